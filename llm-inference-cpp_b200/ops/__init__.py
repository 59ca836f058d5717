"""The CUDA kernels of the library: ``library`` builds and loads them, ``kernels`` calls them."""

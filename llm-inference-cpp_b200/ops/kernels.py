"""Typed Python entry points of the CUDA kernels (``csrc/``), called through ctypes.

Each function checks what the kernel cannot check (device, type, contiguity),
passes raw pointers and the current CUDA stream, and turns a refusal of the
launcher into a :class:`KernelError` that names the kernel and the reason.
There is no other implementation behind these names: without the built library
they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_void_p

import torch

from . import library

OUT_STORE = 0        # y (compute type) = x·Wᵀ
OUT_STORE_F32 = 1    # y (fp32) = x·Wᵀ
OUT_ADD_F32 = 2      # y (fp32) += x·Wᵀ

_ERRORS = {
    -1: "unsupported element type",
    -2: "a size is out of the range this kernel takes",
    -3: "the launch failed (see the CUDA error state)",
    -4: "a pointer or pitch is not aligned as the kernel needs",
    -5: "this combination of options is not supported",
    -6: "a CUDA driver call failed",
}


class KernelError(RuntimeError):
    pass


def _check(name: str, code: int) -> None:
    if code != 0:
        raise KernelError(f"{name}: {_ERRORS.get(code, f'error {code}')}")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported element type {t.dtype}")


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only (there is no CPU path)")


_configured = False


def lib():
    global _configured
    l = library.load()
    if not _configured:
        for name in ("llmi_embed", "llmi_rmsnorm", "llmi_swiglu", "llmi_linear_simt", "llmi_rope_store",
                     "llmi_attention_generic", "llmi_argmax", "llmi_sample"):
            getattr(l, name).restype = c_int
        _configured = True
    return l


# ---------------------------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = fp32(table[ids[t]]); ids int32 [T]; out fp32 [T, W]; a negative id gives zeros."""
    _need_cuda(table, ids, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
    T, W = out.shape
    _check("embed", lib().llmi_embed(c_int(_dtype_code(table)), _ptr(table), _ptr(ids), _ptr(out), c_int(T),
                                     c_int(W), _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = weight * (x[src] * rsqrt(mean(x[src]^2) + eps)), src = rows[r] if rows is given else r."""
    _need_cuda(x, weight, out, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n, W = out.shape
    assert x.shape[1] == W and weight.numel() == W
    _check("rmsnorm", lib().llmi_rmsnorm(c_int(_dtype_code(out)), _ptr(x), _ptr(weight), _ptr(out), _ptr(rows),
                                         c_int(n), c_int(W), c_float(eps), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :F]) * gate_up[:, F:]."""
    _need_cuda(gate_up, out)
    n, F = out.shape
    assert gate_up.shape == (n, 2 * F) and gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype
    _check("swiglu", lib().llmi_swiglu(c_int(_dtype_code(out)), _ptr(gate_up), _ptr(out), c_int(n), c_int(F), _stream()))


def linear_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                mode: int = OUT_STORE) -> None:
    """out (mode) x·wᵀ + bias with fp32 FMA arithmetic; x [M,K], w [N,K], rows may be strided."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and x.dtype == w.dtype
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if mode == OUT_STORE:
        assert out.dtype == x.dtype
    else:
        assert out.dtype == torch.float32
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _check("linear_simt", lib().llmi_linear_simt(
        c_int(_dtype_code(x)), _ptr(x), c_long(x.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(bias), _ptr(out),
        c_long(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(mode), _stream()))


def linear(x, w, out, bias=None, mode: int = OUT_STORE) -> None:
    """The matrix product of the step: picks the kernel for the type and shape."""
    linear_simt(x, w, out, bias, mode)


def rope_store(qkv: torch.Tensor, inv_freq: torch.Tensor | None, rotary_dim: int, tok_seq, tok_pos, seq_pages,
               page_size: int, k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv_heads: int,
               head_dim: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k, and append k, v of each token to its sequence's cache page."""
    _need_cuda(qkv, inv_freq, tok_seq, tok_pos, seq_pages, k_cache, v_cache)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert seq_pages.dtype == torch.int32 and seq_pages.dim() == 2
    _check("rope_store", lib().llmi_rope_store(
        c_int(_dtype_code(qkv)), _ptr(qkv), c_long(qkv.stride(0)), _ptr(inv_freq), c_int(rotary_dim), _ptr(tok_seq),
        _ptr(tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)), c_int(page_size), _ptr(k_cache), _ptr(v_cache),
        c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(1 if write_kv else 0), _stream()))


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, tok_seq, tok_pos, seq_pages,
                      page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of every token over its sequence's cache; q is [T, >= n_heads*head_dim] (row-strided)."""
    _need_cuda(q, out, k_cache, v_cache, tok_seq, tok_pos, seq_pages)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * head_dim)
    assert q.dtype == out.dtype == k_cache.dtype
    _check("attention_generic", lib().llmi_attention_generic(
        c_int(_dtype_code(q)), _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache),
        _ptr(v_cache), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)), c_int(page_size),
        c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r]; logits fp32 [R, V], out int32 [R]."""
    _need_cuda(logits, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check("argmax", lib().llmi_argmax(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _ptr(out), _stream()))


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniforms: torch.Tensor,
           probs_scratch: torch.Tensor, out: torch.Tensor) -> None:
    """Temperature / top-k / top-p sampling; uniforms float64 [R] in [0, 1); probs_scratch fp32 [R, V]."""
    _need_cuda(logits, uniforms, probs_scratch, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert uniforms.dtype == torch.float64 and uniforms.numel() >= R
    assert probs_scratch.dtype == torch.float32 and probs_scratch.numel() >= R * V and probs_scratch.is_contiguous()
    _check("sample", lib().llmi_sample(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V),
                                       c_float(temperature), c_int(top_k), c_float(top_p), _ptr(uniforms),
                                       _ptr(probs_scratch), _ptr(out), _stream()))


def attention(qkv: torch.Tensor, out: torch.Tensor, k_cache, v_cache, ctx, seq_pages, page_size: int, n_heads: int,
              n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Attention of a step's tokens over the cache; q is the first n_heads*head_dim columns of ``qkv``."""
    attention_generic(qkv, out, k_cache, v_cache, ctx.tok_seq, ctx.tok_pos, seq_pages, page_size, n_heads,
                      n_kv_heads, head_dim, scale, window)

"""Typed Python entry points of the CUDA kernels (``csrc/``), called through ctypes.

Each function checks what the kernel cannot check (device, type, contiguity),
passes raw pointers and the current CUDA stream, and turns a refusal of the
launcher into a :class:`KernelError` that names the kernel and the reason.
There is no other implementation behind these names: without the built library
they raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_long, c_void_p

import torch

from . import library

OUT_STORE = 0        # y (compute type) = x·Wᵀ
OUT_STORE_F32 = 1    # y (fp32) = x·Wᵀ
OUT_ADD_F32 = 2      # y (fp32) += x·Wᵀ
OUT_SWIGLU = 3       # y (compute type) = silu(gate)·up, W's rows alternating gate and up rows (tensor-core kernel only)

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


_launches = 0


def launch_count(add: int = 0) -> int:
    """Kernels of this library launched so far in this process (``add`` adjusts it: a graph replay
    adds the kernels it holds)."""
    global _launches
    _launches += add
    return _launches


def _check(name: str, code: int) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"{name}: {_ERRORS.get(code, f'error {code}')}")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported element type {t.dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> c_void_p:
    """The current CUDA stream of the current device (the capture stream while a graph is recorded).  A launch asks
    for it every time; ``torch.cuda.current_stream()`` costs several microseconds a call, which is a quarter of the
    host time of a short prompt's step, so the raw accessor is used where this torch has it."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def _stream_int() -> int:
    """The same as a plain integer, for the functions whose argument types are declared (see ``lib``)."""
    return _stream().value or 0


def copy_to_device(dst_ptr: int, src_ptr: int, n_bytes: int, done: "Mark | None" = None) -> None:
    """``n_bytes`` from pinned host memory at ``src_ptr`` to device memory at ``dst_ptr`` on the current stream (the
    caller keeps both alive and does not touch the host bytes until the copy is done: ``done.wait()`` tells)."""
    code = lib().llmi_copy_to_device(c_void_p(dst_ptr), c_void_p(src_ptr), c_long(n_bytes),
                                     c_void_p(done.handle if done is not None else 0), _stream())
    if code != 0:
        raise KernelError(f"copy_to_device: {_ERRORS.get(code, f'error {code}')}")


class Mark:
    """A point in a stream's work that the host can wait for (set by :func:`copy_to_device`)."""

    def __init__(self):
        fn = lib().llmi_mark_new
        fn.restype = c_void_p
        self.handle = fn()
        if not self.handle:
            raise KernelError("mark: the device gave none")

    def wait(self) -> None:
        if lib().llmi_mark_wait(c_void_p(self.handle)) != 0:
            raise KernelError("mark: the wait failed")

    def __del__(self):
        try:
            if self.handle:
                lib().llmi_mark_free(c_void_p(self.handle))
                self.handle = None
        except Exception:
            pass


def copy_to_host(dst_ptr: int, src_ptr: int, n_bytes: int) -> None:
    """``n_bytes`` from device memory at ``src_ptr`` to pinned host memory at ``dst_ptr`` on the current stream; returns
    when they are there."""
    code = lib().llmi_copy_to_host(c_void_p(dst_ptr), c_void_p(src_ptr), c_long(n_bytes), _stream())
    if code != 0:
        raise KernelError(f"copy_to_host: {_ERRORS.get(code, f'error {code}')}")


def _addr(t) -> int | None:
    return None if t is None else t.data_ptr()


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
                     "llmi_attention_generic", "llmi_argmax", "llmi_sample", "llmi_gemm_tc", "llmi_gemm_tc_splits",
                     "llmi_attention_decode", "llmi_attention_decode_supported", "llmi_attention_decode_resident",
                     "llmi_attention_decode_fused", "llmi_attention_decode_mma", "llmi_attention_decode_mma_supported",
                     "llmi_attention_decode_mma_resident", "llmi_attention_decode_clusters_resident",
                     "llmi_attention_prefill", "llmi_attention_prefill_supported", "llmi_gemm_skinny",
                     "llmi_gemm_skinny_max_tokens", "llmi_attention_prefill_tc", "llmi_attention_prefill_tc_supported",
                     "llmi_sm_count"):
            getattr(l, name).restype = c_int
        l.llmi_gemm_tc_workspace.restype = c_long
        l.llmi_attention_decode_workspace.restype = c_long
        # The launchers of a prompt's step are called a few hundred times per step from Python: with their argument
        # types declared, plain integers go in without a ctypes object being made for each (a third of a call's cost).
        P, L, I, F = c_void_p, c_long, c_int, c_float
        l.llmi_gemm_tc.argtypes = [P, L, P, L, P, P, L, I, I, I, I, P, L, P, I, P, P]
        l.llmi_rmsnorm.argtypes = [I, P, P, P, P, I, I, F, P]
        l.llmi_rope_store.argtypes = [I, P, L, P, I, P, P, P, I, I, P, P, I, I, I, I, I, P]
        l.llmi_attention_prefill_tc.argtypes = [P, L, L, P, L, P, P, L, P, I, P, P, I, I, I, I, I, F, I, I, I, P, L, P, I, P, P]
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
    _check("rmsnorm", lib().llmi_rmsnorm(_dtype_code(out), x.data_ptr(), weight.data_ptr(), out.data_ptr(), _addr(rows), n, W,
                                         eps, _stream_int()))


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


class _TcScratch:
    """Per-device scratch of the tensor-core product: split-K partial tiles, tile tickets (zero between
    launches) and an error word that a bounded wait sets instead of hanging."""
    WORKSPACE_BYTES = 32 << 20
    N_TICKETS = 4096
    N_ATTN_TICKETS = 1 << 16

    def __init__(self, device):
        self.workspace = torch.empty(self.WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        self.tickets = torch.zeros(self.N_TICKETS, dtype=torch.int32, device=device)
        self.attn_tickets = torch.zeros(self.N_ATTN_TICKETS, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)


_tc_scratch: dict = {}


def tc_scratch(device) -> _TcScratch:
    key = torch.device(device).index or 0
    if key not in _tc_scratch:
        _tc_scratch[key] = _TcScratch(device)
    return _tc_scratch[key]


def check_device_errors(device) -> None:
    """Raise if a kernel's bounded wait gave up since the last check (synchronises the device)."""
    sc = _tc_scratch.get(torch.device(device).index or 0)
    if sc is not None:
        code = int(sc.error.item())
        if code:
            sc.error.zero_()
            raise KernelError(f"a bounded wait inside a kernel timed out (code {code}); results are invalid")


_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the device the kernels run on (asked once; a B200 has 148)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = max(1, int(lib().llmi_sm_count()))
    return _sm_count


def gemm_tc_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
            mode: int = OUT_STORE) -> None:
    """out (mode) x·wᵀ + bias on the tcgen05 tensor cores; bf16 inputs, fp32 accumulation."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2 if mode == OUT_SWIGLU else N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert out.dtype == (torch.bfloat16 if mode in (OUT_STORE, OUT_SWIGLU) else torch.float32)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    sc = tc_scratch(x.device)
    _check("gemm_tc", lib().llmi_gemm_tc(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _addr(bias), out.data_ptr(), out.stride(0), M, N, K, mode,
        sc.workspace.data_ptr(), sc.WORKSPACE_BYTES, sc.tickets.data_ptr(), sc.N_TICKETS, sc.error.data_ptr(), _stream_int()))


class DeferredNorm:
    """A row-wise norm y = weight * x / sqrt(mean(x^2) + eps) split over the two products around it.

    The product that last updates x (a residual add) fills ``h`` = compute-type(weight * x) and ``ss`` — the sum
    of x^2 over each 16-row tile of its output, per token — and the product that reads the norm's output
    takes ``h`` as its input and multiplies its accumulators by 1/sqrt(sum(ss)/width + eps) (a reader that cannot
    do that runs the norm the plain way over ``source``, the x the filling product updated).  A norm of a
    handful of rows is all launch and latency; this way it costs no kernel.  Made by a norm part
    (``deferred``), filled by ``linear(..., then_norm=)``, consumed by passing it as ``linear``'s input.
    """
    SS_STRIDE = 64

    def __init__(self, weight: torch.Tensor, eps: float, h: torch.Tensor, ss: torch.Tensor):
        self.weight, self.eps, self.h, self.ss = weight, float(eps), h, ss
        self.source = None       # the x that the filling product updated: a reader that cannot scale normalises from it
        self.n_tiles = (h.shape[1] + 15) // 16
        assert ss.dtype == torch.float32 and ss.numel() >= self.n_tiles * self.SS_STRIDE and weight.dtype == torch.float32

    @property
    def shape(self):
        return self.h.shape

    @property
    def dtype(self):
        return self.h.dtype


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                mode: int = OUT_STORE, then_norm: DeferredNorm | None = None, scale_from: DeferredNorm | None = None) -> None:
    """The same product for at most 64 tokens: the weight-streaming kernel (``csrc/gemm_skinny.cu``).

    ``then_norm`` (mode OUT_ADD_F32): also fill that deferred norm from the updated ``out``.
    ``scale_from``: ``x`` is that deferred norm's ``h``; apply its scale to the accumulators."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2 if mode == OUT_SWIGLU else N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert out.dtype == (torch.bfloat16 if mode in (OUT_STORE, OUT_SWIGLU) else torch.float32)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if then_norm is not None:
        assert mode == OUT_ADD_F32 and then_norm.h.shape == (M, N) and then_norm.h.dtype == torch.bfloat16
        assert then_norm.weight.numel() == N and then_norm.h.stride(1) == 1
    if scale_from is not None:
        assert scale_from.h.data_ptr() == x.data_ptr() and scale_from.h.shape == (M, K)
    sc = tc_scratch(x.device)
    e, f = then_norm, scale_from
    if e is not None:
        e.source = out
    _check("gemm_skinny", lib().llmi_gemm_skinny(
        _ptr(x), c_long(x.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(bias), _ptr(out), c_long(out.stride(0)),
        c_int(M), c_int(N), c_int(K), c_int(mode),
        _ptr(e.weight if e else None), _ptr(e.h if e else None), c_long(e.h.stride(0) if e else 0), _ptr(e.ss if e else None),
        _ptr(f.ss if f else None), c_int(f.n_tiles if f else 0), c_float(f.eps if f else 0.0),
        _ptr(sc.error), _stream()))


SKINNY_MAX_TOKENS = 16
_FORCE_SIMT = os.environ.get("LLMI_LINEAR", "") == "simt"
_NO_SKINNY = os.environ.get("LLMI_LINEAR", "") == "tc"
_FUSE_NORM = os.environ.get("LLMI_FUSE_NORM", "1") != "0"


SKINNY_SMALL_WEIGHT = 16 << 20    # elements: up to here the weight-streaming kernel also takes 17 to 32 tokens
SKINNY_TINY_WEIGHT = 3 << 20      # and up to here 33 to 64 tokens


def skinny_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product x·wᵀ goes to the weight-streaming kernel: up to 16 tokens always; beyond, where the tcgen05
    kernel's fixed cost (cluster, TMEM, exchange of partial tiles over a cluster when there are few 128-row tiles: 4 to
    5 us) is most of its time, or where the norm that rides on the weight-streaming products would cost a kernel of
    its own.  Measured (us, weight-streaming against tcgen05), 32 tokens: 2,048 x 2,048 4.9 / 5.2, 6,144 x 2,048
    10.7 / 8.8 (plus a norm of 3 us), 2,048 x 8,192 11.3 / 11.4, but 16,384 x 2,048 21.2 / 14.8, 6,144 x 4,096
    17.2 / 13.0; 64 tokens: 576 x 1,536 5.3 / 5.5, 1,600 x 960 4.7 / 5.5, 960 x 2,560 6.9 / 6.5, but 2,048 x 2,048
    6.5 / 6.2, 2,048 x 8,192 15.2 / 12.2, 6,144 x 2,048 16.2 / 9.4, 16,384 x 2,048 32.7 / 15.4 (a decode step of the
    1.7B shape at batch 64 with the two 2,048-row products on the tcgen05 kernel: 9.61 -> 9.28 ms)."""
    n = x.shape[0]
    if _FORCE_SIMT or _NO_SKINNY or x.shape[1] % 64 or not gemm_tc_eligible(x, w):
        return False
    return bool(n <= SKINNY_MAX_TOKENS or (n <= 32 and w.numel() <= SKINNY_SMALL_WEIGHT)
                or (n <= 64 and w.numel() <= SKINNY_TINY_WEIGHT))


def norm_deferrable(n_tokens: int, width: int, dtype) -> bool:
    """Whether a norm over ``width`` of ``n_tokens`` rows can be split over the products around it."""
    return bool(_FUSE_NORM and not _FORCE_SIMT and not _NO_SKINNY and dtype == torch.bfloat16
                and n_tokens <= DeferredNorm.SS_STRIDE and width % 64 == 0)


def gemm_bf16(x, w, out, bias=None, mode: int = OUT_STORE, then_norm: DeferredNorm | None = None) -> bool:
    """The bf16 tensor-core product: the weight-streaming kernel for a handful of tokens, the tcgen05
    kernel for more.  ``x`` may be a filled :class:`DeferredNorm`; returns whether ``then_norm`` was filled."""
    pending = x if isinstance(x, DeferredNorm) else None
    xin = pending.h if pending is not None else x
    if skinny_applies(xin, w):
        gemm_skinny(xin, w, out, bias, mode, then_norm, pending)
        return then_norm is not None
    if pending is not None:
        # this reader cannot apply the scale to its accumulators: the norm is run the plain way after all, over the
        # h that the filling product left (one launch, as without the deferral)
        if pending.source is None:
            raise KernelError("a deferred norm that no product has filled")
        rmsnorm(pending.source, pending.weight, pending.h, pending.eps)
    gemm_tc(xin, w, out, bias, mode)
    return False


def linear(x, w, out, bias=None, mode: int = OUT_STORE, then_norm: DeferredNorm | None = None) -> bool:
    """The matrix product of the step: the tensor-core kernels for bf16 operands they can take (16-byte
    aligned rows), the fp32 FMA kernel for the 32-bit path and for everything else.  ``x`` may be a filled
    :class:`DeferredNorm`; returns whether ``then_norm`` was filled (False: run that norm the plain way)."""
    xin = x.h if isinstance(x, DeferredNorm) else x
    if not _FORCE_SIMT and gemm_tc_eligible(xin, w):
        return gemm_bf16(x, w, out, bias, mode, then_norm)
    if isinstance(x, DeferredNorm):      # a reader that cannot scale: the norm the plain way after all
        if x.source is None:
            raise KernelError("a deferred norm that no product has filled")
        rmsnorm(x.source, x.weight, x.h, x.eps)
    linear_simt(xin, w, out, bias, mode)
    return False


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
        _dtype_code(qkv), qkv.data_ptr(), qkv.stride(0), _addr(inv_freq), rotary_dim, tok_seq.data_ptr(), tok_pos.data_ptr(),
        seq_pages.data_ptr(), seq_pages.stride(0), page_size, k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv_heads,
        head_dim, 1 if write_kv else 0, _stream_int()))


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


DECODE_PAGES_PER_SPLIT = 8     # default split of the decode kernel: 512 positions


_resident_cache: dict = {}


# Which decode kernel takes grouped queries (group = query heads per kv head >= 2) of head size 64 or 128: "mma"
# (the group's heads as rows of tensor-core tiles: the work per page does not grow with the group) or "simt"
# (the CUDA-core kernel, which always takes group 1).
_DECODE_ATTENTION = os.environ.get("LLMI_DECODE_ATTENTION", "mma")


def decode_uses_mma(head_dim: int, group: int) -> bool:
    return bool(_DECODE_ATTENTION == "mma" and group >= 2
                and lib().llmi_attention_decode_mma_supported(c_int(head_dim), c_int(group)))


def decode_pages_per_split(n_seqs: int, n_kv_heads: int, max_pages: int, head_dim: int = 64, group: int = 1) -> int:
    """How many pages one work item of the decode kernel covers.

    The kernel is persistent: ``resident`` blocks share the items round-robin.  The split is chosen so
    that the last round of items is nearly full (little idle tail) while an item stays long enough
    (at least 8 pages unless the batch is tiny) that its fixed cost — first load, merge, ticket —
    is small beside its streaming time.  Large batches get no split at all.
    """
    pairs = max(1, n_seqs * n_kv_heads)
    if decode_uses_mma(head_dim, group):
        key = (head_dim, group)
        if key not in _resident_cache:
            _resident_cache[key] = max(1, int(lib().llmi_attention_decode_mma_resident(c_int(head_dim), c_int(group))))
        resident = _resident_cache[key]
        # The tensor-core kernel: the end of an item that is one of several splits costs about six pages of streaming
        # (four warps merged, the partial result written, a ticket), of a whole sequence-head two; the last split to
        # arrive merges two heads and NZ splits per round trip to L2 (about 1.5 pages of head size 64 each).
        # Measured at 4,096 positions: 8 kv heads of size 64, batch 1: 8.7 us at 4 pages a split, 10.6 at 2, 13.1 at
        # 16; batch 64: 84 us without splits, 91 at 16 pages, 119 at 8.
        nz = 16 if head_dim <= 64 else 8
        best, best_cost = max_pages, float("inf")
        for splits in range(1, max(1, max_pages // 4) + 1):
            pps = -(-max_pages // splits)
            n_parts = -(-max_pages // pps)
            rounds = -(-pairs * n_parts // resident)
            cost = rounds * (pps + (2 if n_parts == 1 else 6))
            if n_parts > 1:
                cost += -(-group // 2) * -(-n_parts // nz) * 1.5 * 64 / head_dim
            if cost < best_cost - 1e-9:
                best, best_cost = pps, cost
        return best
    # The CUDA-core kernel has two variants (csrc/attention_decode.cu): with few sequence-heads the one with a producer
    # thread for the key tiles and one for the value tiles, two blocks per SM, whose items may be long.
    key = (head_dim, group, n_seqs, n_kv_heads)
    if key not in _resident_cache:
        two = ctypes.c_int(0)
        resident = int(lib().llmi_attention_decode_plan(c_int(head_dim), c_int(group), c_int(n_seqs), c_int(n_kv_heads), ctypes.byref(two)))
        _resident_cache[key] = (max(1, resident), bool(two.value))
    resident, two_producers = _resident_cache[key]
    best, best_score = max_pages, -1.0
    for splits in range(1, max(1, max_pages // (2 if two_producers else 4)) + 1):
        pps = -(-max_pages // splits)
        n_parts = -(-max_pages // pps)
        items = pairs * n_parts
        rounds = -(-items // resident)
        fill = items / (rounds * resident)                 # how full the rounds are
        # An item costs about two pages of streaming on top; with two producers, where items are read twice as fast,
        # one of several splits about four (partial result, fence, ticket, the last one's merge).  The latter fitted
        # to measurements (32 kv heads of 64; best split measured = chosen): 4,096 positions at batch 1 / 2 / 4 / 8:
        # 8 / 16 / 32 pages / none; 8,192 positions: 16 / 32 / 64 / none; 1,024 positions: 2 / 4 / 8 / none.
        score = fill * pps / (pps + (4.0 if (two_producers and n_parts > 1) else 2.0))
        if score > best_score + 1e-9:
            best, best_score = pps, score
    return best


_PLAN_BY_LIVE = os.environ.get("LLMI_DECODE_PLAN", "live") != "padded"
_plan_cache: dict = {}


def decode_plan(ctx, n_seqs: int, n_pages: int, page_size: int, n_kv_heads: int, head_dim: int, group: int):
    """(pages per item, live sequences) for the decode kernel of a step whose page tables are [n_seqs, n_pages].

    A recorded step is padded to a power of two of sequences.  The kernel skips the padding, but a split chosen for
    16 sequences is a poor one for 9 or 12: so the split (and the kernel's variant) follow the step's LIVE sequences
    (:func:`decode_plan_token` tells recorded steps with different answers apart).  Measured, a decode step of 32
    heads of 64 at 4,096 positions, planned by the padded and by the live number: batch 3 1.334 -> 1.291 ms, 5
    1.754 -> 1.597, 9 2.145 -> 2.025, 12 2.594 -> 2.403, 24 4.264 -> 4.165; 14 and 40 unchanged.  The page tables'
    padded width stays the measure of length: following the live pages too changed the split every few hundred
    tokens (a new recording each time) for no gain at batch 1 to 3.  ``LLMI_DECODE_PLAN=padded`` plans by the
    padded number."""
    n_live = n_seqs
    if _PLAN_BY_LIVE:
        n_live = min(n_seqs, max(1, int(getattr(ctx, "n_real_seqs", 0) or n_seqs)))
    key = (n_live, n_pages, n_kv_heads, head_dim, group)
    plan = _plan_cache.get(key)
    if plan is None:
        pps = decode_pages_per_split(n_live, n_kv_heads, n_pages, head_dim, group)
        cluster = decode_cluster(n_live, n_kv_heads, n_pages, head_dim, group) if pps < n_pages else 0
        if cluster:
            pps = -(-n_pages // cluster)
        plan = _plan_cache[key] = (pps, cluster)
    return plan[0], n_live, plan[1]


_CLUSTER = os.environ.get("LLMI_DECODE_CLUSTER", "1") != "0"
_CLUSTER_MAX_PAGES = int(os.environ.get("LLMI_DECODE_CLUSTER_PAGES", "4"))
_clusters_resident: dict = {}


def decode_cluster(n_live: int, n_kv_heads: int, n_pages: int, head_dim: int, group: int) -> int:
    """The size of the clusters (8, 4 or 2 blocks, one cluster per sequence-head) in which the decode kernel runs a
    step of few sequence-heads and short sequences, or 0 for its persistent form: the largest size whose clusters are
    all resident at once and give a block two to four pages (``LLMI_DECODE_CLUSTER_PAGES``).  Ungrouped queries on the
    CUDA-core kernel only.  With so few pages a block the kernel is as long as the chain behind its last page —
    partial result to memory, fence, ticket, the last block's loads of all partial results — and the clusters replace
    that chain by stores into the first block's shared memory.  A decode step of 32 heads of 64 (24 layers, 2,048
    wide), persistent form -> clusters: batch 1 at 512 / 1,024 / 2,048 positions 0.985 -> 0.933 / 0.999 -> 0.964 /
    1.020 -> 0.995 ms; batch 2 at 512 / 1,024: 0.968 -> 0.941 / 0.997 -> 0.980; batch 4 at 512: 0.994 -> 0.984.  With
    more pages a block it loses (one producer thread a block, few blocks: batch 1 at 4,096 positions, 8 pages a
    block: 1.060 -> 1.084 ms; batch 4: 1.402 -> 1.547), so there the persistent form with its shorter items stays.
    ``LLMI_DECODE_CLUSTER=0`` switches the clusters off."""
    if not _CLUSTER or group != 1 or decode_uses_mma(head_dim, group):
        return 0
    for size in (8, 4, 2):
        if n_pages < 2 * size or -(-n_pages // size) > _CLUSTER_MAX_PAGES:
            continue
        key = (head_dim, size)
        if key not in _clusters_resident:
            _clusters_resident[key] = int(lib().llmi_attention_decode_clusters_resident(c_int(head_dim), c_int(group), c_int(size)))
        if n_live * n_kv_heads <= _clusters_resident[key]:
            return size
    return 0


def decode_plan_token(ctx, n_seqs: int, n_pages: int, page_size: int, n_kv_heads: int, head_dim: int, group: int):
    """What tells two recorded decode steps of the same padded shape apart: the split and the kernel's variant."""
    pps, n_live, cluster = decode_plan(ctx, n_seqs, n_pages, page_size, n_kv_heads, head_dim, group)
    if decode_uses_mma(head_dim, group):
        return (pps,)
    key = (head_dim, group, n_live, n_kv_heads)
    if key not in _resident_cache:
        decode_pages_per_split(n_live, n_kv_heads, n_pages, head_dim, group)
    return (pps, _resident_cache[key][1], cluster)


def attention_decode_supported(head_dim: int, group: int) -> bool:
    return decode_uses_mma(head_dim, group) or bool(lib().llmi_attention_decode_supported(c_int(head_dim), c_int(group)))


def attention_decode_mma(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start,
                         n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, partials: torch.Tensor,
                         pages_per_split: int, rope=None) -> None:
    """:func:`attention_decode` (``rope`` None) or :func:`attention_decode_fused` (``rope = (inv_freq, rotary_dim,
    write_kv)``, ``q`` the un-rotated [q | k | v] rows) by the tensor-core kernel for grouped queries."""
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start, partials)
    S, P = seq_pages.shape
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.shape[-2] == 64 and partials.dtype == torch.float32
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    inv_freq, rotary_dim, write_kv = rope if rope is not None else (None, 0, False)
    assert rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    sc = tc_scratch(q.device)
    _check("attention_decode_mma", lib().llmi_attention_decode_mma(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_long(k_cache.shape[0]), _ptr(seq_pages), c_int(seq_pages.stride(0)), _ptr(seq_kv_len), _ptr(seq_q_start), c_int(S),
        c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window), c_int(P), c_int(pages_per_split),
        c_int(0 if rope is None else 1), _ptr(inv_freq) if rotary_dim else None, c_int(rotary_dim),
        c_int(1 if write_kv else 0), _ptr(partials), c_long(partials.numel()), _ptr(sc.attn_tickets),
        c_int(sc.N_ATTN_TICKETS), _ptr(sc.error), _stream()))


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start,
                     n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, partials: torch.Tensor,
                     pages_per_split: int = DECODE_PAGES_PER_SPLIT, n_live: int = 0, cluster: int = 0) -> None:
    """One token per sequence over its cache pages (bf16, page size 64), split over positions.

    ``partials``: fp32 scratch of at least ``attention_decode_workspace(...)`` floats.  ``n_live``: how many of
    the sequences are not padding, if the caller knows (it decides which variant of the kernel runs, nothing else).
    ``cluster`` (2, 4, 8; ungrouped queries): the form of the kernel with one cluster of that many blocks per
    sequence-head, whose splits meet in shared memory; ``pages_per_split`` x ``cluster`` must cover the page tables.
    """
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start, partials)
    S, P = seq_pages.shape
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.shape[-2] == 64 and partials.dtype == torch.float32
    sc = tc_scratch(q.device)
    _check("attention_decode", lib().llmi_attention_decode(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(seq_pages),
        c_int(seq_pages.stride(0)), _ptr(seq_kv_len), _ptr(seq_q_start), c_int(S), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(P), c_int(pages_per_split), _ptr(partials),
        c_long(partials.numel()), _ptr(sc.attn_tickets), c_int(sc.N_ATTN_TICKETS), _ptr(sc.error), c_int(n_live),
        c_int(cluster), _stream()))


def attention_decode_workspace(n_seqs: int, n_heads: int, head_dim: int, max_pages: int,
                               pages_per_split: int = DECODE_PAGES_PER_SPLIT) -> int:
    return int(lib().llmi_attention_decode_workspace(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(max_pages),
                                                     c_int(pages_per_split)))


def attention_prefill_supported(head_dim: int) -> bool:
    return bool(lib().llmi_attention_prefill_supported(c_int(head_dim)))


def attention_prefill_tc_supported(head_dim: int) -> bool:
    return bool(lib().llmi_attention_prefill_tc_supported(c_int(head_dim)))


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len,
                      n_blocks: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of the prompts of a step over their cache pages (bf16, head size 64 or 128, page 64).

    ``seq_q_start`` [n_seqs + 1] are the sequences' offsets into the step's tokens, ``seq_kv_len`` their
    lengths after the step, ``n_blocks`` the sum over sequences of ceil(tokens / 128).
    """
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len)
    S = seq_pages.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.shape[-2] == 64 and k_cache.is_contiguous() and v_cache.is_contiguous()
    sc = tc_scratch(q.device)
    _check("attention_prefill", lib().llmi_attention_prefill(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_long(k_cache.shape[0]), _ptr(seq_pages), c_int(seq_pages.stride(0)), _ptr(seq_q_start), _ptr(seq_kv_len),
        c_int(S), c_int(n_blocks), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
        _ptr(sc.error), _stream()))


PREFILL_SPLIT_PAGES = 16      # key pages per job when the prompt attention cuts its long query blocks


def prefill_split_jobs(q_lens, kv_lens, window: int, split_pages: int) -> int:
    """How many jobs the prompt attention has along its first grid dimension when every block of 128 queries
    is cut into parts of ``split_pages`` key pages (the kernel's own rule, counted on the host)."""
    jobs = 0
    for q_len, kv_len in zip(q_lens, kv_lens):
        pos0 = kv_len - q_len
        for mb in range((q_len + 127) // 128):
            first_q = pos0 + mb * 128
            last_q = first_q + min(128, q_len - mb * 128) - 1
            lo_key = first_q - window + 1 if (window > 0 and first_q - window + 1 > 0) else 0
            n_pg = last_q // 64 - lo_key // 64 + 1
            jobs += (n_pg + split_pages - 1) // split_pages
    return jobs


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len,
                         n_blocks: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                         split=None) -> None:
    """The same prompt attention on the tcgen05 tensor cores (head size 64 or 128); arguments as ``attention_prefill``.
    ``split = (n_jobs, split_pages, workspace)``: cut the key range of every query block into jobs of
    ``split_pages`` pages (``n_jobs`` from :func:`prefill_split_jobs`, ``workspace`` fp32 of
    n_jobs * n_heads * (head_dim + 2) * 128 floats)."""
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len)
    S = seq_pages.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.shape[-2] == 64 and k_cache.is_contiguous() and v_cache.is_contiguous()
    sc = tc_scratch(q.device)
    n_jobs, split_pages, ws = split if split is not None else (n_blocks, 0, None)
    if ws is not None:
        assert ws.dtype == torch.float32 and ws.is_cuda
    _check("attention_prefill_tc", lib().llmi_attention_prefill_tc(
        q.data_ptr(), q.stride(0), q.shape[0], out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        k_cache.shape[0], seq_pages.data_ptr(), seq_pages.stride(0), seq_q_start.data_ptr(), seq_kv_len.data_ptr(), S,
        n_blocks, n_heads, n_kv_heads, head_dim, scale, window, n_jobs, split_pages, _addr(ws),
        ws.numel() if ws is not None else 0, sc.attn_tickets.data_ptr(), sc.N_ATTN_TICKETS, sc.error.data_ptr(), _stream_int()))


# Which prompt-attention kernel runs: "tc" (tcgen05: about 43 us for a 2,048-token prompt of 32 heads of 64) or
# "mma" (mma.sync: 95 us).
_PREFILL_ATTENTION = os.environ.get("LLMI_PREFILL_ATTENTION", "tc")     # "mma": the mma.sync kernel for every head size
_FORCE_GENERIC_ATTENTION = os.environ.get("LLMI_ATTENTION", "") == "generic"
_PREFILL_SPLIT = os.environ.get("LLMI_PREFILL_SPLIT", "1") != "0"


def attention_decode_fused(qkv: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start,
                           n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, partials: torch.Tensor,
                           pages_per_split: int, inv_freq, rotary_dim: int, write_kv: bool, n_live: int = 0,
                           cluster: int = 0) -> None:
    """:func:`attention_decode` with the step's position encoding done by the same kernel: ``qkv`` holds the
    un-rotated [q | k | v] row of each sequence's token; the new k (rotated) and v are appended to the cache."""
    _need_cuda(qkv, out, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start, partials)
    S, P = seq_pages.shape
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert qkv.stride(1) == 1 and out.stride(1) == 1 and k_cache.shape[-2] == 64 and partials.dtype == torch.float32
    assert rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    sc = tc_scratch(qkv.device)
    _check("attention_decode_fused", lib().llmi_attention_decode_fused(
        _ptr(qkv), c_long(qkv.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(seq_pages),
        c_int(seq_pages.stride(0)), _ptr(seq_kv_len), _ptr(seq_q_start), c_int(S), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(P), c_int(pages_per_split),
        _ptr(inv_freq) if rotary_dim else None, c_int(rotary_dim), c_int(1 if write_kv else 0), _ptr(partials),
        c_long(partials.numel()), _ptr(sc.attn_tickets), c_int(sc.N_ATTN_TICKETS), _ptr(sc.error), c_int(n_live),
        c_int(cluster), _stream()))


_FUSE_ROPE = os.environ.get("LLMI_FUSE_ROPE", "1") != "0"


def _decode_kernel_applies(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rt) -> bool:
    return bool(ctx.decode and qkv.dtype == torch.bfloat16 and page_size == 64 and rt is not None
                and not _FORCE_GENERIC_ATTENTION and seq_pages.shape[0] * n_kv_heads <= _TcScratch.N_ATTN_TICKETS
                and attention_decode_supported(head_dim, n_heads // n_kv_heads))


def attention_fuses_rotation(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rotary_dim, rt) -> bool:
    """Whether :func:`attention` can do this step's rotation and cache append itself (``rope=``): a decode
    step that goes to the split kernel, rotating the whole head or nothing."""
    return bool(_FUSE_ROPE and rotary_dim in (0, head_dim)
                and _decode_kernel_applies(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rt))


def attention(qkv: torch.Tensor, out: torch.Tensor, k_cache, v_cache, ctx, seq_pages, page_size: int, n_heads: int,
              n_kv_heads: int, head_dim: int, scale: float, window: int = 0, rt=None, rope=None) -> None:
    """Attention of a step's tokens over the cache; q is the first n_heads*head_dim columns of ``qkv``.

    In bf16, a decode step goes to the split kernel and a prompt step to the flash kernel when they
    have the head size; everything else (the 32-bit path, other head sizes) goes to the generic kernel.
    ``rope=(inv_freq, rotary_dim, write_kv)``: q, k are not rotated yet and k, v not appended — the kernel
    does it (only where :func:`attention_fuses_rotation` says so).
    """
    if _decode_kernel_applies(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rt):
        S, P = seq_pages.shape
        pps, n_live, cluster = decode_plan(ctx, S, P, page_size, n_kv_heads, head_dim, n_heads // n_kv_heads)
        partials = rt.scratch("attn_partials", (attention_decode_workspace(S, n_heads, head_dim, P, pps),), torch.float32)
        if decode_uses_mma(head_dim, n_heads // n_kv_heads):
            attention_decode_mma(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_kv_len, ctx.seq_q_start, n_heads,
                                 n_kv_heads, head_dim, scale, window, partials, pps, rope)
        elif rope is not None:
            attention_decode_fused(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_kv_len, ctx.seq_q_start, n_heads,
                                   n_kv_heads, head_dim, scale, window, partials, pps, rope[0], rope[1], rope[2], n_live,
                                   cluster)
        else:
            attention_decode(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_kv_len, ctx.seq_q_start, n_heads, n_kv_heads,
                             head_dim, scale, window, partials, pps, n_live, cluster)
        return
    if rope is not None:
        raise RuntimeError("attention: rotation can only be fused into the decode kernel (ask attention_fuses_rotation)")
    if (not ctx.decode and qkv.dtype == torch.bfloat16 and page_size == 64 and not _FORCE_GENERIC_ATTENTION
            and attention_prefill_supported(head_dim)):
        if (_PREFILL_ATTENTION == "tc" and attention_prefill_tc_supported(head_dim) and qkv.stride(0) % 8 == 0
                and out.stride(0) % 8 == 0):
            # A step with fewer (query block, head) jobs than the device has SMs leaves SMs idle and is as long as its
            # longest job: then the key ranges are cut (see the kernel's head).  Measured: 2,048 tokens x 8 heads 28.0 ->
            # 22.2 us, x 4 heads 27.5 -> 21.0 us; with 256 jobs and more the cut gains nothing or costs (4,096 x 8:
            # 49.3 -> 50.5 us; 2,048 x 32: 42.1 -> 49.6 us).
            split = None
            q_lens, kv_lens = getattr(ctx, "host_q_lens", None), getattr(ctx, "host_kv_lens", None)
            if _PREFILL_SPLIT and rt is not None and q_lens is not None and ctx.n_q_blocks * n_heads < sm_count():
                jobs = prefill_split_jobs(q_lens, kv_lens, window, PREFILL_SPLIT_PAGES)
                if jobs > ctx.n_q_blocks:
                    ws = rt.scratch("attn_prefill_partials", (jobs * n_heads * (head_dim + 2) * 128,), torch.float32)
                    split = (jobs, PREFILL_SPLIT_PAGES, ws)
            attention_prefill_tc(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_q_start, ctx.seq_kv_len, ctx.n_q_blocks,
                                 n_heads, n_kv_heads, head_dim, scale, window, split)
            return
        attention_prefill(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_q_start, ctx.seq_kv_len, ctx.n_q_blocks,
                          n_heads, n_kv_heads, head_dim, scale, window)
        return
    attention_generic(qkv, out, k_cache, v_cache, ctx.tok_seq, ctx.tok_pos, seq_pages, page_size, n_heads,
                      n_kv_heads, head_dim, scale, window)

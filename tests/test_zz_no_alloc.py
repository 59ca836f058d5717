"""The decode attention entry point that brings its own scratch memory (GPU).

Some users of the kernel library cannot allocate device memory where they call it — a C program
that links the library without a framework's allocator, a plug-in that is handed its buffers, code
inside a capture or a latency-critical loop where an allocation would stall the device.  For them
``llmi_attention_decode_static`` keeps its scratch in a fixed array inside the library.  This test
calls it the way such a user would: through its exported C symbol, with raw pointers, and nothing
else of the Python package in between.  It must give what the ordinary entry point gives, twice in a
row on different problems (the array keeps the first call's leftovers), and must refuse a problem
that does not fit its array.

The file's name makes pytest collect it last, so that a run stopping at the first failure has
already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_long, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from llmi_b200.ops import library
    lib = ctypes.CDLL(library.build())
    lib.llmi_attention_decode_static.restype = c_int
    lib.llmi_attention_decode.restype = c_int
    lib.llmi_attention_decode_workspace.restype = c_long
    return lib


def _problem(seed, lens, nh, nkv, hd, n_pages):
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    P = max((max(lens) + 63) // 64, 1)
    kc = (torch.randn(n_pages, nkv, 64, hd, generator=g) * 0.7).to(torch.bfloat16).cuda()
    vc = (torch.randn(n_pages, nkv, 64, hd, generator=g) * 0.7).to(torch.bfloat16).cuda()
    perm = torch.randperm(n_pages, generator=g).tolist()
    pages = torch.full((S, P), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for i in range((n + 63) // 64):
            pages[s, i] = perm.pop()
    q = torch.randn(S, nh * hd, generator=g).to(torch.bfloat16).cuda()
    return dict(q=q, kc=kc, vc=vc, pages=pages.cuda(), kvlen=torch.tensor(lens, dtype=torch.int32).cuda(),
                qstart=torch.arange(S, dtype=torch.int32).cuda(), S=S, P=P, nh=nh, nkv=nkv, hd=hd)


def _ptr(t):
    return c_void_p(t.data_ptr())


def _call_static(lib, pr, out, pps, err):
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.llmi_attention_decode_static(
        _ptr(pr["q"]), c_long(pr["q"].stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(pr["kc"]), _ptr(pr["vc"]),
        _ptr(pr["pages"]), c_int(pr["pages"].stride(0)), _ptr(pr["kvlen"]), _ptr(pr["qstart"]), c_int(pr["S"]),
        c_int(pr["nh"]), c_int(pr["nkv"]), c_int(pr["hd"]), c_float(1 / math.sqrt(pr["hd"])), c_int(0), c_int(pr["P"]),
        c_int(pps), _ptr(err), stream)


def _call_ordinary(lib, pr, out, pps):
    n = lib.llmi_attention_decode_workspace(c_int(pr["S"]), c_int(pr["nh"]), c_int(pr["hd"]), c_int(pr["P"]), c_int(pps))
    partials = torch.empty(max(n, 1), device="cuda")
    tickets = torch.zeros(pr["S"] * pr["nkv"], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.llmi_attention_decode(
        _ptr(pr["q"]), c_long(pr["q"].stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(pr["kc"]), _ptr(pr["vc"]),
        _ptr(pr["pages"]), c_int(pr["pages"].stride(0)), _ptr(pr["kvlen"]), _ptr(pr["qstart"]), c_int(pr["S"]),
        c_int(pr["nh"]), c_int(pr["nkv"]), c_int(pr["hd"]), c_float(1 / math.sqrt(pr["hd"])), c_int(0), c_int(pr["P"]),
        c_int(pps), _ptr(partials), c_long(partials.numel()), _ptr(tickets), c_int(tickets.numel()), _ptr(err), c_int(0), c_int(0), stream)
    torch.cuda.synchronize()
    assert rc == 0 and int(err.item()) == 0
    return out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = _library()
    # two different problems back to back: more sequences and splits first, then fewer and another head shape
    problems = [(_problem(1, [700, 64, 1, 333, 1000, 129], 8, 4, 64, 64), 2),
                (_problem(2, [65, 900], 6, 2, 128, 40), 4)]
    for pr, pps in problems:
        ref = _call_ordinary(lib, pr, torch.zeros(pr["S"], pr["nh"] * pr["hd"], dtype=torch.bfloat16, device="cuda"), pps)
        out = torch.full_like(ref, 7.0)
        err = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        rc = _call_static(lib, pr, out, pps, err)
        torch.cuda.synchronize()
        assert rc == 0, f"llmi_attention_decode_static returned {rc}"
        assert int(err.item()) == 0
        a, b = out.double().cpu(), ref.double().cpu()
        assert torch.isfinite(a).all()
        assert float((a - b).abs().max() / b.abs().max()) < 1e-2        # the tolerance of the other bf16 kernel tests
        assert torch.equal(out, ref)                                    # and in fact the same kernel: the same bits


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    pr = _problem(3, [64] * 4, 8, 8, 64, 8)
    out = torch.full((pr["S"], pr["nh"] * pr["hd"]), 7.0, dtype=torch.bfloat16, device="cuda")
    big = dict(pr, S=70000)                       # 70,000 sequences would need more tickets than the array has
    rc = _call_static(lib, big, out, 1, torch.zeros(1, dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert rc == -7                               # LLMI_ERR_STATIC_SCRATCH: refused, nothing launched
    assert (out == 7.0).all()
    # 2,000 sequences of 8 kv heads fit the tickets (16,000 of 16,384) but their partial results do not:
    # 2,000 x 8 heads x 8 splits x (64 + 2) floats are far more than the array's 1,048,576
    wide = dict(pr, S=2000)
    rc = _call_static(lib, wide, out, 1, torch.zeros(1, dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert rc == -7
    assert (out == 7.0).all()
    # and the same sizes with few enough sequences run
    err = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rc = _call_static(lib, pr, out, 1, err)
    torch.cuda.synchronize()
    assert rc == 0 and int(err.item()) == 0 and torch.isfinite(out.float()).all()

"""Each kernel alone against a plain fp32/fp64 PyTorch statement of the same operation, at sizes
other than the engine's test models (GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 1e-2}


def K():
    from llmi_b200.ops import kernels
    return kernels


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    table = torch.randn(301, 72, device="cuda").to(DT[dtype])
    ids = torch.tensor([5, 300, 0, -1, 17], dtype=torch.int32, device="cuda")
    out = torch.full((5, 72), 7.0, device="cuda")
    K().embed(table, ids, out)
    ref = table.float()[ids.clamp_min(0).long()]
    ref[3] = 0
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,eps", [(72, 1e-5), (2048, 1e-6), (1000, 1e-3), (7, 1e-5)])
def test_rmsnorm(dtype, width, eps):
    x = torch.randn(9, width, device="cuda") * 3
    w = 1 + 0.1 * torch.randn(width, device="cuda")
    out = torch.empty(9, width, device="cuda", dtype=DT[dtype])
    K().rmsnorm(x, w, out, eps)
    xd = x.double()
    ref = w.double() * (xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + float(np.float32(eps))))
    assert rel(out, ref) < (1e-6 if dtype == "float32" else 5e-3)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    out2 = torch.empty(3, width, device="cuda", dtype=DT[dtype])
    K().rmsnorm(x, w, out2, eps, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_rows,width", [(700, 2048), (513, 136), (2048, 960)])
def test_rmsnorm_many_rows(dtype, n_rows, width):
    """A prompt's worth of rows (the compute-type output has a kernel of its own from 512 rows on), with padding rows."""
    x = torch.randn(n_rows, width, device="cuda") * 2
    w = 1 + 0.1 * torch.randn(width, device="cuda")
    rows = torch.arange(n_rows, dtype=torch.int32, device="cuda").flip(0).contiguous()
    rows[5] = -1
    out = torch.full((n_rows, width), 7.0, device="cuda", dtype=DT[dtype])
    K().rmsnorm(x, w, out, 1e-5, rows)
    xd = x.double()[rows.long().clamp(min=0)]
    ref = w.double() * (xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + float(np.float32(1e-5))))
    ref[5] = 0
    assert rel(out, ref) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K_", [(1, 200, 72), (5, 64, 64), (70, 129, 1000), (130, 40, 17), (64, 384, 120)])
def test_linear_simt_modes(dtype, M, N, K_):
    k = K()
    x = torch.randn(M, K_, device="cuda").to(DT[dtype])
    w = (torch.randn(N, K_, device="cuda") * 0.1).to(DT[dtype])
    b = torch.randn(N, device="cuda")
    ref = x.double() @ w.double().T
    y = torch.empty(M, N, device="cuda", dtype=DT[dtype])
    k.linear_simt(x, w, y, None, k.OUT_STORE)
    assert rel(y, ref) < (1e-5 if dtype == "float32" else 6e-3)
    y32 = torch.empty(M, N, device="cuda")
    k.linear_simt(x, w, y32, b, k.OUT_STORE_F32)
    assert rel(y32, ref + b.double()) < 1e-5
    acc = torch.randn(M, N, device="cuda")
    before = acc.clone()
    k.linear_simt(x, w, acc, None, k.OUT_ADD_F32)
    assert rel(acc, before.double() + ref) < 1e-5
    # a strided input (columns of a wider matrix) and a batch that is cut differently give the same rows
    wide = torch.randn(M, K_ + 24, device="cuda").to(DT[dtype])
    y1 = torch.empty(M, N, device="cuda")
    k.linear_simt(wide[:, :K_], w, y1, None, k.OUT_STORE_F32)
    y2 = torch.empty(1, N, device="cuda")
    k.linear_simt(wide[M - 1:M, :K_].contiguous(), w, y2, None, k.OUT_STORE_F32)
    assert torch.equal(y1[M - 1:], y2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    gu = (torch.randn(11, 2 * 77, device="cuda") * 4).to(DT[dtype])
    out = torch.empty(11, 77, device="cuda", dtype=DT[dtype])
    K().swiglu(gu, out)
    g, u = gu[:, :77].double(), gu[:, 77:].double()
    assert rel(out, g / (1 + torch.exp(-g)) * u) < (1e-6 if dtype == "float32" else 5e-3)


def paged(n_pages, nkv, hd, dtype, page=64):
    k = torch.full((n_pages, nkv, page, hd), float("nan"), device="cuda", dtype=DT[dtype])
    return k, k.clone()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(6, 2, 48, 48), (5, 5, 16, 16), (4, 1, 80, 32), (3, 3, 24, 0)])
def test_rope_store(dtype, nh, nkv, hd, rot):
    k = K()
    T = 7
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda").to(DT[dtype])
    orig = qkv.clone()
    pos = torch.tensor([0, 1, 63, 64, 130, 5, 2], dtype=torch.int32, device="cuda")
    seq = torch.tensor([0, 0, 0, 0, 0, 1, -1], dtype=torch.int32, device="cuda")
    pages = torch.tensor([[4, 2, 7], [1, -1, -1]], dtype=torch.int32, device="cuda")
    kc, vc = paged(8, nkv, hd, dtype)
    inv = torch.from_numpy(P.rope_inv_freq(rot, 12345.0)).cuda() if rot else None
    k.rope_store(qkv, inv, rot, seq, pos, pages, 64, kc, vc, nh, nkv, hd, True)
    o = orig.double().cpu().numpy()
    for t in range(T):
        if int(seq[t]) < 0:
            assert torch.equal(qkv[t], orig[t])
            continue
        q = o[t, :nh * hd].reshape(1, nh, hd)
        kk = o[t, nh * hd:(nh + nkv) * hd].reshape(1, nkv, hd)
        vv = o[t, (nh + nkv) * hd:].reshape(nkv, hd)
        if rot:
            invn = P.rope_inv_freq(rot, 12345.0)
            q = np.concatenate([P.rope(q[..., :rot], [int(pos[t])], invn), q[..., rot:]], -1)
            kk = np.concatenate([P.rope(kk[..., :rot], [int(pos[t])], invn), kk[..., rot:]], -1)
        page = int(pages[int(seq[t]), int(pos[t]) // 64])
        tol = 2e-6 if dtype == "float32" else 5e-3
        assert rel(qkv[t, :nh * hd].reshape(nh, hd), torch.from_numpy(q[0])) < tol
        assert rel(kc[page, :, int(pos[t]) % 64], torch.from_numpy(kk[0])) < tol
        assert torch.equal(vc[page, :, int(pos[t]) % 64].double().cpu(), torch.from_numpy(vv))
    assert int(torch.isfinite(kc.float()).sum()) == 6 * nkv * hd        # nothing else was written


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd", [(6, 2, 48), (9, 3, 16), (5, 5, 64), (3, 1, 128)])
def test_rope_store_long_prompt_same_bits(dtype, nh, nkv, hd):
    """From 256 tokens on another kernel runs (sines and cosines shared among the heads of a token): it must
    give the bits of the kernel that short steps use, and agree with the plain formulas."""
    k = K()
    T = 300
    gen = torch.Generator(device="cuda").manual_seed(hd)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", generator=gen).to(DT[dtype])
    orig = qkv.clone()
    # two sequences, the second one padding-free but short; one padding token in the middle
    pos = torch.cat([torch.arange(0, 250), torch.arange(0, 50)]).to(torch.int32).cuda()
    seq = torch.cat([torch.zeros(250), torch.ones(50)]).to(torch.int32).cuda()
    seq[123] = -1
    pages = torch.tensor([[5, 0, 3, 6], [2, -1, -1, -1]], dtype=torch.int32, device="cuda")
    inv = torch.from_numpy(P.rope_inv_freq(hd, 54321.0)).cuda()
    kc, vc = paged(7, nkv, hd, dtype)
    k.rope_store(qkv, inv, hd, seq, pos, pages, 64, kc, vc, nh, nkv, hd, True)
    # the same in pieces of fewer than 256 tokens
    q2 = orig.clone()
    kc2, vc2 = paged(7, nkv, hd, dtype)
    for a in range(0, T, 100):
        k.rope_store(q2[a:a + 100], inv, hd, seq[a:a + 100].contiguous(), pos[a:a + 100].contiguous(), pages, 64, kc2, vc2,
                     nh, nkv, hd, True)
    assert torch.equal(qkv, q2)
    assert torch.equal(torch.nan_to_num(kc.float(), nan=-7.0), torch.nan_to_num(kc2.float(), nan=-7.0))
    assert torch.equal(torch.nan_to_num(vc.float(), nan=-7.0), torch.nan_to_num(vc2.float(), nan=-7.0))
    assert torch.equal(qkv[123], orig[123])
    assert int(torch.isfinite(kc.float()).sum()) == 299 * nkv * hd
    o = orig.double().cpu().numpy()
    invn = P.rope_inv_freq(hd, 54321.0)
    tol = 2e-6 if dtype == "float32" else 5e-3
    for t in (0, 1, 63, 64, 200, 249, 250, 299):
        q = P.rope(o[t, :nh * hd].reshape(1, nh, hd), [int(pos[t])], invn)
        kk = P.rope(o[t, nh * hd:(nh + nkv) * hd].reshape(1, nkv, hd), [int(pos[t])], invn)
        page = int(pages[int(seq[t]), int(pos[t]) // 64])
        assert rel(qkv[t, :nh * hd].reshape(nh, hd), torch.from_numpy(q[0])) < tol
        assert rel(kc[page, :, int(pos[t]) % 64], torch.from_numpy(kk[0])) < tol
        assert torch.equal(vc[page, :, int(pos[t]) % 64].double().cpu(),
                           torch.from_numpy(o[t, (nh + nkv) * hd:].reshape(nkv, hd)))


@pytest.mark.parametrize("T,H,K1,M2,mode2", [(5, 320, 192, 96, 0), (8, 2048, 128, 512, 3), (13, 192, 448, 64, 1), (1, 64, 64, 48, 2),
                                             (24, 576, 1536, 1728, 0), (32, 960, 128, 256, 3),
                                             (20, 2048, 128, 6144, 0),      # a reader too large to scale
                                             (64, 576, 1536, 1728, 0), (40, 576, 576, 3072, 3)])
def test_deferred_norm_between_two_products(T, H, K1, M2, mode2):
    """A norm split over the products around it: the first (residual add) also writes weight*x and the tiles'
    sums of squares, the second scales its accumulators.  Against the plain formulas in float64."""
    kk = K()
    gen = torch.Generator(device="cuda").manual_seed(T * H)
    a = torch.randn(T, K1, device="cuda", generator=gen).to(torch.bfloat16)
    w1 = (torch.randn(H, K1, device="cuda", generator=gen) * 0.1).to(torch.bfloat16)
    b1 = torch.randn(H, device="cuda", generator=gen) * 0.1
    x = torch.randn(T, H, device="cuda", generator=gen) * 2
    nw = 1 + 0.2 * torch.randn(H, device="cuda", generator=gen)
    w2 = (torch.randn(M2, H, device="cuda", generator=gen) * 0.1).to(torch.bfloat16)
    eps = 3e-5
    x_ref = x.double() + a.double() @ w1.double().T + b1.double()
    d = kk.DeferredNorm(nw, eps, torch.full((T, H), float("nan"), device="cuda", dtype=torch.bfloat16),
                        torch.full(((H + 15) // 16, kk.DeferredNorm.SS_STRIDE), float("nan"), device="cuda"))
    assert kk.linear(a, w1, x, b1, kk.OUT_ADD_F32, then_norm=d)
    assert rel(x, x_ref) < 1e-6 * 50
    assert rel(d.h, nw.double() * x_ref) < 5e-3
    assert rel(d.ss[:, :T].sum(0), (x_ref ** 2).sum(1)) < 1e-5
    normed = nw.double() * (x_ref / torch.sqrt((x_ref ** 2).mean(1, keepdim=True) + eps))
    if mode2 == 3:
        out = torch.empty(T, M2 // 2, device="cuda", dtype=torch.bfloat16)
        kk.gemm_bf16(d, w2, out, None, kk.OUT_SWIGLU)
        y = normed @ w2.double().T
        g, u = y[:, 0::2], y[:, 1::2]
        ref = g / (1 + torch.exp(-g)) * u
    elif mode2 == 2:
        out = torch.ones(T, M2, device="cuda")
        kk.linear(d, w2, out, None, kk.OUT_ADD_F32)
        ref = 1 + normed @ w2.double().T
    else:
        out = torch.empty(T, M2, device="cuda", dtype=torch.bfloat16 if mode2 == 0 else torch.float32)
        b2 = torch.randn(M2, device="cuda", generator=gen)
        kk.linear(d, w2, out, b2, mode2)
        ref = normed @ w2.double().T + b2.double()
    kk.check_device_errors("cuda:0")
    assert rel(out, ref) < 1e-2
    # and against the norm kernel followed by the same product: the same up to the rounding of h
    hn = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    kk.rmsnorm(x, nw, hn, eps)
    if mode2 in (0, 1):
        out2 = torch.empty_like(out)
        kk.linear(hn, w2, out2, b2, mode2)
        assert rel(out, out2) < 1e-2


def P_inv(hd, theta=23456.0):
    return P.rope_inv_freq(hd, theta)


def plain_attention_rows(q, keys, vals, group, scale, window):
    """q [nh, hd] at the last position of keys/vals [n, nkv, hd]."""
    out = np.zeros_like(q)
    n = keys.shape[0]
    lo = max(0, n - window) if window > 0 else 0
    for h in range(q.shape[0]):
        s = (keys[lo:, h // group] @ q[h]) * scale
        out[h] = P.softmax(s) @ vals[lo:, h // group]
    return out


def plain_attention_all(q, keys, vals, base, group, scale, window):
    """Causal attention of queries q [n, nh, hd] at positions base .. base + n - 1 over keys/vals [base + n, nkv, hd]:
    scores, mask by position (and window), softmax and weighted sum written out with matrix products, in float64."""
    n, nh, hd = q.shape
    tot = keys.shape[0]
    out = np.zeros_like(q)
    qpos = base + np.arange(n)[:, None]
    kpos = np.arange(tot)[None, :]
    seen = kpos <= qpos
    if window > 0:
        seen &= kpos > qpos - window
    for h in range(nh):
        s = (q[:, h] @ keys[:, h // group].T) * scale
        s = np.where(seen, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (e / e.sum(axis=1, keepdims=True)) @ vals[:, h // group]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 2, 48, 0), (5, 1, 24, 0), (4, 4, 128, 0), (2, 2, 16, 0),
                                               (6, 3, 32, 100), (3, 1, 256, 0)])
def test_attention_generic_ragged(dtype, nh, nkv, hd, window):
    """Tokens of three sequences at scattered positions, pages in scrambled order."""
    k = K()
    rng = np.random.default_rng(0)
    lens = [1, 150, 333]
    n_pages = 12
    kc, vc = paged(n_pages, nkv, hd, dtype)
    perm = rng.permutation(n_pages).tolist()
    pages = torch.full((3, 6), -1, dtype=torch.int32)
    store = []
    for s, n in enumerate(lens):
        keys = torch.randn(n, nkv, hd).to(DT[dtype])
        vals = torch.randn(n, nkv, hd).to(DT[dtype])
        store.append((keys, vals))
        for p in range((n + 63) // 64):
            pg = perm.pop()
            pages[s, p] = pg
            m = min(64, n - 64 * p)
            kc[pg, :, :m] = keys[64 * p:64 * p + m].transpose(0, 1).cuda()
            vc[pg, :, :m] = vals[64 * p:64 * p + m].transpose(0, 1).cuda()
    toks = [(0, 0), (1, 0), (1, 63), (1, 64), (1, 149), (2, 332), (2, 100), (-1, 0), (2, 31), (2, 32)]
    T = len(toks)
    q = torch.randn(T, nh * hd + 8).to(DT[dtype]).cuda()
    out = torch.empty(T, nh * hd, device="cuda", dtype=DT[dtype])
    seq = torch.tensor([t[0] for t in toks], dtype=torch.int32, device="cuda")
    pos = torch.tensor([t[1] for t in toks], dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(hd)
    k.attention_generic(q[:, :nh * hd], out, kc, vc, seq, pos, pages.cuda(), 64, nh, nkv, hd, scale, window)
    for t, (s, p) in enumerate(toks):
        if s < 0:
            assert (out[t] == 0).all()
            continue
        keys, vals = store[s]
        ref = plain_attention_rows(q[t, :nh * hd].double().cpu().numpy().reshape(nh, hd), keys[:p + 1].double().numpy(),
                                   vals[:p + 1].double().numpy(), nh // nkv, scale, window)
        assert rel(out[t].reshape(nh, hd), torch.from_numpy(ref)) < (2e-6 if dtype == "float32" else 1e-2), (t, s, p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_far_key_and_window_edge(dtype):
    """One key among hundreds is made to dominate: the output must be its value — unless a window
    excludes it by exactly one position."""
    k = K()
    nh = nkv = 2
    hd = 32
    n = 700
    kc, vc = paged(12, nkv, hd, dtype)
    keys = torch.randn(n, nkv, hd) * 0.1
    vals = torch.randn(n, nkv, hd)
    q = torch.randn(1, nh * hd) * 0.1
    far = 3
    keys[far, 0] = 40 * q[0, :hd] / q[0, :hd].norm() ** 2 * math.sqrt(hd)      # score 40 for head 0 at key 3
    keys, vals, q = keys.to(DT[dtype]), vals.to(DT[dtype]), q.to(DT[dtype]).cuda()
    pages = torch.arange(11, dtype=torch.int32).flip(0).reshape(1, 11).contiguous()
    for p in range(11):
        m = min(64, n - 64 * p)
        kc[int(pages[0, p]), :, :m] = keys[64 * p:64 * p + m].transpose(0, 1).cuda()
        vc[int(pages[0, p]), :, :m] = vals[64 * p:64 * p + m].transpose(0, 1).cuda()
    seq = torch.zeros(1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([n - 1], dtype=torch.int32, device="cuda")
    out = torch.empty(1, nh * hd, device="cuda", dtype=DT[dtype])
    scale = 1 / math.sqrt(hd)
    k.attention_generic(q, out, kc, vc, seq, pos, pages.cuda(), 64, nh, nkv, hd, scale, 0)
    assert rel(out[0, :hd], vals[far, 0]) < 2e-2                  # head 0 sees the far key
    for window, sees in ((n - far, True), (n - far - 1, False)):  # the window's edge, one position either way
        k.attention_generic(q, out, kc, vc, seq, pos, pages.cuda(), 64, nh, nkv, hd, scale, window)
        ref = plain_attention_rows(q.double().cpu().numpy().reshape(nh, hd), keys.double().numpy(), vals.double().numpy(),
                                   1, scale, window)
        assert rel(out.reshape(nh, hd), torch.from_numpy(ref)) < (2e-6 if dtype == "float32" else 1e-2)
        assert (rel(out[0, :hd], vals[far, 0]) < 2e-2) == sees


def test_argmax_first_maximum():
    x = torch.randn(5, 1003, device="cuda")
    x[0, 17] = x[0, 900] = 50.0
    x[1, 1002] = 60.0
    x[2] = -3.0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    K().argmax(x, out)
    assert out.tolist() == [17, 1002, 0, int(x[3].argmax()), int(x[4].argmax())]


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.8, 40, 1.0), (0.7, 0, 0.9), (1.5, 10, 0.3),
                                                     (0.3, 1, 1.0), (1.0, 0, 0.001), (2.0, 5000, 0.95)])
def test_sample_matches_plain(temperature, top_k, top_p):
    torch.manual_seed(1)
    V = 3001
    logits = torch.randn(8, V, device="cuda") * 2.5
    logits[3, 100] = logits[3, 2000] = logits[3, 7] = 9.0          # exact ties at the top
    u = torch.tensor([0.0001, 0.2, 0.5, 0.6, 0.77, 0.9, 0.999, 0.31], dtype=torch.float64, device="cuda")
    out = torch.empty(8, dtype=torch.int32, device="cuda")
    K().sample(logits, temperature, top_k, top_p, u, torch.empty(8, V, device="cuda"), out)
    ref = [P.sample(logits[i].cpu().numpy(), temperature, top_k, top_p, float(u[i])) for i in range(8)]
    assert out.tolist() == ref
    for i, tok in enumerate(out.tolist()):                      # draws stay in the filtered set
        assert P.sampling_probabilities(logits[i].cpu().numpy(), temperature, top_k, top_p)[tok] > 0


@pytest.mark.parametrize("rows", ["A", "B", "ties"])
def test_sample_follows_the_reference_librarys_distribution(rows):
    """The device sampler against the probabilities recorded from the reference's own library
    (tests/golden/make_golden.py: llmi::sampling_probabilities, src/model/sampling.cpp:11-58; exact ties included):
    for a grid of uniform numbers every draw is the first id, in ascending order, at which the recorded cumulative
    probability reaches the number (src/model/sampling.cpp:60-76) — so no token outside the recorded support is ever
    drawn, and none inside it is skipped."""
    import os
    from golden import make_golden as G
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_tiny.npz"))
    logits = gold[f"sampling_{rows}_logits"]
    R, V = logits.shape
    grid = np.concatenate([np.linspace(0.0005, 0.9995, 400), [1e-9, 1 - 1e-9]])
    for i, (temperature, top_k, top_p) in enumerate(G.SAMPLING):
        ref = gold[f"sampling_{rows}_{i}"].astype(np.float64)
        for r in range(R):
            dev = torch.from_numpy(np.repeat(logits[r:r + 1], len(grid), 0)).cuda()
            u = torch.from_numpy(grid).cuda()
            out = torch.empty(len(grid), dtype=torch.int32, device="cuda")
            if temperature <= 0:
                K().argmax(dev, out)
            else:
                K().sample(dev, temperature, top_k, top_p, u, torch.empty(len(grid), V, device="cuda"), out)
            got = out.cpu().numpy()
            cum = np.cumsum(ref[r])
            assert (ref[r][got] > 0).all(), (rows, i, r)
            for g, x in zip(got, grid):
                want = int(np.nonzero((cum >= x) & (ref[r] > 0))[0][0]) if (cum >= x).any() else int(np.nonzero(ref[r] > 0)[0][-1])
                assert g == want or np.min(np.abs(cum - x)) < 2e-6, (rows, i, r, x, g, want)


def test_sample_distribution():
    """Many draws from one row follow the filtered distribution."""
    torch.manual_seed(2)
    V, n = 50, 4000
    row = torch.randn(V) * 2
    logits = row.repeat(n, 1).cuda()
    u = torch.rand(n, dtype=torch.float64, device="cuda")
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    K().sample(logits, 0.9, 12, 0.92, u, torch.empty(n, V, device="cuda"), out)
    p = P.sampling_probabilities(row.numpy(), 0.9, 12, 0.92)
    freq = np.bincount(out.cpu().numpy(), minlength=V) / n
    assert set(np.nonzero(freq)[0]) <= set(np.nonzero(p)[0])
    assert np.abs(freq - p).max() < 0.03


@pytest.mark.parametrize("n_tok,m_out,k", [(1, 200, 72), (5, 64, 64), (16, 128, 64), (17, 384, 120), (70, 129, 1000),
                                           (300, 520, 136), (64, 2048, 8192), (8, 256, 4096), (1000, 136, 264),
                                           (33, 300, 2048), (100, 2048, 2048), (20, 640, 512), (128, 136, 1024),
                                           (600, 1100, 320), (1500, 700, 1088), (512, 256, 64), (256, 2048, 2048),
                                           (300, 2048, 1024), (511, 6144, 512), (256, 16384, 256), (384, 1024, 4096),
                                           (511, 6150, 512), (130, 2048, 8192), (48, 6144, 2048)])
def test_gemm_tc_all_modes(n_tok, m_out, k):
    """The tcgen05 product against fp64 on ragged shapes, with and without split-K."""
    kk = K()
    torch.manual_seed(n_tok + m_out + k)
    x = torch.randn(n_tok, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(m_out, k, device="cuda") * 0.05).to(torch.bfloat16)
    b = torch.randn(m_out, device="cuda")
    ref = x.double() @ w.double().T
    y32 = torch.full((n_tok, m_out), float("nan"), device="cuda")
    kk.gemm_tc(x, w, y32, None, kk.OUT_STORE_F32)
    assert rel(y32, ref) < 2e-5
    y = torch.empty(n_tok, m_out, device="cuda", dtype=torch.bfloat16)
    kk.gemm_tc(x, w, y, b, kk.OUT_STORE)
    assert rel(y, ref + b.double()) < 6e-3
    acc = torch.randn(n_tok, m_out, device="cuda")
    before = acc.clone()
    kk.gemm_tc(x, w, acc, None, kk.OUT_ADD_F32)
    assert rel(acc, before.double() + ref) < 2e-5
    # the same rows whatever else is in the call (a row's value does not depend on the batch)
    y1 = torch.empty(1, m_out, device="cuda")
    kk.gemm_tc(x[n_tok - 1:], w, y1, None, kk.OUT_STORE_F32)
    if kk.lib().llmi_gemm_tc_k_per_cta(n_tok, m_out, k) == kk.lib().llmi_gemm_tc_k_per_cta(1, m_out, k):
        assert torch.equal(y1, y32[n_tok - 1:])
    else:
        assert rel(y1, y32[n_tok - 1:]) < 1e-5
    kk.check_device_errors("cuda:0")
    assert int(kk.tc_scratch("cuda:0").tickets.abs().sum()) == 0


def test_gemm_tc_strided_input_and_refusals():
    kk = K()
    wide = torch.randn(40, 64 + 2 * 64, device="cuda").to(torch.bfloat16)
    w = torch.randn(96, 64, device="cuda").to(torch.bfloat16)
    y = torch.empty(40, 96, device="cuda")
    kk.gemm_tc(wide[:, 64:128], w, y, None, kk.OUT_STORE_F32)
    assert rel(y, wide[:, 64:128].double() @ w.double().T) < 2e-5
    assert not kk.gemm_tc_eligible(torch.empty(4, 20, device="cuda", dtype=torch.bfloat16), w)       # pitch of 40 bytes
    with pytest.raises(kk.KernelError, match="aligned"):
        kk.gemm_tc(torch.empty(4, 20, device="cuda", dtype=torch.bfloat16), torch.empty(8, 20, device="cuda", dtype=torch.bfloat16),
                   torch.empty(4, 8, device="cuda"), None, kk.OUT_STORE_F32)


@pytest.mark.parametrize("lens,nh,nkv,hd", [([2048], 32, 8, 128), ([1500, 548], 32, 8, 128), ([2048], 32, 32, 64)])
def test_attention_prefill_many_blocks_again_and_again(lens, nh, nkv, hd):
    """More (query block, head) jobs than blocks are resident, so that the short query blocks start beside busy
    ones: every launch of many gives the bits of the first, and the first query block (two pages, the job that came
    out wrong now and then when a softmax thread's wait on the finished products could pass two phases behind)
    agrees with the plain formula."""
    kk = K()
    torch.manual_seed(5)
    T, S = sum(lens), len(lens)
    Pg = max((n + 63) // 64 for n in lens)
    kc, vc = paged(S * Pg, nkv, hd, "bfloat16")
    pages = torch.randperm(S * Pg, dtype=torch.int32).reshape(S, Pg)
    keys = [torch.randn(n, nkv, hd).to(torch.bfloat16) for n in lens]
    vals = [torch.randn(n, nkv, hd).to(torch.bfloat16) for n in lens]
    for s_, n in enumerate(lens):
        for pg_i in range((n + 63) // 64):
            m_ = min(64, n - 64 * pg_i)
            kc[pages[s_, pg_i], :, :m_] = keys[s_][64 * pg_i:64 * pg_i + m_].transpose(0, 1).cuda()
            vc[pages[s_, pg_i], :, :m_] = vals[s_][64 * pg_i:64 * pg_i + m_].transpose(0, 1).cuda()
    qkv = torch.randn(T, (nh + 2 * nkv) * hd).to(torch.bfloat16).cuda()
    out = torch.zeros(T, nh * hd, device="cuda", dtype=torch.bfloat16)
    starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    qstart = torch.from_numpy(starts).cuda()
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    nqb = sum((n + 127) // 128 for n in lens)
    scale = 1 / math.sqrt(hd)

    def launch():
        kk.attention_prefill_tc(qkv, out, kc, vc, pages.cuda(), qstart, kvlen, nqb, nh, nkv, hd, scale, 0, None)
    launch()
    first = out.clone()
    for _ in range(60):
        out.zero_()
        launch()
        assert torch.equal(out, first)
    kk.check_device_errors("cuda:0")
    for s_, n in enumerate(lens):          # the first query block of every sequence against the plain formula
        rows = min(128, n)
        for r in (0, 1, 63, 64, rows - 1):
            q = qkv[starts[s_] + r, :nh * hd].double().cpu().numpy().reshape(nh, hd)
            ref = plain_attention_rows(q, keys[s_][:r + 1].double().numpy(), vals[s_][:r + 1].double().numpy(), nh // nkv, scale, 0)
            assert rel(first[starts[s_] + r].reshape(nh, hd), torch.from_numpy(ref)) < 1e-2, (s_, r)


DECODE_SHAPES = [("simt", 32, 32, 64), ("simt", 15, 5, 64), ("simt", 8, 2, 128), ("simt", 8, 8, 32), ("simt", 16, 2, 64),
                 ("mma", 15, 5, 64), ("mma", 8, 2, 128), ("mma", 16, 2, 64), ("mma", 28, 4, 128), ("mma", 32, 2, 64),
                 ("mma", 12, 1, 128), ("mma", 10, 5, 64), ("mma", 3, 3, 64)]


def decode_kernel(kk, kernel):
    """(unfused, fused) launchers of one of the two decode kernels, with the same arguments."""
    if kernel == "simt":
        return kk.attention_decode, kk.attention_decode_fused

    def plain(q, out, kc, vc, pages, kvlen, qstart, nh, nkv, hd, scale, window, part, pps):
        kk.attention_decode_mma(q, out, kc, vc, pages, kvlen, qstart, nh, nkv, hd, scale, window, part, pps, None)

    def fused(q, out, kc, vc, pages, kvlen, qstart, nh, nkv, hd, scale, window, part, pps, inv, rdim, write):
        kk.attention_decode_mma(q, out, kc, vc, pages, kvlen, qstart, nh, nkv, hd, scale, window, part, pps, (inv, rdim, write))

    return plain, fused


@pytest.mark.parametrize("kernel,nh,nkv,hd", DECODE_SHAPES)
@pytest.mark.parametrize("pps,window", [(1, 0), (4, 0), (64, 0), (2, 200)])
def test_attention_decode_ragged(kernel, nh, nkv, hd, pps, window):
    """The split decode kernels (CUDA cores; tensor cores for grouped queries) against the plain formula: sequences
    of very different lengths, a padding sequence, scrambled pages, poisoned cache outside the sequences,
    several split sizes."""
    kk = K()
    attend, _ = decode_kernel(kk, kernel)
    rng = np.random.default_rng(1)
    lens = [1, 64, 65, 700, 0, 129, 1000]
    P = 16
    n_pages = 48
    kc, vc = paged(n_pages, nkv, hd, "bfloat16")
    perm = rng.permutation(n_pages).tolist()
    pages = torch.full((len(lens), P), -1, dtype=torch.int32)
    store = []
    for s_, n in enumerate(lens):
        keys = torch.randn(max(n, 1), nkv, hd).to(torch.bfloat16)
        vals = torch.randn(max(n, 1), nkv, hd).to(torch.bfloat16)
        store.append((keys, vals))
        for pg_i in range((n + 63) // 64):
            pg = perm.pop()
            pages[s_, pg_i] = pg
            m_ = min(64, n - 64 * pg_i)
            kc[pg, :, :m_] = keys[64 * pg_i:64 * pg_i + m_].transpose(0, 1).cuda()
            vc[pg, :, :m_] = vals[64 * pg_i:64 * pg_i + m_].transpose(0, 1).cuda()
    S = len(lens)
    q = torch.randn(S, (nh + 2 * nkv) * hd).to(torch.bfloat16).cuda()
    out = torch.full((S, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qstart = torch.arange(S, dtype=torch.int32, device="cuda")
    part = torch.empty(kk.attention_decode_workspace(S, nh, hd, P, pps), device="cuda")
    scale = 1 / math.sqrt(hd)
    for _ in range(2):          # twice: the tickets must come back to zero
        attend(q, out, kc, vc, pages.cuda(), kvlen, qstart, nh, nkv, hd, scale, window, part, pps)
    kk.check_device_errors("cuda:0")
    assert int(kk.tc_scratch("cuda:0").attn_tickets.abs().sum()) == 0
    for s_, n in enumerate(lens):
        if n == 0:
            assert (out[s_] == 7.0).all()          # a padding sequence is not touched
            continue
        keys, vals = store[s_]
        ref = plain_attention_rows(q[s_, :nh * hd].double().cpu().numpy().reshape(nh, hd), keys[:n].double().numpy(),
                                   vals[:n].double().numpy(), nh // nkv, scale, window)
        assert rel(out[s_].reshape(nh, hd), torch.from_numpy(ref)) < 1e-2, (s_, n)


@pytest.mark.parametrize("nh,hd", [(4, 64), (3, 128), (6, 32), (32, 64)])
@pytest.mark.parametrize("cluster,window", [(2, 0), (4, 0), (8, 0), (4, 200), (8, 300)])
def test_attention_decode_cluster_form_same_bits(nh, hd, cluster, window):
    """The decode kernel run as clusters (one cluster of 2, 4 or 8 blocks per sequence-head, the splits' results
    meeting in the first block's shared memory) gives the bits of its persistent form with the same split: sequences of
    very different lengths (splits that hold nothing, also the FIRST one under a window), a padding sequence,
    position encoding fused in or not; and the plain formula's values."""
    kk = K()
    rng = np.random.default_rng(4)
    lens = [1, 64, 65, 700, 0, 129, 1000, 128, 1024]       # lengths AFTER this step (0: padding)
    P, n_pages = 16, 80
    pps = P // cluster
    gen = torch.Generator().manual_seed(5)
    kc, vc = paged(n_pages, nh, hd, "bfloat16")
    perm = rng.permutation(n_pages).tolist()
    pages = torch.full((len(lens), P), -1, dtype=torch.int32)
    for s_, n in enumerate(lens):
        for pg_i in range((n + 63) // 64):
            pg = perm.pop()
            pages[s_, pg_i] = pg
            m_ = min(64, n - 1 - 64 * pg_i)
            if m_ > 0:
                kc[pg, :, :m_] = torch.randn(nh, m_, hd, generator=gen).to(torch.bfloat16).cuda()
                vc[pg, :, :m_] = torch.randn(nh, m_, hd, generator=gen).to(torch.bfloat16).cuda()
    S = len(lens)
    qkv = torch.randn(S, 3 * nh * hd, generator=gen).to(torch.bfloat16).cuda()
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qstart = torch.arange(S, dtype=torch.int32, device="cuda")
    inv = torch.from_numpy(P_inv(hd)).cuda()
    scale = 1 / math.sqrt(hd)
    part = torch.empty(kk.attention_decode_workspace(S, nh, hd, P, pps), device="cuda")
    pages_d = pages.cuda()
    outs, caches = [], []
    for form in (0, cluster):
        k1, v1 = kc.clone(), vc.clone()
        out = torch.full((S, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
        for _ in range(2):
            kk.attention_decode_fused(qkv, out, k1, v1, pages_d, kvlen, qstart, nh, nh, hd, scale, window, part, pps, inv, hd,
                                      True, cluster=form)
        kk.check_device_errors("cuda:0")
        outs.append(out)
        caches.append((k1, v1))
    assert torch.equal(outs[0], outs[1])
    for a, b in zip(caches[0], caches[1]):
        assert torch.equal(torch.nan_to_num(a.float(), nan=-7.0), torch.nan_to_num(b.float(), nan=-7.0))
    assert (outs[1][4] == 7.0).all()                        # the padding sequence is not touched
    # without the fused position encoding, over the caches that the run above has filled
    k1, v1 = caches[1]
    q_rot = qkv.clone()
    tok_seq = torch.tensor([i if n > 0 else -1 for i, n in enumerate(lens)], dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor([max(n - 1, 0) for n in lens], dtype=torch.int32, device="cuda")
    kk.rope_store(q_rot, inv, hd, tok_seq, tok_pos, pages_d, 64, k1.clone(), v1.clone(), nh, nh, hd, True)
    plain = []
    for form in (0, cluster):
        out = torch.full((S, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
        kk.attention_decode(q_rot, out, k1, v1, pages_d, kvlen, qstart, nh, nh, hd, scale, window, part, pps, cluster=form)
        plain.append(out)
    kk.check_device_errors("cuda:0")
    assert torch.equal(plain[0], plain[1]) and torch.equal(plain[1], outs[1])
    assert int(kk.tc_scratch("cuda:0").attn_tickets.abs().sum()) == 0
    for s_, n in enumerate(lens):                           # and the plain formula
        if n == 0:
            continue
        keys = torch.stack([k1[pages[s_, i // 64], :, i % 64] for i in range(n)]).double().cpu().numpy()
        vals = torch.stack([v1[pages[s_, i // 64], :, i % 64] for i in range(n)]).double().cpu().numpy()
        ref = plain_attention_rows(q_rot[s_, :nh * hd].double().cpu().numpy().reshape(nh, hd), keys, vals, 1, scale, window)
        assert rel(outs[1][s_].reshape(nh, hd), torch.from_numpy(ref)) < 1e-2, (s_, n)


@pytest.mark.parametrize("nh,hd,S,P,cluster", [(32, 64, 1, 16, 8), (32, 64, 3, 8, 4), (8, 128, 2, 32, 8)])
def test_attention_decode_cluster_form_again_and_again(nh, hd, S, P, cluster):
    """The cluster form launched 120 times between other kernels (programmatic dependents, so neighbours overlap):
    every launch gives the first one's bits."""
    kk = K()
    torch.manual_seed(0)
    pps = -(-P // cluster)
    n_pages = S * P + 3
    kc = torch.randn(n_pages, nh, 64, hd, device="cuda").to(torch.bfloat16)
    vc = torch.randn(n_pages, nh, 64, hd, device="cuda").to(torch.bfloat16)
    pages = torch.randperm(n_pages)[:S * P].to(torch.int32).reshape(S, P).cuda()
    kvlen = torch.tensor([P * 64 - 7 * i - 1 for i in range(S)], dtype=torch.int32, device="cuda")
    qstart = torch.arange(S, dtype=torch.int32, device="cuda")
    qkv = torch.randn(S, 3 * nh * hd, device="cuda").to(torch.bfloat16)
    inv = torch.from_numpy(P_inv(hd)).cuda()
    part = torch.empty(kk.attention_decode_workspace(S, nh, hd, P, pps), device="cuda")
    x = torch.randn(8, 2048, device="cuda").to(torch.bfloat16)
    w = torch.randn(2048, 2048, device="cuda").to(torch.bfloat16)
    y = torch.empty(8, 2048, device="cuda", dtype=torch.bfloat16)
    first, differ = None, 0
    for _ in range(120):
        out = torch.full((S, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
        kk.gemm_skinny(x, w, y)
        kk.attention_decode_fused(qkv, out, kc, vc, pages, kvlen, qstart, nh, nh, hd, 1 / math.sqrt(hd), 0, part, pps, inv, hd,
                                  True, cluster=cluster)
        kk.gemm_skinny(x, w, y)
        if first is None:
            first = out.clone()
        elif not torch.equal(out, first):
            differ += 1
    kk.check_device_errors("cuda:0")
    assert differ == 0 and bool(torch.isfinite(first.float()).all())


@pytest.mark.parametrize("kernel,nh,nkv,hd", DECODE_SHAPES)
@pytest.mark.parametrize("pps,window,rot,write", [(1, 0, True, True), (4, 0, True, True), (64, 0, False, True),
                                                  (2, 200, True, True), (4, 0, True, False)])
def test_attention_decode_fused_rotation_same_bits(kernel, nh, nkv, hd, pps, window, rot, write):
    """A decode kernel with the position encoding fused in (q rotated on the fly, the new k and v appended
    by the block that reads their page) gives the bits of the two kernels it replaces: outputs and caches."""
    kk = K()
    attend, attend_fused = decode_kernel(kk, kernel)
    rng = np.random.default_rng(2)
    lens = [1, 64, 65, 700, 0, 129, 1000, 128]       # lengths AFTER this step (0: padding)
    P, n_pages = 16, 56
    gen = torch.Generator().manual_seed(3)
    kc, vc = paged(n_pages, nkv, hd, "bfloat16")
    perm = rng.permutation(n_pages).tolist()
    pages = torch.full((len(lens), P), -1, dtype=torch.int32)
    for s_, n in enumerate(lens):
        for pg_i in range((n + 63) // 64):
            pg = perm.pop()
            pages[s_, pg_i] = pg
            m_ = min(64, n - 1 - 64 * pg_i)           # positions before the newest one are in the cache already
            if m_ > 0:
                kc[pg, :, :m_] = torch.randn(nkv, m_, hd, generator=gen).to(torch.bfloat16).cuda()
                vc[pg, :, :m_] = torch.randn(nkv, m_, hd, generator=gen).to(torch.bfloat16).cuda()
    S = len(lens)
    qkv = torch.randn(S, (nh + 2 * nkv) * hd, generator=gen).to(torch.bfloat16).cuda()
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qstart = torch.arange(S, dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([i if n > 0 else -1 for i, n in enumerate(lens)], dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor([max(n - 1, 0) for n in lens], dtype=torch.int32, device="cuda")
    inv = torch.from_numpy(P_inv(hd)).cuda() if rot else None
    rdim = hd if rot else 0
    scale = 1 / math.sqrt(hd)
    part = torch.empty(kk.attention_decode_workspace(S, nh, hd, P, pps), device="cuda")
    pages_d = pages.cuda()
    # two kernels: rotate and append, then attend
    q2, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
    out2 = torch.full((S, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
    kk.rope_store(q2, inv, rdim, tok_seq, tok_pos, pages_d, 64, kc2, vc2, nh, nkv, hd, True)
    attend(q2, out2, kc2, vc2, pages_d, kvlen, qstart, nh, nkv, hd, scale, window, part, pps)
    # one kernel (write=False: the cache holds the new entries already, as for a call that reads another call's cache)
    q1 = qkv.clone()
    kc1, vc1 = (kc.clone(), vc.clone()) if write else (kc2.clone(), vc2.clone())
    out1 = torch.full((S, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):      # a second run over the cache it has written itself gives the same
        attend_fused(q1, out1, kc1, vc1, pages_d, kvlen, qstart, nh, nkv, hd, scale, window, part, pps, inv, rdim, write)
    kk.check_device_errors("cuda:0")
    assert torch.equal(q1, qkv)                                  # the fused kernel leaves its input alone
    assert torch.equal(out1, out2)
    assert torch.equal(torch.nan_to_num(kc1.float(), nan=-7.0), torch.nan_to_num(kc2.float(), nan=-7.0))
    assert torch.equal(torch.nan_to_num(vc1.float(), nan=-7.0), torch.nan_to_num(vc2.float(), nan=-7.0))
    assert int(kk.tc_scratch("cuda:0").attn_tickets.abs().sum()) == 0


@pytest.mark.parametrize("kernel", ["mma", "tc", "tc-split2", "tc-split3"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 4, 64, 0), (6, 2, 64, 0), (4, 1, 128, 0), (3, 3, 64, 100), (2, 2, 128, 70)])
def test_attention_prefill_ragged(nh, nkv, hd, window, kernel):
    """The flash prompt kernel against the plain formula: prompts of 1..600 tokens in one launch, one of
    them continuing a sequence that already holds 300 positions, scrambled pages, a poisoned cache."""
    kk = K()
    run = kk.attention_prefill_tc if kernel.startswith("tc") else kk.attention_prefill
    rng = np.random.default_rng(2)
    q_lens = [1, 127, 128, 129, 600, 200]
    bases = [0, 0, 0, 0, 0, 300]
    P = 16
    n_pages = 64
    kc, vc = paged(n_pages, nkv, hd, "bfloat16")
    perm = rng.permutation(n_pages).tolist()
    S = len(q_lens)
    pages = torch.full((S, P), -1, dtype=torch.int32)
    store, qs, starts = [], [], [0]
    for s_, (n, b) in enumerate(zip(q_lens, bases)):
        tot = n + b
        keys = torch.randn(tot, nkv, hd).to(torch.bfloat16)
        vals = torch.randn(tot, nkv, hd).to(torch.bfloat16)
        store.append((keys, vals))
        for pg_i in range((tot + 63) // 64):
            pg = perm.pop()
            pages[s_, pg_i] = pg
            m_ = min(64, tot - 64 * pg_i)
            kc[pg, :, :m_] = keys[64 * pg_i:64 * pg_i + m_].transpose(0, 1).cuda()
            vc[pg, :, :m_] = vals[64 * pg_i:64 * pg_i + m_].transpose(0, 1).cuda()
        qs.append(torch.randn(n, nh * hd).to(torch.bfloat16))
        starts.append(starts[-1] + n)
    T = starts[-1]
    q = torch.zeros(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16)
    q[:, :nh * hd] = torch.cat(qs)
    q = q.cuda()
    out = torch.full((T, nh * hd), 7.0, device="cuda", dtype=torch.bfloat16)
    qstart = torch.tensor(starts, dtype=torch.int32, device="cuda")
    kvlen = torch.tensor([n + b for n, b in zip(q_lens, bases)], dtype=torch.int32, device="cuda")
    n_blocks = sum((n + 127) // 128 for n in q_lens)
    scale = 1 / math.sqrt(hd)
    if "split" in kernel:
        # the key range of every query block cut into jobs of 2 or 3 pages, merged by the last one to finish
        sp = int(kernel[-1])
        jobs = kk.prefill_split_jobs(q_lens, [n + b for n, b in zip(q_lens, bases)], window, sp)
        assert jobs > n_blocks
        ws = torch.full((jobs * nh * (hd + 2) * 128,), float("nan"), device="cuda")
        for _ in range(2):      # twice: the tickets must come back to zero
            run(q, out, kc, vc, pages.cuda(), qstart, kvlen, n_blocks, nh, nkv, hd, scale, window, (jobs, sp, ws))
        assert int(kk.tc_scratch("cuda:0").attn_tickets.abs().sum()) == 0
    else:
        run(q, out, kc, vc, pages.cuda(), qstart, kvlen, n_blocks, nh, nkv, hd, scale, window)
    kk.check_device_errors("cuda:0")
    assert torch.isfinite(out.float()).all()
    for s_, (n, b) in enumerate(zip(q_lens, bases)):
        keys, vals = store[s_]
        # every row of every sequence (a row past the first of a 128-row tile, or next to a page's end, is where a
        # wrong mask or a wrong page would show)
        ref = plain_attention_all(qs[s_].double().numpy().reshape(n, nh, hd), keys.double().numpy(), vals.double().numpy(),
                                  b, nh // nkv, scale, window)
        got = out[starts[s_]:starts[s_] + n].reshape(n, nh, hd).double().cpu().numpy()
        err = np.abs(got - ref).reshape(n, -1).max(axis=1) / np.abs(ref).max()
        assert err.max() < 1.5e-2, (s_, int(err.argmax()), float(err.max()))


@pytest.mark.parametrize("n_tok,inner,k", [(1, 100, 72), (8, 8192, 2048), (70, 176, 64), (300, 320, 120), (2048, 512, 256),
                                           (40, 1024, 1024), (24, 72, 2048), (100, 300, 768),
                                           (300, 9728, 128), (300, 9604, 128), (64, 8192, 2048)])
def test_gemm_tc_gated_epilogue(n_tok, inner, k):
    """silu(gate)·up finished inside the product, rows alternating gate and up; with and without split-K."""
    kk = K()
    x = torch.randn(n_tok, k, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(inner, k, device="cuda") * 0.1).to(torch.bfloat16)
    up = (torch.randn(inner, k, device="cuda") * 0.1).to(torch.bfloat16)
    w = torch.stack([gate, up], dim=1).reshape(2 * inner, k).contiguous()
    out = torch.full((n_tok, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
    kk.gemm_tc(x, w, out, None, kk.OUT_SWIGLU)
    g = x.double() @ gate.double().T
    u = x.double() @ up.double().T
    assert rel(out, g / (1 + torch.exp(-g)) * u) < 8e-3
    kk.check_device_errors("cuda:0")


@pytest.mark.parametrize("n_tok,m_out,k", [(16, 49152, 512), (12, 49152, 576), (16, 16384, 768), (8, 49152, 512), (32, 49152, 512)])
def test_gemm_skinny_many_short_row_tiles_again_and_again(n_tok, m_out, k):
    """Many row tiles per block, each of two or three stages, so that the ring of stages wraps around all the time
    while a block's warps are still reading: every launch of many must be right in every element.  (A stage that is
    handed back without ordering the warps' reads before the next copy's writes gave one wrong row tile in thousands
    in a third of the launches of the first shape — a head of 49,152 rows over a narrow model at batch 16.)"""
    kk = K()
    torch.manual_seed(k + n_tok)
    x = torch.randn(n_tok, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(m_out, k, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    scale = float(ref.abs().max())
    y = torch.empty(n_tok, m_out, device="cuda")
    worst = torch.zeros((), device="cuda")
    for _ in range(120):
        y.fill_(float("nan"))
        kk.gemm_skinny(x, w, y, None, kk.OUT_STORE_F32)
        worst = torch.maximum(worst, torch.nan_to_num((y - ref).abs().max(), nan=float("inf")))
    assert float(worst) / scale < 2e-5
    kk.check_device_errors("cuda:0")


@pytest.mark.parametrize("n_tok,m_out,k", [(1, 200, 64), (5, 64, 64), (8, 2048, 2048), (8, 130, 8192), (16, 384, 192),
                                           (17, 6144, 2048), (32, 520, 960), (3, 16, 320), (33, 1728, 576), (64, 576, 1536),
                                           (50, 130, 960), (64, 3072, 576)])
def test_gemm_skinny_all_modes(n_tok, m_out, k):
    """The weight-streaming product (at most 64 tokens) against fp64, ragged shapes, every epilogue."""
    kk = K()
    torch.manual_seed(n_tok * 7 + m_out + k)
    x = torch.randn(n_tok, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(m_out, k, device="cuda") * 0.05).to(torch.bfloat16)
    b = torch.randn(m_out, device="cuda")
    ref = x.double() @ w.double().T
    y32 = torch.full((n_tok, m_out), float("nan"), device="cuda")
    kk.gemm_skinny(x, w, y32, None, kk.OUT_STORE_F32)
    assert rel(y32, ref) < 2e-5
    y = torch.empty(n_tok, m_out, device="cuda", dtype=torch.bfloat16)
    kk.gemm_skinny(x, w, y, b, kk.OUT_STORE)
    assert rel(y, ref + b.double()) < 6e-3
    acc = torch.randn(n_tok, m_out, device="cuda")
    before = acc.clone()
    kk.gemm_skinny(x, w, acc, None, kk.OUT_ADD_F32)
    assert rel(acc, before.double() + ref) < 2e-5
    if m_out % 2 == 0:
        gated = torch.full((n_tok, m_out // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
        kk.gemm_skinny(x, w, gated, None, kk.OUT_SWIGLU)
        g, u = ref[:, 0::2], ref[:, 1::2]
        assert rel(gated, g / (1 + torch.exp(-g)) * u) < 8e-3
    # a row's value does not depend on how many tokens are in the call
    y1 = torch.empty(1, m_out, device="cuda")
    kk.gemm_skinny(x[n_tok - 1:], w, y1, None, kk.OUT_STORE_F32)
    assert torch.equal(y1, y32[n_tok - 1:])
    kk.check_device_errors("cuda:0")

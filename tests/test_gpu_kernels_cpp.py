"""Every CUDA kernel against its plain C++ counterpart (``synaptix_b200/csrc/reference.cpp``, run on the CPU with
the same arguments), at sizes other than the engine's: ragged widths, head sizes in steps of 16, windows, pages in
scrambled order with NaN in every unused row.  ``tests/test_reference_cpp.py`` ties the C++ functions to the plain
Python implementation."""
import math

import pytest
import torch

from synaptix_b200 import reference as R

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-5) if dtype == F32 else dict(atol=2e-2, rtol=2e-2)


def i32(x):
    return torch.as_tensor(x, dtype=torch.int32).cuda()


@pytest.mark.parametrize("dtype", [F32, BF])
def test_embedding_norm_residual_and_silu(dtype):
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(3)
    for H in (50, 100, 2052, 4100):
        E = torch.randn(77, H, generator=g).to(dtype)
        ids = torch.tensor([5, 76, 0, 99, -3, 41])
        assert torch.equal(ops.embed_gather(E.cuda(), i32(ids)).cpu(), R.embed_gather(E, ids))
        h = torch.randn(6, H, generator=g) * 2
        delta = torch.randn(6, H, generator=g).to(dtype)
        gain = 1 + 0.2 * torch.randn(H, generator=g)
        hc, hr = h.clone().cuda(), h.clone()
        y = ops.add_rmsnorm(hc, delta.cuda(), gain.cuda(), 3e-5, dtype)
        yr = R.add_rmsnorm(hr, delta, gain, 3e-5, dtype)
        assert torch.equal(hc.cpu(), hr) and torch.allclose(y.float().cpu(), yr.float(), **tol(dtype))
        rows = torch.tensor([5, 0, 3])
        y2 = ops.add_rmsnorm(h.clone().cuda(), delta.cuda(), gain.cuda(), 3e-5, dtype, rows=i32(rows))
        assert torch.allclose(y2.float().cpu(), R.add_rmsnorm(h.clone(), delta, gain, 3e-5, dtype, rows=rows, write_h=False).float(),
                              **tol(dtype))
        hc, hr = h.clone().cuda(), h.clone()
        ops.residual_add(hc, delta.cuda())
        R.residual_add(hr, delta)
        assert torch.equal(hc.cpu(), hr)
    gu = (torch.randn(9, 2 * 333, generator=g) * 3).to(dtype)
    assert torch.allclose(ops.silu_mul(gu.cuda()).float().cpu(), R.silu_mul(gu).float(), **tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 72, 96), (5, 200, 264), (16, 130, 64), (33, 136, 320), (100, 264, 1224), (128, 72, 8),
                                    (200, 300, 264)])
def test_every_matrix_product_against_the_cpp_loops(M, N, K):
    """The plain product in both dtypes, and whichever fast products take the size (mma.sync stream, tcgen05
    weight stream, tcgen05 tiles), with their epilogues."""
    from synaptix_b200 import ops
    from synaptix_b200.ops.decode import skinny_gemm, skinny_supported
    from synaptix_b200.ops.gemm_tc import gemm_tc
    from synaptix_b200.ops.gemm_ws import gemm_ws, ws_supported
    g = torch.Generator().manual_seed(M + N + K)
    x32 = torch.randn(M, K, generator=g)
    w32 = torch.randn(N, K, generator=g) * 2 / math.sqrt(K)
    want32 = R.gemm(x32, w32)
    assert torch.allclose(ops.gemm_generic(x32.cuda(), w32.cuda()).cpu(), want32, atol=2e-5 * math.sqrt(K), rtol=1e-5)
    x, w = x32.to(BF), w32.to(BF)
    want = R.gemm(x, w, F32)
    want_silu = R.silu_mul(want)
    assert torch.allclose(ops.gemm_generic(x.cuda(), w.cuda(), out_dtype=F32).cpu(), want, atol=2e-5 * math.sqrt(K), rtol=1e-5)
    fast = [("tiles", lambda **kw: gemm_tc(x.cuda(), w.cuda(), **kw))]
    if skinny_supported(M, N, K, BF, BF):
        fast.append(("stream", lambda **kw: skinny_gemm(x.cuda(), w.cuda(), **kw)))
    if ws_supported(M, N, K, BF, BF):
        fast.append(("weight stream", lambda **kw: gemm_ws(x.cuda(), w.cuda(), **kw)))
    for name, f in fast:
        assert torch.allclose(f(epilogue="f32").cpu(), want, atol=2e-5 * math.sqrt(K), rtol=1e-5), name
        assert torch.allclose(f().float().cpu(), want, atol=3e-2, rtol=2e-2), name
        assert torch.allclose(f(epilogue="silu_mul").float().cpu(), want_silu, atol=3e-2, rtol=2e-2), name
    # what the dispatcher picks
    assert torch.allclose(ops.linear(x.cuda(), w.cuda(), out_dtype=F32).cpu(), want, atol=2e-5 * math.sqrt(K), rtol=1e-5)


def _cache(lens, nkv, hd, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    need = [(n + 63) // 64 for n in lens]
    n_pages = sum(need) + 2
    perm = torch.randperm(n_pages - 1, generator=g).add(1).tolist()
    kp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype)
    vp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype)
    bt = torch.zeros((len(lens), max(need)), dtype=torch.int32)
    for s, n in enumerate(lens):
        for i in range(need[s]):
            page = perm.pop()
            bt[s, i] = page
            rows = min(64, n - 64 * i)
            kp[page, :, :rows] = torch.randn(nkv, rows, hd, generator=g).to(dtype)
            vp[page, :, :rows] = torch.randn(nkv, rows, hd, generator=g).to(dtype)
    return kp, vp, bt


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (6, 2, 48, 32), (3, 3, 80, 80), (8, 2, 64, 64), (4, 1, 128, 128),
                                            (2, 2, 112, 0)])
def test_head_preparation_against_the_cpp_loops(dtype, nh, nkv, hd, rot):
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(hd + nh)
    past, new = [3, 64, 0], [70, 2, 5]
    T = sum(new)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    wq, wk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    inv = torch.rand(rot // 2, generator=g) if rot else None
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(past, new)])
    seq_of = torch.cat([torch.full((n,), s) for s, n in enumerate(new)])
    bt = torch.tensor([[2, 5], [3, 1], [4, 0]], dtype=torch.int32)
    kp = torch.full((6, nkv, 64, hd), float("nan"), dtype=dtype)
    vp = kp.clone()
    kc, vc = kp.clone().cuda(), vp.clone().cuda()
    want_q = R.qkv_prepare(qkv, kp, vp, wq, wk, inv, rot, 2e-6, positions, seq_of, bt, nh, nkv, hd)
    q = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
    ops.qkv_prepare(qkv.cuda(), q, kc, vc, wq.cuda(), wk.cuda(), None if inv is None else inv.cuda(), rot, 2e-6, i32(positions),
                    i32(seq_of), bt.cuda(), nh, nkv, hd)
    t = dict(atol=1e-5, rtol=1e-5) if dtype == F32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(q.float().cpu(), want_q.float(), **t)
    assert torch.equal(torch.isnan(kc.float().cpu()), torch.isnan(kp.float()))          # the same places were written
    assert torch.allclose(torch.nan_to_num(kc.float().cpu()), torch.nan_to_num(kp.float()), **t)
    assert torch.equal(torch.nan_to_num(vc.float().cpu()), torch.nan_to_num(vp.float()))


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (6, 2, 48, 50), (8, 2, 32, None), (8, 2, 64, 100), (8, 2, 128, None),
                                               (16, 1, 128, 70), (3, 3, 80, 7)])
def test_every_attention_kernel_against_the_cpp_loops(nh, nkv, hd, window):
    """Prompt steps (packed, unequal lengths, some with keys from before) and single-token steps, through the plain
    kernel and every fast kernel that takes the head size."""
    from synaptix_b200 import ops
    from synaptix_b200.ops.attention import (attn_decode, attn_decode_tma, attn_prefill, attn_prefill_tc, fast_supported,
                                             query_tiles, tc_prefill_supported, tma_decode_supported)
    g = torch.Generator().manual_seed(nh + hd)
    past, new = [0, 130, 64], [200, 3, 70]
    lens = [p + n for p, n in zip(past, new)]
    scale = 1 / math.sqrt(hd)
    for dtype in (F32, BF):
        kp, vp, bt = _cache(lens, nkv, hd, dtype, 11)
        T = sum(new)
        q = torch.randn(T, nh * hd, generator=g).to(dtype)
        positions = torch.cat([torch.arange(p, p + n) for p, n in zip(past, new)])
        seq_of = torch.cat([torch.full((n,), s) for s, n in enumerate(new)])
        want = R.attention(q, kp, vp, positions, seq_of, bt, nh, nkv, hd, scale, window).float()
        t = dict(atol=1e-5, rtol=1e-4) if dtype == F32 else dict(atol=2e-2, rtol=2e-2)
        got = ops.attn_generic(q.cuda(), kp.cuda(), vp.cuda(), i32(positions), i32(seq_of), bt.cuda(), nh, nkv, hd, scale, window)
        assert torch.allclose(got.float().cpu(), want, **t), "plain kernel"
        if dtype != BF or not fast_supported(BF, nh, nkv, hd):
            continue
        cu = [0]
        for n in new:
            cu.append(cu[-1] + n)
        for rows, fn_, ok in ((64, attn_prefill, True), (128, attn_prefill_tc, tc_prefill_supported(BF, nh, nkv, hd))):
            if not ok:
                continue
            ts, t0 = query_tiles(cu, rows)
            got = fn_(q.cuda(), kp.cuda(), vp.cuda(), i32(ts), i32(t0), i32(cu), i32(past), i32(lens), bt.cuda(), nh, nkv, hd,
                      scale, window)
            assert torch.allclose(got.float().cpu(), want, **t), fn_.__name__
        # single-token steps: the last token of every sequence
        last = torch.tensor([c - 1 for c in cu[1:]])
        q1 = q[last].contiguous()
        want1 = want[last]
        for splits in (1, 2, 3, 4):
            got = attn_decode(q1.cuda(), kp.cuda(), vp.cuda(), i32(lens), bt.cuda(), nh, nkv, hd, scale, window, splits)
            assert torch.allclose(got.float().cpu(), want1, **t), f"decode, {splits} splits"
            if tma_decode_supported(BF, nh, nkv, hd):
                got = attn_decode_tma(q1.cuda(), kp.cuda(), vp.cuda(), i32(lens), bt.cuda(), nh, nkv, hd, scale, window, splits)
                assert torch.allclose(got.float().cpu(), want1, **t), f"decode by TMA, {splits} splits"


def test_single_token_attention_that_prepares_its_heads_against_the_cpp_loops():
    """The decode attention that takes the fused projection: C++ head preparation, then C++ attention."""
    from synaptix_b200.ops.attention import attn_decode_prep, attn_decode_tma
    nh, nkv, hd = 8, 2, 128
    g = torch.Generator().manual_seed(5)
    lens = [131, 64, 1, 300]
    S = len(lens)
    kp, vp, bt = _cache(lens, nkv, hd, BF, 3)
    qkv = torch.randn(S, (nh + 2 * nkv) * hd, generator=g).to(BF)
    wq, wk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    inv = torch.rand(hd // 2, generator=g) * 0.1
    positions = torch.tensor([n - 1 for n in lens])
    seq_of = torch.arange(S)
    kr, vr = kp.clone(), vp.clone()
    q = R.qkv_prepare(qkv, kr, vr, wq, wk, inv, hd, 1e-6, positions, seq_of, bt, nh, nkv, hd)
    want = R.attention(q, kr, vr, positions, seq_of, bt, nh, nkv, hd, 0.09, None).float()
    for name, f in (("cp.async", lambda k, v: attn_decode_prep(qkv.cuda(), k, v, i32(lens), bt.cuda(), nh, nkv, hd, 0.09, None, 2,
                                                                 wq.cuda(), wk.cuda(), inv.cuda(), 1e-6, True)),
                    ("TMA", lambda k, v: attn_decode_tma(qkv.cuda(), k, v, i32(lens), bt.cuda(), nh, nkv, hd, 0.09, None, 2,
                                                         prep=True, wq=wq.cuda(), wk=wk.cuda(), inv_freq=inv.cuda(), eps=1e-6,
                                                         write_cache=True))):
        kc, vc = kp.clone().cuda(), vp.clone().cuda()
        got = f(kc, vc)
        assert torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2), name
        assert torch.allclose(torch.nan_to_num(kc.float().cpu()), torch.nan_to_num(kr.float()), atol=3e-2, rtol=2e-2), name
        assert torch.equal(torch.nan_to_num(vc.float().cpu()), torch.nan_to_num(vr.float())), name


def test_sampling_kernels_against_the_cpp_loops():
    from synaptix_b200.ops import sampling as K
    g = torch.Generator().manual_seed(9)
    for V in (301, 40000):
        x = torch.randn(7, V, generator=g) * 2
        x[1, 5] = x[1, V - 2] = 40.0
        x[2, :] = 1.0
        x[3, 9] = float("nan")
        assert K.argmax_rows(x.cuda()).cpu().tolist() == R.argmax_rows(x).tolist()
    V, rows, seed = 2001, 40, 77
    x = torch.randn(rows, V, generator=g) * 2.5
    hist = torch.randint(0, V, (rows, 9), generator=g, dtype=torch.int32)
    hl = torch.randint(0, 10, (rows,), generator=g, dtype=torch.int32)
    for last_n in (0, 3):
        a, b = x.clone().cuda(), x.clone()
        K.apply_penalties(a, hist.cuda(), hl.cuda(), last_n, 1.2, 0.4, 0.3)
        R.apply_penalties(b, hist, hl, last_n, 1.2, 0.4, 0.3)
        assert torch.allclose(a.cpu(), b, atol=1e-6)
    x[0, 17] = x[1, 0] = float("nan")
    x[2, :900] = float("-inf")
    x[3] = (x[3] * 2).round() / 2
    seq, step = torch.arange(rows) % 6, torch.arange(rows) * 3
    for kw in (dict(temperature=1.0), dict(temperature=0.7, top_k=5), dict(temperature=1.2, top_p=0.6),
               dict(temperature=1.0, min_p=0.2), dict(temperature=0.9, top_k=40, top_p=0.8, min_p=0.05), dict(temperature=0.0)):
        args = (kw["temperature"], kw.get("top_k", 0), kw.get("top_p", 1.0), kw.get("min_p", 0.0), seed)
        u_gpu = torch.empty(rows, device="cuda")
        want, u, kept = R.sample_rows(x, *args, seq, step, want_kept=True)
        if kw["temperature"] == 0.0:
            assert torch.equal(K.sample_rows(x.cuda(), *args, i32(seq), i32(step)).cpu(), want)
            continue
        for cluster in (0, 8):
            _sampled_like_the_loops(K.sample_rows(x.cuda(), *args, i32(seq), i32(step), u_out=u_gpu, cluster=cluster).cpu(),
                                    u_gpu, want, u, kept, x, kw)


def _sampled_like_the_loops(got, u_gpu, want, u, kept, x, kw):
    assert torch.equal(u_gpu.cpu(), u)
    # the same token, unless u lies within rounding of an interval's end (the kernel sums in another order)
    xs = x.double() / kw["temperature"]
    p = torch.exp(xs - xs.max(1, keepdim=True).values) * kept.double()
    cum = torch.cumsum(p / p.sum(1, keepdim=True), 1)
    for r in range(x.shape[0]):
        assert kept[r, got[r]] == 1, f"{kw} row {r}: the kernel drew a token the filters drop"
        if got[r] != want[r]:
            edge = cum[r, min(got[r], want[r])].item()
            assert abs(edge - u[r].item()) < 1e-5, f"{kw} row {r}: {got[r]} vs {want[r]}"


def test_decode_bookkeeping_kernels_against_the_cpp_loops():
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(4)
    S, cap = 37, 6
    mk = lambda lo, hi: torch.randint(lo, hi, (S,), generator=g, dtype=torch.int32)
    tok, ctrl, samp = mk(0, 100), mk(-1, 3) * 50, mk(0, 100)
    ctrl[ctrl > 0] += 7
    ctrl[ctrl == 0] = -1
    hist = torch.randint(0, 100, (S, cap), generator=g, dtype=torch.int32)
    hl, pos, rs, adv = mk(0, cap + 1), mk(0, 500), mk(0, 9), mk(0, 2)
    past, lens = pos.clone(), pos + 1
    cpu = [t.clone() for t in (tok, hist, hl, pos, past, lens, rs)]
    gpu = [t.clone().cuda() for t in (tok, hist, hl, pos, past, lens, rs)]
    R.decode_begin(cpu[0], ctrl, cpu[1], cpu[2])
    ops.decode_begin(gpu[0], ctrl.cuda(), gpu[1], gpu[2])
    R.decode_advance(cpu[0], samp, cpu[3], cpu[4], cpu[5], cpu[6], adv, cpu[1], cpu[2])
    ops.decode_advance(gpu[0], samp.cuda(), gpu[3], gpu[4], gpu[5], gpu[6], adv.cuda(), gpu[1], gpu[2])
    for a, b in zip(cpu, gpu):
        assert torch.equal(a, b.cpu())


@pytest.mark.parametrize("M", [129, 300, 1000])
@pytest.mark.parametrize("nh,nkv,K,norm,rot", [(4, 2, 264, True, True), (6, 1, 1224, True, False), (2, 2, 96, False, True)])
def test_projection_with_head_preparation_in_its_epilogue_against_the_cpp_loops(M, nh, nkv, K, norm, rot):
    """The fused q/k/v product of a prompt step whose epilogue norms and rotates the heads and writes the cache: the C++
    product (rounded to bfloat16, as the projection's output would be), then the C++ head preparation; and the two
    kernels it replaces."""
    from synaptix_b200 import ops
    from synaptix_b200.ops.gemm_tc import gemm_tc, gemm_tc_qkv, gemm_tc_status
    hd = 128
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(M, K, generator=g).to(BF)
    w = (torch.randn((nh + 2 * nkv) * hd, K, generator=g) * 2 / math.sqrt(K)).to(BF)
    wq = 1 + 0.3 * torch.randn(hd, generator=g) if norm else None
    wk = 1 + 0.3 * torch.randn(hd, generator=g) if norm else None
    inv = torch.rand(hd // 2, generator=g) * 0.3 if rot else None
    # three sequences, the second with keys from before; pages in scrambled order
    new = [M // 2, M // 3, M - M // 2 - M // 3]
    past = [0, 70, 5]
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(past, new)])
    seq_of = torch.cat([torch.full((n,), s) for s, n in enumerate(new)])
    need = [(p + n + 63) // 64 for p, n in zip(past, new)]
    n_pages = sum(need) + 2
    perm = torch.randperm(n_pages - 1, generator=g).add(1).tolist()
    bt = torch.zeros((3, max(need)), dtype=torch.int32)
    for s in range(3):
        for i in range(need[s]):
            bt[s, i] = perm.pop()
    kp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=BF)
    vp = kp.clone()
    want_q = R.qkv_prepare(R.gemm(x, w), kp, vp, wq, wk, inv, hd if rot else 0, 1e-6, positions, seq_of, bt, nh, nkv, hd)
    dev = lambda t: None if t is None else t.cuda()
    cos, sin = ops.rope_table(i32(positions), inv.cuda()) if rot else (None, None)
    if rot:
        ang = positions.float()[:, None] * inv[None, :]
        assert torch.allclose(cos.cpu(), torch.cos(ang), atol=1e-6) and torch.allclose(sin.cpu(), torch.sin(ang), atol=1e-6)
    kc, vc = torch.full_like(kp, float("nan")).cuda(), torch.full_like(vp, float("nan")).cuda()
    q = torch.full((M, nh * hd), float("nan"), dtype=BF, device="cuda")
    gemm_tc_qkv(x.cuda(), w.cuda(), q, kc, vc, dev(wq), dev(wk), cos, sin, 1e-6, i32(positions), i32(seq_of), bt.cuda(), nh, nkv)
    t = dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(q.float().cpu(), want_q.float(), **t)
    assert torch.equal(torch.isnan(kc.float().cpu()), torch.isnan(kp.float()))          # the same places were written
    assert torch.allclose(torch.nan_to_num(kc.float().cpu()), torch.nan_to_num(kp.float()), **t)
    assert torch.allclose(torch.nan_to_num(vc.float().cpu()), torch.nan_to_num(vp.float()), **t)
    # the two kernels it replaces give the same numbers but for the order of the sums (that product may split K)
    k2, v2 = torch.full_like(kc, float("nan")), torch.full_like(vc, float("nan"))
    q2 = torch.empty_like(q)
    ops.qkv_prepare(gemm_tc(x.cuda(), w.cuda()), q2, k2, v2, dev(wq), dev(wk), dev(inv), hd if rot else 0, 1e-6, i32(positions),
                    i32(seq_of), bt.cuda(), nh, nkv, hd)
    assert torch.allclose(q.float(), q2.float(), atol=2e-2, rtol=1e-2)
    assert torch.allclose(torch.nan_to_num(vc.float()), torch.nan_to_num(v2.float()), atol=2e-2, rtol=1e-2)
    assert torch.allclose(torch.nan_to_num(kc.float()), torch.nan_to_num(k2.float()), atol=2e-2, rtol=1e-2)
    # a layer that reads another layer's cache writes nothing
    q3 = torch.empty_like(q)
    gemm_tc_qkv(x.cuda(), w.cuda(), q3, None, None, dev(wq), dev(wk), cos, sin, 1e-6, i32(positions), i32(seq_of), bt.cuda(), nh, nkv)
    assert torch.equal(q3, q)
    assert gemm_tc_status() == 0

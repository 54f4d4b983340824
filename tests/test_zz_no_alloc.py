"""The decode-attention entry point that allocates nothing, called the way its users call it:
through the exported C symbol of the compiled library, with raw device pointers.

It exists for host programs that cannot bring scratch memory of their own (the device is owned
by someone else's memory pool, or the loop must not call cudaMalloc because that synchronises
the device).  Its partial results go through an array built into the library, so the test
checks it against the ordinary entry point, whose scratch the caller allocates, and against a
plain softmax(q k^T) v written here, on calls in a row with different inputs: a later call finds
the earlier call's leftovers in the array and must not be disturbed by them.  This file sorts
last so that a run which stops at the first failure has already run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = 10005


def _library():
    from synaptix_b200.csrc.build import library_path, load_library
    load_library("attention")                      # compiles it if this is a fresh checkout
    lib = ctypes.CDLL(library_path("attention"))
    lib.sx_attn_decode_noalloc.restype = ctypes.c_int
    lib.sx_attn_decode_noalloc_capacity.restype = ctypes.c_ulonglong
    return lib


def _plain(q, ks, vs, nh, nkv, hd, scale, window):
    """softmax(q k^T * scale) v per head in float64 over each sequence's own keys (the last ``window`` of them)."""
    out = torch.empty(len(ks), nh, hd, dtype=torch.float64)
    g = nh // nkv
    for s, (k, v) in enumerate(zip(ks, vs)):
        n = k.shape[1]
        lo = max(0, n - window) if window else 0
        for h in range(nh):
            sc = (k[h // g, lo:].double() @ q[s].view(nh, hd)[h].double().cpu()) * scale
            out[s, h] = torch.softmax(sc, 0) @ v[h // g, lo:].double()
    return out.float().view(len(ks), nh * hd)


def _case(seed, S, nh, nkv, hd, lens, dense=None):
    """Random queries and a paged cache whose pages are in scrambled order, unused rows NaN.  ``dense``, a
    list, receives each sequence's keys and values ``[nkv, n, hd]`` as the pages hold them."""
    g = torch.Generator().manual_seed(seed)
    need = [(n + 63) // 64 for n in lens]
    n_pages = sum(need) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
    vp = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
    bt = torch.zeros((S, max(need)), dtype=torch.int32)
    for s, n in enumerate(lens):
        for i in range(need[s]):
            page = perm.pop()
            bt[s, i] = page
            rows = min(64, n - 64 * i)
            kp[page, :, :rows] = torch.randn(nkv, rows, hd, generator=g).to(torch.bfloat16)
            vp[page, :, :rows] = torch.randn(nkv, rows, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(S, nh * hd, generator=g).to(torch.bfloat16)
    if dense is not None:
        for s, n in enumerate(lens):
            k = torch.cat([kp[bt[s, i], :, :min(64, n - 64 * i)] for i in range(need[s])], dim=1)
            v = torch.cat([vp[bt[s, i], :, :min(64, n - 64 * i)] for i in range(need[s])], dim=1)
            dense.append((k.float(), v.float()))
    return q.cuda(), kp.cuda(), vp.cuda(), torch.tensor(lens, dtype=torch.int32).cuda(), bt.cuda()


def _call(lib, q, kp, vp, lens, bt, nh, nkv, hd, scale, window, n_splits):
    S = q.shape[0]
    out = torch.full((S, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.sx_attn_decode_noalloc(p(q), p(kp), p(vp), p(out), p(lens), p(bt), ctypes.c_int(bt.shape[1]),
                                    ctypes.c_int(S), ctypes.c_int(nh), ctypes.c_int(nkv), ctypes.c_int(hd),
                                    ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(n_splits),
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_no_alloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    from synaptix_b200.ops.attention import attn_decode
    lib = _library()
    assert lib.sx_attn_decode_noalloc_capacity() == 4 << 20
    # calls in a row, different inputs, head sizes and split counts; the second also with a window
    for seed, nh, nkv, hd, lens, n_splits, window in [(1, 8, 2, 128, [700, 64, 1, 130], 6, 0),
                                                       (2, 8, 2, 128, [33, 900, 257], 9, 100),
                                                       (5, 6, 3, 64, [300, 65], 4, 0), (6, 4, 1, 32, [129, 700, 2], 5, 40)]:
        scale = 1 / math.sqrt(hd)
        dense = []
        q, kp, vp, ln, bt = _case(seed, len(lens), nh, nkv, hd, lens, dense)
        rc, got = _call(lib, q, kp, vp, ln, bt, nh, nkv, hd, scale, window, n_splits)
        assert rc == 0
        want = attn_decode(q, kp, vp, ln, bt, nh, nkv, hd, scale, window or None, n_splits)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = (got.float() - want.float()).abs().max().item()
        assert err < 2e-2, f"call with seed {seed}: {err}"      # the tolerance of the kernel tests
        plain = _plain(q, [d[0] for d in dense], [d[1] for d in dense], nh, nkv, hd, scale, window)
        err = (got.float().cpu() - plain).abs().max().item()
        assert err < 2e-2, f"call with seed {seed} against the plain formula: {err}"
    nh, nkv, hd = 8, 2, 128
    scale = 1 / math.sqrt(hd)
    # one split needs no scratch at all and goes the same way
    q, kp, vp, ln, bt = _case(3, 2, nh, nkv, hd, [100, 5])
    rc, got = _call(lib, q, kp, vp, ln, bt, nh, nkv, hd, scale, 0, 1)
    want = attn_decode(q, kp, vp, ln, bt, nh, nkv, hd, scale, None, 1)
    assert rc == 0 and (got.float() - want.float()).abs().max().item() < 2e-2


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    lib = _library()
    nh, nkv, hd = 32, 8, 128
    q, kp, vp, ln, bt = _case(4, 8, nh, nkv, hd, [70] * 8)
    # 8 sequences x 32 heads x 64 splits x 130 floats = 8.5 MB > 4 MiB
    rc, out = _call(lib, q, kp, vp, ln, bt, nh, nkv, hd, 0.1, 0, 64)
    torch.cuda.synchronize()
    assert rc == TOO_LARGE
    assert torch.isnan(out.float()).all()          # nothing was launched
    rc, _ = _call(lib, q, kp, vp, ln, bt, nh, nkv, hd, 0.1, 0, 16)      # 2.1 MB: fits
    assert rc == 0
    # the most splits whose partial results fit the array are taken, one more is not; and more splits than the
    # merge can hold are refused before anything is launched
    nh, nkv, hd = 16, 1, 32
    per_split = 16 * 34 * 4                            # bytes a split of one sequence takes
    fit = (4 << 20) // per_split                       # 1,927 splits
    q, kp, vp, ln, bt = _case(8, 1, nh, nkv, hd, [200])
    rc_fit, out_fit = _call(lib, q, kp, vp, ln, bt, nh, nkv, hd, 0.1, 0, fit)
    rc_over, out_over = _call(lib, q, kp, vp, ln, bt, nh, nkv, hd, 0.1, 0, fit + 1)
    rc_many, out_many = _call(lib, q, kp, vp, ln, bt, 1, 1, hd, 0.1, 0, 5000)
    torch.cuda.synchronize()
    assert rc_fit == 0 and torch.isfinite(out_fit.float()).all()
    assert rc_over == TOO_LARGE and torch.isnan(out_over.float()).all()
    assert rc_many == 10002 and torch.isnan(out_many.float()).all()

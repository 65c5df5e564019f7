"""lq_attn_decode_static: the decode-attention entry point that allocates nothing.

Some users of the library cannot allocate device memory at the point where they call it (a
fixed memory budget handed out at start-up, a latency-bound loop that must not run into
cudaMalloc's device synchronisation, a host that forbids allocator calls in callbacks).  For
them the scratch of the split-KV attention lives in a static device array inside the library.
This test calls that entry point through its exported C symbol, twice in a row with different
inputs and slice counts (the array keeps the first call's contents), and compares with the
ordinary entry point, whose scratch the caller allocates.  It checks what the entry point is for --
the calls leave the device's free memory and torch's allocation count where they were -- and that a
call too large for the array is refused before anything runs, to the token: the largest call that
fits runs and is right, one token more is refused, and so is a call whose partial results alone
would fit but not together with its counters.

The file's name makes pytest collect it last, so a run that stops at the first failure has
already run every other test.  It passes alone in a fresh process and after the other tests.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

ARGTYPES = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]


def _symbol():
    from longbow_quarrel_b200.kernels import build
    lib = build.load("attn_decode")
    fn = lib.lq_attn_decode_static
    fn.argtypes, fn.restype = ARGTYPES, c_int
    cap = lib.lq_attn_decode_static_floats
    cap.restype = ctypes.c_long
    return fn, int(cap())


def _call(fn, q, case, tok_pos, tok_seq, H, Hkv, hd, scale, window, n_splits, out=None):
    if out is None:
        out = torch.full((q.shape[0], H * hd), float("nan"), dtype=torch.bfloat16, device=q.device)
    p = lambda t: c_void_p(t.data_ptr())  # noqa: E731
    rc = fn(p(q), q.stride(0), p(case.k_pages), p(case.v_pages), p(case.table), case.table.stride(0), p(tok_pos),
            p(tok_seq), p(case.slots), p(out), q.shape[0], H, Hkv, hd, case.page_size, float(scale), int(window or 0),
            n_splits, c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_scratch_entry_point_matches_the_allocating_one():
    from longbow_quarrel_b200.kernels import ops
    from test_gpu_kernels import PagedCase, _attn_tol, _close, _ints, _rand, BF16_ULP
    fn, capacity = _symbol()
    assert capacity == 2 * 1024 * 1024
    H, Hkv, hd = 8, 2, 128
    case = PagedCase([300, 1, 77, 64, 17], Hkv, hd, torch.bfloat16, seed=9)
    tok_seq, tok_pos = _ints([0, 1, 2, 3, 4, 0]), _ints([299, 0, 76, 63, 16, 150])
    scale = hd ** -0.5
    # two calls in a row: other queries, another window and other slice counts the second time,
    # so that what the first call left in the array would show if it were read
    for seed, n_splits, window in ((90, 8, None), (91, 3, 100)):
        q = _rand((6, (H + 2 * Hkv) * hd), torch.bfloat16, seed)
        want = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, tok_pos, tok_seq, case.slots, H, Hkv, hd,
                               case.page_size, scale, window, n_splits)
        out = torch.full((6, H * hd), float("nan"), dtype=torch.bfloat16, device=q.device)
        torch.cuda.synchronize()
        # What the entry point exists for: the call itself allocates nothing, on the device or through torch.
        free_before, count_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_stats()["allocation.all.allocated"]
        rc, got = _call(fn, q, case, tok_pos, tok_seq, H, Hkv, hd, scale, window, n_splits, out=out)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == count_before
        assert rc == 0
        ref = case.reference(q[:, :H * hd].reshape(-1, H, hd).float(), tok_seq.tolist(), tok_pos.tolist(), H, scale,
                             window)
        _close(got.reshape(-1, H, hd), ref, _attn_tol(case, ref), BF16_ULP)      # right against the plain restatement
        assert torch.equal(got, want)                                            # and the same as the other entry point
    # one slice needs no scratch at all
    q = _rand((6, (H + 2 * Hkv) * hd), torch.bfloat16, 92)
    rc, got = _call(fn, q, case, tok_pos, tok_seq, H, Hkv, hd, scale, None, 1)
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.equal(got, ops.attn_decode(q, case.k_pages, case.v_pages, case.table, tok_pos, tok_seq, case.slots,
                                            H, Hkv, hd, case.page_size, scale, None, 1))


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from test_gpu_kernels import PagedCase, _ints, _rand
    fn, capacity = _symbol()
    H, Hkv, hd = 64, 8, 128
    T, n_splits = 64, 32                      # 64 * 64 * 32 * 130 floats = 17 M > 2 M
    assert T * H * n_splits * (hd + 2) > capacity
    case = PagedCase([40] * 2, Hkv, hd, torch.bfloat16, seed=10)
    q = _rand((T, (H + 2 * Hkv) * hd), torch.bfloat16, 93)
    rc, out = _call(fn, q, case, _ints([39] * T), _ints([0] * T), H, Hkv, hd, 1.0, None, n_splits)
    torch.cuda.synchronize()
    assert rc == -4
    assert bool(out.isnan().all())            # nothing ran


def test_static_scratch_capacity_is_exact_to_the_token():
    """16 heads over 2 kv heads of 16, 16 slices: a token needs 16 * 16 * 18 floats of partial results and 2
    counters.  454 tokens fit the 2 Mi floats and run; with 455 the partial results alone would still fit
    (2,096,640) but not with the counters (2,097,550): refused.  Sizes that the kernel does not take are
    refused with -2 and leave the array alone."""
    from longbow_quarrel_b200.kernels import ops
    from test_gpu_kernels import PagedCase, _ints, _rand
    fn, capacity = _symbol()
    H, Hkv, hd, n_splits = 16, 2, 16, 16
    per_token = H * n_splits * (hd + 2) + Hkv
    assert 454 * per_token <= capacity < 455 * per_token and 455 * (per_token - Hkv) <= capacity
    case = PagedCase([200, 90], Hkv, hd, torch.bfloat16, seed=11)
    for T, want_rc in ((454, 0), (455, -4)):
        q = _rand((T, (H + 2 * Hkv) * hd), torch.bfloat16, 94)
        tok_seq = _ints([i % 2 for i in range(T)])
        tok_pos = _ints([(i * 7) % (200 if i % 2 == 0 else 90) for i in range(T)])
        rc, got = _call(fn, q, case, tok_pos, tok_seq, H, Hkv, hd, 0.25, None, n_splits)
        torch.cuda.synchronize()
        assert rc == want_rc
        if rc == 0:
            want = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, tok_pos, tok_seq, case.slots, H, Hkv, hd,
                                   case.page_size, 0.25, None, n_splits)
            assert torch.equal(got, want)
        else:
            assert bool(got.isnan().all())
    q = _rand((4, (H + 2 * Hkv) * hd), torch.bfloat16, 95)
    for bad in (dict(H=15), dict(n_splits=33), dict(hd=12)):
        args = {**dict(H=H, Hkv=Hkv, hd=hd, n_splits=4), **bad}
        rc, got = _call(fn, q, case, _ints([5, 6, 7, 8]), _ints([0, 1, 0, 1]), args["H"], args["Hkv"], args["hd"], 0.25, None,
                        args["n_splits"])
        torch.cuda.synchronize()
        assert rc == -2 and bool(got.isnan().all()), bad

"""Each kernel alone against a plain float32 PyTorch restatement of the same
operation, at sizes other than the engine's tiny configurations."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from longbow_quarrel_b200.kernels import ops
    return ops


BF16_ULP = 2.0 ** -8     # a value stored in bfloat16 is within half of this, relatively, of the exact one


def _close(got, ref, tol, rel=0.0):
    """|got - ref| <= tol * rms(ref) + rel * |ref| everywhere.  `rel` is for results that
    are rounded to bfloat16 on store, whose error is a fraction of each value itself."""
    got, ref = got.float().cpu().double(), ref.float().cpu().double()
    assert torch.isfinite(got).all()
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-30)
    excess = ((got - ref).abs() - rel * ref.abs()) / rms
    err = float(excess.max())
    assert err < tol, err
    return err


def _acc_tol(K):
    """Float32 accumulation of K products: a few times sqrt(K) roundings of 2^-24, relative to
    the result's root mean square."""
    return 8.0 * math.sqrt(K) * 2.0 ** -24


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------ plain kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    ops = _ops()
    table = _rand((301, 72), dtype, 0)
    tokens = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = ops.embedding(table, tokens)
    assert out.dtype == torch.float32
    assert torch.equal(out, table[tokens.long()].float())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [72, 1000, 4096, 70, 8192, 10000])      # 70 and 10000 take the scalar kernel
def test_rmsnorm(out_dtype, D):
    ops = _ops()
    x = _rand((9, D), torch.float32, 1, 3.0)
    gain = 1 + 0.1 * _rand((D,), torch.float32, 2)
    eps = 1e-5
    ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * gain
    rel = 0.0 if out_dtype == torch.float32 else BF16_ULP
    _close(ops.rmsnorm(x, gain, eps, out_dtype), ref, 2e-6, rel)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    _close(ops.rmsnorm(x, gain, eps, out_dtype, rows=rows), ref[rows.long()], 2e-6, rel)


@pytest.mark.parametrize("a_dtype,w_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                             (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 250, 80), (70, 130, 200), (5, 64, 1000)])
def test_gemm_plain(a_dtype, w_dtype, M, N, K):
    ops = _ops()
    a, w = _rand((M, K), a_dtype, 3), _rand((N, K), w_dtype, 4)
    ref = a.float().double() @ w.float().double().T
    _close(ops.gemm_plain(a, w, torch.float32), ref, 1e-5)
    res = _rand((M, N), torch.float32, 5)
    expect = res.double() + ref
    got = ops.gemm_plain(a, w, torch.float32, residual=res)
    assert got.data_ptr() == res.data_ptr()
    _close(got, expect, 1e-5)


def test_gemm_plain_is_independent_of_other_rows():
    """A row's result is bit-equal whether it is computed alone or among others."""
    ops = _ops()
    a, w = _rand((37, 328), torch.float32, 6), _rand((90, 328), torch.float32, 7)
    full = ops.gemm_plain(a, w, torch.float32)
    for r in (0, 11, 36):
        assert torch.equal(ops.gemm_plain(a[r:r + 1].contiguous(), w, torch.float32)[0], full[r])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block", [0, 8])
def test_swiglu(dtype, block):
    ops = _ops()
    F = 40
    g, u = _rand((6, F), dtype, 8, 2.0), _rand((6, F), dtype, 9)
    if block:
        gu = torch.stack([g.reshape(6, F // block, block), u.reshape(6, F // block, block)], dim=2).reshape(6, 2 * F)
    else:
        gu = torch.cat([g, u], dim=1)
    ref = u.float() * (g.float() / (1 + torch.exp(-g.float())))
    _close(ops.swiglu(gu.contiguous(), block), ref, 1e-6, 0.0 if dtype == torch.float32 else BF16_ULP)


# ------------------------------------------------------------------ paged cache helpers
class PagedCase:
    """Random K/V for sequences of given lengths, scattered over shuffled pages."""

    def __init__(self, lens, Hkv, hd, dtype, seed, page_size=64, extra_pages=3, poison=float("nan")):
        rng = np.random.default_rng(seed)
        self.lens, self.Hkv, self.hd, self.page_size = lens, Hkv, hd, page_size
        n_seq = len(lens)
        pages_per = [-(-n // page_size) for n in lens]
        n_pages = sum(pages_per) + extra_pages
        perm = rng.permutation(n_pages)
        self.k = [_rand((n, Hkv, hd), dtype, seed * 100 + i) for i, n in enumerate(lens)]
        self.v = [_rand((n, Hkv, hd), dtype, seed * 100 + 50 + i) for i, n in enumerate(lens)]
        # Unused memory is poisoned so that a read outside a sequence's keys shows.
        self.k_pages = torch.full((n_pages, Hkv, page_size, hd), poison, dtype=dtype, device=DEV)
        self.v_pages = torch.full((n_pages, Hkv, page_size, hd), poison, dtype=dtype, device=DEV)
        self.n_slots = n_seq + 2
        self.slot_of = [int(s) for s in rng.permutation(self.n_slots)[:n_seq]]
        table = np.full((self.n_slots, max(pages_per) + 1), -1, dtype=np.int32)
        nxt = 0
        for i, n in enumerate(lens):
            for p in range(pages_per[i]):
                page = int(perm[nxt]); nxt += 1
                table[self.slot_of[i], p] = page
                lo, hi = p * page_size, min(n, (p + 1) * page_size)
                self.k_pages[page, :, :hi - lo] = self.k[i][lo:hi].transpose(0, 1)
                self.v_pages[page, :, :hi - lo] = self.v[i][lo:hi].transpose(0, 1)
        self.table = torch.from_numpy(table).to(DEV)
        self.slots = torch.tensor(self.slot_of, dtype=torch.int32, device=DEV)

    def reference(self, q, tok_seq, tok_pos, H, scale, window):
        """q [T, H, hd] float; plain softmax attention of each row over keys start..pos."""
        out = torch.empty_like(q, dtype=torch.float64)
        G = H // self.Hkv
        for r in range(q.shape[0]):
            s, p = tok_seq[r], tok_pos[r]
            start = p - window + 1 if (window and p >= window) else 0
            k = self.k[s][start:p + 1].double()
            v = self.v[s][start:p + 1].double()
            for h in range(H):
                sc = (k[:, h // G] @ q[r, h].double()) * scale
                out[r, h] = torch.softmax(sc, 0) @ v[:, h // G]
        return out


def _attn_tol(case, ref):
    """Attention through bfloat16 probabilities: each output is a weighted mean of values whose
    weights carry a relative rounding of 2^-9, so it is off by at most about 2^-8 of the largest
    value; expressed relative to the root mean square of the reference, as _close wants it."""
    vmax = max(float(v.float().abs().max()) for v in case.v)
    rms = float(ref.double().pow(2).mean().sqrt())
    return 2.0 ** -8 * vmax / rms


def _ints(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,hd,window", [(6, 2, 48, None), (4, 4, 16, 37), (8, 1, 128, None), (2, 1, 256, None)])
def test_attention_plain(dtype, H, Hkv, hd, window):
    ops = _ops()
    lens = [130, 1, 77]
    case = PagedCase(lens, Hkv, hd, dtype, seed=1)
    tok_seq = [0, 0, 0, 1, 2, 2]
    tok_pos = [129, 64, 0, 0, 76, 63]
    q = _rand((len(tok_seq), H * hd + 16), dtype, 77)     # wider rows: q is a slice of a qkv buffer
    scale = hd ** -0.5
    out = ops.attention_plain(q, case.k_pages, case.v_pages, case.table, _ints(tok_pos), _ints(tok_seq), case.slots,
                              H, Hkv, hd, case.page_size, scale, window)
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd).float(), tok_seq, tok_pos, H, scale, window)
    _close(out.reshape(-1, H, hd), ref, 2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [32, 128, 20])            # 20: pairs that no 16-byte access covers
def test_rope_kv_write(dtype, hd):
    ops = _ops()
    H, Hkv, page = 3, 2, 64
    T = 5
    tok_seq, tok_pos = [0, 0, 1, 1, 1], [63, 64, 0, 1, 130]
    lens = [65, 131]
    case = PagedCase(lens, Hkv, hd, dtype, seed=2)
    k_before = case.k_pages.clone()
    qkv = _rand((T, (H + 2 * Hkv) * hd), dtype, 5)
    orig = qkv.clone()
    freqs = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    ang = torch.arange(200, dtype=torch.float64)[:, None] * freqs[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    ops.rope_kv_write(qkv, cos, sin, _ints(tok_pos), _ints(tok_seq), case.slots, case.table, case.k_pages,
                      case.v_pages, H, Hkv, hd, page)
    x = orig.float().reshape(T, H + 2 * Hkv, hd)
    c, s = cos[torch.tensor(tok_pos)].unsqueeze(1), sin[torch.tensor(tok_pos)].unsqueeze(1)
    x0, x1 = x[:, :H + Hkv, :hd // 2], x[:, :H + Hkv, hd // 2:]
    rot = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)
    tol, rel = 1e-6, (0.0 if dtype == torch.float32 else BF16_ULP)
    _close(qkv.reshape(T, H + 2 * Hkv, hd)[:, :H + Hkv], rot, tol, rel)
    assert torch.equal(qkv.reshape(T, H + 2 * Hkv, hd)[:, H + Hkv:], orig.reshape(T, H + 2 * Hkv, hd)[:, H + Hkv:])
    changed = torch.zeros_like(case.k_pages, dtype=torch.bool)
    for r in range(T):
        slot = case.slot_of[tok_seq[r]]
        pg = int(case.table[slot, tok_pos[r] // page])
        _close(case.k_pages[pg, :, tok_pos[r] % page], rot[r, H:], tol, rel)
        assert torch.equal(case.v_pages[pg, :, tok_pos[r] % page], orig.reshape(T, H + 2 * Hkv, hd)[r, H + Hkv:])
        changed[pg, :, tok_pos[r] % page] = True
    # Nothing else in the cache was touched.
    same = (case.k_pages == k_before) | (case.k_pages.isnan() & k_before.isnan())
    assert bool((same | changed).all())


# ------------------------------------------------------------------ bfloat16 tensor-core kernels
@pytest.mark.parametrize("M", [1, 3, 8, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(16, 64), (100, 200), (4104, 4096), (250, 80)])
def test_gemm_skinny(M, N, K):
    ops = _ops()
    a, w = _rand((M, K), torch.bfloat16, 10), _rand((N, K), torch.bfloat16, 11)
    ref = a.float().double() @ w.float().double().T
    _close(ops.gemm_skinny(a, w, ops.EPI_F32), ref, _acc_tol(K))
    _close(ops.gemm_skinny(a, w, ops.EPI_BF16), ref, _acc_tol(K), BF16_ULP)
    res = _rand((M, N), torch.float32, 12)
    expect = res.double() + ref
    _close(ops.gemm_skinny(a, w, ops.EPI_RESID, residual=res), expect, _acc_tol(K))


@pytest.mark.parametrize("M,F,K", [(1, 8, 64), (5, 176, 64), (64, 1000, 328)])
def test_gemm_skinny_swiglu(M, F, K):
    ops = _ops()
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    a = _rand((M, K), torch.bfloat16, 13)
    wg, wu = _rand((F, K), torch.bfloat16, 14, 0.2), _rand((F, K), torch.bfloat16, 15, 0.2)
    g = a.float().double() @ wg.float().double().T
    u = a.float().double() @ wu.float().double().T
    ref = u * (g / (1 + torch.exp(-g)))
    out = ops.gemm_skinny(a, interleave_gate_up(wg, wu), ops.EPI_SWIGLU)
    assert out.shape == (M, F)
    _close(out, ref, 1e-4, BF16_ULP)


def test_gemm_skinny_is_independent_of_other_rows():
    ops = _ops()
    a, w = _rand((37, 328), torch.bfloat16, 16), _rand((90, 328), torch.bfloat16, 17)
    full = ops.gemm_skinny(a, w, ops.EPI_F32)
    for r in (0, 11, 36):
        assert torch.equal(ops.gemm_skinny(a[r:r + 1].contiguous(), w, ops.EPI_F32)[0], full[r])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 104, 200), (16, 4104, 328), (8, 4096, 4096)])
def test_gemm_skinny_folds_the_norm_that_follows(M, N, K):
    """The residual epilogue also leaves the next RMS norm's rows (residual * gain, sums of
    squares); a product that reads them finishes the norm.  Against norm and products done apart."""
    ops = _ops()
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    a, w = _rand((M, K), torch.bfloat16, 50), _rand((N, K), torch.bfloat16, 51, 0.2)
    res = _rand((M, N), torch.float32, 52, 3.0)
    res[-1] *= 40.0                                        # rows of very different size
    gain = 1 + 0.1 * _rand((N,), torch.float32, 53)
    eps = 1e-5
    expect = res.double().cpu() + a.float().double().cpu() @ w.float().double().cpu().T
    out, rows = ops.gemm_skinny(a, w, ops.EPI_RESID, residual=res, emit=(gain, eps))
    assert out.data_ptr() == res.data_ptr()
    _close(out, expect, _acc_tol(K))
    new = out.double().cpu()
    _close(rows.data, new * gain.double().cpu(), 1e-6, BF16_ULP)
    assert rows.sums.shape == (M, -(-N // 16))
    sums = rows.sums.double().cpu().sum(1)
    assert float(((sums - new.pow(2).sum(1)).abs() / new.pow(2).sum(1)).max()) < 1e-5
    # the rows as a norm kernel would have left them, from the same bfloat16 values
    rstd = torch.rsqrt(new.pow(2).mean(1, keepdim=True) + eps)
    normed = rows.data.float().double().cpu() * rstd
    _close(rows.finish(), normed, 1e-6, BF16_ULP)
    N2 = 176
    w2 = _rand((N2, N), torch.bfloat16, 54, 0.2)
    ref2 = normed @ w2.float().double().cpu().T
    _close(ops.gemm_skinny(rows, w2, ops.EPI_F32), ref2, _acc_tol(N) + 1e-6)
    _close(ops.gemm_skinny(rows, w2, ops.EPI_BF16), ref2, _acc_tol(N) + 1e-6, BF16_ULP)
    res2 = _rand((M, N2), torch.float32, 55)
    expect2 = res2.double().cpu() + ref2
    _close(ops.gemm_skinny(rows, w2, ops.EPI_RESID, residual=res2), expect2, _acc_tol(N) + 1e-6)
    wg, wu = _rand((N2, N), torch.bfloat16, 56, 0.1), _rand((N2, N), torch.bfloat16, 57, 0.1)
    g, u = normed @ wg.float().double().cpu().T, normed @ wu.float().double().cpu().T
    _close(ops.gemm_skinny(rows, interleave_gate_up(wg, wu), ops.EPI_SWIGLU), u * (g / (1 + torch.exp(-g))), 1e-4, BF16_ULP)
    # a row's result does not depend on the other rows
    one = ops.NormedRows(rows.data[-1:].contiguous(), rows.sums[-1:].contiguous(), eps)
    assert torch.equal(ops.gemm_skinny(one, w2, ops.EPI_F32)[0], ops.gemm_skinny(rows, w2, ops.EPI_F32)[-1])


def test_gemm_skinny_qkv_finishes_a_folded_norm():
    ops = _ops()
    M, H, Hkv, hd, K = 5, 4, 2, 32, 200
    lens = [70 + 5 * i for i in range(M)]
    a = _rand((M, K), torch.bfloat16, 60)
    sums = (_rand((M, 13), torch.float32, 61).abs() * 50 + 1).contiguous()
    eps = 1e-6
    w = _rand(((H + 2 * Hkv) * hd, K), torch.bfloat16, 62, 0.1)
    tok_pos, tok_seq = [n - 1 for n in lens], list(range(M))
    outs = []
    for rows in (ops.NormedRows(a, sums, eps), ops.NormedRows(a, sums, eps).finish()):
        case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=11)
        q = ops.gemm_skinny_qkv(rows, w, None, None, _ints(tok_pos), _ints(tok_seq), case.slots, case.table,
                                case.k_pages, case.v_pages, H, Hkv, hd, 64)
        outs.append((q, case))
    rstd = torch.rsqrt(sums.double().cpu().sum(1, keepdim=True) / K + eps)
    full = ((a.float().double().cpu() * rstd) @ w.float().double().cpu().T).reshape(M, H + 2 * Hkv, hd)
    q, case = outs[0]
    _close(q.reshape(M, H, hd), full[:, :H], _acc_tol(K) + 1e-6, BF16_ULP)
    for m in range(M):
        page = int(case.table[case.slot_of[m], tok_pos[m] // 64])
        _close(case.k_pages[page, :, tok_pos[m] % 64], full[m, H:H + Hkv], _acc_tol(K) + 1e-6, BF16_ULP)
        _close(case.v_pages[page, :, tok_pos[m] % 64], full[m, H + Hkv:], _acc_tol(K) + 1e-6, BF16_ULP)
    # finishing the rows first rounds them once more: close, not equal
    _close(outs[1][0], outs[0][0], 3 * BF16_ULP, BF16_ULP)


@pytest.mark.parametrize("M", [65, 128, 300, 1111])
@pytest.mark.parametrize("N,K", [(16, 64), (250, 80), (1000, 200), (1004, 136), (4104, 1024), (520, 4096)])
def test_gemm_tc(M, N, K):
    ops = _ops()
    a, w = _rand((M, K), torch.bfloat16, 20), _rand((N, K), torch.bfloat16, 21)
    ref = a.float().double() @ w.float().double().T
    _close(ops.gemm_tc(a, w, ops.EPI_F32), ref, _acc_tol(K))
    _close(ops.gemm_tc(a, w, ops.EPI_BF16), ref, _acc_tol(K), BF16_ULP)
    res = _rand((M, N), torch.float32, 22)
    expect = res.double() + ref
    _close(ops.gemm_tc(a, w, ops.EPI_RESID, residual=res), expect, _acc_tol(K))
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M,F,K", [(70, 8, 64), (200, 176, 64), (513, 1000, 328), (2048, 2048, 512)])
def test_gemm_tc_swiglu(M, F, K):
    ops = _ops()
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    a = _rand((M, K), torch.bfloat16, 23)
    wg, wu = _rand((F, K), torch.bfloat16, 24, 0.2), _rand((F, K), torch.bfloat16, 25, 0.2)
    g = a.float().double() @ wg.float().double().T
    u = a.float().double() @ wu.float().double().T
    ref = u * (g / (1 + torch.exp(-g)))
    out = ops.gemm_tc(a, interleave_gate_up(wg, wu), ops.EPI_SWIGLU)
    assert out.shape == (M, F)
    _close(out, ref, 1e-4, BF16_ULP)
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M", [17, 64, 100, 300])
@pytest.mark.parametrize("N,K", [(520, 4096), (4104, 1024), (250, 14336), (1000, 392)])
def test_gemm_tc_cuts_the_contraction_when_tiles_are_few(M, N, K):
    """Few rows and a narrow weight: pieces of work are (tile, range of K), added by a second kernel."""
    ops = _ops()
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    a, w = _rand((M, K), torch.bfloat16, 70), _rand((N, K), torch.bfloat16, 71, 0.3)
    ref = a.float().double() @ w.float().double().T
    _close(ops.gemm_tc(a, w, ops.EPI_F32), ref, _acc_tol(K))
    _close(ops.gemm_tc(a, w, ops.EPI_BF16), ref, _acc_tol(K), BF16_ULP)
    res = _rand((M, N), torch.float32, 72)
    expect = res.double() + ref
    _close(ops.gemm_tc(a, w, ops.EPI_RESID, residual=res), expect, _acc_tol(K))
    F = N // 16 * 8
    if F:
        wg, wu = w[:F].contiguous() * 0.3, w[F:2 * F].contiguous() * 0.3
        g, u = a.float().double() @ wg.float().double().T, a.float().double() @ wu.float().double().T
        out = ops.gemm_tc(a, interleave_gate_up(wg, wu), ops.EPI_SWIGLU)
        assert out.shape == (M, F)
        _close(out, u * (g / (1 + torch.exp(-g))), 1e-4, BF16_ULP)
    full = ops.gemm_tc(a, w, ops.EPI_F32)
    assert torch.equal(ops.gemm_tc(a, w, ops.EPI_F32), full)                               # repeatable
    assert torch.equal(ops.gemm_tc(a[3:4].contiguous(), w, ops.EPI_F32)[0], full[3])       # a row alone
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M", [17, 64])
@pytest.mark.parametrize("N", [33008, 30000, 28000, 26000, 23008, 40000, 18000])   # tile widths 224 ... 128
def test_gemm_tc_one_row_of_tiles_of_every_width(M, N):
    """At most 64 rows: the tile width is chosen so that the rounds over the SMs read the least; a tile
    whose width is no multiple of 32 ends in a half chunk, and the last tile of the row is partial."""
    ops = _ops()
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    K = 136
    a, w = _rand((M, K), torch.bfloat16, 76), _rand((N, K), torch.bfloat16, 77, 0.3)
    ref = (a.float() @ w.float().T).double()
    _close(ops.gemm_tc(a, w, ops.EPI_F32), ref, _acc_tol(K) + 1e-6)
    _close(ops.gemm_tc(a, w, ops.EPI_BF16), ref, _acc_tol(K) + 1e-6, BF16_ULP)
    res = _rand((M, N), torch.float32, 78)
    expect = res.double() + ref
    _close(ops.gemm_tc(a, w, ops.EPI_RESID, residual=res), expect, _acc_tol(K) + 1e-6)
    F = N // 2
    wg, wu = w[:F].contiguous(), w[F:].contiguous()
    g, u = (a.float() @ wg.float().T).double(), (a.float() @ wu.float().T).double()
    out = ops.gemm_tc(a, interleave_gate_up(wg, wu), ops.EPI_SWIGLU)
    assert out.shape == (M, F)
    _close(out, u * (g / (1 + torch.exp(-g))), 1e-4, BF16_ULP)
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M,N,K", [(2048, 4096, 1536),      # 128 tiles of 256 x 256 on 74 pairs: both accumulators, two rounds
                                   (2000, 5008, 520),       # partial tiles at both edges, K no multiple of 64
                                   (256, 18944, 72),        # one row of tiles, two steps along K
                                   (1111, 10000, 4096)])
def test_gemm_pair(M, N, K):
    """Products of many rows on pairs of SMs (tcgen05 with cta_group::2): every epilogue against a product in
    double precision, the same result as the kernel that keeps a tile on one SM up to float32 rounding, and
    the same bits when run again."""
    ops = _ops()
    from longbow_quarrel_b200.kernels.linear import interleave_gate_up
    assert ops.gemm_pair_takes(M, N, K)
    assert not ops.gemm_pair_takes(128, N, K) and not ops.gemm_pair_takes(512, 4096, K)     # too few tiles: gemm_tc's
    a, w = _rand((M, K), torch.bfloat16, 126), _rand((N, K), torch.bfloat16, 127, 0.3)
    ref = a.double() @ w.double().T
    res = _rand((M, N), torch.float32, 128)
    F = N // 2
    wg, wu = w[:F].contiguous(), w[F:].contiguous()
    g, u = a.double() @ wg.double().T, a.double() @ wu.double().T
    inter = interleave_gate_up(wg, wu)
    outs = {}
    for pairs in (True, False, True):
        ops.USE_PAIRS = pairs
        try:
            before = ops.launches_by_name()
            f32 = ops.gemm_tc(a, w, ops.EPI_F32)
            bf = ops.gemm_tc(a, w, ops.EPI_BF16)
            added = ops.gemm_tc(a, w, ops.EPI_RESID, residual=res.clone())
            act = ops.gemm_tc(a, inter, ops.EPI_SWIGLU)
            names = ops.launches_since(before)
        finally:
            ops.USE_PAIRS = True
        assert names.get("gemm_pair", 0) == (4 if pairs else 0), names
        _close(f32, ref, _acc_tol(K) + 1e-6)
        _close(bf, ref, _acc_tol(K) + 1e-6, BF16_ULP)
        _close(added, res.double() + ref, _acc_tol(K) + 1e-6)
        _close(act, u * (g / (1 + torch.exp(-g))), 1e-4, BF16_ULP)
        if pairs in outs:
            for x, y in zip(outs[pairs], (f32, bf, added, act)):
                assert torch.equal(x, y)
        outs[pairs] = (f32, bf, added, act)
    torch.cuda.synchronize()
    assert ops.gemm_pair_status() == 0 and ops.gemm_tc_status() == 0


def test_gemm_pair_leaves_unaligned_outputs_to_gemm_tc():
    """An output whose rows are not 16-byte aligned cannot leave by TMA: the product stays on gemm_tc."""
    ops = _ops()
    M, N, K = 2048, 4098, 128
    a, w = _rand((M, K), torch.bfloat16, 131), _rand((N, K), torch.bfloat16, 132, 0.3)
    before = ops.launches_by_name()
    out = ops.gemm_tc(a, w, ops.EPI_F32)
    assert "gemm_pair" not in ops.launches_since(before)
    _close(out, a.double() @ w.double().T, _acc_tol(K) + 1e-6)


def test_gemm_tc_large_many_tiles_per_block():
    """More tiles than SMs: blocks walk over several tiles and both accumulators are used."""
    ops = _ops()
    M, N, K = 2048, 6144, 512
    a, w = _rand((M, K), torch.bfloat16, 26), _rand((N, K), torch.bfloat16, 27)
    ref = (a.float() @ w.float().T).double()
    _close(ops.gemm_tc(a, w, ops.EPI_F32), ref, _acc_tol(K))
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("H,Hkv,hd,window", [(8, 2, 128, None), (6, 2, 48, None), (4, 4, 16, 37), (3, 1, 32, None),
                                             (40, 2, 64, 100), (8, 8, 80, None)])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
def test_attn_decode(H, Hkv, hd, window, n_splits):
    ops = _ops()
    lens = [300, 1, 77, 64, 17]
    case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=3)
    tok_seq = [0, 1, 2, 3, 4, 0]
    tok_pos = [299, 0, 76, 63, 16, 150]
    q = _rand((len(tok_seq), (H + 2 * Hkv) * hd), torch.bfloat16, 78)
    scale = hd ** -0.5
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd).float(), tok_seq, tok_pos, H, scale, window)
    for early in (False, True):       # with early loads the old keys are requested before the wait for the kernel ahead
        out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _ints(tok_pos), _ints(tok_seq), case.slots,
                              H, Hkv, hd, case.page_size, scale, window, n_splits, early_loads=early)
        _close(out.reshape(-1, H, hd), ref, _attn_tol(case, ref), BF16_ULP)


@pytest.mark.parametrize("H,Hkv,hd,window", [(8, 2, 128, None), (6, 2, 48, None), (4, 4, 16, 37), (3, 1, 32, None),
                                             (40, 2, 64, 100), (8, 8, 80, None)])
@pytest.mark.parametrize("teams", [7, 12, 40, "by hand"])
def test_attn_decode_with_a_work_list(H, Hkv, hd, window, teams):
    """The keys of a long sequence are cut into more parts than those of a short one (the parts merged by
    the block that finishes last); a team of blocks may also be given several segments, one after another."""
    ops = _ops()
    from longbow_quarrel_b200.kernels.attention import cut_decode_work, MAX_SPLITS
    lens = [300, 1, 77, 64, 17, 1500, 33]
    case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=3)
    tok_seq = list(range(len(lens)))
    tok_pos = [n - 1 for n in lens]
    q = _rand((len(tok_seq), (H + 2 * Hkv) * hd), torch.bfloat16, 78)
    scale = hd ** -0.5
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd).float(), tok_seq, tok_pos, H, scale, window)
    if teams == "by hand":
        # three teams: whole short tokens one after another; a token shared by two teams, one of which goes on
        first = [max(0, p - window + 1) // 16 if window and p >= window else 0 for p in tok_pos]
        tiles = [p // 16 + 1 - f for p, f in zip(tok_pos, first)]
        half = tiles[5] // 2
        shared = [(5, 0, half, 0, 2), (5, half, tiles[5], 1, 2)] if half else [(5, 0, tiles[5], 0, 1)]
        segments = [[(b, 0, tiles[b], 0, 1) for b in (0, 1, 2)], shared[:1], shared[1:] + [(b, 0, tiles[b], 0, 1) for b in (3, 4, 6)]]
        teams, offsets = 3, [0, 3, 4, 4 + len(segments[2])]
        work = np.asarray(offsets + [x for team in segments for seg in team for x in seg], dtype=np.int32)
    else:
        work = cut_decode_work(tok_pos, int(window or 0), teams)
        if teams > len(lens) and not window:
            assert work[teams + 1:].reshape(-1, 5)[:work[teams], 4].max() > 1      # the long token has several parts
    for early in (False, True):
        out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _ints(tok_pos), _ints(tok_seq), case.slots,
                              H, Hkv, hd, case.page_size, scale, window, min(MAX_SPLITS, teams), early_loads=early,
                              work=_ints(work.tolist()), teams=teams)
        _close(out.reshape(-1, H, hd), ref, _attn_tol(case, ref), BF16_ULP)
        again = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _ints(tok_pos), _ints(tok_seq), case.slots,
                                H, Hkv, hd, case.page_size, scale, window, min(MAX_SPLITS, teams), early_loads=early,
                                work=_ints(work.tolist()), teams=teams)
        assert torch.equal(out, again)                       # the counters are back at zero; the merge has a fixed order


@pytest.mark.parametrize("far_key", [0, 5, 250, 511, 700])
def test_attn_decode_finds_a_far_key(far_key):
    """One key among hundreds is made to stand out; the output must be its value."""
    ops = _ops()
    H, Hkv, hd = 4, 2, 64
    n = 701
    case = PagedCase([n], Hkv, hd, torch.bfloat16, seed=4)
    q = _rand((1, H * hd), torch.bfloat16, 79)
    # Put a scaled copy of each head's query into the far key of its kv head (both heads of a
    # group then share it: use the group's first head and check that head).
    G = H // Hkv
    slot = case.slot_of[0]
    page = int(case.table[slot, far_key // 64])
    for kvh in range(Hkv):
        qh = q[0, (kvh * G) * hd:(kvh * G + 1) * hd].float()
        key = (qh / qh.norm() * 40.0).to(torch.bfloat16)
        case.k_pages[page, kvh, far_key % 64] = key
        case.k[0][far_key, kvh] = key
    scale = 1.0
    from longbow_quarrel_b200.kernels.attention import cut_decode_work
    for n_splits in (1, 4, "teams"):
        if n_splits == "teams":
            out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _ints([n - 1]), _ints([0]), case.slots,
                                  H, Hkv, hd, 64, scale, None, 5, work=_ints(cut_decode_work([n - 1], 0, 5).tolist()),
                                  teams=5).reshape(H, hd)
        else:
            out = ops.attn_decode(q, case.k_pages, case.v_pages, case.table, _ints([n - 1]), _ints([0]), case.slots,
                                  H, Hkv, hd, 64, scale, None, n_splits).reshape(H, hd)
        for kvh in range(Hkv):
            _close(out[kvh * G], case.v[0][far_key, kvh], 2e-2)


def _query_blocks(tok_seq_lens, past):
    """Blocks of at most 64 rows: (sequence, first packed row, rows, first position)."""
    out, row = [], 0
    for b, (n, p) in enumerate(zip(tok_seq_lens, past)):
        for r in range(0, n, 64):
            out.append((b, row + r, min(64, n - r), p + r))
        row += n
    arr = np.asarray(out, dtype=np.int32)
    return tuple(torch.from_numpy(np.ascontiguousarray(arr[:, i])).to(DEV) for i in range(4))


@pytest.mark.parametrize("H,Hkv,hd,window", [(8, 2, 128, None), (6, 2, 48, None), (4, 4, 16, 37), (3, 1, 32, None),
                                             (4, 2, 64, 100), (2, 2, 80, 64)])
def test_attn_prefill(H, Hkv, hd, window):
    """Three sequences in one call: one whole from position 0, one single token, one that
    continues after 70 cached tokens."""
    ops = _ops()
    lens = [300, 1, 200]            # keys in the cache after the step
    new = [300, 1, 130]             # rows of this step
    past = [0, 0, 70]
    case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=6)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [p + i for n, p in zip(new, past) for i in range(n)]
    q = _rand((sum(new), (H + 2 * Hkv) * hd), torch.bfloat16, 81)
    scale = hd ** -0.5
    out = ops.attn_prefill(q, case.k_pages, case.v_pages, case.table, case.slots, _ints(lens), _query_blocks(new, past),
                           H, Hkv, hd, 64, scale, window)
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd).float(), tok_seq, tok_pos, H, scale, window)
    _close(out.reshape(-1, H, hd), ref, _attn_tol(case, ref), BF16_ULP)


def test_attn_prefill_window_edge_and_far_key():
    """Keys made to stand out just inside and just outside the window, and at position 0
    of a long sequence: the row's output must be the value of the visible one."""
    ops = _ops()
    H = Hkv = 1
    hd, n, W = 64, 400, 50
    case = PagedCase([n], Hkv, hd, torch.bfloat16, seed=7)
    q = _rand((n, hd), torch.bfloat16, 82)
    slot = case.slot_of[0]

    def plant(key_pos, query_row):
        qh = q[query_row].float()
        key = (qh / qh.norm() * 40.0).to(torch.bfloat16)
        case.k_pages[int(case.table[slot, key_pos // 64]), 0, key_pos % 64] = key
        case.k[0][key_pos, 0] = key

    plant(0, 399)            # far key: visible to row 399 without a window, hidden with one
    plant(300, 349)          # distance 49: the last key inside a window of 50
    plant(250, 300)          # distance 50: just outside
    blocks = _query_blocks([n], [0])
    full = ops.attn_prefill(q, case.k_pages, case.v_pages, case.table, case.slots, _ints([n]), blocks, 1, 1, hd, 64,
                            1.0, None)
    win = ops.attn_prefill(q, case.k_pages, case.v_pages, case.table, case.slots, _ints([n]), blocks, 1, 1, hd, 64,
                           1.0, W)
    _close(full[399], case.v[0][0, 0], 2e-2)
    _close(win[349], case.v[0][300, 0], 2e-2)
    ref = case.reference(q.reshape(n, 1, hd).float(), [0] * n, list(range(n)), 1, 1.0, W)
    _close(win.reshape(n, 1, hd), ref, _attn_tol(case, ref), BF16_ULP)
    assert float((win[300].float() - case.v[0][250, 0].float()).abs().max()) > 0.5     # the key outside is not seen
    assert float((win[399].float() - case.v[0][0, 0].float()).abs().max()) > 0.5


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("H,Hkv,hd,rotate", [(4, 2, 32, True), (6, 1, 128, True), (2, 2, 48, False)])
def test_gemm_skinny_qkv_rotates_and_stores(M, H, Hkv, hd, rotate):
    """The fused decode projection against product, rotation and cache write done apart."""
    ops = _ops()
    K = 200
    lens = [70 + 5 * i for i in range(M)]
    case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=11)
    k_before, v_before = case.k_pages.clone(), case.v_pages.clone()
    a = _rand((M, K), torch.bfloat16, 40)
    w = _rand(((H + 2 * Hkv) * hd, K), torch.bfloat16, 41, 0.1)
    tok_pos, tok_seq = [n - 1 for n in lens], list(range(M))
    freqs = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    ang = torch.arange(256, dtype=torch.float64)[:, None] * freqs[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    q = ops.gemm_skinny_qkv(a, w, cos if rotate else None, sin if rotate else None, _ints(tok_pos), _ints(tok_seq),
                            case.slots, case.table, case.k_pages, case.v_pages, H, Hkv, hd, 64)
    full = (a.float().double() @ w.float().double().T).reshape(M, H + 2 * Hkv, hd)
    c = cos[torch.tensor(tok_pos)].double().cpu().unsqueeze(1) if rotate else 1.0
    s = sin[torch.tensor(tok_pos)].double().cpu().unsqueeze(1) if rotate else 0.0
    x0, x1 = full.cpu()[:, :H + Hkv, :hd // 2], full.cpu()[:, :H + Hkv, hd // 2:]
    rot = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)
    _close(q.reshape(M, H, hd), rot[:, :H], _acc_tol(K), BF16_ULP)
    touched = torch.zeros_like(case.k_pages, dtype=torch.bool)
    for m in range(M):
        page = int(case.table[case.slot_of[m], tok_pos[m] // 64])
        _close(case.k_pages[page, :, tok_pos[m] % 64], rot[m, H:], _acc_tol(K), BF16_ULP)
        _close(case.v_pages[page, :, tok_pos[m] % 64], full.cpu()[m, H + Hkv:], _acc_tol(K), BF16_ULP)
        touched[page, :, tok_pos[m] % 64] = True
    for pages, before in ((case.k_pages, k_before), (case.v_pages, v_before)):
        same = (pages == before) | (pages.isnan() & before.isnan())
        assert bool((same | touched).all())          # nothing else in the cache was written


@pytest.mark.parametrize("M,K", [(17, 4096), (64, 328), (300, 200), (1100, 1024)])
@pytest.mark.parametrize("H,Hkv,hd,rotate", [(4, 2, 128, True), (6, 1, 64, True), (3, 3, 128, False)])
def test_gemm_tc_qkv_rotates_and_stores(M, K, H, Hkv, hd, rotate):
    """The fused projection of many rows (tiles, or ranges of K added by the second kernel) against
    product, rotation and cache write done apart; rows of several sequences, some continuing."""
    _check_gemm_tc_qkv(M, K, H, Hkv, hd, rotate)


@pytest.mark.parametrize("M,K,H,Hkv,hd,rotate", [(2500, 1032, 32, 8, 128, True), (1111, 520, 52, 7, 64, True),
                                                 (2048, 256, 24, 8, 128, False)])
def test_gemm_pair_qkv_rotates_and_stores(M, K, H, Hkv, hd, rotate):
    """The same on pairs of SMs (tiles of 256 x 256): enough rows and heads that the pair kernel takes the product."""
    ops = _ops()
    assert ops.gemm_pair_takes(M, (H + 2 * Hkv) * hd, K)
    before = ops.launches_by_name()
    _check_gemm_tc_qkv(M, K, H, Hkv, hd, rotate)
    assert ops.launches_since(before).get("gemm_pair_qkv") == 1
    assert ops.gemm_pair_status() == 0


def _check_gemm_tc_qkv(M, K, H, Hkv, hd, rotate):
    ops = _ops()
    n_seq = 5
    new = [M // n_seq + (1 if b < M % n_seq else 0) for b in range(n_seq)]
    past = [0, 70, 3, 129, 64]
    lens = [p + n for p, n in zip(past, new)]
    case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=21)
    k_before, v_before = case.k_pages.clone(), case.v_pages.clone()
    a = _rand((M, K), torch.bfloat16, 90)
    w = _rand(((H + 2 * Hkv) * hd, K), torch.bfloat16, 91, 0.1)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [past[b] + i for b, n in enumerate(new) for i in range(n)]
    freqs = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    ang = torch.arange(max(lens) + 1, dtype=torch.float64)[:, None] * freqs[None]
    cos, sin = torch.cos(ang).float().to(DEV).contiguous(), torch.sin(ang).float().to(DEV).contiguous()
    q = ops.gemm_tc_qkv(a, w, cos if rotate else None, sin if rotate else None, _ints(tok_pos), _ints(tok_seq),
                        case.slots, case.table, case.k_pages, case.v_pages, H, Hkv, hd, 64)
    torch.cuda.synchronize()
    assert ops.gemm_tc_status() == 0
    full = (a.float().double() @ w.float().double().T).reshape(M, H + 2 * Hkv, hd).cpu()
    c = cos[torch.tensor(tok_pos)].double().cpu().unsqueeze(1) if rotate else 1.0
    s = sin[torch.tensor(tok_pos)].double().cpu().unsqueeze(1) if rotate else 0.0
    x0, x1 = full[:, :H + Hkv, :hd // 2], full[:, :H + Hkv, hd // 2:]
    rot = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)
    tol = _acc_tol(K) + 1e-6
    _close(q.reshape(M, H, hd), rot[:, :H], tol, BF16_ULP)
    touched = torch.zeros_like(case.k_pages, dtype=torch.bool)
    pages = torch.tensor([int(case.table[case.slot_of[tok_seq[m]], tok_pos[m] // 64]) for m in range(M)])
    offs = torch.tensor([p % 64 for p in tok_pos])
    _close(case.k_pages[pages, :, offs], rot[:, H:], tol, BF16_ULP)
    _close(case.v_pages[pages, :, offs], full[:, H + Hkv:], tol, BF16_ULP)
    touched[pages, :, offs] = True
    for pg, before in ((case.k_pages, k_before), (case.v_pages, v_before)):
        same = (pg == before) | (pg.isnan() & before.isnan())
        assert bool((same | touched).all())          # nothing else in the cache was written


def _query_blocks128(new, past):
    out, row = [], 0
    for b, (n, p) in enumerate(zip(new, past)):
        for r in range(0, n, 128):
            out.append((b, row + r, min(128, n - r), p + r))
        row += n
    arr = np.asarray(out, dtype=np.int32)
    return tuple(torch.from_numpy(np.ascontiguousarray(arr[:, i])).to(DEV) for i in range(4))


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("H,Hkv,window", [(8, 2, None), (4, 4, 100), (2, 1, 300)])
def test_attn_prefill_tc(H, Hkv, window, hd):
    """The tcgen05 prefill attention: three sequences in one call (whole from position 0; one
    token; one continuing after 70 cached tokens), unused cache rows poisoned with huge finite
    values, so that a key read beyond a sequence shows."""
    ops = _ops()
    lens, new, past = [700, 1, 330], [700, 1, 260], [0, 0, 70]
    case = PagedCase(lens, Hkv, hd, torch.bfloat16, seed=12, poison=3.0e38)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [p + i for n, p in zip(new, past) for i in range(n)]
    q = _rand((sum(new), (H + 2 * Hkv) * hd), torch.bfloat16, 83)
    scale = hd ** -0.5
    out = ops.attn_prefill_tc(q, case.k_pages, case.v_pages, case.table, case.slots, _ints(lens),
                              _query_blocks128(new, past), H, Hkv, hd, 64, scale, window)
    torch.cuda.synchronize()
    assert ops.attn_prefill_tc_status() == 0
    ref = case.reference(q[:, :H * hd].reshape(-1, H, hd).float(), tok_seq, tok_pos, H, scale, window)
    _close(out.reshape(-1, H, hd), ref, _attn_tol(case, ref), BF16_ULP)


@pytest.mark.parametrize("hd", [128, 64])
def test_attn_prefill_tc_far_key_and_growing_maximum(hd):
    """Scores that grow along the keys (the reference maximum has to move and O be rescaled
    several times), and a key made to stand out at position 0 of a long sequence."""
    ops = _ops()
    H = Hkv = 1
    n = 900
    case = PagedCase([n], Hkv, hd, torch.bfloat16, seed=13, poison=3.0e38)
    q = _rand((n, hd), torch.bfloat16, 84)
    slot = case.slot_of[0]
    # keys aligned with a fixed direction and growing in length: scores rise steadily with the key index
    direction = torch.nn.functional.normalize(_rand((hd,), torch.float32, 85), dim=0)
    q[:, :] = (direction * 6.0).to(torch.bfloat16)
    for pos in range(n):
        key = (direction * (pos / 15.0)).to(torch.bfloat16)
        case.k_pages[int(case.table[slot, pos // 64]), 0, pos % 64] = key
        case.k[0][pos, 0] = key
    blocks = _query_blocks128([n], [0])
    out = ops.attn_prefill_tc(q, case.k_pages, case.v_pages, case.table, case.slots, _ints([n]), blocks, 1, 1, hd, 64,
                              1.0, None)
    ref = case.reference(q.reshape(n, 1, hd).float(), [0] * n, list(range(n)), 1, 1.0, None)
    _close(out.reshape(n, 1, hd), ref, _attn_tol(case, ref), BF16_ULP)
    # a far key: position 0 dominates row 899
    far = (direction * 200.0).to(torch.bfloat16)
    case.k_pages[int(case.table[slot, 0]), 0, 0] = far
    case.k[0][0, 0] = far
    out = ops.attn_prefill_tc(q, case.k_pages, case.v_pages, case.table, case.slots, _ints([n]), blocks, 1, 1, hd, 64,
                              1.0, None)
    _close(out[899], case.v[0][0, 0], 2e-2)
    torch.cuda.synchronize()
    assert ops.attn_prefill_tc_status() == 0

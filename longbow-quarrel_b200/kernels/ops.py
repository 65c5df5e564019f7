"""Python faces of the CUDA kernels.

Every function takes torch tensors that live on the GPU, checks what the kernel
cannot check itself, and launches on torch's current stream.  There is no
fallback: a tensor on the CPU, or a library that cannot be built, is an error.
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor | torch.dtype) -> int:
    dt = t if isinstance(t, torch.dtype) else t.dtype
    try:
        return _CODES[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dt}") from None


def _p(t: torch.Tensor | None):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("the kernels run on the GPU only: got a tensor on " + str(t.device))
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0
_by_name: dict[str, int] = {}


def launch_count() -> int:
    """Kernels launched so far by this process (replays of a captured step count the
    kernels the capture recorded)."""
    return _launches


def launches_by_name() -> dict[str, int]:
    """How often each launcher has run so far (a copy): which kernels a piece of work went through."""
    return dict(_by_name)


def add_launches(n: int, by_name: dict[str, int] | None = None, sign: int = 1) -> None:
    """Count `n` kernels that were recorded or replayed rather than launched here; `by_name` says which."""
    global _launches
    _launches += n
    for name, k in (by_name or {}).items():
        _by_name[name] = _by_name.get(name, 0) + sign * k


def launches_since(before: dict[str, int]) -> dict[str, int]:
    return {name: k - before.get(name, 0) for name, k in _by_name.items() if k != before.get(name, 0)}


def _check(code: int, what: str, kernels: int = 1, variant: str | None = None) -> None:
    """`variant` names the path inside the launcher that the sizes chose (counted beside the launcher)."""
    global _launches
    if code == 0:
        _launches += kernels
        _by_name[what] = _by_name.get(what, 0) + 1
        if variant:
            _by_name[variant] = _by_name.get(variant, 0) + 1
        return
    reason = {-1: "unsupported dtype", -2: "unsupported size", -3: "CUDA driver entry point not found",
              -4: "scratch too small"}.get(code, f"CUDA error {code}")
    raise KernelError(f"{what}: {reason}")


_declared: set[tuple[str, str]] = set()


# Libraries whose kernels wait on barriers with a time limit, and what their status codes mean.
_WATCHED = {"gemm_tc": {1: "the TMA producer waited for a free stage", 2: "the product issuer waited for a free accumulator",
                        3: "the product issuer waited for a stage's copies", 4: "the epilogue waited for an accumulator"},
            "gemm_pair": {1: "a TMA producer waited for a free stage", 2: "the product issuer waited for a free accumulator",
                          3: "the product issuer waited for a stage's copies", 4: "an epilogue waited for an accumulator"},
            "attn_prefill_tc": {}}
_status_words: dict[str, object] = {}


def _watch(lib: str, handle) -> None:
    """Set up the library's status word in mapped host memory (once; not while a stream is being captured,
    since the set-up copies a pointer to the device)."""
    if lib in _status_words or torch.cuda.is_current_stream_capturing():
        return
    from ctypes import POINTER
    fn = getattr(handle, f"lq_{lib}_status_word")
    fn.restype = POINTER(c_int)
    fn.argtypes = []
    _status_words[lib] = fn()


def check_status() -> None:
    """Raise if a bounded wait inside a tensor-core kernel gave up since the last check.  It reads words
    in host memory that such a kernel writes through, so it costs no CUDA call and sees everything that
    ran before the host's last synchronisation: call it where the host has just waited for results."""
    for lib, word in _status_words.items():
        if word and word[0]:
            code = int(word[0])
            word[0] = 0
            why = _WATCHED[lib].get(code, "a wait on a barrier")
            raise KernelError(f"{lib}: {why} for two seconds and gave up (code {code}); the step's results are not valid")


def _fn(lib: str, name: str, argtypes):
    handle = build.load(lib)
    if lib in _WATCHED:
        _watch(lib, handle)
    fn = getattr(handle, name)
    if (lib, name) not in _declared:
        fn.argtypes = argtypes
        fn.restype = c_int
        _declared.add((lib, name))
    return fn


def _contig(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t


def prepare(dtype: torch.dtype, verbose: bool = True) -> None:
    """Build and load the libraries a model of this dtype uses, before the first step."""
    from concurrent.futures import ThreadPoolExecutor
    names = ["plain_kernels"] + (["gemm_skinny", "gemm_tc", "attn_decode", "attn_prefill", "attn_prefill_tc"]
                                             if dtype == torch.bfloat16 else [])
    with ThreadPoolExecutor(max_workers=len(names)) as pool:
        list(pool.map(build.build, names))
    for name in names:
        build.load(name)


# ------------------------------------------------------------------ plain kernels

def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32 (the residual stream starts in 32-bit)."""
    V, D = table.shape
    T = tokens.numel()
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    fn = _fn("plain_kernels", "lq_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(table, "table")), dtype_code(table), _p(tokens), _p(out), T, D, V, _stream()), "embedding")
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMS norm of rows of the float32 stream x [T, D]; `rows` (int32) picks rows."""
    if x.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("rmsnorm reads a float32 stream and float32 gains")
    D = x.shape[-1]
    n = x.shape[0] if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n, D), dtype=out_dtype, device=x.device)
    fn = _fn("plain_kernels", "lq_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_p(_contig(x, "x")), _p(gain), _p(rows), _p(out), dtype_code(out_dtype), n, D, float(eps), _stream()), "rmsnorm")
    return out


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T (+ residual) on the CUDA cores, every product in float32."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: input width {K} does not match weight width {K2}")
    if residual is not None:
        if residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError("linear: residual must be float32 [M, N]")
        if out is None:
            out = residual
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    fn = _fn("plain_kernels", "lq_gemm_plain", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                                c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(a, "a")), dtype_code(a), _p(_contig(w, "w")), dtype_code(w), _p(out), dtype_code(out),
              _p(residual), M, N, K, _stream()), "linear")
    return out


def _check_tables(what: str, cos, sin, hd: int, tok_pos=None) -> None:
    """The fused q/k/v epilogues read cos/sin at [position, head_dim / 2]: tables of another width (a part
    that rotates only some of a head's dimensions) would be read across rows."""
    if cos is None and sin is None:
        return
    if cos is None or sin is None:
        raise KernelError(f"{what}: cos and sin tables come together")
    for t in (cos, sin):
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != hd // 2 or not t.is_contiguous():
            raise KernelError(f"{what}: cos/sin tables must be contiguous float32 [positions, head_dim / 2 = {hd // 2}], "
                              f"found {tuple(t.shape)} {t.dtype}")
    if cos.shape != sin.shape:
        raise KernelError(f"{what}: cos {tuple(cos.shape)} and sin {tuple(sin.shape)} differ")


def rope_kv_write(qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None, tok_pos, tok_seq, slots,
                  page_table: torch.Tensor | None, k_pages: torch.Tensor | None, v_pages: torch.Tensor | None,
                  H: int, Hkv: int, hd: int, page_size: int) -> None:
    """Rotate q and k of every token in place and store k, v into the cache pages."""
    T = qkv.shape[0]
    has_kv = k_pages is not None
    width = (H + (2 * Hkv if has_kv else 0)) * hd
    if qkv.shape[1] != width:
        raise KernelError(f"rope: qkv rows are {qkv.shape[1]} wide, expected {width}")
    if has_kv and (k_pages.dtype != qkv.dtype or v_pages.dtype != qkv.dtype):
        raise KernelError("rope: the cache and the activations must have one dtype")
    _check_tables("rope", cos, sin, hd)
    fn = _fn("plain_kernels", "lq_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                   c_int, c_int, c_void_p])
    _check(fn(_p(_contig(qkv, "qkv")), dtype_code(qkv), _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(slots),
              _p(page_table), page_table.stride(0) if page_table is not None else 0, _p(k_pages), _p(v_pages),
              T, H, Hkv, hd, page_size, int(has_kv), _stream()), "rope_kv_write")


def attention_plain(q: torch.Tensor, k_pages, v_pages, page_table, tok_pos, tok_seq, slots, H: int, Hkv: int,
                    hd: int, page_size: int, scale: float, window: int | None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of every token over its own sequence's cache; q is the left
    H*hd columns of a [T, q_stride] buffer."""
    T = q.shape[0]
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} exceeds 256")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    fn = _fn("plain_kernels", "lq_attention_plain", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                     c_int, c_float, c_int, c_void_p])
    _check(fn(_p(q), q.stride(0), dtype_code(q), _p(k_pages), _p(v_pages), _p(page_table), page_table.stride(0),
              _p(tok_pos), _p(tok_seq), _p(slots), _p(out), T, H, Hkv, hd, page_size, float(scale),
              int(window or 0), _stream()), "attention")
    return out


def swiglu(gu: torch.Tensor, block: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """gu [T, 2F] -> up * silu(gate) [T, F].  block 0: gate columns, then up columns;
    block b: b gate columns, b up columns, alternating."""
    T, F2 = gu.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    fn = _fn("plain_kernels", "lq_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(gu, "gu")), _p(out), dtype_code(gu), T, F, block, _stream()), "swiglu")
    return out


def clear_page_tails(k_pages: torch.Tensor, v_pages: torch.Tensor, items: list[tuple[int, int]]) -> None:
    """Zero the rows [first, page_size) of the pages in `items` = [(page, first)], in every entry and kv
    head of the pools k_pages, v_pages [entries, pages, kv heads, page_size, head_dim]."""
    from ctypes import c_int as _int
    E, P, Hkv, page_size, hd = k_pages.shape
    if v_pages.shape != k_pages.shape or v_pages.dtype != k_pages.dtype:
        raise KernelError("clear_page_tails: keys and values must have one shape and dtype")
    n = len(items)
    pages = (_int * n)(*[int(p) for p, _ in items])
    first = (_int * n)(*[int(f) for _, f in items])
    from ctypes import POINTER
    fn = _fn("plain_kernels", "lq_clear_page_tails", [c_void_p, c_void_p, c_int, POINTER(c_int), POINTER(c_int), c_int,
                                                      c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_p(_contig(k_pages, "k_pages")), _p(_contig(v_pages, "v_pages")), dtype_code(k_pages), pages, first, n,
              E, P, Hkv, page_size, hd, _stream()), "clear_page_tails", -(-n // 120))


# ------------------------------------------------------------------ bfloat16 tensor-core kernels
EPI_BF16, EPI_F32, EPI_RESID, EPI_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_ROWS = 64          # most rows gemm_skinny takes
SKINNY_BEST_ROWS = int(os.environ.get("LQ_SKINNY_BEST_ROWS", "16"))         # up to here streaming W through registers beats the TMA-fed tcgen05 kernel in a step

_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (the current one by default)."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def streams_through_registers(M: int, N: int) -> bool:
    """Whether a product of M rows with a weight of N rows goes to gemm_skinny rather than gemm_tc: up to 16 rows.
    Timed alone at 16 rows gemm_tc is the faster kernel for every weight but the square output projection
    ([28672, 4096]: 48 us against 54; the head [128256, 4096]: 167 against 211), yet a whole model runs no
    faster with it (8B shape, 16 rows, context 2,048: 4.47 ms a step with gemm_tc for every product, 4.40 with
    gemm_skinny), and 15 % slower when only the products of more than one wave of blocks take it, as the single
    timings suggest (6.11 against 5.43 ms at context 4,096): its blocks fill a multiprocessor, so nothing of the
    kernel after it overlaps with it.  From 17 rows on gemm_tc wins (17 rows: 4.50 against 5.69 ms)."""
    return M <= SKINNY_BEST_ROWS


class NormedRows:
    """Rows of an RMS norm whose 1 / rms is still to be applied, as the residual epilogue of
    gemm_skinny leaves them: `data` = residual * gain in bfloat16 [M, width]; `sums` float32
    [M, blocks], each row's sum of squares cut into column blocks; `eps` of the norm.  A product
    that reads them multiplies its result by 1 / sqrt(sum(sums) / width + eps)."""

    __slots__ = ("data", "sums", "eps")

    def __init__(self, data: torch.Tensor, sums: torch.Tensor, eps: float):
        self.data, self.sums, self.eps = data, sums, float(eps)

    @property
    def shape(self):
        return self.data.shape

    @property
    def dtype(self):
        return self.data.dtype

    def finish(self) -> torch.Tensor:
        """The normalised rows themselves (for an operation that cannot take them unfinished)."""
        scale = torch.rsqrt(self.sums.sum(dim=1, keepdim=True) / self.data.shape[1] + self.eps)
        return (self.data.to(torch.float32) * scale).to(self.data.dtype)


def _norm_in(a):
    """(tensor, sums pointer, blocks, 1 / width, eps) of plain or unfinished rows."""
    if isinstance(a, NormedRows):
        if a.sums.dtype != torch.float32 or a.sums.shape[0] != a.data.shape[0] or not a.sums.is_contiguous():
            raise KernelError("unfinished rows: sums must be contiguous float32 [rows, blocks]")
        return a.data, _p(a.sums), a.sums.shape[1], 1.0 / a.data.shape[1], a.eps
    return a, None, 0, 0.0, 0.0


PREFETCH_BYTES = int(float(os.environ.get("LQ_PREFETCH_MB", "8")) * (1 << 20))   # of the weights read next; 0: none


# The same, asked by the decode attention, which leaves HBM a third idle: all of a 34 MB output projection
# (measured: a decode step 0.8 % shorter than with 8 MB).
PREFETCH_BYTES_ATTN = int(float(os.environ.get("LQ_PREFETCH_ATTN_MB", "48")) * (1 << 20))


def _next(next_w, limit=None):
    """(pointer, bytes) of the piece of the next weights to ask into L2."""
    limit = PREFETCH_BYTES if limit is None else limit
    if next_w is None or limit <= 0:
        return None, 0
    return _p(next_w), min(limit, next_w.numel() * next_w.element_size())


def gemm_skinny(a, w: torch.Tensor, epi: int, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, emit: tuple | None = None, next_w: torch.Tensor | None = None):
    """a [M <= 64, K] . w [N, K]^T, both bfloat16, streaming w once from memory.
    epi: EPI_BF16 / EPI_F32 store; EPI_RESID adds into the float32 `residual` in place;
    EPI_SWIGLU reads w as alternating blocks of 8 gate and 8 up rows and stores
    up * silu(gate) [M, N / 2].
    `a` may be NormedRows.  emit = (gain [N] float32, eps), with EPI_RESID only: also returns what the
    RMS norm with that gain makes of the new residual, as NormedRows: (residual, rows).
    next_w: the weights that the stream reads after these; their first bytes are asked into L2."""
    a, in_sums, in_blocks, in_inv, in_eps = _norm_in(a)
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny takes bfloat16 inputs")
    if w.shape[1] != K:
        raise KernelError(f"linear: input width {K} does not match weight width {w.shape[1]}")
    if M > SKINNY_MAX_ROWS or K % 8:
        raise KernelError(f"gemm_skinny: {M} rows (at most {SKINNY_MAX_ROWS}) and width {K} (a multiple of 8)")
    if epi == EPI_RESID:
        if residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError("linear: residual must be float32 [M, N]")
        out = residual
    elif out is None:
        shape = (M, N // 2) if epi == EPI_SWIGLU else (M, N)
        out = torch.empty(shape, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    rows = None
    gain = None
    if emit is not None:
        gain, eps = emit
        if epi != EPI_RESID or gain.dtype != torch.float32 or gain.numel() != N:
            raise KernelError("gemm_skinny: rows for the next norm come with EPI_RESID and a float32 gain [N]")
        rows = NormedRows(torch.empty((M, N), dtype=torch.bfloat16, device=a.device),
                          torch.empty((M, -(-N // 16)), dtype=torch.float32, device=a.device), eps)
    fn = _fn("gemm_skinny", "lq_gemm_skinny", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                               c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_long, c_void_p])
    next_p, next_n = _next(next_w)
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), _p(residual), M, N, K, epi, in_sums, in_blocks, in_inv,
              in_eps, _p(gain), _p(rows.data) if rows else None, _p(rows.sums) if rows else None, next_p, next_n,
              _stream()), "gemm_skinny", 1, f"gemm_skinny:rows{-(-M // 8) * 8}" + (":norm_in" if in_blocks else "")
           + (":norm_out" if rows else ""))
    return (out, rows) if emit is not None else out


def gemm_skinny_qkv(a, w: torch.Tensor, cos, sin, tok_pos, tok_seq, slots, page_table, k_pages, v_pages,
                    H: int, Hkv: int, hd: int, page_size: int, out: torch.Tensor | None = None,
                    next_w: torch.Tensor | None = None) -> torch.Tensor:
    """The q/k/v projection of at most 16 tokens with rotation and cache write in its epilogue:
    returns the rotated q [M, H*hd]; the rotated k and v are stored in each token's cache page.
    `a` may be NormedRows."""
    a, in_sums, in_blocks, in_inv, in_eps = _norm_in(a)
    M, K = a.shape
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny_qkv takes bfloat16 inputs and cache")
    if tuple(w.shape) != ((H + 2 * Hkv) * hd, K):
        raise KernelError(f"gemm_skinny_qkv: weight shape {tuple(w.shape)} is not [(H + 2 Hkv) hd, K]")
    if M > SKINNY_BEST_ROWS or K % 8 or hd % 16:
        raise KernelError(f"gemm_skinny_qkv: {M} rows (at most 16), width {K} (multiple of 8), head_dim {hd} (multiple of 16)")
    _check_tables("gemm_skinny_qkv", cos, sin, hd)
    if out is None:
        out = torch.empty((M, H * hd), dtype=torch.bfloat16, device=a.device)
    fn = _fn("gemm_skinny", "lq_gemm_skinny_qkv", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_void_p, c_int, c_float, c_float, c_void_p, c_long,
                                                   c_void_p])
    next_p, next_n = _next(next_w)
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), M, K, _p(cos), _p(sin), _p(tok_pos), _p(tok_seq),
              _p(slots), _p(page_table), page_table.stride(0), _p(k_pages), _p(v_pages), H, Hkv, hd, page_size,
              in_sums, in_blocks, in_inv, in_eps, next_p, next_n, _stream()), "gemm_skinny_qkv", 1,
           f"gemm_skinny_qkv:rows{-(-M // 8) * 8}" + (":norm_in" if in_blocks else ""))
    return out


USE_PAIRS = True        # many rows: products on pairs of SMs (tcgen05 cta_group::2) where gemm_pair takes the sizes


def gemm_pair_takes(M: int, N: int, K: int) -> bool:
    """Whether the product of these sizes runs on pairs of SMs (256 x 256 tiles fill the pairs at least once)."""
    return USE_PAIRS and bool(_fn("gemm_pair", "lq_gemm_pair_takes", [c_int, c_int, c_int])(M, N, K))


def gemm_pair_status() -> int:
    fn = build.load("gemm_pair").lq_gemm_pair_status
    fn.restype = c_int
    return int(fn())


def _gemm_tc_scratch_floats(M: int, N: int, K: int) -> int:
    fn = build.load("gemm_tc").lq_gemm_tc_scratch_floats
    fn.argtypes, fn.restype = [c_int, c_int, c_int], c_long
    return int(fn(M, N, K))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, epi: int, residual: torch.Tensor | None = None,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T on the tcgen05 tensor cores (TMA-fed, float32 accumulation in
    tensor memory), with the epilogues of gemm_skinny.  For many rows; with few tiles (few rows
    and a narrow weight) the contraction is cut into ranges that a second kernel adds."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 inputs")
    if w.shape[1] != K:
        raise KernelError(f"linear: input width {K} does not match weight width {w.shape[1]}")
    if K % 8:
        raise KernelError(f"gemm_tc: width {K} must be a multiple of 8 (16-byte rows for TMA)")
    if epi == EPI_RESID:
        if residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError("linear: residual must be float32 [M, N]")
        out = residual
    elif out is None:
        shape = (M, N // 2) if epi == EPI_SWIGLU else (M, N)
        out = torch.empty(shape, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    out_cols = N // 2 if epi == EPI_SWIGLU else N
    if (gemm_pair_takes(M, N, K) and out.is_contiguous() and out.data_ptr() % 16 == 0
            and (out_cols * out.element_size()) % 16 == 0 and a.is_contiguous() and w.is_contiguous()):
        # Many rows: tiles of 256 x 256 on pairs of SMs, the output leaving by TMA.
        fn = _fn("gemm_pair", "lq_gemm_pair", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_p(a), _p(w), _p(out), _p(residual), M, N, K, epi, _stream()), "gemm_pair")
        return out
    # Few tiles (few rows, narrow weight): the kernel cuts the contraction into ranges and adds them afterwards.
    splits = int(_fn("gemm_tc", "lq_gemm_tc_splits", [c_int, c_int, c_int])(M, N, K))
    scratch = torch.empty(_gemm_tc_scratch_floats(M, N, K), dtype=torch.float32, device=a.device) if splits > 1 else None
    fn = _fn("gemm_tc", "lq_gemm_tc", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p])
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), _p(residual), M, N, K, epi, _p(scratch), _stream()),
           "gemm_tc", 2 if splits > 1 else 1, "gemm_tc:split_k" if splits > 1 else ("gemm_tc:few_rows" if M <= 64 else None))
    return out


def gemm_tc_qkv(a: torch.Tensor, w: torch.Tensor, cos, sin, tok_pos, tok_seq, slots, page_table, k_pages, v_pages,
                H: int, Hkv: int, hd: int, page_size: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """The q/k/v projection of many rows (or of 17 and more decoded tokens) with rotation and cache
    write in its epilogue, on the tcgen05 kernel: returns the rotated q [M, H*hd]; the rotated k and v
    are stored in each row's cache page.  head_dim 64 or 128."""
    M, K = a.shape
    N = (H + 2 * Hkv) * hd
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_qkv takes bfloat16 inputs and cache")
    if tuple(w.shape) != (N, K):
        raise KernelError(f"gemm_tc_qkv: weight shape {tuple(w.shape)} is not [(H + 2 Hkv) hd, K]")
    if K % 8 or hd not in (64, 128):
        raise KernelError(f"gemm_tc_qkv: width {K} (multiple of 8), head_dim {hd} (64 or 128)")
    _check_tables("gemm_tc_qkv", cos, sin, hd)
    if out is None:
        out = torch.empty((M, H * hd), dtype=torch.bfloat16, device=a.device)
    if gemm_pair_takes(M, N, K) and a.is_contiguous() and w.is_contiguous():
        fn = _fn("gemm_pair", "lq_gemm_pair_qkv", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_void_p])
        _check(fn(_p(a), _p(w), _p(out), M, K, _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(slots), _p(page_table),
                  page_table.stride(0), _p(k_pages), _p(v_pages), H, Hkv, hd, page_size, _stream()), "gemm_pair_qkv")
        return out
    splits = int(_fn("gemm_tc", "lq_gemm_tc_splits", [c_int, c_int, c_int])(M, N, K))
    scratch = torch.empty(_gemm_tc_scratch_floats(M, N, K), dtype=torch.float32, device=a.device) if splits > 1 else None
    fn = _fn("gemm_tc", "lq_gemm_tc_qkv", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                           c_int, c_void_p, c_void_p])
    _check(fn(_p(_contig(a, "a")), _p(_contig(w, "w")), _p(out), M, K, _p(cos), _p(sin), _p(tok_pos), _p(tok_seq),
              _p(slots), _p(page_table), page_table.stride(0), _p(k_pages), _p(v_pages), H, Hkv, hd, page_size,
              _p(scratch), _stream()), "gemm_tc_qkv", 2 if splits > 1 else 1,
           "gemm_tc_qkv:split_k" if splits > 1 else ("gemm_tc_qkv:few_rows" if M <= 64 else None))
    return out


def gemm_tc_status() -> int:
    """0, or the code of a wait inside gemm_tc that gave up (after a synchronize)."""
    fn = build.load("gemm_tc").lq_gemm_tc_status
    fn.restype = c_int
    return int(fn())


def attn_prefill(q: torch.Tensor, k_pages, v_pages, page_table, slots, kv_len, query_blocks, H: int, Hkv: int, hd: int,
                 page_size: int, scale: float, window: int | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of blocks of query rows over the paged bfloat16 cache (flash style:
    tensor-core products, online softmax in float32).  query_blocks = (sequence, first row,
    rows, first position) int32 tensors, one entry for each block of at most 64 rows."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attn_prefill takes bfloat16 queries and cache")
    if hd % 16 or hd > 128 or page_size != 64:
        raise KernelError(f"attn_prefill: head_dim {hd} (multiple of 16, at most 128), page size {page_size} (64)")
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
    qb_seq, qb_row, qb_rows, qb_pos = query_blocks
    fn = _fn("attn_prefill", "lq_attn_prefill", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(page_table), page_table.stride(0), _p(slots), _p(kv_len),
              _p(qb_seq), _p(qb_row), _p(qb_rows), _p(qb_pos), _p(out), qb_seq.numel(), H, Hkv, hd, page_size,
              float(scale), int(window or 0), _stream()), "attn_prefill")
    return out


def attn_prefill_tc(q: torch.Tensor, k_pages, v_pages, page_table, slots, kv_len, query_blocks128, H: int, Hkv: int,
                    hd: int, page_size: int, scale: float, window: int | None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """attn_prefill on the tcgen05 tensor cores (TMA-fed, S and O in tensor memory): blocks of at
    most 128 query rows, head_dim 64 or 128, pages of 64 keys, a cache that is finite everywhere."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_tc takes bfloat16 queries and cache")
    if hd not in (64, 128) or page_size != 64:
        raise KernelError(f"attn_prefill_tc: head_dim {hd} (64 or 128) and page size {page_size} (64)")
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
    qb_seq, qb_row, qb_rows, qb_pos = query_blocks128
    fn = _fn("attn_prefill_tc", "lq_attn_prefill_tc", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_p(q), q.stride(0), T, _p(_contig(k_pages, "k_pages")), _p(_contig(v_pages, "v_pages")), k_pages.shape[0],
              _p(page_table), page_table.stride(0), _p(slots), _p(kv_len), _p(qb_seq), _p(qb_row), _p(qb_rows), _p(qb_pos),
              _p(out), qb_seq.numel(), H, Hkv, hd, page_size, float(scale), int(window or 0), _stream()), "attn_prefill_tc")
    return out


def attn_prefill_tc_status() -> int:
    fn = build.load("attn_prefill_tc").lq_attn_prefill_tc_status
    fn.restype = c_int
    return int(fn())


def attn_decode(q: torch.Tensor, k_pages, v_pages, page_table, tok_pos, tok_seq, slots, H: int, Hkv: int, hd: int,
                page_size: int, scale: float, window: int | None, n_splits: int,
                out: torch.Tensor | None = None, scratch: tuple | None = None,
                next_w: torch.Tensor | None = None, early_loads: bool = False,
                work: torch.Tensor | None = None, teams: int = 0) -> torch.Tensor:
    """Attention of single query rows over the paged bfloat16 cache, the keys of each
    sequence cut into n_splits slices that are merged afterwards.  With `work` (int32: teams + 1 offsets,
    then (token, first tile, last tile + 1, part, parts) per segment) the grid is `teams` blocks per kv
    head and row tile, each walking the segments between its offset and the next, and n_splits is the most
    parts any token has; the list must cover every tile of every token once (the kernel trusts it).  next_w: the weights that the
    stream reads after this; their first bytes are asked into L2 as the blocks finish.
    early_loads: of the keys and values a row reads, only those at its own position can have been
    written by the kernel ahead on the stream (a decode step: one new token per sequence); the kernel
    then requests the others without waiting for that kernel."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attn_decode takes bfloat16 queries and cache")
    if hd % 16 or hd > 128:
        raise KernelError(f"attn_decode: head_dim {hd} must be a multiple of 16 and at most 128")
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        if scratch is None:
            scratch = (torch.empty(T * H * n_splits * hd, dtype=torch.float32, device=q.device),
                       torch.empty(T * H * n_splits * 2, dtype=torch.float32, device=q.device))
        part_o, part_ml = scratch
        if part_o.numel() < T * H * n_splits * hd or part_ml.numel() < T * H * n_splits * 2:
            raise KernelError("attn_decode: scratch too small")
    counters = None
    if n_splits > 1:
        n_counters = T * Hkv * -(-(H // Hkv) // 16)
        counters = _attn_counters(q.device)
        if n_counters > counters.numel():
            if work is not None:
                raise KernelError("attn_decode: more (token, kv head) pairs than counters for a work list")
            counters = None          # more (token, kv head) pairs than counters: merge with the second kernel
    if work is not None and (work.dtype != torch.int32 or not work.is_contiguous() or teams < 1
                             or work.numel() < teams + 1 + 5 * T):
        raise KernelError("attn_decode: the work list must be int32 with teams + 1 offsets and at least a segment per token")
    fn = _fn("attn_decode", "lq_attn_decode_work", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                    c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int,
                                                    c_void_p, c_long, c_int, c_void_p])
    next_p, next_n = _next(next_w, PREFETCH_BYTES_ATTN)
    _check(fn(_p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(page_table), page_table.stride(0), _p(tok_pos),
              _p(tok_seq), _p(slots), _p(part_o), _p(part_ml), _p(counters), _p(out), T, H, Hkv, hd, page_size,
              float(scale), int(window or 0), n_splits, _p(work), int(teams), next_p, next_n, int(early_loads), _stream()),
           "attn_decode", 2 if n_splits > 1 and counters is None else 1,
           "attn_decode:teams" if work is not None else "attn_decode:one_slice" if n_splits == 1 else "attn_decode:slices")
    return out


_counters: dict = {}


def _attn_counters(device) -> torch.Tensor:
    """The counters by which the last block of a (token, kv head) finds out that it is the last:
    zero between calls (the kernel resets what it used), one buffer per device."""
    key = (device.type, device.index)
    if key not in _counters:
        _counters[key] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
    return _counters[key]

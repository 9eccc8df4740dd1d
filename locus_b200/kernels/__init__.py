"""Python entry points of the hand-written CUDA kernels.

Each function takes torch tensors that already live on the GPU, checks what the C entry
point cannot check (devices, contiguity, element types, shapes), and launches on torch's
current stream through ctypes.  Nothing here allocates device memory or falls back to
another implementation: a missing or failing kernel module raises.

The functions are the only way the parts reach the GPU, so a test may replace them by
plain torch functions of the same signature to exercise the engine's host logic.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from ..csrc import build as _build

ERR_UNSUPPORTED = 10001

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"element type {dt} is not supported by the kernels (float32, bfloat16)") from None


_LIBS = {}


def _lib(name: str) -> ctypes.CDLL:
    lib = _LIBS.get(name)
    if lib is None:
        lib = _LIBS[name] = _build.load(name)
    return lib


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_stream_override = None


def _stream():
    if _stream_override is not None:
        return _stream_override
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class pdl_scope:
    """Within the scope, kernels that support it are launched with programmatic dependent
    launch (see csrc/common.cuh): the next kernel's blocks are scheduled while the previous
    kernel still runs.  Used for the CUDA graphs of decode steps."""

    def __enter__(self):
        for lib in _LIBS.values():
            if hasattr(lib, "locus_set_pdl"):
                lib.locus_set_pdl(1)
        return self

    def __exit__(self, *exc):
        for lib in _LIBS.values():
            if hasattr(lib, "locus_set_pdl"):
                lib.locus_set_pdl(0)
        return False


class stream_scope:
    """Within the scope every launch goes to the stream that is torch's current stream when
    the scope is entered (looked up once instead of once per launch)."""

    def __enter__(self):
        global _stream_override
        self._saved = _stream_override
        _stream_override = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        global _stream_override
        _stream_override = self._saved
        return False


class kernel_times:
    """Opt-in table of where the time of eager steps goes, by entry point of this module (the reference has no
    profiler of its own: it prints counters at exit and is timed from outside).  Inside the scope an event is
    recorded behind every entry point's launch, on the stream it went to, and the launch is charged the time from
    the event before it on that stream (the scope's start, for the first launch on the stream that opened the
    scope) to its own: its run and whatever the stream waited for in front of it.  ``ModelRunner.step`` replays no
    graph meanwhile.  ``table()`` waits for the device and returns {entry point: (launches, milliseconds)}; the
    first launch on another stream is counted without a time."""

    def __enter__(self):
        global _TIMES
        _need(_TIMES is None, "kernel_times: scopes do not nest")
        self._spans = []   # (entry point, event before, event behind)
        self._counts = {}
        self._last = {}    # stream -> the event behind its latest launch
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        self._last[torch.cuda.current_stream().cuda_stream] = start
        _TIMES = self
        return self

    def __exit__(self, *exc):
        global _TIMES
        _TIMES = None
        return False

    def _mark(self, what: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        key = torch.cuda.current_stream().cuda_stream
        before = self._last.get(key)
        if before is not None:
            self._spans.append((what, before, ev))
        self._counts[what] = self._counts.get(what, 0) + 1
        self._last[key] = ev

    def restart(self) -> None:
        """The current stream starts a stretch of work of its own (a side stream that has just been told to wait
        for the main one): its next launch is charged from here, not from its last launch long ago."""
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._last[torch.cuda.current_stream().cuda_stream] = ev

    def table(self) -> dict:
        torch.cuda.synchronize()
        ms = {}
        for what, a, b in self._spans:
            ms[what] = ms.get(what, 0.0) + a.elapsed_time(b)
        return {what: (n, ms.get(what, 0.0)) for what, n in self._counts.items()}


_TIMES: Optional[kernel_times] = None


def timing_active() -> bool:
    """Whether a :class:`kernel_times` scope is open (steps then run eagerly)."""
    return _TIMES is not None


def timing_restart() -> None:
    """See :meth:`kernel_times.restart`; nothing without an open scope."""
    if _TIMES is not None:
        _TIMES.restart()


# kernels launched through this module since import (some entry points launch two and count the second themselves)
launches = 0
_LAUNCHES_OF = {}
MOE_SORT_ONE_LAUNCH_EXPERTS = 40 * 1024 // (9 * 4)   # up to this many experts moe_sort is one launch, else two


def _count_launches(n: int) -> None:
    global launches
    launches += n


def _check(code: int, what: str, detail: str = "") -> None:
    global launches
    if code == 0:
        launches += _LAUNCHES_OF.get(what, 1)
        if _TIMES is not None:
            _TIMES._mark(what)
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: sizes or element types outside what the kernel takes {detail}")
    raise KernelError(f"{what}: CUDA error {code} {detail}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda_c(t: torch.Tensor, name: str) -> None:
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.is_contiguous(), f"{name} must be contiguous")


def _i32(t: torch.Tensor, name: str) -> None:
    _cuda_c(t, name)
    _need(t.dtype == torch.int32, f"{name} must be int32")


LL = ctypes.c_longlong
I = ctypes.c_int
F = ctypes.c_float


# ---------------------------------------------------------------------------
def embed_rows(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = table[tokens[t], :] as float32."""
    _i32(tokens, "tokens")
    _cuda_c(table, "table")
    _cuda_c(out, "out")
    T, H = out.shape
    _need(out.dtype == torch.float32, "embed_rows: out must be float32")
    _need(tokens.numel() == T and table.shape[1] == H, "embed_rows: shape mismatch")
    code = _lib("elementwise").locus_embed_rows(
        _p(tokens), _p(table), I(dtype_code(table.dtype)), _p(out), I(T), I(H), _stream()
    )
    _check(code, "embed_rows")


def rmsnorm_adds(x: torch.Tensor) -> bool:
    """Whether :func:`rmsnorm` can fold a pending expert sum into rows like ``x``'s."""
    return x.dtype == torch.float32 and x.shape[-1] % 4 == 0


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, add=None) -> None:
    """out[i] = x[rows[i] if rows else i] * rsqrt(mean(x^2) + eps) * w  (statistics in float32).

    ``add`` = (pair_out, pair_pos, top_k): first x[i] += the sum that :func:`moe_combine` forms (same
    order), written back to ``x``; needs :func:`rmsnorm_adds`.  With ``rows`` the sum enters the norm
    of the gathered rows only and ``x`` stays as it was."""
    _cuda_c(x, "x")
    _cuda_c(w, "w")
    _cuda_c(out, "out")
    H = x.shape[-1]
    n = out.shape[0]
    _need(w.numel() == H and out.shape[-1] == H, "rmsnorm: width mismatch")
    if rows is not None:
        _i32(rows, "rows")
        _need(rows.numel() == n, "rmsnorm: rows/out mismatch")
    else:
        _need(x.shape[0] == n, "rmsnorm: x/out mismatch")
    add_src = add_pos = None
    add_k = 0
    if add is not None:
        add_src, add_pos, add_k = add
        _need(rmsnorm_adds(x), "rmsnorm: cannot fold the expert sum into these rows")
        _cuda_c(add_src, "pair_out")
        _i32(add_pos, "pair_pos")
        _need(add_src.dtype in (torch.float32, torch.bfloat16) and add_src.shape[-1] == H
              and add_pos.numel() >= (n if rows is None else x.shape[0]) * add_k,
              "rmsnorm: expert sum of another shape")
    code = _lib("elementwise").locus_rmsnorm(
        _p(x), I(dtype_code(x.dtype)), _p(w), I(dtype_code(w.dtype)), F(eps), _p(out),
        I(dtype_code(out.dtype)), _p(rows), I(n), I(H), _p(add_src),
        I(dtype_code(add_src.dtype) if add_src is not None else 0), _p(add_pos), I(add_k), _stream()
    )
    _check(code, "rmsnorm")


class ExpertLayout:
    """Device tensors that lay (token, slot) pairs out by expert (see :func:`moe_sort`)."""

    MIN_TILE = 8

    def __init__(self, n_pairs_max: int, n_experts: int, tile_m: int, device) -> None:
        """``tile_m``: rows of a tile; :func:`moe_sort` may be given another one per call
        (at least ``MIN_TILE``), the buffers are sized for the smallest."""
        self.tile_m = tile_m
        self.n_experts = n_experts
        self.max_tiles = (n_pairs_max + self.MIN_TILE - 1) // self.MIN_TILE + n_experts
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(n_experts, **i32)
        self.offsets = torch.zeros(n_experts + 1, **i32)
        self.sorted_pair = torch.zeros(n_pairs_max, **i32)
        self.pair_pos = torch.zeros(n_pairs_max, **i32)
        self.tile_expert = torch.zeros(self.max_tiles, **i32)
        self.tile_row0 = torch.zeros(self.max_tiles, **i32)
        self.tile_rows = torch.zeros(self.max_tiles, **i32)
        self.n_tiles = torch.zeros(1, **i32)
        # a second tile list over the same rows, with tiles of tile2_m rows (0: none; see moe_sort)
        self.tile2_m = 0
        self.tile2_expert = torch.zeros(self.max_tiles, **i32)
        self.tile2_row0 = torch.zeros(self.max_tiles, **i32)
        self.tile2_rows = torch.zeros(self.max_tiles, **i32)
        self.n_tiles2 = torch.zeros(1, **i32)

    def tiles_for(self, n_pairs: int, tile_m: Optional[int] = None) -> int:
        """Upper bound of the number of row tiles (of ``tile_m`` rows, default the layout's) when ``n_pairs``
        pairs are routed."""
        return min(self.max_tiles, n_pairs // (tile_m or self.tile_m) + min(n_pairs, self.n_experts) + 1)


# Tests switch this off to run the CUDA-core product on bfloat16 inputs.
USE_TENSOR_CORES = True


def tensor_cores_take(x: torch.Tensor, w: torch.Tensor, x_rows: Optional[torch.Tensor] = None) -> bool:
    """Whether :func:`linear` runs this product on the tensor cores: bfloat16 activations and
    weights, rows that TMA can address (width and row stride multiples of 8 elements,
    16-byte aligned base), and no row gather (gather into a buffer first)."""
    K = x.shape[-1]
    return (USE_TENSOR_CORES and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x_rows is None
            and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


FEW_ROWS = 8  # rows of x per tile of the row-streaming kernel


def few_rows_take(x: torch.Tensor, w: torch.Tensor, m: int, layout: Optional["ExpertLayout"] = None) -> bool:
    """Whether :func:`linear` runs this product with the row-streaming kernel: at most 8 rows
    (per expert tile when grouped), width a multiple of 8, 32-byte aligned rows."""
    K = x.shape[-1]
    rows_ok = layout.tile_m <= FEW_ROWS if layout is not None else m <= FEW_ROWS
    return (rows_ok and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 32 == 0 and w.data_ptr() % 32 == 0)


# Most rows of a plain product that go to the weight-streaming tensor-core kernel (it takes up to 32, and
# expert tiles of 8, 16 or 32 rows).  The four dense products of a layer at the A2.7B sizes take 46 us with
# either kernel at 16 rows; at 24 rows 59 us there and 47 us on the tcgen05 kernel (cut along K where it has
# few tiles), at 32 rows 61 and 47.
SKINNY_ROWS = 16
SKINNY_TILE_ROWS = 32  # largest expert tile of that kernel's grouped form
SKINNY_MIN_ROWS = 1


def skinny_takes(x: torch.Tensor, w: torch.Tensor, m: int, layout: Optional["ExpertLayout"] = None) -> bool:
    """Whether :func:`linear` runs this product with the weight-streaming tensor-core kernel:
    bfloat16 x bfloat16, at most ``SKINNY_ROWS`` rows (per expert tile of 8, 16 or 32 rows when grouped)."""
    K = x.shape[-1]
    if layout is not None:
        rows_ok = layout.tile_m in (8, 16, 32)
    else:
        rows_ok = SKINNY_MIN_ROWS <= m <= SKINNY_ROWS
    return (USE_TENSOR_CORES and rows_ok and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_N_SM = 0


def _sm_count() -> int:
    global _N_SM
    if _N_SM == 0:
        _N_SM = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _N_SM


SPLIT_SCRATCH_BYTES = 64 << 20   # float32 partial sums of a product split along K
_PLANS: dict = {}
_SPLIT_SCRATCH: dict = {}


def token_tile(m: int, dual: bool = False, n_weight_tiles: int = 0, k: int = 0) -> int:
    """Token tile of a plain product on the tensor cores (see :func:`tc_plan`)."""
    return tc_plan(m, n_weight_tiles * 128, k, dual)[0]


def tc_plan(m: int, n: int, k: int, dual: bool) -> Tuple[int, int]:
    """(token tile, splits along K) of a plain product of ``m`` rows with an [n, k] weight on the
    tcgen05 kernel.  While a tile waits for its weights its time hardly depends on its tokens (measured at
    k = 2048, one tile per SM: 12.7 us with 32 tokens, 13.5 with 64, 15 with 128, 18.3 with 256: 0.38 us
    + 0.75 ns per token for every 64 of k), so what counts is how many rounds the tiles make over the SMs,
    and a product with few tiles (a 2048-row weight has 16) leaves most SMs idle unless it is also cut
    along k; the partial sums then cost a second kernel.  The plan with the least estimated time wins."""
    key = (m, n, k, dual)
    plan = _PLANS.get(key)
    if plan is not None:
        return plan
    top = 128 if dual else 256
    cands = [t for t in (16, 32, 64, 128, 256) if t <= top]
    n_w = max(1, -(-n // 128))
    if k <= 0:  # sizes unknown: the smallest tile that holds the rows
        plan = (next((t for t in cands if m <= t), top), 1)
        _PLANS[key] = plan
        return plan
    n_sm = _sm_count()
    nkb = -(-k // 64)
    best, best_cost = (top, 1), None
    for t in cands:
        if t < 32 and m > t:
            continue
        tiles = -(-m // t) * n_w
        per_kb = (0.38 + 0.00075 * t) * (1.15 if dual else 1.0)
        options = [1]
        if not dual and n % 4 == 0 and tiles * 2 <= n_sm and nkb >= 8:
            s_max = min(n_sm // tiles, nkb // 2, 16, SPLIT_SCRATCH_BYTES // (4 * m * n))
            options += [s for s in range(2, s_max + 1)]
        for sp in options:
            kb = -(-nkb // sp)
            sp = -(-nkb // kb)
            rounds = -(-(tiles * sp) // n_sm)
            cost = rounds * (0.5 + kb * per_kb)
            if sp > 1:
                # the second kernel and its reading of the partial sums (fitted: 64 x 2048 x 2048 in 8 parts
                # takes 9.4 us, 256 x 6144 x 2048 in 3 parts 17.4 us)
                cost += 6.5 + sp * m * n * 4 / 3.5e6
            if best_cost is None or cost < best_cost - 1e-9 or (abs(cost - best_cost) <= 1e-9 and t > best[0]):
                best, best_cost = (t, sp), cost
        if m <= t:
            break
    _PLANS[key] = best
    return best


def _split_scratch(device) -> torch.Tensor:
    """The partial sums' buffer of the stream that launches: products on different streams (the shared expert
    beside the routed ones) must not share one.  Made at a stream's first split product, which is never inside
    a graph capture: a step is run once in the open before it is captured."""
    key = (device, _stream().value)
    t = _SPLIT_SCRATCH.get(key)
    if t is None:
        t = torch.empty(SPLIT_SCRATCH_BYTES // 4, dtype=torch.float32, device=device)
        _SPLIT_SCRATCH[key] = t
    return t


def expert_second_tile(n_pairs: int, n_experts: int) -> int:
    """Row tile of the experts' SECOND product (one accumulator per tile: 256 token rows fit the tensor memory)
    when it pays to walk the layout in larger tiles than the first product's 128, else 0.  With 137 rows per expert
    on average half of the experts need a second 128-row tile, which costs nearly what a full one costs (the tile
    waits for the same weights): measured at 60 x (2048 -> 2048), 4 picks, 2,048 tokens 122 us with 128-row tiles and
    110 us with 256-row tiles, at 64 x (3584 -> 2560), 8 picks 396 and 351 us; at 512 tokens (34 rows per expert)
    87 and 95 us."""
    return 256 if n_pairs >= 96 * n_experts else 0


def expert_tile(n_pairs: int, n_experts: int) -> int:
    """Row tile of a grouped product on the tensor cores.  Always the full 128 rows: a tile reads its
    tokens through a box that fits the rows it really has (16 to 256), so a tile with few rows costs little,
    and every expert's weights stream once.  Measured on the routed experts of 60 x (2048 -> 1408 -> 2048),
    4 picks: 75 us for 8 tokens, 148 us for 32, 173 us for 64, 181 us for 512, 238 us for 2,048 (the
    weight-streaming kernel with tiles of 8 to 32 rows: 79, 167, 219, 626 us)."""
    return 128


def tc_error() -> int:
    """Error word of the tensor-core module (0 = fine); reading it synchronises the device.
    Non-zero: a bounded wait inside a kernel ran out (1 producer, 2 MMA, 3 epilogue)."""
    return int(_lib("gemm_tc").locus_gemm_tc_error())


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, w2: Optional[torch.Tensor] = None,
           bias: Optional[torch.Tensor] = None, accumulate: bool = False,
           row_scale: Optional[torch.Tensor] = None, scale_rows: Optional[torch.Tensor] = None,
           x_rows: Optional[torch.Tensor] = None, x_row_div: int = 1, layout: Optional[ExpertLayout] = None,
           n_rows: Optional[int] = None, lists_ready: bool = False, second_tiles: bool = False) -> None:
    """out = x . w^T with float32 accumulation on CUDA cores (see csrc/gemm_simt.cu).

    ``w2``: out = silu(x . w^T) * (x . w2^T).  ``bias`` [N] is added, ``row_scale`` [M]
    multiplies the row (``scale_rows``: row m uses row_scale[scale_rows[m]]), ``accumulate`` adds the result into the float32 ``out``.
    ``x_rows``: logical row m reads x[x_rows[m] // x_row_div].  ``layout``: grouped product,
    ``w`` is [E, N, K] and logical rows are the expert-sorted pairs of the layout.
    ``n_rows``: number of logical rows (default: rows of ``out``).  ``lists_ready``: the layout was filled by a
    kernel that finished before the kernel in front of this one started (the experts' second product), so a
    kernel launched with programmatic dependent launch may read it before it waits for the one in front.
    ``second_tiles``: a grouped product on the tensor cores walks the layout's second tile list (``moe_sort`` with
    ``tile2_m``) instead of the first.
    """
    _cuda_c(x, "x")
    _cuda_c(w, "w")
    _cuda_c(out, "out")
    K = x.shape[-1]
    N = w.shape[-2]
    _need(w.shape[-1] == K, f"linear: x has width {K} but w has {w.shape[-1]}")
    _need(out.shape[-1] == N, f"linear: out has width {out.shape[-1]} but w has {N} rows")
    M = out.shape[0] if n_rows is None else n_rows
    _need(M <= out.shape[0], "linear: more rows than out holds")
    if x_rows is None and layout is None:
        _need(x.shape[0] >= M, "linear: x has fewer rows than out")
    if w2 is not None:
        _need(w2.shape == w.shape and w2.dtype == w.dtype and w2.is_contiguous(), "linear: w2 must match w")
    if accumulate:
        _need(out.dtype == torch.float32, "linear: accumulate needs a float32 out")
    if bias is not None:
        _need(bias.numel() == N and bias.is_contiguous(), "linear: bias size")
    if row_scale is not None:
        _need(row_scale.dtype == torch.float32 and row_scale.is_contiguous(), "linear: row_scale must be float32")
        if scale_rows is not None:
            _i32(scale_rows, "scale_rows")
        else:
            _need(row_scale.numel() >= M, "linear: row_scale must hold M rows")
    if x_rows is not None:
        _i32(x_rows, "x_rows")
    if layout is not None:
        _need(w.dim() == 3 and w.shape[0] == layout.n_experts, "linear: grouped product needs w [E, N, K]")
    if skinny_takes(x, w, M, layout):
        # bfloat16, up to 32 rows per tile: weight-streaming tensor-core kernel (csrc/gemm_skinny.cu)
        if layout is not None:
            tile = layout.tile_m
            te, t0, tr, nt = layout.tile_expert, layout.tile_row0, layout.tile_rows, layout.n_tiles
            max_tiles, stride = layout.tiles_for(M), N * K
        else:
            _need(w.dim() == 2, "linear: w must be [N, K]")
            tile = 8 if M <= 8 else (16 if M <= 16 else 32)
            te = t0 = tr = nt = None
            max_tiles = stride = 0
        code = _lib("gemm_skinny").locus_gemm_skinny(
            _p(x), _p(w), _p(w2), _p(bias), I(dtype_code(bias.dtype) if bias is not None else 0), _p(out),
            I(dtype_code(out.dtype)), I(1 if accumulate else 0), _p(row_scale), _p(scale_rows), _p(x_rows),
            I(x_row_div), I(M), I(N), I(K), LL(x.stride(0)), LL(out.stride(0)), I(tile), _p(te), _p(t0), _p(tr),
            _p(nt), I(max_tiles), LL(stride), I(1 if (lists_ready and layout is not None) else 0), _stream()
        )
        _check(code, "linear", f"(skinny; M={M}, N={N}, K={K}, tile {tile})")
        return
    if few_rows_take(x, w, M, layout):
        # a handful of rows: bandwidth-bound row-streaming kernel (csrc/gemv.cu)
        if layout is not None:
            te, t0, tr, nt = layout.tile_expert, layout.tile_row0, layout.tile_rows, layout.n_tiles
            max_tiles, stride = layout.tiles_for(M), N * K
        else:
            _need(w.dim() == 2, "linear: w must be [N, K]")
            te = t0 = tr = nt = None
            max_tiles = stride = 0
        code = _lib("gemv").locus_gemv(
            _p(x), I(dtype_code(x.dtype)), _p(w), _p(w2), I(dtype_code(w.dtype)), _p(bias),
            I(dtype_code(bias.dtype) if bias is not None else 0), _p(out), I(dtype_code(out.dtype)),
            I(1 if accumulate else 0), _p(row_scale), _p(scale_rows), _p(x_rows), I(x_row_div), I(M), I(N), I(K),
            LL(x.stride(0)), LL(out.stride(0)), _p(te), _p(t0), _p(tr), _p(nt), I(max_tiles), LL(stride), _stream()
        )
        _check(code, "linear", f"(few rows; M={M}, N={N}, K={K}, x {x.dtype}, w {w.dtype})")
        return
    if tensor_cores_take(x, w, x_rows):
        # bfloat16 x bfloat16: tcgen05 kernel (csrc/gemm_tc.cu)
        if layout is not None and second_tiles and layout.tile2_m > 0:
            TN, splits, scratch = layout.tile2_m, 1, None
            te, t0, tr, nt = layout.tile2_expert, layout.tile2_row0, layout.tile2_rows, layout.n_tiles2
            max_tiles = layout.tiles_for(M, layout.tile2_m)
        elif layout is not None:
            TN, splits, scratch = layout.tile_m, 1, None
            te, t0, tr, nt = layout.tile_expert, layout.tile_row0, layout.tile_rows, layout.n_tiles
            max_tiles = layout.tiles_for(M)
        else:
            _need(w.dim() == 2, "linear: w must be [N, K]")
            TN, splits = tc_plan(M, N, K, w2 is not None)
            if splits > 1:
                scratch = _split_scratch(x.device)
            te = t0 = tr = nt = None
            max_tiles = 0
        code = _lib("gemm_tc").locus_gemm_tc(
            _p(x), LL(M), LL(x.stride(0)), _p(w), _p(w2), LL(w.numel() // K), _p(bias),
            I(dtype_code(bias.dtype) if bias is not None else 0), _p(out), I(dtype_code(out.dtype)),
            I(1 if accumulate else 0), _p(row_scale), _p(scale_rows), I(M), I(N), I(K), LL(out.stride(0)), I(TN),
            _p(te), _p(t0), _p(tr), _p(nt), I(max_tiles), _p(scratch if splits > 1 else None), I(splits), _stream()
        )
        if splits > 1 and code == 0:
            _count_launches(1)   # the kernel that adds the splits up
        _check(code, "linear", f"(tensor cores; M={M}, N={N}, K={K}, token tile {TN}, {splits} splits)")
        return
    if layout is not None:
        _need(layout.tile_m == 64, "linear: the CUDA-core product uses 64-row tiles")
        te, t0, tr, nt = layout.tile_expert, layout.tile_row0, layout.tile_rows, layout.n_tiles
        max_tiles = layout.tiles_for(M)
        stride = N * K
    else:
        _need(w.dim() == 2, "linear: w must be [N, K]")
        te = t0 = tr = nt = None
        max_tiles = 0
        stride = 0
    code = _lib("gemm_simt").locus_gemm_simt(
        _p(x), I(dtype_code(x.dtype)), _p(w), _p(w2), I(dtype_code(w.dtype)), _p(bias),
        I(dtype_code(bias.dtype) if bias is not None else 0), _p(out), I(dtype_code(out.dtype)),
        I(1 if accumulate else 0), _p(row_scale), _p(scale_rows), _p(x_rows), I(x_row_div), I(M), I(N), I(K),
        LL(x.stride(0)), LL(out.stride(0)), _p(te), _p(t0), _p(tr), _p(nt), I(max_tiles), LL(stride),
        _stream()
    )
    _check(code, "linear", f"(M={M}, N={N}, K={K}, x {x.dtype}, w {w.dtype})")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                  q_out: torch.Tensor, pool: torch.Tensor, slots: torch.Tensor, *, n_heads: int,
                  n_kv_heads: int, head_dim: int, rot_dim: int, interleaved: bool,
                  page_tokens: int, write_kv: bool = True) -> None:
    """Rotate q and k by position, write q to ``q_out`` and k, v into the layer's pages.

    ``pool`` is one layer's pages [n_pages, 2, n_kv_heads, page_tokens, head_dim];
    ``slots[t] = page * page_tokens + offset``.  ``inv_freq`` None: no rotation.
    """
    _cuda_c(qkv, "qkv")
    _cuda_c(q_out, "q_out")
    _cuda_c(pool, "pool")
    _i32(positions, "positions")
    _i32(slots, "slots")
    T = qkv.shape[0]
    _need(qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "rope_kv_write: qkv width")
    _need(qkv.dtype == q_out.dtype == pool.dtype, "rope_kv_write: q, k, v and the cache share one element type")
    _need(tuple(pool.shape[1:]) == (2, n_kv_heads, page_tokens, head_dim), "rope_kv_write: pool layout")
    _need(positions.numel() >= T and slots.numel() >= T and q_out.shape[0] >= T, "rope_kv_write: T mismatch")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_cuda,
              "rope_kv_write: inv_freq must be float32 [rot_dim / 2]")
    code = _lib("elementwise").locus_rope_kv_write(
        _p(qkv), I(dtype_code(qkv.dtype)), _p(positions), _p(inv_freq), _p(q_out), _p(pool),
        _p(slots), I(T), I(n_heads), I(n_kv_heads), I(head_dim), I(rot_dim),
        I(1 if interleaved else 0), I(page_tokens), I(1 if write_kv else 0), _stream()
    )
    _check(code, "rope_kv_write")


def attn_chunk(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, *, seg_q0: torch.Tensor,
               seg_qn: torch.Tensor, seg_ctx: torch.Tensor, block_table: torch.Tensor,
               items: torch.Tensor, n_items: int, n_heads: int, n_kv_heads: int, head_dim: int,
               page_tokens: int, window: int, scale: float) -> None:
    """Attention of portions of prompts: ``items`` [n_items, 2] = (segment, first query of a
    16-query tile).  Keys come from the cache through ``block_table`` [n_seg, width]."""
    _cuda_c(q, "q")
    _cuda_c(out, "out")
    _cuda_c(pool, "pool")
    _i32(block_table, "block_table")
    _i32(items, "items")
    _need(q.dtype == pool.dtype == out.dtype, "attn_chunk: q, cache and out share one element type")
    code = _lib("attention").locus_attn_chunk(
        _p(q), I(dtype_code(q.dtype)), _p(pool), _p(out), _p(seg_q0), _p(seg_qn), _p(seg_ctx),
        _p(block_table), I(block_table.shape[1]), _p(items), I(n_items), I(n_heads), I(n_kv_heads),
        I(head_dim), I(page_tokens), I(window), F(scale), _stream()
    )
    _check(code, "attn_chunk", f"(heads {n_heads}/{n_kv_heads}, head_dim {head_dim})")


MMA_HEAD_DIMS = tuple(range(16, 257, 16))
MMA_QUERY_TILE = 64


def attn_chunk_mma_takes(q: torch.Tensor, head_dim: int) -> bool:
    """Whether the tensor-core kernel of prompt portions takes this case (bfloat16, head size
    in ``MMA_HEAD_DIMS``); otherwise :func:`attn_chunk` does it on the CUDA cores."""
    return USE_TENSOR_CORES and q.dtype == torch.bfloat16 and head_dim in MMA_HEAD_DIMS


MMA_ATTN_MAX_SPLITS = 16


def attn_chunk_mma_scratch(head_dim: int) -> Tuple[int, int]:
    """Floats of the two scratch buffers (sums; maxima and denominators) that :func:`attn_chunk_mma` needs
    to cut the keys of a step with few 64-query tiles into ranges (at most two blocks per SM are made)."""
    units = 2 * _sm_count() + MMA_ATTN_MAX_SPLITS
    return units * MMA_QUERY_TILE * head_dim, units * MMA_QUERY_TILE * 2


def attn_chunk_mma_splits(n_items: int, n_heads: int, max_ctx: int) -> int:
    """Ranges the keys of every item are cut into: enough for two blocks per SM when the step has fewer
    blocks than SMs (a short portion behind a long context), down to one tile of 64 keys per range.  A block
    takes about 1.9 us per key tile and the merge 2.5 us, so from four tiles on the cut pays: 64 tokens behind
    1,024 take 35 us in one range and 11 us in 16; 52 behind 30,000, 880 us and 91 us."""
    blocks = n_items * n_heads
    n_sm = _sm_count()
    tiles = -(-max_ctx // MMA_QUERY_TILE)
    if blocks >= n_sm or tiles < 4:
        return 1
    return max(1, min(MMA_ATTN_MAX_SPLITS, (2 * n_sm) // blocks, tiles))


def attn_chunk_mma(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, *, seg_q0: torch.Tensor,
                   seg_qn: torch.Tensor, seg_ctx: torch.Tensor, block_table: torch.Tensor,
                   items: torch.Tensor, n_items: int, n_heads: int, n_kv_heads: int, head_dim: int,
                   page_tokens: int, window: int, scale: float, n_splits: int = 1,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """Attention of portions of prompts on the tensor cores: ``items`` [n_items, 2] =
    (segment, first query of a 64-query tile); otherwise as :func:`attn_chunk`.  ``n_splits`` > 1
    (:func:`attn_chunk_mma_splits`) with scratch of :func:`attn_chunk_mma_scratch` floats: the keys of
    every item are cut into that many ranges, merged in ascending order by a second kernel."""
    _cuda_c(q, "q")
    _cuda_c(out, "out")
    _cuda_c(pool, "pool")
    _i32(block_table, "block_table")
    _i32(items, "items")
    _need(q.dtype == pool.dtype == out.dtype == torch.bfloat16, "attn_chunk_mma: bfloat16 only")
    if n_splits > 1:
        units = n_items * n_heads * n_splits
        _need(part_o is not None and part_ml is not None and part_o.dtype == part_ml.dtype == torch.float32
              and part_o.numel() >= units * MMA_QUERY_TILE * head_dim and part_ml.numel() >= units * MMA_QUERY_TILE * 2,
              "attn_chunk_mma: scratch too small for these ranges")
    code = _lib("attention_mma").locus_attn_chunk_mma(
        _p(q), _p(pool), _p(out), _p(seg_q0), _p(seg_qn), _p(seg_ctx), _p(block_table), I(block_table.shape[1]),
        _p(items), I(n_items), I(n_heads), I(n_kv_heads), I(head_dim), I(page_tokens), I(window), F(scale),
        I(n_splits), _p(part_o if n_splits > 1 else None), _p(part_ml if n_splits > 1 else None), _stream()
    )
    if n_splits > 1 and code == 0:
        _count_launches(1)
    _check(code, "attn_chunk_mma", f"(heads {n_heads}/{n_kv_heads}, head_dim {head_dim}, {n_splits} key ranges)")


TC_ATTN_HEAD_DIM = 128   # the tcgen05 attention kernel: this head size, pages of a multiple of 64 tokens
TC_ATTN_MIN_TOKENS = 256  # from this many new tokens in a step on, the tcgen05 kernel takes every portion


def attn_chunk_tc_takes(q: torch.Tensor, head_dim: int, page_tokens: int, n_tokens: int, max_ctx: int = 0) -> bool:
    """Whether the tcgen05 kernel of prompt portions takes this step: bfloat16, head size 128, pages of a
    multiple of 64 tokens, and either enough new tokens to fill blocks of 128 queries or a context long enough
    that the kernel's faster walk over the keys (cut into ranges, :func:`attn_chunk_tc_splits`) outweighs its
    start-up.  Measured at 16 heads against the mma.sync kernel, both with their key ranges: 128 new tokens
    behind 1,000 / 4,000 / 30,000 cached ones 18.6 / 20.4 / 59.6 us against 15.0 / 31.5 / 153.8 us; 16 new tokens
    14.2 / 16.4 / 53.9 us against 9.0 / 17.4 / 89.4 us."""
    if not (USE_TENSOR_CORES and q.dtype == torch.bfloat16 and head_dim == TC_ATTN_HEAD_DIM and page_tokens % 64 == 0):
        return False
    return n_tokens >= TC_ATTN_MIN_TOKENS or max_ctx >= (2048 if n_tokens >= 128 else 4096)


TC_ATTN_MAX_SPLITS = 16
TC_ATTN_QUERY_BLOCK = 128   # queries of a block of the tcgen05 kernel (two of the 64-query tiles of its item list)


def attn_chunk_tc_splits(n_items: int, n_heads: int, max_ctx: int) -> int:
    """Ranges the key tiles of every block of :func:`attn_chunk_tc` are cut into.  A block takes 128 queries of one
    head, a block per SM: a portion of a few hundred tokens behind a long context makes fewer blocks than the GPU
    has SMs, each walking thousands of keys alone.  Then the keys are cut so that about every SM has a block, down
    to four tiles of 128 keys per range (a block's start and end cost about four tiles' time)."""
    blocks = -(-n_items // 2) * n_heads
    n_sm = _sm_count()
    tiles = -(-max_ctx // TC_ATTN_QUERY_BLOCK)
    if 2 * blocks > n_sm or tiles < 8:
        return 1
    return max(1, min(TC_ATTN_MAX_SPLITS, n_sm // blocks, tiles // 4))


def attn_chunk_tc_scratch() -> Tuple[int, int]:
    """Floats of the two scratch buffers (sums; maxima and denominators) that :func:`attn_chunk_tc` needs for any
    cut that :func:`attn_chunk_tc_splits` chooses: one partial result per (token, head, range), and the ranges
    never outnumber SMs / blocks while a block holds at most 128 tokens of a head."""
    units = TC_ATTN_QUERY_BLOCK * _sm_count()
    return units * TC_ATTN_HEAD_DIM, units * 2


def attn_chunk_tc(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, *, seg_q0: torch.Tensor,
                  seg_qn: torch.Tensor, seg_ctx: torch.Tensor, block_table: torch.Tensor,
                  items: torch.Tensor, n_items: int, n_heads: int, n_kv_heads: int, head_dim: int,
                  page_tokens: int, window: int, scale: float, n_splits: int = 1,
                  part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """Attention of portions of prompts with tcgen05 tensor cores (scores and sums in tensor memory):
    ``items`` as for :func:`attn_chunk_mma` (tiles of 64 queries; a block takes an even one and the 64 queries
    behind it).  ``n_splits`` > 1 (:func:`attn_chunk_tc_splits`) with scratch of :func:`attn_chunk_tc_scratch`
    floats: the key tiles of every block are cut into that many ranges, merged in ascending order by a second
    kernel."""
    _cuda_c(q, "q")
    _cuda_c(out, "out")
    _cuda_c(pool, "pool")
    _i32(block_table, "block_table")
    _i32(items, "items")
    _need(q.dtype == pool.dtype == out.dtype == torch.bfloat16, "attn_chunk_tc: bfloat16 only")
    _need(1 <= n_splits <= TC_ATTN_MAX_SPLITS, f"attn_chunk_tc: 1 to {TC_ATTN_MAX_SPLITS} key ranges")
    if n_splits > 1:
        units = q.shape[0] * n_heads * n_splits
        n_o, n_ml = units * TC_ATTN_HEAD_DIM, units * 2
        _need(part_o is not None and part_ml is not None and part_o.dtype == part_ml.dtype == torch.float32
              and part_o.is_cuda and part_ml.is_cuda and part_o.numel() >= n_o and part_ml.numel() >= n_ml,
              "attn_chunk_tc: scratch too small for these ranges")
    code = _lib("attention_tc").locus_attn_chunk_tc(
        _p(q), LL(q.shape[0]), _p(pool), LL(pool.shape[0]), _p(out), _p(seg_q0), _p(seg_qn), _p(seg_ctx),
        _p(block_table), I(block_table.shape[1]), _p(items), I(n_items), I(n_heads), I(n_kv_heads), I(head_dim),
        I(page_tokens), I(window), F(scale), I(n_splits), _p(part_o if n_splits > 1 else None),
        _p(part_ml if n_splits > 1 else None), _stream()
    )
    if n_splits > 1 and code == 0:
        _count_launches(1)
    _check(code, "attn_chunk_tc", f"(heads {n_heads}/{n_kv_heads}, head_dim {head_dim}, pages of {page_tokens}, "
                                  f"{n_splits} key ranges)")


def attn_tc_error() -> int:
    """Error word of the tcgen05 attention module (0 = fine); reading it synchronises the device."""
    return int(_lib("attention_tc").locus_attn_tc_error())


def attn_error() -> int:
    """Error word of the attention module (0 = fine; 1 = a decode step's ``max_splits`` did not cover its
    longest context); reading it synchronises the device and clears it."""
    return int(_lib("attention").locus_attn_error())


def attn_gqa_error() -> int:
    """Error word of the grouped-query decode attention module (0 = fine; 1 = a wait for a bulk copy ran out);
    reading it synchronises the device and clears it."""
    return int(_lib("attention_gqa").locus_attn_gqa_error())


DECODE_SPLIT = 128


USE_GQA_DECODE = True   # tests switch it off to run grouped-query models on the per-head kernels
# The range cut's cost model of the grouped-query kernel, in keys (csrc/attn_ranges.cuh): the fixed cost of a range,
# and the cost of merging one more range per query head of the group (the merging warp takes the group's heads two
# at a time).  Measured at 28 heads on 4, 8,192 keys: with 2 x 7 = 14 keys per range a call takes 50 / 51 / 52 /
# 65 / 196 us at 1 / 4 / 8 / 16 / 64 requests (2: 51 / 52 / 51 / 66 / 202; 35: 75 / 76 / 74 / 75 / 196).
GQA_COST_RANGE, GQA_COST_MERGE_PER_HEAD = 64, 2
# Fewer (request, key/value head) pairs than this: the per-head kernels, which cut the work G times finer (at 28
# heads on 4 and 8,192 keys: 25 / 37 / 55 / 96 us at 1 / 2 / 4 / 8 requests against 50 / 50 / 51 / 52).
GQA_MIN_UNITS = 16


def attn_decode_gqa_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_tokens: int,
                          n_items: int) -> bool:
    """Whether :func:`attn_decode` runs the grouped-query kernel (csrc/attention_gqa.cu): bfloat16, 2 to 16
    query heads per key/value head, head size 64 or 128, pages of a multiple of 16 tokens, and enough
    (request, key/value head) pairs to fill the GPU with whole groups."""
    g = n_heads // max(1, n_kv_heads)
    return (USE_GQA_DECODE and USE_TENSOR_CORES and dtype == torch.bfloat16 and n_heads % max(1, n_kv_heads) == 0
            and 2 <= g <= 16 and head_dim in (64, 128) and page_tokens % 16 == 0 and n_items <= 1024
            and n_items * n_kv_heads >= GQA_MIN_UNITS)


def decode_streams(head_dim: int, dtype: torch.dtype, page_tokens: int, max_items: int) -> bool:
    """Whether :func:`attn_decode` runs the streaming kernel (the condition of csrc/attention.cu): rows of
    64 to 512 bytes (8, 16 or 32 lanes to a row: its 16-byte pieces rounded up to a power of two), pages that
    are a multiple of that lane count's chunk of 32, 16 or 8 keys, and at most 1024 requests."""
    pieces = head_dim * (4 if dtype == torch.float32 else 2) // 16
    lanes = 0 if pieces < 4 else 8 if pieces <= 8 else 16 if pieces <= 16 else 32 if pieces <= 32 else 0
    return lanes > 0 and page_tokens % (256 // lanes) == 0 and max_items <= 1024


def decode_units(max_items: int, n_heads: int, head_dim: int, dtype: torch.dtype, max_splits: int, device,
                 page_tokens: int = 64, n_kv_heads: int = 0) -> int:
    """How many partial results the scratch of :func:`attn_decode` should hold for batches of up to
    ``max_items`` requests.  The streaming kernels (:func:`decode_streams`, :func:`attn_decode_gqa_takes`) want
    one per (request, head) plus eight rounds of the grid's warps, so that short batches can be cut finely; the
    split kernel (other head and page sizes; and the small batches of a grouped-query model whose rows the
    per-head streaming kernel does not take) wants one per (request, head, split), ``max_splits`` being the
    splits of the longest context that the cache allows."""
    try:
        n_sm = torch.cuda.get_device_properties(device).multi_processor_count
    except Exception:  # no GPU (host tests with emulated kernels)
        n_sm = 148
    streaming = max_items * n_heads + 8 * 16 * n_sm
    if decode_streams(head_dim, dtype, page_tokens, max_items):
        return streaming
    if n_kv_heads > 0 and attn_decode_gqa_takes(dtype, n_heads, n_kv_heads, head_dim, page_tokens,
                                                max(max_items, GQA_MIN_UNITS)):
        # batches below GQA_MIN_UNITS pairs go to the split kernel
        small = min(max_items, max(0, -(-GQA_MIN_UNITS // n_kv_heads) - 1))
        return max(streaming, small * n_heads * max_splits)
    return max_items * n_heads * max_splits


def attn_decode_gqa_variant(few: Optional[bool]) -> None:
    """Force the grouped-query decode kernel's shape for few (request, key/value head) pairs (six warps a block,
    four chunks in flight per warp) on (True) or off (False: ten warps, two chunks), or leave the choice to the
    library (None).  For tests and measurements."""
    _lib("attention_gqa").locus_attn_decode_gqa_set_deep(I(-1 if few is None else 1 if few else 0))


def attn_decode_variant(deep: Optional[bool]) -> None:
    """Force the streaming decode kernel's variant with two chunks in flight per warp on (True) or off (False), or
    leave the choice to the library (None: by the number of (request, head) pairs and the longest context).  For
    tests and measurements."""
    _lib("attention").locus_attn_decode_set_deep(I(-1 if deep is None else 1 if deep else 0))


def attn_decode(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, *, seg_q0: torch.Tensor,
                seg_qn: torch.Tensor, seg_ctx: torch.Tensor, block_table: torch.Tensor,
                items: torch.Tensor, n_items: int, n_heads: int, n_kv_heads: int, head_dim: int,
                page_tokens: int, window: int, scale: float, part_o: torch.Tensor,
                part_ml: torch.Tensor, counters: torch.Tensor, max_splits: int) -> None:
    """Attention of single new tokens: ``items`` [n_items] = segments with one new token.

    ``part_o`` (float32, units * head_dim) and ``part_ml`` (float32, 2 * units) are scratch for
    partial results, ``units`` as :func:`decode_units` gives it (at least n_items * n_heads);
    ``counters`` (int32, n_items * n_heads) must be zero before the call and is zero after it;
    ``max_splits`` must be at least longest_position // DECODE_SPLIT + 1.
    """
    _cuda_c(q, "q")
    _cuda_c(out, "out")
    _cuda_c(pool, "pool")
    _i32(block_table, "block_table")
    _i32(items, "items")
    _need(q.dtype == pool.dtype == out.dtype, "attn_decode: q, cache and out share one element type")
    _need(part_o.dtype == torch.float32 and part_ml.dtype == torch.float32, "attn_decode: float32 scratch")
    max_units = min(part_o.numel() // head_dim, part_ml.numel() // 2)
    _need(max_units >= n_items * n_heads, "attn_decode: scratch too small")
    _need(pool.numel() * pool.element_size() < (64 << 30), "attn_decode: a layer's cache pool of 64 GiB or more")
    _i32(counters, "counters")
    _need(counters.numel() >= n_items * n_heads, "attn_decode: counters too small")
    if attn_decode_gqa_takes(q.dtype, n_heads, n_kv_heads, head_dim, page_tokens, n_items):
        # several query heads per key/value head: the kernel that reads every cache row once for its whole group
        code = _lib("attention_gqa").locus_attn_decode_gqa(
            _p(q), _p(pool), _p(out), _p(seg_q0), _p(seg_ctx), _p(block_table), I(block_table.shape[1]), _p(items),
            I(n_items), I(n_heads), I(n_kv_heads), I(head_dim), I(page_tokens), I(window), F(scale), _p(part_o),
            _p(part_ml), _p(counters), ctypes.c_longlong(max_units), I(GQA_COST_RANGE),
            I(GQA_COST_MERGE_PER_HEAD * (n_heads // n_kv_heads)), _stream()
        )
        _check(code, "attn_decode", f"(grouped queries; heads {n_heads}/{n_kv_heads}, head_dim {head_dim})")
        return
    code = _lib("attention").locus_attn_decode(
        _p(q), I(dtype_code(q.dtype)), _p(pool), _p(out), _p(seg_q0), _p(seg_qn), _p(seg_ctx),
        _p(block_table), I(block_table.shape[1]), _p(items), I(n_items), I(n_heads), I(n_kv_heads),
        I(head_dim), I(page_tokens), I(window), F(scale), _p(part_o), _p(part_ml), _p(counters), I(max_splits),
        ctypes.c_longlong(max_units), _stream()
    )
    _check(code, "attn_decode", f"(heads {n_heads}/{n_kv_heads}, head_dim {head_dim})")


SCORE_FUNCTIONS = {"softmax": 0, "sigmoid": 1}


def _route_rule(score_fn: str, sel_bias: Optional[torch.Tensor], n_group: int, n_group_used: int, n_experts: int,
                what: str):
    """The arguments that say how experts are chosen, checked: (score code, bias pointer, groups, groups used)."""
    _need(score_fn in SCORE_FUNCTIONS, f"{what}: score function {score_fn!r} (known: {', '.join(SCORE_FUNCTIONS)})")
    if sel_bias is not None:
        _need(sel_bias.is_cuda and sel_bias.dtype == torch.float32 and sel_bias.is_contiguous()
              and sel_bias.numel() == n_experts, f"{what}: the selection bias must be float32 [n_experts]")
    _need(1 <= n_group <= 32 and n_experts % n_group == 0,
          f"{what}: {n_group} groups must divide {n_experts} experts (at most 32 groups)")
    _need(n_group == 1 or 1 <= n_group_used <= n_group, f"{what}: groups used must be within 1..{n_group}")
    return I(SCORE_FUNCTIONS[score_fn]), _p(sel_bias), I(n_group), I(n_group_used)


class RouterScratch:
    """Scratch of :func:`router_topk`: the router logits of a step and one counter per tile of
    8 tokens (zero between launches); ``fused_counter``: the counter of :func:`route_fused_small`."""

    def __init__(self, max_tokens: int, n_logits: int, device) -> None:
        self.max_tokens, self.n_logits = max_tokens, n_logits
        self.logits = torch.empty(max_tokens * n_logits, dtype=torch.float32, device=device)
        self.counters = torch.zeros((max_tokens + 7) // 8, dtype=torch.int32, device=device)
        self.fused_counter = torch.zeros(1, dtype=torch.int32, device=device)


def router_topk(h: torch.Tensor, w_router: torch.Tensor, w_gate: Optional[torch.Tensor],
                ids: torch.Tensor, wts: torch.Tensor, gamma: Optional[torch.Tensor], *, top_k: int,
                renorm: bool, scale: float = 1.0, scratch: Optional[RouterScratch] = None, score_fn: str = "softmax",
                sel_bias: Optional[torch.Tensor] = None, n_group: int = 1, n_group_used: int = 1) -> None:
    """Router: scores of all experts (``score_fn``: softmax over them, or a sigmoid of each logit), top-k by
    repeated arg-max, weights; and gamma = sigmoid(w_gate . h) when the shared expert is gated.  All in float32.
    ``sel_bias`` [E] is added to the scores for the selection only; with ``n_group`` > 1 only the
    ``n_group_used`` groups of experts with the best two-score sums are eligible.
    ``scratch`` must hold T tokens of E (+1 with a gate) logits (made on the fly when None)."""
    _cuda_c(h, "h")
    _cuda_c(w_router, "w_router")
    _i32(ids, "ids")
    T, H = h.shape
    E = w_router.shape[0]
    _need(w_router.shape[1] == H, "router_topk: width mismatch")
    _need(wts.dtype == torch.float32 and wts.numel() >= T * top_k and ids.numel() >= T * top_k,
          "router_topk: ids / wts too small")
    if w_gate is not None:
        _need(w_gate.numel() == H and gamma is not None and gamma.dtype == torch.float32 and gamma.numel() >= T,
              "router_topk: gate needs w_gate [H] and gamma [T] float32")
    e1 = E + (1 if w_gate is not None else 0)
    if scratch is None:
        scratch = RouterScratch(T, e1, h.device)
    _need(scratch.n_logits >= e1 and scratch.max_tokens >= T, "router_topk: scratch too small")
    code = _lib("moe_route").locus_router_topk(
        _p(h), I(dtype_code(h.dtype)), _p(w_router), I(dtype_code(w_router.dtype)), _p(w_gate),
        I(dtype_code(w_gate.dtype) if w_gate is not None else 0), _p(scratch.logits), _p(scratch.counters),
        _p(ids), _p(wts), _p(gamma), I(T), I(H), I(E), I(top_k), I(1 if renorm else 0), F(scale),
        *_route_rule(score_fn, sel_bias, n_group, n_group_used, E, "router_topk"), _stream()
    )
    _check(code, "router_topk", f"(H={H}, E={E}, k={top_k})")


def router_logits(h: torch.Tensor, w_all: torch.Tensor, logits: torch.Tensor) -> None:
    """logits[t, e] = w_all[e] . h[t] in float32 with the weight-streaming tensor-core kernel,
    for ANY number of tokens (tiles of up to 16): one kernel, and one order of the sum, for
    every batch shape.  bfloat16 ``h`` [T, H] and ``w_all`` [E (+1), H]; ``logits`` [T, >= E (+1)]."""
    _cuda_c(h, "h")
    _cuda_c(w_all, "w_all")
    T, H = h.shape
    n = w_all.shape[0]
    _need(h.dtype == torch.bfloat16 and w_all.dtype == torch.bfloat16 and H % 8 == 0, "router_logits: bfloat16, H % 8 == 0")
    _need(logits.dtype == torch.float32 and logits.shape[0] >= T and logits.shape[1] >= n and logits.stride(1) == 1,
          "router_logits: logits must be float32 [T, >= rows of w_all]")
    # tiles of 16 tokens from 9 tokens on: with 32 a block's chain is twice as long (64 tokens: 9.1 us against 4.2,
    # 8,192 tokens: 60 against 34), and the order of a sum does not depend on the tile
    tile = 8 if T <= 8 else 16
    code = _lib("gemm_skinny").locus_gemm_skinny(
        _p(h), _p(w_all), None, None, I(0), _p(logits), I(0), I(0), None, None, None, I(1), I(T), I(n), I(H),
        LL(h.stride(0)), LL(logits.stride(0)), I(tile), None, None, None, None, I(0), LL(0), I(0), _stream()
    )
    _check(code, "router_logits", f"(T={T}, H={H}, rows {n})")


def router_select(logits: torch.Tensor, n_experts: int, has_gate: bool, ids: torch.Tensor, wts: torch.Tensor,
                  gamma: Optional[torch.Tensor], *, n_tokens: int, top_k: int, renorm: bool, scale: float = 1.0,
                  score_fn: str = "softmax", sel_bias: Optional[torch.Tensor] = None, n_group: int = 1,
                  n_group_used: int = 1) -> None:
    """Scores from the first ``n_experts`` columns of ``logits``, top-k by repeated arg-max,
    weights (the rule of :func:`router_topk`); gamma = sigmoid(column n_experts) when ``has_gate``."""
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1, "router_select: float32 logits")
    _i32(ids, "ids")
    _need(wts.dtype == torch.float32 and wts.numel() >= n_tokens * top_k and ids.numel() >= n_tokens * top_k,
          "router_select: ids / wts too small")
    if has_gate:
        _need(gamma is not None and gamma.dtype == torch.float32 and gamma.numel() >= n_tokens, "router_select: gamma")
    code = _lib("moe_route").locus_router_select(
        _p(logits), I(logits.stride(0)), _p(ids), _p(wts), _p(gamma), I(n_tokens), I(n_experts), I(top_k),
        I(1 if has_gate else 0), I(1 if renorm else 0), F(scale),
        *_route_rule(score_fn, sel_bias, n_group, n_group_used, n_experts, "router_select"), _stream()
    )
    _check(code, "router_select", f"(E={n_experts}, k={top_k})")


def moe_sort(ids: torch.Tensor, n_pairs: int, layout: ExpertLayout, tile_m: Optional[int] = None,
             tile2_m: int = 0) -> None:
    """Fill ``layout`` from the picked experts ``ids`` (first ``n_pairs`` entries), with row
    tiles of ``tile_m`` rows (default: the layout's).  ``tile2_m`` > 0: also a second tile list over the same
    rows with tiles of that size, for a product that runs with another token tile (``linear(..., second_tiles=True)``)."""
    _i32(ids, "ids")
    _need(n_pairs <= layout.sorted_pair.numel(), "moe_sort: layout too small")
    if tile_m is not None:
        _need(tile_m >= layout.MIN_TILE, f"moe_sort: tiles of at least {layout.MIN_TILE} rows")
        layout.tile_m = tile_m
    _need(tile2_m == 0 or tile2_m >= layout.MIN_TILE, f"moe_sort: tiles of at least {layout.MIN_TILE} rows")
    layout.tile2_m = tile2_m
    code = _lib("moe_route").locus_moe_sort(
        _p(ids), I(n_pairs), I(layout.n_experts), I(layout.tile_m), _p(layout.counts),
        _p(layout.offsets), _p(layout.sorted_pair), _p(layout.pair_pos), _p(layout.tile_expert),
        _p(layout.tile_row0), _p(layout.tile_rows), _p(layout.n_tiles), I(tile2_m), _p(layout.tile2_expert),
        _p(layout.tile2_row0), _p(layout.tile2_rows), _p(layout.n_tiles2), _stream()
    )
    if code == 0 and layout.n_experts > MOE_SORT_ONE_LAUNCH_EXPERTS:
        _count_launches(1)
    _check(code, "moe_sort")


ROUTE_SMALL_PAIRS = 1024  # limits of the one-launch selection + layout
ROUTE_SMALL_EXPERTS = 512


def route_small_takes(n_tokens: int, top_k: int, n_experts: int) -> bool:
    """Whether ``route_small`` handles this batch (a decode-sized batch: its single block would be
    slow for more tokens)."""
    return n_tokens <= 16 and n_tokens * top_k <= ROUTE_SMALL_PAIRS and n_experts <= ROUTE_SMALL_EXPERTS


def route_small(logits: torch.Tensor, n_experts: int, has_gate: bool, ids: torch.Tensor, wts: torch.Tensor,
                gamma: Optional[torch.Tensor], layout: ExpertLayout, *, n_tokens: int, top_k: int, renorm: bool,
                scale: float = 1.0, tile_m: Optional[int] = None, score_fn: str = "softmax",
                sel_bias: Optional[torch.Tensor] = None, n_group: int = 1, n_group_used: int = 1) -> None:
    """``router_select`` followed by ``moe_sort`` in one launch, for batches that
    ``route_small_takes``: same picks, weights and layout."""
    _need(route_small_takes(n_tokens, top_k, n_experts), "route_small: batch too large")
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1, "route_small: float32 logits")
    _i32(ids, "ids")
    _need(wts.dtype == torch.float32 and wts.numel() >= n_tokens * top_k and ids.numel() >= n_tokens * top_k,
          "route_small: ids / wts too small")
    _need(n_tokens * top_k <= layout.sorted_pair.numel() and layout.n_experts == n_experts,
          "route_small: layout does not fit")
    if has_gate:
        _need(gamma is not None and gamma.dtype == torch.float32 and gamma.numel() >= n_tokens, "route_small: gamma")
    if tile_m is not None:
        _need(tile_m >= layout.MIN_TILE, f"route_small: tiles of at least {layout.MIN_TILE} rows")
        layout.tile_m = tile_m
    layout.tile2_m = 0  # this call writes the first tile list only: a second list of an earlier call is stale now
    code = _lib("moe_route").locus_route_small(
        _p(logits), I(logits.stride(0)), _p(ids), _p(wts), _p(gamma), I(n_tokens), I(n_experts), I(top_k),
        I(1 if has_gate else 0), I(1 if renorm else 0), F(scale),
        *_route_rule(score_fn, sel_bias, n_group, n_group_used, n_experts, "route_small"), I(layout.tile_m), _p(layout.counts),
        _p(layout.offsets), _p(layout.sorted_pair), _p(layout.pair_pos), _p(layout.tile_expert),
        _p(layout.tile_row0), _p(layout.tile_rows), _p(layout.n_tiles), _stream()
    )
    _check(code, "route_small", f"(T={n_tokens}, E={n_experts}, k={top_k})")


def route_fused_small(h: torch.Tensor, w_all: torch.Tensor, logits: torch.Tensor, n_experts: int, has_gate: bool,
                      ids: torch.Tensor, wts: torch.Tensor, gamma: Optional[torch.Tensor], layout: ExpertLayout,
                      counter: torch.Tensor, *, n_tokens: int, top_k: int, renorm: bool, scale: float = 1.0,
                      tile_m: Optional[int] = None, score_fn: str = "softmax", sel_bias: Optional[torch.Tensor] = None,
                      n_group: int = 1, n_group_used: int = 1) -> None:
    """:func:`router_logits` followed by :func:`route_small` in ONE launch, for batches that ``route_small_takes``:
    the same logits (the same kernel computes them), picks, weights and layout.  ``counter``: one int32 that is
    zero before the call and zero after it."""
    _need(route_small_takes(n_tokens, top_k, n_experts), "route_fused_small: batch too large")
    _cuda_c(h, "h")
    _cuda_c(w_all, "w_all")
    T, H = n_tokens, h.shape[1]
    n = n_experts + (1 if has_gate else 0)
    _need(h.shape[0] >= T and w_all.shape[0] == n and w_all.shape[1] == H, "route_fused_small: shapes")
    _need(h.dtype == torch.bfloat16 and w_all.dtype == torch.bfloat16 and H % 8 == 0, "route_fused_small: bfloat16, H % 8 == 0")
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.shape[0] >= T and logits.shape[1] >= n
          and logits.stride(1) == 1, "route_fused_small: logits must be float32 [T, >= rows of w_all]")
    _i32(ids, "ids")
    _i32(counter, "counter")
    _need(wts.dtype == torch.float32 and wts.numel() >= T * top_k and ids.numel() >= T * top_k,
          "route_fused_small: ids / wts too small")
    _need(T * top_k <= layout.sorted_pair.numel() and layout.n_experts == n_experts, "route_fused_small: layout does not fit")
    if has_gate:
        _need(gamma is not None and gamma.dtype == torch.float32 and gamma.numel() >= T, "route_fused_small: gamma")
    if tile_m is not None:
        _need(tile_m >= layout.MIN_TILE, f"route_fused_small: tiles of at least {layout.MIN_TILE} rows")
        layout.tile_m = tile_m
    layout.tile2_m = 0  # as in route_small: no second tile list
    code = _lib("gemm_skinny").locus_router_fused_small(
        _p(h), _p(w_all), _p(logits), I(logits.stride(0)), _p(counter), _p(ids), _p(wts), _p(gamma), I(T), I(H),
        LL(h.stride(0)), I(n_experts), I(top_k), I(1 if has_gate else 0), I(1 if renorm else 0), F(scale),
        *_route_rule(score_fn, sel_bias, n_group, n_group_used, n_experts, "route_fused_small"), I(layout.tile_m),
        _p(layout.counts), _p(layout.offsets), _p(layout.sorted_pair), _p(layout.pair_pos), _p(layout.tile_expert),
        _p(layout.tile_row0), _p(layout.tile_rows), _p(layout.n_tiles), _stream()
    )
    _check(code, "route_fused_small", f"(T={T}, E={n_experts}, k={top_k})")


def moe_combine(x: torch.Tensor, pair_out: torch.Tensor, pair_pos: torch.Tensor, top_k: int) -> None:
    """x[t] += sum over slots (in slot order) of pair_out[pair_pos[t * k + slot]] (float32 or bfloat16 rows;
    the sum is float32)."""
    _cuda_c(x, "x")
    _cuda_c(pair_out, "pair_out")
    _i32(pair_pos, "pair_pos")
    T, H = x.shape
    _need(x.dtype == torch.float32 and pair_out.dtype in (torch.float32, torch.bfloat16),
          "moe_combine: float32 x, float32 or bfloat16 pair rows")
    _need(pair_out.shape[-1] == H, "moe_combine: width mismatch")
    code = _lib("elementwise").locus_moe_combine(_p(x), _p(pair_out), I(dtype_code(pair_out.dtype)), _p(pair_pos), I(T),
                                                 I(top_k), I(H), _stream())
    _check(code, "moe_combine")


def gather_rows(src: torch.Tensor, idx: torch.Tensor, div: int, out: torch.Tensor, n: int) -> None:
    """out[i] = src[idx[i] // div] for i < n."""
    _cuda_c(src, "src")
    _cuda_c(out, "out")
    _i32(idx, "idx")
    _need(src.dtype == out.dtype and src.shape[-1] == out.shape[-1], "gather_rows: mismatch")
    code = _lib("elementwise").locus_gather_rows(_p(src), I(dtype_code(src.dtype)), _p(idx), I(div), _p(out),
                                                 I(n), I(src.shape[-1]), _stream())
    _check(code, "gather_rows")


def apply_penalties(logits: torch.Tensor, history: torch.Tensor, repeat: torch.Tensor,
                    freq: torch.Tensor, presence: torch.Tensor) -> None:
    """In place: repetition / frequency / presence penalties over ``history`` [R, n] (-1 = none)."""
    _cuda_c(logits, "logits")
    _i32(history, "history")
    R, V = logits.shape
    _need(logits.dtype == torch.float32, "apply_penalties: float32 logits")
    _need(history.shape[0] == R, "apply_penalties: history rows")
    code = _lib("sampling").locus_apply_penalties(
        _p(logits), LL(logits.stride(0)), I(R), I(V), _p(history), I(history.shape[1]), _p(repeat),
        _p(freq), _p(presence), _stream()
    )
    _check(code, "apply_penalties")


def sample_use_cluster(on: bool) -> None:
    """Let rows of 8,192 to 163,840 tokens be sampled by a cluster of eight blocks per row (the default), or keep
    every row on the one-block kernel.  Both give the same tokens; for tests and measurements."""
    _lib("sampling").locus_sample_use_cluster(I(1 if on else 0))


def sample(logits: torch.Tensor, *, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: torch.Tensor, kept_count: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``logits`` [R, V] float32 (temperature <= 0: arg-max)."""
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1,
          "sample: logits must be float32 CUDA rows")
    R, V = logits.shape
    _i32(out, "out")
    _i32(top_k, "top_k")
    for t, n in ((temperature, "temperature"), (top_p, "top_p"), (min_p, "min_p")):
        _need(t.dtype == torch.float32 and t.numel() >= R and t.is_cuda, f"sample: {n} must be float32 [R]")
    for t, n in ((seeds, "seeds"), (counters, "counters")):
        _need(t.dtype == torch.int64 and t.numel() >= R and t.is_cuda, f"sample: {n} must be int64 [R]")
    code = _lib("sampling").locus_sample(
        _p(logits), LL(logits.stride(0)), I(R), I(V), _p(temperature), _p(top_k), _p(top_p), _p(min_p),
        _p(seeds), _p(counters), _p(out), _p(kept_count), _stream()
    )
    _check(code, "sample")


def modules_for(dtype: torch.dtype) -> list:
    """Kernel modules that a model of element type ``dtype`` needs."""
    return ["elementwise", "gemm_simt", "gemv", "gemm_skinny", "gemm_tc", "attention", "attention_mma", "moe_route", "sampling"]

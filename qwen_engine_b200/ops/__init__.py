"""The engine's operations: thin Python fronts of the hand-written CUDA kernels.

Every function works on CUDA tensors, writes into an output the caller
provides, and launches on torch's current stream.  There is no CPU path and no
library fallback: without the compiled extension, or with a tensor that is not
on a CUDA device, a call raises.  The plain PyTorch restatement of each
operation lives with the tests (tests/ref_ops.py).
"""
from __future__ import annotations

import ctypes
import os
import struct
from typing import Optional

import torch

from ..csrc import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_lib = None

ATTN_TILE_Q = 16        # queries per work item of the generic attention kernel
SMALL_M_MAX = 64        # rows up to which the weight-streaming product is used
SPLITK = True           # products of some tens of rows by clusters of CTAs that share K (gemm_tcgen05_splitk.cu)
SPLITK_MIN_M = 17       # rows from which, up to SPLITK_MAX_M, that kernel serves
SPLITK_MAX_M = 64
SPLITK_MAX_CTAS = 148   # clusters x CTAs at most: all on the GPU at once
SPLITK_LONG_K = 4096    # K from which that kernel serves from SPLITK_LONG_K_MIN_M rows on, where the weight rows / 16 exceed the SMs (0: never)
SPLITK_LONG_K_MIN_M = 9
SPLITK_VERY_LONG_K = 8192   # K from which, under the same conditions, every number of rows goes there (Qwen3-4B's down product)
SPLITK_VERY_LONG_K_MIN_M = 1
SPLITK_MAX_CLUSTERS_OF_8 = 8   # clusters of 8 CTAs at most (16 of them, 2 048 weight rows, took 8.9 us where 16 clusters of 4 take 5.5: a
                               # cluster needs its SMs in one part of the GPU)
SWAP_MIN_M = 17         # rows from which, up to SMALL_M_MAX, wide products go to the swapped tcgen05 kernel
SWAP_MIN_N = 3072       # weight rows from which it has enough CTAs (one per 128) to pull the weights fast enough
SWIGLU_FUSED = True     # SiLU-mul in the epilogue of the gate/up product where the CTA-pair kernel serves it
TCGEN05_PAIRS = True    # CTA pairs for large products
PAIR_MIN_TILES = 74     # 256 x 256 tiles from which they are used (one per pair of SMs)
TCGEN05_ENABLED = True  # the tcgen05 product for more rows (False: the generic kernel serves them)
FLASH_ROWS = 64         # rows (query token x query head of a group) per work item of the flash kernel
FLASH_BN = 64           # keys per tile of the flash kernel
FLASH_ITEM_INTS = 12    # int32 per work item of the flash kernel
FLASH_SPLIT = 256       # keys per part when a decoded token's context is split (reference attn.py:605)
FLASH_TARGET_CTAS = 296  # two CTAs per SM: long contexts are split into as many parts as fit in one wave
DECODE_ATTENTION_CLUSTERS = True    # parts of a request as a thread-block cluster that combines them through distributed shared memory
DECODE_ATTENTION_MMA = True         # decoded tokens (up to 16 rows per kv head, head size 128): warps with key groups and pipelines of their own, mma.sync arithmetic
DECODE_ATTENTION_MMA_MIN_CTAS = 0   # CTAs from which that kernel is used
DECODE_ATTENTION_MMA_STAGES = 3     # key groups a warp of that kernel keeps in flight (2 or 3; measured: 3 is 2.5 % ahead in the step)
DECODE_ATTENTION_MMA_EARLY = True   # that kernel requests earlier steps' keys before it waits for the kernel before it
DECODE_ATTENTION_MMA_BESIDE_TC = True   # also for the decoded tokens of a step whose prompt portions go to the tcgen05 kernel
SHIFTS_IN_ONE_LAUNCH = True          # a mixer that mixes its heads' weights: the shifts of the values' kv head as one launch where the step has no long portion
DECODE_ATTENTION_MMA_WIDE = True    # steps with at most as many attention CTAs as SMs: CTAs of 8 warps, one per SM (and contexts split for 148 CTAs, not 296)
DECODE_PREFETCH_KV_MB = 12          # that kernel asks L2 for the next layer's keys and values when a layer's are at most this many MB (0: never).  Measured (0.6B, context 1 024, asked for before the kernel's dependency wait): 4.4 MB (one request) 0.698 -> 0.690 ms a step, 8.8 MB 0.777 -> 0.765, 17.6 MB equal, 35 MB (eight) 0.915 -> 0.957
TC_ROWS = 256           # rows per work item of the tcgen05 attention kernel (two halves of 128)
TC_BN = 128             # keys per step of the tcgen05 attention kernel
TC_MIN_ROWS = 65        # rows of a request's portion from which the tcgen05 kernel serves it
TC_TARGET_CTAS = 148    # one CTA per SM
TC_MIN_PART_STEPS = 4   # key steps of a part at least, when tiles are cut to fill idle SMs
TC_MAX_PARTS = 8        # parts of one tile at most
TC_BALANCE_BELOW_CTAS = 592   # tiles x kv heads below which the tiles' schedule is laid out and long tiles are cut (4 per SM)
TC_ITEM_COST_STEPS = 2.0      # a work unit's first scores, masked step and output, in key steps
TC_PART_COST_STEPS = 5.0      # a part's scratch or merge on top, in key steps (the parts of a step move through L2 together)
TC_FORCE_CAP = -1       # the most key steps of a work item (0: cut nothing); below 0 the library works it out


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}     # the functions a gated feed-forward may put on its gate
LIMITED_GLU = "swish_limit"    # ("swish_limit", L): g' = min(g, L), u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1)


def gate_activation_known(activation) -> bool:
    if isinstance(activation, (tuple, list)):
        return len(activation) == 2 and activation[0] == LIMITED_GLU and float(activation[1]) > 0.0
    return activation in GATE_ACTIVATIONS


def gate_code(activation) -> int:
    """The number the kernels take for a gated feed-forward's form: 0 silu, 1 the tanh form of gelu, and for the
    limited form the bit pattern of its float32 limit (every positive float's pattern is an integer above 1)."""
    if not gate_activation_known(activation):
        raise KernelRefused(f"unknown activation {activation!r}; known: {sorted(GATE_ACTIVATIONS)} and ({LIMITED_GLU!r}, limit)")
    if isinstance(activation, (tuple, list)):
        import struct
        code = struct.unpack("<i", struct.pack("<f", float(activation[1])))[0]
        if code <= 1:
            raise KernelRefused(f"the limit {activation[1]!r} of a limited feed-forward is too small")
        return code
    return GATE_ACTIVATIONS[activation]


class ExtensionMissing(RuntimeError):
    """The CUDA extension could not be built or loaded."""


class KernelRefused(ValueError):
    """A kernel refused its arguments (a size it does not take, a wrong dtype)."""


def lib():
    """The loaded extension; builds it at the first call."""
    global _lib
    if _lib is None:
        try:
            path = _build.library_path()
            handle = ctypes.CDLL(path)
        except Exception as e:                       # noqa: BLE001 - re-raised with context
            raise ExtensionMissing(
                f"qwen_engine_b200 needs its CUDA extension and could not get it: {e}") from e
        handle.qe_last_error.restype = ctypes.c_char_p
        _lib = handle
    return _lib


def extension_path() -> str:
    return _build.library_path()


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise ExtensionMissing("qwen_engine_b200 ops run on CUDA tensors only (there is no CPU path); "
                               f"got a tensor on {t.device}")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    """The current stream, for a launch."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(_current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# torch's own fast paths to the current device and its current stream's handle (the public
# torch.cuda.current_stream() builds a Stream object per call, which costs more than a launch)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


launch_count = 0        # kernels launched through this module since import (read by the benchmark)
last_attention_kernel = ""   # which kernel the last ``paged_attention`` call went to (read by tests)


def _check(rc: int, name: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        msg = lib().qe_last_error().decode("utf-8", "replace")
        if rc == 1:
            raise KernelRefused(msg or f"{name} refused its arguments")
        raise RuntimeError(msg or f"{name} failed with code {rc}")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelRefused(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelRefused(msg)


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------------------

def prepare_matrix(w: torch.Tensor) -> torch.Tensor:
    """A [out, in] matrix as the product kernels want it (row-major, contiguous)."""
    return w.contiguous()


def embedding(token_ids: torch.Tensor, table: torch.Tensor, out,
              ssq: Optional[torch.Tensor] = None, scale: float = 1.0, accumulate: bool = False) -> None:
    """out[t] = float32(table[token_ids[t]]) * scale; out is the float32 residual stream [T, H].  With ``ssq``
    [T, P] float32, ssq[t, 0] gets the row's sum of squares (one partial sum per row).  ``out`` may be a
    ``ResidualStream``: its rows are written and, if it keeps sums of squares, those too.
    ``accumulate``: the scaled rows are added to what the stream holds (its pending branch output stays
    pending; sums of squares are no longer known)."""
    if isinstance(out, ResidualStream):
        stream = out
        if accumulate:
            embedding(token_ids, table, stream.resid, None, scale, True)
            stream.n_ssq = 0
            return
        embedding(token_ids, table, stream.resid, stream.ssq, scale)
        stream.has_delta, stream.n_ssq = False, (1 if stream.ssq is not None else 0)
        return
    _i32(token_ids, "token_ids")
    T, (V, H) = token_ids.numel(), table.shape
    _need(out.dtype == torch.float32 and out.shape == (T, H) and out.is_contiguous(), "embedding: out must be float32 [T, H]")
    _need(table.is_contiguous(), "embedding: table must be contiguous")
    if ssq is not None:
        _need(ssq.dtype == torch.float32 and ssq.dim() == 2 and ssq.shape[0] == T and ssq.is_contiguous(),
              "embedding: ssq must be float32 [T, P]")
    _check(lib().qe_embedding(_ptr(token_ids), _ptr(table), _ptr(out), T, H, V, _dt(table), _ptr(ssq),
                              int(ssq.shape[1]) if ssq is not None else 0, ctypes.c_float(scale), int(bool(accumulate)),
                              _stream()), "embedding")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """resid += delta (if given), in place in float32; out = rmsnorm(resid) * weight."""
    T, H = resid.shape
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "add_rmsnorm: resid must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (H,), "add_rmsnorm: weight must be float32 [H]")
    _need(out.shape == (T, H) and out.is_contiguous(), "add_rmsnorm: out must be contiguous [T, H]")
    if delta is not None:
        _need(delta.shape == (T, H) and delta.dtype == out.dtype and delta.is_contiguous(),
              "add_rmsnorm: delta must match out")
    _check(lib().qe_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(None), _ptr(weight), ctypes.c_float(eps),
                                _ptr(out), T, H, _dt(out), _stream()), "add_rmsnorm")


def add_rmsnorm_rows(resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                     weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[n] = rmsnorm(resid[rows[n]] + delta[rows[n]]) * weight; resid is not changed."""
    _i32(rows, "rows")
    N, H = out.shape
    _need(rows.numel() >= N, "add_rmsnorm_rows: fewer rows than outputs")
    _need(resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape[1] == H,
          "add_rmsnorm_rows: resid must be contiguous float32 [T, H]")
    _need(weight.dtype == torch.float32 and weight.shape == (H,), "add_rmsnorm_rows: weight must be float32 [H]")
    _need(out.is_contiguous(), "add_rmsnorm_rows: out must be contiguous")
    if delta is not None:
        _need(delta.shape == resid.shape and delta.dtype == out.dtype and delta.is_contiguous(),
              "add_rmsnorm_rows: delta must match")
    _check(lib().qe_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(rows), _ptr(weight), ctypes.c_float(eps),
                                _ptr(out), N, H, _dt(out), _stream()), "add_rmsnorm_rows")


class ResidualStream:
    """The float32 residual stream of a step, with the output of the last branch still to be added.

    ``resid`` [T, H] float32 is the stream.  A branch (mixer or feed-forward) either adds its output
    into it at once (``ResidualSink``), or leaves it in ``delta`` [T, H] (compute dtype) with
    ``has_delta`` set, to be added by the next norm.  ``ssq`` [T, P] float32 holds ``n_ssq`` partial
    sums of squares of every row of ``resid`` when the kernel that last wrote the stream left them
    (``n_ssq`` = 0: unknown); a norm fused into the next product starts from them."""

    def __init__(self, resid: torch.Tensor, delta: torch.Tensor, ssq: Optional[torch.Tensor] = None):
        self.resid, self.delta, self.ssq = resid, delta, ssq
        self.has_delta = False
        self.n_ssq = 0

    @classmethod
    def for_step(cls, alloc, num_tokens: int, width: int, dtype: torch.dtype) -> "ResidualStream":
        """The stream of a step of ``num_tokens`` rows of ``width``, from ``alloc(shape, dtype)``.  For a few rows
        in bfloat16 it also gets room for the partial sums of squares that the products which add into the
        stream leave behind (one per 16 or per 8 columns, padded to whole float4s): their layout is the kernels'
        business, so it is settled here, beside their fronts, and not by the model."""
        ssq = None
        if dtype == torch.bfloat16 and num_tokens <= SMALL_M_MAX:
            ssq = alloc((num_tokens, -(-(-(-width // 8)) // 4) * 4), torch.float32)
        return cls(alloc((num_tokens, width), torch.float32), alloc((num_tokens, width), dtype), ssq)


class ResidualSink:
    """Given to ``linear`` / ``linear_silu_mul`` as ``out``: the product is a branch's output and is to be
    added to the residual stream.  For a few rows in bfloat16 the add happens in the product's epilogue
    (which also leaves the rows' sums of squares for the next norm); otherwise the product goes to
    ``stream.delta`` and the next norm adds it."""

    def __init__(self, stream: ResidualStream):
        self.stream = stream

    def as_delta(self) -> torch.Tensor:
        st = self.stream
        st.has_delta, st.n_ssq = True, 0
        return st.delta


class NormedInput:
    """``rmsnorm(stream.resid + stream.delta) * weight`` that is not computed yet.

    ``linear`` takes it in the place of a tensor: for a few rows in bfloat16, when the stream is up to
    date and its sums of squares are known, the norm runs inside the product kernel (no kernel and no
    buffer between them); otherwise, and for any other consumer, ``materialize`` runs the add-and-norm
    kernel once and returns the tensor."""

    def __init__(self, stream: ResidualStream, weight: torch.Tensor, eps: float, alloc, dtype: torch.dtype):
        self.stream, self.weight, self.eps, self.alloc, self.dtype = stream, weight, float(eps), alloc, dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.stream.resid.shape

    def materialize(self) -> torch.Tensor:
        if self._tensor is None:
            st = self.stream
            out = self.alloc(tuple(st.resid.shape), self.dtype)
            add_rmsnorm(st.resid, st.delta if st.has_delta else None, self.weight, self.eps, out)
            if st.has_delta:
                st.has_delta, st.n_ssq = False, 0
            self._tensor = out
        return self._tensor


# What is fused into the products of a few rows was settled by measurement on a B200 (decode, batch 8,
# context 1024, tokens/s with / without):
#   the norm of the stream into the product that follows it   0.6B 6 480 / 6 920, 1.7B 4 340 / 4 580, 4B 1 570 / 1 970:
#       off.  Every CTA (16 weight rows) reads all of x; in float32 with the norm's arithmetic that costs
#       more than the norm kernel's launch.  Kept as a tested option.
#   SiLU-mul into the product that consumes it               0.6B equal, 4B 1 960 / 2 080: on up to 4 096 columns
#       of gate/up per half (every CTA reads both halves of gate_up).
#   the branch's add into the stream in the product's epilogue   0.6B 6 870 / 6 820, 4B 2 070 / 1 740: on.
SMALL_M_ROWS8 = False   # products of a few rows with so few weight rows that clusters of two share 16: 8 rows a CTA instead (a tested
                        # option that is off: no meeting, but every CTA reads all of x, and the batch-8 step went from 0.919 to 0.941 ms)
FUSED_NORM_MAX_M = 0    # rows up to which a norm is fused into the product that follows (0: never)
FUSED_SILU_MAX_M = 64   # rows up to which SiLU-mul is formed by the product that consumes it ...
FUSED_SILU_MAX_K = 4096  # ... when the activation has at most this many columns
RESID_SINK_MAX_M = 64   # rows up to which a branch's last product adds into the stream itself


def _linear_normed(x: NormedInput, w: torch.Tensor, out: torch.Tensor) -> bool:
    """The fused route of ``linear`` for a NormedInput; False if it does not apply."""
    st = x.stream
    M, K = st.resid.shape
    N = w.shape[0]
    if not (x._tensor is None and not st.has_delta and st.n_ssq > 0 and st.ssq is not None
            and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and M <= FUSED_NORM_MAX_M
            and K % 8 == 0 and st.resid.is_cuda and isinstance(out, torch.Tensor)):
        return False
    _need(w.shape == (N, K) and out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32)
          and w.is_contiguous() and out.is_contiguous(), "linear: operands do not fit the normed input")
    _check(lib().qe_linear_small_m_norm(_ptr(st.resid), _ptr(st.ssq), int(st.n_ssq), int(st.ssq.shape[1]),
                                        _ptr(x.weight), ctypes.c_float(x.eps), _ptr(w), _ptr(out), M, N, K,
                                        int(out.dtype == torch.float32), _stream()), "linear")
    return True


def splitk_splits(M: int, N: int, K: int, dtype: torch.dtype) -> int:
    """How many CTAs share a tile of 128 weight rows, each with a share of K, in the product of some tens
    of rows (``linear_splitk``): as many of 8, 4, 2 as keep all clusters on the GPU at once (8 only for few clusters); 0 where that
    kernel does not apply (few rows, enough weight rows for every SM, other types)."""
    if not (TCGEN05_ENABLED and SPLITK and dtype == torch.bfloat16 and M <= SPLITK_MAX_M and K % 8 == 0 and N % 4 == 0):
        return 0
    # From 9 rows on already (from the first, where K is very long) where the streaming kernel is at its worst: more CTAs of 16 weight rows than SMs (they do not
    # all start at once), a long K, and two tiles of tokens per instruction; then only with 4 or 8 CTAs per cluster.
    early = (SPLITK_LONG_K > 0 and K >= SPLITK_LONG_K and -(-N // 16) > SPLITK_MAX_CTAS
             and M >= (SPLITK_VERY_LONG_K_MIN_M if 0 < SPLITK_VERY_LONG_K <= K else SPLITK_LONG_K_MIN_M))
    if M < SPLITK_MIN_M and not early:
        return 0
    tiles = -(-N // 128)
    for s in (8, 4, 2):
        if s == 8 and tiles > SPLITK_MAX_CLUSTERS_OF_8:
            continue
        if tiles * s <= SPLITK_MAX_CTAS and -(-K // 64) >= 2 * s:
            return s if (M >= SPLITK_MIN_M or s >= 4) else 0
    return 0


def linear_splitk(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int, add: bool = False) -> None:
    """``linear`` in bfloat16 for up to 64 rows by clusters of ``splits`` CTAs that share 128 weight rows
    and meet through distributed shared memory; ``add``: out (float32) += the product."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape == (N, K), "linear_splitk: bfloat16 operands, w [N, K]")
    _need(out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32) and (not add or out.dtype == torch.float32),
          "linear_splitk: out must be [M, N], float32 to be added to")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_splitk: operands must be contiguous")
    mode = 2 if add else int(out.dtype == torch.float32)
    _check(lib().qe_linear_tcgen05_splitk(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(splits), mode, _stream()), "linear_splitk")


def _linear_into_stream(x: torch.Tensor, w: torch.Tensor, sink: ResidualSink, silu: bool) -> bool:
    """The fused route for a ResidualSink: resid += product, sums of squares left behind."""
    st = sink.stream
    M = x.shape[0]
    K = x.shape[1] // 2 if silu else x.shape[1]
    N = w.shape[0]
    if not silu and x.is_cuda and not st.has_delta and st.resid.shape == (M, N) and st.resid.is_contiguous():
        splits = splitk_splits(M, N, K, x.dtype)
        if splits:
            # some tens of rows: clusters that share K add their sum to the stream in their epilogue
            linear_splitk(x, w, st.resid, splits, add=True)
            st.n_ssq = 0
            return True
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= min(SMALL_M_MAX, RESID_SINK_MAX_M) and K % 8 == 0
            and not st.has_delta and st.ssq is not None and st.resid.shape == (M, N)):
        return False
    lib().qe_small_m_rows8(int(SMALL_M_ROWS8))
    cols = int(lib().qe_small_m_tile_cols(N, K))        # columns of a CTA: it leaves one partial sum of squares per row
    if st.ssq.shape[1] < -(-N // cols):
        return False
    _need(w.shape == (N, K) and x.is_contiguous() and w.is_contiguous(), "linear: operands do not fit")
    _hand_over_next_weights()
    _check(lib().qe_linear_small_m_resid(_ptr(x), _ptr(w), _ptr(st.resid), _ptr(st.ssq), int(st.ssq.shape[1]),
                                         M, N, K, int(silu), _stream()), "linear")
    st.n_ssq = -(-N // cols)
    return True


PREFETCH_NEXT_WEIGHTS = True   # products of a few rows ask L2 for the weights of the product that follows them
PREFETCH_NEXT_MAX_MB = 32      # ... when those are at most this many MB


def prefetch_next(w: Optional[torch.Tensor]) -> None:
    """Tell the next ``linear`` / ``linear_silu_mul`` call which weights the step reads after its own
    (None: none).  Where that call is served by the kernel for a few rows, its CTAs ask L2 for them once
    their own weights are on their way; every other kernel ignores the hint.  One call takes it."""
    global _next_w
    _next_w = None
    if (w is not None and PREFETCH_NEXT_WEIGHTS and w.is_cuda and w.is_contiguous()
            and w.numel() * w.element_size() <= PREFETCH_NEXT_MAX_MB << 20):
        _next_w = w


_next_w: Optional[torch.Tensor] = None


def _hand_over_next_weights() -> None:
    """Before a launch of the kernel for a few rows: the pending hint goes to the library (and is cleared)."""
    global _next_w
    if _next_w is not None:
        w, _next_w = _next_w, None
        lib().qe_small_m_prefetch_next(_ptr(w), ctypes.c_ulonglong(w.numel() * w.element_size()))


def linear(x, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] · w[N, K]^T, float32 accumulation; out in x's dtype or float32.
    ``x`` may be a NormedInput (see there)."""
    if isinstance(x, NormedInput):
        if _linear_normed(x, w, out):
            return
        x = x.materialize()
    if isinstance(out, ResidualSink):
        if _linear_into_stream(x, w, out, silu=False):
            return
        out = out.as_delta()
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape == (N, K) and w.dtype == x.dtype, f"linear: w {tuple(w.shape)} {w.dtype} does not fit x {tuple(x.shape)} {x.dtype}")
    _need(out.shape == (M, N) and out.dtype in (x.dtype, torch.float32), "linear: out must be [M, N] in x's dtype or float32")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear: operands must be contiguous")
    out_f32 = int(out.dtype == torch.float32)
    splits = splitk_splits(M, N, K, x.dtype)
    if splits:
        linear_splitk(x, w, out, splits)
        return
    if (x.dtype == torch.bfloat16 and SWAP_MIN_M <= M <= SMALL_M_MAX and N >= SWAP_MIN_N and K % 8 == 0
            and TCGEN05_ENABLED):
        # some tens of rows and many weight rows: the weights on the 128-row side of tcgen05.mma
        _check(lib().qe_linear_tcgen05_swap(_ptr(x), _ptr(w), _ptr(out), M, N, K, out_f32, _stream()), "linear")
        return
    if x.dtype == torch.bfloat16 and M <= SMALL_M_MAX and K % 8 == 0:
        # a few rows: stream every weight once through the tensor cores
        _hand_over_next_weights()
        lib().qe_small_m_rows8(int(SMALL_M_ROWS8))
        _check(lib().qe_linear_small_m(_ptr(x), _ptr(w), _ptr(out), M, N, K, out_f32, _stream()), "linear")
        return
    if (x.dtype == torch.bfloat16 and TCGEN05_PAIRS and TCGEN05_ENABLED and K % 8 == 0
            and (-(-M // 256) * -(-N // 256) >= PAIR_MIN_TILES
                 or (PAIR_PLAN and M > SMALL_M_MAX and tc_product_plan(M, N, K) != 0))):
        # pairs of CTAs share a 256-row tile (tcgen05 cta_group::2): enough 256 x 256 tiles for every pair of SMs,
        # or the library's model of the kernels' times says so (fewer tiles: wide tiles all the same, or 2 or 4 pairs
        # per tile with a share of a long K each, meeting on chip)
        linear_pairs(x, w, out)
        return
    if x.dtype == torch.bfloat16 and M > SMALL_M_MAX and K % 8 == 0 and TCGEN05_ENABLED:
        # many rows: TMA-fed tcgen05 tensor cores with the accumulator in tensor memory
        _check(lib().qe_linear_tcgen05(_ptr(x), _ptr(w), _ptr(out), M, N, K, out_f32, _stream()), "linear")
        return
    _check(lib().qe_linear_generic(_ptr(x), _ptr(w), _ptr(out), M, N, K, _dt(x), out_f32, _stream()), "linear")


PAIR_PLAN = True        # products of many rows with fewer than PAIR_MIN_TILES tiles go where the library's model of the kernels' times sends them


def tc_product_plan(M: int, N: int, K: int) -> int:
    """Which tcgen05 kernel serves a plain bfloat16 product of more than 64 rows: 0 the single-CTA kernel, 1 CTA
    pairs with 256 x 128 tiles, 2 with 256 x 256 tiles, 3 / 4 with K split over 2 / 4 pairs per tile."""
    return int(lib().qe_tc_product_plan(int(M), int(N), int(K), 0))


def pair_k_splits(M: int, N: int, K: int) -> int:
    """Into how many CTA pairs per 256 x 256 tile ``linear_pairs`` splits K for this shape (1: it does not)."""
    return int(lib().qe_pair_k_splits(int(M), int(N), int(K), 0))


def linear_pairs(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``linear`` in bfloat16 by the kernel in which two CTAs share a 256-row tile; any number of rows
    (few tiles: 256 x 128 tiles; ``linear`` itself comes here only for large products)."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape == (N, K) and K % 8 == 0,
          "linear_pairs: bfloat16 operands with K a multiple of 8")
    _need(out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32), "linear_pairs: out must be [M, N]")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_pairs: operands must be contiguous")
    _check(lib().qe_linear_tcgen05_pair(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(out.dtype == torch.float32), _stream()),
           "linear_pairs")


def swiglu_fused_applies(M: int, I: int, K: int, dtype: torch.dtype) -> bool:
    """Whether ``linear_swiglu`` serves this shape: bfloat16, more rows than the weight-streaming products
    take, and enough 256-row x 128-column tiles of the activation for every pair of SMs (the kernel is the
    CTA-pair product)."""
    return (TCGEN05_PAIRS and TCGEN05_ENABLED and SWIGLU_FUSED and dtype == torch.bfloat16 and K % 8 == 0
            and M > SMALL_M_MAX and -(-M // 256) * -(-I // 128) >= PAIR_MIN_TILES)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[M, I] = act(x · w[:I]^T) * (x · w[I:]^T) for the stacked weights w [2 I, K]: the feed-forward's
    activation (``GATE_ACTIVATIONS``) formed in the product's epilogue on its float32 sums (bfloat16, many rows)."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.shape == (2 * I, K) and K % 8 == 0,
          "linear_swiglu: bfloat16 operands, w [2 I, K] with K a multiple of 8")
    _need(out.shape == (M, I) and out.dtype in (torch.bfloat16, torch.float32), "linear_swiglu: out must be [M, I]")
    _need(x.is_contiguous() and w_gate_up.is_contiguous() and out.is_contiguous(), "linear_swiglu: operands must be contiguous")
    _check(lib().qe_linear_swiglu_tcgen05_pair(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K,
                                               int(out.dtype == torch.float32), gate_code(activation), _stream()), "linear_swiglu")


SWIGLU_SMALL_MAX_M = 16     # rows up to which the weight-streaming product forms the activation in its epilogue


def swiglu_small_applies(M: int, I: int, K: int, dtype: torch.dtype) -> bool:
    """Whether ``linear_swiglu_small`` serves this shape: a few rows in bfloat16."""
    return dtype == torch.bfloat16 and 1 <= M <= SWIGLU_SMALL_MAX_M and K % 8 == 0


def linear_swiglu_small(x, w_gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[M, I] = act(x · w[:I]^T) * (x · w[I:]^T) for the stacked weights w [2 I, K] and a few rows (decode steps):
    a CTA streams the gate rows and the up rows of the same 16 columns and forms the activation in its epilogue, so
    that gate and up never exist in memory and the product that follows reads half the bytes, already activated."""
    if isinstance(x, NormedInput):
        x = x.materialize()
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.shape == (2 * I, K) and K % 8 == 0,
          "linear_swiglu_small: bfloat16 operands, w [2 I, K] with K a multiple of 8")
    _need(out.shape == (M, I) and out.dtype == torch.bfloat16 and M <= SWIGLU_SMALL_MAX_M,
          f"linear_swiglu_small: out must be bfloat16 [M, I] with M <= {SWIGLU_SMALL_MAX_M}")
    _need(x.is_contiguous() and w_gate_up.is_contiguous() and out.is_contiguous(), "linear_swiglu_small: operands must be contiguous")
    _hand_over_next_weights()
    _check(lib().qe_linear_small_m_swiglu(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K, gate_code(activation), _stream()),
           "linear_swiglu_small")


QKV_ROPE_FUSED = True       # many rows: per-head norm, rotation and cache write in the epilogue of the QKV product
QKV_ROPE_MIN_TILES = 74     # 256 x 256 tiles of the product from which it is used (one per pair of SMs)


def qkv_rope_fused_applies(M: int, N: int, K: int, dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``linear_qkv_rope`` serves this shape: bfloat16, head size 128 rotated as a whole, and
    enough 256 x 256 tiles for every pair of SMs (the kernel is the CTA-pair product)."""
    return (QKV_ROPE_FUSED and TCGEN05_PAIRS and TCGEN05_ENABLED and dtype == torch.bfloat16
            and head_dim == 128 and rotary_dim == 128 and K % 8 == 0 and N % 128 == 0
            and M > SMALL_M_MAX and -(-M // 256) * -(-N // 256) >= QKV_ROPE_MIN_TILES)


def linear_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                    k_norm_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                    kv_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                    num_heads: int, num_kv_heads: int, write_kv: bool = True) -> None:
    """The QKV product with what ``qk_norm_rope_kv_write`` would do to it afterwards done in its epilogue
    (head size 128, bfloat16): qkv[:, :Hq 128] = rotated, normed q; the rotated, normed k and v go to their
    slots in ``kv_pages`` [pages, 2, Hkv, page, 128] only (the k and v columns of ``qkv`` are not written).
    ``cos_sin``: float32 [T, 64, 2], the step's table of angles (None: no rotation)."""
    M, K = x.shape
    Hq, Hkv = num_heads, num_kv_heads
    N = (Hq + 2 * Hkv) * 128
    _need(x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and w_qkv.shape == (N, K) and K % 8 == 0,
          "linear_qkv_rope: bfloat16 operands, w [(Hq + 2 Hkv) 128, K] with K a multiple of 8")
    _need(qkv.shape == (M, N) and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and x.is_contiguous() and w_qkv.is_contiguous(),
          "linear_qkv_rope: qkv must be contiguous bfloat16 [M, (Hq + 2 Hkv) 128]")
    for wt in (q_norm_w, k_norm_w):
        _need(wt is None or (wt.dtype == torch.float32 and wt.shape == (128,)), "linear_qkv_rope: norm weights must be float32 [128]")
    _need(cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (M, 64, 2) and cos_sin.is_contiguous()),
          "linear_qkv_rope: cos_sin must be float32 [M, 64, 2]")
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None and kv_pages.dtype == torch.bfloat16 and kv_pages.is_contiguous()
              and kv_pages.dim() == 5 and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == 128,
              "linear_qkv_rope: kv_pages must be bfloat16 [pages, 2, Hkv, page, 128]")
        _i32(slot_mapping, "slot_mapping")
        _need(slot_mapping.numel() >= M, "linear_qkv_rope: a slot for every row")
        page_size = int(kv_pages.shape[3])
    _check(lib().qe_linear_qkv_rope_tcgen05_pair(
        _ptr(x), _ptr(w_qkv), _ptr(qkv), M, N, K, _ptr(q_norm_w), _ptr(k_norm_w), ctypes.c_float(eps), _ptr(cos_sin),
        _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None), Hq, Hkv, page_size,
        int(bool(write_kv)), _stream()), "linear_qkv_rope")


QKV_ROPE_SMALL = False       # a few rows: per-head norm, rotation and cache write in the epilogue of the QKV product (clusters of 8 CTAs per head).  Off: measured on a B200 (0.6B sizes, 8 rows, chains of 28): product + rotary kernel 3.83 us, fused 4.54 us (cluster launch + two cluster barriers cost more than the launch they save); the decode step 0.955 -> 0.978 ms.  Kept as a tested option.
QKV_ROPE_SMALL_MAX_M = 16


def qkv_rope_small_applies(M: int, N: int, K: int, dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``linear_qkv_rope_small`` serves this shape: a few rows in bfloat16, head size 128 rotated as a whole."""
    return (QKV_ROPE_SMALL and dtype == torch.bfloat16 and head_dim == 128 and rotary_dim == 128 and K % 8 == 0
            and N % 128 == 0 and 1 <= M <= QKV_ROPE_SMALL_MAX_M)


def linear_qkv_rope_small(x, w_qkv: torch.Tensor, qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                          k_norm_w: Optional[torch.Tensor], eps: float, positions: Optional[torch.Tensor],
                          inv_freq: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                          kv_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                          num_heads: int, num_kv_heads: int, write_kv: bool = True) -> None:
    """The QKV product of a few rows (decode steps) with what ``qk_norm_rope_kv_write`` would do to it afterwards in
    its epilogue (head size 128, bfloat16): a head's 128 columns are the work of a cluster of 8 CTAs, which exchange
    the sums of squares and the rotation's partners through distributed shared memory.  qkv[:, :Hq 128] = rotated,
    normed q; the rotated, normed k and v go to their slots in ``kv_pages`` [pages, 2, Hkv, page, 128] only.  Angles:
    ``cos_sin`` float32 [M, 64, 2] if given, else ``positions`` x ``inv_freq`` [64] (both None: no rotation)."""
    if isinstance(x, NormedInput):
        x = x.materialize()
    M, K = x.shape
    Hq, Hkv = num_heads, num_kv_heads
    N = (Hq + 2 * Hkv) * 128
    _need(x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and w_qkv.shape == (N, K) and K % 8 == 0,
          "linear_qkv_rope_small: bfloat16 operands, w [(Hq + 2 Hkv) 128, K] with K a multiple of 8")
    _need(qkv.shape == (M, N) and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and x.is_contiguous() and w_qkv.is_contiguous()
          and M <= QKV_ROPE_SMALL_MAX_M, f"linear_qkv_rope_small: qkv must be contiguous bfloat16 [M <= {QKV_ROPE_SMALL_MAX_M}, (Hq + 2 Hkv) 128]")
    for wt in (q_norm_w, k_norm_w):
        _need(wt is None or (wt.dtype == torch.float32 and wt.shape == (128,)), "linear_qkv_rope_small: norm weights must be float32 [128]")
    _need(cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (M, 64, 2) and cos_sin.is_contiguous()),
          "linear_qkv_rope_small: cos_sin must be float32 [M, 64, 2]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == 64, "linear_qkv_rope_small: inv_freq must be float32 [64]")
        if cos_sin is None:
            _need(positions is not None and positions.numel() >= M, "linear_qkv_rope_small: a position for every row")
            _i32(positions, "positions")
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None and kv_pages.dtype == torch.bfloat16 and kv_pages.is_contiguous()
              and kv_pages.dim() == 5 and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == 128,
              "linear_qkv_rope_small: kv_pages must be bfloat16 [pages, 2, Hkv, page, 128]")
        _i32(slot_mapping, "slot_mapping")
        _need(slot_mapping.numel() >= M, "linear_qkv_rope_small: a slot for every row")
        page_size = int(kv_pages.shape[3])
    _hand_over_next_weights()
    _check(lib().qe_linear_small_m_qkv_rope(
        _ptr(x), _ptr(w_qkv), _ptr(qkv), M, N, K, _ptr(q_norm_w), _ptr(k_norm_w), ctypes.c_float(eps), _ptr(positions),
        _ptr(inv_freq), _ptr(cos_sin), _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None),
        Hq, Hkv, page_size, int(bool(write_kv)), _stream()), "linear_qkv_rope_small")


def linear_silu_mul(gate_up: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch) -> None:
    """out[M, N] = (silu(gate_up[:, :I]) * gate_up[:, I:]) · w[N, I]^T.  For a few rows in bfloat16 the
    activation is formed while the product loads it; otherwise ``silu_mul`` runs first into a buffer
    that ``scratch(shape, dtype)`` provides."""
    M, I2 = gate_up.shape
    I = I2 // 2
    N = w.shape[0]
    if M > FUSED_SILU_MAX_M or I > FUSED_SILU_MAX_K or splitk_splits(M, N, I, gate_up.dtype):
        act = scratch((M, I), gate_up.dtype)
        silu_mul(gate_up, act)
        linear(act, w, out)
        return
    if isinstance(out, ResidualSink):
        if _linear_into_stream(gate_up, w, out, silu=True):
            return
        out = out.as_delta()
    _need(I2 % 2 == 0 and w.shape == (N, I) and w.dtype == gate_up.dtype, "linear_silu_mul: w must be [N, I] for gate_up [M, 2I]")
    _need(out.shape == (M, N) and out.dtype in (gate_up.dtype, torch.float32), "linear_silu_mul: out must be [M, N]")
    _need(gate_up.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_silu_mul: operands must be contiguous")
    if gate_up.dtype == torch.bfloat16 and M <= SMALL_M_MAX and I % 8 == 0:
        _hand_over_next_weights()
        lib().qe_small_m_rows8(int(SMALL_M_ROWS8))
        _check(lib().qe_linear_small_m_silu(_ptr(gate_up), _ptr(w), _ptr(out), M, N, I,
                                            int(out.dtype == torch.float32), _stream()), "linear_silu_mul")
        return
    act = scratch((M, I), gate_up.dtype)
    silu_mul(gate_up, act)
    linear(act, w, out)


def timeline_begin(capacity: int = 1 << 20) -> None:
    """Start recording in the timeline build of the library (QE_TIMELINE=1 in the environment when it is
    built and loaded): from now on thread 0 of every CTA notes the GPU's clock when it lets its dependents
    start and when its wait for the kernel before it returns.  Raises in the plain build."""
    lib().qe_timeline_begin.restype = ctypes.c_long
    got = int(lib().qe_timeline_begin(ctypes.c_long(int(capacity))))
    if got < 0:
        raise ExtensionMissing("this build of the library records no timeline (build and run with QE_TIMELINE=1)"
                               if got == -1 else "no memory for the timeline")


def timeline_events() -> list[tuple[str, int, int, int, int, int, int]]:
    """The events since ``timeline_begin``, in the order of their times: (source file, line, kind, CTA's linear
    index, CTAs of its grid, ns, SM); kind 0: the CTA let its dependents start (about its start), 1: its wait
    for the predecessor returned."""
    cap = 1 << 20
    buf = (ctypes.c_ulonglong * (4 * cap))()
    lib().qe_timeline_read.restype = ctypes.c_long
    n = int(lib().qe_timeline_read(buf, ctypes.c_long(cap)))
    if n < 0:
        raise ExtensionMissing("this build of the library records no timeline (build and run with QE_TIMELINE=1)")

    def fnv(name: str) -> int:
        h = 2166136261
        for ch in name.encode():
            h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
        return h
    names = {fnv(f): f for f in os.listdir(_build.CSRC_DIR) if f.endswith((".cu", ".cuh", ".h"))}
    out = []
    for i in range(n):
        w, c, t, sm = (int(buf[4 * i + j]) for j in range(4))
        out.append((names.get(w >> 32, hex(w >> 32)), (w >> 16) & 0xFFFF, w & 3, c >> 32, c & 0xFFFFFFFF, t, sm))
    out.sort(key=lambda e: e[5])
    return out


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch of the kernels (on by default): a kernel may start, and a
    product may begin to fetch its weights, while the kernel before it is still running."""
    lib().qe_set_pdl(int(bool(enabled)))


def tc_attention_status() -> int:
    """0, or the code of the first wait inside the tcgen05 attention kernel that ran out."""
    return int(lib().qe_flash_attention_tc_status())


def tcgen05_status() -> int:
    """0 if no bounded wait of the tcgen05 product kernels ever ran out; else the code of the first
    that did (1: a shared-memory slot never came free, 2: TMA bytes never landed, 3: the
    accumulator never completed, 4: an accumulator was never read out; 11-13: the same as 1-3 in the
    kernel for some tens of rows, 21-23 in its form that shares K within a cluster).  Synchronises the device."""
    return (int(lib().qe_gemm_tc_status()) or int(lib().qe_gemm_tc_swap_status()) or int(lib().qe_gemm_tc_pair_status())
            or int(lib().qe_gemm_tc_splitk_status()))


class DeviceWaitTimeout(RuntimeError):
    """A bounded wait inside a kernel ran out: the kernel gave up without storing its output, so what
    the step produced is not to be trusted."""


_STATUS_WORDS = ("qe_gemm_tc", "qe_gemm_tc_swap", "qe_gemm_tc_pair", "qe_gemm_tc_splitk", "qe_flash_attention_tc",
                 "qe_flash_attention", "qe_decode_attention_mma", "qe_small_m")


def device_status() -> dict[str, int]:
    """The status words of the kernels whose waits are bounded that are not zero: kernel family -> code
    of its first wait that ran out.  Synchronises the device (one small copy per word)."""
    if _lib is None:
        return {}                   # nothing was ever launched
    out = {}
    for name in _STATUS_WORDS:
        code = int(getattr(lib(), name + "_status")())
        if code:
            out[name[3:]] = code
    return out


def clear_device_status() -> None:
    """Set the status words back to zero, and the counters by which split contexts find their last part
    (a kernel that gave up may have left them counted up)."""
    if _lib is None:
        return
    for name in _STATUS_WORDS:
        getattr(lib(), name + "_clear_status")()
    for t in _merge_counter_tensors.values():
        t.zero_()


def check_device_status() -> None:
    """Raise ``DeviceWaitTimeout`` if any bounded wait ran out since the words were last cleared (and clear
    them).  The engine calls this where it synchronises anyway: at the end of ``serving``."""
    bad = device_status()
    if bad:
        clear_device_status()
        raise DeviceWaitTimeout(
            "a bounded wait inside a kernel ran out and the kernel returned without its output: "
            + ", ".join(f"{k} (code {v})" for k, v in bad.items())
            + "; the tokens of the steps since the last check are not to be trusted")


def selftest_starved_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, limit: int = 10000) -> None:
    """For tests: one CTA of the tcgen05 product kernel whose loads are withheld, with waits of ``limit``
    polls.  It must give up, store nothing into ``out``, free its tensor memory and leave a code in
    ``tcgen05_status()``; the device stays usable."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (M, N)
          and x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "selftest: contiguous bfloat16 operands")
    _check(lib().qe_gemm_tc_selftest_starved(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(limit), _stream()), "selftest")


ROPE_TABLE_MIN_T = 64   # tokens from which a step's rotation angles are computed once (below: in the kernel)


def rope_table_applies(num_tokens: int, dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether the kernels that rotate q and k take a table of this step's cosines and sines (``rope_table``)
    instead of computing the angles themselves: many tokens, bfloat16, head size 128 rotated as a whole."""
    return num_tokens >= ROPE_TABLE_MIN_T and dtype == torch.bfloat16 and head_dim == 128 and rotary_dim == head_dim


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = (cos, sin)(positions[t] * inv_freq[j]) in float32; out [T, len(inv_freq), 2]."""
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    _need(out.dtype == torch.float32 and out.shape == (T, half, 2) and out.is_contiguous(), "rope_table: out must be float32 [T, half, 2]")
    _check(lib().qe_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rope_table")


def qk_norm_rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                          k_norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor],
                          rotary_dim: int, kv_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                          num_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool = True,
                          cos_sin: Optional[torch.Tensor] = None, norm_dim: Optional[int] = None, magnitude: float = 1.0,
                          value_mix=None) -> None:
    """On the stacked projection output qkv [T, (Hq + 2 Hkv) D] (rows may be strided: the leading columns
    of a wider product), in place: per-head RMS norm of q and k (if weights are given), half-split rotation
    by positions (if inv_freq is given); then k and v are written to the slots of ``slot_mapping`` in
    ``kv_pages`` [pages, 2, Hkv, page, D].  ``norm_dim``: the channels the norm's mean runs over, where a
    head is padded with zero channels up to D.  ``magnitude``: cosines and sines are multiplied by it.
    ``value_mix``: values shared across layers, ("keep", first) copies this layer's values of the step's tokens into
    ``first`` [T, Hkv Dv] (Dv <= D: the heads' own channels, without padding); ("blend", first, lam) caches
    (1 - lam) v + lam first in the place of v."""
    T = qkv.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    _need(qkv.shape == (T, (Hq + 2 * Hkv) * D) and qkv.stride(1) == 1, "qk_norm_rope_kv_write: qkv must be [T, (Hq+2Hkv)D]")
    _i32(positions, "positions")
    stride = qkv.stride(0)
    q = qkv
    k = qkv[:, Hq * D:]
    v = qkv[:, (Hq + Hkv) * D:]
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None, "qk_norm_rope_kv_write: cache write without a cache")
        _need(kv_pages.dtype == qkv.dtype and kv_pages.is_contiguous() and kv_pages.dim() == 5
              and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == D,
              "qk_norm_rope_kv_write: kv_pages must be [pages, 2, Hkv, page, D] in qkv's dtype")
        _i32(slot_mapping, "slot_mapping")
        _need(slot_mapping.numel() >= T, "qk_norm_rope_kv_write: one cache slot per token")
        page_size = kv_pages.shape[3]
    for wt in (q_norm_w, k_norm_w):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.shape == (D,), "qk_norm_rope_kv_write: norm weights must be float32 [D]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "qk_norm_rope_kv_write: inv_freq must be float32 [rotary_dim / 2]")
    v_first, v_mode, v_lambda, v_dim = None, 0, 0.0, D
    if value_mix is not None:
        _need(value_mix[0] in ("keep", "blend"), "qk_norm_rope_kv_write: value_mix is ('keep', first) or ('blend', first, lam)")
        v_first, v_mode = value_mix[1], 1 if value_mix[0] == "keep" else 2
        v_lambda = float(value_mix[2]) if v_mode == 2 else 0.0
        _need(v_first.dim() == 2 and v_first.shape[0] == T and v_first.shape[1] % Hkv == 0 and 1 <= v_first.shape[1] // Hkv <= D
              and v_first.dtype == qkv.dtype and v_first.is_contiguous(),
              "qk_norm_rope_kv_write: the shared values must be contiguous [T, Hkv Dv] in qkv's dtype, Dv <= D")
        v_dim = v_first.shape[1] // Hkv
    _check(lib().qe_qk_norm_rope_kv_write(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(v.data_ptr()),
        ctypes.c_long(stride), ctypes.c_long(stride), ctypes.c_long(stride), _ptr(positions),
        _ptr(q_norm_w), _ptr(k_norm_w), ctypes.c_float(eps), _ptr(inv_freq),
        _ptr(cos_sin if (cos_sin is not None and D == 128 and rotary_dim == D) else None), int(rotary_dim),
        _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None),
        T, Hq, Hkv, D, page_size, int(bool(write_kv)), _dt(qkv), int(norm_dim or D), ctypes.c_float(magnitude), _ptr(v_first),
        v_mode, ctypes.c_float(v_lambda), int(v_dim), _stream()), "qk_norm_rope_kv_write")


def rope_neox(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
              rotary_dim: int) -> None:
    """Half-split rotation of q [T, Hq, D] and k [T, Hkv, D] in place (rows may be strided)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    _need(q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D,
          "rope_neox: heads of a token must be contiguous")
    _i32(positions, "positions")
    _check(lib().qe_qk_norm_rope_kv_write(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(0),
        ctypes.c_long(q.stride(0)), ctypes.c_long(k.stride(0)), ctypes.c_long(0), _ptr(positions),
        _ptr(None), _ptr(None), ctypes.c_float(0.0), _ptr(inv_freq), _ptr(None), int(rotary_dim),
        _ptr(None), _ptr(None), T, Hq, Hkv, D, 1, 0, _dt(q), D, ctypes.c_float(1.0), _ptr(None), 0, ctypes.c_float(0.0), D,
        _stream()), "rope_neox")


def flash_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernel takes this geometry (else the generic kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and num_kv_heads >= 1 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= FLASH_ROWS)


def tc_attention_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernel takes this geometry (prompt portions; else the mma.sync kernel)."""
    if dtype != torch.bfloat16 or head_dim != 128 or num_kv_heads < 1 or num_heads % num_kv_heads:
        return False
    G = num_heads // num_kv_heads
    return G <= 128 and G & (G - 1) == 0 and page_size >= 8 and page_size & (page_size - 1) == 0


def _plan_tc_tiles(tiles: list, Hkv: int) -> tuple[list[int], int, list[int], int]:
    """Work items of the tcgen05 kernel from its tiles (key steps, first key, last key, item fields),
    sorted by their steps, longest first.  Where the tiles alone would leave SMs idle (a short portion
    behind a long context: few tiles; one prompt of a few thousand tokens: tiles as unequal as
    1 : 2 : ... : n), the longer tiles are cut into parts of whole steps; the library works out the most
    steps an item may have by laying out the candidates' schedules (a part costs its scratch and the
    merge, about as much as a step).  The kernel's CTAs, one per SM at most, run the units (an item for one kv
    head) one after the other; the library deals them out, longest first, each to the CTA with the least work
    so far.  Returns the items, the number of parts, the schedule (the CTAs' offsets into the list itself,
    then their unit numbers) and the number of CTAs."""
    cap = TC_FORCE_CAP
    if cap < 0:
        cap = 0
        if tiles and len(tiles) * Hkv < TC_BALANCE_BELOW_CTAS:
            steps = (ctypes.c_int * len(tiles))(*[t[0] for t in tiles])
            cap = int(lib().qe_flash_attention_tc_balance(steps, len(tiles), Hkv, TC_TARGET_CTAS, TC_MIN_PART_STEPS, TC_MAX_PARTS,
                                                          ctypes.c_float(TC_ITEM_COST_STEPS), ctypes.c_float(TC_PART_COST_STEPS)))
    out: list[tuple[int, list[int]]] = []
    n_parts = 0
    for steps, lo, hi, (r, q0, row0, n, c) in tiles:
        parts = min(TC_MAX_PARTS, -(-steps // cap)) if cap else 1
        if parts <= 1:
            out.append((steps, [r, q0, lo, hi, -1, 0, 0, row0, n, c, 0, 0]))
            continue
        per = -(-steps // parts)
        lo_al = lo // TC_BN * TC_BN
        parts = -(-steps // per)
        for sp in range(parts):
            k0 = lo if sp == 0 else lo_al + sp * per * TC_BN
            k1 = min(hi, lo_al + (sp + 1) * per * TC_BN)
            out.append((min(per, steps - sp * per), [r, q0, k0, k1, n_parts + sp, parts, sp, row0, n, c, 0, 0]))
        n_parts += parts
    out.sort(key=lambda kv: -kv[0])
    n_ctas = min(len(out) * Hkv, TC_TARGET_CTAS)
    costs = (ctypes.c_float * len(out))(*[st + TC_ITEM_COST_STEPS + (TC_PART_COST_STEPS if item[4] >= 0 else 0.0) for st, item in out])
    sched = (ctypes.c_int * (n_ctas + 1 + len(out) * Hkv))()
    n = int(lib().qe_flash_attention_tc_schedule(costs, len(out), Hkv, n_ctas, sched))
    _need(n == len(sched), "plan_attention: the schedule of the tcgen05 kernel could not be made")
    return [x for _, item in out for x in item], n_parts, list(sched), n_ctas


def split_geometry(geo) -> tuple:
    """(heads, kv heads, head size, window, biased) of a geometry; the fifth entry (scores biased by distance:
    only some kernels take them) may be left out."""
    Hq, Hkv, D, window = geo[:4]
    return Hq, Hkv, D, window, bool(len(geo) > 4 and geo[4])


def geometry_planes(geo) -> int:
    """The sixth entry of a geometry, if it has one: 1 for a cache whose pages hold one plane per kv head, the values
    being the keys' channels (a latent cache; the tcgen05 kernel does not take it), else 2."""
    return int(geo[5]) if len(geo) > 5 else 2


def plan_attention(q_lens: list[int], ctx_lens: list[int], page_size: int,
                   geometries=(), dtype: torch.dtype = torch.float32,
                   uniform_splits: Optional[dict] = None) -> dict[str, list[int]]:
    """Work lists of the attention kernels for one step's batch, as named int32 lists that the
    step function copies to the device with the rest of the step's metadata.

    ``geometries``: the (heads, kv heads, head size, window[, biased by distance]) of the model's attention layers.
    ``tiles`` serves the generic kernel; for each geometry the flash kernel takes, ``fa<i>_items``
    and ``fa<i>_merge`` hold its work and merge items and ``fa<i>_info`` = [parts, rows per part,
    whether every item has at most 16 rows, the most rows of an item, the number of parts of every
    request if all are cut into the same 2, 4 or 8 parts (they can then form clusters) else 0]; requests that bring many rows go to the tcgen05 kernel
    instead where it takes the geometry: ``tc<i>_items``, ``tc<i>_sched`` (which CTA runs which
    item for which kv head) and ``tc<i>_info`` = [parts, rows per part, CTAs].
    ``uniform_splits`` (geometry -> number of parts) fixes the number of parts of every request,
    so that the lists depend on the batch's shape only (for steps replayed from a CUDA graph)."""
    tiles: list[int] = []
    for r, n in enumerate(q_lens):
        for q0 in range(0, n, ATTN_TILE_Q):
            tiles += [r, q0]
    plan = {"tiles": tiles}
    for gi, geo in enumerate(geometries):
        Hq, Hkv, D, window, biased = split_geometry(geo)
        if not flash_supported(dtype, Hq, Hkv, D):
            continue
        G = Hq // Hkv
        tpt = FLASH_ROWS // G
        use_tc = uniform_splits is None and geometry_planes(geo) == 2 and tc_attention_supported(dtype, Hq, Hkv, D, page_size)
        on_tc = [use_tc and n * G >= TC_MIN_ROWS for n in q_lens]
        tc_tiles: list = []
        base = sum(-(-n // tpt) for n, tc in zip(q_lens, on_tc) if not tc) * Hkv
        items: list[int] = []
        merge: list[int] = []
        n_parts, part_rows, row0, max_rows = 0, 1, 0, 0
        whole: list[tuple[int, list[int]]] = []        # (keys the tile visits, its work item)
        for r, (n, c) in enumerate(zip(q_lens, ctx_lens)):
            total = c + n
            if on_tc[r]:
                tc_tpt = TC_ROWS // G
                for q0 in range(0, n, tc_tpt):
                    lo = max(0, c + q0 - window + 1) if window else 0
                    hi = c + min(n, q0 + tc_tpt)
                    tc_tiles.append((-(-(hi - lo // TC_BN * TC_BN) // TC_BN), lo, hi, (r, q0, row0, n, c)))
                row0 += n
                continue
            if uniform_splits is not None:
                splits = uniform_splits[geo]
            else:
                lo = (max(0, c - window + 1) // FLASH_BN) * FLASH_BN if window else 0
                splits = 1
                if n <= tpt and base < FLASH_TARGET_CTAS and total - lo > FLASH_SPLIT:
                    splits = min(-(-(total - lo) // FLASH_SPLIT), max(1, FLASH_TARGET_CTAS // base))
            if splits > 1:
                for sp in range(splits):
                    items += [r, 0, 0, 0, n_parts + sp, splits, sp, row0, n, c, 0, 0]
                merge += [r, 0, n_parts, splits]
                n_parts += splits
                part_rows = max(part_rows, n * G)
            else:
                for q0 in range(0, n, tpt):
                    whole.append((c + min(n, q0 + tpt), [r, q0, 0, total, -1, 0, 0, row0, n, c, 0, 0]))
            row0 += n
            max_rows = max(max_rows, min(n, tpt) * G)
        # tiles that visit many keys start first, so that the last wave of CTAs is made of short ones
        whole.sort(key=lambda kv: -kv[0])
        items = [x for _, item in whole for x in item] + items
        plan[f"fa{gi}_items"] = items
        plan[f"fa{gi}_merge"] = merge
        sizes = {m for m in merge[3::4]}
        same = sizes.pop() if len(sizes) == 1 and not whole else 0
        plan[f"fa{gi}_info"] = [n_parts, part_rows, int(max_rows <= 16), max_rows, same if same in (2, 4, 8) else 0]
        if tc_tiles:
            tc_items, tc_parts, tc_sched, tc_ctas = _plan_tc_tiles(tc_tiles, Hkv)
            plan[f"tc{gi}_items"] = tc_items
            plan[f"tc{gi}_sched"] = tc_sched
            plan[f"tc{gi}_info"] = [tc_parts, TC_ROWS, tc_ctas]
    return plan


DECODE_CLUSTER4_MAX_SPAN = 4096   # keys up to which 4 parts in a cluster are preferred to more parts merged through memory


def decode_splits(num_reqs: int, max_tokens: int, geometries, dtype: torch.dtype) -> dict:
    """The fixed number of parts per request for a decode step of ``num_reqs`` requests whose block
    tables hold up to ``max_tokens`` tokens: enough parts to fill the GPU, none shorter than a split."""
    out = {}
    for geo in geometries:
        Hq, Hkv, D, window, _ = split_geometry(geo)
        span = min(max_tokens, window) if window else max_tokens
        target = FLASH_TARGET_CTAS
        if (DECODE_ATTENTION_MMA and DECODE_ATTENTION_MMA_WIDE and dtype == torch.bfloat16 and D == 128
                and Hq // Hkv <= 16 and num_reqs * Hkv <= TC_TARGET_CTAS):
            target = TC_TARGET_CTAS                                       # one CTA of 8 warps per SM
        want = max(1, target // max(1, num_reqs * Hkv))                   # all parts run in one wave
        parts = max(1, min(want, -(-span // FLASH_SPLIT)))
        if target == TC_TARGET_CTAS and DECODE_ATTENTION_CLUSTERS and parts > 2:
            # 2, 4 or 8 parts of a request form a thread-block cluster and meet on chip, which beats the merge through
            # global memory (measured at 0.6B sizes, context 1 024: 2 requests in 4 parts each 0.80 ms a step, in 5
            # parts 0.95); clusters of 8 only while all of them still fit the GPU at once (at most 8 of them: 0.95 ms
            # with 16 of them) or where 4 parts would be long ones
            few = num_reqs * Hkv * 8 <= 64
            if parts == 3:
                parts = 4 if num_reqs * Hkv * 4 <= target else 2
            elif parts < 8:
                parts = 8 if few else 4
            elif few or (parts == 8 and span > DECODE_CLUSTER4_MAX_SPAN):
                parts = 8
            elif span <= DECODE_CLUSTER4_MAX_SPAN:
                parts = 4
        out[geo] = parts
    return out


_MERGE_COUNTERS = 1 << 16
_merge_counter_tensors: dict = {}


def _merge_counters(device, kernel: str = "fa") -> torch.Tensor:
    """Zeroed ints, one per (part, kv head), that an attention kernel uses to find the CTA that finishes a
    split context last (it merges the parts and sets its counter back to zero).  One tensor per device
    and kernel for the life of the process, so that its address is the same in every captured step."""
    key = (torch.device(device).index, kernel)
    t = _merge_counter_tensors.get(key)
    if t is None:
        t = torch.zeros(_MERGE_COUNTERS, dtype=torch.int32, device=device)
        _merge_counter_tensors[key] = t
    return t


def _decode_mma_serves(plan, key, qkv: torch.Tensor, Hq: int, Hkv: int, D: int) -> bool:
    """Whether the step's requests that are not on the tcgen05 kernel (geometry index ``key`` of the plan) go to
    the tensor-core kernel for decoded tokens: items of at most 16 rows, head size 128."""
    if not DECODE_ATTENTION_MMA or key is None or f"fa{key}_items" not in plan or D != 128:
        return False
    if f"tc{key}_items" in plan and not DECODE_ATTENTION_MMA_BESIDE_TC:
        return False
    n_parts, part_rows, small_tiles, max_rows, same_parts = plan[f"fa{key}_info_host"]
    n_items = plan[f"fa{key}_items"].numel() // FLASH_ITEM_INTS
    return (1 <= max_rows <= 16 and Hq // Hkv <= 16 and n_items > 0 and n_items * Hkv >= DECODE_ATTENTION_MMA_MIN_CTAS
            and n_parts * Hkv <= _MERGE_COUNTERS and qkv.stride(0) % 8 == 0)


def paged_attention(qkv: torch.Tensor, kv_pages: torch.Tensor, block_tables: torch.Tensor, ctx,
                    out: torch.Tensor, scale: float, window: int, num_heads: int, num_kv_heads: int,
                    head_dim: int, next_pages: Optional[torch.Tensor] = None,
                    slopes: Optional[torch.Tensor] = None, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                    value_shift: int = 0, value_shifts: int = 1) -> None:
    """Attention of the step's queries (the q part of qkv [T, (Hq+2Hkv) D]) over the keys and values
    of their requests in ``kv_pages``; out [T, Hq D].  ``ctx`` is the StepContext (cu_q, ctx_lens,
    the plan that ``plan_attention`` made, and the arena for the parts of split contexts).

    ``slopes`` (float32 [Hq]): the score of query i and key j of head h is scale q.k - slopes[h] (i - j).

    ``softcap`` > 0: the scaled score s becomes softcap tanh(s / softcap).  ``sinks`` (float32 [Hq]): exp(sinks[h])
    joins the softmax's denominator of head h; it has no key and no value.  ``value_shift`` s: the weights of a head
    whose kv head is c meet the values of kv head (c + s) mod Hkv (a mixer that mixes the heads' weights sums such
    outputs).  Every kernel takes the three (not together with a distance bias or a cache of one plane).
    ``value_shifts`` S > 1: out is [S, T, Hq D] and entry s is the output for shift s; where the whole step is served by
    the kernels for few rows, the shifts are one launch (a grid dimension), else one launch each.

    ``next_pages``: the cache of the layer that runs after this one, if it has the same shape (the same
    pages at the same places): a decode step's kernel may ask L2 for that layer's keys and values."""
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    T = qkv.shape[0]
    S = int(value_shifts)
    if S > 1:
        _need(value_shift == 0 and S <= Hkv and out.shape == (S, T, Hq * D) and out.is_contiguous() and out.dtype == qkv.dtype,
              "paged_attention: several shifts write out [S, T, Hq D], S <= Hkv")
        plan0 = ctx.attn_plan
        key0 = plan0.get("geometry_index", {}).get((Hq, Hkv, D, window), plan0.get("geometry_index", {}).get((Hq, Hkv, D, window, False)))
        one_launch = (SHIFTS_IN_ONE_LAUNCH and key0 is not None and f"fa{key0}_items" in plan0 and f"tc{key0}_items" not in plan0
                      and plan0[f"fa{key0}_info_host"][0] * Hkv * S <= _MERGE_COUNTERS and kv_pages.shape[1] == 2 and slopes is None)
        if not one_launch:
            for s in range(S):
                paged_attention(qkv, kv_pages, block_tables, ctx, out[s], scale, window, Hq, Hkv, D, next_pages, slopes, softcap, sinks, s)
            return
    else:
        _need(out.shape == (T, Hq * D) and out.is_contiguous() and out.dtype == qkv.dtype, "paged_attention: out must be [T, Hq D]")
    _need(kv_pages.dtype == qkv.dtype and kv_pages.dim() == 5 and kv_pages.is_contiguous() and kv_pages.shape[1] in (1, 2),
          "paged_attention: kv_pages must be [pages, 2 (or 1: the values are the keys' channels), Hkv, page, D] in q's dtype")
    planes = int(kv_pages.shape[1])
    _i32(block_tables, "block_tables")
    global last_attention_kernel
    plan = ctx.attn_plan
    if slopes is not None:
        _need(slopes.dtype == torch.float32 and slopes.numel() == Hq and slopes.is_contiguous(), "paged_attention: slopes must be float32 [Hq]")
    index = plan.get("geometry_index", {})
    plain = softcap > 0.0 or sinks is not None or value_shift != 0 or S > 1
    if sinks is not None:
        _need(sinks.dtype == torch.float32 and sinks.numel() == Hq and sinks.is_contiguous(), "paged_attention: sinks must be float32 [Hq]")
    if plain:
        _need(planes == 2 and slopes is None and 0 <= value_shift < Hkv,
              "paged_attention: bent scores, sinks and shifted values go with a cache of two planes and no distance bias")
    if planes == 1:
        _need(slopes is None, "paged_attention: no distance bias over a cache of one plane")
        key = index.get((Hq, Hkv, D, window, False, 1))
    else:
        key = index.get((Hq, Hkv, D, window, True)) if slopes is not None else index.get((Hq, Hkv, D, window), index.get((Hq, Hkv, D, window, False)))
    if key is not None and f"tc{key}_items" in plan:
        last_attention_kernel = "flash_attention_tc"
        tc_items = plan[f"tc{key}_items"]
        tc_parts, tc_rows, tc_ctas = plan[f"tc{key}_info_host"]
        part_acc = part_ml = counters = None
        if tc_parts:
            _need(2 * tc_parts * Hkv <= _MERGE_COUNTERS, "paged_attention: too many parts")   # (two counters a tile and kv head)
            part_acc = ctx.arena.alloc((tc_parts * Hkv * tc_rows, D), torch.float32)
            part_ml = ctx.arena.alloc((tc_parts * Hkv * tc_rows, 2), torch.float32)
            counters = _merge_counters(qkv.device, "tc")
        _check(lib().qe_flash_attention_tc(
            _ptr(qkv), ctypes.c_long(qkv.stride(0)), T, _ptr(kv_pages), int(kv_pages.shape[0]), _ptr(block_tables),
            int(block_tables.shape[1]), _ptr(tc_items), tc_items.numel() // FLASH_ITEM_INTS,
            _ptr(plan[f"tc{key}_sched"]), int(tc_ctas), _ptr(out),
            _ptr(part_acc), _ptr(part_ml), int(tc_rows), _ptr(counters), ctypes.c_float(scale), int(window),
            Hq, Hkv, D, int(kv_pages.shape[3]), _ptr(slopes), ctypes.c_float(softcap), _ptr(sinks), int(value_shift), _stream()),
            "flash_attention_tc")
    if key is not None and f"fa{key}_items" in plan:
        items, merge = plan[f"fa{key}_items"], plan[f"fa{key}_merge"]
        n_parts, part_rows, small_tiles, max_rows, same_parts = plan[f"fa{key}_info_host"]
        n_items, n_merge = items.numel() // FLASH_ITEM_INTS, merge.numel() // 4
        if n_items == 0 and f"tc{key}_items" in plan:
            return                      # every request of the step went to the kernel above
        part_acc = part_ml = None
        if n_parts:
            part_acc = ctx.arena.alloc((S * n_parts * Hkv * part_rows, D), torch.float32)
            part_ml = ctx.arena.alloc((S * n_parts * Hkv * part_rows, 2), torch.float32)
        counters = _merge_counters(qkv.device) if 0 < S * n_parts * Hkv <= _MERGE_COUNTERS else None
        # every request in the same few parts: the parts of a request form a cluster and meet on chip
        cluster = int(same_parts) if DECODE_ATTENTION_CLUSTERS and n_items == n_parts else 0
        if _decode_mma_serves(plan, key, qkv, Hq, Hkv, D):
            # decoded tokens: every warp streams key groups of its own through the tensor cores
            last_attention_kernel = "decode_attention_mma"
            lib().qe_decode_attention_mma_stages(int(DECODE_ATTENTION_MMA_STAGES))
            lib().qe_decode_attention_mma_early(int(DECODE_ATTENTION_MMA_EARLY))
            ahead = None
            if (next_pages is not None and DECODE_PREFETCH_KV_MB > 0 and next_pages.shape == kv_pages.shape
                    and next_pages.dtype == kv_pages.dtype and next_pages.is_contiguous()):
                tokens = sum(ctx.ctx_lens_host) + sum(ctx.q_lens_host)
                if tokens * 2 * Hkv * D * kv_pages.element_size() <= DECODE_PREFETCH_KV_MB << 20:
                    ahead = next_pages
            _check(lib().qe_decode_attention_mma(
                _ptr(qkv), ctypes.c_long(qkv.stride(0)), _ptr(kv_pages), _ptr(ahead), _ptr(block_tables), int(block_tables.shape[1]),
                _ptr(items), n_items, _ptr(out), _ptr(part_acc), _ptr(part_ml), int(part_rows), _ptr(counters),
                int(max_rows), cluster, int(DECODE_ATTENTION_MMA_WIDE and n_items * Hkv * S <= TC_TARGET_CTAS),
                ctypes.c_float(scale), int(window), Hq, Hkv, D, int(kv_pages.shape[3]), _ptr(slopes), planes,
                ctypes.c_float(softcap), _ptr(sinks), int(value_shift), S, ctypes.c_long(T * Hq * D), int(n_parts), _stream()),
                "decode_attention_mma")
            return
        last_attention_kernel = "flash_attention"
        _check(lib().qe_flash_attention_fused_merge(
            _ptr(qkv), ctypes.c_long(qkv.stride(0)), _ptr(kv_pages), _ptr(block_tables), int(block_tables.shape[1]),
            _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), _ptr(items), n_items, _ptr(merge), n_merge, _ptr(out),
            _ptr(part_acc), _ptr(part_ml), int(part_rows), _ptr(counters), int(small_tiles), ctypes.c_float(scale), int(window),
            Hq, Hkv, D, int(kv_pages.shape[3]), _ptr(slopes), planes, ctypes.c_float(softcap), _ptr(sinks), int(value_shift),
            S, ctypes.c_long(T * Hq * D), int(n_parts), _stream()), "flash_attention")
        return
    tiles = plan["tiles"]
    n_tiles = tiles.numel() // 2
    last_attention_kernel = "paged_attention_generic"
    _check(lib().qe_paged_attention_generic(
        _ptr(qkv), ctypes.c_long(qkv.stride(0)), _ptr(kv_pages), _ptr(block_tables), int(block_tables.shape[1]),
        _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), _ptr(tiles), n_tiles, _ptr(out), ctypes.c_float(scale), int(window),
        Hq, Hkv, D, int(kv_pages.shape[3]), _dt(qkv), _ptr(slopes), planes, ctypes.c_float(softcap), _ptr(sinks),
        int(value_shift), _stream()), "paged_attention")


def place_tokens(token_ids: torch.Tensor, rows: torch.Tensor, src: torch.Tensor, src_index: torch.Tensor) -> None:
    """token_ids[rows[i]] = src[src_index[i]], all int32 on the device."""
    for t, name in ((token_ids, "token_ids"), (rows, "rows"), (src, "src"), (src_index, "src_index")):
        _i32(t, name)
    _need(rows.numel() == src_index.numel(), "place_tokens: one source index per row")
    _check(lib().qe_place_tokens(_ptr(token_ids), _ptr(rows), _ptr(src), _ptr(src_index), rows.numel(), _stream()),
           "place_tokens")


def copy_pages(cache: torch.Tensor, pairs: torch.Tensor) -> None:
    """cache[s, pairs[2 i + 1]] = cache[s, pairs[2 i]] for every cache slot s of a group's tensor
    [slots, pages, ...] and every pair of the int32 list on the device: whole pages, one launch."""
    _i32(pairs, "pairs")
    _need(cache.dim() >= 3 and cache.is_contiguous(), "copy_pages: cache must be contiguous [slots, pages, ...]")
    _need(pairs.numel() % 2 == 0, "copy_pages: pairs of (source page, destination page)")
    n_slots, n_pages = int(cache.shape[0]), int(cache.shape[1])
    page_bytes = cache[0, 0].numel() * cache.element_size()
    _check(lib().qe_copy_pages(_ptr(cache), n_slots, n_pages, ctypes.c_long(page_bytes), _ptr(pairs), pairs.numel() // 2,
                               _stream()), "copy_pages")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    T, I2 = gate_up.shape
    _need(I2 % 2 == 0 and out.shape == (T, I2 // 2) and out.dtype == gate_up.dtype
          and out.is_contiguous() and gate_up.is_contiguous(), "silu_mul: out must be [T, I] for gate_up [T, 2I]")
    _check(lib().qe_silu_mul(_ptr(gate_up), _ptr(out), T, I2 // 2, _dt(out), _stream()), "silu_mul")


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]; act "silu", or "gelu_tanh":
    0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  Float32 arithmetic, rounded once."""
    T, I2 = gate_up.shape
    _need(gate_activation_known(activation), f"act_mul: unknown activation {activation!r}")
    _need(I2 % 2 == 0 and out.shape == (T, I2 // 2) and out.dtype == gate_up.dtype
          and out.is_contiguous() and gate_up.is_contiguous(), "act_mul: out must be [T, I] for gate_up [T, 2I]")
    _check(lib().qe_act_mul(_ptr(gate_up), _ptr(out), T, I2 // 2, _dt(out), gate_code(activation), _stream()), "act_mul")


def _rows(t: torch.Tensor, name: str) -> None:
    _need(t.dim() == 2 and t.stride(1) == 1, f"{name} must be rows with unit stride along the columns")


def channel_decay(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], tau: float, out: torch.Tensor,
                  log_rate: Optional[torch.Tensor] = None) -> None:
    """out[t, n] = sigmoid(z)^(1 / tau) with z = a[t] . w[n] + bias[n], in float32: the decay of a recurrence
    from the second half of a low-rank pair.  a [T, R] (rows may be strided), w [N, R], out float32 [T, N].
    With ``log_rate`` (float32 [G], G dividing N): out = exp(-exp(log_rate[n // (N / G)]) softplus(z)) instead."""
    _rows(a, "channel_decay: a")
    T, R = a.shape
    N = w.shape[0]
    _need(w.shape == (N, R) and w.dtype == a.dtype and w.is_contiguous(), "channel_decay: w must be [N, R] in a's dtype")
    _need(out.shape == (T, N) and out.dtype == torch.float32 and out.is_contiguous(), "channel_decay: out must be float32 [T, N]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.shape == (N,) and bias.is_contiguous(), "channel_decay: bias must be float32 [N]")
    per = 1
    if log_rate is not None:
        _need(log_rate.dtype == torch.float32 and log_rate.dim() == 1 and log_rate.is_contiguous() and N % log_rate.numel() == 0,
              "channel_decay: log_rate must be float32 [G] with G dividing N")
        per = N // log_rate.numel()
    _check(lib().qe_channel_decay(_ptr(a), ctypes.c_long(a.stride(0)), _ptr(w), _ptr(bias), ctypes.c_float(tau), _ptr(out),
                                  T, N, R, _dt(a), _ptr(log_rate), per, _stream()), "channel_decay")


SCAN_FORMS_DECAY = True     # steps of single tokens: the scan forms the decay from the low-rank pair itself (no decay kernel)


def linear_attention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alpha: Optional[torch.Tensor], state: torch.Tensor,
                          ctx, out: torch.Tensor, q_scale: float, num_heads: int, key_dim: int, value_dim: int,
                          write_state: bool = True, decay=None, head_decay: Optional[torch.Tensor] = None) -> None:
    """The recurrence S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_scale q_t) per head, over the step's
    tokens of every request, from the state its slot holds (zero for a request without context) to the
    state after its last token.  q, k [T, H dk] and v [T, H dv] in the compute type (rows may be strided),
    alpha float32 [T, H dk], state float32 [slots, H, dv, dk], out float32 [T, H dv].
    A step of single tokens may leave ``alpha`` None and give ``decay`` = (a, w, bias, tau) as ``channel_decay``
    takes them: the scan then forms alpha itself, to the same bits.  ``head_decay`` (float32 [H]) in the place of
    both: alpha is one constant per head."""
    H, dk, dv = num_heads, key_dim, value_dim
    T = q.shape[0]
    for t, name, width in ((q, "q", H * dk), (k, "k", H * dk), (v, "v", H * dv)):
        _rows(t, f"linear_attention_scan: {name}")
        _need(t.shape == (T, width) and t.dtype == q.dtype, f"linear_attention_scan: {name} must be [T, {width}]")
    da = dw = db = None
    tau, rank = 1.0, 0
    if head_decay is not None:
        _need(alpha is None and decay is None and head_decay.dtype == torch.float32 and head_decay.shape == (H,)
              and head_decay.is_contiguous(), "linear_attention_scan: head_decay must be float32 [H], alone")
    elif alpha is None:
        _need(decay is not None and int(ctx.max_q_len) <= 1, "linear_attention_scan: without alpha, single tokens and the decay's inputs")
        da, dw, db, tau = decay
        _rows(da, "linear_attention_scan: decay a")
        rank = da.shape[1]
        _need(da.shape[0] == T and da.dtype == q.dtype and dw.dtype == q.dtype and dw.shape == (H * dk, rank) and dw.is_contiguous(),
              "linear_attention_scan: decay a [T, rank] and w [H dk, rank] in q's dtype")
        _need(db is None or (db.dtype == torch.float32 and db.shape == (H * dk,) and db.is_contiguous()),
              "linear_attention_scan: decay bias must be float32 [H dk]")
    else:
        _need(alpha.shape == (T, H * dk) and alpha.dtype == torch.float32 and alpha.is_contiguous(),
              "linear_attention_scan: alpha must be float32 [T, H dk]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dv, dk),
          "linear_attention_scan: state must be float32 [slots, H, dv, dk]")
    _need(out.shape == (T, H * dv) and out.dtype == torch.float32 and out.is_contiguous(),
          "linear_attention_scan: out must be float32 [T, H dv]")
    _check(lib().qe_linear_attention_scan(
        _ptr(q), _ptr(k), _ptr(v), ctypes.c_long(q.stride(0)), ctypes.c_long(k.stride(0)), ctypes.c_long(v.stride(0)),
        _ptr(alpha), _ptr(state), _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), _ptr(ctx.slot_ids), _ptr(out), ctypes.c_float(q_scale),
        int(ctx.num_reqs), int(ctx.max_q_len), H, dk, dv, int(bool(write_state)), _dt(q), _ptr(da),
        ctypes.c_long(da.stride(0) if da is not None else 0), _ptr(dw), _ptr(db), ctypes.c_float(tau), int(rank),
        _ptr(head_decay), _stream()),
        "linear_attention_scan")


_GATES = {None: 0, "silu": 1, "sigmoid": 2}


def head_norm_gate(x: torch.Tensor, gate: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                   out: torch.Tensor, num_heads: int, head_dim: int, gate_kind: Optional[str] = "silu",
                   scale: float = 1.0) -> None:
    """out[t, h] = x[t, h] / rms(x[t, h]) * weight * g(gate[t, h]) * scale for every head of every token:
    the RMS norm over a head's channels (left out when ``weight`` is None) and an output gate (silu or
    sigmoid of ``gate``; left out when ``gate`` is None), float32 arithmetic, rounded once.
    x [T, H D] float32 or the compute type; gate and out in the compute type; rows of all three may be strided."""
    T = x.shape[0]
    H, D = num_heads, head_dim
    _need(gate_kind in _GATES, f"head_norm_gate: unknown gate {gate_kind!r}")
    for t, name in ((x, "x"), (out, "out")) + (((gate, "gate"),) if gate is not None else ()):
        _rows(t, f"head_norm_gate: {name}")
        _need(t.shape == (T, H * D), f"head_norm_gate: {name} must be [T, H D]")
    _need(x.dtype in (torch.float32, out.dtype), "head_norm_gate: x must be float32 or out's dtype")
    if gate is not None:
        _need(gate.dtype == out.dtype, "head_norm_gate: gate must have out's dtype")
    if weight is not None:
        _need(weight.dtype == torch.float32 and weight.shape == (D,) and weight.is_contiguous(), "head_norm_gate: weight must be float32 [D]")
    _check(lib().qe_head_norm_gate(
        _ptr(x), ctypes.c_long(x.stride(0)), int(x.dtype == torch.float32), _ptr(gate),
        ctypes.c_long(gate.stride(0) if gate is not None else 0), _ptr(weight), ctypes.c_float(eps), _ptr(out),
        ctypes.c_long(out.stride(0)), ctypes.c_float(scale), _GATES[gate_kind if gate is not None else None], T, H, D, _dt(out),
        _stream()), "head_norm_gate")


def latent_prepare(down: torch.Tensor, q: torch.Tensor, norm_w: torch.Tensor, eps: float, positions: torch.Tensor,
                   inv_freq: torch.Tensor, rot_dims: int, cache: torch.Tensor, slot_mapping: torch.Tensor,
                   qlat: torch.Tensor, num_heads: int, plain_dim: int, latent_dim: int, rot_dim: int,
                   write_kv: bool = True) -> None:
    """What latent attention does per token before the attention kernel.  ``down`` [T, R + Dr] (rows may be strided): the
    first R channels are RMS-normed (weight ``norm_w``) into the token's cache row, the last Dr are the key part all
    heads share, whose first ``rot_dims`` channels turn (pairs (i, i + rot_dims / 2), angle position x inv_freq[i]) on
    their way into the cache row's tail.  ``q`` [T, H (dn + Dr)]: every head's last Dr channels turn likewise into
    ``qlat`` [T, H, R + Dr] behind the room for the head's folded plain part.  cache [pages, 1, 1, page, R + Dr]."""
    _rows(down, "latent_prepare: down")
    _rows(q, "latent_prepare: q")
    T = q.shape[0]
    H, dn, R, Dr = num_heads, plain_dim, latent_dim, rot_dim
    _need(down.shape == (T, R + Dr) and q.shape == (T, H * (dn + Dr)) and down.dtype == q.dtype == qlat.dtype == cache.dtype,
          "latent_prepare: down [T, R + Dr], q [T, H (dn + Dr)] in the cache's dtype")
    _need(qlat.shape == (T, H * (R + Dr)) and qlat.is_contiguous(), "latent_prepare: qlat must be [T, H (R + Dr)]")
    _need(cache.dim() == 5 and cache.shape[1] == 1 and cache.shape[2] == 1 and cache.shape[4] == R + Dr and cache.is_contiguous(),
          "latent_prepare: cache must be [pages, 1, 1, page, R + Dr]")
    _need(norm_w.dtype == torch.float32 and norm_w.shape == (R,) and inv_freq.dtype == torch.float32
          and inv_freq.numel() >= rot_dims // 2, "latent_prepare: float32 norm weight [R] and inv_freq [rot_dims / 2]")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    _check(lib().qe_latent_prepare(_ptr(down), ctypes.c_long(down.stride(0)), _ptr(q), ctypes.c_long(q.stride(0)), _ptr(norm_w),
                                   ctypes.c_float(eps), _ptr(positions), _ptr(inv_freq), int(rot_dims), _ptr(cache),
                                   _ptr(slot_mapping), _ptr(qlat), T, H, dn, R, Dr, int(bool(write_kv)), _dt(q), _stream()),
           "latent_prepare")


def head_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_head_stride: int, out_head_stride: int) -> None:
    """out[t, h * out_head_stride + n] = sum_k w[h, n, k] x[t, h * x_head_stride + k]: one matrix per head, w [H, N, K];
    x and out are rows (unit stride along columns) in w's dtype, float32 accumulation."""
    _rows(x, "head_linear: x")
    _rows(out, "head_linear: out")
    H, N, K = w.shape
    M = x.shape[0]
    _need(w.is_contiguous() and x.dtype == w.dtype == out.dtype and out.shape[0] == M, "head_linear: operands of one dtype, w contiguous")
    _need((H - 1) * x_head_stride + K <= x.shape[1] and (H - 1) * out_head_stride + N <= out.shape[1],
          "head_linear: the heads do not fit the rows")
    _check(lib().qe_head_linear(_ptr(x), ctypes.c_long(x.stride(0)), ctypes.c_long(x_head_stride), _ptr(w), _ptr(out),
                                ctypes.c_long(out.stride(0)), ctypes.c_long(out_head_stride), M, H, N, K, _dt(x), _stream()),
           "head_linear")


def short_conv(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, ctx, out: torch.Tensor, write_state: bool = True,
               silu: bool = True) -> None:
    """A short causal convolution over the tokens of each request, channel by channel, then silu:
    out[t, c] = silu(sum_j w[c, j] x[t - (taps - 1) + j, c]).  x [T, C] in the compute type (rows may be strided);
    w float32 [C, taps], tap taps - 1 multiplies the token itself; state float32 [slots, taps - 1, C] holds each
    request's last taps - 1 inputs (zeros count for a request without context) and is moved on; out float32 [T, C]."""
    _rows(x, "short_conv: x")
    T, C = x.shape
    taps = w.shape[1]
    _need(w.shape == (C, taps) and w.dtype == torch.float32 and w.is_contiguous(), "short_conv: w must be float32 [C, taps]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, C),
          "short_conv: state must be float32 [slots, taps - 1, C]")
    _need(out.shape == (T, C) and out.dtype == torch.float32 and out.is_contiguous(), "short_conv: out must be float32 [T, C]")
    _check(lib().qe_short_conv(_ptr(x), ctypes.c_long(x.stride(0)), _ptr(w), _ptr(state), _ptr(ctx.cu_q), _ptr(ctx.ctx_lens),
                               _ptr(ctx.slot_ids), _ptr(out), int(ctx.num_reqs), int(ctx.max_q_len), C, taps,
                               int(bool(write_state)), int(bool(silu)), _dt(x), _stream()), "short_conv")


def unit_norm(x: torch.Tensor, num_heads: int, head_dim: int, eps: float, scale: float = 1.0) -> None:
    """x[t, h] <- x[t, h] / sqrt(sum x[t, h]^2 + eps) * scale in place; x float32 [T, H D] (rows may be strided)."""
    _rows(x, "unit_norm: x")
    _need(x.dtype == torch.float32 and x.shape[1] == num_heads * head_dim, "unit_norm: x must be float32 [T, H D]")
    _check(lib().qe_unit_norm(_ptr(x), ctypes.c_long(x.stride(0)), int(x.shape[0]), num_heads, head_dim, ctypes.c_float(eps),
                              ctypes.c_float(scale), _stream()), "unit_norm")


def delta_rule_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: Optional[torch.Tensor], beta: Optional[torch.Tensor],
                    state: torch.Tensor, ctx, out: torch.Tensor, num_heads: int, num_key_heads: int, key_dim: int,
                    value_dim: int, write_state: bool = True, head_decay=None) -> None:
    """The gated delta rule per head over the step's tokens of every request, from the state its slot holds:
    S <- diag(g_t) S; u = sigmoid(beta_t) (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.
    q, k float32 [T, G dk] (head h reads group h // (H / G)), v float32 [T, H dv], g float32 [T, H dk] (None: no
    decay per channel), beta [T, H] before its sigmoid in the compute type (rows may be strided), state float32
    [slots, H, dv, dk], out float32 [T, H dv].  Rows of q, k, v and g may be strided.
    ``head_decay`` = (a, log_rate, bias) in the place of ``g``: one decay per token and head that the scan forms
    itself in float32, exp(-exp(log_rate[h]) softplus(a[t, h] + bias[h])), a [T, H] in the compute type (rows may
    be strided), log_rate and bias float32 [H]."""
    H, G, dk, dv = num_heads, num_key_heads, key_dim, value_dim
    T = q.shape[0]
    for t, name, width in ((q, "q", G * dk), (k, "k", G * dk), (v, "v", H * dv)) + (((g, "g", H * dk),) if g is not None else ()):
        _rows(t, f"delta_rule_scan: {name}")
        _need(t.shape == (T, width) and t.dtype == torch.float32, f"delta_rule_scan: {name} must be float32 [T, {width}]")
    _rows(beta, "delta_rule_scan: beta")
    _need(beta.shape == (T, H), "delta_rule_scan: beta must be [T, H]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dv, dk),
          "delta_rule_scan: state must be float32 [slots, H, dv, dk]")
    _need(out.shape == (T, H * dv) and out.dtype == torch.float32 and out.is_contiguous(), "delta_rule_scan: out must be float32 [T, H dv]")
    da = rate = dbias = None
    if head_decay is not None:
        da, rate, dbias = head_decay
        _need(g is None, "delta_rule_scan: a decay per channel or one per head, not both")
        _rows(da, "delta_rule_scan: the head decay's input")
        _need(da.shape == (T, H) and da.dtype == beta.dtype, "delta_rule_scan: the head decay's input must be [T, H] in beta's type")
        for t_, name in ((rate, "log_rate"), (dbias, "bias")):
            _need(t_.dtype == torch.float32 and t_.shape == (H,) and t_.is_contiguous(), f"delta_rule_scan: the head decay's {name} must be float32 [H]")
    _check(lib().qe_delta_rule_scan(_ptr(q), ctypes.c_long(q.stride(0)), _ptr(k), ctypes.c_long(k.stride(0)), _ptr(v),
                                    ctypes.c_long(v.stride(0)), _ptr(g), ctypes.c_long(g.stride(0) if g is not None else 0),
                                    _ptr(beta), ctypes.c_long(beta.stride(0)), _dt(beta),
                                    ctypes.c_void_p(0), _ptr(state), _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), _ptr(ctx.slot_ids),
                                    _ptr(out), int(ctx.num_reqs), H, G, dk, dv, int(bool(write_state)), 1,
                                    _ptr(da), ctypes.c_long(da.stride(0) if da is not None else 0), _ptr(rate), _ptr(dbias),
                                    _stream()),
           "delta_rule_scan")


ROUTER_SCORINGS = {"softmax_chosen": 0, "softmax_all": 1, "sigmoid": 2}


def moe_route(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], top_idx: torch.Tensor, top_w: torch.Tensor,
              scoring: str = "softmax_chosen", correction: Optional[torch.Tensor] = None) -> None:
    """Router of routed experts: z = w x[t] + bias in float32 (x in the compute type, w float32 [E, W]).
    ``softmax_chosen``: the ``top`` largest logits' experts into top_idx int32 [T, top] (the lower index wins a tie)
    and the softmax over those logits alone into top_w float32 [T, top].
    ``softmax_all``: s = softmax(z) over all E outputs; the ``top`` largest of s + correction (float32 [E], optional)
    are chosen, and their weights are their s as it is (not made to sum to one).
    ``sigmoid``: every output is scored alone, s = sigmoid(z); the ``top`` largest are chosen and their weights are their s."""
    T, W = x.shape
    E = w.shape[0]
    top = top_idx.shape[1]
    _need(scoring in ROUTER_SCORINGS, f"moe_route: unknown scoring {scoring!r}; known: {sorted(ROUTER_SCORINGS)}")
    _need(x.is_contiguous() and w.dtype == torch.float32 and w.shape == (E, W) and w.is_contiguous(), "moe_route: w must be float32 [E, W]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (E,)), "moe_route: bias must be float32 [E]")
    _need(correction is None or (correction.dtype == torch.float32 and correction.shape == (E,) and correction.is_contiguous()
                                 and scoring == "softmax_all"), "moe_route: correction must be float32 [E], with softmax_all")
    _need(top_idx.shape == (T, top) and top_idx.dtype == torch.int32 and top_idx.is_contiguous()
          and top_w.shape == (T, top) and top_w.dtype == torch.float32 and top_w.is_contiguous(), "moe_route: outputs [T, top]")
    _check(lib().qe_moe_route(_ptr(x), _ptr(w), _ptr(bias), _ptr(top_idx), _ptr(top_w), T, W, E, top, _dt(x),
                              ROUTER_SCORINGS[scoring], _ptr(correction), _stream()), "moe_route")


def moe_experts(x: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                out: torch.Tensor, activation, alloc, num_identity: int = 0, weight_inputs: bool = False) -> None:
    """out[t] = sum_j top_w[t, j] * W_down[e] glu(W_gate[e] x[t], W_up[e] x[t]) with e = top_idx[t, j]: the pairs are
    ordered by expert on the device, each expert's rows run as tiles of two grouped products, and the token's choices
    are summed in their order.  w_gate_up [E, 2 I, K] (gate rows, then up rows), w_down [E, N, I]; ``alloc(shape,
    dtype)`` gives scratch memory.  Nothing of the launches depends on the routing.
    ``num_identity``: top_idx may also name E .. E + num_identity - 1, experts without weights whose output is
    x[t] itself (N = K then); their pairs are ordered behind the others and only the weighted sum looks at them.
    ``weight_inputs``: the weight multiplies what the expert reads, not what it returns: out[t] = sum_j expert_e(top_w[t, j]
    x[t]).  The first products are linear, so the weight meets their float32 sums ahead of the activation."""
    T, K = x.shape
    E, I2, _ = w_gate_up.shape
    I, N, top = I2 // 2, w_down.shape[1], top_idx.shape[1]
    P = T * top
    _need(x.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and w_gate_up.shape == (E, 2 * I, K)
          and w_down.shape == (E, N, I) and x.dtype == w_gate_up.dtype == w_down.dtype, "moe_experts: w_gate_up [E, 2 I, K], w_down [E, N, I] in x's dtype")
    _need(out.shape == (T, N) and out.is_contiguous(), "moe_experts: out must be [T, N]")
    _need(num_identity >= 0 and (num_identity == 0 or N == K), "moe_experts: identity experts need outputs of the input's width")
    _need(not (weight_inputs and num_identity), "moe_experts: weighted inputs and identity experts do not go together")
    offsets = alloc((E + num_identity + 1,), torch.int32)
    sorted_pair = alloc((P,), torch.int32)
    place = alloc((P,), torch.int32)
    _check(lib().qe_moe_sort(_ptr(top_idx), _ptr(offsets), _ptr(sorted_pair), _ptr(place), P, E + num_identity, _stream()), "moe_sort")
    act = alloc((P, I), x.dtype)
    _check(lib().qe_moe_gate_up(_ptr(x), _ptr(w_gate_up), _ptr(offsets), _ptr(sorted_pair), _ptr(act), P, E, I, K, top,
                                gate_code(activation), _dt(x), _ptr(top_w if weight_inputs else None), _stream()), "moe_gate_up")
    # a few rows (decoded tokens): the down product cuts K into shares so that enough CTAs pull the weights; the shares' sums
    # are added, in their order, where the token's choices are
    shares = int(lib().qe_moe_down_shares(P, I, _dt(x)))
    y = alloc((shares, P, N), torch.float32)
    _check(lib().qe_moe_down(_ptr(act), _ptr(w_down), _ptr(offsets), _ptr(y), P, E, N, I, shares, _dt(x), _stream()), "moe_down")
    _check(lib().qe_moe_combine(_ptr(y), _ptr(place), _ptr(None if weight_inputs else top_w), _ptr(out), T, N, top, shares, _dt(out),
                                _ptr(top_idx if num_identity else None), E, _ptr(x if num_identity else None), _dt(x), _stream()),
           "moe_combine")


def scaled_add(acc: torch.Tensor, x: torch.Tensor, scale: float, first: bool = False) -> None:
    """acc = (0 if first else acc) + scale * x, element by element in float32; acc and x of one shape, each float32
    or the compute type."""
    _need(acc.shape == x.shape and acc.is_contiguous() and x.is_contiguous(), "scaled_add: two contiguous tensors of one shape")
    _check(lib().qe_scaled_add(_ptr(acc), _dt(acc), _ptr(x), _dt(x), ctypes.c_float(scale), int(bool(first)),
                               ctypes.c_long(acc.numel()), _stream()), "scaled_add")


def qk_bias_norm_kv_write(proj: torch.Tensor, positions: torch.Tensor, q_bias: Optional[torch.Tensor],
                          k_bias: Optional[torch.Tensor], eps: float, q_temp, kv_pages: Optional[torch.Tensor],
                          slot_mapping: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                          write_kv: bool = True) -> None:
    """Attention whose values are its keys as projected: on the leading (Hq + Hkv) D columns of the stacked projection
    output ``proj`` (rows may be strided), in place and in float32: the biases are added (float32 [Hq D], [Hkv D];
    optional); the keys as they then are go to the value plane of ``kv_pages`` [pages, 2, Hkv, page, D]; q and k are
    divided by their root mean square over a head (no weight); q is multiplied by the temperature of its position p,
    1 + coef ln(floor((p + 1) / every) + 1) for ``q_temp`` = (coef, every) (None: none); the normed keys go to the key
    plane."""
    T = proj.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    _rows(proj, "qk_bias_norm_kv_write: proj")
    _need(proj.shape[1] >= (Hq + Hkv) * D, "qk_bias_norm_kv_write: proj must hold q and k side by side")
    _i32(positions, "positions")
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None, "qk_bias_norm_kv_write: cache write without a cache")
        _need(kv_pages.dtype == proj.dtype and kv_pages.is_contiguous() and kv_pages.dim() == 5
              and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == D,
              "qk_bias_norm_kv_write: kv_pages must be [pages, 2, Hkv, page, D] in proj's dtype")
        _i32(slot_mapping, "slot_mapping")
        page_size = kv_pages.shape[3]
    for b, n in ((q_bias, Hq * D), (k_bias, Hkv * D)):
        _need(b is None or (b.dtype == torch.float32 and b.shape == (n,) and b.is_contiguous()),
              "qk_bias_norm_kv_write: biases must be float32 [heads D]")
    coef, every = (0.0, 0) if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
    _need(q_temp is None or every >= 1, "qk_bias_norm_kv_write: the temperature's step must be positive")
    _check(lib().qe_qk_bias_norm_kv_write(_ptr(proj), ctypes.c_long(proj.stride(0)), _ptr(positions), _ptr(q_bias), _ptr(k_bias),
                                          ctypes.c_float(eps), ctypes.c_float(coef), every,
                                          _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None),
                                          T, Hq, Hkv, D, page_size, int(bool(write_kv)), _dt(proj), _stream()),
           "qk_bias_norm_kv_write")


def stream_conv(resid: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], ctx, out_plain: Optional[torch.Tensor],
                out_conv: torch.Tensor, write_state: bool = True) -> None:
    """What a sublayer reads of the float32 residual stream ``resid`` [T, W]: out_plain = resid and out_conv = resid +
    conv(resid), both rounded once to the compute type, conv a causal convolution over the tokens of each request on
    each channel, conv(x)[t, c] = sum_j w[c, j] x[t - (taps - 1) + j, c] with w float32 [W, taps].  state float32
    [slots, taps - 1, W] holds each request's last taps - 1 rows (zeros count for a request without context) and is
    moved on; None where taps = 1."""
    T, W = resid.shape
    taps = w.shape[1]
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "stream_conv: resid must be contiguous float32")
    _need(w.shape == (W, taps) and w.dtype == torch.float32 and w.is_contiguous(), "stream_conv: w must be float32 [W, taps]")
    if taps > 1:
        _need(state is not None and state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, W),
              "stream_conv: state must be float32 [slots, taps - 1, W]")
    for o in (out_plain, out_conv):
        _need(o is None or (o.shape == (T, W) and o.is_contiguous() and o.dtype == out_conv.dtype), "stream_conv: outputs must be contiguous [T, W]")
    _check(lib().qe_stream_conv(_ptr(resid), _ptr(w), _ptr(state if taps > 1 else None), _ptr(ctx.cu_q), _ptr(ctx.ctx_lens),
                                _ptr(ctx.slot_ids), _ptr(out_plain), _ptr(out_conv), int(ctx.num_reqs), int(ctx.max_q_len), W,
                                taps, int(bool(write_state)), _dt(out_conv), _stream()), "stream_conv")


def gated_norm_add(src: torch.Tensor, branch: torch.Tensor, gate: Optional[torch.Tensor], gate_bias: Optional[torch.Tensor],
                   weight: torch.Tensor, eps: float, dst: torch.Tensor, dst_cast: Optional[torch.Tensor] = None,
                   depth_mix=None) -> None:
    """A sublayer's way back into the float32 stream with the norm on the sublayer's side:
    dst[t] = src[t] + rmsnorm(branch[t] * sigmoid(gate[t] + gate_bias)) * weight, float32 arithmetic; ``gate`` None:
    no gate.  src, dst float32 [T, W] (may be the same tensor); branch and gate [T, W] in float32 or the compute
    type; gate_bias, weight float32 [W]; ``dst_cast`` [T, W]: dst once more, rounded to its type.
    ``depth_mix`` = (history, weights, count, mixed): dst is entry count - 1 of history (float32 [L, T, W]), and the
    kernel also leaves mixed = sum over j < count of weights[j] * history[j] (as ``depth_mix`` alone would)."""
    T, W = src.shape
    _need(src.dtype == torch.float32 and dst.dtype == torch.float32 and src.is_contiguous() and dst.is_contiguous()
          and dst.shape == (T, W), "gated_norm_add: src and dst must be contiguous float32 [T, W]")
    _need(branch.shape == (T, W) and branch.is_contiguous(), "gated_norm_add: branch must be contiguous [T, W]")
    _need(weight.dtype == torch.float32 and weight.shape == (W,), "gated_norm_add: weight must be float32 [W]")
    if gate is not None:
        _need(gate.shape == (T, W) and gate.is_contiguous(), "gated_norm_add: gate must be contiguous [T, W]")
        _need(gate_bias is None or (gate_bias.dtype == torch.float32 and gate_bias.shape == (W,)), "gated_norm_add: gate_bias must be float32 [W]")
    if dst_cast is not None:
        _need(dst_cast.shape == (T, W) and dst_cast.is_contiguous(), "gated_norm_add: dst_cast must be contiguous [T, W]")
    history = mix_w = mixed = None
    count = 0
    if depth_mix is not None:
        history, mix_w, count, mixed = depth_mix
        _need(history.dim() == 3 and history.dtype == torch.float32 and history.is_contiguous() and tuple(history.shape[1:]) == (T, W)
              and 1 <= count <= history.shape[0] and dst.data_ptr() == history[count - 1].data_ptr(),
              "gated_norm_add: dst must be the last of the entries of history [L, T, W] that the sum runs over")
        _need(mix_w.dtype == torch.float32 and mix_w.numel() >= count and mix_w.is_contiguous(), "gated_norm_add: the sum's weights must be float32 [count]")
        _need(mixed.shape == (T, W) and mixed.dtype == torch.float32 and mixed.is_contiguous(), "gated_norm_add: mixed must be float32 [T, W]")
    _check(lib().qe_gated_norm_add(_ptr(src), _ptr(branch), _dt(branch), _ptr(gate), _dt(gate) if gate is not None else 0,
                                   _ptr(gate_bias if gate is not None else None), _ptr(weight), ctypes.c_float(eps), _ptr(dst),
                                   _ptr(dst_cast), _dt(dst_cast) if dst_cast is not None else 0, T, W,
                                   _ptr(history), _ptr(mix_w), int(count), _ptr(mixed), _stream()), "gated_norm_add")


def token_side_gate(gate: torch.Tensor, table: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(gate[t, j]) * table[token_ids[t], j]: a second embedding's row, gated; float32 arithmetic,
    rounded once.  gate, out [T, d] and table [V, d] in the compute type."""
    T, d = gate.shape
    _i32(token_ids, "token_ids")
    _need(table.dim() == 2 and table.shape[1] == d and table.is_contiguous() and table.dtype == gate.dtype,
          "token_side_gate: table must be contiguous [V, d] in gate's dtype")
    _need(gate.is_contiguous() and out.shape == (T, d) and out.is_contiguous() and out.dtype == gate.dtype,
          "token_side_gate: gate and out must be contiguous [T, d]")
    _check(lib().qe_token_side_gate(_ptr(gate), _ptr(table), _ptr(token_ids), _ptr(out), T, d, int(table.shape[0]), _dt(gate),
                                    _stream()), "token_side_gate")


def depth_mix(history: torch.Tensor, weights: torch.Tensor, count: int, out: torch.Tensor) -> None:
    """out = sum over j < count of weights[j] * history[j]: a weighted sum of the results of the layers so far.
    history float32 [L, T, W] contiguous, weights float32 [>= count] on the device, out float32 [T, W]; the sum runs in
    the order of j."""
    _need(history.dim() == 3 and history.dtype == torch.float32 and history.is_contiguous() and 1 <= count <= history.shape[0],
          "depth_mix: history must be contiguous float32 [L, T, W] with count <= L")
    _need(weights.dtype == torch.float32 and weights.numel() >= count and weights.is_contiguous(), "depth_mix: weights must be float32 [count]")
    _need(out.shape == history.shape[1:] and out.dtype == torch.float32 and out.is_contiguous(), "depth_mix: out must be float32 [T, W]")
    _check(lib().qe_depth_mix(_ptr(history), _ptr(weights), int(count), _ptr(out), ctypes.c_long(out.numel()), _stream()), "depth_mix")


def group_rmsnorm(x: torch.Tensor, rows: Optional[torch.Tensor], weight: torch.Tensor, eps: float, groups: int,
                  out: torch.Tensor) -> None:
    """RMS norm in groups: every one of ``groups`` equal consecutive parts of a row is divided by its own
    sqrt(mean(part^2) + eps), and the whole row is multiplied by ``weight`` (float32 [W]).  out[n] is the norm of row
    rows[n] of x (of row n without ``rows``); x float32 or the compute type, out float32 or the compute type."""
    N, W = out.shape
    _need(x.dim() == 2 and x.shape[1] == W and x.is_contiguous() and out.is_contiguous(), "group_rmsnorm: x and out must be contiguous rows of one width")
    _need(weight.dtype == torch.float32 and weight.shape == (W,) and weight.is_contiguous(), "group_rmsnorm: weight must be float32 [W]")
    _need(groups >= 1 and W % groups == 0, f"group_rmsnorm: {W} channels do not split into {groups} equal parts")
    if rows is not None:
        _i32(rows, "rows")
        _need(rows.numel() >= N, "group_rmsnorm: fewer rows than outputs")
    else:
        _need(x.shape[0] == N, "group_rmsnorm: x and out must have as many rows")
    _check(lib().qe_group_rmsnorm(_ptr(x), _dt(x), _ptr(rows), _ptr(weight), ctypes.c_float(eps), int(groups), _ptr(out), _dt(out),
                                  N, W, _stream()), "group_rmsnorm")


def group_norm_add(src: torch.Tensor, branch: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, dst: torch.Tensor,
                   next_weight: Optional[torch.Tensor] = None, next_out: Optional[torch.Tensor] = None) -> None:
    """A sublayer's way back into the float32 stream where its result is normed in groups (see ``group_rmsnorm``):
    dst[t] = src[t] + norm(branch[t]) * weight; src and dst float32 [T, W] (may be the same), branch float32 or the
    compute type.  ``next_out`` [T, W] (float32 or the compute type) also gets norm(dst[t]) * next_weight in the same
    pass: what the sublayer after this one reads."""
    T, W = src.shape
    _need(src.dtype == torch.float32 and dst.dtype == torch.float32 and src.is_contiguous() and dst.is_contiguous()
          and dst.shape == (T, W), "group_norm_add: src and dst must be contiguous float32 [T, W]")
    _need(branch.shape == (T, W) and branch.is_contiguous(), "group_norm_add: branch must be contiguous [T, W]")
    _need(groups >= 1 and W % groups == 0, f"group_norm_add: {W} channels do not split into {groups} equal parts")
    for wt in (weight, next_weight):
        _need(wt is None or (wt.dtype == torch.float32 and wt.shape == (W,) and wt.is_contiguous()), "group_norm_add: weights must be float32 [W]")
    if next_out is not None:
        _need(next_weight is not None and next_out.shape == (T, W) and next_out.is_contiguous(), "group_norm_add: next_out must be contiguous [T, W], with its weights")
    _check(lib().qe_group_norm_add(_ptr(src), _ptr(branch), _dt(branch), _ptr(weight), ctypes.c_float(eps), int(groups), _ptr(dst),
                                   _ptr(next_weight if next_out is not None else None), _ptr(next_out),
                                   _dt(next_out) if next_out is not None else 0, T, W, _stream()), "group_norm_add")


def head_mix_gate(partial: torch.Tensor, mix: Optional[torch.Tensor], gate: Optional[torch.Tensor], out: torch.Tensor,
                  num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Attention's heads on their way to the output projection, where a design mixes the heads' attention weights by a
    matrix ``mix`` (float32 [H, H]) and gates every head by one number.  ``partial`` [S, T, H D]: entry s holds, for
    every head g, its weights over the values of kv head (c(g) + s) mod Hkv (``paged_attention`` with ``value_shift``
    s); S = Hkv with ``mix``, else 1.  out[t, h] = sigmoid(gate[t, h]) * sum_g mix[h, g] partial[(c(h) - c(g)) mod Hkv,
    t, g]; ``gate`` [T, H] in the compute type (rows may be strided), None: no gate; ``mix`` None: partial[0] as it is."""
    S, T = partial.shape[0], partial.shape[1]
    H, Hkv, D = num_heads, num_kv_heads, head_dim
    _need(partial.shape == (S, T, H * D) and partial.is_contiguous() and partial.dtype == out.dtype, "head_mix_gate: partial must be contiguous [S, T, H D] in out's dtype")
    _need(S == (Hkv if mix is not None else 1), "head_mix_gate: one set of outputs per kv head with a mixing matrix, else one")
    _need(mix is None or (mix.dtype == torch.float32 and mix.shape == (H, H) and mix.is_contiguous()), "head_mix_gate: mix must be float32 [H, H]")
    _rows(out, "head_mix_gate: out")
    _need(out.shape == (T, H * D), "head_mix_gate: out must be [T, H D]")
    if gate is not None:
        _rows(gate, "head_mix_gate: gate")
        _need(gate.shape == (T, H) and gate.dtype == out.dtype, "head_mix_gate: gate must be [T, H] in out's dtype")
    _check(lib().qe_head_mix_gate(_ptr(partial), ctypes.c_long(T * H * D), S, _ptr(mix), _ptr(gate),
                                  ctypes.c_long(gate.stride(0) if gate is not None else 0), _ptr(out), ctypes.c_long(out.stride(0)),
                                  T, H, Hkv, D, _dt(out), _stream()), "head_mix_gate")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[n] = index of the largest logit of row n (the lowest index on a tie)."""
    N, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "argmax: logits must be contiguous float32")
    _i32(out, "out")
    _check(lib().qe_argmax(_ptr(logits), _ptr(out), N, V, _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor) -> None:
    """Row n: temperature 0 -> argmax; else inverse-CDF sampling of softmax(top-k logits / temperature)
    with the uniform number uniform[n] in [0, 1)."""
    N, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and uniform.dtype == torch.float32, "sample: temperature and uniform must be float32")
    _i32(top_k, "top_k")
    _i32(out, "out")
    _check(lib().qe_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(uniform), _ptr(out), N, V, _stream()), "sample")

"""Python bindings of the CUDA kernels.  Every op here launches this package's own
sm_100a code through ctypes (matrix products of the bfloat16 path may go to cuBLAS, as
they do in tinyserve: serve.py:828-829).  There is no CPU path and no fallback: tensors
must live on a CUDA device and a missing compiler or library raises."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import build

#: gated feed-forwards: act(gate) * up.  "bounded_swish" takes a bound: with g' = min(g, bound) and
#: u' = clamp(u, -bound, bound) it is g' sigmoid(1.702 g') (u' + 1)
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "bounded_swish": 2}
BOUNDED_ACTIVATIONS = ("bounded_swish",)


def activation_code(activation, limit=0.0):
    """(kernel code, bound) of a gated activation; a bounded one needs a positive bound."""
    if activation not in ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}; known: {sorted(ACTIVATIONS)}")
    if activation in BOUNDED_ACTIVATIONS and not limit > 0:
        raise ValueError(f"activation {activation!r} needs a positive bound")
    return ACTIVATIONS[activation], float(limit or 0.0)
SUPPORTED_HEAD_DIMS = tuple(range(16, 513, 16))
_DTYPE = {torch.float32: 0, torch.bfloat16: 1}

_launches = 0
#: bfloat16 matrix products of up to this many rows run on this package's TMA + tcgen05 kernel,
#: larger ones go to cuBLAS (measured on B200 at Qwen3-8B shapes, whole decode steps: 32 tokens
#: +8 %, 48 +4 %, 64 +2 % over cuBLAS)
TCGEN05_MAX_TOKENS = 64
#: bfloat16 attention is chosen by head size: the tcgen05 prefill kernel for these head sizes, the
#: mma.sync kernels (prefill of other head sizes, every decode) up to MMA_MAX_HEAD_DIM, the 32-bit
#: kernel above that
TCGEN05_HEAD_DIMS = (64, 128)
MMA_MAX_HEAD_DIM = 256
MMA_PREFILL_ROWS = 64           # query rows of a block of the mma prefill kernel (4 warps of 16)
#: heads wider than this run the mma prefill kernel with 8 warps (128 rows a block): a block of such
#: heads holds one key tile pair per SM anyway, and twice the rows share its loads and hide its waits
MMA_WIDE_HEAD = 128


def mma_prefill_rows(head_dim: int) -> int:
    return 2 * MMA_PREFILL_ROWS if head_dim > MMA_WIDE_HEAD else MMA_PREFILL_ROWS


def _mma_defines(head_dim: int) -> dict:
    defines = {"TS_HEAD_DIM": head_dim}
    if head_dim > MMA_WIDE_HEAD:
        defines["TS_PREFILL_WARPS"] = 8
    return defines
#: the key ranges of a split-KV decode are the blocks of a thread-block cluster and merge through
#: distributed shared memory when there are at most this many; more are merged by a second kernel
#: (measured on B200 from CUDA graphs, 8 requests x 640 keys: 14.4 us with the second launch,
#: less in the cluster)
CLUSTER_MERGE_MAX_SPLITS = 8
#: the SM count all split heuristics were measured at; the device's own count is used at run time
MEASURED_NUM_SMS = 148
_num_sms = None


def num_sms() -> int:
    """Multiprocessors of the current device (148 where no device is visible)."""
    global _num_sms
    if _num_sms is None:
        if torch.cuda.is_available():
            _num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        else:
            return MEASURED_NUM_SMS
    return _num_sms


# ----------------------------------------------------------------------------- device status
# Kernels never trap: a bounded wait that ran out, or (in a bounds-checking build) an index outside
# its buffer, stores a code into a few words of pinned host memory; see common.cuh.
STATUS_WORDS = 8
_BOUNDS_CODES = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
                 3: "a page number outside the pool", 4: "a position outside the tables",
                 5: "a row outside the batch", 6: "a state slot outside the pool",
                 7: "a request index outside the batch"}
_status = None


def status_words():
    """The int32 status words (a numpy view): pinned host memory that every loaded library writes."""
    global _status
    if _status is None:
        t = torch.zeros(STATUS_WORDS, dtype=torch.int32)
        if torch.cuda.is_available():
            t = t.pin_memory()
        _status = (t, t.numpy())
    return _status[1]


def _register_status(lib):
    if hasattr(lib, "ts_set_status_words") and torch.cuda.is_available():
        status_words()
        if lib.ts_set_status_words(c_void_p(_status[0].data_ptr())) != 0:
            raise RuntimeError("a kernel library did not take the status words")


build.on_load.append(_register_status)


class DeviceError(RuntimeError):
    """A kernel reported that it gave up (a wait ran out) or met an index out of range."""


def raise_on_device_error() -> None:
    """Raise if any kernel has stored a status code since the process started.  Reads host memory
    only; call it after a synchronisation that covers the kernels in question.  The codes stay: an
    engine that has seen one does not go on."""
    w = status_words()
    if w[0]:
        raise DeviceError("a kernel gave up on a bounded wait (mbarrier): its results are not valid; "
                          "the engine stops")
    if w[1]:
        raise DeviceError(f"a kernel met {_BOUNDS_CODES.get(int(w[1]), 'an index out of range')}; "
                          "the access was skipped and the engine stops")


class SplitPartials:
    """The result of a matrix product as split-K partial tiles: the product's kernel stopped
    before adding them up, because the next kernel (residual add + norm, or the q/k norm + rotary
    kernel) adds them while it loads, which is cheaper than reducing inside the product.
    ``materialize()`` adds them up into an ordinary [M, N] tensor for any other consumer."""

    def __init__(self, data, splits, M, N, tile_t, dtype):
        self.data, self.splits, self.M, self.N, self.tile_t, self.dtype = data, splits, M, N, tile_t, dtype
        self.n_tiles, self.t_tiles = -(-N // 128), -(-M // tile_t)
        self.shape = (M, N)
        self.device = data.device

    def args(self):
        return (_ptr(self.data), c_int(self.splits), c_int(self.n_tiles), c_int(self.t_tiles),
                c_int(self.tile_t))

    def materialize(self):
        out = torch.empty(self.M, self.N, dtype=self.dtype, device=self.device)
        lib = _elementwise()
        _check(lib, lib.ts_reduce_partials(c_int(_DTYPE[self.dtype]), *self.args(), _ptr(out),
                                           c_int(self.M), c_int(self.N), _stream()))
        return out


_NO_PARTIALS = (c_void_p(0), c_int(0), c_int(0), c_int(0), c_int(0))

#: up to this many tokens the product before a residual add + norm does the add itself
#: (PendingProduct, ScaledRows), the gate/up product applies the activation in its epilogue and the
#: decode attention kernel takes the q/k/v projection as it is
FUSED_MAX_TOKENS = 16
FUSED_MAX_SPLITS = 8


class PendingProduct:
    """x @ weight^T that has not been launched yet.  ``linear(..., allow_pending=True)`` returns it
    for a few tokens, because the residual add + norm that usually follows can run in the
    product's own kernel: ``add_rmsnorm`` then launches the residual form of the tcgen05 kernel
    (the K cuts of a row tile are a thread-block cluster; they add their partial sums through
    distributed shared memory, add the residual and leave a ScaledRows).  For many tokens
    (``wide``) the paired kernel has the same form.  Any other consumer calls ``partials()`` or
    ``materialize()`` and gets the ordinary product."""

    def __init__(self, x, weight, wide=False):
        self.x, self.weight, self.wide = x, weight, wide         # wide: many tokens, the paired kernel
        self.shape = (x.shape[0], weight.shape[0])
        self.dtype, self.device = x.dtype, x.device

    def splits(self):
        M, K = self.x.shape
        return min(gemm_splits(M, self.weight.shape[0], K, partials=True), FUSED_MAX_SPLITS)

    def partials(self):
        if not self.wide and self.splits() > 1:
            return _linear_tcgen05(self.x, self.weight, False, partials_only=True)
        return self.materialize()

    def materialize(self):
        if self.wide:
            return _linear_pair(self.x, self.weight)
        return _linear_tcgen05(self.x, self.weight, False)


class ScaledRows:
    """Rows that still lack their RMSNorm factor: ``data`` [M, N] holds residual * norm_weight in
    bfloat16 and ``sumsq`` [tiles, 16] the sums of residual^2 over each 128 columns.  ``linear``
    takes it as x and scales every token's result by rsqrt(sum / N + eps) in its epilogue, which
    is the same product as with normalised rows; ``materialize()`` gives the normalised rows."""

    def __init__(self, data, sumsq, tiles, eps):
        self.data, self.sumsq, self.tiles, self.eps = data, sumsq, tiles, eps
        self.shape, self.dtype, self.device = tuple(data.shape), data.dtype, data.device

    @property
    def stride(self):
        """Tokens a tile's sums are apart: 16 from the product for few tokens, more from the paired one."""
        return self.sumsq.shape[1]

    def args(self):
        return (_ptr(self.sumsq), c_int(self.tiles), c_float(self.eps))

    def args_wide(self):
        return (_ptr(self.sumsq), c_int(self.tiles), c_int(self.stride), c_float(self.eps))

    def materialize(self):
        out = torch.empty_like(self.data)
        lib = _elementwise()
        _check(lib, lib.ts_scale_rows(_ptr(self.data), *self.args_wide(), _ptr(out), c_int(self.shape[0]),
                                      c_int(self.shape[1]), _stream()))
        return out


_NO_SCALE = (c_void_p(0), c_int(0), c_float(0.0))


def materialize(x):
    """An ordinary tensor from what a product, a norm or a block returned."""
    return x.materialize() if isinstance(x, (SplitPartials, PendingProduct, ScaledRows, PairSum, NormedAddend, ColumnScaled)) else x


def launch_count() -> int:
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def require_device(device) -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("tinyserve_b200 runs on a CUDA device only (sm_100a); no GPU is visible "
                           "and there is no CPU path")
    if torch.device(device).type != "cuda":
        raise RuntimeError(f"tinyserve_b200 runs on CUDA devices only, got {device!r}")


_STREAM = None


def _stream():
    if _STREAM is not None:
        return _STREAM
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks the current CUDA stream up once for all ops launched inside the scope (the lookup
    costs more than a kernel launch).  The current stream must not change inside the scope."""

    def __enter__(self):
        global _STREAM
        self._outer = _STREAM
        _STREAM = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _STREAM
        _STREAM = self._outer
        return False


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(lib, code, n=1):
    if code != 0:
        raise RuntimeError(lib.ts_last_error().decode())
    count_launches(n)


def _dt(t):
    try:
        return _DTYPE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; kernels take float32 and bfloat16") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("kernel operands must be CUDA tensors: there is no CPU path")


def _vec_flag(w, like):
    """Norm weights are float32 or of the activations' dtype."""
    if w.dtype == torch.float32:
        return 1
    if w.dtype == torch.bfloat16:
        return 0
    raise TypeError(f"norm weight dtype {w.dtype} is not supported")


# ----------------------------------------------------------------------------- libraries
def _elementwise():
    return build.load_unit("elementwise.cu")


def _gemm():
    return build.load_unit("gemm_simt.cu")


def _gemm_tcgen05():
    return build.load_unit("gemm_tcgen05.cu")


_counters: dict = {}


def _tile_counters(device):
    """Zeroed tile counters of the split-K reduction; the kernel returns them to zero."""
    key = str(device)
    if key not in _counters:
        _counters[key] = torch.zeros(16384, dtype=torch.int32, device=device)
    return _counters[key]


def gemm_splits(M, N, K, partials=False):
    """Cuts along K of the tiled product, so that a product with few 128-row tiles still fills
    the SMs.  When the product reduces its own partial tiles: about 160 blocks, at least four
    64-wide slices per cut, wide token tiles cut at most in two (their partial tiles are large).
    When it hands the partial tiles on (``partials``): all 2 x 148 block slots, at most 8 cuts
    (measured on B200 at 8 tokens: 6144x4096 best at 6, 4096x4096 and 4096x12288 at 8)."""
    tile_t = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = -(-N // 128) * -(-M // tile_t)
    slices = -(-K // 64)
    if tiles >= num_sms():
        return 1
    if partials:
        splits = max(1, min(2 * num_sms() // tiles, slices // 4, 8))
    else:
        splits = max(1, min(-(-160 // tiles), slices // 4, 16))
        if tile_t >= 64:
            splits = min(splits, 2)
    per = -(-slices // splits)
    return -(-slices // per)           # no cut without a slice


def gemm_tcgen05_error() -> int:
    """1 if a block of the tcgen05 kernel ever gave up on a wait (synchronises)."""
    return _gemm_tcgen05().ts_gemm_tcgen05_error()


def _tcgen05_ok(x, weight):
    return (x.shape[0] <= TCGEN05_MAX_TOKENS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and weight.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


#: From this many tokens on the gate/up product runs on the paired tcgen05 kernel with the
#: activation in its epilogue.  Measured inside a whole prefill of Qwen3-8B shapes, warm, against
#: the library product + activation kernel: 2,048 tokens +3 %, 4,096 tokens +4.5 %.  Only for
#: rows of PAIR_GATED_MIN_K elements and more: a tile's epilogue (9 to 14 us beside running MMAs)
#: hides behind a mainloop of 64 slices of K, not behind one of 16 (Qwen3-0.6B shapes: slower).
PAIR_GATED_MIN_TOKENS = 2048
PAIR_GATED_MAX_TOKENS = 6144     # (at 8,192 tokens the library's product is 11 % faster, which is what the activation kernel costs)
PAIR_GATED_MIN_K = 4096
#: From this many tokens on every product of a layer runs on the paired kernel, with the residual
#: add, the norm factor and the activation in the products' epilogues.  Off: inside a whole
#: prefill the other three products are 2 to 8 % slower than the library's with the kernels
#: between them (their tiles do not fill whole waves of SM pairs); tests turn it on.
PAIR_MIN_TOKENS = 10 ** 9


def _pair_ok(x, weight):
    return (x.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def _tile_t(M):
    return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128


def _linear_tcgen05(x, weight, out_float32, splits=None, partials_only=False, scale=None, gated=0, bias=None, limit=0.0):
    """``scale``: the ScaledRows whose ``data`` is ``x``; ``gated``: activation code + 1 of the
    gated epilogue (out [M, N / 2]); ``bias`` [N]: added in the epilogue (not with the others)."""
    M, K = x.shape
    N = weight.shape[0]
    out_cols = N // 2 if gated else N
    out = None if partials_only else torch.empty(
        M, out_cols, dtype=torch.float32 if out_float32 else torch.bfloat16, device=x.device)
    lib = _gemm_tcgen05()
    lib.ts_gemm_tcgen05_scratch.restype = c_longlong
    if splits is None:
        splits = gemm_splits(M, N, K, partials=partials_only)
    if partials_only and splits < 2:
        raise ValueError("partial tiles need at least two splits")
    partials = counters = None
    if splits > 1:
        need = lib.ts_gemm_tcgen05_scratch(c_int(M), c_int(N), c_int(splits))
        partials = torch.empty(need, dtype=torch.float32, device=x.device)
        counters = None if partials_only else _tile_counters(x.device)
    if scale is not None or gated:
        if bias is not None:
            raise ValueError("the scaled-rows and gated products take no bias")
        _check(lib, lib.ts_gemm_tcgen05_fused(
            _ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)),
            c_longlong(weight.stride(0)), c_longlong(out_cols), c_int(1 if out_float32 else 0), c_int(splits),
            _ptr(partials), _ptr(counters), *(scale.args() if scale is not None else _NO_SCALE), None, None,
            c_int(0), None, None, c_int(gated), c_float(limit), None, c_int(0), _stream()))
    else:
        _check(lib, lib.ts_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K),
                                        c_longlong(x.stride(0)), c_longlong(weight.stride(0)), c_longlong(N),
                                        c_int(1 if out_float32 else 0), c_int(splits), _ptr(partials),
                                        _ptr(counters), _ptr(bias),
                                        c_int(_vec_flag(bias, torch.bfloat16) if bias is not None else 0), _stream()))
    if partials_only:
        return SplitPartials(partials, splits, M, N, _tile_t(M), torch.bfloat16)
    return out


def _gemm_pair():
    return build.load_unit("gemm_pair_tcgen05.cu")


def gemm_pair_error() -> int:
    """1 if a block of the paired tcgen05 kernel ever gave up on a wait (synchronises)."""
    return _gemm_pair().ts_gemm_pair_error()


_pair_scratch: dict = {}
_pair_count: list = []


def gemm_pairs() -> int:
    """Pairs of blocks of the paired product that the device holds at once (74 on a B200 with all
    148 SMs in pairs)."""
    if not _pair_count:
        n = _gemm_pair().ts_gemm_pair_max_pairs()
        _pair_count.append(n if n > 0 else num_sms() // 2)
    return _pair_count[0]


def _pair_workspace(lib, M, N, K, pairs, halves, out_float32, device):
    """Where the parts of the cut tiles of the last wave are added up, and their counters: zero
    between products (the kernel leaves them so).  One buffer per device, grown on demand:
    products of one stream run one after the other."""
    counters = c_int(0)
    lib.ts_gemm_pair_scratch.restype = c_longlong
    need = lib.ts_gemm_pair_scratch(c_int(M), c_int(N), c_int(K), c_int(pairs), c_int(halves), c_int(1 if out_float32 else 0), ctypes.byref(counters))
    key = str(device)
    have = _pair_scratch.get(key)
    if have is None or have[0].numel() < need or have[1].numel() < counters.value:
        if torch.cuda.is_current_stream_capturing():
            # (a buffer made during a capture belongs to the graph's pool: it must not outlive it here)
            raise RuntimeError("the paired product's scratch would have to grow inside a graph capture: "
                               "run the shape once before it is captured")
        grow = max(need, have[0].numel() if have else 0, 1)
        have = (torch.zeros(grow, dtype=torch.float32, device=device),
                torch.zeros(max(counters.value, 1024), dtype=torch.int32, device=device))
        _pair_scratch[key] = have
    return have


def _linear_pair(x, weight, out_float32=False, bias=None, scale=None, gated=0, limit=0.0, residual=None, norm_weight=None,
                 pairs=None, halves=0):
    """The product for many tokens on pairs of SMs (csrc/gemm_pair_tcgen05.cu).  Plain: returns
    out [M, N]; ``bias`` [N]; ``scale`` the ScaledRows whose ``data`` is ``x``.  ``gated``:
    activation code + 1, out [M, N / 2].  ``residual`` (float32 [M, N], in place) with
    ``norm_weight``: returns (hprime, sumsq) of the new residual.  ``halves``: tiles of 256 (1) or
    512 (2) weight rows, 0: the kernel's estimate decides."""
    M, K = x.shape
    N = weight.shape[0]
    lib = _gemm_pair()
    pairs = pairs or gemm_pairs()
    scratch, counters = _pair_workspace(lib, M, N, K, pairs, halves, out_float32, x.device)
    out = hprime = sumsq = None
    stride = -(-M // 4) * 4
    if residual is not None:
        hprime = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        sumsq = torch.empty(-(-N // 128), stride, dtype=torch.float32, device=x.device)
    else:
        out = torch.empty(M, N // 2 if gated else N, dtype=torch.float32 if out_float32 else torch.bfloat16,
                          device=x.device)
    _check(lib, lib.ts_gemm_pair(
        _ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)),
        c_longlong(weight.stride(0)), c_longlong(out.stride(0) if out is not None else 0),
        c_int(1 if out_float32 else 0), _ptr(bias),
        c_int(_vec_flag(bias, torch.bfloat16) if bias is not None else 0),
        *(scale.args_wide() if scale is not None else (c_void_p(0), c_int(0), c_int(0), c_float(0.0))),
        c_int(gated), _ptr(residual), _ptr(norm_weight),
        c_int(_vec_flag(norm_weight, torch.bfloat16) if norm_weight is not None else 0), _ptr(hprime), _ptr(sumsq),
        c_int(stride), _ptr(scratch), c_longlong(scratch.numel()), _ptr(counters), c_int(counters.numel()),
        c_int(pairs), c_int(halves), c_float(limit), _stream()))
    if residual is not None:
        return hprime, sumsq
    return out


def _attention(head_dim: int):
    if head_dim not in SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head size {head_dim} is not supported: attention takes multiples of 16 "
                         f"up to {SUPPORTED_HEAD_DIMS[-1]}")
    return build.load_unit("attention_simt.cu", {"TS_HEAD_DIM": head_dim})


def _attention_mma(head_dim: int):
    return build.load_unit("attention_mma.cu", _mma_defines(head_dim))


def _attention_tcgen05(head_dim: int):
    return build.load_unit("attention_tcgen05.cu", {"TS_HEAD_DIM": head_dim})


def attention_tcgen05_error(head_dim: int) -> int:
    """1 if a block of the tcgen05 attention kernel ever gave up on a wait (synchronises)."""
    return _attention_tcgen05(head_dim).ts_attention_tcgen05_error()


def attention_mma_error(head_dim: int) -> int:
    """1 if a block of the TMA decode kernel ever gave up on a wait (synchronises)."""
    return _attention_mma(head_dim).ts_attention_mma_error()


def _sampler():
    return build.load_unit("sampler.cu")


def _latent_moe():
    return build.load_unit("latent_moe.cu")


def _sequence():
    return build.load_unit("sequence.cu")


def units_for(head_dims, key_dims=()) -> list:
    """The (source, defines) units a model with these attention head sizes, and these key sizes of
    its matrix-state mixers, needs."""
    units = [("elementwise.cu", {}), ("gemm_simt.cu", {}), ("gemm_tcgen05.cu", {}), ("gemm_pair_tcgen05.cu", {}),
             ("sampler.cu", {}), ("latent_moe.cu", {}), ("sequence.cu", {})]
    units += [("attention_simt.cu", {"TS_HEAD_DIM": d}) for d in sorted(set(head_dims))]
    units += [("attention_mma.cu", _mma_defines(d)) for d in sorted(set(head_dims))
              if d <= MMA_MAX_HEAD_DIM]
    units += [("attention_tcgen05.cu", {"TS_HEAD_DIM": d}) for d in sorted(set(head_dims))
              if d in TCGEN05_HEAD_DIMS]
    units += [("linear_attention.cu", {"TS_KEY_DIM": d}) for d in sorted(set(key_dims))]
    return units


# ----------------------------------------------------------------------------- ops
def block_tables_step(resident, pairs, num_pairs, step_tables, state_slots, num_requests):
    """Apply a step's block-table changes to the resident rows and gather the rows of the step's
    requests.  resident int32 [G, slots + 1, max_blocks]; pairs int32 [capacity, 2] (flat index
    into resident, page); num_pairs int32 [1]; step_tables int32 [G, max_requests, max_blocks];
    state_slots int32 [>= num_requests]: all on the device.  Two small launches."""
    _cuda(resident, pairs, num_pairs, step_tables, state_slots)
    G, slots1, max_blocks = resident.shape
    lib = _elementwise()
    _check(lib, lib.ts_block_tables_step(
        _ptr(resident), _ptr(pairs), _ptr(num_pairs), c_int(pairs.shape[0]), _ptr(step_tables), _ptr(state_slots),
        c_int(num_requests), c_int(step_tables.shape[1]), c_int(slots1 - 1), c_int(max_blocks), c_int(G), _stream()), 2)


def sanitize_step(ctx, vocab_size, num_positions, max_kv_len, num_state_slots):
    """The device half of the index check (see csrc/elementwise.cu): every index of the step in
    ``ctx`` that lies outside its buffer is replaced by a harmless one and reported through the
    status words.  One small kernel, plus one per cache group."""
    lib = _elementwise()
    _cuda(ctx.token_ids, ctx.positions, ctx.cu_q, ctx.kv_lens, ctx.state_slots)
    _check(lib, lib.ts_sanitize_step(
        _ptr(ctx.token_ids), c_int(ctx.num_tokens), c_int(vocab_size), _ptr(ctx.slot_tokens),
        c_int(num_state_slots), _ptr(ctx.positions), c_int(num_positions), _ptr(ctx.logit_rows),
        c_int(ctx.num_logit_rows), _ptr(ctx.cu_q), _ptr(ctx.kv_lens), c_int(ctx.num_requests), c_int(max_kv_len),
        _ptr(ctx.state_slots), _stream()))
    for view in ctx.groups:
        _check(lib, lib.ts_sanitize_group(
            _ptr(view.slot_mapping), c_int(ctx.num_tokens), c_longlong(view.num_pages * view.page_size),
            _ptr(view.block_table), c_int(ctx.num_requests), c_int(view.max_blocks),
            c_int(view.block_table.stride(0)), c_int(view.num_pages), _stream()))


def embed_lookup(table, ids, slot_tokens=None, scale=1.0):
    """float32 [T, n] = table[ids] * scale; ids int32.  An id < 0 names a state slot (-1 - slot) whose
    last sampled token is read from ``slot_tokens`` on the device."""
    _cuda(table, ids, slot_tokens)
    T, n = ids.shape[0], table.shape[1]
    out = torch.empty(T, n, dtype=torch.float32, device=table.device)
    lib = _elementwise()
    _check(lib, lib.ts_embed_lookup(c_int(_dt(table)), _ptr(table), _ptr(ids), _ptr(out), c_int(T),
                                    c_int(n), c_int(table.shape[0]), _ptr(slot_tokens), c_float(scale), _stream()))
    return out


def _product_add_residual(pending, residual, weight, eps, x_scale=None):
    """The residual form of the tcgen05 product: residual += x w^T (times one factor per column
    with ``x_scale``) inside the product's kernel; returns the ScaledRows of the new residual for
    the norm with ``weight``."""
    x, w = pending.x, pending.weight
    M, K = x.shape
    N = w.shape[0]
    tiles = -(-N // 128)
    if pending.wide:
        hprime, sumsq = _linear_pair(x, w, residual=residual, norm_weight=weight)
        return ScaledRows(hprime, sumsq, tiles, eps)
    hprime = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty(tiles, 16, dtype=torch.float32, device=x.device)
    lib = _gemm_tcgen05()
    _check(lib, lib.ts_gemm_tcgen05_fused(
        _ptr(x), _ptr(w), None, c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)), c_longlong(w.stride(0)),
        c_longlong(N), c_int(0), c_int(pending.splits()), None, None, *_NO_SCALE, _ptr(residual), _ptr(weight),
        c_int(_vec_flag(weight, torch.bfloat16)), _ptr(hprime), _ptr(sumsq), c_int(0), c_float(0.0), _ptr(x_scale),
        c_int(_vec_flag(x_scale, torch.bfloat16) if x_scale is not None else 0), _stream()))
    return ScaledRows(hprime, sumsq, tiles, eps)


def add_rmsnorm(x, residual, weight, eps, out_dtype, rows=None, scaled_ok=False):
    """residual (float32, in place) += x; returns rmsnorm(residual) * weight as ``out_dtype``.
    ``x`` None: no add; ``x`` may be the SplitPartials or the PendingProduct of a product, or a
    ColumnScaled of any of these (x times one factor per column is then what is added).  With
    ``rows`` (int32) only those rows are normalised and returned, and the residual is left as it
    is.  With ``scaled_ok`` the caller takes a ScaledRows as well (it hands it to ``linear``)."""
    x_scale = None
    if isinstance(x, ColumnScaled):
        x, x_scale = x.x, x.scale
        if isinstance(x, PendingProduct):
            if (scaled_ok and rows is None and out_dtype == torch.bfloat16 and not x.wide and x.shape == tuple(residual.shape)
                    and residual.dtype == torch.float32 and residual.is_contiguous()
                    and x_scale.shape == (residual.shape[1],) and x_scale.is_contiguous()):
                _cuda(residual, weight, x_scale)
                return _product_add_residual(x, residual, weight, eps, x_scale)
            x = x.partials()
    if isinstance(x, PendingProduct):
        if (scaled_ok and rows is None and out_dtype == torch.bfloat16 and x.shape == tuple(residual.shape)
                and residual.dtype == torch.float32 and residual.is_contiguous()):
            _cuda(residual, weight)
            return _product_add_residual(x, residual, weight, eps)
        x = x.partials()
    parts = _NO_PARTIALS
    if isinstance(x, SplitPartials):
        if x.shape != tuple(residual.shape):
            raise TypeError("add_rmsnorm: the partial tiles do not have the residual's shape")
        parts, x = x.args(), None
    _cuda(x, residual, weight, rows, x_scale)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream is contiguous float32")
    if x is not None and (x.dtype != out_dtype or not x.is_contiguous() or x.shape != residual.shape):
        raise TypeError("add_rmsnorm: x must be contiguous, of the compute dtype and of the residual's shape")
    if x_scale is not None and (x_scale.shape != (residual.shape[1],) or not x_scale.is_contiguous()):
        raise TypeError("add_rmsnorm: the column factors are one contiguous row of the residual's width")
    n = residual.shape[1]
    num_out = residual.shape[0] if rows is None else rows.shape[0]
    out = torch.empty(num_out, n, dtype=out_dtype, device=residual.device)
    lib = _elementwise()
    _check(lib, lib.ts_add_rmsnorm(c_int(_DTYPE[out_dtype]), _ptr(x), _ptr(residual), _ptr(weight),
                                   c_int(_vec_flag(weight, out_dtype)), c_float(eps), _ptr(out),
                                   _ptr(rows), c_int(num_out), c_int(n),
                                   c_int(0 if rows is not None else 1), *parts, _ptr(x_scale),
                                   c_int(_vec_flag(x_scale, out_dtype) if x_scale is not None else 0), _stream()))
    return out


def rmsnorm(x, weight, eps, out=None):
    _cuda(x, weight)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    out = torch.empty_like(x2) if out is None else out
    lib = _elementwise()
    _check(lib, lib.ts_rmsnorm(c_int(_dt(x2)), _ptr(x2), _ptr(weight), c_int(_vec_flag(weight, x.dtype)),
                               c_float(eps), _ptr(out), c_int(x2.shape[0]), c_int(shape[-1]), _stream()))
    return out.view(shape)


def gated_activation(gate_up, activation="silu", block=0, limit=0.0):
    """[rows, 2 I] -> act(gate) * up, [rows, I].  ``block`` 0: the input is gate | up; else gate
    and up columns alternate in blocks of ``block`` (see gated_linear).  ``limit``: the bound of a
    bounded activation."""
    code, limit = activation_code(activation, limit)
    gate_up = materialize(gate_up)
    _cuda(gate_up)
    rows, two_i = gate_up.shape
    out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    lib = _elementwise()
    _check(lib, lib.ts_gated_activation(c_int(_dt(gate_up)), _ptr(gate_up), _ptr(out), c_int(rows),
                                        c_int(two_i // 2), c_int(code), c_int(block), c_float(limit), _stream()))
    return out


#: rows of gate and up alternate in blocks of this many in a fused gate/up weight: half a 128-row
#: tile of the tcgen05 product
GATED_BLOCK = 64


def gated_linear(x, weight, activation="silu", block=0, limit=0.0):
    """act(gate) * up of x @ weight^T, [M, N / 2].  weight [N, K] holds gate rows then up rows
    (``block`` 0) or alternates them in blocks of ``block`` rows.  With blocks of GATED_BLOCK, up
    to FUSED_MAX_TOKENS tokens and a product that needs no cut along K, the tcgen05 product does
    the activation in its epilogue; otherwise the product is followed by the activation kernel.  x may be the
    ScaledRows that add_rmsnorm returned."""
    rows = x.data if isinstance(x, ScaledRows) else x
    N, K = weight.shape
    code, limit = activation_code(activation, limit)
    if (block == GATED_BLOCK and N % 128 == 0 and isinstance(rows, torch.Tensor)
            and rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _pair_ok(rows, weight)
            and (rows.shape[0] >= PAIR_MIN_TOKENS
                 or (rows is x and PAIR_GATED_MIN_TOKENS <= rows.shape[0] <= PAIR_GATED_MAX_TOKENS
                     and K >= PAIR_GATED_MIN_K))):
        _cuda(rows, weight)
        return _linear_pair(rows, weight, gated=code + 1, limit=limit, scale=x if rows is not x else None)
    if (block == GATED_BLOCK and N % 128 == 0 and isinstance(rows, torch.Tensor)
            and rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _tcgen05_ok(rows, weight)
            and rows.shape[0] <= FUSED_MAX_TOKENS          # measured: at 64 tokens the epilogue costs 9 % of the step
            and gemm_splits(rows.shape[0], N, K) == 1):
        _cuda(rows, weight)
        return _linear_tcgen05(rows, weight, False, splits=1, gated=code + 1, limit=limit,
                               scale=x if rows is not x else None)
    return gated_activation(linear(x, weight), activation, block, limit)


def qk_norm_rope_kvwrite(qkv, positions, num_heads, num_kv_heads, head_dim, rotary=None,
                         q_weight=None, k_weight=None, eps=0.0, k_cache=None, v_cache=None,
                         slot_mapping=None, page_size=0):
    """Per-head norm of q and k, rotary encoding, q to a [T, H, D] tensor (returned), k and v
    to the cache slots of ``slot_mapping`` (None: nothing is written)."""
    parts, dtype = _NO_PARTIALS, qkv.dtype
    if isinstance(qkv, SplitPartials):
        if head_dim % 2:
            qkv = qkv.materialize()
        else:
            parts = qkv.args()
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv must be [T, (H + 2 Hkv) * D]")
    device = qkv.device
    if parts is _NO_PARTIALS:
        if not qkv.is_contiguous():
            raise ValueError("qkv must be contiguous")
    else:
        qkv = None
    _cuda(qkv, positions, k_cache, v_cache, slot_mapping)
    q = torch.empty(T, num_heads, head_dim, dtype=dtype, device=device)
    cos = rotary.cos if rotary is not None else None
    sin = rotary.sin if rotary is not None else None
    rot = rotary.rotary_dim if rotary is not None else 0
    inter = int(rotary.interleaved) if rotary is not None else 0
    if k_cache is not None and k_cache.dtype != dtype:
        raise TypeError("cache and activations differ in dtype")
    flag = _vec_flag(q_weight, dtype) if q_weight is not None else 0
    if q_weight is not None and k_weight.dtype != q_weight.dtype:
        raise TypeError("q and k norm weights differ in dtype")
    lib = _elementwise()
    _check(lib, lib.ts_qk_norm_rope_kvwrite(
        c_int(_DTYPE[dtype]), _ptr(qkv), _ptr(q), _ptr(positions), _ptr(cos), _ptr(sin), c_int(rot),
        c_int(inter), _ptr(q_weight), _ptr(k_weight), c_int(flag), c_float(eps), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(k_cache), _ptr(v_cache),
        _ptr(slot_mapping), c_int(page_size), *parts, _stream()))
    return q


def attention_splits(num_requests, max_q_len, max_kv_len, num_heads, num_kv_heads):
    """How many key ranges a launch is cut into so that a small batch still fills the SMs
    (tinykernels.py:865-889, for 148 SMs)."""
    group = num_heads // num_kv_heads
    per_tile = 32 // group if group < 32 else 1
    blocks = -(-max_q_len // per_tile) * num_kv_heads * -(-group // 32) * num_requests
    if blocks >= 2 * num_sms() or max_kv_len < 256:
        return 1
    want = -(-2 * num_sms() // blocks)
    return max(1, min(want, max_kv_len // 128, 32))


class AttentionWork:
    """The work lists of a step's attention launches, built once per step on the host."""
    __slots__ = ("tile_req", "tile_q0", "num_tiles", "dec_req", "dec_tok", "num_decode", "max_decode_kv")


def cut_attention_work(cu, kv, num_requests, queries_per_tile, split_decodes=True):
    """The host half: (tile_req, tile_q0, dec_req, dec_tok, longest decode context) as lists.
    Requests with several tokens are cut into blocks of ``queries_per_tile`` queries, (request,
    first query) each, heaviest (most keys) first, so that a long portion beside many short
    requests launches no block for nothing.  With ``split_decodes``, requests of one token are
    listed apart, (request, token) each, longest context first: they go to the decode kernel,
    which does not spend a block of rows on one query."""
    tiles, decodes = [], []
    for b in range(num_requests):
        n = cu[b + 1] - cu[b]
        if n == 1 and split_decodes:
            decodes.append((kv[b], b, cu[b]))
            continue
        for q0 in range(0, n, queries_per_tile):
            tiles.append((kv[b] - n + q0, b, q0))
    tiles.sort(reverse=True)
    decodes.sort(reverse=True)
    return ([t[1] for t in tiles], [t[2] for t in tiles], [d[1] for d in decodes], [d[2] for d in decodes],
            decodes[0][0] if decodes else 0)


def attention_work(ctx, queries_per_tile, device, split_decodes=True):
    """A step's attention work lists (int32 device tensors) for blocks of ``queries_per_tile``
    queries.  The engine's step function packs them with the rest of the step (one upload) for
    the tile sizes its mixers announce; for any other caller they are cut and uploaded here."""
    cache = getattr(ctx, "tile_cache", None)
    key = (queries_per_tile, split_decodes)
    if cache is not None and key in cache:
        return cache[key]
    host = getattr(ctx, "host", None) or {}
    cu = host.get("cu_q") or ctx.cu_q.tolist()
    kv = host.get("kv_lens") or ctx.kv_lens.tolist()
    tile_req, tile_q0, dec_req, dec_tok, max_decode_kv = cut_attention_work(
        cu, kv, ctx.num_requests, queries_per_tile, split_decodes)
    work = AttentionWork()
    work.num_tiles, work.num_decode, work.max_decode_kv = len(tile_req), len(dec_req), max_decode_kv
    packed = torch.tensor(tile_req + tile_q0 + dec_req + dec_tok, dtype=torch.int32).to(device)
    nt, nd = work.num_tiles, work.num_decode
    work.tile_req, work.tile_q0 = packed[:nt], packed[nt:2 * nt]
    work.dec_req, work.dec_tok = packed[2 * nt:2 * nt + nd], packed[2 * nt + nd:]
    if cache is not None:
        cache[key] = work
    return work


def timeline_read(reset=True):
    """The records of a TINYSERVE_TIMELINE=1 build, from every loaded library, as a numpy structured
    array sorted by time: ns, sm, tag (0 block started, 1 its wait for the predecessor returned,
    2 and 3 marks of the kernel itself), grid and block indices, threads per block."""
    import numpy as np
    dtype = np.dtype([("ns", "<u8"), ("sm", "<i4"), ("tag", "<i4"), ("grid", "<i4", 3), ("block", "<i4", 3),
                      ("threads", "<i4"), ("pad", "<i4")])
    chunks = []
    for lib in build.loaded_units():
        if not hasattr(lib, "ts_timeline_read"):
            continue
        buf = np.zeros(1 << 17, dtype=dtype)
        n = lib.ts_timeline_read(ctypes.c_void_p(buf.ctypes.data), c_int(len(buf)), c_int(1 if reset else 0))
        if n < 0:
            raise RuntimeError("reading the kernel timeline failed")
        chunks.append(buf[:n])
    if not chunks:
        raise RuntimeError("no loaded library records a timeline: set TINYSERVE_TIMELINE=1 before the first kernel is built")
    out = np.concatenate(chunks)
    return out[np.argsort(out["ns"], kind="stable")]


def _tma_pages(k_cache, v_cache):
    """The page count that lets the decode kernel fetch whole pages by TMA, or 0 where the caches
    are not plain [pages, kv heads, page, head] blocks of memory."""
    return k_cache.shape[0] if k_cache.is_contiguous() and v_cache.is_contiguous() else 0


def decode_splits(num_requests, max_kv_len, num_heads, num_kv_heads):
    """Key ranges for the tensor-core decode kernel: as many as fit in one wave of blocks (two
    per SM), with at least two tiles of 64 keys per range."""
    blocks = num_kv_heads * -(-(num_heads // num_kv_heads) // 16) * num_requests
    return max(1, min(2 * num_sms() // blocks, max_kv_len // 128, 32))


def _decode_listed(q, out, k_cache, v_cache, view, ctx, scale, window, work, keep_first=0, sinks=None, chunk=0,
                   slopes=None, softcap=0.0):
    """The one-token requests of a mixed batch, by the tensor-core decode kernel."""
    T, H, D = q.shape
    Hkv = k_cache.shape[1]
    n = work.num_decode
    num_splits = decode_splits(n, work.max_decode_kv, H, Hkv)
    part_o = part_ml = None
    cluster = 1 < num_splits <= CLUSTER_MERGE_MAX_SPLITS
    if num_splits > 1 and not cluster:
        part_o = torch.empty(n * H * num_splits * D, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n * H * num_splits * 2, dtype=torch.float32, device=q.device)
    lib = _attention_mma(D)
    _check(lib, lib.ts_paged_attention_mma(
        _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
        _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(1), c_int(H), c_int(Hkv),
        c_int(view.page_size), c_int(view.block_table.stride(0)), c_float(scale), c_int(window),
        c_int(num_splits), _ptr(part_o), _ptr(part_ml), c_int(2 if cluster else 1), _ptr(work.dec_req),
        _ptr(work.dec_tok), c_int(n), c_int(0), c_int(_tma_pages(k_cache, v_cache)), c_int(keep_first), _ptr(sinks),
        c_int(chunk), _ptr(slopes), c_float(softcap), c_int(Hkv // v_cache.shape[1]), _stream()),
        2 if num_splits > 1 and not cluster else 1)


def attention_backend(dtype, head_dim, page_size=16) -> str:
    """Which kernels attend for this element type and head size: "tcgen05" (prefill on the
    tcgen05 kernel, decode on the mma.sync decode kernel), "mma" (both on the mma.sync kernels) or
    "simt" (the 32-bit kernel: float32, and bfloat16 heads wider than MMA_MAX_HEAD_DIM)."""
    if dtype != torch.bfloat16 or head_dim > MMA_MAX_HEAD_DIM or head_dim not in SUPPORTED_HEAD_DIMS:
        return "simt"
    if head_dim in TCGEN05_HEAD_DIMS and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0:
        return "tcgen05"
    return "mma"


def prefill_tile_queries(dtype, num_heads, num_kv_heads, head_dim, page_size=16) -> int:
    """Queries per block of the prefill kernel that ``attention_backend`` names (0: the kernel
    takes no work list)."""
    group = num_heads // num_kv_heads
    backend = attention_backend(dtype, head_dim, page_size)
    if backend == "tcgen05":
        return 2 * (128 // group if group < 128 else 1)      # two query tiles of 128 rows a block
    if backend == "mma":
        rows = mma_prefill_rows(head_dim)
        return rows // group if group < rows else 1
    return 0


def biased_attention_backends(dtype, head_dim, page_size) -> list:
    """The attention kernels that take a chunk mask and a distance bias at this element type and head
    size (all that take the plain case do), the one the engine picks first."""
    first = attention_backend(dtype, head_dim, page_size)
    return [first] + [b for b in ("mma", "simt") if b != first and (first != "simt")]


def paged_attention(q, k_cache, v_cache, view, ctx, scale, window=0, num_splits=None, backend=None, keep_first=0,
                    sinks=None, chunk=0, slopes=None, softcap=0.0):
    """Attention of this step's queries over their requests' cached keys and values.
    ``chunk`` > 0: a query at position i sees key j <= i only if i // chunk == j // chunk (chunks
    count from position 0 of the sequence; no window beside it).  ``slopes`` float32 [H]: head h's
    score of (i, j) loses slopes[h] * (i - j) after the scale.
    ``keep_first`` (with a window): the first keys of a sequence stay visible to every later query.
    ``sinks`` float32 [H]: head h's softmax sum holds one more term exp(sinks[h]) without key or value.
    ``softcap`` c > 0: the scaled score s becomes c tanh(s / c) (before the slopes' bias).
    A value cache of fewer heads than the key cache (Hkv / s): key head i reads value head i / s.
    q [T, H, D]; caches [pages, Hkv, page_size, D]; ``view`` a GroupView; ``ctx`` gives cu_q,
    kv_lens and the batch's maxima.  bfloat16 runs on the tensor cores (a decode kernel when
    every request brings one token, else a prefill kernel); float32 on the 32-bit kernel.
    ``backend`` overrides ``attention_backend`` (tests run the slower kernels at every size)."""
    _cuda(q, k_cache, v_cache)
    T, H, D = q.shape
    Hkv = k_cache.shape[1]
    if Hkv % v_cache.shape[1]:
        raise ValueError(f"paged_attention: {Hkv} key heads on {v_cache.shape[1]} value heads")
    v_share = Hkv // v_cache.shape[1]          # key head i reads value head i / v_share
    page = view.page_size
    chosen = attention_backend(q.dtype, D, page)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.shape != (H,) or not sinks.is_cuda):
        raise TypeError("paged_attention: sinks are float32 [heads] on the device")
    keep_first = int(keep_first) if window > 0 else 0
    chunk = int(chunk or 0)
    softcap = float(softcap or 0.0)
    if softcap < 0:
        raise ValueError("paged_attention: a soft cap is positive (0: none)")
    if chunk < 0 or (chunk and window > 0):
        raise ValueError("paged_attention: a chunk is positive and comes without a window")
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.shape != (H,) or not slopes.is_cuda):
        raise TypeError("paged_attention: slopes are float32 [heads] on the device")
    if backend is not None and backend != chosen:
        if q.dtype != torch.bfloat16 or (backend == "tcgen05") or (backend == "mma" and chosen == "simt"):
            raise ValueError(f"attention backend {backend!r} does not take {q.dtype}, head size {D}, pages of {page}")
        chosen = backend
    if chosen == "tcgen05" and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        chosen = "mma"
    mma = chosen in ("tcgen05", "mma")
    decode = mma and ctx.max_q_len == 1
    if chosen == "tcgen05" and not decode:
        out = torch.empty_like(q)
        lib = _attention_tcgen05(D)
        tile_queries = prefill_tile_queries(q.dtype, H, Hkv, D, page)
        work = attention_work(ctx, tile_queries, q.device)
        if work.num_decode:
            _decode_listed(q, out, k_cache, v_cache, view, ctx, scale, window, work, keep_first, sinks, chunk, slopes, softcap)
        if work.num_tiles:
            _check(lib, lib.ts_paged_attention_tcgen05(
                _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
                _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(ctx.max_q_len), c_int(H), c_int(Hkv),
                c_int(k_cache.shape[0]), c_int(page), c_int(view.block_table.stride(0)), c_float(scale),
                c_int(window), _ptr(work.tile_req), _ptr(work.tile_q0), c_int(work.num_tiles),
                c_int(tile_queries), c_int(keep_first), _ptr(sinks), c_int(chunk), _ptr(slopes), c_float(softcap),
                c_int(v_share), _stream()))
        return out
    if num_splits is None:
        if decode:
            num_splits = decode_splits(ctx.num_requests, ctx.max_kv_len, H, Hkv)
        elif mma:
            num_splits = 1
        else:
            num_splits = attention_splits(ctx.num_requests, ctx.max_q_len, ctx.max_kv_len, H, Hkv)
    if mma and not decode:
        num_splits = 1
    out = torch.empty_like(q)
    part_o = part_ml = None
    cluster = mma and decode and 1 < num_splits <= CLUSTER_MERGE_MAX_SPLITS
    if num_splits > 1 and not cluster:
        part_o = torch.empty(T * H * num_splits * D, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(T * H * num_splits * 2, dtype=torch.float32, device=q.device)
    launches = 2 if num_splits > 1 and not cluster else 1
    if mma:
        lib = _attention_mma(D)
        tile_req = tile_q0 = None
        num_tiles = tile_queries = 0
        if not decode:
            group = H // Hkv
            rows = mma_prefill_rows(D)
            tile_queries = rows // group if group < rows else 1
            work = attention_work(ctx, tile_queries, q.device)
            if work.num_decode:
                _decode_listed(q, out, k_cache, v_cache, view, ctx, scale, window, work, keep_first, sinks, chunk, slopes, softcap)
            if not work.num_tiles:
                return out
            tile_req, tile_q0, num_tiles = work.tile_req, work.tile_q0, work.num_tiles
        _check(lib, lib.ts_paged_attention_mma(
            _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
            _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(ctx.max_q_len), c_int(H),
            c_int(Hkv), c_int(view.page_size), c_int(view.block_table.stride(0)), c_float(scale),
            c_int(window), c_int(num_splits), _ptr(part_o), _ptr(part_ml),
            c_int((2 if cluster else 1) if decode else 0), _ptr(tile_req), _ptr(tile_q0), c_int(num_tiles), c_int(tile_queries),
            c_int(_tma_pages(k_cache, v_cache)), c_int(keep_first), _ptr(sinks), c_int(chunk), _ptr(slopes),
            c_float(softcap), c_int(v_share), _stream()),
            launches)
        return out
    lib = _attention(D)
    _check(lib, lib.ts_paged_attention_biased(
        c_int(_dt(q)), _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table),
        _ptr(ctx.cu_q), _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(ctx.max_q_len),
        c_int(H), c_int(Hkv), c_int(view.page_size), c_int(view.block_table.stride(0)),
        c_float(scale), c_int(window), c_int(num_splits), _ptr(part_o), _ptr(part_ml), c_int(keep_first),
        _ptr(sinks), c_int(chunk), _ptr(slopes), c_float(softcap), c_int(v_share), _stream()),
        launches)
    return out


def attention_from_qkv(qkv, positions, num_heads, num_kv_heads, head_dim, rotary, q_weight, k_weight, eps,
                       k_cache, v_cache, view, ctx, scale, window=0, write_cache=True, fused=True):
    """Per-head norm of q and k, rotary encoding, cache write of k and v, attention over the cache:
    qkv [T, (H + 2 Hkv) * D] (a tensor, or the SplitPartials of the projection) -> [T, H, D].
    Two kernels (qk_norm_rope_kvwrite, paged_attention), or, when every request brings one token
    (bfloat16, full-width rotary with the (j, j + D/2) pairing), the decode kernel alone: it makes
    its query rows and the newest key and value itself (one kernel fewer per layer; ``fused``
    False keeps the two kernels, for comparison)."""
    dtype = qkv.dtype
    H, Hkv, D = num_heads, num_kv_heads, head_dim
    plain = isinstance(qkv, torch.Tensor)
    # (up to FUSED_MAX_TOKENS requests: measured, at 64 the separate kernel is 4 % of the step faster)
    fused = (fused and write_cache and dtype == torch.bfloat16 and ctx.max_q_len == 1
             and qkv.shape[0] <= FUSED_MAX_TOKENS
             and D in SUPPORTED_HEAD_DIMS and D <= MMA_MAX_HEAD_DIM
             and rotary is not None and rotary.rotary_dim == D and not rotary.interleaved
             and (q_weight is None) == (k_weight is None)
             and k_cache is not None and k_cache.dtype == torch.bfloat16
             and (isinstance(qkv, SplitPartials) or (plain and qkv.is_contiguous()))
             and (q_weight is None or q_weight.dtype == k_weight.dtype))
    if not fused:
        q = qk_norm_rope_kvwrite(qkv, positions, H, Hkv, D, rotary=rotary, q_weight=q_weight, k_weight=k_weight,
                                 eps=eps, k_cache=k_cache, v_cache=v_cache,
                                 slot_mapping=view.slot_mapping if write_cache else None, page_size=view.page_size)
        return paged_attention(q, k_cache, v_cache, view, ctx, scale, window)
    T = qkv.shape[0]
    if qkv.shape[1] != (H + 2 * Hkv) * D:
        raise ValueError("qkv must be [T, (H + 2 Hkv) * D]")
    parts = _NO_PARTIALS if plain else qkv.args()
    _cuda(qkv if plain else None, positions, k_cache, v_cache, view.slot_mapping, view.block_table, rotary.cos, rotary.sin)
    out = torch.empty(T, H, D, dtype=dtype, device=qkv.device)
    num_splits = decode_splits(ctx.num_requests, ctx.max_kv_len, H, Hkv)
    cluster = 1 < num_splits <= CLUSTER_MERGE_MAX_SPLITS
    part_o = part_ml = None
    if num_splits > 1 and not cluster:
        part_o = torch.empty(T * H * num_splits * D, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(T * H * num_splits * 2, dtype=torch.float32, device=qkv.device)
    lib = _attention_mma(D)
    _check(lib, lib.ts_paged_attention_mma_from_qkv(
        _ptr(qkv) if plain else None, *parts, _ptr(positions), _ptr(view.slot_mapping), _ptr(rotary.cos),
        _ptr(rotary.sin), _ptr(q_weight), _ptr(k_weight), c_int(_vec_flag(q_weight, dtype) if q_weight is not None else 0),
        c_float(eps), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
        _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(H), c_int(Hkv), c_int(view.page_size),
        c_int(view.block_table.stride(0)), c_float(scale), c_int(window), c_int(num_splits), _ptr(part_o),
        _ptr(part_ml), c_int(2 if cluster else 1), c_int(_tma_pages(k_cache, v_cache)), _stream()),
        2 if num_splits > 1 and not cluster else 1)
    return out


def linear(x, weight, bias=None, out_float32=False, allow_partials=False, allow_pending=False):
    """x [M, K] @ weight[N, K]^T (+ bias).  float32 operands: this package's 32-bit FMA kernel
    (no tensor cores, no reduced precision).  bfloat16 operands: this package's TMA + tcgen05
    kernel for up to TCGEN05_MAX_TOKENS rows (K and the leading dimensions multiples of 8), cuBLAS
    through torch above that, as in tinyserve (serve.py:828-829).  With ``allow_partials`` the
    result may be a SplitPartials (the caller hands it to add_rmsnorm, qk_norm_rope_kvwrite, or
    calls materialize); with ``allow_pending`` a PendingProduct (for add_rmsnorm, or materialize).
    x may be the ScaledRows that add_rmsnorm returned."""
    scale = None
    if isinstance(x, ScaledRows):
        scale, x = x, x.data
    _cuda(x, weight, bias)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or x.dtype != weight.dtype:
        raise ValueError(f"linear: x {tuple(x.shape)} {x.dtype} does not fit weight {tuple(weight.shape)} {weight.dtype}")
    if bias is not None and tuple(bias.shape) != (N,):
        raise ValueError(f"linear: bias {tuple(bias.shape)} does not fit {N} outputs")
    x = materialize(x)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M >= PAIR_MIN_TOKENS and _pair_ok(x, weight):
        if allow_pending and scale is None and bias is None and not out_float32:
            return PendingProduct(x, weight, wide=True)
        return _linear_pair(x, weight, out_float32, bias=bias, scale=scale)
    if x.dtype == torch.bfloat16 and _tcgen05_ok(x, weight) and (scale is None or M <= FUSED_MAX_TOKENS):
        if bias is not None:
            if scale is not None:
                x, scale = scale.materialize(), None
            return _linear_tcgen05(x, weight, out_float32, bias=bias)
        if allow_pending and scale is None and not out_float32 and M <= FUSED_MAX_TOKENS:
            return PendingProduct(x, weight)
        if (allow_partials or allow_pending) and not out_float32 \
                and gemm_splits(x.shape[0], weight.shape[0], x.shape[1], partials=True) > 1:
            return _linear_tcgen05(x, weight, False, partials_only=True, scale=scale)
        return _linear_tcgen05(x, weight, out_float32, scale=scale)
    if scale is not None:
        x = scale.materialize()
    if x.dtype == torch.bfloat16:
        # a plain library product (and its bias epilogue), as in tinyserve
        if bias is not None and out_float32:
            # the sum stays 32-bit: the library's product, then this package's add of the bias
            return add_row_vector_(torch.mm(x, weight.t(), out_dtype=torch.float32), bias)
        if bias is not None:
            return torch.addmm(bias.to(torch.bfloat16), x, weight.t())
        if out_float32:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return torch.mm(x, weight.t())
    return _linear_simt(x, weight, bias, out_float32)


def _linear_simt(x, weight, bias=None, out_float32=False):
    """The 32-bit FMA product (float32 operands; it takes bfloat16 operands too)."""
    M, K = x.shape
    N = weight.shape[0]
    out_dtype = torch.float32 if out_float32 else x.dtype
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise ValueError("linear: operands must be contiguous along K")
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    lib = _gemm()
    _check(lib, lib.ts_gemm_simt(c_int(_dt(x)), c_int(_DTYPE[out_dtype]), _ptr(x), _ptr(weight),
                                 _ptr(bias), _ptr(out), c_int(M), c_int(N), c_int(K),
                                 c_longlong(x.stride(0)), c_longlong(weight.stride(0)),
                                 c_longlong(N), _stream()))
    return out


def sample(logits, temperature, stream_ids, steps, seed, top_k=None, top_p=None, slot_tokens=None,
           slots=None):
    """One token per row of float32 logits.  temperature float32 [B] (0 = argmax); stream_ids
    int64 [B] and steps int32 [B] select the noise; top_k int32 [B], top_p float32 [B] optional.
    With ``slot_tokens`` (int32 [slots]) and ``slots`` (int32 [B]) row i's token is also stored
    at slot_tokens[slots[i]], for the next step's embedding lookup."""
    _cuda(logits, temperature, stream_ids, steps, top_k, top_p, slot_tokens, slots)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise TypeError("sample: logits must be float32 rows")
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    lib = _sampler()
    _check(lib, lib.ts_sample(_ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V),
                              _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(stream_ids),
                              _ptr(steps), c_ulonglong(seed & (2 ** 64 - 1)), _ptr(out),
                              _ptr(slot_tokens), _ptr(slots), _stream()))
    return out


def apply_repetition_penalty(logits, rows, ids, penalty):
    """In place: rows int32 [R] of logits; ids int32 [R, n] distinct recent tokens (-1 = none);
    penalty float32 [R]."""
    _cuda(logits, rows, ids, penalty)
    lib = _sampler()
    _check(lib, lib.ts_apply_repetition_penalty(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(logits.shape[1]), _ptr(rows), _ptr(ids),
        c_int(rows.shape[0]), c_int(ids.shape[1]), _ptr(penalty), _stream()))
    return logits


# ----------------------------------------------------------------------------- parallel blocks, layer norm, soft cap
class PairSum:
    """The outputs of two sub-layers that read the same input and are summed into the stream
    (a block that runs its mixer and its feed-forward side by side).  The kernel of the next
    norm, or of the next product on the stream, adds both to the 32-bit residual while it loads,
    so the sum is never rounded to the compute dtype; ``materialize()`` adds them for any other
    consumer.  ``b`` may be None."""

    def __init__(self, a, b=None):
        self.a, self.b = materialize(a), materialize(b)
        self.shape, self.dtype, self.device = tuple(self.a.shape), self.a.dtype, self.a.device

    def materialize(self):
        if self.b is None:
            return self.a
        out = torch.empty_like(self.a)
        lib = _elementwise()
        _check(lib, lib.ts_sum2(c_int(_dt(self.a)), _ptr(self.a), _ptr(self.b), _ptr(out), c_longlong(self.a.numel()),
                                _stream()))
        return out


class ColumnScaled:
    """A sub-layer's output that joins the stream multiplied by one learned factor per column
    (a layer scale): the kernel that adds it to the 32-bit residual multiplies while it loads, in
    32-bit, so the product is never rounded to the compute dtype.  ``x`` is a tensor or an
    unfinished product (SplitPartials, PendingProduct); ``materialize()`` gives the scaled tensor
    to any other consumer."""

    def __init__(self, x, scale):
        if isinstance(x, (PairSum, NormedAddend, ScaledRows, ColumnScaled)):
            x = materialize(x)
        self.x, self.scale = x, scale
        self.shape, self.dtype, self.device = tuple(x.shape), x.dtype, x.device

    def materialize(self):
        rows, n = self.shape
        summed = torch.zeros(rows, n, dtype=torch.float32, device=self.device)
        stream_add_(summed, self)
        return summed if self.dtype == torch.float32 else summed.to(self.dtype)


def stream_add_(residual, pending=None, first=None):
    """residual (float32 [rows, n], in place) += pending + first.  ``pending``: None, a tensor of
    the compute dtype, the unfinished product of one, or a ColumnScaled; ``first``: None or
    float32 rows.  One kernel; every addend enters the sum in 32-bit."""
    x_scale = None
    if isinstance(pending, ColumnScaled):
        pending, x_scale = pending.x, pending.scale
    if isinstance(pending, PendingProduct):
        pending = pending.partials()
    parts = _NO_PARTIALS
    if isinstance(pending, SplitPartials):
        if pending.shape != tuple(residual.shape):
            raise TypeError("stream_add: the partial tiles do not have the residual's shape")
        parts, dtype, pending = pending.args(), pending.dtype, None
    else:
        pending = materialize(pending)
        dtype = pending.dtype if pending is not None else torch.float32
    _cuda(residual, pending, x_scale, first)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream is contiguous float32")
    for t in (pending, first):
        if t is not None and (t.shape != residual.shape or not t.is_contiguous()):
            raise TypeError("stream_add: addends are contiguous and of the residual's shape")
    if first is not None and first.dtype != torch.float32:
        raise TypeError("stream_add: the kept stream is float32")
    rows, n = residual.shape
    lib = _elementwise()
    _check(lib, lib.ts_stream_add(c_int(_DTYPE[dtype]), _ptr(residual), _ptr(pending), _ptr(x_scale),
                                  c_int(_vec_flag(x_scale, dtype) if x_scale is not None else 0), _ptr(first),
                                  c_int(rows), c_int(n), *parts, _stream()))
    return residual


def _addends(x):
    if x is None:
        return None, None
    if isinstance(x, PairSum):
        return x.a, x.b
    return materialize(x), None


def add_layernorm(x, residual, weight, eps, out_dtype, bias=None, rows=None):
    """residual (float32, in place) += x; returns (residual - mean) / sqrt(var + eps) * weight
    (+ bias) as ``out_dtype``, var the mean of the squared deviations.  ``x``: None, a tensor of
    the compute dtype or a PairSum.  With ``rows`` (int32) only those rows are normalised and
    returned, and the residual is left as it is."""
    x1, x2 = _addends(x)
    _cuda(x1, x2, residual, weight, bias, rows)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream is contiguous float32")
    for a in (x1, x2):
        if a is not None and (a.dtype != out_dtype or not a.is_contiguous() or a.shape != residual.shape):
            raise TypeError("add_layernorm: addends are contiguous, of the compute dtype and of the residual's shape")
    n = residual.shape[1]
    num_out = residual.shape[0] if rows is None else rows.shape[0]
    out = torch.empty(num_out, n, dtype=out_dtype, device=residual.device)
    lib = _elementwise()
    _check(lib, lib.ts_add_layernorm(
        c_int(_DTYPE[out_dtype]), _ptr(x1), _ptr(x2), _ptr(residual), _ptr(weight), c_int(_vec_flag(weight, out_dtype)),
        _ptr(bias), c_int(_vec_flag(bias, out_dtype) if bias is not None else 0), c_float(eps), _ptr(out), _ptr(rows),
        c_int(num_out), c_int(n), c_int(0 if rows is not None else 1), _stream()))
    return out


def softcap_(logits, cap):
    """logits (float32, in place) <- cap * tanh(logits / cap)."""
    _cuda(logits)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise TypeError("softcap: logits are contiguous float32")
    lib = _elementwise()
    _check(lib, lib.ts_softcap(_ptr(logits), c_longlong(logits.numel()), c_float(cap), _stream()))
    return logits


def add_row_vector_(x, vec):
    """x (float32 [rows, n], in place) += vec [n]."""
    _cuda(x, vec)
    if x.dtype != torch.float32 or not x.is_contiguous() or vec.shape[-1] != x.shape[1]:
        raise TypeError("add_row_vector: contiguous float32 rows and a vector of their length")
    lib = _elementwise()
    _check(lib, lib.ts_add_row_vector(_ptr(x), _ptr(vec), c_int(_vec_flag(vec, torch.bfloat16)), c_int(x.shape[0]),
                                      c_int(x.shape[1]), _stream()))
    return x


def stream_concat(residual, pending, first, out_dtype):
    """[rows, 2 n] of ``out_dtype``: the stream as it stands (residual plus what is still pending:
    None, a tensor or a PairSum) beside ``first`` (float32 [rows, n])."""
    x1, x2 = _addends(pending)
    _cuda(residual, x1, x2, first)
    rows, n = residual.shape
    out = torch.empty(rows, 2 * n, dtype=out_dtype, device=residual.device)
    lib = _elementwise()
    _check(lib, lib.ts_stream_concat(c_int(_DTYPE[out_dtype]), _ptr(residual), _ptr(x1), _ptr(x2), _ptr(first), _ptr(out),
                                     c_int(rows), c_int(n), _stream()))
    return out


def mean_of_normed(xs, weights, eps):
    """mean over i of xs[i] * rsqrt(mean(xs[i]^2) + eps) * weights[i], row by row ([rows, n] each)."""
    xs = [materialize(x) for x in xs]
    _cuda(*xs, *weights)
    if len({(tuple(x.shape), x.dtype) for x in xs}) != 1 or not all(x.is_contiguous() for x in xs):
        raise TypeError("mean_of_normed: branches are contiguous and alike in shape and dtype")
    if len({w.dtype for w in weights}) != 1:
        raise TypeError("mean_of_normed: the branches' weights differ in dtype")
    rows, n = xs[0].shape
    out = torch.empty_like(xs[0])
    count = len(xs)
    xp = (c_void_p * count)(*[x.data_ptr() for x in xs])
    wp = (c_void_p * count)(*[w.data_ptr() for w in weights])
    lib = _elementwise()
    _check(lib, lib.ts_mean_of_normed(c_int(_dt(xs[0])), c_int(count), xp, wp, c_int(_vec_flag(weights[0], xs[0].dtype)),
                                      c_float(eps), _ptr(out), c_int(rows), c_int(n), _stream()))
    return out


def _columns(t):
    """(pointer, row stride) of a 2-d tensor or a column range of one."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("operand must be a 2-d tensor, contiguous along its rows")
    return _ptr(t), c_longlong(t.stride(0))


def rope_unit_kvwrite(q, k, v, positions, num_heads, num_kv_heads, dim, vdim, stored_dim, rotary=None,
                      unit_norm=False, eps=0.0, k_cache=None, v_cache=None, slot_mapping=None, page_size=0,
                      q_weight=None, k_weight=None, pre_eps=0.0, maps=1):
    """Rotary encoding of q and k (first ``rotary.rotary_dim`` elements of every head), then, with
    ``unit_norm``, division of every head of q and k by its root mean square over ``dim``; q goes
    to a [T, H, stored_dim] tensor (returned), k and v to the cache slots of ``slot_mapping``
    (None: nothing is written), heads padded with zeros to ``stored_dim``.  q [T, H dim],
    k [T, Hkv dim], v [T, Hkv vdim] may be column ranges of one projection.

    ``q_weight`` / ``k_weight`` ([dim] each): every head of q and k is RMS-normed with that weight
    (``pre_eps``) before the rotation.  ``maps`` M > 1: every head has M score maps over the same
    values; ``num_heads`` and ``num_kv_heads`` then count (head, map) pairs, laid out head by head
    in q and k, v holds ``num_kv_heads`` / M heads and so does the value cache, and the returned
    query rows are arranged so that the attention kernels pair map m of a head with map m of its
    key/value head (``paged_attention`` gives key head i the value head i / M; ``map_difference``
    reads the output in that order)."""
    _cuda(q, k, v, positions, k_cache, v_cache, slot_mapping, q_weight, k_weight)
    T = q.shape[0]
    if maps < 1 or num_heads % maps or num_kv_heads % maps:
        raise ValueError("rope_unit_kvwrite: the maps do not divide the heads")
    if q.shape[1] != num_heads * dim or k.shape[1] != num_kv_heads * dim or v.shape[1] != num_kv_heads // maps * vdim:
        raise ValueError("rope_unit_kvwrite: q, k, v do not have heads x size columns")
    if (q_weight is None) != (k_weight is None) or (q_weight is not None and (
            q_weight.dtype != k_weight.dtype or q_weight.shape != (dim,) or k_weight.shape != (dim,))):
        raise TypeError("rope_unit_kvwrite: q and k norm weights come together, [dim] each and alike in dtype")
    if k_cache is not None and (k_cache.dtype != q.dtype or k_cache.shape[-1] != stored_dim or not k_cache.is_contiguous()
                                or not v_cache.is_contiguous() or k_cache.shape[1] != num_kv_heads
                                or v_cache.shape[1] != num_kv_heads // maps):
        raise TypeError("rope_unit_kvwrite: the cache does not fit the activations")
    out = torch.empty(T, num_heads, stored_dim, dtype=q.dtype, device=q.device)
    cos = rotary.cos if rotary is not None else None
    sin = rotary.sin if rotary is not None else None
    lib = _elementwise()
    _check(lib, lib.ts_rope_unit_kvwrite(
        c_int(_dt(q)), *_columns(q), *_columns(k), *_columns(v), _ptr(out), _ptr(positions), _ptr(cos), _ptr(sin),
        c_int(rotary.rotary_dim if rotary is not None else 0), c_int(int(rotary.interleaved) if rotary is not None else 0),
        c_int(1 if unit_norm else 0), c_float(eps), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(dim),
        c_int(vdim), c_int(stored_dim), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), c_int(page_size),
        _ptr(q_weight), _ptr(k_weight), c_int(_vec_flag(q_weight, q.dtype) if q_weight is not None else 0),
        c_float(pre_eps), c_int(maps), _stream()))
    return out


def map_difference(attn, num_heads, num_kv_heads, vdim, factor, eps, post):
    """[T, H * vdim] from attn [T, 2 H, D], the outputs of two score maps per head in the row order
    of ``rope_unit_kvwrite(maps=2)``: d = a_0 - factor * a_1 over the first ``vdim`` columns of a
    head, then d / sqrt(mean(d^2) + eps) * post, in 32-bit."""
    _cuda(attn)
    T, rows, D = attn.shape
    if rows != 2 * num_heads or not attn.is_contiguous() or num_heads % num_kv_heads or vdim > D:
        raise ValueError("map_difference: attn is contiguous [T, 2 heads, D]")
    out = torch.empty(T, num_heads * vdim, dtype=attn.dtype, device=attn.device)
    lib = _elementwise()
    _check(lib, lib.ts_map_difference(c_int(_dt(attn)), _ptr(attn), _ptr(out), c_int(T), c_int(num_heads), c_int(num_kv_heads),
                                      c_int(D), c_int(vdim), c_float(factor), c_float(eps), c_float(post), _stream()))
    return out


def head_gate(attn, gate, vdim):
    """[T, H * vdim] = attn [T, H, D][..., :vdim] * sigmoid(gate [T, H]); ``gate`` None: the
    columns are only gathered."""
    _cuda(attn, gate)
    T, H, D = attn.shape
    if not attn.is_contiguous():
        raise ValueError("head_gate: attn must be contiguous")
    out = torch.empty(T, H * vdim, dtype=attn.dtype, device=attn.device)
    gp, ld = _columns(gate) if gate is not None else (c_void_p(0), c_longlong(0))
    lib = _elementwise()
    _check(lib, lib.ts_head_gate(c_int(_dt(attn)), _ptr(attn), gp, ld, _ptr(out), c_int(T), c_int(H), c_int(D),
                                 c_int(vdim), _stream()))
    return out


# ----------------------------------------------------------------------------- linear attention with a matrix state
LINEAR_ATTENTION_MAX_VALUE_DIM = 4096
#: a step whose longest portion has at least LINEAR_ATTENTION_SEGMENT_MIN tokens cuts its portions
#: into segments that run side by side (three launches instead of one: local states, their
#: combination, outputs); the segments are as long as lets the longest portion's blocks fill the
#: SMs once (as many blocks per SM as fit), a multiple of 16 tokens and at least LINEAR_ATTENTION_SEGMENT
LINEAR_ATTENTION_SEGMENT = 64
LINEAR_ATTENTION_SEGMENT_MIN = 256


def linear_attention_segment(longest: int, blocks_per_segment: int, resident: int = 2) -> int:
    """Tokens per segment for a step whose longest portion has ``longest`` tokens and launches
    ``blocks_per_segment`` blocks (heads x column tiles) per segment, ``resident`` of which an SM
    holds at once; 0: one segment, one launch."""
    if longest < LINEAR_ATTENTION_SEGMENT_MIN:
        return 0
    segments = max(1, resident * num_sms() // max(1, blocks_per_segment))
    length = max(LINEAR_ATTENTION_SEGMENT, -(-longest // segments))
    return -(-length // 16) * 16


def linear_attention_supports(key_dim: int) -> bool:
    """Key sizes the scan is built for: those that 1, 2, 4, ... or 32 row groups cut into at most
    64 rows each."""
    return 0 < key_dim <= 2048 and any(key_dim % g == 0 and key_dim // g <= 64 for g in (1, 2, 4, 8, 16, 32))


def _linear_attention(key_dim: int):
    if not linear_attention_supports(key_dim):
        raise ValueError(f"key size {key_dim} is not supported: linear attention takes key sizes that split into "
                         f"1, 2, 4, ... or 32 groups of at most 64 rows")
    return build.load_unit("linear_attention.cu", {"TS_KEY_DIM": key_dim})


def linear_attention(q, k, v, gate, state, ctx, num_heads, key_dim, value_dim, out_dtype, *, decay=None,
                     decay_logits=None, tau=1.0, rotary=None, q_scale=1.0, k_scale=1.0, norm_weight=None, eps=0.0,
                     segment=None, input_activation=None, gate_activation="silu", joint_norm=False,
                     lower=None, tied_key=False, token_keep=None, token_write=None, qk_group=1, value_width=None,
                     raw=False, step_sizes=None):
    """Per request and head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over this step's
    tokens, from and to ``state`` [slots, H, key_dim, value_dim] (float32) at the requests' state
    slots (``ctx.state_slots``, ``ctx.fresh``, ``ctx.cu_q``); returns [T, H * value_dim] =
    o / rms(o) (* norm_weight) * silu(gate).  a_t: ``decay`` float32 [H] (one constant per head)
    or ``decay_logits`` float32 [T, H * key_dim] with a = sigmoid(z)^(1 / tau).  q, k [T, H key_dim],
    v, gate [T, H value_dim] may be column ranges of one projection.  ``rotary``: positions on q
    and k; ``q_scale`` / ``k_scale``: constant factors (after the rotation).  ``segment``: tokens per
    segment of the side-by-side form (None: chosen by the step's longest portion, 0: never).
    ``input_activation`` "silu": q, k and v pass through silu first.  ``gate_activation`` "sigmoid":
    the output is multiplied by sigmoid(gate).  ``joint_norm``: the output norm runs over all heads
    of a token together, with ``norm_weight`` [H * value_dim].  ``input_activation`` may also name
    the operands that pass through silu, as a string of the letters q, k, v.
    ``lower`` float32 [H * key_dim] (with ``decay_logits``): a = lower + (1 - lower) sigmoid(z); with
    ``tied_key`` k = 1 - a and ``k`` is None.  ``token_keep`` / ``token_write`` float32 [T, H]: the decay of
    (token, head) and a factor on its k, S_t = keep_t S_(t-1) + write_t k_t v_t^T.  ``step_sizes`` (raw, bias,
    rate), raw float32 [T, H] (a column range may be given), bias and rate [H]: the kernel makes both itself,
    dt = softplus(raw + bias), keep = exp(-exp(rate) dt), write = dt.  ``qk_group``: heads
    that share one q and one k (q, k [T, H / qk_group * key_dim]).  ``value_width`` < value_dim: v holds
    that many columns per head, the state's next column is fed ones (so that column of S^T q is
    sum of the k . q terms) and the rest zeros.  ``raw``: returns the 32-bit S^T q [T, H * value_dim]
    without norm and gate, for a finishing kernel of the caller's."""
    acts = {None: 0, "silu": 7}
    if isinstance(input_activation, str) and input_activation != "silu" and set(input_activation) <= set("qkv"):
        acts[input_activation] = sum({"q": 1, "k": 2, "v": 4}[c] for c in set(input_activation))
    if input_activation not in acts or gate_activation not in ("silu", "sigmoid"):
        raise ValueError("linear_attention: input activation None, silu or letters of qkv, gate activation silu or sigmoid")
    _cuda(q, k, v, gate, state, decay, decay_logits, norm_weight, lower, token_keep, token_write)
    T = q.shape[0]
    H = num_heads
    vw = value_dim if value_width is None else int(value_width)
    if H % qk_group or q.shape[1] != H // qk_group * key_dim or (k is not None and k.shape[1] != q.shape[1]) \
            or v.shape[1] != H * vw or (k is None) != bool(tied_key):
        raise ValueError("linear_attention: q, k, v do not have heads x size columns")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (H, key_dim, value_dim) or not state.is_contiguous():
        raise TypeError("linear_attention: the state is contiguous float32 [slots, H, key_dim, value_dim]")
    if (decay is not None) + (decay_logits is not None) + (token_keep is not None) + (step_sizes is not None) != 1:
        raise ValueError("linear_attention: per-head decays, per-channel logits, per-token decays or step sizes")
    step_raw = step_bias = step_rate = None
    if step_sizes is not None:
        step_raw, step_bias, step_rate = step_sizes
        _cuda(step_raw, step_bias, step_rate)
        if step_raw.dtype != torch.float32 or tuple(step_raw.shape) != (T, H) or step_raw.stride(1) != 1:
            raise TypeError("linear_attention: step-size logits are float32 [T, H]")
        if step_bias.dtype != step_rate.dtype or step_bias.numel() != H or step_rate.numel() != H:
            raise TypeError("linear_attention: a step-size bias and a rate per head, of one type")
    if decay_logits is not None and (decay_logits.dtype != torch.float32 or decay_logits.shape[1] != H * key_dim):
        raise TypeError("linear_attention: decay logits are float32 [T, H * key_dim]")
    if lower is not None and (lower.dtype != torch.float32 or lower.numel() != H * key_dim or decay_logits is None):
        raise TypeError("linear_attention: the lower bounds are float32 [H * key_dim] and belong to decay logits")
    for name, t in (("token_keep", token_keep), ("token_write", token_write)):
        if token_keep is not None and (t is None or t.dtype != torch.float32 or tuple(t.shape) != (T, H) or not t.is_contiguous()):
            raise TypeError(f"linear_attention: {name} is contiguous float32 [T, H]")
    if vw != value_dim and not raw:
        raise ValueError("linear_attention: constant value columns come with raw outputs")
    out = None if raw else torch.empty(T, H * value_dim, dtype=out_dtype, device=q.device)
    zp, zld = _columns(decay_logits) if decay_logits is not None else (c_void_p(0), c_longlong(0))
    gp, gld = _columns(gate) if gate is not None else (c_void_p(0), c_longlong(0))
    lib = _linear_attention(key_dim)
    # a head of more value columns than a block takes: its output norm runs as a kernel of its own
    tiles = lib.ts_linear_attention_column_tiles(c_int(value_dim))
    wide = tiles > 1 or bool(joint_norm) or bool(raw)
    if segment is None:
        seg_len = linear_attention_segment(getattr(ctx, "max_q_len", 0), H * tiles,
                                           lib.ts_linear_attention_resident_blocks(c_int(value_dim)))
    else:
        seg_len = int(segment)
    max_segments, seg_state, seg_decay = 0, None, None
    if seg_len:
        max_segments = -(-(getattr(ctx, "max_q_len", 0) or T) // seg_len)
        seg_state = torch.empty(ctx.num_requests * H * max_segments * key_dim * value_dim, dtype=torch.float32, device=q.device)
        if decay is None:
            seg_decay = torch.empty(ctx.num_requests * H * max_segments * key_dim, dtype=torch.float32, device=q.device)
    raw_out = torch.empty(T, H * value_dim, dtype=torch.float32, device=q.device) if wide else None
    kp, kld = _columns(k) if k is not None else (c_void_p(0), c_longlong(0))
    _check(lib, lib.ts_linear_attention(
        c_int(_dt(q)), *_columns(q), kp, kld, *_columns(v), gp, gld, zp, zld, c_float(tau), _ptr(decay),
        _ptr(ctx.positions), _ptr(rotary.cos if rotary is not None else None),
        _ptr(rotary.sin if rotary is not None else None), c_int(rotary.rotary_dim if rotary is not None else 0),
        c_float(q_scale), c_float(k_scale), _ptr(state), _ptr(ctx.state_slots), _ptr(ctx.fresh), _ptr(ctx.cu_q),
        c_int(ctx.num_requests), _ptr(norm_weight), c_int(_vec_flag(norm_weight, out_dtype) if norm_weight is not None else 0),
        c_float(eps), _ptr(out), c_longlong(out.stride(0) if out is not None else 0), c_int(H), c_int(value_dim),
        c_int(seg_len), _ptr(seg_state),
        _ptr(seg_decay), c_int(max_segments), c_int(T), _ptr(raw_out), c_int(acts[input_activation]),
        c_int(1 if gate_activation == "sigmoid" else 0), c_int(1 if joint_norm else 0), _ptr(lower),
        c_int(1 if tied_key else 0), _ptr(token_keep), _ptr(token_write), c_int(qk_group), c_int(vw),
        c_int(0 if raw else 1), _ptr(step_raw), c_longlong(step_raw.stride(0) if step_raw is not None else 0),
        _ptr(step_bias), _ptr(step_rate), c_int(_f32(step_bias) if step_bias is not None else 0), _stream()),
        (3 if seg_len else 1) + int(wide and not raw))
    return raw_out if raw else out


# ----------------------------------------------------------------------------- a block that norms what its sub-layers return
class NormedAddend:
    """A sub-layer's output that joins the stream through a norm of its own: residual +=
    y / rms(y) * weight.  The kernel of the next norm does that add while it loads
    (``normed_add_rmsnorm``); ``materialize()`` gives the normed rows to any other consumer."""

    def __init__(self, y, weight, eps):
        self.y, self.weight, self.eps = materialize(y), weight, float(eps)
        self.shape, self.dtype, self.device = tuple(self.y.shape), self.y.dtype, self.y.device

    def materialize(self):
        return rmsnorm(self.y, self.weight, self.eps)


def normed_add_rmsnorm(addend: NormedAddend, residual, weight, eps, out_dtype, rows=None):
    """residual (float32, in place) += y / rms(y) * w_y; returns residual / rms(residual) * weight as
    ``out_dtype`` (``weight`` None: only the add).  With ``rows`` (int32) only those rows are added,
    normalised and returned, and the residual is left as it is."""
    y = addend.y
    _cuda(y, addend.weight, residual, weight, rows)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream is contiguous float32")
    if y.dtype != out_dtype or not y.is_contiguous() or y.shape != residual.shape:
        raise TypeError("normed_add_rmsnorm: the addend is contiguous, of the compute dtype and of the residual's shape")
    n = residual.shape[1]
    num_out = residual.shape[0] if rows is None else rows.shape[0]
    out = torch.empty(num_out, n, dtype=out_dtype, device=residual.device) if weight is not None else None
    lib = _latent_moe()
    _check(lib, lib.ts_normed_add_rmsnorm(
        c_int(_DTYPE[out_dtype]), _ptr(y), _ptr(addend.weight), c_int(_vec_flag(addend.weight, out_dtype)), _ptr(residual),
        _ptr(weight), c_int(_vec_flag(weight, out_dtype) if weight is not None else 0), c_float(addend.eps), c_float(eps),
        _ptr(out), _ptr(rows), c_int(num_out), c_int(n), c_int(0 if rows is not None else 1), _stream()))
    return out


# ----------------------------------------------------------------------------- latent attention
def latent_prepare(proj, q_rank, q_weight, eps, kv_rank=0, rot_dim=0, kv_weight=None, rotary=None, positions=None,
                   cache=None, slot_mapping=None):
    """From the fused projection of every token, proj [T, q_rank (+ kv_rank + rot_dim) + ...]: returns
    the RMS-normed query latent [T, q_rank] and, with ``kv_weight``, writes what the cache keeps of a
    token to its slot of ``cache`` [pages, 1, page, stored]: the RMS-normed key/value latent, then the
    shared key part rotated to the token's position, then zeros."""
    _cuda(proj, q_weight, kv_weight, positions, cache, slot_mapping)
    T = proj.shape[0]
    has_kv = kv_weight is not None
    if proj.stride(1) != 1 or proj.shape[1] < q_rank + (kv_rank + rot_dim if has_kv else 0):
        raise ValueError("latent_prepare: the projection does not hold the latents")
    if has_kv and cache is not None and (cache.dtype != proj.dtype or not cache.is_contiguous() or cache.shape[1] != 1):
        raise TypeError("latent_prepare: the cache is contiguous [pages, 1, page, stored] of the activations' dtype")
    stored = cache.shape[-1] if cache is not None else kv_rank + rot_dim
    q_latent = torch.empty(T, q_rank, dtype=proj.dtype, device=proj.device)
    lib = _latent_moe()
    _check(lib, lib.ts_latent_prepare(
        c_int(_dt(proj)), _ptr(proj), c_longlong(proj.stride(0)), c_int(q_rank), c_int(kv_rank), c_int(rot_dim),
        c_int(stored), c_int(1 if has_kv else 0), _ptr(q_weight), c_int(_vec_flag(q_weight, proj.dtype)), _ptr(kv_weight),
        c_int(_vec_flag(kv_weight, proj.dtype) if has_kv else 0), c_float(eps), _ptr(positions),
        _ptr(rotary.cos if rotary is not None else None), _ptr(rotary.sin if rotary is not None else None), _ptr(q_latent),
        _ptr(cache), _ptr(slot_mapping), c_int(T), c_int(int(rotary.interleaved) if rotary is not None else 0), _stream()))
    return q_latent


def latent_query(carried, q, num_heads, dim, rot_dim, stored, rotary, positions):
    """The attention kernel's query rows [T, H, stored]: per head ``carried`` [H, T, kv_rank] (the
    unrotated query carried into the latent space), then the head's rotated part (columns
    [dim, dim + rot_dim) of its ``dim + rot_dim`` columns of q [T, H (dim + rot_dim)]) turned to the
    token's position, then zeros."""
    _cuda(carried, q, positions)
    H, T, kv_rank = carried.shape
    if H != num_heads or not carried.is_contiguous() or q.stride(1) != 1 or q.shape != (T, H * (dim + rot_dim)):
        raise ValueError("latent_query: operands do not fit")
    out = torch.empty(T, H, stored, dtype=q.dtype, device=q.device)
    lib = _latent_moe()
    _check(lib, lib.ts_latent_query(
        c_int(_dt(q)), _ptr(carried), _ptr(q), c_longlong(q.stride(0)), c_int(H), c_int(dim), c_int(rot_dim), c_int(kv_rank),
        c_int(stored), _ptr(positions), _ptr(rotary.cos if rotary is not None else None),
        _ptr(rotary.sin if rotary is not None else None), _ptr(out), c_int(T),
        c_int(int(rotary.interleaved) if rotary is not None else 0), _stream()))
    return out


def gate_heads(x, gate=None):
    """[T, H * n] = x [H, T, n] * sigmoid(gate [T, H * n]); ``gate`` may be a column range, or None:
    the heads are laid side by side as they are."""
    _cuda(x, gate)
    H, T, n = x.shape
    if not x.is_contiguous() or (gate is not None and (gate.shape != (T, H * n) or gate.stride(1) != 1 or gate.dtype != x.dtype)):
        raise ValueError("gate_heads: operands do not fit")
    out = torch.empty(T, H * n, dtype=x.dtype, device=x.device)
    lib = _latent_moe()
    _check(lib, lib.ts_gate_heads(c_int(_dt(x)), _ptr(x), _ptr(gate), c_longlong(gate.stride(0) if gate is not None else 0),
                                  _ptr(out), c_int(H), c_int(n), c_int(T), _stream()))
    return out


def batched_matmul(a, b, side_by_side=False):
    """[B, M, N] = a [B, M, K] @ b [B, K, N], any strides, 32-bit sums.  bfloat16 operands go to the
    library's batched product (as the plain products of many rows do); float32 operands to this
    package's FMA kernel.  With ``side_by_side`` the result is [M, B * N]: every row's B results
    laid side by side (the library's product writes them there itself)."""
    _cuda(a, b)
    B, M, K = a.shape
    if b.shape[0] != B or b.shape[1] != K or a.dtype != b.dtype:
        raise ValueError(f"batched_matmul: {tuple(a.shape)} does not fit {tuple(b.shape)}")
    if side_by_side:
        if a.dtype != torch.bfloat16:
            return gate_heads(batched_matmul(a, b), None)
        out = torch.empty(M, B, b.shape[2], dtype=a.dtype, device=a.device)
        torch.bmm(a, b, out=out.transpose(0, 1))      # (leading dimension B * N, batches N apart)
        return out.view(M, B * b.shape[2])
    if a.dtype == torch.bfloat16:
        return torch.bmm(a, b)
    N = b.shape[2]
    out = torch.empty(B, M, N, dtype=a.dtype, device=a.device)
    lib = _latent_moe()
    _check(lib, lib.ts_batched_matmul(
        c_int(_dt(a)), _ptr(a), c_longlong(a.stride(0)), c_longlong(a.stride(1)), c_longlong(a.stride(2)), _ptr(b),
        c_longlong(b.stride(0)), c_longlong(b.stride(1)), c_longlong(b.stride(2)), _ptr(out), c_int(B), c_int(M), c_int(N),
        c_int(K), _stream()))
    return out


# ----------------------------------------------------------------------------- mixture of experts
def moe_route(logits, top, renormalize=False, bias=None):
    """float32 [T, E] router logits -> float32 [T, E]: softmax over all experts, the ``top`` largest
    keep their probability as it is, the others become zero.  With ``renormalize`` the kept ones are
    divided by their sum: the softmax over the chosen logits alone.  ``bias`` (float32 [E]) is added
    to the logits first."""
    _cuda(logits, bias)
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (logits.shape[1],)):
        raise TypeError("moe_route: the bias is float32 [experts]")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise TypeError("moe_route: router logits are contiguous float32")
    T, E = logits.shape
    gates = torch.empty_like(logits)
    lib = _latent_moe()
    _check(lib, lib.ts_moe_route(_ptr(logits), _ptr(gates), c_int(T), c_int(E), c_int(top), c_int(1 if renormalize else 0),
                                 _ptr(bias), _stream()))
    return gates


def moe_activate_(a, gates, num_experts, logits=None, top=0):
    """a [T, E * ff] (in place) <- relu(a)^2 * gates[t, e] for the columns of expert e.  With ``logits``
    (float32 [T, E]) and ``top`` in place of ``gates`` the kernel routes every token itself first, as
    ``moe_route`` does: one launch for softmax, choice and activation."""
    _cuda(a, gates, logits)
    T = a.shape[0]
    given = gates if gates is not None else logits
    if (gates is None) == (logits is None) or not a.is_contiguous() or a.shape[1] % num_experts \
            or given.shape != (T, num_experts) or given.dtype != torch.float32 or not given.is_contiguous():
        raise ValueError("moe_activate: operands do not fit")
    lib = _latent_moe()
    _check(lib, lib.ts_moe_activate(c_int(_dt(a)), _ptr(a), _ptr(gates), c_int(T), c_int(num_experts),
                                    c_int(a.shape[1] // num_experts), _ptr(logits), c_int(top), _stream()))
    return a


#: from this many tokens on (bfloat16, fewer experts chosen than there are) a step's tokens are sorted by
#: expert and every expert multiplies its own rows only; below, all experts run on all tokens and the
#: unchosen ones are multiplied by zero (a few decoded tokens touch most experts' weights anyway, and the
#: dense products are this package's tcgen05 kernels)
MOE_GROUPED_MIN_TOKENS = 256


def moe_grouped(h, gates, up, down_side_by_side, top, gated=False, activation="silu", limit=0.0):
    """Mixture of experts over rows sorted by expert.  h [T, n] bfloat16; gates float32 [T, E] (zero:
    not chosen); up [E ff, n] (expert by expert); down_side_by_side [n, E ff].  Returns [T, n]:
    sum over a token's experts of gate * W_down,e relu(W_up,e h)^2, the sum in 32-bit.  The two
    products over ragged row groups are the library's grouped product."""
    _cuda(h, gates, up, down_side_by_side)
    T, n = h.shape
    E = gates.shape[1]
    ff = up.shape[0] // E // (2 if gated else 1)
    lib = _latent_moe()
    align = lib.ts_moe_group_align()
    capacity = -(-(T * top + E * (align - 1)) // align) * align + align
    meta = torch.empty(capacity + T * E + E, dtype=torch.int32, device=h.device)
    row_token, pair_row, ends = meta[:capacity], meta[capacity:capacity + T * E], meta[capacity + T * E:]
    _check(lib, lib.ts_moe_group(_ptr(gates), c_int(T), c_int(E), _ptr(row_token), _ptr(pair_row), _ptr(ends), c_int(capacity),
                                 _stream()))
    x = torch.empty(capacity, n, dtype=h.dtype, device=h.device)
    _check(lib, lib.ts_moe_gather(c_int(_dt(h)), _ptr(h), _ptr(row_token), _ptr(x), c_int(capacity), c_int(n), _stream()))
    if gated:
        a = moe_gated_activate(torch.nn.functional.grouped_mm(x, up.view(E, 2 * ff, n).transpose(1, 2), offs=ends), None, 1,
                               activation, limit)
    else:
        a = torch.nn.functional.grouped_mm(x, up.view(E, ff, n).transpose(1, 2), offs=ends)
        _check(lib, lib.ts_moe_activate(c_int(_dt(a)), _ptr(a), None, c_int(capacity), c_int(1), c_int(ff), None, c_int(0), _stream()))
    y = torch.nn.functional.grouped_mm(a, down_side_by_side.view(n, E, ff).permute(1, 2, 0), offs=ends)
    out = torch.empty(T, n, dtype=h.dtype, device=h.device)
    _check(lib, lib.ts_moe_combine(c_int(_dt(y)), _ptr(y), _ptr(gates), _ptr(pair_row), _ptr(out), c_int(T), c_int(E), c_int(n),
                                   _stream()))
    count_launches(2)
    return out


# ----------------------------------------------------------------------------- rows that depend on their neighbours in time
def _f32(t) -> int:
    if t.dtype == torch.float32:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise TypeError(f"unsupported dtype {t.dtype}; kernels take float32 and bfloat16")


def add_position_rows_(residual, table, positions):
    """residual float32 [T, n] (in place) += table[positions] (a learned vector per position)."""
    _cuda(residual, table, positions)
    T, n = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous() or table.shape[1] != n or not table.is_contiguous():
        raise TypeError("add_position_rows: the residual is contiguous float32 and the table has its width")
    lib = _sequence()
    _check(lib, lib.ts_add_position_rows(_ptr(residual), _ptr(table), c_int(_f32(table)), _ptr(positions),
                                         c_int(table.shape[0]), c_int(T), c_int(n), _stream()))
    return residual


CAUSAL_CONV_MAX_TAPS = 8


def causal_conv(x, weight, state, ctx, out_dtype, bias=None, add_input=False, activation=None):
    """Causal convolution over time on every channel: y_t = sum_j weight[:, j] x_(t - taps + 1 + j)
    (+ bias), zeros before a sequence's start, then silu with ``activation`` "silu", then + x_t with
    ``add_input``.  x [T, C] float32 or of the compute type (a column range is fine); weight
    [C, taps]; ``state`` float32 [slots, taps - 1, C] holds every request's last inputs between
    steps (``ctx.state_slots``, ``ctx.fresh``, ``ctx.cu_q``) and is brought up to date.  Returns
    [T, C] of ``out_dtype``."""
    _cuda(x, weight, bias, state)
    T, C = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != C or not weight.is_contiguous() or x.stride(1) != 1 or activation not in (None, "silu"):
        raise ValueError("causal_conv: weight [channels, taps], x contiguous along its rows, activation None or silu")
    if not 1 <= taps <= CAUSAL_CONV_MAX_TAPS:
        raise ValueError(f"causal_conv: 1 to {CAUSAL_CONV_MAX_TAPS} taps, got {taps}")
    if taps > 1 and (state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps - 1, C) or not state.is_contiguous()):
        raise TypeError("causal_conv: the state is contiguous float32 [slots, taps - 1, channels]")
    if bias is not None and (bias.dtype != weight.dtype or bias.shape != (C,)):
        raise TypeError("causal_conv: the bias is [channels] of the weight's dtype")
    out = torch.empty(T, C, dtype=out_dtype, device=x.device)
    lib = _sequence()
    _check(lib, lib.ts_causal_conv(
        _ptr(x), c_longlong(x.stride(0)), c_int(_f32(x)), _ptr(out), c_longlong(C), c_int(_f32(out)), _ptr(weight),
        c_int(_f32(weight)), _ptr(bias), c_int(taps), _ptr(state), _ptr(ctx.state_slots), _ptr(ctx.fresh), _ptr(ctx.cu_q),
        c_int(ctx.num_requests), c_int(max(1, min(ctx.max_q_len or T, T))), c_int(C), c_int(1 if add_input else 0),
        c_int(1 if activation == "silu" else 0), _stream()))
    return out


def group_norm(x, weight, groups, eps, out_dtype, rows=None):
    """Every one of ``groups`` equal consecutive parts of a row divided by its own root mean
    square, the row times ``weight``.  x [T, n] float32 or of the compute type; with ``rows``
    (int32) only those rows, in that order."""
    _cuda(x, weight, rows)
    n = x.shape[1]
    if x.stride(1) != 1 or weight.shape != (n,) or n % groups:
        raise ValueError(f"group_norm: {n} columns in {groups} groups")
    num_out = x.shape[0] if rows is None else rows.shape[0]
    out = torch.empty(num_out, n, dtype=out_dtype, device=x.device)
    lib = _sequence()
    _check(lib, lib.ts_group_norm(_ptr(x), c_longlong(x.stride(0)), c_int(_f32(x)), _ptr(weight), c_int(_f32(weight)),
                                  _ptr(rows), c_int(groups), c_int(n), c_float(eps), _ptr(out), c_int(_f32(out)),
                                  c_int(num_out), _stream()))
    return out


def group_norm_add_(y, weight, groups, eps, residual):
    """residual float32 [T, n] (in place) += group_norm(y) * weight: the sum stays 32-bit."""
    y = materialize(y)
    _cuda(y, weight, residual)
    T, n = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous() or tuple(y.shape) != (T, n) or y.stride(1) != 1 \
            or weight.shape != (n,) or n % groups:
        raise ValueError(f"group_norm_add: the residual is contiguous float32 [T, {n}], y of its shape, {groups} groups")
    lib = _sequence()
    _check(lib, lib.ts_group_norm_add(_ptr(y), c_longlong(y.stride(0)), c_int(_f32(y)), _ptr(weight), c_int(_f32(weight)),
                                      c_int(groups), c_int(n), c_float(eps), _ptr(residual), c_int(T), _stream()))
    return residual


def axpby(a, x, b, y):
    """a x + b y for two contiguous tensors alike in shape and dtype (32-bit arithmetic)."""
    x, y = materialize(x), materialize(y)
    _cuda(x, y)
    if x.shape != y.shape or x.dtype != y.dtype or not x.is_contiguous() or not y.is_contiguous():
        raise TypeError("axpby: operands are contiguous and alike in shape and dtype")
    out = torch.empty_like(x)
    lib = _sequence()
    _check(lib, lib.ts_axpby(_ptr(x), _ptr(y), c_int(_f32(x)), c_float(a), c_float(b), _ptr(out), c_int(_f32(out)),
                             c_longlong(x.numel()), _stream()))
    return out


def gate_columns(attn, gate, vdim):
    """[T, H * vdim] = attn [T, H, D][..., :vdim] * sigmoid(gate [T, H * vdim]), element by element;
    ``gate`` may be a column range."""
    _cuda(attn, gate)
    T, H, D = attn.shape
    if not attn.is_contiguous() or gate.shape != (T, H * vdim) or gate.stride(1) != 1 or gate.dtype != attn.dtype:
        raise ValueError("gate_columns: operands do not fit")
    out = torch.empty(T, H * vdim, dtype=attn.dtype, device=attn.device)
    lib = _sequence()
    _check(lib, lib.ts_gate_columns(_ptr(attn), _ptr(gate), c_longlong(gate.stride(0)), c_int(_f32(attn)), _ptr(out), c_int(H),
                                    c_int(D), c_int(vdim), c_int(T), _stream()))
    return out


def joint_norm_kvwrite(q, k, v, num_heads, num_kv_heads, dim, vdim, stored_dim, q_weight=None, k_weight=None, eps=0.0,
                       k_cache=None, v_cache=None, slot_mapping=None, page_size=0):
    """q [T, H dim] and k [T, Hkv dim] each divided by the root mean square over the whole row (all
    heads at once) and multiplied by a weight per column (both weights None: no norm); q goes to a
    [T, H, stored_dim] tensor (returned), k and v [T, Hkv vdim] to the cache slots of
    ``slot_mapping`` (None: nothing is written), heads padded with zeros to ``stored_dim``."""
    _cuda(q, k, v, q_weight, k_weight, k_cache, v_cache, slot_mapping)
    T = q.shape[0]
    if q.shape[1] != num_heads * dim or k.shape[1] != num_kv_heads * dim or v.shape[1] != num_kv_heads * vdim:
        raise ValueError("joint_norm_kvwrite: q, k, v do not have heads x size columns")
    if k_cache is not None and (k_cache.dtype != q.dtype or k_cache.shape[-1] != stored_dim or not k_cache.is_contiguous()
                                or not v_cache.is_contiguous()):
        raise TypeError("joint_norm_kvwrite: the cache does not fit the activations")
    if (q_weight is None) != (k_weight is None) or (q_weight is not None and q_weight.dtype != k_weight.dtype):
        raise TypeError("joint_norm_kvwrite: q and k are normed together, with weights of one dtype")
    out = torch.empty(T, num_heads, stored_dim, dtype=q.dtype, device=q.device)
    lib = _sequence()
    _check(lib, lib.ts_joint_norm_kvwrite(
        c_int(_f32(q)), *_columns(q), *_columns(k), *_columns(v), _ptr(q_weight), _ptr(k_weight),
        c_int(_f32(q_weight) if q_weight is not None else 0), c_float(eps), c_int(num_heads), c_int(num_kv_heads),
        c_int(dim), c_int(vdim), c_int(stored_dim), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping),
        c_int(page_size), c_int(T), _stream()))
    return out


def mlstm_gates(raw, cap, m_state, ctx, num_heads):
    """The stabilised gates of a matrix memory with an exponential input gate.  raw float32
    [T, 2 H]: input-gate logits, then forget-gate logits.  i = cap tanh(. / cap),
    f = logsigmoid(cap tanh(. / cap)), m_t = max(f_t + m_(t-1), i_t) with m in ``m_state`` float32
    [slots, H] (zero for a request that starts).  Returns float32 [T, H] each: keep =
    exp(f + m_(t-1) - m_t), write = exp(i - m_t), floor = exp(-m_t).  Steps with a request of 128 tokens
    or more (``ctx.max_q_len``) give a block to each (request, head), whose warps take spans of its tokens."""
    _cuda(raw, m_state)
    T, H = raw.shape[0], num_heads
    if raw.dtype != torch.float32 or raw.shape[1] != 2 * H or raw.stride(1) != 1 or m_state.dtype != torch.float32 \
            or tuple(m_state.shape[1:]) != (H,) or not m_state.is_contiguous():
        raise TypeError("mlstm_gates: raw float32 [T, 2 H], m float32 [slots, H]")
    keep, write, floor = (torch.empty(T, H, dtype=torch.float32, device=raw.device) for _ in range(3))
    lib = _sequence()
    _check(lib, lib.ts_mlstm_gates(_ptr(raw), c_longlong(raw.stride(0)), c_float(cap), _ptr(m_state), _ptr(ctx.state_slots),
                                   _ptr(ctx.fresh), _ptr(ctx.cu_q), c_int(ctx.num_requests), c_int(ctx.max_q_len), c_int(H),
                                   _ptr(keep), _ptr(write), _ptr(floor), _stream()))
    return keep, write, floor


def mlstm_finish(raw, floor, weight, gate, eps, num_heads, value_dim, out_dtype):
    """raw float32 [T, H, wide]: columns [0, value_dim) the numerators, column value_dim the
    normaliser n . q.  Returns [T, H value_dim]: numerator / (max(|n . q|, floor) + 1e-6), divided by
    its root mean square per head, times weight [H value_dim], times sigmoid(gate)."""
    _cuda(raw, floor, weight, gate)
    T, H = floor.shape
    wide = raw.shape[1] // H
    if raw.dtype != torch.float32 or not raw.is_contiguous() or H != num_heads or wide <= value_dim or gate.stride(1) != 1:
        raise TypeError("mlstm_finish: operands do not fit")
    out = torch.empty(T, H * value_dim, dtype=out_dtype, device=raw.device)
    lib = _sequence()
    _check(lib, lib.ts_mlstm_finish(_ptr(raw), c_int(wide), _ptr(floor), _ptr(weight), c_int(_f32(weight)), _ptr(gate),
                                    c_longlong(gate.stride(0)), c_int(_f32(out)), c_float(eps), _ptr(out), c_int(H),
                                    c_int(value_dim), c_int(T), _stream()))
    return out


def ssm_finish(raw, x, skip, z, weight, groups, eps, num_heads, value_dim, out_dtype):
    """(raw + skip[h] x) silu(z), RMS-normed in ``groups`` equal parts over all heads, times weight.
    raw float32 [T, H value_dim]; x, z [T, H value_dim] of the compute type (column ranges are fine)."""
    _cuda(raw, x, skip, z, weight)
    T = raw.shape[0]
    n = num_heads * value_dim
    if raw.dtype != torch.float32 or not raw.is_contiguous() or raw.shape[1] != n or x.shape[1] != n or z.shape[1] != n \
            or x.stride(1) != 1 or z.stride(1) != 1 or skip.dtype != weight.dtype or n % groups:
        raise TypeError("ssm_finish: operands do not fit")
    out = torch.empty(T, n, dtype=out_dtype, device=raw.device)
    lib = _sequence()
    _check(lib, lib.ts_ssm_finish(_ptr(raw), _ptr(x), c_longlong(x.stride(0)), _ptr(skip), _ptr(z), c_longlong(z.stride(0)),
                                  _ptr(weight), c_int(_f32(weight)), c_int(_f32(out)), c_int(groups), c_float(eps), _ptr(out),
                                  c_int(num_heads), c_int(value_dim), c_int(T), _stream()))
    return out


# ----------------------------------------------------------------------------- experts chosen by scores with a correction
def moe_route_scored(logits, correction, top, groups=1, keep=1):
    """float32 [T, E] router logits -> float32 [T, E] weights: s = sigmoid(z) for the ``top`` experts
    with the largest s + correction among the experts of the ``keep`` best of ``groups`` equal groups
    of neighbours (a group's score: the sum of its two largest s + correction), zero elsewhere."""
    _cuda(logits, correction)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise TypeError("moe_route_scored: router logits are contiguous float32")
    T, E = logits.shape
    if correction is not None and (correction.dtype != torch.float32 or correction.shape != (E,)):
        raise TypeError("moe_route_scored: the correction is float32 [experts]")
    gates = torch.empty_like(logits)
    lib = _latent_moe()
    _check(lib, lib.ts_moe_route_scored(_ptr(logits), _ptr(correction), _ptr(gates), c_int(T), c_int(E), c_int(top),
                                        c_int(groups), c_int(keep), _stream()))
    return gates


def moe_gated_activate(a, gates, num_experts, activation="silu", limit=0.0, logits=None, top=0, renormalize=False,
                       bias=None):
    """a [rows, E * 2 ff] (per expert: gate rows, then up rows) -> [rows, E * ff] =
    act(gate) * up * gates[row, e] (``activation`` as in ``gated_activation``); ``gates`` None: no
    weight (rows that are sorted by expert).  With ``logits`` (float32 [rows, E]) and ``top`` in
    place of ``gates`` the kernel routes every row itself first, as ``moe_route`` does with the same
    ``renormalize`` and ``bias``: one launch for softmax, choice and activation."""
    _cuda(a, gates, logits, bias)
    code, limit = activation_code(activation, limit)
    if logits is not None and (gates is not None or logits.shape != (a.shape[0], num_experts) or logits.dtype != torch.float32
                               or not logits.is_contiguous() or not 0 < top <= num_experts
                               or (bias is not None and (bias.dtype != torch.float32 or bias.shape != (num_experts,)))):
        raise ValueError("moe_gated_activate: logits are float32 [rows, experts], with top and without gates")
    rows = a.shape[0]
    ff = a.shape[1] // (2 * num_experts)
    if not a.is_contiguous() or a.shape[1] != 2 * ff * num_experts or \
            (gates is not None and (gates.shape != (rows, num_experts) or gates.dtype != torch.float32 or not gates.is_contiguous())):
        raise ValueError("moe_gated_activate: operands do not fit")
    out = torch.empty(rows, num_experts * ff, dtype=a.dtype, device=a.device)
    lib = _latent_moe()
    _check(lib, lib.ts_moe_gated_activate(c_int(_dt(a)), _ptr(a), _ptr(gates), c_int(rows), c_int(num_experts), c_int(ff),
                                          _ptr(out), c_int(code), c_float(limit), _ptr(logits), _ptr(bias), c_int(top),
                                          c_int(1 if renormalize else 0), _stream()))
    return out

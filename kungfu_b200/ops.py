"""The operations parts are written in, each one a hand-written CUDA kernel of `csrc/`.

Every function here checks its arguments on the host and launches on the current CUDA stream.
There is no CPU implementation and no library fallback: a tensor that is not on a CUDA device, a
missing compiler or a failed build raises.  (Tests that have no GPU replace this table of
functions with a slow emulation of their own through `set_override`; the package ships none.)
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

F32, BF16 = 0, 1
_ACT = {"gelu_tanh": 0, "gelu_erf": 1, "silu": 2, "clamped_swish": 3}      # 3: gated products only, with a limit
_STATUS = {1: "unsupported combination of element types", 2: "unsupported size", 3: "CUDA launch failed",
           4: "alignment rule broken", 5: "one-time set-up failed"}

MAX_HEAD_DIM = 256
MAX_GENERIC_HEAD_DIM = 512      # the generic attention kernel alone takes heads above MAX_HEAD_DIM, up to this


class KernelError(RuntimeError):
    pass


_lib = None
_lib_lock = threading.Lock()
_override = None


def set_override(impl) -> None:
    """Tests without a GPU install an object whose attributes replace the functions of this module."""
    global _override
    _override = impl


def library():
    """The compiled kernel library (built at first use)."""
    global _lib
    if _lib is None:
        with _lib_lock:
            if _lib is None:
                from .csrc import build as _build
                path = _build.build()
                lib = ctypes.CDLL(path)
                lib.kf_last_cuda_error.restype = ctypes.c_char_p
                # kernels may start before their predecessor in the stream has finished (each waits for it before
                # touching dependent memory); KUNGFU_PDL=0 switches that off
                lib.kf_set_pdl(0 if os.environ.get("KUNGFU_PDL", "1") == "0" else 1)
                _lib = lib
    return _lib


class plain_launches:
    """Within this context kernels are launched WITHOUT programmatic dependent launch: each starts only when everything
    before it in the stream has finished.  Needed around a kernel that reads, before its own dependency wait, memory that
    another kernel of the same step wrote: the decode attention kernels request the step's positions that early, which is
    safe for the integers the host copied in and not for integers a kernel derived from them."""

    def __enter__(self):
        if _override is None:
            library().kf_set_pdl(0)
        return self

    def __exit__(self, *exc):
        if _override is None:
            library().kf_set_pdl(0 if os.environ.get("KUNGFU_PDL", "1") == "0" else 1)
        return False


def library_path() -> str:
    from .csrc import build as _build
    return os.path.join(_build.build_dir(), _build.LIB_NAME)


_launches = 0
_fallbacks: dict[str, int] = {}


def note_fallback(what: str) -> None:
    """A bfloat16 operation that ran on a slower generic kernel because the fast one refuses its shape."""
    _fallbacks[what] = _fallbacks.get(what, 0) + 1


def fallbacks() -> dict[str, int]:
    """How often, and why, bfloat16 work left the tensor-core kernels (shown by `describe` and the bench)."""
    return dict(_fallbacks)


def fallback_count() -> int:
    return sum(_fallbacks.values())


def launch_count() -> int:
    """Kernels launched through this module so far (graph replays add the kernels they hold)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    _launches += 1
    if status != 0:
        detail = _STATUS.get(status, f"status {status}")
        if status == 3:
            detail += f" ({library().kf_last_cuda_error().decode()})"
        raise KernelError(f"{what}: {detail}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {t.dtype} is not supported (float32 and bfloat16 are)")


def _p(t: torch.Tensor | None):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kungfu_b200 kernels run on CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernel arguments must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


_pinned_stream = None


def _stream():
    if _pinned_stream is not None:
        return _pinned_stream
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class pinned_stream:
    """Within this context every launch goes to the stream that is current on entry, looked up once (asking torch for the
    current stream costs as much as a launch).  The step function wraps the model's pass in it."""

    def __enter__(self):
        global _pinned_stream
        self._was = _pinned_stream
        _pinned_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._was
        return False


def _f(x: float):
    return ctypes.c_float(x)


# ---- per-kernel timing (the reference's KF_TRACE_KERNELS, crates/kf-backend-cuda/src/exec.rs:2836-2853) -----------
_trace: list | None = None


def trace_begin() -> None:
    """Start timing every operation of this module with CUDA events (steps then run eagerly, not from graphs)."""
    global _trace
    _trace = []


def trace_end() -> list[tuple[str, float]]:
    """Stop timing; returns (operation, milliseconds) in launch order."""
    global _trace
    rec, _trace = _trace or [], None
    if rec:
        torch.cuda.synchronize()
    return [(name, e0.elapsed_time(e1)) for name, e0, e1 in rec]


def tracing() -> bool:
    return _trace is not None


# NVTX ranges around every part and operation, for timelines of a profiler (KUNGFU_NVTX=1 or ops.nvtx_ranges = True).
nvtx_ranges = os.environ.get("KUNGFU_NVTX", "0") == "1"


class nvtx_range:
    """`with ops.nvtx_range("layer 3"):` opens an NVTX range when ranges are switched on, and costs a test otherwise."""

    def __init__(self, name: str):
        self.name = name
        self.on = False

    def __enter__(self):
        self.on = nvtx_ranges and _override is None
        if self.on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()
        return False


def _dispatch(name):
    def deco(fn):
        def wrapper(*a, **k):
            if _override is not None:
                return getattr(_override, name)(*a, **k)
            if nvtx_ranges:
                with nvtx_range(name):
                    return fn(*a, **k)
            if _trace is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = fn(*a, **k)
                e1.record()
                _trace.append((name, e0, e1))
                return out
            return fn(*a, **k)
        wrapper.__name__ = name
        wrapper.__wrapped__ = fn
        wrapper.__doc__ = fn.__doc__
        return wrapper
    return deco


# ---- size rules ---------------------------------------------------------------------------------------

def check_attention_sizes(n_heads: int, n_kv_heads: int, head_dim: int, largest: int = MAX_HEAD_DIM) -> None:
    """Head sizes the attention kernels take: 2..256, even.  Anything else is refused here, at build time.  (`largest` up to
    MAX_GENERIC_HEAD_DIM for a mixer that accepts the generic kernel alone above 256: a latent's stored head.)"""
    if head_dim < 2 or head_dim > min(largest, MAX_GENERIC_HEAD_DIM) or head_dim % 2:
        raise KernelError(f"head_dim {head_dim} is not supported: the attention kernels take even sizes up to {largest}")
    if n_kv_heads < 1 or n_heads % n_kv_heads:
        raise KernelError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")


KERNEL_HEAD_SIZES = (16, 32, 64, 128, 256)


def attention_head_size(n: int) -> int:
    """The smallest head size the tensor-core attention kernels take that holds `n` elements (heads are stored with zero
    tails up to it)."""
    for d in KERNEL_HEAD_SIZES:
        if n <= d:
            return d
    raise KernelError(f"heads of {n} elements are above {MAX_HEAD_DIM}, the largest the attention kernels take")


# ---- operations -----------------------------------------------------------------------------------------

@_dispatch("embed")
def embed(tokens, table, scale: float, out) -> None:
    """out[t, :] = table[tokens[t], :] * scale (32-bit out).  Token ids are validated by the caller on the host."""
    T, (V, H) = out.shape[0], table.shape
    _check(library().kf_embed(_p(tokens), _p(table), _dt(table), _f(scale), _p(out), T, H, V, ctypes.c_void_p(0), _stream()),
           "embed")


@_dispatch("rmsnorm")
def rmsnorm(x, weight, eps: float, plus_one: bool, out, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r]] if rows is given else x[r]) * (weight or 1 + weight)."""
    n, H = out.shape
    _check(library().kf_rmsnorm(_p(x), _p(weight), _dt(weight), _f(eps), int(plus_one), _p(out), _dt(out), _p(rows), n, H,
                                _stream()), "rmsnorm")


@_dispatch("add_rmsnorm")
def add_rmsnorm(branch, weight, eps: float, plus_one: bool, residual, *, next_weight=None, next_eps: float = 0.0,
                next_plus_one: bool = False, next_out=None, copy_out=None) -> None:
    """residual += rmsnorm(branch) * g; if next_out is given, next_out = rmsnorm(residual) * g_next; if copy_out is given
    (instead), copy_out = the new residual rows in copy_out's element type (for a sublayer that reads the stream itself)."""
    T, H = residual.shape
    if copy_out is not None:
        if next_out is not None:
            raise KernelError("add_rmsnorm: either the next norm or a plain copy, not both")
        _check(library().kf_add_rmsnorm(_p(branch), _p(weight), _dt(weight), _f(eps), int(plus_one), _p(residual),
                                        _p(weight), _dt(weight), _f(0.0), 2, _p(copy_out), _dt(copy_out), T, H, _stream()),
               "add_rmsnorm")
        return
    _check(library().kf_add_rmsnorm(_p(branch), _p(weight), _dt(weight), _f(eps), int(plus_one), _p(residual),
                                    _p(next_weight), _dt(next_weight) if next_weight is not None else F32, _f(next_eps),
                                    int(next_plus_one), _p(next_out), _dt(next_out) if next_out is not None else F32,
                                    T, H, _stream()), "add_rmsnorm")


@_dispatch("add")
def add(a, x) -> None:
    """x += a (32-bit)."""
    _check(library().kf_add(_p(a), _p(x), ctypes.c_long(x.numel()), _stream()), "add")


# ---- scratch memory of the split-K products and the device error word ---------------------------------------

_scratch: dict = {}          # device -> {"partial": tensor, "counters": tensor, "error": tensor, "retired": [tensors]}
use_tensor_cores = True      # tests switch this off to reach the generic product with bfloat16 operands
use_fast_attention = True    # likewise for the generic attention kernel
fused_qkv_rope = True        # False: the q,k,v product of a prompt always leaves 32-bit rows for `rope_kv_append`
fused_qkv_rope_launches = 0  # how often the product that rotates and files its own result has run (tests look at it)
prefill_on_tcgen05 = True       # False: the mma.sync prompt kernel for every head and page size
split_prompt_keys = True        # False: one block per (tile of rows, head) however few blocks that makes
decode_on_tensor_cores = True   # False: the SIMT split-KV decode kernel (kept for groups of more than 16 heads)
prefill_plan_override = None    # (runs per tile, key tiles above which a tile is cut): tests reach every launch shape with it


def _dev_scratch(device) -> dict:
    key = (device.type, device.index)
    sc = _scratch.get(key)
    if sc is None:
        sc = {"partial": torch.empty(1 << 20, dtype=torch.float32, device=device),
              "counters": torch.zeros(8192, dtype=torch.int32, device=device),
              "error": torch.zeros(1, dtype=torch.int32, device=device), "retired": []}
        _scratch[key] = sc
    return sc


def _partial(device, n_floats: int) -> torch.Tensor:
    sc = _dev_scratch(device)
    if sc["partial"].numel() < n_floats:
        sc["retired"].append(sc["partial"])          # a captured graph may still point at it
        sc["partial"] = torch.empty(max(n_floats, 2 * sc["partial"].numel()), dtype=torch.float32, device=device)
    return sc["partial"]


def device_error(device=None) -> int:
    """The error word kernels with bounded waits write (0 = none).  Reading it waits for the device."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sc = _scratch.get((device.type, device.index))
    return 0 if sc is None else int(sc["error"].item())


def clear_device_error(device=None) -> None:
    """Set the error word back to 0 (after a failure that was looked at)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sc = _scratch.get((device.type, device.index))
    if sc is not None:
        sc["error"].zero_()


def raise_on_device_error(device=None) -> None:
    code = device_error(device)
    if code:
        raise KernelError(f"a kernel gave up waiting (code {code}: 1 = operands never arrived, 2 = stage never freed, "
                          f"3 = accumulator never completed)")


_rope_plans: dict = {}            # (rows, K, heads, kv heads, head size, rotated) -> whether the fused q,k,v product takes them
_linear_plans: dict = {}          # (rows, features, K, mode) -> (token tile, K splits) as the library plans them


def _linear_tc(x, weight, out, mode: int, N: int, softcap: float, act: int) -> bool:
    """Launch the tcgen05 product if it takes these operands; False if the generic kernel must run."""
    T, K = x.shape
    lib = library()
    if not (use_tensor_cores and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16):
        return False
    if not lib.kf_linear_tc_supported(_p(x), _p(weight), K):
        note_fallback(f"linear: rows of {K} bfloat16 elements are no multiple of 16 bytes (or a base is unaligned)")
        return False
    plan = _linear_plans.get((T, N, K, mode))
    if plan is None:
        bn, splits = ctypes.c_int(0), ctypes.c_int(0)
        lib.kf_linear_tc_plan(T, N, K, int(mode == 2), ctypes.byref(bn), ctypes.byref(splits))
        plan = _linear_plans[(T, N, K, mode)] = (bn.value, splits.value)
    bn, splits = plan
    sc = _dev_scratch(x.device)
    partial = None
    if splits > 1:
        if -(-N // 128) * -(-T // bn) > sc["counters"].numel():
            note_fallback("linear: more output tiles than split counters")
            return False
        partial = _partial(x.device, splits * T * (2 * N if mode == 2 else N))
    _check(lib.kf_linear_tc(_p(x), _p(weight), _p(out), mode, T, N, K, _f(softcap), act, bn, splits,
                            _p(partial), _p(sc["counters"]), _p(sc["error"]), _stream()), "linear (tensor cores)")
    return True


@_dispatch("linear")
def linear(x, weight, out, softcap: float = 0.0) -> None:
    """out[T, N] = x[T, K] . weight[N, K]^T, 32-bit accumulation; softcap > 0 applies cap*tanh(v/cap).
    bfloat16 operands run on the tensor cores (tcgen05) when rows are multiples of 16 bytes; everything else,
    and the whole 32-bit path, runs the generic 32-bit FMA kernel."""
    T, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or tuple(out.shape) != (T, N):
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    if out.dtype == torch.float32 or softcap == 0.0:
        if _linear_tc(x, weight, out, 0 if out.dtype == torch.float32 else 1, N, softcap, 0):
            return
    _check(library().kf_linear_simt(_p(x), _dt(x), _p(weight), _dt(weight), _p(out), _dt(out), T, N, K, _f(softcap),
                                    _stream()), "linear")


@_dispatch("linear_gated")
def linear_gated(x, w_gate_up, out, activation: str, ctx, limit: float = 0.0) -> None:
    """out[T, I] = act(x . Wgate^T) * (x . Wup^T) with w_gate_up = [Wgate; Wup] stacked by rows.  The activation
    'clamped_swish' is the gated form g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1)."""
    T = x.shape[0]
    I = out.shape[1]
    clamped = activation == "clamped_swish"
    if out.dtype == torch.bfloat16 and _linear_tc(x, w_gate_up, out, 2, I, float(limit) if clamped else 0.0, _ACT[activation]):
        return
    gu = ctx.buf("ffn_gate_up", (T, 2 * I), torch.float32)
    linear(x, w_gate_up, gu)
    _check(library().kf_gated_act(_p(gu), _dt(gu), _p(out), _dt(out), T, I, _ACT[activation], _f(limit), _stream()), "gated_act")


@_dispatch("linear_act")
def linear_act(x, w_up, out, activation: str, ctx) -> None:
    """out[T, I] = act(x . Wup^T): the first half of a feed-forward without a gate."""
    T = x.shape[0]
    I = out.shape[1]
    # bfloat16: the activation is the product's own epilogue (the code act + 1 on its bfloat16 store)
    if out.dtype == torch.bfloat16 and _linear_tc(x, w_up, out, 1, I, 0.0, _ACT[activation] + 1):
        return
    up = ctx.buf("ffn_up", (T, I), torch.float32)
    linear(x, w_up, up)
    activation_(up, out, activation)


@_dispatch("rope_table")
def rope_table(positions, inv_freq, cos, sin) -> None:
    """cos/sin[t, i] of positions[t] * inv_freq[i], 32-bit."""
    T, half = cos.shape
    _check(library().kf_rope_table(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, half, _stream()), "rope_table")


@_dispatch("rope_kv_append")
def rope_kv_append(qkv, cos, sin, rot: int, n_heads: int, n_kv_heads: int, head_dim: int, ctx, cache, q_out) -> None:
    """Rotate q and k (pairs i, i+rot/2), write q to q_out and k, v into the pages of `cache` (if it writes)."""
    T = qkv.shape[0]
    table = ctx.block_tables[cache.group]
    _check(library().kf_rope_kv_append(_p(qkv), _p(cos), _p(sin), rot, n_heads, n_kv_heads, head_dim,
                                       _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size,
                                       _p(cache.pages), _dt(cache.pages), _p(q_out), _dt(q_out), int(cache.writes),
                                       T, _stream()), "rope_kv_append")


@_dispatch("linear_rope_kv_append")
def linear_rope_kv_append(x, wqkv, cos, sin, rot: int, n_heads: int, n_kv_heads: int, head_dim: int, ctx, cache, q_out) -> bool:
    """q,k,v = x . wqkv^T, q and k rotated, q to q_out, k and v into the pages of `cache`: one launch whose product files
    its own result (no 32-bit q,k,v rows in memory).  True if it ran; False if this step does not qualify (then the
    caller runs `linear` and `rope_kv_append`): it takes bfloat16 operands, q and pages, head size 256 or 128 rotated in full,
    and so many rows that the product runs as whole tiles on CTA pairs."""
    T, K = x.shape
    if not (use_tensor_cores and fused_qkv_rope and cos is not None and x.dtype == torch.bfloat16
            and wqkv.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16 and cache.pages.dtype == torch.bfloat16):
        return False
    lib = library()
    key = (T, K, n_heads, n_kv_heads, head_dim, rot)
    ok = _rope_plans.get(key)
    if ok is None:
        ok = _rope_plans[key] = bool(lib.kf_linear_rope_append_supported(_p(x), _p(wqkv), T, K, n_heads, n_kv_heads, head_dim, rot))
    if not ok or (x.data_ptr() | wqkv.data_ptr()) & 15:
        return False
    table = ctx.block_tables[cache.group]
    sc = _dev_scratch(x.device)
    global fused_qkv_rope_launches
    fused_qkv_rope_launches += 1
    _check(lib.kf_linear_rope_append(_p(x), _p(wqkv), T, K, n_heads, n_kv_heads, head_dim, _p(cos), _p(sin), _p(ctx.positions),
                                     _p(ctx.row_req), _p(table), table.shape[1], cache.page_size, _p(cache.pages), _p(q_out),
                                     int(cache.writes), _p(sc["error"]), _stream()), "linear_rope_kv_append")
    return True


@_dispatch("paged_attention")
def paged_attention(q, out, ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, softcap: float,
                    window: int | None, value_split: int = 0, keep_first: int = 0, sink: bool = False) -> None:
    """Causal (optionally windowed, softcapped) attention of every row of the step over its request's pages.
    bfloat16: rows of single-row requests run the split-KV decode kernel, the rest the prefill kernel, when the
    head size has an instance of them; the 32-bit path and other head sizes run the generic kernel.
    value_split = G > 0: every query head over every value head.  `out` has n_heads result heads, q n_heads / G heads and
    the pages G heads (n_kv_heads = G * G counts (key head, value head) pairs): result head h, of pair p = h // r with
    r = n_heads // n_kv_heads, is query head (p // G) * r + h % r over the keys of head p // G and the values of head p % G.
    keep_first = K > 0 (with a window): keys 0..K-1 stay visible behind the window, at their true positions.
    sink: one is added to the softmax's denominator (a key of score 0 that has no value)."""
    T = q.shape[0]
    keep_first = int(keep_first) if window else 0
    extras = (keep_first, int(bool(sink)))
    lib = library()
    table = ctx.block_tables[cache.group]
    pages = cache.pages
    common = (_p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size, n_heads, n_kv_heads, head_dim,
              _f(scale), _f(softcap), int(window or 0), int(value_split))
    n_dec = getattr(ctx, "n_dec_rows", 0)
    fast = (use_fast_attention and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16)
    if (keep_first or sink) and (value_split or not extras_on_fast_kernels or not decode_on_tensor_cores
                               or n_heads // n_kv_heads > 16):
        fast = False                                   # the generic kernel: every combination
    vs_splits = ctypes.c_int(0)
    own = decode_value_split_kernel if decode_value_split_kernel is not None else value_split >= 3
    if (fast and n_dec > 0 and value_split and softcap == 0.0 and own
            and lib.kf_attention_decode_vs_plan(n_dec, n_heads // value_split, value_split, head_dim,
                                                int(min(ctx.max_kv_len, window) if window else ctx.max_kv_len),
                                                ctypes.byref(vs_splits)) == 0):
        # one block per tile of 16 query heads and all value heads: scores once, keys and values read once per tile
        partial = _partial(q.device, T * n_heads * vs_splits.value * (head_dim + 4)) if vs_splits.value > 1 else None
        items = None if n_dec == T else ctx.dec_rows
        _check(lib.kf_attention_decode_vs(_p(q), _p(out), _p(pages), _p(items), n_dec, *common[:5], n_heads // value_split,
                                          value_split, head_dim, _f(scale), int(window or 0), vs_splits.value, _p(partial),
                                          _stream()), "attention (decode, every value head)")
        if vs_splits.value > 1:
            add_launches(1)
        if n_dec == T:
            return
        rest, n_rest = ctx.pre_rows, ctx.n_pre_rows
    elif fast and n_dec > 0 and lib.kf_attention_decode_supported(head_dim):
        ht, splits = ctypes.c_int(0), ctypes.c_int(0)
        max_keys = min(ctx.max_kv_len, window + keep_first) if window else ctx.max_kv_len
        group = n_heads // n_kv_heads
        if decode_on_tensor_cores and group <= 16:
            lib.kf_attention_decode_mma_plan(n_dec, n_heads, n_kv_heads, head_dim, int(max_keys), ctypes.byref(splits))
            n_counters = n_dec * n_kv_heads                      # ht stays 0: the tensor-core variant
        else:
            lib.kf_attention_decode_plan(n_dec, n_heads, n_kv_heads, head_dim, int(max_keys), ctypes.byref(ht), ctypes.byref(splits))
            n_counters = n_dec * n_kv_heads * -(-group // ht.value)
        sc = _dev_scratch(q.device)
        if n_counters > sc["counters"].numel():
            rest, n_rest = None, T
        else:
            partial = _partial(q.device, T * n_heads * splits.value * (head_dim + 4)) if splits.value > 1 else None
            items = None if n_dec == T else ctx.dec_rows
            _check(lib.kf_attention_decode(_p(q), _p(out), _p(pages), _p(items), n_dec, *common, ht.value,
                                           splits.value, _p(partial), _p(sc["counters"]), *extras, _stream()), "attention (decode)")
            if n_dec == T:
                return
            rest, n_rest = ctx.pre_rows, ctx.n_pre_rows
    elif fast and n_dec == 0 and getattr(ctx, "n_pre_rows", 0) == T:
        rest, n_rest = ctx.pre_rows, T
    else:
        rest, n_rest = None, T
    prompt_tiles = fast and rest is not None and n_rest == ctx.n_pre_rows and getattr(ctx, "n_tiles", 0) > 0
    if (prompt_tiles and prefill_on_tcgen05 and getattr(ctx, "n_wide", 0) > 0
            and lib.kf_attention_prefill_tc_supported(head_dim, cache.page_size, _p(q), _p(pages))):
        sc = _dev_scratch(q.device)
        max_keys = min(ctx.max_kv_len, window + 128 + -(-keep_first // 64) * 64) if window else ctx.max_kv_len
        run_tiles = ctypes.c_int(0)
        if prefill_plan_override is not None:
            parts, run_tiles = int(prefill_plan_override[0]), ctypes.c_int(int(prefill_plan_override[1]))
        else:
            parts = lib.kf_attention_prefill_tc_plan(ctx.n_wide, n_heads, int(max_keys), ctypes.byref(run_tiles)) if split_prompt_keys else 1
        partial = _partial(q.device, T * n_heads * parts * (head_dim + 4)) if parts > 1 else None
        _check(lib.kf_attention_prefill_tc(_p(q), _p(out), _p(pages), ctypes.c_long(pages.shape[0]), T, _p(ctx.wide_row0),
                                           _p(ctx.wide_nrows), ctx.n_wide, *common, _p(sc["error"]), parts, run_tiles.value,
                                           _p(partial), *extras, _stream()),
               "attention (prefill, tcgen05)")
        if parts > 1:
            add_launches(1)
        return
    if prompt_tiles and lib.kf_attention_prefill_supported(head_dim):
        _check(lib.kf_attention_prefill(_p(q), _p(out), _p(pages), _p(ctx.tile_row0), _p(ctx.tile_nrows), ctx.n_tiles,
                                        *common, *extras, _stream()), "attention (prefill)")
        return
    if fast and use_fast_attention:
        note_fallback(f"attention: head size {head_dim} or page size {cache.page_size} has no tensor-core kernel")
    _check(lib.kf_attention_generic(_p(q), _p(out), _dt(q), _p(pages), _dt(pages), _p(rest), *common, *extras, n_rest, _stream()),
           "attention (generic)")


# Whether the tensor-core attention kernels take `keep_first` and `sink`; False sends such launches to the generic kernel.
extras_on_fast_kernels = os.environ.get("KUNGFU_ATTENTION_EXTRAS_FAST", "1") != "0"

# Decode rows of value-split attention: True, the kernel that owns all value heads of a tile of query heads; False, the
# ordinary decode kernels (one block per pair of a key head and a value head); None, the former from three value heads on
# (at one or two the pairs are so few that the ordinary kernels, which need no merge launch, are faster).
decode_value_split_kernel = {"1": True, "0": False}.get(os.environ.get("KUNGFU_DECODE_VALUE_SPLIT", ""), None)
fuse_rope_into_decode = os.environ.get("KUNGFU_FUSE_ROPE", "1") != "0"   # False: rotation and append always run as their own kernel


def decode_attention_takes_qkv(ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether `rope_append_attend` can run this step's attention: every row is the single row of its request (a decode
    step), bfloat16 pages, and the tensor-core decode kernel has an instance for the head size and group."""
    if _override is not None or not (fuse_rope_into_decode and use_fast_attention and decode_on_tensor_cores):
        return False
    T = ctx.n_rows
    if T <= 0 or getattr(ctx, "n_dec_rows", 0) != T or cache is None or cache.pages.dtype != torch.bfloat16:
        return False
    if n_heads // n_kv_heads > 16 or not library().kf_attention_decode_supported(head_dim):
        return False
    return T * n_kv_heads <= _dev_scratch(cache.pages.device)["counters"].numel()


@_dispatch("rope_append_attend")
def rope_append_attend(qkv, cos, sin, rot: int, out, ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int,
                       scale: float, softcap: float, window: int | None) -> None:
    """For a decode step: rotate q and k, append k and v to the pages and attend, in the split-KV decode kernel itself
    (one launch instead of two).  qkv: 32-bit [T, (n_heads + 2 n_kv_heads) * head_dim]; out: bfloat16 [T, n_heads * head_dim]."""
    T = qkv.shape[0]
    lib = library()
    table = ctx.block_tables[cache.group]
    max_keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
    splits = ctypes.c_int(0)
    lib.kf_attention_decode_mma_plan(T, n_heads, n_kv_heads, head_dim, int(max_keys), ctypes.byref(splits))
    sc = _dev_scratch(qkv.device)
    partial = _partial(qkv.device, T * n_heads * splits.value * (head_dim + 4)) if splits.value > 1 else None
    _check(lib.kf_attention_decode_fused(_p(qkv), _p(cos), _p(sin), int(rot), int(cache.writes), _p(out), _p(cache.pages),
                                         None, T, _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1],
                                         cache.page_size, n_heads, n_kv_heads, head_dim, _f(scale), _f(softcap),
                                         int(window or 0), splits.value, _p(partial), _p(sc["counters"]), _stream()),
           "attention (decode, rotation and append inside)")


# ---- short convolutions, the q|k|v preparation of mixers that convolve and norm their heads, the state-space scan ----

_CONV_ACT = {None: 0, "none": 0, "silu": 1}


@_dispatch("short_conv")
def short_conv(proj, col0: int, in_bias, weight, out_bias, act, state, out, ctx, commit_inline: bool = False) -> bool:
    """out[t, c] = act(sum_j weight[c, j] * u_(t - taps + 1 + j)[c] + out_bias[c]) over the rows of every request of the step,
    u = proj[:, col0 + c] + in_bias[c]; rows before the step come from `state` [requests, taps - 1, C] (32-bit), zeros
    before the sequence's start.  `proj` and `out` are 32-bit.
    `commit_inline` (only for steps in which no request has more than one row): the kernel also moves the state on.
    Returns whether it did; if not, `short_conv_commit` has to run after every reader of the old state."""
    T = out.shape[0]
    C, taps = weight.shape
    inline = bool(commit_inline) and taps > 1
    _check(library().kf_short_conv(_p(proj), proj.shape[1], int(col0), _p(in_bias), _p(weight), _p(out_bias), _dt(weight), C,
                                   taps, _CONV_ACT[act], _p(state), _p(out), out.shape[1], _p(ctx.row_req),
                                   _p(ctx.req_row_start), _p(ctx.req_state_slot), T, int(inline), _stream()), "short_conv")
    return inline


@_dispatch("short_conv_commit")
def short_conv_commit(proj, col0: int, in_bias, n_channels: int, taps: int, state, ctx, w_dtype=None) -> None:
    """After every reader of the old state has been launched: state[slot] <- the last taps - 1 inputs of each request."""
    if taps <= 1:
        return
    dt = _dt(in_bias) if in_bias is not None else (BF16 if w_dtype == torch.bfloat16 else F32)
    _check(library().kf_short_conv_commit(_p(proj), proj.shape[1], int(col0), _p(in_bias), dt, int(n_channels), int(taps),
                                          _p(state), ctx.n_reqs, _p(ctx.req_row_start), _p(ctx.req_n_rows),
                                          _p(ctx.req_state_slot), _stream()), "short_conv_commit")


@_dispatch("qkv_prepare")
def qkv_prepare(proj, col0: int, in_bias, conv_w, conv_state, q_norm, k_norm, eps: float, cos, sin, rot: int,
                interleaved: bool, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, ctx, cache, q_out,
                commit_inline: bool = False) -> bool:
    """From the 32-bit q|k|v projection to the attention's operands: optional bias, short convolution (reading
    `conv_state`), per-head RMS norm of q and k, rotation (interleaved pairs or halves), q into `q_out`
    [T, n_heads * D] and k, v into the pages of `cache`, D = the pages' head size, tails zero.
    `commit_inline` (only for steps in which no request has more than one row): the kernel also moves the convolution's
    state on, when its sizes allow.  Returns whether it did; if not, `short_conv_commit` has to run afterwards."""
    T = q_out.shape[0]
    D = cache.pages.shape[-1]
    if q_out.shape[1] != n_heads * D:
        raise KernelError(f"qkv_prepare: q rows of {q_out.shape[1]} elements for {n_heads} heads of {D}")
    table = ctx.block_tables[cache.group]
    taps = conv_w.shape[1] if conv_w is not None else 1
    wdt = _dt(conv_w) if conv_w is not None else _dt(q_out)
    for w in (in_bias, q_norm, k_norm):
        if w is not None and _dt(w) != wdt:
            raise KernelError("qkv_prepare: bias, convolution and norm weights must share one element type")
    inline = bool(commit_inline and conv_w is not None and taps > 1 and conv_state is not None and
                  library().kf_qkv_prepare_commits_inline(proj.shape[1], int(col0), int(rot), int(interleaved), key_dim, value_dim, D))
    _check(library().kf_qkv_prepare(_p(proj), proj.shape[1], int(col0), _p(in_bias), _p(conv_w), taps, _p(conv_state),
                                    _p(q_norm), _p(k_norm), wdt, _f(eps), _p(cos), _p(sin), int(rot), int(interleaved),
                                    n_heads, n_kv_heads, key_dim, value_dim, D, _p(ctx.positions), _p(ctx.row_req),
                                    _p(ctx.req_row_start), _p(ctx.req_state_slot), _p(table), table.shape[1],
                                    cache.page_size, _p(cache.pages), _dt(cache.pages), _p(q_out), _dt(q_out),
                                    int(cache.writes), T, int(inline), _stream()), "qkv_prepare")
    return inline


@_dispatch("head_gate")
def head_gate(o, proj, gate_col0: int, n_heads: int, value_dim: int, head_dim: int, out, ctx, out_col0: int = 0,
              scale: float = 1.0) -> None:
    """out[t, out_col0 + h * value_dim + i] = o[t, h * head_dim + i] * sigmoid(proj[t, gate_col0 + h]) * scale; proj None:
    packing (and the factor) only.  `out` may be wider than the heads (the joined input of one output product)."""
    T = out.shape[0]
    _check(library().kf_head_gate(_p(o), _p(proj), proj.shape[1] if proj is not None else 0, int(gate_col0), n_heads,
                                  value_dim, head_dim, _p(out), _dt(out), _p(ctx.row_req), T, out.shape[1], int(out_col0),
                                  _f(scale), _stream()), "head_gate")


chunked_scan = True          # False: a long prompt's recurrence is walked by one block per (request, head, 32 columns) only
SCAN_CHUNK_ROWS = 256
SCAN_CHUNKED_FROM = 1024     # rows of a step from which the chunks are walked side by side ...
SCAN_CHUNKED_BLOCKS = 160    # ... if the plain walk would have at most this many blocks (about one per SM); with two per SM
                             # it is already the faster one (736 against 827 us at 128 heads x 64 x 128)


@_dispatch("ssm_scan")
def ssm_scan(xbc, proj, dt_col0: int, dt_bias, a_log, d_skip, state, y, heads: int, groups: int, head_dim: int,
             state_dim: int, ctx, writes: bool = True) -> None:
    """The state-space recurrence over the rows of every request of the step, from and into `state`
    [requests, heads, head_dim, state_dim] (32-bit): S = exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + d_skip x, with
    dt = softplus(proj[:, dt_col0 + h] + dt_bias[h]); xbc rows are [x | B | C] (32-bit).
    Steps of single rows run a kernel without staging; steps of a thousand rows and more whose requests are too few to
    fill the GPU are cut into chunks of 256 rows that are walked side by side (their start states follow from a first
    pass over the chunks): 435 against 590 us for one prompt of 2,048 tokens at 64 heads x 64 x 128; with two such
    prompts the plain walk is already the faster one."""
    T = xbc.shape[0]
    lib = library()
    single = bool(getattr(ctx, "decode_only", False))
    common = (_p(xbc), xbc.shape[1], _p(proj), proj.shape[1], int(dt_col0), _p(dt_bias), _p(a_log), _p(d_skip), _dt(a_log),
              _p(state), _p(y), heads, groups, head_dim, state_dim, ctx.n_reqs, _p(ctx.req_row_start), _p(ctx.req_n_rows),
              _p(ctx.req_state_slot), int(writes))
    few = ctx.n_reqs * heads * -(-head_dim // 32) <= SCAN_CHUNKED_BLOCKS
    if chunked_scan and not single and few and T >= SCAN_CHUNKED_FROM and hasattr(ctx, "buf"):
        n_chunks = T // SCAN_CHUNK_ROWS + ctx.n_reqs
        tab = ctx.buf("ssm_chunk_table", (5 * n_chunks + 2 * ctx.n_reqs,), torch.int32)
        chunk_state = ctx.buf("ssm_chunk_state", (n_chunks, heads, head_dim, state_dim), torch.float32)
        chunk_decay = ctx.buf("ssm_chunk_decay", (n_chunks, heads), torch.float32)
        _check(lib.kf_ssm_scan_chunked(*common, SCAN_CHUNK_ROWS, n_chunks, _p(tab), _p(chunk_state), _p(chunk_decay), _stream()),
               "ssm_scan (chunks side by side)")
        add_launches(3)
        return
    _check(lib.kf_ssm_scan(*common, int(single), _stream()), "ssm_scan")


@_dispatch("gated_group_norm")
def gated_group_norm(y, proj, z_col0: int, weight, eps: float, parts: int, out, ctx) -> None:
    """out = rms norm, in `parts` equal parts of the row, of y * silu(proj[:, z_col0:z_col0 + inner]), times weight."""
    T, inner = out.shape
    _check(library().kf_gated_group_norm(_p(y), _p(proj), proj.shape[1], int(z_col0), _p(weight), _dt(weight), _f(eps), inner,
                                         int(parts), _p(out), _dt(out), _p(ctx.row_req), T, _stream()), "gated_group_norm")


@_dispatch("add2_rmsnorm")
def add2_rmsnorm(a, b, x, *, next_weight=None, next_eps: float = 0.0, next_plus_one: bool = False, next_out=None) -> None:
    """x += a + b (b may be None), 32-bit; if next_out is given, next_out = rmsnorm(x) * g_next in the same pass."""
    T, H = x.shape
    _check(library().kf_add2_rmsnorm(_p(a), _p(b), _p(x), _p(next_weight), _dt(next_weight) if next_weight is not None else F32,
                                     _f(next_eps), int(next_plus_one), _p(next_out),
                                     _dt(next_out) if next_out is not None else F32, T, H, _stream()), "add2_rmsnorm")


# ---- norms in groups, the polynomial activation, attention whose heads' weights are mixed ---------------------------------

@_dispatch("group_rmsnorm")
def group_rmsnorm(x, weight, eps: float, groups: int, out, rows=None) -> None:
    """The row (x[rows[r]] if rows is given else x[r]) cut into `groups` equal parts, each divided by its own
    sqrt(mean(part^2) + eps), times weight."""
    n, H = out.shape
    _check(library().kf_group_rmsnorm(_p(x), _p(weight), _dt(weight), _f(eps), int(groups), _p(out), _dt(out), _p(rows), n, H,
                                      _stream()), "group_rmsnorm")


@_dispatch("add_group_rmsnorm")
def add_group_rmsnorm(branch, weight, eps: float, groups: int, residual, *, shift=None, next_weight=None, next_eps: float = 0.0,
                      next_out=None) -> None:
    """residual += group norm of branch (when branch is given); residual += shift, a constant row (when given);
    next_out = group norm of the residual with next_weight (when given).  One kernel; both norms cut rows alike."""
    T, H = residual.shape
    ws = [w for w in (weight, shift, next_weight) if w is not None]
    if len({w.dtype for w in ws}) > 1:
        raise KernelError("add_group_rmsnorm: weights and shift must share one element type")
    _check(library().kf_add_group_rmsnorm(_p(branch), _p(weight), _dt(ws[0]) if ws else F32, _f(eps), _p(residual), _p(shift),
                                          _p(next_weight), _f(next_eps), _p(next_out),
                                          _dt(next_out) if next_out is not None else F32, int(groups), T, H, _stream()),
           "add_group_rmsnorm")


@_dispatch("poly_norm")
def poly_norm(z, coef, eps: float, out) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e with (a, b, c, e) = coef and N(u) = u / sqrt(mean(u^2) + eps) over a row;
    z 32-bit [T, I]."""
    T, I = out.shape
    _check(library().kf_poly_norm(_p(z), _p(coef), _dt(coef), _f(eps), _p(out), _dt(out), T, I, _stream()), "poly_norm")


@_dispatch("rotate_norm_append")
def rotate_norm_append(proj, col0: int, cos, sin, rot: int, magnitude: float, unit_norm: bool, eps: float, n_heads: int,
                       n_kv_heads: int, key_dim: int, value_dim: int, ctx, cache, q_out) -> None:
    """From the 32-bit q|k|v projection (columns col0.. of proj) to the attention's operands: q and k turned in pairs
    (i, i + rot/2) by cos/sin * magnitude, then (unit_norm) divided by sqrt(mean(head^2) + eps); q into q_out, k and v
    into the pages of `cache`, heads of D = the pages' head size with zero tails."""
    T = q_out.shape[0]
    D = cache.pages.shape[-1]
    if q_out.shape[1] != n_heads * D or cache.pages.shape[2] != n_kv_heads:
        raise KernelError(f"rotate_norm_append: q rows of {q_out.shape[1]} and pages of {cache.pages.shape[2]} heads do not fit "
                          f"{n_heads} query heads and {n_kv_heads} stored heads of {D}")
    table = ctx.block_tables[cache.group]
    _check(library().kf_rotate_norm_append(_p(proj), proj.shape[1], int(col0), _p(cos), _p(sin), int(rot), _f(magnitude),
                                           int(bool(unit_norm)), _f(eps), n_heads, n_kv_heads, key_dim, value_dim, D,
                                           _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size,
                                           _p(cache.pages), _dt(cache.pages), _p(q_out), _dt(q_out), int(cache.writes), T,
                                           _stream()), "rotate_norm_append")


@_dispatch("head_mix_gate")
def head_mix_gate(o, mix, proj, gate_col0: int, n_heads: int, n_kv_heads: int, value_dim: int, head_dim: int, out, ctx) -> None:
    """out[t, h * value_dim + e] = sigmoid(proj[t, gate_col0 + h * value_dim + e]) * sum_g mix[h, g] * o[t, wide(g, kv(h)), e]:
    `o` holds, for every query head g and value head c, head g's weighted sum over the values of c (the result of
    `paged_attention(value_split=n_kv_heads)`), wide(g, c) = ((g // r) * n_kv_heads + c) * r + g % r with
    r = n_heads / n_kv_heads, kv(h) = h // r.  mix None: no mixing (o holds n_heads heads); proj None: no gate."""
    T = out.shape[0]
    _check(library().kf_head_mix_gate(_p(o), _p(mix), _dt(mix) if mix is not None else F32, _p(proj),
                                      proj.shape[1] if proj is not None else 0, int(gate_col0), n_heads, n_kv_heads, value_dim,
                                      head_dim, _p(out), _dt(out), _p(ctx.row_req), T, _stream()), "head_mix_gate")


# ---- the gated delta rule, latent attention, layer scales, per-token side inputs, mixtures of experts ------------------

@_dispatch("linear_cols")
def linear_cols(base, col0: int, weight, out) -> None:
    """out[T, N] = base[:, col0:col0 + K] . weight[N, K]^T, `base` a wider 32-bit matrix (the result of a stacked
    projection): the second half of a factored projection, in 32-bit FMA arithmetic whatever the weights' type."""
    T, N = out.shape
    K = weight.shape[1]
    if base.dtype != torch.float32 or weight.shape[0] != N or base.shape[0] != T:
        raise KernelError(f"linear_cols: base{tuple(base.shape)} {base.dtype} w{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    _check(library().kf_linear_simt_cols(_p(base), ctypes.c_long(base.shape[1]), ctypes.c_long(col0), _p(weight), _dt(weight),
                                         _p(out), _dt(out), T, N, K, _stream()), "linear_cols")


@_dispatch("delta_rule")
def delta_rule(qkv, q0: int, k0: int, v0: int, beta, beta0: int, decay, decay0: int, per_channel: bool, dt_bias, a_log,
               state, out, heads: int, kv_heads: int, dim: int, vdim: int, ctx, writes: bool = True) -> None:
    """The gated delta rule over the rows of every request of the step, from and into `state` [requests, heads, dim, vdim]
    (32-bit): S <- g S (g per head, or per head and key channel = row of S); u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  q, k, v are column ranges of `qkv` (32-bit, after convolution and activation), made unit vectors per head
    here (q also times dim^-1/2); beta = sigmoid(beta[:, beta0 + h]); g = exp(-exp(a_log[h]) softplus(decay[:, decay0 + ...] +
    dt_bias)).  Query/key head of head h: h // (heads // kv_heads).  out: 32-bit [rows, heads * vdim]."""
    T = out.shape[0]
    lib = library()
    # what does not depend on the state (unit vectors, decays, beta) is computed for all rows first, into scratch
    prep = ctx.buf("delta_prep", (T * heads * lib.kf_delta_rule_row_floats(int(dim)),), torch.float32)
    small = ctx.buf("delta_small", (T * heads * 2,), torch.float32)
    _check(lib.kf_delta_rule(_p(qkv), qkv.shape[1], int(q0), int(k0), int(v0), _p(beta), beta.shape[1], int(beta0),
                             _p(decay), decay.shape[1], int(decay0), int(bool(per_channel)), _p(dt_bias), _p(a_log),
                             _dt(a_log), _p(state), _p(out), out.shape[1], heads, kv_heads, dim, vdim, ctx.n_reqs,
                             _p(ctx.req_row_start), _p(ctx.req_n_rows), _p(ctx.req_state_slot), int(writes), T, _p(prep),
                             _p(small), _stream()), "delta_rule")
    add_launches(1)


_GATE_ACT = {"silu": 0, "sigmoid": 1}


@_dispatch("head_norm_gate")
def head_norm_gate(o, weight, eps: float, gate, gate0: int, act: str, out, heads: int, vdim: int, out_col0: int = 0,
                   scale: float = 1.0) -> None:
    """out[t, out_col0 + h * vdim + :] = o[t, h, :] / rms(o[t, h, :]) * weight * act(gate[t, gate0 + h * vdim + :]) * scale;
    act silu or sigmoid.  `weight` holds vdim numbers (shared by the heads) or heads * vdim (one vector per head); `out` may
    be wider than the heads (the joined input of one output product)."""
    T = out.shape[0]
    if weight.numel() not in (vdim, heads * vdim):
        raise KernelError(f"head_norm_gate: {weight.numel()} weights for {heads} heads of {vdim}")
    w_stride = vdim if (weight.numel() == heads * vdim and heads > 1) else 0
    _check(library().kf_head_norm_gate(_p(o), _p(weight), _dt(weight), _f(eps), _p(gate), gate.shape[1], int(gate0),
                                       _GATE_ACT[act], _p(out), _dt(out), heads, vdim, T, w_stride, out.shape[1], int(out_col0),
                                       _f(scale), _stream()), "head_norm_gate")


@_dispatch("latent_append")
def latent_append(proj, c0: int, rank: int, weight, eps: float, ctx, cache) -> None:
    """c = rms_norm(proj[:, c0:c0 + rank]) * weight, written as the key row AND the value row of the single key/value head
    of `cache` (head size D >= rank, tails zero) at every row's position."""
    T = proj.shape[0]
    table = ctx.block_tables[cache.group]
    D = cache.pages.shape[-1]
    _check(library().kf_latent_append(_p(proj), proj.shape[1], int(c0), int(rank), _p(weight), _dt(weight), _f(eps),
                                      _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size,
                                      _p(cache.pages), _dt(cache.pages), D, T, _stream()), "latent_append")


@_dispatch("latent_rope_append")
def latent_rope_append(proj, c0: int, rank: int, rot: int, weight, eps: float, cos, sin, interleaved: bool, magnitude: float,
                       q, q0: int, n_heads: int, q_dim: int, ctx, cache) -> None:
    """The latent with a rotated key part: c = rms_norm(proj[:, c0:c0 + rank]) * weight goes to the key row and the value
    row of the single stored head as `latent_append` does; the `rot` columns after it are turned by the rows' angles and
    filed behind c in the key row (zeros in the value row).  The last `rot` elements of every head of the 32-bit query
    matrix q [T, q0 + n_heads * (q_dim + rot) ..] are turned in place by the same angles."""
    T = proj.shape[0]
    table = ctx.block_tables[cache.group]
    D = cache.pages.shape[-1]
    _check(library().kf_latent_rope_append(_p(proj), proj.shape[1], int(c0), int(rank), int(rot), _p(weight), _dt(weight),
                                           _f(eps), _p(cos), _p(sin), int(bool(interleaved)), _f(magnitude), _p(q), q.shape[1],
                                           int(q0), int(n_heads), int(q_dim), _p(ctx.positions), _p(ctx.row_req), _p(table),
                                           table.shape[1], cache.page_size, _p(cache.pages), _dt(cache.pages), D,
                                           int(cache.writes), T, _stream()), "latent_rope_append")


@_dispatch("cols_rmsnorm")
def cols_rmsnorm(x, c0: int, weight, eps: float, out) -> None:
    """out[t, :] = rms_norm(x[t, c0:c0 + n]) * weight, n = weight's length; x 32-bit."""
    T, n = out.shape
    _check(library().kf_cols_rmsnorm(_p(x), x.shape[1], int(c0), int(n), _p(weight), _dt(weight), _f(eps), _p(out), _dt(out), T,
                                     _stream()), "cols_rmsnorm")


@_dispatch("rownorm_rope_append")
def rownorm_rope_append(proj, col0: int, bias, q_norm, k_norm, eps: float, cos, sin, rot: int, interleaved: bool,
                        magnitude: float, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, ctx, cache, q_out,
                        v_mix=None, v_shared=None, v_mode: int = 0) -> None:
    """From the 32-bit [q | k | v] columns of `proj` to the attention's operands: optional bias, RMS norm of q and of k
    over ALL their heads at once (weights of n_heads * key_dim and n_kv_heads * key_dim; None: no norm), rotation of the
    first `rot` elements of every head (interleaved pairs or halves), q into `q_out` [T, n_heads * D], k and v into the
    pages of `cache`.  v_mode 1: the biased v is also written to `v_shared` [T, n_kv_heads * value_dim] (32-bit);
    v_mode 2: v <- (1 - v_mix) v + v_mix v_shared before it is filed (`v_mix`: one number on the device)."""
    T = q_out.shape[0]
    D = cache.pages.shape[-1]
    if q_out.shape[1] != n_heads * D:
        raise KernelError(f"rownorm_rope_append: q rows of {q_out.shape[1]} elements for {n_heads} heads of {D}")
    table = ctx.block_tables[cache.group]
    ws = [w for w in (bias, q_norm, k_norm, v_mix) if w is not None]
    wdt = _dt(ws[0]) if ws else _dt(q_out)
    if any(_dt(w) != wdt for w in ws):
        raise KernelError("rownorm_rope_append: bias, norm weights and the mixing number must share one element type")
    _check(library().kf_rownorm_rope_append(_p(proj), proj.shape[1], int(col0), _p(bias), _p(q_norm), _p(k_norm), wdt, _f(eps),
                                            _p(cos), _p(sin), int(rot), int(bool(interleaved)), _f(magnitude), n_heads,
                                            n_kv_heads, key_dim, value_dim, D, _p(v_mix), _p(v_shared), int(v_mode),
                                            _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size,
                                            _p(cache.pages), _dt(cache.pages), _p(q_out), _dt(q_out), int(cache.writes), T,
                                            _stream()), "rownorm_rope_append")


MLSTM_COLUMNS = 16          # value columns a block of the matrix memory's walk owns


def mlstm_norm_width(dim: int, vdim: int) -> int:
    """Numbers per head in the matrix memory's second state: a copy of n (dim numbers) per block of MLSTM_COLUMNS value
    columns, then m and three unused numbers."""
    return -(-int(vdim) // MLSTM_COLUMNS) * int(dim) + 4


@_dispatch("mlstm")
def mlstm(proj, q0: int, k0: int, v0: int, i0: int, f0: int, bias_i, bias_f, cap: float, memory, norm_state, out, heads: int,
          dim: int, vdim: int, ctx, writes: bool = True) -> None:
    """The matrix memory with exponential gates over the rows of every request of the step, from and into `memory`
    [requests, heads, dim, vdim] and `norm_state` [requests, heads, mlstm_norm_width(dim, vdim)] (one copy of n per 16 value
    columns, each owned by the block that walks those columns, then the running maximum m), both 32-bit.  q, k, v and the raw gates are column ranges of `proj` (32-bit); q is
    multiplied by dim^-1/2.  gi = cap tanh((zi + bias_i) / cap), gf = logsigmoid(cap tanh((zf + bias_f) / cap));
    m' = max(gf + m, gi); S' = exp(gf + m - m') S + exp(gi - m') k v^T, n' likewise with k;
    out = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6), 32-bit [rows, heads * vdim]."""
    T = out.shape[0]
    lib = library()
    m_at = mlstm_norm_width(dim, vdim) - 4
    if norm_state.shape[2] != m_at + 4:
        raise KernelError(f"mlstm: norm_state rows of {norm_state.shape[2]} numbers, expected {m_at + 4}")
    gates = ctx.buf("mlstm_gates", (T * heads * 4,), torch.float32)
    wdt = _dt(bias_i) if bias_i is not None else F32
    _check(lib.kf_mlstm_gates(_p(proj), proj.shape[1], int(i0), int(f0), _p(bias_i), _p(bias_f), wdt, _f(cap), _p(norm_state),
                              norm_state.shape[2], int(m_at), _p(gates), heads, ctx.n_reqs, _p(ctx.req_row_start),
                              _p(ctx.req_n_rows), _p(ctx.req_state_slot), int(writes), _stream()), "mlstm (gates)")
    _check(lib.kf_mlstm_scan(_p(proj), proj.shape[1], int(q0), int(k0), int(v0), _p(gates), _p(memory), _p(norm_state),
                             norm_state.shape[2], _p(out), heads, dim, vdim, _f(float(dim) ** -0.5), ctx.n_reqs,
                             _p(ctx.req_row_start), _p(ctx.req_n_rows), _p(ctx.req_state_slot), int(writes), _stream()),
           "mlstm (walk)")


@_dispatch("weighted_sum2")
def weighted_sum2(a, sa: float, b, sb: float, out) -> None:
    """out = sa * a + sb * b (32-bit)."""
    _check(library().kf_weighted_sum2(_p(a), _f(sa), _p(b), _f(sb), _p(out), ctypes.c_long(out.numel()), _stream()),
           "weighted_sum2")


@_dispatch("convert")
def convert(src, dst) -> None:
    """dst = src in dst's element type (32-bit <-> bfloat16)."""
    _check(library().kf_convert(_p(src), _dt(src), _p(dst), _dt(dst), ctypes.c_long(src.numel()), _stream()), "convert")


@_dispatch("repeat_rows")
def repeat_rows(a, b, parts: int, out_a, out_b) -> None:
    """out_a[t * parts + j] = a[t], out_b likewise (int32): a step's positions and requests for rows that are presented
    to a kernel as `parts` rows each."""
    T = a.shape[0]
    _check(library().kf_repeat_rows(_p(a), _p(b), _p(out_a), _p(out_b), T, int(parts), _stream()), "repeat_rows")


def _grouped(x, x_off, ldx, x_gstride, row_index, row_div, w, w_gstride, out, o_off, ldo, o_gstride, tiles, max_tiles,
             n_groups, T, N, K, gated, limit, what, row_scale=None):
    tg, tr, tn, nt = tiles if tiles is not None else (None, None, None, None)
    L = ctypes.c_long
    _check(library().kf_grouped_linear(_p(x), _dt(x), L(x_off), L(ldx), L(x_gstride), _p(row_index), int(row_div), _p(w),
                                       _dt(w), L(w_gstride), _p(out), _dt(out), L(o_off), L(ldo), L(o_gstride), _p(tg),
                                       _p(tr), _p(tn), _p(nt), int(max_tiles), int(n_groups), int(T), int(N), int(K),
                                       int(gated), _f(limit), _p(row_scale), _stream()), what)


def grouped_on_tensor_cores(on: bool) -> None:
    """False: grouped products (per-head maps, experts) with bfloat16 weights run the generic 32-bit FMA kernel too
    (tests reach it that way)."""
    library().kf_grouped_use_tensor_cores(int(bool(on)))


@_dispatch("head_linear")
def head_linear(x, col0: int, weight, out) -> None:
    """A linear map per head: out[t, h * O + o] = sum_i x[t, col0 + h * I + i] * weight[h, o, i]; weight [heads, O, I],
    out [rows, heads * O]; x may be wider than heads * I (a column range of a stacked projection's result)."""
    H, O, I = weight.shape
    T = out.shape[0]
    if out.shape[1] != H * O or x.shape[1] < col0 + H * I:
        raise KernelError(f"head_linear: x{tuple(x.shape)} from column {col0}, weight{tuple(weight.shape)}, out{tuple(out.shape)} do not agree")
    _grouped(x, col0, x.shape[1], I, None, 1, weight, O * I, out, 0, out.shape[1], O, None, 0, H, T, O, I, 0, 0.0, "head_linear")


@_dispatch("moe_route")
def moe_route(logits, correction, groups: int, keep: int, top: int, scale: float, ids, weights, *, score: str = "sigmoid",
              group_rank: str = "best_two", normalize: bool = True) -> None:
    """For every row of 32-bit router logits [T, E]: s = sigmoid(logits) (or, score 'softmax', the softmax over all
    experts); the choice is made on s + correction, among the experts of the `keep` groups (of `groups` equal groups of
    neighbours) whose two largest choice scores sum highest (group_rank 'best': whose largest is highest);
    ids [T, top] int32 = the `top` largest; weights [T, top] = s of the chosen * scale, divided by their sum + 1e-20
    when `normalize`."""
    T, E = logits.shape
    if score not in ("sigmoid", "softmax") or group_rank not in ("best_two", "best"):
        raise KernelError(f"moe_route: score {score!r} / group_rank {group_rank!r} are not known")
    _check(library().kf_moe_route(_p(logits), _p(correction), _dt(correction) if correction is not None else F32, T, E,
                                  int(groups), int(keep), int(top), _f(scale), int(score == "softmax"),
                                  int(group_rank == "best"), int(bool(normalize)), _p(ids), _p(weights), _stream()), "moe_route")


@_dispatch("moe_plan")
def moe_plan(ids, n_experts: int, ctx) -> dict:
    """Lay the (token, choice) pairs of `ids` [T, top] out expert by expert.  Returns the device arrays the grouped
    products and the combination read: sorted_pair, inverse, and the list of 64-row tiles per expert."""
    T, top = ids.shape
    P = T * top
    max_tiles = P // 64 + n_experts
    plan = {"pairs": P, "top": top, "max_tiles": max_tiles,
            "sorted_pair": ctx.buf("moe_sorted", (P,), torch.int32), "inverse": ctx.buf("moe_inverse", (P,), torch.int32),
            "tile_group": ctx.buf("moe_tile_group", (max_tiles,), torch.int32),
            "tile_row0": ctx.buf("moe_tile_row0", (max_tiles,), torch.int32),
            "tile_nrows": ctx.buf("moe_tile_nrows", (max_tiles,), torch.int32),
            "n_tiles": ctx.buf("moe_n_tiles", (1,), torch.int32)}
    _check(library().kf_moe_plan(_p(ids), P, int(n_experts), _p(plan["sorted_pair"]), _p(plan["inverse"]), _p(plan["tile_group"]),
                                 _p(plan["tile_row0"]), _p(plan["tile_nrows"]), _p(plan["n_tiles"]), _stream()), "moe_plan")
    return plan


@_dispatch("moe_linear")
def moe_linear(x, plan: dict, weight, out, *, gather: bool, gated: bool = False, limit: float = 0.0,
               activation: str = "clamped_swish", row_scale=None) -> None:
    """out[r] = x_r . weight[e(r)]^T for every sorted pair r of the plan, e(r) its expert; weight [E, N (or 2N: gate rows
    then up rows, when gated), K].  `gather`: x holds one row per TOKEN and pair r reads the row of its token; otherwise
    x holds one row per sorted pair.  gated: out = the clamped gated activation of (gate, up) with `limit`, or, with
    activation 'silu', gate * sigmoid(gate) * up.  `row_scale` [T, top] (32-bit, gathered gated products only): gate and
    up of a pair are multiplied by its number before the activation, which is the expert applied to the scaled input."""
    if row_scale is not None and not (gated and gather):
        raise KernelError("moe_linear: a factor per pair is taken by gathered gated products only")
    if gated and activation not in ("clamped_swish", "silu"):
        raise KernelError(f"moe_linear: gated activation {activation!r} is not one of clamped_swish, silu")
    E, NW, K = weight.shape
    N = NW // 2 if gated else NW
    if out.shape[0] != plan["pairs"] or out.shape[1] != N or x.shape[1] != K:
        raise KernelError(f"moe_linear: x{tuple(x.shape)} weight{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    tiles = (plan["tile_group"], plan["tile_row0"], plan["tile_nrows"], plan["n_tiles"])
    _grouped(x, 0, K, 0, plan["sorted_pair"] if gather else None, plan["top"] if gather else 1, weight, NW * K, out, 0, N, 0,
             tiles, plan["max_tiles"], E, plan["pairs"], N, K, (2 if activation == "silu" else 1) if gated else 0, limit, "moe_linear", row_scale=row_scale)


@_dispatch("moe_combine")
def moe_combine(expert_out, plan: dict, weights, shared, y) -> None:
    """y[t] = sum_j weights[t, j] * expert_out[inverse[t * top + j]] (+ shared[t]), 32-bit, j ascending; `weights` None:
    every weight is one."""
    T, W = y.shape
    _check(library().kf_moe_combine(_p(expert_out), _p(plan["inverse"]), _p(weights), _p(shared), _p(y), T, W, plan["top"],
                                    _stream()), "moe_combine")


@_dispatch("scale_add_rmsnorm")
def scale_add_rmsnorm(a, scale, x, *, next_weight=None, next_eps: float = 0.0, next_plus_one: bool = False, next_out=None,
                      copy_out=None) -> None:
    """x += a * scale (one factor per column), 32-bit; next_out = rmsnorm(x) * g_next and copy_out = x (in its own element
    type) in the same pass when given."""
    T, H = x.shape
    ref = next_out if next_out is not None else copy_out
    if next_out is not None and copy_out is not None and next_out.dtype != copy_out.dtype:
        raise KernelError("scale_add_rmsnorm: next_out and copy_out must share one element type")
    if next_weight is not None and next_weight.dtype != scale.dtype:
        raise KernelError("scale_add_rmsnorm: the scale and the next norm's weight must share one element type")
    _check(library().kf_scale_add_rmsnorm(_p(a), _p(scale), _dt(scale), _p(x), _p(next_weight), _f(next_eps), int(next_plus_one),
                                          _p(next_out), _p(copy_out), _dt(ref) if ref is not None else F32, T, H, _stream()),
           "scale_add_rmsnorm")


@_dispatch("side_gate")
def side_gate(gate, tokens, table, col0: int, out) -> None:
    """out[t, j] = gelu_tanh(gate[t, j]) * table[tokens[t], col0 + j]; gate 32-bit [T, dim]."""
    T, dim = out.shape
    _check(library().kf_side_gate(_p(gate), _p(tokens), _p(table), _dt(table), table.shape[1], int(col0), _p(out), _dt(out),
                                  T, dim, _stream()), "side_gate")


@_dispatch("activation")
def activation_(x, out, act: str) -> None:
    """out = act(x), x 32-bit."""
    _check(library().kf_activation(_p(x), _p(out), _dt(out), ctypes.c_long(x.numel()), _ACT[act], _stream()), "activation")


@_dispatch("argmax")
def argmax(logits, out) -> None:
    """out[r] = index of the first maximum of logits[r, :] (int32)."""
    rows, V = logits.shape
    sc = _dev_scratch(logits.device)
    if "argmax" not in sc or sc["argmax"].numel() < rows * 128:
        if "argmax" in sc:
            sc["retired"].append(sc["argmax"])
        sc["argmax"] = torch.empty(max(rows, 64) * 128, dtype=torch.float32, device=logits.device)
    _check(library().kf_argmax(_p(logits), _p(out), rows, V, _p(sc["argmax"]), _stream()), "argmax")


def _sample_scratch(device, rows: int, V: int, full: bool) -> dict:
    lib = library()
    sc = _dev_scratch(device)
    n_slices = lib.kf_sample_slices(V)
    need = rows * n_slices
    if sc.get("sample_rows", 0) < need:
        for k in ("sample_keys", "sample_stats", "sample_flags"):
            if k in sc:
                sc["retired"].append(sc[k])
        cap = max(need, 64 * n_slices)
        sc["sample_keys"] = torch.empty(cap * 64, dtype=torch.int64, device=device)
        sc["sample_stats"] = torch.empty(cap * 2, dtype=torch.float32, device=device)
        sc["sample_flags"] = torch.zeros(max(rows, 64) * 2, dtype=torch.int32, device=device)
        sc["sample_rows"] = cap
    if sc["sample_flags"].numel() < rows:
        sc["retired"].append(sc["sample_flags"])
        sc["sample_flags"] = torch.zeros(rows * 2, dtype=torch.int32, device=device)
    if full and sc.get("sample_pen_n", 0) < rows * V:
        if "sample_pen" in sc:
            sc["retired"].append(sc["sample_pen"])
        sc["sample_pen"] = torch.empty(rows * V, dtype=torch.float32, device=device)
        sc["sample_pen_n"] = rows * V
    return sc


@_dispatch("sample")
def sample(logits, states, out_ids, *, logit_rows=None, row_req=None, req_slot=None, whole_ranking: bool = False,
           cand_ids=None, cand_vals=None, cand_lse=None) -> None:
    """The end of a step, on the device: out_ids[i] = the token row i of `logits` yields under the rules, generator and
    recent tokens of its request's state (`states` [requests, STATE_WORDS] int32, see sampling/sampler.py), which the
    kernels update.  The request of row i is req_slot[row_req[logit_rows[i]]] (each map None for the identity; rows of
    a negative request are skipped).  `whole_ranking`: some request's rules reach below the 64th candidate (top_k of 0
    or above 64 at a temperature above 0); one more kernel then runs.  cand_*: also write the ranked candidates."""
    rows, V = logits.shape
    sc = _sample_scratch(logits.device, rows, V, whole_ranking)
    k = 0 if cand_ids is None else cand_ids.shape[1]
    _check(library().kf_sample(_p(logits), rows, V, _p(sc["sample_keys"]), _p(sc["sample_stats"]), _p(cand_ids), _p(cand_vals),
                               _p(cand_lse), k, _p(logit_rows), _p(row_req), _p(req_slot), _p(states), _p(out_ids),
                               _p(sc["sample_flags"]), _p(sc["sample_pen"]) if whole_ranking else None,
                               int(whole_ranking), _stream()), "sample")
    add_launches(2 if whole_ranking else 1)


@_dispatch("topk_lse")
def topk_lse(logits, k: int, out_ids, out_vals, out_lse) -> None:
    """Top-k ids (falling value, lower id first among equals), their values, and the row's log-sum-exp; k <= 64."""
    rows, V = logits.shape
    if k < 1 or k > 64 or k > V:
        raise KernelError(f"topk_lse: k = {k} is not in 1..min(64, {V})")
    sc = _sample_scratch(logits.device, rows, V, False)
    _check(library().kf_sample(_p(logits), rows, V, _p(sc["sample_keys"]), _p(sc["sample_stats"]), _p(out_ids), _p(out_vals),
                               _p(out_lse), k, None, None, None, None, None, None, None, 0, _stream()), "topk_lse")
    add_launches(1)


def device_arch() -> int:
    return int(library().kf_device_arch())

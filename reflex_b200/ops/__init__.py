"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, layout), allocates the
output, and launches on torch's current stream, so the calls order with the
library matrix products and can be captured into a CUDA graph.  Sizes a kernel
does not take are refused with an error that names them.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..errors import CudaError, InvalidInput
import os as _os

from . import native, workspace
from .workspace import new as _new

F32, BF16 = 0, 1


def launch_count() -> int:
    """Kernels of this library launched directly so far (graph replays are
    counted by the engine, which knows how many a captured step holds)."""
    return native.LAUNCHES


def dt_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise InvalidInput(f"kernels take float32 or bfloat16, got {dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: Optional[torch.Tensor], name: str, dtype=None) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise CudaError(f"{name} must live on the GPU (there is no CPU path)")
    if not t.is_contiguous():
        raise InvalidInput(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise InvalidInput(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


# ---------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, scale: float, err_flag: torch.Tensor) -> torch.Tensor:
    """hidden[r] = table[ids[r]] * scale, as float32 [R, H]."""
    V, H = table.shape
    R = ids.numel()
    out = _new((R, H), torch.float32, table.device, keep=True)  # the residual stream: lives for the whole step
    st = native.lib().rfx_embed(
        _chk(table, "table"), dt_code(table.dtype), _chk(ids, "ids", torch.int32), R, H, V,
        float(scale), out.data_ptr(), _chk(err_flag, "err_flag", torch.int32), _stream())
    native.check(st, "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, update_residual: bool = True,
            rows: Optional[torch.Tensor] = None, weight_offset: float = 0.0,
            want_out: bool = True) -> Optional[torch.Tensor]:
    """RMSNorm of the float32 residual stream `x` [R, H], with the residual add
    fused in: t = x (+ delta); x <- t (if `update_residual`, in place);
    returns t * rsqrt(mean(t^2) + eps) * (weight_offset + weight) in
    `out_dtype`.  With `rows` only those rows are read and the output has
    `len(rows)` rows (the residual is then left alone)."""
    R, H = x.shape
    _chk(x, "x", torch.float32)
    r_out = R if rows is None else rows.numel()
    out = _new((r_out, H), out_dtype, x.device) if want_out else None
    x_out = x if (delta is not None and update_residual and rows is None) else None
    st = native.lib().rfx_rmsnorm(
        x.data_ptr(), _chk(delta, "delta"), dt_code(delta.dtype) if delta is not None else 0,
        x_out.data_ptr() if x_out is not None else 0, _chk(weight, "weight", torch.float32),
        float(eps), float(weight_offset), out.data_ptr() if out is not None else 0,
        dt_code(out_dtype), _chk(rows, "rows", torch.int32), r_out, H, _stream())
    native.check(st, f"rmsnorm (H={H})")
    return out


def add_(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a += b with a float32."""
    _chk(a, "a", torch.float32)
    st = native.lib().rfx_add(a.data_ptr(), _chk(b, "b"), dt_code(b.dtype), a.numel(), _stream())
    native.check(st, "add")
    return a


def swiglu(gate_up: torch.Tensor, alternating: bool = False) -> torch.Tensor:
    """[R, 2I] -> silu(gate) * up, [R, I].  A row holds the gates in its first
    half and the ups in its second, or (`alternating`) gate_i at 2i and up_i at
    2i + 1."""
    R, two_i = gate_up.shape
    I = two_i // 2
    out = _new((R, I), gate_up.dtype, gate_up.device)
    st = native.lib().rfx_swiglu(_chk(gate_up, "gate_up"), out.data_ptr(), dt_code(gate_up.dtype),
                                 R, I, 1 if alternating else 0, _stream())
    native.check(st, "swiglu")
    return out


# -------------------------------------------------------------------- linear
def _env_int(name: str, default: int, lo: int = 0, hi: int = 1 << 30) -> int:
    """A run-time switch read once from the environment; a bad value is an
    `InvalidInput`, as the reference treats its own switches
    (src/model/kernels.rs:244-259)."""
    raw = _os.environ.get(name)
    if raw is None or raw == "":
        return default
    try:
        v = int(raw)
    except ValueError:
        raise InvalidInput(f"{name} must be an integer, got {raw!r}") from None
    if not (lo <= v <= hi):
        raise InvalidInput(f"{name} must be between {lo} and {hi}, got {v}")
    return v


def _env_flag(name: str, default: bool) -> bool:
    raw = _os.environ.get(name)
    if raw is None or raw == "":
        return default
    if raw not in ("0", "1"):
        raise InvalidInput(f"{name} must be 0 or 1, got {raw!r}")
    return raw == "1"


# `REFLEX_PREFILL_PROFILE=1`: CUDA events at phase marks of every eager step
# (embed, norm, qkv_gemm, norm_rope, attn, o_proj, ffn_gate_up, ffn_down, head, and the
# further phases of other mixers and feed-forwards under their own names),
# totals per phase printed to stderr after the step; a no-op when off and
# inside graph capture (src/model/prefill_profile.rs:1-18, 26-59).
PROFILE = _env_flag("REFLEX_PREFILL_PROFILE", False)
_prof_events: list = []
LAST_PROFILE: dict = {}  # phase -> ms of the last reported step, for callers that want numbers, not lines


def prof_mark(name: str) -> None:
    if not PROFILE or torch.cuda.is_current_stream_capturing():
        return
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    _prof_events.append((name, ev))


def prof_report(label: str) -> None:
    """Waits for the device and prints, per phase, the time between each mark
    and the one before it, summed over the step."""
    import sys

    if not PROFILE or len(_prof_events) < 2:
        _prof_events.clear()
        return
    torch.cuda.synchronize()
    totals, order = {}, []
    for (_, e0), (name, e1) in zip(_prof_events, _prof_events[1:]):
        if name not in totals:
            totals[name] = 0.0
            order.append(name)
        totals[name] += e0.elapsed_time(e1)
    whole = _prof_events[0][1].elapsed_time(_prof_events[-1][1])
    LAST_PROFILE.clear()
    LAST_PROFILE.update(totals, total=whole)
    for name in order:
        print(f"REFLEX_PREFILL_PROFILE step={label} phase={name} ms={totals[name]:.3f}", file=sys.stderr)
    print(f"REFLEX_PREFILL_PROFILE step={label} phase=total ms={whole:.3f}", file=sys.stderr)
    _prof_events.clear()


GEMV_MAX_ROWS = _env_int("REFLEX_B200_GEMV_MAX_ROWS", 64, 0, 64)  # up to here the weight-streaming tensor-core kernel runs

_ERR = {}


def device_error_word(device) -> torch.Tensor:
    """One int32 word per device that kernels with bounded waits set to a
    non-zero code when a wait ran out."""
    key = torch.device(device).index or 0
    if key not in _ERR:
        _ERR[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _ERR[key]


def check_device_errors(device="cuda:0") -> None:
    """Synchronises; raises if a kernel reported that a bounded wait ran out."""
    code = int(device_error_word(device).item())
    if code:
        device_error_word(device).zero_()
        raise CudaError(f"a kernel reported an error (code {code}: a bounded wait that ran out, or a token "
                        f"id outside the vocabulary); the step's results are not valid")


def wait_probe(limit_ns: int, device="cuda:0") -> None:
    """Launches one block that waits, for at most `limit_ns` (clamped to a
    second), on a barrier nothing signals: the bounded wait runs out and the
    kernel records it in the device's error word, as the tensor-core kernels do
    when a copy or a product never arrives."""
    st = native.lib().rfx_wait_probe(int(limit_ns), device_error_word(device).data_ptr(), _stream())
    native.check(st, "wait_probe")


class NormedInput:
    """Rows that still await their RMSNorm factor: `hb` = bfloat16(h * norm
    weight) and `ssq[r][p]`, `n_part` partial sums of squares of h's row r.  The product
    that consumes them multiplies its row r by 1 / sqrt(sum_p ssq[r][p] / size +
    eps), which is the same as normalising first.  Made by `gemm_tc_residual`."""

    def __init__(self, hb: torch.Tensor, ssq: torch.Tensor, n_part: int, size: int, eps: float):
        self.hb, self.ssq, self.n_part, self.size, self.eps = hb, ssq, n_part, size, eps

    @property
    def shape(self):
        return self.hb.shape

    @property
    def dtype(self):
        return self.hb.dtype


def gemm_tc(x, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32,
            ksplit: int = 0, swiglu_pairs: bool = False, own: bool = False) -> torch.Tensor:
    """The tcgen05/TMA product y = x @ weight.T (bfloat16 in, float32 accumulate).
    With `swiglu_pairs` the weight's rows alternate gate, up and the result is
    silu(gate) * up, [R, N / 2].  `x` may be a `NormedInput`."""
    normed = x if isinstance(x, NormedInput) else None
    if normed is not None:
        x = normed.hb
    R, K = x.shape
    N = weight.shape[0]
    _chk(x, "x", torch.bfloat16)
    _chk(weight, "weight", torch.bfloat16)
    y = _new((R, N // 2 if swiglu_pairs else N), out_dtype, x.device, own=own)
    st = native.lib().rfx_gemm_bf16_tc(
        x.data_ptr(), weight.data_ptr(), y.data_ptr(), dt_code(out_dtype), R, N, K, ksplit,
        1 if swiglu_pairs else 0, normed.ssq.data_ptr() if normed is not None else 0,
        normed.n_part if normed is not None else 0, normed.size if normed is not None else 0,
        float(normed.eps) if normed is not None else 0.0, device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gemm_bf16_tc (R={R}, N={N}, K={K})")
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           own: bool = False) -> torch.Tensor:
    """y = x @ weight.T for weight [N, K] row-major.

    float32: this library's own CUDA-core product (no reduced-precision matrix
    mode; each output element reduced over k in index order).
    bfloat16: the weight-streaming tcgen05 kernel for up to GEMV_MAX_ROWS rows
    (decode), the library matrix product (cuBLAS, 32-bit accumulation) above
    that, where the reference uses a library product too
    (src/model/kernels.rs:2518-2561).  The result comes from the step's workspace;
    with `own` it gets memory of its own (what a step hands to its caller)."""
    R, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise InvalidInput(f"linear: x has {K} columns, weight has {K2}")
    if x.dtype != weight.dtype:
        raise InvalidInput(f"linear: x is {x.dtype}, weight is {weight.dtype}")
    if isinstance(x, NormedInput):
        return gemm_tc(x, weight, out_dtype or torch.bfloat16, own=own)
    _chk(x, "x")
    _chk(weight, "weight")
    if x.dtype == torch.float32:
        y = _new((R, N), torch.float32, x.device, own=own)
        st = native.lib().rfx_gemm_f32(x.data_ptr(), weight.data_ptr(), y.data_ptr(), R, N, K, _stream())
        native.check(st, f"gemm_f32 (R={R}, N={N}, K={K})")
        return y
    out_dtype = out_dtype or torch.bfloat16
    if R <= GEMV_MAX_ROWS and K % 8 == 0 and (x.data_ptr() | weight.data_ptr()) % 16 == 0:
        return gemm_tc(x, weight, out_dtype, own=own)
    y = _new((R, N), out_dtype, x.device, own=own)
    if out_dtype == torch.float32:
        return torch.mm(x, weight.t(), out_dtype=torch.float32, out=y)
    return torch.mm(x, weight.t(), out=y)


def gather_dot(x: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """y[j] = x[j] . weight[ids[j]], float32 [P]: row j of `x` against one row of
    the matrix, chosen by id.  Scoring given continuations needs the head's rows
    of a handful of ids, not the whole vocabulary
    (src/kernels_cuda/gemv_gather.cu:10-51).  In 32-bit the bits are those of
    `linear(x, weight)[j, ids[j]]`."""
    P, K = x.shape
    V, K2 = weight.shape
    if K != K2 or ids.numel() != P:
        raise InvalidInput("gather_dot: x [P, K], weight [V, K] and P ids are needed")
    if x.dtype != weight.dtype:
        raise InvalidInput(f"gather_dot: x is {x.dtype}, weight is {weight.dtype}")
    y = torch.empty((P,), dtype=torch.float32, device=x.device)
    st = native.lib().rfx_gather_dot(_chk(x, "x"), _chk(weight, "weight"), dt_code(x.dtype),
                                     _chk(ids, "ids", torch.int32), y.data_ptr(), P, K, V,
                                     device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gather_dot (P={P}, K={K})")
    return y


def gemm_tc_residual(x: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor,
                     norm_weight: torch.Tensor, norm_offset: float, eps: float, ksplit: int = 0) -> NormedInput:
    """hidden += x @ weight.T in place (float32), and the rows of the new hidden
    as a `NormedInput` for the product after the norm whose weight is given: the
    residual add and the RMSNorm between two products without a launch."""
    import ctypes

    R, K = x.shape
    N = weight.shape[0]
    _chk(x, "x", torch.bfloat16)
    _chk(weight, "weight", torch.bfloat16)
    _chk(hidden, "hidden", torch.float32)
    _chk(norm_weight, "norm_weight", torch.float32)
    if tuple(hidden.shape) != (R, N) or norm_weight.numel() != N:
        raise InvalidInput("gemm_tc_residual: hidden must be [rows, out] and the norm weight [out]")
    hb = _new((R, N), torch.bfloat16, x.device)
    ssq = _new((R * native.lib().rfx_gemm_bf16_tc_max_parts(N),), torch.float32, x.device)
    n_part = ctypes.c_int(0)
    st = native.lib().rfx_gemm_bf16_tc_residual(
        x.data_ptr(), weight.data_ptr(), hidden.data_ptr(), norm_weight.data_ptr(), float(norm_offset),
        hb.data_ptr(), ssq.data_ptr(), ctypes.addressof(n_part), R, N, K, ksplit,
        device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gemm_bf16_tc_residual (R={R}, N={N}, K={K})")
    return NormedInput(hb, ssq, n_part.value, N, eps)


ADDED = object()  # what `linear_residual` returns when it added into `hidden` and began no norm


def linear_residual(x: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor, next_norm):
    """The fused forms of `hidden += linear(x, weight)`.

    A few bfloat16 rows and an RMSNorm with a plain weight next: the product
    kernel's epilogue adds into `hidden` and begins `next_norm`; returns a
    `NormedInput`.  More bfloat16 rows than that kernel takes: the library
    product accumulates onto the 32-bit `hidden` in place (C = A B + C with
    32-bit C, so the sum is never rounded to bfloat16); returns `ADDED`.
    Otherwise None, and the caller takes the two-launch way."""
    if x.dtype != torch.bfloat16 or not FUSE_NORM:
        return None
    if x.shape[0] > GEMV_MAX_ROWS or x.shape[1] % 8:
        _chk(x, "x")
        _chk(weight, "weight", torch.bfloat16)
        _chk(hidden, "hidden", torch.float32)
        torch.addmm(hidden, x, weight.t(), out_dtype=torch.float32, out=hidden)
        return ADDED
    if next_norm is None or weight.shape[0] % 8:
        return None  # the product that takes these rows streams them by TMA: whole 16-byte units
    w = getattr(next_norm, "weight", None)
    spec = getattr(next_norm, "spec", None)
    if w is None or spec is None or getattr(spec, "kind", None) != "rmsnorm" or w.numel() != weight.shape[0]:
        return None
    return gemm_tc_residual(x, weight, hidden, w, spec.weight_offset, spec.eps)


FUSE_NORM = _env_flag("REFLEX_B200_FUSE_NORM", True)


def linear_swiglu(x: torch.Tensor, weight_pairs: torch.Tensor) -> torch.Tensor:
    """silu(x @ gate.T) * (x @ up.T) for a weight whose rows alternate gate_j,
    up_j; [R, I] in x's dtype.  For a few bfloat16 rows the activation is the
    product kernel's epilogue; otherwise product, then the SwiGLU kernel."""
    R, K = x.shape
    if x.dtype == torch.bfloat16 and R <= GEMV_MAX_ROWS and K % 8 == 0:
        return gemm_tc(x, weight_pairs, torch.bfloat16, swiglu_pairs=True)
    if isinstance(x, NormedInput):
        raise InvalidInput("a NormedInput is only made for sizes the fused product takes")
    return swiglu(linear(x, weight_pairs), alternating=True)


# ----------------------------------------------------------------- attention
def qkv_post(qkv: torch.Tensor, q_weight, k_weight, eps: float, weight_offset: float,
             rotation, row_pos: torch.Tensor, row_slot: torch.Tensor,
             k_pages, v_pages, page_table: torch.Tensor, page_size: int, nq: int, nkv: int,
             head_dim: int, writes_cache: bool, out_dtype: torch.dtype, values_are_keys: bool = False,
             ld: Optional[int] = None) -> torch.Tensor:
    """Per-head q/k norm, rotary encoding, q out, k and v into the cache.
    `rotation`: a `parts.Rotation` (denominators, rotary_dim, pairing,
    magnitude) or None for no rotary encoding.  `values_are_keys`: the rows hold
    no value columns; a value head is its key head as projected, before the norm
    and the rotation.  `ld`: the rows are the first columns of a wider stacked
    product (the row stride is then `qkv.shape[1]`, the q | k | v columns `ld`)."""
    from ..parts.registry import PAIRINGS

    R = qkv.shape[0]
    rope_denom, rotary_dim, pairing, magnitude = None, 0, 0, 1.0
    if rotation is not None:
        if rotation.pairing not in PAIRINGS:
            raise InvalidInput(f"qkv_post: pairing must be one of {sorted(PAIRINGS)}, got {rotation.pairing!r}")
        rope_denom, rotary_dim = rotation.denominators, int(rotation.rotary_dim)
        pairing, magnitude = PAIRINGS[rotation.pairing], float(rotation.magnitude)
        if rope_denom is not None and rope_denom.numel() != rotary_dim // 2:
            raise InvalidInput("qkv_post: one denominator per rotary pair is needed")
    nkv_in = nkv if writes_cache else 0
    if (qkv.shape[1] if ld is None else ld) != (nq + (1 if values_are_keys else 2) * nkv_in) * head_dim:
        raise InvalidInput("qkv_post: qkv width does not match the head counts")
    if ld is not None and ld > qkv.shape[1]:
        raise InvalidInput("qkv_post: the q | k | v columns do not fit into the rows")
    q = _new((R, nq * head_dim), out_dtype, qkv.device)
    st = native.lib().rfx_qkv_post_kv(
        _chk(qkv, "qkv"), dt_code(qkv.dtype), qkv.shape[1], _chk(q_weight, "q_norm", torch.float32),
        _chk(k_weight, "k_norm", torch.float32), float(eps), float(weight_offset),
        _chk(rope_denom, "rope_denom", torch.float32), int(rotary_dim),
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32),
        q.data_ptr(), _chk(k_pages, "k_pages"), _chk(v_pages, "v_pages"), dt_code(out_dtype),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size, R, nq, nkv_in,
        nkv, head_dim, pairing, magnitude, 1 if values_are_keys else 0, _stream())
    native.check(st, f"qkv_post (head_dim={head_dim})")
    return q


def qkv_fused_takes(x, head_dim: int, rotation, qkv_weight: torch.Tensor) -> bool:
    """Whether `qkv_fused` takes this call: a few bfloat16 rows (decode), a head
    size of 64 or 128, and a rotation, if any, over the whole head in half-split
    pairs."""
    rows, K = x.shape
    if not FUSE_QKV or x.dtype != torch.bfloat16 or qkv_weight.dtype != torch.bfloat16:
        return False
    if rows > min(GEMV_MAX_ROWS, FUSE_QKV_ROWS) or K % 8 or head_dim not in (64, 128):
        return False
    if rotation is not None and (rotation.pairing != "half" or rotation.rotary_dim != head_dim
                                 or rotation.denominators is None):
        return False
    return True


def qkv_fused(x, qkv_weight: torch.Tensor, q_weight, k_weight, eps: float, weight_offset: float,
              rotation, row_pos: torch.Tensor, row_slot: torch.Tensor, k_pages, v_pages,
              page_table: torch.Tensor, page_size: int, nq: int, nkv: int, head_dim: int,
              writes_cache: bool) -> torch.Tensor:
    """The q/k/v product of a decode step and what follows it, in one launch:
    per-head q/k norm, rotary encoding, q out (bfloat16 [R, nq * head_dim]), k and
    v into the cache.  `x`: bfloat16 rows or a `NormedInput`.  What `linear` +
    `qkv_post` give, without the launch between them and without the 32-bit
    q/k/v rows in memory."""
    normed = x if isinstance(x, NormedInput) else None
    if normed is not None:
        x = normed.hb
    R, K = x.shape
    nkv_in = nkv if writes_cache else 0
    if qkv_weight.shape[0] != (nq + 2 * nkv_in) * head_dim or qkv_weight.shape[1] != K:
        raise InvalidInput("qkv_fused: the weight's shape does not match the head counts")
    _chk(x, "x", torch.bfloat16)
    _chk(qkv_weight, "qkv_weight", torch.bfloat16)
    denom = None if rotation is None else rotation.denominators
    q = _new((R, nq * head_dim), torch.bfloat16, x.device)
    st = native.lib().rfx_gemm_bf16_tc_qkv(
        x.data_ptr(), qkv_weight.data_ptr(), R, K,
        normed.ssq.data_ptr() if normed is not None else 0, normed.n_part if normed is not None else 0,
        normed.size if normed is not None else 0, float(normed.eps) if normed is not None else 0.0,
        _chk(q_weight, "q_norm", torch.float32), _chk(k_weight, "k_norm", torch.float32), float(eps),
        float(weight_offset), _chk(denom, "rope_denom", torch.float32),
        float(rotation.magnitude) if rotation is not None else 1.0,
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), q.data_ptr(),
        _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size, nq, nkv_in, nkv,
        head_dim, device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gemm_bf16_tc_qkv (R={R}, K={K}, head_dim={head_dim})")
    return q


FUSE_QKV = _env_flag("REFLEX_B200_FUSE_QKV", True)
# Up to this many rows the fused form is the faster one (measured on a B200 at
# Qwen3-8B sizes: 2.3 % of a step at batch 1, 0.7 % at batch 8, level at 16, behind
# from 32 on).  With more rows the attention kernel that follows is the
# step's largest after the feed-forward, and it gains more from starting early,
# beside the light `qkv_post` launch, and fetching its cached pages meanwhile,
# than the step gains from one launch less.
FUSE_QKV_ROWS = _env_int("REFLEX_B200_FUSE_QKV_ROWS", 8, 0, 64)


def attention_plain(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    page_table: torch.Tensor, page_size: int, row_pos: torch.Tensor,
                    row_slot: torch.Tensor, nq: int, nkv: int, head_dim: int,
                    window: Optional[int], scale: float,
                    sink: Optional[torch.Tensor] = None,
                    slopes: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """`keep_first`: with a window, the first so many positions of a sequence
    stay visible beyond it.  `sink` (float32, one per query head): exp(sink) joins the softmax's
    denominator once, with no key and no value.  `slopes` (float32, one per
    query head): slope * (query position - key position) is taken off every
    score, a linear distance bias."""
    R = q.shape[0]
    out = _new(q.shape, q.dtype, q.device)
    st = native.lib().rfx_attention_plain(
        _chk(q, "q"), _chk(k_pages, "k_pages", q.dtype), _chk(v_pages, "v_pages", q.dtype),
        dt_code(q.dtype), _chk(page_table, "page_table", torch.int32), page_table.shape[1],
        page_size, _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32),
        out.data_ptr(), R, nq, nkv, head_dim, int(window or 0), int(keep_first if window else 0), float(scale),
        _chk(sink, "sink", torch.float32), _chk(slopes, "slopes", torch.float32), _stream())
    native.check(st, f"attention_plain (head_dim={head_dim})")
    return out


def gemv_simple(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The plain CUDA-core bfloat16 product (one warp per output column); kept
    as the readable counterpart of `gemm_tc` for tests."""
    R, K = x.shape
    N = weight.shape[0]
    y = torch.empty((R, N), dtype=out_dtype, device=x.device)
    st = native.lib().rfx_gemv_bf16(_chk(x, "x", torch.bfloat16), _chk(weight, "weight", torch.bfloat16),
                                    y.data_ptr(), dt_code(out_dtype), R, N, K, _stream())
    native.check(st, f"gemv_bf16 (R={R}, N={N}, K={K})")
    return y


_SM_COUNT = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked once."""
    global _SM_COUNT
    if not _SM_COUNT:
        _SM_COUNT = int(native.lib().rfx_sm_count())
    return _SM_COUNT


def decode_splits(n_rows: int, nq: int, nkv: int, max_pages: int = 64) -> int:
    """Key-range splits of the decode kernel for rows whose longest context has
    `max_pages` pages.  A split buys parallelism and costs a CTA's fixed work
    (query load, the warps' merge, the exchange of partials) once more.  Fitted
    to kernel times on a B200 at batches of 1 to 64 and contexts of 640 to
    16,384: two CTAs fit an SM; a CTA walks its pages at 0.6 us a page with an
    SM to itself and 0.85 us beside another (its tile code, not the memory);
    the pages of all CTAs together cannot come faster than the memory gives
    them, 1.35 us per page and CTA slot; a CTA's fixed work is 3 to 4 us; 4 us
    for the launch; the merge 1 us + 0.12 us a split inside a cluster of up to
    8, 5 us in one of 16, 3 us + 0.25 us a split through the combine kernel.
    The smallest estimate wins."""
    forced = _env_int("REFLEX_B200_DECODE_SPLITS", 0, 0, 64)  # tuning aid
    if forced > 0:
        return forced
    ctas = n_rows * nkv * ((nq // nkv + 7) // 8)
    sms = sm_count()
    slots = 2 * sms
    best, best_cost = 1, None
    for s in (1, 2, 4, 8, 16, 32, 64):
        if s > max(1, max_pages):
            break
        n = ctas * s
        per_split = -(-max_pages // s)
        resident = per_split * (0.6 if n <= sms else 0.85) + 4.0
        streaming = n * (per_split * 1.35 + 3.0) / slots
        if s == 1:
            merge = 0.0
        elif s <= 8:
            merge = 1.0 + 0.12 * s
        elif s == 16:
            merge = 5.0
        else:
            merge = 3.0 + 0.25 * s
        cost = 4.0 + max(resident, streaming) + merge
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def attention_decode(q, k_pages, v_pages, page_table, page_size, row_pos, row_slot, nq, nkv,
                     head_dim, window, scale, n_splits: Optional[int] = None,
                     sink: Optional[torch.Tensor] = None,
                     slopes: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """bfloat16 tensor-core attention for rows that are each one query
    position (decode), split over the keys."""
    keep_first = int(keep_first) if window else 0
    R = q.shape[0]
    _chk(q, "q", torch.bfloat16)
    if head_dim % 16 or not (16 <= head_dim <= 256):
        raise InvalidInput(f"attention_decode takes head_dim in steps of 16 up to 256, got {head_dim}")
    n_splits = n_splits or decode_splits(R, nq, nkv)
    out = _new(q.shape, q.dtype, q.device)
    # pages of the store, for the kernel's TMA maps: [pages, kv heads, page, head_dim], one piece
    pool_pages = int(k_pages.shape[0]) if (k_pages.dim() == 4 and k_pages.is_contiguous()
                                           and v_pages.is_contiguous() and v_pages.shape == k_pages.shape) else 0
    if CLUSTER_MERGE and n_splits in (2, 4, 8, 16):
        # the splits as one thread-block cluster that merges its partials itself
        st = native.lib().rfx_attention_decode_kf(
            q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
            _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
            _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), out.data_ptr(), 0,
            R, nq, nkv, head_dim, n_splits, int(window or 0), keep_first, float(scale),
            _chk(sink, "sink", torch.float32), _chk(slopes, "slopes", torch.float32), pool_pages, 1,
            device_error_word(q.device).data_ptr(), _stream())
        if st != native.ERR_UNSUPPORTED:
            native.check(st, f"attention_decode_cluster (head_dim={head_dim}, splits={n_splits})")
            return out
    partial = _new((R * nq * n_splits * (head_dim + 2),), torch.float32, q.device) if n_splits > 1 else None
    st = native.lib().rfx_attention_decode_kf(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), out.data_ptr(),
        partial.data_ptr() if partial is not None else 0, R, nq, nkv, head_dim, n_splits,
        int(window or 0), keep_first, float(scale), _chk(sink, "sink", torch.float32),
        _chk(slopes, "slopes", torch.float32), pool_pages, 0, device_error_word(q.device).data_ptr(), _stream())
    native.check(st, f"attention_decode (head_dim={head_dim}, splits={n_splits})")
    return out


CLUSTER_MERGE = _env_flag("REFLEX_B200_CLUSTER_MERGE", True)


def attention_prefill(q, k_pages, v_pages, page_table, page_size, seq_slot, seq_start, seq_new,
                      seq_row0, max_new: int, nq, nkv, head_dim, window, scale, sink=None,
                      slopes=None, keep_first: int = 0) -> torch.Tensor:
    """bfloat16 tensor-core attention for a packed batch of sequences that
    each bring one or more rows (prefill, chunks, mixed steps)."""
    _chk(q, "q", torch.bfloat16)
    if head_dim % 16 or not (16 <= head_dim <= 256):
        raise InvalidInput(f"attention_prefill takes head_dim in steps of 16 up to 256, got {head_dim}")
    if nq // nkv > 128:
        raise InvalidInput(f"attention_prefill takes up to 128 query heads per kv head, got {nq // nkv}")
    out = _new(q.shape, q.dtype, q.device)
    S = seq_slot.numel()
    st = native.lib().rfx_attention_prefill_kf(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(seq_slot, "seq_slot", torch.int32), _chk(seq_start, "seq_start", torch.int32),
        _chk(seq_new, "seq_new", torch.int32), _chk(seq_row0, "seq_row0", torch.int32), out.data_ptr(),
        S, int(max_new), nq, nkv, head_dim, int(window or 0), int(keep_first) if window else 0, float(scale),
        _chk(sink, "sink", torch.float32), _chk(slopes, "slopes", torch.float32), _stream())
    native.check(st, f"attention_prefill (head_dim={head_dim})")
    return out


def attention_prefill_tc(q, k_pages, v_pages, page_table, page_size, seq_slot, seq_start, seq_new,
                         seq_row0, max_new: int, nq, nkv, head_dim, window, scale, sink=None,
                         slopes=None, keep_first: int = 0) -> torch.Tensor:
    """The tcgen05/TMEM form of `attention_prefill`, for head sizes 64 and 128
    (with `slopes` the scale must be positive)."""
    _chk(q, "q", torch.bfloat16)
    if head_dim not in (64, 128):
        raise InvalidInput(f"attention_prefill_tc takes head_dim 64 or 128, got {head_dim}")
    if nq // nkv > 128:
        raise InvalidInput(f"attention_prefill_tc takes up to 128 query heads per kv head, got {nq // nkv}")
    out = _new(q.shape, q.dtype, q.device)
    st = native.lib().rfx_attention_prefill_tc_kf(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        k_pages.shape[0], _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(seq_slot, "seq_slot", torch.int32), _chk(seq_start, "seq_start", torch.int32),
        _chk(seq_new, "seq_new", torch.int32), _chk(seq_row0, "seq_row0", torch.int32), out.data_ptr(),
        seq_slot.numel(), int(max_new), q.shape[0], nq, nkv, head_dim, int(window or 0),
        int(keep_first) if window else 0, float(scale),
        _chk(sink, "sink", torch.float32), _chk(slopes, "slopes", torch.float32),
        device_error_word(q.device).data_ptr(), _stream())
    native.check(st, f"attention_prefill_tc (head_dim={head_dim})")
    return out


def attention(q, k_pages, v_pages, page_table, page_size, batch, nq, nkv, head_dim, window, scale,
              sink=None, slopes=None, keep_first: int = 0):
    """Attention of the step's rows over their sequences' cached keys and
    values; picks the kernel for the dtype and the kind of step.  `sink`: one
    float32 per query head whose exponential joins the softmax's denominator.
    `slopes`: one float32 per query head; slope * (query position - key
    position) is taken off every score.  `keep_first`: with a window, the first
    so many positions of a sequence stay visible beyond it."""
    fast = q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
    keep_first = int(keep_first) if window else 0
    if fast and batch.is_decode:
        pages = -(-min(batch.max_context, window or batch.max_context) // page_size) + (1 if window else 0)
        pages += -(-keep_first // page_size)
        return attention_decode(q, k_pages, v_pages, page_table, page_size, batch.row_pos,
                                batch.row_slot, nq, nkv, head_dim, window, scale,
                                n_splits=decode_splits(q.shape[0], nq, nkv, pages), sink=sink, slopes=slopes,
                                keep_first=keep_first)
    if fast and nq // nkv <= 128 and head_dim in (64, 128) and scale > 0:
        return attention_prefill_tc(q, k_pages, v_pages, page_table, page_size, batch.seq_slot,
                                    batch.seq_start, batch.seq_new, batch.seq_row0, batch.max_new, nq,
                                    nkv, head_dim, window, scale, sink, slopes, keep_first)
    if fast and nq // nkv <= 128:
        return attention_prefill(q, k_pages, v_pages, page_table, page_size, batch.seq_slot,
                                 batch.seq_start, batch.seq_new, batch.seq_row0, batch.max_new, nq,
                                 nkv, head_dim, window, scale, sink, slopes, keep_first)
    return attention_plain(q, k_pages, v_pages, page_table, page_size, batch.row_pos,
                           batch.row_slot, nq, nkv, head_dim, window, scale, sink, slopes, keep_first)


# ------------------------------------------------- further norms and embedding terms
def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
              delta: Optional[torch.Tensor] = None, update_residual: bool = True,
              rows: Optional[torch.Tensor] = None, want_out: bool = True) -> Optional[torch.Tensor]:
    """Layer norm with a weight and no bias of the float32 residual stream `x`
    [R, H], the residual add fused in as in `rmsnorm`: t = x (+ delta);
    returns (t - mean) / sqrt(var + eps) * weight in `out_dtype`."""
    R, H = x.shape
    _chk(x, "x", torch.float32)
    r_out = R if rows is None else rows.numel()
    out = _new((r_out, H), out_dtype, x.device) if want_out else None
    x_out = x if (delta is not None and update_residual and rows is None) else None
    st = native.lib().rfx_layernorm(
        x.data_ptr(), _chk(delta, "delta"), dt_code(delta.dtype) if delta is not None else 0,
        x_out.data_ptr() if x_out is not None else 0, _chk(weight, "weight", torch.float32),
        float(eps), out.data_ptr() if out is not None else 0, dt_code(out_dtype),
        _chk(rows, "rows", torch.int32), r_out, H, _stream())
    native.check(st, f"layernorm (H={H})")
    return out


def bigram_add(hidden: torch.Tensor, table: torch.Tensor, batch, prev_state: torch.Tensor,
               mul_prev: int, mul_cur: int, vocab: int) -> torch.Tensor:
    """hidden[r] += table[(prev * mul_prev + token * mul_cur) mod buckets], the
    table's last row at a sequence's first position; `prev_state` (int32, one
    word a slot) holds each sequence's last token between steps."""
    R, H = hidden.shape
    buckets = table.shape[0] - 1
    st = native.lib().rfx_bigram_add(
        _chk(hidden, "hidden", torch.float32), _chk(table, "table"), dt_code(table.dtype),
        _chk(batch.tokens, "tokens", torch.int32), _chk(batch.row_pos, "row_pos", torch.int32),
        _chk(batch.row_slot, "row_slot", torch.int32), _chk(batch.seq_row0, "seq_row0", torch.int32),
        batch.seq_slot.numel(), _chk(prev_state, "prev_state", torch.int32), R, H, buckets,
        int(mul_prev), int(mul_cur), int(vocab), _stream())
    native.check(st, "bigram_add")
    return hidden


def sinusoid_add(hidden: torch.Tensor, row_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """hidden[r, 2i] += sin(p f_i), hidden[r, 2i + 1] += cos(p f_i); `inv_freq`
    float64 [ceil(H / 2)]."""
    R, H = hidden.shape
    if inv_freq.numel() != (H + 1) // 2:
        raise InvalidInput("sinusoid_add: one frequency per pair of columns is needed")
    st = native.lib().rfx_sinusoid_add(_chk(hidden, "hidden", torch.float32),
                                       _chk(row_pos, "row_pos", torch.int32),
                                       _chk(inv_freq, "inv_freq", torch.float64), R, H, _stream())
    native.check(st, "sinusoid_add")
    return hidden


# ---------------------------------------------------------- latent attention
def latent_post(proj: torch.Tensor, q_weight: torch.Tensor, kv_weight: torch.Tensor, eps: float,
                row_pos, row_slot, pages, page_table, page_size: int, q_rank: int, kv_rank: int,
                n_gate: int, writes_cache: bool, out_dtype: torch.dtype):
    """A row of the stacked product [query latent | key/value latent | gates]:
    RMSNorm of the query latent (returned, `out_dtype`), RMSNorm of the
    key/value latent into the cache at the row's position, sigmoid of the gates
    (returned, float32 [R, n_gate])."""
    R = proj.shape[0]
    q = _new((R, q_rank), out_dtype, proj.device)
    gate = _new((R, max(1, n_gate)), torch.float32, proj.device)
    st = native.lib().rfx_latent_post(
        _chk(proj, "proj"), dt_code(proj.dtype), proj.shape[1], _chk(q_weight, "q_weight", torch.float32),
        _chk(kv_weight, "kv_weight", torch.float32), float(eps), _chk(row_pos, "row_pos", torch.int32),
        _chk(row_slot, "row_slot", torch.int32), q.data_ptr(), _chk(pages, "pages", out_dtype),
        dt_code(out_dtype), _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        gate.data_ptr(), R, q_rank, kv_rank, n_gate, 1 if writes_cache else 0, _stream())
    native.check(st, "latent_post")
    return q, gate


HEADS_LINEAR_MAX_ROWS = _env_int("REFLEX_B200_HEADS_LINEAR_MAX_ROWS", 64, 0, 1 << 30)


def heads_linear(x: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y[r, b, :] = x[r, b, :] @ weight[b].T for every head b: x [R, heads * K],
    weight [heads, N, K], y [R, heads * N]; with `scale` (float32 [R, heads])
    y[r, b, :] is multiplied by scale[r, b].  float32 and a few bfloat16 rows:
    this library's kernel (32-bit accumulation in index order); more bfloat16
    rows: the library's batched product, then the scaling kernel.  `out_dtype`
    float32 with bfloat16 operands (many rows only): the batched product's
    32-bit sums come out unrounded."""
    heads, N, K = weight.shape
    R = x.shape[0]
    if x.shape[1] != heads * K or x.dtype != weight.dtype:
        raise InvalidInput("heads_linear: x must be [rows, heads * K] in the weight's dtype")
    _chk(x, "x")
    _chk(weight, "weight")
    wide = out_dtype == torch.float32 and x.dtype == torch.bfloat16
    if wide and R <= HEADS_LINEAR_MAX_ROWS:
        raise InvalidInput("heads_linear: 32-bit results of bfloat16 operands need more rows than its own kernel takes")
    y = _new((R, heads * N), torch.float32 if wide else x.dtype, x.device)
    if wide:
        torch.bmm(x.view(R, heads, K).transpose(0, 1), weight.transpose(1, 2), out_dtype=torch.float32,
                  out=y.view(R, heads, N).transpose(0, 1))
        if scale is not None:
            st = native.lib().rfx_scale_heads(y.data_ptr(), dt_code(y.dtype), _chk(scale, "scale", torch.float32),
                                              y.numel(), N, _stream())
            native.check(st, "scale_heads")
        return y
    if x.dtype == torch.bfloat16 and R > HEADS_LINEAR_MAX_ROWS:
        torch.bmm(x.view(R, heads, K).transpose(0, 1), weight.transpose(1, 2),
                  out=y.view(R, heads, N).transpose(0, 1))
        if scale is not None:
            st = native.lib().rfx_scale_heads(y.data_ptr(), dt_code(y.dtype), _chk(scale, "scale", torch.float32),
                                              y.numel(), N, _stream())
            native.check(st, "scale_heads")
        return y
    st = native.lib().rfx_heads_linear(x.data_ptr(), heads * K, weight.data_ptr(), y.data_ptr(), heads * N,
                                       dt_code(x.dtype), _chk(scale, "scale", torch.float32), R, N, K, heads,
                                       _stream())
    native.check(st, f"heads_linear (heads={heads}, N={N}, K={K})")
    return y


# --------------------------------------------------------------------- mLSTM
MLSTM_SLICE = 64  # columns of the memory a block of the scan owns; each slice keeps its own copy of m


def mlstm_state_floats(dim: int, vdim: int) -> int:
    """Floats of state per head and slot: S [dim, vdim], n [dim], m once per slice."""
    return dim * vdim + dim + (vdim + MLSTM_SLICE - 1) // MLSTM_SLICE


MLSTM_CHUNK_MIN_ROWS = _env_int("REFLEX_B200_MLSTM_CHUNK_MIN_ROWS", 48, 1, 1 << 30)


def mlstm_scan(proj: torch.Tensor, offsets, bias_i, bias_f, cap: float, q_scale: float, batch,
               state: torch.Tensor, heads: int, dim: int, vdim: int, max_rows: Optional[int] = None):
    """The recurrence over the step's rows, sequence by sequence.  `proj`
    float32 [R, ld] holds q, k, v and the two gate pre-activations at the
    column offsets `offsets` = (q, k, v, i, f); `state` [slots, heads, floats].
    Returns the numerators S^T q [R, heads * vdim] and denominators [R, heads].
    `max_rows`: the most rows any sequence brings; from `MLSTM_CHUNK_MIN_ROWS`
    on (and dim up to 256) the chunkwise kernel runs, else the row-by-row walk:
    the same function, rounded differently."""
    R = proj.shape[0]
    _chk(proj, "proj", torch.float32)
    if state.shape[-1] != mlstm_state_floats(dim, vdim) or state.shape[-2] != heads:
        raise InvalidInput("mlstm_scan: the state's shape does not match the sizes")
    num = _new((R, heads * vdim), torch.float32, proj.device)
    den = _new((R, heads), torch.float32, proj.device)
    q_off, k_off, v_off, i_off, f_off = (int(o) for o in offsets)
    chunked = max_rows is not None and max_rows >= MLSTM_CHUNK_MIN_ROWS and dim <= 256
    fn = native.lib().rfx_mlstm_chunk if chunked else native.lib().rfx_mlstm_scan
    st = fn(
        proj.data_ptr(), proj.shape[1], q_off, k_off, v_off, i_off, f_off,
        _chk(bias_i, "bias_i", torch.float32), _chk(bias_f, "bias_f", torch.float32), float(cap),
        float(q_scale), _chk(batch.seq_slot, "seq_slot", torch.int32),
        _chk(batch.seq_row0, "seq_row0", torch.int32), batch.seq_slot.numel(),
        _chk(state, "state", torch.float32), num.data_ptr(), den.data_ptr(), heads, dim, vdim, _stream())
    native.check(st, f"mlstm_scan (dim={dim}, vdim={vdim})")
    return num, den


def mlstm_out(num, den, proj, g_off: int, weight, eps: float, heads: int, vdim: int,
              out_dtype: torch.dtype) -> torch.Tensor:
    """o = num / den, each head's o over its root mean square, times the norm
    weight [heads * vdim], times sigmoid of the gate columns of `proj`."""
    R = num.shape[0]
    out = _new((R, heads * vdim), out_dtype, num.device)
    st = native.lib().rfx_mlstm_out(num.data_ptr(), den.data_ptr(), _chk(proj, "proj", torch.float32),
                                    proj.shape[1], int(g_off), _chk(weight, "weight", torch.float32),
                                    float(eps), out.data_ptr(), dt_code(out_dtype), R, heads, vdim, _stream())
    native.check(st, "mlstm_out")
    return out


# ------------------------------------------------------- mixture of experts
MOE_ACTIVATIONS = {"relu2": 0, "silu": 1, "glu_clamped": 2, "swiglu": 3}


MOE_SCORES = {"softmax_top": 0, "sigmoid": 1, "softmax_all": 2}


def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, experts: Optional[int] = None,
              scores: str = "softmax_top", col0: int = 0, scale: float = 1.0):
    """Router logits float32 [R, experts] (+ bias) -> ids int32 [R, top], the
    experts with the largest logits, and weights float32 [R, top]: the softmax
    over the chosen logits only ("softmax_top"), or each chosen logit's sigmoid
    as it is ("sigmoid"), or the softmax over all experts with the chosen ones'
    scores divided by their sum + 1e-20 ("softmax_all"); `scale` multiplies the
    weights.  With `experts` only that many columns of `logits`,
    from column `col0` on, are router logits (the rest belongs to the caller: a
    product stacked with others')."""
    R, ld = logits.shape
    E = ld if experts is None else int(experts)
    if not (0 <= col0 <= ld - E):
        raise InvalidInput("moe_route: the router's columns do not fit into the logits' rows")
    ids = _new((R, top), torch.int32, logits.device)
    wts = _new((R, top), torch.float32, logits.device)
    st = native.lib().rfx_moe_route_scaled(_chk(logits, "logits", torch.float32) + 4 * int(col0), ld,
                                           _chk(bias, "bias", torch.float32), ids.data_ptr(), wts.data_ptr(), R, E,
                                           int(top), MOE_SCORES[scores], float(scale), _stream())
    native.check(st, f"moe_route (experts={E}, top={top})")
    return ids, wts


def moe_experts(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor,
                wts: torch.Tensor, activation: str = "relu2", weight_input: bool = False,
                alpha: float = 1.0, limit: float = 0.0) -> torch.Tensor:
    """sum_k wts[r, k] down[e] act(up[e] x[r]), e = ids[r, k]; up [experts, ff,
    width], down [experts, width, ff]; float32 [R, width].  Every (row, choice)
    reads its expert's matrices itself: the form for a few rows, and the exact
    one in 32-bit.  "glu_clamped": `up` is [experts, 2 ff, width], an expert's
    gate rows and then its up rows, and act is the clamped gated form with
    `alpha` and `limit` (`glu_clamped`); "swiglu": the same layout, silu(gate) * up.  `weight_input`: the weight multiplies
    the expert's input instead of its output, sum_k down[e] act(up[e] (wts[r, k]
    x[r]))."""
    R, width = x.shape
    E, ff, _w = up.shape
    gated = activation in ("glu_clamped", "swiglu")
    if gated:
        ff //= 2
    top = ids.shape[1]
    in_scale, out_wts = (wts, None) if weight_input else (None, wts)
    if x.dtype == torch.bfloat16 and MOE_GROUPED and R >= MOE_GROUPED_MIN_ROWS:
        # captured steps too, as long as the library's grouped product (no wait for the host) is there
        if not torch.cuda.is_current_stream_capturing() or (_GROUPED_MM[0] and width % 8 == 0 and ff % 8 == 0):
            return moe_experts_grouped(x, up, down, ids, wts, activation, weight_input, alpha, limit)
    act = _new((R * top, ff), x.dtype, x.device)
    st = native.lib().rfx_moe_up(_chk(x, "x"), _chk(up, "up", x.dtype), _chk(ids, "ids", torch.int32),
                                 _chk(in_scale, "wts", torch.float32), act.data_ptr(), dt_code(x.dtype), R, top,
                                 ff, width, MOE_ACTIVATIONS[activation], float(alpha), float(limit), _stream())
    native.check(st, "moe_up")
    y = _new((R, width), torch.float32, x.device)
    st = native.lib().rfx_moe_down(act.data_ptr(), _chk(down, "down", x.dtype), ids.data_ptr(),
                                   _chk(out_wts, "wts", torch.float32), y.data_ptr(), dt_code(x.dtype), R, top,
                                   ff, width, _stream())
    native.check(st, "moe_down")
    return y


MOE_GROUPED = _env_flag("REFLEX_B200_MOE_GROUPED", True)
# From two rows on, experts are likely shared between rows, and the grouped form reads each
# expert's matrices once (measured at batch 8 with 16 experts, 4 chosen: a decode step 1.41 ->
# 1.05 ms at width 2048); one row streams its own experts directly.
MOE_GROUPED_MIN_ROWS = _env_int("REFLEX_B200_MOE_GROUPED_MIN_ROWS", 2, 1, 1 << 30)


def moe_experts_grouped(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor,
                        wts: torch.Tensor, activation: str = "relu2", weight_input: bool = False,
                        alpha: float = 1.0, limit: float = 0.0) -> torch.Tensor:
    """The same sum for many bfloat16 rows (prefill): the (row, choice) pairs are
    placed expert by expert on the device, each expert's block of rows goes
    through its two matrices as library products (where the dense layers use
    them too: the library's grouped product, or one product an expert where it
    has none, for which the host reads the experts' offsets once), and a row's
    results are summed in the order of their rank."""
    R, width = x.shape
    E, ff, _w = up.shape
    gated = activation in ("glu_clamped", "swiglu")
    if gated:
        ff //= 2
    top = ids.shape[1]
    n = R * top
    lib = native.lib()
    in_scale, out_wts = (wts, None) if weight_input else (None, wts)

    def activate(a):
        """The experts' activation on the up product's rows: in place, or (gated) [n, 2 ff] -> [n, ff]."""
        if activation == "swiglu":
            return swiglu(a)
        if gated:
            return glu_clamped(a, alpha, limit)
        native.check(lib.rfx_moe_activation(a.data_ptr(), dt_code(a.dtype), a.numel(),
                                            MOE_ACTIVATIONS[activation], _stream()), "moe_activation")
        return a

    offsets = _new((E + 1,), torch.int32, x.device)
    place = _new((n,), torch.int32, x.device)
    native.check(lib.rfx_moe_group(_chk(ids, "ids", torch.int32), n, E, offsets.data_ptr(), place.data_ptr(),
                                   _stream()), "moe_group")
    xg = _new((n, width), x.dtype, x.device)
    native.check(lib.rfx_moe_gather(_chk(x, "x"), place.data_ptr(), _chk(in_scale, "wts", torch.float32),
                                    xg.data_ptr(), dt_code(x.dtype), n, top, width, _stream()), "moe_gather")
    grouped = getattr(torch, "_grouped_mm", None) if _GROUPED_MM[0] else None
    if grouped is not None and width % 8 == 0 and ff % 8 == 0:
        # the library's grouped product reads the experts' offsets on the device: no wait for the host
        try:
            ends = offsets[1:]
            act = activate(grouped(xg, up.transpose(1, 2), offs=ends))
            try:  # 32-bit results where the library gives them: the weighted sum then rounds once
                yg = grouped(act, down.transpose(1, 2), offs=ends, out_dtype=torch.float32) if _GROUPED_MM[1] else None
            except (RuntimeError, TypeError, NotImplementedError):
                _GROUPED_MM[1] = False
                yg = None
            if yg is None:
                yg = grouped(act, down.transpose(1, 2), offs=ends)
        except (RuntimeError, TypeError, NotImplementedError):
            _GROUPED_MM[0] = False  # this build of the library has none for these operands: one product an expert
            yg = None
        if yg is not None:
            y = _new((R, width), torch.float32, x.device)
            native.check(lib.rfx_moe_combine(_chk(yg, "yg"), dt_code(yg.dtype), place.data_ptr(),
                                             _chk(out_wts, "wts", torch.float32), y.data_ptr(), R, top, width,
                                             _stream()), "moe_combine")
            return y
    off = offsets.tolist()  # the one wait for the device
    act = _new((n, up.shape[1]), x.dtype, x.device)
    for e in range(E):
        if off[e + 1] > off[e]:
            torch.mm(xg[off[e]:off[e + 1]], up[e].t(), out=act[off[e]:off[e + 1]])
    act = activate(act)
    yg = _new((n, width), torch.float32, x.device)
    for e in range(E):
        if off[e + 1] > off[e]:
            torch.mm(act[off[e]:off[e + 1]], down[e].t(), out_dtype=torch.float32, out=yg[off[e]:off[e + 1]])
    y = _new((R, width), torch.float32, x.device)
    native.check(lib.rfx_moe_combine(yg.data_ptr(), dt_code(yg.dtype), place.data_ptr(),
                                     _chk(out_wts, "wts", torch.float32), y.data_ptr(), R, top, width, _stream()),
                 "moe_combine")
    return y


_GROUPED_MM = [True, True]  # whether the library's grouped product is tried, and its 32-bit output


# ------------------------------------------- clamped gated activation, row gates
def glu_clamped(gate_up: torch.Tensor, alpha: float, limit: float, alternating: bool = False) -> torch.Tensor:
    """[R, 2I] -> g' sigmoid(alpha g') (u' + 1), [R, I], with g' = min(g, limit)
    and u' = clamp(u, -limit, limit).  A row holds the gates in its first half
    and the ups in its second, or (`alternating`) gate_i at 2i and up_i at 2i + 1."""
    R, two_i = gate_up.shape
    I = two_i // 2
    out = _new((R, I), gate_up.dtype, gate_up.device)
    st = native.lib().rfx_glu_clamped(_chk(gate_up, "gate_up"), out.data_ptr(), dt_code(gate_up.dtype), R, I,
                                      1 if alternating else 0, float(alpha), float(limit), _stream())
    native.check(st, "glu_clamped")
    return out


def linear_glu_clamped(x: torch.Tensor, weight_pairs: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    """glu_clamped(x @ W.T) for a weight whose rows alternate gate_j, up_j; [R, I]
    in x's dtype.  For a few bfloat16 rows the activation is the product
    kernel's epilogue; otherwise product, then `glu_clamped`."""
    R, K = x.shape
    if x.dtype == torch.bfloat16 and R <= GEMV_MAX_ROWS and K % 8 == 0 and FUSE_GLU:
        N = weight_pairs.shape[0]
        _chk(x, "x", torch.bfloat16)
        _chk(weight_pairs, "weight", torch.bfloat16)
        y = _new((R, N // 2), torch.bfloat16, x.device)
        st = native.lib().rfx_gemm_bf16_tc_glu_clamped(
            x.data_ptr(), weight_pairs.data_ptr(), y.data_ptr(), BF16, R, N, K, 0, float(alpha), float(limit),
            device_error_word(x.device).data_ptr(), _stream())
        native.check(st, f"gemm_bf16_tc_glu_clamped (R={R}, N={N}, K={K})")
        return y
    return glu_clamped(linear(x, weight_pairs), alpha, limit, alternating=True)


FUSE_GLU = _env_flag("REFLEX_B200_FUSE_GLU", True)  # 0: product and activation apart (tests compare the two)


def row_gate_add_(y: torch.Tensor, rows: torch.Tensor, z: torch.Tensor, col: int,
                  extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[r] += sigmoid(z[r, col]) * rows[r] (+ extra[r]): y, extra float32 [R, H], z float32 [R, *]."""
    R, H = y.shape
    st = native.lib().rfx_row_gate_add(_chk(y, "y", torch.float32), _chk(rows, "rows"), dt_code(rows.dtype),
                                       _chk(z, "z", torch.float32), z.shape[1], int(col),
                                       _chk(extra, "extra", torch.float32), R, H, _stream())
    native.check(st, "row_gate_add")
    return y


# ------------------------------------------------------------ the residual stream
def stream_concat(x: torch.Tensor, delta: Optional[torch.Tensor], x0: torch.Tensor,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """[x (+ delta) | x0] row by row, [R, 2H] in `out_dtype`: the input of a
    product that mixes the stream with the embedding output."""
    R, H = x.shape
    out = _new((R, 2 * H), out_dtype, x.device)
    st = native.lib().rfx_stream_concat(_chk(x, "x", torch.float32), _chk(delta, "delta"),
                                        dt_code(delta.dtype) if delta is not None else 0,
                                        _chk(x0, "x0", torch.float32), out.data_ptr(), dt_code(out_dtype), R, H,
                                        _stream())
    native.check(st, "stream_concat")
    return out


def keep_copy(x: torch.Tensor) -> torch.Tensor:
    """A copy of `x` that lives for the whole step."""
    out = _new(tuple(x.shape), x.dtype, x.device, keep=True)
    out.copy_(x)
    return out


def logit_finish_(z: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """z <- z * scale, then cap * tanh(z / cap) when cap > 0; float32, in place."""
    if scale == 1.0 and not cap:
        return z
    st = native.lib().rfx_logit_finish(_chk(z, "z", torch.float32), z.numel(), float(scale), float(cap or 0.0),
                                       _stream())
    native.check(st, "logit_finish")
    return z


def branch_norm_mean(a: torch.Tensor, a_bias: Optional[torch.Tensor], wa: torch.Tensor, b: torch.Tensor,
                     wb: torch.Tensor, eps: float) -> torch.Tensor:
    """((a + a_bias) / rms(a + a_bias) * wa + b / rms(b) * wb) / 2, float32 [R, H]:
    two branches' outputs, each RMS-normed with its own weight, averaged."""
    R, H = a.shape
    out = _new((R, H), torch.float32, a.device)
    st = native.lib().rfx_branch_norm_mean(_chk(a, "a", torch.float32), _chk(a_bias, "a_bias", torch.float32),
                                           _chk(wa, "wa", torch.float32), _chk(b, "b", torch.float32),
                                           _chk(wb, "wb", torch.float32), float(eps), out.data_ptr(), R, H,
                                           _stream())
    native.check(st, "branch_norm_mean")
    return out


# ------------------------------------------- short convolutions, gated recurrence
def short_conv(proj: torch.Tensor, col0: int, channels: int, bias: Optional[torch.Tensor], filters_t: torch.Tensor,
               conv_bias: Optional[torch.Tensor], state: Optional[torch.Tensor], batch, also_bf16: bool = False,
               activation: Optional[str] = None, update_state: bool = False):
    """A causal convolution over time of columns [col0, col0 + channels) of
    `proj` (float32 [R, ld]) plus `bias`, one filter a channel (`filters_t`
    float32 [taps, channels], transposed; the last tap on the current token)
    plus `conv_bias`; what lies before a step's rows comes from `state` ([slots,
    n] float32, whose first (taps - 1) * channels floats are the sequence's last
    inputs, oldest first).  float32 [R, channels]; with `also_bf16` a pair, the
    second the same values rounded to bfloat16.  `activation` "silu": y / (1 +
    e^-y) of the result (after `conv_bias`).  `update_state`: the step has one
    row a sequence, and the launch also moves each sequence's last inputs on by
    its row (no `conv_state_update` is then needed)."""
    if update_state and proj.shape[0] != batch.seq_slot.numel():
        raise InvalidInput("short_conv: update_state is for steps of one row a sequence")
    if activation not in (None, "silu"):
        raise InvalidInput(f"short_conv: activation must be None or 'silu', got {activation!r}")
    R = proj.shape[0]
    taps = filters_t.shape[0]
    if filters_t.shape[1] != channels:
        raise InvalidInput("short_conv: the filters must be [taps, channels]")
    out = _new((R, channels), torch.float32, proj.device)
    lo = _new((R, channels), torch.bfloat16, proj.device) if also_bf16 else None
    st = native.lib().rfx_short_conv_act(
        _chk(proj, "proj", torch.float32), proj.shape[1], int(col0), _chk(bias, "bias", torch.float32),
        _chk(filters_t, "filters_t", torch.float32), _chk(conv_bias, "conv_bias", torch.float32), taps,
        _chk(state, "state", torch.float32), state.stride(0) if state is not None else 0,
        _chk(batch.row_slot, "row_slot", torch.int32), out.data_ptr(), lo.data_ptr() if lo is not None else 0,
        R, channels, 1 if activation == "silu" else 0, 1 if update_state else 0, _stream())
    native.check(st, f"short_conv (taps={taps})")
    return (out, lo) if also_bf16 else out


def conv_state_update(proj: torch.Tensor, col0: int, channels: int, bias: Optional[torch.Tensor], taps: int,
                      state: torch.Tensor, batch) -> None:
    """After a step's rows have been convolved: the sequences' new last taps - 1
    inputs into `state`."""
    if taps <= 1:
        return
    st = native.lib().rfx_conv_state_update(
        _chk(proj, "proj", torch.float32), proj.shape[1], int(col0), _chk(bias, "bias", torch.float32), int(taps),
        _chk(state, "state", torch.float32), state.stride(0), _chk(batch.seq_slot, "seq_slot", torch.int32),
        _chk(batch.seq_row0, "seq_row0", torch.int32), batch.seq_slot.numel(), channels, _stream())
    native.check(st, "conv_state_update")


def conv_qkv_post(proj: torch.Tensor, bias: Optional[torch.Tensor], filters_t: torch.Tensor,
                  state: Optional[torch.Tensor], batch, k_pages, v_pages, page_table, page_size: int, nq: int,
                  nkv: int, dim: int, vdim: int, pad: int, temp_coef: float, temp_every: int, writes_cache: bool,
                  out_dtype: torch.dtype, col0: int = 0) -> torch.Tensor:
    """The stacked q | k | v columns of `proj` (float32) plus `bias` through
    their short convolutions (`filters_t` float32 [taps, channels]); q times the
    temperature 1 + coef * ln(floor((p + 1) / every) + 1) at position p, out as
    [R, nq * pad]; k and v into the cache at the rows' positions, heads `pad`
    wide (zeros beyond `dim` and `vdim`).  `col0`: where the q | k | v columns
    begin in `proj` (a product stacked with others')."""
    R = proj.shape[0]
    taps = filters_t.shape[0]
    if filters_t.shape[1] != nq * dim + nkv * (dim + vdim):
        raise InvalidInput("conv_qkv_post: the filters must be [taps, channels of q, k and v]")
    q = _new((R, nq * pad), out_dtype, proj.device)
    if not (0 <= col0 <= proj.shape[1] - filters_t.shape[1]):
        raise InvalidInput("conv_qkv_post: the q | k | v columns do not fit into proj")
    st = native.lib().rfx_conv_qkv_post(
        _chk(proj, "proj", torch.float32) + 4 * int(col0), proj.shape[1], _chk(bias, "bias", torch.float32),
        _chk(filters_t, "filters_t", torch.float32), taps, _chk(state, "state", torch.float32),
        state.stride(0) if state is not None else 0, _chk(batch.row_pos, "row_pos", torch.int32),
        _chk(batch.row_slot, "row_slot", torch.int32), q.data_ptr(), _chk(k_pages, "k_pages", out_dtype),
        _chk(v_pages, "v_pages", out_dtype), dt_code(out_dtype), _chk(page_table, "page_table", torch.int32),
        page_table.shape[1], page_size, R, nq, nkv, dim, vdim, pad, float(temp_coef), int(temp_every),
        1 if writes_cache else 0, _stream())
    native.check(st, f"conv_qkv_post (dim={dim}, vdim={vdim})")
    return q


RGLRU_CHUNK_MIN_ROWS = _env_int("REFLEX_B200_RGLRU_CHUNK_MIN_ROWS", 16, 1, 1 << 30)


def rglru_scan(u: torch.Tensor, gates: torch.Tensor, r_bias, i_bias, lam: torch.Tensor, decay_scale: float,
               proj: torch.Tensor, y_off: int, y_bias, state: torch.Tensor, state_off: int, batch, blocks: int,
               out_dtype: torch.dtype, max_rows: Optional[int] = None, conv_tail=None) -> torch.Tensor:
    """The gated linear recurrence over the step's rows, sequence by sequence
    (csrc/rglru.cu): `u` float32 [R, W] its input, `gates` float32 [R, blocks,
    2 W / blocks] the two gates' pre-activations, `proj` holds the other
    branch's pre-activation at column `y_off`; the running S is `state[slot,
    state_off : state_off + W]`.  Returns S * gelu_tanh(y), [R, W].  `max_rows`:
    the most rows any sequence brings; from `RGLRU_CHUNK_MIN_ROWS` on the kernel
    that folds 128 rows at a time runs, else the row-by-row walk: the same
    function, rounded differently.  `conv_tail` = (x_off, x_bias, taps,
    tail_off): the kernel also stores the sequences' new last taps - 1 inputs of
    the convolution that made `u` (columns x_off.. of `proj` plus `x_bias`) at
    `state[slot, tail_off:]`, what `conv_state_update` does in a launch of its own."""
    R, W = u.shape
    chunked = max_rows is not None and max_rows >= RGLRU_CHUNK_MIN_ROWS
    x_off, x_bias, taps, tail_off = conv_tail if conv_tail is not None else (-1, None, 1, 0)
    out = _new((R, W), out_dtype, u.device)
    st = native.lib().rfx_rglru_scan(
        _chk(u, "u", torch.float32), _chk(gates, "gates", torch.float32), _chk(r_bias, "r_bias", torch.float32),
        _chk(i_bias, "i_bias", torch.float32), _chk(lam, "lam", torch.float32), float(decay_scale),
        _chk(proj, "proj", torch.float32), proj.shape[1], int(y_off), _chk(y_bias, "y_bias", torch.float32),
        _chk(state, "state", torch.float32), state.stride(0), int(state_off),
        _chk(batch.seq_slot, "seq_slot", torch.int32), _chk(batch.seq_row0, "seq_row0", torch.int32),
        batch.seq_slot.numel(), out.data_ptr(), dt_code(out_dtype), W, int(blocks), 1 if chunked else 0,
        int(x_off), _chk(x_bias, "x_bias", torch.float32), int(taps), int(tail_off), _stream())
    native.check(st, f"rglru_scan (width={W}, blocks={blocks})")
    return out


# -------------------------------------------------------- several residual streams
def hyper_expand(x: torch.Tensor, streams: int) -> torch.Tensor:
    """The embedding output [R, W] copied into every one of `streams` residual
    streams, float32 [R, streams * W]; lives for the whole step."""
    R, W = x.shape
    out = _new((R, streams * W), torch.float32, x.device, keep=True)
    st = native.lib().rfx_hyper_expand(_chk(x, "x", torch.float32), out.data_ptr(), R, int(streams), W, _stream())
    native.check(st, f"hyper_expand (streams={streams})")
    return out


class StreamWrite:
    """A sublayer's result that still has to go into the residual streams:
    x_t <- sum_s mix[s, t] x_s + out[t] * (scale * y), with `y` [R, W], `scale`
    float32 [W] or None, `mix` float32 [S, S] (from, to), `out` float32 [S]."""

    def __init__(self, y: torch.Tensor, scale: Optional[torch.Tensor], mix: torch.Tensor, out: torch.Tensor):
        self.y, self.scale, self.mix, self.out = y, scale, mix, out


def hyper_step(streams: torch.Tensor, write: Optional["StreamWrite"], read: torch.Tensor, norm_weight: torch.Tensor,
               eps: float, weight_offset: float, out_dtype: torch.dtype, n_streams: int) -> torch.Tensor:
    """`streams` float32 [R, S * W], updated in place by `write` (if any); then
    u = sum_s read[s] x_s and its RMS norm, u / sqrt(mean(u^2) + eps) *
    (weight_offset + norm_weight), [R, W] in `out_dtype`: one launch."""
    R = streams.shape[0]
    S = int(n_streams)
    W = streams.shape[1] // S
    out = _new((R, W), out_dtype, streams.device)
    y = write.y if write is not None else None
    if y is not None and tuple(y.shape) != (R, W):
        raise InvalidInput("hyper_step: the sublayer's result must be [rows, width]")
    st = native.lib().rfx_hyper_step(
        _chk(streams, "streams", torch.float32), _chk(y, "y"), dt_code(y.dtype) if y is not None else 0,
        _chk(write.scale, "scale", torch.float32) if write is not None else 0,
        _chk(write.mix, "mix", torch.float32) if write is not None else 0,
        _chk(write.out, "out", torch.float32) if write is not None else 0,
        _chk(read, "read", torch.float32), _chk(norm_weight, "norm_weight", torch.float32), float(eps),
        float(weight_offset), out.data_ptr(), dt_code(out_dtype), R, S, W, _stream())
    native.check(st, f"hyper_step (streams={S}, width={W})")
    return out


def hyper_collapse(streams: torch.Tensor, write: Optional["StreamWrite"], n_streams: int,
                   rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The sum of the residual streams after `write` (if any), float32 [R, W];
    `streams` itself is left as it is.  `rows` (int32 on the device): only those
    rows, in that order, [len(rows), W]."""
    R = streams.shape[0] if rows is None else rows.numel()
    S = int(n_streams)
    W = streams.shape[1] // S
    out = _new((R, W), torch.float32, streams.device, keep=True)
    y = write.y if write is not None else None
    st = native.lib().rfx_hyper_collapse(
        _chk(streams, "streams", torch.float32), _chk(y, "y"), dt_code(y.dtype) if y is not None else 0,
        _chk(write.scale, "scale", torch.float32) if write is not None else 0,
        _chk(write.mix, "mix", torch.float32) if write is not None else 0,
        _chk(write.out, "out", torch.float32) if write is not None else 0, out.data_ptr(),
        _chk(rows, "rows", torch.int32), R, S, W, _stream())
    native.check(st, f"hyper_collapse (streams={S}, width={W})")
    return out


# ------------------------------------------------------------ gates, activations
def sigmoid_gate_mul_(a: torch.Tensor, z: torch.Tensor, col: int) -> torch.Tensor:
    """a[r, c] *= sigmoid(z[r, col + c]), in place; the sigmoid is 32-bit."""
    R, H = a.shape
    if col < 0 or col + H > z.shape[1] or z.shape[0] != R:
        raise InvalidInput("sigmoid_gate_mul: the gate's columns do not fit into z")
    st = native.lib().rfx_sigmoid_gate_mul(_chk(a, "a"), dt_code(a.dtype), _chk(z, "z"), dt_code(z.dtype),
                                           z.shape[1], int(col), R, H, _stream())
    native.check(st, "sigmoid_gate_mul")
    return a


def relu2_(a: torch.Tensor) -> torch.Tensor:
    """a <- max(a, 0)^2, in place."""
    st = native.lib().rfx_moe_activation(_chk(a, "a"), dt_code(a.dtype), a.numel(), MOE_ACTIVATIONS["relu2"],
                                         _stream())
    native.check(st, "relu2")
    return a


def linear_relu2(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """relu(x @ W.T)^2, [R, I] in x's dtype.  For a few bfloat16 rows the
    activation is the product kernel's epilogue (on the 32-bit sums, rounded
    once); otherwise product, then the activation in place."""
    R, K = x.shape
    if x.dtype == torch.bfloat16 and R <= GEMV_MAX_ROWS and K % 8 == 0 and FUSE_GLU:
        N = weight.shape[0]
        _chk(x, "x", torch.bfloat16)
        _chk(weight, "weight", torch.bfloat16)
        y = _new((R, N), torch.bfloat16, x.device)
        st = native.lib().rfx_gemm_bf16_tc_relu2(
            x.data_ptr(), weight.data_ptr(), y.data_ptr(), BF16, R, N, K, 0,
            device_error_word(x.device).data_ptr(), _stream())
        native.check(st, f"gemm_bf16_tc_relu2 (R={R}, N={N}, K={K})")
        return y
    return relu2_(linear(x, weight))


# ------------------------------------------------------------- selective scan
def mamba_scan(x: torch.Tensor, dtpre: torch.Tensor, dt_bias: Optional[torch.Tensor], bc: torch.Tensor, b_off: int,
               c_off: int, z: torch.Tensor, z_off: int, A: torch.Tensor, D: Optional[torch.Tensor],
               state: torch.Tensor, state_off: int, batch, out_dtype: torch.dtype,
               dt_weight: Optional[torch.Tensor] = None, dt_low_off: int = 0) -> torch.Tensor:
    """The selective scan over the step's rows, sequence by sequence
    (csrc/mamba.cu): `x`, `dtpre` float32 [R, channels]; `bc` float32 rows with B
    at column `b_off` and C at `c_off` (N each); `z` float32 rows with the gate's
    pre-activation at `z_off`; `A` float32 [channels, N]; the running state is
    `state[slot, state_off : state_off + channels * N]`.  Returns (S . C + D x) *
    silu(z), [R, channels] in `out_dtype`.  With `dt_weight` ([channels, rank],
    float32 or bfloat16; steps of a row or two a sequence only) `dtpre` is None:
    the rows of `bc` hold the step sizes' low-rank vector at column `dt_low_off`
    and the kernel makes dtpre = dt_weight . vector itself (the vector rounded to
    bfloat16 first where the weights are bfloat16)."""
    R, C = x.shape
    N = A.shape[1]
    if dt_weight is None:
        if dtpre is None or tuple(dtpre.shape) != (R, C):
            raise InvalidInput("mamba_scan: dtpre must be [rows, channels]")
    elif dt_weight.shape[0] != C or dt_low_off + dt_weight.shape[1] > bc.shape[1] or \
            dt_weight.dtype not in (torch.float32, torch.bfloat16):
        raise InvalidInput("mamba_scan: dt_weight must be [channels, rank] and its vector fit into the rows of bc")
    if A.shape[0] != C or x.dtype != torch.float32:
        raise InvalidInput("mamba_scan: x must be float32 [rows, channels] and A [channels, states]")
    if max(b_off, c_off) + N > bc.shape[1] or z_off + C > z.shape[1]:
        raise InvalidInput("mamba_scan: B, C or z do not fit into their rows")
    out = _new((R, C), out_dtype, x.device)
    n_seq = batch.seq_slot.numel()
    # a prompt's rows are cut into segments that run side by side: their folded states
    want = int(native.lib().rfx_mamba_scan_scratch(n_seq, R, C, N))
    scratch = _new((want,), torch.float32, x.device) if want > 0 else None
    st = native.lib().rfx_mamba_scan(
        _chk(x, "x", torch.float32), _chk(dtpre, "dtpre", torch.float32), _chk(dt_bias, "dt_bias", torch.float32),
        _chk(bc, "bc", torch.float32), bc.shape[1], int(b_off), int(c_off), _chk(z, "z", torch.float32),
        z.shape[1], int(z_off), _chk(A, "A", torch.float32), _chk(D, "D", torch.float32),
        _chk(state, "state", torch.float32), state.stride(0), int(state_off),
        _chk(batch.seq_slot, "seq_slot", torch.int32), _chk(batch.seq_row0, "seq_row0", torch.int32),
        n_seq, R, out.data_ptr(), dt_code(out_dtype), C, N, scratch.data_ptr() if scratch is not None else None,
        _chk(dt_weight, "dt_weight"), dt_code(dt_weight.dtype) if dt_weight is not None else 0,
        dt_weight.shape[1] if dt_weight is not None else 0, int(dt_low_off), _stream())
    native.check(st, f"mamba_scan (channels={C}, states={N})")
    return out


# ------------------------------------------- norms around a sublayer, small companions
def sandwich_norm(y: torch.Tensor, x: torch.Tensor, post_weight: torch.Tensor, mult: float, eps: float,
                  next_weight: Optional[torch.Tensor], next_eps: float, out_dtype: torch.dtype):
    """x <- x + mult * rms_norm(y) * post_weight in place (`y`, `x` float32 [R, H]);
    with `next_weight` also returns rms_norm(x) * next_weight in `out_dtype`: the
    norm after one sublayer and the norm before the next in one pass over the row."""
    R, H = x.shape
    if tuple(y.shape) != (R, H):
        raise InvalidInput("sandwich_norm: y and x must have the same shape")
    out = _new((R, H), out_dtype, x.device) if next_weight is not None else None
    st = native.lib().rfx_sandwich_norm(
        _chk(y, "y", torch.float32), _chk(x, "x", torch.float32), _chk(post_weight, "post_weight", torch.float32),
        float(mult), float(eps), _chk(next_weight, "next_weight", torch.float32), float(next_eps),
        out.data_ptr() if out is not None else 0, dt_code(out_dtype), R, H, _stream())
    native.check(st, f"sandwich_norm (H={H})")
    return out


def group_norm_gate(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out_dtype: torch.dtype,
                    gate: Optional[torch.Tensor] = None, gate_col: int = 0) -> torch.Tensor:
    """`x` float32 [R, C] in `groups` equal parts, each divided by its own root mean
    square, times weight[c]; with `gate` (float32 rows, the gate's pre-activations
    from column `gate_col` on) also times their sigmoid."""
    R, C = x.shape
    if C % groups or weight.numel() != C:
        raise InvalidInput("group_norm_gate: the groups must divide the row and the weight match it")
    if gate is not None and gate_col + C > gate.shape[1]:
        raise InvalidInput("group_norm_gate: the gate's columns do not fit into its rows")
    out = _new((R, C), out_dtype, x.device)
    st = native.lib().rfx_group_norm_gate(
        _chk(x, "x", torch.float32), _chk(weight, "weight", torch.float32), float(eps),
        _chk(gate, "gate", torch.float32), gate.shape[1] if gate is not None else 0, int(gate_col),
        out.data_ptr(), dt_code(out_dtype), R, C, int(groups), _stream())
    native.check(st, f"group_norm_gate (C={C}, groups={groups})")
    return out


def xielu_(a: torch.Tensor, alpha_pos: float, alpha_neg: float) -> torch.Tensor:
    """In place: z > 0: alpha_pos z^2 + z / 2; else alpha_neg (e^z - 1 - z) + z / 2."""
    st = native.lib().rfx_xielu(_chk(a, "a"), dt_code(a.dtype), a.numel(), float(alpha_pos), float(alpha_neg),
                                _stream())
    native.check(st, "xielu")
    return a


def linear_xielu(x: torch.Tensor, weight: torch.Tensor, alpha_pos: float, alpha_neg: float) -> torch.Tensor:
    """xielu(x @ W.T), [R, I] in x's dtype.  For a few bfloat16 rows the activation is
    the product kernel's epilogue (on the 32-bit sums, rounded once); otherwise product,
    then the activation in place."""
    R, K = x.shape
    if (x.dtype == torch.bfloat16 and R <= GEMV_MAX_ROWS and K % 8 == 0 and FUSE_GLU
            and (x.data_ptr() | weight.data_ptr()) % 16 == 0):
        N = weight.shape[0]
        _chk(x, "x", torch.bfloat16)
        _chk(weight, "weight", torch.bfloat16)
        y = _new((R, N), torch.bfloat16, x.device)
        st = native.lib().rfx_gemm_bf16_tc_xielu(
            x.data_ptr(), weight.data_ptr(), y.data_ptr(), BF16, R, N, K, 0, float(alpha_pos), float(alpha_neg),
            device_error_word(x.device).data_ptr(), _stream())
        native.check(st, f"gemm_bf16_tc_xielu (R={R}, N={N}, K={K})")
        return y
    return xielu_(linear(x, weight), alpha_pos, alpha_neg)


def loop_input_(x: torch.Tensor, x0: Optional[torch.Tensor], vec: torch.Tensor) -> torch.Tensor:
    """x[r] += x0[r] (when given) + vec, float32: the start of a pass over a repeated stretch."""
    R, H = x.shape
    if vec.numel() != H or (x0 is not None and x0.shape != x.shape):
        raise InvalidInput("loop_input: the vector must match a row and x0 the rows")
    st = native.lib().rfx_loop_input(_chk(x, "x", torch.float32), _chk(x0, "x0", torch.float32),
                                     _chk(vec, "vec", torch.float32), R, H, _stream())
    native.check(st, "loop_input")
    return x


def tanh_cols(rows: torch.Tensor, col: int, n: int, out_dtype: torch.dtype) -> torch.Tensor:
    """tanh of columns [col, col + n) of float32 `rows`, [R, n] in `out_dtype`."""
    R, ld = rows.shape
    if col + n > ld:
        raise InvalidInput("tanh_cols: the columns do not fit into the rows")
    out = _new((R, n), out_dtype, rows.device)
    st = native.lib().rfx_tanh_cols(_chk(rows, "rows", torch.float32), ld, int(col), out.data_ptr(),
                                    dt_code(out_dtype), R, int(n), _stream())
    native.check(st, "tanh_cols")
    return out


def scaled_sum_(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float) -> torch.Tensor:
    """a <- sa * a + sb * b, both float32."""
    if a.shape != b.shape:
        raise InvalidInput("scaled_sum: shapes differ")
    st = native.lib().rfx_scaled_sum(_chk(a, "a", torch.float32), _chk(b, "b", torch.float32), float(sa), float(sb),
                                     a.numel(), _stream())
    native.check(st, "scaled_sum")
    return a


# ------------------------------------------- attention with sigmoid weights
def sig_qkv_post(proj: torch.Tensor, col0: int, rotation, row_pos: torch.Tensor, row_slot: torch.Tensor,
                 k_pages, v_pages, page_table: torch.Tensor, page_size: int, nq: int, nkv: int, dim: int,
                 vdim: int, writes_cache: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """Columns [q | k | v] of `proj` from `col0` on (keys `dim` wide, values `vdim`):
    the rotation of q and k (a half-split `parts.Rotation` or None), q out
    [R, nq * dim], k and v into their pages at the rows' positions."""
    R = proj.shape[0]
    need = nq * dim + (nkv * (dim + vdim) if writes_cache else 0)
    if col0 + need > proj.shape[1]:
        raise InvalidInput("sig_qkv_post: the q | k | v columns do not fit into the rows")
    denom, rot = None, 0
    if rotation is not None:
        if rotation.pairing != "half" or rotation.magnitude != 1.0:
            raise InvalidInput("sig_qkv_post: takes a plain half-split rotation")
        denom, rot = rotation.denominators, int(rotation.rotary_dim)
    q = _new((R, nq * dim), out_dtype, proj.device)
    st = native.lib().rfx_sig_qkv_post(
        _chk(proj, "proj"), dt_code(proj.dtype), proj.shape[1], int(col0), _chk(denom, "denominators", torch.float32),
        rot, _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), q.data_ptr(),
        _chk(k_pages, "k_pages", out_dtype), _chk(v_pages, "v_pages", out_dtype), dt_code(out_dtype),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size, R, nq, nkv, dim, vdim,
        1 if writes_cache else 0, _stream())
    native.check(st, f"sig_qkv_post (dim={dim}, vdim={vdim})")
    return q


def attention_sigmoid_plain(q, k_pages, v_pages, page_table, page_size, row_pos, row_slot, nq, nkv, dim, vdim,
                            window, scale, bias) -> torch.Tensor:
    """out = sum over the visible keys of sigmoid(q . k * scale + bias[head]) v, a
    warp per (row, head): the 32-bit path and every head size up to 512."""
    R = q.shape[0]
    out = _new((R, nq * vdim), q.dtype, q.device)
    st = native.lib().rfx_attention_sigmoid_plain(
        _chk(q, "q"), _chk(k_pages, "k_pages", q.dtype), _chk(v_pages, "v_pages", q.dtype), dt_code(q.dtype),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), out.data_ptr(), R, nq, nkv,
        dim, vdim, int(window or 0), float(scale), _chk(bias, "bias", torch.float32), _stream())
    native.check(st, f"attention_sigmoid_plain (dim={dim}, vdim={vdim})")
    return out


def attention_sigmoid_mma(q, k_pages, v_pages, page_table, page_size, seq_slot, seq_start, seq_new, seq_row0,
                          max_new: int, nq, nkv, dim, vdim, window, scale, bias) -> torch.Tensor:
    """The bfloat16 tensor-core form (csrc/sigmoid_attention_mma.cu) for a packed batch of
    sequences that each bring one or more rows: key sizes in steps of 8 up to 256, value
    sizes up to 128, up to 128 query heads a key head."""
    _chk(q, "q", torch.bfloat16)
    R = q.shape[0]
    out = _new((R, nq * vdim), q.dtype, q.device)
    st = native.lib().rfx_attention_sigmoid_mma(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(seq_slot, "seq_slot", torch.int32), _chk(seq_start, "seq_start", torch.int32),
        _chk(seq_new, "seq_new", torch.int32), _chk(seq_row0, "seq_row0", torch.int32), out.data_ptr(),
        seq_slot.numel(), int(max_new), nq, nkv, dim, vdim, int(window or 0), float(scale),
        _chk(bias, "bias", torch.float32), _stream())
    native.check(st, f"attention_sigmoid_mma (dim={dim}, vdim={vdim})")
    return out


def attention_sigmoid(q, k_pages, v_pages, page_table, page_size, batch, nq, nkv, dim, vdim, window, scale, bias):
    """Attention with sigmoid weights for the step's rows; picks the kernel."""
    if (q.dtype == torch.bfloat16 and dim % 8 == 0 and vdim % 8 == 0 and dim <= 256 and vdim <= 128
            and nq // nkv <= 128 and page_size == 64):
        return attention_sigmoid_mma(q, k_pages, v_pages, page_table, page_size, batch.seq_slot, batch.seq_start,
                                     batch.seq_new, batch.seq_row0, batch.max_new, nq, nkv, dim, vdim, window,
                                     scale, bias)
    return attention_sigmoid_plain(q, k_pages, v_pages, page_table, page_size, batch.row_pos, batch.row_slot,
                                   nq, nkv, dim, vdim, window, scale, bias)


# ------------------------------------------- recurrences with a matrix state a head
def ssd_scan(xbc: torch.Tensor, proj: torch.Tensor, z_off: int, dt_off: int, dt_bias: torch.Tensor, A: torch.Tensor,
             D: Optional[torch.Tensor], state: torch.Tensor, state_off: int, batch, heads: int, vdim: int,
             states: int, groups: int, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The state-space recurrence with one decay a head (csrc/ssd.cu): `xbc` float32
    rows [x | B | C], `proj` float32 rows with z at `z_off` and the step sizes'
    pre-activations at `dt_off`; `A` float32 [heads], negative; the running state is
    `state[slot, state_off : state_off + heads * states * vdim]`.  Returns
    (S^T C + D x) * silu(z), [R, heads * vdim]."""
    R = xbc.shape[0]
    inner = heads * vdim
    if xbc.shape[1] != inner + 2 * groups * states:
        raise InvalidInput("ssd_scan: xbc must be [rows, heads * vdim + 2 * groups * states]")
    if z_off + inner > proj.shape[1] or dt_off + heads > proj.shape[1]:
        raise InvalidInput("ssd_scan: z or dt do not fit into the rows of proj")
    out = _new((R, inner), out_dtype, xbc.device)
    st = native.lib().rfx_ssd_scan(
        _chk(xbc, "xbc", torch.float32), xbc.shape[1], _chk(proj, "proj", torch.float32), proj.shape[1], int(z_off),
        int(dt_off), _chk(dt_bias, "dt_bias", torch.float32), _chk(A, "A", torch.float32), _chk(D, "D", torch.float32),
        _chk(state, "state", torch.float32), state.stride(0), int(state_off),
        _chk(batch.seq_slot, "seq_slot", torch.int32), _chk(batch.seq_row0, "seq_row0", torch.int32),
        batch.seq_slot.numel(), out.data_ptr(), dt_code(out_dtype), heads, vdim, states, groups, _stream())
    native.check(st, f"ssd_scan (heads={heads}, vdim={vdim}, states={states})")
    return out


def delta_rule(proj: torch.Tensor, r_off: int, k_off: int, v_off: int, a_off: int, wpre: torch.Tensor,
               w_bias: torch.Tensor, a_bias: torch.Tensor, rate: float, unit_eps: float, state: torch.Tensor,
               state_off: int, batch, heads: int, dim: int) -> torch.Tensor:
    """The generalized delta rule (csrc/delta_rule.cu): `proj` float32 rows with r, k,
    v and the removal rate's pre-activation at their column offsets (heads * dim
    each), `wpre` float32 [R, heads * dim] the decay's; the running state is
    `state[slot, state_off : state_off + heads * dim * dim]`.  Returns S^T r,
    float32 [R, heads * dim]."""
    R = proj.shape[0]
    hd = heads * dim
    if max(r_off, k_off, v_off, a_off) + hd > proj.shape[1] or tuple(wpre.shape) != (R, hd):
        raise InvalidInput("delta_rule: the columns do not fit into the rows")
    out = _new((R, hd), torch.float32, proj.device)
    st = native.lib().rfx_delta_rule(
        _chk(proj, "proj", torch.float32), proj.shape[1], int(r_off), int(k_off), int(v_off), int(a_off),
        _chk(wpre, "wpre", torch.float32), _chk(w_bias, "w_bias", torch.float32), _chk(a_bias, "a_bias", torch.float32),
        float(rate), float(unit_eps), _chk(state, "state", torch.float32), state.stride(0), int(state_off),
        _chk(batch.seq_slot, "seq_slot", torch.int32), _chk(batch.seq_row0, "seq_row0", torch.int32),
        batch.seq_slot.numel(), out.data_ptr(), dt_code(torch.float32), heads, dim, _stream())
    native.check(st, f"delta_rule (heads={heads}, dim={dim})")
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None,
           scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit per row (ties: the highest index).  `out`
    (int32 [B]) and `scratch` (float32, B * 128) may be given to spare the
    allocations of a call a step."""
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    if scratch is None:
        scratch = torch.empty((B * 64 * 2,), dtype=torch.float32, device=logits.device)
    st = native.lib().rfx_argmax(logits.data_ptr(), V, B, V, _chk(out, "out", torch.int32),
                                 _chk(scratch, "scratch", torch.float32), _stream())
    native.check(st, "argmax")
    return out


def sample_work_bytes(B: int, V: int) -> int:
    """Bytes of working memory `sample` needs for B rows of V entries."""
    return int(native.lib().rfx_sample_work_bytes(int(B), int(V)))


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           work: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token a row: temperature softmax, optional top-k and top-p cuts, and an
    inverse-CDF draw with the row's uniform number.  `scratch` (float32 [B, V])
    and `work` (uint8, `sample_work_bytes(B, V)`) may be given to spare the
    allocations of a call a step."""
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    if scratch is None:
        scratch = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    need = sample_work_bytes(B, V)
    if work is None:
        work = torch.empty((need,), dtype=torch.uint8, device=logits.device)
    elif work.numel() < need or work.dtype != torch.uint8:
        raise InvalidInput(f"sample: work must hold {need} bytes")
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    _chk(out, "out", torch.int32)
    st = native.lib().rfx_sample(
        logits.data_ptr(), V, B, V, _chk(temperature, "temperature", torch.float32),
        _chk(top_k, "top_k", torch.int32), _chk(top_p, "top_p", torch.float32),
        _chk(uniform, "uniform", torch.float32), _chk(scratch, "scratch", torch.float32),
        _chk(work, "work", torch.uint8), out.data_ptr(), _stream())
    native.check(st, "sample")
    return out

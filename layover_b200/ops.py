"""The engine's device operations: thin, checked wrappers over the CUDA kernels of `csrc/`.

Every function takes CUDA tensors, launches on torch's current stream and returns without
synchronising. There is no other implementation behind them: if the kernels cannot be
compiled or loaded, or a tensor is not on a CUDA device, the call raises. A size or alignment
that a kernel does not support is refused with a ValueError before or by the launch.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from .csrc import build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_REFUSALS = {-1: "unsupported dtype", -2: "unsupported size", -3: "unsupported alignment"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; the engine runs float32 or bfloat16") from None


LAUNCHES = 0   # kernels of this package launched (or captured into a graph) so far


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code in _REFUSALS:
        raise ValueError(f"{what}: {_REFUSALS[code]}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("layover_b200 kernels need CUDA tensors: there is no CPU path")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


_signatures_done: set[str] = set()


def _fn(lib_name: str, fn_name: str, argtypes):
    lib = build.load(lib_name)
    fn = getattr(lib, fn_name)
    key = lib_name + "." + fn_name
    if key not in _signatures_done:
        fn.argtypes = argtypes
        fn.restype = c_int
        _signatures_done.add(key)
    return fn


# ------------------------------------------------------------------ elementwise
RECORD_WORDS = 8                 # int32 words of a request's record on the device (csrc/common.cuh)
RECORD_POSITION, RECORD_SEED_LO, RECORD_SEED_HI, RECORD_COUNT, RECORD_TEMPERATURE, RECORD_LAST_TOKEN = range(6)


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, token_src: torch.Tensor | None = None,
          records: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[id]; ids int32 [T], table [V, H], out [T, H] of the table's type, or float32 (a
    32-bit residual stream). Where token_src[t] >= 0 the id is the last token in row token_src[t] of
    `records` (int32 [slots, RECORD_WORDS]) instead of ids[t]."""
    _need(ids, torch.int32, "ids"); _need(table, None, "table")
    wide = out.dtype == torch.float32 and table.dtype != torch.float32     # a 32-bit residual stream over a narrower table
    _need(out, torch.float32 if wide else table.dtype, "out")
    if (token_src is None) != (records is None):
        raise ValueError("embed: token_src and records come together")
    if token_src is not None:
        _need(token_src, torch.int32, "token_src"); _need(records, torch.int32, "records")
        if records.dim() != 2 or records.shape[1] != RECORD_WORDS or token_src.shape[0] != ids.shape[0]:
            raise ValueError("embed: records must be [slots, RECORD_WORDS] and token_src one entry per token")
    fn = _fn("elementwise", "lb_embed_wide" if wide else "lb_embed",
             [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(table.dtype), _ptr(ids), _ptr(token_src), _ptr(records), _ptr(table), _ptr(out), ids.shape[0],
              table.shape[1], table.shape[0], _stream()), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (in place, unless `rows` picks source rows), out = rmsnorm(x) * weight.

    x, delta [T, H]; weight float32 [H]; out [T or len(rows), H]."""
    _need(x, None, "x"); _need(weight, torch.float32, "weight"); _need(out, x.dtype, "out")
    if delta is not None:
        _need(delta, x.dtype, "delta")
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if out.shape[0] < n_rows or out.shape[-1] != x.shape[-1] or weight.shape[0] != x.shape[-1]:
        raise ValueError("add_rmsnorm: shapes do not agree")
    fn = _fn("elementwise", "lb_add_rmsnorm",
             [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_rows, x.shape[-1],
              float(eps), _stream()), "add_rmsnorm")
    return out


def residual_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, delta_weight: torch.Tensor | None, delta_eps: float,
                     extra: torch.Tensor | None, weight: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                     rows: torch.Tensor | None = None, delta_scale: float = 1.0) -> torch.Tensor | None:
    """The add + RMSNorm of a 32-bit residual stream x (float32 [T, H], updated in place unless `rows`
    picks source rows):

        x += delta_scale * (delta * delta_weight * rsqrt(mean(delta^2) + delta_eps))     (delta_weight None: x += delta)
        x += extra                                                       (float32 [T, H], e.g. the embedding output)
        out = weight * x * rsqrt(mean(x^2) + eps)                        (weight None: out = x in the run's type, or no output)

    delta and out are in the run's type (bfloat16 or float32); all arithmetic is 32-bit."""
    _need(x, torch.float32, "x")
    hidden = x.shape[-1]
    run = out.dtype if out is not None else (delta.dtype if delta is not None else torch.float32)
    if delta is not None:
        _need(delta, run, "delta")
        if delta.shape != x.shape:
            raise ValueError("residual_rmsnorm: delta must have x's shape")
    for name, t in (("delta_weight", delta_weight), ("weight", weight)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.shape[0] != hidden:
                raise ValueError(f"residual_rmsnorm: {name} must have one entry per channel")
    if extra is not None:
        _need(extra, torch.float32, "extra")
        if extra.shape != x.shape:
            raise ValueError("residual_rmsnorm: extra must have x's shape")
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if (weight is not None and out is None) or (out is not None and (out.shape[0] < n_rows or out.shape[-1] != hidden)):
        raise ValueError("residual_rmsnorm: a norm of the sum needs out [rows, H]")
    if delta_scale != 1.0 and delta_weight is None:
        raise ValueError("residual_rmsnorm: delta_scale scales a normed delta")
    if out is not None:
        _need(out, run, "out")
    fn = _fn("elementwise", "lb_residual_rmsnorm",
             [c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
              c_float, c_void_p])
    _check(fn(dtype_code(run), _ptr(x), _ptr(delta), _ptr(delta_weight), float(delta_eps), _ptr(extra), _ptr(weight),
              _ptr(out), _ptr(rows), n_rows, hidden, float(eps), float(delta_scale), _stream()), "residual_rmsnorm")
    return out


def qk_rownorm_kv(proj: torch.Tensor, q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                  q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None, slot_map: torch.Tensor,
                  gates: torch.Tensor | None, q_heads: int, kv_heads: int, dim: int, vdim: int, page_tokens: int,
                  eps: float) -> None:
    """RMSNorm of q and of k over the whole projection (all heads at once, a weight per channel), no
    rotation; q to q_out, k and v to their pages, sigmoid of the per-head gate logits to `gates`.

    proj [T, >= q_heads*dim + kv_heads*(dim + vdim) (+ q_heads)], rows may be padded; q_out [T, q_heads*R];
    k_pool [pages, kv_heads, page_tokens, R]; v_pool [pages, kv_heads, page_tokens, R]; gates float32 [T, q_heads].
    R is each tensor's own room per head, at least dim (vdim for values): what is beyond the head's
    channels is filled with zeros."""
    _need(q_out, proj.dtype, "q_out"); _need(k_pool, proj.dtype, "k_pool"); _need(v_pool, proj.dtype, "v_pool")
    _need(slot_map, torch.int32, "slot_map")
    tokens = proj.shape[0]
    used = q_heads * dim + kv_heads * (dim + vdim) + (q_heads if gates is not None else 0)
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < used or q_out.shape[0] != tokens or q_out.shape[1] % q_heads:
        raise ValueError("qk_rownorm_kv: the projection row does not hold these heads")
    q_room, k_room, v_room = q_out.shape[1] // q_heads, k_pool.shape[-1], v_pool.shape[-1]
    if tuple(k_pool.shape[1:3]) != (kv_heads, page_tokens) or tuple(v_pool.shape[1:3]) != (kv_heads, page_tokens) \
            or q_room < dim or k_room < dim or v_room < vdim:
        raise ValueError("qk_rownorm_kv: the pools do not match the heads")
    for name, t, n in (("q_norm_w", q_norm_w, q_heads * dim), ("k_norm_w", k_norm_w, kv_heads * dim)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != n:
                raise ValueError(f"qk_rownorm_kv: {name} must have {n} entries")
    if gates is not None:
        _need(gates, torch.float32, "gates")
        if tuple(gates.shape) != (tokens, q_heads):
            raise ValueError("qk_rownorm_kv: gates must be [tokens, q_heads]")
    fn = _fn("elementwise", "lb_qk_rownorm_kv",
             [c_int, c_void_p, c_long] + [c_void_p] * 7 + [c_int] * 6 + [c_float, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(proj.dtype), _ptr(proj), proj.stride(0), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_norm_w),
              _ptr(k_norm_w), _ptr(slot_map), _ptr(gates), tokens, q_heads, kv_heads, dim, vdim, page_tokens, float(eps),
              q_room, k_room, v_room, _stream()), "qk_rownorm_kv")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, 0, i] = cos(positions[t] * inv_freq[i]), out[t, 1, i] = sin(...); out float32 [T, 2, n_freq]."""
    _need(positions, torch.int32, "positions"); _need(inv_freq, torch.float32, "inv_freq"); _need(out, torch.float32, "out")
    tokens, n_freq = positions.shape[0], inv_freq.shape[0]
    if tuple(out.shape) != (tokens, 2, n_freq):
        raise ValueError("rope_table: out must be [tokens, 2, n_freq]")
    fn = _fn("elementwise", "lb_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(positions), _ptr(inv_freq), _ptr(out), tokens, n_freq, _stream()), "rope_table")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor | None, k_pool: torch.Tensor | None,
                    v_pool: torch.Tensor | None, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None,
                    table: torch.Tensor | None, slot_map: torch.Tensor | None, q_heads: int, kv_heads: int, dim: int,
                    page_tokens: int, eps: float) -> None:
    """Per-head norm and rotation of q and k in a fused projection row, q to q_out, k and v to their pages.

    qkv [T, (q_heads + 2 kv_heads) * dim]; q_out [T, q_heads * dim]; pools [pages, kv_heads, page_tokens, dim];
    table float32 [T, 2, dim / 2] from `rope_table` (None: no rotation)."""
    tokens = qkv.shape[0]
    _need(qkv, None, "qkv")
    if q_out is not None:
        _need(q_out, qkv.dtype, "q_out")
    if qkv.shape[1] != (q_heads + 2 * kv_heads) * dim:
        raise ValueError("qk_norm_rope_kv: projection row does not match the head counts")
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        if t is not None:
            _need(t, torch.float32, name)
    if table is not None and (table.dim() != 3 or table.shape[0] != tokens or table.shape[1] != 2):
        raise ValueError("qk_norm_rope_kv: the rotary table must be [tokens, 2, n_freq]")
    if k_pool is not None:
        _need(k_pool, qkv.dtype, "k_pool"); _need(v_pool, qkv.dtype, "v_pool"); _need(slot_map, torch.int32, "slot_map")
    n_freq = 0 if table is None else table.shape[2]
    fn = _fn("elementwise", "lb_qk_norm_rope_kv",
             [c_int] + [c_void_p] * 8 + [c_int] * 6 + [c_float, c_void_p])
    _check(fn(dtype_code(qkv.dtype), _ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_norm_w),
              _ptr(k_norm_w), _ptr(table), _ptr(slot_map), tokens, q_heads, kv_heads, dim, n_freq,
              page_tokens, float(eps), _stream()), "qk_norm_rope_kv")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> torch.Tensor:
    """out = silu(gate) * up, gate_up [T, 2 I], out [T, I]. block 0: the row is [all gates | all ups];
    block b: gates and ups alternate in blocks of b features (`interleave_gate_up`'s layout)."""
    _need(gate_up, None, "gate_up"); _need(out, gate_up.dtype, "out")
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] != 2 * inter or out.shape[1] != inter or out.shape[0] != gate_up.shape[0]:
        raise ValueError("swiglu: shapes do not agree")
    fn = _fn("elementwise", "lb_swiglu", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(gate_up.dtype), _ptr(gate_up), _ptr(out), gate_up.shape[0], inter, int(block), _stream()),
           "swiglu")
    return out


GATE_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str, block: int = 0) -> torch.Tensor:
    """out = act(gate) * up with act "silu", "relu" or "gelu_tanh"; layouts as `swiglu`."""
    _need(gate_up, None, "gate_up"); _need(out, gate_up.dtype, "out")
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] != 2 * inter or out.shape[1] != inter or out.shape[0] != gate_up.shape[0]:
        raise ValueError("gated_act: shapes do not agree")
    if activation not in GATE_ACTIVATIONS:
        raise ValueError(f"gated_act: unknown activation {activation!r}")
    fn = _fn("elementwise", "lb_gated_act", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(gate_up.dtype), _ptr(gate_up), _ptr(out), gate_up.shape[0], inter, int(block),
              GATE_ACTIVATIONS[activation], _stream()), "gated_act")
    return out


def residual_layernorm(x: torch.Tensor, delta_a: torch.Tensor | None, delta_b: torch.Tensor | None,
                       weight: torch.Tensor | None, bias: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                       rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """The add + LayerNorm of a 32-bit residual stream x (float32 [T, H], updated in place unless `rows`
    picks source rows):

        x += delta_a + delta_b                                   (either may be None: two sub-layers' outputs at once)
        out = (x - mean) * rsqrt(mean((x - mean)^2) + eps) * weight + bias       (weight None: no output)

    delta_a, delta_b and out are in the run's type (bfloat16 or float32); all arithmetic is 32-bit."""
    _need(x, torch.float32, "x")
    hidden = x.shape[-1]
    given = [t for t in (out, delta_a, delta_b) if t is not None]
    run = given[0].dtype if given else torch.float32
    for name, t in (("delta_a", delta_a), ("delta_b", delta_b)):
        if t is not None:
            _need(t, run, name)
            if t.shape != x.shape:
                raise ValueError(f"residual_layernorm: {name} must have x's shape")
    for name, t in (("weight", weight), ("bias", bias)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.shape[0] != hidden:
                raise ValueError(f"residual_layernorm: {name} must have one entry per channel")
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if (weight is None) != (out is None) or (out is not None and (out.shape[0] < n_rows or out.shape[-1] != hidden)):
        raise ValueError("residual_layernorm: weight and out come together, out [rows, H]")
    if out is not None:
        _need(out, run, "out")
    fn = _fn("elementwise", "lb_residual_layernorm",
             [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(run), _ptr(x), _ptr(delta_a), _ptr(delta_b), _ptr(weight), _ptr(bias), _ptr(out), _ptr(rows),
              n_rows, hidden, float(eps), _stream()), "residual_layernorm")
    return out


def heads_bias_rope_kv(proj: torch.Tensor, q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                       q_bias: torch.Tensor | None, k_bias: torch.Tensor | None, v_bias: torch.Tensor | None,
                       table: torch.Tensor | None, slot_map: torch.Tensor, first_v: torch.Tensor | None, blend: int,
                       blend_weight: torch.Tensor | None, q_heads: int, kv_heads: int, dim: int, vdim: int,
                       page_tokens: int, q_norm_w: torch.Tensor | None = None, k_norm_w: torch.Tensor | None = None,
                       norm_eps: float = 0.0, neighbours: bool = False, values_from_keys: bool = False) -> None:
    """Biases, a rotation of the first channels of every q and k head, an optional blend of the values with an
    earlier layer's, q to q_out and k, v to their pages.

    proj float32 [T, >= q_heads*dim + kv_heads*(dim + vdim)] (rows may be wider); q_out [T, q_heads*R]; k_pool
    [pages, kv_heads, page_tokens, R]; v_pool likewise (R: each tensor's own room per head, zero-filled beyond the
    head's channels); biases float32 per channel or None; table float32 [T, 2, n_freq] from `rope_table` (channels i
    and i + n_freq turn, i < n_freq; None: no rotation); first_v float32 [T, kv_heads*vdim]: `blend` 1 writes this
    layer's values there, `blend` 2 stores (1 - w) v + w first_v with w = blend_weight (a float32 scalar on the device).
    q_norm_w / k_norm_w float32 [dim] (each may be None): every q (k) head is RMS-normed over its `dim` channels with that
    weight and `norm_eps`, after the biases and before the rotation. `neighbours`: channels 2i and 2i + 1 turn together
    (i < n_freq) instead of i and i + n_freq. `values_from_keys`: the row holds no values; a value head is its key head as
    projected (with the key's bias), before norm and rotation, so vdim = dim."""
    _need(proj, torch.float32, "proj"); _need(k_pool, q_out.dtype, "k_pool"); _need(v_pool, q_out.dtype, "v_pool")
    _need(q_out, None, "q_out"); _need(slot_map, torch.int32, "slot_map")
    tokens = proj.shape[0]
    if values_from_keys and (vdim != dim or v_bias is not None):
        raise ValueError("heads_bias_rope_kv: values that are the keys have the keys' size and no bias of their own")
    used = q_heads * dim + kv_heads * (dim + (0 if values_from_keys else vdim))
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < used or q_out.shape[0] != tokens or q_out.shape[1] % q_heads:
        raise ValueError("heads_bias_rope_kv: the projection row does not hold these heads")
    q_room, k_room, v_room = q_out.shape[1] // q_heads, k_pool.shape[-1], v_pool.shape[-1]
    if tuple(k_pool.shape[1:3]) != (kv_heads, page_tokens) or tuple(v_pool.shape[1:3]) != (kv_heads, page_tokens) \
            or q_room < dim or k_room < dim or v_room < vdim:
        raise ValueError("heads_bias_rope_kv: the pools do not match the heads")
    for name, t, n in (("q_bias", q_bias, q_heads * dim), ("k_bias", k_bias, kv_heads * dim), ("v_bias", v_bias, kv_heads * vdim)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != n:
                raise ValueError(f"heads_bias_rope_kv: {name} must have {n} entries")
    n_freq = 0
    if table is not None:
        _need(table, torch.float32, "table")
        if table.dim() != 3 or table.shape[0] != tokens or table.shape[1] != 2 or 2 * table.shape[2] > dim:
            raise ValueError("heads_bias_rope_kv: the rotary table must be [tokens, 2, n_freq] with 2 n_freq <= dim")
        n_freq = table.shape[2]
    if blend not in (0, 1, 2):
        raise ValueError("heads_bias_rope_kv: blend is 0 (none), 1 (keep these values) or 2 (blend with the kept ones)")
    if blend:
        _need(first_v, torch.float32, "first_v")
        if tuple(first_v.shape) != (tokens, kv_heads * vdim):
            raise ValueError("heads_bias_rope_kv: first_v must be [tokens, kv_heads * vdim]")
    if blend == 2:
        _need(blend_weight, torch.float32, "blend_weight")
        if blend_weight.numel() != 1:
            raise ValueError("heads_bias_rope_kv: blend_weight is one number")
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != dim:
                raise ValueError(f"heads_bias_rope_kv: {name} must have {dim} entries")
    fn = _fn("elementwise", "lb_heads_bias_rope_kv",
             [c_int, c_void_p, c_long] + [c_void_p] * 7 + [c_int, c_void_p, c_void_p, c_int, c_void_p] + [c_int] * 9
             + [c_void_p, c_void_p, c_float, c_int, c_void_p])
    _check(fn(dtype_code(q_out.dtype), _ptr(proj), proj.stride(0), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_bias),
              _ptr(k_bias), _ptr(v_bias), _ptr(table), n_freq, _ptr(slot_map), _ptr(first_v if blend else None), int(blend),
              _ptr(blend_weight if blend == 2 else None), tokens, q_heads, kv_heads, dim, vdim, page_tokens, q_room, k_room,
              v_room, _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps), (1 if neighbours else 0) | (2 if values_from_keys else 0),
              _stream()), "heads_bias_rope_kv")


def channel_gate(heads: torch.Tensor, logits: torch.Tensor, out: torch.Tensor, q_heads: int, vdim: int) -> torch.Tensor:
    """out[t, h*vdim + c] = heads[t, h*R + c] * sigmoid(logits[t, h*vdim + c]): heads [T, q_heads*R] (R >= vdim), logits
    float32 [T, q_heads*vdim] (a view into wider rows is fine), out [T, q_heads*vdim] of heads' type."""
    _need(heads, None, "heads"); _need(out, heads.dtype, "out")
    tokens = heads.shape[0]
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1 or tuple(logits.shape) != (tokens, q_heads * vdim) \
            or tuple(out.shape) != (tokens, q_heads * vdim) or heads.shape[1] % q_heads or heads.shape[1] // q_heads < vdim:
        raise ValueError("channel_gate: shapes do not agree")
    fn = _fn("elementwise", "lb_channel_gate", [c_int, c_void_p, c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(heads.dtype), _ptr(heads), _ptr(logits), logits.stride(0), _ptr(out), tokens, q_heads, vdim,
              heads.shape[1] // q_heads, _stream()), "channel_gate")
    return out


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(x) element by element: "relu2" (relu(z)^2), "gelu_tanh", "silu"; 32-bit arithmetic."""
    _need(x, None, "x"); _need(out, x.dtype, "out")
    if kind not in ACTIVATIONS or out.shape != x.shape:
        raise ValueError(f"activation: unknown kind {kind!r} or shapes that do not agree")
    fn = _fn("elementwise", "lb_activation", [c_int, c_void_p, c_void_p, c_long, c_int, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), _ptr(out), x.numel(), ACTIVATIONS[kind], _stream()), "activation")
    return out


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """logits <- cap * tanh(logits / cap) in place (float32)."""
    _need(logits, torch.float32, "logits")
    if not cap > 0:
        raise ValueError("softcap: the cap must be positive")
    fn = _fn("elementwise", "lb_softcap", [c_void_p, c_long, c_float, c_void_p])
    _check(fn(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap")
    return logits


# ------------------------------------------------------------------ routed experts
EXPERT_ACTIVATIONS = {"silu": 0, "relu": 1, "relu2": 2}


def _route_options(experts: int, correction, groups, keep_groups, renormalize, route_scale, what: str):
    """The router's further options as the kernels take them (see `moe_route`)."""
    groups = int(groups or 0)
    keep = int(keep_groups or groups or 0)
    if correction is not None:
        _need(correction, torch.float32, "correction")
        if correction.numel() != experts:
            raise ValueError(f"{what}: correction must have one entry per expert")
    if groups > 1 and (experts % groups or not 0 < keep <= groups):
        raise ValueError(f"{what}: the experts must form equal groups of which 1..groups are kept")
    if not float(route_scale) > 0:
        raise ValueError(f"{what}: route_scale must be positive")
    return [_ptr(correction), groups, keep, int(bool(renormalize)), float(route_scale)]


def moe_route(h: torch.Tensor, router: torch.Tensor, top: int, ids: torch.Tensor, scores: torch.Tensor,
              shared_w: torch.Tensor | None = None, shared_factor: torch.Tensor | None = None,
              correction: torch.Tensor | None = None, groups: int | None = None, keep_groups: int | None = None,
              renormalize: bool = False, route_scale: float = 1.0) -> None:
    """ids[t, k], scores[t, k]: the `top` experts with the largest router logits of token t (ties: the lower index) and
    sigmoid of those logits. h [T, H] in the run's type; router float32 [experts, H]; logits are 32-bit dot products.
    `shared_w` float32 [H]: also shared_factor[t] = sigmoid(shared_w . h[t]).
    `correction` float32 [experts]: the choice is made on sigmoid + correction, the scores stay the sigmoids. `groups` > 1:
    the experts form that many equal groups of neighbours, a group's score is the sum of its two largest choice scores,
    and only experts of the `keep_groups` best groups can be chosen. `renormalize`: the chosen scores are divided by their
    sum (+ 1e-20); `route_scale` then multiplies them."""
    _need(h, None, "h"); _need(router, torch.float32, "router"); _need(ids, torch.int32, "ids"); _need(scores, torch.float32, "scores")
    tokens, hidden = h.shape
    experts = router.shape[0]
    if router.shape[1] != hidden or tuple(ids.shape) != (tokens, top) or tuple(scores.shape) != (tokens, top) or not 0 < top <= experts:
        raise ValueError("moe_route: shapes do not agree")
    if shared_w is not None:
        _need(shared_w, torch.float32, "shared_w"); _need(shared_factor, torch.float32, "shared_factor")
        if shared_w.numel() != hidden or shared_factor.numel() != tokens:
            raise ValueError("moe_route: shared_w [H] and shared_factor [T]")
    options = _route_options(experts, correction, groups, keep_groups, renormalize, route_scale, "moe_route")
    fn = _fn("moe", "lb_moe_route", [c_int] + [c_void_p] * 6 + [c_int] * 4 + [c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(h.dtype), _ptr(h), _ptr(router), _ptr(shared_w), _ptr(ids), _ptr(scores), _ptr(shared_factor), tokens,
              hidden, experts, int(top), *options, _stream()), "moe_route")


def moe_select(logits: torch.Tensor, experts: int, top: int, ids: torch.Tensor, scores: torch.Tensor,
               shared_factor: torch.Tensor | None = None, correction: torch.Tensor | None = None, groups: int | None = None,
               keep_groups: int | None = None, renormalize: bool = False, route_scale: float = 1.0) -> None:
    """What `moe_route` chooses, from router logits that a matrix product left in float32 [T, >= experts (+ 1)]: the
    `top` largest of the first `experts` columns (ties: the lower index), their sigmoids, and, with `shared_factor`,
    sigmoid of column `experts`."""
    _need(ids, torch.int32, "ids"); _need(scores, torch.float32, "scores")
    tokens = logits.shape[0]
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1 or tuple(ids.shape) != (tokens, top) \
            or tuple(scores.shape) != (tokens, top) or logits.shape[1] < experts + (1 if shared_factor is not None else 0):
        raise ValueError("moe_select: shapes do not agree")
    if shared_factor is not None:
        _need(shared_factor, torch.float32, "shared_factor")
    options = _route_options(experts, correction, groups, keep_groups, renormalize, route_scale, "moe_select")
    fn = _fn("moe", "lb_moe_select", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), _ptr(ids), _ptr(scores), _ptr(shared_factor), tokens, int(experts), int(top),
              *options, _stream()), "moe_select")


def moe_group(ids: torch.Tensor, experts: int, offsets: torch.Tensor, order: torch.Tensor) -> None:
    """Group the (token, k) pairs by expert: order int32 [pairs] lists the pairs expert by expert, expert e's at places
    offsets[e] .. offsets[e + 1] (offsets int32 [experts + 1])."""
    _need(ids, torch.int32, "ids"); _need(offsets, torch.int32, "offsets"); _need(order, torch.int32, "order")
    if offsets.numel() != experts + 1 or order.numel() != ids.numel():
        raise ValueError("moe_group: offsets [experts + 1], order one entry per pair")
    fn = _fn("moe", "lb_moe_group", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(ids), ids.numel(), int(experts), _ptr(offsets), _ptr(order), _stream()), "moe_group")


def moe_expert_up(h: torch.Tensor, order: torch.Tensor, offsets: torch.Tensor, scores: torch.Tensor | None,
                  gate_up: torch.Tensor, act: torch.Tensor, top: int, activation: str = "silu",
                  interleaved: bool = False, gated: bool = True) -> torch.Tensor:
    """act[place] = act_fn(s * gate_e h[token]) * (s * up_e h[token]) for every place of `order` (pair = token * top + k, s =
    scores[pair] or 1): gate_up [experts, 2 * inter, H] (gate rows, then up rows; `interleaved`: every expert's rows in
    `interleave_gate_up`'s layout), act [pairs, inter] in the run's type. `gated` False: experts without a gate, gate_up
    [experts, inter, H] and act[place] = relu(up_e h[token])^2 (activation "relu2", no scores)."""
    _need(h, None, "h"); _need(gate_up, h.dtype, "gate_up"); _need(act, h.dtype, "act")
    experts, rows, hidden = gate_up.shape
    pairs = order.numel()
    inter = rows // 2 if gated else rows
    if hidden != h.shape[1] or (gated and rows % 2) or tuple(act.shape) != (pairs, inter) or pairs != h.shape[0] * top \
            or activation not in EXPERT_ACTIVATIONS or (not gated and (activation != "relu2" or interleaved or scores is not None)):
        raise ValueError("moe_expert_up: shapes do not agree")
    fn = _fn("moe", "lb_moe_expert_up", [c_int, c_void_p, c_long] + [c_void_p] * 5 + [c_int] * 8 + [c_void_p])
    _check(fn(dtype_code(h.dtype), _ptr(h), h.stride(0), _ptr(order), _ptr(offsets), _ptr(scores), _ptr(gate_up), _ptr(act),
              pairs, int(top), experts, hidden, inter, EXPERT_ACTIVATIONS[activation], int(bool(interleaved)), int(bool(gated)),
              _stream()), "moe_expert_up")
    return act


def moe_expert_down(act: torch.Tensor, order: torch.Tensor, offsets: torch.Tensor, down: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y[pair] = down_e act[place] in 32-bit: down [experts, H, inter], y float32 [pairs, H] indexed by pair."""
    _need(act, None, "act"); _need(down, act.dtype, "down"); _need(y, torch.float32, "y")
    experts, hidden, inter = down.shape
    pairs = order.numel()
    if tuple(act.shape) != (pairs, inter) or tuple(y.shape) != (pairs, hidden):
        raise ValueError("moe_expert_down: shapes do not agree")
    fn = _fn("moe", "lb_moe_expert_down", [c_int] + [c_void_p] * 5 + [c_int] * 4 + [c_void_p])
    _check(fn(dtype_code(act.dtype), _ptr(act), _ptr(order), _ptr(offsets), _ptr(down), _ptr(y), pairs, experts, hidden, inter,
              _stream()), "moe_expert_down")
    return y


def moe_combine(y: torch.Tensor, out: torch.Tensor, top: int, pair_scale: torch.Tensor | None = None,
                shared_out: torch.Tensor | None = None, shared_factor: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = sum_k c_k y[row(t * top + k)] + f_t shared_out[t], c = pair_scale or 1, f = shared_factor or 1; y (float32,
    or of out's type) [T * top, H] (row(pair) = pair), or with `rows` (int32 [T * top]) any [R, H] with row(pair) =
    rows[pair]; out and shared_out [T, H] in the run's type. The sum is 32-bit."""
    _need(y, None, "y"); _need(out, None, "out")
    if y.dtype not in (torch.float32, out.dtype):
        raise ValueError("moe_combine: y must be float32 or of out's type")
    tokens, hidden = out.shape
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if y.dim() != 2 or y.shape[1] != hidden or (rows is None and y.shape[0] != tokens * top) or (rows is not None and rows.numel() != tokens * top):
        raise ValueError("moe_combine: y must be [tokens * top, H], or rows one entry per pair")
    if shared_out is not None:
        _need(shared_out, out.dtype, "shared_out")
        if shared_out.shape != out.shape:
            raise ValueError("moe_combine: shared_out must have out's shape")
    for name, t in (("pair_scale", pair_scale), ("shared_factor", shared_factor)):
        if t is not None:
            _need(t, torch.float32, name)
    fn = _fn("moe", "lb_moe_combine", [c_int, c_void_p, c_int] + [c_void_p] * 4 + [c_int] * 3 + [c_void_p, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(y), dtype_code(y.dtype), _ptr(pair_scale), _ptr(shared_out), _ptr(shared_factor), _ptr(out),
              tokens, hidden, int(top), _ptr(rows), _stream()), "moe_combine")
    return out


MOE_TILE_ROWS = 128     # the tensor-core products take the pairs in tiles of this many rows, each of one expert


def moe_padded_rows(pairs: int, experts: int) -> int:
    """Rows of the buffers of the grouped tensor-core products: room for every expert's pairs rounded up to whole tiles."""
    return -(-(pairs + (MOE_TILE_ROWS - 1) * experts) // MOE_TILE_ROWS) * MOE_TILE_ROWS


def moe_group_tiles(ids: torch.Tensor, experts: int, place_of: torch.Tensor, tile_up: torch.Tensor, tile_down: torch.Tensor,
                    rows_up: int, rows_down: int) -> None:
    """The grouping for the tensor-core products: place_of[pair] = the pair's row in buffers of `moe_padded_rows` rows where
    every tile of 128 rows belongs to one expert; tile_up[i] / tile_down[i] = expert * rows_up / expert * rows_down for tile
    i (the row where that expert's weights begin in the stacked matrices), -1 for a tile without pairs; the lists have one
    more entry than the buffers have tiles, the number of tiles in use (all at the front)."""
    for name, t in (("ids", ids), ("place_of", place_of), ("tile_up", tile_up), ("tile_down", tile_down)):
        _need(t, torch.int32, name)
    if place_of.numel() != ids.numel() or tile_up.numel() != tile_down.numel() \
            or (tile_up.numel() - 1) * MOE_TILE_ROWS < moe_padded_rows(ids.numel(), experts):
        raise ValueError("moe_group_tiles: place_of one entry per pair, the tile lists one per tile of the padded buffers and one more")
    fn = _fn("moe", "lb_moe_group_tiles", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(ids), ids.numel(), int(experts), _ptr(place_of), _ptr(tile_up), _ptr(tile_down), tile_up.numel() - 1, int(rows_up),
              int(rows_down), _stream()), "moe_group_tiles")


def moe_scatter_rows(h: torch.Tensor, place_of: torch.Tensor, scale: torch.Tensor | None, rows: torch.Tensor, top: int) -> torch.Tensor:
    """rows[place_of[pair]] = scale[pair] * h[pair // top] (scale None: a copy): h [T, H], rows [R, H] of h's type."""
    _need(h, None, "h"); _need(rows, h.dtype, "rows"); _need(place_of, torch.int32, "place_of")
    pairs = place_of.numel()
    if pairs != h.shape[0] * top or rows.shape[1] != h.shape[1]:
        raise ValueError("moe_scatter_rows: shapes do not agree")
    if scale is not None:
        _need(scale, torch.float32, "scale")
    fn = _fn("moe", "lb_moe_scatter_rows", [c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(h.dtype), _ptr(h), h.stride(0), _ptr(place_of), _ptr(scale), _ptr(rows), pairs, h.shape[1], int(top),
              _stream()), "moe_scatter_rows")
    return rows


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_rows: torch.Tensor, groups: int,
                         epilogue: str | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w_g[N, K]^T tile by tile: every tile of 128 rows of `a` is multiplied by the weights of ONE
    group, the [N, K] matrix that begins at row tile_rows[tile] of w [groups * N, K]; tile_rows [M / 128 + 1] ends with the
    number of tiles in use (all at the front; the others are skipped). It is int32 on the device, written by an earlier kernel. M is a multiple of 128. epilogue "swiglu" as in
    `gemm_tcgen05` (each group's rows interleaved by `interleave_gate_up`)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        raise ValueError("gemm_tcgen05_grouped: operands must be 2-D bfloat16")
    m, k = a.shape
    if w.shape[0] % groups or w.shape[1] != k or m % MOE_TILE_ROWS:
        raise ValueError("gemm_tcgen05_grouped: shapes do not agree")
    n = w.shape[0] // groups
    if epilogue not in (None, "swiglu"):
        raise ValueError(f"gemm_tcgen05_grouped: unknown epilogue {epilogue!r}")
    out_cols = n // 2 if epilogue == "swiglu" else n
    if epilogue == "swiglu" and (n % (2 * SWIGLU_BLOCK) or out.dtype != torch.bfloat16):
        raise ValueError("gemm_tcgen05_grouped: the swiglu epilogue needs interleaved weights and a bfloat16 output")
    _need(tile_rows, torch.int32, "tile_rows")
    if tuple(out.shape) != (m, out_cols) or out.stride(1) != 1 or tile_rows.numel() != m // MOE_TILE_ROWS + 1:
        raise ValueError("gemm_tcgen05_grouped: out [M, N], one tile entry per 128 rows and the count of tiles in use behind them")
    partials, counters, sms = gemm_scratch(a.device)
    fn = _fn("gemm_tcgen05", "lb_gemm_tcgen05_grouped",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_long, c_long, c_long, c_void_p, c_void_p, c_long,
              c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), m, n, k, int(groups), a.stride(0), w.stride(0), out.stride(0),
              _ptr(tile_rows), _ptr(partials), partials.numel(), _ptr(counters), counters.numel(), sms,
              1 if epilogue == "swiglu" else 0, _stream()), "gemm_tcgen05_grouped")
    return out


# ------------------------------------------------------------------ linear attention (a recurrence over state slots)
SCAN_ACTIVATIONS = {None: 0, "none": 0, "silu": 1}


def decay_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, out: torch.Tensor, state: torch.Tensor,
               cu_q: torch.Tensor, state_slots: torch.Tensor, decay: torch.Tensor, n_seqs: int, heads: int, dim: int,
               vdim: int, activation: str | None = None, segment_tokens: int = 0,
               segment_state: torch.Tensor | None = None) -> torch.Tensor:
    """Per sequence and head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over the step's tokens, from and
    to the requests' state slots.

    proj [T, N] holds q at column q_off (heads*dim), k at k_off, v at v_off (heads*vdim), each passed through
    `activation` on the way in; out float32 [T, heads*vdim]; state float32 [slots, heads, dim, vdim];
    decay float32 [heads]; cu_q int32 [S + 1]; state_slots int32 [S].

    With `segment_tokens` > 0 every sequence's tokens are cut into segments of that many that are scanned at once
    (three launches; for steps with long portions, where one chain per sequence and head would leave most of
    the device idle): `segment_state` is float32 scratch [sum over sequences of max(1, ceil(tokens / segment_tokens)),
    heads, dim, vdim] (`scan_segments` counts them). The result agrees with the single pass within rounding."""
    _need(out, torch.float32, "out"); _need(state, torch.float32, "state"); _need(decay, torch.float32, "decay")
    total_segments = 0
    if segment_tokens:
        _need(segment_state, torch.float32, "segment_state")
        total_segments = segment_state.shape[0]
        if tuple(segment_state.shape[1:]) != (heads, dim, vdim) or total_segments < n_seqs:
            raise ValueError("decay_scan: segment_state must be [segments, heads, dim, vdim] with a segment or more per sequence")
    _need(cu_q, torch.int32, "cu_q"); _need(state_slots, torch.int32, "state_slots")
    tokens = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or max(q_off, k_off) + heads * dim > proj.shape[1] \
            or v_off + heads * vdim > proj.shape[1] or min(q_off, k_off, v_off) < 0:
        raise ValueError("decay_scan: the projection row does not hold these heads")
    if tuple(out.shape) != (tokens, heads * vdim) or tuple(state.shape[1:]) != (heads, dim, vdim) or decay.numel() != heads:
        raise ValueError("decay_scan: out, state or decay do not match the heads")
    if activation not in SCAN_ACTIVATIONS:
        raise ValueError(f"decay_scan: unknown activation {activation!r}")
    fn = _fn("linear_attention", "lb_decay_scan",
             [c_int, c_void_p, c_long, c_int, c_int, c_int] + [c_void_p] * 5 + [c_int] * 5 + [c_void_p, c_int, c_int, c_void_p])
    _check(fn(dtype_code(proj.dtype), _ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(out), _ptr(state), _ptr(cu_q),
              _ptr(state_slots), _ptr(decay), n_seqs, heads, dim, vdim, SCAN_ACTIVATIONS[activation],
              _ptr(segment_state), int(segment_tokens), total_segments, _stream()), "decay_scan")
    if total_segments:
        global LAUNCHES
        LAUNCHES += 2          # the segmented form is three kernels
    return out


SCAN_SEGMENT_TOKENS = 128      # the shortest segment of the segmented scan
SCAN_SEGMENT_BYTES = 1 << 30   # the most scratch its segments' states may take; longer segments beyond


def scan_segments(q_lens: list[int], state_bytes: int) -> tuple[int, int]:
    """(tokens per segment, number of segments) for a step whose sequences bring `q_lens` tokens, or (0, 0)
    when no portion is long enough for the segmented scan to pay (two segments or more)."""
    longest = max(q_lens)
    if longest < 2 * SCAN_SEGMENT_TOKENS:
        return 0, 0
    tokens = SCAN_SEGMENT_TOKENS
    while True:
        total = sum(max(1, -(-n // tokens)) for n in q_lens)
        if total * state_bytes <= SCAN_SEGMENT_BYTES or 2 * tokens > longest:
            return tokens, total
        tokens *= 2


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = rmsnorm(x) * weight * sigmoid(gate): x float32 [T, n]; gate [T, n] in the run's type, a view into
    wider rows is fine; out [T, n] in the run's type."""
    _need(x, torch.float32, "x"); _need(weight, torch.float32, "weight"); _need(out, gate.dtype, "out")
    tokens, n = x.shape
    if gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (tokens, n) or tuple(out.shape) != (tokens, n) \
            or weight.numel() != n:
        raise ValueError("gated_rmsnorm: shapes do not agree")
    fn = _fn("linear_attention", "lb_gated_rmsnorm",
             [c_int, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(gate.dtype), _ptr(x), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), tokens, n, float(eps),
              _stream()), "gated_rmsnorm")
    return out


def add_position_rows(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, lowered: torch.Tensor | None = None) -> torch.Tensor:
    """x[t] += table[positions[t]] over a float32 stream x [T, H] (table [rows, H] in the run's type); `lowered` [T, H] in
    the table's type, if given, receives the sum as the matrix products read it."""
    _need(x, torch.float32, "x"); _need(positions, torch.int32, "positions"); _need(table, None, "table")
    if table.dim() != 2 or table.shape[1] != x.shape[1] or positions.shape[0] != x.shape[0]:
        raise ValueError("add_position_rows: the table must be [rows, H] and positions one entry per token")
    if lowered is not None:
        _need(lowered, table.dtype, "lowered")
        if lowered.shape != x.shape:
            raise ValueError("add_position_rows: lowered must have x's shape")
    fn = _fn("elementwise", "lb_add_position_rows", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(dtype_code(table.dtype), _ptr(x), _ptr(positions), _ptr(table), table.shape[0], _ptr(lowered), x.shape[0],
              x.shape[1], _stream()), "add_position_rows")
    return x


def lower_rows(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = x in out's type: a float32 stream as the run's matrix products read it."""
    _need(x, torch.float32, "x"); _need(out, None, "out")
    if out.shape != x.shape:
        raise ValueError("lower_rows: out must have x's shape")
    fn = _fn("elementwise", "lb_lower_rows", [c_int, c_void_p, c_void_p, c_long, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(x), _ptr(out), x.numel(), _stream()), "lower_rows")
    return out


def scaled_add_rmsnorm(x: torch.Tensor, a: torch.Tensor | None, a_weight: torch.Tensor | None, b: torch.Tensor | None,
                       b_weight: torch.Tensor | None, part_eps: float, factor: float, alpha: float, weight: torch.Tensor,
                       eps: float, out: torch.Tensor | None, run_dtype: torch.dtype | None = None) -> torch.Tensor:
    """The norm AFTER the sum over a float32 stream x [T, H], in place:

        x = weight * v * rsqrt(mean(v^2) + eps),   v = alpha * x + factor * (norm_a(a) + norm_b(b))
        norm_a(a) = a * a_weight * rsqrt(mean(a^2) + part_eps)      (a_weight None: a itself; the same for b; b may be None)

    a, b in the run's type; `out` [T, H] in the run's type, if given, receives a copy of the new x."""
    _need(x, torch.float32, "x"); _need(weight, torch.float32, "weight")
    run = run_dtype or (out.dtype if out is not None else (a.dtype if a is not None else torch.float32))
    hidden = x.shape[-1]
    if b is not None and a is None:
        raise ValueError("scaled_add_rmsnorm: b comes with a")
    for name, t in (("a", a), ("b", b), ("out", out)):
        if t is not None:
            _need(t, run, name)
            if t.shape != x.shape:
                raise ValueError(f"scaled_add_rmsnorm: {name} must have x's shape")
    for name, t in (("a_weight", a_weight), ("b_weight", b_weight), ("weight", weight)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != hidden:
                raise ValueError(f"scaled_add_rmsnorm: {name} must have one entry per channel")
    fn = _fn("elementwise", "lb_scaled_add_rmsnorm",
             [c_int] + [c_void_p] * 5 + [c_float, c_float, c_float, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(fn(dtype_code(run), _ptr(x), _ptr(a), _ptr(a_weight), _ptr(b), _ptr(b_weight), float(part_eps), float(factor),
              float(alpha), _ptr(weight), float(eps), _ptr(out), x.shape[0], hidden, _stream()), "scaled_add_rmsnorm")
    return x


# ------------------------------------------------------------------ attention over a latent
def latent_rows(proj: torch.Tensor, q_off: int, dkv_off: int, norm_w: torch.Tensor | None, eps: float, table: torch.Tensor,
                slot_map: torch.Tensor | None, k_pool: torch.Tensor | None, q_out: torch.Tensor, q_heads: int, dim: int,
                rot: int, rank: int, page_tokens: int) -> None:
    """A token's cache row [normed latent | rotated key part | zeros] into `k_pool` [pages, 1, page_tokens, room] (not with
    dkv_off < 0: a layer that reads another layer's rows), and the rotated part of every query head into channels
    [rank, rank + rot) of q_out [T, q_heads * room] (zeros behind it; channels [0, rank) are left alone).
    proj float32 rows: q_heads x [dim | rot] at q_off, [rank | rot] at dkv_off; table float32 [T, 2, rot / 2] from
    `rope_table`: channels 2i and 2i + 1 of a rotated part turn by angle i."""
    _need(proj, torch.float32, "proj"); _need(table, torch.float32, "table"); _need(q_out, None, "q_out")
    tokens = proj.shape[0]
    room = q_out.shape[1] // q_heads
    if proj.dim() != 2 or proj.stride(1) != 1 or q_out.shape[0] != tokens or q_out.shape[1] != q_heads * room or room < rank + rot:
        raise ValueError("latent_rows: q_out must be [tokens, q_heads * room] with room >= rank + rot")
    if tuple(table.shape) != (tokens, 2, rot // 2) or rot % 2:
        raise ValueError("latent_rows: the rotary table must be [tokens, 2, rot / 2]")
    if dkv_off >= 0:
        _need(norm_w, torch.float32, "norm_w"); _need(slot_map, torch.int32, "slot_map"); _need(k_pool, q_out.dtype, "k_pool")
        if norm_w.numel() != rank or tuple(k_pool.shape[1:]) != (1, page_tokens, room):
            raise ValueError("latent_rows: the pool must be [pages, 1, page_tokens, room] and the norm weight [rank]")
    fn = _fn("latent", "lb_latent_rows", [c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                          c_void_p] + [c_int] * 7 + [c_void_p])
    _check(fn(dtype_code(q_out.dtype), _ptr(proj), proj.stride(0), int(q_off), int(dkv_off), _ptr(norm_w), float(eps), _ptr(table),
              _ptr(slot_map), _ptr(k_pool), _ptr(q_out), tokens, q_heads, dim, rot, rank, room, page_tokens, _stream()),
           "latent_rows")


def heads_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h, :] = a[t, h, :] @ w[h]^T, one product per head: a [T, heads, K] and out [T, heads, N] may be views into wider
    rows (the last axis contiguous), w [heads, N, K] dense. a is of w's type, or float32 (unrounded projection rows); out of
    w's type. `gate` float32 [T, heads * N] (a view into wider rows is fine): out *= sigmoid(gate). 32-bit sums in the
    order of K."""
    _need(w, None, "w")
    tokens, heads, k_dim = a.shape
    n_out = w.shape[1]
    if w.dim() != 3 or w.shape[0] != heads or w.shape[2] != k_dim or not w.is_contiguous() or tuple(out.shape) != (tokens, heads, n_out):
        raise ValueError("heads_linear: shapes do not agree")
    if a.device != w.device or out.device != w.device or a.stride(2) != 1 or out.stride(2) != 1 or out.dtype != w.dtype \
            or a.dtype not in (w.dtype, torch.float32):
        raise ValueError("heads_linear: a and out must be on the device, contiguous along the last axis, out of w's type")
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (tokens, heads * n_out):
            raise ValueError("heads_linear: gate must be [tokens, heads * N]")
    fn = _fn("latent", "lb_heads_linear", [c_int, c_int, c_void_p, c_long, c_long, c_void_p, c_void_p, c_long, c_long, c_void_p,
                                           c_long, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(w.dtype), int(a.dtype == torch.float32), _ptr(a), a.stride(0), a.stride(1), _ptr(w), _ptr(out),
              out.stride(0), out.stride(1), _ptr(gate), gate.stride(0) if gate is not None else 0, tokens, heads, n_out, k_dim,
              _stream()), "heads_linear")
    return out


# ------------------------------------------------------------------ the gated delta rule
def delta_prepare_tokens() -> int:
    lib = build.load("delta_rule")
    lib.lb_delta_prepare_tokens.restype = c_int
    return lib.lb_delta_prepare_tokens()


def delta_prepare(proj: torch.Tensor, b_off: int, a_off: int, taps: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  state: torch.Tensor, conv_off: int, batch, prepared: torch.Tensor, heads: int, kv_heads: int, dim: int,
                  vdim: int, unit_eps: float) -> torch.Tensor:
    """Short causal convolutions with silu over the leading channels [q | k | v] of proj (float32 rows), unit q and k heads
    (q also times dim^-1/2), beta = sigmoid(b) and decay = exp(-exp(A_log) softplus(a + dt_bias)) per head, into
    `prepared` float32 [T, channels + 2 heads]; then every request's last taps - 1 inputs are moved into its state row
    (state float32 [slots, floats], the tail at `conv_off`)."""
    channels = 2 * kv_heads * dim + heads * vdim
    for name, t in (("proj", proj), ("taps", taps), ("a_log", a_log), ("dt_bias", dt_bias), ("state", state), ("prepared", prepared)):
        _need(t, torch.float32, name)
    tokens = proj.shape[0]
    n_taps = taps.shape[1]
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < max(channels, b_off + heads, a_off + heads) \
            or tuple(taps.shape) != (channels, n_taps) or tuple(prepared.shape) != (tokens, channels + 2 * heads) \
            or a_log.numel() != heads or dt_bias.numel() != heads or state.dim() != 2 \
            or state.shape[1] < conv_off + (n_taps - 1) * channels:
        raise ValueError("delta_prepare: shapes do not agree")
    tiles = batch.tiles[delta_prepare_tokens()]
    fn = _fn("delta_rule", "lb_delta_prepare",
             [c_void_p, c_long, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(proj), proj.stride(0), int(b_off), int(a_off), _ptr(taps), n_taps, _ptr(a_log), _ptr(dt_bias), _ptr(state),
              state.stride(0), int(conv_off), _ptr(batch.cu_q), _ptr(batch.state_slots), _ptr(tiles.tile_seq), _ptr(tiles.tile_q0),
              tiles.count, batch.n_seqs, _ptr(prepared), heads, kv_heads, dim, vdim, float(unit_eps), _stream()), "delta_prepare")
    return prepared


def delta_scan(prepared: torch.Tensor, out: torch.Tensor, state: torch.Tensor, batch, heads: int, kv_heads: int, dim: int,
               vdim: int) -> torch.Tensor:
    """The recurrence over every sequence's tokens of the step, from and into the requests' state rows:
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q. out float32 [T, heads * vdim]."""
    for name, t in (("prepared", prepared), ("out", out), ("state", state)):
        _need(t, torch.float32, name)
    channels = 2 * kv_heads * dim + heads * vdim
    if tuple(prepared.shape) != (out.shape[0], channels + 2 * heads) or out.shape[1] != heads * vdim or state.dim() != 2 \
            or state.shape[1] < heads * dim * vdim:
        raise ValueError("delta_scan: shapes do not agree")
    fn = _fn("delta_rule", "lb_delta_scan", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p] + [c_int] * 5 + [c_void_p])
    _check(fn(_ptr(prepared), _ptr(out), _ptr(state), state.stride(0), _ptr(batch.cu_q), _ptr(batch.state_slots), batch.n_seqs,
              heads, kv_heads, dim, vdim, _stream()), "delta_scan")
    return out


def head_gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, heads: int,
                       vdim: int) -> torch.Tensor:
    """out[t, h] = o[t, h] * rsqrt(mean(o[t, h]^2) + eps) * weight * silu(gate[t, h]) per head: o float32 [T, heads * vdim],
    gate float32 [T, heads * vdim] (a view into wider rows is fine), weight float32 [vdim] (shared by the heads) or
    [heads * vdim] (a weight per channel), out in the run's type."""
    _need(o, torch.float32, "o"); _need(weight, torch.float32, "weight"); _need(out, None, "out")
    tokens = o.shape[0]
    if gate.dtype != torch.float32 or tuple(o.shape) != (tokens, heads * vdim) or tuple(out.shape) != (tokens, heads * vdim) or gate.dim() != 2 \
            or gate.stride(1) != 1 or tuple(gate.shape) != (tokens, heads * vdim) or weight.numel() not in (vdim, heads * vdim):
        raise ValueError("head_gated_rmsnorm: shapes do not agree")
    per_channel = weight.numel() == heads * vdim and heads > 1
    fn = _fn("delta_rule", "lb_head_gated_rmsnorm", [c_int, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int,
                                                     c_float, c_int, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), tokens, heads, vdim, float(eps),
              vdim if per_channel else 0, _stream()), "head_gated_rmsnorm")
    return out


# ------------------------------------------------------------------ time mixing with a decay per token and key channel
def wkv_mix_tokens() -> int:
    lib = build.load("wkv")
    lib.lb_wkv_mix_tokens.restype = c_int
    return lib.lb_wkv_mix_tokens()


def wkv_shift_mix(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, shift_off: int, batch, mixes: torch.Tensor) -> torch.Tensor:
    """mixes[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]: h [T, W] in the run's type, mu float32 [n, W], mixes [n, T, W] of h's
    type. The input before a step's first token of a request is the tail of its state row (state float32 [slots, floats],
    the tail of W floats at `shift_off`; zeros when the request starts); afterwards the step's last input is left there."""
    _need(h, None, "h"); _need(mu, torch.float32, "mu"); _need(state, torch.float32, "state"); _need(mixes, h.dtype, "mixes")
    tokens, width = h.shape
    n_mix = mu.shape[0]
    if mu.dim() != 2 or mu.shape[1] != width or tuple(mixes.shape) != (n_mix, tokens, width) or state.dim() != 2 \
            or state.shape[1] < shift_off + width:
        raise ValueError("wkv_shift_mix: shapes do not agree")
    tiles = batch.tiles[wkv_mix_tokens()]
    fn = _fn("wkv", "lb_wkv_shift_mix", [c_int, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(h.dtype), _ptr(h), _ptr(mu), _ptr(state), state.stride(0), int(shift_off), _ptr(batch.cu_q),
              _ptr(batch.state_slots), _ptr(tiles.tile_seq), _ptr(tiles.tile_q0), tiles.count, batch.n_seqs, _ptr(mixes), tokens,
              width, n_mix, _stream()), "wkv_shift_mix")
    return mixes


def wkv_decay(a: torch.Tensor, w2: torch.Tensor, w0: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """decay[t, c] = exp(-exp(w0[c] + sum_j w2[c, j] tanh(a[t, j]))) in 32-bit: a float32 [T, >= rank] (rows may be wider),
    w2 [channels, rank] in the run's type, w0 float32 [channels], decay float32 [T, channels]."""
    _need(w2, None, "w2"); _need(w0, torch.float32, "w0"); _need(decay, torch.float32, "decay")
    channels, rank = w2.shape
    tokens = a.shape[0]
    if a.dtype != torch.float32 or a.dim() != 2 or a.stride(1) != 1 or a.shape[1] < rank or w0.numel() != channels \
            or tuple(decay.shape) != (tokens, channels):
        raise ValueError("wkv_decay: shapes do not agree")
    fn = _fn("wkv", "lb_wkv_decay", [c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(w2.dtype), _ptr(a), a.stride(0), _ptr(w2), _ptr(w0), _ptr(decay), tokens, channels, rank, _stream()), "wkv_decay")
    return decay


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor, out: torch.Tensor,
             state: torch.Tensor, batch, heads: int, dim: int) -> torch.Tensor:
    """The recurrence over every sequence's tokens of the step, from and into the requests' state rows (S of head h at
    h * dim * dim of the row): o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T. r, k, v float32
    [T, heads * dim] (views into wider rows are fine), w float32 [T, heads * dim], u float32 [heads, dim], out float32
    [T, heads * dim]."""
    for name, t in (("w", w), ("u", u), ("out", out), ("state", state)):
        _need(t, torch.float32, name)
    tokens, channels = out.shape
    for name, t in (("r", r), ("k", k), ("v", v)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or tuple(t.shape) != (tokens, channels):
            raise ValueError(f"wkv_scan: {name} must be float32 [tokens, heads * dim] with dense rows")
    if channels != heads * dim or tuple(w.shape) != (tokens, channels) or u.numel() != channels or state.dim() != 2 \
            or state.shape[1] < heads * dim * dim:
        raise ValueError("wkv_scan: shapes do not agree")
    fn = _fn("wkv", "lb_wkv_scan", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(r), r.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(w), _ptr(u), _ptr(out), _ptr(state),
              state.stride(0), _ptr(batch.cu_q), _ptr(batch.state_slots), batch.n_seqs, heads, dim, _stream()), "wkv_scan")
    return out


# ------------------------------------------------------------------ matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit FFMA accumulation (no tensor cores).

    a and w share a dtype (float32 or bfloat16); out has it too, or float32. Rows may be strided."""
    if a.dtype != w.dtype or a.dim() != 2 or w.dim() != 2 or out.dim() != 2:
        raise ValueError("gemm: operands must be 2-D and share a dtype")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise ValueError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("gemm: innermost dimension must be contiguous")
    fn = _fn("gemm_simt", "lb_gemm_simt",
             [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long, c_void_p])
    _check(fn(dtype_code(a.dtype), dtype_code(out.dtype), _ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0),
              w.stride(0), out.stride(0), _stream()), "gemm_simt")
    return out


# ------------------------------------------------------------------ attention
ATTENTION_SIMT_MAX_DIM = 640     # the largest head size of the 32-bit attention kernel (csrc/attention_simt.cu)


def attention_simt_block_queries() -> int:
    lib = build.load("attention_simt")
    lib.lb_attention_simt_block_queries.restype = c_int
    return lib.lb_attention_simt_block_queries()


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                   block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, tile_seq: torch.Tensor,
                   tile_q0: torch.Tensor, n_tiles: int, q_heads: int, kv_heads: int, dim: int, page_tokens: int,
                   scale: float, window: int = 0, vdim: int | None = None, sinks: torch.Tensor | None = None,
                   gates: torch.Tensor | None = None, chunk: int = 0, keep_first: int = 0) -> torch.Tensor:
    """Paged causal attention in 32-bit arithmetic for any mix of segment lengths.

    q [T, q_heads * dim]; out [T, q_heads * vdim] (vdim defaults to dim); pools [pages, kv_heads, page_tokens,
    dim or vdim]; block_table int32 [S, W]; cu_q int32 [S + 1]; ctx_len int32 [S]; (tile_seq, tile_q0) int32
    [n_tiles] list the query tiles. `sinks` float32 [q_heads]: a score per head that joins the softmax's
    denominator only; `gates` float32 [T, q_heads]: a factor on each head's output. `chunk` > 0: a query sees
    only the keys of its own chunk of that many positions (counted from position 0 of its sequence). `keep_first` > 0:
    behind a window the first `keep_first` keys of the sequence stay visible."""
    vdim = dim if vdim is None else int(vdim)
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(k_pool, q.dtype, "k_pool"); _need(v_pool, q.dtype, "v_pool")
    if tuple(out.shape) != (q.shape[0], q_heads * vdim) or k_pool.shape[-1] != dim or v_pool.shape[-1] != vdim:
        raise ValueError("attention_simt: out or the pools do not match the head sizes")
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        if sinks.numel() != q_heads:
            raise ValueError("attention_simt: one sink per query head")
    if gates is not None:
        _need(gates, torch.float32, "gates")
        if tuple(gates.shape) != (q.shape[0], q_heads):
            raise ValueError("attention_simt: gates must be [tokens, q_heads]")
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_simt", "lb_attention_simt",
             [c_int] + [c_void_p] * 5 + [c_int] + [c_void_p] * 4 + [c_int] * 5 + [c_float, c_int, c_int, c_void_p,
                                                                                c_void_p, c_int, c_int, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table),
              block_table.shape[1], _ptr(cu_q), _ptr(ctx_len), _ptr(tile_seq), _ptr(tile_q0), n_tiles, q_heads,
              kv_heads, dim, page_tokens, float(scale), int(window), vdim, _ptr(sinks), _ptr(gates), int(chunk), int(keep_first),
              _stream()),
           "attention_simt")
    return out


def attention_f32(q, cache, out, block_table, batch, q_heads, kv_heads, dim, page_tokens, scale, window, vdim=None,
                  sinks=None, gates=None, chunk=0, keep_first=0):
    """The 32-bit path's attention for one step: one kernel for every mix of segment lengths (and, in
    either precision, the attention with sinks, head gates or values of another size than keys)."""
    tiles = batch.tiles[attention_simt_block_queries()]
    attention_simt(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq, tiles.tile_q0,
                   tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window, vdim, sinks, gates, chunk, keep_first)


# ------------------------------------------------------------------ sampling
def sample(logits: torch.Tensor, tokens: torch.Tensor, records: torch.Tensor | None = None,
           row_slots: torch.Tensor | None = None, positions: torch.Tensor | None = None,
           logit_rows: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """tokens[r] = the next token of row r of logits (float32 [R, V], rows may be strided).

    With `records` (int32 [slots, RECORD_WORDS]) and `row_slots` (int32 [R]) row r belongs to the
    request in slot row_slots[r]: temperature 0 there is the first index of the maximum, otherwise a
    Gumbel-max draw keyed by the record's seed and counter; the kernel stores the token as the
    record's last token, bumps its counter and, given `positions` [T] and `logit_rows` [R], sets its
    position. Without records every row is greedy. `status` (int64 device addresses of other
    libraries' error words, from `status_words`) are copied to tokens[R:], so tokens holds
    R + len(status) ints."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sample: logits must be float32 [rows, vocab] with a contiguous vocabulary")
    _need(tokens, torch.int32, "tokens")
    rows, vocab = logits.shape
    n_status = 0 if status is None else status.shape[0]
    if tokens.shape[0] < rows + n_status:
        raise ValueError("sample: tokens must hold a word per row and per status word")
    if records is not None:
        _need(records, torch.int32, "records"); _need(row_slots, torch.int32, "row_slots")
        if records.dim() != 2 or records.shape[1] != RECORD_WORDS or row_slots.shape[0] < rows:
            raise ValueError("sample: records must be [slots, RECORD_WORDS] and row_slots one entry per row")
    for name, t in (("positions", positions), ("logit_rows", logit_rows)):
        if t is not None:
            _need(t, torch.int32, name)
    if status is not None:
        _need(status, torch.int64, "status")
    fn = _fn("sampling", "lb_sample", [c_void_p, c_long, c_int, c_int] + [c_void_p] * 6 + [c_int, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), rows, vocab, _ptr(records), _ptr(row_slots), _ptr(positions),
              _ptr(logit_rows), _ptr(tokens), _ptr(status), n_status, _stream()), "sample")
    return tokens


# ------------------------------------------------------------------ error words of the tensor-core kernels
# Every wait inside the tcgen05 kernels is bounded; a wait that runs out records a code in the
# library's error word and the block leaves. The sampling kernel copies those words behind the
# tokens it writes, so the host sees them with every step's tokens and without a synchronisation
# of its own (`Sampler`); `status_words` lists them, `explain_status` names a code's library, and
# `reset_after_error` puts back what such a block may have left behind (counters that a launch
# normally returns to zero).
_STATUS_LIBRARIES = (("gemm_tcgen05", "lb_gemm_tcgen05_status_address", "lb_gemm_tcgen05_status"),
                     ("attention_tcgen05", "lb_attention_tcgen05_status_address", "lb_attention_tcgen05_status"))
_status_words: dict[tuple[int, tuple[str, ...]], tuple[torch.Tensor, tuple[str, ...]]] = {}


def status_words(device: torch.device, libraries) -> tuple[torch.Tensor | None, tuple[str, ...]]:
    """(int64 device tensor of the error words' addresses, the libraries they belong to) for those of
    `libraries` that have one; (None, ()) if none has."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    wanted = tuple(name for name, _, _ in _STATUS_LIBRARIES if name in libraries)
    key = (index, wanted)
    if key not in _status_words:
        addresses = []
        with torch.cuda.device(index):
            for name, getter, _ in _STATUS_LIBRARIES:
                if name in wanted:
                    fn = getattr(build.load(name), getter)
                    fn.restype = c_void_p
                    address = fn()
                    if not address:
                        raise KernelError(f"{name}: the address of its error word cannot be had")
                    addresses.append(address)
            tensor = torch.tensor(addresses, dtype=torch.int64, device="cuda") if addresses else None
        _status_words[key] = (tensor, wanted)
    return _status_words[key]


def reset_after_error(device: torch.device) -> None:
    """After a kernel reported a wait that ran out: wait for the device, clear the error words and zero
    the split counters (a block that gave up does not take part in returning them to zero)."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    with torch.cuda.device(index):
        torch.cuda.synchronize()
        for name, _, clear in _STATUS_LIBRARIES:
            if name in build.loaded():
                fn = getattr(build.load(name), clear)
                fn.restype = c_int
                fn()
        if index in _scratch:
            _scratch[index][1].zero_()
        if index in _attn_scratch:
            _attn_scratch[index][1].zero_()
        torch.cuda.synchronize()


# ------------------------------------------------------------------ the bfloat16 path
# Split-K scratch and counters are one set per device, shared by every model, engine and stream of
# the process: a launch leaves its counters at zero for the next one, and two launches that overlap
# on the device would mix their partial tiles. So all launches of a device must be ordered on ONE
# stream (the engine runs everything on torch's current stream; the warm-up of a graph capture runs
# on a side stream only while the main stream waits for it).
_SCRATCH_FLOATS = 8 << 20     # split-K partial tiles (32 MiB)
_SCRATCH_COUNTERS = 4096
_scratch: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = {}


def gemm_scratch(device: torch.device) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Per device: the split-K scratch, its tile counters (zero between launches) and the SM count.
    Made once, outside any graph capture (models call this when their runtime is made)."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if index not in _scratch:
        with torch.cuda.device(index):
            partials = torch.empty(_SCRATCH_FLOATS, dtype=torch.float32, device="cuda")
            counters = torch.zeros(_SCRATCH_COUNTERS, dtype=torch.int32, device="cuda")
        _scratch[index] = (partials, counters, torch.cuda.get_device_properties(index).multi_processor_count)
    return _scratch[index]


def gemm_tcgen05_supports(a: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides: K-contiguous rows whose stride is a multiple of 8."""
    return (a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1)


SWIGLU_BLOCK = 64   # gate and up rows alternate in blocks of this many features for the fused epilogue


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2 I, H] with rows in blocks of 64 gate rows followed by the 64 up rows of the same features:
    the layout `gemm_tcgen05(..., epilogue="swiglu")` wants. I must be a multiple of 64."""
    inter, hidden = gate.shape
    if inter % SWIGLU_BLOCK or up.shape != gate.shape:
        raise ValueError("interleave_gate_up: the width must be a multiple of 64 and the shapes must agree")
    blocks = inter // SWIGLU_BLOCK
    stacked = torch.stack((gate.view(blocks, SWIGLU_BLOCK, hidden), up.view(blocks, SWIGLU_BLOCK, hidden)), dim=1)
    return stacked.reshape(2 * inter, hidden).contiguous()


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, max_splits: int = 0,
                 epilogue: str | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores; bfloat16 in, out bfloat16 or float32.

    epilogue "swiglu": w's rows are interleaved by `interleave_gate_up` and out[M, N / 2] = silu(gate) * up,
    rounded where the reference's bfloat16 tensors round."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        raise ValueError("gemm_tcgen05: operands must be 2-D bfloat16")
    m, k = a.shape
    n = w.shape[0]
    if epilogue not in (None, "swiglu"):
        raise ValueError(f"gemm_tcgen05: unknown epilogue {epilogue!r}")
    out_cols = n // 2 if epilogue == "swiglu" else n
    if epilogue == "swiglu" and (n % (2 * SWIGLU_BLOCK) or out.dtype != torch.bfloat16):
        raise ValueError("gemm_tcgen05: the swiglu epilogue needs interleaved weights (2 I rows, I % 64 == 0) and a bfloat16 output")
    if w.shape[1] != k or tuple(out.shape) != (m, out_cols) or out.stride(1) != 1:
        raise ValueError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    partials, counters, sms = gemm_scratch(a.device)
    fn = _fn("gemm_tcgen05", "lb_gemm_tcgen05",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_long, c_long, c_long, c_void_p, c_long,
              c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0), out.stride(0),
              _ptr(partials), partials.numel(), _ptr(counters), counters.numel(), sms, int(max_splits),
              1 if epilogue == "swiglu" else 0, _stream()), "gemm_tcgen05")
    return out


def gemm_qkv_heads(h: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   q_norm_w: torch.Tensor, k_norm_w: torch.Tensor, table: torch.Tensor, slot_map: torch.Tensor,
                   q_heads: int, kv_heads: int, dim: int, page_tokens: int, eps: float) -> bool:
    """The stacked q/k/v projection of up to 16 tokens, or of 512 and more, with the per-head norm, the
    rotation and the page write in its epilogue (head size 128): leaves in q_out and the pools what
    `gemm_tcgen05` followed by `qk_norm_rope_kv` leaves there, bit for bit. False: these sizes are not
    taken and nothing was launched."""
    tokens = h.shape[0]
    if (dim != 128 or 16 < tokens < 512 or h.dtype != torch.bfloat16 or q_norm_w is None or k_norm_w is None or table is None
            or k_pool is None or not gemm_tcgen05_supports(h, w_qkv)):
        return False
    for name, t in (("h", h), ("w_qkv", w_qkv), ("q_out", q_out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        _need(t, torch.float32, name)
    _need(slot_map, torch.int32, "slot_map")
    if w_qkv.shape != ((q_heads + 2 * kv_heads) * dim, h.shape[1]) or tuple(table.shape) != (tokens, 2, dim // 2) \
            or q_out.shape != (tokens, q_heads * dim) or not q_out.is_contiguous():
        raise ValueError("gemm_qkv_heads: shapes do not agree")
    sms = gemm_scratch(h.device)[2]
    fn = _fn("gemm_tcgen05", "lb_gemm_qkv_heads",
             [c_void_p, c_void_p, c_int, c_int, c_long, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p])
    code = fn(_ptr(h), _ptr(w_qkv), tokens, h.shape[1], h.stride(0), w_qkv.stride(0), q_heads, kv_heads, dim,
              _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table), table.shape[2], _ptr(slot_map), _ptr(q_out), _ptr(k_pool),
              _ptr(v_pool), page_tokens, float(eps), sms, _stream())
    if code == 1:
        return False
    _check(code, "gemm_qkv_heads")
    return True


def gemm_status() -> int:
    """0, or the code a tensor-core product recorded when one of its bounded waits ran out
    (1 loads, 2 MMAs, 3 epilogue). Synchronises; clears the code."""
    lib = build.load("gemm_tcgen05")
    lib.lb_gemm_tcgen05_status.restype = c_int
    torch.cuda.synchronize()
    return lib.lb_gemm_tcgen05_status()


def gemm_set_status(code: int) -> None:
    """Write the tensor-core product's error word from the host (a drill of the reporting path)."""
    lib = build.load("gemm_tcgen05")
    lib.lb_gemm_tcgen05_set_status.restype = c_int
    lib.lb_gemm_tcgen05_set_status.argtypes = [c_int]
    torch.cuda.synchronize()
    if lib.lb_gemm_tcgen05_set_status(int(code)):
        raise KernelError("gemm_tcgen05: cannot write the error word")


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T, bfloat16 operands, 32-bit accumulation; out bfloat16 or float32.
    Shapes that TMA cannot address (a row stride that is no multiple of 16 bytes) take the FFMA kernel."""
    if gemm_tcgen05_supports(a, w):
        return gemm_tcgen05(a, w, out)
    return gemm_simt(a, w, out)


_attn_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
_ATTN_SCRATCH_FLOATS = 8 << 20     # split-K partial outputs (32 MiB)
_ATTN_COUNTERS = 1 << 16


def attention_scratch(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per device: scratch for the decode kernel's split partials and its (sequence, KV head) counters."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if index not in _attn_scratch:
        with torch.cuda.device(index):
            _attn_scratch[index] = (torch.empty(_ATTN_SCRATCH_FLOATS, dtype=torch.float32, device="cuda"),
                                    torch.zeros(_ATTN_COUNTERS, dtype=torch.int32, device="cuda"))
    return _attn_scratch[index]


def attention_mma_block_queries() -> int:
    lib = build.load("attention_mma")
    lib.lb_attention_mma_block_queries.restype = c_int
    return lib.lb_attention_mma_block_queries()


def _sink_arguments(sinks, gates, tokens, q_heads, what):
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        if sinks.numel() != q_heads:
            raise ValueError(f"{what}: one sink per query head")
    if gates is not None:
        _need(gates, torch.float32, "gates")
        if tuple(gates.shape) != (tokens, q_heads):
            raise ValueError(f"{what}: gates must be [tokens, q_heads]")


def attention_prefill_bf16(q, k_pool, v_pool, out, block_table, cu_q, ctx_len, tile_seq, tile_q0, n_tiles, q_heads,
                           kv_heads, dim, page_tokens, scale, window=0, sinks=None, gates=None, exact_weights=False, keep_first=0):
    """Tensor-core paged attention for prompt portions: tiles of 64 queries, any number of queries per sequence.
    `window` > 0: the last `window` keys; `window` < 0: a chunked mask, the keys of the query's own chunk of -window positions.
    `sinks` float32 [q_heads] join the softmax's denominator only, `gates` float32 [T, q_heads] multiply the
    heads' outputs, `exact_weights` keeps 16 bits of the weights' mantissa in the second product. `keep_first` (with a
    window): the first keys of a sequence stay visible behind the window."""
    _sink_arguments(sinks, gates, q.shape[0], q_heads, "attention_prefill_bf16")
    for name, t in (("q", q), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_mma", "lb_attention_prefill_bf16",
             [c_void_p] * 5 + [c_int] + [c_void_p] * 4 + [c_int] * 5 + [c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
              _ptr(ctx_len), _ptr(tile_seq), _ptr(tile_q0), n_tiles, q_heads, kv_heads, dim, page_tokens, float(scale),
              int(window), _ptr(sinks), _ptr(gates), int(bool(exact_weights)), int(keep_first), _stream()), "attention_prefill_bf16")
    return out


def decode_plan(n_seqs: int, q_heads: int, kv_heads: int, dim: int, max_context: int, sm_count: int,
                mean_context: int | None = None) -> tuple[int, int]:
    """(splits, stages): how many ways to split the context of a decode step, and which kernel variant.

    A block is one (sequence, KV head, split). With three K/V tiles in shared memory two blocks fit an
    SM; the variant with two tiles fits three (head size 128, at most 8 heads per KV head) but each
    block is slower (about 1.15x per tile). Blocks run in rounds of blocks-per-SM x SMs. With head size
    128 the kernel runs 2, 4 or 8 splits as a thread-block cluster that merges through distributed
    shared memory (16 where all the launch's blocks still fit one per SM: a single sequence, 8.7
    against 10.6 us at 3,072 keys; two sequences 16.5 against 12.1 us, so not there); more splits merge
    through scratch memory, which costs more. The plan is the one
    with the lowest estimate rounds x (64-key tiles per split + overhead in tiles): 4 for a cluster,
    10 for the scratch merge. That fits what was measured at 3,072 keys (sequences: best splits)
    1: 8, 4: 8, 8: 4, 16: 2, 24: 4, 32: 1, 40: 4, 48: 2, 128: 2, one sequence of 32,768 keys: 32 or
    more through scratch memory, and 64 sequences: 4 splits with three blocks an SM (148 us against
    158 us unsplit with two).

    `mean_context`: the sequences' mean length where it is known to be well below the longest (more
    than 1.5 times). The longest sequence's blocks then run on alone at a lone block's rate after the
    others have finished, so the context is cut further, into about 7 blocks an SM (at least 12 tiles
    each), with three blocks an SM as soon as two do not hold them all. Measured with lengths spread
    evenly over 0.1..1 of 8,192 keys (us, the plan for equal lengths against this one): 8 sequences
    54 -> 47, 16: 106 -> 80, 32: 219 -> 136; over 0.1..1 of 3,072 keys: 16: 41 -> 36, 32: 79 -> 56."""
    natural = n_seqs * kv_heads
    want = max(1, 2 * sm_count // natural)                    # all blocks resident at once, two per SM
    splits = min(want, 128, max(1, max_context // 192))       # at least three 64-key tiles per split
    while splits > 1 and n_seqs * q_heads * splits * (dim + 2) > _ATTN_SCRATCH_FLOATS:
        splits -= 1
    if dim != 128:
        return splits, 3
    tiles = max(1, -(-max_context // 64))

    def estimate(count: int, overhead: int, per_sm: int = 2, tile_cost: float = 1.0) -> float:
        return -(-natural * count // (per_sm * sm_count)) * (-(-tiles // count) * tile_cost + overhead)

    clustered = [c for c in (1, 2, 4, 8) if c <= tiles]
    if 16 <= tiles // 3 and natural * 16 <= sm_count:
        clustered.append(16)
    best = min(clustered, key=lambda c: (estimate(c, 4), c))
    plan, cost = (best, 3), estimate(best, 4)
    if splits > 8 and estimate(splits, 10) < cost:
        plan, cost = (splits, 3), estimate(splits, 10)
    skewed = mean_context is not None and 2 * max_context > 3 * max(1, mean_context)
    if skewed and q_heads // kv_heads <= 8 and 8 * natural > 2 * sm_count and 10 * natural < 34 * sm_count:
        count = 1
        while count < 8 and 2 * count * count * natural * natural <= (7 * sm_count) ** 2:   # nearest power of two to 7 SMs / natural
            count *= 2
        while count > 1 and tiles // count < 12:
            count //= 2
        if count >= 2:
            return (count, 3) if natural * count <= 2 * sm_count else (count, 2)
    if 10 * natural >= 17 * sm_count and natural <= 2 * sm_count and tiles >= 64 and q_heads // kv_heads <= 8:
        # just under two blocks an SM, long contexts: four splits with three blocks an SM measured
        # 200 against 225 us (32 sequences of 8,192 keys; at 3,072 keys the two are equal)
        return 4, 2
    if natural > 2 * sm_count and q_heads // kv_heads <= 8:
        # more blocks than two per SM hold at once: three slower blocks an SM may finish sooner
        packed = min((c for c in (1, 2, 4, 8) if c <= tiles), key=lambda c: (estimate(c, 4, 3, 1.15), c))
        if estimate(packed, 4, 3, 1.15) < cost:
            plan = (packed, 2)
    return plan


def decode_splits(n_seqs: int, q_heads: int, kv_heads: int, dim: int, max_context: int, sm_count: int) -> int:
    return decode_plan(n_seqs, q_heads, kv_heads, dim, max_context, sm_count)[0]


def attention_decode_bf16(q, k_pool, v_pool, out, block_table, cu_q, ctx_len, seq_list, n_seqs, q_heads, kv_heads, dim,
                          page_tokens, scale, window=0, splits=1, stages=3, sinks=None, gates=None, exact_weights=False,
                          keep_first=0, kv_share=1):
    """Tensor-core paged attention for sequences with one new token each, the context split `splits` ways
    (`stages` 2: the variant that fits three blocks an SM, see `decode_plan`). `sinks`, `gates` and
    `exact_weights` as in `attention_prefill_bf16` (those variants merge their splits through scratch memory). `kv_share` > 1:
    `kv_heads` counts groups of at most 16 query heads, and kv_share neighbouring groups read the same stored head (the pools
    hold kv_heads / kv_share heads): more query heads on one key/value head than the kernel's tile has rows."""
    _sink_arguments(sinks, gates, q.shape[0], q_heads, "attention_decode_bf16")
    for name, t in (("q", q), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    if seq_list is not None:
        _need(seq_list, torch.int32, "seq_list")
    partials, counters = attention_scratch(q.device)
    fn = _fn("attention_mma", "lb_attention_decode_bf16",
             [c_void_p] * 5 + [c_int] + [c_void_p] * 3 + [c_int] * 5 + [c_float, c_int, c_int, c_void_p, c_long, c_void_p,
                                                                        c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
              _ptr(ctx_len), _ptr(seq_list), n_seqs, q_heads, kv_heads, dim, page_tokens, float(scale), int(window),
              int(splits), _ptr(partials), partials.numel(), _ptr(counters), counters.numel(), int(stages), _ptr(sinks),
              _ptr(gates), int(bool(exact_weights)), int(keep_first), int(kv_share), _stream()), "attention_decode_bf16")
    return out


# ---- attention on tcgen05 (head size 128, pages of 8..128 tokens dividing 128)
TCGEN05_TILE = 128
_pool_maps: dict[tuple, object] = {}


def attention_tcgen05_takes_heads(q_heads: int, kv_heads: int, dim: int) -> bool:
    """Whether the tcgen05 prompt attention has a kernel for these heads (whatever the page size)."""
    return dim == 128 and kv_heads > 0 and q_heads % kv_heads == 0 and q_heads // kv_heads <= 128


def attention_tcgen05_supports(q_heads: int, kv_heads: int, dim: int, page_tokens: int) -> bool:
    return (attention_tcgen05_takes_heads(q_heads, kv_heads, dim)
            and page_tokens >= 8 and page_tokens % 8 == 0 and 128 % page_tokens == 0)


def _pool_map(pool: torch.Tensor):
    """The TMA tensor map of a cache group's pool [layers, 2, pages, kv_heads, page_tokens, dim], made once."""
    key = (pool.data_ptr(), tuple(pool.shape))
    blob = _pool_maps.get(key)
    if blob is None:
        _need(pool, torch.bfloat16, "pool")
        layers, two, pages, kv_heads, page_tokens, dim = pool.shape
        blob = (ctypes.c_ubyte * 128)()
        fn = _fn("attention_tcgen05", "lb_attention_tcgen05_pool_map", [c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int])
        code = fn(ctypes.addressof(blob), _ptr(pool), layers * two, pages, kv_heads, page_tokens, dim)
        if code:
            raise ValueError(f"attention_tcgen05: cannot describe the pool to TMA ({_REFUSALS.get(code, code)})")
        _pool_maps[key] = blob
    return blob


def attention_tcgen05_status() -> int:
    """0, or which bounded wait of the tensor-core attention ran out. Synchronises; clears the code."""
    lib = build.load("attention_tcgen05")
    lib.lb_attention_tcgen05_status.restype = c_int
    torch.cuda.synchronize()
    return lib.lb_attention_tcgen05_status()


def attention_tcgen05_prefill(q, pool, layer, out, block_table, cu_q, ctx_len, tile_seq, tile_q0, n_tiles, q_heads,
                              kv_heads, dim, page_tokens, scale, window=0):
    """Prompt portions on tcgen05: tiles of 128 queries; pool is the cache group's whole pool."""
    for name, t in (("q", q), ("out", out)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_tcgen05", "lb_attention_tcgen05_prefill",
             [c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_int] + [c_void_p] * 4 + [c_int] * 5 +
             [c_float, c_int, c_void_p])
    _check(fn(_ptr(q), q.shape[0], ctypes.addressof(_pool_map(pool)), int(layer), _ptr(out), _ptr(block_table),
              block_table.shape[1], _ptr(cu_q), _ptr(ctx_len), _ptr(tile_seq), _ptr(tile_q0), n_tiles, q_heads, kv_heads,
              dim, page_tokens, float(scale), int(window), _stream()), "attention_tcgen05_prefill")
    return out


def attention_bf16(q, cache, out, block_table, batch, q_heads, kv_heads, dim, page_tokens, scale, window, sinks=None,
                   gates=None, exact_weights=False, chunk=0, keep_first=0, decode_share=1):
    """The bfloat16 path's attention for one step: prompt portions go through the tcgen05 tile kernel
    where it takes the sizes (head size 128, pages of 8..128 tokens), else through the mma.sync
    one; single tokens, alone or beside prompt portions, go through the split decode kernel. With
    sinks, gates or exact weights the mma.sync kernels' variants for those run everywhere. `decode_share` > 1: the
    decode kernel takes the query heads of a key/value head as that many groups (each at most 16 heads)."""
    plain = sinks is None and gates is None and not exact_weights and not chunk and not keep_first
    extras = dict(sinks=sinks, gates=gates, exact_weights=exact_weights, keep_first=keep_first)
    if chunk:
        if window:
            raise ValueError("attention_bf16: a window and a chunked mask do not combine")
        window = -int(chunk)      # the mma.sync kernels read a negative window as a chunked mask of that size
    # a window (or a chunk) bounds the keys a single token reads, whatever its request's length
    seen = (lambda ctx: min(ctx, abs(window) + 63 + (-(-keep_first // 64) * 64 if keep_first else 0))) if window else (lambda ctx: ctx)
    decode_groups = kv_heads * decode_share
    if batch.all_decode and q_heads // decode_groups <= 16:
        sms = gemm_scratch(q.device)[2]
        # planned for the step's own lengths; a captured step for its class of steps (the widest context
        # its block table can describe, with the mean that the class stands for)
        widest = min(batch.plan_max_ctx or block_table.shape[1] * page_tokens, block_table.shape[1] * page_tokens)
        mean = batch.plan_mean_ctx or None
        splits, stages = decode_plan(batch.n_seqs, q_heads, decode_groups, dim, seen(widest), sms, seen(mean) if mean else None)
        attention_decode_bf16(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, None,
                              batch.n_seqs, q_heads, decode_groups, dim, page_tokens, scale, window, splits, stages,
                              kv_share=decode_share, **extras)
        return
    tiles_of = batch.tiles
    if batch.n_decode_seqs > 0 and q_heads // decode_groups <= 16:
        # a mixed step: the sequences with a single token go through the decode kernel (a tile kernel
        # would spend a whole tile of queries on each), the prompt portions through the tile kernel
        sms = gemm_scratch(q.device)[2]
        mean = batch.plan_mean_ctx or None
        splits, stages = decode_plan(batch.n_decode_seqs, q_heads, decode_groups, dim, seen(batch.decode_max_ctx), sms,
                                     seen(mean) if mean else None)
        attention_decode_bf16(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, batch.decode_seqs,
                              batch.n_decode_seqs, q_heads, decode_groups, dim, page_tokens, scale, window, splits, stages,
                              kv_share=decode_share, **extras)
        tiles_of = batch.portion_tiles
    if plain and cache.pool is not None and attention_tcgen05_supports(q_heads, kv_heads, dim, page_tokens):
        tiles = tiles_of[TCGEN05_TILE]
        attention_tcgen05_prefill(q, cache.pool, cache.layer, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq,
                                  tiles.tile_q0, tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window)
        return
    tiles = tiles_of[attention_mma_block_queries()]
    attention_prefill_bf16(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq,
                           tiles.tile_q0, tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window, **extras)

"""Python entry points of the hand-written kernels.

Each function checks its tensors (device, dtype, layout), calls the C launcher
on the current CUDA stream and raises ``KernelError`` with the launcher's
message if it refuses the sizes.  Tensors must live on a CUDA device: there is
no CPU path.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .build import load_module

DT_F32, DT_BF16 = 0, 1
PAGE_SIZE = 64          # tokens per cache page


class KernelError(RuntimeError):
    pass


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return DT_F32
    if t == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {t}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream of the current device (also inside a graph capture, which runs on a stream of its own)."""
    if _raw_stream is not None:                      # the handle itself: a tenth of the cost of making a Stream object
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None):
    if not t.is_cuda:
        raise KernelError(f"{name}: must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: must have {ndim} dimensions, got {t.dim()}")


LAUNCHES = [0]          # kernels of this library launched so far (through these entry points)


_FUNCTIONS: dict = {}    # (module, name) -> (library, its function), looked up once


def _lookup(module: str, fn: str):
    entry = _FUNCTIONS.get((module, fn))
    if entry is None:
        lib = load_module(module)
        entry = _FUNCTIONS[module, fn] = (lib, getattr(lib, fn))
    return entry


def _call(module: str, fn: str, *args, kernels: int = 1):
    entry = _lookup(module, fn)
    rc = entry[1](*args)
    LAUNCHES[0] += kernels
    if rc != 0:
        raise KernelError(entry[0].qwb_last_error().decode("utf-8", "replace") or f"{fn} failed with code {rc}")


_i = ctypes.c_int
_f = ctypes.c_float


# ----------------------------------------------------------------------------- elementwise
def embed_gather(ids: torch.Tensor, table: torch.Tensor, bad_token: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """Rows of ``table`` [V, D] for int32 ``ids`` [T], times ``scale``, as float32 [T, D]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", ndim=2)
    T, (V, D) = ids.numel(), table.shape
    out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    _call("elementwise", "qwb_embed_gather", _ptr(ids), _ptr(table), _i(_dt(table.dtype)), _ptr(out),
          _i(T), _i(D), _i(V), _ptr(bad_token), _f(scale), _stream())
    return out


def embed_add(h: torch.Tensor, ids: torch.Tensor | None, table: torch.Tensor | None, scale: float = 1.0,
              vec: torch.Tensor | None = None) -> torch.Tensor:
    """In place on the float32 stream ``h`` [T, D]: h[t] += table[ids[t]] * scale + vec.  ``table`` (with ``ids``) or
    ``vec`` (float32 [D]) may be None."""
    _need(h, "h", torch.float32, 2)
    T, D = h.shape
    V = 0
    if table is not None:
        _need(ids, "ids", torch.int32, 1)
        _need(table, "table", ndim=2)
        V = table.shape[0]
        if table.shape[1] != D or ids.numel() != T:
            raise KernelError(f"embed_add: table {tuple(table.shape)}, {ids.numel()} ids for a stream {tuple(h.shape)}")
    if vec is not None:
        _need(vec, "vec", torch.float32, 1)
        if vec.numel() != D:
            raise KernelError(f"embed_add: a vector of {vec.numel()} for rows of {D}")
    _call("elementwise", "qwb_embed_add", _ptr(ids if table is not None else None), _ptr(table),
          _i(_dt(table.dtype) if table is not None else DT_F32), _ptr(vec), _ptr(h), _i(T), _i(D), _i(V), _f(scale), _stream())
    return h


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: torch.Tensor | None = None, write_sum: bool = False,
            rows: torch.Tensor | None = None, delta_scale: float = 1.0) -> torch.Tensor:
    """RMS norm of the rows of float32 ``x`` [T, D] (plus ``delta_scale`` times ``delta``), times ``weight``.

    With ``write_sum`` the sum x + delta replaces x.  With ``rows`` (int32) only
    those rows are normed and the output has one row per entry.  ``delta`` may be a ``SplitSum``
    (a product left as sums over pieces of k): its planes are added in their order.
    """
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    T, D = x.shape
    if weight.numel() != D:
        raise KernelError(f"rmsnorm: weight has {weight.numel()} entries for rows of {D}")
    n_rows = T
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.numel()
    out = torch.empty((n_rows, D), dtype=out_dtype, device=x.device)
    if isinstance(delta, SplitSum):
        if tuple(delta.planes.shape[1:]) != (T, D):
            raise KernelError(f"rmsnorm: planes {tuple(delta.planes.shape)} do not match x {tuple(x.shape)}")
        _call("elementwise", "qwb_rmsnorm_planes", _ptr(x), _ptr(delta.planes), _ptr(delta.plane_count),
              _i(delta.planes.shape[0]), _i(T), _ptr(x if write_sum else None), _ptr(weight), _ptr(out), _i(_dt(out_dtype)),
              _ptr(rows), _i(n_rows), _i(D), _f(eps), _stream())
        return out
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if delta.shape != x.shape:
            raise KernelError(f"rmsnorm: delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    _call("elementwise", "qwb_rmsnorm", _ptr(x), _ptr(delta), _ptr(x if (write_sum and delta is not None) else None),
          _ptr(weight), _ptr(out), _i(_dt(out_dtype)), _ptr(rows), _i(n_rows), _i(D), _f(eps), _f(delta_scale), _stream())
    return out


GATE_UP_GROUP = 8       # the fused products want gate and up rows interleaved in groups of this many features


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """[F, K] gate and up rows as one [2F, K] matrix: for every ``group`` features their gate rows, then their up rows.
    A reordering of rows; the products are the same numbers."""
    F, K = gate.shape
    if up.shape != gate.shape or F % group:
        raise KernelError(f"interleave_gate_up: shapes {tuple(gate.shape)}, {tuple(up.shape)} with groups of {group}")
    return torch.cat([gate.reshape(F // group, group, K), up.reshape(F // group, group, K)], dim=1).reshape(2 * F, K).contiguous()


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}      # what a gated feed-forward may put on its gate


def silu_mul(gate_up: torch.Tensor, out_dtype: torch.dtype, interleave: int = 0, activation: str = "silu",
             limit: float = 0.0) -> torch.Tensor:
    """act(gate) * up from a float32 [T, 2F] matrix: gate columns first (``interleave`` 0), or for every
    ``interleave`` features their gates and then their ups.  ``activation``: one of ``GATE_ACTIVATIONS``;
    "clamped_swish" is g sigmoid(1.702 g) (u + 1) with g = min(gate, ``limit``) and u = up clamped to +-``limit``."""
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"silu_mul: unknown gate activation '{activation}'")
    _need(gate_up, "gate_up", torch.float32, 2)
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError(f"silu_mul: {F2} columns cannot be split into gate and up")
    out = torch.empty((T, F2 // 2), dtype=out_dtype, device=gate_up.device)
    _call("elementwise", "qwb_silu_mul", _ptr(gate_up), _ptr(out), _i(_dt(out_dtype)), _i(T), _i(F2 // 2), _i(interleave),
          _i(GATE_ACTIVATIONS[activation]), _f(limit), _stream())
    return out


def add_inplace(out: torch.Tensor, delta: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out += scale * delta, float32, in place."""
    _need(out, "out", torch.float32)
    _need(delta, "delta", torch.float32)
    if out.shape != delta.shape:
        raise KernelError(f"add_inplace: shapes {tuple(out.shape)} and {tuple(delta.shape)} differ")
    _call("elementwise", "qwb_add_inplace", _ptr(out), _ptr(delta), ctypes.c_longlong(out.numel()), _f(scale), _stream())
    return out


def rmsnorm_onto(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                 cast_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """h += y / rms(y) * weight, row by row, in 32-bit and in place: the norm on a sublayer's output.  With
    ``cast_dtype`` the new h is also returned in that dtype (for the next product); float32 returns h itself."""
    _need(h, "h", torch.float32, 2)
    _need(y, "y", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    T, D = h.shape
    if y.shape != h.shape or weight.numel() != D:
        raise KernelError(f"rmsnorm_onto: h {tuple(h.shape)}, y {tuple(y.shape)}, weight of {weight.numel()}")
    cast = None
    if cast_dtype is not None and cast_dtype != torch.float32:
        cast = torch.empty((T, D), dtype=cast_dtype, device=h.device)
    _call("elementwise", "qwb_rmsnorm_onto", _ptr(y), _ptr(weight), _ptr(h), _ptr(cast),
          _i(_dt(cast_dtype) if cast is not None else DT_F32), _i(T), _i(D), _f(eps), _stream())
    if cast_dtype is None:
        return None
    return h if cast is None else cast


def rmsnorm_mix(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, alpha: float = 1.0,
                cast_dtype: torch.dtype | None = None):
    """The norm after the sum, in place on the float32 stream ``h`` [T, D]: h <- v * rsqrt(mean(v^2) + eps) * weight with
    v = alpha * h + y (``y`` float32 [T, D], a sublayer's output).  With ``cast_dtype`` also returns the new h in that
    dtype (h itself for float32), else None."""
    _need(h, "h", torch.float32, 2)
    _need(y, "y", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    T, D = h.shape
    if y.shape != h.shape or weight.numel() != D:
        raise KernelError(f"rmsnorm_mix: y {tuple(y.shape)}, weight of {weight.numel()} for a stream {tuple(h.shape)}")
    cast = None
    if cast_dtype is not None and cast_dtype != torch.float32:
        cast = torch.empty((T, D), dtype=cast_dtype, device=h.device)
    _call("elementwise", "qwb_rmsnorm_mix", _ptr(y), _ptr(weight), _ptr(h), _ptr(cast),
          _i(_dt(cast.dtype) if cast is not None else DT_F32), _i(T), _i(D), _f(eps), _f(alpha), _stream())
    if cast_dtype is None:
        return None
    return h if cast is None else cast


ACTIVATIONS = {"none": 0, "relu2": 1, "gelu_tanh": 2, "silu": 3, "xielu": 4}
ACTIVATION_PARAMS = {"xielu": 2}    # activations with learned numbers of their own, and how many


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, activation: str, out_dtype: torch.dtype,
             col0: int = 0, n_cols: int | None = None, params: torch.Tensor | None = None) -> torch.Tensor:
    """act(x + bias) for float32 x [T, F], or for its columns ``col0 .. col0 + n_cols``; ``activation`` one of
    ``ACTIVATIONS``.  Returns [T, F] (or [T, n_cols]) in ``out_dtype``; a float32 result of whole rows replaces x.
    With no bias and no activation this is the cast of a (slice of a) 32-bit result to a product's operand dtype."""
    _need(x, "x", torch.float32, 2)
    T, ld = x.shape
    F = ld - col0 if n_cols is None else n_cols
    if col0 < 0 or F <= 0 or col0 + F > ld:
        raise KernelError(f"bias_act: columns {col0}..{col0 + F} of rows of {ld}")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.numel() != F:
            raise KernelError(f"bias_act: bias of {bias.numel()} for rows of {F}")
    if activation not in ACTIVATIONS:
        raise KernelError(f"bias_act: unknown activation '{activation}'")
    if activation in ACTIVATION_PARAMS:
        if params is None:
            raise KernelError(f"bias_act: activation '{activation}' needs its {ACTIVATION_PARAMS[activation]} numbers")
        _need(params, "params", torch.float32, 1)
        if params.numel() != ACTIVATION_PARAMS[activation]:
            raise KernelError(f"bias_act: activation '{activation}' takes {ACTIVATION_PARAMS[activation]} numbers, got {params.numel()}")
    else:
        params = None
    whole = F == ld
    if whole and out_dtype == torch.float32 and bias is None and activation == "none":
        return x
    out = x if (out_dtype == torch.float32 and whole) else torch.empty((T, F), dtype=out_dtype, device=x.device)
    _call("elementwise", "qwb_bias_act", ctypes.c_void_p(x.data_ptr() + 4 * col0), _i(ld), _ptr(bias), _ptr(out),
          _i(_dt(out_dtype)), _i(T), _i(F), _i(ACTIVATIONS[activation]), _ptr(params), _stream())
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, out_dtype: torch.dtype | None = None,
              add: torch.Tensor | None = None, add_weight: torch.Tensor | None = None, add_eps: float | None = None,
              write_sum: bool = False, rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """Layer norm with a weight and no bias over the rows of float32 ``x`` [T, D], 32-bit throughout:
    (v - mean) / sqrt(mean of squared deviations + eps) * weight.

    With ``add`` (float32 [T, D]) the rows normed are x + LN(add) * add_weight: the norm of a sublayer's output is added
    first, and with ``write_sum`` that sum replaces x.  ``weight`` None: only that sum is made (returns None).  With
    ``rows`` (int32) only those rows are normed and the output has one row per entry."""
    _need(x, "x", torch.float32, 2)
    T, D = x.shape
    for name, t in (("weight", weight), ("add_weight", add_weight)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != D:
                raise KernelError(f"layernorm: {name} has {t.numel()} entries for rows of {D}")
    if (add is None) != (add_weight is None):
        raise KernelError("layernorm: a sublayer output and its norm's weight come together")
    if add is not None:
        _need(add, "add", torch.float32, 2)
        if add.shape != x.shape:
            raise KernelError(f"layernorm: add {tuple(add.shape)} does not match x {tuple(x.shape)}")
    n_rows = T
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.numel()
    out = None
    if weight is not None:
        out = torch.empty((n_rows, D), dtype=out_dtype, device=x.device)
    _call("layernorm", "qwb_layernorm", _ptr(x), _ptr(add), _ptr(add_weight), _f(eps if add_eps is None else add_eps),
          _i(1 if write_sum else 0), _ptr(weight), _ptr(out), _i(_dt(out_dtype) if out is not None else DT_F32), _ptr(rows),
          _i(n_rows), _i(D), _f(eps), _stream())
    return out


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32 ``x``: x * scale, then cap * tanh(x / cap) if ``cap`` > 0 (logits)."""
    _need(x, "x", torch.float32)
    if scale != 1.0 or cap > 0:
        _call("elementwise", "qwb_scale_softcap", _ptr(x), ctypes.c_longlong(x.numel()), _f(scale), _f(cap), _stream())
    return x


# ----------------------------------------------------------------------------- rope + cache write
def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, factor: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of positions[t] * inv_freq[i], times ``factor``, as float32 [T, half]; the angles are formed in
    float64."""
    _need(positions, "positions", torch.int32, 1)
    _need(inv_freq, "inv_freq", torch.float64, 1)
    T, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((T, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _call("rope_kv", "qwb_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), _i(T), _i(half),
          ctypes.c_double(factor), _stream())
    return cos, sin


def qk_norm_rope_store(qkv: torch.Tensor, q_weight, k_weight, cos, sin, tok_seq, tok_pos, page_table,
                       k_pool, v_pool, n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                       eps: float, store_kv: bool = True) -> torch.Tensor:
    """Per-head norm, rotation and cache write.  ``qkv`` float32 [T, (Hq + 2 Hkv) * hd];
    returns the rotated queries [T, Hq, hd] in the cache's dtype."""
    _need(qkv, "qkv", torch.float32, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope_store: qkv has {qkv.shape[1]} columns, expected "
                          f"{(n_heads + 2 * n_kv_heads) * head_dim}")
    _need(k_pool, "k_pool", ndim=4)
    _need(v_pool, "v_pool", k_pool.dtype, 4)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"qk_norm_rope_store: cache pool {tuple(k_pool.shape)} does not fit "
                          f"{n_kv_heads} heads of {head_dim}")
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != head_dim:
                raise KernelError(f"qk_norm_rope_store: {name} has {t.numel()} entries for heads of {head_dim}")
    if rotary_dim:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, rotary_dim // 2) or sin.shape != cos.shape:
            raise KernelError(f"qk_norm_rope_store: cos/sin {tuple(cos.shape)} do not fit {T} tokens and "
                              f"rotary size {rotary_dim}")
    _need(tok_seq, "tok_seq", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    q_out = torch.empty((T, n_heads, head_dim), dtype=k_pool.dtype, device=qkv.device)
    _call("rope_kv", "qwb_qk_norm_rope_store", _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(page_table), _ptr(q_out), _ptr(k_pool), _ptr(v_pool),
          _i(_dt(k_pool.dtype)), _i(T), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(rotary_dim), _f(eps),
          _i(k_pool.shape[2]), _i(page_table.shape[1]), _i(1 if store_kv else 0), _stream())
    return q_out


# ----------------------------------------------------------------------------- attention
def mma_attention_fits(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels take this case (else the plain ones do)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def tc_attention_fits(dtype: torch.dtype, head_dim: int, page_size: int, group: int) -> bool:
    """Whether the tcgen05 prefill attention kernel takes this case."""
    return mma_attention_fits(dtype, head_dim, page_size) and 1 <= group <= 64


def attn_prefill(q, k_pool, v_pool, page_table, cu_seqlens, pos0, max_new: int, scale: float,
                 window: int = 0, impl: str = "auto", chunk: int = 0, slopes=None, sinks=None) -> torch.Tensor:
    """Causal attention of new tokens over the cache.  q [T, Hq, hd]; returns [T, Hq * hd].
    impl: "auto" (the fastest that fits), "tc" (tcgen05), "mma" (mma.sync), or "plain".  ``chunk`` > 0: a query sees only
    the keys of its own block of ``chunk`` positions, counted from position 0; ``slopes`` / ``sinks`` (float32 [Hq]): a
    bias slopes[h] * distance off the scaled score, and exp(sinks[h]) in the softmax's denominator (all three: the
    tcgen05 kernel only)."""
    _need(q, "q", k_pool.dtype, 3)
    _need(k_pool, "k_pool", ndim=4)
    _need(v_pool, "v_pool", k_pool.dtype, 4)
    _need(page_table, "page_table", torch.int32, 2)
    _need(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _need(pos0, "pos0", torch.int32, 1)
    T, Hq, hd = q.shape
    B = pos0.numel()
    if cu_seqlens.numel() != B + 1 or page_table.shape[0] < B:
        raise KernelError("attn_prefill: cu_seqlens / page_table do not fit the batch")
    out = torch.empty((T, Hq * hd), dtype=q.dtype, device=q.device)
    group = Hq // max(1, k_pool.shape[1])
    # the tcgen05 kernel works on tiles of 128 rows: it pays from a few dozen new tokens per sequence on
    use_tc = impl == "tc" or (impl == "auto" and max_new * group >= 64 and
                              tc_attention_fits(q.dtype, hd, k_pool.shape[2], group))
    if use_tc:
        if q.dtype != torch.bfloat16:
            raise KernelError("attn_prefill: the tensor-core kernel takes bfloat16 only")
        for name, t in (("slopes", slopes), ("sinks", sinks)):
            if t is not None:
                _need(t, name, torch.float32, 1)
                if t.numel() != Hq:
                    raise KernelError(f"attn_prefill: {name} of {t.numel()} for {Hq} heads")
        _call("attention_tc", "qwb_attn_tc_prefill_shaped", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
              _ptr(cu_seqlens), _ptr(pos0), _ptr(out), _i(B), _i(T), _i(max_new), _i(k_pool.shape[0]), _i(Hq),
              _i(k_pool.shape[1]), _i(hd), _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _i(chunk),
              _ptr(slopes), _ptr(sinks), _ptr(gemm_tc_error_word(q.device)), _stream())
        return out
    if chunk or slopes is not None or sinks is not None:
        raise KernelError("attn_prefill: only the tcgen05 kernel masks by chunks, biases by distance or has a sink")
    use_mma = impl == "mma" or (impl == "auto" and mma_attention_fits(q.dtype, hd, k_pool.shape[2]))
    if use_mma:
        if q.dtype != torch.bfloat16:
            raise KernelError("attn_prefill: the tensor-core kernel takes bfloat16 only")
        _call("attention_mma", "qwb_attn_mma_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
              _ptr(cu_seqlens), _ptr(pos0), _ptr(out), _i(B), _i(max_new), _i(Hq), _i(k_pool.shape[1]), _i(hd),
              _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _stream())
        return out
    _call("attention", "qwb_attn_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(cu_seqlens),
          _ptr(pos0), _ptr(out), _i(_dt(q.dtype)), _i(B), _i(max_new), _i(Hq), _i(k_pool.shape[1]), _i(hd),
          _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _stream())
    return out


def attn_decode_scratch_floats(B: int, Hq: int, hd: int, max_runs: int) -> int:
    return B * Hq * max_runs * (hd + 2)


MMA_RUNS_TARGET = 16        # the tensor-core decode kernel cuts a sequence into about this many runs of keys ...
MMA_RUN_PAGES_MAX = 8       # ... of at most this many pages each (more runs beyond that)


def mma_decode_runs(max_len: int, runs_target: int = MMA_RUNS_TARGET, run_pages_max: int = MMA_RUN_PAGES_MAX) -> int:
    """The most runs that the tensor-core decode kernel cuts a sequence of up to ``max_len`` keys into."""
    return int(load_module("attention_mma").qwb_attn_mma_decode_runs(_i(max_len), _i(runs_target), _i(run_pages_max)))


def attn_decode(q, k_pool, v_pool, page_table, seq_len, scale: float, max_len: int, window: int = 0,
                split_tokens: int = 256, scratch: torch.Tensor | None = None, impl: str = "auto",
                runs_target: int = MMA_RUNS_TARGET, run_pages_max: int = MMA_RUN_PAGES_MAX) -> torch.Tensor:
    """Attention of one new token per sequence over the cache.  q [B, Hq, hd]; ``seq_len`` counts
    the new token; ``max_len`` bounds every entry of ``seq_len``.  Returns [B, Hq * hd].

    The keys are cut into runs whose partial results are merged.  The plain kernel cuts into runs of
    ``split_tokens`` keys.  The tensor-core kernel cuts a sequence of p pages into runs of
    clamp(ceil(p / runs_target), 1, run_pages_max) pages (``runs_target`` 1: runs of exactly ``run_pages_max``
    pages): by the sequence's own length, never by what else is in the batch."""
    _need(q, "q", k_pool.dtype, 3)
    _need(k_pool, "k_pool", ndim=4)
    _need(v_pool, "v_pool", k_pool.dtype, 4)
    _need(page_table, "page_table", torch.int32, 2)
    _need(seq_len, "seq_len", torch.int32, 1)
    B, Hq, hd = q.shape
    use_mma = impl == "mma" or (impl == "auto" and mma_attention_fits(q.dtype, hd, k_pool.shape[2]))
    if use_mma and q.dtype != torch.bfloat16:
        raise KernelError("attn_decode: the tensor-core kernel takes bfloat16 only")
    if use_mma:
        max_runs = max(1, mma_decode_runs(max_len, runs_target, run_pages_max))
    else:
        max_runs = max(1, math.ceil(max_len / split_tokens))
    need = attn_decode_scratch_floats(B, Hq, hd, max_runs) if max_runs > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if scratch is not None:
        _need(scratch, "scratch", torch.float32)
    out = torch.empty((B, Hq * hd), dtype=q.dtype, device=q.device)
    if use_mma:
        _call("attention_mma", "qwb_attn_mma_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
              _ptr(seq_len), _ptr(scratch), _ptr(out), _i(B), _i(Hq), _i(k_pool.shape[1]), _i(hd), _i(k_pool.shape[2]),
              _i(page_table.shape[1]), _f(scale), _i(window), _i(runs_target), _i(run_pages_max), _i(max_len), _stream(),
              kernels=2 if max_runs > 1 else 1)
        return out
    _call("attention", "qwb_attn_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(seq_len),
          _ptr(scratch), _ptr(out), _i(_dt(q.dtype)), _i(B), _i(Hq), _i(k_pool.shape[1]), _i(hd),
          _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _i(split_tokens), _i(max_runs),
          _stream(), kernels=2 if max_runs > 1 else 1)
    return out


def attn_decode_fused(qkv: torch.Tensor, q_weight, k_weight, cos, sin, eps: float, k_pool, v_pool, page_table, seq_len,
                      scale: float, max_len: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int = 0,
                      store_kv: bool = True, scratch: torch.Tensor | None = None,
                      runs_target: int = MMA_RUNS_TARGET, run_pages_max: int = MMA_RUN_PAGES_MAX) -> torch.Tensor:
    """``qk_norm_rope_store`` and ``attn_decode`` in one kernel, for a step of one token per sequence on the tensor-core
    path (bfloat16 cache, head size 64 or 128, rotation over the whole head or none): ``qkv`` float32
    [B, (Hq + 2 Hkv) * hd] is the q/k/v projection's output; the new keys and values are written into the cache at
    position ``seq_len - 1`` (unless ``store_kv`` is False).  Returns [B, Hq * hd] bfloat16."""
    _need(qkv, "qkv", torch.float32, 2)
    _need(k_pool, "k_pool", torch.bfloat16, 4)
    _need(v_pool, "v_pool", torch.bfloat16, 4)
    _need(page_table, "page_table", torch.int32, 2)
    _need(seq_len, "seq_len", torch.int32, 1)
    B = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim or seq_len.numel() != B or page_table.shape[0] != B:
        raise KernelError(f"attn_decode_fused: qkv {tuple(qkv.shape)}, {seq_len.numel()} lengths, page table "
                          f"{tuple(page_table.shape)} do not fit {n_heads}+2x{n_kv_heads} heads of {head_dim}")
    if not mma_attention_fits(k_pool.dtype, head_dim, k_pool.shape[2]):
        raise KernelError(f"attn_decode_fused: head size {head_dim} with pages of {k_pool.shape[2]} is not taken")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attn_decode_fused: cache pool {tuple(k_pool.shape)} does not fit {n_kv_heads} heads of {head_dim}")
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != head_dim:
                raise KernelError(f"attn_decode_fused: {name} has {t.numel()} entries for heads of {head_dim}")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("attn_decode_fused: the norm weights of q and k come together")
    if cos is not None:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (B, head_dim // 2) or sin.shape != cos.shape:
            raise KernelError(f"attn_decode_fused: cos/sin {tuple(cos.shape)} do not fit {B} tokens and a rotation "
                              f"over all {head_dim} values")
    max_runs = max(1, mma_decode_runs(max_len, runs_target, run_pages_max))
    need = attn_decode_scratch_floats(B, n_heads, head_dim, max_runs) if max_runs > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
    out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    _call("attention_mma", "qwb_attn_mma_decode_fused", _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
          _f(eps), _i(1 if store_kv else 0), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(seq_len), _ptr(scratch),
          _ptr(out), _i(B), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(k_pool.shape[2]), _i(page_table.shape[1]),
          _f(scale), _i(window), _i(runs_target), _i(run_pages_max), _i(max_len), _stream(),
          kernels=2 if max_runs > 1 else 1)
    return out


# ----------------------------------------------------------------------------- matrix products
SMALL_M = 16            # at most this many rows go to the weight-streaming kernel


def gemm_small(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed, as float32 [M, N] (+ residual), for few rows."""
    _need(x, "x", weight.dtype, 2)
    _need(weight, "weight", ndim=2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_small: x has {K} columns, the weight {weight.shape[1]}")
    if out is None:
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, 2)
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
    _call("gemm_small", "qwb_gemm_small", _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), _i(_dt(x.dtype)),
          _i(M), _i(N), _i(K), _stream(), kernels=(M + 7) // 8)
    return out


STREAM_M = 16           # at most this many bfloat16 rows go to the tensor-core weight-streaming kernel


STREAM_CONFIGS = ((2, 8), (4, 8), (8, 8), (2, 16), (4, 16), (2, 32))   # (blocks of 32 k in flight per warp, warps) that exist


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, config: tuple | None = None) -> torch.Tensor:
    """bfloat16 x [M, K] times bfloat16 weight [N, K] transposed, as float32 [M, N] (+ residual), M <= 16.
    ``config``: one of ``STREAM_CONFIGS`` (default: the kernel's own choice by shape)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_stream: x has {K} columns, the weight {weight.shape[1]}")
    if out is None:
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, 2)
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
    u, w = config or (0, 0)
    _call("gemm_stream", "qwb_gemm_stream", _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), _i(M), _i(N), _i(K),
          _i(u), _i(w), _stream())
    return out


def gemm_stream_swiglu(x: torch.Tensor, weight: torch.Tensor, config: tuple | None = None) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) as bfloat16 [M, F] for bfloat16 x [M, K], M <= 16, and the weight [2F, K] with gate and up
    rows interleaved in groups of 8 features (``interleave_gate_up``)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    if weight.shape[1] != K or weight.shape[0] % 2:
        raise KernelError(f"gemm_stream_swiglu: x is {tuple(x.shape)}, the weight {tuple(weight.shape)}")
    F = weight.shape[0] // 2
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    u, w = config or (0, 0)
    _call("gemm_stream", "qwb_gemm_stream_swiglu", _ptr(x), _ptr(weight), _ptr(out), _i(M), _i(F), _i(K), _i(u), _i(w), _stream())
    return out


RING_STAGE_K = 256              # k per stage of gemm_ring's ring; with 8 or 16 stages a row of W (rows of up to 2,048 or 4,096
RING_KEEPS_X_STAGES = (1, 2, 4, 8, 16)   # values) a warp meets the same k in every tile and keeps its pieces of x in registers


def gemm_ring(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """As ``gemm_stream``, by the kernel that streams W through a ring in shared memory filled by bulk copies and is built
    to overlap with the kernels before and after it.  A wait that gave up shows in ``gemm_tc_check``."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_ring: x has {K} columns, the weight {weight.shape[1]}")
    if out is None:
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, 2)
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
    _call("gemm_ring", "qwb_gemm_ring", _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), _i(M), _i(N), _i(K),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


class SplitSum:
    """A product [T, D] that its kernel left as sums over pieces of k: ``planes`` float32 [P, T, D], of which columns
    16 t .. 16 t + 15 have ``plane_count[t]`` (uint8); the product is the sum of a column's planes in their order.
    The kernel that consumes it adds them (``rmsnorm`` does; ``add_onto`` for any other consumer)."""
    __slots__ = ("planes", "plane_count")

    def __init__(self, planes: torch.Tensor, plane_count: torch.Tensor):
        self.planes, self.plane_count = planes, plane_count

    def add_onto(self, x: torch.Tensor) -> torch.Tensor:
        """x += the product, in place."""
        _need(x, "x", torch.float32, 2)
        if tuple(self.planes.shape[1:]) != tuple(x.shape):
            raise KernelError(f"SplitSum: planes {tuple(self.planes.shape)} do not match x {tuple(x.shape)}")
        _call("elementwise", "qwb_add_planes", _ptr(x), _ptr(self.planes), _ptr(self.plane_count), _i(x.shape[0]),
              _i(x.shape[1]), _stream())
        return x

    def total(self) -> torch.Tensor:
        """The product as one tensor (a new one)."""
        return self.add_onto(torch.zeros(self.planes.shape[1:], dtype=torch.float32, device=self.planes.device))


RING_TILE_ROWS = 16             # rows of W per tile of gemm_ring
RING_SPLIT_MAX_PLANES = 4       # the most planes that the consumers of a SplitSum add
RING_SPLIT_BELOW = 0.8          # the split form is used when whole tiles would keep the SMs busy for less than this share of
                                # their rounds (5,120 rows on 148 SMs: 0.72, where it takes 16.0 and 42.4 us for the o and down
                                # projections of the Qwen3-32B sizes against 19.5 and 54.4 us; 4,096 rows: 0.86, where the
                                # pieces' extra epilogues cost what the even shares save: 7.8 and 18.2 against 6.9 and 18.8 us,
                                # and a step with the down projection alone split 2,457 against 2,485 tokens/s)
_RING_PLANS: dict = {}


def ring_split_plan(N: int, K: int, device):
    """How gemm_ring's split form cuts an [N, K] matrix on this device: ``(blocks, n_planes, plane_count)``, or None when
    whole tiles are as good (they fill the SMs' rounds to RING_SPLIT_BELOW or more, or a tile would be cut into more
    than RING_SPLIT_MAX_PLANES pieces).  Block b takes stages [b * all / blocks, (b + 1) * all / blocks) of the
    ceil(N / 16) * ceil(K / 256) stages, counted tile by tile; a tile's planes are the blocks that hold a part of it."""
    dev = torch.device(device)
    key = (N, K, dev.index or 0)
    if key not in _RING_PLANS:
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        _RING_PLANS[key] = _ring_split_plan(N, K, n_sm, dev)
    return _RING_PLANS[key]


def ring_split_counts(N: int, K: int, blocks: int):
    """plane_count of every tile (a list), for ``blocks`` blocks: pure arithmetic, the same as the kernel's."""
    n_tiles, n_stages = -(-N // RING_TILE_ROWS), -(-K // RING_STAGE_K)
    all_stages = n_tiles * n_stages
    counts = []
    for t in range(n_tiles):
        first = ((t * n_stages + 1) * blocks - 1) // all_stages            # the block that holds the tile's first stage
        last = (((t + 1) * n_stages - 1 + 1) * blocks - 1) // all_stages   # ... and its last
        counts.append(last - first + 1)
    return counts


def _ring_split_plan(N: int, K: int, n_sm: int, device):
    n_tiles, n_stages = -(-N // RING_TILE_ROWS), -(-K // RING_STAGE_K)
    rounds = -(-n_tiles // n_sm)
    if n_tiles <= n_sm or n_tiles / (rounds * n_sm) >= RING_SPLIT_BELOW:
        return None
    counts = ring_split_counts(N, K, n_sm)
    if max(counts) > RING_SPLIT_MAX_PLANES:
        return None
    return n_sm, max(counts), torch.tensor(counts, dtype=torch.uint8, device=device)


def gemm_ring_split(x: torch.Tensor, weight: torch.Tensor, plan=None) -> SplitSum:
    """x W^T by the ring kernel's split form: every block streams an equal share of W and leaves its sums over pieces of
    tiles as planes (see ``SplitSum``).  ``plan``: from ``ring_split_plan`` (default: for this weight, which must have one)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_ring_split: x has {K} columns, the weight {weight.shape[1]}")
    if plan is None:
        plan = ring_split_plan(N, K, x.device)
        if plan is None:
            raise KernelError(f"gemm_ring_split: no split plan for a weight of {N} x {K}")
    blocks, n_planes, plane_count = plan
    planes = torch.empty((n_planes, M, N), dtype=torch.float32, device=x.device)
    _call("gemm_ring", "qwb_gemm_ring_split", _ptr(x), _ptr(weight), _ptr(planes), _i(M), _i(N), _i(K), _i(blocks),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return SplitSum(planes, plane_count)


def gemm_ring_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """As ``gemm_stream_swiglu``, by the ring kernel (see ``gemm_ring``)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    if weight.shape[1] != K or weight.shape[0] % 2:
        raise KernelError(f"gemm_ring_swiglu: x is {tuple(x.shape)}, the weight {tuple(weight.shape)}")
    F = weight.shape[0] // 2
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    _call("gemm_ring", "qwb_gemm_ring_swiglu", _ptr(x), _ptr(weight), _ptr(out), _i(M), _i(F), _i(K),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


def gemm_ring_xielu(x: torch.Tensor, weight: torch.Tensor, params: torch.Tensor) -> torch.Tensor:
    """bfloat16 xIELU(x W^T) [M, N] for up to 16 rows by the ring kernel, the activation in its epilogue."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    _need(params, "params", torch.float32, 1)
    M, K = x.shape
    if weight.shape[1] != K or params.numel() != 2:
        raise KernelError(f"gemm_ring_xielu: x is {tuple(x.shape)}, the weight {tuple(weight.shape)}, {params.numel()} numbers")
    out = torch.empty((M, weight.shape[0]), dtype=torch.bfloat16, device=x.device)
    _call("gemm_ring", "qwb_gemm_ring_xielu", _ptr(x), _ptr(weight), _ptr(out), _ptr(params), _i(M), _i(weight.shape[0]), _i(K),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


_TC_ERROR: dict = {}    # device -> one int32 that a gemm_tc kernel sets when one of its waits gives up
TC_EPILOGUES = {"store": 0, "add": 1, "swiglu": 2}


def gemm_tc_error_word(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _TC_ERROR:
        _TC_ERROR[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _TC_ERROR[key]


def gemm_tc_check(device) -> None:
    """Raise if a tcgen05 kernel (product or attention) on this device gave up a wait since the last check (reads one
    int: synchronises)."""
    word = gemm_tc_error_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        where = {1: "the loader waiting for a free stage", 2: "the tensor-core issuer waiting for its operands",
                 3: "the epilogue or softmax warps waiting for the tensor core",
                 7: "shared memory was not aligned to 1024 bytes"}.get(code, f"code {code}")
        raise KernelError(f"a bounded wait in a tcgen05 kernel ran out ({where}); that kernel's result is not valid")


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, epilogue: str = "store", out: torch.Tensor | None = None,
            tile_n: int | None = None) -> torch.Tensor:
    """bfloat16 x [M, K] times bfloat16 weight transposed on the tcgen05 tensor cores.

    "store": weight [N, K] -> float32 [M, N].  "add": the same, added onto ``out``.
    "swiglu": weight [2F, K] (gate and up rows interleaved in groups of 8 features, ``interleave_gate_up``)
    -> bfloat16 [M, F] = silu(gate) * up.
    """
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    if weight.shape[1] != K:
        raise KernelError(f"gemm_tc: x has {K} columns, the weight {weight.shape[1]}")
    if epilogue not in TC_EPILOGUES:
        raise KernelError(f"gemm_tc: unknown epilogue '{epilogue}'")
    if epilogue == "swiglu":
        if weight.shape[0] % 2:
            raise KernelError(f"gemm_tc: {weight.shape[0]} rows cannot be split into gate and up")
        N = weight.shape[0] // 2
        out_dtype = torch.bfloat16
    else:
        N = weight.shape[0]
        out_dtype = torch.float32
    if out is None:
        if epilogue == "add":
            raise KernelError("gemm_tc: the 'add' epilogue needs the tensor to add onto")
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, 2)
    if tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_tc: out is {tuple(out.shape)}, expected {(M, N)}")
    if tile_n is None:
        tile_n = 128 if epilogue == "swiglu" else (128 if N >= 1024 else 64)
    _call("gemm_tc", "qwb_gemm_tc", _ptr(x), _ptr(weight), _ptr(out), _i(TC_EPILOGUES[epilogue]), _i(M), _i(N), _i(K),
          _i(tile_n), _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


def gemm_tc_xielu(x: torch.Tensor, weight: torch.Tensor, params: torch.Tensor, tile_n: int = 256) -> torch.Tensor:
    """bfloat16 xIELU(x W^T) [M, N] on the tcgen05 tensor cores, the activation in the product's epilogue; ``params``:
    the activation's two learned numbers, float32 on the device."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    _need(params, "params", torch.float32, 1)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or params.numel() != 2:
        raise KernelError(f"gemm_tc_xielu: x {tuple(x.shape)}, weight {tuple(weight.shape)}, {params.numel()} numbers")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _call("gemm_tc", "qwb_gemm_tc_xielu", _ptr(x), _ptr(weight), _ptr(out), _ptr(params), _i(M), _i(N), _i(K), _i(tile_n),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


# ----------------------------------------------------------------------------- recurrent mixers
CONV_MAX_TAPS = 16


def short_conv(x: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: torch.Tensor | None,
               tail: torch.Tensor, ctx, activation: bool = True, update_tail: bool = True,
               in_bias: torch.Tensor | None = None, plus_input: bool = False,
               out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Causal convolution over time, per channel, of columns ``col0 .. col0 + channels`` of float32 ``x`` [T, ld], with
    SiLU after it (``activation``), or (``plus_input``, no activation) with the token's own input added to it:
    x + conv(x).  ``weight`` [channels, taps]: the last tap is the current token's.  ``tail``
    [slots, taps - 1, channels] float32 holds each sequence's last inputs (zero for a new one) and is brought up to
    date (``update_tail``).  ``in_bias`` [channels] is added to every input before the convolution (the bias of the
    projection that made x; the tail holds inputs with it).  ``ctx``: the step (tok_seq, cu_seqlens, slots).
    Returns [T, channels] in ``out_dtype`` (float32 or bfloat16)."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", torch.float32, 2)
    _need(tail, "tail", torch.float32, 3)
    if plus_input and activation:
        raise KernelError("short_conv: the input is added to a convolution without an activation")
    T, ld = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != channels or col0 < 0 or col0 + channels > ld:
        raise KernelError(f"short_conv: weight {tuple(weight.shape)} for columns {col0}..{col0 + channels} of {ld}")
    if tuple(tail.shape[1:]) != (taps - 1, channels):
        raise KernelError(f"short_conv: tail {tuple(tail.shape)} does not fit {taps} taps of {channels} channels")
    for name, t in (("bias", bias), ("in_bias", in_bias)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != channels:
                raise KernelError(f"short_conv: {name} of {t.numel()} for {channels} channels")
    out = torch.empty((T, channels), dtype=out_dtype, device=x.device)
    _call("recurrent", "qwb_short_conv", ctypes.c_void_p(x.data_ptr() + 4 * col0), _i(ld), _ptr(weight), _ptr(bias),
          _ptr(in_bias), _ptr(tail), _ptr(ctx.tok_seq), _ptr(ctx.cu_seqlens), _ptr(ctx.slots), _ptr(out), _i(_dt(out_dtype)),
          _i(T), _i(ctx.n_seqs), _i(channels), _i(taps), _i(2 if plus_input else (1 if activation else 0)),
          _i(1 if update_tail else 0),
          _i(1 if ctx.single_token else 0), _stream(),
          kernels=2 if (update_tail and taps > 1 and not ctx.single_token) else 1)
    return out


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_col0: int, dt_bias, a_log, d_skip, state: torch.Tensor, ctx,
             heads: int, vdim: int, n_state: int, groups: int, write_state: bool = True) -> torch.Tensor:
    """The Mamba-2 recurrence over a step's tokens.  ``xbc`` float32 [T, heads * vdim + 2 * groups * n_state] (x | B | C,
    after convolution and SiLU); the raw step sizes are columns ``dt_col0 ..`` of float32 ``dt`` [T, ld]; ``state``
    float32 [slots, heads, vdim, n_state] (column by column) is read and written back.  Returns y float32 [T, heads * vdim]."""
    _need(xbc, "xbc", torch.float32, 2)
    _need(dt, "dt", torch.float32, 2)
    _need(state, "state", torch.float32, 4)
    T = xbc.shape[0]
    if xbc.shape[1] != heads * vdim + 2 * groups * n_state or tuple(state.shape[1:]) != (heads, vdim, n_state):
        raise KernelError(f"ssm_scan: xbc {tuple(xbc.shape)}, state {tuple(state.shape)} do not fit {heads} heads of "
                          f"{vdim}, state {n_state}, {groups} groups")
    for name, t in (("dt_bias", dt_bias), ("A_log", a_log), ("D", d_skip)):
        _need(t, name, torch.float32, 1)
        if t.numel() != heads:
            raise KernelError(f"ssm_scan: {name} has {t.numel()} entries for {heads} heads")
    y = torch.empty((T, heads * vdim), dtype=torch.float32, device=xbc.device)
    _call("recurrent", "qwb_ssm_scan", _ptr(xbc), _i(xbc.shape[1]), ctypes.c_void_p(dt.data_ptr() + 4 * dt_col0),
          _i(dt.shape[1]), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), _ptr(ctx.cu_seqlens), _ptr(ctx.slots),
          _ptr(y), _i(ctx.n_seqs), _i(heads), _i(vdim), _i(n_state), _i(groups), _i(1 if write_state else 0), _stream())
    return y


def delta_rule(qkv: torch.Tensor, b_raw: torch.Tensor, b_col0: int, a_raw: torch.Tensor, dt_bias, a_log,
               state: torch.Tensor, ctx, heads: int, key_heads: int, key_dim: int, vdim: int, unit_eps: float,
               q_scale: float, write_state: bool = True, per_head: bool = False, a_col0: int = 0) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel, over a step's tokens.  ``qkv`` float32
    [T, 2 * key_heads * key_dim + heads * vdim] (q | k | v after convolution and SiLU; q and k are made unit vectors
    in place, q times ``q_scale``); columns ``b_col0 .. b_col0 + heads`` of ``b_raw`` [T, ld] and ``a_raw``
    [T, heads * key_dim] are the raw write strengths and decays; ``state`` float32 [slots, heads, vdim, key_dim] (column by column).  Returns o float32 [T, heads * vdim].
    ``per_head``: one decay per head instead: the raw decays are columns ``a_col0 .. a_col0 + heads`` of ``a_raw`` [T, ld],
    ``dt_bias`` has ``heads`` entries."""
    _need(qkv, "qkv", torch.float32, 2)
    _need(b_raw, "b_raw", torch.float32, 2)
    _need(a_raw, "a_raw", torch.float32, 2)
    _need(state, "state", torch.float32, 4)
    _need(dt_bias, "dt_bias", torch.float32, 1)
    _need(a_log, "A_log", torch.float32, 1)
    T = qkv.shape[0]
    decay_k = 1 if per_head else key_dim
    if (qkv.shape[1] != 2 * key_heads * key_dim + heads * vdim or b_raw.shape[0] != T or b_col0 + heads > b_raw.shape[1]
            or a_raw.shape[0] != T or a_col0 < 0 or a_col0 + heads * decay_k > a_raw.shape[1]
            or (not per_head and a_raw.shape[1] != heads * key_dim) or tuple(state.shape[1:]) != (heads, vdim, key_dim)
            or dt_bias.numel() != heads * decay_k or a_log.numel() != heads):
        raise KernelError(f"delta_rule: qkv {tuple(qkv.shape)}, b {tuple(b_raw.shape)}, a {tuple(a_raw.shape)}, state "
                          f"{tuple(state.shape)} do not fit {heads} heads ({key_heads} key heads) of {key_dim} x {vdim}")
    dev = qkv.device
    kq = torch.empty((T, key_heads), dtype=torch.float32, device=dev)
    beta = torch.empty((T, heads), dtype=torch.float32, device=dev)
    decay = torch.empty((T, heads * decay_k), dtype=torch.float32, device=dev)
    _call("recurrent", "qwb_delta_prep", _ptr(qkv), _i(qkv.shape[1]), _ptr(kq), ctypes.c_void_p(b_raw.data_ptr() + 4 * b_col0),
          _i(b_raw.shape[1]), _ptr(beta), ctypes.c_void_p(a_raw.data_ptr() + 4 * a_col0), _i(a_raw.shape[1]),
          _ptr(dt_bias), _ptr(a_log), _ptr(decay), _i(T), _i(heads), _i(key_heads), _i(key_dim), _i(decay_k), _f(unit_eps),
          _f(q_scale), _stream())
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=dev)
    _call("recurrent", "qwb_delta_scan", _ptr(qkv), _i(qkv.shape[1]), _ptr(kq), _ptr(beta), _ptr(decay), _ptr(state),
          _ptr(ctx.cu_seqlens), _ptr(ctx.slots), _ptr(o), _i(ctx.n_seqs), _i(heads), _i(key_heads), _i(key_dim), _i(vdim),
          _i(1 if write_state else 0), _i(heads * decay_k), _i(decay_k), _stream())
    return o


RETENTION_CHUNK = 64            # tokens per chunk of the chunked form of retention (csrc/recurrent.cu: QWB_CHUNK) ...
RETENTION_CHUNKED_FROM = 128    # ... which steps whose longest sequence brings at least this many tokens take


def retention_chunked_fits(key_dim: int, vdim: int) -> bool:
    """Whether the chunked form takes a state of key_dim x vdim per head (its tiles must fit in shared memory)."""
    return bool(_lookup("recurrent", "qwb_retention_chunked_fits")[1](_i(key_dim), _i(vdim)))


def retention_scan(qkv: torch.Tensor, cos, sin, rotary_dim: int, decay: torch.Tensor, state: torch.Tensor, ctx, heads: int,
                   key_dim: int, vdim: int, q_scale: float, k_scale: float, write_state: bool = True,
                   chunked: bool | None = None) -> torch.Tensor:
    """Linear attention with a fixed decay per head over a step's tokens: per head S = decay_h S + k v^T, o = S^T q.
    ``qkv`` float32 [T, ld] whose first 2 * heads * key_dim + heads * vdim columns are q | k | v; the first
    ``rotary_dim`` values of every head of q and k are turned by the tokens' angles (``cos``, ``sin`` float32
    [T, rotary_dim / 2]; value i with value i + rotary_dim / 2), then q is multiplied by ``q_scale`` and k by ``k_scale``,
    in place.  ``decay`` float32 [heads]; ``state`` float32 [slots, heads, vdim, key_dim] (column by column) is read and
    written back.  Returns o float32 [T, heads * vdim].  The recurrence is the delta rule's kernel without its correction
    term; steps that bring long prompts (``chunked`` None: from ``RETENTION_CHUNKED_FROM`` tokens on) take the chunked
    form instead, where its sizes fit."""
    _need(qkv, "qkv", torch.float32, 2)
    _need(state, "state", torch.float32, 4)
    _need(decay, "decay", torch.float32, 1)
    T = qkv.shape[0]
    if (qkv.shape[1] < heads * (2 * key_dim + vdim) or decay.numel() != heads
            or tuple(state.shape[1:]) != (heads, vdim, key_dim)):
        raise KernelError(f"retention_scan: qkv {tuple(qkv.shape)}, {decay.numel()} decays, state {tuple(state.shape)} do not "
                          f"fit {heads} heads of {key_dim} x {vdim}")
    if cos is None:
        rotary_dim = 0
    for name, t in (("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32, 2)
            if tuple(t.shape) != (T, rotary_dim // 2):
                raise KernelError(f"retention_scan: table {name} {tuple(t.shape)} for {T} tokens and {rotary_dim} turned values")
    dev = qkv.device
    kq = torch.empty((T, heads), dtype=torch.float32, device=dev)
    _call("recurrent", "qwb_turn_qk_prep", _ptr(qkv), _i(qkv.shape[1]), _ptr(kq), _ptr(cos), _ptr(sin), _i(T), _i(heads),
          _i(key_dim), _i(rotary_dim), _f(q_scale), _f(k_scale), _stream())
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=dev)
    if chunked is None:
        chunked = ctx.max_new >= RETENTION_CHUNKED_FROM
    if chunked and qkv.shape[1] % 4 == 0 and retention_chunked_fits(key_dim, vdim):
        # long prompts: chunks of 64 tokens side by side (three kernels) instead of a chain through every token
        n_chunks = -(-ctx.max_new // RETENTION_CHUNK)
        scratch = torch.empty((2, ctx.n_seqs * n_chunks, heads, vdim, key_dim), dtype=torch.float32, device=dev)
        _call("recurrent", "qwb_retention_chunked", _ptr(qkv), _i(qkv.shape[1]), _ptr(decay), _ptr(state), _ptr(ctx.cu_seqlens),
              _ptr(ctx.slots), _ptr(scratch), _ptr(o), _i(ctx.n_seqs), _i(ctx.max_new), _i(heads), _i(key_dim), _i(vdim),
              _i(1 if write_state else 0), _stream(), kernels=3)
        return o
    _call("recurrent", "qwb_delta_scan", _ptr(qkv), _i(qkv.shape[1]), _ptr(kq), _ptr(None), _ptr(decay), _ptr(state),
          _ptr(ctx.cu_seqlens), _ptr(ctx.slots), _ptr(o), _i(ctx.n_seqs), _i(heads), _i(heads), _i(key_dim), _i(vdim),
          _i(1 if write_state else 0), _i(0), _i(1), _stream())
    return o


def gla_scan(qkv: torch.Tensor, a_raw: torch.Tensor, a_bias: torch.Tensor | None, state: torch.Tensor, ctx, heads: int,
             key_dim: int, vdim: int, q_scale: float, tau: float, write_state: bool = True) -> torch.Tensor:
    """Gated linear attention over a step's tokens: per head S = diag(decay) S + k v^T, o = S^T (q * q_scale), with one
    decay per head and key channel, decay = sigmoid(a_raw + a_bias)^(1 / tau).  ``qkv`` float32 [T, ld] whose first
    2 * heads * key_dim + heads * vdim columns are q | k | v (q is scaled in place; further columns are left alone);
    ``a_raw`` float32 [T, heads * key_dim]; ``state`` float32 [slots, heads, vdim, key_dim] (column by column) is read and
    written back.  Returns o float32 [T, heads * vdim].  The recurrence is the delta rule's kernel without its correction
    term."""
    _need(qkv, "qkv", torch.float32, 2)
    _need(a_raw, "a_raw", torch.float32, 2)
    _need(state, "state", torch.float32, 4)
    T = qkv.shape[0]
    if (qkv.shape[1] < heads * (2 * key_dim + vdim) or tuple(a_raw.shape) != (T, heads * key_dim)
            or tuple(state.shape[1:]) != (heads, vdim, key_dim)):
        raise KernelError(f"gla_scan: qkv {tuple(qkv.shape)}, a {tuple(a_raw.shape)}, state {tuple(state.shape)} do not fit "
                          f"{heads} heads of {key_dim} x {vdim}")
    if a_bias is not None:
        _need(a_bias, "a_bias", torch.float32, 1)
        if a_bias.numel() != heads * key_dim:
            raise KernelError(f"gla_scan: a bias of {a_bias.numel()} for {heads} heads of {key_dim}")
    dev = qkv.device
    kq = torch.empty((T, heads), dtype=torch.float32, device=dev)
    decay = torch.empty((T, heads * key_dim), dtype=torch.float32, device=dev)
    _call("recurrent", "qwb_gla_prep", _ptr(qkv), _i(qkv.shape[1]), _ptr(kq), _ptr(a_raw), _ptr(a_bias), _ptr(decay), _i(T),
          _i(heads), _i(key_dim), _f(q_scale), _f(tau), _stream())
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=dev)
    _call("recurrent", "qwb_delta_scan", _ptr(qkv), _i(qkv.shape[1]), _ptr(kq), _ptr(None), _ptr(decay), _ptr(state),
          _ptr(ctx.cu_seqlens), _ptr(ctx.slots), _ptr(o), _i(ctx.n_seqs), _i(heads), _i(heads), _i(key_dim), _i(vdim),
          _i(1 if write_state else 0), _i(heads * key_dim), _i(key_dim), _stream())
    return o


def gated_part_norm(y: torch.Tensor, gate: torch.Tensor, gate_col0: int, weight: torch.Tensor, n_parts: int, eps: float,
                    gate_first: bool, out_dtype: torch.dtype, gate_activation: str = "sigmoid") -> torch.Tensor:
    """RMS norm over ``n_parts`` equal parts of every row of float32 ``y`` [T, D], with a gate from columns
    ``gate_col0 ..`` of float32 ``gate`` [T, ld].  ``gate_first``: y * silu(gate) is normed, times the weight; else y is
    normed, times the weight, times sigmoid(gate) (or silu(gate): ``gate_activation`` "silu").  ``weight`` has D entries,
    or D / n_parts shared by all parts."""
    if gate_activation not in ("sigmoid", "silu"):
        raise KernelError(f"gated_part_norm: unknown gate activation '{gate_activation}'")
    _need(y, "y", torch.float32, 2)
    _need(gate, "gate", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    T, D = y.shape
    if D % n_parts or weight.numel() not in (D, D // n_parts) or gate_col0 + D > gate.shape[1] or gate.shape[0] != T:
        raise KernelError(f"gated_part_norm: y {tuple(y.shape)} in {n_parts} parts, weight of {weight.numel()}, gate "
                          f"{tuple(gate.shape)} from column {gate_col0}")
    out = torch.empty((T, D), dtype=out_dtype, device=y.device)
    _call("recurrent", "qwb_gated_part_norm", _ptr(y), ctypes.c_void_p(gate.data_ptr() + 4 * gate_col0), _i(gate.shape[1]),
          _ptr(weight), _i(weight.numel()), _ptr(out), _i(_dt(out_dtype)), _i(T), _i(n_parts), _i(D // n_parts), _f(eps),
          _i(0 if gate_first else (2 if gate_activation == "silu" else 1)), _stream())
    return out


# ----------------------------------------------------------------------------- real-gated linear recurrent unit
RGLRU_CHUNK = 64            # tokens per chunk of the three-pass scan ...
RGLRU_CHUNKED_FROM = 256    # ... which steps whose longest sequence brings at least this many tokens take


def block_gates(u: torch.Tensor, w_a: torch.Tensor, b_a: torch.Tensor, w_i: torch.Tensor, b_i: torch.Tensor):
    """Two gates from block-diagonal matrices: float32 ``u`` [T, C] is cut into ``blocks`` equal parts, part b goes through
    ``w_a[b]`` / ``w_i[b]`` ([blocks, n, n], stored [out, in], float32 or bfloat16; multiplied in float) plus the biases
    [blocks, n] (float32), then sigmoid.  Returns (r, i), float32 [T, C]."""
    _need(u, "u", torch.float32, 2)
    T, C = u.shape
    blocks = w_a.shape[0]
    n = C // blocks if blocks else 0
    for name, w, b in (("w_a", w_a, b_a), ("w_i", w_i, b_i)):
        _need(w, name, w_a.dtype, 3)
        _need(b, name + " bias", torch.float32)
        if blocks * n != C or tuple(w.shape) != (blocks, n, n) or b.numel() != C:
            raise KernelError(f"block_gates: {name} {tuple(w.shape)} with bias of {b.numel()} for {C} channels")
    r = torch.empty((T, C), dtype=torch.float32, device=u.device)
    i = torch.empty_like(r)
    _call("rglru", "qwb_block_gates", _ptr(u), _ptr(w_a), _ptr(b_a), _ptr(w_i), _ptr(b_i), _ptr(r), _ptr(i), _i(_dt(w_a.dtype)),
          _i(T), _i(C), _i(blocks), _stream())
    return r, i


def rglru_scan(u: torch.Tensor, r: torch.Tensor, i: torch.Tensor, lam: torch.Tensor, y: torch.Tensor, y_col0: int,
               y_bias: torch.Tensor | None, state: torch.Tensor, ctx, sharpness: float, out_dtype: torch.dtype,
               write_state: bool = True) -> torch.Tensor:
    """The real-gated linear recurrence over a step's tokens, per channel: a = exp(-sharpness * r * softplus(lam)),
    S = a S + sqrt(1 - a^2) * i * u, read out as S * gelu_tanh(y + y_bias).  ``u``, ``r``, ``i`` float32 [T, C]; the
    second branch is columns ``y_col0 .. y_col0 + C`` of float32 ``y`` [T, ld]; ``state`` float32 [slots, C] is read and
    written back.  Returns [T, C] in ``out_dtype``.  Long prompts go in chunks (three passes), everything else in order."""
    for name, t in (("u", u), ("r", r), ("i", i)):
        _need(t, name, torch.float32, 2)
    _need(y, "y", torch.float32, 2)
    _need(lam, "lam", torch.float32, 1)
    _need(state, "state", torch.float32, 2)
    T, C = u.shape
    if r.shape != u.shape or i.shape != u.shape or lam.numel() != C or state.shape[1] != C or y.shape[0] != T or y_col0 + C > y.shape[1]:
        raise KernelError(f"rglru_scan: u {tuple(u.shape)}, r {tuple(r.shape)}, i {tuple(i.shape)}, lam of {lam.numel()}, state "
                          f"{tuple(state.shape)}, y {tuple(y.shape)} from column {y_col0}")
    if y_bias is not None:
        _need(y_bias, "y_bias", torch.float32, 1)
    out = torch.empty((T, C), dtype=out_dtype, device=u.device)
    chunk = max_chunks = 0
    tables = scratch = None
    if ctx.max_new >= RGLRU_CHUNKED_FROM:
        chunk = RGLRU_CHUNK
        max_chunks = -(-T // chunk) + ctx.n_seqs
        tables = torch.empty((2 * max_chunks + ctx.n_seqs + 1,), dtype=torch.int32, device=u.device)
        scratch = torch.empty((2 * max_chunks * C,), dtype=torch.float32, device=u.device)
    _call("rglru", "qwb_rglru_scan", _ptr(u), _ptr(r), _ptr(i), _ptr(lam), ctypes.c_void_p(y.data_ptr() + 4 * y_col0),
          _i(y.shape[1]), _ptr(y_bias), _ptr(state), _ptr(ctx.cu_seqlens), _ptr(ctx.slots), _ptr(out), _i(_dt(out_dtype)),
          _i(ctx.n_seqs), _i(C), _f(sharpness), _i(1 if write_state else 0), _i(chunk), _i(max_chunks), _ptr(tables),
          _ptr(scratch), _stream(), kernels=4 if chunk else 1)
    return out


# ----------------------------------------------------------------------------- window + pooled blocks attention
POOL_MAX_DIM = 256          # csrc/attention_pool.cu: QWB_POOL_MAX_DIM


def pool_prep(qkv: torch.Tensor, q_weight, k_weight, cos_qk, sin_qk, cos_v, sin_v, ctx, page_table, k_pool, v_pool,
              n_heads: int, n_kv_heads: int, dim: int, vdim: int, rotary_dim: int, interleaved: bool, eps: float,
              store_kv: bool = True) -> torch.Tensor:
    """Per-head RMS norm of q and k (weights [dim] shared by the heads, or None), rotation of their first ``rotary_dim``
    values, rotation of every value by its own position (``cos_v`` given), cache write.  ``qkv`` float32
    [T, (H + G) * dim + G * vdim]; the pools [pages, G, 64, dim] / [pages, G, 64, vdim].  Returns q [T, H, dim] in the
    cache's dtype."""
    _need(qkv, "qkv", torch.float32, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + n_kv_heads) * dim + n_kv_heads * vdim:
        raise KernelError(f"pool_prep: qkv {tuple(qkv.shape)} for {n_heads}+{n_kv_heads} heads of {dim}, values of {vdim}")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_SIZE, dim) or tuple(v_pool.shape[1:]) != (n_kv_heads, PAGE_SIZE, vdim):
        raise KernelError(f"pool_prep: pools {tuple(k_pool.shape)}, {tuple(v_pool.shape)} do not fit")
    for name, t, n in (("q_weight", q_weight, dim), ("k_weight", k_weight, dim)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != n:
                raise KernelError(f"pool_prep: {name} of {t.numel()} for heads of {n}")
    for name, t, n in (("cos_qk", cos_qk, rotary_dim), ("sin_qk", sin_qk, rotary_dim), ("cos_v", cos_v, vdim), ("sin_v", sin_v, vdim)):
        if t is not None:
            _need(t, name, torch.float32, 2)
            if tuple(t.shape) != (T, n // 2):
                raise KernelError(f"pool_prep: table {name} {tuple(t.shape)} for {T} tokens and {n} turned values")
    q = torch.empty((T, n_heads, dim), dtype=k_pool.dtype, device=qkv.device)
    _call("attention_pool", "qwb_pool_prep", _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos_qk), _ptr(sin_qk), _ptr(cos_v),
          _ptr(sin_v), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(page_table), _i(page_table.shape[1]), _ptr(q), _ptr(k_pool),
          _ptr(v_pool), _i(_dt(k_pool.dtype)), _i(T), _i(n_heads), _i(n_kv_heads), _i(dim), _i(vdim),
          _i(rotary_dim if cos_qk is not None else 0), _i(1 if interleaved else 0), _i(1 if cos_v is not None else 0), _f(eps),
          _i(1 if store_kv else 0), _stream())
    return q


def pool_update(k_pool, v_pool, pk_pool, pv_pool, page_table, block_table, ctx, pool: int) -> None:
    """The block rows (means of ``pool`` consecutive cached keys and values) of the blocks that this step completes."""
    G, dim, vdim = k_pool.shape[1], k_pool.shape[3], v_pool.shape[3]
    max_blocks = ctx.max_new // pool + 1
    _call("attention_pool", "qwb_pool_update", _ptr(k_pool), _ptr(v_pool), _ptr(pk_pool), _ptr(pv_pool), _ptr(page_table),
          _ptr(block_table), _i(page_table.shape[1]), _ptr(ctx.pos0), _ptr(ctx.seq_len), _i(_dt(k_pool.dtype)), _i(ctx.n_seqs),
          _i(max_blocks), _i(G), _i(dim), _i(vdim), _i(pool), _stream())


def pool_prefill_mma_fits(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether prompts take the tensor-core kernel: bfloat16, keys in multiples of 16, values of 8, tiles that fit."""
    if dtype != torch.bfloat16:
        return False
    return bool(_lookup("attention_pool", "qwb_pool_prefill_mma_fits")[1](_i(DT_BF16), _i(dim), _i(vdim)))


def pool_attention(q: torch.Tensor, k_pool, v_pool, pk_pool, pv_pool, page_table, block_table, ctx, cos_v, sin_v,
                   scale: float, window: int, pool: int, interleaved: bool, impl: str = "auto") -> torch.Tensor:
    """Attention of a step's tokens over their window and the block rows before it.  ``q`` [T, H, dim] in the cache's
    dtype; returns [T, H * vdim] in that dtype, each head turned back by the query's position if ``cos_v`` is given.
    Steps of one token per sequence take the kernel that cuts the keys into runs (sizes that are multiples of 8); other
    steps the tensor-core kernel where it fits (``impl`` "auto" or "mma"), else the plain one ("plain")."""
    _need(q, "q", k_pool.dtype, 3)
    T, H, dim = q.shape
    G, vdim = k_pool.shape[1], v_pool.shape[3]
    out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    width = page_table.shape[1]
    if block_table is not None and block_table.shape[1] != width:
        raise KernelError("pool_attention: the two page tables differ in width")
    if ctx.single_token:
        lib = _lookup("attention_pool", "qwb_pool_decode_runs")[0]
        block_runs = ctypes.c_int(0)
        n_runs = lib.qwb_pool_decode_runs(_i(ctx.max_len), _i(window), _i(pool), ctypes.byref(block_runs))
        lib.qwb_pool_decode_scratch_floats.restype = ctypes.c_longlong
        scratch = torch.empty((lib.qwb_pool_decode_scratch_floats(_i(T), _i(H), _i(vdim), _i(n_runs)),), dtype=torch.float32,
                              device=q.device)
        _call("attention_pool", "qwb_pool_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(pk_pool), _ptr(pv_pool),
              _ptr(page_table), _ptr(block_table), _ptr(ctx.seq_len), _ptr(cos_v), _ptr(sin_v), _ptr(scratch), _ptr(out),
              _i(_dt(q.dtype)), _i(T), _i(H), _i(G), _i(dim), _i(vdim), _i(width), _f(scale), _i(window), _i(pool),
              _i(block_runs.value), _i(n_runs), _i(1 if interleaved else 0), _stream(), kernels=2)
        return out
    if impl == "mma" or (impl == "auto" and pool_prefill_mma_fits(q.dtype, dim, vdim)):
        _call("attention_pool", "qwb_pool_prefill_mma", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(pk_pool), _ptr(pv_pool),
              _ptr(page_table), _ptr(block_table), _ptr(ctx.cu_seqlens), _ptr(ctx.pos0), _ptr(cos_v), _ptr(sin_v), _ptr(out),
              _i(ctx.n_seqs), _i(ctx.max_new), _i(H), _i(G), _i(dim), _i(vdim), _i(width), _f(scale), _i(window), _i(pool),
              _i(1 if interleaved else 0), _stream())
        return out
    _call("attention_pool", "qwb_pool_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(pk_pool), _ptr(pv_pool), _ptr(page_table),
          _ptr(block_table), _ptr(ctx.cu_seqlens), _ptr(ctx.pos0), _ptr(cos_v), _ptr(sin_v), _ptr(out), _i(_dt(q.dtype)),
          _i(ctx.n_seqs), _i(ctx.max_new), _i(H), _i(G), _i(dim), _i(vdim), _i(width), _f(scale), _i(window), _i(pool),
          _i(1 if interleaved else 0), _stream())
    return out


# ----------------------------------------------------------------------------- attention with score maps
MAPS_MAX_DIM = 256          # csrc/attention_maps.cu: QWB_MAPS_MAX_DIM
MAPS_MAX = 2                # ... QWB_MAPS_MAX: score maps per head
MAPS_PREFILL_MMA = True     # bfloat16 prompts take the tensor-core kernel where it fits; False: always the plain one
MAPS_FAST_STEP = 8          # key and value sizes that are multiples of this take the kernels that copy 16 bytes at a time


def maps_prep(qkv: torch.Tensor, bias, q_weight, k_weight, cos, sin, ctx, page_table, k_pool, v_pool, n_heads: int,
              n_kv_heads: int, maps: int, dim: int, vdim: int, rotary_dim: int, interleaved: bool, eps: float,
              store_kv: bool = True) -> torch.Tensor:
    """Bias (float32 over all columns, or None), per-map RMS norm of q and k (weights [dim] shared by heads and maps, or
    None), rotation of the first ``rotary_dim`` values of every map of q and k, cache write.  ``qkv`` float32
    [T, (H + G) * maps * dim + G * vdim]; the pools [pages, G, 64, maps * dim] / [pages, G, 64, vdim].  Returns q
    [T, H, maps * dim] in the cache's dtype."""
    _need(qkv, "qkv", torch.float32, 2)
    T = qkv.shape[0]
    ld = (n_heads + n_kv_heads) * maps * dim + n_kv_heads * vdim
    if qkv.shape[1] != ld:
        raise KernelError(f"maps_prep: qkv {tuple(qkv.shape)} for {n_heads}+{n_kv_heads} heads of {maps} x {dim}, values of {vdim}")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_SIZE, maps * dim) or tuple(v_pool.shape[1:]) != (n_kv_heads, PAGE_SIZE, vdim):
        raise KernelError(f"maps_prep: pools {tuple(k_pool.shape)}, {tuple(v_pool.shape)} do not fit")
    for name, t, n in (("bias", bias, ld), ("q_weight", q_weight, dim), ("k_weight", k_weight, dim)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != n:
                raise KernelError(f"maps_prep: {name} of {t.numel()}, wanted {n}")
    if cos is None:
        rotary_dim = 0
    for name, t in (("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32, 2)
            if tuple(t.shape) != (T, rotary_dim // 2):
                raise KernelError(f"maps_prep: table {name} {tuple(t.shape)} for {T} tokens and {rotary_dim} turned values")
    q = torch.empty((T, n_heads, maps * dim), dtype=k_pool.dtype, device=qkv.device)
    _call("attention_maps", "qwb_maps_prep", _ptr(qkv), _ptr(bias), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
          _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(page_table), _i(page_table.shape[1]), _ptr(q), _ptr(k_pool), _ptr(v_pool),
          _i(_dt(k_pool.dtype)), _i(T), _i(n_heads), _i(n_kv_heads), _i(maps), _i(dim), _i(vdim), _i(rotary_dim),
          _i(1 if interleaved else 0), _f(eps), _i(1 if store_kv else 0), _stream())
    return q


def maps_prefill_mma_fits(dtype: torch.dtype, maps: int, dim: int, vdim: int) -> bool:
    """Whether prompts take the tensor-core kernel: bfloat16, keys in multiples of 16, values of 8, tiles that fit."""
    if dtype != torch.bfloat16 or not MAPS_PREFILL_MMA:
        return False
    return bool(_lookup("attention_maps", "qwb_maps_prefill_mma_fits")[1](_i(DT_BF16), _i(maps), _i(dim), _i(vdim)))


def maps_attention(q: torch.Tensor, k_pool, v_pool, page_table, ctx, maps: int, scale: float, softcap: float = 0.0,
                   chunk: int = 0, lam: float = 0.0, norm_out: bool = False, eps: float = 0.0, out_scale: float = 1.0,
                   impl: str = "auto") -> torch.Tensor:
    """Attention of a step's tokens with ``maps`` score maps per head over the same values.  ``q`` [T, H, maps * dim] in
    the cache's dtype; returns [T, H * vdim] in that dtype: map 0's output, minus ``lam`` times map 1's if there are two,
    then (``norm_out``) divided by its root mean square over vdim and multiplied by ``out_scale``.  Scores are scaled,
    soft-capped (``softcap`` > 0) and masked causally, and to the query's chunk of ``chunk`` positions if that is > 0.
    Steps of one token per sequence take the kernel that cuts the keys into runs (sizes that are multiples of 8); other
    steps the tensor-core kernels where they fit (``impl`` "auto"; "tc": tcgen05, for one uncapped map with keys and values
    of 64 or 128; "mma": mma.sync), else the plain one ("plain")."""
    _need(q, "q", k_pool.dtype, 3)
    T, H, kdim = q.shape
    G, vdim = k_pool.shape[1], v_pool.shape[3]
    if kdim % maps or k_pool.shape[3] != kdim:
        raise KernelError(f"maps_attention: q {tuple(q.shape)} and keys {tuple(k_pool.shape)} with {maps} maps")
    dim = kdim // maps
    out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    width = page_table.shape[1]
    if ctx.single_token and dim % MAPS_FAST_STEP == 0 and vdim % MAPS_FAST_STEP == 0:
        lib = _lookup("attention_maps", "qwb_maps_decode_runs")[0]
        n_runs = lib.qwb_maps_decode_runs(_i(ctx.max_len), _i(chunk))
        lib.qwb_maps_decode_scratch_floats.restype = ctypes.c_longlong
        scratch = torch.empty((lib.qwb_maps_decode_scratch_floats(_i(T), _i(H), _i(maps), _i(vdim), _i(n_runs)),),
                              dtype=torch.float32, device=q.device)
        _call("attention_maps", "qwb_maps_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.seq_len),
              _ptr(scratch), _ptr(out), _i(_dt(q.dtype)), _i(T), _i(H), _i(G), _i(maps), _i(dim), _i(vdim), _i(width), _f(scale),
              _f(softcap), _i(chunk), _i(n_runs), _f(lam), _i(1 if norm_out else 0), _f(eps), _f(out_scale), _stream(), kernels=2)
        return out
    # one map, no cap, keys and values of one size: the prompt kernel of plain grouped-query attention, with the chunk mask
    if (impl in ("auto", "tc") and maps == 1 and softcap <= 0.0 and dim == vdim and q.dtype == torch.bfloat16
            and ctx.max_new * (H // G) >= 64 and tc_attention_fits(q.dtype, dim, k_pool.shape[2], H // G)):
        return attn_prefill(q, k_pool, v_pool, page_table, ctx.cu_seqlens, ctx.pos0, ctx.max_new, scale, impl="tc", chunk=chunk)
    if impl == "mma" or (impl == "auto" and maps_prefill_mma_fits(q.dtype, maps, dim, vdim)):
        _call("attention_maps", "qwb_maps_prefill_mma", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.cu_seqlens),
              _ptr(ctx.pos0), _ptr(out), _i(ctx.n_seqs), _i(ctx.max_new), _i(H), _i(G), _i(maps), _i(dim), _i(vdim), _i(width),
              _f(scale), _f(softcap), _i(chunk), _f(lam), _i(1 if norm_out else 0), _f(eps), _f(out_scale), _stream())
        return out
    _call("attention_maps", "qwb_maps_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.cu_seqlens),
          _ptr(ctx.pos0), _ptr(out), _i(_dt(q.dtype)), _i(ctx.n_seqs), _i(ctx.max_new), _i(H), _i(G), _i(maps), _i(dim), _i(vdim),
          _i(width), _f(scale), _f(softcap), _i(chunk), _f(lam), _i(1 if norm_out else 0), _f(eps), _f(out_scale), _stream())
    return out


# ----------------------------------------------------------------------------- attention with shaped scores
BIAS_ATTN_MAX_DIM = 256     # csrc/attention_bias.cu: QWB_BIAS_MAX_DIM
BIAS_ATTN_FAST_STEP = 8     # key and value sizes that are multiples of this take the kernels that copy 16 bytes at a time
BIAS_PREFILL_MMA = True     # bfloat16 prompts take the tensor-core kernel where it fits; False: always the plain one
BIAS_MMA_MIN_NEW = 16       # ... from this many new tokens of the longest sequence on (a tile is 64 queries)
BIAS_DECODE_TWO_PASS = True # single tokens with mixed heads take the two-pass kernels where they fit (False: all value heads) ...
BIAS_TWO_PASS_FROM_KEYS = 24576     # ... from this many keys in the step (sequences x the bound on their lengths): below, the
                                    # form with all value heads has 16 times the blocks and one kernel less, and is faster
                                    # (8 sequences of 1,024 tokens: 0.495 against 0.515 ms a step; one: 0.391 against 0.460)


def bias_prefill_mma_fits(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether prompts take the tensor-core kernel: bfloat16, keys in multiples of 16, values of 8, tiles that fit."""
    if dtype != torch.bfloat16 or not BIAS_PREFILL_MMA:
        return False
    return bool(_lookup("attention_bias", "qwb_bias_prefill_mma_fits")[1](_i(DT_BF16), _i(dim), _i(vdim)))


def bias_prep(qkv: torch.Tensor, bias, q_weight, k_weight, cos, sin, ctx, page_table, k_pool, v_pool, n_heads: int,
              n_kv_heads: int, dim: int, vdim: int, rotary_dim: int, interleaved: bool, eps: float, store_kv: bool = True,
              values_are_keys: bool = False) -> torch.Tensor:
    """Bias (float32 over all columns, or None), per-head RMS norm of q and k (weights [dim] shared by the heads, or None),
    rotation of the first ``rotary_dim`` values of every head of q and k, cache write.  ``qkv`` float32 [T, ld]: its
    first (H + G) * dim + G * vdim columns, or (H + G) * dim with ``values_are_keys``: the cached value of a token is then
    the raw output of its key projection (with the bias): what the key was ahead of its norm and its turn.  The pools [pages, G, 64, dim] / [pages, G, 64, vdim].
    Returns q [T, H, dim] in the cache's dtype."""
    _need(qkv, "qkv", torch.float32, 2)
    T = qkv.shape[0]
    ld = (n_heads + n_kv_heads) * dim + (0 if values_are_keys else n_kv_heads * vdim)
    if qkv.shape[1] < ld:
        raise KernelError(f"bias_prep: qkv {tuple(qkv.shape)} for {n_heads}+{n_kv_heads} heads of {dim}, values of {vdim}")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_SIZE, dim) or tuple(v_pool.shape[1:]) != (n_kv_heads, PAGE_SIZE, vdim):
        raise KernelError(f"bias_prep: pools {tuple(k_pool.shape)}, {tuple(v_pool.shape)} do not fit")
    for name, t, n in (("bias", bias, ld), ("q_weight", q_weight, dim), ("k_weight", k_weight, dim)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != n:
                raise KernelError(f"bias_prep: {name} of {t.numel()}, wanted {n}")
    if cos is None:
        rotary_dim = 0
    for name, t in (("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32, 2)
            if tuple(t.shape) != (T, rotary_dim // 2):
                raise KernelError(f"bias_prep: table {name} {tuple(t.shape)} for {T} tokens and {rotary_dim} turned values")
    q = torch.empty((T, n_heads, dim), dtype=k_pool.dtype, device=qkv.device)
    _call("attention_bias", "qwb_bias_prep", _ptr(qkv), _ptr(bias), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
          _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(page_table), _i(page_table.shape[1]), _ptr(q), _ptr(k_pool), _ptr(v_pool),
          _i(_dt(k_pool.dtype)), _i(T), _i(n_heads), _i(n_kv_heads), _i(dim), _i(vdim), _i(rotary_dim),
          _i(1 if interleaved else 0), _f(eps), _i(1 if store_kv else 0), _i(1 if values_are_keys else 0), _i(qkv.shape[1]), _stream())
    return q


def bias_tc_fits(q: torch.Tensor, n_kv_heads: int, vdim: int, head_scale, softcap: float, raw: bool) -> bool:
    """Whether a prompt's attention with shaped scores is what the tcgen05 prompt kernel computes: bfloat16, keys and
    values of one size that it takes, scores shaped by a distance bias, a window and a sink only."""
    T, H, dim = q.shape
    return (head_scale is None and softcap <= 0.0 and not raw and dim == vdim and q.dtype == torch.bfloat16
            and tc_attention_fits(q.dtype, dim, PAGE_SIZE, H // n_kv_heads))


def bias_attention(q: torch.Tensor, k_pool, v_pool, page_table, ctx, scale: float, head_scale=None, softcap: float = 0.0,
                   slopes=None, window: int = 0, sinks=None, head_mix=None, gate=None, gate_col0: int = 0,
                   impl: str = "auto") -> torch.Tensor:
    """Softmax attention of a step's tokens with scores shaped head by head.  ``q`` [T, H, dim] in the cache's dtype;
    returns [T, H * vdim] in that dtype.  score = q . k * ``scale`` * ``head_scale``[h]; capped (``softcap`` > 0:
    c tanh(s / c)); minus ``slopes``[h] times the key's distance from the query; causal, and within the last ``window``
    positions if that is > 0; ``sinks``[h]: one more term exp(sink) in the softmax's denominator.  ``head_mix`` [H, H]:
    the heads' weights are mixed after the softmax, w'_h = sum_g mix[h, g] w_g, each head still reading its own value
    head.  ``gate``: head h's output times sigmoid of column ``gate_col0 + h`` of the float32 matrix ``gate`` [T, ld].
    The per-head vectors are float32 [H].  Steps of one token per sequence take the kernel that cuts the keys into runs
    (sizes that are multiples of 8); other steps the tensor-core kernels where they fit (``impl`` "auto"; "tc": tcgen05,
    for scores shaped by a distance bias, a window and a sink only, keys and values of 64 or 128; "mma": mma.sync), else
    the plain prompt kernel ("plain")."""
    _need(q, "q", k_pool.dtype, 3)
    T, H, dim = q.shape
    G, vdim = k_pool.shape[1], v_pool.shape[3]
    if k_pool.shape[3] != dim or v_pool.shape[1] != G:
        raise KernelError(f"bias_attention: q {tuple(q.shape)}, keys {tuple(k_pool.shape)}, values {tuple(v_pool.shape)}")
    for name, t in (("head_scale", head_scale), ("slopes", slopes), ("sinks", sinks)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != H:
                raise KernelError(f"bias_attention: {name} of {t.numel()} for {H} heads")
    if head_mix is not None:
        _need(head_mix, "head_mix", torch.float32, 2)
        if tuple(head_mix.shape) != (H, H):
            raise KernelError(f"bias_attention: a mix {tuple(head_mix.shape)} for {H} heads")
    if gate is not None:
        _need(gate, "gate", torch.float32, 2)
        if gate.shape[0] != T or gate_col0 < 0 or gate_col0 + H > gate.shape[1]:
            raise KernelError(f"bias_attention: gate {tuple(gate.shape)} from column {gate_col0} for {T} tokens of {H} heads")
    width = page_table.shape[1]
    if (head_mix is not None and ctx.single_token and BIAS_DECODE_TWO_PASS and T * ctx.max_len >= BIAS_TWO_PASS_FROM_KEYS
            and _lookup("attention_bias", "qwb_bias_decode_mixed_fits")[1](_i(_dt(q.dtype)), _i(H), _i(G), _i(dim), _i(vdim))):
        # mixed heads, one token per sequence: every head's maximum and sum first, then all heads' final weights mixed in
        # shared memory and applied to their own value heads (keys twice, values once)
        lib = _lookup("attention_bias", "qwb_bias_decode_runs")[0]
        n_runs = lib.qwb_bias_decode_runs(_i(ctx.max_len), _i(window))
        lib.qwb_bias_decode_mixed_scratch_floats.restype = ctypes.c_longlong
        scratch = torch.empty((lib.qwb_bias_decode_mixed_scratch_floats(_i(T), _i(H), _i(vdim), _i(n_runs)),),
                              dtype=torch.float32, device=q.device)
        out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
        _call("attention_bias", "qwb_bias_decode_mixed", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.seq_len),
              _ptr(scratch), _ptr(out), _i(_dt(q.dtype)), _i(T), _i(H), _i(G), _i(dim), _i(vdim), _i(width), _f(scale),
              _ptr(head_scale), _f(softcap), _ptr(slopes), _i(window), _ptr(sinks), _ptr(head_mix),
              ctypes.c_void_p(gate.data_ptr() + 4 * gate_col0) if gate is not None else _ptr(None),
              _i(gate.shape[1] if gate is not None else 0), _i(n_runs), _stream(), kernels=4)
        return out
    all_values = head_mix is not None
    raw = all_values or gate is not None
    C = G if all_values else 1
    width = page_table.shape[1]
    dev = q.device
    att = torch.empty((T, H, C, vdim) if raw else (T, H * vdim), dtype=torch.float32 if raw else q.dtype, device=dev)
    if ctx.single_token and dim % BIAS_ATTN_FAST_STEP == 0 and vdim % BIAS_ATTN_FAST_STEP == 0:
        lib = _lookup("attention_bias", "qwb_bias_decode_runs")[0]
        n_runs = lib.qwb_bias_decode_runs(_i(ctx.max_len), _i(window))
        lib.qwb_bias_decode_scratch_floats.restype = ctypes.c_longlong
        scratch = torch.empty((lib.qwb_bias_decode_scratch_floats(_i(T), _i(H), _i(C), _i(vdim), _i(n_runs)),),
                              dtype=torch.float32, device=dev)
        _call("attention_bias", "qwb_bias_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.seq_len),
              _ptr(scratch), _ptr(att), _i(_dt(q.dtype)), _i(1 if raw else 0), _i(T), _i(H), _i(G), _i(1 if all_values else 0),
              _i(dim), _i(vdim), _i(width), _f(scale), _ptr(head_scale), _f(softcap), _ptr(slopes), _i(window), _ptr(sinks),
              _i(n_runs), _stream(), kernels=2)
    elif (impl in ("auto", "tc") and bias_tc_fits(q, G, vdim, head_scale, softcap, raw)
          and (impl == "tc" or ctx.max_new * (H // G) >= 64)):
        # no number per head, no cap, no mix, no gate, keys and values of 64 or 128: plain grouped-query attention whose
        # softmax takes the distance bias and the sink, on tcgen05
        return attn_prefill(q, k_pool, v_pool, page_table, ctx.cu_seqlens, ctx.pos0, ctx.max_new, scale, window=window, impl="tc",
                            slopes=slopes, sinks=sinks)
    elif impl == "mma" or (impl == "auto" and ctx.max_new >= BIAS_MMA_MIN_NEW and bias_prefill_mma_fits(q.dtype, dim, vdim)):
        _call("attention_bias", "qwb_bias_prefill_mma", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.cu_seqlens),
              _ptr(ctx.pos0), _ptr(att), _i(1 if raw else 0), _i(ctx.n_seqs), _i(ctx.max_new), _i(H), _i(G),
              _i(1 if all_values else 0), _i(dim), _i(vdim), _i(width), _f(scale), _ptr(head_scale), _f(softcap), _ptr(slopes),
              _i(window), _ptr(sinks), _stream())
    else:
        _call("attention_bias", "qwb_bias_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(ctx.cu_seqlens),
              _ptr(ctx.pos0), _ptr(att), _i(_dt(q.dtype)), _i(1 if raw else 0), _i(ctx.n_seqs), _i(ctx.max_new), _i(H), _i(G),
              _i(1 if all_values else 0), _i(dim), _i(vdim), _i(width), _f(scale), _ptr(head_scale), _f(softcap), _ptr(slopes),
              _i(window), _ptr(sinks), _stream())
    if not raw:
        return att
    out = torch.empty((T, H * vdim), dtype=q.dtype, device=dev)
    _call("attention_bias", "qwb_bias_head_mix", _ptr(att), _ptr(head_mix),
          ctypes.c_void_p(gate.data_ptr() + 4 * gate_col0) if gate is not None else _ptr(None),
          _i(gate.shape[1] if gate is not None else 0), _ptr(out), _i(_dt(q.dtype)), _i(T), _i(H), _i(G),
          _i(1 if all_values else 0), _i(vdim), _stream())
    return out


# ----------------------------------------------------------------------------- latent attention
LATENT_MAX_RANK = 512       # csrc/attention_latent.cu: QWB_LATENT_MAX_L
LATENT_MAX_ROW = 1024       # ... QWB_LATENT_MAX_ROW: latent + rotated key part
LATENT_RUN_KEYS = 64        # ... QWB_LATENT_RUN_KEYS: keys per block in a step of one token per sequence


def latent_prep(q: torch.Tensor, dkv: torch.Tensor, c_weight: torch.Tensor, cos, sin, ctx, page_table, pool,
                heads: int, dim: int, rot_dim: int, rank: int, eps: float, store: bool = True, whole_heads: bool = False):
    """Per token: the latent (``dkv[:, :rank]``, RMS-normed, times ``c_weight``) and the rotated shared key part
    (``dkv[:, rank:]``, pairs (2i, 2i + 1) turned by cos/sin [T, half]) go into the cache row of the token's position;
    each head's rotated query part is turned the same way.  ``q`` float32 [T, heads * (dim + rot_dim)].
    Returns (q_plain [heads, T, dim] in the pool's dtype, q_rot float32 [T, heads, rot_dim]); or, with ``whole_heads``
    (for the tensor-core prompt kernel), (q [T, heads, dim + rot_dim] with the rotated parts turned, the tokens' cache
    rows once more as [T, rank + rot_dim]), both in the pool's dtype."""
    _need(q, "q", torch.float32, 2)
    _need(dkv, "dkv", torch.float32, 2)
    _need(c_weight, "c_weight", torch.float32, 1)
    _need(pool, "pool", ndim=4)
    _need(page_table, "page_table", torch.int32, 2)
    T = q.shape[0]
    half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        half = cos.shape[1]
        if cos.shape[0] != T or sin.shape != cos.shape or 2 * half > rot_dim:
            raise KernelError(f"latent_prep: cos/sin {tuple(cos.shape)} do not fit {T} tokens and {rot_dim} rotated values")
    if (q.shape[1] != heads * (dim + rot_dim) or tuple(dkv.shape) != (T, rank + rot_dim) or c_weight.numel() != rank
            or pool.shape[1] != 1 or pool.shape[3] != rank + rot_dim):
        raise KernelError(f"latent_prep: q {tuple(q.shape)}, dkv {tuple(dkv.shape)}, pool {tuple(pool.shape)} do not fit "
                          f"{heads} heads of {dim} + {rot_dim}, latent {rank}")
    q_plain = q_rot = q_full = row_new = None
    if whole_heads:
        q_full = torch.empty((T, heads, dim + rot_dim), dtype=pool.dtype, device=q.device)
        row_new = torch.empty((T, rank + rot_dim), dtype=pool.dtype, device=q.device)
    else:
        q_plain = torch.empty((heads, T, dim), dtype=pool.dtype, device=q.device)
        q_rot = torch.empty((T, heads, rot_dim), dtype=torch.float32, device=q.device)
    _call("attention_latent", "qwb_latent_prep", _ptr(q), _ptr(dkv), _ptr(c_weight), _ptr(cos), _ptr(sin), _ptr(ctx.tok_seq),
          _ptr(ctx.tok_pos), _ptr(page_table), _ptr(pool), _i(_dt(pool.dtype)), _ptr(q_plain), _ptr(q_rot), _ptr(q_full),
          _ptr(row_new), _i(T), _i(heads), _i(dim), _i(rot_dim), _i(rank), _i(half), _f(eps), _i(pool.shape[2]),
          _i(page_table.shape[1]), _i(1 if store else 0), _stream())
    return (q_full, row_new) if whole_heads else (q_plain, q_rot)


def latent_prefill_fits(dtype: torch.dtype, dim: int, rot_dim: int, vdim: int, rank: int) -> bool:
    """Whether the tensor-core prompt kernel takes these head sizes (else the plain kernel does)."""
    tiles = (3 * 64 * (dim + rot_dim + 8) + 2 * 64 * (vdim + 8)) * 2       # bytes of shared memory: Q, two K, two V tiles
    return (dtype == torch.bfloat16 and dim % 8 == 0 and rot_dim % 8 == 0 and vdim % 8 == 0 and (dim + rot_dim) % 16 == 0
            and vdim <= 256 and rank % 8 == 0 and tiles <= 220 * 1024)


def latent_prefill(q: torch.Tensor, k_plain: torch.Tensor, rows: torch.Tensor, v: torch.Tensor, ctx, sink, scale: float,
                   window: int, heads: int, dim: int, rot_dim: int, vdim: int) -> torch.Tensor:
    """Attention of prompts that START their sequences (every position 0 is in this step), on the tensor cores.
    bfloat16: ``q`` [T, heads, dim + rot_dim]; ``k_plain`` [T, heads * dim] and ``v`` [T, heads * vdim], the keys' unrotated
    parts and the values made from the latents; ``rows`` [T, rank + rot_dim], whose last ``rot_dim`` values are the
    rotated key part that the heads share.  Returns [T, heads * vdim]."""
    for name, t in (("q", q), ("k_plain", k_plain), ("rows", rows), ("v", v)):
        _need(t, name, torch.bfloat16)
    T = q.shape[0]
    if (tuple(q.shape) != (T, heads, dim + rot_dim) or tuple(k_plain.shape) != (T, heads * dim) or tuple(v.shape) != (T, heads * vdim)
            or rows.shape[0] != T or rows.shape[1] < rot_dim):
        raise KernelError(f"latent_prefill: q {tuple(q.shape)}, k {tuple(k_plain.shape)}, rows {tuple(rows.shape)}, v {tuple(v.shape)}")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
    out = torch.empty((T, heads * vdim), dtype=torch.bfloat16, device=q.device)
    ld = rows.shape[1]
    _call("attention_latent_mma", "qwb_latent_prefill_mma", _ptr(q), _ptr(k_plain),
          ctypes.c_void_p(rows.data_ptr() + 2 * (ld - rot_dim)), _i(ld), _ptr(v), _ptr(ctx.cu_seqlens), _ptr(sink), _ptr(out),
          _i(ctx.n_seqs), _i(ctx.max_new), _i(heads), _i(dim), _i(rot_dim), _i(vdim), _f(scale), _i(window), _stream())
    return out


def latent_attention(q_abs: torch.Tensor, q_rot: torch.Tensor, pool: torch.Tensor, page_table, ctx, sink, scale: float,
                     window: int = 0) -> torch.Tensor:
    """Attention of every head over the shared cached rows [latent | rotated key part]; the values are the latents.
    ``q_abs`` float32 [heads, T, rank] (the queries taken into the latent space), ``q_rot`` float32 [T, heads, rot_dim];
    ``sink`` float32 [heads] or None: one more term exp(sink) in the softmax's denominator.  Causal; ``window`` > 0:
    a position sees itself and the window - 1 before it.  Returns [heads, T, rank] in the pool's dtype."""
    _need(q_abs, "q_abs", torch.float32, 3)
    _need(q_rot, "q_rot", torch.float32, 3)
    _need(pool, "pool", ndim=4)
    _need(page_table, "page_table", torch.int32, 2)
    H, T, L = q_abs.shape
    R = q_rot.shape[2]
    if tuple(q_rot.shape[:2]) != (T, H) or pool.shape[1] != 1 or pool.shape[3] != L + R:
        raise KernelError(f"latent_attention: q_abs {tuple(q_abs.shape)}, q_rot {tuple(q_rot.shape)}, pool {tuple(pool.shape)}")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.numel() != H:
            raise KernelError(f"latent_attention: {sink.numel()} sinks for {H} heads")
    out = torch.empty((H, T, L), dtype=pool.dtype, device=q_abs.device)
    max_runs, scratch = 0, None
    if ctx.single_token and ctx.max_len > LATENT_RUN_KEYS:
        # one token per sequence over more than one run of keys: a block a run (cut by the key's index, so a sequence's
        # result does not depend on the batch), then a merge; ctx.max_len bounds every sequence's length
        max_runs = -(-ctx.max_len // LATENT_RUN_KEYS)
        scratch = torch.empty((max_runs * T * H * (L + 2),), dtype=torch.float32, device=q_abs.device)
    _call("attention_latent", "qwb_latent_attn", _ptr(q_abs), _ptr(q_rot), _ptr(pool), _ptr(page_table), _ptr(ctx.cu_seqlens),
          _ptr(ctx.pos0), _ptr(sink), _ptr(out), _i(_dt(pool.dtype)), _i(ctx.n_seqs), _i(T), _i(ctx.max_new), _i(H), _i(L),
          _i(R), _i(pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _i(max_runs), _ptr(scratch), _stream(),
          kernels=2 if max_runs else 1)
    return out


# ----------------------------------------------------------------------------- routed experts
MOE_MAX_TOP = 16            # csrc/moe.cu: QWB_MOE_MAX_TOP
_MOE_SLOTS_PER_LAUNCH = 65535


def moe_route(logits: torch.Tensor, top: int, renormalize: bool = False):
    """softmax over float32 ``logits`` [T, E]; the ``top`` largest per row (ties to the lower index).  Returns
    (chosen int32 [T, top], weight float32 [T, top]): the chosen scores, divided by their sum if ``renormalize``."""
    _need(logits, "logits", torch.float32, 2)
    T, E = logits.shape
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _call("moe", "qwb_moe_route", _ptr(logits), _ptr(chosen), _ptr(weight), _i(T), _i(E), _i(top),
          _i(1 if renormalize else 0), _stream())
    return chosen, weight


def moe_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor,
                weight: torch.Tensor) -> torch.Tensor:
    """sum_k weight[t, k] * down_e(silu(gate_e x_t) * up_e x_t), e = chosen[t, k].  ``x`` [T, D] and the stacked
    weights (``w_gate_up`` [E, 2F, D]: gate rows, then up rows; ``w_down`` [E, D, F]) in one dtype.  Returns float32 [T, D]."""
    _need(x, "x", w_gate_up.dtype, 2)
    _need(w_gate_up, "w_gate_up", ndim=3)
    _need(w_down, "w_down", w_gate_up.dtype, 3)
    _need(chosen, "chosen", torch.int32, 2)
    _need(weight, "weight", torch.float32, 2)
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    F, top = F2 // 2, chosen.shape[1]
    if w_gate_up.shape[2] != D or tuple(w_down.shape) != (E, D, F) or tuple(chosen.shape) != (T, top) or weight.shape != chosen.shape:
        raise KernelError(f"moe_experts: x {tuple(x.shape)}, gate/up {tuple(w_gate_up.shape)}, down {tuple(w_down.shape)}, "
                          f"chosen {tuple(chosen.shape)}")
    act = torch.empty((T * top, F), dtype=x.dtype, device=x.device)
    out = torch.empty((T, D), dtype=torch.float32, device=x.device)
    per = max(1, _MOE_SLOTS_PER_LAUNCH // top)
    for t0 in range(0, T, per):
        n = min(per, T - t0)
        _call("moe", "qwb_moe_experts", _ptr(x[t0:t0 + n]), _ptr(w_gate_up), _ptr(w_down), _ptr(chosen[t0:t0 + n]),
              _ptr(weight[t0:t0 + n]), _ptr(act[t0 * top:(t0 + n) * top]), _ptr(out[t0:t0 + n]), _i(_dt(x.dtype)), _i(n),
              _i(D), _i(F), _i(top), _stream(), kernels=2)
    return out


MOE_GROUPED_MIN_TOKENS = 17     # from here on bfloat16 tokens are sorted by expert and go through the library's grouped product


def moe_grouped_fits(x: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    """Whether a step's tokens take the sorted, grouped form (else the expert-streaming kernels do)."""
    D, F = w_gate_up.shape[2], w_gate_up.shape[1] // 2
    return (x.dtype == torch.bfloat16 and x.shape[0] >= MOE_GROUPED_MIN_TOKENS and D % 8 == 0 and F % 8 == 0
            and hasattr(torch, "_grouped_mm"))


def moe_experts_grouped(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor,
                        weight: torch.Tensor) -> torch.Tensor:
    """``moe_experts`` for many bfloat16 tokens: the tokens' copies are sorted by expert (a stable sort: nothing depends
    on the order in which blocks finish), each expert's run goes through the library's grouped matrix product (32-bit
    sums, bfloat16 results) for gate/up and for down, with the gated SiLU between them and the weighted sum of every
    token's copies after them in kernels of this library.  No value is read on the host."""
    _need(x, "x", torch.bfloat16, 2)
    _need(w_gate_up, "w_gate_up", torch.bfloat16, 3)
    _need(w_down, "w_down", torch.bfloat16, 3)
    _need(chosen, "chosen", torch.int32, 2)
    _need(weight, "weight", torch.float32, 2)
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    F, top = F2 // 2, chosen.shape[1]
    flat = chosen.view(-1)
    order = torch.argsort(flat, stable=True)                        # sorted row -> copy (t * top + k)
    ends = torch.searchsorted(flat.index_select(0, order), torch.arange(E, dtype=torch.int32, device=x.device),
                              right=True).to(torch.int32)           # where each expert's run ends (no value read on the host)
    place = torch.empty_like(order)
    place[order] = torch.arange(order.numel(), device=x.device)     # copy -> sorted row
    xs = x.index_select(0, order // top)
    gu = torch._grouped_mm(xs, w_gate_up.transpose(1, 2), offs=ends).contiguous()
    act = torch.empty((T * top, F), dtype=torch.bfloat16, device=x.device)
    _call("moe", "qwb_moe_gated_act", _ptr(gu), _ptr(act), _i(T * top), _i(F), _stream())
    y = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends).contiguous()
    out = torch.empty((T, D), dtype=torch.float32, device=x.device)
    _call("moe", "qwb_moe_combine", _ptr(y), _ptr(place), _ptr(weight), _ptr(out), _i(T), _i(D), _i(top), _stream())
    return out


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
           sequence_index: torch.Tensor | None = None, step: int = 0, recent: torch.Tensor | None = None,
           repeat_penalty: float = 1.0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
           out_u: torch.Tensor | None = None, step_add: torch.Tensor | None = None,
           out: torch.Tensor | None = None, split: bool = True, seed_from: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of float32 ``logits`` [B, V] (changed in place by penalties).
    ``seed_from``: one int64 on the device that holds the seed (``seed`` is then not used); ``step_add``: one int32 on
    the device that is added to ``step``.  With both, a captured graph holds neither the seed nor the step.
    ``split`` False: one block per row whatever the sizes (the result is the same).  With few rows the kernels cut
    every row into chunks and count into one buffer per device: such calls must follow one another on one stream."""
    _need(logits, "logits", torch.float32, 2)
    B, V = logits.shape
    window = 0
    if recent is not None:
        _need(recent, "recent", torch.int32, 2)
        window = recent.shape[1]
    if sequence_index is not None:
        _need(sequence_index, "sequence_index", torch.int32, 1)
    if out_u is not None:
        _need(out_u, "out_u", torch.float64, 1)
    if seed_from is not None:
        _need(seed_from, "seed_from", torch.int64, 1)
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    # few rows and a small top-k: the kernels cut every row into chunks and want scratch memory for what the chunks find
    scratch_bytes = (_lookup("sampling", "qwb_sample_scratch_bytes")[1](_i(B), _i(V), _f(temperature), _i(top_k), _f(top_p))
                     if split else 0)
    scratch = counters = None
    if scratch_bytes:
        scratch = torch.empty((scratch_bytes,), dtype=torch.uint8, device=logits.device)
        if temperature > 0:
            counters = _sample_counters(logits.device, B)
    _call("sampling", "qwb_sample", _ptr(logits), _i(B), _i(V), _ptr(recent), _i(window), _f(repeat_penalty),
          _f(presence_penalty), _f(frequency_penalty), _f(temperature), _i(top_k), _f(top_p),
          ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_from), _ptr(sequence_index), ctypes.c_uint(step & 0xFFFFFFFF),
          _ptr(step_add), _ptr(out), _ptr(out_u), _ptr(scratch), _ptr(counters), _stream(),
          kernels=(3 if temperature > 0 else 2) if scratch_bytes else 1)
    return out


SAMPLE_SPLIT_MAX_ROWS = 592     # the split sampling kernels are used for fewer rows than this (four blocks an SM, two chunks a row)
_SAMPLE_COUNTERS: dict = {}     # device -> zeros [SAMPLE_SPLIT_MAX_ROWS * 1025]: the split sampling kernels count into them (a
                                # counter and 1,024 bins a row) and leave them zero; made once and kept, since captured
                                # graphs hold their address


def _sample_counters(device, rows: int) -> torch.Tensor:
    if rows > SAMPLE_SPLIT_MAX_ROWS:
        raise KernelError(f"sample: {rows} rows cannot be cut into chunks (at most {SAMPLE_SPLIT_MAX_ROWS})")
    key = torch.device(device).index or 0
    have = _SAMPLE_COUNTERS.get(key)
    if have is None:
        have = _SAMPLE_COUNTERS[key] = torch.zeros((SAMPLE_SPLIT_MAX_ROWS * 1025,), dtype=torch.int32, device=device)
    return have


def decode_advance(sampled, token_ids, tok_pos, pos0, seq_len, step_counter=None, recent=None, n_seen=None) -> None:
    """The sampled ids become the next inputs; positions and lengths go up by one."""
    B = sampled.numel()
    window = recent.shape[1] if recent is not None else 0
    _call("elementwise", "qwb_decode_advance", _ptr(sampled), _ptr(token_ids), _ptr(tok_pos), _ptr(pos0),
          _ptr(seq_len), _ptr(step_counter), _ptr(recent), _ptr(n_seen), _i(window), _i(B), _stream())

"""ctypes bindings of the CUDA library: one Python function per kernel entry point.

Every function takes CUDA tensors, checks types, shapes and contiguity on the host,
launches on torch's current stream and returns nothing (outputs are arguments).  There
is no CPU path: a call with a CPU tensor, or on a machine where the library cannot be
built or loaded, raises.
"""

from __future__ import annotations

import ctypes
import logging
from typing import Optional

import torch

from . import build

ABI_VERSION = 11
log = logging.getLogger("miniserve_b200")
_library: Optional[ctypes.CDLL] = None

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def library() -> ctypes.CDLL:
    """The loaded CUDA library (built on first use)."""
    global _library
    if _library is None:
        path = build.library_path()
        lib = ctypes.CDLL(str(path))
        lib.ms_last_error.restype = ctypes.c_char_p
        lib.ms_abi_version.restype = ctypes.c_int
        if lib.ms_abi_version() != ABI_VERSION:
            raise KernelError(f"{path} reports ABI {lib.ms_abi_version()}, bindings expect {ABI_VERSION}; rebuild it")
        # argument and result types from the prototypes in the sources: calls then pass plain Python numbers
        kinds = {"pointer": ctypes.c_void_p, "int": ctypes.c_int, "float": ctypes.c_float, "longlong": ctypes.c_longlong,
                 "string": ctypes.c_char_p, "void": None}
        for name, (result, arguments) in build.exported_signatures().items():
            function = getattr(lib, name)
            function.restype = kinds[result]
            function.argtypes = [kinds[a] for a in arguments]
        _library = lib
    return _library


launch_count = 0   # entry points of this library called so far (each launches one kernel, or a fixed few)


def _check(code: int) -> None:
    global launch_count
    if code != 0:
        raise KernelError(library().ms_last_error().decode())
    launch_count += 1


_device_index: Optional[int] = None


def _stream() -> int:
    """torch's current stream on the library's device (the raw handle: this is called for every launch)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(_device_index)


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The tensor's address (None: a null pointer); the entry points' argument types are known to ctypes."""
    return None if tensor is None else tensor.data_ptr()


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)") from None


def _want(tensor: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if (tensor.is_cuda and tensor.is_contiguous() and (dtype is None or tensor.dtype is dtype)
            and (shape is None or tensor.shape == shape)):
        return                      # (one test for the usual case; what follows words the refusal)
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")


_i = int        # (arguments are converted by ctypes from the prototypes' types; these only coerce)
_f = float


# --------------------------------------------------------------------------- memory-bound kernels


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """``out[n] = scale * float32(table[tokens[n]])``; tokens int32 ``[N]``, out float32 ``[N, H]``."""
    n, hidden = tokens.numel(), table.shape[1]
    _want(tokens, "tokens", torch.int32)
    _want(table, "table")
    _want(out, "out", torch.float32, (n, hidden))
    _check(library().ms_embedding(_ptr(tokens), _ptr(table), _i(_code(table.dtype)), _ptr(out), _i(n), _i(hidden),
                                  _f(scale), _stream()))


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: Optional[float] = None) -> None:
    """In place on float32 ``x``: ``x *= scale``, then with ``cap``: ``x = cap * tanh(x / cap)``."""
    _want(x, "x", torch.float32)
    _check(library().ms_scale_softcap(_ptr(x), x.numel(), _f(scale), _f(cap if cap else 0.0), _stream()))


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, delta2: Optional[torch.Tensor] = None) -> None:
    """Adds ``delta`` into the float32 ``residual`` (in place) and writes its RMSNorm to ``out``.  With ``delta2``
    (a second output of the same layer) the stream receives ``delta + delta2``, summed in float32.

    With ``rows`` (int32 ``[K]``) only those rows are normalised, into ``out [K, H]``, and
    the residual is left untouched.  ``weight`` may be float32 or bfloat16 whatever ``out`` is.
    """
    hidden = residual.shape[1]
    n_out = residual.shape[0] if rows is None else rows.numel()
    _want(residual, "residual", torch.float32)
    _want(out, "out", None, (n_out, hidden))
    _want(weight, "weight", None, (hidden,))
    if delta is not None:
        _want(delta, "delta", out.dtype, residual.shape)
    if delta2 is not None:
        if delta is None:
            delta, delta2 = delta2, None
        else:
            _want(delta2, "delta2", out.dtype, residual.shape)
    if rows is not None:
        _want(rows, "rows", torch.int32)
    _check(library().ms_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(delta2), _i(_code(out.dtype)), _ptr(weight),
                                    _i(_code(weight.dtype)), _ptr(rows), _ptr(out), _i(n_out), _i(hidden), _f(eps),
                                    _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """RMSNorm over the last dim of ``x [rows, size]`` into ``out`` of the same type and shape."""
    _want(x, "x")
    _want(out, "out", x.dtype, x.shape)
    size = x.shape[-1]
    _want(weight, "weight", None, (size,))
    _check(library().ms_rmsnorm(_ptr(x), _i(_code(x.dtype)), _ptr(weight), _i(_code(weight.dtype)), _ptr(out),
                                _i(x.numel() // size), _i(size), _f(eps), _stream()))


def postnorm_add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], post_weight: Optional[torch.Tensor],
                         post_eps: float, weight: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                         rows: Optional[torch.Tensor] = None, post_scale: float = 1.0, post_norm: bool = True) -> None:
    """``residual += post_scale * post_weight * delta / rms(delta)`` (float32, in place), ``out = weight * residual /
    rms(residual)``: a sublayer's output passes a norm of its own on its way into the stream, and the stream is normed for
    the next sublayer.  ``post_norm=False``: the output is not divided by its root mean square, ``residual += post_scale *
    post_weight * delta`` (a scale per channel on what a sublayer adds).  ``delta`` None: nothing is added.  ``weight`` None: the stream is not normed, ``out`` is the stream
    rounded once to ``out``'s type (a sublayer that reads the stream itself).  With ``rows`` (int32 ``[K]``) only those
    rows are computed, into ``out [K, H]``, and the residual is left untouched.  The weights may be float32 or bfloat16
    whatever ``out`` is."""
    hidden = residual.shape[1]
    n_out = residual.shape[0] if rows is None else rows.numel()
    _want(residual, "residual", torch.float32)
    _want(out, "out", None, (n_out, hidden))
    if delta is not None:
        _want(delta, "delta", out.dtype, residual.shape)
        _want(post_weight, "post_weight", None, (hidden,))
    if weight is not None:
        _want(weight, "weight", None, (hidden,))
    if rows is not None:
        _want(rows, "rows", torch.int32)
    _check(library().ms_postnorm_add_rmsnorm(
        _ptr(residual), _ptr(delta), _i(_code(out.dtype)), _ptr(post_weight) if delta is not None else None,
        _i(_code(post_weight.dtype)) if delta is not None else 0, _f(post_eps if post_norm else -1.0), _f(post_scale), _ptr(weight),
        _i(_code(weight.dtype)) if weight is not None else 0, _f(eps), _ptr(rows), _ptr(out), _i(n_out), _i(hidden), _stream()))


def qkv_prepare(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, n_q: int, n_kv: int, head_dim: int, value_dim: int,
                slots: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                cos_sin: Optional[torch.Tensor], rotary_dim: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                q_out: torch.Tensor, interleaved: bool = False, bias: Optional[torch.Tensor] = None,
                value_heads: Optional[int] = None) -> None:
    """Per-head RMSNorm of q and k, rotation of their first ``rotary_dim`` entries (entry i with entry i + rotary_dim / 2,
    or, ``interleaved``, entry 2i with entry 2i + 1), and the append of k and v
    to one layer's pools, for a projection ``proj [N, ld]`` whose columns are laid out freely: query head h at
    ``q_col + h * head_dim``, key head g at ``k_col + g * head_dim``, value head g at ``v_col + g * value_dim``.
    ``k_col < 0``: the projection holds no keys and values (the layer reads another layer's) and only ``q_out
    [N, n_q, head_dim]`` is written.  Key pool ``[pages, n_kv, page_size, head_dim]``, value pool ``[.., value_dim]``;
    norm weights float32 ``[head_dim]`` or None; ``cos_sin`` float32 ``[N, rotary_dim / 2, 2]`` or None.  ``bias`` (float32
    ``[ld]``, column by column as ``proj``): the projection's bias, added in float32 as the heads are read.  ``value_heads``
    (a divisor of ``n_kv``; None: ``n_kv``): the projection and the value pool ``[pages, value_heads, page_size, value_dim]`` hold
    that many value heads (key heads that share values: key head g reads value head ``g % value_heads``)."""
    n, ld = proj.shape
    value_heads = n_kv if value_heads is None else int(value_heads)
    if value_heads < 1 or n_kv % value_heads:
        raise KernelError(f"qkv_prepare: {value_heads} value heads for {n_kv} key heads")
    if bias is not None:
        _want(bias, "bias", torch.float32, (ld,))
    _want(proj, "proj")
    _want(q_out, "q_out", proj.dtype, (n, n_q, head_dim))
    own = k_col >= 0
    if q_col < 0 or q_col + n_q * head_dim > ld or (own and (k_col + n_kv * head_dim > ld or v_col < 0 or v_col + value_heads * value_dim > ld)):
        raise KernelError(f"qkv_prepare: columns {q_col}, {k_col}, {v_col} of {n_q}/{n_kv} heads of {head_dim}/{value_dim} in rows of {ld}")
    if own:
        _want(slots, "slots", torch.int32, (n,))
        _want(k_pool, "k_pool", proj.dtype)
        _want(v_pool, "v_pool", proj.dtype)
        if (k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, k_pool.shape[2], head_dim)
                or tuple(v_pool.shape) != (k_pool.shape[0], value_heads, k_pool.shape[2], value_dim)):
            raise KernelError(f"pool shapes {tuple(k_pool.shape)}, {tuple(v_pool.shape)} are not [pages, {n_kv} | {value_heads}, page_size, "
                              f"{head_dim} | {value_dim}]")
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _want(weight, name, torch.float32, (head_dim,))
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (n, rotary_dim // 2, 2))
    else:
        rotary_dim = 0
    _check(library().ms_qkv_prepare(
        _ptr(proj), _i(_code(proj.dtype)), _i(ld), _i(q_col), _i(k_col if own else -1), _i(v_col if own else -1), _i(n_q), _i(n_kv),
        _i(head_dim), _i(value_dim), _ptr(slots) if own else None, _ptr(q_weight), _ptr(k_weight) if own else None, _f(eps),
        _ptr(cos_sin), _i(rotary_dim), _ptr(k_pool) if own else None, _ptr(v_pool) if own else None,
        _i(k_pool.shape[2]) if own else 1, _ptr(q_out), _i(n), _i(1 if interleaved else 0), _ptr(bias), _i(value_heads), _stream()))


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos_sin: torch.Tensor, magnitude: float = 1.0) -> None:
    """``cos_sin[n, j] = magnitude * (cos, sin)(positions[n] * inv_freq[j])`` in float32; cos_sin ``[N, half, 2]``."""
    n, half = positions.numel(), inv_freq.numel()
    _want(positions, "positions", torch.int32)
    _want(inv_freq, "inv_freq", torch.float32)
    _want(cos_sin, "cos_sin", torch.float32, (n, half, 2))
    _check(library().ms_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(cos_sin), _i(n), _i(half), _f(magnitude), _stream()))


def qk_norm_rope_append(qkv: torch.Tensor, slots: torch.Tensor, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                        rotary_dim: int, interleaved: bool, k_pool: torch.Tensor, v_pool: torch.Tensor,
                        n_q: int, n_kv: int, head_dim: int, q_out: torch.Tensor) -> None:
    """Per-head RMSNorm of q and k, rotation, and the append of k and v to one layer's pools.

    qkv ``[N, (n_q + 2 n_kv) * d]``; slots int32 ``[N]`` (page * page_size + offset, negative:
    no write); pools ``[pages, n_kv, page_size, d]``; q_out ``[N, n_q, d]``; cos_sin float32
    ``[N, rotary_dim / 2, 2]`` or None for no rotation; norm weights ``[d]`` or None.
    """
    n = qkv.shape[0]
    _want(qkv, "qkv", None, (n, (n_q + 2 * n_kv) * head_dim))
    _want(slots, "slots", torch.int32, (n,))
    _want(k_pool, "k_pool", qkv.dtype)
    _want(v_pool, "v_pool", qkv.dtype, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[3] != head_dim:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, {n_kv}, page_size, {head_dim}]")
    _want(q_out, "q_out", qkv.dtype, (n, n_q, head_dim))
    weight_code = 0
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _want(weight, name, None, (head_dim,))
            weight_code = _code(weight.dtype)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share one element type")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (n, rotary_dim // 2, 2))
    else:
        rotary_dim = 0
    _check(library().ms_qk_norm_rope_append(
        _ptr(qkv), _i(_code(qkv.dtype)), _ptr(slots), _ptr(q_weight), _ptr(k_weight), _i(weight_code), _f(eps),
        _ptr(cos_sin), _i(rotary_dim), _i(1 if interleaved else 0), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[2]),
        _i(n_q), _i(n_kv), _i(head_dim), _ptr(q_out), _i(n), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, paired: bool = False, bias: Optional[torch.Tensor] = None) -> None:
    """``out[n, c] = silu(gate_up[n, c]) * gate_up[n, I + c]`` for gate_up ``[N, 2 I]``.  With ``bias`` (float32 ``[2 I]``,
    not with ``paired``) it is added to both halves first, in float32.

    ``paired``: the columns come as :func:`interleave_gate_up` orders a weight's rows (eight gate columns, then
    the up columns of the same features, and so on): ``out[n, 8 j + r] = silu(gate_up[n, 16 j + r]) *
    gate_up[n, 16 j + 8 + r]``.
    """
    n, inter = out.shape
    _want(gate_up, "gate_up", None, (n, 2 * inter))
    _want(out, "out", gate_up.dtype)
    if bias is not None:
        _want(bias, "bias", torch.float32, (2 * inter,))
        if paired:
            raise KernelError("silu_mul: a bias goes with the plain layout (gate columns, then up columns)")
        _check(library().ms_silu_mul_bias(_ptr(gate_up), _i(_code(gate_up.dtype)), _ptr(bias), _ptr(out), _i(n), _i(inter), _stream()))
        return
    _check(library().ms_silu_mul(_ptr(gate_up), _i(_code(gate_up.dtype)), _ptr(out), _i(n), _i(inter),
                                 _i(1 if paired else 0), _stream()))


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """In place: ``x[n, c] += bias[c]`` (float32 ``[C]``), added in float32."""
    _want(x, "x")
    _want(bias, "bias", torch.float32, (x.shape[-1],))
    _check(library().ms_add_bias(_ptr(x), _i(_code(x.dtype)), _ptr(bias), _i(x.numel() // x.shape[-1]), _i(x.shape[-1]), _stream()))


def scaled_sum(a: torch.Tensor, a_scale: float, b: torch.Tensor, b_scale: float, out: torch.Tensor) -> None:
    """``out = a_scale * a + b_scale * b`` elementwise, formed in float32; ``out`` may be ``a`` or ``b``."""
    _want(a, "a")
    _want(b, "b", a.dtype, a.shape)
    _want(out, "out", a.dtype, a.shape)
    _check(library().ms_scaled_sum(_ptr(a), _f(a_scale), _ptr(b), _f(b_scale), _ptr(out), _i(_code(a.dtype)), a.numel(), _stream()))


def normed_sum(a: torch.Tensor, a_weight: torch.Tensor, a_scale: float, b: torch.Tensor, b_weight: torch.Tensor, b_scale: float,
               eps: float, out: torch.Tensor) -> None:
    """``out = a_scale * a_weight * a / rms(a) + b_scale * b_weight * b / rms(b)`` row by row (``eps`` inside the roots): two
    outputs, each normed over the row with a float32 weight of its own, summed."""
    rows, hidden = a.shape
    _want(a, "a")
    _want(b, "b", a.dtype, a.shape)
    _want(out, "out", a.dtype, a.shape)
    _want(a_weight, "a_weight", torch.float32, (hidden,))
    _want(b_weight, "b_weight", torch.float32, (hidden,))
    _check(library().ms_normed_sum(_ptr(a), _ptr(a_weight), _f(a_scale), _ptr(b), _ptr(b_weight), _f(b_scale), _f(eps), _ptr(out),
                                   _i(_code(a.dtype)), _i(rows), _i(hidden), _stream()))


def sigmoid_gate_mul(x: torch.Tensor, gate: torch.Tensor, gate_col: int, out: torch.Tensor) -> None:
    """``out[n, c] = x[n, c] * sigmoid(gate[n, gate_col + c])``: a gate per entry; ``out`` may be ``x``."""
    rows, width = x.shape
    _want(x, "x")
    _want(gate, "gate", x.dtype)
    _want(out, "out", x.dtype, x.shape)
    if gate.dim() != 2 or gate.shape[0] != rows or gate_col < 0 or gate_col + width > gate.shape[1]:
        raise KernelError(f"sigmoid_gate_mul: gate {tuple(gate.shape)} from column {gate_col} for rows of {width}")
    _check(library().ms_sigmoid_gate_mul(_ptr(x), _ptr(gate), _i(gate.shape[1]), _i(gate_col), _ptr(out), _i(_code(x.dtype)), _i(rows),
                                         _i(width), _stream()))


def differential_combine(a: torch.Tensor, lam: float, eps: float, out_scale: float, gate: Optional[torch.Tensor], gate_col: int,
                         out: torch.Tensor) -> None:
    """``a [N, 2 H, dv]`` holds the outputs of two score maps over the same values (the first map's heads, then the second's):
    ``o = a[:, h] - lam * a[:, H + h]``, each head divided by its root mean square (``eps`` inside the root), times ``out_scale``,
    times ``sigmoid(gate[n, gate_col + h dv + c])`` where ``gate`` is given.  ``out [N, H, dv]``."""
    n, both, dv = a.shape
    heads = both // 2
    _want(a, "a")
    _want(out, "out", a.dtype, (n, heads, dv))
    gate_ld = 0
    if gate is not None:
        _want(gate, "gate", a.dtype)
        if gate.dim() != 2 or gate.shape[0] != n or gate_col < 0 or gate_col + heads * dv > gate.shape[1]:
            raise KernelError(f"differential_combine: gate {tuple(gate.shape)} from column {gate_col} for {heads} heads of {dv}")
        gate_ld = gate.shape[1]
    if both != 2 * heads:
        raise KernelError(f"differential_combine: {both} heads are not two maps")
    _check(library().ms_differential_combine(_ptr(a), _i(heads), _i(dv), _f(lam), _f(eps), _f(out_scale), _ptr(gate), _i(gate_ld),
                                             _i(gate_col), _ptr(out), _i(_code(a.dtype)), _i(n), _stream()))


def token_shift(x: torch.Tensor, shift: torch.Tensor, states: torch.Tensor, state_offset: int, state_slots: torch.Tensor,
                query_start: torch.Tensor, request_of_token: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t] = x[t] + (x[t - 1] - x[t]) * shift`` per channel along each request's tokens; the token before a portion's
    first is what ``states[slot, state_offset:]`` (float32 ``[hidden]``, zero for a new sequence) holds, and the portion's last
    ``x`` is left there.  ``shift`` float32 ``[hidden]``; ``out`` is not ``x``."""
    n, hidden = x.shape
    _want(x, "x")
    _want(out, "out", x.dtype, x.shape)
    _want(shift, "shift", torch.float32, (hidden,))
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    _want(request_of_token, "request_of_token", torch.int32, (n,))
    stride = _state_rows(states, state_offset, hidden)
    _check(library().ms_token_shift(_ptr(x), _i(_code(x.dtype)), _ptr(shift), _ptr(states), stride, _i(state_offset),
                                    _ptr(state_slots), _ptr(query_start), _ptr(request_of_token), _ptr(out), _i(n), _i(hidden),
                                    _stream()))


def pair_embedding(tokens: torch.Tensor, table: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int, states: torch.Tensor,
                   state_slots: torch.Tensor, query_start: torch.Tensor, request_of_token: torch.Tensor,
                   residual: torch.Tensor) -> None:
    """``residual[t] += table[(token[t - 1] * mul_prev + token[t] * mul_cur) % buckets]``; a sequence's first token takes row
    ``buckets``.  ``states`` int32 ``[slots, 1]`` holds each request's last token + 1 (0: none yet) and is updated."""
    n, hidden = residual.shape
    _want(tokens, "tokens", torch.int32, (n,))
    _want(table, "table", None, (buckets + 1, hidden))
    _want(residual, "residual", torch.float32)
    _want(states, "states", torch.int32)
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    _want(request_of_token, "request_of_token", torch.int32, (n,))
    if states.dim() != 2 or states.shape[1] < 1:
        raise KernelError(f"pair_embedding: states {tuple(states.shape)} do not hold a token per slot")
    _check(library().ms_pair_embedding(_ptr(tokens), _ptr(table), _i(_code(table.dtype)), _i(buckets), _i(mul_prev), _i(mul_cur),
                                       _ptr(states), states.shape[1], _i(0), _ptr(state_slots), _ptr(query_start),
                                       _ptr(request_of_token), _ptr(residual), _i(n), _i(hidden), _stream()))


# --------------------------------------------------------------------------- attention

MAX_HEAD_DIM = 512      # of the general attention kernel (attention_generic.cu: 16 output lanes per thread)


USE_MMA_ANY = __import__("os").environ.get("MINISERVE_B200_MMA_ANY", "1") == "1"


def attention_kernels(dtype: torch.dtype, head_dim: int, n_q: int, n_kv: int, page_size: int,
                      modified_scores: bool = False, value_dim: Optional[int] = None, extended: bool = False,
                      chunk: Optional[int] = None, shared_values: bool = False) -> dict:
    """Which kernel :func:`paged_attention` runs for these sizes: ``{"decode": name, "prompt": name}`` with the
    names ``tcgen05``, ``mma.sync`` and ``general`` (float32 arithmetic, any size; the only one of the float32
    path, and what bfloat16 falls back to for head sizes the tensor-core kernels are not built for and for
    scores with a soft cap or a distance bias)."""
    lib = library()
    value_dim = head_dim if value_dim is None else value_dim
    chunk = chunk or (1 if shared_values else None)      # (key heads that share value heads: the same two kernels)
    extended = extended or bool(chunk)
    if (USE_MMA_ANY and extended and not modified_scores and dtype == torch.bfloat16
            and (value_dim != head_dim or bool(chunk) or not lib.ms_attention_mma_supports(_i(head_dim)))
            and lib.ms_attention_mma_any_supports(_i(head_dim), _i(value_dim))):
        # (``extended``: the attention has a sink, a gate or value heads of their own size)
        return {"decode": "mma.sync (any size)", "prompt": "mma.sync (any size)"}
    if modified_scores or value_dim != head_dim or chunk or dtype != torch.bfloat16 or not lib.ms_attention_mma_supports(_i(head_dim)):
        return {"decode": "general", "prompt": "general"}
    prompt = "mma.sync"
    if USE_TCGEN05_ATTENTION and lib.ms_attention_tcgen05_supports(_i(head_dim), _i(n_q), _i(n_kv), _i(page_size)):
        prompt = "tcgen05"
    return {"decode": "mma.sync", "prompt": prompt}



def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                    request_of_token: torch.Tensor, positions: torch.Tensor, query_start: torch.Tensor,
                    context_lens: torch.Tensor, max_query_len: int, max_context_len: int, scale: float,
                    window: Optional[int], out: torch.Tensor, host_query_start: Optional[list] = None,
                    softcap: Optional[float] = None, bias_slopes: Optional[torch.Tensor] = None, sink: bool = False,
                    gate: Optional[torch.Tensor] = None, gate_col: int = 0, chunk: Optional[int] = None) -> None:
    """Causal grouped-query attention of every token over its request's paged keys and values.

    ``chunk``: a token at position p sees only the keys of its own chunk, ``p - p % chunk .. p`` (chunks are counted from
    position 0 of the sequence).  A value pool with fewer heads than the key pool (a divisor): key head g reads value head
    ``g % value heads``.  The general kernel and the tensor-core kernel for any head size implement both.

    q ``[N, n_q, d]``, out ``[N, n_q, dv]`` (dv: the value pool's last dimension, usually d); pools of one layer
    ``[pages, n_kv, page_size, d | dv]``.  ``sink``: the softmax's denominator gets one more term ``exp(0)`` (a key of
    score 0 without a value).  ``gate [N, ld]`` with ``gate_col``: head h's output is multiplied by
    ``sigmoid(gate[n, gate_col + h])`` as it is stored.  block_tables
    int32 ``[R, width]``; request_of_token, positions int32 ``[N]``; query_start ``[R + 1]`` and
    context_lens ``[R]`` describe the same batch per request (a request's tokens are the last
    ones of its context).  A token at position p sees keys ``max(0, p - window + 1) .. p`` of
    its own request, which must be in the pool already.

    Score modifiers, both off by default: ``softcap`` turns a scaled score ``s`` into ``softcap * tanh(s /
    softcap)``; ``bias_slopes`` (float32 ``[n_q]``) adds ``slope[head] * (key position - query position)``
    after it.  The general kernel implements them; the tensor-core kernels do not, so a call with either
    runs the general kernel whatever the sizes.

    bfloat16 with a head size the tensor-core kernels are built for runs there
    (``max_query_len``/``max_context_len`` are upper bounds used to shape their grids); everything
    else runs the general float32-arithmetic kernel.  With ``host_query_start`` (the same numbers
    as ``query_start``, on the host) a batch that begins with single-token requests and goes on
    with prompt portions is run as two launches, so that the single tokens get their keys split
    over many thread blocks instead of one block walking a whole context.
    """
    n, n_q, head_dim = q.shape
    _want(q, "q")
    _want(k_pool, "k_pool", q.dtype)
    if k_pool.dim() != 4 or k_pool.shape[3] != head_dim:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, n_kv, page_size, {head_dim}]")
    _want(v_pool, "v_pool", q.dtype)
    if (v_pool.dim() != 4 or v_pool.shape[0] != k_pool.shape[0] or v_pool.shape[2] != k_pool.shape[2]
            or v_pool.shape[1] < 1 or k_pool.shape[1] % v_pool.shape[1]):
        raise KernelError(f"value pool {tuple(v_pool.shape)} does not go with key pool {tuple(k_pool.shape)}")
    value_dim, n_v = v_pool.shape[3], v_pool.shape[1]
    _want(out, "out", q.dtype, (n, n_q, value_dim))
    gate_ptr, gate_ld = None, 0
    if gate is not None:
        _want(gate, "gate", q.dtype)
        if gate.dim() != 2 or gate.shape[0] != n or gate_col < 0 or gate_col + n_q > gate.shape[1]:
            raise KernelError(f"paged_attention: gate logits {tuple(gate.shape)} for {n} tokens of {n_q} heads from column {gate_col}")
        gate_ptr, gate_ld = gate.data_ptr() + gate_col * gate.element_size(), gate.shape[1]
    _want(block_tables, "block_tables", torch.int32)
    _want(request_of_token, "request_of_token", torch.int32, (n,))
    _want(positions, "positions", torch.int32, (n,))
    n_requests = context_lens.numel()
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    _want(context_lens, "context_lens", torch.int32, (n_requests,))
    lib = library()
    n_kv = k_pool.shape[1]
    modified = bool(softcap) or bias_slopes is not None
    if bias_slopes is not None:
        _want(bias_slopes, "bias_slopes", torch.float32, (n_q,))
    # the general form (a sink, a gate, value heads of their own size) at sizes the unrolled tensor-core kernels are not built
    # for: the tensor-core kernel whose head sizes are run-time numbers (multiples of 16 up to 128)
    shared_values = n_v != n_kv
    extended = sink or gate is not None or value_dim != head_dim or bool(chunk) or shared_values
    if (USE_MMA_ANY and extended and not modified and q.dtype == torch.bfloat16
            and (value_dim != head_dim or bool(chunk) or shared_values or not lib.ms_attention_mma_supports(_i(head_dim)))
            and lib.ms_attention_mma_any_supports(_i(head_dim), _i(value_dim))):
        reach = min(max_context_len, chunk) if chunk else max_context_len      # the most keys a token sees
        def run_any(first: int, last: int, longest: int, rows: int, first_row: int = 0) -> None:
            count = last - first
            splits = lib.ms_attention_mma_any_splits(_i(count), _i(n_kv), _i(n_q), _i(longest), _i(reach))
            part_o = part_lse = None
            if splits > 1:
                part_o = torch.empty((rows * n_q * splits, value_dim), dtype=torch.float32, device=q.device)
                part_lse = torch.empty((rows * n_q * splits,), dtype=torch.float32, device=q.device)
            _check(lib.ms_paged_attention_mma_any(
                _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables[first:last]), _i(block_tables.shape[1]),
                _ptr(query_start[first:last + 1]), _ptr(context_lens[first:last]), _i(k_pool.shape[2]), _i(n_q), _i(n_kv),
                _i(head_dim), _i(value_dim), _f(scale), _i(window if window else 0), _ptr(out), _ptr(part_o), _ptr(part_lse),
                _i(splits), _i(count), _i(longest), _i(rows), _i(1 if sink else 0), gate_ptr, _i(gate_ld), _i(first_row),
                _i(chunk or 0), _i(n_v), _stream()))

        single = 0
        if host_query_start and max_query_len > 1 and len(host_query_start) == n_requests + 1:
            while single < n_requests and host_query_start[single + 1] - host_query_start[single] == 1:
                single += 1
        if 0 < single < n_requests:
            run_any(0, single, 1, single)
            run_any(single, n_requests, max_query_len, n, single)
        else:
            run_any(0, n_requests, max_query_len, n)
        return
    general = modified or value_dim != head_dim or bool(chunk) or shared_values      # (the unrolled tensor-core kernels take the sink and the gate, not these)
    if general or q.dtype != torch.bfloat16 or not lib.ms_attention_mma_supports(_i(head_dim)):
        _check(lib.ms_paged_attention_generic(
            _ptr(q), _i(_code(q.dtype)), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _i(block_tables.shape[1]),
            _ptr(request_of_token), _ptr(positions), _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim),
            _f(scale), _i(window if window else 0), _f(softcap if softcap else 0.0), _ptr(bias_slopes), _ptr(out),
            _i(n), _i(value_dim), _i(1 if sink else 0), gate_ptr, _i(gate_ld), _i(chunk or 0), _i(n_v), _stream()))
        return

    def run(first: int, last: int, longest: int, rows: int, first_row: int = 0) -> None:
        """Requests first .. last - 1 (their tokens are found through query_start, which holds absolute rows);
        ``rows``: one past the last row of the batch that these requests own, which sizes the scratch of the
        key splits and the merge that follows them; ``first_row``: their first row (the merge leaves the rows
        before it alone: they belong to the requests of another launch)."""
        tables, starts, lens = block_tables[first:last], query_start[first:last + 1], context_lens[first:last]
        count = last - first
        group = n_q // n_kv
        if (USE_TCGEN05_ATTENTION and longest * group > 16 and (ATTENTION_IN_TURNS or not (sink or gate is not None))
                and lib.ms_attention_tcgen05_supports(_i(head_dim), _i(n_q), _i(n_kv), _i(k_pool.shape[2]))):
            # prompt portions: the TMA + tcgen05 + tensor-memory kernel, its softmax groups taking the key tiles in
            # turn (that form also takes the sink and the gate) or working on each together
            if ATTENTION_IN_TURNS:
                _check(lib.ms_paged_attention_turns(
                    _ptr(q), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[0]), _ptr(tables), _i(block_tables.shape[1]),
                    _ptr(starts), _ptr(lens), _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale),
                    _i(window if window else 0), _ptr(out), _i(count), _i(longest), _i(n),
                    _ptr(device_error_flag(q.device)), _i(1 if sink else 0), gate_ptr, _i(gate_ld), _stream()))
                return
            _check(lib.ms_paged_attention_tcgen05(
                _ptr(q), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[0]), _ptr(tables), _i(block_tables.shape[1]),
                _ptr(starts), _ptr(lens), _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale),
                _i(window if window else 0), _ptr(out), _i(count), _i(longest), _i(n),
                _ptr(device_error_flag(q.device)), _stream()))
            return
        splits = lib.ms_attention_mma_splits(_i(head_dim), _i(count), _i(n_kv), _i(n_q), _i(longest), _i(max_context_len))
        part_o = part_lse = None
        if splits > 1:
            part_o = torch.empty((rows * n_q * splits, head_dim), dtype=torch.float32, device=q.device)
            part_lse = torch.empty((rows * n_q * splits,), dtype=torch.float32, device=q.device)
        _check(lib.ms_paged_attention_mma(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(tables), _i(block_tables.shape[1]), _ptr(starts), _ptr(lens),
            _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale), _i(window if window else 0), _ptr(out),
            _ptr(part_o), _ptr(part_lse), _i(splits), _i(count), _i(longest), _i(rows), _i(1 if sink else 0), gate_ptr,
            _i(gate_ld), _i(first_row), _stream()))

    leading_single = 0
    if host_query_start and max_query_len > 1 and len(host_query_start) == n_requests + 1:
        while (leading_single < n_requests
               and host_query_start[leading_single + 1] - host_query_start[leading_single] == 1):
            leading_single += 1
    if 0 < leading_single < n_requests:
        run(0, leading_single, 1, leading_single)      # single tokens are the batch's first rows, one each
        run(leading_single, n_requests, max_query_len, n, leading_single)
    else:
        run(0, n_requests, max_query_len, n)


FUSED_DECODE_ATTENTION = __import__("os").environ.get("MINISERVE_B200_FUSED_DECODE_ATTENTION", "1") == "1"


# Steps of this many requests run :func:`decode_attention_fused` where it takes the sizes.  Measured at Qwen3-1.7B
# sizes, context 4,096 (ms per step with / without): 1 request 1.341 / 1.330, 2: 1.370 / 1.366, 4: 1.490 / 1.549,
# 8: 1.731 / 1.801, 16: 2.807 / 2.789, 64: 6.441 / 6.371.  With one or two requests there are few blocks and each
# repeats the queries' norm and rotation; with many the kernel's larger register count costs residency.
FUSED_DECODE_ROWS = (3, 8)


def decode_attention_fused_supported(dtype: torch.dtype, head_dim: int, n_q: int, n_kv: int) -> bool:
    """Whether :func:`decode_attention_fused` takes these sizes (bfloat16, head size 64 or 128, at most 16
    query heads per key/value head); MINISERVE_B200_FUSED_DECODE_ATTENTION=0 turns it off."""
    return bool(FUSED_DECODE_ATTENTION and dtype == torch.bfloat16
                and library().ms_attention_decode_fused_supports(_i(head_dim), _i(n_q), _i(n_kv)))


def decode_attention_fused_preferred(rows: int) -> bool:
    """Whether a step of ``rows`` single tokens is faster with :func:`decode_attention_fused` (see FUSED_DECODE_ROWS)."""
    return FUSED_DECODE_ROWS[0] <= rows <= FUSED_DECODE_ROWS[1]


def decode_attention_fused(qkv: torch.Tensor, slots: torch.Tensor, q_weight: Optional[torch.Tensor],
                           k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                           k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                           query_start: torch.Tensor, context_lens: torch.Tensor, max_context_len: int, scale: float,
                           window: Optional[int], n_q: int, n_kv: int, head_dim: int, out: torch.Tensor) -> None:
    """A decode step's attention for requests of ONE new token each, from the projection's output: what
    :func:`qk_norm_rope_append` followed by :func:`paged_attention` computes (per-head RMSNorm of q and k,
    half-split rotation over the whole head, the append of k and v at ``slots``, attention over the cache with the
    keys split over many blocks, and the merge of the splits), with the first of the three kernels folded into
    the second.  Arguments as there; ``cos_sin`` float32 ``[N, d / 2, 2]`` or None; ``max_context_len`` an upper
    bound that the split count is derived from."""
    n = qkv.shape[0]
    _want(qkv, "qkv", torch.bfloat16, (n, (n_q + 2 * n_kv) * head_dim))
    _want(slots, "slots", torch.int32, (n,))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[3] != head_dim:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, {n_kv}, page_size, {head_dim}]")
    _want(out, "out", torch.bfloat16, (n, n_q, head_dim))
    _want(block_tables, "block_tables", torch.int32)
    _want(query_start, "query_start", torch.int32, (n + 1,))
    _want(context_lens, "context_lens", torch.int32, (n,))
    weight_code = 0
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _want(weight, name, None, (head_dim,))
            weight_code = _code(weight.dtype)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share one element type")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (n, head_dim // 2, 2))
    lib = library()
    splits = lib.ms_attention_decode_fused_splits(_i(head_dim), _i(n), _i(n_kv), _i(max_context_len))
    part_o = part_lse = None
    if splits > 1:
        part_o = torch.empty((n * n_q * splits, head_dim), dtype=torch.float32, device=qkv.device)
        part_lse = torch.empty((n * n_q * splits,), dtype=torch.float32, device=qkv.device)
    _check(lib.ms_attention_decode_fused(
        _ptr(qkv), _ptr(slots), _ptr(q_weight), _ptr(k_weight), _i(weight_code), _f(eps), _ptr(cos_sin), _ptr(k_pool),
        _ptr(v_pool), _ptr(block_tables), _i(block_tables.shape[1]), _ptr(query_start), _ptr(context_lens),
        _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale), _i(window if window else 0), _ptr(out),
        _ptr(part_o), _ptr(part_lse), _i(splits), _i(n), _stream()))



# --------------------------------------------------------------------------- latent attention


def latent_prepare(proj: torch.Tensor, q_col: int, dkv_col: int, heads: int, dim: int, rot: int, rank: int,
                   slots: torch.Tensor, norm_weight: torch.Tensor, eps: float, cos_sin: Optional[torch.Tensor],
                   rot_dims: int, cache: torch.Tensor, q_full: torch.Tensor) -> None:
    """What a latent-attention layer does between its input projection and its attention, for every token:
    the latent ``proj[n, dkv_col : dkv_col + rank]`` is RMS-normed with ``norm_weight`` and, followed by the rotated
    key part ``proj[n, dkv_col + rank : + rot]``, written to row ``slots[n]`` of ``cache [pages, page_size, rank + rot]``
    (negative slot: no write); the rotated part of every query head (``proj[n, q_col + h (dim + rot) + dim : + rot]``)
    is rotated into ``q_full[n, h, rank:]``.  The rotation acts on the first ``rot_dims`` entries of a rotated part,
    entry i paired with i + rot_dims / 2, by ``cos_sin`` float32 ``[N, rot_dims / 2, 2]``."""
    n, ld = proj.shape
    _want(proj, "proj")
    _want(slots, "slots", torch.int32, (n,))
    _want(norm_weight, "norm_weight", None, (rank,))
    _want(cache, "cache", proj.dtype)
    if cache.dim() != 3 or cache.shape[2] != rank + rot:
        raise KernelError(f"cache shape {tuple(cache.shape)} is not [pages, page_size, {rank + rot}]")
    _want(q_full, "q_full", proj.dtype, (n, heads, rank + rot))
    if q_col + heads * (dim + rot) > ld or dkv_col + rank + rot > ld:
        raise KernelError(f"latent_prepare: the projections do not fit rows of {ld} numbers")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (n, rot_dims // 2, 2))
    else:
        rot_dims = 0
    _check(library().ms_latent_prepare(_ptr(proj), _i(_code(proj.dtype)), _i(ld), _i(q_col), _i(dkv_col), _i(heads), _i(dim),
                                       _i(rot), _i(rank), _ptr(slots), _ptr(norm_weight), _i(_code(norm_weight.dtype)), _f(eps),
                                       _ptr(cos_sin), _i(rot_dims), _ptr(cache), _ptr(q_full), _i(n), _stream()))


def latent_attention_kernels(dtype: torch.dtype, rank: int, rot: int, heads: int, page_size: int) -> dict:
    """Which kernel :func:`latent_attention` runs for these sizes, as :func:`attention_kernels` says it for keys and
    values: ``{"decode": name, "prompt": name}`` with ``mma.sync`` or ``general``."""
    if dtype == torch.bfloat16 and USE_LATENT_MMA and library().ms_latent_attention_mma_supports(_i(rank), _i(rot), _i(heads)):
        return {"decode": "mma.sync", "prompt": "mma.sync"}
    return {"decode": "general", "prompt": "general"}


USE_LATENT_MMA = __import__("os").environ.get("MINISERVE_B200_LATENT_MMA", "1") == "1"


def latent_attention(q_full: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, request_of_token: torch.Tensor,
                     positions: torch.Tensor, query_start: torch.Tensor, context_lens: torch.Tensor, max_query_len: int,
                     max_context_len: int, rank: int, scale: float, window: Optional[int], out: torch.Tensor) -> None:
    """Causal attention of every token's heads over its request's cached rows ``[c ; k_r]``: the score of head h is
    ``q_full[n, h] . row * scale``, the result the softmax-weighted sum of the rows' first ``rank`` numbers.

    q_full ``[N, H, rank + rot]``; cache of one layer ``[pages, page_size, rank + rot]``; out ``[N, H, rank]``; the
    batch is described as for :func:`paged_attention`.  bfloat16 with sizes that the tensor-core kernel takes runs
    there; everything else runs the general float32-arithmetic kernel."""
    n, heads, dk = q_full.shape
    _want(q_full, "q_full")
    _want(cache, "cache", q_full.dtype)
    if cache.dim() != 3 or cache.shape[2] != dk:
        raise KernelError(f"cache shape {tuple(cache.shape)} is not [pages, page_size, {dk}]")
    _want(out, "out", q_full.dtype, (n, heads, rank))
    _want(block_tables, "block_tables", torch.int32)
    _want(request_of_token, "request_of_token", torch.int32, (n,))
    _want(positions, "positions", torch.int32, (n,))
    n_requests = context_lens.numel()
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    _want(context_lens, "context_lens", torch.int32, (n_requests,))
    lib = library()
    page_size = cache.shape[1]
    if q_full.dtype == torch.bfloat16 and USE_LATENT_MMA and lib.ms_latent_attention_mma_supports(_i(rank), _i(dk - rank), _i(heads)):
        splits = lib.ms_latent_attention_mma_splits(_i(rank), _i(dk - rank), _i(heads), _i(n_requests), _i(max_query_len),
                                                    _i(max_context_len))
        part_o = part_lse = None
        if splits > 1:
            part_o = torch.empty((n * heads * splits, rank), dtype=torch.float32, device=q_full.device)
            part_lse = torch.empty((n * heads * splits,), dtype=torch.float32, device=q_full.device)
        _check(lib.ms_latent_attention_mma(
            _ptr(q_full), _ptr(cache), _ptr(block_tables), _i(block_tables.shape[1]), _ptr(query_start), _ptr(context_lens),
            _i(page_size), _i(heads), _i(rank), _i(dk - rank), _f(scale), _i(window if window else 0), _ptr(out),
            _ptr(part_o), _ptr(part_lse), _i(splits), _i(n_requests), _i(max_query_len), _i(n), _stream()))
        return
    _check(lib.ms_latent_attention_generic(
        _ptr(q_full), _i(_code(q_full.dtype)), _ptr(cache), _ptr(block_tables), _i(block_tables.shape[1]),
        _ptr(request_of_token), _ptr(positions), _i(page_size), _i(heads), _i(dk), _i(rank), _f(scale),
        _i(window if window else 0), _ptr(out), _i(n), _stream()))


def head_gate(x: torch.Tensor, gate: torch.Tensor, gate_col: int) -> None:
    """In place on ``x [N, H, vdim]``: head h of token n is multiplied by ``sigmoid(gate[n, gate_col + h])``."""
    n, heads, vdim = x.shape
    _want(x, "x")
    _want(gate, "gate", x.dtype)
    if gate.dim() != 2 or gate.shape[0] != n or gate_col + heads > gate.shape[1]:
        raise KernelError(f"head_gate: gate logits {tuple(gate.shape)} for {n} tokens of {heads} heads from column {gate_col}")
    _check(library().ms_head_gate(_ptr(x), gate.data_ptr() + gate_col * gate.element_size(), _i(_code(x.dtype)),
                                  _i(gate.shape[1]), _i(heads), _i(vdim), _i(n), _stream()))


def linear_batched(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out[b] = x[b] @ weight[b]^T`` for ``x [B, M, K]``, ``weight [B, N, K]``, ``out [B, M, N]``; ``x`` and ``out`` may be
    strided views (a head's columns of wider rows) as long as their last dimension is dense.  float32 runs the
    library's own FFMA kernel (one thread per output element, k ascending); bfloat16 goes to cuBLAS (``torch.bmm``)."""
    b, m, k = x.shape
    n = weight.shape[1]
    if weight.shape != (b, n, k) or out.shape != (b, m, n) or x.stride(2) != 1 or out.stride(2) != 1 or not weight.is_contiguous():
        raise KernelError(f"linear_batched: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if x.dtype == torch.float32:
        if weight.dtype != torch.float32 or out.dtype != torch.float32 or not (x.is_cuda and weight.is_cuda and out.is_cuda):
            raise KernelError("linear_batched: float32 CUDA tensors expected")
        _check(library().ms_gemm_f32_batched(_ptr(x), _ptr(weight), _ptr(out), _i(m), _i(n), _i(k), _i(x.stride(1)), _i(k),
                                             _i(out.stride(1)), _i(b), x.stride(0), n * k, out.stride(0), _stream()))
        return
    torch.bmm(x, weight.transpose(1, 2), out=out)


# --------------------------------------------------------------------------- state-space mixer

MAX_SCAN_STATE = 256     # numbers of state per channel that selective_scan keeps in registers (8 lanes x 32)
MAX_CONV_TAPS = 8


def _state_rows(states: torch.Tensor, offset: int, length: int) -> int:
    _want(states, "states", torch.float32)
    if states.dim() != 2 or offset < 0 or offset + length > states.shape[1]:
        raise KernelError(f"states {tuple(states.shape)} do not hold {length} numbers from column {offset} per slot")
    return states.shape[1]


CONV_ACTIVATIONS = {"none": 0, "silu": 1}


def causal_conv_silu(proj: torch.Tensor, col: int, weight: torch.Tensor, bias: torch.Tensor, states: torch.Tensor,
                     state_offset: int, state_slots: torch.Tensor, query_start: torch.Tensor, max_query_len: int,
                     out: torch.Tensor) -> None:
    """:func:`causal_conv` with a bias and SiLU."""
    causal_conv(proj, col, weight, bias, states, state_offset, state_slots, query_start, max_query_len, out)


def causal_conv(proj: torch.Tensor, col: int, weight: torch.Tensor, bias: Optional[torch.Tensor], states: torch.Tensor,
                state_offset: int, state_slots: torch.Tensor, query_start: torch.Tensor, max_query_len: int,
                out: torch.Tensor, activation: str = "silu", in_bias: Optional[torch.Tensor] = None) -> None:
    """Causal convolution per channel, then the activation (``"silu"`` or ``"none"``), over each request's tokens, continued
    from the request's state: ``out[t, c] = act(bias[c] + sum_k weight[c, k] * u[t - (taps - 1 - k), c])`` with ``u`` the
    columns ``col .. col + channels`` of ``proj [N, ld]`` (plus ``in_bias[c]``, float32 ``[channels]``: the bias of the
    projection that made them; the zeros before a sequence's start do not get it); inputs before the portion come from
    ``states[slot, state_offset:]`` (float32 ``[taps - 1, channels]``, oldest first), which afterwards holds the last
    ``taps - 1`` inputs seen.  ``weight`` float32 ``[channels, taps]``, ``bias`` float32 ``[channels]`` or None;
    ``state_slots`` int32 ``[R]``, ``query_start`` int32 ``[R + 1]``; ``out [N, channels]`` float32 or of ``proj``'s type."""
    n, ld = proj.shape
    channels, taps = weight.shape
    _want(proj, "proj")
    _want(weight, "weight", torch.float32)
    for name, tensor in (("bias", bias), ("in_bias", in_bias)):
        if tensor is not None:
            _want(tensor, name, torch.float32, (channels,))
    _want(out, "out", None, (n, channels))
    if out.dtype not in (torch.float32, proj.dtype):
        raise KernelError(f"causal_conv: out is float32 or {proj.dtype}, got {out.dtype}")
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    if col < 0 or col + channels > ld or not 1 <= taps <= MAX_CONV_TAPS:
        raise KernelError(f"causal_conv_silu: {channels} channels from column {col} of rows of {ld}, {taps} taps")
    stride = _state_rows(states, state_offset, (taps - 1) * channels)
    _check(library().ms_causal_conv(_ptr(proj), _i(_code(proj.dtype)), _i(ld), _i(col), _i(channels), _i(taps), _ptr(weight),
                                    _ptr(bias), _ptr(in_bias), _i(CONV_ACTIVATIONS[activation]), _ptr(states), stride,
                                    _i(state_offset), _ptr(state_slots), _ptr(query_start), _i(n_requests), _i(max_query_len),
                                    _ptr(out), _i(0 if out.dtype == torch.float32 else 1), _stream()))


def selective_scan(conv: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
                   d: torch.Tensor, states: torch.Tensor, state_offset: int, state_slots: torch.Tensor,
                   query_start: torch.Tensor, heads: int, head_dim: int, state: int, groups: int, y: torch.Tensor,
                   max_query_len: Optional[int] = None) -> None:
    """The selective recurrence over each request's tokens, from and into the request's state.  ``conv`` float32
    ``[N, heads * head_dim + 2 * groups * state]`` = ``[x | B | C]``; the step size of head h is ``softplus(proj[t,
    dt_col + h] + dt_bias[h])``; per head (group ``h // (heads / groups)``) ``S = exp(-exp(a_log) dt) S + dt B x^T`` and
    ``y = S^T C + d x``.  ``states[slot, state_offset:]`` holds float32 ``[heads, head_dim, state]``.  ``y`` float32
    ``[N, heads * head_dim]``.  ``max_query_len``: an upper bound of the tokens a request brings (None: the batch's size); the
    kernel sizes its chunks by it, so a step of single tokens should say 1."""
    n, ld = proj.shape
    inner = heads * head_dim
    _want(proj, "proj")
    _want(conv, "conv", torch.float32, (n, inner + 2 * groups * state))
    for name, tensor in (("dt_bias", dt_bias), ("a_log", a_log), ("d", d)):
        _want(tensor, name, torch.float32, (heads,))
    _want(y, "y", torch.float32, (n, inner))
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    if dt_col < 0 or dt_col + heads > ld or heads % groups or state > MAX_SCAN_STATE:
        raise KernelError(f"selective_scan: {heads} heads in {groups} groups, state {state}, dt from column {dt_col} of rows of {ld}")
    stride = _state_rows(states, state_offset, inner * state)
    _check(library().ms_selective_scan(_ptr(conv), _i(conv.shape[1]), _ptr(proj), _i(_code(proj.dtype)), _i(ld), _i(dt_col),
                                       _ptr(dt_bias), _ptr(a_log), _ptr(d), _ptr(states), stride, _i(state_offset),
                                       _ptr(state_slots), _ptr(query_start), _i(n_requests), _i(n if max_query_len is None else max_query_len),
                                       _i(heads), _i(head_dim), _i(state), _i(groups), _ptr(y), _stream()))


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, z_col: int, weight: torch.Tensor, groups: int, eps: float,
                     out: torch.Tensor) -> None:
    """``v = y * silu(z)`` with ``z`` the columns ``z_col .. z_col + inner`` of ``proj``; ``out = weight * v / rms(v)``,
    the root mean square taken over each of ``groups`` equal parts of a row.  ``y`` float32 ``[N, inner]``, ``weight``
    float32 ``[inner]``, ``out [N, inner]`` in ``proj``'s type."""
    n, inner = y.shape
    _want(y, "y", torch.float32)
    _want(proj, "proj")
    _want(weight, "weight", torch.float32, (inner,))
    _want(out, "out", proj.dtype, (n, inner))
    if proj.shape[0] != n or z_col < 0 or z_col + inner > proj.shape[1] or groups < 1 or inner % groups:
        raise KernelError(f"gated_group_norm: {inner} channels in {groups} groups, z from column {z_col} of {tuple(proj.shape)}")
    _check(library().ms_gated_group_norm(_ptr(y), _ptr(proj), _i(_code(proj.dtype)), _i(proj.shape[1]), _i(z_col), _ptr(weight),
                                         _i(groups), _i(inner), _f(eps), _ptr(out), _i(n), _stream()))


# --------------------------------------------------------------------------- recurrences that carry a matrix or a vector

MAX_MATRIX_SCAN_DIM = 512     # entries of a query or key that matrix_scan spreads over a column's lanes (16 lanes x 32)
MATRIX_SCAN_MODES = {"memory": 0, "delta": 1, "decay": 2, "channel_delta": 3}
HEAD_GATE_ACTIVATIONS = {"sigmoid": 0, "silu": 1}


def small_linear_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out[n, r] = sum_c x[n, c] weight[r, c] + bias[r]`` in float32 for a float32 weight of few rows (gate logits of a
    recurrence: what the router's logits are to a mixture); ``x`` in the compute type, ``out`` float32 ``[N, R]``."""
    n, width = x.shape
    rows = weight.shape[0]
    _want(x, "x")
    _want(weight, "weight", torch.float32, (rows, width))
    if bias is not None:
        _want(bias, "bias", torch.float32, (rows,))
    _want(out, "out", torch.float32, (n, rows))
    _check(library().ms_small_linear_f32(_ptr(x), _i(_code(x.dtype)), _ptr(weight), _ptr(bias), _i(width), _i(rows), _ptr(out),
                                         _i(n), _stream()))


def unit_norm_heads(x: torch.Tensor, col: int, heads: int, dim: int, eps: float, scale: float) -> None:
    """In place on float32 ``x [N, ld]``: head j's entries (columns ``col + j dim ..``) become ``scale * v / sqrt(sum v^2 +
    eps)``."""
    _want(x, "x", torch.float32)
    if x.dim() != 2 or col < 0 or col + heads * dim > x.shape[1]:
        raise KernelError(f"unit_norm_heads: {heads} heads of {dim} from column {col} of {tuple(x.shape)}")
    _check(library().ms_unit_norm_heads(_ptr(x), _i(x.shape[1]), _i(col), _i(heads), _i(dim), _f(eps), _f(scale), _i(x.shape[0]),
                                        _stream()))


def exponential_gates(logits: torch.Tensor, cap: float, states: torch.Tensor, state_offset: int, state_slots: torch.Tensor,
                      query_start: torch.Tensor, max_query_len: int, gates: torch.Tensor) -> None:
    """The gates of a matrix memory with exponential gating, stabilised by a running maximum that the request carries.
    ``logits`` float32 ``[N, 2 H]`` = ``[input | forget]``; ``i = cap tanh(x / cap)``, ``f = logsigmoid(cap tanh(x / cap))``;
    ``m_t = max(f_t + m_(t-1), i_t)`` from ``states[slot, state_offset + head]`` (which receives the last ``m``);
    ``gates [N, H, 3]`` = ``(exp(f_t + m_(t-1) - m_t), exp(i_t - m_t), exp(-m_t))``."""
    n, heads = gates.shape[0], gates.shape[1]
    _want(logits, "logits", torch.float32, (n, 2 * heads))
    _want(gates, "gates", torch.float32, (n, heads, 3))
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    stride = _state_rows(states, state_offset, heads)
    _check(library().ms_exponential_gates(_ptr(logits), _f(cap), _ptr(states), stride, _i(state_offset), _ptr(state_slots),
                                          _ptr(query_start), _i(n_requests), _i(heads), _ptr(gates), _stream()))


def decay_gates(logits: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, gates: torch.Tensor) -> None:
    """The gates of the delta rule: ``logits`` float32 ``[N, 2 H]`` = ``[b | a]``; ``gates [N, H, 2]`` = ``(exp(-exp(a_log)
    softplus(a + dt_bias)), sigmoid(b))``."""
    n, heads = gates.shape[0], gates.shape[1]
    _want(logits, "logits", torch.float32, (n, 2 * heads))
    _want(gates, "gates", torch.float32, (n, heads, 2))
    _want(a_log, "a_log", torch.float32, (heads,))
    _want(dt_bias, "dt_bias", torch.float32, (heads,))
    _check(library().ms_decay_gates(_ptr(logits), _ptr(a_log), _ptr(dt_bias), _ptr(gates), _i(n), _i(heads), _stream()))


def matrix_scan(mode: str, q: torch.Tensor, q_col: int, k: torch.Tensor, k_col: int, v: torch.Tensor, v_col: int,
                gates: torch.Tensor, states: torch.Tensor, state_offset: int, state_slots: torch.Tensor,
                query_start: torch.Tensor, max_query_len: int, heads: int, kv_heads: int, dim: int, vdim: int, y: torch.Tensor,
                q_scale: float = 1.0, bottom: Optional[torch.Tensor] = None, gate_col: int = 0,
                channel_decay: Optional[torch.Tensor] = None, input_activation: str = "none") -> None:
    """A recurrence that carries a ``dim x vdim`` matrix ``S`` per head, walked over each request's tokens from and into the
    request's state.  Queries and keys of head j are the columns ``q_col + (j // (heads / kv_heads)) dim ..`` of ``q`` (and
    ``k``), its values the columns ``v_col + j vdim ..`` of ``v`` (``q``, ``k``, ``v``: one 2-d tensor, float32 or the compute
    type; the queries are multiplied by ``q_scale``).

    ``"memory"``: ``gates [N, H, 3]`` = (keep, write, floor); ``S = keep S + write k v^T``, ``n = keep n + write k``, ``y = S^T q``
    and ``bottom [N, H] = max(|n . q|, floor) + 1e-6``.  The state holds ``[H, vdim + 1, dim]``: the columns of ``S``, then ``n``.
    ``"delta"``: ``gates [N, H, 2]`` = (decay, beta); ``S = decay S``, ``u = beta (v - S^T k)``, ``S = S + k u^T``, ``y = S^T q``.
    The state holds ``[H, vdim, dim]``.  ``y`` float32 ``[N, H, vdim]``.
    ``"decay"``: ``gates [H]``, a constant decay per head; ``S = decay S + k v^T``, ``y = S^T q`` (a linear attention).
    ``"channel_delta"``: the delta form with a decay per head and key channel, ``channel_decay`` float32 ``[N, H * dim]``, acting on
    the rows of ``S``; ``gates`` is float32 ``[N, ld]`` whose columns ``gate_col .. gate_col + H`` hold the logits of beta.  Both
    keep ``[H, vdim, dim]``.  ``input_activation="silu"``: q, k and v pass SiLU as they are read."""
    code = MATRIX_SCAN_MODES[mode]
    n = y.shape[0]
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        _want(tensor, name)
        if tensor.dim() != 2 or tensor.shape[0] != n or tensor.dtype != q.dtype:
            raise KernelError(f"matrix_scan: {name} {tuple(tensor.shape)} {tensor.dtype} for {n} tokens")
    if (heads % kv_heads or q_col < 0 or k_col < 0 or v_col < 0 or q_col + kv_heads * dim > q.shape[1]
            or k_col + kv_heads * dim > k.shape[1] or v_col + heads * vdim > v.shape[1] or not 1 <= dim <= MAX_MATRIX_SCAN_DIM):
        raise KernelError(f"matrix_scan: {heads}/{kv_heads} heads of {dim}/{vdim} at columns {q_col}, {k_col}, {v_col}")
    gate_ld = 0
    if code == 2:
        _want(gates, "gates", torch.float32, (heads,))
    elif code == 3:
        _want(gates, "gates", torch.float32)
        _want(channel_decay, "channel_decay", torch.float32, (n, heads * dim))
        if gates.dim() != 2 or gates.shape[0] != n or gate_col < 0 or gate_col + heads > gates.shape[1]:
            raise KernelError(f"matrix_scan: the logits of beta from column {gate_col} of {tuple(gates.shape)} for {heads} heads")
        gate_ld = gates.shape[1]
    else:
        _want(gates, "gates", torch.float32, (n, heads, 3 if code == 0 else 2))
    _want(y, "y", torch.float32, (n, heads, vdim))
    if code == 0:
        _want(bottom, "bottom", torch.float32, (n, heads))
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    columns = vdim + 1 if code == 0 else vdim
    stride = _state_rows(states, state_offset, heads * columns * dim)
    _check(library().ms_matrix_scan(_i(code), _ptr(q), _i(q.shape[1]), _i(q_col), _ptr(k), _i(k.shape[1]), _i(k_col), _ptr(v),
                                    _i(v.shape[1]), _i(v_col), _i(_code(q.dtype)), _f(q_scale), _ptr(gates), _ptr(states), stride,
                                    _i(state_offset), _ptr(state_slots), _ptr(query_start), _i(n_requests), _i(max_query_len),
                                    _i(heads), _i(kv_heads), _i(dim), _i(vdim), _ptr(y), _ptr(bottom), _i(gate_ld), _i(gate_col),
                                    _ptr(channel_decay) if code == 3 else None, _i(CONV_ACTIVATIONS[input_activation]), _stream()))


def channel_decays(logits: torch.Tensor, col: int, a_log: torch.Tensor, dt_bias: torch.Tensor, per_head: int, out: torch.Tensor) -> None:
    """``out[n, r] = exp(-exp(a_log[r // per_head]) softplus(logits[n, col + r] + dt_bias[r]))``: a decay per head and channel
    from float32 logits ``[N, ld]``; ``out`` float32 ``[N, R]``."""
    n, ld = logits.shape
    rows = out.shape[1]
    _want(logits, "logits", torch.float32)
    _want(out, "out", torch.float32, (n, rows))
    _want(a_log, "a_log", torch.float32, (rows // max(per_head, 1),))
    _want(dt_bias, "dt_bias", torch.float32, (rows,))
    _check(library().ms_low_rank_expand(_ptr(logits), _i(ld), _i(col), _i(rows), None, _i(rows), _i(1), _ptr(a_log), _ptr(dt_bias),
                                        _i(per_head), _ptr(out), _i(0), _i(n), _stream()))


def low_rank_expand(mid: torch.Tensor, col: int, weight_t: torch.Tensor, out: torch.Tensor, a_log: Optional[torch.Tensor] = None,
                    bias: Optional[torch.Tensor] = None, per_head: int = 0) -> None:
    """The second product of a projection made in two steps: ``value[n, r] = sum_j mid[n, col + j] weight_t[j, r]`` with ``mid``
    float32 ``[N, ld]`` and ``weight_t`` float32 ``[rank, R]``, the second matrix TRANSPOSED (the kernel's threads then read
    consecutive numbers).  Without ``a_log``: ``out [N, R]`` (any type) receives the values.
    With ``a_log`` (float32 ``[R / per_head]``) and ``bias`` (float32 ``[R]``): ``out`` float32 receives the decays
    ``exp(-exp(a_log[r // per_head]) softplus(value + bias[r]))``."""
    n, ld = mid.shape
    rank, rows = weight_t.shape
    _want(mid, "mid", torch.float32)
    _want(weight_t, "weight_t", torch.float32)
    decay = a_log is not None
    if decay:
        _want(a_log, "a_log", torch.float32, (rows // max(per_head, 1),))
        _want(bias, "bias", torch.float32, (rows,))
    _want(out, "out", torch.float32 if decay else None, (n, rows))
    _check(library().ms_low_rank_expand(_ptr(mid), _i(ld), _i(col), _i(rank), _ptr(weight_t), _i(rows), _i(1 if decay else 0),
                                        _ptr(a_log), _ptr(bias), _i(per_head), _ptr(out), _i(_code(out.dtype)), _i(n), _stream()))


def head_norm_gate(y: torch.Tensor, bottom: Optional[torch.Tensor], weight: torch.Tensor, gate: torch.Tensor, gate_col: int,
                   activation: str, eps: float, out: torch.Tensor) -> None:
    """``v = y / bottom`` (per token and head; ``bottom`` None: ``y`` itself), each head divided by its root mean square
    (``eps`` inside the root), times ``weight`` (float32: ``[H * vdim]``, or ``[vdim]`` shared by the heads), times
    ``act(gate[n, gate_col + j])`` with ``act`` ``"sigmoid"`` or ``"silu"``.  ``y`` float32 ``[N, H, vdim]``; ``gate`` and ``out [N, H *
    vdim]`` in the compute type."""
    n, heads, vdim = y.shape
    _want(y, "y", torch.float32)
    if bottom is not None:
        _want(bottom, "bottom", torch.float32, (n, heads))
    _want(weight, "weight", torch.float32)
    if weight.numel() not in (vdim, heads * vdim):
        raise KernelError(f"head_norm_gate: a weight of {weight.numel()} numbers for {heads} heads of {vdim}")
    _want(gate, "gate")
    _want(out, "out", gate.dtype, (n, heads * vdim))
    if gate.dim() != 2 or gate.shape[0] != n or gate_col < 0 or gate_col + heads * vdim > gate.shape[1]:
        raise KernelError(f"head_norm_gate: gate {tuple(gate.shape)} from column {gate_col} for {heads} heads of {vdim}")
    _check(library().ms_head_norm_gate(_ptr(y), _ptr(bottom), _ptr(weight), _i(1 if weight.numel() == heads * vdim and heads > 1 else 0),
                                       _ptr(gate), _i(_code(gate.dtype)), _i(gate.shape[1]), _i(gate_col),
                                       _i(HEAD_GATE_ACTIVATIONS[activation]), _f(eps), _ptr(out), _i(n), _i(heads), _i(vdim), _stream()))


def gated_recurrence_scan(u: torch.Tensor, pre: torch.Tensor, gate_bias: torch.Tensor, rate: torch.Tensor, proj: torch.Tensor,
                          y_col: int, y_bias: Optional[torch.Tensor], states: torch.Tensor, state_offset: int,
                          state_slots: torch.Tensor, query_start: torch.Tensor, max_query_len: int, out: torch.Tensor) -> None:
    """The real-gated linear recurrence per channel over each request's tokens, from and into the request's state:
    ``r = sigmoid(pre[0] + gate_bias[0])``, ``i = sigmoid(pre[1] + gate_bias[1])``, ``log a = rate r``, ``S = a S + sqrt(1 - a^2)
    i u``, and ``out = S gelu_tanh(proj[:, y_col + c] + y_bias[c])``.  ``u`` float32 ``[N, W]``, ``pre`` float32 ``[2, N, W]``,
    ``gate_bias`` float32 ``[2, W]``, ``rate`` float32 ``[W]`` (negative), ``states[slot, state_offset:]`` float32 ``[W]``; ``out [N,
    W]`` in ``proj``'s type."""
    n, width = u.shape
    _want(u, "u", torch.float32)
    _want(pre, "pre", torch.float32, (2, n, width))
    _want(gate_bias, "gate_bias", torch.float32, (2, width))
    _want(rate, "rate", torch.float32, (width,))
    _want(proj, "proj")
    if y_bias is not None:
        _want(y_bias, "y_bias", torch.float32, (width,))
    _want(out, "out", proj.dtype, (n, width))
    if proj.dim() != 2 or proj.shape[0] != n or y_col < 0 or y_col + width > proj.shape[1]:
        raise KernelError(f"gated_recurrence_scan: {width} channels from column {y_col} of {tuple(proj.shape)}")
    n_requests = state_slots.numel()
    _want(state_slots, "state_slots", torch.int32)
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    stride = _state_rows(states, state_offset, width)
    _check(library().ms_gated_recurrence_scan(_ptr(u), _ptr(pre), _ptr(gate_bias), _ptr(rate), _ptr(proj), _i(_code(proj.dtype)),
                                              _i(proj.shape[1]), _i(y_col), _ptr(y_bias), _ptr(states), stride, _i(state_offset),
                                              _ptr(state_slots), _ptr(query_start), _i(n_requests), _i(n), _i(width),
                                              _ptr(out), _stream()))


# --------------------------------------------------------------------------- routed experts


def router_topk(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor,
                weights: torch.Tensor, logits: Optional[torch.Tensor] = None, *, choose_from: Optional[int] = None,
                scoring: str = "chosen_softmax", correction: Optional[torch.Tensor] = None, groups: tuple = (1, 1)) -> None:
    """Router of a mixture of experts: float32 logits ``x @ weight^T + bias`` (``weight`` float32 ``[E, width]``), the
    ``top`` experts with the largest logits into ``ids`` int32 ``[N, top]`` (ties: the lower index) and the softmax over
    those logits alone into ``weights`` float32 ``[N, top]``.  ``logits`` float32 ``[N, E]``: scratch that is left holding
    the logits (allocated here if not given).

    ``scoring="all_softmax"``: scores are the softmax over the first ``choose_from`` logits of a row (all, if None;
    further rows of ``weight`` only ride along in the product and leave their logits in ``logits``); the choice goes by
    ``score + correction`` (float32 ``[choose_from]`` or None) among the members of the ``groups[1]`` best of
    ``groups[0]`` equal groups of neighbours (a group's score: its largest choice score), and ``weights`` are the chosen
    outputs' scores as they are.  ``scoring="sigmoid"``: the same with ``sigmoid(logit)`` of every output on its own as its
    score."""
    n, width = x.shape
    experts = weight.shape[0]
    if scoring in ("all_softmax", "sigmoid"):
        total = experts if choose_from is None else choose_from
        if logits is None:
            logits = torch.empty((n, experts), dtype=torch.float32, device=x.device)
        _want(logits, "logits", torch.float32, (n, experts))
        _want(x, "x")
        _want(weight, "weight", torch.float32, (experts, width))
        if bias is not None:
            _want(bias, "bias", torch.float32, (experts,))
        if correction is not None:
            _want(correction, "correction", torch.float32, (total,))
        _want(ids, "ids", torch.int32, (n, top))
        _want(weights, "weights", torch.float32, (n, top))
        _check(library().ms_router_choose(_ptr(x), _i(_code(x.dtype)), _ptr(weight), _ptr(bias), _i(width), _i(experts), _i(total),
                                          _i(top), _ptr(correction), _i(groups[0]), _i(groups[1]), _ptr(logits), _ptr(ids),
                                          _ptr(weights), _i(n), _i(1 if scoring == "sigmoid" else 0), _stream()))
        return
    if scoring != "chosen_softmax" or correction is not None or tuple(groups) != (1, 1) or choose_from not in (None, experts):
        raise KernelError("router_topk: a correction, groups and rows that ride along need scoring='all_softmax'")
    if logits is None:
        logits = torch.empty((n, experts), dtype=torch.float32, device=x.device)
    _want(logits, "logits", torch.float32, (n, experts))
    _want(x, "x")
    _want(weight, "weight", torch.float32, (experts, width))
    if bias is not None:
        _want(bias, "bias", torch.float32, (experts,))
    _want(ids, "ids", torch.int32, (n, top))
    _want(weights, "weights", torch.float32, (n, top))
    _check(library().ms_router_topk(_ptr(x), _i(_code(x.dtype)), _ptr(weight), _ptr(bias), _i(width), _i(experts), _i(top),
                                    _ptr(logits), _ptr(ids), _ptr(weights), _i(n), _stream()))


def expert_route(ids: torch.Tensor, experts: int, offsets: torch.Tensor, order: torch.Tensor, place: torch.Tensor) -> None:
    """Sorts the (token, choice) pairs of ``ids [N, top]`` by expert: ``offsets`` int32 ``[E + 1]`` bounds each expert's
    segment, ``order [N * top]`` lists the pairs (token * top + choice) segment by segment, ``place`` is its inverse."""
    pairs = ids.numel()
    _want(ids, "ids", torch.int32)
    _want(offsets, "offsets", torch.int32, (experts + 1,))
    _want(order, "order", torch.int32, (pairs,))
    _want(place, "place", torch.int32, (pairs,))
    _check(library().ms_expert_route(_ptr(ids), _i(pairs), _i(experts), _ptr(offsets), _ptr(order), _ptr(place), _stream()))


EXPERT_ACTIVATIONS = {"none": 0, "relu_square": 1, "clamped_glu": 2, "silu_glu": 3}


def expert_linear(x: torch.Tensor, order: Optional[torch.Tensor], top: int, weight: torch.Tensor, out: torch.Tensor,
                  offsets: torch.Tensor, relu_square: bool = False, activation: str = "none", limit: float = 0.0,
                  pair_scale: Optional[torch.Tensor] = None) -> None:
    """One product per expert over its segment of the sorted pairs: ``out[i] = act(x[src(i)] @ weight[e]^T)`` for every
    place ``i`` of expert ``e``'s segment, ``weight [E, N, K]``, ``out [pairs, N]``.  With ``order`` the rows are gathered from
    the tokens (``src(i) = order[i] // top``, ``x [tokens, K]``), without it ``x [pairs, K]`` is in sorted order already.
    ``activation``: ``"relu_square"`` (or ``relu_square=True``): ``act(z) = max(z, 0)^2``; ``"clamped_glu"``: the rows of
    ``weight[e]`` alternate (gate row j, up row j) and ``out [pairs, N / 2]`` receives ``g sigmoid(1.702 g) (u + 1)`` with
    ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``; ``"silu_glu"``: the same layout, ``out`` receives
    ``silu(s gate) (s up)`` where ``s`` is the pair's entry of ``pair_scale`` (float32 ``[tokens, top]``, needs ``order``; 1
    without it): the expert computed on ``s`` times its input.  ``offsets`` may bound more segments than ``weight`` has
    experts (identity experts, sorted behind the others): their rows are left alone."""
    experts, n, k = weight.shape
    pairs = out.shape[0]
    if relu_square:
        activation = "relu_square"
    code = EXPERT_ACTIVATIONS[activation]
    _want(x, "x", None)
    _want(weight, "weight", x.dtype)
    _want(out, "out", x.dtype, (pairs, n // 2 if code >= 2 else n))
    if pair_scale is not None:
        if code != 3 or order is None:
            raise KernelError("expert_linear: a scale per pair goes with 'silu_glu' and rows gathered through `order`")
        _want(pair_scale, "pair_scale", torch.float32)
        if pair_scale.numel() != pairs:
            raise KernelError(f"expert_linear: {pair_scale.numel()} scales for {pairs} pairs")
    _want(offsets, "offsets", torch.int32)
    if offsets.numel() < experts + 1:
        raise KernelError(f"expert_linear: {offsets.numel()} offsets for {experts} experts")
    if x.shape[1] != k or (order is None and x.shape[0] != pairs):
        raise KernelError(f"expert_linear: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if order is not None:
        _want(order, "order", torch.int32, (pairs,))
    _check(library().ms_expert_linear(_ptr(x), _i(_code(x.dtype)), _i(k), _ptr(order), _i(top), _ptr(weight), _ptr(out),
                                      _i(out.shape[1]), _ptr(offsets), _i(experts), _i(pairs), _i(n), _i(k), _i(code), _f(limit),
                                      _ptr(pair_scale), _stream()))


def expert_combine(y: torch.Tensor, place: torch.Tensor, weights: Optional[torch.Tensor], shared: Optional[torch.Tensor],
                   out: torch.Tensor, ids: Optional[torch.Tensor] = None, first_identity: int = 0,
                   x: Optional[torch.Tensor] = None, shared_gate: Optional[torch.Tensor] = None, shared_gate_col: int = 0) -> None:
    """``out[n] = sum_k weights[n, k] * y[place[n * top + k]] (+ shared[n])``, summed in float32 in the order of k.
    With ``ids`` (int32 ``[N, top]``) a choice whose id is ``first_identity`` or more is an identity expert and adds
    ``weights[n, k] * x[n]`` instead.  With ``shared_gate`` (float32 ``[N, ld]``) the shared expert's output is multiplied
    by ``sigmoid(shared_gate[n, shared_gate_col])``.  ``weights`` None: every weight is 1 (the experts' inputs carried
    them)."""
    width = out.shape[1]
    n = out.shape[0]
    top = place.numel() // max(n, 1) if weights is None else weights.shape[1]
    _want(y, "y", out.dtype, (n * top, width))
    _want(place, "place", torch.int32, (n * top,))
    if weights is not None:
        _want(weights, "weights", torch.float32, (n, top))
    _want(out, "out", None, (n, width))
    if shared is not None:
        _want(shared, "shared", out.dtype, (n, width))
    gate_ptr, gate_ld = None, 0
    if ids is not None:
        _want(ids, "ids", torch.int32, (n, top))
        _want(x, "x", out.dtype, (n, width))
    if shared_gate is not None:
        _want(shared_gate, "shared_gate", torch.float32)
        if shared_gate.dim() != 2 or shared_gate.shape[0] != n or not 0 <= shared_gate_col < shared_gate.shape[1]:
            raise KernelError(f"expert_combine: gate logits {tuple(shared_gate.shape)}, column {shared_gate_col}, for {n} tokens")
        gate_ptr, gate_ld = shared_gate.data_ptr() + 4 * shared_gate_col, shared_gate.shape[1]
    _check(library().ms_expert_combine(_ptr(y), _i(_code(out.dtype)), _i(width), _ptr(place), _ptr(weights), _i(top), _ptr(shared),
                                       _ptr(out), _i(width), _i(n), _ptr(ids), _i(first_identity),
                                       _ptr(x) if ids is not None else None, gate_ptr, _i(gate_ld), _stream()))


def clamped_glu(both: torch.Tensor, limit: float, out: torch.Tensor) -> None:
    """``out[n, j] = g sigmoid(1.702 g) (u + 1)`` with ``g = min(both[n, 2 j], limit)`` and ``u = clamp(both[n, 2 j + 1],
    -limit, limit)``: the gated activation of a product whose weight alternates gate and up rows."""
    n, inter = out.shape
    _want(both, "both", None, (n, 2 * inter))
    _want(out, "out", both.dtype)
    _check(library().ms_clamped_glu(_ptr(both), _i(_code(both.dtype)), _ptr(out), _i(n), _i(inter), _f(limit), _stream()))


def relu_square(x: torch.Tensor) -> None:
    """In place: ``x = max(x, 0)^2``."""
    _want(x, "x")
    _check(library().ms_relu_square(_ptr(x), _i(_code(x.dtype)), x.numel(), _stream()))

# --------------------------------------------------------------------------- matrix products


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_stats: Optional["RowStats"] = None) -> None:
    """``out[M, N] = x[M, K] @ weight[N, K]^T``.  (``row_stats``: see :func:`linear_wide`; the caller has asked
    :func:`fold_supported` first.)

    float32 operands run through the library's own FFMA kernel (true 32-bit, no tensor-core
    mode).  bfloat16 operands go to cuBLAS through ``torch.mm`` with float32 accumulation;
    ``out`` may then be bfloat16 or float32.
    """
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or tuple(out.shape) != (m, n):
        raise KernelError(f"linear: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if row_stats is not None:
        if row_stats.per_row:
            linear_pair(x, weight, out, row_stats=row_stats)
        else:
            linear_wide(x, weight, out, row_stats=row_stats)
        return
    if x.dtype == torch.float32:
        _want(x, "x", torch.float32)
        _want(weight, "weight", torch.float32)
        _want(out, "out", torch.float32)
        _check(library().ms_gemm_f32(_ptr(x), _ptr(weight), _ptr(out), _i(m), _i(n), _i(k), _i(k), _i(k), _i(n),
                                     _stream()))
        return
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16)
    _want(out, "out")
    if m <= STREAM_MAX_ROWS and k % 8 == 0:
        # few rows (decode steps): one of the two weight-streaming kernels, or the library, by measurement
        choice = _few_rows_choice(x, weight, m)
        if choice == "stream":
            linear_stream(x, weight, out)
            return
        if choice == "skinny":
            _check(library().ms_gemm_skinny(_ptr(x), _i(0), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(m),
                                            _i(n), _i(k), _stream()))
            return
        if choice == "wide":
            linear_wide(x, weight, out)
            return
    if k % 8 == 0 and out.dtype == torch.bfloat16 and pair_preferred(x.device, m, n):
        choice = _pair_or_library("plain", m, weight)
        if choice != "library":
            linear_pair(x, weight, out, wide=choice == "wide")
            return
    if USE_TCGEN05_GEMM and m >= 128 and k % 8 == 0:
        linear_tcgen05(x, weight, out)
        return
    if out.dtype == torch.bfloat16:
        torch.mm(x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)


# Products of many rows (prompt portions).  The kernel in which two thread blocks share a 256 x 256 tile
# (linear_pair) is level with cuBLAS where its tiles fill the pairs of multiprocessors (measured at 2,048 rows:
# 29.3 / 17.7 / 76.5 / 39.3 us against 29.7 / 17.8 / 76.2 / 37.8 us for the four products of a Qwen3-1.7B layer), and
# it can apply the gated activation as it stores, which the library cannot.  With few tiles, or a last round of
# tiles that leaves most pairs idle, cuBLAS' smaller tiles win, so those shapes stay there
# (MINISERVE_B200_PAIR_GEMM=0: all of them do).  The one-block tcgen05 kernel (linear_tcgen05) reaches 77-92 % of
# cuBLAS and runs only on request (MINISERVE_B200_TCGEN05_GEMM=1).
USE_PAIR_GEMM = __import__("os").environ.get("MINISERVE_B200_PAIR_GEMM", "1") == "1"
USE_TCGEN05_GEMM = __import__("os").environ.get("MINISERVE_B200_TCGEN05_GEMM", "0") == "1"
PAIR_MIN_FILL = 0.8            # of the pairs' time in use, by the count of tiles


_many_row_choices: dict = {}         # (device index, kind, row tiles, N, K) -> "pair" | "wide" | "library"
_many_row_times: dict = {}           # the same keys -> {candidate: microseconds} as measured


def many_row_choices() -> dict:
    """What was chosen for the many-row products so far, with the measured times in microseconds."""
    return {key: (choice, _many_row_times.get(key)) for key, choice in _many_row_choices.items()}


def _pair_or_library(kind: str, rows: int, weight: torch.Tensor, n_q: int = 0, n_kv: int = 0) -> str:
    """For a product of ``rows`` rows that :func:`pair_preferred` lets through: the two-block kernel with the
    element-wise work of ``kind`` in its epilogue ("pair"; "wide": with tiles of 256 x 512, which fetch a quarter less
    from the L2 cache but are fewer), or cuBLAS followed by the separate kernel ("library").
    Measured once per kind, count of 256-row tiles and weight shape, on the weight itself, at the first eager call
    that meets it (kept in the choices file like the few-row choices); with MINISERVE_B200_LINEAR_TUNING=0 it is
    the two-block kernel.  Kinds: "plain" (store), "gated" (against the product and the activation kernel), "add"
    (product adding into the residual stream and the norm that reads it, against product, and norm that adds),
    "qkv" (against product and the norm + rotation + append kernel)."""
    n, k = weight.shape
    tiles_m = (rows + 255) // 256
    key = (torch.device(weight.device).index or 0, kind, tiles_m, n, k)
    choice = _many_row_choices.get(key)
    if choice is None:
        if not LINEAR_TUNING or torch.cuda.is_current_stream_capturing():
            return "pair"
        stored_as = f"rows{tiles_m} {kind}"
        choice = _stored_choice(stored_as, n, k)
        if choice is None:
            choice = _measure_many_rows(key, rows, weight, n_q, n_kv)
            _store_choice(stored_as, n, k, choice)
            log.info("%s products of %d rows with a %d x %d weight run %s (measured, us: %s)", kind, rows, n, k,
                     "the two-block kernel" if choice == "pair" else "cuBLAS and the separate kernel", _many_row_times.get(key))
        _many_row_choices[key] = choice
    return choice


def _measure_many_rows(key: tuple, rows: int, weight: torch.Tensor, n_q: int, n_kv: int) -> str:
    kind = key[1]
    n, k = weight.shape
    device = weight.device
    generator = torch.Generator(device=device).manual_seed(0)
    source = torch.randn((rows, k), dtype=torch.float32, device=device, generator=generator).to(torch.bfloat16)
    x = torch.empty_like(source)
    whole = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
    if kind == "plain":
        candidates = {"pair": lambda: linear_pair(x, weight, whole, wide=False),
                      "wide": lambda: linear_pair(x, weight, whole, wide=True),
                      "library": lambda: torch.mm(x, weight.t(), out=whole)}
    elif kind == "gated":
        half = torch.empty((rows, n // 2), dtype=torch.bfloat16, device=device)

        def by_library() -> None:
            torch.mm(x, weight.t(), out=whole)
            silu_mul(whole, half, paired=True)
        candidates = {"pair": lambda: linear_pair(x, weight, half, gated=True, wide=False),
                      "wide": lambda: linear_pair(x, weight, half, gated=True, wide=True), "library": by_library}
    elif kind == "add":
        residual = torch.zeros((rows, n), dtype=torch.float32, device=device)
        norm_weight = torch.ones(n, dtype=torch.bfloat16, device=device)

        def by_pair(wide: bool) -> None:
            linear_pair(x, weight, residual, add=True, wide=wide)
            add_rmsnorm(residual, None, norm_weight, 1e-6, whole)

        def by_library() -> None:
            delta = torch.mm(x, weight.t())
            add_rmsnorm(residual, delta, norm_weight, 1e-6, whole)
        candidates = {"pair": lambda: by_pair(False), "wide": lambda: by_pair(True), "library": by_library}
    elif kind == "qkv":
        d, page = 128, 64
        q = torch.empty((rows, n_q, d), dtype=torch.bfloat16, device=device)
        pools = [torch.empty(((rows + page - 1) // page, n_kv, page, d), dtype=torch.bfloat16, device=device) for _ in range(2)]
        slots = torch.arange(rows, dtype=torch.int32, device=device)
        norm_weight = torch.ones(d, dtype=torch.bfloat16, device=device)
        cos_sin = torch.zeros((rows, d // 2, 2), dtype=torch.float32, device=device)

        def by_library() -> None:
            torch.mm(x, weight.t(), out=whole)
            qk_norm_rope_append(whole, slots, norm_weight, norm_weight, 1e-6, cos_sin, d, False, pools[0], pools[1], n_q, n_kv, d, q)
        candidates = {"pair": lambda: linear_pair_qkv(x, weight, slots, norm_weight, norm_weight, 1e-6, cos_sin, pools[0],
                                                      pools[1], n_q, n_kv, q),
                      "library": by_library}
    else:
        raise KernelError(f"no many-row product of kind {kind!r}")
    times = _sample_times(candidates, x, rounds=4, source=source)
    _many_row_times[key] = {name: round(1e3 * t, 1) for name, t in times.items()}
    return min(times, key=times.get)


def pair_fill(device: torch.device, m: int, n: int) -> float:
    """The share of the pairs' time that the 256 x 256 tiles of an ``m x n`` product keep busy: tiles / (rounds x pairs)."""
    key = torch.device(device).index or 0
    if key not in _multiprocessors:
        _multiprocessors[key] = torch.cuda.get_device_properties(device).multi_processor_count
    pairs = max(_multiprocessors[key] // 2, 1)
    tiles = ((m + 255) // 256) * ((n + 255) // 256)
    return tiles / (((tiles + pairs - 1) // pairs) * pairs)


def pair_rounds(device: torch.device, m: int, n: int) -> int:
    """Tiles that the busiest pair of multiprocessors works on, one after the other, in an ``m x n`` product."""
    key = torch.device(device).index or 0
    if key not in _multiprocessors:
        _multiprocessors[key] = torch.cuda.get_device_properties(device).multi_processor_count
    pairs = max(_multiprocessors[key] // 2, 1)
    return (((m + 255) // 256) * ((n + 255) // 256) + pairs - 1) // pairs


def pair_preferred(device: torch.device, m: int, n: int, gated: bool = False) -> bool:
    """Whether a bfloat16 product of ``m`` rows with an ``n``-row weight goes to :func:`linear_pair`.  The gated form
    also saves the activation kernel and its traffic, so it is taken at a lower fill."""
    return USE_PAIR_GEMM and m >= 256 and pair_fill(device, m, n) >= (0.6 if gated else PAIR_MIN_FILL)

# Prompt portions in bfloat16 run the tcgen05 attention kernel where it takes the sizes (head size 64 or 128,
# group size dividing 128, pages of 8..128 tokens); MINISERVE_B200_TCGEN05_ATTENTION=0 keeps them on the
# mma.sync kernel.
USE_TCGEN05_ATTENTION = __import__("os").environ.get("MINISERVE_B200_TCGEN05_ATTENTION", "1") == "1"
# ... in the form in which two groups of softmax threads take the key tiles in turn, one thread per query row, with
# three score buffers; MINISERVE_B200_ATTENTION_IN_TURNS=0: all softmax threads on every tile, two per row.
ATTENTION_IN_TURNS = __import__("os").environ.get("MINISERVE_B200_ATTENTION_IN_TURNS", "1") == "1"

_error_flags: dict = {}


def device_error_flag(device: torch.device) -> torch.Tensor:
    """One int32 on the device that kernels with bounded waits set when a wait runs out (0: all well)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_device_errors(device: torch.device) -> None:
    """Raises if a kernel gave up waiting since the last check (synchronises the device)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        return                      # no kernel with bounded waits has run on this device
    flag = _error_flags[key]
    code = int(flag.item())
    if code:
        flag.zero_()
        raise KernelError(f"a kernel gave up a bounded wait (code {code}: 1 producer, 2 MMA issue, 3 epilogue, "
                          "4 copies in flight at the end)")


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, add: bool = False) -> None:
    """``out = x @ weight^T`` (``add``: ``out += ...`` on a float32 ``out``) by the library's tcgen05 kernel.

    bfloat16 operands with an inner size that is a multiple of 8; meant for 128 rows and more.
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(out, "out", torch.float32 if add else None, (m, n))
    _check(library().ms_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(1 if add else 0), _i(m),
                                     _i(n), _i(k), _ptr(device_error_flag(x.device)), _stream()))


PAIR_WIDE = __import__("os").environ.get("MINISERVE_B200_PAIR_WIDE", "0") == "1"


def linear_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, add: bool = False, gated: bool = False,
                row_stats: Optional["RowStats"] = None, wide: Optional[bool] = None) -> None:
    """``out = x @ weight^T`` by the kernel in which two thread blocks share each 256 x 256 tile (tcgen05 with
    ``cta_group::2``).  ``add``: ``out += ...`` on a float32 ``out``.  ``gated``: ``weight`` is
    :func:`interleave_gate_up` of a gate and an up projection and ``out [M, N / 2] = silu(gate) * up``.
    ``row_stats`` (from :func:`linear_pair_residual`): ``x`` still lacks the division by its rows' root mean square,
    and the results are multiplied by it before they are rounded.

    bfloat16 operands with an inner size that is a multiple of 8; meant for 256 rows and more.
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    if gated:
        _want(out, "out", torch.bfloat16, (m, n // 2))
    else:
        _want(out, "out", torch.float32 if add else None, (m, n))
    if row_stats is not None:
        _want(row_stats.partials, "row_stats.partials", torch.float32)
        if add or not row_stats.per_row or row_stats.partials.dim() != 2 or row_stats.partials.shape[1] != m \
                or row_stats.partials.shape[0] < row_stats.count:
            raise KernelError(f"linear_pair: row statistics of shape {tuple(row_stats.partials.shape)} for {m} rows, "
                              f"{row_stats.count} tiles")
    _check(library().ms_gemm_pair(_ptr(x), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(2 if gated else 1 if add else 0),
                                  _i(1 if (PAIR_WIDE if wide is None else wide) else 0),
                                  _i(m), _i(n), _i(k), _ptr(row_stats.partials if row_stats else None),
                                  _i(row_stats.count if row_stats else 0), _f(row_stats.eps if row_stats else 0.0), None, None,
                                  _i(0), None, _ptr(device_error_flag(x.device)), _stream()))


QKV_IN_PRODUCT = __import__("os").environ.get("MINISERVE_B200_QKV_IN_PRODUCT", "1") == "1"


def qkv_in_product_supported(rows: int, dtype: torch.dtype, weight: torch.Tensor, head_dim: int, n_q: int, n_kv: int,
                             cos_sin, rotary_dim: int, interleaved: bool) -> bool:
    """Whether a q/k/v projection of ``rows`` rows can norm, rotate and append its heads as it stores them
    (:func:`linear_pair_qkv`): bfloat16, so many rows that it goes to :func:`linear_pair`, heads of 128, and no
    rotation or the half-split one over the whole head."""
    if rows < 256 or not QKV_IN_PRODUCT or dtype != torch.bfloat16:
        return False
    n, k = weight.shape
    return (head_dim == 128 and k % 8 == 0
            and (cos_sin is None or (rotary_dim == head_dim and not interleaved))
            and pair_preferred(weight.device, rows, n) and _pair_or_library("qkv", rows, weight, n_q, n_kv) == "pair")


def linear_pair_qkv(x: torch.Tensor, weight: torch.Tensor, slots: torch.Tensor, q_weight: Optional[torch.Tensor],
                    k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor], k_pool: torch.Tensor,
                    v_pool: torch.Tensor, n_q: int, n_kv: int, q_out: torch.Tensor, row_stats: Optional["RowStats"] = None) -> None:
    """The q/k/v projection ``x @ weight^T`` with :func:`qk_norm_rope_append` applied to the tiles as they leave the
    tensor cores (heads of 128; the arguments mean what they mean there): q heads to ``q_out``, k and v heads to the
    pools, and the projection itself is never written out.  ``row_stats`` as in :func:`linear_pair`."""
    m, k = x.shape
    d = 128
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, ((n_q + 2 * n_kv) * d, k))
    _want(slots, "slots", torch.int32, (m,))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[3] != d:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, {n_kv}, page_size, {d}]")
    _want(q_out, "q_out", torch.bfloat16, (m, n_q, d))
    weight_code = 0
    for name, norm_weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if norm_weight is not None:
            _want(norm_weight, name, None, (d,))
            weight_code = _code(norm_weight.dtype)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share one element type")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (m, d // 2, 2))
    if row_stats is not None:
        _want(row_stats.partials, "row_stats.partials", torch.float32)
        if not row_stats.per_row or row_stats.partials.dim() != 2 or row_stats.partials.shape[1] != m \
                or row_stats.partials.shape[0] < row_stats.count:
            raise KernelError(f"linear_pair_qkv: row statistics of shape {tuple(row_stats.partials.shape)} for {m} rows")
    _check(library().ms_gemm_pair_qkv(
        _ptr(x), _ptr(weight), _ptr(q_out), _i(m), _i(k), _ptr(row_stats.partials if row_stats else None),
        _i(row_stats.count if row_stats else 0), _f(row_stats.eps if row_stats else 0.0), _ptr(slots), _ptr(q_weight),
        _ptr(k_weight), _i(weight_code), _f(eps), _ptr(cos_sin), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[2]), _i(n_q),
        _i(n_kv), _ptr(device_error_flag(x.device)), _stream()))


def pair_column_tiles(n: int) -> int:
    """Rows of ``partials`` that :func:`linear_pair_residual` writes for a weight of ``n`` rows."""
    return (n + 255) // 256


def linear_pair_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                         eps: float, x_next: torch.Tensor, partials: torch.Tensor) -> "RowStats":
    """:func:`linear_wide_residual` for many rows, by the kernel of :func:`linear_pair`: ``residual += x @ weight^T``
    (float32, in place), ``x_next = bfloat16(residual * norm_weight)`` and the rows' sums of squares, one row of
    ``partials [>= pair_column_tiles(N), M]`` per 256 columns.  ``N`` a multiple of 8."""
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(residual, "residual", torch.float32, (m, n))
    _want(norm_weight, "norm_weight", None, (n,))
    _want(x_next, "x_next", torch.bfloat16, (m, n))
    _want(partials, "partials", torch.float32)
    tiles = pair_column_tiles(n)
    if n % 8 or partials.dim() != 2 or partials.shape[1] != m or partials.shape[0] < tiles:
        raise KernelError(f"linear_pair_residual: weight {tuple(weight.shape)}, partials {tuple(partials.shape)} for {tiles} "
                          f"tiles of {m} rows")
    _check(library().ms_gemm_pair(_ptr(x), _ptr(weight), _ptr(x_next), _i(1), _i(3), _i(0), _i(m), _i(n), _i(k), None, _i(0),
                                  _f(0.0), _ptr(residual), _ptr(norm_weight), _i(_code(norm_weight.dtype)), _ptr(partials),
                                  _ptr(device_error_flag(x.device)), _stream()))
    return RowStats(partials, tiles, eps, per_row=True)


_stream_buffers: dict = {}

# Products of few rows (decode steps) read every weight once; which kernel streams a given weight fastest
# depends on its shape.  For up to SKINNY_MAX_ROWS rows the choice between the mma.sync kernel ("skinny":
# many small blocks, K split over a cluster for narrow weights), the tcgen05 kernel ("stream": one block
# per multiprocessor, its start and the sum over blocks sharing a tile cost some microseconds, which only a
# large weight wins back) and the library is measured once per weight shape, on the weight itself, in captured
# graphs as a decode step runs them (_sample_times), at the first eager call that meets the shape;
# MINISERVE_B200_LINEAR_TUNING=0 turns the measurement off, and then (and while a graph is being captured
# before any eager call) the rule below decides.  From SKINNY_MAX_ROWS + 1 to STREAM_MAX_ROWS rows it is the
# rule alone.  The gated product of a feed-forward (gated_up) chooses the same way between the kernel that
# applies the activation as it stores ("wide") and a plain product followed by the activation kernel.
STREAM_MAX_ROWS = int(__import__("os").environ.get("MINISERVE_B200_STREAM_MAX_ROWS", "16"))
STREAM_MIN_UNITS = int(__import__("os").environ.get("MINISERVE_B200_STREAM_MIN_UNITS", "32"))
LINEAR_TUNING = __import__("os").environ.get("MINISERVE_B200_LINEAR_TUNING", "1") == "1"
FEW_ROWS_KERNEL = __import__("os").environ.get("MINISERVE_B200_FEW_ROWS", "")     # "skinny" | "stream" | "wide" | "library"
if FEW_ROWS_KERNEL not in ("", "skinny", "stream", "wide", "library"):
    raise ValueError(f"MINISERVE_B200_FEW_ROWS={FEW_ROWS_KERNEL!r}: expected skinny, stream, wide or library")
_multiprocessors: dict = {}
_linear_choices: dict = {}           # (device index, N, K) -> "skinny" | "stream" | "wide" | "library"
_gated_choices: dict = {}            # (device index, 2 I, K) -> "wide" | "separate"
_choice_times: dict = {}             # the same keys -> {candidate: microseconds} as measured
FLUSH_BYTES = 256 << 20              # larger than the L2 cache
DRAW = 1.03                          # two measured times closer than this count as level


def _stream_units_per_block(device: torch.device, n: int, k: int) -> float:
    key = torch.device(device).index or 0
    if key not in _multiprocessors:
        _multiprocessors[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return ((n + 255) // 256) * ((k + 63) // 64) / _multiprocessors[key]


def _few_rows_rule(device: torch.device, m: int, n: int, k: int) -> str:
    if m <= SKINNY_MAX_ROWS and wide_supports(n, k) == 2:
        return "wide"                # one wave of blocks, each with its whole share of the weight on the way early
    if _stream_units_per_block(device, n, k) >= STREAM_MIN_UNITS:
        return "stream"
    return "skinny" if m <= SKINNY_MAX_ROWS else "library"


def _few_rows_choice(x: torch.Tensor, weight: torch.Tensor, m: int) -> str:
    n, k = weight.shape
    if FEW_ROWS_KERNEL and m <= SKINNY_MAX_ROWS and (FEW_ROWS_KERNEL != "wide" or wide_supports(n, k)):
        return FEW_ROWS_KERNEL      # pinned (to profile one kernel on every product, or to compare)
    if m > SKINNY_MAX_ROWS:
        return _few_rows_rule(x.device, m, n, k)
    key = (torch.device(x.device).index or 0, n, k)
    choice = _linear_choices.get(key)
    if choice is None:
        if not LINEAR_TUNING or torch.cuda.is_current_stream_capturing():
            return _few_rows_rule(x.device, m, n, k)
        choice = _stored_choice("linear", n, k)
        if choice is not None and (choice != "wide" or wide_supports(n, k)):
            _linear_choices[key] = choice
            return choice
        choice = _linear_choices[key] = _measure_few_rows(weight)
        _store_choice("linear", n, k, choice)
        log.info("products of up to %d rows with a %d x %d weight run the %s kernel (measured, us: %s)", SKINNY_MAX_ROWS, n, k,
                 choice, _choice_times.get(key))
    return choice


def linear_choices() -> dict:
    """What was measured so far: (device index, N, K) -> the kernel chosen for products of few rows."""
    return dict(_linear_choices)


# A measured choice can differ between runs where two kernels are level, and with it the order of a product's sums.
# MINISERVE_B200_CHOICES_FILE names a JSON file that keeps the choices: what it holds is used instead of measuring,
# and what is measured is added to it, so that later runs (and other processes) repeat the first one's choices.
CHOICES_FILE = __import__("os").environ.get("MINISERVE_B200_CHOICES_FILE", "")


def _stored_choice(kind: str, n: int, k: int) -> Optional[str]:
    if not CHOICES_FILE:
        return None
    import json
    try:
        with open(CHOICES_FILE, encoding="utf-8") as handle:
            value = json.load(handle).get(f"{kind} {n}x{k}")
    except (OSError, ValueError):
        return None
    allowed = (("skinny", "stream", "wide", "library") if kind == "linear" else ("pair", "wide", "library") if kind.startswith("rows")
               else ("wide", "separate"))
    return value if value in allowed else None


def _store_choice(kind: str, n: int, k: int, choice: str) -> None:
    if not CHOICES_FILE:
        return
    import json
    import os
    try:
        try:
            with open(CHOICES_FILE, encoding="utf-8") as handle:
                stored = json.load(handle)
        except (OSError, ValueError):
            stored = {}
        stored[f"{kind} {n}x{k}"] = choice
        temporary = f"{CHOICES_FILE}.{os.getpid()}"
        with open(temporary, "w", encoding="utf-8") as handle:
            json.dump(stored, handle, indent=1, sort_keys=True)
        os.replace(temporary, CHOICES_FILE)
    except OSError as error:
        log.warning("cannot keep the kernel choices in %s: %s", CHOICES_FILE, error)


TUNING_REPEATS = 8      # a candidate this many times in one captured graph


def _sample_times(candidates: dict, x: torch.Tensor, rounds: int = 7, source: Optional[torch.Tensor] = None) -> dict:
    """Device time in milliseconds of each of ``candidates`` (name -> callable reading ``x``), measured the way
    a decode step runs them: in a captured graph, after a small kernel of this library that writes ``x`` (so
    that a candidate which can start before its predecessor ends does so), with the L2 cache overwritten
    before it.  A graph holds that sequence TUNING_REPEATS times; the same graph without the candidate is
    timed too and subtracted.  The graphs take turns, round after round, so that a clock that is still rising
    meets all of them alike; the figure is the lower quartile of a graph's samples."""
    device = x.device
    flush = torch.empty(FLUSH_BYTES // 4, dtype=torch.float32, device=device)
    # (``source``: what ``x`` is made from before every run; zeros unless the candidates' speed depends on the data,
    # as that of tensor-core products under the power limit does)
    source = torch.zeros_like(x) if source is None else source
    weight = torch.ones(x.shape[-1], dtype=x.dtype, device=device)

    def capture(run) -> torch.cuda.CUDAGraph:
        def sequence() -> None:
            for _ in range(TUNING_REPEATS):
                flush.zero_()
                rmsnorm(source, weight, 1e-6, x)
                if run is not None:
                    run()
        sequence()                                          # lazy set-up outside the capture
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sequence()
        return graph

    graphs = {name: capture(run) for name, run in candidates.items()}
    graphs[None] = capture(None)
    samples = {name: [] for name in graphs}
    for round_index in range(rounds + 2):
        for name, graph in graphs.items():
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            end.synchronize()
            if round_index >= 2:                            # the first rounds bring the clocks up
                samples[name].append(start.elapsed_time(end))
    quartile = {name: sorted(times)[len(times) // 4] for name, times in samples.items()}
    return {name: (quartile[name] - quartile[None]) / TUNING_REPEATS for name in candidates}


def _measure_few_rows(weight: torch.Tensor) -> str:
    """Times the candidates for ``[8, K] @ weight[N, K]^T`` on the device and names the one to use: the fastest
    of this library's kernels or the vendor library's."""
    n, k = weight.shape
    device = weight.device
    x = torch.zeros((SKINNY_MAX_ROWS, k), dtype=torch.bfloat16, device=device)
    out = torch.empty((SKINNY_MAX_ROWS, n), dtype=torch.bfloat16, device=device)
    candidates = {
        "skinny": lambda: _check(library().ms_gemm_skinny(_ptr(x), _i(0), _ptr(weight), _ptr(out), _i(_code(out.dtype)),
                                                          _i(SKINNY_MAX_ROWS), _i(n), _i(k), _stream())),
        "stream": lambda: linear_stream(x, weight, out),
        "library": lambda: torch.mm(x, weight.t(), out=out),
    }
    if wide_supports(n, k) == 2:
        candidates["wide"] = lambda: linear_wide(x, weight, out)
    times = _sample_times(candidates, x)
    _choice_times[(torch.device(device).index or 0, n, k)] = {name: round(1e3 * t, 2) for name, t in times.items()}
    own = min((name for name in candidates if name != "library"), key=lambda name: times[name])
    # Whole steps decide what the measurement leaves open.  The two kernels that stream weights by TMA and ask
    # for the first of them before their predecessor has ended have kept in the step what they showed here (the
    # output matrix, level with the vendor library here, is 4 % of a step faster with the tcgen05 kernel), so
    # they also win a draw; the mma.sync kernel has lost to the library in the step where it was level with it
    # here (the 8B gate/up projection: 12 us a layer), so it has to be clearly faster.
    if own == "skinny":
        return own if DRAW * times[own] < times["library"] else "library"
    return own if times[own] <= DRAW * times["library"] else "library"


def linear_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ weight^T`` for up to 64 rows of bfloat16 ``x`` (inner size a multiple of 8) by the
    library's weight-streaming tcgen05 kernel; ``out`` bfloat16 or float32."""
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(out, "out", None, (m, n))
    key = torch.device(x.device).index or 0
    tiles = (n + 255) // 256
    buffers = _stream_buffers.get(key)
    if buffers is None or buffers[1].numel() < tiles:
        floats, ints = ctypes.c_longlong(0), ctypes.c_longlong(0)
        _check(library().ms_gemm_stream_buffers(_i(max(n, 1 << 20)), ctypes.addressof(floats), ctypes.addressof(ints)))
        buffers = (torch.empty(floats.value, dtype=torch.float32, device=x.device),
                   torch.zeros(ints.value, dtype=torch.int32, device=x.device))
        _stream_buffers[key] = buffers
    _check(library().ms_gemm_stream(_ptr(x), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(m), _i(n), _i(k),
                                    _ptr(buffers[0]), _ptr(buffers[1]), _ptr(device_error_flag(x.device)), _stream()))


_wide_supports: dict = {}


def wide_supports(n: int, k: int) -> int:
    """0: :func:`linear_wide` does not take a weight of ``n`` rows and inner size ``k``; 1: it does, in several
    waves of blocks; 2: with at most one block per multiprocessor, which is what it is made for."""
    answer = _wide_supports.get((n, k))
    if answer is None:
        answer = _wide_supports[(n, k)] = int(library().ms_gemm_wide_supports(_i(n), _i(k)))
    return answer


class RowStats:
    """What is still missing from activations whose norm is folded into the products around it: ``x`` holds
    ``residual * norm weight`` and every row has yet to be divided by the root of its mean square.
    ``partials`` (float32) holds sums of squares of the residual's rows, one row of partial sums per block (or
    column tile) of the product that wrote ``x``: ``[count, 8]`` from the few-row product, ``[count, rows]`` from
    the many-row one (``per_row``).  The product that reads ``x`` adds them up in order and applies
    ``1 / sqrt(total / size + eps)`` to its own results."""

    __slots__ = ("partials", "count", "eps", "per_row")

    def __init__(self, partials: torch.Tensor, count: int, eps: float, per_row: bool = False) -> None:
        self.partials, self.count, self.eps, self.per_row = partials, count, eps, per_row


def wide_blocks(n: int, k: int) -> int:
    """Blocks that :func:`linear_wide` runs for a weight ``[n, k]``: the rows of ``partials`` that
    :func:`linear_wide_residual` writes."""
    return int(library().ms_gemm_wide_blocks(_i(n), _i(k)))


def _wide_call(x, weight, out, out_code: int, mode: int, m: int, n: int, k: int, row_stats: Optional[RowStats],
               residual=None, norm_weight=None, x_next=None, out_partials=None) -> None:
    if row_stats is not None:
        _want(row_stats.partials, "row_stats.partials", torch.float32)
        if row_stats.partials.dim() != 2 or row_stats.partials.shape[1] != 8 or row_stats.partials.shape[0] < row_stats.count:
            raise KernelError(f"row statistics of shape {tuple(row_stats.partials.shape)} for {row_stats.count} blocks")
    _check(library().ms_gemm_wide(
        _ptr(x), _ptr(weight), _ptr(out), _i(out_code), _i(mode), _i(m), _i(n), _i(k),
        _ptr(row_stats.partials if row_stats else None), _i(row_stats.count if row_stats else 0),
        _f(row_stats.eps if row_stats else 0.0), _ptr(residual), _ptr(norm_weight),
        _i(_code(norm_weight.dtype) if norm_weight is not None else 0), _ptr(x_next), _ptr(out_partials),
        _ptr(device_error_flag(x.device)), _stream()))


def linear_wide(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
                row_stats: Optional[RowStats] = None) -> None:
    """``out = x @ weight^T`` for up to 8 rows of bfloat16 ``x`` by the library's kernel for weights of many
    rows (no sum across blocks); ``out`` bfloat16 or float32.

    ``gated``: ``weight [2 I, K]`` holds a gated feed-forward's two projections in blocks of sixteen rows,
    eight gate rows followed by the up rows of the same features (:func:`interleave_gate_up`), and
    ``out [M, I]`` bfloat16 receives ``silu(gate) * up``.  ``row_stats``: ``x`` comes from
    :func:`linear_wide_residual`; its rows' norm is completed on the results (before the activation).
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(out, "out", torch.bfloat16 if gated else None, (m, n // 2 if gated else n))
    _wide_call(x, weight, out, _code(out.dtype), 1 if gated else 0, m, n, k, row_stats)


def linear_wide_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                         eps: float, x_next: torch.Tensor, partials: torch.Tensor) -> RowStats:
    """``residual += x @ weight^T`` (float32, in place) for up to 8 rows of bfloat16 ``x``, and the input of
    whatever follows an RMSNorm of the new residual: ``x_next = bfloat16(residual * norm_weight)`` with the rows'
    sums of squares left in ``partials`` (float32 ``[>= wide_blocks(N, K), 8]``).  The returned statistics go
    with ``x_next`` into :func:`linear_wide` or :func:`gated_up`.  Only for weights with ``wide_supports == 2``.
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(residual, "residual", torch.float32, (m, n))
    _want(norm_weight, "norm_weight", None, (n,))
    _want(x_next, "x_next", torch.bfloat16, (m, n))
    _want(partials, "partials", torch.float32)
    blocks = wide_blocks(n, k)
    if wide_supports(n, k) != 2 or partials.dim() != 2 or partials.shape[1] != 8 or partials.shape[0] < blocks:
        raise KernelError(f"linear_wide_residual: weight {tuple(weight.shape)} (one wave of blocks only), partials "
                          f"{tuple(partials.shape)} for {blocks} blocks")
    _wide_call(x, weight, None, 1, 2, m, n, k, None, residual, norm_weight, x_next, partials)
    return RowStats(partials, blocks, eps)


ADD_IN_PRODUCT = __import__("os").environ.get("MINISERVE_B200_ADD_IN_PRODUCT", "1") == "1"


def add_in_product_supported(rows: int, dtype: torch.dtype, weight: torch.Tensor) -> bool:
    """Whether a product of ``rows`` rows with ``weight`` can add its results into a float32 matrix as it stores
    them (:func:`linear_add`): bfloat16, and so many rows that it goes to :func:`linear_pair`, whose read-out hands
    its tiles to TMA as additions.  The norm that follows then reads the residual stream and writes its output,
    and no longer reads a separate output, adds it and writes the stream back (at Qwen3-1.7B sizes and 2,048 rows:
    25 MB instead of 50 MB a norm)."""
    if rows < 256 or not ADD_IN_PRODUCT or dtype != torch.bfloat16:      # (what decides for steps of few rows, first)
        return False
    n, k = weight.shape
    return (n % 4 == 0 and k % 8 == 0
            and pair_preferred(weight.device, rows, n) and _pair_or_library("add", rows, weight) != "library")


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> None:
    """``residual += x @ weight^T`` (float32, in place), where :func:`add_in_product_supported` said so."""
    linear_pair(x, weight, residual, add=True, wide=_pair_or_library("add", x.shape[0], weight) == "wide")


def residual_partials_shape(rows: int, n: int, k: int) -> tuple:
    """The shape of the float32 ``partials`` that :func:`linear_residual` wants for ``rows`` rows and a weight ``[n, k]``."""
    return (wide_blocks(n, k), 8) if rows <= SKINNY_MAX_ROWS else (pair_column_tiles(n), rows)


def linear_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                    x_next: torch.Tensor, partials: torch.Tensor) -> RowStats:
    """A product whose results join the residual stream, with the norm that follows folded in (where
    :func:`fold_supported` said so): :func:`linear_wide_residual` for up to 8 rows, :func:`linear_pair_residual`
    for many."""
    if x.shape[0] <= SKINNY_MAX_ROWS:
        return linear_wide_residual(x, weight, residual, norm_weight, eps, x_next, partials)
    return linear_pair_residual(x, weight, residual, norm_weight, eps, x_next, partials)


def fold_supported(rows: int, dtype: torch.dtype, producer: torch.Tensor, consumer: torch.Tensor,
                   consumer_gated: bool = False) -> bool:
    """Whether, in a step of ``rows`` rows, an RMSNorm between the product with the weight ``producer`` and the
    one with ``consumer`` can be folded into the two (:func:`linear_residual`, then ``row_stats``): bfloat16, and
    either at most 8 rows and both weights ones that :func:`linear_wide` is (or would be) chosen for, or so many
    rows that both products go to :func:`linear_pair`."""
    if not FOLD_NORMS or dtype != torch.bfloat16 or rows <= 0:
        return False
    if rows > SKINNY_MAX_ROWS:
        if not FOLD_NORMS_MANY_ROWS or producer.shape[0] % 8 or producer.shape[1] % 8 or consumer.shape[1] % 8:
            return False
        # The folded epilogue moves 10 bytes per element against 2; it pays where a pair has a next tile to
        # accumulate meanwhile (measured at Qwen3-1.7B sizes: 4,096 rows 39.3 against 46.1 us for the o projection and
        # the norm kernel, 8,192 rows 71.9 against 89.4 us; 2,048 rows, one tile per pair, 25.8 against 26.1 us)
        return (pair_preferred(producer.device, rows, producer.shape[0])
                and pair_rounds(producer.device, rows, producer.shape[0]) >= 2
                and pair_preferred(consumer.device, rows, consumer.shape[0], gated=consumer_gated)
                and _pair_or_library("add", rows, producer) != "library"
                and _pair_or_library("gated" if consumer_gated else "plain", rows, consumer) != "library")
    for weight, gated in ((producer, False), (consumer, consumer_gated)):
        n, k = weight.shape
        if k % 8 or wide_supports(n, k) != 2:
            return False
        key = (torch.device(weight.device).index or 0, n, k)
        if FEW_ROWS_KERNEL:
            chosen = FEW_ROWS_KERNEL
        else:
            chosen = (_gated_choices if gated else _linear_choices).get(key, "wide")    # not measured yet: the rule says wide
        if chosen != "wide":
            return False
    return True


FOLD_NORMS = __import__("os").environ.get("MINISERVE_B200_FOLD_NORMS", "1") == "1"
FOLD_NORMS_MANY_ROWS = __import__("os").environ.get("MINISERVE_B200_FOLD_NORMS_MANY_ROWS", "1") == "1"


GATE_UP_BLOCK = 8    # rows of the gate projection beside as many of the up projection, for linear_wide(gated=True)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``[2 I, K]``: rows 16 j .. 16 j + 7 are the gate rows 8 j .. 8 j + 7, the next eight the same up rows."""
    inter, k = gate.shape
    if inter % GATE_UP_BLOCK != 0 or up.shape != gate.shape:
        raise KernelError(f"interleave_gate_up: {tuple(gate.shape)} and {tuple(up.shape)}; rows must be a multiple of 8")
    blocks = inter // GATE_UP_BLOCK
    return torch.stack((gate.reshape(blocks, GATE_UP_BLOCK, k), up.reshape(blocks, GATE_UP_BLOCK, k)), dim=1).reshape(2 * inter, k)


WIDE_GATED_MIN_ROWS = 8192     # of the paired weight: the rule when nothing was measured


def gated_up(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_stats: Optional[RowStats] = None) -> None:
    """``out[M, I] = silu(x @ gate^T) * (x @ up^T)`` with ``weight = interleave_gate_up(gate, up)``.
    (``row_stats``: see :func:`linear_wide`; the caller has asked :func:`fold_supported` first.)

    Few rows of bfloat16 go through :func:`linear_wide`, which applies the activation as it stores, where that
    is faster than the product (:func:`linear`) followed by :func:`silu_mul`: measured once per weight shape
    like the choice among the plain products, with the same switch.
    """
    m, k = x.shape
    two_i = weight.shape[0]
    _want(out, "out", x.dtype, (m, two_i // 2))
    if row_stats is not None:
        if row_stats.per_row:
            linear_pair(x, weight, out, gated=True, row_stats=row_stats)
        else:
            linear_wide(x, weight, out, gated=True, row_stats=row_stats)
        return
    if x.dtype == torch.bfloat16 and 0 < m <= SKINNY_MAX_ROWS and _gated_choice(x, weight) == "wide":
        linear_wide(x, weight, out, gated=True)
        return
    if x.dtype == torch.bfloat16 and k % 8 == 0 and pair_preferred(x.device, m, two_i, gated=True):
        choice = _pair_or_library("gated", m, weight)
        if choice != "library":
            linear_pair(x, weight, out, gated=True, wide=choice == "wide")    # many rows: the activation is applied as the tiles are stored
            return
    gate_up = torch.empty((m, two_i), dtype=x.dtype, device=x.device)
    linear(x, weight, gate_up)
    silu_mul(gate_up, out, paired=True)


def _gated_choice(x: torch.Tensor, weight: torch.Tensor) -> str:
    n, k = weight.shape
    key = (torch.device(x.device).index or 0, n, k)
    choice = _gated_choices.get(key)
    if choice is None:
        fits = wide_supports(n, k) if k % 8 == 0 and n % (2 * GATE_UP_BLOCK) == 0 else 0
        if not fits:
            choice = _gated_choices[key] = "separate"
        elif not LINEAR_TUNING or torch.cuda.is_current_stream_capturing():
            return "wide" if fits == 2 and n >= WIDE_GATED_MIN_ROWS else "separate"
        else:
            choice = _stored_choice("gated", n, k)
            if choice is not None:
                _gated_choices[key] = choice
                return choice
            choice = _gated_choices[key] = _measure_gated(weight)
            _store_choice("gated", n, k, choice)
            log.info("gated products of up to %d rows with a %d x %d weight run %s (measured, us: %s)", SKINNY_MAX_ROWS, n, k,
                     "the kernel that applies the activation" if choice == "wide" else "a plain product and the activation kernel",
                     _choice_times.get(key + ("gated",)))
    return choice


def _measure_gated(weight: torch.Tensor) -> str:
    n, k = weight.shape
    device = weight.device
    x = torch.zeros((SKINNY_MAX_ROWS, k), dtype=torch.bfloat16, device=device)
    gate_up = torch.empty((SKINNY_MAX_ROWS, n), dtype=torch.bfloat16, device=device)
    out = torch.empty((SKINNY_MAX_ROWS, n // 2), dtype=torch.bfloat16, device=device)

    def separate() -> None:
        linear(x, weight, gate_up)
        silu_mul(gate_up, out, paired=True)

    separate()                                              # the plain product's own choice is made outside the timing
    times = _sample_times({"wide": lambda: linear_wide(x, weight, out, gated=True), "separate": separate}, x)
    _choice_times[(torch.device(device).index or 0, n, k, "gated")] = {name: round(1e3 * t, 2) for name, t in times.items()}
    return "wide" if times["wide"] <= times["separate"] else "separate"


def choice_times() -> dict:
    """The measurements behind :func:`linear_choices` and :func:`gated_choices`: key -> {candidate: microseconds}
    (gated products have a fourth key element)."""
    return {key: dict(times) for key, times in _choice_times.items()}


def gated_choices() -> dict:
    """What was measured so far: (device index, 2 I, K) -> how the gated product of few rows runs."""
    return dict(_gated_choices)


SKINNY_MAX_ROWS = 8    # above this the weight-streaming kernel re-reads the activations too often


FUSE_GATED_INPUT = False    # applying the activation while streaming recomputes it in every block: slower (measured twice)


def gated_linear(gate_up: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out = (silu(gate_up[:, :I]) * gate_up[:, I:]) @ weight[N, I]^T``.

    With few rows in bfloat16 the activation is applied while the product streams the weights;
    otherwise it is one kernel (:func:`silu_mul`) followed by :func:`linear`.
    """
    m, two_i = gate_up.shape
    inter = two_i // 2
    n = weight.shape[0]
    if two_i != 2 * inter or weight.shape[1] != inter or tuple(out.shape) != (m, n):
        raise KernelError(f"gated_linear: gate_up {tuple(gate_up.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if FUSE_GATED_INPUT and gate_up.dtype == torch.bfloat16 and m <= SKINNY_MAX_ROWS and inter % 8 == 0:
        _want(gate_up, "gate_up", torch.bfloat16)
        _want(weight, "weight", torch.bfloat16)
        _want(out, "out")
        _check(library().ms_gemm_skinny(_ptr(gate_up), _i(1), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(m),
                                        _i(n), _i(inter), _stream()))
        return
    hidden = torch.empty((m, inter), dtype=gate_up.dtype, device=gate_up.device)
    silu_mul(gate_up, hidden)
    linear(hidden, weight, out)


# --------------------------------------------------------------------------- sampling

SAMPLING_RECORD_WORDS = 8


def sample(logits: torch.Tensor, records: Optional[torch.Tensor], slot_of_row: Optional[torch.Tensor],
           draw_index: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """Chooses one token per row of float32 ``logits [K, V]`` into int32 ``out [K]``.

    ``records`` int32 ``[slots, 8]`` holds per state slot the bit patterns of (temperature,
    top_p) and the integers (top_k, seed low word, seed high word); ``slot_of_row`` and
    ``draw_index`` are int32 ``[K]``.  ``records=None`` means argmax for every row.
    """
    k, vocab = logits.shape
    _want(logits, "logits", torch.float32)
    _want(out, "out", torch.int32, (k,))
    if records is not None:
        _want(records, "records", torch.int32)
        if records.dim() != 2 or records.shape[1] != SAMPLING_RECORD_WORDS:
            raise KernelError(f"records must be [slots, {SAMPLING_RECORD_WORDS}] int32")
        _want(slot_of_row, "slot_of_row", torch.int32, (k,))
        _want(draw_index, "draw_index", torch.int32, (k,))
    # candidates of the first of the two kernels: (value, index) for every chunk of every row
    scratch = torch.empty((k, library().ms_sample_chunks(_i(vocab)), 2), dtype=torch.int32, device=logits.device)
    _check(library().ms_sample(_ptr(logits), _i(logits.stride(0)), _i(vocab), _ptr(records), _ptr(slot_of_row),
                               _ptr(draw_index), _ptr(out), _i(k), _ptr(scratch), _stream()))

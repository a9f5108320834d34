"""Python bindings of the CUDA kernels.

Each function checks its arguments, passes raw pointers, sizes and the current CUDA stream to
an ``extern "C"`` launcher, and raises if the launcher reports an error.  There is no other
implementation behind these names: without a GPU, a compiler or a successful build they
raise.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Any

import torch

from mini_engine_b200.csrc import build
from mini_engine_b200.csrc.build import load_library

F32, BF16 = 0, 1
_ERRORS = {1001: "sizes not supported by this kernel", 1002: "bad argument"}


class KernelError(RuntimeError):
    pass


def _type_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())


_scoped_stream: c_void_p | None = None


def _stream() -> c_void_p:
    """The stream that launches go to: torch's current one, looked up once per `stream_scope`
    (the lookup costs about as much as the rest of a launch's Python)."""
    if _scoped_stream is not None:
        return _scoped_stream
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """While open, every launch of this package goes to the stream that was torch's current one
    when the scope was opened.  The model's forward pass opens one: nothing inside it changes the
    current stream (a graph capture changes it around the whole pass)."""

    def __enter__(self) -> None:
        global _scoped_stream
        self.previous = _scoped_stream
        _scoped_stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def __exit__(self, *exc) -> None:
        global _scoped_stream
        _scoped_stream = self.previous


class programmatic_launch:
    """While open, the package's kernels are launched as programmatic dependents of their predecessors
    (``True``, the default outside any scope) or in plain stream order (``False``).  The model's forward
    pass opens one with what its parts say."""

    def __init__(self, enabled: bool):
        self.enabled = bool(enabled)

    def __enter__(self) -> None:
        from mini_engine_b200.csrc.build import set_programmatic_launch

        self.previous = set_programmatic_launch(self.enabled)

    def __exit__(self, *exc) -> None:
        from mini_engine_b200.csrc.build import set_programmatic_launch

        set_programmatic_launch(self.previous)


class _Counter:
    """Kernel launches issued through this package's bindings since import."""

    launches = 0


def launch_count() -> int:
    return _Counter.launches


def _check(code: int, what: str) -> None:
    _Counter.launches += 1
    if code == 0:
        return
    if code in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[code]}")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def raise_on_device_error() -> None:
    """Ask the tensor-core and attention libraries that are loaded whether a kernel gave up a
    bounded wait since the last call, and raise if one did: what such a kernel wrote is invalid.
    Reads a flag from the device, so it waits for the work in flight."""
    latent_tc = 0
    if "latent_attention_tcgen05" in build._loaded:
        held = c_int(0)
        status = _fn("latent_attention_tcgen05", "me_latent_attention_tcgen05_take_error", [ctypes.POINTER(c_int)])(ctypes.byref(held))
        if status != 0:
            raise KernelError(f"could not read the latent attention kernel's error flag (CUDA error {status})")
        latent_tc = held.value
    latent = 0
    if "latent_attention_bf16" in build._loaded:
        held = c_int(0)
        status = _fn("latent_attention_bf16", "me_latent_attention_bf16_take_error", [ctypes.POINTER(c_int)])(ctypes.byref(held))
        if status != 0:
            raise KernelError(f"could not read the latent attention kernel's error flag (CUDA error {status})")
        latent = held.value
    for what, code in (("tensor-core product", tensor_core.take_error()), ("attention", attention_bf16.take_error()),
                       ("latent attention", latent), ("latent attention (tcgen05)", latent_tc)):  # fmt: skip
        if code:
            raise KernelError(
                f"a {what} kernel ran into the limit of a wait (code {code}): the results since the last check are invalid"
            )


def _cuda_error_name(code: int) -> str:
    try:
        runtime = ctypes.CDLL("libcudart.so")
        runtime.cudaGetErrorString.restype = ctypes.c_char_p
        return runtime.cudaGetErrorString(code).decode()
    except OSError:
        return "unknown"


def _need(tensor: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


_signatures_done: set[str] = set()


def _fn(library: str, name: str, argtypes: list[Any]):
    lib = load_library(library)
    fn = getattr(lib, name)
    if name not in _signatures_done:
        fn.argtypes = argtypes
        fn.restype = c_int
        _signatures_done.add(name)
    return fn


# ------------------------------------------------------------------------------ size rules


def check_attention_sizes(head_dim: int, heads: int, kv_heads: int) -> None:
    """Sizes that some attention kernel of this package takes; a clear error otherwise."""
    if head_dim < 16 or head_dim % 16 or head_dim > 512:
        raise ValueError(f"head_dim must be a multiple of 16 between 16 and 512, got {head_dim}")
    if heads < 1 or kv_heads < 1 or heads % kv_heads:
        raise ValueError(f"heads ({heads}) must be a positive multiple of kv_heads ({kv_heads})")


# ------------------------------------------------------------------------------ elementwise


def embedding(table: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor, multiplier: float = 1.0) -> None:
    """``out[t] = table[token_ids[t]] * multiplier`` widened to float32."""
    _need(table, None, "table"), _need(token_ids, torch.int32, "token_ids"), _need(out, torch.float32, "out")
    fn = _fn("elementwise", "me_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    vocab, hidden = table.shape
    code = fn(_ptr(table), _type_code(table.dtype), _ptr(token_ids), _ptr(out), out.shape[0], hidden, vocab,
              float(multiplier), _stream())  # fmt: skip
    _check(code, "embedding")


def logits_finish(logits: torch.Tensor, bias: torch.Tensor | None, scale: float = 1.0, soft_cap: float = 0.0) -> None:
    """In place on float32 ``logits [N, vocab]``: ``y = x * scale + bias``, then ``soft_cap *
    tanh(y / soft_cap)`` when ``soft_cap > 0``."""
    _need(logits, torch.float32, "logits")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.shape != (logits.shape[1],):
            raise KernelError("the bias must have one value per logit")
    fn = _fn("elementwise", "me_logits_finish", [c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p])
    code = fn(_ptr(logits), _ptr(bias) if bias is not None else None, float(scale), float(soft_cap),
              logits.shape[0], logits.shape[1], _stream())  # fmt: skip
    _check(code, "logits_finish")


def pick_tokens(tokens: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """``out[i] = tokens[rows[i]]``, all int32 on the device."""
    _need(tokens, torch.int32, "tokens"), _need(rows, torch.int32, "rows"), _need(out, torch.int32, "out")
    if rows.shape[0] != out.shape[0]:
        raise KernelError("one row index per output")
    fn = _fn("sampling", "me_pick_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(tokens), _ptr(rows), _ptr(out), out.shape[0], _stream()), "pick_tokens")


def add_rmsnorm(
    x: torch.Tensor,
    pending: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: torch.Tensor | None = None,
    pending_scale: torch.Tensor | None = None,
    x_scale: float = 1.0,
    keep_normed: bool = False,
) -> None:
    """``x += sum_s pending[s]`` (in place, float32) and ``out = weight * rmsnorm(x)``.

    With ``x_scale`` the sum is ``x_scale * x + sum_s pending[s]``; with ``keep_normed`` it is the
    normalised row (float32) that is written back to ``x`` instead of the sum (a layer whose norm
    follows the sum).

    With ``rows`` only ``x[rows]`` (+ pending) are normalised into ``out[0..len(rows))`` and
    ``x`` is not modified.  With ``pending_scale`` (float32 ``[hidden]``) the sum that is added is
    ``pending_scale * sum_s pending[s]``, column by column."""
    _need(x, torch.float32, "x"), _need(weight, torch.float32, "weight"), _need(out, None, "out")
    hidden = x.shape[-1]
    splits, stride = 0, 0
    if pending is not None:
        _need(pending, torch.float32, "pending")
        splits, stride = pending.shape[0], pending.stride(0)
        if pending.shape[1:] != x.shape:
            raise KernelError(f"pending {tuple(pending.shape)} does not fit x {tuple(x.shape)}")
    if weight.shape != (hidden,) or out.shape[-1] != hidden:
        raise KernelError("add_rmsnorm: weight/out width does not match x")
    count = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if pending_scale is not None:
        _need(pending_scale, torch.float32, "pending_scale")
        if pending_scale.shape != (hidden,):
            raise KernelError("add_rmsnorm: pending_scale must have one value per column")
    fn = _fn(
        "elementwise",
        "me_add_rmsnorm",
        [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_float, c_int, c_void_p],
    )
    code = fn(
        _ptr(x), _ptr(pending), splits, stride, _ptr(weight), eps, _ptr(out), _type_code(out.dtype),
        _ptr(rows), count, hidden, _ptr(pending_scale), float(x_scale), 1 if keep_normed else 0, _stream(),
    )  # fmt: skip
    _check(code, "add_rmsnorm")


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def add_layernorm(
    x: torch.Tensor,
    pending: torch.Tensor | None,
    weight: torch.Tensor,
    bias: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: torch.Tensor | None = None,
    pending_more: torch.Tensor | None = None,
    pending_bias: torch.Tensor | None = None,
) -> None:
    """``x += pending_bias + sum_s pending[s] + sum_s pending_more[s]`` (in place, float32) and ``out = (x - mean) /
    sqrt(var + eps) * weight + bias`` with the variance as the mean of the squared deviations.  With ``rows`` only
    ``x[rows]`` (+ the pending sums) are normalised into ``out[0..len(rows))`` and ``x`` is not modified."""
    _need(x, torch.float32, "x"), _need(weight, torch.float32, "weight"), _need(bias, torch.float32, "bias"), _need(out, None, "out")
    hidden = x.shape[-1]
    sums = []
    for name, part in (("pending", pending), ("pending_more", pending_more)):
        if part is None:
            sums += [None, 0, 0]
            continue
        _need(part, torch.float32, name)
        if part.shape[1:] != x.shape:
            raise KernelError(f"{name} {tuple(part.shape)} does not fit x {tuple(x.shape)}")
        sums += [part, part.shape[0], part.stride(0)]
    if weight.shape != (hidden,) or bias.shape != (hidden,) or out.shape[-1] != hidden:
        raise KernelError("add_layernorm: weight/bias/out width does not match x")
    if pending_bias is not None:
        _need(pending_bias, torch.float32, "pending_bias")
        if pending_bias.shape != (hidden,):
            raise KernelError("add_layernorm: pending_bias must have one value per column")
    count = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn(
        "elementwise",
        "me_add_layernorm",
        [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    )
    code = fn(
        _ptr(x), _ptr(sums[0]), sums[1], sums[2], _ptr(sums[3]), sums[4], sums[5], _ptr(pending_bias), _ptr(weight), _ptr(bias),
        float(eps), _ptr(out), _type_code(out.dtype), _ptr(rows), count, hidden, _stream(),
    )  # fmt: skip
    _check(code, "add_layernorm")


def swiglu(
    partials: torch.Tensor, out: torch.Tensor, slope: float = 1.0, limit: float | None = None, offset: float = 0.0,
    group_weight: torch.Tensor | None = None, activation: str = "silu",
) -> None:
    """``out = g * sigmoid(slope * g) * (u + offset)`` where gate/up are the halves of ``sum_s
    partials[s]``, ``g = min(gate, limit)`` and ``u = clamp(up, -limit, limit)`` when a limit is
    given, else ``g = gate``, ``u = up``.  The defaults are ``silu(gate) * up``.  With ``group_weight``
    (float32 ``[T, groups]``) the features form ``groups`` equal runs and feature ``i`` of token ``t`` is
    multiplied by ``group_weight[t, i // (inter / groups)]`` (routed units side by side).  ``activation``
    ``"gelu_tanh"`` puts ``0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))`` in the place of ``g * sigmoid(slope * g)``."""
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"swiglu: activation must be one of {sorted(GATE_ACTIVATIONS)}, got {activation!r}")
    _need(partials, torch.float32, "partials"), _need(out, None, "out")
    splits, tokens, width = partials.shape
    inter = width // 2
    if out.shape != (tokens, inter):
        raise KernelError(f"swiglu: out {tuple(out.shape)} does not fit partials {tuple(partials.shape)}")
    if limit is not None and not limit > 0:
        raise KernelError("the limit of a gated activation must be positive (or absent)")
    group_size = 0
    if group_weight is not None:
        _need(group_weight, torch.float32, "group_weight")
        if group_weight.dim() != 2 or group_weight.shape[0] != tokens or inter % group_weight.shape[1]:
            raise KernelError(f"swiglu: group_weight {tuple(group_weight.shape)} does not fit {tokens} tokens of {inter} features")
        group_size = inter // group_weight.shape[1]
    fn = _fn("elementwise", "me_swiglu", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p, c_int, c_int, c_void_p])
    code = fn(_ptr(partials), splits, partials.stride(0), _ptr(out), _type_code(out.dtype), tokens, inter,
              float(slope), float(limit or 0.0), float(offset), _ptr(group_weight), group_size,
              GATE_ACTIVATIONS[activation], _stream())  # fmt: skip
    _check(code, "swiglu")


def qk_norm_rope_store(
    *,
    qkv: torch.Tensor,
    heads: int,
    kv_heads: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos_sin: torch.Tensor | None,
    positions: torch.Tensor,
    q_out: torch.Tensor,
    page_size: int,
    slot_mapping: torch.Tensor | None = None,
    k_pages: torch.Tensor | None = None,
    v_pages: torch.Tensor | None = None,
    k_dense: torch.Tensor | None = None,
    v_dense: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    value_dim: int | None = None,
) -> None:
    """Per-head RMSNorm of q and k, rotation, and the write of k and v to their cache slots
    (or to dense ``[T, kv_heads * head_dim]`` buffers when ``slot_mapping`` is ``None``).
    ``qkv`` is ``[S, T, (heads + kv_heads) * head_dim + kv_heads * value_dim]`` float32 partial sums
    (``value_dim`` is ``head_dim`` unless given); ``bias`` (float32, one value per column of ``qkv``) is
    added to their sum before anything else."""
    _need(qkv, torch.float32, "qkv"), _need(q_out, None, "q_out"), _need(positions, torch.int32, "positions")
    splits, tokens, width = qkv.shape
    value_dim = head_dim if value_dim is None else value_dim
    if width != (heads + kv_heads) * head_dim + kv_heads * value_dim:
        raise KernelError(f"qkv width {width} is not (heads + kv_heads) * head_dim + kv_heads * value_dim")
    if kv_heads and slot_mapping is None and (k_dense is None or v_dense is None):
        raise KernelError("either slot_mapping with pages or dense outputs must be given")
    if kv_heads and slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
        if k_pages is None or v_pages is None or k_pages.dtype != q_out.dtype:
            raise KernelError("pages must be given in the dtype of q_out")
        if k_pages.shape[1:] != (kv_heads, page_size, head_dim) or v_pages.shape[1:] != (kv_heads, page_size, value_dim):
            raise KernelError(f"pages {tuple(k_pages.shape)}, {tuple(v_pages.shape)} do not fit kv_heads/page_size/head_dim")
    rotary_dim = head_dim
    if cos_sin is not None:
        # a rotation of the first rotary_dim <= head_dim elements of every head; the rest pass through
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= head_dim:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= head_dim")
    for w in (q_weight, k_weight, cos_sin, bias):
        if w is not None:
            _need(w, torch.float32, "weight/table")
    if bias is not None and bias.shape != (width,):
        raise KernelError(f"bias {tuple(bias.shape)} does not fit the {width} columns of qkv")
    fn = _fn(
        "elementwise",
        "me_qk_norm_rope_store",
        [c_void_p, c_int, c_longlong] + [c_void_p] * 2 + [c_float] + [c_void_p] * 8 + [c_int] * 7 + [c_void_p, c_int, c_void_p],
    )
    code = fn(
        _ptr(qkv), splits, qkv.stride(0), _ptr(q_weight), _ptr(k_weight), eps, _ptr(cos_sin), _ptr(positions),
        _ptr(slot_mapping if kv_heads else None), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(k_dense),
        _ptr(v_dense), _type_code(q_out.dtype), tokens, heads, kv_heads, head_dim, page_size, rotary_dim, _ptr(bias), value_dim, _stream(),
    )  # fmt: skip
    _check(code, "qk_norm_rope_store")


def rope_table(inv_freq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, i] = (cos, sin)(positions[t] * inv_freq[i])`` in float32, ``[T, rotary_dim / 2, 2]``."""
    _need(inv_freq, torch.float32, "inv_freq"), _need(positions, torch.int32, "positions"), _need(out, torch.float32, "out")
    tokens, half = positions.shape[0], inv_freq.shape[0]
    if tuple(out.shape) != (tokens, half, 2):
        raise KernelError(f"rope_table: out {tuple(out.shape)} is not [{tokens}, {half}, 2]")
    fn = _fn("elementwise", "me_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(inv_freq), _ptr(positions), _ptr(out), tokens, half, _stream()), "rope_table")


def kv_store(k_dense, v_dense, slot_mapping, k_pages, v_pages, kv_heads: int, head_dim: int, page_size: int) -> None:
    """Dense new keys/values ``[T, kv_heads * head_dim]`` into their cache slots."""
    for name, t in (("k_dense", k_dense), ("v_dense", v_dense), ("k_pages", k_pages), ("v_pages", v_pages)):
        _need(t, k_dense.dtype, name)
    _need(slot_mapping, torch.int32, "slot_mapping")
    fn = _fn("elementwise", "me_kv_store", [c_void_p] * 5 + [c_int] * 5 + [c_void_p])
    code = fn(
        _ptr(k_dense), _ptr(v_dense), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages), _type_code(k_dense.dtype),
        k_dense.shape[0], kv_heads, head_dim, page_size, _stream(),
    )  # fmt: skip
    _check(code, "kv_store")


# ----------------------------------------------------------------------------------- GEMMs


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out[T, N] (float32) = x[T, K] @ weight[N, K]^T`` on CUDA cores, ascending-k sums."""
    _need(x, weight.dtype, "x"), _need(weight, None, "weight"), _need(out, torch.float32, "out")
    tokens, inner = x.shape
    outs = weight.shape[0]
    if weight.shape[1] != inner or out.shape != (tokens, outs):
        raise KernelError(f"gemm_simt: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)}")
    fn = _fn("gemm_simt", "me_gemm_simt", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    code = fn(_ptr(x), _ptr(weight), _ptr(out), _type_code(x.dtype), tokens, outs, inner, _stream())
    _check(code, "gemm_simt")


def tensor_core_gemm_supports(outs: int, inner: int) -> bool:
    """TMA addresses rows whose pitch is a multiple of 16 bytes: ``inner % 8 == 0`` for
    bfloat16.  Other shapes take the CUDA-core kernel."""
    return tensor_core.supports(outs, inner)


def choose_splits(tokens: int, outs: int, inner: int, max_splits: int = 8) -> int:
    return tensor_core.choose_splits(tokens, outs, inner, max_splits)


def GemmPlan(weight: torch.Tensor, dual_rows: int | None = None):  # noqa: N802 - constructs a plan object
    return tensor_core.GemmPlan(weight, dual_rows)


def gemm_tensor_core(plan, x: torch.Tensor, out: torch.Tensor, splits: int) -> None:
    tensor_core.gemm(plan, x, out, splits)


def gemm_tensor_core_swiglu(plan, x: torch.Tensor, act: torch.Tensor, activation: str = "silu") -> None:
    tensor_core.gemm_swiglu(plan, x, act, activation=activation)


# -------------------------------------------------------------------------------- attention


def paged_attention_generic(
    q, k_pages, v_pages, block_table, entry_of_token, positions, out, heads, kv_heads, head_dim, scale, window,
    value_dim: int | None = None, sink: bool = False, gate: torch.Tensor | None = None,
    slopes: torch.Tensor | None = None, sink_values: torch.Tensor | None = None, softcap: float = 0.0,
) -> None:
    """One warp per (token, head), any head size; ``softcap`` > 0: a scaled score ``s`` becomes ``softcap * tanh(s /
    softcap)``; ``value_dim``: width of a value head when it differs;
    ``sink``: one more participant of score zero and no value in the softmax, or of the learned score
    ``sink_values[h]`` (float32 ``[heads]``); ``gate`` (float32 ``[T, heads]`` or ``[T, heads * value_dim]``): a
    multiplier on each head's output, or on each of its elements; ``slopes`` (float32 ``[heads]``): ``slopes[h] *
    (p - j)`` is taken off the scaled score of query ``p`` and key ``j``.  ``v_pages=None``: the values are the first
    ``value_dim`` elements of the key rows."""
    value_dim = head_dim if value_dim is None else value_dim
    gate_width = 1
    if gate is not None:
        _need(gate, torch.float32, "gate")
        if gate.shape == (q.shape[0], heads * value_dim) and value_dim > 1:
            gate_width = value_dim
        elif gate.shape != (q.shape[0], heads):
            raise KernelError("gate must be [tokens, heads] or [tokens, heads * value_dim]")
    for name, vector in (("slopes", slopes), ("sink_values", sink_values)):
        if vector is not None:
            _need(vector, torch.float32, name)
            if vector.shape != (heads,):
                raise KernelError(f"{name} must have one value per head")
    value_stride = value_dim
    if v_pages is None:
        if value_dim > head_dim:
            raise KernelError("values inside the key rows cannot be wider than the keys")
        v_pages, value_stride = k_pages, head_dim
    elif v_pages.shape[1:] != (kv_heads, k_pages.shape[2], value_dim):
        raise KernelError(f"value pages {tuple(v_pages.shape)} do not fit the head sizes")
    if k_pages.shape[1:] != (kv_heads, k_pages.shape[2], head_dim):
        raise KernelError(f"key pages {tuple(k_pages.shape)} do not fit the head sizes")
    _need(q, None, "q"), _need(out, q.dtype, "out"), _need(k_pages, q.dtype, "k_pages"), _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"), _need(entry_of_token, torch.int32, "entry_of_token")
    _need(positions, torch.int32, "positions")
    fn = _fn(
        "attention_generic",
        "me_paged_attention_generic",
        [c_void_p] * 7 + [c_int, c_float] + [c_int] * 9 + [c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p],
    )
    code = fn(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), _ptr(entry_of_token), _ptr(positions), _ptr(out),
        _type_code(q.dtype), scale, q.shape[0], heads, kv_heads, head_dim, k_pages.shape[2], block_table.shape[1],
        window, value_dim, 1 if (sink or sink_values is not None) else 0, _ptr(gate), gate_width, value_stride,
        _ptr(slopes), _ptr(sink_values), float(softcap or 0.0), _stream(),
    )  # fmt: skip
    _check(code, "paged_attention_generic")


def paged_attention(
    *, q, k_pages, v_pages, block_table, ctx, out, heads: int, kv_heads: int, head_dim: int, scale: float, window: int,
    value_dim: int | None = None, sink: bool = False, gate: torch.Tensor | None = None,
    slopes: torch.Tensor | None = None, sink_values: torch.Tensor | None = None, softcap: float = 0.0,
) -> None:  # fmt: skip
    """Causal attention of the batch's new tokens over their requests' cached keys (the new
    tokens' own keys are already in the cache).  Chooses the kernel by dtype and sizes.  ``value_dim``,
    ``sink``, ``gate``, ``slopes`` and ``sink_values`` as in :func:`paged_attention_generic`; value heads of another
    width than the key heads and values inside the key rows (``v_pages=None``) take that kernel."""
    if v_pages is None and q.dtype == torch.bfloat16 and latent_attention_supports(head_dim, value_dim, kv_heads):
        if sink or slopes is not None or sink_values is not None or softcap:
            raise KernelError("attention over latent rows takes a window and a gate per head, no sink, no distance bias and no cap")
        latent_attention_bf16(q, k_pages, block_table, ctx, out, heads, head_dim, value_dim, scale, window, gate)
        return
    if v_pages is not None and q.dtype == torch.bfloat16 and value_dim in (None, head_dim):
        if attention_bf16.supports(head_dim, heads, kv_heads):
            attention_bf16.paged_attention(
                q, k_pages, v_pages, block_table, ctx, out, heads, kv_heads, head_dim, scale, window, sink=sink, gate=gate,
                slopes=slopes, sink_values=sink_values, softcap=softcap,
            )  # fmt: skip
            return
    paged_attention_generic(
        q, k_pages, v_pages, block_table, ctx.entry_of_token, ctx.positions, out, heads, kv_heads, head_dim,
        scale, window, value_dim=value_dim, sink=sink, gate=gate, slopes=slopes, sink_values=sink_values, softcap=softcap,
    )  # fmt: skip


LATENT_ROWS, LATENT_SPAN = 32, 128  # (token, head) pairs of a CTA of the kernel below; keys of a CTA of a split request


def latent_attention_supports(width: int, rank: int | None, kv_heads: int = 1) -> bool:
    """Whether the tensor-core kernel takes rows of ``width`` elements whose first ``rank`` are the values."""
    return kv_heads == 1 and rank in (128, 256, 384, 512) and width % 64 == 0 and rank <= width and (160 * width + 2048) * 2 + 1024 <= 226 * 1024


LATENT_TENSOR_MEMORY = True  # tests set it to False to run the mma.sync kernel where the tcgen05 one would be taken
LATENT_TENSOR_MEMORY_MIN_ROWS = 64  # (token, head) pairs of the longest portion from which the tcgen05 kernel is taken
_latent_query_maps: dict[tuple[int, int, int], Any] = {}


def latent_tensor_memory_takes(width: int, rank: int, page_size: int, rows: int) -> bool:
    """Whether prompt portions whose longest has ``rows`` (token, head) pairs take the tcgen05 kernel: the query rows
    and one key tile must fit in shared memory, the output's halves must be whole 64-column blocks, pages whole
    parts of a 64-key tile."""
    return (LATENT_TENSOR_MEMORY and width % 64 == 0 and width <= 576 and rank in (128, 256, 384, 512) and rank <= width
            and page_size in (8, 16, 32, 64) and rows >= LATENT_TENSOR_MEMORY_MIN_ROWS)  # fmt: skip


def _latent_attention_tcgen05(q, pages, block_table, ctx, out, heads, width, rank, scale, window, gate, entries, ids, longest) -> None:
    key = (q.data_ptr(), q.shape[0], q.shape[1])
    q_map = _latent_query_maps.get(key)
    if q_map is None:
        if len(_latent_query_maps) > 8192:
            _latent_query_maps.clear()
        q_map = _latent_query_maps[key] = tensor_core._make_map(q.view(q.shape[0] * heads, width), 128)
    fn = _fn("latent_attention_tcgen05", "me_latent_attention_tcgen05",
             [c_void_p] * 8 + [c_float] + [c_int] * 8 + [c_void_p])  # fmt: skip
    code = fn(
        q_map, attention_bf16._page_map(pages), _ptr(block_table), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), _ptr(out),
        _ptr(gate), _ptr(ids), scale, entries, longest, heads, width, rank, pages.shape[2], block_table.shape[1], window,
        _stream(),
    )  # fmt: skip
    _check(code, "latent_attention_tcgen05")


def latent_attention_bf16(q, pages, block_table, ctx, out, heads: int, width: int, rank: int, scale: float, window: int,
                          gate: torch.Tensor | None = None) -> None:  # fmt: skip
    """Attention of the batch's new tokens over a cache of one latent row per token (``pages [pages, 1, page_size,
    width]``) that is key and, in its first ``rank`` elements, value for every head; ``q [T, heads * width]``, ``out [T,
    heads * rank]``, ``gate`` float32 ``[T, heads]``.  Entries that bring one token split their keys over several CTAs
    (spans of ``LATENT_SPAN`` keys by absolute position); the others take the tcgen05 kernel (two CTAs per 128 (token,
    head) pairs) when :func:`latent_tensor_memory_takes` says so, else one CTA per 32 pairs of the ``mma.sync`` kernel; a
    step that holds both kinds is two launches, each over its own list of entries."""
    for name, t in (("q", q), ("out", out), ("pages", pages)):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous bfloat16")
    if pages.dim() != 4 or pages.shape[1] != 1 or pages.shape[3] != width:
        raise KernelError(f"latent pages {tuple(pages.shape)} are not [pages, 1, page_size, {width}]")
    if q.shape != (out.shape[0], heads * width) or out.shape[1] != heads * rank:
        raise KernelError("q must be [tokens, heads * width] and out [tokens, heads * rank]")
    if gate is not None:
        _need(gate, torch.float32, "gate")
        if gate.shape != (q.shape[0], heads):
            raise KernelError("gate must be [tokens, heads]")
    _need(block_table, torch.int32, "block_table")
    fn = _fn("latent_attention_bf16", "me_latent_attention_bf16",
             [c_void_p] * 10 + [c_float] + [c_int] * 10 + [c_void_p])  # fmt: skip
    decodes = ctx.num_entries if ctx.all_decode else getattr(ctx, "num_decode_entries", 0)
    if decodes == ctx.num_entries:
        launches = [(True, decodes, None, 1)]
    elif decodes:
        launches = [(True, decodes, ctx.decode_entries, 1), (False, ctx.num_entries - decodes, ctx.portion_entries, ctx.max_query_len)]
    else:
        launches = [(False, ctx.num_entries, None, ctx.max_query_len)]
    for split, entries, ids, longest in launches:
        if not split and latent_tensor_memory_takes(width, rank, pages.shape[2], longest * heads):
            _latent_attention_tcgen05(q, pages, block_table, ctx, out, heads, width, rank, scale, window, gate, entries, ids, longest)
            continue
        partials = counters = None
        max_splits = 1
        if split:
            keys = min(window, ctx.max_context_len) if window > 0 else ctx.max_context_len
            max_splits = (keys - 1) // LATENT_SPAN + 2 if window > 0 else -(-keys // LATENT_SPAN)
            partials = ctx.workspace.growing("latent.partials", (ctx.num_entries, heads, max_splits, rank + 2), torch.float32)
        code = fn(
            _ptr(q), _ptr(pages), _ptr(block_table), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), _ptr(out), _ptr(gate),
            _ptr(partials), _ptr(counters), _ptr(ids), scale, entries, longest, heads, width, rank, pages.shape[2],
            block_table.shape[1], window, 1 if split else 0, max_splits, _stream(),
        )  # fmt: skip
        _check(code, "latent_attention_bf16")


def latent_down_finish(
    *, down: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, q_weight: torch.Tensor | None, kv_weight: torch.Tensor,
    eps: float, cos_sin: torch.Tensor | None, slot_mapping: torch.Tensor, q_latent: torch.Tensor | None, k_pages: torch.Tensor,
    gates: int = 0, gate_out: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """The row ``[query latent | c | k_rot | gates]`` of a fused down projection (``down``: ``[S, T, width]`` float32
    partial sums): RMS norm of the query latent into ``q_latent [T, q_rank]`` and of ``c`` (each with its weight),
    rotation of the first ``rotary_dim`` elements of ``k_rot``, the write of ``[c | k_rot]`` to the token's slot of
    ``k_pages [pages, 1, page_size, kv_rank + rot_dim]``, and ``sigmoid`` of the gates into ``gate_out [T, gates]``.
    ``q_rank=0``: the row has no query latent (``q_weight`` and ``q_latent`` are ``None``)."""
    _need(down, torch.float32, "down"), _need(k_pages, None, "k_pages"), _need(kv_weight, torch.float32, "kv_weight")
    if q_rank:
        _need(q_latent, k_pages.dtype, "q_latent"), _need(q_weight, torch.float32, "q_weight")
    elif q_latent is not None or q_weight is not None:
        raise KernelError("latent_down_finish: without a query latent there is neither its weight nor its output")
    _need(slot_mapping, torch.int32, "slot_mapping")
    splits, tokens, width = down.shape
    if width != q_rank + kv_rank + rot_dim + gates:
        raise KernelError(f"the down projection's width {width} is not q_rank + kv_rank + rot_dim + gates")
    if kv_weight.shape != (kv_rank,) or (q_rank and (q_weight.shape != (q_rank,) or q_latent.shape != (tokens, q_rank))):
        raise KernelError("latent_down_finish: norm weights or q_latent do not fit the ranks")
    if k_pages.dim() != 4 or k_pages.shape[1] != 1 or k_pages.shape[3] != kv_rank + rot_dim:
        raise KernelError(f"key pages {tuple(k_pages.shape)} are not [pages, 1, page_size, kv_rank + rot_dim]")
    rotary_dim = 0
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos_sin")
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= rot_dim:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= rot_dim")
    if gates:
        _need(gate_out, torch.float32, "gate_out")
        if gate_out.shape != (tokens, gates):
            raise KernelError("gate_out must be [tokens, gates]")
    fn = _fn("latent_attention", "me_latent_down_finish",
             [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_float] + [c_void_p] * 5 + [c_int] * 7 + [c_void_p])  # fmt: skip
    code = fn(
        _ptr(down), splits, down.stride(0), width, _ptr(q_weight), _ptr(kv_weight), float(eps), _ptr(cos_sin),
        _ptr(slot_mapping), _ptr(q_latent), _ptr(k_pages), _ptr(gate_out), _type_code(k_pages.dtype), tokens, q_rank,
        kv_rank, rot_dim, rotary_dim, gates, _stream(),
    )  # fmt: skip
    _check(code, "latent_down_finish")


HEAD_PRODUCT_TENSOR = True  # tests set it to False to run the plain kernel where the tensor-core one would be taken


def head_product(
    x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, *, tail: int = 0, cos_sin: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """``out[t, h, n] = sum_k x[t, h, k] * weight[h, k, n]`` for every head, ascending ``k``, float32 sums.  ``x`` is
    ``[T, heads * (inner + tail)]`` in the dtype of ``weight``, or float32 partial sums ``[S, T, heads * (inner +
    tail)]``; ``out`` is ``[T, heads * (outs + tail)]``.  The ``tail`` last columns of every head of ``x`` are appended to
    the head's output, the first ``rotary_dim`` of them rotated by ``cos_sin [T, rotary_dim / 2, 2]``."""
    _need(weight, None, "weight"), _need(out, weight.dtype, "out"), _need(x, None, "x")
    heads, inner, outs = weight.shape
    if x.dim() == 3:
        _need(x, torch.float32, "x")
        splits, stride, tokens = x.shape[0], x.stride(0), x.shape[1]
    else:
        splits, stride, tokens = 1, 0, x.shape[0]
        if x.dtype not in (torch.float32, weight.dtype):
            raise KernelError("head_product: x must be float32 or have the dtype of the weight")
    if x.shape[-1] != heads * (inner + tail) or out.shape != (tokens, heads * (outs + tail)):
        raise KernelError(f"head_product: {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} with a tail of {tail}")
    rotary_dim = 0
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos_sin")
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= tail:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= tail")
    if HEAD_PRODUCT_TENSOR and weight.dtype == torch.bfloat16 and inner % 64 == 0 and outs % 8 == 0 and tail % 8 == 0 and 64 * inner * 2 + 32768 <= 200 * 1024:
        fn = _fn("latent_attention_bf16", "me_head_product_bf16",
                 [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p])  # fmt: skip
        code = fn(
            _ptr(x), _type_code(x.dtype), splits, stride, _ptr(weight), _ptr(cos_sin), _ptr(out), tokens, heads, inner,
            outs, tail, rotary_dim, _stream(),
        )  # fmt: skip
        _check(code, "head_product_bf16")
        return
    fn = _fn("latent_attention", "me_head_product",
             [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p])  # fmt: skip
    code = fn(
        _ptr(x), _type_code(x.dtype), splits, stride, _ptr(weight), _ptr(cos_sin), _ptr(out), _type_code(weight.dtype),
        tokens, heads, inner, outs, tail, rotary_dim, _stream(),
    )  # fmt: skip
    _check(code, "head_product")


def biased_attention(
    *, q, k_pages, v_pages, block_table, entry_of_token, positions, out, heads: int, kv_heads: int, head_dim: int,
    value_dim: int, scale: float, window: int = 0, keep_first: int = 0, r1: torch.Tensor | None = None,
    r2: torch.Tensor | None = None, talk: torch.Tensor | None = None, spread: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """Attention of the batch's new tokens over their requests' cached keys with value heads of
    their own width, a window that keeps the first ``keep_first`` tokens, a distance bias ``r1[h] *
    ln(1 + r2[h] * distance)`` taken off the scores, and the heads' softmax weights mixed by
    ``talk [heads, heads]`` before they meet the values.  ``out`` is ``[T, heads * value_dim]`` in
    the dtype of ``q``; with ``talk``, ``spread`` is float32 scratch ``[T, heads, kv_heads,
    value_dim]``."""
    _need(q, None, "q"), _need(out, q.dtype, "out"), _need(k_pages, q.dtype, "k_pages"), _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"), _need(entry_of_token, torch.int32, "entry_of_token")
    _need(positions, torch.int32, "positions")
    tokens = q.shape[0]
    for name, vector in (("r1", r1), ("r2", r2)):
        if vector is not None:
            _need(vector, torch.float32, name)
            if vector.shape != (heads,):
                raise KernelError(f"{name} must have one value per head")
    if (r1 is None) != (r2 is None):
        raise KernelError("the distance bias takes both of its constants or none")
    if k_pages.shape[1:] != (kv_heads, k_pages.shape[2], head_dim) or v_pages.shape[1:] != (kv_heads, k_pages.shape[2], value_dim):
        raise KernelError(f"pages {tuple(k_pages.shape)}, {tuple(v_pages.shape)} do not fit the head sizes")
    if talk is not None:
        _need(talk, torch.float32, "talk"), _need(spread, torch.float32, "spread")
        if talk.shape != (heads, heads) or spread.numel() < tokens * heads * kv_heads * value_dim:
            raise KernelError("talk must be [heads, heads] and spread hold [T, heads, kv_heads, value_dim]")
    fn = _fn(
        "attention_biased",
        "me_biased_attention",
        [c_void_p] * 9 + [c_int, c_float] + [c_int] * 10 + [c_void_p],
    )
    code = fn(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), _ptr(entry_of_token), _ptr(positions), _ptr(r1), _ptr(r2),
        _ptr(spread if talk is not None else out), _type_code(q.dtype), float(scale), tokens, heads, kv_heads, head_dim,
        value_dim, k_pages.shape[2], block_table.shape[1], int(window), int(keep_first), 1 if talk is not None else 0, _stream(),
    )  # fmt: skip
    _check(code, "biased_attention")
    if talk is not None:
        mix = _fn("attention_biased", "me_mix_heads", [c_void_p] * 3 + [c_int] * 5 + [c_void_p])
        code = mix(_ptr(spread), _ptr(talk), _ptr(out), _type_code(out.dtype), tokens, heads, kv_heads, value_dim, _stream())
        _check(code, "mix_heads")


MIXED_ATTENTION_MAX_GROUP, MIXED_ATTENTION_MAX_VALUE_DIM = 8, 256


def mixed_attention(
    *, q, k_pages, v_pages, block_table, entry_of_token, positions, out, heads: int, kv_heads: int, head_dim: int,
    value_dim: int, scale: float, window: int, keep_first: int, r1: torch.Tensor | None, r2: torch.Tensor | None,
    talk: torch.Tensor, scores: torch.Tensor, stats: torch.Tensor, stride: int,
) -> None:  # fmt: skip
    """The attention of :func:`biased_attention` with mixed heads, in two kernels that keep the scores
    (``scores``: float32 scratch of ``T * heads * stride`` values, ``stride`` the most keys a query can see;
    ``stats``: ``T * heads * 2``) and apply every value once.  Groups of up to 8 query heads per KV head,
    value heads up to 256 wide."""
    _need(q, None, "q"), _need(out, q.dtype, "out"), _need(k_pages, q.dtype, "k_pages"), _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"), _need(entry_of_token, torch.int32, "entry_of_token")
    _need(positions, torch.int32, "positions"), _need(talk, torch.float32, "talk")
    _need(scores, torch.float32, "scores"), _need(stats, torch.float32, "stats")
    tokens = q.shape[0]
    for name, vector in (("r1", r1), ("r2", r2)):
        if vector is not None:
            _need(vector, torch.float32, name)
            if vector.shape != (heads,):
                raise KernelError(f"{name} must have one value per head")
    if k_pages.shape[1:] != (kv_heads, k_pages.shape[2], head_dim) or v_pages.shape[1:] != (kv_heads, k_pages.shape[2], value_dim):
        raise KernelError(f"pages {tuple(k_pages.shape)}, {tuple(v_pages.shape)} do not fit the head sizes")
    if talk.shape != (heads, heads) or scores.numel() < tokens * heads * stride or stats.numel() < tokens * heads * 2:
        raise KernelError("talk must be [heads, heads]; scores and stats must hold the step's (token, head) pairs")
    fn = _fn(
        "attention_biased",
        "me_mixed_attention",
        [c_void_p] * 11 + [c_int, c_void_p, c_int, c_float] + [c_int] * 9 + [c_void_p],
    )
    code = fn(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), _ptr(entry_of_token), _ptr(positions), _ptr(r1), _ptr(r2),
        _ptr(talk), _ptr(scores), _ptr(stats), int(stride), _ptr(out), _type_code(q.dtype), float(scale), tokens, heads,
        kv_heads, head_dim, value_dim, k_pages.shape[2], block_table.shape[1], int(window), int(keep_first), _stream(),
    )  # fmt: skip
    _check(code, "mixed_attention")


def branch_sum(branches: list[tuple[torch.Tensor, float]], out: torch.Tensor) -> None:
    """``out [T, width] = sum_b factor_b * sum_s partial_b[s]`` for up to four ``[S, T, width]`` float32
    partial-sum arrays."""
    _need(out, torch.float32, "out")
    count = len(branches)
    if not 1 <= count <= 4:
        raise KernelError("branch_sum takes one to four branches")
    for partial, _factor in branches:
        _need(partial, torch.float32, "partial")
        if partial.dim() != 3 or tuple(partial.shape[1:]) != tuple(out.shape):
            raise KernelError(f"branch {tuple(partial.shape)} does not fit out {tuple(out.shape)}")
    pointers = (c_void_p * count)(*[p.data_ptr() for p, _ in branches])
    splits = (c_int * count)(*[p.shape[0] for p, _ in branches])
    strides = (c_longlong * count)(*[p.stride(0) for p, _ in branches])
    factors = (c_float * count)(*[float(f) for _, f in branches])
    fn = _fn("elementwise", "me_branch_sum", [c_void_p] * 4 + [c_int, c_void_p, c_int, c_int, c_void_p])
    code = fn(pointers, splits, strides, factors, count, _ptr(out), out.shape[0], out.shape[1], _stream())
    _check(code, "branch_sum")


def gla_scan(
    *, proj: torch.Tensor, columns: dict[str, int], a2t: torch.Tensor, a2_bias: torch.Tensor, ctx, state: torch.Tensor,
    out: torch.Tensor, prepared: torch.Tensor, q_scale: float, tau: float, heads: int, dim: int, vdim: int,
) -> None:  # fmt: skip
    """The recurrence of gated linear attention over the batch's tokens, entry by entry, from and
    into each request's state slot.  ``proj`` is ``[S, T, width]`` float32 partial sums whose
    ``columns`` ``q, k, v, a`` say where each projection starts; ``a2t`` is the decay's second factor
    transposed, ``[rank, heads * dim]``; ``out`` is float32 ``[T, heads, vdim]``; ``prepared`` is float32
    scratch of ``T * heads * 3 * dim`` values (q, k and decay of every token, made by a first kernel)."""
    _need(proj, torch.float32, "proj"), _need(a2t, torch.float32, "a2t"), _need(a2_bias, torch.float32, "a2_bias")
    _need(state, torch.float32, "state"), _need(out, torch.float32, "out"), _need(prepared, torch.float32, "prepared")
    rank, tokens = a2t.shape[0], proj.shape[1]
    if a2t.shape != (rank, heads * dim) or a2_bias.shape != (heads * dim,) or state.shape[1:] != (heads, dim, vdim):
        raise KernelError("gla_scan: decay weights or state do not fit heads/dim/vdim")
    if prepared.numel() < tokens * heads * 3 * dim or out.numel() < tokens * heads * vdim:
        raise KernelError("gla_scan: scratch or output too small")
    fn = _fn(
        "linear_attention",
        "me_gla_scan",
        [c_void_p, c_int, c_longlong] + [c_int] * 5 + [c_void_p] * 8 + [c_float, c_float] + [c_int] * 6 + [c_void_p],
    )
    code = fn(
        _ptr(proj), proj.shape[0], proj.stride(0), proj.shape[2], columns["q"], columns["k"], columns["v"], columns["a"],
        _ptr(a2t), _ptr(a2_bias), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots), _ptr(ctx.fresh), _ptr(state), _ptr(out),
        _ptr(prepared), float(q_scale), float(tau), tokens, ctx.num_entries, heads, dim, vdim, rank, _stream(),
    )  # fmt: skip
    _check(code, "gla_scan")


def gla_finish(
    *, o: torch.Tensor, proj: torch.Tensor, gate_column: int, weight: torch.Tensor | None, eps: float, out: torch.Tensor,
    heads: int, vdim: int,
) -> None:  # fmt: skip
    """``out = weight * o / rms(o) * silu(gate)`` per (token, head); the gate is a column range of ``proj``;
    ``weight=None`` is a weight of ones."""
    _need(o, torch.float32, "o"), _need(proj, torch.float32, "proj"), _need(out, None, "out")
    if weight is not None:
        _need(weight, torch.float32, "weight")
    tokens = o.shape[0]
    fn = _fn(
        "linear_attention",
        "me_gla_finish",
        [c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_float, c_void_p] + [c_int] * 4 + [c_void_p],
    )
    code = fn(
        _ptr(o), _ptr(proj), proj.shape[0], proj.stride(0), proj.shape[2], gate_column, _ptr(weight), float(eps), _ptr(out),
        _type_code(out.dtype), tokens, heads, vdim, _stream(),
    )  # fmt: skip
    _check(code, "gla_finish")


RETENTION_CHUNK = 64  # tokens of a chunk of the chunked retention kernels


def retention_chunked_supports(dim: int, vdim: int) -> bool:
    """Whether the chunked kernels take these head sizes (multiples of four that fit a block's shared memory)."""
    fn = load_library("linear_attention").me_retention_chunked_supports
    fn.argtypes, fn.restype = [c_int, c_int], c_int
    return bool(fn(int(dim), int(vdim)))


def retention_scan(
    *, proj: torch.Tensor, columns: dict[str, int], cos_sin: torch.Tensor | None, decay: torch.Tensor, k_scale: float, ctx,
    state: torch.Tensor, out: torch.Tensor, prepared: torch.Tensor, heads: int, dim: int, vdim: int,
    chunk_min: int = 0, chunk_state: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """The recurrence ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` over the batch's tokens, entry by entry,
    from and into each request's state slot.  ``proj`` is ``[S, T, width]`` float32 partial sums whose ``columns`` ``q, k,
    v`` say where each projection starts; q and k are rotated by ``cos_sin [T, rotary_dim / 2, 2]`` (their first
    ``rotary_dim`` elements per head, rotate-half) and k is multiplied by ``k_scale``; ``decay`` is float32 ``[heads]``;
    ``out`` is float32 ``[T, heads, vdim]``; ``prepared`` is float32 scratch of ``T * heads * 3 * dim`` values.
    ``chunk_min`` > 0: entries of at least that many tokens run in chunks of ``RETENTION_CHUNK`` tokens whose blocks work
    side by side (the closed form of the recurrence over a chunk), with ``chunk_state [chunks, heads, dim, vdim]`` float32 as
    scratch for at least ``sum ceil(tokens / RETENTION_CHUNK)`` chunks; the other entries walk token by token."""
    _need(proj, torch.float32, "proj"), _need(decay, torch.float32, "decay"), _need(state, torch.float32, "state")
    max_chunks = 0
    if chunk_min:
        _need(chunk_state, torch.float32, "chunk_state")
        if chunk_state.dim() != 4 or chunk_state.shape[1:] != (heads, dim, vdim) or not retention_chunked_supports(dim, vdim):
            raise KernelError("retention_scan: the chunks' scratch is [chunks, heads, dim, vdim], and the head sizes must be ones the chunked kernels take")
        max_chunks = chunk_state.shape[0]
    _need(out, torch.float32, "out"), _need(prepared, torch.float32, "prepared")
    tokens = proj.shape[1]
    if decay.shape != (heads,) or state.shape[1:] != (heads, dim, vdim):
        raise KernelError("retention_scan: decay or state do not fit heads/dim/vdim")
    if prepared.numel() < tokens * heads * 3 * dim or out.numel() < tokens * heads * vdim:
        raise KernelError("retention_scan: scratch or output too small")
    rotary_dim = 0
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos_sin")
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= dim:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= dim")
    fn = _fn(
        "linear_attention",
        "me_retention_scan",
        [c_void_p, c_int, c_longlong] + [c_int] * 4 + [c_void_p, c_int, c_void_p, c_float] + [c_void_p] * 6 + [c_int] * 6
        + [c_void_p, c_int, c_void_p],
    )
    code = fn(
        _ptr(proj), proj.shape[0], proj.stride(0), proj.shape[2], columns["q"], columns["k"], columns["v"], _ptr(cos_sin),
        rotary_dim, _ptr(decay), float(k_scale), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots), _ptr(ctx.fresh), _ptr(state),
        _ptr(out), _ptr(prepared), tokens, ctx.num_entries, heads, dim, vdim, int(chunk_min), _ptr(chunk_state), max_chunks,
        _stream(),
    )  # fmt: skip
    _check(code, "retention_scan")


def _hyper_update(pending, mix, share, count):
    if pending is None:
        return 0, 0
    _need(pending, torch.float32, "pending"), _need(mix, torch.float32, "mix"), _need(share, torch.float32, "share")
    if mix.shape != (count, count) or share.shape != (count,):
        raise KernelError("hyper-connections: the mixing matrix is [streams, streams] and there is one share per stream")
    return pending.shape[0], pending.stride(0)


def hyper_step(
    *, streams: torch.Tensor, seed: torch.Tensor | None, pending: torch.Tensor | None, mix: torch.Tensor | None,
    share: torch.Tensor | None, mult: float, read: torch.Tensor | None, weight: torch.Tensor, eps: float,
    out: torch.Tensor, rows: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """One sublayer boundary of a model with several residual streams ``streams [S, T, hidden]`` (float32).  First the
    update that the previous sublayer's output ``pending [P, T, hidden]`` (partial sums) is owed: ``x_t = sum_s mix[s,
    t] x_s + mult * share[t] * sum_p pending[p]``, written back; then ``out = weight * rmsnorm(sum_t read[t] x_t)``.
    ``seed [T, hidden]``: the streams have not been written yet and all equal these rows.  ``pending=None``: no update,
    nothing is written.  ``read=None``: the plain sum of the streams.  ``rows`` (int32): only these rows, nothing is
    written back."""
    _need(streams, torch.float32, "streams"), _need(weight, torch.float32, "weight"), _need(out, None, "out")
    count, tokens, hidden = streams.shape
    splits, stride = _hyper_update(pending, mix, share, count)
    if pending is not None and pending.shape[1:] != (tokens, hidden):
        raise KernelError(f"hyper_step: pending {tuple(pending.shape)} does not fit the streams {tuple(streams.shape)}")
    if seed is not None:
        _need(seed, torch.float32, "seed")
        if seed.shape != (tokens, hidden):
            raise KernelError("hyper_step: the seed rows must be [tokens, hidden]")
    if read is not None:
        _need(read, torch.float32, "read")
        if read.shape != (count,):
            raise KernelError("hyper_step: one read weight per stream")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    produced = tokens if rows is None else rows.shape[0]
    if weight.shape != (hidden,) or out.shape != (produced, hidden):
        raise KernelError("hyper_step: weight or out do not fit")
    fn = _fn(
        "hyper_connections",
        "me_hyper_step",
        [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float,
         c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    )  # fmt: skip
    code = fn(
        _ptr(streams), streams.stride(0), _ptr(seed), _ptr(pending), splits, stride, _ptr(mix), _ptr(share), float(mult),
        _ptr(read), _ptr(weight), float(eps), _ptr(out), _type_code(out.dtype), _ptr(rows), produced, hidden, count, _stream(),
    )  # fmt: skip
    _check(code, "hyper_step")


def hyper_sum(
    *, streams: torch.Tensor, seed: torch.Tensor | None, pending: torch.Tensor | None, mix: torch.Tensor | None,
    share: torch.Tensor | None, mult: float, out: torch.Tensor,
) -> None:  # fmt: skip
    """``out [T, hidden]`` (float32): the sum of the residual streams after the update that ``pending`` is owed (see
    :func:`hyper_step`); nothing else is written."""
    _need(streams, torch.float32, "streams"), _need(out, torch.float32, "out")
    count, tokens, hidden = streams.shape
    splits, stride = _hyper_update(pending, mix, share, count)
    if out.shape != (tokens, hidden):
        raise KernelError("hyper_sum: out must be [tokens, hidden]")
    fn = _fn(
        "hyper_connections",
        "me_hyper_sum",
        [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    )
    code = fn(
        _ptr(streams), streams.stride(0), _ptr(seed), _ptr(pending), splits, stride, _ptr(mix), _ptr(share), float(mult),
        _ptr(out), tokens, hidden, count, _stream(),
    )  # fmt: skip
    _check(code, "hyper_sum")


PLAIN_ACTIVATIONS = {"relu_squared": 0, "silu": 1, "gelu_tanh": 2, "relu": 3}


def activation(partials: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """``out = act(sum_s partials[s])`` in the dtype of ``out``: ``relu_squared`` (``max(z, 0)^2``), ``silu``,
    ``gelu_tanh`` or ``relu``, for a feed-forward without a gate."""
    if kind not in PLAIN_ACTIVATIONS:
        raise KernelError(f"activation: kind must be one of {sorted(PLAIN_ACTIVATIONS)}, got {kind!r}")
    _need(partials, torch.float32, "partials"), _need(out, None, "out")
    splits, tokens, width = partials.shape
    if out.shape != (tokens, width):
        raise KernelError(f"activation: out {tuple(out.shape)} does not fit partials {tuple(partials.shape)}")
    fn = _fn("elementwise", "me_activation", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    code = fn(_ptr(partials), splits, partials.stride(0), _ptr(out), _type_code(out.dtype), tokens, width,
              PLAIN_ACTIVATIONS[kind], _stream())  # fmt: skip
    _check(code, "activation")


def qkv_rope_unit_store(
    *, qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int, value_dim: int, bias: torch.Tensor | None,
    cos_sin: torch.Tensor | None, unit_norm_eps: float | None, q_out: torch.Tensor, page_size: int,
    slot_mapping: torch.Tensor | None = None, k_pages: torch.Tensor | None = None, v_pages: torch.Tensor | None = None,
    k_dense: torch.Tensor | None = None, v_dense: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """``qkv [S, T, width]`` float32 partial sums with the columns ``[q | k | v]``: add ``bias`` (float32 ``[width]``),
    rotate the first ``rotary_dim`` elements of every q and k head by ``cos_sin [T, rotary_dim / 2, 2]``, then (with
    ``unit_norm_eps``) divide every rotated q and k head by its root mean square over ``head_dim``, eps inside the root;
    q goes to ``q_out``, k and v to their cache slots (or dense buffers)."""
    _need(qkv, torch.float32, "qkv"), _need(q_out, None, "q_out")
    splits, tokens, width = qkv.shape
    if width != (heads + kv_heads) * head_dim + kv_heads * value_dim:
        raise KernelError(f"qkv width {width} does not fit the head sizes")
    if slot_mapping is None and (k_dense is None or v_dense is None):
        raise KernelError("either slot_mapping with pages or dense outputs must be given")
    if slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
        if k_pages is None or v_pages is None or k_pages.dtype != q_out.dtype or v_pages.dtype != q_out.dtype:
            raise KernelError("pages must be given in the dtype of q_out")
        if k_pages.shape[1:] != (kv_heads, page_size, head_dim) or v_pages.shape[1:] != (kv_heads, page_size, value_dim):
            raise KernelError(f"pages {tuple(k_pages.shape)}, {tuple(v_pages.shape)} do not fit kv_heads/page_size/head_dim")
    rotary_dim = 0
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos_sin")
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= head_dim:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= head_dim")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.shape != (width,):
            raise KernelError(f"bias {tuple(bias.shape)} does not fit the {width} columns of qkv")
    fn = _fn("elementwise", "me_qkv_rope_unit_store",
             [c_void_p, c_int, c_longlong, c_int] + [c_void_p] * 8 + [c_float] + [c_int] * 9 + [c_void_p])  # fmt: skip
    code = fn(
        _ptr(qkv), splits, qkv.stride(0), width, _ptr(bias), _ptr(cos_sin), _ptr(slot_mapping), _ptr(q_out), _ptr(k_pages),
        _ptr(v_pages), _ptr(k_dense), _ptr(v_dense), float(unit_norm_eps or 0.0), _type_code(q_out.dtype), tokens, heads,
        kv_heads, head_dim, value_dim, page_size, rotary_dim, 1 if unit_norm_eps is not None else 0, _stream(),
    )  # fmt: skip
    _check(code, "qkv_rope_unit_store")


def pair_embedding(
    *, table: torch.Tensor, pair_table: torch.Tensor, ctx, last_token: torch.Tensor, out: torch.Tensor,
    rounded: torch.Tensor | None, multiplier: float, buckets: int, mul_prev: int, mul_cur: int,
) -> None:  # fmt: skip
    """``out[t] = table[id_t] * multiplier + pair_table[(previous id * mul_prev + id_t * mul_cur) mod buckets]`` in
    float32 (row ``buckets`` of ``pair_table`` for a sequence's first token).  The id in front of an entry's first
    token is read from ``last_token[slot]`` (int32 ``[slots + 1]``) unless the entry starts its sequence, and the
    entry's last id is left there.  ``rounded``: the same rows in the compute dtype, or ``None``."""
    _need(table, None, "table"), _need(pair_table, table.dtype, "pair_table"), _need(out, torch.float32, "out")
    _need(last_token, torch.int32, "last_token")
    vocab, hidden = table.shape
    if pair_table.shape != (buckets + 1, hidden):
        raise KernelError(f"pair_table {tuple(pair_table.shape)} is not [{buckets + 1}, {hidden}]")
    if rounded is not None:
        _need(rounded, None, "rounded")
    fn = _fn("elementwise", "me_pair_embedding",
             [c_void_p, c_void_p, c_int] + [c_void_p] * 8 + [c_int] * 5 + [c_longlong, c_longlong, c_float, c_void_p])  # fmt: skip
    code = fn(
        _ptr(table), _ptr(pair_table), _type_code(table.dtype), _ptr(ctx.token_ids), _ptr(ctx.entry_of_token),
        _ptr(ctx.cu_tokens), _ptr(ctx.state_slots), _ptr(ctx.fresh), _ptr(last_token), _ptr(out), _ptr(rounded),
        _type_code(rounded.dtype) if rounded is not None else F32, out.shape[0], hidden, vocab, int(buckets),
        int(mul_prev), int(mul_cur), float(multiplier), _stream(),
    )  # fmt: skip
    _check(code, "pair_embedding")


def round_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x`` (float32 ``[T, width]``) in the dtype of ``out``."""
    _need(x, torch.float32, "x"), _need(out, None, "out")
    if out.shape != x.shape:
        raise KernelError("round_rows: shapes differ")
    fn = _fn("elementwise", "me_round_rows", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(out), _type_code(out.dtype), x.shape[0], x.shape[1], _stream()), "round_rows")


def qk_wide_norm_rope_store(
    *, qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int, value_dim: int, q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None, q_out: torch.Tensor, page_size: int,
    slot_mapping: torch.Tensor | None = None, k_pages: torch.Tensor | None = None, v_pages: torch.Tensor | None = None,
    k_dense: torch.Tensor | None = None, v_dense: torch.Tensor | None = None, gates: int = 0,
    gate_out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """RMSNorm of q over all its ``heads * head_dim`` columns at once (weight of that size) and of k over its
    ``kv_heads * head_dim`` columns, rotation of the first ``rotary_dim`` elements of every head, and the write
    of k and v to their cache slots (or dense buffers).  ``qkv`` is ``[S, T, width]`` float32 partial sums with the
    columns ``[q | k | v | gates]``; the ``gates`` trailing columns come out as ``sigmoid`` in ``gate_out [T, gates]``.
    ``bias`` (float32, one value per column of ``qkv``) is added to the sums before anything else."""
    _need(qkv, torch.float32, "qkv"), _need(q_out, None, "q_out")
    splits, tokens, width = qkv.shape
    if width != (heads + kv_heads) * head_dim + kv_heads * value_dim + gates:
        raise KernelError(f"qkv width {width} does not fit the head sizes and {gates} gates")
    if kv_heads and slot_mapping is None and (k_dense is None or v_dense is None):
        raise KernelError("either slot_mapping with pages or dense outputs must be given")
    if kv_heads and slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
        if k_pages is None or v_pages is None or k_pages.dtype != q_out.dtype:
            raise KernelError("pages must be given in the dtype of q_out")
        if k_pages.shape[1:] != (kv_heads, page_size, head_dim) or v_pages.shape[1:] != (kv_heads, page_size, value_dim):
            raise KernelError(f"pages {tuple(k_pages.shape)}, {tuple(v_pages.shape)} do not fit kv_heads/page_size/head_dim")
    rotary_dim = 0
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos_sin")
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= head_dim:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= head_dim")
    if q_weight is not None:
        _need(q_weight, torch.float32, "q_weight")
        if q_weight.shape != (heads * head_dim,):
            raise KernelError("q_weight must have one value per column of q")
    if k_weight is not None and kv_heads:
        _need(k_weight, torch.float32, "k_weight")
        if k_weight.shape != (kv_heads * head_dim,):
            raise KernelError("k_weight must have one value per column of k")
    if gates:
        _need(gate_out, torch.float32, "gate_out")
        if gate_out.shape != (tokens, gates):
            raise KernelError("gate_out must be [tokens, gates]")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.shape != (width,):
            raise KernelError(f"bias {tuple(bias.shape)} does not fit the {width} columns of qkv")
    fn = _fn("elementwise", "me_qk_wide_norm_rope_store",
             [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_float] + [c_void_p] * 8 + [c_int] * 9 + [c_void_p, c_void_p])  # fmt: skip
    code = fn(
        _ptr(qkv), splits, qkv.stride(0), width, _ptr(q_weight), _ptr(k_weight if kv_heads else None), float(eps),
        _ptr(cos_sin), _ptr(slot_mapping if kv_heads else None), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(k_dense),
        _ptr(v_dense), _ptr(gate_out), _type_code(q_out.dtype), tokens, heads, kv_heads, head_dim, value_dim, page_size,
        rotary_dim, gates, _ptr(bias), _stream(),
    )  # fmt: skip
    _check(code, "qk_wide_norm_rope_store")


def rglru(
    *, proj: torch.Tensor, in_bias: torch.Tensor, taps: torch.Tensor, conv_bias: torch.Tensor, ra_t: torch.Tensor,
    ra_bias: torch.Tensor, ri_t: torch.Tensor, ri_bias: torch.Tensor, lam: torch.Tensor, ctx, state: torch.Tensor,
    decay: torch.Tensor, driven: torch.Tensor, conv: torch.Tensor, out: torch.Tensor, sharpness: float,
) -> None:  # fmt: skip
    """A gated linear recurrence per channel over the batch's tokens, entry by entry, from and into each request's
    state slot.  ``proj`` is ``[S, T, 2 C]`` float32 partial sums (gate branch, then recurrent branch); ``taps [C, K]``
    a causal convolution on the recurrent branch; ``ra_t``, ``ri_t`` ``[blocks, in, out]`` the two gates' block
    matrices, transposed; ``state`` is ``[slots + 1, K, C]`` float32 (row 0 the recurrence, then the convolution's
    last ``K - 1`` inputs); ``decay``, ``driven`` and ``conv`` are float32 scratch ``[T, C]``; ``out [T, C]`` is the state
    times ``gelu_tanh`` of the gate branch in the compute dtype; ``sharpness`` is ``c`` of ``a = exp(-c r softplus(lam))``."""
    for name, t in (("proj", proj), ("in_bias", in_bias), ("taps", taps), ("conv_bias", conv_bias), ("ra_t", ra_t),
                    ("ra_bias", ra_bias), ("ri_t", ri_t), ("ri_bias", ri_bias), ("lam", lam), ("state", state),
                    ("decay", decay), ("driven", driven), ("conv", conv)):  # fmt: skip
        _need(t, torch.float32, name)
    _need(out, None, "out")
    splits, tokens, width = proj.shape
    channels, taps_count = taps.shape
    blocks = ra_t.shape[0]
    block_width = channels // blocks
    if width != 2 * channels or in_bias.shape != (width,) or channels % blocks:
        raise KernelError("rglru: the projection must hold two branches of `channels` columns")
    if ra_t.shape != (blocks, block_width, block_width) or ri_t.shape != ra_t.shape:
        raise KernelError("rglru: the gates' matrices must be [blocks, channels / blocks, channels / blocks]")
    for name, t in (("conv_bias", conv_bias), ("ra_bias", ra_bias), ("ri_bias", ri_bias), ("lam", lam)):
        if t.shape != (channels,):
            raise KernelError(f"rglru: {name} must have one value per channel")
    if state.shape[1:] != (taps_count, channels) or out.shape != (tokens, channels):
        raise KernelError("rglru: state must be [slots + 1, taps, channels] and out [tokens, channels]")
    if min(decay.numel(), driven.numel(), conv.numel()) < tokens * channels:
        raise KernelError("rglru: scratch too small")
    fn = _fn("recurrent", "me_rglru", [c_void_p, c_int, c_longlong] + [c_void_p] * 17 + [c_int] * 6 + [c_float, c_void_p])
    code = fn(
        _ptr(proj), splits, proj.stride(0), _ptr(in_bias), _ptr(taps), _ptr(conv_bias), _ptr(ra_t), _ptr(ra_bias),
        _ptr(ri_t), _ptr(ri_bias), _ptr(lam), _ptr(ctx.entry_of_token), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots),
        _ptr(ctx.fresh), _ptr(state), _ptr(decay), _ptr(driven), _ptr(conv), _ptr(out), _type_code(out.dtype), tokens,
        ctx.num_entries, channels, blocks, taps_count, float(sharpness), _stream(),
    )  # fmt: skip
    _check(code, "rglru")


ROUTE_SCORINGS = {"sigmoid": 0, "softmax_chosen": 1}


def route(
    *, h: torch.Tensor, router: torch.Tensor, weights: torch.Tensor, chosen: torch.Tensor, chosen_weight: torch.Tensor,
    top: int, group_count: int, group_keep: int, weight_scale: float, bias: torch.Tensor | None = None,
    scoring: str = "sigmoid",
) -> None:  # fmt: skip
    """Per token the ``top`` units with the largest ``sigmoid(router h)`` among the units of the ``group_keep`` best
    of ``group_count`` equal groups of neighbours (a group's value: the sum of its two largest scores); weights are
    the chosen scores over their sum, times ``weight_scale``.  ``weights [T, units]`` float32 gets them densely (zero
    elsewhere), ``chosen`` (int32) and ``chosen_weight`` (float32) ``[T, top]`` as lists.  ``bias`` (float32 ``[units]``)
    is added to ``router h``.  ``scoring="softmax_chosen"``: the units with the largest logits are chosen and their weights
    are the softmax over the chosen logits only (times ``weight_scale``)."""
    if scoring not in ROUTE_SCORINGS:
        raise KernelError(f"route: scoring must be one of {sorted(ROUTE_SCORINGS)}, got {scoring!r}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.shape != (router.shape[0],):
            raise KernelError("route: one bias per unit")
    _need(h, None, "h"), _need(router, torch.float32, "router"), _need(weights, torch.float32, "weights")
    _need(chosen, torch.int32, "chosen"), _need(chosen_weight, torch.float32, "chosen_weight")
    tokens, hidden = h.shape
    units = router.shape[0]
    if router.shape != (units, hidden) or weights.shape != (tokens, units) or chosen.shape != (tokens, top) or chosen_weight.shape != (tokens, top):
        raise KernelError("route: shapes do not fit")
    fn = _fn("routing", "me_route", [c_void_p, c_int, c_void_p, c_void_p, c_int] + [c_void_p] * 3 + [c_int] * 6 + [c_float, c_void_p])
    code = fn(
        _ptr(h), _type_code(h.dtype), _ptr(router), _ptr(bias), ROUTE_SCORINGS[scoring], _ptr(weights), _ptr(chosen), _ptr(chosen_weight), tokens, hidden,
        units, int(top), int(group_count), int(group_keep), float(weight_scale), _stream(),
    )  # fmt: skip
    _check(code, "route")


def sort_by_unit(*, chosen: torch.Tensor, units: int, pad: int, row_of: torch.Tensor, token_of: torch.Tensor,
                 unit_of_block: torch.Tensor) -> None:  # fmt: skip
    """Rows sorted by unit for grouped products: every (token, choice) of ``chosen [T, top]`` gets a row, each unit's
    run padded to a multiple of ``pad``.  ``row_of [T, top]``, ``token_of [capacity]`` (-1: no token) and
    ``unit_of_block [capacity / pad]`` (-1: no rows) are int32 outputs; ``capacity >= T * top + units * (pad - 1)``."""
    for name, t in (("chosen", chosen), ("row_of", row_of), ("token_of", token_of), ("unit_of_block", unit_of_block)):
        _need(t, torch.int32, name)
    tokens, top = chosen.shape
    capacity = token_of.shape[0]
    if row_of.shape != chosen.shape or capacity % pad or unit_of_block.shape[0] < capacity // pad:
        raise KernelError("sort_by_unit: shapes do not fit")
    fn = _fn("routing", "me_sort_by_unit", [c_void_p] + [c_int] * 5 + [c_void_p] * 4)
    code = fn(_ptr(chosen), tokens, top, int(units), int(pad), capacity, _ptr(row_of), _ptr(token_of), _ptr(unit_of_block), _stream())
    _check(code, "sort_by_unit")


def gather_rows(h: torch.Tensor, token_of: torch.Tensor, out: torch.Tensor) -> None:
    """``out[r] = h[token_of[r]]``, zeros where ``token_of[r] < 0``; rows of a multiple of 16 bytes."""
    _need(h, None, "h"), _need(out, h.dtype, "out"), _need(token_of, torch.int32, "token_of")
    if out.shape != (token_of.shape[0], h.shape[1]):
        raise KernelError("gather_rows: shapes do not fit")
    fn = _fn("routing", "me_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(h), _ptr(token_of), _ptr(out), out.shape[0], h.shape[1] * h.element_size(), _stream()), "gather_rows")


def combine_rows(sorted_out: torch.Tensor, row_of: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t] = sum_k weight[t, k] * sorted_out[row_of[t, k]]`` in the order of ``k``, float32."""
    _need(sorted_out, torch.float32, "sorted_out"), _need(row_of, torch.int32, "row_of")
    _need(weight, torch.float32, "weight"), _need(out, torch.float32, "out")
    tokens, top = row_of.shape
    if weight.shape != row_of.shape or out.shape != (tokens, sorted_out.shape[1]):
        raise KernelError("combine_rows: shapes do not fit")
    fn = _fn("routing", "me_combine_rows", [c_void_p] * 4 + [c_int] * 3 + [c_void_p])
    _check(fn(_ptr(sorted_out), _ptr(row_of), _ptr(weight), _ptr(out), tokens, top, out.shape[1], _stream()), "combine_rows")


def gemm_tensor_core_grouped(plan, x, out, group_of_block, group_rows, outs, dual_rows=0, slope=1.0, limit=None, offset=0.0) -> None:
    tensor_core.gemm_grouped(plan, x, out, group_of_block, group_rows, outs, dual_rows, slope, limit, offset)


GROUP_PAD = 128  # rows of a run of sorted rows (tensor_core.GROUP_PAD)


# --------------------------------------------------------------------------------- sampling


def sample(logits: torch.Tensor, temperatures: torch.Tensor | None, uniforms: torch.Tensor | None, out: torch.Tensor) -> None:
    """Per row: argmax (lowest index among maxima) when its temperature is 0, else the token
    at which the cumulative distribution of ``softmax(logits / T)`` passes ``uniforms[row]``."""
    _need(logits, torch.float32, "logits"), _need(out, torch.int32, "out")
    rows, vocab = logits.shape
    if temperatures is not None:
        _need(temperatures, torch.float32, "temperatures"), _need(uniforms, torch.float32, "uniforms")
    fn = _fn("sampling", "me_sample", [c_void_p] * 4 + [c_int, c_int, c_void_p])
    code = fn(_ptr(logits), _ptr(temperatures), _ptr(uniforms), _ptr(out), rows, vocab, _stream())
    _check(code, "sample")


# The bindings of the tensor-core and attention libraries use this module's helpers and are used
# by its wrappers: they are imported last, when everything above exists.
from mini_engine_b200.csrc import attention_bf16, tensor_core  # noqa: E402

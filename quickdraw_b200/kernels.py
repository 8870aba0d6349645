"""Host side of the operator table: the reference's six operator names, its extra
matvec/routing entry points and the composed token step, each a thin ctypes call into
the sm_100a library (reference surface: quickdraw/kernel/__init__.py:6-28,
quickdraw/kernel/triton/__init__.py:4-13, quickdraw/kernel/cute/matvec.py:146-159,
quickdraw/kernel/cute/moe.py:87-116).

Contract violations raise ``AssertionError`` before any launch, as the reference's
wrappers do.  Outputs are fresh tensors; state tensors are updated in place; every
launch goes to the current CUDA stream of the input's device and is graph-capturable.
There is no CPU execution path: tensors must live on a CUDA device.
"""

from __future__ import annotations

from functools import partial

import torch

from . import _lib
from ._lib import call, ptr, stream_of
from .weights import FP8Linear, NVFP4Linear

BF16 = torch.bfloat16


def _is_cuda_bf16(x):
    return x.is_cuda and x.dtype == BF16 and x.is_contiguous()


def _check_fp4(x, proj: NVFP4Linear):
    assert _is_cuda_bf16(x), "activations must be contiguous bf16 on a CUDA device"
    assert x.shape[-1] == proj.in_features
    assert proj.weight.dtype == torch.uint8 and proj.weight.is_contiguous()
    assert proj.weight_scale.dtype == torch.float8_e4m3fn and proj.weight_scale.is_contiguous()
    assert proj.weight_scale_2.dtype == torch.float32
    assert proj.group_size % 2 == 0 and proj.in_features % proj.group_size == 0
    assert proj.weight_scale.shape == (*proj.weight.shape[:-1], proj.in_features // proj.group_size)
    assert x.device == proj.weight.device == proj.weight_scale.device == proj.weight_scale_2.device


# ------------------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis with an explicit gamma; bf16 or fp32 in, same out."""
    assert x.is_cuda and x.is_contiguous() and x.dtype in (BF16, torch.float32)
    width = x.shape[-1]
    assert gamma.numel() == width and gamma.device == x.device
    gamma = gamma.float().contiguous()
    out = torch.empty_like(x)
    call("qd_rms_norm", ptr(x), ptr(gamma), ptr(out), x.numel() // width, width, float(eps),
         int(x.dtype == torch.float32), stream_of(x))
    return out


def add_rms_norm(x, residual, gamma, eps):
    """(bf16(rms_norm(x + residual) * gamma), bf16(x + residual)); residual may be None."""
    assert _is_cuda_bf16(x) and x.ndim == 1
    assert residual is None or (_is_cuda_bf16(residual) and residual.shape == x.shape)
    assert gamma.dtype == torch.float32 and gamma.is_contiguous() and gamma.numel() == x.numel()
    normed, new_residual = torch.empty_like(x), torch.empty_like(x)
    call("qd_add_rms_norm", ptr(x), ptr(residual), ptr(gamma), ptr(normed), ptr(new_residual),
         x.numel(), float(eps), stream_of(x))
    return normed, new_residual


# ----------------------------------------------------------------------------- matvec
def _scalar_f32(value, device):
    if isinstance(value, torch.Tensor):
        assert value.numel() == 1
        return value.to(device=device, dtype=torch.float32).reshape(1).contiguous()
    return torch.tensor([float(value)], dtype=torch.float32, device=device)


def bf16_gemv(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """bf16 [in] times bf16 [out, in] -> bf16 [out], fp32 accumulation."""
    assert _is_cuda_bf16(x) and x.ndim == 1 and _is_cuda_bf16(weight) and weight.ndim == 2
    assert weight.shape[1] == x.numel() and weight.device == x.device
    out = torch.empty(weight.shape[0], dtype=BF16, device=x.device)
    call("qd_bf16_gemv", ptr(x), ptr(weight), ptr(out), weight.shape[0], weight.shape[1], stream_of(x))
    return out


def nvfp4_gemv(x: torch.Tensor, proj, *, routing_weight=None, force_generic: bool = False) -> torch.Tensor:
    """Single bf16 vector times a packed NVFP4 matrix (or, for a bf16 LM head, a plain
    bf16 matrix); with ``routing_weight`` the routed double rounding applies."""
    if isinstance(proj, torch.Tensor):
        assert routing_weight is None
        return bf16_gemv(x, proj)
    if x.ndim == 2:            # a chunk of tokens (prefill): the tensor-core path
        assert routing_weight is None
        return matmul(x, proj)
    assert x.ndim == 1 and proj.weight.ndim == 2
    _check_fp4(x, proj)
    assert proj.weight_scale_2.numel() == 1
    routing = None if routing_weight is None else _scalar_f32(routing_weight, x.device)
    out = torch.empty(proj.out_features, dtype=BF16, device=x.device)
    call("qd_nvfp4_gemv", ptr(x), ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.weight_scale_2),
         ptr(routing), ptr(out), proj.out_features, proj.in_features, proj.group_size,
         int(force_generic), stream_of(x))
    return out


_matmul_status: dict = {}


def matmul(x: torch.Tensor, proj: NVFP4Linear) -> torch.Tensor:
    """bf16 [tokens, in] times a packed NVFP4 matrix on the tensor cores (prefill projection;
    reference: quickdraw/kernel/triton/matvec.py:153-163): weights expanded to
    bf16(code * block scale), fp32 accumulation, global scale last, bf16 output [tokens, out]."""
    assert isinstance(proj, NVFP4Linear) and x.ndim == 2 and proj.weight.ndim == 2
    assert x.is_cuda and x.dtype == BF16 and x.is_contiguous() and x.shape[1] == proj.in_features
    assert proj.weight.is_contiguous() and proj.weight_scale.is_contiguous() and proj.group_size == 16
    assert proj.weight_scale_2.numel() == 1 and proj.in_features % 64 == 0 and proj.out_features % 8 == 0
    status = _matmul_status.get(x.device)
    if status is None:
        status = _matmul_status[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    out = torch.empty((x.shape[0], proj.out_features), dtype=BF16, device=x.device)
    call("qd_nvfp4_matmul", ptr(x), ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.weight_scale_2),
         ptr(out), x.shape[0], proj.out_features, proj.in_features, proj.group_size, ptr(status), stream_of(x))
    return out


def matmul_rows(x: torch.Tensor, proj: NVFP4Linear, scratch: torch.Tensor | None = None, *, convert: bool = True,
                x_up: torch.Tensor | None = None):
    """``matmul`` for at most 32 token rows (a decode batch): the weights are decoded once on the
    warp-level tensor-core instruction with the tokens as columns.  ``scratch`` (uint8,
    ``rows_scratch_bytes(in_features)``) receives the f16 copy of the rows; ``convert=False``
    reuses what the previous call left there (several projections of the same input).
    ``x_up``: the input rows are bf16(bf16(silu(x)) * x_up), formed on the way in.
    in_features a multiple of 512, out_features of 16.  Returns (y, scratch)."""
    assert isinstance(proj, NVFP4Linear) and x.ndim == 2 and proj.weight.ndim == 2 and x.shape[0] <= 32
    assert x.is_cuda and x.dtype == BF16 and x.is_contiguous() and x.shape[1] == proj.in_features
    assert proj.weight.is_contiguous() and proj.weight_scale.is_contiguous() and proj.group_size == 16
    assert proj.weight_scale_2.numel() == 1 and proj.in_features % 512 == 0 and proj.out_features % 16 == 0
    if scratch is None:
        assert convert
        scratch = torch.empty(rows_scratch_bytes(proj.in_features), dtype=torch.uint8, device=x.device)
    assert scratch.is_cuda and scratch.numel() >= rows_scratch_bytes(proj.in_features)
    out = torch.empty((x.shape[0], proj.out_features), dtype=BF16, device=x.device)
    assert x_up is None or (x_up.shape == x.shape and x_up.dtype == BF16 and x_up.is_contiguous() and x_up.device == x.device)
    call("qd_nvfp4_matmul_rows", ptr(x), ptr(x_up), ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.weight_scale_2), ptr(out),
         x.shape[0], proj.out_features, proj.in_features, proj.group_size, ptr(scratch), int(convert), stream_of(x))
    return out, scratch


def rows_scratch_bytes(in_features: int) -> int:
    return int(_lib.lib().qd_nvfp4_matmul_rows_scratch_bytes(in_features))


def quantize_act(x: torch.Tensor):
    """bf16 [tokens, in] -> the activation operand of the FP4 x FP4 product: (codes uint8
    [tokens, in/2], E4M3 block scales [tokens, in/16], fp32 tensor scale), the layout of an
    ``NVFP4Linear`` (quickdraw/models/weights.py:29-47); every rounding to nearest even."""
    assert x.is_cuda and x.dtype == BF16 and x.ndim == 2 and x.is_contiguous() and x.shape[1] % 16 == 0
    tokens, width = x.shape
    codes = torch.empty((tokens, width // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((tokens, width // 16), dtype=torch.float8_e4m3fn, device=x.device)
    scale_2 = torch.empty((), dtype=torch.float32, device=x.device)
    scratch = torch.empty(1, dtype=torch.int32, device=x.device)
    call("qd_nvfp4_quantize_act", ptr(x), tokens, width, ptr(codes), ptr(scales), ptr(scale_2), ptr(scratch), stream_of(x))
    return codes, scales, scale_2


def matmul_w4a4(xq, proj: NVFP4Linear, *, wide_tiles: bool | None = None) -> torch.Tensor:
    """Quantised activations (``quantize_act``) times a packed NVFP4 matrix on the block-scaled
    FP4 tensor core: neither operand is expanded.  Differs from ``matmul`` by the activation
    rounding only (the W4A4 variant quickdraw's notes ask to validate separately from W4A16);
    in_features a multiple of 256, out_features a multiple of 128.  ``wide_tiles``: 256 weight rows
    per block and MMA (needs out_features % 256 == 0) instead of 128; None lets the library choose."""
    codes, scales, scale_2 = xq
    assert isinstance(proj, NVFP4Linear) and proj.weight.ndim == 2 and proj.group_size == 16
    assert codes.is_cuda and codes.dtype == torch.uint8 and codes.is_contiguous() and scales.is_contiguous()
    assert codes.shape[1] * 2 == proj.in_features and proj.in_features % 256 == 0 and proj.out_features % 128 == 0
    assert proj.weight.is_contiguous() and proj.weight_scale.is_contiguous() and proj.weight_scale_2.numel() == 1
    status = _matmul_status.get(codes.device)
    if status is None:
        status = _matmul_status[codes.device] = torch.zeros(1, dtype=torch.int32, device=codes.device)
    out = torch.empty((codes.shape[0], proj.out_features), dtype=BF16, device=codes.device)
    call("qd_nvfp4_matmul_w4a4", ptr(codes), ptr(scales), ptr(scale_2), ptr(proj.weight), ptr(proj.weight_scale),
         ptr(proj.weight_scale_2), ptr(out), codes.shape[0], proj.out_features, proj.in_features,
         -1 if wide_tiles is None else int(wide_tiles), ptr(status), stream_of(codes))
    return out


def matmul_status(device) -> int:
    """Status word of the tensor-core matmul on ``device`` (0 = clean; bit 0 = a bounded wait ran out)."""
    status = _matmul_status.get(torch.device(device))
    return 0 if status is None else int(status.item())


def expert_gemv(x, proj: NVFP4Linear, ids, weights=None, *, force_generic: bool = False):
    """Rows of the selected experts of a bank: y[slot] = W[ids[slot]] x (or x[slot])."""
    _check_fp4(x, proj)
    assert proj.weight.ndim == 3 and x.ndim in (1, 2)
    assert ids.device == x.device and ids.dtype == torch.int32 and ids.ndim == 1 and ids.is_contiguous()
    slots = ids.numel()
    assert x.ndim == 1 or x.shape[0] == slots
    assert proj.weight_scale_2.numel() in (1, proj.weight.shape[0])
    if weights is not None:
        assert weights.device == x.device and weights.dtype == torch.float32
        assert weights.shape == ids.shape and weights.is_contiguous()
    out = torch.empty((slots, proj.out_features), dtype=BF16, device=x.device)
    call("qd_nvfp4_expert_gemv", ptr(x), ptr(proj.weight), ptr(proj.weight_scale),
         ptr(proj.weight_scale_2), ptr(ids), ptr(weights), ptr(out), proj.out_features,
         proj.in_features, proj.group_size, slots, int(x.ndim == 2),
         int(proj.weight_scale_2.numel() != 1), int(force_generic), stream_of(x))
    return out


def gate_up(x, gate: NVFP4Linear, up: NVFP4Linear, ids=None, *, force_generic: bool = False):
    """bf16(silu(bf16 gate.x)) * bf16(up.x) for one projection pair or selected experts."""
    _check_fp4(x, gate)
    _check_fp4(x, up)
    assert x.ndim == 1 and up.weight.shape == gate.weight.shape and up.group_size == gate.group_size
    assert up.weight_scale_2.shape == gate.weight_scale_2.shape
    bank = ids is not None
    assert gate.weight.ndim == (3 if bank else 2)
    if bank:
        assert ids.device == x.device and ids.dtype == torch.int32 and ids.ndim == 1 and ids.is_contiguous()
        assert gate.weight_scale_2.numel() in (1, gate.weight.shape[0])
    else:
        assert gate.weight_scale_2.numel() == 1
    slots = ids.numel() if bank else 1
    out = torch.empty((slots, gate.out_features) if bank else (gate.out_features,), dtype=BF16, device=x.device)
    call("qd_nvfp4_gate_up", ptr(x), ptr(gate.weight), ptr(gate.weight_scale), ptr(gate.weight_scale_2),
         ptr(up.weight), ptr(up.weight_scale), ptr(up.weight_scale_2), ptr(ids), ptr(out),
         gate.out_features, gate.in_features, gate.group_size, slots,
         int(bank and gate.weight_scale_2.numel() != 1), int(force_generic), stream_of(x))
    return out


def dequantize(proj: NVFP4Linear, *, hardware_convert: bool = True) -> torch.Tensor:
    """fp32 dequantisation of a 2-D projection or of every expert of a bank (scalar global)."""
    assert proj.weight.is_cuda and proj.weight.is_contiguous() and proj.weight_scale.is_contiguous()
    assert proj.weight_scale_2.numel() == 1
    out = torch.empty((*proj.weight.shape[:-1], proj.in_features), dtype=torch.float32,
                      device=proj.weight.device)
    rows = proj.weight.numel() // proj.weight.shape[-1]
    call("qd_nvfp4_dequantize", ptr(proj.weight), ptr(proj.weight_scale), float(proj.weight_scale_2),
         ptr(out), rows, proj.in_features, proj.group_size, int(hardware_convert), stream_of(proj.weight))
    return out


def fp8_gemv(x: torch.Tensor, proj) -> torch.Tensor:
    """Static-FP8 projection; an NVFP4 container in its place is routed to nvfp4_gemv so
    mixers accept either kind of projection."""
    if isinstance(proj, NVFP4Linear):
        return nvfp4_gemv(x, proj)
    assert x.is_cuda and x.ndim == 1 and x.is_contiguous() and x.dtype in (BF16, torch.float32)
    assert proj.weight.ndim == 2 and proj.weight.is_contiguous() and proj.weight.dtype == torch.float8_e4m3fn
    assert x.numel() == proj.in_features
    assert proj.input_scale is not None and proj.input_scale.numel() == 1 and proj.weight_scale.numel() == 1
    w_scale = proj.weight_scale.to(device=x.device, dtype=torch.float32).reshape(1)
    in_scale = proj.input_scale.to(device=x.device, dtype=torch.float32).reshape(1)
    out = torch.empty(proj.out_features, dtype=x.dtype, device=x.device)
    call("qd_fp8_gemv", ptr(x), ptr(proj.weight), ptr(w_scale), ptr(in_scale), ptr(out),
         proj.out_features, proj.in_features, int(x.dtype == torch.float32), stream_of(x))
    return out


def _project(x, proj):
    return fp8_gemv(x, proj) if isinstance(proj, FP8Linear) else nvfp4_gemv(x, proj)


# -------------------------------------------------------------------------------- MoE
def route(logits: torch.Tensor, topk: int):
    """(int32 ids in selection order, fp32 renormalised weights); lowest index wins ties."""
    assert logits.is_cuda and logits.is_contiguous() and logits.ndim == 1
    assert logits.dtype in (BF16, torch.float32)
    experts = logits.numel()
    assert 1 <= topk <= experts and topk <= 32 and experts <= 1024
    ids = torch.empty(topk, dtype=torch.int32, device=logits.device)
    weights = torch.empty(topk, dtype=torch.float32, device=logits.device)
    call("qd_route_topk", ptr(logits), int(logits.dtype == torch.float32), experts, topk, ptr(ids),
         ptr(weights), stream_of(logits))
    return ids, weights


def moe_block(w, x: torch.Tensor, *, config) -> torch.Tensor:
    """Router, top-k NVFP4 experts, gated shared expert (quickdraw/models/qwen.py:168-193).

    Launch plan: router and shared-gate logits, routing, fused gate/up of the selected
    experts and of the shared expert, then one launch for all down projections and the
    combine when the intermediate width is 512 (otherwise per-operator launches).
    """
    assert _is_cuda_bf16(x) and x.ndim == 1
    k = config.num_experts_per_tok
    assert 1 <= k <= config.num_experts
    ids, weights = route(bf16_gemv(x, w.router), k)
    strength = bf16_gemv(x, w.shared_expert_gate)
    inter = w.experts_gate.out_features
    hidden = torch.empty((k + 1, inter), dtype=BF16, device=x.device)
    hidden[:k] = gate_up(x, w.experts_gate, w.experts_up, ids)
    hidden[k] = gate_up(x, w.shared_gate, w.shared_up)
    out = torch.empty_like(x)
    per_expert = int(w.experts_down.weight_scale_2.numel() != 1)
    if inter == 512 and k <= 8 and w.shared_down.in_features == 512:
        lo, hi = 0, config.num_experts
        call("qd_moe_down_combine", ptr(hidden), ptr(ids), ptr(weights), ptr(w.experts_down.weight),
             ptr(w.experts_down.weight_scale), ptr(w.experts_down.weight_scale_2),
             ptr(w.shared_down.weight), ptr(w.shared_down.weight_scale), ptr(w.shared_down.weight_scale_2),
             ptr(strength), ptr(out), None, None, x.numel(), inter, k, per_expert, lo, hi, 0, stream_of(x))
        return out
    contributions = expert_gemv(hidden[:k].contiguous(), w.experts_down, ids, weights)
    shared = nvfp4_gemv(hidden[k].contiguous(), w.shared_down)
    call("qd_moe_combine", ptr(contributions), ptr(ids), ptr(shared), ptr(strength), ptr(out),
         x.numel(), k, stream_of(x))
    return out


# ----------------------------------------------------------------------------- mixers
_ATTN_SPLITS = 32
_scratch: dict = {}


def _attn_scratch(device, floats: int, kv_heads: int):
    key = (device, floats, kv_heads, torch.cuda.current_stream(device).cuda_stream)
    if key not in _scratch:
        _scratch[key] = (torch.empty(floats, dtype=torch.float32, device=device),
                         torch.zeros(kv_heads, dtype=torch.int32, device=device))
    return _scratch[key]


def full_attention_block(w, x, kv_cache, position, *, config) -> torch.Tensor:
    """Gated GQA decode step; writes the key/value row at ``position`` (an int, or a 0-d
    int32 CUDA tensor so a captured graph can be replayed at other positions)."""
    assert _is_cuda_bf16(x) and x.ndim == 1
    keys, values = kv_cache
    assert keys.is_contiguous() and values.is_contiguous() and keys.dtype == BF16 and values.dtype == BF16
    hq, hk, d = config.num_attention_heads, config.num_key_value_heads, config.head_dim
    assert hk > 0 and hq % hk == 0
    capacity = min(keys.shape[0], values.shape[0])
    device_position = isinstance(position, torch.Tensor)
    if device_position:
        assert position.dtype == torch.int32 and position.is_cuda and position.numel() == 1
    else:
        assert 0 <= position < capacity
    qg = _project(x, w.q_proj)
    k_new = _project(x, w.k_proj)
    v_new = _project(x, w.v_proj)
    rotary = int(d * config.partial_rotary_factor)
    assert rotary % 2 == 0 and 0 <= rotary <= d
    lib = _lib.lib()
    floats = lib.qd_attn_scratch_floats(hq, hk, d, _ATTN_SPLITS)
    scratch, counters = _attn_scratch(x.device, floats, hk)
    gated = torch.empty(hq * d, dtype=BF16, device=x.device)
    call("qd_attn_decode", ptr(qg), ptr(k_new), ptr(v_new), ptr(w.q_norm), ptr(w.k_norm), ptr(keys),
         ptr(values), ptr(gated), ptr(scratch), ptr(counters),
         ptr(position) if device_position else None, 0 if device_position else int(position),
         capacity, hq, hk, d, rotary, float(config.rope_theta), float(config.rms_norm_eps),
         _ATTN_SPLITS, 0, stream_of(x))
    return _project(gated, w.o_proj)


def gated_delta_net_block(w, x, rec_state, conv_state, position, *, config) -> torch.Tensor:
    """Gated-DeltaNet decode step; updates the fp32 recurrent state and the bf16 conv
    history in place (``position`` is unused, kept for the table's uniform signature)."""
    assert _is_cuda_bf16(x) and x.ndim == 1
    assert rec_state.is_contiguous() and conv_state.is_contiguous()
    assert rec_state.dtype == torch.float32 and conv_state.dtype == BF16
    hk, dk = config.linear_num_key_heads, config.linear_key_head_dim
    hv, dv = config.linear_num_value_heads, config.linear_value_head_dim
    assert hv % hk == 0
    mixed = _project(x, w.in_proj_qkv)
    z = _project(x, w.in_proj_z)
    a = bf16_gemv(x, w.in_proj_a)
    b = bf16_gemv(x, w.in_proj_b)
    channels, width = mixed.numel(), config.linear_conv_kernel_dim
    assert conv_state.shape == (channels, width - 1) and rec_state.shape == (hv, dk, dv)
    taps = w.conv1d.reshape(channels, width)
    assert taps.is_contiguous() and taps.dtype == BF16
    conv = torch.empty_like(mixed)
    s = stream_of(x)
    call("qd_gdn_conv", ptr(mixed), ptr(taps), ptr(conv_state), ptr(conv), channels, width, s)
    core = torch.empty(hv * dv, dtype=BF16, device=x.device)
    call("qd_gdn_recurrence", ptr(conv), ptr(a), ptr(b), ptr(w.A_log), ptr(w.dt_bias), ptr(rec_state),
         ptr(core), hk, hv, dk, dv, 0, s)
    gated = torch.empty_like(core)
    call("qd_gdn_gated_norm", ptr(core), ptr(z), ptr(w.norm), ptr(gated), hv, dv,
         float(config.rms_norm_eps), s)
    return _project(gated, w.out_proj)


# ------------------------------------------------------------------------------- step
def forward_step(ckpt, token_id, position, state, *, normalize=rms_norm,
                 attention=full_attention_block, delta_net=gated_delta_net_block,
                 experts=moe_block, project_fp4=nvfp4_gemv, prepared=None, logits=True):
    """Composed token step over the operator table (quickdraw/models/qwen.py:196-241):
    one launch group per operator, every operator replaceable.  The engine's default path
    is the fused step in ``fused.py``; this one serves operator overrides and shapes the
    fused step does not cover."""
    config = ckpt.config
    assert len(ckpt.layers) == config.num_hidden_layers
    assert all(layer.idx == i and layer.layer_type == config.layer_types[i]
               for i, layer in enumerate(ckpt.layers)), "complete checkpoint required"
    assert token_id.ndim == 0 and token_id.dtype == torch.long, "one token per step"
    if isinstance(position, int):
        assert 0 <= position < state.kv_k.shape[1]
    x = ckpt.embed_tokens[token_id]
    residual = None
    full = linear = 0
    eps = config.rms_norm_eps

    def add_norm(x, residual, gamma):
        if normalize is rms_norm:
            return add_rms_norm(x, residual, gamma, eps)
        total = x.float() if residual is None else x.float() + residual.float()
        return normalize(total, gamma, eps).to(x.dtype), total.to(x.dtype)

    for layer in ckpt.layers:
        gamma = prepared[0][layer.idx][0] if prepared else 1 + layer.input_layernorm.float()
        normed, residual = add_norm(x, residual, gamma)
        if layer.layer_type == "full_attention":
            mixed = attention(layer.attn, normed, (state.kv_k[full], state.kv_v[full]), position, config=config)
            full += 1
        else:
            assert layer.layer_type == "linear_attention"
            mixed = delta_net(layer.attn, normed, state.rec_state[linear], state.conv_state[linear],
                              position, config=config)
            linear += 1
        gamma = prepared[0][layer.idx][1] if prepared else 1 + layer.post_attention_layernorm.float()
        normed, residual = add_norm(mixed, residual, gamma)
        x = experts(layer.moe, normed, config=config)
    if not logits:
        return None
    gamma = prepared[1] if prepared else 1 + ckpt.final_norm.float()
    normed, _ = add_norm(x, residual, gamma)
    return project_fp4(normed, ckpt.lm_head)


OPERATOR_NAMES = ("rms_norm", "fp8_gemv", "nvfp4_gemv", "full_attention_block",
                  "gated_delta_net_block", "moe_block")


def kernels() -> dict:
    """The six-name operator table of this backend."""
    return dict(rms_norm=rms_norm, fp8_gemv=fp8_gemv, nvfp4_gemv=nvfp4_gemv,
                full_attention_block=full_attention_block,
                gated_delta_net_block=gated_delta_net_block, moe_block=moe_block)


def bind_kernels(*, prepared=None, **overrides) -> dict:
    """Operator table plus a ``forward_step`` bound to it.  Unknown names are rejected;
    an overridden whole block owns its internal projections; an overridden ``fp8_gemv`` /
    ``nvfp4_gemv`` is not injected into this backend's fused blocks (they call the CUDA
    projections directly), it replaces the LM-head projection only."""
    assert overrides.keys() <= set(OPERATOR_NAMES), "unknown kernel operation"
    ops = kernels() | overrides
    ops["forward_step"] = partial(
        forward_step, normalize=ops["rms_norm"], attention=ops["full_attention_block"],
        delta_net=ops["gated_delta_net_block"], experts=ops["moe_block"],
        project_fp4=ops["nvfp4_gemv"], prepared=prepared)
    return ops

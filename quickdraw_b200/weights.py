"""Weight containers for the batch-one decode path (the data contract of the kernels).

Field names, shapes and dtypes follow the reference containers so that a checkpoint
object built for the reference can be handed to this package unchanged
(reference: quickdraw/models/weights.py:29-166).  Only the containers live here; the
arithmetic that consumes them is in the CUDA library.

NVFP4 storage (reference: quickdraw/models/weights.py:14-55):
  * ``weight``         uint8 ``[..., out, in/2]``; byte j holds input 2j in its low
                       nibble and input 2j+1 in its high nibble, each an E2M1 code
                       (bit 3 sign, bits 2:1 exponent, bit 0 mantissa);
  * ``weight_scale``   float8_e4m3fn ``[..., out, in/group_size]``;
  * ``weight_scale_2`` fp32 scalar, or ``[E]`` for an expert bank;
  * the value of weight (o, i) is ``e2m1 * weight_scale[o, i // group] * weight_scale_2``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from pathlib import Path

import torch

E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


@dataclass
class NVFP4Linear:
    """Weight-only FP4 projection; activations stay bf16 (W4A16)."""
    weight: torch.Tensor
    weight_scale: torch.Tensor
    weight_scale_2: torch.Tensor
    input_scale: torch.Tensor | None = None
    group_size: int = 16

    @property
    def out_features(self) -> int:
        return self.weight.shape[-2]

    @property
    def in_features(self) -> int:
        return 2 * self.weight.shape[-1]

    def nbytes(self) -> int:
        return self.weight.nbytes + self.weight_scale.nbytes + self.weight_scale_2.nbytes


@dataclass
class FP8Linear:
    """Static E4M3 projection with scalar weight and activation scales."""
    weight: torch.Tensor
    weight_scale: torch.Tensor
    input_scale: torch.Tensor | None = None

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]


@dataclass
class GDNWeights:
    """Gated-DeltaNet mixer: fused q|k|v projection, output-gate projection z,
    decay/beta projections a/b, depthwise conv taps, per-head decay parameters,
    per-head norm gamma and the output projection."""
    in_proj_qkv: NVFP4Linear | FP8Linear
    in_proj_z: NVFP4Linear | FP8Linear
    in_proj_a: torch.Tensor
    in_proj_b: torch.Tensor
    conv1d: torch.Tensor
    A_log: torch.Tensor
    dt_bias: torch.Tensor
    norm: torch.Tensor
    out_proj: NVFP4Linear | FP8Linear


@dataclass
class FullAttnWeights:
    """GQA mixer; every q_proj head stores its query rows then its gate rows."""
    q_proj: NVFP4Linear | FP8Linear
    k_proj: NVFP4Linear | FP8Linear
    v_proj: NVFP4Linear | FP8Linear
    o_proj: NVFP4Linear | FP8Linear
    q_norm: torch.Tensor
    k_norm: torch.Tensor


@dataclass
class MoEWeights:
    """Router, expert banks (leading expert axis) and the gated shared expert."""
    router: torch.Tensor
    shared_expert_gate: torch.Tensor
    experts_gate: NVFP4Linear
    experts_up: NVFP4Linear
    experts_down: NVFP4Linear
    shared_gate: NVFP4Linear
    shared_up: NVFP4Linear
    shared_down: NVFP4Linear


@dataclass
class LayerWeights:
    idx: int
    layer_type: str
    input_layernorm: torch.Tensor
    post_attention_layernorm: torch.Tensor
    attn: GDNWeights | FullAttnWeights
    moe: MoEWeights


@dataclass
class ModelConfig:
    hidden_size: int
    num_hidden_layers: int
    layer_types: list[str]
    full_attention_interval: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    linear_num_key_heads: int
    linear_key_head_dim: int
    linear_num_value_heads: int
    linear_value_head_dim: int
    linear_conv_kernel_dim: int
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    rms_norm_eps: float
    partial_rotary_factor: float
    rope_theta: float
    vocab_size: int

    @classmethod
    def from_json(cls, path: str | Path) -> "ModelConfig":
        """Read the ``text_config`` block of a Hugging Face ``config.json``
        (reference: quickdraw/models/weights.py:149-156)."""
        text = json.loads(Path(path).read_text())["text_config"]
        rope = text.get("rope_parameters", {})
        special = {"partial_rotary_factor": text.get("partial_rotary_factor", 0.25),
                   "rope_theta": rope.get("rope_theta", 1.0e7)}
        plain = {f.name: text[f.name] for f in fields(cls) if f.name not in special}
        return cls(**plain, **special)

    @property
    def conv_channels(self) -> int:
        return (2 * self.linear_num_key_heads * self.linear_key_head_dim
                + self.linear_num_value_heads * self.linear_value_head_dim)

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)


@dataclass
class Checkpoint:
    """``lm_head`` is an NVFP4Linear in the published checkpoint and a bf16
    ``[vocab, hidden]`` tensor in the synthetic 36B-A3B model; both are accepted."""
    config: ModelConfig
    embed_tokens: torch.Tensor
    final_norm: torch.Tensor
    lm_head: NVFP4Linear | torch.Tensor
    layers: list[LayerWeights]
    mtp: dict[str, torch.Tensor] = field(default_factory=dict)


CONTAINERS = {cls.__name__: cls for cls in (
    NVFP4Linear, FP8Linear, GDNWeights, FullAttnWeights, MoEWeights, LayerWeights,
    ModelConfig, Checkpoint)}

"""Seeded synthetic weights for the 36B-A3B hybrid MoE model and its sub-blocks.

No checkpoint of the model family ships with this package, so every benchmark and
parity test runs on random weights of the published shapes: NVFP4 codes uniform over
the 16 E2M1 codes, one E4M3 block scale per 16 inputs drawn as ``|N(0,1)| * 0.05``
(saturated at the E4M3 maximum 448), fp32 global scale 1.0, bf16 tensors normal with
the standard deviation given below.  Each tensor has its own generator seeded from
``(seed, layer, tensor name)`` so a single layer can be regenerated without the rest;
the CPU and CUDA generators of PyTorch produce different streams, so a test that needs
the same tensors on both sides generates once and copies.

The container shapes follow quickdraw/models/weights.py:77-166 of the reference.
"""

from __future__ import annotations

import zlib

import torch

from .weights import (Checkpoint, FP8Linear, FullAttnWeights, GDNWeights, LayerWeights, ModelConfig,
                      MoEWeights, NVFP4Linear)

BF16 = torch.bfloat16


def model_config(num_layers: int = 48, vocab_size: int = 151936, *, hidden: int = 2048,
                 experts: int = 256, topk: int = 8, intermediate: int = 512,
                 interval: int = 4) -> ModelConfig:
    """36B-A3B hybrid: groups of ``interval - 1`` gated-DeltaNet layers then one GQA layer."""
    kinds = ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
             for i in range(num_layers)]
    return ModelConfig(
        hidden_size=hidden, num_hidden_layers=num_layers, layer_types=kinds,
        full_attention_interval=interval, num_attention_heads=16, num_key_value_heads=2,
        head_dim=256, linear_num_key_heads=16, linear_key_head_dim=128,
        linear_num_value_heads=32, linear_value_head_dim=128, linear_conv_kernel_dim=4,
        num_experts=experts, num_experts_per_tok=topk, moe_intermediate_size=intermediate,
        shared_expert_intermediate_size=intermediate, rms_norm_eps=1e-6,
        partial_rotary_factor=0.25, rope_theta=1.0e7, vocab_size=vocab_size)


class Source:
    """Named, independently seeded random tensors on one device."""

    def __init__(self, seed: int, device):
        self.seed, self.device = seed, torch.device(device)

    def _gen(self, name: str) -> torch.Generator:
        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed << 32) ^ zlib.crc32(name.encode()))
        return g

    def normal(self, name: str, *shape, std: float = 1.0, mean: float = 0.0) -> torch.Tensor:
        t = torch.randn(shape, generator=self._gen(name), device=self.device,
                        dtype=torch.float32)
        return (t * std + mean).to(BF16)

    def nvfp4(self, name: str, out: int, inp: int, experts: int | None = None,
              global_scale: float = 1.0, per_expert_global: bool = False) -> NVFP4Linear:
        lead = () if experts is None else (experts,)
        g = self._gen(name)
        codes = torch.randint(0, 256, (*lead, out, inp // 2), generator=g,
                              device=self.device, dtype=torch.uint8)
        scales = torch.randn((*lead, out, inp // 16), generator=g, device=self.device,
                             dtype=torch.float32).abs_().mul_(0.05).clamp_(max=448.0)
        if per_expert_global and experts is not None:
            gs = torch.full((experts,), global_scale, dtype=torch.float32, device=self.device)
        else:
            gs = torch.tensor(global_scale, dtype=torch.float32, device=self.device)
        return NVFP4Linear(codes, scales.to(torch.float8_e4m3fn), gs)


def _fp8(src: "Source", name: str, out: int, inp: int, input_scale: float = 4.0 / 448.0) -> FP8Linear:
    """Static E4M3 projection of about the same real magnitude as the NVFP4 ones (weights ~
    N(0, 0.1)); activations up to +-4 fill the E4M3 range, larger ones clamp."""
    g = src._gen(name)
    w = torch.randn((out, inp), generator=g, device=src.device, dtype=torch.float32).mul_(64.0).clamp_(-448, 448)
    return FP8Linear(w.to(torch.float8_e4m3fn), torch.tensor(0.1 / 64.0, dtype=torch.float32, device=src.device),
                     torch.tensor(input_scale, dtype=torch.float32, device=src.device))


def expert_slice(bank: NVFP4Linear, lo: int, hi: int) -> NVFP4Linear:
    """Experts [lo, hi) of a bank as an independent (contiguous) bank."""
    g = bank.weight_scale_2
    return NVFP4Linear(bank.weight[lo:hi].clone(), bank.weight_scale[lo:hi].clone(),
                       g if g.numel() == 1 else g[lo:hi].clone(), group_size=bank.group_size)


def make_moe(cfg: ModelConfig, src: Source, tag: str = "moe",
             expert_range: tuple[int, int] | None = None) -> MoEWeights:
    """``expert_range`` keeps only the experts [lo, hi) of each bank (expert parallelism);
    the values are those of the full bank, so ranks hold slices of one model."""
    h, m, s, e = (cfg.hidden_size, cfg.moe_intermediate_size,
                  cfg.shared_expert_intermediate_size, cfg.num_experts)

    def bank(name, out, inp):
        full = src.nvfp4(name, out, inp, e)
        return full if expert_range is None else expert_slice(full, *expert_range)
    return MoEWeights(
        router=src.normal(f"{tag}.router", e, h, std=0.02),
        shared_expert_gate=src.normal(f"{tag}.shared_expert_gate", 1, h, std=0.02),
        experts_gate=bank(f"{tag}.experts_gate", m, h),
        experts_up=bank(f"{tag}.experts_up", m, h),
        experts_down=bank(f"{tag}.experts_down", h, m),
        shared_gate=src.nvfp4(f"{tag}.shared_gate", s, h),
        shared_up=src.nvfp4(f"{tag}.shared_up", s, h),
        shared_down=src.nvfp4(f"{tag}.shared_down", h, s))


def make_gdn(cfg: ModelConfig, src: Source, tag: str = "gdn", fp8: bool = False) -> GDNWeights:
    h = cfg.hidden_size
    linear = (lambda name, out, inp: _fp8(src, name, out, inp)) if fp8 else src.nvfp4
    kw = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    vw = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    hv = cfg.linear_num_value_heads
    return GDNWeights(
        in_proj_qkv=linear(f"{tag}.in_proj_qkv", 2 * kw + vw, h),
        in_proj_z=linear(f"{tag}.in_proj_z", vw, h),
        in_proj_a=src.normal(f"{tag}.in_proj_a", hv, h, std=0.02),
        in_proj_b=src.normal(f"{tag}.in_proj_b", hv, h, std=0.02),
        conv1d=src.normal(f"{tag}.conv1d", 2 * kw + vw, 1, cfg.linear_conv_kernel_dim, std=0.5),
        A_log=src.normal(f"{tag}.A_log", hv, std=0.5),
        dt_bias=src.normal(f"{tag}.dt_bias", hv, std=0.5),
        norm=src.normal(f"{tag}.norm", cfg.linear_value_head_dim, std=0.02, mean=1.0),
        out_proj=linear(f"{tag}.out_proj", h, vw))


def make_attention(cfg: ModelConfig, src: Source, tag: str = "attn", fp8: bool = False) -> FullAttnWeights:
    h = cfg.hidden_size
    linear = (lambda name, out, inp: _fp8(src, name, out, inp)) if fp8 else src.nvfp4
    qw = cfg.num_attention_heads * cfg.head_dim
    kvw = cfg.num_key_value_heads * cfg.head_dim
    return FullAttnWeights(
        q_proj=linear(f"{tag}.q_proj", 2 * qw, h),
        k_proj=linear(f"{tag}.k_proj", kvw, h),
        v_proj=linear(f"{tag}.v_proj", kvw, h),
        o_proj=linear(f"{tag}.o_proj", h, qw),
        q_norm=src.normal(f"{tag}.q_norm", cfg.head_dim, std=0.02),
        k_norm=src.normal(f"{tag}.k_norm", cfg.head_dim, std=0.02))


def make_layer(cfg: ModelConfig, src: Source, idx: int, expert_range=None, fp8_mixers: bool = False) -> LayerWeights:
    kind = cfg.layer_types[idx]
    tag = f"layer{idx}"
    mixer = (make_attention(cfg, src, f"{tag}.attn", fp8_mixers) if kind == "full_attention"
             else make_gdn(cfg, src, f"{tag}.gdn", fp8_mixers))
    return LayerWeights(
        idx=idx, layer_type=kind,
        input_layernorm=src.normal(f"{tag}.input_layernorm", cfg.hidden_size, std=0.02),
        post_attention_layernorm=src.normal(f"{tag}.post_attention_layernorm",
                                            cfg.hidden_size, std=0.02),
        attn=mixer, moe=make_moe(cfg, src, f"{tag}.moe", expert_range))


def make_checkpoint(cfg: ModelConfig, seed: int = 0, device="cuda", expert_range=None,
                    vocab_range=None, fp8_mixers: bool = False, nvfp4_head: bool = False) -> Checkpoint:
    """Whole model with a bf16 embedding and a bf16 LM head (about 23 GB at 48 layers);
    with ``expert_range`` only that slice of every expert bank is kept, with ``vocab_range``
    only those rows of the LM head (the values are those of the whole model)."""
    src = Source(seed, device)
    if nvfp4_head:      # the published checkpoint's head format; weights of about the bf16 head's magnitude
        assert vocab_range is None
        lm_head = src.nvfp4("lm_head.fp4", cfg.vocab_size, cfg.hidden_size, global_scale=0.2)
    else:
        lm_head = src.normal("lm_head", cfg.vocab_size, cfg.hidden_size, std=0.02)
    if vocab_range is not None:
        lm_head = lm_head[vocab_range[0]:vocab_range[1]].clone()
    return Checkpoint(
        config=cfg,
        embed_tokens=src.normal("embed_tokens", cfg.vocab_size, cfg.hidden_size, std=0.02),
        final_norm=src.normal("final_norm", cfg.hidden_size, std=0.02),
        lm_head=lm_head,
        layers=[make_layer(cfg, src, i, expert_range, fp8_mixers) for i in range(cfg.num_hidden_layers)])


def to_device(obj, device):
    """Deep copy of a container tree onto ``device`` (used to hand the same tensors to a
    CPU checker layer by layer)."""
    from dataclasses import fields, is_dataclass
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if is_dataclass(obj):
        return type(obj)(**{f.name: to_device(getattr(obj, f.name), device)
                            for f in fields(obj)})
    if isinstance(obj, (list, tuple)):
        return type(obj)(to_device(v, device) for v in obj)
    if isinstance(obj, dict):
        return {k: to_device(v, device) for k, v in obj.items()}
    return obj


def matvec_case(seed: int = 0, out: int = 1024, inp: int = 2048, device="cpu"):
    """The single-matvec configuration: x bf16 [inp] ~ N(0,1) and one fused gate+up
    sized NVFP4 matrix, drawn from the global generator after ``torch.manual_seed``."""
    torch.manual_seed(seed)
    x = torch.randn(inp).to(BF16)
    codes = torch.randint(0, 256, (out, inp // 2), dtype=torch.uint8)
    scales = (torch.randn(out, inp // 16).abs() * 0.05).clamp(max=448.0).to(torch.float8_e4m3fn)
    proj = NVFP4Linear(codes, scales, torch.tensor(1.0))
    return x.to(device), to_device(proj, device)

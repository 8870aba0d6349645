"""The safetensors loader on CPU: a small checkpoint directory in the published layout (sharded
safetensors, index, config.json with a text_config block, a vision tensor and MTP tensors to be
skipped, per-expert projection tensors) is written from seeded tensors and read back."""

import json

import pytest
import torch
from safetensors.torch import save_file

from quickdraw_b200.loader import load_checkpoint, merge_fp8_scales
from quickdraw_b200.weights import FP8Linear, NVFP4Linear

E4M3 = torch.float8_e4m3fn
CONFIG = dict(hidden_size=64, num_hidden_layers=4, layer_types=["linear_attention", "linear_attention",
              "linear_attention", "full_attention"], full_attention_interval=4, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, linear_num_key_heads=2, linear_key_head_dim=8,
              linear_num_value_heads=4, linear_value_head_dim=8, linear_conv_kernel_dim=4, num_experts=6,
              num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
              rms_norm_eps=1e-6, vocab_size=96)


def _fp8(g, tensors, prefix, rows, cols):
    tensors[prefix + ".weight"] = (torch.randn(rows, cols, generator=g) * 50).to(E4M3)
    tensors[prefix + ".weight_scale"] = torch.rand((), generator=g) * 0.01 + 0.001
    tensors[prefix + ".input_scale"] = torch.rand((), generator=g) * 0.1 + 0.01


def _nvfp4(g, tensors, prefix, rows, cols, activation=False):
    tensors[prefix + ".weight"] = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8)
    tensors[prefix + ".weight_scale"] = (torch.rand(rows, cols // 16, generator=g) * 4 + 0.25).to(E4M3)
    tensors[prefix + ".weight_scale_2"] = torch.rand((), generator=g) * 0.01
    if activation:
        tensors[prefix + ".input_scale"] = torch.rand((), generator=g)


@pytest.fixture(scope="module")
def checkpoint_dir(tmp_path_factory):
    g = torch.Generator().manual_seed(3)
    c = CONFIG
    bf = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
    tensors = {"model.visual.patch_embed.weight": bf(4, 4), "mtp.fc.weight": bf(8, 8), "mtp.norm.weight": bf(8)}
    root = "model.language_model."
    tensors[root + "embed_tokens.weight"] = bf(c["vocab_size"], c["hidden_size"])
    tensors[root + "norm.weight"] = bf(c["hidden_size"])
    _nvfp4(g, tensors, "lm_head", c["vocab_size"], c["hidden_size"])
    for index, kind in enumerate(c["layer_types"]):
        at = f"{root}layers.{index}."
        tensors[at + "input_layernorm.weight"] = bf(c["hidden_size"])
        tensors[at + "post_attention_layernorm.weight"] = bf(c["hidden_size"])
        if kind == "linear_attention":
            m = at + "linear_attn."
            _fp8(g, tensors, m + "in_proj_qkv", 64, 64)
            _fp8(g, tensors, m + "in_proj_z", 32, 64)
            _fp8(g, tensors, m + "out_proj", 64, 32)
            for name, shape in (("in_proj_a.weight", (4, 64)), ("in_proj_b.weight", (4, 64)), ("conv1d.weight", (64, 1, 4)),
                                ("A_log", (4,)), ("dt_bias", (4,)), ("norm.weight", (8,))):
                tensors[m + name] = bf(*shape)
        else:
            m = at + "self_attn."
            _fp8(g, tensors, m + "q_proj", 128, 64)
            _fp8(g, tensors, m + "k_proj", 32, 64)
            _fp8(g, tensors, m + "v_proj", 32, 64)
            _fp8(g, tensors, m + "o_proj", 64, 64)
            tensors[m + "q_norm.weight"], tensors[m + "k_norm.weight"] = bf(16), bf(16)
        tensors[at + "mlp.gate.weight"] = bf(c["num_experts"], c["hidden_size"])
        tensors[at + "mlp.shared_expert_gate.weight"] = bf(1, c["hidden_size"])
        for proj, (rows, cols) in (("gate", (32, 64)), ("up", (32, 64)), ("down", (64, 32))):
            _nvfp4(g, tensors, f"{at}mlp.shared_expert.{proj}_proj", rows, cols)
            for e in range(c["num_experts"]):
                _nvfp4(g, tensors, f"{at}mlp.experts.{e}.{proj}_proj", rows, cols, activation=True)
    directory = tmp_path_factory.mktemp("ckpt")
    names = sorted(tensors)
    shards = {f"model-{i + 1:05d}-of-00003.safetensors": names[i::3] for i in range(3)}      # interleaved on purpose
    weight_map = {}
    for shard, members in shards.items():
        save_file({n: tensors[n].contiguous() for n in members}, str(directory / shard))
        weight_map.update({n: shard for n in members})
    (directory / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (directory / "config.json").write_text(json.dumps({"text_config": dict(CONFIG, rope_parameters={"rope_theta": 5.0e6})}))
    return directory, tensors


def _same(a, b):
    return a.dtype == b.dtype and a.shape == b.shape and torch.equal(a.view(torch.uint8) if a.dtype == E4M3 else a,
                                                                      b.view(torch.uint8) if b.dtype == E4M3 else b)


def test_every_tensor_lands_in_its_container(checkpoint_dir):
    directory, tensors = checkpoint_dir
    ckpt = load_checkpoint(directory, device="cpu")
    c = ckpt.config
    assert c.rope_theta == 5.0e6 and c.partial_rotary_factor == 0.25 and c.num_experts == 6
    assert [l.idx for l in ckpt.layers] == [0, 1, 2, 3] and ckpt.mtp == {}
    assert isinstance(ckpt.lm_head, NVFP4Linear) and _same(ckpt.lm_head.weight, tensors["lm_head.weight"])
    root = "model.language_model."
    assert _same(ckpt.embed_tokens, tensors[root + "embed_tokens.weight"]) and _same(ckpt.final_norm, tensors[root + "norm.weight"])
    first, last = ckpt.layers[0], ckpt.layers[3]
    at = root + "layers.0."
    assert isinstance(first.attn.in_proj_qkv, FP8Linear)
    assert _same(first.attn.in_proj_qkv.weight, tensors[at + "linear_attn.in_proj_qkv.weight"])
    assert float(first.attn.in_proj_z.input_scale) == float(tensors[at + "linear_attn.in_proj_z.input_scale"])
    assert _same(first.attn.conv1d, tensors[at + "linear_attn.conv1d.weight"])
    assert _same(first.attn.A_log, tensors[at + "linear_attn.A_log"])
    assert _same(last.attn.k_norm, tensors[root + "layers.3.self_attn.k_norm.weight"])
    assert _same(last.attn.o_proj.weight, tensors[root + "layers.3.self_attn.o_proj.weight"])
    bank = first.moe.experts_down
    assert bank.weight.shape == (6, 64, 16) and bank.weight_scale.shape == (6, 64, 2) and bank.weight_scale_2.shape == (6,)
    for e in range(6):
        assert _same(bank.weight[e], tensors[f"{at}mlp.experts.{e}.down_proj.weight"])
        assert _same(bank.weight_scale[e], tensors[f"{at}mlp.experts.{e}.down_proj.weight_scale"])
        assert float(bank.weight_scale_2[e]) == float(tensors[f"{at}mlp.experts.{e}.down_proj.weight_scale_2"])
        assert float(bank.input_scale[e]) == float(tensors[f"{at}mlp.experts.{e}.down_proj.input_scale"])
    assert first.moe.shared_up.input_scale is None
    assert _same(first.moe.router, tensors[at + "mlp.gate.weight"])


def test_layer_subset_mtp_and_rank_slices(checkpoint_dir):
    directory, tensors = checkpoint_dir
    part = load_checkpoint(directory, device="cpu", include_mtp=True, layers=[3, 1], expert_range=(2, 5), vocab_range=(32, 64))
    assert [l.idx for l in part.layers] == [1, 3]
    assert sorted(part.mtp) == ["mtp.fc.weight", "mtp.norm.weight"]
    bank = part.layers[0].moe.experts_gate
    assert bank.weight.shape[0] == 3
    for local, e in enumerate(range(2, 5)):
        assert _same(bank.weight[local], tensors[f"model.language_model.layers.1.mlp.experts.{e}.gate_proj.weight"])
    assert _same(part.lm_head.weight, tensors["lm_head.weight"][32:64])
    assert _same(part.lm_head.weight_scale, tensors["lm_head.weight_scale"][32:64])


def test_merged_fp8_scales(checkpoint_dir):
    directory, tensors = checkpoint_dir
    ckpt = load_checkpoint(directory, device="cpu")
    before = {name: (getattr(ckpt.layers[3].attn, name).weight.float() * getattr(ckpt.layers[3].attn, name).weight_scale)
              for name in ("q_proj", "k_proj", "v_proj")}
    merge_fp8_scales(ckpt)
    at = "model.language_model.layers.3.self_attn."
    want_w = max(float(tensors[at + f"{n}.weight_scale"]) for n in ("q_proj", "k_proj", "v_proj"))
    want_x = max(float(tensors[at + f"{n}.input_scale"]) for n in ("q_proj", "k_proj", "v_proj"))
    for name in ("q_proj", "k_proj", "v_proj"):
        proj = getattr(ckpt.layers[3].attn, name)
        assert float(proj.weight_scale) == pytest.approx(want_w) and float(proj.input_scale) == pytest.approx(want_x)
        after = proj.weight.float() * proj.weight_scale
        # re-expressed in a coarser scale: within one E4M3 step of the new grid
        assert (after - before[name]).abs().max() <= 0.0626 * before[name].abs().max() + 1e-6
    # the out projection reads a different activation and keeps its own scales
    assert float(ckpt.layers[3].attn.o_proj.weight_scale) == float(tensors[at + "o_proj.weight_scale"])
    qkv, z = ckpt.layers[0].attn.in_proj_qkv, ckpt.layers[0].attn.in_proj_z
    assert float(qkv.weight_scale) == float(z.weight_scale) and float(qkv.input_scale) == float(z.input_scale)


def test_saved_synthetic_model_reads_back_identically(tmp_path):
    from quickdraw_b200 import synthetic
    from quickdraw_b200.loader import save_checkpoint
    cfg = synthetic.model_config(num_layers=4, vocab_size=64, hidden=256, experts=8, topk=3, intermediate=64)
    ckpt = synthetic.make_checkpoint(cfg, seed=5, device="cpu")
    save_checkpoint(ckpt, tmp_path, shards=3)
    back = load_checkpoint(tmp_path, device="cpu")
    assert back.config == ckpt.config
    assert _same(back.lm_head, ckpt.lm_head) and _same(back.embed_tokens, ckpt.embed_tokens)
    for a, b in zip(back.layers, ckpt.layers):
        assert a.layer_type == b.layer_type and _same(a.input_layernorm, b.input_layernorm)
        for name in ("experts_gate", "experts_up", "experts_down", "shared_gate", "shared_up", "shared_down"):
            x, y = getattr(a.moe, name), getattr(b.moe, name)
            assert _same(x.weight, y.weight) and _same(x.weight_scale, y.weight_scale)
            # a bank-wide scale comes back as one (equal) scale per expert
            assert torch.equal(x.weight_scale_2.flatten(), y.weight_scale_2.flatten().expand(x.weight_scale_2.numel()))
        for name, value in vars(b.attn).items():
            got = getattr(a.attn, name)
            if isinstance(value, torch.Tensor):
                assert _same(got, value), name
            else:
                assert _same(got.weight, value.weight) and _same(got.weight_scale, value.weight_scale), name

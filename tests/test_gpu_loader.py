"""`Engine.from_pretrained` on a checkpoint directory: a synthetic model of the 36B-A3B widths is
written to safetensors shards, loaded through the streaming loader (expert banks filled through
pinned staging on a copy stream) and must generate exactly what the in-memory model generates."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_from_pretrained_generates_like_the_in_memory_model(cuda_device, tmp_path):
    from quickdraw_b200 import synthetic
    from quickdraw_b200.engine import Engine
    from quickdraw_b200.loader import save_checkpoint
    cfg = synthetic.model_config(num_layers=4, vocab_size=2048, experts=16, topk=8)
    ckpt = synthetic.make_checkpoint(cfg, seed=11, device="cuda")
    prompt, steps = [5, 1900, 77, 1033, 8, 640], 16
    direct = Engine(ckpt, max_context=64, device="cuda")
    direct.state.kv_k.zero_()
    direct.state.kv_v.zero_()
    want = direct.generate(prompt, steps)
    save_checkpoint(ckpt, tmp_path, shards=3)
    del direct
    loaded = Engine.from_pretrained(str(tmp_path), max_context=64, device="cuda")
    assert loaded.fused is not None, "the loaded model must take the one-launch step"
    bank = loaded.ckpt.layers[0].moe.experts_gate
    assert bank.weight.is_cuda and bank.weight.shape[0] == 16
    assert torch.equal(bank.weight, ckpt.layers[0].moe.experts_gate.weight)
    loaded.state.kv_k.zero_()
    loaded.state.kv_v.zero_()
    assert loaded.generate(prompt, steps) == want

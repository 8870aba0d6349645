"""Pin the CPU oracle: it must reproduce the reference's saved fixtures, its known-answer
tests and the outputs its own functions gave on seeded NVFP4 inputs."""

import torch

from oracle import decode_oracle as O
from tests.golden.fixture_io import from_tree

STATE_ARGS = {"full_attention_block": ("kv_cache",),
              "gated_delta_net_block": ("rec_state", "conv_state"),
              "forward_step": ("state",)}


def _compare(actual, expected, rtol, atol, where="result"):
    from dataclasses import fields, is_dataclass
    if isinstance(expected, torch.Tensor):
        assert actual.shape == expected.shape and actual.dtype == expected.dtype, where
        if expected.is_floating_point():
            torch.testing.assert_close(actual.double(), expected.double(), rtol=rtol, atol=atol, msg=lambda m: f"{where}: {m}")
        else:
            assert torch.equal(actual, expected), where
    elif is_dataclass(expected):
        for f in fields(expected):
            _compare(getattr(actual, f.name), getattr(expected, f.name), rtol, atol, f"{where}.{f.name}")
    elif isinstance(expected, (list, tuple)):
        assert len(actual) == len(expected)
        for i, (a, e) in enumerate(zip(actual, expected)):
            _compare(a, e, rtol, atol, f"{where}[{i}]")
    elif isinstance(expected, dict):
        for k in expected:
            _compare(actual[k], expected[k], rtol, atol, f"{where}.{k}")
    else:
        assert actual == expected, where


def test_saved_reference_fixtures(reference_fixtures):
    """All 15 saved fixtures: output and post-call state within the stored tolerances."""
    assert len(reference_fixtures) == 15
    for name, tree in sorted(reference_fixtures.items()):
        data = from_tree(tree)
        fn = getattr(O, data["function"])
        actual = fn(**data["kwargs"])
        _compare(actual, data["expected"], data["rtol"], data["atol"], name)
        for arg in STATE_ARGS.get(data["function"], ()):
            _compare(data["kwargs"][arg], data["after"][arg], data["rtol"], data["atol"], f"{name}.after.{arg}")


def test_unpack_all_codes_exact():
    table = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    packed = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    values = O.unpack_fp4(packed.reshape(256, 1))
    for byte in range(256):
        for half, code in enumerate((byte & 15, byte >> 4)):
            want = table[code & 7] * (-1.0 if code & 8 else 1.0)
            got = values[byte, half].item()
            assert got == want and (torch.signbit(values[byte, half]).item() == bool(code & 8))


def test_gemv_matches_reference_bit_exact(reference_outputs):
    for case in from_tree(reference_outputs["gemv"]):
        got = O.nvfp4_gemv(case["x"], case["proj"], routing_weight=case["routing"])
        assert torch.equal(got, case["expected"])
    case = from_tree(reference_outputs["all_codes"])
    assert torch.equal(O.nvfp4_gemv(case["x"], case["proj"]), case["expected"])


def test_routed_double_rounding_known_answer(reference_outputs):
    case = from_tree(reference_outputs["routed_kat"])
    got = O.nvfp4_gemv(case["x"], case["proj"], routing_weight=case["routing"])
    assert got.item() == 5.5625 == case["expected"].item()


def test_config1_rows(reference_outputs):
    from quickdraw_b200 import synthetic
    case = from_tree(reference_outputs["config1_head"])
    x, proj = synthetic.matvec_case(0)
    got = O.nvfp4_gemv(x, proj)
    assert torch.equal(got[:case["rows"]], case["expected"])
    assert got.float().sum().item() == case["checksum"].item()
    assert O.rel_l2(got, O.fp32_dequant_matvec(x, proj)) < 1e-2


def test_expert_bank(reference_outputs):
    for case in from_tree(reference_outputs["expert_gemv"]):
        x, ids, r = case["x"], case["ids"], case["routing"]
        rows = [O.nvfp4_gemv(x if x.ndim == 1 else x[s], O.expert_view(case["proj"], e),
                             routing_weight=None if r is None else r[s])
                for s, e in enumerate(ids.tolist())]
        assert torch.equal(torch.stack(rows), case["expected"])


def test_route_ids_exact(reference_outputs):
    for case in from_tree(reference_outputs["route"]):
        ids, weights = O.route(case["logits"], case["topk"])
        assert torch.equal(ids, case["ids"])
        torch.testing.assert_close(weights, case["weights"], rtol=0, atol=0)
    ids, _ = O.route(torch.ones(6).bfloat16(), 3)
    assert ids.tolist() == [0, 1, 2]
    ids, _ = O.route(torch.tensor([-4., 2., .5, -1., 3., 1.]).bfloat16(), 3)
    assert ids.tolist() == [4, 1, 5]


def test_moe_blocks(reference_outputs):
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    case = from_tree(reference_outputs["moe"])
    got = O.moe_block(ckpt.layers[0].moe, case["x"], config=ckpt.config)
    assert torch.equal(got, case["expected"])
    ties = from_tree(reference_outputs["moe_ties"])
    assert torch.equal(O.moe_block(ties["w"], ties["x"], config=ckpt.config), ties["expected"])


def test_expert_parallel_partition_sums_to_whole(reference_outputs):
    """Rank-local routed sums over disjoint expert slices add up to the unsharded sum."""
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    moe, cfg = ckpt.layers[0].moe, ckpt.config
    x = from_tree(reference_outputs["moe"])["x"]
    whole = O.moe_block(moe, x, config=cfg, partial=True)
    for world in (2, 4):
        per = cfg.num_experts // world
        parts = [O.moe_block(moe, x, config=cfg, partial=True, experts=range(r * per, (r + 1) * per))
                 for r in range(world)]
        total = torch.stack(parts).sum(0)
        torch.testing.assert_close(total, whole, rtol=1e-6, atol=1e-6)
        # the partial sums add in another order than the unsharded fp32 sum: the combined
        # block agrees to bf16 rounding level, not bit for bit
        assert O.rel_l2(O.combine_shared(moe, x, total), O.moe_block(moe, x, config=cfg)) < 1e-2


def test_gdn_block(reference_outputs):
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    data = from_tree(reference_outputs["gdn"])
    rec, conv = data["rec0"].clone(), data["conv0"].clone()
    for step, entry in enumerate(data["steps"]):
        got = O.gated_delta_net_block(ckpt.layers[0].attn, entry["x"], rec, conv, step, config=ckpt.config)
        torch.testing.assert_close(got.float(), entry["expected"].float(), rtol=0.02, atol=0.002)
        assert torch.equal(conv, entry["conv_after"])
    torch.testing.assert_close(rec, data["rec_after"], rtol=2e-5, atol=1e-6)


def test_attention_block(reference_outputs):
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    data = from_tree(reference_outputs["attention"])
    for case in data["cases"]:
        k, v = data["k"].clone(), data["v"].clone()
        got = O.full_attention_block(ckpt.layers[1].attn, case["x"], (k, v), case["position"], config=ckpt.config)
        torch.testing.assert_close(got.float(), case["expected"].float(), rtol=0.02, atol=0.002)
        assert torch.equal(k[case["position"]], case["k_row"]) and torch.equal(v[case["position"]], case["v_row"])
        untouched = [i for i in range(k.shape[0]) if i != case["position"]]
        assert torch.equal(k[untouched], data["k"][untouched]) and torch.equal(v[untouched], data["v"][untouched])


def test_generation_tokens(reference_outputs):
    from quickdraw_b200.state import DecodeState
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    gen = from_tree(reference_outputs["generation"])
    state = DecodeState.allocate(ckpt.config, 32, "cpu")
    state.kv_k.fill_(9.0)
    state.kv_v.fill_(-11.0)
    tokens = O.greedy_decode(ckpt, state, gen["prompt"], len(gen["tokens"]))
    assert tokens == gen["tokens"]
    torch.testing.assert_close(state.rec_state, gen["rec_after"], rtol=1e-3, atol=1e-5)
    assert O.rel_l2(state.kv_k, gen["k_after"]) < 1e-2


def test_chunk_matmul_equals_token_loop():
    """The prefill form of a projection against the single-token function it is pinned to."""
    from quickdraw_b200 import synthetic
    src = synthetic.Source(5, "cpu")
    proj = src.nvfp4("w", 96, 256, global_scale=1.25)
    x = src.normal("x", 9, 256)
    chunk = O.nvfp4_matmul(x, proj)
    rows = torch.stack([O.nvfp4_gemv(x[t], proj) for t in range(9)])
    torch.testing.assert_close(chunk.float(), rows.float(), rtol=0.025, atol=0.003)

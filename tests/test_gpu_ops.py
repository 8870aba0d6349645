"""GPU parity of the operator table against the CPU oracle and the golden fixtures.
Every call goes through the C-ABI library (ctypes); tolerances are the reference's own
(rtol 0.02 / atol 0.002 on bf16 outputs, 2e-5 / 1e-6 on the fp32 state) plus the 1e-2
relative-L2 bound against an fp32-dequantised product."""

import pytest
import torch

from oracle import decode_oracle as O
from quickdraw_b200 import synthetic
from quickdraw_b200.synthetic import to_device
from quickdraw_b200.weights import NVFP4Linear
from tests.golden.fixture_io import from_tree

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(cuda_device):
    from quickdraw_b200 import kernels
    return kernels


def close(actual, expected, rtol=0.02, atol=0.002):
    torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), rtol=rtol, atol=atol)


# ----------------------------------------------------------------------------- formats
def test_dequant_all_codes_all_scales_bit_exact(K, cuda_device):
    scale_codes = [c for c in range(256) if (c & 0x7F) != 0x7F]
    rows = len(scale_codes)
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat(rows, 1)          # in = 512
    scales = torch.tensor(scale_codes, dtype=torch.uint8).view(torch.float8_e4m3fn).reshape(rows, 1).repeat(1, 32)
    proj = NVFP4Linear(codes, scales.contiguous(), torch.tensor(1.0))
    expected = O.dequantize_fp32(proj)
    dev = to_device(proj, cuda_device)
    for hardware in (False, True):
        got = K.dequantize(dev, hardware_convert=hardware).cpu()
        assert torch.equal(got, expected)
        assert torch.equal(torch.signbit(got), torch.signbit(expected))


# ------------------------------------------------------------------------------ matvec
def test_gemv_golden_cases(K, cuda_device, reference_outputs):
    for case in from_tree(reference_outputs["gemv"]):
        x, proj = case["x"].to(cuda_device), to_device(case["proj"], cuda_device)
        routing = case["routing"]
        for generic in (True, False):
            got = K.nvfp4_gemv(x, proj, routing_weight=None if routing is None else routing.to(cuda_device),
                               force_generic=generic)
            close(got, case["expected"])
    case = from_tree(reference_outputs["all_codes"])
    close(K.nvfp4_gemv(case["x"].to(cuda_device), to_device(case["proj"], cuda_device)), case["expected"])


def test_routed_double_rounding_known_answer(K, cuda_device, reference_outputs):
    case = from_tree(reference_outputs["routed_kat"])
    got = K.nvfp4_gemv(case["x"].to(cuda_device), to_device(case["proj"], cuda_device),
                       routing_weight=case["routing"].to(cuda_device))
    assert got.item() == 5.5625


@pytest.mark.parametrize("rows,width", [(1024, 2048), (2048, 4096), (333, 2048), (8192, 2048), (77, 4096)])
def test_streaming_gemv_matches_oracle(K, cuda_device, rows, width):
    torch.manual_seed(rows + width)
    x = torch.randn(width).bfloat16()
    codes = torch.randint(0, 256, (rows, width // 2), dtype=torch.uint8)
    scales = (torch.randn(rows, width // 16).abs() * 0.05).to(torch.float8_e4m3fn)
    proj = NVFP4Linear(codes, scales, torch.tensor(0.75))
    expected = O.nvfp4_gemv(x, proj)
    got = K.nvfp4_gemv(x.to(cuda_device), to_device(proj, cuda_device))
    close(got, expected)
    assert O.rel_l2(got.cpu(), O.fp32_dequant_matvec(x, proj)) < 1e-2
    generic = K.nvfp4_gemv(x.to(cuda_device), to_device(proj, cuda_device), force_generic=True)
    close(generic, expected)
    # the two CUDA paths differ only in fp32 summation order
    assert O.rel_l2(got.cpu(), generic.cpu()) < 4e-3


def test_config1_single_matvec(K, cuda_device, reference_outputs):
    case = from_tree(reference_outputs["config1_head"])
    x, proj = synthetic.matvec_case(0)
    got = K.nvfp4_gemv(x.to(cuda_device), to_device(proj, cuda_device)).cpu()
    close(got[:case["rows"]], case["expected"])
    close(got, O.nvfp4_gemv(x, proj))
    assert O.rel_l2(got, O.fp32_dequant_matvec(x, proj)) < 1e-2


def test_large_activations_do_not_overflow_f16(K, cuda_device):
    torch.manual_seed(3)
    x = (torch.randn(2048) * 3.0e5).bfloat16()
    proj = synthetic.Source(1, "cpu").nvfp4("big", 64, 2048)
    got = K.nvfp4_gemv(x.to(cuda_device), to_device(proj, cuda_device))
    want = O.nvfp4_gemv(x, proj)
    assert torch.isfinite(got).all()
    assert O.rel_l2(got.cpu(), want) < 1e-2


def test_expert_bank_cases(K, cuda_device, reference_outputs):
    for case in from_tree(reference_outputs["expert_gemv"]):
        got = K.expert_gemv(case["x"].to(cuda_device), to_device(case["proj"], cuda_device),
                            case["ids"].to(cuda_device),
                            None if case["routing"] is None else case["routing"].to(cuda_device))
        close(got, case["expected"])


def test_gate_up_plain_and_bank(K, cuda_device):
    src = synthetic.Source(9, "cpu")
    x = src.normal("x", 2048)
    for experts in (None, 6):
        gate, up = src.nvfp4("g", 96, 2048, experts), src.nvfp4("u", 96, 2048, experts)
        ids = None if experts is None else torch.tensor([5, 0, 3], dtype=torch.int32)
        if experts is None:
            want = O.swiglu(O.nvfp4_gemv(x, gate), O.nvfp4_gemv(x, up))
        else:
            want = torch.stack([O.swiglu(O.nvfp4_gemv(x, O.expert_view(gate, e)), O.nvfp4_gemv(x, O.expert_view(up, e)))
                                for e in ids.tolist()])
        for generic in (False, True):
            got = K.gate_up(x.to(cuda_device), to_device(gate, cuda_device), to_device(up, cuda_device),
                            None if ids is None else ids.to(cuda_device), force_generic=generic)
            close(got, want)


def test_bf16_gemv_and_fp8_gemv(K, cuda_device):
    torch.manual_seed(5)
    x = torch.randn(2048).bfloat16()
    w = (torch.randn(300, 2048) * 0.02).bfloat16()
    close(K.bf16_gemv(x.to(cuda_device), w.to(cuda_device)), O.bf16_gemv(x, w))
    from quickdraw_b200.weights import FP8Linear
    eye = FP8Linear(torch.eye(3).to(torch.float8_e4m3fn), torch.tensor(1.0), torch.tensor(1.0))
    got = K.fp8_gemv(torch.tensor([1.0625, 1.1875, -1.0625], device=cuda_device), to_device(eye, cuda_device))
    assert got.cpu().tolist() == [1.0, 1.25, -1.0]       # ties round to even
    proj = FP8Linear((torch.randn(40, 96) * 0.5).to(torch.float8_e4m3fn), torch.tensor(0.125), torch.tensor(0.25))
    xs = torch.randn(96).bfloat16()
    close(K.fp8_gemv(xs.to(cuda_device), to_device(proj, cuda_device)), O.fp8_gemv(xs, proj))


def test_rms_norm(K, cuda_device):
    torch.manual_seed(6)
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(5, 2048).to(dtype)
        gamma = 1 + torch.randn(2048) * 0.1
        got = K.rms_norm(x.to(cuda_device), gamma.to(cuda_device), 1e-6)
        close(got, O.rms_norm(x, gamma, 1e-6), rtol=0.016 if dtype == torch.bfloat16 else 2e-5, atol=1e-6)
    x, r = torch.randn(2048).bfloat16(), torch.randn(2048).bfloat16()
    normed, res = K.add_rms_norm(x.to(cuda_device), r.to(cuda_device), gamma.to(cuda_device), 1e-6)
    want_n, want_r = O.add_norm(x, r, gamma, 1e-6)
    close(normed, want_n, rtol=0.016, atol=1e-6)
    assert torch.equal(res.cpu(), want_r)


# ----------------------------------------------------------------------------- routing
def test_route_ids_exact(K, cuda_device, reference_outputs):
    for case in from_tree(reference_outputs["route"]):
        ids, weights = K.route(case["logits"].to(cuda_device), case["topk"])
        assert torch.equal(ids.cpu(), case["ids"])
        torch.testing.assert_close(weights.cpu(), case["weights"], rtol=2e-6, atol=1e-7)


# --------------------------------------------------------------------------------- MoE
def test_moe_golden(K, cuda_device, reference_outputs):
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    case = from_tree(reference_outputs["moe"])
    got = K.moe_block(to_device(ckpt.layers[0].moe, cuda_device), case["x"].to(cuda_device), config=ckpt.config)
    close(got, case["expected"])
    ties = from_tree(reference_outputs["moe_ties"])
    close(K.moe_block(to_device(ties["w"], cuda_device), ties["x"].to(cuda_device), config=ckpt.config), ties["expected"])


def test_moe_layer_full_width(K, cuda_device):
    """One MoE layer of the 36B-A3B shape (256 experts, top-8, intermediate 512)."""
    cfg = synthetic.model_config(num_layers=1)
    src = synthetic.Source(2, cuda_device)
    moe = synthetic.make_moe(cfg, src)
    x = src.normal("x", cfg.hidden_size)
    got = K.moe_block(moe, x, config=cfg).cpu()
    want = O.moe_block(to_device(moe, "cpu"), x.cpu(), config=cfg)
    close(got, want)
    assert O.rel_l2(got, want) < 1e-2
    logits = K.bf16_gemv(x, moe.router)
    ids, _ = K.route(logits, cfg.num_experts_per_tok)
    want_ids, _ = O.route(O.bf16_gemv(x.cpu(), moe.router.cpu()), cfg.num_experts_per_tok)
    assert torch.equal(ids.cpu(), want_ids)


# ------------------------------------------------------------------------------ mixers
def test_gdn_golden(K, cuda_device, reference_outputs):
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    data = from_tree(reference_outputs["gdn"])
    w = to_device(ckpt.layers[0].attn, cuda_device)
    rec, conv = data["rec0"].to(cuda_device), data["conv0"].to(cuda_device)
    for step, entry in enumerate(data["steps"]):
        got = K.gated_delta_net_block(w, entry["x"].to(cuda_device), rec, conv, step, config=ckpt.config)
        close(got, entry["expected"])
        assert torch.equal(conv.cpu(), entry["conv_after"])
    torch.testing.assert_close(rec.cpu(), data["rec_after"], rtol=1e-3, atol=1e-5)


def test_gdn_full_width(K, cuda_device):
    cfg = synthetic.model_config(num_layers=1)
    src = synthetic.Source(4, cuda_device)
    w = synthetic.make_gdn(cfg, src)
    rec = (torch.randn(32, 128, 128, device=cuda_device) * 0.01)
    conv = src.normal("conv", cfg.conv_channels, 3)
    rec_c, conv_c, w_c = rec.cpu().clone(), conv.cpu().clone(), to_device(w, "cpu")
    for step in range(2):
        x = src.normal(f"x{step}", cfg.hidden_size)
        got = K.gated_delta_net_block(w, x, rec, conv, step, config=cfg)
        want = O.gated_delta_net_block(w_c, x.cpu(), rec_c, conv_c, step, config=cfg)
        assert O.rel_l2(got.cpu(), want) < 1e-2
        close(got, want, rtol=0.05, atol=0.05)
    assert O.rel_l2(rec.cpu(), rec_c) < 1e-3
    assert O.rel_l2(conv.cpu(), conv_c) < 1e-2


def test_attention_golden(K, cuda_device, reference_outputs):
    ckpt = from_tree(reference_outputs["mini_ckpt"])
    data = from_tree(reference_outputs["attention"])
    w = to_device(ckpt.layers[1].attn, cuda_device)
    for case in data["cases"]:
        k, v = data["k"].to(cuda_device), data["v"].to(cuda_device)
        got = K.full_attention_block(w, case["x"].to(cuda_device), (k, v), case["position"], config=ckpt.config)
        close(got, case["expected"])
        p = case["position"]
        close(k[p], case["k_row"])
        assert torch.equal(v[p].cpu(), case["v_row"])
        others = [i for i in range(k.shape[0]) if i != p]
        assert torch.equal(k[others].cpu(), data["k"][others]) and torch.equal(v[others].cpu(), data["v"][others])
        # device-scalar position gives the same result
        k2, v2 = data["k"].to(cuda_device), data["v"].to(cuda_device)
        pos = torch.tensor(p, dtype=torch.int32, device=cuda_device)
        again = K.full_attention_block(w, case["x"].to(cuda_device), (k2, v2), pos, config=ckpt.config)
        assert torch.equal(again, got)


@pytest.mark.parametrize("position", [0, 63, 64, 700, 4095])
def test_attention_full_width(K, cuda_device, position):
    cfg = synthetic.model_config(num_layers=4)
    src = synthetic.Source(8, cuda_device)
    w = synthetic.make_attention(cfg, src)
    capacity = 4096
    k = src.normal("k", capacity, 2, 256)
    v = src.normal("v", capacity, 2, 256)
    x = src.normal("x", cfg.hidden_size)
    kc, vc = k.cpu().clone(), v.cpu().clone()
    got = K.full_attention_block(w, x, (k, v), position, config=cfg)
    want = O.full_attention_block(to_device(w, "cpu"), x.cpu(), (kc, vc), position, config=cfg)
    assert O.rel_l2(got.cpu(), want) < 1e-2
    assert O.rel_l2(k[position].cpu(), kc[position]) < 1e-2
    assert torch.equal(v[position].cpu(), vc[position])


@pytest.mark.parametrize("capacity,position", [(8192, 8191), (8192, 5000), (32768, 32767), (32768, 20011)])
def test_attention_long_context(K, cuda_device, capacity, position):
    """The attention configurations of the baseline: 16 query / 2 KV heads of 256, bf16 cache of
    8192 and 32768 positions ~ N(0, 1), decode at the last position and at one in the middle;
    against the oracle within 1e-2 relative L2 (fp32 softmax over the whole history on the CPU)."""
    cfg = synthetic.model_config(num_layers=4)
    src = synthetic.Source(9, cuda_device)
    w = synthetic.make_attention(cfg, src)
    k = src.normal("k", capacity, 2, 256)
    v = src.normal("v", capacity, 2, 256)
    x = src.normal("x", cfg.hidden_size)
    kc, vc = k.cpu().clone(), v.cpu().clone()
    got = K.full_attention_block(w, x, (k, v), position, config=cfg)
    want = O.full_attention_block(to_device(w, "cpu"), x.cpu(), (kc, vc), position, config=cfg)
    assert O.rel_l2(got.cpu(), want) < 1e-2
    assert O.rel_l2(k[position].cpu(), kc[position]) < 1e-2
    assert torch.equal(v[position].cpu(), vc[position])
    untouched = [position - 1, 0] if position else []
    for t in untouched:
        assert torch.equal(k[t].cpu(), kc[t]) and torch.equal(v[t].cpu(), vc[t])


# ----------------------------------------------------- the reference's saved fixtures
def test_reference_fixtures_through_the_operator_table(K, cuda_device, reference_fixtures):
    """The 15 saved block/step fixtures (tiny shapes, FP8 mixer projections) through
    bind_kernels(): output and post-call state within the stored tolerances."""
    from dataclasses import fields, is_dataclass
    table = K.bind_kernels()

    def compare(a, e, rtol, atol):
        if isinstance(e, torch.Tensor):
            if e.is_floating_point():
                torch.testing.assert_close(a.double().cpu(), e.double().cpu(), rtol=rtol, atol=atol)
            else:
                assert torch.equal(a.cpu(), e.cpu())
        elif is_dataclass(e):
            for f in fields(e):
                compare(getattr(a, f.name), getattr(e, f.name), rtol, atol)
        elif isinstance(e, (list, tuple)):
            for x, y in zip(a, e):
                compare(x, y, rtol, atol)
        elif isinstance(e, dict):
            for key in e:
                compare(a[key], e[key], rtol, atol)
        else:
            assert a == e

    state_args = {"full_attention_block": ("kv_cache",), "gated_delta_net_block": ("rec_state", "conv_state"),
                  "forward_step": ("state",)}
    for name, tree in sorted(reference_fixtures.items()):
        data = from_tree(tree, cuda_device)
        fn = data["function"]
        kwargs = data["kwargs"]
        actual = table[fn](**kwargs)
        compare(actual, data["expected"], data["rtol"], data["atol"])
        for arg in state_args.get(fn, ()):
            compare(kwargs[arg], data["after"][arg], data["rtol"], data["atol"])

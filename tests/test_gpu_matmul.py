"""The tensor-core projection of a chunk of tokens (prefill) against the CPU oracle: the
restated prefill matmul and, row by row, the single-token matvec the reference pins it to."""

import pytest
import torch

from oracle import decode_oracle as O
from quickdraw_b200 import synthetic
from quickdraw_b200.synthetic import to_device

pytestmark = pytest.mark.gpu

SHAPES = [(1, 256, 512), (7, 512, 2048), (128, 256, 2048), (129, 1024, 2048), (300, 2048, 4096), (64, 264, 512)]


@pytest.mark.parametrize("tokens,out_features,in_features", SHAPES)
def test_matmul_matches_oracle(cuda_device, tokens, out_features, in_features):
    from quickdraw_b200 import kernels
    src = synthetic.Source(21, "cpu")
    proj = src.nvfp4(f"w{out_features}x{in_features}", out_features, in_features, global_scale=0.75)
    x = src.normal(f"x{tokens}", tokens, in_features)
    got = kernels.matmul(x.to(cuda_device), to_device(proj, cuda_device)).cpu()
    assert kernels.matmul_status(cuda_device) == 0
    want = O.nvfp4_matmul(x, proj)
    assert got.shape == want.shape
    torch.testing.assert_close(got.float(), want.float(), rtol=0.02, atol=0.002)
    assert O.rel_l2(got, want) < 2e-3
    # the single-token function, the reference's own anchor for the chunked path
    for t in sorted({0, tokens // 2, tokens - 1}):
        row = O.nvfp4_gemv(x[t], proj)
        torch.testing.assert_close(got[t].float(), row.float(), rtol=0.025, atol=0.003)
    exact = (x.float() @ O.dequantize_fp32(proj).T)
    assert O.rel_l2(got, exact) < 1e-2


ROWS_SHAPES = [(1, 16, 512), (7, 528, 2048), (32, 8192, 2048), (32, 2048, 4096), (19, 96, 1024), (32, 9472, 512)]


@pytest.mark.parametrize("tokens,out_features,in_features", ROWS_SHAPES)
def test_few_rows_matmul_matches_oracle(cuda_device, tokens, out_features, in_features):
    """The decode-batch form (mma.sync, tokens as columns; 32- and 64-row weight tiles, ragged
    last tiles) against the restated matmul and the single-token matvec; a second projection
    reuses the converted rows."""
    from quickdraw_b200 import kernels
    src = synthetic.Source(23, "cpu")
    proj = src.nvfp4(f"w{out_features}x{in_features}", out_features, in_features, global_scale=0.75)
    other = src.nvfp4(f"v{in_features}", 64, in_features, global_scale=1.5)
    x = src.normal(f"x{tokens}", tokens, in_features)
    x[0, :5] = torch.tensor([7.0e4, -3.0e5, 1.0e-6, 0.0, 2.5])       # a row that would leave f16
    got, scratch = kernels.matmul_rows(x.to(cuda_device), to_device(proj, cuda_device))
    again, _ = kernels.matmul_rows(x.to(cuda_device), to_device(other, cuda_device), scratch, convert=False)
    got, again = got.cpu(), again.cpu()
    want = O.nvfp4_matmul(x, proj)
    assert got.shape == want.shape and torch.isfinite(got.float()).all()
    torch.testing.assert_close(got[1:].float(), want[1:].float(), rtol=0.02, atol=0.002)
    assert O.rel_l2(got, want) < 2e-3
    assert O.rel_l2(again, O.nvfp4_matmul(x, other)) < 2e-3
    for t in sorted({0, tokens // 2, tokens - 1}):
        row = O.nvfp4_gemv(x[t], proj)
        assert O.rel_l2(got[t], row) < 2e-3
    # three matrices of one input in one launch: bit-identical to the single launches
    from quickdraw_b200._lib import call, lib, ptr, stream_of
    third = src.nvfp4(f"u{in_features}", 48, in_features, global_scale=0.3)
    devs = [to_device(p_, cuda_device) for p_ in (proj, other, third)]
    xd = x.to(cuda_device)
    outs = [torch.empty(tokens, p_.out_features, dtype=torch.bfloat16, device=cuda_device) for p_ in devs]
    args = []
    for p_, out in zip(devs, outs):
        args += [ptr(p_.weight), ptr(p_.weight_scale), ptr(p_.weight_scale_2), ptr(out), p_.out_features]
    call("qd_nvfp4_matmul_rows3", ptr(xd), None, tokens, in_features, 16, ptr(scratch), 1, 3, *args, stream_of(xd))
    single, _ = kernels.matmul_rows(xd, devs[2], scratch, convert=False)
    assert torch.equal(outs[0].cpu(), got) and torch.equal(outs[1].cpu(), again) and torch.equal(outs[2], single)
    # SwiGLU of two inputs formed on the way in: the same as the product of the explicit SwiGLU rows
    gate, up = src.normal(f"g{tokens}", tokens, in_features), src.normal(f"u{tokens}", tokens, in_features)
    hidden = (torch.nn.functional.silu(gate.float()).to(torch.bfloat16).float() * up.float()).to(torch.bfloat16)
    fused, _ = kernels.matmul_rows(gate.to(cuda_device), to_device(proj, cuda_device), x_up=up.to(cuda_device))
    plain, _ = kernels.matmul_rows(hidden.to(cuda_device), to_device(proj, cuda_device))
    assert O.rel_l2(fused.cpu(), plain.cpu()) < 2e-3


@pytest.mark.parametrize("tokens,out_features,in_features", [(1, 2, 128), (37, 514, 2048), (128, 128, 256), (300, 2048, 4096)])
def test_fp8_matmul_matches_row_by_row_oracle(cuda_device, tokens, out_features, in_features):
    """The static-FP8 projection of a chunk (E4M3 x E4M3 on mma.sync, ragged tiles on both sides)
    against the oracle's fp8_gemv row by row; activations beyond the E4M3 range saturate."""
    from quickdraw_b200._lib import call, ptr, stream_of
    from quickdraw_b200.weights import FP8Linear
    gen = torch.Generator().manual_seed(33)
    w = (torch.randn(out_features, in_features, generator=gen) * 64).clamp(-448, 448).to(torch.float8_e4m3fn)
    proj = FP8Linear(w, torch.tensor(0.1 / 64), torch.tensor(4.0 / 448))
    x = (torch.randn(tokens, in_features, generator=gen) * 1.5).to(torch.bfloat16)
    x[0, :3] = torch.tensor([9.0, -30.0, 4.0])          # saturate at +-448 input-scale units
    dev = cuda_device
    xd, wd = x.to(dev), w.to(dev)
    ws, xs = proj.weight_scale.to(dev), proj.input_scale.to(dev)
    y = torch.empty(tokens, out_features, dtype=torch.bfloat16, device=dev)
    scratch = torch.empty(tokens * in_features, dtype=torch.uint8, device=dev)
    call("qd_fp8_matmul", ptr(xd), ptr(wd), ptr(ws), ptr(xs), ptr(y), tokens, out_features, in_features, ptr(scratch), 1,
         stream_of(xd))
    again = torch.empty_like(y)
    call("qd_fp8_matmul", ptr(xd), ptr(wd), ptr(ws), ptr(xs), ptr(again), tokens, out_features, in_features, ptr(scratch), 0,
         stream_of(xd))
    torch.cuda.synchronize()
    want_q, _ = O.quantize_fp8(x, proj.input_scale)
    assert torch.equal(scratch.view(tokens, in_features).cpu(), want_q.view(torch.uint8))
    assert torch.equal(y, again)
    for t in sorted({0, tokens // 2, tokens - 1}):
        row = O.fp8_gemv(x[t], proj)
        assert O.rel_l2(y[t].cpu(), row) < 2e-3, t


def test_two_dimensional_input_takes_the_matmul_path(cuda_device):
    from quickdraw_b200 import kernels
    src = synthetic.Source(22, "cpu")
    proj = src.nvfp4("w", 512, 2048)
    x = src.normal("x", 5, 2048)
    dev_proj = to_device(proj, cuda_device)
    chunk = kernels.nvfp4_gemv(x.to(cuda_device), dev_proj).cpu()
    for t in range(5):
        single = kernels.nvfp4_gemv(x[t].to(cuda_device), dev_proj).cpu()
        torch.testing.assert_close(chunk[t].float(), single.float(), rtol=0.025, atol=0.003)


W4A4_SHAPES = [(1, 128, 256), (7, 256, 512), (128, 256, 2048), (129, 1024, 2048), (300, 2048, 4096), (515, 512, 2048)]


@pytest.mark.parametrize("tokens,width", [(1, 256), (5, 2048), (130, 4096), (64, 512)])
def test_activation_quantiser_is_bit_exact(cuda_device, tokens, width):
    """Codes, block scales and tensor scale of the activation operand against the oracle's
    restatement: identical bytes (round to nearest even everywhere), incl. an all-zero block,
    a block of equal magnitudes and values on rounding ties."""
    from quickdraw_b200 import kernels
    src = synthetic.Source(31, "cpu")
    x = src.normal(f"x{tokens}x{width}", tokens, width)
    x[0, :16] = 0
    x[0, 16:32] = 0.375
    x[-1, -16:] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    codes, scales, g = kernels.quantize_act(x.to(cuda_device))
    want_codes, want_scales, want_g = O.quantize_act_nvfp4(x)
    assert float(g.cpu()) == float(want_g)
    assert torch.equal(scales.cpu().view(torch.uint8), want_scales)
    assert torch.equal(codes.cpu(), want_codes)
    # the quantised chunk is the input within FP4's resolution
    back = O.dequantize_act_nvfp4(want_codes, want_scales, want_g) * want_g
    assert O.rel_l2(back, x.float()) < 0.12


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("tokens,out_features,in_features", W4A4_SHAPES)
def test_w4a4_matmul_matches_oracle(cuda_device, tokens, out_features, in_features, wide):
    """The block-scaled FP4 x FP4 product against the oracle's product of the same quantised
    operands (fp32-accumulation tolerance), and its distance from the exact W4A16 product (the
    activation rounding: about one tenth relative L2 for Gaussian inputs)."""
    from quickdraw_b200 import kernels
    src = synthetic.Source(32, "cpu")
    proj = src.nvfp4(f"w{out_features}x{in_features}", out_features, in_features, global_scale=0.75)
    x = src.normal(f"x{tokens}", tokens, in_features)
    if wide and out_features % 256:
        pytest.skip("256-row tiles need out_features % 256 == 0")
    xq = kernels.quantize_act(x.to(cuda_device))
    got = kernels.matmul_w4a4(xq, to_device(proj, cuda_device), wide_tiles=wide).cpu()
    assert kernels.matmul_status(cuda_device) == 0
    want = O.nvfp4_matmul_w4a4(*O.quantize_act_nvfp4(x), proj)
    assert got.shape == want.shape
    torch.testing.assert_close(got.float(), want.float(), rtol=0.02, atol=0.002)
    assert O.rel_l2(got, want) < 2e-3
    exact = O.nvfp4_matmul(x, proj)
    assert O.rel_l2(got, exact) < 0.2

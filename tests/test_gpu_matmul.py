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

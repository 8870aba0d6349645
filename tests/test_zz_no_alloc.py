"""The allocation-free attention entry point (``qd_attn_decode_static``) against the regular
one.  Some callers cannot allocate device memory - a plugin living inside another runtime's
pool, a latency path that must stay clear of the CUDA allocator - so this variant keeps its
split-context scratch in an array compiled into the library.  Both entry points are called
through the C ABI on the same inputs, twice in a row (the built-in array keeps the previous
call's contents, so the second call checks that nothing stale leaks), and must agree within
the tolerance the other block tests use.  This file sorts last on purpose."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(device, seed, capacity=512):
    g = torch.Generator(device=device).manual_seed(seed)
    rnd = lambda *shape, s=1.0: (torch.randn(shape, generator=g, device=device) * s).bfloat16()
    return dict(qg=rnd(16, 512), k_new=rnd(2, 256), v_new=rnd(2, 256), q_norm=rnd(256, s=0.02),
                k_norm=rnd(256, s=0.02), k=rnd(capacity, 2, 256), v=rnd(capacity, 2, 256))


def _run(entry, case, position, device):
    from quickdraw_b200 import _lib
    from quickdraw_b200._lib import call, ptr, stream_of
    lib = _lib.lib()
    k, v = case["k"].clone(), case["v"].clone()
    out = torch.empty(16 * 256, dtype=torch.bfloat16, device=device)
    common = (ptr(case["qg"]), ptr(case["k_new"]), ptr(case["v_new"]), ptr(case["q_norm"]), ptr(case["k_norm"]),
              ptr(k), ptr(v), ptr(out))
    tail = (None, position, k.shape[0], 16, 2, 256, 64, 1.0e7, 1.0e-6, 32)
    if entry == "static":
        call("qd_attn_decode_static", *common, *tail, stream_of(out))
    else:
        floats = lib.qd_attn_scratch_floats(16, 2, 256, 32)
        scratch = torch.empty(floats, dtype=torch.float32, device=device)
        counters = torch.zeros(2, dtype=torch.int32, device=device)
        call("qd_attn_decode", *common, ptr(scratch), ptr(counters), *tail, 0, stream_of(out))
    torch.cuda.synchronize(device)
    return out, k, v


def test_static_scratch_matches_regular_entry_point_twice(cuda_device):
    for seed, position in ((1, 300), (2, 37)):          # two calls in a row on the shared array
        case = _case(cuda_device, seed)
        want, wk, wv = _run("regular", case, position, cuda_device)
        got, gk, gv = _run("static", case, position, cuda_device)
        torch.testing.assert_close(got.float(), want.float(), rtol=0.02, atol=0.002)
        assert torch.equal(gk, wk) and torch.equal(gv, wv)


def test_static_scratch_at_a_long_context(cuda_device):
    """8192 cached positions: every one of the 32 context splits is many chunks long."""
    case = _case(cuda_device, 4, capacity=8192)
    want, wk, wv = _run("regular", case, 8191, cuda_device)
    got, gk, gv = _run("static", case, 8191, cuda_device)
    torch.testing.assert_close(got.float(), want.float(), rtol=0.02, atol=0.002)
    assert torch.equal(gk, wk) and torch.equal(gv, wv)


def test_static_scratch_rejects_oversized_shapes(cuda_device):
    from quickdraw_b200 import _lib
    from quickdraw_b200._lib import ptr, stream_of
    case = _case(cuda_device, 3, capacity=64)
    out = torch.empty(16 * 256, dtype=torch.bfloat16, device=cuda_device)
    rc = _lib.lib().qd_attn_decode_static(
        ptr(case["qg"]), ptr(case["k_new"]), ptr(case["v_new"]), ptr(case["q_norm"]), ptr(case["k_norm"]),
        ptr(case["k"]), ptr(case["v"]), ptr(out), None, 5, 64, 16, 2, 256, 64, 1.0e7, 1.0e-6, 128,
        stream_of(out))
    assert rc == 5          # QD_ERR_TOO_LARGE: 128 splits need 2 MiB
    assert b"capacity" in _lib.lib().qd_error_string(rc)

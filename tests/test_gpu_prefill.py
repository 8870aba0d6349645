"""Chunked prefill (sequence kernels + tensor-core products) against the token loop through the
decode step: same state and same logits for the next token, up to fp32 summation order — the
reference's own criterion for its chunked path (tests/engine/test_cuda.py:132-147), loosened the
way the whole-step tests are, because bf16 rounding points amplify last-bit differences."""

import pytest
import torch

from oracle import decode_oracle as O
from quickdraw_b200 import synthetic
from quickdraw_b200.state import DecodeState

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunk,fp8_mixers", [(5, False), (16, False), (39, False), (16, True), (39, True)])
def test_chunked_prefill_matches_token_loop(cuda_device, chunk, fp8_mixers):
    """NVFP4 mixers, and the published checkpoint's static-FP8 mixers (the chunk takes them through
    the E4M3 x E4M3 product, the token loop quantises the vector in the step's phase prologue)."""
    from quickdraw_b200.fused import FusedStep
    from quickdraw_b200.prefill import ChunkPrefill
    cfg = synthetic.model_config(num_layers=4, vocab_size=2048, experts=16, topk=8)
    ckpt = synthetic.make_checkpoint(cfg, seed=11, device="cuda", fp8_mixers=fp8_mixers)
    step, prefill = FusedStep(ckpt), ChunkPrefill(ckpt)
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=gen).to("cuda")
    loop_state, chunk_state = (DecodeState.allocate(cfg, 64, "cuda") for _ in range(2))
    for s in (loop_state, chunk_state):
        s.kv_k.zero_()
        s.kv_v.zero_()
    for position in range(40):
        want = step(ckpt, prompt[position], position, loop_state, logits=position == 39)
    for start in range(0, 39, chunk):
        stop = min(39, start + chunk)
        prefill.run(prompt[start:stop], start, chunk_state)
    got = step(ckpt, prompt[39], 39, chunk_state)
    assert prefill.check() == 0 and step.status() == 0
    if fp8_mixers:
        # E4M3 activations turn last-bit differences of a layer's output into 6 % steps of single inputs of
        # the next, and a router near-tie that falls the other way into a different expert: the first layer
        # agrees to rounding, the whole model only loosely (the blocks are compared one by one below)
        assert O.rel_l2(chunk_state.conv_state[0].cpu(), loop_state.conv_state[0].cpu()) < 1e-3
        assert O.rel_l2(chunk_state.rec_state[0].cpu(), loop_state.rec_state[0].cpu()) < 1e-3
        assert O.rel_l2(chunk_state.kv_k[:, :40].cpu(), loop_state.kv_k[:, :40].cpu()) < 0.35
        assert O.rel_l2(got.cpu(), want.cpu()) < 0.35
        return
    assert O.rel_l2(chunk_state.conv_state.cpu(), loop_state.conv_state.cpu()) < 2e-2
    assert O.rel_l2(chunk_state.rec_state.cpu(), loop_state.rec_state.cpu()) < 2e-2
    assert O.rel_l2(chunk_state.kv_k[:, :40].cpu(), loop_state.kv_k[:, :40].cpu()) < 2e-2
    assert O.rel_l2(chunk_state.kv_v[:, :40].cpu(), loop_state.kv_v[:, :40].cpu()) < 2e-2
    assert O.rel_l2(got.cpu(), want.cpu()) < 5e-2


def test_fp8_mixer_blocks_of_a_chunk_match_the_oracle(cuda_device):
    """Static-FP8 mixers in the chunk forms, block by block on the same inputs (no propagation through
    E4M3 rounding steps and router ties): a DeltaNet block and an attention block over 20 tokens
    against the oracle's single-token blocks walked over the tokens."""
    from quickdraw_b200.prefill import ChunkPrefill
    from quickdraw_b200.synthetic import to_device
    cfg = synthetic.model_config(num_layers=4, vocab_size=2048, experts=16, topk=8)
    ckpt = synthetic.make_checkpoint(cfg, seed=11, device="cuda", fp8_mixers=True)
    cpu = to_device(ckpt, "cpu")
    prefill = ChunkPrefill(ckpt)
    tokens = 20
    x = synthetic.Source(3, "cpu").normal("x", tokens, cfg.hidden_size)
    state, ref = DecodeState.allocate(cfg, 32, "cuda"), DecodeState.allocate(cfg, 32, "cpu")
    for s in (state, ref):
        for t in (s.kv_k, s.kv_v, s.rec_state, s.conv_state):
            t.zero_()
    got = prefill._delta_net(ckpt.layers[0].attn, x.to("cuda"), state, 0).cpu()
    for t in range(tokens):
        want = O.gated_delta_net_block(cpu.layers[0].attn, x[t], ref.rec_state[0], ref.conv_state[0], t, config=cfg)
        assert O.rel_l2(got[t], want) < 1e-2, t
    assert O.rel_l2(state.rec_state[0].cpu(), ref.rec_state[0]) < 1e-2
    assert O.rel_l2(state.conv_state[0].cpu(), ref.conv_state[0]) < 1e-3
    attention = next(layer for layer in ckpt.layers if layer.layer_type == "full_attention")
    got = prefill._attention(attention.attn, x.to("cuda"), state, 0, 0).cpu()
    for t in range(tokens):
        want = O.full_attention_block(cpu.layers[attention.idx].attn, x[t], (ref.kv_k[0], ref.kv_v[0]), t, config=cfg)
        assert O.rel_l2(got[t], want) < 1e-2, t
    assert O.rel_l2(state.kv_k[0, :tokens].cpu(), ref.kv_k[0, :tokens]) < 1e-3
    assert prefill.check() == 0


@pytest.mark.parametrize("experts,topk,tokens,width,rows,few_rows", [
    (8, 3, 21, 512, 264, 0),       # few tiles: 64-row weight tiles
    (40, 2, 30, 256, 256, 0),      # 128-row weight tiles
    (64, 2, 40, 256, 768, 0),      # every SM busy: 256-row (or balanced 128-row) weight tiles
    (8, 3, 21, 512, 272, 32),      # the few-rows form: up to eight routes per expert, a ragged last weight tile
    (4, 2, 50, 2048, 512, 32),     # ... 25 routes per expert: four groups of eight, the last one with a single route
    (40, 8, 3, 512, 2048, 32),     # ... most experts without a route
    (8, 3, 21, 512, 272, 0),       # the same shape through the tcgen05 form
    (4, 2, 50, 2048, 512, -32),    # 32 routes per pass: 25 routes per expert in one pass
    (3, 2, 100, 1024, 144, -32),   # ... 67 routes per expert: three passes, the last one with three routes
    (40, 8, 3, 512, 2048, -32),    # ... most experts without a route
    (300, 8, 40, 2048, 1024, 32),  # more experts than SMs
])
def test_grouped_matmul_matches_per_route_matvec(cuda_device, experts, topk, tokens, width, rows, few_rows):
    """The grouped product of the routed experts (tcgen05 tiles, or the mma.sync form for few
    routes per expert) against the single-token expert matvec."""
    from quickdraw_b200 import kernels
    from quickdraw_b200.prefill import ChunkPrefill
    from quickdraw_b200.synthetic import to_device
    src = synthetic.Source(31, "cpu")
    bank = to_device(src.nvfp4("bank", rows, width, experts, global_scale=0.5, per_expert_global=True), cuda_device)
    x = src.normal("x", tokens, width).to(cuda_device)
    gen = torch.Generator().manual_seed(3)
    ids = torch.stack([torch.randperm(experts, generator=gen)[:topk] for _ in range(tokens)]).to(torch.int32).to(cuda_device)
    weights = torch.rand(tokens, topk, generator=gen).to(cuda_device)
    sorted_ids, order = ids.flatten().sort(stable=True)
    boundaries = torch.searchsorted(sorted_ids, torch.arange(experts + 1, device=cuda_device, dtype=torch.int32)).to(torch.int32)
    helper = ChunkPrefill.__new__(ChunkPrefill)
    helper.device = cuda_device
    helper.status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    helper.FEW_ROWS = abs(few_rows) or 0
    helper.ROUTES_PER_PASS = 32 if few_rows < 0 else (8 if few_rows > 0 else 0)
    if few_rows < 0:
        helper.FEW_ROWS = 10 ** 6
    routes = tokens * topk
    plain = helper._grouped(x, bank, order.to(torch.int32), boundaries, routes, topk, by_token=True, scatter=False)
    sorted_rows = x.repeat_interleave(topk, 0)[order].contiguous()
    routed = helper._grouped(sorted_rows, bank, order.to(torch.int32), boundaries, routes, topk, routing=weights.flatten(),
                             by_token=False, scatter=True)
    assert int(helper.status.item()) == 0
    for r in range(routes):
        route = int(order[r])
        token, expert = route // topk, int(ids.flatten()[route])
        want = kernels.expert_gemv(x[token], bank, ids.flatten()[route:route + 1])[0]
        torch.testing.assert_close(plain[r].float(), want.float(), rtol=0.025, atol=0.003)
        want_routed = kernels.expert_gemv(x[token], bank, ids.flatten()[route:route + 1], weights.flatten()[route:route + 1])[0]
        torch.testing.assert_close(routed[route].float(), want_routed.float(), rtol=0.025, atol=0.003)
    if few_rows:
        # a token row beyond the f16 range: its f16 copy is scaled down by a power of two and the sums back up
        big = x.clone()
        big[0] *= 2.0 ** 17
        scaled = helper._grouped(big, bank, order.to(torch.int32), boundaries, routes, topk, by_token=True, scatter=False)
        of_token_0 = (order // topk == 0)
        assert O.rel_l2(scaled[of_token_0].float().cpu(), (plain[of_token_0].float() * 2.0 ** 17).cpu()) < 1e-3
        assert torch.equal(scaled[~of_token_0], plain[~of_token_0])
    # two banks against the same routes (gate and up): one launch in the few-rows form, the same bits either way
    bank2 = to_device(src.nvfp4("bank2", rows, width, experts, global_scale=0.25, per_expert_global=True), cuda_device)
    first, second = helper._grouped_pair(x, bank, bank2, order.to(torch.int32), boundaries, routes, topk)
    alone = helper._grouped(x, bank2, order.to(torch.int32), boundaries, routes, topk, by_token=True, scatter=False)
    assert torch.equal(first, plain) and torch.equal(second, alone)
    # SwiGLU of two inputs formed on the way in (either form; the tcgen05 form runs the SwiGLU kernel first)
    up = src.normal("up", routes, width).to(cuda_device)
    hidden = (torch.nn.functional.silu(sorted_rows.float()).to(torch.bfloat16).float() * up.float()).to(torch.bfloat16)
    fused = helper._grouped(sorted_rows, bank, order.to(torch.int32), boundaries, routes, topk, by_token=False, scatter=True, x_up=up)
    explicit = helper._grouped(hidden, bank, order.to(torch.int32), boundaries, routes, topk, by_token=False, scatter=True)
    assert O.rel_l2(fused.cpu(), explicit.cpu()) < 2e-3


@pytest.mark.parametrize("key_dim,value_dim,tokens", [(128, 128, 37), (128, 128, 3), (128, 96, 16), (64, 64, 21)])
def test_sequence_conv_and_recurrence_match_single_token_kernels(cuda_device, key_dim, value_dim, tokens):
    """The chunk forms of the DeltaNet convolution and recurrence against the single-token
    kernels walked over the same tokens (convolution bit-exact; recurrence up to summation
    order).  Key dimension 128 takes the register-resident kernel, 64 the general one."""
    from quickdraw_b200._lib import call, ptr, stream_of
    hk, hv, width = 2, 4, 4
    channels = 2 * hk * key_dim + hv * value_dim
    src = synthetic.Source(17, "cpu")
    mixed = src.normal("mixed", tokens, channels).to(cuda_device)
    taps = src.normal("taps", channels, width, std=0.5).to(cuda_device)
    a, b = src.normal("a", tokens, hv).to(cuda_device), src.normal("b", tokens, hv).to(cuda_device)
    a_log, dt_bias = src.normal("alog", hv, std=0.5).to(cuda_device), src.normal("dt", hv).to(cuda_device)
    conv0 = src.normal("conv0", channels, width - 1).to(cuda_device)
    rec0 = src.normal("rec0", hv, key_dim, value_dim, std=0.1).float().to(cuda_device)
    s = stream_of(mixed)

    conv_loop, rec_loop = conv0.clone(), rec0.clone()
    conv_rows, out_rows = torch.empty_like(mixed), torch.empty(tokens, hv * value_dim, dtype=torch.bfloat16, device=cuda_device)
    for t in range(tokens):
        call("qd_gdn_conv", ptr(mixed[t]), ptr(taps), ptr(conv_loop), ptr(conv_rows[t]), channels, width, s)
        call("qd_gdn_recurrence", ptr(conv_rows[t]), ptr(a[t]), ptr(b[t]), ptr(a_log), ptr(dt_bias), ptr(rec_loop),
             ptr(out_rows[t]), hk, hv, key_dim, value_dim, 0, s)

    conv_seq, rec_seq = conv0.clone(), rec0.clone()
    conv_out, out = torch.empty_like(mixed), torch.empty_like(out_rows)
    call("qd_seq_gdn_conv", ptr(mixed), ptr(taps), ptr(conv_seq), ptr(conv_out), tokens, channels, width, s)
    call("qd_seq_gdn_recurrence", ptr(conv_out), ptr(a), ptr(b), ptr(a_log), ptr(dt_bias), ptr(rec_seq), ptr(out),
         tokens, hk, hv, key_dim, value_dim, s)
    torch.cuda.synchronize()
    assert torch.equal(conv_out, conv_rows) and torch.equal(conv_seq, conv_loop)
    assert O.rel_l2(rec_seq.cpu(), rec_loop.cpu()) < 1e-4
    assert O.rel_l2(out.cpu(), out_rows.cpu()) < 1e-2


@pytest.mark.parametrize("value_dim,tokens", [(128, 64), (128, 100), (96, 515), (128, 1030)])
def test_chunked_recurrence_matches_token_by_token(cuda_device, value_dim, tokens):
    """The chunked form of the delta rule (64 tokens at a time, tf32 operands on the tensor
    cores) against the token-by-token sequence kernel: outputs and final state within 5e-3
    (tf32 rounding), for runs that end on a chunk boundary and inside a chunk."""
    from quickdraw_b200._lib import call, lib, ptr, stream_of
    hk, hv, key_dim = 2, 4, 128
    channels = 2 * hk * key_dim + hv * value_dim
    src = synthetic.Source(19, "cpu")
    conv = src.normal("conv", tokens, channels).to(cuda_device)
    a, b = src.normal("a", tokens, hv).to(cuda_device), src.normal("b", tokens, hv).to(cuda_device)
    a_log, dt_bias = src.normal("alog", hv, std=0.5).to(cuda_device), src.normal("dt", hv).to(cuda_device)
    rec0 = src.normal("rec0", hv, key_dim, value_dim, std=0.1).float().to(cuda_device)
    s = stream_of(conv)
    rec_seq, rec_chunk = rec0.clone(), rec0.clone()
    out_seq = torch.empty(tokens, hv * value_dim, dtype=torch.bfloat16, device=cuda_device)
    out_chunk = torch.full_like(out_seq, float("nan"))
    call("qd_seq_gdn_recurrence", ptr(conv), ptr(a), ptr(b), ptr(a_log), ptr(dt_bias), ptr(rec_seq), ptr(out_seq),
         tokens, hk, hv, key_dim, value_dim, s)
    scratch = torch.empty(lib().qd_seq_gdn_chunk_scratch_bytes(tokens, hv), dtype=torch.uint8, device=cuda_device)
    call("qd_seq_gdn_recurrence_chunked", ptr(conv), ptr(a), ptr(b), ptr(a_log), ptr(dt_bias), ptr(rec_chunk),
         ptr(out_chunk), tokens, hk, hv, key_dim, value_dim, ptr(scratch), s)
    torch.cuda.synchronize()
    assert torch.isfinite(out_chunk.float()).all() and torch.isfinite(rec_chunk).all()
    errors = (O.rel_l2(out_chunk.cpu(), out_seq.cpu()), O.rel_l2(rec_chunk.cpu(), rec_seq.cpu()))
    assert max(errors) < 5e-3, errors
    # token by token as well: no single row is far off
    rows = (out_chunk.float() - out_seq.float()).norm(dim=1) / out_seq.float().norm(dim=1).clamp_min(1e-6)
    assert float(rows.max()) < 3e-2, float(rows.max())


@pytest.mark.parametrize("routes,experts", [(4088, 256), (24, 16), (5000, 7), (1, 3)])
def test_group_routes_is_the_stable_sort_by_expert(cuda_device, routes, experts):
    from quickdraw_b200._lib import call, ptr, stream_of
    gen = torch.Generator().manual_seed(routes)
    ids = torch.randint(0, experts, (routes,), generator=gen).to(torch.int32).to(cuda_device)
    if routes > 100:
        ids[ids == 3] = 2                                   # an expert without routes
    order = torch.empty(routes, dtype=torch.int32, device=cuda_device)
    boundaries = torch.empty(experts + 1, dtype=torch.int32, device=cuda_device)
    call("qd_seq_group_routes", ptr(ids), routes, experts, ptr(order), ptr(boundaries), stream_of(ids))
    sorted_ids, want_order = ids.sort(stable=True)
    want_boundaries = torch.searchsorted(sorted_ids, torch.arange(experts + 1, device=cuda_device, dtype=torch.int32))
    assert torch.equal(order.long(), want_order) and torch.equal(boundaries.long(), want_boundaries)


@pytest.mark.parametrize("tokens,hidden,topk", [(5, 2048, 8), (33, 4096, 2), (1, 520, 3)])
def test_combine_with_the_next_norm_equals_the_two_calls(cuda_device, tokens, hidden, topk):
    """The MoE combine with the residual add + RMSNorm of the next layer in its launch: the same bits as
    qd_seq_moe_combine followed by qd_seq_add_rms_norm."""
    from quickdraw_b200._lib import call, ptr, stream_of
    src = synthetic.Source(43, cuda_device)
    contributions = src.normal("c", tokens * topk, hidden)
    shared, residual = src.normal("s", tokens, hidden), src.normal("r", tokens, hidden)
    strength = src.normal("g", tokens, 1)
    gamma = (1 + src.normal("w", hidden, std=0.1).float()).contiguous()
    gen = torch.Generator().manual_seed(tokens)
    ids = torch.stack([torch.randperm(64, generator=gen)[:topk] for _ in range(tokens)]).to(torch.int32).to(cuda_device)
    out, normed, new_residual = (torch.empty(tokens, hidden, dtype=torch.bfloat16, device=cuda_device) for _ in range(3))
    fused_normed, fused_residual = torch.empty_like(normed), torch.empty_like(normed)
    call("qd_seq_moe_combine", ptr(contributions), ptr(ids), ptr(shared), ptr(strength), ptr(out), tokens, hidden, topk,
         stream_of(out))
    call("qd_seq_add_rms_norm", ptr(out), ptr(residual), ptr(gamma), ptr(normed), ptr(new_residual), tokens, hidden, 1e-6,
         stream_of(out))
    call("qd_seq_moe_combine_norm", ptr(contributions), ptr(ids), ptr(shared), ptr(strength), ptr(residual), ptr(gamma),
         ptr(fused_normed), ptr(fused_residual), tokens, hidden, topk, 1e-6, stream_of(out))
    assert torch.equal(fused_normed, normed) and torch.equal(fused_residual, new_residual)


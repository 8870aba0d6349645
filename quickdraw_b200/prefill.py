"""Prompt tokens in chunks: the sequence form of the token step (no logits).

The reference prefills in chunks of 128 tokens (quickdraw/engine/engine.py:98-104): every
projection of a chunk is one matrix product, the token-sequential parts (DeltaNet convolution
and recurrence, causal attention) walk the chunk inside one kernel, the routed experts run as
a grouped product over the chunk's (token, slot) routes sorted by expert
(quickdraw/kernel/triton/moe.py:60-151).  Here the products run on the tensor cores
(``qd_nvfp4_matmul`` / ``qd_nvfp4_grouped_matmul``, tcgen05) and the glue kernels apply the
single-token arithmetic row by row; the state (KV cache, recurrent state, convolution
history) ends up where the token loop would leave it, up to fp32 summation order.

``ChunkPrefill.run`` advances the state over a chunk and returns nothing: the engine feeds
the last prompt token through the decode step, which produces the logits.
"""

from __future__ import annotations

import torch

from ._lib import call, lib, ptr, stream_of
from .weights import Checkpoint, FP8Linear, NVFP4Linear

BF16 = torch.bfloat16


class ChunkPrefill:
    """``expert_range`` / ``group``: expert parallel.  The checkpoint holds the banks of experts
    [lo, hi) only; every rank routes all tokens (the router is replicated), multiplies the routes
    of its own experts and leaves zero rows for the others; one all-reduce per layer moves the
    bf16 contribution rows (every row has exactly one writer, so the sum is a copy) and every
    rank combines them in ascending expert id like a single GPU."""

    sliced, group, expert_range = False, None, None      # defaults of a whole model on one GPU
    total_experts = None                                  # experts of the whole model (None: the bank's own count)
    _rows_scratch = None
    _expert_scratch = None
    _retired = None
    _fp8_rows = None
    CHUNKED_FROM = 64                                     # tokens from which the DeltaNet recurrence takes the chunked form
    FEW_TOKENS = 32                                       # token rows up to which a dense product takes the mma.sync form
    ROUTES_PER_PASS = 0                                   # 8 / 32 routes per decoding of a weight tile; 0: the library chooses
    FEW_ROWS = 20                                         # mean routes per expert up to which the mma.sync form is used

    def __init__(self, ckpt: Checkpoint, expert_range: tuple[int, int] | None = None, group=None):
        c = ckpt.config
        self.ckpt, self.device = ckpt, ckpt.embed_tokens.device
        self.expert_range = expert_range or (0, c.num_experts)
        self.sliced = self.expert_range != (0, c.num_experts)
        self.total_experts = c.num_experts
        self.group = group
        self.gammas = [((1 + layer.input_layernorm.float()).contiguous(),
                        (1 + layer.post_attention_layernorm.float()).contiguous()) for layer in ckpt.layers]
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._rows_scratch, self._expert_scratch, self._retired = {}, {}, []
        for layer in ckpt.layers:
            assert layer.moe.experts_gate.weight.shape[0] == self.expert_range[1] - self.expert_range[0], \
                "the expert banks must hold exactly the owned range"

    # ------------------------------------------------------------------ building blocks
    def _empty(self, *shape, dtype=BF16):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _retire(self, scratch):
        """Keep a scratch area that is being replaced by a larger one: a captured graph may still write to it."""
        if scratch is not None:
            self._retired = (self._retired or []) + [scratch]

    def _rows_form(self, tokens, proj):
        return tokens <= self.FEW_TOKENS and proj.in_features % 512 == 0 and proj.out_features % 16 == 0

    def _matmul(self, x, proj: NVFP4Linear, x_up=None):
        """x W^T; with ``x_up`` the input is the SwiGLU of (x, x_up), formed on the way in by the
        decode-batch form and by a separate kernel otherwise."""
        out = self._empty(x.shape[0], proj.out_features)
        if isinstance(proj, FP8Linear):
            # a static-FP8 mixer projection: the rows are quantised once per input and input scale
            if x_up is not None:
                x = self._swiglu(x, x_up)
            scratch, source, scale = self._fp8_rows or (None, None, None)
            if scratch is None or scratch.numel() < x.numel():
                self._retire(scratch)
                scratch = torch.empty(x.numel(), dtype=torch.uint8, device=self.device)
                source = None
            fresh = source is not x or scale != proj.input_scale.data_ptr()      # (no host read of the scale: capturable)
            call("qd_fp8_matmul", ptr(x), ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.input_scale), ptr(out),
                 x.shape[0], proj.out_features, proj.in_features, ptr(scratch), int(fresh), stream_of(x))
            self._fp8_rows = (scratch, x, proj.input_scale.data_ptr())
            return out
        if self._rows_form(x.shape[0], proj):
            # a decode batch: weights decoded once on mma.sync with the tokens as columns; the f16
            # copy of the token rows is shared by the projections of the same input
            if self._rows_scratch is None:
                self._rows_scratch = {}
            scratch, source = self._rows_scratch.get(proj.in_features, (None, None))
            fresh = x_up is not None or source is not x      # a SwiGLU input is converted every time
            if scratch is None:
                size = lib().qd_nvfp4_matmul_rows_scratch_bytes(proj.in_features)
                scratch = torch.empty(size, dtype=torch.uint8, device=self.device)
            call("qd_nvfp4_matmul_rows", ptr(x), ptr(x_up), ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.weight_scale_2),
                 ptr(out), x.shape[0], proj.out_features, proj.in_features, proj.group_size, ptr(scratch),
                 int(fresh), stream_of(x))
            self._rows_scratch[proj.in_features] = (scratch, None if x_up is not None else x)
            return out
        if x_up is not None:
            x = self._swiglu(x, x_up)
        call("qd_nvfp4_matmul", ptr(x), ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.weight_scale_2),
             ptr(out), x.shape[0], proj.out_features, proj.in_features, proj.group_size, ptr(self.status),
             stream_of(x))
        return out

    def _matmul_many(self, x, projections):
        """The products of one input with up to three matrices; in the decode-batch form they share a launch."""
        if not (len(projections) <= 3 and all(isinstance(proj, NVFP4Linear) and self._rows_form(x.shape[0], proj)
                                              and proj.in_features == projections[0].in_features for proj in projections)):
            return [self._matmul(x, proj) for proj in projections]
        first = projections[0]
        if self._rows_scratch is None:
            self._rows_scratch = {}
        scratch, source = self._rows_scratch.get(first.in_features, (None, None))
        if scratch is None:
            scratch = torch.empty(lib().qd_nvfp4_matmul_rows_scratch_bytes(first.in_features), dtype=torch.uint8, device=self.device)
        outs = [self._empty(x.shape[0], proj.out_features) for proj in projections]
        args = []
        for proj, out in zip(projections, outs):
            args += [ptr(proj.weight), ptr(proj.weight_scale), ptr(proj.weight_scale_2), ptr(out), proj.out_features]
        args += [None, None, None, None, 0] * (3 - len(projections))
        call("qd_nvfp4_matmul_rows3", ptr(x), None, x.shape[0], first.in_features, first.group_size, ptr(scratch),
             int(source is not x), len(projections), *args, stream_of(x))
        self._rows_scratch[first.in_features] = (scratch, x)
        return outs

    def _small(self, x, weight):
        rows = weight.shape[0]
        out = self._empty(x.shape[0], rows)
        call("qd_seq_bf16_matmul", ptr(x), ptr(weight), ptr(out), x.shape[0], rows, x.shape[1], stream_of(x))
        return out

    def _small_pair(self, x, weight0, weight1):
        """Two small bf16 projections of the same input in one launch."""
        out0, out1 = self._empty(x.shape[0], weight0.shape[0]), self._empty(x.shape[0], weight1.shape[0])
        call("qd_seq_bf16_matmul2", ptr(x), ptr(weight0), ptr(out0), weight0.shape[0], ptr(weight1), ptr(out1), weight1.shape[0],
             x.shape[0], x.shape[1], stream_of(x))
        return out0, out1

    def _add_norm(self, x, residual, gamma, eps):
        normed, new_residual = torch.empty_like(x), torch.empty_like(x)
        call("qd_seq_add_rms_norm", ptr(x), ptr(residual), ptr(gamma), ptr(normed), ptr(new_residual),
             x.shape[0], x.shape[1], eps, stream_of(x))
        return normed, new_residual

    def _swiglu(self, gate, up):
        out = torch.empty_like(gate)
        call("qd_swiglu", ptr(gate), ptr(up), ptr(out), gate.numel(), stream_of(gate))
        return out

    def _few_rows(self, routes, bank):
        return (routes <= self.FEW_ROWS * (self.total_experts or bank.weight.shape[0]) and bank.in_features in (512, 1024, 2048)
                and bank.out_features % 16 == 0)

    def _expert_rows_scratch(self, in_rows, in_features):
        """The area for the f16 copy of the input rows of the few-rows form, and the input it holds."""
        if self._expert_scratch is None:
            self._expert_scratch = {}
        scratch, source = self._expert_scratch.get(in_features, (None, None))
        need = lib().qd_nvfp4_expert_rows_scratch_bytes(in_rows, in_features)
        if scratch is None or scratch.numel() < need:
            self._retire(scratch)
            scratch, source = torch.empty(need, dtype=torch.uint8, device=self.device), None
        return scratch, source

    def _grouped_pair(self, x, bank, bank2, order, boundaries, routes, topk):
        """The gate and up products of the routed experts (token rows in, sorted order out); one launch in the few-rows form."""
        if not (self._few_rows(routes, bank) and bank.weight.shape == bank2.weight.shape):
            return (self._grouped(x, bank, order, boundaries, routes, topk, by_token=True, scatter=False),
                    self._grouped(x, bank2, order, boundaries, routes, topk, by_token=True, scatter=False))
        out, out2 = self._empty(routes, bank.out_features), self._empty(routes, bank.out_features)
        scratch, source = self._expert_rows_scratch(routes // topk, bank.in_features)
        call("qd_nvfp4_expert_rows2", ptr(x), ptr(bank.weight), ptr(bank.weight_scale), ptr(bank.weight_scale_2), ptr(out),
             ptr(bank2.weight), ptr(bank2.weight_scale), ptr(bank2.weight_scale_2), ptr(out2), ptr(order), ptr(boundaries),
             routes, bank.weight.shape[0], topk, bank.out_features, bank.in_features, bank.group_size,
             int(bank.weight_scale_2.numel() != 1), self.ROUTES_PER_PASS, ptr(scratch), int(source is not x), stream_of(x))
        self._expert_scratch[bank.in_features] = (scratch, x)
        return out, out2

    def _grouped(self, x, bank: NVFP4Linear, order, boundaries, routes, topk, *, routing=None, by_token, scatter, x_up=None):
        # rows of experts another rank owns stay zero in the scattered (route-order) output
        out = (torch.zeros if self.sliced and scatter else torch.empty)((routes, bank.out_features), dtype=BF16, device=self.device)
        experts = bank.weight.shape[0]
        if self._few_rows(routes, bank):
            # few rows per expert: weights decoded once per 8 or 32 routes on mma.sync, no 128-token tiles;
            # the f16 copy of the input rows is shared by the products of the same input (gate, up)
            scratch, source = self._expert_rows_scratch(routes // topk if by_token else routes, bank.in_features)
            fresh = x_up is not None or source is not x
            # 512 inputs (the down product) and eight or more routes per expert: 32 routes per decoding of a tile
            # (measured at 16 routes per expert: 91 against 105 us; the 2048-input products: 245 against 201 us)
            per_pass = self.ROUTES_PER_PASS or (32 if bank.in_features == 512 and routes >= 8 * (self.total_experts or experts) else 0)
            call("qd_nvfp4_expert_rows", ptr(x), ptr(x_up), ptr(bank.weight), ptr(bank.weight_scale), ptr(bank.weight_scale_2),
                 ptr(order), ptr(boundaries), ptr(routing), ptr(out), routes, experts, topk, bank.out_features,
                 bank.in_features, bank.group_size, int(by_token), int(scatter),
                 int(bank.weight_scale_2.numel() != 1), per_pass, ptr(scratch), int(fresh), stream_of(x))
            self._expert_scratch[bank.in_features] = (scratch, None if x_up is not None else x)
            return out
        if x_up is not None:
            x = self._swiglu(x, x_up)
        call("qd_nvfp4_grouped_matmul", ptr(x), ptr(bank.weight), ptr(bank.weight_scale), ptr(bank.weight_scale_2),
             ptr(order), ptr(boundaries), ptr(routing), ptr(out), routes, bank.weight.shape[0], topk,
             bank.out_features, bank.in_features, bank.group_size, int(by_token), int(scatter),
             int(bank.weight_scale_2.numel() != 1), routes, ptr(self.status), stream_of(x))
        return out

    # --------------------------------------------------------------------------- blocks
    def _delta_net(self, w, x, state, index):
        c = self.ckpt.config
        tokens = x.shape[0]
        hv, dv = c.linear_num_value_heads, c.linear_value_head_dim
        qkv, z = self._matmul_many(x, [w.in_proj_qkv, w.in_proj_z])
        a, b = self._small_pair(x, w.in_proj_a, w.in_proj_b)
        conv = torch.empty_like(qkv)
        call("qd_seq_gdn_conv", ptr(qkv), ptr(w.conv1d), ptr(state.conv_state[index]), ptr(conv), tokens,
             qkv.shape[1], c.linear_conv_kernel_dim, stream_of(x))
        core = self._empty(tokens, hv * dv)
        if tokens >= self.CHUNKED_FROM and c.linear_key_head_dim == 128 and dv % 32 == 0:
            # 64 tokens at a time on the tensor cores (closed form of the delta rule within a chunk)
            scratch = torch.empty(lib().qd_seq_gdn_chunk_scratch_bytes(tokens, hv), dtype=torch.uint8, device=self.device)
            call("qd_seq_gdn_recurrence_chunked", ptr(conv), ptr(a), ptr(b), ptr(w.A_log), ptr(w.dt_bias),
                 ptr(state.rec_state[index]), ptr(core), tokens, c.linear_num_key_heads, hv,
                 c.linear_key_head_dim, dv, ptr(scratch), stream_of(x))
        else:
            call("qd_seq_gdn_recurrence", ptr(conv), ptr(a), ptr(b), ptr(w.A_log), ptr(w.dt_bias),
                 ptr(state.rec_state[index]), ptr(core), tokens, c.linear_num_key_heads, hv,
                 c.linear_key_head_dim, dv, stream_of(x))
        gated = torch.empty_like(core)
        call("qd_gdn_gated_norm", ptr(core), ptr(z), ptr(w.norm), ptr(gated), tokens * hv, dv, c.rms_norm_eps,
             stream_of(x))
        return self._matmul(gated, w.out_proj)

    def _attention(self, w, x, state, index, position0):
        c = self.ckpt.config
        tokens = x.shape[0]
        qg, k, v = self._matmul_many(x, [w.q_proj, w.k_proj, w.v_proj])
        q_scratch = self._empty(tokens, c.num_attention_heads * c.head_dim)
        out = torch.empty_like(q_scratch)
        # q/k norm + RoPE + cache rows, then causal attention on the tensor cores: every cache tile
        # is read once per sixteen tokens
        call("qd_seq_attention", ptr(qg), ptr(k), ptr(v), ptr(w.q_norm), ptr(w.k_norm), ptr(state.kv_k[index]),
             ptr(state.kv_v[index]), ptr(q_scratch), ptr(out), tokens, position0, state.kv_k.shape[1],
             c.num_attention_heads, c.num_key_value_heads, c.head_dim, int(c.head_dim * c.partial_rotary_factor),
             c.rope_theta, c.rms_norm_eps, stream_of(x))
        return self._matmul(out, w.o_proj)

    def _moe(self, w, x, follow=None):
        """The MoE block; with ``follow`` = (residual, gamma of the next norm) the residual add and RMSNorm in front
        of the next layer run in the combine's launch and (normed, new residual) is returned."""
        c = self.ckpt.config
        tokens, topk = x.shape[0], c.num_experts_per_tok
        logits, strength = self._small_pair(x, w.router, w.shared_expert_gate)
        ids = self._empty(tokens, topk, dtype=torch.int32)
        weights = self._empty(tokens, topk, dtype=torch.float32)
        call("qd_seq_route_topk", ptr(logits), tokens, c.num_experts, topk, ptr(ids), ptr(weights), stream_of(x))
        # the routes sorted by expert (stable), as the reference groups them
        routes = tokens * topk
        order = self._empty(routes, dtype=torch.int32)
        boundaries = self._empty(c.num_experts + 1, dtype=torch.int32)
        call("qd_seq_group_routes", ptr(ids), routes, c.num_experts, ptr(order), ptr(boundaries), stream_of(x))
        if self.sliced:      # this rank's experts: their slice of the boundaries, indices local to the bank
            boundaries = boundaries[self.expert_range[0]:self.expert_range[1] + 1]
        gate, up = self._grouped_pair(x, w.experts_gate, w.experts_up, order, boundaries, routes, topk)
        # the SwiGLU is formed while the rows of the down product are written as f16 (a separate kernel where
        # the 128-token tiles take the product)
        contributions = self._grouped(gate, w.experts_down, order, boundaries, routes, topk, x_up=up,
                                      routing=weights.flatten(), by_token=False, scatter=True)
        if self.sliced:
            import torch.distributed as dist
            dist.all_reduce(contributions, group=self.group)
        shared_gate, shared_up = self._matmul_many(x, [w.shared_gate, w.shared_up])
        shared = self._matmul(shared_gate, w.shared_down, x_up=shared_up)
        if follow is not None and x.shape[1] % 8 == 0 and x.shape[1] <= 4096:
            residual, gamma = follow
            normed, new_residual = torch.empty_like(x), torch.empty_like(x)
            call("qd_seq_moe_combine_norm", ptr(contributions), ptr(ids), ptr(shared), ptr(strength), ptr(residual), ptr(gamma),
                 ptr(normed), ptr(new_residual), tokens, x.shape[1], topk, c.rms_norm_eps, stream_of(x))
            return normed, new_residual
        out = torch.empty_like(x)
        call("qd_seq_moe_combine", ptr(contributions), ptr(ids), ptr(shared), ptr(strength), ptr(out), tokens,
             x.shape[1], topk, stream_of(x))
        return out if follow is None else self._add_norm(out, follow[0], follow[1], c.rms_norm_eps)

    # ------------------------------------------------------------------------------ run
    @torch.inference_mode()
    def run(self, token_ids: torch.Tensor, position0: int, state) -> None:
        """Advance ``state`` over the tokens at positions position0 .. position0 + len - 1."""
        c = self.ckpt.config
        assert token_ids.ndim == 1 and token_ids.dtype == torch.long and token_ids.is_cuda
        assert 0 <= position0 and position0 + token_ids.numel() <= state.kv_k.shape[1]
        x = self.ckpt.embed_tokens[token_ids].contiguous()
        normed, residual = self._add_norm(x, None, self.gammas[0][0], c.rms_norm_eps)
        for number, (layer, (_, gamma_post)) in enumerate(zip(self.ckpt.layers, self.gammas)):
            if layer.layer_type == "full_attention":
                index = sum(1 for k in c.layer_types[:layer.idx] if k == "full_attention")
                mixed = self._attention(layer.attn, normed, state, index, position0)
            else:
                index = sum(1 for k in c.layer_types[:layer.idx] if k != "full_attention")
                mixed = self._delta_net(layer.attn, normed, state, index)
            if number + 1 == len(self.ckpt.layers):
                break             # the chunk step returns nothing: behind the last mixer no state is written
            normed, residual = self._add_norm(mixed, residual, gamma_post, c.rms_norm_eps)
            # the norm in front of the next layer rides on the combine
            normed, residual = self._moe(layer.moe, normed, follow=(residual, self.gammas[number + 1][0]))

    def check(self) -> int:
        """Status word of the tensor-core products (0 = clean)."""
        return int(self.status.item())

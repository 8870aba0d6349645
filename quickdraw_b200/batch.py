"""Small-batch decode: one token of each of B independent sequences per step, every sequence
with its own KV cache, recurrent state, convolution history and position.

The reference decodes one sequence (quickdraw/engine/engine.py:114-127); its per-layer math
(quickdraw/models/qwen.py:196-241) is applied here to B rows at a time.  Row-independent
operators are the chunk forms of the prefill (tensor-core products with B rows, residual add +
RMSNorm, routing, routes grouped by expert, grouped expert products, combine); the three
operators that touch per-sequence state (DeltaNet convolution and recurrence, attention) are
the single-token kernels with the sequence as one more grid dimension.  The LM head reads every
weight row once for all sequences; the next token of each sequence is the greedy argmax.

``BatchState`` stacks the reference's ``DecodeState`` buffers along a leading sequence axis;
``sequence(b)`` is a ``DecodeState`` view of one sequence, so a prompt is prefilled with the
single-sequence chunk prefill and a sequence can be continued by the single-sequence step.
"""

from __future__ import annotations

import torch

from ._lib import call, lib, ptr, stream_of
from .prefill import ChunkPrefill
from .state import DecodeState
from .weights import Checkpoint

BF16 = torch.bfloat16
MAX_ATTN_SPLITS = 16    # context splits per (sequence, KV head), at most


class BatchState:
    def __init__(self, config, batch: int, max_context: int, device):
        one = DecodeState.allocate(config, 1, "meta")
        full = one.kv_k.shape[0]
        kv_shape = (batch, full, max_context, config.num_key_value_heads, config.head_dim)
        self.kv_k = torch.zeros(kv_shape, dtype=BF16, device=device)
        self.kv_v = torch.zeros(kv_shape, dtype=BF16, device=device)
        self.rec_state = torch.zeros((batch, *one.rec_state.shape), dtype=torch.float32, device=device)
        self.conv_state = torch.zeros((batch, *one.conv_state.shape), dtype=BF16, device=device)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=device)
        self.batch, self.max_context = batch, max_context

    def sequence(self, b: int) -> DecodeState:
        """The buffers of sequence b as the single-sequence container (views, no copy)."""
        return DecodeState(self.kv_k[b], self.kv_v[b], self.rec_state[b], self.conv_state[b],
                           int(self.positions[b].item()))

    def memory_bytes(self) -> int:
        return sum(t.nbytes for t in (self.kv_k, self.kv_v, self.rec_state, self.conv_state))


class BatchDecode(ChunkPrefill):
    """``step(tokens[B], state)`` -> (next tokens [B] int64, logits [B, vocab] bf16)."""

    def __init__(self, ckpt: Checkpoint, expert_range: tuple[int, int] | None = None,
                 vocab_range: tuple[int, int] | None = None, group=None):
        """``expert_range`` / ``vocab_range`` / ``group``: expert parallel (the checkpoint is this
        rank's slice): the routed experts as in ``ChunkPrefill``, the LM head by vocabulary rows
        with one all-gather of the logit shards."""
        super().__init__(ckpt, expert_range=expert_range, group=group)
        self.vocab_range = vocab_range
        c = ckpt.config
        self.final_gamma = (1 + ckpt.final_norm.float()).contiguous()
        self._scratch = None
        self._graphs = {}

    def _attn_splits(self, batch, context):
        """Context splits per (sequence, KV head): the count whose blocks fill whole waves of the
        GPU best (one block per SM; a split costs a merge, 16 at most)."""
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        pairs = batch * self.ckpt.config.num_key_value_heads
        cost = lambda s: -(-pairs * s // sms) * (-(-context // s) + 64)
        return min(range(1, MAX_ATTN_SPLITS + 1), key=cost)

    def _attn_scratch(self, batch):
        c = self.ckpt.config
        if self._scratch is None or self._scratch[0] < batch:
            floats = lib().qd_attn_scratch_floats(c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                                                  MAX_ATTN_SPLITS)
            self._scratch = (batch, torch.empty(batch * floats, dtype=torch.float32, device=self.device),
                             torch.zeros(batch * c.num_key_value_heads, dtype=torch.int32, device=self.device))
        return self._scratch[1], self._scratch[2]

    # ------------------------------------------------------------- per-sequence-state blocks
    def _delta_net_batch(self, w, x, state: BatchState, index):
        c = self.ckpt.config
        batch = x.shape[0]
        hv, dv = c.linear_num_value_heads, c.linear_value_head_dim
        qkv, z = self._matmul_many(x, [w.in_proj_qkv, w.in_proj_z])
        a, b = self._small_pair(x, w.in_proj_a, w.in_proj_b)
        conv = torch.empty_like(qkv)
        conv_state, rec_state = state.conv_state[:, index], state.rec_state[:, index]
        call("qd_batch_gdn_conv", ptr(qkv), ptr(w.conv1d), ptr(conv_state[0]), conv_state.stride(0), ptr(conv),
             batch, qkv.shape[1], c.linear_conv_kernel_dim, stream_of(x))
        core = self._empty(batch, hv * dv)
        call("qd_batch_gdn_recurrence", ptr(conv), ptr(a), ptr(b), ptr(w.A_log), ptr(w.dt_bias),
             ptr(rec_state[0]), rec_state.stride(0), ptr(core), batch, c.linear_num_key_heads, hv,
             c.linear_key_head_dim, dv, stream_of(x))
        gated = torch.empty_like(core)
        call("qd_gdn_gated_norm", ptr(core), ptr(z), ptr(w.norm), ptr(gated), batch * hv, dv, c.rms_norm_eps,
             stream_of(x))
        return self._matmul(gated, w.out_proj)

    def _attention_batch(self, w, x, state: BatchState, index):
        c = self.ckpt.config
        batch = x.shape[0]
        qg, k, v = self._matmul_many(x, [w.q_proj, w.k_proj, w.v_proj])
        out = self._empty(batch, c.num_attention_heads * c.head_dim)
        q_scratch = torch.empty_like(out)
        scratch, counters = self._attn_scratch(batch)
        k_cache, v_cache = state.kv_k[:, index], state.kv_v[:, index]
        call("qd_batch_attention", ptr(qg), ptr(k), ptr(v), ptr(w.q_norm), ptr(w.k_norm), ptr(k_cache[0]),
             ptr(v_cache[0]), k_cache.stride(0), ptr(q_scratch), ptr(out), ptr(scratch), ptr(counters),
             ptr(state.positions), batch, state.max_context, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
             int(c.head_dim * c.partial_rotary_factor), c.rope_theta, c.rms_norm_eps,
             self._attn_splits(batch, state.max_context), stream_of(x))
        return self._matmul(out, w.o_proj)

    # ------------------------------------------------------------------------------ step
    @torch.inference_mode()
    def step(self, tokens: torch.Tensor, state: BatchState, *, positions_checked: bool = False):
        """Feed tokens[b] to sequence b at state.positions[b]; advances every position by one."""
        c = self.ckpt.config
        assert tokens.shape == (state.batch,) and tokens.dtype == torch.long and tokens.is_cuda
        if not positions_checked:
            assert int(state.positions.max().item()) < state.max_context, "a sequence has filled its cache"
        x = self.ckpt.embed_tokens[tokens].contiguous()
        normed, residual = self._add_norm(x, None, self.gammas[0][0], c.rms_norm_eps)
        # the norm after a layer's MoE block (in front of the next layer, or the final one) rides on its combine
        following = [gamma_in for gamma_in, _ in self.gammas[1:]] + [self.final_gamma]
        for (layer, (_, gamma_post)), gamma_next in zip(zip(self.ckpt.layers, self.gammas), following):
            if layer.layer_type == "full_attention":
                index = sum(1 for k in c.layer_types[:layer.idx] if k == "full_attention")
                mixed = self._attention_batch(layer.attn, normed, state, index)
            else:
                index = sum(1 for k in c.layer_types[:layer.idx] if k != "full_attention")
                mixed = self._delta_net_batch(layer.attn, normed, state, index)
            normed, residual = self._add_norm(mixed, residual, gamma_post, c.rms_norm_eps)
            normed, residual = self._moe(layer.moe, normed, follow=(residual, gamma_next))
        final = normed
        head = self.ckpt.lm_head
        logits = self._small(final, head) if isinstance(head, torch.Tensor) else self._matmul(final, head)   # bf16 / NVFP4 head
        if self.vocab_range is not None and logits.shape[1] != c.vocab_size:
            import torch.distributed as dist
            world = dist.get_world_size(self.group)
            shards = torch.empty((world, *logits.shape), dtype=logits.dtype, device=logits.device)
            dist.all_gather_into_tensor(shards, logits.contiguous(), group=self.group)
            logits = shards.permute(1, 0, 2).reshape(logits.shape[0], c.vocab_size)
        state.positions += 1
        return logits.float().argmax(dim=-1), logits

    def graph_step(self, tokens: torch.Tensor, state: BatchState):
        """``step`` replayed from a CUDA graph: a step is some 1 100 launches, which the host
        issues more slowly than the GPU runs them.  The first call with a state runs eagerly (it
        also loads and configures every kernel), the second captures, later ones replay; the
        results live in buffers that the next call overwrites.  ``state.positions`` may only be
        written by the steps themselves once a state has been captured (call ``forget`` after
        writing them)."""
        entry = self._graphs.get(id(state))
        if entry is None:
            out = self.step(tokens, state)
            # host-side bound of the largest position: the device value is read again only when
            # the bound reaches the end of the cache
            self._graphs[id(state)] = {"state": state, "bound": int(state.positions.max().item()), "graph": None}
            return out
        if entry["bound"] >= state.max_context:
            entry["bound"] = int(state.positions.max().item())
            assert entry["bound"] < state.max_context, "a sequence has filled its cache"
        if entry["graph"] is None:
            entry["tokens"] = tokens.clone()
            graph = torch.cuda.CUDAGraph()
            # ordinary edges between the kernels of the graph: measured faster than programmatic ones
            chained = lib().qd_set_chained_launches(0)
            try:
                with torch.cuda.graph(graph):
                    entry["out"] = self.step(entry["tokens"], state, positions_checked=True)
            finally:
                lib().qd_set_chained_launches(chained)
            entry["graph"] = graph
        entry["tokens"].copy_(tokens)
        entry["graph"].replay()
        entry["bound"] += 1
        return entry["out"]

    def forget(self, state: BatchState) -> None:
        """Drop the captured graph of a state (its positions were written from outside)."""
        self._graphs.pop(id(state), None)

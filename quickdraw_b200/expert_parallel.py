"""Expert-parallel decode across the GPUs of one node (one process per GPU).

Partition: rank r of W owns experts [r*E/W, (r+1)*E/W) of every layer's banks; router,
shared expert, mixers, norms, embedding, LM head and the whole decode state are replicated,
so every rank runs the identical step on identical inputs and arrives at the same routing.
A rank multiplies only the selected experts it owns; the fp32 partial sums [hidden] meet in
one NCCL all-reduce per layer, after which every rank rounds the sum to bf16 and adds the
gated shared row exactly as the single-GPU kernel does.  The reference has no distributed
path (it is a single-GPU library); this module is the multi-GPU extension of its engine.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .engine import Engine
from .fused import FusedStep
from .weights import Checkpoint


def expert_range(rank: int, world: int, experts: int) -> tuple[int, int]:
    assert world >= 1 and 0 <= rank < world and experts % world == 0, "experts must split evenly"
    per = experts // world
    return rank * per, (rank + 1) * per


class ExpertParallelStep:
    """``step(ckpt, token_id, position, state, *, logits=True)`` over a sharded checkpoint."""

    def __init__(self, ckpt: Checkpoint, rank: int, world: int, group=None, pdl: bool = True):
        self.rank, self.world, self.group = rank, world, group
        self.fused = FusedStep(ckpt, expert_range=expert_range(rank, world, ckpt.config.num_experts), pdl=pdl)
        self.ckpt = ckpt
        self.next_token = self.fused.next_token
        layers = ckpt.config.num_hidden_layers
        self.launches_per_step = self.fused.launches_per_step + layers + 1   # + one finish per exchange

    def __call__(self, ckpt, token_id, position, state, *, logits=True):
        assert ckpt is self.ckpt
        layers = ckpt.config.num_hidden_layers
        for layer in range(layers):
            self.fused.run_layers(token_id, position, state, layer, layer + 1)
            if layer == layers - 1 and not logits:
                return None        # the last MoE output only feeds the LM head
            dist.all_reduce(self.fused.routed_partial, op=dist.ReduceOp.SUM, group=self.group)
        out = torch.empty(ckpt.config.vocab_size, dtype=torch.bfloat16, device=self.fused.device)
        self.fused.run_layers(token_id, position, state, layers, layers, out)
        return out

    def status(self) -> int:
        return self.fused.status()


class ExpertParallelEngine(Engine):
    """Engine whose step is expert parallel.  Build it on every rank of an initialised NCCL
    process group; ``cfg`` and ``seed`` describe the synthetic model, of which each rank
    generates its own slice (pass ``ckpt=`` to supply an already sharded checkpoint)."""

    def __init__(self, cfg, seed: int = 0, max_context: int = 32768, device="cuda", *, ckpt=None,
                 group=None, cuda_graph: bool = True):
        from . import synthetic
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if ckpt is None:
            ckpt = synthetic.make_checkpoint(cfg, seed, device,
                                             expert_range=expert_range(rank, world, cfg.num_experts))
        step = ExpertParallelStep(ckpt, rank, world, group)
        super().__init__(ckpt, max_context, str(device), "b200", cuda_graph=cuda_graph, _step_object=step)
        self.launches_per_step = step.launches_per_step

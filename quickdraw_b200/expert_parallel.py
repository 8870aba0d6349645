"""Expert-parallel decode across the GPUs of one node (one process per GPU).

Partition: rank r of W owns experts [r*E/W, (r+1)*E/W) of every layer's banks; router,
shared expert, mixers, norms, embedding, LM head and the whole decode state are replicated,
so every rank runs the identical step on identical inputs and arrives at the same routing.
A rank multiplies only the selected experts it owns; the fp32 partial sums [hidden] meet in
one exchange per layer, after which every rank rounds the sum to bf16 and adds the gated
shared row exactly as the single-GPU kernel does.  The exchange is the library's own kernel
over peer memory (every rank stores its vector into every rank's symmetric buffer over NVLink,
flags, bounded wait, sum in rank order: ``qd_peer_all_reduce``) when the symmetric allocation
can be set up on every rank and the group has at most four ranks (the sizes it was run on;
``QD_EP_EXCHANGE=peer`` asks for it on larger groups), else one NCCL all-reduce
(``QD_EP_EXCHANGE=nccl`` forces that).
Measured per token: 3.96 ms (peer) against 4.00 ms (NCCL) on two GPUs, 3.94 ms against 4.36 ms
on four.  The reference has no distributed
path (it is a single-GPU library); this module is the multi-GPU extension of its engine.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ._lib import call, lib, ptr

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
        self.peer = self._peer_exchange(group) if world > 1 else None
        if self.peer is not None:
            self.launches_per_step += layers                                   # the exchange kernels

    def _peer_exchange(self, group):
        """Symmetric buffer + peer pointers for ``qd_peer_all_reduce``, or None (NCCL instead).
        Every rank must come to the same answer: the outcome is agreed on with an all-reduce."""
        ok, state = 1, None
        # the peer kernel was run on 2 and 4 GPUs; larger groups take NCCL unless asked otherwise
        choice = os.environ.get("QD_EP_EXCHANGE", "peer" if self.world <= 4 else "nccl")
        if choice != "peer" or dist.get_backend(group) != "nccl":
            ok = 0
        else:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                n = self.fused.routed_partial.numel()
                nbytes = lib().qd_peer_all_reduce_bytes(self.world, n)
                assert nbytes > 0
                buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.fused.device)
                buffer.zero_()
                name = (group or dist.group.WORLD).group_name
                handle = symm_mem.rendezvous(buffer, name)
                peers = (ctypes.c_ulonglong * self.world)(*[int(a) for a in handle.buffer_ptrs])
                epoch = torch.zeros(1, dtype=torch.int32, device=self.fused.device)
                status = torch.zeros(1, dtype=torch.int32, device=self.fused.device)
                state = (buffer, handle, peers, epoch, status, n)
            except Exception:                      # no symmetric memory on this system
                ok = 0
        agreed = torch.tensor([ok], dtype=torch.int32, device=self.fused.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)      # also orders the zero fill before any exchange
        torch.cuda.synchronize(self.fused.device)
        return state if int(agreed.item()) == 1 else None

    def _exchange(self):
        if self.peer is None:
            dist.all_reduce(self.fused.routed_partial, op=dist.ReduceOp.SUM, group=self.group)
            return
        _, _, peers, epoch, status, n = self.peer
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.fused.device).cuda_stream)
        call("qd_peer_all_reduce", ptr(self.fused.routed_partial), peers, self.rank, self.world, n, ptr(epoch),
             ptr(status), stream)

    def __call__(self, ckpt, token_id, position, state, *, logits=True):
        assert ckpt is self.ckpt
        layers = ckpt.config.num_hidden_layers
        for layer in range(layers):
            self.fused.run_layers(token_id, position, state, layer, layer + 1)
            if layer == layers - 1 and not logits:
                return None        # the last MoE output only feeds the LM head
            self._exchange()
        out = torch.empty(ckpt.config.vocab_size, dtype=torch.bfloat16, device=self.fused.device)
        self.fused.run_layers(token_id, position, state, layers, layers, out)
        return out

    def status(self) -> int:
        exchange = int(self.peer[4].item()) if self.peer is not None else 0
        return self.fused.status() | exchange


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

"""Expert-parallel decode across the GPUs of one node (one process per GPU).

Partition: rank r of W owns experts [r*E/W, (r+1)*E/W) of every layer's banks and rows
[r*V/W, (r+1)*V/W) of the LM head; router, shared expert, mixers, norms, embedding and the
whole decode state are replicated, so every rank runs the identical token step on identical
inputs and arrives at the same routing.  The step stays ONE persistent launch per token on
every rank: in the MoE tail a rank multiplies only the selected experts it owns and stores
their bf16 contribution rows straight into every rank's exchange area (plain stores over
NVLink into peer-mapped memory, every word carrying its tag), each rank then adds all eight
rows from its own area in ascending expert id, exactly the sum a single GPU forms; after
the LM head the ranks' best (logit, index) pairs meet the same way and every rank ends the
step with the same next token.  There is no collective call on the token path.

The exchange areas are one symmetric-memory allocation (torch symmetric memory supplies the
peer mappings; multicast binding is switched off, only unicast peer pointers are used).
Full logits (the end of a prompt) are assembled with one all-gather of the vocabulary shards.
The reference has no distributed path (it is a single-GPU library); this module is the
multi-GPU extension of its engine.
"""

from __future__ import annotations

import os
import threading
import time

import torch
import torch.distributed as dist

from .engine import Engine
from .fused import FusedStep
from .weights import Checkpoint


def expert_range(rank: int, world: int, experts: int) -> tuple[int, int]:
    assert world >= 1 and 0 <= rank < world and experts % world == 0, "experts must split evenly"
    per = experts // world
    return rank * per, (rank + 1) * per


def vocab_range(rank: int, world: int, vocab: int) -> tuple[int, int]:
    assert world >= 1 and 0 <= rank < world and vocab % world == 0, "vocabulary must split evenly"
    per = vocab // world
    return rank * per, (rank + 1) * per


class PeerLost(RuntimeError):
    """A rank of the group stopped answering (or said goodbye) between steps."""


class RankWatchdog:
    """Host-side liveness of the ranks of one group, over a key-value store (a
    ``torch.distributed`` ``TCPStore`` or anything with ``set`` / ``get`` / ``add``).

    Every rank bumps its own counter from a daemon thread every ``interval`` seconds;
    ``check()`` (called before a launch) reads every peer's counter and raises ``PeerLost``
    when a counter has not moved for ``timeout`` seconds, when its rank has left with
    ``leave()``, or when the store itself is gone (the rank that hosts it died).  A launch
    that a lost peer would have stalled is therefore never issued; the bounded waits inside
    the kernel (status bit 0) cover a peer lost in mid-step.  Nothing here touches a GPU.
    """

    def __init__(self, store, rank: int, world: int, *, interval: float = 0.05, timeout: float = 1.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout = interval, timeout
        self._stop = threading.Event()
        self._seen = {r: (-1, time.monotonic()) for r in range(world) if r != rank}
        self.store.add(f"qd/alive/{rank}", 1)
        self._thread = threading.Thread(target=self._beat, name="qd-watchdog", daemon=True)
        self._thread.start()

    def _beat(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self.store.add(f"qd/alive/{self.rank}", 1)
            except Exception:       # the store is gone: check() reports it
                return

    def check(self) -> None:
        now = time.monotonic()
        for peer, (count, since) in self._seen.items():
            try:
                if int(self.store.add(f"qd/left/{peer}", 0)) > 0:
                    raise PeerLost(f"rank {peer} left the group")
                current = int(self.store.add(f"qd/alive/{peer}", 0))
            except PeerLost:
                raise
            except Exception as error:
                raise PeerLost(f"the group's store stopped answering ({type(error).__name__}): "
                               f"the rank that hosts it is gone") from error
            if current != count:
                self._seen[peer] = (current, now)
            elif now - since > self.timeout:
                raise PeerLost(f"rank {peer} has not answered for {now - since:.2f} s")

    def leave(self) -> None:
        """Ordered goodbye: the peers' next ``check()`` names this rank."""
        self._stop.set()
        try:
            self.store.add(f"qd/left/{self.rank}", 1)
        except Exception:
            pass

    def stop(self) -> None:
        self._stop.set()


class ExpertParallelStep:
    """``step(ckpt, token_id, position, state, *, logits=True)`` over a model slice."""

    def __init__(self, ckpt: Checkpoint, rank: int, world: int, group=None, watchdog: RankWatchdog | None = None):
        cfg = ckpt.config
        self.rank, self.world, self.group = rank, world, group
        self.watchdog = watchdog
        self.ckpt = ckpt
        self.vocab = vocab_range(rank, world, cfg.vocab_size)
        self.fused = FusedStep(ckpt, expert_range=expert_range(rank, world, cfg.num_experts),
                               vocab_range=self.vocab, persistent=True)
        self.next_token = self.fused.next_token
        self.launches_per_step = 1
        self.device = self.fused.device
        self.gather_logits = True                 # False: return this rank's shard view only (decode replay)
        self._keep = self._exchange_area(group)

    def _exchange_area(self, group):
        """One symmetric allocation; every rank learns every rank's mapping of it."""
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        nbytes = self.fused.exchange_bytes()
        buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        buffer.zero_()
        name = (group or dist.group.WORLD).group_name
        handle = symm_mem.rendezvous(buffer, name)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)                       # every area is zero before any step stores into it
        self.fused.set_exchange(self.rank, self.world, [int(a) for a in handle.buffer_ptrs])
        return buffer, handle

    def __call__(self, ckpt, token_id, position, state, *, logits=True):
        assert ckpt is self.ckpt
        if self.watchdog is not None:
            self.watchdog.check()                 # raises PeerLost instead of launching into a stall
        out = self.fused(ckpt, token_id, position, state, logits=logits)
        if out is None or not self.gather_logits:
            return out
        lo, hi = self.vocab
        full = torch.empty_like(out)
        dist.all_gather_into_tensor(full, out[lo:hi].contiguous(), group=self.group)
        return full

    def status(self) -> int:
        return self.fused.status()

    def close(self) -> None:
        """Ordered teardown: call on every rank, between steps, before the process group goes."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        if self.watchdog is not None:
            self.watchdog.stop()
        self.fused.exchange = None
        self._keep = None


class ExpertParallelEngine(Engine):
    """Engine whose step is expert parallel.  Build it on every rank of an initialised NCCL
    process group; ``cfg`` and ``seed`` describe the synthetic model, of which each rank
    generates its own slice (pass ``ckpt=`` to supply an already sliced checkpoint)."""

    def __init__(self, cfg, seed: int = 0, max_context: int = 32768, device="cuda", *, ckpt=None,
                 group=None, cuda_graph: bool = True, watchdog: RankWatchdog | None = None):
        from . import synthetic
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if ckpt is None:
            ckpt = synthetic.make_checkpoint(cfg, seed, device,
                                             expert_range=expert_range(rank, world, cfg.num_experts),
                                             vocab_range=vocab_range(rank, world, cfg.vocab_size))
        step = ExpertParallelStep(ckpt, rank, world, group, watchdog)
        super().__init__(ckpt, max_context, str(device), "b200", cuda_graph=cuda_graph, _step_object=step)
        self.launches_per_step = step.launches_per_step
        # prompts in chunks through the sequence kernels, the routed experts split over the ranks
        from .prefill import ChunkPrefill
        self.chunk_prefill = ChunkPrefill(ckpt, expert_range=expert_range(rank, world, ckpt.config.num_experts), group=group)
        self.sequence_prefill = True

    def close(self) -> None:
        self.graph = None
        self.step.close()

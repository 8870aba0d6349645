"""Host-side logic of the expert-parallel path on CPU (gloo, world size 2): the expert
ranges tile the bank, and the ranks' fp32 partial sums over their own experts, all-reduced,
reproduce the unsharded MoE block of the oracle."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import decode_oracle as O
from quickdraw_b200 import synthetic
from quickdraw_b200.expert_parallel import expert_range


def test_expert_ranges_tile_the_bank():
    for world in (1, 2, 4, 8):
        spans = [expert_range(r, world, 256) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 256
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cfg = synthetic.model_config(num_layers=1, vocab_size=64, hidden=256, experts=8, topk=3, intermediate=64)
    src = synthetic.Source(7, "cpu")
    lo, hi = expert_range(rank, world, cfg.num_experts)
    full = synthetic.make_moe(cfg, src)                      # same seed on every rank
    mine = synthetic.make_moe(cfg, src, expert_range=(lo, hi))
    assert torch.equal(mine.experts_gate.weight, full.experts_gate.weight[lo:hi])
    x = src.normal("x", cfg.hidden_size)
    with torch.inference_mode():
        partial = O.moe_block(full, x, config=cfg, experts=range(lo, hi), partial=True)
        dist.all_reduce(partial, op=dist.ReduceOp.SUM)
        combined = O.combine_shared(full, x, partial)
        whole = O.moe_block(full, x, config=cfg)
    import json
    with open(os.path.join(outdir, f"rank{rank}.json"), "w") as f:
        json.dump([O.rel_l2(combined, whole), bool(torch.equal(combined, whole))], f)
    dist.barrier()
    dist.destroy_process_group()


def test_partial_sums_all_reduce_to_the_whole_block():
    world = 2
    import json
    import tempfile
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_rank_main, args=(world, _free_port(), outdir), nprocs=world, join=True)
        for rank in range(world):
            err, exact = json.load(open(os.path.join(outdir, f"rank{rank}.json")))
            assert exact or err < 4e-3, (rank, err)

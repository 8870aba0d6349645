"""Host-side logic of the expert-parallel path on CPU (gloo, world size 2).

  * the expert and vocabulary ranges tile the bank and the LM head;
  * the exchange the persistent kernel performs, restated with gloo: every rank fills the
    rows of the per-layer contribution table that belong to experts it owns, the tables meet
    (each row has exactly one writer, so a sum over ranks moves them unchanged), and every rank
    adds the rows in ascending expert id: bit-identical to the oracle's unsharded MoE block;
  * the vocabulary-sharded greedy choice: best (logit, index) per rank, highest value and
    lowest index win: the oracle's argmax;
  * failure detection: a rank that exits between steps (no goodbye) or says goodbye is
    reported by the survivor's watchdog before its next launch, instead of a stall.
"""

import json
import os
import socket
import tempfile
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import decode_oracle as O
from quickdraw_b200 import synthetic
from quickdraw_b200.expert_parallel import PeerLost, RankWatchdog, expert_range, vocab_range


def test_expert_ranges_tile_the_bank():
    for world in (1, 2, 4, 8):
        spans = [expert_range(r, world, 256) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 256
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        rows = [vocab_range(r, world, 151936) for r in range(world)]
        assert rows[0][0] == 0 and rows[-1][1] == 151936
        assert all(a[1] == b[0] for a, b in zip(rows, rows[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _exchange_rank(rank, world, port, outdir):
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
        ids, weights = O.route(O.bf16_gemv(x, full.router), cfg.num_experts_per_tok)
        order = sorted(zip(ids.tolist(), weights))                       # ascending expert id, as the kernel's table
        table = torch.zeros(len(order), cfg.hidden_size, dtype=torch.float32)
        for slot, (expert, weight) in enumerate(order):
            if lo <= expert < hi:                                         # this rank's rows, from its own slice
                local = expert - lo
                hidden = O.swiglu(O.nvfp4_gemv(x, O.expert_view(mine.experts_gate, local)),
                                  O.nvfp4_gemv(x, O.expert_view(mine.experts_up, local)))
                table[slot] = O.nvfp4_gemv(hidden, O.expert_view(mine.experts_down, local), routing_weight=weight).float()
        dist.all_reduce(table, op=dist.ReduceOp.SUM)                      # one writer per row: rows arrive unchanged
        routed = torch.zeros(cfg.hidden_size, dtype=torch.float32)
        for row in table:
            routed = routed + row
        combined = O.combine_shared(full, x, routed)
        whole = O.moe_block(full, x, config=cfg)
        # the vocabulary-sharded greedy choice
        logits = src.normal("logits", cfg.vocab_size).float()
        logits[[5, 40]] = logits.max() + 1                                # a tie across the shards: lowest index wins
        vlo, vhi = vocab_range(rank, world, cfg.vocab_size)
        best = torch.tensor([float(logits[vlo:vhi].max()), float(vlo + int(logits[vlo:vhi].argmax()))], dtype=torch.float64)
        pairs = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(pairs, best)
        choice = min(pairs, key=lambda p: (-float(p[0]), float(p[1])))
    with open(os.path.join(outdir, f"rank{rank}.json"), "w") as f:
        json.dump({"exact": bool(torch.equal(combined, whole)), "token": int(choice[1]), "want": int(logits.argmax())}, f)
    dist.barrier()
    dist.destroy_process_group()


def test_contribution_rows_exchanged_and_added_in_expert_order_are_the_whole_block():
    world = 2
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_exchange_rank, args=(world, _free_port(), outdir), nprocs=world, join=True)
        for rank in range(world):
            out = json.load(open(os.path.join(outdir, f"rank{rank}.json")))
            assert out["exact"], f"rank {rank}: the exchanged sum differs from the unsharded block"
            assert out["token"] == out["want"] == 5


def _watchdog_rank(rank, world, port, outdir, goodbye):
    """Ranks take `steps` of a stub step (no GPU); rank 1 goes away after its third step."""
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    dog = RankWatchdog(store, rank, world, interval=0.02, timeout=0.5)
    store.add("qd/test/ready", 1)
    while int(store.add("qd/test/ready", 0)) < world:
        time.sleep(0.01)
    report = {"steps": 0, "lost": None}
    started = time.monotonic()
    try:
        for step in range(400):
            dog.check()                 # what ExpertParallelStep does before every launch
            time.sleep(0.01)            # the launch
            report["steps"] += 1
            if rank == 1 and step == 2:
                if goodbye:
                    dog.leave()
                    break
                os._exit(0)             # gone without a word, between steps
    except PeerLost as lost:
        report["lost"] = str(lost)
    report["seconds"] = time.monotonic() - started
    with open(os.path.join(outdir, f"rank{rank}.json"), "w") as f:
        json.dump(report, f)
    if rank == 0:
        time.sleep(0.2)                 # the store lives in this process: let the peer finish reading
    dog.stop()


@pytest.mark.parametrize("goodbye", [False, True])
def test_a_rank_that_goes_away_between_steps_is_reported_not_waited_for(goodbye):
    world = 2
    with tempfile.TemporaryDirectory() as outdir:
        context = mp.spawn(_watchdog_rank, args=(world, _free_port(), outdir, goodbye), nprocs=world, join=False)
        deadline = time.monotonic() + 60
        while not context.join(timeout=1):
            assert time.monotonic() < deadline, "the surviving rank stalled"
        survivor = json.load(open(os.path.join(outdir, "rank0.json")))
    assert survivor["lost"] is not None, "the survivor took every step although its peer was gone"
    assert "rank 1" in survivor["lost"]
    assert ("left the group" in survivor["lost"]) == goodbye
    assert 3 <= survivor["steps"] < 400 and survivor["seconds"] < 10


def test_the_store_going_away_is_a_lost_peer():
    class DeadStore:
        def __init__(self):
            self.calls = 0

        def add(self, key, value):
            self.calls += 1
            if self.calls > 1:
                raise ConnectionError("connection reset")
            return 1
    dog = RankWatchdog(DeadStore(), 1, 2, interval=10.0)
    with pytest.raises(PeerLost, match="store stopped answering"):
        dog.check()
    dog.stop()

"""Expert parallelism on the GPUs of one box against the single-GPU engine (one process per
GPU; the ranks are child processes with a time limit: a rank that does not finish is killed by
its own process id and the test fails with the ranks' output).  Group sizes above the box's
GPU count are skipped; host-side coverage is in test_expert_parallel_cpu.py.

The last test makes a bounded wait of the persistent kernel run out on ONE GPU without
faulting anything: rank 0 of a two-rank group whose second exchange area is an ordinary
local buffer that nobody ever writes."""

import json
import os
import socket
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
RANK_TIMEOUT_S = 180

RANK_PROGRAM = r"""
import json, os, sys
rank, world, port, outdir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
prompt, steps = json.loads(sys.argv[5]), int(sys.argv[6])
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, NCCL_NVLS_ENABLE="0",
                  TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
import torch
import torch.distributed as dist
from quickdraw_b200 import synthetic
from quickdraw_b200.expert_parallel import ExpertParallelEngine
torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
cfg = synthetic.model_config(num_layers=4, vocab_size=2048, experts=16, topk=8)
engine = ExpertParallelEngine(cfg, seed=11, max_context=64, device=f"cuda:{rank}")
engine.state.kv_k.zero_()
engine.state.kv_v.zero_()
tokens = engine.generate(prompt, steps)            # prompt through the chunked prefill, then the captured graph
print("rank", rank, "generated", flush=True)
# the full logits of the last prompt token, gathered from the ranks' vocabulary shards
engine.reset()
engine.state.kv_k.zero_()
engine.state.kv_v.zero_()
with torch.inference_mode():
    for position, token in enumerate(prompt):
        logits = engine.step(engine.ckpt, torch.tensor(token, device=f"cuda:{rank}"), position, engine.state)
# three sequences stepped together (the batched decode), experts and LM head split the same way
from quickdraw_b200.batch import BatchDecode, BatchState
from quickdraw_b200.expert_parallel import expert_range, vocab_range
batch = BatchDecode(engine.ckpt, expert_range=expert_range(rank, world, cfg.num_experts),
                    vocab_range=vocab_range(rank, world, cfg.vocab_size))
sequences = BatchState(cfg, 3, 64, f"cuda:{rank}")
fed = torch.tensor([5, 77, 1900], device=f"cuda:{rank}")
for _ in range(3):
    fed, batch_logits = batch.step(fed, sequences)
torch.cuda.synchronize()
with open(os.path.join(outdir, f"rank{rank}.json"), "w") as f:
    json.dump({"tokens": tokens, "status": engine.fused.status(), "launches": engine.launches_per_step,
               "logits": logits.float().cpu().tolist(), "batch_logits": batch_logits.float().cpu().tolist(),
               "batch_status": batch.check()}, f)
# ordered teardown: every rank is between steps; the exchange areas go before the group does
engine.close()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "left", flush=True)
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_generation_matches_single_gpu(world):
    """Tokens and the gathered logits of the expert-parallel engine are the single GPU's, bit
    for bit: every rank adds the same eight bf16 contribution rows in the same order, in the
    chunked prefill of the prompt (one all-reduce of the contribution rows per layer) as in the
    one-launch decode step (rows stored into every rank's exchange area)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from quickdraw_b200 import synthetic
    from quickdraw_b200.engine import Engine
    prompt, steps = [5, 1900, 77, 1033, 8, 640, 12, 2001, 333, 90, 1500, 41, 7, 7, 1999, 250, 3], 24
    cfg = synthetic.model_config(num_layers=4, vocab_size=2048, experts=16, topk=8)
    single = Engine(synthetic.make_checkpoint(cfg, seed=11, device="cuda:0"), max_context=64, device="cuda:0")
    single.state.kv_k.zero_()
    single.state.kv_v.zero_()
    want = single.generate(prompt, steps)
    single.reset()
    single.state.kv_k.zero_()
    single.state.kv_v.zero_()
    with torch.inference_mode():
        for position, token in enumerate(prompt):
            want_logits = single.step(single.ckpt, torch.tensor(token, device="cuda:0"), position, single.state)
    want_logits = want_logits.float().cpu().tolist()
    from quickdraw_b200.batch import BatchDecode, BatchState
    batch = BatchDecode(single.ckpt)
    sequences = BatchState(cfg, 3, 64, "cuda:0")
    fed = torch.tensor([5, 77, 1900], device="cuda:0")
    for _ in range(3):
        fed, batch_logits = batch.step(fed, sequences)
    want_batch = batch_logits.float().cpu().tolist()
    del single, batch, sequences
    torch.cuda.empty_cache()
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    with tempfile.TemporaryDirectory() as outdir:
        port = str(_free_port())
        logs = [open(os.path.join(outdir, f"rank{r}.log"), "w") for r in range(world)]
        ranks = [subprocess.Popen([sys.executable, "-c", RANK_PROGRAM, str(r), str(world), port, outdir,
                                   json.dumps(prompt), str(steps)], env=env, stdout=logs[r],
                                  stderr=subprocess.STDOUT, cwd=str(ROOT)) for r in range(world)]
        failed = []
        deadline = time.monotonic() + RANK_TIMEOUT_S
        for r, proc in enumerate(ranks):
            try:
                if proc.wait(timeout=max(1.0, deadline - time.monotonic())) != 0:
                    failed.append(f"rank {r} exited with {proc.returncode}")
            except subprocess.TimeoutExpired:
                failed.append(f"rank {r} did not finish within {RANK_TIMEOUT_S} s")
        for proc in ranks:
            if proc.poll() is None:
                proc.kill()          # this process id only
                proc.wait()
        for f in logs:
            f.close()
        text = "\n".join(f"--- rank {r}\n" + open(os.path.join(outdir, f"rank{r}.log")).read()[-2000:] for r in range(world))
        assert not failed, "; ".join(failed) + "\n" + text
        out = [json.load(open(os.path.join(outdir, f"rank{r}.json"))) for r in range(world)]
    for r in range(world):
        assert out[r]["status"] == 0, f"rank {r}: device status {out[r]['status']}"
        assert out[r]["launches"] == 1, "the expert-parallel step is one launch per token"
        assert out[r]["tokens"] == want, f"rank {r}: {out[r]['tokens']} vs single GPU {want}"
        assert out[r]["logits"] == want_logits, f"rank {r}: gathered logits differ from the single GPU's"
        assert out[r]["batch_status"] == 0
        assert out[r]["batch_logits"] == want_batch, f"rank {r}: batched-decode logits differ from the single GPU's"


def test_a_wait_that_nothing_answers_runs_out_and_the_next_call_works(cuda_device):
    """Rank 0 of a two-rank group on one GPU; the area that stands for rank 1 is local memory
    nobody writes, so rank 1's contribution rows and best logit never arrive.  With the wait
    limit set to 20 ms the launch must come back on its own with the wait-timeout bit in the
    status word, the context must stay usable, and an ordinary step afterwards must be exact."""
    from quickdraw_b200 import _lib, synthetic
    from quickdraw_b200.expert_parallel import expert_range, vocab_range
    from quickdraw_b200.fused import FusedStep
    from quickdraw_b200.state import DecodeState
    cfg = synthetic.model_config(num_layers=4, vocab_size=2048, experts=16, topk=8)
    whole = synthetic.make_checkpoint(cfg, seed=11, device="cuda")
    part = synthetic.make_checkpoint(cfg, seed=11, device="cuda", expert_range=expert_range(0, 2, cfg.num_experts),
                                     vocab_range=vocab_range(0, 2, cfg.vocab_size))
    step = FusedStep(part, expert_range=expert_range(0, 2, cfg.num_experts), vocab_range=vocab_range(0, 2, cfg.vocab_size))
    areas = [torch.zeros(step.exchange_bytes(), dtype=torch.uint8, device="cuda") for _ in range(2)]
    step.set_exchange(0, 2, [a.data_ptr() for a in areas])
    state = DecodeState.allocate(cfg, 64, "cuda")
    state.kv_k.zero_()
    state.kv_v.zero_()
    token = torch.tensor(5, device="cuda")
    lib = _lib.lib()
    try:
        assert lib.qd_set_wait_limit_us(20000) == 0
        torch.cuda.synchronize()
        started = time.monotonic()
        step(part, token, 0, state)
        torch.cuda.synchronize()                   # returns: the kernel gave up by itself
        elapsed = time.monotonic() - started
    finally:
        lib.qd_set_wait_limit_us(200000)
    assert step.status() & 1, "the wait-timeout bit is not set"
    assert elapsed < 5.0, f"the launch took {elapsed:.1f} s to give up"
    # the context is intact: an ordinary single-GPU step is bit-identical to a fresh object's
    fresh = [DecodeState.allocate(cfg, 64, "cuda") for _ in range(2)]
    for s in fresh:
        s.kv_k.zero_()
        s.kv_v.zero_()
    a = FusedStep(whole)(whole, token, 0, fresh[0])
    b = FusedStep(whole, persistent=False)(whole, token, 0, fresh[1])
    torch.cuda.synchronize()
    assert torch.isfinite(a.float()).all()
    from oracle import decode_oracle as O
    assert O.rel_l2(a.cpu(), b.cpu()) < 2e-2

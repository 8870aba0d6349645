#!/usr/bin/env python
"""Batch-one greedy decode benchmark of the synthetic 36B-A3B NVFP4 hybrid MoE model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one decode token through all 48 layers and the LM head.  The model is
generated on the device from a fixed seed (no checkpoint ships with the package), the
prompt is 512 uniform random token ids.  Rank 0 prints one JSON line:

  value      decode tokens/s, device-timed (CUDA events around K graph replays, inputs
             resident in HBM), max over ranks;
  e2e        the same through ``Engine.decode_step`` with the token and position coming
             from pinned host memory and the selected token read back every step;
  roofline   the token-step kernel (one launch per token): algorithmic bytes of a token /
             CUDA-event time per launch against the measured HBM copy bandwidth;
  matvec_roofline  the NVFP4 matvec kernel alone (FP4 tensor core), 128 units of the
             single-matvec configuration ([1024, 2048]) per launch over two 151 MB matrices;
  kernels    per-kernel legs: the phases of the token step from the kernel's own timestamps
             (MoE layer = router + gate/up + down phases, DeltaNet state update, attention,
             LM head), and decode attention alone at contexts 8192 and 32768;
  cpu_baseline  the reference's PyTorch path on this host's cores on a bounded sample: one
             4-layer group and the LM head, scaled to 48 layers (extrapolated, said so).

``--impl reference`` times only that CPU path and prints the same line shape: the
reference's own ``quickdraw.models.qwen`` when a checkout is importable (``baseline/_ref``),
else the oracle port of it.
With N > 1 (torchrun) the routed experts and the LM-head rows are sharded across ranks
(expert parallel); the step stays one launch per token on every rank, the ranks exchange
their routed contributions and best logits through peer memory inside that launch.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 512
BF16 = torch.bfloat16
CONFIG1_BYTES = 1024 * 1024 + 1024 * 128 + 4 + 4096 + 2048     # weights + x + y of one matvec
# DRAM bytes (read + write) of one token step: captured with ncu on an 8-layer model of the
# same widths (a full-size capture would hold 24 GB through the replay passes) and scaled to
# the full model by the algorithmic bytes, to which it is proportional.
STEP_TRAFFIC_RATIO = 1.035       # ncu: (dram read + write) / algorithmic bytes of one persistent launch


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a cuBLAS GEMM timed alone on this pool (burst figure)."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        if "bf16_tflops" in data:
            return float(data["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def bytes_per_token(cfg, position: int) -> int:
    """Algorithmic HBM bytes of one decode token: every weight the token touches once
    (selected experts only), recurrent/conv state read and written, KV history read."""
    h, inter = cfg.hidden_size, cfg.moe_intermediate_size
    fp4 = lambda out, inp: out * inp // 2 + out * inp // 16 + 4
    moe = (cfg.num_experts * h * 2 + h * 2
           + (cfg.num_experts_per_tok + 1) * (2 * fp4(inter, h) + fp4(h, inter)))
    kw = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    vw = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    gdn_w = fp4(2 * kw + vw, h) + fp4(vw, h) + fp4(h, vw) + 2 * cfg.linear_num_value_heads * h * 2 \
        + (2 * kw + vw) * cfg.linear_conv_kernel_dim * 2
    rec = cfg.linear_num_value_heads * cfg.linear_key_head_dim * cfg.linear_value_head_dim * 4
    conv = (2 * kw + vw) * (cfg.linear_conv_kernel_dim - 1) * 2
    gdn = gdn_w + 2 * rec + 2 * conv
    qw, kvw = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    attn = fp4(2 * qw, h) + 2 * fp4(kvw, h) + fp4(h, qw) + 2 * kvw * 2 * (position + 1)
    n_full = cfg.layer_types.count("full_attention")
    n_lin = cfg.num_hidden_layers - n_full
    norms = (2 * cfg.num_hidden_layers + 1) * h * 4
    return (cfg.num_hidden_layers * moe + n_lin * gdn + n_full * attn
            + cfg.vocab_size * h * 2 + norms + h * 2)


def bytes_per_batch_step(cfg, batch: int, context: int) -> int:
    """Algorithmic HBM bytes of one batched decode step: every weight once (of the routed experts the
    expected number of distinct ones that `batch` tokens with top-k routing touch), every
    sequence's recurrent / convolution state read and written and its KV history read."""
    h, inter = cfg.hidden_size, cfg.moe_intermediate_size
    fp4 = lambda out, inp: out * inp // 2 + out * inp // 16 + 4
    expert = 2 * fp4(inter, h) + fp4(h, inter)
    distinct = cfg.num_experts * (1.0 - (1.0 - cfg.num_experts_per_tok / cfg.num_experts) ** batch)
    moe = cfg.num_experts * h * 2 + h * 2 + (distinct + 1) * expert
    kw = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    vw = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    gdn_w = fp4(2 * kw + vw, h) + fp4(vw, h) + fp4(h, vw) + 2 * cfg.linear_num_value_heads * h * 2 \
        + (2 * kw + vw) * cfg.linear_conv_kernel_dim * 2
    rec = cfg.linear_num_value_heads * cfg.linear_key_head_dim * cfg.linear_value_head_dim * 4
    conv = (2 * kw + vw) * (cfg.linear_conv_kernel_dim - 1) * 2
    qw, kvw = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    attn_w = fp4(2 * qw, h) + 2 * fp4(kvw, h) + fp4(h, qw)
    kv = 2 * kvw * 2 * (context + 1)
    n_full = cfg.layer_types.count("full_attention")
    n_lin = cfg.num_hidden_layers - n_full
    return int(cfg.num_hidden_layers * moe + n_lin * (gdn_w + batch * 2 * (rec + conv)) + n_full * (attn_w + batch * kv)
               + cfg.vocab_size * h * 2)


class ClockSampler:
    """nvidia-smi SM clock / throttle-reason samples while a timed region runs.  The process is
    started ahead of the region (it needs some hundred milliseconds to come up, longer with eight
    of them on one host); every sample carries its arrival time and `summary()` keeps those of the
    marked window.  A region too short for two samples is followed by untimed replays of the same
    step until there are three (`extended` then counts the samples taken after the region)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.begin = self.end = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark_begin(self):
        self.begin = time.perf_counter()

    def mark_end(self):
        self.end = time.perf_counter()

    def in_window(self, extended=False):
        if self.begin is None:
            return [r for _, r in self.rows]
        stop = float("inf") if extended or self.end is None else self.end + 0.05
        return [r for at, r in self.rows if self.begin <= at <= stop]

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        timed = self.in_window()
        rows = timed if len(timed) >= 2 else self.in_window(extended=True)
        sm = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in rows if len(r) >= 6
                          for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        mx = max((int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()), default=None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(sm), "extended": len(rows) - len(timed)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------ CPU baseline timing
def reference_module():
    """The reference's own step function when the installed copy under baseline/_ref is importable, else None."""
    for root in (ROOT / "baseline" / "_ref",):
        if (root / "quickdraw" / "models" / "qwen.py").exists():
            sys.path.insert(0, str(root))
            try:
                from quickdraw.models import qwen      # noqa: PLC0415
                return qwen
            except Exception:                           # missing dependency of the checkout
                sys.path.remove(str(root))
    return None


def cpu_sample(cfg, threads: int):
    """Seconds per token of the CPU path, from one 4-layer group and the LM head.  Returns
    (seconds per token, seconds actually timed, kind)."""
    from oracle import decode_oracle as O
    from quickdraw_b200 import synthetic
    from quickdraw_b200.state import DecodeState
    torch.set_num_threads(threads)
    group = cfg.full_attention_interval
    sub = synthetic.model_config(num_layers=group, vocab_size=cfg.vocab_size, interval=group)
    ckpt = synthetic.make_checkpoint(sub, seed=0, device="cpu")
    state = DecodeState.allocate(sub, 1024, "cpu")
    state.kv_k.normal_()
    state.kv_v.normal_()
    ref = reference_module()
    kind = "reference" if ref is not None else "port"
    step_fn = O.forward_step
    if ref is not None:
        # the reference's own functions; its blocks take the projection as an argument, and this
        # model's mixer projections are NVFP4 (the LM head, bf16 here, is timed below)
        import functools
        step_fn = functools.partial(
            ref.forward_step,
            attention=functools.partial(ref.full_attention_block, project_fp8=ref.nvfp4_gemv),
            delta_net=functools.partial(ref.gated_delta_net_block, project_fp8=ref.nvfp4_gemv))
    with torch.inference_mode():
        x = torch.nn.functional.embedding(torch.tensor(7), ckpt.embed_tokens)

        def layers_once():
            return step_fn(ckpt, torch.tensor(7), PROMPT_LEN + 128, state, logits=False)

        def head_once():
            normed, _ = O.add_norm(x, torch.zeros_like(x), 1 + ckpt.final_norm.float(), sub.rms_norm_eps)
            return O.project(normed, ckpt.lm_head)
        t_all = time.perf_counter()
        try:
            layers_once()
        except Exception:                                # the checkout does not take these containers
            kind, step_fn = "port", O.forward_step
            layers_once()
        times = []
        for _ in range(2):
            t = time.perf_counter()
            layers_once()
            times.append(time.perf_counter() - t)
        t = time.perf_counter()
        head_once()
        head = time.perf_counter() - t
        timed = time.perf_counter() - t_all
    per_group = sorted(times)[0]
    return per_group * (cfg.num_hidden_layers / group) + head, timed, kind


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    from quickdraw_b200 import synthetic
    cfg = synthetic.model_config()
    threads = len(os.sched_getaffinity(0))
    t0 = time.perf_counter()
    samples, timed, kind = [], 0.0, "port"
    for _ in range(max(1, min(args.steps, 3))):
        per_token, seconds, kind = cpu_sample(cfg, threads)
        samples.append(per_token)
        timed += seconds
        if time.perf_counter() - t0 > 150:
            break
    per_token = sorted(samples)[len(samples) // 2]
    value = 1.0 / per_token
    sample = ("one 4-layer group (3 DeltaNet + 1 attention + 4 MoE blocks) and the bf16 LM head at "
              "position 640, group time x12 + head time")
    line = {
        "impl": "reference", "metric": "batch-1 decode tok/s (36B-A3B NVFP4 MoE)", "value": value,
        "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_token * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 activations, NVFP4 (E2M1 + E4M3 block scale) weights, fp32 accumulate",
        "data": "synthetic", "config": workload_config(cfg, world),
        # a token is extrapolated from the sample: value = 1 / (group time x 12 + head time)
        "extrapolated": True, "seconds_timed": timed,
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample,
                         "extrapolated": True},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, world, prompt=PROMPT_LEN):
    full = cfg.layer_types.count("full_attention")
    name = "config 4: " if (cfg.num_hidden_layers, cfg.vocab_size) == (48, 151936) else "REDUCED (profiling only): "
    return {"workload": f"{name}synthetic 36B-A3B hybrid ({cfg.num_hidden_layers - full} gated-DeltaNet + {full} GQA "
                        f"layers, {cfg.num_experts}-expert top-{cfg.num_experts_per_tok} NVFP4 MoE, vocab "
                        f"{cfg.vocab_size}), 512-token prompt then greedy decode, batch 1",
            "layers": cfg.num_hidden_layers, "prompt": prompt,
            "parallelism": "single GPU" if world == 1 else f"expert parallel x{world} (experts sharded, rest replicated)",
            "l2": "every token streams ~2.5 GB of weights, far beyond the 126 MB L2; no flush needed"}


# ----------------------------------------------------------------------- GPU benchmark
def matvec_roofline(device, rows=131072, width=2048, mats=2, reps=10, kernel=0):
    """The NVFP4 streaming matvec kernel alone: `mats` distinct [rows, width] matrices
    (2 x 151 MB by default, more than L2), one launch each, alternating.  A launch does
    rows / 1024 units of the single-matvec configuration ([1024, 2048])."""
    from quickdraw_b200 import synthetic
    from quickdraw_b200._lib import call, ptr, stream_of
    src = synthetic.Source(1, device)
    bank = src.nvfp4("roofline.bank", rows, width, mats)
    x = src.normal("roofline.x", width)
    y = torch.empty(mats, rows, dtype=BF16, device=device)

    def launch(i):
        call("qd_nvfp4_gemv", ptr(x), ptr(bank.weight[i]), ptr(bank.weight_scale[i]), ptr(bank.weight_scale_2),
             None, ptr(y[i]), rows, width, 16, kernel, stream_of(x))
    for i in range(3 * mats):
        launch(i % mats)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps * mats):
        launch(i % mats)
    e1.record()
    torch.cuda.synchronize(device)
    per_launch_s = e0.elapsed_time(e1) * 1e-3 / (reps * mats)
    units = rows // 1024
    return units * CONFIG1_BYTES / per_launch_s / 1e9, per_launch_s, units


def prefill_gemm_roofline(device, tokens=8192, rows=8192, width=2048, reps=10):
    """The prefill projection on the tensor cores (tcgen05): an 8192-token chunk through the
    largest projection shape of the model ([8192, 2048], the DeltaNet qkv / attention q
    projection), NVFP4 weights expanded to bf16 on the fly."""
    from quickdraw_b200 import kernels, synthetic
    src = synthetic.Source(2, device)
    proj = src.nvfp4("prefill.w", rows, width)
    x = src.normal("prefill.x", tokens, width)
    for _ in range(3):
        kernels.matmul(x, proj)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        kernels.matmul(x, proj)
    e1.record()
    torch.cuda.synchronize(device)
    assert kernels.matmul_status(device) == 0
    per_launch_s = e0.elapsed_time(e1) * 1e-3 / reps
    return 2.0 * tokens * rows * width / per_launch_s / 1e12, per_launch_s


def w4a4_gemm_roofline(device, tokens=8192, rows=8192, width=2048, reps=10):
    """The same projection with BOTH operands NVFP4 on the block-scaled FP4 tensor core
    (tcgen05 kind::mxf4nvf4): the activation chunk quantised once (timed apart), weights and
    activations multiplied without any expansion.  Returns TFLOP/s and seconds of the product,
    and seconds of the quantiser."""
    from quickdraw_b200 import kernels, synthetic
    src = synthetic.Source(2, device)
    proj = src.nvfp4("prefill.w", rows, width)
    x = src.normal("prefill.x", tokens, width)
    xq = kernels.quantize_act(x)
    out = {}
    for name, fn in (("product", lambda: kernels.matmul_w4a4(xq, proj)), ("quantiser", lambda: kernels.quantize_act(x))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        out[name] = e0.elapsed_time(e1) * 1e-3 / reps
    assert kernels.matmul_status(device) == 0
    return 2.0 * tokens * rows * width / out["product"] / 1e12, out["product"], out["quantiser"]


def attention_leg(cfg, device, context, peak, reps=24):
    """Decode attention alone (the split-context kernel of the operator table) at one context
    length: 16 query / 2 KV heads of 256, bf16 cache ~ N(0, 1); the caches rotate over more than
    L2 holds.  Algorithmic bytes per launch: the K and V rows of the history, 2048 B per position."""
    from quickdraw_b200._lib import call, lib, ptr, stream_of
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_cache = 2 * context * hkv * d * 2
    n = max(2, -(-(300 << 20) // per_cache))
    gen = torch.Generator(device=device).manual_seed(7)
    k = torch.randn(n, context, hkv, d, generator=gen, device=device).to(BF16)
    v = torch.randn(n, context, hkv, d, generator=gen, device=device).to(BF16)
    qg = torch.randn(hq, 2 * d, generator=gen, device=device).to(BF16)
    kn = torch.randn(hkv, d, generator=gen, device=device).to(BF16)
    vn = torch.randn(hkv, d, generator=gen, device=device).to(BF16)
    norm = torch.zeros(d, dtype=BF16, device=device)
    out = torch.empty(hq * d, dtype=BF16, device=device)
    splits = 32
    scratch = torch.empty(lib().qd_attn_scratch_floats(hq, hkv, d, splits), dtype=torch.float32, device=device)
    counters = torch.zeros(hkv, dtype=torch.int32, device=device)

    def launch(i):
        call("qd_attn_decode", ptr(qg), ptr(kn), ptr(vn), ptr(norm), ptr(norm), ptr(k[i % n]), ptr(v[i % n]), ptr(out),
             ptr(scratch), ptr(counters), None, context - 1, context, hq, hkv, d, int(d * cfg.partial_rotary_factor),
             float(cfg.rope_theta), float(cfg.rms_norm_eps), splits, 0, stream_of(out))
    for i in range(n):
        launch(i)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        launch(i)
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / reps
    nbytes = 2 * context * hkv * d * 2
    return {"kernel": "attn_decode_kernel (split-context decode attention alone)", "context": context, "launch_us": us,
            "bytes_per_launch": nbytes, "achieved": nbytes / us / 1e3, "peak": peak, "unit": "GB/s",
            "frac": nbytes / us / 1e3 / peak, "caches_rotated": n}


def batch_attention_leg(cfg, device, batch, context, peak, reps=12):
    """The batched decode attention alone (tensor-core form, `qd_batch_attention`): `batch` sequences
    with `context` cached positions each, caches ~ N(0, 1), 2 x 537 MB of them alternating (beyond L2)."""
    from quickdraw_b200._lib import call, lib, ptr, stream_of
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    capacity = context + 1
    gen = torch.Generator(device=device).manual_seed(9)
    k = torch.randn(2, batch, capacity, hkv, d, generator=gen, device=device).to(BF16)
    v = torch.randn(2, batch, capacity, hkv, d, generator=gen, device=device).to(BF16)
    qg = torch.randn(batch, hq, 2 * d, generator=gen, device=device).to(BF16)
    kn = torch.randn(batch, hkv, d, generator=gen, device=device).to(BF16)
    vn = torch.randn(batch, hkv, d, generator=gen, device=device).to(BF16)
    norm = torch.zeros(d, dtype=BF16, device=device)
    out, q_scratch = (torch.empty(batch, hq * d, dtype=BF16, device=device) for _ in range(2))
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    pairs = batch * hkv
    splits = min(range(1, 17), key=lambda s: -(-pairs * s // sms) * (-(-context // s) + 64))
    scratch = torch.empty(batch * lib().qd_attn_scratch_floats(hq, hkv, d, 16), dtype=torch.float32, device=device)
    counters = torch.zeros(batch * hkv, dtype=torch.int32, device=device)
    positions = torch.full((batch,), context, dtype=torch.int32, device=device)

    def launch(i):
        call("qd_batch_attention", ptr(qg), ptr(kn), ptr(vn), ptr(norm), ptr(norm), ptr(k[i % 2]), ptr(v[i % 2]),
             k.stride(1), ptr(q_scratch), ptr(out), ptr(scratch), ptr(counters), ptr(positions), batch, capacity, hq, hkv, d,
             int(d * cfg.partial_rotary_factor), float(cfg.rope_theta), float(cfg.rms_norm_eps), splits, stream_of(out))
    for i in range(3):
        launch(i)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        launch(i)
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / reps
    nbytes = batch * 2 * (context + 1) * hkv * d * 2
    return {"kernel": "seq_attn_prepare_kernel + batch_attn_mma_kernel (mma.sync, rows straight from the cache)", "batch": batch,
            "context": context, "splits": splits, "launch_us": us, "bytes_per_launch": nbytes, "achieved": nbytes / us / 1e3,
            "peak": peak, "unit": "GB/s", "frac": nbytes / us / 1e3 / peak}


def kernel_legs(engine, ckpt, cfg, device, peak):
    """Per-kernel legs: the phases of one token step from the persistent kernel's own timestamps
    (time on the critical path per phase kind; algorithmic bytes / that time), and decode
    attention alone at the baseline's contexts."""
    from quickdraw_b200.trace import phase_summary, traced_step
    position = engine.state.position
    marks = traced_step(engine.fused, ckpt, engine.pending_token, position, engine.state)
    phases = phase_summary(cfg, marks, position)

    def leg(kinds, what):
        us = sum(phases[k]["us"] for k in kinds if k in phases)
        nbytes = sum(phases[k]["bytes"] for k in kinds if k in phases)
        return {"what": what, "us": us, "bytes": nbytes, "achieved": nbytes / us / 1e3 if us else None, "peak": peak,
                "unit": "GB/s", "frac": nbytes / us / 1e3 / peak if us else None}
    def attention_phase(context):
        """The attention phases of the token-step kernel (the product path) with `context` cached
        positions: a traced step at position context - 1 on a state of that capacity whose caches
        hold N(0, 1) values; mean over the model's attention layers."""
        from quickdraw_b200.state import DecodeState
        state = DecodeState.allocate(cfg, context, device)
        state.kv_k.normal_()
        state.kv_v.normal_()
        for _ in range(2):
            engine.fused(ckpt, engine.pending_token, context - 1, state, logits=False)
        long_marks = traced_step(engine.fused, ckpt, engine.pending_token, context - 1, state)
        ph = phase_summary(cfg, long_marks, context - 1)
        us, nbytes = ph["Ma"]["us"] + ph["Na"]["us"], ph["Ma"]["bytes"]
        return {"what": "split-context attention + merge phases of the token-step kernel, %d cached positions" % context,
                "us": us, "bytes": nbytes, "achieved": nbytes / us / 1e3, "peak": peak, "unit": "GB/s", "frac": nbytes / us / 1e3 / peak}
    return {
        "source": "timestamps inside the token-step kernel, one traced step at position %d" % position,
        "attention_phase_8192": attention_phase(8192),
        "attention_phase_32768": attention_phase(32768),
        "moe_layer": leg(["C", "D", "E"], "router + gate/up + down/combine phases of one layer (256 experts, top-8 + shared)"),
        "deltanet_step": leg(["M"], "gated-DeltaNet recurrence of one layer: fp32 state [32,128,128] read + written"),
        "deltanet_in_projections": leg(["A"], "qkv + z + a/b projections with the short convolution"),
        "out_projection": leg(["B"], "gated norm + out projection (4096 inputs)"),
        "attention_layer_core": leg(["Ma", "Na"], "split-context attention + merge of one layer at this position"),
        "lm_head": leg(["H"], "final norm + bf16 LM head + greedy argmax"),
        # the operator-table kernel (composed path, cross-check), not on the product path
        "attention_batch_32x8192": batch_attention_leg(cfg, device, 32, 8192, peak),
        "attention_operator_8192": attention_leg(cfg, device, 8192, peak),
        "attention_operator_32768": attention_leg(cfg, device, 32768, peak),
    }


def batch_decode_leg(ckpt, cfg, device, batch=32, context=8192, steps=8, warmup=2, slices=None, group=None):
    """Small-batch decode with per-sequence state: `batch` sequences that each hold `context`
    tokens (caches filled with N(0,1) values, as the attention configuration of the baseline
    does), one token per sequence per step; device-timed."""
    from quickdraw_b200.batch import BatchDecode, BatchState
    decoder = BatchDecode(ckpt, **(slices or {}), group=group)
    state = BatchState(cfg, batch, context + max(warmup, 3) + steps, device)
    state.kv_k.normal_()
    state.kv_v.normal_()
    state.positions.fill_(context)
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, cfg.vocab_size, (batch,), generator=gen).to(device)
    for _ in range(max(warmup, 3)):      # eager, capture, first replay
        tokens, _ = decoder.graph_step(tokens, state)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        tokens, _ = decoder.graph_step(tokens, state)
    e1.record()
    torch.cuda.synchronize(device)
    assert decoder.check() == 0
    ms = e0.elapsed_time(e1) / steps
    if slices:      # every rank runs the same sequences: the slowest rank's time counts
        worst = torch.tensor([ms], device=device)
        torch.distributed.all_reduce(worst, op=torch.distributed.ReduceOp.MAX, group=group)
        ms = float(worst.item())
    step_bytes = bytes_per_batch_step(cfg, batch, context)
    peak, _ = measured_peaks()
    return {"batch": batch, "context": context, "steps": steps, "ms_per_step": ms, "tok_s": batch / (ms * 1e-3),
            "bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms * 1e-3) / 1e9,
            "frac_of_measured_hbm": (step_bytes / (ms * 1e-3) / 1e9 / peak) if not slices else None,
            "state_bytes": state.memory_bytes(), "path": "one CUDA graph per step: tensor-core products with %d rows + batched state kernels" % batch
            + (", routed experts and LM head split over the ranks" if slices else "")}


def run_gpu(args):
    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    from quickdraw_b200 import synthetic
    cfg = synthetic.model_config(num_layers=args.layers, vocab_size=args.vocab)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
        from quickdraw_b200.expert_parallel import ExpertParallelEngine
        engine = ExpertParallelEngine(cfg, seed=0, max_context=args.context, device=device)
    else:
        from quickdraw_b200.engine import Engine
        ckpt = synthetic.make_checkpoint(cfg, seed=0, device=device)
        engine = Engine(ckpt, max_context=args.context, device=str(device))
    gen = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=gen).tolist()
    torch.cuda.synchronize(device)
    # the prompt twice: the first request of a process also pays for the lazy loading of every
    # kernel it touches; the second is the steady state that `prefill.ms` reports
    t_prefill = time.perf_counter()
    engine.prefill(prompt)
    torch.cuda.synchronize(device)
    first_prefill_s = time.perf_counter() - t_prefill
    engine.reset()
    if world > 1:
        torch.distributed.barrier()
    t_prefill = time.perf_counter()
    logits = engine.prefill(prompt)
    engine.pending_token = torch.argmax(logits)
    torch.cuda.synchronize(device)
    prefill_s = time.perf_counter() - t_prefill

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize(device)

    # ---- device-timed decode: graph replays with the token fed back on the device
    clocks = ClockSampler(local).__enter__()          # ahead of the timed region: nvidia-smi takes a while to start
    for _ in range(args.warmup):
        engine.decode_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks.mark_begin()
    e0.record()
    for _ in range(args.steps):
        engine.decode_step()
    e1.record()
    barrier()
    clocks.mark_end()
    device_ms = e0.elapsed_time(e1)
    # a region too short for two clock samples: the same step, untimed, until there are three
    more, extra = time.perf_counter(), 0
    room = args.context - int(engine.state.position) - args.steps - 4      # the e2e leg below still needs its rows
    while extra + 16 <= room:
        need = len(clocks.in_window(extended=True)) < 3 and time.perf_counter() - more < 3.0 and clocks.proc is not None
        if world > 1:       # every rank takes the same number of steps (they meet inside the step)
            flag = torch.tensor([int(need)], device=device)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
            need = bool(flag.item())
        if not need:
            break
        for _ in range(16):
            engine.decode_step()
        torch.cuda.synchronize(device)
        extra += 16
    clocks.__exit__()
    # ---- end to end through the engine's own API: the pending token comes from pinned host
    #      memory every step, the selected token is read back to the host every step
    token_host = torch.zeros((), dtype=torch.long).pin_memory()
    token_host.fill_(int(engine.pending_token.item()))
    generated = []
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        engine.pending_token = token_host.to(device, non_blocking=True)
        token = int(engine.decode_step().item())
        token_host.fill_(token)
        generated.append(token)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    times = torch.tensor([device_ms, e2e_ms], device=device)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    device_ms, e2e_ms = times.tolist()
    step_status = engine.fused.status() if getattr(engine, "fused", None) is not None else 0
    assert step_status == 0, f"the decode step reported status {step_status} (a bounded wait ran out)"
    tokens_match = None
    if world > 1:
        # every rank must have generated the same tokens (they never talk about tokens: each
        # rank derives them from the exchanged contributions and best logits)
        mine = torch.tensor(generated[:64], dtype=torch.long, device=device)
        lo, hi = mine.clone(), mine.clone()
        torch.distributed.all_reduce(lo, op=torch.distributed.ReduceOp.MIN)
        torch.distributed.all_reduce(hi, op=torch.distributed.ReduceOp.MAX)
        tokens_match = bool(torch.equal(lo, hi))
        # the batch-32 leg under expert parallelism: every rank steps the same 32 sequences
        from quickdraw_b200.expert_parallel import expert_range, vocab_range
        ep_batch_leg = batch_decode_leg(engine.ckpt, cfg, device, slices={
            "expert_range": expert_range(rank, world, cfg.num_experts),
            "vocab_range": vocab_range(rank, world, cfg.vocab_size)})
        engine.close()
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    mv_gbs, mv_launch_s, mv_units = matvec_roofline(device, rows=args.matvec_rows or 131072)
    stream_gbs, stream_launch_s, _ = matvec_roofline(device, rows=args.matvec_rows or 131072, kernel=2)
    gemm_tflops, gemm_launch_s = prefill_gemm_roofline(device)
    w4a4_tflops, w4a4_launch_s, w4a4_quant_s = w4a4_gemm_roofline(device)
    tensor_peak, tensor_peak_kind = measured_tensor_peak()
    batch_leg, legs = (ep_batch_leg if world > 1 else None), None
    if world == 1:
        legs = kernel_legs(engine, ckpt, cfg, device, peak)
        batch_leg = batch_decode_leg(ckpt, cfg, device)
    position = args.prompt + args.warmup + args.steps // 2
    token_bytes = bytes_per_token(cfg, position)
    tok_s = args.steps / (device_ms * 1e-3)
    threads = len(os.sched_getaffinity(0))
    per_token_cpu, cpu_seconds, cpu_kind = (float('nan'), 0.0, "port") if args.no_cpu_baseline else cpu_sample(cfg, threads)
    launches = getattr(engine, "launches_per_step", None) or engine.fused.launches_per_step
    line = {
        "metric": "batch-1 decode tok/s (36B-A3B NVFP4 MoE)", "value": tok_s, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_ms / args.steps, "higher_is_better": True,
        # one token stream however many GPUs: expert parallelism divides a fixed amount of work
        "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 activations, NVFP4 (E2M1 + E4M3 block scale) weights, fp32 accumulate",
        "data": "synthetic", "config": workload_config(cfg, world, args.prompt),
        "e2e": {"value": args.steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": 8},
        "tokens_match": tokens_match,
        "gpu_launches": launches * args.steps,
        # outside the timed region: the prompt (chunks of up to 2048 tokens through the tensor-core
        # products on one GPU; token by token under expert parallelism) up to the first token
        "prefill": {"tokens": args.prompt, "ms": prefill_s * 1e3, "tok_s": args.prompt / prefill_s,
                    "first_request_ms": first_prefill_s * 1e3,
                    "path": "chunked" if getattr(engine, "sequence_prefill", False) else "token loop"},
        "clocks": clocks.summary(),
        # the dominant kernel is the token step itself: one launch = one token = every weight
        # the token touches, read once (single GPU: the persistent kernel; expert parallel: the
        # per-rank share of the launches of one step)
        "roofline": {"bound": "hbm",
                     "kernel": "mega_kernel (one launch per token)" if world == 1 else "decode step, per rank",
                     "achieved": token_bytes * tok_s / 1e9 / world, "peak": peak, "unit": "GB/s",
                     "frac": token_bytes * tok_s / 1e9 / world / peak,
                     "peak_source": f"{peak_kind} copy bandwidth", "traffic": int(token_bytes * STEP_TRAFFIC_RATIO) if world == 1 else None,
                     "launch_us": device_ms / args.steps * 1e3, "bytes_per_launch": token_bytes,
                     "frac_of_8tbs": token_bytes * tok_s / 8e12 / world},
        "matvec_roofline": {"kernel": "nvfp4_umma_matvec_kernel (tcgen05 kind::mxf4nvf4, %d x [1024,2048] per launch, 2 matrices alternating)" % mv_units,
                            "achieved": mv_gbs, "peak": peak, "unit": "GB/s", "frac": mv_gbs / peak,
                            "launch_us": mv_launch_s * 1e6, "bytes_per_launch": mv_units * CONFIG1_BYTES},
        # the second matvec kernel (operands the tensor-core kernel does not cover take it: expert
        # banks, gate/up pairs, fused prologues and epilogues)
        "stream_matvec_roofline": {"kernel": "stream_kernel (mma.sync row engine), same matrices", "achieved": stream_gbs,
                                   "peak": peak, "unit": "GB/s", "frac": stream_gbs / peak, "launch_us": stream_launch_s * 1e6},
        "prefill_gemm_roofline": {"bound": "tensor", "kernel": "nvfp4_gemm_kernel (tcgen05, 8192 tokens x [8192, 2048])",
                                  "achieved": gemm_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                                  "frac": gemm_tflops / tensor_peak, "peak_source": f"{tensor_peak_kind} cuBLAS bf16",
                                  "launch_us": gemm_launch_s * 1e6},
        # both operands NVFP4 (activations quantised per chunk): no measured FP4 peak exists on this
        # pool, so the fraction is given against the measured bf16 burst (the nominal FP4 dense
        # rate is four times the bf16 one) and against the nominal 9 PFLOP/s
        "w4a4_gemm_roofline": {"bound": "tensor", "kernel": "nvfp4_gemm_w4a4_kernel (tcgen05 kind::mxf4nvf4, 8192 tokens x [8192, 2048])",
                               "achieved": w4a4_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                               "frac": w4a4_tflops / tensor_peak, "peak_source": f"{tensor_peak_kind} cuBLAS bf16",
                               "frac_of_nominal_fp4": w4a4_tflops / 9000.0, "launch_us": w4a4_launch_s * 1e6,
                               "quantiser_us": w4a4_quant_s * 1e6},
        # widening row: batch-32 decode with per-sequence KV and DeltaNet state (tok/s over all
        # sequences); not part of `value`
        "batch_decode": batch_leg,
        "kernels": legs,
        "cpu_baseline": {"value": 1.0 / per_token_cpu, "unit": "tok/s", "cores": threads, "kind": cpu_kind,
                         "sample": "one 4-layer group and the LM head at position 640, group time x12 + head time",
                         "extrapolated": True, "seconds_timed": cpu_seconds},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    ap.add_argument("--prompt", type=int, default=PROMPT_LEN, help="prompt length (512 in the headline workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU sample (profiling runs)")
    ap.add_argument("--layers", type=int, default=48, help="model depth (48 in the headline workload; fewer for profiling)")
    ap.add_argument("--vocab", type=int, default=151936, help="vocabulary (151936 in the headline workload)")
    ap.add_argument("--matvec-rows", type=int, default=0, help="rows of the matvec roofline matrices (default 131072)")
    ap.add_argument("--context", type=int, default=2048, help="KV-cache capacity of the decode engine")
    args = ap.parse_args()
    assert args.warmup >= 0 and args.steps > 0
    if args.impl == "reference":
        run_reference(args)
    else:
        with torch.inference_mode():
            run_gpu(args)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

"""Per-phase timeline of one token step of the persistent kernel.

    python -m quickdraw_b200.trace [--layers 8] [--position 600] [--show 1,3]

Runs a few steps of a synthetic model of the 36B-A3B widths, then one step with the
kernel's timestamp buffer attached (sixteen nanosecond marks per phase and block: 0 start
after the grid barrier, 1 end, 2 activation vector ready, 3 first weight tile landed,
4 / 5 first and last tile issued by the producer) and prints, per phase kind, the mean
work time (last block's end - last block's start) and the mean barrier gap (last block's
start - last block's end of the phase before).  Phase kinds: A in-projections, M mixer core
(a = attention layer), N attention split merge, B out-projection, C router, D gate/up,
E down + combine, H LM head.
"""

from __future__ import annotations

import argparse

import numpy as np
import torch

from . import synthetic
from .fused import FusedStep
from .state import DecodeState

SLOTS = 16


def phase_plan(cfg) -> list[tuple[str, int]]:
    plan = []
    for index, kind in enumerate(cfg.layer_types):
        attn = kind == "full_attention"
        for k in (["A", "M", "N", "B", "C", "D", "E"] if attn else ["A", "M", "B", "C", "D", "E"]):
            plan.append((k + ("a" if attn and k in "AMNB" else ""), index))
    plan.append(("H", len(cfg.layer_types)))
    return plan


def traced_step(step, ckpt, token, position: int, state) -> np.ndarray:
    """One step with the kernel's timestamp buffer attached: marks [phase][16][blocks], ns."""
    cfg = ckpt.config
    grid = torch.cuda.get_device_properties(step.device).multi_processor_count
    plan = phase_plan(cfg)
    step.trace = torch.zeros(len(plan) * SLOTS * grid, dtype=torch.int64, device=step.device)
    try:
        step(ckpt, token, position, state)
        torch.cuda.synchronize(step.device)
        return step.trace.cpu().numpy().reshape(len(plan), SLOTS, grid).astype(np.int64)
    finally:
        step.trace = None


def phase_summary(cfg, marks: np.ndarray, position: int) -> dict[str, dict]:
    """Per phase kind: mean time on the critical path (the last block's end minus the last
    block's end of the phase before: these add up to the whole step), algorithmic bytes and
    the bandwidth that makes."""
    plan = phase_plan(cfg)
    nbytes = phase_bytes(cfg, position)
    spans: dict[str, list[int]] = {}
    previous_end = int(marks[0, 0].min())
    for index, (kind, _) in enumerate(plan):
        end = int(marks[index, 1].max())
        spans.setdefault(kind, []).append(end - previous_end)
        previous_end = end
    out = {}
    for kind, values in spans.items():
        us = float(np.mean(values)) / 1e3
        out[kind] = {"count": len(values), "us": us, "bytes": int(nbytes.get(kind, 0)),
                     "gbs": (nbytes[kind] / us / 1e3) if nbytes.get(kind) else None}
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--position", type=int, default=600)
    ap.add_argument("--context", type=int, default=0, help="KV capacity (default: position + 64)")
    ap.add_argument("--interval", type=int, default=4, help="every interval-th layer is an attention layer")
    ap.add_argument("--show", default="", help="comma-separated layers to print phase by phase")
    ap.add_argument("--dump", default="", help="save the raw marks [phase][16][blocks] to this .npy file")
    args = ap.parse_args()
    dev = "cuda"
    cfg = synthetic.model_config(num_layers=args.layers, vocab_size=args.vocab, interval=args.interval)
    ckpt = synthetic.make_checkpoint(cfg, seed=0, device=dev)
    step = FusedStep(ckpt, persistent=True)
    state = DecodeState.allocate(cfg, args.context or args.position + 64, dev)
    state.kv_k.normal_()
    state.kv_v.normal_()
    grid = torch.cuda.get_device_properties(0).multi_processor_count
    plan = phase_plan(cfg)
    token = torch.tensor(11, device=dev)
    for position in range(args.position, args.position + 4):
        step(ckpt, token, position, state)
    step.trace = torch.zeros(len(plan) * SLOTS * grid, dtype=torch.int64, device=dev)
    step(ckpt, token, args.position + 4, state)
    torch.cuda.synchronize()
    assert step.status() == 0
    marks = step.trace.cpu().numpy().reshape(len(plan), SLOTS, grid).astype(np.int64)
    if args.dump:
        np.save(args.dump, marks)
    origin = marks[0, 0].min()
    marks = np.where(marks > 0, marks - origin, -1)
    show = {int(v) for v in args.show.split(",") if v}
    print("ns since the first block started; per phase: start(min max) x-ready(median) tile0(median) end(min median max)")
    totals: dict[str, list[tuple[int, int]]] = {}
    previous_end = 0
    for index, (kind, layer) in enumerate(plan):
        start, end = marks[index, 0], marks[index, 1]
        if layer in show or kind == "H":
            print(f"{index:4d} {kind:3s} L{layer:<3d} {start.min():8d} {start.max():8d}  {int(np.median(marks[index, 2])):8d} "
                  f"{int(np.median(marks[index, 3])):8d}  {end.min():8d} {int(np.median(end)):8d} {end.max():8d}")
        totals.setdefault(kind, []).append((int(end.max() - start.max()), int(start.max() - previous_end)))
        previous_end = int(end.max())
    print(f"whole step: {marks[-1, 1].max() / 1e3:.1f} us")
    nbytes = phase_bytes(cfg, args.position + 4)
    for kind, rows in totals.items():
        a = np.array(rows[1:] if len(rows) > 1 else rows)
        work = a[:, 0].mean() / 1e3
        rate = f"{nbytes[kind] / work / 1e6:7.2f} TB/s of {nbytes[kind] / 1e6:8.2f} MB" if nbytes.get(kind) else ""
        print(f"{kind:3s} x{len(rows):3d}  work {work:7.2f} us   barrier gap {a[:, 1].mean() / 1e3:6.2f} us   {rate}")


def phase_bytes(cfg, position: int) -> dict[str, float]:
    """Algorithmic bytes of each phase kind (weights once, state read + write, KV history)."""
    h, inter = cfg.hidden_size, cfg.moe_intermediate_size
    fp4 = lambda out, inp: out * inp // 2 + out * inp // 16
    kw = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    vw = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    qw, kvw = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    rec = cfg.linear_num_value_heads * cfg.linear_key_head_dim * cfg.linear_value_head_dim * 4
    return {
        "A": fp4(2 * kw + vw, h) + fp4(vw, h) + 2 * cfg.linear_num_value_heads * h * 2,
        "Aa": fp4(2 * qw, h) + 2 * fp4(kvw, h),
        "M": 2 * rec,
        "Ma": 2 * kvw * 2 * (position + 1),
        "B": fp4(h, vw), "Ba": fp4(h, qw),
        "C": (cfg.num_experts + 1) * h * 2,
        "D": (cfg.num_experts_per_tok + 1) * 2 * fp4(inter, h),
        "E": (cfg.num_experts_per_tok + 1) * fp4(h, inter),
        "H": cfg.vocab_size * h * 2,
    }


if __name__ == "__main__":
    with torch.inference_mode():
        main()

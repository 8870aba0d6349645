"""Regenerate the golden fixtures from the reference project.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/quickdraw

It writes two files beside this script:

``reference_fixtures.pt``
    The reference's own saved block/step fixtures (its ``references/model/*.pt``:
    inputs, expected output, expected post-call state, tolerances), re-saved as plain
    tensor trees under their original names.

``reference_outputs.pt``
    Outputs of the reference's own functions (``quickdraw.models.qwen``), run by this
    script on seeded inputs that exercise the NVFP4 path at shapes the saved fixtures
    do not cover: matvec tails, expert banks, routed rounding, all 256 byte codes,
    router ties, NVFP4 mixers, a bf16 LM head and a short greedy generation.

The reference is only imported here; the test-suite reads the two files.
"""

import argparse
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from quickdraw_b200 import synthetic  # noqa: E402
from quickdraw_b200.state import DecodeState  # noqa: E402
from quickdraw_b200.weights import NVFP4Linear  # noqa: E402
from tests.golden.fixture_io import to_tree  # noqa: E402


def small_fp4(out, inp, experts=None, group=16, bank_global=False):
    lead = () if experts is None else (experts,)
    codes = torch.randint(0, 256, (*lead, out, inp // 2), dtype=torch.uint8)
    scales = (torch.randint(1, 9, (*lead, out, inp // group)).float() / 8).to(torch.float8_e4m3fn)
    g = torch.rand(experts if bank_global else ()) * 0.25 + 0.01
    return NVFP4Linear(codes, scales, g.float(), group_size=group)


def mini_config():
    """Real head geometry (128-wide DeltaNet heads, 256-wide attention heads, conv
    width 4) on a narrow hidden size so the fixture stays small."""
    cfg = synthetic.model_config(num_layers=2, vocab_size=384, hidden=256, experts=8,
                                 topk=3, intermediate=64, interval=2)
    cfg.num_attention_heads, cfg.num_key_value_heads = 4, 2
    cfg.linear_num_key_heads, cfg.linear_num_value_heads = 1, 2
    return cfg


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", type=Path, required=True, help="checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, str(args.reference))
    sys.dont_write_bytecode = True
    from quickdraw.models import qwen  # the reference implementation

    torch.set_num_threads(1)
    # ---- 1. the reference's saved fixtures
    saved = {}
    for path in sorted((args.reference / "references/model").glob("*.pt")):
        saved[path.stem] = torch.load(path, map_location="cpu", weights_only=True)
    torch.save(saved, HERE / "reference_fixtures.pt")

    def shim(x, proj, **kw):
        if isinstance(proj, torch.Tensor):
            return F.linear(x.unsqueeze(0), proj).squeeze(0)
        return qwen.nvfp4_gemv(x, proj, **kw)

    out = {}
    with torch.inference_mode():
        # ---- 2. matvec cases (tails, routing, big rows)
        torch.manual_seed(7)
        cases = []
        for rows, width in ((13, 16), (17, 48), (5, 32), (64, 512), (48, 2048), (24, 4096)):
            proj = small_fp4(rows, width)
            x = torch.randn(width).bfloat16()
            for routing in (None, torch.tensor(0.317)):
                cases.append(dict(x=x, proj=proj, routing=routing,
                                  expected=qwen.nvfp4_gemv(x, proj, routing_weight=routing)))
        out["gemv"] = cases
        # all 256 byte codes through a group of two
        proj = NVFP4Linear(torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(256, 1),
                           torch.ones(256, 1).to(torch.float8_e4m3fn), torch.ones(()), group_size=2)
        x = torch.tensor([1.0, 3.0]).bfloat16()
        out["all_codes"] = dict(x=x, proj=proj, expected=qwen.nvfp4_gemv(x, proj))
        # routed double rounding known answer
        proj = NVFP4Linear(torch.full((1, 8), 0x77, dtype=torch.uint8),
                           torch.tensor([[0.5]]).to(torch.float8_e4m3fn), torch.tensor(0.137))
        x = torch.arange(1, 17).bfloat16()
        out["routed_kat"] = dict(x=x, proj=proj, routing=torch.tensor(0.1),
                                 expected=qwen.nvfp4_gemv(x, proj, routing_weight=torch.tensor(0.1)))
        # the single-matvec benchmark configuration, first rows only
        x, proj = synthetic.matvec_case(0)
        out["config1_head"] = dict(rows=64, expected=qwen.nvfp4_gemv(x, proj)[:64].clone(),
                                   checksum=qwen.nvfp4_gemv(x, proj).float().sum())
        # expert banks: ids, per-slot inputs, routing, per-expert global scales
        torch.manual_seed(14)
        bank_cases = []
        for bank_global in (False, True):
            bank = small_fp4(17, 48, experts=5, bank_global=bank_global)
            ids = torch.tensor([4, 1, 3], dtype=torch.int32)
            routing = torch.tensor([0.2, 0.3, 0.5])
            for per_slot in (False, True):
                x = torch.randn((3, 48) if per_slot else (48,)).bfloat16()
                for r in (None, routing):
                    expected = torch.stack([
                        qwen.nvfp4_gemv(x[s] if per_slot else x, qwen._expert_projection(bank, e),
                                       routing_weight=None if r is None else r[s])
                        for s, e in enumerate(ids.tolist())])
                    bank_cases.append(dict(x=x, proj=bank, ids=ids, routing=r, expected=expected))
        out["expert_gemv"] = bank_cases
        # ---- 3. routing
        routes = []
        torch.manual_seed(21)
        for experts, topk in ((6, 3), (7, 1), (33, 8), (256, 8), (7, 7)):
            for logits in (torch.zeros(experts), torch.randn(experts), torch.ones(experts),
                           torch.arange(experts).float() * 100,
                           (torch.randn(experts) * 4).round() / 4):
                logits = logits.bfloat16()
                p = torch.softmax(logits.float(), -1)
                ids = p.argsort(descending=True, stable=True)[:topk]
                w = p[ids]
                routes.append(dict(logits=logits, topk=topk, ids=ids.to(torch.int32), weights=w / w.sum()))
        out["route"] = routes
        # ---- 4. blocks with NVFP4 projections at real head geometry
        cfg = mini_config()
        src = synthetic.Source(5, "cpu")
        ckpt = synthetic.make_checkpoint(cfg, seed=5, device="cpu")
        out["mini_ckpt"] = ckpt
        x = src.normal("x", cfg.hidden_size)
        moe = ckpt.layers[0].moe
        out["moe"] = dict(x=x, expected=qwen.moe_block(moe, x, config=cfg))
        zero_router = synthetic.make_moe(cfg, src, "ties")
        zero_router.router.zero_()
        out["moe_ties"] = dict(w=zero_router, x=x, expected=qwen.moe_block(zero_router, x, config=cfg))
        gdn = ckpt.layers[0].attn
        torch.manual_seed(31)
        rec0 = torch.randn(cfg.linear_num_value_heads, 128, 128) * 0.01
        conv0 = src.normal("conv_state", cfg.conv_channels, 3)
        rec, conv, steps = rec0.clone(), conv0.clone(), []
        for step in range(3):
            xs = src.normal(f"gx{step}", cfg.hidden_size)
            y = qwen.gated_delta_net_block(gdn, xs, rec, conv, step, config=cfg,
                                           project_fp8=qwen.nvfp4_gemv)
            steps.append(dict(x=xs, expected=y, conv_after=conv.clone()))
        out["gdn"] = dict(rec0=rec0, conv0=conv0, steps=steps, rec_after=rec.clone())
        attn = ckpt.layers[1].attn
        capacity = 48
        kk = torch.full((capacity, cfg.num_key_value_heads, cfg.head_dim), 9.0).bfloat16()
        vv = torch.full((capacity, cfg.num_key_value_heads, cfg.head_dim), -11.0).bfloat16()
        kk[:37] = src.normal("k_hist", 37, cfg.num_key_value_heads, cfg.head_dim)
        vv[:37] = src.normal("v_hist", 37, cfg.num_key_value_heads, cfg.head_dim)
        attn_cases = []
        for position in (0, 5, 37):
            k1, v1 = kk.clone(), vv.clone()
            xs = src.normal(f"ax{position}", cfg.hidden_size)
            y = qwen.full_attention_block(attn, xs, (k1, v1), position, config=cfg,
                                          project_fp8=qwen.nvfp4_gemv)
            attn_cases.append(dict(x=xs, position=position, expected=y,
                                   k_row=k1[position].clone(), v_row=v1[position].clone()))
        out["attention"] = dict(k=kk, v=vv, cases=attn_cases)
        # ---- 5. whole step and a short greedy generation on the mini model
        from quickdraw.kernel import bind_kernels
        step = bind_kernels(fp8_gemv=shim, nvfp4_gemv=shim)["forward_step"]
        state = DecodeState.allocate(cfg, 32, "cpu")
        state.kv_k.fill_(9.0)
        state.kv_v.fill_(-11.0)
        prompt = [3, 77, 191, 5, 300]
        logits_trace, tokens, position, token = [], [], 0, None
        for t in prompt:
            logits = step(ckpt, torch.tensor(t), position, state)
            position += 1
        logits_trace.append(logits.clone())
        token = int(logits.argmax())
        tokens.append(token)
        for _ in range(15):
            logits = step(ckpt, torch.tensor(token), position, state)
            position += 1
            token = int(logits.argmax())
            tokens.append(token)
        logits_trace.append(logits.clone())
        out["generation"] = dict(prompt=prompt, tokens=tokens, first_logits=logits_trace[0],
                                 last_logits=logits_trace[1], rec_after=state.rec_state.clone(),
                                 conv_after=state.conv_state.clone(),
                                 k_after=state.kv_k.clone(), v_after=state.kv_v.clone())
    torch.save(to_tree(out), HERE / "reference_outputs.pt")
    for name in ("reference_fixtures.pt", "reference_outputs.pt"):
        print(name, (HERE / name).stat().st_size, "bytes")


if __name__ == "__main__":
    main()

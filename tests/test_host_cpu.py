"""Host-side logic that needs no GPU: the C-ABI library loads and exports every symbol the
header declares, a missing library fails loudly (there is no fallback path), and the engine's
request control flow (reference behaviour: quickdraw/engine/engine.py:93-148, exercised the way
tests/engine/test_engine.py of the reference does, with an injected step)."""

import re
from pathlib import Path

import pytest
import torch

from quickdraw_b200 import _lib, synthetic
from quickdraw_b200.engine import Engine
from quickdraw_b200.weights import Checkpoint

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "quickdraw_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(qd_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 30 and "qd_decode_step_persistent" in names and "qd_attn_decode_static" in names
    handle = _lib.lib()
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert handle.qd_version() >= 1
    assert handle.qd_error_string(3) == b"bounded device wait ran out"


def test_binding_table_covers_the_header():
    assert set(declared_symbols()) == set(_lib.exported_symbols())


def test_binding_argument_types_follow_the_header():
    """Every ctypes signature has the header's parameters, in order: pointers, int, unsigned, float, long long."""
    import ctypes
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    kinds = {ctypes.c_void_p: "pointer", ctypes.c_int: "int", ctypes.c_float: "float", ctypes.c_longlong: "long long",
             ctypes.c_uint: "unsigned int"}
    checked = 0
    for result, name, params in re.findall(r"\b(int|long long|const char\*)\s+(qd_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        if name == "qd_error_string":
            continue
        declared = []
        for param in (piece.strip() for piece in params.split(",")):
            if param in ("", "void"):
                continue
            if "*" in param:
                declared.append("pointer")
            else:
                declared.append(re.sub(r"\s+\w+$", "", param).replace("const ", "").strip())
        bound = [kinds[t] for t in _lib.SIGNATURES[name]]
        assert bound == declared, (name, bound, declared)
        assert (name in _lib.LONG_RESULTS) == (result == "long long"), name
        checked += 1
    assert checked == len(_lib.SIGNATURES)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libquickdraw_b200.so")
    with pytest.raises(_lib.LibraryMissing, match="no fallback"):
        _lib.lib()
    from quickdraw_b200 import kernels
    x = torch.zeros(2048, dtype=torch.bfloat16)
    with pytest.raises((_lib.LibraryMissing, AssertionError)):
        kernels.rms_norm(x, torch.ones(2048), 1e-6)


# ------------------------------------------------------------------------- engine control flow
class CountingStep:
    """A step that emits a fixed token sequence: logits peak at script[position]."""

    def __init__(self, vocab, script):
        self.vocab, self.script, self.calls = vocab, script, []

    def __call__(self, ckpt, token_id, position, state, **kwargs):
        self.calls.append((int(token_id), int(position)))
        state.rec_state.add_(1.0)
        logits = torch.zeros(self.vocab)
        logits[self.script[int(position) % len(self.script)]] = 1.0
        return logits


def make_engine(script, max_context=16):
    cfg = synthetic.model_config(num_layers=4, vocab_size=64)
    ckpt = Checkpoint(config=cfg, embed_tokens=None, final_norm=None, lm_head=None, layers=[])
    step = CountingStep(cfg.vocab_size, script)
    return Engine(ckpt, max_context=max_context, device="cpu", step=step), step


def test_custom_step_selects_custom_backend_without_graph():
    engine, _ = make_engine([1])
    assert engine.backend == "custom" and engine.graph is None and engine.state.position == 0


def test_b200_backend_refuses_a_cpu_device():
    cfg = synthetic.model_config(num_layers=4, vocab_size=64)
    ckpt = Checkpoint(config=cfg, embed_tokens=None, final_norm=None, lm_head=None, layers=[])
    with pytest.raises(AssertionError, match="no CPU path"):
        Engine(ckpt, max_context=8, device="cpu")


def test_generate_runs_the_prompt_once_then_decodes():
    engine, step = make_engine([3, 4, 5, 6, 7, 8, 9, 10])
    out = engine.generate([20, 21, 22], 4)
    # prompt tokens at positions 0..2; the logits after position 2 pick script[2] = 5; every
    # decode step feeds the previous choice at the next position
    assert out == [5, 6, 7, 8]
    assert step.calls == [(20, 0), (21, 1), (22, 2), (5, 3), (6, 4), (7, 5)]
    assert engine.state.position == 6


def test_generate_stops_at_eos_and_keeps_it():
    engine, _ = make_engine([3, 4, 5, 6, 7, 8])
    engine.eos_token_ids = {6}
    assert engine.generate([1, 2], 10) == [4, 5, 6]


def test_generate_stops_at_capacity():
    engine, _ = make_engine([1, 2, 3, 4, 5, 6, 7, 8], max_context=5)
    out = engine.generate([9, 9, 9], 10)
    assert len(out) == 3 and engine.state.position == 5       # prompt 3 + two decode steps fit


def test_generate_argument_contract():
    engine, step = make_engine([1])
    assert engine.generate([1, 2], 0) == [] and step.calls == []
    with pytest.raises(AssertionError, match="nonnegative"):
        engine.generate([1], -1)
    with pytest.raises(AssertionError, match="prompt must fit"):
        engine.prefill([])
    with pytest.raises(AssertionError, match="prompt must fit"):
        engine.prefill(list(range(17)))
    with pytest.raises(AssertionError, match="pending token"):
        engine.decode_step()


def test_reset_zeroes_history_and_keeps_the_buffers():
    engine, _ = make_engine([1, 2, 3])
    engine.generate([5, 6], 2)
    addresses = [t.data_ptr() for t in (engine.state.kv_k, engine.state.rec_state, engine.state.conv_state)]
    assert float(engine.state.rec_state.abs().sum()) > 0
    engine.reset()
    assert engine.state.position == 0 and engine.pending_token is None
    assert float(engine.state.rec_state.abs().sum()) == 0 and float(engine.state.conv_state.abs().sum()) == 0
    assert addresses == [t.data_ptr() for t in (engine.state.kv_k, engine.state.rec_state, engine.state.conv_state)]


def test_prefill_starts_a_fresh_request():
    engine, step = make_engine([1, 2, 3, 4])
    engine.generate([7, 7, 7], 1)
    engine.prefill([8])
    assert engine.state.position == 1 and step.calls[-1] == (8, 0)


# ----------------------------------------------------------------- conversation reuse (host logic)
def test_prefix_reuse_processes_only_the_new_suffix():
    engine, step = make_engine([3, 4, 5, 6, 7, 8, 9, 10], max_context=32)
    engine.prefill_reuse([20, 21, 22])
    assert engine.reused_tokens == 0 and [c for c in step.calls] == [(20, 0), (21, 1), (22, 2)]
    before = engine.state.rec_state.clone()
    step.calls.clear()
    logits = engine.prefill_reuse([20, 21, 22, 30, 31])                # extends the previous prompt
    assert engine.reused_tokens == 3 and step.calls == [(30, 3), (31, 4)]
    assert engine.state.position == 5 and int(logits.argmax()) == 7    # script[4]
    assert torch.equal(engine.state.rec_state, before + 2)             # restored, then two more steps
    step.calls.clear()
    engine.prefill_reuse([20, 21, 99, 30])                             # diverges inside the old prompt: fresh
    assert engine.reused_tokens == 0 and step.calls[0] == (20, 0) and len(step.calls) == 4
    assert torch.equal(engine.state.rec_state, torch.full_like(before, 4.0))


def test_snapshot_restore_round_trip_and_binding():
    engine, step = make_engine([3, 4, 5, 6, 7, 8, 9, 10], max_context=32)
    first = engine.generate([1, 2], 3)                                  # prompt 2 + decode steps at positions 2, 3
    snap = engine.snapshot()
    assert snap.tokens == (1, 2, first[0], first[1]) and snap.position == 4
    assert snap.nbytes() == engine.state.rec_state.nbytes + engine.state.conv_state.nbytes
    rec = engine.state.rec_state.clone()
    engine.decode_step()
    engine.decode_step()
    engine.restore(snap)                                                # back to the snapshot: buffers reused
    assert engine.state.position == 4 and torch.equal(engine.state.rec_state, rec)
    assert int(engine.pending_token) == first[2]
    assert int(engine.decode_step()) == 7                               # continues as it did the first time (script[4])
    # a new conversation overwrites the cache rows the snapshot relies on
    engine.prefill([9, 9, 9, 9, 9])
    with pytest.raises(AssertionError, match="overwritten"):
        engine.restore(snap)
    other, _ = make_engine([1], max_context=32)
    with pytest.raises(AssertionError, match="another checkpoint"):
        other.restore(snap)


def test_reuse_survives_a_reset_when_the_cache_rows_are_intact():
    engine, step = make_engine([3, 4, 5, 6], max_context=32)
    engine.prefill_reuse([5, 6, 7])
    engine.reset()                                                      # history cleared, cache rows untouched
    step.calls.clear()
    engine.prefill_reuse([5, 6, 7, 8])
    assert engine.reused_tokens == 3 and step.calls == [(8, 3)]


def test_bench_byte_counts_of_a_step_and_of_a_batched_step():
    """The algorithmic bytes bench.py divides by: one sequence of the batched count is the single-token
    count (up to the norm vectors and the embedding row), more sequences add their own state and KV
    history and touch more distinct experts, never more than all of them."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = synthetic.model_config()
    one, single = bench.bytes_per_batch_step(cfg, 1, 639), bench.bytes_per_token(cfg, 639)
    assert abs(one - single) < 1e-3 * single
    small, large = bench.bytes_per_batch_step(cfg, 32, 8192), bench.bytes_per_batch_step(cfg, 64, 8192)
    assert one < small < large
    # 32 more sequences: their state and KV history, and fewer than 32 x 8 more experts per layer
    h, inter = cfg.hidden_size, cfg.moe_intermediate_size
    expert = 3 * (inter * h // 2 + inter * h // 16 + 4)
    per_sequence = (large - small) / 32
    state = 36 * 2 * (32 * 128 * 128 * 4 + 8192 * 3 * 2) + 12 * 2 * 2 * 256 * 2 * 8193
    assert state < per_sequence < state + cfg.num_hidden_layers * 8 * expert


@pytest.mark.parametrize("tokens,fp8", [(3, False), (70, False), (3, True), (40, True)])
def test_chunk_and_batch_paths_pass_the_declared_number_of_arguments(monkeypatch, tokens, fp8):
    """The Python drivers of the prompt-chunk and batched-decode paths, run on CPU tensors with the library
    call replaced by a recorder: every call names a bound entry point and passes as many arguments as the
    header declares for it (ctypes would not notice a missing trailing argument), and both paths reach
    their few-row and many-row forms."""
    from quickdraw_b200 import batch, prefill
    from quickdraw_b200.state import DecodeState
    seen = {}

    def record(name, *args):
        assert name in _lib.SIGNATURES, name
        assert len(args) == len(_lib.SIGNATURES[name]), (name, len(args), len(_lib.SIGNATURES[name]))
        seen[name] = seen.get(name, 0) + 1

    class FakeLibrary:
        def __getattr__(self, name):
            assert name in _lib.SIGNATURES, name
            return lambda *args: 4096 if name.endswith("_bytes") else 1

    for module in (prefill, batch):
        monkeypatch.setattr(module, "call", record)
        monkeypatch.setattr(module, "lib", lambda: FakeLibrary())
        monkeypatch.setattr(module, "stream_of", lambda t: None)
    class AsIfOnGpu(torch.Tensor):         # the drivers refuse token ids that are not on a GPU
        is_cuda = property(lambda self: True)

    cfg = synthetic.model_config(num_layers=4, vocab_size=512, experts=16, topk=4)
    ckpt = synthetic.make_checkpoint(cfg, seed=2, device="cpu", fp8_mixers=fp8, nvfp4_head=fp8)
    state = DecodeState.allocate(cfg, 128, "cpu")
    prefill.ChunkPrefill(ckpt).run((torch.arange(tokens) % cfg.vocab_size).as_subclass(AsIfOnGpu), 0, state)
    assert seen.get("qd_seq_moe_combine_norm", 0) == 3 and "qd_seq_moe_combine" not in seen      # the last MoE block is not run
    assert ("qd_fp8_matmul" in seen) == fp8
    assert ("qd_nvfp4_expert_rows2" in seen) or ("qd_nvfp4_grouped_matmul" in seen)
    chunk_calls = dict(seen)
    seen.clear()
    many = batch.BatchState(cfg, 3, 64, "cpu")
    decoder = batch.BatchDecode(ckpt)
    monkeypatch.setattr(decoder, "_attn_splits", lambda *a: 1, raising=False)
    picked, logits = decoder.step(torch.tensor([1, 2, 3]).as_subclass(AsIfOnGpu), many)
    assert picked.shape == (3,) and logits.shape == (3, cfg.vocab_size) and many.positions.tolist() == [1, 1, 1]
    assert seen["qd_seq_moe_combine_norm"] == 4 and seen["qd_nvfp4_expert_rows2"] == 4 and seen["qd_seq_bf16_matmul2"] >= 4
    assert "qd_nvfp4_matmul_rows3" in seen or fp8
    assert chunk_calls


def test_every_kernel_launched_as_a_programmatic_dependent_waits_for_its_predecessor():
    """Source check: a kernel that qd_launch may start before the kernel in front of it has finished
    (pdl argument other than false / 0) contains the wait, as chain_enter() or grid_dependency_wait()."""
    sources = {path.name: path.read_text() for path in (ROOT / "quickdraw_b200" / "csrc").glob("*.cu*")}

    def arguments(text, start):          # top-level arguments of the call whose "(" ends at `start`
        depth, current, found, i = 0, "", [], start
        while True:
            ch = text[i]
            if ch in "([":
                depth += 1
            elif ch in ")]":
                if depth == 0:
                    return found + [current.strip()]
                depth -= 1
            if ch == "," and depth == 0 and (found or current.count("<") == current.count(">")):      # template arguments of the kernel
                found.append(current.strip())
                current = ""
            else:
                current += ch
            i += 1

    def bodies(kernel):
        for text in sources.values():
            for match in re.finditer(r"__global__[^{;]*?\b" + kernel + r"\s*\(", text, flags=re.S):
                start = text.index("{", match.end())
                depth, end = 0, start
                while True:
                    depth += {"{": 1, "}": -1}.get(text[end], 0)
                    if depth == 0:
                        break
                    end += 1
                yield text[start:end]

    dependents = 0
    for name, text in sources.items():
        for match in re.finditer(r"(?<!int )qd_launch\(", text):
            args = arguments(text, match.end())
            kernel, pdl = re.match(r"\w+", args[0]).group(0), args[5]
            if pdl in ("false", "0"):
                continue
            found = list(bodies(kernel))
            assert found, (name, kernel)
            assert all("chain_enter();" in body or "grid_dependency_wait();" in body for body in found), (name, kernel)
            dependents += 1
    assert dependents >= 30


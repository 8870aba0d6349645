"""Single-request greedy generation on the B200 decode kernels.

Same surface and behaviour as the reference engine (quickdraw/engine/engine.py:10-148):
``Engine(ckpt, max_context, device, backend, *, kernels, step, cuda_graph, ...)``, the
attributes ``state, pending_token, eos_token_ids, graph, step, ckpt, max_context, backend``
and the methods ``capture_decode, prefill, decode_step, generate, reset``.  The engine
owns ``state.position``; a step never touches it.  ``reset`` zeroes the recurrent and
convolution history, keeps every buffer address (a captured graph stays valid) and leaves
the KV cache alone (slots at or beyond the position are never read).

Prompts run in chunks of ``prefill_chunk_size`` tokens through the sequence path
(tensor-core products; the reference's default chunk is 128, here 2048 because larger chunks
amortise the expert weights better) where the fused step applies, token by token otherwise.

Backends: ``"b200"`` (default) runs the fused CUDA step where the checkpoint has the
36B-A3B widths and the composed operator table otherwise; passing ``kernels=`` or
``step=`` gives the ``"custom"`` backend used by tests (no graph).  There is no CPU
backend: on a CPU device only a caller-supplied ``step`` can run.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .state import DecodeState
from .weights import Checkpoint


@dataclass
class Snapshot:
    """A request's history at one point: the token ids processed so far, the recurrent and
    convolution tensors (copies), the position and the pending token.  The KV cache is not
    copied: its rows below ``position`` stay valid as long as the engine only continues from a
    restored snapshot or starts over (rows at or beyond the position are rewritten before they
    are read).  Bound to the checkpoint and the execution settings it was taken under."""
    tokens: tuple[int, ...]
    position: int
    pending_token: torch.Tensor | None
    rec_state: torch.Tensor
    conv_state: torch.Tensor
    binding: tuple

    def nbytes(self) -> int:
        return self.rec_state.nbytes + self.conv_state.nbytes


class Engine:
    def __init__(self, ckpt: Checkpoint, max_context: int = 32768, device: str = "cuda",
                 backend: str | None = None, *, kernels: dict | None = None, step=None,
                 cuda_graph: bool = True, prefill_chunk_size: int = 2048,
                 sequence_prefill: bool = True, _step_object=None):
        custom = kernels is not None or step is not None
        if backend is None:
            backend = "custom" if custom else "b200"
        assert backend in ("b200", "custom")
        assert kernels is None or step is None
        assert backend == "custom" or not custom
        assert max_context > 0 and prefill_chunk_size > 0
        self.ckpt, self.max_context, self.device, self.backend = ckpt, max_context, device, backend
        self.prefill_chunk_size = prefill_chunk_size
        self.sequence_prefill = False      # set below where the chunked path applies
        self.chunk_prefill = None
        self.graph = None
        self.fused = None
        on_cuda = torch.device(device).type == "cuda"
        if _step_object is not None:      # a prebuilt fused-style step (expert parallel)
            assert on_cuda and not custom
            self.fused = _step_object
            self.step = _step_object
        elif step is not None:
            self.step = step
        else:
            assert on_cuda, "the b200 backend needs a CUDA device; there is no CPU path"
            from . import fused
            from .kernels import bind_kernels
            if kernels is None and fused.supports(ckpt):
                self.fused = fused.FusedStep(ckpt)
                self.step = self.fused
                if sequence_prefill and all(fused.mixer_format(layer) in ("nvfp4", "fp8") for layer in ckpt.layers):
                    from .prefill import ChunkPrefill     # NVFP4 or static-FP8 mixers; the last token goes through the step
                    self.chunk_prefill = ChunkPrefill(ckpt)
                    self.sequence_prefill = True
            else:
                prepared = ([(1 + l.input_layernorm.float(), 1 + l.post_attention_layernorm.float())
                             for l in ckpt.layers], 1 + ckpt.final_norm.float())
                self.step = bind_kernels(prepared=prepared, **(kernels or {}))["forward_step"]
        self.state = DecodeState.allocate(ckpt.config, max_context, device)
        self.history: list[int] = []            # token ids processed since the last reset (prompt part; see _fold)
        self._decoded: list[torch.Tensor] = []  # tokens processed by decode steps, still on the device
        self._kv_tokens: list[int] = []         # the token sequence the cache rows [0, n) were computed from
        self.pending_token: torch.Tensor | None = None
        self.eos_token_ids: set[int] = set()
        if backend == "b200" and cuda_graph:
            self.capture_decode()

    # ----------------------------------------------------------------- graph capture
    @torch.inference_mode()
    def capture_decode(self):
        """Capture one decode step (position read from a device scalar) plus the greedy
        selection; three warm-up steps run on a scratch state first
        (quickdraw/engine/engine.py:65-83)."""
        assert self.backend == "b200" and self.state.position == 0
        dev = self.device
        self._decode_input = torch.zeros((), dtype=torch.long, device=dev)
        self._device_position = torch.zeros((), dtype=torch.int32, device=dev)
        self._decode_output = torch.empty((), dtype=torch.long, device=dev)
        scratch = DecodeState(torch.empty_like(self.state.kv_k), torch.empty_like(self.state.kv_v),
                              torch.zeros_like(self.state.rec_state),
                              torch.zeros_like(self.state.conv_state), 0)
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream):
            for _ in range(3):
                self.step(self.ckpt, self._decode_input, self._device_position, scratch)
        torch.cuda.current_stream(dev).wait_stream(stream)
        self.graph = torch.cuda.CUDAGraph()
        # an expert-parallel step leaves the greedy token on every rank without assembling the
        # full logits: keep the all-gather of the vocabulary shards out of the replayed step
        gathers = getattr(self.step, "gather_logits", None)
        if gathers is not None:
            self.step.gather_logits = False
        with torch.cuda.graph(self.graph, stream=stream):
            logits = self.step(self.ckpt, self._decode_input, self._device_position, self.state)
            if self.fused is not None:
                self._decode_output.copy_(self.fused.next_token)
            else:
                torch.argmax(logits, out=self._decode_output)
            self._decode_logits = logits
        if gathers is not None:
            self.step.gather_logits = gathers
        del scratch
        self.reset()

    # ----------------------------------------------------------------------- requests
    @torch.inference_mode()
    def prefill(self, token_ids: list[int]) -> torch.Tensor:
        """Start a fresh request: run the prompt, return the logits after its last token
        (quickdraw/engine/engine.py:93-111).  With the chunked path all tokens but the last
        go through the sequence kernels ``prefill_chunk_size`` at a time; the last one, and
        every token otherwise, goes through the decode step."""
        assert 0 < len(token_ids) <= self.max_context, "prompt must fit within max_context"
        self.reset()
        return self._extend(list(token_ids))

    def _extend(self, token_ids: list[int]) -> torch.Tensor:
        """Process ``token_ids`` after the current position; logits after the last one."""
        start = self.state.position
        tokens = torch.tensor(token_ids, dtype=torch.long, device=self.device)
        logits = None
        done = 0
        if self.sequence_prefill and len(token_ids) > 1:
            while done < len(token_ids) - 1:
                stop = min(len(token_ids) - 1, done + self.prefill_chunk_size)
                self.chunk_prefill.run(tokens[done:stop], start + done, self.state)
                done = stop
            self.state.position = start + done
        for index, token in enumerate(tokens[done:], start=done):
            if self.backend == "b200":
                logits = self.step(self.ckpt, token, self.state.position, self.state,
                                   logits=index == len(tokens) - 1)
            else:
                logits = self.step(self.ckpt, token, self.state.position, self.state)
            self.state.position += 1
        self._note([int(t) for t in token_ids])
        return logits

    def _note(self, ids: list[int]) -> None:
        """Record tokens processed at the positions after ``history`` and what that did to the
        cache: a row is rewritten with the same content exactly when the whole prefix is the same."""
        for token in ids:
            at = len(self.history)
            if not (at < len(self._kv_tokens) and self._kv_tokens[at] == token):
                del self._kv_tokens[at:]
                self._kv_tokens.append(token)
            self.history.append(token)

    def _fold(self) -> None:
        """Bring ``history`` up to date with the decode steps taken (their tokens stay on the
        device until somebody needs them as numbers: one transfer here, none per step)."""
        if self._decoded:
            ids = torch.stack([t.reshape(()) for t in self._decoded]).tolist()
            self._decoded = []
            self._note([int(t) for t in ids])

    # ------------------------------------------------------------- conversation reuse
    def _binding(self) -> tuple:
        return (id(self.ckpt), self.backend, str(self.device), self.max_context, self.sequence_prefill)

    @torch.inference_mode()
    def snapshot(self) -> Snapshot:
        """The history of the current request, to come back to later (the reference plans this:
        todo.md "Conversation reuse").  75 MB of copies for the 36B-A3B model, no KV copy."""
        self._fold()
        pending = None if self.pending_token is None else self.pending_token.clone()
        return Snapshot(tuple(self.history), self.state.position, pending, self.state.rec_state.clone(),
                        self.state.conv_state.clone(), self._binding())

    @torch.inference_mode()
    def restore(self, snap: Snapshot) -> None:
        """Copy a snapshot back into the existing buffers (a captured graph stays valid).  Refused
        when the snapshot belongs to another checkpoint or other execution settings, or when the
        cache rows it relies on have been overwritten by a different prefix since."""
        self._fold()
        assert snap.binding == self._binding(), "snapshot taken under another checkpoint or other settings"
        assert self._kv_covers(snap.tokens), "the cache rows of this snapshot have been overwritten"
        self.state.rec_state.copy_(snap.rec_state)
        self.state.conv_state.copy_(snap.conv_state)
        self.state.position = snap.position
        self.pending_token = None if snap.pending_token is None else snap.pending_token.clone()
        self.history = list(snap.tokens)

    def _kv_covers(self, tokens) -> bool:
        return len(tokens) <= len(self._kv_tokens) and list(tokens) == self._kv_tokens[:len(tokens)]

    @torch.inference_mode()
    def prefill_reuse(self, token_ids: list[int], snap: Snapshot | None = None) -> torch.Tensor:
        """Like ``prefill``, but when ``snap`` (default: the snapshot this method took after the
        previous prompt) holds a proper prefix of ``token_ids`` only the new suffix is processed.
        Anything else - no snapshot, different tokens, foreign binding, overwritten cache rows -
        is a fresh ``prefill``.  Leaves a snapshot of the whole prompt in ``last_snapshot``."""
        assert 0 < len(token_ids) <= self.max_context, "prompt must fit within max_context"
        self._fold()
        snap = snap if snap is not None else getattr(self, "last_snapshot", None)
        usable = (snap is not None and snap.binding == self._binding() and 0 < len(snap.tokens) < len(token_ids)
                  and list(token_ids[:len(snap.tokens)]) == list(snap.tokens) and snap.position == len(snap.tokens)
                  and self._kv_covers(snap.tokens))
        if usable:
            self.restore(snap)
            self.reused_tokens = len(snap.tokens)
            logits = self._extend(list(token_ids[len(snap.tokens):]))
        else:
            self.reused_tokens = 0
            logits = self.prefill(token_ids)
        self.last_snapshot = self.snapshot()
        return logits

    @classmethod
    def from_pretrained(cls, path: str, **kwargs) -> "Engine":
        """Load a checkpoint directory (safetensors shards), merge the static FP8 scales of the
        projections that share an activation, and build the engine (reference:
        quickdraw/engine/engine.py:85-90)."""
        from .loader import load_checkpoint, merge_fp8_scales
        ckpt = load_checkpoint(path, device=kwargs.get("device", "cuda"))
        merge_fp8_scales(ckpt)
        return cls(ckpt, **kwargs)

    @torch.inference_mode()
    def decode_step(self) -> torch.Tensor:
        """Process the pending token, select and return its successor (0-d int64)."""
        assert self.pending_token is not None, "select a pending token before decode"
        assert self.state.position < self.max_context, "context capacity reached"
        self._decoded.append(self.pending_token)          # becomes a number only when a snapshot asks
        if self.graph is None:
            logits = self.step(self.ckpt, self.pending_token, self.state.position, self.state)
            self.pending_token = torch.argmax(logits)
        else:
            watchdog = getattr(self.step, "watchdog", None)
            if watchdog is not None:
                watchdog.check()        # expert parallel: a lost peer raises here, before the launch
            self._decode_input.copy_(self.pending_token)
            self._device_position.fill_(self.state.position)
            self.graph.replay()
            self.pending_token = self._decode_output.clone()
        self.state.position += 1
        return self.pending_token

    @torch.inference_mode()
    def generate(self, token_ids: list[int], max_tokens: int) -> list[int]:
        """New token ids, EOS included; stops before a step would exceed the capacity."""
        assert max_tokens >= 0, "max_tokens must be nonnegative"
        if max_tokens == 0:
            return []
        logits = self.prefill(token_ids)
        self.pending_token = torch.argmax(logits)
        output = [int(self.pending_token.item())]
        while (len(output) < max_tokens and output[-1] not in self.eos_token_ids
               and self.state.position < self.max_context):
            output.append(int(self.decode_step().item()))
        return output

    def reset(self) -> None:
        self.state.rec_state.zero_()
        self.state.conv_state.zero_()
        self.state.position = 0
        self.pending_token = None
        self._fold()                # what the cache rows hold outlives the request
        self.history = []

"""The fused decode step: the whole token step as one C-ABI call (``qd_decode_step``).

``FusedStep(ckpt)`` builds the library's host-side pointer table from a checkpoint whose
mixer projections are NVFP4 and whose LM head is bf16 (the 36B-A3B layout) and is itself
the ``step(ckpt, token_id, position, state, *, logits=True)`` callable the engine
expects (reference boundary: quickdraw/engine/engine.py:15-16, qwen.py:196-199).  The
checkpoint keeps ownership of every weight; this object owns one small zero-initialised
device workspace per instance and the fp32 ``1 + gamma`` norm vectors.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong, c_void_p

import torch

from . import _lib
from ._lib import check, ptr
from .weights import Checkpoint, NVFP4Linear

BF16 = torch.bfloat16
FLAG_PDL, FLAG_NO_LOGITS = 1, 2


class QdFp4(Structure):
    _fields_ = [("codes", c_void_p), ("scales", c_void_p), ("global_", c_void_p)]


class QdLayer(Structure):
    _fields_ = [("is_attention", c_int), ("gamma_in", c_void_p), ("gamma_post", c_void_p),
                ("proj_a", QdFp4), ("proj_b", QdFp4), ("proj_c", QdFp4), ("proj_out", QdFp4),
                ("in_proj_a", c_void_p), ("in_proj_b", c_void_p), ("conv1d", c_void_p),
                ("a_log", c_void_p), ("dt_bias", c_void_p), ("head_norm", c_void_p),
                ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("router", c_void_p), ("shared_expert_gate", c_void_p),
                ("experts_gate", QdFp4), ("experts_up", QdFp4), ("experts_down", QdFp4),
                ("shared_gate", QdFp4), ("shared_up", QdFp4), ("shared_down", QdFp4),
                ("experts_global_per_expert", c_int), ("state_index", c_int),
                ("mixers_fp8", c_int), ("mixer_input_scale", c_void_p), ("out_input_scale", c_void_p)]


class QdModelConfig(Structure):
    _fields_ = [("hidden", c_int), ("layers", c_int), ("vocab", c_int),
                ("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("rotary_dim", c_int),
                ("key_heads", c_int), ("value_heads", c_int), ("key_dim", c_int), ("value_dim", c_int),
                ("conv_width", c_int), ("experts", c_int), ("topk", c_int), ("intermediate", c_int),
                ("eps", c_float), ("rope_theta", c_float), ("expert_lo", c_int), ("expert_hi", c_int),
                ("vocab_lo", c_int), ("vocab_hi", c_int),
                ("embed", c_void_p), ("final_gamma", c_void_p), ("lm_head", c_void_p), ("lm_head_fp4", QdFp4)]


class QdExchange(Structure):
    _fields_ = [("rank", c_int), ("world", c_int), ("peer_base", ctypes.c_ulonglong * 8)]


class QdState(Structure):
    _fields_ = [("kv_k", c_void_p), ("kv_v", c_void_p), ("rec_state", c_void_p),
                ("conv_state", c_void_p), ("capacity", c_int)]


def _fp4(proj: NVFP4Linear) -> QdFp4:
    assert isinstance(proj, NVFP4Linear), "the fused step needs NVFP4 projections"
    assert proj.group_size == 16 and proj.weight.is_cuda
    assert proj.weight.is_contiguous() and proj.weight_scale.is_contiguous()
    assert proj.weight.dtype == torch.uint8 and proj.weight_scale.dtype == torch.float8_e4m3fn
    assert proj.weight_scale_2.dtype == torch.float32
    assert proj.weight.data_ptr() % 16 == 0 and proj.weight_scale.data_ptr() % 16 == 0
    return QdFp4(proj.weight.data_ptr(), proj.weight_scale.data_ptr(), proj.weight_scale_2.data_ptr())


def _fp8(proj) -> QdFp4:
    """A static FP8 projection in the descriptor of a mixer projection: E4M3 weights in ``codes``,
    no block scales, the fp32 weight scale in ``global``."""
    assert proj.weight.is_cuda and proj.weight.is_contiguous() and proj.weight.dtype == torch.float8_e4m3fn
    assert proj.weight_scale.dtype == torch.float32 and proj.weight_scale.numel() == 1
    assert proj.input_scale is not None and proj.input_scale.dtype == torch.float32 and proj.input_scale.numel() == 1
    assert proj.weight.data_ptr() % 16 == 0
    return QdFp4(proj.weight.data_ptr(), None, proj.weight_scale.data_ptr())


MIXER_NAMES = {"full_attention": ("q_proj", "k_proj", "v_proj", "o_proj"),
               "linear_attention": ("in_proj_qkv", "in_proj_z", "out_proj")}


def mixer_format(layer) -> str:
    """'nvfp4', 'fp8' (all projections of the mixer static FP8 with one input scale for those
    that read the layer input) or 'mixed' (not covered by the fused step)."""
    from .weights import FP8Linear
    projections = [getattr(layer.attn, name) for name in MIXER_NAMES[layer.layer_type]]
    if all(isinstance(p, NVFP4Linear) for p in projections):
        return "nvfp4"
    if all(isinstance(p, FP8Linear) and p.input_scale is not None for p in projections):
        readers = projections[:-1]
        if all(float(p.input_scale) == float(readers[0].input_scale) for p in readers):
            return "fp8"
    return "mixed"


def supports(ckpt: Checkpoint) -> bool:
    """Shapes the fused step covers: the 36B-A3B widths (any depth, vocabulary, expert
    count up to 256, top-k up to 8); mixers NVFP4 or static FP8 whose input-reading projections
    share one activation scale (``loader.merge_fp8_scales``), NVFP4 experts, a bf16 or NVFP4 LM head."""
    c = ckpt.config
    head_ok = isinstance(ckpt.lm_head, torch.Tensor) or (isinstance(ckpt.lm_head, NVFP4Linear) and ckpt.lm_head.weight.ndim == 2
                                                         and ckpt.lm_head.weight_scale_2.numel() == 1)
    return (head_ok and c.hidden_size == 2048
            and c.linear_num_value_heads * c.linear_value_head_dim == 4096
            and c.num_attention_heads * c.head_dim == 4096 and c.moe_intermediate_size == 512
            and c.shared_expert_intermediate_size == 512 and c.linear_value_head_dim == 128
            and c.linear_key_head_dim <= 128 and c.num_experts <= 256 and c.num_experts_per_tok <= 8
            and c.head_dim <= 256 and c.num_attention_heads // c.num_key_value_heads <= 8
            and all(mixer_format(layer) != "mixed" for layer in ckpt.layers))


class FusedStep:
    """``expert_range`` / ``vocab_range``: the slice of the routed experts and of the LM-head
    rows this checkpoint holds (expert parallel; banks and ``lm_head`` are local to the slice).
    A sliced model runs through the persistent kernel only and needs ``set_exchange``."""

    def __init__(self, ckpt: Checkpoint, *, expert_range: tuple[int, int] | None = None,
                 vocab_range: tuple[int, int] | None = None, pdl: bool = True, persistent: bool | None = None):
        assert supports(ckpt), "checkpoint shapes are outside the fused step; use kernels.forward_step"
        self.ckpt, self.pdl = ckpt, pdl
        c = ckpt.config
        self.lib = _lib.lib()
        self.device = ckpt.embed_tokens.device
        lo, hi = expert_range or (0, c.num_experts)
        self.expert_range = (lo, hi)
        self.vocab_range = vocab_range
        self.sliced = expert_range is not None or vocab_range is not None
        self.exchange = None
        self._keep = []      # fp32 gammas and anything else the pointer table refers to

        def gamma(weight):
            g = (1 + weight.float()).contiguous()
            self._keep.append(g)
            return g.data_ptr()

        self.head_fp4 = isinstance(ckpt.lm_head, NVFP4Linear)
        head_rows = ckpt.lm_head.out_features if self.head_fp4 else ckpt.lm_head.shape[0]
        assert ckpt.embed_tokens.dtype == BF16 and ckpt.embed_tokens.is_contiguous()
        assert self.head_fp4 or (ckpt.lm_head.dtype == BF16 and ckpt.lm_head.is_contiguous())
        assert head_rows == ((vocab_range[1] - vocab_range[0]) if vocab_range else c.vocab_size), \
            "lm_head must hold exactly the owned rows"
        cfg = QdModelConfig(
            hidden=c.hidden_size, layers=c.num_hidden_layers, vocab=c.vocab_size,
            q_heads=c.num_attention_heads, kv_heads=c.num_key_value_heads, head_dim=c.head_dim,
            rotary_dim=int(c.head_dim * c.partial_rotary_factor), key_heads=c.linear_num_key_heads,
            value_heads=c.linear_num_value_heads, key_dim=c.linear_key_head_dim,
            value_dim=c.linear_value_head_dim, conv_width=c.linear_conv_kernel_dim,
            experts=c.num_experts, topk=c.num_experts_per_tok, intermediate=c.moe_intermediate_size,
            eps=c.rms_norm_eps, rope_theta=c.rope_theta, expert_lo=lo, expert_hi=hi,
            vocab_lo=vocab_range[0] if vocab_range else 0, vocab_hi=vocab_range[1] if vocab_range else 0,
            embed=ckpt.embed_tokens.data_ptr(), final_gamma=gamma(ckpt.final_norm),
            lm_head=None if self.head_fp4 else ckpt.lm_head.data_ptr(),
            lm_head_fp4=_fp4(ckpt.lm_head) if self.head_fp4 else QdFp4())
        self.model = c_void_p()
        check(self.lib.qd_model_create(byref(cfg), byref(self.model)), "qd_model_create")
        full = linear = 0
        for layer in ckpt.layers:
            moe, at = layer.moe, layer.attn
            assert moe.experts_gate.weight.shape[0] == hi - lo, "expert banks must hold the owned range"
            d = QdLayer()
            d.gamma_in, d.gamma_post = gamma(layer.input_layernorm), gamma(layer.post_attention_layernorm)
            fp8 = mixer_format(layer) == "fp8"
            describe = _fp8 if fp8 else _fp4
            if fp8:
                names = MIXER_NAMES[layer.layer_type]
                d.mixers_fp8 = 1
                d.mixer_input_scale = getattr(at, names[0]).input_scale.data_ptr()
                d.out_input_scale = getattr(at, names[-1]).input_scale.data_ptr()
            if layer.layer_type == "full_attention":
                d.is_attention = 1
                d.proj_a, d.proj_b, d.proj_c, d.proj_out = map(describe, (at.q_proj, at.k_proj, at.v_proj, at.o_proj))
                d.q_norm, d.k_norm = at.q_norm.data_ptr(), at.k_norm.data_ptr()
                d.state_index, full = full, full + 1
            else:
                d.is_attention = 0
                d.proj_a, d.proj_b, d.proj_out = describe(at.in_proj_qkv), describe(at.in_proj_z), describe(at.out_proj)
                for name in ("in_proj_a", "in_proj_b", "conv1d", "A_log", "dt_bias", "norm"):
                    t = getattr(at, name)
                    assert t.dtype == BF16 and t.is_contiguous() and t.is_cuda
                d.in_proj_a, d.in_proj_b = at.in_proj_a.data_ptr(), at.in_proj_b.data_ptr()
                d.conv1d, d.a_log, d.dt_bias = at.conv1d.data_ptr(), at.A_log.data_ptr(), at.dt_bias.data_ptr()
                d.head_norm = at.norm.data_ptr()
                d.state_index, linear = linear, linear + 1
            assert moe.router.dtype == BF16 and moe.router.is_contiguous()
            d.router, d.shared_expert_gate = moe.router.data_ptr(), moe.shared_expert_gate.data_ptr()
            d.experts_gate, d.experts_up, d.experts_down = map(
                _fp4, (moe.experts_gate, moe.experts_up, moe.experts_down))
            d.shared_gate, d.shared_up, d.shared_down = map(_fp4, (moe.shared_gate, moe.shared_up, moe.shared_down))
            d.experts_global_per_expert = int(moe.experts_gate.weight_scale_2.numel() != 1)
            check(self.lib.qd_model_set_layer(self.model, layer.idx, byref(d)), "qd_model_set_layer")
        nbytes = self.lib.qd_decode_workspace_bytes(self.model)
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self.next_token = torch.zeros((), dtype=torch.long, device=self.device)
        self.launches_per_step = 6 * c.num_hidden_layers + 1
        # One cooperative launch per token; the launch-per-phase path stays as a cross-check
        # (whole models only).
        self.program = None
        self.trace = None
        if persistent is None:
            persistent = True
        assert persistent or not self.sliced, "a model slice runs through the persistent kernel only"
        assert persistent or (not self.head_fp4 and all(mixer_format(layer) == "nvfp4" for layer in ckpt.layers)), \
            "static FP8 mixers and an NVFP4 LM head run through the persistent kernel only"
        if persistent:
            size = self.lib.qd_program_bytes(self.model)
            host = torch.zeros(size, dtype=torch.uint8)
            check(self.lib.qd_program_build(self.model, ptr(self.workspace), c_void_p(host.data_ptr()), size),
                  "qd_program_build")
            self.program = host.to(self.device)
            self.launches_per_step = 1
        self.persistent = bool(persistent)

    def __del__(self):
        model = getattr(self, "model", None)
        if model:
            self.lib.qd_model_destroy(model)
            self.model = None

    def _state(self, state) -> QdState:
        for t in (state.kv_k, state.kv_v, state.rec_state, state.conv_state):
            assert t.is_cuda and t.is_contiguous()
        assert state.kv_k.dtype == BF16 and state.rec_state.dtype == torch.float32
        return QdState(state.kv_k.data_ptr(), state.kv_v.data_ptr(), state.rec_state.data_ptr(),
                       state.conv_state.data_ptr(), state.kv_k.shape[1])

    def _position(self, position, state):
        if isinstance(position, torch.Tensor):
            assert position.dtype == torch.int32 and position.is_cuda and position.numel() == 1
            return ptr(position), 0
        assert 0 <= position < state.kv_k.shape[1]
        return None, int(position)

    def __call__(self, ckpt, token_id, position, state, *, logits=True):
        """One token; returns bf16 logits [vocab] (fresh tensor) or None.  The greedy next
        token of the step is left in ``self.next_token`` (int64 device scalar)."""
        assert ckpt is self.ckpt, "bound to a different checkpoint"
        assert token_id.ndim == 0 and token_id.dtype == torch.long and token_id.is_cuda
        pos_dev, pos_host = self._position(position, state)
        st = self._state(state)
        out = torch.empty(ckpt.config.vocab_size, dtype=BF16, device=self.device) if logits else None
        flags = (FLAG_PDL if self.pdl else 0) | (0 if logits else FLAG_NO_LOGITS)
        stream = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        if self.persistent:
            assert self.exchange is not None or not self.sliced, "a model slice needs set_exchange() first"
            if self.exchange is not None and out is None:
                out = self._scratch_logits      # the LM head (and its exchange) runs on every token
            check(self.lib.qd_decode_step_persistent(
                self.model, byref(st), ptr(token_id), pos_dev, pos_host, ptr(self.workspace),
                ptr(self.program), byref(self.exchange) if self.exchange is not None else None, ptr(out),
                ptr(self.next_token), flags, ptr(self.trace), stream),
                "qd_decode_step_persistent")
            return out if logits else None
        check(self.lib.qd_decode_step(self.model, byref(st), ptr(token_id), pos_dev, pos_host,
                                      ptr(self.workspace), ptr(out) if logits else ptr(self.workspace),
                                      ptr(self.next_token), flags, stream), "qd_decode_step")
        return out

    def exchange_bytes(self) -> int:
        """Bytes of this rank's exchange area (expert parallel)."""
        return int(self.lib.qd_exchange_bytes(self.model))

    def set_exchange(self, rank: int, world: int, peer_addresses: list[int]) -> None:
        """Expert parallel: ``peer_addresses[r]`` = address in this process of rank r's
        zero-initialised exchange area (``exchange_bytes()`` bytes, peer-mapped)."""
        assert 1 < world <= 8 and 0 <= rank < world and len(peer_addresses) == world
        ex = QdExchange(rank=rank, world=world)
        for r, address in enumerate(peer_addresses):
            ex.peer_base[r] = int(address)
        self.exchange = ex
        self._scratch_logits = torch.empty(self.ckpt.config.vocab_size, dtype=BF16, device=self.device)

    def status(self) -> int:
        """Device status word (0 = clean; bit 0 = a bounded wait ran out)."""
        return int(self.workspace[256:260].view(torch.int32).item())

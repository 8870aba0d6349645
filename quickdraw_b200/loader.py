"""Checkpoint loading: a Hugging Face style directory of safetensors shards -> ``Checkpoint``.

Same contract as the reference loader (quickdraw/models/weights.py:187-330): ``config.json``
(``text_config`` block), ``model.safetensors.index.json`` (``weight_map``: tensor name ->
shard), language-model tensors under ``model.language_model.``, the vision tower
(``model.visual.``) skipped, ``mtp.*`` tensors only on request, ``layers=`` to load a subset,
the per-expert projections ``...mlp.experts.<e>.<gate|up|down>_proj.*`` stacked into one bank
per projection with a leading expert axis.  A projection is NVFP4 when it carries a
``weight_scale_2`` tensor and static FP8 otherwise (the published checkpoint: FP8 mixers, NVFP4
experts and LM head; the synthetic 36B-A3B layout: NVFP4 everywhere, bf16 LM head).

Built for a 180 GB device: nothing is stacked on the host.  Every bank is allocated once at
its final size on the device and filled expert by expert through two pinned staging buffers on
a copy stream, so reading the next expert from the page cache overlaps the previous expert's
host-to-device copy; ``expert_range`` / ``vocab_range`` read only the experts and LM-head rows
one rank of an expert-parallel group owns (the rest of the shards is never touched).
"""

from __future__ import annotations

import json
import re
from contextlib import ExitStack
from pathlib import Path

import torch

from .weights import (Checkpoint, FP8Linear, FullAttnWeights, GDNWeights, LayerWeights, ModelConfig,
                      MoEWeights, NVFP4Linear)

ROOT = "model.language_model."
LAYER_NAME = re.compile(r"model\.language_model\.layers\.(\d+)\.")

# field of the container -> tensor name below the layer's mixer prefix; "linear" entries are
# quantised projections (format decided by the tensors present), the others plain tensors
GDN_FIELDS = {"in_proj_qkv": "linear", "in_proj_z": "linear", "out_proj": "linear",
              "in_proj_a": "in_proj_a.weight", "in_proj_b": "in_proj_b.weight", "conv1d": "conv1d.weight",
              "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm.weight"}
ATTN_FIELDS = {"q_proj": "linear", "k_proj": "linear", "v_proj": "linear", "o_proj": "linear",
               "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}


class ShardReader:
    """Opens the shards of a checkpoint on first use and hands out tensors by name."""

    def __init__(self, directory: Path, stack: ExitStack):
        from safetensors import safe_open
        self.directory, self.stack, self._open = directory, stack, safe_open
        self.weight_map: dict[str, str] = json.loads((directory / "model.safetensors.index.json").read_text())["weight_map"]
        self.handles: dict[str, object] = {}

    def __contains__(self, name: str) -> bool:
        return name in self.weight_map

    def _handle(self, name: str):
        shard = self.weight_map[name]
        if shard not in self.handles:
            self.handles[shard] = self.stack.enter_context(self._open(self.directory / shard, framework="pt"))
        return self.handles[shard]

    def tensor(self, name: str) -> torch.Tensor:
        return self._handle(name).get_tensor(name)

    def rows(self, name: str, lo: int, hi: int) -> torch.Tensor:
        """Rows [lo, hi) of a tensor without reading the others."""
        return self._handle(name).get_slice(name)[lo:hi]


class BankFiller:
    """Stacks per-expert tensors into one device tensor through double-buffered pinned staging."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device) if self.cuda else None
        self.staging: dict[tuple, list] = {}
        self.turn = 0

    def fill(self, parts) -> torch.Tensor:
        """parts: an iterable of equally shaped host tensors, one per expert."""
        parts = iter(parts)
        first = next(parts)
        rest = list(parts)
        bank = torch.empty((1 + len(rest), *first.shape), dtype=first.dtype, device=self.device)
        for index, part in enumerate([first, *rest]):
            self._copy(bank[index], part)
        return bank

    def _copy(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        if not self.cuda:
            dst.copy_(src)
            return
        key = (tuple(src.shape), src.dtype)
        if key not in self.staging:
            self.staging[key] = [(torch.empty(src.shape, dtype=src.dtype).pin_memory(), torch.cuda.Event()) for _ in range(2)]
        buffer, event = self.staging[key][self.turn & 1]
        self.turn += 1
        event.synchronize()                      # the copy that last used this buffer has finished
        buffer.copy_(src)
        with torch.cuda.stream(self.stream):
            dst.copy_(buffer, non_blocking=True)
            event.record(self.stream)

    def finish(self) -> None:
        if self.cuda:
            self.stream.synchronize()


def _scalar(reader: ShardReader, name: str, device) -> torch.Tensor:
    return reader.tensor(name).float().to(device)


def _linear(reader: ShardReader, prefix: str, device, rows: tuple[int, int] | None = None):
    """One quantised projection: NVFP4 if it has a second-level scale, static FP8 otherwise."""
    def body(suffix):
        name = f"{prefix}.{suffix}"
        return (reader.rows(name, *rows) if rows else reader.tensor(name)).to(device)
    activation = _scalar(reader, prefix + ".input_scale", device) if prefix + ".input_scale" in reader else None
    if prefix + ".weight_scale_2" in reader:
        return NVFP4Linear(weight=body("weight"), weight_scale=body("weight_scale"),
                           weight_scale_2=_scalar(reader, prefix + ".weight_scale_2", device), input_scale=activation)
    assert rows is None, "row slices are for NVFP4 / bf16 matrices"
    return FP8Linear(weight=body("weight"), weight_scale=_scalar(reader, prefix + ".weight_scale", device),
                     input_scale=activation)


def _expert_bank(reader: ShardReader, filler: BankFiller, base: str, proj: str, experts: range, device) -> NVFP4Linear:
    names = lambda suffix: [f"{base}.{e}.{proj}_proj.{suffix}" for e in experts]
    weight = filler.fill(reader.tensor(n) for n in names("weight"))
    scale = filler.fill(reader.tensor(n) for n in names("weight_scale"))
    second = torch.stack([reader.tensor(n).float().reshape(()) for n in names("weight_scale_2")]).to(device)
    activation = None
    if all(n in reader for n in names("input_scale")):
        activation = torch.stack([reader.tensor(n).float().reshape(()) for n in names("input_scale")]).to(device)
    return NVFP4Linear(weight=weight, weight_scale=scale, weight_scale_2=second, input_scale=activation)


def _mixer(reader: ShardReader, prefix: str, fields: dict[str, str], device) -> dict:
    return {field: (_linear(reader, prefix + field, device) if where == "linear" else reader.tensor(prefix + where).to(device))
            for field, where in fields.items()}


def load_checkpoint(path: str | Path, device: str | torch.device = "cuda", include_mtp: bool = False,
                    layers: list[int] | None = None, *, expert_range: tuple[int, int] | None = None,
                    vocab_range: tuple[int, int] | None = None) -> Checkpoint:
    """Language weights of the checkpoint directory ``path`` on ``device``
    (reference: quickdraw/models/weights.py:187-330; same arguments, plus the two slices)."""
    directory = Path(path)
    device = torch.device(device)
    config = ModelConfig.from_json(directory / "config.json")
    wanted = set(range(config.num_hidden_layers)) if layers is None else set(layers)
    experts = range(*(expert_range or (0, config.num_experts)))
    with ExitStack() as stack:
        reader = ShardReader(directory, stack)
        present = sorted({int(m.group(1)) for m in map(LAYER_NAME.match, reader.weight_map) if m} & wanted)
        filler = BankFiller(device)
        built = []
        for index in present:
            at = f"{ROOT}layers.{index}."
            kind = config.layer_types[index]
            assert kind in ("linear_attention", "full_attention"), kind
            if kind == "linear_attention":
                mixer = GDNWeights(**_mixer(reader, at + "linear_attn.", GDN_FIELDS, device))
            else:
                mixer = FullAttnWeights(**_mixer(reader, at + "self_attn.", ATTN_FIELDS, device))
            bank = lambda proj: _expert_bank(reader, filler, at + "mlp.experts", proj, experts, device)
            shared = lambda proj: _linear(reader, f"{at}mlp.shared_expert.{proj}_proj", device)
            moe = MoEWeights(router=reader.tensor(at + "mlp.gate.weight").to(device),
                             shared_expert_gate=reader.tensor(at + "mlp.shared_expert_gate.weight").to(device),
                             experts_gate=bank("gate"), experts_up=bank("up"), experts_down=bank("down"),
                             shared_gate=shared("gate"), shared_up=shared("up"), shared_down=shared("down"))
            built.append(LayerWeights(idx=index, layer_type=kind,
                                      input_layernorm=reader.tensor(at + "input_layernorm.weight").to(device),
                                      post_attention_layernorm=reader.tensor(at + "post_attention_layernorm.weight").to(device),
                                      attn=mixer, moe=moe))
        if "lm_head.weight_scale_2" in reader:
            head = _linear(reader, "lm_head", device, rows=vocab_range)
        else:
            head = (reader.rows("lm_head.weight", *vocab_range) if vocab_range else reader.tensor("lm_head.weight")).to(device)
        extra = {}
        if include_mtp:
            extra = {name: reader.tensor(name).to(device) for name in reader.weight_map if name.startswith("mtp.")}
        checkpoint = Checkpoint(config=config, embed_tokens=reader.tensor(ROOT + "embed_tokens.weight").to(device),
                                final_norm=reader.tensor(ROOT + "norm.weight").to(device), lm_head=head,
                                layers=built, mtp=extra)
        filler.finish()
    return checkpoint


def merge_fp8_scales(ckpt: Checkpoint) -> None:
    """The projections that read the same activation (q, k, v of an attention layer; qkv and z of
    a DeltaNet layer) get one weight scale and one input scale, the largest of the group; a
    projection whose weight scale changes is re-expressed in the new scale (dequantise through
    f16, divide, clamp to +-448, round to E4M3).  Reference: quickdraw/models/weights.py:169-184.
    After this the group's activation is quantised once for all its members."""
    for layer in ckpt.layers:
        group = ("q_proj", "k_proj", "v_proj") if layer.layer_type == "full_attention" else ("in_proj_qkv", "in_proj_z")
        members = [getattr(layer.attn, name) for name in group]
        if not all(isinstance(m, FP8Linear) for m in members):
            continue
        shared_weight = torch.stack([m.weight_scale.reshape(()) for m in members]).max()
        shared_input = torch.stack([m.input_scale.reshape(()) for m in members]).max()
        changed = any(float(m.weight_scale) != float(shared_weight) for m in members)
        for m in members:
            if changed:
                real = m.weight.half() * m.weight_scale.reshape(())
                m.weight = (real.float() * shared_weight.reciprocal()).clamp(-448, 448).to(torch.float8_e4m3fn)
            m.weight_scale, m.input_scale = shared_weight, shared_input


def save_checkpoint(ckpt: Checkpoint, path: str | Path, shards: int = 2, text_config: dict | None = None) -> None:
    """Write ``ckpt`` as a directory ``load_checkpoint`` reads: the inverse naming, tensors dealt
    round-robin over ``shards`` safetensors files, ``config.json`` and the index.  Used to put
    synthetic models on disk (the published checkpoint is not redistributed with this package)."""
    from dataclasses import asdict
    from safetensors.torch import save_file
    directory = Path(path)
    directory.mkdir(parents=True, exist_ok=True)
    tensors: dict[str, torch.Tensor] = {}

    def put_linear(prefix: str, proj) -> None:
        tensors[prefix + ".weight"] = proj.weight
        tensors[prefix + ".weight_scale"] = proj.weight_scale
        if isinstance(proj, NVFP4Linear):
            tensors[prefix + ".weight_scale_2"] = proj.weight_scale_2.reshape(())
        if proj.input_scale is not None:
            tensors[prefix + ".input_scale"] = proj.input_scale.reshape(())

    tensors[ROOT + "embed_tokens.weight"] = ckpt.embed_tokens
    tensors[ROOT + "norm.weight"] = ckpt.final_norm
    if isinstance(ckpt.lm_head, NVFP4Linear):
        put_linear("lm_head", ckpt.lm_head)
    else:
        tensors["lm_head.weight"] = ckpt.lm_head
    for layer in ckpt.layers:
        at = f"{ROOT}layers.{layer.idx}."
        tensors[at + "input_layernorm.weight"] = layer.input_layernorm
        tensors[at + "post_attention_layernorm.weight"] = layer.post_attention_layernorm
        linear_mixer = layer.layer_type == "linear_attention"
        prefix = at + ("linear_attn." if linear_mixer else "self_attn.")
        for field, where in (GDN_FIELDS if linear_mixer else ATTN_FIELDS).items():
            value = getattr(layer.attn, field)
            if where == "linear":
                put_linear(prefix + field, value)
            else:
                tensors[prefix + where] = value
        moe = layer.moe
        tensors[at + "mlp.gate.weight"] = moe.router
        tensors[at + "mlp.shared_expert_gate.weight"] = moe.shared_expert_gate
        for proj in ("gate", "up", "down"):
            put_linear(f"{at}mlp.shared_expert.{proj}_proj", getattr(moe, f"shared_{proj}"))
            bank = getattr(moe, f"experts_{proj}")
            per_expert_scale = bank.weight_scale_2.numel() == bank.weight.shape[0]
            for e in range(bank.weight.shape[0]):
                name = f"{at}mlp.experts.{e}.{proj}_proj"
                tensors[name + ".weight"] = bank.weight[e]
                tensors[name + ".weight_scale"] = bank.weight_scale[e]
                tensors[name + ".weight_scale_2"] = (bank.weight_scale_2[e] if per_expert_scale else bank.weight_scale_2).reshape(())
                if bank.input_scale is not None:
                    tensors[name + ".input_scale"] = bank.input_scale[e].reshape(())
    tensors.update(ckpt.mtp)
    names = sorted(tensors)
    weight_map = {}
    for i in range(shards):
        shard = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        members = names[i::shards]
        save_file({n: tensors[n].detach().cpu().contiguous().clone() for n in members}, str(directory / shard))
        weight_map.update({n: shard for n in members})
    (directory / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    config = asdict(ckpt.config)
    theta = config.pop("rope_theta")
    (directory / "config.json").write_text(json.dumps({"text_config": dict(config, rope_parameters={"rope_theta": theta}, **(text_config or {}))}))

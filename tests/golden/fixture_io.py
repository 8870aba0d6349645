"""Tensor-tree (de)serialisation for golden fixtures.

A fixture file is a ``torch.save`` of nested dicts / lists / tensors / scalars only, so
it loads with ``weights_only=True``.  Dataclass instances are written as
``{"__type__": <class name>, "fields": {...}}`` and rebuilt with the containers of
``quickdraw_b200`` (the class names are those of the reference's containers).
"""

from dataclasses import fields, is_dataclass

import torch

from quickdraw_b200.state import DecodeState
from quickdraw_b200.weights import CONTAINERS

_TYPES = dict(CONTAINERS, DecodeState=DecodeState)


def to_tree(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu().clone()
    if is_dataclass(obj):
        return {"__type__": type(obj).__name__,
                "fields": {f.name: to_tree(getattr(obj, f.name)) for f in fields(obj)}}
    if isinstance(obj, dict):
        return {key: to_tree(value) for key, value in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(to_tree(value) for value in obj)
    return obj


def from_tree(tree, device="cpu"):
    if isinstance(tree, torch.Tensor):
        return tree.to(device).clone()
    if isinstance(tree, dict):
        if "__type__" in tree:
            return _TYPES[tree["__type__"]](**from_tree(tree["fields"], device))
        return {key: from_tree(value, device) for key, value in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(from_tree(value, device) for value in tree)
    return tree


def load(path, device="cpu"):
    return from_tree(torch.load(path, map_location="cpu", weights_only=True), device)

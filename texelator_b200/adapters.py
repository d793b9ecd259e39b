"""Which linears of a decoder model the BC4 operator replaces.

Same contract as ``texelator/adapters.py`` of the reference: ``discover_linears``
(:57-87) lists q/k/v/o/gate/up/down projections that sit inside a numbered layer
and marks them unsupported when K is not a multiple of one BC4 block (16);
``artifact_key`` (:51-54) names the files; ``resolve_parent`` (:90-96) finds the
module to patch.
"""
from __future__ import annotations

import hashlib
import re
from collections.abc import Iterable
from dataclasses import asdict, dataclass

from torch import nn

DEFAULT_SUFFIXES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
FUSED_SUFFIXES = ("qkv_proj", "query_key_value", "c_attn", "Wqkv", "gate_up_proj", "dense_h_to_4h", "dense_4h_to_h")

_LAYER_RE = re.compile(r"(?:^|\.)(?:decoder\.layers|layers|h|blocks)\.(\d+)(?:\.|$)")


@dataclass(frozen=True)
class LinearSpec:
    module_name: str
    artifact_key: str
    layer: int
    op: str
    M: int
    K: int
    bias: bool
    supported: bool
    reason: str

    def to_dict(self) -> dict:
        return asdict(self)


def layer_index(name: str) -> int | None:
    match = _LAYER_RE.search(name)
    return int(match.group(1)) if match else None


def artifact_key(name: str) -> str:
    stem = re.sub(r"[^A-Za-z0-9_.-]+", "_", name).replace(".", "__")
    return f"{stem}--{hashlib.sha256(name.encode()).hexdigest()[:10]}"


def discover_linears(model: nn.Module, suffixes: Iterable[str] = DEFAULT_SUFFIXES,
                     include_regex: str | None = None) -> list[LinearSpec]:
    wanted = tuple(suffixes)
    extra = re.compile(include_regex) if include_regex else None
    specs = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear):
            continue
        layer = layer_index(name)
        op = name.rsplit(".", 1)[-1]
        if layer is None or not (op in wanted or (extra and extra.search(name))):
            continue
        rows, cols = (int(v) for v in module.weight.shape)
        ok = cols % 16 == 0
        specs.append(LinearSpec(name, artifact_key(name), layer, op, rows, cols, module.bias is not None, ok,
                                "ok" if ok else "input dimension K is not divisible by 16"))
    specs.sort(key=lambda spec: (spec.layer, spec.module_name))
    return specs


def resolve_parent(model: nn.Module, module_name: str) -> tuple[nn.Module, str]:
    parent_name, _, child = module_name.rpartition(".")
    if not parent_name:
        if not hasattr(model, child):
            raise RuntimeError(f"model module does not exist: {module_name}")
        return model, child
    return model.get_submodule(parent_name), child

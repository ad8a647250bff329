"""Neburax configuration: the keys of its config.json.

A small decoder-only family that lists its layers one by one and mixes three kinds of token mixing::

    architecture   "Neburax"
    vocab, width
    layers         [{"type": "mamba2" | "parallel", "mixer": {...}, "mlp": {...} | null, "weights_of": j}, ...]
    norm           {"eps"}

``mixer`` of a ``mamba2`` layer: heads, vdim, state, groups, norm_groups, conv (taps).
``mixer`` of a ``parallel`` layer: left {heads, kv_heads, dim, vdim, scale, mask {size}}, right {width, blocks,
conv}, left_scale, right_scale: chunked attention and a gated linear recurrence side by side.
``mlp``: kind "dense" {ff}, or kind "moe" {expert {ff}, router {experts, top, identity}, shared {ff} | absent}.
A layer with ``weights_of: j`` runs layer j's tensors over a cache and state of its own.

No size has a default: a key that the model needs and config.json lacks is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig

LAYER_TYPES = ("mamba2", "parallel")
MLP_KINDS = ("dense", "moe")
WHO = "NeburaxConfig"


def _need(d: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"{WHO}: {where} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"{WHO}: {where}.{key} has the wrong type: {v!r}")
    return v


def _positive(d: Any, keys, where: str) -> None:
    for k in keys:
        if _need(d, k, where, int) <= 0:
            raise ConfigError(f"{WHO}: {where}.{k} must be positive")


def _check_mamba2(m: Any, where: str) -> None:
    _positive(m, ("heads", "vdim", "state", "groups", "norm_groups", "conv"), where)
    if m["heads"] % m["groups"]:
        raise ConfigError(f"{WHO}: {where}.heads must be a multiple of groups")
    if (m["heads"] * m["vdim"]) % m["norm_groups"]:
        raise ConfigError(f"{WHO}: {where}: heads * vdim must be a multiple of norm_groups")


def _check_parallel(m: Any, where: str) -> None:
    left, right = (m or {}).get("left"), (m or {}).get("right")
    _positive(left, ("heads", "kv_heads", "dim", "vdim"), where + ".left")
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"{WHO}: {where}.left.heads must be a multiple of kv_heads")
    if not _need(left, "scale", where + ".left") > 0:
        raise ConfigError(f"{WHO}: {where}.left.scale must be positive")
    if left.get("mask") is not None and _need(left["mask"], "size", where + ".left.mask", int) < 1:
        raise ConfigError(f"{WHO}: {where}.left.mask.size must be at least 1")
    _positive(right, ("width", "blocks", "conv"), where + ".right")
    if right["width"] % right["blocks"]:
        raise ConfigError(f"{WHO}: {where}.right.width must be a multiple of blocks")
    for k in ("left_scale", "right_scale"):
        _need(m, k, where)


def _check_mlp(mlp: Any, where: str) -> None:
    if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"{WHO}: {where}.kind must be one of {MLP_KINDS}")
    if mlp["kind"] == "dense":
        _positive(mlp, ("ff",), where)
        return
    _positive(mlp.get("expert"), ("ff",), where + ".expert")
    router = mlp.get("router")
    n = _need(router, "experts", where + ".router", int)
    top = _need(router, "top", where + ".router", int)
    ident = router.get("identity") or 0
    if isinstance(ident, bool) or not isinstance(ident, int) or ident < 0 or n < 0 or n + ident < 1:
        raise ConfigError(f"{WHO}: {where}.router needs experts + identity >= 1, neither negative")
    if not 1 <= top <= n + ident:
        raise ConfigError(f"{WHO}: {where}.router needs 1 <= top <= experts + identity")
    if mlp.get("shared") is not None:
        _positive(mlp["shared"], ("ff",), where + ".shared")


@dataclasses.dataclass
class NeburaxConfig(ModelConfig):
    architecture: ClassVar[str] = "Neburax"
    model_types: ClassVar[tuple[str, ...]] = ("neburax",)

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    norm: Optional[dict] = None

    def to_dict(self) -> dict[str, Any]:
        out = super().to_dict()
        out["architecture"] = self.architecture
        out["layers"] = list(self.layers)
        return out

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{WHO}: vocab and width must be positive")
        if not self.layers:
            raise ConfigError(f"{WHO}: 'layers' is empty")
        if not _need(self.norm, "eps", "norm") > 0:
            raise ConfigError(f"{WHO}: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{WHO}: {where}.type is {layer.get('type') if isinstance(layer, dict) else layer!r}; "
                                  f"known: {LAYER_TYPES}")
            if layer["type"] == "mamba2":
                _check_mamba2(layer.get("mixer"), where + ".mixer")
            else:
                _check_parallel(layer.get("mixer"), where + ".mixer")
            if layer.get("mlp") is not None:
                _check_mlp(layer["mlp"], where + ".mlp")
            j = layer.get("weights_of")
            if j is not None:
                if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(self.layers) or j == i:
                    raise ConfigError(f"{WHO}: {where}.weights_of must name another layer")
                if self.layers[j].get("weights_of") is not None:
                    raise ConfigError(f"{WHO}: {where}.weights_of names layer {j}, which has no tensors of its own")

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs."""
        j = self.layers[i].get("weights_of")
        return i if j is None else int(j)

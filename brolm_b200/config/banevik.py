"""Banevik configuration: the keys of its config.json.

A small decoder-only family whose config.json lists its layers one by one::

    architecture   "Banevik"
    vocab, width
    embedding      {"bigram": {"buckets", "mul_prev", "mul_cur"}}     a hashed table of token pairs
    layers         [{"type": "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]
    loop           {"start", "stop", "times"}    layers start .. stop-1 run ``times`` times (null: no loop)
    norm           {"eps"}
    logit_softcap

``mixer`` of a latent-attention layer: heads, dim (unrotated query/key size per head), rot_dim
(rotated), vdim, kv_rank, scale, rot {base, dims}, mask {size} (absent: every earlier token is seen).
``mlp``: kind "moe", expert {ff}, router {experts, top}.

No size has a default: a key that the model needs and config.json lacks is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig

LAYER_TYPES = ("latent_attention",)
MLP_KINDS = ("moe",)


def _need(d: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"BanevikConfig: {where} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"BanevikConfig: {where}.{key} has the wrong type: {v!r}")
    return v


@dataclasses.dataclass
class BanevikConfig(ModelConfig):
    architecture: ClassVar[str] = "Banevik"
    model_types: ClassVar[tuple[str, ...]] = ("banevik",)

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    loop: Optional[dict] = None
    norm: Optional[dict] = None
    embedding: Optional[dict] = None
    logit_softcap: float = 0.0

    def to_dict(self) -> dict[str, Any]:
        out = super().to_dict()
        out["architecture"] = self.architecture
        out["layers"] = list(self.layers)
        return out

    def validate(self) -> None:
        who = "BanevikConfig"
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{who}: vocab and width must be positive")
        if not self.layers:
            raise ConfigError(f"{who}: 'layers' is empty")
        if not _need(self.norm, "eps", "norm") > 0:
            raise ConfigError(f"{who}: norm.eps must be positive")
        if self.logit_softcap < 0:
            raise ConfigError(f"{who}: logit_softcap must be >= 0 (0 switches it off)")
        bg = self.bigram
        if bg is not None:
            if _need(bg, "buckets", "embedding.bigram", int) <= 0:
                raise ConfigError(f"{who}: embedding.bigram.buckets must be positive")
            for k in ("mul_prev", "mul_cur"):
                if _need(bg, k, "embedding.bigram", int) < 0:
                    raise ConfigError(f"{who}: embedding.bigram.{k} must not be negative")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{who}: {where}.type is {layer.get('type') if isinstance(layer, dict) else layer!r}; "
                                  f"known: {LAYER_TYPES}")
            m = layer.get("mixer")
            for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                if _need(m, k, f"{where}.mixer", int) <= 0:
                    raise ConfigError(f"{who}: {where}.mixer.{k} must be positive")
            if not _need(m, "scale", f"{where}.mixer") > 0:
                raise ConfigError(f"{who}: {where}.mixer.scale must be positive")
            rot = m.get("rot")
            dims = _need(rot, "dims", f"{where}.mixer.rot", int)
            if not _need(rot, "base", f"{where}.mixer.rot") > 0:
                raise ConfigError(f"{who}: {where}.mixer.rot.base must be positive")
            if dims < 0 or dims % 2 or dims > m["rot_dim"]:
                raise ConfigError(f"{who}: {where}.mixer.rot.dims must be even and at most rot_dim")
            if m.get("mask") is not None and _need(m["mask"], "size", f"{where}.mixer.mask", int) < 1:
                raise ConfigError(f"{who}: {where}.mixer.mask.size must be at least 1")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"{who}: {where}.mlp.kind must be one of {MLP_KINDS}")
                if _need(mlp.get("expert"), "ff", f"{where}.mlp.expert", int) <= 0:
                    raise ConfigError(f"{who}: {where}.mlp.expert.ff must be positive")
                n = _need(mlp.get("router"), "experts", f"{where}.mlp.router", int)
                top = _need(mlp.get("router"), "top", f"{where}.mlp.router", int)
                if not 1 <= top <= n:
                    raise ConfigError(f"{who}: {where}.mlp.router needs 1 <= top <= experts")
        if self.loop is not None:
            start, stop = _need(self.loop, "start", "loop", int), _need(self.loop, "stop", "loop", int)
            times = _need(self.loop, "times", "loop", int)
            if not (0 <= start <= stop <= len(self.layers)) or times < 1:
                raise ConfigError(f"{who}: loop needs 0 <= start <= stop <= {len(self.layers)} and times >= 1")

    # derived ---------------------------------------------------------------
    @property
    def bigram(self) -> Optional[dict]:
        return (self.embedding or {}).get("bigram")

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def runs(self) -> list[tuple[int, bool]]:
        """The order of the layer runs: (layer, whether the run opens a pass of the loop)."""
        n = len(self.layers)
        if self.loop is None or self.loop["stop"] <= self.loop["start"]:
            return [(i, False) for i in range(n)]
        start, stop = self.loop["start"], self.loop["stop"]
        out = [(i, False) for i in range(start)]
        for _ in range(self.loop["times"]):
            out += [(i, i == start) for i in range(start, stop)]
        return out + [(i, False) for i in range(stop, n)]

"""Banevik as a layout of parts.

Embedding plus a hashed table of token pairs; layers in the parallel arrangement (mixer and feed-forward
read the same stream through a norm each); latent attention with a sliding window and a sink; routed
experts with a logistic gate on the expert's input; a span of layers that runs several times with the
same weights, every pass with caches of its own and opened by a product over [stream; embedding output];
the embedding as output matrix, with soft-capped logits.  Every size and constant comes from config.json.

Tensor names: ``embed``, ``bigram``, ``loop.in``, ``final.norm`` and, for layer i, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{up,down}``.
"""
from __future__ import annotations

from ..config import BanevikConfig, register_architecture
from ..parts import BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, PairTableSpec, PartSpec

LOOP_ENTRY = "loop_in"


def banevik_layout(cfg: BanevikConfig) -> ModelLayout:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("norm", "rmsnorm", dict(size=W, eps=cfg.eps, offset=1.0), {"weight": name})

    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        rot = m["rot"]
        position = None
        if rot["dims"] > 0:
            position = PartSpec("position", "rope", dict(head_dim=m["rot_dim"], theta=float(rot["base"]),
                                                         rotary_dim=rot["dims"]))
        mixer = PartSpec(
            "mixer", "latent_attention",
            dict(hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"],
                 scale=float(m["scale"]), eps=cfg.eps, window=(m.get("mask") or {}).get("size"), sink=True,
                 position=position),
            {"q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk",
             "uv": p + "mix.uv", "sink": p + "mix.sink", "o": p + "mix.o"})
        ffn = pre_ffn = None
        mlp = layer.get("mlp")
        if mlp is not None:
            n = mlp["router"]["experts"]
            names = {"router": p + "mlp.router"}
            for e in range(n):
                names[f"e{e}.up"] = f"{p}mlp.e{e}.up"
                names[f"e{e}.down"] = f"{p}mlp.e{e}.down"
            ffn = PartSpec("feedforward", "routed_experts",
                           dict(hidden=W, inter=mlp["expert"]["ff"], experts=n, top=mlp["router"]["top"],
                                activation="relu2", scale_input=True), names)
            pre_ffn = norm(p + "norm2")
        blocks.append(BlockSpec(kind="parallel", mixer=mixer, feedforward=ffn, pre_mixer_norm=norm(p + "norm1"),
                                pre_ffn_norm=pre_ffn))
    runs = cfg.runs()
    looped = any(opens for _, opens in runs)
    stream_parts = {}
    if looped:
        stream_parts[LOOP_ENTRY] = PartSpec("stream", "concat_linear", dict(hidden=W), {"weight": "loop.in"})
    pairs = None
    if cfg.bigram is not None:
        bg = cfg.bigram
        pairs = PairTableSpec("bigram", bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    return ModelLayout(
        embedding=EmbeddingSpec("embed", cfg.vocab, W, scale=1.0, pairs=pairs),
        blocks=blocks,
        schedule=[LayerCall(i, before=LOOP_ENTRY if opens else None) for i, opens in runs],
        final_norm=norm("final.norm"),
        head=HeadSpec("head", tied_to="embed", softcap=float(cfg.logit_softcap or 0.0)),
        stream_parts=stream_parts)


register_architecture(BanevikConfig, banevik_layout)

"""Neburax as a layout of parts.

Layers whose sublayers read the residual stream itself and whose results alone are normed (x += n1(mixer(x)),
x += n2(ff(x))); two kinds of mixer: a selective state space, or chunked attention (a norm over the whole query
and key rows, no positions, value heads of their own size) side by side with a gated linear recurrence; a dense
feed-forward with biases, or routed experts with a softmax router, identity experts and a shared expert; a layer
may run another layer's tensors over a cache and state of its own; the embedding is the output matrix.  Every
size and constant comes from config.json.

Tensor names: ``embed``, ``final.norm`` and, for layer i, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}`` (state space) or
``l<i>.mix.left.{q,k,v,q.norm,k.norm,o}`` and ``l<i>.mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}``,
``l<i>.mlp.{up,up.b,down,down.b}`` (dense) or ``l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down}}``.
"""
from __future__ import annotations

from ..config import NeburaxConfig, register_architecture
from ..parts import BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, PartSpec

DECAY_SCALE = 8.0        # log a = -8 r softplus(lam): fixed by the design


def _state_space(W: int, m: dict, eps: float, p: str) -> PartSpec:
    return PartSpec("mixer", "state_space",
                    dict(hidden=W, heads=m["heads"], head_size=m["vdim"], state=m["state"], groups=m["groups"],
                         norm_groups=m["norm_groups"], taps=m["conv"], eps=eps),
                    {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
                     "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "o": p + "o"})


def _side_by_side(W: int, m: dict, eps: float, p: str) -> PartSpec:
    a, r = m["left"], m["right"]
    left = PartSpec("mixer", "attention",
                    dict(hidden=W, n_q=a["heads"], n_kv=a["kv_heads"], head_dim=a["dim"], scale=float(a["scale"]),
                         v_dim=a["vdim"], qk_norm="whole", eps=eps, chunk=(a.get("mask") or {}).get("size")),
                    {n: f"{p}left.{n}" for n in ("q", "k", "v", "o")} | {"q_norm": p + "left.q.norm",
                                                                        "k_norm": p + "left.k.norm"})
    q = p + "right."
    right = PartSpec("mixer", "gated_recurrence",
                     dict(hidden=W, width=r["width"], blocks=r["blocks"], taps=r["conv"], decay_scale=DECAY_SCALE),
                     {"y": q + "y", "y_bias": q + "y.b", "x": q + "x", "x_bias": q + "x.b", "conv": q + "conv",
                      "conv_bias": q + "conv.b", "ra": q + "ra", "ra_bias": q + "ra.b", "ri": q + "ri",
                      "ri_bias": q + "ri.b", "lam": q + "lam", "o": q + "o"})
    return PartSpec("mixer", "side_by_side", dict(left=left, right=right, left_scale=float(m["left_scale"]),
                                                  right_scale=float(m["right_scale"])))


def _feedforward(W: int, mlp: dict, p: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("feedforward", "dense", dict(hidden=W, inter=mlp["ff"], activation="relu2", bias=True),
                        {"up": p + "up", "up_bias": p + "up.b", "down": p + "down", "down_bias": p + "down.b"})
    router = mlp["router"]
    n, ident = router["experts"], router.get("identity") or 0
    names = {"router": p + "router", "correction": p + "correction"}
    for e in range(n):
        for mat in ("gate", "up", "down"):
            names[f"e{e}.{mat}"] = f"{p}e{e}.{mat}"
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("feedforward", "gated", dict(hidden=W, inter=mlp["shared"]["ff"], activation="silu"),
                          {mat: f"{p}shared.{mat}" for mat in ("gate", "up", "down")})
    return PartSpec("feedforward", "routed_experts",
                    dict(hidden=W, inter=mlp["expert"]["ff"], experts=n, top=router["top"], activation="silu",
                         scale_input=False, router="softmax", correction=True, gated=True, identity=ident,
                         shared=shared), names)


def neburax_layout(cfg: NeburaxConfig) -> ModelLayout:
    W, eps = cfg.width, cfg.eps

    def norm(name: str) -> PartSpec:
        return PartSpec("norm", "rmsnorm", dict(size=W, eps=eps, offset=0.0), {"weight": name})

    blocks, block_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if cfg.owner(i) != i:
            continue
        p = f"l{i}."
        m = layer["mixer"]
        mixer = _state_space(W, m, eps, p + "mix.") if layer["type"] == "mamba2" else _side_by_side(W, m, eps, p + "mix.")
        mlp = layer.get("mlp")
        more = {"entry": PartSpec("norm", "cast", dict(size=W))}
        block_of[i] = len(blocks)
        blocks.append(BlockSpec(kind="postnorm", mixer=mixer, post_mixer_norm=norm(p + "norm1"),
                                feedforward=_feedforward(W, mlp, p + "mlp.") if mlp is not None else None,
                                post_ffn_norm=norm(p + "norm2") if mlp is not None else None, more=more))
    return ModelLayout(
        embedding=EmbeddingSpec("embed", cfg.vocab, W, scale=1.0),
        blocks=blocks,
        schedule=[LayerCall(block_of[cfg.owner(i)]) for i in range(len(cfg.layers))],
        final_norm=norm("final.norm"),
        head=HeadSpec("head", tied_to="embed"))


register_architecture(NeburaxConfig, neburax_layout)

"""Banevik, restated plainly: one function per mechanism, whole sequences, float64 torch on the CPU.

Nothing here is shared with the framework.  A model is (config dict, {tensor name: tensor}).
Notation: T tokens, D width, H heads, dn / dr unrotated / rotated query-key sizes, dv value size,
R latent size, E experts.

    embedding      x_t = embed[tok_t] + bigram[(tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets]
                   (t = 0: the table's last row, number ``buckets``)
    norm           n(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w)
    layer          x <- x + mixer(n(x; norm1)) + ff(n(x; norm2))        (ff absent: the mixer alone)
    loop           layers start..stop-1 run ``times`` times; before each run  x <- W_in [x; x0]
    latent mixer   q = Wq h  ->  per head [qn (dn) | qr (dr)];  Wdkv h -> [a (R) | kr (dr)]
                   c = a / sqrt(mean(a^2) + eps) * g;  kn_h = Wuk_h c;  v_h = Wuv_h c
                   s_ij = (qn_i . kn_j + rot(qr_i, i) . rot(kr_j, j)) * scale   for 0 <= i - j < window
                   p_ij = exp(s_ij) / (exp(sink_h) + sum_j exp(s_ij));   o_i = sum_j p_ij v_j;   y = Wo [o_1 .. o_H]
    experts        z = Wr h; s = sigmoid(z); the ``top`` largest s; y = sum_e Wdown_e relu(Wup_e (s_e h))^2
    output         logits = cap * tanh(embed n(x; final.norm) / cap)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def embed(config, w, tokens):
    """Token rows plus the rows of the bigram table."""
    bg = (config.get("embedding") or {}).get("bigram")
    if bg is None:
        return torch.stack([w["embed"][tok].to(F) for tok in tokens])
    rows = []
    for t, tok in enumerate(tokens):
        if t == 0:
            row = bg["buckets"]
        else:
            row = (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]
        rows.append(w["embed"][tok].to(F) + w["bigram"][row].to(F))
    return torch.stack(rows)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, weight, eps):
    return rms(x, eps) * (1.0 + weight.to(F))


def rotate(x, positions, base, dims):
    """x [T, n]: the first ``dims`` entries turn as pairs (i, i + dims/2) by position * base^(-2i/dims); the rest pass."""
    if dims == 0:
        return x.clone()
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = torch.tensor(list(positions), dtype=F)[:, None] * freq[None, :]
    u, v = x[:, :half], x[:, half:dims]
    return torch.cat([u * a.cos() - v * a.sin(), v * a.cos() + u * a.sin(), x[:, dims:]], dim=1)


def latent_attention(m, w, pre, h, eps):
    """h [T, D] -> [T, D].  ``pre``: the tensors' prefix ('l3.mix.')."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window = (m.get("mask") or {}).get("size")
    q = (h @ w[pre + "q"].to(F).T).view(T, H, dn + dr)
    dkv = h @ w[pre + "dkv"].to(F).T
    c = rms(dkv[:, :R], eps) * w[pre + "dkv.norm"].to(F)
    pos = list(range(T))
    rot = m["rot"]
    kr = rotate(dkv[:, R:], pos, rot["base"], rot["dims"])
    kn = (c @ w[pre + "uk"].to(F).T).view(T, H, dn)
    v = (c @ w[pre + "uv"].to(F).T).view(T, H, dv)
    sink = w[pre + "sink"].to(F)
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        qr = rotate(q[:, hd, dn:], pos, rot["base"], rot["dims"])
        s = (q[:, hd, :dn] @ kn[:, hd].T + qr @ kr.T) * m["scale"]
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            e = torch.exp(s[i, lo:i + 1])
            p = e / (math.exp(float(sink[hd])) + e.sum())
            out[i, hd] = p @ v[lo:i + 1, hd]
    return out.reshape(T, H * dv) @ w[pre + "o"].to(F).T


def experts(m, w, pre, h, margins=None):
    """Routed feed-forward; h [T, D] -> [T, D].  ``pre``: 'l3.mlp.'.  ``margins``: a list that receives, per
    token, how far the last chosen score is above the first one left out, relative to the largest |z|
    (infinite when every expert is chosen): a rounded run may choose otherwise where this is tiny."""
    E, top = m["router"]["experts"], m["router"]["top"]
    z = h @ w[pre + "router"].to(F).T
    s = torch.sigmoid(z)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(s[t], top).indices.tolist()
        if margins is not None:
            zs = torch.sort(z[t], descending=True).values
            margins.append(float("inf") if top == E else float((zs[top - 1] - zs[top]) / z[t].abs().max()))
        for e in chosen:
            x = s[t, e] * h[t]
            u = torch.relu(w[f"{pre}e{e}.up"].to(F) @ x) ** 2
            out[t] += w[f"{pre}e{e}.down"].to(F) @ u
    return out


def layer(config, w, i, x):
    spec = config["layers"][i]
    eps = config["norm"]["eps"]
    if spec["type"] != "latent_attention":
        raise ValueError(f"unknown layer type {spec['type']}")
    y = latent_attention(spec["mixer"], w, f"l{i}.mix.", norm(x, w[f"l{i}.norm1"], eps), eps)
    if spec.get("mlp") is not None:
        y = y + experts(spec["mlp"], w, f"l{i}.mlp.", norm(x, w[f"l{i}.norm2"], eps))
    return x + y


def order(config):
    """The layer runs: (layer number, whether the run opens a pass of the loop)."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    runs += [(i, False) for i in range(loop["stop"], n)]
    return runs


def forward(config, w, tokens, streams=None):
    """Logits [T, vocab] of one sequence; ``streams``: a list that receives the stream after every run."""
    x0 = embed(config, w, tokens)
    x = x0
    for i, opens in order(config):
        if opens:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].to(F).T
        x = layer(config, w, i, x)
        if streams is not None:
            streams.append(x.clone())
    logits = norm(x, w["final.norm"], config["norm"]["eps"]) @ w["embed"].to(F).T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits

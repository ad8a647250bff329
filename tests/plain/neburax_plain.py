"""Neburax restated plainly: whole sequences, float64, one function per mechanism.

Nothing here is shared with the package: the functions take the tensors of a checkpoint by name (a dict
of float64 tensors) and the configuration as the dict config.json holds.  Notation: T tokens, W width,
x the residual stream (T, W).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, taps, bias):
    """u (T, C); taps (C, K), column K-1 weighs the current token; zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out + bias


def chunk_mask(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def chunked_attention(h, t, p, m, eps):
    """Grouped-query attention without positions: scores only inside a chunk of ``mask.size`` places."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = unit_rms(h @ t[p + "q"].T, eps) * t[p + "q.norm"]
    k = unit_rms(h @ t[p + "k"].T, eps) * t[p + "k.norm"]
    v = h @ t[p + "v"].T
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    seen = chunk_mask(T, m["mask"]["size"])
    outs = []
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.cat(outs, dim=-1) @ t[p + "o"].T


def gated_recurrence(h, t, p, m):
    """Two branches: a gelu gate, and a convolved branch that drives a diagonal recurrence whose decay
    and input gate come from block-diagonal products of the branch itself."""
    T = h.shape[0]
    nb, width = m["blocks"], m["width"]
    y = gelu_tanh(h @ t[p + "y"].T + t[p + "y.b"])
    u = causal_conv(h @ t[p + "x"].T + t[p + "x.b"], t[p + "conv"], t[p + "conv.b"])
    ub = u.view(T, nb, width // nb)
    r = torch.sigmoid(torch.einsum("bok,tbk->tbo", t[p + "ra"], ub) + t[p + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("bok,tbk->tbo", t[p + "ri"], ub) + t[p + "ri.b"]).reshape(T, width)
    log_a = -8.0 * r * softplus(t[p + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    s = torch.zeros(width, dtype=h.dtype)
    states = []
    for n in range(T):
        s = a[n] * s + drive[n]
        states.append(s)
    return (torch.stack(states) * y) @ t[p + "o"].T


def parallel_mixer(h, t, p, m, eps):
    left = chunked_attention(h, t, p + "left.", m["left"], eps)
    right = gated_recurrence(h, t, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def state_space(h, t, p, m, eps):
    """A selective state space per head: S <- decay S + dt B x^T, y = S^T C + D x."""
    T = h.shape[0]
    nh, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = nh * dv
    proj = h @ t[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, t[p + "conv"], t[p + "conv.b"]))
    x = xbc[:, :inner].view(T, nh, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + t[p + "dt_bias"])
    decay = torch.exp(-torch.exp(t[p + "A_log"]) * dt)          # (T, nh)
    ys = torch.zeros(T, nh, dv, dtype=h.dtype)
    for head in range(nh):
        g = head // (nh // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for n in range(T):
            S = decay[n, head] * S + dt[n, head] * torch.outer(B[n, g], x[n, head])
            ys[n, head] = S.T @ C[n, g] + t[p + "D"][head] * x[n, head]
    y = ys.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


def dense_ff(h, t, p):
    a = torch.relu(h @ t[p + "up"].T + t[p + "up.b"]) ** 2
    return a @ t[p + "down"].T + t[p + "down.b"]


def gated_ff(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def mixture_ff(h, t, p, mlp, choices=None):
    """``choices``: if a list is given, the chosen experts of every token are appended to it."""
    n_real, n_id, top = mlp["router"]["experts"], mlp["router"].get("identity", 0), mlp["router"]["top"]
    s = torch.softmax(h @ t[p + "router"].T, dim=-1)              # over real and identity experts alike
    pick = torch.topk(s + t[p + "correction"], top, dim=-1).indices
    w = torch.gather(s, 1, pick)
    w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    if choices is not None:
        choices.append((pick, s + t[p + "correction"]))
    out = torch.zeros_like(h)
    for e in range(n_real + n_id):
        hit = pick == e
        rows = hit.any(dim=-1)
        if not rows.any():
            continue
        we = (w * hit).sum(dim=-1, keepdim=True)[rows]
        ye = gated_ff(h[rows], t, f"{p}e{e}.") if e < n_real else h[rows]
        out[rows] = out[rows] + we * ye
    if mlp.get("shared") is not None:
        out = out + gated_ff(h, t, p + "shared.")
    return out


def forward(config, tensors, tokens, streams=None, choices=None):
    """Logits (T, vocab) of one sequence that starts at position 0.  ``streams``: a list that receives the
    residual stream after every layer run."""
    t = {k: v.to(F64) if v.is_floating_point() else v for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        m = layer["mixer"]
        if layer["type"] == "parallel":
            y = parallel_mixer(x, t, p + "mix.", m, eps)
        elif layer["type"] == "mamba2":
            y = state_space(x, t, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + unit_rms(y, eps) * t[p + "norm1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, t, p + "mlp.") if mlp["kind"] == "dense" else mixture_ff(x, t, p + "mlp.", mlp, choices)
            x = x + unit_rms(y, eps) * t[p + "norm2"]
        if streams is not None:
            streams.append(x.clone())
    return (unit_rms(x, eps) * t["final.norm"]) @ t["embed"].T

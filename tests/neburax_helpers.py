"""Shared by the Neburax tests: small configurations that differ from one another in every size and option,
model folders with random weights, and the oracle's view of them."""
from __future__ import annotations

import json
import os

import torch

import brolm_b200 as bb


def ssm(heads, vdim, state, groups, norm_groups, conv, mlp=None, **more):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups,
                                          conv=conv), mlp=mlp, **more)


def pair(heads, kv_heads, dim, vdim, scale, chunk, width, blocks, conv, ls, rs, mlp=None, **more):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask=dict(size=chunk))
    return dict(type="parallel", mixer=dict(left=left, right=dict(width=width, blocks=blocks, conv=conv),
                                            left_scale=ls, right_scale=rs), mlp=mlp, **more)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, identity=0, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, identity=identity))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


# S: every routed layer uses all of its experts (identity ones included), so nothing hangs on a discrete choice and a
# rounded run can be held against the oracle.  A layer that runs another's tensors; a layer without a feed-forward; a
# chunk far below a page (9); a state size that is no power of two (12) with three norm groups; five taps.
CFG_S = dict(
    architecture="Neburax", vocab=96, width=48, norm=dict(eps=1e-5),
    layers=[pair(4, 2, 8, 16, 0.3, 9, 32, 2, 4, 0.7, 1.3, mlp=dense(40)),
            ssm(4, 8, 16, 2, 1, 2, mlp=moe(24, 3, 4, identity=1, shared=16)),
            pair(4, 2, 8, 16, 0.3, 9, 32, 2, 4, 0.7, 1.3, mlp=dense(40), weights_of=0),
            ssm(2, 24, 12, 1, 3, 5)])

# T: real routing (2 of 5 + 2 identity, 1 of 4), a chunk of one page exactly (64) and one across a page border (70),
# as many key heads as query heads, key and value heads of one size, head sizes that are no multiples of 8, one block, a convolution of one tap (no kept
# inputs), no shared expert, no identity experts, sizes that are no multiples of 16.
CFG_T = dict(
    architecture="Neburax", vocab=50, width=40, norm=dict(eps=1e-6),
    layers=[ssm(5, 8, 40, 5, 5, 3, mlp=moe(20, 5, 2, identity=2)),
            pair(3, 3, 24, 24, 0.2, 64, 40, 1, 1, 1.0, 0.5, mlp=moe(36, 4, 1)),
            pair(6, 1, 12, 6, 0.25, 70, 24, 3, 2, 1.5, 1.0, mlp=dense(56))])

# U: one layer run three times, each run with a state of its own; a chunk of one (a token sees itself alone) and,
# in another layer, a chunk longer than any prompt of the tests; a router with identity experts only; two layers whose
# key and value heads have one size that is a multiple of 16 (in bfloat16 their attention runs on the tensor cores).
CFG_U = dict(
    architecture="Neburax", vocab=64, width=32, norm=dict(eps=1e-5),
    layers=[pair(2, 1, 16, 32, 0.35, 1, 16, 4, 3, 0.9, 1.1, mlp=moe(16, 0, 2, identity=2, shared=24)),
            pair(2, 1, 16, 32, 0.35, 1, 16, 4, 3, 0.9, 1.1, mlp=moe(16, 0, 2, identity=2, shared=24), weights_of=0),
            ssm(1, 32, 64, 1, 2, 4, mlp=dense(16)),
            pair(2, 1, 16, 32, 0.35, 1, 16, 4, 3, 0.9, 1.1, mlp=moe(16, 0, 2, identity=2, shared=24), weights_of=0),
            pair(4, 2, 16, 16, 0.5, 1000, 48, 2, 2, 1.0, 1.0),
            pair(2, 2, 32, 32, 0.3, 40, 32, 2, 2, 1.0, 1.0, mlp=dense(24))])

CONFIGS = {"S": (CFG_S, 3, 0.15), "T": (CFG_T, 4, 0.2), "U": (CFG_U, 5, 0.2)}      # name -> (config, seed, weight std)


def make_folder(tmp_path, name: str, store=torch.float32) -> str:
    cfg, seed, std = CONFIGS[name]
    folder = os.path.join(str(tmp_path), f"neburax_{name}_{str(store).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        bb.write_random_model(bb.NeburaxConfig.from_dict(cfg), folder, seed=seed, weight_std=std, norm_std=0.5,
                              dtype=store)
    return folder


def oracle_inputs(folder: str):
    """(config dict, {name: tensor}) read without the framework's own reader."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        config = json.load(fh)
    return config, load_file(os.path.join(folder, "model.safetensors"))


def random_prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]

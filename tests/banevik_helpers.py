"""Shared by the Banevik tests: small configurations that differ from one another in every size and
option, model folders with random weights, and the oracle's view of them."""
from __future__ import annotations

import json
import os

import torch

import brolm_b200 as bb


def _layer(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims, window, ff=None, experts=None, top=None):
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                 rot=dict(base=base, dims=dims))
    if window is not None:
        mixer["mask"] = dict(size=window)
    mlp = None
    if ff is not None:
        mlp = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    return dict(type="latent_attention", mixer=mixer, mlp=mlp)


# P: every routed layer uses all of its experts, so no result hangs on a discrete choice and a rounded
# (bfloat16) run can be held against the oracle.  A looped span that does not start at layer 0 and runs three
# times; a layer without a feed-forward; a layer without a window; rotated sizes below the rotated part;
# a window that crosses a page border (70) and one far below a page (9).
CFG_P = dict(
    architecture="Banevik", vocab=96, width=48,
    embedding=dict(bigram=dict(buckets=31, mul_prev=5, mul_cur=3)),
    layers=[_layer(3, 8, 16, 24, 24, 0.2, 100.0, 8, 9, ff=40, experts=2, top=2),
            _layer(2, 16, 8, 8, 40, 0.3, 10000.0, 8, 70),
            _layer(5, 8, 8, 16, 16, 0.25, 500.0, 8, None, ff=24, experts=3, top=3)],
    loop=dict(start=1, stop=3, times=3), norm=dict(eps=1e-5), logit_softcap=12.0)

# Q: real routing (2 of 5, 1 of 4), more heads than a tensor-core decode tile has rows (18), sizes that are
# no multiples of 8, no loop, a window of one page exactly and a window of 1 (a token sees itself alone).
CFG_Q = dict(
    architecture="Banevik", vocab=50, width=40,
    embedding=dict(bigram=dict(buckets=7, mul_prev=11, mul_cur=1)),
    layers=[_layer(18, 6, 4, 10, 12, 0.4, 50.0, 4, 64, ff=20, experts=5, top=2),
            _layer(4, 12, 12, 4, 20, 0.15, 1000.0, 6, 1, ff=36, experts=4, top=1),
            _layer(1, 24, 8, 32, 56, 0.2, 300.0, 8, 5)],
    loop=None, norm=dict(eps=1e-6), logit_softcap=0.0)

# R: the whole model is the looped span, twice; one layer.
CFG_R = dict(
    architecture="Banevik", vocab=64, width=32,
    embedding=dict(bigram=dict(buckets=13, mul_prev=3, mul_cur=2)),
    layers=[_layer(4, 8, 8, 8, 16, 0.35, 20.0, 8, 17, ff=16, experts=3, top=3)],
    loop=dict(start=0, stop=1, times=2), norm=dict(eps=1e-5), logit_softcap=8.0)

CONFIGS = {"P": (CFG_P, 3, 0.15), "Q": (CFG_Q, 4, 0.2), "R": (CFG_R, 5, 0.2)}      # name -> (config, seed, weight std)


def make_folder(tmp_path, name: str, store=torch.float32) -> str:
    cfg, seed, std = CONFIGS[name]
    folder = os.path.join(str(tmp_path), f"banevik_{name}_{str(store).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        bb.write_random_model(bb.BanevikConfig.from_dict(cfg), folder, seed=seed, weight_std=std, norm_std=0.3,
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

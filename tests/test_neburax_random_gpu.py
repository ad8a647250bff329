"""Neburax models drawn at random (layer order, every size, taps, chunks, experts, shared layers) through the engine in
float32 against the plain implementation: a prompt step of three unequal requests, twelve tokens one by one, and the
same once more on the slots, pages and states that were given back.  The bar of a request is the larger of 2e-5 and
eight times the error the plain implementation itself makes when it runs in float32 (a drawn model may norm a vector
of two numbers that are both near zero; no arithmetic in 32 bits gets that to 2e-5)."""
import os
import random

import pytest
import torch

import brolm_b200 as bb
from tests.neburax_helpers import dense, moe, oracle_inputs, pair, random_prompts, ssm
from tests.plain import neburax_plain as plain

pytestmark = pytest.mark.gpu


def draw_mlp(rng):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return dense(rng.choice([8, 20, 48, 130]))
    experts, ident = rng.choice([1, 2, 3, 6, 9]), rng.choice([0, 0, 1, 3])
    return moe(rng.choice([8, 12, 40, 72]), experts, rng.randint(1, min(experts + ident, 4)), identity=ident,
               shared=rng.choice([None, 8, 56]))


def draw_layer(rng):
    if rng.random() < 0.5:
        groups = rng.choice([1, 2, 3])
        heads = groups * rng.choice([1, 2, 3])
        vdim = rng.choice([4, 6, 8, 20, 32, 64])
        norm_groups = rng.choice([g for g in (1, 2, 3, 4, 6) if (heads * vdim) % g == 0])
        return ssm(heads, vdim, rng.choice([2, 5, 12, 16, 24, 48, 64, 100, 128]), groups, norm_groups,
                   rng.choice([1, 2, 3, 4, 6]), mlp=draw_mlp(rng))
    kv = rng.choice([1, 2, 3])
    d = rng.choice([4, 6, 8, 16, 20, 32, 64])
    blocks = rng.choice([1, 2, 3, 4])
    return pair(kv * rng.choice([1, 2, 4]), kv, d, rng.choice([d, d, 4, 8, 12, 32, 128]), rng.choice([0.1, 0.3, 1.0]),
                rng.choice([1, 2, 7, 31, 64, 65, 100, 128, 129, 500]), blocks * rng.choice([1, 5, 8, 16, 48]), blocks,
                rng.choice([1, 2, 3, 4, 5]), rng.choice([0.5, 1.0, 1.7]), rng.choice([0.6, 1.0, 1.2]), mlp=draw_mlp(rng))


def draw_config(seed):
    rng = random.Random(seed)
    layers = [draw_layer(rng) for _ in range(rng.randint(1, 5))]
    for i in range(1, len(layers)):
        j = rng.randrange(0, i)
        if rng.random() < 0.3 and "weights_of" not in layers[j]:
            layers[i] = dict(layers[j], weights_of=j)
    return dict(architecture="Neburax", vocab=rng.choice([37, 64, 200, 577]), width=rng.choice([24, 40, 72, 136, 320]),
                norm=dict(eps=rng.choice([1e-5, 1e-6])), layers=layers)


@pytest.mark.parametrize("seed", range(16))
def test_a_drawn_model_prompt_decode_and_the_same_again(tmp_path, seed):
    folder = os.path.join(str(tmp_path), "drawn")
    bb.write_random_model(bb.NeburaxConfig.from_dict(draw_config(seed)), folder, seed=seed, weight_std=0.15, norm_std=0.5,
                          dtype=torch.float32)
    config, weights = oracle_inputs(folder)
    rng = random.Random(seed + 1000)
    lens = [rng.choice([1, 2, 17, 40, 66, 130, 200]) for _ in range(3)]
    reqs = random_prompts(config["vocab"], [n + 12 for n in lens], seed)
    refs = [plain.forward(config, weights, p) for p in reqs]
    plain.F64 = torch.float32
    try:
        own = [float((plain.forward(config, weights, p).double() - r).abs().max() / r.abs().max()) for p, r in zip(reqs, refs)]
    finally:
        plain.F64 = torch.float64
    bars = [max(2e-5, 8 * e) for e in own]
    eng = bb.Engine(bb.load_model(folder, dtype="float32"), max_tokens=1024, max_slots=3)
    rounds = []
    for _ in range(2):
        slots = eng.open(3)
        got = [[] for _ in reqs]
        first = eng.step(slots, [p[:n] for p, n in zip(reqs, lens)], want=[list(range(n)) for n in lens])
        at = 0
        for b, n in enumerate(lens):
            got[b].append(first[at:at + n].clone())
            at += n
        for j in range(12):
            out = eng.step(slots, [[p[n + j]] for p, n in zip(reqs, lens)])
            for b in range(3):
                got[b].append(out[b:b + 1].clone())
        eng.close(slots)
        rounds.append([torch.cat(g).cpu() for g in got])
    for b, (r, bar) in enumerate(zip(refs, bars)):
        err = float((rounds[0][b].double() - r).abs().max() / r.abs().max())
        assert err <= bar, f"request {b} of {lens[b]} + 12 tokens: {err:.2e} against a bar of {bar:.1e}"
        assert torch.equal(rounds[0][b], rounds[1][b]), "the second tenants of the slots see something of the first"

"""Banevik without a GPU: configuration, layout, tensor names, the oracle's own consistency."""
import copy
import json
import os

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.config import ConfigError
from tests.banevik_helpers import CFG_P, CFG_Q, CFG_R, make_folder, oracle_inputs
from tests.plain import banevik_plain as plain


def test_config_is_chosen_by_its_architecture_key(tmp_path):
    path = os.path.join(str(tmp_path), "config.json")
    with open(path, "w") as fh:
        json.dump(CFG_P, fh)
    cfg = bb.load_config(path)
    assert isinstance(cfg, bb.BanevikConfig) and cfg.width == 48 and len(cfg.layers) == 3
    again = bb.BanevikConfig.from_dict(cfg.to_dict())
    assert again == cfg


def test_runs_follow_the_loop():
    assert bb.BanevikConfig.from_dict(CFG_P).runs() == [(0, False), (1, True), (2, False), (1, True), (2, False),
                                                        (1, True), (2, False)]
    assert bb.BanevikConfig.from_dict(CFG_Q).runs() == [(0, False), (1, False), (2, False)]
    assert bb.BanevikConfig.from_dict(CFG_R).runs() == [(0, True), (0, True)]
    assert plain.order(CFG_P) == bb.BanevikConfig.from_dict(CFG_P).runs()


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
])
def test_bad_configurations_are_named(edit, what):
    c = copy.deepcopy(CFG_P)
    edit(c)
    with pytest.raises(ConfigError) as e:
        bb.BanevikConfig.from_dict(c)
    assert what.split(".")[-1] in str(e.value)


def test_layout_names_and_caches():
    m = bb.Model(bb.BanevikConfig.from_dict(CFG_P), dtype="float32", device="cpu")
    names = m.expected_tensors()
    for n in ("embed", "bigram", "loop.in", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv",
              "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o", "l0.mlp.router", "l0.mlp.e1.up",
              "l2.mlp.e2.down", "l1.norm1"):
        assert n in names, n
    assert "l1.norm2" not in names and "l1.mlp.router" not in names          # a layer without a feed-forward
    assert names["bigram"].shape == (32, 48) and names["loop.in"].shape == (48, 96)
    assert names["l0.mix.q"].shape == (3 * 24, 48) and names["l0.mix.dkv"].shape == (24 + 16, 48)
    assert names["l2.mix.uv"].shape == (5 * 16, 16) and names["l2.mix.sink"].shape == (5,)
    specs = m.cache_specs()
    assert len(specs) == 7                                                   # every run has a cache of its own
    assert specs[0].head_dim == 48 and specs[0].window == 9 and not specs[0].values
    assert specs[2].window is None and specs[1] == specs[3] == specs[5]
    # no loop: no entry matrix
    q = bb.Model(bb.BanevikConfig.from_dict(CFG_Q), dtype="float32", device="cpu")
    assert "loop.in" not in q.expected_tensors() and not q.layout.stream_parts


def test_oracle_token_by_token_equals_whole(tmp_path):
    """The oracle itself: a prefix's logits do not depend on what follows (causality), the window hides what
    it should, and the sink takes weight away."""
    config, w = oracle_inputs(make_folder(tmp_path, "P"))
    toks = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(config, w, toks)
    part = plain.forward(config, w, toks[:23])
    assert float((whole[:23] - part).abs().max()) < 1e-9
    m = dict(config["layers"][0]["mixer"])
    h = torch.randn(30, config["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    a = plain.latent_attention(m, w, "l0.mix.", h, 1e-5)
    h2 = h.clone()
    h2[:10] += 1.0                                       # tokens 0..9: out of a window of 9 from position 18 on
    b = plain.latent_attention(m, w, "l0.mix.", h2, 1e-5)
    assert float((a[18:] - b[18:]).abs().max()) < 1e-12 and float((a[17] - b[17]).abs().max()) > 1e-9
    w2 = dict(w)
    w2["l0.mix.sink"] = w["l0.mix.sink"] + 50.0          # the sink swallows everything
    assert float(plain.latent_attention(m, w2, "l0.mix.", h, 1e-5).abs().max()) < 1e-12

"""Neburax without a GPU: configuration, layout, tensor names, what the cache keeps, the oracle's own consistency."""
import copy
import json
import os

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.cache import Cache, CacheEntries, KVSpec, StateSpec
from brolm_b200.config import ConfigError
from tests.neburax_helpers import CFG_S, CFG_T, CFG_U, make_folder, oracle_inputs
from tests.plain import neburax_plain as plain


def test_config_is_chosen_by_its_architecture_key(tmp_path):
    path = os.path.join(str(tmp_path), "config.json")
    with open(path, "w") as fh:
        json.dump(CFG_S, fh)
    cfg = bb.load_config(path)
    assert isinstance(cfg, bb.NeburaxConfig) and cfg.width == 48 and len(cfg.layers) == 4
    assert bb.NeburaxConfig.from_dict(cfg.to_dict()) == cfg
    assert [cfg.owner(i) for i in range(4)] == [0, 1, 0, 3]


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][3]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "kind"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][3].update(weights_of=2), "weights_of"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_are_named(edit, what):
    c = copy.deepcopy(CFG_S)
    edit(c)
    with pytest.raises(ConfigError) as e:
        bb.NeburaxConfig.from_dict(c)
    assert what in str(e.value)


def test_layout_names_and_caches():
    m = bb.Model(bb.NeburaxConfig.from_dict(CFG_S), dtype="float32", device="cpu")
    names = m.expected_tensors()
    for n in ("embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.left.q", "l0.mix.left.q.norm", "l0.mix.left.k.norm",
              "l0.mix.left.o", "l0.mix.right.y.b", "l0.mix.right.conv.b", "l0.mix.right.ra", "l0.mix.right.ri.b",
              "l0.mix.right.lam", "l0.mlp.up.b", "l0.mlp.down.b", "l1.mix.in", "l1.mix.conv", "l1.mix.dt_bias",
              "l1.mix.A_log", "l1.mix.D", "l1.mix.norm", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e2.gate",
              "l1.mlp.shared.down", "l3.mix.o"):
        assert n in names, n
    assert not any(n.startswith("l2.") for n in names)                  # a layer that runs another's tensors has none
    assert "l3.norm2" not in names and "l1.mlp.e3.up" not in names       # no feed-forward; identity experts have none
    assert names["l0.mix.left.q"].shape == (32, 48) and names["l0.mix.left.v"].shape == (32, 48)
    assert names["l0.mix.left.o"].shape == (48, 64) and names["l0.mix.left.k.norm"].shape == (16,)
    assert names["l0.mix.right.ra"].shape == (2, 16, 16) and names["l0.mix.right.conv"].shape == (32, 4)
    assert names["l1.mix.in"].shape == (2 * 32 + 2 * 2 * 16 + 4, 48) and names["l1.mix.conv"].shape == (32 + 64, 2)
    assert names["l1.mlp.router"].shape == (4, 48) and names["l1.mlp.correction"].shape == (4,)
    assert [c.block for c in m.layout.schedule] == [0, 1, 0, 2]
    specs = m.cache_specs()
    assert specs[0] == specs[2] and isinstance(specs[0], tuple)           # runs 0 and 2: equal needs, places of their own
    kv, st = specs[0]
    assert kv == KVSpec(2, 8, None, True, 16, 9) and st == StateSpec((32 * 4,), torch.float32)
    assert specs[1] == StateSpec((4 * 8 * 16 + 1 * (32 + 64),), torch.float32)
    assert specs[3] == StateSpec((2 * 24 * 12 + 4 * (48 + 24),), torch.float32)


def test_a_tuple_of_specs_gives_one_entry_per_spec():
    kv, st = KVSpec(2, 8, None, True, 16, 70), StateSpec((10,), torch.float32)
    c = Cache([(kv, st), st, (kv, st), None], max_tokens=640, dtype=torch.float32, device="cpu", max_slots=2)
    e0, e2 = c.entries[0], c.entries[2]
    assert isinstance(e0, CacheEntries) and len(e0.parts) == 2 and c.entries[3] is None
    assert e0.parts[0].group is e2.parts[0].group and (e0.parts[0].index, e2.parts[0].index) == (0, 1)
    assert e0.parts[1].group is c.entries[1].group and sorted([e0.parts[1].index, c.entries[1].index, e2.parts[1].index]) == [0, 1, 2]
    g = c.kv_groups[0]
    assert g.ring == 128 and g.pool.num_pages == 4                         # a chunk of 70 is kept like a window of 70
    assert tuple(g.k.shape) == (2, 4, 2, 64, 8) and tuple(g.v.shape) == (2, 4, 2, 64, 16)
    s = c.alloc_slot()
    c.reserve({s: 500})
    assert len(g.pages[s]) == 2
    c.state_groups[0].data[:, s] = 1.0
    c.free_slot(s)
    assert c.alloc_slot() == s and float(c.state_groups[0].data[:, s].abs().max()) == 0.0      # zero again for the next tenant


def test_oracle_is_causal_and_its_parts_do_what_they_say(tmp_path):
    config, w = oracle_inputs(make_folder(tmp_path, "S"))
    w = {k: v.double() for k, v in w.items()}
    toks = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(config, w, toks)
    part = plain.forward(config, w, toks[:23])
    assert float((whole[:23] - part).abs().max()) < 1e-9
    # the chunk of 9: position 20 (chunk 18..26) sees 18, 19, 20 and nothing before
    m = config["layers"][0]["mixer"]["left"]
    h = torch.randn(30, config["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    a = plain.chunked_attention(h, w, "l0.mix.left.", m, 1e-5)
    h2 = h.clone()
    h2[:18] += 1.0
    b = plain.chunked_attention(h2, w, "l0.mix.left.", m, 1e-5)
    assert float((a[18:] - b[18:]).abs().max()) < 1e-12 and float((a[17] - b[17]).abs().max()) > 1e-9
    # the first token of a chunk sees itself alone: its result is its own value through W_o
    v = (h @ w["l0.mix.left.v"].T).view(30, 2, 16)
    want = torch.cat([v[18, hd // 2] for hd in range(4)]) @ w["l0.mix.left.o"].T
    assert float((a[18] - want).abs().max()) < 1e-12
    # the convolution: the last column weighs the token itself, nothing comes from before the start
    taps = torch.tensor([[0.0, 0.0, 2.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    u = torch.arange(1.0, 9.0, dtype=torch.float64).view(4, 2)
    got = plain.causal_conv(u, taps, torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert got[:, 0].tolist() == [2.5, 6.5, 10.5, 14.5] and got[:, 1].tolist() == [0.0, 0.0, 2.0, 4.0]
    # identity experts alone, two of two chosen: the weights sum to one and the result is the input
    cu, wu = oracle_inputs(make_folder(tmp_path, "U"))
    wu = {k: v.double() for k, v in wu.items()}
    mlp = dict(cu["layers"][0]["mlp"], shared=None)
    x = torch.randn(7, cu["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    assert float((plain.mixture_ff(x, wu, "l0.mlp.", mlp) - x).abs().max()) < 1e-12


def test_state_space_matches_its_quadratic_form():
    """The recurrence of a head against the same result written as a sum over earlier tokens:
    y_t = sum_{s<=t} (prod_{s<r<=t} decay_r) dt_s (B_s . C_t) x_s + D x_t."""
    g = torch.Generator().manual_seed(4)
    T, W = 12, 16
    m = dict(heads=2, vdim=4, state=6, groups=1, norm_groups=1, conv=1)
    inner, cols = 8, 8 + 12
    t = {"p.in": torch.randn(2 * inner + 12 + 2, W, generator=g, dtype=torch.float64) * 0.3,
         "p.conv": torch.ones(cols, 1, dtype=torch.float64), "p.conv.b": torch.zeros(cols, dtype=torch.float64),
         "p.dt_bias": torch.randn(2, generator=g, dtype=torch.float64), "p.A_log": torch.randn(2, generator=g, dtype=torch.float64),
         "p.D": torch.randn(2, generator=g, dtype=torch.float64), "p.norm": torch.ones(inner, dtype=torch.float64),
         "p.o": torch.eye(inner, dtype=torch.float64)}
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    got = plain.state_space(h, t, "p.", m, 1e-5)
    proj = h @ t["p.in"].T
    z, xbc, dt = proj[:, :inner], plain.silu(proj[:, inner:inner + cols]), plain.softplus(proj[:, inner + cols:] + t["p.dt_bias"])
    x, B, C = xbc[:, :inner].view(T, 2, 4), xbc[:, inner:inner + 6], xbc[:, inner + 6:]
    y = torch.zeros(T, 2, 4, dtype=torch.float64)
    for hd in range(2):
        la = -torch.exp(t["p.A_log"][hd]) * dt[:, hd]
        for a in range(T):
            for s in range(a + 1):
                y[a, hd] += torch.exp(la[s + 1:a + 1].sum()) * dt[s, hd] * (B[s] @ C[a]) * x[s, hd]
            y[a, hd] += t["p.D"][hd] * x[a, hd]
    want = plain.unit_rms(y.reshape(T, inner) * plain.silu(z), 1e-5)
    assert float((got - want).abs().max()) < 1e-10

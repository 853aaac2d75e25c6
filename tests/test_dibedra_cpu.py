"""Host-side parts of the Dibedra design: config.json parsing and validation, the registry, tensor names and shapes, the
page manager's rule for pages a sliding window has left, and the oracle's own mechanisms on hand-made inputs. No GPU."""
import json
import math

import pytest
import torch

import dibedra_cases as K
import dibedra_oracle as O
from livecc_b200 import registry
from livecc_b200.checkpoint import seq_param_specs, synthetic_seq_tensors
from livecc_b200.config import SeqModelConfig
from livecc_b200.kv_cache import PAGE_SIZE, SeqStatePool


@pytest.mark.parametrize("name", sorted(K.CASES))
def test_config_round_trip_and_validation(name):
    d = K.CASES[name]
    cfg = SeqModelConfig.from_json(json.loads(json.dumps(d)))
    cfg.validate()
    assert SeqModelConfig.from_json(cfg.to_json()) == cfg
    assert cfg.block == "parallel" and cfg.norm == "dyt" and cfg.dense == "mlp" and cfg.logit_scale == d["logit_scale"]
    for L, e in zip(cfg.layers, d["layers"]):
        assert L.attn.window == e["mixer"]["mask"]["size"] and L.attn.value_keys and L.attn.gate == "channel" and not L.attn.sink
        assert L.weights_of == e.get("weights_of", -1)
        if e["mlp"] and e["mlp"]["kind"] == "moe":
            r = e["mlp"]["router"]
            assert (L.moe.experts, L.moe.identity, L.moe.top) == (r["experts"], r.get("identity", 0), r["top"])
            assert L.moe.router == "softmax" and L.moe.act == "clamp_glu" and L.moe.limit == e["mlp"]["expert"]["limit"]
            assert (L.moe.groups, L.moe.keep) == ((r["groups"]["count"], r["groups"]["keep"]) if "groups" in r else (0, 0))


def test_random_configurations_are_valid():
    for seed in range(40):
        cfg = SeqModelConfig.from_json(K.random_config(seed))
        cfg.validate()
        assert SeqModelConfig.from_json(cfg.to_json()) == cfg


def test_bad_configurations_are_refused():
    def bad(change):
        d = json.loads(json.dumps(K.CASES["moe"]))
        change(d)
        with pytest.raises((ValueError, NotImplementedError, KeyError)):
            SeqModelConfig.from_json(d).validate()

    bad(lambda d: d["layers"][0]["mixer"].update(kv_heads=2))                      # 3 query heads over 2 key heads
    bad(lambda d: d["layers"][0]["mixer"].update(vdim=12))                         # the values are the keys
    bad(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3))                   # pairs
    bad(lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4))       # 9 outputs in 4 groups
    bad(lambda d: (d["layers"][0]["mlp"]["router"]["groups"].update(keep=1), d["layers"][0]["mlp"]["router"].update(top=4)))   # 3 kept, 4 wanted
    bad(lambda d: d["layers"][1].update(weights_of=1))                             # itself
    bad(lambda d: d["layers"][1].update(weights_of=7))                             # no such layer
    bad(lambda d: d["layers"][0].update(type="mamba3"))


def test_registry_and_tensor_names():
    assert "Dibedra" in registry.architectures()
    d = K.CASES["looped"]
    cfg = SeqModelConfig.from_json(d)
    names = {n: s for n, s, _ in seq_param_specs(cfg)}
    assert names["l0.norm1"] == (32,) and names["l0.norm1.b"] == (32,) and names["l0.norm1.alpha"] == ()
    assert names["l1.mix.q"] == (24, 32) and names["l1.mix.k"] == (12, 32) and names["l1.mix.g"] == (24, 32) and names["l1.mix.o"] == (32, 24)
    assert names["l1.mix.q.norm"] == (6,) and "l1.mix.v" not in names and "l1.norm2" not in names
    assert names["l1.mlp.router"] == (8, 32) and names["l1.mlp.correction"] == (8,) and names["l1.mlp.e5.gate"] == (10, 32)
    assert "l1.mlp.e6.up" not in names                                             # identity experts have no tensors
    assert names["l3.mlp.up"] == (20, 32) and "l3.mlp.gate" not in names
    assert not any(n.startswith(("l2.", "l4.", "l5.")) for n in names)             # layers that run with another layer's weights
    assert names["final.norm.alpha"] == () and names["head"] == (96, 32)
    t = synthetic_seq_tensors(cfg, seed=1)
    assert set(t) == set(names) and all(tuple(t[n].shape) == s for n, s in names.items())


def test_pages_behind_every_window_are_given_back():
    pool = SeqStatePool({0: (1, 8, 8, 0, 70), 1: (2, 4, 4, 0, 20)}, [0, 0], torch.float32, "cpu", initial_pages=8)
    assert pool.keep_from(10) == 0 and pool.keep_from(70) == 1 and pool.keep_from(300) == 231
    assert SeqStatePool({0: (1, 8, 8, 0, 70), 1: (1, 8, 8, 0, 0)}, [0, 0], torch.float32, "cpu").keep_from(300) == 0   # one layer sees everything
    assert SeqStatePool({0: (1, 8, 8, 128, 70)}, [0], torch.float32, "cpu").keep_from(300) == 256                       # chunks and a window
    from livecc_b200.kv_cache import SeqCache

    c = SeqCache(pool)
    c.ensure_tokens(300)
    c.advance(300)
    assert [p is None for p in c.pages] == [True, True, True, False, False] and 231 // PAGE_SIZE == 3
    c.release()
    assert len(pool.free) == pool.num_pages


# ---- the oracle's mechanisms on hand-made inputs ----------------------------------------------------------------------------
def test_oracle_rotation_pairs_neighbours_and_keeps_the_rest():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 1, 12).repeat(3, 1, 1)
    rot = {"dims": 4, "base": 100.0}
    y = O.rotate_pairs(x, rot)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])       # position 0 and the channels past dims
    f = [1.0, 100.0 ** -0.5]
    for i in range(2):
        a = 2 * f[i]
        u, v = x[2, 0, 2 * i], x[2, 0, 2 * i + 1]
        assert abs(y[2, 0, 2 * i] - (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(y[2, 0, 2 * i + 1] - (v * math.cos(a) + u * math.sin(a))) < 1e-12


def test_oracle_long_context_frequencies():
    f, mag = O.pair_frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    plain, one = O.pair_frequencies({"dims": 8, "base": 10000.0})
    assert one == 1.0 and abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert abs(f[0] - plain[0]) < 1e-15 and abs(f[-1] - plain[-1] / 4.0) < 1e-15   # fast pairs kept, slow pairs divided
    assert all(plain[i] / 4.0 - 1e-15 <= f[i] <= plain[i] + 1e-15 for i in range(4))
    from livecc_b200.config import RotaryConfig

    g, m2 = RotaryConfig(8, 10000.0, {"factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}).frequencies()
    assert max(abs(a - float(b)) for a, b in zip(g, f)) < 1e-15 and m2 == mag


def test_oracle_window_and_router():
    q = torch.zeros(5, 1, 2, dtype=torch.float64)
    k = torch.zeros(5, 1, 2, dtype=torch.float64)
    v = torch.arange(5, dtype=torch.float64).reshape(5, 1, 1)
    out = O.window_attention(q, k, v, 1.0, 2)[:, 0, 0]
    assert torch.allclose(out, torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5], dtype=torch.float64))   # the mean of itself and one before
    mlp = {"router": {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 1}}, "expert": {"limit": 1.0}}
    t = {"router": torch.eye(6, dtype=torch.float64)[:, :6] * 3.0, "correction": torch.tensor([0.0, 0.0, 0.0, 0.9, 0.0, 0.0], dtype=torch.float64)}
    h = torch.zeros(1, 6, dtype=torch.float64)
    h[0, 0] = 1.0                                                                  # output 0 has the best score, output 3 the best choice score
    idx, w = O.route(h, mlp, t, "")
    assert sorted(idx[0].tolist()) == [2, 3]                                       # only group 1 = outputs (2, 3) stays
    s = torch.softmax(h @ t["router"].T, -1)[0]
    assert torch.allclose(w[0].sort().values, s[[2, 3]].sort().values)             # weights are the scores, without the correction
    idx, _ = O.route(h, mlp, t, "", use_groups=False)
    assert sorted(idx[0].tolist()) == [0, 3]

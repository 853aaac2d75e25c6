"""Host-side parts of the Lugizen design: config.json parsing and validation, the registry, tensor names and shapes, the
weight layout the library reads, the page manager's rule for pages a latent window has left, and the oracle's own
mechanisms on hand-made inputs. No GPU."""
import json
import math

import pytest
import torch

import lugizen_cases as K
import lugizen_oracle as O
from livecc_b200 import registry
from livecc_b200.checkpoint import seq_param_specs, synthetic_seq_tensors
from livecc_b200.config import SeqModelConfig
from livecc_b200.kv_cache import PAGE_SIZE, SeqCache, SeqStatePool

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(K.CASES))
def test_config_round_trip_and_validation(name):
    d = K.CASES[name]
    cfg = SeqModelConfig.from_json(json.loads(json.dumps(d)))
    cfg.validate()
    assert SeqModelConfig.from_json(cfg.to_json()) == cfg
    assert cfg.block == "branchnorm" and cfg.norm == "rms" and cfg.norm_scalar and cfg.dense == "mlp"
    assert cfg.canon_taps == d.get("canon", {}).get("taps", 0)
    for L, e in zip(cfg.layers, d["layers"]):
        mx = e["mixer"]
        if e["type"] == "channel_delta":
            assert (L.delta.heads, L.delta.kv_heads, L.delta.dim, L.delta.vdim, L.delta.conv) == tuple(mx[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
        elif e["type"] == "attention":
            a = L.attn
            assert a.window == 0 and not a.value_keys and a.gate == "none" and not a.sink and a.unit_norm and a.temp and not a.rot_pairs
            assert a.v_mix == bool(mx.get("v_mix")) and a.rot.dims == mx["rot"]["dims"] and a.scale == mx["scale"]
        else:
            a = L.latent
            assert (a.q_rank, a.window, a.gate, a.sink, a.kv_from) == (mx["q_rank"], mx["mask"]["size"], False, False, -1)
        if e["mlp"] and e["mlp"]["kind"] == "moe":
            r = e["mlp"]["router"]
            assert (L.moe.experts, L.moe.top, L.moe.ff) == (r["experts"], r["top"], e["mlp"]["expert"]["ff"])
            assert L.moe.router == "topk_softmax" and L.moe.act == "silu_glu" and L.moe.shared_ff == 0


def test_random_configurations_are_valid():
    for seed in range(40):
        cfg = SeqModelConfig.from_json(K.random_config(seed))
        cfg.validate()
        assert SeqModelConfig.from_json(cfg.to_json()) == cfg


def test_bad_configurations_are_refused():
    def bad(change, case="mixed"):
        d = json.loads(json.dumps(K.CASES[case]))
        change(d)
        with pytest.raises((ValueError, NotImplementedError, KeyError)):
            SeqModelConfig.from_json(d).validate()

    bad(lambda d: d["layers"][0]["mixer"].update(heads=3, kv_heads=2))             # 3 value heads over 2 key heads
    bad(lambda d: d["layers"][0]["mixer"].update(conv=9))                          # more taps than the kernels keep
    bad(lambda d: d["layers"][1]["mixer"].update(kv_heads=2))                      # 3 query heads over 2 key heads
    bad(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=3))                   # pairs
    bad(lambda d: d["layers"][3]["mixer"].update(vdim=7))                          # mixed values of another shape
    bad(lambda d: d["layers"][2]["mixer"].update(rot_dim=6))                       # rot.dims says 4
    bad(lambda d: d["layers"][1]["mlp"]["router"].update(top=9))                   # 5 experts
    bad(lambda d: d["canon"].update(taps=9))
    bad(lambda d: d["layers"][0].update(type="mamba3"))


def test_registry_and_tensor_names():
    assert "Lugizen" in registry.architectures()
    cfg = SeqModelConfig.from_json(K.CASES["mixed"])
    names = {n: s for n, s, _ in seq_param_specs(cfg)}
    assert names["l0.norm1"] == () and names["l0.norm2"] == () and names["final.norm"] == () and names["l0.canon1"] == (32, 3)
    assert names["l0.mix.q"] == (8, 32) and names["l0.mix.v"] == (12, 32) and names["l0.mix.q.conv"] == (8, 3) and names["l0.mix.v.conv"] == (12, 3)
    assert names["l0.mix.b"] == (2, 32) and names["l0.mix.A_log"] == (2,) and names["l0.mix.a1"] == (5, 32) and names["l0.mix.a2"] == (16, 5)
    assert names["l0.mix.dt_bias"] == (16,) and names["l0.mix.g1"] == (3, 32) and names["l0.mix.g2"] == (12, 3) and names["l0.mix.norm"] == (6,)
    assert names["l0.mlp.up"] == (20, 32) and "l0.mlp.gate" not in names
    assert names["l1.mix.q"] == (24, 32) and names["l1.mix.k"] == (8, 32) and names["l1.mix.v"] == (6, 32) and names["l1.mix.o"] == (32, 18)
    assert names["l1.mix.temp"] == (3,) and names["l1.mix.vmix"] == () and "l1.mix.q.norm" not in names and "l1.mix.g" not in names
    assert names["l1.mlp.router"] == (5, 32) and names["l1.mlp.e4.gate"] == (12, 32) and "l1.mlp.correction" not in names
    assert names["l2.mix.dq"] == (10, 32) and names["l2.mix.dq.norm"] == (10,) and names["l2.mix.uq"] == (20, 10)
    assert names["l2.mix.dkv"] == (16, 32) and names["l2.mix.dkv.norm"] == (12,) and names["l2.mix.uk"] == (12, 12) and names["l2.mix.uv"] == (10, 12)
    assert "l2.mix.q" not in names and "l2.mix.sink" not in names and "l2.mix.g" not in names
    assert "l3.norm2" not in names and names["head"] == (96, 32)
    t = synthetic_seq_tensors(cfg, seed=1)
    assert set(t) == set(names) and all(tuple(t[n].shape) == s for n, s in names.items())
    no_canon = SeqModelConfig.from_json(K.config([K.att(mlp=None)], taps=0))
    assert not any("canon" in n for n, _, _ in seq_param_specs(no_canon))


def test_weight_layout_the_library_reads():
    """Blocks of the delta rule's input projection start at multiples of 8 rows (zero rows between them), the convolution's
    taps follow the same layout, a norm's single number becomes a row of the model's width, and the first layer that mixes
    values is the one that keeps them."""
    from livecc_b200.seq_engine import SeqWeights

    d = K.config([K.lat(mlp=None), K.delta(heads=3, kv_heads=3, dim=5, vdim=3, decay_rank=2, gate_rank=9, mlp=None), K.att(v_mix=True, mlp="moe"),
                  K.att(mlp=None), K.att(v_mix=True, mlp=None)], width=16, vocab=40)
    cfg = SeqModelConfig.from_json(d)
    t = synthetic_seq_tensors(cfg, seed=2)
    w = SeqWeights(cfg, t, torch.float32, "cpu")
    assert not w.unused
    dl = w.layers[1]
    assert dl["d_in"].shape == (16 + 16 + 16 + 8 + 8 + 16, 16) and dl["d_conv_w"].shape == (48, 3)
    assert torch.equal(dl["d_in"][:15], t["l1.mix.q"].float()) and not dl["d_in"][15].any()
    assert torch.equal(dl["d_in"][16:31], t["l1.mix.k"].float()) and torch.equal(dl["d_in"][32:41], t["l1.mix.v"].float())
    assert torch.equal(dl["d_in"][48:51], t["l1.mix.b"].float()) and torch.equal(dl["d_in"][56:58], t["l1.mix.a1"].float())
    assert torch.equal(dl["d_in"][64:73], t["l1.mix.g1"].float()) and not dl["d_in"][73:].any()
    assert torch.equal(dl["d_conv_w"][16:31], t["l1.mix.k.conv"].float()) and not dl["d_conv_w"][41:].any()
    assert w.layers[0]["norm1"].shape == (16,) and bool((w.layers[0]["norm1"] == t["l0.norm1"].float()).all())
    assert [w.layers[i].get("m_vmix_role", 0) for i in (2, 3, 4)] == [1, 0, 2]
    assert abs(w.layers[4]["m_vmix"] - float(t["l4.mix.vmix"])) < 1e-9
    la = w.layers[0]
    assert la["a_in"].shape == (10 + 16 + 6, 16) and torch.equal(la["a_in"][:10], t["l0.mix.dq"].float()) and "a_sink" not in la
    assert w.layers[2]["e_up"].shape == (5, 24, 16) and "e_correction" not in w.layers[2]


def test_pages_behind_a_latent_window_are_given_back():
    pool = SeqStatePool({0: (1, 16, 0, 0, 70), 2: (1, 6, 0, 0, 20)}, [0, 8, 0], torch.float32, "cpu", initial_pages=8)
    assert pool.keep_from(10) == 0 and pool.keep_from(70) == 1 and pool.keep_from(300) == 231
    assert SeqStatePool({0: (1, 16, 0, 0, 70), 1: (2, 8, 4, 0, 0)}, [0, 0], torch.float32, "cpu").keep_from(300) == 0   # plain attention sees everything
    c = SeqCache(pool)
    c.ensure_tokens(300)
    c.advance(300)
    assert [p is None for p in c.pages] == [True, True, True, False, False] and 231 // PAGE_SIZE == 3
    slot = c.slot
    pool.state[1][slot].fill_(3.0)
    c.release()
    assert len(pool.free) == pool.num_pages
    c2 = SeqCache(pool)
    assert c2.slot == slot and not pool.state[1][slot].any()       # a slot that is used again starts from zero
    c2.release()


# ---- the oracle's mechanisms on hand-made inputs ----------------------------------------------------------------------------
def test_oracle_rotation_pairs_halves_and_keeps_the_rest():
    x = torch.arange(12, dtype=F64).reshape(1, 1, 12).repeat(3, 1, 1)
    y = O.rotate_half(x, 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])       # position 0 and the channels past dims
    f = [1.0, 100.0 ** -0.5]
    for i in range(2):
        a = 2 * f[i]
        u, v = x[2, 0, i], x[2, 0, i + 2]                                          # channel i turns with channel i + dims / 2
        assert abs(y[2, 0, i] - (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(y[2, 0, i + 2] - (v * math.cos(a) + u * math.sin(a))) < 1e-12
    assert torch.allclose(O.rotate_half(x, 4, 100.0, start=5)[0], O.rotate_half(x.repeat(2, 1, 1), 4, 100.0)[5])


def test_oracle_convolution_reads_the_current_token_last():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=F64)                                 # the last tap is the current token's
    assert O.time_conv(x, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_oracle_delta_rule_overwrites_what_a_key_held():
    """With decay 1 and beta 1, writing v2 under a unit key that already holds v1 replaces v1; an orthogonal key is untouched;
    the read-out of a token sees its own write; a decay of 0 on every channel forgets everything before the token."""
    e1, e2 = torch.tensor([1.0, 0.0], dtype=F64), torch.tensor([0.0, 1.0], dtype=F64)
    k = torch.stack([e1, e2, e1, e1])
    q = torch.stack([e1, e1, e1, e2])
    v = torch.tensor([[1.0, 2.0], [5.0, 6.0], [7.0, 8.0], [9.0, 9.0]], dtype=F64)
    ones = torch.ones(4, 2, dtype=F64)
    out = O.delta_rule(q, k, v, torch.ones(4, dtype=F64), ones)
    assert out.tolist() == [[1.0, 2.0], [1.0, 2.0], [7.0, 8.0], [5.0, 6.0]]
    half = O.delta_rule(q, k, v, torch.full((4,), 0.5, dtype=F64), ones)
    assert half[2].tolist() == [0.5 * (7.0 - 0.5) + 0.5, 0.5 * (8.0 - 1.0) + 1.0]  # S k = v1 / 2, then half of the difference lands
    dec = ones.clone()
    dec[3] = 0.0
    assert O.delta_rule(q, k, v, torch.ones(4, dtype=F64), dec)[3].tolist() == [0.0, 0.0]


def test_oracle_window_values_and_router():
    q = torch.zeros(5, 1, 2, dtype=F64)
    k = torch.zeros(5, 1, 2, dtype=F64)
    v = torch.arange(5, dtype=F64).reshape(5, 1, 1)
    assert torch.allclose(O.softmax_attention(q, k, v, 1.0, 2)[:, 0, 0], torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5], dtype=F64))
    assert torch.allclose(O.softmax_attention(q, k, v, 1.0)[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0], dtype=F64))
    mlp = {"router": {"experts": 4, "top": 2}}
    t = {"router": torch.eye(4, dtype=F64)}
    h = torch.tensor([[2.0, -1.0, 1.0, 0.0]], dtype=F64)
    idx, w = O.route(h, mlp, t, "")
    assert idx[0].tolist() == [0, 2] and torch.allclose(w[0], torch.softmax(torch.tensor([2.0, 1.0], dtype=F64), 0)) and abs(float(w.sum()) - 1) < 1e-12
    assert O.route(h, mlp, t, "", equal_weights=True)[1][0].tolist() == [0.5, 0.5]
    y = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(O.scalar_norm(y, torch.tensor(2.0, dtype=F64), 0.0), y / math.sqrt(12.5) * 2.0)

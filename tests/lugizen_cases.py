"""Small Lugizen configurations and inputs for the tests (config.json dictionaries; none of them is a served model's
combination of sizes). Sizes are deliberately unequal where a served model might make them equal or 1."""
from __future__ import annotations

import torch


def rot(dims, base=10000.0):
    return {"dims": dims, "base": base}


def moe(experts=5, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def dense(ff=20):
    return {"kind": "dense", "ff": ff}


def _mlp(mlp):
    return dense() if mlp == "dense" else (moe() if mlp == "moe" else mlp)


def delta(heads=2, kv_heads=1, dim=8, vdim=6, conv=3, decay_rank=5, gate_rank=3, mlp="dense"):
    return {"type": "channel_delta", "mlp": _mlp(mlp),
            "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank, gate_rank=gate_rank)}


def att(heads=3, kv_heads=1, dim=8, vdim=6, rot_dims=4, base=300.0, scale=0.3, v_mix=False, mlp="dense"):
    mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot(rot_dims, base), scale=scale)
    if v_mix:
        mx["v_mix"] = True
    return {"type": "attention", "mixer": mx, "mlp": _mlp(mlp)}


def lat(heads=2, dim=6, rot_dim=4, vdim=5, kv_rank=12, q_rank=10, window=9, base=500.0, scale=0.25, mlp="dense"):
    return {"type": "latent_attention", "mlp": _mlp(mlp),
            "mixer": dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, mask={"size": window},
                          rot=rot(rot_dim, base), scale=scale)}


def config(layers, width=24, vocab=80, eps=1e-5, taps=3):
    d = {"architecture": "Lugizen", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if taps:          # 0: the mixers read the residual stream itself
        d["canon"] = {"taps": taps}
    return d


CASES = {
    "delta_only": config([delta(mlp=None), delta(heads=4, kv_heads=4, dim=5, vdim=9, conv=2, mlp=None)]),
    "attention_only": config([att(mlp=None, v_mix=True), att(heads=4, kv_heads=2, dim=6, vdim=6, rot_dims=6, scale=0.5, mlp=None),
                              att(heads=2, kv_heads=1, dim=10, vdim=6, rot_dims=2, v_mix=True, mlp=None),
                              att(heads=1, kv_heads=1, dim=4, vdim=6, rot_dims=0, v_mix=True, mlp=None)], taps=2),
    "latent_only": config([lat(mlp=None), lat(heads=3, dim=4, rot_dim=2, vdim=7, kv_rank=9, q_rank=6, window=70, mlp=None)], taps=4),
    "mixed": config([delta(), att(v_mix=True, mlp="moe"), lat(mlp="moe"), att(heads=2, kv_heads=1, dim=6, rot_dims=6, v_mix=True, mlp=None),
                     delta(heads=3, kv_heads=3, dim=6, vdim=4, conv=4, mlp=moe(experts=3, top=3, ff=9))], width=32, vocab=96),
    "dense": config([delta(), lat(), att(heads=2, kv_heads=2, dim=6, rot_dims=2, mlp=dense(37)), delta(heads=2, kv_heads=2, dim=12, vdim=4, mlp=None)],
                    width=40),
    "moe": config([att(mlp=moe(experts=7, top=3, ff=10)), delta(mlp=moe(experts=3, top=1, ff=20)),
                   lat(mlp=moe(experts=4, top=4, ff=9))], width=24),
    "odd": config([lat(heads=5, dim=10, rot_dim=6, vdim=3, kv_rank=17, q_rank=7, window=129, scale=1.25, mlp=moe(experts=33, top=5, ff=6)),
                   delta(heads=6, kv_heads=2, dim=18, vdim=5, conv=1, decay_rank=2, gate_rank=7, mlp=dense(7)),
                   att(heads=6, kv_heads=2, dim=5, vdim=11, rot_dims=4, mlp=moe(experts=2, top=1, ff=7)),
                   delta(heads=1, kv_heads=1, dim=40, vdim=33, conv=5, mlp=None)], width=18, vocab=50, eps=1e-6, taps=1),
    # a sharp softmax (large score scale) with channels that do not turn: one key can dominate wherever it sits
    "sharp": config([att(heads=2, kv_heads=1, dim=8, vdim=8, rot_dims=4, scale=3.0, mlp=None)], width=16, vocab=64),
    "sharp_latent": config([lat(heads=2, dim=6, rot_dim=4, vdim=5, kv_rank=12, q_rank=10, window=100, scale=0.3, mlp=None)], width=16, vocab=64),
}


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(5000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(seed):
    """A random stack: 2 to 6 layers of the three mixers in any order, head counts and sizes that are and are not multiples of
    8, windows from 1 token to beyond the prompt, rotated parts from none to the whole head, 0 to 5 taps, dense, routed or no
    feed-forward."""
    import random

    rng = random.Random(seed)

    def rmlp():
        x = rng.random()
        if x < 0.2:
            return None
        if x < 0.5:
            return dense(rng.choice([8, 20, 37, 64]))
        E = rng.choice([1, 2, 3, 6, 8, 12, 17, 40])
        return moe(experts=E, top=rng.randint(1, min(E, 5)), ff=rng.choice([8, 12, 16, 40, 64]))

    layers = []
    mixes = rng.random() < 0.7
    vshape = (rng.choice([1, 2, 3]), rng.choice([4, 6, 8, 20]))          # layers that mix values share their values' shape
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice(["delta", "att", "lat"])
        if kind == "delta":
            G = rng.choice([1, 2, 3])
            layers.append(delta(heads=G * rng.choice([1, 2]), kv_heads=G, dim=rng.choice([4, 6, 16, 20, 33]), vdim=rng.choice([3, 8, 12, 17]),
                                conv=rng.choice([1, 2, 3, 4]), decay_rank=rng.choice([1, 4, 9]), gate_rank=rng.choice([2, 8]), mlp=rmlp()))
        elif kind == "att":
            vm = mixes and rng.random() < 0.7
            G, dv = vshape if vm else (rng.choice([1, 2, 3]), rng.choice([4, 6, 8, 20]))
            dim = rng.choice([4, 6, 8, 16, 20, 32, 72])
            layers.append(att(heads=G * rng.choice([1, 2, 4]), kv_heads=G, dim=dim, vdim=dv, rot_dims=rng.choice([0, 2, dim // 2 // 2 * 2, dim]),
                              base=rng.choice([100.0, 1e4, 2.5e5]), scale=rng.uniform(0.05, 0.5), v_mix=vm, mlp=rmlp()))
        else:
            rd = rng.choice([2, 4, 8])
            layers.append(lat(heads=rng.choice([1, 2, 5]), dim=rng.choice([3, 8, 16]), rot_dim=rd, vdim=rng.choice([4, 7, 16]),
                              kv_rank=rng.choice([5, 16, 24]), q_rank=rng.choice([3, 8, 20]), window=rng.choice([1, 2, 7, 31, 64, 65, 100, 400]),
                              base=rng.choice([100.0, 1e4]), scale=rng.uniform(0.05, 0.5), mlp=rmlp()))
    return config(layers, width=rng.choice([16, 24, 40, 64, 100, 136]), vocab=rng.choice([50, 96, 200]), eps=rng.choice([1e-6, 1e-5]),
                  taps=rng.choice([0, 1, 2, 3, 5]))

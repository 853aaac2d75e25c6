"""Small Dibedra configurations and inputs for the tests (config.json dictionaries; none of them is a served model's
combination of sizes). Sizes are deliberately unequal where a served model might make them equal or 1."""
from __future__ import annotations

import torch


def rot(dims, base=10000.0, scaling=None):
    d = {"dims": dims, "base": base}
    if scaling:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def moe(experts=5, top=2, ff=12, limit=1.5, identity=1, groups=None):
    r = {"experts": experts, "top": top}
    if identity:
        r["identity"] = identity
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def dense(ff=20):
    return {"kind": "dense", "ff": ff}


def att(heads=3, kv_heads=1, dim=8, window=10, rot_dims=4, base=300.0, scaling=(4.0, 32, 8.0, 2.0), scale=0.3, mlp="dense", weights_of=None):
    L = {"type": "attention",
         "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, mask={"size": window}, rot=rot(rot_dims, base, scaling), scale=scale),
         "mlp": dense() if mlp == "dense" else (moe() if mlp == "moe" else mlp)}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def shared(layers, j):
    """A copy of layer j's entry that runs with layer j's weights."""
    L = {k: v for k, v in layers[j].items()}
    L["weights_of"] = j
    return L


def config(layers, width=24, vocab=80, eps=1e-5, logit_scale=0.7):
    return {"architecture": "Dibedra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "logit_scale": logit_scale}


def _looped():
    base = [att(mlp=None), att(heads=4, kv_heads=2, dim=6, window=17, rot_dims=6, mlp=moe(experts=6, top=3, ff=10, identity=2, groups=(4, 3)))]
    return base + [shared(base, 1), att(heads=2, kv_heads=2, dim=12, window=5, rot_dims=2, scaling=None, mlp="dense"), shared(base, 1), shared(base, 0)]


CASES = {
    "attention_only": config([att(mlp=None), att(heads=4, kv_heads=4, dim=6, window=70, rot_dims=6, scaling=None, scale=0.5, mlp=None)]),
    "dense": config([att(window=33), att(heads=2, kv_heads=1, dim=16, window=3, rot_dims=16, mlp=dense(37))], width=40),
    "moe": config([att(mlp=moe(experts=7, top=3, ff=10, limit=0.8, identity=2, groups=(3, 2))),
                   att(mlp=moe(experts=3, top=1, ff=20, limit=4.0, identity=0)),
                   att(mlp=moe(experts=4, top=4, ff=9, limit=1.0, identity=4, groups=(8, 8)))], width=24),
    "looped": config(_looped(), width=32, vocab=96),
    "odd": config([att(heads=5, kv_heads=5, dim=10, window=129, rot_dims=6, scale=1.25, scaling=(2.0, 64, 16.0, 1.0),
                       mlp=moe(experts=33, top=5, ff=6, limit=2.0, identity=3, groups=(6, 4))),
                   att(heads=1, kv_heads=1, dim=18, window=1, rot_dims=0, scaling=None, mlp=dense(7)),
                   att(heads=6, kv_heads=2, dim=5, window=64, rot_dims=4, mlp=moe(experts=2, top=1, ff=7, limit=0.5, identity=0))],
                  width=18, vocab=50, eps=1e-6, logit_scale=1.0),
    # a sharp softmax (large score scale) with channels that do not turn: one key can dominate wherever it sits
    "sharp": config([att(heads=2, kv_heads=1, dim=8, window=100, rot_dims=4, scaling=None, scale=3.0, mlp=None)], width=16, vocab=64),
}


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(3000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(seed):
    """A random stack: 2 to 7 layers, some running with an earlier layer's weights, head counts and sizes that are and are not
    multiples of 8, windows from 1 token to beyond the prompt, rotated parts from none to the whole head, dense, routed or no
    feed-forward, routers with and without groups and identity experts."""
    import random

    rng = random.Random(seed)

    def rmlp():
        x = rng.random()
        if x < 0.2:
            return None
        if x < 0.5:
            return dense(rng.choice([8, 20, 37, 64]))
        ident = rng.choice([0, 0, 1, 3, 4])
        E = rng.choice([1, 2, 3, 6, 8, 12, 17, 40])
        n = E + ident
        counts = [c for c in (1, 2, 3, 4, 5, 6, 8) if n % c == 0]
        top = rng.randint(1, min(n, 5))
        groups = None
        if rng.random() < 0.6:
            c = rng.choice(counts)
            keeps = [k for k in range(1, c + 1) if k * (n // c) >= top]
            groups = (c, rng.choice(keeps))
        return moe(experts=E, top=top, ff=rng.choice([8, 12, 16, 40, 64]), limit=rng.choice([0.5, 1.0, 3.0]), identity=ident, groups=groups)

    layers, owners = [], []
    for i in range(rng.randint(2, 7)):
        if owners and rng.random() < 0.35:
            layers.append(shared(layers, rng.choice(owners)))
            continue
        owners.append(i)
        G = rng.choice([1, 2, 3])
        dim = rng.choice([4, 6, 8, 16, 20, 32, 72])
        layers.append(att(heads=G * rng.choice([1, 2, 4]), kv_heads=G, dim=dim, window=rng.choice([1, 2, 7, 31, 64, 65, 100, 400]),
                          rot_dims=rng.choice([0, 2, dim // 2 // 2 * 2, dim]), base=rng.choice([100.0, 1e4, 2.5e5]),
                          scaling=rng.choice([None, (2.0, 64, 16.0, 1.0), (4.0, 32, 8.0, 2.0), (8.0, 1024, 32.0, 0.5)]),
                          scale=rng.uniform(0.05, 0.5), mlp=rmlp()))
    return config(layers, width=rng.choice([16, 24, 40, 64, 100, 136]), vocab=rng.choice([50, 96, 200]), eps=rng.choice([1e-6, 1e-5]),
                  logit_scale=rng.choice([0.25, 1.0, 1.7]))

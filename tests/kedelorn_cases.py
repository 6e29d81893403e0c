"""Small Kedelorn configurations and inputs for the tests (config.json dictionaries; none of them is a served model's
combination of sizes). Sizes are deliberately unequal where a served model might make them equal or 1."""
from __future__ import annotations

import torch


def rot(dims, base=10000.0, scaling=None):
    d = {"dims": dims, "base": base}
    if scaling:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def moe(experts=5, top=2, ff=12, scale=1.5, shared=20):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def ret(heads=3, dim=8, vdim=6, decay=(0.9, 0.97, 0.999), rot_dims=4, base=500.0, mlp="moe"):
    return {"type": "retention", "mixer": dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay), rot=rot(rot_dims, base)),
            "mlp": moe() if mlp == "moe" else mlp}


def lat(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=12, scale=0.3, base=300.0, scaling=(4.0, 32, 8.0, 2.0), kv_from=None, mlp="moe"):
    mx = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale, rot=rot(rot_dim, base, scaling))
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx, "mlp": moe() if mlp == "moe" else mlp}


def config(layers, width=24, vocab=80, streams=2, eps=1e-5):
    return {"architecture": "Kedelorn", "vocab": vocab, "width": width, "streams": streams, "layers": layers, "norm": {"eps": eps}}


CASES = {
    "retention_only": config([ret(mlp=None), ret(heads=2, dim=12, vdim=16, decay=(0.5, 1.0), rot_dims=12, mlp=None)], width=24, streams=3),
    "latent_only": config([lat(mlp=None), lat(heads=2, dim=4, rot_dim=8, vdim=10, kv_rank=20, scaling=None, mlp=None)], width=24),
    "shared_cache": config([lat(mlp=None), lat(heads=5, dim=6, vdim=3, kv_from=0, scale=0.5, mlp=None),
                            lat(heads=1, dim=16, vdim=16, kv_from=0, mlp=None)], width=16, streams=1),
    "moe_only": config([ret(heads=1, dim=4, vdim=4, decay=(0.8,), rot_dims=0, mlp=moe(experts=7, top=3, ff=10, scale=0.7, shared=0)),
                        ret(heads=1, dim=4, vdim=4, decay=(0.8,), rot_dims=2, mlp=moe(experts=3, top=1, ff=20, scale=2.0, shared=9))],
                       width=24, streams=2),
    "mixed": config([ret(), lat(), lat(kv_from=1, heads=2), ret(heads=2, dim=16, vdim=4, decay=(0.99, 0.6), rot_dims=16, mlp=None), lat(mlp=moe(experts=4, top=4))],
                    width=40, streams=2),
    "odd": config([lat(heads=3, dim=5, rot_dim=6, vdim=7, kv_rank=9, scale=1.25, scaling=(2.0, 64, 16.0, 1.0), mlp=moe(experts=33, top=5, ff=6, shared=3)),
                   ret(heads=1, dim=17, vdim=5, decay=(0.93,), rot_dims=2, mlp=moe(experts=2, top=1, ff=7, shared=0))],
                  width=18, vocab=50, streams=4, eps=1e-6),
    # a sharp softmax (large score scale): one key dominates the weights, so a key that is missed or misplaced changes the
    # output by far more than the tolerance
    "sharp": config([lat(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, scale=6.0, base=10000.0, scaling=None, mlp=None)],
                    width=16, vocab=64, streams=2),
}


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(2000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(seed):
    """A random stack: 2 to 6 layers in any order, 1 to 8 streams, head counts, key / value / latent / rotary sizes that are
    and are not multiples of 8, caches read by later layers, routers from 1 to 40 experts, layers without feed-forward."""
    import random

    rng = random.Random(seed)

    def rmoe():
        if rng.random() < 0.2:
            return None
        E = rng.choice([1, 2, 3, 6, 8, 12, 17, 40])
        return moe(experts=E, top=rng.randint(1, min(E, 5)), ff=rng.choice([8, 12, 16, 40, 64]), scale=rng.choice([0.5, 1.0, 2.5]),
                   shared=rng.choice([0, 8, 20, 64]))

    layers, owners = [], []
    for i in range(rng.randint(2, 6)):
        if rng.random() < 0.5:
            H, dim = rng.choice([1, 2, 3, 5]), rng.choice([6, 8, 16, 20, 32, 72])
            layers.append(ret(heads=H, dim=dim, vdim=rng.choice([4, 8, 12, 40, 72]), decay=[1.0 - 2.0 ** -rng.uniform(1, 10) for _ in range(H)],
                              rot_dims=rng.choice([0, 2, dim // 2 // 2 * 2, dim]), base=rng.choice([100.0, 1e4, 1e6]), mlp=rmoe()))
        elif owners and rng.random() < 0.4:
            j = rng.choice(owners)              # reads layer j's cache: same latent and rotary geometry, its own heads
            g = layers[j]["mixer"]
            L = lat(heads=rng.choice([1, 2, 4, 7]), dim=rng.choice([4, 8, 12, 32]), rot_dim=g["rot_dim"], vdim=rng.choice([4, 8, 20, 32]),
                    kv_rank=g["kv_rank"], scale=rng.uniform(0.05, 0.5), kv_from=j, mlp=rmoe())
            L["mixer"]["rot"] = dict(g["rot"])
            layers.append(L)
        else:
            owners.append(i)
            layers.append(lat(heads=rng.choice([1, 2, 3, 6]), dim=rng.choice([4, 8, 12, 32, 64]), rot_dim=rng.choice([2, 6, 8, 16, 32]),
                              vdim=rng.choice([4, 8, 20, 32]), kv_rank=rng.choice([8, 12, 20, 64, 136]), scale=rng.uniform(0.05, 0.5),
                              base=rng.choice([300.0, 1e4, 5e5]),
                              scaling=rng.choice([None, (2.0, 64, 16.0, 1.0), (4.0, 32, 8.0, 2.0), (8.0, 1024, 32.0, 0.5)]), mlp=rmoe()))
    return config(layers, width=rng.choice([16, 24, 40, 64, 100, 136]), vocab=rng.choice([50, 96, 200]), streams=rng.choice([1, 2, 3, 4, 5, 8]),
                  eps=rng.choice([1e-6, 1e-5]))

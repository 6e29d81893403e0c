"""Small configurations and inputs for the hybrid sequence model tests (config.json dictionaries; none of them is a
served model's combination of sizes)."""
from __future__ import annotations

import torch


def ssd(heads=4, vdim=8, state=12, groups=2, conv=4, norm_groups=2, ff=None):
    return {"type": "mamba2", "mixer": dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups),
            "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def par(heads=4, kv_heads=2, dim=16, vdim=8, chunk=24, scale=0.5, r_heads=2, r_dim=8, r_vdim=12, tau=4.0, ff=48):
    return {"type": "parallel",
            "mixer": {"left": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask={"size": chunk}, scale=scale),
                      "right": dict(heads=r_heads, dim=r_dim, vdim=r_vdim, tau=tau)},
            "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def config(layers, width=40, vocab=96, eps=1e-5, alpha=2.0, embed_scale=3.0, softcap=20.0):
    return {"architecture": "Bimopel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "postln_alpha": alpha, "embedding": {"scale": embed_scale}, "logit_softcap": softcap}


# name -> config.json dictionary. Sizes are deliberately unequal where a served model might make them equal or 1.
CASES = {
    "ssd_only": config([ssd(), ssd(heads=3, vdim=5, state=20, groups=3, conv=2, norm_groups=1, ff=24)], width=24),
    "parallel_only": config([par()], width=40),
    "mixed": config([ssd(), par(), ssd(heads=6, vdim=4, state=7, groups=1, conv=3, norm_groups=3), par(chunk=10, kv_heads=4, ff=None)],
                    width=48, alpha=3.0),
    "odd": config([par(heads=3, kv_heads=1, dim=10, vdim=6, chunk=7, scale=1.25, r_heads=1, r_dim=17, r_vdim=5, tau=1.0, ff=20),
                   ssd(heads=2, vdim=18, state=33, groups=1, conv=5, norm_groups=4, ff=None)],
                  width=18, vocab=50, alpha=1.0, embed_scale=1.0, softcap=0.0),
    # a sharp softmax (large score scale): one key dominates, so a chunk edge or a page border that is off by one token
    # changes the output by far more than the tolerance. Chunks of 40 against pages of 64: borders never coincide.
    "sharp": config([par(heads=2, kv_heads=1, dim=8, vdim=8, chunk=40, scale=6.0, r_heads=1, r_dim=4, r_vdim=4, ff=None)],
                    width=16, vocab=64, alpha=0.5),
}


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

"""Tiny Zimupel configurations for the tests.  Their layers differ in every size, constant and
order and include the values a model could happen to make equal or 1: one stream, no streams at
all (the single residual), one head, one kv head, as many kv heads as heads, keys larger and smaller
than values, rotation of a part of a head and of all of it and none, a decay of exactly 1 and a fast
one, one group of experts, one chosen expert, all experts chosen, a layer without feed-forward, a
layer that reads another layer's keys and values, no logit scale or cap, every mixer as the first
layer, and sizes that fit no 16-byte access."""

from __future__ import annotations


def retention(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return "retention", m


def lightning(heads, dim, vdim, decay):
    return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def attention(heads, kv, dim, vdim, scale, diff, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if kv is not None:
        m["kv_heads"] = kv
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "attention", m


def moe(experts, top, ff, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


P = {"architecture": "Zimupel", "vocab": 211, "width": 48, "norm": {"eps": 1e-6}, "streams": 2,
     "logit_scale": 1.5, "logit_softcap": 20.0,
     "layers": [layer(lightning(3, 8, 12, (0.9, 1.0, 0.5)), moe(6, 2, 16, (3, 2))),
                layer(attention(4, 2, 16, 8, 0.25, 0.2), dense(40)),
                layer(retention(2, 16, 8, (0.97, 0.999), rot=(500.0, 8)), moe(4, 1, 24)),
                layer(attention(4, 2, 16, 8, 0.3, 0.35, kv_from=1), None),
                layer(retention(1, 24, 40, (0.95,)), moe(5, 5, 8))]}
# no streams: the single residual; no logit scale, no cap
Q = {"architecture": "Zimupel", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
     "layers": [layer(retention(4, 16, 16, (0.9, 0.99, 0.999, 0.8), rot=(200000.0, 16)), dense(96)),
                layer(attention(3, None, 8, 24, 0.35, 0.5), moe(8, 3, 16, (4, 2))),
                layer(lightning(1, 32, 16, (0.98,)), moe(10, 2, 32, (2, 1))),
                layer(attention(3, None, 8, 24, 0.2, 0.1, kv_from=1), dense(32)),
                layer(lightning(2, 8, 8, (0.93, 0.75)), None),
                layer(attention(2, 1, 32, 32, 0.18, 0.8), moe(4, 2, 16, (4, 2)))]}
# one stream (with its weights), and sizes that no 16-byte access fits
R = {"architecture": "Zimupel", "vocab": 97, "width": 50, "norm": {"eps": 1e-5}, "streams": 1,
     "logit_softcap": 12.0,
     "layers": [layer(attention(3, 3, 10, 6, 0.3, 0.4), moe(3, 2, 10)),
                layer(retention(3, 10, 6, (0.9, 0.95, 0.99), rot=(900.0, 4)), dense(22)),
                layer(lightning(2, 6, 14, (0.7, 0.995)), moe(6, 2, 14, (2, 1)))]}
# four streams and sizes in multiples of 16 and 64
S = {"architecture": "Zimupel", "vocab": 150, "width": 128, "norm": {"eps": 1e-5}, "streams": 4,
     "logit_scale": 0.5,
     "layers": [layer(retention(2, 64, 64, (0.99, 0.9999), rot=(10000.0, 32)), moe(4, 2, 32, (2, 2))),
                layer(attention(4, 1, 64, 128, 0.125, 0.6), dense(64)),
                layer(lightning(2, 128, 64, (0.96, 0.999)), moe(8, 4, 16, (2, 1))),
                layer(attention(4, 1, 64, 128, 0.1, 0.28, kv_from=1), moe(4, 1, 48))]}
# sizes in multiples of 16 but not of 64 (the mma.sync attention in prompts, the maps as rows of one
# block in single tokens), attention first, three groups of experts, two cache readers of one layer
T = {"architecture": "Zimupel", "vocab": 320, "width": 192, "norm": {"eps": 1e-6}, "streams": 2,
     "logit_scale": 3.0, "logit_softcap": 40.0,
     "layers": [layer(attention(6, 3, 32, 64, 0.15, 0.45), dense(80)),
                layer(lightning(3, 48, 48, (0.9, 0.97, 0.999)), moe(6, 2, 40, (3, 1))),
                layer(attention(6, 3, 32, 64, 0.2, 0.15, kv_from=0), dense(64)),
                layer(retention(4, 32, 80, (0.95, 0.99, 0.995, 0.9995), rot=(50000.0, 16)), moe(12, 3, 24, (3, 2))),
                layer(attention(12, 3, 32, 64, 0.17, 0.7, kv_from=0), None)]}
CASES = {"P": (P, 5, 8), "Q": (Q, 9, 16), "R": (R, 13, 4), "S": (S, 17, 16), "T": (T, 21, 32)}   # config, seed, page size
# projections drawn large enough that the softmax of a tiny model is peaked and the router's
# choice is clear of ties
STD_OF = {"embed": 0.5, ".mix.q": 0.3, ".mix.k": 0.3, ".router": 0.4, ".correction": 0.3, ".hc": 0.5,
          ".mix.lq": 0.2, ".mix.lk": 0.2}


def make_model(folder: str, cfg: dict, seed: int) -> str:
    """The weights are stored in bfloat16, as a served model's are: what the engine's bfloat16 path
    computes then differs from the oracle by the rounding of activations only."""
    import torch
    from servelab_b200.config import config_from_dict
    from servelab_b200.weights import write_random_model
    return write_random_model(folder, config_from_dict(cfg), seed, dtype=torch.bfloat16, std=0.15,
                              norm_std=0.3, std_of=STD_OF)

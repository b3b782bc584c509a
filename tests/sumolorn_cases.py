"""Tiny Sumolorn configurations for the tests.  Their layers differ in every size, constant and
order and include the values a model could happen to make equal or 1: one head, one kv head, as many
kv heads as heads, keys larger and smaller than values, a rotation of part of a head, of all of it
and none, stretched and plain frequencies, windows of 1, 5, 9, 33, 70 and one beyond every request,
no window, one tap, two taps and five, no loop, a loop over one layer, over all layers and an empty
one, a layer without feed-forward, every mixer as the first layer, no logit scale, and sizes that
fit no 16-byte access."""

from __future__ import annotations

import json
import os


def attention(heads, kv, dim, vdim, scale, window=None, rot=None, softcap=None):
    m = {"heads": heads, "dim": dim, "scale": scale}
    if kv is not None:
        m["kv_heads"] = kv
    if vdim is not None:
        m["vdim"] = vdim
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    if softcap is not None:
        m["softcap"] = softcap
    return "attention", m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale):
    return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                "q_rank": q_rank, "rot": {"base": base, "dims": rot_dim}, "scale": scale}


def parallel(left, right):
    """left: (taps, heads, kv, dim, vdim, scale, window, rot); right: (heads, dim, vdim, tau, rank)."""
    taps, heads, kv, dim, vdim, scale, window, rot = left
    lm = attention(heads, kv, dim, vdim, scale, window, rot)[1]
    lm["conv"] = taps
    rh, rd, rv, tau, rank = right
    return "parallel", {"left": lm, "right": {"heads": rh, "dim": rd, "vdim": rv, "tau": tau, "rank": rank}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


STRETCH = (8.0, 1.0, 4.0, 16)          # wavelengths beyond 16 positions are stretched eight times

# the latent attention first; the two middle layers run three times
A = {"architecture": "Sumolorn", "vocab": 211, "width": 48, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
     "loop": {"start": 1, "stop": 3, "times": 3},
     "layers": [layer(latent(3, 8, 4, 12, 20, 10, 1000.0, 0.3), dense(40, 1.0)),
                layer(attention(4, 2, 16, 8, 0.25, window=5, rot=(500.0, 8, STRETCH), softcap=5.0), dense(24, 0.7)),
                layer(parallel((3, 2, 1, 16, 16, 0.2, 9, (100.0, 16)), (3, 8, 12, 4.0, 6)), None),
                layer(attention(2, None, 8, None, 0.35, rot=(10000.0, 8)), dense(32, 2.5))]}
# no loop, no logit scale, sizes that no 16-byte access fits; a window of one token; one tap
B = {"architecture": "Sumolorn", "vocab": 97, "width": 50, "norm": {"eps": 1e-5},
     "layers": [layer(parallel((1, 3, 3, 10, 6, 0.3, 1, (900.0, 4)), (1, 6, 14, 1.0, 3)), dense(22, 1.5)),
                layer(attention(3, 3, 10, 6, 0.3, window=1, softcap=2.0), dense(14, 0.5)),
                layer(latent(1, 6, 2, 10, 14, 7, 50.0, 0.4), None),
                layer(parallel((2, 2, 1, 6, 10, 0.4, 13, None), (2, 10, 6, 30.0, 5)), dense(18, 1.0))]}
# sizes in multiples of 64 (the tensor-core attentions of every kind), the whole model twice
C = {"architecture": "Sumolorn", "vocab": 150, "width": 128, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
     "loop": {"start": 0, "stop": 3, "times": 2},
     "layers": [layer(attention(4, 1, 64, 64, 0.06, window=70, rot=(1e6, 32, (4.0, 1.0, 4.0, 64)), softcap=15.0),
                      dense(64, 1.2)),
                layer(parallel((5, 4, 2, 64, 64, 0.08, 33, (3e5, 64)), (2, 64, 128, 12.0, 16)), dense(96, 3.0)),
                layer(latent(4, 64, 64, 64, 64, 48, 1.5e5, 0.05), dense(64, 0.9))]}
# sizes in multiples of 16 but not of 64, an empty loop, a window beyond every request
D = {"architecture": "Sumolorn", "vocab": 320, "width": 192, "norm": {"eps": 1e-6}, "logit_scale": 0.125,
     "loop": {"start": 2, "stop": 2, "times": 4},
     "layers": [layer(attention(6, 3, 32, 64, 0.15, window=1000, rot=(1e4, 32), softcap=30.0), dense(80, 1.0)),
                layer(latent(6, 16, 16, 32, 48, 32, 1e4, 0.2), dense(64, 2.0)),
                layer(parallel((4, 6, 3, 48, 32, 0.14, 40, (2e5, 16)), (4, 32, 48, 8.0, 8)), dense(48, 1.5)),
                layer(attention(12, 3, 16, 48, 0.08, window=33, rot=(3e4, 16, (2.0, 1.0, 2.0, 32))), None)]}
CASES = {"A": (A, 5, 8), "B": (B, 9, 4), "C": (C, 13, 16), "D": (D, 17, 32)}   # config, seed, page size
# projections drawn large enough that the softmax of a tiny model is peaked; sinks, taps and the
# decays' offsets large enough that leaving one out moves the logits
STD_OF = {"embed": 0.5, ".sink": 1.5, ".conv": 0.5, ".a2.b": 1.5, ".a1": 0.4, ".a2": 0.6,
          ".q": 0.3, ".k": 0.3, ".uq": 0.3, ".uk": 0.3, ".dq": 0.3, ".dkv": 0.3}


def make_model(folder: str, cfg: dict, seed: int, drop_rank: bool = False) -> str:
    """The weights are stored in bfloat16, as a served model's are.  ``drop_rank``: config.json is
    written without the bottleneck size of the decays, which the loader then reads from the tensor."""
    import torch
    from servelab_b200.config import config_from_dict
    from servelab_b200.weights import write_random_model
    write_random_model(folder, config_from_dict(cfg), seed, dtype=torch.bfloat16, std=0.15, norm_std=0.3,
                       std_of=STD_OF)
    if drop_rank:
        path = os.path.join(folder, "config.json")
        with open(path) as f:
            written = json.load(f)
        for entry in written["layers"]:
            if entry["type"] == "parallel":
                entry["mixer"]["right"].pop("rank", None)
        with open(path, "w") as f:
            json.dump(written, f, indent=1)
    return folder

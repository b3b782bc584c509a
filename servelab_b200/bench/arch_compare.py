"""Prefill and decode throughput of the Dezelorn design beside the Qwen2 decoder at equal layer
sizes (random weights), with the attention kernels' own times and roofline fractions.

Both models get the same width, heads, kv heads, head size, feed-forward size, layer count,
vocabulary and sliding window, so the matrix products do nearly the same work (Dezelorn has a
gate projection instead of a value projection) and what differs is the mixer: a convolution
on q and k, keys that are also the values (half the cache bytes), the distance bias, and the
heads mixed after the softmax -- which this package computes as one attention result per
(query head, kv head) pair, so its attention does kv_heads times the arithmetic of the plain
one.  ``python bench.py --compare dezelorn`` prints one JSON line with, per size and model:
prefill tokens per second (one 2,048-token prompt), decode tokens per second at batch 8 and 64
(contexts of 1,536 tokens, graphs), and per-kernel microseconds of an eager prefill and of
eager decode steps of 8 and of 64 requests.
"""

from __future__ import annotations

from typing import Dict

PROMPT, CONTEXT, PAGE, WINDOW, LAYERS, VOCAB = 2048, 1536, 16, 1024, 4, 32000
SIZES = {                       # width, heads, kv heads, head size, feed-forward
    "1b-like": (2048, 16, 4, 128, 5632),
    "3b-like": (2048, 16, 2, 128, 11008),
    "7b-like": (3584, 28, 4, 128, 18944),
    "small-heads": (1536, 24, 4, 64, 4096),
}


def dezelorn_config(width, heads, kv, dim, ff, layers=LAYERS) -> dict:
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "conv": 4, "scale": dim ** -0.5,
             "mask": {"size": WINDOW}, "q_temp": {"coef": 0.3, "every": 128}}
    return {"architecture": "Dezelorn", "vocab": VOCAB, "width": width, "embedding": {"scale": 8.0},
            "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}}
                       for _ in range(layers)]}


def qwen2_config(width, heads, kv, dim, ff, layers=LAYERS) -> dict:
    from .workloads import QWEN2
    return dict(QWEN2, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads,
                num_key_value_heads=kv, head_dim=dim, intermediate_size=ff, vocab_size=VOCAB,
                tie_word_embeddings=False, use_sliding_window=True, sliding_window=WINDOW,
                max_window_layers=0)


# Daferax: layers alternate between the latent attention (windowed) and the grouped-query
# attention (every earlier key), each followed by routed experts with a shared expert.  The Qwen2
# model beside it has the same width, heads, kv heads, head size and layer count, a dense
# feed-forward of the size a Daferax token ACTIVATES (top experts + shared), and its upper half of
# layers windowed.  width, heads, kv heads, head size (keys = values), latent size, rotated part,
# experts, groups, kept groups, top, expert size, shared size
DAFERAX_SIZES = {
    "lite-2048": (2048, 16, 4, 128, 256, 64, 32, 4, 2, 4, 1408, 2816),
    "small-1024": (1024, 8, 2, 64, 192, 64, 16, 2, 1, 2, 512, 1024),
}


def daferax_config(width, heads, kv, dim, rank, rot, experts, groups, keep, top, eff, sff, layers=LAYERS) -> dict:
    mlp = {"kind": "moe", "expert": {"ff": eff}, "shared": {"ff": sff},
           "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "scale": 2.0, "top": top}}
    latent = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank,
              "scale": (dim + rot) ** -0.5, "mask": {"size": WINDOW},
              "rot": {"base": 250000.0, "dims": rot,
                      "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    attn = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "v_mix": True,
            "rot": {"base": 2000000.0, "dims": dim}}
    return {"architecture": "Daferax", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention" if i % 2 == 0 else "attention",
                        "mixer": latent if i % 2 == 0 else attn, "mlp": mlp} for i in range(layers)]}


def qwen2_like_daferax(width, heads, kv, dim, rank, rot, experts, groups, keep, top, eff, sff, layers=LAYERS) -> dict:
    cfg = qwen2_config(width, heads, kv, dim, top * eff + sff, layers)
    cfg["max_window_layers"] = layers // 2            # the upper half of the layers is windowed
    return cfg


def _daferax_rooflines(size, res, peaks) -> Dict[str, object]:
    """Microseconds per launch and achieved fractions of the measured peaks for the kernels of the
    Daferax layers beside their Qwen2 counterparts, from the eager profiles.  Prefill attention:
    flops of the visible (query, key) pairs, 2 (Dk + Dv) per pair and head, of the bf16 peak -- for
    the latent attention Dk and Dv are what the absorbed form multiplies (latent + rotated part,
    latent).  Decode attention: bytes of the cached rows the 8 requests may see, of the copy
    bandwidth.  Elementwise kernels: bytes they must move, of the copy bandwidth.  Experts
    (prefill): 6 tokens top width expert_size flops of the bf16 peak; (decode, 8 tokens): bytes of
    the weights of the experts that at most 8 top pairs can touch."""
    width, heads, kv, dim, rank, rot, experts, groups, keep, top, eff, sff = DAFERAX_SIZES[size]
    out: Dict[str, object] = {}
    pk, dk = res["daferax"]["prefill_kernels_us"], res["daferax"]["decode_b8_kernels_us"]
    qk, qd = res["qwen2"]["prefill_kernels_us"], res["qwen2"]["decode_b8_kernels_us"]
    n_lat, n_att = (LAYERS + 1) // 2, LAYERS // 2
    full_pairs = PROMPT * (PROMPT + 1) / 2
    win_pairs = sum(min(t + 1, WINDOW) for t in range(PROMPT))

    def hbm(nbytes, us):
        return round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)

    def tf(flops, us):
        return round(flops / (us * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)

    # the latent layers run this design's kernel; the grouped layers, whose keys and values are of one
    # size here, the kernels of the other models (when they are of two sizes: this design's kernel too)
    lat = (pk.get("attention_kv_tc") or 0) + (pk.get("attention_kv_mma") or 0) + (pk.get("attention_kv") or 0)
    grp = (pk.get("prefill_attention_tc") or 0) + (pk.get("prefill_attention") or 0)
    lat_flops = n_lat * win_pairs * heads * 2 * (2 * rank + rot)
    grp_flops = n_att * full_pairs * heads * 2 * 2 * dim
    if lat and grp:
        out["daferax_latent_prefill_attention_us_per_layer"] = round(lat / n_lat, 1)
        out["daferax_latent_prefill_attention_bf16_frac"] = tf(lat_flops, lat)
        out["daferax_grouped_prefill_attention_us_per_layer"] = round(grp / n_att, 1)
        out["daferax_grouped_prefill_attention_bf16_frac"] = tf(grp_flops, grp)
    elif lat:
        out["daferax_prefill_attention_us_per_layer"] = round(lat / LAYERS, 1)
        out["daferax_prefill_attention_bf16_frac"] = tf(lat_flops + grp_flops, lat)
    qatt = (qk.get("prefill_attention_tc") or 0) + (qk.get("prefill_attention") or 0)
    if qatt:
        flops = (LAYERS // 2 * win_pairs + (LAYERS - LAYERS // 2) * full_pairs) * heads * 4 * dim
        out["qwen2_prefill_attention_us_per_layer"] = round(qatt / LAYERS, 1)
        out["qwen2_prefill_attention_bf16_frac"] = tf(flops, qatt)
    dlat = dk.get("attention_kv_mma") or dk.get("attention_kv")
    dgrp = dk.get("decode_attention")
    lat_bytes = 8 * 2 * n_lat * min(CONTEXT, WINDOW) * (rank + rot)
    grp_bytes = 8 * 2 * n_att * CONTEXT * kv * 2 * dim
    if dlat and dgrp:
        out["daferax_latent_decode_attention_us_per_layer"] = round(dlat / n_lat, 2)
        out["daferax_latent_decode_attention_hbm_frac"] = hbm(lat_bytes, dlat)
        out["daferax_grouped_decode_attention_us_per_layer"] = round(dgrp / n_att, 2)
        out["daferax_grouped_decode_attention_hbm_frac"] = hbm(grp_bytes, dgrp)
    elif dlat:
        out["daferax_decode_attention_us_per_layer"] = round(dlat / LAYERS, 2)
        out["daferax_decode_attention_hbm_frac"] = hbm(lat_bytes + grp_bytes, dlat)
    qdatt = qd.get("decode_attention")
    if qdatt:
        nbytes = 8 * 2 * kv * 2 * dim * (LAYERS // 2 * min(CONTEXT, WINDOW) + (LAYERS - LAYERS // 2) * CONTEXT)
        out["qwen2_decode_attention_us_per_layer"] = round(qdatt / LAYERS, 2)
        out["qwen2_decode_attention_hbm_frac"] = hbm(nbytes, qdatt)
    if pk.get("ln_add_norm"):
        us = pk["ln_add_norm"] / (2 * LAYERS + 1)
        out["daferax_norm_us"], out["daferax_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if qk.get("add_rmsnorm"):
        us = qk["add_rmsnorm"] / (2 * LAYERS + 1)
        out["qwen2_norm_us"], out["qwen2_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if pk.get("head_prep"):
        us = pk["head_prep"] / LAYERS
        moved = PROMPT * 4 * (n_lat * (heads * rot + rank + rot) + n_att * (heads + 2 * kv) * dim) / LAYERS
        out["daferax_head_prep_us"], out["daferax_head_prep_hbm_frac"] = round(us, 2), hbm(moved, us)
    if qk.get("qkv_rope_cache"):
        us = qk["qkv_rope_cache"] / LAYERS
        out["qwen2_rope_cache_us"], out["qwen2_rope_cache_hbm_frac"] = round(us, 2), hbm(PROMPT * 4 * (heads + 2 * kv) * dim, us)
    for name in ("moe_gate_up", "moe_down"):
        if pk.get(name):
            share = 2.0 / 3.0 if name == "moe_gate_up" else 1.0 / 3.0
            out[f"daferax_{name}_prefill_us"] = round(pk[name] / LAYERS, 1)
            out[f"daferax_{name}_prefill_bf16_frac"] = tf(share * 6.0 * PROMPT * top * width * eff * LAYERS, pk[name])
        if dk.get(name):
            share = 2.0 / 3.0 if name == "moe_gate_up" else 1.0 / 3.0
            touched = min(experts, 8 * top)
            out[f"daferax_{name}_decode_us"] = round(dk[name] / LAYERS, 2)
            out[f"daferax_{name}_decode_hbm_frac"] = hbm(share * touched * 3 * width * eff * 2 * LAYERS, dk[name])
    for tag, prof in (("prefill", pk), ("decode_b8", dk)):
        out[f"daferax_{tag}_small_kernels_us"] = {k: round(v / LAYERS, 2) for k, v in prof.items()
                                                  if k in ("moe_route", "moe_plan", "moe_combine", "router_logits",
                                                           "sigmoid_gate", "gemm_simt_batched")}
    return out


# Zimupel: four layers -- linear attention with a decay and rotation, differential attention, linear
# attention on activated q, k, v, differential attention that reads the second layer's cache -- each
# followed by routed experts; the residual kept as `streams` copies.  A differential head has two
# maps of `dim` elements and values of 2 dim, so half as many heads give the projections of a plain
# attention.  Beside it the closest model the package has: Daferax with grouped-query attention in
# every layer (keys = values = dim) and the same routed experts (no shared expert, no value mixing).
# width, heads, kv heads, head size, experts, groups, kept groups, top, expert size, streams
ZIMUPEL_SIZES = {
    "lite-2048": (2048, 16, 4, 128, 32, 4, 2, 4, 1408, 4),
    "small-1024": (1024, 8, 2, 64, 16, 2, 1, 2, 512, 2),
}


def zimupel_config(width, heads, kv, dim, experts, groups, keep, top, eff, streams, layers=LAYERS) -> dict:
    mlp = {"kind": "moe", "expert": {"ff": eff},
           "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "top": top}}
    decay = [1.0 - 2.0 ** (-4.75 - 0.5 * i) for i in range(heads)]
    ret = {"heads": heads, "dim": dim, "vdim": dim, "decay": decay, "rot": {"base": 500000.0, "dims": dim}}
    lig = {"heads": heads, "dim": dim, "vdim": dim, "decay": decay}
    att = {"heads": heads // 2, "kv_heads": max(1, kv // 2), "dim": dim, "vdim": 2 * dim, "scale": dim ** -0.5,
           "diff": 0.25}
    kinds = [("retention", ret), ("attention", att), ("lightning", lig), ("attention", dict(att, kv_from=1))]
    return {"architecture": "Zimupel", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5}, "streams": streams,
            "logit_scale": 1.0, "logit_softcap": 25.0,
            "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": mlp} for i in range(layers)]}


def daferax_like_zimupel(width, heads, kv, dim, experts, groups, keep, top, eff, streams, layers=LAYERS) -> dict:
    mlp = {"kind": "moe", "expert": {"ff": eff},
           "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "scale": 1.0, "top": top}}
    attn = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
            "rot": {"base": 1000000.0, "dims": dim}}
    return {"architecture": "Daferax", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": attn, "mlp": mlp} for _ in range(layers)]}


def _zimupel_rooflines(size, res, peaks) -> Dict[str, object]:
    """Microseconds per launch and achieved fractions of the measured peaks for the kernels of the
    Zimupel layers beside their Daferax counterparts, from the eager profiles.  Linear attention,
    prefill: 4 T H D Dv flops (state update and output, the recurrence's own arithmetic; the chunked
    kernels spend more, on the tensor cores) of the bf16 peak, beside the softmax attention's
    2 (Dk + Dv) flops per visible pair and head; decode: the state read and written once, of the copy bandwidth, beside the cached
    rows the requests may see.  Elementwise kernels: the bytes they must move, of the copy
    bandwidth."""
    width, heads, kv, dim, experts, groups, keep, top, eff, streams = ZIMUPEL_SIZES[size]
    out: Dict[str, object] = {}
    zp, zd = res["zimupel"]["prefill_kernels_us"], res["zimupel"]["decode_b8_kernels_us"]
    dp, dd = res["daferax"]["prefill_kernels_us"], res["daferax"]["decode_b8_kernels_us"]
    n_lin, n_att = 2, 2
    pairs = PROMPT * (PROMPT + 1) / 2

    def hbm(nbytes, us):
        return round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)

    def tf(flops, us):
        return round(flops / (us * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)

    lin = (zp.get("decay_attention (chunked)") or 0) + (zp.get("decay_attention") or 0)
    if lin:
        us = lin / n_lin
        out["zimupel_linear_prefill_us_per_layer"] = round(us, 1)
        out["zimupel_linear_prefill_bf16_frac"] = tf(4.0 * PROMPT * heads * dim * dim, us)
    if zd.get("decay_attention"):
        us = zd["decay_attention"] / n_lin
        out["zimupel_linear_decode_us_per_layer"] = round(us, 2)
        out["zimupel_linear_decode_hbm_frac"] = hbm(8 * 2 * heads * dim * dim * 4, us)
    zatt = zp.get("attention_kv_tc") or zp.get("attention_kv_mma") or zp.get("attention_kv_maps")
    if zatt:
        us = zatt / n_att
        out["zimupel_differential_prefill_us_per_layer"] = round(us, 1)
        out["zimupel_differential_prefill_bf16_frac"] = tf(pairs * (heads // 2) * 2 * 2 * (dim + 2 * dim), us)
    zdatt = zd.get("attention_kv_mma") or zd.get("attention_kv_maps")
    if zdatt:
        us = zdatt / n_att
        out["zimupel_differential_decode_us_per_layer"] = round(us, 2)
        out["zimupel_differential_decode_hbm_frac"] = hbm(8 * CONTEXT * max(1, kv // 2) * 4 * dim * 2, us)
    datt = (dp.get("prefill_attention_tc") or 0) + (dp.get("prefill_attention") or 0) + (dp.get("attention_kv_mma") or 0)
    if datt:
        us = datt / LAYERS
        out["daferax_prefill_attention_us_per_layer"] = round(us, 1)
        out["daferax_prefill_attention_bf16_frac"] = tf(pairs * heads * 4 * dim, us)
    ddatt = dd.get("decode_attention") or dd.get("attention_kv_mma")
    if ddatt:
        us = ddatt / LAYERS
        out["daferax_decode_attention_us_per_layer"] = round(us, 2)
        out["daferax_decode_attention_hbm_frac"] = hbm(8 * CONTEXT * kv * 2 * dim * 2, us)
    if zp.get("hyper_mix_norm"):
        us = zp["hyper_mix_norm"] / (2 * LAYERS + 1)
        out["zimupel_streams_norm_us"] = round(us, 2)
        out["zimupel_streams_norm_hbm_frac"] = hbm(PROMPT * width * (8 * streams + 4), us)
    if dp.get("ln_add_norm"):
        us = dp["ln_add_norm"] / (2 * LAYERS + 1)
        out["daferax_norm_us"], out["daferax_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if zp.get("group_norm_gate"):
        us = zp["group_norm_gate"] / LAYERS
        out["zimupel_norm_gate_us"] = round(us, 2)
        # linear layers: float32 row and gate in, row out; differential layers: two float32 maps in, row out
        moved = PROMPT * heads * dim * ((4 + 2 + 2) * n_lin + (8 + 2) * n_att) / LAYERS
        out["zimupel_norm_gate_hbm_frac"] = hbm(moved, us)
    if zp.get("head_prep"):
        us = zp["head_prep"] / n_att
        out["zimupel_head_prep_us"] = round(us, 2)
        out["zimupel_head_prep_hbm_frac"] = hbm(PROMPT * 4 * (heads * dim + 1.5 * kv * dim) , us)
    if dp.get("head_prep"):
        us = dp["head_prep"] / LAYERS
        out["daferax_head_prep_us"] = round(us, 2)
        out["daferax_head_prep_hbm_frac"] = hbm(PROMPT * 4 * (heads + 2 * kv) * dim, us)
    for tag, a, b in (("prefill", zp, dp), ("decode_b8", zd, dd)):
        for name in ("moe_route", "router_logits", "moe_gate_up", "moe_down", "moe_combine", "moe_plan", "gated_act",
                     "embed_norm_streams"):
            if a.get(name) or b.get(name):
                out[f"{tag}_{name}_us_per_layer"] = {"zimupel": round((a.get(name) or 0) / LAYERS, 2),
                                                     "daferax": round((b.get(name) or 0) / LAYERS, 2)}
    return out


# Sumolorn: four layers -- soft-capped windowed attention with sinks, a parallel layer (convolved
# windowed attention beside a linear attention with learned decays), a latent attention with latent
# queries, the windowed attention again -- each with the clamped feed-forward.  Beside it the closest
# model the package has: Daferax with a grouped-query attention where Sumolorn has its attention and
# its parallel layer, a latent attention where it has one, and a dense feed-forward of the same size.
# width, heads, kv heads, head size, feed-forward, latent size, rotated part, queries' latent,
# heads / key size / value size of the linear branch
SUMOLORN_SIZES = {
    "1b-like": (2048, 16, 4, 128, 5632, 256, 64, 768, 8, 128, 256),
    "small-1024": (1024, 8, 2, 64, 2816, 192, 64, 384, 4, 64, 128),
}


def sumolorn_config(width, heads, kv, dim, ff, rank, rot, q_rank, lh, ld, lv, layers=LAYERS) -> dict:
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    attn = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
            "mask": {"size": WINDOW},
            "rot": {"base": 2000000.0, "dims": dim,
                    "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    left = {"conv": 4, "heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
            "mask": {"size": WINDOW}, "rot": {"base": 400000.0, "dims": dim // 2}}
    right = {"heads": lh, "dim": ld, "vdim": lv, "tau": 8.0, "rank": 32}
    latent = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank, "q_rank": q_rank,
              "scale": (dim + rot) ** -0.5, "rot": {"base": 100000.0, "dims": rot}}
    kinds = [("attention", attn), ("parallel", {"left": left, "right": right}), ("latent_attention", latent),
             ("attention", attn)]
    return {"architecture": "Sumolorn", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": mlp} for i in range(layers)]}


def daferax_like_sumolorn(width, heads, kv, dim, ff, rank, rot, q_rank, lh, ld, lv, layers=LAYERS) -> dict:
    mlp = {"kind": "dense", "ff": ff}
    attn = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
            "mask": {"size": WINDOW}, "rot": {"base": 1000000.0, "dims": dim}}
    latent = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank,
              "scale": (dim + rot) ** -0.5, "rot": {"base": 250000.0, "dims": rot}}
    kinds = [("attention", attn), ("attention", attn), ("latent_attention", latent), ("attention", attn)]
    return {"architecture": "Daferax", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": mlp} for i in range(layers)]}


def _sumolorn_rooflines(size, res, peaks) -> Dict[str, object]:
    """Microseconds per launch and achieved fractions of the measured peaks for the kernels of the
    Sumolorn layers beside their Daferax counterparts, from the eager profiles.  Softmax attention,
    prefill: 2 (Dk + Dv) flops per visible pair and head of the bf16 peak (for the latent form, what
    the absorbed form multiplies); decode: the cached rows 8 requests may see, of the copy bandwidth.
    Linear attention, prefill: 4 T H D Dv flops (the recurrence's own arithmetic); decode: the state
    read and written once.  Elementwise kernels: the bytes they must move, of the copy bandwidth."""
    width, heads, kv, dim, ff, rank, rot, q_rank, lh, ld, lv = SUMOLORN_SIZES[size]
    out: Dict[str, object] = {}
    sp, sd = res["sumolorn"]["prefill_kernels_us"], res["sumolorn"]["decode_b8_kernels_us"]
    dp, dd = res["daferax"]["prefill_kernels_us"], res["daferax"]["decode_b8_kernels_us"]
    win_pairs = sum(min(t + 1, WINDOW) for t in range(PROMPT))
    full_pairs = PROMPT * (PROMPT + 1) / 2

    def hbm(nbytes, us):
        return round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)

    def tf(flops, us):
        return round(flops / (us * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)

    def total(table, *names):
        return sum(table.get(n) or 0 for n in names)

    # prefill attention, all softmax layers of a model together (the kernels' names do not tell the layers apart)
    s_flops = (3 * win_pairs * heads * 4 * dim) + full_pairs * heads * 2 * (2 * rank + rot)
    d_flops = (3 * win_pairs * heads * 4 * dim) + full_pairs * heads * 2 * (2 * rank + rot)
    s_att = total(sp, "attention_kv_mma", "attention_kv_tc", "attention_kv", "prefill_attention_tc", "prefill_attention")
    d_att = total(dp, "attention_kv_mma", "attention_kv_tc", "attention_kv", "prefill_attention_tc", "prefill_attention")
    if s_att and d_att:
        out["prefill_softmax_attention_us_all_layers"] = {"sumolorn": round(s_att, 1), "daferax": round(d_att, 1)}
        out["prefill_softmax_attention_bf16_frac"] = {"sumolorn": tf(s_flops, s_att), "daferax": tf(d_flops, d_att)}
    rows = 8 * (3 * min(CONTEXT, WINDOW) * kv * 2 * dim + CONTEXT * (rank + rot)) * 2
    s_dec = total(sd, "attention_kv_mma", "attention_kv", "decode_attention")
    d_dec = total(dd, "attention_kv_mma", "attention_kv", "decode_attention")
    if s_dec and d_dec:
        out["decode_b8_softmax_attention_us_all_layers"] = {"sumolorn": round(s_dec, 2), "daferax": round(d_dec, 2)}
        out["decode_b8_softmax_attention_hbm_frac"] = {"sumolorn": hbm(rows, s_dec), "daferax": hbm(rows, d_dec)}
    if sp.get("decay_attention (gated chunks)") or sp.get("decay_attention"):
        us = sp.get("decay_attention (gated chunks)") or sp["decay_attention"]
        out["sumolorn_linear_prefill_us"] = round(us, 1)
        out["sumolorn_linear_prefill_bf16_frac"] = tf(4.0 * PROMPT * lh * ld * lv, us)
    if sd.get("decay_attention"):
        us = sd["decay_attention"]
        out["sumolorn_linear_decode_b8_us"] = round(us, 2)
        out["sumolorn_linear_decode_b8_hbm_frac"] = hbm(8 * lh * ld * lv * 4 * 2, us)
    if sp.get("short_conv"):
        us = sp["short_conv"]
        chans = (heads + 2 * kv) * dim
        out["sumolorn_conv_us"], out["sumolorn_conv_hbm_frac"] = round(us, 2), hbm(PROMPT * chans * 4, us)
    if sp.get("norm_sum2"):
        us = sp["norm_sum2"]
        out["sumolorn_branch_norms_us"], out["sumolorn_branch_norms_hbm_frac"] = round(us, 2), hbm(PROMPT * width * 10, us)
    if sp.get("head_prep"):
        us = sp["head_prep"] / 5                # (three grouped layers, and two launches of the latent layer)
        out["sumolorn_head_prep_us"] = round(us, 2)
        moved = PROMPT * 4 * (3 * (heads + 2 * kv) * dim + heads * (dim + rot) + rank + rot) / 5
        out["sumolorn_head_prep_hbm_frac"] = hbm(moved, us)
    if dp.get("head_prep"):
        us = dp["head_prep"] / LAYERS
        out["daferax_head_prep_us"] = round(us, 2)
        moved = PROMPT * 4 * (3 * (heads + 2 * kv) * dim + heads * (dim + rot) + rank + rot) / LAYERS
        out["daferax_head_prep_hbm_frac"] = hbm(moved, us)
    if sp.get("add_rmsnorm"):
        us = sp["add_rmsnorm"] / (2 * LAYERS + 1)
        out["sumolorn_norm_us"], out["sumolorn_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if dp.get("ln_add_norm"):
        us = dp["ln_add_norm"] / (2 * LAYERS + 1)
        out["daferax_norm_us"], out["daferax_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if sp.get("gated_act"):
        us = sp["gated_act"] / LAYERS
        out["sumolorn_activation_us"], out["sumolorn_activation_hbm_frac"] = round(us, 2), hbm(PROMPT * ff * 6, us)
    if dp.get("swiglu"):
        us = dp["swiglu"] / LAYERS
        out["daferax_activation_us"], out["daferax_activation_hbm_frac"] = round(us, 2), hbm(PROMPT * ff * 6, us)
    for name in ("group_norm_gate", "rms_norm_rows", "sigmoid_gate"):
        if sp.get(name) or dp.get(name):
            out[f"prefill_{name}_us"] = {"sumolorn": round(sp.get(name) or 0, 2), "daferax": round(dp.get(name) or 0, 2)}
    return out


def _measure(cfg: dict, note, graph_prefill: bool = False) -> Dict[str, object]:
    """``graph_prefill``: the prompt's step replays the graph captured for its padded sizes where the
    model allows it (the eager step of a small model is bound by the host's launches); the eager
    time is reported beside it."""
    import torch
    from ..ops import kernels as K
    from ..ops.profile import StepProfile
    from . import workloads as W
    pages = 64 * (-(-(CONTEXT + 64) // PAGE)) + PROMPT // PAGE + 8
    engine = W.make_engine(cfg, pages, 64, PROMPT, 4096, weights_seed=3, page_size=PAGE)
    runner = engine.runner
    gen = torch.Generator().manual_seed(2)
    vocab = runner.spec.vocab_size
    out: Dict[str, object] = {}

    def timed(fn, repeats, warmup):
        for _ in range(warmup):
            fn()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeats):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / repeats

    # prefill: one prompt, whole, through the step function
    ids = torch.randint(0, vocab, (PROMPT,), generator=gen).tolist()
    runner.cache.open("p")
    runner.cache.ensure("p", PROMPT)
    entry = runner.entry("p", ids, 0, (PROMPT - 1,))
    saved = runner.cuda_graphs
    if graph_prefill and saved:
        ms = timed(lambda: runner.step([entry]), 10, 4)
        out["prefill_graph_replays"] = runner.portion_graph_replays
        out["prefill_graph_ms"] = round(ms, 3)
    runner.cuda_graphs = False                    # (a step with a state record runs eagerly anyway)
    ms = timed(lambda: runner.step([entry]), 5, 3)
    out["prefill_eager_ms"] = round(ms, 3)
    ms = out.get("prefill_graph_ms", ms) if out.get("prefill_graph_replays") else ms
    out["prefill_ms"] = round(ms, 3)
    out["prefill_tok_s"] = round(PROMPT / (ms * 1e-3), 1)
    with StepProfile() as prof:
        runner.step([entry])
    out["prefill_kernels_us"] = prof.summary(1)
    runner.cuda_graphs = saved
    runner.cache.release("p")

    # decode: requests that hold CONTEXT tokens (pages taken, not prefilled: a step's time does
    # not depend on the values in the cache)
    for batch in (8, 64):
        rids = [f"d{batch}-{i}" for i in range(batch)]
        for rid in rids:
            assert runner.cache.open(rid) and runner.cache.ensure(rid, CONTEXT)
            runner.cache.trim(rid, CONTEXT - 1)
        entries = [runner.entry(rid, [1 + i], CONTEXT - 1, (0,)) for i, rid in enumerate(rids)]
        tok = torch.empty(batch, dtype=torch.int32, device="cuda:0")
        ms = timed(lambda: K.sample_rows(runner.step(entries), tok), 50, 10)
        out[f"decode_b{batch}_ms"] = round(ms, 4)
        out[f"decode_b{batch}_tok_s"] = round(batch / (ms * 1e-3), 1)
        runner.cuda_graphs = False
        runner.step(entries)
        with StepProfile() as prof:
            for _ in range(5):
                runner.step(entries)
        out[f"decode_b{batch}_kernels_us"] = prof.summary(5)
        runner.cuda_graphs = saved
        for rid in rids:
            runner.cache.release(rid)
    del engine, runner
    torch.cuda.empty_cache()
    return out


def _kernel_rooflines(size, res: Dict[str, Dict[str, object]], peaks) -> Dict[str, object]:
    """Achieved fractions of the measured peaks for the kernels that differ between the two
    models, per launch.  Attention, decode: bytes of the visible keys (and values, where they
    are stored) of 8 requests over the kernel's time, of the copy bandwidth.  Attention,
    prefill: 4 T W' H D flops (scores and weighted values of the visible pairs; W' the mean
    number of visible keys) over the kernel's time, of the bf16 peak -- the same count for both
    models, so that the fraction says how far each is from the arithmetic the design needs, not
    from what the kernel happens to do.  Elementwise kernels of the 2,048-token prefill: the
    bytes they must move (float32 stream in and out, update in, normed rows out; projection in,
    queries and cache rows out; pair results and gate in, rows out) of the copy bandwidth."""
    width, heads, kv, dim, ff = SIZES[size]
    seen = min(CONTEXT, WINDOW)
    pairs = sum(min(t + 1, WINDOW) for t in range(PROMPT))
    flops = 4.0 * pairs * heads * dim
    qs, ks = heads * dim, kv * dim
    out = {}

    def hbm(nbytes, us):
        return round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)

    for arch, stored, names in (("dezelorn", 1, ("talk_decode_attention", "talk_prefill_attention")),
                                ("qwen2", 2, ("decode_attention", "prefill_attention_tc"))):
        pk, dk = res[arch]["prefill_kernels_us"], res[arch]["decode_b8_kernels_us"]
        dec = dk.get(names[0])
        pre = pk.get(names[1]) or pk.get("prefill_attention")
        if dec:
            out[f"{arch}_decode_attention_us"] = round(dec / LAYERS, 2)
            out[f"{arch}_decode_attention_hbm_frac"] = hbm(8 * seen * kv * dim * 2 * stored, dec / LAYERS)
        if pre:
            out[f"{arch}_prefill_attention_us"] = round(pre / LAYERS, 1)
            out[f"{arch}_prefill_attention_bf16_frac"] = round(
                flops / (pre / LAYERS * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)
    pk = res["dezelorn"]["prefill_kernels_us"]
    if pk.get("dyt_add_norm"):
        us = pk["dyt_add_norm"] / (2 * LAYERS + 1)          # (the last one norms one row only)
        out["dezelorn_norm_us"], out["dezelorn_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if pk.get("qk_conv_cache"):
        us = pk["qk_conv_cache"] / LAYERS
        out["dezelorn_conv_cache_us"], out["dezelorn_conv_cache_hbm_frac"] = round(us, 2), hbm(PROMPT * 4 * (qs + ks), us)
    if pk.get("mix_heads_gate"):
        us = pk["mix_heads_gate"] / LAYERS
        out["dezelorn_mix_gate_us"] = round(us, 2)
        out["dezelorn_mix_gate_hbm_frac"] = hbm(PROMPT * (4 * heads * kv * dim + 4 * qs), us)
    pk = res["qwen2"]["prefill_kernels_us"]
    if pk.get("add_rmsnorm"):
        us = pk["add_rmsnorm"] / (2 * LAYERS + 1)
        out["qwen2_norm_us"], out["qwen2_norm_hbm_frac"] = round(us, 2), hbm(PROMPT * 12 * width, us)
    if pk.get("qkv_rope_cache"):
        us = pk["qkv_rope_cache"] / LAYERS
        out["qwen2_rope_cache_us"], out["qwen2_rope_cache_hbm_frac"] = round(us, 2), hbm(PROMPT * 4 * (qs + 2 * ks), us)
    return out


def run(peaks, note=lambda m: None, sizes=None, design: str = "dezelorn") -> Dict[str, object]:
    if design == "sumolorn":
        result = {"compare": "sumolorn vs daferax (grouped-query and latent attention, dense feed-forward) at equal "
                             "layer sizes", "layers": LAYERS, "prompt": PROMPT, "decode_context": CONTEXT,
                  "window": WINDOW, "vocab": VOCAB, "dtype": "bf16",
                  "data": "synthetic: random weights, token ids uniform over the vocabulary",
                  "peaks": peaks.get("source"), "sizes": {}}
        for size in (sizes or SUMOLORN_SIZES):
            dims = SUMOLORN_SIZES[size]
            res = {}
            for arch, make in (("sumolorn", sumolorn_config), ("daferax", daferax_like_sumolorn)):
                note(f"{size}: {arch}")
                res[arch] = _measure(make(*dims), note, graph_prefill=True)
            res["kernels"] = _sumolorn_rooflines(size, res, peaks)
            res["dims"] = dict(zip(("width", "heads", "kv_heads", "head_dim", "ff", "kv_rank", "rot_dim", "q_rank",
                                    "linear_heads", "linear_key_dim", "linear_value_dim"), dims))
            result["sizes"][size] = res
        return result
    if design == "zimupel":
        result = {"compare": "zimupel vs daferax (grouped-query attention in every layer) at equal layer sizes",
                  "layers": LAYERS, "prompt": PROMPT, "decode_context": CONTEXT, "vocab": VOCAB, "dtype": "bf16",
                  "data": "synthetic: random weights, token ids uniform over the vocabulary",
                  "peaks": peaks.get("source"), "sizes": {}}
        for size in (sizes or ZIMUPEL_SIZES):
            dims = ZIMUPEL_SIZES[size]
            res = {}
            for arch, make in (("zimupel", zimupel_config), ("daferax", daferax_like_zimupel)):
                note(f"{size}: {arch}")
                res[arch] = _measure(make(*dims), note)
            res["kernels"] = _zimupel_rooflines(size, res, peaks)
            res["dims"] = dict(zip(("width", "heads", "kv_heads", "head_dim", "experts", "groups", "keep", "top",
                                    "expert_ff", "streams"), dims))
            result["sizes"][size] = res
        return result
    if design == "daferax":
        result = {"compare": "daferax vs qwen2 at equal layer sizes", "layers": LAYERS, "prompt": PROMPT,
                  "decode_context": CONTEXT, "window": WINDOW, "vocab": VOCAB, "dtype": "bf16",
                  "data": "synthetic: random weights, token ids uniform over the vocabulary",
                  "peaks": peaks.get("source"), "sizes": {}}
        for size in (sizes or DAFERAX_SIZES):
            dims = DAFERAX_SIZES[size]
            res = {}
            for arch, make in (("daferax", daferax_config), ("qwen2", qwen2_like_daferax)):
                note(f"{size}: {arch}")
                res[arch] = _measure(make(*dims), note)
            res["kernels"] = _daferax_rooflines(size, res, peaks)
            res["dims"] = dict(zip(("width", "heads", "kv_heads", "head_dim", "kv_rank", "rot_dim", "experts",
                                    "groups", "keep", "top", "expert_ff", "shared_ff"), dims))
            result["sizes"][size] = res
        return result
    result = {"compare": "dezelorn vs qwen2 at equal layer sizes", "layers": LAYERS, "prompt": PROMPT,
              "decode_context": CONTEXT, "window": WINDOW, "vocab": VOCAB, "dtype": "bf16",
              "data": "synthetic: random weights, token ids uniform over the vocabulary",
              "peaks": peaks.get("source"), "sizes": {}}
    for size in (sizes or SIZES):
        dims = SIZES[size]
        res = {}
        for arch, make in (("dezelorn", dezelorn_config), ("qwen2", qwen2_config)):
            note(f"{size}: {arch}")
            res[arch] = _measure(make(*dims), note)
        res["kernels"] = _kernel_rooflines(size, res, peaks)
        res["dims"] = dict(zip(("width", "heads", "kv_heads", "head_dim", "ff"), dims))
        result["sizes"][size] = res
    return result

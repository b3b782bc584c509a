"""Sumolorn on the CPU: config keys and refusals, the spec it turns into, the order its layers run
in, the tensors it declares, what its mixers ask of the cache, and the oracle's own pieces on cases
worked by hand."""

import copy
import json
import math

import pytest
import torch

import plain_sumolorn as plain
import sumolorn_cases as C
from servelab_b200.cache import CacheManager
from servelab_b200.cache.manager import FixedStateRequest, PagedKVRequest, paged_part, state_part
from servelab_b200.cache.storage import plan_groups
from servelab_b200.config import ConfigError, SumolornConfig, config_from_dict, load_config
from servelab_b200.models.causal_lm import declare_tensors
from servelab_b200.parts import BLOCKS, part_class

F64 = torch.float64


def test_round_trip_and_registry(tmp_path):
    for cfg, _, _ in C.CASES.values():
        typed = config_from_dict(cfg)
        assert isinstance(typed, SumolornConfig) and typed.to_dict() == cfg
        assert hash(typed) == hash(config_from_dict(copy.deepcopy(cfg)))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(C.A, f)
    assert load_config(str(tmp_path)).to_dict() == C.A


def test_every_size_and_constant_reaches_the_spec():
    spec = config_from_dict(C.A).to_model_spec()
    assert spec.vocab_size == 211 and spec.hidden_size == 48 and not spec.tie_word_embeddings
    assert spec.logit_scale == 0.5 and spec.logit_softcap is None and spec.residual_streams is None
    assert all(b.kind == "pre_norm" and b.mixer_norm.unit_offset and b.mixer_norm.eps == 1e-6 for b in spec.layers)
    assert spec.final_norm.unit_offset
    assert [b.mixer.kind for b in spec.layers] == ["latent_attention", "normed_attention", "parallel_mixers",
                                                   "normed_attention"]
    la = spec.layers[0].mixer
    assert (la.num_heads, la.head_dim, la.rope_dim, la.value_dim, la.kv_rank, la.q_rank) == (3, 8, 4, 12, 20, 10)
    assert la.scale == 0.3 and la.window is None and la.sink and la.head_gate and not la.element_gate
    assert (la.position.kind, la.position.dims, la.position.theta) == ("rotary_pairs", 4, 1000.0)
    at = spec.layers[1].mixer
    assert (at.num_heads, at.num_kv_heads, at.head_dim, at.value_dim, at.window, at.scale, at.softcap) == \
        (4, 2, 16, 8, 5, 0.25, 5.0)
    assert at.sink and at.head_gate and not at.qk_unit_norm and not at.qk_norm and at.conv_taps == 0
    p = at.position
    assert (p.kind, p.rotary_dim, p.theta, p.stretch_factor, p.stretch_low, p.stretch_high, p.stretch_original) == \
        ("rotary", 8, 500.0, 8.0, 1.0, 4.0, 16.0)
    par = spec.layers[2].mixer
    assert par.factor == 0.5 and par.eps == 1e-6
    lf, rt = par.left, par.right
    assert (lf.conv_taps, lf.num_heads, lf.num_kv_heads, lf.head_dim, lf.value_dim, lf.scale, lf.window) == \
        (3, 2, 1, 16, 16, 0.2, 9)
    assert lf.qk_unit_norm and not lf.sink and not lf.head_gate and lf.softcap is None
    assert (lf.position.rotary_dim, lf.position.theta, lf.position.stretch_factor) == (16, 100.0, None)
    assert (rt.num_heads, rt.head_dim, rt.value_dim, rt.decay_gate_tau, rt.decay_gate_rank) == (3, 8, 12, 4.0, 6)
    assert rt.decay == () and rt.query_scale == 8 ** -0.5 and rt.key_scale is None
    assert (rt.out_norm, rt.out_norm_weight, rt.out_norm_per_head, rt.gate_activation) == ("head", True, True, "silu")
    last = spec.layers[3].mixer            # kv_heads and vdim left out: as many as heads, as large as dim
    assert (last.num_kv_heads, last.value_dim, last.window, last.softcap) == (2, 8, None, None)
    assert spec.layers[2].feed_forward is None and spec.layers[2].ff_norm is None
    f = spec.layers[1].feed_forward
    assert (f.activation, f.intermediate_size, f.limit, f.swish_alpha) == ("swish_clamped", 24, 0.7, 1.702)


def test_the_order_in_which_layers_run():
    runs = lambda cfg: [r.layer for r in config_from_dict(cfg).to_model_spec().run_order]
    assert runs(C.A) == [0, 1, 2, 1, 2, 1, 2, 3] == plain.layer_runs(C.A)
    assert runs(C.B) == [0, 1, 2, 3]
    assert runs(C.C) == [0, 1, 2, 0, 1, 2]
    assert runs(C.D) == [0, 1, 2, 3] == plain.layer_runs(C.D)           # an empty range, however often
    one = dict(C.B, loop={"start": 3, "stop": 4, "times": 3})
    assert runs(one) == [0, 1, 2, 3, 3, 3] == plain.layer_runs(one)
    assert all(r.cache_of is None for r in config_from_dict(C.A).to_model_spec().run_order)   # a cache a pass


@pytest.mark.parametrize("change, word", [
    (lambda c: c.update(extra=1), "unknown key"),
    (lambda c: c["layers"][1]["mixer"].update(bias=True), "unknown key"),
    (lambda c: c["layers"][1]["mixer"].update(conv=3), "unknown key"),          # taps belong to a left branch
    (lambda c: c["layers"][2]["mixer"]["left"].update(softcap=3.0), "unknown key"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(scaling={"factor": 2.0, "slow": 1}), "unknown key"),
    (lambda c: c["layers"][0].update(type="conv"), "not known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not known"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "malformed"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(tau=0.0), "positive"),
    (lambda c: c["layers"][1]["mlp"].update(limit=0.0), "limit"),
    (lambda c: c.pop("norm"), "missing"),
])
def test_refusals(change, word):
    cfg = copy.deepcopy(C.A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_declared_tensors():
    decls = {d.name: tuple(d.shape) for d in declare_tensors(config_from_dict(C.A).to_model_spec())}
    assert decls["embed"] == (211, 48) and decls["head"] == (211, 48) and decls["final.norm"] == (48,)
    for name, shape in {"l0.mix.dq": (10, 48), "l0.mix.dq.norm": (10,), "l0.mix.uq": (36, 10), "l0.mix.dkv": (24, 48),
                        "l0.mix.dkv.norm": (20,), "l0.mix.uk": (24, 20), "l0.mix.uv": (36, 20), "l0.mix.sink": (3,),
                        "l0.mix.g": (3, 48), "l0.mix.o": (48, 36),
                        "l1.mix.q": (64, 48), "l1.mix.k": (32, 48), "l1.mix.v": (16, 48), "l1.mix.o": (48, 32),
                        "l1.mix.sink": (4,), "l1.mix.g": (4, 48),
                        "l2.mix.left.q": (32, 48), "l2.mix.left.q.conv": (32, 3), "l2.mix.left.k.conv": (16, 3),
                        "l2.mix.left.v.conv": (16, 3), "l2.mix.left.o": (48, 32), "l2.mix.left.out": (48,),
                        "l2.mix.right.out": (48,), "l2.mix.right.q": (24, 48), "l2.mix.right.v": (36, 48),
                        "l2.mix.right.g": (36, 48), "l2.mix.right.o": (48, 36), "l2.mix.right.norm": (12,),
                        "l2.mix.right.a1": (6, 48), "l2.mix.right.a2": (24, 6), "l2.mix.right.a2.b": (24,),
                        "l1.mlp.gate": (24, 48), "l1.mlp.down": (48, 24), "l3.norm2": (48,)}.items():
        assert decls[name] == shape, name
    assert "l2.norm2" not in decls and "l2.mlp.gate" not in decls and "l3.mix.sink" in decls
    assert not any(".left.sink" in n or ".left.g" in n for n in decls)
    # without the key, the bottleneck of the decays is whatever the checkpoint holds
    cfg = copy.deepcopy(C.A)
    cfg["layers"][2]["mixer"]["right"].pop("rank")
    decls = {d.name: tuple(d.shape) for d in declare_tensors(config_from_dict(cfg).to_model_spec())}
    assert decls["l2.mix.right.a1"] == (-1, 48) and decls["l2.mix.right.a2"] == (24, -1)


def test_what_the_mixers_ask_of_the_cache():
    spec = config_from_dict(C.A).to_model_spec()
    req = [part_class(BLOCKS, spec.layers[r.layer]).cache_request(spec.layers[r.layer]) for r in spec.run_order]
    assert req[0] == PagedKVRequest(1, 24, None, tied_values=True)             # one row a token: latent | rotated
    assert req[1] == PagedKVRequest(2, 16, 5, value_dim=8)
    pages, state = paged_part(req[2]), state_part(req[2])
    assert pages == PagedKVRequest(1, 16, 9, value_dim=16)
    conv = (3 - 1) * (2 * 16 + 1 * 16 + 1 * 16)
    assert state == FixedStateRequest((conv + 3 * 8 * 12,))                    # both branches' records, side by side
    assert req[3] == req[1] and req[5] == req[1] and req[4] == req[2]          # every pass its own cache
    groups, of_run = plan_groups(req)
    assert len(groups) == 4 and of_run[1] == of_run[3] == of_run[5] and of_run[2] == of_run[4] == of_run[6]
    # one tap: no record for the convolution; the linear branch still has its state
    spec = config_from_dict(C.B).to_model_spec()
    first = part_class(BLOCKS, spec.layers[0]).cache_request(spec.layers[0])
    assert paged_part(first) == PagedKVRequest(3, 10, 1, value_dim=6)
    assert state_part(first) == FixedStateRequest((1 * 6 * 14,))
    cm = CacheManager([g.request.window for g in plan_groups([first])[0]], 8, 4, 2)
    assert cm.open("a") and cm.ensure("a", 9)
    cm.trim("a", 9)
    assert cm.block_table("a", 0)[:2] == [-1, -1]                              # a window of one token
    cm.release("a")
    cm.check_invariants()


# ------------------------------------------------- the oracle's pieces by hand
def test_oracle_stretched_frequencies():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 16}
    f = plain.scaled_frequencies(8, 500.0, sc)
    raw = [500.0 ** (-2.0 * i / 8) for i in range(4)]
    wl = [2 * math.pi / r for r in raw]
    assert 16 / 4 < wl[0] < 16 / 1 < wl[1]               # the first is blended, the others are stretched
    s0 = (16 / wl[0] - 1.0) / 3.0
    assert abs(float(f[0]) - ((1 - s0) * raw[0] / 8 + s0 * raw[0])) < 1e-15
    assert abs(float(f[0]) - 0.5761) < 1e-4
    assert all(abs(float(f[i]) - raw[i] / 8) < 1e-15 for i in (1, 2, 3))
    short = plain.scaled_frequencies(4, 2.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 4096})
    assert torch.equal(short, 2.0 ** (-2.0 * torch.arange(2, dtype=F64) / 4))          # short wavelengths stay


def test_oracle_convolution_and_recurrence():
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=F64)
    w = torch.tensor([[0.5, 2.0], [1.0, -1.0]], dtype=F64)              # [channels, taps]; the last tap is "now"
    y = plain.short_conv(u, w)
    assert torch.equal(y, torch.tensor([[2.0, -10.0], [4.5, -10.0], [7.0, -10.0]], dtype=F64))
    q = torch.ones(2, 1, 2, dtype=F64)
    k = torch.tensor([[[1.0, 2.0]], [[0.0, 0.0]]], dtype=F64)
    v = torch.tensor([[[3.0]], [[0.0]]], dtype=F64)
    alpha = torch.tensor([[[1.0, 1.0]], [[0.5, 0.25]]], dtype=F64)
    o = plain.gated_linear_attention(q, k, v, alpha)
    assert torch.equal(o.flatten(), torch.tensor([9.0, 0.5 * 3.0 + 0.25 * 6.0], dtype=F64))


def test_oracle_sink_and_cap():
    q = torch.tensor([[[2.0]]], dtype=F64)
    k = torch.tensor([[[3.0]]], dtype=F64)
    v = torch.tensor([[[5.0]]], dtype=F64)
    o = plain.softmax_attention(q, k, v, 0.5, None, 2.0, torch.tensor([1.0]))
    s = 2.0 * math.tanh(3.0 / 2.0)
    assert abs(float(o) - 5.0 * math.exp(s) / (math.exp(s) + math.exp(1.0))) < 1e-12
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(plain.rms_norm(x, torch.tensor([0.5, -0.5], dtype=F64), 0.0, one_plus=True),
                          torch.tensor([[3.0 * 1.5, 4.0 * 0.5]], dtype=F64) / math.sqrt(12.5))

"""Zimupel on the CPU: config keys and refusals, the spec it turns into, the tensors it declares,
what its mixers ask of the cache, and the oracle's own pieces on cases worked by hand."""

import copy
import json
import math

import pytest
import torch

import plain_zimupel as plain
import zimupel_cases as C
from servelab_b200.cache import CacheManager
from servelab_b200.cache.manager import FixedStateRequest, PagedKVRequest, paged_part, state_part
from servelab_b200.cache.storage import plan_groups
from servelab_b200.config import ConfigError, ZimupelConfig, config_from_dict, load_config
from servelab_b200.models.causal_lm import declare_tensors
from servelab_b200.parts import BLOCKS, part_class

F64 = torch.float64


def test_round_trip_and_registry(tmp_path):
    for cfg, _, _ in C.CASES.values():
        typed = config_from_dict(cfg)
        assert isinstance(typed, ZimupelConfig) and typed.to_dict() == cfg
        assert hash(typed) == hash(config_from_dict(copy.deepcopy(cfg)))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(C.P, f)
    assert load_config(str(tmp_path)).to_dict() == C.P


def test_every_size_and_constant_reaches_the_spec():
    spec = config_from_dict(C.P).to_model_spec()
    assert spec.vocab_size == 211 and spec.hidden_size == 48 and not spec.tie_word_embeddings
    assert spec.residual_streams == 2 and spec.logit_scale == 1.5 and spec.logit_softcap == 20.0
    assert spec.embedding_norm.kind == "rmsnorm" and spec.embedding_norm.eps == 1e-6
    assert [b.kind for b in spec.layers] == ["hyper_connections"] * 5 and all(b.streams == 2 for b in spec.layers)
    assert [b.mixer.kind for b in spec.layers] == ["decay_attention", "differential_attention", "decay_attention",
                                                   "differential_attention", "decay_attention"]
    li = spec.layers[0].mixer
    assert (li.num_heads, li.head_dim, li.value_dim, li.decay) == (3, 8, 12, (0.9, 1.0, 0.5))
    assert (li.qkv_activation, li.key_scale, li.out_norm, li.out_norm_weight, li.gate_activation) == \
        ("silu", None, "row", True, "sigmoid")
    assert li.position.kind == "none" and li.out_norm_eps == 1e-6
    re = spec.layers[2].mixer
    assert (re.num_heads, re.head_dim, re.value_dim, re.decay) == (2, 16, 8, (0.97, 0.999))
    assert (re.qkv_activation, re.out_norm, re.out_norm_weight, re.gate_activation) == (None, "head", False, "silu")
    assert re.key_scale == 16 ** -0.5 and (re.position.rotary_dim, re.position.theta) == (8, 500.0)
    assert spec.layers[4].mixer.position.kind == "none"
    a = spec.layers[1].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.scale, a.lambda_init) == (4, 2, 16, 8, 0.25, 0.2)
    assert a.own_kv and a.qkv_bias and not spec.layers[3].mixer.own_kv
    assert [(r.layer, r.cache_of) for r in spec.run_order] == [(0, None), (1, None), (2, None), (3, 1), (4, None)]
    f = spec.layers[0].feed_forward
    assert (f.num_experts, f.top, f.expert_size, f.num_groups, f.keep_groups) == (6, 2, 16, 3, 2)
    assert (f.score_fn, f.correction_name, f.group_best, f.norm_eps, f.renormalize, f.shared) == \
        ("sigmoid", "correction", 2, 1e-20, True, None)
    assert (spec.layers[2].feed_forward.num_groups, spec.layers[2].feed_forward.top) == (1, 1)
    d = spec.layers[1].feed_forward
    assert (d.kind, d.intermediate_size, d.activation) == ("gated_mlp", 40, "gelu_tanh")
    assert spec.layers[3].feed_forward is None
    # without the keys: one residual, no scale, no cap, as many kv heads as heads
    q = config_from_dict(C.Q).to_model_spec()
    assert q.residual_streams is None and q.logit_scale is None and q.logit_softcap is None
    assert [b.kind for b in q.layers] == ["pre_norm"] * 6 and q.layers[4].feed_forward is None and q.layers[1].mixer.num_kv_heads == 3
    assert config_from_dict(C.R).to_model_spec().residual_streams == 1


@pytest.mark.parametrize("change, text", [
    (lambda c: c.update(rope=1), "unknown key"),
    (lambda c: c["layers"][0].update(type="recurrent"), "not known"),
    (lambda c: c["layers"][0]["mixer"].update(window=3), "unknown key"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay factors"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "earlier attention layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier attention layer"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "differs"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "not known"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "kept groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(scale=2.0), "unknown key"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.pop("norm"), "missing key"),
])
def test_refusals(change, text):
    cfg = copy.deepcopy(C.P)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(cfg)


def test_a_chain_of_borrowed_caches_is_refused():
    cfg = copy.deepcopy(C.P)
    cfg["layers"].append(C.layer(C.attention(4, 2, 16, 8, 0.3, 0.1, kv_from=3), None))
    with pytest.raises(ConfigError, match="projections of its own"):
        config_from_dict(cfg)


def test_declared_tensors():
    spec = config_from_dict(C.P).to_model_spec()
    d = {t.name: tuple(t.shape) for t in declare_tensors(spec)}
    assert d["embed"] == (211, 48) and d["head"] == (211, 48) and d["embed.norm"] == (48,) and d["final.norm"] == (48,)
    assert d["l0.mix.q"] == (24, 48) and d["l0.mix.v"] == (36, 48) and d["l0.mix.g"] == (36, 48)
    assert d["l0.mix.o"] == (48, 36) and d["l0.mix.norm"] == (36,)
    assert d["l0.hc1.in"] == (2,) and d["l0.hc2.out"] == (2,) and d["l0.hc1.mix"] == (2, 2)
    assert d["l0.mlp.router"] == (6, 48) and d["l0.mlp.correction"] == (6,) and d["l0.mlp.e5.down"] == (48, 16)
    assert d["l1.mix.q"] == (128, 48) and d["l1.mix.q.b"] == (128,) and d["l1.mix.k"] == (64, 48)
    assert d["l1.mix.v.b"] == (16,) and d["l1.mix.o"] == (48, 32) and d["l1.mix.lk2"] == (16,)
    assert d["l1.mlp.gate"] == (40, 48) and "l2.mix.norm" not in d and d["l2.mix.g"] == (16, 48)
    # the layer that borrows keys and values has no projections for them, and no feed-forward
    assert "l3.mix.k" not in d and "l3.mix.v.b" not in d and d["l3.mix.q"] == (128, 48)
    assert "l3.hc2.in" not in d and "l3.norm2" not in d and "l3.mlp.gate" not in d
    # no streams: no hyper-connection weights at all
    dq = {t.name for t in declare_tensors(config_from_dict(C.Q).to_model_spec())}
    assert not any(".hc" in n for n in dq) and "l0.norm2" in dq
    dr = {t.name: tuple(t.shape) for t in declare_tensors(config_from_dict(C.R).to_model_spec())}
    assert dr["l0.hc1.mix"] == (1, 1)


def test_cache_requests():
    spec = config_from_dict(C.P).to_model_spec()
    reqs = [part_class(BLOCKS, b).cache_request(b) for b in spec.layers]
    assert state_part(reqs[0]) == FixedStateRequest((3, 8, 12)) and paged_part(reqs[0]) is None
    assert state_part(reqs[2]) == FixedStateRequest((2, 16, 8))
    # a kv head's two maps are one cached key row
    assert paged_part(reqs[1]) == PagedKVRequest(2, 32, None, value_dim=8) and state_part(reqs[1]) is None
    from servelab_b200.models.causal_lm import CausalLM
    from servelab_b200.parts import BuildEnv
    model = CausalLM(spec, BuildEnv(device="cpu", dtype=torch.float32, page_size=8))
    per_run = model.cache_requests()
    assert per_run[3] is None and per_run[1] is not None
    groups, of_layer = plan_groups(per_run)
    assert len(groups) == 1 and of_layer == {1: 0}
    cm = CacheManager([None], 6, 8, 2)
    assert cm.open("a") and cm.ensure("a", 40) and not cm.ensure("a", 49)
    cm.release("a")
    cm.check_invariants()


# ------------------------------------------------------------ the oracle itself
def test_the_closed_form_of_the_recurrence_equals_its_steps():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(9, 3, 5, generator=g, dtype=F64), torch.randn(9, 3, 5, generator=g, dtype=F64)
    v = torch.randn(9, 3, 4, generator=g, dtype=F64)
    for decay in ((0.9, 1.0, 0.25), (1.0, 1.0, 1.0)):
        assert (plain.decayed_sum(q, k, v, decay) - plain.decayed_sum_stepwise(q, k, v, decay)).abs().max() < 1e-12
    # by hand: two tokens, one head of one element
    one = lambda *x: torch.tensor(x, dtype=F64).view(-1, 1, 1)
    o = plain.decayed_sum(one(2.0, 3.0), one(5.0, 7.0), one(11.0, 13.0), (0.5,))
    assert o.flatten().tolist() == [2 * 5 * 11, 3 * (0.5 * 5 * 11 + 7 * 13)]


def test_rotation_pairs_element_i_with_i_plus_half():
    x = torch.zeros(1, 1, 6, dtype=F64)
    x[0, 0] = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0])
    out = plain.rotate_halves(x, torch.tensor([3]), 4, 100.0)[0, 0]
    f = [1.0, 100.0 ** -0.5]
    for i in range(2):
        a = 3 * f[i]
        u, v = [1.0, 2.0][i], [3.0, 4.0][i]
        assert abs(out[i] - (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(out[i + 2] - (v * math.cos(a) + u * math.sin(a))) < 1e-12
    assert out[4:].tolist() == [5.0, 6.0]


def test_router_by_hand():
    # scores 0.5 everywhere but where stated; offsets decide the choice, not the weights
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    z = torch.zeros(1, 6, dtype=F64)
    z[0, 4] = math.log(3.0)                 # sigmoid = 0.75
    corr = torch.tensor([0.4, 0.4, 0.0, 0.0, 0.0, 0.0], dtype=F64)
    ids, w = plain.route(z, corr, r)
    # groups score 0.9 + 0.9, 0.5 + 0.5, 0.75 + 0.5: the first wins although expert 4 is the best alone
    assert sorted(ids[0].tolist()) == [0, 1] and torch.allclose(w, torch.full((1, 2), 0.5, dtype=F64))
    # negative choice scores: experts outside the kept group must count as minus infinity, not 0
    corr = torch.tensor([-2.0, -2.0, -3.0, -3.0, -3.0, -3.5], dtype=F64)
    ids, w = plain.route(z, corr, r)
    assert sorted(ids[0].tolist()) == [0, 1]
    ids, w = plain.route(z, torch.zeros(6, dtype=F64), {"experts": 6, "top": 3})
    assert ids[0, 0] == 4 and abs(float(w.sum()) - 1.0) < 1e-12 and abs(float(w[0, 0]) - 0.75 / 1.75) < 1e-12


def test_lambda_and_the_tanh_form_of_gelu():
    W = {"m.lq1": torch.tensor([0.5, 1.0]), "m.lk1": torch.tensor([2.0, -1.0]),
         "m.lq2": torch.tensor([1.0, 1.0]), "m.lk2": torch.tensor([0.0, 0.5])}
    assert abs(plain.differential_lambda(W, "m.", 0.3) - (1.0 - math.exp(0.5) + 0.3)) < 1e-12
    z = torch.tensor([-3.0, 0.0, 0.7, 4.0], dtype=F64)
    assert (plain.gelu_tanh(z) - torch.nn.functional.gelu(z, approximate="tanh")).abs().max() < 1e-12

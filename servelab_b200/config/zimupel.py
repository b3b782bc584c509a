"""Typed configuration of the Zimupel decoder, read from its config.json keys.

A Zimupel model is a stack of pre-norm layers that config.json lists one by one (``layers[i]``:
``type`` names the mixer, ``mixer`` holds its sizes and constants, ``mlp`` the feed-forward or null).
Layers may differ in every size and in their order.  With ``streams`` the residual is kept as that
many parallel copies (hyper-connections: learned read, write and mixing weights per sublayer);
without the key it is the usual single stream, x <- x + f(norm(x)).  The embedded tokens pass an RMS
norm of their own; the output is the final RMS norm, an untied head, ``logit_scale`` and the soft cap
``logit_softcap`` (each applied only if the key is there).

Mixers: ``retention`` -- linear attention with a fixed decay per head (``decay``), rotate-half
rotation on the first ``rot.dims`` elements of q and k, keys times dim^-1/2, every head's result
divided by its root mean square, a SiLU gate; ``lightning`` -- the same recurrence on SiLU-activated
q, k and v with no rotation and no key factor, an RMS norm with a weight over all heads together, a
sigmoid gate; ``attention`` -- differential attention: grouped-query softmax attention with two maps
a head, biases on q, k and v, no rotation, ``scale`` on the scores, o = a_1 - lambda a_2 normed per
head and times 1 - ``diff``; with ``kv_from: j`` the layer has no key and value projections and reads
the cache of layer j.  Feed-forward ``dense``: a gated feed-forward with the tanh form of GELU;
``moe``: sigmoid router, a learned offset per expert in the choice only, groups that score as the sum
of their two best, the chosen experts' scores renormalised (sum + 1e-20), SiLU experts.

Any other key is an error: a key that is not read would be a mechanism that is not computed.

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``head``, and under ``l<i>.``: ``norm1``,
``norm2``, ``hc1.{in,out,mix}``, ``hc2.{in,out,mix}``; ``mix.{q,k,v,g,o}`` (+ ``mix.norm``);
``mix.{q,k,v}`` (+ ``.b``), ``mix.o``, ``mix.{lq1,lk1,lq2,lk2}``; ``mlp.{gate,up,down}``;
``mlp.router``, ``mlp.correction``, ``mlp.e<j>.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .daferax import _freeze, _only, _thaw
from .qwen2 import ConfigError
from .specs import (BlockSpec, DecayAttentionSpec, DifferentialAttentionSpec, GatedMLPSpec, LayerRun,
                    ModelSpec, NoPositionSpec, RMSNormSpec, RotarySpec, RoutedExpertsSpec)

_MAX_POSITIONS = 1 << 20          # nothing in the model bounds the positions

_MIXER_KEYS = {
    "retention": ("heads", "dim", "vdim", "decay", "rot"),
    "lightning": ("heads", "dim", "vdim", "decay"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "diff", "kv_from"),
}
GROUP_BEST = 2                    # a group of experts scores as the sum of its two best
ROUTE_NORM_EPS = 1e-20            # in the denominator of the renormalised weights


@dataclass(frozen=True)
class ZimupelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]               # the entries of config.json's ``layers``, frozen
    streams: Optional[int] = None
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Zimupel"
    model_type = "zimupel"

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "ZimupelConfig":
        p = []
        _only(cfg, ("architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "streams",
                    "logit_scale", "logit_softcap", "eos_token_id"), "config", p)
        for key in ("vocab", "width", "norm", "layers"):
            if key not in cfg:
                p.append(f"missing key '{key}'")
        if p:
            raise ConfigError("invalid Zimupel config: " + "; ".join(p))
        _only(cfg["norm"], ("eps",), "norm", p)
        if p:
            raise ConfigError("invalid Zimupel config: " + "; ".join(p))
        eos = cfg.get("eos_token_id", ())
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)

        def number(key, kind):
            return None if cfg.get(key) is None else kind(cfg[key])
        out = cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]),
                  layers=tuple(_freeze(layer) for layer in cfg["layers"]), streams=number("streams", int),
                  logit_scale=number("logit_scale", float), logit_softcap=number("logit_softcap", float),
                  eos_token_ids=eos_ids)
        out.to_model_spec()                # every per-layer check happens there
        return out

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": [_thaw(layer) for layer in self.layers]}
        for key in ("streams", "logit_scale", "logit_softcap"):
            if getattr(self, key) is not None:
                d[key] = getattr(self, key)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------- the model as plain data
    def _mixer(self, i: int, kind: str, m: dict, entries, p):
        where = f"layers[{i}].mixer"
        _only(m, _MIXER_KEYS[kind], where, p)
        heads, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        if min(heads, dim, vdim) <= 0:
            p.append(f"{where}: heads, dim and vdim must be positive")
        if kind in ("retention", "lightning"):
            decay = tuple(float(d) for d in m["decay"])
            if len(decay) != heads:
                p.append(f"{where}: {len(decay)} decay factors for {heads} heads")
            if kind == "lightning":
                return DecayAttentionSpec(
                    hidden_size=self.width, num_heads=heads, head_dim=dim, value_dim=vdim, decay=decay,
                    qkv_activation="silu", out_norm="row", out_norm_weight=True, out_norm_eps=self.norm_eps,
                    gate_activation="sigmoid")
            position = NoPositionSpec()
            rot = m.get("rot")
            if rot:
                _only(rot, ("base", "dims"), where + ".rot", p)
                dims = int(rot["dims"])
                if dims % 2 or not 0 < dims <= dim:
                    p.append(f"{where}.rot.dims must be even, positive and at most dim")
                position = RotarySpec(head_dim=dim, rotary_dim=dims, theta=float(rot["base"]))
            return DecayAttentionSpec(
                hidden_size=self.width, num_heads=heads, head_dim=dim, value_dim=vdim, decay=decay,
                position=position, key_scale=dim ** -0.5, out_norm="head", out_norm_weight=False,
                out_norm_eps=self.norm_eps, gate_activation="silu")
        kv_heads = int(m.get("kv_heads", heads))
        if kv_heads <= 0 or heads % kv_heads:
            p.append(f"{where}: heads must be a multiple of kv_heads")
        src = m.get("kv_from")
        if src is not None:
            src = int(src)
            other = entries[src] if 0 <= src < i else None
            om = (other or {}).get("mixer") or {}
            if other is None or other.get("type") != "attention" or om.get("kv_from") is not None:
                p.append(f"{where}.kv_from must name an earlier attention layer with projections of its own")
            elif (int(om.get("kv_heads", om["heads"])), int(om["dim"]), int(om["vdim"])) != (kv_heads, dim, vdim):
                p.append(f"{where}.kv_from: layer {src} differs in kv_heads, dim or vdim")
        return DifferentialAttentionSpec(
            hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
            scale=float(m["scale"]), lambda_init=float(m["diff"]), norm_eps=self.norm_eps, qkv_bias=True,
            own_kv=src is None)

    def _feed_forward(self, i: int, mlp: dict, p):
        where = f"layers[{i}].mlp"
        kind = mlp.get("kind")
        if kind == "dense":
            _only(mlp, ("kind", "ff"), where, p)
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="gelu_tanh",
                                gate_name="gate", up_name="up", down_name="down", weight_suffix="")
        if kind != "moe":
            p.append(f"{where}: kind {kind!r} is not known (moe, dense)")
            return None
        _only(mlp, ("kind", "expert", "router"), where, p)
        r = mlp.get("router") or {}
        _only(r, ("experts", "groups", "top"), where + ".router", p)
        _only(mlp.get("expert") or {}, ("ff",), where + ".expert", p)
        groups = r.get("groups") or {}
        _only(groups, ("count", "keep"), where + ".router.groups", p)
        experts, top = int(r["experts"]), int(r["top"])
        count = int(groups.get("count", 1))
        keep = int(groups.get("keep", count))
        if experts <= 0 or count <= 0 or experts % count or not 0 < keep <= count \
                or not 0 < top <= experts // count * keep:
            p.append(f"{where}.router: experts must split into groups.count equal groups, "
                     f"0 < keep <= count, and top experts must fit into the kept groups")
        return RoutedExpertsSpec(
            hidden_size=self.width, num_experts=experts, top=top, expert_size=int(mlp["expert"]["ff"]),
            num_groups=count, keep_groups=keep, route_scale=1.0, renormalize=True, score_fn="sigmoid",
            correction_name="correction", group_best=GROUP_BEST, norm_eps=ROUTE_NORM_EPS)

    def to_model_spec(self) -> ModelSpec:
        p = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not self.layers:
            p.append("the model has no layers")
        if self.streams is not None and self.streams < 1:
            p.append("streams must be at least 1")
        norm = RMSNormSpec(dim=self.width, eps=self.norm_eps, weight_suffix="")
        entries = [_thaw(layer) for layer in self.layers]
        layers, runs = [], []
        for i, entry in enumerate(entries):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}]", p)
            kind = entry.get("type")
            if kind not in _MIXER_KEYS:
                p.append(f"layers[{i}]: mixer type {kind!r} is not known ({', '.join(_MIXER_KEYS)})")
                continue
            try:
                mixer = self._mixer(i, kind, entry.get("mixer") or {}, entries, p)
                ff = self._feed_forward(i, entry["mlp"], p) if entry.get("mlp") else None
            except (KeyError, TypeError, ValueError) as e:
                p.append(f"layers[{i}]: missing or malformed key {e}")
                continue
            layers.append(BlockSpec(
                kind="pre_norm" if self.streams is None else "hyper_connections", mixer=mixer, feed_forward=ff,
                mixer_norm=norm, ff_norm=None if ff is None else norm, mixer_norm_name="norm1",
                mixer_name="mix", ff_norm_name="norm2", feed_forward_name="mlp", streams=self.streams or 1))
            src = (entry.get("mixer") or {}).get("kv_from") if kind == "attention" else None
            runs.append(LayerRun(i, cache_of=None if src is None else int(src)))
        if p:
            raise ConfigError("invalid Zimupel config: " + "; ".join(p))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            layers=tuple(layers), run_order=tuple(runs), final_norm=norm, tie_word_embeddings=False,
            max_position_embeddings=_MAX_POSITIONS, eos_token_ids=self.eos_token_ids, embed_name="embed",
            lm_head_name="head", final_norm_prefix="final.norm", layer_prefix="l{}",
            embedding_norm=norm, embedding_norm_prefix="embed.norm", residual_streams=self.streams,
            logit_scale=self.logit_scale, logit_softcap=self.logit_softcap,
            # a layer without a feed-forward has no use for its second norm and stream weights; a
            # checkpoint may hold them all the same
            ignored_suffixes=(".norm2", ".hc2.in", ".hc2.out", ".hc2.mix"))

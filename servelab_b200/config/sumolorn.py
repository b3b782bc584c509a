"""Typed configuration of the Sumolorn decoder, read from its config.json keys.

A Sumolorn model is a stack of pre-norm layers that config.json lists one by one (``layers[i]``:
``type`` names the mixer, ``mixer`` holds its sizes and constants, ``mlp`` the feed-forward or null),
x <- x + mix(N(x)), x <- x + ff(N(x)) with RMS norms whose stored weight lies around zero (the factor
is 1 + w).  ``loop`` = {start, stop, times}: the layers start .. stop - 1 run ``times`` times in a row
with the same weights, each pass with a cache and state of its own.  The output is the final norm, an
untied head and ``logit_scale``.

Mixers: ``attention`` -- grouped-query softmax attention, rotation of element i with element
i + dims / 2 over the first ``rot.dims`` elements of a head (``rot.scaling``: long wavelengths
stretched), scores times ``scale`` then soft-capped by ``softcap``, a sliding window ``mask.size``, a
learned sink a head in the softmax's denominator, a sigmoid gate a head; ``latent_attention`` -- keys
and values expanded from one cached latent a token (``kv_rank``) plus a rotated part shared by the
heads (``rot_dim``, neighbouring pairs), queries through a latent of their own (``q_rank``), every
earlier key, a sink and a gate a head; ``parallel`` -- two mixers on the same input, each result
RMS-normed over the width, half their sum: ``left`` a windowed grouped-query attention with a causal
convolution of ``conv`` taps on q, k and v, rotation, then q and k divided by their root mean square
a head; ``right`` a linear attention whose state decays per key channel and token,
alpha = sigmoid(z)^(1 / ``tau``), results normed a head and gated by SiLU.  Feed-forward ``dense``:
g = min(gate, limit), u = clamp(up, -limit, limit), down(g sigmoid(1.702 g) (u + 1)).

Any other key is an error: a key that is not read would be a mechanism that is not computed.

Tensor names: ``embed``, ``final.norm``, ``head``, and under ``l<i>.``: ``norm1``, ``norm2``;
``mix.{q,k,v,o,g,sink}``; ``mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o,g,sink}``;
``mix.left.{q,k,v,o}`` with ``.conv`` taps, ``mix.right.{q,k,v,g,o,norm,a1,a2,a2.b}``,
``mix.left.out``, ``mix.right.out``; ``mlp.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .daferax import _freeze, _only, _thaw
from .qwen2 import ConfigError
from .specs import (BlockSpec, DecayAttentionSpec, GatedMLPSpec, LatentAttentionSpec, LayerRun, ModelSpec,
                    NoPositionSpec, NormedAttentionSpec, PairRotarySpec, ParallelMixersSpec, RMSNormSpec,
                    RotarySpec)

_MAX_POSITIONS = 1 << 20          # nothing in the model bounds the positions
SWISH_ALPHA = 1.702               # g sigmoid(1.702 g) in the feed-forward
BRANCH_FACTOR = 0.5               # a parallel mixer returns half the sum of its two normed branches

_MIXER_TYPES = ("attention", "latent_attention", "parallel")


def _stretch(rot: dict, where: str, p) -> dict:
    sc = rot.get("scaling")
    if not sc:
        return {}
    _only(sc, ("factor", "low", "high", "original"), where + ".scaling", p)
    return dict(stretch_factor=float(sc["factor"]), stretch_low=float(sc["low"]),
                stretch_high=float(sc["high"]), stretch_original=float(sc["original"]))


def _window(m: dict, where: str, p) -> Optional[int]:
    mask = m.get("mask")
    if not mask:
        return None
    _only(mask, ("size",), where + ".mask", p)
    size = int(mask["size"])
    if size < 1:
        p.append(f"{where}.mask.size must be at least 1")
    return size


@dataclass(frozen=True)
class SumolornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]               # the entries of config.json's ``layers``, frozen
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    logit_scale: Optional[float] = None
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Sumolorn"
    model_type = "sumolorn"

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "SumolornConfig":
        p = []
        _only(cfg, ("architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "loop",
                    "logit_scale", "eos_token_id"), "config", p)
        for key in ("vocab", "width", "norm", "layers"):
            if key not in cfg:
                p.append(f"missing key '{key}'")
        if p:
            raise ConfigError("invalid Sumolorn config: " + "; ".join(p))
        _only(cfg["norm"], ("eps",), "norm", p)
        loop = cfg.get("loop")
        if loop:
            _only(loop, ("start", "stop", "times"), "loop", p)
        if p:
            raise ConfigError("invalid Sumolorn config: " + "; ".join(p))
        eos = cfg.get("eos_token_id", ())
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        try:
            out = cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]),
                      layers=tuple(_freeze(layer) for layer in cfg["layers"]),
                      loop=(int(loop["start"]), int(loop["stop"]), int(loop["times"])) if loop else None,
                      logit_scale=None if cfg.get("logit_scale") is None else float(cfg["logit_scale"]),
                      eos_token_ids=eos_ids)
        except (KeyError, TypeError, ValueError) as e:
            raise ConfigError(f"invalid Sumolorn config: missing or malformed key {e}") from None
        out.to_model_spec()                # every per-layer check happens there
        return out

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": [_thaw(layer) for layer in self.layers]}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.logit_scale is not None:
            d["logit_scale"] = self.logit_scale
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------- the model as plain data
    def _softmax_attention(self, m: dict, where: str, p, branch: bool) -> NormedAttentionSpec:
        """The grouped-query attention: the ``attention`` mixer (soft cap, sink, gate a head), or the
        left branch of a ``parallel`` mixer (convolution, unit-normed heads, plain softmax)."""
        keys = ("heads", "kv_heads", "dim", "vdim", "mask", "rot", "scale")
        _only(m, keys + (("conv",) if branch else ("softcap",)), where, p)
        heads, dim = int(m["heads"]), int(m["dim"])
        kv_heads, vdim = int(m.get("kv_heads", heads)), int(m.get("vdim", dim))
        if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
            p.append(f"{where}: heads must be a positive multiple of kv_heads; dim and vdim positive")
        position = NoPositionSpec()
        rot = m.get("rot")
        if rot:
            _only(rot, ("base", "dims", "scaling"), where + ".rot", p)
            dims = int(rot["dims"])
            if dims % 2 or not 0 < dims <= dim:
                p.append(f"{where}.rot.dims must be even, positive and at most dim")
            position = RotarySpec(head_dim=dim, rotary_dim=dims, theta=float(rot["base"]), precise=True,
                                  **_stretch(rot, where + ".rot", p))
        taps = int(m.get("conv", 0)) if branch else 0
        if taps < 0:
            p.append(f"{where}.conv must not be negative")
        cap = m.get("softcap")
        return NormedAttentionSpec(
            hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
            window=_window(m, where, p), scale=float(m["scale"]), qk_norm=False, qk_norm_eps=self.norm_eps,
            position=position, head_gate=not branch, conv_taps=taps, qk_unit_norm=branch,
            softcap=None if cap is None else float(cap), sink=not branch)

    def _latent(self, m: dict, where: str, p) -> LatentAttentionSpec:
        _only(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "rot", "scale", "mask"), where, p)
        heads, dim, rot_dim, vdim, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        if min(heads, dim, rot_dim, vdim, rank) <= 0 or rot_dim % 2:
            p.append(f"{where}: heads, dim, vdim, kv_rank must be positive and rot_dim positive and even")
        rot = m.get("rot") or {}
        _only(rot, ("base", "dims", "scaling"), where + ".rot", p)
        if int(rot.get("dims", rot_dim)) != rot_dim:
            p.append(f"{where}.rot.dims must equal rot_dim")
        position = PairRotarySpec(dims=rot_dim, theta=float(rot["base"]), **_stretch(rot, where + ".rot", p))
        q_rank = m.get("q_rank")
        return LatentAttentionSpec(
            hidden_size=self.width, num_heads=heads, head_dim=dim, rope_dim=rot_dim, value_dim=vdim, kv_rank=rank,
            window=_window(m, where, p), scale=float(m["scale"]), latent_norm_eps=self.norm_eps, position=position,
            head_gate=True, q_rank=None if q_rank is None else int(q_rank), sink=True)

    def _gated_decay(self, m: dict, where: str, p) -> DecayAttentionSpec:
        # (``rank``, the bottleneck of the decay's projection, is optional: a checkpoint's a1 decides it)
        _only(m, ("heads", "dim", "vdim", "tau", "rank"), where, p)
        heads, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        if min(heads, dim, vdim) <= 0 or float(m["tau"]) <= 0:
            p.append(f"{where}: heads, dim, vdim and tau must be positive")
        return DecayAttentionSpec(
            hidden_size=self.width, num_heads=heads, head_dim=dim, value_dim=vdim, decay=(),
            out_norm="head", out_norm_weight=True, out_norm_per_head=True, out_norm_eps=self.norm_eps,
            gate_activation="silu", decay_gate_rank=int(m.get("rank", -1)), decay_gate_tau=float(m["tau"]), query_scale=dim ** -0.5)

    def _mixer(self, i: int, kind: str, m: dict, p):
        where = f"layers[{i}].mixer"
        if kind == "attention":
            return self._softmax_attention(m, where, p, branch=False)
        if kind == "latent_attention":
            return self._latent(m, where, p)
        _only(m, ("left", "right"), where, p)
        return ParallelMixersSpec(
            hidden_size=self.width, left=self._softmax_attention(m["left"], where + ".left", p, branch=True),
            right=self._gated_decay(m["right"], where + ".right", p), eps=self.norm_eps, factor=BRANCH_FACTOR)

    def _feed_forward(self, i: int, mlp: dict, p):
        where = f"layers[{i}].mlp"
        kind = mlp.get("kind", "dense")
        if kind != "dense":
            p.append(f"{where}: kind {kind!r} is not known (dense)")
            return None
        _only(mlp, ("kind", "ff", "limit"), where, p)
        if float(mlp["limit"]) <= 0:
            p.append(f"{where}.limit must be positive")
        return GatedMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="swish_clamped",
                            limit=float(mlp["limit"]), swish_alpha=SWISH_ALPHA, gate_name="gate", up_name="up",
                            down_name="down", weight_suffix="")

    def run_layers(self) -> Tuple[int, ...]:
        """The layers in the order they run, a looped layer once per pass."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, n))

    def to_model_spec(self) -> ModelSpec:
        p = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not self.layers:
            p.append("the model has no layers")
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start <= stop <= len(self.layers) or times < 1:
                p.append("loop: 0 <= start <= stop <= number of layers and times >= 1 are needed")
        norm = RMSNormSpec(dim=self.width, eps=self.norm_eps, weight_suffix="", unit_offset=True)
        layers = []
        for i, entry in enumerate(_thaw(layer) for layer in self.layers):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}]", p)
            kind = entry.get("type")
            if kind not in _MIXER_TYPES:
                p.append(f"layers[{i}]: mixer type {kind!r} is not known ({', '.join(_MIXER_TYPES)})")
                continue
            try:
                mixer = self._mixer(i, kind, entry.get("mixer") or {}, p)
                ff = self._feed_forward(i, entry["mlp"], p) if entry.get("mlp") else None
            except (KeyError, TypeError, ValueError) as e:
                p.append(f"layers[{i}]: missing or malformed key {e}")
                continue
            layers.append(BlockSpec(kind="pre_norm", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    ff_norm=None if ff is None else norm, mixer_norm_name="norm1",
                                    mixer_name="mix", ff_norm_name="norm2", feed_forward_name="mlp"))
        if p:
            raise ConfigError("invalid Sumolorn config: " + "; ".join(p))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            layers=tuple(layers), run_order=tuple(LayerRun(i) for i in self.run_layers()), final_norm=norm,
            tie_word_embeddings=False, max_position_embeddings=_MAX_POSITIONS, eos_token_ids=self.eos_token_ids,
            embed_name="embed", lm_head_name="head", final_norm_prefix="final.norm", layer_prefix="l{}",
            logit_scale=self.logit_scale,
            # a layer without a feed-forward has no use for its second norm; a checkpoint may hold it
            ignored_suffixes=(".norm2",))

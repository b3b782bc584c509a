"""Linear attention with a fixed decay per head (spec: ``DecayAttentionSpec``): the mixer of
retention-like and lightning-like layers.

Per step, with h the mixer's input [T, hidden]:

  1. one product for q | k | v | gate (their matrices are concatenated at load);
  2. one kernel for the recurrence S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t over the
     tokens of every request in order, with the optional activation, rotation and key factor
     applied to q, k and v as they are loaded; S lives in the request's state slot (float32) and is
     carried from step to step, so a prompt may be cut anywhere;
  3. one kernel for the norm of the result (per head without a weight, or over the whole row with
     one) times act(gate);
  4. the output projection.

Nothing is paged: a request holds ``heads x head_dim x value_dim`` floats per layer whatever its
length.
"""

from __future__ import annotations

import torch

from ..cache.manager import FixedStateRequest
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.source import MATRIX, NORM, TensorDecl
from .base import Mixer
from .normed_attention import pad_rows
from .registry import register_mixer


@register_mixer("decay_attention")
class DecayAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        s = spec
        if min(s.num_heads, s.head_dim, s.value_dim) <= 0:
            raise ValueError("decay_attention: heads, head_dim and value_dim must be positive")
        if len(s.decay) != s.num_heads:
            raise ValueError(f"decay_attention: {len(s.decay)} decay factors for {s.num_heads} heads")
        if s.qkv_activation not in (None, "silu"):
            raise ValueError(f"decay_attention: qkv_activation {s.qkv_activation!r} (None, 'silu')")
        if s.out_norm not in ("head", "row"):
            raise ValueError(f"decay_attention: out_norm {s.out_norm!r} ('head', 'row')")
        if s.gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"decay_attention: gate_activation {s.gate_activation!r} ('silu', 'sigmoid')")
        self.rot_dims, self.freq = 0, None
        if s.position.kind == "rotary":
            rd = s.position.rotary_dim or s.head_dim
            if rd % 2 or not 0 < rd <= s.head_dim:
                raise ValueError(f"decay_attention: rotary_dim {rd} must be even and at most head_dim")
            # frequencies formed in float64 and rounded once
            f = float(s.position.theta) ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / rd)
            self.rot_dims, self.freq = rd, f.to(torch.float32).to(env.device)
        elif s.position.kind != "none":
            raise ValueError(f"decay_attention: position {s.position.kind!r} (rotary or none)")
        self.decay = torch.tensor(list(s.decay), dtype=torch.float64).to(torch.float32).to(env.device)
        self.q_size = s.num_heads * s.head_dim
        self.v_size = s.num_heads * s.value_dim
        self.key_scale = 1.0 if s.key_scale is None else float(s.key_scale)

    @classmethod
    def _names(cls, spec, prefix):
        return {n: f"{prefix}.{getattr(spec, n + '_name')}" for n in ("q", "k", "v", "gate", "o", "out_norm")}

    @classmethod
    def declare(cls, spec, prefix):
        h, qs, vs = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_heads * spec.value_dim
        n = cls._names(spec, prefix)
        out = [TensorDecl(n["q"], (qs, h), MATRIX), TensorDecl(n["k"], (qs, h), MATRIX),
               TensorDecl(n["v"], (vs, h), MATRIX), TensorDecl(n["gate"], (vs, h), MATRIX),
               TensorDecl(n["o"], (h, vs), MATRIX)]
        if spec.out_norm_weight:
            out.append(TensorDecl(n["out_norm"], (vs,), NORM))
        return out

    @classmethod
    def cache_request(cls, spec):
        return FixedStateRequest((spec.num_heads, spec.head_dim, spec.value_dim))

    def load(self, store):
        n = self._names(self.spec, self.prefix)
        self.w_in = pad_rows(store.cat([n["q"], n["k"], n["v"], n["gate"]]))
        self.w_o = store.get(n["o"])
        self.norm_w = store.get(n["out_norm"]) if self.spec.out_norm_weight else None

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T = x.shape[0]
        proj = K.plain_unless(None, linear(x, self.w_in))              # [T, q | k | v | gate]
        o = torch.empty((T, self.v_size), dtype=torch.float32, device=x.device)
        K.decay_attention(proj, ctx, cache.state, self.decay, o, q_off=0, k_off=self.q_size,
                          v_off=2 * self.q_size, num_heads=s.num_heads, head_dim=s.head_dim,
                          value_dim=s.value_dim, activation=s.qkv_activation, freq=self.freq,
                          rot_dims=self.rot_dims, key_scale=self.key_scale)
        gate = proj[:, 2 * self.q_size + self.v_size:2 * self.q_size + 2 * self.v_size]
        out = torch.empty((T, self.v_size), dtype=x.dtype, device=x.device)
        groups, size = (s.num_heads, s.value_dim) if s.out_norm == "head" else (1, self.v_size)
        K.group_norm_gate(o, groups, size, out, eps=s.out_norm_eps, weight=self.norm_w, gate=gate,
                          gate_activation=s.gate_activation)
        return linear(out, self.w_o, consumer="norm")

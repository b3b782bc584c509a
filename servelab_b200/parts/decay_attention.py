"""Linear attention with a fixed decay per head (spec: ``DecayAttentionSpec``): the mixer of
retention-like and lightning-like layers -- or, with ``decay_gate_rank``, with a decay of its own
for every token and key channel, alpha_t = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau) (the product with
W_a1 is part of the first product; the one with W_a2 returns float32, and the sigmoid, its
logarithm and the power are formed in float32 inside the recurrence's kernel).

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
from ..weights.source import BIAS, MATRIX, NORM, TensorDecl
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
        self.gated = s.decay_gate_rank is not None
        # (the kernels for learned decays skip requests without tokens and tiles of padding)
        self.padded_steps_safe = self.gated
        if self.gated and (s.decay or not s.decay_gate_tau > 0):
            raise ValueError("decay_attention: learned decays take no fixed ``decay`` and a positive tau")
        if not self.gated and len(s.decay) != s.num_heads:
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
        self.decay = (None if self.gated else
                      torch.tensor(list(s.decay), dtype=torch.float64).to(torch.float32).to(env.device))
        self.out_dtype = None                  # (set by a mixer that wraps this one)
        self.query_scale = 1.0 if s.query_scale is None else float(s.query_scale)
        self.q_size = s.num_heads * s.head_dim
        self.v_size = s.num_heads * s.value_dim
        self.key_scale = 1.0 if s.key_scale is None else float(s.key_scale)

    @classmethod
    def _names(cls, spec, prefix):
        return {n: f"{prefix}.{getattr(spec, n + '_name')}"
                for n in ("q", "k", "v", "gate", "o", "out_norm", "decay_down", "decay_up", "decay_bias")}

    @classmethod
    def declare(cls, spec, prefix):
        h, qs, vs = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_heads * spec.value_dim
        n = cls._names(spec, prefix)
        out = [TensorDecl(n["q"], (qs, h), MATRIX), TensorDecl(n["k"], (qs, h), MATRIX),
               TensorDecl(n["v"], (vs, h), MATRIX), TensorDecl(n["gate"], (vs, h), MATRIX),
               TensorDecl(n["o"], (h, vs), MATRIX)]
        if spec.out_norm_weight:
            out.append(TensorDecl(n["out_norm"], (spec.value_dim if spec.out_norm_per_head else vs,), NORM))
        if spec.decay_gate_rank is not None:
            r = spec.decay_gate_rank            # (-1: the checkpoint's tensor decides)
            out += [TensorDecl(n["decay_down"], (r, h), MATRIX), TensorDecl(n["decay_up"], (qs, r), MATRIX),
                    TensorDecl(n["decay_bias"], (qs,), BIAS)]
        return out

    @classmethod
    def cache_request(cls, spec):
        return FixedStateRequest((spec.num_heads, spec.head_dim, spec.value_dim))

    def load(self, store):
        n = self._names(self.spec, self.prefix)
        s = self.spec
        names = [n["q"], n["k"], n["v"], n["gate"]] + ([n["decay_down"]] if self.gated else [])
        self.w_in = pad_rows(store.cat(names))
        self.w_o = store.get(n["o"])
        self.norm_w = store.get(n["out_norm"]) if s.out_norm_weight else None
        if self.norm_w is not None and s.out_norm_per_head:
            self.norm_w = self.norm_w.repeat(s.num_heads).contiguous()       # one weight vector, every head
        if self.gated:
            self.rank = store.get(n["decay_down"]).shape[0]
            self.w_a2 = store.get(n["decay_up"])
            self.a2_bias = store.get(n["decay_bias"]).to(torch.float32).contiguous()

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T = x.shape[0]
        proj = K.plain_unless(None, linear(x, self.w_in))              # [T, q | k | v | gate]
        o = torch.empty((T, self.v_size), dtype=torch.float32, device=x.device)
        gate_z = None
        if self.gated:
            low = proj[:, 2 * self.q_size + 2 * self.v_size:2 * self.q_size + 2 * self.v_size + self.rank]
            if self.rank < 64:
                # a bottleneck this narrow: the CUDA-core product (float32 sums in k order)
                gate_z = torch.empty((T, self.q_size), dtype=torch.float32, device=x.device)
                K.gemm_simt(low, self.w_a2, gate_z)
            else:
                gate_z = linear(low if low.data_ptr() % 16 == 0 else low.contiguous(), self.w_a2,
                                out_dtype=torch.float32)
        state = cache.state if cache.state.dim() == 2 else cache.state.view(cache.state.shape[0], -1)
        K.decay_attention(proj, ctx, state, self.decay, o, q_off=0, k_off=self.q_size,
                          v_off=2 * self.q_size, num_heads=s.num_heads, head_dim=s.head_dim,
                          value_dim=s.value_dim, activation=s.qkv_activation, freq=self.freq,
                          rot_dims=self.rot_dims, key_scale=self.key_scale, query_scale=self.query_scale,
                          gate_z=gate_z, gate_bias=self.a2_bias if self.gated else None,
                          gate_tau=s.decay_gate_tau)
        gate = proj[:, 2 * self.q_size + self.v_size:2 * self.q_size + 2 * self.v_size]
        out = torch.empty((T, self.v_size), dtype=x.dtype, device=x.device)
        groups, size = (s.num_heads, s.value_dim) if s.out_norm == "head" else (1, self.v_size)
        K.group_norm_gate(o, groups, size, out, eps=s.out_norm_eps, weight=self.norm_w, gate=gate,
                          gate_activation=s.gate_activation)
        if self.out_dtype is not None:
            return linear(out, self.w_o, out_dtype=self.out_dtype)
        return linear(out, self.w_o, consumer="norm")

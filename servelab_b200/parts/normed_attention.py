"""Grouped-query attention with normed and rotated queries and keys, keys and values of
different sizes, values mixed across layers and a gate per head (spec: ``NormedAttentionSpec``).

Per step, with h the mixer's input [T, hidden]:

  1. one product for q | k | v | gate (their matrices are concatenated at load);
  1b. with ``conv_taps``: a causal convolution over time on every q, k and v channel; the rows
     before a portion come from the request's state record, which is left holding the last
     taps - 1 projected rows;
  2. one kernel: RMS norm of every query and key head (one weight vector each, shared by the
     heads), rotation on the first ``dims`` elements (neighbouring pairs, or element i with
     element i + dims / 2), with ``qk_unit_norm`` every rotated head divided by its root mean
     square, q into its buffer, k into the request's pages; the values -- kept for later layers
     ("source") or replaced by (1 - lambda) v + lambda v_source ("mix") -- into the pages, so the
     cache holds what the attention uses;
  3. attention of every query over its request's visible keys, softmax in float32 (scores
     soft-capped, a sink a head in the denominator: each optional), head h's row times
     sigmoid(gate_h);
  4. the output projection (``out_dtype``: a mixer that norms the result asks for float32).

The values of the source layer travel to the mixing layers through the step's scratch
(``ctx.scratch``): they are needed for the step's own tokens only, because every layer caches its
mixed values.
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import FixedStateRequest, PagedKVRequest
from ..ops import attention as A
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.source import BIAS, MATRIX, NORM, POSITIVE, TensorDecl
from .base import Mixer
from .registry import POSITIONS, build_part, register_mixer


def pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """``w`` with zero rows appended up to a multiple (the library's products want one)."""
    extra = -w.shape[0] % multiple
    if not extra:
        return w
    return torch.cat([w, torch.zeros((extra, w.shape[1]), dtype=w.dtype, device=w.device)]).contiguous()


@register_mixer("normed_attention")
class NormedAttention(Mixer):
    graph_safe = True
    padded_steps_safe = True      # the convolution's record is written per request with tokens only

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.value_mix not in (None, "source", "mix"):
            raise ValueError(f"normed_attention: value_mix {spec.value_mix!r} (None, 'source', 'mix')")
        if spec.conv_taps < 0 or spec.conv_taps > K.CONV_MAX_TAPS:
            raise ValueError(f"normed_attention: 0..{K.CONV_MAX_TAPS} taps, got {spec.conv_taps}")
        if spec.softcap is not None and not spec.softcap > 0:
            raise ValueError("normed_attention: a soft cap must be positive")
        self.position = build_part(POSITIONS, spec.position, f"{prefix}.rot", env)
        self.out_dtype = None                  # (set by a mixer that wraps this one)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.q_size = spec.num_heads * spec.head_dim
        self.k_size = spec.num_kv_heads * spec.head_dim
        self.v_size = spec.num_kv_heads * spec.value_dim
        A.check_kv_supported(spec.head_dim, spec.value_dim)
        A.prepare_kv_attention(spec.head_dim, spec.value_dim, env.dtype)
        if (spec.head_dim == spec.value_dim and env.dtype == torch.bfloat16 and spec.head_dim in (64, 128)
                and spec.softcap is None and not spec.sink and torch.cuda.is_available()):
            from ..ops import library
            library.attention(spec.head_dim)      # the kernels for equal sizes, built now

    @classmethod
    def _names(cls, spec, prefix):
        return {n: f"{prefix}.{getattr(spec, n + '_name')}"
                for n in ("q", "k", "v", "o", "gate", "q_norm", "k_norm", "value_mix")}

    @classmethod
    def declare(cls, spec, prefix):
        h, H, G, D, Dv = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        n = cls._names(spec, prefix)
        out = [TensorDecl(n["q"], (H * D, h), MATRIX), TensorDecl(n["k"], (G * D, h), MATRIX),
               TensorDecl(n["v"], (G * Dv, h), MATRIX), TensorDecl(n["o"], (h, H * Dv), MATRIX)]
        if spec.qk_norm:
            out += [TensorDecl(n["q_norm"], (D,), NORM), TensorDecl(n["k_norm"], (D,), NORM)]
        if spec.value_mix == "mix":
            out.append(TensorDecl(n["value_mix"], (), POSITIVE))
        if spec.head_gate:
            out.append(TensorDecl(n["gate"], (H, h), MATRIX))
        if spec.conv_taps >= 1:
            out += [TensorDecl(n[x] + spec.conv_suffix, (rows, spec.conv_taps), BIAS)
                    for x, rows in (("q", H * D), ("k", G * D), ("v", G * Dv))]
        if spec.sink:
            out.append(TensorDecl(f"{prefix}.{spec.sink_name}", (H,), BIAS))
        return out

    @classmethod
    def cache_request(cls, spec):
        pages = PagedKVRequest(spec.num_kv_heads, spec.head_dim, spec.window, value_dim=spec.value_dim)
        if spec.conv_taps <= 1:
            return pages
        width = spec.num_heads * spec.head_dim + spec.num_kv_heads * (spec.head_dim + spec.value_dim)
        return (pages, FixedStateRequest((spec.conv_taps - 1, width)))

    def load(self, store):
        s = self.spec
        n = self._names(s, self.prefix)
        self.w_in = pad_rows(store.cat([n["q"], n["k"], n["v"]] + ([n["gate"]] if s.head_gate else [])))
        self.w_o = store.get(n["o"])
        self.q_norm = store.get(n["q_norm"]) if s.qk_norm else None
        self.k_norm = store.get(n["k_norm"]) if s.qk_norm else None
        self.lam = store.get(n["value_mix"]).reshape(1) if s.value_mix == "mix" else None
        self.taps = None
        if s.conv_taps >= 1:
            # [taps, channels]: a tap's weights of neighbouring channels are neighbours
            self.taps = store.cat([n[x] + s.conv_suffix for x in ("q", "k", "v")]).t().contiguous()
        self.sink = store.get(f"{self.prefix}.{s.sink_name}").to(torch.float32).contiguous() if s.sink else None

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T = x.shape[0]
        table = ctx.block_tables[cache.group]
        proj = K.plain_unless(None, linear(x, self.w_in))             # [T, q | k | v | gate]
        gate = proj[:, self.q_size + self.k_size + self.v_size:] if s.head_gate else None
        if self.taps is not None:
            if not owns_cache:
                raise NotImplementedError("normed_attention: a convolution in a run that reads another run's cache")
            conv = torch.empty((T, self.q_size + self.k_size + self.v_size), dtype=x.dtype, device=x.device)
            state = cache.state
            if state is not None and state.dim() > 2:
                state = state.view(state.shape[0], -1)
            K.short_conv(proj, self.taps, state, ctx, conv)
            proj = conv
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=x.device)
        key = "value_mix:" + s.value_mix_key
        v_keep = v_first = None
        if s.value_mix == "source":
            v_keep = ctx.scratch[key] = torch.empty((T, self.v_size), dtype=x.dtype, device=x.device)
        elif s.value_mix == "mix":
            v_first = ctx.scratch[key]
        pairs = getattr(self.position, "pair_table", None)
        freq, rot_dims, mag = pairs() if pairs is not None else (None, 0, 1.0)
        halves = pairs is None and self.position.rotary_table() is not None
        if halves:                                 # element i with element i + dims / 2
            freq, rot_dims = self.position.rotary_table()
        norm_dims = s.head_dim if s.qk_norm else 0
        unit_dims = s.head_dim if s.qk_unit_norm else 0
        K.head_prep(proj, ctx, table, cache.page_size,
                    q_off=0, num_heads=s.num_heads, q_dim=s.head_dim, q_norm_w=self.q_norm,
                    q_norm_dims=norm_dims, q_rot_off=0,
                    k_off=self.q_size, num_kv_heads=s.num_kv_heads, k_dim=s.head_dim, k_norm_w=self.k_norm,
                    k_norm_dims=norm_dims, k_rot_off=0,
                    v_off=self.q_size + self.k_size, v_dim=s.value_dim,
                    freq=freq, rot_dims=rot_dims, rot_mag=mag, eps=s.qk_norm_eps, q_out=q,
                    k_cache=cache.k if owns_cache else None, v_cache=cache.v if owns_cache else None,
                    lam=self.lam, v_first=v_first, v_keep=v_keep, rot_half=halves,
                    q_unit_dims=unit_dims, k_unit_dims=unit_dims)
        out = torch.empty((T, s.num_heads * s.value_dim), dtype=x.dtype, device=x.device)
        A.kv_attention(ctx, q, cache.k, cache.v, s.value_dim, out, table, s.num_heads, s.num_kv_heads,
                       s.head_dim, s.value_dim, cache.page_size, self.scale, s.window or 0, gate,
                       s.softcap, self.sink)
        if self.out_dtype is not None:
            return linear(out, self.w_o, out_dtype=self.out_dtype)
        return linear(out, self.w_o, consumer="norm")

"""Differential attention (spec: ``DifferentialAttentionSpec``): two softmax attention maps a
head over one set of values, combined as a_1 - lambda a_2, normed per head and scaled.

Per step, with h the mixer's input [T, hidden]:

  1. one product with bias for q | k | v (q alone in a layer that reads another layer's cache);
  2. one kernel that copies the queries out and writes the keys -- a kv head's two maps side by side
     as one cached row of 2 x head_dim elements -- and the values into the request's pages;
  3. attention of every (query head, map) over its request's keys of that map, causal, softmax in
     float32, results float32 per map;
  4. one kernel: o = a_1 - lambda a_2, divided by its root mean square over the head, times
     1 - lambda_init; lambda is one number a layer, formed from four learned vectors at load;
  5. the output projection.
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import PagedKVRequest
from ..ops import attention as A
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.source import BIAS, MATRIX, TensorDecl
from .base import Mixer
from .normed_attention import pad_rows
from .registry import register_mixer


@register_mixer("differential_attention")
class DifferentialAttention(Mixer):
    graph_safe = True
    MAPS = 2

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        s = spec
        if min(s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim) <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError("differential_attention: heads must be a positive multiple of kv heads")
        self.scale = s.scale if s.scale is not None else 1.0 / math.sqrt(s.head_dim)
        self.q_size = s.num_heads * self.MAPS * s.head_dim
        self.k_size = s.num_kv_heads * self.MAPS * s.head_dim
        self.v_size = s.num_kv_heads * s.value_dim
        A.check_kv_supported(s.head_dim, s.value_dim)
        A.prepare_maps_attention(s.head_dim, s.value_dim, env.dtype, maps=2, group=s.num_heads // s.num_kv_heads)

    @classmethod
    def _names(cls, spec, prefix):
        return {n: f"{prefix}.{getattr(spec, n + '_name')}" for n in ("q", "k", "v", "o")}

    @classmethod
    def declare(cls, spec, prefix):
        h, H, G, D, Dv = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        n = cls._names(spec, prefix)
        sizes = [("q", H * cls.MAPS * D)] + ([("k", G * cls.MAPS * D), ("v", G * Dv)] if spec.own_kv else [])
        out = [TensorDecl(n[key], (rows, h), MATRIX) for key, rows in sizes]
        if spec.qkv_bias:
            out += [TensorDecl(n[key] + spec.bias_suffix, (rows,), BIAS) for key, rows in sizes]
        out.append(TensorDecl(n["o"], (h, H * Dv), MATRIX))
        out += [TensorDecl(f"{prefix}.{name}", (D,), BIAS) for name in spec.lambda_names]
        return out

    @classmethod
    def cache_request(cls, spec):
        # a kv head's maps side by side are one cached key row
        return PagedKVRequest(spec.num_kv_heads, cls.MAPS * spec.head_dim, spec.window, value_dim=spec.value_dim)

    def load(self, store):
        s = self.spec
        n = self._names(s, self.prefix)
        keys = ["q", "k", "v"] if s.own_kv else ["q"]
        self.w_in = pad_rows(store.cat([n[k] for k in keys]))
        self.b_in = None
        if s.qkv_bias:
            b = torch.cat([store.get(n[k] + s.bias_suffix) for k in keys])
            extra = self.w_in.shape[0] - b.shape[0]
            self.b_in = torch.cat([b, b.new_zeros(extra)]).contiguous() if extra else b.contiguous()
        self.w_o = store.get(n["o"])
        lq1, lk1, lq2, lk2 = (store.get(f"{self.prefix}.{name}").double() for name in s.lambda_names)
        lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + s.lambda_init
        self.lam = torch.tensor([lam], dtype=torch.float32, device=self.w_o.device)

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T = x.shape[0]
        if owns_cache != s.own_kv:
            raise ValueError("differential_attention: a layer with key and value projections owns its "
                             "cache, one without reads another layer's")
        table = ctx.block_tables[cache.group]
        proj = K.plain_unless(None, linear(x, self.w_in, self.b_in))       # [T, q | k | v]
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=x.device)
        K.head_prep(proj, ctx, table, cache.page_size,
                    q_off=0, num_heads=s.num_heads * self.MAPS, q_dim=s.head_dim, q_norm_w=None,
                    q_norm_dims=0, q_rot_off=0,
                    k_off=self.q_size, num_kv_heads=s.num_kv_heads if owns_cache else 0,
                    k_dim=self.MAPS * s.head_dim, k_norm_w=None, k_norm_dims=0, k_rot_off=0,
                    v_off=self.q_size + self.k_size if owns_cache else -1, v_dim=s.value_dim,
                    freq=None, rot_dims=0, rot_mag=1.0, eps=0.0, q_out=q,
                    k_cache=cache.k if owns_cache else None, v_cache=cache.v if owns_cache else None)
        per_map = torch.empty((T, s.num_heads * self.MAPS * s.value_dim), dtype=torch.float32, device=x.device)
        A.maps_attention(ctx, q, cache.k, cache.v, per_map, table, s.num_heads, s.num_kv_heads, self.MAPS,
                         s.head_dim, s.value_dim, cache.page_size, self.scale, s.window or 0)
        out = torch.empty((T, s.num_heads * s.value_dim), dtype=x.dtype, device=x.device)
        K.group_norm_gate(per_map, s.num_heads, s.value_dim, out, eps=s.norm_eps,
                          factor=1.0 - s.lambda_init, maps=self.MAPS, lam=self.lam)
        return linear(out, self.w_o, consumer="norm")

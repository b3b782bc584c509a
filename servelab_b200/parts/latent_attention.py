"""Latent attention (spec: ``LatentAttentionSpec``): the cache holds, per token, one normed latent
vector c of ``kv_rank`` elements and one rotated key part of ``rope_dim`` elements; head h's
unrotated key is W_uk[h] c and its value W_uv[h] c.

Neither is ever expanded.  Because q.(W_uk[h] c) = (W_uk[h]^T q).c, the unrotated part of a query
is multiplied by its head's W_uk once, and the attention runs over the cached rows themselves:

  1. one product for q | dkv | gate (with ``q_rank``: dq | dkv | gate, then the RMS norm of the
     queries' latent and the product with W_uq);
  2. one kernel: RMS norm of the latent part of dkv, rotation of its last ``rope_dim`` elements
     (neighbouring pairs), the row [c | rotated part] into the request's page; rotation of the last
     ``rope_dim`` elements of every query head, written behind where the absorbed part will go;
  3. per head: q'[h] = W_uk[h]^T q_unrotated[h]   (``kv_rank`` elements);
  4. attention with ONE kv head for all query heads, keys = cached rows (kv_rank + rope_dim
     elements), values = the first kv_rank elements of the same rows, float32 softmax, window;
  5. per head: o[h] = W_uv[h] o'[h], times sigmoid(gate), and the output projection.  A gate of
     one number a head (``head_gate``) and a sink a head in the softmax's denominator (``sink``)
     act inside the attention kernel of step 4: a number a head commutes with W_uv[h].

The scores and results equal those of the expanded form exactly (up to rounding), for prompts and
single tokens alike, so no per-head key or value is cached or recomputed for earlier tokens.
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import PagedKVRequest
from ..ops import attention as A
from ..ops import kernels as K
from ..ops.linear import batched_head_linear, linear
from ..weights.source import BIAS, MATRIX, NORM, TensorDecl
from .base import Mixer
from .normed_attention import pad_rows
from .registry import POSITIONS, build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.element_gate and spec.head_gate:
            raise ValueError("latent_attention: a gate per element or a gate per head, not both")
        self.position = build_part(POSITIONS, spec.position, f"{prefix}.rot", env)
        self.q_head = spec.head_dim + spec.rope_dim
        self.row = spec.kv_rank + spec.rope_dim                    # a cached row; a query row after step 3
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.q_head)
        A.check_kv_supported(self.row, spec.kv_rank)
        A.prepare_kv_attention(self.row, spec.kv_rank, env.dtype)

    @classmethod
    def _names(cls, spec, prefix):
        return {n: f"{prefix}.{getattr(spec, n + '_name')}"
                for n in ("q", "down", "latent_norm", "up_k", "up_v", "o", "gate", "q_down", "q_norm", "q_up",
                          "sink")}

    @classmethod
    def declare(cls, spec, prefix):
        h, H, D, Dr, Dv, R = (spec.hidden_size, spec.num_heads, spec.head_dim, spec.rope_dim,
                              spec.value_dim, spec.kv_rank)
        n = cls._names(spec, prefix)
        if spec.q_rank is None:
            out = [TensorDecl(n["q"], (H * (D + Dr), h), MATRIX)]
        else:
            out = [TensorDecl(n["q_down"], (spec.q_rank, h), MATRIX), TensorDecl(n["q_norm"], (spec.q_rank,), NORM),
                   TensorDecl(n["q_up"], (H * (D + Dr), spec.q_rank), MATRIX)]
        out += [TensorDecl(n["down"], (R + Dr, h), MATRIX),
               TensorDecl(n["latent_norm"], (R,), NORM), TensorDecl(n["up_k"], (H * D, R), MATRIX),
               TensorDecl(n["up_v"], (H * Dv, R), MATRIX), TensorDecl(n["o"], (h, H * Dv), MATRIX)]
        if spec.element_gate:
            out.append(TensorDecl(n["gate"], (H * Dv, h), MATRIX))
        if spec.head_gate:
            out.append(TensorDecl(n["gate"], (H, h), MATRIX))
        if spec.sink:
            out.append(TensorDecl(n["sink"], (H,), BIAS))
        return out

    @classmethod
    def cache_request(cls, spec):
        return PagedKVRequest(1, spec.kv_rank + spec.rope_dim, spec.window, tied_values=True)

    def load(self, store):
        s = self.spec
        n = self._names(s, self.prefix)
        gated = s.element_gate or s.head_gate
        first = n["q"] if s.q_rank is None else n["q_down"]
        self.first_rows = store.get(first).shape[0]      # H (D + Dr) query columns, or the queries' latent
        self.w_in = pad_rows(store.cat([first, n["down"]] + ([n["gate"]] if gated else [])))
        self.q_norm = store.get(n["q_norm"]) if s.q_rank is not None else None
        self.w_uq = pad_rows(store.get(n["q_up"])) if s.q_rank is not None else None
        self.sink = store.get(n["sink"]).to(torch.float32).contiguous() if s.sink else None
        self.latent_norm = store.get(n["latent_norm"])
        # [H, kv_rank, head_dim]: q' = q_unrotated . this^T per head
        self.w_uk_t = store.get(n["up_k"]).view(s.num_heads, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = store.get(n["up_v"]).view(s.num_heads, s.value_dim, s.kv_rank).contiguous()
        self.w_o = store.get(n["o"])

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T, H, D, Dr, R = x.shape[0], s.num_heads, s.head_dim, s.rope_dim, s.kv_rank
        table = ctx.block_tables[cache.group]
        proj = K.plain_unless(None, linear(x, self.w_in))             # [T, q (or its latent) | dkv | gate]
        q_size = H * self.q_head
        first = self.first_rows
        q_abs = torch.empty((T, H * self.row), dtype=x.dtype, device=x.device)
        pairs = getattr(self.position, "pair_table", None)
        freq, rot_dims, mag = pairs() if pairs is not None else (None, 0, 1.0)
        kw = dict(num_kv_heads=1, k_dim=self.row, k_norm_w=self.latent_norm, k_norm_dims=R, k_rot_off=R,
                  v_off=-1, v_dim=0, freq=freq, rot_dims=rot_dims, rot_mag=mag, eps=s.latent_norm_eps,
                  k_cache=cache.k if owns_cache else None, v_cache=None)
        qkw = dict(q_off=0, num_heads=H, q_dim=self.q_head, q_norm_w=None, q_norm_dims=0, q_rot_off=D,
                   q_out=q_abs[:, R:], q_head_stride=self.row, q_skip=D)
        if s.q_rank is None:
            queries = proj
            K.head_prep(proj, ctx, table, cache.page_size, k_off=first, **qkw, **kw)
        else:
            # the queries' latent: norm, then the product with W_uq; the keys' row and the queries are
            # then prepared from two tensors (two launches of the head kernel)
            cq = torch.empty((T, s.q_rank), dtype=x.dtype, device=x.device)
            K.rms_norm_rows(proj[:, :first], self.q_norm, s.latent_norm_eps, cq)
            queries = K.plain_unless(None, linear(cq, self.w_uq))
            K.head_prep(queries, ctx, table, cache.page_size, k_off=0, num_kv_heads=0, k_dim=0, k_norm_w=None,
                        k_norm_dims=0, k_rot_off=0, v_off=-1, v_dim=0, freq=freq, rot_dims=rot_dims, rot_mag=mag,
                        eps=s.latent_norm_eps, k_cache=None, v_cache=None, **qkw)
            K.head_prep(proj, ctx, table, cache.page_size, q_off=0, num_heads=0, q_dim=0, q_norm_w=None,
                        q_norm_dims=0, q_rot_off=0, q_out=q_abs, k_off=first, **kw)
        # q'[:, h, :R] = q[:, h, :D] . W_uk[h]
        batched_head_linear(queries[:, :q_size].view(T, H, self.q_head)[:, :, :D], self.w_uk_t,
                            q_abs.view(T, H, self.row)[:, :, :R])
        o_lat = torch.empty((T, H * R), dtype=x.dtype, device=x.device)
        gate_cols = proj[:, first + self.row:]
        A.kv_attention(ctx, q_abs, cache.k, cache.k, self.row, o_lat, table, H, 1, self.row, R,
                       cache.page_size, self.scale, s.window or 0, gate_cols if s.head_gate else None,
                       None, self.sink)
        out = torch.empty((T, H * s.value_dim), dtype=x.dtype, device=x.device)
        batched_head_linear(o_lat.view(T, H, R), self.w_uv, out.view(T, H, s.value_dim))
        if s.element_gate:
            K.sigmoid_gate(out, gate_cols[:, :H * s.value_dim], out)
        return linear(out, self.w_o, consumer="norm")

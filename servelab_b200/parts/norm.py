"""Norms fused with the residual add that precedes them: RMSNorm and Dynamic Tanh.

y = x * rsqrt(mean(x^2) + eps) * w in float32 (tests/test_triton_kernels.py:57-59,
servelab/attention/triton/paged_attention.py:76-91 in the reference); the weight
is held in float32.
"""

from __future__ import annotations

import torch

from ..ops import kernels as K
from ..weights.source import BIAS, NORM, POSITIVE, TensorDecl
from .base import Norm
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    accepts_split_sum = True      # ``delta`` may be a SplitSum (parts of a K-split product)
    accepts_deferred_linear = True    # ... or a product not launched yet, which then runs with the
                                      # add and this norm in its epilogue; the result is ScaledRows

    accepts_hyper_pending = True      # ... or the update of a residual kept as several streams

    @classmethod
    def declare(cls, spec, prefix):
        # (a weight stored around zero is drawn around zero in random models: the role of a bias)
        return [TensorDecl(prefix + spec.weight_suffix, (spec.dim,), BIAS if spec.unit_offset else NORM)]

    def load(self, store):
        self.weight = store.get(self.prefix + self.spec.weight_suffix)
        if self.spec.unit_offset:             # the stored weight lies around zero: the factor is 1 + w
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()

    def read_streams(self, ctx, streams, pending, read_weights, out_rows=None):
        """For a residual kept as streams [T, n, dim]: folds the pending update in (``HyperPending``
        or None), then norms sum_s read_weights[s] x_s (None: the plain sum) -- one launch.  With
        ``out_rows`` only those rows are produced and the streams are left as they are."""
        rows = streams.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((rows, self.spec.dim), dtype=self.env.dtype, device=streams.device)
        update = mix = out_w = None
        if pending is not None:
            update, mix, out_w = K.plain_unless(None, pending.value), pending.mix, pending.out_weights
        K.hyper_mix_norm(streams, update, mix, out_w, read_weights, self.weight, self.spec.eps, out, out_rows)
        return out

    def forward(self, ctx, resid, delta, out_rows=None):
        if resid.dim() == 3:              # several streams: their sum is what a model's last norm reads
            return self.read_streams(ctx, resid, delta, None, out_rows)
        if isinstance(delta, K.DeferredLinear):
            if out_rows is None and self.env.dtype == torch.bfloat16:
                return K.gemm_tc_resid_norm(delta.x, delta.w, delta.bias, resid, self.weight,
                                            self.spec.eps)
            delta = delta.materialize()
        rows = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((rows, self.spec.dim), dtype=self.env.dtype, device=resid.device)
        K.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out, out_rows)
        return out


class HyperPending:
    """A sublayer's result that has not been folded into a residual kept as several streams yet:
    x_t <- sum_s mix[s, t] x_s + out_weights[t] value.  The kernel that prepares the next reader's
    input does it on the way (``RMSNorm.read_streams``)."""

    accept_flag = "accepts_hyper_pending"

    def __init__(self, value, mix: torch.Tensor, out_weights: torch.Tensor):
        self.value, self.mix, self.out_weights = value, mix, out_weights

    def materialize(self):
        raise TypeError("an update of several residual streams can only be handed to a part that folds "
                        "it in (a norm with read_streams)")


fuse_product_norms = True     # Dynamic Tanh: a deferred product runs with the norms in its epilogue


class PostNormed:
    """A sublayer's result that still lacks the norm it must pass before it is added to the
    stream (the "b" norm of a sandwich block): the next norm kernel applies that norm, the add
    and itself in one pass if it is of a kind that can (``accepts_post_normed``); otherwise
    ``materialize()`` runs the norm on the result alone."""

    accept_flag = "accepts_post_normed"

    def __init__(self, ctx, value: torch.Tensor, norm: "Norm"):
        self.ctx, self.value, self.norm = ctx, value, norm

    @property
    def shape(self):
        return self.value.shape

    def materialize(self) -> torch.Tensor:
        return self.norm.apply(self.ctx, K.plain_unless(None, self.value))


@register_norm("dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha x) w + b, float32 arithmetic, nothing reduced over the row.  Being
    elementwise it also takes a ``PostNormed`` update whose pending norm is a Dynamic Tanh:
    one kernel then norms the update, adds it and norms the sum."""
    graph_safe = True
    accepts_post_normed = True
    accepts_deferred_linear = True    # as the pending norm of a PostNormed value: the value may be a
                                      # product not launched yet, which then runs with both norms
                                      # and the add in its epilogue

    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + spec.weight_suffix, (spec.dim,), NORM),
                TensorDecl(prefix + spec.bias_suffix, (spec.dim,), BIAS),
                TensorDecl(prefix + spec.alpha_suffix, (), POSITIVE)]

    def load(self, store):
        s = self.spec
        self.weight = store.get(self.prefix + s.weight_suffix)
        self.bias = store.get(self.prefix + s.bias_suffix)
        self.alpha = store.get(self.prefix + s.alpha_suffix).reshape(1)
        self.params = (self.alpha, self.weight, self.bias)

    def forward(self, ctx, resid, delta, out_rows=None):
        post = None
        if isinstance(delta, PostNormed):
            if isinstance(delta.norm, DynamicTanh):
                post, delta = delta.norm.params, delta.value
                if isinstance(delta, K.DeferredLinear):
                    if (out_rows is None and self.env.dtype == torch.bfloat16 and delta.bias is None
                            and fuse_product_norms):
                        return K.gemm_tc_resid_dyt(delta.x, delta.w, resid, post, self.params)
                    delta = delta.materialize()
            else:
                delta = delta.materialize()
        elif isinstance(delta, K.DeferredLinear):
            delta = delta.materialize()
        rows = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((rows, self.spec.dim), dtype=self.env.dtype, device=resid.device)
        K.dyt_add_norm(resid, delta, post, self.params, out, out_rows)
        return out

    def apply(self, ctx, x):
        """The norm of ``x`` [T, dim] alone (no stream, no add), in the compute dtype."""
        stream = x.to(torch.float32)
        out = torch.empty((x.shape[0], self.spec.dim), dtype=self.env.dtype, device=x.device)
        K.dyt_add_norm(stream, None, None, self.params, out, None)
        return out

    def add_into(self, ctx, resid, delta) -> None:
        """resid += this norm of ``delta`` (the close of a branch that nothing norms after)."""
        K.dyt_add_norm(resid, delta, self.params, None, None, None)


@register_norm("layernorm")
class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w + b in float32.  As the pending norm of a ``PostNormed``
    update it runs inside the kernel that adds the update to the stream (``close``), which also
    hands the stream to the next reader in the compute dtype."""
    graph_safe = True
    accepts_post_normed = True

    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + spec.weight_suffix, (spec.dim,), NORM),
                TensorDecl(prefix + spec.bias_suffix, (spec.dim,), BIAS)]

    def load(self, store):
        self.weight = store.get(self.prefix + self.spec.weight_suffix)
        self.bias = store.get(self.prefix + self.spec.bias_suffix)
        self.params = (self.weight, self.bias, self.spec.eps)

    @staticmethod
    def _pending(delta):
        """(update tensor or None, its pending layer norm's parameters or None)."""
        if isinstance(delta, PostNormed):
            if isinstance(delta.norm, LayerNorm):
                return K.plain_unless(None, delta.value), delta.norm.params
            return delta.materialize(), None
        return (None if delta is None else K.plain_unless(None, delta)), None

    def forward(self, ctx, resid, delta, out_rows=None):
        """The norm of the stream's rows (after the update) -- the use as a model's final norm."""
        delta, post = self._pending(delta)
        if delta is not None and post is None:
            if out_rows is not None:                  # a plain update and selected rows: add first
                resid = resid + delta.to(torch.float32)
            else:
                resid += delta.to(torch.float32)
            delta = None
        rows = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((rows, self.spec.dim), dtype=self.env.dtype, device=resid.device)
        K.ln_add_norm(resid, delta, post, self.params, out, out_rows)
        return out

    def apply(self, ctx, x):
        stream = x.to(torch.float32)
        out = torch.empty((x.shape[0], self.spec.dim), dtype=self.env.dtype, device=x.device)
        K.ln_add_norm(stream, None, None, self.params, out, None)
        return out

    @classmethod
    def close(cls, ctx, resid, delta, dtype):
        """Adds a pending update into the float32 stream (its layer norm applied on the way) and
        returns the stream for the next reader: the stream itself in float32, else a copy in
        ``dtype``.  One launch."""
        delta, post = cls._pending(delta)
        if delta is not None and post is None:
            resid += delta.to(torch.float32)
            delta = None
        if dtype == torch.float32:
            if delta is not None:
                K.ln_add_norm(resid, delta, post, None, None, None)
            return resid
        out = torch.empty(resid.shape, dtype=dtype, device=resid.device)
        K.ln_add_norm(resid, delta, post, None, out, None)
        return out

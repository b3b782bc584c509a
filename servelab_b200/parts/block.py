"""Arrangement of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += ff(norm2(x)) -- the order of the
reference's layer body (servelab/parallel/tp_model.py:125-133); ``feed_forward``
None: the layer ends after the mixer.  The stream x is
float32; an update that has not been added yet travels beside it so that the add
happens inside the next norm kernel.
"""

from __future__ import annotations

from ..ops.kernels import plain_unless
from .base import Block
from ..weights.source import BIAS, MIXING, TensorDecl
from .norm import HyperPending, PostNormed
from .registry import FEED_FORWARDS, MIXERS, NORMS, build_part, part_class, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self._build(spec, prefix, env)
        # a step of this block may be captured in a CUDA graph iff every part only
        # launches kernels whose arguments are device buffers of the step context
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self._present())

    @staticmethod
    def _members(spec, prefix):
        """(registry, spec, prefix) of the four parts; the names under the layer's prefix are
        the spec's, so the block knows no checkpoint's naming."""
        out = ((NORMS, spec.mixer_norm, f"{prefix}.{spec.mixer_norm_name}"),
               (MIXERS, spec.mixer, f"{prefix}.{spec.mixer_name}"))
        if spec.feed_forward is None:                 # the layer ends after the mixer
            return out
        return out + ((NORMS, spec.ff_norm, f"{prefix}.{spec.ff_norm_name}"),
                      (FEED_FORWARDS, spec.feed_forward, f"{prefix}.{spec.feed_forward_name}"))

    def _build(self, spec, prefix, env):
        parts = [build_part(table, part, name, env) for table, part, name in self._members(spec, prefix)]
        self.mixer_norm, self.mixer = parts[:2]
        self.ff_norm, self.feed_forward = parts[2:] if len(parts) > 2 else (None, None)

    def _present(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    @classmethod
    def declare(cls, spec, prefix):
        out = []
        for table, part, name in cls._members(spec, prefix):
            out += part_class(table, part).declare(part, name)
        return out

    @classmethod
    def cache_request(cls, spec):
        return part_class(MIXERS, spec.mixer).cache_request(spec.mixer)

    def load(self, store):
        for p in self._present():
            p.load(store)

    accepts_split_sum = True          # the incoming ``delta`` may be a SplitSum
    accepts_deferred_linear = True    # ... or a DeferredLinear

    def forward(self, ctx, resid, delta, cache, owns_cache):
        # An update may arrive in an unfinished form (the partial sums of a K-split product, a
        # product not launched yet), and a norm may return its rows in one (ScaledRows): a part
        # that does not say that it takes the form gets the plain tensor.
        x = self.mixer_norm.forward(ctx, resid, plain_unless(self.mixer_norm, delta))
        a = self.mixer.forward(ctx, plain_unless(self.mixer, x), cache, owns_cache)
        if self.feed_forward is None:
            return resid, a
        x = self.ff_norm.forward(ctx, resid, plain_unless(self.ff_norm, a))
        return resid, self.feed_forward.forward(ctx, plain_unless(self.feed_forward, x))


@register_block("sandwich_norm")
class SandwichNormBlock(PreNormBlock):
    """x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))): each sublayer's result passes
    a norm of its own before it is added.  The result travels to the next norm kernel as a
    ``PostNormed`` value, so norm-of-result, add and norm-of-next-input are one launch where
    the norms' kind allows.  ``feed_forward`` None: the layer ends after the mixer."""

    @staticmethod
    def _members(spec, prefix):
        out = [(NORMS, spec.mixer_norm, f"{prefix}.{spec.mixer_norm_name}"),
               (MIXERS, spec.mixer, f"{prefix}.{spec.mixer_name}"),
               (NORMS, spec.mixer_post_norm, f"{prefix}.{spec.mixer_post_norm_name}")]
        if spec.feed_forward is not None:
            out += [(NORMS, spec.ff_norm, f"{prefix}.{spec.ff_norm_name}"),
                    (FEED_FORWARDS, spec.feed_forward, f"{prefix}.{spec.feed_forward_name}"),
                    (NORMS, spec.ff_post_norm, f"{prefix}.{spec.ff_post_norm_name}")]
        return tuple(out)

    def _build(self, spec, prefix, env):
        parts = [build_part(table, part, name, env) for table, part, name in self._members(spec, prefix)]
        self.mixer_norm, self.mixer, self.mixer_post_norm = parts[:3]
        self.ff_norm, self.feed_forward, self.ff_post_norm = (parts[3:] if len(parts) > 3
                                                              else (None, None, None))
        self._parts = parts

    def __init__(self, spec, prefix, env):
        Block.__init__(self, spec, prefix, env)
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and
                                            (spec.ff_norm is None or spec.ff_post_norm is None)):
            raise ValueError("sandwich_norm: every sublayer needs a norm before and after it")
        self._build(spec, prefix, env)
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self._parts)

    def load(self, store):
        for p in self._parts:
            p.load(store)

    accepts_split_sum = False
    accepts_deferred_linear = False
    accepts_post_normed = True        # the incoming ``delta`` may be a PostNormed value

    def forward(self, ctx, resid, delta, cache, owns_cache):
        x = self.mixer_norm.forward(ctx, resid, plain_unless(self.mixer_norm, delta))
        # (a sublayer's result may be a product not launched yet, if its pending norm takes that)
        a = plain_unless(self.mixer_post_norm, self.mixer.forward(ctx, plain_unless(self.mixer, x), cache, owns_cache))
        a = PostNormed(ctx, a, self.mixer_post_norm)
        if self.feed_forward is None:
            return resid, a
        x = self.ff_norm.forward(ctx, resid, plain_unless(self.ff_norm, a))
        f = plain_unless(self.ff_post_norm, self.feed_forward.forward(ctx, plain_unless(self.feed_forward, x)))
        return resid, PostNormed(ctx, f, self.ff_post_norm)


@register_block("result_norm")
class ResultNormBlock(Block):
    """x += norm1(mixer(x)); x += norm2(ff(x)): the sublayers read the stream itself and only
    their results are normed.  A result travels as a ``PostNormed`` value to the kernel that adds
    it, which also produces the next reader's copy of the stream (``LayerNorm.close``).
    ``feed_forward`` None: the layer ends after the mixer."""
    accepts_post_normed = True

    @staticmethod
    def _members(spec, prefix):
        out = [(MIXERS, spec.mixer, f"{prefix}.{spec.mixer_name}"),
               (NORMS, spec.mixer_post_norm, f"{prefix}.{spec.mixer_post_norm_name}")]
        if spec.feed_forward is not None:
            out += [(FEED_FORWARDS, spec.feed_forward, f"{prefix}.{spec.feed_forward_name}"),
                    (NORMS, spec.ff_post_norm, f"{prefix}.{spec.ff_post_norm_name}")]
        return tuple(out)

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and spec.ff_post_norm is None):
            raise ValueError("result_norm: every sublayer needs a norm on its result")
        self._parts = [build_part(t, part, name, env) for t, part, name in self._members(spec, prefix)]
        self.mixer, self.mixer_post_norm = self._parts[:2]
        self.feed_forward, self.ff_post_norm = self._parts[2:] if len(self._parts) > 2 else (None, None)
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self._parts)

    @classmethod
    def declare(cls, spec, prefix):
        out = []
        for table, part, name in cls._members(spec, prefix):
            out += part_class(table, part).declare(part, name)
        return out

    @classmethod
    def cache_request(cls, spec):
        return part_class(MIXERS, spec.mixer).cache_request(spec.mixer)

    def load(self, store):
        for p in self._parts:
            p.load(store)

    def forward(self, ctx, resid, delta, cache, owns_cache):
        from .norm import LayerNorm
        h = LayerNorm.close(ctx, resid, delta, self.env.dtype)
        a = K_plain(self.mixer.forward(ctx, h, cache, owns_cache))
        a = PostNormed(ctx, a, self.mixer_post_norm)
        if self.feed_forward is None:
            return resid, a
        h = LayerNorm.close(ctx, resid, a, self.env.dtype)
        f = K_plain(self.feed_forward.forward(ctx, h))
        return resid, PostNormed(ctx, f, self.ff_post_norm)


@register_block("hyper_connections")
class HyperConnectionsBlock(Block):
    """The residual is ``streams`` parallel copies X [T, n, w].  Sublayer f with norm N and the
    learned vectors in, out [n] and matrix mix [n, n] (indexed [from, to]):

        u = sum_s in[s] X_s;   y = f(N(u));   X_t <- sum_s mix[s, t] X_s + out[t] y   (all t at once)

    A sublayer's y travels as a ``HyperPending`` value to the kernel that prepares the next
    reader's input, which folds it in on the way.  ``feed_forward`` None: the layer ends after the
    mixer."""
    accepts_hyper_pending = True

    @staticmethod
    def _members(spec, prefix):
        out = [(NORMS, spec.mixer_norm, f"{prefix}.{spec.mixer_norm_name}"),
               (MIXERS, spec.mixer, f"{prefix}.{spec.mixer_name}")]
        if spec.feed_forward is not None:
            out += [(NORMS, spec.ff_norm, f"{prefix}.{spec.ff_norm_name}"),
                    (FEED_FORWARDS, spec.feed_forward, f"{prefix}.{spec.feed_forward_name}")]
        return tuple(out)

    @staticmethod
    def _hyper_names(spec, prefix):
        names = [spec.mixer_hyper_name] + ([spec.ff_hyper_name] if spec.feed_forward is not None else [])
        return [f"{prefix}.{n}" for n in names]

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.streams < 1:
            raise ValueError("hyper_connections: at least one stream")
        if spec.mixer_norm is None or (spec.feed_forward is not None and spec.ff_norm is None):
            raise ValueError("hyper_connections: every sublayer needs a norm before it")
        self._parts = [build_part(t, part, name, env) for t, part, name in self._members(spec, prefix)]
        for norm in self._parts[0::2]:
            if not hasattr(norm, "read_streams"):
                raise ValueError(f"hyper_connections: the norm {norm.spec.kind!r} cannot read several streams")
        self.mixer_norm, self.mixer = self._parts[:2]
        self.ff_norm, self.feed_forward = self._parts[2:] if len(self._parts) > 2 else (None, None)
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self._parts)

    @classmethod
    def declare(cls, spec, prefix):
        out = []
        for table, part, name in cls._members(spec, prefix):
            out += part_class(table, part).declare(part, name)
        n = spec.streams
        for h in cls._hyper_names(spec, prefix):
            out += [TensorDecl(h + ".in", (n,), BIAS), TensorDecl(h + ".out", (n,), BIAS),
                    TensorDecl(h + ".mix", (n, n), MIXING)]
        return out

    @classmethod
    def cache_request(cls, spec):
        return part_class(MIXERS, spec.mixer).cache_request(spec.mixer)

    def load(self, store):
        for p in self._parts:
            p.load(store)
        self.hyper = [(store.get(h + ".in"), store.get(h + ".mix").contiguous(), store.get(h + ".out"))
                      for h in self._hyper_names(self.spec, self.prefix)]

    def forward(self, ctx, streams, pending, cache, owns_cache):
        if streams.dim() != 3 or streams.shape[1] != self.spec.streams:
            raise ValueError("hyper_connections: the residual must be [tokens, streams, hidden]")
        read, mix, out_w = self.hyper[0]
        x = self.mixer_norm.read_streams(ctx, streams, pending, read)
        pending = HyperPending(self.mixer.forward(ctx, x, cache, owns_cache), mix, out_w)
        if self.feed_forward is None:
            return streams, pending
        read, mix, out_w = self.hyper[1]
        x = self.ff_norm.read_streams(ctx, streams, pending, read)
        return streams, HyperPending(self.feed_forward.forward(ctx, x), mix, out_w)


def K_plain(value):
    """A part's result as a plain tensor (unfinished forms are finished)."""
    return plain_unless(None, value)

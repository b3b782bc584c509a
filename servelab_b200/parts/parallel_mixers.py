"""Two mixers side by side on the same input (spec: ``ParallelMixersSpec``):

    y = factor (RMSnorm(left(h)) w_left + RMSnorm(right(h)) w_right)

Both branches are mixers of the registry, built from their own specs under
``<prefix>.<left_name>`` and ``<prefix>.<right_name>``; each returns its projected result in
float32 and one kernel norms both over the model width and adds them.

What the branches ask of the cache is merged into one request of this mixer: pages from the one
branch that wants pages (two paged branches would need two block tables a layer, which is not
built), and ONE per-request state record that holds the branches' records side by side.  Each
branch sees its own slice of the record through a ``LayerCache`` of its own (the rows of a slice
are the whole record's length apart, which the kernels that index state take as a stride).
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import FixedStateRequest, paged_part, state_part
from ..ops import kernels as K
from ..weights.source import NORM, TensorDecl
from .base import LayerCache, Mixer
from .registry import MIXERS, build_part, part_class, register_mixer


def _record_sizes(spec):
    """Floats of each branch's state record, rounded up to 4 (16-byte aligned slices)."""
    sizes = []
    for branch in (spec.left, spec.right):
        st = state_part(part_class(MIXERS, branch).cache_request(branch))
        sizes.append(0 if st is None else -(-math.prod(st.shape) // 4) * 4)
    return sizes


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.left = build_part(MIXERS, spec.left, f"{prefix}.{spec.left_name}", env)
        self.right = build_part(MIXERS, spec.right, f"{prefix}.{spec.right_name}", env)
        for branch in (self.left, self.right):
            if not hasattr(branch, "out_dtype"):
                raise ValueError(f"parallel_mixers: the mixer {branch.spec.kind!r} cannot return float32 results")
            branch.out_dtype = torch.float32
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in (self.left, self.right))
        self.padded_steps_safe = all(getattr(b, "padded_steps_safe", False) for b in (self.left, self.right))
        self.sizes = _record_sizes(spec)

    @classmethod
    def _norm_names(cls, spec, prefix):
        return (f"{prefix}.{spec.left_name}{spec.out_suffix}", f"{prefix}.{spec.right_name}{spec.out_suffix}")

    @classmethod
    def declare(cls, spec, prefix):
        out = []
        for branch, name in ((spec.left, spec.left_name), (spec.right, spec.right_name)):
            out += part_class(MIXERS, branch).declare(branch, f"{prefix}.{name}")
        return out + [TensorDecl(n, (spec.hidden_size,), NORM) for n in cls._norm_names(spec, prefix)]

    @classmethod
    def cache_request(cls, spec):
        requests = [part_class(MIXERS, b).cache_request(b) for b in (spec.left, spec.right)]
        pages = [p for p in (paged_part(r) for r in requests) if p is not None]
        if len(pages) > 1:
            raise ValueError("parallel_mixers: only one branch may keep pages of keys")
        total = sum(_record_sizes(spec))
        out = tuple(pages) + ((FixedStateRequest((total,)),) if total else ())
        return out[0] if len(out) == 1 else (out or None)

    def load(self, store):
        self.left.load(store)
        self.right.load(store)
        self.w_left, self.w_right = (store.get(n) for n in self._norm_names(self.spec, self.prefix))

    def _branch_cache(self, cache: LayerCache, index: int) -> LayerCache:
        start = sum(self.sizes[:index])
        state = cache.state[:, start:start + self.sizes[index]] if self.sizes[index] else None
        return LayerCache(group=cache.group, k=cache.k, v=cache.v, state=state, page_size=cache.page_size)

    def forward(self, ctx, x, cache, owns_cache):
        a = K.plain_unless(None, self.left.forward(ctx, x, self._branch_cache(cache, 0), owns_cache))
        b = K.plain_unless(None, self.right.forward(ctx, x, self._branch_cache(cache, 1), owns_cache))
        out = torch.empty((x.shape[0], self.spec.hidden_size), dtype=x.dtype, device=x.device)
        K.norm_sum2(a, b, self.w_left, self.w_right, self.spec.eps, self.spec.factor, out)
        return out

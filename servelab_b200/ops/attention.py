"""Chooses and launches the attention kernel for a step.

  float32                      plain kernel (CUDA cores, float32 throughout)
  bfloat16, all q_len == 1     split-KV decode kernel (tensor cores)
  bfloat16, otherwise          tensor-core prefill kernel
  bfloat16, head size not a    plain kernel
  multiple of 16

``force_generic`` switches every call to the plain kernel (tests and
measurements compare the fast kernels with it).
"""

from __future__ import annotations

import torch

from . import kernels as K
from . import library as L

force_generic = False
use_decode_kernel = True
use_prefill_kernel = True
MAX_HEAD_DIM = 256


def check_supported(head_dim: int, dtype: torch.dtype) -> None:
    if head_dim < 1 or head_dim > MAX_HEAD_DIM:
        raise L.KernelError(f"attention kernels take head sizes 1..{MAX_HEAD_DIM}, got {head_dim}")


def _generic(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale, window):
    g = H // Hkv
    tile_seq, tile_row0, n = ctx.attention_tiles(g, K.generic_attention_tile_rows())
    K.paged_attention_generic(q, k_cache, v_cache, out, table, ctx.cu_q, ctx.ctx_len, tile_seq,
                              tile_row0, n, H, Hkv, D, page_size, scale, window)


def paged_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale,
                    window) -> None:
    if q.dtype == torch.bfloat16 and not force_generic and K.has_fast_attention(D):
        if ctx.decode_only and use_decode_kernel:
            K.decode_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale,
                               window)
            return
        if use_prefill_kernel:
            K.prefill_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size,
                                scale, window)
            return
    _generic(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale, window)


# ---------------------------------------------- attention with mixed heads
use_talk_fast = True       # bfloat16: the tensor-core instances (off: the plain kernel, their twin)


def _talk_fast(head_dim: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and use_talk_fast and not force_generic and K.has_fast_attention(head_dim)


def prepare_talk_attention(head_dim: int, dtype: torch.dtype) -> None:
    """Builds what ``talk_attention`` will launch for this head size (at load, not in a step)."""
    if _talk_fast(head_dim, dtype) and torch.cuda.is_available():
        L.attention(head_dim)


def talk_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale, window,
                   bias_r1, bias_r2, talk, gate) -> None:
    """Windowed attention with a log-distance bias, then the heads' softmax weights mixed by
    ``talk`` [H, H] (None: not mixed) and the result multiplied by sigmoid(``gate``) (None:
    not gated), into ``out`` [T, H D].  Mixed heads go through the results of every (query
    head, kv head) pair, float32 [T, H, Hkv, D], which ``mix_heads_gate`` combines (with the
    key splits of a decode step).  float32: the plain kernel; bfloat16: the tensor-core
    instances (decode kernel for steps of single tokens, prefill kernel otherwise)."""
    T = q.shape[0]
    nvh = Hkv if talk is not None else 1
    if _talk_fast(D, q.dtype):
        if ctx.decode_only and use_decode_kernel:
            pairs, pair_ml = K.talk_decode_attention(ctx, q, k_cache, v_cache, table, H, Hkv, D,
                                                     page_size, scale, window, bias_r1, bias_r2, nvh)
            K.mix_heads_gate(pairs, None, talk, gate, out, H, Hkv, D, pair_ml)
            return
        pairs = torch.empty((T, H, nvh, D), dtype=torch.float32, device=q.device)
        K.talk_prefill_attention(ctx, q, k_cache, v_cache, table, H, Hkv, D, page_size, scale, window,
                                 bias_r1, bias_r2, pairs)
        K.mix_heads_gate(pairs, None, talk, gate, out, H, Hkv, D)
        return
    tile_seq, tile_row0, n = ctx.attention_tiles(H // Hkv, K.generic_attention_tile_rows())
    if talk is None:
        K.paged_attention_generic(q, k_cache, v_cache, out, table, ctx.cu_q, ctx.ctx_len, tile_seq,
                                  tile_row0, n, H, Hkv, D, page_size, scale, window, bias_r1, bias_r2)
        if gate is not None:
            K.mix_heads_gate(None, out, None, gate, out, H, Hkv, D)
        return
    pairs = torch.empty((T, H, Hkv, D), dtype=torch.float32, device=q.device)
    K.paged_attention_generic(q, k_cache, v_cache, None, table, ctx.cu_q, ctx.ctx_len, tile_seq,
                              tile_row0, n, H, Hkv, D, page_size, scale, window, bias_r1, bias_r2, pairs)
    K.mix_heads_gate(pairs, None, talk, gate, out, H, Hkv, D)


# ------------------------------- attention with keys and values of two sizes
KV_MAX_KEY_DIM, KV_MAX_VALUE_DIM = 1088, 512


def check_kv_supported(key_dim: int, value_dim: int) -> None:
    if not 0 < key_dim <= KV_MAX_KEY_DIM or not 0 < value_dim <= KV_MAX_VALUE_DIM:
        raise L.KernelError(f"attention kernels take keys of 1..{KV_MAX_KEY_DIM} and values of "
                            f"1..{KV_MAX_VALUE_DIM} elements, got {key_dim} and {value_dim}")


use_equal_size_kernels = True
use_kv_tc_capped = True    # a cap or a sink in steps with prompt portions: the tcgen05 kernel (off: mma.sync)
use_kv_fast = True         # bfloat16: the tensor-core kernel (off: the plain kernel, its twin)
KV_FAST_MAX_KEY_DIM, KV_FAST_MAX_VALUE_DIM = 320, 256


def _kv_fast(key_dim: int, value_dim: int, dtype: torch.dtype) -> bool:
    return (dtype == torch.bfloat16 and use_kv_fast and not force_generic
            and key_dim % 16 == 0 and value_dim % 16 == 0
            and key_dim <= KV_FAST_MAX_KEY_DIM and value_dim <= KV_FAST_MAX_VALUE_DIM)


def prepare_kv_attention(key_dim: int, value_dim: int, dtype: torch.dtype) -> None:
    """Builds what ``kv_attention`` will launch for these sizes (at load, not in a step)."""
    if _kv_fast(key_dim, value_dim, dtype) and torch.cuda.is_available():
        L.attention_kv(key_dim, value_dim)


def kv_attention(ctx, q, k_cache, v_cache, v_row_stride, out, table, H, Hkv, Dk, Dv, page_size, scale,
                 window, head_gate, softcap=None, sink=None) -> None:
    """Attention with keys of ``Dk`` and values of ``Dv`` elements (value rows ``v_row_stride``
    apart in ``v_cache``, which may be the key cache: the values are then a prefix of the key
    rows), causal with an optional window, head h's row times sigmoid(head_gate[t, h]) if given.
    ``softcap``: a scaled score s becomes softcap tanh(s / softcap); ``sink`` float32 [H]: a
    number a head whose exponential joins the softmax's denominator.  The tcgen05 kernel for two
    sizes, the mma.sync kernel and the plain kernel take both; the kernels for equal sizes of the
    other models take neither, so a mixer that has one does not reach them.
    float32, or sizes the tensor-core kernel does not take: the plain kernel."""
    tied = v_cache.data_ptr() == k_cache.data_ptr() and v_row_stride == Dk
    modified = bool(softcap) or sink is not None
    if (Dk == Dv and not tied and not modified and v_row_stride == Dv and q.dtype == torch.bfloat16 and not force_generic
            and use_equal_size_kernels and K.has_fast_attention(Dk) and Dk in (64, 128)):
        # keys and values of one size the tcgen05 kernels take: the framework's attention for
        # equal sizes (tcgen05 prefill, one-launch decode), then the gate in a pass of its own
        paged_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, Dk, page_size, scale, window)
        if head_gate is not None:
            K.sigmoid_gate(out, head_gate, out, group=Dv)
        return
    if _kv_fast(Dk, Dv, q.dtype) and (tied or v_row_stride == Dv) and q.stride(0) % 8 == 0 \
            and out.stride(0) % 2 == 0:
        if (not ctx.decode_only and out.stride(0) % 8 == 0 and (use_kv_tc_capped or not modified)
                and K.attention_kv_tc_takes(Dk, Dv, page_size, H // Hkv, tied)):
            K.attention_kv_tc(ctx, q, k_cache, v_cache, tied, out, table, H, Hkv, Dk, Dv, page_size, scale,
                              window, head_gate, softcap or 0.0, sink)
            return
        K.attention_kv_mma(ctx, q, k_cache, v_cache, tied, out, table, H, Hkv, Dk, Dv, page_size, scale,
                           window, head_gate, softcap or 0.0, sink)
        return
    K.attention_kv(ctx, q, k_cache, v_cache, v_row_stride, out, table, H, Hkv, Dk, Dv, page_size, scale,
                   window, head_gate, softcap or 0.0, sink)


# ------------------------------------------------- several attention maps a head
use_maps_tc = True         # steps with prompt portions: the tcgen05 kernel where it takes the sizes
def prepare_maps_attention(key_dim: int, value_dim: int, dtype: torch.dtype, maps: int = 1, group: int = 1) -> None:
    """Builds what ``maps_attention`` will launch for these sizes (at load, not in a step)."""
    if _kv_fast(key_dim, value_dim, dtype) and torch.cuda.is_available():
        L.attention_kv(key_dim, value_dim)
        if K.attention_kv_folds(group, maps, key_dim, value_dim):
            L.attention_kv(maps * key_dim, value_dim)     # steps of single tokens


def maps_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, maps, Dk, Dv, page_size, scale, window) -> None:
    """Attention with ``maps`` maps a head (q [T, H, maps, Dk]; a cached key row holds a kv head's
    maps side by side; one set of values a kv head), causal with an optional window; float32
    results per map, [T, H, maps, Dv].  bfloat16 with sizes in multiples of 16: the tensor-core
    kernels built for the pair of sizes (tcgen05 for prompt portions with sizes in multiples of
    64, mma.sync otherwise); float32 or other sizes: the plain kernel."""
    if _kv_fast(Dk, Dv, q.dtype) and q.stride(0) % 8 == 0 and out.stride(0) % 2 == 0:
        if (use_maps_tc and not ctx.decode_only and out.stride(0) % 4 == 0
                and K.attention_kv_tc_takes(Dk, Dv, page_size, H // Hkv, False)):
            # steps with portions of prompts, sizes in multiples of 64: the tcgen05 kernel
            K.attention_kv_tc_maps(ctx, q, k_cache, v_cache, out, table, H, Hkv, maps, Dk, Dv, page_size, scale,
                                   window)
            return
        K.attention_kv_mma_maps(ctx, q, k_cache, v_cache, out, table, H, Hkv, maps, Dk, Dv, page_size, scale, window)
        return
    K.attention_kv_maps(ctx, q, k_cache, v_cache, out, table, H, Hkv, maps, Dk, Dv, page_size, scale, window)

"""Python entry points of the CUDA kernels (thin: pointer passing, no math).

Every function launches on torch's current CUDA stream and returns without
synchronising.  Tensors must be CUDA tensors, contiguous in their last dimension.
The dtype of the activations selects the float32 or the bfloat16 instance.
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from . import library as L

_F32, _BF16 = torch.float32, torch.bfloat16


launch_count = 0       # launches of this package's kernels (library GEMMs not included)


class SplitSum:
    """A [M, N] result that exists as float32 partial sums ``parts`` [splits, M, N]
    of a matrix product split along K (plus an optional float32 ``bias`` [N] still
    to be added).  Kernels that consume it add the parts in order, so no separate
    reduction is launched; ``materialize()`` produces the plain tensor."""

    accept_flag = "accepts_split_sum"

    def __init__(self, parts: torch.Tensor, bias: Optional[torch.Tensor], dtype: torch.dtype):
        self.parts, self.bias, self.dtype = parts, bias, dtype

    @property
    def shape(self):
        return self.parts.shape[1:]

    def materialize(self) -> torch.Tensor:
        S, M, N = self.parts.shape
        out = torch.empty((M, N), dtype=self.dtype, device=self.parts.device)
        L.check(L.core().slb_split_sum(self.parts.data_ptr(), out.data_ptr(), out.stride(0),
                                       _p(self.bias), 1 if self.dtype == _F32 else 0, M, N, S,
                                       _stream()), "split_sum")
        return out


class DeferredLinear:
    """A [M, N] result x . w^T (+ bias) whose product has not been launched: the consumer
    (a norm that takes it) launches the product with its own work in the product's epilogue
    (``gemm_tc_resid_norm``).  ``materialize()`` runs the plain product."""

    accept_flag = "accepts_deferred_linear"

    def __init__(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]):
        self.x, self.w, self.bias = x, w, bias

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])

    def materialize(self) -> torch.Tensor:
        return gemm_tc_cluster(self.x, self.w, None, self.bias)


class ScaledRows:
    """Normed rows [M, h] without their factor 1 / rms: ``z`` = bfloat16(resid * weight) and
    ``sumsq`` [M, tiles], the sums of squares of resid per 128-column tile, as
    ``gemm_tc_resid_norm`` leaves them.  A matrix product that takes this form multiplies
    its result by 1 / sqrt(sum(sumsq) / h + eps) per token in its epilogue, which equals the
    product of the normed rows because the factor is one number a row.  ``materialize()``
    runs the norm kernel on the (already updated) residual stream."""

    accept_flag = "accepts_scaled_rows"

    def __init__(self, z, sumsq, eps: float, resid, weight):
        self.z, self.sumsq, self.eps, self.resid, self.weight = z, sumsq, eps, resid, weight

    @property
    def shape(self):
        return self.z.shape

    @property
    def dtype(self):
        return self.z.dtype

    @property
    def device(self):
        return self.z.device

    def materialize(self) -> torch.Tensor:
        out = torch.empty_like(self.z)
        add_rmsnorm(self.resid, None, self.weight, self.eps, out)
        return out


def plain_unless(part, value):
    """``value`` as a tensor unless it is an unfinished form (``SplitSum``, ``DeferredLinear``,
    ``ScaledRows``) and ``part`` says (by the form's flag) that it takes it."""
    flag = getattr(type(value), "accept_flag", None)
    if flag is not None and not getattr(part, flag, False):
        return value.materialize()
    return value


# the current stream's handle without building a torch.cuda.Stream object for it (a few
# microseconds a launch, which a step of a small model notices)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    global launch_count
    launch_count += 1
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _suffix(dt: torch.dtype) -> str:
    if dt == _F32:
        return "f32"
    if dt == _BF16:
        return "bf16"
    raise L.KernelError(f"kernels take float32 or bfloat16, not {dt}")


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise L.KernelsUnavailable(
            "servelab_b200 needs a CUDA device (sm_100a): there is no CPU path")
    L.core()


# ------------------------------------------------------------- elementwise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as float32; ids int32 [T], out float32 [T, h]."""
    fn = getattr(L.core(), "slb_embedding_" + _suffix(table.dtype))
    L.check(fn(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(), table.shape[1],
               table.shape[0], float(scale), _stream()), "embedding")


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> None:
    """In place on float32 logits [R, V]: times ``scale``, then with ``softcap`` > 0 bounded to
    softcap * tanh(x / softcap)."""
    if logits.dtype != _F32:
        raise L.KernelError("logit_transform: float32 logits only")
    L.check(L.core().slb_logit_transform(logits.data_ptr(), logits.stride(0), logits.shape[0],
                                         logits.shape[1], float(scale), float(softcap), _stream()),
            "logit_transform")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, row_map: Optional[torch.Tensor] = None) -> None:
    """resid += delta (in place, float32; skipped when ``row_map`` selects rows);
    out[r] = rmsnorm(resid[src(r)] (+ delta)) * weight."""
    rows = out.shape[0]
    if isinstance(delta, SplitSum):
        if out.dtype != _BF16:
            delta = delta.materialize()
        else:
            S, M, N = delta.parts.shape
            L.check(L.core().slb_add_rmsnorm_parts_bf16(
                resid.data_ptr(), delta.parts.data_ptr(), S, M * N, _p(delta.bias),
                weight.data_ptr(), out.data_ptr(), _p(row_map), rows, out.shape[1], float(eps),
                _stream()), "add_rmsnorm")
            return
    fn = getattr(L.core(), "slb_add_rmsnorm_" + _suffix(out.dtype))
    L.check(fn(resid.data_ptr(), _p(delta), weight.data_ptr(), out.data_ptr(), _p(row_map),
               rows, out.shape[1], float(eps), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t, i] = silu(gate_i) * up_i of row t of ``gate_up`` ([T, 2 I], I = out.shape[1]).
    ``block`` == 0: a row holds all gates, then all ups; ``block`` > 0: gates and ups
    alternate in runs of ``block`` elements."""
    fn = getattr(L.core(), "slb_swiglu_" + _suffix(out.dtype))
    L.check(fn(gate_up.data_ptr(), out.data_ptr(), out.shape[0], out.shape[1],
               gate_up.stride(0), out.stride(0), int(block), _stream()), "swiglu")


# ----------------------------------------------------- rotary + cache write
def _num_pages(cache: Optional[torch.Tensor]) -> int:
    """Pages in a layer's cache [pages, kv heads, page size, head size]: the kernels skip a
    block-table entry beyond it (and set a status word) instead of touching memory outside."""
    return 0 if cache is None else cache.shape[0]


def cache_write_status(reset: bool = False) -> int:
    """0 unless the q/k/v kernel met a block-table entry outside the cache (synchronises)."""
    return L.core().slb_cache_write_status(1 if reset else 0)


def generic_attention_status(reset: bool = False) -> int:
    """0 unless the plain attention kernel met a block-table entry outside the cache."""
    return L.core().slb_paged_attention_generic_status(1 if reset else 0)


def qkv_rope_cache(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                   seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                   inv_freq: Optional[torch.Tensor], rotary_dim: int, q_out: torch.Tensor,
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    if isinstance(qkv, SplitSum):
        if bias is not None and qkv.bias is not None:
            raise L.KernelError("qkv_rope_cache: two biases")
        if q_out.dtype != _BF16:
            qkv = qkv.materialize()
        else:
            S, M, N = qkv.parts.shape
            L.check(L.core().slb_qkv_rope_cache_parts_bf16(
                qkv.parts.data_ptr(), S, M * N, N, _p(bias if bias is not None else qkv.bias),
                positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                block_table.shape[1], page_size, _num_pages(k_cache), _p(inv_freq), rotary_dim,
                q_out.data_ptr(), q_out.stride(0), _p(k_cache), _p(v_cache), M, num_heads,
                num_kv_heads, head_dim, _stream()), "qkv_rope_cache")
            return
    fn = getattr(L.core(), "slb_qkv_rope_cache_" + _suffix(qkv.dtype))
    L.check(fn(qkv.data_ptr(), qkv.stride(0), _p(bias), positions.data_ptr(),
               seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
               _num_pages(k_cache), _p(inv_freq), rotary_dim, q_out.data_ptr(), q_out.stride(0), _p(k_cache),
               _p(v_cache), qkv.shape[0], num_heads, num_kv_heads, head_dim, _stream()),
            "qkv_rope_cache")


# ---------------------------------------------------------------- attention
def generic_attention_tile_rows() -> int:
    return L.core().slb_paged_attention_generic_tile_rows()


def paged_attention_generic(q, k_cache, v_cache, out, block_table, cu_q, ctx_len, tile_seq,
                            tile_row0, num_tiles: int, num_heads: int, num_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int,
                            bias_r1: Optional[torch.Tensor] = None,
                            bias_r2: Optional[torch.Tensor] = None,
                            pair_out: Optional[torch.Tensor] = None) -> None:
    """``bias_r1`` / ``bias_r2`` (float32 [H]): r1_h ln(1 + r2_h distance) is subtracted from the
    scaled scores.  ``pair_out`` (float32 [T, H, Hkv, D]): instead of ``out`` (may be None then)
    the result of every query head's weights applied to every kv head's values."""
    fn = getattr(L.core(), "slb_paged_attention_generic_" + _suffix(q.dtype))
    L.check(fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), _p(out),
               out.stride(0) if out is not None else 0, block_table.data_ptr(), block_table.shape[1],
               cu_q.data_ptr(), ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), num_tiles,
               num_heads, num_kv_heads, head_dim, page_size, k_cache.shape[0], float(scale),
               int(window), _p(bias_r1), _p(bias_r2), _p(pair_out), _stream()), "paged_attention_generic")


def mix_heads_gate(pairs: Optional[torch.Tensor], direct: Optional[torch.Tensor],
                   talk: Optional[torch.Tensor], gate: Optional[torch.Tensor], out: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int,
                   pair_ml: Optional[torch.Tensor] = None) -> None:
    """out[t, h] = (sum_g talk[h, g] pairs[t, g, c(h)]) * sigmoid(gate[t, h]); with ``pairs``
    None, ``direct`` [T, H D] takes the place of the sum.  ``pairs`` float32 [T, H, nvh, D]
    (nvh = Hkv, or 1 without ``talk``), or with ``pair_ml`` [T, H, nvh, splits, 2] the
    unnormalised partials [T, H, nvh, splits, D] of split key ranges, combined here.  ``gate``
    [T, H D] may be a view of a wider projection (its row stride is passed); ``talk`` float32
    [H, H]."""
    fn = getattr(L.core(), "slb_mix_heads_gate_" + _suffix(out.dtype))
    splits = pair_ml.shape[3] if pair_ml is not None else 0
    nvh = pairs.shape[2] if pairs is not None else 0
    L.check(fn(_p(pairs), _p(pair_ml), splits, nvh, _p(direct),
               direct.stride(0) if direct is not None else 0, _p(talk),
               _p(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0),
               out.shape[0], num_heads, num_kv_heads, head_dim, _stream()), "mix_heads_gate")


def talk_prefill_attention(ctx, q, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim,
                           page_size, scale, window, bias_r1, bias_r2, pairs: torch.Tensor) -> None:
    """The tensor-core prefill attention with a distance bias, results per (query head, value
    head) pair in ``pairs`` float32 [T, H, nvh, D] (nvh = Hkv: every pair; 1: own kv head)."""
    lib = L.attention(head_dim)
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads,
                                                 lib.slb_prefill_attention_tile_rows())
    L.check(lib.slb_talk_prefill_attention_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_len.data_ptr(), tile_seq.data_ptr(),
        tile_row0.data_ptr(), n, num_heads, num_kv_heads, page_size, k_cache.shape[0], float(scale),
        int(window), _p(bias_r1), _p(bias_r2), pairs.data_ptr(), 1 if pairs.shape[2] > 1 or num_kv_heads == 1 else 0,
        _stream()), "talk_prefill_attention")


def talk_decode_splits(num_seqs: int, num_kv_heads: int, group: int, value_groups: int,
                       longest_context: int, window: int, max_splits: int) -> int:
    """Key splits of the decode kernel for mixed heads: enough blocks for ``decode_ctas_per_sm``
    per SM, at most one split per 64 keys a query can see.  ``value_groups``: blocks per (request,
    kv head), each finishing a group of value heads."""
    seen = min(longest_context, window + 63) if window > 0 else longest_context
    ctas = num_seqs * num_kv_heads * value_groups * ((group + 15) // 16)
    want = max(1, (decode_ctas_per_sm * _num_sms()) // max(ctas, 1))
    return max(1, min(want, max_splits, -(-seen // 64)))


def talk_decode_attention(ctx, q, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim,
                          page_size, scale, window, bias_r1, bias_r2, nvh: int):
    """The split-key decode attention with a distance bias for steps of single tokens; returns
    (pairs [S, H, nvh, splits, D], pair_ml [S, H, nvh, splits, 2]), float32 partials that
    ``mix_heads_gate`` combines."""
    lib = L.attention(head_dim)
    S = ctx.num_seqs
    per_block = lib.slb_talk_attention_value_heads()
    splits = talk_decode_splits(S, num_kv_heads, num_heads // num_kv_heads, -(-nvh // per_block),
                                ctx.split_hint_len, window, lib.slb_decode_attention_max_splits())
    pairs = torch.empty((S, num_heads, nvh, splits, head_dim), dtype=_F32, device=q.device)
    pair_ml = torch.empty((S, num_heads, nvh, splits, 2), dtype=_F32, device=q.device)
    L.check(lib.slb_talk_decode_attention_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], ctx.ctx_len.data_ptr(), S, num_heads, num_kv_heads, page_size,
        k_cache.shape[0], float(scale), int(window), splits, _p(bias_r1), _p(bias_r2),
        pairs.data_ptr(), pair_ml.data_ptr(), 1 if nvh > 1 or num_kv_heads == 1 else 0, _stream()),
        "talk_decode_attention")
    return pairs, pair_ml


def dyt_add_norm(resid: torch.Tensor, delta: Optional[torch.Tensor], post, pre,
                 out: Optional[torch.Tensor], row_map: Optional[torch.Tensor] = None) -> None:
    """Dynamic Tanh around a residual add.  ``post`` / ``pre`` are (alpha, weight, bias)
    float32 device tensors or None.  d = post(delta) (or delta); resid += d in place (not when
    ``row_map`` selects rows); out[r] = pre(resid[src(r)] + d)."""
    dtype = out.dtype if out is not None else delta.dtype
    rows = out.shape[0] if out is not None else resid.shape[0]
    pa, pw, pb = post if post is not None else (None, None, None)
    a, w, b = pre if pre is not None else (None, None, None)
    fn = getattr(L.core(), "slb_dyt_add_norm_" + _suffix(dtype))
    L.check(fn(resid.data_ptr(), resid.stride(0), _p(delta), delta.stride(0) if delta is not None else 0,
               _p(pa), _p(pw), _p(pb), _p(a), _p(w), _p(b), _p(out),
               out.stride(0) if out is not None else 0, _p(row_map), rows, resid.shape[1], _stream()),
            "dyt_add_norm")


def qk_conv_cache(proj: torch.Tensor, taps_w: torch.Tensor, state: Optional[torch.Tensor], ctx,
                  block_table: torch.Tensor, page_size: int, temp_coef: float, temp_every: int,
                  q_out: torch.Tensor, k_cache: Optional[torch.Tensor], num_kv_heads: int,
                  head_dim: int) -> None:
    """Causal convolution over time (``taps_w`` float32 [taps, C]: transposed) on the first C = q width +
    kv width columns of ``proj``, with the rows before a portion taken from ``state``
    (float32 [slots, taps - 1, C], indexed by ``ctx.state_slots`` and updated); queries times
    their temperature into ``q_out``, keys into the pages of ``k_cache`` (None: not written)."""
    fn = getattr(L.core(), "slb_qk_conv_cache_" + _suffix(proj.dtype))
    n = 1 if (taps_w.shape[0] == 1 or ctx.decode_only) else 2
    L.check(fn(proj.data_ptr(), proj.stride(0), taps_w.data_ptr(), taps_w.shape[0], _p(state),
               ctx.state_slots.data_ptr(), ctx.cu_q.data_ptr(), ctx.seq_of_token.data_ptr(),
               ctx.positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
               _num_pages(k_cache), float(temp_coef), int(temp_every), q_out.data_ptr(), q_out.stride(0),
               _p(k_cache), proj.shape[0], ctx.num_seqs, q_out.shape[1], num_kv_heads, head_dim,
               1 if ctx.decode_only else 0, state.stride(0) if state is not None else 0, _stream()),
            "qk_conv_cache")
    global launch_count
    launch_count += n - 1


def short_conv(proj: torch.Tensor, taps_w: torch.Tensor, state: Optional[torch.Tensor], ctx,
               out: torch.Tensor) -> None:
    """The convolution alone: y_t = sum_i taps_w[i] u_(t - taps + 1 + i) on the first C = out.shape[1]
    columns of ``proj`` into ``out`` [T, C]; the rows before a portion come from ``state`` (float32
    [slots, >= (taps - 1) * C], a request's record at ``ctx.state_slots``; rows of the record may be
    ``state.stride(0)`` apart, so it can be a slice of a larger record), which is left holding the
    last taps - 1 projected rows."""
    fn = getattr(L.core(), "slb_qk_conv_cache_" + _suffix(proj.dtype))
    n = 1 if (taps_w.shape[0] == 1 or ctx.decode_only) else 2
    L.check(fn(proj.data_ptr(), proj.stride(0), taps_w.data_ptr(), taps_w.shape[0], _p(state),
               ctx.state_slots.data_ptr(), ctx.cu_q.data_ptr(), ctx.seq_of_token.data_ptr(),
               ctx.positions.data_ptr(), None, 0, 1, 0, 0.0, 1, out.data_ptr(), out.stride(0),
               None, proj.shape[0], ctx.num_seqs, out.shape[1], 0, 0,
               1 if ctx.decode_only else 0, state.stride(0) if state is not None else 0, _stream()),
            "short_conv")
    global launch_count
    launch_count += n - 1


CONV_MAX_TAPS = 64             # most taps the convolution kernel is launched with


def conv_cache_status(reset: bool = False) -> int:
    """0 unless the convolution kernel met a block-table entry outside the cache."""
    return L.core().slb_conv_cache_status(1 if reset else 0)


# ---------------------------------------------------------- matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = a[M,K] . w[N,K]^T (+ bias) on CUDA cores, float32 accumulation."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype == _F32 and out.dtype == _F32:
        fn = L.core().slb_gemm_simt_f32
    elif a.dtype == _BF16 and out.dtype == _BF16:
        fn = L.core().slb_gemm_simt_bf16
    elif a.dtype == _BF16 and out.dtype == _F32:
        fn = L.core().slb_gemm_simt_bf16_f32out
    else:
        raise L.KernelError(f"gemm_simt: unsupported dtypes {a.dtype} -> {out.dtype}")
    L.check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
               out.stride(0), _p(bias), M, N, K, _stream()), "gemm_simt")


# ----------------------------------------------------------------- sampling
def sample_rows(logits: torch.Tensor, out: torch.Tensor, temperature=None, top_k=None,
                top_p=None, seed=None, stream=None, position=None) -> None:
    """out[r] = sampled token of row r; all per-row parameter arrays live on the
    device (float32 / int32 / int64); ``temperature=None`` means greedy rows."""
    R, V = logits.shape
    L.check(L.core().slb_sample_rows(
        logits.data_ptr(), logits.stride(0), R, V, _p(temperature), _p(top_k), _p(top_p),
        _p(seed), _p(stream), _p(position), out.data_ptr(), _stream()), "sample_rows")


# ------------------------------------- tensor-core attention (bfloat16 only)
_sm_count = None
decode_ctas_per_sm = 2      # blocks per SM the split heuristic aims for


def _num_sms() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def attention_status(head_dim: int, reset: bool = False) -> int:
    """0 unless a bounded wait inside the tensor-core attention kernels for this head
    size gave up (synchronises with the device)."""
    return L.attention(head_dim).slb_attention_status(1 if reset else 0)


def prefill_attention_tc_status(head_dim: int, reset: bool = False) -> int:
    """0 unless a bounded wait inside the tcgen05 prefill attention gave up."""
    return L.attention(head_dim).slb_prefill_attention_tc_status(1 if reset else 0)


def prefill_attention_tc_where(head_dim: int) -> dict:
    """Where the roles of the tcgen05 prefill attention gave up a bounded wait last:
    per role (code, block, key tile, key tiles of the block); zeros if never."""
    import ctypes
    buf = (ctypes.c_int * 12)()
    L.attention(head_dim).slb_prefill_attention_tc_where(ctypes.cast(buf, ctypes.c_void_p))
    out = {}
    for i, role in enumerate(("loader", "mma", "softmax")):
        code, block, tile, ntiles = buf[4 * i:4 * i + 4]
        out[role] = {"code": hex(code), "block": block, "tile": tile, "tiles": ntiles}
    return out


def has_fast_attention(head_dim: int) -> bool:
    """The tensor-core kernels exist for head sizes that are multiples of 16 up to
    256; the library for a head size is built when it is first asked for."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


use_tc_prefill = True       # tcgen05 prefill attention where it applies (head size 64/128)


def prefill_attention(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                      head_dim, page_size, scale, window) -> None:
    lib = L.attention(head_dim)
    group = num_heads // num_kv_heads
    if (use_tc_prefill and hasattr(lib, "slb_prefill_attention_tc_bf16")
            and lib.slb_prefill_attention_tc_supported(page_size, group)):
        tile_seq, tile_row0, n = ctx.attention_tiles(group, lib.slb_prefill_attention_tc_tile_rows(group))
        L.check(lib.slb_prefill_attention_tc_bf16(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
            out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(),
            ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads,
            num_kv_heads, page_size, k_cache.shape[0], float(scale), int(window), _stream()),
            "prefill_attention_tc")
        return
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads,
                                                 lib.slb_prefill_attention_tile_rows())
    L.check(lib.slb_prefill_attention_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(),
        ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads,
        num_kv_heads, page_size, k_cache.shape[0], float(scale), int(window), _stream()),
        "prefill_attention")


def decode_splits(num_seqs: int, num_kv_heads: int, group: int, longest_context: int,
                  max_splits: int) -> int:
    """How many ways the keys of each request are split: enough blocks for
    ``decode_ctas_per_sm`` per SM, at most one split per 64 keys of the longest
    context."""
    ctas = num_seqs * num_kv_heads * ((group + 15) // 16)
    want = max(1, (decode_ctas_per_sm * _num_sms()) // max(ctas, 1))
    return max(1, min(want, max_splits, -(-longest_context // 64)))


def decode_attention_split(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                           head_dim, page_size, scale, window) -> None:
    """Attention for a step of single tokens, earlier form: four warps share every
    64-key tile behind a block-wide barrier and a second kernel combines the splits.
    Kept as the twin of ``decode_attention``."""
    lib = L.attention(head_dim)
    S = ctx.num_seqs
    splits = decode_splits(S, num_kv_heads, num_heads // num_kv_heads, ctx.split_hint_len,
                           lib.slb_decode_attention_max_splits())
    scratch = None
    if splits > 1:
        nbytes = lib.slb_decode_attention_scratch_bytes(S, num_heads, splits)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
    L.check(lib.slb_decode_attention_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.ctx_len.data_ptr(),
        _p(scratch), S, num_heads, num_kv_heads, page_size, k_cache.shape[0], float(scale),
        int(window), splits, _stream()), "decode_attention")
    global launch_count
    launch_count += 1 if splits > 1 else 0          # the combine kernel


decode_ws_stages = 3           # depth of the kernel's shared-memory ring (2..4)
decode_ws_force_splits = 0     # measurements: launch this many splits instead of the choice below
# The kernel picks each request's number of splits itself, from the request's own length: one
# while it has at most `decode_ws_unsplit_tiles` 64-key tiles, and never more splits than were
# launched.  In the cluster form (the default) a split has two tiles at least, and a request
# takes more splits than one cluster holds only when that saves a block four tiles or more
# (a tile costs a block about 0.8 us while the GPU is not full, a second level of combining
# about 3 us).  In the arrival-counter form (the twin) a split has about
# `decode_ws_split_coef` * sqrt(tiles) tiles: there one block combines every split.
decode_ws_split_coef = 0.8
decode_ws_unsplit_tiles = 6    # (us at 256 / 512 keys, batch 8: 5.4 / 8.4 with 12, 5.4 / 6.0 with 6, 5.9 / 6.0 with 3)

_DECODE_COUNTERS = 1 << 16     # arrival counters held per device (256 KiB)
_decode_counters: Dict[int, torch.Tensor] = {}


def _decode_counter_buffer(device: torch.device) -> torch.Tensor:
    """Zeroed once; every launch of the decode kernel leaves the counters zero.  One
    fixed buffer per device, so addresses captured in CUDA graphs stay valid."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    buf = _decode_counters.get(index)
    if buf is None:
        buf = _decode_counters[index] = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32,
                                                    device=device)
    return buf


def decode_ws_splits(num_seqs: int, num_kv_heads: int, group: int, longest_context: int,
                     max_splits: int, tile_keys: int, cluster: bool = False) -> int:
    """The most splits a request may use (the launch's grid): as many as keep all
    blocks of the step resident at once (two per SM), 1 for short contexts.  ``cluster``:
    the kernel's rule for the cluster form (two tiles a split at least) instead of the one
    for the arrival counter (about ``decode_ws_split_coef`` * sqrt(tiles) tiles a split)."""
    head_rows = 8 if group <= 8 else 16
    pairs = num_seqs * num_kv_heads * (-(-group // head_rows))
    tiles = max(1, -(-longest_context // tile_keys))
    if tiles <= decode_ws_unsplit_tiles:
        return 1
    slots = 2 * _num_sms()                      # two blocks of three stages fit on an SM
    per = 2 if cluster else max(1, math.ceil(decode_ws_split_coef * math.sqrt(tiles)))
    longest_uses = -(-tiles // per)             # the kernel's own rule for the longest context
    return max(1, min(max_splits, slots // max(pairs, 1), longest_uses))


def decode_attention_takes(head_dim: int, page_size: int) -> bool:
    """Whether the one-launch decode kernel takes this head size and page size."""
    return has_fast_attention(head_dim) and \
        bool(L.attention(head_dim).slb_decode_attention_ws_supported(page_size))


# The splits of a request combine through the shared memory of a thread-block cluster when
# there are at most eight of them (no scratch, no arrival counter, no round trip through the
# L2 cache: 7 us -> 2 us after the last key at batch 8 on the 7B shape).  A step that would
# like more splits but already has enough blocks to fill the GPU with eight takes eight; one
# with few requests and long contexts takes several clusters a request (up to 64 splits), whose
# partial results meet in global memory: every block of the cluster that finishes a slice of
# the outputs last combines that slice (at batch 1 the arrival-counter form, where one block
# combined everything, spent 16 us there whatever the number of splits).
decode_ws_cluster = True


def _decode_launch_shape(ctx, lib, q_device, num_heads, num_kv_heads):
    """(splits, scratch, counters, cluster) of a launch of the one-launch decode kernel."""
    S = ctx.num_seqs
    group = num_heads // num_kv_heads
    splits = decode_ws_force_splits or decode_ws_splits(
        S, num_kv_heads, group, ctx.split_hint_len, lib.slb_decode_attention_ws_max_splits(),
        lib.slb_decode_attention_ws_tile_keys(), decode_ws_cluster)
    scratch = counters = None
    cluster = False
    most = lib.slb_decode_attention_ws_max_cluster_splits()
    if splits > 1 and decode_ws_cluster:
        pairs = S * num_kv_heads * (-(-group // (8 if group <= 8 else 16)))
        if splits > most and pairs * most >= _num_sms():
            splits = most
        if splits > most:
            splits = splits // most * most          # whole clusters: their results meet in global memory
        cluster = True
    if splits > 1 and (not cluster or splits > most):
        if lib.slb_decode_attention_ws_counters(S, num_heads, num_kv_heads) > _DECODE_COUNTERS:
            splits = 1
        else:
            nbytes = lib.slb_decode_attention_ws_scratch_bytes(S, num_heads, splits)
            scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=q_device)
            counters = _decode_counter_buffer(q_device)
    return splits, scratch, counters, cluster


def decode_attention(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                     head_dim, page_size, scale, window) -> None:
    """Attention for a step of single tokens (every q_len == 1): one launch; the
    splits of a request are combined by the block that finishes last.  Head sizes
    that are no multiple of 64 and page sizes that are no power of two from 8 go to
    ``decode_attention_split``."""
    lib = L.attention(head_dim)
    if not lib.slb_decode_attention_ws_supported(page_size):
        decode_attention_split(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                               head_dim, page_size, scale, window)
        return
    S = ctx.num_seqs
    splits, scratch, counters, cluster = _decode_launch_shape(ctx, lib, q.device, num_heads, num_kv_heads)
    L.check(lib.slb_decode_attention_ws_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.ctx_len.data_ptr(),
        _p(scratch), _p(counters), S, num_heads, num_kv_heads, page_size, k_cache.shape[0],
        float(scale), int(window), splits, int(decode_ws_stages), float(decode_ws_split_coef),
        int(decode_ws_unsplit_tiles), 1 if cluster else 0, _stream()), "decode_attention")


def decode_attention_status(head_dim: int, reset: bool = False) -> int:
    """0 unless a bounded wait inside the decode attention kernel gave up (or a block-table
    entry pointed outside the cache: 0x40)."""
    return L.attention(head_dim).slb_decode_attention_ws_status(1 if reset else 0)


def decode_attention_splits_used(head_dim: int, reset: bool = False) -> int:
    """The most splits any request has used in a launch of the one-launch decode kernel
    since the last reset; 0 if every request ran unsplit (synchronises)."""
    return L.attention(head_dim).slb_decode_attention_ws_splits_used(1 if reset else 0)


# ------------------------------------ tcgen05 weight-streaming product (decode)
TC_MAX_TOKENS = 64
tc_max_stages = 4          # cap on the kernel's shared-memory ring: with four stages two blocks fit
                           # on an SM, and the blocks of the next product become resident (and
                           # request their first weight tiles) beside those of a draining one


tc_blocks_per_sm = 2       # blocks of a product the K split aims at per SM.  Measured on the 7B
                           # shape (ms per decode step at batch 8 / batch 1): 1 block and 6 stages
                           # 3.48 / 3.31, 2 and 4: 3.39 / 3.20, 2 and 5: 3.66 / 3.45, 3 and 3:
                           # 3.45 / 3.22, 4 and 2: 3.48 / 3.26


tc_token_group = 16            # tokens a block takes when a step's tokens are cut into groups
tc_token_group_bytes = 20 << 20    # ... which happens for matrices up to this size from 17 tokens on: every
                                   # group reads the matrix again, from the L2 cache


def tc_token_groups(m: int, w) -> int:
    """Into how many groups of ``tc_token_group`` tokens the tcgen05 products cut a step of
    ``m`` tokens for the matrix ``w`` (1: not at all).  Small matrices only: with few row
    tiles a product has few blocks, and each would finish many tokens one after the other;
    cut into groups it has as many blocks again per group, at the price of reading the
    matrix once per group."""
    if m <= tc_token_group or w.numel() * w.element_size() > tc_token_group_bytes:
        return 1
    return -(-m // tc_token_group)


def tc_decode_splits(n_out: int, k: int, groups: int = 1) -> int:
    """K splits so that (row tiles x token groups x splits) is about ``tc_blocks_per_sm``
    blocks per SM."""
    tiles = -(-n_out // 128) * groups
    kblocks = -(-k // 64)
    slots = tc_blocks_per_sm * _num_sms()
    want = max(1, slots // tiles) if tiles < slots else 1      # all blocks resident at once
    return max(1, min(want, kblocks // 4 if kblocks >= 8 else 1))


# rows of gates, then as many of ups, and so on: the layout for which the tcgen05 product
# applies the activation in its epilogue (half of its 128-row tile)
SWIGLU_BLOCK = 64


def _row_scale(x):
    """(x as the tensor a product reads, sumsq pointer, tiles, eps)"""
    if isinstance(x, ScaledRows):
        return x.z, x.sumsq.data_ptr(), x.sumsq.shape[1], float(x.eps)
    return x, None, 0, 0.0


def gemm_tc_decode(x, w: torch.Tensor, out: Optional[torch.Tensor],
                   bias: Optional[torch.Tensor] = None, splits: int = 0,
                   defer_sum: bool = False, out_dtype: Optional[torch.dtype] = None,
                   swiglu: bool = False):
    """out[M,N] = x[M,K] . w[N,K]^T (+ bias) for up to 64 tokens on tcgen05 tensor
    cores with TMA-streamed weights; bfloat16 operands, float32 or bfloat16 output.
    With ``defer_sum`` and more than one K split the partial sums are returned as a
    ``SplitSum`` (no reduction is launched); otherwise ``out`` (allocated if None).
    ``swiglu``: ``w`` holds gate and up rows alternating in runs of ``SWIGLU_BLOCK``; the
    result is silu(gate) * up, [M, N / 2] (one K split, no bias).  ``x`` may be ``ScaledRows``."""
    global launch_count
    x, sumsq, tiles, eps = _row_scale(x)
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_decode_splits(N, Kd, groups)
    if swiglu:
        if splits != 1 or bias is not None or N % (2 * SWIGLU_BLOCK):
            raise ValueError("gemm_tc_decode: the fused activation needs one K split, no bias and "
                             f"a multiple of {2 * SWIGLU_BLOCK} rows")
        if out is None:
            out = torch.empty((M, N // 2), dtype=out_dtype or x.dtype, device=x.device)
    out_dtype = out.dtype if out is not None else (out_dtype or x.dtype)
    ws = torch.empty((splits, M, N), dtype=_F32, device=x.device) if splits > 1 else None
    deferred = defer_sum and splits > 1
    if out is None and not deferred:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    L.check(L.core().slb_gemm_tc_decode_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _p(out),
        out.stride(0) if out is not None else N,
        _p(bias), _p(ws), 1 if out_dtype == _F32 else 0, M, N, Kd, splits, tc_max_stages,
        1 if deferred else 0, 1 if swiglu else 0, sumsq, tiles, eps,
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_decode")
    if deferred:
        return SplitSum(ws, bias, out_dtype)
    launch_count += 1 if splits > 1 else 0
    return out


TC_MAX_CLUSTER = 8             # K splits that can share a row tile as one thread-block cluster
TC_ROPE_HEAD_DIMS = (16, 32, 64, 128)   # a 128-row tile of the q|k|v product holds whole heads


def tc_cluster_splits(n_out: int, k: int, groups: int = 1) -> int:
    return min(tc_decode_splits(n_out, k, groups), TC_MAX_CLUSTER)


def gemm_tc_cluster(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                    bias: Optional[torch.Tensor] = None, splits: int = 0) -> torch.Tensor:
    """out[M,N] = x . w^T (+ bias) in bfloat16 for up to 64 tokens, like
    ``gemm_tc_decode``, but the K splits of a row tile form a thread-block cluster and
    add their results up through one another's shared memory: no partial sums in
    global memory and no reduction kernel; a fixed order of additions.  ``x`` may be
    ``ScaledRows``."""
    x, sumsq, tiles, eps = _row_scale(x)
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_cluster_splits(N, Kd, groups)
    if out is None:
        out = torch.empty((M, N), dtype=_BF16, device=x.device)
    L.check(L.core().slb_gemm_tc_cluster_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), _p(bias),
        M, N, Kd, splits, _cluster_stages(M, groups), sumsq, tiles, eps,
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_cluster")
    return out


def gemm_tc_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                     positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                     page_size: int, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                     q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                     head_dim: int, splits: int = 0) -> None:
    """The q|k|v product of up to 64 tokens together with ``qkv_rope_cache``: the product's
    epilogue adds the bias, rotates q and k, writes q to ``q_out`` and k, v into the paged
    cache.  Head sizes in ``TC_ROPE_HEAD_DIMS``.  ``x`` may be ``ScaledRows``."""
    x, sumsq, tiles, eps = _row_scale(x)
    M, Kd = x.shape
    groups = tc_token_groups(M, w_qkv)
    splits = splits or tc_cluster_splits(w_qkv.shape[0], Kd, groups)
    L.check(L.core().slb_gemm_tc_qkv_rope_bf16(
        x.data_ptr(), x.stride(0), w_qkv.data_ptr(), w_qkv.stride(0),
        _p(bias), positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, _num_pages(k_cache), _p(inv_freq), rotary_dim,
        q_out.data_ptr(), q_out.stride(0), _p(k_cache), _p(v_cache), M, num_heads, num_kv_heads,
        head_dim, Kd, splits, _cluster_stages(M, groups), sumsq, tiles, eps,
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_qkv_rope")


tc_cluster_many_token_stages = 3   # ring depth of the cluster products above 16 tokens: their x tiles grow
                                   # with the tokens, and with four stages only two blocks fit on an SM,
                                   # which is fewer clusters of eight than a 36-tile product has at once
                                   # (the rest started when the first had finished: 38 against 25 us for
                                   # q|k|v at 64 tokens)


def _cluster_stages(M: int, groups: int = 1) -> int:
    if M <= 16 or (groups > 1 and tc_token_group <= 16):    # (what a block sees)
        return tc_max_stages
    return min(tc_max_stages, tc_cluster_many_token_stages)


def gemm_tc_resid_norm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                       resid: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                       splits: int = 0) -> ScaledRows:
    """The product that closes a residual branch with the add and the RMS norm that follow
    it, in one kernel: resid (float32, in place) += x . w^T (+ bias); the result is the normed
    rows in the form ``ScaledRows`` (bfloat16(resid * norm_weight) and per-tile sums of
    squares), whose factor 1 / rms the next product applies.  Up to 64 tokens."""
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_cluster_splits(N, Kd, groups)
    z = torch.empty((M, N), dtype=_BF16, device=x.device)
    sumsq = torch.empty((M, -(-N // 128)), dtype=_F32, device=x.device)
    L.check(L.core().slb_gemm_tc_resid_norm_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _p(bias), resid.data_ptr(),
        resid.stride(0), norm_weight.data_ptr(), z.data_ptr(), z.stride(0), sumsq.data_ptr(),
        M, N, Kd, splits, _cluster_stages(M, groups), tc_token_group if groups > 1 else 0,
        _stream()), "gemm_tc_resid_norm")
    return ScaledRows(z, sumsq, eps, resid, norm_weight)


def gemm_tc_resid_dyt(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, post, pre,
                      splits: int = 0) -> torch.Tensor:
    """The product that closes a residual branch of a block with Dynamic Tanh norms, in one
    kernel: resid (float32, in place) += post(x . w^T); returns pre(resid) in bfloat16, the
    finished normed rows.  ``post`` / ``pre`` are (alpha, weight, bias) float32 device tensors.
    Up to 64 tokens."""
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_cluster_splits(N, Kd, groups)
    z = torch.empty((M, N), dtype=_BF16, device=x.device)
    L.check(L.core().slb_gemm_tc_resid_dyt_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), resid.data_ptr(), resid.stride(0),
        post[0].data_ptr(), post[1].data_ptr(), post[2].data_ptr(), pre[0].data_ptr(), pre[1].data_ptr(),
        pre[2].data_ptr(), z.data_ptr(), z.stride(0), M, N, Kd, splits, _cluster_stages(M, groups),
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_resid_dyt")
    return z


def gemm_tc_status(reset: bool = False) -> int:
    """0 unless a bounded wait inside the tcgen05 kernels ran out, or the q|k|v epilogue met a
    block-table entry outside the cache (synchronises)."""
    return L.core().slb_gemm_tc_status(1 if reset else 0)


# ------------------------------------------- layer norm around the residual add
def ln_add_norm(resid: torch.Tensor, delta: Optional[torch.Tensor], post, pre,
                out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> None:
    """x = resid (+ LN_post(delta)); resid = x unless ``rows`` selects rows; out = LN_pre(x) or,
    without ``pre``, x in ``out``'s dtype.  ``post`` / ``pre``: (weight, bias, eps) float32, or
    None.  Layer norm: mean and variance over the row, float32."""
    dt = out.dtype if out is not None else delta.dtype
    fn = getattr(L.core(), "slb_ln_add_norm_" + _suffix(dt))
    n = (rows.numel() if rows is not None else resid.shape[0])
    pw, pb, pe = post if post is not None else (None, None, 0.0)
    qw, qb, qe = pre if pre is not None else (None, None, 0.0)
    L.check(fn(resid.data_ptr(), resid.stride(0), _p(delta), delta.stride(0) if delta is not None else 0,
               _p(pw), _p(pb), float(pe), _p(qw), _p(qb), float(qe), _p(out),
               out.stride(0) if out is not None else 0, _p(rows), n, resid.shape[1], _stream()),
            "ln_add_norm")


# ------------------------------- head norms, pair rotation, value mix, cache write
import ctypes as _ct


class _HeadPrepArgs(_ct.Structure):
    _fields_ = [
        ("proj", _ct.c_void_p), ("ld", _ct.c_int),
        ("q_off", _ct.c_int), ("H", _ct.c_int), ("Dq", _ct.c_int), ("q_norm_dims", _ct.c_int),
        ("q_rot_off", _ct.c_int), ("q_norm_w", _ct.c_void_p),
        ("k_off", _ct.c_int), ("G", _ct.c_int), ("Dk", _ct.c_int), ("k_norm_dims", _ct.c_int),
        ("k_rot_off", _ct.c_int), ("k_norm_w", _ct.c_void_p),
        ("v_off", _ct.c_int), ("Dv", _ct.c_int),
        ("lam", _ct.c_void_p), ("v_first", _ct.c_void_p), ("ld_vf", _ct.c_int),
        ("v_keep", _ct.c_void_p), ("ld_vk", _ct.c_int),
        ("freq", _ct.c_void_p), ("rot_dims", _ct.c_int), ("rot_mag", _ct.c_float), ("eps", _ct.c_float),
        ("positions", _ct.c_void_p), ("seq_of_token", _ct.c_void_p), ("block_table", _ct.c_void_p),
        ("max_pages", _ct.c_int), ("page_size", _ct.c_int), ("num_pages", _ct.c_int),
        ("q_out", _ct.c_void_p), ("ldq", _ct.c_int), ("k_cache", _ct.c_void_p), ("v_cache", _ct.c_void_p),
        ("q_head_stride", _ct.c_int), ("q_skip", _ct.c_int),
        ("rot_half", _ct.c_int), ("q_unit_dims", _ct.c_int), ("k_unit_dims", _ct.c_int),
    ]


def head_prep(proj: torch.Tensor, ctx, block_table: torch.Tensor, page_size: int, *,
              q_off: int, num_heads: int, q_dim: int, q_norm_w, q_norm_dims: int, q_rot_off: int,
              k_off: int, num_kv_heads: int, k_dim: int, k_norm_w, k_norm_dims: int, k_rot_off: int,
              v_off: int, v_dim: int, freq, rot_dims: int, rot_mag: float, eps: float,
              q_out: torch.Tensor, k_cache, v_cache, lam=None, v_first=None, v_keep=None,
              q_head_stride: Optional[int] = None, q_skip: int = 0, rot_half: bool = False,
              q_unit_dims: int = 0, k_unit_dims: int = 0) -> None:
    """One launch between a mixer's first product and its attention: RMS norm of the first
    ``*_norm_dims`` elements of every query / key head (weight shared by the heads; 0: none),
    rotation of ``rot_dims`` elements from ``*_rot_off`` on (neighbouring pairs, or with
    ``rot_half`` element i with element i + rot_dims / 2; ``freq`` float32
    [rot_dims / 2]; cos and sin times ``rot_mag``), then the first ``*_unit_dims`` elements divided
    by their root mean square (0: not), queries into ``q_out``, keys into the pages;
    (head h at ``q_out[t, h * q_head_stride:]``, without its first ``q_skip`` elements);
    values (``v_off`` < 0: none) mixed with ``v_first`` by ``lam`` (a float32 scalar on the
    device) or copied to ``v_keep``, and into the pages.  A cache that is None is not written."""
    a = _HeadPrepArgs()
    a.proj, a.ld = proj.data_ptr(), proj.stride(0)
    a.q_off, a.H, a.Dq, a.q_norm_dims, a.q_rot_off, a.q_norm_w = (q_off, num_heads, q_dim, q_norm_dims,
                                                                  q_rot_off, _p(q_norm_w))
    a.k_off, a.G, a.Dk, a.k_norm_dims, a.k_rot_off, a.k_norm_w = (k_off, num_kv_heads, k_dim, k_norm_dims,
                                                                  k_rot_off, _p(k_norm_w))
    a.v_off, a.Dv = v_off, (v_dim if v_off >= 0 else 0)
    a.lam, a.v_first = _p(lam), _p(v_first)
    a.ld_vf = v_first.stride(0) if v_first is not None else 0
    a.v_keep = _p(v_keep)
    a.ld_vk = v_keep.stride(0) if v_keep is not None else 0
    a.freq, a.rot_dims, a.rot_mag, a.eps = _p(freq), rot_dims, float(rot_mag), float(eps)
    a.positions, a.seq_of_token = ctx.positions.data_ptr(), ctx.seq_of_token.data_ptr()
    a.block_table, a.max_pages, a.page_size = block_table.data_ptr(), block_table.shape[1], page_size
    cache = k_cache if k_cache is not None else v_cache
    a.num_pages = cache.shape[0] if cache is not None else 0
    a.q_out, a.ldq = q_out.data_ptr(), q_out.stride(0)
    a.k_cache, a.v_cache = _p(k_cache), _p(v_cache)
    a.q_head_stride, a.q_skip = (q_dim if q_head_stride is None else q_head_stride), q_skip
    a.rot_half, a.q_unit_dims, a.k_unit_dims = int(bool(rot_half)), int(q_unit_dims), int(k_unit_dims)
    fn = getattr(L.core(), "slb_head_prep_" + _suffix(proj.dtype))
    L.check(fn(_ct.byref(a), proj.shape[0], _stream()), "head_prep")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, group: int = 1) -> None:
    """out = x * sigmoid(gate) ([T, N] views with any row stride); ``group``: neighbouring elements
    that share a gate value (1: element by element; a head's size: one number a head)."""
    fn = getattr(L.core(), "slb_sigmoid_gate_" + _suffix(x.dtype))
    L.check(fn(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), out.data_ptr(), out.stride(0),
               x.shape[0], x.shape[1], int(group), _stream()), "sigmoid_gate")


def head_prep_status(reset: bool = False) -> int:
    return L.core().slb_head_prep_status(1 if reset else 0)


# ------------------------------------ attention with keys and values of two sizes
def attention_kv_tile_rows() -> int:
    return L.core().slb_attention_kv_tile_rows()


def attention_kv_status(reset: bool = False) -> int:
    return L.core().slb_attention_kv_status(1 if reset else 0)


def attention_kv(ctx, q, k_cache, v_cache, v_row_stride: int, out, block_table, num_heads: int,
                 num_kv_heads: int, k_dim: int, v_dim: int, page_size: int, scale: float, window: int,
                 head_gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                 sink: Optional[torch.Tensor] = None) -> None:
    """The plain kernel: float32 arithmetic; keys of ``k_dim``, values of ``v_dim`` elements at
    ``v_cache`` with rows ``v_row_stride`` apart (the key cache itself for values that are a
    prefix of the keys); ``head_gate`` [T, >= H]: head h's row times sigmoid(head_gate[t, h]);
    ``softcap`` > 0: a scaled score s becomes softcap tanh(s / softcap); ``sink`` float32 [H]: its
    exponential joins the softmax's denominator."""
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads, attention_kv_tile_rows())
    fn = getattr(L.core(), "slb_attention_kv_" + _suffix(q.dtype))
    L.check(fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), v_row_stride,
               out.data_ptr(), out.stride(0), block_table.data_ptr(), block_table.shape[1],
               ctx.cu_q.data_ptr(), ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n,
               num_heads, num_kv_heads, k_dim, v_dim, page_size, k_cache.shape[0], float(scale),
               int(window), _p(head_gate), head_gate.stride(0) if head_gate is not None else 0,
               float(softcap), _p(sink), _stream()), "attention_kv")


def attention_kv_splits(num_seqs: int, num_kv_heads: int, longest_context: int, window: int,
                        tile_keys: int = 64, max_splits: int = 32, resident: int = 2) -> int:
    """Blocks a request's keys are split over in a step of single tokens.  With ``resident``
    blocks an SM the step takes (waves of blocks) x (key tiles a block): the fewest splits with
    the smallest such product, at least two key tiles a block."""
    seen = min(longest_context, window + tile_keys) if window > 0 else longest_context
    tiles = -(-seen // tile_keys)
    units = max(1, num_seqs * num_kv_heads)
    slots = max(1, _num_sms() * resident)
    best, best_cost = 1, None
    for s in range(1, max(1, min(max_splits, tiles // 2)) + 1):
        cost = -(-units * s // slots) * -(-tiles // s)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


_kv_resident = {}


def attention_kv_resident(lib, k_dim: int, v_dim: int, narrow: bool, group: int) -> int:
    """Blocks of the tensor-core kernel for these sizes that an SM holds at once."""
    key = (k_dim, v_dim, bool(narrow), group <= 8)
    if key not in _kv_resident:
        _kv_resident[key] = int(lib.slb_attention_kv_mma_resident(1 if narrow else 0, group))
    return _kv_resident[key]


def attention_kv_mma(ctx, q, k_cache, v_cache, tied: bool, out, block_table, num_heads: int,
                     num_kv_heads: int, k_dim: int, v_dim: int, page_size: int, scale: float, window: int,
                     head_gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                     sink: Optional[torch.Tensor] = None) -> None:
    """The tensor-core kernel (bfloat16), for prompt portions and single tokens; in a step of
    single tokens the keys of a request are split over several blocks when the requests alone
    would not fill the device.  ``softcap`` and ``sink`` as in ``attention_kv``."""
    lib = L.attention_kv(k_dim, v_dim)
    rows = lib.slb_attention_kv_mma_tile_rows()
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads, rows)
    splits, part_o, part_ml = 1, None, None
    if ctx.decode_only and attention_kv_split and num_heads // num_kv_heads <= rows:
        narrow = attention_kv_narrow and num_heads // num_kv_heads <= 16
        splits = attention_kv_splits(ctx.num_seqs, num_kv_heads, ctx.split_hint_len, window,
                                     max_splits=lib.slb_attention_kv_mma_max_splits(),
                                     resident=attention_kv_resident(lib, k_dim, v_dim, narrow,
                                                                    num_heads // num_kv_heads))
        if splits > 1:
            T = q.shape[0]
            part_o = torch.empty((T, num_heads, splits, v_dim), dtype=_F32, device=q.device)
            part_ml = torch.empty((T, num_heads, splits, 2), dtype=_F32, device=q.device)
    args = (q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), 1 if tied else 0, out.data_ptr(),
            out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(),
            ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads, num_kv_heads,
            page_size, k_cache.shape[0], float(scale), int(window), _p(head_gate),
            head_gate.stride(0) if head_gate is not None else 0, splits, _p(part_o), _p(part_ml),
            1 if ctx.decode_only and attention_kv_narrow and num_heads // num_kv_heads <= 16 else 0)
    if softcap or sink is not None:
        L.check(lib.slb_attention_kv_mma_capped_bf16(*args, float(softcap or 0.0), _p(sink), _stream()),
                "attention_kv_mma")
        return
    L.check(lib.slb_attention_kv_mma_bf16(*args, _stream()), "attention_kv_mma")


attention_kv_split = True      # (off: one block a request and kv head, the twin)
# steps of single tokens with at most 16 query heads a kv head: the block's warps share the rows
# and split the value columns (off: a warp 16 rows, the twin)
attention_kv_narrow = True


# steps of single tokens with several maps a head: the maps become rows of one block (a library
# built for keys of maps x the map's size), which reads a kv head's values once (off: a block a
# map, the twin)
attention_kv_fold = True
ATTENTION_KV_FOLD_MAX_KEY = 320


def attention_kv_folds(group: int, maps: int, k_dim: int, v_dim: int) -> bool:
    """Whether a step of single tokens with ``maps`` maps a head and ``group`` heads a kv head
    runs with the maps as rows of one block."""
    return (attention_kv_fold and maps > 1 and group * maps <= 16 and k_dim % 8 == 0
            and (maps * k_dim) % 16 == 0 and maps * k_dim <= ATTENTION_KV_FOLD_MAX_KEY and v_dim % 16 == 0)


attention_kv_use_tc = True     # steps with prompt portions: the tcgen05 kernel where it takes the sizes


def attention_kv_tc_takes(k_dim: int, v_dim: int, page_size: int, group: int, tied: bool) -> bool:
    return bool(attention_kv_use_tc and L.attention_kv(k_dim, v_dim).slb_attention_kv_tc_supported(
        page_size, group, 1 if tied else 0))


def attention_kv_tc(ctx, q, k_cache, v_cache, tied: bool, out, block_table, num_heads: int,
                    num_kv_heads: int, k_dim: int, v_dim: int, page_size: int, scale: float, window: int,
                    head_gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                    sink: Optional[torch.Tensor] = None) -> None:
    """The tcgen05 kernel (bfloat16; key and value sizes multiples of 64; steps with prompt
    portions): 128 flattened rows a block, accumulators in tensor memory.  ``softcap`` and ``sink``
    as in ``attention_kv``."""
    lib = L.attention_kv(k_dim, v_dim)
    group = num_heads // num_kv_heads
    tile_seq, tile_row0, n = ctx.attention_tiles(group, lib.slb_attention_kv_tc_tile_rows(group))
    args = (q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), 1 if tied else 0, out.data_ptr(),
            out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(),
            ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads, num_kv_heads,
            page_size, k_cache.shape[0], float(scale), int(window), _p(head_gate),
            head_gate.stride(0) if head_gate is not None else 0)
    if softcap or sink is not None:
        L.check(lib.slb_attention_kv_tc_capped_bf16(*args, float(softcap or 0.0), _p(sink), _stream()),
                "attention_kv_tc")
        return
    L.check(lib.slb_attention_kv_tc_bf16(*args, _stream()), "attention_kv_tc")


def attention_kv_tc_maps(ctx, q, k_cache, v_cache, out, block_table, num_heads: int, num_kv_heads: int,
                         maps: int, k_dim: int, v_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """The tcgen05 kernel with ``maps`` attention maps a head (layouts as ``attention_kv_maps``): a
    block takes 128 flattened rows of one map of a kv head; float32 results per map."""
    lib = L.attention_kv(k_dim, v_dim)
    group = num_heads // num_kv_heads
    tile_seq, tile_row0, n = ctx.attention_tiles(group, lib.slb_attention_kv_tc_tile_rows(group))
    L.check(lib.slb_attention_kv_tc_maps_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), out.stride(0),
        block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_len.data_ptr(),
        tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads, num_kv_heads, maps, page_size,
        k_cache.shape[0], float(scale), int(window), _stream()), "attention_kv_tc")


def attention_kv_tc_status(k_dim: int, v_dim: int, reset: bool = False) -> int:
    """0, or the code of the first bounded wait of the tcgen05 kernel that gave up."""
    return L.attention_kv(k_dim, v_dim).slb_attention_kv_tc_status(1 if reset else 0)


def attention_kv_mma_status(k_dim: int, v_dim: int, reset: bool = False) -> int:
    return L.attention_kv(k_dim, v_dim).slb_attention_kv_mma_status(1 if reset else 0)


# ----------------------------------------------------- per-head batches of products
def gemm_simt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, b, :] = a[:, b, :] . w[b]^T for a [M, B, K], w [B, N, K], out [M, B, N] (views with
    any row stride; the last dimension contiguous), on CUDA cores with float32 accumulation."""
    M, B, Kd = a.shape
    N = w.shape[1]
    fn = getattr(L.core(), "slb_gemm_simt_batched_" + _suffix(a.dtype))
    L.check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(1), out.data_ptr(), out.stride(0),
               M, N, Kd, B, a.stride(1), w.stride(0), out.stride(1), _stream()), "gemm_simt_batched")


router_vendor_min_tokens = 512


def router_logits(x: torch.Tensor, w_f32: torch.Tensor) -> torch.Tensor:
    """float32 logits x . w^T of a float32 router matrix (activations float32 or bfloat16); a
    token's sums run in a fixed order."""
    M, Kd = x.shape
    if x.dtype == _BF16 and M >= router_vendor_min_tokens:
        # a large step in the bfloat16 path: the vendor's float32 product (no reduced-precision
        # mode: torch's default for float32 products) on the widened rows
        from .profile import mark
        out = torch.mm(x.float(), w_f32.t())
        mark("library gemm")
        return out
    out = torch.empty((M, w_f32.shape[0]), dtype=_F32, device=x.device)
    fn = getattr(L.core(), "slb_router_logits_" + _suffix(x.dtype))
    L.check(fn(x.data_ptr(), x.stride(0), w_f32.data_ptr(), w_f32.stride(0), out.data_ptr(), out.stride(0),
               M, w_f32.shape[0], Kd, _stream()), "router_logits")
    return out


# ------------------------------------------------------------- routed experts
def moe_route(logits: torch.Tensor, groups: int, keep: int, top: int, route_scale: float,
              renormalize: bool):
    """(ids int32 [T, top], weights float32 [T, top]) of the softmax router with group-limited
    choice."""
    T, E = logits.shape
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=_F32, device=logits.device)
    L.check(L.core().slb_moe_route(logits.data_ptr(), logits.stride(0), T, E, groups, keep, top,
                                   float(route_scale), 1 if renormalize else 0, ids.data_ptr(),
                                   weights.data_ptr(), _stream()), "moe_route")
    return ids, weights


moe_vendor_grouped = True      # bfloat16 steps of many rows: the vendor's grouped product (off: this package's)
moe_vendor_min_pairs = 1024    # (token, choice) pairs from which it is taken ...
moe_vendor_min_expert_elements = 1 << 21   # ... for experts of at least this many elements a matrix (measured:
                                           # width 2,048 x 1,408: 2.8 -> 1.1 ms a 2,048-token step of 4 layers;
                                           # 1,024 x 512: 0.40 -> 0.62 ms with the copies around it)
moe_tensor_cores = True        # bfloat16: the experts' products on mma.sync (off: CUDA cores, the twin)


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, shared: Optional[torch.Tensor]) -> torch.Tensor:
    """sum_k weights[t, k] * down_e(silu(gate_e x_t) * up_e x_t) (+ shared[t]), e = ids[t, k];
    ``w_gate_up`` [E, 2 I, h] (gate rows, then up rows), ``w_down`` [E, h, I]."""
    T, top = ids.shape
    E, two_i, h = w_gate_up.shape
    inter = two_i // 2
    n_out = w_down.shape[1]
    P = T * top
    lib = L.core()
    plan = torch.empty(lib.slb_moe_plan_ints(P, E), dtype=torch.int32, device=x.device)
    L.check(lib.slb_moe_plan(ids.data_ptr(), P, E, plan.data_ptr(), _stream()), "moe_plan")
    if (x.dtype == _BF16 and moe_vendor_grouped and P >= moe_vendor_min_pairs
            and h * inter >= moe_vendor_min_expert_elements and h % 8 == 0
            and inter % 8 == 0 and n_out % 8 == 0 and hasattr(torch, "_grouped_mm")):
        # Large steps: the vendor's grouped product over the rows sorted by expert (the plan's list
        # and offsets stay on the device), as the dense products of large steps go to the vendor's
        # GEMM; gathering and scattering rows are copies.
        from .profile import mark
        nt = (plan.numel() - 4 * E - 1 - P) // 2
        ends = plan[E + 1:2 * E + 1]                                   # cumulative row counts
        order = plan[3 * E + 1 + 2 * nt:3 * E + 1 + 2 * nt + P]        # pairs sorted by expert
        xs = x.index_select(0, torch.div(order, top, rounding_mode="floor"))
        gu = torch._grouped_mm(xs, w_gate_up.transpose(1, 2), offs=ends)
        mark("library grouped gemm")
        act = torch.empty((P, inter), dtype=x.dtype, device=x.device)
        swiglu(gu, act, 0)
        ys = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends)
        mark("library grouped gemm")
        y = torch.empty_like(ys)
        y.index_copy_(0, order.long(), ys)
        out = torch.empty((T, n_out), dtype=x.dtype, device=x.device)
        L.check(lib.slb_moe_combine_bf16_rows(
            y.data_ptr(), y.stride(0), weights.data_ptr(), _p(shared),
            shared.stride(0) if shared is not None else 0, out.data_ptr(), out.stride(0), T, top, n_out,
            _stream()), "moe_combine")
        return out
    act = torch.empty((P, inter), dtype=x.dtype, device=x.device)
    sfx = _suffix(x.dtype)
    # bfloat16 with rows of whole 16-byte chunks: the tensor-core products; else CUDA cores
    mma = (x.dtype == _BF16 and moe_tensor_cores and h % 8 == 0 and inter % 8 == 0 and n_out % 2 == 0
           and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)
    up_sfx = "mma_bf16" if mma else sfx
    L.check(getattr(lib, "slb_moe_gate_up_" + up_sfx)(
        x.data_ptr(), x.stride(0), w_gate_up.data_ptr(), w_gate_up.stride(1), act.data_ptr(), act.stride(0),
        plan.data_ptr(), E, P, top, inter, h, _stream()), "moe_gate_up")
    y = torch.empty((P, n_out), dtype=_F32, device=x.device)
    L.check(getattr(lib, "slb_moe_down_" + up_sfx)(
        act.data_ptr(), act.stride(0), w_down.data_ptr(), w_down.stride(1), y.data_ptr(), y.stride(0),
        plan.data_ptr(), E, P, top, n_out, inter, _stream()), "moe_down")
    out = torch.empty((T, n_out), dtype=x.dtype, device=x.device)
    L.check(getattr(lib, "slb_moe_combine_" + sfx)(
        y.data_ptr(), y.stride(0), weights.data_ptr(), _p(shared),
        shared.stride(0) if shared is not None else 0, out.data_ptr(), out.stride(0), T, top, n_out,
        _stream()), "moe_combine")
    return out


def moe_route_scored(logits: torch.Tensor, groups: int, keep: int, top: int, route_scale: float,
                     renormalize: bool, score_fn: str = "softmax", correction: Optional[torch.Tensor] = None,
                     group_best: int = 1, norm_eps: float = 0.0):
    """(ids int32 [T, top], weights float32 [T, top]) with every choice of the route kernel as an
    argument: ``score_fn`` "softmax" or "sigmoid"; ``correction`` float32 [E], added to the scores
    for the choice only; a group scores as the sum of its ``group_best`` largest choice scores;
    ``norm_eps`` in the denominator of the renormalised weights."""
    T, E = logits.shape
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=_F32, device=logits.device)
    fn_code = {"softmax": 0, "sigmoid": 1}[score_fn]
    L.check(L.core().slb_moe_route_scored(
        logits.data_ptr(), logits.stride(0), T, E, groups, keep, top, float(route_scale),
        1 if renormalize else 0, fn_code, _p(correction), int(group_best), float(norm_eps),
        ids.data_ptr(), weights.data_ptr(), _stream()), "moe_route")
    return ids, weights


GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0, activation: str = "silu",
              limit: Optional[float] = None, alpha: float = 1.0) -> None:
    """out[t, i] = act(gate_i) * up_i (layout as ``swiglu``); ``activation`` "silu", "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) or "swish_clamped": with g = min(gate, limit)
    and u = clamp(up, -limit, limit), out = g sigmoid(alpha g) (u + 1)."""
    if activation == "swish_clamped":
        fn = getattr(L.core(), "slb_gated_act_clamped_" + _suffix(out.dtype))
        L.check(fn(gate_up.data_ptr(), out.data_ptr(), out.shape[0], out.shape[1], gate_up.stride(0),
                   out.stride(0), int(block), float(limit), float(alpha), _stream()), "gated_act")
        return
    fn = getattr(L.core(), "slb_gated_act_" + _suffix(out.dtype))
    L.check(fn(gate_up.data_ptr(), out.data_ptr(), out.shape[0], out.shape[1], gate_up.stride(0),
               out.stride(0), int(block), GATED_ACTIVATIONS[activation], _stream()), "gated_act")


# ------------------------------------------- several residual streams, embedding norm
def hyper_max_streams() -> int:
    return L.core().slb_hyper_max_streams()


def embed_norm_streams(ids: torch.Tensor, table: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                       out: torch.Tensor) -> None:
    """out[t, s] = rmsnorm(table[ids[t]]) * weight for every stream s (weight None: the embedding
    itself); out float32 [T, n, h] or [T, h]."""
    n = out.shape[1] if out.dim() == 3 else 1
    fn = getattr(L.core(), "slb_embed_norm_streams_" + _suffix(table.dtype))
    L.check(fn(ids.data_ptr(), table.data_ptr(), _p(weight), float(eps), out.data_ptr(), ids.numel(), n,
               table.shape[1], table.shape[0], _stream()), "embed_norm_streams")


def hyper_mix_norm(streams: torch.Tensor, update: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                   out_w: Optional[torch.Tensor], read_w: Optional[torch.Tensor],
                   norm_w: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor],
                   row_map: Optional[torch.Tensor] = None) -> None:
    """``streams`` float32 [T, n, w]: with ``update`` [T, w], X_t <- sum_s mix[s, t] X_s + out_w[t] update
    (in place; not written when ``row_map`` selects rows); then out[r] = rmsnorm(sum_s read_w[s] X_s)
    * norm_w (``read_w`` None: the plain sum; ``norm_w`` None: no norm)."""
    T, n, w = streams.shape
    rows = T if row_map is None else row_map.numel()
    dt = out.dtype if out is not None else update.dtype
    fn = getattr(L.core(), "slb_hyper_mix_norm_" + _suffix(dt))
    L.check(fn(streams.data_ptr(), _p(update), update.stride(0) if update is not None else 0, _p(mix),
               _p(out_w), _p(read_w), _p(norm_w), float(eps), _p(out),
               out.stride(0) if out is not None else 0, _p(row_map), rows, n, w, _stream()), "hyper_mix_norm")


def rms_norm_rows(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out: torch.Tensor) -> None:
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight over the columns of ``x`` [T, n] (a view with any
    row stride: a latent inside a wider projection); float32 arithmetic."""
    fn = getattr(L.core(), "slb_rms_norm_rows_" + _suffix(x.dtype))
    L.check(fn(x.data_ptr(), x.stride(0), _p(weight), float(eps), out.data_ptr(), out.stride(0), x.shape[0],
               x.shape[1], _stream()), "rms_norm_rows")


def norm_sum2(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, factor: float,
              out: torch.Tensor) -> None:
    """out = factor (rmsnorm(a) wa + rmsnorm(b) wb) row by row; a, b float32 [T, n]."""
    if a.dtype != _F32 or b.dtype != _F32:
        raise L.KernelError("norm_sum2 takes float32 branches")
    fn = getattr(L.core(), "slb_norm_sum2_" + _suffix(out.dtype))
    L.check(fn(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), wa.data_ptr(), wb.data_ptr(), float(eps),
               float(factor), out.data_ptr(), out.stride(0), a.shape[0], a.shape[1], _stream()), "norm_sum2")


GATE_ACTIVATIONS = {None: 0, "sigmoid": 1, "silu": 2}


def group_norm_gate(x: torch.Tensor, groups: int, size: int, out: torch.Tensor, *, eps: float,
                    weight: Optional[torch.Tensor] = None, factor: float = 1.0,
                    gate: Optional[torch.Tensor] = None, gate_activation: Optional[str] = None,
                    maps: int = 1, lam: Optional[torch.Tensor] = None) -> None:
    """out[t, g, :] = y / sqrt(mean(y^2) + eps) * weight * factor * act(gate) over ``groups`` groups of
    ``size`` elements; y = x (float32 [T, groups * size]) or, with ``maps`` 2, x[t, g, 0] - lam *
    x[t, g, 1] of x [T, groups, 2, size] (``lam`` a float32 scalar on the device)."""
    fn = getattr(L.core(), "slb_group_norm_gate_" + _suffix(out.dtype))
    L.check(fn(x.data_ptr(), x.stride(0), maps, _p(lam), _p(weight), float(eps), float(factor), _p(gate),
               gate.stride(0) if gate is not None else 0, GATE_ACTIVATIONS[gate_activation if gate is not None else None],
               out.data_ptr(), out.stride(0), x.shape[0], groups, size, _stream()), "group_norm_gate")


# ----------------------------------------------- linear attention with a decay
class _DecayAttnArgs(_ct.Structure):
    _fields_ = [
        ("proj", _ct.c_void_p), ("ld", _ct.c_int),
        ("q_off", _ct.c_int), ("k_off", _ct.c_int), ("v_off", _ct.c_int),
        ("H", _ct.c_int), ("D", _ct.c_int), ("Dv", _ct.c_int), ("act", _ct.c_int),
        ("freq", _ct.c_void_p), ("rot_dims", _ct.c_int), ("k_scale", _ct.c_float),
        ("decay", _ct.c_void_p),
        ("positions", _ct.c_void_p), ("cu_q", _ct.c_void_p), ("state_slots", _ct.c_void_p),
        ("state", _ct.c_void_p), ("num_slots", _ct.c_int),
        ("out", _ct.c_void_p), ("ldo", _ct.c_int),
        ("gate_z", _ct.c_void_p), ("ld_gate", _ct.c_int), ("gate_bias", _ct.c_void_p),
        ("gate_inv_tau", _ct.c_float), ("q_scale", _ct.c_float), ("state_stride", _ct.c_longlong),
    ]


class _DecayChunkArgs(_ct.Structure):
    _fields_ = [("a", _DecayAttnArgs), ("tile_seq", _ct.c_void_p), ("tile_row0", _ct.c_void_p),
                ("num_tiles", _ct.c_int), ("work", _ct.c_void_p)]


class _GatedChunkArgs(_ct.Structure):
    _fields_ = [("a", _DecayAttnArgs), ("tile_seq", _ct.c_void_p), ("tile_row0", _ct.c_void_p),
                ("num_tiles", _ct.c_int), ("work", _ct.c_void_p), ("qdec", _ct.c_void_p), ("kdec", _ct.c_void_p),
                ("dtot", _ct.c_void_p), ("scores", _ct.c_void_p)]


# Learned decays: steps that bring portions of prompts in bfloat16 take the chunked kernels (float32
# arithmetic on the CUDA cores, chunks of 32 tokens) from the same number of tokens a request on.
decay_gated_chunked = True
force_gated_chunks = False       # (tests: the chunked kernels also for float32 rows)


# Steps that bring portions of prompts in bfloat16 take the chunked tensor-core kernels when the
# step has at least this many tokens a request (shorter portions: the recurrent kernel, which is
# also the float32 path and the one for steps of single tokens).
decay_attention_chunked = True
decay_attention_chunk_min_tokens = 16
# operands of the chunked kernels' products as two bfloat16 numbers each (three MMAs a product)
decay_attention_split = True


def decay_attention_max_dim() -> int:
    return L.core().slb_decay_attention_max_dim()


def decay_attention(proj: torch.Tensor, ctx, state: torch.Tensor, decay: Optional[torch.Tensor], out: torch.Tensor, *,
                    q_off: int, k_off: int, v_off: int, num_heads: int, head_dim: int, value_dim: int,
                    activation: Optional[str] = None, freq: Optional[torch.Tensor] = None, rot_dims: int = 0,
                    key_scale: float = 1.0, query_scale: float = 1.0, gate_z: Optional[torch.Tensor] = None,
                    gate_bias: Optional[torch.Tensor] = None, gate_tau: float = 1.0) -> None:
    """o_t = S_t^T q_t with S_t = decay_h S_{t-1} + k_t v_t^T per head over the tokens of every request
    of the step, in order; q, k, v are columns of ``proj`` [T, ...]; ``state`` float32
    [slots, H, D, Dv] (or [slots, >= H * D * Dv]: a slice of a larger record) is read at
    ``ctx.state_slots`` and left advanced; ``out`` float32 [T, H * Dv].  With ``gate_z`` (float32
    [T, H * D]; ``decay`` None) every key channel of every token has its own decay
    sigmoid(gate_z + gate_bias)^(1 / gate_tau): S_t = diag(alpha_t) S_{t-1} + k_t v_t^T."""
    a = _DecayAttnArgs()
    a.proj, a.ld = proj.data_ptr(), proj.stride(0)
    a.q_off, a.k_off, a.v_off = q_off, k_off, v_off
    a.H, a.D, a.Dv = num_heads, head_dim, value_dim
    a.act = {None: 0, "silu": 1}[activation]
    a.freq, a.rot_dims, a.k_scale = _p(freq), rot_dims, float(key_scale)
    a.decay = _p(decay)
    a.positions, a.cu_q, a.state_slots = ctx.positions.data_ptr(), ctx.cu_q.data_ptr(), ctx.state_slots.data_ptr()
    a.state, a.num_slots = state.data_ptr(), state.shape[0]
    a.out, a.ldo = out.data_ptr(), out.stride(0)
    a.gate_z, a.ld_gate = _p(gate_z), (gate_z.stride(0) if gate_z is not None else 0)
    a.gate_bias, a.gate_inv_tau, a.q_scale = _p(gate_bias), 1.0 / float(gate_tau), float(query_scale)
    a.state_stride = state.stride(0)
    if gate_z is not None and gate_z.dtype != _F32:
        raise L.KernelError("decay_attention: the decays' logits must be float32")
    plain = (gate_z is None and query_scale == 1.0
             and state.stride(0) == num_heads * head_dim * value_dim)
    if (gate_z is not None and not ctx.decode_only and head_dim <= L.core().slb_decay_gated_chunk_max_dim()
            and ctx.num_tokens >= decay_attention_chunk_min_tokens * ctx.num_seqs
            and (force_gated_chunks or (decay_gated_chunked and proj.dtype == torch.bfloat16))):
        chunk = L.core().slb_decay_gated_chunk_tokens()
        tile_seq, tile_row0, n = ctx.attention_tiles(1, chunk)
        c = _GatedChunkArgs()
        c.a = a
        c.tile_seq, c.tile_row0, c.num_tiles = tile_seq.data_ptr(), tile_row0.data_ptr(), n
        dev = proj.device
        work = torch.empty((max(n, 1), num_heads, head_dim, value_dim), dtype=_F32, device=dev)
        qk_dec = torch.empty((2, proj.shape[0], num_heads * head_dim), dtype=_F32, device=dev)
        dtot = torch.empty((max(n, 1), num_heads, head_dim), dtype=_F32, device=dev)
        scores = torch.empty((max(n, 1), num_heads, chunk, chunk), dtype=_F32, device=dev)
        c.work, c.dtot, c.scores = work.data_ptr(), dtot.data_ptr(), scores.data_ptr()
        c.qdec, c.kdec = qk_dec[0].data_ptr(), qk_dec[1].data_ptr()
        fn = getattr(L.core(), "slb_decay_gated_chunk_" + _suffix(proj.dtype))
        L.check(fn(_ct.byref(c), ctx.num_seqs, _stream()), "decay_attention (gated chunks)")
        global launch_count
        launch_count += 3
        return
    if (decay_attention_chunked and plain and proj.dtype == torch.bfloat16 and not ctx.decode_only
            and head_dim <= L.core().slb_decay_chunk_max_dim()
            and ctx.num_tokens >= decay_attention_chunk_min_tokens * ctx.num_seqs):
        # portions of prompts: the chunked form on the tensor cores
        tile_seq, tile_row0, n = ctx.attention_tiles(1, L.core().slb_decay_chunk_tokens())
        c = _DecayChunkArgs()
        c.a = a
        c.tile_seq, c.tile_row0, c.num_tiles = tile_seq.data_ptr(), tile_row0.data_ptr(), n
        work = torch.empty((max(n, 1), num_heads, head_dim, value_dim), dtype=torch.float32, device=proj.device)
        c.work = work.data_ptr()
        L.check(L.core().slb_decay_chunk_bf16(_ct.byref(c), ctx.num_seqs, int(decay_attention_split), _stream()),
                "decay_attention (chunked)")
        return
    fn = getattr(L.core(), "slb_decay_attention_" + _suffix(proj.dtype))
    L.check(fn(_ct.byref(a), ctx.num_seqs, _stream()), "decay_attention")


def attention_kv_maps(ctx, q, k_cache, v_cache, out, block_table, num_heads: int, num_kv_heads: int,
                      maps: int, k_dim: int, v_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """The plain kernel with ``maps`` attention maps a head: q [T, H, maps, k_dim], cached key rows
    [maps, k_dim] per kv head, one set of values per kv head; ``out`` float32 [T, H, maps, v_dim]."""
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads, attention_kv_tile_rows())
    fn = getattr(L.core(), "slb_attention_kv_maps_" + _suffix(q.dtype))
    L.check(fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), maps * k_dim, maps, v_cache.data_ptr(), v_dim,
               out.data_ptr(), out.stride(0), block_table.data_ptr(), block_table.shape[1],
               ctx.cu_q.data_ptr(), ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n,
               num_heads, num_kv_heads, k_dim, v_dim, page_size, k_cache.shape[0], float(scale), int(window),
               _stream()), "attention_kv_maps")


def attention_kv_mma_maps(ctx, q, k_cache, v_cache, out, block_table, num_heads: int, num_kv_heads: int,
                          maps: int, k_dim: int, v_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """The tensor-core kernel (bfloat16) with ``maps`` attention maps a head, layouts as
    ``attention_kv_maps``; in a step of single tokens the keys of a request are split over several
    blocks when the requests alone would not fill the device."""
    if ctx.decode_only and attention_kv_folds(num_heads // num_kv_heads, maps, k_dim, v_dim):
        # a step of single tokens: the maps are rows of one block, which reads the values once
        lib = L.attention_kv(maps * k_dim, v_dim)
        group = num_heads // num_kv_heads * maps
        tile_seq, tile_row0, n = ctx.attention_tiles(group, lib.slb_attention_kv_mma_tile_rows())
        splits, part_o, part_ml = 1, None, None
        if attention_kv_split:
            splits = attention_kv_splits(ctx.num_seqs, num_kv_heads, ctx.split_hint_len, window,
                                         max_splits=lib.slb_attention_kv_mma_max_splits(),
                                         resident=attention_kv_resident(lib, maps * k_dim, v_dim,
                                                                        attention_kv_narrow, group))
            if splits > 1:
                T = q.shape[0]
                part_o = torch.empty((T, num_heads * maps, splits, v_dim), dtype=_F32, device=q.device)
                part_ml = torch.empty((T, num_heads * maps, splits, 2), dtype=_F32, device=q.device)
        L.check(lib.slb_attention_kv_mma_folded_bf16(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), maps, out.data_ptr(), out.stride(0),
            block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_len.data_ptr(),
            tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads, num_kv_heads, page_size, k_cache.shape[0],
            float(scale), int(window), splits, _p(part_o), _p(part_ml), 1 if attention_kv_narrow else 0,
            _stream()), "attention_kv_mma")
        return
    lib = L.attention_kv(k_dim, v_dim)
    rows = lib.slb_attention_kv_mma_tile_rows()
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads, rows)
    splits, part_o, part_ml = 1, None, None
    if ctx.decode_only and attention_kv_split and num_heads // num_kv_heads <= rows:
        splits = attention_kv_splits(ctx.num_seqs, num_kv_heads * maps, ctx.split_hint_len, window,
                                     max_splits=lib.slb_attention_kv_mma_max_splits(),
                                     resident=attention_kv_resident(
                                         lib, k_dim, v_dim, attention_kv_narrow and num_heads // num_kv_heads <= 16,
                                         num_heads // num_kv_heads))
        if splits > 1:
            T = q.shape[0]
            part_o = torch.empty((T, num_heads * maps, splits, v_dim), dtype=_F32, device=q.device)
            part_ml = torch.empty((T, num_heads * maps, splits, 2), dtype=_F32, device=q.device)
    L.check(lib.slb_attention_kv_mma_maps_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), maps, out.data_ptr(), out.stride(0),
        block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_len.data_ptr(),
        tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads, num_kv_heads, page_size, k_cache.shape[0],
        float(scale), int(window), splits, _p(part_o), _p(part_ml),
        1 if ctx.decode_only and attention_kv_narrow and num_heads // num_kv_heads <= 16 else 0, _stream()),
        "attention_kv_mma")

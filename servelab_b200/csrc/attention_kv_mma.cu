// Tensor-core paged attention (bf16, mma.sync m16n8k16, float32 softmax and accumulation) for
// mixers whose keys and values differ in size, compiled for one pair of sizes (SLB_KEY_DIM,
// SLB_VALUE_DIM: multiples of 16, at most 320 and 256).  It serves prompt portions and single
// tokens alike, and the absorbed form of a latent attention: with `tied` the values are the
// first SLB_VALUE_DIM elements of the cached key rows, so a tile is fetched once and read by
// both products.
//
// Work unit: (tile of 64 flattened query rows rho = local_token * g + head_in_group, kv head);
// a warp owns 16 rows.  Keys are visited in tiles of 64 aligned to absolute positions through a
// two-stage cp.async ring; Q fragments are re-read from shared memory k-step by k-step, so large
// key sizes cost no registers; scores and the online softmax live in registers in the base-2
// domain; P is rounded to bf16 as the operand of P.V.  Optional epilogue: head h's row times
// sigmoid(gate[token][h]).
//
// Steps of few single tokens split every request's keys over `splits` blocks (grid y): a block
// leaves its unnormalised rows with their running maxima and sums in scratch, and a second small
// kernel combines them (and applies the gate).
//
// In a step of single tokens a tile holds the g query heads of one request that share the kv
// head (all heads of a latent attention): the rows of the MMA are heads.  When they are at most
// 16 (`narrow`), the four warps share them: each forms the tile's scores and softmax weights (the
// same numbers in every warp) and multiplies them with its quarter of the value columns, so the
// long product of a tile is spread over the warps; the Q tile takes 16 rows of shared memory, so
// that two blocks fit an SM at the largest sizes.
//
// Several attention maps a head (`maps`; not with `tied`): every query head and every kv head
// carries `maps` query / key vectors side by side ([head][map][DK]; a cached key row is
// [map][DK]), each map is an attention of its own over the kv head's one set of values, and a
// block owns (tile, kv head, map).  The results go out map by map, [token][head][map][DV], as
// float32 when `out_f32` is given, for the kernel that combines the maps.
//
// Maps folded into the rows (`fold` maps, a library built for SLB_KEY_DIM = fold * the map's key
// size): a (head, map) is a row of its own, and its query stands in the map's columns of an
// otherwise zero row of SLB_KEY_DIM, so that the product with the whole cached key row
// [map][key size] is that map's score.  One block then serves all maps of a kv head and reads
// the values once; in a step of single tokens (memory-bound) that is the point.
#include "mma_util.cuh"

#ifndef SLB_KEY_DIM
#error "compile with -DSLB_KEY_DIM=<key size> -DSLB_VALUE_DIM=<value size>"
#endif

SLB_DEFINE_PDL_SWITCH

namespace {

constexpr int DK = SLB_KEY_DIM, DV = SLB_VALUE_DIM;
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK >= 16 && DV >= 16 && DK <= 320 && DV <= 256,
              "key and value sizes must be multiples of 16, at most 320 and 256");
constexpr int LDK = DK + 8, LDV = DV + 8;      // shared-memory row strides (16-byte pad)
// (keys per tile: 32 for large keys, so that two blocks fit an SM's shared memory)
constexpr int BM = 64, BN = SLB_KEY_DIM > 192 ? 32 : 64, NTHREADS = 128;
constexpr int KCH = DK / 8, VCH = DV / 8;      // 16-byte chunks per row
constexpr int KSTEPS = DK / 16, NT_O = DV / 8, NT_S = BN / 8;
// a stage of the ring: a K tile and, unless the values are part of the key rows, a V tile
__host__ __device__ constexpr int stage_elems(bool tied) { return BN * LDK + (tied ? 0 : BN * LDV); }

using namespace slb_mma;

__device__ int kv_attn_status_word = 0;

__device__ __forceinline__ void load_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ kc,
                                          const bf16* __restrict__ vc, bool tied,
                                          const int* __restrict__ table, int k0, int kend, int kvh,
                                          int Hkv, int ps, int num_pages, int ldk, int koff) {
    // NTHREADS / BN threads a key: its page is looked up once, then its 16-byte chunks are shared out
    constexpr int TPR = NTHREADS / BN;
    static_assert(NTHREADS % BN == 0, "whole threads per key row");
    const int per_row = tied ? KCH : KCH + VCH;
    const int r = threadIdx.x / TPR, sub = threadIdx.x % TPR;
    const int kp = k0 + r;
    bool ok = kp < kend;
    int page = -1;
    if (ok) page = table[kp / ps];
    if (page >= num_pages) {
        atomicCAS(&kv_attn_status_word, 0, 0x40);
        page = -1;
    }
    ok = ok && page >= 0;
    const size_t slot = ok ? ((size_t)page * Hkv + kvh) * ps + kp % ps : 0;
    const bf16* krow = kc + slot * ldk + koff;
    const bf16* vrow = vc + slot * DV;
    for (int c = sub; c < per_row; c += TPR) {
        if (c < KCH) cp_async16(Ks + r * LDK + c * 8, krow + c * 8, ok);
        else cp_async16(Vs + r * LDV + (c - KCH) * 8, vrow + (c - KCH) * 8, ok);
    }
}

// NARROW: at most 16 rows a tile, shared by the warps; a warp then holds only its share of the
// value columns (16-column pairs np with np % 4 == warp), and the Q tile takes `q_rows` = 8 or 16
// rows of shared memory (with 8, the MMA's upper rows re-read the lower ones and are masked).
template <bool NARROW>
__global__ void __launch_bounds__(NTHREADS) attention_kv_mma_kernel(
    const bf16* __restrict__ q, int ldq, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
    int tied, bf16* __restrict__ out, int ldo, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ cu_q, const int* __restrict__ ctx_len, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_row0, int H, int Hkv, int ps, int num_pages, float scale_log2,
    int window, const bf16* __restrict__ gate, int ldg, int splits, float* __restrict__ part_o,
    float* __restrict__ part_ml, int maps, float* __restrict__ out_f32, int q_rows, int fold,
    float softcap, float scale, const float* __restrict__ sink) {
    // softcap > 0: a scaled score s becomes softcap tanh(s / softcap); sink: one number a head whose
    // exponential joins the softmax's denominator (added where the row is finished: here without
    // key splits, in the combine kernel with them)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_wait();
    constexpr int NO = NARROW ? ((NT_O / 2 + 3) / 4) * 2 : NT_O;      // 8-column tiles of O a warp holds
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [q_rows][LDK]
    bf16* stage0 = Qs + q_rows * LDK;                      // 2 x (K tile | V tile)
    const int STAGE_ELEMS = stage_elems(tied != 0);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int units = Hkv * maps;
    const int kvh = (blockIdx.x % units) / maps, map = (blockIdx.x % units) % maps;
    const int ldk = maps * DK, koff = map * DK;
    const int tile = (int)(gridDim.x / units) - 1 - (int)(blockIdx.x / units);   // the longest first
    const int s = tile_seq[tile];
    const int row0 = tile_row0[tile];
    const int g = H / Hkv;
    const int q0 = cu_q[s];
    const int qlen = cu_q[s + 1] - q0;
    const int ctx = ctx_len[s];
    const int nrows = min(q_rows, qlen * g - row0);
    if (nrows <= 0) return;
    const int pos_base = ctx - qlen;
    const int* table = block_table + (size_t)s * max_pages;

    for (int idx = tid; idx < q_rows * KCH; idx += NTHREADS) {
        const int r = idx / KCH, c = idx - r * KCH;
        const bool ok = r < nrows;
        const int rho = row0 + (ok ? r : 0);
        const int tl = rho / g, hg = rho - tl * g;
        if (fold > 1) {
            // H counts (head, map) pairs; the pair's query of DK / fold elements goes to its map's columns
            const int dks = DK / fold, pair = kvh * g + hg, at = c * 8 - (pair % fold) * dks;
            const bool mine = ok && at >= 0 && at < dks;
            cp_async16(Qs + r * LDK + c * 8, q + (size_t)(q0 + tl) * ldq + (size_t)pair * dks + (mine ? at : 0), mine);
            continue;
        }
        cp_async16(Qs + r * LDK + c * 8, q + (size_t)(q0 + tl) * ldq + (size_t)((kvh * g + hg) * maps + map) * DK + c * 8, ok);
    }
    cp_async_commit();

    const int p_first = pos_base + row0 / g;
    const int p_last = pos_base + (row0 + nrows - 1) / g;
    int kbeg = 0;
    if (window > 0) kbeg = max(0, p_first - window + 1) / BN * BN;
    const int kend = p_last + 1;
    int ntiles = (kend - kbeg + BN - 1) / BN;
    if (splits > 1) {                                      // this block's share of the key tiles
        const int per = (ntiles + splits - 1) / splits;
        const int first = min(ntiles, (int)blockIdx.y * per);
        ntiles = min(ntiles, first + per) - first;
        kbeg += first * BN;
    }

    if (ntiles > 0)
        load_tile(stage0, stage0 + BN * LDK, kc, vc, tied != 0, table, kbeg, kend, kvh, Hkv, ps, num_pages, ldk, koff);
    cp_async_commit();

    const int wrow = NARROW ? 0 : warp;                    // the warp's 16 rows of the tile
    const int r_lo = wrow * 16 + (lane >> 2), r_hi = r_lo + 8;
    const int pos_lo = r_lo < nrows ? pos_base + (row0 + r_lo) / g : -1;
    const int pos_hi = r_hi < nrows ? pos_base + (row0 + r_hi) / g : -1;
    const int wr_last = min(nrows - 1, wrow * 16 + 15);
    const int warp_pos_max = wrow * 16 < nrows ? pos_base + (row0 + wr_last) / g : -1;
    const int warp_pos_min = pos_base + (row0 + wrow * 16) / g;
    const int tig = lane & 3;

    float o[NO][4];
#pragma unroll
    for (int n = 0; n < NO; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const bf16* Qw = Qs + wrow * 16 * LDK + ((lane & 15) & (q_rows - 1)) * LDK;   // this lane's row of the A tiles

    for (int t = 0; t < ntiles; ++t) {
        bf16* Ks = stage0 + (t & 1) * STAGE_ELEMS;
        const bf16* Vs = tied ? Ks : Ks + BN * LDK;
        const int ldv_s = tied ? LDK : LDV;
        if (t + 1 < ntiles) {
            bf16* Kn = stage0 + ((t + 1) & 1) * STAGE_ELEMS;
            load_tile(Kn, Kn + BN * LDK, kc, vc, tied != 0, table, kbeg + (t + 1) * BN, kend, kvh, Hkv, ps,
                      num_pages, ldk, koff);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int k0 = kbeg + t * BN;
        // (a warp whose rows all lie before the tile, or beyond the window's reach of it, skips it)
        if (k0 <= warp_pos_max && (window <= 0 || warp_pos_min - (k0 + BN - 1) < window)) {
            float sc[NT_S][4];
#pragma unroll
            for (int j = 0; j < NT_S; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
            // (the fragment loads are issued one k-step ahead of the MMAs that use them: the
            // instructions keep their program order, so the order is written out here)
            unsigned af[2][4], bf[2][NT_S / 2][4];
            ldmatrix_x4(af[0], Qw + (lane >> 4) * 8);
#pragma unroll
            for (int jp = 0; jp < NT_S / 2; ++jp)
                ldmatrix_x4(bf[0][jp], Ks + (jp * 16 + (lane >> 4) * 8 + (lane & 7)) * LDK + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                const int cur = kk & 1, nxt = cur ^ 1;
                if (kk + 1 < KSTEPS) {
                    ldmatrix_x4(af[nxt], Qw + (kk + 1) * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int jp = 0; jp < NT_S / 2; ++jp)
                        ldmatrix_x4(bf[nxt][jp], Ks + (jp * 16 + (lane >> 4) * 8 + (lane & 7)) * LDK + (kk + 1) * 16 +
                                                     ((lane >> 3) & 1) * 8);
                }
#pragma unroll
                for (int jp = 0; jp < NT_S / 2; ++jp) {
                    mma_bf16(sc[2 * jp], af[cur], bf[cur][jp][0], bf[cur][jp][1]);
                    mma_bf16(sc[2 * jp + 1], af[cur], bf[cur][jp][2], bf[cur][jp][3]);
                }
            }
            if (softcap > 0.f) {
                // (what follows multiplies by scale * log2 e: the capped score divided by scale)
                const float in = scale / softcap, back = softcap / scale;
#pragma unroll
                for (int j = 0; j < NT_S; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[j][e] = back * tanhf(sc[j][e] * in);
            }
            // mask, online softmax (base-2 domain)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NT_S; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kp = k0 + j * 8 + tig * 2 + (e & 1);
                    const int pos = (e < 2) ? pos_lo : pos_hi;
                    const bool vis = kp < kend && kp <= pos && (window <= 0 || pos - kp < window);
                    if (!vis) sc[j][e] = -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sc[j][e]);
                }
            float alpha[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m[h], mx[h] * scale_log2);
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                alpha[h] = exp2f(m[h] - m_use);
                m[h] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
                    sc[j][2 * h] = exp2f(fmaf(sc[j][2 * h], scale_log2, -m_use));
                    sc[j][2 * h + 1] = exp2f(fmaf(sc[j][2 * h + 1], scale_log2, -m_use));
                    sum += sc[j][2 * h] + sc[j][2 * h + 1];
                }
                l[h] = l[h] * alpha[h] + sum;
            }
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int n = 0; n < NO; ++n) {
                    o[n][0] *= alpha[0];
                    o[n][1] *= alpha[0];
                    o[n][2] *= alpha[1];
                    o[n][3] *= alpha[1];
                }
            }
            // O += P . V
#pragma unroll
            for (int ks = 0; ks < NT_S / 2; ++ks) {
                unsigned a[4];
                a[0] = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
                a[1] = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
                a[2] = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
                a[3] = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
                unsigned vf[2][4];
                if constexpr (NARROW) {                    // this warp's share of the value columns
#pragma unroll
                    for (int i = 0; i < NO / 2; ++i) {
                        const int np = i * 4 + warp;
                        if (np < NT_O / 2) {
                            ldmatrix_x4_trans(vf[i & 1], Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv_s +
                                                             np * 16 + (lane >> 4) * 8);
                            mma_bf16(o[2 * i], a, vf[i & 1][0], vf[i & 1][1]);
                            mma_bf16(o[2 * i + 1], a, vf[i & 1][2], vf[i & 1][3]);
                        }
                    }
                    continue;
                }
                if constexpr (!NARROW) {
                    ldmatrix_x4_trans(vf[0], Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv_s + (lane >> 4) * 8);
#pragma unroll
                    for (int np = 0; np < NT_O / 2; ++np) {
                        const int cur = np & 1, nxt = cur ^ 1;
                        if (np + 1 < NT_O / 2)
                            ldmatrix_x4_trans(vf[nxt], Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv_s +
                                                           (np + 1) * 16 + (lane >> 4) * 8);
                        mma_bf16(o[2 * np], a, vf[cur][0], vf[cur][1]);
                        mma_bf16(o[2 * np + 1], a, vf[cur][2], vf[cur][3]);
                    }
                }
            }
        }
        __syncthreads();
    }

    cp_async_wait<0>();                                    // (a block without key tiles fetched Q all the same)
    pdl_launch_dependents();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = h ? r_hi : r_lo;
        if (row >= nrows) continue;
        const int rho = row0 + row;
        const int tl = rho / g, hg = rho - tl * g;
        const int head = (kvh * g + hg) * maps + map;
        if (splits > 1) {
            const size_t pi = ((size_t)(q0 + tl) * H * maps + head) * splits + blockIdx.y;
            if (tig == 0 && (!NARROW || warp == 0)) {
                part_ml[2 * pi] = m[h];
                part_ml[2 * pi + 1] = l[h];
            }
            float* po = part_o + pi * DV + tig * 2;
#pragma unroll
            for (int i = 0; i < NO; ++i) {
                const int n = NARROW ? ((i >> 1) * 4 + warp) * 2 + (i & 1) : i;     // the tile's place in the row
                if (n < NT_O) *reinterpret_cast<float2*>(po + n * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
            }
            continue;
        }
        if (sink != nullptr)
            l[h] += (m[h] == -INFINITY) ? 1.f : exp2f(sink[head] * 1.4426950408889634f - m[h]);
        float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
        if (gate != nullptr) {
            const float z = __bfloat162float(gate[(size_t)(q0 + tl) * ldg + head]);
            inv *= 1.0f / (1.0f + __expf(-z));
        }
        if (out_f32 != nullptr) {
            float* dst = out_f32 + (size_t)(q0 + tl) * ldo + (size_t)head * DV + tig * 2;
#pragma unroll
            for (int i = 0; i < NO; ++i) {
                const int n = NARROW ? ((i >> 1) * 4 + warp) * 2 + (i & 1) : i;
                if (n < NT_O)
                    *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
            }
            continue;
        }
        bf16* dst = out + (size_t)(q0 + tl) * ldo + (size_t)head * DV + tig * 2;
#pragma unroll
        for (int i = 0; i < NO; ++i) {
            const int n = NARROW ? ((i >> 1) * 4 + warp) * 2 + (i & 1) : i;
            if (n < NT_O) *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        }
    }
}

// out[t][h] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) (times the gate): one block a (token,
// head), a thread two neighbouring columns; the splits' weights are formed once per block.
__global__ void __launch_bounds__(128) attention_kv_combine_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits, bf16* __restrict__ out,
    int ldo, int H, const bf16* __restrict__ gate, int ldg, float* __restrict__ out_f32,
    const float* __restrict__ sink) {
    __shared__ float wgt[32];
    __shared__ float inv_s;
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    const int head = blockIdx.y;
    const size_t base = (t * H + head) * splits;
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        const float ms = s < splits ? part_ml[2 * (base + s)] : -INFINITY;
        const float ls = s < splits ? part_ml[2 * (base + s) + 1] : 0.f;
        const float M = warp_max(ms);
        const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
        float L = warp_sum(ls * w);
        wgt[s] = w;
        if (s == 0) {
            if (sink != nullptr) L += (M == -INFINITY) ? 1.f : exp2f(sink[head] * 1.4426950408889634f - M);
            float inv = L > 0.f ? 1.f / L : 0.f;
            if (gate != nullptr) inv *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[t * ldg + head])));
            inv_s = inv;
        }
    }
    __syncthreads();
    for (int c = threadIdx.x * 2; c < DV; c += blockDim.x * 2) {
        float a0 = 0.f, a1 = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float2 v = *reinterpret_cast<const float2*>(part_o + (base + s) * DV + c);
            a0 += v.x * wgt[s];
            a1 += v.y * wgt[s];
        }
        if (out_f32 != nullptr)
            *reinterpret_cast<float2*>(out_f32 + t * ldo + (size_t)head * DV + c) = make_float2(a0 * inv_s, a1 * inv_s);
        else
            *reinterpret_cast<unsigned*>(out + t * ldo + (size_t)head * DV + c) = pack_bf16(a0 * inv_s, a1 * inv_s);
    }
}

}  // namespace

extern "C" {
int slb_attention_kv_mma_max_splits() { return 32; }
int slb_attention_kv_mma_key_dim() { return DK; }
int slb_attention_kv_mma_value_dim() { return DV; }
int slb_attention_kv_mma_tile_rows() { return BM; }
int slb_attention_kv_mma_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, kv_attn_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(kv_attn_status_word, &zero, sizeof(int));
    }
    return v;
}
// Blocks of the kernel an SM holds at once (separate keys and values), for the choice of splits:
// `group` rows a tile in the narrow form.
int slb_attention_kv_mma_resident(int narrow, int group) {
    const int q_rows = narrow ? (group <= 8 ? 8 : 16) : BM;
    const size_t smem = ((size_t)q_rows * LDK + 2 * stage_elems(false)) * sizeof(bf16);
    static unsigned long long configured = 0, configured_narrow = 0;       // (sizes above 48 KB need the opt-in first)
    const int rc = narrow ? slb_configure(&configured_narrow, attention_kv_mma_kernel<true>,
                                          ((size_t)16 * LDK + 2 * stage_elems(false)) * sizeof(bf16))
                          : slb_configure(&configured, attention_kv_mma_kernel<false>,
                                          ((size_t)BM * LDK + 2 * stage_elems(false)) * sizeof(bf16));
    if (rc != 0) return 1;
    int n = 0;
    const cudaError_t e = narrow
        ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_kv_mma_kernel<true>, NTHREADS, smem)
        : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_kv_mma_kernel<false>, NTHREADS, smem);
    return e == cudaSuccess && n > 0 ? n : 1;
}
static int launch_attention_kv_mma(const bf16* q, int ldq, const bf16* kc, const bf16* vc, int tied, bf16* out,
                                   float* out_f32, int ldo, const int* block_table, int max_pages, const int* cu_q,
                                   const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                                   int H, int Hkv, int maps, int ps, int num_pages, float scale, int window,
                                   const bf16* gate, int ldg, int splits, float* part_o, float* part_ml,
                                   int narrow, int fold, cudaStream_t st, float softcap = 0.f,
                                   const float* sink = nullptr) {
    // `fold` > 1: H counts (head, map) pairs, `maps` is 1, DK is fold times a map's key size.
    // `narrow`: every tile of the list holds at most 16 rows (a step of single tokens with at most
    // 16 query heads a kv head).
    // `splits` > 1 (steps of single tokens only: a tile is one token's heads): scratch part_o
    // [tokens][H * maps][splits][DV] and part_ml [tokens][H * maps][splits][2], float32.
    if (num_tiles <= 0) return 0;
    if (splits < 1 || splits > 32 || (splits > 1 && (part_o == nullptr || part_ml == nullptr || H / Hkv > BM)))
        return SLB_ERR_BAD_ARG;
    if (narrow && H / Hkv > 16) return SLB_ERR_BAD_ARG;
    if (softcap < 0.f || (sink != nullptr && (maps != 1 || fold != 1))) return SLB_ERR_BAD_ARG;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || ps <= 0 || max_pages <= 0 || num_pages <= 0 || scale <= 0.f ||
        (tied && DV > DK) || ldq % 8 != 0 || ldo % 2 != 0 || maps < 1 || (maps > 1 && tied) || fold < 1 ||
        (fold > 1 && (maps != 1 || tied || DK % (8 * fold) != 0 || H % fold != 0)))
        return SLB_ERR_BAD_ARG;
    if ((long long)num_tiles * Hkv * maps > 2147483647LL) return SLB_ERR_TOO_LARGE;
    // (a narrow tile of at most 8 rows keeps 8 rows of Q: a third block fits an SM at the largest sizes)
    const int q_rows = narrow ? (H / Hkv <= 8 ? 8 : 16) : BM;
    const size_t smem = ((size_t)q_rows * LDK + 2 * stage_elems(tied != 0)) * sizeof(bf16);
    static unsigned long long configured = 0, configured_narrow = 0;
    const int rc = narrow ? slb_configure(&configured_narrow, attention_kv_mma_kernel<true>,
                                          ((size_t)16 * LDK + 2 * stage_elems(false)) * sizeof(bf16))
                          : slb_configure(&configured, attention_kv_mma_kernel<false>,
                                          ((size_t)BM * LDK + 2 * stage_elems(false)) * sizeof(bf16));
    if (rc != 0) return rc;
    const int e = slb_launch(narrow ? attention_kv_mma_kernel<true> : attention_kv_mma_kernel<false>,
                             dim3(num_tiles * Hkv * maps, splits), dim3(NTHREADS), smem, st,
                             q, ldq, kc, tied ? kc : vc, tied, out, ldo, block_table, max_pages, cu_q, ctx_len,
                             tile_seq, tile_row0, H, Hkv, ps, num_pages, scale * 1.4426950408889634f, window,
                             gate, ldg, splits, part_o, part_ml, maps, out_f32, q_rows, fold, softcap, scale, sink);
    if (e != 0 || splits == 1) return e;
    // (one tile a token: num_tiles is the number of tokens)
    return slb_launch(attention_kv_combine_kernel, dim3(num_tiles, H * maps), dim3(128), 0, st, (const float*)part_o,
                      (const float*)part_ml, splits, out, ldo, H * maps, gate, ldg, out_f32, sink);
}
// `tied`: the values are the first DV elements of the key rows (vc is ignored).
int slb_attention_kv_mma_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, int tied, bf16* out,
                              int ldo, const int* block_table, int max_pages, const int* cu_q,
                              const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                              int H, int Hkv, int ps, int num_pages, float scale, int window,
                              const bf16* gate, int ldg, int splits, float* part_o, float* part_ml,
                              int narrow, cudaStream_t st) {
    return launch_attention_kv_mma(q, ldq, kc, vc, tied, out, nullptr, ldo, block_table, max_pages, cu_q, ctx_len,
                                   tile_seq, tile_row0, num_tiles, H, Hkv, 1, ps, num_pages, scale, window, gate,
                                   ldg, splits, part_o, part_ml, narrow, 1, st);
}
// The same with a soft cap on the scaled scores (`softcap` > 0: s <- softcap tanh(s / softcap)) and a
// sink a head (`sink` [H] float32 or null) in the softmax's denominator.
int slb_attention_kv_mma_capped_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, int tied, bf16* out,
                                     int ldo, const int* block_table, int max_pages, const int* cu_q,
                                     const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                                     int H, int Hkv, int ps, int num_pages, float scale, int window,
                                     const bf16* gate, int ldg, int splits, float* part_o, float* part_ml,
                                     int narrow, float softcap, const float* sink, cudaStream_t st) {
    return launch_attention_kv_mma(q, ldq, kc, vc, tied, out, nullptr, ldo, block_table, max_pages, cu_q, ctx_len,
                                   tile_seq, tile_row0, num_tiles, H, Hkv, 1, ps, num_pages, scale, window, gate,
                                   ldg, splits, part_o, part_ml, narrow, 1, st, softcap, sink);
}
// `maps` attention maps a head; float32 results [token][head][map][DV] with rows `ldo` floats apart
int slb_attention_kv_mma_maps_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, int maps, float* out,
                                   int ldo, const int* block_table, int max_pages, const int* cu_q,
                                   const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                                   int H, int Hkv, int ps, int num_pages, float scale, int window, int splits,
                                   float* part_o, float* part_ml, int narrow, cudaStream_t st) {
    return launch_attention_kv_mma(q, ldq, kc, vc, 0, nullptr, out, ldo, block_table, max_pages, cu_q, ctx_len,
                                   tile_seq, tile_row0, num_tiles, H, Hkv, maps, ps, num_pages, scale, window,
                                   nullptr, 0, splits, part_o, part_ml, narrow, 1, st);
}
// The same results from a library built for keys of maps * (a map's key size): the maps are rows
// of one block (H and Hkv are the model's head counts; q [token][head][map][DK / maps]).
int slb_attention_kv_mma_folded_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, int maps, float* out,
                                     int ldo, const int* block_table, int max_pages, const int* cu_q,
                                     const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                                     int H, int Hkv, int ps, int num_pages, float scale, int window, int splits,
                                     float* part_o, float* part_ml, int narrow, cudaStream_t st) {
    if (maps < 1) return SLB_ERR_BAD_ARG;
    return launch_attention_kv_mma(q, ldq, kc, vc, 0, nullptr, out, ldo, block_table, max_pages, cu_q, ctx_len,
                                   tile_seq, tile_row0, num_tiles, H * maps, Hkv, 1, ps, num_pages, scale, window,
                                   nullptr, 0, splits, part_o, part_ml, narrow, maps, st);
}
}

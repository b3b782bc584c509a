// Linear attention with a fixed decay per head for steps that bring portions of prompts, in its
// chunked form on the tensor cores (bf16 mma.sync, float32 accumulators).
//
// A request's portion is cut into chunks of 64 tokens from its first token on.  With S the state
// [D, Dv] that enters a chunk of n tokens, g the head's decay and i, j token indices in the chunk:
//
//     o_i   = g^(i+1) S^T q_i  +  sum_{j <= i} g^(i-j) (q_i . k_j) v_j
//     S_out = g^n S  +  sum_j g^(n-1-j) k_j v_j^T
//
// which is the recurrence S_t = g S_{t-1} + k_t v_t^T, o_t = S_t^T q_t written out.  Three launches:
//
//   1. local sums   a block per (chunk, head, 64 value columns): L = sum_j g^(n-1-j) k_j v_j^T, float32
//                   into a work buffer [chunks, H, D, Dv];
//   2. scan         a thread per state element of a (request, head): walks the request's chunks
//                   in order, S <- g^n S + L in float32, leaves in the work buffer the state that ENTERS
//                   each chunk, and the final state in the request's slot;
//   3. outputs      a block per (chunk, head, 64 value columns): the formula for o_i above.
//
// The state, the decay powers, the decay mask of the scores and all sums are float32.  Activation,
// rotation (float32 angles, sincosf) and the key factor are applied in float32 as q, k and v are
// staged.  An operand of a tensor-core product is a float32 number x, which bfloat16 cannot hold:
// it is staged as two bfloat16 numbers, hi = bf16(x) and lo = bf16(x - hi), and a product a . b
// is three MMAs, a_hi b_hi + a_hi b_lo + a_lo b_hi, which leaves an error of about 2^-16 of the
// product's terms (`split` = 0 stages hi alone: one MMA, operands rounded to 8 bits).  So the
// result differs from the recurrent kernel beside this one by float32-like rounding, however a
// prompt is cut; that kernel is the bit-exact twin and the float32 path.
#include "decay_attention.cuh"
#include "mma_util.cuh"

using namespace slb_mma;

#define DC_CHUNK 64
#define DC_THREADS 256
#define DC_PAD 8                   // bf16 elements added to every shared row (ldmatrix without bank conflicts)
#define DC_MAX_D 128
#define DC_EV 64                   // value columns a block
#define DC_LDV (DC_EV + DC_PAD)
#define DC_SCAN_BATCH 16

struct DecayChunkArgs {
    DecayAttnArgs a;
    const int* tile_seq; const int* tile_row0; int num_tiles;
    float* work;                   // [num_tiles][H][D][Dv] float32
};

// g^m for m = 0 .. 64
__device__ __forceinline__ void dc_powers(float* pw, float g) {
    for (int m = threadIdx.x; m <= DC_CHUNK; m += DC_THREADS) pw[m] = powf(g, (float)m);
}

__device__ __forceinline__ void dc_zero(void* p, int bytes) {          // bytes a multiple of 16, p 16-byte aligned
    uint4* q = reinterpret_cast<uint4*>(p);
    for (int i = threadIdx.x; i < bytes / 16; i += DC_THREADS) q[i] = make_uint4(0, 0, 0, 0);
}

// x as hi (+ lo) at index idx of two arrays `lo_off` elements apart
template <bool SPLIT>
__device__ __forceinline__ void dc_put(bf16* hi, int lo_off, int idx, float x) {
    const bf16 h = __float2bfloat16(x);
    hi[idx] = h;
    if (SPLIT) hi[lo_off + idx] = __float2bfloat16(x - __bfloat162float(h));
}

template <bool SPLIT>
__device__ __forceinline__ void dc_mma(float (&c)[4], const unsigned (&ah)[4], const unsigned (&al)[4],
                                       unsigned bh0, unsigned bh1, unsigned bl0, unsigned bl1) {
    if (SPLIT) {
        mma_bf16(c, al, bh0, bh1);
        mma_bf16(c, ah, bl0, bl1);
    }
    mma_bf16(c, ah, bh0, bh1);
}

// eight neighbours at index idx (a multiple of 8; the arrays are 16-byte aligned)
template <bool SPLIT>
__device__ __forceinline__ void dc_put8(bf16* hi, int lo_off, int idx, const float (&x)[8]) {
    unsigned h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        h[e] = pack_bf16(x[2 * e], x[2 * e + 1]);
        if (SPLIT) {
            const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162*>(&h[e]);
            l[e] = pack_bf16(x[2 * e] - __low2float(hv), x[2 * e + 1] - __high2float(hv));
        }
    }
    *reinterpret_cast<uint4*>(hi + idx) = make_uint4(h[0], h[1], h[2], h[3]);
    if (SPLIT) *reinterpret_cast<uint4*>(hi + lo_off + idx) = make_uint4(l[0], l[1], l[2], l[3]);
}

__device__ __forceinline__ void dc_load8(float (&x)[8], const bf16* p, bool act) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
        x[2 * e] = act ? da_silu(f.x) : f.x;
        x[2 * e + 1] = act ? da_silu(f.y) : f.y;
    }
}

// Prepared q and / or k of the chunk's n tokens into shared rows of `ld` elements (rows from n on
// and columns from D on are zeroed by the caller); the lo halves sit `lo_off` elements behind the
// hi ones.  Eight elements a load where the sizes and offsets are multiples of 8 (and the rotated
// part of 16), else one.
template <bool SPLIT, bool WITH_Q>
__device__ __forceinline__ void dc_stage_qk(bf16* qs, bf16* ks, int ld, int lo_off, const bf16* proj, int tok0, int n,
                                            int h, const DecayAttnArgs& a) {
    const int D = a.D, half = a.rot_dims >> 1, rest = D - a.rot_dims;
    const bool act = a.act == 1;
    const bool wide = ((a.ld | a.q_off | a.k_off | D | half) & 7) == 0 && (reinterpret_cast<size_t>(proj) & 15) == 0;
    if (wide) {
        const int hv = half >> 3, rv = rest >> 3;
        for (int idx = threadIdx.x; idx < n * hv; idx += DC_THREADS) {
            const int j = idx / hv, i = (idx - j * hv) << 3;
            const bf16* row = proj + (size_t)(tok0 + j) * a.ld + h * D + i;
            float qu[8], qv[8], ku[8], kv[8], sn[8], cs[8], x[8], y[8];
            if (WITH_Q) { dc_load8(qu, row + a.q_off, act); dc_load8(qv, row + a.q_off + half, act); }
            dc_load8(ku, row + a.k_off, act);
            dc_load8(kv, row + a.k_off + half, act);
            const float pos = (float)a.positions[tok0 + j];
#pragma unroll
            for (int e = 0; e < 8; ++e) sincosf(pos * a.freq[i + e], &sn[e], &cs[e]);
            if (WITH_Q) {
#pragma unroll
                for (int e = 0; e < 8; ++e) { x[e] = qu[e] * cs[e] - qv[e] * sn[e]; y[e] = qv[e] * cs[e] + qu[e] * sn[e]; }
                dc_put8<SPLIT>(qs, lo_off, j * ld + i, x);
                dc_put8<SPLIT>(qs, lo_off, j * ld + i + half, y);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x[e] = (ku[e] * cs[e] - kv[e] * sn[e]) * a.k_scale;
                y[e] = (kv[e] * cs[e] + ku[e] * sn[e]) * a.k_scale;
            }
            dc_put8<SPLIT>(ks, lo_off, j * ld + i, x);
            dc_put8<SPLIT>(ks, lo_off, j * ld + i + half, y);
        }
        for (int idx = threadIdx.x; idx < n * rv; idx += DC_THREADS) {
            const int j = idx / rv, d = a.rot_dims + ((idx - j * rv) << 3);
            const bf16* row = proj + (size_t)(tok0 + j) * a.ld + h * D + d;
            float x[8];
            if (WITH_Q) {
                dc_load8(x, row + a.q_off, act);
                dc_put8<SPLIT>(qs, lo_off, j * ld + d, x);
            }
            dc_load8(x, row + a.k_off, act);
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] *= a.k_scale;
            dc_put8<SPLIT>(ks, lo_off, j * ld + d, x);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < n * half; idx += DC_THREADS) {
        const int j = idx / half, i = idx - j * half;
        const bf16* row = proj + (size_t)(tok0 + j) * a.ld;
        float sn, cs;
        sincosf((float)a.positions[tok0 + j] * a.freq[i], &sn, &cs);
        if (WITH_Q) {
            float u = to_float(row[a.q_off + h * D + i]), v = to_float(row[a.q_off + h * D + i + half]);
            if (act) { u = da_silu(u); v = da_silu(v); }
            dc_put<SPLIT>(qs, lo_off, j * ld + i, u * cs - v * sn);
            dc_put<SPLIT>(qs, lo_off, j * ld + i + half, v * cs + u * sn);
        }
        float u = to_float(row[a.k_off + h * D + i]), v = to_float(row[a.k_off + h * D + i + half]);
        if (act) { u = da_silu(u); v = da_silu(v); }
        dc_put<SPLIT>(ks, lo_off, j * ld + i, (u * cs - v * sn) * a.k_scale);
        dc_put<SPLIT>(ks, lo_off, j * ld + i + half, (v * cs + u * sn) * a.k_scale);
    }
    for (int idx = threadIdx.x; idx < n * rest; idx += DC_THREADS) {
        const int j = idx / rest, d = a.rot_dims + (idx - j * rest);
        const bf16* row = proj + (size_t)(tok0 + j) * a.ld;
        if (WITH_Q) {
            float u = to_float(row[a.q_off + h * D + d]);
            if (act) u = da_silu(u);
            dc_put<SPLIT>(qs, lo_off, j * ld + d, u);
        }
        float u = to_float(row[a.k_off + h * D + d]);
        if (act) u = da_silu(u);
        dc_put<SPLIT>(ks, lo_off, j * ld + d, u * a.k_scale);
    }
}

// v of the chunk's tokens, columns e0 .. e0 + 63, row j times pw[n - 1 - j] if `pw` is given
template <bool SPLIT>
__device__ __forceinline__ void dc_stage_v(bf16* vs, int lo_off, const bf16* proj, int tok0, int n, int h, int e0,
                                           const float* pw, const DecayAttnArgs& a) {
    const int width = min(DC_EV, a.Dv - e0);
    const bool act = a.act == 1;
    if (((a.ld | a.v_off | a.Dv) & 7) == 0 && (reinterpret_cast<size_t>(proj) & 15) == 0) {
        const int wv = width >> 3;
        for (int idx = threadIdx.x; idx < n * wv; idx += DC_THREADS) {
            const int j = idx / wv, col = (idx - j * wv) << 3;
            float x[8];
            dc_load8(x, proj + (size_t)(tok0 + j) * a.ld + a.v_off + h * a.Dv + e0 + col, act);
            if (pw != nullptr) {
                const float w = pw[n - 1 - j];
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] *= w;
            }
            dc_put8<SPLIT>(vs, lo_off, j * DC_LDV + col, x);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < n * width; idx += DC_THREADS) {
        const int j = idx / width, col = idx - j * width;
        float v = to_float(proj[(size_t)(tok0 + j) * a.ld + a.v_off + h * a.Dv + e0 + col]);
        if (act) v = da_silu(v);
        if (pw != nullptr) v *= pw[n - 1 - j];
        dc_put<SPLIT>(vs, lo_off, j * DC_LDV + col, v);
    }
}

// ------------------------------------------------------------------ 1. local sums of a chunk
template <bool SPLIT>
__global__ void __launch_bounds__(DC_THREADS) decay_chunk_local_kernel(const DecayChunkArgs c) {
    extern __shared__ __align__(16) unsigned char dc_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const DecayAttnArgs& a = c.a;
    const int tile = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * DC_EV;
    const int s = c.tile_seq[tile], row0 = c.tile_row0[tile];
    const int q0 = a.cu_q[s];
    const int n = min(DC_CHUNK, a.cu_q[s + 1] - q0 - row0);
    if (n <= 0) return;
    const int D = a.D, Dv = a.Dv, Dp = (D + 15) & ~15;
    const int ldk = Dp + DC_PAD;
    const int k_elems = DC_CHUNK * ldk, v_elems = DC_CHUNK * DC_LDV;
    const int parts = SPLIT ? 2 : 1;
    bf16* ks = reinterpret_cast<bf16*>(dc_smem);            // [parts][64][ldk]
    bf16* vs = ks + parts * k_elems;                        // [parts][64][DC_LDV]
    float* pw = reinterpret_cast<float*>(vs + parts * v_elems);
    dc_powers(pw, a.decay[h]);
    if (n < DC_CHUNK || D < Dp || Dv - e0 < DC_EV)          // (a full tile is written whole)
        dc_zero(ks, parts * (k_elems + v_elems) * (int)sizeof(bf16));
    __syncthreads();
    const bf16* proj = reinterpret_cast<const bf16*>(a.proj);
    dc_stage_qk<SPLIT, false>(nullptr, ks, ldk, k_elems, proj, q0 + row0, n, h, a);
    dc_stage_v<SPLIT>(vs, v_elems, proj, q0 + row0, n, h, e0, pw, a);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int ksteps = (n + 15) >> 4;
    float* dst = c.work + ((size_t)tile * a.H + h) * (size_t)D * Dv;
    for (int mt = warp; mt < Dp / 16; mt += DC_THREADS / 32) {
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        for (int kk = 0; kk < ksteps; ++kk) {
            // A[m = d][k = token] from rows stored [token][d]
            const int a_at = (kk * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * ldk + mt * 16 + ((lane >> 3) & 1) * 8;
            unsigned ah[4], al[4] = {0, 0, 0, 0};
            ldmatrix_x4_trans(ah, ks + a_at);
            if (SPLIT) ldmatrix_x4_trans(al, ks + k_elems + a_at);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                // B[k = token][n = e] from rows stored [token][e]
                const int b_at = (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DC_LDV + np * 16 + ((lane >> 4) & 1) * 8;
                unsigned bh[4], bl[4] = {0, 0, 0, 0};
                ldmatrix_x4_trans(bh, vs + b_at);
                if (SPLIT) ldmatrix_x4_trans(bl, vs + v_elems + b_at);
                dc_mma<SPLIT>(acc[2 * np], ah, al, bh[0], bh[1], bl[0], bl[1]);
                dc_mma<SPLIT>(acc[2 * np + 1], ah, al, bh[2], bh[3], bl[2], bl[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int e = e0 + nt * 8 + 2 * t;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int d = mt * 16 + g + half * 8;
                if (d < D) {
                    if (e + 1 < Dv && !(Dv & 1))
                        *reinterpret_cast<float2*>(dst + (size_t)d * Dv + e) = make_float2(acc[nt][2 * half], acc[nt][2 * half + 1]);
                    else {
                        if (e < Dv) dst[(size_t)d * Dv + e] = acc[nt][2 * half];
                        if (e + 1 < Dv) dst[(size_t)d * Dv + e + 1] = acc[nt][2 * half + 1];
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------ 2. the states that enter the chunks
// A request's chunks are neighbours in the tile list, in order; the first one is found by a walk
// over the list.  The next chunk's local sums are fetched while this chunk's are used.
__global__ void __launch_bounds__(256) decay_chunk_scan_kernel(const DecayChunkArgs c) {
    pdl_wait();
    pdl_launch_dependents();
    const DecayAttnArgs& a = c.a;
    const int s = blockIdx.x, h = blockIdx.y;
    const int qlen = a.cu_q[s + 1] - a.cu_q[s];
    if (qlen <= 0) return;
    const int slot = a.state_slots[s];
    if (slot < 0 || slot >= a.num_slots) return;
    const int elems = a.D * a.Dv;
    const int idx = blockIdx.z * blockDim.x + threadIdx.x;
    if (idx >= elems) return;
    int first = 0;
    while (first < c.num_tiles && c.tile_seq[first] != s) ++first;
    const int count = (qlen + DC_CHUNK - 1) / DC_CHUNK;
    if (first + count > c.num_tiles) return;
    const float g = a.decay[h];
    const float g_full = powf(g, (float)DC_CHUNK);
    float* sp = a.state + ((size_t)slot * a.H + h) * (size_t)elems + idx;
    float* wp = c.work + ((size_t)first * a.H + h) * (size_t)elems + idx;
    const size_t step = (size_t)a.H * elems;
    float S = *sp;
    // (the loads of a batch do not wait for one another: one memory latency a batch, not a chunk)
    for (int k0 = 0; k0 < count; k0 += DC_SCAN_BATCH) {
        float L[DC_SCAN_BATCH];
#pragma unroll
        for (int u = 0; u < DC_SCAN_BATCH; ++u) L[u] = k0 + u < count ? wp[u * step] : 0.f;
#pragma unroll
        for (int u = 0; u < DC_SCAN_BATCH; ++u) {
            if (k0 + u < count) {
                const int n = min(DC_CHUNK, qlen - (k0 + u) * DC_CHUNK);
                wp[u * step] = S;
                S = fmaf(n == DC_CHUNK ? g_full : powf(g, (float)n), S, L[u]);
            }
        }
        wp += DC_SCAN_BATCH * step;
    }
    *sp = S;
}

// ------------------------------------------------------------------ 3. the chunk's outputs
// Eight warps: 16 tokens and 32 of the value columns each (the scores of 16 tokens are formed by the
// two warps that share them).  The masked scores stay in registers: the accumulator of q . k^T of
// 16 tokens x 16 keys has the layout of the A operand of the product with v.  The entering state's
// tile takes the place of the keys once the scores are formed (two blocks fit an SM that way).
template <bool SPLIT>
__global__ void __launch_bounds__(DC_THREADS) decay_chunk_out_kernel(const DecayChunkArgs c) {
    extern __shared__ __align__(16) unsigned char dc_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const DecayAttnArgs& a = c.a;
    const int tile = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * DC_EV;
    const int s = c.tile_seq[tile], row0 = c.tile_row0[tile];
    const int q0 = a.cu_q[s];
    const int n = min(DC_CHUNK, a.cu_q[s + 1] - q0 - row0);
    if (n <= 0) return;
    const int slot = a.state_slots[s];
    if (slot < 0 || slot >= a.num_slots) return;
    const int D = a.D, Dv = a.Dv, Dp = (D + 15) & ~15;
    const int ldk = Dp + DC_PAD;
    const int qk_elems = DC_CHUNK * ldk, v_elems = DC_CHUNK * DC_LDV, s_elems = Dp * DC_LDV;
    const int ks_elems = max(qk_elems, s_elems);            // a part of the queries, and of the keys, then the state's tile
    const int parts = SPLIT ? 2 : 1;
    bf16* qs = reinterpret_cast<bf16*>(dc_smem);            // [parts][64][ldk] (parts ks_elems apart)
    bf16* ks = qs + parts * ks_elems;                       // [parts][64][ldk], later [parts][Dp][DC_LDV]
    bf16* vs = ks + parts * ks_elems;                       // [parts][64][DC_LDV]
    float* pw = reinterpret_cast<float*>(vs + parts * v_elems);
    const int width = min(DC_EV, Dv - e0);
    dc_powers(pw, a.decay[h]);
    if (n < DC_CHUNK || D < Dp || width < DC_EV)            // (a full tile is written whole)
        dc_zero(qs, parts * (2 * ks_elems + v_elems) * (int)sizeof(bf16));
    __syncthreads();
    const bf16* proj = reinterpret_cast<const bf16*>(a.proj);
    const int tok0 = q0 + row0;
    dc_stage_qk<SPLIT, true>(qs, ks, ldk, ks_elems, proj, tok0, n, h, a);
    dc_stage_v<SPLIT>(vs, v_elems, proj, tok0, n, h, e0, nullptr, a);
    __syncthreads();

    const int warp = (threadIdx.x >> 5) & 3, wc = threadIdx.x >> 7;     // token group, half of the columns
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bool live = warp * 16 < n;
    const int a_row = (warp * 16 + (lane & 15)) * ldk + ((lane >> 4) & 1) * 8;   // A[m = token][k = d], + kk * 16

    // scores of this warp's tokens against the keys up to its own 16
    float p[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) p[nt][0] = p[nt][1] = p[nt][2] = p[nt][3] = 0.f;
    if (live) {
        for (int kk = 0; kk < Dp / 16; ++kk) {
            unsigned ah[4], al[4] = {0, 0, 0, 0};
            ldmatrix_x4(ah, qs + a_row + kk * 16);
            if (SPLIT) ldmatrix_x4(al, qs + ks_elems + a_row + kk * 16);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                if (np <= warp) {
                    // B[k = d][n = key] from rows stored [key][d]
                    const int b_at = (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * ldk + kk * 16 + ((lane >> 3) & 1) * 8;
                    unsigned bh[4], bl[4] = {0, 0, 0, 0};
                    ldmatrix_x4(bh, ks + b_at);
                    if (SPLIT) ldmatrix_x4(bl, ks + ks_elems + b_at);
                    dc_mma<SPLIT>(p[2 * np], ah, al, bh[0], bh[1], bl[0], bl[1]);
                    dc_mma<SPLIT>(p[2 * np + 1], ah, al, bh[2], bh[3], bl[2], bl[3]);
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = warp * 16 + g + 8 * (r >> 1), j = nt * 8 + 2 * t + (r & 1);
                p[nt][r] = (j <= i && i < n) ? p[nt][r] * pw[i - j] : 0.f;
            }
    }
    __syncthreads();                                        // every warp is done with the keys

    // the entering state's tile [d][e] over them (padding rows and columns zero)
    {
        const float* src = c.work + ((size_t)tile * a.H + h) * (size_t)D * Dv + e0;
        if (D < Dp || width < DC_EV) dc_zero(ks, parts * ks_elems * (int)sizeof(bf16));
        if (D < Dp || width < DC_EV) __syncthreads();
        if ((Dv & 7) == 0) {
            const int wv = width >> 3;
#pragma unroll 4
            for (int idx = threadIdx.x; idx < D * wv; idx += DC_THREADS) {
                const int d = idx / wv, col = (idx - d * wv) << 3;
                const float4 lo4 = *reinterpret_cast<const float4*>(src + (size_t)d * Dv + col);
                const float4 hi4 = *reinterpret_cast<const float4*>(src + (size_t)d * Dv + col + 4);
                const float x[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
                dc_put8<SPLIT>(ks, ks_elems, d * DC_LDV + col, x);
            }
        } else {
            for (int idx = threadIdx.x; idx < D * width; idx += DC_THREADS) {
                const int d = idx / width, col = idx - d * width;
                dc_put<SPLIT>(ks, ks_elems, d * DC_LDV + col, src[(size_t)d * Dv + col]);
            }
        }
    }
    __syncthreads();
    if (!live) return;                                      // (no barrier follows)

    // what the entering state gives: q . S, each token's row times g^(i + 1)
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    for (int kk = 0; kk < Dp / 16; ++kk) {
        unsigned ah[4], al[4] = {0, 0, 0, 0};
        ldmatrix_x4(ah, qs + a_row + kk * 16);
        if (SPLIT) ldmatrix_x4(al, qs + ks_elems + a_row + kk * 16);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
            // B[k = d][n = e] from rows stored [d][e]
            const int b_at = (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DC_LDV + (wc * 2 + np) * 16 + ((lane >> 4) & 1) * 8;
            unsigned bh[4], bl[4] = {0, 0, 0, 0};
            ldmatrix_x4_trans(bh, ks + b_at);
            if (SPLIT) ldmatrix_x4_trans(bl, ks + ks_elems + b_at);
            dc_mma<SPLIT>(acc[2 * np], ah, al, bh[0], bh[1], bl[0], bl[1]);
            dc_mma<SPLIT>(acc[2 * np + 1], ah, al, bh[2], bh[3], bl[2], bl[3]);
        }
    }
    {
        const float f0 = pw[warp * 16 + g + 1], f1 = pw[warp * 16 + g + 9];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            acc[nt][0] *= f0; acc[nt][1] *= f0;
            acc[nt][2] *= f1; acc[nt][3] *= f1;
        }
    }

    // plus the masked scores times v
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        if (kk <= warp) {
            unsigned ah[4], al[4] = {0, 0, 0, 0};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float x0 = p[2 * kk + (r >> 1)][2 * (r & 1)], x1 = p[2 * kk + (r >> 1)][2 * (r & 1) + 1];
                ah[r] = pack_bf16(x0, x1);
                if (SPLIT) {
                    const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162*>(&ah[r]);
                    al[r] = pack_bf16(x0 - __low2float(hv), x1 - __high2float(hv));
                }
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                // B[k = key][n = e] from rows stored [key][e]
                const int b_at = (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DC_LDV + (wc * 2 + np) * 16 + ((lane >> 4) & 1) * 8;
                unsigned bh[4], bl[4] = {0, 0, 0, 0};
                ldmatrix_x4_trans(bh, vs + b_at);
                if (SPLIT) ldmatrix_x4_trans(bl, vs + v_elems + b_at);
                dc_mma<SPLIT>(acc[2 * np], ah, al, bh[0], bh[1], bl[0], bl[1]);
                dc_mma<SPLIT>(acc[2 * np + 1], ah, al, bh[2], bh[3], bl[2], bl[3]);
            }
        }
    }
    const bool pairs = !((Dv | a.ldo) & 1);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const int e = e0 + (wc * 4 + nt) * 8 + 2 * t;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int i = warp * 16 + g + half * 8;
            if (i < n) {
                float* o = a.out + (size_t)(tok0 + i) * a.ldo + h * Dv;
                if (pairs && e + 1 < Dv) *reinterpret_cast<float2*>(o + e) = make_float2(acc[nt][2 * half], acc[nt][2 * half + 1]);
                else {
                    if (e < Dv) o[e] = acc[nt][2 * half];
                    if (e + 1 < Dv) o[e + 1] = acc[nt][2 * half + 1];
                }
            }
        }
    }
}

static size_t dc_local_smem(int D, bool split) {
    const int Dp = (D + 15) & ~15, parts = split ? 2 : 1;
    return (size_t)parts * (DC_CHUNK * (Dp + DC_PAD) + DC_CHUNK * DC_LDV) * sizeof(bf16) + (DC_CHUNK + 4) * sizeof(float);
}
static size_t dc_out_smem(int D, bool split) {
    const int Dp = (D + 15) & ~15, parts = split ? 2 : 1;
    const int qk = DC_CHUNK * (Dp + DC_PAD), st = Dp * DC_LDV;
    return (size_t)parts * (2 * (qk > st ? qk : st) + DC_CHUNK * DC_LDV) * sizeof(bf16) + (DC_CHUNK + 4) * sizeof(float);
}

template <bool SPLIT>
static int launch_decay_chunks(const DecayChunkArgs* c, int num_seqs, cudaStream_t st) {
    static unsigned long long done_local = 0, done_out = 0;
    const DecayAttnArgs& a = c->a;
    const size_t smem_local = dc_local_smem(a.D, SPLIT), smem_out = dc_out_smem(a.D, SPLIT);
    int rc = slb_configure(&done_local, decay_chunk_local_kernel<SPLIT>, dc_local_smem(DC_MAX_D, SPLIT));
    if (rc != 0) return rc;
    rc = slb_configure(&done_out, decay_chunk_out_kernel<SPLIT>, dc_out_smem(DC_MAX_D, SPLIT));
    if (rc != 0) return rc;
    const int vz = (a.Dv + DC_EV - 1) / DC_EV;
    const dim3 grid(c->num_tiles, a.H, vz);
    rc = slb_launch(decay_chunk_local_kernel<SPLIT>, grid, dim3(DC_THREADS), smem_local, st, *c);
    if (rc != 0) return rc;
    const int sz = (a.D * a.Dv + 255) / 256;
    rc = slb_launch(decay_chunk_scan_kernel, dim3(num_seqs, a.H, sz), dim3(256), 0, st, *c);
    if (rc != 0) return rc;
    return slb_launch(decay_chunk_out_kernel<SPLIT>, grid, dim3(DC_THREADS), smem_out, st, *c);
}

extern "C" {
int slb_decay_chunk_max_dim() { return DC_MAX_D; }
int slb_decay_chunk_tokens() { return DC_CHUNK; }
// proj bfloat16; `work` float32 [num_tiles][H][D][Dv]; the tile list cuts every request's tokens of
// the step into chunks of slb_decay_chunk_tokens() (request, first row), a request's in order.
int slb_decay_chunk_bf16(const DecayChunkArgs* c, int num_seqs, int split, cudaStream_t st) {
    const DecayAttnArgs& a = c->a;
    if (num_seqs <= 0 || c->num_tiles <= 0) return 0;
    if (a.H <= 0 || a.D <= 0 || a.Dv <= 0 || a.num_slots <= 0 || (a.rot_dims & 1) || a.rot_dims < 0 ||
        a.rot_dims > a.D || (a.rot_dims > 0 && a.freq == nullptr) || a.act < 0 || a.act > 1 || c->work == nullptr ||
        c->tile_seq == nullptr || c->tile_row0 == nullptr)
        return SLB_ERR_BAD_ARG;
    if (a.D > DC_MAX_D || a.H > 65535 || (a.Dv + DC_EV - 1) / DC_EV > 65535 || (a.D * a.Dv + 255) / 256 > 65535)
        return SLB_ERR_TOO_LARGE;
    return split ? launch_decay_chunks<true>(c, num_seqs, st) : launch_decay_chunks<false>(c, num_seqs, st);
}
}

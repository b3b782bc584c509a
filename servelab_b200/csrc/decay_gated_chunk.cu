// Linear attention with a decay of its own for every token and key channel, for portions of
// prompts: the recurrence
//
//     S_t = diag(alpha_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t
//
// cut into chunks of 32 tokens.  With l_t = log alpha_t and L_t = l_first + ... + l_t inside a chunk
// (per key channel d), and S the state that enters the chunk,
//
//     o_t   = sum_d q_t[d] e^(L_t[d]) S[d][:]  +  sum_{j <= t} A[t][j] v_j,
//     A[t][j] = sum_d q_t[d] k_j[d] e^(L_t[d] - L_j[d]),
//     S_out = diag(e^(L_last)) S + sum_j diag(e^(L_last - L_j)) k_j v_j^T.
//
// Every exponent is a difference L_t - L_j with j <= t, or L_t itself: never positive, so nothing
// overflows however fast a channel decays (a factorised form q e^L . k e^-L would).  All
// arithmetic is float32 on the CUDA cores: the logarithms of the decays, their sums, the
// exponentials, the products and the state (what enters a recurrence stays 32-bit also where the
// projections are bfloat16).
//
// Four launches:
//   1. per (chunk, head): L for the chunk's tokens, e^(L_last), the masked scores A, and -- kept for
//      launches 2 and 4, so that they only copy -- the queries times e^(L_t) and the keys times
//      e^(L_last - L_j);
//   2. per (chunk, head, 64 value columns): the chunk's own sum  sum_j e^(L_last - L_j) k_j v_j^T
//      into a work buffer;
//   3. per state element: the walk over a request's chunks, S <- e^(L_last) S + sum; the work
//      buffer is left holding the state that ENTERS every chunk, the slot the final state;
//   4. per (chunk, head, 64 value columns): the outputs.
// The result differs from the token-by-token kernel by float32 rounding only, and so does the
// result of a prompt cut elsewhere.
#include "decay_attention.cuh"

#define GC_CHUNK 32
#define GC_EV 64
#define GC_MAX_D 256
#define GC_SCAN_BATCH 16

struct GatedChunkArgs {
    DecayAttnArgs a;
    const int* tile_seq; const int* tile_row0; int num_tiles;
    float* work;        // [num_tiles][H][D][Dv]
    float* qdec;        // [tokens][H * D]: q_t[d] e^(L_t[d])
    float* kdec;        // [tokens][H * D]: k_j[d] e^(L_last[d] - L_j[d])
    float* dtot;        // [num_tiles][H][D]
    float* scores;      // [num_tiles][H][GC_CHUNK][GC_CHUNK]
};

__device__ __forceinline__ bool gc_tile(const GatedChunkArgs& c, int tile, int& t0, int& n) {
    const DecayAttnArgs& a = c.a;
    const int s = c.tile_seq[tile];
    const int q0 = a.cu_q[s];
    const int row0 = c.tile_row0[tile];
    n = min(GC_CHUNK, a.cu_q[s + 1] - q0 - row0);
    t0 = q0 + row0;
    return n > 0;
}

// ------------------------------------------------------------------ 1. logarithms and scores
template <typename T>
__global__ void __launch_bounds__(256) gated_chunk_prep_kernel(const GatedChunkArgs c) {
    extern __shared__ float gc_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const DecayAttnArgs& a = c.a;
    const int tile = blockIdx.x, h = blockIdx.y;
    int t0, n;
    if (!gc_tile(c, tile, t0, n)) return;
    const int D = a.D, LD = D + 1;
    float* Ls = gc_smem;                         // [GC_CHUNK][D + 1]
    float* qs = Ls + GC_CHUNK * LD;
    float* ks = qs + GC_CHUNK * LD;
    const T* proj = reinterpret_cast<const T*>(a.proj);
    // the logarithms of the decays, every (token, channel) on a thread of its own ...
#pragma unroll 4
    for (int idx = threadIdx.x; idx < n * D; idx += blockDim.x) {
        const int j = idx / D, d = idx - j * D;
        float z = a.gate_z[(size_t)(t0 + j) * a.ld_gate + h * D + d];
        if (a.gate_bias != nullptr) z += a.gate_bias[h * D + d];
        Ls[j * LD + d] = (fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * a.gate_inv_tau;      // log sigmoid(z) / tau
    }
    __syncthreads();
    // ... then their running sums, a channel a thread, in the order of the tokens
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float run = 0.f;
        for (int j = 0; j < n; ++j) {
            run += Ls[j * LD + d];
            Ls[j * LD + d] = run;
        }
        c.dtot[((size_t)tile * a.H + h) * D + d] = expf(run);
    }
    __syncthreads();
    const size_t ldl = (size_t)a.H * D;
#pragma unroll 4
    for (int idx = threadIdx.x; idx < n * D; idx += blockDim.x) {
        const int j = idx / D, d = idx - j * D;
        const T* row = proj + (size_t)(t0 + j) * a.ld;
        const int pos = a.positions[t0 + j];
        const float qv = da_prepared(row + a.q_off + h * D, d, pos, a) * a.q_scale;
        const float kv = da_prepared(row + a.k_off + h * D, d, pos, a) * a.k_scale;
        const float L = Ls[j * LD + d];
        qs[j * LD + d] = qv;
        ks[j * LD + d] = kv;
        c.qdec[(size_t)(t0 + j) * ldl + h * D + d] = qv * expf(L);
        c.kdec[(size_t)(t0 + j) * ldl + h * D + d] = kv * expf(Ls[(n - 1) * LD + d] - L);
    }
    __syncthreads();
    float* A = c.scores + ((size_t)tile * a.H + h) * (GC_CHUNK * GC_CHUNK);
    for (int e = threadIdx.x; e < GC_CHUNK * GC_CHUNK; e += blockDim.x) A[e] = 0.f;      // (above the diagonal)
    // The pairs (t, j <= t) of the chunk, numbered along the rows of the triangle so that every
    // thread gets as many: pair e sits in row t with t (t + 1) / 2 <= e.
    const int pairs = n * (n + 1) / 2;
    for (int e = threadIdx.x; e < pairs; e += blockDim.x) {
        int t = (int)((sqrtf(8.0f * (float)e + 1.0f) - 1.0f) * 0.5f);
        while (t * (t + 1) / 2 > e) --t;                   // (the root's rounding)
        while ((t + 1) * (t + 2) / 2 <= e) ++t;
        const int j = e - t * (t + 1) / 2;
        const float* qt = qs + t * LD;
        const float* kj = ks + j * LD;
        const float* Lt = Ls + t * LD;
        const float* Lj = Ls + j * LD;
        float sum = 0.f;
        // (the exponent is <= 0; the one-instruction 2^x is exact to 2 ulp there, and its argument's
        // rounding weighs on terms that are small by the same factor)
        for (int d = 0; d < D; ++d) sum = fmaf(qt[d] * kj[d], __expf(Lt[d] - Lj[d]), sum);
        A[t * GC_CHUNK + j] = sum;
    }
}

// ------------------------------------------------------------------ 2. a chunk's own sum
// Thread (dy, ex): state rows dy, dy + 16, ... and value columns 4 ex .. 4 ex + 3 of the slice.
template <typename T, int R>
__global__ void __launch_bounds__(256) gated_chunk_local_kernel(const GatedChunkArgs c) {
    extern __shared__ float gc_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const DecayAttnArgs& a = c.a;
    const int tile = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * GC_EV;
    int t0, n;
    if (!gc_tile(c, tile, t0, n)) return;
    const int D = a.D, Dv = a.Dv;
    float* kk = gc_smem;                         // [GC_CHUNK][D]: k_j[d] e^(L_last[d] - L_j[d])
    float* vs = kk + GC_CHUNK * D;               // [GC_CHUNK][GC_EV]
    const T* proj = reinterpret_cast<const T*>(a.proj);
    const size_t ldl = (size_t)a.H * D;
    const float* kd = c.kdec + (size_t)t0 * ldl + h * D;
    if ((D & 3) == 0) {                                   // (rows of launch 1's decayed keys, 16 bytes a load)
#pragma unroll 4
        for (int idx = threadIdx.x; idx < n * (D / 4); idx += blockDim.x) {
            const int j = idx / (D / 4), d4 = idx - j * (D / 4);
            *reinterpret_cast<float4*>(kk + j * D + d4 * 4) = *reinterpret_cast<const float4*>(kd + j * ldl + d4 * 4);
        }
    } else {
#pragma unroll 4
        for (int idx = threadIdx.x; idx < n * D; idx += blockDim.x) {
            const int j = idx / D, d = idx - j * D;
            kk[idx] = kd[j * ldl + d];
        }
    }
#pragma unroll 4
    for (int idx = threadIdx.x; idx < n * GC_EV; idx += blockDim.x) {
        const int j = idx / GC_EV, e = e0 + (idx - j * GC_EV);
        float v = 0.f;
        if (e < Dv) {
            v = to_float(proj[(size_t)(t0 + j) * a.ld + a.v_off + h * Dv + e]);
            if (a.act == 1) v = da_silu(v);
        }
        vs[idx] = v;
    }
    __syncthreads();
    const int ex = threadIdx.x & 15, dy = threadIdx.x >> 4;
    float acc[R][4];
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int j = 0; j < n; ++j) {
        const float4 v4 = *reinterpret_cast<const float4*>(vs + j * GC_EV + ex * 4);
        const float* kj = kk + j * D + dy;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            if (dy + 16 * i < D) {
                const float kv = kj[16 * i];
                acc[i][0] = fmaf(kv, v4.x, acc[i][0]);
                acc[i][1] = fmaf(kv, v4.y, acc[i][1]);
                acc[i][2] = fmaf(kv, v4.z, acc[i][2]);
                acc[i][3] = fmaf(kv, v4.w, acc[i][3]);
            }
        }
    }
    float* w = c.work + ((size_t)tile * a.H + h) * (size_t)D * Dv;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = dy + 16 * i;
        if (d < D) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = e0 + ex * 4 + u;
                if (e < Dv) w[(size_t)d * Dv + e] = acc[i][u];
            }
        }
    }
}

// ------------------------------------------------------------------ 3. the states that enter the chunks
// A request's chunks are neighbours in the tile list, in order; the first one is found by a walk
// over the list.
__global__ void __launch_bounds__(256) gated_chunk_scan_kernel(const GatedChunkArgs c) {
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
    const int d = idx / a.Dv;
    int first = 0;
    while (first < c.num_tiles && c.tile_seq[first] != s) ++first;
    const int count = (qlen + GC_CHUNK - 1) / GC_CHUNK;
    if (first + count > c.num_tiles) return;
    float* sp = a.state + (size_t)slot * (size_t)a.state_stride + (size_t)h * elems + idx;
    float* wp = c.work + ((size_t)first * a.H + h) * (size_t)elems + idx;
    const float* dp = c.dtot + ((size_t)first * a.H + h) * a.D + d;
    const size_t step = (size_t)a.H * elems, dstep = (size_t)a.H * a.D;
    float S = *sp;
    for (int k0 = 0; k0 < count; k0 += GC_SCAN_BATCH) {
        float L[GC_SCAN_BATCH], g[GC_SCAN_BATCH];
#pragma unroll
        for (int u = 0; u < GC_SCAN_BATCH; ++u) {
            L[u] = k0 + u < count ? wp[u * step] : 0.f;
            g[u] = k0 + u < count ? dp[u * dstep] : 1.f;
        }
#pragma unroll
        for (int u = 0; u < GC_SCAN_BATCH; ++u) {
            if (k0 + u < count) {
                wp[u * step] = S;
                S = fmaf(g[u], S, L[u]);
            }
        }
        wp += GC_SCAN_BATCH * step;
        dp += GC_SCAN_BATCH * dstep;
    }
    *sp = S;
}

// ------------------------------------------------------------------ 4. the chunk's outputs
// Thread (ty, ex): tokens ty and ty + 16 of the chunk, value columns 4 ex .. 4 ex + 3 of the slice.
template <typename T>
__global__ void __launch_bounds__(256) gated_chunk_out_kernel(const GatedChunkArgs c) {
    extern __shared__ float gc_smem[];
    pdl_wait();
    const DecayAttnArgs& a = c.a;
    const int tile = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * GC_EV;
    int t0, n;
    if (!gc_tile(c, tile, t0, n)) return;
    const int D = a.D, Dv = a.Dv, LD = (D + 3) & ~3;
    float* qt = gc_smem;                         // [GC_CHUNK][LD]: q_t[d] e^(L_t[d]); zero rows beyond n
    float* Sin = qt + GC_CHUNK * LD;             // [D][GC_EV]: the entering state's slice
    float* vs = Sin + (size_t)D * GC_EV;         // [GC_CHUNK][GC_EV]
    float* As = vs + GC_CHUNK * GC_EV;           // [GC_CHUNK][GC_CHUNK + 1]
    const T* proj = reinterpret_cast<const T*>(a.proj);
    const size_t ldl = (size_t)a.H * D;
    const float* qd = c.qdec + (size_t)t0 * ldl + h * D;
    if ((D & 3) == 0) {                                   // (rows of launch 1's decayed queries, 16 bytes a load)
#pragma unroll 4
        for (int idx = threadIdx.x; idx < GC_CHUNK * (D / 4); idx += blockDim.x) {
            const int j = idx / (D / 4), d4 = idx - j * (D / 4);
            *reinterpret_cast<float4*>(qt + j * LD + d4 * 4) =
                j < n ? *reinterpret_cast<const float4*>(qd + j * ldl + d4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
#pragma unroll 4
        for (int idx = threadIdx.x; idx < GC_CHUNK * D; idx += blockDim.x) {
            const int j = idx / D, d = idx - j * D;
            qt[j * LD + d] = j < n ? qd[j * ldl + d] : 0.f;
        }
    }
    const float* w = c.work + ((size_t)tile * a.H + h) * (size_t)D * Dv;
    if ((Dv & 3) == 0 && e0 + GC_EV <= Dv) {               // whole rows of the slice, 16 bytes a load
#pragma unroll 4
        for (int idx = threadIdx.x; idx < D * (GC_EV / 4); idx += blockDim.x) {
            const int d = idx / (GC_EV / 4), e4 = idx - d * (GC_EV / 4);
            *reinterpret_cast<float4*>(Sin + d * GC_EV + e4 * 4) =
                *reinterpret_cast<const float4*>(w + (size_t)d * Dv + e0 + e4 * 4);
        }
    } else {
#pragma unroll 4
        for (int idx = threadIdx.x; idx < D * GC_EV; idx += blockDim.x) {
            const int d = idx / GC_EV, e = e0 + (idx - d * GC_EV);
            Sin[idx] = e < Dv ? w[(size_t)d * Dv + e] : 0.f;
        }
    }
#pragma unroll 4
    for (int idx = threadIdx.x; idx < GC_CHUNK * GC_EV; idx += blockDim.x) {
        const int j = idx / GC_EV, e = e0 + (idx - j * GC_EV);
        float v = 0.f;
        if (j < n && e < Dv) {
            v = to_float(proj[(size_t)(t0 + j) * a.ld + a.v_off + h * Dv + e]);
            if (a.act == 1) v = da_silu(v);
        }
        vs[idx] = v;
    }
    const float* A = c.scores + ((size_t)tile * a.H + h) * (GC_CHUNK * GC_CHUNK);
    for (int idx = threadIdx.x; idx < GC_CHUNK * GC_CHUNK; idx += blockDim.x)
        As[(idx / GC_CHUNK) * (GC_CHUNK + 1) + idx % GC_CHUNK] = A[idx];
    __syncthreads();
    pdl_launch_dependents();
    const int ex = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const float* q0 = qt + ty * LD;
    const float* q1 = qt + (ty + 16) * LD;
#define GC_ROW(a0, a1, s4)                                                                  \
    acc[0][0] = fmaf(a0, s4.x, acc[0][0]); acc[0][1] = fmaf(a0, s4.y, acc[0][1]);           \
    acc[0][2] = fmaf(a0, s4.z, acc[0][2]); acc[0][3] = fmaf(a0, s4.w, acc[0][3]);           \
    acc[1][0] = fmaf(a1, s4.x, acc[1][0]); acc[1][1] = fmaf(a1, s4.y, acc[1][1]);           \
    acc[1][2] = fmaf(a1, s4.z, acc[1][2]); acc[1][3] = fmaf(a1, s4.w, acc[1][3]);
    int d = 0;
    for (; d + 4 <= D; d += 4) {                           // (four state rows a step: the queries 16 bytes a load)
        const float4 qa = *reinterpret_cast<const float4*>(q0 + d);
        const float4 qb = *reinterpret_cast<const float4*>(q1 + d);
        const float4 s0 = *reinterpret_cast<const float4*>(Sin + d * GC_EV + ex * 4);
        const float4 s1 = *reinterpret_cast<const float4*>(Sin + (d + 1) * GC_EV + ex * 4);
        const float4 s2 = *reinterpret_cast<const float4*>(Sin + (d + 2) * GC_EV + ex * 4);
        const float4 s3 = *reinterpret_cast<const float4*>(Sin + (d + 3) * GC_EV + ex * 4);
        GC_ROW(qa.x, qb.x, s0) GC_ROW(qa.y, qb.y, s1) GC_ROW(qa.z, qb.z, s2) GC_ROW(qa.w, qb.w, s3)
    }
    for (; d < D; ++d) {
        const float4 s4 = *reinterpret_cast<const float4*>(Sin + d * GC_EV + ex * 4);
        const float a0 = q0[d], a1 = q1[d];
        GC_ROW(a0, a1, s4)
    }
    const float* A0 = As + ty * (GC_CHUNK + 1);
    const float* A1 = As + (ty + 16) * (GC_CHUNK + 1);
    for (int j = 0; j < n; ++j) {
        const float4 v4 = *reinterpret_cast<const float4*>(vs + j * GC_EV + ex * 4);
        const float a0 = A0[j], a1 = A1[j];
        GC_ROW(a0, a1, v4)
    }
#undef GC_ROW
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int t = ty + 16 * r;
        if (t < n) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = e0 + ex * 4 + u;
                if (e < Dv) a.out[(size_t)(t0 + t) * a.ldo + h * Dv + e] = acc[r][u];
            }
        }
    }
}

template <typename T>
static int launch_gated_chunk(const GatedChunkArgs* c_in, int num_seqs, cudaStream_t st) {
    if (num_seqs <= 0 || c_in->num_tiles <= 0) return 0;
    GatedChunkArgs c = *c_in;
    DecayAttnArgs& a = c.a;
    if (a.state_stride <= 0) a.state_stride = (long long)a.H * a.D * a.Dv;
    if (a.H <= 0 || a.D <= 0 || a.Dv <= 0 || a.num_slots <= 0 || (a.rot_dims & 1) || a.rot_dims < 0 ||
        a.rot_dims > a.D || (a.rot_dims > 0 && a.freq == nullptr) || a.act < 0 || a.act > 1 ||
        a.gate_z == nullptr || a.ld_gate < a.H * a.D || !(a.gate_inv_tau > 0.f) ||
        a.state_stride < (long long)a.H * a.D * a.Dv || c.work == nullptr || c.qdec == nullptr || c.kdec == nullptr ||
        c.dtot == nullptr || c.scores == nullptr || c.tile_seq == nullptr || c.tile_row0 == nullptr)
        return SLB_ERR_BAD_ARG;
    if (a.D > GC_MAX_D || a.H > 65535 || num_seqs > 65535) return SLB_ERR_TOO_LARGE;
    const int vz = (a.Dv + GC_EV - 1) / GC_EV;
    const int ez = (a.D * a.Dv + 255) / 256;
    if (vz > 65535 || ez > 65535) return SLB_ERR_TOO_LARGE;
    const size_t smem1 = (size_t)3 * GC_CHUNK * (a.D + 1) * sizeof(float);
    const size_t smem2 = ((size_t)GC_CHUNK * a.D + GC_CHUNK * GC_EV) * sizeof(float);
    const size_t smem4 = ((size_t)GC_CHUNK * ((a.D + 3) & ~3) + (size_t)a.D * GC_EV + GC_CHUNK * GC_EV +
                          GC_CHUNK * (GC_CHUNK + 1)) * sizeof(float);
    constexpr size_t MAX1 = (size_t)3 * GC_CHUNK * (GC_MAX_D + 1) * sizeof(float);
    constexpr size_t MAX4 = ((size_t)GC_CHUNK * (GC_MAX_D + 1) + (size_t)GC_MAX_D * GC_EV + GC_CHUNK * GC_EV +
                             GC_CHUNK * (GC_CHUNK + 1)) * sizeof(float);
    static unsigned long long conf1 = 0, conf4 = 0;
    int rc = slb_configure(&conf1, gated_chunk_prep_kernel<T>, MAX1);
    if (rc != 0) return rc;
    rc = slb_configure(&conf4, gated_chunk_out_kernel<T>, MAX4);
    if (rc != 0) return rc;
    rc = slb_launch(gated_chunk_prep_kernel<T>, dim3(c.num_tiles, a.H), dim3(256), smem1, st, c);
    if (rc != 0) return rc;
    if (a.D <= 128)
        rc = slb_launch(gated_chunk_local_kernel<T, 8>, dim3(c.num_tiles, a.H, vz), dim3(256), smem2, st, c);
    else
        rc = slb_launch(gated_chunk_local_kernel<T, GC_MAX_D / 16>, dim3(c.num_tiles, a.H, vz), dim3(256), smem2, st, c);
    if (rc != 0) return rc;
    rc = slb_launch(gated_chunk_scan_kernel, dim3(num_seqs, a.H, ez), dim3(256), 0, st, c);
    if (rc != 0) return rc;
    return slb_launch(gated_chunk_out_kernel<T>, dim3(c.num_tiles, a.H, vz), dim3(256), smem4, st, c);
}

extern "C" {
int slb_decay_gated_chunk_max_dim() { return GC_MAX_D; }
int slb_decay_gated_chunk_tokens() { return GC_CHUNK; }
int slb_decay_gated_chunk_f32(const GatedChunkArgs* c, int num_seqs, cudaStream_t st) {
    return launch_gated_chunk<float>(c, num_seqs, st);
}
int slb_decay_gated_chunk_bf16(const GatedChunkArgs* c, int num_seqs, cudaStream_t st) {
    return launch_gated_chunk<bf16>(c, num_seqs, st);
}
}

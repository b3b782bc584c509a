// Short causal convolution over time on the projected queries and keys, the query
// temperature, and the write of the keys into their pages.
//
// Input is the fused projection of each token, [T, C] with C = H D query channels followed
// by Hkv D key channels (more columns may follow; they are not touched).  Per channel c and
// token t at index j of its request's portion (the taps are passed transposed, w[i][c]):
//
//   y_t = sum_i w[i][c] * u_(j - (taps - 1) + i)
//
// where u comes from the portion for indices >= 0 and from the request's state record for
// the taps - 1 rows before it: state[slot][i][c] is the projected row taps - 1 - i places
// before the portion (zeros for a new request: a cleared slot).  Everything is float32.
// Query channels are then multiplied by 1 + coef * ln(floor((p + 1) / every) + 1) at position
// p and stored to q_out; key channels go to the page the block table names,
// k_cache[page][kv head][p % page_size][D].
//
// The state must end up as the last taps - 1 rows of (old state, portion).  In a step of
// single tokens the thread that computes (request, channel) is the only one that reads that
// column of the record, so it shifts it on the spot (`update_inline`).  With portions other
// blocks may still read the old record, so a second, small kernel writes it afterwards.
//
// With no key heads (Hkv = 0) every channel is a "query" channel: the kernel is then a plain
// convolution of the first q_size columns into q_out, which a mixer runs on q | k | v before its
// head kernel.  The records of two requests lie `state_stride` floats apart (a record may be part of
// a larger one).
#include "common.cuh"

#define SC_MAX_TAPS 64

SLB_DEFINE_STATUS_WORD(conv_cache_status_word, slb_conv_cache_status)

// VEC consecutive elements as floats, by 16-byte accesses where VEC allows
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[VEC]) {
    if constexpr (VEC == 1) {
        v[0] = to_float(p[0]);
    } else if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float4 x = *reinterpret_cast<const float4*>(p + i);
            v[i] = x.x; v[i + 1] = x.y; v[i + 2] = x.z; v[i + 3] = x.w;
        }
    } else {
        static_assert(VEC == 8, "bfloat16 vectors are 8 wide");
        const uint4 x = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[VEC]) {
    if constexpr (VEC == 1) {
        p[0] = from_float<T>(v[0]);
    } else if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4)
            *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
        uint4 x;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = x;
    }
}

// taps_w is [taps][C] (a tap's weights of neighbouring channels are neighbours).  A thread owns
// VEC neighbouring channels of one token; a vector never straddles the q | k border or a head.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) qk_conv_cache_kernel(
    const T* __restrict__ proj, int ldp, const float* __restrict__ taps_w, int taps,
    float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_q,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
    float temp_coef, int temp_every, T* __restrict__ q_out, int ldq, T* __restrict__ k_cache,
    int q_size, int Hkv, int D, int update_inline, long long state_stride) {
    const int C = q_size + Hkv * D;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int t = blockIdx.y;
    const int s = seq_of_token[t];
    const int q0 = cu_q[s];
    const int j = t - q0;
    const int pos = positions[t];
    const int hist = taps - 1;
    float* st = state != nullptr ? state + (size_t)state_slots[s] * state_stride + c : nullptr;
    float y[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) y[v] = 0.f;
    for (int i = 0; i < taps; ++i) {
        const int jj = j - hist + i;
        float u[VEC], w[VEC];
        if (jj >= 0) {
            load_vec<T, VEC>(proj + (size_t)(q0 + jj) * ldp + c, u);
        } else if (st != nullptr) {
            load_vec<float, VEC>(st + (size_t)(hist + jj) * C, u);
        } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) u[v] = 0.f;
        }
        load_vec<float, VEC>(taps_w + (size_t)i * C + c, w);
#pragma unroll
        for (int v = 0; v < VEC; ++v) y[v] = fmaf(w[v], u[v], y[v]);
        // a step of single tokens: row i - 1 of the new record is row i of (record, token); this
        // thread alone reads and writes these columns of the record, in this order
        if (update_inline && i >= 1 && st != nullptr) store_vec<float, VEC>(st + (size_t)(i - 1) * C, u);
    }
    if (c < q_size) {
        if (temp_coef != 0.f) {
            const float f = 1.f + temp_coef * logf(floorf((float)(pos + 1) / (float)temp_every) + 1.f);
#pragma unroll
            for (int v = 0; v < VEC; ++v) y[v] *= f;
        }
        store_vec<T, VEC>(q_out + (size_t)t * ldq + c, y);
    } else if (k_cache != nullptr) {
        const int cc = c - q_size;
        const int kvh = cc / D, d = cc - kvh * D;
        const int page = block_table[(size_t)s * max_pages + pos / page_size];
        if (page >= num_pages) atomicCAS(&conv_cache_status_word, 0, 1);
        else if (page >= 0)
            store_vec<T, VEC>(k_cache + (((size_t)page * Hkv + kvh) * page_size + pos % page_size) * D + d, y);
    }
}

// new record = last taps - 1 rows of (old record, this step's portion), per request and channel
template <typename T>
__global__ void __launch_bounds__(256) conv_state_update_kernel(
    const T* __restrict__ proj, int ldp, int taps, float* __restrict__ state,
    const int* __restrict__ state_slots, const int* __restrict__ cu_q, int C, long long state_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = blockIdx.y;
    const int q0 = cu_q[s], n = cu_q[s + 1] - q0;
    if (n <= 0) return;
    const int hist = taps - 1;
    float* st = state + (size_t)state_slots[s] * state_stride + c;
    // ascending i: row i + n of the old record is read before any row >= i + 1 is written
    for (int i = 0; i < hist; ++i) {
        const int src = i + n - hist;              // index into the portion, or before it
        st[(size_t)i * C] = src >= 0 ? to_float(proj[(size_t)(q0 + src) * ldp + c]) : st[(size_t)(i + n) * C];
    }
}

template <typename T>
static int launch_conv(const T* proj, int ldp, const float* taps_w, int taps, float* state,
                       const int* state_slots, const int* cu_q, const int* seq_of_token,
                       const int* positions, const int* block_table, int max_pages, int page_size,
                       int num_pages, float temp_coef, int temp_every, T* q_out, int ldq, T* k_cache,
                       int T_tokens, int S, int q_size, int Hkv, int D, int decode_only, long long state_stride,
                       cudaStream_t st) {
    if (T_tokens <= 0) return 0;
    if (state_stride <= 0) state_stride = (long long)(taps - 1) * (q_size + Hkv * D);
    if (state_stride < (long long)(taps - 1) * (q_size + Hkv * D)) return SLB_ERR_BAD_ARG;
    if (Hkv == 0) { D = 0; page_size = 1; }             // (no key channels: a convolution alone)
    if (taps < 1 || q_size < 0 || Hkv < 0 || (Hkv > 0 && D <= 0) || q_size + Hkv * D <= 0 || page_size <= 0 ||
        temp_every <= 0 ||
        (taps > 1 && state == nullptr) || T_tokens > 65535 || S > 65535)
        return SLB_ERR_BAD_ARG;
    if (taps > SC_MAX_TAPS) return SLB_ERR_TOO_LARGE;
    const int C = q_size + Hkv * D;
    const int inline_update = decode_only && taps > 1 ? 1 : 0;
    constexpr int V = 16 / (int)sizeof(T);             // channels of one 16-byte access
    const bool vec = q_size % V == 0 && D % V == 0 && ldp % V == 0 && ldq % V == 0 && C % 4 == 0 &&
                     state_stride % 4 == 0 &&
                     (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)state |
                       (uintptr_t)taps_w) & 15) == 0;
    int rc;
    if (vec) {
        const int threads = C / V >= 256 ? 256 : 64;
        rc = slb_launch(qk_conv_cache_kernel<T, V>, dim3((C / V + threads - 1) / threads, T_tokens), dim3(threads),
                        0, st, proj, ldp, taps_w, taps, state, state_slots, cu_q, seq_of_token, positions,
                        block_table, max_pages, page_size, num_pages, temp_coef, temp_every, q_out, ldq,
                        k_cache, q_size, Hkv, D, inline_update, state_stride);
    } else {
        rc = slb_launch(qk_conv_cache_kernel<T, 1>, dim3((C + 255) / 256, T_tokens), dim3(256), 0, st, proj,
                        ldp, taps_w, taps, state, state_slots, cu_q, seq_of_token, positions, block_table,
                        max_pages, page_size, num_pages, temp_coef, temp_every, q_out, ldq, k_cache, q_size,
                        Hkv, D, inline_update, state_stride);
    }
    if (rc != 0 || taps == 1 || inline_update) return rc;
    return slb_launch(conv_state_update_kernel<T>, dim3((C + 255) / 256, S), dim3(256), 0, st, proj, ldp,
                      taps, state, state_slots, cu_q, C, state_stride);
}

extern "C" {
int slb_qk_conv_cache_f32(const float* proj, int ldp, const float* taps_w, int taps, float* state,
                          const int* state_slots, const int* cu_q, const int* seq_of_token,
                          const int* positions, const int* block_table, int max_pages, int page_size,
                          int num_pages, float temp_coef, int temp_every, float* q_out, int ldq,
                          float* k_cache, int T_tokens, int S, int q_size, int Hkv, int D,
                          int decode_only, long long state_stride, cudaStream_t st) {
    return launch_conv<float>(proj, ldp, taps_w, taps, state, state_slots, cu_q, seq_of_token, positions,
                              block_table, max_pages, page_size, num_pages, temp_coef, temp_every, q_out,
                              ldq, k_cache, T_tokens, S, q_size, Hkv, D, decode_only, state_stride, st);
}
int slb_qk_conv_cache_bf16(const bf16* proj, int ldp, const float* taps_w, int taps, float* state,
                           const int* state_slots, const int* cu_q, const int* seq_of_token,
                           const int* positions, const int* block_table, int max_pages, int page_size,
                           int num_pages, float temp_coef, int temp_every, bf16* q_out, int ldq,
                           bf16* k_cache, int T_tokens, int S, int q_size, int Hkv, int D,
                           int decode_only, long long state_stride, cudaStream_t st) {
    return launch_conv<bf16>(proj, ldp, taps_w, taps, state, state_slots, cu_q, seq_of_token, positions,
                             block_table, max_pages, page_size, num_pages, temp_coef, temp_every, q_out,
                             ldq, k_cache, T_tokens, S, q_size, Hkv, D, decode_only, state_stride, st);
}
}

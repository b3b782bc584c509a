// Plain paged attention for mixers whose keys and values have different sizes: keys of Dk
// elements (up to 1,088), values of Dv (up to 512), grouped heads, causal with an optional window,
// any page size, any mix of prompt portions and single tokens.  float32 arithmetic throughout;
// inputs and outputs float32 or bfloat16.
//
// The values may live in the key cache itself: `ldv` is the row stride of a value row, so a
// latent attention whose cached row is [latent | rotated part] passes the key cache as the value
// cache with ldv = Dk and Dv = the latent's size (keys and values are then one kv head that every
// query head shares).
//
// Optional epilogue: the row of head h is multiplied by sigmoid(gate[token][h]) (one number a
// head).
//
// Optional in the scores: a soft cap, s <- cap tanh(s / cap) on the scaled score (`softcap` > 0),
// and a sink, one number a head whose exponential is added to the softmax's denominator once (it
// has no key and no value and is neither scaled nor capped).
//
// Several attention maps a head (`maps`, the differential form): every query head and every kv
// head carries `maps` query / key vectors side by side ([head][map][Dk], key rows `ldk` apart),
// each map is an attention of its own over the kv head's one set of values, and the results are
// written map by map ([token][head][map][Dv], float32 if asked for), for the kernel that combines
// them.  A block then owns (tile, kv head, map).
//
// Work unit: (tile of 32 flattened query rows rho = local_token * g + head_in_group, kv head).
// Keys are visited in tiles of 32 aligned to absolute positions, in increasing order, with an
// online softmax per row; the head dimension is walked in chunks of 64 through one shared
// buffer, so large heads need no more shared memory than small ones.  A row's result depends
// only on its query and the keys it may see: not on the other rows, the cut of the prompt, or
// the pages.
#include "common.cuh"

#define AK_BM 32
#define AK_BN 32
#define AK_DC 64
#define AK_THREADS 256
#define AK_MAX_DK 1088
#define AK_MAX_DV 512

SLB_DEFINE_STATUS_WORD(attention_kv_status_word, slb_attention_kv_status)

template <typename T, typename TO>
__global__ void __launch_bounds__(AK_THREADS) attention_kv_kernel(
    const T* __restrict__ q, int ldq, const T* __restrict__ kc, int ldk, int maps, const T* __restrict__ vc, int ldv,
    TO* __restrict__ out, int ldo, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
    int H, int Hkv, int Dk, int Dv, int ps, int num_pages, float scale, int window,
    const T* __restrict__ gate, int ldg, float softcap, const float* __restrict__ sink) {
    extern __shared__ float ak_smem[];
    pdl_wait();
    const int ldq_s = Dk + 1;
    float* Qs = ak_smem;                              // [AK_BM][Dk + 1]
    float* Cs = Qs + AK_BM * ldq_s;                   // [AK_BN][AK_DC + 1]: a chunk of keys or values
    float* Ps = Cs + AK_BN * (AK_DC + 1);             // [AK_BM][AK_BN + 1]
    __shared__ int page_of[AK_BN];

    const int tid = threadIdx.x;
    const int kvh = blockIdx.y / maps, map = blockIdx.y - kvh * maps;
    const int s = tile_seq[blockIdx.x];
    const int row0 = tile_row0[blockIdx.x];
    const int g = H / Hkv;
    const int q0 = cu_q[s];
    const int qlen = cu_q[s + 1] - q0;
    const int ctx = ctx_len[s];
    const int nrows = min(AK_BM, qlen * g - row0);
    if (nrows <= 0) return;
    const int pos_base = ctx - qlen;

    for (int idx = tid; idx < AK_BM * Dk; idx += AK_THREADS) {
        const int r = idx / Dk, d = idx - r * Dk;
        float v = 0.f;
        if (r < nrows) {
            const int rho = row0 + r;
            const int tl = rho / g, hg = rho - tl * g;
            v = to_float(q[(size_t)(q0 + tl) * ldq + (size_t)((kvh * g + hg) * maps + map) * Dk + d]);
        }
        Qs[r * ldq_s + d] = v;
    }

    const int r = tid >> 3, c0 = tid & 7;
    const bool row_valid = r < nrows;
    const int my_pos = row_valid ? pos_base + (row0 + r) / g : -1;
    const int p_first = pos_base + row0 / g;
    const int p_last = pos_base + (row0 + nrows - 1) / g;
    int kbeg = 0;
    if (window > 0) kbeg = max(0, p_first - window + 1) / AK_BN * AK_BN;
    const int kend = p_last + 1;
    const int nvc = (Dv + AK_DC - 1) / AK_DC;

    float m = -INFINITY, l = 0.f;
    float acc[AK_MAX_DV / AK_DC][AK_DC / 8];
#pragma unroll
    for (int i = 0; i < AK_MAX_DV / AK_DC; ++i)
#pragma unroll
        for (int j = 0; j < AK_DC / 8; ++j) acc[i][j] = 0.f;

    const int* table = block_table + (size_t)s * max_pages;
    for (int k0 = kbeg; k0 < kend; k0 += AK_BN) {
        __syncthreads();
        if (tid < AK_BN) {
            const int kp = k0 + tid;
            int page = -1;
            if (kp < kend) {
                page = table[kp / ps];
                if (page >= num_pages) {
                    atomicCAS(&attention_kv_status_word, 0, 1);
                    page = -1;
                }
            }
            page_of[tid] = page;
        }
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int d0 = 0; d0 < Dk; d0 += AK_DC) {
            __syncthreads();
            for (int idx = tid; idx < AK_BN * AK_DC; idx += AK_THREADS) {
                const int kr = idx / AK_DC, d = idx - kr * AK_DC;
                const int page = page_of[kr];
                float kv = 0.f;
                if (page >= 0 && d0 + d < Dk) {
                    const size_t slot = ((size_t)page * Hkv + kvh) * ps + (k0 + kr) % ps;
                    kv = to_float(kc[slot * ldk + map * Dk + d0 + d]);
                }
                Cs[kr * (AK_DC + 1) + d] = kv;
            }
            __syncthreads();
            const int dn = min(AK_DC, Dk - d0);
            for (int d = 0; d < dn; ++d) {
                const float qv = Qs[r * ldq_s + d0 + d];
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[j] += qv * Cs[(c0 + 8 * j) * (AK_DC + 1) + d];
            }
        }
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kp = k0 + c0 + 8 * j;
            const bool vis = row_valid && kp <= my_pos && (window <= 0 || my_pos - kp < window);
            float sv = sc[j] * scale;
            if (softcap > 0.f) sv = softcap * tanhf(sv / softcap);
            sc[j] = vis ? sv : -INFINITY;
            tmax = fmaxf(tmax, sc[j]);
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        const float m_new = fmaxf(m, tmax);
        float alpha = 1.f, psum = 0.f;
        float p[4] = {0.f, 0.f, 0.f, 0.f};
        if (m_new != -INFINITY) {
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                p[j] = (sc[j] == -INFINITY) ? 0.f : expf(sc[j] - m_new);
                psum += p[j];
            }
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int j = 0; j < 4; ++j) Ps[r * (AK_BN + 1) + c0 + 8 * j] = p[j];

#pragma unroll
        for (int vci = 0; vci < AK_MAX_DV / AK_DC; ++vci) {
            if (vci < nvc) {
                const int d0 = vci * AK_DC;
                __syncthreads();                       // the chunk buffer is free; Ps is written
                for (int idx = tid; idx < AK_BN * AK_DC; idx += AK_THREADS) {
                    const int kr = idx / AK_DC, d = idx - kr * AK_DC;
                    const int page = page_of[kr];
                    float vv = 0.f;
                    if (page >= 0 && d0 + d < Dv) {
                        const size_t slot = ((size_t)page * Hkv + kvh) * ps + (k0 + kr) % ps;
                        vv = to_float(vc[slot * ldv + d0 + d]);
                    }
                    Cs[kr * (AK_DC + 1) + d] = vv;
                }
                __syncthreads();
#pragma unroll
                for (int j = 0; j < AK_DC / 8; ++j) acc[vci][j] *= alpha;
                for (int k = 0; k < AK_BN; ++k) {
                    const float pv = Ps[r * (AK_BN + 1) + k];
#pragma unroll
                    for (int j = 0; j < AK_DC / 8; ++j) acc[vci][j] += pv * Cs[k * (AK_DC + 1) + c0 + 8 * j];
                }
            }
        }
    }

    if (row_valid) {
        const int rho = row0 + r;
        const int tl = rho / g, hg = rho - tl * g;
        const int head = (kvh * g + hg) * maps + map;
        if (sink != nullptr) l += (m == -INFINITY) ? 1.f : expf(sink[head] - m);
        float inv = l > 0.f ? 1.0f / l : 0.f;
        if (gate != nullptr) {
            const float z = to_float(gate[(size_t)(q0 + tl) * ldg + head]);
            inv *= 1.0f / (1.0f + expf(-z));
        }
        TO* o = out + (size_t)(q0 + tl) * ldo + (size_t)head * Dv;
#pragma unroll
        for (int vci = 0; vci < AK_MAX_DV / AK_DC; ++vci)
#pragma unroll
            for (int j = 0; j < AK_DC / 8; ++j) {
                const int c = vci * AK_DC + c0 + 8 * j;
                if (vci < nvc && c < Dv) o[c] = from_float<TO>(acc[vci][j] * inv);
            }
    }
}

template <typename T, typename TO>
static int launch_attention_kv(const T* q, int ldq, const T* kc, int ldk, int maps, const T* vc, int ldv, TO* out, int ldo,
                               const int* block_table, int max_pages, const int* cu_q,
                               const int* ctx_len, const int* tile_seq, const int* tile_row0,
                               int num_tiles, int H, int Hkv, int Dk, int Dv, int ps, int num_pages,
                               float scale, int window, const T* gate, int ldg, float softcap,
                               const float* sink, cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (softcap < 0.f || (sink != nullptr && maps != 1)) return SLB_ERR_BAD_ARG;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || Dk <= 0 || Dv <= 0 || ps <= 0 || max_pages <= 0 ||
        num_pages <= 0 || ldv < Dv || maps <= 0 || ldk < maps * Dk)
        return SLB_ERR_BAD_ARG;
    if (Dk > AK_MAX_DK || Dv > AK_MAX_DV || Hkv * maps > 65535) return SLB_ERR_TOO_LARGE;
    const size_t smem = ((size_t)AK_BM * (Dk + 1) + AK_BN * (AK_DC + 1) + AK_BM * (AK_BN + 1)) * sizeof(float);
    constexpr size_t SMEM_MAX =
        ((size_t)AK_BM * (AK_MAX_DK + 1) + AK_BN * (AK_DC + 1) + AK_BM * (AK_BN + 1)) * sizeof(float);
    static unsigned long long configured = 0;
    const int rc = slb_configure(&configured, attention_kv_kernel<T, TO>, SMEM_MAX);
    if (rc != 0) return rc;
    return slb_launch(attention_kv_kernel<T, TO>, dim3(num_tiles, Hkv * maps), dim3(AK_THREADS), smem, st, q, ldq,
                      kc, ldk, maps, vc, ldv, out, ldo, block_table, max_pages, cu_q, ctx_len, tile_seq, tile_row0,
                      H, Hkv, Dk, Dv, ps, num_pages, scale, window, gate, ldg, softcap, sink);
}

extern "C" {
int slb_attention_kv_tile_rows() { return AK_BM; }
int slb_attention_kv_f32(const float* q, int ldq, const float* kc, const float* vc, int ldv, float* out,
                         int ldo, const int* block_table, int max_pages, const int* cu_q,
                         const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                         int H, int Hkv, int Dk, int Dv, int ps, int num_pages, float scale, int window,
                         const float* gate, int ldg, float softcap, const float* sink, cudaStream_t st) {
    return launch_attention_kv<float, float>(q, ldq, kc, Dk, 1, vc, ldv, out, ldo, block_table, max_pages, cu_q,
                                      ctx_len, tile_seq, tile_row0, num_tiles, H, Hkv, Dk, Dv, ps,
                                      num_pages, scale, window, gate, ldg, softcap, sink, st);
}
int slb_attention_kv_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, int ldv, bf16* out,
                          int ldo, const int* block_table, int max_pages, const int* cu_q,
                          const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                          int H, int Hkv, int Dk, int Dv, int ps, int num_pages, float scale, int window,
                          const bf16* gate, int ldg, float softcap, const float* sink, cudaStream_t st) {
    return launch_attention_kv<bf16, bf16>(q, ldq, kc, Dk, 1, vc, ldv, out, ldo, block_table, max_pages, cu_q,
                                     ctx_len, tile_seq, tile_row0, num_tiles, H, Hkv, Dk, Dv, ps,
                                     num_pages, scale, window, gate, ldg, softcap, sink, st);
}
// several maps a head (see the top of the file); the results are float32 in both forms
int slb_attention_kv_maps_f32(const float* q, int ldq, const float* kc, int ldk, int maps, const float* vc, int ldv,
                              float* out, int ldo, const int* block_table, int max_pages, const int* cu_q,
                              const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                              int H, int Hkv, int Dk, int Dv, int ps, int num_pages, float scale, int window,
                              cudaStream_t st) {
    return launch_attention_kv<float, float>(q, ldq, kc, ldk, maps, vc, ldv, out, ldo, block_table, max_pages, cu_q,
                                             ctx_len, tile_seq, tile_row0, num_tiles, H, Hkv, Dk, Dv, ps,
                                             num_pages, scale, window, nullptr, 0, 0.f, nullptr, st);
}
int slb_attention_kv_maps_bf16(const bf16* q, int ldq, const bf16* kc, int ldk, int maps, const bf16* vc, int ldv,
                               float* out, int ldo, const int* block_table, int max_pages, const int* cu_q,
                               const int* ctx_len, const int* tile_seq, const int* tile_row0, int num_tiles,
                               int H, int Hkv, int Dk, int Dv, int ps, int num_pages, float scale, int window,
                               cudaStream_t st) {
    return launch_attention_kv<bf16, float>(q, ldq, kc, ldk, maps, vc, ldv, out, ldo, block_table, max_pages, cu_q,
                                            ctx_len, tile_seq, tile_row0, num_tiles, H, Hkv, Dk, Dv, ps,
                                            num_pages, scale, window, nullptr, 0, 0.f, nullptr, st);
}
}

// What happens to the projected queries, keys and values of a step between the product and the
// attention, for mixers that norm heads and rotate neighbouring pairs:
//
//   per query head and per key head (a "vector" of D elements of the product's row):
//     * RMS norm over its first `norm_dims` elements with a weight shared by the heads
//       (x / sqrt(mean(x^2) + eps) * w; 0: no norm);
//     * rotation of `rot_dims` elements starting at `rot_off`: element 2i is paired with element
//       2i + 1 (or, with `rot_half`, element i with element i + rot_dims / 2), the pair (u, v) at
//       position p becomes (u c - v s, v c + u s) with
//       c = mag cos(p f_i), s = mag sin(p f_i) (a table of frequencies, one factor on both);
//     * after the rotation, division of the first `unit_dims` elements by their root mean square
//       (no weight; 0: none);
//     * queries go to the q buffer -- head h at h * q_head_stride, without its first `q_skip`
//       elements (a latent attention replaces them by their product with a matrix and keeps the
//       rotated rest) --, keys into the request's page (block-table look-up here);
//   per value head (optional):
//     * v <- (1 - lambda) v + lambda v_first with the values another layer computed for the same
//       token (optional), or a copy of v kept for the layers that will ask for it;
//     * into the request's page.
//
// The same kernel serves a grouped-query attention (queries and keys normed over the whole head
// and rotated from element 0) and a latent attention (one "key" of latent + rotated part: norm
// over the latent, rotation of the rest; queries rotated from `rot_off` on, not normed).
// One block a token (and group of vectors), one warp a vector at a time; the token's sines and
// cosines are formed once a block; float32 arithmetic, angles in float32.
#include "common.cuh"

#define HP_WARPS 4
#define HP_MAX_D 1152

SLB_DEFINE_STATUS_WORD(head_prep_status_word, slb_head_prep_status)

struct HeadPrepArgs {
    const void* proj; int ld;
    int q_off, H, Dq, q_norm_dims, q_rot_off; const float* q_norm_w;
    int k_off, G, Dk, k_norm_dims, k_rot_off; const float* k_norm_w;
    int v_off, Dv;
    const float* lambda; const void* v_first; int ld_vf; void* v_keep; int ld_vk;
    const float* freq; int rot_dims; float rot_mag; float eps;
    const int* positions; const int* seq_of_token; const int* block_table;
    int max_pages, page_size, num_pages;
    void* q_out; int ldq; void* k_cache; void* v_cache;
    int q_head_stride, q_skip;
    int rot_half, q_unit_dims, k_unit_dims;
};

template <typename T>
__global__ void __launch_bounds__(HP_WARPS * 32) head_prep_kernel(const HeadPrepArgs a) {
    extern __shared__ float hp_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int maxd = max(max(a.Dq, a.Dk), a.Dv);
    float* buf = hp_smem + (size_t)warp * maxd;
    float* cs_tab = hp_smem + (size_t)HP_WARPS * maxd;     // cos and sin of the token's angles, once a block
    float* sn_tab = cs_tab + a.rot_dims / 2;
    const T* row = reinterpret_cast<const T*>(a.proj) + (size_t)t * a.ld;
    const int pos = a.positions[t];
    for (int i = threadIdx.x; i < a.rot_dims / 2; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * a.freq[i], &sn, &cs);
        cs_tab[i] = cs * a.rot_mag;
        sn_tab[i] = sn * a.rot_mag;
    }
    __syncthreads();
    // where this token's key and value go
    long long slot = -1;
    if (a.k_cache != nullptr || a.v_cache != nullptr) {
        const int page = a.block_table[(size_t)a.seq_of_token[t] * a.max_pages + pos / a.page_size];
        if (page >= a.num_pages) {
            if (lane == 0) atomicCAS(&head_prep_status_word, 0, 1);
        } else if (page >= 0) {
            slot = (long long)page * a.G * a.page_size + pos % a.page_size;
        }
    }
    const int nv = a.v_off >= 0 ? a.G : 0;
    const int units = a.H + a.G + nv;
    // (grid y: groups of HP_WARPS vectors, so that a step of few tokens still fills the device)
    for (int u = blockIdx.y * HP_WARPS + warp; u < units; u += gridDim.y * HP_WARPS) {
        const T* src;
        T* dst = nullptr;
        int D, norm_dims = 0, rot_off = 0, unit_dims = 0;
        const float* nw = nullptr;
        bool rotate = a.rot_dims > 0;
        int vhead = -1, skip = 0;
        if (u < a.H) {
            D = a.Dq; norm_dims = a.q_norm_dims; nw = a.q_norm_w; rot_off = a.q_rot_off; unit_dims = a.q_unit_dims;
            src = row + a.q_off + (size_t)u * D;
            dst = reinterpret_cast<T*>(a.q_out) + (size_t)t * a.ldq + (size_t)u * a.q_head_stride;
            skip = a.q_skip;
        } else if (u < a.H + a.G) {
            const int g = u - a.H;
            D = a.Dk; norm_dims = a.k_norm_dims; nw = a.k_norm_w; rot_off = a.k_rot_off; unit_dims = a.k_unit_dims;
            src = row + a.k_off + (size_t)g * D;
            if (a.k_cache != nullptr && slot >= 0)
                dst = reinterpret_cast<T*>(a.k_cache) + (size_t)(slot + (long long)g * a.page_size) * D;
        } else {
            vhead = u - a.H - a.G;
            D = a.Dv; rotate = false;
            src = row + a.v_off + (size_t)vhead * D;
            if (a.v_cache != nullptr && slot >= 0)
                dst = reinterpret_cast<T*>(a.v_cache) + (size_t)(slot + (long long)vhead * a.page_size) * D;
        }
        __syncwarp();
        for (int i = lane; i < D; i += 32) buf[i] = to_float(src[i]);
        __syncwarp();
        if (vhead >= 0) {
            if (a.v_keep != nullptr) {
                T* keep = reinterpret_cast<T*>(a.v_keep) + (size_t)t * a.ld_vk + (size_t)vhead * D;
                for (int i = lane; i < D; i += 32) keep[i] = from_float<T>(buf[i]);
            }
            if (a.v_first != nullptr) {
                const float lam = a.lambda[0];
                const T* vf = reinterpret_cast<const T*>(a.v_first) + (size_t)t * a.ld_vf + (size_t)vhead * D;
                for (int i = lane; i < D; i += 32) buf[i] = (1.0f - lam) * buf[i] + lam * to_float(vf[i]);
            }
        } else {
            if (norm_dims > 0) {
                float ss = 0.f;
                for (int i = lane; i < norm_dims; i += 32) ss += buf[i] * buf[i];
                ss = warp_sum(ss);
                const float r = 1.0f / sqrtf(ss / (float)norm_dims + a.eps);
                for (int i = lane; i < norm_dims; i += 32) buf[i] = buf[i] * r * (nw != nullptr ? nw[i] : 1.f);
            }
            if (rotate) {
                __syncwarp();                          // (the norm wrote elements other lanes rotate)
                const int half = a.rot_dims / 2;
                for (int i = lane; i < half; i += 32) {
                    const float sn = sn_tab[i], cs = cs_tab[i];
                    const int ix = a.rot_half ? rot_off + i : rot_off + 2 * i;
                    const int iy = a.rot_half ? rot_off + i + half : rot_off + 2 * i + 1;
                    const float x = buf[ix], y = buf[iy];
                    buf[ix] = x * cs - y * sn;
                    buf[iy] = y * cs + x * sn;
                }
            }
            if (unit_dims > 0) {
                __syncwarp();
                float ss = 0.f;
                for (int i = lane; i < unit_dims; i += 32) ss += buf[i] * buf[i];
                ss = warp_sum(ss);
                const float r = 1.0f / sqrtf(ss / (float)unit_dims + a.eps);
                for (int i = lane; i < unit_dims; i += 32) buf[i] *= r;
            }
        }
        __syncwarp();
        if (dst != nullptr)
            for (int i = skip + lane; i < D; i += 32) dst[i - skip] = from_float<T>(buf[i]);
    }
}

// out = x * sigmoid(gate), float32 arithmetic; one gate value per `group` neighbouring elements
// (1: element by element; a head's size: one number a head).
template <typename T>
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(const T* __restrict__ x, int ldx,
                                                           const T* __restrict__ gate, int ldg,
                                                           T* __restrict__ out, int ldo, int N, int group) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < N; c += blockDim.x) {
        const float z = to_float(gate[t * ldg + c / group]);
        out[t * ldo + c] = from_float<T>(to_float(x[t * ldx + c]) / (1.0f + expf(-z)));
    }
}

template <typename T>
static int launch_head_prep(const HeadPrepArgs& a, int num_tokens, cudaStream_t st) {
    if (num_tokens <= 0) return 0;
    const int maxd = a.Dq > a.Dk ? (a.Dq > a.Dv ? a.Dq : a.Dv) : (a.Dk > a.Dv ? a.Dk : a.Dv);
    if (a.H < 0 || a.G < 0 || a.Dq < 0 || a.Dk < 0 || maxd <= 0 || (a.rot_dims & 1)) return SLB_ERR_BAD_ARG;
    if (maxd > HP_MAX_D) return SLB_ERR_TOO_LARGE;
    if (a.rot_dims > 0 && (a.freq == nullptr || (a.H > 0 && a.q_rot_off + a.rot_dims > a.Dq) ||
                           (a.G > 0 && a.k_rot_off + a.rot_dims > a.Dk)))
        return SLB_ERR_BAD_ARG;
    if (a.q_norm_dims > a.Dq || a.k_norm_dims > a.Dk || a.q_skip < 0 || a.q_skip > a.Dq) return SLB_ERR_BAD_ARG;
    if (a.q_unit_dims < 0 || a.q_unit_dims > a.Dq || a.k_unit_dims < 0 || a.k_unit_dims > a.Dk) return SLB_ERR_BAD_ARG;
    if ((a.k_cache != nullptr || a.v_cache != nullptr) && (a.block_table == nullptr || a.page_size <= 0))
        return SLB_ERR_BAD_ARG;
    const size_t smem = ((size_t)HP_WARPS * maxd + a.rot_dims) * sizeof(float);
    const int units = a.H + a.G + (a.v_off >= 0 ? a.G : 0);
    const int gy = num_tokens < 512 ? (units + HP_WARPS - 1) / HP_WARPS : 1;
    return slb_launch(head_prep_kernel<T>, dim3(num_tokens, gy), dim3(HP_WARPS * 32), smem, st, a);
}

extern "C" {
int slb_head_prep_f32(const HeadPrepArgs* a, int num_tokens, cudaStream_t st) {
    return launch_head_prep<float>(*a, num_tokens, st);
}
int slb_head_prep_bf16(const HeadPrepArgs* a, int num_tokens, cudaStream_t st) {
    return launch_head_prep<bf16>(*a, num_tokens, st);
}
int slb_sigmoid_gate_f32(const float* x, int ldx, const float* gate, int ldg, float* out, int ldo, int T,
                         int N, int group, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (group <= 0) return SLB_ERR_BAD_ARG;
    return slb_launch(sigmoid_gate_kernel<float>, dim3(T), dim3(256), 0, st, x, ldx, gate, ldg, out, ldo, N, group);
}
int slb_sigmoid_gate_bf16(const bf16* x, int ldx, const bf16* gate, int ldg, bf16* out, int ldo, int T,
                          int N, int group, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (group <= 0) return SLB_ERR_BAD_ARG;
    return slb_launch(sigmoid_gate_kernel<bf16>, dim3(T), dim3(256), 0, st, x, ldx, gate, ldg, out, ldo, N, group);
}
}

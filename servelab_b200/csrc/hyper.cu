// Kernels around a residual that is kept as several parallel streams (hyper-connections), the
// RMS norm of an embedding, and the norm + gate that follows a head-wise mixer.
//
//   embed_norm_streams   out[t][s][:] = rmsnorm(table[ids[t]]) * w for s = 0..n-1 (w null: the
//                        embedding itself), float32: gather, norm and the copies in one pass.
//   hyper_mix_norm       with X [T][n][w] the float32 streams: an update y [T][w] that a sublayer
//                        left is folded in, X_t <- sum_s M[s][t] X_s + b[t] y (all streams at once
//                        from the old ones; M indexed [from][to]), then the next reader's input
//                        u = sum_s a[s] X_s (a null: the plain sum) is RMS-normed with a weight
//                        (null: u itself) into rows of the compute dtype.  With a row selection
//                        only those rows are produced and X is left as it is.  Each step optional.
//   group_norm_gate      y = x / sqrt(mean_group(x^2) + eps) * w * factor * act(gate) over groups of
//                        neighbouring elements (a head, or the whole row), where x is a float32 row
//                        or the difference a_1 - lambda a_2 of two maps stored side by side
//                        ([group][2][size]); w and gate optional; act: sigmoid or SiLU.
//
// All arithmetic float32; sums over a row run in an order that depends only on the row's size.
#include "common.cuh"

#define HY_MAX_STREAMS 8

template <typename T>
__global__ void __launch_bounds__(256) embed_norm_streams_kernel(
    const int* __restrict__ ids, const T* __restrict__ table, const float* __restrict__ w, float eps,
    float* __restrict__ out, int n, int h, int vocab) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * h;
    float rstd = 1.f;
    if (w != nullptr) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < h; c += blockDim.x) {
            const float x = ok ? to_float(row[c]) : 0.f;
            ss += x * x;
        }
        ss = block_sum(ss, scratch);
        rstd = 1.0f / sqrtf(ss / (float)h + eps);
    }
    float* o = out + (size_t)t * n * h;
    for (int c = threadIdx.x; c < h; c += blockDim.x) {
        float x = ok ? to_float(row[c]) : 0.f;
        if (w != nullptr) x = x * rstd * w[c];
        for (int s = 0; s < n; ++s) o[(size_t)s * h + c] = x;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) hyper_mix_norm_kernel(
    float* __restrict__ X, const T* __restrict__ y, int ldy, const float* __restrict__ M,
    const float* __restrict__ b, const float* __restrict__ a, const float* __restrict__ norm_w, float eps,
    T* __restrict__ out, int ldo, const int* __restrict__ row_map, int n, int w) {
    extern __shared__ float hy_u[];               // [w]: the reader's input before the norm
    __shared__ float scratch[33];
    __shared__ float sM[HY_MAX_STREAMS * HY_MAX_STREAMS], sb[HY_MAX_STREAMS], sa[HY_MAX_STREAMS];
    // (the small vectors are weights: read before the wait for the preceding kernel)
    for (int i = threadIdx.x; i < n * n; i += blockDim.x) sM[i] = M != nullptr ? M[i] : (i / n == i % n ? 1.f : 0.f);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        sb[i] = b != nullptr ? b[i] : 1.f;
        sa[i] = a != nullptr ? a[i] : 1.f;
    }
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    const int r = blockIdx.x;
    const int t = row_map != nullptr ? row_map[r] : r;
    float* x = X + (size_t)t * n * w;
    const bool fold = y != nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < w; c += blockDim.x) {
        float old[HY_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HY_MAX_STREAMS; ++s) old[s] = s < n ? x[(size_t)s * w + c] : 0.f;
        float u = 0.f;
        if (fold) {
            const float yv = to_float(y[(size_t)t * ldy + c]);
#pragma unroll
            for (int to = 0; to < HY_MAX_STREAMS; ++to) {
                if (to < n) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < HY_MAX_STREAMS; ++s)
                        if (s < n) v = fmaf(sM[s * n + to], old[s], v);
                    v = fmaf(sb[to], yv, v);
                    if (row_map == nullptr) x[(size_t)to * w + c] = v;
                    u = fmaf(sa[to], v, u);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < HY_MAX_STREAMS; ++s)
                if (s < n) u = fmaf(sa[s], old[s], u);
        }
        hy_u[c] = u;
        ss += u * u;
    }
    if (out == nullptr) return;
    float rstd = 1.f;
    if (norm_w != nullptr) {
        ss = block_sum(ss, scratch);
        rstd = 1.0f / sqrtf(ss / (float)w + eps);
    }
    T* o = out + (size_t)r * ldo;
    for (int c = threadIdx.x; c < w; c += blockDim.x)     // (a thread reads back what it wrote itself)
        o[c] = from_float<T>(norm_w != nullptr ? hy_u[c] * rstd * norm_w[c] : hy_u[c]);
}

// a warp a (token, group)
template <typename T>
__global__ void __launch_bounds__(128) group_norm_gate_kernel(
    const float* __restrict__ in, int ldi, int maps, const float* __restrict__ lam,
    const float* __restrict__ w, float eps, float factor, const T* __restrict__ gate, int ldg, int gate_act,
    T* __restrict__ out, int ldo, int T_, int groups, int size) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * 4 + warp;
    if (unit >= (long long)T_ * groups) return;
    const int t = (int)(unit / groups), g = (int)(unit - (long long)t * groups);
    const float* x1 = in + (size_t)t * ldi + (size_t)g * maps * size;
    const float* x2 = x1 + size;
    const float l = maps == 2 ? lam[0] : 0.f;
    float ss = 0.f;
    for (int c = lane; c < size; c += 32) {
        const float x = maps == 2 ? x1[c] - l * x2[c] : x1[c];
        ss += x * x;
    }
    ss = warp_sum(ss);
    const float rstd = factor / sqrtf(ss / (float)size + eps);
    for (int c = lane; c < size; c += 32) {
        float x = (maps == 2 ? x1[c] - l * x2[c] : x1[c]) * rstd;
        const int col = g * size + c;
        if (w != nullptr) x *= w[col];
        if (gate != nullptr) {
            const float z = to_float(gate[(size_t)t * ldg + col]);
            const float sg = 1.0f / (1.0f + expf(-z));
            x *= gate_act == 2 ? z * sg : sg;
        }
        out[(size_t)t * ldo + col] = from_float<T>(x);
    }
}

template <typename T>
static int launch_hyper_mix_norm(float* X, const T* y, int ldy, const float* M, const float* b, const float* a,
                                 const float* norm_w, float eps, T* out, int ldo, const int* row_map, int rows,
                                 int n, int w, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (n <= 0 || w <= 0 || (y != nullptr && ldy < w) || (out != nullptr && ldo < w)) return SLB_ERR_BAD_ARG;
    if (n > HY_MAX_STREAMS || (size_t)w * sizeof(float) > 200 * 1024) return SLB_ERR_TOO_LARGE;
    const size_t smem = (size_t)w * sizeof(float);
    static unsigned long long configured = 0;
    if (smem > 48 * 1024) {
        const int rc = slb_configure(&configured, hyper_mix_norm_kernel<T>, 200 * 1024);
        if (rc != 0) return rc;
    }
    int threads = ((w + 3) / 4 + 31) / 32 * 32;
    threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
    return slb_launch(hyper_mix_norm_kernel<T>, dim3(rows), dim3(threads), smem, st, X, y, ldy, M, b, a, norm_w,
                      eps, out, ldo, row_map, n, w);
}

template <typename T>
static int launch_group_norm_gate(const float* in, int ldi, int maps, const float* lam, const float* w, float eps,
                                  float factor, const T* gate, int ldg, int gate_act, T* out, int ldo, int T_,
                                  int groups, int size, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (groups <= 0 || size <= 0 || (maps != 1 && maps != 2) || (maps == 2 && lam == nullptr) ||
        gate_act < 0 || gate_act > 2 || (gate != nullptr && gate_act == 0))
        return SLB_ERR_BAD_ARG;
    const long long units = (long long)T_ * groups;
    if ((units + 3) / 4 > 2147483647LL) return SLB_ERR_TOO_LARGE;
    return slb_launch(group_norm_gate_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, st, in, ldi, maps,
                      lam, w, eps, factor, gate, ldg, gate_act, out, ldo, T_, groups, size);
}

// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w over the first n columns of every row (a latent
// inside a wider projection); a block a row, float32 arithmetic.
template <typename T>
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(const T* __restrict__ x, int ldx,
                                                            const float* __restrict__ w, float eps,
                                                            T* __restrict__ out, int ldo, int n) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const T* row = x + (size_t)blockIdx.x * ldx;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = to_float(row[c]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x)
        out[(size_t)blockIdx.x * ldo + c] = from_float<T>(to_float(row[c]) * rstd * (w != nullptr ? w[c] : 1.f));
}

// out[t] = factor * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb): the results of two branches
// that read the same input, each RMS-normed over the row with a weight of its own, summed.
// a and b float32 [T, n]; a block a row; float32 arithmetic.
template <typename T>
__global__ void __launch_bounds__(256) norm_sum2_kernel(const float* __restrict__ a, int lda,
                                                        const float* __restrict__ b, int ldb,
                                                        const float* __restrict__ wa, const float* __restrict__ wb,
                                                        float eps, float factor, T* __restrict__ out, int ldo, int n) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const float* ra = a + (size_t)blockIdx.x * lda;
    const float* rb = b + (size_t)blockIdx.x * ldb;
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        sa += ra[c] * ra[c];
        sb += rb[c] * rb[c];
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float fa = 1.0f / sqrtf(sa / (float)n + eps), fb = 1.0f / sqrtf(sb / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x)
        out[(size_t)blockIdx.x * ldo + c] = from_float<T>(factor * (ra[c] * fa * wa[c] + rb[c] * fb * wb[c]));
}

extern "C" {
int slb_rms_norm_rows_f32(const float* x, int ldx, const float* w, float eps, float* out, int ldo, int T, int n,
                          cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || ldx < n || ldo < n) return SLB_ERR_BAD_ARG;
    return slb_launch(rms_norm_rows_kernel<float>, dim3(T), dim3(n >= 1024 ? 256 : 128), 0, st, x, ldx, w, eps, out,
                      ldo, n);
}
int slb_rms_norm_rows_bf16(const bf16* x, int ldx, const float* w, float eps, bf16* out, int ldo, int T, int n,
                           cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || ldx < n || ldo < n) return SLB_ERR_BAD_ARG;
    return slb_launch(rms_norm_rows_kernel<bf16>, dim3(T), dim3(n >= 1024 ? 256 : 128), 0, st, x, ldx, w, eps, out,
                      ldo, n);
}
int slb_norm_sum2_f32(const float* a, int lda, const float* b, int ldb, const float* wa, const float* wb, float eps,
                      float factor, float* out, int ldo, int T, int n, cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || lda < n || ldb < n || ldo < n || wa == nullptr || wb == nullptr) return SLB_ERR_BAD_ARG;
    return slb_launch(norm_sum2_kernel<float>, dim3(T), dim3(256), 0, st, a, lda, b, ldb, wa, wb, eps, factor, out,
                      ldo, n);
}
int slb_norm_sum2_bf16(const float* a, int lda, const float* b, int ldb, const float* wa, const float* wb, float eps,
                       float factor, bf16* out, int ldo, int T, int n, cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || lda < n || ldb < n || ldo < n || wa == nullptr || wb == nullptr) return SLB_ERR_BAD_ARG;
    return slb_launch(norm_sum2_kernel<bf16>, dim3(T), dim3(256), 0, st, a, lda, b, ldb, wa, wb, eps, factor, out,
                      ldo, n);
}
int slb_hyper_max_streams() { return HY_MAX_STREAMS; }
int slb_embed_norm_streams_f32(const int* ids, const float* table, const float* w, float eps, float* out, int T,
                               int n, int h, int vocab, cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || h <= 0 || vocab <= 0) return SLB_ERR_BAD_ARG;
    return slb_launch(embed_norm_streams_kernel<float>, dim3(T), dim3(256), 0, st, ids, table, w, eps, out, n, h, vocab);
}
int slb_embed_norm_streams_bf16(const int* ids, const bf16* table, const float* w, float eps, float* out, int T,
                                int n, int h, int vocab, cudaStream_t st) {
    if (T <= 0) return 0;
    if (n <= 0 || h <= 0 || vocab <= 0) return SLB_ERR_BAD_ARG;
    return slb_launch(embed_norm_streams_kernel<bf16>, dim3(T), dim3(256), 0, st, ids, table, w, eps, out, n, h, vocab);
}
int slb_hyper_mix_norm_f32(float* X, const float* y, int ldy, const float* M, const float* b, const float* a,
                           const float* norm_w, float eps, float* out, int ldo, const int* row_map, int rows, int n,
                           int w, cudaStream_t st) {
    return launch_hyper_mix_norm<float>(X, y, ldy, M, b, a, norm_w, eps, out, ldo, row_map, rows, n, w, st);
}
int slb_hyper_mix_norm_bf16(float* X, const bf16* y, int ldy, const float* M, const float* b, const float* a,
                            const float* norm_w, float eps, bf16* out, int ldo, const int* row_map, int rows, int n,
                            int w, cudaStream_t st) {
    return launch_hyper_mix_norm<bf16>(X, y, ldy, M, b, a, norm_w, eps, out, ldo, row_map, rows, n, w, st);
}
int slb_group_norm_gate_f32(const float* in, int ldi, int maps, const float* lam, const float* w, float eps,
                            float factor, const float* gate, int ldg, int gate_act, float* out, int ldo, int T,
                            int groups, int size, cudaStream_t st) {
    return launch_group_norm_gate<float>(in, ldi, maps, lam, w, eps, factor, gate, ldg, gate_act, out, ldo, T, groups,
                                         size, st);
}
int slb_group_norm_gate_bf16(const float* in, int ldi, int maps, const float* lam, const float* w, float eps,
                             float factor, const bf16* gate, int ldg, int gate_act, bf16* out, int ldo, int T,
                             int groups, int size, cudaStream_t st) {
    return launch_group_norm_gate<bf16>(in, ldi, maps, lam, w, eps, factor, gate, ldg, gate_act, out, ldo, T, groups,
                                        size, st);
}
}

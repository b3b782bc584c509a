// Routed experts: the router's choice, the plan of a step (which rows each expert gets), the
// experts' products on CUDA cores, and the weighted sum.
//
//   slb_moe_route      scores = softmax(logits) in float32 per token; experts form `groups` equal
//                      groups of neighbours, a group's score is its largest score, only experts of
//                      the `keep` best groups can be chosen; the `top` largest scores among those
//                      are the choice (ties: the lower index); weight = score * route_scale
//                      (optionally divided by the sum of the chosen scores).
//   slb_moe_route_scored  the same with sigmoid scores, an offset per expert that enters the choice
//                      only, groups that score as the sum of their best few, and a constant in the
//                      denominator of the renormalised weights, each an argument.
//   slb_moe_plan       (token, choice) pairs sorted by expert: counts, offsets, the list, and the
//                      row tiles of the products (tile -> expert, first row), of a length that
//                      depends only on the number of pairs and experts (a fixed grid).
//   slb_moe_gate_up    act[pair] = silu(W_gate[e] x) * (W_up[e] x) for the pair's expert e;
//   slb_moe_down       y[pair] = W_down[e] act[pair], float32;
//   slb_moe_combine    out[t] = (shared[t]) + sum_k weight[t][k] * y[t * top + k], in the order k.
//
// Each output element of a product is a sum over k = 0..K-1 in that order (plain FFMA), and the
// combine adds a token's experts in the order of its choice, so a token's result does not depend
// on what else is in the batch.
#include "mma_util.cuh"

#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 32
#define MOE_BM 64
#define MOE_BN 64
#define MOE_BK 16

// ------------------------------------------------------------------- route
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
        }
    }
}

// One warp a token.  `score_fn` 0: scores = softmax(logits); 1: scores = sigmoid(logits).  The
// choice runs on choice scores c = score (+ correction[e], a learned offset that enters the choice
// only); a group's score is the sum of its `group_best` largest choice scores (1: its maximum);
// experts outside the `keep` best groups count as minus infinity (choice scores may be negative);
// the weights are the chosen experts' scores without the offset, divided by their sum + `norm_eps`
// with `renormalize`, times `route_scale`.  Ties: the lower index.
__global__ void __launch_bounds__(128) moe_route_kernel(
    const float* __restrict__ logits, int ldl, int T, int E, int groups, int keep, int top,
    float route_scale, int renormalize, int score_fn, const float* __restrict__ correction, int group_best,
    float norm_eps, int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float route_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* s = route_smem + (size_t)warp * (2 * E + 2 * groups);   // scores, choice scores,
    float* c = s + E;                                                // the groups' scores and marks
    float* gs = c + E;
    float* gmark = gs + groups;
    const float* z = logits + (size_t)t * ldl;
    if (score_fn == 0) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(z[e] - mx);
            s[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) s[e] *= inv;
    } else {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-z[e]));
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) c[e] = correction != nullptr ? s[e] + correction[e] : s[e];
    __syncwarp();
    const int per = E / groups;
    if (groups > 1) {
        for (int g = lane; g < groups; g += 32) {
            // the sum of the group's `group_best` largest choice scores (all of them if it has fewer)
            float total = 0.f;
            int prev_i = -1;
            float prev_v = INFINITY;
            const int take = group_best < per ? group_best : per;
            for (int r = 0; r < take; ++r) {
                float b = -INFINITY;
                int bi = -1;
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    const float v = c[e];
                    const bool after = v < prev_v || (v == prev_v && e > prev_i);   // not yet taken
                    if (after && (bi < 0 || v > b)) {
                        b = v;
                        bi = e;
                    }
                }
                if (bi < 0) break;
                total += b;
                prev_v = b;
                prev_i = bi;
            }
            gs[g] = total;
            gmark[g] = 0.f;
        }
        __syncwarp();
        for (int round = 0; round < keep; ++round) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gmark[g] == 0.f && (gs[g] > bv || (gs[g] == bv && g < bi) || bi == 0x7fffffff) && gs[g] == gs[g]) {
                    bv = gs[g];
                    bi = g;
                }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < groups) gmark[bi] = 1.f;   // (no group found: logits that are no numbers)
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gmark[e / per] == 0.f) c[e] = -INFINITY;
        __syncwarp();
    }
    float chosen_sum = 0.f;
    for (int round = 0; round < top; ++round) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (v > -INFINITY && (v > bv || (v == bv && e < bi) || bi == 0x7fffffff)) {
                bv = v;
                bi = e;
            }
        }
        warp_argmax(bv, bi);
        float w = 0.f;
        if (bi >= E) {                                     // nothing left to choose (logits that are no
            bi = 0;                                        // numbers, as the rows of a padded step may
        } else {                                           // hold): expert 0 with weight 0
            w = s[bi];
        }
        __syncwarp();
        if (lane == 0) {
            ids[(size_t)t * top + round] = bi;
            weights[(size_t)t * top + round] = w;
            if (w == w && c[bi] > -INFINITY) c[bi] = -INFINITY;      // taken
        }
        chosen_sum += w;
        __syncwarp();
    }
    if (lane < top) {
        float w = weights[(size_t)t * top + lane];
        if (renormalize) w /= (chosen_sum + norm_eps);
        weights[(size_t)t * top + lane] = w * route_scale;
    }
}

// ----------------------------------------------------------- router logits
// logits[t][e] = sum_k x[t][k] * w[e][k] in float32 (w float32, x float32 or bfloat16).  A block
// owns ROUTER_TOK tokens and one expert; its eight warps take an eighth of k each (lanes stride,
// coalesced) and the partial sums are added in a fixed order, so a token's logits do not depend
// on the batch.
#define ROUTER_TOK 4
template <typename T>
__global__ void __launch_bounds__(256) router_logits_kernel(const T* __restrict__ x, int ldx,
                                                            const float* __restrict__ w, int ldw,
                                                            float* __restrict__ logits, int ldl, int M,
                                                            int E, int K) {
    __shared__ float part[8][ROUTER_TOK];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * ROUTER_TOK;
    const int e = blockIdx.y;
    const T* xr[ROUTER_TOK];
#pragma unroll
    for (int i = 0; i < ROUTER_TOK; ++i) xr[i] = x + (size_t)min(t0 + i, M - 1) * ldx;
    const float* wr = w + (size_t)e * ldw;
    const int per = (K + 7) / 8;
    const int k_end = min(K, (warp + 1) * per);
    float acc[ROUTER_TOK];
#pragma unroll
    for (int i = 0; i < ROUTER_TOK; ++i) acc[i] = 0.f;
#pragma unroll 4
    for (int k = warp * per + lane; k < k_end; k += 32) {
        const float wv = wr[k];
#pragma unroll
        for (int i = 0; i < ROUTER_TOK; ++i) acc[i] = fmaf(to_float(xr[i][k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < ROUTER_TOK; ++i) {
        const float v = warp_sum(acc[i]);
        if (lane == 0) part[warp][i] = v;
    }
    __syncthreads();
    if (threadIdx.x < ROUTER_TOK && t0 + threadIdx.x < M) {
        float v = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) v += part[j][threadIdx.x];
        logits[(size_t)(t0 + threadIdx.x) * ldl + e] = v;
    }
}

// -------------------------------------------------------------------- plan
// One block.  plan = [counts E | offsets E + 1 | cursor E | tile_expert NT | tile_row0 NT |
// sorted P] (int32), NT = ceil(P / MOE_BM) + E.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, int P, int E,
                                                        int num_tiles, int* __restrict__ plan) {
    pdl_wait();
    pdl_launch_dependents();
    int* counts = plan;
    int* offsets = plan + E;
    int* cursor = offsets + E + 1;
    int* tile_expert = cursor + E;
    int* tile_row0 = tile_expert + num_tiles;
    int* sorted = tile_row0 + num_tiles;
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) counts[e] = 0;
    for (int i = tid; i < num_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int p = tid; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int off = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = off;
            cursor[e] = off;
            const int n = counts[e];
            for (int r0 = 0; r0 < n; r0 += MOE_BM, ++tile) {
                tile_expert[tile] = e;
                tile_row0[tile] = r0;
            }
            off += n;
        }
        offsets[E] = off;
    }
    __syncthreads();
    // (a product's result is written per pair, so the order within an expert changes no value)
    for (int p = tid; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e < 0 || e >= E) continue;
        sorted[atomicAdd(&cursor[e], 1)] = p;
    }
}

// ---------------------------------------------------------------- products
// MODE 0: gate|up with the activation: A rows are x[pair / top], W = w_gu[e] ([2 I, K]: I gate
// rows, then I up rows), C = act[pair][I].  MODE 1: down: A rows are act[pair], W = w_down[e]
// ([N, K = I]), C = y[pair][N] float32.
template <typename T, typename TC, int MODE>
__global__ void __launch_bounds__(256) moe_product_kernel(
    const T* __restrict__ A, int lda, const T* __restrict__ W, long long w_expert_stride, int ldw,
    TC* __restrict__ C, int ldc, const int* __restrict__ plan, int E, int num_tiles, int P, int top,
    int N, int K) {
    __shared__ __align__(16) float As[MOE_BK][MOE_BM + 4];
    __shared__ __align__(16) float Ws[MOE_BK][MOE_BN + 4];
    __shared__ __align__(16) float Us[MODE == 0 ? MOE_BK : 1][MOE_BN + 4];
    __shared__ int rows[MOE_BM];
    pdl_wait();
    const int* counts = plan;
    const int* offsets = plan + E;
    const int* tile_expert = offsets + E + 1 + E;
    const int* tile_row0 = tile_expert + num_tiles;
    const int* sorted = tile_row0 + num_tiles;
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    const int r0 = tile_row0[blockIdx.y];
    const int nrows = min(MOE_BM, counts[e] - r0);
    const int tid = threadIdx.x;
    if (tid < MOE_BM) rows[tid] = tid < nrows ? sorted[offsets[e] + r0 + tid] : -1;
    __syncthreads();
    const T* We = W + (size_t)e * w_expert_stride;
    const int ty = tid >> 4, tx = tid & 15;
    const int n0 = blockIdx.x * MOE_BN;
    float acc[4][4], acu[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = acu[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int row = idx >> 4, kk = idx & 15;
            const int gk = k0 + kk, gn = n0 + row;
            const int pr = rows[row];
            float av = 0.f;
            if (pr >= 0 && gk < K) av = to_float(A[(size_t)(MODE == 0 ? pr / top : pr) * lda + gk]);
            As[kk][row] = av;
            const bool in = gn < N && gk < K;
            Ws[kk][row] = in ? to_float(We[(size_t)gn * ldw + gk]) : 0.f;
            if (MODE == 0) Us[kk][row] = in ? to_float(We[(size_t)(N + gn) * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            if (MODE == 0) {
                const float4 u = *reinterpret_cast<const float4*>(&Us[kk][tx * 4]);
                const float uv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acu[i][j] = fmaf(av[i], uv[j], acu[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int pr = rows[ty * 4 + i];
        if (pr < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (MODE == 0) {
                // the gate and the up value are rounded to the activations' type first, as two
                // separate products would leave them
                const float gte = to_float(from_float<T>(v)), up = to_float(from_float<T>(acu[i][j]));
                v = gte / (1.0f + expf(-gte)) * up;
            }
            C[(size_t)pr * ldc + gn] = from_float<TC>(v);
        }
    }
}

// ------------------------------------------------- products on tensor cores
// The same two products in bfloat16 on mma.sync (m16n8k16, float32 accumulation): a block owns
// 64 sorted rows of one expert and 64 output columns (MODE 0: 64 gate columns AND their 64 up
// columns, the activation in the epilogue), a warp 16 rows; A rows (gathered by the plan) and W
// rows arrive by 16-byte cp.async through a two-stage ring of 32-element k-blocks.  Rows, K and
// the leading dimensions must be multiples of 8 elements.
#define MM_BM 64
#define MM_BN 64
#define MM_BK 32
#define MM_LD (MM_BK + 8)

template <int MODE>
__global__ void __launch_bounds__(128) moe_product_mma_kernel(
    const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, long long w_expert_stride, int ldw,
    void* __restrict__ Cv, int ldc, const int* __restrict__ plan, int E, int num_tiles, int top, int N,
    int K) {
    using namespace slb_mma;
    __shared__ __align__(16) bf16 As[2][MM_BM][MM_LD];
    __shared__ __align__(16) bf16 Ws[2][MM_BN][MM_LD];
    __shared__ __align__(16) bf16 Us[MODE == 0 ? 2 : 1][MODE == 0 ? MM_BN : 1][MM_LD];
    __shared__ int rows[MM_BM];
    pdl_wait();
    const int* counts = plan;
    const int* offsets = plan + E;
    const int* tile_expert = offsets + E + 1 + E;
    const int* tile_row0 = tile_expert + num_tiles;
    const int* sorted = tile_row0 + num_tiles;
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    const int r0 = tile_row0[blockIdx.y];
    const int nrows = min(MM_BM, counts[e] - r0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MM_BM) rows[tid] = tid < nrows ? sorted[offsets[e] + r0 + tid] : -1;
    __syncthreads();
    const bf16* We = W + (size_t)e * w_expert_stride;
    const int n0 = blockIdx.x * MM_BN;

    auto load = [&](int stage, int k0) {
        // 64 rows x 4 chunks of 8 elements for each of A, W (and U)
        for (int idx = tid; idx < MM_BM * 4; idx += 128) {
            const int r = idx >> 2, c = idx & 3;
            const int gk = k0 + c * 8;
            const int pr = rows[r];
            const bool oka = pr >= 0 && gk < K;
            cp_async16(&As[stage][r][c * 8], A + (oka ? (size_t)(MODE == 0 ? pr / top : pr) * lda + gk : 0), oka);
            const bool okw = n0 + r < N && gk < K;
            cp_async16(&Ws[stage][r][c * 8], We + (okw ? (size_t)(n0 + r) * ldw + gk : 0), okw);
            if (MODE == 0)
                cp_async16(&Us[stage][r][c * 8], We + (okw ? (size_t)(N + n0 + r) * ldw + gk : 0), okw);
        }
    };

    float acc[MM_BN / 8][4], acu[MODE == 0 ? MM_BN / 8 : 1][4];
#pragma unroll
    for (int j = 0; j < MM_BN / 8; ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[j][x] = 0.f;
#pragma unroll
    for (int j = 0; j < (MODE == 0 ? MM_BN / 8 : 1); ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) acu[j][x] = 0.f;

    const int nk = (K + MM_BK - 1) / MM_BK;
    load(0, 0);
    cp_async_commit();
    const bool active = warp * 16 < nrows;
    for (int kb = 0; kb < nk; ++kb) {
        if (kb + 1 < nk) {
            load((kb + 1) & 1, (kb + 1) * MM_BK);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int st = kb & 1;
        if (active) {
#pragma unroll
            for (int kk = 0; kk < MM_BK / 16; ++kk) {
                unsigned a[4];
                ldmatrix_x4(a, &As[st][warp * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
                for (int jp = 0; jp < MM_BN / 16; ++jp) {
                    unsigned b[4];
                    ldmatrix_x4(b, &Ws[st][jp * 16 + (lane >> 4) * 8 + (lane & 7)][kk * 16 + ((lane >> 3) & 1) * 8]);
                    mma_bf16(acc[2 * jp], a, b[0], b[1]);
                    mma_bf16(acc[2 * jp + 1], a, b[2], b[3]);
                    if (MODE == 0) {
                        ldmatrix_x4(b, &Us[st][jp * 16 + (lane >> 4) * 8 + (lane & 7)][kk * 16 + ((lane >> 3) & 1) * 8]);
                        mma_bf16(acu[2 * jp], a, b[0], b[1]);
                        mma_bf16(acu[2 * jp + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    if (!active) return;
    const int tig = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int pr = rows[warp * 16 + (lane >> 2) + 8 * h];
        if (pr < 0) continue;
#pragma unroll
        for (int j = 0; j < MM_BN / 8; ++j) {
            const int gn = n0 + j * 8 + tig * 2;
            if (gn >= N) continue;                        // (N is even: both columns exist or neither)
            float v0 = acc[j][2 * h], v1 = acc[j][2 * h + 1];
            if (MODE == 0) {
                const float g0 = __bfloat162float(__float2bfloat16_rn(v0)), g1 = __bfloat162float(__float2bfloat16_rn(v1));
                const float u0 = __bfloat162float(__float2bfloat16_rn(acu[j][2 * h]));
                const float u1 = __bfloat162float(__float2bfloat16_rn(acu[j][2 * h + 1]));
                v0 = g0 / (1.0f + expf(-g0)) * u0;
                v1 = g1 / (1.0f + expf(-g1)) * u1;
                *reinterpret_cast<unsigned*>(reinterpret_cast<bf16*>(Cv) + (size_t)pr * ldc + gn) = pack_bf16(v0, v1);
            } else {
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(Cv) + (size_t)pr * ldc + gn) = make_float2(v0, v1);
            }
        }
    }
}

// ----------------------------------------------------------------- combine
template <typename T, typename TY>
__global__ void __launch_bounds__(256) moe_combine_kernel(
    const TY* __restrict__ y, int ldy, const float* __restrict__ weights, const T* __restrict__ shared,
    int lds, T* __restrict__ out, int ldo, int top, int N) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < N; c += gridDim.y * blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) v += weights[(size_t)t * top + k] * to_float(y[((size_t)t * top + k) * ldy + c]);
        if (shared != nullptr) v += to_float(shared[(size_t)t * lds + c]);
        out[(size_t)t * ldo + c] = from_float<T>(v);
    }
}

static int moe_num_tiles(int P, int E) { return (P + MOE_BM - 1) / MOE_BM + E; }

template <typename T>
static int launch_moe_gate_up(const T* x, int ldx, const T* w_gu, int ldw, T* act, int lda,
                              const int* plan, int E, int P, int top, int I, int K, cudaStream_t st) {
    if (P <= 0) return 0;
    if (E <= 0 || top <= 0 || I <= 0 || K <= 0) return SLB_ERR_BAD_ARG;
    const int nt = moe_num_tiles(P, E);
    if (nt > 65535) return SLB_ERR_TOO_LARGE;
    return slb_launch(moe_product_kernel<T, T, 0>, dim3((I + MOE_BN - 1) / MOE_BN, nt), dim3(256), 0, st, x,
                      ldx, w_gu, (long long)2 * I * ldw, ldw, act, lda, plan, E, nt, P, top, I, K);
}

template <typename T>
static int launch_moe_down(const T* act, int lda, const T* w_down, int ldw, float* y, int ldy,
                           const int* plan, int E, int P, int top, int N, int I, cudaStream_t st) {
    if (P <= 0) return 0;
    if (E <= 0 || top <= 0 || I <= 0 || N <= 0) return SLB_ERR_BAD_ARG;
    const int nt = moe_num_tiles(P, E);
    if (nt > 65535) return SLB_ERR_TOO_LARGE;
    return slb_launch(moe_product_kernel<T, float, 1>, dim3((N + MOE_BN - 1) / MOE_BN, nt), dim3(256), 0, st,
                      act, lda, w_down, (long long)N * ldw, ldw, y, ldy, plan, E, nt, P, top, N, I);
}

template <int MODE>
static int launch_moe_mma(const bf16* A, int lda, const bf16* W, long long stride, int ldw, void* C, int ldc,
                          const int* plan, int E, int P, int top, int N, int K, cudaStream_t st) {
    if (P <= 0) return 0;
    if (E <= 0 || top <= 0 || N <= 0 || K <= 0 || K % 8 || lda % 8 || ldw % 8 || N % 2 || ldc % 2 ||
        ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || (stride % 8))
        return SLB_ERR_BAD_ARG;
    const int nt = moe_num_tiles(P, E);
    if (nt > 65535) return SLB_ERR_TOO_LARGE;
    return slb_launch(moe_product_mma_kernel<MODE>, dim3((N + MM_BN - 1) / MM_BN, nt), dim3(128), 0, st, A, lda,
                      W, stride, ldw, C, ldc, plan, E, nt, top, N, K);
}

extern "C" {
int slb_moe_gate_up_mma_bf16(const bf16* x, int ldx, const bf16* w_gu, int ldw, bf16* act, int lda,
                             const int* plan, int E, int P, int top, int I, int K, cudaStream_t st) {
    return launch_moe_mma<0>(x, ldx, w_gu, (long long)2 * I * ldw, ldw, act, lda, plan, E, P, top, I, K, st);
}
int slb_moe_down_mma_bf16(const bf16* act, int lda, const bf16* w_down, int ldw, float* y, int ldy,
                          const int* plan, int E, int P, int top, int N, int I, cudaStream_t st) {
    return launch_moe_mma<1>(act, lda, w_down, (long long)N * ldw, ldw, y, ldy, plan, E, P, top, N, I, st);
}
int slb_moe_tile_rows() { return MOE_BM; }
static int launch_moe_route(const float* logits, int ldl, int T, int E, int groups, int keep, int top,
                            float route_scale, int renormalize, int score_fn, const float* correction,
                            int group_best, float norm_eps, int* ids, float* weights, cudaStream_t st) {
    if (T <= 0) return 0;
    if (E <= 0 || groups <= 0 || E % groups != 0 || keep <= 0 || keep > groups || top <= 0 ||
        top > (E / groups) * keep || score_fn < 0 || score_fn > 1 || group_best < 1)
        return SLB_ERR_BAD_ARG;
    if (E > MOE_MAX_EXPERTS || top > MOE_MAX_TOP) return SLB_ERR_TOO_LARGE;
    const size_t smem = (size_t)4 * (2 * E + 2 * groups) * sizeof(float);
    return slb_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), smem, st, logits, ldl, T, E, groups,
                      keep, top, route_scale, renormalize, score_fn, correction, group_best, norm_eps, ids,
                      weights);
}
// the softmax router whose groups score as their best expert
int slb_moe_route(const float* logits, int ldl, int T, int E, int groups, int keep, int top,
                  float route_scale, int renormalize, int* ids, float* weights, cudaStream_t st) {
    return launch_moe_route(logits, ldl, T, E, groups, keep, top, route_scale, renormalize, 0, nullptr, 1, 0.f,
                            ids, weights, st);
}
// every choice of the route kernel as an argument
int slb_moe_route_scored(const float* logits, int ldl, int T, int E, int groups, int keep, int top,
                         float route_scale, int renormalize, int score_fn, const float* correction,
                         int group_best, float norm_eps, int* ids, float* weights, cudaStream_t st) {
    return launch_moe_route(logits, ldl, T, E, groups, keep, top, route_scale, renormalize, score_fn, correction,
                            group_best, norm_eps, ids, weights, st);
}
int slb_router_logits_f32(const float* x, int ldx, const float* w, int ldw, float* logits, int ldl, int M,
                          int E, int K, cudaStream_t st) {
    if (M <= 0 || E <= 0) return 0;
    if (K <= 0) return SLB_ERR_BAD_ARG;
    return slb_launch(router_logits_kernel<float>, dim3((M + ROUTER_TOK - 1) / ROUTER_TOK, E), dim3(256), 0, st, x,
                      ldx, w, ldw, logits, ldl, M, E, K);
}
int slb_router_logits_bf16(const bf16* x, int ldx, const float* w, int ldw, float* logits, int ldl, int M,
                           int E, int K, cudaStream_t st) {
    if (M <= 0 || E <= 0) return 0;
    if (K <= 0) return SLB_ERR_BAD_ARG;
    return slb_launch(router_logits_kernel<bf16>, dim3((M + ROUTER_TOK - 1) / ROUTER_TOK, E), dim3(256), 0, st, x,
                      ldx, w, ldw, logits, ldl, M, E, K);
}
int slb_moe_plan_ints(int P, int E) { return 4 * E + 1 + 2 * moe_num_tiles(P, E) + P; }
int slb_moe_plan(const int* ids, int P, int E, int* plan, cudaStream_t st) {
    if (P <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS) return SLB_ERR_BAD_ARG;
    return slb_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, st, ids, P, E, moe_num_tiles(P, E), plan);
}
int slb_moe_gate_up_f32(const float* x, int ldx, const float* w_gu, int ldw, float* act, int lda,
                        const int* plan, int E, int P, int top, int I, int K, cudaStream_t st) {
    return launch_moe_gate_up<float>(x, ldx, w_gu, ldw, act, lda, plan, E, P, top, I, K, st);
}
int slb_moe_gate_up_bf16(const bf16* x, int ldx, const bf16* w_gu, int ldw, bf16* act, int lda,
                         const int* plan, int E, int P, int top, int I, int K, cudaStream_t st) {
    return launch_moe_gate_up<bf16>(x, ldx, w_gu, ldw, act, lda, plan, E, P, top, I, K, st);
}
int slb_moe_down_f32(const float* act, int lda, const float* w_down, int ldw, float* y, int ldy,
                     const int* plan, int E, int P, int top, int N, int I, cudaStream_t st) {
    return launch_moe_down<float>(act, lda, w_down, ldw, y, ldy, plan, E, P, top, N, I, st);
}
int slb_moe_down_bf16(const bf16* act, int lda, const bf16* w_down, int ldw, float* y, int ldy,
                      const int* plan, int E, int P, int top, int N, int I, cudaStream_t st) {
    return launch_moe_down<bf16>(act, lda, w_down, ldw, y, ldy, plan, E, P, top, N, I, st);
}
int slb_moe_combine_f32(const float* y, int ldy, const float* weights, const float* shared, int lds,
                        float* out, int ldo, int T, int top, int N, cudaStream_t st) {
    if (T <= 0) return 0;
    return slb_launch(moe_combine_kernel<float, float>, dim3(T, T < 256 ? (N + 255) / 256 : 1), dim3(256), 0, st, y, ldy, weights, shared, lds,
                      out, ldo, top, N);
}
int slb_moe_combine_bf16(const float* y, int ldy, const float* weights, const bf16* shared, int lds,
                         bf16* out, int ldo, int T, int top, int N, cudaStream_t st) {
    if (T <= 0) return 0;
    return slb_launch(moe_combine_kernel<bf16, float>, dim3(T, T < 256 ? (N + 255) / 256 : 1), dim3(256), 0, st, y, ldy, weights, shared, lds,
                      out, ldo, top, N);
}
// the experts' rows in bfloat16 (a library product left them so)
int slb_moe_combine_bf16_rows(const bf16* y, int ldy, const float* weights, const bf16* shared, int lds,
                              bf16* out, int ldo, int T, int top, int N, cudaStream_t st) {
    if (T <= 0) return 0;
    return slb_launch(moe_combine_kernel<bf16, bf16>, dim3(T, T < 256 ? (N + 255) / 256 : 1), dim3(256), 0, st,
                      y, ldy, weights, shared, lds, out, ldo, top, N);
}
}

// Linear attention with a fixed decay per head, as a recurrence over a per-request state:
//
//     S_t = decay_h S_{t-1} + k_t v_t^T        (S: D x Dv per head, float32, kept in a state slot)
//     o_t = S_t^T q_t
//
// or, with `gate_z`, with a decay of its own for every token and key channel (the rows of S that
// belong to key channel d are multiplied by alpha_t[d] = sigmoid(z_t[d])^(1 / tau)):
//
//     S_t = diag(alpha_t) S_{t-1} + k_t v_t^T
//
// q, k and v are columns of one projected row per token.  Before they enter the recurrence the
// kernel applies, each optional: an activation (SiLU) on q, k and v; a rotation of the first
// `rot_dims` elements of every query and key head (element i with element i + rot_dims / 2, angle
// position * freq[i]); a factor on the keys.  Everything after the load is float32: activations,
// angles, the state, the products and the sums.  No softmax, no denominator.
//
// A block owns (request, head, 32 value columns); thread (part, column) keeps the state elements
// S[d][column] of its part's run of ceil(D / 8) neighbouring d in registers, so a token costs D / 8
// multiply-adds for the state and as many for the output (q and k are read from shared memory four
// at a time, the same address for a whole warp), and the eight parts of an output are added through
// shared memory in a fixed order.  Tokens of the request's portion are taken in
// order, eight at a time (their prepared q, k, v rows staged in shared memory).  The state is
// read from the request's slot at the start and written back at the end, so a request can be cut
// anywhere: the result of a token is bit-identical however the prompt is cut and whatever else is
// in the batch.  Steps of single tokens run the same kernel: then it is one read and one write of
// the state.
#include "decay_attention.cuh"

#define DA_EV 32
#define DA_PARTS 8
#define DA_TT 8
#define DA_MAX_D 256

// R: state rows a thread holds (head size / DA_PARTS, rounded up to 16 or 32): with 16 the kernel
// fits 64 registers, so four blocks an SM keep their state slices in flight.
template <typename T, int R>
__global__ void __launch_bounds__(DA_EV * DA_PARTS, R <= 16 ? 4 : 2) decay_attention_kernel(const DecayAttnArgs a) {
    extern __shared__ float da_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * DA_EV;
    const int q0 = a.cu_q[s];
    const int qlen = a.cu_q[s + 1] - q0;
    if (qlen <= 0) return;
    const int slot = a.state_slots[s];
    if (slot < 0 || slot >= a.num_slots) return;
    const int D = a.D, Dv = a.Dv;
    const int Dp = (D + DA_PARTS - 1) / DA_PARTS;          // state rows a part owns: d = p * Dp + i
    const int Dpad = (Dp + 3) / 4 * 4;                     // a part's q and k in shared memory, 16-byte aligned
    const int LD = DA_PARTS * Dpad;
    float* qs = da_smem;                         // [DA_TT][LD]: element d at (d / Dp) * Dpad + d % Dp, zeros between
    float* ks = qs + DA_TT * LD;                 // [DA_TT][LD]
    float* vs = ks + DA_TT * LD;                 // [DA_TT][DA_EV]
    float* part = vs + DA_TT * DA_EV;            // [DA_TT][DA_PARTS][DA_EV]
    float* as = part + DA_TT * DA_PARTS * DA_EV; // [DA_TT][LD]: the decays of a token's key channels (gated form)
    const bool gated = a.gate_z != nullptr;
    const int tid = threadIdx.x, p = tid >> 5, e = tid & 31;
    const int col = e0 + e;
    const bool live = col < Dv;
    const float dec = gated ? 1.f : a.decay[h];
    float* srow = a.state + (size_t)slot * (size_t)a.state_stride + (size_t)h * D * Dv;

    float st[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = p * Dp + i;
        st[i] = (live && i < Dp && d < D) ? srow[(size_t)d * Dv + col] : 0.f;
    }
    const T* proj = reinterpret_cast<const T*>(a.proj);
    for (int t0 = 0; t0 < qlen; t0 += DA_TT) {
        const int n = min(DA_TT, qlen - t0);
        for (int idx = tid; idx < n * LD; idx += DA_EV * DA_PARTS) {
            const int j = idx / LD, c = idx - j * LD;
            const int pp = c / Dpad, i = c - pp * Dpad;
            const int d = pp * Dp + i;
            float qv = 0.f, kv = 0.f, av = 1.f;            // (the padding multiplies state elements that stay 0)
            if (i < Dp && d < D) {
                const T* row = proj + (size_t)(q0 + t0 + j) * a.ld;
                const int pos = a.positions[q0 + t0 + j];
                qv = da_prepared(row + a.q_off + h * D, d, pos, a) * a.q_scale;
                kv = da_prepared(row + a.k_off + h * D, d, pos, a) * a.k_scale;
                if (gated) {
                    float z = a.gate_z[(size_t)(q0 + t0 + j) * a.ld_gate + h * D + d];
                    if (a.gate_bias != nullptr) z += a.gate_bias[h * D + d];
                    // log sigmoid(z) = min(z, 0) - log(1 + exp(-|z|))
                    av = expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * a.gate_inv_tau);
                }
            }
            qs[idx] = qv;
            ks[idx] = kv;
            if (gated) as[idx] = av;
        }
        for (int idx = tid; idx < n * DA_EV; idx += DA_EV * DA_PARTS) {
            const int j = idx / DA_EV, c = e0 + (idx - j * DA_EV);
            float v = 0.f;
            if (c < Dv) {
                v = to_float(proj[(size_t)(q0 + t0 + j) * a.ld + a.v_off + h * Dv + c]);
                if (a.act == 1) v = da_silu(v);
            }
            vs[idx] = v;
        }
        __syncthreads();
        for (int j = 0; j < n; ++j) {
            const float v = vs[j * DA_EV + e];
            const float4* qj = reinterpret_cast<const float4*>(qs + j * LD + p * Dpad);
            const float4* kj = reinterpret_cast<const float4*>(ks + j * LD + p * Dpad);
            float acc = 0.f;
            if (gated) {
                const float4* aj = reinterpret_cast<const float4*>(as + j * LD + p * Dpad);
#pragma unroll
                for (int i4 = 0; i4 < R / 4; ++i4) {
                    if (i4 * 4 < Dp) {
                        const float4 k4 = kj[i4], q4 = qj[i4], a4 = aj[i4];
                        st[4 * i4] = fmaf(a4.x, st[4 * i4], k4.x * v);
                        acc = fmaf(st[4 * i4], q4.x, acc);
                        st[4 * i4 + 1] = fmaf(a4.y, st[4 * i4 + 1], k4.y * v);
                        acc = fmaf(st[4 * i4 + 1], q4.y, acc);
                        st[4 * i4 + 2] = fmaf(a4.z, st[4 * i4 + 2], k4.z * v);
                        acc = fmaf(st[4 * i4 + 2], q4.z, acc);
                        st[4 * i4 + 3] = fmaf(a4.w, st[4 * i4 + 3], k4.w * v);
                        acc = fmaf(st[4 * i4 + 3], q4.w, acc);
                    }
                }
                part[(j * DA_PARTS + p) * DA_EV + e] = acc;
                continue;
            }
#pragma unroll
            for (int i4 = 0; i4 < R / 4; ++i4) {
                if (i4 * 4 < Dp) {                         // (the same for every thread)
                    const float4 k4 = kj[i4], q4 = qj[i4];
                    st[4 * i4] = fmaf(dec, st[4 * i4], k4.x * v);
                    acc = fmaf(st[4 * i4], q4.x, acc);
                    st[4 * i4 + 1] = fmaf(dec, st[4 * i4 + 1], k4.y * v);
                    acc = fmaf(st[4 * i4 + 1], q4.y, acc);
                    st[4 * i4 + 2] = fmaf(dec, st[4 * i4 + 2], k4.z * v);
                    acc = fmaf(st[4 * i4 + 2], q4.z, acc);
                    st[4 * i4 + 3] = fmaf(dec, st[4 * i4 + 3], k4.w * v);
                    acc = fmaf(st[4 * i4 + 3], q4.w, acc);
                }
            }
            part[(j * DA_PARTS + p) * DA_EV + e] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < n * DA_EV; idx += DA_EV * DA_PARTS) {
            const int j = idx / DA_EV, c = idx - j * DA_EV;
            if (e0 + c < Dv) {
                float o = 0.f;
#pragma unroll
                for (int pp = 0; pp < DA_PARTS; ++pp) o += part[(j * DA_PARTS + pp) * DA_EV + c];
                a.out[(size_t)(q0 + t0 + j) * a.ldo + h * Dv + e0 + c] = o;
            }
        }
        // (the next tile's loads touch qs, ks and vs, which every thread has finished reading
        // before the second barrier; `part` is written again only after the next first barrier)
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = p * Dp + i;
        if (live && i < Dp && d < D) srow[(size_t)d * Dv + col] = st[i];
    }
}

template <typename T>
static int launch_decay_attention(const DecayAttnArgs* a_in, int num_seqs, cudaStream_t st) {
    if (num_seqs <= 0) return 0;
    DecayAttnArgs args = *a_in;
    if (args.state_stride <= 0) args.state_stride = (long long)args.H * args.D * args.Dv;
    const DecayAttnArgs* a = &args;
    if (a->state_stride < (long long)a->H * a->D * a->Dv) return SLB_ERR_BAD_ARG;
    if ((a->gate_z == nullptr) == (a->decay == nullptr)) return SLB_ERR_BAD_ARG;      // one of the two
    if (a->gate_z != nullptr && (a->ld_gate < a->H * a->D || !(a->gate_inv_tau > 0.f))) return SLB_ERR_BAD_ARG;
    if (a->H <= 0 || a->D <= 0 || a->Dv <= 0 || a->num_slots <= 0 || (a->rot_dims & 1) || a->rot_dims < 0 ||
        a->rot_dims > a->D || (a->rot_dims > 0 && a->freq == nullptr) || a->act < 0 || a->act > 1)
        return SLB_ERR_BAD_ARG;
    if (a->D > DA_MAX_D || a->H > 65535) return SLB_ERR_TOO_LARGE;
    const int vz = (a->Dv + DA_EV - 1) / DA_EV;
    if (vz > 65535) return SLB_ERR_TOO_LARGE;
    const int dpad = ((a->D + DA_PARTS - 1) / DA_PARTS + 3) / 4 * 4;
    const size_t smem = ((size_t)(a->gate_z != nullptr ? 3 : 2) * DA_TT * DA_PARTS * dpad + DA_TT * DA_EV +
                         DA_TT * DA_PARTS * DA_EV) * sizeof(float);
    if (a->D <= 16 * DA_PARTS)
        return slb_launch(decay_attention_kernel<T, 16>, dim3(num_seqs, a->H, vz), dim3(DA_EV * DA_PARTS), smem, st, *a);
    return slb_launch(decay_attention_kernel<T, DA_MAX_D / DA_PARTS>, dim3(num_seqs, a->H, vz), dim3(DA_EV * DA_PARTS),
                      smem, st, *a);
}

extern "C" {
int slb_decay_attention_max_dim() { return DA_MAX_D; }
int slb_decay_attention_f32(const DecayAttnArgs* a, int num_seqs, cudaStream_t st) {
    return launch_decay_attention<float>(a, num_seqs, st);
}
int slb_decay_attention_bf16(const DecayAttnArgs* a, int num_seqs, cudaStream_t st) {
    return launch_decay_attention<bf16>(a, num_seqs, st);
}
}

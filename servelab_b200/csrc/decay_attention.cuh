// What the kernels of the linear attention with a decay share: their argument block and the
// preparation of an element of q or k (activation, rotation) in float32.
#pragma once

#include "common.cuh"

struct DecayAttnArgs {
    const void* proj; int ld;
    int q_off, k_off, v_off;
    int H, D, Dv;
    int act;                       // 0: none; 1: SiLU on q, k and v
    const float* freq; int rot_dims;
    float k_scale;
    const float* decay;            // [H]
    const int* positions; const int* cu_q; const int* state_slots;
    float* state; int num_slots;   // [num_slots][H][D][Dv]
    float* out; int ldo;           // [T][H * Dv] float32
    // appended: a decay of its own for every token and key channel instead of `decay` (which is
    // then null), alpha = sigmoid(z)^(1 / tau) with z = gate_z[token][h * D + d] + gate_bias[h * D + d]
    // (float32), formed in float32 as exp(log sigmoid(z) / tau); a factor on the queries; and the
    // distance in floats between the records of two slots (0: H * D * Dv)
    const float* gate_z; int ld_gate; const float* gate_bias; float gate_inv_tau;
    float q_scale;
    long long state_stride;
};

__device__ __forceinline__ float da_silu(float z) { return z / (1.0f + expf(-z)); }

// element d of a query or key head of token `row` (a pointer to the head's first element)
template <typename T>
__device__ __forceinline__ float da_prepared(const T* head, int d, int pos, const DecayAttnArgs& a) {
    float x = to_float(head[d]);
    if (a.act == 1) x = da_silu(x);
    if (d < a.rot_dims) {
        const int half = a.rot_dims >> 1;
        const int i = d < half ? d : d - half;
        float other = to_float(head[d < half ? d + half : d - half]);
        if (a.act == 1) other = da_silu(other);
        float sn, cs;
        sincosf((float)pos * a.freq[i], &sn, &cs);
        x = d < half ? x * cs - other * sn : x * cs + other * sn;
    }
    return x;
}

// rowquant.cuh — the per-32 int8 activation quantizer as the row kernels use it (backend/cuda/actgroup.cu:32-54:
// sc = max/127, inv = sc>0 ? 1/sc : 0, round to nearest even, clamp +-127, asum = sc*sum), and the f64 warp sum of the
// RMSNorm's sum of squares. Shared by the row kernels of a step and by the tensor-parallel reduce + norm + quantize kernel.
#pragma once
#include "common.cuh"

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Quantizes one group of 32 values held one per lane. Lane 0 writes the scale and the group sum.
__device__ __forceinline__ void quant_group_warp(float y, int8_t* codes_g, float* sc_out, float* asum_out, int lane) {
    float ma = fabsf(y);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
    float sc = __fdiv_rn(ma, 127.f);
    float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
    int q = __float2int_rn(__fmul_rn(y, inv));
    q = max(-127, min(127, q));
    int sum = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    codes_g[lane] = (int8_t)q;
    if (lane == 0) {
        *sc_out = sc;
        *asum_out = __fmul_rn(sc, (float)sum);
    }
}

// The same quantizer for a group held 8 values per lane by four consecutive lanes (q4 = lane & 3 is the lane's place in
// its group). The maximum and the integer sum do not depend on the order they are taken in, so the codes, scale and sum
// are those of quant_group_warp. Every lane of the warp must call it (lanes past the row pass zeros). The lane's eight
// codes come back packed in w[2], the group's scale and sum in sc and asum (the same in its four lanes).
__device__ __forceinline__ void quant_group_quad_regs(const float (&y)[8], unsigned (&w)[2], float& sc, float& asum,
                                                      float* deq = nullptr /* [8]: code * scale */) {
    float ma = 0.f;
#pragma unroll
    for (int u = 0; u < 8; u++) ma = fmaxf(ma, fabsf(y[u]));
    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 1));
    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 2));
    sc = __fdiv_rn(ma, 127.f);
    const float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
    int sum = 0;
    w[0] = w[1] = 0u;
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int q = __float2int_rn(__fmul_rn(y[u], inv));
        q = max(-127, min(127, q));
        sum += q;
        w[u >> 2] |= (unsigned)(q & 0xff) << (8 * (u & 3));
        if (deq) deq[u] = __fmul_rn((float)q, sc);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    asum = __fmul_rn(sc, (float)sum);
}

// ... stored: the codes at codes_g + 8*q4, the scale and the sum by the group's first lane (`live` false: nothing is stored)
__device__ __forceinline__ void quant_group_quad(const float (&y)[8], int8_t* codes_g, float* sc_out, float* asum_out, int q4, bool live,
                                                 float* deq = nullptr /* [8]: code * scale */) {
    unsigned w[2];
    float sc, asum;
    quant_group_quad_regs(y, w, sc, asum, deq);
    if (live) {
        *reinterpret_cast<uint2*>(codes_g + 8 * q4) = make_uint2(w[0], w[1]);
        if (q4 == 0) {
            *sc_out = sc;
            *asum_out = asum;
        }
    }
}

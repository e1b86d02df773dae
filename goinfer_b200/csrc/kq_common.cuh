// kq_common.cuh — the pieces of the K-quant block formats every kernel of this library shares.
//
// Q4_K and Q5_K super-blocks start with a 16-byte header: d and dmin (f16), then 12 bytes that pack eight 6-bit scales and
// eight 6-bit minima (the GGUF file's own layout; the reference's host twin is backend/cuda/kernels/ks_a1_test.go:62-67).
#pragma once
#include <cuda_fp16.h>

// byte k (0..11) of the 12 packed scale bytes, given as the header's three little-endian words after d|dmin
__device__ __forceinline__ unsigned kq_byte(int k, unsigned s0, unsigned s1, unsigned s2) {
    const unsigned w = k < 4 ? s0 : (k < 8 ? s1 : s2);
    return (w >> ((k & 3) << 3)) & 0xffu;
}

// 6-bit scale and minimum of sub-block j: sub-blocks 0..3 sit in the low six bits of bytes j and j+4; sub-blocks 4..7 take
// their low four bits from byte j+4 (scale: low nibble, minimum: high nibble) and their top two bits from the top two bits of
// bytes j-4 and j.
__device__ __forceinline__ void kq_scale_min(int j, unsigned s0, unsigned s1, unsigned s2, int* sc, int* m) {
    if (j < 4) {
        *sc = (int)(kq_byte(j, s0, s1, s2) & 63u);
        *m = (int)(kq_byte(j + 4, s0, s1, s2) & 63u);
    } else {
        const unsigned hi = kq_byte(j + 4, s0, s1, s2);
        *sc = (int)((hi & 0x0Fu) | ((kq_byte(j - 4, s0, s1, s2) >> 6) << 4));
        *m = (int)((hi >> 4) | ((kq_byte(j, s0, s1, s2) >> 6) << 4));
    }
}

__device__ __forceinline__ float kq_h2f(unsigned short b) { return __half2float(__ushort_as_half(b)); }

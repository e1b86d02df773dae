// kquant.cu — the GGUF Q5_K and Q6_K lanes: weight rows in the file's 5- and 6-bit super-blocks times the per-32 int8
// activations of the step. A Q4_K_M checkpoint keeps some projections (attn_v, ffn_down in half the layers, the head)
// in these formats; they are multiplied as they are, not through an int8 or fp16 copy.
//
//   Q5_K  (176 B / 256 weights: d, dmin, 12 bytes of 6-bit scales and minimums, qh[32], qs[128]):
//         y += (d*sc_g*aS_g) * idot_g - (dmin*m_g) * asum_g   per group g of 32, codes 0..31   (backend/cuda/actgroup.cu:77-143)
//   Q6_K  (210 B / 256 weights: ql[128], qh[64], 16 int8 sub-scales, d) kept as the blocks' first 208 bytes row by row
//         (16-byte aligned, so a lane's loads are 16-byte ones) followed by the blocks' d values:
//         y += (d*sc_h*aS_g) * idot_h   per half-group h of 16, codes -32..31   (the W6A8 product of backend/cuda/actgroup.cu:145-205)
//
// One warp owns one weight row and up to four activation rows; integer dots by dp4a, f32 terms, a shuffle tree at the
// end. A token's sum does not depend on the other tokens of the launch, so a row's bits do not depend on its batch.
// The bar is the reference's own for these kernels: |y - f64 product| <= 1e-5 * sum |w*a|
// (backend/cuda/kernels/kso1c_kernels_test.go:146-151).
#include "common.cuh"
#include "kq_common.cuh"

namespace {

__device__ __forceinline__ int kq_dp4a_us(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int kq_dp4a_ss(int a, int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Q5_K. Lane: super-block b0 + (lane >> 2) of the row (eight in flight), pair j = lane & 3 (sub-blocks 2j and 2j+1: the low and
// high nibbles of code bytes 32j .. 32j+31, whose fifth bits are bits 2j and 2j+1 of the 32 qh bytes).
template <int TT>
__global__ void __launch_bounds__(256) q5k_gemv_kernel(const uint8_t* __restrict__ W, int N, int nSB, const int8_t* __restrict__ codes,
                                                       const float* __restrict__ scales, int T, float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5), t0 = blockIdx.y * TT;
    if (n >= N) return;
    const int j = lane & 3, sub = lane >> 2, K = nSB * 256, nG = nSB * 8;
    const uint8_t* row = W + (size_t)n * nSB * 176;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.f;
    for (int b = sub; b < nSB; b += 8) {
        const uint8_t* blk = row + (size_t)b * 176;
        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
        const uint4 qh0 = *reinterpret_cast<const uint4*>(blk + 16), qh1 = *reinterpret_cast<const uint4*>(blk + 32);
        const uint4 q0 = *reinterpret_cast<const uint4*>(blk + 48 + 32 * j), q1 = *reinterpret_cast<const uint4*>(blk + 64 + 32 * j);
        const float d = kq_h2f((unsigned short)(hdr.x & 0xffffu)), dmin = kq_h2f((unsigned short)(hdr.x >> 16));
        int scLo, mLo, scHi, mHi;
        kq_scale_min(2 * j, hdr.y, hdr.z, hdr.w, &scLo, &mLo);
        kq_scale_min(2 * j + 1, hdr.y, hdr.z, hdr.w, &scHi, &mHi);
        const float dsLo = __fmul_rn(d, (float)scLo), dsHi = __fmul_rn(d, (float)scHi);
        const float nmLo = -__fmul_rn(dmin, (float)mLo), nmHi = -__fmul_rn(dmin, (float)mHi);
        const unsigned qs[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const unsigned qh[8] = {qh0.x, qh0.y, qh0.z, qh0.w, qh1.x, qh1.y, qh1.z, qh1.w};
        unsigned wl[8], wh[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            wl[i] = (qs[i] & 0x0F0F0F0Fu) | (((qh[i] >> (2 * j)) & 0x01010101u) << 4);
            wh[i] = ((qs[i] >> 4) & 0x0F0F0F0Fu) | (((qh[i] >> (2 * j + 1)) & 0x01010101u) << 4);
        }
        const int g = 8 * b + 2 * j;
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (t0 + t >= T) break;
            const int4* av = reinterpret_cast<const int4*>(codes + (size_t)(t0 + t) * K + 256 * b + 64 * j);
            const int4 l0 = av[0], l1 = av[1], h0 = av[2], h1 = av[3];
            const float* sp = scales + (size_t)(t0 + t) * 2 * nG;
            const float2 aS = *reinterpret_cast<const float2*>(sp + g), as = *reinterpret_cast<const float2*>(sp + nG + g);
            int pl = 0, ph = 0;
            pl = kq_dp4a_us(wl[0], l0.x, pl); pl = kq_dp4a_us(wl[1], l0.y, pl); pl = kq_dp4a_us(wl[2], l0.z, pl); pl = kq_dp4a_us(wl[3], l0.w, pl);
            pl = kq_dp4a_us(wl[4], l1.x, pl); pl = kq_dp4a_us(wl[5], l1.y, pl); pl = kq_dp4a_us(wl[6], l1.z, pl); pl = kq_dp4a_us(wl[7], l1.w, pl);
            ph = kq_dp4a_us(wh[0], h0.x, ph); ph = kq_dp4a_us(wh[1], h0.y, ph); ph = kq_dp4a_us(wh[2], h0.z, ph); ph = kq_dp4a_us(wh[3], h0.w, ph);
            ph = kq_dp4a_us(wh[4], h1.x, ph); ph = kq_dp4a_us(wh[5], h1.y, ph); ph = kq_dp4a_us(wh[6], h1.z, ph); ph = kq_dp4a_us(wh[7], h1.w, ph);
            float f = acc[t];
            f = __fmaf_rn((float)pl, __fmul_rn(dsLo, aS.x), f);
            f = __fmaf_rn((float)ph, __fmul_rn(dsHi, aS.y), f);
            f = __fmaf_rn(nmLo, as.x, f);
            acc[t] = __fmaf_rn(nmHi, as.y, f);
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        float f = acc[t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) f += __shfl_down_sync(0xffffffffu, f, off);
        if (lane == 0 && t0 + t < T) dst[(size_t)(t0 + t) * ldd + n] = f;
    }
}

// Q6_K on the device: per weight row, the file's blocks with their trailing d taken out, [row][super-block][208 B] (ql[128],
// qh[64], 16 int8 sub-scales: 16-byte aligned, so every load below is a 16-byte one), followed by one fp16 d per block
// ([row][super-block]). A block's 256 weights: half n = e / 128, then four groups of 32 (gq), element l of a group:
// low four bits in ql[64 n + 32 (gq & 1) + l] (low nibble for gq < 2, high for gq >= 2), two more bits in qh[32 n + l] at
// shift 2 gq; value = d * sc[8 n + 2 gq + l / 16] * (q - 32).
//
// Lane map: lane = 4 * (super-block of the pass) + 2 * n + h owns l = 16 h .. 16 h + 15 of half n, i.e. 64 weights of one
// super-block (16 of each group), eight super-blocks a pass; one sub-scale per group (index 8 n + 2 gq + h). The 6-bit codes
// stay unsigned: sum (q - 32) a = dp4a(q, a) - 32 * dp4a(1, a).
constexpr size_t kQ6Body = 208;
template <int TT>
__global__ void __launch_bounds__(256) q6k_gemv_kernel(const uint8_t* __restrict__ W, int N, int nSB, const int8_t* __restrict__ codes,
                                                       const float* __restrict__ scales, int T, float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5), t0 = blockIdx.y * TT;
    if (n >= N) return;
    const int half = (lane >> 1) & 1, h = lane & 1, K = nSB * 256, nG = nSB * 8;
    const uint8_t* body = W + (size_t)n * nSB * kQ6Body;
    const unsigned short* dp = reinterpret_cast<const unsigned short*>(W + (size_t)N * nSB * kQ6Body) + (size_t)n * nSB;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.f;
    for (int b = lane >> 2; b < nSB; b += 8) {
        const uint8_t* blk = body + (size_t)b * kQ6Body;
        const uint4 la = *reinterpret_cast<const uint4*>(blk + 64 * half + 16 * h);         // groups 0 (low nibbles) and 2 (high)
        const uint4 lb = *reinterpret_cast<const uint4*>(blk + 64 * half + 32 + 16 * h);    // groups 1 and 3
        const uint4 hb = *reinterpret_cast<const uint4*>(blk + 128 + 32 * half + 16 * h);   // the two upper bits of all four groups
        const uint2 sw = *reinterpret_cast<const uint2*>(blk + 192 + 8 * half);            // the half's eight sub-scales
        const float d = kq_h2f(dp[b]);
        const unsigned lo_a[4] = {la.x, la.y, la.z, la.w}, lo_b[4] = {lb.x, lb.y, lb.z, lb.w}, up[4] = {hb.x, hb.y, hb.z, hb.w};
        // sub-scale of group gq: byte 2 gq + h of the eight
        float dsc[4];
#pragma unroll
        for (int gq = 0; gq < 4; gq++) {
            const unsigned w = gq < 2 ? sw.x : sw.y;
            dsc[gq] = __fmul_rn(d, (float)(int)(signed char)((w >> (8 * (2 * (gq & 1) + h))) & 0xffu));
        }
        unsigned q6[4][4];   // [group][word of four codes], 0..63
#pragma unroll
        for (int i = 0; i < 4; i++) {
            q6[0][i] = (lo_a[i] & 0x0F0F0F0Fu) | ((up[i] << 4) & 0x30303030u);
            q6[1][i] = (lo_b[i] & 0x0F0F0F0Fu) | ((up[i] << 2) & 0x30303030u);
            q6[2][i] = ((lo_a[i] >> 4) & 0x0F0F0F0Fu) | (up[i] & 0x30303030u);
            q6[3][i] = ((lo_b[i] >> 4) & 0x0F0F0F0Fu) | ((up[i] >> 2) & 0x30303030u);
        }
        const int g0 = 8 * b + 4 * half;
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (t0 + t >= T) break;
            const int8_t* ab = codes + (size_t)(t0 + t) * K + 256 * b + 128 * half + 16 * h;
            const float* sp = scales + (size_t)(t0 + t) * 2 * nG + g0;
            float f = acc[t];
#pragma unroll
            for (int gq = 0; gq < 4; gq++) {
                const int4 a = *reinterpret_cast<const int4*>(ab + 32 * gq);
                int dot = kq_dp4a_us(q6[gq][0], a.x, 0), sum = kq_dp4a_ss(0x01010101, a.x, 0);
                dot = kq_dp4a_us(q6[gq][1], a.y, dot); sum = kq_dp4a_ss(0x01010101, a.y, sum);
                dot = kq_dp4a_us(q6[gq][2], a.z, dot); sum = kq_dp4a_ss(0x01010101, a.z, sum);
                dot = kq_dp4a_us(q6[gq][3], a.w, dot); sum = kq_dp4a_ss(0x01010101, a.w, sum);
                f = __fmaf_rn((float)(dot - 32 * sum), __fmul_rn(dsc[gq], sp[gq]), f);
            }
            acc[t] = f;
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        float f = acc[t];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) f += __shfl_xor_sync(0xffffffffu, f, off);
        if (lane == 0 && t0 + t < T) dst[(size_t)(t0 + t) * ldd + n] = f;
    }
}

// int8 rows with a scale per row (W8A8). Lane: 16 consecutive codes (half a group of 32) of every 32nd half-group of the row:
// four dp4a, one f32 term with the group's activation scale; the row scale multiplies the warp's total.
template <int TT>
__global__ void __launch_bounds__(256) i8_gemv_kernel(const uint8_t* __restrict__ W, int N, int K, const int8_t* __restrict__ codes,
                                                      const float* __restrict__ scales, int T, float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5), t0 = blockIdx.y * TT;
    if (n >= N) return;
    const int nG = K >> 5, nH = K >> 4;
    const uint4* row = reinterpret_cast<const uint4*>(W + (size_t)n * K);
    const float ws = reinterpret_cast<const float*>(W + (size_t)N * K)[n];
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.f;
    for (int c = lane; c < nH; c += 32) {
        const uint4 w = row[c];
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (t0 + t >= T) break;
            const int4 a = reinterpret_cast<const int4*>(codes + (size_t)(t0 + t) * K)[c];
            int p = kq_dp4a_ss((int)w.x, a.x, 0);
            p = kq_dp4a_ss((int)w.y, a.y, p);
            p = kq_dp4a_ss((int)w.z, a.z, p);
            p = kq_dp4a_ss((int)w.w, a.w, p);
            acc[t] = __fmaf_rn((float)p, scales[(size_t)(t0 + t) * 2 * nG + (c >> 1)], acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        float f = acc[t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) f += __shfl_down_sync(0xffffffffu, f, off);
        if (lane == 0 && t0 + t < T) dst[(size_t)(t0 + t) * ldd + n] = __fmul_rn(f, ws);
    }
}

__global__ void __launch_bounds__(256) i8_to_f16_kernel(const uint8_t* __restrict__ W, int N, int K, __half* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)N * K) return;
    const float ws = reinterpret_cast<const float*>(W + (size_t)N * K)[i / K];
    out[i] = __float2half_rn(__fmul_rn((float)reinterpret_cast<const int8_t*>(W)[i], ws));
}

// ---- fp16 copies for the tensor-core path at dense row counts (fast class): one thread per 32 weights ----
__global__ void __launch_bounds__(256) q5k_to_f16_kernel(const uint8_t* __restrict__ W, size_t n_blocks, __half* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (block, sub-block)
    if (i >= n_blocks * 8) return;
    const size_t g = i >> 3;
    const int j = (int)(i & 7);
    const uint8_t* blk = W + g * 176;
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    const float d = kq_h2f((unsigned short)(hdr.x & 0xffffu)), dmin = kq_h2f((unsigned short)(hdr.x >> 16));
    int sc, mn;
    kq_scale_min(j, hdr.y, hdr.z, hdr.w, &sc, &mn);
    const float ds = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)mn);
    const uint8_t *qh = blk + 16, *qs = blk + 48 + 32 * (j >> 1);
    __half* o = out + g * 256 + 32 * j;
    for (int l = 0; l < 32; l++) {
        const int code = ((j & 1) ? (qs[l] >> 4) : (qs[l] & 15)) | (((qh[l] >> j) & 1) << 4);
        o[l] = __float2half_rn(__fmaf_rn(ds, (float)code, -dm));
    }
}

__global__ void __launch_bounds__(256) q6k_to_f16_kernel(const uint8_t* __restrict__ W, size_t n_blocks, __half* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (block, group of 32)
    if (i >= n_blocks * 8) return;
    const size_t g = i >> 3;
    const int grp = (int)(i & 7), half = grp >> 2, gq = grp & 3;
    const uint8_t* blk = W + g * kQ6Body;
    const uint8_t* ql = blk + 64 * half + 32 * (gq & 1);
    const uint8_t* qh = blk + 128 + 32 * half;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + 8 * half + 2 * gq);
    const float d = kq_h2f(reinterpret_cast<const unsigned short*>(W + n_blocks * kQ6Body)[g]);
    __half* o = out + g * 256 + 32 * grp;
    for (int l = 0; l < 32; l++) {
        const int lo = (gq & 2) ? (ql[l] >> 4) : (ql[l] & 15);
        const int code = (lo | (((qh[l] >> (2 * gq)) & 3) << 4)) - 32;
        o[l] = __float2half_rn(__fmul_rn(__fmul_rn(d, (float)sc[l >> 4]), (float)code));
    }
}

// x[t][k] = code * scale of its group: the activations as the K-quant lanes see them, for the fp16 tensor-core path
__global__ void act_dequant_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales, int K, float* __restrict__ out) {
    const int t = blockIdx.y, k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= K) return;
    out[(size_t)t * K + k] = __fmul_rn((float)codes[(size_t)t * K + k], scales[(size_t)t * 2 * (K >> 5) + (k >> 5)]);
}

// the file's 210-byte blocks -> 208-byte bodies, then the blocks' d values
__global__ void q6k_repack_kernel(const uint8_t* __restrict__ raw, size_t TB, uint8_t* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (block, byte)
    if (i >= TB * 210) return;
    const size_t g = i / 210;
    const int o = (int)(i % 210);
    if (o < 208) out[g * kQ6Body + o] = raw[i];
    else out[TB * kQ6Body + g * 2 + (o - 208)] = raw[i];
}

}  // namespace

// W: Q5_K as in the file; Q6_K as 208-byte bodies + d (launch_q6k_repack). Any T: the rows go four at a time.
int launch_kq_matmul(b200_ctx* ctx, int kind, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd) {
    if (kind == B200_K_I8) {
        if (K % 32 || T < 1) B200_FAIL(ctx, B200_BAD_ARGUMENT, "int8 matmul needs K %% 32 == 0 and at least one row");
        if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(aq.codes)) & 15) B200_FAIL(ctx, B200_BAD_ARGUMENT, "int8 matmul wants 16-byte aligned buffers");
        ProfScope ps(ctx, PROF_HEAD_GEMM);
        const int tt = T == 1 ? 1 : (T == 2 ? 2 : 4);
        dim3 grid(ceil_div(N, 8), ceil_div(T, tt));
        if (tt == 1) i8_gemv_kernel<1><<<grid, 256, 0, ctx->stream>>>(W, N, K, aq.codes, aq.scales, T, dst, ldd);
        else if (tt == 2) i8_gemv_kernel<2><<<grid, 256, 0, ctx->stream>>>(W, N, K, aq.codes, aq.scales, T, dst, ldd);
        else i8_gemv_kernel<4><<<grid, 256, 0, ctx->stream>>>(W, N, K, aq.codes, aq.scales, T, dst, ldd);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    if (K % 256 || T < 1) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K-quant matmul needs K %% 256 == 0 and at least one row");
    if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(aq.codes)) & 15) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K-quant matmul wants 16-byte aligned buffers");
    const int nSB = K / 256;
    ProfScope ps(ctx, PROF_Q4K_GEMM);
    const int tt = T == 1 ? 1 : (T == 2 ? 2 : 4);
    dim3 grid(ceil_div(N, 8), ceil_div(T, tt));
    if (kind == B200_K_Q5K) {
        if (tt == 1) q5k_gemv_kernel<1><<<grid, 256, 0, ctx->stream>>>(W, N, nSB, aq.codes, aq.scales, T, dst, ldd);
        else if (tt == 2) q5k_gemv_kernel<2><<<grid, 256, 0, ctx->stream>>>(W, N, nSB, aq.codes, aq.scales, T, dst, ldd);
        else q5k_gemv_kernel<4><<<grid, 256, 0, ctx->stream>>>(W, N, nSB, aq.codes, aq.scales, T, dst, ldd);
    } else if (kind == B200_K_Q6K) {
        if (tt == 1) q6k_gemv_kernel<1><<<grid, 256, 0, ctx->stream>>>(W, N, nSB, aq.codes, aq.scales, T, dst, ldd);
        else if (tt == 2) q6k_gemv_kernel<2><<<grid, 256, 0, ctx->stream>>>(W, N, nSB, aq.codes, aq.scales, T, dst, ldd);
        else q6k_gemv_kernel<4><<<grid, 256, 0, ctx->stream>>>(W, N, nSB, aq.codes, aq.scales, T, dst, ldd);
    } else {
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "not a Q5_K / Q6_K matrix");
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_kq_to_f16(b200_ctx* ctx, int kind, const uint8_t* W, int N, int K, __half* out) {
    if (kind == B200_K_I8) {
        i8_to_f16_kernel<<<(unsigned)(((size_t)N * K + 255) / 256), 256, 0, ctx->stream>>>(W, N, K, out);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    const size_t nb = (size_t)N * K / 256;
    const unsigned grid = (unsigned)((nb * 8 + 255) / 256);
    if (kind == B200_K_Q5K) q5k_to_f16_kernel<<<grid, 256, 0, ctx->stream>>>(W, nb, out);
    else if (kind == B200_K_Q6K) q6k_to_f16_kernel<<<grid, 256, 0, ctx->stream>>>(W, nb, out);
    else B200_FAIL(ctx, B200_BAD_ARGUMENT, "not a Q5_K / Q6_K matrix");
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_act_dequant(b200_ctx* ctx, ActQ aq, int T, int K, float* out) {
    dim3 grid(ceil_div(K, 256), T);
    act_dequant_kernel<<<grid, 256, 0, ctx->stream>>>(aq.codes, aq.scales, K, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_q6k_repack(b200_ctx* ctx, const uint8_t* raw, size_t n_blocks, uint8_t* planes) {  // planes: n_blocks * 210 bytes
    const size_t n = n_blocks * 210;
    q6k_repack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(raw, n_blocks, planes);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

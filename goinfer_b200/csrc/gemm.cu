// gemm.cu — weight matmuls of the step.
//
// Q4_K x per-32-int8 activations, exact class (backend/cuda/actgroup.cu:311-355 rowQ4K's arithmetic):
//   dst[t][n] = sum over groups g, ascending:  fma(idot_g, (d*sc_g)*aS[t][g], .) then fma(-(dmin*m_g), asum[t][g], .)
// with idot_g the exact int32 dot of 32 weight codes and 32 activation codes. The integer dots run on the
// tensor cores (mma.sync m16n8k32 u8 x s8), the per-group rescale on the CUDA cores. Weights are the MMA's
// 16-row operand, packed tokens its 8-column operand, so one warp streams 16 weight rows once for up to
// 8*NT tokens. With SPLITK (small token counts, HBM-bound) the 8 warps of a CTA take super-blocks
// round-robin and fold their partials in warp order; without it every (row, token) sum is one ascending
// chain, the same order the CPU oracle uses, so the result is bit-identical to it.
//
// f16 weights (LM head): mma.sync m16n8k16 with the f32 activation split into f16 hi + lo parts, fp32
// accumulate. f32 weights (router, f32 test models): f64 accumulate on the CUDA cores.
#include <cstdlib>

#include "common.cuh"
#include "kq_common.cuh"

namespace {

#define MAGIC_I 0x4B400000
#define MAGIC_F 12582912.0f

__device__ __forceinline__ void mma_u8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d = a*b + c with c a separate (constant) operand: the magic-number bias costs no moves
__device__ __forceinline__ void mma_u8s8_c(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1,
                                           int c) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

// grid.x: 16-row weight tiles (8 per CTA without SPLITK, 1 per CTA with it); grid.y: token tiles of 8*NT;
// grid.z: experts when GROUPED.
template <int NT, bool SPLITK, bool GROUPED>
__global__ void __launch_bounds__(256) q4k_gemm_mma_kernel(const uint8_t* __restrict__ W, const uint8_t* const* __restrict__ Wptrs,
                                                           int N, int nSB, const int8_t* __restrict__ codes,
                                                           const float* __restrict__ scales, int T,
                                                           const int32_t* __restrict__ offs, const int32_t* __restrict__ rows,
                                                           float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
    const int n0 = SPLITK ? blockIdx.x * 16 : (blockIdx.x * 8 + warp) * 16;
    if (!SPLITK && n0 >= N) return;
    int t_base, t_end;
    const uint8_t* Wm = W;
    if (GROUPED) {
        const int e = blockIdx.z;
        t_base = offs[e] + blockIdx.y * 8 * NT;
        t_end = offs[e + 1];
        if (t_base >= t_end) return;
        Wm = Wptrs[e];
    } else {
        t_base = blockIdx.y * 8 * NT;
        t_end = T;
    }
    const int K = nSB * 256, nG = nSB * 8;
    const int r0 = min(n0 + gid, N - 1), r1 = min(n0 + gid + 8, N - 1);
    const uint8_t* w0 = Wm + (size_t)r0 * nSB * 144;
    const uint8_t* w1 = Wm + (size_t)r1 * nSB * 144;

    const int8_t* ab[NT];   // activation codes of the token this lane feeds the MMA with
    const float* sc0[NT];   // scale rows of the two tokens this lane's accumulators belong to
    const float* sc1[NT];
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        int tb = min(t_base + 8 * j + gid, t_end - 1);
        int tc0 = min(t_base + 8 * j + 2 * tig, t_end - 1), tc1 = min(t_base + 8 * j + 2 * tig + 1, t_end - 1);
        if (GROUPED && rows) { tb = rows[tb]; tc0 = rows[tc0]; tc1 = rows[tc1]; }
        ab[j] = codes + (size_t)tb * K + 8 * tig;
        sc0[j] = scales + (size_t)tc0 * 2 * nG;
        sc1[j] = scales + (size_t)tc1 * 2 * nG;
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    }

    const int b_begin = SPLITK ? warp : 0, b_step = SPLITK ? 8 : 1;
    for (int b = b_begin; b < nSB; b += b_step) {
        const uint4 h0 = *reinterpret_cast<const uint4*>(w0 + (size_t)b * 144);
        const uint4 h1 = *reinterpret_cast<const uint4*>(w1 + (size_t)b * 144);
        // this lane decodes sub-blocks 2*tig and 2*tig+1 of its two rows; the quad shares them by shuffle
        float my_ds[2][2], my_nm[2][2];
        {
            int s, m;
            const float d0 = kq_h2f((unsigned short)(h0.x & 0xffffu)), dm0 = kq_h2f((unsigned short)(h0.x >> 16));
            const float d1 = kq_h2f((unsigned short)(h1.x & 0xffffu)), dm1 = kq_h2f((unsigned short)(h1.x >> 16));
            kq_scale_min(2 * tig, h0.y, h0.z, h0.w, &s, &m);
            my_ds[0][0] = __fmul_rn(d0, (float)s); my_nm[0][0] = -__fmul_rn(dm0, (float)m);
            kq_scale_min(2 * tig + 1, h0.y, h0.z, h0.w, &s, &m);
            my_ds[0][1] = __fmul_rn(d0, (float)s); my_nm[0][1] = -__fmul_rn(dm0, (float)m);
            kq_scale_min(2 * tig, h1.y, h1.z, h1.w, &s, &m);
            my_ds[1][0] = __fmul_rn(d1, (float)s); my_nm[1][0] = -__fmul_rn(dm1, (float)m);
            kq_scale_min(2 * tig + 1, h1.y, h1.z, h1.w, &s, &m);
            my_ds[1][1] = __fmul_rn(d1, (float)s); my_nm[1][1] = -__fmul_rn(dm1, (float)m);
        }
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int src = (lane & ~3) | p;
            const float ds0lo = __shfl_sync(0xffffffffu, my_ds[0][0], src), ds0hi = __shfl_sync(0xffffffffu, my_ds[0][1], src);
            const float ds1lo = __shfl_sync(0xffffffffu, my_ds[1][0], src), ds1hi = __shfl_sync(0xffffffffu, my_ds[1][1], src);
            const float nm0lo = __shfl_sync(0xffffffffu, my_nm[0][0], src), nm0hi = __shfl_sync(0xffffffffu, my_nm[0][1], src);
            const float nm1lo = __shfl_sync(0xffffffffu, my_nm[1][0], src), nm1hi = __shfl_sync(0xffffffffu, my_nm[1][1], src);
            // code words 2*tig, 2*tig+1 of the pair: low nibbles = sub-block 2p, high = 2p+1. The k order inside a
            // group is permuted the same way for weights and activations, which an integer dot does not see.
            const uint2 q0 = *reinterpret_cast<const uint2*>(w0 + (size_t)b * 144 + 16 + 32 * p + 8 * tig);
            const uint2 q1 = *reinterpret_cast<const uint2*>(w1 + (size_t)b * 144 + 16 + 32 * p + 8 * tig);
            const unsigned al0 = q0.x & 0x0F0F0F0Fu, al1 = q1.x & 0x0F0F0F0Fu, al2 = q0.y & 0x0F0F0F0Fu, al3 = q1.y & 0x0F0F0F0Fu;
            const unsigned ah0 = (q0.x >> 4) & 0x0F0F0F0Fu, ah1 = (q1.x >> 4) & 0x0F0F0F0Fu, ah2 = (q0.y >> 4) & 0x0F0F0F0Fu,
                           ah3 = (q1.y >> 4) & 0x0F0F0F0Fu;
            const int g = 8 * b + 2 * p;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const int2 blo = *reinterpret_cast<const int2*>(ab[j] + 256 * b + 64 * p);
                const int2 bhi = *reinterpret_cast<const int2*>(ab[j] + 256 * b + 64 * p + 32);
                int cl[4] = {MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I}, ch[4] = {MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I};
                mma_u8s8(cl, al0, al1, al2, al3, (unsigned)blo.x, (unsigned)blo.y);
                mma_u8s8(ch, ah0, ah1, ah2, ah3, (unsigned)bhi.x, (unsigned)bhi.y);
                const float2 aS0 = *reinterpret_cast<const float2*>(sc0[j] + g);       // token 2*tig: scales of groups g, g+1
                const float2 aS1 = *reinterpret_cast<const float2*>(sc1[j] + g);       // token 2*tig+1
                const float2 as0 = *reinterpret_cast<const float2*>(sc0[j] + nG + g);  // group sums
                const float2 as1 = *reinterpret_cast<const float2*>(sc1[j] + nG + g);
                float f;
                // (row gid, token 2*tig)
                f = acc[j][0];
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[0]), MAGIC_F), __fmul_rn(ds0lo, aS0.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[0]), MAGIC_F), __fmul_rn(ds0hi, aS0.y), f);
                f = __fmaf_rn(nm0lo, as0.x, f);
                acc[j][0] = __fmaf_rn(nm0hi, as0.y, f);
                // (row gid, token 2*tig+1)
                f = acc[j][1];
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[1]), MAGIC_F), __fmul_rn(ds0lo, aS1.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[1]), MAGIC_F), __fmul_rn(ds0hi, aS1.y), f);
                f = __fmaf_rn(nm0lo, as1.x, f);
                acc[j][1] = __fmaf_rn(nm0hi, as1.y, f);
                // (row gid+8, token 2*tig)
                f = acc[j][2];
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[2]), MAGIC_F), __fmul_rn(ds1lo, aS0.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[2]), MAGIC_F), __fmul_rn(ds1hi, aS0.y), f);
                f = __fmaf_rn(nm1lo, as0.x, f);
                acc[j][2] = __fmaf_rn(nm1hi, as0.y, f);
                // (row gid+8, token 2*tig+1)
                f = acc[j][3];
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[3]), MAGIC_F), __fmul_rn(ds1lo, aS1.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[3]), MAGIC_F), __fmul_rn(ds1hi, aS1.y), f);
                f = __fmaf_rn(nm1lo, as1.x, f);
                acc[j][3] = __fmaf_rn(nm1hi, as1.y, f);
            }
        }
    }

    if (SPLITK) {
        // fold the 8 warps' partials in warp order (fixed, so a row's value does not depend on the batch)
        __shared__ float red[8][NT][4][32];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[warp][j][i][lane] = acc[j][i];
        __syncthreads();
        if (warp != 0) return;
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float s = red[0][j][i][lane];
#pragma unroll
                for (int w = 1; w < 8; w++) s = __fadd_rn(s, red[w][j][i][lane]);
                acc[j][i] = s;
            }
    }
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int t0 = t_base + 8 * j + 2 * tig, t1 = t0 + 1;
        const int na = n0 + gid, nb = n0 + gid + 8;
        if (t0 < t_end) {
            if (na < N) dst[(size_t)t0 * ldd + na] = acc[j][0];
            if (nb < N) dst[(size_t)t0 * ldd + nb] = acc[j][2];
        }
        if (t1 < t_end) {
            if (na < N) dst[(size_t)t1 * ldd + na] = acc[j][1];
            if (nb < N) dst[(size_t)t1 * ldd + nb] = acc[j][3];
        }
    }
}


// ---- tiled exact-class kernel for more than 8 rows ----
// CTA = 8 warps x 16 weight rows against BT = 8*NT tokens. Per super-block the tokens' 256 activation codes and their
// 8 scales / 8 group sums are staged in shared memory by cp.async (two stages), each token's codes padded to 288 bytes
// so the 8-byte fragment loads of a half-warp fall in distinct banks. Weights stream from global memory straight into
// registers, one super-block ahead. Arithmetic and its order are q4k_gemm_mma_kernel's: one ascending chain per output.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gsrc) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N_>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N_)); }

struct WRegs {
    uint4 h0, h1;
    uint2 q0[4], q1[4];
};

__device__ __forceinline__ void load_wregs(WRegs& w, const uint8_t* w0, const uint8_t* w1, int b, int tig) {
    w.h0 = *reinterpret_cast<const uint4*>(w0 + (size_t)b * 144);
    w.h1 = *reinterpret_cast<const uint4*>(w1 + (size_t)b * 144);
#pragma unroll
    for (int p = 0; p < 4; p++) {
        w.q0[p] = *reinterpret_cast<const uint2*>(w0 + (size_t)b * 144 + 16 + 32 * p + 8 * tig);
        w.q1[p] = *reinterpret_cast<const uint2*>(w1 + (size_t)b * 144 + 16 + 32 * p + 8 * tig);
    }
}

template <int NT, bool GROUPED>
__global__ void __launch_bounds__(256, (NT <= 8 ? 2 : 1)) q4k_gemm_tile_kernel(
    const uint8_t* __restrict__ W, const uint8_t* const* __restrict__ Wptrs, int N, int nSB, const int8_t* __restrict__ codes,
    const float* __restrict__ scales, int T, const int32_t* __restrict__ offs, const int32_t* __restrict__ rows,
    float* __restrict__ dst, int ldd) {
    constexpr int BT = 8 * NT, CS = 288, SS = 80, STAGE = BT * CS + BT * SS;  // SS: 64 bytes of scales padded so 4 tokens' float4 loads miss each other's banks
    extern __shared__ __align__(16) uint8_t tile_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
    const int n0 = (blockIdx.x * 8 + warp) * 16;
    int t_base, t_end;
    const uint8_t* Wm = W;
    if (GROUPED) {
        const int e = blockIdx.z;
        t_base = offs[e] + blockIdx.y * BT;
        t_end = offs[e + 1];
        if (t_base >= t_end) return;
        Wm = Wptrs[e];
    } else {
        t_base = blockIdx.y * BT;
        t_end = T;
    }
    const int K = nSB * 256, nG = nSB * 8;
    const bool active = n0 < N;
    const int r0 = min(n0 + gid, N - 1), r1 = min(n0 + gid + 8, N - 1);
    const uint8_t* w0 = Wm + (size_t)r0 * nSB * 144;
    const uint8_t* w1 = Wm + (size_t)r1 * nSB * 144;

    auto load_stage = [&](int b, int st) {
        uint8_t* sc = tile_smem + st * STAGE;
        uint8_t* ss = sc + BT * CS;
        for (int i = threadIdx.x; i < BT * 16; i += 256) {
            const int tok = i >> 4, c = i & 15;
            int t = min(t_base + tok, t_end - 1);
            if (GROUPED && rows) t = rows[t];
            cp_async16(sc + tok * CS + c * 16, codes + (size_t)t * K + 256 * b + 16 * c);
        }
        for (int i = threadIdx.x; i < BT * 8; i += 256) {
            const int tok = i >> 3, q = i & 7, p = q >> 1, half = q & 1;  // half 0: scales of groups 2p,2p+1; 1: their sums
            int t = min(t_base + tok, t_end - 1);
            if (GROUPED && rows) t = rows[t];
            cp_async8(ss + tok * SS + p * 16 + half * 8, scales + (size_t)t * 2 * nG + (half ? nG : 0) + 8 * b + 2 * p);
        }
    };

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    WRegs wc, wn;
    load_stage(0, 0);
    cp_async_commit();
    if (active) load_wregs(wc, w0, w1, 0, tig);
    for (int b = 0; b < nSB; b++) {
        if (b + 1 < nSB) {
            load_stage(b + 1, (b + 1) & 1);
            cp_async_commit();
            if (active) load_wregs(wn, w0, w1, b + 1, tig);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (active) {
            const uint8_t* sc = tile_smem + (b & 1) * STAGE;
            const uint8_t* ss = sc + BT * CS;
            float my_ds[2][2], my_nm[2][2];
            {
                int s_, m_;
                const float d0 = kq_h2f((unsigned short)(wc.h0.x & 0xffffu)), dm0 = kq_h2f((unsigned short)(wc.h0.x >> 16));
                const float d1 = kq_h2f((unsigned short)(wc.h1.x & 0xffffu)), dm1 = kq_h2f((unsigned short)(wc.h1.x >> 16));
                kq_scale_min(2 * tig, wc.h0.y, wc.h0.z, wc.h0.w, &s_, &m_);
                my_ds[0][0] = __fmul_rn(d0, (float)s_); my_nm[0][0] = -__fmul_rn(dm0, (float)m_);
                kq_scale_min(2 * tig + 1, wc.h0.y, wc.h0.z, wc.h0.w, &s_, &m_);
                my_ds[0][1] = __fmul_rn(d0, (float)s_); my_nm[0][1] = -__fmul_rn(dm0, (float)m_);
                kq_scale_min(2 * tig, wc.h1.y, wc.h1.z, wc.h1.w, &s_, &m_);
                my_ds[1][0] = __fmul_rn(d1, (float)s_); my_nm[1][0] = -__fmul_rn(dm1, (float)m_);
                kq_scale_min(2 * tig + 1, wc.h1.y, wc.h1.z, wc.h1.w, &s_, &m_);
                my_ds[1][1] = __fmul_rn(d1, (float)s_); my_nm[1][1] = -__fmul_rn(dm1, (float)m_);
            }
#pragma unroll
            for (int p = 0; p < 4; p++) {
                const int src = (lane & ~3) | p;
                const float ds0lo = __shfl_sync(0xffffffffu, my_ds[0][0], src), ds0hi = __shfl_sync(0xffffffffu, my_ds[0][1], src);
                const float ds1lo = __shfl_sync(0xffffffffu, my_ds[1][0], src), ds1hi = __shfl_sync(0xffffffffu, my_ds[1][1], src);
                const float nm0lo = __shfl_sync(0xffffffffu, my_nm[0][0], src), nm0hi = __shfl_sync(0xffffffffu, my_nm[0][1], src);
                const float nm1lo = __shfl_sync(0xffffffffu, my_nm[1][0], src), nm1hi = __shfl_sync(0xffffffffu, my_nm[1][1], src);
                const uint2 q0 = wc.q0[p], q1 = wc.q1[p];
                const unsigned al0 = q0.x & 0x0F0F0F0Fu, al1 = q1.x & 0x0F0F0F0Fu, al2 = q0.y & 0x0F0F0F0Fu, al3 = q1.y & 0x0F0F0F0Fu;
                const unsigned ah0 = (q0.x >> 4) & 0x0F0F0F0Fu, ah1 = (q1.x >> 4) & 0x0F0F0F0Fu, ah2 = (q0.y >> 4) & 0x0F0F0F0Fu,
                               ah3 = (q1.y >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    const uint8_t* tb = sc + (8 * j + gid) * CS + 64 * p + 8 * tig;
                    const int2 blo = *reinterpret_cast<const int2*>(tb);
                    const int2 bhi = *reinterpret_cast<const int2*>(tb + 32);
                    int cl[4], ch[4];
                    mma_u8s8_c(cl, al0, al1, al2, al3, (unsigned)blo.x, (unsigned)blo.y, MAGIC_I);
                    mma_u8s8_c(ch, ah0, ah1, ah2, ah3, (unsigned)bhi.x, (unsigned)bhi.y, MAGIC_I);
                    // {aS[g], aS[g+1], asum[g], asum[g+1]} of tokens 2*tig and 2*tig+1 of this tile
                    const float4 s0 = *reinterpret_cast<const float4*>(ss + (8 * j + 2 * tig) * SS + p * 16);
                    const float4 s1 = *reinterpret_cast<const float4*>(ss + (8 * j + 2 * tig + 1) * SS + p * 16);
                    float f;
                    f = acc[j][0];
                    f = __fmaf_rn(__fsub_rn(__int_as_float(cl[0]), MAGIC_F), __fmul_rn(ds0lo, s0.x), f);
                    f = __fmaf_rn(__fsub_rn(__int_as_float(ch[0]), MAGIC_F), __fmul_rn(ds0hi, s0.y), f);
                    f = __fmaf_rn(nm0lo, s0.z, f);
                    acc[j][0] = __fmaf_rn(nm0hi, s0.w, f);
                    f = acc[j][1];
                    f = __fmaf_rn(__fsub_rn(__int_as_float(cl[1]), MAGIC_F), __fmul_rn(ds0lo, s1.x), f);
                    f = __fmaf_rn(__fsub_rn(__int_as_float(ch[1]), MAGIC_F), __fmul_rn(ds0hi, s1.y), f);
                    f = __fmaf_rn(nm0lo, s1.z, f);
                    acc[j][1] = __fmaf_rn(nm0hi, s1.w, f);
                    f = acc[j][2];
                    f = __fmaf_rn(__fsub_rn(__int_as_float(cl[2]), MAGIC_F), __fmul_rn(ds1lo, s0.x), f);
                    f = __fmaf_rn(__fsub_rn(__int_as_float(ch[2]), MAGIC_F), __fmul_rn(ds1hi, s0.y), f);
                    f = __fmaf_rn(nm1lo, s0.z, f);
                    acc[j][2] = __fmaf_rn(nm1hi, s0.w, f);
                    f = acc[j][3];
                    f = __fmaf_rn(__fsub_rn(__int_as_float(cl[3]), MAGIC_F), __fmul_rn(ds1lo, s1.x), f);
                    f = __fmaf_rn(__fsub_rn(__int_as_float(ch[3]), MAGIC_F), __fmul_rn(ds1hi, s1.y), f);
                    f = __fmaf_rn(nm1lo, s1.z, f);
                    acc[j][3] = __fmaf_rn(nm1hi, s1.w, f);
                }
            }
            wc = wn;
        }
        __syncthreads();
    }
    if (!active) return;
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int t0 = t_base + 8 * j + 2 * tig, t1 = t0 + 1;
        const int na = n0 + gid, nb = n0 + gid + 8;
        if (t0 < t_end) {
            if (na < N) dst[(size_t)t0 * ldd + na] = acc[j][0];
            if (nb < N) dst[(size_t)t0 * ldd + nb] = acc[j][2];
        }
        if (t1 < t_end) {
            if (na < N) dst[(size_t)t1 * ldd + na] = acc[j][1];
            if (nb < N) dst[(size_t)t1 * ldd + nb] = acc[j][3];
        }
    }
}

template <int NT>
int run_q4k_tile(b200_ctx* ctx, const uint8_t* W, int N, int nSB, ActQ aq, int T, float* dst, int ldd) {
    constexpr int smem = 2 * (8 * NT) * (288 + 80);
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        cudaFuncSetAttribute(q4k_gemm_tile_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    dim3 grid(ceil_div(N, 128), ceil_div(T, 8 * NT));
    ProfScope ps(ctx, PROF_Q4K_GEMM);
    q4k_gemm_tile_kernel<NT, false><<<grid, 256, smem, ctx->stream>>>(W, nullptr, N, nSB, aq.codes, aq.scales, T, nullptr, nullptr,
                                                                     dst, ldd);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}


// ---- small-batch GEMV (fast class, up to 3 rows): HBM-bound, CUDA-core integer dots ----
// One warp per R weight rows; lane l owns sub-block pair (l & 3) of super-block b0 + (l >> 2), eight super-blocks a
// pass (the lane partition of backend/cuda/actgroup.cu:302-316); U passes are loaded before any is used. High nibbles
// are not shifted down: dp4a runs on q & 0xF0F0F0F0 and the scale carries the exact factor 1/16. Lane partials are
// folded by shfl_down 16..1. These matrices are 9-57 MB, where a launch's fixed ~4 us shows: a plain streaming read of
// the same bytes reaches 2.1 / 3.5 / 4.6 TB/s at 9.4 / 28 / 57 MB on this GPU, and this kernel 73-79% of that.
// unsigned weight bytes x signed activation bytes
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int TT, int R, int U>
__global__ void __launch_bounds__(256) q4k_gemv_dp4a_kernel(const uint8_t* __restrict__ W, int N, int nSB,
                                                            const int8_t* __restrict__ codes, const float* __restrict__ scales,
                                                            float* __restrict__ dst, int ldd) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = (blockIdx.x * 8 + warp) * R;
    if (n0 >= N) return;
    const int j = lane & 3, sub = lane >> 2;
    const int K = nSB * 256, nG = nSB * 8;
    const uint8_t* wr[R];
#pragma unroll
    for (int r = 0; r < R; r++) wr[r] = W + (size_t)min(n0 + r, N - 1) * nSB * 144;
    float acc[R][TT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < TT; t++) acc[r][t] = 0.f;

    for (int b0 = 0; b0 < nSB; b0 += 8 * U) {
        uint4 hdr[U][R], q0[U][R], q1[U][R];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int b = b0 + 8 * u + sub;
            ok[u] = b < nSB;
            const int bb = ok[u] ? b : nSB - 1;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint8_t* blk = wr[r] + (size_t)bb * 144;
                hdr[u][r] = *reinterpret_cast<const uint4*>(blk);
                q0[u][r] = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j);
                q1[u][r] = *reinterpret_cast<const uint4*>(blk + 32 + 32 * j);
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (!ok[u]) continue;
            const int b = b0 + 8 * u + sub, g = 8 * b + 2 * j;
            int4 al[TT][2], ah[TT][2];
            float2 aS[TT], as[TT];
#pragma unroll
            for (int t = 0; t < TT; t++) {
                const int4* av = reinterpret_cast<const int4*>(codes + (size_t)t * K + 256 * b + 64 * j);
                al[t][0] = av[0]; al[t][1] = av[1]; ah[t][0] = av[2]; ah[t][1] = av[3];
                aS[t] = *reinterpret_cast<const float2*>(scales + (size_t)t * 2 * nG + g);
                as[t] = *reinterpret_cast<const float2*>(scales + (size_t)t * 2 * nG + nG + g);
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint4 h = hdr[u][r];
                const float d = kq_h2f((unsigned short)(h.x & 0xffffu)), dmin = kq_h2f((unsigned short)(h.x >> 16));
                int scLo, mLo, scHi, mHi;
                kq_scale_min(2 * j, h.y, h.z, h.w, &scLo, &mLo);
                kq_scale_min(2 * j + 1, h.y, h.z, h.w, &scHi, &mHi);
                const float dsLo = __fmul_rn(d, (float)scLo), dsHi = __fmul_rn(d, (float)scHi);
                const float nmLo = -__fmul_rn(dmin, (float)mLo), nmHi = -__fmul_rn(dmin, (float)mHi);
                const uint4 a = q0[u][r], c = q1[u][r];
                const unsigned wl[8] = {a.x & 0x0F0F0F0Fu, a.y & 0x0F0F0F0Fu, a.z & 0x0F0F0F0Fu, a.w & 0x0F0F0F0Fu,
                                        c.x & 0x0F0F0F0Fu, c.y & 0x0F0F0F0Fu, c.z & 0x0F0F0F0Fu, c.w & 0x0F0F0F0Fu};
                const unsigned wh[8] = {a.x & 0xF0F0F0F0u, a.y & 0xF0F0F0F0u, a.z & 0xF0F0F0F0u, a.w & 0xF0F0F0F0u,
                                        c.x & 0xF0F0F0F0u, c.y & 0xF0F0F0F0u, c.z & 0xF0F0F0F0u, c.w & 0xF0F0F0F0u};
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    int pl = 0, ph = 0;
                    pl = dp4a_us(wl[0], al[t][0].x, pl); pl = dp4a_us(wl[1], al[t][0].y, pl);
                    pl = dp4a_us(wl[2], al[t][0].z, pl); pl = dp4a_us(wl[3], al[t][0].w, pl);
                    pl = dp4a_us(wl[4], al[t][1].x, pl); pl = dp4a_us(wl[5], al[t][1].y, pl);
                    pl = dp4a_us(wl[6], al[t][1].z, pl); pl = dp4a_us(wl[7], al[t][1].w, pl);
                    ph = dp4a_us(wh[0], ah[t][0].x, ph); ph = dp4a_us(wh[1], ah[t][0].y, ph);
                    ph = dp4a_us(wh[2], ah[t][0].z, ph); ph = dp4a_us(wh[3], ah[t][0].w, ph);
                    ph = dp4a_us(wh[4], ah[t][1].x, ph); ph = dp4a_us(wh[5], ah[t][1].y, ph);
                    ph = dp4a_us(wh[6], ah[t][1].z, ph); ph = dp4a_us(wh[7], ah[t][1].w, ph);
                    float f = acc[r][t];
                    f = __fmaf_rn((float)pl, __fmul_rn(dsLo, aS[t].x), f);
                    f = __fmaf_rn((float)ph, __fmul_rn(__fmul_rn(dsHi, aS[t].y), 0.0625f), f);  // ph = 16 * idot, 1/16 is exact
                    f = __fmaf_rn(nmLo, as[t].x, f);
                    acc[r][t] = __fmaf_rn(nmHi, as[t].y, f);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < TT; t++) {
            float f = acc[r][t];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) f += __shfl_down_sync(0xffffffffu, f, off);
            if (lane == 0 && n0 + r < N) dst[(size_t)t * ldd + n0 + r] = f;
        }
}


// The same products from the tile-major copy ([16-row tile][super-block][16 rows][144 B], what a fast-class model keeps):
// a CTA takes one 16-row tile, warp w the super-blocks w, w+8, ...; lane l owns rows (l >> 2) and (l >> 2) + 8 and the
// sub-block pair (l & 3), so a warp's loads of one super-block are the tile's 2304 contiguous bytes and the CTA's eight
// warps read 18 KB in one piece. The eight row-lanes of a pair read the same activations (one broadcast). Lane partials
// fold over the four pairs by two xor shuffles, warp partials through shared memory in warp order.
template <int TT>
__global__ void __launch_bounds__(256) q4k_gemv_tiles_kernel(const uint8_t* __restrict__ W16, int N, int nSB,
                                                             const int8_t* __restrict__ codes, const float* __restrict__ scales,
                                                             float* __restrict__ dst, int ldd) {
    pdl_trigger();
    pdl_wait();
    __shared__ float part[8][16][TT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = lane & 3, r0 = lane >> 2;
    const int K = nSB * 256, nG = nSB * 8;
    const uint8_t* tile = W16 + (size_t)blockIdx.x * nSB * (16 * 144);
    float acc[2][TT];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int t = 0; t < TT; t++) acc[r][t] = 0.f;
    constexpr int U = 2;  // super-blocks in flight per warp
    for (int b0 = warp; b0 < nSB; b0 += 8 * U) {
        uint4 hdr[U][2], q0[U][2], q1[U][2];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int b = b0 + 8 * u;
            ok[u] = b < nSB;
            const uint8_t* blk0 = tile + (size_t)(ok[u] ? b : b0) * (16 * 144);
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint8_t* blk = blk0 + (r0 + 8 * r) * 144;
                hdr[u][r] = *reinterpret_cast<const uint4*>(blk);
                q0[u][r] = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j);
                q1[u][r] = *reinterpret_cast<const uint4*>(blk + 32 + 32 * j);
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (!ok[u]) continue;
            const int b = b0 + 8 * u, g = 8 * b + 2 * j;
            int4 al[TT][2], ah[TT][2];
            float2 aS[TT], as[TT];
#pragma unroll
            for (int t = 0; t < TT; t++) {
                const int4* av = reinterpret_cast<const int4*>(codes + (size_t)t * K + 256 * b + 64 * j);
                al[t][0] = av[0]; al[t][1] = av[1]; ah[t][0] = av[2]; ah[t][1] = av[3];
                aS[t] = *reinterpret_cast<const float2*>(scales + (size_t)t * 2 * nG + g);
                as[t] = *reinterpret_cast<const float2*>(scales + (size_t)t * 2 * nG + nG + g);
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint4 h = hdr[u][r];
                const float d = kq_h2f((unsigned short)(h.x & 0xffffu)), dmin = kq_h2f((unsigned short)(h.x >> 16));
                int scLo, mLo, scHi, mHi;
                kq_scale_min(2 * j, h.y, h.z, h.w, &scLo, &mLo);
                kq_scale_min(2 * j + 1, h.y, h.z, h.w, &scHi, &mHi);
                const float dsLo = __fmul_rn(d, (float)scLo), dsHi = __fmul_rn(d, (float)scHi);
                const float nmLo = -__fmul_rn(dmin, (float)mLo), nmHi = -__fmul_rn(dmin, (float)mHi);
                const uint4 a = q0[u][r], c = q1[u][r];
                const unsigned wl[8] = {a.x & 0x0F0F0F0Fu, a.y & 0x0F0F0F0Fu, a.z & 0x0F0F0F0Fu, a.w & 0x0F0F0F0Fu,
                                        c.x & 0x0F0F0F0Fu, c.y & 0x0F0F0F0Fu, c.z & 0x0F0F0F0Fu, c.w & 0x0F0F0F0Fu};
                const unsigned wh[8] = {a.x & 0xF0F0F0F0u, a.y & 0xF0F0F0F0u, a.z & 0xF0F0F0F0u, a.w & 0xF0F0F0F0u,
                                        c.x & 0xF0F0F0F0u, c.y & 0xF0F0F0F0u, c.z & 0xF0F0F0F0u, c.w & 0xF0F0F0F0u};
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    int pl = 0, ph = 0;
                    pl = dp4a_us(wl[0], al[t][0].x, pl); pl = dp4a_us(wl[1], al[t][0].y, pl);
                    pl = dp4a_us(wl[2], al[t][0].z, pl); pl = dp4a_us(wl[3], al[t][0].w, pl);
                    pl = dp4a_us(wl[4], al[t][1].x, pl); pl = dp4a_us(wl[5], al[t][1].y, pl);
                    pl = dp4a_us(wl[6], al[t][1].z, pl); pl = dp4a_us(wl[7], al[t][1].w, pl);
                    ph = dp4a_us(wh[0], ah[t][0].x, ph); ph = dp4a_us(wh[1], ah[t][0].y, ph);
                    ph = dp4a_us(wh[2], ah[t][0].z, ph); ph = dp4a_us(wh[3], ah[t][0].w, ph);
                    ph = dp4a_us(wh[4], ah[t][1].x, ph); ph = dp4a_us(wh[5], ah[t][1].y, ph);
                    ph = dp4a_us(wh[6], ah[t][1].z, ph); ph = dp4a_us(wh[7], ah[t][1].w, ph);
                    float f = acc[r][t];
                    f = __fmaf_rn((float)pl, __fmul_rn(dsLo, aS[t].x), f);
                    f = __fmaf_rn((float)ph, __fmul_rn(__fmul_rn(dsHi, aS[t].y), 0.0625f), f);  // ph = 16 * idot, 1/16 is exact
                    f = __fmaf_rn(nmLo, as[t].x, f);
                    acc[r][t] = __fmaf_rn(nmHi, as[t].y, f);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int t = 0; t < TT; t++) {
            float f = acc[r][t];
            f += __shfl_xor_sync(0xffffffffu, f, 1);
            f += __shfl_xor_sync(0xffffffffu, f, 2);
            if (j == 0) part[warp][r0 + 8 * r][t] = f;
        }
    __syncthreads();
    if (threadIdx.x < 16 * TT) {
        const int row = threadIdx.x / TT, t = threadIdx.x % TT, n = blockIdx.x * 16 + row;
        float f = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) f += part[w][row][t];
        if (n < N) dst[(size_t)t * ldd + n] = f;
    }
}

template <int TT>
int run_q4k_gemv(b200_ctx* ctx, const uint8_t* W, int N, int nSB, ActQ aq, float* dst, int ldd, int tiled = 0) {
    ProfScope ps(ctx, PROF_Q4K_GEMM);
    if (tiled) {
        launch_pdl(q4k_gemv_tiles_kernel<TT>, dim3(ceil_div(N, 16)), dim3(256), 0, ctx->stream, W, N, nSB, aq.codes, aq.scales, dst, ldd);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    // 2 rows per warp at one token, 4 at two or three (the activation loads are shared by a warp's rows)
    if (TT == 1) launch_pdl(q4k_gemv_dp4a_kernel<TT, 2, 1>, dim3(ceil_div(N, 16)), dim3(256), 0, ctx->stream, W, N, nSB, aq.codes, aq.scales, dst, ldd);
    else launch_pdl(q4k_gemv_dp4a_kernel<TT, 4, 1>, dim3(ceil_div(N, 32)), dim3(256), 0, ctx->stream, W, N, nSB, aq.codes, aq.scales, dst, ldd);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ---- f16 weights ----
__global__ void split_f16_kernel(const float* __restrict__ x, size_t n, __half* __restrict__ hi, __half* __restrict__ lo) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    __half h = __float2half_rn(v);
    hi[i] = h;
    lo[i] = __float2half_rn(__fsub_rn(v, __half2float(h)));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// dst[t][n] = sum_k W[n][k] * x[t][k], W f16, x as f16 hi + lo. K a multiple of 32. One warp per 16 weight rows.
template <int NT>
__global__ void __launch_bounds__(256) f16w_gemm_mma_kernel(const __half* __restrict__ W, int N, int K,
                                                            const __half* __restrict__ xhi, const __half* __restrict__ xlo,
                                                            int T, float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
    const int n0 = (blockIdx.x * 8 + warp) * 16;
    if (n0 >= N) return;
    const int t_base = blockIdx.y * 8 * NT;
    const __half* w0 = W + (size_t)min(n0 + gid, N - 1) * K + 8 * tig;
    const __half* w1 = W + (size_t)min(n0 + gid + 8, N - 1) * K + 8 * tig;
    const __half* bh[NT];
    const __half* bl[NT];
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        size_t t = (size_t)min(t_base + 8 * j + gid, T - 1);
        bh[j] = xhi + t * K + 8 * tig;
        bl[j] = xlo + t * K + 8 * tig;
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    }
    for (int k = 0; k < K; k += 32) {
        // halves [k+8*tig, +8) of both rows; the k order inside the 32-chunk is permuted alike for W and x
        const uint4 a = *reinterpret_cast<const uint4*>(w0 + k);
        const uint4 b = *reinterpret_cast<const uint4*>(w1 + k);
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const uint4 xh = *reinterpret_cast<const uint4*>(bh[j] + k);
            const uint4 xl = *reinterpret_cast<const uint4*>(bl[j] + k);
            mma_f16(acc[j], a.x, b.x, a.y, b.y, xh.x, xh.y);
            mma_f16(acc[j], a.z, b.z, a.w, b.w, xh.z, xh.w);
            mma_f16(acc[j], a.x, b.x, a.y, b.y, xl.x, xl.y);
            mma_f16(acc[j], a.z, b.z, a.w, b.w, xl.z, xl.w);
        }
    }
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int t0 = t_base + 8 * j + 2 * tig, t1 = t0 + 1;
        const int na = n0 + gid, nb = n0 + gid + 8;
        if (t0 < T) {
            if (na < N) dst[(size_t)t0 * ldd + na] = acc[j][0];
            if (nb < N) dst[(size_t)t0 * ldd + nb] = acc[j][2];
        }
        if (t1 < T) {
            if (na < N) dst[(size_t)t1 * ldd + na] = acc[j][1];
            if (nb < N) dst[(size_t)t1 * ldd + nb] = acc[j][3];
        }
    }
}

// generic fallback: one warp per output, f64 accumulate (any K; f16 or f32 weights)
template <typename WT>
__global__ void __launch_bounds__(256) dense_matmul_f64_kernel(const WT* __restrict__ W, int N, int K, const float* __restrict__ x,
                                                               float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), t = blockIdx.y;
    if (n >= N) return;
    const WT* w = W + (size_t)n * K;
    const float* xr = x + (size_t)t * K;
    double s = 0;
    for (int k = lane; k < K; k += 32) s += (double)xr[k] * (double)(float)w[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) dst[(size_t)t * ldd + n] = (float)s;
}

// The same sums for four tokens a warp (f32 weights: the router): a weight is loaded once for the four, and every
// output keeps the kernel above's order of additions (lane-strided partial sums in f64, then the xor fold), hence its bits.
__global__ void __launch_bounds__(256) dense_matmul_f64_tok4_kernel(const float* __restrict__ W, int N, int K, const float* __restrict__ x, int T,
                                                                    float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), t0 = blockIdx.y * 4;
    if (n >= N) return;
    const float* w = W + (size_t)n * K;
    const float* xr[4];
#pragma unroll
    for (int i = 0; i < 4; i++) xr[i] = x + (size_t)min(t0 + i, T - 1) * K;
    double s[4] = {0, 0, 0, 0};
    for (int k = lane; k < K; k += 32) {
        const double wv = (double)w[k];
#pragma unroll
        for (int i = 0; i < 4; i++) s[i] += (double)xr[i][k] * wv;
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s[i] += __shfl_xor_sync(0xffffffffu, s[i], o);
        if (lane == 0 && t0 + i < T) dst[(size_t)(t0 + i) * ldd + n] = (float)s[i];
    }
}

// The same sums again for a tile of TT tokens x 16 weight rows a block: the tokens' rows are brought into shared memory once
// as f64 (exact), a warp takes two of the 16 weight rows and reads each weight once for the TT tokens. A
// 128 x 128 router product over K = 2048 moves 25 MB through L2 instead of the 164 MB of the four-tokens-a-warp kernel.
// Dynamic shared memory: TT * K doubles.
template <int TT>
__global__ void __launch_bounds__(256) dense_matmul_f64_tile_kernel(const float* __restrict__ W, int N, int K, const float* __restrict__ x, int T,
                                                                    float* __restrict__ dst, int ldd) {
    extern __shared__ double xs[];   // [TT][K]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.y * TT;
    for (int tt = warp; tt < TT; tt += 8) {   // a warp brings a token's row in, several loads in flight a lane
        const float* xr = x + (size_t)min(t0 + tt, T - 1) * K;
        double* xd = xs + (size_t)tt * K;
        if ((K & 3) == 0 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
#pragma unroll 8
            for (int k = 4 * lane; k < K; k += 128) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(xr + k));
                *reinterpret_cast<double2*>(xd + k) = make_double2((double)v.x, (double)v.y);
                *reinterpret_cast<double2*>(xd + k + 2) = make_double2((double)v.z, (double)v.w);
            }
        } else {
#pragma unroll 8
            for (int k = lane; k < K; k += 32) xd[k] = (double)__ldg(xr + k);
        }
    }
    __syncthreads();
    // the warp's two weight rows side by side, four steps of K's loads in flight (a lane's weights are 128 bytes apart: the
    // loads' latency, not their count, is what a lane waits for)
    const int n0 = blockIdx.x * 16 + 2 * warp;
    if (n0 >= N) return;
    const bool two = n0 + 1 < N;
    const float* w0 = W + (size_t)n0 * K;
    const float* w1 = W + (size_t)(two ? n0 + 1 : n0) * K;
    double s0[TT], s1[TT];
#pragma unroll
    for (int i = 0; i < TT; i++) s0[i] = s1[i] = 0;
    int k = lane;
    float a[4], b[4], an[4], bn[4];   // this batch of four steps' weights and the next one's, already on their way
    if (k + 96 < K) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            a[u] = __ldg(w0 + k + 32 * u);
            b[u] = __ldg(w1 + k + 32 * u);
        }
    }
    for (; k + 96 < K; k += 128) {
        const bool more = k + 128 + 96 < K;
        if (more) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                an[u] = __ldg(w0 + k + 128 + 32 * u);
                bn[u] = __ldg(w1 + k + 128 + 32 * u);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const double av = (double)a[u], bv = (double)b[u];
#pragma unroll
            for (int i = 0; i < TT; i++) {
                const double xv = xs[i * K + k + 32 * u];
                s0[i] += xv * av;
                s1[i] += xv * bv;
            }
        }
        if (more) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                a[u] = an[u];
                b[u] = bn[u];
            }
        }
    }
    for (; k < K; k += 32) {
        const double av = (double)w0[k], bv = (double)w1[k];
#pragma unroll
        for (int i = 0; i < TT; i++) {
            const double xv = xs[i * K + k];
            s0[i] += xv * av;
            s1[i] += xv * bv;
        }
    }
#pragma unroll
    for (int i = 0; i < TT; i++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s0[i] += __shfl_xor_sync(0xffffffffu, s0[i], o);
            s1[i] += __shfl_xor_sync(0xffffffffu, s1[i], o);
        }
        if (lane == 0 && t0 + i < T) {
            dst[(size_t)(t0 + i) * ldd + n0] = (float)s0[i];
            if (two) dst[(size_t)(t0 + i) * ldd + n0 + 1] = (float)s1[i];
        }
    }
}

__global__ void __launch_bounds__(256) dense_matmul_f64_grouped_kernel(const float* const* __restrict__ Wptrs, int N, int K,
                                                                       const float* __restrict__ x,
                                                                       const int32_t* __restrict__ offs,
                                                                       const int32_t* __restrict__ rows,
                                                                       float* __restrict__ dst, int ldd) {
    const int lane = threadIdx.x & 31, e = blockIdx.z;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), a = offs[e] + blockIdx.y;
    if (n >= N || a >= offs[e + 1]) return;
    const float* w = Wptrs[e] + (size_t)n * K;
    const float* xr = x + (size_t)(rows ? rows[a] : a) * K;
    double s = 0;
    for (int k = lane; k < K; k += 32) s += (double)xr[k] * (double)w[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) dst[(size_t)a * ldd + n] = (float)s;
}

// ---- Q4_K block utilities ----
__global__ void q4k_dequant_kernel(const uint8_t* __restrict__ W, size_t n_blocks, float* __restrict__ out) {
    const size_t blk = blockIdx.x;
    if (blk >= n_blocks) return;
    const uint8_t* b = W + blk * 144;
    const uint4 h = *reinterpret_cast<const uint4*>(b);
    const float d = kq_h2f((unsigned short)(h.x & 0xffffu)), dmin = kq_h2f((unsigned short)(h.x >> 16));
    const int e = threadIdx.x;  // 0..255
    const int j = e >> 5, p = e >> 6, l = e & 31;
    int sc, m;
    kq_scale_min(j, h.y, h.z, h.w, &sc, &m);
    const uint8_t q = b[16 + 32 * p + l];
    const int code = (j & 1) ? (q >> 4) : (q & 0x0F);
    out[blk * 256 + e] = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)code), __fmul_rn(dmin, (float)m));
}

// One thread per super-block; the arithmetic is the host quantizer's, operation for operation.
__device__ void q4k_quantize_block_dev(const float* __restrict__ w, uint8_t* __restrict__ blk) {
    float scale[8], mn[8];
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; j++) {
        float lo = w[32 * j], hi = w[32 * j];
        for (int i = 1; i < 32; i++) {
            lo = fminf(lo, w[32 * j + i]);
            hi = fmaxf(hi, w[32 * j + i]);
        }
        float m = lo < 0.f ? -lo : 0.f;
        float s = __fdiv_rn(__fadd_rn(hi, m), 15.f);
        if (s < 0.f) s = 0.f;
        scale[j] = s;
        mn[j] = m;
        max_scale = fmaxf(max_scale, s);
        max_min = fmaxf(max_min, m);
    }
    const __half hd = __float2half_rn(__fdiv_rn(max_scale, 63.f)), hm = __float2half_rn(__fdiv_rn(max_min, 63.f));
    const float d = __half2float(hd), dmin = __half2float(hm);
    int sc[8], m6[8];
    for (int j = 0; j < 8; j++) {
        sc[j] = d > 0.f ? max(0, min(63, __float2int_rn(__fdiv_rn(scale[j], d)))) : 0;
        m6[j] = dmin > 0.f ? max(0, min(63, __float2int_rn(__fdiv_rn(mn[j], dmin)))) : 0;
    }
    uint8_t hdr[16];
    const unsigned short hdb = __half_as_ushort(hd), hmb = __half_as_ushort(hm);
    hdr[0] = hdb & 0xff; hdr[1] = hdb >> 8; hdr[2] = hmb & 0xff; hdr[3] = hmb >> 8;
    for (int i = 4; i < 16; i++) hdr[i] = 0;
    for (int j = 0; j < 8; j++) {
        if (j < 4) {
            hdr[4 + j] |= (uint8_t)(sc[j] & 63);
            hdr[4 + j + 4] |= (uint8_t)(m6[j] & 63);
        } else {
            hdr[4 + j + 4] |= (uint8_t)((sc[j] & 0x0F) | ((m6[j] & 0x0F) << 4));
            hdr[4 + j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
            hdr[4 + j] |= (uint8_t)((m6[j] >> 4) << 6);
        }
    }
    for (int i = 0; i < 16; i++) blk[i] = hdr[i];
    for (int p = 0; p < 4; p++) {
        const float dsl = __fmul_rn(d, (float)sc[2 * p]), dml = __fmul_rn(dmin, (float)m6[2 * p]);
        const float dsh = __fmul_rn(d, (float)sc[2 * p + 1]), dmh = __fmul_rn(dmin, (float)m6[2 * p + 1]);
        const float il = dsl > 0.f ? __fdiv_rn(1.f, dsl) : 0.f, ih = dsh > 0.f ? __fdiv_rn(1.f, dsh) : 0.f;
        for (int l = 0; l < 32; l++) {
            int cl = __float2int_rn(__fmul_rn(__fadd_rn(w[64 * p + l], dml), il));
            int ch = __float2int_rn(__fmul_rn(__fadd_rn(w[64 * p + 32 + l], dmh), ih));
            cl = max(0, min(15, cl));
            ch = max(0, min(15, ch));
            blk[16 + 32 * p + l] = (uint8_t)(cl | (ch << 4));
        }
    }
}

__global__ void q4k_quantize_kernel(const float* __restrict__ w, size_t n_blocks, uint8_t* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_blocks) q4k_quantize_block_dev(w + i * 256, out + i * 144);
}

// counter-based normal generator (splitmix64 hash -> Box-Muller)
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t i) {
    uint64_t r = mix64(seed * 0xD1342543DE82EF95ull + i);
    float u1 = ((float)((r >> 40) + 1)) * (1.0f / 16777217.0f);
    float u2 = ((float)((r >> 8) & 0xFFFFFF)) * (1.0f / 16777216.0f);
    return sqrtf(-2.f * logf(u1)) * cospif(2.f * u2);
}

__global__ void synth_f32_kernel(float* out, size_t n, float sigma, uint64_t seed) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = sigma * normal_at(seed, i);
}
__global__ void synth_f16_kernel(__half* out, size_t n, float sigma, uint64_t seed) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(sigma * normal_at(seed, i));
}
__global__ void synth_q4k_kernel(uint8_t* out, size_t n_blocks, float sigma, uint64_t seed) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks) return;
    float w[256];
    for (int e = 0; e < 256; e++) w[e] = sigma * normal_at(seed, i * 256 + e);
    q4k_quantize_block_dev(w, out + i * 144);
}

template <int NT, bool SPLITK>
int run_q4k(b200_ctx* ctx, const uint8_t* W, int N, int nSB, ActQ aq, int T, float* dst, int ldd) {
    dim3 grid(SPLITK ? ceil_div(N, 16) : ceil_div(N, 128), ceil_div(T, 8 * NT));
    ProfScope ps(ctx, PROF_Q4K_GEMM);
    q4k_gemm_mma_kernel<NT, SPLITK, false><<<grid, 256, 0, ctx->stream>>>(W, nullptr, N, nSB, aq.codes, aq.scales, T, nullptr,
                                                                         nullptr, dst, ldd);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

int launch_q4k_matmul(b200_ctx* ctx, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, int klass, const uint8_t* W_tiles) {
    if (K % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "Q4_K needs K %% 256 == 0");
    const int nSB = K / 256;
    // Fast class from 33 rows (or when asked for by klass 2): tcgen05 fp16 matmul, if its scratch is in place. (Measured:
    // at 45 rows it takes 111 us on a 28672x8192 matrix against 214 us for the integer kernels; below 33 rows the
    // streaming integer kernel is the faster one.)
    static const bool no_umma_env = getenv("B200_NO_UMMA") != nullptr;
    if (klass != B200_CLASS_EXACT && klass != 3 && klass != 4 && klass != 5 && klass != 6 && (T >= 33 || klass == 2) && ctx->umma_scratch && !no_umma_env &&
        q4k_umma_scratch_bytes(T, K, N) <= ctx->umma_scratch_bytes)
        return launch_q4k_matmul_umma(ctx, W, N, K, aq, T, dst, ldd, ctx->umma_scratch, ctx->umma_scratch_bytes, ctx->err_flag, W_tiles);
    // Fast class, up to 32 rows (klass 5 forces it): fp16 dequant in registers + mma.sync, the weights streamed once
    {
        const int small_min = q4k_small_min_rows();
        const bool fast = klass == 0 || klass == 2;
        if (W_tiles && (klass == 5 || (fast && small_min > 0 && T >= small_min)) && T <= 32 && ctx->umma_scratch && !no_umma_env &&
            q4k_umma_scratch_bytes(T, K, N) <= ctx->umma_scratch_bytes)
            return launch_q4k_matmul_small(ctx, W_tiles, N, K, aq, T, dst, ldd);
        if (klass == 5) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the small-batch Q4_K matmul needs the tiled weights, 1..32 rows and the fast class's scratch");
    }
    if (!W) {
        // only the tile-major copy is resident (a fast-class model drops the row-major one): the kernels that read it
        if (!W_tiles) B200_FAIL(ctx, B200_BAD_ARGUMENT, "no weights");
        if (T == 1) return run_q4k_gemv<1>(ctx, W_tiles, N, nSB, aq, dst, ldd, 1);
        if (T == 2) return run_q4k_gemv<2>(ctx, W_tiles, N, nSB, aq, dst, ldd, 1);
        if (T == 3) return run_q4k_gemv<3>(ctx, W_tiles, N, nSB, aq, dst, ldd, 1);
        if (T <= 32 && ctx->umma_scratch) return launch_q4k_matmul_small(ctx, W_tiles, N, K, aq, T, dst, ldd);
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "this row count or kernel class needs the row-major Q4_K matrix, which this model did not keep");
    }
    // Rows up to 8 are HBM-bound: split K over the CTA's warps (unless the exact class asks for the one ascending
    // chain per output that every larger batch uses, so a row's bits do not depend on its batch).
    if (T <= 8 && klass == B200_CLASS_EXACT) return run_q4k<1, false>(ctx, W, N, nSB, aq, T, dst, ldd);
    if (klass == 4 && T <= 64 && (reinterpret_cast<uintptr_t>(W) & 15) == 0) return launch_q4k_matmul_stream(ctx, W, N, K, aq, T, dst, ldd, false);
    if (T == 1) return run_q4k_gemv<1>(ctx, W, N, nSB, aq, dst, ldd);
    if (T == 2) return run_q4k_gemv<2>(ctx, W, N, nSB, aq, dst, ldd);
    if (T == 3) return run_q4k_gemv<3>(ctx, W, N, nSB, aq, dst, ldd);
    // 4..63 rows, fast class: the weights stream through a TMA ring (klass 3 forces the older kernels for comparison)
    static const bool no_stream = getenv("B200_NO_STREAM") != nullptr;
    if (T <= 63 && klass != B200_CLASS_EXACT && klass != 3 && !no_stream && (reinterpret_cast<uintptr_t>(W) & 15) == 0)
        return launch_q4k_matmul_stream(ctx, W, N, K, aq, T, dst, ldd, klass != 4);  // klass 4: the one-chain form (the exact class's bits); 6: split
    if (T <= 8) return run_q4k<1, true>(ctx, W, N, nSB, aq, T, dst, ldd);
    if (T <= 16) return run_q4k<2, false>(ctx, W, N, nSB, aq, T, dst, ldd);
    if (T <= 32) return run_q4k_tile<4>(ctx, W, N, nSB, aq, T, dst, ldd);
    return run_q4k_tile<8>(ctx, W, N, nSB, aq, T, dst, ldd);
}

int launch_q4k_matmul_grouped(b200_ctx* ctx, const uint8_t* const* Wptrs, int n_experts, int N, int K, ActQ aq,
                              const int32_t* offs, const int32_t* rows, int max_rows_per_expert, float* dst, int ldd) {
    if (K % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "Q4_K needs K %% 256 == 0");
    constexpr int NT = 2, smem = 2 * (8 * NT) * (288 + 80);
    dim3 grid(ceil_div(N, 128), ceil_div(max_rows_per_expert, 8 * NT), n_experts);
    ProfScope ps(ctx, PROF_Q4K_GEMM);
    q4k_gemm_tile_kernel<NT, true><<<grid, 256, smem, ctx->stream>>>(nullptr, Wptrs, N, K / 256, aq.codes, aq.scales, 0, offs,
                                                                     rows, dst, ldd);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

// split_scratch: 2*T*K halves (the activation's f16 hi and lo parts), owned by the caller.
int launch_f16w_matmul(b200_ctx* ctx, const __half* W, int N, int K, const float* x, int T, float* dst, int ldd,
                       __half* split_scratch, int klass) {
    // fast class, dense row counts (or forced with klass 2): the tcgen05 kernel
    static const bool no_umma = getenv("B200_NO_UMMA") != nullptr;
    if (klass != B200_CLASS_EXACT && (T >= 32 || klass == 2) && !no_umma && ctx->umma_scratch && f16w_umma_supported(W, N, K) &&
        f16w_umma_scratch_bytes(T, K) <= ctx->umma_scratch_bytes)
        return launch_f16w_matmul_umma(ctx, W, N, K, x, T, dst, ldd, ctx->umma_scratch, ctx->umma_scratch_bytes, ctx->err_flag);
    if (K % 32) {
        dim3 grid(ceil_div(N, 8), T);
        dense_matmul_f64_kernel<__half><<<grid, 256, 0, ctx->stream>>>(W, N, K, x, dst, ldd);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    size_t n = (size_t)T * K;
    __half* hi = split_scratch;
    __half* lo = split_scratch + n;
    split_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x, n, hi, lo);
    LAUNCH_CHECK(ctx);
    ProfScope ps(ctx, PROF_HEAD_GEMM);
    if (T <= 8) {
        dim3 grid(ceil_div(N, 128), ceil_div(T, 8));
        f16w_gemm_mma_kernel<1><<<grid, 256, 0, ctx->stream>>>(W, N, K, hi, lo, T, dst, ldd);
    } else if (T <= 32) {
        dim3 grid(ceil_div(N, 128), ceil_div(T, 32));
        f16w_gemm_mma_kernel<4><<<grid, 256, 0, ctx->stream>>>(W, N, K, hi, lo, T, dst, ldd);
    } else {
        dim3 grid(ceil_div(N, 128), ceil_div(T, 64));
        f16w_gemm_mma_kernel<8><<<grid, 256, 0, ctx->stream>>>(W, N, K, hi, lo, T, dst, ldd);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_f32w_matmul(b200_ctx* ctx, const float* W, int N, int K, const float* x, int T, float* dst, int ldd) {
    if (T >= 8 && (size_t)8 * K * sizeof(double) <= 200 * 1024) {   // the tokens' rows fit a block's shared memory as f64
        const size_t smem = (size_t)8 * K * sizeof(double);
        static PerDeviceOnce attr_once;  // the attribute belongs to the device
        if (attr_once.first(ctx->device))
            CUDA_TRY(ctx, cudaFuncSetAttribute(dense_matmul_f64_tile_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        dense_matmul_f64_tile_kernel<8><<<dim3(ceil_div(N, 16), ceil_div(T, 8)), 256, smem, ctx->stream>>>(W, N, K, x, T, dst, ldd);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    if (T >= 4) {
        dense_matmul_f64_tok4_kernel<<<dim3(ceil_div(N, 8), ceil_div(T, 4)), 256, 0, ctx->stream>>>(W, N, K, x, T, dst, ldd);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    dim3 grid(ceil_div(N, 8), T);
    dense_matmul_f64_kernel<float><<<grid, 256, 0, ctx->stream>>>(W, N, K, x, dst, ldd);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_f32w_matmul_grouped(b200_ctx* ctx, const float* const* Wptrs, int n_experts, int N, int K, const float* x,
                               const int32_t* offs, const int32_t* rows, int max_rows_per_expert, float* dst, int ldd) {
    dim3 grid(ceil_div(N, 8), max_rows_per_expert, n_experts);
    dense_matmul_f64_grouped_kernel<<<grid, 256, 0, ctx->stream>>>(Wptrs, N, K, x, offs, rows, dst, ldd);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_q4k_dequant(b200_ctx* ctx, const uint8_t* W, size_t n_blocks, float* out) {
    q4k_dequant_kernel<<<(unsigned)n_blocks, 256, 0, ctx->stream>>>(W, n_blocks, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_q4k_quantize(b200_ctx* ctx, const float* w, size_t n_blocks, uint8_t* out) {
    q4k_quantize_kernel<<<(unsigned)((n_blocks + 127) / 128), 128, 0, ctx->stream>>>(w, n_blocks, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_synth_normal_f32(b200_ctx* ctx, float* out, size_t n, float sigma, uint64_t seed) {
    synth_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(out, n, sigma, seed);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}
int launch_synth_f16(b200_ctx* ctx, __half* out, size_t n, float sigma, uint64_t seed) {
    synth_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(out, n, sigma, seed);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}
int launch_synth_q4k(b200_ctx* ctx, uint8_t* out, size_t n_blocks, float sigma, uint64_t seed) {
    synth_q4k_kernel<<<(unsigned)((n_blocks + 63) / 64), 64, 0, ctx->stream>>>(out, n_blocks, sigma, seed);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

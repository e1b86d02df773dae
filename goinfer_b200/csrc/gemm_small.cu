// gemm_small.cu — fast-class Q4_K matmul for up to 32 packed rows (decode at small batch): the weight matrix is streamed
// exactly once and the kernel is meant to run at the speed of that stream.
//
//   dst[t][n] = sum_k W[n][k] * x[t][k],   W Q4_K,   x = fp16(code * scale) of the per-32 quantizer
//
// What is built around the hardware here:
//  * Weight layout. The matrix is kept tile by tile: [row tile of 16][super-block][16 rows][144 B] (the GGUF blocks unchanged,
//    reordered at finalize by q4k_to_tiles_kernel). A warp owns a row tile, so everything it reads is one contiguous run and a
//    stage of its ring is a single bulk copy of 2 super-blocks x 16 rows = 4608 bytes. (Measured: 144-byte-wide tiled TMA boxes
//    of the row-major matrix reach 2.8-4.2 TB/s on this part however deep the ring, the copy engine spends its time on box rows;
//    contiguous copies of the same bytes run at the speed of a plain read.)
//  * Weights never pass through a dequantized copy. Lanes read their 32 code bytes and the 16-byte header from the ring with
//    bank-conflict-free 16-byte loads, turn nibbles into fp16 in registers and feed them to mma.sync m16n8k16 as the 16-row
//    operand straight from registers.
//  * The sum over K does not care about the order of its terms, so the order is chosen for the loads: lane (gid, p) of a
//    warp owns sub-block pair p of rows gid and gid + 8, i.e. 32 consecutive code bytes per row, and an MMA's sixteen k
//    positions are four consecutive code bytes of each of the four pairs. The activation tiles are written in that order by
//    the kernels that quantize activations (x16_store8 in common.cuh), so a lane's eight-token operand is one 16-byte load
//    per two MMAs.
//  * The activation tiles of a stage ([tokens][512] fp16) are shared by the CTA's warps through a second ring, filled by plain
//    bulk copies and handed back with an mbarrier on which every warp arrives.
//  * Several CTAs per SM: the loads of one overlap the arithmetic of another; narrow matrices are split over K so that every
//    SM has work, with the partial sums left for the consumer kernel (or summed by a small kernel) in a fixed order.
// Every wait is bounded: on expiry the CTA raises the error flag, waits (bounded) for the copies it started and returns.
//
// Arithmetic: w = d sc q - dmin m is split into its two terms. The code term runs on the tensor cores as (q * ds) x
// activation with ds = fp16(d sc): a nibble is or-ed into the mantissa of a half whose unit in the last place is 1 (1024 for
// low nibbles, 64 for high ones, so no shift is needed), and one half2 fma computes (M + q) * ds - M * ds = q * ds with a
// single rounding. The minimum term is a second, small product: -(dmin m)[row][sub-block] x asum[sub-block][token], one
// m16n8k8 MMA per super-block, with asum the per-32 sums the quantizer already wrote. fp16 operands, fp32 accumulation: the
// fast class's tolerance, the same as the tcgen05 matmul's for 33 rows and more. The reference's per-group integer formula
// (backend/cuda/actgroup.cu:311-355) stays with the exact class.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kq_common.cuh"
#include "umma.cuh"

namespace {

constexpr int kSmWarps = 8;
constexpr int kSmThreads = kSmWarps * 32;
constexpr int kTileBytes16 = 16 * 144;   // one super-block of a 16-row tile

template <int NT, int MT>
struct SmallCfg {
    static constexpr int kTpad = 8 * NT;                        // token rows an MMA column operand covers
    static constexpr int kSbw = MT == 2 ? 1 : 2;                // super-blocks per ring stage
    static constexpr int kWStage = MT * kSbw * kTileBytes16;    // a stage of a warp's weight ring: [MT row tiles][kSbw super-blocks][16 rows][144]
    static constexpr int kWDepth = 2;
    static constexpr int kChunk = kTpad * 128 + 32;             // 64 k of every token row; 32 bytes of skew keep the four pairs' loads off each other's banks
    static constexpr int kAStage = kSbw * 4 * kChunk;           // the activation tiles of a stage
    static constexpr int kADepth = 2;
    static constexpr int kSmem = kSmWarps * kWDepth * kWStage + kADepth * kAStage + 1024;
};

__device__ __forceinline__ void mma_f16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16_k8(float (&d)[4], unsigned a0, unsigned a1, unsigned b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

__device__ __forceinline__ __half2 as_h2(unsigned u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ unsigned as_u32(__half2 h) { return *reinterpret_cast<unsigned*>(&h); }
__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// (w & mask) | magic in one LOP3: both constants must sit in registers for that (as immediates the compiler spends two
// instructions per nibble pair, and this is the kernel's hottest line), so they are handed over as opaque values
__device__ __forceinline__ unsigned and_or(unsigned w, unsigned mask, unsigned magic) {
    unsigned r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "r"(mask), "r"(magic));
    return r;
}
__device__ __forceinline__ unsigned opaque(unsigned v) {
    unsigned r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
struct NibbleConsts {
    unsigned mask_lo, magic_lo, mask_hi, magic_hi;   // 0x000F000F | 1024.0 halves; 0x00F000F0 | 64.0 halves
};
// low nibbles of bytes 0 and 2 of w -> {q0, q2} * ds (the half 1024 + q, times ds, minus 1024 ds: one rounding)
__device__ __forceinline__ unsigned deq_lo(unsigned w, __half2 ds, __half2 c, const NibbleConsts& k) {
    return as_u32(__hfma2(as_h2(and_or(w, k.mask_lo, k.magic_lo)), ds, c));
}
// high nibbles of bytes 0 and 2 (the half 64 + q)
__device__ __forceinline__ unsigned deq_hi(unsigned w, __half2 ds, __half2 c, const NibbleConsts& k) {
    return as_u32(__hfma2(as_h2(and_or(w, k.mask_hi, k.magic_hi)), ds, c));
}

struct RowScales {
    __half2 ds_lo, c_lo, ds_hi, c_hi;  // sub-block 2p: scale and -1024 * scale; sub-block 2p+1: scale and -64 * scale
    unsigned neg_dm;                   // {-(dmin m)(2p), -(dmin m)(2p+1)} as a half2: this lane's part of the minimum term's operand
};

// scales and minima of sub-blocks 2p and 2p+1 of one row's super-block, from its 16-byte header (the 6-bit fields of both
// sub-blocks are pulled out two at a time: they sit in neighbouring bytes)
__device__ __forceinline__ RowScales row_scales(const uint4 hdr, int p) {
    unsigned scs, ms;   // {sc(2p), sc(2p+1)} and {m(2p), m(2p+1)} in the two low bytes
    if (p < 2) {
        scs = (hdr.y >> (16 * p)) & 0x3F3Fu;
        ms = (hdr.z >> (16 * p)) & 0x3F3Fu;
    } else {
        const int sh = 16 * (p - 2);
        const unsigned lo = hdr.w >> sh;
        scs = (lo & 0x0F0Fu) | (((hdr.y >> sh) >> 2) & 0x3030u);
        ms = ((lo >> 4) & 0x0F0Fu) | (((hdr.z >> sh) >> 2) & 0x3030u);
    }
    // bytes -> halves: the byte or-ed into the mantissa of 1024, minus 1024
    const __half2 k1024 = __float2half2_rn(1024.f);
    const __half2 sc2 = __hsub2(as_h2(prmt(scs, 0u, 0x4140u) | 0x64006400u), k1024);
    const __half2 m2 = __hsub2(as_h2(prmt(ms, 0u, 0x4140u) | 0x64006400u), k1024);
    const __half2 d2 = as_h2(prmt(hdr.x, 0u, 0x1010u)), dmin2 = as_h2(prmt(hdr.x, 0u, 0x3232u));
    const __half2 ds2 = __hmul2(d2, sc2);          // {ds(2p), ds(2p+1)}, each rounded to fp16 once
    RowScales r;
    r.ds_lo = as_h2(prmt(as_u32(ds2), 0u, 0x1010u));
    r.ds_hi = as_h2(prmt(as_u32(ds2), 0u, 0x3232u));
    r.c_lo = __hmul2(r.ds_lo, __float2half2_rn(-1024.f));   // exact: a power of two
    r.c_hi = __hmul2(r.ds_hi, __float2half2_rn(-64.f));
    r.neg_dm = as_u32(__hmul2(dmin2, m2)) ^ 0x80008000u;
    return r;
}

// grid (groups of 8*MT row tiles, K ranges); block 256. w16: the matrix tile by tile; n_tiles = ceil(N / 16).
// GROUPED (routed experts): grid (groups of row tiles, 1, experts); w16 holds the experts' matrices one after the other
// (n_tiles tiles each), x16 / scales / out rows are the token-expert pairs in expert order, and expert e owns rows
// offs[e] .. offs[e+1]: the CTA walks them 8*NT at a time (the weights of a second pass come out of L2) and skips the
// MMAs of 8-row groups past the expert's last row; an expert without rows costs its CTAs one load of offs.
template <int NT, int MT, bool GROUPED>
__global__ void __launch_bounds__(kSmThreads, 2) q4k_small_kernel(const uint8_t* __restrict__ w16, int n_tiles,
                                                                                               const __half* __restrict__ x16,
                                                                                               const float* __restrict__ scales, int N, int nSB,
                                                                                               int sb_per_split, int T, float* __restrict__ out, int ldo,
                                                                                               size_t split_stride, int* __restrict__ err_flag,
                                                                                               const int32_t* __restrict__ offs) {
    using Cfg = SmallCfg<NT, MT>;
    constexpr int kSbw = Cfg::kSbw;
    pdl_trigger();
    extern __shared__ __align__(1024) uint8_t sm_raw[];
    __shared__ __align__(8) uint64_t wfull[kSmWarps][3], afull[3], aempty[3];
    __shared__ int abort_s;
    uint8_t* smem = sm_raw + ((1024u - (smem_u32(sm_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, p = lane & 3;
    const int tile_l = (blockIdx.x * kSmWarps + warp) * MT;          // first 16-row tile of this warp (within its matrix)
    const int tile0 = tile_l + (GROUPED ? (int)blockIdx.z * n_tiles : 0);
    const int row0 = tile_l * 16;
    const int b_lo = GROUPED ? 0 : blockIdx.y * sb_per_split, n_sb = max(0, min(nSB, b_lo + sb_per_split) - b_lo);
    const int n_it = (n_sb + kSbw - 1) / kSbw;                       // stages; the last may hold fewer super-blocks
    uint8_t* wring = smem + (size_t)warp * Cfg::kWDepth * Cfg::kWStage;
    uint8_t* aring = smem + (size_t)kSmWarps * Cfg::kWDepth * Cfg::kWStage;
    volatile int* abort_v = &abort_s;

    if (tid == 0) {
        for (int w = 0; w < kSmWarps; w++)
            for (int s = 0; s < Cfg::kWDepth; s++) mbar_init(smem_u32(&wfull[w][s]), 1);
        for (int s = 0; s < Cfg::kADepth; s++) {
            mbar_init(smem_u32(&afull[s]), 1);
            mbar_init(smem_u32(&aempty[s]), kSmWarps);
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    int rbase = 0;   // first activation / output row of the pass

    // stage i of this warp: super-blocks b_lo + kSbw i .. of its row tiles, one contiguous run per tile
    auto issue_w = [&](int i, int stage) {
        const int b = b_lo + kSbw * i, nb = min(kSbw, b_lo + n_sb - b);
        const unsigned bar = smem_u32(&wfull[warp][stage]);
        int live = 0;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) live += (tile_l + mt < n_tiles) ? 1 : 0;
        mbar_arrive_expect_tx(bar, (unsigned)(live * nb * kTileBytes16));   // a warp past the matrix arrives with no bytes to wait for
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
            if (tile_l + mt < n_tiles)
                bulk_g2s(smem_u32(wring + (size_t)stage * Cfg::kWStage + (size_t)mt * kSbw * kTileBytes16),
                         w16 + ((size_t)(tile0 + mt) * nSB + b) * kTileBytes16, (unsigned)(nb * kTileBytes16), bar);
    };
    // the CTA's activation tiles of stage i: per super-block four 64-wide chunks of kTpad token rows from row rbase on (the
    // fp16 matrix is [token tile of 256][chunk of 64 along K][256 rows][64]: a run of rows that crosses a token tile is two copies)
    auto issue_a = [&](int i, int stage) {
        const int b = b_lo + kSbw * i, nb = min(kSbw, b_lo + n_sb - b);
        const unsigned bar = smem_u32(&afull[stage]);
        mbar_arrive_expect_tx(bar, (unsigned)(nb * 4 * Cfg::kTpad * 128));
        const int tt = rbase >> 8, r_in = rbase & 255, n1 = min(Cfg::kTpad, 256 - r_in);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(x16) + ((size_t)tt * (4 * nSB) + 4 * b) * (256 * 128) + (size_t)r_in * 128;
        const unsigned dst = smem_u32(aring + (size_t)stage * Cfg::kAStage);
        for (int c = 0; c < 4 * nb; c++) {
            bulk_g2s(dst + c * Cfg::kChunk, src + (size_t)c * (256 * 128), n1 * 128, bar);
            if (n1 < Cfg::kTpad)
                bulk_g2s(dst + c * Cfg::kChunk + n1 * 128, src + ((size_t)(4 * nSB) + c) * (256 * 128) - (size_t)r_in * 128, (Cfg::kTpad - n1) * 128, bar);
        }
    };

    // weights are written by nobody: their first stages start before the wait on the kernel ahead of this one (a routed
    // expert's CTAs first have to learn whether the expert has rows at all)
    int w_issued = 0, a_issued = 0;
    if (!GROUPED && lane == 0)
        for (; w_issued < min(Cfg::kWDepth, n_it); w_issued++) issue_w(w_issued, w_issued);
    pdl_wait();
    int r_begin = 0, T_e = T;
    if (GROUPED) {
        r_begin = offs[blockIdx.z];
        T_e = offs[blockIdx.z + 1] - r_begin;
    }
    const int sg = GROUPED ? ((gid + (r_begin & 7)) & 7) : gid;   // the activation rows' swizzle goes by their place in the whole matrix; passes are 8*NT rows apart

    // two accumulators per output tile where the registers allow: the low and the high sub-block of a pair feed different
    // ones, which halves the chain of dependent MMAs; they are added at the end
    constexpr bool kTwoAcc = MT * NT <= 2;
    constexpr int NA = kTwoAcc ? NT : 1, MA = kTwoAcc ? MT : 1;
    const NibbleConsts kc{opaque(0x000F000Fu), opaque(0x64006400u), opaque(0x00F000F0u), opaque(0x54005400u)};
    const float* asum_base = scales + (size_t)8 * nSB + 2 * p;
    int ws = 0, as = 0;
    unsigned wph = 0, aph = 0;   // ring positions and the phase parities of their barriers: they run on from pass to pass
    const int n_pass = GROUPED ? (T_e + Cfg::kTpad - 1) / Cfg::kTpad : 1;
#pragma unroll 1
    for (int pass = 0; pass < n_pass; pass++) {
    rbase = r_begin + pass * Cfg::kTpad;
    const int Tc = min(Cfg::kTpad, T_e - pass * Cfg::kTpad), nt_live = (Tc + 7) >> 3;
    const int ws0 = ws, as0 = as;
    const unsigned wph0 = wph, aph0 = aph;
    if (GROUPED || pass > 0) {   // (a dense launch started its first weight stages above)
        w_issued = 0;
        if (lane == 0)
            for (; w_issued < min(Cfg::kWDepth, n_it); w_issued++) issue_w(w_issued, (ws0 + w_issued) % Cfg::kWDepth);
    }
    a_issued = 0;
    if (tid == 0)
        for (; a_issued < min(Cfg::kADepth, n_it); a_issued++) issue_a(a_issued, (as0 + a_issued) % Cfg::kADepth);
    float acc[MT][NT][4], acc2[MA][NA][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[mt][nt][e] = 0.f;
#pragma unroll
    for (int mt = 0; mt < MA; mt++)
#pragma unroll
        for (int nt = 0; nt < NA; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc2[mt][nt][e] = 0.f;

    // group sums of this lane's token rows for sub-blocks 2p, 2p+1 of a super-block (the minimum term's operand); a stage's
    // sums are loaded while the stage before it is multiplied
    auto load_asum = [&](int i, unsigned (&dst)[kSbw][NT]) {
#pragma unroll
        for (int u = 0; u < kSbw; u++) {
            const int b = b_lo + kSbw * i + u;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int tl = 8 * nt + gid;
                const float2 v = (tl < Tc && b < b_lo + n_sb) ? __ldg(reinterpret_cast<const float2*>(asum_base + (size_t)(rbase + tl) * 16 * nSB + 8 * b)) : make_float2(0.f, 0.f);
                dst[u][nt] = as_u32(__floats2half2_rn(v.x, v.y));
            }
        }
    };
    unsigned asum[kSbw][NT], asum_next[kSbw][NT];
    load_asum(0, asum_next);

    int done = 0;
#pragma unroll 1
    for (int i = 0; i < n_it; i++) {
#pragma unroll
        for (int u = 0; u < kSbw; u++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) asum[u][nt] = asum_next[u][nt];
        load_asum(i + 1, asum_next);
        bool ok = mbar_wait(smem_u32(&wfull[warp][ws]), wph, abort_v);
        ok = ok && mbar_wait(smem_u32(&afull[as]), aph, abort_v);
        if (!__all_sync(0xffffffffu, ok)) {
            abort_s = 1;
            break;
        }
        const int nb = min(kSbw, n_sb - kSbw * i);
#pragma unroll
        for (int u = 0; u < kSbw; u++) {
            if (u >= nb) break;
            const uint8_t* wst = wring + (size_t)ws * Cfg::kWStage + (size_t)u * kTileBytes16;
            const uint8_t* ast = aring + (size_t)as * Cfg::kAStage + (size_t)(4 * u + p) * Cfg::kChunk + (size_t)gid * 128;
            // raw code words and scales of this lane's rows: row (gid + 8 hr) of tile mt, bytes 32 p .. 32 p + 31 of its code block
            unsigned wq[MT][2][8];
            RowScales rs[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    const uint8_t* rowp = wst + (size_t)mt * kSbw * kTileBytes16 + (size_t)(gid + 8 * hr) * 144;
                    const uint4 hdr = *reinterpret_cast<const uint4*>(rowp);
                    const uint4 qa = *reinterpret_cast<const uint4*>(rowp + 16 + 32 * p);
                    const uint4 qb = *reinterpret_cast<const uint4*>(rowp + 32 + 32 * p);
                    wq[mt][hr][0] = qa.x; wq[mt][hr][1] = qa.y; wq[mt][hr][2] = qa.z; wq[mt][hr][3] = qa.w;
                    wq[mt][hr][4] = qb.x; wq[mt][hr][5] = qb.y; wq[mt][hr][6] = qb.z; wq[mt][hr][7] = qb.w;
                    rs[mt][hr] = row_scales(hdr, p);
                }
            // the minimum term: -(dmin m)[rows][sub-blocks 2p, 2p+1] x asum[sub-blocks][tokens], k = the super-block's 8 sub-blocks
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                    if (!GROUPED || nt < nt_live) mma_f16_k8(acc[mt][nt], rs[mt][0].neg_dm, rs[mt][1].neg_dm, asum[u][nt]);
            }
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                // 16-byte pieces jj (elements 8 jj .. 8 jj + 7 of the low sub-block) and jj + 4 (of the high one) of this lane's
                // token rows: {x, y} is the operand of code word 2 jj, {z, w} of code word 2 jj + 1
                uint4 bl[NT], bh[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    bl[nt] = *reinterpret_cast<const uint4*>(ast + (size_t)nt * (8 * 128) + ((jj ^ sg) << 4));
                    bh[nt] = *reinterpret_cast<const uint4*>(ast + (size_t)nt * (8 * 128) + (((jj + 4) ^ sg) << 4));
                }
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
#pragma unroll
                    for (int hw = 0; hw < 2; hw++) {
                        const unsigned w0 = wq[mt][0][2 * jj + hw], w1 = wq[mt][1][2 * jj + hw];
                        const unsigned w0s = w0 >> 8, w1s = w1 >> 8;   // bytes 1 and 3 where bytes 0 and 2 were
                        {   // low nibbles: sub-block 2p
                            const unsigned a0 = deq_lo(w0, rs[mt][0].ds_lo, rs[mt][0].c_lo, kc), a1 = deq_lo(w1, rs[mt][1].ds_lo, rs[mt][1].c_lo, kc);
                            const unsigned a2 = deq_lo(w0s, rs[mt][0].ds_lo, rs[mt][0].c_lo, kc), a3 = deq_lo(w1s, rs[mt][1].ds_lo, rs[mt][1].c_lo, kc);
#pragma unroll
                            for (int nt = 0; nt < NT; nt++)
                                if (!GROUPED || nt < nt_live) mma_f16(acc[mt][nt], a0, a1, a2, a3, hw ? bl[nt].z : bl[nt].x, hw ? bl[nt].w : bl[nt].y);
                        }
                        {   // high nibbles: sub-block 2p + 1
                            const unsigned a0 = deq_hi(w0, rs[mt][0].ds_hi, rs[mt][0].c_hi, kc), a1 = deq_hi(w1, rs[mt][1].ds_hi, rs[mt][1].c_hi, kc);
                            const unsigned a2 = deq_hi(w0s, rs[mt][0].ds_hi, rs[mt][0].c_hi, kc), a3 = deq_hi(w1s, rs[mt][1].ds_hi, rs[mt][1].c_hi, kc);
#pragma unroll
                            for (int nt = 0; nt < NT; nt++)
                                if (!GROUPED || nt < nt_live)
                                    mma_f16(kTwoAcc ? acc2[kTwoAcc ? mt : 0][kTwoAcc ? nt : 0] : acc[mt][nt], a0, a1, a2, a3, hw ? bh[nt].z : bh[nt].x,
                                            hw ? bh[nt].w : bh[nt].y);
                        }
                    }
                }
            }
        }
        done = i + 1;
        // the reads of both stages are ordered before the copy engine's writes of their refills
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(smem_u32(&aempty[as]));
            if (w_issued < n_it) {
                issue_w(w_issued, ws);   // the stage just read takes the stage `depth` further on
                w_issued++;
            }
            if (warp == 0 && a_issued < n_it) {
                // the stage just read is refilled once every warp has let go of it
                if (mbar_wait(smem_u32(&aempty[as]), aph, abort_v)) {
                    issue_a(a_issued, as);
                    a_issued++;
                } else {
                    abort_s = 1;
                }
            }
        }
        __syncwarp();
        if (++ws == Cfg::kWDepth) { ws = 0; wph ^= 1u; }
        if (++as == Cfg::kADepth) { as = 0; aph ^= 1u; }
    }
    if (*abort_v && lane == 0) {
        // copies this warp started and did not consume must land before the CTA may leave: bounded waits on their barriers
        for (int k = done; k < w_issued; k++)
            mbar_wait(smem_u32(&wfull[warp][(ws0 + k) % Cfg::kWDepth]), wph0 ^ (unsigned)(((ws0 + k) / Cfg::kWDepth) & 1));
    }
    __syncthreads();   // (also: every warp is done with both rings before the next pass refills them)
    if (abort_s) {
        if (tid == 0) {
            // activation stages nobody will read: the earliest unread one of any warp is not known here, so wait for all issued
            for (int k = max(0, a_issued - Cfg::kADepth); k < a_issued; k++)
                mbar_wait(smem_u32(&afull[(as0 + k) % Cfg::kADepth]), aph0 ^ (unsigned)(((as0 + k) / Cfg::kADepth) & 1));
            if (err_flag) atomicExch(err_flag, 1);
        }
        return;
    }
    float* o = out + (GROUPED ? (size_t)0 : (size_t)blockIdx.y * split_stride);
    if (kTwoAcc) {
#pragma unroll
        for (int mt = 0; mt < MA; mt++)
#pragma unroll
            for (int nt = 0; nt < NA; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[mt][nt][e] += acc2[mt][nt][e];
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const int r0 = row0 + 16 * mt + gid, r1 = r0 + 8;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int t0 = 8 * nt + 2 * p, t1 = t0 + 1;
            if (t0 < Tc) {
                if (r0 < N) o[(size_t)(rbase + t0) * ldo + r0] = acc[mt][nt][0];
                if (r1 < N) o[(size_t)(rbase + t0) * ldo + r1] = acc[mt][nt][2];
            }
            if (t1 < Tc) {
                if (r0 < N) o[(size_t)(rbase + t1) * ldo + r0] = acc[mt][nt][1];
                if (r1 < N) o[(size_t)(rbase + t1) * ldo + r1] = acc[mt][nt][3];
            }
        }
    }
    }   // pass
}

// [N][nSB][144] -> [ceil(N/16)][nSB][16][144]: one 16-byte piece per thread; rows past N become zero blocks (zero weights)
__global__ void q4k_to_tiles_kernel(const uint8_t* __restrict__ rm, int N, int nSB, uint8_t* __restrict__ tiles, size_t n_pieces) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pieces) return;
    const int piece = (int)(i % 9);
    const size_t blk = i / 9;                  // (tile, b, r) in the output's order
    const int r = (int)(blk % 16);
    const size_t tb = blk / 16;
    const int b = (int)(tb % nSB);
    const size_t tile = tb / nSB;
    const size_t row = tile * 16 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < (size_t)N) v = *reinterpret_cast<const uint4*>(rm + (row * nSB + b) * 144 + piece * 16);
    *reinterpret_cast<uint4*>(tiles + i * 16) = v;
}

// dst[t][n] = sum over the K ranges, in range order
__global__ void small_reduce_kernel(const float* __restrict__ part, size_t split_stride, int splits, int T, int N, float* __restrict__ dst, int ldd) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * N) return;
    const int t = (int)(i / N), n = (int)(i % N);
    float s = 0.f;
    for (int k = 0; k < splits; k++) s += part[(size_t)k * split_stride + i];
    dst[(size_t)t * ldd + n] = s;
}

template <int NT, int MT>
int run_small(b200_ctx* ctx, const uint8_t* W, int N, int nSB, const __half* x16, const float* scales, int T, float* out, int ldo, size_t stride, int splits,
              int sb_per_split) {
    using Cfg = SmallCfg<NT, MT>;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_small_kernel<NT, MT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
    }
    const int n_tiles = ceil_div(N, 16);
    dim3 grid(ceil_div(n_tiles, kSmWarps * MT), splits);
    {
        ProfScope ps(ctx, PROF_Q4K_GEMM);
        const int32_t* const no_offs = nullptr;
        launch_pdl(q4k_small_kernel<NT, MT, false>, grid, dim3(kSmThreads), (size_t)Cfg::kSmem, ctx->stream, W, n_tiles, x16, scales, N, nSB, sb_per_split, T, out, ldo,
                   stride, ctx->err_flag, no_offs);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

// The row count from which the fast class takes this kernel. Below it the dp4a lanes are faster (their work grows with the
// row count, this kernel's is that of eight rows at any count up to eight): measured on 151936 x 4096, 88 us (dp4a) against
// 99 us at two rows, 164 us against 99 us at three. B200_SMALL_MIN_ROWS overrides it for comparisons; 0 turns the kernel off.
int q4k_small_min_rows() {
    static const int v = [] {
        const char* e = getenv("B200_SMALL_MIN_ROWS");
        return e ? atoi(e) : 3;
    }();
    return v;
}

size_t q4k_tiles_bytes(int N, int K) { return (size_t)ceil_div(N, 16) * 16 * (K / 256) * 144; }

// row-major Q4_K [N][K/256][144] -> the tile-by-tile layout this file's kernel streams (q4k_tiles_bytes(N, K) bytes)
int launch_q4k_to_tiles(b200_ctx* ctx, const uint8_t* row_major, int N, int K, uint8_t* tiles) {
    if (K % 256 || ((reinterpret_cast<uintptr_t>(row_major) | reinterpret_cast<uintptr_t>(tiles)) & 15))
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "Q4_K re-layout wants K %% 256 == 0 and 16-byte aligned buffers");
    const size_t n_pieces = q4k_tiles_bytes(N, K) / 16;
    q4k_to_tiles_kernel<<<(unsigned)((n_pieces + 255) / 256), 256, 0, ctx->stream>>>(row_major, N, K / 256, tiles, n_pieces);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

// W: the matrix in the tile-by-tile layout (launch_q4k_to_tiles). Needs the context's tcgen05 scratch (the fp16 activation
// tiles and the K-range partials live there).
int launch_q4k_matmul_small(b200_ctx* ctx, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd) {
    ST_TRY(flush_pending_parts(ctx));  // the scratch is about to be reused
    if (K % 256 || T < 1 || T > 32) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the small-batch Q4_K matmul takes 1..32 rows and K %% 256 == 0");
    if (reinterpret_cast<uintptr_t>(W) & 15) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the small-batch Q4_K matmul wants 16-byte aligned weights");
    if (!ctx->umma_scratch) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the small-batch Q4_K matmul needs the fast class's scratch");
    const int nSB = K / 256;
    const int NT = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    // two m-tiles a warp (half the activation traffic) where the matrix is tall enough to cover the SMs that way
    const int MT = (NT == 4 && ceil_div(N, 256) >= ctx->sm_count) ? 2 : 1;
    const int tiles = ceil_div(ceil_div(N, 16), kSmWarps * MT);
    // K ranges. Two CTAs share an SM (their rings take 94 KB each), so the grid runs in waves of 2 * SMs CTAs and a wave
    // that is a third full costs a whole one (a 24576 x 4096 matrix in two ranges: 384 CTAs on 296 places, 1.3 waves).
    // Every count of ranges is priced as waves x (super-blocks per CTA + 2 for a CTA's fixed cost: ring fill, epilogue)
    // and the cheapest is taken; a count whose partials (written and read back: 8 bytes per range, row and column)
    // would pass a third of the weights' bytes is left out.
    const int kSbw = MT == 2 ? 1 : 2;   // SmallCfg<NT, MT>::kSbw
    const int places = 2 * ctx->sm_count;
    const double wbytes = (double)N * K * 0.5625;
    int splits = 1;
    double best = 1e30;
    if (NT == 4) {  // 17 to 32 rows (one CTA an SM): enough CTAs for two per SM, fewer while the partials' traffic would pass a third of the weights'
        splits = std::max(1, std::min(std::max(1, nSB / kSbw), ceil_div(2 * ctx->sm_count, tiles)));
        while (splits > 1 && 8.0 * splits * T * N > 0.33 * wbytes && tiles * (splits - 1) >= ctx->sm_count) splits--;
    }
    for (int sp = 1; NT < 4 && sp <= std::max(1, nSB / kSbw); sp++) {
        const int per = ceil_div(ceil_div(nSB, sp), kSbw) * kSbw, real = ceil_div(nSB, per);
        if (real != sp) continue;
        if (sp > 1 && 8.0 * sp * T * N > 0.33 * wbytes) break;
        const double cost = (double)ceil_div(tiles * sp, places) * (per + 2);
        if (cost < best - 1e-9) { best = cost; splits = sp; }
    }
    static const int splits_env = getenv("B200_SMALL_SPLITS") ? atoi(getenv("B200_SMALL_SPLITS")) : 0;   // for measurements
    if (splits_env > 0) splits = std::min(splits_env, nSB);
    int sb_per_split = ceil_div(ceil_div(nSB, splits), kSbw) * kSbw;   // whole stages
    splits = ceil_div(nSB, sb_per_split);
    const size_t x_bytes = (size_t)256 * K * 2;
    const bool slots = ctx->x16_slot_bytes > 0;
    const size_t part_off = slots ? 2 * ctx->x16_slot_bytes : ((x_bytes + 255) & ~(size_t)255);
    while (splits > 1 && part_off + (size_t)splits * T * N * 4 + 256 > ctx->umma_scratch_bytes) {
        sb_per_split = ceil_div(ceil_div(nSB, splits - 1), kSbw) * kSbw;
        splits = ceil_div(nSB, sb_per_split);
    }
    if ((slots && x_bytes > ctx->x16_slot_bytes) || part_off + (splits > 1 ? (size_t)splits * T * N * 4 : 0) + 256 > ctx->umma_scratch_bytes)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "small-batch Q4_K matmul: scratch too small");
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ctx->umma_scratch) + part_off);
    const __half* x16 = ctx->x16_ready;   // laid out by the kernel that quantized these activations (or by the caller)
    if (!x16) {
        __half* mine = slots ? x16_next_slot(ctx) : reinterpret_cast<__half*>(ctx->umma_scratch);
        ST_TRY(launch_act_to_f16(ctx, aq, T, K, mine));
        x16 = mine;
    }
    float* out = splits > 1 ? part : dst;
    const int ldo = splits > 1 ? N : ldd;
    const size_t stride = splits > 1 ? (size_t)T * N : 0;
    int st;
    if (NT == 1) st = run_small<1, 1>(ctx, W, N, nSB, x16, aq.scales, T, out, ldo, stride, splits, sb_per_split);
    else if (NT == 2) st = run_small<2, 1>(ctx, W, N, nSB, x16, aq.scales, T, out, ldo, stride, splits, sb_per_split);
    else if (MT == 1) st = run_small<4, 1>(ctx, W, N, nSB, x16, aq.scales, T, out, ldo, stride, splits, sb_per_split);
    else st = run_small<4, 2>(ctx, W, N, nSB, x16, aq.scales, T, out, ldo, stride, splits, sb_per_split);
    ST_TRY(st);
    if (splits > 1) {
        if (ctx->defer_reduce && ldd == N) {  // the consumer adds the partials (same order, same bits)
            ctx->pending = Parts{part, stride, splits, dst, T, N};
        } else {
            launch_pdl(small_reduce_kernel, dim3((unsigned)(((size_t)T * N + 255) / 256)), dim3(256), 0, ctx->stream, part, stride, splits, T, N, dst, ldd);
            LAUNCH_CHECK(ctx);
        }
    }
    return B200_OK;
}

// Routed experts' activations: sorted slot s takes token row rows_tok[s]: its fp16 tiles (code * scale, the layout the
// kernels above read) and its scales and group sums. One block per slot.
__global__ void gather_rows_x16_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales, const int32_t* __restrict__ rows_tok, int K,
                                       __half* __restrict__ x16, float* __restrict__ scales_out) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, r = rows_tok[s], nG = K >> 5;
    for (int c = threadIdx.x; c < (K >> 3); c += blockDim.x) {
        const int2 cw = *reinterpret_cast<const int2*>(codes + (size_t)r * K + 8 * c);
        const float sc = scales[(size_t)r * 2 * nG + (c >> 2)];
        const int8_t* cb = reinterpret_cast<const int8_t*>(&cw);
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = __fmul_rn((float)cb[u], sc);
        x16_store8(x16, K, s, 8 * c, v);
    }
    for (int i = threadIdx.x; i < 2 * nG; i += blockDim.x) scales_out[(size_t)s * 2 * nG + i] = scales[(size_t)r * 2 * nG + i];
}

int launch_gather_rows_x16(b200_ctx* ctx, ActQ src, const int32_t* rows_tok, int n_rows, int K, __half* x16, float* scales_out) {
    if (n_rows <= 0) return B200_OK;
    if (K % 32) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K %% 32");
    launch_pdl(gather_rows_x16_kernel, dim3(n_rows), dim3(128), 0, ctx->stream, (const int8_t*)src.codes, (const float*)src.scales, rows_tok, K, x16, scales_out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

// Routed experts. W_all: the experts' matrices one after the other, each tile by tile (launch_q4k_to_tiles over the stacked
// [n_experts * N][K] matrix gives exactly that when N is a multiple of 16). x16 / scales: the activation rows of the
// token-expert pairs in expert order (expert e owns rows offs[e] .. offs[e+1], a device array), the fp16 tiles padded so
// that rows up to n_rows + 16 can be read. dst rows are the same pairs.
bool q4k_small_grouped_supported(const uint8_t* W_all, int N, int K) { return N % 16 == 0 && K % 256 == 0 && (reinterpret_cast<uintptr_t>(W_all) & 15) == 0; }

int launch_q4k_matmul_small_grouped(b200_ctx* ctx, const uint8_t* W_all, int n_experts, int N, int K, const __half* x16, const float* scales,
                                    const int32_t* offs, int n_rows, float* dst, int ldd) {
    if (!q4k_small_grouped_supported(W_all, N, K)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "grouped small-batch matmul: N %% 16, K %% 256 or alignment");
    if (n_rows <= 0) return B200_OK;
    // passes of 16 rows (NT = 2): at 8 rows an expert on average, most experts take one. A warp takes two row tiles (MT = 2) where
    // the matrix has enough of them: an expert's share of a launch is small (a 1536 x 2048 gate|up stack is 1.8 MB), so fewer,
    // longer CTAs spend less of their time on set-up and on the first copies' latency.
    static const int mt_env = getenv("B200_EXPERT_MT") ? atoi(getenv("B200_EXPERT_MT")) : 0;
    const int n_tiles = N / 16, nSB = K / 256;
    const int MTsel = mt_env ? mt_env : (n_tiles >= 32 ? 2 : 1);
    ProfScope ps(ctx, PROF_Q4K_GEMM);
    if (MTsel == 2) {
        using Cfg = SmallCfg<2, 2>;
        static PerDeviceOnce attr_once;  // the attribute belongs to the device
        if (attr_once.first(ctx->device))
            CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_small_kernel<2, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        dim3 grid(ceil_div(n_tiles, kSmWarps * 2), 1, n_experts);
        launch_pdl(q4k_small_kernel<2, 2, true>, grid, dim3(kSmThreads), (size_t)Cfg::kSmem, ctx->stream, W_all, n_tiles, x16, scales, N, nSB, nSB, n_rows, dst, ldd,
                   (size_t)0, ctx->err_flag, offs);
    } else {
        using Cfg = SmallCfg<2, 1>;
        static PerDeviceOnce attr_once;
        if (attr_once.first(ctx->device))
            CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_small_kernel<2, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        dim3 grid(ceil_div(n_tiles, kSmWarps), 1, n_experts);
        launch_pdl(q4k_small_kernel<2, 1, true>, grid, dim3(kSmThreads), (size_t)Cfg::kSmem, ctx->stream, W_all, n_tiles, x16, scales, N, nSB, nSB, n_rows, dst, ldd,
                   (size_t)0, ctx->err_flag, offs);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

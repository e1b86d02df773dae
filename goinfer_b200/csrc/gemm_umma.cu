// gemm_umma.cu — fast-class Q4_K matmul for dense token counts: tcgen05 tensor cores with TMEM accumulators.
//
//   dst[t][n] = sum_k X[t][k] * W[n][k],   W Q4_K [N][K],  X = code * scale of the per-32 int8 activations
//
// Both operands are brought to fp16 in shared memory and multiplied by tcgen05.mma (kind::f16, fp32 accumulate in
// tensor memory). This is the non-bit-exact class the reference also has for large row counts (its int4 mma.sync GEMM,
// backend/cuda/gemm_w4a8_mma.cu:21-27, reported through Caps.HasFastPrefill): the integer group dots of the exact class
// are replaced by fp16 products of the dequantized values, each within 2^-11 of the exact operand.
//
// One CTA owns a [256 tokens] x [128*NT weight rows] output tile: per token tile an accumulator of 128*NT fp32 columns x
// 128 lanes (NT = 2: all of the SM's tensor memory; NT = 1 when that is what it takes to cover the SMs). K is walked in
// chunks of 64 (one sub-block pair of a super-block):
//   A ring: slots of one token tile ([128 tokens][64] fp16; a chunk takes two slots when the CTA has two token tiles,
//            else one): 6 slots, 3 in a launch of 128 rows or fewer. The fp16 activation matrix is written tile by tile
//            in the MMA's swizzled order by the kernels that quantize activations, so a slot is ONE contiguous 16 KB
//            bulk copy, issued by one thread.
//   raw weights: the 144-byte super-blocks of the tile's rows, per super-block one bulk copy of 2304 contiguous bytes
//            per 16 rows of the tile-major copy (or one tiled TMA copy, box 144 B x 128*NT rows, of the row-major matrix),
//            issued by one thread into a slot (two slots in a launch of 128 rows or fewer); each producer thread keeps
//            its row's current super-block in registers.
//   B ring: stages of [128*NT weight rows][64] fp16 (2; 3 in a launch of 128 rows or fewer), dequantized by eight
//            producer warps (a thread = a weight row; nibbles become fp16 by a mantissa trick, three instructions per
//            pair of weights).
// The producers arrive on a `full` mbarrier per chunk (the activation copy's bytes are counted on the same barrier); the
// MMA warp's elected thread waits for it, issues the chunk's 8 tcgen05.mma (M128, N = 128*NT, K = 16 each) and a
// tcgen05.commit that arrives on the `empty` mbarrier producers and loaders wait on before they reuse a stage. Nothing
// in the loop is a block-wide barrier. The epilogue reads the accumulators with tcgen05.ld (each warp its 32 TMEM lanes =
// 32 tokens), turns the 32x32 blocks around in shared memory and writes whole fp32 rows. With split-K (gridDim.z > 1)
// each split writes its own partial matrix; a second kernel adds the splits in order, unless the caller's next kernel
// does that itself (b200_ctx::defer_reduce).
//
// Every mbarrier wait is bounded: on expiry the CTA raises an error flag, frees its TMEM and returns.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "umma.cuh"
#include "kq_common.cuh"

namespace {

constexpr int kStages = 4;    // barrier slots: a chunk's full / empty barriers are slot it % kStages (four: a chunk's slot is its place in its super-block)
#ifndef B200_UMMA_A_SLOTS
#define B200_UMMA_A_SLOTS 6
#define B200_UMMA_B_STAGES 2
#define B200_UMMA_RAW_SLOTS 1
#endif
// The activation ring is counted in token tiles of 16 KB (a chunk with two token tiles takes two slots, with one tile one), the
// dequantized weight ring in stages of 128*NT rows, the raw super-blocks in slots of 128*NT x 144 bytes. Build parameters, for
// measurement: 5 slots + 3 weight stages, 5 + 2 with two raw slots and 6 + 2 + 1 all run a 256-row launch on 24576 x 4096 in
// 57-59 us and a 2048-row one in 358-374 us; 4 activation slots lose 6-10 % at 2048 rows.
constexpr int kASlotsQ4 = B200_UMMA_A_SLOTS, kBStagesQ4 = B200_UMMA_B_STAGES, kRawSlotsQ4 = B200_UMMA_RAW_SLOTS;
constexpr int kASlotsKQ = 6, kBStagesKQ = 2;
constexpr int kOneASlots = 3, kOneBStages = 3, kOneRawSlots = 2;   // launches of 128 rows or fewer (Q4_K)
static_assert(kBStagesQ4 <= kStages && kBStagesKQ <= kStages, "a ring cannot be deeper than the barrier slots");

// 8 weights of one 16-byte chunk (nibbles of words w0, w1) -> fp16, two at a time in half2 arithmetic. A nibble q is
// placed at mantissa bits [6,10) of the half 16.0 (0x4C00), which makes the half 16 + q with no int->float conversion, and
// w = (16 + q) * ds + c with c = -(16 ds + mn) is one half2 fma (c carries an extra rounding of about ds/128).
// Nibbles come out paired (0,2),(1,3) per word, so the tile's K order inside every group of four is 0,2,1,3; the activation
// matrix is written in the same order (a dot product does not care).
// (x & mask) | magic in one LOP3: with both constants in registers (as immediates the compiler spends two instructions a pair)
__device__ __forceinline__ unsigned and_or_u(unsigned x, unsigned mask, unsigned magic) {
    unsigned r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(x), "r"(mask), "r"(magic));
    return r;
}
__device__ __forceinline__ unsigned opaque_u(unsigned v) {
    unsigned r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
template <bool HIGH>
__device__ __forceinline__ uint4 dequant8(unsigned w0, unsigned w1, __half2 ds, __half2 c, unsigned mask, unsigned magic) {
    auto cv = [&](unsigned w, int byte1) -> unsigned {
        // nibble of bytes (0,2) or (1,3), low or high, moved to bits [6,10) and [22,26)
        const int from = (byte1 ? 8 : 0) + (HIGH ? 4 : 0);
        const unsigned sh = from <= 6 ? (w << (6 - from)) : (w >> (from - 6));
        unsigned t = and_or_u(sh, mask, magic);
        __half2 h = __hfma2(*reinterpret_cast<__half2*>(&t), ds, c);
        return *reinterpret_cast<unsigned*>(&h);
    };
    uint4 o;
    o.x = cv(w0, 0);
    o.y = cv(w0, 1);
    o.z = cv(w1, 0);
    o.w = cv(w1, 1);
    return o;
}

// scales and minima of sub-blocks 2p and 2p+1 from the header's 12 packed bytes, two at a time (the 6-bit fields of a pair sit
// in neighbouring bytes): {sc(2p), sc(2p+1)} and {m(2p), m(2p+1)} in the two low bytes. p is a literal at every call site.
__device__ __forceinline__ void pair_scale_min(const uint4 hdr, int p, unsigned* scs, unsigned* ms) {
    if (p < 2) {
        *scs = (hdr.y >> (16 * p)) & 0x3F3Fu;
        *ms = (hdr.z >> (16 * p)) & 0x3F3Fu;
    } else {
        const int sh = 16 * (p - 2);
        const unsigned lo = hdr.w >> sh;
        *scs = (lo & 0x0F0Fu) | (((hdr.y >> sh) >> 2) & 0x3030u);
        *ms = ((lo >> 4) & 0x0F0Fu) | (((hdr.z >> sh) >> 2) & 0x3030u);
    }
}

constexpr int kProducerWarps = 8;
constexpr int kProducers = kProducerWarps * 32;
constexpr int kUmmaThreads = kProducers + 96;  // 8 producer warps + the MMA-issuing, activation-loading and weight-loading warps
constexpr int kRawRow = 144;                   // one Q4_K super-block

// fast class: silu in f32 with the hardware exponential and reciprocal (about 1e-6 relative of the f64 value), the same
// expression as the stand-alone SwiGLU kernel's, so that the two give the same bits
__device__ __forceinline__ float umma_silu(float x) { return __fdividef(x, __fadd_rn(1.f, __expf(-x))); }

// NT: weight tiles of 128 rows per CTA: 2 when the grid still covers the SMs, else 1.
// SWIGLU (NT = 2, no K split): the weight rows are gate|up interleaved by 128 (tile t = gate rows 128t.. then up rows 128t..),
// so a thread of the epilogue holds, for its token, gate and up of the same 32 columns: it writes silu(gate) * up quantized
// per 32 (codes [T][F], scales and group sums [T][2*F/32]) and the f32 gate|up matrix never exists.
// FMT 4: Q4_K rows (144-byte super-blocks). FMT 6: Q6_K rows as the device keeps them, 208-byte bodies (ql[128], qh[64],
// sixteen int8 sub-scales) with the super-blocks' d values in `dvals` ([N][nSB] halves): w = d * sc * (q - 32), the six-bit
// q put together from a nibble and two upper bits; (q - 32) is exact in fp16 and takes the one rounding of the product with
// fp16(d * sc). FMT 5: Q5_K rows as in the file (176-byte super-blocks: d, dmin, the 12 scale bytes of Q4_K, qh[32], qs[128]):
// Q4_K's nibbles with a fifth bit from qh, the five-bit code placed in the mantissa of the half 32 + q.
// The rest of the kernel (activation ring, MMAs, epilogue) does not know the format.
// ONE (Q4_K, launches of 128 rows or fewer: every CTA has one token tile): the shared memory the second token tile's slots
// would take goes to a third weight stage and a second slot of raw super-blocks (3 activation slots + 3 + 2).
template <int NT, bool SWIGLU, int FMT = 4, bool ONE = false>
__global__ void __launch_bounds__(kUmmaThreads, 1) q4k_umma_gemm_kernel(const __grid_constant__ CUtensorMap wmap, int N, int nSB,
                                                                        const __half* __restrict__ X16, int T,
                                                                        float* __restrict__ dst, int ldd, size_t split_stride,
                                                                        int* __restrict__ err_flag, int8_t* __restrict__ sw_codes,
                                                                        float* __restrict__ sw_scales, __half* __restrict__ sw_x16,
                                                                        const uint8_t* __restrict__ w16, const unsigned short* __restrict__ dvals) {
    constexpr int RAW = FMT == 6 ? 208 : (FMT == 5 ? 176 : kRawRow);   // raw bytes of one super-block of a weight row
    pdl_trigger();  // the next kernel's blocks may be placed as ours retire; they wait for our completion before they touch data
    extern __shared__ __align__(1024) uint8_t umma_smem[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], raw_full[2], raw_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    constexpr int STAGE = 2 * kTileBytes;       // a chunk of the activation matrix in global memory: two token tiles
    static_assert(!ONE || FMT == 4, "the one-token-tile rings are the Q4_K kernel's");
    constexpr int kASlots = ONE ? kOneASlots : (FMT == 4 ? kASlotsQ4 : kASlotsKQ), kBStages = ONE ? kOneBStages : (FMT == 4 ? kBStagesQ4 : kBStagesKQ);
    constexpr int RAWST = ONE ? kOneRawSlots : (FMT == 4 ? kRawSlotsQ4 : 1), RAWSLOT = 128 * NT * RAW;   // slots of raw super-blocks (beside the one in registers)
    static_assert(RAWST <= 2, "two barriers for the raw slots");
    constexpr int BSTAGE = NT * kTileBytes;     // a B stage = NT weight tiles, contiguous: one K-major tile of 128*NT rows
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * 128 * NT, t0 = blockIdx.y * 256;
    // split-K ranges are whole super-blocks (4 chunks of 64)
    const int splits = gridDim.z, sb0 = (int)((long long)nSB * blockIdx.z / splits),
              sb1 = (int)((long long)nSB * (blockIdx.z + 1) / splits);
    const int n_sb = sb1 - sb0, n_it = 4 * n_sb;
    // token tiles of 128 this CTA really has: with 128 rows or fewer left, the second tile's copies, MMAs and epilogue are left out
    const int mt_count = (!ONE && T - t0 > 128) ? 2 : 1;
    // the swizzle atoms want 1024-byte aligned tiles; the launch reserves 1024 spare bytes for this round-up
    uint8_t* smem = umma_smem + ((1024u - (smem_u32(umma_smem) & 1023u)) & 1023u);
    uint8_t* bring = smem + (size_t)kASlots * kTileBytes;  // kBStages B stages of BSTAGE bytes
    uint8_t* raw = bring + kBStages * BSTAGE;                // the raw super-block (144 bytes) of each of the tile's 128*NT weight rows

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            // per chunk: the loader's arrival that announces the A bytes + 8 warp arrivals after the B stores
            mbar_init(smem_u32(&full_bar[s]), kProducerWarps + 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);  // one tcgen05.commit
        }
        for (int s = 0; s < RAWST; s++) {
            mbar_init(smem_u32(&raw_full[s]), 1);                 // the weight loader's announcement (+ the box's bytes)
            mbar_init(smem_u32(&raw_empty[s]), kProducerWarps);   // every producer warp has taken its rows out
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {  // TMEM: per token tile one accumulator of 128*NT fp32 columns x 128 lanes (NT = 2: all 512 columns)
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(256 * NT));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    volatile int* abort_v = &abort_s;
    pdl_wait();  // barriers and tensor memory were set up while the kernel before this one drained; its outputs are complete from here

    if (warp < kProducerWarps) {
        // ---- producers ----
        // B: NT = 2: thread = weight row tid, both sub-blocks of the chunk's pair. NT = 1: row tid & 127, sub-block
        // tid >> 7 of the pair. Each thread keeps its row's current super-block (144 raw bytes) in registers; the weight
        // loader fetches the tile's next super-blocks into `raw` meanwhile.
        const int wr = NT == 2 ? tid : tid & 127, hf1 = (tid >> 7) & 1;
        const unsigned b_off = (unsigned)wr * 128u, sw = (unsigned)(wr & 7);
        bool ok = true;
        if constexpr (FMT == 6) {
            uint4 q[13];      // the row's current super-block: ql (8 x 16 bytes), qh (4), sub-scales (1)
            float d = 0.f, d_next = 0.f;
            const bool row_in = n0 + wr < N;
            const unsigned short* dp = dvals + (size_t)min(n0 + wr, N - 1) * nSB + sb0;
            if (n_sb > 0 && row_in) d_next = __half2float(__ushort_as_half(dp[0]));
            const unsigned k_nib = opaque_u(0x00F000F0u), k_up = opaque_u(0x03000300u), k_magic = opaque_u(0x54005400u);   // registers: one LOP3 per use
            const __half2 k96 = __float2half2_rn(96.f);
            auto step6 = [&](int it, int p) -> bool {  // p = it & 3, a literal at every call site
                if (it >= kBStages) {
                    const bool w_ok = mbar_wait(smem_u32(&empty_bar[(it - kBStages) % kStages]), (unsigned)(((it - kBStages) / kStages) & 1), abort_v);
                    if (!__all_sync(0xffffffffu, w_ok)) return false;
                }
                if (p == 0) {
                    const int sb = it >> 2;
                    const bool w_ok = mbar_wait(smem_u32(&raw_full[0]), (unsigned)(sb & 1), abort_v);
                    if (!__all_sync(0xffffffffu, w_ok)) return false;
                    const uint4* rp = reinterpret_cast<const uint4*>(raw + (size_t)wr * RAW);
#pragma unroll
                    for (int i = 0; i < 13; i++) q[i] = rp[i];
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&raw_empty[0]));
                    d = d_next;
                    if (sb + 1 < n_sb && row_in) d_next = __half2float(__ushort_as_half(dp[sb + 1]));
                }
                {
                    // chunk p = elements 64 p .. 64 p + 63 of the block: half p >> 1 of the block; its first 32 elements take the
                    // low (p even) or high (p odd) nibbles of ql[64 half + l] and bit pair (p & 1) * 2 of qh[32 half + l], the
                    // other 32 those of ql[64 half + 32 + l] and the next bit pair; sub-scales 8 half + 4 (p & 1) + {0,1 | 2,3}
                    const int half = p >> 1, odd = p & 1;
                    uint8_t* rowp = bring + (size_t)(it % kBStages) * BSTAGE + b_off;
                    const unsigned scw = (&q[12].x)[2 * half + odd];
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        if (NT == 1 && hf != hf1) continue;
                        const uint4 la = q[4 * half + 2 * hf], lb = q[4 * half + 2 * hf + 1];   // ql of l = 0..15, 16..31
                        const uint4 ua = q[8 + 2 * half], ub = q[8 + 2 * half + 1];               // qh of the same l
                        const unsigned lw[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
                        const unsigned uw[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
                        const int ush = 4 * odd + 2 * hf;   // the bit pair's place in a qh byte
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {     // 8 elements a piece: l = 8 ch .. 8 ch + 7, sub-scale l / 16
                            const int sc = (int)(signed char)((scw >> (8 * (2 * hf + (ch >> 1)))) & 0xffu);
                            const __half2 ds = __half2half2(__float2half_rn(d * (float)sc));
                            uint4 o;
                            unsigned* ov = &o.x;
#pragma unroll
                            for (int wi = 0; wi < 2; wi++) {
                                const unsigned w = lw[2 * ch + wi], u = uw[2 * ch + wi];
#pragma unroll
                                for (int b1 = 0; b1 < 2; b1++) {   // bytes (0,2) then (1,3) of the word: the tile's order inside every four
                                    // nibble to bits [4,8) of each half, the two upper bits to [8,10): the half 64 + q
                                    const int nfrom = 8 * b1 + 4 * odd;      // where the nibble starts in the 16-bit lane
                                    const unsigned nsh = nfrom <= 4 ? (w << (4 - nfrom)) : (w >> (nfrom - 4));
                                    const int ufrom = 8 * b1 + ush;
                                    const unsigned us = ufrom <= 8 ? (u << (8 - ufrom)) : (u >> (ufrom - 8));
                                    unsigned t = and_or_u(nsh, k_nib, k_magic);
                                    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(us), "r"(k_up), "r"(t));   // (us & k_up) | t
                                    const __half2 hq = __hsub2(*reinterpret_cast<__half2*>(&t), k96);   // q - 32, exact
                                    const __half2 hv = __hmul2(hq, ds);
                                    ov[2 * wi + b1] = *reinterpret_cast<const unsigned*>(&hv);
                                }
                            }
                            *reinterpret_cast<uint4*>(rowp + (((unsigned)(4 * hf + ch) ^ sw) << 4)) = o;
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&full_bar[it % kStages]));
                return true;
            };
            for (int it = 0; it < n_it && ok; it += 4) {
                ok = step6(it, 0);
                if (ok) ok = step6(it + 1, 1);
                if (ok) ok = step6(it + 2, 2);
                if (ok) ok = step6(it + 3, 3);
            }
        } else if constexpr (FMT == 5) {
            uint4 hdr, uq[2], q[8];   // the row's current super-block: d, dmin, scale bytes; the fifth bits; the nibbles
            const unsigned k_nib = opaque_u(0x01E001E0u), k_bit = opaque_u(0x02000200u), k_magic = opaque_u(0x50005000u);
            auto step5 = [&](int it, int p) -> bool {  // p = it & 3, a literal at every call site
                if (it >= kBStages) {
                    const bool w_ok = mbar_wait(smem_u32(&empty_bar[(it - kBStages) % kStages]), (unsigned)(((it - kBStages) / kStages) & 1), abort_v);
                    if (!__all_sync(0xffffffffu, w_ok)) return false;
                }
                if (p == 0) {
                    const int sb = it >> 2;
                    const bool w_ok = mbar_wait(smem_u32(&raw_full[0]), (unsigned)(sb & 1), abort_v);
                    if (!__all_sync(0xffffffffu, w_ok)) return false;
                    const uint4* rp = reinterpret_cast<const uint4*>(raw + (size_t)wr * RAW);
                    hdr = rp[0];
                    uq[0] = rp[1]; uq[1] = rp[2];
#pragma unroll
                    for (int i = 0; i < 8; i++) q[i] = rp[3 + i];
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&raw_empty[0]));
                }
                {   // sub-blocks 2p (low nibbles of code bytes 32p.., bit 2p of qh[l]) and 2p+1 (high nibbles, bit 2p+1)
                    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
                    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                    uint8_t* rowp = bring + (size_t)(it % kBStages) * BSTAGE + b_off;
                    const uint4 qa = q[2 * p], qb = q[2 * p + 1];
                    const unsigned wq[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    const unsigned uw[8] = {uq[0].x, uq[0].y, uq[0].z, uq[0].w, uq[1].x, uq[1].y, uq[1].z, uq[1].w};
                    unsigned scs, ms;
                    pair_scale_min(hdr, p, &scs, &ms);
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        if (NT == 1 && hf != hf1) continue;
                        const int sc = (int)((scs >> (8 * hf)) & 0xffu), mn = (int)((ms >> (8 * hf)) & 0xffu);
                        const __half dsh = __float2half_rn(d * (float)sc);
                        const __half2 ds = __half2half2(dsh), c = __float2half2_rn(-(32.f * __half2float(dsh) + dmin * (float)mn));
                        const int bit = 2 * p + hf;
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            uint4 o;
                            unsigned* ov = &o.x;
#pragma unroll
                            for (int wi = 0; wi < 2; wi++) {
                                const unsigned w = wq[2 * ch + wi], u = uw[2 * ch + wi];
#pragma unroll
                                for (int b1 = 0; b1 < 2; b1++) {   // bytes (0,2) then (1,3): the tile's order inside every four
                                    const int nfrom = 8 * b1 + 4 * hf;   // the nibble's first bit in the 16-bit lane; it goes to bit 5
                                    const unsigned nsh = nfrom <= 5 ? (w << (5 - nfrom)) : (w >> (nfrom - 5));
                                    const int ufrom = 8 * b1 + bit;      // the fifth bit's place; it goes to bit 9
                                    const unsigned us = ufrom <= 9 ? (u << (9 - ufrom)) : (u >> (ufrom - 9));
                                    unsigned t = and_or_u(nsh, k_nib, k_magic);
                                    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(us), "r"(k_bit), "r"(t));   // (us & k_bit) | t
                                    const __half2 hv = __hfma2(*reinterpret_cast<__half2*>(&t), ds, c);
                                    ov[2 * wi + b1] = *reinterpret_cast<const unsigned*>(&hv);
                                }
                            }
                            *reinterpret_cast<uint4*>(rowp + (((unsigned)(4 * hf + ch) ^ sw) << 4)) = o;
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&full_bar[it % kStages]));
                return true;
            };
            for (int it = 0; it < n_it && ok; it += 4) {
                ok = step5(it, 0);
                if (ok) ok = step5(it + 1, 1);
                if (ok) ok = step5(it + 2, 2);
                if (ok) ok = step5(it + 3, 3);
            }
        } else {
        uint4 hdr, q[8];  // the current super-block: d, dmin, 12 scale bytes; 128 code bytes
        const unsigned k_mask = opaque_u(0x03C003C0u), k_magic = opaque_u(0x4C004C00u);   // registers, so that mask-and-or is one LOP3
        static_assert(kStages == 4, "a chunk's barrier slot is its place p in its super-block");
        // where this thread's eight 16-byte pieces of a row go inside a B stage (the 128-byte swizzle), computed once
        uint8_t* piece[8];
#pragma unroll
        for (int c8 = 0; c8 < 8; c8++) piece[c8] = bring + b_off + (((unsigned)c8 ^ sw) << 4);

        auto step = [&](int sb, int p) -> bool {  // chunk it = 4 * sb + p; p is a literal at every call site, so slots and stages are too
            const int it = 4 * sb + p;
            // the B stage was last read by the MMAs of chunk it - kBStages
            if (it >= kBStages) {  // the answer is made warp-uniform: the lanes meet in __syncwarp below
                const int back = p - kBStages;   // negative: a chunk of the super-block before
                const bool w_ok = mbar_wait(smem_u32(&empty_bar[back & 3]), (unsigned)((sb + (back >> 2)) & 1), abort_v);
                if (!__all_sync(0xffffffffu, w_ok)) return false;
            }
            if (p == 0) {  // take the row's next super-block out of its raw slot, then hand the slot back to the weight loader
                const int slot = sb % RAWST;
                const bool w_ok = mbar_wait(smem_u32(&raw_full[slot]), (unsigned)((sb / RAWST) & 1), abort_v);
                if (!__all_sync(0xffffffffu, w_ok)) return false;
                const uint4* rp = reinterpret_cast<const uint4*>(raw + (size_t)slot * RAWSLOT + (size_t)wr * RAW);
                hdr = rp[0];
#pragma unroll
                for (int i = 0; i < 8; i++) q[i] = rp[1 + i];
                // these reads are ordered before the copy engine's writes of the refill
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&raw_empty[slot]));
            }
            {   // dequantize the chunk's sub-blocks 2p (low nibbles of code bytes 32p..32p+31) and 2p+1 (high nibbles)
                const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
                const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                const int stage_off = (kBStages == 2 ? (p & 1) : it % kBStages) * BSTAGE;
                const uint4 qa = q[2 * p], qb = q[2 * p + 1];
                const unsigned wq[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                unsigned scs, ms;
                pair_scale_min(hdr, p, &scs, &ms);
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    if (NT == 1 && hf != hf1) continue;
                    const int sc = (int)((scs >> (8 * hf)) & 0xffu), mn = (int)((ms >> (8 * hf)) & 0xffu);
                    const __half dsh = __float2half_rn(d * (float)sc);
                    // the offset uses the rounded scale, so that the 16 * scale part cancels exactly
                    const __half2 ds = __half2half2(dsh), c = __float2half2_rn(-(16.f * __half2float(dsh) + dmin * (float)mn));
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        const uint4 v = hf ? dequant8<true>(wq[2 * ch], wq[2 * ch + 1], ds, c, k_mask, k_magic)
                                           : dequant8<false>(wq[2 * ch], wq[2 * ch + 1], ds, c, k_mask, k_magic);
                        *reinterpret_cast<uint4*>(piece[4 * hf + ch] + stage_off) = v;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy stores -> visible to the tensor core
            __syncwarp();  // every lane's stores are fenced: one arrival stands for the warp
            if (lane == 0) mbar_arrive(smem_u32(&full_bar[p]));
            return true;
        };
        for (int sb = 0; sb < n_sb && ok; sb++) {
            ok = step(sb, 0);
            if (ok) ok = step(sb, 1);
            if (ok) ok = step(sb, 2);
            if (ok) ok = step(sb, 3);
        }
        }
        if (!ok) abort_s = 1;
    } else if (warp == kProducerWarps && lane == 0) {
        // ---- the MMA issuer: one thread; waits for a full stage, issues its 8 MMAs, commits to empty[it % 4] ----
        for (int it = 0; it < n_it; it++) {
            if (!mbar_wait(smem_u32(&full_bar[it % kStages]), (unsigned)((it / kStages) & 1), abort_v)) {
                abort_s = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned b0 = smem_u32(bring + (size_t)(it % kBStages) * BSTAGE);
            // one instruction spans all 128*NT weight rows (N = 128*NT): the token tile is fetched once for them
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                if (mt >= mt_count) break;
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    umma_f16(tmem_base + mt * 128 * NT, umma_desc(smem_u32(smem + (size_t)((mt_count * it + mt) % kASlots) * kTileBytes) + ks * 32), umma_desc(b0 + ks * 32),
                             idesc_for(128 * NT), (it > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&empty_bar[it % kStages]));
        }
        // all MMAs done: the last commit covers every earlier one. Only this thread waits for it; everyone else
        // parks in the block barrier below.
        if (n_it > 0 && !*abort_v) {
            const int last = n_it - 1;
            if (!mbar_wait(smem_u32(&empty_bar[last % kStages]), (unsigned)((last / kStages) & 1), abort_v)) abort_s = 1;
        }
    } else if (warp == kProducerWarps + 1 && lane == 0) {
        // ---- the activation loader: one thread, one 32 KB bulk copy per chunk. The fp16 activation matrix is stored
        // tile by tile ([token tile][chunk of K][256 rows][64]) in the swizzled order of the MMA tiles. ----
        const uint8_t* src = reinterpret_cast<const uint8_t*>(X16) + ((size_t)blockIdx.y * (size_t)(4 * nSB) + (size_t)(4 * sb0)) * STAGE;
        int issued = 0;
        for (int it = 0; it < n_it && !abort_s; it++) {
            const unsigned bar = smem_u32(&full_bar[it % kStages]);
            for (int mt = 0; mt < mt_count; mt++) {
                // the slot's last tenant was token tile flat - kASlots, a tile of chunk (flat - kASlots) / mt_count; and the chunk's
                // `full` barrier must have finished the phase of chunk it - kStages before anything of this chunk arrives on it
                const int flat = mt_count * it + mt, prev = max(flat >= kASlots ? (flat - kASlots) / mt_count : -1, it - kStages);
                if (prev >= 0 && !mbar_wait(smem_u32(&empty_bar[prev % kStages]), (unsigned)((prev / kStages) & 1), abort_v)) {
                    abort_s = 1;
                    break;
                }
                if (mt == 0) mbar_arrive_expect_tx(bar, (unsigned)(mt_count * kTileBytes));   // rows 0..127 of a 256-row tile are its first half
                bulk_g2s(smem_u32(smem + (size_t)(flat % kASlots) * kTileBytes), src + (size_t)it * STAGE + (size_t)mt * kTileBytes, kTileBytes, bar);
            }
            issued = it + 1;
        }
        if (abort_s) {  // copies still in flight must land before the CTA may leave: bounded waits on their barriers
            for (int it = max(0, issued - 4); it < issued; it++) mbar_wait(smem_u32(&full_bar[it % kStages]), (unsigned)((it / kStages) & 1));
        }
    } else if (warp == kProducerWarps + 2 && lane == 0) {
        // ---- the weight loader: one thread. From the row-major matrix, one tiled copy per super-block: 144 raw bytes of
        // each of the tile's rows (rows past N read as zeros, which dequantize to zero weights). From the tile-major copy
        // (w16: [16-row tile][super-block][16][144], padded with zero blocks to whole tiles), 2304 contiguous bytes per
        // 16 rows; 16-row tiles past the matrix are not fetched, and their columns of the product are never stored. ----
        int issued = 0;
        const int tile0 = n0 / 16, live = min(8 * NT, (N + 15) / 16 - tile0);
        for (int sb = 0; sb < n_sb; sb++) {
            const int slot = sb % RAWST;
            if (sb >= RAWST && !mbar_wait(smem_u32(&raw_empty[slot]), (unsigned)((sb / RAWST - 1) & 1), abort_v)) {
                abort_s = 1;
                break;
            }
            uint8_t* rslot = raw + (size_t)slot * RAWSLOT;
            if (w16) {
                mbar_arrive_expect_tx(smem_u32(&raw_full[slot]), (unsigned)(live * 16 * kRawRow));
                for (int i = 0; i < live; i++)
                    bulk_g2s(smem_u32(rslot + (size_t)i * 16 * kRawRow), w16 + ((size_t)(tile0 + i) * nSB + sb0 + sb) * (16 * kRawRow), 16 * kRawRow,
                             smem_u32(&raw_full[slot]));
            } else {
                mbar_arrive_expect_tx(smem_u32(&raw_full[slot]), (unsigned)RAWSLOT);
                tensor_g2s_2d(smem_u32(rslot), &wmap, (sb0 + sb) * RAW, n0, smem_u32(&raw_full[slot]));
            }
            issued = sb + 1;
        }
        // copies still in flight must land before the CTA may leave: bounded waits on their barriers
        if (abort_s)
            for (int sb = max(0, issued - RAWST); sb < issued; sb++) mbar_wait(smem_u32(&raw_full[sb % RAWST]), (unsigned)((sb / RAWST) & 1));
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (abort_s) {
        if (tid == 0 && err_flag) atomicExch(err_flag, 1);
    } else if (n_it > 0 && warp < kProducerWarps && (warp >> 2) < mt_count) {
        // warp w reads TMEM lanes 32*(w%4).. of token tile mt = w/4, all 128*NT columns:
        // tokens t0 + 128*mt + 32*(w%4) + lane, output columns n0 + column
        float* out = dst + (size_t)blockIdx.z * split_stride;
        const int mt = warp >> 2, lq = warp & 3;
        const int tbase = t0 + mt * 128 + lq * 32;
        uint8_t* tp = smem + warp * (32 * 144);
        if constexpr (SWIGLU) {
            const int F = N >> 1, nG = F >> 5, tt = tbase + lane;
#pragma unroll 1
            for (int cb = 0; cb < 4; cb++) {
                unsigned rg[32], ru[32];
                const unsigned ta = tmem_base + ((unsigned)(lq * 32) << 16) + (unsigned)(mt * 256 + cb * 32);
#define UMMA_LD32(R, ADDR)                                                                                                          \
    asm volatile(                                                                                                                    \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                                    \
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n" \
        : "=r"(R[0]), "=r"(R[1]), "=r"(R[2]), "=r"(R[3]), "=r"(R[4]), "=r"(R[5]), "=r"(R[6]), "=r"(R[7]), "=r"(R[8]), "=r"(R[9]),      \
          "=r"(R[10]), "=r"(R[11]), "=r"(R[12]), "=r"(R[13]), "=r"(R[14]), "=r"(R[15]), "=r"(R[16]), "=r"(R[17]), "=r"(R[18]),       \
          "=r"(R[19]), "=r"(R[20]), "=r"(R[21]), "=r"(R[22]), "=r"(R[23]), "=r"(R[24]), "=r"(R[25]), "=r"(R[26]), "=r"(R[27]),       \
          "=r"(R[28]), "=r"(R[29]), "=r"(R[30]), "=r"(R[31])                                                                         \
        : "r"(ADDR))
                UMMA_LD32(rg, ta);
                UMMA_LD32(ru, ta + 128u);
#undef UMMA_LD32
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                const int f0 = blockIdx.x * 128 + cb * 32;  // the group's first column of the [T][F] product
                float y[32], ma = 0.f;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    y[i] = __fmul_rn(umma_silu(__uint_as_float(rg[i])), __uint_as_float(ru[i]));
                    ma = fmaxf(ma, fabsf(y[i]));
                }
                // the per-32 quantizer of the step (sc = max/127, round to nearest even, clamp, group sum)
                const float sc = __fdiv_rn(ma, 127.f);
                const float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
                int sum = 0;
                unsigned w[8];
#pragma unroll
                for (int i = 0; i < 8; i++) w[i] = 0u;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    int q = __float2int_rn(__fmul_rn(y[i], inv));
                    q = max(-127, min(127, q));
                    sum += q;
                    w[i >> 2] |= (unsigned)(q & 0xff) << (8 * (i & 3));
                }
                if (tt < T && f0 < F) {
                    uint4* o = reinterpret_cast<uint4*>(sw_codes + (size_t)tt * F + f0);
                    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    o[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    sw_scales[(size_t)tt * 2 * nG + (f0 >> 5)] = sc;
                    sw_scales[(size_t)tt * 2 * nG + nG + (f0 >> 5)] = __fmul_rn(sc, (float)sum);
                    if (sw_x16) {  // the next matmul's fp16 activation tiles, laid out here instead of by a conversion kernel
#pragma unroll
                        for (int c8 = 0; c8 < 4; c8++) {
                            float dq[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const int q = (int)(signed char)((w[(8 * c8 + i) >> 2] >> (8 * (i & 3))) & 0xffu);
                                dq[i] = __fmul_rn((float)q, sc);
                            }
                            x16_store8(sw_x16, F, tt, f0 + 8 * c8, dq);
                        }
                    }
                }
            }
        } else {
#pragma unroll 1
        for (int cb = 0; cb < 4 * NT; cb++) {
            unsigned r[32];
            const unsigned taddr = tmem_base + ((unsigned)(lq * 32) << 16) + (unsigned)(mt * 128 * NT + cb * 32);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                  "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            // lane = token, registers = columns: turn the 32 x 32 block around in shared memory (the rings are idle now;
            // rows 144 bytes apart keep both directions conflict-free) so that a store instruction writes whole rows
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; i++)
                *reinterpret_cast<uint4*>(tp + lane * 144 + i * 16) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            __syncwarp();
            const int nc = n0 + cb * 32 + (lane & 7) * 4;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int row = j * 4 + (lane >> 3), tt = tbase + row;
                const uint4 v = *reinterpret_cast<const uint4*>(tp + row * 144 + (lane & 7) * 16);
                if (tt < T && nc < N) {
                    float* o = out + (size_t)tt * ldd + nc;
                    if (nc + 4 <= N && (ldd & 3) == 0) *reinterpret_cast<uint4*>(o) = v;
                    else {
                        const unsigned e[4] = {v.x, v.y, v.z, v.w};
                        for (int i = 0; i < 4; i++)
                            if (nc + i < N) o[i] = __uint_as_float(e[i]);
                    }
                }
            }
        }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256 * NT));
}

// X16[t][k'] = fp16(code * scale of its group). Two reorderings of K that the weight tiles share: inside every group of
// four, positions 1 and 2 are swapped (the order the nibble pairs come out of a code word); and the matrix is stored as
// the MMA's shared-memory tiles, [token tile of 256][chunk of 64 along K][256 rows][64], the 16-byte chunk c of a row at
// position c ^ (t & 7) (the 128-byte swizzle), so that one contiguous 32 KB copy brings a stage in ready for the tensor
// core. Rows past T in the last token tile are never written: they feed accumulator rows that are never stored.
__global__ void act_to_f16_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales, int K,
                                  __half* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, nG = K >> 5;
    const int k8 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (k8 >= K) return;
    const int2 c = *reinterpret_cast<const int2*>(codes + (size_t)t * K + k8);
    const float s = scales[(size_t)t * 2 * nG + (k8 >> 5)];
    const int8_t* cb = reinterpret_cast<const int8_t*>(&c);
    uint4 o;
    __half2 h;
    h = __floats2half2_rn(__fmul_rn((float)cb[0], s), __fmul_rn((float)cb[2], s)); o.x = *reinterpret_cast<unsigned*>(&h);
    h = __floats2half2_rn(__fmul_rn((float)cb[1], s), __fmul_rn((float)cb[3], s)); o.y = *reinterpret_cast<unsigned*>(&h);
    h = __floats2half2_rn(__fmul_rn((float)cb[4], s), __fmul_rn((float)cb[6], s)); o.z = *reinterpret_cast<unsigned*>(&h);
    h = __floats2half2_rn(__fmul_rn((float)cb[5], s), __fmul_rn((float)cb[7], s)); o.w = *reinterpret_cast<unsigned*>(&h);
    const int seg = k8 >> 6, chunk = (k8 >> 3) & 7;
    const size_t tile = ((size_t)(t >> 8) * (size_t)(K >> 6) + seg) * (256 * 64);
    *reinterpret_cast<uint4*>(out + tile + (size_t)(t & 255) * 64 + ((chunk ^ (t & 7)) << 3)) = o;
}

// dst[t][n] = sum over splits, in split order
__global__ void splitk_reduce_kernel(const float* __restrict__ part, size_t split_stride, int splits, int T, int N,
                                     float* __restrict__ dst, int ldd) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * N) return;
    const int t = (int)(i / N), n = (int)(i % N);
    float s = 0.f;
    for (int k = 0; k < splits; k++) s += part[(size_t)k * split_stride + (size_t)t * N + n];
    dst[(size_t)t * ldd + n] = s;
}

}  // namespace

// The tensor map of a weight matrix seen as bytes, [N rows][nSB * 144], with a box of one super-block x box_rows rows. A map
// depends only on its key, so the cache never goes stale. cuTensorMapEncodeTiled is reached through the runtime's
// driver-entry-point lookup.
const CUtensorMap* q4k_weight_map(b200_ctx* ctx, const uint8_t* W, int N, int nSB, int box_rows, int sb_bytes) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap*> cache;
    std::lock_guard<std::mutex> lock(mu);
    const tensor_map_encode_fn encode = tensor_map_encoder();
    if (!encode) {
        ctx->err = "cuTensorMapEncodeTiled is not available from this driver";
        return nullptr;
    }
    const auto key = std::make_tuple((const void*)W, N, nSB, box_rows, sb_bytes);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    CUtensorMap* m = new CUtensorMap;
    const cuuint64_t dims[2] = {(cuuint64_t)nSB * sb_bytes, (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)nSB * sb_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)sb_bytes, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(W), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        delete m;
        ctx->err = "cuTensorMapEncodeTiled failed with " + std::to_string((int)r) + " (N=" + std::to_string(N) + ", super-blocks=" + std::to_string(nSB) + ")";
        return nullptr;
    }
    cache[key] = m;
    return m;
}

// fp16(code * scale) of the quantized activation rows, in the tile layout the fast-class matmuls read
int launch_act_to_f16(b200_ctx* ctx, ActQ aq, int T, int K, __half* out) {
    dim3 grid(ceil_div(K / 8, 256), T);
    launch_pdl(act_to_f16_kernel, grid, dim3(256), 0, ctx->stream, aq.codes, aq.scales, K, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

size_t q4k_umma_scratch_bytes(int max_rows, int max_k, int max_n) {
    // fp16 activations + split-K partials (up to 4 splits)
    return (size_t)ceil_div(max_rows, 256) * 256 * max_k * 2 + (size_t)4 * max_rows * max_n * 4 + 256;
}

int flush_pending_parts(b200_ctx* ctx) {
    if (ctx->pending.n <= 0) return B200_OK;
    const Parts pt = ctx->pending;
    ctx->pending = Parts{};
    splitk_reduce_kernel<<<(unsigned)(((size_t)pt.rows * pt.cols + 255) / 256), 256, 0, ctx->stream>>>(pt.p, pt.stride, pt.n, pt.rows, pt.cols,
                                                                                                      const_cast<float*>(pt.dst), pt.cols);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_q4k_matmul_umma(b200_ctx* ctx, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, void* scratch,
                           size_t scratch_bytes, int* err_flag, const uint8_t* W_tiles) {
    return launch_q4k_matmul_umma_swiglu(ctx, W, N, K, aq, T, dst, ldd, scratch, scratch_bytes, err_flag, ActQ{}, false, nullptr, nullptr, W_tiles);
}

// With `sw` set and W = gate|up interleaved by 128 rows ([2F][K]): when the launch has two weight tiles per CTA and no K
// split (or `force`), the epilogue writes silu(gate) * up quantized per 32 into `sw` and *fused = true; otherwise the
// f32 product goes to dst as usual (its columns in the interleaved order) and *fused = false.
__half* x16_next_slot(b200_ctx* ctx) {
    if (!ctx->x16_slot_bytes || !ctx->umma_scratch) return nullptr;
    ctx->x16_toggle ^= 1;
    return reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(ctx->umma_scratch) + (size_t)ctx->x16_toggle * ctx->x16_slot_bytes);
}

int launch_q4k_matmul_umma_swiglu(b200_ctx* ctx, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, void* scratch,
                                  size_t scratch_bytes, int* err_flag, ActQ sw, bool force, bool* fused, __half* sw_x16, const uint8_t* W_tiles) {
    if (fused) *fused = false;
    static const bool no_tiles_env = getenv("B200_UMMA_ROW_MAJOR") != nullptr;  // measurement: keep the tiled copies of the row-major matrix
    if (no_tiles_env && W) W_tiles = nullptr;
    if (!W && !W_tiles) B200_FAIL(ctx, B200_BAD_ARGUMENT, "no weights");
    ST_TRY(flush_pending_parts(ctx));  // the scratch is about to be reused
    if (K % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "Q4_K needs K %% 256 == 0");
    if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(W_tiles)) & 15) B200_FAIL(ctx, B200_BAD_ARGUMENT, "tcgen05 matmul wants 16-byte aligned weights");
    const int nSB = K / 256, t_tiles = ceil_div(T, 256);
    // two weight tiles per CTA halve the activation traffic; one per CTA when that is what it takes to cover the SMs
    const int max_splits = std::max(1, std::min(4, nSB / 2));
    int NT = ceil_div(N, 256) * t_tiles * max_splits >= ctx->sm_count * 3 / 4 ? 2 : 1;
    if (sw.codes && force) NT = 2;
    const int n_tiles = ceil_div(N, 128 * NT);
    int splits = std::max(1, std::min(max_splits, ctx->sm_count / std::max(1, n_tiles * t_tiles)));
    if (sw.codes && force) splits = 1;
    const bool fuse = sw.codes && NT == 2 && splits == 1 && N % 256 == 0 && (N / 2) % 32 == 0 && !(reinterpret_cast<uintptr_t>(sw.codes) & 15);
    if (sw.codes && !fuse && !dst) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the fused SwiGLU epilogue does not apply to this shape and no f32 output was given");
    const size_t x_bytes = (size_t)t_tiles * 256 * K * 2;
    const size_t part_bytes = splits > 1 ? (size_t)splits * T * N * 4 : 0;
    // the scratch: with activation slots, two of them and then the partials; else the activations and then the partials
    const bool slots = ctx->x16_slot_bytes > 0 && scratch == ctx->umma_scratch;
    const size_t part_off = slots ? 2 * ctx->x16_slot_bytes : ((x_bytes + 255) & ~(size_t)255);
    if ((slots && x_bytes > ctx->x16_slot_bytes) || part_off + part_bytes + 256 > scratch_bytes)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "tcgen05 matmul scratch too small");
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + part_off);
    const __half* x16 = slots ? ctx->x16_ready : nullptr;  // laid out by the kernel that quantized these activations
    if (!x16) {
        __half* mine = slots ? x16_next_slot(ctx) : reinterpret_cast<__half*>(scratch);
        ST_TRY(launch_act_to_f16(ctx, aq, T, K, mine));
        x16 = mine;
    }
    if (sw_x16 && sw_x16 == x16) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the epilogue's activation slot is the one this matmul reads");
    // A ring + B ring (sized for NT = 2) + one raw super-block per producer thread + round-up room
    constexpr int smem = kASlotsQ4 * kTileBytes + kBStagesQ4 * 2 * kTileBytes + kRawSlotsQ4 * kProducers * kRawRow + 1024;
    static_assert(smem <= 227 * 1024, "a CTA's shared memory");
    constexpr int smem_one = kOneASlots * kTileBytes + kOneBStages * 2 * kTileBytes + kOneRawSlots * kProducers * kRawRow + 1024;
    static_assert(smem_one <= 227 * 1024, "a CTA's shared memory");
    static const bool no_one_env = getenv("B200_UMMA_NO_ONE") != nullptr;   // measurement: the general rings at every row count
    const bool one = T <= 128 && !no_one_env;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<1, false, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_one));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<2, false, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_one));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<2, true, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_one));
    }
    static const CUtensorMap no_map{};  // the tile-major copy is fetched with plain bulk copies
    const CUtensorMap* wmap = W_tiles ? &no_map : q4k_weight_map(ctx, W, N, nSB, 128 * NT, kRawRow);
    if (!wmap) return B200_CUDA_ERROR;
    dim3 grid(n_tiles, t_tiles, splits);
    float* out = splits > 1 ? part : dst;
    const int out_ld = splits > 1 ? N : ldd;
    const size_t stride = splits > 1 ? (size_t)T * N : 0;
    {
        ProfScope ps(ctx, PROF_Q4K_GEMM);
        int8_t* const no_codes = nullptr;
        float* const no_scales = nullptr;
        __half* const no_x16 = nullptr;
        const unsigned short* const no_d = nullptr;
        if (one && fuse) launch_pdl(q4k_umma_gemm_kernel<2, true, 4, true>, grid, dim3(kUmmaThreads), smem_one, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, err_flag, sw.codes, sw.scales, sw_x16, W_tiles, no_d);
        else if (one && NT == 2) launch_pdl(q4k_umma_gemm_kernel<2, false, 4, true>, grid, dim3(kUmmaThreads), smem_one, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, err_flag, no_codes, no_scales, no_x16, W_tiles, no_d);
        else if (one) launch_pdl(q4k_umma_gemm_kernel<1, false, 4, true>, grid, dim3(kUmmaThreads), smem_one, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, err_flag, no_codes, no_scales, no_x16, W_tiles, no_d);
        else if (fuse) launch_pdl(q4k_umma_gemm_kernel<2, true>, grid, dim3(kUmmaThreads), smem, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, err_flag, sw.codes, sw.scales, sw_x16, W_tiles, no_d);
        else if (NT == 2) launch_pdl(q4k_umma_gemm_kernel<2, false>, grid, dim3(kUmmaThreads), smem, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, err_flag, no_codes, no_scales, no_x16, W_tiles, no_d);
        else launch_pdl(q4k_umma_gemm_kernel<1, false>, grid, dim3(kUmmaThreads), smem, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, err_flag, no_codes, no_scales, no_x16, W_tiles, no_d);
    }
    LAUNCH_CHECK(ctx);
    if (fuse && fused) *fused = true;
    if (splits > 1) {
        if (ctx->defer_reduce && ldd == N) {  // the consumer adds the partials (same order, same bits)
            ctx->pending = Parts{part, stride, splits, dst, T, N};
        } else {
            launch_pdl(splitk_reduce_kernel, dim3((unsigned)(((size_t)T * N + 255) / 256)), dim3(256), 0, ctx->stream, part, stride, splits, T, N, dst, ldd);
            LAUNCH_CHECK(ctx);
        }
    }
    return B200_OK;
}

// Q6_K weights (208-byte bodies row by row, d values behind them: launch_q6k_repack) x the per-32 activations as fp16
// tiles, on the same tcgen05 pipeline: the producers put the six-bit codes together and scale them in registers, so no
// dequantized copy of the matrix exists. From 32 rows in the fast class.
size_t q6k_umma_smem_bytes() { return (size_t)kASlotsKQ * kTileBytes + (size_t)kBStagesKQ * 2 * kTileBytes + (size_t)kProducers * 208 + 1024; }

// whether T rows of an [N][K] Q6_K matrix fit a scratch of `scratch_bytes` whose first 2 * slot_bytes hold activation slots
bool q6k_umma_fits(int sm_count, size_t slot_bytes, size_t scratch_bytes, int N, int K, int T) {
    if (K % 256 || T < 1 || !scratch_bytes) return false;
    const int nSB = K / 256, t_tiles = ceil_div(T, 256);
    const int max_splits = std::max(1, std::min(4, nSB / 2));
    const int NT = ceil_div(N, 256) * t_tiles * max_splits >= sm_count * 3 / 4 ? 2 : 1;
    const int n_tiles = ceil_div(N, 128 * NT);
    const int splits = std::max(1, std::min(max_splits, sm_count / std::max(1, n_tiles * t_tiles)));
    const size_t x_bytes = (size_t)t_tiles * 256 * K * 2;
    const size_t part_bytes = splits > 1 ? (size_t)splits * T * N * 4 : 0;
    const size_t part_off = slot_bytes ? 2 * slot_bytes : ((x_bytes + 255) & ~(size_t)255);
    return !(slot_bytes && x_bytes > slot_bytes) && part_off + part_bytes + 256 <= scratch_bytes;
}

int launch_q6k_matmul_umma(b200_ctx* ctx, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd) {
    return launch_kq_matmul_umma(ctx, B200_K_Q6K, W, N, K, aq, T, dst, ldd);
}

// kind B200_K_Q5K (the file's 176-byte blocks) or B200_K_Q6K (208-byte bodies + d values)
int launch_kq_matmul_umma(b200_ctx* ctx, int kind, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd) {
    ST_TRY(flush_pending_parts(ctx));  // the scratch is about to be reused
    if (kind != B200_K_Q5K && kind != B200_K_Q6K) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the K-quant tcgen05 matmul takes Q5_K or Q6_K");
    const int sb_bytes = kind == B200_K_Q6K ? 208 : 176;
    if (K % 256 || (reinterpret_cast<uintptr_t>(W) & 15)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "Q5_K / Q6_K need K %% 256 == 0 and 16-byte aligned weights");
    if (!ctx->umma_scratch) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the tcgen05 matmul needs the fast class's scratch");
    const int nSB = K / 256, t_tiles = ceil_div(T, 256);
    const int max_splits = std::max(1, std::min(4, nSB / 2));
    const int NT = ceil_div(N, 256) * t_tiles * max_splits >= ctx->sm_count * 3 / 4 ? 2 : 1;
    const int n_tiles = ceil_div(N, 128 * NT);
    const int splits = std::max(1, std::min(max_splits, ctx->sm_count / std::max(1, n_tiles * t_tiles)));
    const size_t x_bytes = (size_t)t_tiles * 256 * K * 2;
    const size_t part_bytes = splits > 1 ? (size_t)splits * T * N * 4 : 0;
    const bool slots = ctx->x16_slot_bytes > 0;
    const size_t part_off = slots ? 2 * ctx->x16_slot_bytes : ((x_bytes + 255) & ~(size_t)255);
    if ((slots && x_bytes > ctx->x16_slot_bytes) || part_off + part_bytes + 256 > ctx->umma_scratch_bytes)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "tcgen05 matmul scratch too small");
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ctx->umma_scratch) + part_off);
    const __half* x16 = slots ? ctx->x16_ready : nullptr;
    if (!x16) {
        __half* mine = slots ? x16_next_slot(ctx) : reinterpret_cast<__half*>(ctx->umma_scratch);
        ST_TRY(launch_act_to_f16(ctx, aq, T, K, mine));
        x16 = mine;
    }
    const int smem = (int)q6k_umma_smem_bytes();
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<1, false, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<2, false, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<1, false, 5>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_umma_gemm_kernel<2, false, 5>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    const CUtensorMap* wmap = q4k_weight_map(ctx, W, N, nSB, 128 * NT, sb_bytes);
    if (!wmap) return B200_CUDA_ERROR;
    const unsigned short* dvals = kind == B200_K_Q6K ? reinterpret_cast<const unsigned short*>(W + (size_t)N * nSB * 208) : nullptr;
    dim3 grid(n_tiles, t_tiles, splits);
    float* out = splits > 1 ? part : dst;
    const int out_ld = splits > 1 ? N : ldd;
    const size_t stride = splits > 1 ? (size_t)T * N : 0;
    {
        ProfScope ps(ctx, PROF_Q4K_GEMM);
        int8_t* const no_codes = nullptr;
        float* const no_scales = nullptr;
        __half* const no_x16 = nullptr;
        const uint8_t* const no_tiles = nullptr;
#define KQ_LAUNCH(NTV, FMTV) launch_pdl(q4k_umma_gemm_kernel<NTV, false, FMTV>, grid, dim3(kUmmaThreads), (size_t)smem, ctx->stream, *wmap, N, nSB, x16, T, out, out_ld, stride, ctx->err_flag, no_codes, no_scales, no_x16, no_tiles, dvals)
        if (kind == B200_K_Q6K) { if (NT == 2) KQ_LAUNCH(2, 6); else KQ_LAUNCH(1, 6); }
        else { if (NT == 2) KQ_LAUNCH(2, 5); else KQ_LAUNCH(1, 5); }
#undef KQ_LAUNCH
    }
    LAUNCH_CHECK(ctx);
    if (splits > 1) {
        if (ctx->defer_reduce && ldd == N) {
            ctx->pending = Parts{part, stride, splits, dst, T, N};
        } else {
            launch_pdl(splitk_reduce_kernel, dim3((unsigned)(((size_t)T * N + 255) / 256)), dim3(256), 0, ctx->stream, part, stride, splits, T, N, dst, ldd);
            LAUNCH_CHECK(ctx);
        }
    }
    return B200_OK;
}

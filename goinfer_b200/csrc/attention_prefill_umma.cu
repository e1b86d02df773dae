// attention_prefill_umma.cu — fast-class causal attention of a long prefill run on the 5th-generation tensor cores.
//
// A run is `nrows` query rows of ONE sequence at consecutive positions pos0 .. pos0+nrows-1 (a prefill chunk of the ragged
// step: decoder/resident/forward.go:60-84; the CPU path's per-row loop is decoder/program_cpu_n.go:497-515 over
// attendBatchedHeadsP, decoder/forwardn.go:295-501); row j attends keys 0 .. pos0+j of its slot's paged fp16 K/V. The
// reference's own tensor-core kernel for this is its Turing FlashAttention (backend/cuda/attn_fused.cu); this one is built
// for tcgen05:
//
//   one CTA = 128 query rows of one head; the walk over keys is FlashAttention's, 64 keys a tile
//   S = Q K^T     tcgen05.mma M128 N64 K16 x (HD/16), both operands K-major in shared memory, S in tensor memory (two
//                 buffers, so the next tile's product runs while this tile's softmax does)
//   softmax       four warps, one thread per query row: tcgen05.ld of the row's 64 scores, scale, causal mask, running max
//                 and sum in fp32 registers with no shuffles; P is rounded to fp16 and written to shared memory as the next
//                 product's 128-row operand (the row sums are taken over the rounded values, so the weights stay normalized)
//   O += P V      tcgen05.mma M128 N(HD) K16 x 4, V read as it lies in the cache ([key][dim]: the MN-major operand form,
//                 so nothing is transposed), O in tensor memory for the whole walk; when a row's maximum moves, its warp
//                 rescales its 32 rows of O in place (tcgen05.ld / st) before P is released
//   K/V tiles     two loader warps, cp.async 16 bytes a thread from the paged pool into a 3-stage ring laid out as the MMA
//                 wants it ([dim half][64 keys][128 B], 16-byte chunks XOR-swizzled by key row); tiled TMA boxes over 16-key
//                 blocks were measured far slower than their bytes on this part and are not used
// One thread issues every MMA; mbarriers (bounded waits) carry the hand-offs; tcgen05.commit frees stages.
//
// Q may be split into fp16 hi + lo parts (two products per tile: the scores then carry fp32-level accuracy) and so may P;
// prefill_umma_precision() says what is on and what each form costs.
#include <cstdlib>

#include "common.cuh"
#include "umma.cuh"

namespace {

constexpr int kPuKeys = 64, kPuStages = 3;
constexpr int kPuThreads = 7 * 32;  // warps 0-3 softmax, 4 MMA issue, 5-6 loaders
constexpr int kPuLoaders = 64;

// shared-memory descriptor of an MN-major operand with the 128-byte swizzle: 64 consecutive MN elements are a 128-byte
// line, eight lines (eight K positions) a 1024-byte atom; atoms of the next 64 MN elements lie `lbo` bytes further, atoms of
// the next eight K positions `sbo` bytes further
__device__ __forceinline__ uint64_t umma_desc_mn(unsigned smem_addr, unsigned lbo, unsigned sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) |
           (1ull << 46) | (2ull << 61);
}
// fp32 accumulate, f16 x f16, M = 128; b_mn: the B operand is MN-major
__host__ __device__ constexpr unsigned idesc_pu(unsigned n, bool b_mn) { return (1u << 4) | (b_mn ? (1u << 16) : 0u) | ((n >> 3) << 17) | ((128u >> 4) << 24); }

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ float pu_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// tanh(x) = 1 - 2 / (exp(2x) + 1), on the hardware exponential and reciprocal (about 1e-6 relative; the softcap's own arithmetic)
__device__ __forceinline__ float pu_tanh(float x) {
    const float e = pu_ex2(x * 2.8853900817779268f);
    return 1.f - __fdividef(2.f, e + 1.f);
}

template <int HD, bool QSPLIT, bool PSPLIT>
struct PuCfg {
    static constexpr int kHalves = HD / 64;                  // 64-wide slices of a row (the swizzle's 128-byte lines)
    static constexpr int kQTile = 128 * HD * 2;              // one fp16 part of the Q tile: [half][128 rows][128 B]
    static constexpr int kKVTile = kPuKeys * HD * 2;         // a K or V tile: [half][64 keys][128 B]
    static constexpr int kPTile = 128 * kPuKeys * 2;         // one fp16 part of P: [128 rows][128 B]
    static constexpr int kQBytes = (QSPLIT ? 2 : 1) * kQTile;
    static constexpr int kPBytes = 2 * (PSPLIT ? 2 : 1) * kPTile;   // two buffers
    static constexpr int kSmem = kQBytes + 2 * kPuStages * kKVTile + kPBytes + 1024;
    static constexpr int kTmemCols = HD == 128 ? 256 : 256;  // S0 | S1 (64 each) | O (HD), rounded to a power of two
};

// grid (row tiles of 128, heads); heavy tiles (late rows: most keys) first
template <int HD, bool QSPLIT, bool PSPLIT, bool CAP>
__global__ void __launch_bounds__(kPuThreads, 1) attn_prefill_umma_kernel(const float* __restrict__ q, int ldq, int nrows, int nKV, int G, float scale,
                                                                          float cap, int pos0, const __half* __restrict__ kpool,
                                                                          const __half* __restrict__ vpool, const int32_t* __restrict__ tbl,
                                                                          int block_rows, float* __restrict__ out, int ldo, int* __restrict__ err_flag) {
    using Cfg = PuCfg<HD, QSPLIT, PSPLIT>;
    extern __shared__ __align__(1024) uint8_t pu_smem[];
    __shared__ __align__(8) uint64_t kv_full[kPuStages], kv_empty[kPuStages], s_full[2], s_empty[2], p_full[2], p_empty[2], o_done;
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rt = (int)gridDim.x - 1 - (int)blockIdx.x, head = blockIdx.y, kvh = head / G;
    const int r0 = rt * 128;
    const int rows_here = min(128, nrows - r0);
    const int last_key = pos0 + r0 + rows_here - 1;          // the tile's last visible key
    const int n_tiles = last_key / kPuKeys + 1;
    uint8_t* smem = pu_smem + ((1024u - (smem_u32(pu_smem) & 1023u)) & 1023u);
    uint8_t* q_sm = smem;
    uint8_t* k_sm = q_sm + Cfg::kQBytes;
    uint8_t* v_sm = k_sm + kPuStages * Cfg::kKVTile;
    uint8_t* p_sm = v_sm + kPuStages * Cfg::kKVTile;
    volatile int* abort_v = &abort_s;

    if (tid == 0) {
        for (int s = 0; s < kPuStages; s++) {
            mbar_init(smem_u32(&kv_full[s]), kPuLoaders);   // every loader thread, after its copies landed
            mbar_init(smem_u32(&kv_empty[s]), 1);           // one tcgen05.commit
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&s_full[b]), 1);             // commit after the score MMAs
            mbar_init(smem_u32(&s_empty[b]), 4);            // the four softmax warps have read the buffer
            mbar_init(smem_u32(&p_full[b]), 4);             // ... have written P (and rescaled O)
            mbar_init(smem_u32(&p_empty[b]), 1);            // commit after the P V MMAs
        }
        mbar_init(smem_u32(&o_done), 1);                    // commit after every tile's P V MMAs
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // the Q tile: f32 -> fp16 (hi, and lo = the rounding remainder), [half][128 rows][128 B], 16-byte chunks swizzled by row
    for (int i = tid; i < 128 * (HD / 8); i += kPuThreads) {
        const int row = i / (HD / 8), c = i % (HD / 8);      // chunk c = dims 8c .. 8c+7
        const int r = min(r0 + row, nrows - 1);
        const float4 a = *reinterpret_cast<const float4*>(q + (size_t)r * ldq + (size_t)head * HD + 8 * c);
        const float4 b = *reinterpret_cast<const float4*>(q + (size_t)r * ldq + (size_t)head * HD + 8 * c + 4);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint4 hi, lo;
        unsigned* ph = &hi.x;
        unsigned* pl = &lo.x;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const __half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
            const float2 hf = __half22float2(h);
            const __half2 l = __floats2half2_rn(v[2 * e] - hf.x, v[2 * e + 1] - hf.y);
            ph[e] = *reinterpret_cast<const unsigned*>(&h);
            pl[e] = *reinterpret_cast<const unsigned*>(&l);
        }
        const unsigned off = (unsigned)((c >> 3) * (128 * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
        *reinterpret_cast<uint4*>(q_sm + off) = hi;
        if (QSPLIT) *reinterpret_cast<uint4*>(q_sm + Cfg::kQTile + off) = lo;
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy stores -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    const unsigned tm_s[2] = {tmem_base, tmem_base + 64}, tm_o = tmem_base + 128;

    if (warp >= 5) {
        // ---- loaders: tile j = keys 64j .. 64j+63 of K and of V into stage j % 3 ----
        const int lt = tid - 5 * 32;   // 0..63
        // thread lt copies 16-byte chunk lt % (HD/8) of key rows lt / (HD/8) + (64 / (HD/8)) i: within a 16-key slab (which lies in
        // one block) the block is looked up once
        constexpr int CPR = HD / 8, RSTEP = kPuLoaders / CPR, PER_SLAB = 16 / RSTEP;
        const int c = lt % CPR, ra = lt / CPR;
        auto issue = [&](int j) {
            const unsigned kd = smem_u32(k_sm + (size_t)(j % kPuStages) * Cfg::kKVTile), vd = smem_u32(v_sm + (size_t)(j % kPuStages) * Cfg::kKVTile);
#pragma unroll 1
            for (int sl = 0; sl < kPuKeys / 16; sl++) {
                // a slab wholly past the last visible key repeats the last visible one (finite numbers that the mask then weighs
                // by zero) instead of touching an unmapped block
                const int key_s = min(j * kPuKeys + 16 * sl, last_key & ~15);
                const int blk = tbl[key_s / block_rows];
                const uint8_t* kb = reinterpret_cast<const uint8_t*>(kpool) + ((((size_t)blk * nKV + kvh) * block_rows + (key_s % block_rows)) * HD) * 2 + (size_t)c * 16;
                const uint8_t* vb = reinterpret_cast<const uint8_t*>(vpool) + (kb - reinterpret_cast<const uint8_t*>(kpool));
#pragma unroll
                for (int ii = 0; ii < PER_SLAB; ii++) {
                    const int r = ra + RSTEP * ii, row = 16 * sl + r;
                    const unsigned d = (unsigned)((c >> 3) * (kPuKeys * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(kd + d), "l"(kb + (size_t)r * (HD * 2)));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(vd + d), "l"(vb + (size_t)r * (HD * 2)));
                }
            }
        };
        // A thread's arrival on a stage's barrier is tied to the completion of its own copies (cp.async.mbarrier.arrive), so the
        // loaders never wait for data: they only wait for a stage to be free again.
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; t++) {
            // the stage of tile t was last read by the products of tile t - 3
            if (t >= kPuStages) ok = mbar_wait_spin(smem_u32(&kv_empty[t % kPuStages]), (unsigned)(((t / kPuStages) - 1) & 1), abort_v);
            if (!ok) break;
            issue(t);
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(&kv_full[t % kPuStages])) : "memory");
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");   // nothing of this thread's is in flight when the CTA leaves
        if (!ok) abort_s = 1;
    } else if (warp == 4) {
        if (lane == 0) {
            // ---- the MMA issuer ----
            const unsigned qa = smem_u32(q_sm), pa = smem_u32(p_sm);
            bool ok = true;
            auto issue_pv = [&](int j) {   // O += P_j V_j
                const int b = j & 1;
                const unsigned vb = smem_u32(v_sm + (size_t)(j % kPuStages) * Cfg::kKVTile);
#pragma unroll
                for (int part = 0; part < (PSPLIT ? 2 : 1); part++)
#pragma unroll
                    for (int ks = 0; ks < kPuKeys / 16; ks++)
                        umma_f16(tm_o, umma_desc(pa + (unsigned)((b * (PSPLIT ? 2 : 1) + part) * Cfg::kPTile + ks * 32)),
                                 umma_desc_mn(vb + (unsigned)(ks * 2 * 1024), kPuKeys * 128, 1024), idesc_pu(HD, true), (j > 0 || part > 0 || ks > 0) ? 1u : 0u);
                umma_commit(smem_u32(&kv_empty[j % kPuStages]));
                umma_commit(smem_u32(&p_empty[b]));
                umma_commit(smem_u32(&o_done));
            };
            for (int j = 0; j < n_tiles && ok; j++) {
                const int b = j & 1;
                ok = mbar_wait_spin(smem_u32(&kv_full[j % kPuStages]), (unsigned)((j / kPuStages) & 1), abort_v);
                if (ok && j >= 2) ok = mbar_wait_spin(smem_u32(&s_empty[b]), (unsigned)(((j >> 1) - 1) & 1), abort_v);
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the loaders' copies, seen through the barrier, before the tensor core reads them
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned kb = smem_u32(k_sm + (size_t)(j % kPuStages) * Cfg::kKVTile);
#pragma unroll
                for (int part = 0; part < (QSPLIT ? 2 : 1); part++)
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++)
                        umma_f16(tm_s[b], umma_desc(qa + (unsigned)(part * Cfg::kQTile + (ks >> 2) * (128 * 128) + (ks & 3) * 32)),
                                 umma_desc(kb + (unsigned)((ks >> 2) * (kPuKeys * 128) + (ks & 3) * 32)), idesc_pu(kPuKeys, false),
                                 (part > 0 || ks > 0) ? 1u : 0u);
                umma_commit(smem_u32(&s_full[b]));
                if (j >= 1) {   // the product of the tile before, once its P is there (the scores above run meanwhile)
                    ok = mbar_wait_spin(smem_u32(&p_full[(j - 1) & 1]), (unsigned)(((j - 1) >> 1) & 1), abort_v);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    issue_pv(j - 1);
                }
            }
            if (ok) {
                const int j = n_tiles - 1;
                ok = mbar_wait_spin(smem_u32(&p_full[j & 1]), (unsigned)((j >> 1) & 1), abort_v);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    issue_pv(j);
                }
            }
            if (!ok) abort_s = 1;
        }
    } else {
        // ---- softmax: thread = query row r0 + tid; warp w owns tensor-memory lanes 32w .. 32w+31 ----
        const int row = tid;
        const int kmax = pos0 + min(r0 + row, nrows - 1);   // last key this row sees (rows past the run repeat the last one)
        const unsigned lane_off = (unsigned)(warp * 32) << 16;
        const float sl2 = scale * 1.4426950408889634f;       // scores are kept in units of log2 e, so that exp is one ex2
        const float cap_l2 = cap * 1.4426950408889634f, scale_over_cap = CAP ? scale / cap : 0.f;
        const float mul = CAP ? 1.f : sl2;
        const int kmin_warp = pos0 + min(r0 + warp * 32, nrows - 1);   // the last key the warp's first row sees
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            const int b = j & 1;
            ok = mbar_wait_spin(smem_u32(&s_full[b]), (unsigned)((j >> 1) & 1), abort_v);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            unsigned sr[2][32];
            tmem_ld32(tm_s[b] + lane_off, sr[0]);
            tmem_ld32(tm_s[b] + lane_off + 32, sr[1]);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_empty[b]));   // the buffer may take the scores of tile j + 2
            // scores -> log2 units, causal mask, row maximum
            const int key0 = j * kPuKeys;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains: the maximum is not one long dependency
            float* s = reinterpret_cast<float*>(&sr[0][0]);
            if (CAP) {
#pragma unroll
                for (int i = 0; i < 64; i++) s[i] = cap_l2 * pu_tanh(s[i] * scale_over_cap);
            }
            if (key0 + 63 > kmin_warp) {   // a tile that reaches past some row's last key (the last tiles of a walk): mask
#pragma unroll
                for (int i = 0; i < 64; i++) s[i] = key0 + i <= kmax ? s[i] : -INFINITY;
            }
#pragma unroll
            for (int i = 0; i < 64; i++) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
            // the scores stay as the tensor core left them; scale (and the change to log2 units) rides in the exponent's fma
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * mul;
            // The reference point of the exponentials follows the row maximum lazily: it moves only when the maximum has grown by
            // more than 2^8 past it (weights then stay below 256, far inside fp16 and fp32 range, and the final division by the
            // row sum takes the common factor out exactly as with the true maximum). A moved reference costs a pass over the
            // row's accumulator in tensor memory, so this keeps that pass to the first tiles of a walk.
            // (key 0 is visible to every row: the reference is finite from the first tile on)
            const float m_new = (mx > m_run + 8.f) ? mx : m_run;
            const float alpha = pu_ex2(m_run - m_new);
            // O *= alpha where a row's maximum moved: the warp's 32 rows in place, after the product of the tile before
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                ok = mbar_wait_spin(smem_u32(&o_done), (unsigned)((j - 1) & 1), abort_v);   // P V of tile j-1 has been accumulated
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                for (int cb = 0; cb < HD / 32; cb++) {
                    unsigned orow[32];
                    tmem_ld32(tm_o + lane_off + cb * 32, orow);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; i++) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                    tmem_st32(tm_o + lane_off + cb * 32, orow);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            // the P buffer is read by the product of tile j - 2 until p_empty says otherwise
            if (j >= 2) {
                ok = mbar_wait_spin(smem_u32(&p_empty[b]), (unsigned)(((j >> 1) - 1) & 1), abort_v);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            }
            // P, rounded to fp16 (hi) and, with PSPLIT, the remainder (lo), straight into the buffer; the row sum is taken over
            // what the tensor core will see
            uint8_t* pb = p_sm + (size_t)(b * (PSPLIT ? 2 : 1)) * Cfg::kPTile + (size_t)row * 128;
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 8; c++) {
                uint4 ph, pl;
                unsigned* wh = &ph.x;
                unsigned* wl = &pl.x;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float p0 = pu_ex2(fmaf(s[8 * c + 2 * e], mul, -m_new)), p1 = pu_ex2(fmaf(s[8 * c + 2 * e + 1], mul, -m_new));
                    const __half2 h = __floats2half2_rn(p0, p1);
                    const float2 hf = __half22float2(h);
                    wh[e] = *reinterpret_cast<const unsigned*>(&h);
                    if (PSPLIT) {
                        const __half2 l = __floats2half2_rn(p0 - hf.x, p1 - hf.y);
                        wl[e] = *reinterpret_cast<const unsigned*>(&l);
                        ps4[e] += p0 + p1;
                    } else {
                        ps4[e] += hf.x + hf.y;
                    }
                }
                *reinterpret_cast<uint4*>(pb + ((c ^ (row & 7)) << 4)) = ph;
                if (PSPLIT) *reinterpret_cast<uint4*>(pb + Cfg::kPTile + ((c ^ (row & 7)) << 4)) = pl;
            }
            l_run = l_run * alpha + ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
            m_run = m_new;
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[b]));
        }
        if (ok) {
            // the last product, then the rows: O / l
            ok = mbar_wait_spin(smem_u32(&o_done), (unsigned)((n_tiles - 1) & 1), abort_v);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = 1.f / l_run;
            float* op = out + (size_t)(r0 + row) * ldo + (size_t)head * HD;
#pragma unroll
            for (int cb = 0; cb < HD / 32; cb++) {
                unsigned orow[32];
                tmem_ld32(tm_o + lane_off + cb * 32, orow);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row < rows_here) {
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        *reinterpret_cast<float4*>(op + cb * 32 + 4 * i) =
                            make_float4(__uint_as_float(orow[4 * i]) * inv, __uint_as_float(orow[4 * i + 1]) * inv, __uint_as_float(orow[4 * i + 2]) * inv,
                                        __uint_as_float(orow[4 * i + 3]) * inv);
                }
            }
        } else {
            abort_s = 1;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (abort_s && tid == 0 && err_flag) atomicExch(err_flag, 1);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(Cfg::kTmemCols));
}

template <int HD, bool QSPLIT, bool PSPLIT, bool CAP>
int run_prefill_umma(b200_ctx* ctx, const float* q, int ldq, int nrows, int nH, int nKV, float scale, float cap, int pos0, const int32_t* tbl,
                     KVView kv, float* out, int ldo) {
    using Cfg = PuCfg<HD, QSPLIT, PSPLIT>;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(attn_prefill_umma_kernel<HD, QSPLIT, PSPLIT, CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
    }
    dim3 grid(ceil_div(nrows, 128), nH);
    {
        ProfScope ps(ctx, PROF_ATTN_SPLIT);
        attn_prefill_umma_kernel<HD, QSPLIT, PSPLIT, CAP><<<grid, kPuThreads, Cfg::kSmem, ctx->stream>>>(q, ldq, nrows, nKV, nH / nKV, scale, cap, pos0, kv.k,
                                                                                                   kv.v, tbl, kv.block_rows, out, ldo, ctx->err_flag);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

// Runs of at least this many rows go through the tcgen05 kernel (one CTA per 128 rows and head); shorter runs stay with the
// mma.sync kernel, whose 16-row tiles fill the SMs better.
int prefill_umma_min_rows() {
    static const int v = [] {
        const char* e = getenv("B200_PREFILL_UMMA_MIN_ROWS");
        return e ? atoi(e) : 128;
    }();
    return v;
}

// How the operands are rounded (B200_PREFILL_PREC overrides it for comparisons). Measured on a 2048-row run 4096 rows deep
// (32 query / 8 kv heads of 128, unit-variance q, k, v) against the f64 oracle:
//   0: Q and P single fp16        0.378 ms a layer (455 TFLOP/s)   relative L2 2.6e-4, max |error| 6.8e-4
//   1: Q as fp16 hi + lo          0.458 ms         (376 TFLOP/s)               1.5e-4,             3.5e-4
//   2: Q and P as hi + lo         0.531 ms         (323 TFLOP/s)               1.1e-6,             2.5e-6
// The fast class's matmuls round their operands to fp16 (1.5e-3 relative per product), so the cheapest form is well inside
// the class's tolerance and is the default; the bar it is held to: relative L2 5e-4, max |error| 1e-3 of the value scale.
int prefill_umma_precision() {
    static const int v = [] {
        const char* e = getenv("B200_PREFILL_PREC");
        return e ? atoi(e) : 0;
    }();
    return v;
}

bool prefill_attention_umma_supported(int nH, int nKV, int hd, int block_rows, const void* q, int ldq, const void* kpool, const void* vpool,
                                      const void* out, int ldo) {
    return (hd == 128 || hd == 64) && nKV > 0 && nH % nKV == 0 && block_rows % 16 == 0 && (ldq & 3) == 0 && (ldo & 3) == 0 &&
           ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kpool) | reinterpret_cast<uintptr_t>(vpool) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
}

// precision: 0 = Q and P single fp16, 1 = Q split hi + lo, 2 = Q and P split (fp32-level scores and weights)
int launch_prefill_attention_umma(b200_ctx* ctx, const float* q, int ldq, int nrows, int nH, int nKV, int hd, float scale, float softcap, int slot,
                                  int pos0, KVView kv, float* out, int ldo, int precision) {
    if (nrows <= 0) return B200_OK;
    const int32_t* tbl = kv.table + (size_t)slot * kv.max_blocks;
#define PU_CASE(HD_, QS_, PS_)                                                                                                      \
    return softcap != 0.f ? run_prefill_umma<HD_, QS_, PS_, true>(ctx, q, ldq, nrows, nH, nKV, scale, softcap, pos0, tbl, kv, out, ldo) \
                          : run_prefill_umma<HD_, QS_, PS_, false>(ctx, q, ldq, nrows, nH, nKV, scale, softcap, pos0, tbl, kv, out, ldo)
    if (hd == 128) {
        if (precision == 0) PU_CASE(128, false, false);
        if (precision == 1) PU_CASE(128, true, false);
        PU_CASE(128, true, true);
    }
    if (hd == 64) {
        if (precision == 0) PU_CASE(64, false, false);
        if (precision == 1) PU_CASE(64, true, false);
        PU_CASE(64, true, true);
    }
#undef PU_CASE
    B200_FAIL(ctx, B200_BAD_ARGUMENT, "tcgen05 prefill attention: head_dim %d is not built", hd);
}

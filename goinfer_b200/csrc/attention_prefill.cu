// attention_prefill.cu — fast-class causal attention for a run of query rows of ONE sequence at consecutive positions
// (a prefill chunk of the ragged step: decoder/resident/forward.go:60-84; the CPU path's per-row loop is
// decoder/program_cpu_n.go:497-515 over attendBatchedHeadsP, decoder/forwardn.go:295-501).
//
// Row j of the run sits at position pos0 + j and attends keys 0 .. pos0 + j of its slot's paged fp16 K/V (the run's own
// keys were stored by the RoPE/KV-store kernel just before). One CTA owns 16 consecutive query rows of one kv head; its
// G warps are the G query heads of that kv head's group, so the K/V tiles (32 keys, cp.async into a 3-stage ring shared
// by the warps, 16-byte chunks XOR-swizzled by key row) are fetched once per group. Per warp and tile:
//   S[16 rows][32 keys] = Q K^T   mma.sync m16n8k16, Q held in registers as f16 hi + lo parts (fp32-level accuracy)
//   online softmax in fp32 registers (rows gid and gid+8 of the lane's quad)
//   O[16][HD] += P V              P = the S accumulators re-used as the A fragment, split hi + lo as well
// The walk is flash-attention style, one pass over the keys, nothing written but the final rows. The arithmetic is the
// decode kernel's (same splits, same fp32 softmax); only the grouping of rows differs.
#include <cstdlib>

#include "common.cuh"

namespace {

__device__ __forceinline__ float pf_score(float dot, float scale, float cap) {
    float s = dot * scale;
    if (cap != 0.f) s = cap * tanhf(s / cap);
    return s;
}
__device__ __forceinline__ void pf_ldsm_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_ldsm_x4_t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pf_split(float x, float y, unsigned& hi, unsigned& lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const unsigned*>(&h);
    lo = *reinterpret_cast<const unsigned*>(&l);
}

constexpr int kPfStages = 3, kPfKeys = 32;

template <int HD, int G>
__global__ void __launch_bounds__(32 * G) attn_prefill_kernel(const float* __restrict__ q, int ldq, int nrows, int nH, int nKV,
                                                              float scale, float cap, int pos0, const __half* __restrict__ kpool,
                                                              const __half* __restrict__ vpool, const int32_t* __restrict__ tbl,
                                                              int block_rows, float* __restrict__ out, int ldo) {
    constexpr int KS = HD / 16, CPR = HD / 8, ROWB = HD * 2, TILE = kPfKeys * ROWB, NT = HD / 8;
    constexpr int THREADS = 32 * G, CHUNKS = kPfKeys * CPR;  // 16-byte chunks of one K (or V) tile
    extern __shared__ __align__(128) uint8_t pf_smem[];
    // heavy tiles (late rows: most keys) first, so the tail of the grid is short work
    const int rt = (int)gridDim.x - 1 - (int)blockIdx.x, kvh = blockIdx.y;
    const int r0 = rt * 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
    const int head = kvh * G + warp;
    const unsigned sm_s = (unsigned)__cvta_generic_to_shared(pf_smem);
    const int ra = min(r0 + gid, nrows - 1), rb = min(r0 + gid + 8, nrows - 1);  // this lane's two rows (clamped copies past the end)
    const int last_key = pos0 + min(r0 + 15, nrows - 1);                        // the tile's last visible key
    const int n_tiles = last_key / kPfKeys + 1;

    // Q fragments, hi and lo
    unsigned qh[KS][4], ql[KS][4];
    {
        const float* qa = q + (size_t)ra * ldq + (size_t)head * HD;
        const float* qb = q + (size_t)rb * ldq + (size_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const float2 a0 = *reinterpret_cast<const float2*>(qa + 16 * ks + 2 * tig);
            const float2 a1 = *reinterpret_cast<const float2*>(qb + 16 * ks + 2 * tig);
            const float2 a2 = *reinterpret_cast<const float2*>(qa + 16 * ks + 8 + 2 * tig);
            const float2 a3 = *reinterpret_cast<const float2*>(qb + 16 * ks + 8 + 2 * tig);
            pf_split(a0.x, a0.y, qh[ks][0], ql[ks][0]);
            pf_split(a1.x, a1.y, qh[ks][1], ql[ks][1]);
            pf_split(a2.x, a2.y, qh[ks][2], ql[ks][2]);
            pf_split(a3.x, a3.y, qh[ks][3], ql[ks][3]);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const int kmax_a = pos0 + ra, kmax_b = pos0 + rb;

    auto issue = [&](int it) {
        if (it < n_tiles) {
            const unsigned dst = sm_s + (unsigned)((it % kPfStages) * 2 * TILE);
#pragma unroll
            for (int i = 0; i < (CHUNKS + THREADS - 1) / THREADS; i++) {
                const int ci = threadIdx.x + THREADS * i;
                if (CHUNKS % THREADS == 0 || ci < CHUNKS) {
                    const int row = ci / CPR, c = ci % CPR;
                    // a 16-key slab lies in one block; a slab wholly past the last visible key repeats the last visible
                    // one (finite numbers that the mask then weighs by zero) instead of touching an unmapped block
                    const int key = min(it * kPfKeys + row, (last_key & ~15) + (row & 15));
                    const int blk = tbl[key / block_rows];
                    const size_t off = ((((size_t)blk * nKV + kvh) * block_rows + (key % block_rows)) * HD) * 2 + (size_t)c * 16;
                    const unsigned d = (unsigned)(row * ROWB + ((c ^ (row & 7)) << 4));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + d), "l"(reinterpret_cast<const uint8_t*>(kpool) + off));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + TILE + d), "l"(reinterpret_cast<const uint8_t*>(vpool) + off));
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
#pragma unroll
    for (int s = 0; s < kPfStages - 1; s++) issue(s);

    const int lrow = (lane & 7) + ((lane >> 4) << 3), lsel = (lane >> 3) & 1;
    for (int it = 0; it < n_tiles; it++) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kPfStages - 2));  // this thread's part of tile `it` has landed
        __syncthreads();                                                   // everyone's has; tile it-1 is no longer read
        issue(it + kPfStages - 1);
        const unsigned kb = sm_s + (unsigned)((it % kPfStages) * 2 * TILE), vb = kb + TILE;
        const int key0 = it * kPfKeys;
        // S: 4 key groups of 8; hi and lo products accumulate apart to shorten the dependency chains
        float sh[4][4], sl[4][4];
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) sh[j][i] = sl[j][i] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int sl16 = 0; sl16 < 2; sl16++) {
                unsigned b0, b1, b2, b3;
                const int row = lrow + 16 * sl16;
                pf_ldsm_x4(kb + (unsigned)(row * ROWB + (((2 * ks + lsel) ^ (row & 7)) << 4)), b0, b1, b2, b3);
                pf_mma(sh[2 * sl16], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b0, b1);
                pf_mma(sh[2 * sl16 + 1], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b2, b3);
                pf_mma(sl[2 * sl16], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b0, b1);
                pf_mma(sl[2 * sl16 + 1], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b2, b3);
            }
        }
        // scores, causal mask, running max per row
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int kk = key0 + 8 * j + 2 * tig;
            sh[j][0] = kk <= kmax_a ? pf_score(sh[j][0] + sl[j][0], scale, cap) : -INFINITY;
            sh[j][1] = kk + 1 <= kmax_a ? pf_score(sh[j][1] + sl[j][1], scale, cap) : -INFINITY;
            sh[j][2] = kk <= kmax_b ? pf_score(sh[j][2] + sl[j][2], scale, cap) : -INFINITY;
            sh[j][3] = kk + 1 <= kmax_b ? pf_score(sh[j][3] + sl[j][3], scale, cap) : -INFINITY;
            mx_a = fmaxf(mx_a, fmaxf(sh[j][0], sh[j][1]));
            mx_b = fmaxf(mx_b, fmaxf(sh[j][2], sh[j][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        // key 0 is visible to every row, so after the first tile the running maxima are finite
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float al_a = __expf(m_a - mn_a), al_b = __expf(m_b - mn_b);
        float ps_a = 0.f, ps_b = 0.f;
        unsigned ph[2][4], pl[2][4];  // P as A fragments of the two 16-key steps
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p0 = __expf(sh[j][0] - mn_a), p1 = __expf(sh[j][1] - mn_a);
            const float p2 = __expf(sh[j][2] - mn_b), p3 = __expf(sh[j][3] - mn_b);
            ps_a += p0 + p1;
            ps_b += p2 + p3;
            // key group j is columns (j&1)*8.. of step j>>1: a0/a1 for the low half, a2/a3 for the high half
            pf_split(p0, p1, ph[j >> 1][(j & 1) * 2], pl[j >> 1][(j & 1) * 2]);
            pf_split(p2, p3, ph[j >> 1][(j & 1) * 2 + 1], pl[j >> 1][(j & 1) * 2 + 1]);
        }
        ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 1);
        ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 2);
        ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 1);
        ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 2);
        l_a = l_a * al_a + ps_a;
        l_b = l_b * al_b + ps_b;
        m_a = mn_a;
        m_b = mn_b;
        // O = O * alpha + P V
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; n2++) {
            o[2 * n2][0] *= al_a; o[2 * n2][1] *= al_a; o[2 * n2][2] *= al_b; o[2 * n2][3] *= al_b;
            o[2 * n2 + 1][0] *= al_a; o[2 * n2 + 1][1] *= al_a; o[2 * n2 + 1][2] *= al_b; o[2 * n2 + 1][3] *= al_b;
#pragma unroll
            for (int st = 0; st < 2; st++) {
                unsigned v0, v1, v2, v3;
                const int row = lrow + 16 * st;
                // transposed 8x8 blocks: (keys 0-7, dims 16 n2..), (keys 0-7, dims +8), (keys 8-15, dims ..), (keys 8-15, dims +8)
                pf_ldsm_x4_t(vb + (unsigned)(row * ROWB + (((2 * n2 + lsel) ^ (row & 7)) << 4)), v0, v1, v2, v3);
                pf_mma(o[2 * n2], ph[st][0], ph[st][1], ph[st][2], ph[st][3], v0, v2);
                pf_mma(o[2 * n2 + 1], ph[st][0], ph[st][1], ph[st][2], ph[st][3], v1, v3);
                pf_mma(o[2 * n2], pl[st][0], pl[st][1], pl[st][2], pl[st][3], v0, v2);
                pf_mma(o[2 * n2 + 1], pl[st][0], pl[st][1], pl[st][2], pl[st][3], v1, v3);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    const float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
    if (r0 + gid < nrows) {
        float* op = out + (size_t)(r0 + gid) * ldo + (size_t)head * HD;
#pragma unroll
        for (int n = 0; n < NT; n++) *reinterpret_cast<float2*>(op + 8 * n + 2 * tig) = make_float2(o[n][0] * inv_a, o[n][1] * inv_a);
    }
    if (r0 + gid + 8 < nrows) {
        float* op = out + (size_t)(r0 + gid + 8) * ldo + (size_t)head * HD;
#pragma unroll
        for (int n = 0; n < NT; n++) *reinterpret_cast<float2*>(op + 8 * n + 2 * tig) = make_float2(o[n][2] * inv_b, o[n][3] * inv_b);
    }
}

template <int HD, int G>
int run_prefill(b200_ctx* ctx, const float* q, int ldq, int nrows, int nH, int nKV, float scale, float cap, int pos0,
                const int32_t* tbl, KVView kv, float* out, int ldo) {
    constexpr int smem = kPfStages * 2 * kPfKeys * HD * 2;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(attn_prefill_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    dim3 grid(ceil_div(nrows, 16), nKV);
    {
        ProfScope ps(ctx, PROF_ATTN_SPLIT);
        attn_prefill_kernel<HD, G><<<grid, 32 * G, smem, ctx->stream>>>(q, ldq, nrows, nH, nKV, scale, cap, pos0, kv.k, kv.v, tbl,
                                                                        kv.block_rows, out, ldo);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

bool prefill_attention_supported(int nH, int nKV, int hd, int block_rows) {
    const int G = nKV > 0 ? nH / nKV : 0;
    return (hd == 128 || hd == 64) && (G == 1 || G == 2 || G == 4 || G == 8) && block_rows % 16 == 0;
}

// q: the run's first row ([nrows][ldq] f32, after RoPE); out: the run's first output row ([nrows][ldo] f32); the run is
// `nrows` rows of slot `slot` at positions pos0 .. pos0+nrows-1 whose K/V are already in the pool.
int launch_prefill_attention(b200_ctx* ctx, const float* q, int ldq, int nrows, int nH, int nKV, int hd, float scale,
                             float softcap, int slot, int pos0, KVView kv, float* out, int ldo) {
    if (nrows <= 0) return B200_OK;
    const int G = nH / nKV;
    // long runs: the tcgen05 kernel (128 rows of a head per CTA)
    static const bool no_umma = getenv("B200_NO_UMMA") != nullptr || getenv("B200_NO_PREFILL_UMMA") != nullptr;
    if (!no_umma && nrows >= prefill_umma_min_rows() &&
        prefill_attention_umma_supported(nH, nKV, hd, kv.block_rows, q, ldq, kv.k, kv.v, out, ldo))
        return launch_prefill_attention_umma(ctx, q, ldq, nrows, nH, nKV, hd, scale, softcap, slot, pos0, kv, out, ldo, prefill_umma_precision());
    const int32_t* tbl = kv.table + (size_t)slot * kv.max_blocks;
#define PF_CASE(HD_, G_) \
    if (hd == HD_ && G == G_) return run_prefill<HD_, G_>(ctx, q, ldq, nrows, nH, nKV, scale, softcap, pos0, tbl, kv, out, ldo)
    PF_CASE(128, 1); PF_CASE(128, 2); PF_CASE(128, 4); PF_CASE(128, 8);
    PF_CASE(64, 1); PF_CASE(64, 2); PF_CASE(64, 4); PF_CASE(64, 8);
#undef PF_CASE
    B200_FAIL(ctx, B200_BAD_ARGUMENT, "prefill attention: head_dim %d with group %d is not built", hd, G);
}

// gemm_stream.cu — Q4_K x per-32 int8 matmul for small row counts (4..63 rows), built to keep HBM busy.
//
//   dst[t][n] = sum over groups g of 32:  fma(idot(n,t,g), (d*sc_g)*aS[t][g], .) then fma(-(dmin*m_g), asum[t][g], .)
//
// the W4A8 product of backend/cuda/actgroup.cu:311-355 with one ascending chain per output (so, without a K split, the
// bits are those of the exact class's kernels). At these row counts the matmul is a stream of the weights: what matters
// is bytes in flight. One CTA owns 64 weight rows; a producer thread brings the rows' raw super-blocks in with one tiled
// TMA copy each (box 144 bytes x 64 rows) through a ring of 4 stages (3 at 32 rows; three or four CTAs share an SM), and four consumer
// warps (16 rows each) take their fragments out of the ring, free the stage at once, and run the integer MMAs
// (mma.sync m16n8k32 u8 x s8: one instruction is one 32-group for 16 rows x 8 rows of activations) and the f32 chain.
// The k order inside a group is permuted the same way for weights and activations (8 bytes per lane), which an integer dot
// does not see. The activation rows' codes, scales and group sums of the super-block ride in the same stage (four more
// tiled copies; the codes in the copy engine's 128-byte swizzle, so that fragment loads are free of bank conflicts).
// With splits > 1 every K range writes its own partial matrix and a second kernel adds them in order.
// Every mbarrier wait is bounded: on expiry the CTA raises the error flag and returns.
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "umma.cuh"

namespace {

constexpr int kSRows = 64, kSConsumers = 4, kSThreads = (kSConsumers + 1) * 32, kSWBytes = kSRows * 144;
// a stage: the 64 rows' raw super-blocks (9216 B), then the activation rows' codes as two [8*nt][128 B] halves in the
// copy engine's 128-byte swizzle (fragment loads of 8 rows then miss each other's banks), their 8 scales and their 8
// group sums ([8*nt][32 B] each); rounded up to 1 KB so that every stage's swizzled halves sit on 1 KB boundaries
__host__ __device__ constexpr int stream_stage_bytes(int nt) { return (kSWBytes + 8 * nt * (256 + 64) + 1023) / 1024 * 1024; }
__host__ __device__ constexpr int stream_stages(int nt) { return nt <= 2 ? 4 : 3; }  // 48-87 KB per CTA: two to four CTAs per SM

__device__ __forceinline__ unsigned s_byte(int k, unsigned s0, unsigned s1, unsigned s2) {
    unsigned w = k < 4 ? s0 : (k < 8 ? s1 : s2);
    return (w >> ((k & 3) << 3)) & 0xffu;
}
// 6-bit scale and minimum of sub-block j (ggml get_scale_min_k4; backend/cuda/kernels/ks_a1_test.go:62-67)
__device__ __forceinline__ void s_scale_min(int j, unsigned s0, unsigned s1, unsigned s2, int* sc, int* m) {
    if (j < 4) {
        *sc = (int)(s_byte(j, s0, s1, s2) & 63u);
        *m = (int)(s_byte(j + 4, s0, s1, s2) & 63u);
    } else {
        unsigned hi = s_byte(j + 4, s0, s1, s2);
        *sc = (int)((hi & 0x0Fu) | ((s_byte(j - 4, s0, s1, s2) >> 6) << 4));
        *m = (int)((hi >> 4) | ((s_byte(j, s0, s1, s2) >> 6) << 4));
    }
}
__device__ __forceinline__ float s_h2f(unsigned short b) { return __half2float(__ushort_as_half(b)); }

#define S_MAGIC_I 0x4B400000
#define S_MAGIC_F 12582912.0f

// d = a*b + c, c the magic-number bias that makes the int32 result readable as a float
__device__ __forceinline__ void s_mma(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(S_MAGIC_I));
}

template <int NT>  // token tiles of 8
__global__ void __launch_bounds__(kSThreads) q4k_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap cmap,
                                                               const __grid_constant__ CUtensorMap smap, int N, int nSB,
                                                               int T, float* __restrict__ dst, int ldd, size_t split_stride,
                                                               int* __restrict__ err_flag, const int32_t* __restrict__ offs) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(1024) uint8_t s_ring_raw[];
    uint8_t* s_ring = s_ring_raw + ((1024u - (smem_u32(s_ring_raw) & 1023u)) & 1023u);  // the launch reserves 1 KB for this round-up
    constexpr int kSStages = stream_stages(NT), kSStageBytes = stream_stage_bytes(NT);
    __shared__ __align__(8) uint64_t full[kSStages], empty[kSStages];
    __shared__ int abort_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    const int n0 = blockIdx.x * kSRows;
    // plain: grid.y splits K. Grouped (offs given): grid.y is the expert, whose weights are rows e*N .. of the map and whose
    // activation rows are offs[e] .. offs[e+1] of the (expert-sorted) activation buffers.
    int w_row0 = n0, t_base = 0, splits = gridDim.y, split = blockIdx.y, n_pass = 1;
    if (offs) {
        const int e = blockIdx.y;
        t_base = offs[e];
        T = offs[e + 1] - t_base;   // this expert's rows: walked 8*NT at a time, the weights streamed again for every pass
        if (T <= 0) return;
        n_pass = (T + 8 * NT - 1) / (8 * NT);
        w_row0 = e * N + n0;
        splits = 1;
        split = 0;
    }
    const int sb0 = (int)((long long)nSB * split / splits), sb1 = (int)((long long)nSB * (split + 1) / splits);
    const int n_sb = sb1 - sb0, nG = nSB * 8;
    if (tid == 0) {
        for (int s = 0; s < kSStages; s++) {
            mbar_init(smem_u32(&full[s]), 1);             // the producer's announcement (+ the box's bytes)
            mbar_init(smem_u32(&empty[s]), kSConsumers);  // every consumer warp holds the stage's bytes in registers
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    volatile int* abort_v = &abort_s;

    if (warp == kSConsumers) {
        // ---- producer: one thread; per super-block five tiled copies on the stage's barrier: the 64 rows' raw weights, the
        // activation rows' codes (two 128-byte halves, swizzled), their scales and their group sums. Rows past T read as
        // zeros (they feed accumulators that are never stored). ----
        if (lane == 0) {
            constexpr unsigned tx = (unsigned)(kSWBytes + 8 * NT * (256 + 64));
            int issued = 0;
            for (int i = 0; i < n_pass * n_sb; i++) {
                const int st = i % kSStages, b = sb0 + i % n_sb, t_row = t_base + (i / n_sb) * 8 * NT;
                if (i >= kSStages && !mbar_wait(smem_u32(&empty[st]), (unsigned)(((i - kSStages) / kSStages) & 1), abort_v)) {
                    abort_s = 1;
                    break;
                }
                const unsigned bar = smem_u32(&full[st]), base = smem_u32(s_ring) + (unsigned)st * kSStageBytes;
                mbar_arrive_expect_tx(bar, tx);
                tensor_g2s_2d(base, &wmap, b * 144, w_row0, bar);
                tensor_g2s_2d(base + kSWBytes, &cmap, 256 * b, t_row, bar);
                tensor_g2s_2d(base + kSWBytes + 8 * NT * 128, &cmap, 256 * b + 128, t_row, bar);
                tensor_g2s_2d(base + kSWBytes + 8 * NT * 256, &smap, 8 * b, t_row, bar);
                tensor_g2s_2d(base + kSWBytes + 8 * NT * 288, &smap, nG + 8 * b, t_row, bar);
                issued = i + 1;
            }
            // copies still in flight must land before the CTA may leave: bounded waits on their barriers
            if (abort_s)
                for (int i = max(0, issued - kSStages); i < issued; i++) mbar_wait(smem_u32(&full[i % kSStages]), (unsigned)((i / kSStages) & 1));
        }
        return;
    }

    // ---- consumers: warp w owns rows n0 + 16w .. +15; lane rows gid and gid + 8 ----
    float acc[NT][4];
    const unsigned row_off = (unsigned)(16 * warp + gid) * 144u;
    bool ok = true;
    const int na = n0 + 16 * warp + gid, nb = na + 8;
    for (int pass = 0; pass < n_pass && ok; pass++) {
    const int Tp = T - pass * 8 * NT;  // rows from this pass on (the pass itself takes 8*NT of them)
#pragma unroll
    for (int j = 0; j < NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int i = pass * n_sb; i < (pass + 1) * n_sb; i++) {
        const int st = i % kSStages;
        const bool there = mbar_wait(smem_u32(&full[st]), (unsigned)((i / kSStages) & 1), abort_v);
        if (!__all_sync(0xffffffffu, there)) {
            ok = false;
            break;
        }
        const uint8_t* w0 = s_ring + (size_t)st * kSStageBytes + row_off;
        const uint8_t* w1 = w0 + 8 * 144;
        const uint4 h0 = *reinterpret_cast<const uint4*>(w0);
        const uint4 h1 = *reinterpret_cast<const uint4*>(w1);
        uint2 q0[4], q1[4];
#pragma unroll
        for (int p = 0; p < 4; p++) {
            q0[p] = *reinterpret_cast<const uint2*>(w0 + 16 + 32 * p + 8 * tig);
            q1[p] = *reinterpret_cast<const uint2*>(w1 + 16 + 32 * p + 8 * tig);
        }
        const uint8_t* act = s_ring + (size_t)st * kSStageBytes + kSWBytes;       // codes: two swizzled [8*NT rows][128 B] halves
        const uint8_t* asc = act + 8 * NT * 256;                                  // [8*NT rows][8] scales, then [8*NT rows][8] group sums
        // this lane decodes sub-blocks 2*tig and 2*tig+1 of its two rows; the quad shares them by shuffle
        float my_ds[2][2], my_nm[2][2];
        {
            int s, m;
            const float d0 = s_h2f((unsigned short)(h0.x & 0xffffu)), dm0 = s_h2f((unsigned short)(h0.x >> 16));
            const float d1 = s_h2f((unsigned short)(h1.x & 0xffffu)), dm1 = s_h2f((unsigned short)(h1.x >> 16));
            s_scale_min(2 * tig, h0.y, h0.z, h0.w, &s, &m);
            my_ds[0][0] = __fmul_rn(d0, (float)s); my_nm[0][0] = -__fmul_rn(dm0, (float)m);
            s_scale_min(2 * tig + 1, h0.y, h0.z, h0.w, &s, &m);
            my_ds[0][1] = __fmul_rn(d0, (float)s); my_nm[0][1] = -__fmul_rn(dm0, (float)m);
            s_scale_min(2 * tig, h1.y, h1.z, h1.w, &s, &m);
            my_ds[1][0] = __fmul_rn(d1, (float)s); my_nm[1][0] = -__fmul_rn(dm1, (float)m);
            s_scale_min(2 * tig + 1, h1.y, h1.z, h1.w, &s, &m);
            my_ds[1][1] = __fmul_rn(d1, (float)s); my_nm[1][1] = -__fmul_rn(dm1, (float)m);
        }
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int src = (lane & ~3) | p;
            const float ds0lo = __shfl_sync(0xffffffffu, my_ds[0][0], src), ds0hi = __shfl_sync(0xffffffffu, my_ds[0][1], src);
            const float ds1lo = __shfl_sync(0xffffffffu, my_ds[1][0], src), ds1hi = __shfl_sync(0xffffffffu, my_ds[1][1], src);
            const float nm0lo = __shfl_sync(0xffffffffu, my_nm[0][0], src), nm0hi = __shfl_sync(0xffffffffu, my_nm[0][1], src);
            const float nm1lo = __shfl_sync(0xffffffffu, my_nm[1][0], src), nm1hi = __shfl_sync(0xffffffffu, my_nm[1][1], src);
            // code words 2*tig, 2*tig+1 of the pair: low nibbles = sub-block 2p, high = 2p+1
            const unsigned al0 = q0[p].x & 0x0F0F0F0Fu, al1 = q1[p].x & 0x0F0F0F0Fu, al2 = q0[p].y & 0x0F0F0F0Fu, al3 = q1[p].y & 0x0F0F0F0Fu;
            const unsigned ah0 = (q0[p].x >> 4) & 0x0F0F0F0Fu, ah1 = (q1[p].x >> 4) & 0x0F0F0F0Fu, ah2 = (q0[p].y >> 4) & 0x0F0F0F0Fu,
                           ah3 = (q1[p].y >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                if (8 * j >= Tp) continue;  // a token tile with no rows (uniform over the CTA)
                // bytes 64p + 8tig .. (+32 for the pair's second sub-block) of row 8j + gid: half p >> 1, 16-byte chunk
                // ((64p + 8tig) & 127) >> 4 stored at chunk ^ (row & 7)
                const uint8_t* hb = act + (p >> 1) * (8 * NT * 128) + (8 * j + gid) * 128 + ((8 * tig) & 15);
                const int c_lo = ((64 * (p & 1) + 8 * tig) >> 4), c_hi = c_lo + 2;
                const int2 blo = *reinterpret_cast<const int2*>(hb + ((c_lo ^ gid) << 4));
                const int2 bhi = *reinterpret_cast<const int2*>(hb + ((c_hi ^ gid) << 4));
                int cl[4], ch[4];
                s_mma(cl, al0, al1, al2, al3, (unsigned)blo.x, (unsigned)blo.y);
                s_mma(ch, ah0, ah1, ah2, ah3, (unsigned)bhi.x, (unsigned)bhi.y);
                const uint8_t* s0 = asc + (8 * j + 2 * tig) * 32 + 8 * p;              // row 2*tig: scales of groups 2p, 2p+1
                const uint8_t* s1 = s0 + 32;                                           // row 2*tig+1
                const float2 aS0 = *reinterpret_cast<const float2*>(s0), aS1 = *reinterpret_cast<const float2*>(s1);
                const float2 as0 = *reinterpret_cast<const float2*>(s0 + 8 * NT * 32), as1 = *reinterpret_cast<const float2*>(s1 + 8 * NT * 32);  // group sums
                float f;
                f = acc[j][0];  // (weight row gid, activation row 2*tig)
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[0]), S_MAGIC_F), __fmul_rn(ds0lo, aS0.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[0]), S_MAGIC_F), __fmul_rn(ds0hi, aS0.y), f);
                f = __fmaf_rn(nm0lo, as0.x, f);
                acc[j][0] = __fmaf_rn(nm0hi, as0.y, f);
                f = acc[j][1];  // (gid, 2*tig+1)
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[1]), S_MAGIC_F), __fmul_rn(ds0lo, aS1.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[1]), S_MAGIC_F), __fmul_rn(ds0hi, aS1.y), f);
                f = __fmaf_rn(nm0lo, as1.x, f);
                acc[j][1] = __fmaf_rn(nm0hi, as1.y, f);
                f = acc[j][2];  // (gid+8, 2*tig)
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[2]), S_MAGIC_F), __fmul_rn(ds1lo, aS0.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[2]), S_MAGIC_F), __fmul_rn(ds1hi, aS0.y), f);
                f = __fmaf_rn(nm1lo, as0.x, f);
                acc[j][2] = __fmaf_rn(nm1hi, as0.y, f);
                f = acc[j][3];  // (gid+8, 2*tig+1)
                f = __fmaf_rn(__fsub_rn(__int_as_float(cl[3]), S_MAGIC_F), __fmul_rn(ds1lo, aS1.x), f);
                f = __fmaf_rn(__fsub_rn(__int_as_float(ch[3]), S_MAGIC_F), __fmul_rn(ds1hi, aS1.y), f);
                f = __fmaf_rn(nm1lo, as1.x, f);
                acc[j][3] = __fmaf_rn(nm1hi, as1.y, f);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the stage's reads precede the refill's writes
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[st]));
    }
    if (!ok) break;
    float* out = dst + (size_t)split * split_stride + (size_t)(t_base + pass * 8 * NT) * ldd;
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int t0 = 8 * j + 2 * tig, t1 = t0 + 1;
        if (t0 < Tp) {
            if (na < N) out[(size_t)t0 * ldd + na] = acc[j][0];
            if (nb < N) out[(size_t)t0 * ldd + nb] = acc[j][2];
        }
        if (t1 < Tp) {
            if (na < N) out[(size_t)t1 * ldd + na] = acc[j][1];
            if (nb < N) out[(size_t)t1 * ldd + nb] = acc[j][3];
        }
    }
    }
    if (!ok) {
        abort_s = 1;
        if (lane == 0 && err_flag) atomicExch(err_flag, 1);
    }
}

// dst[t][n] = sum over splits, in split order
__global__ void stream_reduce_kernel(const float* __restrict__ part, size_t split_stride, int splits, int T, int N,
                                     float* __restrict__ dst, int ldd) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * N) return;
    const int t = (int)(i / N), n = (int)(i % N);
    float s = part[i];
    for (int k = 1; k < splits; k++) s = __fadd_rn(s, part[(size_t)k * split_stride + i]);
    dst[(size_t)t * ldd + n] = s;
}

// Cached 2-D tensor maps of the activation buffers: codes [T][K] bytes with a box of 128 x box_rows and the 128-byte
// swizzle; scales [T][2*nG] floats with a box of 8 x box_rows. A map depends only on its key.
const CUtensorMap* act_map(b200_ctx* ctx, const void* ptr, int inner, int T, int box_rows, bool is_codes) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, bool>, CUtensorMap*> cache;
    std::lock_guard<std::mutex> lock(mu);
    const tensor_map_encode_fn encode = tensor_map_encoder();
    if (!encode) {
        ctx->err = "cuTensorMapEncodeTiled is not available from this driver";
        return nullptr;
    }
    const auto key = std::make_tuple(ptr, inner, T, box_rows, is_codes);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    CUtensorMap* m = new CUtensorMap;
    const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)T};
    const cuuint64_t strides[1] = {(cuuint64_t)inner * (is_codes ? 1 : 4)};
    const cuuint32_t box[2] = {is_codes ? 128u : 8u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(m, is_codes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims,
                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, is_codes ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        delete m;
        ctx->err = "cuTensorMapEncodeTiled failed with " + std::to_string((int)r) + " (activation buffer, inner " + std::to_string(inner) + ", rows " + std::to_string(T) + ")";
        return nullptr;
    }
    cache[key] = m;
    return m;
}

template <int NT>
int run_stream(b200_ctx* ctx, const CUtensorMap* wmap, int N, int nSB, ActQ aq, int T, float* dst, int ldd, int splits, float* part) {
    constexpr int smem = stream_stages(NT) * stream_stage_bytes(NT) + 1024;
    const CUtensorMap* cmap = act_map(ctx, aq.codes, nSB * 256, T, 8 * NT, true);
    const CUtensorMap* smap = act_map(ctx, aq.scales, nSB * 16, T, 8 * NT, false);
    if (!cmap || !smap) return B200_CUDA_ERROR;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_stream_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    dim3 grid(ceil_div(N, kSRows), splits);
    float* out = splits > 1 ? part : dst;
    {
        ProfScope ps(ctx, PROF_Q4K_GEMM);
        launch_pdl(q4k_stream_kernel<NT>, grid, dim3(kSThreads), smem, ctx->stream, *wmap, *cmap, *smap, N, nSB, T, out, splits > 1 ? N : ldd,
                   splits > 1 ? (size_t)T * N : (size_t)0, ctx->err_flag, (const int32_t*)nullptr);
    }
    LAUNCH_CHECK(ctx);
    if (splits > 1) {
        launch_pdl(stream_reduce_kernel, dim3((unsigned)(((size_t)T * N + 255) / 256)), dim3(256), 0, ctx->stream, part, (size_t)T * N, splits, T, N, dst, ldd);
        LAUNCH_CHECK(ctx);
    }
    return B200_OK;
}

// sorted[s] = row rows_tok[s] of the activation buffers: codes [.][K] and scales [.][2*nG]
__global__ void gather_act_rows_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales, const int32_t* __restrict__ rows_tok,
                                       int K, int8_t* __restrict__ codes_out, float* __restrict__ scales_out) {
    const int s = blockIdx.x, r = rows_tok[s], nS = K / 16;  // K/32 scales + K/32 sums
    const uint4* src = reinterpret_cast<const uint4*>(codes + (size_t)r * K);
    uint4* dstc = reinterpret_cast<uint4*>(codes_out + (size_t)s * K);
    for (int i = threadIdx.x; i < K / 16; i += blockDim.x) dstc[i] = src[i];
    for (int i = threadIdx.x; i < nS; i += blockDim.x) scales_out[(size_t)s * nS + i] = scales[(size_t)r * nS + i];
}

}  // namespace

int launch_gather_act_rows(b200_ctx* ctx, ActQ src, const int32_t* rows_tok, int n_rows, int K, ActQ dst) {
    if (n_rows <= 0) return B200_OK;
    gather_act_rows_kernel<<<n_rows, 128, 0, ctx->stream>>>(src.codes, src.scales, rows_tok, K, dst.codes, dst.scales);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

bool q4k_stream_grouped_supported(const uint8_t* W_all, int N, int K) { return N % kSRows == 0 && K % 256 == 0 && (reinterpret_cast<uintptr_t>(W_all) & 15) == 0; }

// Experts' matrices stacked in one buffer ([n_experts * N][K] Q4_K); aq holds the activation rows in expert-sorted order
// (rows offs[e] .. offs[e+1] belong to expert e, n_rows in all); dst rows are the sorted slots.
int launch_q4k_matmul_stream_grouped(b200_ctx* ctx, const uint8_t* W_all, int n_experts, int N, int K, ActQ aq, const int32_t* offs,
                                     int n_rows, int max_rows_per_expert, float* dst, int ldd) {
    if (!q4k_stream_grouped_supported(W_all, N, K)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "grouped streaming matmul: N %% 64, K %% 256 or alignment");
    if (n_rows <= 0) return B200_OK;
    constexpr int NT = 2;
    const int nSB = K / 256;
    const CUtensorMap* wmap = q4k_weight_map(ctx, W_all, n_experts * N, nSB, kSRows);
    const CUtensorMap* cmap = act_map(ctx, aq.codes, K, n_rows, 8 * NT, true);
    const CUtensorMap* smap = act_map(ctx, aq.scales, nSB * 16, n_rows, 8 * NT, false);
    if (!wmap || !cmap || !smap) return B200_CUDA_ERROR;
    constexpr int smem = stream_stages(NT) * stream_stage_bytes(NT) + 1024;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(q4k_stream_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    (void)max_rows_per_expert;
    dim3 grid(N / kSRows, n_experts);
    {
        ProfScope ps(ctx, PROF_Q4K_GEMM);
        launch_pdl(q4k_stream_kernel<NT>, grid, dim3(kSThreads), smem, ctx->stream, *wmap, *cmap, *smap, N, nSB, 0, dst, ldd, (size_t)0, ctx->err_flag, offs);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_q4k_matmul_stream(b200_ctx* ctx, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, bool allow_split) {
    if (K % 256 || T < 1 || T > 64) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the streaming Q4_K matmul takes 1..64 rows and K %% 256 == 0");
    if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(aq.codes) | reinterpret_cast<uintptr_t>(aq.scales)) & 15)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "the streaming Q4_K matmul wants 16-byte aligned weights and activation buffers");
    const int nSB = K / 256, tiles = ceil_div(N, kSRows);
    // split K (whole super-blocks, at least four per range) only while the CTAs do not fill three slots per SM
    int splits = 1;
    if (allow_split && ctx->umma_scratch) {
        splits = std::max(1, std::min(std::min(4, nSB / 4), 3 * ctx->sm_count / tiles));
        while (splits > 1 && (size_t)splits * T * N * 4 > ctx->umma_scratch_bytes) splits--;
    }
    const CUtensorMap* wmap = q4k_weight_map(ctx, W, N, nSB, kSRows);
    if (!wmap) return B200_CUDA_ERROR;
    float* part = reinterpret_cast<float*>(ctx->umma_scratch);
    if (T <= 8) return run_stream<1>(ctx, wmap, N, nSB, aq, T, dst, ldd, splits, part);
    if (T <= 16) return run_stream<2>(ctx, wmap, N, nSB, aq, T, dst, ldd, splits, part);
    if (T <= 32) return run_stream<4>(ctx, wmap, N, nSB, aq, T, dst, ldd, splits, part);
    return run_stream<8>(ctx, wmap, N, nSB, aq, T, dst, ldd, splits, part);
}

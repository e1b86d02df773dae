// gemm_f16_umma.cu — fast-class matmul over f16 weights (the LM head: logits = h W^T, decoder/forwardn.go:800-831) for
// dense row counts: tcgen05 tensor cores, TMEM accumulators, both operands brought in by the copy engine.
//
//   dst[t][n] = sum_k x[t][k] * W[n][k],   W f16 [N][K] row-major (K-major, what the MMA wants),  x f32 [T][K]
//
// The f32 activations are split into f16 hi + lo parts (x = hi + lo up to 2^-22 relative), so the product keeps
// fp32-level accuracy over the f16 weights: per chunk of 64 along K the accumulator takes hi x W and lo x W.
// One CTA owns a [128 rows] x [256 weight rows] tile (an accumulator of 256 fp32 columns x 128 lanes of tensor memory).
// Ring of 3 stages, each: A hi and A lo tiles (16 KB each, one contiguous bulk copy each from a tile-major,
// pre-swizzled copy of the split activations) + the weight tile (256 rows x 64, one tiled TMA copy with the 128-byte
// swizzle; rows past N read as zeros). Warp 8's elected thread loads, warp 9's issues the MMAs and commits each stage
// back to the loader; warps 0-7 only run the epilogue (tcgen05.ld, turn the 32x32 blocks around in shared memory, write
// whole rows). Token tiles of the same weight tile are neighbours in the grid, so the second one finds the weights in L2.
// Every mbarrier wait is bounded: on expiry the CTA raises an error flag, frees its TMEM and returns.
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "umma.cuh"

namespace {

constexpr int kHStages = 3;
constexpr int kHStageBytes = 2 * kTileBytes + 2 * kTileBytes;  // A hi, A lo, B (256 rows = two tiles)
constexpr int kHThreads = 10 * 32;

// Test hook for the bounded waits (b200_debug_wait_fault): [0] = how many polls the MMA issuer gives a stage to fill
// (0: the default), [1] = the K chunk from which the loader stops bringing stages in (-1: never). With a chunk withheld
// the issuer's wait runs out, the CTA raises the error flag, waits for the copies it did start, frees its tensor memory
// and returns; nothing spins without a limit.
__device__ int g_wait_fault[2] = {0, -1};

__global__ void __launch_bounds__(kHThreads, 1) f16w_umma_gemm_kernel(const __grid_constant__ CUtensorMap wmap, int N, int K,
                                                                      const __half* __restrict__ xhi, const __half* __restrict__ xlo,
                                                                      int T, float* __restrict__ dst, int ldd,
                                                                      int* __restrict__ err_flag) {
    pdl_trigger();
    extern __shared__ __align__(1024) uint8_t h_smem[];
    __shared__ __align__(8) uint64_t full_bar[kHStages], empty_bar[kHStages];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = blockIdx.x * 128, n0 = blockIdx.y * 256;
    const int n_it = K / 64;
    uint8_t* smem = h_smem + ((1024u - (smem_u32(h_smem) & 1023u)) & 1023u);

    if (tid == 0) {
        for (int s = 0; s < kHStages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);   // the loader's announcement (+ the three copies' bytes)
            mbar_init(smem_u32(&empty_bar[s]), 1);  // one tcgen05.commit
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    volatile int* abort_v = &abort_s;
    pdl_wait();  // set up while the kernel before this one drained; its outputs are complete from here

    if (warp == 8 && lane == 0) {
        // ---- loader ----
        const size_t a_off = (size_t)blockIdx.x * (size_t)n_it * kTileBytes;  // tile-major: [token tile][chunk][128 rows][64]
        const uint8_t* ahi = reinterpret_cast<const uint8_t*>(xhi) + a_off;
        const uint8_t* alo = reinterpret_cast<const uint8_t*>(xlo) + a_off;
        int issued = 0;
        const int withhold_from = g_wait_fault[1];
        for (int it = 0; it < n_it; it++) {
            if (it == withhold_from) break;  // test hook: the stages from here on never fill
            if (it >= kHStages && !mbar_wait(smem_u32(&empty_bar[it % kHStages]), (unsigned)(((it - kHStages) / kHStages) & 1), abort_v)) {
                abort_s = 1;
                break;
            }
            const unsigned bar = smem_u32(&full_bar[it % kHStages]), st = smem_u32(smem + (size_t)(it % kHStages) * kHStageBytes);
            mbar_arrive_expect_tx(bar, (unsigned)kHStageBytes);
            bulk_g2s(st, ahi + (size_t)it * kTileBytes, kTileBytes, bar);
            bulk_g2s(st + kTileBytes, alo + (size_t)it * kTileBytes, kTileBytes, bar);
            tensor_g2s_2d(st + 2 * kTileBytes, &wmap, it * 64, n0, bar);
            issued = it + 1;
        }
        if (abort_s)  // copies still in flight must land before the CTA may leave: bounded waits on their barriers
            for (int it = max(0, issued - kHStages); it < issued; it++) mbar_wait(smem_u32(&full_bar[it % kHStages]), (unsigned)((it / kHStages) & 1));
    } else if (warp == 9 && lane == 0) {
        // ---- MMA issuer ----
        const int polls = g_wait_fault[0] > 0 ? g_wait_fault[0] : kWaitPolls;
        for (int it = 0; it < n_it; it++) {
            if (!mbar_wait(smem_u32(&full_bar[it % kHStages]), (unsigned)((it / kHStages) & 1), abort_v, polls)) {
                abort_s = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned a0 = smem_u32(smem + (size_t)(it % kHStages) * kHStageBytes), b0 = a0 + 2 * kTileBytes;
#pragma unroll
            for (int part = 0; part < 2; part++)
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    umma_f16(tmem_base, umma_desc(a0 + part * kTileBytes + ks * 32), umma_desc(b0 + ks * 32), idesc_for(256),
                             (it > 0 || part > 0 || ks > 0) ? 1u : 0u);
            umma_commit(smem_u32(&empty_bar[it % kHStages]));
        }
        if (n_it > 0 && !*abort_v) {
            const int last = n_it - 1;
            if (!mbar_wait(smem_u32(&empty_bar[last % kHStages]), (unsigned)((last / kHStages) & 1), abort_v)) abort_s = 1;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (abort_s) {
        if (tid == 0 && err_flag) atomicExch(err_flag, 1);
    } else if (n_it > 0 && warp < 8) {
        // warp w reads TMEM lanes 32*(w%4).. (rows t0 + 32*(w%4) + lane), columns 128*(w/4) .. +127
        const int lq = warp & 3, ch = warp >> 2;
        const int tbase = t0 + lq * 32;
        uint8_t* tp = smem + warp * (32 * 144);
#pragma unroll 1
        for (int cb = 4 * ch; cb < 4 * ch + 4; cb++) {
            unsigned r[32];
            const unsigned taddr = tmem_base + ((unsigned)(lq * 32) << 16) + (unsigned)(cb * 32);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                  "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
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
                    float* o = dst + (size_t)tt * ldd + nc;
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
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256));
}

// x f32 [T][K] -> hi and lo f16 parts, each stored as the MMA's shared-memory tiles: [token tile of 128][chunk of 64
// along K][128 rows][64], the 16-byte chunk c of a row at position c ^ (t & 7). Rows past T are written as zeros.
__global__ void split_to_tiles_kernel(const float* __restrict__ x, int T, int K, __half* __restrict__ hi, __half* __restrict__ lo) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int k8 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (k8 >= K) return;
    uint4 oh = make_uint4(0, 0, 0, 0), ol = make_uint4(0, 0, 0, 0);
    if (t < T) {
        const float4 a = *reinterpret_cast<const float4*>(x + (size_t)t * K + k8);
        const float4 b = *reinterpret_cast<const float4*>(x + (size_t)t * K + k8 + 4);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        unsigned* ph = &oh.x;
        unsigned* pl = &ol.x;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            const float2 hf = __half22float2(h);
            const __half2 l = __floats2half2_rn(v[2 * i] - hf.x, v[2 * i + 1] - hf.y);
            ph[i] = *reinterpret_cast<const unsigned*>(&h);
            pl[i] = *reinterpret_cast<const unsigned*>(&l);
        }
    }
    const int seg = k8 >> 6, chunk = (k8 >> 3) & 7;
    const size_t off = ((size_t)(t >> 7) * (size_t)(K >> 6) + seg) * (128 * 64) + (size_t)(t & 127) * 64 + ((chunk ^ (t & 7)) << 3);
    *reinterpret_cast<uint4*>(hi + off) = oh;
    *reinterpret_cast<uint4*>(lo + off) = ol;
}

// The tensor map of an f16 weight matrix [N][K] with a box of 64 x 256 and the 128-byte swizzle. A map depends only on
// its key, so the cache never goes stale.
const CUtensorMap* f16_weight_map(b200_ctx* ctx, const __half* W, int N, int K) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int>, CUtensorMap*> cache;
    std::lock_guard<std::mutex> lock(mu);
    const tensor_map_encode_fn encode = tensor_map_encoder();
    if (!encode) {
        ctx->err = "cuTensorMapEncodeTiled is not available from this driver";
        return nullptr;
    }
    const auto key = std::make_tuple((const void*)W, N, K);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    CUtensorMap* m = new CUtensorMap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {64, 256};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(W), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        delete m;
        ctx->err = "cuTensorMapEncodeTiled failed with " + std::to_string((int)r) + " (f16 weights N=" + std::to_string(N) + ", K=" + std::to_string(K) + ")";
        return nullptr;
    }
    cache[key] = m;
    return m;
}

}  // namespace

size_t f16w_umma_scratch_bytes(int T, int K) { return (size_t)2 * ceil_div(T, 128) * 128 * K * 2 + 256; }

bool f16w_umma_supported(const __half* W, int N, int K) { return K % 64 == 0 && N >= 256 && (reinterpret_cast<uintptr_t>(W) & 15) == 0; }

int launch_f16w_matmul_umma(b200_ctx* ctx, const __half* W, int N, int K, const float* x, int T, float* dst, int ldd, void* scratch,
                            size_t scratch_bytes, int* err_flag) {
    if (!f16w_umma_supported(W, N, K)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "f16 tcgen05 matmul needs K %% 64 == 0, N >= 256 and 16-byte aligned weights");
    if (f16w_umma_scratch_bytes(T, K) > scratch_bytes) B200_FAIL(ctx, B200_BAD_ARGUMENT, "f16 tcgen05 matmul scratch too small");
    const int t_tiles = ceil_div(T, 128);
    __half* hi = reinterpret_cast<__half*>(scratch);
    __half* lo = hi + (size_t)t_tiles * 128 * K;
    {
        dim3 grid(ceil_div(K / 8, 256), t_tiles * 128);
        launch_pdl(split_to_tiles_kernel, grid, dim3(256), 0, ctx->stream, x, T, K, hi, lo);
        LAUNCH_CHECK(ctx);
    }
    constexpr int smem = kHStages * kHStageBytes + 1024;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(f16w_umma_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    const CUtensorMap* wmap = f16_weight_map(ctx, W, N, K);
    if (!wmap) return B200_CUDA_ERROR;
    dim3 grid(t_tiles, ceil_div(N, 256));
    {
        ProfScope ps(ctx, PROF_HEAD_GEMM);
        launch_pdl(f16w_umma_gemm_kernel, grid, dim3(kHThreads), smem, ctx->stream, *wmap, N, K, hi, lo, T, dst, ldd, err_flag);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

// Test hook: arms (or, with polls = 0 and withhold_chunk = -1, disarms) the wait fault of the f16 tcgen05 matmul on the
// context's device. Armed, the loader of every CTA stops bringing stages in at K chunk `withhold_chunk` and the MMA
// issuer gives a stage `polls` polls to fill, so the issuer's bounded wait runs out: the kernel raises the error flag and
// returns, and the entry point that launched it reports B200_TIMEOUT. Nothing faults and nothing waits without a limit.
extern "C" int b200_debug_wait_fault(b200_ctx* ctx, int polls, int withhold_chunk) {
    if (!ctx || polls < 0) return B200_BAD_ARGUMENT;
    const int v[2] = {polls, withhold_chunk};
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyToSymbol(g_wait_fault, v, sizeof v));
    return B200_OK;
}

// ops.cu — operator-level C entry points (host buffers in and out) and device-resident micro-benchmarks.
// They run the same kernels the step uses, the way the reference tests its kernels against host twins
// (backend/cuda/kernels/actgroup_kernel_test.go, moe_route_test.go, gemv_bw_test.go).
#include <algorithm>
#include <cmath>
#include <vector>

#include "common.cuh"

namespace {

struct Tmp {  // device allocations freed at scope exit
    std::vector<void*> ps;
    ~Tmp() {
        for (void* p : ps) cudaFree(p);
    }
    template <typename T>
    cudaError_t get(T** p, size_t n) {
        cudaError_t e = cudaMalloc((void**)p, std::max<size_t>(n * sizeof(T), 16));
        if (e == cudaSuccess) ps.push_back(*p);
        return e;
    }
};

// Lends the context a tcgen05-matmul scratch for the length of an operator call (a model owns its own).
struct UmmaScratch {
    b200_ctx* ctx;
    void* saved_p;
    size_t saved_n;
    int* saved_f;
    size_t saved_slot;
    explicit UmmaScratch(b200_ctx* c) : ctx(c), saved_p(c->umma_scratch), saved_n(c->umma_scratch_bytes), saved_f(c->err_flag), saved_slot(c->x16_slot_bytes) {
        c->x16_slot_bytes = 0;  // operator entry points use the plain layout: activations, then partials
        c->x16_ready = nullptr;
    }
    int ensure(Tmp& t, int M, int K, int N) { return ensure_bytes(t, std::max(q4k_umma_scratch_bytes(M, K, N), f16w_umma_scratch_bytes(M, K))); }
    int ensure_bytes(Tmp& t, size_t need) {
        if (ctx->umma_scratch && ctx->umma_scratch_bytes >= need && ctx->err_flag) return B200_OK;
        uint8_t* p;
        int* f;
        CUDA_TRY(ctx, t.get(&p, need));
        CUDA_TRY(ctx, t.get(&f, 1));
        CUDA_TRY(ctx, cudaMemsetAsync(f, 0, 4, ctx->stream));
        ctx->umma_scratch = p;
        ctx->umma_scratch_bytes = need;
        ctx->err_flag = f;
        return B200_OK;
    }
    int check() {  // after a stream synchronize
        int flag = 0;
        if (ctx->err_flag) cudaMemcpy(&flag, ctx->err_flag, 4, cudaMemcpyDeviceToHost);
        if (flag) B200_FAIL(ctx, B200_TIMEOUT, "a bounded device-side wait in the tcgen05 matmul gave up");
        return B200_OK;
    }
    ~UmmaScratch() {
        ctx->umma_scratch = saved_p;
        ctx->umma_scratch_bytes = saved_n;
        ctx->err_flag = saved_f;
        ctx->x16_slot_bytes = saved_slot;
    }
};

#define TMP_GET(ctx, tmp, ptr, n) CUDA_TRY(ctx, (tmp).get(&(ptr), (n)))
#define H2D(ctx, dst, src, bytes) CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (ctx)->stream))
#define D2H(ctx, dst, src, bytes) CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (ctx)->stream))
#define SYNC(ctx) CUDA_TRY(ctx, cudaStreamSynchronize((ctx)->stream))

__global__ void fill_i32_kernel(int32_t* p, size_t n, int32_t v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
__global__ void iota_blocks_kernel(int32_t* table, int rows, int max_blocks, const int32_t* n_keys, int block_rows) {
    // row r owns blocks 1 + r*max_blocks + b (contiguous identity mapping)
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * max_blocks) return;
    int r = i / max_blocks, b = i % max_blocks;
    table[i] = (b * block_rows < n_keys[r]) ? 1 + r * max_blocks + b : 0;
}
__global__ void scatter_kv_kernel(const float* k, const float* v, __half* kpool, __half* vpool, const int32_t* table, int rows,
                                  int max_keys, int max_blocks, int nKV, int hd, int block_rows, const int32_t* n_keys) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t per_row = (size_t)max_keys * nKV * hd;
    if (i >= (size_t)rows * per_row) return;
    int r = (int)(i / per_row);
    size_t j = i % per_row;
    int e = (int)(j % hd), kvh = (int)((j / hd) % nKV), key = (int)(j / ((size_t)hd * nKV));
    if (key >= n_keys[r]) return;
    int blk = table[(size_t)r * max_blocks + key / block_rows];
    size_t off = (((size_t)blk * nKV + kvh) * block_rows + key % block_rows) * hd + e;
    kpool[off] = __float2half_rn(k[i]);
    vpool[off] = __float2half_rn(v[i]);
}
__global__ void ctx_minus1_kernel(const int32_t* n_keys, int32_t* row_pos, int32_t* row_slot, int rows) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) { row_pos[i] = n_keys[i] - 1; row_slot[i] = i; }
}

}  // namespace

extern "C" {

int b200_op_quant_g32(b200_ctx* ctx, const float* x, int rows, int k, int8_t* codes, float* scales) {
    Tmp t;
    float* dx; ActQ aq;
    const size_t n = (size_t)rows * k, ns = (size_t)rows * 2 * (k / 32);
    TMP_GET(ctx, t, dx, n); TMP_GET(ctx, t, aq.codes, n); TMP_GET(ctx, t, aq.scales, ns);
    H2D(ctx, dx, x, n * 4);
    ST_TRY(launch_quant_g32(ctx, dx, rows, k, aq));
    D2H(ctx, codes, aq.codes, n); D2H(ctx, scales, aq.scales, ns * 4);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_q4k_dequant(b200_ctx* ctx, const uint8_t* w, int rows, int cols, float* out) {
    if (cols % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "cols %% 256");
    Tmp t;
    const size_t nb = (size_t)rows * cols / 256;
    uint8_t* dw; float* dout;
    TMP_GET(ctx, t, dw, nb * 144); TMP_GET(ctx, t, dout, nb * 256);
    H2D(ctx, dw, w, nb * 144);
    ST_TRY(launch_q4k_dequant(ctx, dw, nb, dout));
    D2H(ctx, out, dout, nb * 256 * 4);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_q4k_matmul(b200_ctx* ctx, const uint8_t* w, const float* a, int M, int K, int N, int klass, float* dst) {
    if (K % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K %% 256");
    const bool tiles_only = klass == 7;  // the fast class as a model runs it: only the tile-major copy is given to the kernels
    if (tiles_only) klass = 0;
    Tmp t;
    const size_t wb = (size_t)N * K / 256 * 144;
    uint8_t* dw; float *da, *dd; ActQ aq;
    TMP_GET(ctx, t, dw, wb); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, aq.codes, (size_t)M * K); TMP_GET(ctx, t, aq.scales, (size_t)M * 2 * (K / 32));
    H2D(ctx, dw, w, wb); H2D(ctx, da, a, (size_t)M * K * 4);
    ST_TRY(launch_quant_g32(ctx, da, M, K, aq));
    UmmaScratch us(ctx);
    ST_TRY(us.ensure(t, M, K, N));
    uint8_t* dtiles = nullptr;   // the tile-by-tile copy a model keeps for the small-batch kernel
    if (tiles_only || ((klass == 0 || klass == 2 || klass == 5) && M <= 32)) {
        TMP_GET(ctx, t, dtiles, q4k_tiles_bytes(N, K));
        ST_TRY(launch_q4k_to_tiles(ctx, dw, N, K, dtiles));
    }
    ST_TRY(launch_q4k_matmul(ctx, tiles_only ? nullptr : dw, N, K, aq, M, dd, N, klass, dtiles));
    D2H(ctx, dst, dd, (size_t)M * N * 4);
    SYNC(ctx);
    return us.check();
}

int b200_op_gate_up_swiglu(b200_ctx* ctx, const uint8_t* w, const float* a, int M, int K, int F, int mode, int8_t* codes_out,
                           float* scales_out) {
    if (K % 256 || F % 128 || M <= 0 || mode < 0 || mode > 2) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K %% 256, F %% 128, mode 0..2");
    Tmp t;
    const size_t rb = (size_t)K / 256 * 144, wb = (size_t)2 * F * rb;
    uint8_t *dw, *dil; float *da, *dgu; ActQ aq, mid;
    TMP_GET(ctx, t, dw, wb); TMP_GET(ctx, t, dil, wb); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dgu, (size_t)M * 2 * F);
    TMP_GET(ctx, t, aq.codes, (size_t)M * K); TMP_GET(ctx, t, aq.scales, (size_t)M * 2 * (K / 32));
    TMP_GET(ctx, t, mid.codes, (size_t)M * F); TMP_GET(ctx, t, mid.scales, (size_t)M * 2 * (F / 32));
    H2D(ctx, dw, w, wb); H2D(ctx, da, a, (size_t)M * K * 4);
    ST_TRY(launch_quant_g32(ctx, da, M, K, aq));
    UmmaScratch us(ctx);
    ST_TRY(us.ensure(t, M, K, 2 * F));
    bool fused = false;
    if (mode == 0) {
        // gate rows then up rows, the tcgen05 matmul, then the stand-alone SwiGLU + quantizer
        ST_TRY(launch_q4k_matmul(ctx, dw, 2 * F, K, aq, M, dgu, 2 * F, 2));
        ST_TRY(launch_swiglu_quant(ctx, dgu, M, F, 2 * F, nullptr, mid, false, false));
    } else {
        ST_TRY(launch_interleave_rows128(ctx, dw, dw + (size_t)F * rb, F, rb, dil));
        ST_TRY(launch_q4k_matmul_umma_swiglu(ctx, dil, 2 * F, K, aq, M, dgu, 2 * F, ctx->umma_scratch, ctx->umma_scratch_bytes, ctx->err_flag,
                                             mode == 1 ? mid : ActQ{}, mode == 1, &fused));
        if (mode == 1 && !fused) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the fused epilogue did not apply");
        if (!fused) ST_TRY(launch_swiglu_quant(ctx, dgu, M, F, 2 * F, nullptr, mid, false, true));
    }
    D2H(ctx, codes_out, mid.codes, (size_t)M * F);
    D2H(ctx, scales_out, mid.scales, (size_t)M * 2 * (F / 32) * 4);
    SYNC(ctx);
    return us.check();
}

int b200_op_kq_matmul(b200_ctx* ctx, int kind, const uint8_t* w, const float* a, int M, int K, int N, float* dst) {
    if (kind == B200_K_I8 ? K % 32 != 0 : (K % 256 || (kind != B200_K_Q5K && kind != B200_K_Q6K)))
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "a Q5_K or Q6_K matrix with K %% 256 == 0, or int8 rows with K %% 32 == 0");
    Tmp t;
    const size_t nb = (size_t)N * K / 256, wb = kind == B200_K_I8 ? (size_t)N * K + (size_t)N * 4 : nb * (kind == B200_K_Q5K ? 176 : 210);
    uint8_t *dw, *dp = nullptr; float *da, *dd; ActQ aq;
    TMP_GET(ctx, t, dw, wb); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, aq.codes, (size_t)M * K); TMP_GET(ctx, t, aq.scales, (size_t)M * 2 * (K / 32));
    H2D(ctx, dw, w, wb); H2D(ctx, da, a, (size_t)M * K * 4);
    if (kind == B200_K_Q6K) {
        TMP_GET(ctx, t, dp, wb);
        ST_TRY(launch_q6k_repack(ctx, dw, nb, dp));
    }
    ST_TRY(launch_quant_g32(ctx, da, M, K, aq));
    ST_TRY(launch_kq_matmul(ctx, kind, kind == B200_K_Q6K ? dp : dw, N, K, aq, M, dd, N));
    D2H(ctx, dst, dd, (size_t)M * N * 4);
    SYNC(ctx);
    return B200_OK;
}

// Test hook: the Q6_K matmul on the tcgen05 kernel that puts the codes together itself (what a fast-class model runs from
// 32 rows), at any M, on the file's 210-byte blocks.
int b200_debug_q6k_matmul_umma(b200_ctx* ctx, const uint8_t* w, const float* a, int M, int K, int N, float* dst) {
    return b200_debug_kq_matmul_umma(ctx, B200_K_Q6K, w, a, M, K, N, dst);
}

int b200_debug_kq_matmul_umma(b200_ctx* ctx, int kind, const uint8_t* w, const float* a, int M, int K, int N, float* dst) {
    if (K % 256 || M < 1 || N < 1 || (kind != B200_K_Q5K && kind != B200_K_Q6K)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "a Q5_K or Q6_K matrix with K %% 256 == 0");
    Tmp t;
    const size_t nb = (size_t)N * K / 256, wb = nb * (kind == B200_K_Q6K ? 210 : 176);
    uint8_t *dw, *dp; float *da, *dd; ActQ aq;
    TMP_GET(ctx, t, dw, wb); TMP_GET(ctx, t, dp, wb); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, aq.codes, (size_t)M * K); TMP_GET(ctx, t, aq.scales, (size_t)M * 2 * (K / 32));
    H2D(ctx, dw, w, wb); H2D(ctx, da, a, (size_t)M * K * 4);
    if (kind == B200_K_Q6K) ST_TRY(launch_q6k_repack(ctx, dw, nb, dp));
    ST_TRY(launch_quant_g32(ctx, da, M, K, aq));
    UmmaScratch us(ctx);
    ST_TRY(us.ensure(t, M, K, N));
    ST_TRY(launch_kq_matmul_umma(ctx, kind, kind == B200_K_Q6K ? dp : dw, N, K, aq, M, dd, N));
    D2H(ctx, dst, dd, (size_t)M * N * 4);
    SYNC(ctx);
    return us.check();
}

int b200_op_topk(b200_ctx* ctx, const float* logits, int rows, int vocab, int k, float inv_temperature, int32_t* ids_out,
                 float* logits_out, double* z_out) {
    if (rows <= 0 || vocab <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad top-K shape");
    Tmp t;
    float *dl, *dv; int32_t* di; double* dz;
    TMP_GET(ctx, t, dl, (size_t)rows * vocab); TMP_GET(ctx, t, dv, (size_t)rows * k); TMP_GET(ctx, t, di, (size_t)rows * k);
    TMP_GET(ctx, t, dz, (size_t)rows);
    H2D(ctx, dl, logits, (size_t)rows * vocab * 4);
    ST_TRY(launch_topk(ctx, dl, rows, vocab, k, inv_temperature, z_out != nullptr, di, dv, dz));
    D2H(ctx, ids_out, di, (size_t)rows * k * 4);
    D2H(ctx, logits_out, dv, (size_t)rows * k * 4);
    if (z_out) D2H(ctx, z_out, dz, (size_t)rows * 8);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_philox(b200_ctx* ctx, const uint32_t* ctr, const uint32_t* key, int n, uint32_t* out) {
    if (n <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad count");
    Tmp t;
    uint32_t *dc, *dk, *dout;
    TMP_GET(ctx, t, dc, (size_t)4 * n); TMP_GET(ctx, t, dk, (size_t)2 * n); TMP_GET(ctx, t, dout, (size_t)4 * n);
    H2D(ctx, dc, ctr, (size_t)16 * n); H2D(ctx, dk, key, (size_t)8 * n);
    ST_TRY(launch_philox(ctx, dc, dk, n, dout));
    D2H(ctx, out, dout, (size_t)16 * n);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_f16_matmul(b200_ctx* ctx, const uint16_t* w, const float* a, int M, int K, int N, int klass, float* dst) {
    if (M <= 0 || K <= 0 || N <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad matmul shape");
    Tmp t;
    __half *dw, *split; float *da, *dd;
    TMP_GET(ctx, t, dw, (size_t)N * K); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, split, (size_t)2 * M * K);
    H2D(ctx, dw, w, (size_t)N * K * 2); H2D(ctx, da, a, (size_t)M * K * 4);
    UmmaScratch us(ctx);
    ST_TRY(us.ensure_bytes(t, f16w_umma_scratch_bytes(M, K)));
    if (klass == 2 && !f16w_umma_supported(dw, N, K)) B200_FAIL(ctx, B200_DECLINED, "f16 tcgen05 matmul needs K %% 64 == 0 and N >= 256");
    ST_TRY(launch_f16w_matmul(ctx, dw, N, K, da, M, dd, N, split, klass));
    D2H(ctx, dst, dd, (size_t)M * N * 4);
    SYNC(ctx);
    return us.check();
}

int b200_bench_f16_matmul(b200_ctx* ctx, int M, int K, int N, int klass, int warmup, int iters, float* ms_out) {
    if (M <= 0 || K <= 0 || N <= 0 || iters <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad bench shape");
    Tmp t;
    __half *dw, *split; float *da, *dd;
    TMP_GET(ctx, t, dw, (size_t)N * K); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, split, (size_t)2 * M * K);
    ST_TRY(launch_synth_f16(ctx, dw, (size_t)N * K, 0.02f, 23));
    ST_TRY(launch_synth_normal_f32(ctx, da, (size_t)M * K, 1.f, 5));
    UmmaScratch us(ctx);
    ST_TRY(us.ensure_bytes(t, f16w_umma_scratch_bytes(M, K)));
    cudaEvent_t e0, e1;
    CUDA_TRY(ctx, cudaEventCreate(&e0)); CUDA_TRY(ctx, cudaEventCreate(&e1));
    for (int i = 0; i < warmup; i++) ST_TRY(launch_f16w_matmul(ctx, dw, N, K, da, M, dd, N, split, klass));
    CUDA_TRY(ctx, cudaEventRecord(e0, ctx->stream));
    for (int i = 0; i < iters; i++) ST_TRY(launch_f16w_matmul(ctx, dw, N, K, da, M, dd, N, split, klass));
    CUDA_TRY(ctx, cudaEventRecord(e1, ctx->stream));
    SYNC(ctx);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *ms_out = ms / iters;
    return us.check();
}

int b200_op_q4k_quantize(b200_ctx* ctx, const float* w, int rows, int cols, uint8_t* out) {
    if (cols % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "cols %% 256");
    Tmp t;
    const size_t nb = (size_t)rows * cols / 256;
    float* dw; uint8_t* dq;
    TMP_GET(ctx, t, dw, nb * 256); TMP_GET(ctx, t, dq, nb * 144);
    H2D(ctx, dw, w, nb * 256 * 4);
    ST_TRY(launch_q4k_quantize(ctx, dw, nb, dq));
    D2H(ctx, out, dq, nb * 144);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_rmsnorm(b200_ctx* ctx, const float* x, const float* w, int rows, int dim, float eps, float* out) {
    Tmp t;
    float *dx, *dw, *dout;
    TMP_GET(ctx, t, dx, (size_t)rows * dim); TMP_GET(ctx, t, dw, (size_t)dim); TMP_GET(ctx, t, dout, (size_t)rows * dim);
    H2D(ctx, dx, x, (size_t)rows * dim * 4); H2D(ctx, dw, w, (size_t)dim * 4);
    ST_TRY(launch_add_rmsnorm_quant(ctx, dx, nullptr, dw, rows, dim, eps, dout, ActQ{}, nullptr));
    D2H(ctx, out, dout, (size_t)rows * dim * 4);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_route(b200_ctx* ctx, const float* logits, int rows, int n_experts, int k, int norm_topk, int32_t* idx, float* wts) {
    Tmp t;
    float *dl, *dw; int32_t* di;
    TMP_GET(ctx, t, dl, (size_t)rows * n_experts); TMP_GET(ctx, t, dw, (size_t)rows * k); TMP_GET(ctx, t, di, (size_t)rows * k);
    H2D(ctx, dl, logits, (size_t)rows * n_experts * 4);
    ST_TRY(launch_route(ctx, dl, rows, n_experts, k, norm_topk, di, dw));
    D2H(ctx, idx, di, (size_t)rows * k * 4); D2H(ctx, wts, dw, (size_t)rows * k * 4);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_draw(b200_ctx* ctx, const float* logits, int rows, int vocab, const b200_draw* draws, const int32_t* mask_index,
                 const uint32_t* logit_mask, int n_masks, int32_t* ids) {
    Tmp t;
    float* dl; b200_draw* dd; int32_t *dm, *di; uint32_t* dmk;
    const size_t words = (vocab + 31) / 32;
    TMP_GET(ctx, t, dl, (size_t)rows * vocab); TMP_GET(ctx, t, dd, (size_t)rows); TMP_GET(ctx, t, dm, (size_t)rows);
    TMP_GET(ctx, t, di, (size_t)rows); TMP_GET(ctx, t, dmk, std::max<size_t>(1, (size_t)n_masks * words));
    H2D(ctx, dl, logits, (size_t)rows * vocab * 4); H2D(ctx, dd, draws, (size_t)rows * sizeof(b200_draw));
    if (mask_index && logit_mask && n_masks > 0) {
        H2D(ctx, dm, mask_index, (size_t)rows * 4); H2D(ctx, dmk, logit_mask, (size_t)n_masks * words * 4);
        ST_TRY(launch_mask_logits(ctx, dl, rows, vocab, dm, dmk));
    }
    ST_TRY(launch_draw(ctx, dl, rows, vocab, dd, di, nullptr));
    D2H(ctx, ids, di, (size_t)rows * 4);
    SYNC(ctx);
    return B200_OK;
}

int b200_op_attention(b200_ctx* ctx, const float* q, const float* k, const float* v, const int32_t* n_keys, int rows, int max_keys,
                      int n_heads, int n_kv_heads, int head_dim, float scale, float softcap, int block_rows, int klass,
                      float* out) {
    if (rows <= 0 || max_keys <= 0 || block_rows <= 0 || n_heads % n_kv_heads) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad attention shape");
    Tmp t;
    const int max_blocks = ceil_div(max_keys, block_rows);
    const size_t pool_blocks = 1 + (size_t)rows * max_blocks;
    const size_t pool_elems = pool_blocks * n_kv_heads * block_rows * head_dim;
    const size_t kvn = (size_t)rows * max_keys * n_kv_heads * head_dim, qn = (size_t)rows * n_heads * head_dim;
    float *dq, *dk, *dv, *dout; __half *kp, *vp; int32_t *tbl, *nk, *rpos, *rslot;
    AttnScratch sc;
    sc.max_splits = ceil_div(max_keys, attn_split_keys());
    TMP_GET(ctx, t, dq, qn); TMP_GET(ctx, t, dk, kvn); TMP_GET(ctx, t, dv, kvn); TMP_GET(ctx, t, dout, qn);
    TMP_GET(ctx, t, kp, pool_elems); TMP_GET(ctx, t, vp, pool_elems);
    TMP_GET(ctx, t, tbl, (size_t)rows * max_blocks); TMP_GET(ctx, t, nk, (size_t)rows); TMP_GET(ctx, t, rpos, (size_t)rows);
    TMP_GET(ctx, t, rslot, (size_t)rows);
    TMP_GET(ctx, t, sc.partial, attn_scratch_floats(rows, n_heads, head_dim, sc.max_splits));
    H2D(ctx, dq, q, qn * 4); H2D(ctx, dk, k, kvn * 4); H2D(ctx, dv, v, kvn * 4); H2D(ctx, nk, n_keys, (size_t)rows * 4);
    CUDA_TRY(ctx, cudaMemsetAsync(kp, 0, pool_elems * 2, ctx->stream));
    CUDA_TRY(ctx, cudaMemsetAsync(vp, 0, pool_elems * 2, ctx->stream));
    iota_blocks_kernel<<<ceil_div(rows * max_blocks, 256), 256, 0, ctx->stream>>>(tbl, rows, max_blocks, nk, block_rows);
    LAUNCH_CHECK(ctx);
    scatter_kv_kernel<<<(unsigned)((kvn + 255) / 256), 256, 0, ctx->stream>>>(dk, dv, kp, vp, tbl, rows, max_keys, max_blocks,
                                                                              n_kv_heads, head_dim, block_rows, nk);
    LAUNCH_CHECK(ctx);
    ctx_minus1_kernel<<<ceil_div(rows, 256), 256, 0, ctx->stream>>>(nk, rpos, rslot, rows);
    LAUNCH_CHECK(ctx);
    KVView kv{kp, vp, tbl, max_blocks, block_rows, n_kv_heads, head_dim};
    const float sc_ = scale != 0.f ? scale : (float)(1.0 / std::sqrt((double)head_dim));
    if (klass == B200_CLASS_EXACT) {
        float* scores;
        TMP_GET(ctx, t, scores, (size_t)rows * n_heads * max_keys);
        const double sd = scale != 0.f ? (double)scale : 1.0 / std::sqrt((double)head_dim);
        ST_TRY(launch_paged_attention_exact(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, sd, (double)softcap,
                                            rslot, rpos, max_keys, kv, scores, max_keys, dout, ActQ{}));
    } else {
        ST_TRY(launch_paged_attention(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, sc_, softcap, rslot, rpos,
                                      max_keys, kv, sc, dout, ActQ{}));
    }
    D2H(ctx, out, dout, qn * 4);
    SYNC(ctx);
    return B200_OK;
}

namespace {
// one slot holding `keys` rows of K/V in a fresh pool; fills kv and returns through the Tmp
int build_one_slot_kv(b200_ctx* ctx, Tmp& t, const float* dk, const float* dv, int keys, int n_kv_heads, int head_dim, int block_rows,
                      KVView* kv_out) {
    const int max_blocks = ceil_div(keys, block_rows);
    const size_t pool_elems = (size_t)(1 + max_blocks) * n_kv_heads * block_rows * head_dim;
    __half *kp, *vp; int32_t *tbl, *nk;
    TMP_GET(ctx, t, kp, pool_elems); TMP_GET(ctx, t, vp, pool_elems); TMP_GET(ctx, t, tbl, (size_t)max_blocks); TMP_GET(ctx, t, nk, 1);
    CUDA_TRY(ctx, cudaMemsetAsync(kp, 0, pool_elems * 2, ctx->stream));
    CUDA_TRY(ctx, cudaMemsetAsync(vp, 0, pool_elems * 2, ctx->stream));
    H2D(ctx, nk, &keys, 4);
    iota_blocks_kernel<<<ceil_div(max_blocks, 256), 256, 0, ctx->stream>>>(tbl, 1, max_blocks, nk, block_rows);
    LAUNCH_CHECK(ctx);
    const size_t kvn = (size_t)keys * n_kv_heads * head_dim;
    scatter_kv_kernel<<<(unsigned)((kvn + 255) / 256), 256, 0, ctx->stream>>>(dk, dv, kp, vp, tbl, 1, keys, max_blocks, n_kv_heads,
                                                                              head_dim, block_rows, nk);
    LAUNCH_CHECK(ctx);
    *kv_out = KVView{kp, vp, tbl, max_blocks, block_rows, n_kv_heads, head_dim};
    return B200_OK;
}
}  // namespace

int b200_op_prefill_attention(b200_ctx* ctx, const float* q, const float* k, const float* v, int rows, int pos0, int n_heads,
                              int n_kv_heads, int head_dim, float scale, float softcap, int block_rows, float* out) {
    if (rows <= 0 || pos0 < 0 || block_rows <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad attention shape");
    if (!prefill_attention_supported(n_heads, n_kv_heads, head_dim, block_rows))
        B200_FAIL(ctx, B200_DECLINED, "prefill attention: head_dim %d, group %d, %d-row blocks is not built", head_dim, n_heads / n_kv_heads, block_rows);
    Tmp t;
    const int keys = pos0 + rows;
    const size_t kvn = (size_t)keys * n_kv_heads * head_dim, qn = (size_t)rows * n_heads * head_dim;
    float *dq, *dk, *dv, *dout;
    TMP_GET(ctx, t, dq, qn); TMP_GET(ctx, t, dk, kvn); TMP_GET(ctx, t, dv, kvn); TMP_GET(ctx, t, dout, qn);
    H2D(ctx, dq, q, qn * 4); H2D(ctx, dk, k, kvn * 4); H2D(ctx, dv, v, kvn * 4);
    KVView kv;
    ST_TRY(build_one_slot_kv(ctx, t, dk, dv, keys, n_kv_heads, head_dim, block_rows, &kv));
    const float sc_ = scale != 0.f ? scale : (float)(1.0 / std::sqrt((double)head_dim));
    ST_TRY(launch_prefill_attention(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, sc_, softcap, 0, pos0, kv, dout,
                                    n_heads * head_dim));
    D2H(ctx, out, dout, qn * 4);
    SYNC(ctx);
    return B200_OK;
}

int b200_bench_prefill_attention(b200_ctx* ctx, int rows, int pos0, int n_heads, int n_kv_heads, int head_dim, int block_rows,
                                 int warmup, int iters, float* ms_out) {
    if (rows <= 0 || pos0 < 0 || iters <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad bench shape");
    if (!prefill_attention_supported(n_heads, n_kv_heads, head_dim, block_rows)) B200_FAIL(ctx, B200_DECLINED, "prefill attention shape is not built");
    Tmp t;
    const int keys = pos0 + rows;
    const size_t kvn = (size_t)keys * n_kv_heads * head_dim, qn = (size_t)rows * n_heads * head_dim;
    float *dq, *dk, *dv, *dout;
    TMP_GET(ctx, t, dq, qn); TMP_GET(ctx, t, dk, kvn); TMP_GET(ctx, t, dv, kvn); TMP_GET(ctx, t, dout, qn);
    ST_TRY(launch_synth_normal_f32(ctx, dq, qn, 1.f, 11));
    ST_TRY(launch_synth_normal_f32(ctx, dk, kvn, 0.5f, 12));
    ST_TRY(launch_synth_normal_f32(ctx, dv, kvn, 0.5f, 13));
    KVView kv;
    ST_TRY(build_one_slot_kv(ctx, t, dk, dv, keys, n_kv_heads, head_dim, block_rows, &kv));
    const float sc_ = (float)(1.0 / std::sqrt((double)head_dim));
    cudaEvent_t e0, e1;
    CUDA_TRY(ctx, cudaEventCreate(&e0)); CUDA_TRY(ctx, cudaEventCreate(&e1));
    for (int i = 0; i < warmup; i++)
        ST_TRY(launch_prefill_attention(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, sc_, 0.f, 0, pos0, kv, dout, n_heads * head_dim));
    CUDA_TRY(ctx, cudaEventRecord(e0, ctx->stream));
    for (int i = 0; i < iters; i++)
        ST_TRY(launch_prefill_attention(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, sc_, 0.f, 0, pos0, kv, dout, n_heads * head_dim));
    CUDA_TRY(ctx, cudaEventRecord(e1, ctx->stream));
    SYNC(ctx);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *ms_out = ms / iters;
    return B200_OK;
}

namespace {
__global__ void __launch_bounds__(512) read_sum_kernel(const uint4* __restrict__ p, size_t n, unsigned* __restrict__ sink) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t st = (size_t)gridDim.x * blockDim.x;
    unsigned s = 0;
    for (; i + 3 * st < n; i += 4 * st) {
        const uint4 a = p[i], b = p[i + st], c = p[i + 2 * st], d = p[i + 3 * st];
        s += a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < n; i += st) {
        const uint4 a = p[i];
        s += a.x ^ a.y ^ a.z ^ a.w;
    }
    if (s == 0x12345678u) sink[0] = s;  // keeps the loads alive; practically never taken
}
}  // namespace

int b200_bench_read(b200_ctx* ctx, size_t bytes, int n_copies, int warmup, int iters, float* ms_out) {
    if (bytes < 16 || n_copies <= 0 || iters <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad bench shape");
    Tmp t;
    const size_t n = bytes / 16;
    uint8_t* buf; unsigned* sink;
    TMP_GET(ctx, t, buf, n * 16 * n_copies); TMP_GET(ctx, t, sink, 1);
    CUDA_TRY(ctx, cudaMemsetAsync(buf, 0x11, n * 16 * n_copies, ctx->stream));
    const int grid = ctx->sm_count * 4;
    cudaEvent_t e0, e1;
    CUDA_TRY(ctx, cudaEventCreate(&e0)); CUDA_TRY(ctx, cudaEventCreate(&e1));
    for (int i = 0; i < warmup; i++) read_sum_kernel<<<grid, 512, 0, ctx->stream>>>(reinterpret_cast<const uint4*>(buf) + (size_t)(i % n_copies) * n, n, sink);
    CUDA_TRY(ctx, cudaEventRecord(e0, ctx->stream));
    for (int i = 0; i < iters; i++) read_sum_kernel<<<grid, 512, 0, ctx->stream>>>(reinterpret_cast<const uint4*>(buf) + (size_t)(i % n_copies) * n, n, sink);
    CUDA_TRY(ctx, cudaEventRecord(e1, ctx->stream));
    SYNC(ctx);
    LAUNCH_CHECK(ctx);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *ms_out = ms / iters;
    return B200_OK;
}

namespace {
// random code bytes with scales of a sane size at the f16 fields (Q5_K: d and dmin at 0 and 2; Q6_K: the d values behind the bodies)
__global__ void kq_fill_kernel(uint8_t* __restrict__ w, size_t n_bytes, size_t n_blocks, int kind, uint64_t seed) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_bytes) return;
    uint64_t z = (i + 1) * 0x9E3779B97F4A7C15ull + seed;
    z ^= z >> 31; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 29;
    uint8_t v = (uint8_t)(z >> 24);
    if (kind == B200_K_Q5K) {
        const size_t o = i % 176;
        if (o < 4) v = (o & 1) ? 0x20 : (uint8_t)(z >> 40);   // f16 with exponent byte 0x20: about 0.008 .. 0.016
    } else {
        if (i >= 208 * n_blocks) v = ((i - 208 * n_blocks) & 1) ? 0x20 : (uint8_t)(z >> 40);
    }
    w[i] = v;
}
}  // namespace

int b200_bench_kq_matmul(b200_ctx* ctx, int kind, int M, int K, int N, int n_weight_copies, int warmup, int iters, float* ms_out) {
    if (K % 256 || M <= 0 || N <= 0 || n_weight_copies <= 0 || iters <= 0 || (kind != B200_K_Q5K && kind != B200_K_Q6K))
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad bench shape");
    Tmp t;
    const size_t nb = (size_t)N * K / 256, wb = nb * (kind == B200_K_Q5K ? 176 : 210), wbp = (wb + 255) & ~(size_t)255;
    uint8_t* dw; float *da, *dd; ActQ aq;
    TMP_GET(ctx, t, dw, wbp * n_weight_copies); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, aq.codes, (size_t)M * K); TMP_GET(ctx, t, aq.scales, (size_t)M * 2 * (K / 32));
    for (int c = 0; c < n_weight_copies; c++) {
        kq_fill_kernel<<<(unsigned)((wb + 255) / 256), 256, 0, ctx->stream>>>(dw + (size_t)c * wbp, wb, nb, kind, 17 + c);
        LAUNCH_CHECK(ctx);
    }
    ST_TRY(launch_synth_normal_f32(ctx, da, (size_t)M * K, 1.f, 5));
    ST_TRY(launch_quant_g32(ctx, da, M, K, aq));
    cudaEvent_t e0, e1;
    CUDA_TRY(ctx, cudaEventCreate(&e0)); CUDA_TRY(ctx, cudaEventCreate(&e1));
    for (int i = 0; i < warmup; i++) ST_TRY(launch_kq_matmul(ctx, kind, dw + (size_t)(i % n_weight_copies) * wbp, N, K, aq, M, dd, N));
    CUDA_TRY(ctx, cudaEventRecord(e0, ctx->stream));
    for (int i = 0; i < iters; i++) ST_TRY(launch_kq_matmul(ctx, kind, dw + (size_t)(i % n_weight_copies) * wbp, N, K, aq, M, dd, N));
    CUDA_TRY(ctx, cudaEventRecord(e1, ctx->stream));
    SYNC(ctx);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *ms_out = ms / iters;
    return B200_OK;
}

int b200_bench_q4k_matmul(b200_ctx* ctx, int M, int K, int N, int klass, int n_weight_copies, int warmup, int iters, float* ms_out) {
    if (K % 256 || M <= 0 || N <= 0 || n_weight_copies <= 0 || iters <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad bench shape");
    const bool tiles_only = klass == 7;  // the fast class as a model runs it: only the tile-major copy is given to the kernels
    if (tiles_only) klass = 0;
    Tmp t;
    const size_t wb = (size_t)N * K / 256 * 144;
    uint8_t* dw; float *da, *dd; ActQ aq;
    // several copies of the matrix, cycled, so a launch never finds its weights in L2
    TMP_GET(ctx, t, dw, wb * n_weight_copies); TMP_GET(ctx, t, da, (size_t)M * K); TMP_GET(ctx, t, dd, (size_t)M * N);
    TMP_GET(ctx, t, aq.codes, (size_t)M * K); TMP_GET(ctx, t, aq.scales, (size_t)M * 2 * (K / 32));
    for (int c = 0; c < n_weight_copies; c++) ST_TRY(launch_synth_q4k(ctx, dw + (size_t)c * wb, wb / 144, 0.02f, 17 + c));
    // up to 32 rows the fast class streams the tile-by-tile copy of the matrix a model makes at finalize
    uint8_t* dtiles = nullptr;
    const size_t tb = q4k_tiles_bytes(N, K);
    if (tiles_only || ((klass == 0 || klass == 5) && M <= 32)) {
        TMP_GET(ctx, t, dtiles, tb * n_weight_copies);
        for (int c = 0; c < n_weight_copies; c++) ST_TRY(launch_q4k_to_tiles(ctx, dw + (size_t)c * wb, N, K, dtiles + (size_t)c * tb));
    }
    ST_TRY(launch_synth_normal_f32(ctx, da, (size_t)M * K, 1.f, 5));
    ST_TRY(launch_quant_g32(ctx, da, M, K, aq));
    UmmaScratch us(ctx);
    ST_TRY(us.ensure(t, M, K, N));
    cudaEvent_t e0, e1;
    CUDA_TRY(ctx, cudaEventCreate(&e0)); CUDA_TRY(ctx, cudaEventCreate(&e1));
    // In a step the kernel that quantized the activations has also laid out the fp16 tiles the fast class's matmuls read
    // (up to 32 rows: the small-batch kernel): klass 0 prepares them once, outside the timed launches, the way a step finds
    // them; klass 5 leaves the conversion kernel in every launch.
    struct TilesGiven {
        b200_ctx* c;
        ~TilesGiven() { c->x16_ready = nullptr; }
    } tiles_given{ctx};
    if (klass == 0 && M >= q4k_small_min_rows() && q4k_small_min_rows() > 0 && M <= 32) {
        ST_TRY(launch_act_to_f16(ctx, aq, M, K, reinterpret_cast<__half*>(ctx->umma_scratch)));
        ctx->x16_ready = reinterpret_cast<const __half*>(ctx->umma_scratch);
    }
    auto tiles_of = [&](int i) { return dtiles ? dtiles + (size_t)(i % n_weight_copies) * tb : nullptr; };
    auto rows_of = [&](int i) -> const uint8_t* { return tiles_only ? nullptr : dw + (size_t)(i % n_weight_copies) * wb; };
    for (int i = 0; i < warmup; i++) ST_TRY(launch_q4k_matmul(ctx, rows_of(i), N, K, aq, M, dd, N, klass, tiles_of(i)));
    CUDA_TRY(ctx, cudaEventRecord(e0, ctx->stream));
    for (int i = 0; i < iters; i++) ST_TRY(launch_q4k_matmul(ctx, rows_of(i), N, K, aq, M, dd, N, klass, tiles_of(i)));
    CUDA_TRY(ctx, cudaEventRecord(e1, ctx->stream));
    SYNC(ctx);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *ms_out = ms / iters;
    return us.check();
}

int b200_bench_attention(b200_ctx* ctx, int rows, int ctx_lo, int ctx_hi, int n_heads, int n_kv_heads, int head_dim,
                         int block_rows, uint64_t seed, int warmup, int iters, float* ms_out, double* kv_bytes_out) {
    if (rows <= 0 || ctx_lo <= 0 || ctx_hi < ctx_lo || iters <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad bench shape");
    Tmp t;
    std::vector<int32_t> nk(rows);
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + 1;
    double tot_keys = 0;
    for (int r = 0; r < rows; r++) {
        z ^= z << 13; z ^= z >> 7; z ^= z << 17;
        nk[r] = ctx_lo + (int)(z % (uint64_t)(ctx_hi - ctx_lo + 1));
        tot_keys += nk[r];
    }
    const int max_keys = ctx_hi, max_blocks = ceil_div(max_keys, block_rows);
    const size_t pool_blocks = 1 + (size_t)rows * max_blocks;
    const size_t pool_elems = pool_blocks * n_kv_heads * block_rows * head_dim;
    const size_t qn = (size_t)rows * n_heads * head_dim;
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    if (pool_elems * 4 + ((size_t)2 << 30) > free_b) B200_FAIL(ctx, B200_BAD_ARGUMENT, "attention bench pool does not fit the device");
    float *dq, *dout; __half *kp, *vp; int32_t *tbl, *dnk, *rpos, *rslot;
    AttnScratch sc;
    sc.max_splits = ceil_div(max_keys, attn_split_keys());
    TMP_GET(ctx, t, dq, qn); TMP_GET(ctx, t, dout, qn); TMP_GET(ctx, t, kp, pool_elems); TMP_GET(ctx, t, vp, pool_elems);
    TMP_GET(ctx, t, tbl, (size_t)rows * max_blocks); TMP_GET(ctx, t, dnk, (size_t)rows); TMP_GET(ctx, t, rpos, (size_t)rows);
    TMP_GET(ctx, t, rslot, (size_t)rows);
    TMP_GET(ctx, t, sc.partial, attn_scratch_floats(rows, n_heads, head_dim, sc.max_splits));
    H2D(ctx, dnk, nk.data(), (size_t)rows * 4);
    ST_TRY(launch_synth_normal_f32(ctx, dq, qn, 1.f, seed + 1));
    ST_TRY(launch_synth_f16(ctx, kp, pool_elems, 0.5f, seed + 2));
    ST_TRY(launch_synth_f16(ctx, vp, pool_elems, 0.5f, seed + 3));
    iota_blocks_kernel<<<ceil_div(rows * max_blocks, 256), 256, 0, ctx->stream>>>(tbl, rows, max_blocks, dnk, block_rows);
    LAUNCH_CHECK(ctx);
    ctx_minus1_kernel<<<ceil_div(rows, 256), 256, 0, ctx->stream>>>(dnk, rpos, rslot, rows);
    LAUNCH_CHECK(ctx);
    KVView kv{kp, vp, tbl, max_blocks, block_rows, n_kv_heads, head_dim};
    const float scale = (float)(1.0 / std::sqrt((double)head_dim));
    cudaEvent_t e0, e1;
    CUDA_TRY(ctx, cudaEventCreate(&e0)); CUDA_TRY(ctx, cudaEventCreate(&e1));
    for (int i = 0; i < warmup; i++)
        ST_TRY(launch_paged_attention(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, scale, 0.f, rslot, rpos, max_keys, kv, sc, dout, ActQ{}));
    CUDA_TRY(ctx, cudaEventRecord(e0, ctx->stream));
    for (int i = 0; i < iters; i++)
        ST_TRY(launch_paged_attention(ctx, dq, n_heads * head_dim, rows, n_heads, n_kv_heads, head_dim, scale, 0.f, rslot, rpos, max_keys, kv, sc, dout, ActQ{}));
    CUDA_TRY(ctx, cudaEventRecord(e1, ctx->stream));
    SYNC(ctx);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *ms_out = ms / iters;
    if (kv_bytes_out) *kv_bytes_out = tot_keys * 2.0 * n_kv_heads * head_dim * 2.0;
    return B200_OK;
}

}  // extern "C"

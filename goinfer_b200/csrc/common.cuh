// common.cuh — context, error handling and the launcher table shared by the library's .cu files.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/b200_bench.h"  // brings in b200_resident.h

// Kernel classes the per-launch profiler tells apart.
enum ProfTag { PROF_ATTN_SPLIT = 0, PROF_ATTN_COMBINE, PROF_Q4K_GEMM, PROF_HEAD_GEMM, PROF_NORM_QUANT, PROF_ROPE_KV,
               PROF_SWIGLU, PROF_OTHER, PROF_TAGS };

struct ProfRec {
    int tag;
    cudaEvent_t e0, e1;
};

// The K-split partial matrices a matmul left unsummed for its consumer: n matrices [rows][width of dst] `stride` floats
// apart, to be added in order in place of reading `dst`.
struct Parts {
    const float* p = nullptr;
    size_t stride = 0;
    int n = 0;
    const float* dst = nullptr;
    int rows = 0, cols = 0;  // of dst (row stride = cols)
};

struct b200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    std::string err;
    int64_t launches = 0;  // kernels this library launched on the context
    int sm_count = 148;
    // scratch of the tcgen05 matmul (fp16 activations + split-K partials) and the device flag a bounded wait raises;
    // owned by whoever set them (a model at finalize, or an operator-level entry point for the length of its call)
    void* umma_scratch = nullptr;
    size_t umma_scratch_bytes = 0;
    int* err_flag = nullptr;
    // set around a matmul whose consumer (residual add + norm, RoPE/KV store, residual add) can add the K-split partials
    // itself: the matmul then skips its reduce kernel and leaves `pending`; the consumer that is handed pending.dst takes it
    bool defer_reduce = false;
    Parts pending;
    // fp16 activation tiles made by the kernel that quantized the activations (instead of a conversion kernel ahead of the
    // tcgen05 matmul): when x16_slot_bytes is set the scratch starts with two slots of that size (a matmul reads one while
    // its epilogue or the next producer fills the other) and the K-split partials follow them. x16_ready is set by the
    // caller around the one matmul whose activations a producer has just laid out, and is null otherwise.
    size_t x16_slot_bytes = 0;
    int x16_toggle = 0;
    const __half* x16_ready = nullptr;
    // a request to the attention output's quantizers (the split merge, the per-32 quantizer of a prefill run) to lay rows
    // x16_row0.. of the slot out as they quantize them; each adds the rows it covered to x16_done
    __half* x16_want = nullptr;
    int x16_row0 = 0, x16_done = 0;
    // tensor parallel: the NCCL communicator b200_tp_init made for this context (null on a single GPU)
    void* tp_comm = nullptr;
    int tp_rank = 0, tp_size = 1;
    // per-launch CUDA-event timing of the tagged kernel classes (off unless b200_profile sets a mask)
    unsigned prof_mask = 0;
    std::vector<ProfRec> prof_recs;
    std::vector<cudaEvent_t> prof_pool;
    cudaEvent_t prof_event() {
        if (!prof_pool.empty()) { cudaEvent_t e = prof_pool.back(); prof_pool.pop_back(); return e; }
        cudaEvent_t e;
        cudaEventCreate(&e);
        return e;
    }
};

// Brackets one kernel launch with events when its class is being profiled.
struct ProfScope {
    b200_ctx* ctx;
    ProfRec rec;
    bool on;
    ProfScope(b200_ctx* c, int tag) : ctx(c), on((c->prof_mask >> tag) & 1u) {
        if (on) {
            rec.tag = tag;
            rec.e0 = c->prof_event();
            rec.e1 = c->prof_event();
            cudaEventRecord(rec.e0, c->stream);
        }
    }
    ~ProfScope() {
        if (on) {
            cudaEventRecord(rec.e1, ctx->stream);
            ctx->prof_recs.push_back(rec);
        }
    }
};

#define B200_FAIL(ctx, code, ...)                         \
    do {                                                  \
        char buf_[512];                                   \
        snprintf(buf_, sizeof buf_, __VA_ARGS__);         \
        (ctx)->err = buf_;                                \
        return (code);                                    \
    } while (0)

#define CUDA_TRY(ctx, expr)                                                                              \
    do {                                                                                                 \
        cudaError_t e_ = (expr);                                                                         \
        if (e_ != cudaSuccess) B200_FAIL(ctx, B200_CUDA_ERROR, "%s: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

#define ST_TRY(expr)            \
    do {                        \
        int st_ = (expr);       \
        if (st_ != B200_OK) return st_; \
    } while (0)

// Counts the launch and reports a launch-time error.
#define LAUNCH_CHECK(ctx)                                                                               \
    do {                                                                                                \
        (ctx)->launches++;                                                                              \
        cudaError_t e_ = cudaGetLastError();                                                            \
        if (e_ != cudaSuccess) B200_FAIL(ctx, B200_CUDA_ERROR, "launch failed: %s (%s:%d)", cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// One-time set-up that belongs to a device rather than to the process (cudaFuncSetAttribute): a flag per device ordinal.
// Calls into the library are serialized per context; two contexts of different devices touch different flags.
struct PerDeviceOnce {
    bool done[64] = {};
    bool first(int device) {
        bool& d = done[device & 63];
        const bool was = d;
        d = true;
        return !was;
    }
};

// ---- programmatic dependent launch -------------------------------------------------------------------------------
// A kernel launched with launch_pdl may start while the kernel before it on the stream is still running: its blocks are
// placed as soon as every block of the earlier kernel has called pdl_trigger() (or left), and they must call pdl_wait()
// before they read or write anything an earlier kernel may touch; pdl_wait() returns when the earlier kernels have
// completed and their writes are visible. What runs before the wait (index arithmetic, barrier set-up, loads of weights,
// which no kernel writes) overlaps the earlier kernel's tail, and the launch latency disappears from the chain.
// RULE: only kernels whose every thread reaches pdl_wait() before its first dependent access go through launch_pdl.
// Without the launch attribute both calls do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = getenv("B200_NO_PDL") == nullptr;
    return on;
}

// Eight consecutive activations (k8 a multiple of 8) of row t as the tcgen05 matmul's fp16 tiles hold them: the matrix is
// stored [token tile of 256][chunk of 64 along K][256 rows][64], the 16-byte chunk c of a row at position c ^ (t & 7) (the
// 128-byte swizzle), positions 1 and 2 of every group of four swapped (the order nibble pairs leave a code word in).
// v[i] = code * scale, rounded to fp16 here.
__device__ __forceinline__ void x16_store8(__half* __restrict__ out, int K, int t, int k8, const float (&v)[8]) {
    uint4 o;
    __half2 h;
    h = __floats2half2_rn(v[0], v[2]); o.x = *reinterpret_cast<unsigned*>(&h);
    h = __floats2half2_rn(v[1], v[3]); o.y = *reinterpret_cast<unsigned*>(&h);
    h = __floats2half2_rn(v[4], v[6]); o.z = *reinterpret_cast<unsigned*>(&h);
    h = __floats2half2_rn(v[5], v[7]); o.w = *reinterpret_cast<unsigned*>(&h);
    const int seg = k8 >> 6, chunk = (k8 >> 3) & 7;
    const size_t tile = ((size_t)(t >> 8) * (size_t)(K >> 6) + seg) * (256 * 64);
    *reinterpret_cast<uint4*>(out + tile + (size_t)(t & 255) * 64 + ((chunk ^ (t & 7)) << 3)) = o;
}

// one activation of row t at column k into the same tiles
__device__ __forceinline__ void x16_store1(__half* __restrict__ out, int K, int t, int k, float v) {
    const int i = k & 7, pos = (i == 1 || i == 2) ? 3 - i : ((i == 5 || i == 6) ? 11 - i : i);
    const int seg = k >> 6, chunk = (k >> 3) & 7;
    const size_t tile = ((size_t)(t >> 8) * (size_t)(K >> 6) + seg) * (256 * 64);
    out[tile + (size_t)(t & 255) * 64 + ((chunk ^ (t & 7)) << 3) + pos] = __float2half_rn(v);
}

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // an error surfaces in LAUNCH_CHECK's cudaGetLastError
}
#endif

// ---- device buffers a Q4_K matmul reads: int8 codes [T][K] and scales [T][2*K/32] ----
struct ActQ {
    int8_t* codes = nullptr;
    float* scales = nullptr;
};

// ---- paged KV view of one layer ----
// Pool layout: [block][kv_head][row in block][head_dim] fp16 for K, the same for V. One (block, kv head)
// tile is block_rows*head_dim*2 contiguous bytes.
struct KVView {
    __half* k = nullptr;
    __half* v = nullptr;
    const int32_t* table = nullptr;  // [n_slots][max_blocks]
    int max_blocks = 0, block_rows = 16, n_kv = 0, hd = 0;
};

// ---- launchers (each returns a B200_* status) ----
// elementwise.cu
int launch_embed_gather(b200_ctx*, const void* table, int kind, int n_rows, const int32_t* ids, int T, int H, float scale, float* h);
// h += delta (delta may be null), then RMSNorm(h)*w -> normed f32 (may be null) and/or per-32 int8 (aq.codes may be null).
int launch_add_rmsnorm_quant(b200_ctx*, float* h, const float* delta, const float* w, int T, int H, float eps,
                             float* normed, ActQ aq, const int32_t* gather_rows, __half* x16 = nullptr);
int launch_quant_g32(b200_ctx*, const float* x, int T, int K, ActQ aq);
// f64_silu: the reference's f64 silu (decoder/rmsnorm.go:204-207); false in the fast class (f32 expf, about 2e-7 relative)
int launch_swiglu_quant(b200_ctx*, const float* gate_up, int T, int F, int ld, float* mid_f32, ActQ aq, bool f64_silu = true,
                        bool interleaved128 = false, __half* x16 = nullptr);  // x16: also lay the fp16 tiles out (x16_store8)  // interleaved128: gate f at (f/128)*256 + f%128, up 128 further
int launch_add(b200_ctx*, float* h, const float* delta, size_t n);
// q (in place, f32), k,v -> paged fp16 store; optional per-head RMSNorm, NeoX RoPE with f64 cos/sin.
int launch_qknorm_rope_kvstore(b200_ctx*, float* qkv, int ld, int T, int nH, int nKV, int hd, int rot_half,
                               const double* inv_freq, const float* q_norm, const float* k_norm, float eps,
                               const int32_t* row_slot, const int32_t* row_pos, KVView kv);
int launch_fold_experts(b200_ctx*, const float* eo, const float* wts, const int32_t* slot_of, int T, int k, int H, float* out);
int launch_softcap(b200_ctx*, float* x, size_t n, float cap);

// gemm.cu
// dst[T][N] (ld = ldd) = act . W^T for a Q4_K matrix; klass 0 auto, 1 exact, 2 fast. W_tiles: the same matrix tile by tile
// (launch_q4k_to_tiles) or null; the kernels that stream tiles run only when it is given.
int launch_q4k_matmul(b200_ctx*, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, int klass, const uint8_t* W_tiles = nullptr);
int launch_kq_matmul(b200_ctx*, int kind, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd);  // Q5_K (file blocks) / Q6_K (bodies + d: launch_q6k_repack)
int launch_q6k_repack(b200_ctx*, const uint8_t* raw, size_t n_blocks, uint8_t* planes);
int launch_kq_to_f16(b200_ctx*, int kind, const uint8_t* W, int N, int K, __half* out);  // dequantized fp16 copy [N][K]
int launch_act_dequant(b200_ctx*, ActQ aq, int T, int K, float* out);                    // code * scale, f32 [T][K]
// grouped form: expert e owns assignment rows [offs[e], offs[e+1]); assignment a reads activation row
// rows[a] and writes dst row a. Wptrs[e] is expert e's matrix.
int launch_q4k_matmul_grouped(b200_ctx*, const uint8_t* const* Wptrs, int n_experts, int N, int K, ActQ aq,
                              const int32_t* offs, const int32_t* rows, int max_rows_per_expert, float* dst, int ldd);
// gemm_umma.cu: fast-class tcgen05 matmul; scratch from q4k_umma_scratch_bytes
size_t q4k_umma_scratch_bytes(int max_rows, int max_k, int max_n);
// W_tiles: the tile-major copy (launch_q4k_to_tiles); when given it is what the kernel fetches and W may be null
int launch_q4k_matmul_umma(b200_ctx*, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, void* scratch,
                           size_t scratch_bytes, int* err_flag, const uint8_t* W_tiles = nullptr);
int launch_q4k_matmul_umma_swiglu(b200_ctx*, const uint8_t* W_interleaved, int N, int K, ActQ aq, int T, float* dst, int ldd, void* scratch,
                                  size_t scratch_bytes, int* err_flag, ActQ swiglu_out, bool force, bool* fused, __half* swiglu_x16 = nullptr,
                                  const uint8_t* W_tiles = nullptr);
// Q6_K (bodies + d: launch_q6k_repack) on the same pipeline: the codes are put together and scaled in the kernel
int launch_q6k_matmul_umma(b200_ctx*, const uint8_t* W_bodies, int N, int K, ActQ aq, int T, float* dst, int ldd);
int launch_kq_matmul_umma(b200_ctx*, int kind, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd);  // Q5_K (file blocks) or Q6_K
bool q6k_umma_fits(int sm_count, size_t slot_bytes, size_t scratch_bytes, int N, int K, int T);
int launch_act_to_f16(b200_ctx*, ActQ aq, int T, int K, __half* out);  // the fp16 activation tiles of quantized rows (what the producers otherwise lay out)
// gemm_small.cu: the fast class's matmul for up to 32 rows (fp16 dequant in registers, mma.sync, weights streamed once);
// uses the context's scratch like the tcgen05 matmul and takes the producers' activation tiles the same way
// its weights are kept tile by tile ([row tile of 16][super-block][16 rows][144 B]: launch_q4k_to_tiles, q4k_tiles_bytes)
int q4k_small_min_rows();
bool q4k_small_grouped_supported(const uint8_t* W_all_tiles, int N, int K);
// token rows -> expert-sorted slots: fp16 tiles + scales and group sums (what the grouped kernel below reads)
int launch_gather_rows_x16(b200_ctx*, ActQ src, const int32_t* rows_tok, int n_rows, int K, __half* x16, float* scales_out);
// routed experts on the same kernel: expert e's rows are offs[e] .. offs[e+1] of x16 / scales / dst (expert order)
int launch_q4k_matmul_small_grouped(b200_ctx*, const uint8_t* W_all_tiles, int n_experts, int N, int K, const __half* x16, const float* scales,
                                    const int32_t* offs, int n_rows, float* dst, int ldd);
size_t q4k_tiles_bytes(int N, int K);
int launch_q4k_to_tiles(b200_ctx*, const uint8_t* row_major, int N, int K, uint8_t* tiles);
int launch_q4k_matmul_small(b200_ctx*, const uint8_t* W_tiles, int N, int K, ActQ aq, int T, float* dst, int ldd);
__half* x16_next_slot(b200_ctx*);  // the scratch's other fp16 activation slot (null when the scratch has none)
int launch_interleave_rows128(b200_ctx*, const uint8_t* gate, const uint8_t* up, int F, size_t row_bytes, uint8_t* out);  // tile t: gate rows 128t.., up rows 128t..
int launch_f16w_matmul(b200_ctx*, const __half* W, int N, int K, const float* x, int T, float* dst, int ldd,
                       __half* split_scratch, int klass);
// gemm_f16_umma.cu: the tcgen05 kernel behind it (fast class, dense row counts)
size_t f16w_umma_scratch_bytes(int T, int K);
bool f16w_umma_supported(const __half* W, int N, int K);
int launch_f16w_matmul_umma(b200_ctx*, const __half* W, int N, int K, const float* x, int T, float* dst, int ldd, void* scratch,
                            size_t scratch_bytes, int* err_flag);
int launch_f32w_matmul(b200_ctx*, const float* W, int N, int K, const float* x, int T, float* dst, int ldd);
// grouped f32 form (f32 test models with routed experts): same indirection as the Q4_K grouped matmul
int launch_f32w_matmul_grouped(b200_ctx*, const float* const* Wptrs, int n_experts, int N, int K, const float* x,
                               const int32_t* offs, const int32_t* rows, int max_rows_per_expert, float* dst, int ldd);
int launch_q4k_dequant(b200_ctx*, const uint8_t* W, size_t n_blocks, float* out);
int launch_q4k_quantize(b200_ctx*, const float* w, size_t n_blocks, uint8_t* out);
int launch_synth_normal_f32(b200_ctx*, float* out, size_t n, float sigma, uint64_t seed);
int launch_synth_q4k(b200_ctx*, uint8_t* out, size_t n_blocks, float sigma, uint64_t seed);
int launch_synth_f16(b200_ctx*, __half* out, size_t n, float sigma, uint64_t seed);

// attention.cu
struct AttnScratch {
    float* partial = nullptr;  // [T][nH][max_splits][hd+2]
    int max_splits = 0;
};
size_t attn_scratch_floats(int T, int nH, int hd, int max_splits);
int attn_split_keys();
int launch_paged_attention(b200_ctx*, const float* q, int ldq, int T, int nH, int nKV, int hd, float scale, float softcap,
                           const int32_t* row_slot, const int32_t* row_pos, int max_keys, KVView kv, AttnScratch sc,
                           float* out, ActQ aq);

// gemm_umma.cu: the cached tensor map (a CUtensorMap, opaque here) of a Q4_K matrix seen as bytes [N][nSB*144], box of one
// super-block x box_rows rows; null (and ctx->err) when the driver cannot encode it
const struct CUtensorMap_st* q4k_weight_map(b200_ctx*, const uint8_t* W, int N, int nSB, int box_rows, int sb_bytes = 144);
// gemm_stream.cu: Q4_K x int8 for 4..64 rows, weights streamed through a TMA ring (exact arithmetic; split-K when splits > 1)
int launch_q4k_matmul_stream(b200_ctx*, const uint8_t* W, int N, int K, ActQ aq, int T, float* dst, int ldd, bool allow_split);
// the same kernel over experts stacked in one buffer ([n_experts*N][K]) and expert-sorted activation rows
bool q4k_stream_grouped_supported(const uint8_t* W_all, int N, int K);
int launch_q4k_matmul_stream_grouped(b200_ctx*, const uint8_t* W_all, int n_experts, int N, int K, ActQ aq, const int32_t* offs,
                                     int n_rows, int max_rows_per_expert, float* dst, int ldd);
int launch_gather_act_rows(b200_ctx*, ActQ src, const int32_t* rows_tok, int n_rows, int K, ActQ dst);

// gemm_umma.cu: sums partials nobody took into their dst (a safety net: every deferred matmul has a taker)
int flush_pending_parts(b200_ctx*);

// tp.cu: collectives over the context's communicator, on its stream
int tp_all_reduce_sum(b200_ctx*, float* buf, size_t n);
// A model's peer-visible step buffers (tensor parallel on the GPUs of one host): one device block per rank, each mapped
// into every other rank's process, so that one kernel can sum the ranks' partial o / down products over NVLink, add the
// residual, apply the next RMSNorm, quantize per 32, and store the codes into every rank's activation buffer
// (launch_tp_reduce_norm_quant). Offsets are the same on every rank.
constexpr int kTpMaxRanks = 8;
struct TpFused {
    bool on = false;
    int t = 1, rank = 0, max_rows = 0, H = 0;
    uint8_t* base = nullptr;              // this rank's block (cudaMalloc)
    uint8_t* peer[kTpMaxRanks] = {};      // every rank's block as mapped here; peer[rank] == base
    size_t off_part = 0, off_stage = 0, off_h = 0, off_codes = 0, off_scales = 0, off_row_flags = 0, off_cta_flags = 0, bytes = 0;
    unsigned seq = 0;                     // one more per launch, the same on every rank
    // the flagless form (launch_tp_reduce_norm_quant_ll): staging, codes and scales twice, used in turn; a word that has not
    // arrived yet holds a value no sender ever stores
    size_t off_stage_ll[2] = {0, 0}, off_codes_ll[2] = {0, 0}, off_scales_ll[2] = {0, 0};
    unsigned ll_calls = 0;                // the same on every rank
    int armed[2] = {0, 0};                // leading rows of each codes/scales buffer known to hold the not-arrived value
    bool use_ll = true;
    long long wait_ns = 0;                // how long a rank waits for its peers before it gives up
    long long* phase_ns = nullptr;        // measurement only: where CTA 0 stamps its clock at each stage (5 values)
    float* part() const { return reinterpret_cast<float*>(base + off_part); }
    float* h() const { return reinterpret_cast<float*>(base + off_h); }
    int8_t* codes() const { return reinterpret_cast<int8_t*>(base + off_codes); }
    float* scales() const { return reinterpret_cast<float*>(base + off_scales); }
    ActQ aq_ll(int p) const { return ActQ{reinterpret_cast<int8_t*>(base + off_codes_ll[p]), reinterpret_cast<float*>(base + off_scales_ll[p])}; }
};
void tp_fused_layout(TpFused*, int t, int rank, int max_rows, int H);
// tp.cu: allocates the block, trades the handles over the communicator and maps the peers' blocks; `on` stays false (and
// the step keeps NCCL's all-reduce) when any rank could not, which every rank learns before it returns
int tp_fused_setup(b200_ctx*, TpFused*, int max_rows, int H);
void tp_fused_teardown(b200_ctx*, TpFused*);
// tp_fused.cu. Rank r owns rows [r*ceil(T/t), ...): x = h + sum over ranks (rank order) of part; mode 0: h <- x on the
// owner, RMSNorm(x)*w quantized per 32 into every rank's codes/scales; mode 1: x into every rank's h (no norm).
// Every rank must launch it with the same T and mode, in the same order. phases (1 push, 2 reduce) and use_flags are for
// the one-GPU emulation, which runs every rank's push before any reduce and needs no flags.
int launch_tp_reduce_norm_quant(b200_ctx*, TpFused*, int T, const float* norm_w, float eps, int mode, int phases = 3, bool use_flags = true);
// The same work as mode 0 without flags or fences: the data words announce themselves. Staging and activation buffers
// start out filled with a value no sender stores (a NaN pattern for f32 words, byte -128 for codes); a reader polls a word
// until it differs and, for staging, puts the value back. Buffers alternate between calls, so a buffer is rearmed a whole
// call before it is written again. *out is the activation buffer this call filled (valid when the kernel has ended).
// phases: 1 push, 2 reduce, 4 rearm + wait for every row's codes (7 = all; split only by the one-GPU emulation).
int tp_fused_arm(b200_ctx*, TpFused*);  // fills the flagless form's buffers with the not-arrived values
// given: this rank's product as K-split partials (else the ones the matmul left pending for the block's product, if any).
// x16: also lay the rows out as the fp16 tiles the matmul after this kernel reads (local rows 0..T-1 of that slot).
int launch_tp_reduce_norm_quant_ll(b200_ctx*, TpFused*, int T, const float* norm_w, float eps, ActQ* out, int phases = 7, const Parts* given = nullptr,
                                   __half* x16 = nullptr);
int tp_all_gather_columns(b200_ctx*, const float* local, int rows, int w, float* gathered, float* full);

// attention_prefill.cu: causal attention for a run of rows of one slot at consecutive positions pos0.. (fast class)
bool prefill_attention_supported(int nH, int nKV, int hd, int block_rows);
int launch_prefill_attention(b200_ctx*, const float* q, int ldq, int nrows, int nH, int nKV, int hd, float scale, float softcap,
                             int slot, int pos0, KVView kv, float* out, int ldo);
// attention_prefill_umma.cu: the same for long runs on tcgen05 (precision: 0 = Q and P in single fp16, 1 = Q as fp16 hi + lo,
// 2 = Q and P as hi + lo)
int prefill_umma_min_rows();
int prefill_umma_precision();
bool prefill_attention_umma_supported(int nH, int nKV, int hd, int block_rows, const void* q, int ldq, const void* kpool, const void* vpool,
                                      const void* out, int ldo);
int launch_prefill_attention_umma(b200_ctx*, const float* q, int ldq, int nrows, int nH, int nKV, int hd, float scale, float softcap, int slot,
                                  int pos0, KVView kv, float* out, int ldo, int precision);

// exact class: f64 arithmetic in the CPU path's own order; scores is [T*nH][ld] f32 scratch, ld >= max_keys
int launch_paged_attention_exact(b200_ctx*, const float* q, int ldq, int T, int nH, int nKV, int hd, double scale,
                                 double softcap, const int32_t* row_slot, const int32_t* row_pos, int max_keys, KVView kv,
                                 float* scores, int ld, float* out, ActQ aq);

// sample.cu
int launch_mask_logits(b200_ctx*, float* logits, int R, int V, const int32_t* row_mask, const uint32_t* masks);
int launch_draw(b200_ctx*, const float* logits, int R, int V, const b200_draw* draws, int32_t* ids, float* scratch);
int launch_topk(b200_ctx*, const float* logits, int R, int V, int k, float invT, bool want_z, int32_t* ids, float* vals, double* z);
int launch_philox(b200_ctx*, const uint32_t* ctr, const uint32_t* key, int n, uint32_t* out);
int launch_route(b200_ctx*, const float* logits, int T, int nE, int k, int norm, int32_t* idx, float* wts);
int launch_group_experts(b200_ctx*, const int32_t* idx, int T, int k, int nE, int32_t* offs, int32_t* rows);

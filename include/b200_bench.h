/*
 * b200_bench.h — entry points of libgoinfer_b200.so that serve measurement, synthetic workloads and tests.
 *
 * None of these stands in for an interface of the reference (townsendmerino/goinfer): a host that binds the resident
 * backend needs only b200_resident.h. They exist so that benchmarks can build models and contexts without host copies,
 * time kernels on resident data, and so that tests can reach states a normal run never enters.
 */
#ifndef B200_BENCH_H
#define B200_BENCH_H

#include "b200_resident.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Counts kernels launched by this library on the context since open (bench accounting). */
int64_t b200_launch_count(b200_ctx* ctx);

/* Fills one Q4_K tensor on the device with seeded N(0, sigma) weights quantized by the library's
 * deterministic quantizer (no host copy). The reference has no fp32->Q4_K quantizer (it only reads
 * GGUF, decoder/gguf.go:1508-1537); this exists for synthetic-weight workloads. */
int b200_synth_tensor(b200_model* m, int which, int layer, int expert, int kind,
                      int rows, int cols, float sigma, uint64_t seed);
/* Fills the KV rows [0, n_pos) of a slot in every layer with seeded N(0, sigma) fp16 values (synthetic
 * prefix contexts for a decode benchmark) and maps their blocks. */
int b200_synth_kv(b200_model* m, int slot, int n_pos, float sigma, uint64_t seed);
/* Timed decode steps with everything already on the device (benchmark leg "value"): runs `steps`
 * greedy StepBatch iterations over the given sequences, feeding each drawn id back as the next token,
 * and returns the device time of the whole loop in milliseconds. */
int b200_decode_loop_device(b200_model* m, int n_seqs, const int32_t* slot, const int32_t* pos0,
                            const int32_t* first_ids, int steps, int advance_pos,
                            int32_t* ids_out /*[steps][n_seqs] or NULL*/, float* ms_out);

/* Debug tap for parity work: copies the first n floats of the residual stream ([rows][hidden]) as the latest
 * step left it after its last layer. */
int b200_debug_read_hidden(b200_model* m, float* out, int n);

/* Per-launch CUDA-event timing of kernel classes, on the stream the kernels are launched on (the role of
 * the reference's per-phase decodeTiming clocks, decoder/policy_decode.go:10-14). tag_mask bit i enables
 * class i: 0 attention split, 1 attention combine, 2 Q4_K matmul, 3 LM-head matmul, 4 norm+quant,
 * 5 RoPE+KV store, 6 SwiGLU+quant. b200_profile_read synchronizes, sums milliseconds and launches per class
 * since the last read, and clears the records. */
int b200_profile(b200_ctx* ctx, unsigned tag_mask);
int b200_profile_read(b200_ctx* ctx, double* ms_by_tag, int64_t* launches_by_tag, int n_tags);

/* Device-resident micro-benchmarks: average device milliseconds per launch over `iters` launches after
 * `warmup`, of the kernel the step would pick (or `klass`), on synthetic resident data. */
/* The read-only floor of a streaming kernel over `bytes` bytes: a grid-stride 16-byte-load kernel that only sums what it
 * reads, launched back to back over `n_copies` copies of the buffer like the matmul benchmark launches its weights. */
int b200_bench_read(b200_ctx* ctx, size_t bytes, int n_copies, int warmup, int iters, float* ms_out);
/* The Q5_K / Q6_K matmul (kind B200_K_Q5K / B200_K_Q6K) on random blocks with sane scales, cycled over copies. */
int b200_bench_kq_matmul(b200_ctx* ctx, int kind, int M, int K, int N, int n_weight_copies, int warmup, int iters, float* ms_out);
int b200_bench_q4k_matmul(b200_ctx* ctx, int M, int K, int N, int klass, int n_weight_copies,
                          int warmup, int iters, float* ms_out);
int b200_bench_f16_matmul(b200_ctx* ctx, int M, int K, int N, int klass, int warmup, int iters, float* ms_out);
int b200_bench_attention(b200_ctx* ctx, int rows, int ctx_lo, int ctx_hi, int n_heads, int n_kv_heads,
                         int head_dim, int block_rows, uint64_t seed, int warmup, int iters,
                         float* ms_out, double* kv_bytes_out);
int b200_bench_prefill_attention(b200_ctx* ctx, int rows, int pos0, int n_heads, int n_kv_heads, int head_dim,
                                 int block_rows, int warmup, int iters, float* ms_out);


/* Test hook for the bounded device-side waits. With polls > 0 and withhold_chunk >= 0 the f16 tcgen05 matmul's loader
 * stops bringing stages in at that K chunk and its MMA issuer gives a stage `polls` polls to fill; the issuer's wait then
 * runs out, the kernel raises the error flag, waits for the copies it started, frees its tensor memory and returns, and
 * the entry point that launched it reports B200_TIMEOUT. (0, -1) disarms. Nothing faults or spins without a limit. */
int b200_debug_wait_fault(b200_ctx* ctx, int polls, int withhold_chunk);

/* Test hook: dst[M][N] = a . W^T for W Q6_K given as the file's 210-byte blocks, on the tcgen05 kernel that assembles and
 * scales the six-bit codes itself (what a fast-class model runs for Q6_K tensors from 32 rows), at any M. */
int b200_debug_q6k_matmul_umma(b200_ctx* ctx, const uint8_t* w_host, const float* a_host, int M, int K, int N, float* dst_host);
/* The same for kind B200_K_Q5K (176-byte blocks) or B200_K_Q6K. */
int b200_debug_kq_matmul_umma(b200_ctx* ctx, int kind, const uint8_t* w_host, const float* a_host, int M, int K, int N, float* dst_host);

/* 1 when the model's tensor-parallel layers sum their partial products with the library's own kernel over peer memory
 * (the ranks share a host and could map one another's buffers), 0 when they call NCCL's all-reduce. */
int b200_tp_fused_active(b200_model* m);
/* Average device milliseconds of that kernel alone on T rows of the model's width, `iters` launches back to back after
 * `warmup` (mode 0: norm + quantize to every rank, 1: rows to every rank). Every rank must call it with the same arguments
 * at the same point; it overwrites the model's step scratch. B200_BAD_ARGUMENT when the kernel is not in use.
 * stage_us_out (4 floats, or NULL): from one more launch, how long the kernel's first CTA spent pushing partial rows to
 * their owners, waiting for and reducing its own rows, completing its stores, and waiting for the peers' stores. */
int b200_bench_tp_reduce(b200_model* m, int T, int mode, int warmup, int iters, float* ms_out, float* stage_us_out);

/* Test hook for the tensor-parallel reduce + residual + RMSNorm + quantize kernel on ONE GPU: `t` blocks on this device
 * stand for the ranks' peer-visible blocks, and the kernel is launched once per rank, one launch after the other, with its
 * cross-rank waits left out (kernels that wait for one another must not share a GPU). parts [t][T][H] are the ranks'
 * partial products, h [T][H] the residual rows every rank starts from, w [H] the norm weight. mode 0: every rank's view of
 * the codes [t][T][H] and scales [t][T][2*H/32] and its residual rows h_out [t][T][H] (updated on the owner only);
 * mode 1: h_out holds the summed rows on every rank; mode 2: mode 0's work in the form without flags (words that announce
 * themselves), three calls in a row on the same inputs so that both buffer pairs are used, rearmed and used again; with
 * n_kparts > 0 (mode 2 only) parts is [t][n_kparts][T][H]: each rank's product as the K-split partials a matmul leaves
 * for its consumer, which the kernel adds in split order. */
int b200_debug_tp_reduce_emulated(b200_ctx* ctx, int t, int T, int H, const float* parts, const float* h, const float* w,
                                  float eps, int mode, int n_kparts, int8_t* codes_out, float* scales_out, float* h_out);

#ifdef __cplusplus
}
#endif
#endif /* B200_BENCH_H */

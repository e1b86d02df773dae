/*
 * b200_resident.h — C ABI of the B200 (sm_100a) resident backend for goinfer's ragged batched
 * decode / varlen-prefill step.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an int status and never
 * throws, aborts or calls back into the host. A cgo-free Go host binds these with dlopen/dlsym; the
 * Python package binds them with ctypes. Host buffers passed in stay the caller's and are only read
 * (or written, for outputs) during the call.
 *
 * Each declaration cites the interface of the reference (townsendmerino/goinfer, paths relative to its
 * root) that it stands in for.
 */
#ifndef B200_RESIDENT_H
#define B200_RESIDENT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------------------------------- */
#define B200_OK            0
#define B200_DECLINED      1 /* the model cannot be built resident (decoder.DeclineResident, decoder/residency.go:240-255) */
#define B200_KV_POOL_FULL  2 /* decoder.ErrKVPoolFull: every row's blocks were mapped first and nothing was written (decoder/mc3_batch.go:492-498) */
#define B200_BAD_ARGUMENT  3
#define B200_CUDA_ERROR    4
#define B200_TIMEOUT       5 /* a bounded device-side wait gave up; the context stays usable */
#define B200_NCCL_ERROR    6

/* ---- tensor names (b200_upload_tensor `which`) ----------------------------------------------------
 * The weights a dense or routed-expert decoder layer carries, as decoder.BackendView.Weights() hands
 * them to a resident build (decoder/backend_view.go:120-302). */
#define B200_T_EMBED       0  /* [vocab, hidden]  F32 | F16                                   */
#define B200_T_FINAL_NORM  1  /* [hidden]         F32                                         */
#define B200_T_LM_HEAD     2  /* [vocab, hidden]  F32 | F16 | Q4K                             */
#define B200_T_ATTN_NORM   3  /* [hidden]         F32                                         */
#define B200_T_WQ          4  /* [n_heads*head_dim, hidden]                                   */
#define B200_T_WK          5  /* [n_kv_heads*head_dim, hidden]                                */
#define B200_T_WV          6
#define B200_T_WO          7  /* [hidden, n_heads*head_dim]                                   */
#define B200_T_Q_NORM      8  /* [head_dim] F32, per-head RMSNorm of q (decoder/program_cpu.go:351-364) */
#define B200_T_K_NORM      9
#define B200_T_FFN_NORM    10
#define B200_T_GATE        11 /* [ffn, hidden]                                                */
#define B200_T_UP          12
#define B200_T_DOWN        13 /* [hidden, ffn]                                                */
#define B200_T_ROUTER      14 /* [n_experts, hidden] F32 only (decoder/weightmat.go:61-64)    */
#define B200_T_EXP_GATE    15 /* [moe_ffn, hidden] per expert                                 */
#define B200_T_EXP_UP      16
#define B200_T_EXP_DOWN    17 /* [hidden, moe_ffn] per expert                                 */

/* ---- weight kinds --------------------------------------------------------------------------------- */
#define B200_K_F32 0
#define B200_K_F16 1
#define B200_K_Q4K 2 /* GGUF Q4_K super-blocks, 144 bytes per 256 weights, row-major [rows][cols/256][144]
                        (decoder/gguf.go:1508-1537; device twin backend/cuda/actgroup.cu:311-355). A Q4K
                        matrix multiplies per-32-group int8 activations (backend/cuda/actgroup.cu:32-54). */
#define B200_K_Q5K 3 /* GGUF Q5_K super-blocks, 176 bytes per 256 weights (d, dmin, 12 scale bytes, qh[32], qs[128]), as in
                        the file; x per-32 int8 activations (backend/cuda/actgroup.cu:77-143). */
#define B200_K_Q6K 4 /* GGUF Q6_K super-blocks, 210 bytes per 256 weights (ql[128], qh[64], 16 int8 sub-scales, d), uploaded as in
                        the file; the device keeps each block's first 208 bytes row by row (16-byte aligned) and the d values
                        behind them; x per-32 int8 activations (the W6A8 product, backend/cuda/actgroup.cu:145-205).
                        The Q5_K / Q6_K matmuls are held to the reference's own bar for them: within 1e-5 of sum |w*a| of the
                        f64 product of the dequantized row (backend/cuda/kernels/kso1c_kernels_test.go:146-151). q|k|v and
                        gate|up may mix Q4_K, Q5_K and Q6_K parts, as Q4_K_M files do. */
#define B200_K_I8 5  /* int8 rows with one f32 scale per row (W8A8: what the reference keeps the embedding table, the LM head
                        and every projection without raw K-quant bytes as under q4k, decoder/weightmat.go:74-83): the upload is
                        [rows][cols] int8 followed by rows f32 scales. dst[n] = (sum over groups of 32: aS_g * idot_g) * wScale[n]
                        (backend/cuda/actgroup.cu:287-297,417-432); an embedding row is code * wScale[row]. Held to the reference's
                        GEMV bar: 1e-5 of sum |w*a| against the f64 product (backend/cuda/kernels/actgroup_kernel_test.go:305-364). */

/* ---- draw kinds ----------------------------------------------------------------------------------- */
#define B200_DRAW_LOGITS 0 /* no draw: the row's logits are returned (BatchSeq.Draw == nil)          */
#define B200_DRAW_GREEDY 1 /* BatchDraw.Greedy: first maximal index (internal/runtime/sampling/sampler.go:485-518) */
#define B200_DRAW_MINP   2 /* min-p retained set + CDF walk with the caller's uniform `u`
                              (sampler.go:586-724, drawFiltered :442-458)                            */
#define B200_DRAW_GUMBEL 3 /* temperature-only sampling by Gumbel-max over Philox4x32-10 noise: argmax_i(l_i*invT + G_i)
                              (internal/runtime/sampling/sampler_gumbel.go:37-64,104-110; philox.go:21-36;
                              device twin backend/cuda/gumbel.cu). For this kind `temperature` carries invT =
                              float32(1/T) as the host sampler computed it, the 8 bytes of {min_p, _pad} carry the
                              64-bit seed and the 8 bytes of `u` the 64-bit draw index (Sampler.NextDraw); copy them
                              in with memcpy. */

/* ---- kernel classes (b200_model_cfg.kernel_class) -------------------------------------------------
 * The reference separates exact kernels from fast, non-bit-identical ones by a row floor
 * (resident.Caps.HasFastPrefill / FastPrefillFloor, decoder/resident/forward.go:119-146). */
#define B200_CLASS_AUTO  0 /* fast class: tensor-core flash-decode and tiled prefill attention with fp32 online softmax; Q4_K
                              matmuls by row count: integer-dot kernels with the CPU path's per-group formula at small row
                              counts (f32 sums folded in another order), and from 33 rows a tcgen05 matmul over the
                              dequantized fp16 weights and fp16(code * scale) activations with fp32 accumulation.
                              Held to the logit bar on shallow models and to cosine >= 0.995 / relative L2 <= 0.10
                              (decoder/selftest_gpu.go:30-35) at depth. */
#define B200_CLASS_EXACT 1 /* exact class: attention in f64 in the CPU path's own order (decoder/forwardn.go:379-499)
                              and one ascending f32 chain per matmul output at every row count, so a row's bits do
                              not depend on its batch (decoder/resident/subsystems.go:102-110)             */

typedef struct b200_ctx b200_ctx;
typedef struct b200_model b200_model;

/* Model shape and runtime plan. Mirrors what a resident build reads through BackendView: Dims(),
 * NormEps(), AttnScale(), HasQKNorm(), AttnLogitSoftcap(), MoE() (decoder/backend_view.go:17-76). */
typedef struct {
    int32_t hidden, n_layers, n_heads, n_kv_heads, head_dim, ffn, vocab;
    int32_t rotary_dim;      /* rotated dims per head (== head_dim for full rotary)                    */
    int32_t qk_norm;         /* 1: per-head RMSNorm of q and k before RoPE                             */
    int32_t n_experts, top_k, norm_topk, moe_ffn; /* n_experts == 0: dense gated FFN                   */
    int32_t kv_block_rows;   /* positions per KV block (16 or 64)                                      */
    int32_t kv_pool_blocks;  /* blocks in the pool, the null block 0 included                          */
    int32_t n_slots;         /* KV slots (KVSubsystem.KVSlots, decoder/resident/subsystems.go)         */
    int32_t ctx_cap;         /* Caps.ContextCap: positions per slot                                    */
    int32_t max_rows;        /* most packed rows one step carries                                      */
    int32_t tp_rank, tp_size;/* tensor-parallel rank/size; 1 = replica                                 */
    int32_t kernel_class;    /* B200_CLASS_*                                                           */
    int32_t fast_floor;      /* rows from which the fast class runs (0 = library default)              */
    int32_t kv_dtype;        /* 0 = fp16 paged cache (the only kind this backend builds); 1 = f32, which
                                this backend declines (decoder.DeclineResident) and only the CPU oracle runs */
    float rms_eps, rope_theta;
    float attn_scale;        /* 0 = 1/sqrt(head_dim)                                                   */
    float attn_softcap;      /* 0 = off; else cap*tanh(s/cap) (decoder/attention.go:287-295)           */
    float final_softcap;     /* 0 = off                                                                */
    float embed_scale;       /* 0 or 1 = none (decoder/cpu_batch.go:176-186)                           */
} b200_model_cfg;

/* Per-sequence draw of a step (resident.BatchDraw, decoder/resident/forward.go:43-52). */
typedef struct {
    int32_t kind;        /* B200_DRAW_*                                                               */
    float temperature;   /* min-p only; <= 0 reads as 1                                               */
    float min_p;         /* min-p only; > 1 is clamped to 1 (sampler.go:129-139)                      */
    float _pad;
    double u;            /* min-p only: the uniform in [0,1) the host sampler drew for this token     */
} b200_draw;

/* resident.Caps (decoder/resident/forward.go:119-146). */
typedef struct {
    int32_t context_cap, kv_slots, batch_lo, batch_hi; /* BatchStepRange = (batch_lo, batch_hi)       */
    int32_t has_fast_prefill, fast_prefill_floor, tail_min_rows, batch_greedy_draw;
    int64_t weight_bytes, kv_bytes, scratch_bytes;
} b200_caps;

/* decoder.ResidentBatchStats (decoder/mc3_batch.go:82-94) plus device-side counters. */
typedef struct {
    int64_t steps, rows, prefill_rows, kernel_launches, kv_blocks_in_use, kv_pool_full;
    double last_step_device_ms;
} b200_stats_t;

/* ---- context -------------------------------------------------------------------------------------- */
/* Opens device `device_ordinal`. `stream` is a cudaStream_t the library launches on; NULL makes the
 * library create its own. Replaces gpudev.Open (backend/cuda/internal/gpudev/cuda.go:177-181). */
int b200_open(int device_ordinal, void* stream, b200_ctx** out);
void b200_close(b200_ctx* ctx);
/* Text of the last non-OK status on this context (the Go shim turns it into an error value). */
const char* b200_last_error(b200_ctx* ctx);
/* Tensor parallel (the 70B-class configuration: q/k/v/gate/up split by output rows, o/down by input columns, the KV
 * cache by kv head, an all-reduce of the partial [rows][hidden] products after the o and down projections, the LM head
 * split by vocabulary slice and gathered). No counterpart in the reference's single-GPU CUDA backend. One process per GPU:
 * rank 0 makes the id (b200_tp_unique_id, 128 bytes), the host carries it to the other ranks, every rank calls
 * b200_tp_init on its context, then creates its model with tp_rank / tp_size set and its own share of n_heads,
 * n_kv_heads and ffn in the configuration (vocab stays whole; the LM head tensor is this rank's [vocab/tp_size][hidden]
 * slice). NCCL is opened with dlopen at the first of these calls. Every rank must make the same step calls in the same
 * order. */
int b200_tp_unique_id(b200_ctx* ctx, void* id_out, size_t bytes);
int b200_tp_init(b200_ctx* ctx, const void* id, size_t bytes, int rank, int size);
int b200_tp_destroy(b200_ctx* ctx);

/* ---- model build: ResidencyBackend.BuildResident (decoder/residency.go:208-210) -------------------- */
int b200_model_create(b200_ctx* ctx, const b200_model_cfg* cfg, b200_model** out);
/* Copies one tensor to the device. `layer` is -1 for model-level tensors; `expert` is -1 unless `which`
 * is an expert tensor. The host buffer stays the caller's. */
int b200_upload_tensor(b200_model* m, int which, int layer, int expert, int kind,
                       int rows, int cols, const void* host, size_t bytes);
/* Per-layer RoPE inverse frequencies (BackendView.RopeInvFreq, decoder/residency.go:604-619). `layer`
 * -1 sets every layer. Without a call the table is theta^(-2d/rotary_dim) (decoder/ropescale.go:285-290). */
int b200_set_rope_inv_freq(b200_model* m, int layer, const double* inv_freq, int n);
/* Plans the KV pool and scratch, fuses projection groups, fills Caps. */
int b200_model_finalize(b200_model* m, b200_caps* out);
void b200_model_free(b200_model* m);

/* ---- KVSubsystem (decoder/resident/subsystems.go; backend/cuda/kvpool.go:16-76) --------------------- */
int b200_kv_slots(b200_model* m);
/* Releases a slot's blocks and rewinds it to position 0 (ResidentForward.Reset on that slot). */
int b200_reset_slot(b200_model* m, int slot);
int b200_reset(b200_model* m);
/* Copies a slot's block table (ctx_cap / kv_block_rows entries, 0 = unmapped) to `out`. */
int b200_block_table(b200_model* m, int slot, int32_t* out, int n);
/* ResidentForward.UploadKV (decoder/resident/forward.go:5-33): rows [base, base+n) of one layer, f32
 * [n][n_kv_heads*head_dim], rounded to the cache's fp16. */
int b200_upload_kv(b200_model* m, int slot, int layer, int base, int n, const float* keys, const float* vals);

/* ---- the step: DecodeSubsystem.StepBatch / StepRagged (decoder/resident/subsystems.go:102-117;
 *      wire types decoder/resident/forward.go:35-84; existing implementation backend/cuda/batchstep.go:49-182)
 *
 * n_seqs sequences; sequence i owns n_rows[i] packed rows at positions pos[i], pos[i]+1, ... of KV slot
 * slot[i] (slots distinct). prefill_prompt_len[i] > 0 marks a prefill chunk (at most one, first, no draw,
 * inside its prompt; prefill_last[i] iff it ends it). Inputs are either `embs` (packed rows x hidden f32,
 * the reference's host embedResident rows) or `token_ids` (device table gather; allowed where the lookup
 * is a plain table row, decoder/residency.go:1053-1131); exactly one is non-NULL.
 * draws may be NULL (all rows return logits). mask_index[i] >= 0 selects row mask_index[i] of `logit_mask`
 * ([n_masks][ceil(vocab/32)] words, bit set = token allowed; cleared => logit = -inf before the draw,
 * constrain/constrain.go:233-267).
 *
 * Outputs: logits_out receives, packed in order, one [vocab] row for every row that returns logits
 * (every row of a sequence without a draw; for a draw sequence every row but its last; for a prefill chunk only the
 * final row of a Last pass). ids_out[i] is the drawn id or -1. n_logit_rows_out, if not NULL, receives
 * the number of rows written.
 * StepBatch is this call with n_rows[i] == 1 for all i. */
int b200_step_ragged(b200_model* m, int n_seqs, const int32_t* slot, const int32_t* pos,
                     const int32_t* n_rows, const int32_t* prefill_prompt_len,
                     const uint8_t* prefill_last, const float* embs, const int32_t* token_ids,
                     const b200_draw* draws, const int32_t* mask_index, const uint32_t* logit_mask,
                     int n_masks, float* logits_out, int32_t* ids_out, int32_t* n_logit_rows_out);

/* ResidentForward.Forward / DecodeSubsystem.ForwardArgmax / ForwardNoLogits on one slot
 * (decoder/resident/forward.go:5-33): one row at `pos`. out_kind: 0 logits, 1 argmax id, 2 nothing. */
int b200_forward(b200_model* m, int slot, const float* emb, int token_id, int pos, int out_kind,
                 float* logits_out, int32_t* id_out);
/* DecodeSubsystem.ForwardTopK (decoder/resident/subsystems.go:40-48): one row at `pos`, only its k best logits (and Z when
 * z_out is not NULL) come back instead of the vocabulary-wide row. inv_temperature = float32(1/T). */
int b200_forward_topk(b200_model* m, int slot, const float* emb, int token_id, int pos, int k, float inv_temperature,
                      int32_t* ids_out, float* logits_out, double* z_out);
/* Prefix reuse over paged blocks (KVSubsystem.CopyKV; backend/cuda/kvpool.go:16-27,436-536): dst_slot is reset and then
 * holds the first n_rows rows of src_slot. Whole blocks are shared by reference (a block counts the tables that name it
 * and goes back to the pool when the last one lets go); the rows of a partial last block are copied into a block of
 * dst's own. A slot that later writes into a block another table also names first takes a block of its own and keeps
 * the rows before the write (copy on write), so no slot ever writes a block another slot reads.
 * B200_KV_POOL_FULL (nothing changed) when the one block this may take is not there. */
int b200_copy_kv(b200_model* m, int dst_slot, int src_slot, int n_rows);
/* PrefillSubsystem.PrefillLast (decoder/resident/subsystems.go): n rows from start_pos on one slot, logits of the last row. */
int b200_prefill_last(b200_model* m, int slot, int n, const float* embs, const int32_t* token_ids,
                      int start_pos, float* logits_out);

/* ---- the device batch: admission and retirement applied on the device ------------------------------------------------
 * The reference's serve loop admits a request when a session is free and retires it when its generation ends
 * (scheduler.Admission, internal/runtime/scheduler/admission.go:60-122), and its coalescer packs every step's batch on the
 * host (decoder/mc3_batch.go:358-446). Here a fixed set of SEATS lives on the device: seat i is bound to KV slot
 * first_slot + i; an empty seat runs a throw-away row on `park_slot`, so every step has the same shape and a finished
 * sequence's KV stays in its slot (a follow-up turn continues it, or it serves as a prefix donor).
 *   b200_batch_open   binds the seats (n_seats <= max_rows; park_slot outside the seats' slots; max_steps bounds a run).
 *   b200_batch_admit  after the host has prefilled the seat's slot up to `pos` (b200_prefill_last, b200_step_ragged,
 *                     b200_copy_kv): the sequence continues at `pos` by feeding `token`, for at most `max_new` tokens or
 *                     until it draws `eos_id` (-1: none). The blocks it can still take are reserved against the pool:
 *                     B200_KV_POOL_FULL (nothing changed) when they are not there.
 *   b200_batch_retire takes a sequence off its seat (a cancelled request).
 *   b200_batch_run    applies the commands queued since the last run, in order, then decodes `steps` greedy steps for all
 *                     seats: ids are fed back and positions advance on the device, a seat retires itself when its sequence
 *                     ends, and nothing is packed or uploaded per step. events_out receives one record of four ints per
 *                     live seat and step, in step order then seat order: seat, drawn id, the position that was decoded,
 *                     flags (bit 1: the seat retired after this step). Each record's id is what StepBatch would have
 *                     drawn for that sequence at that position with a Greedy draw.
 * Between runs every other entry point may be used on any slot but a live seat's. */
int b200_batch_open(b200_model* m, int n_seats, int first_slot, int park_slot, int max_steps);
int b200_batch_admit(b200_model* m, int seat, int pos, int token, int max_new, int eos_id);
int b200_batch_retire(b200_model* m, int seat);
int b200_batch_run(b200_model* m, int steps, int32_t* events_out, int max_events, int32_t* n_events_out);
int b200_batch_close(b200_model* m);

int b200_stats(b200_model* m, b200_stats_t* out);
/* ---- operator-level entry points (host buffers in, host buffers out) -------------------------------
 * The reference exposes its matmul as Backend.MatmulBT(a, b, dst, M, K, N) (decoder/backend.go:23-32)
 * and tests kernels against host twins (backend/cuda/kernels/actgroup_kernel_test.go). These run the
 * same device kernels the step uses on caller-supplied data. */
/* Per-32 int8 activation quantizer (backend/cuda/actgroup.cu:32-54): x [rows][k] -> codes int8
 * [rows][k], scales [rows][2*k/32] (k/32 scales then k/32 group sums). */
int b200_op_quant_g32(b200_ctx* ctx, const float* x, int rows, int k, int8_t* codes, float* scales);
/* Q4_K super-blocks -> f32 weights, w = d*sc*q - dmin*m (backend/cuda/kernels/ks_a1_test.go:117-131). */
int b200_op_q4k_dequant(b200_ctx* ctx, const uint8_t* w, int rows, int cols, float* out);
/* dst[M][N] = a[M][K] . W^T, W Q4_K [N][K]; activations quantized per 32 (actgroup.cu:311-355).
 * klass: 0 = library choice by M (fast class), 1 = exact kernels, 2 = the fast class's tcgen05 fp16 kernel at any M; for kernel
 * comparisons: 3 = the register-direct integer kernels, 4 = the streaming integer kernel in its one-chain form (the exact
 * class's bits), 5 = the small-batch fp16 kernel (M <= 32), 6 = the streaming integer kernel with K split, 7 = the fast class
 * given only the tile-major copy of W, as a fast-class model keeps it after b200_finalize_weights. */
int b200_op_q4k_matmul(b200_ctx* ctx, const uint8_t* w, const float* a, int M, int K, int N, int klass,
                       float* dst);
/* dst[M][N] = a[M][K] . w[N][K]^T over f16 weights (the LM head's kind, decoder/forwardn.go:800-831): klass 0 picks by
 * row count as a fast-class step does, 1 the accurate small-batch kernel, 2 forces the tcgen05 kernel. */
int b200_op_f16_matmul(b200_ctx* ctx, const uint16_t* w, const float* a, int M, int K, int N, int klass, float* dst);
/* fp32 -> Q4_K with the library's deterministic quantizer (the reference only reads Q4_K, decoder/gguf.go:1508-1537); out is
 * rows*cols/256*144 bytes. */
int b200_op_q4k_quantize(b200_ctx* ctx, const float* w, int rows, int cols, uint8_t* out);
/* RMSNorm rows (decoder/rmsnorm.go:29-92). */
int b200_op_rmsnorm(b200_ctx* ctx, const float* x, const float* w, int rows, int dim, float eps, float* out);
/* softmax -> top-k router (decoder/mlp.go:130-184, 370-440): logits [rows][n_experts] -> idx, wts [rows][k]. */
int b200_op_route(b200_ctx* ctx, const float* logits, int rows, int n_experts, int k, int norm_topk,
                  int32_t* idx, float* wts);
/* Draw over logits rows with optional masks (sampler.go:485-518, 586-724). */
int b200_op_draw(b200_ctx* ctx, const float* logits, int rows, int vocab, const b200_draw* draws,
                 const int32_t* mask_index, const uint32_t* logit_mask, int n_masks, int32_t* ids);
/* The k best logits of each row ordered (logit descending, token id ascending; -0 and +0 tie) and, when z_out is not
 * NULL, Z = sum exp((l - max) * inv_temperature) over the whole row (decoder/resident/forward.go:91-96; device twin
 * backend/cuda/topk.cu). 1 <= k <= min(1024, vocab). */
int b200_op_topk(b200_ctx* ctx, const float* logits, int rows, int vocab, int k, float inv_temperature,
                 int32_t* ids_out, float* logits_out, double* z_out);
/* Philox4x32-10 (internal/runtime/sampling/philox.go:21-36) on the device: n (counter[4], key[2]) pairs -> out[4] each. */
int b200_op_philox(b200_ctx* ctx, const uint32_t* ctr, const uint32_t* key, int n, uint32_t* out);
/* Paged decode attention over caller-supplied contiguous K/V (f32 rounded to fp16 on upload):
 * q [rows][n_heads*head_dim]; row r attends keys [0, n_keys[r]) of its own K/V
 * (decoder/forwardn.go:295-501, acc64 branch). */
int b200_op_attention(b200_ctx* ctx, const float* q, const float* k, const float* v, const int32_t* n_keys,
                      int rows, int max_keys, int n_heads, int n_kv_heads, int head_dim, float scale,
                      float softcap, int block_rows, int klass /* 0 fast fp32, 1 exact f64 */, float* out);

/* Causal attention of a prefill run: `rows` query rows of one sequence at positions pos0 .. pos0+rows-1 over its
 * K/V [pos0+rows][n_kv_heads*head_dim] (f32 rounded to fp16 on upload, paged); row j attends keys 0 .. pos0+j
 * (the per-row loop of decoder/program_cpu_n.go:497-515 over decoder/forwardn.go:295-501). Fast class. */
int b200_op_prefill_attention(b200_ctx* ctx, const float* q, const float* k, const float* v, int rows, int pos0,
                              int n_heads, int n_kv_heads, int head_dim, float scale, float softcap,
                              int block_rows, float* out);

/* silu(x . Wgate^T) * (x . Wup^T), quantized per 32: codes [M][F], scales then group sums [M][2*F/32]. w = Q4_K gate rows then up
 * rows ([2F][K]). Fast class. mode 0: tcgen05 matmul, then the SwiGLU + quantizer kernel; mode 1: gate|up rows interleaved by 128 and
 * the SwiGLU + quantizer in the matmul's epilogue; mode 2: interleaved rows, separate kernels. The three give the same bytes. */
int b200_op_gate_up_swiglu(b200_ctx* ctx, const uint8_t* w_host, const float* x_host, int M, int K, int F, int mode,
                           int8_t* codes_out, float* scales_out);

/* dst[M][N] = x . W^T for W of kind B200_K_Q5K / B200_K_Q6K given as the file's blocks ([N][K/256][176 or 210] bytes) and f32
 * x [M][K], quantized per 32 on the device like the step does. */
int b200_op_kq_matmul(b200_ctx* ctx, int kind, const uint8_t* w_host, const float* x_host, int M, int K, int N, float* dst_host);

/* Paged decode attention that allocates nothing. No counterpart in the reference (its backends allocate their split
 * buffers when a model is built); it exists for hosts that cannot allocate when they need attention: a serving process
 * whose device memory was handed out once at start-up and is owned by its own pool, or a plug-in living under another
 * program's "no device allocation after init" rule, where a cudaMalloc in the step would break the host's memory budget.
 *
 * All pointers are DEVICE pointers owned by the caller: q [rows][ldq] f32 (query heads of row r at q + r*ldq; 8-byte
 * aligned, ldq even), row_slot/row_pos [rows] (the block-table row and the position, i.e. keys-1, of each query),
 * k_pool/v_pool the fp16 pools laid out [block][kv_head][row_in_block][head_dim] (16-byte aligned), block_table
 * [n_table_rows][max_blocks], out [rows][n_heads*head_dim] f32 (8-byte aligned). scale 0 means 1/sqrt(head_dim). Work is
 * queued on the context's stream; the caller synchronizes that stream before reading `out`. The context's device is made
 * current for the length of the call and the caller's own device is current again when it returns.
 *
 * Preconditions the library cannot check (the arrays live on the device): 0 <= row_pos[r] < max_keys, row_slot[r] names a
 * row of block_table, and every table entry of a row's keys names a block of the pools. A row_pos[r] >= max_keys reads
 * nothing outside the table or the scratch, but that row's output is meaningless.
 *
 * The split partials live in one fixed 16 MiB device array inside the library (every GPU that loads the library holds
 * it until the process exits). Limits: head_dim 64 or 128, n_heads/n_kv_heads in {1,2,4,8}, block_rows a positive multiple
 * of 16, max_blocks * block_rows >= max_keys, and rows * n_heads * ceil(max_keys/512) * (head_dim+2) * 4 bytes <= 16 MiB
 * (e.g. 32 heads of 128: 252 rows at 2048 keys, 63 rows at 8192 keys); anything else returns B200_BAD_ARGUMENT with the
 * sizes in b200_last_error.
 * The first call on a device looks up the array's address (no allocation); make that first call before starting any
 * stream capture. The array is shared by every call and keeps the previous call's bytes; nothing in it needs clearing,
 * but two calls whose kernels overlap on the GPU (different streams or contexts of one device) race on it:
 * serialize them. The entry point calls no cudaMalloc, cudaFree or other allocating routine. */
int b200_attention_noalloc(b200_ctx* ctx, const float* q, int ldq, int rows, int n_heads, int n_kv_heads, int head_dim,
                           float scale, float softcap, const int32_t* row_slot, const int32_t* row_pos, int max_keys,
                           const void* k_pool, const void* v_pool, const int32_t* block_table, int max_blocks,
                           int block_rows, float* out);

#ifdef __cplusplus
}
#endif
#endif /* B200_RESIDENT_H */

// engine.cu — the resident model and its ragged step behind the C ABI of include/b200_resident.h.
//
// What the reference does on the host per step — the slot/position arrays, the per-slot block tables and
// their upload (backend/cuda/batchstep.go:306-381, kvpool.go:16-76), the coalescer's per-token embedding
// rows (decoder/mc3_batch.go:358-366) — lives on the device here: a step uploads one small packed
// descriptor (per-sequence slot, position, row count, token ids), and prepare_step_kernel maps KV blocks
// from the device free list, builds the row->sequence / row->position arrays and the sequence offsets.
// The host keeps only counters (rows stored and blocks mapped per slot, free blocks), which is enough to
// refuse a step with B200_KV_POOL_FULL before anything is launched (decoder/mc3_batch.go:492-498).
//
// Layer program (decoder/program.go:143-166): norm -> QKV -> [QK norm] -> RoPE -> KV append -> attention
// -> O -> residual -> norm -> gated FFN | routed experts -> residual; final norm + LM head on the rows that
// return logits or draw (decoder/forwardn.go:800-831).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace {

constexpr int kKindMixed = 100;  // a projection group whose parts are K-quants of different kinds, multiplied part by part

struct DevMat {
    int kind = -1, rows = 0, cols = 0;
    void* p = nullptr;
    size_t bytes = 0;
    DevMat* seg[3] = {nullptr, nullptr, nullptr};  // kKindMixed: the parts, in row order
    int n_seg = 0;
    __half* f16 = nullptr;  // Q5_K / Q6_K, fast class: a dequantized copy for the tensor-core matmul at dense row counts
    // Q4_K, fast class: the matrix tile by tile (launch_q4k_to_tiles). Every fast-class kernel reads this layout, so the
    // row-major matrix is dropped once it exists (p == nullptr) unless a debugging switch asks for the older kernels.
    uint8_t* tiles = nullptr;
    bool present() const { return kind >= 0 && (p || n_seg > 0 || tiles); }
};

// the kinds that multiply the per-32 int8 activations
bool is_kquant(int kind) { return kind == B200_K_Q4K || kind == B200_K_Q5K || kind == B200_K_Q6K || kind == B200_K_I8 || kind == kKindMixed; }
// the kinds multiplied by the dp4a lanes of kquant.cu (and, from 32 rows in the fast class, through an fp16 copy)
bool is_lane_kind(int kind) { return kind == B200_K_Q5K || kind == B200_K_Q6K || kind == B200_K_I8; }

size_t mat_bytes(int kind, size_t rows, size_t cols) {
    if (kind == B200_K_F32) return rows * cols * 4;
    if (kind == B200_K_F16) return rows * cols * 2;
    if (kind == B200_K_Q5K) return rows * cols / 256 * 176;
    if (kind == B200_K_Q6K) return rows * cols / 256 * 210;
    if (kind == B200_K_I8) return rows * cols + rows * 4;
    return rows * cols / 256 * 144;
}

struct LayerW {
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    DevMat wq, wk, wv, wo, gate, up, down, router;
    std::vector<DevMat> eg, eu, ed;
    DevMat qkv, gu;                         // fused at finalize
    bool gu_il = false;                     // gu's rows are gate|up interleaved by 128 (fast class, Q4_K): tile t = gate rows 128t.. then up rows 128t..
    std::vector<DevMat> egu;                // per expert gate|up
    const uint8_t** d_egu_ptrs = nullptr;   // device arrays of expert matrix pointers
    uint8_t *egu_all = nullptr, *ed_all = nullptr;  // Q4_K experts stacked: [n_experts][2F][.] and [n_experts][H][.]
    uint8_t *egu_tiles = nullptr, *ed_tiles = nullptr;  // fast class: the stacks tile-major (every expert's matrix as launch_q4k_to_tiles lays it), the row-major stacks released
    const uint8_t** d_ed_ptrs = nullptr;
    double* inv_freq = nullptr;             // device, [rot_half]
    std::vector<double> h_inv_freq;
};

__global__ void init_pool_kernel(int32_t* free_stack, int32_t* free_count, int blocks, int32_t* table, size_t table_n,
                                 int32_t* slot_mapped, int n_slots, int32_t* refs) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (size_t)blocks) refs[i] = 0;
    // take pops the last entry: ascending ids 1..blocks-1 (backend/cuda/kvpool.go:50-64)
    if (i < (size_t)blocks - 1) free_stack[i] = (int32_t)(blocks - 1 - i);
    if (i < table_n) table[i] = 0;
    if (i < (size_t)n_slots) slot_mapped[i] = 0;
    if (i == 0) *free_count = blocks - 1;
}

__global__ void reset_slot_kernel(int32_t* free_stack, int32_t* free_count, int32_t* table, int max_blocks,
                                  int32_t* slot_mapped, int slot, int32_t* refs) {
    // single thread: unref in table order, a block whose last reference goes is appended (kvpool.go:58-64,78-84)
    int n = slot_mapped[slot], fc = *free_count;
    int32_t* t = table + (size_t)slot * max_blocks;
    for (int b = 0; b < n; b++) {
        if (t[b] && --refs[t[b]] <= 0) {
            refs[t[b]] = 0;
            free_stack[fc++] = t[b];
        }
        t[b] = 0;
    }
    *free_count = fc;
    slot_mapped[slot] = 0;
}

// dst (empty) takes the first n_full blocks of src by reference and, when tail is set, a block of its own for the rows
// of src's next block that it keeps (the caller copies them): backend/cuda/kvpool.go:511-536 (kvShare).
__global__ void share_prefix_kernel(int32_t* table, int max_blocks, int32_t* slot_mapped, int32_t* refs, int32_t* free_stack,
                                    int32_t* free_count, int src, int dst, int n_full, int tail) {
    const int32_t* st = table + (size_t)src * max_blocks;
    int32_t* dt = table + (size_t)dst * max_blocks;
    for (int b = 0; b < n_full; b++) {
        dt[b] = st[b];
        refs[st[b]]++;
    }
    int fc = *free_count;
    if (tail) {
        const int32_t id = free_stack[--fc];
        refs[id] = 1;
        dt[n_full] = id;
    }
    *free_count = fc;
    slot_mapped[dst] = n_full + (tail ? 1 : 0);
}

// A slot about to write into blocks [b_lo, b_hi) that other tables also name takes blocks of its own first
// (kvpool.go:436-477, kvMap): the caller copies the rows it keeps.
__global__ void cow_kernel(int32_t* table, int max_blocks, int32_t* refs, int32_t* free_stack, int32_t* free_count, int slot, int b_lo,
                           int b_hi) {
    int32_t* t = table + (size_t)slot * max_blocks;
    int fc = *free_count;
    for (int b = b_lo; b < b_hi; b++) {
        const int32_t old = t[b];
        if (old && refs[old] > 1) {
            const int32_t id = free_stack[--fc];
            refs[id] = 1;
            refs[old]--;
            t[b] = id;
        }
    }
    *free_count = fc;
}

// rows [0, rows) of block `from` -> block `to`, every kv head, K and V of one layer (exact copies)
__global__ void copy_block_rows_kernel(__half* kpool, __half* vpool, int from, int to, int rows, int nKV, int block_rows, int hd) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, n = (size_t)nKV * rows * hd;
    if (i >= n) return;
    const int e = (int)(i % hd), r = (int)((i / hd) % rows), kvh = (int)(i / ((size_t)hd * rows));
    const size_t so = (((size_t)from * nKV + kvh) * block_rows + r) * hd + e, dn = (((size_t)to * nKV + kvh) * block_rows + r) * hd + e;
    kpool[dn] = kpool[so];
    vpool[dn] = vpool[so];
}

// Descriptor layout (int32 words): [0] n_seqs, [1] T, then slot[S], pos[S], nrows[S] with S = n_seqs.
// One block. Thread 0 maps blocks in sequence order; then all threads expand rows.
__global__ void __launch_bounds__(256) prepare_step_kernel(const int32_t* __restrict__ desc, int32_t* __restrict__ pos_dev,
                                                           int use_pos_dev, int32_t* __restrict__ table, int max_blocks,
                                                           int block_rows, int32_t* __restrict__ slot_mapped,
                                                           int32_t* __restrict__ free_stack, int32_t* __restrict__ free_count,
                                                           int32_t* __restrict__ seq_row0, int32_t* __restrict__ row_slot,
                                                           int32_t* __restrict__ row_pos, int32_t* __restrict__ status,
                                                           int32_t* __restrict__ refs) {
    const int S = desc[0], T = desc[1];
    const int32_t* slot = desc + 2;
    const int32_t* pos = use_pos_dev ? pos_dev : desc + 2 + S;
    const int32_t* nrows = desc + 2 + 2 * S;
    if (threadIdx.x == 0) {
        int run = 0, fc = *free_count, bad = 0;
        for (int i = 0; i < S; i++) {
            seq_row0[i] = run;
            run += nrows[i];
            const int need = (pos[i] + nrows[i] + block_rows - 1) / block_rows;
            int32_t* t = table + (size_t)slot[i] * max_blocks;
            int mapped = slot_mapped[slot[i]];
            for (int b = mapped; b < need; b++) {
                if (fc <= 0 || b >= max_blocks) { bad = 1; break; }  // the host counters rule this out
                t[b] = free_stack[--fc];
                refs[t[b]] = 1;
            }
            if (need > mapped) slot_mapped[slot[i]] = need;
        }
        seq_row0[S] = run;
        *free_count = fc;
        if (bad || run != T) *status = 1;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < T; r += blockDim.x) {
        int lo = 0, hi = S;  // last i with seq_row0[i] <= r
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (seq_row0[mid] <= r) lo = mid; else hi = mid;
        }
        row_slot[r] = slot[lo];
        row_pos[r] = pos[lo] + (r - seq_row0[lo]);
    }
}

// decode loop feedback: next token = drawn id, position + 1
__global__ void advance_kernel(int32_t* tokens, const int32_t* ids, int32_t* pos_dev, int S, int advance_pos,
                               int32_t* ids_log) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= S) return;
    tokens[i] = ids[i];
    if (ids_log) ids_log[i] = ids[i];
    if (advance_pos) pos_dev[i] += 1;
}

// ---- the device batch: a fixed set of seats that decode step after step with no per-step host packing ----
// A seat is bound to a KV slot. A live seat holds a sequence (position, the token to feed, tokens left, its end-of-sequence
// id); an empty seat runs a throw-away row at position 0 of the parking slot, so a step always has the same rows and a
// finished sequence's KV stays as it was (for a follow-up turn or as a prefix donor). Commands are applied in order at a
// step boundary; a seat retires itself when it draws its end-of-sequence id or runs out of tokens.
struct SeatCmd {
    int32_t op, seat, pos, token, max_new, eos;   // op 1: admit, 2: retire
};
struct SeatEvent {
    int32_t seat, id, pos, flags;                 // flags bit 0: the seat was live in this step, bit 1: it retired after it
};
__global__ void seats_apply_kernel(const SeatCmd* __restrict__ cmds, int n, int32_t* desc_slot, int first_slot, int park_slot,
                                   int32_t* live, int32_t* pos, int32_t* tokens, int32_t* remaining, int32_t* eos) {
    if (threadIdx.x || blockIdx.x) return;
    for (int k = 0; k < n; k++) {
        const SeatCmd c = cmds[k];
        if (c.op == 1) {
            live[c.seat] = 1; pos[c.seat] = c.pos; tokens[c.seat] = c.token; remaining[c.seat] = c.max_new; eos[c.seat] = c.eos;
            desc_slot[c.seat] = first_slot + c.seat;
        } else {
            live[c.seat] = 0; pos[c.seat] = 0; tokens[c.seat] = 0; remaining[c.seat] = 0;
            desc_slot[c.seat] = park_slot;
        }
    }
}
// the step's records go to events[*step][.] (the count of steps lives on the device so that every step is the same launches:
// a run replays one captured graph); seats_next_step_kernel moves it on
__global__ void seats_advance_kernel(int S, const int32_t* __restrict__ ids, int32_t* desc_slot, int park_slot, int32_t* live, int32_t* pos,
                                     int32_t* tokens, int32_t* remaining, const int32_t* __restrict__ eos, SeatEvent* __restrict__ events,
                                     const int32_t* __restrict__ step) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= S) return;
    events += (size_t)(*step) * S;
    SeatEvent ev{i, -1, 0, 0};
    if (live[i]) {
        const int id = ids[i];
        ev.id = id; ev.pos = pos[i]; ev.flags = 1;
        tokens[i] = id;
        pos[i] += 1;
        if (--remaining[i] <= 0 || id == eos[i]) {   // the sequence is over: the seat goes back to the parking slot
            ev.flags |= 2;
            live[i] = 0; pos[i] = 0; tokens[i] = 0;
            desc_slot[i] = park_slot;
        }
    }
    events[i] = ev;
}

__global__ void seats_next_step_kernel(int32_t* step) { *step += 1; }

__global__ void synth_kv_kernel(__half* kpool, __half* vpool, const int32_t* table_row, int n_pos, int nKV, int hd,
                                int block_rows, float sigma, uint64_t seed) {
    // element index over [pos][kvh][e]
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t n = (size_t)n_pos * nKV * hd;
    if (i >= n) return;
    int e = (int)(i % hd), kvh = (int)((i / hd) % nKV), pos = (int)(i / ((size_t)hd * nKV));
    int blk = table_row[pos / block_rows];
    size_t off = (((size_t)blk * nKV + kvh) * block_rows + (pos % block_rows)) * hd + e;
    // two cheap hashed uniforms -> approximately normal (sum of uniforms), enough for synthetic contexts
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + i;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    float u = 0.f;
    for (int k = 0; k < 4; k++) u += (float)((z >> (16 * k)) & 0xFFFF) * (1.f / 65536.f);
    float g = (u - 2.f) * 1.7320508f;  // variance 4/12 -> 1
    kpool[off] = __float2half_rn(sigma * g);
    vpool[off] = __float2half_rn(sigma * (float)(((z >> 7) & 0xFFFF) * (1.f / 65536.f) - 0.5f) * 3.4641016f);
}

__global__ void upload_kv_kernel(__half* kpool, __half* vpool, const int32_t* table_row, const float* keys, const float* vals,
                                 int base, int n, int nKV, int hd, int block_rows) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t tot = (size_t)n * nKV * hd;
    if (i >= tot) return;
    int e = (int)(i % hd), kvh = (int)((i / hd) % nKV), pos = base + (int)(i / ((size_t)hd * nKV));
    int blk = table_row[pos / block_rows];
    size_t off = (((size_t)blk * nKV + kvh) * block_rows + (pos % block_rows)) * hd + e;
    kpool[off] = __float2half_rn(keys[i]);
    vpool[off] = __float2half_rn(vals[i]);
}

}  // namespace

struct b200_model {
    b200_ctx* ctx = nullptr;
    b200_model_cfg c{};
    bool finalized = false;
    DevMat embed, head;
    float* final_norm = nullptr;
    std::vector<LayerW> layers;
    int rot_half = 0;

    // KV
    std::vector<__half*> kpool, vpool;  // per layer
    int32_t *table = nullptr, *free_stack = nullptr, *free_count = nullptr, *slot_mapped = nullptr, *status = nullptr;
    int max_blocks = 0;
    std::vector<int> h_slot_len, h_slot_mapped;
    int h_free = 0;
    // The host's mirror of the device allocator (same order of pops and pushes, so the same ids): what lets the host count a
    // step's block needs before anything is launched, shared and copy-on-write blocks included, and name blocks to copy.
    int32_t* refs = nullptr;                 // device: tables naming each block
    std::vector<int32_t> h_table, h_refs, h_stack;
    int32_t h_pop() {
        const int32_t id = h_stack.back();
        h_stack.pop_back();
        h_refs[id] = 1;
        h_free--;
        return id;
    }
    void h_unref(int32_t id) {
        if (id && --h_refs[id] <= 0) {
            h_refs[id] = 0;
            h_stack.push_back(id);
            h_free++;
        }
    }
    int32_t* h_tab(int slot) { return h_table.data() + (size_t)slot * max_blocks; }
    void h_pool_init() {
        h_table.assign((size_t)c.n_slots * max_blocks, 0);
        h_refs.assign(c.kv_pool_blocks, 0);
        h_stack.clear();
        for (int b = c.kv_pool_blocks - 1; b >= 1; b--) h_stack.push_back(b);
        h_free = c.kv_pool_blocks - 1;
    }
    // the mirror of what prepare_step_kernel does for rows up to `end` of a slot
    void h_append(int slot, int end) {
        const int need = (end + c.kv_block_rows - 1) / c.kv_block_rows;
        for (int b = h_slot_mapped[slot]; b < need; b++) h_tab(slot)[b] = h_pop();
        if (need > h_slot_mapped[slot]) h_slot_mapped[slot] = need;
        h_slot_len[slot] = std::max(h_slot_len[slot], end);
    }
    // blocks of [pos, end) that other tables also name: each costs a block of the slot's own before it is written
    int h_cow_need(int slot, int pos, int end) const {
        const int B = c.kv_block_rows, b_hi = std::min(h_slot_mapped[slot], (end + B - 1) / B);
        int n = 0;
        for (int b = pos / B; b < b_hi; b++) {
            const int32_t id = h_table[(size_t)slot * max_blocks + b];
            if (id && h_refs[id] > 1) n++;
        }
        return n;
    }

    // step buffers (device)
    int MR = 0, MLR = 0;  // max rows, max logit rows per head chunk
    int32_t *d_desc = nullptr, *d_pos = nullptr, *d_tokens = nullptr, *d_seq_row0 = nullptr, *d_row_slot = nullptr,
            *d_row_pos = nullptr, *d_head_rows = nullptr, *d_row_mask = nullptr, *d_ids = nullptr, *d_ids_log = nullptr;
    b200_draw* d_draws = nullptr;
    uint32_t* d_masks = nullptr;
    size_t masks_cap = 0;
    float *h = nullptr, *normed = nullptr, *qkv = nullptr, *ctxb = nullptr, *att = nullptr, *gu = nullptr, *mid = nullptr,
          *hn = nullptr, *logits = nullptr;
    ActQ aq_h, aq_ctx, aq_mid;
    __half* split = nullptr;
    AttnScratch asc;
    float* kq_act = nullptr;       // fast class with Q5_K / Q6_K tensors: code * scale activations for their fp16 matmul
    void* umma_scratch = nullptr;  // fast class: tcgen05 matmul scratch
    size_t x16_slot_bytes = 0;     // its two fp16 activation slots (0: the scratch has none)
    size_t umma_bytes = 0;
    int* err_flag = nullptr;       // raised by a bounded device-side wait that gave up
    ActQ aq_h_local;               // the hidden-width activation buffers this GPU's own kernels fill (aq_h may point at a peer-filled pair)
    TpFused tpf;                   // tensor parallel: the peer-visible h / partial-product / activation buffers (tpf.on) 
    float* exact_scores = nullptr;  // exact class: [MR*nH][ctx_cap]
    void* d_topk = nullptr;  // ForwardTopK's outputs: 1024 ids, 1024 logits, Z
    float *logits_local = nullptr, *logits_gather = nullptr;  // tensor parallel: [MLR][V/t] and the gathered [t][MLR][V/t]
    // the step's leading prefill run (rows of one slot at consecutive positions), 0 rows when there is none;
    // pf_tail_keys = the longest key range among the rows after it
    int pf_rows = 0, pf_slot = 0, pf_pos0 = 0, pf_tail_keys = 1;
    // the decode loop's captured step (b200_decode_loop_device) and what it was captured for
    cudaGraphExec_t loop_graph = nullptr;
    int loop_graph_S = 0, loop_graph_splits = 0, loop_graph_adv = 0;
    int64_t loop_graph_launches = 0;
    // the device batch (b200_batch_*): seats bound to slots first_slot.., empty seats park on park_slot
    struct Seats {
        int n = 0, first_slot = 0, park_slot = 0, max_steps = 0;
        int32_t *live = nullptr, *remaining = nullptr, *eos = nullptr;   // device, [n]
        int32_t *desc = nullptr, *pos = nullptr, *tokens = nullptr, *rows = nullptr;   // device: the seats' step descriptor, positions, tokens to feed, head rows
        b200_draw* draws = nullptr;
        int32_t* step = nullptr;                                         // device: steps done in the current run
        cudaGraphExec_t graph = nullptr;                                 // one captured step and what it was captured for
        int graph_splits = 0;
        int64_t graph_launches = 0;
        void *cmds = nullptr, *events = nullptr;                         // device: SeatCmd[2n], SeatEvent[max_steps][n]
        std::vector<int32_t> h_live, h_pos, h_end;                       // the host's view between runs (h_end: last position + 1 a seat may reach)
        std::vector<int32_t> pending;                                    // commands not yet applied, 6 words each
    } seats;
    // MoE
    float *rl = nullptr, *rw = nullptr, *egu_out = nullptr, *eo = nullptr, *emid = nullptr;
    int32_t *ridx = nullptr, *eoffs = nullptr, *erows = nullptr;
    ActQ aq_emid;
    __half *x16_sorted = nullptr, *x16_emid = nullptr;  // routed experts, fast class: fp16 tiles of the sorted rows and of silu(gate)*up
    ActQ aq_sorted;  // routed experts: the layer's activation rows in expert-sorted order ([max_rows*top_k][hidden])
    // pinned host staging
    int32_t* p_desc = nullptr;
    float* p_logits = nullptr;
    size_t p_logits_cap = 0;
    int32_t* p_ids = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    b200_stats_t stats{};
    size_t weight_bytes = 0, kv_bytes = 0, scratch_bytes = 0;
    std::vector<void*> allocs;

    int dalloc(void** p, size_t bytes, size_t* tally) {
        cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
        if (e != cudaSuccess) B200_FAIL(ctx, B200_CUDA_ERROR, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
        allocs.push_back(*p);
        if (tally) *tally += bytes;
        return B200_OK;
    }
    void dfree(void* p) {
        if (!p) return;
        auto it = std::find(allocs.begin(), allocs.end(), p);
        if (it != allocs.end()) allocs.erase(it);
        cudaFree(p);
    }
};

namespace {

DevMat* tensor_slot(b200_model* m, int which, int layer, int expert, float*** vec, int* veclen) {
    *vec = nullptr;
    const b200_model_cfg& c = m->c;
    if (which == B200_T_EMBED) return &m->embed;
    if (which == B200_T_LM_HEAD) return &m->head;
    if (which == B200_T_FINAL_NORM) { *vec = &m->final_norm; *veclen = c.hidden; return nullptr; }
    if (layer < 0 || layer >= c.n_layers) return nullptr;
    LayerW& L = m->layers[layer];
    switch (which) {
        case B200_T_ATTN_NORM: *vec = &L.attn_norm; *veclen = c.hidden; return nullptr;
        case B200_T_FFN_NORM: *vec = &L.ffn_norm; *veclen = c.hidden; return nullptr;
        case B200_T_Q_NORM: *vec = &L.q_norm; *veclen = c.head_dim; return nullptr;
        case B200_T_K_NORM: *vec = &L.k_norm; *veclen = c.head_dim; return nullptr;
        case B200_T_WQ: return &L.wq;
        case B200_T_WK: return &L.wk;
        case B200_T_WV: return &L.wv;
        case B200_T_WO: return &L.wo;
        case B200_T_GATE: return &L.gate;
        case B200_T_UP: return &L.up;
        case B200_T_DOWN: return &L.down;
        case B200_T_ROUTER: return &L.router;
        case B200_T_EXP_GATE: return expert >= 0 && expert < (int)L.eg.size() ? &L.eg[expert] : nullptr;
        case B200_T_EXP_UP: return expert >= 0 && expert < (int)L.eu.size() ? &L.eu[expert] : nullptr;
        case B200_T_EXP_DOWN: return expert >= 0 && expert < (int)L.ed.size() ? &L.ed[expert] : nullptr;
    }
    return nullptr;
}

// expected [rows, cols] of a matrix tensor
bool expected_shape(const b200_model_cfg& c, int which, int* rows, int* cols) {
    const int qd = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
    switch (which) {
        case B200_T_EMBED: *rows = c.vocab; *cols = c.hidden; return true;
        case B200_T_LM_HEAD: *rows = c.tp_size > 1 ? c.vocab / c.tp_size : c.vocab; *cols = c.hidden; return true;  // a rank holds its vocabulary slice
        case B200_T_WQ: *rows = qd; *cols = c.hidden; return true;
        case B200_T_WK: case B200_T_WV: *rows = kvd; *cols = c.hidden; return true;
        case B200_T_WO: *rows = c.hidden; *cols = qd; return true;
        case B200_T_GATE: case B200_T_UP: *rows = c.ffn; *cols = c.hidden; return true;
        case B200_T_DOWN: *rows = c.hidden; *cols = c.ffn; return true;
        case B200_T_ROUTER: *rows = c.n_experts; *cols = c.hidden; return true;
        case B200_T_EXP_GATE: case B200_T_EXP_UP: *rows = c.moe_ffn; *cols = c.hidden; return true;
        case B200_T_EXP_DOWN: *rows = c.hidden; *cols = c.moe_ffn; return true;
    }
    return false;
}

int prep_mat(b200_model* m, int which, int layer, int expert, int kind, int rows, int cols, DevMat** out) {
    b200_ctx* ctx = m->ctx;
    float** vecp;
    int veclen = 0;
    float*** vp = &vecp;
    DevMat* mat = tensor_slot(m, which, layer, expert, vp, &veclen);
    if (!mat) B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor %d (layer %d, expert %d) is not a matrix of this model", which, layer, expert);
    int er, ec;
    if (!expected_shape(m->c, which, &er, &ec) || er != rows || ec != cols)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor %d: shape [%d,%d], expected [%d,%d]", which, rows, cols, er, ec);
    if (kind < B200_K_F32 || kind > B200_K_I8) B200_FAIL(ctx, B200_BAD_ARGUMENT, "unknown tensor kind %d", kind);
    if (is_kquant(kind) && kind != B200_K_I8 && cols % 256) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K-quants need cols %% 256 == 0");
    if (kind == B200_K_I8 && cols % 32) B200_FAIL(ctx, B200_BAD_ARGUMENT, "int8 rows need cols %% 32 == 0");
    if (which == B200_T_ROUTER && kind != B200_K_F32) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the router stays f32");
    if (which == B200_T_EMBED && is_kquant(kind) && kind != B200_K_I8) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the embedding table is f32, f16 or int8");
    if (is_lane_kind(kind) && (expert >= 0 || m->c.tp_size > 1))
        B200_FAIL(ctx, B200_DECLINED, "Q5_K / Q6_K / int8 tensors are taken for dense, single-GPU models");
    if (mat->p) { m->dfree(mat->p); m->weight_bytes -= mat->bytes; }
    mat->kind = kind; mat->rows = rows; mat->cols = cols;
    mat->bytes = mat_bytes(kind, rows, cols);
    ST_TRY(m->dalloc(&mat->p, mat->bytes, &m->weight_bytes));
    *out = mat;
    return B200_OK;
}

// concatenates matrices of one kind and width row-wise into a new buffer and frees the parts
int fuse_rows(b200_model* m, std::vector<DevMat*> parts, DevMat* out) {
    b200_ctx* ctx = m->ctx;
    size_t bytes = 0;
    int rows = 0;
    bool same = true, all_kq = true;
    for (auto* p : parts) {
        if (!p->present() || p->cols != parts[0]->cols) B200_FAIL(ctx, B200_DECLINED, "projection group with a missing tensor or unequal widths");
        same = same && p->kind == parts[0]->kind;
        all_kq = all_kq && is_kquant(p->kind);
        bytes += p->bytes;
        rows += p->rows;
    }
    if (!same || parts[0]->kind == B200_K_Q6K || parts[0]->kind == B200_K_I8) {
        // K-quants of different kinds (a Q4_K_M file's q|k|v or gate|up), or Q6_K parts (whose d values sit behind the blocks, so two matrices do not concatenate):
        // the parts stay where they are and are multiplied one after the other into their columns of the output
        if (!all_kq || parts.size() > 3) B200_FAIL(ctx, B200_DECLINED, "projection group mixing quantized and float tensors");
        out->kind = kKindMixed; out->cols = parts[0]->cols; out->rows = rows; out->bytes = 0; out->p = nullptr;
        out->n_seg = (int)parts.size();
        for (size_t i = 0; i < parts.size(); i++) out->seg[i] = parts[i];
        return B200_OK;
    }
    out->kind = parts[0]->kind; out->cols = parts[0]->cols; out->rows = rows; out->bytes = bytes;
    ST_TRY(m->dalloc(&out->p, bytes, &m->weight_bytes));
    size_t off = 0;
    for (auto* p : parts) {
        CUDA_TRY(ctx, cudaMemcpyAsync((char*)out->p + off, p->p, p->bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        off += p->bytes;
    }
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    for (auto* p : parts) { m->dfree(p->p); m->weight_bytes -= p->bytes; p->p = nullptr; }
    return B200_OK;
}

// dst[T][N] = x . W^T, picking the kernel by the weight kind
int matmul(b200_model* m, const DevMat& W, const float* xf, ActQ xq, int T, float* dst, int ldd) {
    b200_ctx* ctx = m->ctx;
    if (W.kind == B200_K_Q4K) return launch_q4k_matmul(ctx, (const uint8_t*)W.p, W.rows, W.cols, xq, T, dst, ldd, m->c.kernel_class, W.tiles);
    if (is_lane_kind(W.kind)) {
        // from 32 rows in the fast class: fp16 copy of the weights x (code * scale) activations on the tensor cores (the
        // dp4a lane re-reads the matrix for every four rows); the weights are then within 2^-11 of their values
        static const bool no_umma = getenv("B200_NO_UMMA") != nullptr, q6_copy = getenv("B200_Q6K_F16_COPY") != nullptr;
        // Q5_K / Q6_K: the tcgen05 kernel puts the codes together itself (no dequantized copy of the matrix)
        if ((W.kind == B200_K_Q6K || W.kind == B200_K_Q5K) && !q6_copy && T >= 32 && m->c.kernel_class != B200_CLASS_EXACT && !no_umma && ctx->umma_scratch &&
            q6k_umma_fits(ctx->sm_count, ctx->x16_slot_bytes, ctx->umma_scratch_bytes, W.rows, W.cols, T) && !(reinterpret_cast<uintptr_t>(W.p) & 15))
            return launch_kq_matmul_umma(ctx, W.kind, (const uint8_t*)W.p, W.rows, W.cols, xq, T, dst, ldd);
        if (W.f16 && m->kq_act && T >= 32 && m->c.kernel_class != B200_CLASS_EXACT && !no_umma && ctx->umma_scratch &&
            f16w_umma_supported(W.f16, W.rows, W.cols) && f16w_umma_scratch_bytes(T, W.cols) <= ctx->umma_scratch_bytes) {
            ST_TRY(launch_act_dequant(ctx, xq, T, W.cols, m->kq_act));
            return launch_f16w_matmul_umma(ctx, W.f16, W.rows, W.cols, m->kq_act, T, dst, ldd, ctx->umma_scratch, ctx->umma_scratch_bytes, ctx->err_flag);
        }
        return launch_kq_matmul(ctx, W.kind, (const uint8_t*)W.p, W.rows, W.cols, xq, T, dst, ldd);
    }
    if (W.kind == kKindMixed) {
        const bool defer = ctx->defer_reduce;
        ctx->defer_reduce = false;  // a part's K-split partials cannot stand for the whole output
        int off = 0;
        for (int i = 0; i < W.n_seg; i++) {
            ST_TRY(matmul(m, *W.seg[i], xf, xq, T, dst + off, ldd));
            off += W.seg[i]->rows;
        }
        ctx->defer_reduce = defer;
        return B200_OK;
    }
    if (W.kind == B200_K_F16) return launch_f16w_matmul(ctx, (const __half*)W.p, W.rows, W.cols, xf, T, dst, ldd, m->split, m->c.kernel_class);
    return launch_f32w_matmul(ctx, (const float*)W.p, W.rows, W.cols, xf, T, dst, ldd);
}

// logits[rn][V] of `rn` already-normed rows: the LM head, whose vocabulary slices a tensor-parallel group gathers
int head_logits(b200_model* m, int rn) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    const int V = c.vocab;
    if (c.tp_size <= 1) return matmul(m, m->head, m->hn, m->aq_h, rn, m->logits, V);
    const int Vl = V / c.tp_size;
    ST_TRY(matmul(m, m->head, m->hn, m->aq_h, rn, m->logits_local, Vl));
    return tp_all_gather_columns(ctx, m->logits_local, rn, Vl, m->logits_gather, m->logits);
}

constexpr int kPrefillRunMin = 16;  // shorter runs stay with the flash-decode kernel, a row each

int run_layers(b200_model* m, int T, int max_keys) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    const int H = c.hidden, nH = c.n_heads, nKV = c.n_kv_heads, hd = c.head_dim, qd = nH * hd, ldq = (nH + 2 * nKV) * hd;
    const float scale = c.attn_scale != 0.f ? c.attn_scale : (float)(1.0 / std::sqrt((double)hd));
    const ActQ none{};
    ctx->umma_scratch = m->umma_scratch;  // this model's tcgen05 scratch and error flag serve its launches
    ctx->umma_scratch_bytes = m->umma_bytes;
    ctx->err_flag = m->err_flag;
    ctx->x16_slot_bytes = m->x16_slot_bytes;
    ctx->x16_ready = nullptr;
    struct X16Guard {  // no request, hand-off, deferral or unsummed partial outlives this call, whichever way it returns
        b200_ctx* c;
        ~X16Guard() {
            c->x16_want = nullptr;
            c->x16_ready = nullptr;
            c->defer_reduce = false;
            c->pending = Parts{};   // (the ordinary return has summed them already; an error return abandons the step's results)
        }
    } x16_guard{ctx};
    ctx->x16_want = nullptr;
    // A producer lays out the fp16 activation tiles of the tcgen05 matmul that follows it (no conversion kernel) when that
    // matmul is a plain Q4_K one at a dense row count in the fast class.
    static const bool no_x16_env = getenv("B200_NO_X16_FUSE") != nullptr || getenv("B200_NO_UMMA") != nullptr;
    auto x16_for = [&](const DevMat& W) -> __half* {
        const int x16_from = q4k_small_min_rows() > 0 ? std::min(33, q4k_small_min_rows()) : 33;  // the small-batch kernel reads the same tiles
        if (no_x16_env || !m->x16_slot_bytes || W.kind != B200_K_Q4K || T < x16_from || c.kernel_class == B200_CLASS_EXACT || (W.cols % 256) ||
            (size_t)ceil_div(T, 256) * 256 * W.cols * 2 > m->x16_slot_bytes)
            return nullptr;
        return x16_next_slot(ctx);
    };
    const float* delta = nullptr;  // pending residual add, fused into the next norm
    m->aq_h = m->aq_h_local;
    // tensor parallel on one host: sums the ranks' partial rows in m->att, adds them to the residual rows, norms with w and
    // quantizes; m->aq_h then points at the activation buffers every rank's kernel filled
    auto cross_rank_norm = [&](const float* w, __half* x16_out) -> int {
        if (m->tpf.use_ll) return launch_tp_reduce_norm_quant_ll(ctx, &m->tpf, T, w, c.rms_eps, &m->aq_h, 7, nullptr, x16_out);
        ST_TRY(launch_tp_reduce_norm_quant(ctx, &m->tpf, T, w, c.rms_eps, 0));
        m->aq_h = ActQ{m->tpf.codes(), m->tpf.scales()};
        return B200_OK;
    };
    bool normed_ready = false;     // tensor parallel: the layer's attention norm was applied by the kernel that reduced across the ranks
    __half* x16_carry = nullptr;   // ... and these are the fp16 tiles it laid out for the layer's q|k|v
    for (int l = 0; l < c.n_layers; l++) {
        LayerW& L = m->layers[l];
        bool reduced = false;  // the down products were already added to the residual rows
        const bool q_in = is_kquant(L.qkv.kind);
        __half* x16 = (q_in && !normed_ready) ? x16_for(L.qkv) : x16_carry;   // (or the tiles the cross-rank kernel laid out after the last layer)
        x16_carry = nullptr;
        if (!normed_ready) m->aq_h = m->aq_h_local;
        if (!normed_ready)  // (tensor parallel: the kernel that summed the last layer's down products has normed and quantized already)
            ST_TRY(launch_add_rmsnorm_quant(ctx, m->h, delta, L.attn_norm, T, H, c.rms_eps, q_in ? nullptr : m->normed,
                                            q_in ? m->aq_h : none, nullptr, x16));
        normed_ready = false;
        // the consumers of the q|k|v, o and down products can add their K-split partials themselves (no reduce kernel)
        static const bool tap_env = getenv("B200_DEBUG_TAP") != nullptr || getenv("B200_NO_DEFER") != nullptr;
        // (tensor parallel: only where the cross-rank kernel, which adds them like the norm kernel does, is the consumer)
        const bool can_defer = !m->exact_scores && !tap_env;
        const bool tp_ll = m->tpf.on && m->tpf.use_ll;
        const bool defer = can_defer && (c.tp_size <= 1 || m->tpf.on);
        const bool defer_o = can_defer && (c.tp_size <= 1 || (tp_ll && c.n_experts == 0 && is_kquant(L.gu.kind)));
        const bool defer_down = can_defer && (c.tp_size <= 1 || (tp_ll && l + 1 < c.n_layers && is_kquant(m->layers[l + 1].qkv.kind)));
        ctx->defer_reduce = defer;
        ctx->x16_ready = x16;
        ST_TRY(matmul(m, L.qkv, m->normed, m->aq_h, T, m->qkv, ldq));
        ctx->x16_ready = nullptr;
        ctx->defer_reduce = false;
        KVView kv{m->kpool[l], m->vpool[l], m->table, m->max_blocks, c.kv_block_rows, nKV, hd};
        ST_TRY(launch_qknorm_rope_kvstore(ctx, m->qkv, ldq, T, nH, nKV, hd, m->rot_half, L.inv_freq,
                                          c.qk_norm ? L.q_norm : nullptr, c.qk_norm ? L.k_norm : nullptr, c.rms_eps,
                                          m->d_row_slot, m->d_row_pos, kv));
        const bool o_q = is_kquant(L.wo.kind);
        __half* x16o = nullptr;
        if (m->exact_scores) {
            const double scale_d = c.attn_scale != 0.f ? (double)c.attn_scale : 1.0 / std::sqrt((double)hd);
            ST_TRY(launch_paged_attention_exact(ctx, m->qkv, ldq, T, nH, nKV, hd, scale_d, (double)c.attn_softcap, m->d_row_slot,
                                                m->d_row_pos, max_keys, kv, m->exact_scores, c.ctx_cap, m->ctxb,
                                                o_q ? m->aq_ctx : none));
        } else {
            // a leading run of rows of one sequence (a prefill chunk) goes through the tiled causal kernel, the rest through
            // flash-decode; both write f32 context rows and their per-32 codes
            const int pf = m->pf_rows;
            x16o = o_q ? x16_for(L.wo) : nullptr;   // the o projection's tiles: laid out by whoever quantizes the context rows
            ctx->x16_want = x16o;
            ctx->x16_done = 0;
            ctx->x16_row0 = 0;
            if (pf > 0) {
                ST_TRY(launch_prefill_attention(ctx, m->qkv, ldq, pf, nH, nKV, hd, scale, c.attn_softcap, m->pf_slot, m->pf_pos0, kv,
                                                m->ctxb, qd));
                if (o_q) ST_TRY(launch_quant_g32(ctx, m->ctxb, pf, qd, m->aq_ctx));
            }
            ctx->x16_row0 = pf;
            if (T > pf) {
                ActQ aq_tail = none;
                if (o_q) aq_tail = ActQ{m->aq_ctx.codes + (size_t)pf * qd, m->aq_ctx.scales + (size_t)pf * 2 * (qd / 32)};
                ST_TRY(launch_paged_attention(ctx, m->qkv + (size_t)pf * ldq, ldq, T - pf, nH, nKV, hd, scale, c.attn_softcap,
                                              m->d_row_slot + pf, m->d_row_pos + pf, pf > 0 ? m->pf_tail_keys : max_keys, kv, m->asc,
                                              m->ctxb + (size_t)pf * qd, aq_tail));
            }
        }
        ctx->x16_want = nullptr;
        ctx->defer_reduce = defer_o;
        ctx->x16_ready = (x16o && ctx->x16_done == T) ? x16o : nullptr;   // every context row was laid out
        ST_TRY(matmul(m, L.wo, m->ctxb, m->aq_ctx, T, m->att, H));
        ctx->x16_ready = nullptr;
        ctx->defer_reduce = false;
        // o is split by input columns: the ranks hold partial sums. On one host one kernel sums them over peer memory, adds
        // the residual, norms and quantizes (rows/t of the rows per rank, the codes stored to every rank); else NCCL sums.
        if (c.tp_size > 1 && !m->tpf.on) ST_TRY(tp_all_reduce_sum(ctx, m->att, (size_t)T * H));
        if (c.n_experts == 0) {
            const bool g_q = is_kquant(L.gu.kind), d_q = is_kquant(L.down.kind);
            __half* x16g = nullptr;
            if (m->tpf.on && g_q) {
                x16g = m->tpf.use_ll ? x16_for(L.gu) : nullptr;   // laid out by the cross-rank kernel as the codes arrive
                ST_TRY(cross_rank_norm(L.ffn_norm, x16g));
            } else {
                m->aq_h = m->aq_h_local;
                const float* add = m->att;
                if (m->tpf.on) {  // the summed rows go to every rank's residual stream; the norm below then adds nothing
                    ST_TRY(launch_tp_reduce_norm_quant(ctx, &m->tpf, T, nullptr, c.rms_eps, 1));
                    add = nullptr;
                }
                x16g = g_q ? x16_for(L.gu) : nullptr;
                ST_TRY(launch_add_rmsnorm_quant(ctx, m->h, add, L.ffn_norm, T, H, c.rms_eps, g_q ? nullptr : m->normed,
                                                g_q ? m->aq_h : none, nullptr, x16g));
            }
            __half* x16d = d_q ? x16_for(L.down) : nullptr;   // the other slot: laid out by whoever quantizes silu(gate) * up
            bool fused = false;
            ctx->x16_ready = x16g;
            ctx->defer_reduce = can_defer && d_q;   // the SwiGLU kernel adds the gate|up partials (each rank's columns are whole)
            static const bool no_umma_env = getenv("B200_NO_UMMA") != nullptr, no_fuse_env = getenv("B200_NO_FUSED_SWIGLU") != nullptr;
            if (L.gu_il && d_q && T >= 33 && !tap_env && !no_umma_env && ctx->umma_scratch &&
                q4k_umma_scratch_bytes(T, H, 2 * c.ffn) <= ctx->umma_scratch_bytes) {
                // the tcgen05 GEMM; where it runs two weight tiles per CTA without a K split its epilogue is the SwiGLU and the
                // quantizer (the f32 gate|up matrix is never written), else the product lands in m->gu, interleaved
                ST_TRY(launch_q4k_matmul_umma_swiglu(ctx, (const uint8_t*)L.gu.p, 2 * c.ffn, H, m->aq_h, T, m->gu, 2 * c.ffn, ctx->umma_scratch,
                                                     ctx->umma_scratch_bytes, ctx->err_flag, no_fuse_env ? ActQ{} : m->aq_mid, false, &fused, x16d, L.gu.tiles));
            } else {
                ST_TRY(matmul(m, L.gu, m->normed, m->aq_h, T, m->gu, 2 * c.ffn));
            }
            ctx->x16_ready = nullptr;
            ctx->defer_reduce = false;
            if (!fused)
                ST_TRY(launch_swiglu_quant(ctx, m->gu, T, c.ffn, 2 * c.ffn, d_q ? nullptr : m->mid, d_q ? m->aq_mid : none,
                                           c.kernel_class == B200_CLASS_EXACT, L.gu_il, x16d));
            ctx->defer_reduce = defer_down;
            ctx->x16_ready = x16d;
            ST_TRY(matmul(m, L.down, m->mid, m->aq_mid, T, m->att, H));
            ctx->x16_ready = nullptr;
            ctx->defer_reduce = false;
            if (m->tpf.on) {
                // the down products: summed, added and, when a quantized q|k|v follows, normed with the next layer's weight
                if (l + 1 < c.n_layers && is_kquant(m->layers[l + 1].qkv.kind)) {
                    x16_carry = m->tpf.use_ll ? x16_for(m->layers[l + 1].qkv) : nullptr;
                    ST_TRY(cross_rank_norm(m->layers[l + 1].attn_norm, x16_carry));
                    normed_ready = true;
                } else {
                    ST_TRY(launch_tp_reduce_norm_quant(ctx, &m->tpf, T, nullptr, c.rms_eps, 1));  // every rank gets the updated rows
                }
                reduced = true;
            } else if (c.tp_size > 1) {
                ST_TRY(tp_all_reduce_sum(ctx, m->att, (size_t)T * H));
            }
        } else {
            // routed experts (decoder/mlp.go:36-120): f32 router on the f32 normed row, top-k, grouped expert GEMMs,
            // fold in routing-rank order
            const int nE = c.n_experts, kk = c.top_k, F = c.moe_ffn;
            ST_TRY(launch_add_rmsnorm_quant(ctx, m->h, m->att, L.ffn_norm, T, H, c.rms_eps, m->normed,
                                            (H % 32 == 0) ? m->aq_h : none, nullptr));
            ST_TRY(launch_f32w_matmul(ctx, (const float*)L.router.p, nE, H, m->normed, T, m->rl, nE));
            ST_TRY(launch_route(ctx, m->rl, T, nE, kk, c.norm_topk, m->ridx, m->rw));
            ST_TRY(launch_group_experts(ctx, m->ridx, T, kk, nE, m->eoffs, m->erows));
            const int32_t* rows_tok = m->erows;
            const int32_t* slot_of = m->erows + (size_t)T * kk;
            if (L.egu_tiles) {
                // the experts' matmuls on the small-batch tensor-core kernel, grouped: token rows go to expert order as fp16
                // tiles (with their scales and group sums), the SwiGLU lays out the down projection's tiles itself
                ST_TRY(launch_gather_rows_x16(ctx, m->aq_h, rows_tok, T * kk, H, m->x16_sorted, m->aq_sorted.scales));
                ST_TRY(launch_q4k_matmul_small_grouped(ctx, L.egu_tiles, nE, 2 * F, H, m->x16_sorted, m->aq_sorted.scales, m->eoffs, T * kk, m->egu_out, 2 * F));
                ST_TRY(launch_swiglu_quant(ctx, m->egu_out, T * kk, F, 2 * F, nullptr, m->aq_emid, false, false, m->x16_emid));
                ST_TRY(launch_q4k_matmul_small_grouped(ctx, L.ed_tiles, nE, H, F, m->x16_emid, m->aq_emid.scales, m->eoffs, T * kk, m->eo, H));
            } else if (L.egu[0].kind == B200_K_Q4K) {
                static const bool no_stream = getenv("B200_NO_STREAM") != nullptr;
                if (L.egu_all && m->aq_sorted.codes && !no_stream && q4k_stream_grouped_supported(L.egu_all, 2 * F, H) &&
                    q4k_stream_grouped_supported(L.ed_all, H, F)) {
                    // weights stream through the TMA ring: the activation rows go into expert-sorted order first, so that an
                    // expert's rows are one tile of the buffer (same arithmetic and chain order as the kernel below)
                    ST_TRY(launch_gather_act_rows(ctx, m->aq_h, rows_tok, T * kk, H, m->aq_sorted));
                    ST_TRY(launch_q4k_matmul_stream_grouped(ctx, L.egu_all, nE, 2 * F, H, m->aq_sorted, m->eoffs, T * kk, T, m->egu_out, 2 * F));
                    ST_TRY(launch_swiglu_quant(ctx, m->egu_out, T * kk, F, 2 * F, nullptr, m->aq_emid, c.kernel_class == B200_CLASS_EXACT));
                    ST_TRY(launch_q4k_matmul_stream_grouped(ctx, L.ed_all, nE, H, F, m->aq_emid, m->eoffs, T * kk, T, m->eo, H));
                } else {
                    ST_TRY(launch_q4k_matmul_grouped(ctx, L.d_egu_ptrs, nE, 2 * F, H, m->aq_h, m->eoffs, rows_tok, T, m->egu_out, 2 * F));
                    ST_TRY(launch_swiglu_quant(ctx, m->egu_out, T * kk, F, 2 * F, nullptr, m->aq_emid, c.kernel_class == B200_CLASS_EXACT));
                    ST_TRY(launch_q4k_matmul_grouped(ctx, L.d_ed_ptrs, nE, H, F, m->aq_emid, m->eoffs, nullptr, T, m->eo, H));
                }
            } else if (L.egu[0].kind == B200_K_F32) {
                ST_TRY(launch_f32w_matmul_grouped(ctx, (const float* const*)L.d_egu_ptrs, nE, 2 * F, H, m->normed, m->eoffs, rows_tok, T, m->egu_out, 2 * F));
                ST_TRY(launch_swiglu_quant(ctx, m->egu_out, T * kk, F, 2 * F, m->emid, ActQ{}));
                ST_TRY(launch_f32w_matmul_grouped(ctx, (const float* const*)L.d_ed_ptrs, nE, H, F, m->emid, m->eoffs, nullptr, T, m->eo, H));
            } else {
                B200_FAIL(ctx, B200_DECLINED, "routed experts run as Q4_K or f32");
            }
            ST_TRY(launch_fold_experts(ctx, m->eo, m->rw, slot_of, T, kk, H, m->att));
        }
        delta = reduced ? nullptr : m->att;
    }
    if (delta) ST_TRY(launch_add(ctx, m->h, delta, (size_t)T * H));
    ST_TRY(flush_pending_parts(ctx));
    m->aq_h = m->aq_h_local;
    return B200_OK;
}

}  // namespace

extern "C" {

int b200_open(int device_ordinal, void* stream, b200_ctx** out) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device_ordinal < 0 || device_ordinal >= n) return B200_CUDA_ERROR;
    if (cudaSetDevice(device_ordinal) != cudaSuccess) return B200_CUDA_ERROR;
    auto* ctx = new b200_ctx();
    ctx->device = device_ordinal;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { delete ctx; return B200_CUDA_ERROR; }
        ctx->own_stream = true;
    }
    *out = ctx;
    return B200_OK;
}

void b200_close(b200_ctx* ctx) {
    if (!ctx) return;
    b200_tp_destroy(ctx);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char* b200_last_error(b200_ctx* ctx) { return ctx ? ctx->err.c_str() : "no context"; }
int64_t b200_launch_count(b200_ctx* ctx) { return ctx ? ctx->launches : 0; }

int b200_model_create(b200_ctx* ctx, const b200_model_cfg* cfg, b200_model** out) {
    const b200_model_cfg& c = *cfg;
    if (c.hidden <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.vocab <= 0 ||
        c.n_heads % c.n_kv_heads || c.n_slots <= 0 || c.ctx_cap <= 0 || c.kv_block_rows <= 0 || c.kv_pool_blocks < 2)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad model configuration");
    if (c.kv_dtype != 0) B200_FAIL(ctx, B200_DECLINED, "only the fp16 paged KV cache is built");
    if (c.tp_size > 1) {
        // a tensor-parallel shard: the configuration carries this rank's share of heads, kv heads and FFN columns and the
        // whole vocabulary; the context must hold the communicator of that size (b200_tp_init)
        if (!ctx->tp_comm || ctx->tp_size != c.tp_size || ctx->tp_rank != c.tp_rank)
            B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor-parallel rank %d of %d needs b200_tp_init with the same rank and size first", c.tp_rank, c.tp_size);
        if (c.n_experts > 0) B200_FAIL(ctx, B200_DECLINED, "tensor parallel is built for dense models");
        if (c.vocab % c.tp_size) B200_FAIL(ctx, B200_DECLINED, "the vocabulary does not divide over %d ranks", c.tp_size);
    }
    if (c.head_dim > 256) B200_FAIL(ctx, B200_DECLINED, "head_dim above 256");
    if (c.n_experts > 512) B200_FAIL(ctx, B200_DECLINED, "more than 512 experts");
    auto* m = new b200_model();
    m->ctx = ctx;
    m->c = c;
    if (m->c.rotary_dim <= 0) m->c.rotary_dim = c.head_dim;
    m->rot_half = m->c.rotary_dim / 2;
    m->layers.resize(c.n_layers);
    for (auto& L : m->layers) {
        L.h_inv_freq.resize(m->rot_half);
        for (int d = 0; d < m->rot_half; d++)  // decoder/ropescale.go:285-290
            L.h_inv_freq[d] = std::pow((double)c.rope_theta, -(double)(2 * d) / (double)(2 * m->rot_half));
        if (c.n_experts > 0) { L.eg.resize(c.n_experts); L.eu.resize(c.n_experts); L.ed.resize(c.n_experts); }
    }
    *out = m;
    return B200_OK;
}

int b200_upload_tensor(b200_model* m, int which, int layer, int expert, int kind, int rows, int cols, const void* host,
                       size_t bytes) {
    b200_ctx* ctx = m->ctx;
    if (m->finalized) B200_FAIL(ctx, B200_BAD_ARGUMENT, "model already finalized");
    float** vecp = nullptr;
    int veclen = 0;
    DevMat* probe = tensor_slot(m, which, layer, expert, &vecp, &veclen);
    if (vecp) {
        if (kind != B200_K_F32 || (size_t)rows * cols != (size_t)veclen || bytes != (size_t)veclen * 4)
            B200_FAIL(ctx, B200_BAD_ARGUMENT, "norm tensor %d must be f32[%d]", which, veclen);
        if (!*vecp) ST_TRY(m->dalloc((void**)vecp, bytes, &m->weight_bytes));
        CUDA_TRY(ctx, cudaMemcpy(*vecp, host, bytes, cudaMemcpyHostToDevice));
        return B200_OK;
    }
    (void)probe;
    DevMat* mat;
    ST_TRY(prep_mat(m, which, layer, expert, kind, rows, cols, &mat));
    if (bytes != mat->bytes) B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor %d: %zu bytes, expected %zu", which, bytes, mat->bytes);
    if (kind == B200_K_Q6K) {
        // the file's 210-byte blocks become 208-byte bodies followed by their d values on the device (16-byte aligned loads): through a staging copy
        void* stage = nullptr;
        CUDA_TRY(ctx, cudaMalloc(&stage, bytes));
        // on the model's own stream, so that the re-layout kernel is ordered after the copy (a plain cudaMemcpy from pageable
        // memory may return while its DMA is still in flight, and this stream does not wait for the default stream)
        cudaError_t e = cudaMemcpyAsync(stage, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
        int st = e == cudaSuccess ? launch_q6k_repack(ctx, (const uint8_t*)stage, bytes / 210, (uint8_t*)mat->p) : B200_CUDA_ERROR;
        if (st == B200_OK) e = cudaStreamSynchronize(ctx->stream);
        cudaFree(stage);
        if (e != cudaSuccess) B200_FAIL(ctx, B200_CUDA_ERROR, "Q6_K upload: %s", cudaGetErrorString(e));
        return st;
    }
    CUDA_TRY(ctx, cudaMemcpy(mat->p, host, bytes, cudaMemcpyHostToDevice));
    return B200_OK;
}

int b200_synth_tensor(b200_model* m, int which, int layer, int expert, int kind, int rows, int cols, float sigma, uint64_t seed) {
    b200_ctx* ctx = m->ctx;
    if (m->finalized) B200_FAIL(ctx, B200_BAD_ARGUMENT, "model already finalized");
    DevMat* mat;
    ST_TRY(prep_mat(m, which, layer, expert, kind, rows, cols, &mat));
    const size_t n = (size_t)rows * cols;
    if (is_lane_kind(kind)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "no device synthesis for Q5_K / Q6_K / int8 tensors: upload them");
    if (kind == B200_K_Q4K) return launch_synth_q4k(ctx, (uint8_t*)mat->p, n / 256, sigma, seed);
    if (kind == B200_K_F16) return launch_synth_f16(ctx, (__half*)mat->p, n, sigma, seed);
    return launch_synth_normal_f32(ctx, (float*)mat->p, n, sigma, seed);
}

int b200_set_rope_inv_freq(b200_model* m, int layer, const double* f, int n) {
    if (n != m->rot_half) B200_FAIL(m->ctx, B200_BAD_ARGUMENT, "inv_freq needs %d entries", m->rot_half);
    for (int l = 0; l < m->c.n_layers; l++)
        if (layer < 0 || l == layer) {
            m->layers[l].h_inv_freq.assign(f, f + n);
            if (m->layers[l].inv_freq)
                CUDA_TRY(m->ctx, cudaMemcpy(m->layers[l].inv_freq, f, n * sizeof(double), cudaMemcpyHostToDevice));
        }
    return B200_OK;
}

int b200_model_finalize(b200_model* m, b200_caps* out) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (m->finalized) B200_FAIL(ctx, B200_BAD_ARGUMENT, "model already finalized");
    const int H = c.hidden, nH = c.n_heads, nKV = c.n_kv_heads, hd = c.head_dim;
    CUDA_TRY(ctx, cudaDeviceSynchronize());  // every upload's copy has landed before this stream touches the tensors
    if (!m->embed.present() || !m->head.present() || !m->final_norm) B200_FAIL(ctx, B200_DECLINED, "embedding, head or final norm missing");
    for (int l = 0; l < c.n_layers; l++) {
        LayerW& L = m->layers[l];
        if (!L.attn_norm || !L.ffn_norm || (c.qk_norm && (!L.q_norm || !L.k_norm))) B200_FAIL(ctx, B200_DECLINED, "layer %d: norm weights missing", l);
        if (!L.wo.present()) B200_FAIL(ctx, B200_DECLINED, "layer %d: o projection missing", l);
        ST_TRY(fuse_rows(m, {&L.wq, &L.wk, &L.wv}, &L.qkv));
        if (c.n_experts == 0) {
            if (!L.down.present()) B200_FAIL(ctx, B200_DECLINED, "layer %d: down projection missing", l);
            if (c.kernel_class != B200_CLASS_EXACT && L.gate.present() && L.up.present() && L.gate.kind == B200_K_Q4K && L.up.kind == B200_K_Q4K &&
                L.down.kind == B200_K_Q4K && c.ffn % 128 == 0 && L.gate.cols == L.up.cols && !getenv("B200_NO_INTERLEAVE")) {
                // fast class: gate and up rows interleaved by 128, so that one 256-row tile of the tcgen05 GEMM holds gate and
                // up of the same 128 columns and its epilogue can apply the SwiGLU; every other consumer reads the same order
                L.gu.kind = B200_K_Q4K; L.gu.cols = L.gate.cols; L.gu.rows = 2 * c.ffn; L.gu.bytes = L.gate.bytes + L.up.bytes;
                ST_TRY(m->dalloc(&L.gu.p, L.gu.bytes, &m->weight_bytes));
                ST_TRY(launch_interleave_rows128(ctx, (const uint8_t*)L.gate.p, (const uint8_t*)L.up.p, c.ffn, (size_t)L.gate.cols / 256 * 144, (uint8_t*)L.gu.p));
                CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                for (DevMat* p : {&L.gate, &L.up}) { m->dfree(p->p); m->weight_bytes -= p->bytes; p->p = nullptr; }
                L.gu_il = true;
            } else {
                ST_TRY(fuse_rows(m, {&L.gate, &L.up}, &L.gu));
            }
        } else {
            if (!L.router.present()) B200_FAIL(ctx, B200_DECLINED, "layer %d: router missing", l);
            L.egu.resize(c.n_experts);
            std::vector<const uint8_t*> pg(c.n_experts), pd(c.n_experts);
            for (int e = 0; e < c.n_experts; e++) {
                if (!L.ed[e].present()) B200_FAIL(ctx, B200_DECLINED, "layer %d expert %d: down missing", l, e);
                ST_TRY(fuse_rows(m, {&L.eg[e], &L.eu[e]}, &L.egu[e]));
                pg[e] = (const uint8_t*)L.egu[e].p;
                pd[e] = (const uint8_t*)L.ed[e].p;
            }
            if (L.egu[0].kind == B200_K_Q4K && L.ed[0].kind == B200_K_Q4K) {
                // stack the experts' matrices in one buffer each, so that one tensor map addresses every expert's rows
                const size_t gb = L.egu[0].bytes, db = L.ed[0].bytes;
                bool same = true;
                for (int e = 0; e < c.n_experts; e++) same = same && L.egu[e].bytes == gb && L.ed[e].bytes == db && L.ed[e].kind == B200_K_Q4K;
                if (same) {
                    ST_TRY(m->dalloc((void**)&L.egu_all, gb * c.n_experts, &m->weight_bytes));
                    ST_TRY(m->dalloc((void**)&L.ed_all, db * c.n_experts, &m->weight_bytes));
                    for (int e = 0; e < c.n_experts; e++) {
                        CUDA_TRY(ctx, cudaMemcpyAsync(L.egu_all + gb * e, L.egu[e].p, gb, cudaMemcpyDeviceToDevice, ctx->stream));
                        CUDA_TRY(ctx, cudaMemcpyAsync(L.ed_all + db * e, L.ed[e].p, db, cudaMemcpyDeviceToDevice, ctx->stream));
                    }
                    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                    for (int e = 0; e < c.n_experts; e++) {
                        m->dfree(L.egu[e].p); m->weight_bytes -= gb; L.egu[e].p = L.egu_all + gb * e;
                        m->dfree(L.ed[e].p); m->weight_bytes -= db; L.ed[e].p = L.ed_all + db * e;
                        pg[e] = (const uint8_t*)L.egu[e].p;
                        pd[e] = (const uint8_t*)L.ed[e].p;
                    }
                    // fast class: the experts run on the small-batch tensor-core kernel in grouped form, which streams the
                    // tile-major layout; the row-major stacks are released (one copy of 16 GB of experts, not two)
                    const bool small_experts = (c.kernel_class == B200_CLASS_AUTO || c.kernel_class == 2) && !getenv("B200_NO_SMALL_EXPERTS") &&
                                               c.hidden % 256 == 0 && c.moe_ffn % 256 == 0 && q4k_small_grouped_supported(L.egu_all, 2 * c.moe_ffn, c.hidden) &&
                                               q4k_small_grouped_supported(L.ed_all, c.hidden, c.moe_ffn);
                    if (small_experts) {
                        ST_TRY(m->dalloc((void**)&L.egu_tiles, gb * c.n_experts, &m->weight_bytes));
                        ST_TRY(launch_q4k_to_tiles(ctx, L.egu_all, c.n_experts * 2 * c.moe_ffn, c.hidden, L.egu_tiles));
                        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                        m->dfree(L.egu_all); m->weight_bytes -= gb * c.n_experts; L.egu_all = nullptr;
                        ST_TRY(m->dalloc((void**)&L.ed_tiles, db * c.n_experts, &m->weight_bytes));
                        ST_TRY(launch_q4k_to_tiles(ctx, L.ed_all, c.n_experts * c.hidden, c.moe_ffn, L.ed_tiles));
                        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                        m->dfree(L.ed_all); m->weight_bytes -= db * c.n_experts; L.ed_all = nullptr;
                        for (int e = 0; e < c.n_experts; e++) { L.egu[e].p = nullptr; L.ed[e].p = nullptr; pg[e] = nullptr; pd[e] = nullptr; }
                    }
                }
            }
            ST_TRY(m->dalloc((void**)&L.d_egu_ptrs, c.n_experts * sizeof(void*), &m->weight_bytes));
            ST_TRY(m->dalloc((void**)&L.d_ed_ptrs, c.n_experts * sizeof(void*), &m->weight_bytes));
            CUDA_TRY(ctx, cudaMemcpy(L.d_egu_ptrs, pg.data(), c.n_experts * sizeof(void*), cudaMemcpyHostToDevice));
            CUDA_TRY(ctx, cudaMemcpy(L.d_ed_ptrs, pd.data(), c.n_experts * sizeof(void*), cudaMemcpyHostToDevice));
        }
        ST_TRY(m->dalloc((void**)&L.inv_freq, std::max(1, m->rot_half) * sizeof(double), &m->weight_bytes));
        CUDA_TRY(ctx, cudaMemcpy(L.inv_freq, L.h_inv_freq.data(), m->rot_half * sizeof(double), cudaMemcpyHostToDevice));
    }
    // KV pool
    m->max_blocks = ceil_div(c.ctx_cap, c.kv_block_rows);
    const size_t per_layer = (size_t)c.kv_pool_blocks * nKV * c.kv_block_rows * hd * sizeof(__half);
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    if (2 * per_layer * c.n_layers + ((size_t)1 << 30) > free_b)
        B200_FAIL(ctx, B200_DECLINED, "KV pool of %.1f GB does not fit the %.1f GB free on the device",
                  2.0 * per_layer * c.n_layers / 1e9, free_b / 1e9);
    m->kpool.resize(c.n_layers);
    m->vpool.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        ST_TRY(m->dalloc((void**)&m->kpool[l], per_layer, &m->kv_bytes));
        ST_TRY(m->dalloc((void**)&m->vpool[l], per_layer, &m->kv_bytes));
        // Block 0 is the all-zero null block (backend/cuda/kvpool.go:16-27). The whole pool starts zeroed: the attention
        // kernels load whole 16-key tiles and weight the rows past a sequence's end by zero, so every row must hold
        // finite values from the start (a reused block holds a previous sequence's finite rows).
        CUDA_TRY(ctx, cudaMemsetAsync(m->kpool[l], 0, per_layer, ctx->stream));
        CUDA_TRY(ctx, cudaMemsetAsync(m->vpool[l], 0, per_layer, ctx->stream));
    }
    ST_TRY(m->dalloc((void**)&m->table, (size_t)c.n_slots * m->max_blocks * 4, &m->kv_bytes));
    ST_TRY(m->dalloc((void**)&m->free_stack, (size_t)c.kv_pool_blocks * 4, &m->kv_bytes));
    ST_TRY(m->dalloc((void**)&m->free_count, 4, nullptr));
    ST_TRY(m->dalloc((void**)&m->slot_mapped, (size_t)c.n_slots * 4, nullptr));
    ST_TRY(m->dalloc((void**)&m->refs, (size_t)c.kv_pool_blocks * 4, &m->kv_bytes));
    ST_TRY(m->dalloc((void**)&m->status, 4, nullptr));
    CUDA_TRY(ctx, cudaMemsetAsync(m->status, 0, 4, ctx->stream));
    m->h_slot_len.assign(c.n_slots, 0);
    m->h_slot_mapped.assign(c.n_slots, 0);
    m->h_pool_init();
    // step buffers
    const int MR = m->MR = std::max(1, c.max_rows);
    const int MLR = m->MLR = std::min(MR, std::max(c.n_slots, 64));
    size_t* sb = &m->scratch_bytes;
    const int qd = nH * hd, ldq = (nH + 2 * nKV) * hd;
    const int F = c.n_experts ? 0 : c.ffn;
    ST_TRY(m->dalloc((void**)&m->d_desc, (size_t)(2 + 3 * MR) * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_pos, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_tokens, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_seq_row0, (size_t)(MR + 1) * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_row_slot, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_row_pos, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_head_rows, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_row_mask, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_ids, (size_t)MR * 4, sb));
    ST_TRY(m->dalloc((void**)&m->d_draws, (size_t)MR * sizeof(b200_draw), sb));
    // tensor parallel on one host: the residual rows, the o / down partial products and the activations that follow them
    // live in a block the other ranks have mapped, for the kernel that sums, norms and quantizes across the ranks
    if (c.tp_size > 1 && c.n_experts == 0) ST_TRY(tp_fused_setup(ctx, &m->tpf, MR, H));
    if (m->tpf.on) {
        m->h = m->tpf.h();
        if (sb) *sb += m->tpf.bytes;
    } else {
        ST_TRY(m->dalloc((void**)&m->h, (size_t)MR * H * 4, sb));
    }
    ST_TRY(m->dalloc((void**)&m->normed, (size_t)MR * H * 4, sb));
    ST_TRY(m->dalloc((void**)&m->qkv, (size_t)MR * ldq * 4, sb));
    ST_TRY(m->dalloc((void**)&m->ctxb, (size_t)MR * qd * 4, sb));
    if (m->tpf.on) m->att = m->tpf.part();
    else ST_TRY(m->dalloc((void**)&m->att, (size_t)MR * H * 4, sb));
    ST_TRY(m->dalloc((void**)&m->aq_h.codes, (size_t)MR * H, sb));
    ST_TRY(m->dalloc((void**)&m->aq_h.scales, (size_t)MR * 2 * ceil_div(H, 32) * 4, sb));
    m->aq_h_local = m->aq_h;
    ST_TRY(m->dalloc((void**)&m->aq_ctx.codes, (size_t)MR * qd, sb));
    ST_TRY(m->dalloc((void**)&m->aq_ctx.scales, (size_t)MR * 2 * ceil_div(qd, 32) * 4, sb));
    if (F) {
        ST_TRY(m->dalloc((void**)&m->gu, (size_t)MR * 2 * F * 4, sb));
        ST_TRY(m->dalloc((void**)&m->mid, (size_t)MR * F * 4, sb));
        ST_TRY(m->dalloc((void**)&m->aq_mid.codes, (size_t)MR * F, sb));
        ST_TRY(m->dalloc((void**)&m->aq_mid.scales, (size_t)MR * 2 * ceil_div(F, 32) * 4, sb));
    } else {
        const int nE = c.n_experts, kk = c.top_k, EF = c.moe_ffn;
        ST_TRY(m->dalloc((void**)&m->rl, (size_t)MR * nE * 4, sb));
        ST_TRY(m->dalloc((void**)&m->rw, (size_t)MR * kk * 4, sb));
        ST_TRY(m->dalloc((void**)&m->ridx, (size_t)MR * kk * 4, sb));
        ST_TRY(m->dalloc((void**)&m->eoffs, (size_t)(nE + 1) * 4, sb));
        ST_TRY(m->dalloc((void**)&m->erows, (size_t)2 * MR * kk * 4, sb));
        ST_TRY(m->dalloc((void**)&m->egu_out, (size_t)MR * kk * 2 * EF * 4, sb));
        ST_TRY(m->dalloc((void**)&m->eo, (size_t)MR * kk * H * 4, sb));
        if (m->layers[0].egu[0].kind != B200_K_Q4K) ST_TRY(m->dalloc((void**)&m->emid, (size_t)MR * kk * EF * 4, sb));
        if (H % 256 == 0) {
            ST_TRY(m->dalloc((void**)&m->aq_sorted.codes, (size_t)MR * kk * H, sb));
            ST_TRY(m->dalloc((void**)&m->aq_sorted.scales, (size_t)MR * kk * 2 * (H / 32) * 4, sb));
        }
        if (m->layers[0].egu_tiles) {   // rows padded to whole 256-row tiles with room for a 16-row pass past the last row
            const size_t rows_pad = (size_t)ceil_div(MR * kk + 16, 256) * 256;
            ST_TRY(m->dalloc((void**)&m->x16_sorted, rows_pad * H * 2, sb));
            ST_TRY(m->dalloc((void**)&m->x16_emid, rows_pad * EF * 2, sb));
            CUDA_TRY(ctx, cudaMemsetAsync(m->x16_sorted, 0, rows_pad * H * 2, ctx->stream));
            CUDA_TRY(ctx, cudaMemsetAsync(m->x16_emid, 0, rows_pad * EF * 2, ctx->stream));
        }
        ST_TRY(m->dalloc((void**)&m->aq_emid.codes, (size_t)MR * kk * EF, sb));
        ST_TRY(m->dalloc((void**)&m->aq_emid.scales, (size_t)MR * kk * 2 * ceil_div(EF, 32) * 4, sb));
    }
    const bool fast_attn = (hd == 64 || hd == 128) && ((nH / nKV) == 1 || (nH / nKV) == 2 || (nH / nKV) == 4 || (nH / nKV) == 8);
    if (c.kernel_class == B200_CLASS_EXACT || (!fast_attn && hd > 64)) {
        ST_TRY(m->dalloc((void**)&m->exact_scores, (size_t)MR * nH * c.ctx_cap * 4, sb));
    } else {
        m->asc.max_splits = ceil_div(c.ctx_cap, attn_split_keys());
        ST_TRY(m->dalloc((void**)&m->asc.partial, attn_scratch_floats(MR, nH, hd, m->asc.max_splits) * 4, sb));
    }
    if (c.kernel_class != B200_CLASS_EXACT && MR >= 4) {
        // fast class: scratch of the tcgen05 matmul (fp16 activations + split-K partials), sized for the widest projection
        int max_k = std::max(H, qd), max_n = std::max(ldq, H);
        if (F) { max_k = std::max(max_k, F); max_n = std::max(max_n, 2 * F); }
        m->umma_bytes = q4k_umma_scratch_bytes(MR, max_k, max_n);
        // two fp16 activation slots ahead of the partials: producers lay the tiles out for the matmul that follows them
        m->x16_slot_bytes = ((size_t)ceil_div(MR, 256) * 256 * max_k * 2 + 255) & ~(size_t)255;
        m->umma_bytes += m->x16_slot_bytes;
        // Q4_K projections are re-laid tile by tile, the layout the fast class's kernels fetch with plain bulk copies (the
        // one- and two-row dp4a kernel, the small-batch kernel up to 32 rows, the tcgen05 kernel above). The row-major
        // matrix is then released, unless the kernel class or a debugging switch can route a step to the older kernels
        // that read it, or the scratch cannot hold the matrix's worst case.
        if (q4k_small_min_rows() > 0) {
            const bool may_drop = (c.kernel_class == B200_CLASS_AUTO || c.kernel_class == 2) && !getenv("B200_KEEP_ROW_MAJOR") && !getenv("B200_NO_UMMA") &&
                                  !getenv("B200_UMMA_ROW_MAJOR") && !getenv("B200_DEBUG_TAP");
            auto to_tiles = [&](DevMat* d, int max_rows) -> int {
                if (!d->p || d->kind != B200_K_Q4K || d->cols % 256) return B200_OK;
                ST_TRY(m->dalloc((void**)&d->tiles, q4k_tiles_bytes(d->rows, d->cols), &m->weight_bytes));
                ST_TRY(launch_q4k_to_tiles(ctx, (const uint8_t*)d->p, d->rows, d->cols, d->tiles));
                if (may_drop && q4k_umma_scratch_bytes(max_rows, d->cols, d->rows) <= m->umma_bytes) {
                    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                    m->dfree(d->p);
                    d->p = nullptr;
                    m->weight_bytes -= d->bytes;
                }
                return B200_OK;
            };
            for (int l = 0; l < c.n_layers; l++) {
                LayerW& L = m->layers[l];
                for (DevMat* d : {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down, &L.qkv, &L.gu}) ST_TRY(to_tiles(d, MR));
            }
            ST_TRY(to_tiles(&m->head, MLR));
        }
        // W8A8 tensors: fp16 copies for the tensor-core matmul from 32 rows on. Q5_K and Q6_K tensors need none: the tcgen05
        // kernel takes their blocks as they are (a copy is made only where the scratch cannot hold the matrix's partials)
        std::vector<DevMat*> kq;
        const size_t scratch_now = m->umma_bytes;
        auto wants_copy = [&](const DevMat* d, int rows_max) {
            if (!d->p || !is_lane_kind(d->kind)) return false;
            if ((d->kind != B200_K_Q6K && d->kind != B200_K_Q5K) || getenv("B200_Q6K_F16_COPY")) return true;
            return !q6k_umma_fits(ctx->sm_count, m->x16_slot_bytes, scratch_now, d->rows, d->cols, rows_max) || (reinterpret_cast<uintptr_t>(d->p) & 15);
        };
        for (int l = 0; l < c.n_layers; l++) {
            LayerW& L = m->layers[l];
            for (DevMat* d : {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down, &L.qkv, &L.gu})
                if (wants_copy(d, MR)) kq.push_back(d);
        }
        if (wants_copy(&m->head, MLR)) kq.push_back(&m->head);
        if (!kq.empty() && MR >= 32) {
            for (DevMat* d : kq) {
                ST_TRY(m->dalloc((void**)&d->f16, (size_t)d->rows * d->cols * 2, &m->weight_bytes));
                ST_TRY(launch_kq_to_f16(ctx, d->kind, (const uint8_t*)d->p, d->rows, d->cols, d->f16));
            }
            ST_TRY(m->dalloc((void**)&m->kq_act, (size_t)MR * max_k * 4, sb));
            m->umma_bytes = std::max(m->umma_bytes, f16w_umma_scratch_bytes(MR, max_k));
        }
        ST_TRY(m->dalloc(&m->umma_scratch, m->umma_bytes, sb));
    }
    ST_TRY(m->dalloc((void**)&m->err_flag, 4, nullptr));
    CUDA_TRY(ctx, cudaMemsetAsync(m->err_flag, 0, 4, ctx->stream));
    ST_TRY(m->dalloc((void**)&m->hn, (size_t)MLR * H * 4, sb));
    ST_TRY(m->dalloc((void**)&m->logits, (size_t)MLR * c.vocab * 4, sb));
    if (c.tp_size > 1) {
        ST_TRY(m->dalloc((void**)&m->logits_local, (size_t)MLR * (c.vocab / c.tp_size) * 4, sb));
        ST_TRY(m->dalloc((void**)&m->logits_gather, (size_t)MLR * c.vocab * 4, sb));
    }
    ST_TRY(m->dalloc((void**)&m->split, (size_t)2 * MLR * H * 2, sb));
    CUDA_TRY(ctx, cudaMallocHost((void**)&m->p_desc, (size_t)(2 + 3 * MR) * 4 + (size_t)MR * (4 + 4 + 4 + sizeof(b200_draw))));
    CUDA_TRY(ctx, cudaMallocHost((void**)&m->p_ids, (size_t)(MR + 2) * 4));  // ids, then the error flag and the allocator status
    CUDA_TRY(ctx, cudaEventCreate(&m->ev0));
    CUDA_TRY(ctx, cudaEventCreate(&m->ev1));
    m->finalized = true;
    ST_TRY(b200_reset(m));
    if (out) {
        memset(out, 0, sizeof *out);
        out->context_cap = c.ctx_cap;
        out->kv_slots = c.n_slots;
        out->batch_lo = 2;  // BatchStepRange = (2, KVSlots), backend/cuda/batchstep.go:36-44
        out->batch_hi = c.n_slots;
        // the fast class (fp32 flash attention, split-K small-batch matmul) is not bit-identical to the exact one
        out->has_fast_prefill = c.kernel_class == B200_CLASS_EXACT ? 0 : 1;
        out->fast_prefill_floor = c.kernel_class == B200_CLASS_EXACT ? 0 : 1;
        out->tail_min_rows = 1;
        out->batch_greedy_draw = 1;
        out->weight_bytes = (int64_t)m->weight_bytes;
        out->kv_bytes = (int64_t)m->kv_bytes;
        out->scratch_bytes = (int64_t)m->scratch_bytes;
    }
    return B200_OK;
}

void b200_model_free(b200_model* m) {
    if (!m) return;
    cudaStreamSynchronize(m->ctx->stream);
    tp_fused_teardown(m->ctx, &m->tpf);
    if (m->loop_graph) cudaGraphExecDestroy(m->loop_graph);
    if (m->seats.graph) cudaGraphExecDestroy(m->seats.graph);
    for (void* p : m->allocs) cudaFree(p);
    if (m->p_desc) cudaFreeHost(m->p_desc);
    if (m->p_ids) cudaFreeHost(m->p_ids);
    if (m->p_logits) cudaFreeHost(m->p_logits);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    delete m;
}

int b200_kv_slots(b200_model* m) { return m->c.n_slots; }
int b200_tp_fused_active(b200_model* m) { return m && m->tpf.on ? 1 : 0; }

int b200_bench_tp_reduce(b200_model* m, int T, int mode, int warmup, int iters, float* ms_out, float* stage_us_out) {
    b200_ctx* ctx = m->ctx;
    if (!m->finalized || !m->tpf.on || T < 1 || T > m->MR || iters < 1 || !ms_out) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the cross-rank kernel is not in use, or bad arguments");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ctx->err_flag = m->err_flag;
    const float* w = m->layers[0].ffn_norm;
    auto one = [&]() -> int {  // the form the model's steps use
        if (mode == 0 && m->tpf.use_ll) return launch_tp_reduce_norm_quant_ll(ctx, &m->tpf, T, w, m->c.rms_eps, nullptr);
        return launch_tp_reduce_norm_quant(ctx, &m->tpf, T, w, m->c.rms_eps, mode);
    };
    for (int i = 0; i < warmup; i++) ST_TRY(one());
    CUDA_TRY(ctx, cudaEventRecord(m->ev0, ctx->stream));
    for (int i = 0; i < iters; i++) ST_TRY(one());
    CUDA_TRY(ctx, cudaEventRecord(m->ev1, ctx->stream));
    CUDA_TRY(ctx, cudaEventSynchronize(m->ev1));
    float ms = 0.f;
    CUDA_TRY(ctx, cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    *ms_out = ms / iters;
    if (stage_us_out) {  // one more launch with CTA 0's clock stamped at each stage
        long long* d_ns = nullptr;
        long long ns[5] = {0, 0, 0, 0, 0};
        CUDA_TRY(ctx, cudaMalloc((void**)&d_ns, sizeof ns));
        CUDA_TRY(ctx, cudaMemsetAsync(d_ns, 0, sizeof ns, ctx->stream));
        m->tpf.phase_ns = d_ns;
        const int st = one();
        m->tpf.phase_ns = nullptr;
        if (st == B200_OK) cudaMemcpyAsync(ns, d_ns, sizeof ns, cudaMemcpyDeviceToHost, ctx->stream);
        cudaStreamSynchronize(ctx->stream);
        cudaFree(d_ns);
        ST_TRY(st);
        for (int i = 0; i < 4; i++) stage_us_out[i] = (float)(ns[i + 1] - ns[i]) * 1e-3f;
    }
    int gave_up = 0;
    CUDA_TRY(ctx, cudaMemcpyAsync(&gave_up, m->err_flag, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (gave_up) {
        cudaMemsetAsync(m->err_flag, 0, 4, ctx->stream);
        B200_FAIL(ctx, B200_TIMEOUT, "a rank waited for its peers longer than its limit");
    }
    return B200_OK;
}

int b200_reset_slot(b200_model* m, int slot) {
    b200_ctx* ctx = m->ctx;
    if (!m->finalized || slot < 0 || slot >= m->c.n_slots) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad slot %d", slot);
    reset_slot_kernel<<<1, 1, 0, ctx->stream>>>(m->free_stack, m->free_count, m->table, m->max_blocks, m->slot_mapped, slot, m->refs);
    LAUNCH_CHECK(ctx);
    for (int b = 0; b < m->h_slot_mapped[slot]; b++) {
        m->h_unref(m->h_tab(slot)[b]);
        m->h_tab(slot)[b] = 0;
    }
    m->h_slot_mapped[slot] = 0;
    m->h_slot_len[slot] = 0;
    return B200_OK;
}

int b200_reset(b200_model* m) {
    b200_ctx* ctx = m->ctx;
    if (!m->finalized) B200_FAIL(ctx, B200_BAD_ARGUMENT, "model not finalized");
    const size_t tn = (size_t)m->c.n_slots * m->max_blocks;
    const size_t n = std::max<size_t>(std::max<size_t>(tn, m->c.kv_pool_blocks), m->c.n_slots);
    init_pool_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(m->free_stack, m->free_count, m->c.kv_pool_blocks,
                                                                           m->table, tn, m->slot_mapped, m->c.n_slots, m->refs);
    LAUNCH_CHECK(ctx);
    std::fill(m->h_slot_len.begin(), m->h_slot_len.end(), 0);
    std::fill(m->h_slot_mapped.begin(), m->h_slot_mapped.end(), 0);
    m->h_pool_init();
    return B200_OK;
}

int b200_block_table(b200_model* m, int slot, int32_t* out, int n) {
    b200_ctx* ctx = m->ctx;
    if (!m->finalized || slot < 0 || slot >= m->c.n_slots) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad slot %d", slot);
    const int k = std::min(n, m->max_blocks);
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaMemcpy(out, m->table + (size_t)slot * m->max_blocks, (size_t)k * 4, cudaMemcpyDeviceToHost));
    for (int i = k; i < n; i++) out[i] = 0;
    return B200_OK;
}

}  // extern "C"

namespace {

// host-side block accounting for rows [0, end) of a slot; returns blocks still to map
int blocks_needed(const b200_model* m, int slot, int end) {
    return std::max(0, ceil_div(end, m->c.kv_block_rows) - m->h_slot_mapped[slot]);
}

// rows [0, rows) of block `from` -> block `to` in every layer
int copy_block_rows(b200_model* m, int from, int to, int rows) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (rows <= 0) return B200_OK;
    const size_t n = (size_t)c.n_kv_heads * rows * c.head_dim;
    for (int l = 0; l < c.n_layers; l++) {
        copy_block_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(m->kpool[l], m->vpool[l], from, to, rows, c.n_kv_heads,
                                                                                    c.kv_block_rows, c.head_dim);
        LAUNCH_CHECK(ctx);
    }
    return B200_OK;
}

// Before a slot writes rows [pos, end): blocks of that range other tables also name are replaced by blocks of its own, the
// rows before pos kept (backend/cuda/kvpool.go:436-477). The caller has counted the blocks this takes (h_cow_need).
int make_private(b200_model* m, int slot, int pos, int end) {
    b200_ctx* ctx = m->ctx;
    if (m->h_cow_need(slot, pos, end) == 0) return B200_OK;
    const int B = m->c.kv_block_rows, b_lo = pos / B, b_hi = std::min(m->h_slot_mapped[slot], ceil_div(end, B));
    cow_kernel<<<1, 1, 0, ctx->stream>>>(m->table, m->max_blocks, m->refs, m->free_stack, m->free_count, slot, b_lo, b_hi);
    LAUNCH_CHECK(ctx);
    for (int b = b_lo; b < b_hi; b++) {
        const int32_t old = m->h_tab(slot)[b];
        if (old && m->h_refs[old] > 1) {
            const int32_t id = m->h_pop();
            m->h_refs[old]--;
            m->h_tab(slot)[b] = id;
            if (b == b_lo) ST_TRY(copy_block_rows(m, old, id, pos - b * B));
        }
    }
    return B200_OK;
}

// After a synchronize that brought the device's error flag (p_ids[MR]) and allocator status (p_ids[MR+1]) back: a bounded
// wait that gave up is B200_TIMEOUT; a prepare_step_kernel that found its free stack empty, a table full or a row count
// unlike the descriptor's means the host's counters and the device allocator disagree, which no later step can repair.
int check_device_flags(b200_model* m, const char* what) {
    b200_ctx* ctx = m->ctx;
    const int timed_out = m->p_ids[m->MR], alloc_bad = m->p_ids[m->MR + 1];
    if (timed_out) cudaMemsetAsync(m->err_flag, 0, 4, ctx->stream);
    if (alloc_bad) cudaMemsetAsync(m->status, 0, 4, ctx->stream);
    if (alloc_bad) B200_FAIL(ctx, B200_CUDA_ERROR, "the device block allocator disagreed with the host's counters during %s; reset the model", what);
    if (timed_out) B200_FAIL(ctx, B200_TIMEOUT, "a bounded device-side wait gave up during %s", what);
    return B200_OK;
}

// Maps the blocks of rows [0, end) of one slot on the device and makes the blocks of [base, end) its own (used by the KV
// upload/synthesis entry points, which write those rows).
int map_slot_rows(b200_model* m, int slot, int base, int end) {
    b200_ctx* ctx = m->ctx;
    const int fresh = blocks_needed(m, slot, end), need = fresh + m->h_cow_need(slot, base, end);
    if (need > m->h_free) { m->stats.kv_pool_full++; B200_FAIL(ctx, B200_KV_POOL_FULL, "kv pool full: %d blocks needed, %d free", need, m->h_free); }
    ST_TRY(make_private(m, slot, base, end));
    if (fresh == 0) return B200_OK;
    int32_t* d = m->p_desc;
    d[0] = 1; d[1] = 1; d[2] = slot; d[3] = end - 1; d[4] = 1;
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_desc, d, 5 * 4, cudaMemcpyHostToDevice, ctx->stream));
    prepare_step_kernel<<<1, 256, 0, ctx->stream>>>(m->d_desc, m->d_pos, 0, m->table, m->max_blocks, m->c.kv_block_rows,
                                                    m->slot_mapped, m->free_stack, m->free_count, m->d_seq_row0, m->d_row_slot,
                                                    m->d_row_pos, m->status, m->refs);
    LAUNCH_CHECK(ctx);
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR + 1, m->status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));  // p_desc is reused by the next call
    m->p_ids[m->MR] = 0;
    ST_TRY(check_device_flags(m, "a KV upload"));
    {
        const int keep_len = m->h_slot_len[slot];
        m->h_append(slot, end);
        m->h_slot_len[slot] = keep_len;  // the callers set the stored length themselves
    }
    return B200_OK;
}

}  // namespace

extern "C" {

int b200_synth_kv(b200_model* m, int slot, int n_pos, float sigma, uint64_t seed) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (!m->finalized || slot < 0 || slot >= c.n_slots || n_pos < 0 || n_pos > c.ctx_cap) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad slot or length");
    if (n_pos == 0) return B200_OK;
    ST_TRY(map_slot_rows(m, slot, 0, n_pos));
    const size_t n = (size_t)n_pos * c.n_kv_heads * c.head_dim;
    for (int l = 0; l < c.n_layers; l++) {
        synth_kv_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(m->kpool[l], m->vpool[l],
                                                                              m->table + (size_t)slot * m->max_blocks, n_pos,
                                                                              c.n_kv_heads, c.head_dim, c.kv_block_rows, sigma,
                                                                              seed * 1315423911ull + (uint64_t)l);
        LAUNCH_CHECK(ctx);
    }
    m->h_slot_len[slot] = std::max(m->h_slot_len[slot], n_pos);
    return B200_OK;
}

int b200_upload_kv(b200_model* m, int slot, int layer, int base, int n, const float* keys, const float* vals) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (!m->finalized || slot < 0 || slot >= c.n_slots || layer < 0 || layer >= c.n_layers || base < 0 || n <= 0 || base + n > c.ctx_cap)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad slot, layer or range");
    ST_TRY(map_slot_rows(m, slot, base, base + n));
    const size_t cnt = (size_t)n * c.n_kv_heads * c.head_dim;
    struct Staging {  // freed on every way out
        float *k = nullptr, *v = nullptr;
        ~Staging() { cudaFree(k); cudaFree(v); }
    } stg;
    CUDA_TRY(ctx, cudaMalloc(&stg.k, cnt * 4));
    CUDA_TRY(ctx, cudaMalloc(&stg.v, cnt * 4));
    CUDA_TRY(ctx, cudaMemcpyAsync(stg.k, keys, cnt * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(stg.v, vals, cnt * 4, cudaMemcpyHostToDevice, ctx->stream));
    upload_kv_kernel<<<(unsigned)((cnt + 255) / 256), 256, 0, ctx->stream>>>(m->kpool[layer], m->vpool[layer],
                                                                             m->table + (size_t)slot * m->max_blocks, stg.k, stg.v, base, n,
                                                                             c.n_kv_heads, c.head_dim, c.kv_block_rows);
    LAUNCH_CHECK(ctx);
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    m->h_slot_len[slot] = std::max(m->h_slot_len[slot], base + n);
    return B200_OK;
}

int b200_copy_kv(b200_model* m, int dst_slot, int src_slot, int n_rows) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (!m->finalized || dst_slot < 0 || dst_slot >= c.n_slots || src_slot < 0 || src_slot >= c.n_slots || dst_slot == src_slot)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad slots %d <- %d", dst_slot, src_slot);
    if (n_rows < 0 || n_rows > m->h_slot_len[src_slot]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "slot %d stores %d rows, %d asked", src_slot, m->h_slot_len[src_slot], n_rows);
    const int B = c.kv_block_rows, n_full = n_rows / B, tail = n_rows % B;
    // what dst holds now goes back to the pool first (in the mirror too), then the budget is checked: nothing is written on refusal
    const int freed_after_reset = [&] {
        int n = 0;
        for (int b = 0; b < m->h_slot_mapped[dst_slot]; b++) {
            const int32_t id = m->h_tab(dst_slot)[b];
            if (id && m->h_refs[id] == 1) n++;
        }
        return n;
    }();
    if ((tail ? 1 : 0) > m->h_free + freed_after_reset) {
        m->stats.kv_pool_full++;
        B200_FAIL(ctx, B200_KV_POOL_FULL, "kv pool full: 1 block needed, %d free", m->h_free + freed_after_reset);
    }
    ST_TRY(b200_reset_slot(m, dst_slot));
    if (n_rows == 0) return B200_OK;
    share_prefix_kernel<<<1, 1, 0, ctx->stream>>>(m->table, m->max_blocks, m->slot_mapped, m->refs, m->free_stack, m->free_count, src_slot,
                                                  dst_slot, n_full, tail ? 1 : 0);
    LAUNCH_CHECK(ctx);
    for (int b = 0; b < n_full; b++) {
        const int32_t id = m->h_tab(src_slot)[b];
        m->h_tab(dst_slot)[b] = id;
        m->h_refs[id]++;
    }
    m->h_slot_mapped[dst_slot] = n_full;
    if (tail) {
        const int32_t id = m->h_pop();
        m->h_tab(dst_slot)[n_full] = id;
        m->h_slot_mapped[dst_slot] = n_full + 1;
        ST_TRY(copy_block_rows(m, m->h_tab(src_slot)[n_full], id, tail));
    }
    m->h_slot_len[dst_slot] = n_rows;
    return B200_OK;
}

int b200_step_ragged(b200_model* m, int n_seqs, const int32_t* slot, const int32_t* pos, const int32_t* n_rows,
                     const int32_t* prefill_prompt_len, const uint8_t* prefill_last, const float* embs, const int32_t* token_ids,
                     const b200_draw* draws, const int32_t* mask_index, const uint32_t* logit_mask, int n_masks, float* logits_out,
                     int32_t* ids_out, int32_t* n_logit_rows_out) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (!m->finalized) B200_FAIL(ctx, B200_BAD_ARGUMENT, "model not finalized");
    if (n_seqs <= 0 || (!embs) == (!token_ids)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "a step takes exactly one of embs / token_ids");
    const int H = c.hidden, V = c.vocab;
    // ---- checks on the sequences alone (backend/cuda/batchstep.go:184-211) and the block budget ----
    int T = 0, need = 0, max_keys = 0;
    {
        std::vector<char> seen(c.n_slots, 0);
        for (int i = 0; i < n_seqs; i++) {
            if (slot[i] < 0 || slot[i] >= c.n_slots || seen[slot[i]]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "sequence %d: slot %d out of range or repeated", i, slot[i]);
            seen[slot[i]] = 1;
            if (n_rows[i] <= 0 || pos[i] < 0 || pos[i] + n_rows[i] > c.ctx_cap)
                B200_FAIL(ctx, B200_BAD_ARGUMENT, "sequence %d: rows [%d,%d) outside the context cap %d", i, pos[i], pos[i] + n_rows[i], c.ctx_cap);
            if (pos[i] > m->h_slot_len[slot[i]]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "sequence %d: position %d past the slot's %d stored rows", i, pos[i], m->h_slot_len[slot[i]]);
            const int pl = prefill_prompt_len ? prefill_prompt_len[i] : 0;
            if (pl > 0) {
                const bool last = prefill_last && prefill_last[i];
                const bool has_draw = draws && draws[i].kind != B200_DRAW_LOGITS;
                if (i != 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "a step takes one prefill chunk and it goes first");
                if (has_draw) B200_FAIL(ctx, B200_BAD_ARGUMENT, "a prefill chunk carries no draw");
                if (pl < pos[i] + n_rows[i]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the chunk ends at %d, past its prompt's %d", pos[i] + n_rows[i], pl);
                if (last != (pos[i] + n_rows[i] == pl)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the chunk ends at %d of a %d-row prompt with Last %d", pos[i] + n_rows[i], pl, (int)last);
            }
            T += n_rows[i];
            need += blocks_needed(m, slot[i], pos[i] + n_rows[i]) + m->h_cow_need(slot[i], pos[i], pos[i] + n_rows[i]);
            max_keys = std::max(max_keys, pos[i] + n_rows[i]);
        }
    }
    if (T > m->MR) B200_FAIL(ctx, B200_BAD_ARGUMENT, "%d rows exceed max_rows %d", T, m->MR);
    if (token_ids)
        for (int r = 0; r < T; r++)
            if (token_ids[r] < 0 || token_ids[r] >= V) B200_FAIL(ctx, B200_BAD_ARGUMENT, "token id %d out of range", token_ids[r]);
    if (need > m->h_free) { m->stats.kv_pool_full++; B200_FAIL(ctx, B200_KV_POOL_FULL, "kv pool full: %d blocks needed, %d free", need, m->h_free); }

    // ---- rows that reach the LM head: logits rows first, then the drawn rows ----
    std::vector<int> head_rows, head_seq;
    int n_out = 0;
    {
        std::vector<int> draw_rows, draw_seq;
        int r0 = 0;
        for (int i = 0; i < n_seqs; i++) {
            const int pl = prefill_prompt_len ? prefill_prompt_len[i] : 0;
            const int dk = draws ? draws[i].kind : B200_DRAW_LOGITS;
            const int lastr = r0 + n_rows[i] - 1;
            if (pl > 0) {
                if (prefill_last && prefill_last[i]) { head_rows.push_back(lastr); head_seq.push_back(i); }
            } else {
                for (int r = r0; r < lastr; r++) { head_rows.push_back(r); head_seq.push_back(i); }
                if (dk == B200_DRAW_LOGITS) { head_rows.push_back(lastr); head_seq.push_back(i); }
                else { draw_rows.push_back(lastr); draw_seq.push_back(i); }
            }
            r0 += n_rows[i];
        }
        n_out = (int)head_rows.size();
        head_rows.insert(head_rows.end(), draw_rows.begin(), draw_rows.end());
        head_seq.insert(head_seq.end(), draw_seq.begin(), draw_seq.end());
    }
    const int R = (int)head_rows.size();

    // ---- upload the step descriptor ----
    int32_t* d = m->p_desc;
    d[0] = n_seqs; d[1] = T;
    memcpy(d + 2, slot, (size_t)n_seqs * 4);
    memcpy(d + 2 + n_seqs, pos, (size_t)n_seqs * 4);
    memcpy(d + 2 + 2 * n_seqs, n_rows, (size_t)n_seqs * 4);
    CUDA_TRY(ctx, cudaEventRecord(m->ev0, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_desc, d, (size_t)(2 + 3 * n_seqs) * 4, cudaMemcpyHostToDevice, ctx->stream));
    int32_t* p_tail = d + 2 + 3 * m->MR;  // head_rows[MR], row_mask[MR], tokens[MR], draws[MR]
    int32_t* p_head = p_tail;
    int32_t* p_mask = p_tail + m->MR;
    int32_t* p_tok = p_tail + 2 * m->MR;
    b200_draw* p_draw = (b200_draw*)(p_tail + 3 * m->MR);
    for (int j = 0; j < R; j++) {
        p_head[j] = head_rows[j];
        p_mask[j] = (mask_index && logit_mask && mask_index[head_seq[j]] >= 0 && mask_index[head_seq[j]] < n_masks) ? mask_index[head_seq[j]] : -1;
        p_draw[j] = (j >= n_out) ? draws[head_seq[j]] : b200_draw{B200_DRAW_LOGITS, 0, 0, 0, 0};
    }
    bool any_mask = false;
    for (int j = 0; j < R; j++) any_mask |= p_mask[j] >= 0;
    if (R) {
        CUDA_TRY(ctx, cudaMemcpyAsync(m->d_head_rows, p_head, (size_t)R * 4, cudaMemcpyHostToDevice, ctx->stream));
        CUDA_TRY(ctx, cudaMemcpyAsync(m->d_row_mask, p_mask, (size_t)R * 4, cudaMemcpyHostToDevice, ctx->stream));
        CUDA_TRY(ctx, cudaMemcpyAsync(m->d_draws, p_draw, (size_t)R * sizeof(b200_draw), cudaMemcpyHostToDevice, ctx->stream));
    }
    if (any_mask) {
        const size_t mb = (size_t)n_masks * ((V + 31) / 32) * 4;
        if (mb > m->masks_cap) {
            if (m->d_masks) m->dfree(m->d_masks);
            ST_TRY(m->dalloc((void**)&m->d_masks, mb, &m->scratch_bytes));
            m->masks_cap = mb;
        }
        CUDA_TRY(ctx, cudaMemcpyAsync(m->d_masks, logit_mask, mb, cudaMemcpyHostToDevice, ctx->stream));
    }
    if (token_ids) {
        memcpy(p_tok, token_ids, (size_t)T * 4);
        CUDA_TRY(ctx, cudaMemcpyAsync(m->d_tokens, p_tok, (size_t)T * 4, cudaMemcpyHostToDevice, ctx->stream));
    } else {
        CUDA_TRY(ctx, cudaMemcpyAsync(m->h, embs, (size_t)T * H * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    // ---- device: map blocks, build row arrays, run the layers ----
    for (int i = 0; i < n_seqs; i++) ST_TRY(make_private(m, slot[i], pos[i], pos[i] + n_rows[i]));  // blocks shared with other slots
    prepare_step_kernel<<<1, 256, 0, ctx->stream>>>(m->d_desc, m->d_pos, 0, m->table, m->max_blocks, c.kv_block_rows,
                                                    m->slot_mapped, m->free_stack, m->free_count, m->d_seq_row0, m->d_row_slot,
                                                    m->d_row_pos, m->status, m->refs);
    LAUNCH_CHECK(ctx);
    // the host counters follow what the kernel does
    for (int i = 0; i < n_seqs; i++) m->h_append(slot[i], pos[i] + n_rows[i]);
    if (token_ids) ST_TRY(launch_embed_gather(ctx, m->embed.p, m->embed.kind, m->embed.rows, m->d_tokens, T, H, c.embed_scale, m->h));
    // the first sequence's rows, when they are many, form the tiled prefill run (fast class only)
    m->pf_rows = 0;
    if (!m->exact_scores && n_rows[0] >= kPrefillRunMin && prefill_attention_supported(c.n_heads, c.n_kv_heads, c.head_dim, c.kv_block_rows) &&
        !getenv("B200_NO_PREFILL_ATTN")) {
        m->pf_rows = n_rows[0];
        m->pf_slot = slot[0];
        m->pf_pos0 = pos[0];
        m->pf_tail_keys = 1;
        for (int i = 1; i < n_seqs; i++) m->pf_tail_keys = std::max(m->pf_tail_keys, pos[i] + n_rows[i]);
    }
    const int st_layers = run_layers(m, T, max_keys);
    m->pf_rows = 0;
    if (st_layers != B200_OK) return st_layers;
    // ---- head, in chunks of MLR rows ----
    if ((size_t)std::max(n_out, 1) * V * 4 > m->p_logits_cap) {
        if (m->p_logits) cudaFreeHost(m->p_logits);
        m->p_logits_cap = (size_t)std::max(n_out, 1) * V * 4;
        CUDA_TRY(ctx, cudaMallocHost((void**)&m->p_logits, m->p_logits_cap));
    }
    for (int j0 = 0; j0 < R; j0 += m->MLR) {
        const int rn = std::min(m->MLR, R - j0);
        const bool hq = is_kquant(m->head.kind);
        ST_TRY(launch_add_rmsnorm_quant(ctx, m->h, nullptr, m->final_norm, rn, H, c.rms_eps, hq ? nullptr : m->hn,
                                        hq ? m->aq_h : ActQ{}, m->d_head_rows + j0));
        ST_TRY(head_logits(m, rn));
        if (c.final_softcap > 0.f) ST_TRY(launch_softcap(ctx, m->logits, (size_t)rn * V, c.final_softcap));
        if (any_mask) ST_TRY(launch_mask_logits(ctx, m->logits, rn, V, m->d_row_mask + j0, m->d_masks));
        const int out_here = std::max(0, std::min(n_out, j0 + rn) - j0);
        if (out_here && logits_out)
            CUDA_TRY(ctx, cudaMemcpyAsync(m->p_logits + (size_t)j0 * V, m->logits, (size_t)out_here * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (j0 + rn > n_out) ST_TRY(launch_draw(ctx, m->logits, rn, V, m->d_draws + j0, m->d_ids + j0, nullptr));
    }
    if (R > n_out) CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids, m->d_ids, (size_t)R * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR, m->err_flag, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR + 1, m->status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaEventRecord(m->ev1, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    ST_TRY(check_device_flags(m, "the step"));
    if (n_out && logits_out) memcpy(logits_out, m->p_logits, (size_t)n_out * V * 4);
    if (ids_out) {
        for (int i = 0; i < n_seqs; i++) ids_out[i] = -1;
        for (int j = n_out; j < R; j++) ids_out[head_seq[j]] = m->p_ids[j];
    }
    if (n_logit_rows_out) *n_logit_rows_out = n_out;
    float ms = 0;
    cudaEventElapsedTime(&ms, m->ev0, m->ev1);
    m->stats.steps++;
    m->stats.rows += T;
    if (prefill_prompt_len && prefill_prompt_len[0] > 0) m->stats.prefill_rows += n_rows[0];
    m->stats.last_step_device_ms = ms;
    return B200_OK;
}

int b200_forward(b200_model* m, int slot, const float* emb, int token_id, int pos, int out_kind, float* logits_out, int32_t* id_out) {
    const int32_t one = 1, s = slot, p = pos, tok = token_id;
    b200_draw dr{out_kind == 1 ? B200_DRAW_GREEDY : B200_DRAW_LOGITS, 0, 0, 0, 0};
    int32_t id = -1;
    // ForwardNoLogits still runs the LM head here; its result is simply not copied out
    int st = b200_step_ragged(m, 1, &s, &p, &one, nullptr, nullptr, emb, emb ? nullptr : &tok, &dr, nullptr, nullptr, 0,
                              out_kind == 0 ? logits_out : nullptr, &id, nullptr);
    if (id_out) *id_out = id;
    return st;
}

int b200_forward_topk(b200_model* m, int slot, const float* emb, int token_id, int pos, int k, float inv_temperature,
                      int32_t* ids_out, float* logits_out, double* z_out) {
    b200_ctx* ctx = m->ctx;
    if (!ids_out || !logits_out) B200_FAIL(ctx, B200_BAD_ARGUMENT, "top-K needs its output buffers");
    // the row's logits stay on the device (a greedy-draw step reads nothing back but an id); the selection runs over them
    const int32_t one = 1, s = slot, p = pos, tok = token_id;
    b200_draw dr{B200_DRAW_GREEDY, 0, 0, 0, 0};
    int32_t id = -1;
    ST_TRY(b200_step_ragged(m, 1, &s, &p, &one, nullptr, nullptr, emb, emb ? nullptr : &tok, &dr, nullptr, nullptr, 0, nullptr, &id, nullptr));
    if (!m->d_topk) {
        ST_TRY(m->dalloc((void**)&m->d_topk, (size_t)1024 * 8 + 8, &m->scratch_bytes));
    }
    int32_t* di = reinterpret_cast<int32_t*>(m->d_topk);
    float* dv = reinterpret_cast<float*>(di + 1024);
    double* dz = reinterpret_cast<double*>(dv + 1024);
    ST_TRY(launch_topk(ctx, m->logits, 1, m->c.vocab, k, inv_temperature, z_out != nullptr, di, dv, dz));
    CUDA_TRY(ctx, cudaMemcpyAsync(ids_out, di, (size_t)k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(logits_out, dv, (size_t)k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (z_out) CUDA_TRY(ctx, cudaMemcpyAsync(z_out, dz, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return B200_OK;
}

int b200_prefill_last(b200_model* m, int slot, int n, const float* embs, const int32_t* token_ids, int start_pos, float* logits_out) {
    const int32_t s = slot, p = start_pos, nr = n, pl = start_pos + n;
    const uint8_t last = 1;
    return b200_step_ragged(m, 1, &s, &p, &nr, &pl, &last, embs, token_ids, nullptr, nullptr, nullptr, 0, logits_out, nullptr, nullptr);
}

int b200_decode_loop_device(b200_model* m, int n_seqs, const int32_t* slot, const int32_t* pos0, const int32_t* first_ids, int steps,
                            int advance_pos, int32_t* ids_out, float* ms_out) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    if (!m->finalized || n_seqs <= 0 || n_seqs > m->MR || n_seqs > m->MLR || steps <= 0) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad decode loop arguments");
    const int H = c.hidden, V = c.vocab, S = n_seqs;
    int need = 0, max_keys = 0;
    {
        std::vector<char> seen(c.n_slots, 0);
        for (int i = 0; i < S; i++) {
            if (slot[i] < 0 || slot[i] >= c.n_slots || seen[slot[i]]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "slot %d out of range or repeated", slot[i]);
            seen[slot[i]] = 1;
            const int end = pos0[i] + (advance_pos ? steps : 1);
            if (pos0[i] < 0 || end > c.ctx_cap || pos0[i] > m->h_slot_len[slot[i]]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "sequence %d outside its slot", i);
            if (first_ids[i] < 0 || first_ids[i] >= V) B200_FAIL(ctx, B200_BAD_ARGUMENT, "token id out of range");
            need += blocks_needed(m, slot[i], end) + m->h_cow_need(slot[i], pos0[i], end);
            max_keys = std::max(max_keys, end);
        }
    }
    if (need > m->h_free) { m->stats.kv_pool_full++; B200_FAIL(ctx, B200_KV_POOL_FULL, "kv pool full: %d blocks needed, %d free", need, m->h_free); }
    for (int i = 0; i < S; i++) ST_TRY(make_private(m, slot[i], pos0[i], pos0[i] + (advance_pos ? steps : 1)));
    if (ids_out && !m->d_ids_log) ST_TRY(m->dalloc((void**)&m->d_ids_log, (size_t)m->MR * 4, &m->scratch_bytes));
    int32_t* d = m->p_desc;
    d[0] = S; d[1] = S;
    memcpy(d + 2, slot, (size_t)S * 4);
    memcpy(d + 2 + S, pos0, (size_t)S * 4);
    for (int i = 0; i < S; i++) d[2 + 2 * S + i] = 1;
    int32_t* p_tail = d + 2 + 3 * m->MR;
    b200_draw* p_draw = (b200_draw*)(p_tail + 3 * m->MR);
    for (int i = 0; i < S; i++) { p_tail[i] = i; p_tail[2 * m->MR + i] = first_ids[i]; p_draw[i] = b200_draw{B200_DRAW_GREEDY, 0, 0, 0, 0}; }
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_desc, d, (size_t)(2 + 3 * S) * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_pos, pos0, (size_t)S * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_head_rows, p_tail, (size_t)S * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_tokens, p_tail + 2 * m->MR, (size_t)S * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->d_draws, p_draw, (size_t)S * sizeof(b200_draw), cudaMemcpyHostToDevice, ctx->stream));
    std::vector<int32_t> log;
    if (ids_out) log.resize((size_t)steps * S);
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaEventRecord(m->ev0, ctx->stream));
    auto one_step = [&](int st) -> int {
        prepare_step_kernel<<<1, 256, 0, ctx->stream>>>(m->d_desc, m->d_pos, 1, m->table, m->max_blocks, c.kv_block_rows,
                                                        m->slot_mapped, m->free_stack, m->free_count, m->d_seq_row0,
                                                        m->d_row_slot, m->d_row_pos, m->status, m->refs);
        LAUNCH_CHECK(ctx);
        ST_TRY(launch_embed_gather(ctx, m->embed.p, m->embed.kind, m->embed.rows, m->d_tokens, S, H, c.embed_scale, m->h));
        ST_TRY(run_layers(m, S, max_keys));
        const bool hq = is_kquant(m->head.kind);
        ST_TRY(launch_add_rmsnorm_quant(ctx, m->h, nullptr, m->final_norm, S, H, c.rms_eps, hq ? nullptr : m->hn,
                                        hq ? m->aq_h : ActQ{}, m->d_head_rows));
        ST_TRY(head_logits(m, S));
        if (c.final_softcap > 0.f) ST_TRY(launch_softcap(ctx, m->logits, (size_t)S * V, c.final_softcap));
        ST_TRY(launch_draw(ctx, m->logits, S, V, m->d_draws, m->d_ids, nullptr));
        advance_kernel<<<ceil_div(S, 256), 256, 0, ctx->stream>>>(m->d_tokens, m->d_ids, m->d_pos, S, advance_pos, ids_out ? m->d_ids_log : nullptr);
        LAUNCH_CHECK(ctx);
        if (ids_out) CUDA_TRY(ctx, cudaMemcpyAsync(log.data() + (size_t)st * S, m->d_ids_log, (size_t)S * 4, cudaMemcpyDeviceToHost, ctx->stream));
        return B200_OK;
    };
    // A step's launches do not depend on the step (positions and tokens advance on the device), so from the second step on
    // the loop replays one captured CUDA graph: several hundred launches become one. Kept off when ids are logged to the
    // host every step, when kernels are being event-profiled, and under tensor parallel (the collectives stay eager).
    static const bool no_graph = getenv("B200_NO_GRAPH") != nullptr;
    const bool use_graph = steps >= 3 && !ids_out && ctx->prof_mask == 0 && c.tp_size <= 1 && !no_graph;
    int done = 0;
    if (use_graph) {
        ST_TRY(one_step(0));  // eager: first-use set-up (function attributes, tensor maps) happens outside the capture
        done = 1;
        // grids depend on the key count only through the attention kernels' split count (the exact class: through the count itself)
        const int key_splits = m->exact_scores ? max_keys : ceil_div(max_keys, 512);
        if (!m->loop_graph || m->loop_graph_S != S || m->loop_graph_splits != key_splits || m->loop_graph_adv != advance_pos) {
            if (m->loop_graph) { cudaGraphExecDestroy(m->loop_graph); m->loop_graph = nullptr; }
            const int64_t l0 = ctx->launches;
            CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
            const int st_cap = one_step(1);
            cudaGraph_t g = nullptr;
            const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &g);
            if (st_cap != B200_OK) {
                if (g) cudaGraphDestroy(g);
                return st_cap;
            }
            if (ce != cudaSuccess || !g) B200_FAIL(ctx, B200_CUDA_ERROR, "capturing the decode step failed: %s", cudaGetErrorString(ce));
            m->loop_graph_launches = ctx->launches - l0;
            ctx->launches = l0;  // capturing launched nothing
            const cudaError_t ie = cudaGraphInstantiate(&m->loop_graph, g, 0);
            cudaGraphDestroy(g);
            if (ie != cudaSuccess) {
                m->loop_graph = nullptr;
                B200_FAIL(ctx, B200_CUDA_ERROR, "instantiating the decode step's graph failed: %s", cudaGetErrorString(ie));
            }
            m->loop_graph_S = S;
            m->loop_graph_splits = key_splits;
            m->loop_graph_adv = advance_pos;
        }
        for (; done < steps; done++) {
            CUDA_TRY(ctx, cudaGraphLaunch(m->loop_graph, ctx->stream));
            ctx->launches += m->loop_graph_launches;
        }
    }
    for (int st = done; st < steps; st++) ST_TRY(one_step(st));
    CUDA_TRY(ctx, cudaEventRecord(m->ev1, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR, m->err_flag, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR + 1, m->status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    ST_TRY(check_device_flags(m, "the decode loop"));
    float ms = 0;
    cudaEventElapsedTime(&ms, m->ev0, m->ev1);
    if (ms_out) *ms_out = ms;
    if (ids_out) memcpy(ids_out, log.data(), log.size() * 4);
    // The mirror pops blocks in the order the device did: step by step, and within a step sequence by sequence (a sequence
    // by sequence replay would hand two sequences that cross block edges in different steps each other's ids).
    for (int st = 0; st < (advance_pos ? steps : 1); st++)
        for (int i = 0; i < S; i++) m->h_append(slot[i], pos0[i] + st + 1);
    m->stats.steps += steps;
    m->stats.rows += (int64_t)steps * S;
    m->stats.last_step_device_ms = ms / steps;
    return B200_OK;
}

// ---- the device batch (scheduler.Admission's admit / retire mapped onto the device: internal/runtime/scheduler/admission.go:60-122) ----
// b200_batch_open binds seats to slots; between runs the host prefills a seat's slot (b200_prefill_last / b200_step_ragged)
// and admits the sequence at its next position with the token to feed; b200_batch_run then decodes `steps` greedy steps for
// every seat with nothing packed or uploaded per step: commands are applied on the device at the first step's boundary,
// ids are fed back, positions advance, a seat retires itself at its end-of-sequence id or token budget, and one record per
// seat and step comes back. The blocks a seat's sequence can still take are reserved at admission, so a run cannot find
// the pool empty.
int b200_batch_open(b200_model* m, int n_seats, int first_slot, int park_slot, int max_steps) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    auto& q = m->seats;
    if (!m->finalized || q.n || n_seats < 1 || n_seats > m->MR || n_seats > m->MLR || first_slot < 0 || first_slot + n_seats > c.n_slots || park_slot < 0 ||
        park_slot >= c.n_slots || (park_slot >= first_slot && park_slot < first_slot + n_seats) || max_steps < 1)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: %d seats from slot %d, parking slot %d, %d steps a run", n_seats, first_slot, park_slot, max_steps);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    size_t* sb = &m->scratch_bytes;
    const int S = n_seats;
    ST_TRY(m->dalloc((void**)&q.live, (size_t)S * 4, sb));
    ST_TRY(m->dalloc((void**)&q.remaining, (size_t)S * 4, sb));
    ST_TRY(m->dalloc((void**)&q.eos, (size_t)S * 4, sb));
    ST_TRY(m->dalloc((void**)&q.desc, (size_t)(2 + 3 * S) * 4, sb));
    ST_TRY(m->dalloc((void**)&q.pos, (size_t)S * 4, sb));
    ST_TRY(m->dalloc((void**)&q.tokens, (size_t)S * 4, sb));
    ST_TRY(m->dalloc((void**)&q.rows, (size_t)S * 4, sb));
    ST_TRY(m->dalloc((void**)&q.draws, (size_t)S * sizeof(b200_draw), sb));
    ST_TRY(m->dalloc((void**)&q.step, 4, sb));
    ST_TRY(m->dalloc(&q.cmds, (size_t)2 * S * sizeof(SeatCmd), sb));
    ST_TRY(m->dalloc(&q.events, (size_t)max_steps * S * sizeof(SeatEvent), sb));
    std::vector<int32_t> d(2 + 3 * S), iota(S);
    std::vector<b200_draw> dr(S, b200_draw{B200_DRAW_GREEDY, 0, 0, 0, 0});
    d[0] = S; d[1] = S;
    for (int i = 0; i < S; i++) { d[2 + i] = park_slot; d[2 + S + i] = 0; d[2 + 2 * S + i] = 1; iota[i] = i; }
    CUDA_TRY(ctx, cudaMemcpyAsync(q.desc, d.data(), d.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(q.rows, iota.data(), (size_t)S * 4, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(q.draws, dr.data(), (size_t)S * sizeof(b200_draw), cudaMemcpyHostToDevice, ctx->stream));
    for (int32_t* z : {q.live, q.remaining, q.eos, q.pos, q.tokens}) CUDA_TRY(ctx, cudaMemsetAsync(z, 0, (size_t)S * 4, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    q.n = S; q.first_slot = first_slot; q.park_slot = park_slot; q.max_steps = max_steps;
    q.h_live.assign(S, 0); q.h_pos.assign(S, 0); q.h_end.assign(S, 0);
    q.pending.clear();
    return B200_OK;
}

namespace {
// blocks the seats' sequences (and the parking slot) may still take, seat `skip` left out
int seats_reserved(b200_model* m, int skip) {
    auto& q = m->seats;
    int need = blocks_needed(m, q.park_slot, 1);
    for (int i = 0; i < q.n; i++)
        if (i != skip && q.h_live[i]) need += blocks_needed(m, q.first_slot + i, q.h_end[i]);
    return need;
}
}  // namespace

int b200_batch_admit(b200_model* m, int seat, int pos, int token, int max_new, int eos_id) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    auto& q = m->seats;
    if (!q.n || seat < 0 || seat >= q.n) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: no seat %d", seat);
    const int slot = q.first_slot + seat, end = pos + max_new;
    if (q.h_live[seat]) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: seat %d holds a sequence", seat);
    if (pos < 0 || max_new < 1 || end > c.ctx_cap || pos > m->h_slot_len[slot] || token < 0 || token >= c.vocab)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: seat %d cannot continue at position %d for %d tokens (its slot stores %d rows, capacity %d)", seat, pos,
                  max_new, m->h_slot_len[slot], c.ctx_cap);
    if ((int)q.pending.size() / 6 >= 2 * q.n) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: too many commands before a run");
    // the blocks this sequence can still take (and the copies a shared block costs) must be there beside every other seat's
    const int need = blocks_needed(m, slot, end) + m->h_cow_need(slot, pos, end);
    if (need + seats_reserved(m, seat) > m->h_free) {
        m->stats.kv_pool_full++;
        B200_FAIL(ctx, B200_KV_POOL_FULL, "kv pool full: seat %d needs %d blocks, %d are reserved, %d free", seat, need, seats_reserved(m, seat), m->h_free);
    }
    ST_TRY(make_private(m, slot, pos, end));
    q.h_live[seat] = 1; q.h_pos[seat] = pos; q.h_end[seat] = end;
    const int32_t cmd[6] = {1, seat, pos, token, max_new, eos_id};
    q.pending.insert(q.pending.end(), cmd, cmd + 6);
    return B200_OK;
}

int b200_batch_retire(b200_model* m, int seat) {
    b200_ctx* ctx = m->ctx;
    auto& q = m->seats;
    if (!q.n || seat < 0 || seat >= q.n) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: no seat %d", seat);
    if ((int)q.pending.size() / 6 >= 2 * q.n) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: too many commands before a run");
    q.h_live[seat] = 0;
    const int32_t cmd[6] = {2, seat, 0, 0, 0, 0};
    q.pending.insert(q.pending.end(), cmd, cmd + 6);
    return B200_OK;
}

int b200_batch_run(b200_model* m, int steps, int32_t* events_out, int max_events, int32_t* n_events_out) {
    b200_ctx* ctx = m->ctx;
    const b200_model_cfg& c = m->c;
    auto& q = m->seats;
    const int S = q.n, H = c.hidden, V = c.vocab;
    if (!S || steps < 1 || steps > q.max_steps || !n_events_out || (max_events > 0 && !events_out))
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: %d steps (at most %d a run)", steps, q.max_steps);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ctx->umma_scratch = m->umma_scratch;
    ctx->umma_scratch_bytes = m->umma_bytes;
    ctx->x16_slot_bytes = m->x16_slot_bytes;
    ctx->err_flag = m->err_flag;
    if (seats_reserved(m, -1) > m->h_free) {   // (other calls took blocks since the admissions)
        m->stats.kv_pool_full++;
        B200_FAIL(ctx, B200_KV_POOL_FULL, "kv pool full: the seats' sequences may take %d blocks, %d free", seats_reserved(m, -1), m->h_free);
    }
    const int n_cmd = (int)q.pending.size() / 6;
    if (n_cmd) {
        CUDA_TRY(ctx, cudaMemcpyAsync(q.cmds, q.pending.data(), q.pending.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        seats_apply_kernel<<<1, 32, 0, ctx->stream>>>((const SeatCmd*)q.cmds, n_cmd, q.desc + 2, q.first_slot, q.park_slot, q.live, q.pos, q.tokens, q.remaining, q.eos);
        LAUNCH_CHECK(ctx);
        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));   // the commands' host buffer is reused
        q.pending.clear();
    }
    int max_keys = 1;
    for (int i = 0; i < S; i++)
        if (q.h_live[i]) max_keys = std::max(max_keys, std::min(q.h_end[i], q.h_pos[i] + steps));
    // rounded up to whole attention splits, so that a captured step's arguments hold for every run with that split count
    if (!m->exact_scores) max_keys = std::min(c.ctx_cap, ceil_div(max_keys, 512) * 512);
    CUDA_TRY(ctx, cudaMemsetAsync(q.step, 0, 4, ctx->stream));
    CUDA_TRY(ctx, cudaEventRecord(m->ev0, ctx->stream));
    auto one_step = [&]() -> int {
        prepare_step_kernel<<<1, 256, 0, ctx->stream>>>(q.desc, q.pos, 1, m->table, m->max_blocks, c.kv_block_rows, m->slot_mapped, m->free_stack,
                                                        m->free_count, m->d_seq_row0, m->d_row_slot, m->d_row_pos, m->status, m->refs);
        LAUNCH_CHECK(ctx);
        ST_TRY(launch_embed_gather(ctx, m->embed.p, m->embed.kind, m->embed.rows, q.tokens, S, H, c.embed_scale, m->h));
        ST_TRY(run_layers(m, S, max_keys));
        const bool hq = is_kquant(m->head.kind);
        ST_TRY(launch_add_rmsnorm_quant(ctx, m->h, nullptr, m->final_norm, S, H, c.rms_eps, hq ? nullptr : m->hn, hq ? m->aq_h : ActQ{}, q.rows));
        ST_TRY(head_logits(m, S));
        if (c.final_softcap > 0.f) ST_TRY(launch_softcap(ctx, m->logits, (size_t)S * V, c.final_softcap));
        ST_TRY(launch_draw(ctx, m->logits, S, V, q.draws, m->d_ids, nullptr));
        seats_advance_kernel<<<ceil_div(S, 256), 256, 0, ctx->stream>>>(S, m->d_ids, q.desc + 2, q.park_slot, q.live, q.pos, q.tokens, q.remaining, q.eos,
                                                                       (SeatEvent*)q.events, q.step);
        LAUNCH_CHECK(ctx);
        seats_next_step_kernel<<<1, 1, 0, ctx->stream>>>(q.step);
        LAUNCH_CHECK(ctx);
        return B200_OK;
    };
    // Every step is the same launches (who is seated, positions, tokens and the step count live on the device), so from its
    // second step on a run replays one captured CUDA graph, kept from run to run while the attention kernels' split count
    // stays. Off while kernels are being event-profiled and under tensor parallel (the collectives stay eager).
    static const bool no_graph = getenv("B200_NO_GRAPH") != nullptr;
    const bool use_graph = steps >= 3 && ctx->prof_mask == 0 && c.tp_size <= 1 && !no_graph;
    int done = 0;
    if (use_graph) {
        ST_TRY(one_step());  // eager: first-use set-up (function attributes, tensor maps) happens outside the capture
        done = 1;
        const int key_splits = m->exact_scores ? max_keys : ceil_div(max_keys, 512);
        if (!q.graph || q.graph_splits != key_splits) {
            if (q.graph) { cudaGraphExecDestroy(q.graph); q.graph = nullptr; }
            const int64_t l0 = ctx->launches;
            CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
            const int st_cap = one_step();
            cudaGraph_t gr = nullptr;
            const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &gr);
            if (st_cap != B200_OK) {
                if (gr) cudaGraphDestroy(gr);
                return st_cap;
            }
            if (ce != cudaSuccess || !gr) B200_FAIL(ctx, B200_CUDA_ERROR, "capturing the batch step failed: %s", cudaGetErrorString(ce));
            q.graph_launches = ctx->launches - l0;
            ctx->launches = l0;  // capturing launched nothing
            const cudaError_t ie = cudaGraphInstantiate(&q.graph, gr, 0);
            cudaGraphDestroy(gr);
            if (ie != cudaSuccess) {
                q.graph = nullptr;
                B200_FAIL(ctx, B200_CUDA_ERROR, "instantiating the batch step's graph failed: %s", cudaGetErrorString(ie));
            }
            q.graph_splits = key_splits;
        }
        for (; done < steps; done++) {
            CUDA_TRY(ctx, cudaGraphLaunch(q.graph, ctx->stream));
            ctx->launches += q.graph_launches;
        }
    }
    for (; done < steps; done++) ST_TRY(one_step());
    CUDA_TRY(ctx, cudaEventRecord(m->ev1, ctx->stream));
    std::vector<SeatEvent> ev((size_t)steps * S);
    CUDA_TRY(ctx, cudaMemcpyAsync(ev.data(), q.events, ev.size() * sizeof(SeatEvent), cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR, m->err_flag, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(m->p_ids + m->MR + 1, m->status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    ST_TRY(check_device_flags(m, "a run of the device batch"));
    // The mirror pops blocks in the order the device did (step by step, seat by seat), and the host's view of the seats
    // follows the records.
    int n_out = 0;
    for (int st = 0; st < steps; st++)
        for (int i = 0; i < S; i++) {
            const SeatEvent& e = ev[(size_t)st * S + i];
            if (e.flags & 1) {
                m->h_append(q.first_slot + i, e.pos + 1);
                q.h_pos[i] = e.pos + 1;
                if (e.flags & 2) q.h_live[i] = 0;
                if (n_out < max_events) {
                    events_out[4 * n_out] = i; events_out[4 * n_out + 1] = e.id; events_out[4 * n_out + 2] = e.pos; events_out[4 * n_out + 3] = e.flags;
                }
                n_out++;
                m->stats.rows++;
            } else {
                m->h_append(q.park_slot, 1);
            }
        }
    *n_events_out = n_out;
    float ms = 0;
    cudaEventElapsedTime(&ms, m->ev0, m->ev1);
    m->stats.steps += steps;
    m->stats.last_step_device_ms = ms / steps;
    if (n_out > max_events) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device batch: %d records, room for %d", n_out, max_events);
    return B200_OK;
}

int b200_batch_close(b200_model* m) {
    auto& q = m->seats;
    if (!q.n) return B200_OK;
    cudaStreamSynchronize(m->ctx->stream);
    if (q.graph) cudaGraphExecDestroy(q.graph);
    for (void* p : {(void*)q.live, (void*)q.remaining, (void*)q.eos, (void*)q.desc, (void*)q.pos, (void*)q.tokens, (void*)q.rows, (void*)q.draws, (void*)q.step, q.cmds, q.events})
        m->dfree(p);
    q = b200_model::Seats{};
    return B200_OK;
}

// Debug tap: the residual stream after the last layer of the latest step, [rows][hidden].
int b200_debug_read_hidden(b200_model* m, float* out, int n) {
    CUDA_TRY(m->ctx, cudaStreamSynchronize(m->ctx->stream));
    const float* src = m->h;
    if (const char* w = getenv("B200_DEBUG_TAP")) {  // qkv | ctx | att: the last layer's buffers
        if (!strcmp(w, "qkv")) src = m->qkv;
        if (!strcmp(w, "ctx")) src = m->ctxb;
        if (!strcmp(w, "att")) src = m->att;
    }
    CUDA_TRY(m->ctx, cudaMemcpy(out, src, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return B200_OK;
}

int b200_profile(b200_ctx* ctx, unsigned tag_mask) {
    ctx->prof_mask = tag_mask;
    return B200_OK;
}

int b200_profile_read(b200_ctx* ctx, double* ms_by_tag, int64_t* launches_by_tag, int n_tags) {
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < n_tags; i++) { ms_by_tag[i] = 0; launches_by_tag[i] = 0; }
    for (auto& r : ctx->prof_recs) {
        float ms = 0;
        cudaEventElapsedTime(&ms, r.e0, r.e1);
        if (r.tag < n_tags) { ms_by_tag[r.tag] += ms; launches_by_tag[r.tag]++; }
        ctx->prof_pool.push_back(r.e0);
        ctx->prof_pool.push_back(r.e1);
    }
    ctx->prof_recs.clear();
    return B200_OK;
}

int b200_stats(b200_model* m, b200_stats_t* out) {
    *out = m->stats;
    out->kernel_launches = m->ctx->launches;
    out->kv_blocks_in_use = m->c.kv_pool_blocks - 1 - m->h_free;
    return B200_OK;
}

}  // extern "C"

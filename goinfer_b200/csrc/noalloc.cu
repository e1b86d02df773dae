// noalloc.cu — paged decode attention for callers that cannot allocate device memory.
//
// The split-K attention kernels park per-split partial results (an accumulator row, a running maximum and a running
// sum per head and split) in global scratch before a second kernel merges them. Everywhere else in this library that
// scratch comes from cudaMalloc at model build time. Some hosts never get to call an allocator at the moment they
// need attention: a step that runs inside a memory-frozen serving process whose pool was carved up at start-up, or a
// plug-in loaded into somebody else's process under a "no device allocations after init" rule, where a cudaMalloc in
// the step would break the host's memory budget. For them b200_attention_noalloc uses the fixed array below.
//
// The array is part of the library image: every GPU that loads the library carries its 16 MiB until the process exits,
// whether or not the entry point is ever called.
#include <mutex>

#include "common.cuh"

#define NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)  // 16 MiB

// Device storage. In host code the name is only a handle for the runtime's symbol table, never an address a kernel
// may be given; the address is asked for once per device with cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;
}  // namespace

namespace {
// Makes `want` the calling thread's current device for the length of a call and puts the caller's own back afterwards.
struct DeviceScope {
    int prev = -1;
    bool switched = false;
    cudaError_t enter(int want) {
        cudaError_t e = cudaGetDevice(&prev);
        if (e != cudaSuccess) return e;
        if (prev == want) return cudaSuccess;
        e = cudaSetDevice(want);
        switched = e == cudaSuccess;
        return e;
    }
    ~DeviceScope() {
        if (switched) cudaSetDevice(prev);
    }
};
}  // namespace

extern "C" int b200_attention_noalloc(b200_ctx* ctx, const float* q, int ldq, int rows, int n_heads, int n_kv_heads,
                                      int head_dim, float scale, float softcap, const int32_t* row_slot,
                                      const int32_t* row_pos, int max_keys, const void* k_pool, const void* v_pool,
                                      const int32_t* block_table, int max_blocks, int block_rows, float* out) {
    if (!ctx) return B200_BAD_ARGUMENT;
    if (!q || !row_slot || !row_pos || !k_pool || !v_pool || !block_table || !out || rows <= 0 || max_keys <= 0 ||
        n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_heads % n_kv_heads || ldq < n_heads * head_dim)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "b200_attention_noalloc: null pointer or bad shape");
    const int G = n_heads / n_kv_heads;
    if (!((head_dim == 64 || head_dim == 128) && (G == 1 || G == 2 || G == 4 || G == 8)) || block_rows <= 0 || block_rows % 16 != 0)
        B200_FAIL(ctx, B200_BAD_ARGUMENT,
                  "b200_attention_noalloc: only head_dim 64/128, group size 1/2/4/8 and KV blocks of a positive multiple of 16 rows "
                  "use the split kernels this entry point serves (got head_dim %d, group %d, block_rows %d)", head_dim, G, block_rows);
    // every key below max_keys must have a table entry: the kernels index block_table[key / block_rows] of a row's table
    if (max_blocks <= 0 || (long long)max_blocks * block_rows < (long long)max_keys)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "b200_attention_noalloc: %d table entries of %d rows cannot hold %d keys", max_blocks, block_rows, max_keys);
    // the kernels read q in 8-byte pairs, the pools in 16-byte tile chunks and write out in 8-byte pairs
    if ((reinterpret_cast<uintptr_t>(q) & 7) || (ldq & 1) || (reinterpret_cast<uintptr_t>(k_pool) & 15) ||
        (reinterpret_cast<uintptr_t>(v_pool) & 15) || (reinterpret_cast<uintptr_t>(out) & 7) ||
        (reinterpret_cast<uintptr_t>(row_slot) & 3) || (reinterpret_cast<uintptr_t>(row_pos) & 3) || (reinterpret_cast<uintptr_t>(block_table) & 3))
        B200_FAIL(ctx, B200_BAD_ARGUMENT,
                  "b200_attention_noalloc: q and out must be 8-byte aligned with an even ldq, the pools 16-byte aligned, the int arrays 4-byte aligned");
    if (ctx->device < 0 || ctx->device >= kMaxDevices) B200_FAIL(ctx, B200_BAD_ARGUMENT, "device ordinal out of range");
    // the partials of every row, head and split must fit the fixed array
    const int max_splits = ceil_div(max_keys, attn_split_keys());
    const size_t need = attn_scratch_floats(rows, n_heads, head_dim, max_splits);
    if (need > (size_t)NOALLOC_SCRATCH_FLOATS)
        B200_FAIL(ctx, B200_BAD_ARGUMENT,
                  "b200_attention_noalloc: %d rows x %d heads x %d splits need %zu bytes of scratch, the fixed array holds %zu; "
                  "use fewer rows per call or the allocating path", rows, n_heads, max_splits, need * 4,
                  (size_t)NOALLOC_SCRATCH_FLOATS * 4);
    // The context's device is made current for this call (its stream and the array's address belong to it) and the
    // caller's own device is current again when the call returns.
    DeviceScope dev;
    CUDA_TRY(ctx, dev.enter(ctx->device));
    // One-time set-up on this device (first call only): resolve the array's device address with this device current.
    float* scratch;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        scratch = g_scratch_ptr[ctx->device];
        if (!scratch) {
            void* p = nullptr;
            CUDA_TRY(ctx, cudaGetSymbolAddress(&p, g_noalloc_scratch));
            scratch = g_scratch_ptr[ctx->device] = static_cast<float*>(p);
        }
    }
    // Nothing in the scratch has to start at zero: each (row, head, split) slot that the merge kernel reads is written
    // in full by the split kernel of the same call, so leftovers of an earlier call are never read. (A row whose
    // position is not below max_keys breaks the caller's side of the contract; the kernels then stay inside the table
    // and the array, and that row's output is meaningless.)
    KVView kv{const_cast<__half*>(static_cast<const __half*>(k_pool)), const_cast<__half*>(static_cast<const __half*>(v_pool)),
              block_table, max_blocks, block_rows, n_kv_heads, head_dim};
    AttnScratch sc;
    sc.partial = scratch;
    sc.max_splits = max_splits;
    const float s = scale != 0.f ? scale : 1.0f / sqrtf((float)head_dim);
    return launch_paged_attention(ctx, q, ldq, rows, n_heads, n_kv_heads, head_dim, s, softcap, row_slot, row_pos, max_keys, kv, sc,
                                  out, ActQ{});
}

// tp.cu — tensor-parallel plumbing: one NCCL communicator per context, looked up at run time.
//
// The 70B-class configuration splits every layer over t GPUs, one process per GPU: q/k/v/gate/up by output rows
// (heads, FFN columns), o/down by input columns, the KV cache by kv head; the partial [rows][hidden] products of the
// o and down projections are summed across ranks (all-reduce) and the LM head's vocabulary slices are gathered. The
// reference's CUDA backend is single-GPU; the split follows its column/row-split description of the tensor-parallel
// configuration. NCCL is not linked: libnccl.so.2 is opened with dlopen when the first communicator is made (the copy a
// host process already loaded, e.g. PyTorch's, is the one found), so a single-GPU host needs no NCCL at all.
#include <dlfcn.h>

#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace {

// the slice of NCCL's C API this file uses (nccl.h: ncclGetUniqueId, ncclCommInitRank, ncclCommDestroy, ncclAllReduce,
// ncclAllGather, ncclGetErrorString)
struct NcclUniqueId { char internal[128]; };
typedef void* NcclComm;
typedef int (*get_unique_id_fn)(NcclUniqueId*);
typedef int (*comm_init_rank_fn)(NcclComm*, int, NcclUniqueId, int);
typedef int (*comm_destroy_fn)(NcclComm);
typedef int (*all_reduce_fn)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*all_gather_fn)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
typedef const char* (*error_string_fn)(int);
constexpr int kNcclFloat32 = 7, kNcclSum = 0, kNcclUint8 = 1;

struct NcclApi {
    void* lib = nullptr;
    get_unique_id_fn get_unique_id = nullptr;
    comm_init_rank_fn comm_init_rank = nullptr;
    comm_destroy_fn comm_destroy = nullptr;
    all_reduce_fn all_reduce = nullptr;
    all_gather_fn all_gather = nullptr;
    error_string_fn error_string = nullptr;
    std::string why;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names)
            if ((api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
        if (!api.lib) {
            api.why = std::string("libnccl.so.2 could not be opened: ") + dlerror();
            return;
        }
        api.get_unique_id = (get_unique_id_fn)dlsym(api.lib, "ncclGetUniqueId");
        api.comm_init_rank = (comm_init_rank_fn)dlsym(api.lib, "ncclCommInitRank");
        api.comm_destroy = (comm_destroy_fn)dlsym(api.lib, "ncclCommDestroy");
        api.all_reduce = (all_reduce_fn)dlsym(api.lib, "ncclAllReduce");
        api.all_gather = (all_gather_fn)dlsym(api.lib, "ncclAllGather");
        api.error_string = (error_string_fn)dlsym(api.lib, "ncclGetErrorString");
        if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_reduce || !api.all_gather || !api.error_string) {
            api.why = "libnccl lacks a symbol this library needs";
            api.lib = nullptr;
        }
    });
    return &api;
}

#define NCCL_TRY(ctx, api, expr)                                                                         \
    do {                                                                                                 \
        int r_ = (expr);                                                                                 \
        if (r_ != 0) B200_FAIL(ctx, B200_NCCL_ERROR, "NCCL: %s (%s)", (api)->error_string(r_), #expr);   \
    } while (0)

// [t][rows][w] -> [rows][t*w]
__global__ void interleave_slices_kernel(const float* __restrict__ in, int t, int rows, int w, float* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = (size_t)t * rows * w;
    if (i >= n) return;
    const int c = (int)(i % w);
    const int r = (int)((i / w) % rows);
    const int k = (int)(i / ((size_t)w * rows));
    out[(size_t)r * t * w + (size_t)k * w + c] = in[i];
}

}  // namespace

int b200_tp_unique_id(b200_ctx* ctx, void* id_out, size_t bytes) {
    if (!id_out || bytes < sizeof(NcclUniqueId)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the unique id takes %zu bytes", sizeof(NcclUniqueId));
    NcclApi* api = nccl_api();
    if (!api->lib) B200_FAIL(ctx, B200_NCCL_ERROR, "%s", api->why.c_str());
    NCCL_TRY(ctx, api, api->get_unique_id(reinterpret_cast<NcclUniqueId*>(id_out)));
    return B200_OK;
}

int b200_tp_init(b200_ctx* ctx, const void* id, size_t bytes, int rank, int size) {
    if (!id || bytes < sizeof(NcclUniqueId) || size < 1 || rank < 0 || rank >= size) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad tensor-parallel rank %d of %d", rank, size);
    if (ctx->tp_comm) B200_FAIL(ctx, B200_BAD_ARGUMENT, "the context already has a communicator");
    NcclApi* api = nccl_api();
    if (!api->lib) B200_FAIL(ctx, B200_NCCL_ERROR, "%s", api->why.c_str());
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    NcclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    NcclComm comm = nullptr;
    NCCL_TRY(ctx, api, api->comm_init_rank(&comm, size, uid, rank));
    ctx->tp_comm = comm;
    ctx->tp_rank = rank;
    ctx->tp_size = size;
    return B200_OK;
}

int b200_tp_destroy(b200_ctx* ctx) {
    if (!ctx->tp_comm) return B200_OK;
    NcclApi* api = nccl_api();
    cudaStreamSynchronize(ctx->stream);
    const int r = api->comm_destroy(ctx->tp_comm);
    ctx->tp_comm = nullptr;
    ctx->tp_size = 1;
    ctx->tp_rank = 0;
    if (r != 0) B200_FAIL(ctx, B200_NCCL_ERROR, "NCCL: %s (ncclCommDestroy)", api->error_string(r));
    return B200_OK;
}

// ---- the peer-visible step buffers of launch_tp_reduce_norm_quant ----
// Every rank allocates its block, the 64-byte inter-process handles are traded with one all-gather on the communicator,
// and each rank maps the others' blocks (which also turns peer access on). Whether every rank managed is then agreed
// with one all-reduce, so that either all of them run the fused kernel or all of them keep NCCL's all-reduce.
int tp_fused_setup(b200_ctx* ctx, TpFused* f, int max_rows, int H) {
    f->on = false;
    if (!ctx->tp_comm || ctx->tp_size < 2) return B200_OK;
    NcclApi* api = nccl_api();
    const int t = ctx->tp_size, rank = ctx->tp_rank;
    // the same answer on every rank: the environment is the launcher's, the shape is the model's
    bool want = t <= kTpMaxRanks && H % 256 == 0 && H <= 8192 && !getenv("B200_TP_NO_FUSED");
    tp_fused_layout(f, t, rank, max_rows, H);
    const char* wait_ms = getenv("B200_TP_WAIT_MS");
    f->wait_ns = (long long)(wait_ms && atoi(wait_ms) > 0 ? atoi(wait_ms) : 5000) * 1000000ll;
    if (!want) return B200_OK;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int ok = 1;
    cudaIpcMemHandle_t mine{};
    if (cudaMalloc((void**)&f->base, f->bytes) != cudaSuccess) { cudaGetLastError(); f->base = nullptr; ok = 0; }
    // flags at zero and the flagless form's buffers armed, on the stream the handle exchange below runs on: no peer has
    // this block's handle before these fills are done
    if (ok && (cudaMemsetAsync(f->base, 0, f->bytes, ctx->stream) != cudaSuccess || tp_fused_arm(ctx, f) != B200_OK ||
               cudaIpcGetMemHandle(&mine, f->base) != cudaSuccess)) { cudaGetLastError(); ok = 0; }
    // trade the handles (a rank that failed sends zeros and says so in the agreement below)
    uint8_t* d_all = nullptr;
    float* d_ok = nullptr;
    CUDA_TRY(ctx, cudaMalloc((void**)&d_all, (size_t)(t + 1) * sizeof mine));
    CUDA_TRY(ctx, cudaMalloc((void**)&d_ok, 4));
    CUDA_TRY(ctx, cudaMemcpyAsync(d_all + (size_t)t * sizeof mine, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream));
    NCCL_TRY(ctx, api, api->all_gather(d_all + (size_t)t * sizeof mine, d_all, sizeof mine, kNcclUint8, ctx->tp_comm, ctx->stream));
    std::vector<cudaIpcMemHandle_t> all(t);
    CUDA_TRY(ctx, cudaMemcpyAsync(all.data(), d_all, (size_t)t * sizeof mine, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    for (int k = 0; k < t && ok; k++) {
        if (k == rank) { f->peer[k] = f->base; continue; }
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[k], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = 0; break; }
        f->peer[k] = reinterpret_cast<uint8_t*>(p);
    }
    // the agreement: the sum of the ranks' "I can" is t or it is not
    const float okf = ok ? 1.f : 0.f;
    CUDA_TRY(ctx, cudaMemcpyAsync(d_ok, &okf, 4, cudaMemcpyHostToDevice, ctx->stream));
    NCCL_TRY(ctx, api, api->all_reduce(d_ok, d_ok, 1, kNcclFloat32, kNcclSum, ctx->tp_comm, ctx->stream));
    float sum = 0.f;
    CUDA_TRY(ctx, cudaMemcpyAsync(&sum, d_ok, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(d_all);
    cudaFree(d_ok);
    if ((int)(sum + 0.5f) == t) {
        f->on = true;
        f->use_ll = !getenv("B200_TP_FLAGS");   // measurement: the form with flags and fences for every call
        return B200_OK;
    }
    tp_fused_teardown(ctx, f);
    return B200_OK;
}

// Unmaps the peers' blocks, waits (on the communicator, when it is still there) until every rank has, and frees this one's.
void tp_fused_teardown(b200_ctx* ctx, TpFused* f) {
    if (!f->base && !f->on) return;
    cudaStreamSynchronize(ctx->stream);
    for (int k = 0; k < f->t; k++)
        if (k != f->rank && f->peer[k]) cudaIpcCloseMemHandle(f->peer[k]);
    bool peers_done = true;
    if (f->t > 1 && ctx->tp_comm) {  // every rank comes here (the ranks agreed on the outcome of the setup)
        NcclApi* api = nccl_api();
        float* d = nullptr;
        if (cudaMalloc((void**)&d, 4) == cudaSuccess) {
            cudaMemsetAsync(d, 0, 4, ctx->stream);
            api->all_reduce(d, d, 1, kNcclFloat32, kNcclSum, ctx->tp_comm, ctx->stream);
            // a rank that is gone never joins: the wait is bounded, and a block whose peers may still have it mapped is
            // left to the process's exit rather than freed under them
            const auto t0 = std::chrono::steady_clock::now();
            cudaError_t q;
            while ((q = cudaStreamQuery(ctx->stream)) == cudaErrorNotReady) {
                if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(10)) { peers_done = false; break; }
                std::this_thread::sleep_for(std::chrono::milliseconds(1));
            }
            if (q != cudaSuccess && q != cudaErrorNotReady) cudaGetLastError();
            if (peers_done) cudaFree(d);
        }
    }
    if (!peers_done) {
        *f = TpFused{};
        return;
    }
    if (f->base) cudaFree(f->base);
    *f = TpFused{};
}

// buf[n] <- sum over ranks, in place, on the context's stream
int tp_all_reduce_sum(b200_ctx* ctx, float* buf, size_t n) {
    if (!ctx->tp_comm) B200_FAIL(ctx, B200_BAD_ARGUMENT, "no tensor-parallel communicator on this context");
    NcclApi* api = nccl_api();
    ProfScope ps(ctx, PROF_OTHER);
    NCCL_TRY(ctx, api, api->all_reduce(buf, buf, n, kNcclFloat32, kNcclSum, ctx->tp_comm, ctx->stream));
    ctx->launches++;
    return B200_OK;
}

// local [rows][w] of every rank -> full [rows][t*w] on every rank (rank k's slice at columns k*w ..); gathered is
// scratch of t*rows*w floats
int tp_all_gather_columns(b200_ctx* ctx, const float* local, int rows, int w, float* gathered, float* full) {
    if (!ctx->tp_comm) B200_FAIL(ctx, B200_BAD_ARGUMENT, "no tensor-parallel communicator on this context");
    NcclApi* api = nccl_api();
    const size_t n = (size_t)rows * w;
    NCCL_TRY(ctx, api, api->all_gather(local, gathered, n, kNcclFloat32, ctx->tp_comm, ctx->stream));
    ctx->launches++;
    const size_t tot = n * ctx->tp_size;
    interleave_slices_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, ctx->stream>>>(gathered, ctx->tp_size, rows, w, full);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

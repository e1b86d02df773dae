// tp_fused.cu — tensor parallel on the GPUs of one host: the all-reduce of the o / down partial products, the residual
// add, the RMSNorm that follows and the per-32 quantizer as ONE kernel over peer memory.
//
// NCCL's form of the same work is an f32 all-reduce of [rows][hidden] (every rank ends with every row) followed by a
// norm + quantize kernel that every rank runs on every row. Here a rank owns rows/t of the rows. The kernel has two
// stages. Push: every rank stores each of its partial rows into a staging area of the row's owner (plain 16-byte stores
// to the owner's block, mapped into this process; stores are posted, so they pipeline where loads from a peer would wait
// 1.7 us each and are held to about 9 GB/s per SM by the loads an SM can keep in flight), then raises the row's flag on the
// owner. Reduce: the owner waits for a row's flags, adds the staged rows and its own in rank order, adds its residual row,
// norms, quantizes and stores the int8 codes and the scales into every rank's activation buffer: 4 bytes per value travel
// in and 1.25 out, against 8 for the all-reduce, and the norm is computed once. The residual stream stays sharded by rows
// between layers; the last layer's call hands the updated rows to every rank instead (mode 1), for the final norm and the
// vocabulary-split head.
//
// Synchronisation. Row flags (pushed -> owner) and CTA flags (a rank's CTA j has stored its codes -> CTA j of every rank)
// carry the launch's sequence number and only grow, so nothing is ever reset. The grid is the same on every rank and no
// larger than the SM count, so all CTAs run at once and the push stage, which waits for nothing, always completes. A
// kernel ends only when every rank's CTAs have stored, so a peer's pushes for the next call cannot land in a staging
// area that is still being read, nor its codes in a buffer the consumers of this call still read (the next call's pushes
// and stores come after that call's kernels have started, which on this rank is after those consumers). Every wait is
// bounded by wall time; a rank that gives up raises the context's error flag, stores nothing more and returns, and its
// peers then give up the same way.
//
// The arithmetic is the row kernels' (elementwise.cu): f64 sum of squares, y = (x*inv)*w, the quantizer of rowquant.cuh.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "rowquant.cuh"

namespace {

constexpr int kTpMaxCtas = 128;  // the grid's cap: one CTA per SM at most, so the CTAs that wait for one another all run

struct TpPeers {
    uint8_t* p[kTpMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// waits until *flag has reached seq (bounded by wall time)
__device__ __forceinline__ bool wait_flag(const unsigned* flag, unsigned seq, long long wait_ns) {
    if ((int)(ld_acquire_sys(flag) - seq) >= 0) return true;
    const long long t0 = global_ns();
    while ((int)(ld_acquire_sys(flag) - seq) < 0) {
        if (global_ns() - t0 > wait_ns) return false;
        __nanosleep(64);
    }
    return true;
}

struct TpOffsets {
    size_t part, stage, h, codes, scales, row_flags, cta_flags;
};

// One thread per 8 consecutive values of a row (H/8 threads, at most 1024).
// phases: 1 = push only, 2 = reduce only, 3 = both (the one-GPU emulation runs every rank's push before any reduce).
__global__ void __launch_bounds__(1024) tp_reduce_norm_quant_kernel(TpPeers peers, TpOffsets off, int rank, int t, unsigned seq, int T, int H,
                                                                    const float* __restrict__ w, float eps, int mode, int phases,
                                                                    int use_flags, long long wait_ns, int* __restrict__ err_flag,
                                                                    long long* __restrict__ stage_ns) {
    __shared__ double red[32];
    const int rows_per = (T + t - 1) / t, nG = H >> 5, c = threadIdx.x, nW = blockDim.x >> 5;
    const int q4 = threadIdx.x & 3, g = c >> 2;
    const bool stamp = stage_ns && blockIdx.x == 0 && threadIdx.x == 0;  // measurement: CTA 0's clock at each stage
    if (stamp) stage_ns[0] = global_ns();
    if (*reinterpret_cast<volatile int*>(err_flag)) return;  // a wait already gave up in this step: the later launches do not wait again
    uint8_t* const me = peers.p[rank];
    // ---- push: this rank's partial rows go to their owners' staging areas ([source rank][owner's row][H]) ----
    if (phases & 1) {
        for (int r = blockIdx.x; r < T; r += gridDim.x) {
            const int o = r / rows_per, b = r - o * rows_per;
            if (o == rank) continue;
            const float* src = reinterpret_cast<const float*>(me + off.part) + (size_t)r * H + 8 * c;
            float* dst = reinterpret_cast<float*>(peers.p[o] + off.stage) + ((size_t)rank * rows_per + b) * H + 8 * c;
            const float4 a0 = *reinterpret_cast<const float4*>(src), a1 = *reinterpret_cast<const float4*>(src + 4);
            *reinterpret_cast<float4*>(dst) = a0;
            *reinterpret_cast<float4*>(dst + 4) = a1;
            __syncthreads();
            if (threadIdx.x == 0 && use_flags) {
                __threadfence_system();  // the CTA's stores (ordered before this thread by the barrier) ahead of the flag
                st_release_sys(reinterpret_cast<unsigned*>(peers.p[o] + off.row_flags) + (size_t)b * kTpMaxRanks + rank, seq);
            }
        }
    }
    if (stamp) stage_ns[1] = global_ns();
    bool ok = true;
    if (phases & 2) {
        float wv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (mode == 0) {
            const float4 a = *reinterpret_cast<const float4*>(w + 8 * c), bb = *reinterpret_cast<const float4*>(w + 8 * c + 4);
            wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = bb.x; wv[5] = bb.y; wv[6] = bb.z; wv[7] = bb.w;
        }
        // ---- reduce: this rank's rows, dealt over the grid ----
        for (int b = blockIdx.x; b < rows_per && ok; b += gridDim.x) {
            const int r = rank * rows_per + b;
            if (r >= T) break;
            float* hr = reinterpret_cast<float*>(me + off.h) + (size_t)r * H + 8 * c;
            const float4 h0 = *reinterpret_cast<const float4*>(hr), h1 = *reinterpret_cast<const float4*>(hr + 4);
            if (use_flags) {
                bool mine_ok = true;
                if (threadIdx.x < t && threadIdx.x != rank)
                    mine_ok = wait_flag(reinterpret_cast<const unsigned*>(me + off.row_flags) + (size_t)b * kTpMaxRanks + threadIdx.x, seq, wait_ns);
                ok = __syncthreads_and(mine_ok) != 0;
                if (!ok) break;
            }
            // the ranks' partial rows, added in rank order starting from rank 0's, then the residual row
            float4 a0[kTpMaxRanks], a1[kTpMaxRanks];
#pragma unroll
            for (int k = 0; k < kTpMaxRanks; k++) {
                if (k < t) {
                    const float* src = k == rank ? reinterpret_cast<const float*>(me + off.part) + (size_t)r * H + 8 * c
                                                 : reinterpret_cast<const float*>(me + off.stage) + ((size_t)k * rows_per + b) * H + 8 * c;
                    a0[k] = __ldcg(reinterpret_cast<const float4*>(src));
                    a1[k] = __ldcg(reinterpret_cast<const float4*>(src + 4));
                }
            }
            float d[8] = {a0[0].x, a0[0].y, a0[0].z, a0[0].w, a1[0].x, a1[0].y, a1[0].z, a1[0].w};
#pragma unroll
            for (int k = 1; k < kTpMaxRanks; k++) {
                if (k < t) {
                    d[0] = __fadd_rn(d[0], a0[k].x); d[1] = __fadd_rn(d[1], a0[k].y); d[2] = __fadd_rn(d[2], a0[k].z); d[3] = __fadd_rn(d[3], a0[k].w);
                    d[4] = __fadd_rn(d[4], a1[k].x); d[5] = __fadd_rn(d[5], a1[k].y); d[6] = __fadd_rn(d[6], a1[k].z); d[7] = __fadd_rn(d[7], a1[k].w);
                }
            }
            const float x[8] = {__fadd_rn(h0.x, d[0]), __fadd_rn(h0.y, d[1]), __fadd_rn(h0.z, d[2]), __fadd_rn(h0.w, d[3]),
                                __fadd_rn(h1.x, d[4]), __fadd_rn(h1.y, d[5]), __fadd_rn(h1.z, d[6]), __fadd_rn(h1.w, d[7])};
            const float4 o0 = make_float4(x[0], x[1], x[2], x[3]), o1 = make_float4(x[4], x[5], x[6], x[7]);
            if (mode == 1) {
                for (int k = 0; k < t; k++) {
                    float* dst = reinterpret_cast<float*>(peers.p[k] + off.h) + (size_t)r * H + 8 * c;
                    *reinterpret_cast<float4*>(dst) = o0;
                    *reinterpret_cast<float4*>(dst + 4) = o1;
                }
                continue;
            }
            *reinterpret_cast<float4*>(hr) = o0;
            *reinterpret_cast<float4*>(hr + 4) = o1;
            double ss = 0;
#pragma unroll
            for (int u = 0; u < 8; u++) ss += (double)x[u] * (double)x[u];
            ss = warp_sum_f64(ss);
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
            __syncthreads();
            double tot = 0;
            for (int k = 0; k < nW; k++) tot += red[k];
            __syncthreads();  // red is reused by the CTA's next row
            const float inv = (float)(1.0 / sqrt(tot / (double)H + (double)eps));
            float y[8];
#pragma unroll
            for (int u = 0; u < 8; u++) y[u] = __fmul_rn(__fmul_rn(x[u], inv), wv[u]);
            unsigned cw[2];
            float sc, asum;
            quant_group_quad_regs(y, cw, sc, asum);
            for (int k = 0; k < t; k++) {
                *reinterpret_cast<uint2*>(reinterpret_cast<int8_t*>(peers.p[k] + off.codes) + (size_t)r * H + 8 * c) = make_uint2(cw[0], cw[1]);
                if (q4 == 0) {
                    float* sk = reinterpret_cast<float*>(peers.p[k] + off.scales) + (size_t)r * 2 * nG;
                    sk[g] = sc;
                    sk[nG + g] = asum;
                }
            }
        }
    }
    if (stamp) stage_ns[2] = global_ns();
    // ---- every rank's CTA j tells CTA j of every rank that its stores are done, and waits for theirs ----
    if (use_flags && (phases & 2)) {
        __syncthreads();
        bool mine_ok = true;
        if (threadIdx.x == 0) __threadfence_system();
        __syncthreads();
        if (stamp) stage_ns[3] = global_ns();
        if (threadIdx.x < t && ok) {
            const size_t slot = (size_t)blockIdx.x * kTpMaxRanks;
            st_release_sys(reinterpret_cast<unsigned*>(peers.p[threadIdx.x] + off.cta_flags) + slot + rank, seq);
            mine_ok = wait_flag(reinterpret_cast<const unsigned*>(me + off.cta_flags) + slot + threadIdx.x, seq, wait_ns);
        }
        ok = __syncthreads_and(mine_ok && ok) != 0;
    }
    if (!ok && threadIdx.x == 0) atomicExch(err_flag, 1);
    if (stamp) stage_ns[4] = global_ns();
}


// ---- the flagless form ----
constexpr unsigned kNoF32 = 0xFFFFFFFFu;   // a NaN pattern no sender stores (a value with these bits is sent as the default NaN)
constexpr unsigned kNoCodes = 0x80808080u; // four codes of -128: the quantizer clamps to +-127
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_volatile_v2(void* p, unsigned a, unsigned b) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_volatile_u32(void* p, unsigned a) { asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(a) : "memory"); }
__device__ __forceinline__ unsigned sendable(unsigned bits) { return bits == kNoF32 ? 0x7FC00000u : bits; }
__device__ __forceinline__ bool arrived(uint4 v, unsigned none) { return v.x != none && v.y != none && v.z != none && v.w != none; }
// polls 16 bytes until none of its words holds `none` (bounded by wall time)
__device__ __forceinline__ bool poll_v4(const void* p, unsigned none, long long wait_ns, uint4* out) {
    uint4 v = ld_volatile_v4(p);
    if (!arrived(v, none)) {
        const long long t0 = global_ns();
        int spins = 0;
        do {
            v = ld_volatile_v4(p);
            if ((++spins & 63) == 0 && global_ns() - t0 > wait_ns) { *out = v; return false; }
        } while (!arrived(v, none));
    }
    *out = v;
    return true;
}

// eight values of this rank's partial product at element i: the matmul's output, or, when it left its K-split partials for
// this kernel, their sum in split order starting from the first
__device__ __forceinline__ void own_partial8(const float* __restrict__ part, const float* __restrict__ kparts, int n_kparts, size_t kpart_stride,
                                             size_t i, float (&v)[8]) {
    const float* src = n_kparts ? kparts + i : part + i;
    float4 a = __ldcg(reinterpret_cast<const float4*>(src)), b = __ldcg(reinterpret_cast<const float4*>(src + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    for (int k = 1; k < n_kparts; k++) {
        a = __ldcg(reinterpret_cast<const float4*>(src + (size_t)k * kpart_stride));
        b = __ldcg(reinterpret_cast<const float4*>(src + (size_t)k * kpart_stride + 4));
        v[0] = __fadd_rn(v[0], a.x); v[1] = __fadd_rn(v[1], a.y); v[2] = __fadd_rn(v[2], a.z); v[3] = __fadd_rn(v[3], a.w);
        v[4] = __fadd_rn(v[4], b.x); v[5] = __fadd_rn(v[5], b.y); v[6] = __fadd_rn(v[6], b.z); v[7] = __fadd_rn(v[7], b.w);
    }
}

struct TpLLOffsets {
    size_t part, h, stage, codes, scales, next_codes, next_scales;  // of this call's buffers and of the next call's
};

__global__ void __launch_bounds__(1024) tp_ll_reduce_norm_quant_kernel(TpPeers peers, TpLLOffsets off, int rank, int t, int T, int H,
                                                                       const float* __restrict__ w, float eps, int phases, long long wait_ns,
                                                                       int* __restrict__ err_flag, long long* __restrict__ stage_ns,
                                                                       const float* __restrict__ kparts, int n_kparts, size_t kpart_stride,
                                                                       __half* __restrict__ x16) {
    __shared__ double red[32];
    const int rows_per = (T + t - 1) / t, nG = H >> 5, c = threadIdx.x, nW = blockDim.x >> 5;
    const int q4 = threadIdx.x & 3, g = c >> 2;
    const bool stamp = stage_ns && blockIdx.x == 0 && threadIdx.x == 0;
    pdl_trigger();
    // the norm weight is written by no kernel: fetched while the kernel ahead on the stream drains
    const float4 wa = *reinterpret_cast<const float4*>(w + 8 * c), wb = *reinterpret_cast<const float4*>(w + 8 * c + 4);
    pdl_wait();
    if (stamp) stage_ns[0] = global_ns();
    if (*reinterpret_cast<volatile int*>(err_flag)) return;  // a wait already gave up in this step: the later launches do not wait again
    uint8_t* const me = peers.p[rank];
    bool ok = true;
    // ---- push: this rank's partial rows into their owners' staging ([source rank][owner's row][H]) ----
    if (phases & 1) {
        // the rows are walked from the next rank's on (rank s starts with the rows of rank s + 1), so that at any moment the
        // ranks send to different owners instead of all to the owners of the first rows
        for (int r0 = blockIdx.x; r0 < t * rows_per; r0 += gridDim.x) {
            int r = r0 + (rank + 1) * rows_per;
            if (r >= t * rows_per) r -= t * rows_per;
            if (r >= T) continue;
            const int o = r / rows_per, b = r - o * rows_per;
            if (o == rank) continue;
            float* dst = reinterpret_cast<float*>(peers.p[o] + off.stage) + ((size_t)rank * rows_per + b) * H + 8 * c;
            float pv[8];
            own_partial8(reinterpret_cast<const float*>(me + off.part), kparts, n_kparts, kpart_stride, (size_t)r * H + 8 * c, pv);
            uint4 a0 = make_uint4(__float_as_uint(pv[0]), __float_as_uint(pv[1]), __float_as_uint(pv[2]), __float_as_uint(pv[3]));
            uint4 a1 = make_uint4(__float_as_uint(pv[4]), __float_as_uint(pv[5]), __float_as_uint(pv[6]), __float_as_uint(pv[7]));
            a0.x = sendable(a0.x); a0.y = sendable(a0.y); a0.z = sendable(a0.z); a0.w = sendable(a0.w);
            a1.x = sendable(a1.x); a1.y = sendable(a1.y); a1.z = sendable(a1.z); a1.w = sendable(a1.w);
            st_volatile_v4(dst, a0);
            st_volatile_v4(dst + 4, a1);
        }
    }
    if (stamp) stage_ns[1] = global_ns();
    // ---- reduce: this rank's rows, dealt over the grid ----
    if (phases & 2) {
        const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
        for (int b = blockIdx.x; b < rows_per; b += gridDim.x) {
            const int r = rank * rows_per + b;
            if (r >= T) break;
            float* hr = reinterpret_cast<float*>(me + off.h) + (size_t)r * H + 8 * c;
            const float4 h0 = *reinterpret_cast<const float4*>(hr), h1 = *reinterpret_cast<const float4*>(hr + 4);
            float pv[8];
            own_partial8(reinterpret_cast<const float*>(me + off.part), kparts, n_kparts, kpart_stride, (size_t)r * H + 8 * c, pv);
            // the ranks' partial rows, added in rank order starting from rank 0's; a staged word is put back once it has been read
            float d[8];
#pragma unroll
            for (int k = 0; k < kTpMaxRanks; k++) {
                if (k < t) {
                    float v[8];
                    if (k == rank) {
#pragma unroll
                        for (int u = 0; u < 8; u++) v[u] = pv[u];
                    } else {
                        float* st = reinterpret_cast<float*>(me + off.stage) + ((size_t)k * rows_per + b) * H + 8 * c;
                        uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                        ok = ok && poll_v4(st, kNoF32, wait_ns, &a0);   // (a thread that gave up once does not wait again)
                        ok = ok && poll_v4(st + 4, kNoF32, wait_ns, &a1);
                        const uint4 none = make_uint4(kNoF32, kNoF32, kNoF32, kNoF32);
                        st_volatile_v4(st, none);
                        st_volatile_v4(st + 4, none);
                        v[0] = __uint_as_float(a0.x); v[1] = __uint_as_float(a0.y); v[2] = __uint_as_float(a0.z); v[3] = __uint_as_float(a0.w);
                        v[4] = __uint_as_float(a1.x); v[5] = __uint_as_float(a1.y); v[6] = __uint_as_float(a1.z); v[7] = __uint_as_float(a1.w);
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) d[u] = k == 0 ? v[u] : __fadd_rn(d[u], v[u]);
                }
            }
            const float x[8] = {__fadd_rn(h0.x, d[0]), __fadd_rn(h0.y, d[1]), __fadd_rn(h0.z, d[2]), __fadd_rn(h0.w, d[3]),
                                __fadd_rn(h1.x, d[4]), __fadd_rn(h1.y, d[5]), __fadd_rn(h1.z, d[6]), __fadd_rn(h1.w, d[7])};
            *reinterpret_cast<float4*>(hr) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(hr + 4) = make_float4(x[4], x[5], x[6], x[7]);
            double ss = 0;
#pragma unroll
            for (int u = 0; u < 8; u++) ss += (double)x[u] * (double)x[u];
            ss = warp_sum_f64(ss);
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
            __syncthreads();
            double tot = 0;
            for (int k = 0; k < nW; k++) tot += red[k];
            __syncthreads();  // red is reused by the CTA's next row
            const float inv = (float)(1.0 / sqrt(tot / (double)H + (double)eps));
            float y[8];
#pragma unroll
            for (int u = 0; u < 8; u++) y[u] = __fmul_rn(__fmul_rn(x[u], inv), wv[u]);
            unsigned cw[2];
            float sc, asum;
            quant_group_quad_regs(y, cw, sc, asum);
            const unsigned scb = sendable(__float_as_uint(sc)), asb = sendable(__float_as_uint(asum));
            for (int k = 0; k < t; k++) {
                st_volatile_v2(reinterpret_cast<int8_t*>(peers.p[k] + off.codes) + (size_t)r * H + 8 * c, cw[0], cw[1]);
                if (q4 == 0) {
                    float* sk = reinterpret_cast<float*>(peers.p[k] + off.scales) + (size_t)r * 2 * nG;
                    st_volatile_u32(sk + g, scb);
                    st_volatile_u32(sk + nG + g, asb);
                }
            }
        }
    }
    if (stamp) stage_ns[2] = global_ns();
    if (phases & 4) {
        // ---- rearm the other pair of activation buffers for the next call (rows [0, T)) ----
        const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
        const size_t n_codes16 = (size_t)T * H / 16, n_scales16 = (size_t)T * 2 * nG * 4 / 16;
        for (size_t i = tid; i < n_codes16; i += nthr)
            reinterpret_cast<uint4*>(me + off.next_codes)[i] = make_uint4(kNoCodes, kNoCodes, kNoCodes, kNoCodes);
        for (size_t i = tid; i < n_scales16; i += nthr) reinterpret_cast<uint4*>(me + off.next_scales)[i] = make_uint4(kNoF32, kNoF32, kNoF32, kNoF32);
        if (stamp) stage_ns[3] = global_ns();
        // ---- wait until every row's codes and scales, from every owner, are here; with x16 set, the thread that saw 16
        // codes arrive also lays them out as the fp16 tiles (code * scale) the matmul after this kernel reads, so no
        // conversion kernel runs between the two ----
        uint4 v;
        for (size_t i = tid; i < n_codes16 && ok; i += nthr) {
            ok = poll_v4(me + off.codes + i * 16, kNoCodes, wait_ns, &v);
            if (x16 && ok) {
                const int r = (int)(i / (size_t)(H >> 4)), k16 = (int)(i % (size_t)(H >> 4)) << 4;
                const unsigned* scp = reinterpret_cast<const unsigned*>(me + off.scales) + (size_t)r * 2 * nG + (k16 >> 5);
                unsigned sb = *reinterpret_cast<const volatile unsigned*>(scp);
                if (sb == kNoF32) {   // the group's scale has not landed yet (bounded like every wait)
                    const long long t0 = global_ns();
                    while ((sb = *reinterpret_cast<const volatile unsigned*>(scp)) == kNoF32) {
                        if (global_ns() - t0 > wait_ns) { ok = false; break; }
                    }
                }
                if (ok) {
                    const float sc = __uint_as_float(sb);
                    const unsigned cw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        float f[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) f[u] = __fmul_rn((float)(int)(signed char)((cw[2 * hh + (u >> 2)] >> (8 * (u & 3))) & 0xffu), sc);
                        x16_store8(x16, H, r, k16 + 8 * hh, f);
                    }
                }
            }
        }
        for (size_t i = tid; i < n_scales16 && ok; i += nthr) ok = poll_v4(me + off.scales + i * 16, kNoF32, wait_ns, &v);
    }
    if (!ok) atomicExch(err_flag, 1);
    if (stamp) stage_ns[4] = global_ns();
}

}  // namespace

void tp_fused_layout(TpFused* f, int t, int rank, int max_rows, int H) {
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    f->t = t; f->rank = rank; f->max_rows = max_rows; f->H = H;
    f->off_part = 0;
    f->off_stage = up(f->off_part + (size_t)max_rows * H * 4);
    f->off_h = up(f->off_stage + (size_t)(max_rows + kTpMaxRanks) * H * 4);   // t * ceil(T/t) rows at most
    f->off_codes = up(f->off_h + (size_t)max_rows * H * 4);
    f->off_scales = up(f->off_codes + (size_t)max_rows * H);
    f->off_row_flags = up(f->off_scales + (size_t)max_rows * 2 * (H / 32) * 4);
    f->off_cta_flags = up(f->off_row_flags + (size_t)max_rows * kTpMaxRanks * 4);
    size_t at = up(f->off_cta_flags + (size_t)kTpMaxCtas * kTpMaxRanks * 4);
    for (int p = 0; p < 2; p++) {
        f->off_stage_ll[p] = at; at = up(at + (size_t)(max_rows + kTpMaxRanks) * H * 4);
        f->off_codes_ll[p] = at; at = up(at + (size_t)max_rows * H);
        f->off_scales_ll[p] = at; at = up(at + (size_t)max_rows * 2 * (H / 32) * 4);
    }
    f->bytes = at;
}

// Fills the flagless form's buffers with the not-arrived values (the block was just allocated, or a wait gave up).
int tp_fused_arm(b200_ctx* ctx, TpFused* f) {
    for (int p = 0; p < 2; p++) {
        CUDA_TRY(ctx, cudaMemsetAsync(f->base + f->off_stage_ll[p], 0xFF, (size_t)(f->max_rows + kTpMaxRanks) * f->H * 4, ctx->stream));
        CUDA_TRY(ctx, cudaMemsetAsync(f->base + f->off_codes_ll[p], 0x80, (size_t)f->max_rows * f->H, ctx->stream));
        CUDA_TRY(ctx, cudaMemsetAsync(f->base + f->off_scales_ll[p], 0xFF, (size_t)f->max_rows * 2 * (f->H / 32) * 4, ctx->stream));
        f->armed[p] = f->max_rows;
    }
    return B200_OK;
}

int launch_tp_reduce_norm_quant_ll(b200_ctx* ctx, TpFused* f, int T, const float* norm_w, float eps, ActQ* out, int phases, const Parts* given,
                                   __half* x16) {
    if (!f->base || T < 1 || T > f->max_rows || f->H % 256 || f->H > 8192 || f->t < 1 || f->t > kTpMaxRanks || !norm_w)
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor-parallel reduce: %d rows of %d (at most %d), %d ranks", T, f->H, f->max_rows, f->t);
    if (!ctx->err_flag) B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor-parallel reduce: the context has no error flag");
    const int p = (int)(f->ll_calls & 1u);
    if ((phases & 1) && f->armed[p] < T) {
        // the step's row count grew: this call's activation buffers are rearmed here. No peer can store into them before it
        // has this rank's partial rows, which are pushed after these fills in stream order.
        CUDA_TRY(ctx, cudaMemsetAsync(f->base + f->off_codes_ll[p], 0x80, (size_t)T * f->H, ctx->stream));
        CUDA_TRY(ctx, cudaMemsetAsync(f->base + f->off_scales_ll[p], 0xFF, (size_t)T * 2 * (f->H / 32) * 4, ctx->stream));
    }
    TpPeers peers;
    for (int k = 0; k < kTpMaxRanks; k++) peers.p[k] = f->peer[k < f->t ? k : 0];
    const TpLLOffsets off{f->off_part, f->off_h, f->off_stage_ll[p], f->off_codes_ll[p], f->off_scales_ll[p], f->off_codes_ll[1 - p], f->off_scales_ll[1 - p]};
    const int grid = std::min(std::min(kTpMaxCtas, ctx->sm_count), T);
    Parts pt{};
    if (given) {
        pt = *given;
    } else if (ctx->pending.n > 0 && ctx->pending.dst == f->part() && ctx->pending.rows == T && ctx->pending.cols == f->H && !(ctx->pending.stride & 3)) {
        pt = ctx->pending;  // the matmul left its K-split partials for this kernel to add
        ctx->pending = Parts{};
    } else {
        ST_TRY(flush_pending_parts(ctx));
    }
    {
        ProfScope ps(ctx, PROF_OTHER);  // counted with the collectives it replaces
        launch_pdl(tp_ll_reduce_norm_quant_kernel, dim3(grid), dim3(f->H / 8), 0, ctx->stream, peers, off, f->rank, f->t, T, f->H, norm_w, eps, phases,
                   f->wait_ns, ctx->err_flag, f->phase_ns, pt.p, pt.n, pt.stride, x16);
    }
    LAUNCH_CHECK(ctx);
    if (phases & 4) {
        f->armed[p] = 0;
        f->armed[1 - p] = T;
        f->ll_calls++;
    }
    if (out) *out = f->aq_ll(p);
    return B200_OK;
}

int launch_tp_reduce_norm_quant(b200_ctx* ctx, TpFused* f, int T, const float* norm_w, float eps, int mode, int phases, bool use_flags) {
    if (!f->base || T < 1 || T > f->max_rows || f->H % 256 || f->H > 8192 || f->t < 1 || f->t > kTpMaxRanks || (mode == 0 && !norm_w))
        B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor-parallel reduce: %d rows of %d (at most %d), %d ranks", T, f->H, f->max_rows, f->t);
    if (!ctx->err_flag) B200_FAIL(ctx, B200_BAD_ARGUMENT, "tensor-parallel reduce: the context has no error flag");
    TpPeers peers;
    for (int k = 0; k < kTpMaxRanks; k++) peers.p[k] = f->peer[k < f->t ? k : 0];
    const TpOffsets off{f->off_part, f->off_stage, f->off_h, f->off_codes, f->off_scales, f->off_row_flags, f->off_cta_flags};
    ST_TRY(flush_pending_parts(ctx));  // this form reads the finished product
    if (phases & 1) ++f->seq;
    const int grid = std::min(std::min(kTpMaxCtas, ctx->sm_count), T);
    ProfScope ps(ctx, PROF_OTHER);  // counted with the collectives it replaces
    tp_reduce_norm_quant_kernel<<<grid, f->H / 8, 0, ctx->stream>>>(peers, off, f->rank, f->t, f->seq, T, f->H, norm_w, eps, mode, phases,
                                                                   use_flags ? 1 : 0, f->wait_ns, ctx->err_flag, f->phase_ns);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

extern "C" int b200_debug_tp_reduce_emulated(b200_ctx* ctx, int t, int T, int H, const float* parts, const float* h, const float* w,
                                             float eps, int mode, int n_kparts, int8_t* codes_out, float* scales_out, float* h_out) {
    if (t < 1 || t > kTpMaxRanks || T < 1 || H < 256 || H % 256 || H > 8192) B200_FAIL(ctx, B200_BAD_ARGUMENT, "bad emulated shape");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (n_kparts < 0 || n_kparts > 8 || (n_kparts > 0 && mode != 2)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K-split partials go with mode 2");
    struct Blocks {
        TpFused f[kTpMaxRanks];
        float* kp[kTpMaxRanks] = {};
        __half* x16[kTpMaxRanks] = {};
        float* dw = nullptr;
        int* flag = nullptr;
        ~Blocks() {
            for (auto& x : f) cudaFree(x.base);
            for (auto* x : kp) cudaFree(x);
            for (auto* x : x16) cudaFree(x);
            cudaFree(dw);
            cudaFree(flag);
        }
    } bl;
    for (int k = 0; k < t; k++) {
        tp_fused_layout(&bl.f[k], t, k, T, H);
        CUDA_TRY(ctx, cudaMalloc((void**)&bl.f[k].base, bl.f[k].bytes));
        CUDA_TRY(ctx, cudaMemsetAsync(bl.f[k].base, 0, bl.f[k].bytes, ctx->stream));
        if (n_kparts > 0) {  // rank k's product as n_kparts partial matrices, T*H floats apart
            CUDA_TRY(ctx, cudaMalloc((void**)&bl.kp[k], (size_t)n_kparts * T * H * 4));
            CUDA_TRY(ctx, cudaMemcpyAsync(bl.kp[k], parts + (size_t)k * n_kparts * T * H, (size_t)n_kparts * T * H * 4, cudaMemcpyHostToDevice, ctx->stream));
        } else {
            CUDA_TRY(ctx, cudaMemcpyAsync(bl.f[k].part(), parts + (size_t)k * T * H, (size_t)T * H * 4, cudaMemcpyHostToDevice, ctx->stream));
        }
        CUDA_TRY(ctx, cudaMemcpyAsync(bl.f[k].h(), h, (size_t)T * H * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    for (int k = 0; k < t; k++)
        for (int j = 0; j < t; j++) bl.f[k].peer[j] = bl.f[j].base;
    CUDA_TRY(ctx, cudaMalloc((void**)&bl.dw, (size_t)H * 4));
    CUDA_TRY(ctx, cudaMalloc((void**)&bl.flag, 4));
    CUDA_TRY(ctx, cudaMemsetAsync(bl.flag, 0, 4, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(bl.dw, w, (size_t)H * 4, cudaMemcpyHostToDevice, ctx->stream));
    int* const saved = ctx->err_flag;
    ctx->err_flag = bl.flag;
    int st = B200_OK;
    ActQ got[kTpMaxRanks];
    if (mode == 2) {
        // the flagless form, three calls in a row on the same inputs (each of the two buffer pairs is used, rearmed and used
        // again); a word that never arrives makes a wait run out, which the flag reports
        for (int k = 0; k < t && st == B200_OK; k++) {
            bl.f[k].wait_ns = 50ll * 1000000ll;
            st = tp_fused_arm(ctx, &bl.f[k]);
        }
        const size_t x_bytes = (size_t)ceil_div(T, 256) * 256 * H * 2;
        for (int k = 0; k < t; k++) {
            CUDA_TRY(ctx, cudaMalloc((void**)&bl.x16[k], 2 * x_bytes));   // what the kernel lays out | what the conversion kernel makes of the codes
            CUDA_TRY(ctx, cudaMemsetAsync(bl.x16[k], 0, 2 * x_bytes, ctx->stream));
        }
        for (int round = 0; round < 3 && st == B200_OK; round++) {
            for (int k = 0; k < t; k++) CUDA_TRY(ctx, cudaMemcpyAsync(bl.f[k].h(), h, (size_t)T * H * 4, cudaMemcpyHostToDevice, ctx->stream));
            for (int ph = 1; ph <= 4; ph *= 2)  // every rank's push, then every rank's reduce, then every rank's rearm + wait
                for (int k = 0; k < t && st == B200_OK; k++) {
                    const Parts given{bl.kp[k], (size_t)T * H, n_kparts, bl.f[k].part(), T, H};
                    st = launch_tp_reduce_norm_quant_ll(ctx, &bl.f[k], T, bl.dw, eps, &got[k], ph, &given, bl.x16[k]);
                }
        }
        // the fp16 tiles every rank laid out as the codes arrived are the conversion kernel's, bit for bit
        std::vector<uint8_t> ha(x_bytes), hb(x_bytes);
        for (int k = 0; k < t && st == B200_OK; k++) {
            st = launch_act_to_f16(ctx, got[k], T, H, bl.x16[k] + x_bytes / 2);
            if (st != B200_OK) break;
            CUDA_TRY(ctx, cudaMemcpyAsync(ha.data(), bl.x16[k], x_bytes, cudaMemcpyDeviceToHost, ctx->stream));
            CUDA_TRY(ctx, cudaMemcpyAsync(hb.data(), bl.x16[k] + x_bytes / 2, x_bytes, cudaMemcpyDeviceToHost, ctx->stream));
            CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            if (memcmp(ha.data(), hb.data(), x_bytes)) {
                ctx->err_flag = saved;
                B200_FAIL(ctx, B200_CUDA_ERROR, "rank %d: the fp16 tiles laid out by the cross-rank kernel differ from the conversion kernel's", k);
            }
        }
    } else {
        for (int ph = 1; ph <= 2; ph++)  // every rank's push, then every rank's reduce
            for (int k = 0; k < t && st == B200_OK; k++) st = launch_tp_reduce_norm_quant(ctx, &bl.f[k], T, bl.dw, eps, mode, ph, false);
        for (int k = 0; k < t; k++) got[k] = ActQ{bl.f[k].codes(), bl.f[k].scales()};
    }
    ctx->err_flag = saved;
    if (st != B200_OK) return st;
    int gave_up = 0;
    CUDA_TRY(ctx, cudaMemcpyAsync(&gave_up, bl.flag, 4, cudaMemcpyDeviceToHost, ctx->stream));
    for (int k = 0; k < t; k++) {
        if (mode != 1) {
            CUDA_TRY(ctx, cudaMemcpyAsync(codes_out + (size_t)k * T * H, got[k].codes, (size_t)T * H, cudaMemcpyDeviceToHost, ctx->stream));
            CUDA_TRY(ctx, cudaMemcpyAsync(scales_out + (size_t)k * T * 2 * (H / 32), got[k].scales, (size_t)T * 2 * (H / 32) * 4, cudaMemcpyDeviceToHost, ctx->stream));
        }
        CUDA_TRY(ctx, cudaMemcpyAsync(h_out + (size_t)k * T * H, bl.f[k].h(), (size_t)T * H * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (gave_up) B200_FAIL(ctx, B200_TIMEOUT, "a wait of the emulated ranks ran out");
    return B200_OK;
}

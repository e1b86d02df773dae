// sample.cu — device-side draws, logit masks and the routed-expert bookkeeping.
//
//   mask      constrain/constrain.go:233-267 maskID: a rejected token's logit becomes -inf before the draw
//   greedy    internal/runtime/sampling/sampler.go:485-518 Argmax: first maximal index
//   min-p     sampler.go:586-647 (candidates logit >= max + T*ln(minP)), :654-724 finishFilter (order by
//             (prob desc, id asc), cut p < minP*p0, drop zeros, renormalise), :442-458 drawFiltered (first
//             prefix whose cumulative probability exceeds the caller's uniform u)
//   route     decoder/mlp.go:130-184 routeExperts (softmax path), :370-411 softmaxF32, :415-440 topK
#include <algorithm>

#include "common.cuh"

namespace {

__global__ void mask_logits_kernel(float* __restrict__ logits, int V, const int32_t* __restrict__ row_mask,
                                   const uint32_t* __restrict__ masks) {
    const int r = blockIdx.y;
    const int mi = row_mask[r];
    if (mi < 0) return;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= V) return;
    const int words = (V + 31) / 32;
    if (!((masks[(size_t)mi * words + (t >> 5)] >> (t & 31)) & 1u)) logits[(size_t)r * V + t] = -INFINITY;
}

constexpr int kDrawThreads = 1024;

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0;
    for (int w = 0; w < kDrawThreads / 32; w++) t += red[w];
    return t;
}

__device__ __forceinline__ long long block_sum_i64(long long v, long long* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    long long t = 0;
    for (int w = 0; w < kDrawThreads / 32; w++) t += red[w];
    return t;
}

// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11; the host's statement is
// internal/runtime/sampling/philox.go:21-36). Integer only, so every backend draws the same words. One round: the two
// 32 x 32 -> 64 bit products M0 * c0 and M1 * c2; the new counter is (hi(M1 c2) ^ c1 ^ k0, lo(M1 c2), hi(M0 c0) ^ c3 ^ k1,
// lo(M0 c0)). Round r runs under the key k + r * W (the Weyl sequence: the key is bumped between rounds, not before the first).
struct PhiloxState {
    unsigned c[4];
};
__device__ __forceinline__ PhiloxState philox_round(PhiloxState s, unsigned key0, unsigned key1) {
    const unsigned long long prod_a = (unsigned long long)0xD2511F53u * s.c[0];
    const unsigned long long prod_b = (unsigned long long)0xCD9E8D57u * s.c[2];
    PhiloxState n;
    n.c[0] = (unsigned)(prod_b >> 32) ^ s.c[1] ^ key0;
    n.c[1] = (unsigned)prod_b;
    n.c[2] = (unsigned)(prod_a >> 32) ^ s.c[3] ^ key1;
    n.c[3] = (unsigned)prod_a;
    return n;
}
__device__ __forceinline__ void philox4x32(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0, unsigned k1, unsigned* out) {
    PhiloxState s{{c0, c1, c2, c3}};
#pragma unroll
    for (unsigned r = 0; r < 10u; r++) s = philox_round(s, k0 + r * 0x9E3779B9u, k1 + r * 0xBB67AE85u);
#pragma unroll
    for (int i = 0; i < 4; i++) out[i] = s.c[i];
}

// 32 random bits -> a standard Gumbel variate G = -ln(-ln(w)), w = (h + 0.5) / 2^32 in (0, 1), in f32 without cancellation.
// The f32 operations and their order are the host sampler's (internal/runtime/sampling/sampler_gumbel.go:37-64; device twin
// backend/cuda/gumbel.cu:50-60), because a draw must pick the same token on every backend: E = -ln(1 - w) is taken from log1p
// on the lower half of the range, and on the upper half from 1 - w = (~h + 0.5) / 2^32, which is exact.
__device__ __forceinline__ float gumbel_noise(unsigned h) {
    const bool lower = (h >> 31) == 0u;
    const float unit = __fmul_rn(__fadd_rn((float)(lower ? h : ~h), 0.5f), 2.3283064365386963e-10f);   // w below, 1 - w above
    const float e = lower ? -log1pf(-unit) : -logf(unit);
    return -logf(e);
}

// ---- top-K rows (decoder/resident/subsystems.go:40-48, forward.go:91-96; device twin backend/cuda/topk.cu) ----
// The K highest logits of a row ordered (logit descending, token id ascending), and Z = sum exp((l - max) * invT) over
// the whole row. -0 and +0 tie, as on the host. One block per row: an exact 3-pass radix select (11 + 11 + 10 bits of an
// order-preserving key) finds the K-th largest key; every entry above it and the first `need` entries equal to it by
// ascending id are gathered and a bitonic sort orders the K survivors.
constexpr int kTopKThreads = 1024, kTopKMax = 1024;

__device__ __forceinline__ unsigned topk_key(float x) {
    if (x == 0.0f) x = 0.0f;  // -0 -> +0
    const unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kTopKThreads) topk_kernel(const float* __restrict__ logits, int V, int K, float invT, int want_z,
                                                            int32_t* __restrict__ ids, float* __restrict__ vals, double* __restrict__ z) {
    __shared__ unsigned hist[2048];
    __shared__ unsigned long long cand[kTopKMax];  // (key << 32) | ~id : sorts by key desc, id asc when sorted descending
    __shared__ unsigned s_prefix, s_need, s_cnt_gt, s_cnt_eq;
    __shared__ double s_red[kTopKThreads / 32];
    __shared__ float s_maxv;
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)r * V;
    // radix select: after the passes, s_prefix is the K-th largest key and s_need how many entries equal to it are kept
    unsigned prefix = 0, need = (unsigned)K;
    const int shifts[3] = {21, 10, 0}, bits[3] = {11, 11, 10};
    unsigned mask_hi = 0;  // the bits already fixed
    for (int pass = 0; pass < 3; pass++) {
        const int nb = 1 << bits[pass];
        for (int i = tid; i < nb; i += kTopKThreads) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < V; i += kTopKThreads) {
            const unsigned k = topk_key(l[i]);
            if ((k & mask_hi) == prefix) atomicAdd(&hist[(k >> shifts[pass]) & (nb - 1)], 1u);
        }
        __syncthreads();
        if (tid == 0) {  // walk the bins from the top: the bin where the running count reaches `need`
            unsigned run = 0;
            int b = nb - 1;
            for (; b > 0; b--) {
                if (run + hist[b] >= need) break;
                run += hist[b];
            }
            s_prefix = prefix | ((unsigned)b << shifts[pass]);
            s_need = need - run;
        }
        __syncthreads();
        prefix = s_prefix;
        need = s_need;
        mask_hi |= (unsigned)(nb - 1) << shifts[pass];
        __syncthreads();
    }
    // gather: every key above the K-th, in any order; then the `need` lowest ids among the equal ones
    if (tid == 0) { s_cnt_gt = 0; s_cnt_eq = 0; }
    __syncthreads();
    const unsigned n_gt = (unsigned)K - need;
    for (int i = tid; i < V; i += kTopKThreads) {
        const unsigned k = topk_key(l[i]);
        if (k > prefix) cand[atomicAdd(&s_cnt_gt, 1u)] = ((unsigned long long)k << 32) | (unsigned)(~i);
    }
    __syncthreads();
    // equal keys by ascending id: a block-wide ordered scan in chunks of the block size
    for (int base = 0; base < V && s_cnt_eq < need; base += kTopKThreads) {
        const int i = base + tid;
        const bool eq = i < V && topk_key(l[i]) == prefix;
        // rank among this chunk's equal entries (ids ascend with tid)
        const unsigned bal = __ballot_sync(0xffffffffu, eq);
        const int lane = tid & 31, warp = tid >> 5;
        if (lane == 0) hist[warp] = __popc(bal);
        __syncthreads();
        unsigned before = 0;
        for (int w = 0; w < warp; w++) before += hist[w];
        const unsigned rank = s_cnt_eq + before + __popc(bal & ((1u << lane) - 1));
        unsigned chunk_total = 0;
        for (int w = 0; w < kTopKThreads / 32; w++) chunk_total += hist[w];
        if (eq && rank < need) cand[n_gt + rank] = ((unsigned long long)prefix << 32) | (unsigned)(~i);
        __syncthreads();
        if (tid == 0) s_cnt_eq += chunk_total;
        __syncthreads();
    }
    // pad to a power of two and bitonic sort descending
    int n2 = 1;
    while (n2 < K) n2 <<= 1;
    for (int i = K + tid; i < n2; i += kTopKThreads) cand[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < n2; i += kTopKThreads) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const unsigned long long a = cand[i], b = cand[j];
                    if (desc ? a < b : a > b) { cand[i] = b; cand[j] = a; }
                }
            }
            __syncthreads();
        }
    for (int i = tid; i < K; i += kTopKThreads) {
        const int id = (int)(~(unsigned)(cand[i] & 0xffffffffull));
        ids[(size_t)r * K + i] = id;
        vals[(size_t)r * K + i] = l[id];
    }
    if (want_z) {
        if (tid == 0) s_maxv = l[(int)(~(unsigned)(cand[0] & 0xffffffffull))];
        __syncthreads();
        const double mx = (double)s_maxv, it = (double)invT;
        double acc = 0;
        for (int i = tid; i < V; i += kTopKThreads) acc += exp(((double)l[i] - mx) * it);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if ((tid & 31) == 0) s_red[tid >> 5] = acc;
        __syncthreads();
        if (tid == 0) {
            double t = 0;
            for (int w = 0; w < kTopKThreads / 32; w++) t += s_red[w];
            z[r] = t;
        }
    }
}

__global__ void philox_kernel(const uint32_t* __restrict__ ctr, const uint32_t* __restrict__ key, int n, uint32_t* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned r[4];
    philox4x32(ctr[4 * i], ctr[4 * i + 1], ctr[4 * i + 2], ctr[4 * i + 3], key[2 * i], key[2 * i + 1], r);
    for (int k = 0; k < 4; k++) out[4 * i + k] = r[k];
}

// One block per row.
__global__ void __launch_bounds__(kDrawThreads) draw_kernel(const float* __restrict__ logits, int V,
                                                            const b200_draw* __restrict__ draws, int32_t* __restrict__ ids) {
    __shared__ float s_val[kDrawThreads / 32];
    __shared__ int s_idx[kDrawThreads / 32];
    __shared__ double s_red[kDrawThreads / 32];
    __shared__ float s_max;
    __shared__ int s_arg;
    const int r = blockIdx.x;
    const float* l = logits + (size_t)r * V;
    const b200_draw dr = draws[r];
    if (dr.kind == B200_DRAW_LOGITS) {
        if (threadIdx.x == 0) ids[r] = -1;
        return;
    }
    // first maximum
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += kDrawThreads) {
        float v = l[i];
        if (v > best || bi == 0x7fffffff) {
            if (v > best || bi == 0x7fffffff) { best = v; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = s_val[0];
        int k = s_idx[0];
        for (int w = 1; w < kDrawThreads / 32; w++)
            if (s_val[w] > b || (s_val[w] == b && s_idx[w] < k)) { b = s_val[w]; k = s_idx[w]; }
        s_max = b;
        s_arg = k;
    }
    __syncthreads();
    if (dr.kind == B200_DRAW_GREEDY) {
        if (threadIdx.x == 0) ids[r] = s_arg;
        return;
    }
    if (dr.kind == B200_DRAW_GUMBEL) {
        // argmax_i(l_i * invT + G_i): a thread walks groups of four tokens (one Philox call each) in ascending order with a
        // strict >, and ties between threads go to the lower index: the lowest index among the maxima, as on the host
        // (sampler_gumbel.go:52-64). The seed and the draw index ride in the struct's bytes 8..23.
        const unsigned* raw = reinterpret_cast<const unsigned*>(&draws[r]);
        const unsigned k0 = raw[2], k1 = raw[3], d0 = raw[4], d1 = raw[5];
        const float invT = dr.temperature;
        float gb = -INFINITY;
        int gi = -1;
        for (int b = threadIdx.x; b * 4 < V; b += kDrawThreads) {
            unsigned h[4];
            philox4x32((unsigned)b, d0, d1, 0u, k0, k1, h);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int i = b * 4 + q;
                if (i < V) {
                    const float k = __fadd_rn(__fmul_rn(l[i], invT), gumbel_noise(h[q]));
                    if (k > gb) { gb = k; gi = i; }
                }
            }
        }
        auto better = [](float ak, int ai, float bk, int bi2) { return ai >= 0 && (bi2 < 0 || ak > bk || (ak == bk && ai < bi2)); };
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ok_ = __shfl_xor_sync(0xffffffffu, gb, o);
            const int oi = __shfl_xor_sync(0xffffffffu, gi, o);
            if (better(ok_, oi, gb, gi)) { gb = ok_; gi = oi; }
        }
        __syncthreads();  // s_val / s_idx were read by thread 0 above
        if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = gb; s_idx[threadIdx.x >> 5] = gi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float b = s_val[0];
            int k = s_idx[0];
            for (int w = 1; w < kDrawThreads / 32; w++)
                if (better(s_val[w], s_idx[w], b, k)) { b = s_val[w]; k = s_idx[w]; }
            ids[r] = k >= 0 ? k : s_arg;  // nothing comparable (an all -inf row): the plain argmax
        }
        return;
    }
    // min-p
    const double texp = dr.temperature > 0.f ? (double)dr.temperature : 1.0;
    const double minp = dr.min_p > 1.f ? 1.0 : (double)dr.min_p;
    const double maxL = (double)s_max;
    const double thr = minp > 0 ? maxL + texp * log(minp) : -INFINITY;
    // e of a retained token, else 0: candidate by logit, not cut by minP*p0 (p0 = e of the top token = 1), nonzero
    auto e_of = [&](int i) -> double {
        const double li = (double)l[i];
        if (!(li >= thr)) return 0.0;
        const double e = exp((li - maxL) / texp);
        if (minp > 0 && e < minp * 1.0) return 0.0;
        return e;
    };
    double part = 0;
    for (int i = threadIdx.x; i < V; i += kDrawThreads) part += e_of(i);
    const double total = block_sum_f64(part, s_red);
    if (!(total > 0)) {
        if (threadIdx.x == 0) ids[r] = s_arg;
        return;
    }
    const double target = dr.u * total;
    // largest key X (bit pattern of a positive double) with mass{e >= X} > target
    long long lo = 1, hi = __double_as_longlong(1.0) + 1;
    while (hi - lo > 1) {
        const long long mid = lo + (hi - lo) / 2;
        const double x = __longlong_as_double(mid);
        double p2 = 0;
        for (int i = threadIdx.x; i < V; i += kDrawThreads) {
            const double e = e_of(i);
            if (e >= x) p2 += e;
        }
        const double g = block_sum_f64(p2, s_red);
        if (g > target) lo = mid; else hi = mid;
    }
    const double X = __longlong_as_double(lo);
    // mass strictly above X, and the ties at X
    double pa = 0;
    long long ties = 0;
    for (int i = threadIdx.x; i < V; i += kDrawThreads) {
        const double e = e_of(i);
        if (e > X) pa += e;
        if (e == X) ties++;
    }
    const double above = block_sum_f64(pa, s_red);
    const long long n_ties = block_sum_i64(ties, (long long*)s_red);
    if (n_ties == 0) {  // u at or past the retained mass: the reference returns the last retained token
        if (threadIdx.x == 0) ids[r] = s_arg;
        return;
    }
    // ties share one e: after t of them the running mass is above + t*X; take the first t that exceeds target
    long long t = (long long)floor((target - above) / X) + 1;
    if (t < 1) t = 1;
    if (t > n_ties) t = n_ties;
    // t-th smallest id among the ties: bisection on the id
    int ilo = -1, ihi = V - 1;  // count(id <= ilo) < t <= count(id <= ihi)
    while (ihi - ilo > 1) {
        const int mid = ilo + (ihi - ilo) / 2;
        long long c = 0;
        for (int i = threadIdx.x; i <= mid; i += kDrawThreads)
            if (e_of(i) == X) c++;
        const long long cnt = block_sum_i64(c, (long long*)s_red);
        if (cnt >= t) ihi = mid; else ilo = mid;
    }
    if (threadIdx.x == 0) ids[r] = ihi;
}

// One warp per row. n_experts <= 512.
__global__ void __launch_bounds__(32) route_kernel(const float* __restrict__ logits, int nE, int k, int norm,
                                                   int32_t* __restrict__ idx, float* __restrict__ wts) {
    __shared__ float p[512];
    __shared__ double e64[512];
    const int r = blockIdx.x, lane = threadIdx.x;
    const float* lg = logits + (size_t)r * nE;
    float mx = -INFINITY;
    for (int i = lane; i < nE; i += 32) mx = fmaxf(mx, lg[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int i = lane; i < nE; i += 32) {
        const double e = exp((double)__fsub_rn(lg[i], mx));
        e64[i] = e;
        p[i] = (float)e;
    }
    __syncwarp();
    double sum = 0;
    if (lane == 0)
        for (int i = 0; i < nE; i++) sum += e64[i];  // index order, as the reference sums
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inv = (float)(1.0 / sum);
    for (int i = lane; i < nE; i += 32) p[i] = __fmul_rn(p[i], inv);
    __syncwarp();
    float wsum = 0.f;
    for (int j = 0; j < k; j++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < nE; i += 32) {
            const float v = p[i];
            if (v > best) { best = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) {  // fewer than k finite scores
            if (lane == 0) { idx[(size_t)r * k + j] = -1; wts[(size_t)r * k + j] = 0.f; }
            continue;
        }
        if (lane == 0) {
            idx[(size_t)r * k + j] = bi;
            wts[(size_t)r * k + j] = best;
            p[bi] = -INFINITY;  // used
        }
        wsum = __fadd_rn(wsum, best);
        __syncwarp();
    }
    if (norm && wsum > 0.f && lane == 0)
        for (int j = 0; j < k; j++)
            if (idx[(size_t)r * k + j] >= 0) wts[(size_t)r * k + j] = __fdiv_rn(wts[(size_t)r * k + j], wsum);
}

// One block of 1024 threads: a counting sort that keeps an expert's rows in the order of their assignments. The experts'
// totals come from shared-memory atomics (a count does not depend on the order), their offsets from a warp scan; then the
// assignments are walked 1024 at a time, a thread each: lanes that name the same expert find one another with match_any (a
// lane's place among them is its rank in the warp), the warps' counts per expert are scanned over the 32 warps by a thread
// per expert, and slot = the expert's running offset + the warps before + the rank. offs[nE+1]; rows_tok[s] = token row of
// sorted slot s; slot_of[a] = sorted slot of assignment a = row*k + rank (-1 when the rank is empty).
// Dynamic shared memory: 33 * nE ints.
__global__ void __launch_bounds__(1024) group_experts_kernel(const int32_t* __restrict__ idx, int n_assign, int k, int nE, int32_t* __restrict__ offs,
                                                             int32_t* __restrict__ rows_tok, int32_t* __restrict__ slot_of) {
    extern __shared__ int s_base[];    // nE running offsets, then [32 warps][nE] counts
    int* wcnt = s_base + nE;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < nE; e += 1024) s_base[e] = 0;
    __syncthreads();
    for (int a = tid; a < n_assign; a += 1024) {
        const int e = idx[a];
        if (e >= 0) atomicAdd(&s_base[e], 1);
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int e0 = 0; e0 < nE; e0 += 32) {
            const int c = e0 + lane < nE ? s_base[e0 + lane] : 0;
            int v = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += u;
            }
            if (e0 + lane < nE) {
                offs[e0 + lane] = carry + v - c;
                s_base[e0 + lane] = carry + v - c;
            }
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) offs[nE] = carry;
    }
    __syncthreads();
    for (int a0 = 0; a0 < n_assign; a0 += 1024) {
        const int a = a0 + tid, e = a < n_assign ? idx[a] : -1;
        for (int i = tid; i < 32 * nE; i += 1024) wcnt[i] = 0;
        __syncthreads();
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && rank == 0) wcnt[warp * nE + e] = __popc(peers);
        __syncthreads();
        for (int ee = tid; ee < nE; ee += 1024) {   // the warps' counts become the warps' first slots; the expert's offset moves on
            int run = s_base[ee];
            for (int w = 0; w < 32; w++) {
                const int c = wcnt[w * nE + ee];
                wcnt[w * nE + ee] = run;
                run += c;
            }
            s_base[ee] = run;
        }
        __syncthreads();
        if (e >= 0) {
            const int slot = wcnt[warp * nE + e] + rank;
            rows_tok[slot] = a / k;
            slot_of[a] = slot;
        } else if (a < n_assign) {
            slot_of[a] = -1;
        }
        __syncthreads();
    }
}

}  // namespace

int launch_mask_logits(b200_ctx* ctx, float* logits, int R, int V, const int32_t* row_mask, const uint32_t* masks) {
    mask_logits_kernel<<<dim3(ceil_div(V, 256), R), 256, 0, ctx->stream>>>(logits, V, row_mask, masks);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_draw(b200_ctx* ctx, const float* logits, int R, int V, const b200_draw* draws, int32_t* ids, float*) {
    draw_kernel<<<R, kDrawThreads, 0, ctx->stream>>>(logits, V, draws, ids);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_topk(b200_ctx* ctx, const float* logits, int R, int V, int k, float invT, bool want_z, int32_t* ids, float* vals, double* z) {
    if (k < 1 || k > kTopKMax || k > V) B200_FAIL(ctx, B200_BAD_ARGUMENT, "top-K takes 1 <= k <= min(%d, vocab)", kTopKMax);
    topk_kernel<<<R, kTopKThreads, 0, ctx->stream>>>(logits, V, k, invT, want_z ? 1 : 0, ids, vals, z);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_philox(b200_ctx* ctx, const uint32_t* ctr, const uint32_t* key, int n, uint32_t* out) {
    philox_kernel<<<ceil_div(n, 128), 128, 0, ctx->stream>>>(ctr, key, n, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_route(b200_ctx* ctx, const float* logits, int T, int nE, int k, int norm, int32_t* idx, float* wts) {
    if (nE > 512) B200_FAIL(ctx, B200_DECLINED, "router: more than 512 experts");
    route_kernel<<<T, 32, 0, ctx->stream>>>(logits, nE, k, norm, idx, wts);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_group_experts(b200_ctx* ctx, const int32_t* idx, int T, int k, int nE, int32_t* offs, int32_t* rows) {
    // rows holds rows_tok[T*k] followed by slot_of[T*k]
    if (nE > 512) B200_FAIL(ctx, B200_DECLINED, "expert grouping: more than 512 experts");
    const size_t smem = (size_t)33 * nE * sizeof(int);
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device))
        CUDA_TRY(ctx, cudaFuncSetAttribute(group_experts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 33 * 512 * (int)sizeof(int)));
    group_experts_kernel<<<1, 1024, smem, ctx->stream>>>(idx, T * k, k, nE, offs, rows, rows + (size_t)T * k);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

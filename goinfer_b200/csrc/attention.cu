// attention.cu — paged attention for decode rows and the causal rows of a prefill chunk.
//
// Every packed row r is one query at position row_pos[r] of KV slot row_slot[r]; it attends keys
// [0, row_pos[r]] of that slot through the block table (the rows of a chunk were stored before this runs).
// Semantics follow decoder/forwardn.go:295-501: score = (q.k)*scale, optional cap*tanh(s/cap)
// (decoder/attention.go:287-295), softmax over the causal range, context = sum w*v. The reference folds
// in f64; here the dot, the online softmax and the AV sum run in fp32 over fp16 K/V.
//
// attn_split_kernel: flash-decode. One CTA per (key split, kv head, row): the G query heads of the group
// share every K and V load; each lane owns HD/32 dims of every key, scores are reduced across the warp by a
// transposing butterfly, softmax is online, and the 4 warps' states are merged in shared memory. Partials
// (acc[HD], max, sum) go to scratch and attn_combine_kernel merges the splits in split order, normalises and
// (optionally) quantizes the context row per 32 for the O projection.
// attn_generic_kernel: any head_dim up to 64 and any group size, one warp per (row, head); used for tiny test
// models and as the independent implementation the parity tests cross-check the fast kernel with.
#include "common.cuh"

namespace {

constexpr int kSplitKeys = 512;

__device__ __forceinline__ float score_of(float dot, float scale, float cap) {
    float s = dot * scale;
    if (cap != 0.f) s = cap * tanhf(s / cap);
    return s;
}

// v[i] summed over the warp's lanes; lane L receives the total of v[L].
__device__ __forceinline__ float reduce_scatter32(float (&v)[32], int lane) {
#pragma unroll
    for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
        const bool up = lane & off;
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            float a = v[i], b = v[i + n / 2];
            float send = up ? a : b, keep = up ? b : a;
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return v[0];
}

template <int DPL>
__device__ __forceinline__ void load_halves(const __half* p, float (&out)[DPL]) {
    if constexpr (DPL == 4) {
        uint2 u = *reinterpret_cast<const uint2*>(p);
        float2 a = __half22float2(*reinterpret_cast<__half2*>(&u.x)), b = __half22float2(*reinterpret_cast<__half2*>(&u.y));
        out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
    } else if constexpr (DPL == 2) {
        unsigned u = *reinterpret_cast<const unsigned*>(p);
        float2 a = __half22float2(*reinterpret_cast<__half2*>(&u));
        out[0] = a.x; out[1] = a.y;
    } else {
#pragma unroll
        for (int d = 0; d < DPL; d++) out[d] = __half2float(p[d]);
    }
}

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_split_kernel(const float* __restrict__ q, int ldq, int nH, int nKV, float scale,
                                                         float cap, const int32_t* __restrict__ row_slot,
                                                         const int32_t* __restrict__ row_pos, const __half* __restrict__ kpool,
                                                         const __half* __restrict__ vpool, const int32_t* __restrict__ table,
                                                         int max_blocks, int block_rows, float* __restrict__ partial,
                                                         int max_splits) {
    constexpr int DPL = HD / 32, KB = 32 / G;
    const int r = blockIdx.z, kvh = blockIdx.y, split = blockIdx.x;
    const int nkeys = row_pos[r] + 1;
    const int k0 = split * kSplitKeys;
    if (k0 >= nkeys) return;
    const int k1 = min(nkeys, k0 + kSplitKeys);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int32_t* tbl = table + (size_t)row_slot[r] * max_blocks;

    float qr[G][DPL];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int d = 0; d < DPL; d++) qr[g][d] = q[(size_t)r * ldq + (size_t)(kvh * G + g) * HD + lane * DPL + d];
    const int my_kk = lane / G;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[g][d] = 0.f;

    for (int kb = k0 + warp * KB; kb < k1; kb += 4 * KB) {
        size_t off[KB];
        float part[32];
#pragma unroll
        for (int kk = 0; kk < KB; kk++) {
            const int key = min(kb + kk, k1 - 1);
            const int blk = tbl[key / block_rows];
            off[kk] = (((size_t)blk * nKV + kvh) * block_rows + (key % block_rows)) * HD + lane * DPL;
            float kf[DPL];
            load_halves<DPL>(kpool + off[kk], kf);
#pragma unroll
            for (int g = 0; g < G; g++) {
                float s = 0.f;
#pragma unroll
                for (int d = 0; d < DPL; d++) s = fmaf(qr[g][d], kf[d], s);
                part[kk * G + g] = s;
            }
        }
        float s = reduce_scatter32(part, lane);  // this lane: key kb + my_kk, head lane % G
        const bool valid = kb + my_kk < k1;
        s = valid ? score_of(s, scale, cap) : -INFINITY;
        float mx = s;
#pragma unroll
        for (int o = G; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run, mx);  // finite: the batch holds at least one valid key
        const float alpha = __expf(m_run - m_new);
        const float p = valid ? __expf(s - m_new) : 0.f;
        float ps = p;
#pragma unroll
        for (int o = G; o < 32; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l_run = l_run * alpha + ps;
        m_run = m_new;
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float a = __shfl_sync(0xffffffffu, alpha, g);
#pragma unroll
            for (int d = 0; d < DPL; d++) acc[g][d] *= a;
        }
#pragma unroll
        for (int kk = 0; kk < KB; kk++) {
            float vf[DPL];
            load_halves<DPL>(vpool + off[kk], vf);
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float pg = __shfl_sync(0xffffffffu, p, kk * G + g);
#pragma unroll
                for (int d = 0; d < DPL; d++) acc[g][d] = fmaf(pg, vf[d], acc[g][d]);
            }
        }
    }

    __shared__ float sm_m[4][G], sm_l[4][G];
    __shared__ float sm_acc[4][G][HD];
    if (lane < G) {
        sm_m[warp][lane] = m_run;
        sm_l[warp][lane] = l_run;
    }
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int d = 0; d < DPL; d++) sm_acc[warp][g][lane * DPL + d] = acc[g][d];
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += 128) {
        const int g = idx / HD, e = idx % HD;
        float M = sm_m[0][g];  // warp 0 always saw a key
#pragma unroll
        for (int w = 1; w < 4; w++) M = fmaxf(M, sm_m[w][g]);
        float tot = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = __expf(sm_m[w][g] - M);
            tot += sm_acc[w][g][e] * f;
            l += sm_l[w][g] * f;
        }
        float* out = partial + (((size_t)r * nH + kvh * G + g) * max_splits + split) * (HD + 2);
        out[e] = tot;
        if (e == 0) {
            out[HD] = M;
            out[HD + 1] = l;
        }
    }
}

// grid (nH, T), HD threads. Merges a row's splits in split order; optional per-32 quantization.
template <int HD>
__global__ void attn_combine_kernel(const float* __restrict__ partial, int nH, int max_splits,
                                    const int32_t* __restrict__ row_pos, float* __restrict__ out, int8_t* __restrict__ codes,
                                    float* __restrict__ scales) {
    const int h = blockIdx.x, r = blockIdx.y, e = threadIdx.x;
    const int nsp = (row_pos[r] + 1 + kSplitKeys - 1) / kSplitKeys;
    const float* p = partial + ((size_t)r * nH + h) * max_splits * (HD + 2);
    float M = -INFINITY;
    for (int s = 0; s < nsp; s++) M = fmaxf(M, p[(size_t)s * (HD + 2) + HD]);
    float tot = 0.f, l = 0.f;
    for (int s = 0; s < nsp; s++) {
        const float f = __expf(p[(size_t)s * (HD + 2) + HD] - M);
        tot += p[(size_t)s * (HD + 2) + e] * f;
        l += p[(size_t)s * (HD + 2) + HD + 1] * f;
    }
    const float y = tot / l;
    const int D = nH * HD;
    out[(size_t)r * D + h * HD + e] = y;
    if (codes) {
        const int lane = e & 31, g = (h * HD + e) >> 5, nG = D >> 5;
        float ma = fabsf(y);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
        const float sc = __fdiv_rn(ma, 127.f);
        const float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
        int qv = max(-127, min(127, __float2int_rn(__fmul_rn(y, inv))));
        int sum = qv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        codes[(size_t)r * D + h * HD + e] = (int8_t)qv;
        if (lane == 0) {
            scales[(size_t)r * 2 * nG + g] = sc;
            scales[(size_t)r * 2 * nG + nG + g] = __fmul_rn(sc, (float)sum);
        }
    }
}

// One warp per (row, head); lanes stride the keys. head_dim <= 64.
__global__ void __launch_bounds__(32) attn_generic_kernel(const float* __restrict__ q, int ldq, int nH, int nKV, int hd,
                                                          float scale, float cap, const int32_t* __restrict__ row_slot,
                                                          const int32_t* __restrict__ row_pos, const __half* __restrict__ kpool,
                                                          const __half* __restrict__ vpool, const int32_t* __restrict__ table,
                                                          int max_blocks, int block_rows, float* __restrict__ out) {
    const int h = blockIdx.x, r = blockIdx.y, lane = threadIdx.x;
    const int kvh = h / (nH / nKV);
    const int nkeys = row_pos[r] + 1;
    const int32_t* tbl = table + (size_t)row_slot[r] * max_blocks;
    const float* qh = q + (size_t)r * ldq + (size_t)h * hd;
    float m = -INFINITY, l = 0.f, acc[64];
    for (int e = 0; e < 64; e++) acc[e] = 0.f;
    for (int key = lane; key < nkeys; key += 32) {
        const int blk = tbl[key / block_rows];
        const size_t off = (((size_t)blk * nKV + kvh) * block_rows + (key % block_rows)) * hd;
        float dot = 0.f;
        for (int e = 0; e < hd; e++) dot = fmaf(qh[e], __half2float(kpool[off + e]), dot);
        const float s = score_of(dot, scale, cap);
        const float mn = fmaxf(m, s);
        const float a = __expf(m - mn), p = __expf(s - mn);
        l = l * a + p;
        for (int e = 0; e < hd; e++) acc[e] = acc[e] * a + p * __half2float(vpool[off + e]);
        m = mn;
    }
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float f = (m == -INFINITY) ? 0.f : __expf(m - M);
    float L = l * f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    for (int e = 0; e < hd; e++) {
        float v = acc[e] * f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) out[(size_t)r * nH * hd + (size_t)h * hd + e] = v / L;
    }
}

// ---- exact class: f64 dot, softmax and AV fold, the CPU path's own arithmetic (decoder/forwardn.go:379-499) ----
// scores[(r*nH + h)*ld + key] = f32(sum_d q_d*k_d in f64, d ascending)
__global__ void __launch_bounds__(128) attn_exact_scores_kernel(const float* __restrict__ q, int ldq, int nH, int nKV, int hd,
                                                                double scale, double cap, const int32_t* __restrict__ row_slot,
                                                                const int32_t* __restrict__ row_pos,
                                                                const __half* __restrict__ kpool, const int32_t* __restrict__ table,
                                                                int max_blocks, int block_rows, float* __restrict__ scores, int ld) {
    const int h = blockIdx.y, r = blockIdx.z;
    const int key = blockIdx.x * 128 + threadIdx.x;
    if (key > row_pos[r]) return;
    const int kvh = h / (nH / nKV);
    const int blk = table[(size_t)row_slot[r] * max_blocks + key / block_rows];
    const __half* kr = kpool + (((size_t)blk * nKV + kvh) * block_rows + key % block_rows) * hd;
    const float* qh = q + (size_t)r * ldq + (size_t)h * hd;
    double d = 0;
    for (int i = 0; i < hd; i++) d = __dadd_rn(d, __dmul_rn((double)qh[i], (double)__half2float(kr[i])));
    (void)scale; (void)cap;
    scores[((size_t)r * nH + h) * ld + key] = (float)d;  // the f32-rounded dot; scale and cap are applied in f64 below
}

// per (head, row): x = cap(f64(dot)*scale); max over the unrounded x; e = exp(f64(f32 x) - max) stored as f32; f64 sum of
// the unrounded e; w = f32(f64(f32 e) / sum) -- the rounding points of decoder/forwardn.go:437-470
__device__ __forceinline__ double exact_score(float dot, double scale, double cap) {
    double x = __dmul_rn((double)dot, scale);
    if (cap != 0.0) x = cap * tanh(x / cap);
    return x;
}
__global__ void __launch_bounds__(256) attn_exact_softmax_kernel(const int32_t* __restrict__ row_pos, int nH, double scale,
                                                                 double cap, float* __restrict__ scores, int ld) {
    __shared__ double red[8];
    const int h = blockIdx.x, r = blockIdx.y, nkeys = row_pos[r] + 1;
    float* s = scores + ((size_t)r * nH + h) * ld;
    double mx = -INFINITY;
    for (int t = threadIdx.x; t < nkeys; t += 256) mx = fmax(mx, exact_score(s[t], scale, cap));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; w++) mx = fmax(mx, red[w]);
    __syncthreads();
    double sum = 0;
    for (int t = threadIdx.x; t < nkeys; t += 256) {
        const double e = exp((double)(float)exact_score(s[t], scale, cap) - mx);
        s[t] = (float)e;
        sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = 0;
    for (int w = 0; w < 8; w++) sum += red[w];
    const double inv = 1.0 / sum;
    for (int t = threadIdx.x; t < nkeys; t += 256) s[t] = (float)((double)s[t] * inv);
}

// per (head, row), one thread per dim: ctx_d = f32( sum over keys ascending of w_t * v_t[d] in f64 )
__global__ void attn_exact_av_kernel(const float* __restrict__ scores, int ld, int nH, int nKV, int hd,
                                     const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                     const __half* __restrict__ vpool, const int32_t* __restrict__ table, int max_blocks,
                                     int block_rows, float* __restrict__ out) {
    const int h = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
    if (d >= hd) return;
    const int kvh = h / (nH / nKV), nkeys = row_pos[r] + 1;
    const float* w = scores + ((size_t)r * nH + h) * ld;
    const int32_t* tbl = table + (size_t)row_slot[r] * max_blocks;
    double acc = 0;
    for (int k0 = 0; k0 < nkeys; k0 += block_rows) {
        const __half* vb = vpool + (((size_t)tbl[k0 / block_rows] * nKV + kvh) * block_rows) * hd + d;
        const int n = min(block_rows, nkeys - k0);
        for (int i = 0; i < n; i++) acc = __dadd_rn(acc, __dmul_rn((double)w[k0 + i], (double)__half2float(vb[(size_t)i * hd])));
    }
    out[(size_t)r * nH * hd + (size_t)h * hd + d] = (float)acc;
}

template <int HD, int G>
int run_split(b200_ctx* ctx, const float* q, int ldq, int T, int nH, int nKV, float scale, float cap, const int32_t* row_slot,
              const int32_t* row_pos, int max_keys, KVView kv, AttnScratch sc, float* out, ActQ aq) {
    const int nsp = ceil_div(max_keys, kSplitKeys);
    if (nsp > sc.max_splits) B200_FAIL(ctx, B200_BAD_ARGUMENT, "attention scratch too small for %d keys", max_keys);
    dim3 grid(nsp, nKV, T);
    {
        ProfScope ps(ctx, PROF_ATTN_SPLIT);
        attn_split_kernel<HD, G><<<grid, 128, 0, ctx->stream>>>(q, ldq, nH, nKV, scale, cap, row_slot, row_pos, kv.k, kv.v,
                                                               kv.table, kv.max_blocks, kv.block_rows, sc.partial, sc.max_splits);
    }
    LAUNCH_CHECK(ctx);
    {
        ProfScope ps(ctx, PROF_ATTN_COMBINE);
        attn_combine_kernel<HD><<<dim3(nH, T), HD, 0, ctx->stream>>>(sc.partial, nH, sc.max_splits, row_pos, out, aq.codes, aq.scales);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

int launch_paged_attention_exact(b200_ctx* ctx, const float* q, int ldq, int T, int nH, int nKV, int hd, double scale,
                                 double softcap, const int32_t* row_slot, const int32_t* row_pos, int max_keys, KVView kv,
                                 float* scores, int ld, float* out, ActQ aq) {
    if (max_keys > ld) B200_FAIL(ctx, B200_BAD_ARGUMENT, "exact attention scratch holds %d keys, %d asked", ld, max_keys);
    attn_exact_scores_kernel<<<dim3(ceil_div(max_keys, 128), nH, T), 128, 0, ctx->stream>>>(
        q, ldq, nH, nKV, hd, scale, softcap, row_slot, row_pos, kv.k, kv.table, kv.max_blocks, kv.block_rows, scores, ld);
    LAUNCH_CHECK(ctx);
    attn_exact_softmax_kernel<<<dim3(nH, T), 256, 0, ctx->stream>>>(row_pos, nH, scale, softcap, scores, ld);
    LAUNCH_CHECK(ctx);
    attn_exact_av_kernel<<<dim3(nH, T), ((hd + 31) / 32) * 32, 0, ctx->stream>>>(scores, ld, nH, nKV, hd, row_slot, row_pos, kv.v,
                                                                                 kv.table, kv.max_blocks, kv.block_rows, out);
    LAUNCH_CHECK(ctx);
    if (aq.codes) return launch_quant_g32(ctx, out, T, nH * hd, aq);
    return B200_OK;
}

int attn_split_keys() { return kSplitKeys; }

size_t attn_scratch_floats(int T, int nH, int hd, int max_splits) { return (size_t)T * nH * max_splits * (hd + 2); }

int launch_paged_attention(b200_ctx* ctx, const float* q, int ldq, int T, int nH, int nKV, int hd, float scale, float softcap,
                           const int32_t* row_slot, const int32_t* row_pos, int max_keys, KVView kv, AttnScratch sc, float* out,
                           ActQ aq) {
    const int G = nH / nKV;
#define SPLIT_CASE(HD_, G_) \
    if (hd == HD_ && G == G_) return run_split<HD_, G_>(ctx, q, ldq, T, nH, nKV, scale, softcap, row_slot, row_pos, max_keys, kv, sc, out, aq)
    SPLIT_CASE(128, 1); SPLIT_CASE(128, 2); SPLIT_CASE(128, 4); SPLIT_CASE(128, 8);
    SPLIT_CASE(64, 1); SPLIT_CASE(64, 2); SPLIT_CASE(64, 4); SPLIT_CASE(64, 8);
#undef SPLIT_CASE
    if (hd > 64) B200_FAIL(ctx, B200_DECLINED, "attention: head_dim %d with group %d is not built", hd, G);
    attn_generic_kernel<<<dim3(nH, T), 32, 0, ctx->stream>>>(q, ldq, nH, nKV, hd, scale, softcap, row_slot, row_pos, kv.k, kv.v,
                                                             kv.table, kv.max_blocks, kv.block_rows, out);
    LAUNCH_CHECK(ctx);
    if (aq.codes) return launch_quant_g32(ctx, out, T, nH * hd, aq);
    return B200_OK;
}

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
#include <cstdlib>

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
    const int nkeys = min(row_pos[r] + 1, max_blocks * block_rows);  // a position past the table reads no block outside it
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


// ---- tensor-core flash-decode (fast class) ----
// One CTA per (key split, kv head, row), 4 warps; each warp walks 16-key tiles of its own (a KV block, or a 16-row slab
// of one, is contiguous per kv head: 16*HD fp16) through a private 3-stage cp.async ring in shared memory, 16-byte
// chunks XOR-swizzled by the key row so ldmatrix reads are conflict-free. Scores S[head][key] = Q K^T run as
// mma.sync m16n8k16 with the group's query heads in the 16-row operand (f32 q split into f16 hi + lo parts, so the
// product keeps fp32-level accuracy over the fp16 keys); the context is accumulated transposed, O^T[dim][head] = V^T P^T,
// so that the score fragment of a lane is already the B fragment of the second product and the 8-column operand holds
// the (up to 8) heads of the group. Online softmax in fp32 registers; P is also split hi + lo. G <= 8.
__device__ __forceinline__ void ldsm_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16f32(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(unsigned smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_dst), "l"(gsrc));
}
// f32 pair -> f16 hi pair and f16 lo pair (x = hi + lo up to 2^-22 relative)
__device__ __forceinline__ void split_hi_lo(float x, float y, unsigned& hi, unsigned& lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const unsigned*>(&h);
    lo = *reinterpret_cast<const unsigned*>(&l);
}

constexpr int kMmaStages = 3;

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_mma_kernel(const float* __restrict__ q, int ldq, int nH, int nKV, float scale, float cap,
                                                       const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                                       const __half* __restrict__ kpool, const __half* __restrict__ vpool,
                                                       const int32_t* __restrict__ table, int max_blocks, int block_rows,
                                                       float* __restrict__ partial, int max_splits, int split_keys) {
    pdl_trigger();
    pdl_wait();
    constexpr int KS = HD / 16, CPR = HD / 8, ROWB = HD * 2, TILE = 16 * ROWB, CPL = 16 * CPR / 32;
    extern __shared__ __align__(128) uint8_t attn_smem[];
    const int r = blockIdx.z, kvh = blockIdx.y, split = blockIdx.x;
    const int nkeys = min(row_pos[r] + 1, max_blocks * block_rows);  // a position past the table reads no block outside it
    const int k0 = split * split_keys;
    if (k0 >= nkeys) return;
    const int k1 = min(nkeys, k0 + split_keys);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
    const int32_t* tbl = table + (size_t)row_slot[r] * max_blocks;
    uint8_t* wsm = attn_smem + (size_t)warp * kMmaStages * 2 * TILE;
    const unsigned wsm_s = (unsigned)__cvta_generic_to_shared(wsm);

    // Q fragments: row gid = head gid of the group (zero rows beyond the group), dims 16ks+2tig(+1) and 16ks+8+2tig(+1)
    unsigned qh0[KS], qh2[KS], ql0[KS], ql2[KS];
    {
        const float* qp = q + (size_t)r * ldq + (size_t)(kvh * G + (gid < G ? gid : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            float2 a = *reinterpret_cast<const float2*>(qp + 16 * ks + 2 * tig);
            float2 b = *reinterpret_cast<const float2*>(qp + 16 * ks + 8 + 2 * tig);
            if (gid >= G) { a.x = a.y = b.x = b.y = 0.f; }
            split_hi_lo(a.x, a.y, qh0[ks], ql0[ks]);
            split_hi_lo(b.x, b.y, qh2[ks], ql2[ks]);
        }
    }
    float o[KS][4];
#pragma unroll
    for (int mt = 0; mt < KS; mt++) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    const int c_first = k0 / 16 + warp, c_end = (k1 + 15) / 16;   // this warp's tiles: c_first, c_first+4, ...
    const int n_tiles = c_first < c_end ? (c_end - c_first + 3) / 4 : 0;
    auto issue = [&](int it) {
        if (it < n_tiles) {
            const int key0 = (c_first + 4 * it) * 16;
            const int blk = tbl[key0 / block_rows];
            const size_t off = (((size_t)blk * nKV + kvh) * block_rows + (key0 % block_rows)) * HD;
            const uint8_t* ksrc = reinterpret_cast<const uint8_t*>(kpool + off);
            const uint8_t* vsrc = reinterpret_cast<const uint8_t*>(vpool + off);
            const unsigned dst = wsm_s + (unsigned)((it % kMmaStages) * 2 * TILE);
#pragma unroll
            for (int i = 0; i < CPL; i++) {
                const int ci = lane + 32 * i, row = ci / CPR, c = ci % CPR;
                const unsigned d = (unsigned)(row * ROWB + ((c ^ (row & 7)) << 4));
                cp16(dst + d, ksrc + ci * 16);
                cp16(dst + TILE + d, vsrc + ci * 16);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
#pragma unroll
    for (int s = 0; s < kMmaStages - 1; s++) issue(s);

    // per-lane ldmatrix geometry (same for K and V tiles)
    const int lrow = (lane & 7) + ((lane >> 4) << 3), lsel = (lane >> 3) & 1;
    for (int it = 0; it < n_tiles; it++) {
        issue(it + kMmaStages - 1);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kMmaStages - 1));
        __syncwarp();
        const unsigned kb = wsm_s + (unsigned)((it % kMmaStages) * 2 * TILE), vb = kb + TILE;
        const int key0 = (c_first + 4 * it) * 16;
        // S0 = keys 0-7 of the tile, S1 = keys 8-15; hi and lo parts accumulate apart to shorten the dependency chains
        float s0h[4] = {0, 0, 0, 0}, s0l[4] = {0, 0, 0, 0}, s1h[4] = {0, 0, 0, 0}, s1l[4] = {0, 0, 0, 0};
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            unsigned b0, b1, b2, b3;
            ldsm_x4(kb + (unsigned)(lrow * ROWB + (((2 * ks + lsel) ^ (lrow & 7)) << 4)), b0, b1, b2, b3);
            mma_f16f32(s0h, qh0[ks], 0u, qh2[ks], 0u, b0, b1);
            mma_f16f32(s1h, qh0[ks], 0u, qh2[ks], 0u, b2, b3);
            mma_f16f32(s0l, ql0[ks], 0u, ql2[ks], 0u, b0, b1);
            mma_f16f32(s1l, ql0[ks], 0u, ql2[ks], 0u, b2, b3);
        }
        float sv[4];
        sv[0] = s0h[0] + s0l[0]; sv[1] = s0h[1] + s0l[1]; sv[2] = s1h[0] + s1l[0]; sv[3] = s1h[1] + s1l[1];
        const int kk[4] = {key0 + 2 * tig, key0 + 2 * tig + 1, key0 + 8 + 2 * tig, key0 + 9 + 2 * tig};
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            sv[i] = kk[i] < k1 ? score_of(sv[i], scale, cap) : -INFINITY;
            mx = fmaxf(mx, sv[i]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float alpha = __expf(m_run - m_new);
        float pv[4], ps = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            pv[i] = __expf(sv[i] - m_new);   // exp(-inf) = 0 for masked keys
            ps += pv[i];
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * alpha + ps;
        m_run = m_new;
        unsigned ph0, pl0, ph1, pl1;
        split_hi_lo(pv[0], pv[1], ph0, pl0);
        split_hi_lo(pv[2], pv[3], ph1, pl1);
        // rescale the context columns of heads 2*tig and 2*tig+1
        const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * tig) * 4), a1 = __shfl_sync(0xffffffffu, alpha, (2 * tig + 1) * 4);
#pragma unroll
        for (int mt = 0; mt < KS; mt++) {
            o[mt][0] *= a0; o[mt][1] *= a1; o[mt][2] *= a0; o[mt][3] *= a1;
            unsigned v0, v1, v2, v3;
            ldsm_x4_t(vb + (unsigned)(lrow * ROWB + (((2 * mt + lsel) ^ (lrow & 7)) << 4)), v0, v1, v2, v3);
            mma_f16f32(o[mt], v0, v1, v2, v3, ph0, ph1);
            mma_f16f32(o[mt], v0, v1, v2, v3, pl0, pl1);
        }
        __syncwarp();
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();
    // merge the 4 warps (reusing the ring): sm_acc[warp][head][dim], sm_m/sm_l[warp][head]
    float* sm_acc = reinterpret_cast<float*>(attn_smem);
    float* sm_m = sm_acc + 4 * G * HD;
    float* sm_l = sm_m + 4 * G;
    if (tig == 0 && gid < G) {
        sm_m[warp * G + gid] = m_run;
        sm_l[warp * G + gid] = l_run;
    }
#pragma unroll
    for (int mt = 0; mt < KS; mt++) {
        const int h0 = 2 * tig, h1 = 2 * tig + 1, d0 = 16 * mt + gid;
        if (h0 < G) { sm_acc[(warp * G + h0) * HD + d0] = o[mt][0]; sm_acc[(warp * G + h0) * HD + d0 + 8] = o[mt][2]; }
        if (h1 < G) { sm_acc[(warp * G + h1) * HD + d0] = o[mt][1]; sm_acc[(warp * G + h1) * HD + d0 + 8] = o[mt][3]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += 128) {
        const int g = idx / HD, e = idx % HD;
        float M = sm_m[g];  // warp 0 always holds a tile
#pragma unroll
        for (int w = 1; w < 4; w++) M = fmaxf(M, sm_m[w * G + g]);
        float tot = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = __expf(sm_m[w * G + g] - M);
            tot += sm_acc[(w * G + g) * HD + e] * f;
            l += sm_l[w * G + g] * f;
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
__global__ void attn_combine_kernel(const float* __restrict__ partial, int nH, int max_splits, int split_keys,
                                    const int32_t* __restrict__ row_pos, float* __restrict__ out, int8_t* __restrict__ codes,
                                    float* __restrict__ scales) {
    const int h = blockIdx.x, r = blockIdx.y, e = threadIdx.x;
    const int nsp = min((row_pos[r] + 1 + split_keys - 1) / split_keys, max_splits);  // never past the row's slots of the array
    const float* p = partial + ((size_t)r * nH + h) * max_splits * (HD + 2);
    // eight splits' loads are in flight at a time; the sums keep the split order
    float M = -INFINITY;
    for (int s0 = 0; s0 < nsp; s0 += 8) {
        float mv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) mv[u] = s0 + u < nsp ? p[(size_t)(s0 + u) * (HD + 2) + HD] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; u++) M = fmaxf(M, mv[u]);
    }
    float tot = 0.f, l = 0.f;
    for (int s0 = 0; s0 < nsp; s0 += 8) {
        float mv[8], av[8], lv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const bool in = s0 + u < nsp;
            const float* ps = p + (size_t)(s0 + u) * (HD + 2);
            mv[u] = in ? ps[HD] : 0.f;
            av[u] = in ? ps[e] : 0.f;
            lv[u] = in ? ps[HD + 1] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (s0 + u < nsp) {
                const float f = __expf(mv[u] - M);
                tot += av[u] * f;
                l += lv[u] * f;
            }
        }
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

// The same merge with two values per thread and four heads per block (grid (nH/4, T), 2*HD threads): with up to eight
// splits every load of the row is issued at once, before the maximum is known. Same sums in the same order, same codes.
template <int HD>
__global__ void __launch_bounds__(2 * HD) attn_combine2_kernel(const float* __restrict__ partial, int nH, int max_splits, int split_keys,
                                                               const int32_t* __restrict__ row_pos, float* __restrict__ out,
                                                               int8_t* __restrict__ codes, float* __restrict__ scales,
                                                               __half* __restrict__ x16, int x16_row0) {
    pdl_trigger();
    pdl_wait();
    constexpr int TPH = HD / 2;  // threads per head
    const int h = blockIdx.x * 4 + threadIdx.x / TPH, r = blockIdx.y, e = 2 * (threadIdx.x % TPH);
    const int nsp = min((row_pos[r] + 1 + split_keys - 1) / split_keys, max_splits);  // never past the row's slots of the array
    const float* p = partial + ((size_t)r * nH + h) * max_splits * (HD + 2);
    float M = -INFINITY, tot0 = 0.f, tot1 = 0.f, l = 0.f;
    if (nsp <= 8) {
        float mv[8], lv[8];
        float2 av[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const bool in = u < nsp;
            const float* ps = p + (size_t)u * (HD + 2);
            const float2 ml = in ? *reinterpret_cast<const float2*>(ps + HD) : make_float2(-INFINITY, 0.f);
            mv[u] = ml.x;
            lv[u] = ml.y;
            av[u] = in ? *reinterpret_cast<const float2*>(ps + e) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 8; u++) M = fmaxf(M, mv[u]);
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (u < nsp) {
                const float f = __expf(mv[u] - M);
                tot0 += av[u].x * f;
                tot1 += av[u].y * f;
                l += lv[u] * f;
            }
        }
    } else {
        for (int s = 0; s < nsp; s++) M = fmaxf(M, p[(size_t)s * (HD + 2) + HD]);
        for (int s = 0; s < nsp; s++) {
            const float* ps = p + (size_t)s * (HD + 2);
            const float f = __expf(ps[HD] - M);
            const float2 a = *reinterpret_cast<const float2*>(ps + e);
            tot0 += a.x * f;
            tot1 += a.y * f;
            l += ps[HD + 1] * f;
        }
    }
    const float y0 = tot0 / l, y1 = tot1 / l;
    const int D = nH * HD;
    *reinterpret_cast<float2*>(out + (size_t)r * D + h * HD + e) = make_float2(y0, y1);
    if (codes) {
        const int g = (h * HD + e) >> 5, nG = D >> 5;
        float ma = fmaxf(fabsf(y0), fabsf(y1));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
        const float sc = __fdiv_rn(ma, 127.f);
        const float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
        const int q0 = max(-127, min(127, __float2int_rn(__fmul_rn(y0, inv)))), q1 = max(-127, min(127, __float2int_rn(__fmul_rn(y1, inv))));
        int sum = q0 + q1;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        *reinterpret_cast<uint16_t*>(codes + (size_t)r * D + h * HD + e) = (uint16_t)((q0 & 0xff) | ((q1 & 0xff) << 8));
        if (x16) {  // the o projection's fp16 activation tiles
            x16_store1(x16, D, x16_row0 + r, h * HD + e, __fmul_rn((float)q0, sc));
            x16_store1(x16, D, x16_row0 + r, h * HD + e + 1, __fmul_rn((float)q1, sc));
        }
        if ((threadIdx.x & 15) == 0) {
            scales[(size_t)r * 2 * nG + g] = sc;
            scales[(size_t)r * 2 * nG + nG + g] = __fmul_rn(sc, (float)sum);
        }
    }
}

template <int HD>
void launch_combine(b200_ctx* ctx, const float* partial, int nH, int T, int max_splits, int split_keys, const int32_t* row_pos, float* out, ActQ aq) {
    if (nH % 4 == 0 && !((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(out)) & 7) && !(reinterpret_cast<uintptr_t>(aq.codes) & 1)) {
        __half* x16 = aq.codes ? ctx->x16_want : nullptr;
        launch_pdl(attn_combine2_kernel<HD>, dim3(nH / 4, T), dim3(2 * HD), 0, ctx->stream, partial, nH, max_splits, split_keys, row_pos, out, aq.codes, aq.scales,
                   x16, ctx->x16_row0);
        if (x16) ctx->x16_done += T;
    } else
        attn_combine_kernel<HD><<<dim3(nH, T), HD, 0, ctx->stream>>>(partial, nH, max_splits, split_keys, row_pos, out, aq.codes, aq.scales);
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

// ---- exact class, tiled: the same arithmetic with the K and V rows read once for the G query heads of a kv head ----
// Scores. Grid (key tiles of 256, kv heads, rows), 128 threads, two keys a thread (tid and tid + 128 of the tile). The G
// heads' query rows sit in shared memory as f64; a thread reads its keys' rows 16 bytes at a time and runs G ascending f64
// chains per key (fused multiply-adds: the f64 value may differ from a separate multiply and add in its last bit, which the
// rounding to f32 hides except for values within 2^-29 of a rounding boundary).
template <int HD, int G>
__global__ void __launch_bounds__(128) attn_exact_scores_tile_kernel(const float* __restrict__ q, int ldq, int nH, int nKV,
                                                                     const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                                                     const __half* __restrict__ kpool, const int32_t* __restrict__ table,
                                                                     int max_blocks, int block_rows, float* __restrict__ scores, int ld) {
    __shared__ double2 qs[G][HD / 2];
    const int r = blockIdx.z, kvh = blockIdx.y, key0 = blockIdx.x * 256;
    const int nkeys = min(row_pos[r] + 1, max_blocks * block_rows);
    if (key0 >= nkeys) return;
    for (int i = threadIdx.x; i < G * HD / 2; i += 128) {
        const int g = i / (HD / 2), d2 = i % (HD / 2);
        const float2 v = *reinterpret_cast<const float2*>(q + (size_t)r * ldq + (size_t)(kvh * G + g) * HD + 2 * d2);
        qs[g][d2] = make_double2((double)v.x, (double)v.y);
    }
    __syncthreads();
    const int32_t* tbl = table + (size_t)row_slot[r] * max_blocks;
    const int ka = key0 + threadIdx.x, kb = ka + 128;
    const bool has_a = ka < nkeys, has_b = kb < nkeys;
    if (!has_a) return;
    const int kbc = has_b ? kb : ka;  // a thread without a second key reads its first one twice and drops the result
    const uint4* ra = reinterpret_cast<const uint4*>(kpool + (((size_t)tbl[ka / block_rows] * nKV + kvh) * block_rows + ka % block_rows) * HD);
    const uint4* rb = reinterpret_cast<const uint4*>(kpool + (((size_t)tbl[kbc / block_rows] * nKV + kvh) * block_rows + kbc % block_rows) * HD);
    double acc_a[G], acc_b[G];
#pragma unroll
    for (int g = 0; g < G; g++) acc_a[g] = acc_b[g] = 0.0;
#pragma unroll 2
    for (int c = 0; c < HD / 8; c++) {
        const uint4 va = ra[c], vb = rb[c];
        const __half2* ha = reinterpret_cast<const __half2*>(&va);
        const __half2* hb = reinterpret_cast<const __half2*>(&vb);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 fa = __half22float2(ha[i]), fb = __half22float2(hb[i]);
            const double a0 = fa.x, a1 = fa.y, b0 = fb.x, b1 = fb.y;
#pragma unroll
            for (int g = 0; g < G; g++) {
                const double2 qq = qs[g][4 * c + i];
                acc_a[g] = fma(qq.x, a0, acc_a[g]);
                acc_b[g] = fma(qq.x, b0, acc_b[g]);
                acc_a[g] = fma(qq.y, a1, acc_a[g]);
                acc_b[g] = fma(qq.y, b1, acc_b[g]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
        float* s = scores + ((size_t)r * nH + kvh * G + g) * ld;
        s[ka] = (float)acc_a[g];
        if (has_b) s[kb] = (float)acc_b[g];
    }
}

// Weighted sum of the V rows. Grid (kv heads, rows), 256 threads: thread (dg, kl) owns dims 8*dg .. 8*dg+7 of the G heads and
// the keys kl, kl + KL, ... of every 256-key chunk, whose weights sit in shared memory as f64. Each thread folds its keys in
// ascending order in f64; the KL partial sums (KL consecutive lanes of a warp) are then added in a fixed butterfly. (The CPU path folds all keys in one ascending
// chain: the f64 sums differ in their last bits, the f32 results only where the f64 value lies within 2^-29 of a rounding
// boundary.)
template <int HD, int G>
__global__ void __launch_bounds__(256) attn_exact_av_tile_kernel(const float* __restrict__ w, int ld, int nH, int nKV,
                                                                 const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                                                 const __half* __restrict__ vpool, const int32_t* __restrict__ table,
                                                                 int max_blocks, int block_rows, float* __restrict__ out) {
    constexpr int DG = HD / 8, KL = 256 / DG, CH = 256;
    static_assert(KL <= 32, "the key lanes of a dim group are lanes of one warp");
    __shared__ double ws[G][CH];
    __shared__ int vrow[CH];   // the chunk's keys as rows of the pool (block id and row in the block resolved once a chunk)
    const int kvh = blockIdx.x, r = blockIdx.y;
    const int nkeys = min(row_pos[r] + 1, max_blocks * block_rows);
    const int kl = threadIdx.x % KL, dg = threadIdx.x / KL;
    const int32_t* tbl = table + (size_t)row_slot[r] * max_blocks;
    double acc[G][8];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[g][j] = 0.0;
    for (int kc = 0; kc < nkeys; kc += CH) {
        __syncthreads();
        for (int i = threadIdx.x; i < G * CH; i += 256) {
            const int g = i / CH, kk = i % CH;
            ws[g][kk] = kc + kk < nkeys ? (double)w[((size_t)r * nH + kvh * G + g) * ld + kc + kk] : 0.0;
        }
        {
            const int key = min(kc + (int)threadIdx.x, nkeys - 1);   // (CH == the block's 256 threads)
            vrow[threadIdx.x] = (tbl[key / block_rows] * nKV + kvh) * block_rows + key % block_rows;
        }
        __syncthreads();
        const int n = min(CH, nkeys - kc);
        auto fold = [&](const uint4& v, int kk) {
            const __half2* hv = reinterpret_cast<const __half2*>(&v);
            double vd[8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(hv[i]);
                vd[2 * i] = f.x;
                vd[2 * i + 1] = f.y;
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                const double wg = ws[g][kk];
#pragma unroll
                for (int j = 0; j < 8; j++) acc[g][j] = fma(wg, vd[j], acc[g][j]);
            }
        };
        // four keys' loads in flight per thread (ascending keys, the same chain of sums)
        int kk = kl;
        for (; kk + 3 * KL < n; kk += 4 * KL) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = *reinterpret_cast<const uint4*>(vpool + (size_t)vrow[kk + u * KL] * HD + 8 * dg);
#pragma unroll
            for (int u = 0; u < 4; u++) fold(v[u], kk + u * KL);
        }
        for (; kk < n; kk += KL) fold(*reinterpret_cast<const uint4*>(vpool + (size_t)vrow[kk] * HD + 8 * dg), kk);
    }
    // fold the KL key lanes
#pragma unroll
    for (int off = KL / 2; off >= 1; off >>= 1)
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[g][j] += __shfl_xor_sync(0xffffffffu, acc[g][j], off);
    if (kl == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            float* o = out + (size_t)r * nH * HD + (size_t)(kvh * G + g) * HD + 8 * dg;
            *reinterpret_cast<float4*>(o) = make_float4((float)acc[g][0], (float)acc[g][1], (float)acc[g][2], (float)acc[g][3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4((float)acc[g][4], (float)acc[g][5], (float)acc[g][6], (float)acc[g][7]);
        }
    }
}

template <int HD, int G>
int run_exact_tiled(b200_ctx* ctx, const float* q, int ldq, int T, int nH, int nKV, const int32_t* row_slot, const int32_t* row_pos,
                    int max_keys, KVView kv, float* scores, int ld, float* out, double scale, double softcap) {
    {
        ProfScope ps(ctx, PROF_ATTN_SPLIT);
        attn_exact_scores_tile_kernel<HD, G><<<dim3(ceil_div(max_keys, 256), nKV, T), 128, 0, ctx->stream>>>(
            q, ldq, nH, nKV, row_slot, row_pos, kv.k, kv.table, kv.max_blocks, kv.block_rows, scores, ld);
    }
    LAUNCH_CHECK(ctx);
    {
        ProfScope ps(ctx, PROF_ATTN_COMBINE);
        attn_exact_softmax_kernel<<<dim3(nH, T), 256, 0, ctx->stream>>>(row_pos, nH, scale, softcap, scores, ld);
    }
    LAUNCH_CHECK(ctx);
    {
        ProfScope ps(ctx, PROF_OTHER);
        attn_exact_av_tile_kernel<HD, G><<<dim3(nKV, T), 256, 0, ctx->stream>>>(scores, ld, nH, nKV, row_slot, row_pos, kv.v, kv.table,
                                                                               kv.max_blocks, kv.block_rows, out);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
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
        launch_combine<HD>(ctx, sc.partial, nH, T, sc.max_splits, kSplitKeys, row_pos, out, aq);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

constexpr int kMmaSplitKeys = 1024;

template <int HD, int G>
int run_mma(b200_ctx* ctx, const float* q, int ldq, int T, int nH, int nKV, float scale, float cap, const int32_t* row_slot,
            const int32_t* row_pos, int max_keys, KVView kv, AttnScratch sc, float* out, ActQ aq) {
    const int nsp = ceil_div(max_keys, kMmaSplitKeys);
    if (nsp > sc.max_splits) B200_FAIL(ctx, B200_BAD_ARGUMENT, "attention scratch too small for %d keys", max_keys);
    constexpr int smem = 4 * kMmaStages * 2 * 16 * HD * 2;
    static PerDeviceOnce attr_once;  // the attribute belongs to the device
    if (attr_once.first(ctx->device)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(attn_mma_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    dim3 grid(nsp, nKV, T);
    {
        ProfScope ps(ctx, PROF_ATTN_SPLIT);
        launch_pdl(attn_mma_kernel<HD, G>, grid, dim3(128), smem, ctx->stream, q, ldq, nH, nKV, scale, cap, row_slot, row_pos, kv.k, kv.v, kv.table,
                   kv.max_blocks, kv.block_rows, sc.partial, sc.max_splits, kMmaSplitKeys);
    }
    LAUNCH_CHECK(ctx);
    {
        ProfScope ps(ctx, PROF_ATTN_COMBINE);
        launch_combine<HD>(ctx, sc.partial, nH, T, sc.max_splits, kMmaSplitKeys, row_pos, out, aq);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

int launch_paged_attention_exact(b200_ctx* ctx, const float* q, int ldq, int T, int nH, int nKV, int hd, double scale,
                                 double softcap, const int32_t* row_slot, const int32_t* row_pos, int max_keys, KVView kv,
                                 float* scores, int ld, float* out, ActQ aq) {
    if (max_keys > ld) B200_FAIL(ctx, B200_BAD_ARGUMENT, "exact attention scratch holds %d keys, %d asked", ld, max_keys);
    // the usual head shapes: tiled kernels that read a K or V row once for the G heads of its kv head (16-byte row pieces:
    // the pools and q must be 16- and 8-byte aligned, which the engine's buffers are)
    const int G = nH / nKV;
    const bool aligned = (reinterpret_cast<uintptr_t>(kv.k) & 15) == 0 && (reinterpret_cast<uintptr_t>(kv.v) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(q) & 7) == 0 && (ldq & 1) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    static const bool no_tiled = getenv("B200_EXACT_ATTN_PLAIN") != nullptr;
    if (aligned && !no_tiled) {
        int st = -1;
#define EXACT_CASE(HD_, G_) \
    if (hd == HD_ && G == G_) st = run_exact_tiled<HD_, G_>(ctx, q, ldq, T, nH, nKV, row_slot, row_pos, max_keys, kv, scores, ld, out, scale, softcap)
        EXACT_CASE(128, 1); EXACT_CASE(128, 2); EXACT_CASE(128, 4); EXACT_CASE(128, 8);
        EXACT_CASE(64, 1); EXACT_CASE(64, 2); EXACT_CASE(64, 4); EXACT_CASE(64, 8);
#undef EXACT_CASE
        if (st >= 0) {
            if (st != B200_OK) return st;
            if (aq.codes) return launch_quant_g32(ctx, out, T, nH * hd, aq);
            return B200_OK;
        }
    }
    {
        ProfScope ps(ctx, PROF_ATTN_SPLIT);
        attn_exact_scores_kernel<<<dim3(ceil_div(max_keys, 128), nH, T), 128, 0, ctx->stream>>>(
            q, ldq, nH, nKV, hd, scale, softcap, row_slot, row_pos, kv.k, kv.table, kv.max_blocks, kv.block_rows, scores, ld);
    }
    LAUNCH_CHECK(ctx);
    {
        ProfScope ps(ctx, PROF_ATTN_COMBINE);
        attn_exact_softmax_kernel<<<dim3(nH, T), 256, 0, ctx->stream>>>(row_pos, nH, scale, softcap, scores, ld);
    }
    LAUNCH_CHECK(ctx);
    {
        ProfScope ps(ctx, PROF_OTHER);
        attn_exact_av_kernel<<<dim3(nH, T), ((hd + 31) / 32) * 32, 0, ctx->stream>>>(scores, ld, nH, nKV, hd, row_slot, row_pos, kv.v,
                                                                                     kv.table, kv.max_blocks, kv.block_rows, out);
    }
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
    // tensor-core kernel: 16-key tiles must be contiguous, i.e. the block size a multiple of 16
    static const bool use_mma = !getenv("B200_ATTN_SIMT");
    if (use_mma && kv.block_rows % 16 == 0) {
#define MMA_CASE(HD_, G_) \
    if (hd == HD_ && G == G_) return run_mma<HD_, G_>(ctx, q, ldq, T, nH, nKV, scale, softcap, row_slot, row_pos, max_keys, kv, sc, out, aq)
        MMA_CASE(128, 1); MMA_CASE(128, 2); MMA_CASE(128, 4); MMA_CASE(128, 8);
        MMA_CASE(64, 1); MMA_CASE(64, 2); MMA_CASE(64, 4); MMA_CASE(64, 8);
#undef MMA_CASE
    }
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

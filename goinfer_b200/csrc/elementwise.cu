// elementwise.cu — the HBM-bound row kernels of the step: embedding gather, residual + RMSNorm + per-32
// int8 activation quantization, SwiGLU + quantization, per-head QK RMSNorm + NeoX RoPE + paged fp16 KV
// store, expert fold. Each is one pass over its rows; arithmetic follows the reference's CPU path:
//   RMSNorm      decoder/rmsnorm.go:29-92      (f64 sum of squares, y = (x*inv)*w)
//   quantizer    backend/cuda/actgroup.cu:32-54 (sc = max/127, inv = sc>0 ? 1/sc : 0, RNE, clamp +-127, asum = sc*sum)
//   SwiGLU       decoder/mlp.go:269-290, silu in f64 decoder/rmsnorm.go:204-207
//   QK norm      decoder/program_cpu.go:351-364
//   RoPE         decoder/rope.go:28-64 (split-half, cos/sin and the rotation in f64)
//   residual     decoder/model_forward.go:98-119
//   expert fold  decoder/mlp.go:729-745 (out += w*src, rank order, no contraction)
#include "common.cuh"
#include "rowquant.cuh"

namespace {

__global__ void embed_gather_kernel(const void* __restrict__ table, int kind, int n_rows, const int32_t* __restrict__ ids, int H,
                                    float scale, float* __restrict__ h) {
    pdl_trigger();
    pdl_wait();
    int r = blockIdx.x;
    size_t id = (size_t)ids[r];
    float* out = h + (size_t)r * H;
    if (kind == B200_K_I8) {  // int8 rows, then one f32 scale per row
        const int8_t* row = (const int8_t*)table + id * H;
        const float ws = reinterpret_cast<const float*>((const int8_t*)table + (size_t)n_rows * H)[id];
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = __fmul_rn((float)row[i], ws);
            out[i] = scale != 1.f ? __fmul_rn(v, scale) : v;
        }
    } else if (kind == B200_K_F32) {
        const float* row = (const float*)table + id * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = scale != 1.f ? __fmul_rn(row[i], scale) : row[i];
    } else {
        const __half* row = (const __half*)table + id * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = __half2float(row[i]);
            out[i] = scale != 1.f ? __fmul_rn(v, scale) : v;
        }
    }
}

// value i of a matrix kept as n K-split partials `stride` floats apart: added in order, starting from the first
__device__ __forceinline__ float parts_at(const float* __restrict__ p, size_t stride, int n, size_t i) {
    float s = p[i];
    for (int k = 1; k < n; k++) s = __fadd_rn(s, p[(size_t)k * stride + i]);
    return s;
}

// One block per output row. Dynamic shared memory: H floats (the normed row) + 8 doubles.
__global__ void __launch_bounds__(256) add_rmsnorm_quant_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                                const float* __restrict__ w, int H, float eps,
                                                                float* __restrict__ normed, int8_t* __restrict__ codes,
                                                                float* __restrict__ scales,
                                                                const int32_t* __restrict__ gather_rows, int n_parts,
                                                                size_t part_stride) {
    extern __shared__ double smem_d[];
    double* red = smem_d;                 // 8 doubles
    float* row = (float*)(smem_d + 8);    // H floats
    const int j = blockIdx.x;
    const int r = gather_rows ? gather_rows[j] : j;
    float* hr = h + (size_t)r * H;
    double ss = 0;
    // eight elements a pass: their loads are all in flight before the first dependent add (the sum keeps its order)
    const float* dr = delta ? delta + (size_t)r * H : nullptr;
    int i = threadIdx.x;
    for (; i + 7 * (int)blockDim.x < H; i += 8 * blockDim.x) {
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; u++) x[u] = hr[i + u * blockDim.x];
        if (dr) {
            float d[8];
#pragma unroll
            for (int u = 0; u < 8; u++) d[u] = n_parts ? parts_at(dr, part_stride, n_parts, i + u * blockDim.x) : dr[i + u * blockDim.x];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                x[u] = __fadd_rn(x[u], d[u]);
                hr[i + u * blockDim.x] = x[u];
            }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            row[i + u * blockDim.x] = x[u];
            ss += (double)x[u] * (double)x[u];
        }
    }
    for (; i < H; i += blockDim.x) {
        float x = hr[i];
        if (dr) {
            x = __fadd_rn(x, n_parts ? parts_at(dr, part_stride, n_parts, i) : dr[i]);
            hr[i] = x;
        }
        row[i] = x;
        ss += (double)x * (double)x;
    }
    ss = warp_sum_f64(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    double tot = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) tot += red[k];
    const float inv = (float)(1.0 / sqrt(tot / (double)H + (double)eps));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nG = H >> 5;
#pragma unroll 4
    for (int g = warp; g < nG; g += 8) {  // unrolled: the groups' shuffle and divide chains interleave
        int i = g * 32 + lane;
        float y = __fmul_rn(__fmul_rn(row[i], inv), w[i]);
        if (normed) normed[(size_t)j * H + i] = y;
        if (codes) quant_group_warp(y, codes + (size_t)j * H + g * 32, scales + (size_t)j * 2 * nG + g,
                                    scales + (size_t)j * 2 * nG + nG + g, lane);
    }
    // tail for H not a multiple of 32 (f32-weight models only; no quantized output there)
    for (int i = nG * 32 + threadIdx.x; i < H; i += blockDim.x)
        if (normed) normed[(size_t)j * H + i] = __fmul_rn(__fmul_rn(row[i], inv), w[i]);
}

// The same row pass for widths that are a multiple of 32 and at most 8 * 256 * P: a thread keeps its P chunks of eight
// consecutive values in registers from the loads to the stores (no shared row buffer, every load of the row in flight at
// once), and a group of 32 is four lanes, so its maximum and sum take two shuffles each. The sum of squares is added in
// another order than the kernel above adds it, in f64, which the rounded f32 factor does not see.
template <int P>
__global__ void __launch_bounds__(256) add_rmsnorm_quant_vec_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                                    const float* __restrict__ w, int H, float eps,
                                                                    float* __restrict__ normed, int8_t* __restrict__ codes,
                                                                    float* __restrict__ scales, const int32_t* __restrict__ gather_rows,
                                                                    int n_parts, size_t part_stride, __half* __restrict__ x16) {
    pdl_trigger();
    pdl_wait();
    __shared__ double red[8];
    const int j = blockIdx.x, r = gather_rows ? gather_rows[j] : j, nC = H >> 3, nG = H >> 5;
    float* hr = h + (size_t)r * H;
    const float* dr = delta ? delta + (size_t)r * H : nullptr;
    float x[P][8];
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int c = p * 256 + threadIdx.x;
        if (c < nC) {
            const float4 a = *reinterpret_cast<const float4*>(hr + 8 * c), b = *reinterpret_cast<const float4*>(hr + 8 * c + 4);
            x[p][0] = a.x; x[p][1] = a.y; x[p][2] = a.z; x[p][3] = a.w; x[p][4] = b.x; x[p][5] = b.y; x[p][6] = b.z; x[p][7] = b.w;
        } else {
#pragma unroll
            for (int u = 0; u < 8; u++) x[p][u] = 0.f;
        }
    }
    if (dr) {
        float d[P][8];
        const int np = n_parts ? n_parts : 1;
#pragma unroll
        for (int p = 0; p < P; p++) {
            const int c = p * 256 + threadIdx.x;
#pragma unroll
            for (int u = 0; u < 8; u++) d[p][u] = 0.f;
            if (c < nC) {
                for (int k = 0; k < np; k++) {  // the partials are added in split order, starting from the first
                    const float* src = dr + (size_t)k * part_stride + 8 * c;
                    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
                    if (k == 0) {
                        d[p][0] = a.x; d[p][1] = a.y; d[p][2] = a.z; d[p][3] = a.w; d[p][4] = b.x; d[p][5] = b.y; d[p][6] = b.z; d[p][7] = b.w;
                    } else {
                        d[p][0] = __fadd_rn(d[p][0], a.x); d[p][1] = __fadd_rn(d[p][1], a.y); d[p][2] = __fadd_rn(d[p][2], a.z);
                        d[p][3] = __fadd_rn(d[p][3], a.w); d[p][4] = __fadd_rn(d[p][4], b.x); d[p][5] = __fadd_rn(d[p][5], b.y);
                        d[p][6] = __fadd_rn(d[p][6], b.z); d[p][7] = __fadd_rn(d[p][7], b.w);
                    }
                }
            }
        }
#pragma unroll
        for (int p = 0; p < P; p++) {
            const int c = p * 256 + threadIdx.x;
            if (c < nC) {
#pragma unroll
                for (int u = 0; u < 8; u++) x[p][u] = __fadd_rn(x[p][u], d[p][u]);
                *reinterpret_cast<float4*>(hr + 8 * c) = make_float4(x[p][0], x[p][1], x[p][2], x[p][3]);
                *reinterpret_cast<float4*>(hr + 8 * c + 4) = make_float4(x[p][4], x[p][5], x[p][6], x[p][7]);
            }
        }
    }
    double ss = 0;
#pragma unroll
    for (int p = 0; p < P; p++)
#pragma unroll
        for (int u = 0; u < 8; u++) ss += (double)x[p][u] * (double)x[p][u];
    ss = warp_sum_f64(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    double tot = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) tot += red[k];
    const float inv = (float)(1.0 / sqrt(tot / (double)H + (double)eps));
    const int q4 = threadIdx.x & 3;
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int c = p * 256 + threadIdx.x;
        if (p * 256 + (int)(threadIdx.x & ~31u) >= nC) break;  // a whole warp past the row (uniform)
        const bool live = c < nC;
        float y[8];
        if (live) {
            const float4 a = *reinterpret_cast<const float4*>(w + 8 * c), b = *reinterpret_cast<const float4*>(w + 8 * c + 4);
            const float wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int u = 0; u < 8; u++) y[u] = __fmul_rn(__fmul_rn(x[p][u], inv), wv[u]);
            if (normed) {
                *reinterpret_cast<float4*>(normed + (size_t)j * H + 8 * c) = make_float4(y[0], y[1], y[2], y[3]);
                *reinterpret_cast<float4*>(normed + (size_t)j * H + 8 * c + 4) = make_float4(y[4], y[5], y[6], y[7]);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 8; u++) y[u] = 0.f;
        }
        if (codes) {
            const int g = c >> 2;
            float dq[8];
            quant_group_quad(y, codes + (size_t)j * H + (size_t)g * 32, scales + (size_t)j * 2 * nG + g, scales + (size_t)j * 2 * nG + nG + g, q4, live,
                             x16 ? dq : nullptr);
            if (x16 && live) x16_store8(x16, H, j, 8 * c, dq);
        }
    }
}

__global__ void __launch_bounds__(256) quant_g32_kernel(const float* __restrict__ x, int K, int8_t* __restrict__ codes,
                                                        float* __restrict__ scales) {
    const int r = blockIdx.y, lane = threadIdx.x & 31, nG = K >> 5;
    const int g = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (g >= nG) return;
    float y = x[(size_t)r * K + g * 32 + lane];
    quant_group_warp(y, codes + (size_t)r * K + g * 32, scales + (size_t)r * 2 * nG + g, scales + (size_t)r * 2 * nG + nG + g, lane);
}

// The same quantizer with eight values per thread (K a multiple of 32, aligned rows); optionally lays the rows out as the
// tcgen05 matmul's fp16 tiles, rows x16_row0.. of the slot.
__global__ void __launch_bounds__(256) quant_g32_vec_kernel(const float* __restrict__ x, int K, int8_t* __restrict__ codes,
                                                            float* __restrict__ scales, __half* __restrict__ x16, int x16_row0) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, nG = K >> 5, nC = K >> 3;
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (blockIdx.x * 256 + (int)(threadIdx.x & ~31u) >= nC) return;  // a whole warp past the row
    const bool live = c < nC;
    float y[8];
    if (live) {
        const float4 a = *reinterpret_cast<const float4*>(x + (size_t)r * K + 8 * c), b = *reinterpret_cast<const float4*>(x + (size_t)r * K + 8 * c + 4);
        y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w; y[4] = b.x; y[5] = b.y; y[6] = b.z; y[7] = b.w;
    } else {
#pragma unroll
        for (int u = 0; u < 8; u++) y[u] = 0.f;
    }
    const int g = c >> 2;
    float dq[8];
    quant_group_quad(y, codes + (size_t)r * K + (size_t)g * 32, scales + (size_t)r * 2 * nG + g, scales + (size_t)r * 2 * nG + nG + g, threadIdx.x & 3,
                     live, x16 ? dq : nullptr);
    if (x16 && live) x16_store8(x16, K, x16_row0 + r, 8 * c, dq);
}

__device__ __forceinline__ float silu_f64(float x) {
    double x64 = (double)x;
    return (float)(x64 / (1.0 + exp(-x64)));
}

// fast class: silu in f32 with the hardware exponential and reciprocal (about 1e-6 relative of the f64 value); the tcgen05
// GEMM's fused epilogue uses the same expression
__device__ __forceinline__ float silu_f32(float x) { return __fdividef(x, __fadd_rn(1.f, __expf(-x))); }

// gate at gate_up[r*ld + f], up at gate_up[r*ld + F + f].
template <bool F64>
__global__ void __launch_bounds__(256) swiglu_quant_kernel(const float* __restrict__ gate_up, int F, int ld,
                                                           float* __restrict__ mid, int8_t* __restrict__ codes,
                                                           float* __restrict__ scales, int il) {
    const int r = blockIdx.y, lane = threadIdx.x & 31, nG = F >> 5;
    const int g = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (g >= nG) return;
    const int f = g * 32 + lane;
    const size_t gi = il ? (size_t)(f >> 7) * 256 + (f & 127) : (size_t)f;  // il: gate|up interleaved by 128 columns
    const float gt = gate_up[(size_t)r * ld + gi], up = gate_up[(size_t)r * ld + gi + (il ? 128 : F)];
    float y = __fmul_rn(F64 ? silu_f64(gt) : silu_f32(gt), up);
    if (mid) mid[(size_t)r * F + f] = y;
    if (codes) quant_group_warp(y, codes + (size_t)r * F + g * 32, scales + (size_t)r * 2 * nG + g, scales + (size_t)r * 2 * nG + nG + g, lane);
}

// The same with eight consecutive values per thread (vector loads, a group is four lanes). F a multiple of 32.
template <bool F64>
__global__ void __launch_bounds__(256) swiglu_quant_vec_kernel(const float* __restrict__ gate_up, int F, int ld, float* __restrict__ mid,
                                                               int8_t* __restrict__ codes, float* __restrict__ scales, int il,
                                                               __half* __restrict__ x16, int n_parts, size_t part_stride) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, nG = F >> 5, nC = F >> 3;
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (blockIdx.x * 256 + (int)(threadIdx.x & ~31u) >= nC) return;  // a whole warp past the row
    const bool live = c < nC;
    float y[8];
    if (live) {
        const int f = 8 * c, up_off = il ? 128 : F;
        const float* gp = gate_up + (size_t)r * ld + (il ? (size_t)(f >> 7) * 256 + (f & 127) : (size_t)f);
        const float4 g0 = *reinterpret_cast<const float4*>(gp), g1 = *reinterpret_cast<const float4*>(gp + 4);
        const float4 u0 = *reinterpret_cast<const float4*>(gp + up_off), u1 = *reinterpret_cast<const float4*>(gp + up_off + 4);
        float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        for (int k = 1; k < n_parts; k++) {  // gate_up is the first of the matmul's K-split partials: added in their order
            const float* pp = gp + (size_t)k * part_stride;
            const float4 a0 = *reinterpret_cast<const float4*>(pp), a1 = *reinterpret_cast<const float4*>(pp + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(pp + up_off), b1 = *reinterpret_cast<const float4*>(pp + up_off + 4);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int u = 0; u < 8; u++) {
                gv[u] = __fadd_rn(gv[u], av[u]);
                uv[u] = __fadd_rn(uv[u], bv[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) y[u] = __fmul_rn(F64 ? silu_f64(gv[u]) : silu_f32(gv[u]), uv[u]);
        if (mid) {
            *reinterpret_cast<float4*>(mid + (size_t)r * F + 8 * c) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4*>(mid + (size_t)r * F + 8 * c + 4) = make_float4(y[4], y[5], y[6], y[7]);
        }
    } else {
#pragma unroll
        for (int u = 0; u < 8; u++) y[u] = 0.f;
    }
    const int g = c >> 2;
    float dq[8];
    quant_group_quad(y, codes + (size_t)r * F + (size_t)g * 32, scales + (size_t)r * 2 * nG + g, scales + (size_t)r * 2 * nG + nG + g,
                     threadIdx.x & 3, live, x16 ? dq : nullptr);
    if (x16 && live) x16_store8(x16, F, r, 8 * c, dq);
}

// plain SwiGLU for widths that are not a multiple of 32 (f32-weight models)
__global__ void swiglu_plain_kernel(const float* __restrict__ gate_up, int F, int ld, float* __restrict__ mid) {
    const int r = blockIdx.y;
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f < F) mid[(size_t)r * F + f] = __fmul_rn(silu_f64(gate_up[(size_t)r * ld + f]), gate_up[(size_t)r * ld + F + f]);
}

__global__ void add_kernel(float* __restrict__ h, const float* __restrict__ d, size_t n, int n_parts, size_t part_stride) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] = __fadd_rn(h[i], n_parts ? parts_at(d, part_stride, n_parts, i) : d[i]);
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// One block per packed row. Shared: cos/sin of the row's position (f64), one head buffer per warp.
__global__ void __launch_bounds__(256) qknorm_rope_kvstore_kernel(
    float* __restrict__ qkv, int ld, int nH, int nKV, int hd, int half, const double* __restrict__ inv_freq,
    const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, const int32_t* __restrict__ row_slot,
    const int32_t* __restrict__ row_pos, __half* __restrict__ kpool, __half* __restrict__ vpool,
    const int32_t* __restrict__ table, int max_blocks, int block_rows, const float* __restrict__ parts, int n_parts,
    size_t part_stride) {
    extern __shared__ double smem_d[];
    double* cs = smem_d;                         // [half] cos, [half] sin
    float* hb = (float*)(smem_d + 2 * half);     // [8][hd]
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = row_pos[r], slot = row_slot[r];
    for (int d = threadIdx.x; d < half; d += blockDim.x) {
        double th = (double)pos * inv_freq[d];
        double s, c;
        sincos(th, &s, &c);
        cs[d] = c;
        cs[half + d] = s;
    }
    __syncthreads();
    const int blk = table[(size_t)slot * max_blocks + pos / block_rows];
    const int rib = pos % block_rows;
    float* buf = hb + warp * hd;
    float* rowp = qkv + (size_t)r * ld;
    for (int hh = warp; hh < nH + 2 * nKV; hh += 8) {
        const bool is_q = hh < nH, is_k = !is_q && hh < nH + nKV;
        float* src = rowp + (size_t)hh * hd;
        double ss = 0;
        for (int e = lane; e < hd; e += 32) {
            float x = n_parts ? parts_at(parts, part_stride, n_parts, (size_t)r * ld + (size_t)hh * hd + e) : src[e];
            buf[e] = x;
            ss += (double)x * (double)x;
        }
        const float* nw = is_q ? q_norm : (is_k ? k_norm : nullptr);
        if (nw) {  // per-head RMSNorm before RoPE
            ss = warp_sum_f64(ss);
            float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)eps));
            __syncwarp();
            for (int e = lane; e < hd; e += 32) buf[e] = __fmul_rn(__fmul_rn(buf[e], inv), nw[e]);
        }
        __syncwarp();
        if (is_q || is_k) {
            for (int d = lane; d < half; d += 32) {
                double x1 = buf[d], x2 = buf[half + d], c = cs[d], s = cs[half + d];
                float y1 = (float)(x1 * c - x2 * s), y2 = (float)(x2 * c + x1 * s);
                buf[d] = y1;
                buf[half + d] = y2;
            }
            __syncwarp();
        }
        if (is_q) {
            for (int e = lane; e < hd; e += 32) src[e] = buf[e];
        } else {
            const int kvh = is_k ? hh - nH : hh - nH - nKV;
            __half* dst = (is_k ? kpool : vpool) + (((size_t)blk * nKV + kvh) * block_rows + rib) * hd;
            for (int e = lane; e < hd; e += 32) dst[e] = __float2half_rn(buf[e]);
        }
        __syncwarp();
    }
}

// The same for head_dim 128 or 64 with two heads per warp and sixteen per block (grid.y walks the heads): a lane keeps
// HD/32 consecutive values of a head, the loads of both heads (and of every K-split partial) are in flight while the block's
// cos/sin table is computed, and the rotation partner comes by shuffle. Same arithmetic, expression by expression.
template <int HD>
__global__ void __launch_bounds__(256) qknorm_rope_kvstore_vec_kernel(
    float* __restrict__ qkv, int ld, int nH, int nKV, int half, const double* __restrict__ inv_freq,
    const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, const int32_t* __restrict__ row_slot,
    const int32_t* __restrict__ row_pos, __half* __restrict__ kpool, __half* __restrict__ vpool,
    const int32_t* __restrict__ table, int max_blocks, int block_rows, const float* __restrict__ parts, int n_parts,
    size_t part_stride) {
    pdl_trigger();
    pdl_wait();
    constexpr int hd = HD, V = HD / 32;   // values a lane
    __shared__ double cs[2 * 64];  // [half] cos, [half] sin
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_heads = nH + 2 * nKV;
    const int pos = row_pos[r], slot = row_slot[r];
    float x[2][V];
    const float* base = n_parts ? parts : qkv;
    const int np = n_parts ? n_parts : 1;
    auto load = [&](const float* p, float (&o)[V]) {
        if constexpr (V == 4) {
            const float4 a = *reinterpret_cast<const float4*>(p);
            o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
        } else {
            const float2 a = *reinterpret_cast<const float2*>(p);
            o[0] = a.x; o[1] = a.y;
        }
    };
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const int hh = blockIdx.y * 16 + 2 * warp + u;
#pragma unroll
        for (int i = 0; i < V; i++) x[u][i] = 0.f;
        if (hh < n_heads) {
            const size_t off = (size_t)r * ld + (size_t)hh * hd + V * lane;
            for (int k = 0; k < np; k++) {
                float a[V];
                load(base + (size_t)k * part_stride + off, a);
#pragma unroll
                for (int i = 0; i < V; i++) x[u][i] = k == 0 ? a[i] : __fadd_rn(x[u][i], a[i]);
            }
        }
    }
    for (int d = threadIdx.x; d < half; d += blockDim.x) {
        double th = (double)pos * inv_freq[d];
        double sn, c;
        sincos(th, &sn, &c);
        cs[d] = c;
        cs[half + d] = sn;
    }
    __syncthreads();
    const int blk = table[(size_t)slot * max_blocks + pos / block_rows];
    const int rib = pos % block_rows;
    const int e0 = V * lane;                       // this lane's first element
    const bool first = e0 < half, second = !first && e0 < 2 * half;
    const int partner = first ? lane + half / V : lane - half / V;
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const int hh = blockIdx.y * 16 + 2 * warp + u;
        if (hh >= n_heads) break;  // uniform over the warp
        const bool is_q = hh < nH, is_k = !is_q && hh < nH + nKV;
        const float* nw = is_q ? q_norm : (is_k ? k_norm : nullptr);
        float v[V];
#pragma unroll
        for (int i = 0; i < V; i++) v[i] = x[u][i];
        if (nw) {
            double ss = 0;
#pragma unroll
            for (int i = 0; i < V; i++) ss += (double)v[i] * (double)v[i];
            ss = warp_sum_f64(ss);
            const float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)eps));
            float wv[V];
            load(nw + e0, wv);
#pragma unroll
            for (int i = 0; i < V; i++) v[i] = __fmul_rn(__fmul_rn(v[i], inv), wv[i]);
        }
        if (is_q || is_k) {
#pragma unroll
            for (int i = 0; i < V; i++) {
                const float other = __shfl_sync(0xffffffffu, v[i], partner & 31);
                if (first) {
                    const double x1 = v[i], x2 = other, c = cs[e0 + i], sn = cs[half + e0 + i];
                    v[i] = (float)(x1 * c - x2 * sn);
                } else if (second) {
                    const double x1 = other, x2 = v[i], c = cs[e0 + i - half], sn = cs[e0 + i];
                    v[i] = (float)(x2 * c + x1 * sn);
                }
            }
        }
        if (is_q) {
            float* dq = qkv + (size_t)r * ld + (size_t)hh * hd + e0;
            if constexpr (V == 4) *reinterpret_cast<float4*>(dq) = make_float4(v[0], v[1], v[2], v[3]);
            else *reinterpret_cast<float2*>(dq) = make_float2(v[0], v[1]);
        } else {
            const int kvh = is_k ? hh - nH : hh - nH - nKV;
            __half* dst = (is_k ? kpool : vpool) + (((size_t)blk * nKV + kvh) * block_rows + rib) * hd + e0;
            const __half2 h0 = __floats2half2_rn(v[0], v[1]);
            if constexpr (V == 4) {
                const __half2 h1 = __floats2half2_rn(v[2], v[3]);
                *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const unsigned*>(&h0), *reinterpret_cast<const unsigned*>(&h1));
            } else {
                *reinterpret_cast<unsigned*>(dst) = *reinterpret_cast<const unsigned*>(&h0);
            }
        }
    }
}

// out row 256t + j = gate row 128t + j, out row 256t + 128 + j = up row 128t + j (rows of row_bytes bytes, a multiple of 16)
__global__ void interleave_rows128_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up, size_t row_bytes,
                                          uint8_t* __restrict__ out) {
    const int o = blockIdx.x, t = o >> 8, j = o & 255;
    const uint8_t* src = (j < 128 ? gate : up) + (size_t)(128 * t + (j & 127)) * row_bytes;
    uint4* d = reinterpret_cast<uint4*>(out + (size_t)o * row_bytes);
    const uint4* s = reinterpret_cast<const uint4*>(src);
    for (size_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d[i] = s[i];
}

// eo rows are in expert-sorted slot order; slot_of[row*k + rank] names the slot (-1: empty rank).
__global__ void fold_experts_kernel(const float* __restrict__ eo, const float* __restrict__ wts,
                                    const int32_t* __restrict__ slot_of, int k, int H, float* __restrict__ out) {
    const int r = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    float acc = 0.f;
    for (int j = 0; j < k; j++) {
        const int s = slot_of[(size_t)r * k + j];
        if (s >= 0) acc = __fadd_rn(acc, __fmul_rn(wts[(size_t)r * k + j], eo[(size_t)s * H + i]));
    }
    out[(size_t)r * H + i] = acc;
}

}  // namespace

int launch_embed_gather(b200_ctx* ctx, const void* table, int kind, int n_rows, const int32_t* ids, int T, int H, float scale, float* h) {
    launch_pdl(embed_gather_kernel, dim3(T), dim3(256), 0, ctx->stream, table, kind, n_rows, ids, H, (scale == 0.f ? 1.f : scale), h);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_add_rmsnorm_quant(b200_ctx* ctx, float* h, const float* delta, const float* w, int T, int H, float eps,
                             float* normed, ActQ aq, const int32_t* gather_rows, __half* x16) {
    if (aq.codes && (H % 32)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "quantized rows need a width that is a multiple of 32");
    size_t smem = 8 * sizeof(double) + (size_t)H * sizeof(float);
    ProfScope ps(ctx, PROF_NORM_QUANT);
    Parts pt{};
    if (delta && ctx->pending.n > 0 && ctx->pending.dst == delta && !gather_rows) {  // the matmul left its K-split partials for us
        pt = ctx->pending;
        ctx->pending = Parts{};
    }
    const float* dl = pt.n ? pt.p : delta;
    const bool vec = H % 32 == 0 && H <= 8192 && !((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(dl) | reinterpret_cast<uintptr_t>(w) |
                                                    reinterpret_cast<uintptr_t>(normed) | (uintptr_t)(pt.stride * 4)) & 15) &&
                     !(reinterpret_cast<uintptr_t>(aq.codes) & 7);
    if (vec && H <= 2048)
        launch_pdl(add_rmsnorm_quant_vec_kernel<1>, dim3(T), dim3(256), 0, ctx->stream, h, dl, w, H, eps, normed, aq.codes, aq.scales, gather_rows, pt.n, pt.stride, x16);
    else if (vec && H <= 4096)
        launch_pdl(add_rmsnorm_quant_vec_kernel<2>, dim3(T), dim3(256), 0, ctx->stream, h, dl, w, H, eps, normed, aq.codes, aq.scales, gather_rows, pt.n, pt.stride, x16);
    else if (vec)
        launch_pdl(add_rmsnorm_quant_vec_kernel<4>, dim3(T), dim3(256), 0, ctx->stream, h, dl, w, H, eps, normed, aq.codes, aq.scales, gather_rows, pt.n, pt.stride, x16);
    else {
        if (x16) B200_FAIL(ctx, B200_BAD_ARGUMENT, "fp16 activation tiles are laid out by the vector kernel only (width %% 32, aligned buffers)");
        add_rmsnorm_quant_kernel<<<T, 256, smem, ctx->stream>>>(h, dl, w, H, eps, normed, aq.codes, aq.scales, gather_rows, pt.n, pt.stride);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_quant_g32(b200_ctx* ctx, const float* x, int T, int K, ActQ aq) {
    if (K % 32) B200_FAIL(ctx, B200_BAD_ARGUMENT, "K must be a multiple of 32");
    if (!((reinterpret_cast<uintptr_t>(x) | (uintptr_t)((size_t)K * 4)) & 15) && !(reinterpret_cast<uintptr_t>(aq.codes) & 7)) {
        __half* x16 = ctx->x16_want;
        launch_pdl(quant_g32_vec_kernel, dim3(ceil_div(K / 8, 256), T), dim3(256), 0, ctx->stream, x, K, aq.codes, aq.scales, x16, ctx->x16_row0);
        if (x16) ctx->x16_done += T;
    } else {
        dim3 grid(ceil_div(K / 32, 8), T);
        quant_g32_kernel<<<grid, 256, 0, ctx->stream>>>(x, K, aq.codes, aq.scales);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_swiglu_quant(b200_ctx* ctx, const float* gate_up, int T, int F, int ld, float* mid, ActQ aq, bool f64_silu, bool interleaved128,
                        __half* x16) {
    ProfScope ps(ctx, PROF_SWIGLU);
    const int il = interleaved128 ? 1 : 0;
    if (il && (!aq.codes || F % 128)) B200_FAIL(ctx, B200_BAD_ARGUMENT, "interleaved gate|up needs a quantized output and F %% 128 == 0");
    const bool vec = aq.codes && F % 32 == 0 &&
                     !((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(mid) | (uintptr_t)((size_t)ld * 4)) & 15) &&
                     !(reinterpret_cast<uintptr_t>(aq.codes) & 7);
    Parts pt{};
    if (ctx->pending.n > 0 && ctx->pending.dst == gate_up) {  // the matmul left its K-split partials
        if (vec && ld == ctx->pending.cols && !((reinterpret_cast<uintptr_t>(ctx->pending.p) | (uintptr_t)(ctx->pending.stride * 4)) & 15)) {
            pt = ctx->pending;
            ctx->pending = Parts{};
        } else {
            ST_TRY(flush_pending_parts(ctx));
        }
    }
    if (aq.codes) {
        if (F % 32) B200_FAIL(ctx, B200_BAD_ARGUMENT, "F must be a multiple of 32");
        if (vec) {
            dim3 grid(ceil_div(F / 8, 256), T);
            const float* src = pt.n ? pt.p : gate_up;
            if (f64_silu) launch_pdl(swiglu_quant_vec_kernel<true>, grid, dim3(256), 0, ctx->stream, src, F, ld, mid, aq.codes, aq.scales, il, x16, pt.n, pt.stride);
            else launch_pdl(swiglu_quant_vec_kernel<false>, grid, dim3(256), 0, ctx->stream, src, F, ld, mid, aq.codes, aq.scales, il, x16, pt.n, pt.stride);
        } else {
            if (x16) B200_FAIL(ctx, B200_BAD_ARGUMENT, "fp16 activation tiles are laid out by the vector kernel only (aligned buffers)");
            dim3 grid(ceil_div(F / 32, 8), T);
            if (f64_silu) swiglu_quant_kernel<true><<<grid, 256, 0, ctx->stream>>>(gate_up, F, ld, mid, aq.codes, aq.scales, il);
            else swiglu_quant_kernel<false><<<grid, 256, 0, ctx->stream>>>(gate_up, F, ld, mid, aq.codes, aq.scales, il);
        }
    } else {
        dim3 grid(ceil_div(F, 256), T);
        swiglu_plain_kernel<<<grid, 256, 0, ctx->stream>>>(gate_up, F, ld, mid);
    }
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_interleave_rows128(b200_ctx* ctx, const uint8_t* gate, const uint8_t* up, int F, size_t row_bytes, uint8_t* out) {
    if (F % 128 || row_bytes % 16) B200_FAIL(ctx, B200_BAD_ARGUMENT, "row interleave needs F %% 128 == 0 and 16-byte rows");
    interleave_rows128_kernel<<<2 * F, 128, 0, ctx->stream>>>(gate, up, row_bytes, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_add(b200_ctx* ctx, float* h, const float* delta, size_t n) {
    Parts pt{};
    if (ctx->pending.n > 0 && ctx->pending.dst == delta) {
        pt = ctx->pending;
        ctx->pending = Parts{};
    }
    launch_pdl(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ctx->stream, h, pt.n ? pt.p : delta, n, pt.n, pt.stride);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_softcap(b200_ctx* ctx, float* x, size_t n, float cap) {
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x, n, cap);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_qknorm_rope_kvstore(b200_ctx* ctx, float* qkv, int ld, int T, int nH, int nKV, int hd, int rot_half,
                               const double* inv_freq, const float* q_norm, const float* k_norm, float eps,
                               const int32_t* row_slot, const int32_t* row_pos, KVView kv) {
    if (hd > 256 || 2 * rot_half > hd) B200_FAIL(ctx, B200_BAD_ARGUMENT, "head_dim up to 256, rotary_dim <= head_dim");
    size_t smem = 2 * (size_t)rot_half * sizeof(double) + 8 * (size_t)hd * sizeof(float);
    ProfScope ps(ctx, PROF_ROPE_KV);
    Parts pt{};
    if (ctx->pending.n > 0 && ctx->pending.dst == qkv) {  // the q|k|v matmul left its K-split partials for us
        pt = ctx->pending;
        ctx->pending = Parts{};
    }
    const bool vec = (hd == 128 || hd == 64) && rot_half % (hd / 32) == 0 && rot_half <= 64 && ld % 4 == 0 &&
                     !((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(pt.p) | (uintptr_t)(pt.stride * 4) |
                        reinterpret_cast<uintptr_t>(q_norm) | reinterpret_cast<uintptr_t>(k_norm)) & 15) &&
                     !((reinterpret_cast<uintptr_t>(kv.k) | reinterpret_cast<uintptr_t>(kv.v)) & 7);
    if (vec) {
        dim3 grid(T, ceil_div(nH + 2 * nKV, 16));
        if (hd == 128)
            launch_pdl(qknorm_rope_kvstore_vec_kernel<128>, grid, dim3(256), 0, ctx->stream, qkv, ld, nH, nKV, rot_half, inv_freq, q_norm, k_norm, eps, row_slot,
                       row_pos, kv.k, kv.v, kv.table, kv.max_blocks, kv.block_rows, pt.p, pt.n, pt.stride);
        else
            launch_pdl(qknorm_rope_kvstore_vec_kernel<64>, grid, dim3(256), 0, ctx->stream, qkv, ld, nH, nKV, rot_half, inv_freq, q_norm, k_norm, eps, row_slot,
                       row_pos, kv.k, kv.v, kv.table, kv.max_blocks, kv.block_rows, pt.p, pt.n, pt.stride);
    } else
    qknorm_rope_kvstore_kernel<<<T, 256, smem, ctx->stream>>>(qkv, ld, nH, nKV, hd, rot_half, inv_freq, q_norm, k_norm, eps,
                                                              row_slot, row_pos, kv.k, kv.v, kv.table, kv.max_blocks,
                                                              kv.block_rows, pt.p, pt.n, pt.stride);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

int launch_fold_experts(b200_ctx* ctx, const float* eo, const float* wts, const int32_t* slot_of, int T, int k, int H,
                        float* out) {
    dim3 grid(ceil_div(H, 256), T);
    fold_experts_kernel<<<grid, 256, 0, ctx->stream>>>(eo, wts, slot_of, k, H, out);
    LAUNCH_CHECK(ctx);
    return B200_OK;
}

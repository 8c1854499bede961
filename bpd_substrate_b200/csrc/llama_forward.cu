// Q8_0 Llama forward on the device: the composition of bpd_llama_block_cpu / bpd_llama_forward_cpu
// (bench/bpd_cpu.c:5608-5798 of the reference) out of the Q8_0 products of q8_0.cu / gemv_batch.cu and
// the small kernels below, which restate the reference's own steps:
//   rms_norm with a binary64 sum of squares        bench/bpd_cpu.c:4959-4988
//   rotary embedding, NORM pairing, freq factors   bench/bpd_cpu.c:5146-5183
//   f16 KV-cache write (round to nearest even)     bench/bpd_cpu.c:5240-5257
//   grouped-query attention, three-pass softmax    bench/bpd_cpu.c:5370-5433
//   SwiGLU, residual add, argmax (lowest index)    bench/bpd_cpu.c:5504-5507, 5466, 4512-4529
// Weights, caches and activations are device memory; the descriptor structs are host memory holding
// device pointers, with the reference's field order.  Everything runs on one stream in the reference's
// order; no kernel waits on another.  The small kernels are launched programmatically like the products: each lets the
// launch behind it be scheduled at once (a product then fetches its first weights meanwhile) and waits for the
// launch ahead of it before it touches memory, so activations and caches are read with plain loads, never through
// the read-only path (only weights are).
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

#include <cuda_fp16.h>

namespace bpdq {

// One CTA per row.  The reference adds the squares in binary64 in index order and rounds the mean
// to fp32; here 256 threads add strided partial sums in binary64 and a tree joins them.  The
// binary64 sums differ by ~1e-16 relative, which vanishes in the rounding to fp32 except when the
// mean sits within that distance of a rounding boundary.
__device__ __forceinline__ void cta_rmsnorm_row(const float* x, const float* __restrict__ w, float* y, int cols, float eps,
                                                double t)
{
    __shared__ double s_part[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = t;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += s_part[i];
    const float mean = (float)(tot / (double)cols);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    // eight loads in flight before the stores (x, y and, in the fused kernel, the residual may be the same memory,
    // so the compiler would otherwise wait for every store before the next load)
    for (int c0 = threadIdx.x; c0 < cols; c0 += 256 * 8) {
        float xv[8], wv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c = c0 + 256 * j;
            xv[j] = c < cols ? x[c] : 0.0f;
            wv[j] = (w && c < cols) ? w[c] : 1.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c = c0 + 256 * j;
            if (c < cols) {
                const float v = __fmul_rn(xv[j], scale);
                y[c] = w ? __fmul_rn(v, wv[j]) : v;
            }
        }
    }
}

// Rows of up to 4096 columns: every thread keeps its sixteen elements in registers and fetches their weights before
// the sum is joined, so the row is read once and the weights' latency runs under the reduction.  r: the residual to
// add first (x_io = x + r is written back), or null.  Same operations on the same values, in the same order, as the
// general path (thread t: columns t, t + 256, ...).
__device__ __forceinline__ void cta_add_rmsnorm_row_4096(float* x_io, const float* x, const float* r, const float* __restrict__ w,
                                                         float* y, int cols, float eps)
{
    __shared__ double s_part[8];
    float v[16], wv[16];
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int c = (int)threadIdx.x + 256 * i;
        v[i] = c < cols ? x[c] : 0.0f;
        wv[i] = (w && c < cols) ? w[c] : 1.0f;
    }
    if (r) {
        float rv[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int c = (int)threadIdx.x + 256 * i;
            rv[i] = c < cols ? r[c] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int c = (int)threadIdx.x + 256 * i;
            if (c < cols) {
                v[i] = __fadd_rn(v[i], rv[i]);
                x_io[c] = v[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; i++)
        if ((int)threadIdx.x + 256 * i < cols) t += (double)v[i] * (double)v[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = t;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += s_part[i];
    const float mean = (float)(tot / (double)cols);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int c = (int)threadIdx.x + 256 * i;
        if (c < cols) {
            const float u = __fmul_rn(v[i], scale);
            y[c] = w ? __fmul_rn(u, wv[i]) : u;
        }
    }
}

__global__ void __launch_bounds__(256) k_rmsnorm_llama(const float* in, const float* __restrict__ w, float* out, int cols, float eps)
{
    pdl_launch_dependents();
    pdl_wait();
    if (cols <= 4096) {
        cta_add_rmsnorm_row_4096(nullptr, in + (size_t)blockIdx.x * cols, nullptr, w, out + (size_t)blockIdx.x * cols, cols, eps);
        return;
    }
    const float* x = in + (size_t)blockIdx.x * cols;
    double t = 0.0;
    for (int c = threadIdx.x; c < cols; c += 256) {
        const double v = (double)x[c];
        t += v * v;
    }
    cta_rmsnorm_row(x, w, out + (size_t)blockIdx.x * cols, cols, eps, t);
}

// The residual add and the norm that follows it in one launch: x = x + r (kept), out = rms_norm(x) * w.
// Every thread squares and later re-reads the elements it has just written, in k_rmsnorm_llama's order.
__global__ void __launch_bounds__(256) k_add_rmsnorm_llama(float* x_io, const float* r, const float* __restrict__ w, float* out,
                                                            int cols, float eps)   // out may be r
{
    pdl_launch_dependents();
    pdl_wait();
    float* x = x_io + (size_t)blockIdx.x * cols;
    const float* rr = r + (size_t)blockIdx.x * cols;
    if (cols <= 4096) {
        cta_add_rmsnorm_row_4096(x, x, rr, w, out + (size_t)blockIdx.x * cols, cols, eps);
        return;
    }
    double t = 0.0;
    for (int c0 = threadIdx.x; c0 < cols; c0 += 256 * 8) {
        float xv[8], rv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c = c0 + 256 * j;
            xv[j] = c < cols ? x[c] : 0.0f;
            rv[j] = c < cols ? rr[c] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c = c0 + 256 * j;
            if (c < cols) {
                const float v = __fadd_rn(xv[j], rv[j]);
                x[c] = v;
                t += (double)v * (double)v;
            }
        }
    }
    cta_rmsnorm_row(x, w, out + (size_t)blockIdx.x * cols, cols, eps, t);
}

// The reference's libm returns the correctly rounded fp32 value of expf / cosf / sinf for all but
// a fraction of a percent of arguments; the device's fp32 versions are 1-2 ulp off for about half of
// them.  Such last-bit differences are harmless by themselves, but every product that follows
// re-quantizes its input to int8, where a last-bit difference now and then flips a rounding and
// becomes a 1e-3 difference.  So these small kernels evaluate in binary64 and round once.
__device__ __forceinline__ float exp_rounded(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float cos_rounded(float x) { return (float)cos((double)x); }
__device__ __forceinline__ float sin_rounded(float x) { return (float)sin((double)x); }

// In place or out of place.  Thread = (token, head, pair).  theta is reached as the reference reaches
// it, by repeated multiplication from (float)pos, so that the angle has the same bits.
__device__ __forceinline__ void rope_pair(float x0, float x1, int pair, int half, int pos, const float* __restrict__ freq_factors,
                                          float theta_scale, float& y0, float& y1)
{
    if (pair < half) {
        float theta = (float)pos;
        for (int i = 0; i < pair; i++) theta = __fmul_rn(theta, theta_scale);
        const float ff = freq_factors ? freq_factors[pair] : 1.0f;
        const float te = __fdiv_rn(theta, ff);
        const float c = cos_rounded(te), s = sin_rounded(te);
        y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    } else {
        y0 = x0;
        y1 = x1;
    }
}

__global__ void __launch_bounds__(256) k_rope_norm(const float* in, float* out, const int32_t* pos_ids,
                                                    const float* __restrict__ freq_factors,
                                                    int n_tokens, int n_heads, int head_dim, int n_dims, float theta_scale)
{
    pdl_launch_dependents();
    pdl_wait();
    const int half = n_dims / 2;
    const long total = (long)n_tokens * n_heads * (head_dim / 2);
    for (long u = (long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long)gridDim.x * blockDim.x) {
        const int pair = (int)(u % (head_dim / 2));
        const long th = u / (head_dim / 2);
        const int t = (int)(th / n_heads);
        const float* src = in + th * head_dim;
        float* dst = out + th * head_dim;
        float y0, y1;
        rope_pair(src[2 * pair], src[2 * pair + 1], pair, half, pos_ids[t], freq_factors, theta_scale, y0, y1);
        dst[2 * pair] = y0;
        dst[2 * pair + 1] = y1;
    }
}

// The three steps between the q/k/v products and attention in one launch: q rotated in place, k rotated
// and stored to its cache row, v stored to its cache row (f16 rounding of the same fp32 values the separate
// steps round).  Thread = (token, head of q|k|v, pair).
template <int F16>
__global__ void __launch_bounds__(256) k_rope_qk_store_kv(float* q, const float* k, const float* v, void* k_cache, void* v_cache,
                                                           const int32_t* pos_ids,
                                                           const float* __restrict__ freq_factors, int n_tokens, int n_heads,
                                                           int n_kv_heads, int head_dim, int n_dims, float theta_scale,
                                                           int max_seq_len, int* err)
{
    pdl_launch_dependents();
    pdl_wait();
    const int half = n_dims / 2, pairs = head_dim / 2, heads = n_heads + 2 * n_kv_heads;
    const long total = (long)n_tokens * heads * pairs;
    for (long u = (long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long)gridDim.x * blockDim.x) {
        const int pair = (int)(u % pairs);
        const long th = u / pairs;
        const int t = (int)(th / heads), h = (int)(th - (long)t * heads);
        const int pos = pos_ids[t];
        if (h < n_heads) {
            float* p = q + ((size_t)t * n_heads + h) * head_dim + 2 * pair;
            float y0, y1;
            rope_pair(p[0], p[1], pair, half, pos, freq_factors, theta_scale, y0, y1);
            p[0] = y0;
            p[1] = y1;
        } else {
            const bool is_k = h < n_heads + n_kv_heads;
            const int hk = h - n_heads - (is_k ? 0 : n_kv_heads);
            const float* p = (is_k ? k : v) + ((size_t)t * n_kv_heads + hk) * head_dim + 2 * pair;
            float y0 = p[0], y1 = p[1];
            if (pos < 0 || pos >= max_seq_len) {      // no cache row of that index: nothing is stored, code 20 is recorded
                if (pair == 0 && hk == 0 && err) atomicCAS(err, 0, 20);
                continue;
            }
            if (is_k) rope_pair(p[0], p[1], pair, half, pos, freq_factors, theta_scale, y0, y1);
            const size_t at = ((size_t)pos * n_kv_heads + hk) * head_dim + 2 * pair;
            void* cache = is_k ? k_cache : v_cache;
            if (F16) {
                reinterpret_cast<__half*>(cache)[at] = __float2half_rn(y0);
                reinterpret_cast<__half*>(cache)[at + 1] = __float2half_rn(y1);
            } else {
                reinterpret_cast<float*>(cache)[at] = y0;
                reinterpret_cast<float*>(cache)[at + 1] = y1;
            }
        }
    }
}

// cache[pos[t]][:] = f16(src[t][:]) (round to nearest even) or the fp32 copy.  A position outside
// [0, max_seq_len) has no cache row: nothing is stored for that token and code 20 is recorded.
template <int F16>
__global__ void __launch_bounds__(256) k_kv_write(void* cache, const float* src, const int32_t* pos_ids, int n_tokens, int row,
                                                   int max_seq_len, int* err)
{
    pdl_launch_dependents();
    pdl_wait();
    const long total = (long)n_tokens * row;
    for (long u = (long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long)gridDim.x * blockDim.x) {
        const int t = (int)(u / row), i = (int)(u - (long)t * row);
        const int pos = pos_ids[t];
        if (pos < 0 || pos >= max_seq_len) {
            if (i == 0 && err) atomicCAS(err, 0, 20);
            continue;
        }
        const size_t at = (size_t)pos * row + i;
        if (F16) reinterpret_cast<__half*>(cache)[at] = __float2half_rn(src[u]);
        else reinterpret_cast<float*>(cache)[at] = src[u];
    }
}

// One CTA per (query token, query head).  In the reference ALL n_kv cache rows take part: rows past
// the query's position score -1e38 and weigh exp(-huge) = 0, so they add exact zeros to the sum and to
// the output (the cache holds finite values); they are skipped here, which leaves every bit as it is.
// Scores: raw dot products (multiply, then add, in index order, one thread per cache row, the row read
// 16 bytes at a time), scaled afterwards; maximum; exp and sum (added in index order by one thread, as
// the reference adds them); normalisation by the reciprocal; then thread d adds v[ic][d] * w[ic] over
// the rows in order.
template <int F16>
__global__ void __launch_bounds__(256) k_gqa_attn(const float* q, const void* kc, const void* vc, float* dst, int n_kv,
                                                   int n_q_heads, int n_kv_heads, int head_dim, float scale, int kv_offset)
{
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sh[];
    float* scores = sh;                   // [n_kv]
    float* sq = sh + n_kv;                // [head_dim]
    __shared__ float s_red[8];
    const int qt = blockIdx.x / n_q_heads, iq = blockIdx.x % n_q_heads;
    const int kv_head = iq / (n_q_heads / n_kv_heads);
    const int q_pos = kv_offset + qt;
    const float* pq = q + ((size_t)qt * n_q_heads + iq) * head_dim;
    float* pdst = dst + ((size_t)qt * n_q_heads + iq) * head_dim;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int d = tid; d < head_dim; d += 256) sq[d] = pq[d];
    __syncthreads();
    auto load = [&](const void* base, size_t idx) -> float {
        return F16 ? __half2float(reinterpret_cast<const __half*>(base)[idx]) : reinterpret_cast<const float*>(base)[idx];
    };
    n_kv = n_kv < q_pos + 1 ? n_kv : q_pos + 1;      // the rows that can weigh more than zero
    constexpr int kVec = F16 ? 8 : 4;                 // elements per 16-byte load
    const bool vec_ok = (head_dim % kVec) == 0 && ((uintptr_t)kc & 15) == 0;
    float mx = -1e38f;
    for (int ic = tid; ic < n_kv; ic += 256) {
        const size_t row = ((size_t)ic * n_kv_heads + kv_head) * head_dim;
        float s = 0.0f;
        if (vec_ok) {
            const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(kc) + row * (F16 ? 2 : 4));
            for (int j = 0; j < head_dim / kVec; j++) {
                const uint4 w = __ldcg(p + j);     // the cache rows may have been written by the launch before this one
                float kf[kVec];
                if (F16) {
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
                        kf[(2 * i) % kVec] = f2.x;
                        kf[(2 * i + 1) % kVec] = f2.y;
                    }
                } else {
                    kf[0] = __uint_as_float(w.x); kf[1] = __uint_as_float(w.y);
                    kf[2] = __uint_as_float(w.z); kf[3] = __uint_as_float(w.w);
                }
#pragma unroll
                for (int i = 0; i < kVec; i++) s = __fadd_rn(s, __fmul_rn(sq[j * kVec + i], kf[i]));
            }
        } else {
            for (int d = 0; d < head_dim; d++) s = __fadd_rn(s, __fmul_rn(sq[d], load(kc, row + d)));
        }
        const float sv = __fmul_rn(s, scale);
        scores[ic] = sv;
        mx = fmaxf(mx, sv);
    }
    mx = warp_max(mx);
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, s_red[i]);
    __syncthreads();
    for (int ic = tid; ic < n_kv; ic += 256) scores[ic] = exp_rounded(__fsub_rn(scores[ic], mx));
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
        int ic = 0;
        for (; ic + 8 <= n_kv; ic += 8) {            // eight loads in flight, the additions in index order
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = scores[ic + i];
#pragma unroll
            for (int i = 0; i < 8; i++) t = __fadd_rn(t, e[i]);
        }
        for (; ic < n_kv; ic++) t = __fadd_rn(t, scores[ic]);
        s_red[0] = t;
    }
    __syncthreads();
    const float sum = s_red[0];
    const float inv = (sum == 0.0f) ? 0.0f : __fdiv_rn(1.0f, sum);
    for (int ic = tid; ic < n_kv; ic += 256) scores[ic] = __fmul_rn(scores[ic], inv);
    __syncthreads();
    for (int d = tid; d < head_dim; d += 256) {
        float acc = 0.0f;
        int ic = 0;
        for (; ic + 8 <= n_kv; ic += 8) {            // eight rows' loads in flight, the additions in index order
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = load(vc, ((size_t)(ic + i) * n_kv_heads + kv_head) * head_dim + d);
#pragma unroll
            for (int i = 0; i < 8; i++) acc = __fadd_rn(acc, __fmul_rn(e[i], scores[ic + i]));
        }
        for (; ic < n_kv; ic++)
            acc = __fadd_rn(acc, __fmul_rn(load(vc, ((size_t)ic * n_kv_heads + kv_head) * head_dim + d), scores[ic]));
        pdst[d] = acc;
    }
}

__global__ void __launch_bounds__(256) k_swiglu_f32(const float* gate, const float* up, float* dst, long n)   // dst may be gate
{
    pdl_launch_dependents();
    pdl_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float g = gate[i];
        dst[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, exp_rounded(-g))), up[i]);
    }
}
__global__ void __launch_bounds__(256) k_add_f32(const float* a, const float* b, float* dst, long n)
{
    pdl_launch_dependents();
    pdl_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        dst[i] = __fadd_rn(a[i], b[i]);
}

// One CTA per row; the largest value wins, the lowest index among equals (v > best in index order).
__global__ void __launch_bounds__(256) k_argmax_rows(const float* x, long long* out, int n)
{
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_v[256];
    __shared__ int s_i[256];
    const float* row = x + (size_t)blockIdx.x * n;
    float best = row[0];
    int bi = 0;
    for (int k = threadIdx.x; k < n; k += 256) {
        const float v = row[k];
        if (v > best || (v == best && k < bi)) { best = v; bi = k; }
    }
    s_v[threadIdx.x] = best;
    s_i[threadIdx.x] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v = s_v[threadIdx.x + o];
            const int i = s_i[threadIdx.x + o];
            if (v > s_v[threadIdx.x] || (v == s_v[threadIdx.x] && i < s_i[threadIdx.x])) {
                s_v[threadIdx.x] = v;
                s_i[threadIdx.x] = i;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = s_i[0];
}

// A launch that may be scheduled while the launch ahead of it on the stream still runs (every kernel here waits for that
// launch before it touches memory).
template <typename... KArgs, typename... Args>
static int launch_ordered(void (*kern)(KArgs...), int grid, int block, size_t smem, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
}

static int grid_1d(long n)
{
    long want = (n + 255) / 256, cap = (long)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

static int launch_attn(const float* q, const void* kc, const void* vc, float* dst, int n_q, int n_kv, int H, int HKV, int D,
                       float scale, int kv_offset, int f16, cudaStream_t s)
{
    const size_t sh = (size_t)(n_kv + D) * sizeof(float);
    if (sh > 200 * 1024) return BPDQ_ERR_RANGE;      // scores live in shared memory
    static bool attr_set[2][64] = {{false}};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[f16 ? 1 : 0][dev]) {
        int rc = f16 ? check_cuda(cudaFuncSetAttribute(k_gqa_attn<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024))
                     : check_cuda(cudaFuncSetAttribute(k_gqa_attn<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (rc) return rc;
        attr_set[f16 ? 1 : 0][dev] = true;
    }
    if (f16) launch_ordered(k_gqa_attn<1>, n_q * H, 256, sh, s, q, kc, vc, dst, n_kv, H, HKV, D, scale, kv_offset);
    else launch_ordered(k_gqa_attn<0>, n_q * H, 256, sh, s, q, kc, vc, dst, n_kv, H, HKV, D, scale, kv_offset);
    return check_cuda(cudaGetLastError());
}

static int launch_rope(const float* in, float* out, const int32_t* pos_ids, const float* ff, int n_tokens, int n_heads,
                       int head_dim, int n_dims, float freq_base, cudaStream_t s)
{
    // the step between consecutive pairs' angles, computed where the reference computes it: on the host
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    launch_ordered(k_rope_norm, grid_1d((long)n_tokens * n_heads * head_dim / 2), 256, 0, s, in, out, pos_ids, ff, n_tokens, n_heads,
                                                                                 head_dim, n_dims, theta_scale);
    return check_cuda(cudaGetLastError());
}

static int launch_kv_write(void* cache, const float* src, const int32_t* pos_ids, int n_tokens, int row, int f16, int max_seq_len,
                           cudaStream_t s)
{
    if (f16) launch_ordered(k_kv_write<1>, grid_1d((long)n_tokens * row), 256, 0, s, cache, src, pos_ids, n_tokens, row, max_seq_len, device_error_flag());
    else launch_ordered(k_kv_write<0>, grid_1d((long)n_tokens * row), 256, 0, s, cache, src, pos_ids, n_tokens, row, max_seq_len, device_error_flag());
    return check_cuda(cudaGetLastError());
}

// One product: on the re-tiled copy of the matrix (tensor cores, every token in one pass over the weights)
// when there is one and enough tokens to pay for it, else on the rows (one pass per token).
constexpr int kTilesMinTokens = 3;
static int product(const uint8_t* rows, const uint8_t* tiles, const float* x, float* out, int n_tokens, int N, int K,
                   cudaStream_t s, Workspace* ws)
{
    if (tiles && n_tokens >= kTilesMinTokens) {
        // consecutive products share one piece of scratch: they are ordered on the stream
        Workspace one = ws ? *ws : Workspace{nullptr, 0, 0};
        return gemm_q8_0_tiles(tiles, x, out, n_tokens, N, K, s, ws ? &one : nullptr);
    }
    return bpd_qmatmul_q8_0_cuda(rows, x, out, n_tokens, N, K, s);
}

// Products that read the same vector: one launch where the fast Q8_0 kernel applies (one token, K a
// multiple of 256, aligned pointers), else one call each.  Same arithmetic either way.
static int products_shared_input(int n, const uint8_t* const* Ws, const uint8_t* const* Ts, float* const* outs, const int* Ns,
                                 const float* x, int n_tokens, int K, cudaStream_t s, Workspace* ws)
{
    if (n_tokens == 1 && gemv_q8_0_fast_multi(n, Ws, outs, Ns, x, K, s) == 0) return 0;
    for (int j = 0; j < n; j++) {
        int rc = product(Ws[j], Ts[j], x, outs[j], n_tokens, Ns[j], K, s, ws);
        if (rc) return rc;
    }
    return 0;
}

static int check_cfg(const bpd_llama_config* c, int n_tokens, int kv_pos)
{
    if (!c || n_tokens < 1 || kv_pos < 0) return BPDQ_ERR_ARG;
    if (c->n_layers < 0 || c->n_heads < 1 || c->n_kv_heads < 1 || c->head_dim < 2 || (c->head_dim & 1)) return BPDQ_ERR_ARG;
    if (c->n_heads % c->n_kv_heads) return BPDQ_ERR_ARG;
    if (c->embed_dim != c->n_heads * c->head_dim || (c->embed_dim % 32) || c->ffn_dim < 32 || (c->ffn_dim % 32)) return BPDQ_ERR_ARG;
    if (c->rope_dim < 0 || c->rope_dim > c->head_dim || (c->rope_dim & 1)) return BPDQ_ERR_ARG;
    if (c->max_seq_len < 1 || kv_pos + n_tokens > c->max_seq_len) return BPDQ_ERR_RANGE;
    if ((size_t)(c->max_seq_len + c->head_dim) * sizeof(float) > 200 * 1024) return BPDQ_ERR_RANGE;   // scores live in shared memory
    return 0;
}

static int launch_rope_qk_store_kv(float* q, const float* k, const float* v, void* k_cache, void* v_cache, const int32_t* pos_ids,
                                   const float* ff, int n_tokens, int H, int HKV, int D, int n_dims, float freq_base, int f16,
                                   int max_seq_len, cudaStream_t s)
{
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    const int grid = grid_1d((long)n_tokens * (H + 2 * HKV) * (D / 2));
    if (f16) launch_ordered(k_rope_qk_store_kv<1>, grid, 256, 0, s, q, k, v, k_cache, v_cache, pos_ids, ff, n_tokens, H, HKV, D, n_dims, theta_scale,
                                                        max_seq_len, device_error_flag());
    else launch_ordered(k_rope_qk_store_kv<0>, grid, 256, 0, s, q, k, v, k_cache, v_cache, pos_ids, ff, n_tokens, H, HKV, D, n_dims, theta_scale,
                                                    max_seq_len, device_error_flag());
    return check_cuda(cudaGetLastError());
}

// One transformer block.  x_normed: s1 already holds rms_norm(x) * attn_norm_w (the block before fused it
// with its last residual add).  fuse_next: the last residual add also writes rms_norm(x) * next_norm_w to s1.
// The fused launches do the same operations on the same values as the separate steps.
static int block_forward(float* x, const bpd_llama_layer_weights* lw, const bpd_llama_layer_weights* lt,
                         const bpd_llama_config* cfg, const int32_t* pos_ids,
                         int n_tokens, int kv_pos, void* k_cache, void* v_cache, float* s1, float* s2, float* s3,
                         const float* rope_freqs, bool x_normed, bool fuse_next, const float* next_norm_w, cudaStream_t s,
                         Workspace* ws)
{
    const int E = cfg->embed_dim, H = cfg->n_heads, HKV = cfg->n_kv_heads, D = cfg->head_dim, F = cfg->ffn_dim;
    const int n_kv_full = cfg->max_seq_len;
    int rc;
    const int row = HKV * D;
    // scratch3 holds K and, behind it, V (it is at least n_tokens * H*D floats and H*D >= 2 * HKV*D
    // whenever two or more query heads share a KV head; otherwise V is computed after K is stored)
    const bool kv_together = (size_t)2 * row <= (size_t)H * D;
    float* vbuf = kv_together ? s3 + (size_t)n_tokens * row : s3;
    if (!x_normed) launch_ordered(k_rmsnorm_llama, n_tokens, 256, 0, s, x, lw->attn_norm_w, s1, E, cfg->rms_eps);
    {
        const uint8_t* Ws[3] = {lw->w_q, lw->w_k, lw->w_v};
        const uint8_t* Ts[3] = {lt ? lt->w_q : nullptr, lt ? lt->w_k : nullptr, lt ? lt->w_v : nullptr};
        float* outs[3] = {s2, s3, vbuf};
        const int Ns[3] = {H * D, row, row};
        if ((rc = products_shared_input(kv_together ? 3 : 2, Ws, Ts, outs, Ns, s1, n_tokens, E, s, ws))) return rc;
    }
    if (kv_together) {
        if ((rc = launch_rope_qk_store_kv(s2, s3, vbuf, k_cache, v_cache, pos_ids, rope_freqs, n_tokens, H, HKV, D, cfg->rope_dim,
                                          cfg->rope_base, cfg->kv_cache_f16, cfg->max_seq_len, s)))
            return rc;
    } else {
        if ((rc = launch_rope(s2, s2, pos_ids, rope_freqs, n_tokens, H, D, cfg->rope_dim, cfg->rope_base, s))) return rc;
        if ((rc = launch_rope(s3, s3, pos_ids, rope_freqs, n_tokens, HKV, D, cfg->rope_dim, cfg->rope_base, s))) return rc;
        if ((rc = launch_kv_write(k_cache, s3, pos_ids, n_tokens, row, cfg->kv_cache_f16, cfg->max_seq_len, s))) return rc;
        if ((rc = product(lw->w_v, lt ? lt->w_v : nullptr, s1, vbuf, n_tokens, row, E, s, ws))) return rc;
        if ((rc = launch_kv_write(v_cache, vbuf, pos_ids, n_tokens, row, cfg->kv_cache_f16, cfg->max_seq_len, s))) return rc;
    }
    if ((rc = launch_attn(s2, k_cache, v_cache, s1, n_tokens, n_kv_full, H, HKV, D, 1.0f / sqrtf((float)D), kv_pos,
                          cfg->kv_cache_f16, s)))
        return rc;
    if ((rc = product(lw->w_o, lt ? lt->w_o : nullptr, s1, s2, n_tokens, E, H * D, s, ws))) return rc;
    launch_ordered(k_add_rmsnorm_llama, n_tokens, 256, 0, s, x, s2, lw->ffn_norm_w, s1, E, cfg->rms_eps);
    {
        const uint8_t* Ws[2] = {lw->w_gate, lw->w_up};
        const uint8_t* Ts[2] = {lt ? lt->w_gate : nullptr, lt ? lt->w_up : nullptr};
        float* outs[2] = {s2, s3};
        const int Ns[2] = {F, F};
        if ((rc = products_shared_input(2, Ws, Ts, outs, Ns, s1, n_tokens, E, s, ws))) return rc;
    }
    launch_ordered(k_swiglu_f32, grid_1d((long)n_tokens * F), 256, 0, s, s2, s3, s2, (long)n_tokens * F);
    if ((rc = product(lw->w_down, lt ? lt->w_down : nullptr, s2, s1, n_tokens, E, F, s, ws))) return rc;
    if (fuse_next) launch_ordered(k_add_rmsnorm_llama, n_tokens, 256, 0, s, x, s1, next_norm_w, s1, E, cfg->rms_eps);
    else launch_ordered(k_add_f32, grid_1d((long)n_tokens * E), 256, 0, s, x, s1, x, (long)n_tokens * E);
    return check_cuda(cudaGetLastError());
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

/* device-pointer twins of the steps' _cpu entry points (same argument order, plus the stream) */
int bpd_rmsnorm_llama_cuda(const float* input, const float* weight, float* output, int n_rows, int row_len, float eps,
                           void* stream)
{
    if (n_rows < 0 || row_len <= 0 || (n_rows > 0 && (!input || !output))) return latch(BPDQ_ERR_ARG);
    if (n_rows == 0) return 0;
    launch_ordered(k_rmsnorm_llama, n_rows, 256, 0, (cudaStream_t)stream, input, weight, output, row_len, eps);
    int rc = check_cuda(cudaGetLastError());
    return rc ? latch(rc) : 0;
}
int bpd_rope_norm_freqs_cuda(const float* input, float* output, const int32_t* pos_ids, const float* freq_factors,
                             int n_tokens, int n_heads, int head_dim, int n_dims, float freq_base, void* stream)
{
    if (n_tokens < 0 || n_heads < 1 || head_dim < 2 || (head_dim & 1) || n_dims < 0 || n_dims > head_dim || (n_dims & 1))
        return latch(BPDQ_ERR_ARG);
    if (n_tokens == 0) return 0;
    if (!input || !output || !pos_ids) return latch(BPDQ_ERR_ARG);
    int rc = launch_rope(input, output, pos_ids, freq_factors, n_tokens, n_heads, head_dim, n_dims, freq_base, (cudaStream_t)stream);
    return rc ? latch(rc) : 0;
}
int bpd_kv_cache_write_f16_cuda(uint16_t* cache, const float* src, const int32_t* pos_ids, int n_tokens, int n_kv_heads,
                                int head_dim, int max_seq_len, void* stream)
{
    if (n_tokens < 0 || n_kv_heads < 1 || head_dim < 1 || max_seq_len < 1 || (n_tokens > 0 && (!cache || !src || !pos_ids)))
        return latch(BPDQ_ERR_ARG);
    if (n_tokens == 0) return 0;
    int rc = launch_kv_write(cache, src, pos_ids, n_tokens, n_kv_heads * head_dim, 1, max_seq_len, (cudaStream_t)stream);
    return rc ? latch(rc) : 0;
}
int bpd_kv_cache_write_cuda(float* cache, const float* src, const int32_t* pos_ids, int n_tokens, int n_kv_heads, int head_dim,
                            int max_seq_len, void* stream)
{
    if (n_tokens < 0 || n_kv_heads < 1 || head_dim < 1 || max_seq_len < 1 || (n_tokens > 0 && (!cache || !src || !pos_ids)))
        return latch(BPDQ_ERR_ARG);
    if (n_tokens == 0) return 0;
    int rc = launch_kv_write(cache, src, pos_ids, n_tokens, n_kv_heads * head_dim, 0, max_seq_len, (cudaStream_t)stream);
    return rc ? latch(rc) : 0;
}
int bpd_gqa_attn_cuda(const float* q, const void* k, const void* v, float* dst, int n_q_tokens, int n_kv, int n_q_heads,
                      int n_kv_heads, int head_dim, float scale, int kv_offset, int kv_is_f16, void* stream)
{
    if (n_q_tokens < 0 || n_kv < 1 || n_q_heads < 1 || n_kv_heads < 1 || (n_q_heads % n_kv_heads) || head_dim < 1)
        return latch(BPDQ_ERR_ARG);
    if (n_q_tokens == 0) return 0;
    if (!q || !k || !v || !dst) return latch(BPDQ_ERR_ARG);
    int rc = launch_attn(q, k, v, dst, n_q_tokens, n_kv, n_q_heads, n_kv_heads, head_dim, scale, kv_offset, kv_is_f16,
                         (cudaStream_t)stream);
    return rc ? latch(rc) : 0;
}
int bpd_swiglu_fuse_cuda(const float* gate, const float* up, float* dst, int n, void* stream)
{
    if (n < 0 || (n > 0 && (!gate || !up || !dst))) return latch(BPDQ_ERR_ARG);
    if (n == 0) return 0;
    launch_ordered(k_swiglu_f32, grid_1d(n), 256, 0, (cudaStream_t)stream, gate, up, dst, n);
    int rc = check_cuda(cudaGetLastError());
    return rc ? latch(rc) : 0;
}
int bpd_argmax_dim_cuda(const float* x, long long* out, int outer, int dim_size, int inner, void* stream)
{
    if (outer < 0 || dim_size < 1 || inner != 1 || (outer > 0 && (!x || !out))) return latch(BPDQ_ERR_ARG);
    if (outer == 0) return 0;
    launch_ordered(k_argmax_rows, outer, 256, 0, (cudaStream_t)stream, x, out, dim_size);
    int rc = check_cuda(cudaGetLastError());
    return rc ? latch(rc) : 0;
}

int bpd_llama_block_cuda(float* x, const bpd_llama_layer_weights* lw, const bpd_llama_config* cfg, const int32_t* pos_ids,
                         int n_tokens, int kv_pos, void* k_cache, void* v_cache, float* scratch1, float* scratch2,
                         float* scratch3, const float* rope_freqs, void* stream)
{
    int rc = check_cfg(cfg, n_tokens, kv_pos);
    if (rc) return latch(rc);
    if (!x || !lw || !pos_ids || !k_cache || !v_cache || !scratch1 || !scratch2 || !scratch3) return latch(BPDQ_ERR_ARG);
    rc = block_forward(x, lw, nullptr, cfg, pos_ids, n_tokens, kv_pos, k_cache, v_cache, scratch1, scratch2, scratch3, rope_freqs,
                       false, false, nullptr, (cudaStream_t)stream, nullptr);
    return rc ? latch(rc) : 0;
}

// floats of the forward's own vectors (x and the reference's three scratch vectors)
static void forward_floats(const bpd_llama_config* cfg, int n_tokens, size_t& nx, size_t& n1, size_t& n2)
{
    const int E = cfg->embed_dim, F = cfg->ffn_dim, H = cfg->n_heads, D = cfg->head_dim;
    const size_t max_dim = (size_t)(E > F ? E : F), max_proj = (size_t)(H * D > F ? H * D : F);
    nx = ((size_t)n_tokens * E + 63) / 64 * 64;
    n1 = ((size_t)n_tokens * max_dim + 63) / 64 * 64;
    n2 = ((size_t)n_tokens * max_proj + 63) / 64 * 64;
}

static int llama_forward(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights, const bpd_llama_weights* tiles,
                         const bpd_llama_config* cfg, const int32_t* pos_ids, int kv_pos, void* k_cache, void* v_cache,
                         float* logits_out, long long* token_out, Workspace* ws, cudaStream_t s)
{
    int rc = check_cfg(cfg, n_tokens, kv_pos);
    if (rc) return latch(rc);
    if (!token_ids || !weights || !pos_ids || !k_cache || !v_cache || !logits_out || !weights->token_embd ||
        !weights->output_w || (cfg->n_layers > 0 && !weights->layers))
        return latch(BPDQ_ERR_ARG);
    const int E = cfg->embed_dim, D = cfg->head_dim, HKV = cfg->n_kv_heads;
    size_t nx, n1, n2;
    forward_floats(cfg, n_tokens, nx, n1, n2);
    float* base = reinterpret_cast<float*>(scratch_take(ws, kScratchForward, (nx + n1 + 2 * n2) * sizeof(float), s, &rc));
    if (!base) return rc;
    float *x = base, *s1 = x + nx, *s2 = s1 + n1, *s3 = s2 + n2;
    if ((rc = bpd_embed_lookup_q8_0_vocab_cuda(weights->token_embd, token_ids, x, n_tokens, E, cfg->vocab_size, s))) return rc;
    const size_t kv_layer = (size_t)cfg->max_seq_len * HKV * D * (cfg->kv_cache_f16 ? 2 : 4);
    // every block's last residual add also computes the norm that follows it: the next block's, or the output norm
    for (int layer = 0; layer < cfg->n_layers; layer++) {
        const bool last = layer + 1 == cfg->n_layers;
        rc = block_forward(x, &weights->layers[layer], tiles && tiles->layers ? &tiles->layers[layer] : nullptr, cfg, pos_ids,
                           n_tokens, kv_pos, (uint8_t*)k_cache + layer * kv_layer, (uint8_t*)v_cache + layer * kv_layer, s1, s2, s3,
                           weights->rope_freqs, layer > 0, true,
                           last ? weights->output_norm_w : weights->layers[layer + 1].attn_norm_w, s, ws);
        if (rc) return latch(rc);
    }
    if (cfg->n_layers == 0) launch_ordered(k_rmsnorm_llama, n_tokens, 256, 0, s, x, weights->output_norm_w, s1, E, cfg->rms_eps);
    if ((rc = product(weights->output_w, tiles ? tiles->output_w : nullptr, s1, logits_out, n_tokens, cfg->vocab_size, E, s, ws)))
        return rc;
    if (token_out) launch_ordered(k_argmax_rows, n_tokens, 256, 0, s, logits_out, token_out, cfg->vocab_size);
    rc = check_cuda(cudaGetLastError());
    return rc ? latch(rc) : 0;
}

int bpd_llama_forward_tiles_cuda(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights,
                                 const bpd_llama_weights* tiles, const bpd_llama_config* cfg, const int32_t* pos_ids,
                                 int kv_pos, void* k_cache, void* v_cache, float* logits_out, long long* token_out,
                                 void* stream)
{
    return llama_forward(token_ids, n_tokens, weights, tiles, cfg, pos_ids, kv_pos, k_cache, v_cache, logits_out, token_out,
                         nullptr, (cudaStream_t)stream);
}

// The same with caller-owned scratch (bpdq_llama_forward_workspace_bytes; 16-byte aligned): no allocation, no
// state shared with other calls.
size_t bpdq_llama_forward_workspace_bytes(const bpd_llama_config* cfg, int n_tokens)
{
    if (!cfg || n_tokens < 1 || check_cfg(cfg, n_tokens, 0) == BPDQ_ERR_ARG) return 0;
    size_t nx, n1, n2;
    forward_floats(cfg, n_tokens, nx, n1, n2);
    const int kmax = cfg->embed_dim > cfg->ffn_dim ? cfg->embed_dim : cfg->ffn_dim;
    return (nx + n1 + 2 * n2) * sizeof(float) + 512 + gemm_q8_0_tiles_workspace(n_tokens, 0, kmax) + 256;
}
int bpd_llama_forward_ws_cuda(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights,
                              const bpd_llama_weights* tiles, const bpd_llama_config* cfg, const int32_t* pos_ids, int kv_pos,
                              void* k_cache, void* v_cache, float* logits_out, long long* token_out, void* workspace,
                              size_t workspace_bytes, void* stream)
{
    if (!workspace || ((uintptr_t)workspace & 15)) return latch(workspace ? BPDQ_ERR_ALIGN : BPDQ_ERR_ARG);
    Workspace ws = {(uint8_t*)workspace, workspace_bytes, 0};
    return llama_forward(token_ids, n_tokens, weights, tiles, cfg, pos_ids, kv_pos, k_cache, v_cache, logits_out, token_out, &ws,
                         (cudaStream_t)stream);
}

int bpd_llama_forward_cuda(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights,
                           const bpd_llama_config* cfg, const int32_t* pos_ids, int kv_pos, void* k_cache, void* v_cache,
                           float* logits_out, long long* token_out, void* stream)
{
    return bpd_llama_forward_tiles_cuda(token_ids, n_tokens, weights, nullptr, cfg, pos_ids, kv_pos, k_cache, v_cache, logits_out,
                                        token_out, stream);
}

}  // extern "C"

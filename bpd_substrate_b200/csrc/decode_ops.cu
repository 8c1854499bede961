// fp32 operators of the decode dispatch: the symbol surface that
// inference/llamatov_gpu_llama.py:15-31 of the reference binds from its generated kernel
// library (lib/kernel_templates_llama.pl: k_vecmat :107-158, k_rms_norm :529-593, elementwise
// :600-830, k_matmul :1104-1290).  They sit either side of the quantized GEMVs in a decode
// step; all are memory bound and small.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

// c[col] = sum_k a[k] * b[k*n + col]   (weights fp32 [k][n], the reference's layout).
// A CTA covers 32 consecutive columns; its 8 warps take k = w, w+8, ... (coalesced 128-byte
// rows of b), keep 4 loads in flight, and are added in warp order 0..7 through shared memory.
__global__ void __launch_bounds__(256) k_vecmat_f32(const float* __restrict__ a, const float* __restrict__ b,
                                                    float* __restrict__ c, int k, int n)
{
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane;
    float acc = 0.0f;
    if (col < n) {
        int i = warp;
        for (; i + 24 < k; i += 32) {
            const float b0 = __ldg(b + (size_t)i * n + col), b1 = __ldg(b + (size_t)(i + 8) * n + col);
            const float b2 = __ldg(b + (size_t)(i + 16) * n + col), b3 = __ldg(b + (size_t)(i + 24) * n + col);
            acc = fmaf(__ldg(a + i), b0, acc);
            acc = fmaf(__ldg(a + i + 8), b1, acc);
            acc = fmaf(__ldg(a + i + 16), b2, acc);
            acc = fmaf(__ldg(a + i + 24), b3, acc);
        }
        for (; i < k; i += 8) acc = fmaf(__ldg(a + i), __ldg(b + (size_t)i * n + col), acc);
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < n) {
        float s = part[0][lane];
#pragma unroll
        for (int w = 1; w < 8; w++) s += part[w][lane];
        c[col] = s;
    }
}

// out[row][col] = in[row][col] * rsqrt(mean(in[row]^2) + eps) * weight[col]; one CTA per row.
__global__ void __launch_bounds__(256) k_rms_norm(const float* __restrict__ in, const float* __restrict__ w,
                                                  float* __restrict__ out, int cols, float eps)
{
    __shared__ float s_sum[8];
    const float* x = in + (size_t)blockIdx.x * cols;
    float t = 0.0f;
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float v = x[c];
        t = fmaf(v, v, t);
    }
    t = warp_sum(t);
    if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = t;
    __syncthreads();
    float tot = s_sum[0];
#pragma unroll
    for (int i = 1; i < 8; i++) tot += s_sum[i];
    const float scale = rsqrtf(tot / (float)cols + eps);
    for (int c = threadIdx.x; c < cols; c += 256) out[(size_t)blockIdx.x * cols + c] = x[c] * scale * w[c];
}

enum { OP_ADD = 0, OP_MUL = 1, OP_SILU = 2 };
template <int OP>
__global__ void __launch_bounds__(256) k_elementwise(const float* __restrict__ a, const float* __restrict__ b,
                                                     float* __restrict__ out, long n)
{
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float x = a[i];
        float r;
        if (OP == OP_ADD) r = x + b[i];
        else if (OP == OP_MUL) r = x * b[i];
        else r = x / (1.0f + expf(-x));   // lib/kernel_templates_llama.pl:668
        out[i] = r;
    }
}

// C[M][N] = A[M][K] @ B[K][N], 32x32 shared-memory tiles (lib/kernel_templates_llama.pl:1104-1290).
__global__ void __launch_bounds__(1024) k_matmul_f32(const float* __restrict__ A, const float* __restrict__ B,
                                                     float* __restrict__ C, int M, int N, int K)
{
    __shared__ float sA[32][33], sB[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int row = blockIdx.y * 32 + ty, col = blockIdx.x * 32 + tx;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        sA[ty][tx] = (row < M && k0 + tx < K) ? A[(size_t)row * K + k0 + tx] : 0.0f;
        sB[ty][tx] = (k0 + ty < K && col < N) ? B[(size_t)(k0 + ty) * N + col] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 32; i++) acc = fmaf(sA[ty][i], sB[i][tx], acc);
        __syncthreads();
    }
    if (row < M && col < N) C[(size_t)row * N + col] = acc;
}

static int ew_grid(long n)
{
    long want = (n + 255) / 256, cap = (long)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

void gpu_vecmat(const float* a, const float* b, float* c, int k, int n)
{
    if (k < 0 || n < 0 || (n > 0 && k > 0 && (!a || !b || !c))) { latch(BPDQ_ERR_ARG); return; }
    if (n == 0) return;
    k_vecmat_f32<<<(n + 31) / 32, 256, 0, current_stream()>>>(a, b, c, k, n);
    check_cuda(cudaGetLastError());
}
void gpu_rms_norm(const float* in, const float* w, float* out, int rows, int cols, float eps)
{
    if (rows < 0 || cols <= 0 || (rows > 0 && (!in || !w || !out))) { latch(BPDQ_ERR_ARG); return; }
    if (rows == 0) return;
    k_rms_norm<<<rows, 256, 0, current_stream()>>>(in, w, out, cols, eps);
    check_cuda(cudaGetLastError());
}
void gpu_add(const float* a, const float* b, float* out, int n)
{
    if (n < 0 || (n > 0 && (!a || !b || !out))) { latch(BPDQ_ERR_ARG); return; }
    if (n == 0) return;
    k_elementwise<OP_ADD><<<ew_grid(n), 256, 0, current_stream()>>>(a, b, out, n);
    check_cuda(cudaGetLastError());
}
void gpu_mul(const float* a, const float* b, float* out, int n)
{
    if (n < 0 || (n > 0 && (!a || !b || !out))) { latch(BPDQ_ERR_ARG); return; }
    if (n == 0) return;
    k_elementwise<OP_MUL><<<ew_grid(n), 256, 0, current_stream()>>>(a, b, out, n);
    check_cuda(cudaGetLastError());
}
void gpu_silu(const float* in, float* out, int n)
{
    if (n < 0 || (n > 0 && (!in || !out))) { latch(BPDQ_ERR_ARG); return; }
    if (n == 0) return;
    k_elementwise<OP_SILU><<<ew_grid(n), 256, 0, current_stream()>>>(in, in, out, n);
    check_cuda(cudaGetLastError());
}
void gpu_matmul(const float* A, const float* B, float* C, int M, int N, int K)
{
    if (M < 0 || N < 0 || K < 0 || (M > 0 && N > 0 && (!A || !B || !C))) { latch(BPDQ_ERR_ARG); return; }
    if (M == 0 || N == 0) return;
    k_matmul_f32<<<dim3((N + 31) / 32, (M + 31) / 32), dim3(32, 32), 0, current_stream()>>>(A, B, C, M, N, K);
    check_cuda(cudaGetLastError());
}
void gpu_matmul_opt(const float* A, const float* B, float* C, int M, int N, int K) { gpu_matmul(A, B, C, M, N, K); }

}  // extern "C"

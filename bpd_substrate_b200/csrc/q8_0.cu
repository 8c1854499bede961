// Q8_0 on device pointers: the `_cuda` twins of the reference's CPU entry points
// bpd_dequant_q8_0_cpu (bench/bpd_cpu.c:3960-3973), bpd_quant_q8_0_cpu (:4106-4136),
// bpd_qmatmul_q8_0_cpu (:4295-4315), bpd_embed_lookup_q8_0_cpu (:4002-4013), plus the exact
// int32 block dots of bpd_qdot_q8_0_q8_0_cpu (:4263-4280) for parity checks.
//
// A Q8_0 block is 34 bytes (fp16 scale, 32 int8) and only 2-byte aligned, so the simple kernels
// here move 16-bit words; the GEMV fast path (gemv_batch.cu) stages whole rows in shared memory
// and realigns there.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

// One thread = 4 consecutive outputs (float4 store); 8 threads per block.
__global__ void __launch_bounds__(256) k_dequant_q8_0(const uint8_t* __restrict__ raw, float* __restrict__ out,
                                                      long n_blocks)
{
    const long n_items = n_blocks * 8;
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long)gridDim.x * blockDim.x) {
        const long b = it >> 3;
        const int q = (int)(it & 7);
        const unsigned short* blk = reinterpret_cast<const unsigned short*>(raw + b * BPDQ_Q80_BYTES);
        const float s = f16_bits_to_f32(__ldg(blk));
        const unsigned short lo = __ldg(blk + 1 + 2 * q), hi = __ldg(blk + 2 + 2 * q);
        float4 o;
        o.x = (float)(signed char)(lo & 0xFF) * s;
        o.y = (float)(signed char)(lo >> 8) * s;
        o.z = (float)(signed char)(hi & 0xFF) * s;
        o.w = (float)(signed char)(hi >> 8) * s;
        __stcs(reinterpret_cast<float4*>(out) + it, o);
    }
}

// Rows gathered by token id, then dequantized: out[t][embed_dim].  An id outside [0, vocab) reads nothing and
// writes nothing (the row of `out` keeps its contents); the kernel records code 21 in the error word instead.
__global__ void __launch_bounds__(256) k_embed_lookup_q8_0(const uint8_t* __restrict__ table,
                                                           const int32_t* __restrict__ ids, float* __restrict__ out,
                                                           int n_tokens, int blocks_per_row, int vocab, int* __restrict__ err)
{
    const long per_tok = (long)blocks_per_row * 8;
    const long n_items = per_tok * n_tokens;
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long)gridDim.x * blockDim.x) {
        const long t = it / per_tok, r = it - t * per_tok;
        const long b = r >> 3;
        const int q = (int)(r & 7);
        const int id = __ldg(ids + t);
        if (id < 0 || id >= vocab) {
            if (r == 0 && err) atomicCAS(err, 0, 21);
            continue;
        }
        const unsigned short* blk = reinterpret_cast<const unsigned short*>(
            table + ((size_t)id * blocks_per_row + b) * BPDQ_Q80_BYTES);
        const float s = f16_bits_to_f32(__ldg(blk));
        const unsigned short lo = __ldg(blk + 1 + 2 * q), hi = __ldg(blk + 2 + 2 * q);
        float4 o;
        o.x = (float)(signed char)(lo & 0xFF) * s;
        o.y = (float)(signed char)(lo >> 8) * s;
        o.z = (float)(signed char)(hi & 0xFF) * s;
        o.w = (float)(signed char)(hi >> 8) * s;
        reinterpret_cast<float4*>(out)[it] = o;
    }
}

// Quantizer: 8 lanes per 32-value block, byte-identical to bpd_quant_q8_0_cpu
// (IEEE division, round-half-even, scale stored as fp16 of amax/127).
__global__ void __launch_bounds__(256) k_quant_q8_0(const float* __restrict__ x, uint8_t* __restrict__ y, long n_blocks)
{
    const long n_items = (n_blocks * 8 + 31) / 32 * 32;   // whole warps, so that shuffles see all lanes
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long)gridDim.x * blockDim.x) {
        const long b = it >> 3;
        const int q = (int)(it & 7);
        const bool live = b < n_blocks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = __ldg(reinterpret_cast<const float4*>(x) + it);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        if (!live) continue;
        const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        auto qz = [mul](float f) -> unsigned { return (unsigned)__float2int_rn(__fmul_rn(f, mul)) & 0xFFu; };
        unsigned short* blk = reinterpret_cast<unsigned short*>(y + b * BPDQ_Q80_BYTES);
        if (q == 0) blk[0] = __half_as_ushort(__float2half_rn(__fdiv_rn(amax, 127.0f)));
        blk[1 + 2 * q] = (unsigned short)(qz(v.x) | (qz(v.y) << 8));
        blk[2 + 2 * q] = (unsigned short)(qz(v.z) | (qz(v.w) << 8));
    }
}

// Exact int32 dot of every block pair (w[b] . a[b]).
__global__ void __launch_bounds__(256) k_q8_0_block_dots(const uint8_t* __restrict__ w, const uint8_t* __restrict__ a,
                                                         int32_t* __restrict__ dots, long n_blocks)
{
    for (long b = (long)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (long)gridDim.x * blockDim.x) {
        const unsigned short* wb = reinterpret_cast<const unsigned short*>(w + b * BPDQ_Q80_BYTES) + 1;
        const unsigned short* ab = reinterpret_cast<const unsigned short*>(a + b * BPDQ_Q80_BYTES) + 1;
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t ww = __ldg(wb + 2 * i) | ((uint32_t)__ldg(wb + 2 * i + 1) << 16);
            const uint32_t aa = __ldg(ab + 2 * i) | ((uint32_t)__ldg(ab + 2 * i + 1) << 16);
            s = dp4a_ss(ww, aa, s);
        }
        dots[b] = s;
    }
}

// Generic GEMV for any K that is a multiple of 32 (slow path: byte-granular loads, every warp
// quantizes the activation blocks it touches).  One warp per weight row; lane l takes blocks
// l, l+32, ...; lanes are summed by a butterfly (xor 16 .. 1).
__global__ void __launch_bounds__(256) k_gemv_q8_0_generic(const uint8_t* __restrict__ W, const float* __restrict__ x,
                                                           float* __restrict__ out, int N, int nbk)
{
    const int lane = threadIdx.x & 31;
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= N) return;
    const uint8_t* wr = W + (size_t)row * nbk * BPDQ_Q80_BYTES;
    float acc = 0.0f;
    for (int b = lane; b < nbk; b += 32) {
        const float* xb = x + (size_t)b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(__ldg(xb + i)));
        const float ad = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
        const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        const unsigned short* wb = reinterpret_cast<const unsigned short*>(wr + (size_t)b * BPDQ_Q80_BYTES);
        int s = 0;
        for (int i = 0; i < 16; i++) {
            const unsigned short ww = __ldg(wb + 1 + i);
            s += (int)(signed char)(ww & 0xFF) * __float2int_rn(__fmul_rn(__ldg(xb + 2 * i), mul));
            s += (int)(signed char)(ww >> 8) * __float2int_rn(__fmul_rn(__ldg(xb + 2 * i + 1), mul));
        }
        acc = fmaf((float)s, f16_bits_to_f32(__ldg(wb)) * ad, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc;
}

// Q8_0 weights times activations that are ALREADY Q8_0 blocks (the dispatcher and tile kernels of
// bench/bpd_gemm_q8_0_cpu.c:32-207 take them so): out[j * ldc + i] for weight row i (rows w_stride bytes
// apart) and activation row j (a_stride bytes apart).  The reference keeps, per output cell, eight fp32 lanes:
// lane q adds, block after block, (wd * ad) * (float)(sum of the four products of elements 4q..4q+3), multiply
// and add rounded separately; the lanes are then summed as (c_q + c_{q+4}), (s_0 + s_2, s_1 + s_3), t_0 + t_1
// (bench/bpd_gemm_q8_0_cpu.c:44-85).  Eight threads per cell play those lanes, in that order: the reference's
// AVX result bit for bit.  Rows are 2-byte aligned only.
__global__ void __launch_bounds__(256) k_qmatmul_q8_0_q8_0(const uint8_t* __restrict__ W, const uint8_t* __restrict__ Xq,
                                                           float* __restrict__ out, int m_weight, int m_tokens, int nbk,
                                                           long w_stride, long a_stride, int ldc)
{
    const long n_cells = (long)m_weight * m_tokens;
    const long n_items = (n_cells * 8 + 31) / 32 * 32;      // whole warps, so that the shuffles see all lanes
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long)gridDim.x * blockDim.x) {
        const long cell = it >> 3;
        const int q = (int)(it & 7);
        const bool live = cell < n_cells;
        const int j = live ? (int)(cell / m_weight) : 0, i = live ? (int)(cell - (long)j * m_weight) : 0;
        const uint8_t* wr = W + (size_t)i * w_stride;
        const uint8_t* ar = Xq + (size_t)j * a_stride;
        float c = 0.0f;
        if (live) {
            for (int b = 0; b < nbk; b++) {
                const unsigned short* wb = reinterpret_cast<const unsigned short*>(wr + (size_t)b * BPDQ_Q80_BYTES);
                const unsigned short* ab = reinterpret_cast<const unsigned short*>(ar + (size_t)b * BPDQ_Q80_BYTES);
                const uint32_t ww = __ldg(wb + 1 + 2 * q) | ((uint32_t)__ldg(wb + 2 + 2 * q) << 16);
                const uint32_t aa = __ldg(ab + 1 + 2 * q) | ((uint32_t)__ldg(ab + 2 + 2 * q) << 16);
                const float scale = __fmul_rn(f16_bits_to_f32(__ldg(wb)), f16_bits_to_f32(__ldg(ab)));
                c = __fadd_rn(__fmul_rn(scale, (float)dp4a_ss(ww, aa, 0)), c);
            }
        }
        c = __fadd_rn(c, __shfl_xor_sync(0xFFFFFFFFu, c, 4));
        c = __fadd_rn(c, __shfl_xor_sync(0xFFFFFFFFu, c, 2));
        c = __fadd_rn(c, __shfl_xor_sync(0xFFFFFFFFu, c, 1));
        if (live && q == 0) out[(size_t)j * ldc + i] = c;
    }
}

static int qmatmul_q8_0_q8_0(const uint8_t* W, const uint8_t* Xq, float* out, int m_weight, int m_tokens, int nbk, long w_stride,
                             long a_stride, int ldc, cudaStream_t s)
{
    if (m_weight < 0 || m_tokens < 0 || nbk <= 0 || ldc < m_weight || w_stride < 0 || a_stride < 0) return latch(BPDQ_ERR_ARG);
    if (m_weight == 0 || m_tokens == 0) return 0;
    if (!W || !Xq || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)W & 1) || ((uintptr_t)Xq & 1) || (w_stride & 1) || (a_stride & 1) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    const long want = ((long)m_weight * m_tokens * 8 + 255) / 256, cap = (long)sm_count() * 16;
    k_qmatmul_q8_0_q8_0<<<(unsigned)(want < cap ? want : cap), 256, 0, s>>>(W, Xq, out, m_weight, m_tokens, nbk, w_stride, a_stride, ldc);
    int rc = check_cuda(cudaGetLastError());
    return rc ? latch(rc) : 0;
}

static int grid_for(long items, int threads = 256)
{
    long want = (items + threads - 1) / threads, cap = (long)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

int bpd_qmatmul_q8_0_dispatch_cuda(const uint8_t* Wq, const uint8_t* Xq, float* out, int m_weight, int m_tokens, int K, void* stream);

int bpd_dequant_q8_0_cuda(const uint8_t* raw, float* out, size_t n_blocks, void* stream)
{
    if (n_blocks && (!raw || !out)) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)raw & 1) || ((uintptr_t)out & 15)) return latch(BPDQ_ERR_ALIGN);
    if (!n_blocks) return 0;
    k_dequant_q8_0<<<grid_for((long)n_blocks * 8), 256, 0, (cudaStream_t)stream>>>(raw, out, (long)n_blocks);
    return check_cuda(cudaGetLastError());
}

int bpd_quant_q8_0_cuda(const float* x, uint8_t* y, size_t n_elements, void* stream)
{
    if ((n_elements % 32) != 0 || (n_elements && (!x || !y))) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 1)) return latch(BPDQ_ERR_ALIGN);
    if (!n_elements) return 0;
    const long nb = (long)(n_elements / 32);
    k_quant_q8_0<<<grid_for(nb * 8), 256, 0, (cudaStream_t)stream>>>(x, y, nb);
    return check_cuda(cudaGetLastError());
}

int bpd_q8_0_block_dots_cuda(const uint8_t* w, const uint8_t* a, int32_t* dots, size_t n_blocks, void* stream)
{
    if (n_blocks && (!w || !a || !dots)) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)w & 1) || ((uintptr_t)a & 1)) return latch(BPDQ_ERR_ALIGN);
    if (!n_blocks) return 0;
    k_q8_0_block_dots<<<grid_for((long)n_blocks), 256, 0, (cudaStream_t)stream>>>(w, a, dots, (long)n_blocks);
    return check_cuda(cudaGetLastError());
}

// out[m*N + n] = W row n . q8_0(X row m), as bpd_qmatmul_q8_0_cpu(W, X, out, M, N, K).
int bpd_qmatmul_q8_0_cuda(const uint8_t* W, const float* X, float* out, int M, int N, int K, void* stream)
{
    if (M < 0 || N < 0 || K <= 0 || (K % 32) != 0) return latch(BPDQ_ERR_ARG);
    if (M == 0 || N == 0) return 0;
    if (!W || !X || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)W & 1) || ((uintptr_t)X & 3) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    cudaStream_t s = (cudaStream_t)stream;
    for (int m = 0; m < M; m++) {
        const float* x = X + (size_t)m * K;
        float* o = out + (size_t)m * N;
        int rc = gemv_q8_0_fast(W, x, o, N, K, s);
        if (rc == BPDQ_ERR_RANGE) {
            k_gemv_q8_0_generic<<<(N + 7) / 8, 256, 0, s>>>(W, x, o, N, K / 32);
            rc = check_cuda(cudaGetLastError());
        }
        if (rc) return latch(rc);
    }
    return 0;
}

int bpd_embed_lookup_q8_0_vocab_cuda(const uint8_t* table, const int32_t* ids, float* out, int n_tokens, int embed_dim,
                                     int vocab_size, void* stream)
{
    if (n_tokens < 0 || embed_dim <= 0 || (embed_dim % 32) != 0 || vocab_size < 1) return latch(BPDQ_ERR_ARG);
    if (n_tokens == 0) return 0;
    if (!table || !ids || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)table & 1) || ((uintptr_t)out & 15)) return latch(BPDQ_ERR_ALIGN);
    const long items = (long)n_tokens * (embed_dim / 4);
    k_embed_lookup_q8_0<<<grid_for(items), 256, 0, (cudaStream_t)stream>>>(table, ids, out, n_tokens, embed_dim / 32, vocab_size,
                                                                            device_error_flag());
    return check_cuda(cudaGetLastError());
}
// The reference's signature has no table size (bench/bpd_cpu.c:4002): only negative ids can be refused.
int bpd_embed_lookup_q8_0_cuda(const uint8_t* table, const int32_t* ids, float* out, int n_tokens, int embed_dim,
                               void* stream)
{
    return bpd_embed_lookup_q8_0_vocab_cuda(table, ids, out, n_tokens, embed_dim, 0x7FFFFFFF, stream);
}

// bench/bpd_cpu.c:4428-4459  bpd_qmatmul_q8_0_llamafile_cpu(W, X, out, m_weight, m_tokens, K): fp32 activations,
// out[token * m_weight + weight_row]
int bpd_qmatmul_q8_0_llamafile_cuda(const uint8_t* W, const float* X, float* out, int m_weight, int m_tokens, int K, void* stream)
{
    if (m_weight < 0 || m_tokens < 0 || K <= 0 || (K % 32) != 0) return latch(BPDQ_ERR_ARG);
    if (m_weight == 0 || m_tokens == 0) return 0;
    if (!W || !X || !out) return latch(BPDQ_ERR_ARG);
    // as the reference does: quantize the activation rows to Q8_0 (library-owned scratch of this stream), then the dispatcher
    const size_t row = (size_t)(K / 32) * BPDQ_Q80_BYTES;
    int rc = 0;
    uint8_t* xq = scratch_take(nullptr, kScratchQ80Acts, (size_t)m_tokens * row, (cudaStream_t)stream, &rc);
    if (!xq) return rc;
    if ((rc = bpd_quant_q8_0_cuda(X, xq, (size_t)m_tokens * K, stream))) return rc;
    return bpd_qmatmul_q8_0_dispatch_cuda(W, xq, out, m_weight, m_tokens, K, stream);
}
// bench/bpd_gemm_q8_0_cpu.c:159-207  bpd_qmatmul_q8_0_dispatch_cpu(Wq, Xq, out, m_weight, m_tokens, K): activations
// already quantized to Q8_0 rows [m_tokens][K/32][34]
int bpd_qmatmul_q8_0_dispatch_cuda(const uint8_t* Wq, const uint8_t* Xq, float* out, int m_weight, int m_tokens, int K, void* stream)
{
    if (K <= 0 || (K % 32) != 0) return latch(BPDQ_ERR_ARG);
    const long row = (long)(K / 32) * BPDQ_Q80_BYTES;
    return qmatmul_q8_0_q8_0(Wq, Xq, out, m_weight, m_tokens, K / 32, row, row, m_weight, (cudaStream_t)stream);
}
// bench/bpd_gemm_q8_0_cpu.c:32-157  bpd_gemm_q8_0_{RM}_{RN}_cpu(W_tile, B_tile, k, w_stride, a_stride, out, ldc): one
// tile of RM weight rows x RN activation rows over k blocks, out[j * ldc + i]
#define BPDQ_Q8_0_TILE(RM, RN)                                                                                                  \
    int bpd_gemm_q8_0_##RM##_##RN##_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride,       \
                                         float* out, int ldc, void* stream)                                                     \
    {                                                                                                                           \
        return qmatmul_q8_0_q8_0(W_tile, B_tile, out, RM, RN, k, w_stride, a_stride, ldc, (cudaStream_t)stream);               \
    }
BPDQ_Q8_0_TILE(1, 1) BPDQ_Q8_0_TILE(1, 2) BPDQ_Q8_0_TILE(1, 4)
BPDQ_Q8_0_TILE(2, 1) BPDQ_Q8_0_TILE(2, 2) BPDQ_Q8_0_TILE(2, 4)
BPDQ_Q8_0_TILE(4, 1) BPDQ_Q8_0_TILE(4, 2) BPDQ_Q8_0_TILE(4, 4)
#undef BPDQ_Q8_0_TILE

// gpu_vecmat-shaped: (activations, weights, out, k, n)  -- lib/kernel_templates_llama.pl:147-158
void gpu_vecmat_q8_0(const float* a, const uint8_t* wq, float* c, int k, int n)
{
    bpd_qmatmul_q8_0_cuda(wq, a, c, 1, n, k, (void*)current_stream());
}

}  // extern "C"

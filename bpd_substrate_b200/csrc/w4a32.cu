// Q4_K weights times fp32 activations (no activation quantization): the drop-in semantics of
// bpd_qmatmul_q4k_gpu / k_qmatmul_q4k (bench/bpd_quant_gpu.cu:90-154,166-169) and a device twin
// of bpd_qmm_q4k (bench/bpd_quant.c:114-137) of the reference.
//
// Every weight is dequantized exactly as bench/bpd_quant.c:64-71 does (one rounding:
// scale*q - min) and multiplied into an fp32 accumulator.  Accumulation order (the reference's
// CPU code sums strictly left to right, its GPU kernel per thread and then by a shared-memory
// tree; fp32 results of different orders agree to ~1e-6 norm-wise, not bit for bit):
//   one warp per weight row; lane l takes half-super-blocks l, l+32, ... in ascending order
//   and within one its 128 elements in ascending order, acc = fma(w, x, acc); lanes are then
//   added by a butterfly (xor 16, 8, 4, 2, 1).
//
// This path is bound by instruction issue (about six instructions per weight), not by HBM; the
// bandwidth-bound GEMV is the Q8_K-activation kernel in gemv_q4k.cu.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

// Nibble n (0..15) as a float without the conversion pipe: 2^23 + n has n in its low mantissa bits.
__device__ __forceinline__ float nibble_to_float(uint32_t n) { return __uint_as_float(0x4B000000u | n) - 8388608.0f; }

// COLS activations vectors at once: x(k, c) = xs[k * ldx + c * cstride]
template <int COLS>
__global__ void __launch_bounds__(256) k_w4a32(const uint8_t* __restrict__ W, const float* __restrict__ xs, long ldx,
                                               long cstride, float* __restrict__ out, long ldo, long ostride, int M,
                                               int nb)
{
    const int lane = threadIdx.x & 31;
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= M) return;
    const uint8_t* wr = W + (size_t)row * nb * BPDQ_Q4K_BYTES;
    float acc[COLS];
#pragma unroll
    for (int c = 0; c < COLS; c++) acc[c] = 0.0f;
    for (int hb = lane; hb < 2 * nb; hb += 32) {
        const uint8_t* blk = wr + (size_t)(hb >> 1) * BPDQ_Q4K_BYTES;
        const int half = hb & 1;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
        const float d = f16_bits_to_f32(hdr.x & 0xFFFFu), dmin = f16_bits_to_f32(hdr.x >> 16);
        uint32_t sc4, mn4;
        q4k_scales4(hdr.y, hdr.z, hdr.w, half, sc4, mn4);
        const uint4* qs = reinterpret_cast<const uint4*>(blk + 16 + 64 * half);
        const long k0 = (long)hb * 128;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint4 qv = __ldg(qs + j);
            const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
            const float scale = d * (float)byte_of(sc4, j);
            const float minv = dmin * (float)byte_of(mn4, j);
            // bytes 0..15 of the sub-block: low nibble = element k, high nibble = element k+16
#pragma unroll
            for (int b = 0; b < 16; b++) {
                const uint32_t byte = (qw[b >> 2] >> (8 * (b & 3))) & 0xFFu;
                const float wlo = fmaf(scale, nibble_to_float(byte & 15u), -minv);
                const float whi = fmaf(scale, nibble_to_float(byte >> 4), -minv);
                const long klo = k0 + 32 * j + b, khi = klo + 16;
#pragma unroll
                for (int c = 0; c < COLS; c++) {
                    acc[c] = fmaf(wlo, __ldg(xs + klo * ldx + c * cstride), acc[c]);
                    acc[c] = fmaf(whi, __ldg(xs + khi * ldx + c * cstride), acc[c]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < COLS; c++) {
        const float v = warp_sum(acc[c]);
        if (lane == 0) out[(long)row * ldo + c * ostride] = v;
    }
}

// GEMV fast path (contiguous x): a warp owns R consecutive rows; lane l takes half-super-blocks
// l, l+32, ...  The activations of a sub-block are loaded once and used by all R rows; a nibble
// becomes a float with one byte-permute (0x4B0000qq = 2^23 + q) and one subtraction.  Per
// sub-block the lane forms S1 = sum q*x and S0 = sum x, then acc += (d*sc)*S1 - (dmin*mn)*S0,
// half-blocks ascending; lanes are added by a butterfly (xor 16 .. 1).
template <int R>
__global__ void __launch_bounds__(256) k_w4a32_gemv(const uint8_t* __restrict__ W, const float* __restrict__ x,
                                                    float* __restrict__ out, int M, int nb)
{
    const int lane = threadIdx.x & 31;
    const int row0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * R;
    if (row0 >= M) return;
    const size_t row_bytes = (size_t)nb * BPDQ_Q4K_BYTES;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.0f;
    for (int hb = lane; hb < 2 * nb; hb += 32) {
        const int half = hb & 1;
        const uint8_t* blk0 = W + (size_t)row0 * row_bytes + (size_t)(hb >> 1) * BPDQ_Q4K_BYTES;
        uint4 hdr[R];
#pragma unroll
        for (int r = 0; r < R; r++)
            hdr[r] = (row0 + r < M) ? __ldg(reinterpret_cast<const uint4*>(blk0 + r * row_bytes)) : make_uint4(0, 0, 0, 0);
        const float4* xs = reinterpret_cast<const float4*>(x + (size_t)hb * 128);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float xv[32];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 v = __ldg(xs + 8 * j + i);
                xv[4 * i + 0] = v.x;
                xv[4 * i + 1] = v.y;
                xv[4 * i + 2] = v.z;
                xv[4 * i + 3] = v.w;
            }
            float s0 = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; i++) s0 += xv[i];
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (row0 + r >= M) continue;
                const uint4 qv = __ldg(reinterpret_cast<const uint4*>(blk0 + r * row_bytes + 16 + 64 * half) + j);
                const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
                float s1 = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const uint32_t lo = qw[w] & 0x0F0F0F0Fu, hi = (qw[w] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        // bytes {q, 0, 0, 0x4B}: selector picks byte b of the nibble word, then 0x4B000000's bytes
                        const uint32_t sel = 0x7440u | (uint32_t)b;
                        const float fl = __uint_as_float(__byte_perm(lo, 0x4B000000u, sel)) - 8388608.0f;
                        const float fh = __uint_as_float(__byte_perm(hi, 0x4B000000u, sel)) - 8388608.0f;
                        s1 = fmaf(fl, xv[4 * w + b], s1);
                        s1 = fmaf(fh, xv[16 + 4 * w + b], s1);
                    }
                }
                uint32_t sc4, mn4;
                q4k_scales4(hdr[r].y, hdr[r].z, hdr[r].w, half, sc4, mn4);
                const float d = f16_bits_to_f32(hdr[r].x & 0xFFFFu), dmin = f16_bits_to_f32(hdr[r].x >> 16);
                acc[r] = fmaf(d * (float)byte_of(sc4, j), s1, acc[r]);
                acc[r] = fmaf(-(dmin * (float)byte_of(mn4, j)), s0, acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && row0 + r < M) out[row0 + r] = v;
    }
}

// Generic driver: n_cols activation vectors; element (k, c) at xs[k*ldx + c*cstride]; result
// (row, c) at out[row*ldo + c*ostride].
static int w4a32(const uint8_t* W, const float* xs, long ldx, long cstride, float* out, long ldo, long ostride, int M,
                 int K, int n_cols, cudaStream_t s)
{
    if (M < 0 || n_cols < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (M == 0 || n_cols == 0) return 0;
    if (!W || !xs || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)W & 15) || ((uintptr_t)xs & 3) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    if (n_cols == 1 && ldx == 1 && !((uintptr_t)xs & 15)) {
        constexpr int R = 4;
        const int warps = (M + R - 1) / R;
        k_w4a32_gemv<R><<<(warps + 7) / 8, 256, 0, s>>>(W, xs, out, M, K / 256);
        return check_cuda(cudaGetLastError());
    }
    const int grid = (M + 7) / 8;
    for (int c0 = 0; c0 < n_cols; c0 += 4) {
        const int nc = n_cols - c0 < 4 ? n_cols - c0 : 4;
        const float* x0 = xs + c0 * cstride;
        float* o0 = out + c0 * ostride;
        switch (nc) {
            case 1: k_w4a32<1><<<grid, 256, 0, s>>>(W, x0, ldx, cstride, o0, ldo, ostride, M, K / 256); break;
            case 2: k_w4a32<2><<<grid, 256, 0, s>>>(W, x0, ldx, cstride, o0, ldo, ostride, M, K / 256); break;
            case 3: k_w4a32<3><<<grid, 256, 0, s>>>(W, x0, ldx, cstride, o0, ldo, ostride, M, K / 256); break;
            default: k_w4a32<4><<<grid, 256, 0, s>>>(W, x0, ldx, cstride, o0, ldo, ostride, M, K / 256); break;
        }
        int rc = check_cuda(cudaGetLastError());
        if (rc) return rc;
    }
    return 0;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

// bench/bpd_quant_gpu.cu:166-169: output[M] = dequant(qweight[M][K]) . x[K]
void bpd_qmatmul_q4k_gpu(const uint8_t* qweight, const float* x, float* output, int M, int K)
{
    w4a32(qweight, x, 1, 0, output, 1, 0, M, K, 1, current_stream());
}
int bpd_qmatmul_q4k_gpu_st(const uint8_t* qweight, const float* x, float* output, int M, int K, void* stream)
{
    return w4a32(qweight, x, 1, 0, output, 1, 0, M, K, 1, (cudaStream_t)stream);
}
// bench/bpd_quant.c:114-137 on device pointers: C[M][N] = dequant(qA[M][K]) @ B[K][N]
int bpd_qmm_q4k_cuda(const uint8_t* qA, const float* B, float* C, int M, int N, int K, void* stream)
{
    return w4a32(qA, B, N, 1, C, N, 1, M, K, N, (cudaStream_t)stream);
}

}  // extern "C"

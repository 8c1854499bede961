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
// The GEMV fast path (k_w4a32_ring) streams the weights through per-warp ring slots as the W4A8 kernels do
// and spends 2.5 instructions per weight; it is bound by instruction issue, not by HBM (the bandwidth-bound
// GEMV is the Q8_K-activation kernel).  Its accumulation order is described at the kernel.
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

// ---- GEMV fast path: weights through the shared-memory ring.
//
// Structure: one CTA per SM, nw warps, each with its own ring slots that it refills itself with 1-D bulk copies of
// tiles of R whole rows (gemv_batch.cu's scheme).  The activation vector sits in shared memory as fp32, every
// half-super-block's 128 floats padded to 132 so that the 16-byte reads of 32 lanes hit distinct banks, next to the
// sum of every sub-block's 32 activations (S0).
// Arithmetic per row: lane l takes half-super-blocks l, l + 32, ... in ascending order; per sub-block
//     S1' = sum_k (1 + q_k / 16) * x_k      (the nibble goes into the top mantissa bits of 1.0f with two bit
//                                            operations per four weights and one byte permute per weight: no
//                                            conversion, no subtraction per weight)
//     acc = fma(16 * d * sc, S1' - S0, acc);  acc = fma(-(dmin * mn), S0, acc)
// i.e. sum q*x = 16 (S1' - S0) with S0 summed once per launch; lanes are added by fold_rows' fixed butterfly.
// Against the reference's strictly sequential fp32 sum and against binary64 the result agrees to ~1e-6 norm-wise
// (the stated bar is 1e-5): the re-association costs about one more bit than the per-weight form.
constexpr int kW4XPad = 132;            // floats per half-super-block of x in shared memory

struct W4Plan {
    const uint8_t* W;
    const float* x;
    float* out;
    int M, nb, row_bytes, rt, n_tiles;
    int nw, slots, slot_bytes;
    int off_ring, off_x, off_s0, off_bar;
    size_t smem;
};

__device__ __forceinline__ float w4_fold(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

template <int R>
__device__ __forceinline__ void w4_tile(const uint8_t* tile, const float* xs, const float* s0s, const W4Plan& p, int row0, int lane)
{
    const int rows = min(R, p.M - row0);
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.0f;
    for (int hb = lane; hb < 2 * p.nb; hb += 32) {
        const int half = hb & 1;
        const uint8_t* blk0 = tile + (size_t)(hb >> 1) * BPDQ_Q4K_BYTES;
        const float4* xv4 = reinterpret_cast<const float4*>(xs + (size_t)hb * kW4XPad);
        const float4 s0v = *reinterpret_cast<const float4*>(s0s + 4 * hb);
        const float s0a[4] = {s0v.x, s0v.y, s0v.z, s0v.w};
        float dsc[R][4], dmn[R][4];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint4 hdr = *reinterpret_cast<const uint4*>(blk0 + (size_t)r * p.row_bytes);
            const float d16 = 16.0f * f16_bits_to_f32(hdr.x & 0xFFFFu), dmin = f16_bits_to_f32(hdr.x >> 16);
            uint32_t sc4, mn4;
            q4k_scales4(hdr.y, hdr.z, hdr.w, half, sc4, mn4);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                dsc[r][j] = d16 * (float)byte_of(sc4, j);
                dmn[r][j] = dmin * (float)byte_of(mn4, j);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float xv[32];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 v = xv4[8 * j + i];
                xv[4 * i + 0] = v.x;
                xv[4 * i + 1] = v.y;
                xv[4 * i + 2] = v.z;
                xv[4 * i + 3] = v.w;
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (r >= rows) continue;
                const uint4 qv = *reinterpret_cast<const uint4*>(blk0 + (size_t)r * p.row_bytes + 16 + 64 * half + 16 * j);
                const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
                float s1a = 0.0f, s1b = 0.0f;     // two chains: low-nibble and high-nibble elements
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    // byte = 0x80 | q << 3: with 0x3F on top, the float 1 + q / 16
                    const uint32_t lo = ((qw[w] << 3) & 0x78787878u) | 0x80808080u;
                    const uint32_t hi = ((qw[w] >> 1) & 0x78787878u) | 0x80808080u;
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        const uint32_t sel = 0x7044u | ((uint32_t)b << 8);
                        s1a = fmaf(__uint_as_float(__byte_perm(lo, 0x3F000000u, sel)), xv[4 * w + b], s1a);
                        s1b = fmaf(__uint_as_float(__byte_perm(hi, 0x3F000000u, sel)), xv[16 + 4 * w + b], s1b);
                    }
                }
                const float t = (s1a + s1b) - s0a[j];
                acc[r] = fmaf(dsc[r][j], t, acc[r]);
                acc[r] = fmaf(-dmn[r][j], s0a[j], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const float v = w4_fold(acc[r]);
        if (lane == 0 && r < rows) p.out[row0 + r] = v;
    }
}

__global__ void __launch_bounds__(352, 1) k_w4a32_ring(const W4Plan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;
    float* xs = reinterpret_cast<float*>(smem + p.off_x);        // [2 nb][132]
    float* s0s = reinterpret_cast<float*>(smem + p.off_s0);      // [8 nb]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < p.nw * p.slots; s++) mbar_init(&full[s], 1);
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();
    const int stride = p.nw * (int)gridDim.x;
    const int first = warp * (int)gridDim.x + (int)blockIdx.x;
    uint8_t* my_ring = ring + (size_t)warp * p.slots * p.slot_bytes;
    uint64_t* my_full = full + warp * p.slots;
    int lv = first;
    auto issue = [&](int slot) {
        const int row0 = lv * p.rt;
        const uint32_t bytes = (uint32_t)min(p.rt, p.M - row0) * p.row_bytes;
        if (lane == 0) {
            mbar_expect_tx(&my_full[slot], bytes);
            bulk_g2s(my_ring + (size_t)slot * p.slot_bytes, p.W + (size_t)row0 * p.row_bytes, bytes, &my_full[slot]);
        }
        lv += stride;
    };
    for (int k = 0; k < p.slots && lv < p.n_tiles; k++) issue(k);     // weights never depend on the launch before
    // the activation vector may come from the launch before: wait for it, then stage it (padded) and the sub-block sums
    pdl_wait();
    for (int sub = warp; sub < 8 * p.nb; sub += p.nw) {
        const float v = __ldcg(p.x + (size_t)sub * 32 + lane);
        xs[(size_t)(sub >> 2) * kW4XPad + 32 * (sub & 3) + lane] = v;
        // fixed order: butterfly over the 32 lanes
        const float s = w4_fold(v);
        if (lane == 0) s0s[sub] = s;
    }
    __syncthreads();
    int slot = 0;
    uint32_t parity = 0;
    for (int v = first; v < p.n_tiles; v += stride) {
        if (!mbar_wait_bounded(&my_full[slot], parity, err, 2)) return;
        const uint8_t* tile = my_ring + (size_t)slot * p.slot_bytes;
        const int row0 = v * p.rt;
        if (p.rt == 4) w4_tile<4>(tile, xs, s0s, p, row0, lane);
        else if (p.rt == 2) w4_tile<2>(tile, xs, s0s, p, row0, lane);
        else w4_tile<1>(tile, xs, s0s, p, row0, lane);
        __syncwarp();
        if (lv < p.n_tiles) issue(slot);
        if (++slot == p.slots) {
            slot = 0;
            parity ^= 1u;
        }
    }
}

// Plans and launches the ring kernel; BPDQ_ERR_RANGE when the shape does not fit it (the caller then uses the generic kernel).
static int w4a32_ring(const uint8_t* W, const float* x, float* out, int M, int K, cudaStream_t s)
{
    W4Plan p;
    p.W = W;
    p.x = x;
    p.out = out;
    p.M = M;
    p.nb = K / 256;
    p.row_bytes = p.nb * BPDQ_Q4K_BYTES;
    if (p.row_bytes > 32 * 1024) return BPDQ_ERR_RANGE;
    const int budget = 9216;
    p.rt = 4 * p.row_bytes <= budget ? 4 : (2 * p.row_bytes <= budget ? 2 : 1);
    p.slot_bytes = p.rt * p.row_bytes;
    p.n_tiles = (M + p.rt - 1) / p.rt;
    p.slots = 2;
    p.nw = 10;
    const size_t x_bytes = (size_t)2 * p.nb * kW4XPad * sizeof(float), s0_bytes = (size_t)8 * p.nb * sizeof(float);
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_x = take(x_bytes);
        p.off_s0 = take(s0_bytes);
        p.off_bar = take((size_t)p.nw * p.slots * 8);
        p.smem = off;
        if (p.smem <= (size_t)227 * 1024) break;
        if (p.nw > 4) p.nw--;
        else return BPDQ_ERR_RANGE;
    }
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(k_w4a32_ring, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    long want = ((long)p.n_tiles + p.nw - 1) / p.nw;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(want < 1 ? 1 : (want < sm_count() ? want : sm_count())));
    cfg.blockDim = dim3((unsigned)p.nw * 32);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, k_w4a32_ring, p, device_error_flag()));
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
        int rc = w4a32_ring(W, xs, out, M, K, s);
        if (rc != BPDQ_ERR_RANGE) return rc;
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

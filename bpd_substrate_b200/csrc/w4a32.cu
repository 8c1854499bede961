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
// The GEMV fast path (k_w4a32_ring) streams the weights through per-warp ring slots as the W4A8 kernels do and
// multiplies them with a 24-bit block-fixed-point copy of the activations, exactly, by integer dot products; its
// arithmetic and accumulation order are described at the kernel.  The generic kernels below (several activation
// vectors, strided activations) multiply in fp32, weight by weight.
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

// ---- GEMV fast path: weights through the shared-memory ring, activations as 24-bit block fixed point.
//
// Structure: one CTA per SM, nw warps, each with its own ring slots that it refills itself with 1-D bulk copies of
// tiles of R whole rows (gemv_batch.cu's scheme).
//
// Arithmetic.  Multiplying every 4-bit weight with an fp32 activation costs a conversion and an FMA per weight, which
// is more than HBM leaves time for.  Instead every CTA first rewrites the activation vector, per sub-block of 32, as
//     x_k = s * X_k,   s = amax / (2^23 - 256),   X_k = rint(x_k / s)  (a 24-bit signed integer),
// split into three byte planes X = 65536 H + 256 M + L (H signed, M and L unsigned), and keeps S0 = sum x_k per
// sub-block in fp32.  The products are then exact integer dot products of the nibbles with the three planes (dp4a:
// 24 per 32 weights), joined as D = 65536 D_H + 256 D_M + D_L in fp32, and per sub-block
//     acc = fma((d * sc) * s, D, acc);   acc = fma(-(dmin * mn), S0, acc),
// lane l taking half-super-blocks l, l + 32, ... in ascending order, lanes added by a fixed butterfly.
// The only approximation is the rounding of x_k to 24 bits relative to its sub-block's largest element (fp32 itself
// carries 24 bits per element): against binary64 the result is closer than the reference's own sequential fp32 sum,
// norm-wise about 1e-7 (the stated bar is 1e-5).  Inputs must be finite.
constexpr int kW4RecBytes = 432;        // per half-super-block: three planes of 128 bytes, four scales, four sums, 16 spare
constexpr float kW4Range = 8388352.0f;  // 2^23 - 256: rint(x * range / amax) stays below 2^23 whatever the roundings

struct W4Plan {
    const uint8_t* W;
    const float* x;
    float* out;
    int M, nb, row_bytes, rt, n_tiles;
    int nw, slots, slot_bytes;
    int off_ring, off_x, off_bar;
    size_t smem;
};

__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 256 activations held by a warp (lane l: elements 4l..4l+3 in v0, 128 + 4l.. in v1) -> the two records of the block
__device__ __forceinline__ void w4_write_records(const float4& v0, const float4& v1, uint8_t* rec0, int lane)
{
    const float4 v[2] = {v0, v1};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint8_t* rec = rec0 + h * kW4RecBytes;
        float amax = fmaxf(fmaxf(fabsf(v[h].x), fabsf(v[h].y)), fmaxf(fabsf(v[h].z), fabsf(v[h].w)));
        float s0 = (v[h].x + v[h].y) + (v[h].z + v[h].w);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {            // eight lanes = one sub-block
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, o);
        }
        const float scale = __fdiv_rn(amax, kW4Range);
        const float inv = amax != 0.0f ? __fdiv_rn(kW4Range, amax) : 0.0f;
        const int q0 = __float2int_rn(v[h].x * inv), q1 = __float2int_rn(v[h].y * inv), q2 = __float2int_rn(v[h].z * inv),
                  q3 = __float2int_rn(v[h].w * inv);
        // byte b of the four integers -> one word per plane
        const uint32_t a01 = __byte_perm((uint32_t)q0, (uint32_t)q1, 0x5140), a23 = __byte_perm((uint32_t)q2, (uint32_t)q3, 0x5140);   // L M L M
        const uint32_t b01 = __byte_perm((uint32_t)q0, (uint32_t)q1, 0x6262), b23 = __byte_perm((uint32_t)q2, (uint32_t)q3, 0x6262);   // H H (bytes 0, 1)
        const uint32_t pl = __byte_perm(a01, a23, 0x5410), pm = __byte_perm(a01, a23, 0x7632), ph = __byte_perm(b01, b23, 0x5410);
        const int w = lane & 31;                      // word index inside the 128-byte plane = lane (elements 4 lane ..)
        reinterpret_cast<uint32_t*>(rec)[w] = ph;
        reinterpret_cast<uint32_t*>(rec + 128)[w] = pm;
        reinterpret_cast<uint32_t*>(rec + 256)[w] = pl;
        if ((lane & 7) == 0) {
            reinterpret_cast<float*>(rec + 384)[lane >> 3] = scale;
            reinterpret_cast<float*>(rec + 400)[lane >> 3] = s0;
        }
    }
}

template <int R>
__device__ __forceinline__ void w4_tile(const uint8_t* tile, const uint8_t* xs, const W4Plan& p, int row0, int lane)
{
    const int rows = min(R, p.M - row0);
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.0f;
    for (int hb = lane; hb < 2 * p.nb; hb += 32) {
        const int half = hb & 1;
        const uint8_t* blk0 = tile + (size_t)(hb >> 1) * BPDQ_Q4K_BYTES;
        const uint8_t* rec = xs + (size_t)hb * kW4RecBytes;
        const float4 sc4f = *reinterpret_cast<const float4*>(rec + 384);
        const float4 s04f = *reinterpret_cast<const float4*>(rec + 400);
        const float xs_scale[4] = {sc4f.x, sc4f.y, sc4f.z, sc4f.w}, xs_s0[4] = {s04f.x, s04f.y, s04f.z, s04f.w};
        float dd[R], dm[R];
        uint32_t sc4[R], mn4[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint4 hdr = *reinterpret_cast<const uint4*>(blk0 + (size_t)r * p.row_bytes);
            dd[r] = f16_bits_to_f32(hdr.x & 0xFFFFu);
            dm[r] = f16_bits_to_f32(hdr.x >> 16);
            q4k_scales4(hdr.y, hdr.z, hdr.w, half, sc4[r], mn4[r]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // the sub-block's 32 activations as three byte planes: words 0..3 = elements 0..15, 4..7 = 16..31
            uint32_t pl[3][8];
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const uint4 a = *reinterpret_cast<const uint4*>(rec + 128 * k + 32 * j);
                const uint4 b = *reinterpret_cast<const uint4*>(rec + 128 * k + 32 * j + 16);
                pl[k][0] = a.x; pl[k][1] = a.y; pl[k][2] = a.z; pl[k][3] = a.w;
                pl[k][4] = b.x; pl[k][5] = b.y; pl[k][6] = b.z; pl[k][7] = b.w;
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (r >= rows) continue;
                const uint4 qv = *reinterpret_cast<const uint4*>(blk0 + (size_t)r * p.row_bytes + 16 + 64 * half + 16 * j);
                const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
                int lo[3] = {0, 0, 0}, hi[3] = {0, 0, 0};
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const uint32_t ql = qw[w] & 0x0F0F0F0Fu, qh = qw[w] & 0xF0F0F0F0u;     // hi: 16 x the nibble
                    lo[0] = dp4a_us(ql, pl[0][w], lo[0]);
                    hi[0] = dp4a_us(qh, pl[0][4 + w], hi[0]);
                    lo[1] = dp4a_uu(ql, pl[1][w], lo[1]);
                    hi[1] = dp4a_uu(qh, pl[1][4 + w], hi[1]);
                    lo[2] = dp4a_uu(ql, pl[2][w], lo[2]);
                    hi[2] = dp4a_uu(qh, pl[2][4 + w], hi[2]);
                }
                // exact integers: hi[] are multiples of 16
                const float dH = (float)(lo[0] + (hi[0] >> 4)), dM = (float)(lo[1] + (int)((unsigned)hi[1] >> 4)),
                            dL = (float)(lo[2] + (int)((unsigned)hi[2] >> 4));
                const float D = fmaf(65536.0f, dH, fmaf(256.0f, dM, dL));
                acc[r] = fmaf((dd[r] * (float)byte_of(sc4[r], j)) * xs_scale[j], D, acc[r]);
                acc[r] = fmaf(-(dm[r] * (float)byte_of(mn4[r], j)), xs_s0[j], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        float v = acc[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (lane == 0 && r < rows) p.out[row0 + r] = v;
    }
}

__global__ void __launch_bounds__(352, 1) k_w4a32_ring(const W4Plan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;
    uint8_t* xs = smem + p.off_x;                                // [2 nb][432]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int b = tid; b < p.nw * p.slots; b += blockDim.x) {     // the barriers are set up by as many threads
        mbar_init(&full[b], 1);
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
    // the activation vector may come from the launch before: wait for it, then every CTA makes its own fixed-point copy
    pdl_wait();
    for (int b0 = warp; b0 < p.nb; b0 += 4 * p.nw) {      // four blocks' loads in flight per warp
        float4 v[4][2];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int b = b0 + i * p.nw;
            if (b < p.nb) {
                const float4* xb = reinterpret_cast<const float4*>(p.x + (size_t)b * 256);
                v[i][0] = __ldcg(xb + lane);
                v[i][1] = __ldcg(xb + 32 + lane);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int b = b0 + i * p.nw;
            if (b < p.nb) w4_write_records(v[i][0], v[i][1], xs + (size_t)(2 * b) * kW4RecBytes, lane);
        }
    }
    __syncthreads();
    int slot = 0;
    uint32_t parity = 0;
    for (int v = first; v < p.n_tiles; v += stride) {
        if (!mbar_wait_bounded(&my_full[slot], parity, err, 2)) return;
        const uint8_t* tile = my_ring + (size_t)slot * p.slot_bytes;
        const int row0 = v * p.rt;
        if (p.rt == 4) w4_tile<4>(tile, xs, p, row0, lane);
        else if (p.rt == 2) w4_tile<2>(tile, xs, p, row0, lane);
        else w4_tile<1>(tile, xs, p, row0, lane);
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
    const size_t x_bytes = (size_t)2 * p.nb * kW4RecBytes;
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_x = take(x_bytes);
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

// Q4_K weights x Q8_K activations: decode GEMV (1 token) and small-batch GEMM (2..4 tokens
// per pass), with the activations quantized to Q8_K inside the kernel.
//
// The reference has no Q4_K x Q8_K kernel (docs/llama-kernel-audit.md:65 lists it as an
// unbuilt design); its Q4_K GEMV is the dequantize-to-fp32 kernel k_qmatmul_q4k
// (bench/bpd_quant_gpu.cu:90-154), which this file's bpd_qmatmul_q4k_q8k_* entry points
// stand beside.  The arithmetic is this library's own definition, built from the
// reference's Q8_0 quantizer (bench/bpd_cpu.c:4106-4136) and scalar block dot
// (bench/bpd_cpu.c:4263-4280):
//
//   Q8_K block (292 B / 256 activations): float d = amax/127; int8 qs[256] =
//   round-half-even(x * (127/amax)); int16 bsums[16] (sums of 16 consecutive qs).
//   Per weight row and super-block b:
//       isum = sum_j sc_j * (sum over sub-block j of nibble * qs)          (int32, exact)
//       msum = sum_j mn_j * (sum over sub-block j of qs)                   (int32, exact)
//       term = (d*dA) * float(isum) - (dmin*dA) * float(msum)
//   out[row] = sum_b term.
//
// Accumulation order on the GPU (documented because fp32 addition is not associative):
//   lane l of the warp that owns K-chunk c (4096 consecutive K) owns half-super-block
//   hb = 32c + l (sub-blocks 4(hb&1) .. +3 of super-block hb>>1) and computes
//       acc = fma(d*dA, float(isum_half), 0); acc = fma(-(dmin*dA), float(msum_half), acc)
//   the 32 lanes are combined by a butterfly (xor 16, 8, 4, 2, 1), and the K-chunks of a row
//   are added in ascending order starting from chunk 0.
//
// Data movement: the rows a CTA owns are one contiguous byte span (row stride K/256*144 B,
// no padding), so a tile of R rows is fetched with ONE 1-D bulk asynchronous copy
// (cp.async.bulk, completion on an mbarrier) into a ring of shared-memory slots by a
// producer warp; consumer warps unpack from shared memory.  The quantized activations live
// in registers for the whole kernel (32 words per lane per token), so the inner loop reads
// only weights from shared memory.  Bytes per weight row: K/256*144 read once from HBM.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

constexpr int kMaxTokens = 4;       // tokens per pass (activation registers: 32 words each)
constexpr int kXqStride = 144;      // 128 int8 + 16 B pad per half-super-block: conflict-free 16 B reads

struct GemvPlan {
    int nb;          // super-blocks per row
    int row_bytes;   // nb * 144
    int kc;          // K-chunks (warps) per row, ceil(nb / 16)
    int rw;          // row-warps: rows processed concurrently inside a tile
    int nw;          // consumer warps = kc * rw
    int rt;          // rows per tile (multiple of rw)
    int stages;
    int n_tiles;
    int grid;
    size_t smem;
    // smem offsets
    int off_ring, off_xq, off_xd, off_part, off_bar;
};

// ---------------------------------------------------------------- activation quantizer (device)

// Quantize one 256-float block with a warp (rule of bench/bpd_cpu.c:4106-4136, fp32 scale).
// Lane l holds elements 4l..4l+3 (v0) and 128+4l..128+4l+3 (v1).  Returns the two packed
// int8 words and the block scale d (same value in every lane).
__device__ __forceinline__ void quantize_block_256(const float4& v0, const float4& v1, uint32_t& p0, uint32_t& p1,
                                                   float& d)
{
    float amax = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w)));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    amax = warp_max(amax);
    d = __fdiv_rn(amax, 127.0f);
    const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
    auto q = [mul](float x) -> uint32_t { return (uint32_t)__float2int_rn(__fmul_rn(x, mul)) & 0xFFu; };
    p0 = q(v0.x) | (q(v0.y) << 8) | (q(v0.z) << 16) | (q(v0.w) << 24);
    p1 = q(v1.x) | (q(v1.y) << 8) | (q(v1.z) << 16) | (q(v1.w) << 24);
}

// Standalone quantizer to the 292-byte Q8_K block format: one warp per block.
__global__ void __launch_bounds__(256) k_quant_q8_K(const float* __restrict__ x, uint8_t* __restrict__ y,
                                                    long n_blocks)
{
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
    for (long b = warp; b < n_blocks; b += n_warps) {
        const float4* xb = reinterpret_cast<const float4*>(x + b * 256);
        const float4 v0 = __ldg(xb + lane), v1 = __ldg(xb + 32 + lane);
        uint32_t p0, p1;
        float d;
        quantize_block_256(v0, v1, p0, p1, d);
        uint8_t* yb = y + b * BPDQ_Q8K_BYTES;          // 292 = 4*73: word aligned
        uint32_t* yw = reinterpret_cast<uint32_t*>(yb);
        if (lane == 0) yw[0] = __float_as_uint(d);
        yw[1 + lane] = p0;
        yw[33 + lane] = p1;
        // bsums: 16 values = 4 lanes each; groups 0..7 from p0, 8..15 from p1
        int s0 = dp4a_ss(p0, 0x01010101u, 0), s1 = dp4a_ss(p1, 0x01010101u, 0);
        s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 1);
        s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 2);
        s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 1);
        s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 2);
        // pack two int16 per word: lanes 0,8,16,24 write words for group pairs
        const int g = lane >> 2;  // group index within each half
        const int s0n = __shfl_down_sync(0xFFFFFFFFu, s0, 4), s1n = __shfl_down_sync(0xFFFFFFFFu, s1, 4);
        if ((lane & 7) == 0) {
            yw[65 + (g >> 1)] = ((uint32_t)s0 & 0xFFFFu) | ((uint32_t)s0n << 16);
            yw[69 + (g >> 1)] = ((uint32_t)s1 & 0xFFFFu) | ((uint32_t)s1n << 16);
        }
    }
}

// ---------------------------------------------------------------- inner product of one half-super-block

// sbp: shared-memory super-block (144 B).  half: which four sub-blocks.  xr[t]: this lane's
// 128 quantized activations of token t, bs[t][j]: their per-sub-block sums, xd[t]: the Q8_K
// block scale.  dbg: optional global int32[8] slot of this (row, super-block) for the exact
// sub-block dots of token 0.
template <int T, int LAYOUT>
__device__ __forceinline__ void half_block_fma(const uint8_t* sbp, int half, const uint32_t (&xr)[T][32],
                                               const int (&bs)[T][4], const float (&xd)[T], float (&acc)[T],
                                               int32_t* dbg)
{
    const uint4 hdr = *reinterpret_cast<const uint4*>(sbp);
    const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
    const float dmin = f16_bits_to_f32(hdr.x >> 16);
    uint32_t sc4, mn4;
    q4k_scales4(hdr.y, hdr.z, hdr.w, half, sc4, mn4);
    const uint4* qs = reinterpret_cast<const uint4*>(sbp + 16 + 64 * half);

    int isum[T];
#pragma unroll
    for (int t = 0; t < T; t++) isum[t] = 0;

    if (LAYOUT == BPDQ_LAYOUT_BPD) {
        // uint4 i = sub-block i of this half: low nibbles <-> x[32i .. 32i+15], high <-> x[32i+16 .. 32i+31]
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 qv = qs[i];
            const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
            const int sc = (int)byte_of(sc4, i);
#pragma unroll
            for (int t = 0; t < T; t++) {
                int lo = 0, hi = 0;
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    lo = dp4a_us(qw[w] & 0x0F0F0F0Fu, xr[t][8 * i + w], lo);
                    hi = dp4a_us(qw[w] & 0xF0F0F0F0u, xr[t][8 * i + 4 + w], hi);  // 16 x the high-nibble dot
                }
                const int dot = lo + (hi >> 4);  // exact: hi is a multiple of 16
                isum[t] += sc * dot;
                if (dbg && t == 0) dbg[4 * half + i] = dot;
            }
        }
    } else {
        // ggml order: 32 bytes (two uint4) = sub-block 2c (low nibbles) and sub-block 2c+1 (high nibbles)
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint4 qa = qs[2 * c], qb = qs[2 * c + 1];
            const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const int sc_lo = (int)byte_of(sc4, 2 * c), sc_hi = (int)byte_of(sc4, 2 * c + 1);
#pragma unroll
            for (int t = 0; t < T; t++) {
                int lo = 0, hi = 0;
#pragma unroll
                for (int w = 0; w < 8; w++) {
                    lo = dp4a_us(qw[w] & 0x0F0F0F0Fu, xr[t][16 * c + w], lo);
                    hi = dp4a_us(qw[w] & 0xF0F0F0F0u, xr[t][16 * c + 8 + w], hi);
                }
                hi >>= 4;
                isum[t] += sc_lo * lo + sc_hi * hi;
                if (dbg && t == 0) {
                    dbg[4 * half + 2 * c] = lo;
                    dbg[4 * half + 2 * c + 1] = hi;
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < T; t++) {
        int msum = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) msum += (int)byte_of(mn4, j) * bs[t][j];
        acc[t] = fmaf(d * xd[t], (float)isum[t], acc[t]);
        acc[t] = fmaf(-(dmin * xd[t]), (float)msum, acc[t]);
    }
}

// ---------------------------------------------------------------- the GEMV / small-batch GEMM kernel

// XSRC: 0 = x is fp32 [T][K], quantized here; 1 = x is Q8_K blocks [T][K/256][292].
// MAXTHREADS bounds the CTA size (and so the registers the compiler may use per thread).
template <int T, int LAYOUT, int XSRC, int MAXTHREADS>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_gemv_q4k_q8k(const uint8_t* __restrict__ W, const void* __restrict__ xin, float* __restrict__ out, int M, int K,
               GemvPlan p, int* __restrict__ err, int32_t* __restrict__ dbg)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;
    uint8_t* xq = smem + p.off_xq;                               // [T][n_hb][144]
    float* xds = reinterpret_cast<float*>(smem + p.off_xd);      // [T][nb]
    float* part = reinterpret_cast<float*>(smem + p.off_part);   // [2][rt][kc][T]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);
    uint64_t* empty = full + p.stages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + p.stages);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_threads = blockDim.x;
    const bool is_producer = (warp == p.nw);
    const int n_hb = 2 * p.nb;
    const uint32_t tile_bytes_full = (uint32_t)p.rt * p.row_bytes;

    if (tid == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.nw);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // Tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int my_tiles = (p.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    // Let the next kernel in the stream start its own weight prefetch as early as possible.
    pdl_launch_dependents();

    // Producer: start the first ring fills before anything else so HBM latency overlaps the
    // activation quantization below.  Weights never depend on the previous kernel.
    int issued = 0;
    if (is_producer && lane == 0) {
        for (; issued < my_tiles && issued < p.stages; issued++) {
            const int tile = blockIdx.x + issued * gridDim.x;
            const int row0 = tile * p.rt;
            const int rows = min(p.rt, M - row0);
            const uint32_t bytes = (uint32_t)rows * p.row_bytes;
            mbar_expect_tx(&full[issued], bytes);
            bulk_g2s(ring + (size_t)issued * tile_bytes_full, W + (size_t)row0 * p.row_bytes, bytes, &full[issued]);
        }
    }

    // Activations may be produced by the previous kernel: wait for it here.
    pdl_wait();

    // ---- stage the quantized activations in shared memory (padded half-block layout)
    if (XSRC == 0) {
        const float* x = reinterpret_cast<const float*>(xin);
        const int n_warps = n_threads >> 5;
        for (int blk = warp; blk < T * p.nb; blk += n_warps) {
            const int t = blk / p.nb, b = blk - t * p.nb;
            const float4* xb = reinterpret_cast<const float4*>(x + (size_t)t * K + (size_t)b * 256);
            const float4 v0 = __ldg(xb + lane), v1 = __ldg(xb + 32 + lane);
            uint32_t p0, p1;
            float d;
            quantize_block_256(v0, v1, p0, p1, d);
            uint8_t* dst = xq + ((size_t)t * n_hb + 2 * b) * kXqStride;
            reinterpret_cast<uint32_t*>(dst)[lane] = p0;
            reinterpret_cast<uint32_t*>(dst + kXqStride)[lane] = p1;
            if (lane == 0) xds[t * p.nb + b] = d;
        }
    } else {
        const uint8_t* xb = reinterpret_cast<const uint8_t*>(xin);
        for (int i = tid; i < T * p.nb * 64; i += n_threads) {
            const int blk = i >> 6, w = i & 63;  // word w of the 64 qs words of block blk = t*nb + b
            const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(xb + (size_t)blk * BPDQ_Q8K_BYTES + 4) + w);
            uint8_t* dst = xq + ((size_t)2 * blk + (w >> 5)) * kXqStride;  // half-block index t*n_hb + 2b + (w>>5)
            reinterpret_cast<uint32_t*>(dst)[w & 31] = v;
        }
        for (int i = tid; i < T * p.nb; i += n_threads)
            xds[i] = __uint_as_float(__ldg(reinterpret_cast<const uint32_t*>(xb + (size_t)i * BPDQ_Q8K_BYTES)));
    }
    __syncthreads();

    if (is_producer) {
        // ---- producer warp: keep the ring full
        if (lane == 0) {
            for (int it = issued; it < my_tiles; it++) {
                const int s = it % p.stages;
                const uint32_t parity = ((it / p.stages) - 1) & 1;
                if (!mbar_wait_bounded(&empty[s], parity, err, 1)) break;
                const int tile = blockIdx.x + it * gridDim.x;
                const int row0 = tile * p.rt;
                const int rows = min(p.rt, M - row0);
                const uint32_t bytes = (uint32_t)rows * p.row_bytes;
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(ring + (size_t)s * tile_bytes_full, W + (size_t)row0 * p.row_bytes, bytes, &full[s]);
            }
        }
        return;
    }

    // ---- consumer warps
    const int kc = warp % p.kc;     // K-chunk of this warp (fixed for the whole kernel)
    const int rwi = warp / p.kc;    // row-warp index
    const int hb = 32 * kc + lane;  // half-super-block of this lane
    const bool active = hb < n_hb;
    const int sb = hb >> 1, half = hb & 1;

    uint32_t xr[T][32];
    int bs[T][4];
    float xd[T];
#pragma unroll
    for (int t = 0; t < T; t++) {
        if (active) {
            const uint4* src = reinterpret_cast<const uint4*>(xq + ((size_t)t * n_hb + hb) * kXqStride);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint4 v = src[i];
                xr[t][4 * i + 0] = v.x;
                xr[t][4 * i + 1] = v.y;
                xr[t][4 * i + 2] = v.z;
                xr[t][4 * i + 3] = v.w;
            }
            xd[t] = xds[t * p.nb + sb];
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++) xr[t][i] = 0;
            xd[t] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < 8; w++) s = dp4a_ss(xr[t][8 * j + w], 0x01010101u, s);
            bs[t][j] = s;
        }
    }

    const int n_consumer_threads = p.nw * 32;
    for (int it = 0; it < my_tiles; it++) {
        const int s = it % p.stages;
        const uint32_t parity = (it / p.stages) & 1;
        const int tile = blockIdx.x + it * gridDim.x;
        const int row0 = tile * p.rt;
        const int rows = min(p.rt, M - row0);
        const bool ok = mbar_wait_bounded(&full[s], parity, err, 2);
        if (!ok) *abort_flag = 1;
        const uint8_t* tile_smem = ring + (size_t)s * tile_bytes_full;
        float* part_it = part + (size_t)(it & 1) * p.rt * p.kc * T;

        if (ok) {
            for (int r = rwi; r < rows; r += p.rw) {
                float acc[T];
#pragma unroll
                for (int t = 0; t < T; t++) acc[t] = 0.0f;
                if (active) {
                    int32_t* d = dbg ? dbg + ((size_t)(row0 + r) * p.nb + sb) * 8 : nullptr;
                    half_block_fma<T, LAYOUT>(tile_smem + (size_t)r * p.row_bytes + (size_t)sb * BPDQ_Q4K_BYTES, half,
                                              xr, bs, xd, acc, d);
                }
#pragma unroll
                for (int t = 0; t < T; t++) acc[t] = warp_sum(acc[t]);
                if (lane == 0) {
                    if (p.kc == 1) {
#pragma unroll
                        for (int t = 0; t < T; t++) out[(size_t)t * M + row0 + r] = acc[t];
                    } else {
#pragma unroll
                        for (int t = 0; t < T; t++) part_it[((size_t)r * p.kc + kc) * T + t] = acc[t];
                    }
                }
            }
        }
        // this warp no longer reads the slot
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

        if (p.kc > 1) {
            // K-chunks of a row live in different warps: combine them in ascending chunk order.
            named_bar_sync(1, n_consumer_threads);
            if (*abort_flag) return;  // every consumer warp sees the same value after the barrier
            for (int i = tid; i < rows * T; i += n_consumer_threads) {
                const int r = i / T, t = i - r * T;
                float v = part_it[((size_t)r * p.kc + 0) * T + t];
                for (int c = 1; c < p.kc; c++) v += part_it[((size_t)r * p.kc + c) * T + t];
                out[(size_t)t * M + row0 + r] = v;
            }
        } else if (!ok) {
            return;
        }
    }
}

// ---------------------------------------------------------------- host side

constexpr int kSmemLimit = 227 * 1024;
constexpr int kSmallCtaThreads = 320;   // up to 9 consumer warps + the producer: K <= 36864

// consumer warps for rows of K weights: kc warps cover a row, rw rows run side by side
static int consumer_warps(int K)
{
    const int kc = (K / 256 + 15) / 16;
    return kc * (kc >= 8 ? 1 : 8 / kc);
}

static size_t plan_smem(GemvPlan& p, int T)
{
    size_t off = 0;
    auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
    p.off_ring = take((size_t)p.stages * p.rt * p.row_bytes);
    p.off_xq = take((size_t)T * 2 * p.nb * kXqStride);
    p.off_xd = take((size_t)T * p.nb * 4);
    p.off_part = take((size_t)2 * p.rt * p.kc * T * 4);
    p.off_bar = take((size_t)2 * p.stages * 8 + 8);
    return off;
}

static int make_plan(int M, int K, int T, GemvPlan& p)
{
    if (M < 0 || K <= 0 || (K % 256) != 0 || T < 1 || T > kMaxTokens) return BPDQ_ERR_ARG;
    const Tuning& tu = tuning();
    p.nb = K / 256;
    p.row_bytes = p.nb * BPDQ_Q4K_BYTES;
    p.kc = (p.nb + 15) / 16;
    if (p.kc > 31) return BPDQ_ERR_RANGE;  // K > 126976: one warp per 4096 K, 31 consumer warps at most
    p.rw = p.kc >= 8 ? 1 : (8 / p.kc);
    p.nw = p.kc * p.rw;
    int rows_per_warp = tu.tile_bytes / (p.rw * p.row_bytes);
    if (rows_per_warp < 1) rows_per_warp = 1;
    p.rt = p.rw * rows_per_warp;
    // small matrices: shrink tiles until every SM has at least one
    while (p.rt > p.rw && (long)((M + p.rt - 1) / p.rt) < (long)sm_count()) p.rt -= p.rw;
    p.n_tiles = (M + p.rt - 1) / p.rt;
    p.stages = tu.stages < 2 ? 2 : tu.stages;
    p.smem = plan_smem(p, T);
    while (p.smem > (size_t)kSmemLimit && p.stages > 2) {
        p.stages--;
        p.smem = plan_smem(p, T);
    }
    if (p.smem > (size_t)kSmemLimit) return BPDQ_ERR_RANGE;
    const int threads = (p.nw + 1) * 32;
    int per_sm = kSmemLimit / (int)p.smem;
    if (per_sm > 2048 / threads) per_sm = 2048 / threads;
    if (per_sm > tu.ctas_per_sm) per_sm = tu.ctas_per_sm;
    if (per_sm < 1) per_sm = 1;
    const long cap = (long)sm_count() * per_sm;
    p.grid = (int)(p.n_tiles < cap ? p.n_tiles : cap);
    if (p.grid < 1) p.grid = 1;
    return 0;
}

template <int T, int LAYOUT, int XSRC, int MAXTHREADS>
static int launch_one(const uint8_t* W, const void* x, float* out, int M, int K, const GemvPlan& p, int32_t* dbg,
                      cudaStream_t s)
{
    auto kern = k_gemv_q4k_q8k<T, LAYOUT, XSRC, MAXTHREADS>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3((p.nw + 1) * 32);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, W, x, out, M, K, p, device_error_flag(), dbg));
}

template <int LAYOUT, int XSRC>
static int launch_T(int T, const uint8_t* W, const void* x, float* out, int M, int K, const GemvPlan& p, int32_t* dbg,
                    cudaStream_t s)
{
    if ((p.nw + 1) * 32 > kSmallCtaThreads) {
        // very long rows: many warps per row, one token per pass
        if (T != 1) return BPDQ_ERR_ARG;
        return launch_one<1, LAYOUT, XSRC, 1024>(W, x, out, M, K, p, dbg, s);
    }
    switch (T) {
        case 1: return launch_one<1, LAYOUT, XSRC, kSmallCtaThreads>(W, x, out, M, K, p, dbg, s);
        case 2: return launch_one<2, LAYOUT, XSRC, kSmallCtaThreads>(W, x, out, M, K, p, dbg, s);
        case 3: return launch_one<3, LAYOUT, XSRC, kSmallCtaThreads>(W, x, out, M, K, p, dbg, s);
        case 4: return launch_one<4, LAYOUT, XSRC, kSmallCtaThreads>(W, x, out, M, K, p, dbg, s);
    }
    return BPDQ_ERR_ARG;
}

// out is [tokens][M]; x is fp32 [tokens][K] (xsrc 0) or Q8_K blocks [tokens][K/256] (xsrc 1).
// More than kMaxTokens tokens run as several passes over the weights.
int gemm_q4k_q8k(const uint8_t* W, const void* x, float* out, int tokens, int M, int K, int layout, int xsrc,
                 int32_t* dbg, cudaStream_t s)
{
    if (tokens < 0 || M < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (M == 0 || tokens == 0) return 0;
    if (!W || !x || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)W & 15) || ((uintptr_t)x & 15) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    const size_t x_stride = xsrc == 0 ? (size_t)K * 4 : (size_t)(K / 256) * BPDQ_Q8K_BYTES;
    const bool long_rows = (consumer_warps(K) + 1) * 32 > kSmallCtaThreads;
    const int per_pass = long_rows ? 1 : kMaxTokens;
    for (int t0 = 0; t0 < tokens; t0 += per_pass) {
        const int T = (tokens - t0) < per_pass ? (tokens - t0) : per_pass;
        GemvPlan p;
        int rc = make_plan(M, K, T, p);
        if (rc) return latch(rc);
        const void* xt = (const uint8_t*)x + (size_t)t0 * x_stride;
        float* ot = out + (size_t)t0 * M;
        if (layout == BPDQ_LAYOUT_GGML)
            rc = xsrc == 0 ? launch_T<BPDQ_LAYOUT_GGML, 0>(T, W, xt, ot, M, K, p, dbg, s)
                           : launch_T<BPDQ_LAYOUT_GGML, 1>(T, W, xt, ot, M, K, p, dbg, s);
        else
            rc = xsrc == 0 ? launch_T<BPDQ_LAYOUT_BPD, 0>(T, W, xt, ot, M, K, p, dbg, s)
                           : launch_T<BPDQ_LAYOUT_BPD, 1>(T, W, xt, ot, M, K, p, dbg, s);
        if (rc) return latch(rc);
        dbg = nullptr;  // sub-block dots are reported for token 0 only
    }
    return 0;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

int bpd_quant_q8_K_cuda(const float* x, uint8_t* y, size_t n_elements, void* stream)
{
    if ((n_elements % 256) != 0 || (n_elements && (!x || !y))) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return latch(BPDQ_ERR_ALIGN);
    const long nb = (long)(n_elements / 256);
    if (nb == 0) return 0;
    long want = (nb + 7) / 8, cap = (long)sm_count() * 8;
    int grid = (int)(want < cap ? want : cap);
    k_quant_q8_K<<<grid, 256, 0, (cudaStream_t)stream>>>(x, y, nb);
    return check_cuda(cudaGetLastError());
}

// Decode GEMV: out[M] = W[M][K] (Q4_K, C-ABI nibble order) . quantize_q8_K(x[K]).
int bpd_qmatmul_q4k_q8k_cuda(const uint8_t* qweight, const float* x, float* out, int M, int K, void* stream)
{
    return gemm_q4k_q8k(qweight, x, out, 1, M, K, BPDQ_LAYOUT_BPD, 0, nullptr, (cudaStream_t)stream);
}
// Full-control form: tokens >= 1, layout 0/1, xsrc 0 (fp32) / 1 (pre-quantized Q8_K), optional
// int32 [M][K/256][8] buffer receiving token 0's exact sub-block dots.
int bpd_qmm_q4k_q8k_cuda(const uint8_t* qweight, const void* x, float* out, int tokens, int M, int K, int layout,
                         int xsrc, int32_t* subdots, void* stream)
{
    if ((layout != 0 && layout != 1) || (xsrc != 0 && xsrc != 1)) return latch(BPDQ_ERR_ARG);
    return gemm_q4k_q8k(qweight, x, out, tokens, M, K, layout, xsrc, subdots, (cudaStream_t)stream);
}

// Dispatch-shaped entries (argument order of gpu_vecmat / gpu_matmul,
// lib/kernel_templates_llama.pl:147-158, 1104-1112): activations first, weights second.
void gpu_vecmat_q4k(const float* a, const uint8_t* wq, float* c, int k, int n)
{
    gemm_q4k_q8k(wq, a, c, 1, n, k, BPDQ_LAYOUT_BPD, 0, nullptr, current_stream());
}
void gpu_matmul_q4k(const float* A, const uint8_t* wq, float* Cout, int M, int N, int K)
{
    gemm_q4k_q8k(wq, A, Cout, M, N, K, BPDQ_LAYOUT_BPD, 0, nullptr, current_stream());
}

}  // extern "C"

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

#include <cstring>
#include <vector>

namespace bpdq {

constexpr int kMaxTokens = 4;       // tokens per pass (activation registers: 32 words each)

constexpr int kMaxProblems = 4;     // weight matrices per launch that share one activation vector

// One weight matrix of a launch.  All matrices of a launch have the same K and read the same
// activations; their rows are cut into tiles of rt rows and numbered consecutively.
struct GemvProblem {
    const uint8_t* W;   // [M][K/256][144]
    float* out;         // [T][M]
    int M;
    int tile_begin;     // first tile number of this matrix
};

struct GemvPlan {
    int nb;          // super-blocks per row
    int row_bytes;   // nb * 144
    int kc;          // K-chunks (warps) per row, ceil(nb / 16)
    int ng;          // consumer groups per CTA (each owns whole tiles)
    int nw;          // consumer warps = ng * kc
    int rt;          // rows per tile (1, 2 or 4)
    int slots;       // ring slots per group
    int n_tiles;     // tiles of all matrices together
    int n_problems;
    int grid;
    size_t smem;
    // smem offsets
    int off_ring, off_xq, off_xd, off_part, off_bar;
    // Tile hand-out is static: round n gives group g of CTA c tile (n*ng + g)*grid + c.
    // optional timeline capture (debug): 8 global-timer stamps per CTA, or null
    unsigned long long* trace;
    GemvProblem prob[kMaxProblems];
};

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define BPDQ_TRACE(slot)                                                              \
    do {                                                                              \
        if (p.trace && lane == 0 && (warp == 0 || (slot) == 7))                       \
            p.trace[(size_t)blockIdx.x * 8 + (slot)] = global_timer_ns();             \
    } while (0)


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

// Stages the quantized activations of all T tokens in shared memory, cooperatively by the
// consumer warps of the CTA: xq is [T][2*nb] half-super-blocks of 128 int8 padded to 144 B (so
// that the 16-byte reads of 32 consecutive lanes hit distinct banks), xds is [T][nb] block
// scales.  XSRC 0: x is fp32 and is quantized here, one warp per 256-block, UNR blocks in
// flight per warp so that the loop costs about one L2 round trip; XSRC 1: x is Q8_K blocks.
constexpr int kXqStride = 144;

template <int T, int XSRC>
__device__ __forceinline__ void stage_activations(const void* __restrict__ xin, int K, int nb, uint8_t* xq,
                                                  float* xds, int warp, int lane, int n_warps)
{
    const int n_hb = 2 * nb;
    if (XSRC == 0) {
        constexpr int UNR = 4;
        const float* x = reinterpret_cast<const float*>(xin);
        const int total = T * nb;
        for (int blk0 = warp; blk0 < total; blk0 += n_warps * UNR) {
            float4 v0[UNR], v1[UNR];
#pragma unroll
            for (int u = 0; u < UNR; u++) {
                const int blk = blk0 + u * n_warps;
                if (blk < total) {
                    // blk = t*nb + b and x is [T][K] with K = 256*nb: block blk starts at 256*blk
                    const float4* xb = reinterpret_cast<const float4*>(x + (size_t)blk * 256);
                    v0[u] = __ldg(xb + lane);
                    v1[u] = __ldg(xb + 32 + lane);
                }
            }
#pragma unroll
            for (int u = 0; u < UNR; u++) {
                const int blk = blk0 + u * n_warps;
                if (blk < total) {
                    uint32_t p0, p1;
                    float d;
                    quantize_block_256(v0[u], v1[u], p0, p1, d);
                    uint8_t* dst = xq + (size_t)2 * blk * kXqStride;  // half-block index t*n_hb + 2b = 2*blk
                    reinterpret_cast<uint32_t*>(dst)[lane] = p0;
                    reinterpret_cast<uint32_t*>(dst + kXqStride)[lane] = p1;
                    if (lane == 0) xds[blk] = d;
                }
            }
        }
    } else {
        const uint8_t* xb = reinterpret_cast<const uint8_t*>(xin);
        const int tid = warp * 32 + lane, n_threads = n_warps * 32;
        for (int i = tid; i < T * nb * 64; i += n_threads) {
            const int blk = i >> 6, w = i & 63;  // word w of the 64 qs words of block blk = t*nb + b
            const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(xb + (size_t)blk * BPDQ_Q8K_BYTES + 4) + w);
            uint8_t* dst = xq + ((size_t)2 * blk + (w >> 5)) * kXqStride;
            reinterpret_cast<uint32_t*>(dst)[w & 31] = v;
        }
        for (int i = tid; i < T * nb; i += n_threads)
            xds[i] = __uint_as_float(__ldg(reinterpret_cast<const uint32_t*>(xb + (size_t)i * BPDQ_Q8K_BYTES)));
    }
    (void)n_hb;
    (void)K;
}

// Sums R per-lane partials across the 32 lanes of a warp.  After the call the total of row
// rr sits in lane rr*(32/R) (the other lanes hold partial garbage).  Fixed order: for R=4
// lanes are folded by xor 16 (rows split 0,1 | 2,3), xor 8 (row split), then xor 4, 2, 1; for
// R=2 by xor 16 (row split) then 8, 4, 2, 1; for R=1 a plain butterfly 16, 8, 4, 2, 1.
template <int R>
__device__ __forceinline__ float fold_rows(const float (&v)[R], int lane)
{
    float c;
    if constexpr (R == 4) {
        const bool up = (lane & 16) != 0;
        float a = (up ? v[2] : v[0]) + __shfl_xor_sync(0xFFFFFFFFu, up ? v[0] : v[2], 16);
        float b = (up ? v[3] : v[1]) + __shfl_xor_sync(0xFFFFFFFFu, up ? v[1] : v[3], 16);
        const bool up2 = (lane & 8) != 0;
        c = (up2 ? b : a) + __shfl_xor_sync(0xFFFFFFFFu, up2 ? a : b, 8);
        c += __shfl_xor_sync(0xFFFFFFFFu, c, 4);
    } else if constexpr (R == 2) {
        const bool up = (lane & 16) != 0;
        c = (up ? v[R - 1] : v[0]) + __shfl_xor_sync(0xFFFFFFFFu, up ? v[0] : v[R - 1], 16);
        c += __shfl_xor_sync(0xFFFFFFFFu, c, 8);
        c += __shfl_xor_sync(0xFFFFFFFFu, c, 4);
    } else {
        c = v[0] + __shfl_xor_sync(0xFFFFFFFFu, v[0], 16);
        c += __shfl_xor_sync(0xFFFFFFFFu, c, 8);
        c += __shfl_xor_sync(0xFFFFFFFFu, c, 4);
    }
    c += __shfl_xor_sync(0xFFFFFFFFu, c, 2);
    c += __shfl_xor_sync(0xFFFFFFFFu, c, 1);
    return c;
}


// Kernel structure.  A CTA has `ng` consumer groups of `kc` warps and one producer warp.  A
// group owns whole tiles of R consecutive weight rows (one contiguous byte span) and has its
// own ring of `slots` shared-memory slots with full/empty mbarriers, so groups never wait for
// each other.  Tile hand-out is static (round n gives group g of CTA c tile (n*ng + g)*grid + c),
// so producer and consumers walk the same sequence without talking; lane g of the producer
// warp feeds group g, which keeps the copy issue rate above what HBM can deliver.
// Inside a group, warp c covers K-chunk c of all R rows; the R rows are independent
// instruction streams, which is what hides shared-memory and dot-product latency.
// MAXTHREADS / MINBLOCKS bound the CTA size and the registers per thread so that CTAs of
// consecutive launches can be resident on one SM together (programmatic dependent launch).
template <int T, int R, int LAYOUT, int XSRC, int MAXTHREADS, int MINBLOCKS>
__global__ void __launch_bounds__(MAXTHREADS, MINBLOCKS)
k_gemv_q4k_q8k(const void* __restrict__ xin, int K, const GemvPlan p, int* __restrict__ err,
               int32_t* __restrict__ dbg)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                           // [ng][slots][R*row_bytes]
    uint8_t* xq = smem + p.off_xq;                               // [T][n_hb][144]
    float* xds = reinterpret_cast<float*>(smem + p.off_xd);      // [T][nb]
    float* part = reinterpret_cast<float*>(smem + p.off_part);   // [ng][2][R][kc][T]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);   // [ng*slots]
    uint64_t* empty = full + p.ng * p.slots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + p.ng * p.slots);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_producer = (warp == p.nw);
    const int n_hb = 2 * p.nb;
    const uint32_t tile_bytes_full = (uint32_t)R * p.row_bytes;
    BPDQ_TRACE(0);

    if (tid == 0) {
        for (int s = 0; s < p.ng * p.slots; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.kc);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // Programmatic dependent launch: the next kernel in the stream may start once every CTA
    // of this one has got here.  Its CTAs fill their weight rings while we compute and then
    // block in pdl_wait() until this grid has finished.
    pdl_launch_dependents();
    BPDQ_TRACE(1);

    if (is_producer) {
        if (lane < p.ng) {
            // Weights never depend on the previous kernel: no pdl_wait on this path.
            const int g = lane;
            int slot = 0;
            uint32_t wait_parity = 0;   // phase of empty[] that frees a slot for its next use
            bool wrapped = false;       // false during the first pass over the ring: slots are free
            for (int v = g * (int)gridDim.x + (int)blockIdx.x; v < p.n_tiles; v += p.ng * (int)gridDim.x) {
                const int s = g * p.slots + slot;
                if (wrapped && !mbar_wait_bounded(&empty[s], wait_parity, err, 1)) break;
                const uint8_t* Wj = p.prob[0].W;
                int Mj = p.prob[0].M, tb = 0;
#pragma unroll
                for (int q = 1; q < kMaxProblems; q++)
                    if (q < p.n_problems && v >= p.prob[q].tile_begin) {
                        Wj = p.prob[q].W;
                        Mj = p.prob[q].M;
                        tb = p.prob[q].tile_begin;
                    }
                const int row0 = (v - tb) * R;
                const uint32_t bytes = (uint32_t)min(R, Mj - row0) * p.row_bytes;
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(ring + (size_t)s * tile_bytes_full, Wj + (size_t)row0 * p.row_bytes, bytes, &full[s]);
                if (++slot == p.slots) {
                    slot = 0;
                    if (wrapped) wait_parity ^= 1u;
                    wrapped = true;
                }
            }
            if (lane == 0) BPDQ_TRACE(7);
        }
        return;
    }

    // Activations may be written by the previous kernel: wait for it before the first read.
    pdl_wait();
    BPDQ_TRACE(2);

    // ---- consumer warps
    const int g = warp / p.kc;      // group
    const int kc = warp % p.kc;     // K-chunk of this warp (fixed for the whole kernel)
    const int hb = 32 * kc + lane;  // half-super-block of this lane
    const bool active = hb < n_hb;
    const int sb = hb >> 1, half = hb & 1;
    const int n_consumer_threads = p.nw * 32;

    stage_activations<T, XSRC>(xin, K, p.nb, xq, xds, warp, lane, p.nw);
    named_bar_sync(2, n_consumer_threads);
    BPDQ_TRACE(3);

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
    BPDQ_TRACE(4);

    constexpr int kLanesPerRow = 32 / R;
    const int my_row = lane / kLanesPerRow;                  // row whose total this lane ends up holding
    const bool row_leader = (lane % kLanesPerRow) == 0;
    float* part_g = part + (size_t)g * 2 * R * p.kc * T;

    int slot = 0;
    uint32_t parity = 0;
    int n = 0;
    for (int v = g * (int)gridDim.x + (int)blockIdx.x; v < p.n_tiles; v += p.ng * (int)gridDim.x, n++) {
        const int s = g * p.slots + slot;
        const bool ok = mbar_wait_bounded(&full[s], parity, err, 2);
        if (!ok) {
            // gave up: tell the group mates (they may be past the wait) and meet them once more
            *abort_flag = 1;
            if (p.kc > 1) named_bar_sync(3 + g, p.kc * 32);
            return;
        }
        if (n == 0) BPDQ_TRACE(5);
        if (++slot == p.slots) {
            slot = 0;
            parity ^= 1u;
        }
        int M = p.prob[0].M, tb = 0;
        float* __restrict__ out = p.prob[0].out;
        bool first_matrix = true;
#pragma unroll
        for (int q = 1; q < kMaxProblems; q++)
            if (q < p.n_problems && v >= p.prob[q].tile_begin) {
                M = p.prob[q].M;
                tb = p.prob[q].tile_begin;
                out = p.prob[q].out;
                first_matrix = false;
            }
        const int row0 = (v - tb) * R;
        const int rows = min(R, M - row0);
        const uint8_t* tile_smem = ring + (size_t)s * tile_bytes_full + (size_t)sb * BPDQ_Q4K_BYTES;
        float* part_n = part_g + (size_t)(n & 1) * R * p.kc * T;

        float acc[R][T];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int t = 0; t < T; t++) acc[r][t] = 0.0f;
        if (active) {
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (r < rows) {
                    // sub-block dots are reported for the first matrix of a launch only
                    int32_t* d = (dbg && first_matrix) ? dbg + ((size_t)(row0 + r) * p.nb + sb) * 8 : nullptr;
                    half_block_fma<T, LAYOUT>(tile_smem + (size_t)r * p.row_bytes, half, xr, bs, xd, acc[r], d);
                }
            }
        }
        // this warp no longer reads the slot
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

#pragma unroll
        for (int t = 0; t < T; t++) {
            float vv[R];
#pragma unroll
            for (int r = 0; r < R; r++) vv[r] = acc[r][t];
            const float total = fold_rows<R>(vv, lane);
            if (row_leader && my_row < rows) {
                if (p.kc == 1) out[(size_t)t * M + row0 + my_row] = total;
                else part_n[((size_t)my_row * p.kc + kc) * T + t] = total;
            }
        }

        if (p.kc > 1) {
            // K-chunks of a row live in the kc warps of this group: add them in ascending order.
            named_bar_sync(3 + g, p.kc * 32);
            if (*abort_flag) return;
            const int gt = kc * 32 + lane;
            for (int e = gt; e < rows * T; e += p.kc * 32) {
                const int r = e / T, t = e - r * T;
                float sum = part_n[((size_t)r * p.kc + 0) * T + t];
                for (int c = 1; c < p.kc; c++) sum += part_n[((size_t)r * p.kc + c) * T + t];
                out[(size_t)t * M + row0 + r] = sum;
            }
        }
    }
    BPDQ_TRACE(6);
}

// ---------------------------------------------------------------- host side

// Timeline capture for tuning: when set, launch k writes 8 stamps per CTA at
// trace_base + k * trace_stride.
static unsigned long long* g_trace_base = nullptr;
static size_t g_trace_stride = 0;
static int g_trace_left = 0;

constexpr int kSmemLimit = 227 * 1024;
constexpr int kSmallCtaThreads = 288;   // up to 8 consumer warps + the producer
constexpr int kMidCtaThreads = 544;     // up to 16 consumer warps + the producer

static int rows_per_tile(int row_bytes)
{
    const int cap = tuning().tile_bytes;
    if (4 * row_bytes <= cap) return 4;
    if (2 * row_bytes <= cap) return 2;
    return 1;
}

static size_t plan_smem(GemvPlan& p, int T)
{
    size_t off = 0;
    auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
    p.off_ring = take((size_t)p.ng * p.slots * p.rt * p.row_bytes);
    p.off_xq = take((size_t)T * 2 * p.nb * kXqStride);
    p.off_xd = take((size_t)T * p.nb * 4);
    p.off_part = take((size_t)p.ng * 2 * p.rt * p.kc * T * 4);
    p.off_bar = take((size_t)2 * p.ng * p.slots * 8 + 8);
    return off;
}

// Fills everything but the problem table's pointers.  Ms: rows of each matrix.
static int make_plan(const int* Ms, int n_problems, int K, int T, GemvPlan& p)
{
    if (K <= 0 || (K % 256) != 0 || T < 1 || T > kMaxTokens) return BPDQ_ERR_ARG;
    if (n_problems < 1 || n_problems > kMaxProblems) return BPDQ_ERR_ARG;
    const Tuning& tu = tuning();
    p.nb = K / 256;
    p.row_bytes = p.nb * BPDQ_Q4K_BYTES;
    p.kc = (p.nb + 15) / 16;
    if (p.kc > 31) return BPDQ_ERR_RANGE;  // K > 126976: one warp per 4096 K, 31 consumer warps at most
    p.ng = (T > 2 && tu.warps > 8 ? 8 : tu.warps) / p.kc;   // 3-4 tokens need the registers of a small CTA
    if (p.ng < 1) p.ng = 1;
    if (p.ng > 12 && p.kc > 1) p.ng = 12;  // named barriers 3 .. 3+ng-1 (used only when kc > 1)
    if (p.ng > 31) p.ng = 31;
    p.nw = p.ng * p.kc;
    p.rt = rows_per_tile(p.row_bytes);
    p.n_problems = n_problems;
    p.n_tiles = 0;
    for (int j = 0; j < kMaxProblems; j++) {
        p.prob[j].W = nullptr;
        p.prob[j].out = nullptr;
        p.prob[j].M = 0;
        p.prob[j].tile_begin = 0x7FFFFFFF;
    }
    for (int j = 0; j < n_problems; j++) {
        if (Ms[j] < 0) return BPDQ_ERR_ARG;
        p.prob[j].M = Ms[j];
        p.prob[j].tile_begin = p.n_tiles;
        p.n_tiles += (Ms[j] + p.rt - 1) / p.rt;
    }
    p.slots = tu.stages < 2 ? 2 : tu.stages;
    p.smem = plan_smem(p, T);
    while (p.smem > (size_t)kSmemLimit && (p.slots > 2 || p.ng > 1)) {
        if (p.slots > 2) p.slots--;
        else { p.ng--; p.nw = p.ng * p.kc; }
        p.smem = plan_smem(p, T);
    }
    if (p.smem > (size_t)kSmemLimit) return BPDQ_ERR_RANGE;
    const int threads = (p.nw + 1) * 32;
    int per_sm = kSmemLimit / (int)p.smem;
    if (per_sm > 2048 / threads) per_sm = 2048 / threads;
    if (per_sm > tu.ctas_per_sm) per_sm = tu.ctas_per_sm;
    if (per_sm < 1) per_sm = 1;
    const long cap = (long)sm_count() * per_sm;
    // one tile per group at least; small launches still spread over all SMs
    long want = (p.n_tiles + p.ng - 1) / p.ng;
    if (want < sm_count()) want = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
    if (want < 1) want = 1;
    p.grid = (int)(want < cap ? want : cap);
    p.trace = nullptr;
    return 0;
}

template <int T, int R, int LAYOUT, int XSRC, int MAXTHREADS, int MINBLOCKS>
static int launch_one(const void* x, int K, const GemvPlan& p, int32_t* dbg, cudaStream_t s)
{
    auto kern = k_gemv_q4k_q8k<T, R, LAYOUT, XSRC, MAXTHREADS, MINBLOCKS>;
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
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, x, K, p, device_error_flag(), dbg));
}

template <int T, int LAYOUT, int XSRC, int MAXTHREADS, int MB>
static int launch_R2(const void* x, int K, const GemvPlan& p, int32_t* dbg, cudaStream_t s)
{
    switch (p.rt) {
        case 4: return launch_one<T, 4, LAYOUT, XSRC, MAXTHREADS, MB>(x, K, p, dbg, s);
        case 2: return launch_one<T, 2, LAYOUT, XSRC, MAXTHREADS, MB>(x, K, p, dbg, s);
        case 1: return launch_one<T, 1, LAYOUT, XSRC, MAXTHREADS, MB>(x, K, p, dbg, s);
    }
    return BPDQ_ERR_ARG;
}

template <int T, int LAYOUT, int XSRC>
static int launch_R(const void* x, int K, const GemvPlan& p, int32_t* dbg, cudaStream_t s)
{
    const int threads = (p.nw + 1) * 32;
    if (threads > kMidCtaThreads) {
        // very long rows (K > 65536): many warps per row; registers capped by the CTA size
        if (T != 1 || p.rt != 1) return BPDQ_ERR_RANGE;
        return launch_one<1, 1, LAYOUT, XSRC, 1024, 1>(x, K, p, dbg, s);
    }
    if (threads > kSmallCtaThreads) {
        if (T > 2) return BPDQ_ERR_RANGE;
        return launch_R2<(T > 2 ? 1 : T), LAYOUT, XSRC, kMidCtaThreads, 1>(x, K, p, dbg, s);
    }
    return launch_R2<T, LAYOUT, XSRC, kSmallCtaThreads, (T == 1 ? 2 : 1)>(x, K, p, dbg, s);
}

template <int LAYOUT, int XSRC>
static int launch_T(int T, const void* x, int K, const GemvPlan& p, int32_t* dbg, cudaStream_t s)
{
    switch (T) {
        case 1: return launch_R<1, LAYOUT, XSRC>(x, K, p, dbg, s);
        case 2: return launch_R<2, LAYOUT, XSRC>(x, K, p, dbg, s);
        case 3: return launch_R<3, LAYOUT, XSRC>(x, K, p, dbg, s);
        case 4: return launch_R<4, LAYOUT, XSRC>(x, K, p, dbg, s);
    }
    return BPDQ_ERR_ARG;
}

// n matrices W[j] ([Ms[j]][K], Q4_K) against the same activations.  outs[j] is [tokens][Ms[j]];
// x is fp32 [tokens][K] (xsrc 0) or Q8_K blocks [tokens][K/256] (xsrc 1).  More than
// kMaxTokens tokens run as several passes over the weights.
int gemm_q4k_q8k_multi(int n, const uint8_t* const* Ws, float* const* outs, const int* Ms, const void* x, int tokens,
                       int K, int layout, int xsrc, int32_t* dbg, cudaStream_t s)
{
    if (n < 1 || n > kMaxProblems || tokens < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    long total_rows = 0;
    for (int j = 0; j < n; j++) {
        if (Ms[j] < 0) return latch(BPDQ_ERR_ARG);
        total_rows += Ms[j];
    }
    if (total_rows == 0 || tokens == 0) return 0;
    if (!x) return latch(BPDQ_ERR_ARG);
    if ((uintptr_t)x & 15) return latch(BPDQ_ERR_ALIGN);
    for (int j = 0; j < n; j++) {
        if (Ms[j] > 0 && (!Ws[j] || !outs[j])) return latch(BPDQ_ERR_ARG);
        if (((uintptr_t)Ws[j] & 15) || ((uintptr_t)outs[j] & 3)) return latch(BPDQ_ERR_ALIGN);
    }
    const size_t x_stride = xsrc == 0 ? (size_t)K * 4 : (size_t)(K / 256) * BPDQ_Q8K_BYTES;
    int per_pass = kMaxTokens;
    {
        GemvPlan probe;
        int rc = make_plan(Ms, n, K, tokens < kMaxTokens ? tokens : kMaxTokens, probe);
        if (rc) return latch(rc);
        const int threads = (probe.nw + 1) * 32;
        if (threads > kMidCtaThreads) per_pass = 1;
        else if (threads > kSmallCtaThreads) per_pass = 2;
    }
    for (int t0 = 0; t0 < tokens; t0 += per_pass) {
        const int T = (tokens - t0) < per_pass ? (tokens - t0) : per_pass;
        GemvPlan p;
        int rc = make_plan(Ms, n, K, T, p);
        if (rc) return latch(rc);
        if (g_trace_base && g_trace_left > 0) {
            p.trace = g_trace_base;
            g_trace_base += g_trace_stride;
            g_trace_left--;
        }
        for (int j = 0; j < n; j++) {
            p.prob[j].W = Ws[j];
            p.prob[j].out = outs[j] + (size_t)t0 * Ms[j];
        }
        const void* xt = (const uint8_t*)x + (size_t)t0 * x_stride;
        if (layout == BPDQ_LAYOUT_GGML)
            rc = xsrc == 0 ? launch_T<BPDQ_LAYOUT_GGML, 0>(T, xt, K, p, dbg, s)
                           : launch_T<BPDQ_LAYOUT_GGML, 1>(T, xt, K, p, dbg, s);
        else
            rc = xsrc == 0 ? launch_T<BPDQ_LAYOUT_BPD, 0>(T, xt, K, p, dbg, s)
                           : launch_T<BPDQ_LAYOUT_BPD, 1>(T, xt, K, p, dbg, s);
        if (rc) return latch(rc);
        dbg = nullptr;  // sub-block dots are reported for token 0 only
    }
    return 0;
}

int gemm_q4k_q8k(const uint8_t* W, const void* x, float* out, int tokens, int M, int K, int layout, int xsrc,
                 int32_t* dbg, cudaStream_t s)
{
    if (M < 0) return latch(BPDQ_ERR_ARG);
    // many tokens: the weights would be streamed once per four tokens here; the tensor-core
    // kernels read them once per 64.  Measured on 14336x4096, 4096x14336, 4096x4096 and 1024x4096:
    // the tcgen05 kernel (128-row tiles, split K) is ahead from 24 tokens on matrices of 2^25
    // weights and more (from 33 when there are fewer than 8192 rows), mma.sync everywhere else.
    if (tokens > 4 && layout == BPDQ_LAYOUT_BPD && xsrc == 0 && !dbg) {
        const bool large = (long)M * K >= (1L << 25);
        if (large && (tokens >= 33 || (tokens >= 24 && M >= 8192)))
            return gemm_q4k_q8k_tc5(W, reinterpret_cast<const float*>(x), out, tokens, M, K, s);
        return gemm_q4k_q8k_mma(W, reinterpret_cast<const float*>(x), out, tokens, M, K, s);
    }
    return gemm_q4k_q8k_multi(1, &W, &out, &M, x, tokens, K, layout, xsrc, dbg, s);
}


// ================================================================ batched independent GEMVs
//
// One launch runs up to kMaxBatch independent products out_j = W_j . q8K(x_j), each with its
// own shape (M_j, K_j); several may name the same x_j.  This is the shape of a decoder layer's
// seven projections when nothing in between is computed (the benchmark workload), and of any
// set of matrices that are known to be independent.
//
// Differences from the kernel above:
//  * every consumer warp owns whole tiles and whole rows: a row longer than 4096 weights is
//    walked in K-chunks of 4096 by the same warp (lane l takes half-super-block 32c + l of
//    chunk c), so no warp ever waits for another one and the mapping does not depend on K;
//  * all activation vectors of the launch are quantized once, up front, into shared memory
//    as 144-byte records per half-super-block: 128 int8, then the four sub-block sums as
//    int16 and the block scale (the padding of the layout above, put to use).  A lane fetches
//    its record (nine 16-byte reads, conflict-free) once per tile and K-chunk;
//  * accumulation order: a lane adds its half-blocks in ascending chunk order with the two
//    FMAs of half_block_fma, then the rows are folded over the lanes by fold_rows.

constexpr int kMaxBatch = 8;
constexpr size_t kBigLaunchBytes = 8u << 20;       // Q4_K weights of a launch from which the larger tile budget applies
constexpr size_t kBigLaunchBytesQ80 = 48u << 20;   // the same for Q8_0 weights (two rows of K = 4096 per tile)
constexpr int kBigLaunchTileBytes = 9216;

struct BatchProblem {
    const uint8_t* W;
    float* out;
    int M, nb, row_bytes, rt;     // rows, super-blocks per row, bytes per row, rows per tile
    int tile_begin;
    int xq_off;                   // byte offset of this problem's activation records in shared memory
    int accumulate;               // 1: out[row] += result (residual connection folded into the product)
};
struct BatchVector {              // one distinct activation vector
    const float* x;
    int nb, xq_off;
};
struct BatchPlan {
    int n_problems, n_vectors, n_tiles, total_blocks;
    int nw, slots, slot_bytes, grid;
    int off_ring, off_xq, off_bar;
    size_t smem;
    unsigned long long* trace;
    // activation records already quantized by k_quant_records (same layout as the shared-memory
    // records, xq_bytes in all), or null: quantize inside this kernel
    const uint8_t* records;
    int xq_bytes;
    // what the CTAs do to the launch's single input vector before they quantize it themselves (records
    // null): 0 nothing, 1 rms_norm(pro_a, weights pro_b, pro_eps), 2 silu(pro_a) * pro_b
    int prologue;
    const float* pro_a;
    const float* pro_b;
    float pro_eps;
    BatchProblem prob[kMaxBatch];
    BatchVector vec[kMaxBatch];
};


// Quantizes one 256-block held by a warp (lane l: elements 4l..4l+3 in v0, 128+4l.. in v1) and
// writes its two 144-byte records: 128 int8, four int16 sub-block sums, the fp32 block scale.
__device__ __forceinline__ void write_records(const float4& v0, const float4& v1, uint8_t* rec0, int lane)
{
    uint32_t p0, p1;
    float d;
    quantize_block_256(v0, v1, p0, p1, d);
    uint8_t* rec1 = rec0 + kXqStride;
    reinterpret_cast<uint32_t*>(rec0)[lane] = p0;
    reinterpret_cast<uint32_t*>(rec1)[lane] = p1;
    int s0 = dp4a_ss(p0, 0x01010101u, 0), s1 = dp4a_ss(p1, 0x01010101u, 0);   // 8 lanes = one sub-block
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, o);
        s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
    }
    if ((lane & 7) == 0) {
        reinterpret_cast<short*>(rec0 + 128)[lane >> 3] = (short)s0;
        reinterpret_cast<short*>(rec1 + 128)[lane >> 3] = (short)s1;
    }
    if (lane == 0) {
        reinterpret_cast<float*>(rec0 + 128)[2] = d;
        reinterpret_cast<float*>(rec0 + 128)[3] = 0.0f;
        reinterpret_cast<float*>(rec1 + 128)[2] = d;
        reinterpret_cast<float*>(rec1 + 128)[3] = 0.0f;
    }
}

// ---- Q8_0 weights (34-byte blocks: fp16 scale + 32 int8; bench/bpd_cpu.c:3886-3890 of the
// reference) against Q8_0-quantized activations (rule of bench/bpd_cpu.c:4106-4136: stored
// scale f16(amax/127), multiplier 127/amax, round half to even).  Same kernel skeleton; a lane
// owns a PAIR of blocks (68 bytes = 17 aligned words of a row) and the activation record of a
// pair is 80 bytes: 64 int8, the two block scales as fp32 (already widened from fp16), 8 spare.
constexpr int kQ80PairStride = 80;

// Quantizes 256 consecutive activations held by a warp (v0: elements 4l.., v1: 128+4l..) into
// the four pair records starting at rec.  Eight lanes share one 32-element block.
__device__ __forceinline__ void write_records_q80(const float4& v0, const float4& v1, uint8_t* rec, int lane)
{
    const float4 v[2] = {v0, v1};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        float amax = fmaxf(fmaxf(fabsf(v[h].x), fabsf(v[h].y)), fmaxf(fabsf(v[h].z), fabsf(v[h].w)));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        const __half d16 = __float2half_rn(__fdiv_rn(amax, 127.0f));
        const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        auto q = [mul](float x) -> uint32_t { return (uint32_t)__float2int_rn(__fmul_rn(x, mul)) & 0xFFu; };
        const uint32_t packed = q(v[h].x) | (q(v[h].y) << 8) | (q(v[h].z) << 16) | (q(v[h].w) << 24);
        const int blk = 4 * h + (lane >> 3);          // block 0..7 of the 256
        uint8_t* pr = rec + (size_t)(blk >> 1) * kQ80PairStride;
        reinterpret_cast<uint32_t*>(pr + 32 * (blk & 1))[lane & 7] = packed;
        if ((lane & 7) == 0) reinterpret_cast<float*>(pr + 64)[blk & 1] = __half2float(d16);
    }
}

template <int R>
__device__ __forceinline__ void batch_tile_q80(const uint8_t* tile_smem, const uint8_t* xq, const BatchProblem& pb,
                                               int row0, int lane)
{
    const int rows = min(R, pb.M - row0);
    const int n_pairs = 4 * pb.nb;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.0f;
    for (int pp = lane; pp < n_pairs; pp += 32) {
        const uint4* rec = reinterpret_cast<const uint4*>(xq + (size_t)pp * kQ80PairStride);
        uint32_t xr[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 t = rec[i];
            xr[4 * i + 0] = t.x;
            xr[4 * i + 1] = t.y;
            xr[4 * i + 2] = t.z;
            xr[4 * i + 3] = t.w;
        }
        const uint4 sc = rec[4];
        const float ad0 = __uint_as_float(sc.x), ad1 = __uint_as_float(sc.y);
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (r < rows) {
                const uint32_t* w = reinterpret_cast<const uint32_t*>(tile_smem + (size_t)r * pb.row_bytes) + 17 * pp;
                uint32_t ww[17];
#pragma unroll
                for (int i = 0; i < 17; i++) ww[i] = w[i];
                // block 0: scale = low half of word 0, quants = bytes 2..33 (realign by 16 bits)
                int s0 = 0, s1 = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    s0 = dp4a_ss(__funnelshift_r(ww[i], ww[i + 1], 16), xr[i], s0);
                    s1 = dp4a_ss(ww[9 + i], xr[8 + i], s1);   // block 1: quants are words 9..16
                }
                const float wd0 = f16_bits_to_f32(ww[0] & 0xFFFFu), wd1 = f16_bits_to_f32(ww[8] >> 16);
                acc[r] = fmaf((float)s0, wd0 * ad0, acc[r]);
                acc[r] = fmaf((float)s1, wd1 * ad1, acc[r]);
            }
        }
    }
    const float total = fold_rows<R>(acc, lane);
    constexpr int kLanesPerRow = 32 / R;
    const int my_row = lane / kLanesPerRow;
    if ((lane % kLanesPerRow) == 0 && my_row < rows) pb.out[row0 + my_row] = total;
}


struct QuantVectors {
    int n_vectors, total_blocks;
    BatchVector vec[kMaxBatch];
};

// Activation quantizer of the batched path: one warp per 256-block, records go to global
// scratch memory in the layout the GEMV kernel keeps in shared memory.  The inputs are not
// written by the kernel before it in the stream in any way this kernel could know, so it reads
// them at once and only joins the stream order (pdl_wait) before it ends; the scratch it
// writes must therefore not be in use by an earlier launch.
template <int FMT>
__global__ void __launch_bounds__(256) k_quant_records(const QuantVectors q, uint8_t* __restrict__ records,
                                                        int wait_first)
{
    pdl_launch_dependents();
    if (wait_first) pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    for (int b = warp; b < q.total_blocks; b += n_warps) {
        int blk = b, k = 0;
        while (k + 1 < q.n_vectors && blk >= q.vec[k].nb) { blk -= q.vec[k].nb; k++; }
        const float4* xb = reinterpret_cast<const float4*>(q.vec[k].x + (size_t)blk * 256);
        const float4 v0 = __ldg(xb + lane), v1 = __ldg(xb + 32 + lane);
        if (FMT == 0) write_records(v0, v1, records + q.vec[k].xq_off + (size_t)(2 * blk) * kXqStride, lane);
        else write_records_q80(v0, v1, records + q.vec[k].xq_off + (size_t)(4 * blk) * kQ80PairStride, lane);
    }
    if (!wait_first) pdl_wait();
}


// ---- Decode glue: the elementwise steps either side of a product write the product's activation
// records directly, so the fp32 vector between them never goes to memory and the step is one launch.
//
// rms_norm fused with the record quantizer.  One CTA per row; arithmetic and summation order are
// those of k_rms_norm in decode_ops.cu (lib/kernel_templates_llama.pl:529-593 of the reference):
// per-thread fmaf chain over c = t, t+256, ..., butterfly over the warp, the eight warp sums added
// in order, scale = rsqrtf(sum/cols + eps), y = (x*scale)*w; then the rule of quantize_block_256.
__global__ void __launch_bounds__(256) k_rmsnorm_records(const float* __restrict__ in, const float* __restrict__ w,
                                                          uint8_t* __restrict__ records, int cols, float eps)
{
    __shared__ float s_sum[8];
    pdl_launch_dependents();
    pdl_wait();   // the row is the previous product's output (residual stream)
    const float* x = in + (size_t)blockIdx.x * cols;
    uint8_t* rec = records + (size_t)blockIdx.x * (cols / 256) * 2 * kXqStride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float t = 0.0f;
    // (data written by the launch before this one is read past L1: ld.global.cg)
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float v = __ldcg(x + c);
        t = fmaf(v, v, t);
    }
    t = warp_sum(t);
    if (lane == 0) s_sum[warp] = t;
    __syncthreads();
    float tot = s_sum[0];
#pragma unroll
    for (int i = 1; i < 8; i++) tot += s_sum[i];
    const float scale = rsqrtf(tot / (float)cols + eps);
    for (int b = warp; b < cols / 256; b += 8) {
        const float4* xb = reinterpret_cast<const float4*>(x + (size_t)b * 256);
        const float4* wb = reinterpret_cast<const float4*>(w + (size_t)b * 256);
        const float4 a0 = __ldcg(xb + lane), a1 = __ldcg(xb + 32 + lane), w0 = __ldg(wb + lane), w1 = __ldg(wb + 32 + lane);
        const float4 v0 = make_float4(a0.x * scale * w0.x, a0.y * scale * w0.y, a0.z * scale * w0.z, a0.w * scale * w0.w);
        const float4 v1 = make_float4(a1.x * scale * w1.x, a1.y * scale * w1.y, a1.z * scale * w1.z, a1.w * scale * w1.w);
        write_records(v0, v1, rec + (size_t)(2 * b) * kXqStride, lane);
    }
}

// silu(gate) * up fused with the record quantizer (the arithmetic of k_elementwise's OP_SILU then
// OP_MUL: x / (1 + expf(-x)), lib/kernel_templates_llama.pl:668).  One warp per 256-block.
__global__ void __launch_bounds__(256) k_swiglu_records(const float* __restrict__ gate, const float* __restrict__ up,
                                                         uint8_t* __restrict__ records, long n_blocks)
{
    pdl_launch_dependents();
    pdl_wait();   // gate and up come from the product launched just before
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
    auto act = [](float g, float u) { return (g / (1.0f + expf(-g))) * u; };
    for (long b = warp; b < n_blocks; b += n_warps) {
        const float4* gb = reinterpret_cast<const float4*>(gate + (size_t)b * 256);
        const float4* ub = reinterpret_cast<const float4*>(up + (size_t)b * 256);
        const float4 g0 = __ldcg(gb + lane), g1 = __ldcg(gb + 32 + lane), u0 = __ldcg(ub + lane), u1 = __ldcg(ub + 32 + lane);
        const float4 v0 = make_float4(act(g0.x, u0.x), act(g0.y, u0.y), act(g0.z, u0.z), act(g0.w, u0.w));
        const float4 v1 = make_float4(act(g1.x, u1.x), act(g1.y, u1.y), act(g1.z, u1.z), act(g1.w, u1.w));
        write_records(v0, v1, records + (size_t)(2 * b) * kXqStride, lane);
    }
}

// Plain quantizer to records for a vector that the previous launch produced.
__global__ void __launch_bounds__(256) k_vector_records(const float* __restrict__ x, uint8_t* __restrict__ records,
                                                         long n_blocks)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
    for (long b = warp; b < n_blocks; b += n_warps) {
        const float4* xb = reinterpret_cast<const float4*>(x + (size_t)b * 256);
        write_records(__ldcg(xb + lane), __ldcg(xb + 32 + lane), records + (size_t)(2 * b) * kXqStride, lane);
    }
}

template <int R, int LAYOUT, int ACC>
__device__ __forceinline__ void batch_tile(const uint8_t* tile_smem, const uint8_t* xq, const BatchProblem& pb, int row0,
                                           int lane)
{
    const int rows = min(R, pb.M - row0);
    const int n_hb = 2 * pb.nb;
    float acc[R][1];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r][0] = 0.0f;
    for (int hb = lane; hb < n_hb; hb += 32) {
        const uint4* rec = reinterpret_cast<const uint4*>(xq + (size_t)hb * kXqStride);
        uint32_t xr[1][32];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint4 v = rec[i];
            xr[0][4 * i + 0] = v.x;
            xr[0][4 * i + 1] = v.y;
            xr[0][4 * i + 2] = v.z;
            xr[0][4 * i + 3] = v.w;
        }
        const uint4 tail = rec[8];
        int bs[1][4];
        bs[0][0] = (int)(short)(tail.x & 0xFFFFu);
        bs[0][1] = (int)(short)(tail.x >> 16);
        bs[0][2] = (int)(short)(tail.y & 0xFFFFu);
        bs[0][3] = (int)(short)(tail.y >> 16);
        float xd[1] = {__uint_as_float(tail.z)};
        const uint8_t* sbp = tile_smem + (size_t)(hb >> 1) * BPDQ_Q4K_BYTES;
#pragma unroll
        for (int r = 0; r < R; r++)
            if (r < rows) half_block_fma<1, LAYOUT>(sbp + (size_t)r * pb.row_bytes, hb & 1, xr, bs, xd, acc[r], nullptr);
    }
    float v[R];
#pragma unroll
    for (int r = 0; r < R; r++) v[r] = acc[r][0];
    const float total = fold_rows<R>(v, lane);
    constexpr int kLanesPerRow = 32 / R;
    const int my_row = lane / kLanesPerRow;
    // ACC: launches with a residual epilogue are a separate instantiation (the conditional costs the
    // plain product 2 % of its bandwidth); the residual stream was written by an earlier launch: read it past L1
    if ((lane % kLanesPerRow) == 0 && my_row < rows)
        pb.out[row0 + my_row] = (ACC && pb.accumulate) ? __ldcg(pb.out + row0 + my_row) + total : total;
}

// ---- Elementwise steps done by the consumer warps of a product kernel itself (every CTA repeats
// them): the records of the step's result are written to shared memory.  `warp` of `nw` consumer
// warps; barrier 2 is the consumers' named barrier.
//
// rms_norm: the sum of squares is formed exactly as k_rms_norm (decode_ops.cu) forms it with 256
// threads: thread t chains c = t, t+256, ...; butterfly over each warp of 32; the eight warp sums
// added in order.  Consumer warps play those eight warps in turn.
__device__ __forceinline__ void cta_rmsnorm_records(const float* __restrict__ a, const float* __restrict__ w, float eps, int nb,
                                                    uint8_t* xq, float* s_sum, int warp, int lane, int nw)
{
    const int cols = nb * 256;
    for (int vw = warp; vw < 8; vw += nw) {
        float t = 0.0f;
        for (int c = vw * 32 + lane; c < cols; c += 256) {
            const float v = __ldcg(a + c);
            t = fmaf(v, v, t);
        }
        t = warp_sum(t);
        if (lane == 0) s_sum[vw] = t;
    }
    named_bar_sync(2, nw * 32);
    float tot = s_sum[0];
#pragma unroll
    for (int i = 1; i < 8; i++) tot += s_sum[i];
    const float scale = rsqrtf(tot / (float)cols + eps);
    for (int b = warp; b < nb; b += nw) {
        const float4* xb = reinterpret_cast<const float4*>(a + (size_t)b * 256);
        const float4* wb = reinterpret_cast<const float4*>(w + (size_t)b * 256);
        const float4 a0 = __ldcg(xb + lane), a1 = __ldcg(xb + 32 + lane), w0 = __ldg(wb + lane), w1 = __ldg(wb + 32 + lane);
        const float4 v0 = make_float4(a0.x * scale * w0.x, a0.y * scale * w0.y, a0.z * scale * w0.z, a0.w * scale * w0.w);
        const float4 v1 = make_float4(a1.x * scale * w1.x, a1.y * scale * w1.y, a1.z * scale * w1.z, a1.w * scale * w1.w);
        write_records(v0, v1, xq + (size_t)(2 * b) * kXqStride, lane);
    }
}
// silu(gate) * up with k_elementwise's arithmetic
__device__ __forceinline__ void cta_swiglu_records(const float* __restrict__ gate, const float* __restrict__ up, int nb,
                                                   uint8_t* xq, int warp, int lane, int nw)
{
    auto act = [](float g, float u) { return (g / (1.0f + expf(-g))) * u; };
    for (int b = warp; b < nb; b += nw) {
        const float4* gb = reinterpret_cast<const float4*>(gate + (size_t)b * 256);
        const float4* ub = reinterpret_cast<const float4*>(up + (size_t)b * 256);
        const float4 g0 = __ldcg(gb + lane), g1 = __ldcg(gb + 32 + lane), u0 = __ldcg(ub + lane), u1 = __ldcg(ub + 32 + lane);
        const float4 v0 = make_float4(act(g0.x, u0.x), act(g0.y, u0.y), act(g0.z, u0.z), act(g0.w, u0.w));
        const float4 v1 = make_float4(act(g1.x, u1.x), act(g1.y, u1.y), act(g1.z, u1.z), act(g1.w, u1.w));
        write_records(v0, v1, xq + (size_t)(2 * b) * kXqStride, lane);
    }
}
__device__ __forceinline__ void cta_vector_records(const float* __restrict__ x, int nb, uint8_t* xq, int warp, int lane, int nw)
{
    for (int b = warp; b < nb; b += nw) {
        const float4* xb = reinterpret_cast<const float4*>(x + (size_t)b * 256);
        write_records(__ldcg(xb + lane), __ldcg(xb + 32 + lane), xq + (size_t)(2 * b) * kXqStride, lane);
    }
}

template <int FMT, int LAYOUT, int MAXTHREADS, int ACC>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_gemv_batch_q4k_q8k(const BatchPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                 // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                     // activation records
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);    // [nw*slots]
    uint64_t* empty = full + p.nw * p.slots;
    uint64_t* xbar = empty + p.nw * p.slots;                           // activation records have landed

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_producer = (warp == p.nw);
    BPDQ_TRACE(0);
    if (tid == 0) {
        for (int s = 0; s < p.nw * p.slots; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(xbar, 1);
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();
    BPDQ_TRACE(1);

    if (is_producer) {
        if (lane < p.nw) {
            // lane g feeds consumer warp g; weights never depend on the previous kernel
            const int g = lane;
            int slot = 0;
            uint32_t wait_parity = 0;
            bool wrapped = false;
            for (int v = g * (int)gridDim.x + (int)blockIdx.x; v < p.n_tiles; v += p.nw * (int)gridDim.x) {
                const int s = g * p.slots + slot;
                if (wrapped && !mbar_wait_bounded(&empty[s], wait_parity, err, 1)) break;
                int j = 0;
#pragma unroll
                for (int q = 1; q < kMaxBatch; q++)
                    if (q < p.n_problems && v >= p.prob[q].tile_begin) j = q;
                const BatchProblem& pb = p.prob[j];
                const int row0 = (v - pb.tile_begin) * pb.rt;
                const uint32_t bytes = (uint32_t)min(pb.rt, pb.M - row0) * pb.row_bytes;
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(ring + (size_t)s * p.slot_bytes, pb.W + (size_t)row0 * pb.row_bytes, bytes, &full[s]);
                if (++slot == p.slots) {
                    slot = 0;
                    if (wrapped) wait_parity ^= 1u;
                    wrapped = true;
                }
            }
            if (lane == 0) BPDQ_TRACE(7);
        }
        return;
    }

    if (p.records) {
        // Records were written by the quantizer kernel launched just before this one: one thread
        // waits for it (and so for everything earlier in the stream) and pulls them in with one
        // bulk copy; everybody else waits for the bytes.
        if (tid == 0) {
            pdl_wait();
            mbar_expect_tx(xbar, (uint32_t)p.xq_bytes);
            bulk_g2s(xq, p.records, (uint32_t)p.xq_bytes, xbar);
        }
        BPDQ_TRACE(2);
        if (!mbar_wait_bounded(xbar, 0, err, 3)) return;
    } else {
        // Activations may be written by the previous kernel: wait for it before the first read.
        pdl_wait();
        BPDQ_TRACE(2);
        if (p.prologue == 1) {
            cta_rmsnorm_records(p.pro_a, p.pro_b, p.pro_eps, p.vec[0].nb, xq, reinterpret_cast<float*>(xbar + 1), warp, lane, p.nw);
        } else if (p.prologue == 2) {
            cta_swiglu_records(p.pro_a, p.pro_b, p.vec[0].nb, xq, warp, lane, p.nw);
        } else {
        // ---- quantize every activation vector of the launch into shared memory (all consumer warps)
        constexpr int UNR = 4;
        for (int blk0 = warp; blk0 < p.total_blocks; blk0 += p.nw * UNR) {
            float4 v0[UNR], v1[UNR];
            int vb[UNR], vq[UNR];
#pragma unroll
            for (int u = 0; u < UNR; u++) {
                int blk = blk0 + u * p.nw;
                vb[u] = -1;
                if (blk < p.total_blocks) {
                    // every CTA reads the same vectors: start each one at a different block so
                    // that the SMs do not all ask the same L2 lines at the same moment
                    blk = (blk + (int)blockIdx.x * 5) % p.total_blocks;
                    int k = 0;
                    while (k + 1 < p.n_vectors && blk >= p.vec[k].nb) { blk -= p.vec[k].nb; k++; }
                    const float4* xb = reinterpret_cast<const float4*>(p.vec[k].x + (size_t)blk * 256);
                    v0[u] = __ldcg(xb + lane);      // may be the output of the launch before this one
                    v1[u] = __ldcg(xb + 32 + lane);
                    vb[u] = blk;
                    vq[u] = p.vec[k].xq_off;
                }
            }
#pragma unroll
            for (int u = 0; u < UNR; u++) {
                if (vb[u] < 0) continue;
                if (FMT == 0) write_records(v0[u], v1[u], xq + vq[u] + (size_t)(2 * vb[u]) * kXqStride, lane);
                else write_records_q80(v0[u], v1[u], xq + vq[u] + (size_t)(4 * vb[u]) * kQ80PairStride, lane);
            }
        }
        }
        named_bar_sync(2, p.nw * 32);
    }
    BPDQ_TRACE(3);

    int slot = 0;
    uint32_t parity = 0;
    bool first = true;
    for (int v = warp * (int)gridDim.x + (int)blockIdx.x; v < p.n_tiles; v += p.nw * (int)gridDim.x) {
        const int s = warp * p.slots + slot;
        if (!mbar_wait_bounded(&full[s], parity, err, 2)) return;
        if (first) { BPDQ_TRACE(5); first = false; }
        if (++slot == p.slots) {
            slot = 0;
            parity ^= 1u;
        }
        int j = 0;
#pragma unroll
        for (int q = 1; q < kMaxBatch; q++)
            if (q < p.n_problems && v >= p.prob[q].tile_begin) j = q;
        const BatchProblem& pb = p.prob[j];
        const int row0 = (v - pb.tile_begin) * pb.rt;
        const uint8_t* tile_smem = ring + (size_t)s * p.slot_bytes;
        if (FMT == 0) {
            if (pb.rt == 4) batch_tile<4, LAYOUT, ACC>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else if (pb.rt == 2) batch_tile<2, LAYOUT, ACC>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else batch_tile<1, LAYOUT, ACC>(tile_smem, xq + pb.xq_off, pb, row0, lane);
        } else {
            if (pb.rt == 4) batch_tile_q80<4>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else if (pb.rt == 2) batch_tile_q80<2>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else batch_tile_q80<1>(tile_smem, xq + pb.xq_off, pb, row0, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    BPDQ_TRACE(6);
}

struct BatchDesc {
    const uint8_t* W;
    const float* x;
    float* out;
    int M, K;
};

// Builds the launch plan for descs[0..n); returns BPDQ_ERR_RANGE when the set does not fit one
// launch (too many activations for shared memory, or rows longer than a ring slot).
static int make_batch_plan(const BatchDesc* d, int n, BatchPlan& p, int fmt = 0)
{
    if (n < 1 || n > kMaxBatch) return BPDQ_ERR_RANGE;
    const Tuning& tu = tuning();
    const int slot_cap = 32 * 1024;
    p.n_problems = n;
    p.n_vectors = 0;
    p.n_tiles = 0;
    p.total_blocks = 0;
    p.slot_bytes = 0;
    p.trace = nullptr;
    p.records = nullptr;
    p.prologue = 0;
    p.pro_a = p.pro_b = nullptr;
    p.pro_eps = 0.0f;
    int xq_bytes = 0;
    // Rows per tile: as many as fit tile_bytes (1, 2 or 4).  A launch with a lot of work gets a
    // slightly larger budget, 4 rows of K = 4096 (9216 bytes): the per-tile work of a consumer warp
    // (barrier wait, record loads, fold, store) is then spread over four rows, worth 8 % of bandwidth
    // on a 123 MB layer, while a small launch keeps the smaller tiles that balance better over the SMs.
    size_t launch_bytes = 0;
    for (int j = 0; j < n; j++)
        if (d[j].M > 0 && d[j].K > 0)
            launch_bytes += (size_t)d[j].M * (fmt == 0 ? d[j].K / 256 * BPDQ_Q4K_BYTES : d[j].K / 32 * BPDQ_Q80_BYTES);
    const int tile_budget = (launch_bytes >= (fmt == 0 ? kBigLaunchBytes : kBigLaunchBytesQ80) && tu.tile_bytes < kBigLaunchTileBytes)
                                ? kBigLaunchTileBytes : tu.tile_bytes;
    for (int j = 0; j < n; j++) {
        if (d[j].M <= 0 || d[j].K <= 0 || (d[j].K % 256) != 0) return BPDQ_ERR_ARG;
        BatchProblem& pb = p.prob[j];
        pb.W = d[j].W;
        pb.out = d[j].out;
        pb.accumulate = 0;
        pb.M = d[j].M;
        pb.nb = d[j].K / 256;
        pb.row_bytes = fmt == 0 ? pb.nb * BPDQ_Q4K_BYTES : pb.nb * 8 * BPDQ_Q80_BYTES;
        if (pb.row_bytes > slot_cap) return BPDQ_ERR_RANGE;
        pb.rt = 4 * pb.row_bytes <= tile_budget ? 4 : (2 * pb.row_bytes <= tile_budget ? 2 : 1);
        if (pb.rt * pb.row_bytes > p.slot_bytes) p.slot_bytes = pb.rt * pb.row_bytes;
        pb.tile_begin = p.n_tiles;
        p.n_tiles += (pb.M + pb.rt - 1) / pb.rt;
        int k = 0;
        for (; k < p.n_vectors; k++)
            if (p.vec[k].x == d[j].x && p.vec[k].nb == pb.nb) break;
        if (k == p.n_vectors) {
            p.vec[k].x = d[j].x;
            p.vec[k].nb = pb.nb;
            p.vec[k].xq_off = xq_bytes;
            xq_bytes += fmt == 0 ? 2 * pb.nb * kXqStride : 4 * pb.nb * kQ80PairStride;
            p.total_blocks += pb.nb;
            p.n_vectors++;
        }
        pb.xq_off = p.vec[k].xq_off;
    }
    for (int j = n; j < kMaxBatch; j++) {
        p.prob[j] = p.prob[0];
        p.prob[j].tile_begin = 0x7FFFFFFF;
    }
    for (int k = p.n_vectors; k < kMaxBatch; k++) p.vec[k] = p.vec[0];
    p.xq_bytes = xq_bytes;
    p.slots = tu.stages < 2 ? 2 : tu.stages;
    p.nw = tu.warps < 1 ? 1 : (tu.warps > 16 ? 16 : tu.warps);
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_xq = take((size_t)xq_bytes);
        p.off_bar = take((size_t)2 * p.nw * p.slots * 8 + 8 + 64);   // barriers, then nine floats of the rms_norm prologue
        p.smem = off;
        if (p.smem <= (size_t)kSmemLimit) break;
        if (p.slots > 2) p.slots--;
        else if (p.nw > 4) p.nw--;
        else return BPDQ_ERR_RANGE;
    }
    long want = (p.n_tiles + p.nw - 1) / p.nw;
    if (want < 1) want = 1;
    p.grid = (int)(want < sm_count() ? want : sm_count());
    return 0;
}

template <int FMT, int LAYOUT, int ACC = 0>
static int launch_batch(const BatchPlan& p, cudaStream_t s)
{
    if (ACC == 0) {
        for (int j = 0; j < p.n_problems; j++)
            if (p.prob[j].accumulate) return launch_batch<FMT, LAYOUT, 1>(p, s);
    }
    auto kern = k_gemv_batch_q4k_q8k<FMT, LAYOUT, kMidCtaThreads, ACC>;
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
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p, device_error_flag()));
}

static int launch_quant_records(const BatchPlan& p, uint8_t* records, int wait_first, cudaStream_t s)
{
    QuantVectors q;
    q.n_vectors = p.n_vectors;
    q.total_blocks = p.total_blocks;
    for (int k = 0; k < kMaxBatch; k++) q.vec[k] = p.vec[k];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.total_blocks + 7) / 8);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, k_quant_records<0>, q, records, wait_first));
}

// Independent GEMVs: as many launches as needed, each covering as many consecutive
// descriptors as fit; a product that does not fit the batched kernel at all (K > 58254) runs
// through the single-matrix kernel.
//
// ws / ws_bytes: optional scratch for the quantized activation records (144 bytes per 128
// activations of every distinct vector of a launch).  With scratch, a small kernel quantizes
// the activations once and the GEMV kernel bulk-copies the records; without it every CTA of the
// GEMV kernel quantizes them itself.  ws_private: the caller promises that no earlier launch
// still reads this scratch, so the quantizer need not wait for the stream before writing it.
int gemv_q4k_q8k_batch(const BatchDesc* d, int n, int layout, uint8_t* ws, size_t ws_bytes, int ws_private,
                       cudaStream_t s)
{
    if (n < 0 || (n > 0 && !d)) return latch(BPDQ_ERR_ARG);
    if (ws && ((uintptr_t)ws & 15)) return latch(BPDQ_ERR_ALIGN);
    for (int j = 0; j < n; j++) {
        if (d[j].M < 0 || d[j].K <= 0 || (d[j].K % 256) != 0) return latch(BPDQ_ERR_ARG);
        if (d[j].M > 0 && (!d[j].W || !d[j].x || !d[j].out)) return latch(BPDQ_ERR_ARG);
        if (((uintptr_t)d[j].W & 15) || ((uintptr_t)d[j].x & 15) || ((uintptr_t)d[j].out & 3)) return latch(BPDQ_ERR_ALIGN);
    }
    int i = 0;
    size_t ws_used = 0;
    while (i < n) {
        if (d[i].M == 0) { i++; continue; }
        // longest run starting at i that fits one launch
        BatchDesc run[kMaxBatch];
        BatchPlan plan, good;
        int len = 0;
        while (i + len < n && len < kMaxBatch && d[i + len].M > 0) {
            run[len] = d[i + len];
            if (make_batch_plan(run, len + 1, plan) != 0) break;
            // do not let a long run squeeze the consumer warps out of shared memory: split instead
            if (len > 0 && plan.nw < (tuning().warps < 8 ? tuning().warps : 8)) break;
            good = plan;
            len++;
        }
        if (len == 0) {
            int rc = gemm_q4k_q8k(d[i].W, d[i].x, d[i].out, 1, d[i].M, d[i].K, layout, 0, nullptr, s);
            if (rc) return rc;
            i++;
            continue;
        }
        if (ws && ws_used + (size_t)good.xq_bytes <= ws_bytes) {
            uint8_t* rec = ws + ws_used;
            ws_used += ((size_t)good.xq_bytes + 127) / 128 * 128;
            int rc = launch_quant_records(good, rec, ws_private ? 0 : 1, s);
            if (rc) return latch(rc);
            good.records = rec;
        }
        if (g_trace_base && g_trace_left > 0) {
            good.trace = g_trace_base;
            g_trace_base += g_trace_stride;
            g_trace_left--;
        }
        int rc = layout == BPDQ_LAYOUT_GGML ? launch_batch<0, BPDQ_LAYOUT_GGML>(good, s) : launch_batch<0, BPDQ_LAYOUT_BPD>(good, s);
        if (rc) return latch(rc);
        i += len;
    }
    return 0;
}

// Products over records that an earlier launch wrote (k_rmsnorm_records, k_swiglu_records,
// k_vector_records): up to kMaxBatch matrices with the same K sharing one record vector, one
// launch.  Bit j of accumulate_mask: out_j[row] += result (the residual connection).
int gemv_q4k_records(const BatchDesc* d, int n, const uint8_t* records, unsigned accumulate_mask, int layout, cudaStream_t s)
{
    if (n < 1 || n > kMaxBatch || !d || !records) return latch(BPDQ_ERR_ARG);
    if ((uintptr_t)records & 15) return latch(BPDQ_ERR_ALIGN);
    BatchDesc run[kMaxBatch];
    for (int j = 0; j < n; j++) {
        if (d[j].M <= 0 || d[j].K <= 0 || (d[j].K % 256) != 0 || d[j].K != d[0].K) return latch(BPDQ_ERR_ARG);
        if (!d[j].W || !d[j].out) return latch(BPDQ_ERR_ARG);
        if (((uintptr_t)d[j].W & 15) || ((uintptr_t)d[j].out & 3)) return latch(BPDQ_ERR_ALIGN);
        run[j] = d[j];
        run[j].x = reinterpret_cast<const float*>(records);   // one shared vector: identical key for the planner
    }
    BatchPlan plan;
    int rc = make_batch_plan(run, n, plan);
    if (rc) return latch(rc);
    plan.records = records;
    for (int j = 0; j < n; j++) plan.prob[j].accumulate = (accumulate_mask >> j) & 1u;
    rc = layout == BPDQ_LAYOUT_GGML ? launch_batch<0, BPDQ_LAYOUT_GGML>(plan, s) : launch_batch<0, BPDQ_LAYOUT_BPD>(plan, s);
    return rc ? latch(rc) : 0;
}

// One launch for "elementwise step, quantize, products, residual add": the CTAs of the product
// kernel apply the step to the single input vector themselves (each CTA redundantly: the vector is
// 16-56 KB and comes from L2) while their producer warp is already filling the weight ring.
// prologue 0: records of a;  1: records of rms_norm(a, weights b, eps);  2: records of silu(a) * b.
int gemv_q4k_fused(const BatchDesc* d, int n, int prologue, const float* a, const float* b, float eps,
                   unsigned accumulate_mask, int layout, cudaStream_t s)
{
    if (n < 1 || n > kMaxBatch || !d || !a || prologue < 0 || prologue > 2 || (prologue && !b)) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)a & 15) || (b && ((uintptr_t)b & 15))) return latch(BPDQ_ERR_ALIGN);
    BatchDesc run[kMaxBatch];
    for (int j = 0; j < n; j++) {
        if (d[j].M <= 0 || d[j].K <= 0 || (d[j].K % 256) != 0 || d[j].K != d[0].K) return latch(BPDQ_ERR_ARG);
        if (!d[j].W || !d[j].out) return latch(BPDQ_ERR_ARG);
        if (((uintptr_t)d[j].W & 15) || ((uintptr_t)d[j].out & 3)) return latch(BPDQ_ERR_ALIGN);
        run[j] = d[j];
        run[j].x = a;
    }
    BatchPlan plan;
    int rc = make_batch_plan(run, n, plan);
    if (rc) return latch(rc);
    plan.prologue = prologue;
    plan.pro_a = a;
    plan.pro_b = b;
    plan.pro_eps = eps;
    for (int j = 0; j < n; j++) plan.prob[j].accumulate = (accumulate_mask >> j) & 1u;
    rc = layout == BPDQ_LAYOUT_GGML ? launch_batch<0, BPDQ_LAYOUT_GGML>(plan, s) : launch_batch<0, BPDQ_LAYOUT_BPD>(plan, s);
    return rc ? latch(rc) : 0;
}

// ---- Persistent decode chain: ONE cooperative launch walks a whole program of dependent phases
// (per decoder layer: rms_norm -> q,k,v | q -> o, += x | rms_norm -> gate,up | silu(gate)*up -> down, += x).
// The weights of a phase do not depend on the phase before it, so the producer warp streams the
// tiles of all phases back to back into the ring and HBM never waits for a launch boundary; only
// the consumer warps wait, at a grid-wide barrier between phases (one counter per phase: every CTA
// adds one when its rows are written and fenced, thread 0 of every CTA polls with an acquire load,
// bounded), then rebuild the phase's activation records in shared memory from the vector the
// previous phase produced.  A cooperative launch keeps all CTAs resident, which the barrier needs.
constexpr int kChainMaxProblems = 3;
struct ChainPhase {
    int n_problems, prologue, nb, n_tiles;   // prologue as in BatchPlan: 0 records of a, 1 rms_norm(a, b, eps), 2 silu(a)*b
    const float* a;
    const float* b;
    float eps;
    int pad;
    BatchProblem prob[kChainMaxProblems];
};
struct ChainPlan {
    const ChainPhase* phases;   // device array
    unsigned* arrive;           // [n_phases] grid-barrier counters, zero at launch
    int n_phases;
    int nw, slots, slot_bytes;
    int off_ring, off_xq, off_bar;
    size_t smem;
    unsigned long long* trace;  // tuning aid: SM-clock stamps of CTA 0, [phase < 64][4], or null
};
#define CHAIN_TRACE(ph, k)                                                                     \
    do {                                                                                       \
        if (p.trace && blockIdx.x == 0 && tid == 0 && (ph) < 64) p.trace[(ph) * 4 + (k)] = clock64(); \
    } while (0)

template <int LAYOUT, int MAXTHREADS>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_decode_chain(const ChainPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                 // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                     // activation records of the current phase
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);    // [nw*slots]
    uint64_t* empty = full + p.nw * p.slots;
    float* s_sum = reinterpret_cast<float*>(empty + p.nw * p.slots);   // nine floats of the rms_norm step
    volatile int* dead = reinterpret_cast<volatile int*>(s_sum + 12);  // a wait gave up: everybody leaves at the next barrier

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = p.nw, grid = (int)gridDim.x;
    if (tid == 0) {
        for (int s = 0; s < nw * p.slots; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *dead = 0;
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == nw) {
        // ---- producer: lane g feeds consumer warp g, phase after phase without a pause
        if (lane < nw) {
            const int g = lane;
            int slot = 0;
            uint32_t wait_parity = 0;
            bool wrapped = false;
            for (int ph = 0; ph < p.n_phases; ph++) {
                const ChainPhase& P = p.phases[ph];
                const int n_tiles = P.n_tiles, n_prob = P.n_problems;
                for (int v = g * grid + (int)blockIdx.x; v < n_tiles; v += nw * grid) {
                    const int s = g * p.slots + slot;
                    if (wrapped && !mbar_wait_bounded(&empty[s], wait_parity, err, 23)) return;
                    int j = 0;
#pragma unroll
                    for (int q = 1; q < kChainMaxProblems; q++)
                        if (q < n_prob && v >= P.prob[q].tile_begin) j = q;
                    const BatchProblem& pb = P.prob[j];
                    const int row0 = (v - pb.tile_begin) * pb.rt;
                    const uint32_t bytes = (uint32_t)min(pb.rt, pb.M - row0) * pb.row_bytes;
                    mbar_expect_tx(&full[s], bytes);
                    bulk_g2s(ring + (size_t)s * p.slot_bytes, pb.W + (size_t)row0 * pb.row_bytes, bytes, &full[s]);
                    if (++slot == p.slots) {
                        slot = 0;
                        if (wrapped) wait_parity ^= 1u;
                        wrapped = true;
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();   // the first phase's input vector comes from whatever ran before this launch
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < p.n_phases; ph++) {
        const ChainPhase& P = p.phases[ph];
        if (ph > 0) {
            // grid-wide barrier: every CTA has written and fenced the rows of phase ph-1
            if (tid == 0) {
                bool ok = false;
                for (uint32_t it = 0; it < (1u << 22); it++) {
                    unsigned seen;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.arrive + ph - 1) : "memory");
                    if (seen >= (unsigned)grid) { ok = true; break; }
                    if ((it & 255u) == 255u && *reinterpret_cast<volatile int*>(err) != 0) break;
                    __nanosleep(20);
                }
                if (!ok) {
                    atomicCAS(err, 0, 21);
                    *dead = 1;
                }
            }
            named_bar_sync(3, nw * 32);
            if (*dead) break;
        }
        CHAIN_TRACE(ph, 0);
        // ---- the phase's activation records
        if (P.prologue == 1) cta_rmsnorm_records(P.a, P.b, P.eps, P.nb, xq, s_sum, warp, lane, nw);
        else if (P.prologue == 2) cta_swiglu_records(P.a, P.b, P.nb, xq, warp, lane, nw);
        else cta_vector_records(P.a, P.nb, xq, warp, lane, nw);
        named_bar_sync(2, nw * 32);
        CHAIN_TRACE(ph, 1);
        // ---- this warp's tiles of the phase
        const int n_tiles = P.n_tiles, n_prob = P.n_problems;
        for (int v = warp * grid + (int)blockIdx.x; v < n_tiles; v += nw * grid) {
            const int s = warp * p.slots + slot;
            if (!mbar_wait_bounded(&full[s], parity, err, 22)) {
                *dead = 1;
                break;
            }
            if (++slot == p.slots) {
                slot = 0;
                parity ^= 1u;
            }
            int j = 0;
#pragma unroll
            for (int q = 1; q < kChainMaxProblems; q++)
                if (q < n_prob && v >= P.prob[q].tile_begin) j = q;
            const BatchProblem& pb = P.prob[j];
            const int row0 = (v - pb.tile_begin) * pb.rt;
            const uint8_t* tile_smem = ring + (size_t)s * p.slot_bytes;
            if (pb.rt == 4) batch_tile<4, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            else if (pb.rt == 2) batch_tile<2, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            else batch_tile<1, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        // ---- publish: rows written by this CTA are visible device-wide before its arrival counts
        CHAIN_TRACE(ph, 2);
        __threadfence();
        named_bar_sync(2, nw * 32);
        if (*dead) break;
        if (tid == 0) atomicAdd(p.arrive + ph, 1u);
        CHAIN_TRACE(ph, 3);
    }
}

struct ChainHandle {
    ChainPlan plan;
    ChainPhase* d_phases;
    unsigned* d_arrive;
    int device;
};

// Host side of the persistent chain: the program is planned and uploaded once, then launched per token.
struct ChainPhaseDesc {          // mirrors bpdq_chain_phase of the header
    int n, prologue;
    const float* a;
    const float* b;
    float eps;
    unsigned accumulate_mask;
    BatchDesc prod[kChainMaxProblems];
};

static ChainHandle* chain_create(int n_phases, const ChainPhaseDesc* ph)
{
    if (n_phases < 1 || !ph) { latch(BPDQ_ERR_ARG); return nullptr; }
    const Tuning& tu = tuning();
    std::vector<ChainPhase> prog((size_t)n_phases);
    int slot_bytes = 0, xq_bytes = 0;
    for (int i = 0; i < n_phases; i++) {
        const ChainPhaseDesc& d = ph[i];
        ChainPhase& P = prog[i];
        if (d.n < 1 || d.n > kChainMaxProblems || d.prologue < 0 || d.prologue > 2 || !d.a || (d.prologue && !d.b) ||
            ((uintptr_t)d.a & 15) || ((uintptr_t)d.b & 15)) { latch(BPDQ_ERR_ARG); return nullptr; }
        P.n_problems = d.n;
        P.prologue = d.prologue;
        P.a = d.a;
        P.b = d.b;
        P.eps = d.eps;
        P.pad = 0;
        P.n_tiles = 0;
        const int K = d.prod[0].K;
        if (K <= 0 || (K % 256) != 0) { latch(BPDQ_ERR_ARG); return nullptr; }
        P.nb = K / 256;
        size_t phase_bytes = 0;
        for (int j = 0; j < d.n; j++) phase_bytes += (size_t)(d.prod[j].M > 0 ? d.prod[j].M : 0) * P.nb * BPDQ_Q4K_BYTES;
        const int tile_budget = (phase_bytes >= kBigLaunchBytes && tu.tile_bytes < kBigLaunchTileBytes) ? kBigLaunchTileBytes : tu.tile_bytes;
        for (int j = 0; j < kChainMaxProblems; j++) {
            const BatchDesc& q = d.prod[j < d.n ? j : 0];
            BatchProblem& pb = P.prob[j];
            if (j < d.n && (q.M <= 0 || q.K != K || !q.W || !q.out || ((uintptr_t)q.W & 15) || ((uintptr_t)q.out & 3))) {
                latch(BPDQ_ERR_ARG);
                return nullptr;
            }
            pb.W = q.W;
            pb.out = q.out;
            pb.M = q.M;
            pb.nb = P.nb;
            pb.row_bytes = P.nb * BPDQ_Q4K_BYTES;
            if (pb.row_bytes > 32 * 1024) { latch(BPDQ_ERR_RANGE); return nullptr; }
            pb.rt = 4 * pb.row_bytes <= tile_budget ? 4 : (2 * pb.row_bytes <= tile_budget ? 2 : 1);
            pb.xq_off = 0;
            pb.accumulate = (j < d.n) ? (int)((d.accumulate_mask >> j) & 1u) : 0;
            if (j < d.n) {
                pb.tile_begin = P.n_tiles;
                P.n_tiles += (pb.M + pb.rt - 1) / pb.rt;
                if (pb.rt * pb.row_bytes > slot_bytes) slot_bytes = pb.rt * pb.row_bytes;
            } else {
                pb.tile_begin = 0x7FFFFFFF;
            }
        }
        if (2 * P.nb * kXqStride > xq_bytes) xq_bytes = 2 * P.nb * kXqStride;
    }
    ChainHandle* h = new ChainHandle();
    ChainPlan& p = h->plan;
    p.n_phases = n_phases;
    p.slot_bytes = slot_bytes;
    p.slots = tu.stages < 2 ? 2 : tu.stages;
    p.nw = tu.warps < 1 ? 1 : (tu.warps > 16 ? 16 : tu.warps);
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_xq = take((size_t)xq_bytes);
        p.off_bar = take((size_t)2 * p.nw * p.slots * 8 + 64);
        p.smem = off;
        if (p.smem <= (size_t)kSmemLimit) break;
        if (p.slots > 2) p.slots--;
        else if (p.nw > 4) p.nw--;
        else { delete h; latch(BPDQ_ERR_RANGE); return nullptr; }
    }
    cudaGetDevice(&h->device);
    void* dp = nullptr;
    void* da = nullptr;
    if (check_cuda(cudaMalloc(&dp, sizeof(ChainPhase) * (size_t)n_phases)) || check_cuda(cudaMalloc(&da, sizeof(unsigned) * (size_t)n_phases)) ||
        check_cuda(cudaMemcpy(dp, prog.data(), sizeof(ChainPhase) * (size_t)n_phases, cudaMemcpyHostToDevice))) {
        if (dp) cudaFree(dp);
        if (da) cudaFree(da);
        delete h;
        latch(BPDQ_ERR_CUDA);
        return nullptr;
    }
    h->d_phases = (ChainPhase*)dp;
    h->d_arrive = (unsigned*)da;
    p.phases = h->d_phases;
    p.arrive = h->d_arrive;
    p.trace = nullptr;
    return h;
}

static int chain_run(ChainHandle* h, cudaStream_t s)
{
    if (!h) return latch(BPDQ_ERR_ARG);
    auto kern = k_decode_chain<BPDQ_LAYOUT_BPD, kMidCtaThreads>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != h->device) return latch(BPDQ_ERR_ARG);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        if (rc) return latch(rc);
        attr_set[dev] = true;
    }
    int rc = check_cuda(cudaMemsetAsync(h->d_arrive, 0, sizeof(unsigned) * (size_t)h->plan.n_phases, s));
    if (rc) return latch(rc);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count());     // one CTA per SM, all resident: the barrier between phases needs that
    cfg.blockDim = dim3((unsigned)(h->plan.nw + 1) * 32);
    cfg.dynamicSmemBytes = h->plan.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    ChainPlan plan = h->plan;
    plan.trace = nullptr;
    if (g_trace_base && g_trace_left > 0) {
        plan.trace = g_trace_base;
        g_trace_base += g_trace_stride;
        g_trace_left--;
    }
    rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, plan, device_error_flag()));
    return rc ? latch(rc) : 0;
}

static void chain_destroy(ChainHandle* h)
{
    if (!h) return;
    cudaFree(h->d_phases);
    cudaFree(h->d_arrive);
    delete h;
}

template <typename Kern, typename... Args>
static int launch_glue(Kern kern, int grid, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, args...));
}

static int glue_grid(long n_blocks)
{
    long want = (n_blocks + 7) / 8, cap = (long)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

// ---- Stream of independent products: ONE persistent launch for any number of them.
// The batched kernel above covers up to kMaxBatch products; a step of the benchmark has 224, i.e. 32
// launches, and each launch boundary drains the weight ring: the SM idles from its CTA's last tile
// until the next launch's first tile has arrived.  Here the products are cut into phases (as many
// consecutive products as the shared-memory record buffer holds), the producer warp streams the tiles
// of all phases back to back, and the consumer warps only pause between phases to swap the
// activation records (a CTA-local barrier and one pass over <= 48 KB from L2).  All activation vectors
// are quantized beforehand by one launch of k_quant_records_table.  No CTA waits for another.
struct StreamPhase {            // device program entry
    int n_problems, n_tiles, rec_bytes, pad;
    const uint8_t* records;     // this phase's activation records in global scratch (16-byte aligned)
    long long pad2;
    BatchProblem prob[kMaxBatch];
};
static_assert(sizeof(StreamPhase) % 16 == 0, "phase descriptors are copied in 16-byte pieces");
struct StreamPlan {
    const StreamPhase* phases;
    int n_phases;
    int nw, slots, slot_bytes;
    int off_ring, off_xq, off_desc, off_bar;
    size_t smem;
};
struct VecEntry {               // one distinct activation vector of a stream
    const float* x;
    int nb, block_begin;        // 256-blocks of this vector, index of its first block among all
    size_t rec_off;             // byte offset of its records in the scratch
};

__global__ void __launch_bounds__(256) k_quant_records_table(const VecEntry* __restrict__ table, int n_vec, int total_blocks,
                                                              uint8_t* __restrict__ records)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    for (int b = warp; b < total_blocks; b += n_warps) {
        int lo = 0, hi = n_vec - 1;          // last entry whose block_begin <= b
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (table[mid].block_begin <= b) lo = mid;
            else hi = mid - 1;
        }
        const VecEntry e = table[lo];
        const int blk = b - e.block_begin;
        const float4* xb = reinterpret_cast<const float4*>(e.x + (size_t)blk * 256);
        write_records(__ldcg(xb + lane), __ldcg(xb + 32 + lane), records + e.rec_off + (size_t)(2 * blk) * kXqStride, lane);
    }
}

template <int LAYOUT, int MAXTHREADS>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_gemv_stream_q4k_q8k(const StreamPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                 // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                     // activation records of the consumers' phase
    StreamPhase* desc_p = reinterpret_cast<StreamPhase*>(smem + p.off_desc);   // the producer's phase
    StreamPhase* desc_c = desc_p + 1;                                           // the consumers' phase
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);    // [nw*slots]
    uint64_t* empty = full + p.nw * p.slots;
    volatile int* dead = reinterpret_cast<volatile int*>(empty + p.nw * p.slots);   // a wait gave up: leave at the next barrier

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = p.nw, grid = (int)gridDim.x;
    constexpr int kDescWords = sizeof(StreamPhase) / 16;
    if (tid == 0) {
        for (int s = 0; s < nw * p.slots; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *dead = 0;
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == nw) {
        // ---- producer: lane g feeds consumer warp g; weights never depend on the launch before
        int slot = 0;
        uint32_t wait_parity = 0;
        bool wrapped = false, ok = true;
        for (int ph = 0; ph < p.n_phases; ph++) {
            __syncwarp();
            for (int w = lane; w < kDescWords; w += 32)
                reinterpret_cast<uint4*>(desc_p)[w] = __ldg(reinterpret_cast<const uint4*>(p.phases + ph) + w);
            __syncwarp();
            if (lane < nw && ok) {
                const int g = lane;
                for (int v = g * grid + (int)blockIdx.x; v < desc_p->n_tiles; v += nw * grid) {
                    const int s = g * p.slots + slot;
                    if (wrapped && !mbar_wait_bounded(&empty[s], wait_parity, err, 1)) { ok = false; break; }
                    int j = 0;
#pragma unroll
                    for (int q = 1; q < kMaxBatch; q++)
                        if (q < desc_p->n_problems && v >= desc_p->prob[q].tile_begin) j = q;
                    const BatchProblem& pb = desc_p->prob[j];
                    const int row0 = (v - pb.tile_begin) * pb.rt;
                    const uint32_t bytes = (uint32_t)min(pb.rt, pb.M - row0) * pb.row_bytes;
                    mbar_expect_tx(&full[s], bytes);
                    bulk_g2s(ring + (size_t)s * p.slot_bytes, pb.W + (size_t)row0 * pb.row_bytes, bytes, &full[s]);
                    if (++slot == p.slots) {
                        slot = 0;
                        if (wrapped) wait_parity ^= 1u;
                        wrapped = true;
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();   // the records come from the quantizer launched just before
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < p.n_phases; ph++) {
        // everybody has finished the previous phase: descriptor and records may be replaced
        named_bar_sync(2, nw * 32);
        if (*dead) break;
        if (warp == 0)
            for (int w = lane; w < kDescWords; w += 32)
                reinterpret_cast<uint4*>(desc_c)[w] = __ldg(reinterpret_cast<const uint4*>(p.phases + ph) + w);
        {
            const StreamPhase* gp = p.phases + ph;
            const int n16 = gp->rec_bytes >> 4;
            const uint4* src = reinterpret_cast<const uint4*>(gp->records);
            for (int w = tid; w < n16; w += nw * 32) reinterpret_cast<uint4*>(xq)[w] = __ldcg(src + w);
        }
        named_bar_sync(2, nw * 32);
        const int n_tiles = desc_c->n_tiles, n_prob = desc_c->n_problems;
        for (int v = warp * grid + (int)blockIdx.x; v < n_tiles; v += nw * grid) {
            const int s = warp * p.slots + slot;
            if (!mbar_wait_bounded(&full[s], parity, err, 2)) {
                *dead = 1;      // keep meeting the others at the barriers; everybody leaves at the next one
                break;
            }
            if (++slot == p.slots) {
                slot = 0;
                parity ^= 1u;
            }
            int j = 0;
#pragma unroll
            for (int q = 1; q < kMaxBatch; q++)
                if (q < n_prob && v >= desc_c->prob[q].tile_begin) j = q;
            const BatchProblem& pb = desc_c->prob[j];
            const int row0 = (v - pb.tile_begin) * pb.rt;
            const uint8_t* tile_smem = ring + (size_t)s * p.slot_bytes;
            if (pb.rt == 4) batch_tile<4, LAYOUT, 0>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else if (pb.rt == 2) batch_tile<2, LAYOUT, 0>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else batch_tile<1, LAYOUT, 0>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
    }
}

struct StreamHandle {
    StreamPlan plan;
    StreamPhase* d_phases;
    VecEntry* d_table;
    uint8_t* records;
    int n_vec, total_blocks, device;
};

// Plans `n` independent products as phases of consecutive products (at most kMaxBatch per phase and
// at most kStreamXqBytes of activation records), lays their records out in `ws` and uploads the program.
constexpr int kStreamXqBytes = 48 * 1024;
static StreamHandle* stream_create(int n, const BatchDesc* d, uint8_t* ws, size_t ws_bytes)
{
    if (n < 1 || !d || !ws || ((uintptr_t)ws & 15)) { latch(BPDQ_ERR_ARG); return nullptr; }
    const Tuning& tu = tuning();
    std::vector<StreamPhase> prog;
    std::vector<VecEntry> table;
    int slot_bytes = 0, xq_max = 0, total_blocks = 0;
    size_t ws_used = 0;
    size_t stream_bytes = 0;
    for (int j = 0; j < n; j++)
        if (d[j].M > 0 && d[j].K > 0) stream_bytes += (size_t)d[j].M * (d[j].K / 256) * BPDQ_Q4K_BYTES;
    const int tile_budget = (stream_bytes >= kBigLaunchBytes && tu.tile_bytes < kBigLaunchTileBytes) ? kBigLaunchTileBytes : tu.tile_bytes;
    int i = 0;
    while (i < n) {
        StreamPhase P;
        memset(&P, 0, sizeof(P));
        const size_t vec_first = table.size();
        int xq_bytes = 0;
        while (i < n && P.n_problems < kMaxBatch) {
            const BatchDesc& q = d[i];
            if (q.M <= 0 || q.K <= 0 || (q.K % 256) != 0 || !q.W || !q.x || !q.out) { latch(BPDQ_ERR_ARG); return nullptr; }
            if (((uintptr_t)q.W & 15) || ((uintptr_t)q.x & 15) || ((uintptr_t)q.out & 3)) { latch(BPDQ_ERR_ALIGN); return nullptr; }
            const int nb = q.K / 256, row_bytes = nb * BPDQ_Q4K_BYTES;
            if (row_bytes > 32 * 1024) { latch(BPDQ_ERR_RANGE); return nullptr; }
            size_t k = vec_first;
            for (; k < table.size(); k++)
                if (table[k].x == q.x && table[k].nb == nb) break;
            const int add = k == table.size() ? 2 * nb * kXqStride : 0;
            if (P.n_problems > 0 && xq_bytes + add > kStreamXqBytes) break;
            if (add > kStreamXqBytes) { latch(BPDQ_ERR_RANGE); return nullptr; }
            if (k == table.size()) {
                VecEntry e;
                e.x = q.x;
                e.nb = nb;
                e.block_begin = total_blocks;
                e.rec_off = ws_used + (size_t)xq_bytes;
                table.push_back(e);
                total_blocks += nb;
            }
            BatchProblem& pb = P.prob[P.n_problems];
            pb.W = q.W;
            pb.out = q.out;
            pb.M = q.M;
            pb.nb = nb;
            pb.row_bytes = row_bytes;
            pb.rt = 4 * row_bytes <= tile_budget ? 4 : (2 * row_bytes <= tile_budget ? 2 : 1);
            pb.tile_begin = P.n_tiles;
            pb.xq_off = (int)(table[k].rec_off - ws_used);
            pb.accumulate = 0;
            P.n_tiles += (pb.M + pb.rt - 1) / pb.rt;
            if (pb.rt * row_bytes > slot_bytes) slot_bytes = pb.rt * row_bytes;
            xq_bytes += add;
            P.n_problems++;
            i++;
        }
        for (int j = P.n_problems; j < kMaxBatch; j++) {
            P.prob[j] = P.prob[0];
            P.prob[j].tile_begin = 0x7FFFFFFF;
        }
        P.rec_bytes = xq_bytes;
        P.records = ws + ws_used;
        ws_used += ((size_t)xq_bytes + 127) / 128 * 128;
        if (ws_used > ws_bytes) { latch(BPDQ_ERR_RANGE); return nullptr; }
        if (xq_bytes > xq_max) xq_max = xq_bytes;
        prog.push_back(P);
    }
    StreamHandle* h = new StreamHandle();
    StreamPlan& p = h->plan;
    p.n_phases = (int)prog.size();
    p.slot_bytes = slot_bytes;
    p.slots = tu.stages < 2 ? 2 : tu.stages;
    p.nw = tu.warps < 1 ? 1 : (tu.warps > 16 ? 16 : tu.warps);
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_xq = take((size_t)xq_max);
        p.off_desc = take(2 * sizeof(StreamPhase));
        p.off_bar = take((size_t)2 * p.nw * p.slots * 8 + 16);
        p.smem = off;
        if (p.smem <= (size_t)kSmemLimit) break;
        if (p.slots > 2) p.slots--;
        else if (p.nw > 4) p.nw--;
        else { delete h; latch(BPDQ_ERR_RANGE); return nullptr; }
    }
    cudaGetDevice(&h->device);
    void *dp = nullptr, *dt = nullptr;
    if (check_cuda(cudaMalloc(&dp, sizeof(StreamPhase) * prog.size())) || check_cuda(cudaMalloc(&dt, sizeof(VecEntry) * table.size())) ||
        check_cuda(cudaMemcpy(dp, prog.data(), sizeof(StreamPhase) * prog.size(), cudaMemcpyHostToDevice)) ||
        check_cuda(cudaMemcpy(dt, table.data(), sizeof(VecEntry) * table.size(), cudaMemcpyHostToDevice))) {
        if (dp) cudaFree(dp);
        if (dt) cudaFree(dt);
        delete h;
        latch(BPDQ_ERR_CUDA);
        return nullptr;
    }
    h->d_phases = (StreamPhase*)dp;
    h->d_table = (VecEntry*)dt;
    h->records = ws;
    h->n_vec = (int)table.size();
    h->total_blocks = total_blocks;
    p.phases = h->d_phases;
    return h;
}

static int stream_run(StreamHandle* h, cudaStream_t s)
{
    if (!h) return latch(BPDQ_ERR_ARG);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != h->device) return latch(BPDQ_ERR_ARG);
    auto kern = k_gemv_stream_q4k_q8k<BPDQ_LAYOUT_BPD, kMidCtaThreads>;
    static bool attr_set[64] = {false};
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        if (rc) return latch(rc);
        attr_set[dev] = true;
    }
    // quantizer: stream-ordered (its inputs may be anything the stream produced before)
    const int qgrid = glue_grid(h->total_blocks);
    k_quant_records_table<<<qgrid, 256, 0, s>>>(h->d_table, h->n_vec, h->total_blocks, h->records);
    int rc = check_cuda(cudaGetLastError());
    if (rc) return latch(rc);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count());
    cfg.blockDim = dim3((unsigned)(h->plan.nw + 1) * 32);
    cfg.dynamicSmemBytes = h->plan.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, h->plan, device_error_flag()));
    return rc ? latch(rc) : 0;
}

static void stream_destroy(StreamHandle* h)
{
    if (!h) return;
    cudaFree(h->d_phases);
    cudaFree(h->d_table);
    delete h;
}

// Q8_0 weights [N][K/32][34] times one activation vector, activations quantized to Q8_0 inside
// the kernel.  Fast path only: K a multiple of 256 (rows are then 16-byte multiples and can be
// bulk-copied); returns BPDQ_ERR_RANGE otherwise so that the caller can take the generic kernel.
int gemv_q8_0_fast(const uint8_t* W, const float* x, float* out, int N, int K, cudaStream_t s)
{
    if ((K % 256) != 0 || ((uintptr_t)W & 15) || ((uintptr_t)x & 15)) return BPDQ_ERR_RANGE;
    BatchDesc d = {W, x, out, N, K};
    BatchPlan plan;
    int rc = make_batch_plan(&d, 1, plan, 1);
    if (rc) return rc;
    return launch_batch<1, BPDQ_LAYOUT_BPD>(plan, s);
}

// Up to kMaxBatch Q8_0 matrices that read the same activation vector, one launch (q/k/v, gate/up).
int gemv_q8_0_fast_multi(int n, const uint8_t* const* Ws, float* const* outs, const int* Ns, const float* x, int K,
                         cudaStream_t s)
{
    if (n < 1 || n > kMaxBatch || (K % 256) != 0 || ((uintptr_t)x & 15)) return BPDQ_ERR_RANGE;
    BatchDesc d[kMaxBatch];
    for (int j = 0; j < n; j++) {
        if ((uintptr_t)Ws[j] & 15) return BPDQ_ERR_RANGE;
        d[j] = {Ws[j], x, outs[j], Ns[j], K};
    }
    BatchPlan plan;
    int rc = make_batch_plan(d, n, plan, 1);
    if (rc) return rc;
    return launch_batch<1, BPDQ_LAYOUT_BPD>(plan, s);
}

// ---------------------------------------------------------------- scratch without an allocator
//
// Scratch for the quantized activation records of bpd_qmatmul_q4k_q8k_batch_static_cuda: a
// fixed array inside the library image.  Every GPU that loads the library carries these bytes
// until the process exits.
constexpr size_t kStaticRecordBytes = 256 * 1024;   // room for 233,016 activations per call
static __device__ __align__(256) uint8_t g_static_records[kStaticRecordBytes];

// In host code the name g_static_records is only a handle for the runtime, not a device
// address: it must be translated once per device, with that device current.
static uint8_t* static_records_address(int* status)
{
    static uint8_t* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        *status = e != cudaSuccess ? check_cuda(e) : latch(BPDQ_ERR_RANGE);
        return nullptr;
    }
    if (!cached[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_records);
        if (e != cudaSuccess || !p) {
            *status = e != cudaSuccess ? check_cuda(e) : latch(BPDQ_ERR_CUDA);
            return nullptr;
        }
        cached[dev] = (uint8_t*)p;
    }
    *status = 0;
    return cached[dev];
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

// Debug aid: the next `launches` GEMV launches each write 8 global-timer stamps per CTA
// (ns) into dev_buf, `stride_u64` 64-bit words apart.  Pass NULL to stop.
void bpdq_debug_trace(void* dev_buf, size_t stride_u64, int launches)
{
    g_trace_base = (unsigned long long*)dev_buf;
    g_trace_stride = stride_u64;
    g_trace_left = dev_buf ? launches : 0;
}

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
// Several weight matrices against one activation vector in one launch (the q/k/v and the
// gate/up projections of a decoder layer): out[j][Ms[j]] = W[j][Ms[j]][K] . quantize_q8_K(x[K]).
int bpd_qmatmul_q4k_q8k_multi_cuda(int n, const uint8_t* const* qweights, float* const* outs, const int* Ms,
                                   const float* x, int K, void* stream)
{
    return gemm_q4k_q8k_multi(n, qweights, outs, Ms, x, 1, K, BPDQ_LAYOUT_BPD, 0, nullptr, (cudaStream_t)stream);
}
// n independent products in as few launches as possible (one, for a decoder layer's seven
// projections).  descs is a HOST array of {W, x, out, M, K}.
int bpd_qmatmul_q4k_q8k_batch_cuda(int n, const bpdq_gemv_desc* descs, void* stream)
{
    static_assert(sizeof(bpdq_gemv_desc) == sizeof(BatchDesc), "descriptor layouts must match");
    return gemv_q4k_q8k_batch(reinterpret_cast<const BatchDesc*>(descs), n, BPDQ_LAYOUT_BPD, nullptr, 0, 0,
                              (cudaStream_t)stream);
}
// Same, with caller-owned scratch for the quantized activations (bpdq_batch_workspace_bytes
// says how much).  Ordered like any launch: the quantizer waits for the work ahead of it in the
// stream before it reads the activations or writes the scratch.
int bpd_qmatmul_q4k_q8k_batch_ws_cuda(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes,
                                      void* stream)
{
    return gemv_q4k_q8k_batch(reinterpret_cast<const BatchDesc*>(descs), n, BPDQ_LAYOUT_BPD, (uint8_t*)workspace,
                              workspace_bytes, 0, (cudaStream_t)stream);
}
// Same, for activation vectors that are complete when the call is made (nothing still in flight on
// the stream writes them) and scratch that no launch still in flight uses: the quantizer then
// runs under the tail of the launch ahead of it instead of after it.
int bpd_qmatmul_q4k_q8k_batch_ready_cuda(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes,
                                         void* stream)
{
    return gemv_q4k_q8k_batch(reinterpret_cast<const BatchDesc*>(descs), n, BPDQ_LAYOUT_BPD, (uint8_t*)workspace,
                              workspace_bytes, 1, (cudaStream_t)stream);
}
size_t bpdq_batch_workspace_bytes(int n, const bpdq_gemv_desc* descs)
{
    // upper bound: every vector distinct, each launch's share rounded up to 128 bytes
    size_t total = 0;
    for (int j = 0; j < n; j++) total += (size_t)(descs[j].K / 128) * kXqStride + 128;
    return total;
}
// Batched GEMVs for callers that must not allocate device memory (see include/bpdq.h).
int bpd_qmatmul_q4k_q8k_batch_static_cuda(int n, const bpdq_gemv_desc* descs, void* stream)
{
    if (n < 0 || (n > 0 && !descs)) return latch(BPDQ_ERR_ARG);
    // the records of all launches of this call sit side by side in the fixed array
    if (bpdq_batch_workspace_bytes(n, descs) > kStaticRecordBytes) return latch(BPDQ_ERR_RANGE);
    int rc = 0;
    uint8_t* records = static_records_address(&rc);
    if (!records) return rc;
    // ws_private = 0: the quantizer waits for everything earlier in the stream before it writes,
    // because the previous call on this stream may still be reading the same array
    return gemv_q4k_q8k_batch(reinterpret_cast<const BatchDesc*>(descs), n, BPDQ_LAYOUT_BPD, records,
                              kStaticRecordBytes, 0, (cudaStream_t)stream);
}
size_t bpdq_batch_static_capacity(void) { return kStaticRecordBytes; }

// Full-control form: tokens >= 1, layout 0/1, xsrc 0 (fp32) / 1 (pre-quantized Q8_K), optional
// int32 [M][K/256][8] buffer receiving token 0's exact sub-block dots.
size_t bpdq_records_bytes(int K) { return K > 0 && (K % 256) == 0 ? (size_t)(K / 256) * 2 * kXqStride : 0; }
int bpd_quant_q8k_records_cuda(const float* x, void* records, int K, void* stream)
{
    if (!x || !records || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)x & 15) || ((uintptr_t)records & 15)) return latch(BPDQ_ERR_ALIGN);
    int rc = launch_glue(k_vector_records, glue_grid(K / 256), (cudaStream_t)stream, x, (uint8_t*)records, (long)(K / 256));
    return rc ? latch(rc) : 0;
}
int bpd_rmsnorm_q8k_records_cuda(const float* x, const float* w, void* records, int rows, int K, float eps, void* stream)
{
    if (rows < 0 || K <= 0 || (K % 256) != 0 || (rows > 0 && (!x || !w || !records))) return latch(BPDQ_ERR_ARG);
    if (rows == 0) return 0;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)records & 15)) return latch(BPDQ_ERR_ALIGN);
    int rc = launch_glue(k_rmsnorm_records, rows, (cudaStream_t)stream, x, w, (uint8_t*)records, K, eps);
    return rc ? latch(rc) : 0;
}
int bpd_swiglu_q8k_records_cuda(const float* gate, const float* up, void* records, int K, void* stream)
{
    if (!gate || !up || !records || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)gate & 15) || ((uintptr_t)up & 15) || ((uintptr_t)records & 15)) return latch(BPDQ_ERR_ALIGN);
    int rc = launch_glue(k_swiglu_records, glue_grid(K / 256), (cudaStream_t)stream, gate, up, (uint8_t*)records, (long)(K / 256));
    return rc ? latch(rc) : 0;
}
int bpd_qmatmul_q4k_fused_cuda(int n, const bpdq_gemv_desc* descs, int prologue, const float* a, const float* b, float eps,
                               unsigned accumulate_mask, void* stream)
{
    if (n < 1 || n > kMaxBatch || !descs) return latch(BPDQ_ERR_ARG);
    BatchDesc d[kMaxBatch];
    for (int j = 0; j < n; j++) d[j] = {descs[j].W, nullptr, descs[j].out, descs[j].M, descs[j].K};
    return gemv_q4k_fused(d, n, prologue, a, b, eps, accumulate_mask, BPDQ_LAYOUT_BPD, (cudaStream_t)stream);
}
void* bpdq_gemv_stream_create(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes)
{
    return stream_create(n, reinterpret_cast<const BatchDesc*>(descs), (uint8_t*)workspace, workspace_bytes);
}
int bpdq_gemv_stream_run(void* handle, void* stream) { return stream_run((StreamHandle*)handle, (cudaStream_t)stream); }
void bpdq_gemv_stream_destroy(void* handle) { stream_destroy((StreamHandle*)handle); }
void* bpdq_chain_create(int n_phases, const bpdq_chain_phase* phases)
{
    static_assert(sizeof(bpdq_chain_phase) == sizeof(ChainPhaseDesc), "phase descriptor layouts must match");
    return chain_create(n_phases, reinterpret_cast<const ChainPhaseDesc*>(phases));
}
int bpdq_chain_run(void* chain, void* stream) { return chain_run((ChainHandle*)chain, (cudaStream_t)stream); }
void bpdq_chain_destroy(void* chain) { chain_destroy((ChainHandle*)chain); }
int bpd_qmatmul_q4k_records_cuda(int n, const bpdq_gemv_desc* descs, const void* records, unsigned accumulate_mask,
                                 void* stream)
{
    if (n < 1 || n > kMaxBatch || !descs) return latch(BPDQ_ERR_ARG);
    BatchDesc d[kMaxBatch];
    for (int j = 0; j < n; j++) d[j] = {descs[j].W, nullptr, descs[j].out, descs[j].M, descs[j].K};
    return gemv_q4k_records(d, n, (const uint8_t*)records, accumulate_mask, BPDQ_LAYOUT_BPD, (cudaStream_t)stream);
}
int bpd_qmm_q4k_q8k_cuda(const uint8_t* qweight, const void* x, float* out, int tokens, int M, int K, int layout,
                         int xsrc, int32_t* subdots, void* stream)
{
    if ((layout != 0 && layout != 1) || (xsrc != 0 && xsrc != 1)) return latch(BPDQ_ERR_ARG);
    return gemm_q4k_q8k(qweight, x, out, tokens, M, K, layout, xsrc, subdots, (cudaStream_t)stream);
}

// The tensor-core kernel at any token count (the dispatcher above picks it for more than 8).
int bpd_qmm_q4k_q8k_mma_cuda(const uint8_t* qweight, const float* X, float* out, int tokens, int M, int K, void* stream)
{
    return gemm_q4k_q8k_mma(qweight, X, out, tokens, M, K, (cudaStream_t)stream);
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

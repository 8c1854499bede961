// Device-side building blocks shared by the Q4_K x Q8_K product kernels (gemv_q4k.cu: one matrix or a
// group sharing a vector; gemv_batch.cu: independent products per launch, decode glue;
// gemv_persistent.cu: whole chains or streams of products per launch) and the launch plan of the
// batched kernel.  Arithmetic and accumulation order are described at the top of gemv_q4k.cu.
#ifndef BPDQ_GEMV_Q4K_DEVICE_CUH
#define BPDQ_GEMV_Q4K_DEVICE_CUH

#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

constexpr int kSmemLimit = 227 * 1024;
constexpr int kSmallCtaThreads = 288;   // up to 8 consumer warps + the producer
constexpr int kMidCtaThreads = 544;     // up to 16 consumer warps + the producer

// Activation records are 128 int8 padded to 144 bytes, so that the 16-byte reads of 32 consecutive
// lanes hit distinct banks (the padding carries the sub-block sums and the block scale).
constexpr int kXqStride = 144;

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Timeline stamps of the tuning builds (-DBPDQ_TRACE_BUILD); nothing in the default build.
#ifdef BPDQ_TRACE_BUILD
#define BPDQ_TRACE(slot)                                                              \
    do {                                                                              \
        if (p.trace && lane == 0 && (warp == 0 || (slot) == 7))                       \
            p.trace[(size_t)blockIdx.x * 8 + (slot)] = global_timer_ns();             \
    } while (0)
#else
#define BPDQ_TRACE(slot) do { } while (0)
#endif


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

// ---------------------------------------------------------------- inner product of one half-super-block

// sbp: shared-memory super-block (144 B).  half: which four sub-blocks.  xr[t]: this lane's
// 128 quantized activations of token t, bs[t][j]: their per-sub-block sums, xd[t]: the Q8_K
// block scale.  dbg: optional global int32[8] slot of this (row, super-block) for the exact
// sub-block dots of token 0.  (Tried on this loop and not kept: the high nibbles by a full-rate subtraction
// q - (q & 0x0F..) instead of a second mask, within +-1 % on the benchmark step depending on how the compiler
// schedules around it; the mins through two dp2a on packed sub-block sums instead of four multiply-adds, -3.5 %.)
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

// ---- the batched kernel's launch plan (up to kMaxBatch products per launch)
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
    // n > 0: every result is also stored at its output address + shift[t] (the gathered buffers of the ranks
    // of a row-sharded model, peer memory included); used by the EPI = 2 instantiation
    PeerTargets peers;
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

template <int R, int LAYOUT, int ACC>
__device__ __forceinline__ void batch_tile(const uint8_t* tile_smem, const uint8_t* xq, const BatchProblem& pb, int row0,
                                           int lane, const PeerTargets* peers = nullptr)
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
    if constexpr (ACC == 2) {
        // The exchange step of row sharding, folded into the product: the tile's R results go to the rank's own output
        // and to every rank's gathered buffer (peer memory is written, never read).  The row totals are gathered into
        // every lane, then lane 0 stores to the own output and lane t to target t - 1, each with ONE store of R floats:
        // one store instruction per tile for all targets together.
        float vals[R];
#pragma unroll
        for (int rr = 0; rr < R; rr++) vals[rr] = __shfl_sync(0xFFFFFFFFu, total, rr * kLanesPerRow);
        if (lane <= peers->n) {
            char* dst = reinterpret_cast<char*>(pb.out + row0) + (lane == 0 ? 0ll : peers->shift[lane > 0 ? lane - 1 : 0]);
            if (rows == R && (reinterpret_cast<uintptr_t>(dst) & (4 * R - 1)) == 0) {
                if constexpr (R == 4) *reinterpret_cast<float4*>(dst) = make_float4(vals[0], vals[1], vals[2], vals[3]);
                else if constexpr (R == 2) *reinterpret_cast<float2*>(dst) = make_float2(vals[0], vals[1]);
                else *reinterpret_cast<float*>(dst) = vals[0];
            } else {
#pragma unroll
                for (int rr = 0; rr < R; rr++)
                    if (rr < rows) reinterpret_cast<float*>(dst)[rr] = vals[rr];
            }
        }
    } else {
        if ((lane % kLanesPerRow) == 0 && my_row < rows)
            pb.out[row0 + my_row] = (ACC && pb.accumulate) ? __ldcg(pb.out + row0 + my_row) + total : total;
    }
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
    // the values this warp scales after the sum is known are fetched now: their latency (the vector was written by
    // other SMs a moment ago, the weights come from HBM) runs under the sum of squares instead of after it
    constexpr int kPre = 2;
    float4 pa[kPre][2], pw[kPre][2];
#pragma unroll
    for (int i = 0; i < kPre; i++) {
        const int b = warp + i * nw;
        if (b < nb) {
            const float4* xb = reinterpret_cast<const float4*>(a + (size_t)b * 256);
            const float4* wb = reinterpret_cast<const float4*>(w + (size_t)b * 256);
            pa[i][0] = __ldcg(xb + lane);
            pa[i][1] = __ldcg(xb + 32 + lane);
            pw[i][0] = __ldg(wb + lane);
            pw[i][1] = __ldg(wb + 32 + lane);
        }
    }
    for (int vw = warp; vw < 8; vw += nw) {
        float t = 0.0f;
        for (int base = 0; base < cols; base += 16 * 256) {     // sixteen loads in flight, same chain of FMAs
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int c = base + i * 256 + vw * 32 + lane;
                v[i] = c < cols ? __ldcg(a + c) : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 16; i++) t = fmaf(v[i], v[i], t);
        }
        t = warp_sum(t);
        if (lane == 0) s_sum[vw] = t;
    }
    named_bar_sync(2, nw * 32);
    float tot = s_sum[0];
#pragma unroll
    for (int i = 1; i < 8; i++) tot += s_sum[i];
    const float scale = rsqrtf(tot / (float)cols + eps);
    auto emit = [&](int b, const float4& a0, const float4& a1, const float4& w0, const float4& w1) {
        const float4 v0 = make_float4(a0.x * scale * w0.x, a0.y * scale * w0.y, a0.z * scale * w0.z, a0.w * scale * w0.w);
        const float4 v1 = make_float4(a1.x * scale * w1.x, a1.y * scale * w1.y, a1.z * scale * w1.z, a1.w * scale * w1.w);
        write_records(v0, v1, xq + (size_t)(2 * b) * kXqStride, lane);
    };
#pragma unroll
    for (int i = 0; i < kPre; i++) {
        const int b = warp + i * nw;
        if (b < nb) emit(b, pa[i][0], pa[i][1], pw[i][0], pw[i][1]);
    }
    for (int b = warp + kPre * nw; b < nb; b += nw) {
        const float4* xb = reinterpret_cast<const float4*>(a + (size_t)b * 256);
        const float4* wb = reinterpret_cast<const float4*>(w + (size_t)b * 256);
        emit(b, __ldcg(xb + lane), __ldcg(xb + 32 + lane), __ldg(wb + lane), __ldg(wb + 32 + lane));
    }
}
// silu(gate) * up with k_elementwise's arithmetic; three blocks' loads in flight per warp
__device__ __forceinline__ void cta_swiglu_records(const float* __restrict__ gate, const float* __restrict__ up, int nb,
                                                   uint8_t* xq, int warp, int lane, int nw)
{
    auto act = [](float g, float u) { return (g / (1.0f + expf(-g))) * u; };
    constexpr int kPre = 3;
    for (int b0 = warp; b0 < nb; b0 += kPre * nw) {
        float4 g[kPre][2], u[kPre][2];
#pragma unroll
        for (int i = 0; i < kPre; i++) {
            const int b = b0 + i * nw;
            if (b < nb) {
                const float4* gb = reinterpret_cast<const float4*>(gate + (size_t)b * 256);
                const float4* ub = reinterpret_cast<const float4*>(up + (size_t)b * 256);
                g[i][0] = __ldcg(gb + lane);
                g[i][1] = __ldcg(gb + 32 + lane);
                u[i][0] = __ldcg(ub + lane);
                u[i][1] = __ldcg(ub + 32 + lane);
            }
        }
#pragma unroll
        for (int i = 0; i < kPre; i++) {
            const int b = b0 + i * nw;
            if (b < nb) {
                const float4 v0 = make_float4(act(g[i][0].x, u[i][0].x), act(g[i][0].y, u[i][0].y), act(g[i][0].z, u[i][0].z), act(g[i][0].w, u[i][0].w));
                const float4 v1 = make_float4(act(g[i][1].x, u[i][1].x), act(g[i][1].y, u[i][1].y), act(g[i][1].z, u[i][1].z), act(g[i][1].w, u[i][1].w));
                write_records(v0, v1, xq + (size_t)(2 * b) * kXqStride, lane);
            }
        }
    }
}
// records of a plain vector; three blocks per warp are in flight before the first is quantized
__device__ __forceinline__ void cta_vector_records(const float* __restrict__ x, int nb, uint8_t* xq, int warp, int lane, int nw)
{
    constexpr int kPre = 3;
    for (int b0 = warp; b0 < nb; b0 += kPre * nw) {
        float4 v[kPre][2];
#pragma unroll
        for (int i = 0; i < kPre; i++) {
            const int b = b0 + i * nw;
            if (b < nb) {
                const float4* xb = reinterpret_cast<const float4*>(x + (size_t)b * 256);
                v[i][0] = __ldcg(xb + lane);
                v[i][1] = __ldcg(xb + 32 + lane);
            }
        }
#pragma unroll
        for (int i = 0; i < kPre; i++) {
            const int b = b0 + i * nw;
            if (b < nb) write_records(v[i][0], v[i][1], xq + (size_t)(2 * b) * kXqStride, lane);
        }
    }
}

struct BatchDesc {
    const uint8_t* W;
    const float* x;
    float* out;
    int M, K;
};

// ---- host side shared by the three files
// gemv_q4k.cu: next timeline buffer of a tuning build, else null
unsigned long long* trace_take();
// gemv_q4k.cu: one matrix (or tokens > 1), any shape
int gemm_q4k_q8k(const uint8_t* W, const void* x, float* out, int tokens, int M, int K, int layout, int xsrc,
                 int32_t* dbg, cudaStream_t s, Workspace* ws = nullptr);
// gemv_batch.cu: plan and launch of the batched kernel (fmt 0: Q4_K weights, 1: Q8_0)
int make_batch_plan(const BatchDesc* d, int n, BatchPlan& p, int fmt = 0, int ctas_per_sm = 1);
int launch_batch_plan(const BatchPlan& p, int fmt, int layout, cudaStream_t s);

// a small kernel (256 threads per CTA unless said otherwise) launched programmatically behind the launch before it
template <int THREADS = 256, typename Kern, typename... Args>
static int launch_glue(Kern kern, int grid, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, args...));
}
// grid of a kernel that gives one warp (of eight per CTA) to each of n_blocks work items
static inline int glue_grid(long n_blocks)
{
    long want = (n_blocks + 7) / 8, cap = (long)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace bpdq

#endif  // BPDQ_GEMV_Q4K_DEVICE_CUH

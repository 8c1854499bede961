// ================================================================ Q4_K re-tiled in groups of 16 rows
//
// The reference's idea of a weight layout made for the kernel that reads it ("Q8 padded 64B coalesced
// [nb,N,64]", inference/llamatov_c_inference.py:88-100), applied to Q4_K for products with 2..64 activation
// rows: a pure, exactly invertible permutation of the 144-byte super-blocks.
//
// Layout ("rg16"): rows are taken in groups of 16 (the M of one int8 tensor-core MMA, m16n8k32); the unit of
// (group G, super-block b) is 16 x 144 = 2304 bytes at ((G * K/256) + b) * 2304:
//     bytes    0..255   the 16 block headers (fp16 d, fp16 dmin, 12 scale bytes), row r at 16 r
//     bytes  256..2303  the nibble words in MMA fragment order: for q = 0..3, lane L = 0..31 (g = L / 4, t = L % 4)
//                       16 bytes at 256 + 512 q + 16 L = words  (j = 2q, row g) (2q, g + 8) (2q + 1, g) (2q + 1, g + 8),
//                       "word t of sub-block j" being bytes 16 + 16 j + 4 t .. + 3 of the row's original block:
//                       elements 32 j + 4 t .. + 3 in its low nibbles, 32 j + 16 + 4 t .. + 3 in its high nibbles.
// Rows beyond N are zero.  A thread of the MMA then fetches, with ONE 16-byte shared-memory load that is free of
// bank conflicts, the A fragments of two sub-blocks (rows g and g + 8), and the units of a row group follow each
// other along K, so any K range of a group is ONE contiguous span for a 1-D bulk copy: no tensor maps, no per-row
// requests.
//
// Kernel (k_gemm_q4k_rg16<NT>, NT tiles of 8 tokens): the streaming structure of gemv_stream.cu with the
// arithmetic of gemm_q4k_mma.cu.  A CTA takes "CTA tiles" (nw row groups of one matrix, one per warp) in turn and
// walks K in chunks of kc super-blocks.  Every warp owns ring slots that it refills itself with the next chunks of
// its own row groups (one bulk copy each); the quantized activations of a chunk (288-byte records per super-block
// and token, written by k_quant_rg16_records) are shared by the CTA's warps and swapped through two buffers by a
// records warp, with one mbarrier pair per buffer and no CTA-wide barrier.  Per sub-block and token tile: one MMA
// on the raw nibbles, the 6-bit scale applied to its int32 result; per super-block the mins through the
// activations' sub-block sums, then acc = fma(dA, d * float(isum) - dmin * float(msum), acc), super-blocks
// ascending: the arithmetic and order of gemm_q4k_mma.cu, same bits.  All waits are bounded.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

#include <cstring>
#include <vector>

namespace bpdq {

constexpr int kRgRows = 16;
constexpr int kRgUnit = kRgRows * BPDQ_Q4K_BYTES;    // 2304
constexpr int kRgActPitch = 288;                     // bytes per (super-block, token) record
constexpr int kRgInline = 8;                         // products whose table travels as kernel parameters
constexpr int kRgMaxProblems = 128;                  // products per launch
constexpr int kRgMaxThreads = 352;

struct RgProblem {            // 32 bytes
    const uint8_t* W;         // re-tiled weights
    float* out;               // [tokens][M]
    int M;
    int tile_begin;           // index of the product's first CTA tile
    unsigned short nb, pad;
    unsigned rec_off16;       // offset of its activation records in the launch's scratch, in 16-byte units
};
static_assert(sizeof(RgProblem) == 32, "table entries are copied in 16-byte pieces");

struct RgPlan {
    const RgProblem* table;                   // device table (n_problems + 1 entries), or null: inline_tab
    RgProblem inline_tab[kRgInline + 1];
    const uint8_t* records;
    int n_problems, n_tiles;                  // CTA tiles over all products
    int tokens, tok_pad;
    int nw, slots, kc;                        // row groups per CTA tile (= consumer warps), ring slots per warp, super-blocks per chunk
    int slot_bytes, xq_bytes;                 // kc * 2304, kc * tok_pad * 288
    int off_ring, off_xq, off_tab, off_bar;
    size_t smem;
    int32_t* ints;                            // optional [tokens][M][nb][2] of product 0: exact (isum, msum)
};

struct RgVec {                // one distinct activation matrix X [tokens][K] of a launch
    const float* X;
    int nb, unit_begin;       // unit = (super-block, padded token)
    unsigned rec_off16, pad;
};

// ---- the permutation, both ways: one thread per 16-byte piece of a unit
template <bool FORWARD>
__global__ void __launch_bounds__(256) k_q4k_rg16_permute(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int nb,
                                                         long n_pieces)
{
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_pieces; it += (long)gridDim.x * blockDim.x) {
        const long unit = it / 144;
        const int pi = (int)(it - unit * 144);
        const long G = unit / nb;
        const int b = (int)(unit - G * nb);
        const size_t tile_at = (size_t)unit * kRgUnit + (size_t)pi * 16;
        if (pi < 16) {
            const long row = G * kRgRows + pi;
            const size_t raw_at = ((size_t)row * nb + b) * BPDQ_Q4K_BYTES;
            if (FORWARD) *reinterpret_cast<uint4*>(dst + tile_at) = row < N ? *reinterpret_cast<const uint4*>(src + raw_at) : make_uint4(0, 0, 0, 0);
            else if (row < N) *reinterpret_cast<uint4*>(dst + raw_at) = *reinterpret_cast<const uint4*>(src + tile_at);
        } else {
            const int pp = pi - 16, q = pp >> 5, L = pp & 31, g = L >> 2, t = L & 3;
            uint32_t w[4];
            if (!FORWARD) {
                const uint4 v = *reinterpret_cast<const uint4*>(src + tile_at);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int j = 2 * q + (e >> 1);
                const long row = G * kRgRows + g + 8 * (e & 1);
                const size_t raw_at = ((size_t)row * nb + b) * BPDQ_Q4K_BYTES + 16 + 16 * j + 4 * t;
                if (FORWARD) w[e] = row < N ? *reinterpret_cast<const uint32_t*>(src + raw_at) : 0u;
                else if (row < N) *reinterpret_cast<uint32_t*>(dst + raw_at) = w[e];
            }
            if (FORWARD) *reinterpret_cast<uint4*>(dst + tile_at) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// ---- activation quantizer: one warp per (super-block, padded token) of every distinct activation matrix of the
// launch.  Record (288 bytes): 256 int8 with word w of the 64 (elements 4w..4w+3) stored at position
// 8 (w / 8) + 2 (w % 4) + (w % 8) / 4, so that a thread's two B-fragment words of a sub-block are adjacent; then the
// fp32 block scale and, at byte 272, the eight int16 sub-block sums.  The Q8_K rule of gemv_q4k.cu.
__global__ void __launch_bounds__(256) k_quant_rg16_records(const RgVec* __restrict__ vecs, const RgVec one, int n_vec,
                                                             long total_units, uint8_t* __restrict__ records, int tokens, int tok_pad)
{
    // ordered like any launch: the activations may come from the launch ahead, which may also still read the scratch.
    // vecs == null: the single entry `one` came with the launch.
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
    for (long u = warp; u < total_units; u += n_warps) {
        int lo = 0, hi = n_vec - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if ((long)vecs[mid].unit_begin <= u) lo = mid;
            else hi = mid - 1;
        }
        const RgVec v = vecs ? vecs[lo] : one;
        const int local = (int)(u - v.unit_begin);
        const int b = local / tok_pad, t = local - b * tok_pad;
        uint32_t* rec = reinterpret_cast<uint32_t*>(records + (size_t)v.rec_off16 * 16 + ((size_t)b * tok_pad + t) * kRgActPitch);
        if (t >= tokens) {
            rec[lane] = 0;
            rec[32 + lane] = 0;
            if (lane < 8) rec[64 + lane] = 0;
            continue;
        }
        const float4* xb = reinterpret_cast<const float4*>(v.X + (size_t)t * v.nb * 256 + (size_t)b * 256);
        const float4 v0 = __ldcg(xb + lane), v1 = __ldcg(xb + 32 + lane);
        float amax = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w)));
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
        amax = warp_max(amax);
        const float d = __fdiv_rn(amax, 127.0f);
        const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        auto q = [mul](float x) -> uint32_t { return (uint32_t)__float2int_rn(__fmul_rn(x, mul)) & 0xFFu; };
        const uint32_t p0 = q(v0.x) | (q(v0.y) << 8) | (q(v0.z) << 16) | (q(v0.w) << 24);   // word lane
        const uint32_t p1 = q(v1.x) | (q(v1.y) << 8) | (q(v1.z) << 16) | (q(v1.w) << 24);   // word 32 + lane
        const int pos = 8 * (lane >> 3) + 2 * (lane & 3) + ((lane & 7) >> 2);
        rec[pos] = p0;
        rec[32 + pos] = p1;
        int s0 = dp4a_ss(p0, 0x01010101u, 0), s1 = dp4a_ss(p1, 0x01010101u, 0);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, o);
            s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
        }
        short* bs = reinterpret_cast<short*>(rec + 68);           // bytes 272..287
        if ((lane & 7) == 0) {
            bs[lane >> 3] = (short)s0;                            // sub-blocks 0..3
            bs[4 + (lane >> 3)] = (short)s1;                      // sub-blocks 4..7
        }
        if (lane == 0) rec[64] = __float_as_uint(d);
        if (lane > 0 && lane < 4) rec[64 + lane] = 0;
    }
}

__device__ __forceinline__ void rg_mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    // (not volatile: a pure function of its operands, so that independent MMAs can be scheduled back to back)
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ int rg_dp2a_lo(uint32_t a16x2, uint32_t b8x4, int c)
{
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a16x2), "r"(b8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int rg_dp2a_hi(uint32_t a16x2, uint32_t b8x4, int c)
{
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a16x2), "r"(b8x4), "r"(c));
    return d;
}

// Position of a CTA in its sequence of (CTA tile, K chunk) phases.
struct RgWalk {
    int tile, j, chunk, nch;
};

template <int NT>
__global__ void __launch_bounds__(kRgMaxThreads, 1)
k_gemm_q4k_rg16(const RgPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                            // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                                // [2][xq_bytes]
    const RgProblem* tab = reinterpret_cast<const RgProblem*>(smem + p.off_tab);  // [n_problems + 1]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);               // [nw*slots] a chunk of weights has landed
    uint64_t* xfull = full + p.nw * p.slots;                                      // [2] a chunk's records have landed
    uint64_t* xempty = xfull + 2;                                                 // [2] every warp is done with them

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = p.nw, grid = (int)gridDim.x;
    {
        const int n16 = (p.n_problems + 1) * 2;
        const uint4* src = p.table ? reinterpret_cast<const uint4*>(p.table) : nullptr;
        for (int w = tid; w < n16; w += blockDim.x)
            reinterpret_cast<uint4*>(smem + p.off_tab)[w] = src ? __ldg(src + w) : reinterpret_cast<const uint4*>(p.inline_tab)[w];
    }
    {
        // the barriers are set up by as many threads: full[nw*slots], xfull[2], xempty[2] (one arrival per consumer warp)
        const int n_bars = nw * p.slots + 4, first_xempty = nw * p.slots + 2;
        for (int b = tid; b < n_bars; b += blockDim.x) {
            mbar_init(&full[b], b >= first_xempty ? nw : 1);
            mbar_init_fence();
        }
    }
    __syncthreads();

    auto start = [&](RgWalk& w) {
        w.tile = (int)blockIdx.x;
        w.j = 0;
        w.chunk = 0;
        w.nch = 1;
        if (w.tile < p.n_tiles) {
            while (w.tile >= tab[w.j + 1].tile_begin) w.j++;
            w.nch = ((int)tab[w.j].nb + p.kc - 1) / p.kc;
        }
    };
    auto advance = [&](RgWalk& w) {
        if (++w.chunk == w.nch) {
            w.chunk = 0;
            w.tile += grid;
            if (w.tile < p.n_tiles) {
                while (w.tile >= tab[w.j + 1].tile_begin) w.j++;
                w.nch = ((int)tab[w.j].nb + p.kc - 1) / p.kc;
            }
        }
    };

    if (warp == nw) {
        // ---- records warp: one lane walks the phases and keeps the two record buffers filled
        if (lane == 0) {
            RgWalk rw;
            start(rw);
            pdl_wait();                 // the records come from the quantizer launched just before
            pdl_launch_dependents();
            for (int ph = 0; rw.tile < p.n_tiles; ph++) {
                const int b = ph & 1;
                if (ph >= 2 && !mbar_wait_bounded(&xempty[b], (uint32_t)((ph >> 1) - 1) & 1u, err, 4)) break;
                const RgProblem& q = tab[rw.j];
                const int sb0 = rw.chunk * p.kc;
                const int nsb = min(p.kc, (int)q.nb - sb0);
                const uint32_t bytes = (uint32_t)nsb * p.tok_pad * kRgActPitch;
                mbar_expect_tx(&xfull[b], bytes);
                bulk_g2s(xq + (size_t)b * p.xq_bytes, p.records + (size_t)q.rec_off16 * 16 + (size_t)sb0 * p.tok_pad * kRgActPitch,
                         bytes, &xfull[b]);
                advance(rw);
            }
        }
        return;
    }

    // ---- consumer warps: warp w takes row group w of every CTA tile
    const int g = lane >> 2, t = lane & 3;
    uint8_t* my_ring = ring + (size_t)warp * p.slots * p.slot_bytes;
    uint64_t* my_full = full + warp * p.slots;
    RgWalk lw, cw;                      // the chunk to load next, the chunk to compute next
    start(lw);
    start(cw);
    int load_slot = 0, pending = 0;
    auto group_of = [&](const RgWalk& w) -> int {      // this warp's row group in the walk's CTA tile, or -1
        const RgProblem& q = tab[w.j];
        const int G = (w.tile - q.tile_begin) * nw + warp;
        return G < (q.M + kRgRows - 1) / kRgRows ? G : -1;
    };
    auto pump = [&]() {                 // keep `slots` chunks of this warp's own weights on their way
        while (pending < p.slots && lw.tile < p.n_tiles) {
            const int G = group_of(lw);
            if (G >= 0) {
                const RgProblem& q = tab[lw.j];
                const int sb0 = lw.chunk * p.kc;
                const uint32_t bytes = (uint32_t)min(p.kc, (int)q.nb - sb0) * kRgUnit;
                if (lane == 0) {
                    mbar_expect_tx(&my_full[load_slot], bytes);
                    bulk_g2s(my_ring + (size_t)load_slot * p.slot_bytes, q.W + ((size_t)G * q.nb + sb0) * kRgUnit, bytes,
                             &my_full[load_slot]);
                }
                if (++load_slot == p.slots) load_slot = 0;
                pending++;
            }
            advance(lw);
        }
    };
    pump();                             // weights never depend on the launch before this one

    float facc[NT][4];
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; cw.tile < p.n_tiles; ph++) {
        if (ph == 0) pdl_wait();        // join the stream order (unbounded by design) before the bounded wait
        if (!mbar_wait_bounded(&xfull[ph & 1], (uint32_t)(ph >> 1) & 1u, err, 3)) return;
        if (ph == 0) pdl_launch_dependents();
        const int G = group_of(cw);
        if (G >= 0) {
            if (!mbar_wait_bounded(&my_full[slot], parity, err, 2)) return;
            const RgProblem& q = tab[cw.j];
            if (cw.chunk == 0) {
#pragma unroll
                for (int n = 0; n < NT; n++)
#pragma unroll
                    for (int i = 0; i < 4; i++) facc[n][i] = 0.0f;
            }
            const int sb0 = cw.chunk * p.kc;
            const int nsb = min(p.kc, (int)q.nb - sb0);
            const uint8_t* chunk = my_ring + (size_t)slot * p.slot_bytes;
            const uint8_t* recs = xq + (size_t)(ph & 1) * p.xq_bytes;
            for (int s = 0; s < nsb; s++) {
                const uint8_t* unit = chunk + (size_t)s * kRgUnit;
                const uint8_t* xa = recs + (size_t)s * p.tok_pad * kRgActPitch;
                const uint4 h0 = *reinterpret_cast<const uint4*>(unit + 16 * g);
                const uint4 h1 = *reinterpret_cast<const uint4*>(unit + 16 * (g + 8));
                uint32_t sca[2], mna[2], scb[2], mnb[2];   // packed scales / mins of rows g and g + 8, halves 0 / 1
                q4k_scales4(h0.y, h0.z, h0.w, 0, sca[0], mna[0]);
                q4k_scales4(h0.y, h0.z, h0.w, 1, sca[1], mna[1]);
                q4k_scales4(h1.y, h1.z, h1.w, 0, scb[0], mnb[0]);
                q4k_scales4(h1.y, h1.z, h1.w, 1, scb[1], mnb[1]);
                int isum[NT][4];
#pragma unroll
                for (int n = 0; n < NT; n++)
#pragma unroll
                    for (int i = 0; i < 4; i++) isum[n][i] = 0;
                // The MMAs of a group of sub-blocks are issued back to back, each into its own registers, and only then
                // are their results scaled and added: the tensor pipe's latency is paid once per group, not per MMA.
                constexpr int GS = NT == 1 ? 8 : (NT == 2 ? 4 : 2);          // sub-blocks per group
#pragma unroll
                for (int j0 = 0; j0 < 8; j0 += GS) {
                    int c[GS][NT][4];
#pragma unroll
                    for (int jj = 0; jj < GS; jj += 2) {
                        const int qq = (j0 + jj) >> 1;
                        const uint4 wv = *reinterpret_cast<const uint4*>(unit + 256 + 512 * qq + 16 * lane);
                        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                        for (int e2 = 0; e2 < 2; e2++) {
                            const int j = j0 + jj + e2;
                            const uint32_t wa = ww[2 * e2], wb = ww[2 * e2 + 1];
                            // fragment order: {row g k 0-15, row g+8 k 0-15, row g k 16-31, row g+8 k 16-31}
                            const uint32_t af[4] = {wa & 0x0F0F0F0Fu, wb & 0x0F0F0F0Fu, (wa >> 4) & 0x0F0F0F0Fu, (wb >> 4) & 0x0F0F0F0Fu};
#pragma unroll
                            for (int n = 0; n < NT; n++) {
                                const uint2 bf = *reinterpret_cast<const uint2*>(xa + (size_t)(8 * n + g) * kRgActPitch + 32 * j + 8 * t);
                                rg_mma_s8(c[jj + e2][n], af, bf.x, bf.y);
                            }
                        }
                    }
#pragma unroll
                    for (int jj = 0; jj < GS; jj++) {
                        const int j = j0 + jj;
                        const int sa = (int)byte_of(sca[j >> 2], j & 3), sb_ = (int)byte_of(scb[j >> 2], j & 3);
#pragma unroll
                        for (int n = 0; n < NT; n++) {
                            isum[n][0] += sa * c[jj][n][0];
                            isum[n][1] += sa * c[jj][n][1];
                            isum[n][2] += sb_ * c[jj][n][2];
                            isum[n][3] += sb_ * c[jj][n][3];
                        }
                    }
                }
                const float d0 = f16_bits_to_f32(h0.x & 0xFFFFu), m0 = f16_bits_to_f32(h0.x >> 16);
                const float d1 = f16_bits_to_f32(h1.x & 0xFFFFu), m1 = f16_bits_to_f32(h1.x >> 16);
#pragma unroll
                for (int n = 0; n < NT; n++) {
                    // accumulator i: row g (i < 2) or g + 8, token 8n + 2t + (i & 1)
                    const uint8_t* r0 = xa + (size_t)(8 * n + 2 * t) * kRgActPitch;
                    const uint8_t* r1 = r0 + kRgActPitch;
                    const float dA0 = *reinterpret_cast<const float*>(r0 + 256);
                    const float dA1 = *reinterpret_cast<const float*>(r1 + 256);
                    const uint4 bs0 = *reinterpret_cast<const uint4*>(r0 + 272);   // eight int16 sub-block sums
                    const uint4 bs1 = *reinterpret_cast<const uint4*>(r1 + 272);
                    auto msum = [](const uint4& bs, uint32_t mlo, uint32_t mhi) {
                        int v = rg_dp2a_lo(bs.x, mlo, 0);
                        v = rg_dp2a_hi(bs.y, mlo, v);
                        v = rg_dp2a_lo(bs.z, mhi, v);
                        return rg_dp2a_hi(bs.w, mhi, v);
                    };
                    const int ms[4] = {msum(bs0, mna[0], mna[1]), msum(bs1, mna[0], mna[1]), msum(bs0, mnb[0], mnb[1]),
                                       msum(bs1, mnb[0], mnb[1])};
                    if (p.ints && cw.j == 0) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int row = G * kRgRows + g + (i >> 1) * 8, tok = 8 * n + 2 * t + (i & 1);
                            if (row < q.M && tok < p.tokens)
                                *reinterpret_cast<int2*>(p.ints + (((size_t)tok * q.M + row) * q.nb + (sb0 + s)) * 2) =
                                    make_int2(isum[n][i], ms[i]);
                        }
                    }
                    const float v0 = d0 * (float)isum[n][0] - m0 * (float)ms[0];
                    const float v1 = d0 * (float)isum[n][1] - m0 * (float)ms[1];
                    const float v2 = d1 * (float)isum[n][2] - m1 * (float)ms[2];
                    const float v3 = d1 * (float)isum[n][3] - m1 * (float)ms[3];
                    facc[n][0] = fmaf(dA0, v0, facc[n][0]);
                    facc[n][1] = fmaf(dA1, v1, facc[n][1]);
                    facc[n][2] = fmaf(dA0, v2, facc[n][2]);
                    facc[n][3] = fmaf(dA1, v3, facc[n][3]);
                }
            }
            if (cw.chunk == cw.nch - 1) {
                // out is [tokens][M]
#pragma unroll
                for (int n = 0; n < NT; n++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int row = G * kRgRows + g + (i >> 1) * 8, tok = 8 * n + 2 * t + (i & 1);
                        if (row < q.M && tok < p.tokens) q.out[(size_t)tok * q.M + row] = facc[n][i];
                    }
            }
            pending--;
            if (++slot == p.slots) {
                slot = 0;
                parity ^= 1u;
            }
        }
        // every lane is done with the chunk's records and with the ring slot
        __syncwarp();
        if (lane == 0) mbar_arrive(&xempty[ph & 1]);
        pump();
        advance(cw);
    }
}

// ------------------------------------------------------------------ host side

static size_t rg16_bytes(int N, int K) { return (size_t)((N + kRgRows - 1) / kRgRows) * (size_t)(K / 256) * kRgUnit; }

static int rg16_permute(bool forward, const uint8_t* src, uint8_t* dst, int N, int K, cudaStream_t s)
{
    if (N < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (N == 0) return 0;
    if (!src || !dst) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return latch(BPDQ_ERR_ALIGN);
    const int nb = K / 256;
    const long n_pieces = (long)((N + kRgRows - 1) / kRgRows) * nb * 144;
    const long want = (n_pieces + 255) / 256, cap = (long)sm_count() * 16;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    if (forward) k_q4k_rg16_permute<true><<<grid, 256, 0, s>>>(src, dst, N, nb, n_pieces);
    else k_q4k_rg16_permute<false><<<grid, 256, 0, s>>>(src, dst, N, nb, n_pieces);
    int rc = check_cuda(cudaGetLastError());
    return rc ? latch(rc) : 0;
}

struct RgDesc {               // = bpdq_gemv_desc with W pointing to re-tiled weights and x to X [tokens][K]
    const uint8_t* W;
    const float* x;
    float* out;
    int M, K;
};

// Shapes a launch for n products at `tokens` (1..64) activation rows; fills table / vecs (host) and the plan.
static int rg16_plan(const RgDesc* d, int n, int tokens, RgPlan& p, std::vector<RgProblem>& table, std::vector<RgVec>& vecs,
                     size_t& records_bytes, long& total_units)
{
    if (n < 1 || n > kRgMaxProblems || tokens < 1 || tokens > 64) return BPDQ_ERR_RANGE;
    const int nt = tokens <= 8 ? 1 : (tokens <= 16 ? 2 : (tokens <= 32 ? 4 : 8));
    p.tokens = tokens;
    p.tok_pad = 8 * nt;
    p.kc = nt >= 4 ? 2 : 4;
    p.slot_bytes = p.kc * kRgUnit;
    p.xq_bytes = p.kc * p.tok_pad * kRgActPitch;
    p.n_problems = n;
    p.ints = nullptr;
    p.table = nullptr;
    long groups_total = 0;
    for (int j = 0; j < n; j++) {
        if (d[j].M <= 0 || d[j].K <= 0 || (d[j].K % 256) != 0 || d[j].K / 256 > 65535) return BPDQ_ERR_ARG;
        if (!d[j].W || !d[j].x || !d[j].out) return BPDQ_ERR_ARG;
        if (((uintptr_t)d[j].W & 15) || ((uintptr_t)d[j].x & 15) || ((uintptr_t)d[j].out & 3)) return BPDQ_ERR_ALIGN;
        groups_total += (d[j].M + kRgRows - 1) / kRgRows;
    }
    // Row groups per CTA tile (= consumer warps): the SMs' warps run side by side and share the SM's issue slots and
    // bandwidth, so the time of a launch goes with (tiles per SM) x (groups per tile); among equal costs, more warps.
    const int nw_max = 10;
    long cost_of[nw_max + 1];
    long best_cost = -1;
    for (int w = 1; w <= nw_max; w++) {
        long tiles = 0;
        for (int j = 0; j < n; j++) tiles += ((d[j].M + kRgRows - 1) / kRgRows + w - 1) / w;
        cost_of[w] = ((tiles + sm_count() - 1) / sm_count()) * w;
        if (best_cost < 0 || cost_of[w] < best_cost) best_cost = cost_of[w];
    }
    // more warps hide the MMA's latency: the widest tile within 3 % of the cheapest
    int best_nw = 1;
    for (int w = nw_max; w >= 1; w--)
        if (cost_of[w] * 100 <= best_cost * 103) { best_nw = w; break; }
    p.nw = best_nw;
    const size_t tab_bytes = ((size_t)(n + 1) * sizeof(RgProblem) + 127) / 128 * 128;
    for (;;) {
        const size_t fixed = 2 * (size_t)p.xq_bytes + tab_bytes + 1024;     // + barriers
        long slots = (227L * 1024 - (long)fixed) / ((long)p.nw * p.slot_bytes);
        if (slots > 6) slots = 6;
        if (slots >= 2) { p.slots = (int)slots; break; }
        if (p.nw > 1) p.nw--;
        else return BPDQ_ERR_RANGE;
    }
    size_t off = 0;
    auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
    p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
    p.off_xq = take((size_t)2 * p.xq_bytes);
    p.off_tab = take((size_t)(n + 1) * sizeof(RgProblem));
    p.off_bar = take((size_t)(p.nw * p.slots + 4) * 8);
    p.smem = off;
    table.assign(n + 1, RgProblem());
    vecs.clear();
    size_t rec_used = 0;
    long units = 0;
    int tiles = 0;
    for (int j = 0; j < n; j++) {
        const int nb = d[j].K / 256;
        size_t k = 0;
        for (; k < vecs.size(); k++)
            if (vecs[k].X == d[j].x && vecs[k].nb == nb) break;
        if (k == vecs.size()) {
            RgVec v;
            v.X = d[j].x;
            v.nb = nb;
            v.unit_begin = (int)units;
            v.rec_off16 = (unsigned)(rec_used / 16);
            v.pad = 0;
            vecs.push_back(v);
            units += (long)nb * p.tok_pad;
            rec_used += (size_t)nb * p.tok_pad * kRgActPitch;
            if (units > 0x7FFFFFFFL) return BPDQ_ERR_RANGE;
        }
        RgProblem& q = table[j];
        q.W = d[j].W;
        q.out = d[j].out;
        q.M = d[j].M;
        q.tile_begin = tiles;
        q.nb = (unsigned short)nb;
        q.pad = 0;
        q.rec_off16 = vecs[k].rec_off16;
        tiles += ((d[j].M + kRgRows - 1) / kRgRows + p.nw - 1) / p.nw;
    }
    table[n] = table[n - 1];
    table[n].tile_begin = 0x7FFFFFFF;
    p.n_tiles = tiles;
    records_bytes = rec_used;
    total_units = units;
    (void)groups_total;
    return 0;
}

template <int NT>
static int rg16_launch_nt(const RgPlan& p, cudaStream_t s)
{
    auto kern = k_gemm_q4k_rg16<NT>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.n_tiles < sm_count() ? p.n_tiles : sm_count()));
    cfg.blockDim = dim3((unsigned)(p.nw + 1) * 32);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p, device_error_flag()));
}

static int rg16_launch(const RgPlan& p, cudaStream_t s)
{
    switch (p.tok_pad) {
        case 8: return rg16_launch_nt<1>(p, s);
        case 16: return rg16_launch_nt<2>(p, s);
        case 32: return rg16_launch_nt<4>(p, s);
        default: return rg16_launch_nt<8>(p, s);
    }
}

static int rg16_quantize(const RgVec* d_vecs, const RgVec& one, int n_vec, long total_units, uint8_t* records, int tokens, int tok_pad,
                         cudaStream_t s)
{
    const long want = (total_units + 7) / 8, cap = (long)sm_count() * 8;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(want < 1 ? 1 : (want < cap ? want : cap)));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, k_quant_rg16_records, d_vecs, one, n_vec, total_units, records, tokens, tok_pad));
}

// One product, any number of tokens (passes of 64): no tables in device memory (they travel as kernel parameters;
// the one vector entry of the quantizer sits at the head of the scratch).
int gemm_q4k_q8k_rg16(const uint8_t* tiles, const float* X, float* out, int tokens, int N, int K, cudaStream_t s, Workspace* ws,
                      int32_t* sb_ints)
{
    if (tokens < 0 || N < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (tokens == 0 || N == 0) return 0;
    if (!tiles || !X || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)tiles & 15) || ((uintptr_t)X & 15) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    for (int t0 = 0; t0 < tokens; t0 += 64) {
        const int T = tokens - t0 < 64 ? tokens - t0 : 64;
        RgDesc d = {tiles, X + (size_t)t0 * K, out + (size_t)t0 * N, N, K};
        RgPlan p;
        std::vector<RgProblem> table;
        std::vector<RgVec> vecs;
        size_t rec_bytes = 0;
        long units = 0;
        int rc = rg16_plan(&d, 1, T, p, table, vecs, rec_bytes, units);
        if (rc) return latch(rc);
        // every pass of 64 tokens reuses the scratch (the quantizer waits for the pass before it)
        Workspace pass_ws = ws ? *ws : Workspace{nullptr, 0, 0};
        uint8_t* scratch = scratch_take(ws ? &pass_ws : nullptr, kScratchQ4ktActs, rec_bytes, s, &rc);
        if (!scratch) return rc;
        rc = rg16_quantize(nullptr, vecs[0], 1, units, scratch, T, p.tok_pad, s);
        if (rc) return latch(rc);
        p.records = scratch;
        for (int j = 0; j <= 1; j++) p.inline_tab[j] = table[j];
        p.ints = sb_ints ? sb_ints + (size_t)t0 * N * (K / 256) * 2 : nullptr;
        rc = rg16_launch(p, s);
        if (rc) return latch(rc);
    }
    return 0;
}

size_t gemm_q4k_q8k_rg16_workspace(int tokens, int K)
{
    const int T = tokens < 64 ? tokens : 64;
    const int nt = T <= 8 ? 1 : (T <= 16 ? 2 : (T <= 32 ? 4 : 8));
    return (size_t)(K / 256) * (8 * nt) * kRgActPitch + 256;
}

// ---- many products, one launch per 128 of them: tables in device memory, made once
struct RgLaunch {
    RgPlan plan;
    RgProblem* d_table;
    RgVec* d_vecs;
    int n_vec;
    long units;
};
struct RgHandle {
    std::vector<RgLaunch> launches;
    int device, tokens;
};

static void rg16_stream_destroy(RgHandle* h)
{
    if (!h) return;
    for (auto& L : h->launches) {
        if (L.d_table) cudaFree(L.d_table);
        if (L.d_vecs) cudaFree(L.d_vecs);
    }
    delete h;
}

static size_t rg16_stream_workspace(int n, const RgDesc* d, int tokens)
{
    const int T = tokens < 64 ? tokens : 64;
    const int nt = T <= 8 ? 1 : (T <= 16 ? 2 : (T <= 32 ? 4 : 8));
    size_t total = 0;
    for (int j = 0; j < n; j++) total += (size_t)(d[j].K / 256) * (8 * nt) * kRgActPitch;
    return total + 256;
}

static RgHandle* rg16_stream_create(int n, const RgDesc* d, int tokens, uint8_t* ws, size_t ws_bytes)
{
    if (n < 1 || !d || !ws || ((uintptr_t)ws & 15) || tokens < 1 || tokens > 64) { latch(BPDQ_ERR_ARG); return nullptr; }
    RgHandle* h = new RgHandle();
    h->tokens = tokens;
    cudaGetDevice(&h->device);
    const int n_launches = (n + kRgMaxProblems - 1) / kRgMaxProblems;
    const int per_launch = (n + n_launches - 1) / n_launches;
    size_t ws_used = 0;
    for (int i0 = 0; i0 < n; i0 += per_launch) {
        const int cnt = n - i0 < per_launch ? n - i0 : per_launch;
        RgLaunch L;
        memset(&L, 0, sizeof(L));
        std::vector<RgProblem> table;
        std::vector<RgVec> vecs;
        size_t rec_bytes = 0;
        int rc = rg16_plan(d + i0, cnt, tokens, L.plan, table, vecs, rec_bytes, L.units);
        if (rc) { rg16_stream_destroy(h); latch(rc); return nullptr; }
        if (ws_used + rec_bytes > ws_bytes) { rg16_stream_destroy(h); latch(BPDQ_ERR_RANGE); return nullptr; }
        L.plan.records = ws + ws_used;
        ws_used += (rec_bytes + 255) / 256 * 256;
        void *dt = nullptr, *dv = nullptr;
        if (check_cuda(cudaMalloc(&dt, sizeof(RgProblem) * table.size())) || check_cuda(cudaMalloc(&dv, sizeof(RgVec) * vecs.size())) ||
            check_cuda(cudaMemcpy(dt, table.data(), sizeof(RgProblem) * table.size(), cudaMemcpyHostToDevice)) ||
            check_cuda(cudaMemcpy(dv, vecs.data(), sizeof(RgVec) * vecs.size(), cudaMemcpyHostToDevice))) {
            if (dt) cudaFree(dt);
            if (dv) cudaFree(dv);
            rg16_stream_destroy(h);
            latch(BPDQ_ERR_CUDA);
            return nullptr;
        }
        L.d_table = (RgProblem*)dt;
        L.d_vecs = (RgVec*)dv;
        L.n_vec = (int)vecs.size();
        L.plan.table = L.d_table;
        h->launches.push_back(L);
    }
    return h;
}

static int rg16_stream_run(RgHandle* h, cudaStream_t s)
{
    if (!h) return latch(BPDQ_ERR_ARG);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != h->device) return latch(BPDQ_ERR_ARG);
    for (auto& L : h->launches) {
        int rc = rg16_quantize(L.d_vecs, RgVec(), L.n_vec, L.units, const_cast<uint8_t*>(L.plan.records), h->tokens, L.plan.tok_pad, s);
        if (rc) return latch(rc);
        rc = rg16_launch(L.plan, s);
        if (rc) return latch(rc);
    }
    return 0;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

size_t bpd_q4k_rg16_bytes(int N, int K)
{
    if (N < 0 || K <= 0 || (K % 256) != 0) return 0;
    return rg16_bytes(N, K);
}
int bpd_repack_q4k_rg16_cuda(const uint8_t* raw, uint8_t* tiles, int N, int K, void* stream)
{
    return rg16_permute(true, raw, tiles, N, K, (cudaStream_t)stream);
}
int bpd_unrepack_q4k_rg16_cuda(const uint8_t* tiles, uint8_t* raw, int N, int K, void* stream)
{
    return rg16_permute(false, tiles, raw, N, K, (cudaStream_t)stream);
}
int bpd_qmm_q4k_q8k_rg16_cuda(const uint8_t* tiles, const float* X, float* out, int tokens, int M, int K, void* stream)
{
    return gemm_q4k_q8k_rg16(tiles, X, out, tokens, M, K, (cudaStream_t)stream, nullptr, nullptr);
}
size_t bpdq_qmm_q4k_q8k_rg16_workspace_bytes(int tokens, int K)
{
    return tokens > 0 && K > 0 && (K % 256) == 0 ? gemm_q4k_q8k_rg16_workspace(tokens, K) : 0;
}
int bpd_qmm_q4k_q8k_rg16_ws_cuda(const uint8_t* tiles, const float* X, float* out, int tokens, int M, int K, void* workspace,
                                 size_t workspace_bytes, void* stream)
{
    if (!workspace || ((uintptr_t)workspace & 15)) return latch(workspace ? BPDQ_ERR_ALIGN : BPDQ_ERR_ARG);
    Workspace ws = {(uint8_t*)workspace, workspace_bytes, 0};
    return gemm_q4k_q8k_rg16(tiles, X, out, tokens, M, K, (cudaStream_t)stream, &ws, nullptr);
}
int bpd_qmm_q4k_q8k_rg16_ints_cuda(const uint8_t* tiles, const float* X, float* out, int32_t* sb_ints, int tokens, int M, int K,
                                   void* stream)
{
    if (!sb_ints || ((uintptr_t)sb_ints & 7)) return latch(sb_ints ? BPDQ_ERR_ALIGN : BPDQ_ERR_ARG);
    return gemm_q4k_q8k_rg16(tiles, X, out, tokens, M, K, (cudaStream_t)stream, nullptr, sb_ints);
}
size_t bpdq_gemm_rg16_stream_workspace_bytes(int n, const bpdq_gemv_desc* descs, int tokens)
{
    return n > 0 && descs && tokens > 0 ? rg16_stream_workspace(n, reinterpret_cast<const RgDesc*>(descs), tokens) : 0;
}
void* bpdq_gemm_rg16_stream_create(int n, const bpdq_gemv_desc* descs, int tokens, void* workspace, size_t workspace_bytes)
{
    static_assert(sizeof(bpdq_gemv_desc) == sizeof(RgDesc), "descriptor layouts must match");
    return rg16_stream_create(n, reinterpret_cast<const RgDesc*>(descs), tokens, (uint8_t*)workspace, workspace_bytes);
}
int bpdq_gemm_rg16_stream_run(void* handle, void* stream) { return rg16_stream_run((RgHandle*)handle, (cudaStream_t)stream); }
int bpdq_gemm_rg16_stream_launches(void* handle) { return handle ? 2 * (int)((RgHandle*)handle)->launches.size() : 0; }
void bpdq_gemm_rg16_stream_destroy(void* handle) { rg16_stream_destroy((RgHandle*)handle); }

}  // extern "C"

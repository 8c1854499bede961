// Many-token Q4_K x Q8_K product on the fifth-generation tensor cores (tcgen05, accumulators in
// tensor memory).  Same arithmetic as gemm_q4k_mma.cu and gemv_q4k.cu, every integer exact:
//
//   out[t][n] = sum_b dA_tb * ( d_nb * isum - dmin_nb * msum )
//   isum = sum_j sc_j * dot_j = 8 * sum_k (q_k * sh_j(k)) * x_k + sum_k (q_k * sl_j(k)) * x_k,   sc = 8*sh + sl
//   msum = sum_j mn_j * bsum_j = 64 * sum_j mn_j * bh_j + sum_j mn_j * bl_j,                     bsum = 64*bh + bl
//
// q*sl and q*sh are below 128, mn, bl, bh fit a signed byte, so all four sums are kind::i8 MMAs
// (int8 x int8 -> int32 in TMEM) that accumulate over a whole super-block: D_lo, D_hi over its
// eight K=32 steps, D_ml, D_mh in one step each.  The fp32 scales are applied once per
// super-block by the epilogue warps after tcgen05.ld.
//
// One CTA = 128 weight rows (the MMA M) x all tokens (the MMA N, 16..64), fourteen warps:
//   warps 0-7   transform: two threads per row turn its packed nibbles into the two int8 A planes
//               and store them straight into tensor memory (tcgen05.st: lane = row, one 32-bit
//               column = four K elements), half a super-block at a time.  The A operand never
//               touches shared memory: expanded to two bytes per weight it would cost four times
//               the shared-memory traffic of the packed rows and bound the kernel there.
//   warps 8-11  epilogue: thread r owns TMEM lane r: tcgen05.ld 16 columns of the four
//               accumulators at a time, scale, accumulate up to 64 fp32 outputs in registers
//   warp 12     producer: per super-block one tiled TMA request for the 128 x 144-byte block of
//               raw rows and one bulk copy of the activations' block (the B operand, already in the
//               canonical K-major core-matrix layout: 8 tokens x 16 bytes per 128-byte core matrix,
//               written by k_quant_tc5_acts)
//   warp 13     allocates tensor memory; one lane issues the MMAs and commits to mbarriers
// Rings: raw rows + activations in shared memory (2-6 stages) -> A planes in TMEM (3-4 half-
// super-block stages of 64 columns, plus two 8-column stages for the mins) -> accumulators in
// TMEM (two sets of 4 x tokens columns; one set at 64 tokens, where two would not fit 512 columns).
// All mbarrier waits are bounded; on a timeout the role records an error code and leaves, the
// others time out in turn, and warp 13 frees the tensor memory before it returns.
#include "bpdq_common.cuh"
#include "tcgen05_device.cuh"
#include "../../include/bpdq.h"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace bpdq {

constexpr int kRows = 128;
constexpr int kMaxRawStages = 6, kMaxOpStages = 4, kSideSlots = 8;
constexpr int kOpCols = 64;                        // TMEM columns of one A stage: lo plane 32 (4 sub-blocks x K=32 bytes), hi plane 32
constexpr int kMinCols = 8;                        // one K=32 step: columns 0,1 = the eight mins, rest zero
constexpr int kRowsBytes = kRows * BPDQ_Q4K_BYTES; // 18432

struct Tc5Plan {
    int N, nb, tokens, npad;      // weight rows, super-blocks per row, valid / padded tokens (16, 32 or 64)
    int n_tiles, grid, raw_stages;
    int splits, sb_per_unit, n_units;   // K is cut into `splits` ranges of sb_per_unit super-blocks; unit = (tile, range)
    float* partials;              // [splits][tokens][N] fp32, used when splits > 1
    unsigned* arrivals;           // [n_tiles][2] units of a tile (and token half) that have stored their partial
    int act_bytes;                // scratch bytes per super-block: 324 * npad
    int raw_bytes;                // ring slot: rows + activations
    int off_raw, off_side, off_bar;
    size_t smem;
    unsigned long long* trace;    // tuning aid (BPDQ_TC5_TRACE builds): stamps of CTA 0, [role 0..4][super-block 0..31], or null
    int32_t* ints;                // optional [tokens][N][nb][2]: the exact (isum, msum) of every super-block, or null
};

__device__ __forceinline__ unsigned long long tc5_timer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
    return t;
}
#ifdef BPDQ_TC5_TRACE
#define TC5_TRACE(role, i) do { if (p.trace && blockIdx.x == 0 && (i) < 32) p.trace[(role) * 32 + (i)] = tc5_timer(); } while (0)
#else
#define TC5_TRACE(role, i) do { } while (0)
#endif

// Activation quantizer: warp per (super-block, token).  Scratch per super-block:
//   [256*npad] int8 B operand, canonical: element (tok,k) at (k/16)*16*npad + (tok/8)*128 + (tok%8)*16 + k%16
//   [32*npad]  bl plane, [32*npad] bh plane (K = 32 bytes per token, bytes 0..7 = sub-blocks 0..7, rest 0)
//   [4*npad]   fp32 block scales
__global__ void __launch_bounds__(256) k_quant_tc5_acts(const float* __restrict__ X, uint8_t* __restrict__ scratch,
                                                        int tokens, int npad, int K, unsigned* __restrict__ arrivals,
                                                        int n_arrivals)
{
    // Programmatic launch on both sides: the product's CTAs may start their weight loads while this
    // kernel runs, and this kernel is resident before the launch ahead of it has finished, which it
    // waits for here because that launch may produce X and may still read the scratch.
    pdl_launch_dependents();
    pdl_wait();
    // the split-K arrival counters of the product that follows start at zero
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < n_arrivals; q += gridDim.x * blockDim.x) arrivals[q] = 0u;
    const int nb = K / 256;
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
    const int chunk_stride = 16 * npad;
    for (long u = warp; u < (long)nb * npad; u += n_warps) {
        const int b = (int)(u / npad), t = (int)(u - (long)b * npad);
        uint8_t* base = scratch + (size_t)b * 324 * npad;
        uint8_t* rowp = base + (t >> 3) * 128 + (t & 7) * 16;
        uint32_t p0 = 0, p1 = 0;
        float d = 0.0f;
        if (t < tokens) {
            const float4* xb = reinterpret_cast<const float4*>(X + (size_t)t * K + (size_t)b * 256);
            const float4 v0 = __ldg(xb + lane), v1 = __ldg(xb + 32 + lane);
            float amax = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w)));
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
            amax = warp_max(amax);
            d = __fdiv_rn(amax, 127.0f);
            const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
            auto q = [mul](float x) -> uint32_t { return (uint32_t)__float2int_rn(__fmul_rn(x, mul)) & 0xFFu; };
            p0 = q(v0.x) | (q(v0.y) << 8) | (q(v0.z) << 16) | (q(v0.w) << 24);
            p1 = q(v1.x) | (q(v1.y) << 8) | (q(v1.z) << 16) | (q(v1.w) << 24);
        }
        // word `lane` = elements 4*lane.. -> K-chunk lane/4, byte 4*(lane%4); word 32+lane -> chunk 8 + lane/4
        *reinterpret_cast<uint32_t*>(rowp + (lane >> 2) * chunk_stride + 4 * (lane & 3)) = p0;
        *reinterpret_cast<uint32_t*>(rowp + (8 + (lane >> 2)) * chunk_stride + 4 * (lane & 3)) = p1;
        int s0 = dp4a_ss(p0, 0x01010101u, 0), s1 = dp4a_ss(p1, 0x01010101u, 0);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, o);
            s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
        }
        // gather the eight sub-block sums into every lane, then lane 0 writes the two planes
        uint32_t bl_lo = 0, bl_hi = 0, bh_lo = 0, bh_hi = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int a = __shfl_sync(0xFFFFFFFFu, s0, 8 * j), c = __shfl_sync(0xFFFFFFFFu, s1, 8 * j);
            bl_lo |= (uint32_t)(a & 63) << (8 * j);
            bh_lo |= ((uint32_t)(a >> 6) & 0xFFu) << (8 * j);
            bl_hi |= (uint32_t)(c & 63) << (8 * j);
            bh_hi |= ((uint32_t)(c >> 6) & 0xFFu) << (8 * j);
        }
        uint8_t* blp = base + 256 * npad + (t >> 3) * 128 + (t & 7) * 16;
        uint8_t* bhp = blp + 32 * npad;
        if (lane == 0) {
            *reinterpret_cast<uint4*>(blp) = make_uint4(bl_lo, bl_hi, 0, 0);
            *reinterpret_cast<uint4*>(blp + chunk_stride) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(bhp) = make_uint4(bh_lo, bh_hi, 0, 0);
            *reinterpret_cast<uint4*>(bhp + chunk_stride) = make_uint4(0, 0, 0, 0);
            reinterpret_cast<float*>(base + 320 * npad)[t] = d;
        }
    }
}

// Warp roles per padded token count.  Sixteen transform warps (four threads per weight row) hide the
// shared-memory and tcgen05.st latencies; at 64 tokens the epilogue is the heavier side and gets
// eight warps (two per TMEM lane quadrant, half of the columns each) while the transform keeps eight.
template <int NPAD> struct Tc5Shape {
    static constexpr int kTransformWarps = NPAD == 64 ? 8 : 16;
    static constexpr int kEpilogueWarps = NPAD == 64 ? 8 : 4;
    static constexpr int kThreads = (kTransformWarps + kEpilogueWarps + 2) * 32;
};

template <int NPAD>
__global__ void __launch_bounds__(Tc5Shape<NPAD>::kThreads, 1)
k_gemm_q4k_q8k_tc5(const __grid_constant__ CUtensorMap wmap, const uint8_t* __restrict__ acts, float* __restrict__ out,
                   const Tc5Plan p, int* __restrict__ err)
{
    constexpr int kTransformWarps = Tc5Shape<NPAD>::kTransformWarps;
    constexpr int kEpilogueWarps = Tc5Shape<NPAD>::kEpilogueWarps;
    constexpr int kProducerWarp = kTransformWarps + kEpilogueWarps, kMmaWarp = kProducerWarp + 1;
    // transform warps work in groups of eight (two threads per weight row, two sub-blocks each per half
    // super-block); with two groups they take alternate super-blocks, so that one group's chain of
    // waits, loads, stores and arrivals overlaps the other's
    constexpr int kGroups = kTransformWarps / 8;
    constexpr int kParts = 2, kSubs = 2;
    // Two accumulator sets of four (lo, hi, ml, mh) x kAccCols columns.  Up to 32 tokens they alternate by
    // super-block; at 64 tokens two such pairs would not fit 512 columns, so the sets are the two token halves:
    // each super-block is issued as two passes of N = 32 over the same A operand, and the epilogue of one
    // half runs while the other half's MMAs execute.
    constexpr int kPasses = NPAD == 64 ? 2 : 1;
    constexpr int kAccCols = NPAD / kPasses;                // MMA N = token columns per accumulator
    constexpr int kEpiCols = kAccCols;                      // token columns per epilogue warp
    static_assert(kEpilogueWarps == 4 * kPasses, "one epilogue warp per TMEM lane quadrant and pass");
    // tensor-memory columns: accumulator sets, then the A stages, then the two mins stages
    constexpr int kAccSets = 2;
    constexpr int kOpStages = NPAD == 16 ? 4 : 3;
    constexpr uint32_t kColOps = kAccSets * 4 * kAccCols;
    constexpr uint32_t kColMins = kColOps + kOpStages * kOpCols;
    static_assert(kColMins + 2 * kMinCols <= 512, "tensor memory has 512 columns");
    static_assert(kOpStages <= kMaxOpStages && kOpStages <= 4, "a mins stage is reused two super-blocks later");

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* raw = smem + p.off_raw;
    float* side = reinterpret_cast<float*>(smem + p.off_side);   // [kSideSlots][256 hdr floats + NPAD dA floats]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);
    const int kRawStages = p.raw_stages;
    uint64_t* w_full = bars;                         // [raw_stages] weight rows of a slot have landed (TMA bytes)
    uint64_t* a_full = w_full + kMaxRawStages;       // [raw_stages] activation block of a slot has landed
    uint64_t* raw_empty = a_full + kMaxRawStages;    // MMA commit (its MMAs follow the transform's reads of the slot)
    uint64_t* xf_full = raw_empty + kMaxRawStages;   // [2] by super-block parity: the eight warps of a transform group
    uint64_t* op_empty = xf_full + 2;                // [kOpStages] MMA commit
    uint64_t* acc_full = op_empty + kMaxOpStages;    // [kAccSets] MMA commit + the issuer's arrival after it wrote the token scales
    uint64_t* acc_empty = acc_full + 2;              // epilogue warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    constexpr int kSideFloats = 256 + NPAD;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kMaxRawStages; s++) { mbar_init(&w_full[s], 1); mbar_init(&a_full[s], 1); mbar_init(&raw_empty[s], 1); }
        for (int s = 0; s < kMaxOpStages; s++) mbar_init(&op_empty[s], 1);
        for (int s = 0; s < 2; s++) { mbar_init(&xf_full[s], 8); mbar_init(&acc_full[s], 2); mbar_init(&acc_empty[s], 4); }
        mbar_init_fence();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    // Everything up to here, the weight loads of the first ring round and their transform overlap the
    // activation quantizer launched just before this kernel: only what that kernel wrote (the
    // activation blocks, the split-K counters) waits for it, in the producer and the epilogue warps.

    const int my_units = (p.n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total_sb = my_units * p.sb_per_unit;   // super-blocks this CTA walks, over all its units

    if (warp == kProducerWarp) {
        // ---------------- producer
        if (lane == 0) {
            // two walks over the same sequence of (tile, super-block): weights may run ahead of the
            // activations by the ring's depth, and do so before the quantizer has finished
            struct Walk { int q, unit, tile, b; };
            auto start = [&]() { Walk w; w.q = 0; w.unit = blockIdx.x; w.tile = w.unit / p.splits; w.b = (w.unit - w.tile * p.splits) * p.sb_per_unit; return w; };
            auto step = [&](Walk& w) {
                w.b++;
                if (++w.q == p.sb_per_unit) {
                    w.q = 0;
                    w.unit += gridDim.x;
                    w.tile = w.unit / p.splits;
                    w.b = (w.unit - w.tile * p.splits) * p.sb_per_unit;
                }
            };
            Walk ww = start(), wa = start();
            const int ahead = total_sb < kRawStages ? total_sb : kRawStages;
            for (int i = 0; i < ahead; i++) {
                mbar_expect_tx(&w_full[i], (uint32_t)kRowsBytes);
                tma_rows_2d(raw + (size_t)i * p.raw_bytes, &wmap, ww.b * (BPDQ_Q4K_BYTES / 4), ww.tile * kRows, &w_full[i]);
                TC5_TRACE(0, i);
                step(ww);
            }
            pdl_wait();
            int s = 0;
            uint32_t par = 1;   // parity of the consumers' release one round of stages back
            for (int i = 0; i < total_sb; i++) {
                uint8_t* slot = raw + (size_t)s * p.raw_bytes;
                if (i >= kRawStages) {
                    if (!mbar_wait_sleepy(&raw_empty[s], par, err, 11)) break;
                    mbar_expect_tx(&w_full[s], (uint32_t)kRowsBytes);
                    tma_rows_2d(slot, &wmap, ww.b * (BPDQ_Q4K_BYTES / 4), ww.tile * kRows, &w_full[s]);
                    TC5_TRACE(0, i);
                    step(ww);
                }
                mbar_expect_tx(&a_full[s], (uint32_t)p.act_bytes);
                bulk_g2s(slot + kRowsBytes, acts + (size_t)wa.b * p.act_bytes, (uint32_t)p.act_bytes, &a_full[s]);
                step(wa);
                if (++s == kRawStages) { s = 0; par ^= 1u; }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer.  The whole warp walks the loop so that addresses, descriptors and
        // ring counters stay warp-uniform (the MMA takes them from uniform registers); one elected lane issues.
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kAccCols >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        const uint64_t b_desc0 = umma_desc(smem_addr(raw + kRowsBytes), 16 * NPAD, 128);
        const uint32_t b_step = (uint32_t)p.raw_bytes >> 4;
        int s = 0, o = 0;
        uint32_t raw_par = 0;
        bool gave_up = false;
        for (int i = 0; i < total_sb && !gave_up; i++) {
            if (!mbar_wait_bounded(&a_full[s], raw_par, err, 12)) break;
            // the tokens' block scales go from the activation block to the side ring for the epilogue
            {
                const float* dA = reinterpret_cast<const float*>(raw + (size_t)s * p.raw_bytes + kRowsBytes + 320 * NPAD);
                float* sd = side + (size_t)(i % kSideSlots) * kSideFloats + 256;
#pragma unroll
                for (int q = lane; q < NPAD; q += 32) sd[q] = dA[q];
            }
            if (!mbar_wait_bounded(&xf_full[i & 1], (uint32_t)(i >> 1) & 1u, err, 14)) break;
            __syncwarp();
            TC5_TRACE(5, i);
            const int o1 = (o + 1 == kOpStages) ? 0 : o + 1;
#pragma unroll
            for (int pass = 0; pass < kPasses; pass++) {
                // set and the parity of its release by the epilogue one use back
                const int a = kPasses == 2 ? pass : (i & 1);
                const int use = kPasses == 2 ? i : (i >> 1);
                if (use >= 1 && !mbar_wait_bounded(&acc_empty[a], (uint32_t)(use - 1) & 1u, err, 13)) { gave_up = true; break; }
                if (pass == 0) TC5_TRACE(9, i);
                // first of the two arrivals on acc_full: publishes the side ring's scales (and, through the
                // transform's arrival seen above, its d/dmin) to the epilogue; the MMA commit is the second
                if (lane == 0) mbar_arrive(&acc_full[a]);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // the B descriptors differ only in their 14-bit start-address field (bytes >> 4); tokens
                // 32.. of the second pass start four 128-byte core matrices further on
                const uint64_t b_base = b_desc0 + (uint64_t)((uint32_t)s * b_step + (uint32_t)pass * (4u * 128u >> 4));
                const uint32_t d_lo = tmem_base + (uint32_t)(a * 4) * kAccCols, d_hi = d_lo + kAccCols;
                const uint32_t d_ml = d_lo + 2 * kAccCols, d_mh = d_lo + 3 * kAccCols;
                if (elect_one()) {
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int oh = half ? o1 : o;
                        const uint32_t a_lo = tmem_base + kColOps + (uint32_t)oh * kOpCols, a_hi = a_lo + 32;
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const int j = 4 * half + k;   // sub-block: K-chunks 2j, 2j+1 of the B operand
                            const uint64_t bdesc = b_base + (uint64_t)((2 * j * 16 * NPAD) >> 4);
                            if (half == 0 && k == 0) {
                                umma_i8_ts<0>(d_lo, a_lo, bdesc, idesc);
                                umma_i8_ts<0>(d_hi, a_hi, bdesc, idesc);
                            } else {
                                umma_i8_ts<1>(d_lo, a_lo + 8 * k, bdesc, idesc);
                                umma_i8_ts<1>(d_hi, a_hi + 8 * k, bdesc, idesc);
                            }
                        }
                        if (half == 1) {
                            const uint32_t a_mn = tmem_base + kColMins + (uint32_t)(i & 1) * kMinCols;
                            umma_i8_ts<0>(d_ml, a_mn, b_base + (uint64_t)((256 * NPAD) >> 4), idesc);
                            umma_i8_ts<0>(d_mh, a_mn, b_base + (uint64_t)((288 * NPAD) >> 4), idesc);
                        }
                        if (pass == kPasses - 1) umma_commit(&op_empty[oh]);
                    }
                    if (pass == kPasses - 1) umma_commit(&raw_empty[s]);
                    umma_commit(&acc_full[a]);
                }
                __syncwarp();
            }
            TC5_TRACE(2, i);
            o = (o1 + 1 == kOpStages) ? 0 : o1 + 1;
            if (++s == kRawStages) { s = 0; raw_par ^= 1u; }
        }
    } else if (warp < kTransformWarps) {
        // ---------------- transform: two threads share row r of the tile (kSubs sub-blocks each per half);
        // warp w may touch TMEM lanes 32*(w%4)..+31, which are its rows
        const int group = warp >> 3, part = (warp >> 2) & 1;
        const int r = 32 * (warp & 3) + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
        int s = group, o = (2 * group) % kOpStages;
        uint32_t raw_par = 0, op_par = 1;   // op_par: parity of the issuer's release one round of stages back
        for (int i = group; i < total_sb; i += kGroups) {
            if (!mbar_wait_sleepy(&w_full[s], raw_par, err, 15)) break;
            if ((tid & 255) == 0) TC5_TRACE(1, i);
            // both A stages of this super-block must be free
            const int o1 = (o + 1 == kOpStages) ? 0 : o + 1;
            const uint32_t op_par1 = (o + 1 == kOpStages) ? op_par ^ 1u : op_par;
            // (the issuer commits in order: the release of the second stage implies that of the first)
            if (2 * i + 1 >= kOpStages && !mbar_wait_sleepy(&op_empty[o1], op_par1, err, 16)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint8_t* slot = raw + (size_t)s * p.raw_bytes;
            const uint8_t* row = slot + (size_t)r * BPDQ_Q4K_BYTES;
            const uint4 hdr = *reinterpret_cast<const uint4*>(row);
            uint4 qv[2][kSubs];
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int kk = 0; kk < kSubs; kk++)
                    qv[half][kk] = *reinterpret_cast<const uint4*>(row + 16 + 64 * half + 16 * (kSubs * part + kk));
            float* sd = side + (size_t)(i % kSideSlots) * kSideFloats;
            if (part == 0)
                *reinterpret_cast<float2*>(sd + 2 * r) = make_float2(f16_bits_to_f32(hdr.x & 0xFFFFu), f16_bits_to_f32(hdr.x >> 16));
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t lo[8 * kSubs], hi[8 * kSubs];
                uint32_t sc4 = 0;
                if (kSubs > 1) {
                    uint32_t mn4;
                    q4k_scales4(hdr.y, hdr.z, hdr.w, half, sc4, mn4);
                }
#pragma unroll
                for (int kk = 0; kk < kSubs; kk++) {
                    const int k = kSubs * part + kk;
                    const uint4 q = qv[half][kk];
                    uint32_t sc;
                    if (kSubs > 1) {
                        sc = byte_of(sc4, k);
                    } else {
                        // the one 6-bit scale of sub-block 4*half + part: byte `part` of the scale words
                        const uint32_t y = hdr.y >> (8 * part);
                        sc = half == 0 ? (y & 63u) : (((hdr.w >> (8 * part)) & 0xFu) | ((y >> 2) & 0x30u));
                    }
                    const uint32_t sl = sc & 7u, sh = sc >> 3;
                    const uint32_t l0 = q.x & 0x0F0F0F0Fu, l1 = q.y & 0x0F0F0F0Fu, l2 = q.z & 0x0F0F0F0Fu, l3 = q.w & 0x0F0F0F0Fu;
                    const uint32_t h0 = (q.x >> 4) & 0x0F0F0F0Fu, h1 = (q.y >> 4) & 0x0F0F0F0Fu, h2 = (q.z >> 4) & 0x0F0F0F0Fu,
                                   h3 = (q.w >> 4) & 0x0F0F0F0Fu;
                    // columns 0..3 of a K=32 step = elements 0..15 of the sub-block (low nibbles), 4..7 = elements 16..31 (high)
                    lo[8 * kk + 0] = l0 * sl; lo[8 * kk + 1] = l1 * sl; lo[8 * kk + 2] = l2 * sl; lo[8 * kk + 3] = l3 * sl;
                    lo[8 * kk + 4] = h0 * sl; lo[8 * kk + 5] = h1 * sl; lo[8 * kk + 6] = h2 * sl; lo[8 * kk + 7] = h3 * sl;
                    hi[8 * kk + 0] = l0 * sh; hi[8 * kk + 1] = l1 * sh; hi[8 * kk + 2] = l2 * sh; hi[8 * kk + 3] = l3 * sh;
                    hi[8 * kk + 4] = h0 * sh; hi[8 * kk + 5] = h1 * sh; hi[8 * kk + 6] = h2 * sh; hi[8 * kk + 7] = h3 * sh;
                }
                const uint32_t a_lo = lane_base + kColOps + (uint32_t)(half ? o1 : o) * kOpCols + (uint32_t)(8 * kSubs) * (uint32_t)part;
                tmem_st(a_lo, lo);
                tmem_st(a_lo + 32, hi);
            }
            op_par = op_par1;
            o = o1;
#pragma unroll
            for (int q = 0; q < 2 * kGroups - 1; q++)
                if (++o == kOpStages) { o = 0; op_par ^= 1u; }
            if (part == kParts - 1) {
                uint32_t sca, mna, scb, mnb;
                q4k_scales4(hdr.y, hdr.z, hdr.w, 0, sca, mna);
                q4k_scales4(hdr.y, hdr.z, hdr.w, 1, scb, mnb);
                const uint32_t mins[8] = {mna, mnb, 0, 0, 0, 0, 0, 0};    // mins of sub-blocks 0..7, then zero K padding
                tmem_st(lane_base + kColMins + (uint32_t)(i & 1) * kMinCols, mins);
            }
            // the stores must have landed before the issuer's MMAs may read them
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&xf_full[i & 1]);
            if ((tid & 255) == 0) TC5_TRACE(3, i);
            s += kGroups;
            if (s >= kRawStages) { s -= kRawStages; raw_par ^= 1u; }
        }
    } else {
        // ---------------- epilogue: a thread owns one TMEM lane (output row) and kEpiCols token columns
        const int e = warp - kTransformWarps, pass = e >> 2;
        const int r = 32 * (e & 3) + lane, c0 = pass * kEpiCols;
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * (e & 3)) << 16);
        float facc[kEpiCols];
        int i = 0;
        int* last_flag = reinterpret_cast<int*>(tmem_slot + 2) + pass;
        pdl_wait();   // the quantizer zeroed the split-K counters
        for (int ul = 0; ul < my_units; ul++) {
#pragma unroll
            for (int t = 0; t < kEpiCols; t++) facc[t] = 0.0f;
            bool gave_up = false;
            const int unit = blockIdx.x + ul * gridDim.x;
            const int tile = unit / p.splits, split = unit - tile * p.splits;
            const int rowg = tile * kRows + r;
            for (int b = 0; b < p.sb_per_unit; b++, i++) {
                const int a = kPasses == 2 ? pass : (i & 1);
                const int use = kPasses == 2 ? i : (i >> 1);
                if (!mbar_wait_sleepy(&acc_full[a], (uint32_t)use & 1u, err, 17)) { gave_up = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float* sd = side + (size_t)(i % kSideSlots) * kSideFloats;
                const float2 dd = *reinterpret_cast<const float2*>(sd + 2 * r);
                const float d = dd.x, dmin = dd.y;
                const uint32_t col0 = lane_base + (uint32_t)(a * 4) * kAccCols;
#pragma unroll
                for (int c = 0; c < kEpiCols / 8; c++) {
                    int lo[8], hi[8], ml[8], mh[8];
                    tmem_ld(col0 + 8 * c, lo);
                    tmem_ld(col0 + kAccCols + 8 * c, hi);
                    tmem_ld(col0 + 2 * kAccCols + 8 * c, ml);
                    tmem_ld(col0 + 3 * kAccCols + 8 * c, mh);
                    const float4 dA0 = *reinterpret_cast<const float4*>(sd + 256 + c0 + 8 * c);
                    const float4 dA1 = *reinterpret_cast<const float4*>(sd + 256 + c0 + 8 * c + 4);
                    const float dA[8] = {dA0.x, dA0.y, dA0.z, dA0.w, dA1.x, dA1.y, dA1.z, dA1.w};
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int t = 0; t < 8; t++) {
                        const float v = d * (float)(8 * hi[t] + lo[t]) - dmin * (float)(64 * mh[t] + ml[t]);
                        facc[8 * c + t] = fmaf(dA[t], v, facc[8 * c + t]);
                    }
                    if (p.ints && rowg < p.N) {
#pragma unroll
                        for (int t = 0; t < 8; t++)
                            if (c0 + 8 * c + t < p.tokens)
                                *reinterpret_cast<int2*>(p.ints + (((size_t)(c0 + 8 * c + t) * p.N + rowg) * p.nb + (split * p.sb_per_unit + b)) * 2) =
                                    make_int2(8 * hi[t] + lo[t], 64 * mh[t] + ml[t]);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[a]);
                if (tid == 32 * kTransformWarps) TC5_TRACE(4, i);
            }
            if (gave_up) break;
            if (p.splits == 1) {
                if (rowg < p.N) {
#pragma unroll
                    for (int t = 0; t < kEpiCols; t++)
                        if (c0 + t < p.tokens) out[(size_t)(c0 + t) * p.N + rowg] = facc[t];
                }
            } else {
                // split K: store this range's partial sums; the unit that arrives last adds the ranges in
                // their fixed order 0, 1, ..., so the result does not depend on which one that was
                if (rowg < p.N) {
#pragma unroll
                    for (int t = 0; t < kEpiCols; t++)
                        if (c0 + t < p.tokens) __stcg(p.partials + ((size_t)split * p.tokens + (c0 + t)) * p.N + rowg, facc[t]);
                }
                __threadfence();
                named_bar_sync(1 + pass, 128);
                if ((e & 3) == 0 && lane == 0) {
                    const unsigned before = atomicAdd(p.arrivals + 2 * tile + pass, 1u);
                    *last_flag = (before == (unsigned)p.splits - 1u) ? 1 : 0;
                }
                named_bar_sync(1 + pass, 128);
                const bool last = *last_flag != 0;
                named_bar_sync(1 + pass, 128);   // everybody has read the flag before the next unit rewrites it
                if (last) {
                    __threadfence();
                    if (rowg < p.N) {
                        // four tokens x up to eight ranges of loads in flight, then the sums in range order
#pragma unroll 1
                        for (int t0 = 0; t0 < kEpiCols && c0 + t0 < p.tokens; t0 += 4) {
                            float v[4][8];
#pragma unroll
                            for (int tt = 0; tt < 4; tt++)
#pragma unroll
                                for (int q = 0; q < 8; q++)
                                    v[tt][q] = (q < p.splits && c0 + t0 + tt < p.tokens)
                                                   ? __ldcg(p.partials + ((size_t)q * p.tokens + (c0 + t0 + tt)) * p.N + rowg)
                                                   : 0.0f;
#pragma unroll
                            for (int tt = 0; tt < 4; tt++) {
                                float sum = 0.0f;
#pragma unroll
                                for (int q = 0; q < 8; q++)
                                    if (q < p.splits) sum += v[tt][q];
                                if (c0 + t0 + tt < p.tokens) out[(size_t)(c0 + t0 + tt) * p.N + rowg] = sum;
                            }
                        }
                    }
                }
            }
        }
    }
    // ---------------- teardown: everybody meets, then the allocating warp frees tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

#ifdef BPDQ_TC5_TRACE
static unsigned long long* g_tc5_trace = nullptr;
#endif

static int tc5_weight_map(CUtensorMap* map, const uint8_t* W, int N, int nb)
{
    static PFN_cuTensorMapEncodeTiled encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return latch(BPDQ_ERR_CUDA);
        encode = (PFN_cuTensorMapEncodeTiled)fn;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)nb * (BPDQ_Q4K_BYTES / 4), (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)nb * BPDQ_Q4K_BYTES};
    const cuuint32_t box[2] = {(cuuint32_t)(BPDQ_Q4K_BYTES / 4), (cuuint32_t)kRows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(W), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : latch(BPDQ_ERR_CUDA - 900 - (int)r);
}

template <int NPAD>
static int launch_tc5(const CUtensorMap& wmap, const uint8_t* acts, float* out, const Tc5Plan& p, cudaStream_t s)
{
    auto kern = k_gemm_q4k_q8k_tc5<NPAD>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(Tc5Shape<NPAD>::kThreads);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, wmap, acts, out, p, device_error_flag()));
}

// out[tokens][N], X fp32 [tokens][K], C-ABI nibble order; N >= 128 rows (the TMA box), up to 64 tokens per pass.
int gemm_q4k_q8k_tc5(const uint8_t* W, const float* X, float* out, int tokens, int N, int K, cudaStream_t s, Workspace* ws,
                     int32_t* sb_ints)
{
    if (tokens < 0 || N < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (tokens == 0 || N == 0) return 0;
    if (!W || !X || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)W & 15) || ((uintptr_t)X & 15) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    if (N < kRows) return latch(BPDQ_ERR_RANGE);
    CUtensorMap wmap;
    int rc = tc5_weight_map(&wmap, W, N, K / 256);
    if (rc) return rc;
    for (int t0 = 0; t0 < tokens; t0 += 64) {
        const int T = tokens - t0 < 64 ? tokens - t0 : 64;
        Tc5Plan p;
        p.N = N;
        p.nb = K / 256;
        p.tokens = T;
#ifdef BPDQ_TC5_TRACE
        p.trace = g_tc5_trace;
#else
        p.trace = nullptr;
#endif
        p.ints = sb_ints ? sb_ints + (size_t)t0 * N * p.nb * 2 : nullptr;
        p.npad = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
        p.n_tiles = (N + kRows - 1) / kRows;
        // Split K so that every SM has work and the per-CTA chain of super-blocks is short: pick the
        // number of ranges (a power of two dividing the super-blocks per row, at least two per range)
        // with the fewest super-block steps on the busiest SM, charging each unit two steps of set-up.
        p.splits = 1;
        {
            long best = -1;
            for (int sp = 1; sp <= 8; sp *= 2) {
                if (p.nb % sp != 0 || p.nb / sp < 2) break;
                const long units = (long)p.n_tiles * sp;
                const long waves = (units + sm_count() - 1) / sm_count();
                const long cost = waves * (p.nb / sp + 2);
                if (best < 0 || cost < best) { best = cost; p.splits = sp; }
            }
        }
        p.sb_per_unit = p.nb / p.splits;
        p.n_units = p.n_tiles * p.splits;
        p.grid = p.n_units < sm_count() ? p.n_units : sm_count();
        p.act_bytes = 324 * p.npad;
        p.raw_bytes = (kRowsBytes + p.act_bytes + 127) / 128 * 128;
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        const size_t fixed = ((size_t)kSideSlots * (256 + p.npad) * 4 + 127) / 128 * 128 + 256;
        p.raw_stages = (int)((227 * 1024 - fixed) / p.raw_bytes);
        if (p.raw_stages > kMaxRawStages) p.raw_stages = kMaxRawStages;
        if (p.raw_stages < 2) return latch(BPDQ_ERR_RANGE);
        p.off_raw = take((size_t)p.raw_stages * p.raw_bytes);
        p.off_side = take((size_t)kSideSlots * (256 + p.npad) * 4);
        p.off_bar = take(256);
        p.smem = off;
        if (p.smem > 227 * 1024) return latch(BPDQ_ERR_RANGE);
        // every pass of 64 tokens uses the same scratch: the quantizer waits for the pass before it
        Workspace pass_ws = ws ? *ws : Workspace{nullptr, 0, 0};
        int src = 0;
        uint8_t* acts = scratch_take(ws ? &pass_ws : nullptr, kScratchTc5Acts, (size_t)p.nb * p.act_bytes, s, &src);
        if (!acts) return src;
        const size_t arrivals_bytes = ((size_t)p.n_tiles * 2 * sizeof(unsigned) + 255) / 256 * 256;
        uint8_t* red = scratch_take(ws ? &pass_ws : nullptr, kScratchTc5Reduce,
                                    arrivals_bytes + (p.splits > 1 ? (size_t)p.splits * T * N * sizeof(float) : 0), s, &src);
        if (!red) return src;
        p.arrivals = reinterpret_cast<unsigned*>(red);
        p.partials = reinterpret_cast<float*>(red + arrivals_bytes);
        const long units = (long)p.nb * p.npad;
        long want = (units + 7) / 8, cap = (long)sm_count() * 8;
        {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(want < cap ? want : cap));
            cfg.blockDim = dim3(256);
            cfg.stream = s;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = at;
            cfg.numAttrs = tuning().pdl ? 1 : 0;
            rc = check_cuda(cudaLaunchKernelEx(&cfg, k_quant_tc5_acts, (const float*)(X + (size_t)t0 * K), acts, T, p.npad, K,
                                               p.arrivals, p.n_tiles * 2));
            if (rc) return rc;
        }
        float* o = out + (size_t)t0 * N;
        rc = p.npad == 16 ? launch_tc5<16>(wmap, acts, o, p, s) : (p.npad == 32 ? launch_tc5<32>(wmap, acts, o, p, s) : launch_tc5<64>(wmap, acts, o, p, s));
        if (rc) return latch(rc);
    }
    return 0;
}

// scratch bytes of gemm_q4k_q8k_tc5 (an upper bound: widest token padding, eight K ranges)
size_t gemm_q4k_q8k_tc5_workspace(int tokens, int N, int K)
{
    const int T = tokens < 64 ? tokens : 64;
    const int n_tiles = (N + kRows - 1) / kRows;
    return (size_t)(K / 256) * 324 * 64 + 256 + ((size_t)n_tiles * 2 * sizeof(unsigned) + 255) / 256 * 256 +
           (size_t)8 * T * N * sizeof(float) + 512;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {
#ifdef BPDQ_TC5_TRACE
// Tuning aid of trace builds: CTA 0 of later tcgen05 launches writes 5 x 32 clock stamps to dev_buf; NULL stops.
void bpdq_debug_trace_tc5(void* dev_buf) { g_tc5_trace = (unsigned long long*)dev_buf; }
#endif
// The tcgen05 kernel directly (bpd_qmm_q4k_q8k_cuda's dispatcher decides when to use it).
int bpd_qmm_q4k_q8k_tc5_cuda(const uint8_t* qweight, const float* X, float* out, int tokens, int M, int K, void* stream)
{
    return gemm_q4k_q8k_tc5(qweight, X, out, tokens, M, K, (cudaStream_t)stream);
}
// Checking forms of the two tensor-core kernels: besides out they store, for every (token, row, super-block), the
// exact int32 pair (isum, msum) that the fp32 scales are applied to; sb_ints is [tokens][M][K/256][2].
int bpd_qmm_q4k_q8k_tc5_ints_cuda(const uint8_t* qweight, const float* X, float* out, int32_t* sb_ints, int tokens, int M, int K,
                                  void* stream)
{
    if (!sb_ints || ((uintptr_t)sb_ints & 7)) return latch(sb_ints ? BPDQ_ERR_ALIGN : BPDQ_ERR_ARG);
    return gemm_q4k_q8k_tc5(qweight, X, out, tokens, M, K, (cudaStream_t)stream, nullptr, sb_ints);
}
int bpd_qmm_q4k_q8k_mma_ints_cuda(const uint8_t* qweight, const float* X, float* out, int32_t* sb_ints, int tokens, int M, int K,
                                  void* stream)
{
    if (!sb_ints || ((uintptr_t)sb_ints & 7)) return latch(sb_ints ? BPDQ_ERR_ALIGN : BPDQ_ERR_ARG);
    return gemm_q4k_q8k_mma(qweight, X, out, tokens, M, K, (cudaStream_t)stream, nullptr, sb_ints);
}
}

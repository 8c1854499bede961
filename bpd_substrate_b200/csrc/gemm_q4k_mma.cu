// Batched Q4_K x Q8_K product for many tokens: int8 tensor-core MMA on raw nibbles.
//
// out[t][n] = sum_b dA_tb * ( d_nb * isum - dmin_nb * msum ),
//   isum = sum_j sc_j * sum_{k in sub-block j} q_k * x_k,   msum = sum_j mn_j * bsum_tj
// (the definition of gemv_q4k.cu; every integer is exact).  A sub-block is exactly the K depth
// of one mma.sync.m16n8k32 (s8 x s8 -> s32): the raw nibbles 0..15 are the A operand, built in
// registers straight from the packed bytes (thread (g,t) needs word t of the 16-byte
// sub-block of rows g and g+8: low nibbles are k = 4t..4t+3, high nibbles k = 16+4t..), the
// int8 activations the B operand; the 6-bit scale multiplies the int32 result (4 IMAD per
// MMA), and the min term uses the activations' sub-block sums with dp2a.  A warp owns 16
// weight rows and all tokens (NT n-tiles of 8).
//
// Data movement: activations are quantized once by k_quant_gemm_acts into global scratch laid
// out [K/256][tokens_padded][288 B]: 256 int8 (words permuted so that a thread's two B words
// are adjacent: one 8-byte read, conflict-free at this pitch), fp32 scale, eight int16
// sub-block sums.  A CTA of W warps (16*W rows) walks K in stages of two super-blocks; per
// stage the producer issues TWO requests: a tiled TMA copy (cp.async.bulk.tensor.2d, box
// 288 bytes x 16*W rows of the [N][K/256*144] byte matrix; rows past the end are zero-filled)
// and one bulk copy of the stage's activations, into a ring with full/empty mbarriers.
// Accumulation order: super-blocks ascending, one fp32 accumulator per output,
// acc = fma(dA, d * float(isum) - dmin * float(msum), acc).
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace bpdq {

constexpr int kActPitch = 288;     // bytes per (super-block, token) in scratch and in shared memory
constexpr int kSbPerStage = 2;

struct GemmPlan {
    int N, K, nb, tokens, tok_pad;   // weight rows, K, super-blocks per row, valid tokens, padded tokens (8*NT)
    int warps;                       // consumer warps per CTA = row groups (16 rows each) x ts
    int ts;                          // warps that share a row group, each taking NT n-tiles of the tokens
    int stages, n_tiles, grid;
    int stage_bytes, act_bytes;      // bytes per ring slot, of which activations
    int row_pitch, box_rows;         // TMA box: bytes per row piece (144 or 288), rows (<= N)
    size_t smem;
    int32_t* ints;                   // optional [tokens][N][nb][2]: the exact (isum, msum) of every super-block, or null
};

// D = A x B (no accumulator input: the C operand is the zero register)
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// Activation quantizer for the GEMM path: one warp per (token, super-block); writes the
// 288-byte record at [b][t] (tokens >= `tokens` up to tok_pad are written as zeros).  Word w of
// the 64 quant words (elements 4w..4w+3) is stored at position 8*(w/8) + 2*(w%4) + (w%8)/4, so
// that words 8j+t and 8j+4+t (one thread's B fragment of sub-block j) sit side by side.
__global__ void __launch_bounds__(256) k_quant_gemm_acts(const float* __restrict__ X, uint8_t* __restrict__ scratch,
                                                         int tokens, int tok_pad, int K)
{
    // Programmatic launch on both sides: the product's CTAs may set up while this kernel runs, and this
    // kernel is resident before the launch ahead of it has finished, which it waits for here because
    // that launch may produce X and may still read the scratch.
    pdl_launch_dependents();
    pdl_wait();
    const int nb = K / 256;
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
    for (long u = warp; u < (long)nb * tok_pad; u += n_warps) {
        const int b = (int)(u / tok_pad), t = (int)(u - (long)b * tok_pad);
        uint32_t* rec = reinterpret_cast<uint32_t*>(scratch + ((size_t)b * tok_pad + t) * kActPitch);
        if (t >= tokens) {
            rec[lane] = 0;
            rec[32 + lane] = 0;
            if (lane < 8) rec[64 + lane] = 0;
            continue;
        }
        const float4* xb = reinterpret_cast<const float4*>(X + (size_t)t * K + (size_t)b * 256);
        const float4 v0 = __ldg(xb + lane), v1 = __ldg(xb + 32 + lane);
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
        // sub-block sums: sub-block j = words 8j..8j+7 = 8 consecutive lanes
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

__device__ __forceinline__ int dp2a_lo(uint32_t a16x2, uint32_t b8x4, int c)
{
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a16x2), "r"(b8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi(uint32_t a16x2, uint32_t b8x4, int c)
{
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a16x2), "r"(b8x4), "r"(c));
    return d;
}
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_addr(dst_smem)),
        "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}

template <int NT>
__global__ void __launch_bounds__(544, 1)
k_gemm_q4k_q8k_mma(const __grid_constant__ CUtensorMap wmap, const uint8_t* __restrict__ acts, float* __restrict__ out,
                   const GemmPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + p.stages;
    uint8_t* ring = smem + 128;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool is_producer = warp == p.warps;
    const int rows_per_cta = 16 * (p.warps / p.ts);
    const int rg = warp / p.ts;                 // row group of this warp
    const int tok0 = (warp % p.ts) * 8 * NT;    // first token of this warp
    const int n_stage_steps = (p.nb + kSbPerStage - 1) / kSbPerStage;   // stages per row tile

    if (tid == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.warps);
        }
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();   // activations in scratch come from the quantizer launched just before

    if (is_producer) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
                const int row0 = tile * rows_per_cta;
                for (int st = 0; st < n_stage_steps; st++, it++) {
                    const int s = it % p.stages;
                    if (it >= p.stages && !mbar_wait_bounded(&empty[s], ((it / p.stages) - 1) & 1, err, 1)) return;
                    const int sb0 = st * kSbPerStage;
                    const int nsb = min(kSbPerStage, p.nb - sb0);
                    uint8_t* slot = ring + (size_t)s * p.stage_bytes;
                    const uint32_t act_bytes = (uint32_t)nsb * p.tok_pad * kActPitch;
                    // the box is always whole: columns past the row end and rows past N arrive as zeros
                    mbar_expect_tx(&full[s], act_bytes + (uint32_t)p.box_rows * p.row_pitch);
                    bulk_g2s(slot, acts + (size_t)sb0 * p.tok_pad * kActPitch, act_bytes, &full[s]);
                    // x coordinate in 4-byte elements: 36 words per super-block (a multiple of 16 bytes)
                    tma_load_2d(slot + p.act_bytes, &wmap, sb0 * (BPDQ_Q4K_BYTES / 4), row0, &full[s]);
                }
            }
        }
        return;
    }

    int it = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
        const int row0 = tile * rows_per_cta + 16 * rg;
        float facc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) facc[n][i] = 0.0f;

        for (int st = 0; st < n_stage_steps; st++, it++) {
            const int s = it % p.stages;
            if (!mbar_wait_bounded(&full[s], (it / p.stages) & 1, err, 2)) return;
            const uint8_t* slot = ring + (size_t)s * p.stage_bytes;
            const int nsb = min(kSbPerStage, p.nb - st * kSbPerStage);
            if (row0 < p.N) {   // warps past the end of the matrix only keep the ring moving
                for (int sb = 0; sb < nsb; sb++) {
                    const uint8_t* xa = slot + (size_t)sb * p.tok_pad * kActPitch;
                    const uint8_t* w0 = slot + p.act_bytes + (size_t)(16 * rg + g) * p.row_pitch + sb * BPDQ_Q4K_BYTES;
                    const uint8_t* w1 = w0 + 8 * p.row_pitch;
                    const uint4 h0 = *reinterpret_cast<const uint4*>(w0);
                    const uint4 h1 = *reinterpret_cast<const uint4*>(w1);
                    uint32_t sca[2], mna[2], scb[2], mnb[2];   // packed scales/mins of rows g and g+8, halves 0/1
                    q4k_scales4(h0.y, h0.z, h0.w, 0, sca[0], mna[0]);
                    q4k_scales4(h0.y, h0.z, h0.w, 1, sca[1], mna[1]);
                    q4k_scales4(h1.y, h1.z, h1.w, 0, scb[0], mnb[0]);
                    q4k_scales4(h1.y, h1.z, h1.w, 1, scb[1], mnb[1]);
                    int isum[NT][4];
#pragma unroll
                    for (int n = 0; n < NT; n++)
#pragma unroll
                        for (int i = 0; i < 4; i++) isum[n][i] = 0;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int sa = (int)byte_of(sca[j >> 2], j & 3), sb_ = (int)byte_of(scb[j >> 2], j & 3);
                        const uint32_t wa = *reinterpret_cast<const uint32_t*>(w0 + 16 + 16 * j + 4 * t);
                        const uint32_t wb = *reinterpret_cast<const uint32_t*>(w1 + 16 + 16 * j + 4 * t);
                        // fragment order: {row g k 0-15, row g+8 k 0-15, row g k 16-31, row g+8 k 16-31}
                        const uint32_t af[4] = {wa & 0x0F0F0F0Fu, wb & 0x0F0F0F0Fu, (wa >> 4) & 0x0F0F0F0Fu,
                                                (wb >> 4) & 0x0F0F0F0Fu};
#pragma unroll
                        for (int n = 0; n < NT; n++) {
                            const uint2 bf =
                                *reinterpret_cast<const uint2*>(xa + (size_t)(tok0 + 8 * n + g) * kActPitch + 32 * j + 8 * t);
                            int c[4];
                            mma_s8(c, af, bf.x, bf.y);
                            isum[n][0] += sa * c[0];
                            isum[n][1] += sa * c[1];
                            isum[n][2] += sb_ * c[2];
                            isum[n][3] += sb_ * c[3];
                        }
                    }
                    const float d0 = f16_bits_to_f32(h0.x & 0xFFFFu), m0 = f16_bits_to_f32(h0.x >> 16);
                    const float d1 = f16_bits_to_f32(h1.x & 0xFFFFu), m1 = f16_bits_to_f32(h1.x >> 16);
#pragma unroll
                    for (int n = 0; n < NT; n++) {
                        // accumulator i: row g (i<2) or g+8, token 8n + 2t + (i&1)
                        const uint8_t* r0 = xa + (size_t)(tok0 + 8 * n + 2 * t) * kActPitch;
                        const uint8_t* r1 = r0 + kActPitch;
                        const float dA0 = *reinterpret_cast<const float*>(r0 + 256);
                        const float dA1 = *reinterpret_cast<const float*>(r1 + 256);
                        const uint4 bs0 = *reinterpret_cast<const uint4*>(r0 + 272);   // eight int16 sub-block sums
                        const uint4 bs1 = *reinterpret_cast<const uint4*>(r1 + 272);
                        auto msum = [](const uint4& bs, uint32_t mlo, uint32_t mhi) {
                            int v = dp2a_lo(bs.x, mlo, 0);
                            v = dp2a_hi(bs.y, mlo, v);
                            v = dp2a_lo(bs.z, mhi, v);
                            return dp2a_hi(bs.w, mhi, v);
                        };
                        const int ms[4] = {msum(bs0, mna[0], mna[1]), msum(bs1, mna[0], mna[1]), msum(bs0, mnb[0], mnb[1]),
                                           msum(bs1, mnb[0], mnb[1])};
                        if (p.ints) {
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const int row = row0 + g + (i >> 1) * 8, tok = tok0 + 8 * n + 2 * t + (i & 1);
                                if (row < p.N && tok < p.tokens)
                                    *reinterpret_cast<int2*>(p.ints + (((size_t)tok * p.N + row) * p.nb + (st * kSbPerStage + sb)) * 2) =
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
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        // out is [tokens][N]
#pragma unroll
        for (int n = 0; n < NT; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = row0 + g + (i >> 1) * 8, tok = tok0 + 8 * n + 2 * t + (i & 1);
                if (row < p.N && tok < p.tokens) out[(size_t)tok * p.N + row] = facc[n][i];
            }
    }
}

// The weight matrix as a 2-D tensor of 4-byte elements [N][K/256*36] for the tiled copy.
static int make_weight_map(CUtensorMap* map, const uint8_t* W, int N, int nb, int box_rows, int row_pitch)
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
    const cuuint32_t box[2] = {(cuuint32_t)(row_pitch / 4), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(W), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : latch(BPDQ_ERR_CUDA - 900 - (int)r);
}

template <int NT>
static int launch_gemm(const uint8_t* W, const uint8_t* acts, float* out, const GemmPlan& p, cudaStream_t s)
{
    CUtensorMap wmap;
    int mrc = make_weight_map(&wmap, W, p.N, p.nb, p.box_rows, p.row_pitch);
    if (mrc) return mrc;
    auto kern = k_gemm_q4k_q8k_mma<NT>;
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
    cfg.blockDim = dim3((p.warps + 1) * 32);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, wmap, acts, out, p, device_error_flag()));
}

// out[tokens][N] for up to 64 tokens per pass.  C-ABI nibble order only.
int gemm_q4k_q8k_mma(const uint8_t* W, const float* X, float* out, int tokens, int N, int K, cudaStream_t s, Workspace* ws,
                     int32_t* sb_ints)
{
    if (tokens < 0 || N < 0 || K <= 0 || (K % 256) != 0) return latch(BPDQ_ERR_ARG);
    if (tokens == 0 || N == 0) return 0;
    if (!W || !X || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)W & 15) || ((uintptr_t)X & 15) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    for (int t0 = 0; t0 < tokens; t0 += 64) {
        const int T = tokens - t0 < 64 ? tokens - t0 : 64;
        GemmPlan p;
        p.N = N;
        p.K = K;
        p.nb = K / 256;
        p.tokens = T;
        // tokens are split over `ts` warps per row group, NT n-tiles of 8 tokens each
        const int nt = T <= 8 ? 1 : (T <= 32 ? 2 : 4);
        p.ts = T <= 16 ? 1 : 2;
        p.tok_pad = 8 * nt * p.ts;
        // rows per CTA: 16 * groups, chosen so that the tiles fill the SMs in as few equal rounds as possible
        // (warps of a CTA run side by side, so a tile's time grows slowly with its height: model it as 4 + w)
        int best_w = 8;
        long best_cost = -1;
        for (int w = 8; w >= 1; w--) {
            const long tiles = (N + 16 * w - 1) / (16 * w);
            const long rounds = (tiles + sm_count() - 1) / sm_count();
            const long cost = rounds * (4 + w);
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_w = w; }
        }
        p.warps = best_w * p.ts;
        p.n_tiles = (N + 16 * best_w - 1) / (16 * best_w);
        p.grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
        p.act_bytes = kSbPerStage * p.tok_pad * kActPitch;
        p.act_bytes = (p.act_bytes + 127) / 128 * 128;   // the weight box must start on a 128-byte boundary
        p.row_pitch = (p.nb < kSbPerStage ? p.nb : kSbPerStage) * BPDQ_Q4K_BYTES;
        p.box_rows = 16 * best_w < N ? 16 * best_w : N;
        p.stage_bytes = (p.act_bytes + 16 * best_w * p.row_pitch + 127) / 128 * 128;
        p.stages = (227 * 1024 - 128) / p.stage_bytes;
        if (p.stages > 6) p.stages = 6;
        if (p.stages < 2) return latch(BPDQ_ERR_RANGE);
        p.smem = 128 + (size_t)p.stages * p.stage_bytes;
        p.ints = sb_ints ? sb_ints + (size_t)t0 * N * p.nb * 2 : nullptr;
        const size_t scratch_bytes = (size_t)p.nb * p.tok_pad * kActPitch;
        // every pass of 64 tokens uses the same scratch: the quantizer waits for the pass before it
        Workspace pass_ws = ws ? *ws : Workspace{nullptr, 0, 0};
        int src = 0;
        uint8_t* acts = scratch_take(ws ? &pass_ws : nullptr, kScratchGemmActs, scratch_bytes, s, &src);
        if (!acts) return src;
        const long units = (long)p.nb * p.tok_pad;
        long want = (units + 7) / 8, cap = (long)sm_count() * 8;
        int rc;
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
            rc = check_cuda(cudaLaunchKernelEx(&cfg, k_quant_gemm_acts, (const float*)(X + (size_t)t0 * K), acts, T, p.tok_pad, K));
            if (rc) return rc;
        }
        float* o = out + (size_t)t0 * N;
        rc = nt == 1 ? launch_gemm<1>(W, acts, o, p, s) : (nt == 2 ? launch_gemm<2>(W, acts, o, p, s) : launch_gemm<4>(W, acts, o, p, s));
        if (rc) return latch(rc);
    }
    return 0;
}

// scratch bytes of gemm_q4k_q8k_mma for these sizes (an upper bound over its token passes)
size_t gemm_q4k_q8k_mma_workspace(int tokens, int K)
{
    const int T = tokens < 64 ? tokens : 64;
    const int nt = T <= 8 ? 1 : (T <= 32 ? 2 : 4), ts = T <= 16 ? 1 : 2;
    return (size_t)(K / 256) * (8 * nt * ts) * kActPitch + 256;
}

}  // namespace bpdq

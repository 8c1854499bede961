// Batched Q4_K x Q8_K product for 8 < tokens: int8 tensor-core MMA on raw nibbles.
//
// out[t][n] = sum_b [ (d_nb * dA_tb) * isum - (dmin_nb * dA_tb) * msum ],
//   isum = sum_j sc_j * sum_{k in sub-block j} q_k * x_k,   msum = sum_j mn_j * sum_{k in j} x_k
// (the definition of gemv_q4k.cu, exact integers inside a super-block).  The integer sums run
// on the tensor cores without ever leaving the integer domain:
//   * a 6-bit scale is split sc = 8*sh + sl; the byte-wise products q*sl and q*sh are < 128, so
//     (w & 0x0F0F0F0F) * sl is four int8 operands from ONE 32-bit multiply;
//   * isum = 8 * acc_hi + acc_lo with two int32 accumulators that run over the eight
//     sub-blocks of a super-block; msum comes from a third accumulator whose A operand is mn_j
//     replicated over the sub-block;
//   * the fp32 scales are applied once per super-block.
// MMA shape: mma.sync.m16n8k32 s8 x s8 -> s32.  A warp owns 16 weight rows (A fragments are built
// in registers straight from the packed nibbles: thread (g,t) needs word t of the 16-byte
// sub-block of rows g and g+8), and all tokens (NT n-tiles of 8).
//
// Data movement: activations are quantized once by k_quant_gemm_acts into global scratch laid
// out [K/256][tokens_padded][272 B] (256 int8, fp32 scale, pad: the 272-byte pitch makes the
// B-fragment reads conflict-free); a CTA of W warps (16*W rows) walks K in stages of two
// super-blocks: the producer warp bulk-copies each row's 288-byte piece (pitch 304 B in shared
// memory, conflict-free A reads) and the stage's activation chunk into a ring with full/empty
// mbarriers.  Accumulation order: super-blocks in ascending order, one fp32 accumulator per
// output, acc += dA * (d * float(isum) - dmin * float(msum)).
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

constexpr int kActPitch = 272;     // bytes per (super-block, token) in scratch and in shared memory
constexpr int kRowPitch = 304;     // shared-memory pitch of a row's two-super-block piece (288 B + 16)
constexpr int kSbPerStage = 2;

struct GemmPlan {
    int N, K, nb, tokens, tok_pad;   // weight rows, K, super-blocks per row, valid tokens, padded tokens (8*NT)
    int warps;                       // consumer warps per CTA (16 rows each)
    int stages, n_tiles, grid;
    int stage_bytes, act_bytes;      // bytes per ring slot, of which activations
    size_t smem;
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Activation quantizer for the GEMM path: one warp per (token, super-block); writes the
// 272-byte record at [b][t] (tokens >= `tokens` up to tok_pad are written as zeros).
__global__ void __launch_bounds__(256) k_quant_gemm_acts(const float* __restrict__ X, uint8_t* __restrict__ scratch,
                                                         int tokens, int tok_pad, int K)
{
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
            if (lane < 4) rec[64 + lane] = 0;
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
        rec[lane] = q(v0.x) | (q(v0.y) << 8) | (q(v0.z) << 16) | (q(v0.w) << 24);
        rec[32 + lane] = q(v1.x) | (q(v1.y) << 8) | (q(v1.z) << 16) | (q(v1.w) << 24);
        if (lane == 0) rec[64] = __float_as_uint(d);
        if (lane > 0 && lane < 4) rec[64 + lane] = 0;
    }
}

template <int NT>
__global__ void __launch_bounds__(288, 1)
k_gemm_q4k_q8k_mma(const uint8_t* __restrict__ W, const uint8_t* __restrict__ acts, float* __restrict__ out,
                   const GemmPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + p.stages;
    uint8_t* ring = smem + 128;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool is_producer = warp == p.warps;
    const int rows_per_cta = 16 * p.warps;
    const int row_bytes = p.nb * BPDQ_Q4K_BYTES;
    const int n_stage_steps = (p.nb + kSbPerStage - 1) / kSbPerStage;   // stages per row tile

    if (tid == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 32);          // every producer lane arrives (with its own byte count)
            mbar_init(&empty[s], p.warps);
        }
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();   // activations in scratch come from the quantizer launched just before

    if (is_producer) {
        int it = 0;
        for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
            const int row0 = tile * rows_per_cta;
            const int rows = min(rows_per_cta, p.N - row0);
            for (int st = 0; st < n_stage_steps; st++, it++) {
                const int s = it % p.stages;
                if (it >= p.stages) {
                    if (!mbar_wait_bounded(&empty[s], ((it / p.stages) - 1) & 1, err, 1)) return;
                }
                const int sb0 = st * kSbPerStage;
                const int nsb = min(kSbPerStage, p.nb - sb0);
                uint8_t* slot = ring + (size_t)s * p.stage_bytes;
                uint32_t my_bytes = 0;
                // lane 0 also brings this stage's activations: [nsb][tok_pad][272] is contiguous
                if (lane == 0) my_bytes += (uint32_t)nsb * p.tok_pad * kActPitch;
                for (int r = lane; r < rows; r += 32) my_bytes += (uint32_t)nsb * BPDQ_Q4K_BYTES;
                mbar_expect_tx(&full[s], my_bytes);
                if (lane == 0)
                    bulk_g2s(slot, acts + (size_t)sb0 * p.tok_pad * kActPitch, (uint32_t)nsb * p.tok_pad * kActPitch,
                             &full[s]);
                for (int r = lane; r < rows; r += 32)
                    bulk_g2s(slot + p.act_bytes + (size_t)r * kRowPitch,
                             W + (size_t)(row0 + r) * row_bytes + (size_t)sb0 * BPDQ_Q4K_BYTES,
                             (uint32_t)nsb * BPDQ_Q4K_BYTES, &full[s]);
            }
        }
        return;
    }

    int it = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
        const int row0 = tile * rows_per_cta + 16 * warp;
        float facc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) facc[n][i] = 0.0f;

        for (int st = 0; st < n_stage_steps; st++, it++) {
            const int s = it % p.stages;
            if (!mbar_wait_bounded(&full[s], (it / p.stages) & 1, err, 2)) return;
            const uint8_t* slot = ring + (size_t)s * p.stage_bytes;
            const int sb0 = st * kSbPerStage;
            const int nsb = min(kSbPerStage, p.nb - sb0);
            if (row0 < p.N) {   // warps past the end of the matrix only keep the ring moving
                for (int sb = 0; sb < nsb; sb++) {
                    const uint8_t* xa = slot + (size_t)sb * p.tok_pad * kActPitch;
                    const uint8_t* w0 = slot + p.act_bytes + (size_t)(16 * warp + g) * kRowPitch + sb * BPDQ_Q4K_BYTES;
                    const uint8_t* w1 = w0 + 8 * kRowPitch;
                    const uint4 h0 = *reinterpret_cast<const uint4*>(w0);
                    const uint4 h1 = *reinterpret_cast<const uint4*>(w1);
                    int lo[NT][4], hi[NT][4], mm[NT][4];
#pragma unroll
                    for (int n = 0; n < NT; n++)
#pragma unroll
                        for (int i = 0; i < 4; i++) lo[n][i] = hi[n][i] = mm[n][i] = 0;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        uint32_t sc4a, mn4a, sc4b, mn4b;
                        q4k_scales4(h0.y, h0.z, h0.w, j >> 2, sc4a, mn4a);
                        q4k_scales4(h1.y, h1.z, h1.w, j >> 2, sc4b, mn4b);
                        const uint32_t sca = byte_of(sc4a, j & 3), scb = byte_of(sc4b, j & 3);
                        const uint32_t mna = byte_of(mn4a, j & 3) * 0x01010101u, mnb = byte_of(mn4b, j & 3) * 0x01010101u;
                        const uint32_t wa = *reinterpret_cast<const uint32_t*>(w0 + 16 + 16 * j + 4 * t);
                        const uint32_t wb = *reinterpret_cast<const uint32_t*>(w1 + 16 + 16 * j + 4 * t);
                        const uint32_t qa_lo = wa & 0x0F0F0F0Fu, qa_hi = (wa >> 4) & 0x0F0F0F0Fu;
                        const uint32_t qb_lo = wb & 0x0F0F0F0Fu, qb_hi = (wb >> 4) & 0x0F0F0F0Fu;
                        // fragment order: {row g k 0-15, row g+8 k 0-15, row g k 16-31, row g+8 k 16-31}
                        const uint32_t a_lo[4] = {qa_lo * (sca & 7u), qb_lo * (scb & 7u), qa_hi * (sca & 7u), qb_hi * (scb & 7u)};
                        const uint32_t a_hi[4] = {qa_lo * (sca >> 3), qb_lo * (scb >> 3), qa_hi * (sca >> 3), qb_hi * (scb >> 3)};
                        const uint32_t a_mn[4] = {mna, mnb, mna, mnb};
#pragma unroll
                        for (int n = 0; n < NT; n++) {
                            const uint32_t* xr = reinterpret_cast<const uint32_t*>(xa + (size_t)(8 * n + g) * kActPitch);
                            const uint32_t b0 = xr[8 * j + t], b1 = xr[8 * j + 4 + t];
                            mma_s8(lo[n], a_lo, b0, b1);
                            mma_s8(hi[n], a_hi, b0, b1);
                            mma_s8(mm[n], a_mn, b0, b1);
                        }
                    }
                    const float d0 = f16_bits_to_f32(h0.x & 0xFFFFu), m0 = f16_bits_to_f32(h0.x >> 16);
                    const float d1 = f16_bits_to_f32(h1.x & 0xFFFFu), m1 = f16_bits_to_f32(h1.x >> 16);
#pragma unroll
                    for (int n = 0; n < NT; n++) {
                        // accumulator i: row g (i<2) or g+8, token 8n + 2t + (i&1)
                        const float dA0 = *reinterpret_cast<const float*>(xa + (size_t)(8 * n + 2 * t) * kActPitch + 256);
                        const float dA1 = *reinterpret_cast<const float*>(xa + (size_t)(8 * n + 2 * t + 1) * kActPitch + 256);
                        const float v0 = d0 * (float)(8 * hi[n][0] + lo[n][0]) - m0 * (float)mm[n][0];
                        const float v1 = d0 * (float)(8 * hi[n][1] + lo[n][1]) - m0 * (float)mm[n][1];
                        const float v2 = d1 * (float)(8 * hi[n][2] + lo[n][2]) - m1 * (float)mm[n][2];
                        const float v3 = d1 * (float)(8 * hi[n][3] + lo[n][3]) - m1 * (float)mm[n][3];
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
                const int row = row0 + g + (i >> 1) * 8, tok = 8 * n + 2 * t + (i & 1);
                if (row < p.N && tok < p.tokens) out[(size_t)tok * p.N + row] = facc[n][i];
            }
    }
}

// Scratch for the quantized activations of the GEMM path: grown on demand, kept per device.
static uint8_t* gemm_scratch(size_t bytes)
{
    static uint8_t* buf[64] = {nullptr};
    static size_t cap[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cap[dev] < bytes) {
        if (buf[dev]) {
            cudaDeviceSynchronize();
            cudaFree(buf[dev]);
            buf[dev] = nullptr;
            cap[dev] = 0;
        }
        size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
        void* p = nullptr;
        if (check_cuda(cudaMalloc(&p, want)) != 0) return nullptr;
        buf[dev] = (uint8_t*)p;
        cap[dev] = want;
    }
    return buf[dev];
}

template <int NT>
static int launch_gemm(const uint8_t* W, const uint8_t* acts, float* out, const GemmPlan& p, cudaStream_t s)
{
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
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, W, acts, out, p, device_error_flag()));
}

// out[tokens][N] for up to 64 tokens per pass.  C-ABI nibble order only.
int gemm_q4k_q8k_mma(const uint8_t* W, const float* X, float* out, int tokens, int N, int K, cudaStream_t s)
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
        const int nt = T <= 16 ? 2 : (T <= 32 ? 4 : 8);
        p.tok_pad = 8 * nt;
        // rows per CTA: 16 * warps, chosen so that the tiles fill the SMs in as few equal rounds as possible
        int best_w = 8;
        long best_cost = -1;
        for (int w = 4; w <= 8; w++) {
            const long tiles = (N + 16 * w - 1) / (16 * w);
            const long rounds = (tiles + sm_count() - 1) / sm_count();
            const long cost = rounds * w;
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_w = w; }
        }
        p.warps = best_w;
        p.n_tiles = (N + 16 * p.warps - 1) / (16 * p.warps);
        p.grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
        p.act_bytes = kSbPerStage * p.tok_pad * kActPitch;
        p.stage_bytes = (p.act_bytes + 16 * p.warps * kRowPitch + 127) / 128 * 128;
        p.stages = (227 * 1024 - 128) / p.stage_bytes;
        if (p.stages > 6) p.stages = 6;
        if (p.stages < 2) return latch(BPDQ_ERR_RANGE);
        p.smem = 128 + (size_t)p.stages * p.stage_bytes;
        const size_t scratch_bytes = (size_t)p.nb * p.tok_pad * kActPitch;
        uint8_t* acts = gemm_scratch(scratch_bytes);
        if (!acts) return latch(BPDQ_ERR_CUDA);
        const long units = (long)p.nb * p.tok_pad;
        long want = (units + 7) / 8, cap = (long)sm_count() * 8;
        k_quant_gemm_acts<<<(int)(want < cap ? want : cap), 256, 0, s>>>(X + (size_t)t0 * K, acts, T, p.tok_pad, K);
        int rc = check_cuda(cudaGetLastError());
        if (rc) return rc;
        float* o = out + (size_t)t0 * N;
        rc = nt == 2 ? launch_gemm<2>(W, acts, o, p, s) : (nt == 4 ? launch_gemm<4>(W, acts, o, p, s) : launch_gemm<8>(W, acts, o, p, s));
        if (rc) return latch(rc);
    }
    return 0;
}

}  // namespace bpdq

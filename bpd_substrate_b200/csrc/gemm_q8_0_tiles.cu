// Many-token Q8_0 x Q8_0 product on the fifth-generation tensor cores over weights re-tiled once at
// load ("Q8_0 tiles").  Same arithmetic, in the same order, as the scalar bpd_qmatmul_q8_0_cpu of the
// reference (bench/bpd_cpu.c:4263-4280, 4295-4315): every activation row is quantized to Q8_0
// (bench/bpd_cpu.c:4106-4136), then per 32-element block
//
//   sumi = sum_j w_j * a_j                      (int32, exact: one kind::i8 MMA with K = 32)
//   out  = out + (float)sumi * (wd * ad)        (fp32, blocks in order, multiply then add)
//
// so the result is the reference's bit for bit, not only within a tolerance.
//
// The re-tiled layout is a pure permutation of the Q8_0 bytes (34 bytes per row and block stay 34),
// the idea of the reference's own "Q8 padded 64B coalesced [nb,N,64]" upload
// (inference/llamatov_c_inference.py:88-100) taken to what tcgen05 wants: for a tile of 128 rows and
// one block, a unit of 4352 bytes
//   [0, 4096)     the 128 x 32 int8 quants in the MMA's canonical K-major core-matrix order:
//                 element (r, k) at (k/16)*2048 + (r/8)*128 + (r%8)*16 + k%16
//   [4096, 4352)  the 128 fp16 block scales, row r at 4096 + 2r
// and units ordered [row tile][block], so that a CTA streams its tile with plain 1-D bulk copies and the
// bytes land in shared memory exactly as the MMA's A descriptor reads them: no transform warps, no
// per-weight instructions.  Rows beyond N in the last tile are zero.
//
// Kernel: one CTA = one tile of 128 rows x one tile of T tokens (16, 32 or 64), ten or eighteen warps:
//   warp 0     producer: per ring stage one bulk copy of four weight units and one of four activation units
//   warp 1     allocates tensor memory; one lane issues one MMA per block into a ring of eight
//              accumulators (T columns each) and commits each to an mbarrier
//   warps 2-   epilogue (8 warps at 16 tokens, else 16): thread r of a TMEM lane quarter owns row r; the two
//              or four warps of a quarter split the tokens; tcgen05.ld, then the fp32 operations above per
//              (row, token, block)
// All mbarrier waits are bounded; on a timeout the role records an error code and leaves, the others
// time out in turn, and warp 1 frees the tensor memory before it returns.
#include "bpdq_common.cuh"
#include "tcgen05_device.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

constexpr int kTileRows = 128;
constexpr int kTileQuants = kTileRows * 32;              // 4096
constexpr int kTileUnit = kTileRows * BPDQ_Q80_BYTES;    // 4352

template <int T>
struct Q8tShape {
    static constexpr int kEpiWarps = T == 16 ? 8 : 16;   // two or four per TMEM lane quarter (per scheduler): the
                                                         // epilogue's dependent fp32 chains need that many to keep issuing
    static constexpr int kThreads = 32 * (2 + kEpiWarps);
    static constexpr int kCols = T / (kEpiWarps / 4);    // token columns per epilogue warp: 8, 8, 16
    static constexpr int kChunk = T == 64 ? 4 : 8;       // blocks per ring stage = per accumulator set = per barrier round
    static constexpr int kActUnit = 36 * T;              // T x 32 int8 (canonical order) + T fp32 scales
    static constexpr int kStageBytes = kChunk * (kTileUnit + kActUnit);
    static constexpr int kStages = T == 64 ? 8 : 5;      // 213, 220 and 197 KB of ring
    static constexpr int kTmemCols = 2 * kChunk * T;     // two accumulator sets: 256 or 512 columns
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 8 * (2 * kStages + 4) + 16;
};

// ------------------------------------------------------------------ re-tiling (and its inverse)

// One thread per (tile, block, row): 34 bytes in, two 16-byte stores and one fp16 out.
template <bool FORWARD>
__global__ void __launch_bounds__(256) k_q8_0_tiles_permute(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N,
                                                           int nb, long n_items)
{
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long)gridDim.x * blockDim.x) {
        const int r = (int)(it & (kTileRows - 1));
        const long ub = it >> 7;                          // tile * nb + block
        const long tile = ub / nb;
        const int b = (int)(ub - tile * nb);
        const long n = tile * kTileRows + r;
        const size_t unit = (size_t)ub * kTileUnit;
        const size_t q0 = unit + (size_t)(r >> 3) * 128 + (size_t)(r & 7) * 16;
        const size_t raw = ((size_t)n * nb + b) * BPDQ_Q80_BYTES;
        if (FORWARD) {
            unsigned short h[17];
#pragma unroll
            for (int i = 0; i < 17; i++) h[i] = n < N ? *reinterpret_cast<const unsigned short*>(src + raw + 2 * i) : (unsigned short)0;
            uint4 lo, hi;
            lo.x = h[1] | ((uint32_t)h[2] << 16);   lo.y = h[3] | ((uint32_t)h[4] << 16);
            lo.z = h[5] | ((uint32_t)h[6] << 16);   lo.w = h[7] | ((uint32_t)h[8] << 16);
            hi.x = h[9] | ((uint32_t)h[10] << 16);  hi.y = h[11] | ((uint32_t)h[12] << 16);
            hi.z = h[13] | ((uint32_t)h[14] << 16); hi.w = h[15] | ((uint32_t)h[16] << 16);
            *reinterpret_cast<uint4*>(dst + q0) = lo;
            *reinterpret_cast<uint4*>(dst + q0 + 2048) = hi;
            *reinterpret_cast<unsigned short*>(dst + unit + kTileQuants + 2 * r) = h[0];
        } else if (n < N) {
            const uint4 lo = *reinterpret_cast<const uint4*>(src + q0);
            const uint4 hi = *reinterpret_cast<const uint4*>(src + q0 + 2048);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            unsigned short* o = reinterpret_cast<unsigned short*>(dst + raw);
            o[0] = *reinterpret_cast<const unsigned short*>(src + unit + kTileQuants + 2 * r);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                o[1 + 2 * i] = (unsigned short)(w[i] & 0xFFFFu);
                o[2 + 2 * i] = (unsigned short)(w[i] >> 16);
            }
        }
    }
}

// ------------------------------------------------------------------ activation quantizer

// X fp32 [M][K] -> per (token tile, block) a unit of 36*T bytes: the T x 32 int8 B operand in the
// canonical K-major order (element (t, k) at (k/16)*16*T + (t/8)*128 + (t%8)*16 + k%16), then T fp32
// scales holding the value of the fp16 scale a Q8_0 block would store.  Eight lanes per block, the
// rule of k_quant_q8_0 (byte-identical to bpd_quant_q8_0_cpu).  Tokens beyond M quantize zeros.
__global__ void __launch_bounds__(256) k_quant_q8_0_tiles(const float* __restrict__ X, uint8_t* __restrict__ acts, int M, int K,
                                                          int T, long n_items)
{
    // Programmatic launch on both sides: the product may start loading weights while this kernel runs;
    // this kernel waits for the launch ahead of it, which may produce X and may still read the scratch.
    pdl_launch_dependents();
    pdl_wait();
    const int nb = K / 32;
    for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long)gridDim.x * blockDim.x) {
        const int l = (int)(it & 7);
        const long bt = it >> 3;                          // (tile * nb + block) * T + t
        const int t = (int)(bt % T);
        const long ub = bt / T;
        const long tile = ub / nb;
        const int b = (int)(ub - tile * nb);
        const long tok = tile * T + t;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tok < M) v = __ldg(reinterpret_cast<const float4*>(X + (size_t)tok * K + (size_t)b * 32) + l);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        const float mul = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        auto qz = [mul](float f) -> uint32_t { return (uint32_t)__float2int_rn(__fmul_rn(f, mul)) & 0xFFu; };
        uint8_t* unit = acts + (size_t)ub * 36 * T;
        *reinterpret_cast<uint32_t*>(unit + (l >> 2) * 16 * T + (t >> 3) * 128 + (t & 7) * 16 + 4 * (l & 3)) =
            qz(v.x) | (qz(v.y) << 8) | (qz(v.z) << 16) | (qz(v.w) << 24);
        if (l == 0) reinterpret_cast<float*>(unit + 32 * T)[t] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
    }
}

// ------------------------------------------------------------------ the product

template <int T>
__global__ void __launch_bounds__(Q8tShape<T>::kThreads, 1)
k_gemm_q8_0_tiles(const uint8_t* __restrict__ tiles, const uint8_t* __restrict__ acts, float* __restrict__ out, int M, int N,
                  int nb, int* err)
{
    using S = Q8tShape<T>;
    constexpr int kStages = S::kStages, G = S::kChunk;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * S::kStageBytes);   // [kStages] bulk copies landed
    uint64_t* empty = full + kStages;                 // [kStages] all epilogue warps are done with the stage
    uint64_t* acc_full = empty + kStages;             // [2] MMA commit: the accumulators of a chunk are complete
    uint64_t* acc_empty = acc_full + 2;               // [2] all epilogue warps have read them
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kStages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], S::kEpiWarps); }
        for (int s = 0; s < 2; s++) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], S::kEpiWarps); }
        mbar_init_fence();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(S::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    const int n_chunks = (nb + G - 1) / G;
    auto blocks_in = [nb](int c) { const int g = nb - c * G; return g < G ? g : G; };
    constexpr int kActOff = G * kTileUnit;            // activation units follow the weight units of a stage

    if (warp == 0) {
        // ---------------- producer.  The weights of the first ring round are requested before the
        // activation quantizer launched ahead of this kernel has finished; only its output waits for it.
        if (lane == 0) {
            const uint8_t* wsrc = tiles + (size_t)blockIdx.x * nb * kTileUnit;
            const uint8_t* asrc = acts + (size_t)blockIdx.y * nb * S::kActUnit;
            const int ahead = n_chunks < kStages ? n_chunks : kStages;
            for (int i = 0; i < ahead; i++) {
                const uint32_t g = (uint32_t)blocks_in(i);
                mbar_expect_tx(&full[i], g * (uint32_t)(kTileUnit + S::kActUnit));
                bulk_g2s(ring + (size_t)i * S::kStageBytes, wsrc + (size_t)i * G * kTileUnit, g * kTileUnit, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < ahead; i++)
                bulk_g2s(ring + (size_t)i * S::kStageBytes + kActOff, asrc + (size_t)i * G * S::kActUnit,
                         (uint32_t)blocks_in(i) * S::kActUnit, &full[i]);
            int s = 0;
            uint32_t par = 0;      // parity of the epilogue's release one ring round back
            for (int i = kStages; i < n_chunks; i++) {
                if (!mbar_wait_sleepy(&empty[s], par, err, 31)) break;   // the ring has slack: poll gently
                const uint32_t g = (uint32_t)blocks_in(i);
                uint8_t* stage = ring + (size_t)s * S::kStageBytes;
                mbar_expect_tx(&full[s], g * (uint32_t)(kTileUnit + S::kActUnit));
                bulk_g2s(stage, wsrc + (size_t)i * G * kTileUnit, g * kTileUnit, &full[s]);
                bulk_g2s(stage + kActOff, asrc + (size_t)i * G * S::kActUnit, g * S::kActUnit, &full[s]);
                if (++s == kStages) { s = 0; par ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer.  The whole warp walks the loop so that descriptors and ring
        // counters stay warp-uniform; one elected lane issues a chunk's MMAs and one commit.
        const uint32_t idesc = umma_i8_idesc(kTileRows, T);
        int s = 0;
        uint32_t full_par = 0;
        for (int c = 0; c < n_chunks; c++) {
            const int a = c & 1;
            if (!mbar_wait_bounded(&full[s], full_par, err, 32)) break;
            if (c >= 2 && !mbar_wait_bounded(&acc_empty[a], (uint32_t)((c >> 1) - 1) & 1u, err, 33)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // Few instructions per MMA: this warp shares its scheduler with four busy epilogue warps and gets
            // about one issue slot in five.  Descriptors differ between blocks only in their address field
            // (low word, no carry: shared memory addresses / 16 stay below 2^14).
            const uint32_t stage = smem_addr(ring + (size_t)s * S::kStageBytes);
            const uint64_t a0 = umma_desc(stage, 2048, 128), b0 = umma_desc(stage + kActOff, 16 * T, 128);
            const uint32_t a_lo = (uint32_t)a0, a_hi = (uint32_t)(a0 >> 32), b_lo = (uint32_t)b0, b_hi = (uint32_t)(b0 >> 32);
            const uint32_t d0 = tmem_base + (uint32_t)(a * G * T);
            const int g_n = blocks_in(c);
            if (elect_one()) {
                if (g_n == G) {
#pragma unroll
                    for (int g = 0; g < G; g++)
                        umma_i8_ss<0>(d0 + (uint32_t)(g * T), ((uint64_t)a_hi << 32) | (a_lo + (uint32_t)(g * (kTileUnit >> 4))),
                                      ((uint64_t)b_hi << 32) | (b_lo + (uint32_t)(g * (S::kActUnit >> 4))), idesc);
                } else {
                    for (int g = 0; g < g_n; g++)
                        umma_i8_ss<0>(d0 + (uint32_t)(g * T), ((uint64_t)a_hi << 32) | (a_lo + (uint32_t)(g * (kTileUnit >> 4))),
                                      ((uint64_t)b_hi << 32) | (b_lo + (uint32_t)(g * (S::kActUnit >> 4))), idesc);
                }
                umma_commit(&acc_full[a]);
            }
            __syncwarp();
            if (++s == kStages) { s = 0; full_par ^= 1u; }
        }
    } else {
        // ---------------- epilogue
        constexpr int kCols = S::kCols;
        const int e = warp - 2;
        const int quarter = warp & 3;                     // the TMEM lanes this warp may read: 32*(warp%4)..
        const int c0 = (e >> 2) * kCols;                  // first token column of this warp
        const int r = 32 * quarter + lane;
        const uint32_t taddr0 = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c0;
        float acc[kCols];
#pragma unroll
        for (int t = 0; t < kCols; t++) acc[t] = 0.0f;
        int s = 0;
        uint32_t full_par = 0;
        bool gave_up = false;
        pdl_wait();
        for (int c = 0; c < n_chunks; c++) {
            const int a = c & 1;
            if (!mbar_wait_bounded(&full[s], full_par, err, 34)) { gave_up = true; break; }
            if (!mbar_wait_bounded(&acc_full[a], (uint32_t)(c >> 1) & 1u, err, 35)) { gave_up = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint8_t* stage = ring + (size_t)s * S::kStageBytes;
            const int g_n = blocks_in(c);
            int v[G][kCols];
#pragma unroll
            for (int g = 0; g < G; g++) {
                const uint32_t ta = taddr0 + (uint32_t)((a * G + g) * T);
                if constexpr (kCols >= 16) {
#pragma unroll
                    for (int j = 0; j < kCols / 16; j++) tmem_ld(ta + 16 * j, *reinterpret_cast<int(*)[16]>(&v[g][16 * j]));
                } else {
                    tmem_ld(ta, *reinterpret_cast<int(*)[8]>(&v[g][0]));
                }
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[a]);
            // one block: the reference's three roundings as scalar instructions (the packed f32x2 forms run on
            // half of the fp32 lanes only, and the assembler merges mul.rn.f32x2 + add.rn.f32x2 into one fma,
            // which rounds once where the reference rounds twice).  (float)sumi without the slow conversion
            // instruction: an integer add on the bits gives 1.5*2^23 + sumi exactly (|sumi| < 2^22), and taking
            // 1.5*2^23 off again is exact too.
            auto block = [&](int g) {
                const float wd = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(stage + g * kTileUnit + kTileQuants + 2 * r));
                const float* ad = reinterpret_cast<const float*>(stage + kActOff + g * S::kActUnit + 32 * T) + c0;
#pragma unroll
                for (int t4 = 0; t4 < kCols / 4; t4++) {
                    const float4 a4 = *reinterpret_cast<const float4*>(ad + 4 * t4);
                    const float a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float f = __fadd_rn(__int_as_float(v[g][4 * t4 + j] + 0x4B400000), -12582912.0f);
                        acc[4 * t4 + j] = __fadd_rn(acc[4 * t4 + j], __fmul_rn(f, __fmul_rn(wd, a[j])));
                    }
                }
            };
            if (g_n == G) {
                // whole chunk: no conditions between the blocks, so that the scale loads of all of them can be
                // issued ahead of the arithmetic
#pragma unroll
                for (int g = 0; g < G; g++) block(g);
            } else {
#pragma unroll
                for (int g = 0; g < G; g++)
                    if (g < g_n) block(g);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == kStages) { s = 0; full_par ^= 1u; }
        }
        const long n = (long)blockIdx.x * kTileRows + r;
        if (!gave_up && n < N) {
#pragma unroll
            for (int t = 0; t < kCols; t++) {
                const long tok = (long)blockIdx.y * T + c0 + t;
                if (tok < M) out[(size_t)tok * N + n] = acc[t];
            }
        }
    }
    // ---------------- teardown: everybody meets, then the allocating warp frees tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------ host side

static size_t tiles_bytes(int N, int K)
{
    return (size_t)((N + kTileRows - 1) / kTileRows) * (size_t)(K / 32) * kTileUnit;
}

static int permute_tiles(bool forward, const uint8_t* src, uint8_t* dst, int N, int K, cudaStream_t s)
{
    if (N < 0 || K <= 0 || (K % 32) != 0) return latch(BPDQ_ERR_ARG);
    if (N == 0) return 0;
    if (!src || !dst) return latch(BPDQ_ERR_ARG);
    const uint8_t* tiles = forward ? dst : src;
    const uint8_t* raw = forward ? src : dst;
    if (((uintptr_t)tiles & 15) || ((uintptr_t)raw & 1)) return latch(BPDQ_ERR_ALIGN);
    const int nb = K / 32;
    const long n_items = (long)((N + kTileRows - 1) / kTileRows) * nb * kTileRows;
    const long want = (n_items + 255) / 256, cap = (long)sm_count() * 16;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    if (forward) k_q8_0_tiles_permute<true><<<grid, 256, 0, s>>>(src, dst, N, nb, n_items);
    else k_q8_0_tiles_permute<false><<<grid, 256, 0, s>>>(src, dst, N, nb, n_items);
    return check_cuda(cudaGetLastError());
}

template <int T>
static int launch_q8t(const uint8_t* tiles, const uint8_t* acts, float* out, int M, int N, int nb, cudaStream_t s)
{
    using S = Q8tShape<T>;
    auto kern = k_gemm_q8_0_tiles<T>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::kSmem));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((N + kTileRows - 1) / kTileRows), (unsigned)((M + T - 1) / T));
    cfg.blockDim = dim3(S::kThreads);
    cfg.dynamicSmemBytes = S::kSmem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, tiles, acts, out, M, N, nb, device_error_flag()));
}

// out[m*N + n] = W row n . q8_0(X row m), W in the re-tiled layout.
int gemm_q8_0_tiles(const uint8_t* tiles, const float* X, float* out, int M, int N, int K, cudaStream_t s, Workspace* ws)
{
    if (M < 0 || N < 0 || K <= 0 || (K % 32) != 0) return latch(BPDQ_ERR_ARG);
    if (M == 0 || N == 0) return 0;
    if (!tiles || !X || !out) return latch(BPDQ_ERR_ARG);
    if (((uintptr_t)tiles & 15) || ((uintptr_t)X & 15) || ((uintptr_t)out & 3)) return latch(BPDQ_ERR_ALIGN);
    const int nb = K / 32;
    // Token tile: 16, 32 or 64, whichever needs the least time by a model of waves of CTAs over the SMs
    // times the measured cost of one block at that width (1 : 1.5 : 2.95); a narrower tile re-reads the
    // weights once more per tile, from L2, and spreads the epilogue's work over more SMs.
    int T = 16;
    {
        const long row_tiles = (N + kTileRows - 1) / kTileRows;
        const int widths[3] = {16, 32, 64};
        const double rel[3] = {1.0, 1.5, 2.95};
        double best = -1.0;
        for (int i = 0; i < 3; i++) {
            if (i > 0 && M <= widths[i - 1]) break;
            const long ctas = row_tiles * ((M + widths[i] - 1) / widths[i]);
            const double cost = (double)((ctas + sm_count() - 1) / sm_count()) * rel[i];
            if (best < 0.0 || cost <= best) { best = cost; T = widths[i]; }
        }
    }
    const long token_tiles = (M + T - 1) / T;
    if (token_tiles > 65535) return latch(BPDQ_ERR_RANGE);
    int src = 0;
    uint8_t* acts = scratch_take(ws, kScratchTilesActs, (size_t)token_tiles * nb * 36 * T, s, &src);
    if (!acts) return src;
    {
        const long n_items = token_tiles * nb * T * 8;
        const long want = (n_items + 255) / 256, cap = (long)sm_count() * 8;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(want < cap ? want : cap));
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = tuning().pdl ? 1 : 0;
        int rc = check_cuda(cudaLaunchKernelEx(&cfg, k_quant_q8_0_tiles, X, acts, M, K, T, n_items));
        if (rc) return latch(rc);
    }
    int rc = T == 16 ? launch_q8t<16>(tiles, acts, out, M, N, nb, s)
                     : (T == 32 ? launch_q8t<32>(tiles, acts, out, M, N, nb, s) : launch_q8t<64>(tiles, acts, out, M, N, nb, s));
    return rc ? latch(rc) : 0;
}

// scratch bytes of gemm_q8_0_tiles: 36 bytes per 32 activations, tokens padded to the widest token tile
size_t gemm_q8_0_tiles_workspace(int M, int N, int K)
{
    (void)N;
    return (size_t)((M + 63) / 64) * (size_t)(K / 32) * 36 * 64 + 256;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {
// Bytes of the re-tiled form of an N x K Q8_0 matrix (rows padded to whole tiles of 128).
size_t bpd_q8_0_tiles_bytes(int N, int K)
{
    if (N < 0 || K <= 0 || (K % 32) != 0) return 0;
    return tiles_bytes(N, K);
}
// Q8_0 rows [N][K/32][34] -> tiles; and back, bit for bit.
int bpd_repack_q8_0_tiles_cuda(const uint8_t* raw, uint8_t* tiles, int N, int K, void* stream)
{
    return permute_tiles(true, raw, tiles, N, K, (cudaStream_t)stream);
}
int bpd_unrepack_q8_0_tiles_cuda(const uint8_t* tiles, uint8_t* raw, int N, int K, void* stream)
{
    return permute_tiles(false, tiles, raw, N, K, (cudaStream_t)stream);
}
// bpd_qmatmul_q8_0_cpu's arguments and result (bench/bpd_cpu.c:4295-4315) with W re-tiled: out[m*N + n].
int bpd_qmatmul_q8_0_tiles_cuda(const uint8_t* tiles, const float* X, float* out, int M, int N, int K, void* stream)
{
    return gemm_q8_0_tiles(tiles, X, out, M, N, K, (cudaStream_t)stream);
}
// the same with caller-owned scratch (bpdq_qmatmul_q8_0_tiles_workspace_bytes; 16-byte aligned)
size_t bpdq_qmatmul_q8_0_tiles_workspace_bytes(int M, int N, int K)
{
    return M > 0 && K > 0 ? gemm_q8_0_tiles_workspace(M, N, K) : 0;
}
int bpd_qmatmul_q8_0_tiles_ws_cuda(const uint8_t* tiles, const float* X, float* out, int M, int N, int K, void* workspace,
                                   size_t workspace_bytes, void* stream)
{
    if (!workspace || ((uintptr_t)workspace & 15)) return latch(workspace ? BPDQ_ERR_ALIGN : BPDQ_ERR_ARG);
    Workspace ws = {(uint8_t*)workspace, workspace_bytes, 0};
    return gemm_q8_0_tiles(tiles, X, out, M, N, K, (cudaStream_t)stream, &ws);
}
}

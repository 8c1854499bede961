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
#include "gemv_q4k_device.cuh"

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

// ---------------------------------------------------------------- the GEMV / small-batch GEMM kernel

// Stages the quantized activations of all T tokens in shared memory, cooperatively by the
// consumer warps of the CTA: xq is [T][2*nb] half-super-blocks of 128 int8 padded to 144 B (so
// that the 16-byte reads of 32 consecutive lanes hit distinct banks), xds is [T][nb] block
// scales.  XSRC 0: x is fp32 and is quantized here, one warp per 256-block, UNR blocks in
// flight per warp so that the loop costs about one L2 round trip; XSRC 1: x is Q8_K blocks.
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

    for (int s = tid; s < p.ng * p.slots; s += blockDim.x) {     // the barriers are set up by as many threads
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], p.kc);
        mbar_init_fence();
    }
    if (tid == 0) *abort_flag = 0;
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

// Timeline capture of the tuning builds: launch k writes its stamps at trace_base + k * trace_stride.
#ifdef BPDQ_TRACE_BUILD
static unsigned long long* g_trace_base = nullptr;
static size_t g_trace_stride = 0;
static int g_trace_left = 0;

unsigned long long* trace_take()
{
    if (!g_trace_base || g_trace_left <= 0) return nullptr;
    unsigned long long* at = g_trace_base;
    g_trace_base += g_trace_stride;
    g_trace_left--;
    return at;
}
#else
unsigned long long* trace_take() { return nullptr; }
#endif

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
        p.trace = trace_take();
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
                 int32_t* dbg, cudaStream_t s, Workspace* ws)
{
    if (M < 0) return latch(BPDQ_ERR_ARG);
    // many tokens: the weights would be streamed once per four tokens here; the tensor-core
    // kernels read them once per 64.  Measured on 14336x4096, 4096x14336, 4096x4096 and 1024x4096:
    // the tcgen05 kernel (128-row tiles, split K) is ahead from 24 tokens on matrices of 2^25
    // weights and more (from 33 when there are fewer than 8192 rows), mma.sync everywhere else.
    const bool large = (long)M * K >= (1L << 25);
    // 3 and 4 tokens on such matrices: 13.3 / 18.6 us here (the dp4a work grows with the tokens)
    // against 10.8 us for the mma.sync kernel; smaller matrices stay here (4096x4096: 9.0 against 10.2)
    if (tokens > (large ? 2 : 4) && layout == BPDQ_LAYOUT_BPD && xsrc == 0 && !dbg) {
        if (large && (tokens >= 33 || (tokens >= 24 && M >= 8192)))
            return gemm_q4k_q8k_tc5(W, reinterpret_cast<const float*>(x), out, tokens, M, K, s, ws);
        return gemm_q4k_q8k_mma(W, reinterpret_cast<const float*>(x), out, tokens, M, K, s, ws);
    }
    return gemm_q4k_q8k_multi(1, &W, &out, &M, x, tokens, K, layout, xsrc, dbg, s);
}


}  // namespace bpdq

using namespace bpdq;

extern "C" {

#ifdef BPDQ_TRACE_BUILD
// Tuning builds only: the next `launches` GEMV launches each write 8 global-timer stamps per CTA
// (ns) into dev_buf, `stride_u64` 64-bit words apart.  Pass NULL to stop.
void bpdq_debug_trace(void* dev_buf, size_t stride_u64, int launches)
{
    g_trace_base = (unsigned long long*)dev_buf;
    g_trace_stride = stride_u64;
    g_trace_left = dev_buf ? launches : 0;
}
#endif

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

int bpd_qmm_q4k_q8k_cuda(const uint8_t* qweight, const void* x, float* out, int tokens, int M, int K, int layout,
                         int xsrc, int32_t* subdots, void* stream)
{
    if ((layout != 0 && layout != 1) || (xsrc != 0 && xsrc != 1)) return latch(BPDQ_ERR_ARG);
    return gemm_q4k_q8k(qweight, x, out, tokens, M, K, layout, xsrc, subdots, (cudaStream_t)stream);
}

// The same with caller-owned scratch: nothing is allocated and no state is shared with other calls, so
// calls on different streams may overlap as long as their workspaces differ.
size_t bpdq_qmm_q4k_q8k_workspace_bytes(int tokens, int M, int K)
{
    if (tokens <= 0 || M <= 0 || K <= 0 || (K % 256) != 0) return 0;
    const size_t a = gemm_q4k_q8k_mma_workspace(tokens, K), b = M >= 128 ? gemm_q4k_q8k_tc5_workspace(tokens, M, K) : 0;
    return a > b ? a : b;
}
int bpd_qmm_q4k_q8k_ws_cuda(const uint8_t* qweight, const void* x, float* out, int tokens, int M, int K, int layout,
                            int xsrc, int32_t* subdots, void* workspace, size_t workspace_bytes, void* stream)
{
    if ((layout != 0 && layout != 1) || (xsrc != 0 && xsrc != 1) || !workspace) return latch(BPDQ_ERR_ARG);
    if ((uintptr_t)workspace & 15) return latch(BPDQ_ERR_ALIGN);
    Workspace ws = {(uint8_t*)workspace, workspace_bytes, 0};
    return gemm_q4k_q8k(qweight, x, out, tokens, M, K, layout, xsrc, subdots, (cudaStream_t)stream, &ws);
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

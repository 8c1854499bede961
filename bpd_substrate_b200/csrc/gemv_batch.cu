// ================================================================ batched independent GEMVs
//
// One launch runs up to kMaxBatch independent products out_j = W_j . q8K(x_j), each with its
// own shape (M_j, K_j); several may name the same x_j.  This is the shape of a decoder layer's
// seven projections when nothing in between is computed (the benchmark workload), and of any
// set of matrices that are known to be independent.
//
// Differences from the kernel of gemv_q4k.cu:
//  * every consumer warp owns whole tiles and whole rows: a row longer than 4096 weights is
//    walked in K-chunks of 4096 by the same warp (lane l takes half-super-block 32c + l of
//    chunk c), so no warp ever waits for another one and the mapping does not depend on K;
//  * all activation vectors of the launch are quantized once, up front, into shared memory
//    as 144-byte records per half-super-block: 128 int8, then the four sub-block sums as
//    int16 and the block scale (the padding of the layout above, put to use).  A lane fetches
//    its record (nine 16-byte reads, conflict-free) once per tile and K-chunk;
//  * accumulation order: a lane adds its half-blocks in ascending chunk order with the two
//    FMAs of half_block_fma, then the rows are folded over the lanes by fold_rows.

#include "gemv_q4k_device.cuh"

namespace bpdq {

struct QuantVectors {
    int n_vectors, total_blocks;
    BatchVector vec[kMaxBatch];
};

// Activation quantizer of the batched path: one warp per 256-block, records go to global
// scratch memory in the layout the GEMV kernel keeps in shared memory.  wait_first = 1: ordered
// like any launch (the vectors may be written, and the scratch read, by the launch ahead of it).
// wait_first = 0: the caller promises that the vectors are complete and the scratch unused, so the
// kernel reads at once and only joins the stream order (pdl_wait) before it ends.  The vectors are
// read past L1 (ld.global.cg): with programmatic launch this kernel can be resident while the
// launch that writes them is still running, which rules out the non-coherent path.
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
        const float4 v0 = __ldcg(xb + lane), v1 = __ldcg(xb + 32 + lane);
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
__global__ void __launch_bounds__(512) k_rmsnorm_records(const float* __restrict__ in, const float* __restrict__ w,
                                                          uint8_t* __restrict__ records, int cols, float eps)
{
    __shared__ float s_sum[8];
    pdl_launch_dependents();
    pdl_wait();   // the row is the previous product's output (residual stream)
    const float* x = in + (size_t)blockIdx.x * cols;
    uint8_t* rec = records + (size_t)blockIdx.x * (cols / 256) * 2 * kXqStride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (int)blockDim.x >> 5, nb = cols / 256;
    // Sixteen warps: the first eight form the sum of squares the way k_rms_norm's 256 threads do; all sixteen then scale
    // and quantize a 256-block each.  The block a warp will scale is fetched before the sum (it comes from L2, its
    // weights from HBM), so that latency runs under the sum instead of after it.
    float4 a0, a1, w0, w1;
    if (warp < nb) {
        const float4* xb = reinterpret_cast<const float4*>(x + (size_t)warp * 256);
        const float4* wb = reinterpret_cast<const float4*>(w + (size_t)warp * 256);
        a0 = __ldcg(xb + lane);
        a1 = __ldcg(xb + 32 + lane);
        w0 = __ldg(wb + lane);
        w1 = __ldg(wb + 32 + lane);
    }
    if (threadIdx.x < 256) {
        float t = 0.0f;
        // (data written by the launch before this one is read past L1: ld.global.cg).  The chain of FMAs
        // is k_rms_norm's, but sixteen loads go out before the first of them is used: one L2 round trip
        // per 4096 columns instead of sixteen.  A column past the end contributes fmaf(0, 0, t) = t.
        for (int base = 0; base < cols; base += 16 * 256) {
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int c = base + i * 256 + (int)threadIdx.x;
                v[i] = c < cols ? __ldcg(x + c) : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 16; i++) t = fmaf(v[i], v[i], t);
        }
        t = warp_sum(t);
        if (lane == 0) s_sum[warp] = t;
    }
    __syncthreads();
    float tot = s_sum[0];
#pragma unroll
    for (int i = 1; i < 8; i++) tot += s_sum[i];
    const float scale = rsqrtf(tot / (float)cols + eps);
    for (int b = warp; b < nb; b += n_warps) {
        if (b != warp) {
            const float4* xb = reinterpret_cast<const float4*>(x + (size_t)b * 256);
            const float4* wb = reinterpret_cast<const float4*>(w + (size_t)b * 256);
            a0 = __ldcg(xb + lane);
            a1 = __ldcg(xb + 32 + lane);
            w0 = __ldg(wb + lane);
            w1 = __ldg(wb + 32 + lane);
        }
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

// Every consumer warp owns `slots` ring slots and fills them itself: after it has used a slot it issues the
// bulk copy of the tile it will need `slots` turns later, so a freed slot is on its way to being full again at
// once and nobody has to notice that it became free.  (A producer warp polling the slots' "empty" barriers
// reacted too slowly for tiles of a few KB: the weight stream then ran at 85 % of what HBM delivers.)
template <int FMT, int LAYOUT, int MAXTHREADS, int ACC>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_gemv_batch_q4k_q8k(const BatchPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                 // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                     // activation records
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);    // [nw*slots]
    uint64_t* xbar = full + 2 * p.nw * p.slots;                        // activation records have landed

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    BPDQ_TRACE(0);
    // the barriers are set up by as many threads as there are barriers
    for (int b = tid; b <= p.nw * p.slots; b += blockDim.x) {
        mbar_init(b < p.nw * p.slots ? &full[b] : xbar, 1);
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();
    BPDQ_TRACE(1);

    // ---- the tiles of this warp, in order; `lv` runs `slots` tiles ahead of the tile being computed
    const int stride = p.nw * (int)gridDim.x;
    const int first = warp * (int)gridDim.x + (int)blockIdx.x;
    uint8_t* my_ring = ring + (size_t)warp * p.slots * p.slot_bytes;
    uint64_t* my_full = full + warp * p.slots;
    int lv = first;
    auto issue = [&](int slot) {
        int j = 0;
#pragma unroll
        for (int q = 1; q < kMaxBatch; q++)
            if (q < p.n_problems && lv >= p.prob[q].tile_begin) j = q;
        const BatchProblem& pb = p.prob[j];
        const int row0 = (lv - pb.tile_begin) * pb.rt;
        const uint32_t bytes = (uint32_t)min(pb.rt, pb.M - row0) * pb.row_bytes;
        if (lane == 0) {
            mbar_expect_tx(&my_full[slot], bytes);
            bulk_g2s(my_ring + (size_t)slot * p.slot_bytes, pb.W + (size_t)row0 * pb.row_bytes, bytes, &my_full[slot]);
        }
        lv += stride;
    };
    // weights never depend on the launch before this one: the first tiles are requested at once
    for (int k = 0; k < p.slots && lv < p.n_tiles; k++) issue(k);

    if (p.records) {
        // Records were written by the quantizer kernel launched just before this one: every thread waits
        // for it (and so for everything earlier in the stream; unbounded by design, it is the stream
        // order), one of them pulls the records in with one bulk copy, and the bounded wait that follows
        // covers nothing but that copy.
        pdl_wait();
        if (tid == 0) {
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
        // ---- quantize every activation vector of the launch into shared memory (all warps)
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
    bool first_tile = true;
    for (int v = first; v < p.n_tiles; v += stride) {
        if (!mbar_wait_bounded(&my_full[slot], parity, err, 2)) return;
        if (first_tile) { BPDQ_TRACE(5); first_tile = false; }
        int j = 0;
#pragma unroll
        for (int q = 1; q < kMaxBatch; q++)
            if (q < p.n_problems && v >= p.prob[q].tile_begin) j = q;
        const BatchProblem& pb = p.prob[j];
        const int row0 = (v - pb.tile_begin) * pb.rt;
        const uint8_t* tile_smem = my_ring + (size_t)slot * p.slot_bytes;
        const PeerTargets* peers = ACC == 2 ? &p.peers : nullptr;
        if (FMT == 0) {
            if (pb.rt == 4) batch_tile<4, LAYOUT, ACC>(tile_smem, xq + pb.xq_off, pb, row0, lane, peers);
            else if (pb.rt == 2) batch_tile<2, LAYOUT, ACC>(tile_smem, xq + pb.xq_off, pb, row0, lane, peers);
            else batch_tile<1, LAYOUT, ACC>(tile_smem, xq + pb.xq_off, pb, row0, lane, peers);
        } else {
            if (pb.rt == 4) batch_tile_q80<4>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else if (pb.rt == 2) batch_tile_q80<2>(tile_smem, xq + pb.xq_off, pb, row0, lane);
            else batch_tile_q80<1>(tile_smem, xq + pb.xq_off, pb, row0, lane);
        }
        // every lane has read the slot (its values went into the row sums, which were folded over the lanes
        // and stored): refill it
        __syncwarp();
        if (lv < p.n_tiles) issue(slot);
        if (++slot == p.slots) {
            slot = 0;
            parity ^= 1u;
        }
    }
    BPDQ_TRACE(6);
}

// Builds the launch plan for descs[0..n); returns BPDQ_ERR_RANGE when the set does not fit one
// launch (too many activations for shared memory, or rows longer than a ring slot).
int make_batch_plan(const BatchDesc* d, int n, BatchPlan& p, int fmt, int ctas_per_sm)
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
        // ctas_per_sm = 2: a CTA takes less than half of the SM's shared memory (1 KB per CTA is the system's), so that
        // the CTAs of the NEXT launch become resident while this launch still runs and have their first weight tiles in
        // shared memory by the time the data they depend on is complete.  Measured on the dependent decode chain: slower
        // (1.67 against 1.32 ms per token; half a ring per launch streams too slowly), so no caller asks for it.
        const size_t limit = ctas_per_sm > 1 ? (size_t)(228 * 1024 / ctas_per_sm - 1024) : (size_t)kSmemLimit;
        if (p.smem <= limit) break;
        if (p.slots > 2) p.slots--;
        else if (p.nw > (ctas_per_sm > 1 ? 2 : 4)) p.nw--;
        else if (ctas_per_sm > 1) { ctas_per_sm = 1; p.slots = tu.stages < 2 ? 2 : tu.stages; p.nw = tu.warps < 1 ? 1 : (tu.warps > 16 ? 16 : tu.warps); }
        else return BPDQ_ERR_RANGE;
    }
    long want = (p.n_tiles + p.nw - 1) / p.nw;
    if (want < 1) want = 1;
    // (still one CTA of THIS launch per SM: the other half of the SM is for the launch behind it)
    p.grid = (int)(want < sm_count() ? want : sm_count());
    // outputs inside the range registered with bpdq_set_peer_outputs: results are stored to every target too
    p.peers.n = 0;
    if (fmt == 0) {
        const char *lo = nullptr, *hi = nullptr;
        bool plain = true;
        for (int j = 0; j < n; j++) {
            const char* a = (const char*)p.prob[j].out;
            const char* b = a + (size_t)p.prob[j].M * sizeof(float);
            if (!lo || a < lo) lo = a;
            if (!hi || b > hi) hi = b;
            if (p.prob[j].accumulate) plain = false;
        }
        PeerTargets t;
        bool all_inside = plain;
        for (int j = 0; j < n && all_inside; j++)
            all_inside = peer_targets_for(p.prob[j].out, p.prob[j].out + p.prob[j].M, t);
        if (all_inside && n > 0) p.peers = t;
        (void)lo; (void)hi;
    }
    return 0;
}

template <int FMT, int LAYOUT, int ACC = 0>
static int launch_batch(const BatchPlan& p, cudaStream_t s)
{
    if (ACC == 0) {
        for (int j = 0; j < p.n_problems; j++)
            if (p.prob[j].accumulate) return launch_batch<FMT, LAYOUT, 1>(p, s);
        // results also go to the ranks' gathered buffers: its own instantiation, so that the single-GPU
        // kernel stays as it is (Q4_K in the C-ABI nibble order only)
        if constexpr (FMT == 0 && LAYOUT == BPDQ_LAYOUT_BPD) {
            if (p.peers.n > 0) return launch_batch<FMT, LAYOUT, 2>(p, s);
        }
    }
    auto kern = k_gemv_batch_q4k_q8k<FMT, LAYOUT, kMidCtaThreads, ACC>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        if (rc) return rc;
        // the SM's whole shared memory, also when one CTA asks for less than half of it (two launches side by side)
        rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(p.nw * 32);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p, device_error_flag()));
}

int launch_batch_plan(const BatchPlan& p, int fmt, int layout, cudaStream_t s)
{
    if (fmt == 1) return launch_batch<1, BPDQ_LAYOUT_BPD>(p, s);
    return layout == BPDQ_LAYOUT_GGML ? launch_batch<0, BPDQ_LAYOUT_GGML>(p, s) : launch_batch<0, BPDQ_LAYOUT_BPD>(p, s);
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
        good.trace = trace_take();
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
    for (int j = 0; j < n; j++) {     // malformed descriptors are an argument error, whatever their size
        if (descs[j].M < 0 || descs[j].K <= 0 || (descs[j].K % 256) != 0) return latch(BPDQ_ERR_ARG);
        if (descs[j].M > 0 && (!descs[j].W || !descs[j].x || !descs[j].out)) return latch(BPDQ_ERR_ARG);
    }
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
    int rc = launch_glue<512>(k_rmsnorm_records, rows, (cudaStream_t)stream, x, w, (uint8_t*)records, K, eps);
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

int bpd_qmatmul_q4k_records_cuda(int n, const bpdq_gemv_desc* descs, const void* records, unsigned accumulate_mask,
                                 void* stream)
{
    if (n < 1 || n > kMaxBatch || !descs) return latch(BPDQ_ERR_ARG);
    BatchDesc d[kMaxBatch];
    for (int j = 0; j < n; j++) d[j] = {descs[j].W, nullptr, descs[j].out, descs[j].M, descs[j].K};
    return gemv_q4k_records(d, n, (const uint8_t*)records, accumulate_mask, BPDQ_LAYOUT_BPD, (cudaStream_t)stream);
}

}  // extern "C"

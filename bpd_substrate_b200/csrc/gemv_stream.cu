// ================================================================ streams of independent GEMVs
//
// Any number of independent products out_j = W_j . q8K(x_j) as ONE persistent launch (plus one small
// launch that quantizes their activation vectors).  A decode step of the benchmark is 224 such
// products; launched layer by layer (gemv_batch.cu) every launch boundary drains the weight stream:
// an SM idles from its CTA's last tile until the next launch's first tile has crossed HBM.  Here the
// weights of all products flow through the shared-memory ring without a gap.
//
// Structure (one CTA per SM, nw consumer warps + one records warp):
//  * Tiles (1, 2 or 4 whole rows of one matrix) are numbered over the whole stream and dealt round robin
//    to the nw * gridDim.x consumer warps, so the load is balanced over the stream, not per product.
//  * Every consumer warp owns `slots` ring slots and fills them ITSELF: after it has used a slot it issues
//    the bulk copy (cp.async.bulk, completion counted on the slot's mbarrier) of the tile it will need
//    `slots` turns later.  No producer warp has to notice that a slot became free, so the refill starts
//    the moment the slot is free and slots - 1 tiles per warp are always in flight.
//  * The quantized activations (144-byte records per 128 activations, written by k_quant_stream_records)
//    are too many for shared memory, so the stream is cut into phases of consecutive products whose
//    records fit one of TWO record buffers.  The records warp bulk-copies phase p + 1 into the buffer
//    that phase p - 1 used as soon as every consumer warp has left phase p - 1 (an mbarrier counted by
//    the warps); a consumer warp waits for a phase's records once, when it enters the phase.  There is
//    no CTA-wide barrier anywhere in the stream and no CTA waits for another.
//  * The table of products (32 bytes each) sits in shared memory; a warp walks it monotonically.
//  * A row longer than a ring slot (more than 64 super-blocks: K > 16384) is a tile of its own that arrives in
//    pieces of 64 super-blocks, one ring turn each; the warp carries the row's partial sums from piece to piece.
//    A lane still owns the half-blocks l, l + 32, ... of the row in ascending order: the same sums, the same bits.
//
// Arithmetic and accumulation order are those of the batched kernel (batch_tile): same bits.
// Every wait is bounded; a warp that gives up records an error code and leaves.
#include "gemv_q4k_device.cuh"

#include <cstring>
#include <vector>

namespace bpdq {

constexpr int kStreamMaxProblems = 128;    // products per launch (their table must fit shared memory)

struct StreamProblem {          // 32 bytes
    const uint8_t* W;
    float* out;
    int M;
    int tile_begin;             // index of this product's first tile in the launch
    unsigned short nb;          // super-blocks per row
    unsigned char rt, pieces;   // rows per tile; pieces > 1: a row longer than a ring slot arrives in pieces of 64 super-blocks
    unsigned short xq_off16;    // offset of its activation records inside the phase's buffer, in 16-byte units
    unsigned short phase;
};
static_assert(sizeof(StreamProblem) == 32, "table entries are copied in 16-byte pieces");
struct StreamPhaseRec {         // 8 bytes
    unsigned rec_off;           // byte offset of the phase's records in the launch's record scratch (16-byte aligned)
    unsigned rec_bytes;
};

struct StreamPlan {
    const StreamProblem* problems;   // device arrays
    const StreamPhaseRec* phases;
    const uint8_t* records;          // record scratch of this launch
    int n_problems, n_phases, n_tiles;
    int nw, slots, slot_bytes, xq_bytes;   // xq_bytes: size of ONE record buffer
    int off_ring, off_xq, off_prob, off_phase, off_bar;
    size_t smem;
    PeerTargets peers;               // n > 0: results also go to the ranks' gathered buffers (ACC = 2)
};

struct VecEntry {               // one distinct activation vector of a stream
    const float* x;
    int nb, block_begin;        // 256-blocks of this vector, index of its first block among all
    size_t rec_off;             // byte offset of its records in the scratch
};

// Quantizer of a stream's activation vectors: one warp per 256-block.  early_read = 1: the caller promises
// that the vectors are complete (nothing in flight writes them), so they are read and quantized at once, under
// the tail of the launch ahead; the records are written only after that launch has completed, because it may
// still read the same scratch.  early_read = 0: ordered like any launch.
template <int FMT>
__global__ void __launch_bounds__(256) k_quant_stream_records(const VecEntry* __restrict__ table, int n_vec, int total_blocks,
                                                               uint8_t* __restrict__ records, int early_read)
{
    pdl_launch_dependents();
    if (!early_read) pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    constexpr int kHold = 4;     // blocks a warp reads before it has to wait
    for (int b0 = warp; b0 < total_blocks; b0 += n_warps * kHold) {
        float4 v0[kHold], v1[kHold];
        uint8_t* dst[kHold];
#pragma unroll
        for (int u = 0; u < kHold; u++) {
            const int b = b0 + u * n_warps;
            dst[u] = nullptr;
            if (b < total_blocks) {
                int lo = 0, hi = n_vec - 1;          // last entry whose block_begin <= b
                while (lo < hi) {
                    const int mid = (lo + hi + 1) >> 1;
                    if (__ldg(&table[mid].block_begin) <= b) lo = mid;
                    else hi = mid - 1;
                }
                const VecEntry e = table[lo];
                const int blk = b - e.block_begin;
                const float4* xb = reinterpret_cast<const float4*>(e.x + (size_t)blk * 256);
                v0[u] = __ldcg(xb + lane);
                v1[u] = __ldcg(xb + 32 + lane);
                dst[u] = records + e.rec_off + (FMT == 0 ? (size_t)(2 * blk) * kXqStride : (size_t)(4 * blk) * kQ80PairStride);
            }
        }
        if (early_read) pdl_wait();      // (returns at once after the first time)
#pragma unroll
        for (int u = 0; u < kHold; u++) {
            if (!dst[u]) continue;
            if (FMT == 0) write_records(v0[u], v1[u], dst[u], lane);
            else write_records_q80(v0[u], v1[u], dst[u], lane);
        }
    }
    if (early_read) pdl_wait();          // a warp without blocks still joins the stream order
}

// One piece (nsb super-blocks, in shared memory) of a long row against the records of the same K range: lane l
// adds the piece's half-blocks l, l + 32, ... to the row's running sum.
template <int LAYOUT>
__device__ __forceinline__ void row_piece(const uint8_t* piece, const uint8_t* xq, int nsb, int lane, float (&acc)[1])
{
    for (int hb = lane; hb < 2 * nsb; hb += 32) {
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
        half_block_fma<1, LAYOUT>(piece + (size_t)(hb >> 1) * BPDQ_Q4K_BYTES, hb & 1, xr, bs, xd, acc, nullptr);
    }
}
// The end of a row that arrived in pieces: batch_tile<1>'s fold over the lanes and its store (peer targets included).
template <int ACC>
__device__ __forceinline__ void store_row(float partial, const BatchProblem& pb, int row0, int lane, const PeerTargets* peers)
{
    const float v[1] = {partial};
    const float total = fold_rows<1>(v, lane);
    if constexpr (ACC == 2) {
        const float val = __shfl_sync(0xFFFFFFFFu, total, 0);
        if (lane <= peers->n)
            *reinterpret_cast<float*>(reinterpret_cast<char*>(pb.out + row0) + (lane == 0 ? 0ll : peers->shift[lane > 0 ? lane - 1 : 0])) = val;
    } else {
        if (lane == 0) pb.out[row0] = total;
    }
}

// FMT 0: Q4_K weights against Q8_K records; FMT 1: Q8_0 weights (rows of 34-byte blocks, K a multiple of 256) against
// Q8_0 pair records -- the two modes of the batched kernel.
template <int FMT, int LAYOUT, int ACC>
__global__ void __launch_bounds__(kMidCtaThreads, 1)
k_gemv_stream_q4k_q8k(const StreamPlan p, int* __restrict__ err)
{
    constexpr int kRowUnit = FMT == 0 ? BPDQ_Q4K_BYTES : 8 * BPDQ_Q80_BYTES;     // bytes of 256 weights
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                            // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                                // [2][xq_bytes]
    const StreamProblem* prob = reinterpret_cast<const StreamProblem*>(smem + p.off_prob);   // [n_problems + 1]
    const StreamPhaseRec* phase = reinterpret_cast<const StreamPhaseRec*>(smem + p.off_phase);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);               // [nw*slots] a tile has landed
    uint64_t* xfull = full + p.nw * p.slots;                                      // [2] a phase's records have landed
    uint64_t* xempty = xfull + 2;                                                 // [2] every consumer warp has left the phase

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = p.nw, grid = (int)gridDim.x;
    // the tables: plain loads (they were uploaded when the plan was made, long before this launch)
    {
        const int n16 = (p.n_problems + 1) * (int)(sizeof(StreamProblem) / 16);
        for (int w = tid; w < n16; w += blockDim.x)
            reinterpret_cast<uint4*>(smem + p.off_prob)[w] = __ldg(reinterpret_cast<const uint4*>(p.problems) + w);
        for (int w = tid; w < p.n_phases; w += blockDim.x)
            reinterpret_cast<uint2*>(smem + p.off_phase)[w] = __ldg(reinterpret_cast<const uint2*>(p.phases) + w);
    }
    // the barriers are set up by as many threads: full[nw*slots], xfull[2], xempty[2] (an arrival per consumer warp)
    for (int b = tid; b < nw * p.slots + 4; b += blockDim.x) {
        mbar_init(&full[b], b >= nw * p.slots + 2 ? nw : 1);
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == nw) {
        // ---- records warp: one lane walks the phases
        if (lane == 0) {
            pdl_wait();                 // the records come from the quantizer launched just before
            pdl_launch_dependents();    // (a launch behind this one may be scheduled from here on)
            for (int ph = 0; ph < p.n_phases; ph++) {
                const int b = ph & 1;
                // buffer b held phase ph - 2: every consumer warp must have left it
                if (ph >= 2 && !mbar_wait_bounded(&xempty[b], (uint32_t)((ph >> 1) - 1) & 1u, err, 4)) break;
                const StreamPhaseRec r = phase[ph];
                mbar_expect_tx(&xfull[b], r.rec_bytes);
                bulk_g2s(xq + (size_t)b * p.xq_bytes, p.records + r.rec_off, r.rec_bytes, &xfull[b]);
            }
        }
        return;
    }

    // ---- consumer warps
    const int W = nw * grid;                       // warps that share the stream
    const int first = warp * grid + (int)blockIdx.x;
    uint8_t* my_ring = ring + (size_t)warp * p.slots * p.slot_bytes;
    uint64_t* my_full = full + warp * p.slots;

    // the tile (and piece of it) this warp will LOAD next: runs `slots` ring turns ahead of the one it computes
    constexpr int kPieceSb = 64;                   // super-blocks per piece of a long row
    int lg = first, lj = 0, lpiece = 0;
    auto issue = [&](int slot) {
        // all lanes walk the table (uniform); lane 0 issues
        while (lg >= prob[lj + 1].tile_begin) lj++;
        const StreamProblem& q = prob[lj];
        const int row_bytes = (int)q.nb * kRowUnit;
        const int row0 = (lg - q.tile_begin) * (int)q.rt;
        uint32_t bytes = (uint32_t)min((int)q.rt, q.M - row0) * (uint32_t)row_bytes;
        size_t at = (size_t)row0 * row_bytes;
        if (q.pieces > 1) {
            const int sb0 = lpiece * kPieceSb;
            bytes = (uint32_t)min(kPieceSb, (int)q.nb - sb0) * kRowUnit;
            at += (size_t)sb0 * kRowUnit;
        }
        if (lane == 0) {
            mbar_expect_tx(&my_full[slot], bytes);
            bulk_g2s(my_ring + (size_t)slot * p.slot_bytes, q.W + at, bytes, &my_full[slot]);
        }
        if (++lpiece >= (int)q.pieces) {
            lpiece = 0;
            lg += W;
        }
    };
    for (int k = 0; k < p.slots && lg < p.n_tiles; k++) issue(k);    // weights never depend on the launch before

    int cj = 0, ph = 0, slot = 0;
    uint32_t parity = 0;
    bool have_records = false, ok = true;
    // wait once for the records of the phase this warp is in
    auto enter_phase = [&]() -> bool {
        if (!have_records) {
            // the first records come from the quantizer launched just before: join the stream order first
            // (unbounded by design), so that the bounded wait covers nothing but the records' copy
            if (ph == 0) pdl_wait();
            if (!mbar_wait_bounded(&xfull[ph & 1], (uint32_t)(ph >> 1) & 1u, err, 3)) return false;
            if (ph == 0) pdl_launch_dependents();
            have_records = true;
        }
        return true;
    };
    // leave the phase: this warp will not read its records again
    auto leave_phase = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&xempty[ph & 1]);
        ph++;
        have_records = false;
    };
    for (int g = first; g < p.n_tiles; g += W) {
        while (g >= prob[cj + 1].tile_begin) cj++;
        const StreamProblem& q = prob[cj];
        // every phase is entered and left in order, also those in which this warp has no tile: the buffers'
        // barriers count one arrival per warp and phase
        while (ph < (int)q.phase) {
            if (!(ok = enter_phase())) break;
            leave_phase();
        }
        if (!ok || !(ok = enter_phase())) break;
        BatchProblem pb;
        pb.W = q.W;
        pb.out = q.out;
        pb.M = q.M;
        pb.nb = q.nb;
        pb.row_bytes = (int)q.nb * kRowUnit;
        pb.rt = q.rt;
        pb.accumulate = 0;
        const int row0 = (g - q.tile_begin) * (int)q.rt;
        const uint8_t* rec = xq + (size_t)(ph & 1) * p.xq_bytes + (size_t)q.xq_off16 * 16;
        const PeerTargets* peers = ACC == 2 ? &p.peers : nullptr;
        if (FMT == 0 && q.pieces > 1) {
            // one long row, piece by piece: lane l adds its half-blocks l, l + 32, ... of the row in ascending order
            float acc[1] = {0.0f};
            for (int piece = 0; piece < (int)q.pieces && ok; piece++) {
                if (!(ok = mbar_wait_bounded(&my_full[slot], parity, err, 2))) break;
                const uint8_t* tile_smem = my_ring + (size_t)slot * p.slot_bytes;
                const int sb0 = piece * kPieceSb, nsb = min(kPieceSb, (int)q.nb - sb0);
                row_piece<LAYOUT>(tile_smem, rec + (size_t)(2 * sb0) * kXqStride, nsb, lane, acc);
                __syncwarp();
                if (lg < p.n_tiles) issue(slot);
                if (++slot == p.slots) {
                    slot = 0;
                    parity ^= 1u;
                }
            }
            if (!ok) break;
            store_row<ACC>(acc[0], pb, row0, lane, peers);
            continue;
        }
        if (!(ok = mbar_wait_bounded(&my_full[slot], parity, err, 2))) break;
        const uint8_t* tile_smem = my_ring + (size_t)slot * p.slot_bytes;
        if constexpr (FMT == 0) {
            if (q.rt == 4) batch_tile<4, LAYOUT, ACC>(tile_smem, rec, pb, row0, lane, peers);
            else if (q.rt == 2) batch_tile<2, LAYOUT, ACC>(tile_smem, rec, pb, row0, lane, peers);
            else batch_tile<1, LAYOUT, ACC>(tile_smem, rec, pb, row0, lane, peers);
        } else {
            (void)peers;
            if (q.rt == 4) batch_tile_q80<4>(tile_smem, rec, pb, row0, lane);
            else if (q.rt == 2) batch_tile_q80<2>(tile_smem, rec, pb, row0, lane);
            else batch_tile_q80<1>(tile_smem, rec, pb, row0, lane);
        }
        // every lane has read the slot (its values went into the row sums that were folded over the lanes and
        // stored): the slot can take the tile this warp needs `slots` turns from now
        __syncwarp();
        if (lg < p.n_tiles) issue(slot);
        if (++slot == p.slots) {
            slot = 0;
            parity ^= 1u;
        }
    }
    // pass through the phases that are left, so that the records warp and the other warps can go on
    while (ok && ph < p.n_phases) {
        if (!(ok = enter_phase())) break;
        leave_phase();
    }
}

struct StreamLaunch {
    StreamPlan plan;
    StreamProblem* d_problems;
    StreamPhaseRec* d_phases;
    VecEntry* d_table;
    int n_vec, total_blocks;
};
struct StreamHandle {
    std::vector<StreamLaunch> launches;
    uint8_t* records;
    int device, fmt;
};

static void stream_destroy(StreamHandle* h)
{
    if (!h) return;
    for (auto& L : h->launches) {
        if (L.d_problems) cudaFree(L.d_problems);
        if (L.d_phases) cudaFree(L.d_phases);
        if (L.d_table) cudaFree(L.d_table);
    }
    delete h;
}

// Plans `n` independent products as launches of at most kStreamMaxProblems consecutive products, each cut into
// record phases; lays the records out in `ws` and uploads the tables.
static StreamHandle* stream_create(int n, const BatchDesc* d, uint8_t* ws, size_t ws_bytes, int fmt)
{
    if (n < 1 || !d || !ws || ((uintptr_t)ws & 15) || (fmt != 0 && fmt != 1)) { latch(BPDQ_ERR_ARG); return nullptr; }
    const Tuning& tu = tuning();
    const int row_unit = fmt == 0 ? BPDQ_Q4K_BYTES : 8 * BPDQ_Q80_BYTES;                 // bytes of 256 weights
    const int rec_unit = fmt == 0 ? 2 * kXqStride : 4 * kQ80PairStride;                  // record bytes of 256 activations
    size_t stream_bytes = 0;
    int biggest_vec = 0;
    for (int j = 0; j < n; j++) {
        const BatchDesc& q = d[j];
        if (q.M <= 0 || q.K <= 0 || (q.K % 256) != 0 || !q.W || !q.x || !q.out) { latch(BPDQ_ERR_ARG); return nullptr; }
        if (((uintptr_t)q.W & 15) || ((uintptr_t)q.x & 15) || ((uintptr_t)q.out & 3)) { latch(BPDQ_ERR_ALIGN); return nullptr; }
        if (q.K / 256 > 255 * 64 || (fmt == 1 && q.K / 256 * row_unit > 32 * 1024)) { latch(BPDQ_ERR_RANGE); return nullptr; }
        stream_bytes += (size_t)q.M * (q.K / 256) * row_unit;
        if (q.K / 256 * rec_unit > biggest_vec) biggest_vec = q.K / 256 * rec_unit;
    }
    const int tile_budget = (stream_bytes >= (fmt == 0 ? kBigLaunchBytes : kBigLaunchBytesQ80) && tu.tile_bytes < kBigLaunchTileBytes)
                                ? kBigLaunchTileBytes : tu.tile_bytes;
    // one record buffer: 20 KB, or the largest single vector
    const int xq_cap = biggest_vec > 20 * 1024 ? (biggest_vec + 127) / 128 * 128 : 20 * 1024;
    StreamHandle* h = new StreamHandle();
    h->records = ws;
    h->fmt = fmt;
    cudaGetDevice(&h->device);
    size_t ws_used = 0;
    // as few launches as the table size allows, of equal length
    const int n_launches = (n + kStreamMaxProblems - 1) / kStreamMaxProblems;
    const int per_launch = (n + n_launches - 1) / n_launches;
    for (int i0 = 0; i0 < n; i0 += per_launch) {
        const int cnt = n - i0 < per_launch ? n - i0 : per_launch;
        std::vector<StreamProblem> prob(cnt + 1);
        std::vector<StreamPhaseRec> phases;
        std::vector<VecEntry> table;
        int n_tiles = 0, slot_bytes = 0, total_blocks = 0;
        int ph_bytes = 0;
        size_t vec_first = 0;
        size_t launch_base = ws_used;
        phases.push_back({(unsigned)0, 0u});
        bool plain = true;
        PeerTargets peers;
        peers.n = 0;
        for (int j = 0; j < cnt; j++) {
            const BatchDesc& q = d[i0 + j];
            const int nb = q.K / 256, row_bytes = nb * row_unit, rec = nb * rec_unit;
            size_t k = vec_first;
            for (; k < table.size(); k++)
                if (table[k].x == q.x && table[k].nb == nb) break;
            if (k == table.size() && ph_bytes + rec > xq_cap) {
                // new phase
                ws_used += (size_t)(ph_bytes + 127) / 128 * 128;
                phases.back().rec_bytes = (unsigned)ph_bytes;
                phases.push_back({(unsigned)(ws_used - launch_base), 0u});
                ph_bytes = 0;
                vec_first = table.size();
                k = table.size();
            }
            if (k == table.size()) {
                VecEntry e;
                e.x = q.x;
                e.nb = nb;
                e.block_begin = total_blocks;
                e.rec_off = (ws_used - launch_base) + (size_t)ph_bytes;
                table.push_back(e);
                total_blocks += nb;
                ph_bytes += rec;
            }
            StreamProblem& pb = prob[j];
            pb.W = q.W;
            pb.out = q.out;
            pb.M = q.M;
            pb.tile_begin = n_tiles;
            pb.nb = (unsigned short)nb;
            pb.rt = (unsigned char)(4 * row_bytes <= tile_budget ? 4 : (2 * row_bytes <= tile_budget ? 2 : 1));
            // Q4_K rows of more than 64 super-blocks arrive in pieces of 64 (9216 bytes), so the ring slots stay small
            pb.pieces = (unsigned char)((fmt == 0 && nb > 64) ? (nb + 63) / 64 : 1);
            pb.xq_off16 = (unsigned short)((table[k].rec_off - phases.back().rec_off) / 16);
            pb.phase = (unsigned short)(phases.size() - 1);
            n_tiles += (q.M + pb.rt - 1) / pb.rt;
            const int tile_bytes = pb.pieces > 1 ? 64 * row_unit : (int)pb.rt * row_bytes;
            if (tile_bytes > slot_bytes) slot_bytes = tile_bytes;
            PeerTargets t;
            if (plain && fmt == 0 && peer_targets_for(q.out, q.out + q.M, t)) peers = t;
            else plain = false;
        }
        phases.back().rec_bytes = (unsigned)ph_bytes;
        ws_used += (size_t)(ph_bytes + 127) / 128 * 128;
        if (ws_used > ws_bytes) { stream_destroy(h); latch(BPDQ_ERR_RANGE); return nullptr; }
        // sentinel entry: ends the walk over the table
        prob[cnt] = prob[cnt - 1];
        prob[cnt].tile_begin = 0x7FFFFFFF;
        prob[cnt].phase = (unsigned short)(phases.size() - 1);
        StreamLaunch L;
        memset(&L, 0, sizeof(L));
        StreamPlan& p = L.plan;
        p.n_problems = cnt;
        p.n_phases = (int)phases.size();
        p.n_tiles = n_tiles;
        p.slot_bytes = slot_bytes;
        p.xq_bytes = xq_cap;
        p.slots = tu.stages < 2 ? 2 : tu.stages;
        p.nw = tu.warps < 1 ? 1 : (tu.warps > 16 ? 16 : tu.warps);
        p.peers.n = 0;
        if (plain && peers.n > 0) p.peers = peers;
        for (;;) {
            size_t off = 0;
            auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
            p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
            p.off_xq = take((size_t)2 * p.xq_bytes);
            p.off_prob = take((size_t)(cnt + 1) * sizeof(StreamProblem));
            p.off_phase = take((size_t)p.n_phases * sizeof(StreamPhaseRec));
            p.off_bar = take((size_t)(p.nw * p.slots + 4) * 8);
            p.smem = off;
            if (p.smem <= (size_t)kSmemLimit) break;
            if (p.slots > 2) p.slots--;
            else if (p.nw > 2) p.nw--;
            else { stream_destroy(h); latch(BPDQ_ERR_RANGE); return nullptr; }
        }
        p.records = ws + launch_base;
        void *dp = nullptr, *dph = nullptr, *dt = nullptr;
        if (check_cuda(cudaMalloc(&dp, sizeof(StreamProblem) * prob.size())) ||
            check_cuda(cudaMalloc(&dph, sizeof(StreamPhaseRec) * phases.size())) ||
            check_cuda(cudaMalloc(&dt, sizeof(VecEntry) * table.size())) ||
            check_cuda(cudaMemcpy(dp, prob.data(), sizeof(StreamProblem) * prob.size(), cudaMemcpyHostToDevice)) ||
            check_cuda(cudaMemcpy(dph, phases.data(), sizeof(StreamPhaseRec) * phases.size(), cudaMemcpyHostToDevice)) ||
            check_cuda(cudaMemcpy(dt, table.data(), sizeof(VecEntry) * table.size(), cudaMemcpyHostToDevice))) {
            if (dp) cudaFree(dp);
            if (dph) cudaFree(dph);
            if (dt) cudaFree(dt);
            stream_destroy(h);
            latch(BPDQ_ERR_CUDA);
            return nullptr;
        }
        L.d_problems = (StreamProblem*)dp;
        L.d_phases = (StreamPhaseRec*)dph;
        L.d_table = (VecEntry*)dt;
        L.n_vec = (int)table.size();
        L.total_blocks = total_blocks;
        p.problems = L.d_problems;
        p.phases = L.d_phases;
        h->launches.push_back(L);
    }
    return h;
}

template <int FMT, int ACC>
static int launch_stream(const StreamPlan& plan, cudaStream_t s)
{
    auto kern = k_gemv_stream_q4k_q8k<FMT, BPDQ_LAYOUT_BPD, ACC>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    long want = ((long)plan.n_tiles + plan.nw - 1) / plan.nw;
    if (want < 1) want = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(want < sm_count() ? want : sm_count()));
    cfg.blockDim = dim3((unsigned)(plan.nw + 1) * 32);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, plan, device_error_flag()));
}

static int stream_run(StreamHandle* h, int early_read, cudaStream_t s)
{
    if (!h) return latch(BPDQ_ERR_ARG);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != h->device) return latch(BPDQ_ERR_ARG);
    for (auto& L : h->launches) {
        int rc = h->fmt == 0 ? launch_glue(k_quant_stream_records<0>, glue_grid(L.total_blocks), s, (const VecEntry*)L.d_table, L.n_vec,
                                           L.total_blocks, const_cast<uint8_t*>(L.plan.records), early_read)
                             : launch_glue(k_quant_stream_records<1>, glue_grid(L.total_blocks), s, (const VecEntry*)L.d_table, L.n_vec,
                                           L.total_blocks, const_cast<uint8_t*>(L.plan.records), early_read);
        if (rc) return latch(rc);
        rc = h->fmt == 1 ? launch_stream<1, 0>(L.plan, s) : (L.plan.peers.n > 0 ? launch_stream<0, 2>(L.plan, s) : launch_stream<0, 0>(L.plan, s));
        if (rc) return latch(rc);
    }
    return 0;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

void* bpdq_gemv_stream_create(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes)
{
    return stream_create(n, reinterpret_cast<const BatchDesc*>(descs), (uint8_t*)workspace, workspace_bytes, 0);
}

// The same stream for Q8_0 weights (rows of 34-byte blocks, K a multiple of 256; descs[j].W = the Q8_0 rows): the
// product of bpd_qmatmul_q8_0_cuda at one token, many matrices per launch.  Workspace: bpdq_gemv_stream_q8_0_workspace_bytes.
size_t bpdq_gemv_stream_q8_0_workspace_bytes(int n, const bpdq_gemv_desc* descs)
{
    size_t total = 0;
    for (int j = 0; j < n; j++) total += (size_t)(descs[j].K / 256) * 4 * kQ80PairStride + 128;
    return total;
}
void* bpdq_gemv_stream_create_q8_0(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes)
{
    return stream_create(n, reinterpret_cast<const BatchDesc*>(descs), (uint8_t*)workspace, workspace_bytes, 1);
}

int bpdq_gemv_stream_run(void* handle, void* stream) { return stream_run((StreamHandle*)handle, 0, (cudaStream_t)stream); }

// For callers that can promise more (as bpd_qmatmul_q4k_q8k_batch_ready_cuda): every activation vector is complete
// when the call is made.  The quantizer then reads them under the tail of the launch ahead of it.
int bpdq_gemv_stream_run_ready(void* handle, void* stream) { return stream_run((StreamHandle*)handle, 1, (cudaStream_t)stream); }

int bpdq_gemv_stream_launches(void* handle) { return handle ? 2 * (int)((StreamHandle*)handle)->launches.size() : 0; }

void bpdq_gemv_stream_destroy(void* handle) { stream_destroy((StreamHandle*)handle); }

}  // extern "C"

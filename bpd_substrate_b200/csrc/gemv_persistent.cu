// A whole program of dependent Q4_K x Q8_K products in ONE launch, built from the batched kernel's pieces
// (gemv_q4k_device.cuh): k_decode_chain walks dependent phases with a grid-wide barrier between them
// (cooperative launch).  Streams of independent products are in gemv_stream.cu.
#include "gemv_q4k_device.cuh"

#include <cstring>
#include <vector>

namespace bpdq {

// ---- Persistent decode chain: ONE cooperative launch walks a whole program of dependent phases
// (per decoder layer: rms_norm -> q,k,v | q -> o, += x | rms_norm -> gate,up | silu(gate)*up -> down, += x).
// The weights of a phase do not depend on the phase before it.  Every consumer warp owns a private ring
// that it refills itself: when it has folded a tile it issues the bulk copy of the tile it needs `slots`
// turns later, which may belong to a later phase, so the ring is full again when the warp comes back from
// the barrier between phases and HBM works through the barrier and the next phase's records step.  The
// barrier is grid-wide (one counter per phase: every CTA adds one when its rows are written and fenced,
// thread 0 of every CTA polls with an acquire load, bounded); after it the CTA rebuilds the phase's
// activation records in shared memory from the vector the previous phase produced.  A cooperative launch
// keeps all CTAs resident, which the barrier needs.
//
// A gate/up phase followed by a silu(gate)*up phase is planned as PAIRED tiles: a tile holds the same rows
// of both matrices, the warp folds them together and writes gate, up and silu(gate)*up, and the phase
// after it quantizes that one vector instead of evaluating 2 x 14336 exponentials in every CTA.  The bits
// are those of the unpaired program: a row's lanes, its fold and the activation's arithmetic are the same.
constexpr int kChainMaxProblems = 3;
constexpr int kChainThreads = 384;   // at most twelve warps, all consumers: 170 registers each
struct ChainPhase {
    int n_problems, prologue, nb, n_tiles;   // prologue as in BatchPlan: 0 records of a, 1 rms_norm(a, b, eps), 2 silu(a)*b
    const float* a;
    const float* b;
    float eps;
    int pair;                                // 1: tiles hold rt/2 rows of prob[0] and the same rows of prob[1]
    float* act;                              // paired phases: silu(out0) * out1
    BatchProblem prob[kChainMaxProblems];
};
static_assert(sizeof(ChainPhase) % 16 == 0, "phase descriptors are copied to shared memory 16 bytes at a time");
static_assert(sizeof(ChainPhase) / 16 <= 32, "one warp copies a descriptor, a lane per 16 bytes");
constexpr int kChainWindow = 8;   // descriptors of the current phase and the seven after it are held in shared memory
struct ChainPlan {
    const ChainPhase* phases;   // device array
    unsigned* arrive;           // [n_phases] grid-barrier counters, zero at launch
    int n_phases;
    int nw, slots, slot_bytes;
    int off_ring, off_xq, off_win, off_bar;
    size_t smem;
    unsigned long long* trace;  // tuning aid: SM-clock stamps of CTA 0, [phase < 64][8], or null
};
#ifdef BPDQ_TRACE_BUILD
#define CHAIN_TRACE(ph, k)                                                                     \
    do {                                                                                       \
        if (p.trace && blockIdx.x == 0 && tid == 0 && (ph) < 64) p.trace[(ph) * 8 + (k)] = clock64(); \
    } while (0)
#else
#define CHAIN_TRACE(ph, k) do { } while (0)
#endif

// A paired tile: rows [row0, row0 + H) of the gate matrix, then the same rows of the up matrix, H = R / 2.
// Lane l adds its half-blocks l, l + 32, ... of every row and the rows are folded as batch_tile<R> folds them.
template <int R, int LAYOUT>
__device__ __forceinline__ void pair_tile(const uint8_t* tile_smem, const uint8_t* xq, const BatchProblem& g,
                                          const BatchProblem& u, float* __restrict__ act, int row0, int lane)
{
    constexpr int H = R / 2;
    const int rows = min(H, g.M - row0);
    const int n_hb = 2 * g.nb;
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
            if ((r % H) < rows) half_block_fma<1, LAYOUT>(sbp + (size_t)r * g.row_bytes, hb & 1, xr, bs, xd, acc[r], nullptr);
    }
    float v[R];
#pragma unroll
    for (int r = 0; r < R; r++) v[r] = acc[r][0];
    const float total = fold_rows<R>(v, lane);
    constexpr int kLanesPerRow = 32 / R;
    // the lanes that hold a gate row fetch the up row of the same index
    const float other = __shfl_sync(0xFFFFFFFFu, total, (lane + H * kLanesPerRow) & 31);
    const int my_row = lane / kLanesPerRow;
    if ((lane % kLanesPerRow) == 0) {
        if (my_row < H) {
            if (my_row < rows) {
                g.out[row0 + my_row] = total;
                act[row0 + my_row] = (total / (1.0f + expf(-total))) * other;   // cta_swiglu_records' arithmetic
            }
        } else if (my_row - H < rows) {
            u.out[row0 + my_row - H] = total;
        }
    }
}

template <int LAYOUT, int MAXTHREADS>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_decode_chain(const ChainPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                 // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                     // activation records of the current phase
    ChainPhase* win = reinterpret_cast<ChainPhase*>(smem + p.off_win); // [kChainWindow] descriptor of phase q at q % kChainWindow
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);    // [nw*slots]
    float* s_sum = reinterpret_cast<float*>(full + p.nw * p.slots);    // nine floats of the rms_norm step
    volatile int* dead = reinterpret_cast<volatile int*>(s_sum + 12);  // a wait gave up: everybody leaves at the next barrier

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = p.nw, grid = (int)gridDim.x;
    constexpr int kDesc16 = (int)(sizeof(ChainPhase) / 16);
    // the program was uploaded when the chain was planned: plain loads
    for (int w = tid; w < min(p.n_phases, kChainWindow) * kDesc16; w += blockDim.x)
        reinterpret_cast<uint4*>(win)[w] = __ldg(reinterpret_cast<const uint4*>(p.phases) + w);
    for (int b = tid; b < nw * p.slots; b += blockDim.x) {       // the barriers are set up by as many threads
        mbar_init(&full[b], 1);
        mbar_init_fence();
    }
    if (tid == 0) *dead = 0;
    __syncthreads();
    pdl_launch_dependents();

    const int first = warp * grid + (int)blockIdx.x, stride = nw * grid;
    uint8_t* my_ring = ring + (size_t)warp * p.slots * p.slot_bytes;
    uint64_t* my_full = full + warp * p.slots;

    // the tile this warp will LOAD next: runs `slots` ring turns ahead of the one it folds, across phases
    // (lph, lv) always names a tile that exists, or lph == n_phases: the walker never looks back at a phase
    // that the warp has left, so the window may drop that phase's descriptor
    int lph = 0, lv = first, cur = 0;
    auto desc = [&](int q) -> const ChainPhase* { return q < cur + kChainWindow ? &win[q % kChainWindow] : &p.phases[q]; };
    auto skip = [&]() {
        while (lph < p.n_phases && lv >= desc(lph)->n_tiles) {
            lph++;
            lv = first;
        }
    };
    skip();
    auto issue = [&](int slot) {
        if (lph >= p.n_phases) return;
        if (lane == 0) {
            const ChainPhase& P = *desc(lph);
            uint8_t* dst = my_ring + (size_t)slot * p.slot_bytes;
            if (P.pair) {
                const BatchProblem& g = P.prob[0];
                const int half = g.rt >> 1, row0 = lv * half;
                const uint32_t bytes = (uint32_t)min(half, g.M - row0) * g.row_bytes;
                mbar_expect_tx(&my_full[slot], 2 * bytes);
                bulk_g2s(dst, g.W + (size_t)row0 * g.row_bytes, bytes, &my_full[slot]);
                bulk_g2s(dst + (size_t)half * g.row_bytes, P.prob[1].W + (size_t)row0 * g.row_bytes, bytes, &my_full[slot]);
            } else {
                int j = 0;
#pragma unroll
                for (int q = 1; q < kChainMaxProblems; q++)
                    if (q < P.n_problems && lv >= P.prob[q].tile_begin) j = q;
                const BatchProblem& pb = P.prob[j];
                const int row0 = (lv - pb.tile_begin) * pb.rt;
                const uint32_t bytes = (uint32_t)min(pb.rt, pb.M - row0) * pb.row_bytes;
                mbar_expect_tx(&my_full[slot], bytes);
                bulk_g2s(dst, pb.W + (size_t)row0 * pb.row_bytes, bytes, &my_full[slot]);
            }
        }
        lv += stride;
        skip();
    };
    for (int k = 0; k < p.slots; k++) issue(k);    // weights never depend on what ran before this launch

    pdl_wait();   // the first phase's input vector comes from whatever ran before this launch
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < p.n_phases; ph++) {
        const ChainPhase& P = win[ph % kChainWindow];
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
            // the window moves on: the slot of phase ph-1 takes phase ph-1+kChainWindow (complete before the
            // barrier that ends the records step; nobody reads descriptors in between)
            cur = ph;
            const int q = ph - 1 + kChainWindow;
            if (q < p.n_phases && warp == nw - 1 && lane < kDesc16)
                reinterpret_cast<uint4*>(&win[q % kChainWindow])[lane] = __ldg(reinterpret_cast<const uint4*>(p.phases + q) + lane);
        }
        CHAIN_TRACE(ph, 0);
        // ---- the phase's activation records
        if (P.prologue == 1) cta_rmsnorm_records(P.a, P.b, P.eps, P.nb, xq, s_sum, warp, lane, nw);
        else if (P.prologue == 2) cta_swiglu_records(P.a, P.b, P.nb, xq, warp, lane, nw);
        else cta_vector_records(P.a, P.nb, xq, warp, lane, nw);
        named_bar_sync(2, nw * 32);
        CHAIN_TRACE(ph, 1);
        // ---- this warp's tiles of the phase
        const int n_tiles = P.n_tiles, n_prob = P.n_problems, pair = P.pair;
        for (int v = first; v < n_tiles; v += stride) {
            if (!mbar_wait_bounded(&my_full[slot], parity, err, 22)) {
                *dead = 1;
                break;
            }
            if (v == first) CHAIN_TRACE(ph, 4);
            const uint8_t* tile_smem = my_ring + (size_t)slot * p.slot_bytes;
            if (pair) {
                const BatchProblem& g = P.prob[0];
                const int row0 = v * (g.rt >> 1);
                if (g.rt == 4) pair_tile<4, LAYOUT>(tile_smem, xq, g, P.prob[1], P.act, row0, lane);
                else pair_tile<2, LAYOUT>(tile_smem, xq, g, P.prob[1], P.act, row0, lane);
            } else {
                int j = 0;
#pragma unroll
                for (int q = 1; q < kChainMaxProblems; q++)
                    if (q < n_prob && v >= P.prob[q].tile_begin) j = q;
                const BatchProblem& pb = P.prob[j];
                const int row0 = (v - pb.tile_begin) * pb.rt;
                if (pb.rt == 4) batch_tile<4, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
                else if (pb.rt == 2) batch_tile<2, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
                else batch_tile<1, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            }
            // every lane has read the slot: it takes the tile this warp needs `slots` turns from now
            __syncwarp();
            if (v == first) CHAIN_TRACE(ph, 5);
            issue(slot);
            if (v == first) CHAIN_TRACE(ph, 6);
            if (++slot == p.slots) {
                slot = 0;
                parity ^= 1u;
            }
        }
        // ---- publish: rows written by this CTA are visible device-wide before its arrival counts
        // (the CTA's barrier orders every warp's stores before thread 0, whose fence is cumulative: one fence per CTA)
        CHAIN_TRACE(ph, 2);
        named_bar_sync(2, nw * 32);
        if (*dead) break;
        if (tid == 0) {
            __threadfence();
            atomicAdd(p.arrive + ph, 1u);
        }
        CHAIN_TRACE(ph, 3);
    }
}

struct ChainHandle {
    ChainPlan plan;
    ChainPhase* d_phases;
    unsigned* d_arrive;
    float* d_act;      // silu(gate)*up vectors of the paired phases, one after the other
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
        P.pair = 0;
        P.act = nullptr;
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
    // gate/up followed by silu(gate)*up: paired tiles, and the next phase reads the product's own activation vector
    size_t act_floats = 0;
    std::vector<size_t> act_at((size_t)n_phases, 0);
    for (int i = 0; i + 1 < n_phases; i++) {
        const ChainPhaseDesc& d = ph[i];
        const ChainPhaseDesc& e = ph[i + 1];
        ChainPhase& P = prog[i];
        if (d.n != 2 || d.accumulate_mask || d.prod[0].M != d.prod[1].M || P.prob[0].rt < 2 || e.prologue != 2 ||
            e.a != d.prod[0].out || e.b != d.prod[1].out || e.prod[0].K != d.prod[0].M) continue;
        P.pair = 1;
        P.n_tiles = (P.prob[0].M + P.prob[0].rt / 2 - 1) / (P.prob[0].rt / 2);
        act_at[i] = act_floats;
        act_floats += ((size_t)P.prob[0].M + 63) / 64 * 64;
    }
    ChainHandle* h = new ChainHandle();
    ChainPlan& p = h->plan;
    p.n_phases = n_phases;
    p.slot_bytes = slot_bytes;
    p.slots = tu.stages < 2 ? 2 : tu.stages;
    p.nw = tu.warps < 1 ? 1 : (tu.warps > kChainThreads / 32 ? kChainThreads / 32 : tu.warps);
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_xq = take((size_t)xq_bytes);
        p.off_win = take(sizeof(ChainPhase) * kChainWindow);
        p.off_bar = take((size_t)p.nw * p.slots * 8 + 128);
        p.smem = off;
        if (p.smem <= (size_t)kSmemLimit) break;
        if (p.slots > 2) p.slots--;
        else if (p.nw > 4) p.nw--;
        else { delete h; latch(BPDQ_ERR_RANGE); return nullptr; }
    }
    cudaGetDevice(&h->device);
    void* dp = nullptr;
    void* da = nullptr;
    void* dv = nullptr;
    bool bad = check_cuda(cudaMalloc(&dp, sizeof(ChainPhase) * (size_t)n_phases)) || check_cuda(cudaMalloc(&da, sizeof(unsigned) * (size_t)n_phases)) ||
               (act_floats && check_cuda(cudaMalloc(&dv, sizeof(float) * act_floats)));
    if (!bad) {
        for (int i = 0; i + 1 < n_phases; i++) {
            if (!prog[i].pair) continue;
            prog[i].act = (float*)dv + act_at[i];
            prog[i + 1].prologue = 0;
            prog[i + 1].a = prog[i].act;
        }
        bad = check_cuda(cudaMemcpy(dp, prog.data(), sizeof(ChainPhase) * (size_t)n_phases, cudaMemcpyHostToDevice)) != 0;
    }
    if (bad) {
        if (dp) cudaFree(dp);
        if (da) cudaFree(da);
        if (dv) cudaFree(dv);
        delete h;
        latch(BPDQ_ERR_CUDA);
        return nullptr;
    }
    h->d_phases = (ChainPhase*)dp;
    h->d_arrive = (unsigned*)da;
    h->d_act = (float*)dv;
    p.phases = h->d_phases;
    p.arrive = h->d_arrive;
    p.trace = nullptr;
    return h;
}

static int chain_run(ChainHandle* h, cudaStream_t s)
{
    if (!h) return latch(BPDQ_ERR_ARG);
    auto kern = k_decode_chain<BPDQ_LAYOUT_BPD, kChainThreads>;
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
    cfg.blockDim = dim3((unsigned)h->plan.nw * 32);
    cfg.dynamicSmemBytes = h->plan.smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    ChainPlan plan = h->plan;
    plan.trace = nullptr;
    plan.trace = trace_take();
    rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, plan, device_error_flag()));
    return rc ? latch(rc) : 0;
}

static void chain_destroy(ChainHandle* h)
{
    if (!h) return;
    cudaFree(h->d_phases);
    cudaFree(h->d_arrive);
    if (h->d_act) cudaFree(h->d_act);
    delete h;
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

void* bpdq_chain_create(int n_phases, const bpdq_chain_phase* phases)
{
    static_assert(sizeof(bpdq_chain_phase) == sizeof(ChainPhaseDesc), "phase descriptor layouts must match");
    return chain_create(n_phases, reinterpret_cast<const ChainPhaseDesc*>(phases));
}

int bpdq_chain_run(void* chain, void* stream) { return chain_run((ChainHandle*)chain, (cudaStream_t)stream); }

void bpdq_chain_destroy(void* chain) { chain_destroy((ChainHandle*)chain); }

}  // extern "C"

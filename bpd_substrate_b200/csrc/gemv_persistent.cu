// A whole program of dependent Q4_K x Q8_K products in ONE launch, built from the batched kernel's pieces
// (gemv_q4k_device.cuh): k_decode_chain walks dependent phases with a grid-wide barrier between them
// (cooperative launch).  Streams of independent products are in gemv_stream.cu.
#include "gemv_q4k_device.cuh"

#include <cstring>
#include <vector>

namespace bpdq {

// ---- Persistent decode chain: ONE cooperative launch walks a whole program of dependent phases
// (per decoder layer: rms_norm -> q,k,v | q -> o, += x | rms_norm -> gate,up | silu(gate)*up -> down, += x).
// The weights of a phase do not depend on the phase before it, so the producer warp streams the
// tiles of all phases back to back into the ring and HBM never waits for a launch boundary; only
// the consumer warps wait, at a grid-wide barrier between phases (one counter per phase: every CTA
// adds one when its rows are written and fenced, thread 0 of every CTA polls with an acquire load,
// bounded), then rebuild the phase's activation records in shared memory from the vector the
// previous phase produced.  A cooperative launch keeps all CTAs resident, which the barrier needs.
constexpr int kChainMaxProblems = 3;
struct ChainPhase {
    int n_problems, prologue, nb, n_tiles;   // prologue as in BatchPlan: 0 records of a, 1 rms_norm(a, b, eps), 2 silu(a)*b
    const float* a;
    const float* b;
    float eps;
    int pad;
    BatchProblem prob[kChainMaxProblems];
};
struct ChainPlan {
    const ChainPhase* phases;   // device array
    unsigned* arrive;           // [n_phases] grid-barrier counters, zero at launch
    int n_phases;
    int nw, slots, slot_bytes;
    int off_ring, off_xq, off_bar;
    size_t smem;
    unsigned long long* trace;  // tuning aid: SM-clock stamps of CTA 0, [phase < 64][4], or null
};
#ifdef BPDQ_TRACE_BUILD
#define CHAIN_TRACE(ph, k)                                                                     \
    do {                                                                                       \
        if (p.trace && blockIdx.x == 0 && tid == 0 && (ph) < 64) p.trace[(ph) * 4 + (k)] = clock64(); \
    } while (0)
#else
#define CHAIN_TRACE(ph, k) do { } while (0)
#endif

template <int LAYOUT, int MAXTHREADS>
__global__ void __launch_bounds__(MAXTHREADS, 1)
k_decode_chain(const ChainPlan p, int* __restrict__ err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem + p.off_ring;                                 // [nw][slots][slot_bytes]
    uint8_t* xq = smem + p.off_xq;                                     // activation records of the current phase
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.off_bar);    // [nw*slots]
    uint64_t* empty = full + p.nw * p.slots;
    float* s_sum = reinterpret_cast<float*>(empty + p.nw * p.slots);   // nine floats of the rms_norm step
    volatile int* dead = reinterpret_cast<volatile int*>(s_sum + 12);  // a wait gave up: everybody leaves at the next barrier

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = p.nw, grid = (int)gridDim.x;
    if (tid == 0) {
        for (int s = 0; s < nw * p.slots; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *dead = 0;
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == nw) {
        // ---- producer: lane g feeds consumer warp g, phase after phase without a pause
        if (lane < nw) {
            const int g = lane;
            int slot = 0;
            uint32_t wait_parity = 0;
            bool wrapped = false;
            for (int ph = 0; ph < p.n_phases; ph++) {
                const ChainPhase& P = p.phases[ph];
                const int n_tiles = P.n_tiles, n_prob = P.n_problems;
                for (int v = g * grid + (int)blockIdx.x; v < n_tiles; v += nw * grid) {
                    const int s = g * p.slots + slot;
                    if (wrapped && !mbar_wait_bounded(&empty[s], wait_parity, err, 23)) return;
                    int j = 0;
#pragma unroll
                    for (int q = 1; q < kChainMaxProblems; q++)
                        if (q < n_prob && v >= P.prob[q].tile_begin) j = q;
                    const BatchProblem& pb = P.prob[j];
                    const int row0 = (v - pb.tile_begin) * pb.rt;
                    const uint32_t bytes = (uint32_t)min(pb.rt, pb.M - row0) * pb.row_bytes;
                    mbar_expect_tx(&full[s], bytes);
                    bulk_g2s(ring + (size_t)s * p.slot_bytes, pb.W + (size_t)row0 * pb.row_bytes, bytes, &full[s]);
                    if (++slot == p.slots) {
                        slot = 0;
                        if (wrapped) wait_parity ^= 1u;
                        wrapped = true;
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();   // the first phase's input vector comes from whatever ran before this launch
    int slot = 0;
    uint32_t parity = 0;
    for (int ph = 0; ph < p.n_phases; ph++) {
        const ChainPhase& P = p.phases[ph];
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
        }
        CHAIN_TRACE(ph, 0);
        // ---- the phase's activation records
        if (P.prologue == 1) cta_rmsnorm_records(P.a, P.b, P.eps, P.nb, xq, s_sum, warp, lane, nw);
        else if (P.prologue == 2) cta_swiglu_records(P.a, P.b, P.nb, xq, warp, lane, nw);
        else cta_vector_records(P.a, P.nb, xq, warp, lane, nw);
        named_bar_sync(2, nw * 32);
        CHAIN_TRACE(ph, 1);
        // ---- this warp's tiles of the phase
        const int n_tiles = P.n_tiles, n_prob = P.n_problems;
        for (int v = warp * grid + (int)blockIdx.x; v < n_tiles; v += nw * grid) {
            const int s = warp * p.slots + slot;
            if (!mbar_wait_bounded(&full[s], parity, err, 22)) {
                *dead = 1;
                break;
            }
            if (++slot == p.slots) {
                slot = 0;
                parity ^= 1u;
            }
            int j = 0;
#pragma unroll
            for (int q = 1; q < kChainMaxProblems; q++)
                if (q < n_prob && v >= P.prob[q].tile_begin) j = q;
            const BatchProblem& pb = P.prob[j];
            const int row0 = (v - pb.tile_begin) * pb.rt;
            const uint8_t* tile_smem = ring + (size_t)s * p.slot_bytes;
            if (pb.rt == 4) batch_tile<4, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            else if (pb.rt == 2) batch_tile<2, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            else batch_tile<1, LAYOUT, 1>(tile_smem, xq, pb, row0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        // ---- publish: rows written by this CTA are visible device-wide before its arrival counts
        CHAIN_TRACE(ph, 2);
        __threadfence();
        named_bar_sync(2, nw * 32);
        if (*dead) break;
        if (tid == 0) atomicAdd(p.arrive + ph, 1u);
        CHAIN_TRACE(ph, 3);
    }
}

struct ChainHandle {
    ChainPlan plan;
    ChainPhase* d_phases;
    unsigned* d_arrive;
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
        P.pad = 0;
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
    ChainHandle* h = new ChainHandle();
    ChainPlan& p = h->plan;
    p.n_phases = n_phases;
    p.slot_bytes = slot_bytes;
    p.slots = tu.stages < 2 ? 2 : tu.stages;
    p.nw = tu.warps < 1 ? 1 : (tu.warps > 16 ? 16 : tu.warps);
    for (;;) {
        size_t off = 0;
        auto take = [&off](size_t bytes) { size_t at = off; off += (bytes + 127) / 128 * 128; return (int)at; };
        p.off_ring = take((size_t)p.nw * p.slots * p.slot_bytes);
        p.off_xq = take((size_t)xq_bytes);
        p.off_bar = take((size_t)2 * p.nw * p.slots * 8 + 64);
        p.smem = off;
        if (p.smem <= (size_t)kSmemLimit) break;
        if (p.slots > 2) p.slots--;
        else if (p.nw > 4) p.nw--;
        else { delete h; latch(BPDQ_ERR_RANGE); return nullptr; }
    }
    cudaGetDevice(&h->device);
    void* dp = nullptr;
    void* da = nullptr;
    if (check_cuda(cudaMalloc(&dp, sizeof(ChainPhase) * (size_t)n_phases)) || check_cuda(cudaMalloc(&da, sizeof(unsigned) * (size_t)n_phases)) ||
        check_cuda(cudaMemcpy(dp, prog.data(), sizeof(ChainPhase) * (size_t)n_phases, cudaMemcpyHostToDevice))) {
        if (dp) cudaFree(dp);
        if (da) cudaFree(da);
        delete h;
        latch(BPDQ_ERR_CUDA);
        return nullptr;
    }
    h->d_phases = (ChainPhase*)dp;
    h->d_arrive = (unsigned*)da;
    p.phases = h->d_phases;
    p.arrive = h->d_arrive;
    p.trace = nullptr;
    return h;
}

static int chain_run(ChainHandle* h, cudaStream_t s)
{
    if (!h) return latch(BPDQ_ERR_ARG);
    auto kern = k_decode_chain<BPDQ_LAYOUT_BPD, kMidCtaThreads>;
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
    cfg.blockDim = dim3((unsigned)(h->plan.nw + 1) * 32);
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

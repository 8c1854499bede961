// Shared definitions for the quantized-inference kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#define BPDQ_Q4K_BYTES 144
#define BPDQ_Q4K_ELEMS 256
#define BPDQ_Q80_BYTES 34
#define BPDQ_Q80_ELEMS 32
#define BPDQ_Q8K_BYTES 292

// Nibble orders of a Q4_K super-block.
//   0: byte 16j+k  holds element 32j+k (low nibble) and 32j+16+k (high)   [the C-ABI order]
//   1: byte 32c+l  holds element 64c+l (low nibble) and 64c+32+l (high)   [the ggml order]
#define BPDQ_LAYOUT_BPD  0
#define BPDQ_LAYOUT_GGML 1

// Status codes returned by the *_st entry points and latched for the legacy void ones.
enum {
    BPDQ_OK = 0,
    BPDQ_ERR_ARG = -1,        // null pointer, negative size, K not a block multiple
    BPDQ_ERR_ALIGN = -2,      // a pointer that must be 16-byte aligned is not
    BPDQ_ERR_RANGE = -3,      // shape beyond what the kernel supports
    BPDQ_ERR_DEVICE = -4,     // a kernel gave up on a bounded wait, or skipped an out-of-range index
    BPDQ_ERR_CAPTURE = -5,    // library-owned scratch would have to grow while the stream is being captured
    BPDQ_ERR_CUDA = -1000     // BPDQ_ERR_CUDA - cudaError_t
};

namespace bpdq {

// Host-side library state (runtime.cu).
cudaStream_t current_stream();
int latch(int status);                 // remembers the first non-zero status; returns status
int check_cuda(cudaError_t e);         // maps and latches
int sm_count();
int* device_error_flag();              // device pointer to the kernels' error word

struct Tuning {
    int tile_bytes;     // weight bytes staged per ring slot (target)
    int stages;         // ring depth
    int ctas_per_sm;    // persistent CTAs per SM (upper bound)
    int warps;          // consumer warps per CTA (target)
    int pdl;            // launch GEMVs with programmatic dependent launch
    int dequant_variant;   // 0: four outputs per thread, 1: eight outputs per thread
    int dequant_ctas;      // CTAs per SM of the dequant grid
};
Tuning& tuning();

// Scratch memory of the compute entry points (runtime.cu).  A caller-owned workspace is a plain byte
// range that the entry carves up; without one, the library keeps a block per (device, stream, purpose).
// Such a block only grows, and a block that has been handed out is never freed before the process
// ends (a larger replacement is a new allocation; launches in flight and captured graphs that hold
// the old address stay valid).  Growing is refused while the stream is being captured.
enum ScratchKind { kScratchGemmActs = 0, kScratchTc5Acts, kScratchTc5Reduce, kScratchTilesActs, kScratchForward,
                   kScratchQ4ktActs, kScratchQ4ktReduce, kScratchQ80Acts, kScratchKinds };
struct Workspace {
    uint8_t* base;
    size_t bytes, used;
};
// `bytes` of scratch for `kind`: from *ws when ws is given (BPDQ_ERR_RANGE if it does not fit), else the
// library's block for (current device, s, kind).  Returns null and sets *status on failure.
uint8_t* scratch_take(Workspace* ws, int kind, size_t bytes, cudaStream_t s, int* status);

// gemv_batch.cu: bulk-copy GEMV for Q8_0 weights (BPDQ_ERR_RANGE when the shape needs the generic kernel)
int gemv_q8_0_fast(const uint8_t* W, const float* x, float* out, int N, int K, cudaStream_t s);
int gemv_q8_0_fast_multi(int n, const uint8_t* const* Ws, float* const* outs, const int* Ns, const float* x, int K,
                         cudaStream_t s);
// peer_exchange.cu: where a product's results are stored besides its own output (gathered buffers of all
// ranks, byte shifts from the output address), and the flag slots of the per-step signal
constexpr int kMaxPeerTargets = 8;
struct PeerTargets {
    int n;
    long long shift[kMaxPeerTargets];
};
struct PeerFlagSlots {
    int n;
    unsigned* slot[kMaxPeerTargets];
};
bool peer_targets_for(const void* lo, const void* hi, PeerTargets& t);
// gemm_q4k_mma.cu: tensor-core path for many tokens, out[tokens][N], C-ABI nibble order.  ws: caller-owned scratch or
// null (library-owned); sb_ints: optional int32 [tokens][N][K/256][2], the exact (isum, msum) of every super-block
int gemm_q4k_q8k_mma(const uint8_t* W, const float* X, float* out, int tokens, int N, int K, cudaStream_t s,
                     Workspace* ws = nullptr, int32_t* sb_ints = nullptr);
size_t gemm_q4k_q8k_mma_workspace(int tokens, int K);
int gemm_q4k_q8k_tc5(const uint8_t* W, const float* X, float* out, int tokens, int N, int K, cudaStream_t s,
                     Workspace* ws = nullptr, int32_t* sb_ints = nullptr);
size_t gemm_q4k_q8k_tc5_workspace(int tokens, int N, int K);
// gemm_q8_0_tiles.cu: tcgen05 product on re-tiled Q8_0 weights, out[m*N + n], the scalar reference's fp32 order
int gemm_q8_0_tiles(const uint8_t* tiles, const float* X, float* out, int M, int N, int K, cudaStream_t s,
                    Workspace* ws = nullptr);
size_t gemm_q8_0_tiles_workspace(int M, int N, int K);

#ifdef __CUDACC__

// ------------------------------------------------------------------ small device helpers

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h)
{
    // cvt.f32.f16 is exact for every finite binary16 value, subnormals included.
    return __half2float(__ushort_as_half((unsigned short)h));
}

// Six-bit unpack of the 12 scale bytes, four sub-blocks at a time, as packed bytes.
// w0,w1,w2 are the three little-endian words of scales[12]; half 0 = sub-blocks 0..3,
// half 1 = sub-blocks 4..7.  Byte lane j of the result belongs to sub-block 4*half+j.
__device__ __forceinline__ void q4k_scales4(uint32_t w0, uint32_t w1, uint32_t w2, int half,
                                            uint32_t& sc4, uint32_t& mn4)
{
    if (half == 0) {
        sc4 = w0 & 0x3F3F3F3Fu;
        mn4 = w1 & 0x3F3F3F3Fu;
    } else {
        sc4 = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
        mn4 = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
    }
}

__device__ __forceinline__ uint32_t byte_of(uint32_t w, int j) { return (w >> (8 * j)) & 0xFFu; }

// unsigned bytes x signed bytes -> int32
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ------------------------------------------------------------------ mbarrier + bulk copy

__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls, records `code` in the device error word and
// returns false so that the caller can leave the kernel instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* err, int code,
                                                  uint32_t limit = (1u << 22))
{
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    if (err) atomicCAS(err, 0, code);
    return false;
}
// 1-D bulk asynchronous copy global -> this CTA's shared memory, completion counted in bytes
// on an mbarrier.  Source, destination and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}
// Programmatic dependent launch: no-ops unless the launch carried the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

#endif  // __CUDACC__

}  // namespace bpdq

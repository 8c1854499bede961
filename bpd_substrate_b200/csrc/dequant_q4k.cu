// Q4_K super-block dequantization on device pointers.
//
// Replaces k_dequant_q4k (bench/bpd_quant_gpu.cu:35-84), the launch-shape variants of
// bench/bpd_quant_gpu_sweep.cu:36-143 and the two kernels of
// bench/bench_dequant_gpu_h2h.cu:27-72 of the reference.
//
// The value of element e of a super-block is (d*sc_j)*nibble(e) - dmin*mn_j with j = e>>5
// (bench/bpd_quant.c:64-71).  d*sc_j, (d*sc_j)*nibble and dmin*mn_j are exact in binary32
// (11 x 6 x 4 significant bits), so the single rounding is the final subtraction and any
// instruction selection (separate multiply/subtract or fused) gives the same bits.
//
// Memory bound, 144 B in and 1024 B out per super-block, write dominated.  Default kernel
// (k_dequant_q4k_w8): one thread turns one 4-byte nibble word into eight outputs, two float4
// streaming stores (64-byte runs per four lanes, every 32-byte sector written whole); the
// 16-byte header is a load shared by the 32 threads of a super-block through L1; each thread
// keeps four items in flight.  k_dequant_q4k (four outputs per thread, 512 contiguous bytes
// per warp store) is kept selectable; on B200 the eight-output form with 32 CTAs per SM
// measured 5.9 TB/s against 5.3 TB/s.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

// One item = (super-block sb, quad t of 64): outputs 4t .. 4t+3 of that super-block.
template <int LAYOUT>
__device__ __forceinline__ void dequant_item_load(const uint8_t* __restrict__ q, long sb, int t, uint4& hdr,
                                                  uint32_t& w)
{
    const uint8_t* blk = q + sb * BPDQ_Q4K_BYTES;
    hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    // word of qs that holds this quad's four nibbles
    const int widx = (LAYOUT == BPDQ_LAYOUT_BPD) ? (4 * (t >> 3) + (t & 3)) : (8 * (t >> 4) + (t & 7));
    w = __ldg(reinterpret_cast<const uint32_t*>(blk + 16) + widx);
}

template <int LAYOUT>
__device__ __forceinline__ float4 dequant_item_math(const uint4& hdr, uint32_t w, int t)
{
    const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
    const float dmin = f16_bits_to_f32(hdr.x >> 16);
    const int j = t >> 3;  // sub-block of outputs 4t..4t+3
    uint32_t sc4, mn4;
    q4k_scales4(hdr.y, hdr.z, hdr.w, j >> 2, sc4, mn4);
    const float scale = d * (float)byte_of(sc4, j & 3);
    const float minv = dmin * (float)byte_of(mn4, j & 3);
    const bool high = (LAYOUT == BPDQ_LAYOUT_BPD) ? ((t & 4) != 0) : ((t & 8) != 0);
    const uint32_t n = (high ? (w >> 4) : w) & 0x0F0F0F0Fu;
    float4 o;
    o.x = scale * (float)(n & 0xFFu) - minv;
    o.y = scale * (float)((n >> 8) & 0xFFu) - minv;
    o.z = scale * (float)((n >> 16) & 0xFFu) - minv;
    o.w = scale * (float)(n >> 24) - minv;
    return o;
}

template <int LAYOUT, int UNROLL>
__global__ void __launch_bounds__(256) k_dequant_q4k(const uint8_t* __restrict__ q, float* __restrict__ out,
                                                     long n_blocks)
{
    // Items are numbered sb*64 + t; consecutive threads take consecutive items so that the
    // float4 stores of a warp are contiguous.
    const long n_items = n_blocks * 64;
    const long stride = (long)gridDim.x * blockDim.x;
    long item = (long)blockIdx.x * blockDim.x + threadIdx.x;
    float4* out4 = reinterpret_cast<float4*>(out);

    for (; item + (UNROLL - 1) * stride < n_items; item += UNROLL * stride) {
        uint4 hdr[UNROLL];
        uint32_t w[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long it = item + u * stride;
            dequant_item_load<LAYOUT>(q, it >> 6, (int)(it & 63), hdr[u], w[u]);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long it = item + u * stride;
            __stcs(out4 + it, dequant_item_math<LAYOUT>(hdr[u], w[u], (int)(it & 63)));
        }
    }
    for (; item < n_items; item += stride) {
        uint4 hdr;
        uint32_t w;
        dequant_item_load<LAYOUT>(q, item >> 6, (int)(item & 63), hdr, w);
        __stcs(out4 + item, dequant_item_math<LAYOUT>(hdr, w, (int)(item & 63)));
    }
}

// Variant with eight outputs per thread: one nibble word gives four low-nibble and four
// high-nibble elements (two float4 stores 64 bytes apart in the C-ABI order, 128 bytes apart in
// the ggml order), which halves the loads per output.  Item = (super-block, word 0..31).
template <int LAYOUT, int UNROLL>
__global__ void __launch_bounds__(256) k_dequant_q4k_w8(const uint8_t* __restrict__ q, float* __restrict__ out,
                                                        long n_blocks)
{
    const long n_items = n_blocks * 32;
    const long stride = (long)gridDim.x * blockDim.x;
    float4* out4 = reinterpret_cast<float4*>(out);
    for (long item0 = (long)blockIdx.x * blockDim.x + threadIdx.x; item0 < n_items; item0 += UNROLL * stride) {
        uint4 hdr[UNROLL];
        uint32_t w[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long it = item0 + u * stride;
            if (it < n_items) {
                const uint8_t* blk = q + (it >> 5) * BPDQ_Q4K_BYTES;
                hdr[u] = __ldg(reinterpret_cast<const uint4*>(blk));
                w[u] = __ldg(reinterpret_cast<const uint32_t*>(blk + 16) + (it & 31));
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long it = item0 + u * stride;
            if (it >= n_items) continue;
            const int wi = (int)(it & 31);
            const float d = f16_bits_to_f32(hdr[u].x & 0xFFFFu), dmin = f16_bits_to_f32(hdr[u].x >> 16);
            // sub-blocks and float4 positions of the low and the high nibbles of word wi
            int j_lo, j_hi, p_lo, p_hi;
            if (LAYOUT == BPDQ_LAYOUT_BPD) {
                j_lo = j_hi = wi >> 2;
                p_lo = 8 * (wi >> 2) + (wi & 3);
                p_hi = p_lo + 4;
            } else {
                j_lo = 2 * (wi >> 3);
                j_hi = j_lo + 1;
                p_lo = 16 * (wi >> 3) + (wi & 7);
                p_hi = p_lo + 8;
            }
            uint32_t sc4, mn4;
            q4k_scales4(hdr[u].y, hdr[u].z, hdr[u].w, j_lo >> 2, sc4, mn4);
            const float s_lo = d * (float)byte_of(sc4, j_lo & 3), m_lo = dmin * (float)byte_of(mn4, j_lo & 3);
            const float s_hi = d * (float)byte_of(sc4, j_hi & 3), m_hi = dmin * (float)byte_of(mn4, j_hi & 3);
            const uint32_t lo = w[u] & 0x0F0F0F0Fu, hi = (w[u] >> 4) & 0x0F0F0F0Fu;
            float4 a, b;
            a.x = s_lo * (float)(lo & 0xFFu) - m_lo;
            a.y = s_lo * (float)((lo >> 8) & 0xFFu) - m_lo;
            a.z = s_lo * (float)((lo >> 16) & 0xFFu) - m_lo;
            a.w = s_lo * (float)(lo >> 24) - m_lo;
            b.x = s_hi * (float)(hi & 0xFFu) - m_hi;
            b.y = s_hi * (float)((hi >> 8) & 0xFFu) - m_hi;
            b.z = s_hi * (float)((hi >> 16) & 0xFFu) - m_hi;
            b.w = s_hi * (float)(hi >> 24) - m_hi;
            float4* o = out4 + (it >> 5) * 64;
            __stcs(o + p_lo, a);
            __stcs(o + p_hi, b);
        }
    }
}

// Launch-shape study kernels (the sweep entry points).  EPT = outputs per thread per step:
//   1: thread -> one output (the "v1" shape), 2: thread -> one qs byte, two outputs (the
//   "ilp2"/"multi" shape).  A CTA of blockDim.x threads covers sb_per_cta super-blocks and
//   always writes all 256 outputs of each, whatever the CTA size.
template <int EPT>
__global__ void k_dequant_q4k_shape(const uint8_t* __restrict__ q, float* __restrict__ out, int n_blocks,
                                    int sb_per_cta)
{
    const long first = (long)blockIdx.x * sb_per_cta;
    const int units_per_sb = 256 / EPT;
    for (int u = threadIdx.x; u < sb_per_cta * units_per_sb; u += blockDim.x) {
        const long sb = first + u / units_per_sb;
        if (sb >= n_blocks) break;
        const int r = u % units_per_sb;
        const uint8_t* blk = q + sb * BPDQ_Q4K_BYTES;
        const uint32_t* hw = reinterpret_cast<const uint32_t*>(blk);
        const uint32_t h0 = __ldg(hw);
        const float d = f16_bits_to_f32(h0 & 0xFFFFu), dmin = f16_bits_to_f32(h0 >> 16);
        // byte index k within the sub-block and sub-block j
        const int j = (EPT == 1) ? (r >> 5) : (r >> 4);
        const int k = (EPT == 1) ? (r & 15) : (r & 15);
        uint32_t sc4, mn4;
        q4k_scales4(__ldg(hw + 1), __ldg(hw + 2), __ldg(hw + 3), j >> 2, sc4, mn4);
        const float scale = d * (float)byte_of(sc4, j & 3);
        const float minv = dmin * (float)byte_of(mn4, j & 3);
        const uint32_t b = __ldg(blk + 16 + 16 * j + k);
        float* o = out + sb * 256 + 32 * j;
        if (EPT == 1) {
            const bool high = (r & 16) != 0;
            o[k + (high ? 16 : 0)] = scale * (float)(high ? (b >> 4) : (b & 15u)) - minv;
        } else {
            o[k] = scale * (float)(b & 15u) - minv;
            o[k + 16] = scale * (float)(b >> 4) - minv;
        }
    }
}

static int check_args(const void* q, const void* out, long n_blocks)
{
    if (n_blocks < 0 || (n_blocks > 0 && (!q || !out))) return BPDQ_ERR_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return BPDQ_ERR_ALIGN;
    return 0;
}

static int launch_dequant(const void* q, float* out, long n_blocks, int layout, cudaStream_t s)
{
    int rc = check_args(q, out, n_blocks);
    if (rc) return latch(rc);
    if (n_blocks == 0) return 0;
    constexpr int UNROLL = 4;
    const int variant = tuning().dequant_variant;
    const long n_items = n_blocks * (variant == 1 ? 32 : 64);
    // Persistent-style grid: a whole number of waves of CTAs of 256 threads per SM.
    long want = (n_items + 256L * UNROLL - 1) / (256L * UNROLL);
    long cap = (long)sm_count() * tuning().dequant_ctas;
    int grid = (int)(want < cap ? (want < 1 ? 1 : want) : cap);
    const uint8_t* qq = (const uint8_t*)q;
    if (variant == 1) {
        if (layout == BPDQ_LAYOUT_GGML) k_dequant_q4k_w8<BPDQ_LAYOUT_GGML, UNROLL><<<grid, 256, 0, s>>>(qq, out, n_blocks);
        else k_dequant_q4k_w8<BPDQ_LAYOUT_BPD, UNROLL><<<grid, 256, 0, s>>>(qq, out, n_blocks);
    } else {
        if (layout == BPDQ_LAYOUT_GGML) k_dequant_q4k<BPDQ_LAYOUT_GGML, UNROLL><<<grid, 256, 0, s>>>(qq, out, n_blocks);
        else k_dequant_q4k<BPDQ_LAYOUT_BPD, UNROLL><<<grid, 256, 0, s>>>(qq, out, n_blocks);
    }
    return check_cuda(cudaGetLastError());
}

template <int EPT>
static void launch_shape(const uint8_t* q, float* o, int nb, int threads, int sb_per_cta)
{
    if (nb < 0 || (nb > 0 && (!q || !o))) { latch(BPDQ_ERR_ARG); return; }
    if (nb == 0) return;
    int grid = (nb + sb_per_cta - 1) / sb_per_cta;
    k_dequant_q4k_shape<EPT><<<grid, threads, 0, current_stream()>>>(q, o, nb, sb_per_cta);
    check_cuda(cudaGetLastError());
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

// bench/bpd_quant_gpu.cu:162-164
void bpd_dequant_q4k_gpu(const uint8_t* qdata, float* output, int n_blocks)
{
    launch_dequant(qdata, output, n_blocks, BPDQ_LAYOUT_BPD, current_stream());
}
int bpd_dequant_q4k_gpu_st(const uint8_t* qdata, float* output, size_t n_blocks, int layout, void* stream)
{
    if (layout != BPDQ_LAYOUT_BPD && layout != BPDQ_LAYOUT_GGML) return latch(BPDQ_ERR_ARG);
    return launch_dequant(qdata, output, (long)n_blocks, layout, (cudaStream_t)stream);
}

// bench/bench_dequant_gpu_h2h.cu:74-76 -- both names run the ggml nibble order, as both do there.
void run_llamacpp(const void* q, float* o, int nb) { launch_dequant(q, o, nb, BPDQ_LAYOUT_GGML, current_stream()); }
void run_bpd(const void* q, float* o, int nb) { launch_dequant(q, o, nb, BPDQ_LAYOUT_GGML, current_stream()); }

// bench/bpd_quant_gpu_sweep.cu:134-143 -- same launch shapes; every shape writes whole blocks.
void dequant_v1_256(const uint8_t* q, float* o, int nb) { launch_shape<1>(q, o, nb, 256, 1); }
void dequant_v1_128(const uint8_t* q, float* o, int nb) { launch_shape<1>(q, o, nb, 128, 1); }
void dequant_v1_64(const uint8_t* q, float* o, int nb) { launch_shape<1>(q, o, nb, 64, 1); }
void dequant_v1_32(const uint8_t* q, float* o, int nb) { launch_shape<1>(q, o, nb, 32, 1); }
void dequant_ilp2(const uint8_t* q, float* o, int nb) { launch_shape<2>(q, o, nb, 128, 1); }
void dequant_multi2(const uint8_t* q, float* o, int nb) { launch_shape<2>(q, o, nb, 128, 2); }
void dequant_multi4(const uint8_t* q, float* o, int nb) { launch_shape<2>(q, o, nb, 128, 4); }
void dequant_multi8(const uint8_t* q, float* o, int nb) { launch_shape<2>(q, o, nb, 128, 8); }

}  // extern "C"

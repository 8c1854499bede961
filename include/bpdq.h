/* bpdq.h -- C ABI of libbpdq.so: B200 (sm_100a) kernels for BPD's quantized-inference path.
 *
 * Every function is plain C: raw pointers and sizes, no C++ or torch types.  "device"
 * pointers are CUDA device addresses (from the *_alloc helpers below, or from any other
 * allocator in the same process, e.g. a torch tensor's data_ptr()).
 *
 * Two kinds of entry point:
 *   1. Drop-ins with the reference's own names and signatures (void return, int sizes).  They
 *      launch on the library's current stream (bpdq_set_stream; default: the legacy default
 *      stream, as in the reference) and latch any error for bpdq_last_status().
 *   2. Additive *_st / *_cuda forms that return a status (0 = ok, negative = error, see the
 *      BPDQ_ERR_* list), take size_t sizes where an int would overflow, and an explicit
 *      stream (a cudaStream_t passed as void*).
 *
 * There is no CPU fallback anywhere: every compute entry launches a CUDA kernel.
 *
 * Each declaration names the reference interface it replaces (path:line inside
 * heath-hunnicutt-ruach-tov/bpd-substrate).
 */
#ifndef BPDQ_H
#define BPDQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes */
#define BPDQ_STATUS_OK 0
#define BPDQ_STATUS_ERR_ARG (-1)     /* null pointer, negative size, K not a block multiple */
#define BPDQ_STATUS_ERR_ALIGN (-2)   /* pointer not aligned as the kernel needs (16 B for weights) */
#define BPDQ_STATUS_ERR_RANGE (-3)   /* shape beyond what the kernel supports */
#define BPDQ_STATUS_ERR_DEVICE (-4)  /* a kernel gave up on a bounded wait, or skipped an out-of-range index */
#define BPDQ_STATUS_ERR_CAPTURE (-5) /* library-owned scratch would have to grow while the stream is being captured */
#define BPDQ_STATUS_ERR_CUDA (-1000) /* minus the cudaError_t value */

/* ---- library state (additive; the reference keeps none) ------------------------------ */
void bpdq_set_stream(void* cuda_stream);   /* stream used by the void drop-ins */
void* bpdq_get_stream(void);
int bpdq_last_status(void);                /* first error since the last clear (synchronizes) */
int bpdq_device_error_word(void);
void bpdq_clear_status(void);
/* Launch tuning, process-wide (set it once, before the launches it should apply to; not per stream): max bytes
 * per weight tile of the GEMV ring, ring slots per warp, CTAs per SM, consumer warps per CTA, programmatic
 * dependent launch on/off.  <=0 (pdl: <0) keeps a field. */
void bpdq_set_tuning(int tile_bytes, int slots, int ctas_per_sm, int warps, int pdl);
/* dequant launch tuning: variant 0 = four outputs per thread, 1 = eight; CTAs per SM of the grid */
void bpdq_set_dequant_tuning(int variant, int ctas_per_sm);
int bpdq_sm_count(void);

/* ---- scratch memory of the compute entries -------------------------------------------------
 * Three kinds of entry need device scratch beyond their inputs and outputs (quantized activations,
 * split-K partial sums, the forward pass's vectors): the many-token products bpd_qmm_q4k_q8k_cuda /
 * _mma_cuda / _tc5_cuda / gpu_matmul_q4k, bpd_qmatmul_q8_0_tiles_cuda and bpd_qmatmul_q8_0_llamafile_cuda,
 * and bpd_llama_forward*_cuda.  Each has two forms:
 *   *_ws_cuda(..., workspace, workspace_bytes, stream): the caller owns the scratch (16-byte aligned, at
 *     least the matching *_workspace_bytes()).  Nothing is allocated and no state is shared between calls:
 *     calls on different streams may overlap if their workspaces differ; BPDQ_STATUS_ERR_RANGE if too small.
 *   the plain form: the library keeps one block per (device, stream, purpose).  Calls on one stream are ordered
 *     by the stream; calls on different streams use different blocks.  A block grows by replacement the first
 *     time a larger size is asked for on that stream (cudaMalloc, which synchronizes the device); a block that
 *     was handed out is never freed before the process ends, so launches in flight and captured graphs that
 *     hold its address stay valid.  While a stream is being captured a block cannot grow: the call returns
 *     BPDQ_STATUS_ERR_CAPTURE and launches nothing -- make one call of that size on the stream before the
 *     capture (a warm-up run), or use the *_ws_cuda form. */

/* ---- device memory helpers (additive, size_t) ------------------------------------------ */
void* bpdq_alloc(size_t bytes);
void bpdq_free(void* dev);
void bpdq_h2d(void* dev, const void* host, size_t bytes);
void bpdq_d2h(void* host, const void* dev, size_t bytes);
void bpdq_d2d(void* dst, const void* src, size_t bytes);
int bpdq_h2d_async(void* dev, const void* host, size_t bytes, void* stream);
int bpdq_d2h_async(void* host, const void* dev, size_t bytes, void* stream);
void* bpdq_host_alloc(size_t bytes);       /* pinned host memory */
void bpdq_host_free(void* host);
void bpdq_sync(void);
int bpdq_stream_sync(void* stream);

/* ---- events, memset, streams, CUDA graphs (additive) ------------------------------------ */
void* bpdq_event_create(void);
void bpdq_event_destroy(void* ev);
int bpdq_event_record(void* ev, void* stream);
float bpdq_event_elapsed_ms(void* start, void* stop);  /* waits for stop */
int bpdq_memset_async(void* dev, int value, size_t bytes, void* stream);
void* bpdq_stream_create(void);
int bpdq_stream_wait_event(void* stream, void* ev);    /* later work on stream waits for the event */
void bpdq_stream_destroy(void* stream);
int bpdq_graph_begin(void* stream);        /* start capturing launches made on stream */
void* bpdq_graph_end(void* stream);        /* -> executable graph handle, NULL on error */
int bpdq_graph_launch(void* graph, void* stream);
void bpdq_graph_destroy(void* graph);
int bpdq_set_device(int device);
int bpdq_mem_info(size_t* free_bytes, size_t* total_bytes);   /* cudaMemGetInfo of the current device */
int bpdq_l2_bytes(void);

/* ---- reference memory helpers, name for name ------------------------------------------- */
/* bench/bpd_quant_gpu.cu:172-176 (first argument of h2d/d2h is the destination) */
void* qgpu_alloc(int bytes);
void qgpu_free(void* p);
void qgpu_h2d(void* dev, const void* host, int bytes);
void qgpu_d2h(void* host, const void* dev, int bytes);
void qgpu_sync(void);
/* bench/bpd_quant_gpu_sweep.cu:145-149 */
void* sgpu_alloc(int bytes);
void sgpu_free(void* p);
void sgpu_h2d(void* dev, const void* host, int bytes);
void sgpu_d2h(void* host, const void* dev, int bytes);
void sgpu_sync(void);
/* bench/bench_dequant_gpu_h2h.cu:77-81 */
void* galloc(int bytes);
void gfree(void* p);
void gh2d(void* dev, const void* host, int bytes);
void gd2h(void* host, const void* dev, int bytes);
void gsync(void);
/* generators/generate_llama_kernels.pl:32-60 */
void* gpu_alloc(int bytes);
void gpu_free(void* p);
void gpu_copy_h2d(void* dev, const void* host, int bytes);
void gpu_copy_d2h(void* host, const void* dev, int bytes);
void gpu_copy_d2d(void* dst, const void* src, int bytes);
void gpu_sync(void);

/* ---- Q4_K dequantization (device pointers) --------------------------------------------- */
/* bench/bpd_quant_gpu.cu:162-164 -- 144-byte super-blocks -> 256 floats each, the nibble
 * order of bench/bpd_quant.c:68-72.  Bit-exact with bpd_dequant_q4k (bench/bpd_quant.c:77). */
void bpd_dequant_q4k_gpu(const uint8_t* qdata, float* output, int n_blocks);
/* layout 0 = that order, 1 = the ggml order of bench/bench_dequant_gpu_h2h.cu:35-46 */
int bpd_dequant_q4k_gpu_st(const uint8_t* qdata, float* output, size_t n_blocks, int layout, void* stream);
/* bench/bench_dequant_gpu_h2h.cu:74-76 (ggml nibble order, both names) */
void run_llamacpp(const void* q, float* out, int nb);
void run_bpd(const void* q, float* out, int nb);
/* bench/bpd_quant_gpu_sweep.cu:134-143 -- the launch-shape study; unlike the reference's
 * v1_128/64/32 every shape here writes all 256 outputs of every block. */
void dequant_v1_256(const uint8_t* q, float* out, int nb);
void dequant_v1_128(const uint8_t* q, float* out, int nb);
void dequant_v1_64(const uint8_t* q, float* out, int nb);
void dequant_v1_32(const uint8_t* q, float* out, int nb);
void dequant_ilp2(const uint8_t* q, float* out, int nb);
void dequant_multi2(const uint8_t* q, float* out, int nb);
void dequant_multi4(const uint8_t* q, float* out, int nb);
void dequant_multi8(const uint8_t* q, float* out, int nb);

/* ---- Q4_K x Q8_K (weights 4-bit, activations quantized to 8-bit in the kernel) ---------- */
/* No counterpart in the reference (docs/llama-kernel-audit.md:65 "Q4_K . Q8_K direct" is an
 * unbuilt design); defined from its Q8_0 analogues bench/bpd_cpu.c:4106-4136, 4263-4280.
 * Q8_K block = 292 B: float d, int8 qs[256], int16 bsums[16] (size: lib/gguf_emit_manifest.pl:142). */
int bpd_quant_q8_K_cuda(const float* x, uint8_t* y, size_t n_elements, void* stream);
/* out[M] = W[M][K] . q8K(x[K]); W in the nibble order of bench/bpd_quant.c:68-72 */
int bpd_qmatmul_q4k_q8k_cuda(const uint8_t* qweight, const float* x, float* out, int M, int K, void* stream);
/* n <= 4 matrices that read the same x in ONE launch (q/k/v, gate/up): outs[j][Ms[j]] */
int bpd_qmatmul_q4k_q8k_multi_cuda(int n, const uint8_t* const* qweights, float* const* outs, const int* Ms,
                                   const float* x, int K, void* stream);
/* n independent products out_j[M_j] = W_j[M_j][K_j] . q8K(x_j[K_j]) in as few launches as
 * possible (shapes may differ; several may share x).  descs is a host array. */
typedef struct bpdq_gemv_desc {
    const uint8_t* W;
    const float* x;
    float* out;
    int M, K;
} bpdq_gemv_desc;
int bpd_qmatmul_q4k_q8k_batch_cuda(int n, const bpdq_gemv_desc* descs, void* stream);
/* same with caller-owned device scratch for the quantized activations: a small kernel quantizes
 * each distinct x once and the GEMV kernel bulk-copies the result, instead of every CTA
 * quantizing every x.  Ordered after everything ahead of it in the stream, like any launch. */
int bpd_qmatmul_q4k_q8k_batch_ws_cuda(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes,
                                      void* stream);
/* same, for callers that can promise more: every x is complete when the call is made (no launch
 * still in flight on the stream writes it) and no launch still in flight uses the scratch.  The
 * quantizer then reads x ahead of stream order, under the tail of the launch before it.  Right for
 * independent products whose inputs were uploaded beforehand; WRONG for a dependent chain. */
int bpd_qmatmul_q4k_q8k_batch_ready_cuda(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes,
                                         void* stream);
size_t bpdq_batch_workspace_bytes(int n, const bpdq_gemv_desc* descs);
/* No counterpart in the reference.  The same batched product for callers that cannot allocate
 * device memory at the time of the call: plugins of a host application that owns every byte of
 * the GPU and hands out none, code in a region where the CUDA allocator must not be entered
 * (cudaMalloc and cudaFree synchronize the whole device), and latency-bound loops that may not
 * pay for an allocation.  The scratch for the quantized activations
 * is a fixed 256 KiB array inside the library (bpdq_batch_static_capacity(); every GPU that
 * loads the library holds it until the process ends), so this entry point allocates nothing
 * and frees nothing; inputs and outputs are still the caller's.
 *  - Limit: bpdq_batch_workspace_bytes(n, descs) must not exceed the capacity (about 233,000
 *    activations over the call's vectors); a larger call returns -3 and launches nothing.
 *  - The first call on a device looks up the array's device address and sets kernel
 *    attributes; make that first call before any stream capture begins.
 *  - Every call uses the same array and overwrites what the previous call left there (nothing
 *    in it needs to start at zero).  Calls on ONE stream are ordered by the library; calls that
 *    can overlap on the GPU (different streams, different host threads) race on the array and
 *    must be serialized by the caller. */
int bpd_qmatmul_q4k_q8k_batch_static_cuda(int n, const bpdq_gemv_desc* descs, void* stream);
size_t bpdq_batch_static_capacity(void);
/* Any number of independent products as ONE persistent launch per 128 products (plus one launch that quantizes
 * their activation vectors): the weights of all products stream through the shared-memory ring without a launch
 * boundary in between, every consumer warp refilling its own ring slots, and the activation records are swapped
 * through two shared-memory buffers phase by phase without any CTA-wide barrier.  bpdq_gemv_stream_create plans
 * the products (same descriptors as the batched entries), lays the activation records out in `workspace`
 * (bpdq_batch_workspace_bytes(n, descs) bytes, 16-byte aligned, must stay allocated) and uploads the plan (it
 * allocates device memory; peer targets registered with bpdq_set_peer_outputs are read here);
 * bpdq_gemv_stream_run launches it, stream-ordered like any launch; bpdq_gemv_stream_run_ready is for callers who
 * can promise that every activation vector is complete when the call is made (nothing in flight writes them): the
 * quantizer then reads them under the tail of the launch ahead.  Same bits as the batched entries.
 * bpdq_gemv_stream_launches: kernel launches one run makes. */
void* bpdq_gemv_stream_create(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes);   /* NULL on error */
int bpdq_gemv_stream_run(void* handle, void* stream);
int bpdq_gemv_stream_run_ready(void* handle, void* stream);
int bpdq_gemv_stream_launches(void* handle);
void bpdq_gemv_stream_destroy(void* handle);
/* the same stream for Q8_0 weights (bench/bpd_cpu.c:4295-4315 at one activation row, many matrices per launch):
 * descs[j].W = Q8_0 rows [M][K/32][34], K a multiple of 256; run / run_ready / destroy as above */
size_t bpdq_gemv_stream_q8_0_workspace_bytes(int n, const bpdq_gemv_desc* descs);
void* bpdq_gemv_stream_create_q8_0(int n, const bpdq_gemv_desc* descs, void* workspace, size_t workspace_bytes);

/* ---- Decode glue.  Replaces, around the products of a decoder layer, the separate elementwise
 * launches of the reference's decode loop (inference/llamatov_gpu_llama.py:119-166: gpu_rms_norm,
 * gpu_silu, gpu_mul, gpu_add; kernels lib/kernel_templates_llama.pl:529-593, :600-830): each step
 * writes the next product's quantized activation records (144 bytes per 128 activations: int8
 * values, four int16 sub-block sums, the fp32 block scale) instead of an fp32 vector, and the
 * residual add is the product's own epilogue.  Same arithmetic as the separate calls, bit for bit.
 * All launch asynchronously on `stream` and are ordered after the launch before them. */
size_t bpdq_records_bytes(int K);                       /* bytes of the records of K activations */
/* records = q8K(x) */
int bpd_quant_q8k_records_cuda(const float* x, void* records, int K, void* stream);
/* records[r] = q8K(rms_norm(x[r], w, eps)), rows of K floats (gpu_rms_norm's arithmetic) */
int bpd_rmsnorm_q8k_records_cuda(const float* x, const float* w, void* records, int rows, int K, float eps, void* stream);
/* records = q8K(silu(gate) * up) (gpu_silu then gpu_mul) */
int bpd_swiglu_q8k_records_cuda(const float* gate, const float* up, void* records, int K, void* stream);
/* out_j[M_j] (+)= W_j[M_j][K] . records for n <= 8 matrices with the same K in one launch; descs[j].x is
 * ignored; bit j of accumulate_mask: add to out_j instead of overwriting it (gpu_add folded in) */
int bpd_qmatmul_q4k_records_cuda(int n, const bpdq_gemv_desc* descs, const void* records, unsigned accumulate_mask,
                                 void* stream);
/* The step, its quantization, the products and the residual add as ONE launch: every CTA of the
 * product kernel applies the step to the input vector itself while its weight ring fills.
 * prologue 0: x = a;  1: x = rms_norm(a, weights b, eps);  2: x = silu(a) * b;  then
 * out_j[M_j] (+)= W_j[M_j][K] . q8K(x), n <= 8 matrices with the same K.  Same bits as the separate calls. */
int bpd_qmatmul_q4k_fused_cuda(int n, const bpdq_gemv_desc* descs, int prologue, const float* a, const float* b, float eps,
                               unsigned accumulate_mask, void* stream);
/* A whole chain of dependent phases (each: step, quantize, up to three products with the same K,
 * optional residual adds) as ONE cooperative launch of one CTA per SM: the weights of all phases
 * stream back to back through the shared-memory ring, the consumer warps meet at a grid-wide barrier
 * (bounded wait, status -4 on a timeout) between phases.  The program is planned and uploaded once
 * (bpdq_chain_create, which allocates device memory), then run once per token.  Phase fields as the
 * arguments of bpd_qmatmul_q4k_fused_cuda.  Same bits as the separate calls. */
typedef struct bpdq_chain_phase {
    int n, prologue;
    const float* a;
    const float* b;
    float eps;
    unsigned accumulate_mask;
    bpdq_gemv_desc prod[3];
} bpdq_chain_phase;
void* bpdq_chain_create(int n_phases, const bpdq_chain_phase* phases);   /* NULL on error (bpdq_last_status) */
int bpdq_chain_run(void* chain, void* stream);
void bpdq_chain_destroy(void* chain);
/* out[tokens][M]; layout 0/1 as above; xsrc 0: x is float [tokens][K], 1: x is Q8_K blocks
 * [tokens][K/256]; subdots (may be NULL): int32 [M][K/256][8], token 0's exact sub-block dots */
int bpd_qmm_q4k_q8k_cuda(const uint8_t* qweight, const void* x, float* out, int tokens, int M, int K, int layout,
                         int xsrc, int32_t* subdots, void* stream);
/* the same with caller-owned scratch (see "scratch memory" above) */
size_t bpdq_qmm_q4k_q8k_workspace_bytes(int tokens, int M, int K);
int bpd_qmm_q4k_q8k_ws_cuda(const uint8_t* qweight, const void* x, float* out, int tokens, int M, int K, int layout,
                            int xsrc, int32_t* subdots, void* workspace, size_t workspace_bytes, void* stream);
/* the int8 tensor-core kernel behind bpd_qmm_q4k_q8k_cuda for more than 8 tokens, callable at any
 * token count: out[tokens][M], X float [tokens][K], nibble order of bench/bpd_quant.c:68-72 */
int bpd_qmm_q4k_q8k_mma_cuda(const uint8_t* qweight, const float* X, float* out, int tokens, int M, int K, void* stream);
/* the same product on tcgen05 tensor cores with TMEM accumulators (M >= 128 weight rows) */
int bpd_qmm_q4k_q8k_tc5_cuda(const uint8_t* qweight, const float* X, float* out, int tokens, int M, int K, void* stream);
/* checking forms of the two tensor-core kernels: besides out they store, for every (token, row, super-block),
 * the exact int32 pair (isum, msum) the fp32 scales are applied to; sb_ints is int32 [tokens][M][K/256][2] */
int bpd_qmm_q4k_q8k_mma_ints_cuda(const uint8_t* qweight, const float* X, float* out, int32_t* sb_ints, int tokens, int M, int K,
                                  void* stream);
int bpd_qmm_q4k_q8k_tc5_ints_cuda(const uint8_t* qweight, const float* X, float* out, int32_t* sb_ints, int tokens, int M, int K,
                                  void* stream);
/* ---- Q4_K re-tiled in groups of 16 rows ("rg16"), for products with 2..64 activation rows and more.
 * The idea of inference/llamatov_c_inference.py:88-100 (a weight layout made for the kernel that reads it) applied to
 * Q4_K as a pure, exactly invertible permutation: per group of 16 rows and super-block a unit of 2304 bytes = the 16
 * block headers (row r at 16 r), then the nibble words in the order the int8 MMA m16n8k32 takes its A fragments: for
 * q = 0..3 and lane L = 0..31 (g = L / 4, t = L % 4) the 16 bytes at 256 + 512 q + 16 L hold word t of sub-block 2q of
 * rows g and g + 8, then of sub-block 2q + 1 (word t of sub-block j = bytes 16 + 16 j + 4 t .. + 3 of the row's block);
 * units ordered [row group][super-block]; rows beyond N are zero.  tiles: 16-byte aligned, bpd_q4k_rg16_bytes(N, K). */
size_t bpd_q4k_rg16_bytes(int N, int K);
int bpd_repack_q4k_rg16_cuda(const uint8_t* raw, uint8_t* tiles, int N, int K, void* stream);
int bpd_unrepack_q4k_rg16_cuda(const uint8_t* tiles, uint8_t* raw, int N, int K, void* stream);
/* out[tokens][M] = q8K(X[tokens][K]) . W^T on re-tiled weights, any number of tokens (64 per pass over the weights): a
 * streaming kernel (every warp refills its own ring slots with 1-D bulk copies of its row group's units; quantized
 * activations swapped through two shared-memory buffers) around mma.sync int8 MMAs; the arithmetic, order and bits of
 * bpd_qmm_q4k_q8k_mma_cuda.  The plain form uses library-owned scratch of the stream (see "scratch memory"). */
int bpd_qmm_q4k_q8k_rg16_cuda(const uint8_t* tiles, const float* X, float* out, int tokens, int M, int K, void* stream);
size_t bpdq_qmm_q4k_q8k_rg16_workspace_bytes(int tokens, int K);
int bpd_qmm_q4k_q8k_rg16_ws_cuda(const uint8_t* tiles, const float* X, float* out, int tokens, int M, int K, void* workspace,
                                 size_t workspace_bytes, void* stream);
int bpd_qmm_q4k_q8k_rg16_ints_cuda(const uint8_t* tiles, const float* X, float* out, int32_t* sb_ints, int tokens, int M, int K,
                                   void* stream);    /* + the exact (isum, msum) pairs, as the _ints forms above */
/* Any number of independent products on re-tiled weights, each with its own X [tokens][K_j] (tokens 1..64), as one
 * persistent launch per 128 products (plus one launch that quantizes the activations): descs[j].W = re-tiled weights,
 * descs[j].x = X_j, out_j [tokens][M_j].  create plans and uploads the tables (it allocates device memory); workspace:
 * bpdq_gemm_rg16_stream_workspace_bytes, 16-byte aligned, must stay allocated.  run is stream-ordered like any launch. */
size_t bpdq_gemm_rg16_stream_workspace_bytes(int n, const bpdq_gemv_desc* descs, int tokens);
void* bpdq_gemm_rg16_stream_create(int n, const bpdq_gemv_desc* descs, int tokens, void* workspace, size_t workspace_bytes);
int bpdq_gemm_rg16_stream_run(void* handle, void* stream);
int bpdq_gemm_rg16_stream_launches(void* handle);
void bpdq_gemm_rg16_stream_destroy(void* handle);
/* dispatch-shaped forms: argument order of gpu_vecmat (lib/kernel_templates_llama.pl:147-158)
 * and gpu_matmul (lib/kernel_templates_llama.pl:1104-1112) with the fp32 [K][N] weight
 * replaced by Q4_K rows [N][K/256][144] */
void gpu_vecmat_q4k(const float* a, const uint8_t* wq, float* c, int k, int n);
void gpu_matmul_q4k(const float* A, const uint8_t* wq, float* C, int M, int N, int K);

/* ---- Q4_K weights x fp32 activations (no activation quantization) --------------------------- */
/* bench/bpd_quant_gpu.cu:166-169  output[M] = dequant(qweight[M][K]) . x[K] */
void bpd_qmatmul_q4k_gpu(const uint8_t* qweight, const float* x, float* output, int M, int K);
int bpd_qmatmul_q4k_gpu_st(const uint8_t* qweight, const float* x, float* output, int M, int K, void* stream);
/* bench/bpd_quant.c:114-137 (bpd_qmm_q4k) on device pointers: C[M][N] = dequant(qA[M][K]) @ B[K][N] */
int bpd_qmm_q4k_cuda(const uint8_t* qA, const float* B, float* C, int M, int N, int K, void* stream);

/* ---- Q8_0 (34-byte blocks: fp16 scale + 32 int8), device-pointer twins of the CPU entries --- */
/* bench/bpd_cpu.c:3960-3973  bpd_dequant_q8_0_cpu */
int bpd_dequant_q8_0_cuda(const uint8_t* raw, float* out, size_t n_blocks, void* stream);
/* bench/bpd_cpu.c:4106-4136  bpd_quant_q8_0_cpu (byte-identical blocks) */
int bpd_quant_q8_0_cuda(const float* x, uint8_t* y, size_t n_elements, void* stream);
/* the exact int32 core of bench/bpd_cpu.c:4263-4280 bpd_qdot_q8_0_q8_0_cpu, per block */
int bpd_q8_0_block_dots_cuda(const uint8_t* w, const uint8_t* a, int32_t* dots, size_t n_blocks, void* stream);
/* bench/bpd_cpu.c:4295-4315  bpd_qmatmul_q8_0_cpu: out[m*N+n] = W row n . q8_0(X row m) */
int bpd_qmatmul_q8_0_cuda(const uint8_t* W, const float* X, float* out, int M, int N, int K, void* stream);
/* bench/bpd_cpu.c:4428-4459  bpd_qmatmul_q8_0_llamafile_cpu: fp32 activations X[m_tokens][K], out[token*m_weight + row];
 * quantizes X to Q8_0 (library-owned scratch of the stream) and runs the dispatcher below */
int bpd_qmatmul_q8_0_llamafile_cuda(const uint8_t* W, const float* X, float* out, int m_weight, int m_tokens, int K, void* stream);
/* bench/bpd_gemm_q8_0_cpu.c:159-207  bpd_qmatmul_q8_0_dispatch_cpu: activations already Q8_0 rows [m_tokens][K/32][34].
 * Eight fp32 partial sums per output, added in the order of the reference's AVX lanes: its result bit for bit. */
int bpd_qmatmul_q8_0_dispatch_cuda(const uint8_t* Wq, const uint8_t* Xq, float* out, int m_weight, int m_tokens, int K, void* stream);
/* bench/bpd_gemm_q8_0_cpu.c:32-97  bpd_gemm_q8_0_{RM}_{RN}_cpu: one tile of RM weight rows (w_stride bytes apart) x RN
 * activation rows (a_stride bytes apart) over k blocks, out[j*ldc + i] */
int bpd_gemm_q8_0_1_1_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_1_2_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_1_4_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_2_1_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_2_2_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_2_4_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_4_1_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_4_2_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
int bpd_gemm_q8_0_4_4_cuda(const uint8_t* W_tile, const uint8_t* B_tile, int k, int w_stride, int a_stride, float* out, int ldc, void* stream);
/* bench/bpd_cpu.c:4002-4013  bpd_embed_lookup_q8_0_cpu.  An id below zero (and, in the _vocab form, at or above
 * vocab_size) is not looked up: that row of `out` is left as it was and bpdq_last_status() reports -4. */
int bpd_embed_lookup_q8_0_cuda(const uint8_t* table, const int32_t* ids, float* out, int n_tokens, int embed_dim,
                               void* stream);
int bpd_embed_lookup_q8_0_vocab_cuda(const uint8_t* table, const int32_t* ids, float* out, int n_tokens, int embed_dim,
                                     int vocab_size, void* stream);
/* Q8_0 re-tiled for the tensor cores: the idea of inference/llamatov_c_inference.py:88-100 ("Q8 padded 64B
 * coalesced [nb,N,64]") as a pure permutation of the Q8_0 bytes.  Per tile of 128 rows and block of 32
 * elements a unit of 4352 bytes: the 128x32 int8 quants, element (r,k) at (k/16)*2048 + (r/8)*128 +
 * (r%8)*16 + k%16, then the 128 fp16 scales; units ordered [row tile][block]; rows beyond N are zero.
 * tiles must be 16-byte aligned and bpd_q8_0_tiles_bytes(N, K) long. */
size_t bpd_q8_0_tiles_bytes(int N, int K);
int bpd_repack_q8_0_tiles_cuda(const uint8_t* raw, uint8_t* tiles, int N, int K, void* stream);
int bpd_unrepack_q8_0_tiles_cuda(const uint8_t* tiles, uint8_t* raw, int N, int K, void* stream);
/* bench/bpd_cpu.c:4295-4315  bpd_qmatmul_q8_0_cpu on re-tiled weights, any number of tokens M, on the
 * tcgen05 tensor cores; the fp32 operations per block are the scalar reference's, in its order */
int bpd_qmatmul_q8_0_tiles_cuda(const uint8_t* tiles, const float* X, float* out, int M, int N, int K, void* stream);
size_t bpdq_qmatmul_q8_0_tiles_workspace_bytes(int M, int N, int K);
int bpd_qmatmul_q8_0_tiles_ws_cuda(const uint8_t* tiles, const float* X, float* out, int M, int N, int K, void* workspace,
                                   size_t workspace_bytes, void* stream);
/* gpu_vecmat's argument order (lib/kernel_templates_llama.pl:147-158) with Q8_0 rows [n][k/32][34] */
void gpu_vecmat_q8_0(const float* a, const uint8_t* wq, float* c, int k, int n);

/* ---- fp32 operators of the decode dispatch (inference/llamatov_gpu_llama.py:15-31) ----------- */
/* lib/kernel_templates_llama.pl:147-158  c[n] = a[k] . b[k][n] */
void gpu_vecmat(const float* a, const float* b, float* c, int k, int n);
/* lib/kernel_templates_llama.pl:583-593 */
void gpu_rms_norm(const float* in, const float* w, float* out, int rows, int cols, float eps);
/* lib/kernel_templates_llama.pl:600-830 (binary elementwise; silu = x / (1 + expf(-x)), :668) */
void gpu_add(const float* a, const float* b, float* out, int n);
void gpu_mul(const float* a, const float* b, float* out, int n);
void gpu_silu(const float* in, float* out, int n);
/* lib/kernel_templates_llama.pl:1104-1290, lib/kernel_templates_blas.pl:2146-2153  C[M][N] = A[M][K] @ B[K][N] */
void gpu_matmul(const float* A, const float* B, float* C, int M, int N, int K);
void gpu_matmul_opt(const float* A, const float* B, float* C, int M, int N, int K);

/* ---- Q8_0 Llama forward (bench/bpd_cpu.c:5537-5798: bpd_llama_config, bpd_llama_layer_weights,
 * bpd_llama_weights, bpd_llama_block_cpu, bpd_llama_forward_cpu).  Same structs (host memory, field
 * for field), same argument order; every pointer inside them and every array argument is DEVICE
 * memory; the KV caches are [n_layers][max_seq_len][n_kv_heads*head_dim] f16 (kv_cache_f16 = 1) or f32
 * and must be zero where nothing has been written (all max_seq_len rows take part in the softmax,
 * masked, as in the reference).  token_out may be NULL.  Asynchronous on `stream`; 0 or a status.
 * Indices that come from device memory are checked on the device: a token id outside [0, vocab_size) is not looked
 * up and a position outside [0, max_seq_len) is not stored (the embedding row / cache row is left untouched), and
 * bpdq_last_status() then reports -4.  Attention takes query t to sit at position kv_pos + t: pos_ids must be
 * kv_pos, kv_pos + 1, ... (as the reference's callers pass them); the rotary embedding uses pos_ids itself. */
typedef struct {
    int n_layers, n_heads, n_kv_heads, head_dim, embed_dim, ffn_dim, vocab_size, max_seq_len;
    float rms_eps, rope_base;
    int rope_dim, kv_cache_f16;
} bpd_llama_config;
typedef struct {
    const float* attn_norm_w;
    const uint8_t *w_q, *w_k, *w_v, *w_o;
    const float* ffn_norm_w;
    const uint8_t *w_gate, *w_up, *w_down;
} bpd_llama_layer_weights;
typedef struct {
    const uint8_t* token_embd;
    const bpd_llama_layer_weights* layers;   /* HOST array of n_layers descriptors */
    const float* output_norm_w;
    const uint8_t* output_w;
    const float* rope_freqs;                 /* [rope_dim/2] or NULL */
} bpd_llama_weights;
/* the steps on device pointers, as the reference's _cpu entries (bench/bpd_cpu.c:4959, 5146, 5240, 5204,
 * 5370, 5504, 4512) plus the stream; bpd_gqa_attn_cuda reads f16 caches directly when kv_is_f16 (the
 * reference widens them to fp32 copies first); bpd_argmax_dim_cuda supports inner = 1 */
int bpd_rmsnorm_llama_cuda(const float* input, const float* weight, float* output, int n_rows, int row_len, float eps,
                           void* stream);
int bpd_rope_norm_freqs_cuda(const float* input, float* output, const int32_t* pos_ids, const float* freq_factors,
                             int n_tokens, int n_heads, int head_dim, int n_dims, float freq_base, void* stream);
int bpd_kv_cache_write_f16_cuda(uint16_t* cache, const float* src, const int32_t* pos_ids, int n_tokens, int n_kv_heads,
                                int head_dim, int max_seq_len, void* stream);
int bpd_kv_cache_write_cuda(float* cache, const float* src, const int32_t* pos_ids, int n_tokens, int n_kv_heads, int head_dim,
                            int max_seq_len, void* stream);
int bpd_gqa_attn_cuda(const float* q, const void* k, const void* v, float* dst, int n_q_tokens, int n_kv, int n_q_heads,
                      int n_kv_heads, int head_dim, float scale, int kv_offset, int kv_is_f16, void* stream);
int bpd_swiglu_fuse_cuda(const float* gate, const float* up, float* dst, int n, void* stream);
int bpd_argmax_dim_cuda(const float* x, long long* out, int outer, int dim_size, int inner, void* stream);
int bpd_llama_block_cuda(float* x, const bpd_llama_layer_weights* lw, const bpd_llama_config* cfg, const int32_t* pos_ids,
                         int n_tokens, int kv_pos, void* k_cache, void* v_cache, float* scratch1, float* scratch2,
                         float* scratch3, const float* rope_freqs, void* stream);
int bpd_llama_forward_cuda(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights,
                           const bpd_llama_config* cfg, const int32_t* pos_ids, int kv_pos, void* k_cache, void* v_cache,
                           float* logits_out, long long* token_out, void* stream);
/* The same forward with a second set of weights: `tiles` has the layout of `weights`, its Q8_0 matrix
 * pointers (w_q .. w_down of every layer, output_w) refer to copies re-tiled by bpd_repack_q8_0_tiles_cuda, or
 * are NULL; its other fields are not read.  With three or more tokens (a prefill) every product that has a
 * re-tiled copy runs once over the weights on the tensor cores (bpd_qmatmul_q8_0_tiles_cuda) instead of once
 * per token; single tokens use the rows as before.  tiles == NULL is bpd_llama_forward_cuda. */
int bpd_llama_forward_tiles_cuda(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights,
                                 const bpd_llama_weights* tiles, const bpd_llama_config* cfg, const int32_t* pos_ids,
                                 int kv_pos, void* k_cache, void* v_cache, float* logits_out, long long* token_out,
                                 void* stream);

/* the forward with caller-owned scratch (see "scratch memory" above); tiles may be NULL */
size_t bpdq_llama_forward_workspace_bytes(const bpd_llama_config* cfg, int n_tokens);
int bpd_llama_forward_ws_cuda(const int32_t* token_ids, int n_tokens, const bpd_llama_weights* weights,
                              const bpd_llama_weights* tiles, const bpd_llama_config* cfg, const int32_t* pos_ids, int kv_pos,
                              void* k_cache, void* v_cache, float* logits_out, long long* token_out, void* workspace,
                              size_t workspace_bytes, void* stream);

/* ---- row-sharded products on several GPUs without a collective.
 * The reference's decode loop runs on one GPU; with the rows of every matrix sharded over ranks (one
 * process per GPU) each rank needs the other ranks' output slices.  Instead of an all-gather after the
 * products, the batched product kernel stores each result, besides its own output, into every rank's
 * gathered buffer (peer memory mapped through CUDA IPC), and a flag per rank and step replaces the
 * collective's rendezvous.
 *   bpdq_ipc_export / bpdq_ipc_import / bpdq_ipc_close: cudaIpcGetMemHandle / cudaIpcOpenMemHandle (with lazy
 *     peer access) / cudaIpcCloseMemHandle on a bpdq_alloc allocation; the handle is 64 bytes.
 *   bpdq_set_peer_outputs: for this device, every batched Q4_K product (bpd_qmatmul_q4k_q8k_batch*_cuda,
 *     C-ABI nibble order, no accumulate) whose outputs all lie in [local_base, local_base + bytes) also
 *     stores result i to targets[t] + (address of result i - local_base) for t < n_targets (<= 8; 16-byte
 *     aligned; a rank's own gathered buffer is one of the targets).  n_targets = 0 clears.  Read when a launch
 *     is planned, so set it before the launches are made or captured into a graph.
 *   bpdq_peer_signal: after all earlier work of the stream, writes `value` to each of the n slots (this rank's
 *     flag in each rank's flag array).  bpdq_peer_wait: returns when the n flags at local_flags have all
 *     reached `value` (flags only grow); gives up after about a second and latches status -4. */
int bpdq_ipc_export(const void* dev_ptr, void* handle64);
void* bpdq_ipc_import(const void* handle64);
int bpdq_ipc_close(void* imported);
int bpdq_set_peer_outputs(const void* local_base, size_t bytes, int n_targets, void* const* targets);
int bpdq_peer_signal(unsigned* const* slots, int n, unsigned value, void* stream);
int bpdq_peer_wait(const unsigned* local_flags, int n, unsigned value, void* stream);
/* both in one launch (slot i belongs to the rank whose flag is local_flags[i]) */
int bpdq_peer_signal_wait(unsigned* const* slots, const unsigned* local_flags, int n, unsigned value, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BPDQ_H */

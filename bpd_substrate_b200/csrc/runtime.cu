// Host-side runtime of the C-ABI library: stream selection, status latch, device memory
// helpers.  This is the Python-facing replacement for the reference's SWI-Prolog launch shim
// (lib/cuda_launch.c:39-307): the same duties (context, alloc/free, H2D/D2H, sync, launch)
// behind plain C symbols that ctypes can bind.
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

#include <atomic>
#include <mutex>
#include <vector>

namespace bpdq {

static std::atomic<cudaStream_t> g_stream{nullptr};
static std::atomic<int> g_status{0};
static Tuning g_tuning = {8192, 2, 1, 16, 1, 1, 32};

__device__ int g_dev_error = 0;

cudaStream_t current_stream() { return g_stream.load(std::memory_order_relaxed); }

int latch(int status)
{
    if (status != 0) {
        int expected = 0;
        g_status.compare_exchange_strong(expected, status);
    }
    return status;
}

int check_cuda(cudaError_t e)
{
    if (e == cudaSuccess) return 0;
    return latch(BPDQ_ERR_CUDA - (int)e);
}

int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int* device_error_flag()
{
    static int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dev_error) != cudaSuccess) return nullptr;
        cached[dev] = (int*)p;
    }
    return cached[dev];
}

Tuning& tuning() { return g_tuning; }

// ---- library-owned scratch: one block per (device, stream, purpose), grown by replacement
namespace {
struct ScratchBlock {
    int dev, kind;
    cudaStream_t stream;
    uint8_t* ptr;
    size_t cap;
};
std::mutex g_scratch_mutex;
std::vector<ScratchBlock> g_scratch;     // live blocks
std::vector<void*> g_scratch_retired;    // replaced blocks: kept allocated, earlier launches and graphs may use them
}  // namespace

uint8_t* scratch_take(Workspace* ws, int kind, size_t bytes, cudaStream_t s, int* status)
{
    *status = 0;
    if (bytes == 0) bytes = 16;
    if (ws) {
        const size_t at = (ws->used + 255) / 256 * 256;
        const size_t pad = (256 - ((uintptr_t)ws->base & 255)) & 255;   // the carved pieces are 256-byte aligned
        if (!ws->base || at + pad + bytes > ws->bytes) {
            *status = latch(BPDQ_ERR_RANGE);
            return nullptr;
        }
        ws->used = at + bytes;
        return ws->base + pad + at;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *status = check_cuda(e);
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    ScratchBlock* blk = nullptr;
    for (auto& b : g_scratch)
        if (b.dev == dev && b.kind == kind && b.stream == s) { blk = &b; break; }
    if (blk && blk->cap >= bytes) return blk->ptr;
    // a new or larger block is an allocation: not while the stream records a graph
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) (void)cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone) {
        *status = latch(BPDQ_ERR_CAPTURE);
        return nullptr;
    }
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    if (blk && want < 2 * blk->cap) want = 2 * blk->cap;
    void* p = nullptr;
    e = cudaMalloc(&p, want);
    if (e != cudaSuccess && want > bytes) e = cudaMalloc(&p, want = bytes);
    if (e != cudaSuccess) {
        *status = check_cuda(e);
        return nullptr;
    }
    if (blk) {
        g_scratch_retired.push_back(blk->ptr);
        blk->ptr = (uint8_t*)p;
        blk->cap = want;
    } else {
        g_scratch.push_back({dev, kind, s, (uint8_t*)p, want});
    }
    return (uint8_t*)p;
}

static void* dev_alloc(size_t bytes)
{
    void* p = nullptr;
    if (check_cuda(cudaMalloc(&p, bytes ? bytes : 1)) != 0) return nullptr;
    return p;
}
static void dev_free(void* p) { check_cuda(cudaFree(p)); }
static void copy_sync(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind)
{
    // Ordered after work queued on the library's stream, then blocking like the reference's
    // cudaMemcpy helpers (bench/bpd_quant_gpu.cu:172-175).
    cudaStream_t s = current_stream();
    if (check_cuda(cudaMemcpyAsync(dst, src, bytes, kind, s)) != 0) return;
    check_cuda(cudaStreamSynchronize(s));
}
static void sync_all() { check_cuda(cudaDeviceSynchronize()); }

}  // namespace bpdq

using namespace bpdq;

extern "C" {

// ---- library state ---------------------------------------------------------------------
void bpdq_set_stream(void* stream) { g_stream.store((cudaStream_t)stream); }
void* bpdq_get_stream(void) { return (void*)current_stream(); }

int bpdq_last_status(void)
{
    // Folds in the device-side error word (set when a kernel gave up on a bounded wait).
    int* flag = device_error_flag();
    int dev_err = 0;
    if (flag && cudaMemcpy(&dev_err, flag, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && dev_err != 0)
        latch(BPDQ_ERR_DEVICE);
    return g_status.load();
}
int bpdq_device_error_word(void)
{
    int* flag = device_error_flag();
    int dev_err = 0;
    if (flag) cudaMemcpy(&dev_err, flag, sizeof(int), cudaMemcpyDeviceToHost);
    return dev_err;
}
void bpdq_clear_status(void)
{
    g_status.store(0);
    int* flag = device_error_flag();
    if (flag) cudaMemset(flag, 0, sizeof(int));
    (void)cudaGetLastError();
}
void bpdq_set_tuning(int tile_bytes, int stages, int ctas_per_sm, int warps, int pdl)
{
    Tuning& t = tuning();
    if (tile_bytes > 0) t.tile_bytes = tile_bytes;
    if (stages > 0) t.stages = stages;
    if (ctas_per_sm > 0) t.ctas_per_sm = ctas_per_sm;
    if (warps > 0) t.warps = warps;
    if (pdl >= 0) t.pdl = pdl;
}
void bpdq_set_dequant_tuning(int variant, int ctas_per_sm)
{
    if (variant == 0 || variant == 1) tuning().dequant_variant = variant;
    if (ctas_per_sm > 0) tuning().dequant_ctas = ctas_per_sm;
}
int bpdq_sm_count(void) { return sm_count(); }

void* bpdq_alloc(size_t bytes) { return dev_alloc(bytes); }
void bpdq_free(void* p) { dev_free(p); }
void bpdq_h2d(void* dev, const void* host, size_t bytes) { copy_sync(dev, host, bytes, cudaMemcpyHostToDevice); }
void bpdq_d2h(void* host, const void* dev, size_t bytes) { copy_sync(host, dev, bytes, cudaMemcpyDeviceToHost); }
void bpdq_d2d(void* dst, const void* src, size_t bytes) { copy_sync(dst, src, bytes, cudaMemcpyDeviceToDevice); }
int bpdq_h2d_async(void* dev, const void* host, size_t bytes, void* stream)
{
    return check_cuda(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
}
int bpdq_d2h_async(void* host, const void* dev, size_t bytes, void* stream)
{
    return check_cuda(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
}
void* bpdq_host_alloc(size_t bytes)
{
    void* p = nullptr;
    if (check_cuda(cudaMallocHost(&p, bytes ? bytes : 1)) != 0) return nullptr;
    return p;
}
void bpdq_host_free(void* p) { check_cuda(cudaFreeHost(p)); }
void bpdq_sync(void) { sync_all(); }
int bpdq_stream_sync(void* stream) { return check_cuda(cudaStreamSynchronize((cudaStream_t)stream)); }

// ---- events, memset, CUDA graphs (additive) -----------------------------------------------
void* bpdq_event_create(void)
{
    cudaEvent_t e = nullptr;
    if (check_cuda(cudaEventCreate(&e)) != 0) return nullptr;
    return (void*)e;
}
void bpdq_event_destroy(void* ev) { if (ev) check_cuda(cudaEventDestroy((cudaEvent_t)ev)); }
int bpdq_event_record(void* ev, void* stream) { return check_cuda(cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)stream)); }
// Waits for `stop`, then returns the milliseconds between the two events (negative on error).
float bpdq_event_elapsed_ms(void* start, void* stop)
{
    if (check_cuda(cudaEventSynchronize((cudaEvent_t)stop)) != 0) return -1.0f;
    float ms = -1.0f;
    if (check_cuda(cudaEventElapsedTime(&ms, (cudaEvent_t)start, (cudaEvent_t)stop)) != 0) return -1.0f;
    return ms;
}
int bpdq_memset_async(void* dev, int value, size_t bytes, void* stream)
{
    return check_cuda(cudaMemsetAsync(dev, value, bytes, (cudaStream_t)stream));
}
void* bpdq_stream_create(void)
{
    cudaStream_t s = nullptr;
    if (check_cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking)) != 0) return nullptr;
    return (void*)s;
}
void bpdq_stream_destroy(void* s) { if (s) check_cuda(cudaStreamDestroy((cudaStream_t)s)); }
// Work queued on `stream` after this call waits for the work that `ev` was recorded behind.
int bpdq_stream_wait_event(void* stream, void* ev)
{
    return check_cuda(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0));
}

// Capture everything launched on `stream` between begin and end into an executable graph.
int bpdq_graph_begin(void* stream)
{
    return check_cuda(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
}
void* bpdq_graph_end(void* stream)
{
    cudaGraph_t g = nullptr;
    if (check_cuda(cudaStreamEndCapture((cudaStream_t)stream, &g)) != 0 || !g) return nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = check_cuda(cudaGraphInstantiate(&exec, g, 0));
    cudaGraphDestroy(g);
    return rc == 0 ? (void*)exec : nullptr;
}
int bpdq_graph_launch(void* exec, void* stream)
{
    return check_cuda(cudaGraphLaunch((cudaGraphExec_t)exec, (cudaStream_t)stream));
}
void bpdq_graph_destroy(void* exec) { if (exec) check_cuda(cudaGraphExecDestroy((cudaGraphExec_t)exec)); }
int bpdq_set_device(int dev) { return check_cuda(cudaSetDevice(dev)); }
// Free and total device memory of the current device as the driver reports them.
int bpdq_mem_info(size_t* free_bytes, size_t* total_bytes)
{
    size_t f = 0, t = 0;
    int rc = check_cuda(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return rc;
}
int bpdq_l2_bytes(void)
{
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrL2CacheSize, dev) != cudaSuccess) return 0;
    return n;
}

// ---- the reference's memory helpers, name for name ----------------------------------------
// bench/bpd_quant_gpu.cu:172-176
void* qgpu_alloc(int bytes) { return bytes < 0 ? (latch(BPDQ_ERR_ARG), nullptr) : dev_alloc((size_t)bytes); }
void qgpu_free(void* p) { dev_free(p); }
void qgpu_h2d(void* d, const void* s, int bytes) { if (bytes >= 0) copy_sync(d, s, (size_t)bytes, cudaMemcpyHostToDevice); else latch(BPDQ_ERR_ARG); }
void qgpu_d2h(void* d, const void* s, int bytes) { if (bytes >= 0) copy_sync(d, s, (size_t)bytes, cudaMemcpyDeviceToHost); else latch(BPDQ_ERR_ARG); }
void qgpu_sync(void) { sync_all(); }
// bench/bpd_quant_gpu_sweep.cu:145-149
void* sgpu_alloc(int bytes) { return qgpu_alloc(bytes); }
void sgpu_free(void* p) { dev_free(p); }
void sgpu_h2d(void* d, const void* s, int bytes) { qgpu_h2d(d, s, bytes); }
void sgpu_d2h(void* d, const void* s, int bytes) { qgpu_d2h(d, s, bytes); }
void sgpu_sync(void) { sync_all(); }
// bench/bench_dequant_gpu_h2h.cu:77-81
void* galloc(int b) { return qgpu_alloc(b); }
void gfree(void* p) { dev_free(p); }
void gh2d(void* d, const void* s, int b) { qgpu_h2d(d, s, b); }
void gd2h(void* d, const void* s, int b) { qgpu_d2h(d, s, b); }
void gsync(void) { sync_all(); }
// generators/generate_llama_kernels.pl:32-60
void* gpu_alloc(int bytes) { return qgpu_alloc(bytes); }
void gpu_free(void* p) { dev_free(p); }
void gpu_copy_h2d(void* d, const void* h, int b) { qgpu_h2d(d, h, b); }
void gpu_copy_d2h(void* h, const void* d, int b) { qgpu_d2h(h, d, b); }
void gpu_copy_d2d(void* dst, const void* src, int b) { if (b >= 0) copy_sync(dst, src, (size_t)b, cudaMemcpyDeviceToDevice); else latch(BPDQ_ERR_ARG); }
void gpu_sync(void) { sync_all(); }

}  // extern "C"

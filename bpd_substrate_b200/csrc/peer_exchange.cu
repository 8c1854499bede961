// Row-sharded products over several GPUs without a collective: every rank's product kernels store
// each result, next to their own output, straight into the gathered buffer of every rank (peer
// memory over NVLink, mapped through CUDA IPC), so the exchange rides on the products' epilogue.
// What is left of the all-gather is one flag per rank and step: a rank raises its flag in every
// peer's memory after its last product of the step, and waits (bounded) for all flags in its own.
//
// This file holds the plumbing: IPC export / import of an allocation, the per-device table of store
// targets that the batched product's planner reads, and the two flag kernels.  The stores themselves
// are in batch_tile (gemv_q4k_device.cuh).
#include "bpdq_common.cuh"
#include "../../include/bpdq.h"

namespace bpdq {

struct PeerTable {
    const char* base;
    size_t bytes;
    int n;
    const char* target[kMaxPeerTargets];
};
static PeerTable g_peer_table[64];

static PeerTable* table_of_current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return &g_peer_table[dev];
}

// The targets for a launch whose outputs span [lo, hi): all of it must lie inside the registered range.
bool peer_targets_for(const void* lo, const void* hi, PeerTargets& t)
{
    t.n = 0;
    const PeerTable* tab = table_of_current_device();
    if (!tab || tab->n == 0) return false;
    const char *a = (const char*)lo, *b = (const char*)hi;
    if (a < tab->base || b > tab->base + tab->bytes || a > b) return false;
    t.n = tab->n;
    for (int i = 0; i < tab->n; i++) t.shift[i] = (long long)(tab->target[i] - tab->base);
    return true;
}

// Raise this rank's flag in every peer's flag array: all earlier work of the stream (the products and
// their peer stores) has completed before this launch starts; the fence orders the flag behind it at
// system scope.
__global__ void k_peer_signal(PeerFlagSlots slots, unsigned value)
{
    __threadfence_system();
    const int i = threadIdx.x;
    if (i < slots.n) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(slots.slot[i]), "r"(value) : "memory");
    }
}

// Wait until every flag has reached `value` (flags only grow).  Bounded: about a second of polling,
// then the launch records an error and returns, so a missing rank cannot hang the device.
__global__ void k_peer_wait(const unsigned* flags, int n, unsigned value, int* err)
{
    const int i = threadIdx.x;
    if (i >= n) return;
    for (unsigned poll = 0; poll < (1u << 22); poll++) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
        if ((int)(v - value) >= 0) return;
        __nanosleep(200);
    }
    if (err) atomicCAS(err, 0, 51);
}

// Both in one launch: thread i raises this rank's flag at rank i, then waits for rank i's flag here.
__global__ void k_peer_signal_wait(PeerFlagSlots slots, const unsigned* flags, unsigned value, int* err)
{
    __threadfence_system();
    const int i = threadIdx.x;
    if (i >= slots.n) return;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(slots.slot[i]), "r"(value) : "memory");
    for (unsigned poll = 0; poll < (1u << 22); poll++) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
        if ((int)(v - value) >= 0) return;
        __nanosleep(200);
    }
    if (err) atomicCAS(err, 0, 51);
}

}  // namespace bpdq

using namespace bpdq;

extern "C" {

int bpdq_ipc_export(const void* dev_ptr, void* handle64)
{
    if (!dev_ptr || !handle64) return latch(BPDQ_ERR_ARG);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    int rc = check_cuda(cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr)));
    if (rc) return latch(rc);
    memcpy(handle64, &h, 64);
    return 0;
}

void* bpdq_ipc_import(const void* handle64)
{
    if (!handle64) { latch(BPDQ_ERR_ARG); return nullptr; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (check_cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess)) != 0) { latch(BPDQ_ERR_CUDA); return nullptr; }
    return p;
}

int bpdq_ipc_close(void* imported)
{
    if (!imported) return 0;
    return check_cuda(cudaIpcCloseMemHandle(imported));
}

int bpdq_set_peer_outputs(const void* local_base, size_t bytes, int n_targets, void* const* targets)
{
    PeerTable* tab = table_of_current_device();
    if (!tab) return latch(BPDQ_ERR_CUDA);
    if (n_targets == 0 || !local_base) { tab->n = 0; return 0; }
    if (n_targets < 0 || n_targets > kMaxPeerTargets || !targets || bytes == 0) return latch(BPDQ_ERR_ARG);
    if ((uintptr_t)local_base & 15) return latch(BPDQ_ERR_ALIGN);
    for (int i = 0; i < n_targets; i++)
        if (!targets[i] || ((uintptr_t)targets[i] & 15)) return latch(BPDQ_ERR_ALIGN);
    tab->base = (const char*)local_base;
    tab->bytes = bytes;
    for (int i = 0; i < n_targets; i++) tab->target[i] = (const char*)targets[i];
    tab->n = n_targets;
    return 0;
}

int bpdq_peer_signal(unsigned* const* slots, int n, unsigned value, void* stream)
{
    if (n < 0 || n > kMaxPeerTargets || (n > 0 && !slots)) return latch(BPDQ_ERR_ARG);
    if (n == 0) return 0;
    PeerFlagSlots s;
    s.n = n;
    for (int i = 0; i < n; i++) {
        if (!slots[i] || ((uintptr_t)slots[i] & 3)) return latch(BPDQ_ERR_ALIGN);
        s.slot[i] = slots[i];
    }
    k_peer_signal<<<1, 32, 0, (cudaStream_t)stream>>>(s, value);
    return check_cuda(cudaGetLastError());
}

int bpdq_peer_signal_wait(unsigned* const* slots, const unsigned* local_flags, int n, unsigned value, void* stream)
{
    if (n < 0 || n > kMaxPeerTargets || (n > 0 && (!slots || !local_flags))) return latch(BPDQ_ERR_ARG);
    if (n == 0) return 0;
    PeerFlagSlots s;
    s.n = n;
    for (int i = 0; i < n; i++) {
        if (!slots[i] || ((uintptr_t)slots[i] & 3)) return latch(BPDQ_ERR_ALIGN);
        s.slot[i] = slots[i];
    }
    k_peer_signal_wait<<<1, 32, 0, (cudaStream_t)stream>>>(s, local_flags, value, device_error_flag());
    return check_cuda(cudaGetLastError());
}

int bpdq_peer_wait(const unsigned* local_flags, int n, unsigned value, void* stream)
{
    if (n < 0 || n > 32 || (n > 0 && !local_flags)) return latch(BPDQ_ERR_ARG);
    if (n == 0) return 0;
    k_peer_wait<<<1, 32, 0, (cudaStream_t)stream>>>(local_flags, n, value, device_error_flag());
    return check_cuda(cudaGetLastError());
}

}  // extern "C"

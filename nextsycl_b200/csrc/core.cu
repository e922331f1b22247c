// core.cu: devices, memory, copies and tickets of the C ABI (include/ns.h) on the CUDA runtime.
// Behaviour follows the reference's kernels/ns/ns.cpp call by call (cited per function); the mechanism is CUDA's:
// streams for queues, events for tickets, peer copies over NVLink for ns_copy_peer.
#include "ns_internal.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {
thread_local std::string g_err;

// A ticket names one of the last NS_RING events; an older one's slot has been reused by a newer mark, so it is refused
// rather than silently standing for that newer event.
bool ticket_live(const ns_gpu* g, int64_t ticket) { return ticket >= 0 && ticket < g->next_ticket && ticket >= g->next_ticket - NS_RING; }

cudaEvent_t ticket_event(ns_gpu* g, int64_t ticket) {
    // caller holds g->mu
    if (g->ring.empty()) g->ring.assign((size_t) NS_RING, nullptr);
    cudaEvent_t& e = g->ring[(size_t) (ticket % NS_RING)];
    if (!e) cudaEventCreate(&e);
    return e;
}
}  // namespace

int ns_fail(const std::string& what) {
    g_err = what;
    return -1;
}

int ns_cuda(cudaError_t e, const char* where) {
    return ns_fail(std::string(where) + ": cuda: " + cudaGetErrorString(e));
}

int ns_enter(ns_gpu* g, const char* where) {
    if (!g) return ns_fail(std::string(where) + ": no gpu");
    NS_CUDA(cudaSetDevice(g->dev), where);
    return 0;
}

int ns_launched(const char* where) {
    NS_CUDA(cudaGetLastError(), where);
    return 0;
}

int ns_kept(ns_gpu* g, size_t bytes, void** out) {
    std::lock_guard<std::mutex> lk(g->mu);
    if (g->kept_bytes < bytes) {
        if (g->kept) {
            NS_CUDA(cudaStreamSynchronize(g->compute), "ns_kept");
            cudaFree(g->kept);
            g->kept = nullptr;
            g->kept_bytes = 0;
        }
        const size_t want = (bytes + (size_t) (1 << 20) - 1) / (1 << 20) * (1 << 20);
        if (cudaMalloc(&g->kept, want) != cudaSuccess) {
            cudaGetLastError();
            return ns_fail("device allocation of " + std::to_string(want) + " bytes failed");
        }
        g->kept_bytes = want;
    }
    *out = g->kept;
    return 0;
}

int ns_kept_kv(ns_gpu* g, size_t bytes, void** out) {
    std::lock_guard<std::mutex> lk(g->mu);
    if (g->kept_kv_bytes < bytes) {
        if (g->kept_kv) {
            NS_CUDA(cudaStreamSynchronize(g->compute), "ns_kept_kv");
            cudaFree(g->kept_kv);
            g->kept_kv = nullptr;
            g->kept_kv_bytes = 0;
        }
        const size_t want = (bytes + (size_t) (1 << 20) - 1) / (1 << 20) * (1 << 20);
        if (cudaMalloc(&g->kept_kv, want) != cudaSuccess) {
            cudaGetLastError();
            return ns_fail("device allocation of " + std::to_string(want) + " bytes failed");
        }
        g->kept_kv_bytes = want;
    }
    *out = g->kept_kv;
    return 0;
}

extern "C" {

const char* ns_last_error(void) { return g_err.c_str(); }
const char* ns_version(void) { return "nextsycl-b200 0.1 (cuda, sm_100a)"; }

// kernels/ns/ns.cpp:41-77
int ns_gpu_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int ns_gpu_name(int index, char* buf, size_t len) {
    cudaDeviceProp p;
    NS_CUDA(cudaGetDeviceProperties(&p, index), "ns_gpu_name");
    if (!buf || len == 0) return ns_fail("ns_gpu_name: no buffer");
    snprintf(buf, len, "%s", p.name);
    return 0;
}

int ns_gpu_pci(int index, char* buf, size_t len) {
    if (!buf || len == 0) return ns_fail("ns_gpu_pci: no buffer");
    char id[32] = {0};
    NS_CUDA(cudaDeviceGetPCIBusId(id, (int) sizeof(id), index), "ns_gpu_pci");
    snprintf(buf, len, "%s", id);
    return 0;
}

int ns_gpu_units(int index, int* units, int* mhz) {
    int sms = 0, khz = 0;
    NS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, index), "ns_gpu_units");
    NS_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, index), "ns_gpu_units");
    if (units) *units = sms;
    if (mhz) *mhz = khz / 1000;
    return 0;
}

// kernels/ns/ns.cpp:79-94: the compute queue and the two copy lanes
int ns_gpu_open(int index, ns_gpu** out) {
    NS_TRY
    if (!out) return ns_fail("ns_gpu_open: no out");
    int n = ns_gpu_count();
    if (index < 0 || index >= n) return ns_fail("ns_gpu_open: no GPU " + std::to_string(index) + " (" + std::to_string(n) + " found)");
    NS_CUDA(cudaSetDevice(index), "ns_gpu_open");
    ns_gpu* g = new ns_gpu();
    g->dev = index;
    cudaDeviceGetAttribute(&g->sms, cudaDevAttrMultiProcessorCount, index);
    cudaError_t e = cudaStreamCreateWithFlags(&g->compute, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g->lane[0], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g->lane[1], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaHostAlloc((void**) &g->status_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
    if (e == cudaSuccess) {
        *g->status_host = 0;
        e = cudaHostGetDevicePointer((void**) &g->status_dev, g->status_host, 0);
    }
    if (e == cudaSuccess) e = cudaMalloc((void**) &g->dec_sync, 2 * NS_DEC_SYNC_SLOTS * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(g->dec_sync, 0, 2 * NS_DEC_SYNC_SLOTS * sizeof(unsigned int));
    if (e != cudaSuccess) {
        delete g;
        return ns_cuda(e, "ns_gpu_open");
    }
    *out = g;
    return 0;
    NS_CATCH("ns_gpu_open")
}

// kernels/ns/ns.cpp:96-100: waits for all three queues
void ns_gpu_close(ns_gpu* g) {
    if (!g) return;
    cudaSetDevice(g->dev);
    cudaStreamSynchronize(g->compute);
    cudaStreamSynchronize(g->lane[0]);
    cudaStreamSynchronize(g->lane[1]);
    for (cudaEvent_t e : g->ring)
        if (e) cudaEventDestroy(e);
    if (g->kept) cudaFree(g->kept);
    if (g->kept_kv) cudaFree(g->kept_kv);
    if (g->dec_sync) cudaFree(g->dec_sync);
    if (g->status_host) cudaFreeHost(g->status_host);
    cudaStreamDestroy(g->compute);
    cudaStreamDestroy(g->lane[0]);
    cudaStreamDestroy(g->lane[1]);
    cudaGetLastError();
    delete g;
}

void* ns_gpu_queue(ns_gpu* g) { return g ? (void*) &g->compute : nullptr; }

// kernels/ns/ns.cpp:104-113
int ns_gpu_memory(ns_gpu* g, uint64_t* total, int64_t* free_bytes) {
    if (ns_enter(g, "ns_gpu_memory")) return -1;
    size_t f = 0, t = 0;
    NS_CUDA(cudaMemGetInfo(&f, &t), "ns_gpu_memory");
    if (total) *total = (uint64_t) t;
    if (free_bytes) *free_bytes = (int64_t) f;
    return 0;
}

// kernels/ns/ns.cpp:115-128
int ns_alloc(ns_gpu* g, size_t bytes, void** out) {
    if (ns_enter(g, "ns_alloc")) return -1;
    if (!out) return ns_fail("ns_alloc: no out");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess || !p) {
        cudaGetLastError();
        return ns_fail("device allocation of " + std::to_string(bytes) + " bytes failed");
    }
    *out = p;
    return 0;
}

int ns_free(ns_gpu* g, void* p) {
    if (ns_enter(g, "ns_free")) return -1;
    if (p) NS_CUDA(cudaFree(p), "ns_free");
    return 0;
}

// kernels/ns/ns.cpp:130-138: pinned and readable from the device in place
int ns_alloc_host(ns_gpu* g, size_t bytes, void** out) {
    if (ns_enter(g, "ns_alloc_host")) return -1;
    if (!out) return ns_fail("ns_alloc_host: no out");
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess || !p) {
        cudaGetLastError();
        return ns_fail("host allocation of " + std::to_string(bytes) + " bytes failed");
    }
    *out = p;
    return 0;
}

int ns_free_host(ns_gpu* g, void* p) {
    if (ns_enter(g, "ns_free_host")) return -1;
    if (p) NS_CUDA(cudaFreeHost(p), "ns_free_host");
    return 0;
}

// kernels/ns/ns.cpp:140-159
int ns_copy_to(ns_gpu* g, void* dst, const void* src_host, size_t bytes) {
    if (ns_enter(g, "ns_copy_to")) return -1;
    if (bytes) NS_CUDA(cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, g->compute), "ns_copy_to");
    return 0;
}

int ns_copy_from(ns_gpu* g, void* dst_host, const void* src, size_t bytes) {
    if (ns_enter(g, "ns_copy_from")) return -1;
    if (bytes) NS_CUDA(cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, g->compute), "ns_copy_from");
    return 0;
}

int ns_copy_dev(ns_gpu* g, void* dst, const void* src, size_t bytes) {
    if (ns_enter(g, "ns_copy_dev")) return -1;
    if (bytes) NS_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, g->compute), "ns_copy_dev");
    return 0;
}

// kernels/ns/ns.cpp:161-174
int ns_copy_2d(ns_gpu* g, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t height) {
    if (ns_enter(g, "ns_copy_2d")) return -1;
    if (width && height)
        NS_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, height, cudaMemcpyDeviceToDevice, g->compute), "ns_copy_2d");
    return 0;
}

// kernels/ns/ns.cpp:185-190
int ns_mark(ns_gpu* g, int64_t* ticket) {
    if (ns_enter(g, "ns_mark")) return -1;
    if (!ticket) return ns_fail("ns_mark: no ticket");
    std::lock_guard<std::mutex> lk(g->mu);
    const int64_t t = g->next_ticket++;
    NS_CUDA(cudaEventRecord(ticket_event(g, t), g->compute), "ns_mark");
    *ticket = t;
    return 0;
}

// kernels/ns/ns.cpp:193-201
int ns_stream_copy(ns_gpu* g, void* dst, const void* src, size_t bytes, const int64_t* after, int ndeps, int lane, int64_t* ticket) {
    if (ns_enter(g, "ns_stream_copy")) return -1;
    if (lane < 0 || lane > 1) return ns_fail("ns_stream_copy: lane 0 or 1");
    std::lock_guard<std::mutex> lk(g->mu);
    cudaStream_t s = g->lane[lane];
    for (int i = 0; i < ndeps; ++i) {
        if (!ticket_live(g, after[i])) return ns_fail("ns_stream_copy: no such ticket (or older than the last 65,536 marks)");
        NS_CUDA(cudaStreamWaitEvent(s, ticket_event(g, after[i]), 0), "ns_stream_copy");
    }
    if (bytes) NS_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, s), "ns_stream_copy");
    const int64_t t = g->next_ticket++;
    NS_CUDA(cudaEventRecord(ticket_event(g, t), s), "ns_stream_copy");
    if (ticket) *ticket = t;
    return 0;
}

// kernels/ns/ns.cpp:223-228: the wait happens on the device, the host does not block
int ns_await(ns_gpu* g, int64_t ticket) {
    if (ns_enter(g, "ns_await")) return -1;
    std::lock_guard<std::mutex> lk(g->mu);
    if (!ticket_live(g, ticket)) return ns_fail("ns_await: no such ticket (or older than the last 65,536 marks)");
    NS_CUDA(cudaStreamWaitEvent(g->compute, ticket_event(g, ticket), 0), "ns_await");
    return 0;
}

// kernels/ns/ns.cpp:204-220
int ns_stamp(ns_gpu* g, int64_t* ticket) { return ns_mark(g, ticket); }

int ns_elapsed(ns_gpu* g, int64_t t0, int64_t t1, double* ns) {
    if (ns_enter(g, "ns_elapsed")) return -1;
    if (!ns) return ns_fail("ns_elapsed: no out");
    cudaEvent_t a, b;
    {
        std::lock_guard<std::mutex> lk(g->mu);
        if (!ticket_live(g, t0) || !ticket_live(g, t1)) return ns_fail("ns_elapsed: no such ticket (or older than the last 65,536 marks)");
        a = ticket_event(g, t0);
        b = ticket_event(g, t1);
    }
    NS_CUDA(cudaEventSynchronize(a), "ns_elapsed");
    NS_CUDA(cudaEventSynchronize(b), "ns_elapsed");
    float ms = 0.f;
    NS_CUDA(cudaEventElapsedTime(&ms, a, b), "ns_elapsed");
    *ns = (double) ms * 1e6;
    return 0;
}

// kernels/ns/ns.cpp:230-242
int ns_fill(ns_gpu* g, void* dst, uint8_t value, size_t bytes) {
    if (ns_enter(g, "ns_fill")) return -1;
    if (bytes) NS_CUDA(cudaMemsetAsync(dst, value, bytes, g->compute), "ns_fill");
    return 0;
}

int ns_sync(ns_gpu* g) {
    if (ns_enter(g, "ns_sync")) return -1;
    NS_CUDA(cudaStreamSynchronize(g->compute), "ns_sync");
    NS_CUDA(cudaGetLastError(), "ns_sync");
    if (g->status_host && *(volatile int*) g->status_host != 0) {
        const int code = *(volatile int*) g->status_host;
        *(volatile int*) g->status_host = 0;
        if (g->dec_sync) cudaMemset(g->dec_sync, 0, 2 * NS_DEC_SYNC_SLOTS * sizeof(unsigned int));   // counters a failed step may have left set
        if (code == 802)
            return ns_fail("ns_sync: a decode row needed more key splits than its call's max_kv laid out (code 802): a sequence is longer than "
                           "max_kv; its output is not valid");
        if (code == 803) return ns_fail("ns_sync: a batched cache write would have passed a cache's capacity (code 803); those rows were not written");
        return ns_fail("ns_sync: a kernel gave up a bounded wait (code " + std::to_string(code) + "); its output is not valid");
    }
    return 0;
}

// kernels/ns/ns.cpp:244-250 copies through host memory and waits twice; here one peer copy over NVLink, then a wait
int ns_copy_peer(ns_gpu* to, void* dst, ns_gpu* from, const void* src, size_t bytes, void* staging) {
    (void) staging;
    if (!to || !from) return ns_fail("ns_copy_peer: no gpu");
    if (ns_enter(from, "ns_copy_peer")) return -1;
    NS_CUDA(cudaStreamSynchronize(from->compute), "ns_copy_peer");
    if (ns_enter(to, "ns_copy_peer")) return -1;
    if (bytes) NS_CUDA(cudaMemcpyPeerAsync(dst, to->dev, src, from->dev, bytes, to->compute), "ns_copy_peer");
    NS_CUDA(cudaStreamSynchronize(to->compute), "ns_copy_peer");
    return 0;
}

}  // extern "C"

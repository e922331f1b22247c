// ns_internal.cuh: what the library's translation units share (not part of the ABI).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "ns.h"

// One opened GPU: a device ordinal, the compute stream every kernel and ordered copy goes to, two copy lanes
// (ns_stream_copy), and the ticket ring. Buffers the library keeps for the process (query staging, counters) hang off
// it and are freed by ns_gpu_close.
// (sequence, key head) pairs the decode kernels' completion counters cover; larger batches use the plain dependent merge
constexpr int NS_DEC_SYNC_SLOTS = 65536;

struct ns_gpu {
    int dev = 0;
    int sms = 0;
    cudaStream_t compute = nullptr;
    cudaStream_t lane[2] = {nullptr, nullptr};
    std::mutex mu;                       // guards the ring and the kept buffers
    std::vector<cudaEvent_t> ring;       // 65,536 slots, created on first use
    int64_t next_ticket = 0;
    void* kept = nullptr;                // grow-only staging buffer (compat entry points: fp32 -> fp16 queries)
    size_t kept_bytes = 0;
    unsigned int* dec_sync = nullptr;    // 2 x NS_DEC_SYNC_SLOTS counters: decode CTAs done / merge blocks done, per (sequence, key head)
    void* kept_kv = nullptr;             // a second one: quantised caches expanded to fp16 for the tensor-core kernels
    size_t kept_kv_bytes = 0;
    int* status_host = nullptr;          // one word of mapped pinned memory: a kernel whose bounded wait gave up writes its code
    int* status_dev = nullptr;           // the same word as the device sees it; ns_sync reports and clears it
};

static constexpr int64_t NS_RING = 1 << 16;

// sets the calling thread's message and returns -1
int ns_fail(const std::string& what);
// -1 with "<where>: <cuda error string>" when e is an error
int ns_cuda(cudaError_t e, const char* where);

#define NS_CUDA(call, where)                          \
    do {                                              \
        cudaError_t e__ = (call);                     \
        if (e__ != cudaSuccess) return ns_cuda(e__, where); \
    } while (0)

// makes g's device current for the calling thread; -1 on a null handle
int ns_enter(ns_gpu* g, const char* where);
// the kept staging buffer grown to at least `bytes` (stream-ordered with the compute stream: growth frees the old
// buffer only after the stream has drained)
int ns_kept(ns_gpu* g, size_t bytes, void** out);
int ns_kept_kv(ns_gpu* g, size_t bytes, void** out);
// after a kernel launch: surfaces a launch-configuration error as -1
int ns_launched(const char* where);

// C++ exceptions never cross the ABI
#define NS_TRY try {
#define NS_CATCH(where)                                                                    \
    }                                                                                      \
    catch (const std::exception& e) { return ns_fail(std::string(where) + ": " + e.what()); } \
    catch (...) { return ns_fail(std::string(where) + ": unknown failure"); }

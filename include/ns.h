/* ns.h: the device / memory / copy part of the C ABI, on CUDA.
 *
 * Same names, argument meaning and error behaviour as the reference's kernels/ns/ns.h:18-56, so the reference's
 * loader (crates/sys/src/lib.rs:200-236, one dlsym per name below) binds this library unchanged. Every call returns 0,
 * or -1 with the reason available from ns_last_error() on the calling thread (kernels/ns/ns.h:3).
 *
 * What differs underneath: an ns_gpu is a CUDA device ordinal with one compute stream and two copy streams
 * (the reference: one in-order SYCL queue and two copy queues, kernels/ns/ns_internal.hpp:8-16); tickets are CUDA
 * events in a 65,536-slot ring; ns_copy_peer goes over NVLink and ignores its staging argument.
 */
#ifndef NS_H
#define NS_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ns_gpu ns_gpu;

/* kernels/ns/ns.h:20-21. The message stays valid until the thread's next failing call. */
const char* ns_last_error(void);
const char* ns_version(void);

/* kernels/ns/ns.h:24-27: CUDA devices in ordinal order; units = SM count, mhz = SM clock. */
int ns_gpu_count(void);
int ns_gpu_name(int index, char* buf, size_t len);
int ns_gpu_pci(int index, char* buf, size_t len);
int ns_gpu_units(int index, int* units, int* mhz);
/* kernels/ns/ns.h:29-30 */
int ns_gpu_open(int index, ns_gpu** out);
void ns_gpu_close(ns_gpu* g);
/* kernels/ns/ns.h:32: the native queue; here a pointer to the compute cudaStream_t */
void* ns_gpu_queue(ns_gpu* g);
/* kernels/ns/ns.h:34 */
int ns_gpu_memory(ns_gpu* g, uint64_t* total, int64_t* free_bytes);

/* kernels/ns/ns.h:36-40. A failed device allocation says "device allocation of N bytes failed", which callers
 * classify as retryable (crates/core/src/lib.rs:39-43). */
int ns_alloc(ns_gpu* g, size_t bytes, void** out);
int ns_free(ns_gpu* g, void* p);
int ns_alloc_host(ns_gpu* g, size_t bytes, void** out);
int ns_free_host(ns_gpu* g, void* p);
/* kernels/ns/ns.h:42-46: queued on the compute stream, in order; they return before the copy has run */
int ns_copy_to(ns_gpu* g, void* dst, const void* src_host, size_t bytes);
int ns_copy_from(ns_gpu* g, void* dst_host, const void* src, size_t bytes);
int ns_copy_dev(ns_gpu* g, void* dst, const void* src, size_t bytes);
int ns_copy_2d(ns_gpu* g, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t height);
/* kernels/ns/ns.h:47-51: tickets. ns_mark: everything queued so far; ns_stream_copy: a copy on lane 0 or 1 after
 * `ndeps` tickets, returning its own; ns_await: the compute stream waits on the device; ns_stamp / ns_elapsed:
 * device timestamps, nanoseconds between the ends of two stamps (waits for them). */
int ns_mark(ns_gpu* g, int64_t* ticket);
int ns_stream_copy(ns_gpu* g, void* dst, const void* src, size_t bytes, const int64_t* after, int ndeps, int lane, int64_t* ticket);
int ns_await(ns_gpu* g, int64_t ticket);
int ns_stamp(ns_gpu* g, int64_t* ticket);
int ns_elapsed(ns_gpu* g, int64_t t0, int64_t t1, double* ns);
/* kernels/ns/ns.h:52-53 */
int ns_fill(ns_gpu* g, void* dst, uint8_t value, size_t bytes);
int ns_sync(ns_gpu* g);
/* kernels/ns/ns.h:56: device memory of one GPU into another's; waits. `staging` is accepted and unused. */
int ns_copy_peer(ns_gpu* to, void* dst, ns_gpu* from, const void* src, size_t bytes, void* staging);

#ifdef __cplusplus
}
#endif
#endif

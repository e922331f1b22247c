// tc05.cuh: thin inline-PTX wrappers for the Blackwell (sm_100a) tensor path: mbarriers with bounded waits, TMA tile
// loads, tensor-memory allocation, tcgen05.mma / commit / ld / st, and the shared-memory and instruction descriptors.
// Device code only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace tc05 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarriers -------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) { asm volatile("mbarrier.inval.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase of `parity` to complete, at most `limit` polls. On giving up it raises *abort (shared memory:
// every later wait of the CTA returns at once) and records `code` in *status (global or mapped host memory), so the
// kernel runs to its teardown instead of hanging. Returns false when the wait did not complete.
constexpr uint32_t WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort, int* status, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*abort) return false;
        if (i > 64) __nanosleep(64);
    }
    *abort = 1;
    if (status) {
        *(volatile int*) status = code;
        __threadfence_system();
    }
    return false;
}

// ---- TMA -------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(tmap) : "memory");
}
// a box of a rank-3 tensor into shared memory; x is the innermost coordinate (x * element size a multiple of 16 bytes)
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
                 "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

// the same box only as far as L2: no shared memory, no barrier - a later tma_load_3d of it finds it there
__device__ __forceinline__ void tma_prefetch_3d(const void* tmap, int x, int y, int z) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];\n" ::"l"(tmap), "r"(x), "r"(y), "r"(z) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------------------------------
// one whole warp; ncols a power of two >= 32; the base address lands in *slot (shared memory)
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// this warp's 32 lanes (rows) x 32 consecutive 32-bit columns from taddr (lane field = 32 * (warp % 4))
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---- descriptors -----------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle (tiles as TMA writes them with CU_TENSOR_MAP_SWIZZLE_128B; the
// tile base 1024-byte aligned). Fields: start address >> 4 in bits [0,14), leading byte offset >> 4 in [16,30), stride
// byte offset >> 4 in [32,46), descriptor version 1 in [46,48), layout type 2 (128-byte swizzle) in [61,64).
//   K-major operand (rows of 64 16-bit elements = 128 B): sbo = bytes between 8-row groups (1024 when rows are dense),
//     lbo unused (1). A K-step of 16 elements inside the 128-byte row advances the start address by 32 bytes.
//   MN-major operand (a "row" = 64 contiguous MN elements of one K index): sbo = bytes between groups of 8 K indices,
//     lbo = bytes between 64-element MN chunks.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr >> 4) & 0x3FFF);
    d |= (uint64_t) ((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t) ((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 2 << 61;
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation: D format fp32 (1) in bits [4,6), A format in
// [7,10) and B format in [10,13) (0 fp16, 1 bf16), A major in bit 15 and B major in bit 16 (0 K-major, 1 MN-major),
// N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, int bf16, int a_mn, int b_mn) {
    return (1u << 4) | ((uint32_t) bf16 << 7) | ((uint32_t) bf16 << 10) | ((uint32_t) a_mn << 15) | ((uint32_t) b_mn << 16) |
           ((uint32_t) (n >> 3) << 17) | ((uint32_t) (m >> 4) << 24);
}

// D[tmem] (+)= A[smem] x B[smem]; one thread issues
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] x B[smem]: A is K-major in tensor memory, row = lane, 16-bit elements two a column
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier gets one arrival when every tcgen05.mma this thread issued before has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// a barrier among `threads` threads of the CTA (whole warps); id 0 is __syncthreads's
__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory"); }

// ---- a pair of CTAs (a cluster of two) on one MMA: cta_group::2 ------------------------------------------------------
// The CTA of even rank (the leader) issues the MMAs; an M = 128 product gives each CTA 64 rows of D, A comes from each
// CTA's own shared memory (its 64 rows), B from both (each holds half of N), all at the same offsets in both CTAs.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the address, in the cluster's shared window, of the same shared-memory location in the CTA of rank `rank`
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// one arrival on a barrier of any CTA of the cluster (address from cluster_map)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// writes this thread made to shared memory become visible to the tensor core and TMA (the async proxy)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// one warp in EACH CTA of the pair, the same slot offset in both
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(ncols) : "memory");
}
// a box into this CTA's shared memory; the bytes are counted on the barrier at `bar`'s offset in the LEADER (bar may be
// the local address: the peer bit is cleared here)
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* tmap, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
                 "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar & 0xFEFFFFFFu)
                 : "memory");
}
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with A in tensor memory: each CTA's 64 rows, K-major, 16-bit elements two a column, held twice - lanes 0..63 and
// again lanes 64..127 (the pair's operand form)
__device__ __forceinline__ void mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrival on the barrier at `cluster_addr` (a cluster_map address: either CTA's) when every MMA of the pair that this
// thread issued before has completed
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// ---- two fp32 values a 64-bit register: one instruction of the FMA pipe works on both ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// 2^x for a pair, x <= ~0, on the FMA and integer pipes instead of the special-function unit: x = n + r with n = round(x)
// (the magic-number addition leaves n in the sum's low mantissa bits) and r in [-1/2, 1/2]; 2^r by a cubic fitted to a
// relative error of 7.5e-5 - well inside a 16-bit weight's rounding, 4.9e-4 for fp16 -; n goes into the exponent by an
// integer addition. x is held at -125 from below (2^-125: a weight of zero once rounded).
__device__ __forceinline__ void ex2_pair_fma(uint64_t x2, float& a, float& b) {
    float xa, xb;
    unpack2(x2, xa, xb);
    xa = fmaxf(xa, -125.0f);
    xb = fmaxf(xb, -125.0f);
    const uint64_t x = pack2(xa, xb);
    const uint64_t magic = pack2(12582912.0f, 12582912.0f), neg_magic = pack2(-12582912.0f, -12582912.0f);
    const uint64_t minus1 = pack2(-1.0f, -1.0f);
    const uint64_t t = add2(x, magic);                  // round(x) in the low mantissa bits
    const uint64_t n = add2(t, neg_magic);              // round(x) as a float
    const uint64_t r = fma2(n, minus1, x);              // x - round(x)
    uint64_t q = fma2(pack2(0.05517167f, 0.05517167f), r, pack2(0.24261113f, 0.24261113f));
    q = fma2(q, r, pack2(0.69326097f, 0.69326097f));
    q = fma2(q, r, pack2(0.99992806f, 0.99992806f));
    float qa, qb, ta, tb;
    unpack2(q, qa, qb);
    unpack2(t, ta, tb);
    a = __uint_as_float(__float_as_uint(qa) + (__float_as_uint(ta) << 23));
    b = __uint_as_float(__float_as_uint(qb) + (__float_as_uint(tb) << 23));
}

}  // namespace tc05

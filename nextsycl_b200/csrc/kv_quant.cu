// kv_quant.cu: the quantised forms of the GQA caches (heads of 256): the writer, the reader's values as fp16, and the
// 32-point rotation that goes with them (kernels/llm/qwen35/q35.cpp:281-348, reader silo/attn.cpp:49-78).
//
// A head's row: q8_0 (kt 1) 256 int8 values then 8 fp16 scales = 272 bytes; q4_0 (kt 2) 8 blocks of 16 bytes (byte j of a
// block: value j in the low nibble, value j + 16 in the high one) then 8 fp16 scales = 144 bytes - llama.cpp's blocks of
// 32 with the scales moved behind the values.
#include "kernels.cuh"

namespace {

__host__ __device__ constexpr int64_t q_row_bytes(int kt) { return kt == 1 ? 272 : 144; }

// A warp a head row (256 values = 8 blocks of 32), keys then values; lane j holds value j of each of the 8 blocks, so every
// load is one coalesced 128 bytes and a block's scale is a butterfly of shuffles. The arithmetic is llama.cpp's q8_0 /
// q4_0 as the reference writes it (q35.cpp:289-322), every product and quotient a single rounding: q8_0 d = amax / 127,
// q = round-half-away(x / d ... as x * (1 / d)); q4_0 d = m / -8 with m the FIRST value of largest magnitude, code =
// min(15, trunc(x * (1 / d) + 8.5)), value j in the low nibble of byte j and value j + 16 in the high one.
constexpr int QWARPS = 8;

__global__ void __launch_bounds__(QWARPS * 32) kv_store_q_kernel(int kt, const float* __restrict__ k, int64_t ks, const float* __restrict__ v, int64_t vs,
                                                                 int64_t T, int64_t Hkv, int64_t cap, int64_t p0, uint8_t* __restrict__ kd,
                                                                 uint8_t* __restrict__ vd) {
    const unsigned FULL = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int64_t rows = 2 * T * Hkv;   // (k | v, token, key head)
    const int64_t rb = q_row_bytes(kt);
    for (int64_t r = (int64_t) blockIdx.x * QWARPS + (threadIdx.x >> 5); r < rows; r += (int64_t) gridDim.x * QWARPS) {
        const bool isv = r >= T * Hkv;
        const int64_t th = isv ? r - T * Hkv : r, t = th / Hkv, h = th % Hkv;
        const float* x = (isv ? v + t * vs : k + t * ks) + h * 256;
        uint8_t* row = (isv ? vd : kd) + (h * cap + p0 + t) * rb;
        float xv[8];
#pragma unroll
        for (int b = 0; b < 8; ++b) xv[b] = x[b * 32 + lane];
        float mine = 0.0f;   // lane b < 8 ends up holding block b's scale
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            // the block's largest magnitude and the lowest lane that holds it
            float am = fabsf(xv[b]);
            int at = lane;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float oa = __shfl_xor_sync(FULL, am, o);
                const int oi = __shfl_xor_sync(FULL, at, o);
                if (oa > am || (oa == am && oi < at)) am = oa, at = oi;
            }
            float d;
            if (kt == 1) {
                d = __fdiv_rn(am, 127.0f);
                const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                row[b * 32 + lane] = (uint8_t) (int8_t) roundf(__fmul_rn(xv[b], inv));
            } else {
                const float first = __shfl_sync(FULL, xv[b], at);
                const float m = am > 0.0f ? first : 0.0f;   // a block of zeros keeps the reference's initial m = +0, so d = -0
                d = __fdiv_rn(m, -8.0f);
                const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                const int code = min(15, (int) __fadd_rn(__fmul_rn(xv[b], inv), 8.5f));
                const int hi = __shfl_down_sync(FULL, code, 16);
                if (lane < 16) row[b * 16 + lane] = (uint8_t) (code | (hi << 4));
            }
            if (lane == b) mine = d;
        }
        if (lane < 8) reinterpret_cast<__half*>(row + (kt == 1 ? 256 : 128))[lane] = __float2half_rn(mine);
    }
}

// rows [0, n) of each head as fp16 [Hkv][n][256]: value = half(float(q) * float(d)), one rounding (silo/attn.cpp:57-77).
// A thread 8 values (one 16-byte store).
__global__ void kv_dequant_kernel(int kt, const uint8_t* __restrict__ c, int64_t Hkv, int64_t cap, int64_t n, __half* __restrict__ out) {
    const int64_t total = Hkv * n * 32;
    const int64_t rb = q_row_bytes(kt);
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int u = (int) (id % 32);                 // features 8u .. 8u + 7
        const int64_t j = (id / 32) % n, h = id / (32 * n);
        const uint8_t* row = c + (h * cap + j) * rb;
        float f[8];
        if (kt == 1) {
            const uint2 w = *reinterpret_cast<const uint2*>(row + 8 * u);
            const float d = __half2float(reinterpret_cast<const __half*>(row + 256)[u >> 2]);
            const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __fmul_rn((float) (int8_t) ((ww[i >> 2] >> (8 * (i & 3))) & 0xff), d);
        } else {
            const int blk = u >> 2, sub = u & 3;
            const uint2 w = *reinterpret_cast<const uint2*>(row + blk * 16 + (sub & 1) * 8);
            const float d = __half2float(reinterpret_cast<const __half*>(row + 128)[blk]);
            const int sh = sub >= 2 ? 4 : 0;
            const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __fmul_rn((float) ((int) (((ww[i >> 2] >> (8 * (i & 3))) >> sh) & 15) - 8), d);
        }
        __half2 o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(out + (h * n + j) * 256 + 8 * u) = *reinterpret_cast<uint4*>(o);
    }
}

// The normalised 32-point Walsh-Hadamard transform of every block of 32 (q35.cpp:328-348), a warp a block: lane i holds
// element i and stage o (1, 2, 4, 8, 16) is one exchange with lane i ^ o - the lower lane of a pair keeps a + b, the upper
// a - b, the pairs and their order the reference's, every sum a single rounding - then the factor 1 / sqrt(32).
__global__ void __launch_bounds__(QWARPS * 32) fwht32_kernel(float* __restrict__ x, int64_t rows, int64_t nb, int64_t stride) {
    const int lane = threadIdx.x & 31;
    const int64_t total = rows * nb;
    for (int64_t id = (int64_t) blockIdx.x * QWARPS + (threadIdx.x >> 5); id < total; id += (int64_t) gridDim.x * QWARPS) {
        float* p = x + (id / nb) * stride + (id % nb) * 32;
        float val = p[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, val, o);
            val = (lane & o) ? __fsub_rn(other, val) : __fadd_rn(val, other);
        }
        p[lane] = __fmul_rn(val, 0.17677669529663687f);
    }
}

unsigned blocks_for(int64_t n) { return (unsigned) std::min<int64_t>(8192, (n + 255) / 256); }
unsigned warp_blocks(int64_t warps) { return (unsigned) std::min<int64_t>(8192, (warps + QWARPS - 1) / QWARPS); }

}  // namespace

int ns_launch_kv_dequant(ns_gpu* g, int kt, const void* c, int64_t Hkv, int64_t cap, int64_t n, void* out, const char* where) {
    kv_dequant_kernel<<<blocks_for(Hkv * n * 32), 256, 0, g->compute>>>(kt, (const uint8_t*) c, Hkv, cap, n, (__half*) out);
    return ns_launched(where);
}

extern "C" {

int ns_q35_kv_store_q(ns_gpu* g, int kt, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap,
                      int64_t p0, void* kc, void* vc) {
    NS_TRY
    if (ns_enter(g, "ns_q35_kv_store_q")) return -1;
    if (T <= 0) return 0;
    if (D != 256 || (kt != 1 && kt != 2)) return ns_fail("ns_q35_kv_store_q: heads of 256, form 1 (q8_0) or 2 (q4_0)");
    if (p0 < 0 || p0 + T > cap) return ns_fail("ns_q35_kv_store_q: past the cache's capacity");
    if (!k || !v || !kc || !vc || Hkv < 1) return ns_fail("ns_q35_kv_store_q: a null buffer");
    if (ks % 4 != 0 || vs % 4 != 0 || ((uintptr_t) k & 15) != 0 || ((uintptr_t) v & 15) != 0 || ((uintptr_t) kc & 15) != 0 || ((uintptr_t) vc & 15) != 0)
        return ns_fail("ns_q35_kv_store_q: rows 16-byte aligned");
    kv_store_q_kernel<<<warp_blocks(2 * T * Hkv), QWARPS * 32, 0, g->compute>>>(kt, k, ks, v, vs, T, Hkv, cap, p0, (uint8_t*) kc, (uint8_t*) vc);
    return ns_launched("ns_q35_kv_store_q");
    NS_CATCH("ns_q35_kv_store_q")
}

int ns_q35_fwht32(ns_gpu* g, float* x, int64_t rows, int64_t n, int64_t stride) {
    NS_TRY
    if (ns_enter(g, "ns_q35_fwht32")) return -1;
    if (rows <= 0) return 0;
    if (n % 32) return ns_fail("ns_q35_fwht32: rows of a multiple of 32");
    if (!x || stride < n) return ns_fail("ns_q35_fwht32: rows at least n floats apart");
    fwht32_kernel<<<warp_blocks(rows * (n / 32)), QWARPS * 32, 0, g->compute>>>(x, rows, n / 32, stride);
    return ns_launched("ns_q35_fwht32");
    NS_CATCH("ns_q35_fwht32")
}

}  // extern "C"

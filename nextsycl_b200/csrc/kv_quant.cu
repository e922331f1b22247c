// kv_quant.cu: the quantised forms of the GQA caches (heads of 256): the writer, the reader's values as fp16, and the
// 32-point rotation that goes with them (kernels/llm/qwen35/q35.cpp:281-348, reader silo/attn.cpp:49-78).
//
// A head's row: q8_0 (kt 1) 256 int8 values then 8 fp16 scales = 272 bytes; q4_0 (kt 2) 8 blocks of 16 bytes (byte j of a
// block: value j in the low nibble, value j + 16 in the high one) then 8 fp16 scales = 144 bytes - llama.cpp's blocks of
// 32 with the scales moved behind the values.
#include "kernels.cuh"

namespace {

__host__ __device__ constexpr int64_t q_row_bytes(int kt) { return kt == 1 ? 272 : 144; }

// a thread a block of 32 values, keys then values (q35.cpp:289-322). Products and sums are single roundings (no fused
// multiply-add), as the CPU statement of the same arithmetic computes them.
__global__ void kv_store_q_kernel(int kt, const float* __restrict__ k, int64_t ks, const float* __restrict__ v, int64_t vs, int64_t T, int64_t Hkv,
                                  int64_t cap, int64_t p0, uint8_t* __restrict__ kd, uint8_t* __restrict__ vd) {
    const int64_t total = 2 * T * Hkv * 8;
    const int64_t rb = q_row_bytes(kt);
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        int64_t i = id;
        const int b = (int) (i % 8);
        i /= 8;
        const int64_t h = i % Hkv;
        i /= Hkv;
        const int64_t t = i % T;
        const bool isv = i / T == 1;
        const float* x = (isv ? v + t * vs : k + t * ks) + h * 256 + b * 32;
        uint8_t* row = (isv ? vd : kd) + (h * cap + p0 + t) * rb;
        float xv[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 a = *reinterpret_cast<const float4*>(x + 4 * j);
            xv[4 * j] = a.x, xv[4 * j + 1] = a.y, xv[4 * j + 2] = a.z, xv[4 * j + 3] = a.w;
        }
        if (kt == 1) {
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(xv[j]));
            const float d = __fdiv_rn(amax, 127.0f), inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) word |= ((uint32_t) (uint8_t) (int8_t) roundf(__fmul_rn(xv[4 * j + e], inv))) << (8 * e);
                w[j] = word;
            }
            uint4* dst = reinterpret_cast<uint4*>(row + b * 32);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            reinterpret_cast<__half*>(row + 256)[b] = __float2half_rn(d);
        } else {
            float m = 0.0f, am = 0.0f;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (fabsf(xv[j]) > am) {
                    am = fabsf(xv[j]);
                    m = xv[j];
                }
            const float d = __fdiv_rn(m, -8.0f), inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
            uint32_t w[4];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = 4 * j4 + e;
                    const int lo = min(15, (int) __fadd_rn(__fmul_rn(xv[j], inv), 8.5f)), hi = min(15, (int) __fadd_rn(__fmul_rn(xv[j + 16], inv), 8.5f));
                    word |= (uint32_t) (lo | (hi << 4)) << (8 * e);
                }
                w[j4] = word;
            }
            *reinterpret_cast<uint4*>(row + b * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<__half*>(row + 128)[b] = __float2half_rn(d);
        }
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

// q35.cpp:328-348: a thread a block of 32, the butterflies in the reference's order
__global__ void fwht32_kernel(float* __restrict__ x, int64_t rows, int64_t nb, int64_t stride) {
    const int64_t total = rows * nb;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        float* p = x + (id / nb) * stride + (id % nb) * 32;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = p[i];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (!(i & o)) {
                    const float a = v[i], b = v[i + o];
                    v[i] = __fadd_rn(a, b);
                    v[i + o] = __fsub_rn(a, b);
                }
#pragma unroll
        for (int i = 0; i < 32; ++i) p[i] = __fmul_rn(v[i], 0.17677669529663687f);
    }
}

unsigned blocks_for(int64_t n) { return (unsigned) std::min<int64_t>(8192, (n + 255) / 256); }

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
    kv_store_q_kernel<<<blocks_for(2 * T * Hkv * 8), 256, 0, g->compute>>>(kt, k, ks, v, vs, T, Hkv, cap, p0, (uint8_t*) kc, (uint8_t*) vc);
    return ns_launched("ns_q35_kv_store_q");
    NS_CATCH("ns_q35_kv_store_q")
}

int ns_q35_fwht32(ns_gpu* g, float* x, int64_t rows, int64_t n, int64_t stride) {
    NS_TRY
    if (ns_enter(g, "ns_q35_fwht32")) return -1;
    if (rows <= 0) return 0;
    if (n % 32) return ns_fail("ns_q35_fwht32: rows of a multiple of 32");
    if (!x || stride < n) return ns_fail("ns_q35_fwht32: rows at least n floats apart");
    fwht32_kernel<<<blocks_for(rows * (n / 32)), 256, 0, g->compute>>>(x, rows, n / 32, stride);
    return ns_launched("ns_q35_fwht32");
    NS_CATCH("ns_q35_fwht32")
}

}  // extern "C"

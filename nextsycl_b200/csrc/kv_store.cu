// kv_store.cu: the writers of the caches the attention kernels read.
#include "kernels.cuh"

namespace {
// fp32 rows -> the fp16 caches [Hkv][cap][D] at positions p0 .. (kernels/llm/qwen35/q35.cpp:573-588); a thread 8 values
__global__ void kv_store_kernel(const float* __restrict__ k, int64_t ks, const float* __restrict__ v, int64_t vs, int64_t T, int64_t Hkv, int64_t D,
                                int64_t cap, int64_t p0, __half* __restrict__ kc, __half* __restrict__ vc) {
    const int64_t n8 = T * Hkv * (D / 8);
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t d = (i % (D / 8)) * 8, h = (i / (D / 8)) % Hkv, t = i / ((D / 8) * Hkv);
        const int64_t at = (h * cap + p0 + t) * D + d;
        const float* kr = k + t * ks + h * D + d;
        const float* vr = v + t * vs + h * D + d;
        __half2 ko[4], vo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            ko[e] = __floats2half2_rn(kr[2 * e], kr[2 * e + 1]);
            vo[e] = __floats2half2_rn(vr[2 * e], vr[2 * e + 1]);
        }
        *reinterpret_cast<uint4*>(kc + at) = *reinterpret_cast<uint4*>(ko);
        *reinterpret_cast<uint4*>(vc + at) = *reinterpret_cast<uint4*>(vo);
    }
}
}  // namespace

int ns_launch_kv_store(ns_gpu* g, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap, int64_t p0,
                       void* kc, void* vc) {
    const int64_t n8 = T * Hkv * (D / 8);
    const int threads = 256;
    const int64_t blocks = (n8 + threads - 1) / threads;
    kv_store_kernel<<<(unsigned) (blocks > 4096 ? 4096 : blocks), threads, 0, g->compute>>>(k, ks, v, vs, T, Hkv, D, cap, p0, (__half*) kc, (__half*) vc);
    return ns_launched("ns_q35_kv_store");
}

namespace {
__global__ void scale_to_f16_kernel(const float* __restrict__ src, int64_t src_row, __half* __restrict__ dst, int64_t dst_row, int64_t rows, int64_t cols,
                                    float scale) {
    const int64_t n8 = rows * (cols / 8);
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t r = i / (cols / 8), c = (i % (cols / 8)) * 8;
        const float4 a = *reinterpret_cast<const float4*>(src + r * src_row + c);
        const float4 b = *reinterpret_cast<const float4*>(src + r * src_row + c + 4);
        __half2 o[4] = {__floats2half2_rn(a.x * scale, a.y * scale), __floats2half2_rn(a.z * scale, a.w * scale),
                        __floats2half2_rn(b.x * scale, b.y * scale), __floats2half2_rn(b.z * scale, b.w * scale)};
        *reinterpret_cast<uint4*>(dst + r * dst_row + c) = *reinterpret_cast<uint4*>(o);
    }
}
}  // namespace

int ns_launch_scale_to_f16(ns_gpu* g, const float* src, int64_t src_row, void* dst, int64_t dst_row, int64_t rows, int64_t cols, float scale) {
    const int64_t n8 = rows * (cols / 8);
    const int64_t blocks = (n8 + 255) / 256;
    scale_to_f16_kernel<<<(unsigned) (blocks > 8192 ? 8192 : blocks), 256, 0, g->compute>>>(src, src_row, (__half*) dst, dst_row, rows, cols, scale);
    return ns_launched("scale_to_f16");
}

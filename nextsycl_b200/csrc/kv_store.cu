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
// The same for a batch in one launch: sequence b's T rows go to positions p0 .. of ITS caches, both read from the device
// table the batched decode reads. A row that would land past its cache's capacity is not written and raises status 803.
__global__ void kv_store_batch_kernel(const float* __restrict__ k, int64_t ks, int64_t k_seq, const float* __restrict__ v, int64_t vs, int64_t v_seq,
                                      const ns_b200_seq* __restrict__ seqs, int64_t B, int64_t T, int64_t Hkv, int64_t D, int* status) {
    const int64_t per = T * Hkv * (D / 8), n8 = B * per;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t b = i / per, j = i % per;
        const int64_t d = (j % (D / 8)) * 8, h = (j / (D / 8)) % Hkv, t = j / ((D / 8) * Hkv);
        const ns_b200_seq s = seqs[b];
        if (s.p0 < 0 || s.p0 + t >= s.cap) {
            if (status) *(volatile int*) status = 803;
            continue;
        }
        const int64_t at = (h * s.cap + s.p0 + t) * D + d;
        const float4* kr = reinterpret_cast<const float4*>(k + b * k_seq + t * ks + h * D + d);
        const float4* vr = reinterpret_cast<const float4*>(v + b * v_seq + t * vs + h * D + d);
        const float4 k0 = kr[0], k1 = kr[1], v0 = vr[0], v1 = vr[1];
        __half2 ko[4] = {__floats2half2_rn(k0.x, k0.y), __floats2half2_rn(k0.z, k0.w), __floats2half2_rn(k1.x, k1.y), __floats2half2_rn(k1.z, k1.w)};
        __half2 vo[4] = {__floats2half2_rn(v0.x, v0.y), __floats2half2_rn(v0.z, v0.w), __floats2half2_rn(v1.x, v1.y), __floats2half2_rn(v1.z, v1.w)};
        *reinterpret_cast<uint4*>((__half*) s.kc + at) = *reinterpret_cast<uint4*>(ko);
        *reinterpret_cast<uint4*>((__half*) s.vc + at) = *reinterpret_cast<uint4*>(vo);
    }
}
}  // namespace

int ns_launch_kv_store_batch(ns_gpu* g, const float* k, int64_t ks, int64_t k_seq, const float* v, int64_t vs, int64_t v_seq, const ns_b200_seq* seqs,
                             int64_t B, int64_t T, int64_t Hkv, int64_t D) {
    const int64_t n8 = B * T * Hkv * (D / 8);
    const int64_t blocks = (n8 + 255) / 256;
    kv_store_batch_kernel<<<(unsigned) (blocks > 4096 ? 4096 : blocks), 256, 0, g->compute>>>(k, ks, k_seq, v, vs, v_seq, seqs, B, T, Hkv, D, g->status_dev);
    return ns_launched("ns_b200_kv_store_batch");
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

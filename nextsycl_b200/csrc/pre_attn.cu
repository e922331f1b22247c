// pre_attn.cu: the step before attention - RMS norm of each head of q and k, rotary positions, and the writes that feed
// the attention kernels (kernels/llm/qwen35/q35.cpp:220-279,350-385,573-588). The reference runs it as three or four
// launches a layer (norm+rope of q, of k, the cache store); ns_b200_qkv_prepare is the same arithmetic in one launch,
// with q leaving as the fp16 rows the native attention entry points read and k, v landing in the fp16 caches.
#include "kernels.cuh"

#include <algorithm>
#include <cmath>

namespace {

// Row x [D] of one (row, head), a warp: RMS norm (w null: none), rotate-half over the first n_rot features (pair (i, i +
// n_rot/2) by angle p * theta^(-2i/n_rot)), then `put(i, value)` for every feature. Both features of a pair are read
// before either is written, so src and dst may be the same rows.
template <class Put>
__device__ __forceinline__ void norm_rope_row(const float* __restrict__ x, int64_t D, const float* __restrict__ w, float eps, int64_t n_rot, float theta,
                                              float p_t, const int32_t* pos3, int64_t s0, int64_t s1, int64_t s2, Put put) {
    const int lane = threadIdx.x & 31;
    float inv = 1.0f;
    if (w) {
        float s = 0.0f;
        for (int64_t i = lane; i < D; i += 32) s += x[i] * x[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        inv = rsqrtf(s / (float) D + eps);
    }
    const int64_t half_rot = n_rot / 2, sect = s0 + s1 + s2;
    for (int64_t i = lane; i < half_rot; i += 32) {
        float p = p_t;
        if (pos3) {
            const int64_t sec = i % sect;
            const int c = (sec % 3 == 1 && sec < 3 * s1) ? 1 : (sec % 3 == 2 && sec < 3 * s2) ? 2 : 0;
            p = (float) pos3[c];
        }
        // the frequency as the correctly rounded float of theta^e, e the reference's float exponent: at position 100,000 one
        // unit in the last place of the frequency is 0.008 rad of angle
        const float a = p * (float) pow((double) theta, (double) (-2.0f * (float) i / (float) n_rot));
        float sn, c_;
        sincosf(a, &sn, &c_);
        const float lo = w ? x[i] * inv * w[i] : x[i], hi = w ? x[i + half_rot] * inv * w[i + half_rot] : x[i + half_rot];
        put(i, lo * c_ - hi * sn);
        put(i + half_rot, hi * c_ + lo * sn);
    }
    for (int64_t i = n_rot + lane; i < D; i += 32) put(i, w ? x[i] * inv * w[i] : x[i]);
}

__global__ void __launch_bounds__(256) norm_rope_kernel(const float* __restrict__ src, int64_t ss, int64_t hs, float* __restrict__ dst, int64_t ds, int64_t T,
                                                        int64_t H, int64_t D, const float* __restrict__ w, float eps, int64_t n_rot, float theta, int64_t p0,
                                                        const int32_t* __restrict__ pos, int64_t s0, int64_t s1, int64_t s2) {
    const int64_t th = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (th >= T * H) return;
    const int64_t t = th / H, h = th % H;
    float* y = dst + t * ds + h * D;
    norm_rope_row(src + t * ss + h * hs, D, w, eps, n_rot, theta, (float) (p0 + t), pos ? pos + 3 * t : nullptr, s0, s1, s2,
                  [&](int64_t i, float v) { y[i] = v; });
}

// one launch for a layer's q, k, v rows: heads [0, Hq) are q (norm wq, rope) -> q_out fp16 [T][Hq*D]; heads [Hq, Hq+Hkv) are
// k (norm wk, rope) -> the key cache at position p0 + t; heads [Hq+Hkv, Hq+2Hkv) are v -> the value cache, unchanged
__global__ void __launch_bounds__(256) qkv_prepare_kernel(const float* __restrict__ q, int64_t qs, const float* __restrict__ k, int64_t ks,
                                                          const float* __restrict__ v, int64_t vs, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                                                          const float* __restrict__ wq, const float* __restrict__ wk, float eps, int64_t n_rot, float theta,
                                                          int64_t p0, int64_t cap, __half* __restrict__ q_out, __half* __restrict__ kc,
                                                          __half* __restrict__ vc) {
    const int64_t HT = Hq + 2 * Hkv, th = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (th >= T * HT) return;
    const int64_t t = th / HT, h = th % HT;
    const int lane = threadIdx.x & 31;
    if (h < Hq) {
        __half* y = q_out + (t * Hq + h) * D;
        norm_rope_row(q + t * qs + h * D, D, wq, eps, n_rot, theta, (float) (p0 + t), nullptr, 0, 0, 0, [&](int64_t i, float x) { y[i] = __float2half_rn(x); });
    } else if (h < Hq + Hkv) {
        const int64_t hk = h - Hq;
        __half* y = kc + (hk * cap + p0 + t) * D;
        norm_rope_row(k + t * ks + hk * D, D, wk, eps, n_rot, theta, (float) (p0 + t), nullptr, 0, 0, 0, [&](int64_t i, float x) { y[i] = __float2half_rn(x); });
    } else {
        const int64_t hk = h - Hq - Hkv;
        const float* x = v + t * vs + hk * D;
        __half* y = vc + (hk * cap + p0 + t) * D;
        for (int64_t i = lane; i < D; i += 32) y[i] = __float2half_rn(x[i]);
    }
}

// deepseek2 (kernels/llm/deepseek2/ds2.cpp:15-34): cos and sin of pair i0 (of n_dims) at position p as ggml's rope cache
// computes them - the angle by repeated products from the position, YaRN's ramp between the interpolated and the
// extrapolated angle, mscale on both. Every product and sum is a single rounding, in the reference's order.
__device__ __forceinline__ void yarn_cs(float p, int i0, float theta_scale, float freq_scale, float ext_factor, float mscale, float corr0, float corr1,
                                        float& c, float& s) {
    float theta_extrap = p;
    for (int k = 0; k < i0 / 2; ++k) theta_extrap = __fmul_rn(theta_extrap, theta_scale);
    const float theta_interp = __fmul_rn(freq_scale, theta_extrap);
    float theta = theta_interp;
    if (ext_factor != 0.0f) {
        const float y = __fdiv_rn(__fsub_rn((float) (i0 / 2), corr0), fmaxf(0.001f, __fsub_rn(corr1, corr0)));
        const float ramp_mix = __fmul_rn(__fsub_rn(1.0f, fminf(1.0f, fmaxf(0.0f, y))), ext_factor);
        theta = __fadd_rn(__fmul_rn(theta_interp, __fsub_rn(1.0f, ramp_mix)), __fmul_rn(theta_extrap, ramp_mix));
    }
    float sn, cs;
    sincosf(theta, &sn, &cs);
    c = __fmul_rn(cs, mscale);
    s = __fmul_rn(sn, mscale);
}

// ds2.cpp:58-83: adjacent pairs of the rotated part of each head, in place (and into `out`)
__global__ void ds2_rope_kernel(float* __restrict__ x, int64_t T, int64_t H, int64_t row, int64_t head, int64_t off, int64_t n_dims, int64_t pos0,
                                float theta_scale, float freq_scale, float ext_factor, float mscale, float corr0, float corr1, float* __restrict__ out,
                                int64_t out_row, int64_t out_head) {
    const int64_t pairs = n_dims / 2, total = T * H * pairs;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t i = id % pairs, h = (id / pairs) % H, t = id / (pairs * H);
        const int i0 = (int) (2 * i);
        float c, s;
        yarn_cs((float) (pos0 + t), i0, theta_scale, freq_scale, ext_factor, mscale, corr0, corr1, c, s);
        float* v = x + t * row + h * head + off + i0;
        const float x0 = v[0], x1 = v[1];
        const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)), y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        v[0] = y0, v[1] = y1;
        if (out) {
            float* o = out + t * out_row + h * out_head + i0;
            o[0] = y0, o[1] = y1;
        }
    }
}

// ds2.cpp:85-112: a block a token: the first L values RMS-normed with w, the last R rotated, into the fp16 cache row
__global__ void __launch_bounds__(256) ds2_kv_store_kernel(const float* __restrict__ kv, const float* __restrict__ w, float eps, __half* __restrict__ cache,
                                                           int64_t L, int64_t R, int64_t pos0, float theta_scale, float freq_scale, float ext_factor,
                                                           float mscale, float corr0, float corr1) {
    __shared__ float red[8];
    const int64_t t = blockIdx.x;
    const int lid = threadIdx.x;
    const float* xr = kv + t * (L + R);
    float ss = 0.f;
    for (int64_t i = lid; i < L; i += 256) ss += xr[i] * xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((lid & 31) == 0) red[lid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += red[k];
    const float inv = 1.f / sqrtf(tot / (float) L + eps);
    __half* o = cache + (pos0 + t) * (L + R);
    for (int64_t i = lid; i < L; i += 256) o[i] = __float2half_rn(xr[i] * inv * w[i]);
    for (int64_t i = lid; i < R / 2; i += 256) {
        const int i0 = (int) (2 * i);
        float c, s;
        yarn_cs((float) (pos0 + t), i0, theta_scale, freq_scale, ext_factor, mscale, corr0, corr1, c, s);
        const float x0 = xr[L + i0], x1 = xr[L + i0 + 1];
        o[L + i0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        o[L + i0 + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
    }
}

// deepseek41's E4M3 simulation (kernels/llm/deepseek41/silo/k41.cpp:16-35): a block of 32 values shares a power-of-two
// scale from its largest magnitude; each value becomes the nearest E4M3FN value (ties to even) times the scale
__device__ __forceinline__ float pow2_ceil(float x) {
    int e;
    const float m = frexpf(x, &e);
    if (m == 0.5f) e -= 1;
    return ldexpf(1.0f, e);
}
__device__ __forceinline__ float e4m3_round(float x) {
    const float a = fabsf(x);
    if (a == 0.f) return x;
    int e;
    frexpf(a, &e);
    int be = e - 1;
    if (be < -6) be = -6;
    const float step = ldexpf(1.0f, be - 3);
    float q = __fmul_rn(rintf(__fdiv_rn(a, step)), step);
    q = fminf(q, 448.f);
    return x < 0 ? -q : q;
}
// v of the 32 lanes of a warp = one block
__device__ __forceinline__ float e4m3_sim_warp(float v) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = pow2_ceil(__fdiv_rn(fmaxf(amax, 1e-4f), 448.f));
    return __fmul_rn(e4m3_round(fminf(fmaxf(__fdiv_rn(v, sc), -448.f), 448.f)), sc);
}

// k41.cpp:616-662: a block a token, D <= 512
__global__ void __launch_bounds__(256) ds41_kv_post_kernel(float* __restrict__ kv, const float* __restrict__ w, int64_t D, float eps, int64_t rd, int64_t pos0,
                                                           float theta_scale, float freq_scale, float ext_factor, float mscale, float corr0, float corr1,
                                                           __half* __restrict__ ring, int64_t R) {
    __shared__ float y[512];
    __shared__ float red[8];
    const int64_t t = blockIdx.x;
    const int lid = threadIdx.x;
    float* xr = kv + t * D;
    float s = 0.f;
    for (int64_t c = lid; c < D; c += 256) s += xr[c] * xr[c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((lid & 31) == 0) red[lid >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += red[k];
    const float inv = 1.f / sqrtf(tot / (float) D + eps);
    for (int64_t c = lid; c < D; c += 256) y[c] = xr[c] * inv * w[c];
    __syncthreads();
    const int64_t off = D - rd;
    if (lid < rd / 2) {
        const int i0 = 2 * lid;
        float cs, sn;
        yarn_cs((float) (pos0 + t), i0, theta_scale, freq_scale, ext_factor, mscale, corr0, corr1, cs, sn);
        const float x0 = y[off + i0], x1 = y[off + i0 + 1];
        y[off + i0] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        y[off + i0 + 1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
    }
    __syncthreads();
    for (int64_t c0 = 0; c0 < D; c0 += 256) {
        const int64_t c = c0 + lid;
        const bool in = c < D;               // D is a multiple of 32: a warp is all in or all out
        const float q = e4m3_sim_warp(in ? y[c] : 0.f);
        if (in) {
            xr[c] = q;
            ring[((pos0 + t) % R) * D + c] = __float2half_rn(q);
        }
    }
}

// k41.cpp:776-808: x [T][H][D]; a warp a block of 32 consecutive values; a pair's other value from the neighbouring lane
__global__ void __launch_bounds__(128) ds41_att_post_kernel(float* __restrict__ x, int64_t n, int64_t H, int64_t D, int64_t rd, int64_t pos0,
                                                            float theta_scale, float freq_scale, float ext_factor, float mscale, float corr0, float corr1) {
    const int64_t i = (int64_t) blockIdx.x * 128 + threadIdx.x;
    const bool in = i < n;                   // n is a multiple of 32: a warp is all in or all out
    float v = in ? x[i] : 0.f;
    const int64_t c = i % D, off = D - rd;
    const float o = __shfl_xor_sync(0xffffffffu, v, 1);
    if (in && c >= off) {
        const int i0 = (int) ((c - off) & ~int64_t(1));
        float cs, sn;
        yarn_cs((float) (pos0 + i / (H * D)), i0, theta_scale, freq_scale, ext_factor, mscale, corr0, corr1, cs, sn);
        sn = -sn;
        v = (c - off) % 2 == 0 ? __fsub_rn(__fmul_rn(v, cs), __fmul_rn(o, sn)) : __fadd_rn(__fmul_rn(o, sn), __fmul_rn(v, cs));
    }
    const float q = e4m3_sim_warp(v);
    if (in) x[i] = q;
}

// the reference's float power theta_scale = freq_base^(-2 / n_dims), as the correctly rounded float
float theta_scale_of(float freq_base, int64_t n_dims) { return (float) pow((double) freq_base, (double) (-2.0f / (float) n_dims)); }

int check_rope(const char* name, int64_t D, int64_t n_rot) {
    if (D < 2 || D % 16 != 0 || n_rot < 0 || n_rot > D || n_rot % 2) return ns_fail(std::string(name) + ": D a multiple of 16, n_rot even and at most D");
    return 0;
}

}  // namespace

extern "C" {

int ns_q35_qk_norm_rope(ns_gpu* g, const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, const float* w,
                        float eps, int64_t n_rot, float theta, int64_t p0) {
    NS_TRY
    const char* name = "ns_q35_qk_norm_rope";
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (check_rope(name, D, n_rot)) return -1;
    if (!src || !dst || !w || H < 1) return ns_fail(std::string(name) + ": a null buffer");
    norm_rope_kernel<<<(unsigned) ((T * H + 7) / 8), 256, 0, g->compute>>>(src, ss, hs, dst, ds, T, H, D, w, eps, n_rot, theta, p0, nullptr, 0, 0, 0);
    return ns_launched(name);
    NS_CATCH("ns_q35_qk_norm_rope")
}

int ns_q35_qk_norm_rope_pos(ns_gpu* g, const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, const float* w,
                            float eps, int64_t n_rot, float theta, const int32_t* pos, int64_t s0, int64_t s1, int64_t s2) {
    NS_TRY
    const char* name = "ns_q35_qk_norm_rope_pos";
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (check_rope(name, D, n_rot)) return -1;
    if (s0 < 0 || s1 < 0 || s2 < 0 || s0 + s1 + s2 <= 0) return ns_fail(std::string(name) + ": sections");
    if (!src || !dst || !w || !pos || H < 1) return ns_fail(std::string(name) + ": a null buffer");
    norm_rope_kernel<<<(unsigned) ((T * H + 7) / 8), 256, 0, g->compute>>>(src, ss, hs, dst, ds, T, H, D, w, eps, n_rot, theta, 0, pos, s0, s1, s2);
    return ns_launched(name);
    NS_CATCH("ns_q35_qk_norm_rope_pos")
}

int ns_q35_rope(ns_gpu* g, const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, int64_t n_rot, float theta,
                int64_t p0) {
    NS_TRY
    const char* name = "ns_q35_rope";
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (check_rope(name, D, n_rot)) return -1;
    if (!src || !dst || H < 1) return ns_fail(std::string(name) + ": a null buffer");
    norm_rope_kernel<<<(unsigned) ((T * H + 7) / 8), 256, 0, g->compute>>>(src, ss, hs, dst, ds, T, H, D, nullptr, 0.f, n_rot, theta, p0, nullptr, 0, 0, 0);
    return ns_launched(name);
    NS_CATCH("ns_q35_rope")
}

int ns_ds2_rope(ns_gpu* g, float* x, int64_t T, int64_t H, int64_t row, int64_t head, int64_t off, int64_t n_dims, int64_t pos0, float freq_base,
                float freq_scale, float ext_factor, float mscale, float corr0, float corr1, float* out, int64_t out_row, int64_t out_head) {
    NS_TRY
    if (ns_enter(g, "ns_ds2_rope")) return -1;
    if (T <= 0 || H <= 0 || n_dims <= 0) return 0;
    if (n_dims % 2 != 0) return ns_fail("ns_ds2_rope: an even rotated width");
    if (!x || pos0 < 0) return ns_fail("ns_ds2_rope: a null buffer");
    const int64_t total = T * H * (n_dims / 2);
    ds2_rope_kernel<<<(unsigned) std::min<int64_t>(4096, (total + 255) / 256), 256, 0, g->compute>>>(x, T, H, row, head, off, n_dims, pos0,
                                                                                                    theta_scale_of(freq_base, n_dims), freq_scale, ext_factor,
                                                                                                    mscale, corr0, corr1, out, out_row, out_head);
    return ns_launched("ns_ds2_rope");
    NS_CATCH("ns_ds2_rope")
}

int ns_ds2_kv_store(ns_gpu* g, const float* kv, const float* w, float eps, uint16_t* cache, int64_t T, int64_t L, int64_t R, int64_t pos0, float freq_base,
                    float freq_scale, float ext_factor, float mscale, float corr0, float corr1) {
    NS_TRY
    if (ns_enter(g, "ns_ds2_kv_store")) return -1;
    if (T <= 0) return 0;
    if (R % 2 != 0 || R < 0 || L < 1) return ns_fail("ns_ds2_kv_store: an even rotated width");
    if (!kv || !w || !cache || pos0 < 0) return ns_fail("ns_ds2_kv_store: a null buffer");
    ds2_kv_store_kernel<<<(unsigned) T, 256, 0, g->compute>>>(kv, w, eps, (__half*) cache, L, R, pos0, theta_scale_of(freq_base, R > 0 ? R : 2), freq_scale,
                                                             ext_factor, mscale, corr0, corr1);
    return ns_launched("ns_ds2_kv_store");
    NS_CATCH("ns_ds2_kv_store")
}

int ns_ds41_kv_post(ns_gpu* g, float* kv, const float* w, int64_t T, int64_t D, float eps, int64_t rd, int64_t pos0, float freq_base, float freq_scale,
                    float ext_factor, float mscale, float corr0, float corr1, uint16_t* ring, int64_t R) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_kv_post")) return -1;
    if (T <= 0) return 0;
    if (D < 32 || D % 32 != 0 || D > 512 || rd < 0 || rd % 2 != 0 || rd > D) return ns_fail("ns_ds41_kv_post: a row of at most 512 in blocks of 32");
    if (!kv || !w || !ring || R < 1 || pos0 < 0) return ns_fail("ns_ds41_kv_post: a null buffer");
    ds41_kv_post_kernel<<<(unsigned) T, 256, 0, g->compute>>>(kv, w, D, eps, rd, pos0, theta_scale_of(freq_base, rd > 0 ? rd : 2), freq_scale, ext_factor, mscale,
                                                             corr0, corr1, (__half*) ring, R);
    return ns_launched("ns_ds41_kv_post");
    NS_CATCH("ns_ds41_kv_post")
}

int ns_ds41_att_post(ns_gpu* g, float* x, int64_t T, int64_t H, int64_t D, int64_t rd, int64_t pos0, float freq_base, float freq_scale, float ext_factor,
                     float mscale, float corr0, float corr1) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_att_post")) return -1;
    if (T <= 0 || H <= 0) return 0;
    if (D < 32 || D % 32 != 0 || rd < 0 || rd % 2 != 0 || rd > D) return ns_fail("ns_ds41_att_post: rows in blocks of 32");
    if (!x || pos0 < 0) return ns_fail("ns_ds41_att_post: a null buffer");
    const int64_t n = T * H * D;
    ds41_att_post_kernel<<<(unsigned) ((n + 127) / 128), 128, 0, g->compute>>>(x, n, H, D, rd, pos0, theta_scale_of(freq_base, rd > 0 ? rd : 2), freq_scale,
                                                                              ext_factor, mscale, corr0, corr1);
    return ns_launched("ns_ds41_att_post");
    NS_CATCH("ns_ds41_att_post")
}

int ns_b200_qkv_prepare(ns_gpu* g, const float* q, int64_t qs, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hq, int64_t Hkv,
                        int64_t D, const float* wq, const float* wk, float eps, int64_t n_rot, float theta, int64_t p0, int64_t cap, void* q_out, void* kc,
                        void* vc) {
    NS_TRY
    const char* name = "ns_b200_qkv_prepare";
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (check_rope(name, D, n_rot)) return -1;
    if (Hq < 1 || Hkv < 1 || !q || !k || !v || !q_out || !kc || !vc) return ns_fail(std::string(name) + ": a null buffer");
    if (p0 < 0 || p0 + T > cap) return ns_fail(std::string(name) + ": past the cache's capacity");
    qkv_prepare_kernel<<<(unsigned) ((T * (Hq + 2 * Hkv) + 7) / 8), 256, 0, g->compute>>>(q, qs, k, ks, v, vs, T, Hq, Hkv, D, wq, wk, eps, n_rot, theta, p0, cap,
                                                                                          (__half*) q_out, (__half*) kc, (__half*) vc);
    return ns_launched(name);
    NS_CATCH("ns_b200_qkv_prepare")
}

}  // extern "C"

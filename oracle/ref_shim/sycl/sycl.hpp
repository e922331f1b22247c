// A host stand-in for the handful of SYCL names that the reference's simplest kernels use, so that those kernels - the
// reference's own source lines, taken from its checkout at build time - compile with g++ and run on the CPU as a check on
// this repository's oracle. Test infrastructure only. What it covers: sycl::half (IEEE binary16, round to nearest even),
// vec, uint2 / uint4, bit_cast, a few math functions, and queue::parallel_for over range<1>, range<2> and - for kernels
// whose work-items never talk to one another - nd_range<1>, all run as plain loops. Group operations (barriers,
// reductions, sub-group shuffles, local memory) are deliberately absent: a kernel that needs them does not compile here.
#pragma once
#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace sycl {

struct half {
    uint16_t bits = 0;
    half() = default;
    half(float f) : bits((uint16_t) _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC)) {}
    operator float() const { return _cvtsh_ss(bits); }
};
static_assert(sizeof(half) == 2, "binary16");

template <class T, int N>
struct vec {
    T v[N];
    T& operator[](int i) { return v[i]; }
    const T& operator[](int i) const { return v[i]; }
};

struct uint2 {
    uint32_t v[2];
    uint32_t x() const { return v[0]; }
    uint32_t y() const { return v[1]; }
};
struct uint4 {
    uint32_t v[4];
    uint4() = default;
    uint4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) : v{a, b, c, d} {}
    uint32_t x() const { return v[0]; }
    uint32_t y() const { return v[1]; }
    uint32_t z() const { return v[2]; }
    uint32_t w() const { return v[3]; }
};

template <class To, class From>
To bit_cast(const From& f) {
    static_assert(sizeof(To) == sizeof(From), "bit_cast: equal sizes");
    To t;
    std::memcpy(&t, &f, sizeof(To));
    return t;
}

inline float fmax(float a, float b) { return std::fmax(a, b); }
inline float fabs(float a) { return std::fabs(a); }
inline float round(float a) { return std::round(a); }     // halves away from zero, as SYCL's
inline float clamp(float x, float lo, float hi) { return std::fmin(std::fmax(x, lo), hi); }
template <class T>
T min(T a, T b) { return a < b ? a : b; }
template <class T>
T max(T a, T b) { return a > b ? a : b; }

template <int D>
struct range;
template <>
struct range<1> {
    size_t n[1];
    range(size_t a) : n{a} {}
};
template <>
struct range<2> {
    size_t n[2];
    range(size_t a, size_t b) : n{a, b} {}
};
template <int D>
struct id;
template <>
struct id<1> {
    size_t i[1];
    size_t operator[](int k) const { return i[k]; }
    operator size_t() const { return i[0]; }
};
template <>
struct id<2> {
    size_t i[2];
    size_t operator[](int k) const { return i[k]; }
};
template <int D>
struct nd_range;
template <>
struct nd_range<1> {
    size_t global, local;
    nd_range(range<1> g, range<1> l) : global(g.n[0]), local(l.n[0]) {}
};
template <int D>
struct nd_item;
template <>
struct nd_item<1> {
    size_t group, local;
    size_t get_group(int) const { return group; }
    size_t get_local_id(int) const { return local; }
};

struct queue {
    template <class F>
    void parallel_for(range<1> r, F f) {
        for (size_t a = 0; a < r.n[0]; ++a) f(id<1>{{a}});
    }
    template <class F>
    void parallel_for(range<2> r, F f) {
        for (size_t a = 0; a < r.n[0]; ++a)
            for (size_t b = 0; b < r.n[1]; ++b) f(id<2>{{a, b}});
    }
    template <class F>
    void parallel_for(nd_range<1> r, F f) {
        for (size_t g = 0; g < r.global / r.local; ++g)
            for (size_t l = 0; l < r.local; ++l) f(nd_item<1>{g, l});
    }
};

}  // namespace sycl

// A host stand-in for the SYCL names that the reference's kernels use, so that those kernels - the reference's own source
// lines, taken from its checkout at build time - compile with g++ and run on the CPU as a check on this repository's
// oracle. Test infrastructure only. (joint_matrix, for the matrix-unit kernels: sycl/ext/oneapi/matrix/matrix.hpp.)
//
// What it covers: sycl::half (IEEE binary16, round to nearest even), vec, uint2 / uint4, bit_cast, the math functions the
// kernels call, queue::submit / parallel_for over range<1..3> (plain loops) and over nd_range<1> with work-groups:
// local_accessor, group_barrier, sub-groups, reduce_over_group / permute_group_by_xor / broadcasts over a group or a
// sub-group. A work-group runs as one cooperative fiber (ucontext) a work-item, scheduled round-robin by the calling
// thread: a work-item runs until it reaches a collective, and the collective completes when every member has arrived, so
// execution is deterministic. A reduction folds the members' values in the order of their indices.
// What it does not cover: ESIMD, images, USM allocation, events, oneMKL.
// The sub-group size of the next launch is a setting (sycl::detail::sub_group_size()), because g++ ignores the
// [[sycl::reqd_sub_group_size]] attribute the kernels carry.
#pragma once
#include <immintrin.h>
#include <ucontext.h>

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <type_traits>
#include <vector>

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
    T& x() { return v[0]; }
    T& y() { return v[1]; }
    T& z() { return v[2]; }
    T& w() { return v[3]; }
    const T& x() const { return v[0]; }
    const T& y() const { return v[1]; }
    const T& z() const { return v[2]; }
    const T& w() const { return v[3]; }
    template <class U>
    vec<U, N> convert() const {
        vec<U, N> r;
        for (int i = 0; i < N; ++i) r.v[i] = (U) v[i];
        return r;
    }
};
using float2 = vec<float, 2>;
using float4 = vec<float, 4>;

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
inline float fmin(float a, float b) { return std::fmin(a, b); }
inline float fabs(float a) { return std::fabs(a); }
inline float round(float a) { return std::round(a); }     // halves away from zero, as SYCL's
inline float floor(float a) { return std::floor(a); }
inline float exp(float a) { return std::exp(a); }
inline float exp2(float a) { return std::exp2(a); }
inline float log(float a) { return std::log(a); }
inline float sqrt(float a) { return std::sqrt(a); }
inline float rsqrt(float a) { return 1.0f / std::sqrt(a); }
inline float sin(float a) { return std::sin(a); }
inline float cos(float a) { return std::cos(a); }
inline float pow(float a, float b) { return std::pow(a, b); }
inline float tanh(float a) { return std::tanh(a); }
inline float rint(float a) { return std::nearbyint(a); }      // to nearest, halves to even
inline float ldexp(float a, int e) { return std::ldexp(a, e); }
inline float frexp(float a, int* e) { return std::frexp(a, e); }
inline float clamp(float x, float lo, float hi) { return std::fmin(std::fmax(x, lo), hi); }
template <class T>
T min(T a, T b) { return a < b ? a : b; }
template <class T>
T max(T a, T b) { return a > b ? a : b; }

enum class memory_order { relaxed, acquire, release, acq_rel, seq_cst };
enum class memory_scope { work_item, sub_group, work_group, device, system };
namespace access {
enum class address_space { global_space, local_space, private_space, generic_space };
enum class decorated { no, yes };
}  // namespace access
// work-items are fibers of one thread: an atomic is the plain operation
template <class T, memory_order O, memory_scope S, access::address_space A = access::address_space::generic_space>
struct atomic_ref {
    T& r;
    explicit atomic_ref(T& x) : r(x) {}
    T fetch_add(T v) {
        const T old = r;
        r = old + v;
        return old;
    }
    T load() const { return r; }
    void store(T v) { r = v; }
};

template <class T = void>
struct plus {
    T operator()(T a, T b) const { return a + b; }
};
template <class T = void>
struct maximum {
    T operator()(T a, T b) const { return a > b ? a : b; }
};
template <class T = void>
struct minimum {
    T operator()(T a, T b) const { return a < b ? a : b; }
};

template <int D>
struct range {
    size_t n[D];
    template <class... A, class = typename std::enable_if<sizeof...(A) == D && (std::is_arithmetic<A>::value && ...)>::type>
    range(A... a) : n{(size_t) a...} {}
    size_t operator[](int k) const { return n[k]; }
};
template <int D>
struct id {
    size_t i[D];
    size_t operator[](int k) const { return i[k]; }
};
template <>
struct id<1> {
    size_t i[1];
    size_t operator[](int k) const { return i[k]; }
    operator size_t() const { return i[0]; }
};
template <int D>
struct nd_range;
template <>
struct nd_range<1> {
    size_t global, local;
    nd_range(range<1> g, range<1> l) : global(g.n[0]), local(l.n[0]) {}
};

namespace detail {

inline int& sub_group_size() {
    static int s = 16;
    return s;
}
inline int*& sub_group_size_setting() {      // when set: where the size of the next launch is read from
    static int* p = nullptr;
    return p;
}

// a set of work-items that meet in collectives: the work-group, or one of its sub-groups
struct SyncSet {
    int size = 0, arrived = 0;
    unsigned gen = 0;
    std::vector<unsigned char> slots;     // 16 bytes a member: what each contributes to the collective in progress
};

struct Fiber {
    ucontext_t ctx;
    std::vector<unsigned char> stack;
    bool done = false;
};

struct GroupRun {
    ucontext_t sched;
    std::vector<Fiber> fibers;
    int current = -1;
    SyncSet all;
    std::vector<SyncSet> subs;
    int sg = 16;
};
inline GroupRun*& run() {
    static thread_local GroupRun* r = nullptr;
    return r;
}
inline void yield() {
    GroupRun* r = run();
    swapcontext(&r->fibers[r->current].ctx, &r->sched);
}
// returns when every member of the set has called it the same number of times
inline void sync(SyncSet& s) {
    const unsigned mine = s.gen;
    if (++s.arrived == s.size) {
        s.arrived = 0;
        ++s.gen;
    } else {
        while (s.gen == mine) yield();
    }
}
// every member contributes v; f sees all contributions in member order
template <class T, class F>
auto collective(SyncSet& s, int me, T v, F f) -> decltype(f((const T*) nullptr, 0)) {
    static_assert(sizeof(T) <= 16, "collective: values of at most 16 bytes");
    std::memcpy(s.slots.data() + 16 * me, &v, sizeof(T));
    sync(s);
    T all[1024];
    for (int i = 0; i < s.size; ++i) std::memcpy(&all[i], s.slots.data() + 16 * i, sizeof(T));
    auto r = f(all, s.size);
    sync(s);
    return r;
}

template <class K, class Item>
struct Entry {
    const K* kernel;
    Item item;
};
template <class K, class Item>
void trampoline(unsigned lo, unsigned hi) {
    auto* e = reinterpret_cast<Entry<K, Item>*>(((uintptr_t) hi << 32) | (uintptr_t) lo);
    (*e->kernel)(e->item);
    GroupRun* r = run();
    r->fibers[r->current].done = true;
    swapcontext(&r->fibers[r->current].ctx, &r->sched);
}

}  // namespace detail

template <int D>
struct group {
    size_t id;
    size_t get_group_linear_id() const { return id; }
    size_t get_group_id(int) const { return id; }
    size_t get_local_linear_id() const { return (size_t) detail::run()->current; }
    size_t get_local_linear_range() const { return (size_t) detail::run()->all.size; }
};
struct sub_group {
    int lane, index;
    size_t get_local_linear_id() const { return (size_t) lane; }
    size_t get_group_linear_id() const { return (size_t) index; }
    id<1> get_local_id() const { return id<1>{{(size_t) lane}}; }
    size_t get_local_linear_range() const { return (size_t) detail::run()->subs[index].size; }
    size_t get_max_local_range() const { return (size_t) detail::run()->sg; }
};
template <int D>
struct nd_item;
template <>
struct nd_item<1> {
    size_t group_id, local_id, local_range, group_range;
    size_t get_group(int) const { return group_id; }
    group<1> get_group() const { return group<1>{group_id}; }
    size_t get_local_id(int) const { return local_id; }
    size_t get_local_linear_id() const { return local_id; }
    size_t get_local_range(int) const { return local_range; }
    size_t get_group_range(int) const { return group_range; }
    size_t get_global_id(int) const { return group_id * local_range + local_id; }
    size_t get_global_linear_id() const { return group_id * local_range + local_id; }
    sub_group get_sub_group() const {
        const int sg = detail::run()->sg;
        return sub_group{(int) local_id % sg, (int) local_id / sg};
    }
};

namespace detail {
inline SyncSet& set_of(const group<1>&, int& me) {
    GroupRun* r = run();
    me = r->current;
    return r->all;
}
inline SyncSet& set_of(const sub_group& s, int& me) {
    me = s.lane;
    return run()->subs[s.index];
}
}  // namespace detail

template <class G>
void group_barrier(const G& g) {
    int me;
    detail::sync(detail::set_of(g, me));
}
template <class G, class T, class Op>
T reduce_over_group(const G& g, T v, Op op) {
    int me;
    detail::SyncSet& s = detail::set_of(g, me);
    return detail::collective(s, me, v, [&](const T* all, int n) {
        T a = all[0];
        for (int i = 1; i < n; ++i) a = op(a, all[i]);
        return a;
    });
}
template <class G, class T, class Op>
T exclusive_scan_over_group(const G& g, T v, Op op) {
    int me;
    detail::SyncSet& s = detail::set_of(g, me);
    return detail::collective(s, me, v, [&](const T* all, int) {
        T a = T();
        for (int i = 0; i < me; ++i) a = i == 0 ? all[0] : op(a, all[i]);
        return a;
    });
}
template <class T>
T permute_group_by_xor(const sub_group& g, T v, int mask) {
    int me;
    detail::SyncSet& s = detail::set_of(g, me);
    return detail::collective(s, me, v, [&](const T* all, int) { return all[me ^ mask]; });
}
template <class T>
T select_from_group(const sub_group& g, T v, int from) {
    int me;
    detail::SyncSet& s = detail::set_of(g, me);
    return detail::collective(s, me, v, [&](const T* all, int) { return all[from]; });
}
template <class G, class T>
T group_broadcast(const G& g, T v, int from = 0) {
    int me;
    detail::SyncSet& s = detail::set_of(g, me);
    return detail::collective(s, me, v, [&](const T* all, int) { return all[from]; });
}
template <class G>
bool any_of_group(const G& g, bool v) {
    int me;
    detail::SyncSet& s = detail::set_of(g, me);
    return detail::collective(s, me, (int) v, [&](const int* all, int n) {
        bool a = false;
        for (int i = 0; i < n; ++i) a = a || all[i];
        return a;
    });
}

struct handler;
template <class T, int D>
struct local_accessor {
    std::shared_ptr<std::vector<T>> mem;
    local_accessor(range<1> r, handler&) : mem(std::make_shared<std::vector<T>>(r.n[0])) {}
    T& operator[](size_t i) const { return (*mem)[i]; }
    T* get_pointer() const { return mem->data(); }
    struct raw_ptr {
        T* p;
        T* get() const { return p; }
    };
    template <access::decorated>
    raw_ptr get_multi_ptr() const { return raw_ptr{mem->data()}; }
};
// one address space on the host: the cast is the pointer itself
template <access::address_space, access::decorated, class T>
T* address_space_cast(T* p) { return p; }

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
    void parallel_for(range<3> r, F f) {
        for (size_t a = 0; a < r.n[0]; ++a)
            for (size_t b = 0; b < r.n[1]; ++b)
                for (size_t c = 0; c < r.n[2]; ++c) f(id<3>{{a, b, c}});
    }
    // work-groups one after the other, each as cooperative fibers
    template <class F>
    void parallel_for(nd_range<1> r, const F& f) {
        using Item = nd_item<1>;
        const size_t local = r.local, ngroups = r.global / r.local;
        detail::GroupRun run;
        run.sg = std::min<int>(detail::sub_group_size_setting() ? *detail::sub_group_size_setting() : detail::sub_group_size(), (int) local);
        run.fibers.resize(local);
        for (auto& fb : run.fibers) fb.stack.resize(256 * 1024);
        detail::GroupRun* outer = detail::run();
        detail::run() = &run;
        std::vector<detail::Entry<F, Item>> entries(local);
        for (size_t g = 0; g < ngroups; ++g) {
            run.all.size = (int) local;
            run.all.arrived = 0;
            run.all.slots.assign(16 * local, 0);
            const int nsub = (int) ((local + run.sg - 1) / run.sg);
            run.subs.assign(nsub, detail::SyncSet());
            for (int s = 0; s < nsub; ++s) {
                run.subs[s].size = (int) std::min<size_t>(run.sg, local - (size_t) s * run.sg);
                run.subs[s].slots.assign(16 * run.sg, 0);
            }
            for (size_t l = 0; l < local; ++l) {
                entries[l] = {&f, Item{g, l, local, ngroups}};
                detail::Fiber& fb = run.fibers[l];
                fb.done = false;
                getcontext(&fb.ctx);
                fb.ctx.uc_stack.ss_sp = fb.stack.data();
                fb.ctx.uc_stack.ss_size = fb.stack.size();
                fb.ctx.uc_link = &run.sched;
                const uintptr_t p = (uintptr_t) &entries[l];
                makecontext(&fb.ctx, (void (*)()) detail::trampoline<F, Item>, 2, (unsigned) (p & 0xffffffffu), (unsigned) (p >> 32));
            }
            for (size_t left = local; left > 0;) {
                left = 0;
                for (size_t l = 0; l < local; ++l) {
                    if (run.fibers[l].done) continue;
                    run.current = (int) l;
                    swapcontext(&run.sched, &run.fibers[l].ctx);
                    if (!run.fibers[l].done) ++left;
                }
            }
        }
        detail::run() = outer;
    }
    template <class F>
    void submit(F f);
    void wait() {}
    void memset(void* p, int v, size_t n) { std::memset(p, v, n); }
    void memcpy(void* d, const void* s, size_t n) { std::memcpy(d, s, n); }
};

struct handler {
    queue* q;
    template <class R, class F>
    void parallel_for(R r, const F& f) { q->parallel_for(r, f); }
};
template <class F>
void queue::submit(F f) {
    handler h{this};
    f(h);
}

// device memory is the host's
template <class T>
T* malloc_device(size_t n, const queue&) { return static_cast<T*>(std::malloc(n * sizeof(T))); }
inline void free(void* p, const queue&) { std::free(p); }

}  // namespace sycl

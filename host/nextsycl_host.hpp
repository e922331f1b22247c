// nextsycl_host.hpp: a C++ stand-in for the reference's Rust foundation crates above the C ABI - `nextsycl_sys::Api`
// (crates/sys/src/lib.rs:26-60,138-151,181-250: dlopen RTLD_NOW | RTLD_GLOBAL, one function pointer per name, an error
// naming a missing symbol) and `nextsycl_core::{Gpu, DevBuf, Arena}` (crates/core/src/lib.rs:133-156,217-304,446-503:
// bounds-checked buffers, a 256-byte bump arena). Header only; no CUDA types: the library is reached by name alone, as
// an engine reaches it.
#pragma once
#include <dlfcn.h>

#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

namespace nextsycl {

struct ns_gpu;

class Api {
public:
    // NEXTSYCL_LIB when set, else `fallback` (crates/sys/src/lib.rs:138-151)
    explicit Api(const std::string& fallback = "dist/libnextsycl-llm.so") {
        const char* env = std::getenv("NEXTSYCL_LIB");
        path_ = env && *env ? env : fallback;
        handle_ = dlopen(path_.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (!handle_) throw std::runtime_error(path_ + ": " + dlerror());
        last_error = need<const char* (*)()>("ns_last_error");
        gpu_count = need<int (*)()>("ns_gpu_count");
        gpu_open = need<int (*)(int, ns_gpu**)>("ns_gpu_open");
        gpu_close = need<void (*)(ns_gpu*)>("ns_gpu_close");
        alloc = need<int (*)(ns_gpu*, size_t, void**)>("ns_alloc");
        free_ = need<int (*)(ns_gpu*, void*)>("ns_free");
        copy_to = need<int (*)(ns_gpu*, void*, const void*, size_t)>("ns_copy_to");
        copy_from = need<int (*)(ns_gpu*, void*, const void*, size_t)>("ns_copy_from");
        fill = need<int (*)(ns_gpu*, void*, uint8_t, size_t)>("ns_fill");
        sync = need<int (*)(ns_gpu*)>("ns_sync");
    }
    ~Api() {
        if (handle_) dlclose(handle_);
    }
    Api(const Api&) = delete;
    Api& operator=(const Api&) = delete;

    // null when absent (crates/sys/src/lib.rs:246-250)
    void* symbol(const std::string& name) const { return dlsym(handle_, name.c_str()); }
    // the engines' tables: an error naming the missing symbol (llm/qwen35/src/ffi.rs:76-79)
    template <class F>
    F need(const std::string& name) const {
        void* p = symbol(name);
        if (!p) throw std::runtime_error(path_ + ": " + name + " is missing");
        return reinterpret_cast<F>(p);
    }
    void check(int rc, const std::string& what) const {
        if (rc != 0) throw std::runtime_error(what + ": " + last_error());
    }
    const std::string& path() const { return path_; }

    const char* (*last_error)() = nullptr;
    int (*gpu_count)() = nullptr;
    int (*gpu_open)(int, ns_gpu**) = nullptr;
    void (*gpu_close)(ns_gpu*) = nullptr;
    int (*alloc)(ns_gpu*, size_t, void**) = nullptr;
    int (*free_)(ns_gpu*, void*) = nullptr;
    int (*copy_to)(ns_gpu*, void*, const void*, size_t) = nullptr;
    int (*copy_from)(ns_gpu*, void*, const void*, size_t) = nullptr;
    int (*fill)(ns_gpu*, void*, uint8_t, size_t) = nullptr;
    int (*sync)(ns_gpu*) = nullptr;

private:
    std::string path_;
    void* handle_ = nullptr;
};

class Gpu {
public:
    Gpu(const Api& api, int index) : api(api) { api.check(api.gpu_open(index, &raw), "opening the GPU"); }
    ~Gpu() {
        if (raw) api.gpu_close(raw);
    }
    Gpu(const Gpu&) = delete;
    Gpu& operator=(const Gpu&) = delete;
    void sync() const { api.check(api.sync(raw), "waiting for the GPU"); }
    const Api& api;
    ns_gpu* raw = nullptr;
};

// Device memory of one GPU; a view does not own it. `bounds` as crates/core/src/lib.rs:299-304.
class DevBuf {
public:
    DevBuf(const Gpu& gpu, size_t len) : gpu(&gpu), len(len), owned(true) {
        gpu.api.check(gpu.api.alloc(gpu.raw, len, &ptr), "allocating device memory");
    }
    DevBuf(const Gpu& gpu, void* ptr, size_t len) : gpu(&gpu), ptr(ptr), len(len), owned(false) {}
    DevBuf(DevBuf&& o) noexcept : gpu(o.gpu), ptr(o.ptr), len(o.len), owned(o.owned) { o.owned = false; }
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    ~DevBuf() {
        if (owned && ptr) gpu->api.free_(gpu->raw, ptr);
    }
    void bounds(size_t at, size_t n) const {
        if (at > len || n > len - at) throw std::runtime_error("bytes " + std::to_string(at) + ".." + std::to_string(at + n) + " of a " + std::to_string(len) + "-byte buffer");
    }
    DevBuf view(size_t at, size_t n) const {
        bounds(at, n);
        return DevBuf(*gpu, static_cast<uint8_t*>(ptr) + at, n);
    }
    void write(const void* src, size_t n, size_t at = 0) const {
        bounds(at, n);
        gpu->api.check(gpu->api.copy_to(gpu->raw, static_cast<uint8_t*>(ptr) + at, src, n), "copying to the GPU");
    }
    void read(void* dst, size_t n, size_t at = 0) const {
        bounds(at, n);
        gpu->api.check(gpu->api.copy_from(gpu->raw, dst, static_cast<const uint8_t*>(ptr) + at, n), "copying from the GPU");
        gpu->sync();
    }
    const Gpu* gpu;
    void* ptr = nullptr;
    size_t len;
    bool owned;
};

// A bump allocator over one device allocation, 256-byte aligned; requests that do not fit get their own allocation.
class Arena {
public:
    Arena(const Gpu& gpu, size_t bytes) : buf(gpu, bytes) {}
    DevBuf bytes(size_t n) {
        const size_t at = (off + 255) / 256 * 256;
        if (at + n > buf.len) {
            ++spills;
            return DevBuf(*buf.gpu, n);
        }
        off = at + n;
        if (off > peak) peak = off;
        return buf.view(at, n);
    }
    DevBuf f32(size_t n) { return bytes(n * 4); }
    void reset() { off = 0; }
    size_t mark() const { return off; }
    void rewind(size_t m) {
        if (m < off) off = m;
    }
    DevBuf buf;
    size_t off = 0, peak = 0, spills = 0;
};

}  // namespace nextsycl

// Glue between the host API and the C ABI of the sm_100a backend (include/gradc_b200.h).
// This is the seam the reference's dispatcher (gradc/backend/dispatcher.hpp:43-256) and its CUDAMemPool
// (gradc/backend/cuda/memory_pool.hpp:13-103) occupy: one context per device, status codes turned into
// std::runtime_error like the reference's backend errors.  There is no CPU math behind it: an operation asked
// to run on Device(CPU) throws.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

#include "../../include/gradc_b200.h"
#include "base.hpp"

namespace gradc {

inline void gcb_check(int status, const char* what) {
    if (status != GCB_OK) throw std::runtime_error(std::string(what) + ": " + gcb_last_error_string());
}

class Backend {
    std::map<int, gcb_ctx*> m_ctx;
    std::mutex m_mu;
    Backend() = default;

public:
    Backend(const Backend&) = delete;
    static Backend& get() {
        static Backend b;
        return b;
    }
    gcb_ctx* ctx(Device d) {
        if (!d.is_cuda()) throw std::runtime_error("This build computes on CUDA devices only; a CPU tensor reached a device operation.");
        std::lock_guard<std::mutex> g(m_mu);
        auto it = m_ctx.find(d.index);
        if (it != m_ctx.end()) return it->second;
        gcb_ctx* c = nullptr;
        gcb_check(gcb_ctx_create(d.index, &c), "creating the device context");
        m_ctx[d.index] = c;
        return c;
    }
    // Adopt a context made elsewhere (a trainer that shares it with a DP communicator).
    void adopt(int index, gcb_ctx* c) {
        std::lock_guard<std::mutex> g(m_mu);
        m_ctx[index] = c;
    }
    void* allocate(int64_t bytes, Device d) {
        if (d.is_cpu()) {
            void* p = nullptr;
            if (posix_memalign(&p, 64, bytes > 0 ? (size_t)bytes : 64) != 0) throw std::bad_alloc();
            return p;
        }
        void* p = nullptr;
        gcb_check(gcb_arena_alloc(ctx(d), (size_t)bytes, &p), "arena allocation");
        return p;
    }
    void release(void* p, Device d) noexcept {
        if (!p) return;
        if (d.is_cpu()) { std::free(p); return; }
        std::lock_guard<std::mutex> g(m_mu);
        auto it = m_ctx.find(d.index);
        if (it != m_ctx.end()) gcb_arena_free(it->second, p);
    }
    float hwm_gb(Device d) { return (float)gcb_arena_high_water_bytes(ctx(d)) / (1024.f * 1024.f * 1024.f); }
};

// Same entry points as the reference's CUDAMemPool, for code that logs the pool high-water mark.
class CUDAMemPool {
public:
    static CUDAMemPool& get() { static CUDAMemPool p; return p; }
    float get_hwm_gb(Device d = Device(DeviceType::CUDA, 0)) { return Backend::get().hwm_gb(d); }
    void log_hwm() { std::cout << "Current HWM: " << get_hwm_gb() << " GB" << std::endl; }
    void* allocate(int64_t bytes, Device d) { return Backend::get().allocate(bytes, d); }
    void free(void* p, int64_t, Device d) { Backend::get().release(p, d); }
    void clear(Device d) { gcb_check(gcb_arena_release_cached(Backend::get().ctx(d)), "arena release"); }
};

inline cudaStream_t create_stream() {
    cudaStream_t s;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) throw std::runtime_error("cudaStreamCreate failed");
    return s;
}
inline cudaEvent_t create_event() {
    cudaEvent_t e;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) throw std::runtime_error("cudaEventCreate failed");
    return e;
}

}  // namespace gradc

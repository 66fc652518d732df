// gm_host.cpp -- backend loading, the tiered buffer pool and the state helpers.
// See gm_host.hpp for what this layer mirrors.
#include "gm_host.hpp"

#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>

#include <cmath>

namespace gometal {

// ---------------------------------------------------------------------
// Backend
// ---------------------------------------------------------------------
Backend& backend() {
    static Backend b;
    return b;
}

template <class F>
static bool resolve(void* h, const char* name, F* out, std::string* missing) {
    *out = reinterpret_cast<F>(dlsym(h, name));
    if (!*out) { *missing += std::string(missing->empty() ? "" : ", ") + name; return false; }
    return true;
}

std::string Backend::load(const std::string& path) {
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) return std::string("cannot load backend: ") + dlerror();
    std::string missing;
    Backend b;
    b.handle = h;
    resolve(h, "create_cuda_device", &b.create_device, &missing);
    resolve(h, "destroy_cuda_device", &b.destroy_device, &missing);
    resolve(h, "allocate_cuda_buffer", &b.allocate, &missing);
    resolve(h, "deallocate_cuda_buffer", &b.deallocate, &missing);
    resolve(h, "zero_cuda_buffer", &b.zero, &missing);
    resolve(h, "copy_float32_array_to_cuda_buffer", &b.copy_in, &missing);
    resolve(h, "copy_cuda_buffer_to_float32_array", &b.copy_out, &missing);
    resolve(h, "execute_sgd_step_cuda", &b.sgd, &missing);
    resolve(h, "execute_adam_step_cuda", &b.adam, &missing);
    resolve(h, "execute_adam_step_cuda_pooled", &b.adam_pooled, &missing);
    resolve(h, "execute_rmsprop_step_cuda", &b.rmsprop, &missing);
    resolve(h, "execute_adagrad_step_cuda", &b.adagrad, &missing);
    resolve(h, "execute_adadelta_step_cuda", &b.adadelta, &missing);
    resolve(h, "execute_nadam_step_cuda", &b.nadam, &missing);
    resolve(h, "execute_lbfgs_step_cuda", &b.lbfgs, &missing);
    resolve(h, "gm_last_error", &b.last_error, &missing);
    if (!missing.empty()) {
        dlclose(h);
        return "backend " + path + " lacks: " + missing;
    }
    std::string optional;                                   // absent entries only disable mixed precision
    resolve(h, "gm_mixed_create", &b.mixed_create, &optional);
    resolve(h, "gm_mixed_destroy", &b.mixed_destroy, &optional);
    resolve(h, "gm_mixed_step_async", &b.mixed_step, &optional);
    resolve(h, "gm_mixed_get_state", &b.mixed_get_state, &optional);
    resolve(h, "gm_mixed_set_state", &b.mixed_set_state, &optional);
    resolve(h, "gm_mixed_set_clip", &b.mixed_set_clip, &optional);
    resolve(h, "gm_mixed_last_clip", &b.mixed_last_clip, &optional);
    resolve(h, "gm_tensor_list_create", &b.list_create, &optional);
    resolve(h, "gm_tensor_list_destroy", &b.list_destroy, &optional);
    resolve(h, "gm_device_synchronize", &b.device_synchronize, &optional);
    resolve(h, "gm_arena_create", &b.arena_create, &optional);
    resolve(h, "gm_arena_alloc", &b.arena_alloc, &optional);
    resolve(h, "gm_arena_destroy", &b.arena_destroy, &optional);
    *this = b;
    return "";
}

// ---------------------------------------------------------------------
// memory
// ---------------------------------------------------------------------
namespace memory {

const std::vector<int> kDefaultPoolSizes = {1024, 4096, 16384, 65536, 262144, 1048576, 4194304, 16777216, 67108864};

int findPoolSize(int size) {
    for (int p : kDefaultPoolSizes) if (p >= size) return p;
    return size;                           // larger than the largest tier: exact size
}

int calculateMaxPoolSize(int bufferSize) {
    if (bufferSize <= 4096) return 100;
    if (bufferSize <= 65536) return 50;
    if (bufferSize <= 1048576) return 20;
    if (bufferSize <= 16777216) return 20;
    return 15;
}

MemoryManager::~MemoryManager() {
    Backend& b = backend();
    if (arena_) { if (b.arena_destroy) b.arena_destroy(arena_); return; }      // the buffers go with the arena
    if (!b.deallocate) return;
    for (auto& kv : pools_) for (uintptr_t p : kv.second.free) b.deallocate(p);
}

std::string MemoryManager::UseArena(int64_t bytes) {
    Backend& b = backend();
    std::lock_guard<std::mutex> lk(mu_);
    if (arena_) return "this memory manager already has an arena";
    if (!sizes_.empty() || !pools_.empty()) return "the arena must be chosen before the first allocation";
    if (bytes <= 0) return "arena size must be positive";
    if (!b.has_arena()) return "the loaded backend has no arena entries";
    arena_ = b.arena_create(device_, bytes);
    if (!arena_) return std::string("failed to create the arena: ") + (b.last_error ? b.last_error() : "");
    return "";
}

uintptr_t MemoryManager::AllocateBuffer(int size) {
    if (size <= 0) return 0;
    Backend& b = backend();
    if (!b.allocate) return 0;
    const int tier = findPoolSize(size);
    std::lock_guard<std::mutex> lk(mu_);
    Pool& pool = pools_[tier];
    if (pool.size == 0) { pool.size = tier; pool.maxSize = calculateMaxPoolSize(tier); }
    uintptr_t buf = 0;
    if (!pool.free.empty()) {
        buf = pool.free.back();
        pool.free.pop_back();
    } else {
        if (arena_) {
            buf = b.arena_alloc(arena_, tier);                 // 0 when the arena is full
            if (!buf) return 0;
        } else {
            if (pool.allocated >= pool.maxSize) return 0;      // "buffer pool at capacity"
            buf = b.allocate(device_, tier, 1 /* GPU */);
            if (!buf) return 0;
        }
        pool.allocated++;
    }
    sizes_[buf] = tier;
    return buf;
}

void MemoryManager::ReleaseBuffer(uintptr_t buffer) {
    if (!buffer) return;
    Backend& b = backend();
    std::lock_guard<std::mutex> lk(mu_);
    auto it = sizes_.find(buffer);
    // manager.go:305-313 falls back to a 4 MB guess for an untracked buffer and
    // prints a warning; an untracked pointer is simply handed back to the device here.
    if (it == sizes_.end()) { if (!arena_ && b.deallocate) b.deallocate(buffer); return; }
    const int tier = it->second;
    sizes_.erase(it);
    Pool& pool = pools_[tier];
    if (arena_ || (int)pool.free.size() < pool.maxSize) {     // arena memory can only be reused, not returned
        pool.free.push_back(buffer);
    } else {
        if (b.deallocate) b.deallocate(buffer);
        pool.allocated--;
    }
}

std::map<int, PoolStats> MemoryManager::Stats() {
    std::lock_guard<std::mutex> lk(mu_);
    std::map<int, PoolStats> out;
    for (auto& kv : pools_) {
        PoolStats s;
        s.available = (int)kv.second.free.size();
        s.allocated = kv.second.allocated;
        s.maxSize = kv.second.maxSize;
        out[kv.first] = s;
    }
    return out;
}

int MemoryManager::trackedSize(uintptr_t buffer) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = sizes_.find(buffer);
    return it == sizes_.end() ? -1 : it->second;
}

}  // namespace memory

// ---------------------------------------------------------------------
// state helpers
// ---------------------------------------------------------------------
namespace optimizer {

int extractBufferIndex(const std::string& name) {
    const size_t us = name.rfind('_');
    if (us == std::string::npos) return -1;
    const std::string tail = name.substr(us + 1);
    // fmt.Sscanf("%d"): optional sign, then at least one digit; trailing text is ignored
    size_t i = 0;
    bool neg = false;
    if (i < tail.size() && (tail[i] == '+' || tail[i] == '-')) { neg = tail[i] == '-'; ++i; }
    if (i >= tail.size() || tail[i] < '0' || tail[i] > '9') return -1;
    long v = 0;
    while (i < tail.size() && tail[i] >= '0' && tail[i] <= '9') { v = v * 10 + (tail[i] - '0'); ++i; }
    return (int)(neg ? -v : v);
}

float pow(float x, float y) {
    if (y == 0.0f) return 1.0f;
    if (y == 1.0f) return x;
    float result = 1.0f;
    for (int i = 0; i < (int)y; ++i) result *= x;
    return result;
}

std::string validateStateType(const std::string& optimizerType, const OptimizerState& state) {
    if (state.Type != optimizerType)
        return "state type mismatch: expected " + optimizerType + ", got " + state.Type;
    return "";
}

// JSON decoding hands every number to Go as float64, so only that kind is
// accepted (state_helpers.go:52-74); anything else yields the default.
float extractFloat32Param(const std::map<std::string, Param>& p, const std::string& key, float def) {
    auto it = p.find(key);
    if (it != p.end() && it->second.kind == Param::Float64) return (float)it->second.f;
    return def;
}

bool extractBoolParam(const std::map<std::string, Param>& p, const std::string& key, bool def) {
    auto it = p.find(key);
    if (it != p.end() && it->second.kind == Param::Bool) return it->second.b;
    return def;
}

uint64_t extractUint64Param(const std::map<std::string, Param>& p, const std::string& key, uint64_t def) {
    auto it = p.find(key);
    if (it != p.end() && it->second.kind == Param::Float64) return (uint64_t)it->second.f;
    return def;
}

int calculateTensorSize(const std::vector<int>& shape) {
    int size = 1;
    for (int d : shape) size *= d;
    return size;
}

}  // namespace optimizer
}  // namespace gometal

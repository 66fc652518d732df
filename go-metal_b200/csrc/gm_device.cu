// gm_device.cu -- device handles, the buffer registry, cudaMalloc-backed
// buffers and arenas, host<->device copies and the fp32<->fp16 conversion.
//
// Replaces cgo_bridge/bridge_memory.m (allocate/zero/copy/convert, :4-55,
// :163-188, :221-423) and the device/queue calls of cgo_bridge/bridge_device.m
// for the optimizer-step path.
#include <cuda_fp16.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <thread>

#include <set>

#include "gm_internal.h"

namespace gm {

// ------------------------------------------------------------------
// errors
// ------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return GM_ERR_CUDA;
}

// ------------------------------------------------------------------
// live-handle and buffer registries
// ------------------------------------------------------------------
struct BufInfo { int64_t bytes; int ordinal; bool owned; };
struct Arena {
    uintptr_t base = 0; int64_t cap = 0; int64_t used = 0; int ordinal = 0;
};

static std::mutex g_mu;
static std::set<Device*> g_devices;
static std::set<TensorList*> g_lists;
static std::set<Arena*> g_arenas;
static std::unordered_map<uintptr_t, BufInfo> g_bufs;

Device* as_device(uintptr_t h) {
    if (h == 0) { set_error("device handle is nil"); return nullptr; }
    std::lock_guard<std::mutex> lk(g_mu);
    Device* d = reinterpret_cast<Device*>(h);
    if (!g_devices.count(d)) { set_error("handle %p is not a live device", (void*)h); return nullptr; }
    return d;
}

TensorList* as_list(uintptr_t h) {
    if (h == 0) { set_error("tensor list handle is nil"); return nullptr; }
    std::lock_guard<std::mutex> lk(g_mu);
    TensorList* l = reinterpret_cast<TensorList*>(h);
    if (!g_lists.count(l)) { set_error("handle %p is not a live tensor list", (void*)h); return nullptr; }
    return l;
}

static Arena* as_arena(uintptr_t h) {
    if (h == 0) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    Arena* a = reinterpret_cast<Arena*>(h);
    return g_arenas.count(a) ? a : nullptr;
}

// Bumped by every allocation and release the library performs; a cached tensor
// list validated under the current value needs no second look at the registry.
static std::atomic<uint64_t> g_registry_gen{1};

int64_t registered_size(uintptr_t p) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_bufs.find(p);
    return it == g_bufs.end() ? -1 : it->second.bytes;
}

uint64_t registry_generation() { return g_registry_gen.load(std::memory_order_acquire); }

bool buffer_holds(uintptr_t p, int64_t need, const char* what) {
    const int64_t have = registered_size(p);
    if (have >= 0 && have < need) {
        set_error("%s: buffer holds %lld bytes, the call needs %lld", what, (long long)have, (long long)need);
        return false;
    }
    return true;
}

int registered_ordinal(uintptr_t p) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_bufs.find(p);
    return it == g_bufs.end() ? -1 : it->second.ordinal;
}

static int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

static uintptr_t alloc_registered(Device* d, int64_t bytes) {
    if (bytes <= 0) { set_error("allocation size %lld is not positive", (long long)bytes); return 0; }
    DeviceGuard g(d);
    void* p = nullptr;
    // cudaMalloc returns 256-byte aligned addresses; the reservation is rounded
    // up to the same granule so vector tails never touch a neighbour.
    cudaError_t e = cudaMalloc(&p, (size_t)round_up(bytes, 256));
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc"); cudaGetLastError(); return 0; }
    std::lock_guard<std::mutex> lk(g_mu);
    g_bufs[(uintptr_t)p] = BufInfo{bytes, d->ordinal, true};
    g_registry_gen.fetch_add(1, std::memory_order_release);
    return (uintptr_t)p;
}

static void free_registered(uintptr_t p) {
    if (!p) return;
    BufInfo info{};
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_bufs.find(p);
        if (it == g_bufs.end() || !it->second.owned) return;   // not ours: leave it alone
        info = it->second;
        g_bufs.erase(it);
        g_registry_gen.fetch_add(1, std::memory_order_release);
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != info.ordinal) cudaSetDevice(info.ordinal);
    cudaFree((void*)p);
    if (prev != info.ordinal && prev >= 0) cudaSetDevice(prev);
}

// ------------------------------------------------------------------
// devices
// ------------------------------------------------------------------
static Device* make_device(int ordinal) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0) {
        cudaGetLastError();
        set_error("no CUDA device is visible (%s); this library has no CPU path",
                  e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
        return nullptr;
    }
    if (ordinal < 0 || ordinal >= count) { set_error("device ordinal %d out of range [0,%d)", ordinal, count); return nullptr; }
    e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) { cuda_fail(e, "cudaSetDevice"); return nullptr; }
    Device* d = new Device();
    d->ordinal = ordinal;
    cudaDeviceGetAttribute(&d->sm_count, cudaDevAttrMultiProcessorCount, ordinal);
    if (const char* e2 = getenv("GOMETAL_GRID_WAVES")) d->grid_waves = atoi(e2);
    if (const char* e3 = getenv("GOMETAL_LBFGS_WAVES")) d->lbfgs_waves = atoi(e3);
    if (const char* e4 = getenv("GOMETAL_LBFGS_KEEP_DIR")) d->lbfgs_keep_dir = atoi(e4);
    if (const char* e9 = getenv("GOMETAL_LBFGS_OVERLAP")) d->lbfgs_overlap = atoi(e9);
    if (const char* e = getenv("GOMETAL_LBFGS_PREWAIT")) d->lbfgs_prewait = atoi(e);
    if (const char* e = getenv("GOMETAL_LBFGS_DEFER")) d->lbfgs_defer = atoi(e) != 0;
    if (const char* e5 = getenv("GOMETAL_MIXED_KEEP_G")) d->mixed_keep_g = atoi(e5);
    if (const char* e6 = getenv("GOMETAL_MIXED_OVERLAP")) d->mixed_overlap = atoi(e6);
    if (const char* e8 = getenv("GOMETAL_MIXED_VARIANT")) d->mixed_variant = atoi(e8);
    if (const char* e = getenv("GOMETAL_MIXED_FASTDIV")) d->mixed_fastdiv = atoi(e);
    if (const char* e = getenv("GOMETAL_MIXED_PF")) d->mixed_pf = atoi(e);
    if (const char* e = getenv("GOMETAL_MIXED_RING")) d->mixed_ring = atoi(e);
    if (const char* e = getenv("GOMETAL_LBFGS_COOP")) d->lbfgs_coop = atoi(e);
    if (const char* e = getenv("GOMETAL_BARRIER_BUDGET_CYCLES")) { const long long v = atoll(e); if (v > 0) d->barrier_budget_cycles = v; }
    if (const char* e7 = getenv("GOMETAL_MIXED_CHECK_PERSISTENT")) d->mixed_check_persistent = atoi(e7);
    if (const char* e3 = getenv("GOMETAL_CHUNK_ELEMS")) d->chunk_elems = atoi(e3);
    // A blocking stream on purpose: the synchronous copies of the drop-in ABI
    // (cudaMemcpy/cudaMemset on the legacy default stream) may return before a
    // small transfer has landed, and only a blocking stream is ordered after
    // them.  A non-blocking stream let a kernel read a table a few hundred
    // bytes long before its upload had completed.
    e = cudaStreamCreateWithFlags(&d->stream, cudaStreamDefault);
    if (e != cudaSuccess) { cuda_fail(e, "cudaStreamCreate"); delete d; return nullptr; }
    cudaEventCreate(&d->ev_start);
    cudaEventCreate(&d->ev_stop);
    e = cudaMalloc((void**)&d->ticket, 256);
    if (e == cudaSuccess) e = cudaMalloc((void**)&d->scalars, 4096);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(scratch)"); delete d; return nullptr; }
    cudaMemset(d->ticket, 0, 256);
    cudaMemset(d->scalars, 0, 4096);
    std::lock_guard<std::mutex> lk(g_mu);
    g_devices.insert(d);
    return d;
}

int ensure_partials(Device* d, int64_t count) {
    if (count <= d->partials_cap) return GM_OK;
    DeviceGuard g(d);
    int64_t cap = round_up(count, 4096);
    if (d->partials) { cudaStreamSynchronize(d->stream); cudaFree(d->partials); d->partials = nullptr; d->partials_cap = 0; }
    GM_CUDA_CHECK(cudaMalloc((void**)&d->partials, (size_t)cap * sizeof(float)));
    d->partials_cap = cap;
    return GM_OK;
}

int ensure_tagged(Device* d, int64_t count) {
    if (count <= d->tagged_cap) return GM_OK;
    DeviceGuard g(d);
    int64_t cap = round_up(count, 4096);
    if (d->tagged) { cudaStreamSynchronize(d->stream); cudaFree(d->tagged); d->tagged = nullptr; d->tagged_cap = 0; }
    GM_CUDA_CHECK(cudaMalloc((void**)&d->tagged, (size_t)cap * sizeof(unsigned long long)));
    GM_CUDA_CHECK(cudaMemset(d->tagged, 0, (size_t)cap * sizeof(unsigned long long)));   // epoch 0 is never waited for
    d->tagged_cap = cap;
    return GM_OK;
}

int launch_grid(Device* d, const void* kernel, int threads, int64_t work_items) {
    // grid_waves == 0: one CTA per chunk.  Measured on B200, a large grid of
    // short-lived CTAs streams about 15 % faster than resident CTAs looping
    // over chunks (the block scheduler keeps more loads in flight).
    // grid_waves > 0: that many waves of resident CTAs, each looping.
    int64_t grid = work_items;
    if (d->grid_waves > 0) {
        int per_sm = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0);
        if (e != cudaSuccess || per_sm < 1) { cudaGetLastError(); per_sm = 1; }
        grid = (int64_t)per_sm * d->sm_count * d->grid_waves;
        if (grid > work_items) grid = work_items;
    }
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    if (grid < 1) grid = 1;
    return (int)grid;
}

// ------------------------------------------------------------------
// tensor lists
// ------------------------------------------------------------------
static uint64_t fnv1a(uint64_t h, const void* data, size_t n) {
    const unsigned char* p = (const unsigned char*)data;
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
    return h;
}

void free_list(TensorList* l) {
    if (!l) return;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_lists.erase(l);
    }
    if (l->blob && l->dev) {
        DeviceGuard g(l->dev);
        cudaFree(l->blob);
    }
    delete l;
}

TensorList* build_list(Device* d, int ns, int nt, const uintptr_t* const* sp, const int64_t* numel,
                       const int* elem_bytes, bool cache, int* err) {
    *err = GM_OK;
    if (ns < 1 || ns > kMaxStreams) { set_error("stream count %d outside [1,%d]", ns, kMaxStreams); *err = GM_ERR_BAD_ARG; return nullptr; }
    if (nt < 1) { set_error("tensor count %d is not positive", nt); *err = GM_ERR_BAD_ARG; return nullptr; }
    const uint64_t gen = g_registry_gen.load(std::memory_order_acquire);
    auto validate = [&]() -> bool {
        for (int t = 0; t < nt; ++t) {
            if (numel[t] <= 0) { set_error("tensor %d has %lld elements", t, (long long)numel[t]); *err = GM_ERR_BAD_SIZE; return false; }
            for (int s = 0; s < ns; ++s) {
                uintptr_t p = sp[s][t];
                if (p == 0) { set_error("stream %d tensor %d is a nil buffer", s, t); *err = GM_ERR_NIL_BUFFER; return false; }
                int eb = elem_bytes ? elem_bytes[s] : 4;
                if (p % (uintptr_t)eb) { set_error("stream %d tensor %d address is not %d-byte aligned", s, t, eb); *err = GM_ERR_BAD_ARG; return false; }
                int64_t have = registered_size(p);
                if (have >= 0 && have < numel[t] * eb) {
                    set_error("stream %d tensor %d: buffer holds %lld bytes, step needs %lld", s, t,
                              (long long)have, (long long)(numel[t] * eb));
                    *err = GM_ERR_BAD_SIZE;
                    return false;
                }
            }
        }
        return true;
    };
    uint64_t key = 0xcbf29ce484222325ull;
    key = fnv1a(key, &ns, sizeof(ns));
    key = fnv1a(key, &nt, sizeof(nt));
    for (int s = 0; s < ns; ++s) {
        key = fnv1a(key, sp[s], sizeof(uintptr_t) * nt);
        int eb = elem_bytes ? elem_bytes[s] : 4;
        key = fnv1a(key, &eb, sizeof(eb));
    }
    key = fnv1a(key, numel, sizeof(int64_t) * nt);
    if (key == 0) key = 1;
    if (cache) {
        std::lock_guard<std::mutex> lk(d->mu);
        auto it = d->list_cache.find(key);
        if (it != d->list_cache.end()) {
            TensorList* l = it->second;
            bool same = (int)l->ptrs.size() == ns && (int)l->numel.size() == nt;
            for (int s = 0; same && s < ns; ++s)
                same = memcmp(l->ptrs[s].data(), sp[s], sizeof(uintptr_t) * nt) == 0
                       && l->elem_bytes[s] == (elem_bytes ? elem_bytes[s] : 4);
            if (same) same = memcmp(l->numel.data(), numel, sizeof(int64_t) * nt) == 0;
            if (same) {
                // pointers and sizes are those of the cached list; the registry is consulted
                // again only if something was allocated or released since it was last checked
                if (l->validated_gen != gen) {
                    if (!validate()) return nullptr;
                    l->validated_gen = gen;
                }
                return l;
            }
            d->list_cache.erase(it);   // hash collision: rebuild below
            free_list(l);
        }
    }

    if (!validate()) return nullptr;

    TensorList* l = new TensorList();
    l->dev = d;
    l->validated_gen = gen;
    l->numel.assign(numel, numel + nt);
    l->ptrs.resize(ns);
    for (int s = 0; s < ns; ++s) {
        l->ptrs[s].assign(sp[s], sp[s] + nt);
        l->elem_bytes[s] = elem_bytes ? elem_bytes[s] : 4;
    }
    int64_t total = 0;
    for (int t = 0; t < nt; ++t) total += numel[t];
    l->total = total;

    // Chunk = the elements one CTA pass covers (256 threads x 8 elements).
    // With one CTA per chunk this is also the CTA's whole job.
    const int tile = kApplyThreads * 8;
    int chunk = 2 * tile;                               // 4096: best of a 2048..65536 sweep on B200 (fp32 lists)
    for (int s = 0; s < ns; ++s) if (l->elem_bytes[s] == 2) chunk = 4 * tile;   // fp16 streams: 8192 measured best
    // Small lists are latency-bound, not bandwidth-bound: one pass per CTA (1,024
    // elements) and more CTAs shorten the chain of dependent loads a CTA walks
    // (MLP-sized list: 6 us -> 3 us per launch).
    if (chunk == 2 * tile) {
        const int64_t one_wave = (int64_t)d->sm_count * 5 * 1024;     // every chunk resident at once
        if (total <= one_wave) chunk = 1024;
        else if (total <= (1LL << 27)) chunk = 2048;                  // measured: 1-3 % ahead of 4,096 from 2^24 to 2^27 elements,
                                                                      // level at 2^28, 1.5 % behind at 2^30
    }
    if (chunk == 4 * tile) {
        // Lists with fp16 streams (the mixed-precision update runs 4 CTAs per SM): between 6,144 and
        // 8,192 elements per chunk take the size whose last wave of CTAs is the fuller one (25.2 M
        // parameters in 48 tensors: 6.97 waves and 134.2 us against 5.24 waves and 135.5 us).
        const double resident = 4.0 * d->sm_count;
        auto last_wave = [&](int ch) {
            long long chunks = 0;
            for (int t = 0; t < nt; ++t) chunks += (numel[t] + ch - 1) / ch;
            const double waves = (double)chunks / resident;
            const double frac = waves - (double)(long long)waves;
            return frac == 0.0 ? 1.0 : frac;
        };
        if (total > (int64_t)resident * 4 * tile && last_wave(3 * tile) > last_wave(4 * tile) + 0.15) chunk = 3 * tile;
    }
    if (d->chunk_elems > 0) chunk = (d->chunk_elems + tile - 1) / tile * tile;

    // head[t]: number of leading elements to peel so that every stream of the
    // tensor sits on a 16-byte boundary; the vector tile is 8 elements for
    // lists with 2-byte streams so one 16-byte access covers it.
    std::vector<int> head(nt), prefix(nt + 1), dot_prefix(nt + 1);
    dot_prefix[0] = 0;
    int lanes = 4;
    for (int s = 0; s < ns; ++s) if (l->elem_bytes[s] == 2) lanes = 8;
    prefix[0] = 0;
    for (int t = 0; t < nt; ++t) {
        int h = -1;
        for (int cand = 0; cand < lanes && h < 0; ++cand) {
            bool ok = true;
            for (int s = 0; s < ns && ok; ++s)
                ok = ((sp[s][t] + (uintptr_t)cand * l->elem_bytes[s]) % kVecBytes) == 0;
            if (ok) h = cand;
        }
        if (h >= 0 && h > numel[t]) h = (int)numel[t];
        head[t] = h;
        int64_t body = numel[t] - (h > 0 ? h : 0);
        int64_t nchunks = body > 0 ? (body + chunk - 1) / chunk : 1;
        if ((int64_t)prefix[t] + nchunks > 0x7fffffff) { set_error("tensor list too large"); *err = GM_ERR_BAD_SIZE; delete l; return nullptr; }
        prefix[t + 1] = prefix[t] + (int)nchunks;
        const int64_t ndot = (numel[t] + kDotChunkElems - 1) / kDotChunkElems;
        if ((int64_t)dot_prefix[t] + ndot > 0x7fffffff) { set_error("tensor list too large"); *err = GM_ERR_BAD_SIZE; delete l; return nullptr; }
        dot_prefix[t + 1] = dot_prefix[t] + (int)ndot;
    }

    const int num_chunks = prefix[nt];
    size_t off_ptrs = 0;
    size_t off_numel = off_ptrs + sizeof(unsigned long long) * ns * nt;
    size_t off_rec = off_numel + sizeof(long long) * nt;
    size_t off_head = off_rec + sizeof(int2) * (size_t)num_chunks;
    size_t off_prefix = off_head + sizeof(int) * nt;
    size_t off_dot = off_prefix + sizeof(int) * (nt + 1);
    size_t bytes = off_dot + sizeof(int) * (nt + 1);
    std::vector<unsigned char> host(bytes);
    for (int s = 0; s < ns; ++s)
        for (int t = 0; t < nt; ++t)
            ((unsigned long long*)(host.data() + off_ptrs))[(size_t)s * nt + t] = (unsigned long long)sp[s][t];
    for (int t = 0; t < nt; ++t) ((long long*)(host.data() + off_numel))[t] = numel[t];
    {
        int2* rec = (int2*)(host.data() + off_rec);
        for (int t = 0; t < nt; ++t)
            for (int c = prefix[t]; c < prefix[t + 1]; ++c) rec[c] = make_int2(t, c - prefix[t]);
    }
    memcpy(host.data() + off_head, head.data(), sizeof(int) * nt);
    memcpy(host.data() + off_prefix, prefix.data(), sizeof(int) * (nt + 1));
    memcpy(host.data() + off_dot, dot_prefix.data(), sizeof(int) * (nt + 1));

    {
        DeviceGuard g(d);
        cudaError_t e = cudaMalloc(&l->blob, round_up((int64_t)bytes, 256));
        if (e == cudaSuccess) e = cudaMemcpy(l->blob, host.data(), bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { *err = cuda_fail(e, "tensor list upload"); cudaGetLastError(); if (l->blob) cudaFree(l->blob); delete l; return nullptr; }
    }
    unsigned char* b = (unsigned char*)l->blob;
    l->dl.ptrs = (const unsigned long long*)(b + off_ptrs);
    l->dl.numel = (const long long*)(b + off_numel);
    l->dl.head = (const int*)(b + off_head);
    l->dl.chunk_prefix = (const int*)(b + off_prefix);
    l->dl.chunk_rec = (const int2*)(b + off_rec);
    l->dl.dot_prefix = (const int*)(b + off_dot);
    l->dl.num_dot_chunks = dot_prefix[nt];
    l->chunk_prefix = prefix;
    l->head = head;
    l->dl.num_tensors = nt;
    l->dl.num_chunks = prefix[nt];
    l->dl.chunk_elems = chunk;
    l->dl.num_streams = ns;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_lists.insert(l);
    }
    if (cache) {
        std::lock_guard<std::mutex> lk(d->mu);
        if (d->list_cache.size() >= 64) {
            // Bounded: forget everything, rebuild on demand.  The forgotten lists are parked, not
            // freed: a caller may still hold one between its lookup and its launch.  What the
            // eviction before this one parked is freed now, once the stream has drained.
            cudaStreamSynchronize(d->stream);
            for (TensorList* o : d->retired_lists) free_list(o);
            d->retired_lists.clear();
            for (auto& kv : d->list_cache) d->retired_lists.push_back(kv.second);
            d->list_cache.clear();
        }
        l->key = key;
        auto prev = d->list_cache.find(key);
        // another thread cached the same list meanwhile: its kernels may still read that
        // descriptor, so it is parked until the device handle goes away
        if (prev != d->list_cache.end()) d->parked_lists.push_back(prev->second);
        d->list_cache[key] = l;
    }
    return l;
}

// ------------------------------------------------------------------
// fp32 <-> fp16 conversion (bridge_memory.m:362-376)
// ------------------------------------------------------------------
__global__ void convert_f32_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __float2half_rn(src[i]);
}

__global__ void convert_f16_to_f32_kernel(const __half* __restrict__ src, float* __restrict__ dst, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __half2float(src[i]);
}

// Both buffers on a 16-byte boundary: eight elements per thread per pass (two 16-byte
// fp32 accesses, one 16-byte fp16 access), streamed; the last n % 8 elements one by one.
__global__ void __launch_bounds__(256)
convert_f32_to_f16_vec_kernel(const float* __restrict__ src, __half* __restrict__ dst, long long n) {
    const long long n8 = n >> 3;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const float4* s4 = reinterpret_cast<const float4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const float4 a = __ldcs(s4 + 2 * i), b = __ldcs(s4 + 2 * i + 1);
        const __half2 h0 = __halves2half2(__float2half_rn(a.x), __float2half_rn(a.y));
        const __half2 h1 = __halves2half2(__float2half_rn(a.z), __float2half_rn(a.w));
        const __half2 h2 = __halves2half2(__float2half_rn(b.x), __float2half_rn(b.y));
        const __half2 h3 = __halves2half2(__float2half_rn(b.z), __float2half_rn(b.w));
        uint4 o;
        o.x = *reinterpret_cast<const unsigned*>(&h0); o.y = *reinterpret_cast<const unsigned*>(&h1);
        o.z = *reinterpret_cast<const unsigned*>(&h2); o.w = *reinterpret_cast<const unsigned*>(&h3);
        __stcs(d4 + i, o);
    }
    const long long t = (n8 << 3) + (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) dst[t] = __float2half_rn(src[t]);
}

__global__ void __launch_bounds__(256)
convert_f16_to_f32_vec_kernel(const __half* __restrict__ src, float* __restrict__ dst, long long n) {
    const long long n8 = n >> 3;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 v = __ldcs(s4 + i);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        __stcs(d4 + 2 * i, make_float4(f0.x, f0.y, f1.x, f1.y));
        __stcs(d4 + 2 * i + 1, make_float4(f2.x, f2.y, f3.x, f3.y));
    }
    const long long t = (n8 << 3) + (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) dst[t] = __half2float(src[t]);
}

}  // namespace gm

using namespace gm;

// ======================================================================
// C ABI
// ======================================================================
extern "C" {

const char* gm_last_error(void) { return g_err; }
const char* gm_version(void) { return "gometal_cuda 0.1 (sm_100a)"; }

uintptr_t gm_device_create(int ordinal) { return (uintptr_t)make_device(ordinal); }

uintptr_t create_cuda_device(void) {
    int ordinal = 0;
    const char* e = getenv("GOMETAL_CUDA_DEVICE");
    if (!e || !*e) e = getenv("LOCAL_RANK");
    if (e && *e) ordinal = atoi(e);
    return (uintptr_t)make_device(ordinal);
}

void destroy_cuda_device(uintptr_t h) {
    Device* d = as_device(h);
    if (!d) return;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_devices.erase(d);
    }
    DeviceGuard g(d);
    cudaStreamSynchronize(d->stream);
    std::vector<TensorList*> lists;
    for (auto& kv : d->list_cache) lists.push_back(kv.second);
    d->list_cache.clear();
    for (TensorList* l : d->parked_lists) lists.push_back(l);
    d->parked_lists.clear();
    for (TensorList* l : d->retired_lists) lists.push_back(l);
    d->retired_lists.clear();
    for (TensorList* l : lists) free_list(l);
    lbfgs_release_device(d);
    if (d->partials) cudaFree(d->partials);
    if (d->tagged) cudaFree(d->tagged);
    if (d->ticket) cudaFree(d->ticket);
    if (d->scalars) cudaFree(d->scalars);
    cudaEventDestroy(d->ev_start);
    cudaEventDestroy(d->ev_stop);
    for (cudaEvent_t e : d->slice_events) cudaEventDestroy(e);
    if (d->h2d_stream) cudaStreamDestroy(d->h2d_stream);
    if (d->d2h_stream) cudaStreamDestroy(d->d2h_stream);
    cudaStreamDestroy(d->stream);
    delete d;
}

uintptr_t create_command_queue(uintptr_t h) {
    Device* d = as_device(h);
    return d ? (uintptr_t)d->stream : 0;
}

void release_command_queue(uintptr_t) {}   // the stream belongs to the device handle

int gm_device_ordinal(uintptr_t h) { Device* d = as_device(h); return d ? d->ordinal : GM_ERR_NIL_DEVICE; }
int gm_device_sm_count(uintptr_t h) { Device* d = as_device(h); return d ? d->sm_count : GM_ERR_NIL_DEVICE; }
uintptr_t gm_device_stream(uintptr_t h) { Device* d = as_device(h); return d ? (uintptr_t)d->stream : 0; }
int64_t gm_device_launch_count(uintptr_t h) { Device* d = as_device(h); return d ? d->launches : -1; }

int gm_device_synchronize(uintptr_t h) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return GM_OK;
}

// Waits for the device's stream, but no longer than timeout_ms: polls the stream instead
// of blocking in the driver, so a step that never completes (a peer that never entered
// its collective) gives the caller GM_ERR_TIMEOUT and the choice of what to do next.
int gm_device_synchronize_timeout(uintptr_t h, int timeout_ms) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (timeout_ms < 0) { set_error("timeout %d ms is negative", timeout_ms); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    unsigned spins = 0;
    for (;;) {
        const cudaError_t e = cudaStreamQuery(d->stream);
        if (e == cudaSuccess) return GM_OK;
        if (e != cudaErrorNotReady) return cuda_fail(e, "cudaStreamQuery");
        if (std::chrono::steady_clock::now() >= deadline) {
            set_error("the device stream did not drain within %d ms", timeout_ms);
            return GM_ERR_TIMEOUT;
        }
        if (++spins > 200) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

// Launch-strategy switches of a device handle (the GOMETAL_* environment variables set
// the same fields when the handle is created).  Every setting computes the same bits.
int gm_device_set_tuning(uintptr_t h, const char* name, long long value) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!name) { set_error("name is nil"); return GM_ERR_BAD_ARG; }
    const std::string n(name);
    if (n == "mixed_ring") { if (value < 0 || value > 2) { set_error("mixed_ring is 0, 1 or 2"); return GM_ERR_BAD_ARG; } d->mixed_ring = (int)value; }
    else if (n == "mixed_fastdiv") d->mixed_fastdiv = value ? 1 : 0;
    else if (n == "mixed_pf") d->mixed_pf = value ? 1 : 0;
    else if (n == "mixed_variant") d->mixed_variant = value ? 1 : 0;
    else if (n == "lbfgs_defer") d->lbfgs_defer = value != 0;
    else if (n == "lbfgs_prewait") { if (value < 0 || value > 2) { set_error("lbfgs_prewait is 0, 1 or 2"); return GM_ERR_BAD_ARG; } d->lbfgs_prewait = (int)value; }
    else if (n == "lbfgs_coop") { if (value < 0 || value > 2) { set_error("lbfgs_coop is 0, 1 or 2"); return GM_ERR_BAD_ARG; } d->lbfgs_coop = (int)value; }
    else if (n == "barrier_budget_cycles") { if (value <= 0) { set_error("the budget must be positive"); return GM_ERR_BAD_ARG; } d->barrier_budget_cycles = value; }
    else { set_error("unknown tuning name '%s'", name); return GM_ERR_BAD_ARG; }
    return GM_OK;
}

long long gm_device_get_tuning(uintptr_t h, const char* name) {
    Device* d = as_device(h);
    if (!d || !name) return -1;
    const std::string n(name);
    if (n == "mixed_ring") return d->mixed_ring;
    if (n == "mixed_fastdiv") return d->mixed_fastdiv;
    if (n == "mixed_pf") return d->mixed_pf;
    if (n == "mixed_variant") return d->mixed_variant;
    if (n == "lbfgs_coop") return d->lbfgs_coop;
    if (n == "lbfgs_prewait") return d->lbfgs_prewait;
    if (n == "lbfgs_defer") return d->lbfgs_defer;
    if (n == "barrier_budget_cycles") return d->barrier_budget_cycles;
    set_error("unknown tuning name '%s'", name);
    return -1;
}

int gm_timer_start(uintptr_t h) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaEventRecord(d->ev_start, d->stream));
    return GM_OK;
}

int gm_timer_stop(uintptr_t h, float* elapsed_ms) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!elapsed_ms) { set_error("output is nil"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaEventRecord(d->ev_stop, d->stream));
    GM_CUDA_CHECK(cudaEventSynchronize(d->ev_stop));
    GM_CUDA_CHECK(cudaEventElapsedTime(elapsed_ms, d->ev_start, d->ev_stop));
    return GM_OK;
}

// ---- buffers ----
uintptr_t gm_buffer_alloc(uintptr_t h, int64_t bytes) {
    Device* d = as_device(h);
    return d ? alloc_registered(d, bytes) : 0;
}

void gm_buffer_free(uintptr_t p) { free_registered(p); }
int64_t gm_buffer_size(uintptr_t p) { return registered_size(p); }

// bridge_memory.m:4-42: nil device or size<=0 gives 0; every storage mode maps
// to device memory here.
uintptr_t allocate_cuda_buffer(uintptr_t h, int size, int device_type) {
    (void)device_type;
    if (size <= 0) { set_error("allocation size %d is not positive", size); return 0; }
    return gm_buffer_alloc(h, (int64_t)size);
}

void deallocate_cuda_buffer(uintptr_t p) { free_registered(p); }

int gm_buffer_zero(uintptr_t h, uintptr_t p, int64_t bytes) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!p) { set_error("buffer is nil"); return GM_ERR_NIL_BUFFER; }
    if (bytes <= 0) { set_error("size %lld is not positive", (long long)bytes); return GM_ERR_BAD_SIZE; }
    int64_t have = registered_size(p);
    if (have >= 0 && bytes > have) { set_error("zero of %lld bytes exceeds the %lld-byte buffer", (long long)bytes, (long long)have); return GM_ERR_BAD_SIZE; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaMemsetAsync((void*)p, 0, (size_t)bytes, d->stream));
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return GM_OK;
}

int zero_cuda_buffer(uintptr_t h, uintptr_t p, int size) { return gm_buffer_zero(h, p, (int64_t)size); }

static int copy_sync(uintptr_t p, void* host, int64_t bytes, bool to_device) {
    if (!p) { set_error("buffer is nil"); return GM_ERR_NIL_BUFFER; }
    if (!host) { set_error("host pointer is nil"); return GM_ERR_BAD_ARG; }
    if (bytes <= 0) { set_error("size %lld is not positive", (long long)bytes); return GM_ERR_BAD_SIZE; }
    int64_t have = registered_size(p);
    if (have >= 0 && bytes > have) { set_error("copy of %lld bytes exceeds the %lld-byte buffer", (long long)bytes, (long long)have); return GM_ERR_BAD_SIZE; }
    int ord = registered_ordinal(p);
    int prev = -1;
    if (ord >= 0) { cudaGetDevice(&prev); if (prev != ord) cudaSetDevice(ord); }
    cudaError_t e = to_device ? cudaMemcpy((void*)p, host, (size_t)bytes, cudaMemcpyHostToDevice)
                              : cudaMemcpy(host, (void*)p, (size_t)bytes, cudaMemcpyDeviceToHost);
    if (ord >= 0 && prev != ord && prev >= 0) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy");
    return GM_OK;
}

int copy_data_to_cuda_buffer(uintptr_t p, void* data, int size) { return copy_sync(p, data, size, true); }
int copy_float32_array_to_cuda_buffer(uintptr_t p, float* data, int n) { return copy_sync(p, data, (int64_t)n * 4, true); }
int copy_int32_array_to_cuda_buffer(uintptr_t p, int* data, int n) { return copy_sync(p, data, (int64_t)n * 4, true); }
int copy_cuda_buffer_to_float32_array(uintptr_t p, float* data, int n) { return copy_sync(p, data, (int64_t)n * 4, false); }
int copy_cuda_buffer_to_int32_array(uintptr_t p, int* data, int n) { return copy_sync(p, data, (int64_t)n * 4, false); }

int gm_buffer_upload(uintptr_t h, uintptr_t p, const void* host, int64_t bytes) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));     // never overwrite inputs of a step still in flight
    return copy_sync(p, const_cast<void*>(host), bytes, true);
}

int gm_buffer_download(uintptr_t h, uintptr_t p, void* host, int64_t bytes) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return copy_sync(p, host, bytes, false);
}

int gm_buffer_upload_async(uintptr_t h, uintptr_t p, const void* host, int64_t bytes) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!p || !host || bytes <= 0) { set_error("bad async upload arguments"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaMemcpyAsync((void*)p, host, (size_t)bytes, cudaMemcpyHostToDevice, d->stream));
    return GM_OK;
}

int gm_buffer_download_async(uintptr_t h, uintptr_t p, void* host, int64_t bytes) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!p || !host || bytes <= 0) { set_error("bad async download arguments"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaMemcpyAsync(host, (void*)p, (size_t)bytes, cudaMemcpyDeviceToHost, d->stream));
    return GM_OK;
}

void* gm_host_alloc_pinned(int64_t bytes) {
    void* p = nullptr;
    if (bytes <= 0) return nullptr;
    cudaError_t e = cudaMallocHost(&p, (size_t)bytes);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMallocHost"); cudaGetLastError(); return nullptr; }
    return p;
}

void gm_host_free_pinned(void* p) { if (p) cudaFreeHost(p); }

// ---- arenas ----
// The arena's own allocation stays out of the buffer registry; only the
// sub-buffers handed out are registered (as not separately freeable).
uintptr_t gm_arena_create(uintptr_t h, int64_t bytes) {
    Device* d = as_device(h);
    if (!d) return 0;
    if (bytes <= 0) { set_error("arena size %lld is not positive", (long long)bytes); return 0; }
    DeviceGuard g(d);
    void* p = nullptr;
    int64_t cap = round_up(bytes, 256);
    cudaError_t e = cudaMalloc(&p, (size_t)cap);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(arena)"); cudaGetLastError(); return 0; }
    Arena* a = new Arena();
    a->base = (uintptr_t)p; a->cap = cap; a->used = 0; a->ordinal = d->ordinal;
    std::lock_guard<std::mutex> lk(g_mu);
    g_arenas.insert(a);
    return (uintptr_t)a;
}

uintptr_t gm_arena_alloc(uintptr_t h, int64_t bytes) {
    Arena* a = as_arena(h);
    if (!a) { set_error("not a live arena"); return 0; }
    if (bytes <= 0) { set_error("allocation size %lld is not positive", (long long)bytes); return 0; }
    int64_t need = round_up(bytes, 256);
    std::lock_guard<std::mutex> lk(g_mu);
    if (a->used + need > a->cap) { set_error("arena full: %lld of %lld bytes used, %lld requested", (long long)a->used, (long long)a->cap, (long long)bytes); return 0; }
    uintptr_t p = a->base + (uintptr_t)a->used;
    a->used += need;
    g_bufs[p] = BufInfo{bytes, a->ordinal, false};
    g_registry_gen.fetch_add(1, std::memory_order_release);
    return p;
}

uintptr_t gm_arena_base(uintptr_t h) { Arena* a = as_arena(h); return a ? a->base : 0; }
int64_t gm_arena_capacity(uintptr_t h) { Arena* a = as_arena(h); return a ? a->cap : -1; }
int64_t gm_arena_used(uintptr_t h) { Arena* a = as_arena(h); return a ? a->used : -1; }

static void arena_forget_subbuffers(Arena* a) {     // g_mu held
    for (auto it = g_bufs.begin(); it != g_bufs.end();) {
        bool inside = !it->second.owned && it->first >= a->base && it->first < a->base + (uintptr_t)a->cap;
        if (inside) it = g_bufs.erase(it); else ++it;
    }
    g_registry_gen.fetch_add(1, std::memory_order_release);
}

void gm_arena_reset(uintptr_t h) {
    Arena* a = as_arena(h);
    if (!a) return;
    std::lock_guard<std::mutex> lk(g_mu);
    arena_forget_subbuffers(a);
    a->used = 0;
}

void gm_arena_destroy(uintptr_t h) {
    Arena* a = as_arena(h);
    if (!a) return;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_arenas.erase(a);
        arena_forget_subbuffers(a);
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != a->ordinal) cudaSetDevice(a->ordinal);
    cudaFree((void*)a->base);
    if (prev != a->ordinal && prev >= 0) cudaSetDevice(prev);
    delete a;
}

// ---- conversion ----
int convert_tensor_type_cuda(uintptr_t src, uintptr_t dst, int* shape, int nd, int src_t, int dst_t, uintptr_t h) {
    Device* d = as_device(h);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!src || !dst) { set_error("source or destination buffer is nil"); return GM_ERR_NIL_BUFFER; }
    if (!shape || nd <= 0) { set_error("shape is empty"); return GM_ERR_BAD_ARG; }
    long long n = 1;
    for (int i = 0; i < nd; ++i) {
        if (shape[i] <= 0) { set_error("shape[%d]=%d is not positive", i, shape[i]); return GM_ERR_BAD_SIZE; }
        n *= shape[i];
    }
    const int F32 = 0, F16 = 2;
    if ((src_t == F32 || src_t == F16) && (dst_t == F32 || dst_t == F16)) {
        if (!buffer_holds(src, n * (src_t == F32 ? 4 : 2), "conversion source")) return GM_ERR_BAD_SIZE;
        if (!buffer_holds(dst, n * (dst_t == F32 ? 4 : 2), "conversion destination")) return GM_ERR_BAD_SIZE;
    }
    DeviceGuard g(d);
    int blocks = (int)((n + 255) / 256);
    int cap = d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    const bool vec = src % 16 == 0 && dst % 16 == 0;        // buffers from this library always are
    if (vec) {
        blocks = (int)(((n >> 3) + 255) / 256);
        if (blocks > d->sm_count * 32) blocks = d->sm_count * 32;
        if (blocks < 1) blocks = 1;                           // the tail (n % 8 <= 7 elements) fits in one block
    }
    if (src_t == F32 && dst_t == F16) {
        if (vec) convert_f32_to_f16_vec_kernel<<<blocks, 256, 0, d->stream>>>((const float*)src, (__half*)dst, n);
        else convert_f32_to_f16_kernel<<<blocks, 256, 0, d->stream>>>((const float*)src, (__half*)dst, n);
    } else if (src_t == F16 && dst_t == F32) {
        if (vec) convert_f16_to_f32_vec_kernel<<<blocks, 256, 0, d->stream>>>((const __half*)src, (float*)dst, n);
        else convert_f16_to_f32_kernel<<<blocks, 256, 0, d->stream>>>((const __half*)src, (float*)dst, n);
    } else {
        set_error("conversion %d -> %d is not supported (only Float32<->Float16)", src_t, dst_t);
        return GM_ERR_UNSUPPORTED;
    }
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return GM_OK;
}

// ---- tensor lists ----
uintptr_t gm_tensor_list_create(uintptr_t h, int ns, int nt, const uintptr_t* const* sp,
                                const int64_t* numel, const int* elem_bytes) {
    Device* d = as_device(h);
    if (!d) return 0;
    if (!sp || !numel) { set_error("pointer or size array is nil"); return 0; }
    int err = 0;
    return (uintptr_t)build_list(d, ns, nt, sp, numel, elem_bytes, false, &err);
}

void gm_tensor_list_destroy(uintptr_t h) {
    TensorList* l = as_list(h);
    if (!l || l->key != 0) return;      // cached lists belong to the device
    free_list(l);
}

int64_t gm_tensor_list_total(uintptr_t h) { TensorList* l = as_list(h); return l ? l->total : -1; }
int gm_tensor_list_chunk_elems(uintptr_t h) { TensorList* l = as_list(h); return l ? l->dl.chunk_elems : -1; }
int gm_tensor_list_head(uintptr_t h, int tensor) {
    TensorList* l = as_list(h);
    if (!l) return -2;
    if (tensor < 0 || tensor >= (int)l->head.size()) { set_error("tensor index %d outside the list", tensor); return -2; }
    return l->head[tensor];
}
int gm_tensor_list_num_chunks(uintptr_t h) { TensorList* l = as_list(h); return l ? l->dl.num_chunks : -1; }

}  // extern "C"

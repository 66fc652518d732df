// gm_zero1.cu -- ZeRO-1 style sharding of the optimizer step across the GPUs
// of one node: every rank keeps the full parameter arena, owns the optimizer
// state (and the gradients) of one contiguous shard, updates that shard, and
// the updated parameters are exchanged with an all-gather over NVLink.
//
// The reference has no multi-device code at all; this file has no counterpart
// there.  NCCL is loaded at run time (dlopen of libnccl.so.2) so the library
// itself loads on machines without NCCL; the ZeRO-1 entries then report
// GM_ERR_UNSUPPORTED.
//
// Two exchange paths:
//   * gm_zero1_allgather_async / gm_zero1_adam_step_async: the update kernel
//     followed by ncclAllGather on the same stream (in place: rank r's shard
//     already sits at arena + r*count).
//   * gm_zero1_adam_push_step_async: one kernel that updates the shard and
//     stores each new parameter vector to the local arena and to every peer's
//     arena through peer-mapped pointers (plain st.global over NVLink; no TMA,
//     no multicast), so the transfer overlaps the update tile by tile.  A
//     one-word ncclAllReduce behind it on the same stream is the barrier that
//     tells every rank that all pushes into its arena have landed.  There is
//     no device-side waiting in the kernel.
#include <dlfcn.h>
#include <math.h>
#include <string.h>

#include <set>

#include "gm_apply.cuh"

namespace gm {

// Minimal NCCL surface (matches nccl.h 2.x; types kept opaque).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
constexpr int kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclInt32 = 2, kNcclSum = 0;

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
    std::string load_error;           // why `ok` is false, captured once when the load was tried
};

static NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
            const char* why = dlerror();                 // one call: it also clears the message
            api.load_error = why ? why : "dlopen failed";
        }
        if (!api.handle) return;
        api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
        api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
        api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
        api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
        api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
        api.ReduceScatter = (decltype(api.ReduceScatter))dlsym(api.handle, "ncclReduceScatter");
        api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.AllReduce
                 && api.GetErrorString;
        if (!api.ok) api.load_error = "libnccl was loaded but lacks a required symbol";
    });
    return api;
}

static int nccl_fail(ncclResult_t r, const char* what) {
    set_error("NCCL error %d (%s) in %s", r, nccl().GetErrorString ? nccl().GetErrorString(r) : "?", what);
    return GM_ERR_CUDA;
}

constexpr int kArenaSlots = 2;         // 0: fp32 parameter arena, 1: fp16 parameter arena (mixed precision)

// One exported arena and the peers' mappings of theirs (index = rank; own entry = local base).
struct PeerMap {
    uintptr_t peer_base[kMaxPeers] = {0};
    bool peer_opened[kMaxPeers] = {false};
    uintptr_t local_base = 0;
    size_t local_bytes = 0;            // size of the exported allocation
};

struct Zero1 {
    Device* dev = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    PeerMap map[kArenaSlots];          // peer-mapped arenas for the push paths
    int* barrier_word = nullptr;       // device int used by the closing all-reduce
    bool push_prefetch = true;         // GOMETAL_PUSH_PREFETCH=0 selects the push kernel without the software prefetch
    int push_variant = 2;              // GOMETAL_PUSH_VARIANT (2 measured best on 8 GPUs): how the remote stores of a pass leave (see zero1_adam_push_kernel)
    // copy-engine path: one stream per peer, one event per slice, one "done" event per peer
    cudaStream_t copy_stream[kMaxPeers] = {nullptr};
    cudaEvent_t copy_done[kMaxPeers] = {nullptr};
    std::vector<cudaEvent_t> slice_ready;
};

static std::mutex g_z_mu;
static std::set<Zero1*> g_z;

static Zero1* as_zero1(uintptr_t h) {
    if (!h) { set_error("ZeRO-1 handle is nil"); return nullptr; }
    std::lock_guard<std::mutex> lk(g_z_mu);
    Zero1* z = reinterpret_cast<Zero1*>(h);
    if (!g_z.count(z)) { set_error("handle %p is not a live ZeRO-1 group", (void*)h); return nullptr; }
    return z;
}

// ---- fused update + push ----

// Adam over this rank's shard list; every new parameter vector is stored to the
// local arena and to the same offset of each peer's arena.
// NP = number of peers, a template parameter so that the store loop unrolls
// and the peer offsets stay in registers.  Like mta_apply_kernel, a thread issues
// the loads of its next pass before the arithmetic and the stores of the current
// one, so the remote stores leave while loads are in flight.
//
// VAR picks how the NP remote stores of a pass leave: 0 = plain stores, peers in the order
// rank+1, rank+2, ...; 1 = the same with the evict-first (.cs) qualifier; 2 = plain stores
// whose first peer rotates with the warp and the pass, so that the warps of an SM do not all
// address the same peer at the same moment.
__device__ __forceinline__ void st_remote_cs(float4* a, const float4 v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int NP, int VAR>
__global__ void __launch_bounds__(kApplyThreads, 4)
zero1_adam_push_kernel(const DevList L, const AdamRule::P prm, const PeerDst peers) {
    constexpr int NS = 4;
    constexpr int NT = kApplyThreads;
    const int tid = threadIdx.x;
    const int T = L.num_tensors;
    const long long chunk = L.chunk_elems;

    for (int c = blockIdx.x; c < L.num_chunks; c += gridDim.x) {
        const int2 rec = __ldg(L.chunk_rec + c);
        const int t = rec.x, k = rec.y;
        const long long n = __ldg(L.numel + t);
        const int h = __ldg(L.head + t);
        float* p[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) p[s] = reinterpret_cast<float*>(__ldg(L.ptrs + (size_t)s * T + t));

        auto scalar_at = [&](long long i) {
            float x[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) x[s] = p[s][i];
            AdamRule::elem(x, prm);
            p[0][i] = x[0]; p[2][i] = x[2]; p[3][i] = x[3];
#pragma unroll
            for (int r = 0; r < NP; ++r)
                *reinterpret_cast<float*>(reinterpret_cast<char*>(p[0] + i) + peers.delta[r]) = x[0];
        };

        if (h < 0) {
            const long long b = (long long)k * chunk;
            const long long e = (b + chunk < n) ? b + chunk : n;
            for (long long i = b + tid; i < e; i += NT) scalar_at(i);
            continue;
        }
        const long long b = (long long)h + (long long)k * chunk;
        const long long e = (b + chunk < n) ? b + chunk : n;
        if (k == 0 && tid < h) scalar_at(tid);
        const int nvec = (int)((e - b) >> 2);
        float4* q[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) q[s] = reinterpret_cast<float4*>(p[s] + b);

        int i = tid;
        float4 cur[NS];
        if (i < nvec) {
#pragma unroll
            for (int s = 0; s < NS; ++s) cur[s] = ld_stream(q[s] + i);
        }
        while (i < nvec) {
            const int nx = i + NT;
            float4 nxt[NS];
            if (nx < nvec) {
#pragma unroll
                for (int s = 0; s < NS; ++s) nxt[s] = ld_stream(q[s] + nx);
            }
            float x0[NS], x1[NS], x2[NS], x3[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) { x0[s] = cur[s].x; x1[s] = cur[s].y; x2[s] = cur[s].z; x3[s] = cur[s].w; }
            AdamRule::elem(x0, prm); AdamRule::elem(x1, prm); AdamRule::elem(x2, prm); AdamRule::elem(x3, prm);
            const float4 wn = make_float4(x0[0], x1[0], x2[0], x3[0]);
            if (VAR == 2) {
                int idx = ((i >> 5) + (i / NT)) % NP;
#pragma unroll
                for (int r = 0; r < NP; ++r) {
                    *reinterpret_cast<float4*>(reinterpret_cast<char*>(q[0] + i) + peers.delta[idx]) = wn;
                    idx = idx + 1 == NP ? 0 : idx + 1;
                }
            } else {
#pragma unroll
                for (int r = 0; r < NP; ++r) {
                    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<char*>(q[0] + i) + peers.delta[r]);
                    if (VAR == 1) st_remote_cs(dst, wn); else *dst = wn;
                }
            }
            *(q[0] + i) = wn;                                            // local copy stays cacheable
            st_stream(q[2] + i, make_float4(x0[2], x1[2], x2[2], x3[2]));
            st_stream(q[3] + i, make_float4(x0[3], x1[3], x2[3], x3[3]));
#pragma unroll
            for (int s = 0; s < NS; ++s) cur[s] = nxt[s];
            i = nx;
        }
        const long long tb = b + ((long long)nvec << 2);
        if (tb + tid < e) scalar_at(tb + tid);
    }
}

// The version without the software prefetch (GOMETAL_PUSH_PREFETCH=0), kept for comparison.
template <int NP>
__global__ void __launch_bounds__(kApplyThreads, 4)
zero1_adam_push_plain_kernel(const DevList L, const AdamRule::P prm, const PeerDst peers) {
    constexpr int NS = 4;
    constexpr int NT = kApplyThreads;
    const int tid = threadIdx.x;
    const int T = L.num_tensors;
    const long long chunk = L.chunk_elems;
    for (int c = blockIdx.x; c < L.num_chunks; c += gridDim.x) {
        const int2 rec = __ldg(L.chunk_rec + c);
        const int t = rec.x, k = rec.y;
        const long long n = __ldg(L.numel + t);
        const int h = __ldg(L.head + t);
        float* p[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) p[s] = reinterpret_cast<float*>(__ldg(L.ptrs + (size_t)s * T + t));
        auto scalar_at = [&](long long i) {
            float x[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) x[s] = p[s][i];
            AdamRule::elem(x, prm);
            p[0][i] = x[0]; p[2][i] = x[2]; p[3][i] = x[3];
#pragma unroll
            for (int r = 0; r < NP; ++r)
                *reinterpret_cast<float*>(reinterpret_cast<char*>(p[0] + i) + peers.delta[r]) = x[0];
        };
        if (h < 0) {
            const long long b = (long long)k * chunk;
            const long long e = (b + chunk < n) ? b + chunk : n;
            for (long long i = b + tid; i < e; i += NT) scalar_at(i);
            continue;
        }
        const long long b = (long long)h + (long long)k * chunk;
        const long long e = (b + chunk < n) ? b + chunk : n;
        if (k == 0 && tid < h) scalar_at(tid);
        const long long nvec = (e - b) >> 2;
        float4* q[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) q[s] = reinterpret_cast<float4*>(p[s] + b);
        for (long long i = tid; i < nvec; i += NT) {
            float4 v[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) v[s] = ld_stream(q[s] + i);
            float x0[NS], x1[NS], x2[NS], x3[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) { x0[s] = v[s].x; x1[s] = v[s].y; x2[s] = v[s].z; x3[s] = v[s].w; }
            AdamRule::elem(x0, prm); AdamRule::elem(x1, prm); AdamRule::elem(x2, prm); AdamRule::elem(x3, prm);
            const float4 wn = make_float4(x0[0], x1[0], x2[0], x3[0]);
            *(q[0] + i) = wn;
            st_stream(q[2] + i, make_float4(x0[2], x1[2], x2[2], x3[2]));
            st_stream(q[3] + i, make_float4(x0[3], x1[3], x2[3], x3[3]));
#pragma unroll
            for (int r = 0; r < NP; ++r)
                *reinterpret_cast<float4*>(reinterpret_cast<char*>(q[0] + i) + peers.delta[r]) = wn;
        }
        const long long tb = b + (nvec << 2);
        if (tb + tid < e) scalar_at(tb + tid);
    }
}

using PushFn = void (*)(const DevList, const AdamRule::P, const PeerDst);

template <int NP>
static PushFn push_kernel_np(bool prefetch, int variant) {
    if (!prefetch) return zero1_adam_push_plain_kernel<NP>;
    switch (variant) {
        case 1: return zero1_adam_push_kernel<NP, 1>;
        case 2: return zero1_adam_push_kernel<NP, 2>;
        default: return zero1_adam_push_kernel<NP, 0>;
    }
}

static PushFn push_kernel_for(int peers, bool prefetch, int variant) {
    switch (peers) {
        case 0: case 1: return push_kernel_np<1>(prefetch, variant);
        case 2: return push_kernel_np<2>(prefetch, variant);
        case 3: return push_kernel_np<3>(prefetch, variant);
        case 4: return push_kernel_np<4>(prefetch, variant);
        case 5: return push_kernel_np<5>(prefetch, variant);
        case 6: return push_kernel_np<6>(prefetch, variant);
        default: return push_kernel_np<7>(prefetch, variant);
    }
}

}  // namespace gm

using namespace gm;

extern "C" {

int gm_zero1_unique_id(void* out_id) {
    if (!out_id) { set_error("output is nil"); return GM_ERR_BAD_ARG; }
    if (!nccl().ok) { set_error("libnccl.so.2 could not be loaded: %s", nccl().load_error.c_str()); return GM_ERR_UNSUPPORTED; }
    ncclUniqueId id;
    ncclResult_t r = nccl().GetUniqueId(&id);
    if (r != 0) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(out_id, &id, sizeof(id));
    return GM_OK;
}

uintptr_t gm_zero1_create(uintptr_t device_ptr, const void* unique_id, int rank, int world) {
    Device* d = as_device(device_ptr);
    if (!d) return 0;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) { set_error("bad rank %d / world %d (max %d)", rank, world, kMaxPeers); return 0; }
    Zero1* z = new Zero1();
    z->dev = d; z->rank = rank; z->world = world;
    if (const char* e = getenv("GOMETAL_PUSH_PREFETCH")) z->push_prefetch = atoi(e) != 0;
    if (const char* e = getenv("GOMETAL_PUSH_VARIANT")) z->push_variant = atoi(e);
    DeviceGuard g(d);
    if (cudaMalloc((void**)&z->barrier_word, 256) != cudaSuccess) { cuda_fail(cudaGetLastError(), "cudaMalloc"); delete z; return 0; }
    cudaMemset(z->barrier_word, 0, 256);
    if (world > 1) {
        if (!unique_id) { set_error("unique id is nil"); cudaFree(z->barrier_word); delete z; return 0; }
        if (!nccl().ok) { set_error("libnccl.so.2 could not be loaded: %s", nccl().load_error.c_str()); cudaFree(z->barrier_word); delete z; return 0; }
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        ncclResult_t r = nccl().CommInitRank(&z->comm, world, id, rank);
        if (r != 0) { nccl_fail(r, "ncclCommInitRank"); cudaFree(z->barrier_word); delete z; return 0; }
    }
    std::lock_guard<std::mutex> lk(g_z_mu);
    g_z.insert(z);
    return (uintptr_t)z;
}

void gm_zero1_destroy(uintptr_t h) {
    Zero1* z = as_zero1(h);
    if (!z) return;
    {
        std::lock_guard<std::mutex> lk(g_z_mu);
        g_z.erase(z);
    }
    DeviceGuard g(z->dev);
    cudaStreamSynchronize(z->dev->stream);
    for (int r = 0; r < z->world; ++r) {
        if (z->copy_stream[r]) { cudaStreamSynchronize(z->copy_stream[r]); cudaStreamDestroy(z->copy_stream[r]); }
        if (z->copy_done[r]) cudaEventDestroy(z->copy_done[r]);
        for (int slot = 0; slot < kArenaSlots; ++slot)
            if (z->map[slot].peer_opened[r]) cudaIpcCloseMemHandle((void*)z->map[slot].peer_base[r]);
    }
    for (cudaEvent_t e : z->slice_ready) cudaEventDestroy(e);
    if (z->comm) nccl().CommDestroy(z->comm);
    cudaFree(z->barrier_word);
    delete z;
}

int gm_zero1_rank(uintptr_t h) { Zero1* z = as_zero1(h); return z ? z->rank : -1; }
int gm_zero1_world(uintptr_t h) { Zero1* z = as_zero1(h); return z ? z->world : -1; }

int gm_zero1_allgather_async(uintptr_t h, uintptr_t arena_base, int64_t count, int elem_bytes) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    if (!arena_base) { set_error("arena is nil"); return GM_ERR_NIL_BUFFER; }
    if (count <= 0 || (elem_bytes != 2 && elem_bytes != 4)) { set_error("bad count/element size"); return GM_ERR_BAD_SIZE; }
    if (!buffer_holds(arena_base, (int64_t)z->world * count * elem_bytes, "all-gather arena")) return GM_ERR_BAD_SIZE;
    if (z->world == 1) return GM_OK;
    DeviceGuard g(z->dev);
    const char* send = (const char*)arena_base + (size_t)z->rank * count * elem_bytes;
    ncclResult_t r = nccl().AllGather(send, (void*)arena_base, (size_t)count,
                                      elem_bytes == 4 ? kNcclFloat32 : kNcclFloat16, z->comm, z->dev->stream);
    if (r != 0) return nccl_fail(r, "ncclAllGather");
    z->dev->launches++;
    return GM_OK;
}

int gm_zero1_step_async(uintptr_t h, int rule, uintptr_t shard_list, const gm_hyper_t* hyper, uintptr_t arena_base,
                        int64_t count) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    TensorList* l = as_list(shard_list);
    if (!l || !hyper) { if (l) set_error("hyper-parameters are nil"); return GM_ERR_BAD_ARG; }
    int rc = launch_rule(z->dev, rule, l, *hyper);
    if (rc != GM_OK) return rc;
    return gm_zero1_allgather_async(h, arena_base, count, 4);
}

int gm_zero1_adam_step_async(uintptr_t h, uintptr_t shard_list, const gm_hyper_t* hyper, uintptr_t arena_base,
                             int64_t count) {
    return gm_zero1_step_async(h, GM_RULE_ADAM, shard_list, hyper, arena_base, count);
}

// cudaIpcGetMemHandle describes a whole device allocation, and the peer that opens it
// gets the allocation's first byte back, whatever address inside it was exported.  The
// peers store to "their mapping + the same offset", so the arena has to start where its
// allocation starts; the driver's address-range query (loaded at run time, like NCCL)
// tells.  Returns 1 when arena_base is the base (and the allocation's size), 0 when it
// is not, -1 when unknown.
static int is_allocation_base(uintptr_t arena_base, size_t* alloc_bytes) {
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    static range_fn fn = []() -> range_fn {
        void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        return h ? (range_fn)dlsym(h, "cuMemGetAddressRange_v2") : nullptr;
    }();
    if (!fn) return -1;
    unsigned long long base = 0;
    size_t size = 0;
    if (fn(&base, &size, (unsigned long long)arena_base) != 0) return -1;
    *alloc_bytes = size;
    return base == (unsigned long long)arena_base ? 1 : 0;
}

// ---- peer mapping for the push path ----
int gm_zero1_ipc_handle(uintptr_t h, uintptr_t arena_base, void* out_handle /* 64 bytes */) {
    return gm_zero1_ipc_handle_slot(h, 0, arena_base, out_handle);
}

int gm_zero1_open_peers(uintptr_t h, const void* handles /* world x 64 bytes, rank order */) {
    return gm_zero1_open_peers_slot(h, 0, handles);
}

int gm_zero1_ipc_handle_slot(uintptr_t h, int slot, uintptr_t arena_base, void* out_handle /* 64 bytes */) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    if (slot < 0 || slot >= kArenaSlots) { set_error("arena slot %d outside [0,%d)", slot, kArenaSlots); return GM_ERR_BAD_ARG; }
    if (!arena_base || !out_handle) { set_error("nil argument"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(z->dev);
    size_t alloc_bytes = 0;
    const int at_base = is_allocation_base(arena_base, &alloc_bytes);
    if (at_base == 0) {
        set_error("the parameter arena must start at the first byte of its device allocation: "
                  "an IPC handle maps the whole allocation and the peers would store at the wrong offset");
        return GM_ERR_BAD_ARG;
    }
    cudaIpcMemHandle_t mh;
    GM_CUDA_CHECK(cudaIpcGetMemHandle(&mh, (void*)arena_base));
    static_assert(sizeof(mh) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(out_handle, &mh, sizeof(mh));
    size_t bytes = at_base == 1 ? alloc_bytes : 0;
    if (bytes == 0 && registered_size(arena_base) > 0) bytes = (size_t)registered_size(arena_base);
    if (bytes == 0) {
        // Neither the driver's address-range query nor the library's own registry knows where this
        // allocation starts and ends: the peers' stores could not be checked against it.
        set_error("cannot establish the bounds of the arena's allocation; the peer-store paths need them "
                  "(use gm_zero1_adam_step_async, which exchanges through NCCL, instead)");
        return GM_ERR_UNSUPPORTED;
    }
    z->map[slot].local_base = arena_base;
    z->map[slot].local_bytes = bytes;
    return GM_OK;
}

int gm_zero1_open_peers_slot(uintptr_t h, int slot, const void* handles /* world x 64 bytes, rank order */) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    if (slot < 0 || slot >= kArenaSlots) { set_error("arena slot %d outside [0,%d)", slot, kArenaSlots); return GM_ERR_BAD_ARG; }
    if (!handles) { set_error("handles are nil"); return GM_ERR_BAD_ARG; }
    if (!z->map[slot].local_base) { set_error("call gm_zero1_ipc_handle first"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(z->dev);
    for (int r = 0; r < z->world; ++r) {
        if (r == z->rank) { z->map[slot].peer_base[r] = z->map[slot].local_base; continue; }
        if (z->map[slot].peer_opened[r]) {                 // a new arena replaces an earlier mapping
            cudaStreamSynchronize(z->dev->stream);
            cudaIpcCloseMemHandle((void*)z->map[slot].peer_base[r]);
            z->map[slot].peer_opened[r] = false;
            z->map[slot].peer_base[r] = 0;
        }
        cudaIpcMemHandle_t mh;
        memcpy(&mh, (const char*)handles + (size_t)r * 64, 64);
        void* p = nullptr;
        GM_CUDA_CHECK(cudaIpcOpenMemHandle(&p, mh, cudaIpcMemLazyEnablePeerAccess));
        z->map[slot].peer_base[r] = (uintptr_t)p;
        z->map[slot].peer_opened[r] = true;
    }
    return GM_OK;
}

// Every parameter tensor of the shard must lie inside the exported arena: its address
// minus the arena base is added to each peer's mapping, and a tensor from elsewhere would
// turn into a store to an address no peer mapped.
static int check_inside_arena(const Zero1* z, const TensorList* l, const int slot = 0, const int stream = 0,
                              const int elem_bytes = 4) {
    if (!z->map[slot].local_base) { set_error("call gm_zero1_ipc_handle and gm_zero1_open_peers first"); return GM_ERR_BAD_ARG; }
    for (size_t t = 0; t < l->numel.size(); ++t) {
        const uintptr_t p = l->ptrs[stream][t];
        const uintptr_t end = p + (uintptr_t)l->numel[t] * elem_bytes;
        if (p < z->map[slot].local_base || end > z->map[slot].local_base + z->map[slot].local_bytes) {
            set_error("parameter tensor %zu lies outside the arena exported to the peers", t);
            return GM_ERR_BAD_ARG;
        }
    }
    return GM_OK;
}

// Launches the fused update + push kernel over a window of the shard list (no barrier).
// rank r stores to r+1, r+2, ... so that at any moment the ranks aim at different peers
static int peer_destinations(const Zero1* z, const int slot, PeerDst* peers) {
    peers->count = 0;
    for (int i = 1; i < z->world; ++i) {
        const int r = (z->rank + i) % z->world;
        if (!z->map[slot].peer_base[r]) { set_error("peer %d is not mapped; call gm_zero1_open_peers", r); return GM_ERR_BAD_ARG; }
        peers->delta[peers->count++] = (long long)z->map[slot].peer_base[r] - (long long)z->map[slot].local_base;
    }
    return GM_OK;
}

static int push_launch(Zero1* z, const TensorList* l, const gm_hyper_t& hyper, Window win) {
    Device* d = z->dev;
    PeerDst peers{};
    {
        const int rc = peer_destinations(z, 0, &peers);
        if (rc != GM_OK) return rc;
    }
    AdamRule::P p;
    p.lr = hyper.lr; p.beta1 = hyper.beta1; p.beta2 = hyper.beta2; p.eps = hyper.eps;
    p.wd = hyper.weight_decay; p.use_wd = hyper.weight_decay > 0.0f ? 1 : 0;
    p.bc1 = 1.0f - powf(hyper.beta1, (float)hyper.step);
    p.bc2 = 1.0f - powf(hyper.beta2, (float)hyper.step);
    p.omb1 = 1.0f - hyper.beta1;
    p.omb2 = 1.0f - hyper.beta2;
    p.rbc1 = 0.0f; p.rbc2 = 0.0f;
    DevList dl;
    const int rc = apply_window(l, win, &dl);
    if (rc != GM_OK) return rc;
    if (dl.num_chunks == 0) return GM_OK;
    DeviceGuard g(d);
    const PushFn kernel = push_kernel_for(peers.count, z->push_prefetch, z->push_variant);
    const int grid = launch_grid(d, (const void*)kernel, kApplyThreads, dl.num_chunks);
    kernel<<<grid, kApplyThreads, 0, d->stream>>>(dl, p, peers);
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    return GM_OK;
}

// One-word all-reduce on the device stream: completes only after every rank's pushes
// (everything enqueued before it on each rank's stream) have finished.
static int push_barrier(Zero1* z) {
    if (z->world <= 1) return GM_OK;
    DeviceGuard g(z->dev);
    ncclResult_t r = nccl().AllReduce(z->barrier_word, z->barrier_word, 1, kNcclInt32, kNcclSum, z->comm, z->dev->stream);
    if (r != 0) return nccl_fail(r, "ncclAllReduce(barrier)");
    z->dev->launches++;
    return GM_OK;
}

static int push_validate(Zero1* z, const TensorList* l, const gm_hyper_t* hyper) {
    if (!l || !hyper) { if (l) set_error("hyper-parameters are nil"); return GM_ERR_BAD_ARG; }
    if (l->dev != z->dev) { set_error("tensor list belongs to another device"); return GM_ERR_BAD_ARG; }
    if (l->dl.num_streams != 4) { set_error("Adam shard list needs w,g,m,v"); return GM_ERR_BAD_ARG; }
    for (int s = 0; s < 4; ++s) if (l->elem_bytes[s] != 4) { set_error("stream %d is not fp32", s); return GM_ERR_BAD_ARG; }
    if (hyper->step < 1) { set_error("Adam step count %d must be >= 1", hyper->step); return GM_ERR_BAD_ARG; }
    return check_inside_arena(z, l);
}

int gm_zero1_adam_push_step_async(uintptr_t h, uintptr_t shard_list, const gm_hyper_t* hyper) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    TensorList* l = as_list(shard_list);
    int rc = push_validate(z, l, hyper);
    if (rc != GM_OK) return rc;
    rc = push_launch(z, l, *hyper, Window());
    if (rc != GM_OK) return rc;
    return push_barrier(z);
}

// The sharded step for a caller whose gradients and parameters live in pinned HOST memory:
// the rank's gradient shard is uploaded, updated and pushed to the peers, and the rank's new
// parameters are downloaded, slice by slice on three streams (see gm_step_host); the closing
// barrier tells every rank that its arena is complete.  Synchronous.
int gm_zero1_adam_push_step_host(uintptr_t h, uintptr_t shard_list, const gm_hyper_t* hyper, const void* host_grads,
                                 void* host_params, int num_slices) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    TensorList* l = as_list(shard_list);
    int rc = push_validate(z, l, hyper);
    if (rc != GM_OK) return rc;
    if (!host_grads || !host_params) { set_error("nil host buffer"); return GM_ERR_BAD_ARG; }
    const gm_hyper_t hy = *hyper;
    rc = host_pipelined_step(z->dev, l, host_grads, host_params, num_slices,
                             [&](Window win) { return push_launch(z, l, hy, win); },
                             [&]() { return push_barrier(z); });
    return rc;
}

// Update + exchange with the copy engines: the shard is cut into `num_slices`
// groups of whole tensors; as soon as the update kernel of a slice has finished,
// one cudaMemcpyAsync per peer (each on its own stream) copies the slice's new
// parameters into the same offset of that peer's arena, while the SMs update
// the next slice.  The step ends, like the push path, with a one-word all-reduce
// after the device stream has waited for every copy stream.  The shard's
// parameter tensors must lie back to back in the arena.
int gm_zero1_adam_dma_step_async(uintptr_t h, uintptr_t shard_list, const gm_hyper_t* hyper, int num_slices) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    TensorList* l = as_list(shard_list);
    if (!l || !hyper) { if (l) set_error("hyper-parameters are nil"); return GM_ERR_BAD_ARG; }
    if (l->dl.num_streams != 4) { set_error("Adam shard list needs w,g,m,v"); return GM_ERR_BAD_ARG; }
    Device* d = z->dev;
    const int T = l->dl.num_tensors;
    if (num_slices < 1) num_slices = 1;
    if (num_slices > T) num_slices = T;
    for (int t = 0; t + 1 < T; ++t) {
        if (l->ptrs[0][t] + (uintptr_t)l->numel[t] * 4 != l->ptrs[0][t + 1]) {
            set_error("parameter tensors %d and %d are not contiguous in the arena", t, t + 1);
            return GM_ERR_BAD_ARG;
        }
    }
    const int slot = 0;
    for (int r = 0; r < z->world; ++r) {
        if (r != z->rank && !z->map[slot].peer_base[r]) { set_error("peer %d is not mapped; call gm_zero1_open_peers", r); return GM_ERR_BAD_ARG; }
    }
    {
        const int rc = check_inside_arena(z, l);
        if (rc != GM_OK) return rc;
    }
    DeviceGuard g(d);
    for (int r = 0; r < z->world; ++r) {
        if (r == z->rank || z->copy_stream[r]) continue;
        GM_CUDA_CHECK(cudaStreamCreateWithFlags(&z->copy_stream[r], cudaStreamNonBlocking));
        GM_CUDA_CHECK(cudaEventCreateWithFlags(&z->copy_done[r], cudaEventDisableTiming));
    }
    while ((int)z->slice_ready.size() < num_slices) {
        cudaEvent_t e;
        GM_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        z->slice_ready.push_back(e);
    }
    int rc = GM_OK;
    for (int s = 0; s < num_slices && rc == GM_OK; ++s) {
        const int t0 = (int)((long long)T * s / num_slices), t1 = (int)((long long)T * (s + 1) / num_slices);
        if (t1 <= t0) continue;
        Window win;
        win.begin = l->chunk_prefix[t0];
        win.count = l->chunk_prefix[t1] - l->chunk_prefix[t0];
        rc = launch_rule(d, GM_RULE_ADAM, l, *hyper, win);
        if (rc != GM_OK) break;
        GM_CUDA_CHECK(cudaEventRecord(z->slice_ready[s], d->stream));
        const uintptr_t src = l->ptrs[0][t0];
        const size_t bytes = (size_t)(l->ptrs[0][t1 - 1] + (uintptr_t)l->numel[t1 - 1] * 4 - src);
        for (int r = 0; r < z->world; ++r) {
            if (r == z->rank) continue;
            const uintptr_t dst = src - z->map[slot].local_base + z->map[slot].peer_base[r];
            GM_CUDA_CHECK(cudaStreamWaitEvent(z->copy_stream[r], z->slice_ready[s], 0));
            GM_CUDA_CHECK(cudaMemcpyAsync((void*)dst, (const void*)src, bytes, cudaMemcpyDeviceToDevice, z->copy_stream[r]));
        }
    }
    if (rc != GM_OK) return rc;
    for (int r = 0; r < z->world; ++r) {
        if (r == z->rank) continue;
        GM_CUDA_CHECK(cudaEventRecord(z->copy_done[r], z->copy_stream[r]));
        GM_CUDA_CHECK(cudaStreamWaitEvent(d->stream, z->copy_done[r], 0));
    }
    return push_barrier(z);
}

// Mixed-precision Adam on sharded fp16 gradients: the overflow flag of every
// rank's shard is summed across ranks between the check and the update, so all
// ranks skip or step together and their loss-scale states stay identical; the
// fp16 parameter copies are then all-gathered in place.
static int zero1_flag_hook(void* ctx, unsigned int* d_flag) {
    Zero1* z = static_cast<Zero1*>(ctx);
    if (z->world == 1) return GM_OK;
    ncclResult_t r = nccl().AllReduce(d_flag, d_flag, 1, kNcclInt32, kNcclSum, z->comm, z->dev->stream);
    if (r != 0) return nccl_fail(r, "ncclAllReduce(overflow flag)");
    z->dev->launches++;
    return GM_OK;
}

int gm_zero1_mixed_step_async(uintptr_t h, uintptr_t mixed, uintptr_t shard_list, float lr, float eps, float wd,
                              uintptr_t p16_arena_base, int64_t count_per_rank) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    int rc = mixed_step_with_hook((uintptr_t)z->dev, mixed, shard_list, lr, eps, wd, zero1_flag_hook, z);
    if (rc != GM_OK) return rc;
    return gm_zero1_allgather_async(h, p16_arena_base, count_per_rank, 2);
}

// The same step with the exchange fused into the update kernel: every new fp16 parameter
// vector is stored to the local arena and to the same offset of each peer's fp16 arena
// (arena slot 1, exported with gm_zero1_ipc_handle_slot / gm_zero1_open_peers_slot); the
// closing one-word all-reduce is the barrier.  On a skipped step nothing is stored.
int gm_zero1_mixed_push_step_async(uintptr_t h, uintptr_t mixed, uintptr_t shard_list, float lr, float eps, float wd) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    TensorList* l = as_list(shard_list);
    if (!l) return GM_ERR_BAD_ARG;
    if (l->dl.num_streams != 5) { set_error("mixed-precision list must be g16, master, m, v, p16"); return GM_ERR_BAD_ARG; }
    int rc = check_inside_arena(z, l, 1, 4, 2);
    if (rc != GM_OK) return rc;
    PeerDst peers{};
    rc = peer_destinations(z, 1, &peers);
    if (rc != GM_OK) return rc;
    rc = mixed_step_with_hook((uintptr_t)z->dev, mixed, shard_list, lr, eps, wd, zero1_flag_hook, z, &peers);
    if (rc != GM_OK) return rc;
    return push_barrier(z);
}

// Gradient hand-off for data-parallel training: every rank holds a full gradient
// arena of its own micro-batch; after the call rank r's shard
// [r*count, (r+1)*count) holds the SUM over ranks (in place), which is what the
// sharded update consumes.  The summation order inside NCCL is not specified,
// so results are reproducible run to run on one topology but not bit-defined.
int gm_zero1_reduce_scatter_async(uintptr_t h, uintptr_t grad_arena_base, int64_t count, int elem_bytes) {
    Zero1* z = as_zero1(h);
    if (!z) return GM_ERR_BAD_ARG;
    if (!grad_arena_base) { set_error("arena is nil"); return GM_ERR_NIL_BUFFER; }
    if (count <= 0 || (elem_bytes != 2 && elem_bytes != 4)) { set_error("bad count/element size"); return GM_ERR_BAD_SIZE; }
    if (!buffer_holds(grad_arena_base, (int64_t)z->world * count * elem_bytes, "reduce-scatter arena")) return GM_ERR_BAD_SIZE;
    if (z->world == 1) return GM_OK;
    if (!nccl().ReduceScatter) { set_error("ncclReduceScatter is not available"); return GM_ERR_UNSUPPORTED; }
    DeviceGuard g(z->dev);
    char* recv = (char*)grad_arena_base + (size_t)z->rank * count * elem_bytes;
    ncclResult_t r = nccl().ReduceScatter((const void*)grad_arena_base, recv, (size_t)count,
                                          elem_bytes == 4 ? kNcclFloat32 : kNcclFloat16, kNcclSum, z->comm, z->dev->stream);
    if (r != 0) return nccl_fail(r, "ncclReduceScatter");
    z->dev->launches++;
    return GM_OK;
}

}  // extern "C"

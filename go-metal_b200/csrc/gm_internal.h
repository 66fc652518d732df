// gm_internal.h -- shared host-side structures of libgometal_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <functional>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "gometal_cuda.h"

namespace gm {

constexpr int kMaxStreams = 5;          // pointer arrays one rule can walk
constexpr int kApplyThreads = 256;      // CTA width of the apply kernels
constexpr int kVecBytes = 16;           // 128-bit accesses
constexpr int kMagicDevice = 0x474d4456;   // "GMDV"
constexpr int kMagicList = 0x474d544c;     // "GMTL"

// Descriptor a multi-tensor kernel receives by value.  All arrays live in one
// device allocation owned by the TensorList.
struct DevList {
    const unsigned long long* ptrs;   // [num_streams][num_tensors] device addresses
    const long long* numel;           // [num_tensors]
    const int* head;                  // [num_tensors] scalar elements before the 16-B aligned body; -1 = no aligned body
    const int* chunk_prefix;          // [num_tensors+1] first chunk of each tensor
    const int2* chunk_rec;            // [num_chunks] {tensor, chunk index inside the tensor}
    const int* dot_prefix;            // [num_tensors+1] first 4096-element reduction chunk of each tensor (counted from element 0)
    int num_dot_chunks;
    int num_tensors;
    int num_chunks;
    int chunk_elems;                  // elements per chunk (multiple of the vector tile)
    int num_streams;
};

struct Device;

struct TensorList {
    int magic = kMagicList;
    Device* dev = nullptr;
    DevList dl{};
    void* blob = nullptr;             // device allocation behind dl
    int64_t total = 0;
    int elem_bytes[kMaxStreams] = {4, 4, 4, 4, 4};
    std::vector<int64_t> numel;       // host copy
    std::vector<std::vector<uintptr_t>> ptrs;   // host copy [stream][tensor]
    uint64_t key = 0;                 // cache key (0 = not cached)
    std::vector<int> chunk_prefix;    // host copy: first chunk of each tensor, [num_tensors+1]
    std::vector<int> head;            // host copy of dl.head
    uint64_t validated_gen = 0;       // registry generation under which the buffers were last checked
};

// A launch may cover only chunks [begin, begin + count) of a list (a slice of whole
// tensors in the pipelined entries); count < 0 means the whole list.  Passed by value:
// the list itself is never modified by a launch.
struct Window { int begin = 0; int count = -1; };

struct Device {
    int magic = kMagicDevice;
    int ordinal = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;   // host-buffer steps: copies overlap the kernels
    std::vector<cudaEvent_t> slice_events;
    std::mutex mu;
    std::unordered_map<uint64_t, TensorList*> list_cache;
    std::vector<TensorList*> parked_lists;   // displaced from the cache while possibly still in use
    std::vector<TensorList*> retired_lists;  // the cache's content at its last eviction; freed at the next one
    int64_t launches = 0;
    int mixed_keep_g = 1;               // fp16 gradients marked evict_last by the overflow check (GOMETAL_MIXED_KEEP_G)
    int mixed_check_persistent = 1;     // overflow check as one resident wave of looping CTAs (GOMETAL_MIXED_CHECK_PERSISTENT)
    int mixed_fastdiv = 1;              // divisions by the bias corrections through div_const (GOMETAL_MIXED_FASTDIV)
    int mixed_pf = 1;                   // next-pass L2 prefetch in the update kernel (GOMETAL_MIXED_PF)
    int mixed_ring = 0;                 // 2: the mixed step as one cooperative launch, 1: check kernel + ring update,
                                        // 0: check kernel + one-CTA-per-chunk update (GOMETAL_MIXED_RING)
    long long barrier_budget_cycles = 1LL << 31;   // bound of every device-side barrier wait, about a second
                                        // (GOMETAL_BARRIER_BUDGET_CYCLES)
    int mixed_variant = 0;              // 1: the 4-elements-per-thread update kernel instead of the 8-element one (GOMETAL_MIXED_VARIANT)
    int mixed_overlap = 2;              // update grid launched with programmatic stream serialization: 2 = it may start when the
                                        // check grid's CTAs reach their end (measured best), 1 = from their start, 0 = off
                                        // (GOMETAL_MIXED_OVERLAP)
    int lbfgs_overlap = 2;              // L-BFGS passes launched with programmatic stream serialization: 2 = the next pass may
                                        // start when a pass's CTAs reach their end (measured best), 1 = from their start, 0 = off
                                        // (GOMETAL_LBFGS_OVERLAP)
    int lbfgs_keep_dir = 1;             // L-BFGS direction lines marked evict_last in L2 (GOMETAL_LBFGS_KEEP_DIR=0 turns it off)
    int lbfgs_prewait = 1;              // history loads an L-BFGS pass issues before it waits for the previous pass: 0 none, 1 its first
                                        // chunk, 2 also an L2 prefetch of its second (GOMETAL_LBFGS_PREWAIT)
    int lbfgs_defer = 1;                // an L-BFGS pass whose scalar only the next pass reads leaves the final sum to that pass
                                        // instead of a ticket and a finishing CTA (GOMETAL_LBFGS_DEFER=0 turns it off)
    int lbfgs_waves = 1;                // resident-CTA waves of the pipelined L-BFGS pass (GOMETAL_LBFGS_WAVES)
    int grid_waves = 0;                 // 0: one CTA per chunk; >0: waves of resident CTAs (GOMETAL_GRID_WAVES)
    int chunk_elems = 0;                // 0: default tile; else elements per chunk (GOMETAL_CHUNK_ELEMS)
    int lbfgs_coop = 0;                 // L-BFGS step as one cooperative launch: 2 = direction left in L2, 1 = direction kept on
                                        // chip, 0 = one launch per pass (GOMETAL_LBFGS_COOP)
    unsigned lbfgs_epoch = 0;           // barrier epochs handed to the single-launch L-BFGS step so far
    int lbfgs_mode = 3;                 // bit 0: corrected curvature pair, bit 1: descent direction
    // scratch for reductions (dot partials, tickets); grown on demand
    float* partials = nullptr;
    int64_t partials_cap = 0;
    // chunk sums of the single-launch L-BFGS step, each a 64-bit word {barrier epoch, sum}; zeroed when allocated
    unsigned long long* tagged = nullptr;
    int64_t tagged_cap = 0;
    unsigned int* ticket = nullptr;     // one counter for last-CTA-done finishes
    float* scalars = nullptr;           // small device scratch for L-BFGS scalars
};

// Destinations of a fused update + push kernel: byte offsets from the local arena to each
// peer's mapping of its own arena (plain peer stores over NVLink).
constexpr int kMaxPeers = 8;
struct PeerDst {
    long long delta[kMaxPeers];
    int count;                        // number of peers (excluding self)
};

// ---- error reporting ----
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);   // records and returns GM_ERR_CUDA

#define GM_CUDA_CHECK(call)                                              \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) return ::gm::cuda_fail(e__, #call);       \
    } while (0)

Device* as_device(uintptr_t h);        // nullptr (and error text) if not a live device
TensorList* as_list(uintptr_t h);

// RAII: make the device's ordinal current for the scope.
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(const Device* d) {
        cudaGetDevice(&prev);
        if (prev != d->ordinal) cudaSetDevice(d->ordinal);
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// ---- tensor lists ----
// Builds (or fetches from the device's cache when `cache` is set) the
// descriptor for the given pointer arrays.  Returns nullptr on failure.
TensorList* build_list(Device* d, int num_streams, int num_tensors,
                       const uintptr_t* const* stream_ptrs, const int64_t* numel,
                       const int* elem_bytes, bool cache, int* err);
void free_list(TensorList* l);

// Grid size for a chunked kernel: one CTA per chunk, or waves of resident CTAs when the device asks for it.
int launch_grid(Device* d, const void* kernel, int threads, int64_t work_items);

int ensure_partials(Device* d, int64_t count);
int ensure_tagged(Device* d, int64_t count);
constexpr int kDotChunkElems = 4096;    // elements per chunk of the fixed-order reductions

// ---- rule launchers (gm_rules.cu) ----
void lbfgs_release_device(Device* d);           // frees the L-BFGS pointer tables cached for a device
// clip: device address of the global-norm clipping coefficient every gradient is multiplied
// by first (nullptr: gradients are used as they are)
int launch_rule(Device* d, int rule, const TensorList* l, const gm_hyper_t& h, Window win = Window(),
                const float* clip = nullptr);
// Applies a window to a list's descriptor; GM_ERR_BAD_ARG when it lies outside the list.
int apply_window(const TensorList* l, Window win, DevList* out);

// Host-buffer pipeline shared by gm_step_host and the sharded host step (gm_rules.cu).
int host_pipelined_step(Device* d, const TensorList* l, const void* host_grads, void* host_params, int num_slices,
                        const std::function<int(Window)>& launch, const std::function<int()>& finish);

// ---- mixed precision (gm_mixed.cu) ----
// push: when given, every new fp16 parameter vector is also stored to the peers' arenas
int mixed_step_with_hook(uintptr_t device_ptr, uintptr_t mixed, uintptr_t list, float lr, float eps, float wd,
                         int (*hook)(void* ctx, unsigned int* d_flag), void* ctx, const PeerDst* push = nullptr);

// ---- buffer registry (gm_device.cu) ----
int64_t registered_size(uintptr_t p);   // -1 if unknown
// false (with the error text set) when p is a buffer this library allocated and it holds
// fewer than `need` bytes; buffers from elsewhere cannot be checked and pass
bool buffer_holds(uintptr_t p, int64_t need, const char* what);
// changes whenever the library allocates or releases a buffer: a cached validation made under the
// current value is still good
uint64_t registry_generation();
int registered_ordinal(uintptr_t p);    // -1 if unknown

}  // namespace gm

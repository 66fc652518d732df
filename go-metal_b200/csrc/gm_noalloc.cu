// gm_noalloc.cu -- a dot product entry that never touches the allocator.
//
// gm_dot_canonical() keeps its chunk sums and its "last CTA" ticket in buffers
// obtained with cudaMalloc (through the device handle, and a small table per
// call).  Some hosts cannot afford that: a trainer that has handed every byte
// of HBM to its own arenas has nothing left for cudaMalloc to return, and a
// steady-state training loop that must not stall cannot take the device-wide
// synchronisation cudaMalloc/cudaFree imply.  For those callers this file
// provides the same reduction with its working memory compiled into the
// library: one file-scope __device__ array per GPU that loads the library
// (about 64 KB, held until the process exits).
//
// The summation order is the documented fixed order of gm_lbfgs.cu (4096-element
// chunks, 256 lanes walking (i*256+t)*4+k, xor tree per warp, warp sums in
// order, chunk sums by the CTA that finishes last), so the result has the same
// bits as gm_dot_canonical().
#include <mutex>

#include "gm_apply.cuh"

namespace gm {

constexpr int kStaticDotChunk = 4096;
constexpr int kStaticDotThreads = 256;
constexpr int kStaticMaxChunks = 16384;                       // 64 Mi elements at most
constexpr long long kStaticMaxElems = (long long)kStaticMaxChunks * kStaticDotChunk;
static_assert(kStaticMaxElems == GM_DOT_STATIC_MAX_ELEMENTS, "header and kernel disagree on the limit");
constexpr int kTicketWords = 64;                               // first 256 bytes: the ticket

// Working memory of gm_dot_canonical_static: [0] ticket, [64..] one sum per chunk.
// In host code this name is only a handle for cudaGetSymbolAddress; the device
// address is looked up once per device below and passed to the kernel.
static __device__ __align__(256) float g_static_dot_scratch[kTicketWords + kStaticMaxChunks];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mu;
static float* g_static_ptr[kMaxDevices] = {nullptr};

__device__ __forceinline__ float static_cta_sum(float acc, float* warp_sum) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = add(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.0f;
    if (threadIdx.x == 0) {
        total = warp_sum[0];
#pragma unroll
        for (int w = 1; w < kStaticDotThreads / 32; ++w) total = add(total, warp_sum[w]);
    }
    __syncthreads();
    return total;
}

__global__ void __launch_bounds__(kStaticDotThreads)
dot_static_kernel(const float* __restrict__ a, const float* __restrict__ b, long long n, int num_chunks,
                  int vec_ok, float* __restrict__ scratch, float* __restrict__ out) {
    __shared__ float warp_sum[kStaticDotThreads / 32];
    __shared__ int is_last;
    const int tid = threadIdx.x;
    unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch);
    float* partials = scratch + kTicketWords;

    for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
        const long long base = (long long)c * kStaticDotChunk;
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < kStaticDotChunk / (kStaticDotThreads * 4); ++i) {
            const long long e0 = base + ((long long)i * kStaticDotThreads + tid) * 4;
            if (vec_ok && e0 + 3 < n) {
                const float4 av = *reinterpret_cast<const float4*>(a + e0);
                const float4 bv = *reinterpret_cast<const float4*>(b + e0);
                acc = add(acc, mul(av.x, bv.x)); acc = add(acc, mul(av.y, bv.y));
                acc = add(acc, mul(av.z, bv.z)); acc = add(acc, mul(av.w, bv.w));
            } else {
                for (int k = 0; k < 4; ++k) if (e0 + k < n) acc = add(acc, mul(a[e0 + k], b[e0 + k]));
            }
        }
        const float total = static_cta_sum(acc, warp_sum);
        if (tid == 0) partials[c] = total;
    }

    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned my = atomicAdd(ticket, 1u);
        is_last = (my == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float acc = 0.0f;
    const volatile float* pv = partials;
    for (int c = tid; c < num_chunks; c += kStaticDotThreads) acc = add(acc, pv[c]);
    const float dot = static_cta_sum(acc, warp_sum);
    if (tid == 0) {
        *out = dot;
        *ticket = 0u;
    }
}

}  // namespace gm

using namespace gm;

extern "C" {

// Dot product of two fp32 device vectors in the library's fixed summation
// order, for hosts that must not allocate (all HBM already committed to their
// own arenas, or a loop that cannot afford the device-wide synchronisation of
// cudaMalloc/cudaFree).  Inputs `a`, `b` (n floats each) and the one-float
// output `out` are device pointers on the CURRENT device; `stream` is the
// cudaStream_t to launch on (0 = the default stream).  The call is
// asynchronous: read `out` after the stream has been synchronised.
//
// Working memory is a ~64 KB array compiled into the library, one copy per GPU
// that has loaded it, kept until the process exits.  Limit: n <= 67,108,864
// (GM_DOT_STATIC_MAX_ELEMENTS in the header); larger n is rejected with
// GM_ERR_BAD_SIZE.  The first call on each device looks the array's device
// address up (cudaGetSymbolAddress) with that device current; make that first
// call before starting any stream capture.  All calls on a device share the
// array and it keeps the previous call's chunk sums: the ticket word is cleared
// on the stream before every launch, and two calls whose kernels can overlap on
// the GPU (different streams, no ordering between them) race on it -- order
// them.  No cudaMalloc, cudaFree or other allocating routine is called; the one
// thing that can still reserve device memory is CUDA itself, which on the first
// call per device may load this library's code onto the GPU and, with it, place
// the built-in array (lazy module loading).  The looked-up address is cached per
// process and device ordinal and does not survive a cudaDeviceReset.
int gm_dot_canonical_static(uintptr_t a, uintptr_t b, int64_t n, uintptr_t out, uintptr_t stream) {
    if (!a || !b || !out) { set_error("gm_dot_canonical_static: a, b and out must be device pointers"); return GM_ERR_NIL_BUFFER; }
    if (n <= 0) { set_error("gm_dot_canonical_static: length %lld is not positive", (long long)n); return GM_ERR_BAD_SIZE; }
    if (n > kStaticMaxElems) {
        set_error("gm_dot_canonical_static: %lld elements exceed the built-in scratch (max %lld); "
                  "use gm_dot_canonical for longer vectors", (long long)n, kStaticMaxElems);
        return GM_ERR_BAD_SIZE;
    }
    if (a % 4 || b % 4 || out % 4) { set_error("gm_dot_canonical_static: pointers must be 4-byte aligned"); return GM_ERR_BAD_ARG; }
    int ordinal = -1;
    GM_CUDA_CHECK(cudaGetDevice(&ordinal));
    if (ordinal < 0 || ordinal >= kMaxDevices) { set_error("device ordinal %d out of range", ordinal); return GM_ERR_BAD_ARG; }
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_ptr[ordinal]) {
            float* p = nullptr;
            GM_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, g_static_dot_scratch));   // this device's copy
            g_static_ptr[ordinal] = p;
        }
        scratch = g_static_ptr[ordinal];
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int num_chunks = (int)((n + kStaticDotChunk - 1) / kStaticDotChunk);
    const int vec_ok = (a % 16 == 0 && b % 16 == 0) ? 1 : 0;
    // the ticket must start at zero whatever an earlier call left behind
    GM_CUDA_CHECK(cudaMemsetAsync(scratch, 0, sizeof(unsigned int), s));
    int sms = 0;
    GM_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal));
    int grid = sms * 4;
    if (grid > num_chunks) grid = num_chunks;
    if (grid < 1) grid = 1;
    dot_static_kernel<<<grid, kStaticDotThreads, 0, s>>>((const float*)a, (const float*)b, (long long)n, num_chunks,
                                                         vec_ok, scratch, (float*)out);
    GM_CUDA_CHECK(cudaGetLastError());
    return GM_OK;
}

}  // extern "C"

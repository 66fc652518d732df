// gm_clip.cu -- deterministic gradient norm and global-norm clipping for the
// fp32 rules.
//
// The reference has no clipping code; docs/guides/optimizers.md:568-569 names
// gradient-norm clipping as a concept only.  The formula used here is the
// common one, computed in binary32 on the device:
//     coef = min(1, max_norm / (sqrt(sum g^2) + 1e-6))
// and every gradient is multiplied by coef (one rounding) before the rule.
//
// The sum of squares is taken in the library's fixed order (the list dot
// product of g with itself): 4096-element chunks counted from element 0 of each
// tensor; in a chunk lane t of 256 adds the squares of elements (i*256+t)*4+k
// (i, k = 0..3) in that order, each square rounded before it is added; the 32
// lanes of a warp combine by xor tree (16, 8, 4, 2, 1); the 8 warp sums add in
// ascending order; the CTA that finishes last adds the chunk sums of all
// tensors (lane t takes chunks t, t+256, ..., then the same tree).  No float
// atomics: the value depends neither on the grid nor on the addresses.
#include <math.h>

#include "gm_apply.cuh"

namespace gm {

constexpr int kClipThreads = 256;

// out[0] = sum of squares, out[1] = clipping coefficient, out[2] = norm.
__global__ void __launch_bounds__(kClipThreads)
sumsq_canonical_kernel(const DevList L, const int stream, float* __restrict__ partials,
                       unsigned int* __restrict__ ticket, const float max_norm, float* __restrict__ out) {
    __shared__ float warp_sum[kClipThreads / 32];
    __shared__ int is_last;
    const int tid = threadIdx.x;
    const int T = L.num_tensors;
    constexpr int PASSES = kDotChunkElems / (kClipThreads * 4);

    for (int c = blockIdx.x; c < L.num_dot_chunks; c += gridDim.x) {
        const int t = find_tensor(L.dot_prefix, T, c);
        const long long n = __ldg(L.numel + t);
        const long long base = (long long)(c - __ldg(L.dot_prefix + t)) * kDotChunkElems;
        const float* g = reinterpret_cast<const float*>(__ldg(L.ptrs + (size_t)stream * T + t));
        const bool vec_ok = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
        float acc = 0.0f;
        if (vec_ok && base + kDotChunkElems <= n) {
            float4 v[PASSES];
#pragma unroll
            for (int i = 0; i < PASSES; ++i)
                v[i] = __ldcs(reinterpret_cast<const float4*>(g + base + ((long long)i * kClipThreads + tid) * 4));
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
                acc = add(acc, mul(v[i].x, v[i].x)); acc = add(acc, mul(v[i].y, v[i].y));
                acc = add(acc, mul(v[i].z, v[i].z)); acc = add(acc, mul(v[i].w, v[i].w));
            }
        } else {
            for (int i = 0; i < PASSES; ++i) {
                const long long e0 = base + ((long long)i * kClipThreads + tid) * 4;
                for (int k = 0; k < 4; ++k)
                    if (e0 + k < n) { const float x = g[e0 + k]; acc = add(acc, mul(x, x)); }
            }
        }
        const float total = cta_sum_256(acc, warp_sum);
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
    for (int c = tid; c < L.num_dot_chunks; c += kClipThreads) acc = add(acc, pv[c]);
    const float ss = cta_sum_256(acc, warp_sum);
    if (tid == 0) {
        const float norm = root(ss);
        float coef = dvd(max_norm, add(norm, 1e-6f));
        if (!(coef < 1.0f)) coef = 1.0f;            // also when the coefficient is NaN
        out[0] = ss;
        out[1] = coef;
        out[2] = norm;
        *ticket = 0u;
        __threadfence();
    }
}

}  // namespace gm

using namespace gm;

extern "C" {

int gm_grad_clip_coef_async(uintptr_t device_ptr, uintptr_t list, float max_norm, uintptr_t out3_device) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    TensorList* l = as_list(list);
    if (!l) return GM_ERR_BAD_ARG;
    if (l->dev != d) { set_error("tensor list belongs to another device"); return GM_ERR_BAD_ARG; }
    if (!out3_device) { set_error("output buffer is nil"); return GM_ERR_NIL_BUFFER; }
    if (!buffer_holds(out3_device, 12, "clip output")) return GM_ERR_BAD_SIZE;
    if (l->dl.num_streams < 2 || l->elem_bytes[1] != 4) { set_error("the list needs an fp32 gradient stream (stream 1)"); return GM_ERR_BAD_ARG; }
    if (!(max_norm > 0.0f)) { set_error("max_norm %g is not positive", (double)max_norm); return GM_ERR_BAD_ARG; }
    int rc = ensure_partials(d, l->dl.num_dot_chunks);
    if (rc != GM_OK) return rc;
    DeviceGuard g(d);
    int grid = d->sm_count * 8;
    if (grid > l->dl.num_dot_chunks) grid = l->dl.num_dot_chunks;
    if (grid < 1) grid = 1;
    sumsq_canonical_kernel<<<grid, kClipThreads, 0, d->stream>>>(l->dl, 1, d->partials, d->ticket, max_norm, (float*)out3_device);
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    return GM_OK;
}

int gm_step_clipped_async(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper, uintptr_t coef_device) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    TensorList* l = as_list(list);
    if (!l) return GM_ERR_BAD_ARG;
    if (!hyper) { set_error("hyper-parameters are nil"); return GM_ERR_BAD_ARG; }
    if (l->dev != d) { set_error("tensor list belongs to another device"); return GM_ERR_BAD_ARG; }
    if (!coef_device || coef_device % 4) { set_error("the coefficient must be a 4-byte aligned device address"); return GM_ERR_NIL_BUFFER; }
    return launch_rule(d, rule, l, *hyper, Window(), (const float*)coef_device);
}

// Norm, coefficient and step in one call, all on the device's stream: no host round trip.
int gm_step_with_clip_async(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper, float max_norm) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    const uintptr_t out = (uintptr_t)(d->scalars + 16);          // {sum of squares, coefficient, norm}
    int rc = gm_grad_clip_coef_async(device_ptr, list, max_norm, out);
    if (rc != GM_OK) return rc;
    return gm_step_clipped_async(device_ptr, rule, list, hyper, out + 4);
}

int gm_last_clip(uintptr_t device_ptr, float* out3) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!out3) { set_error("output is nil"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    GM_CUDA_CHECK(cudaMemcpy(out3, d->scalars + 16, 12, cudaMemcpyDeviceToHost));
    return GM_OK;
}

}  // extern "C"

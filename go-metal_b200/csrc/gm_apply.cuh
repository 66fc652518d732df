// gm_apply.cuh -- the multi-tensor-apply skeleton shared by the fp32 rules.
//
// One launch walks a whole tensor list.  Work is cut into fixed-size chunks of
// one tensor each (4096 elements by default) and, by default, the grid has one
// CTA per chunk: measured on B200, many short-lived CTAs stream ~10 % faster
// than resident CTAs looping over chunks.  Inside a chunk every stream is read
// and written with 128-bit accesses, one vector per thread per pass, and the
// loads of the next pass are issued before the arithmetic of the current one.
// The few elements before the first and after the last 16-byte boundary of a
// tensor are handled one at a time.
//
// Arithmetic uses the round-to-nearest intrinsics (__fmul_rn, __fadd_rn,
// __fdiv_rn, __fsqrt_rn): the compiler never contracts them into fused
// multiply-adds, so each operation rounds exactly like the scalar statement
// order of cgo_bridge/bridge_optimizer.m.
#pragma once

#include "gm_internal.h"

namespace gm {

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float dvd(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float root(float a) { return __fsqrt_rn(a); }

// The IEEE division and square root take a long special-case path when an
// operand is zero.  Parameters that a model never touches (zero gradient, zero
// moments) would send every one of their elements down it: measured 1.6x the
// kernel time on a list where half the elements are like that.  dvd0 and root0
// are for the call sites where that can happen: the two shortcuts are exact
// (+-0 / b = +-0 for every b > 0 including +inf, sqrt(+-0) = +-0) and everything
// else goes to the intrinsic unchanged.
__device__ __forceinline__ float dvd0(float a, float b) {
    if (a == 0.0f && b > 0.0f) return a;
    return __fdiv_rn(a, b);
}
__device__ __forceinline__ float root0(float a) {
    if (a == 0.0f) return a;
    return __fsqrt_rn(a);
}

// a / c for a divisor c that is the same for a whole launch, given r = RN(1/c):
//     q0 = RN(a*r); e0 = a - q0*c (one fma); q1 = RN(q0 + e0*r); e1 = a - q1*c; q = RN(q1 + e1*r).
// q0 is within 2^-23 of a/c in relative terms, so q1 = RN((a/c)(1 + d)) with |d| < 2^-46 is a
// faithful quotient, its residual e1 is exact, and by Markstein's theorem (a faithful quotient
// corrected once with the correctly rounded reciprocal) the last step returns RN(a/c): the bits
// of __fdiv_rn(a, c) at five instructions, without the reciprocal estimate and its refinement.
// That needs every intermediate to be a normal number.  The host only enables the path for
// 2^-24 <= c <= 1 with a significand that is not all ones (const_div_ok); here a must lie in
// [2^-100, 2^100), which the exponent test checks (zero, denormals, huge values, inf and NaN
// take the IEEE division).  The selftest entry gm_selftest_const_div compares the two over
// all 2^32 values of a for a given c.
__device__ __forceinline__ float div_const(float a, float c, float r) {
    const unsigned biased = (__float_as_uint(a) >> 23) & 0xffu;
    if (biased - 27u < 200u) {                               // 27 <= exponent field <= 226
        float q = __fmul_rn(a, r);
        float e = __fmaf_rn(-q, c, a);
        q = __fmaf_rn(e, r, q);
        e = __fmaf_rn(-q, c, a);
        return __fmaf_rn(e, r, q);
    }
    return dvd0(a, c);
}
__host__ __device__ __forceinline__ bool const_div_ok(float c) {
    union { float f; unsigned u; } b;
    b.f = c;
    return c >= 5.9604644775390625e-08f && c <= 1.0f && (b.u & 0x7fffffu) != 0x7fffffu;
}

// Sum of the 256 lane values of a CTA in the library's fixed order (xor tree per warp, warp
// sums in ascending order); result valid in thread 0.  warp_sum: 8 floats of shared memory.
__device__ __forceinline__ float cta_sum_256(float acc, float* warp_sum) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = add(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.0f;
    if (threadIdx.x == 0) {
        total = warp_sum[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) total = add(total, warp_sum[w]);
    }
    __syncthreads();
    return total;
}

// ---- pieces of the bounded grid-wide barrier of the single-launch steps ----
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// One 64-bit word read or written as a unit at GPU scope: a value and its tag travel together,
// so a reader that sees the tag has the value and no fence is needed on either side.
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

// Waits until *word == epoch, but no longer than `budget` clock cycles.  False: gave up.
__device__ __forceinline__ bool bounded_wait_for(const unsigned* word, const unsigned epoch, const long long budget) {
    const long long t0 = clock64();
    while (ld_acquire(word) != epoch) {
        if (clock64() - t0 > budget) return false;
        __nanosleep(64);
    }
    return true;
}

// Streaming accesses: every byte is touched once per step, so lines are marked
// evict-first on the way in and on the way out.
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float* p, float v) { __stcs(p, v); }

// Finds the tensor that owns chunk c: the largest t with prefix[t] <= c.
__device__ __forceinline__ int find_tensor(const int* __restrict__ prefix, int num_tensors, int c) {
    int lo = 0, hi = num_tensors;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (__ldg(prefix + mid) <= c) lo = mid; else hi = mid;
    }
    return lo;
}

// ---- Adam (shared by the fp32 and the mixed-precision kernels): bridge_optimizer.m:398-399 (host), :484-550 (graph) ----
struct AdamRule {
    static constexpr int NS = 4;                 // w, g, m, v
    static constexpr unsigned WMASK = 0b1101;
    struct P { float lr, beta1, beta2, omb1, omb2, bc1, bc2, eps, wd; int use_wd; float rbc1, rbc2; };
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) { elem_t<false>(x, p); }
    // FAST: the two divisions by the bias corrections go through div_const with the
    // reciprocals rbc1 and rbc2 (same bits; the caller has checked const_div_ok for both).
    template <bool FAST>
    static __device__ __forceinline__ void elem_t(float (&x)[NS], const P& p) {
        const float w = x[0], g = x[1];
        const float m_new = add(mul(x[2], p.beta1), mul(g, p.omb1));
        const float v_new = add(mul(x[3], p.beta2), mul(mul(g, g), p.omb2));
        const float m_hat = FAST ? div_const(m_new, p.bc1, p.rbc1) : dvd0(m_new, p.bc1);
        const float v_hat = FAST ? div_const(v_new, p.bc2, p.rbc2) : dvd0(v_new, p.bc2);
        float upd = dvd0(m_hat, add(root0(v_hat), p.eps));
        if (p.use_wd) upd = add(upd, mul(w, p.wd));
        x[0] = sub(w, mul(upd, p.lr));
        x[2] = m_new;
        x[3] = v_new;
    }
};

// L2 eviction policies for data that a later launch reads again while other
// data streams past it once (the L-BFGS direction vector between passes, the
// fp16 gradients between the overflow check and the update): lines loaded or
// stored with the evict_last policy stay in L2 ahead of evict-first streams.
__device__ __forceinline__ unsigned long long l2_policy(const bool keep) {
    unsigned long long p;
    if (keep) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    else asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ float4 ld_l2(const float* a, const unsigned long long pol) {
    float4 v;
    asm volatile("ld.global.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(a), "l"(pol));
    return v;
}
__device__ __forceinline__ void st_l2(float* a, const float4 v, const unsigned long long pol) {
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;"
                 :: "l"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "l"(pol) : "memory");
}

__device__ __forceinline__ uint4 ld_l2(const uint4* a, const unsigned long long pol) {
    uint4 v;
    asm volatile("ld.global.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a), "l"(pol));
    return v;
}

// Rule concept:
//   static constexpr int NS;            number of streams (w, g, state...)
//   static constexpr unsigned WMASK;    bit s set => stream s is written back
//   struct P;                           scalars, passed by value
//   static __device__ void elem(float (&x)[NS], const P&);   in-place on x
//
// CLIP: every gradient (stream 1 of every rule) is first multiplied by the
// global-norm clipping coefficient, a device scalar that a reduction launched
// earlier on the same stream has left at `clip` (one rounding per gradient).
template <class Rule, bool CLIP>
__global__ void __launch_bounds__(kApplyThreads, (Rule::NS <= 4 ? 5 : 4))
mta_apply_kernel(const DevList L, const typename Rule::P prm, const float* __restrict__ clip) {
    constexpr int NS = Rule::NS;
    constexpr int NT = kApplyThreads;
    const int tid = threadIdx.x;
    const int T = L.num_tensors;
    const int chunk = L.chunk_elems;
    const float cs = CLIP ? __ldg(clip) : 1.0f;

    for (int c = blockIdx.x; c < L.num_chunks; c += gridDim.x) {
        const int2 rec = __ldg(L.chunk_rec + c);          // {tensor, chunk index inside the tensor}
        const int t = rec.x, k = rec.y;
        const long long n = __ldg(L.numel + t);
        const int h = __ldg(L.head + t);
        float* p[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) p[s] = reinterpret_cast<float*>(__ldg(L.ptrs + (size_t)s * T + t));

        if (h < 0) {
            // streams disagree on alignment: element-wise walk of this chunk
            const long long b = (long long)k * chunk;
            const long long e = (b + chunk < n) ? b + chunk : n;
            for (long long i = b + tid; i < e; i += NT) {
                float x[NS];
#pragma unroll
                for (int s = 0; s < NS; ++s) x[s] = ld_stream(p[s] + i);
                if (CLIP) x[1] = mul(x[1], cs);
                Rule::elem(x, prm);
#pragma unroll
                for (int s = 0; s < NS; ++s) if (Rule::WMASK & (1u << s)) st_stream(p[s] + i, x[s]);
            }
            continue;
        }

        // aligned body of this chunk: elements [b, b+len), b on a 16-byte boundary in every stream
        const long long b = (long long)h + (long long)k * chunk;
        const long long left = n - b;
        const int len = left < (long long)chunk ? (int)(left > 0 ? left : 0) : chunk;
        const int nvec = len >> 2;
#pragma unroll
        for (int s = 0; s < NS; ++s) p[s] += b;

        int i = tid;
        float4 cur[NS];
        if (i < nvec) {
#pragma unroll
            for (int s = 0; s < NS; ++s) cur[s] = ld_stream(reinterpret_cast<const float4*>(p[s]) + i);
        }
        while (i < nvec) {
            const int nx = i + NT;
            float4 nxt[NS];
            if (nx < nvec) {                               // next pass's loads go out first
#pragma unroll
                for (int s = 0; s < NS; ++s) nxt[s] = ld_stream(reinterpret_cast<const float4*>(p[s]) + nx);
            }
            float x0[NS], x1[NS], x2[NS], x3[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) { x0[s] = cur[s].x; x1[s] = cur[s].y; x2[s] = cur[s].z; x3[s] = cur[s].w; }
            if (CLIP) { x0[1] = mul(x0[1], cs); x1[1] = mul(x1[1], cs); x2[1] = mul(x2[1], cs); x3[1] = mul(x3[1], cs); }
            Rule::elem(x0, prm);
            Rule::elem(x1, prm);
            Rule::elem(x2, prm);
            Rule::elem(x3, prm);
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                if (Rule::WMASK & (1u << s))
                    st_stream(reinterpret_cast<float4*>(p[s]) + i, make_float4(x0[s], x1[s], x2[s], x3[s]));
            }
#pragma unroll
            for (int s = 0; s < NS; ++s) cur[s] = nxt[s];
            i = nx;
        }

        // fewer than 4 elements after the last full vector, and the h (< 4)
        // elements before the first boundary of the tensor
        int idx = -1 - h;                                   // nothing to do
        if ((nvec << 2) + tid < len) idx = (nvec << 2) + tid;
        else if (k == 0 && tid >= NT - h) idx = tid - NT;   // -h .. -1: the head, taken by the last h threads
        if (idx >= -h) {
            float x[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) x[s] = ld_stream(p[s] + idx);
            if (CLIP) x[1] = mul(x[1], cs);
            Rule::elem(x, prm);
#pragma unroll
            for (int s = 0; s < NS; ++s) if (Rule::WMASK & (1u << s)) st_stream(p[s] + idx, x[s]);
        }
    }
}

template <class Rule>
int launch_apply(Device* d, const TensorList* l, const typename Rule::P& prm, Window win = Window(),
                 const float* clip = nullptr) {
    if (l->dl.num_streams != Rule::NS) {
        set_error("tensor list has %d streams, rule needs %d", l->dl.num_streams, Rule::NS);
        return GM_ERR_BAD_ARG;
    }
    for (int s = 0; s < Rule::NS; ++s) {
        if (l->elem_bytes[s] != 4) { set_error("stream %d is not fp32", s); return GM_ERR_BAD_ARG; }
    }
    auto kernel = clip ? mta_apply_kernel<Rule, true> : mta_apply_kernel<Rule, false>;
    DevList dl;
    {
        const int rc = apply_window(l, win, &dl);
        if (rc != GM_OK) return rc;
        if (dl.num_chunks == 0) return GM_OK;
    }
    int grid = launch_grid(d, (const void*)kernel, kApplyThreads, dl.num_chunks);
    kernel<<<grid, kApplyThreads, 0, d->stream>>>(dl, prm, clip);
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    return GM_OK;
}

}  // namespace gm

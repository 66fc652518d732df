// gm_mixed.cu -- mixed-precision Adam with a device-resident dynamic loss
// scale, and the gradient sum-of-squares reduction.
//
// The reference only carries the configuration of this feature
// (training/model_trainer.go:79-87, 258-270: scale 65536, growth 2, backoff
// 0.5, interval 2000) and a standalone fp32<->fp16 conversion kernel
// (cgo_bridge/bridge_memory.m:362-376); the policy text is
// docs/tutorials/mixed-precision.md:617-629: on overflow halve the scale and
// skip the update, after N clean steps double it.  One step here is two
// launches and no host synchronisation:
//   1. mixed_check_kernel   reads the fp16 gradients once, ORs an overflow
//                           flag (warp vote, one atomic per CTA at most);
//   2. mixed_update_kernel  if the flag is clear: unscale, Adam on the fp32
//                           master copy (AdamRule, same order as the fp32
//                           path), write master/m/v and the fp16 copy; the
//                           last CTA to finish advances the loss-scale state
//                           machine and the Adam step counter on the device.
// Bias corrections come from a host-computed table indexed by the device-side
// step counter, because libm's powf and CUDA's powf do not round alike.
#include <cuda_fp16.h>
#include <math.h>

#include <algorithm>
#include <set>

#include "gm_apply.cuh"

namespace gm {

constexpr int kMagicMixed = 0x474d4d58;   // "GMMX"

struct Mixed {
    int magic = kMagicMixed;
    Device* dev = nullptr;
    gm_loss_scale_t* d_state = nullptr;
    unsigned int* d_flag = nullptr;        // [0] overflow flag, [1] update ticket, [2] check ticket, [3] sum-of-squares
                                           // accumulator, [16..19] StepPrep, [24] last step's sum of squares
    int want_norm = 0;
    float max_norm = 0.0f;                 // > 0: global-norm clipping with this limit
    float2* d_table = nullptr;             // [table_len+1] {1-b1^t, 1-b2^t}
    int table_len = 0;
    bool saturated = false;                // table[table_len] == {1,1}: later steps reuse it
    float beta1 = 0.9f, beta2 = 0.999f;
    int64_t calls = 0;                     // upper bound of the device step counter
    unsigned epoch = 0;                    // barrier epoch of the last single-launch step
};

static std::mutex g_mixed_mu;
static std::set<Mixed*> g_mixed;

static Mixed* as_mixed(uintptr_t h) {
    if (!h) { set_error("mixed-precision handle is nil"); return nullptr; }
    std::lock_guard<std::mutex> lk(g_mixed_mu);
    Mixed* m = reinterpret_cast<Mixed*>(h);
    if (!g_mixed.count(m)) { set_error("handle %p is not a live mixed-precision state", (void*)h); return nullptr; }
    return m;
}

static int upload_table(Mixed* m, int len) {
    std::vector<float2> host((size_t)len + 1);
    host[0] = make_float2(1.0f, 1.0f);
    for (int t = 1; t <= len; ++t) {
        host[t].x = 1.0f - powf(m->beta1, (float)t);     // bridge_optimizer.m:398
        host[t].y = 1.0f - powf(m->beta2, (float)t);     // bridge_optimizer.m:399
    }
    // From the first step at which both corrections equal 1 they stay 1.
    m->saturated = host[len].x == 1.0f && host[len].y == 1.0f;
    DeviceGuard g(m->dev);
    GM_CUDA_CHECK(cudaStreamSynchronize(m->dev->stream));
    if (m->d_table) cudaFree(m->d_table);
    m->d_table = nullptr;
    GM_CUDA_CHECK(cudaMalloc((void**)&m->d_table, sizeof(float2) * ((size_t)len + 1)));
    GM_CUDA_CHECK(cudaMemcpy(m->d_table, host.data(), sizeof(float2) * ((size_t)len + 1), cudaMemcpyHostToDevice));
    m->table_len = len;
    return GM_OK;
}

// The device counter can be at most `calls` before the next step; the table must reach
// calls + 1 unless its tail is already constant.  Doubles until it does.
static int grow_table(Mixed* m) {
    while (!m->saturated && m->calls + 1 > m->table_len) {
        if (m->table_len > (1 << 28)) { set_error("bias-correction table would exceed 2^29 entries"); return GM_ERR_BAD_SIZE; }
        const int rc = upload_table(m, m->table_len * 2);
        if (rc != GM_OK) return rc;
    }
    return GM_OK;
}

static bool valid_loss_scale(const gm_loss_scale_t& s) {
    return s.scale > 0.0f && isfinite(s.scale) && s.growth >= 1.0f && isfinite(s.growth) && s.backoff > 0.0f
           && s.backoff <= 1.0f && s.interval >= 1 && s.max_scale >= s.scale && isfinite(s.max_scale)
           && s.adam_t >= 0 && s.good_steps >= 0 && s.skipped >= 0;
}

// 1 bits at 0x8000 / 0x80000000 mark halves whose exponent field is all ones.
__device__ __forceinline__ unsigned nonfinite_mask(unsigned w) {
    return ((w & 0x7c007c00u) + 0x04000400u) & 0x80008000u;
}

// What the update kernel needs to know about the step, written once by the
// check kernel so that every update CTA starts with a single 16-byte load.
// r1, r2: reciprocals of the bias corrections; fast: both corrections qualify for div_const;
// clip: the global-norm clipping coefficient of this step (1 when clipping is off).
struct StepPrep { unsigned overflow; float inv_scale; float bc1; float bc2; float r1; float r2; float clip; unsigned fast; };

__device__ __forceinline__ void publish_prep(StepPrep* prep, unsigned overflow, float scale, float2 bc, float clip) {
    StepPrep sp;
    sp.overflow = overflow;
    sp.inv_scale = dvd(1.0f, scale);
    sp.bc1 = bc.x;
    sp.bc2 = bc.y;
    sp.r1 = dvd(1.0f, bc.x);
    sp.r2 = dvd(1.0f, bc.y);
    sp.clip = clip;
    sp.fast = (const_div_ok(bc.x) && const_div_ok(bc.y)) ? 1u : 0u;
    *prep = sp;
}

// acc + (half * inv)^2, the square rounded before the add: the order-defined form the
// deterministic gradient norm uses.
__device__ __forceinline__ float sq_acc1(const unsigned short h, const float inv, float acc) {
    const float a = mul(__half2float(__ushort_as_half(h)), inv);
    return add(acc, mul(a, a));
}
__device__ __forceinline__ float sq_acc2(const unsigned x, const float inv, float acc) {
    return sq_acc1((unsigned short)(x >> 16), inv, sq_acc1((unsigned short)(x & 0xffffu), inv, acc));
}
__device__ __forceinline__ float sq_acc8(const uint4 v, const float inv, float acc) {
    return sq_acc2(v.w, inv, sq_acc2(v.z, inv, sq_acc2(v.y, inv, sq_acc2(v.x, inv, acc))));
}

// acc + the squares of the two halves packed in x, each first multiplied by inv.
__device__ __forceinline__ float sumsq2(const unsigned x, const float inv, float acc) {
    const float a = __half2float(__ushort_as_half((unsigned short)(x & 0xffffu))) * inv;
    const float b = __half2float(__ushort_as_half((unsigned short)(x >> 16))) * inv;
    acc = fmaf(a, a, acc);
    return fmaf(b, b, acc);
}
__device__ __forceinline__ float sumsq8(const uint4 v, const float inv, float acc) {
    return sumsq2(v.w, inv, sumsq2(v.z, inv, sumsq2(v.y, inv, sumsq2(v.x, inv, acc))));
}
__device__ __forceinline__ float sumsq1(const unsigned short h, const float inv, float acc) {
    const float a = __half2float(__ushort_as_half(h)) * inv;
    return fmaf(a, a, acc);
}

// NORM: the same pass also takes the sum of squares of the unscaled gradients, in a
// fixed order and without float atomics: per chunk, lane t of 256 adds the squares of
// the vectors t, t+256, ... it loaded (eight halves each, in memory order), then the
// element it owns in front of the tensor's first 16-byte boundary (first chunk only),
// then the element it owns behind the last whole vector; the lane values combine as in
// cta_sum_256 into partials[chunk]; the CTA that finishes last adds the chunk sums (lane
// t takes chunks t, t+256, ...) and leaves the total in flag[24] and, when max_norm > 0,
// the clipping coefficient min(1, max_norm / (sqrt(total) + 1e-6)) in flag[25] and in the
// published scalars.  The order follows the list's chunking, hence the tensors' offsets
// from a 16-byte boundary: the same layout always gives the same bits.
template <bool NORM>
__global__ void __launch_bounds__(kApplyThreads, NORM ? 6 : 8)
mixed_check_kernel(const DevList L, unsigned int* __restrict__ flag, const gm_loss_scale_t* __restrict__ state,
                   const float2* __restrict__ table, int table_len, StepPrep* __restrict__ prep, const int keep_g,
                   float* __restrict__ partials, const float max_norm) {
    __shared__ float warp_ss[kApplyThreads / 32];
    __shared__ int is_last;
    // flags bit 0: the gradients get the evict_last L2 policy (the update kernel reads them
    // again); bit 1: an update kernel launched with programmatic stream serialization may
    // become resident from the start of this grid, else from the point where its CTAs have
    // finished their chunks.  Either way it waits for this grid to complete before it reads
    // the published scalars; without that launch attribute the trigger has no effect.
    if (keep_g & 2) asm volatile("griddepcontrol.launch_dependents;");
    const unsigned long long pol = l2_policy((keep_g & 1) != 0);
    constexpr int NT = kApplyThreads;
    constexpr int U = 4;                                     // 16-byte loads in flight per thread
    const int tid = threadIdx.x;
    const long long chunk = L.chunk_elems;
    unsigned bad = 0;
    const float inv = NORM ? dvd(1.0f, state->scale) : 0.0f;

    // Each CTA walks chunks blockIdx.x, blockIdx.x + gridDim.x, ...  The table
    // lookups of the next chunk are issued while the current chunk's loads are in
    // flight, and the next chunk's loads before the loop turns, so neither latency
    // is exposed after the first chunk.
    struct Ref { const unsigned short* g; long long n, b, e; int h, k; };
    auto lookup = [&](int c) -> Ref {
        Ref r;
        const int2 rec = __ldg(L.chunk_rec + c);
        r.k = rec.y;
        r.n = __ldg(L.numel + rec.x);
        r.h = __ldg(L.head + rec.x);
        r.g = reinterpret_cast<const unsigned short*>(__ldg(L.ptrs + rec.x));
        r.b = (long long)(r.h > 0 ? r.h : 0) + (long long)r.k * chunk;
        r.e = (r.b + chunk < r.n) ? r.b + chunk : r.n;
        return r;
    };
    uint4 v[U];
    auto issue = [&](const Ref& r) {
        // first U*NT vectors of the chunk's aligned body (all of it at the default chunk size)
        const long long nvec = (r.e - r.b) >> 3;
        const uint4* q = reinterpret_cast<const uint4*>(r.g + r.b);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            v[u] = make_uint4(0u, 0u, 0u, 0u);
            if (r.h >= 0 && tid + u * NT < nvec) v[u] = ld_l2(q + tid + u * NT, pol);
        }
    };

    int c = blockIdx.x;
    Ref cur{};
    if (c < L.num_chunks) { cur = lookup(c); issue(cur); }
    while (c < L.num_chunks) {
        const int cn = c + gridDim.x;
        Ref nxt{};
        if (cn < L.num_chunks) nxt = lookup(cn);
        const unsigned short* g = cur.g;
        float ss = 0.0f;
        if (cur.h < 0) {
            // streams off a common 16-byte boundary: element by element
            for (long long i = cur.b + tid; i < cur.e; i += NT) {
                bad |= ((g[i] & 0x7c00u) == 0x7c00u);
                if (NORM) ss = sq_acc1(g[i], inv, ss);
            }
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                bad |= nonfinite_mask(v[u].x) | nonfinite_mask(v[u].y) | nonfinite_mask(v[u].z) | nonfinite_mask(v[u].w);
                if (NORM) ss = sq_acc8(v[u], inv, ss);                      // lanes past the end hold zeros
            }
            const long long nvec = (cur.e - cur.b) >> 3;
            const uint4* q = reinterpret_cast<const uint4*>(g + cur.b);
            for (long long i = tid + (long long)U * NT; i < nvec; i += NT) {      // chunks larger than U*NT vectors
                const uint4 w = ld_l2(q + i, pol);
                bad |= nonfinite_mask(w.x) | nonfinite_mask(w.y) | nonfinite_mask(w.z) | nonfinite_mask(w.w);
                if (NORM) ss = sq_acc8(w, inv, ss);
            }
            if (cur.k == 0 && tid < cur.h) {                                         // elements before the boundary
                bad |= ((g[tid] & 0x7c00u) == 0x7c00u);
                if (NORM) ss = sq_acc1(g[tid], inv, ss);
            }
            const long long tb = cur.b + (nvec << 3);
            if (tb + tid < cur.e) {                                                  // fewer than 8 after the last vector
                bad |= ((g[tb + tid] & 0x7c00u) == 0x7c00u);
                if (NORM) ss = sq_acc1(g[tb + tid], inv, ss);
            }
        }
        if (cn < L.num_chunks) issue(nxt);                                           // in flight during the reduction below
        if (NORM) {
            const float total = cta_sum_256(ss, warp_ss);
            if (tid == 0) partials[c] = total;
        }
        c = cn;
        cur = nxt;
    }
    if (!(keep_g & 2)) asm volatile("griddepcontrol.launch_dependents;");
    // block vote, then one atomic for the whole CTA (and only when needed)
    const int any_bad = __syncthreads_or(bad != 0);
    if (tid == 0) {
        if (any_bad) atomicOr(flag, 1u);
        __threadfence();
        const unsigned ticket = atomicAdd(flag + 2, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    // last CTA: every vote and every chunk sum is in; publish the step's scalars
    __threadfence();
    float total = 0.0f;
    if (NORM) {
        float acc = 0.0f;
        const volatile float* pv = partials;
        for (int k = tid; k < L.num_chunks; k += NT) acc = add(acc, pv[k]);
        total = cta_sum_256(acc, warp_ss);
    }
    if (tid == 0) {
        const unsigned overflow = *reinterpret_cast<volatile unsigned int*>(flag);
        const int tstep = state->adam_t + 1;
        const float2 bc = table[tstep < table_len ? tstep : table_len];
        float clip = 1.0f;
        if (NORM) {
            if (max_norm > 0.0f) {
                clip = dvd(max_norm, add(root(total), 1e-6f));
                if (!(clip < 1.0f)) clip = 1.0f;
            }
            flag[24] = __float_as_uint(total);
            flag[25] = __float_as_uint(clip);
        }
        publish_prep(prep, overflow, state->scale, bc, clip);
        flag[2] = 0u;
    }
}

// Grid of the check kernel: the CTAs resident at once, trimmed so that every CTA
// walks the same number of chunks.
static int check_grid(Device* d, int num_chunks, bool norm) {
    static thread_local int per_sm_of[2] = {0, 0};      // the two instantiations differ in registers
    int& per_sm = per_sm_of[norm ? 1 : 0];
    if (per_sm == 0) {
        if (norm) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mixed_check_kernel<true>, kApplyThreads, 0);
        else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mixed_check_kernel<false>, kApplyThreads, 0);
        if (per_sm < 1) per_sm = 1;
    }
    const long long resident = (long long)per_sm * d->sm_count;
    if (d->mixed_check_persistent == 0 || num_chunks <= resident) return num_chunks;
    const long long rounds = (num_chunks + resident - 1) / resident;
    return (int)((num_chunks + rounds - 1) / rounds);
}

// Recomputes the published scalars after the overflow flag has been combined
// across ranks (sharded gradients: every rank must take the same decision).
__global__ void mixed_prep_kernel(const unsigned int* __restrict__ flag, const gm_loss_scale_t* __restrict__ state,
                                  const float2* __restrict__ table, int table_len, StepPrep* __restrict__ prep) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const int tstep = state->adam_t + 1;
    const float2 bc = table[tstep < table_len ? tstep : table_len];
    publish_prep(prep, flag[0] != 0u ? 1u : 0u, state->scale, bc, 1.0f);
}

struct MixedScalars { float lr, beta1, beta2, omb1, omb2, eps, wd; int use_wd; };

template <bool FAST, bool CLIP>
__device__ __forceinline__ void mixed_elem(float g16_as_f32, float inv_scale, float clip, float& w, float& m, float& v,
                                           unsigned short& p16, const AdamRule::P& p) {
    float x[4] = {w, mul(g16_as_f32, inv_scale), m, v};
    if (CLIP) x[1] = mul(x[1], clip);
    AdamRule::elem_t<FAST>(x, p);
    w = x[0]; m = x[2]; v = x[3];
    p16 = __half_as_ushort(__float2half_rn(x[0]));
}

__device__ __forceinline__ float half_bits_to_float(unsigned short h) { return __half2float(__ushort_as_half(h)); }

// 256-bit accesses: eight consecutive fp32 values per thread, 32-byte aligned.
struct F8 { float v[8]; };
__device__ __forceinline__ F8 ld256(const float* p) {
    F8 r;
    asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7]) : "l"(p));
    return r;
}
__device__ __forceinline__ void st256(float* p, const F8& r) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7]) : "memory");
}

// WIDE: 8 elements per thread per pass with 256-bit fp32 accesses (else 4 with a software
// prefetch).  FAST: the divisions by the two bias corrections use div_const when the
// published scalars allow it.  PF: while a pass is computed, the lines of the next pass
// are requested into L2 (no registers held).  CLIP: gradients are multiplied by the
// published clipping coefficient.  PUSH: every new fp16 parameter vector is also stored to
// the same offset of each peer's fp16 arena (sharded step; plain stores over NVLink).
template <bool WIDE, int MINB, bool FAST, bool PF, bool CLIP, bool PUSH>
__global__ void __launch_bounds__(kApplyThreads, MINB)
mixed_update_kernel(const DevList L, gm_loss_scale_t* __restrict__ state, unsigned int* __restrict__ flag,
                    const StepPrep* __restrict__ prep, const MixedScalars sc, const PeerDst peers) {
    constexpr int NT = kApplyThreads;
    const int tid = threadIdx.x;
    const int T = L.num_tensors;
    const long long chunk = L.chunk_elems;

    // Under programmatic stream serialization this CTA may start while the check
    // grid is still draining: warm L2 with the first vectors it will read, then wait
    // for the check grid to complete (a no-op after an ordinary launch).
    if (blockIdx.x < L.num_chunks) {
        const int2 rec = __ldg(L.chunk_rec + blockIdx.x);
        const int t = rec.x;
        const int h = __ldg(L.head + t);
        if (h >= 0) {
            const long long off = (long long)h + (long long)rec.y * chunk + 4LL * tid;
            if (off + 4 <= __ldg(L.numel + t)) {
#pragma unroll
                for (int s = 1; s < 4; ++s) {
                    const float* a = reinterpret_cast<const float*>(__ldg(L.ptrs + s * (size_t)T + t)) + off;
                    asm volatile("prefetch.global.L2 [%0];" :: "l"(a));
                }
            }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // The step's scalars were published by the check kernel; the loss-scale
    // state itself is only rewritten by the CTA that finishes last.
    const uint4 raw = *reinterpret_cast<const uint4*>(prep);
    const uint4 raw2 = *(reinterpret_cast<const uint4*>(prep) + 1);
    const unsigned overflow = raw.x;

    if (!overflow) {
        AdamRule::P p;
        p.lr = sc.lr; p.beta1 = sc.beta1; p.beta2 = sc.beta2; p.omb1 = sc.omb1; p.omb2 = sc.omb2;
        p.bc1 = __uint_as_float(raw.z); p.bc2 = __uint_as_float(raw.w);
        p.rbc1 = __uint_as_float(raw2.x); p.rbc2 = __uint_as_float(raw2.y);
        p.eps = sc.eps; p.wd = sc.wd; p.use_wd = sc.use_wd;
        const float inv_scale = __uint_as_float(raw.y);
        const float clip = __uint_as_float(raw2.z);
        const bool fast = FAST && raw2.w != 0u;           // uniform over the grid

        for (int c = blockIdx.x; c < L.num_chunks; c += gridDim.x) {
            const int2 rec = __ldg(L.chunk_rec + c);
            const int t = rec.x, k = rec.y;
            const long long n = __ldg(L.numel + t);
            const int h = __ldg(L.head + t);
            const unsigned short* g = reinterpret_cast<const unsigned short*>(__ldg(L.ptrs + 0 * (size_t)T + t));
            float* w = reinterpret_cast<float*>(__ldg(L.ptrs + 1 * (size_t)T + t));
            float* m = reinterpret_cast<float*>(__ldg(L.ptrs + 2 * (size_t)T + t));
            float* v = reinterpret_cast<float*>(__ldg(L.ptrs + 3 * (size_t)T + t));
            unsigned short* o = reinterpret_cast<unsigned short*>(__ldg(L.ptrs + 4 * (size_t)T + t));

            auto scalar_at = [&](long long i) {
                float wi = w[i], mi = m[i], vi = v[i];
                unsigned short pi;
                mixed_elem<false, CLIP>(half_bits_to_float(g[i]), inv_scale, clip, wi, mi, vi, pi, p);
                w[i] = wi; m[i] = mi; v[i] = vi; o[i] = pi;
                if (PUSH) {
                    for (int r = 0; r < peers.count; ++r)
                        *reinterpret_cast<unsigned short*>(reinterpret_cast<char*>(o + i) + peers.delta[r]) = pi;
                }
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

            // The 256-bit accesses need the fp32 streams on a 32-byte boundary.  The alignment peel
            // guarantees 16 bytes; 32 follow whenever the streams of a tensor share one element
            // offset (the fp16 streams then force a multiple of 8 elements), which is the usual
            // packing.  A tensor whose streams sit at different offsets can miss it and takes the
            // 4-element path below.
            int rot = 0;                                   // PUSH: the peer this thread's next pass addresses first
            if (PUSH && peers.count > 1) rot = ((tid >> 5) + c) % peers.count;
            const bool wide_ok = WIDE && (((reinterpret_cast<uintptr_t>(w + b) | reinterpret_cast<uintptr_t>(m + b) |
                                            reinterpret_cast<uintptr_t>(v + b)) & 31) == 0);
            if (wide_ok) {
                // 8 consecutive elements per thread per pass: one 16-byte access on the fp16
                // streams, one 32-byte access on each fp32 stream, all loads before the arithmetic
                const int nv8 = (int)((e - b) >> 3);
                const uint4* gq8 = reinterpret_cast<const uint4*>(g + b);
                uint4* oq8 = reinterpret_cast<uint4*>(o + b);
                for (int i = tid; i < nv8; i += NT) {
                    const uint4 gc = __ldcs(gq8 + i);
                    F8 W = ld256(w + b + 8LL * i), M = ld256(m + b + 8LL * i), V = ld256(v + b + 8LL * i);
                    if (PF && i + NT < nv8 && (tid & 3) == 0) {
                        // four threads share a 128-byte line of each fp32 stream: one of them asks for
                        // the line the four will load in the next pass
                        const long long nx = b + 8LL * (i + NT);
                        asm volatile("prefetch.global.L2 [%0];" :: "l"(w + nx));
                        asm volatile("prefetch.global.L2 [%0];" :: "l"(m + nx));
                        asm volatile("prefetch.global.L2 [%0];" :: "l"(v + nx));
                    }
                    const unsigned gw[4] = {gc.x, gc.y, gc.z, gc.w};
                    unsigned ow[4];
                    if (fast) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            unsigned short lo, hi;
                            mixed_elem<true, CLIP>(half_bits_to_float((unsigned short)(gw[j] & 0xffffu)), inv_scale, clip, W.v[2 * j], M.v[2 * j], V.v[2 * j], lo, p);
                            mixed_elem<true, CLIP>(half_bits_to_float((unsigned short)(gw[j] >> 16)), inv_scale, clip, W.v[2 * j + 1], M.v[2 * j + 1], V.v[2 * j + 1], hi, p);
                            ow[j] = (unsigned)lo | ((unsigned)hi << 16);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            unsigned short lo, hi;
                            mixed_elem<false, CLIP>(half_bits_to_float((unsigned short)(gw[j] & 0xffffu)), inv_scale, clip, W.v[2 * j], M.v[2 * j], V.v[2 * j], lo, p);
                            mixed_elem<false, CLIP>(half_bits_to_float((unsigned short)(gw[j] >> 16)), inv_scale, clip, W.v[2 * j + 1], M.v[2 * j + 1], V.v[2 * j + 1], hi, p);
                            ow[j] = (unsigned)lo | ((unsigned)hi << 16);
                        }
                    }
                    st256(w + b + 8LL * i, W); st256(m + b + 8LL * i, M); st256(v + b + 8LL * i, V);
                    const uint4 packed = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    if (PUSH) {
                        // the first peer rotates with the warp and the pass, so that the warps of an SM do
                        // not all address the same peer at the same moment
                        int idx = rot;
                        for (int r = 0; r < peers.count; ++r) {
                            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(oq8 + i) + peers.delta[idx]) = packed;
                            idx = idx + 1 == peers.count ? 0 : idx + 1;
                        }
                        rot = rot + 1 == peers.count ? 0 : rot + 1;
                    }
                    __stcs(oq8 + i, packed);
                }
                const long long tb8 = b + ((long long)nv8 << 3);
                if (tb8 + tid < e) scalar_at(tb8 + tid);
                continue;
            }
            // 4 elements per thread per pass: one 8-byte access on the fp16 streams,
            // one 16-byte access on each fp32 stream; the next pass's loads are
            // issued before this pass's arithmetic.
            const int nvec = (int)((e - b) >> 2);
            const uint2* gq = reinterpret_cast<const uint2*>(g + b);
            float4* wq = reinterpret_cast<float4*>(w + b);
            float4* mq = reinterpret_cast<float4*>(m + b);
            float4* vq = reinterpret_cast<float4*>(v + b);
            uint2* oq = reinterpret_cast<uint2*>(o + b);
            int i = tid;
            uint2 gc; float4 wc, mc, vc;
            if (i < nvec) { gc = __ldcs(gq + i); wc = __ldcs(wq + i); mc = __ldcs(mq + i); vc = __ldcs(vq + i); }
            while (i < nvec) {
                const int nx = i + NT;
                uint2 gn; float4 wn, mn, vn;
                if (nx < nvec) { gn = __ldcs(gq + nx); wn = __ldcs(wq + nx); mn = __ldcs(mq + nx); vn = __ldcs(vq + nx); }
                unsigned short h0, h1, h2, h3;
                mixed_elem<false, CLIP>(half_bits_to_float((unsigned short)(gc.x & 0xffffu)), inv_scale, clip, wc.x, mc.x, vc.x, h0, p);
                mixed_elem<false, CLIP>(half_bits_to_float((unsigned short)(gc.x >> 16)), inv_scale, clip, wc.y, mc.y, vc.y, h1, p);
                mixed_elem<false, CLIP>(half_bits_to_float((unsigned short)(gc.y & 0xffffu)), inv_scale, clip, wc.z, mc.z, vc.z, h2, p);
                mixed_elem<false, CLIP>(half_bits_to_float((unsigned short)(gc.y >> 16)), inv_scale, clip, wc.w, mc.w, vc.w, h3, p);
                __stcs(wq + i, wc); __stcs(mq + i, mc); __stcs(vq + i, vc);
                const uint2 packed = make_uint2((unsigned)h0 | ((unsigned)h1 << 16), (unsigned)h2 | ((unsigned)h3 << 16));
                if (PUSH) {
                    int idx = rot;
                    for (int r = 0; r < peers.count; ++r) {
                        *reinterpret_cast<uint2*>(reinterpret_cast<char*>(oq + i) + peers.delta[idx]) = packed;
                        idx = idx + 1 == peers.count ? 0 : idx + 1;
                    }
                    rot = rot + 1 == peers.count ? 0 : rot + 1;
                }
                __stcs(oq + i, packed);
                gc = gn; wc = wn; mc = mn; vc = vn;
                i = nx;
            }
            const long long tb = b + ((long long)nvec << 2);
            if (tb + tid < e) scalar_at(tb + tid);
        }
    }

    // last CTA to arrive runs the loss-scale state machine
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned ticket = atomicAdd(flag + 1, 1u);
        if (ticket == gridDim.x - 1) {
            gm_loss_scale_t s = *state;
            if (overflow) {
                s.scale = mul(s.scale, s.backoff);
                s.good_steps = 0;
                s.skipped += 1;
                s.last_overflow = 1;
            } else {
                s.adam_t += 1;
                s.last_overflow = 0;
                s.good_steps += 1;
                if (s.good_steps >= s.interval) {
                    float grown = mul(s.scale, s.growth);
                    if (grown > s.max_scale) grown = s.max_scale;
                    s.scale = grown;
                    s.good_steps = 0;
                }
            }
            *state = s;
            flag[0] = 0u;
            flag[1] = 0u;
            __threadfence();
        }
    }
}

}  // namespace gm
#include "gm_mixed_ring.cuh"
namespace gm {

// ---- sum of squares (grad-norm): warp shuffle tree, one float atomic per CTA ----
template <bool HALF>
__global__ void __launch_bounds__(kApplyThreads)
sumsq_kernel(const DevList L, float inv_scale, float* __restrict__ out) {
    constexpr int NT = kApplyThreads;
    const int tid = threadIdx.x;
    const long long chunk = L.chunk_elems;
    float acc = 0.0f;
    for (int c = blockIdx.x; c < L.num_chunks; c += gridDim.x) {
        const int2 rec = __ldg(L.chunk_rec + c);
        const int t = rec.x, k = rec.y;
        const long long n = __ldg(L.numel + t);
        const int h = __ldg(L.head + t);
        const long long hh = h > 0 ? h : 0;
        const long long b = (long long)k * chunk + (k > 0 ? hh : 0);     // chunk 0 also takes the h elements before the boundary
        long long e = (long long)(k + 1) * chunk + hh;
        if (e > n) e = n;
        constexpr int V = HALF ? 8 : 4;                                  // elements per 16-byte access
        // [b, a0) before the 16-byte boundary, [a0, a0 + nvec*V) in 16-byte accesses, the rest one by one
        const long long a0 = h < 0 ? e : (k == 0 ? (hh < e ? hh : e) : b);
        const long long nvec = h < 0 ? 0 : (e - a0) / V;
        const long long tail = a0 + nvec * V;
        if (HALF) {
            const unsigned short* g = reinterpret_cast<const unsigned short*>(__ldg(L.ptrs + t));
            for (long long i = b + tid; i < a0; i += NT) acc = sumsq1(g[i], inv_scale, acc);
            const uint4* q = reinterpret_cast<const uint4*>(g + a0);
            for (long long i = tid; i < nvec; i += 2 * NT) {
                const uint4 v0 = __ldcs(q + i);
                const uint4 v1 = i + NT < nvec ? __ldcs(q + i + NT) : make_uint4(0u, 0u, 0u, 0u);
                acc = sumsq8(v1, inv_scale, sumsq8(v0, inv_scale, acc));
            }
            for (long long i = tail + tid; i < e; i += NT) acc = sumsq1(g[i], inv_scale, acc);
        } else {
            const float* g = reinterpret_cast<const float*>(__ldg(L.ptrs + t));
            auto one = [&](long long i) { const float x = g[i] * inv_scale; acc = fmaf(x, x, acc); };
            for (long long i = b + tid; i < a0; i += NT) one(i);
            const float4* q = reinterpret_cast<const float4*>(g + a0);
            for (long long i = tid; i < nvec; i += 2 * NT) {
                const float4 v0 = __ldcs(q + i);
                const float4 v1 = i + NT < nvec ? __ldcs(q + i + NT) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float x[8] = {v0.x * inv_scale, v0.y * inv_scale, v0.z * inv_scale, v0.w * inv_scale,
                                    v1.x * inv_scale, v1.y * inv_scale, v1.z * inv_scale, v1.w * inv_scale};
#pragma unroll
                for (int j = 0; j < 8; ++j) acc = fmaf(x[j], x[j], acc);
            }
            for (long long i = tail + tid; i < e; i += NT) one(i);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    __shared__ float warp_sum[NT / 32];
    if ((tid & 31) == 0) warp_sum[tid >> 5] = acc;
    __syncthreads();
    if (tid == 0) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) total += warp_sum[w];
        atomicAdd(out, total);
    }
}

// One mixed-precision step.  `hook`, when given, runs between the check and the
// update kernels with the device address of the overflow word, so that a sharded
// caller can combine the flag across ranks on the same stream.
int mixed_step_with_hook(uintptr_t device_ptr, uintptr_t mixed, uintptr_t list, float lr, float eps, float wd,
                         int (*hook)(void* ctx, unsigned int* d_flag), void* ctx, const PeerDst* push) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    Mixed* m = as_mixed(mixed);
    TensorList* l = as_list(list);
    if (!m || !l) return GM_ERR_BAD_ARG;
    if (m->dev != d || l->dev != d) { set_error("handles belong to different devices"); return GM_ERR_BAD_ARG; }
    if (l->dl.num_streams != 5 || l->elem_bytes[0] != 2 || l->elem_bytes[1] != 4 || l->elem_bytes[2] != 4
        || l->elem_bytes[3] != 4 || l->elem_bytes[4] != 2) {
        set_error("mixed-precision list must be g16(2B), master, m, v (4B), p16(2B)");
        return GM_ERR_BAD_ARG;
    }
    // The device counter can be at most `calls` before this step; make sure the
    // table reaches calls+1 unless its tail is already constant.
    {
        const int rc = grow_table(m);
        if (rc != GM_OK) return rc;
    }
    m->calls += 1;
    MixedScalars sc;
    sc.lr = lr; sc.beta1 = m->beta1; sc.beta2 = m->beta2; sc.omb1 = 1.0f - m->beta1; sc.omb2 = 1.0f - m->beta2;
    sc.eps = eps; sc.wd = wd; sc.use_wd = wd > 0.0f ? 1 : 0;
    const bool clipping = m->max_norm > 0.0f;
    if (clipping && hook) {
        set_error("clipping is not available in the sharded mixed-precision step: the norm would cover one rank's shard only");
        return GM_ERR_UNSUPPORTED;
    }
    const bool norm = m->want_norm || clipping;
    if (norm) {
        const int rc = ensure_partials(d, l->dl.num_chunks);
        if (rc != GM_OK) return rc;
    }
    DeviceGuard g(d);
    int grid_c = check_grid(d, l->dl.num_chunks, norm);
    StepPrep* prep = reinterpret_cast<StepPrep*>(m->d_flag + 16);
    const int check_flags = (d->mixed_keep_g ? 1 : 0) | (d->mixed_overlap == 1 ? 2 : 0);

    // The ring kernels (gm_mixed_ring.cuh): 2 = the whole step as one cooperative launch, 1 = the
    // check kernel followed by the ring update.  They carry neither the norm nor the clipping, and
    // the sharded step needs the flag exchange between check and update, so those keep two launches.
    int ring = d->mixed_ring;
    if (norm || push) ring = 0;
    if (hook && ring == 2) ring = 1;
    if (l->dl.chunk_elems % kCheckElems) ring = 0;
    using RingFn = void (*)(const DevList, gm_loss_scale_t*, unsigned int*, StepPrep*, const MixedScalars, const float2*,
                            const int, const unsigned, const int, const long long);
    RingFn ring_fn = nullptr;
    int ring_grid = 0;
    if (ring) {
        ring_fn = ring == 2 ? (d->mixed_fastdiv ? mixed_ring_kernel<true, true> : mixed_ring_kernel<true, false>)
                            : (d->mixed_fastdiv ? mixed_ring_kernel<false, true> : mixed_ring_kernel<false, false>);
        static thread_local std::set<const void*> prepared;
        if (!prepared.count((const void*)ring_fn)) {
            GM_CUDA_CHECK(cudaFuncSetAttribute((const void*)ring_fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingBytes));
            prepared.insert((const void*)ring_fn);
        }
        int per_sm = 0;
        GM_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)ring_fn, kApplyThreads, kRingBytes));
        if (per_sm < 1) { ring = 0; }
        const long long tiles = (long long)l->dl.num_chunks * (l->dl.chunk_elems / kTileElems);
        ring_grid = (int)std::min<long long>((long long)per_sm * d->sm_count, tiles);
        if (ring_grid < 1) ring_grid = 1;
    }
    if (ring == 2) {
        int coop = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, d->ordinal);
        if (!coop) ring = 1;
    }
    if (ring == 2) {
        m->epoch += 1;
        DevList dl = l->dl;
        gm_loss_scale_t* st = m->d_state;
        unsigned int* fl = m->d_flag;
        const float2* tb = m->d_table;
        int tlen = m->table_len;
        unsigned ep = m->epoch;
        int kg = check_flags;
        long long budget = d->barrier_budget_cycles;
        void* args[] = {&dl, &st, &fl, &prep, &sc, &tb, &tlen, &ep, &kg, &budget};
        GM_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)ring_fn, dim3(ring_grid), dim3(kApplyThreads), args, kRingBytes, d->stream));
        d->launches++;
        return GM_OK;
    }
    if (norm)
        mixed_check_kernel<true><<<grid_c, kApplyThreads, 0, d->stream>>>(l->dl, m->d_flag, m->d_state, m->d_table, m->table_len,
                                                                          prep, check_flags, d->partials, clipping ? m->max_norm : 0.0f);
    else
        mixed_check_kernel<false><<<grid_c, kApplyThreads, 0, d->stream>>>(l->dl, m->d_flag, m->d_state, m->d_table, m->table_len,
                                                                           prep, check_flags, nullptr, 0.0f);
    d->launches++;
    if (hook) {
        int rc = hook(ctx, m->d_flag);
        if (rc != GM_OK) return rc;
        mixed_prep_kernel<<<1, 32, 0, d->stream>>>(m->d_flag, m->d_state, m->d_table, m->table_len, prep);
        d->launches++;
    }
    if (push && clipping) { set_error("clipping is not available in the sharded mixed-precision step"); return GM_ERR_UNSUPPORTED; }
    using UpdateFn = void (*)(const DevList, gm_loss_scale_t*, unsigned int*, const StepPrep*, const MixedScalars, const PeerDst);
    PeerDst peers{};
    if (push) peers = *push;
    // Variant 0 (default): 8 elements per thread with 256-bit fp32 accesses, the divisions by the
    // bias corrections through div_const, next-pass L2 prefetch.  GOMETAL_MIXED_FASTDIV=0 and
    // GOMETAL_MIXED_PF=0 switch the last two off; GOMETAL_MIXED_VARIANT=1 selects the older
    // 4-elements-per-thread kernel with a software prefetch.  All produce the same bits.
    UpdateFn update;
    if (push) {
        const int sel = (d->mixed_fastdiv ? 1 : 0) | (d->mixed_pf ? 2 : 0);
        switch (sel) {
            case 0: update = mixed_update_kernel<true, 4, false, false, false, true>; break;
            case 1: update = mixed_update_kernel<true, 4, true, false, false, true>; break;
            case 2: update = mixed_update_kernel<true, 4, false, true, false, true>; break;
            default: update = mixed_update_kernel<true, 4, true, true, false, true>; break;
        }
    } else if (d->mixed_variant == 1) {
        update = clipping ? mixed_update_kernel<false, 4, false, false, true, false> : mixed_update_kernel<false, 4, false, false, false, false>;
    } else {
        const int sel = (d->mixed_fastdiv ? 1 : 0) | (d->mixed_pf ? 2 : 0) | (clipping ? 4 : 0);
        switch (sel) {
            case 0: update = mixed_update_kernel<true, 4, false, false, false, false>; break;
            case 1: update = mixed_update_kernel<true, 4, true, false, false, false>; break;
            case 2: update = mixed_update_kernel<true, 4, false, true, false, false>; break;
            case 3: update = mixed_update_kernel<true, 4, true, true, false, false>; break;
            case 4: update = mixed_update_kernel<true, 4, false, false, true, false>; break;
            case 5: update = mixed_update_kernel<true, 4, true, false, true, false>; break;
            case 6: update = mixed_update_kernel<true, 4, false, true, true, false>; break;
            default: update = mixed_update_kernel<true, 4, true, true, true, false>; break;
        }
    }
    int grid_u = launch_grid(d, (const void*)update, kApplyThreads, l->dl.num_chunks);
    if (ring == 1) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(ring_grid); cfg.blockDim = dim3(kApplyThreads); cfg.dynamicSmemBytes = kRingBytes; cfg.stream = d->stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        if (!hook && d->mixed_overlap) { cfg.attrs = &attr; cfg.numAttrs = 1; }
        GM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, ring_fn, l->dl, m->d_state, m->d_flag, prep, sc, (const float2*)m->d_table, m->table_len,
                                         0u, check_flags, d->barrier_budget_cycles));
        d->launches++;
        GM_CUDA_CHECK(cudaGetLastError());
        return GM_OK;
    }
    if (!hook && d->mixed_overlap) {
        // the update grid may become resident while the check grid drains
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid_u); cfg.blockDim = dim3(kApplyThreads); cfg.dynamicSmemBytes = 0; cfg.stream = d->stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        GM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, update, l->dl, m->d_state, m->d_flag, (const StepPrep*)prep, sc, peers));
    } else {
        update<<<grid_u, kApplyThreads, 0, d->stream>>>(l->dl, m->d_state, m->d_flag, prep, sc, peers);
    }
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    return GM_OK;
}

}  // namespace gm

using namespace gm;

extern "C" {

uintptr_t gm_mixed_create(uintptr_t device_ptr, const gm_loss_scale_t* initial, float beta1, float beta2,
                          int table_steps) {
    Device* d = as_device(device_ptr);
    if (!d) return 0;
    gm_loss_scale_t init;
    if (initial) {
        init = *initial;
    } else {                                   // training/model_trainer.go:258-270
        init.scale = 65536.0f; init.growth = 2.0f; init.backoff = 0.5f; init.max_scale = 16777216.0f;
        init.interval = 2000; init.good_steps = 0; init.adam_t = 0; init.skipped = 0; init.last_overflow = 0;
    }
    if (!valid_loss_scale(init)) {
        set_error("invalid loss-scale configuration (scale %g growth %g backoff %g interval %d max %g)",
                  (double)init.scale, (double)init.growth, (double)init.backoff, init.interval, (double)init.max_scale);
        return 0;
    }
    if (!(beta1 >= 0.0f && beta1 < 1.0f && beta2 >= 0.0f && beta2 < 1.0f)) {
        set_error("betas must lie in [0,1)");
        return 0;
    }
    Mixed* m = new Mixed();
    m->dev = d; m->beta1 = beta1; m->beta2 = beta2;
    m->calls = init.adam_t;
    DeviceGuard g(d);
    cudaError_t e = cudaMalloc((void**)&m->d_state, 256);
    if (e == cudaSuccess) e = cudaMalloc((void**)&m->d_flag, 256);
    if (e == cudaSuccess) e = cudaMemset(m->d_flag, 0, 256);
    if (e == cudaSuccess) e = cudaMemcpy(m->d_state, &init, sizeof(init), cudaMemcpyHostToDevice);
    if (e != cudaSuccess || upload_table(m, table_steps > 0 ? table_steps : 32768) != GM_OK || grow_table(m) != GM_OK) {
        if (e != cudaSuccess) cuda_fail(e, "mixed state allocation");
        if (m->d_state) cudaFree(m->d_state);
        if (m->d_flag) cudaFree(m->d_flag);
        if (m->d_table) cudaFree(m->d_table);
        delete m;
        return 0;
    }
    std::lock_guard<std::mutex> lk(g_mixed_mu);
    g_mixed.insert(m);
    return (uintptr_t)m;
}

void gm_mixed_destroy(uintptr_t h) {
    Mixed* m = as_mixed(h);
    if (!m) return;
    {
        std::lock_guard<std::mutex> lk(g_mixed_mu);
        g_mixed.erase(m);
    }
    DeviceGuard g(m->dev);
    cudaStreamSynchronize(m->dev->stream);
    cudaFree(m->d_state); cudaFree(m->d_flag); cudaFree(m->d_table);
    delete m;
}

int gm_mixed_step_async(uintptr_t device_ptr, uintptr_t mixed, uintptr_t list, float lr, float eps, float wd) {
    return gm::mixed_step_with_hook(device_ptr, mixed, list, lr, eps, wd, nullptr, nullptr);
}

int gm_mixed_get_state(uintptr_t device_ptr, uintptr_t mixed, gm_loss_scale_t* out) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    Mixed* m = as_mixed(mixed);
    if (!m || !out) { if (m) set_error("output is nil"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    GM_CUDA_CHECK(cudaMemcpy(out, m->d_state, sizeof(*out), cudaMemcpyDeviceToHost));
    unsigned int ctl[3] = {0, 0, 0};                          // arrive count, go epoch, error word
    GM_CUDA_CHECK(cudaMemcpy(ctl, m->d_flag + kCtlArrive, sizeof(ctl), cudaMemcpyDeviceToHost));
    if (ctl[2]) {
        // a grid-barrier wait of the single-launch step ran out: put the control block back in its
        // initial state so that the handle stays usable, and tell the caller
        GM_CUDA_CHECK(cudaMemset(m->d_flag, 0, 256));
        m->epoch = 0;
        set_error("a grid-barrier wait of the mixed-precision step ran out; that step's buffers are partly updated");
        return GM_ERR_TIMEOUT;
    }
    return GM_OK;
}

int gm_mixed_set_state(uintptr_t device_ptr, uintptr_t mixed, const gm_loss_scale_t* in) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    Mixed* m = as_mixed(mixed);
    if (!m || !in) { if (m) set_error("input is nil"); return GM_ERR_BAD_ARG; }
    if (!valid_loss_scale(*in)) {
        set_error("invalid loss-scale state (scale %g growth %g backoff %g interval %d max %g step %d)", (double)in->scale,
                  (double)in->growth, (double)in->backoff, in->interval, (double)in->max_scale, in->adam_t);
        return GM_ERR_BAD_ARG;
    }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    GM_CUDA_CHECK(cudaMemcpy(m->d_state, in, sizeof(*in), cudaMemcpyHostToDevice));
    m->calls = in->adam_t;
    return grow_table(m);
}

int gm_mixed_enable_grad_norm(uintptr_t mixed, int enable) {
    Mixed* m = as_mixed(mixed);
    if (!m) return GM_ERR_BAD_ARG;
    m->want_norm = enable ? 1 : 0;
    return GM_OK;
}

// A bounded device-side wait on a word that nothing sets: it must give up after
// budget_cycles and report it (gave_up = 1), leaving the context usable.
int gm_selftest_barrier_timeout(uintptr_t device_ptr, long long budget_cycles, int* gave_up) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!gave_up || budget_cycles <= 0 || budget_cycles > (1LL << 33)) { set_error("bad self-test arguments"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    unsigned* word = reinterpret_cast<unsigned*>(d->scalars + 40);
    int* status = reinterpret_cast<int*>(d->scalars + 41);
    GM_CUDA_CHECK(cudaMemsetAsync(word, 0, 8, d->stream));
    barrier_timeout_selftest_kernel<<<1, 32, 0, d->stream>>>(word, budget_cycles, status);
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    GM_CUDA_CHECK(cudaMemcpy(gave_up, status, sizeof(int), cudaMemcpyDeviceToHost));
    return GM_OK;
}

int gm_mixed_set_clip(uintptr_t mixed, float max_norm) {
    Mixed* m = as_mixed(mixed);
    if (!m) return GM_ERR_BAD_ARG;
    if (!(max_norm >= 0.0f) || !isfinite(max_norm)) { set_error("max_norm %g must be finite and >= 0 (0 turns clipping off)", (double)max_norm); return GM_ERR_BAD_ARG; }
    m->max_norm = max_norm;
    return GM_OK;
}

int gm_mixed_last_clip(uintptr_t device_ptr, uintptr_t mixed, float* out_sumsq, float* out_coef) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    Mixed* m = as_mixed(mixed);
    if (!m || !out_sumsq || !out_coef) { if (m) set_error("output is nil"); return GM_ERR_BAD_ARG; }
    if (!(m->max_norm > 0.0f) && !m->want_norm) { set_error("neither clipping nor the gradient norm is enabled on this state"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    float two[2];
    GM_CUDA_CHECK(cudaMemcpy(two, m->d_flag + 24, sizeof(two), cudaMemcpyDeviceToHost));
    *out_sumsq = two[0];
    *out_coef = two[1];
    return GM_OK;
}

int gm_mixed_last_grad_sumsq(uintptr_t device_ptr, uintptr_t mixed, float* out) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    Mixed* m = as_mixed(mixed);
    if (!m || !out) { if (m) set_error("output is nil"); return GM_ERR_BAD_ARG; }
    if (!m->want_norm && !(m->max_norm > 0.0f)) { set_error("the gradient norm is not enabled on this mixed-precision state"); return GM_ERR_BAD_ARG; }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    GM_CUDA_CHECK(cudaMemcpy(out, m->d_flag + 24, sizeof(float), cudaMemcpyDeviceToHost));
    return GM_OK;
}

uintptr_t gm_mixed_state_device_ptr(uintptr_t mixed) {
    Mixed* m = as_mixed(mixed);
    return m ? (uintptr_t)m->d_state : 0;
}

int gm_grad_sumsq_async(uintptr_t device_ptr, uintptr_t list, int elem_bytes, float inv_scale, uintptr_t out) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    TensorList* l = as_list(list);
    if (!l) return GM_ERR_BAD_ARG;
    if (!out) { set_error("output buffer is nil"); return GM_ERR_NIL_BUFFER; }
    if (elem_bytes != l->elem_bytes[0] || (elem_bytes != 2 && elem_bytes != 4)) {
        set_error("gradient stream holds %d-byte elements, caller said %d", l->elem_bytes[0], elem_bytes);
        return GM_ERR_BAD_ARG;
    }
    DeviceGuard g(d);
    GM_CUDA_CHECK(cudaMemsetAsync((void*)out, 0, sizeof(float), d->stream));
    if (elem_bytes == 2) {
        int grid = launch_grid(d, (const void*)sumsq_kernel<true>, kApplyThreads, l->dl.num_chunks);
        sumsq_kernel<true><<<grid, kApplyThreads, 0, d->stream>>>(l->dl, inv_scale, (float*)out);
    } else {
        int grid = launch_grid(d, (const void*)sumsq_kernel<false>, kApplyThreads, l->dl.num_chunks);
        sumsq_kernel<false><<<grid, kApplyThreads, 0, d->stream>>>(l->dl, inv_scale, (float*)out);
    }
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    return GM_OK;
}

}  // extern "C"

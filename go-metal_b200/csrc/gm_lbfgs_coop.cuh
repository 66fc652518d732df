// gm_lbfgs_coop.cuh -- one L-BFGS step as ONE cooperative launch with the direction
// vector kept on chip.  Included by gm_lbfgs.cu (it uses LbfgsTable and the column layout).
//
// MEASURED SLOWER than the multi-launch step and therefore not the default (n = 10^7,
// history 10 on B200: 0.815 ms per step against 0.507 ms; "lbfgs_coop" of
// gm_device_set_tuning selects it).  What it shows: at this size the direction vector
// fills the chip -- 13 chunks of shared memory and 32 registers per thread on every SM --
// and what is left cannot keep enough loads in flight: 512 threads with 64 bytes each are
// 32 KB per SM where a B200 needs about 100 KB to stream at full rate, so a pass costs
// ~37 us instead of the 23 us of the multi-launch pass that re-reads the direction from L2.
// It stays in the library as the step that needs one launch, and for the bounded grid
// barrier it carries.
//
// The multi-launch step (gm_lbfgs.cu) runs 2h+2 passes; in each loop pass the direction
// is read and rewritten (through L2, where it is kept resident) while two history vectors
// stream in from DRAM.  Here the direction never leaves the SMs between passes: every CTA
// owns the 4096-element chunks b, b+G, b+2G, ... (G = one CTA per SM) and holds them for
// the whole step -- up to 13 chunks in shared memory (208 KB) and 4 in registers (two per
// group of 256 threads, 32 values per thread).  A pass then only streams its history
// vectors; the sum a pass needs from all CTAs goes through the chunk sums in global memory
// and one grid-wide barrier, after which EVERY CTA adds the chunk sums in the fixed order
// itself and applies the epilogue, so no second barrier is needed to hand the scalar back.
//
// The chunk -> lane map, the xor tree, the order of the warp sums and of the chunk sums
// are those of the multi-launch kernels, and so is every statement on an element: the two
// produce the same bits (the parity tests run both).
//
// Capacity: 17 chunks per SM, i.e. 17 * 148 * 4096 = 10,305,536 elements on B200; longer
// problems, more than kCoopMaxHistory pairs, or a device without cooperative launch take
// the multi-launch step.  Every barrier wait is bounded; a wait that runs out sets the
// error word, the CTA stops taking part (its chunks keep the values of the last finished
// pass) and the host reports GM_ERR_TIMEOUT.
#pragma once

namespace gm {

constexpr int kCoopThreads = 512;                                  // 128 registers per thread: no spills
constexpr int kCoopGroups = kCoopThreads / kDotThreads;            // 2 groups of 256 lanes
constexpr int kCoopRegChunks = 4;                                  // per CTA: two per group, 32 registers per thread
constexpr int kCoopSmemChunks = 13;
constexpr int kCoopMaxChunksPerCta = kCoopSmemChunks + kCoopRegChunks; // 17
constexpr int kCoopMaxHistory = 12;
constexpr int kCoopMaxPasses = 2 * kCoopMaxHistory + 2;
constexpr size_t kCoopSmemBytes = (size_t)kCoopSmemChunks * kDotChunk * sizeof(float);

// control words behind the device's ticket (Device::ticket is 64 words)
constexpr int kLbArrive = 8, kLbGo = 9, kLbError = 10;

// One pass of the step, with the scalars it reads and writes named by index instead of by
// address: values produced earlier in the same launch live in shared memory, not in global.
struct CoopPass {
    int kind;            // 0 dir = +-g, 1 dir -= c*vec, 2 dir += c*vec, 3 final update
    int col_axpy;        // kinds 1, 2: the vector
    int col_dot;         // column dotted with the new direction (-1: none)
    int rho_axpy;        // kinds 1, 2: history slot whose rho decides whether the pair is skipped
    int rho_dot;         // slot whose rho decides whether the dot is skipped and multiplies it (-1: none)
    int coef_alpha;      // kinds 1, 2: coefficient = alpha[coef_alpha] if >= 0, else the running coefficient
    int epilogue;        // 0 none, 1 alpha[out_alpha] = dot*rho, 2 coefficient = alpha[alpha_in] - dot*rho, 3 rho[prev] = 1/dot
    int out_alpha, alpha_in;
};

struct CoopPlan {
    CoopPass pass[kCoopMaxPasses];
    int num_passes;
    int history;                           // m
    int descent, corrected, have_pair;
    int col_s_new, col_y_prev, col_s_prev; // final pass
    float step;
    unsigned epoch_base;                   // barrier k of this launch is released with epoch_base + k
    const float* rho[kCoopMaxHistory];     // the rho buffers (one float each), by history slot
    float* alpha;                          // [m] alpha buffer
    float* rho_prev;                       // rho[prev], written by the final pass
    long long barrier_budget;
};

// Sum of the first 256 threads' values in the library's fixed order; every thread of the
// (1024-thread) CTA calls it, the result is returned to all of them.
__device__ __forceinline__ float coop_sum_first256(float acc, float* warp_sum, float* result) {
    if (threadIdx.x < kDotThreads) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc = add(acc, __shfl_xor_sync(0xffffffffu, acc, off));
        if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = warp_sum[0];
#pragma unroll
        for (int w = 1; w < kDotThreads / 32; ++w) total = add(total, warp_sum[w]);
        *result = total;
    }
    __syncthreads();
    return *result;
}

// Sum over the 256 lanes of one group (named barrier 1 + group); valid in the group's lane 0.
__device__ __forceinline__ float coop_group_sum(float acc, float* warp_sum8, const int group, const int lane) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = add(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if ((lane & 31) == 0) warp_sum8[lane >> 5] = acc;
    asm volatile("bar.sync %0, %1;" :: "r"(1 + group), "r"(kDotThreads) : "memory");
    float total = 0.0f;
    if (lane == 0) {
        total = warp_sum8[0];
#pragma unroll
        for (int w = 1; w < kDotThreads / 32; ++w) total = add(total, warp_sum8[w]);
    }
    asm volatile("bar.sync %0, %1;" :: "r"(1 + group), "r"(kDotThreads) : "memory");
    return total;
}

// What a group needs to know about one chunk.
struct CoopChunk {
    int t;
    long long n, base;
    bool fast;                 // a whole chunk, 16-byte aligned in every column
};

__device__ __forceinline__ CoopChunk coop_locate(const LbfgsTable& tb, const int c) {
    CoopChunk r;
    r.t = find_tensor(tb.chunk_prefix, tb.T, c);
    r.n = __ldg(tb.numel + r.t);
    r.base = (long long)(c - __ldg(tb.chunk_prefix + r.t)) * kDotChunk;
    r.fast = __ldg(tb.aligned + r.t) != 0 && r.base + kDotChunk <= r.n;
    return r;
}

// Ragged end of a tensor, or columns off a 16-byte boundary: element by element in the same
// order.  Rare (at most one chunk per tensor, or tensors a caller misaligned), so these are
// real calls with the chunk's direction values passed through memory: d16[i * 4 + k] is
// element (i*256+lane)*4+k.
__device__ __noinline__ float coop_loop_chunk_slow(const float* src, const float* vec, const float* dv, const long long base,
                                                   const long long n, const int kind, const int descent, const float coef,
                                                   const int lane, float* d16) {
    float acc = 0.0f;
    for (int i = 0; i < 4; ++i) {
        const long long e0 = base + ((long long)i * kDotThreads + lane) * 4;
        for (int k = 0; k < 4; ++k) {
            const long long e = e0 + k;
            float x = d16[i * 4 + k];
            if (e < n) {
                if (kind == 0) x = descent ? src[e] : -src[e];
                else if (vec) x = kind == 1 ? sub(x, mul(coef, vec[e])) : add(x, mul(coef, vec[e]));
                if (dv) acc = add(acc, mul(dv[e], x));
            } else {
                x = 0.0f;
            }
            d16[i * 4 + k] = x;
        }
    }
    return acc;
}

struct CoopFinalPtrs { float* x; const float* g; float* og; float* dirg; float* s_new; float* y_prev; const float* s_prev; };

__device__ __noinline__ float coop_final_chunk_slow(const CoopFinalPtrs q, const long long base, const long long n, const float step,
                                                    const int have_pair, const int corrected, const int same_slot, const int lane,
                                                    float* d16) {
    float acc = 0.0f;
    for (int i = 0; i < 4; ++i) {
        const long long e0 = base + ((long long)i * kDotThreads + lane) * 4;
        for (int k = 0; k < 4; ++k) {
            const long long e = e0 + k;
            if (e < n) {
                const float p = -d16[i * 4 + k];
                d16[i * 4 + k] = p;
                q.dirg[e] = p;
                const float sv = mul(step, p);
                q.x[e] = add(q.x[e], sv);
                const float gv = q.g[e];
                if (have_pair) {
                    const float spv = same_slot ? sv : q.s_prev[e];
                    float yv;
                    if (corrected) yv = sub(gv, q.og[e]);
                    else yv = sub(gv, gv);
                    q.y_prev[e] = yv;
                    acc = add(acc, mul(spv, yv));
                }
                q.og[e] = gv;
                q.s_new[e] = sv;
            }
        }
    }
    return acc;
}

__device__ __forceinline__ void f4_to_mem(const float4 (&d)[4], float* m) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { m[i * 4] = d[i].x; m[i * 4 + 1] = d[i].y; m[i * 4 + 2] = d[i].z; m[i * 4 + 3] = d[i].w; }
}
__device__ __forceinline__ void f4_from_mem(float4 (&d)[4], const float* m) {
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = make_float4(m[i * 4], m[i * 4 + 1], m[i * 4 + 2], m[i * 4 + 3]);
}

// Kinds 0, 1, 2 on one chunk whose direction values are d[0..3] (lane t holds elements
// (i*256+t)*4 .. +3 in d[i]).  Returns this lane's share of the dot product.
__device__ __forceinline__ float coop_loop_chunk(const LbfgsTable& tb, const CoopChunk& ck, const int kind, const int descent,
                                                 const bool has_vec, const bool want_dot, const int col_axpy, const int col_dot,
                                                 const float coef, const int lane, float4 (&d)[4]) {
    const int T = tb.T;
    auto col = [&](int cidx) -> const float* { return reinterpret_cast<const float*>(__ldg(tb.ptrs + (size_t)cidx * T + ck.t)); };
    const float* src = kind == 0 ? col(COL_G) : nullptr;
    const float* vec = has_vec ? col(col_axpy) : nullptr;
    const float* dv = want_dot ? col(col_dot) : nullptr;
    float acc = 0.0f;
    auto new_dir = [&](float d_old, float v) -> float { return kind == 1 ? sub(d_old, mul(coef, v)) : add(d_old, mul(coef, v)); };
    if (ck.fast) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float4 s4[2], v4[2], o4[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const long long e0 = ck.base + ((long long)(2 * half + u) * kDotThreads + lane) * 4;
                if (kind == 0) s4[u] = __ldcs(reinterpret_cast<const float4*>(src + e0));
                if (has_vec) v4[u] = __ldcs(reinterpret_cast<const float4*>(vec + e0));
                if (want_dot) o4[u] = __ldcs(reinterpret_cast<const float4*>(dv + e0));
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                float4& x = d[2 * half + u];
                if (kind == 0) {
                    x = descent ? s4[u] : make_float4(-s4[u].x, -s4[u].y, -s4[u].z, -s4[u].w);
                } else if (has_vec) {
                    x = make_float4(new_dir(x.x, v4[u].x), new_dir(x.y, v4[u].y), new_dir(x.z, v4[u].z), new_dir(x.w, v4[u].w));
                }
                if (want_dot) {
                    acc = add(acc, mul(o4[u].x, x.x)); acc = add(acc, mul(o4[u].y, x.y));
                    acc = add(acc, mul(o4[u].z, x.z)); acc = add(acc, mul(o4[u].w, x.w));
                }
            }
        }
    } else {
        float m16[16];
        f4_to_mem(d, m16);
        acc = coop_loop_chunk_slow(src, vec, dv, ck.base, ck.n, kind, descent, coef, lane, m16);
        f4_from_mem(d, m16);
    }
    return acc;
}

// The final pass on one chunk: p = -r is written to the direction buffer, x += step*p,
// s[hi] = step*p, y[prev] = g - old_g (or g - g in the reference's statement order),
// old_g = g; returns this lane's share of s[prev].y[prev].  Statement for statement the
// kind-3 branch of lbfgs_pass_kernel.
__device__ __forceinline__ float coop_final_chunk(const LbfgsTable& tb, const CoopChunk& ck, const CoopPlan& plan, const int lane,
                                                  float4 (&d)[4]) {
    const int T = tb.T;
    auto col = [&](int cidx) -> float* { return reinterpret_cast<float*>(__ldg(tb.ptrs + (size_t)cidx * T + ck.t)); };
    float* x = col(COL_W);
    const float* g = col(COL_G);
    float* og = col(COL_OLDG);
    float* dirg = col(COL_DIR);
    float* s_new = col(plan.col_s_new);
    float* y_prev = plan.have_pair ? col(plan.col_y_prev) : nullptr;
    const float* s_prev = plan.have_pair ? col(plan.col_s_prev) : nullptr;
    const bool same_slot = plan.col_s_prev == plan.col_s_new;
    const float step = plan.step;
    float acc = 0.0f;
    if (ck.fast) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long e0 = ck.base + ((long long)i * kDotThreads + lane) * 4;
            float4 xv = *reinterpret_cast<float4*>(x + e0);
            const float4 gv = *reinterpret_cast<const float4*>(g + e0);
            float4 ov = make_float4(0.f, 0.f, 0.f, 0.f), sp = make_float4(0.f, 0.f, 0.f, 0.f);
            if (plan.have_pair && plan.corrected) ov = *reinterpret_cast<const float4*>(og + e0);
            if (plan.have_pair && !same_slot) sp = __ldcs(reinterpret_cast<const float4*>(s_prev + e0));
            float4 dv = d[i];
            dv.x = -dv.x; dv.y = -dv.y; dv.z = -dv.z; dv.w = -dv.w;
            const float4 sv = make_float4(mul(step, dv.x), mul(step, dv.y), mul(step, dv.z), mul(step, dv.w));
            xv.x = add(xv.x, sv.x); xv.y = add(xv.y, sv.y); xv.z = add(xv.z, sv.z); xv.w = add(xv.w, sv.w);
            if (plan.have_pair) {
                float4 yv;
                if (plan.corrected) yv = make_float4(sub(gv.x, ov.x), sub(gv.y, ov.y), sub(gv.z, ov.z), sub(gv.w, ov.w));
                else yv = make_float4(sub(gv.x, gv.x), sub(gv.y, gv.y), sub(gv.z, gv.z), sub(gv.w, gv.w));
                if (same_slot) sp = sv;
                acc = add(acc, mul(sp.x, yv.x)); acc = add(acc, mul(sp.y, yv.y));
                acc = add(acc, mul(sp.z, yv.z)); acc = add(acc, mul(sp.w, yv.w));
                *reinterpret_cast<float4*>(y_prev + e0) = yv;
            }
            *reinterpret_cast<float4*>(dirg + e0) = dv;
            *reinterpret_cast<float4*>(x + e0) = xv;
            *reinterpret_cast<float4*>(og + e0) = gv;
            *reinterpret_cast<float4*>(s_new + e0) = sv;
            d[i] = dv;
        }
    } else {
        float m16[16];
        f4_to_mem(d, m16);
        const CoopFinalPtrs q = {x, g, og, dirg, s_new, y_prev, s_prev};
        acc = coop_final_chunk_slow(q, ck.base, ck.n, step, plan.have_pair, plan.corrected, same_slot ? 1 : 0, lane, m16);
        f4_from_mem(d, m16);
    }
    return acc;
}

__global__ void __launch_bounds__(kCoopThreads, 1)
lbfgs_coop_kernel(const LbfgsTable tb, const CoopPlan plan, float* __restrict__ partials, unsigned int* __restrict__ ctl) {
    extern __shared__ float4 sdir[];                 // [slot][1024]: lane t's d[i] of a chunk at [i * 256 + t]
    __shared__ float s_warp[kCoopGroups][kDotThreads / 32];     // per-group scratch of the chunk sums
    __shared__ float s_red[kDotThreads / 32];
    __shared__ float s_result;
    __shared__ float s_alpha[kCoopMaxHistory];
    __shared__ float s_coef;
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    const int group = tid >> 8, lane = tid & (kDotThreads - 1);
    const int G = gridDim.x;
    const int count = (int)blockIdx.x < tb.num_chunks ? (tb.num_chunks - (int)blockIdx.x + G - 1) / G : 0;
    const int reg_first = count > kCoopRegChunks ? count - kCoopRegChunks : 0;   // local chunks from here on live in registers
    // this group's register chunks: the local indices >= reg_first of its parity
    const int li_a = reg_first + ((group - reg_first) & 1);
    const int li_b = li_a + kCoopGroups;
    float4 dreg_a[4], dreg_b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { dreg_a[i] = make_float4(0.f, 0.f, 0.f, 0.f); dreg_b[i] = dreg_a[i]; }
    if (tid < kCoopMaxHistory) s_alpha[tid] = 0.0f;
    if (tid == 0) s_coef = 0.0f;
    __syncthreads();

    unsigned barrier_no = 0;
    for (int pi = 0; pi < plan.num_passes; ++pi) {
        const CoopPass& ps = plan.pass[pi];
        const bool final_pass = ps.kind == 3;
        bool skip_axpy = false, want_dot = false, has_vec = false;
        float coef = 0.0f, rho_dot = 0.0f;
        if (!final_pass) {
            skip_axpy = ps.kind != 0 && rho_skips(plan.rho[ps.rho_axpy]);
            want_dot = ps.col_dot >= 0 && !(ps.rho_dot >= 0 && rho_skips(plan.rho[ps.rho_dot]));
            has_vec = ps.kind != 0 && !skip_axpy;
            if (ps.kind != 0) coef = ps.coef_alpha >= 0 ? s_alpha[ps.coef_alpha] : s_coef;
            if (ps.rho_dot >= 0) rho_dot = *plan.rho[ps.rho_dot];
        } else {
            want_dot = plan.have_pair != 0;
        }

        // the chunk sums of consecutive barriers alternate between two buffers: a CTA that is
        // already writing the next pass's sums must not disturb one still adding up this pass's
        float* psum = partials + ((barrier_no + 1) & 1u) * (size_t)tb.num_chunks;
        // one chunk of this group, its direction values in d
        auto run_chunk = [&](const int li, float4 (&d)[4]) {
            const int c = blockIdx.x + li * G;
            const CoopChunk ck = coop_locate(tb, c);
            const float acc = final_pass ? coop_final_chunk(tb, ck, plan, lane, d)
                                         : coop_loop_chunk(tb, ck, ps.kind, plan.descent, has_vec, want_dot, ps.col_axpy, ps.col_dot, coef, lane, d);
            if (want_dot) {
                const float total = coop_group_sum(acc, s_warp[group], group, lane);
                if (lane == 0) psum[c] = total;
            }
        };
        if (final_pass || ps.kind == 0 || has_vec || want_dot) {
            for (int li = group; li < reg_first; li += kCoopGroups) {
                float4* slot = sdir + (size_t)li * (kDotChunk / 4) + lane;
                float4 d[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) d[i] = slot[i * kDotThreads];
                run_chunk(li, d);
                if (!final_pass && (ps.kind == 0 || has_vec)) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) slot[i * kDotThreads] = d[i];
                }
            }
            if (li_a < count) run_chunk(li_a, dreg_a);
            if (li_b < count) run_chunk(li_b, dreg_b);
        }
        if (ps.epilogue == 0) continue;

        // every CTA's chunk sums are needed: one bounded grid-wide barrier, then every CTA adds
        // them up itself in the fixed order
        float dot = 0.0f;
        if (want_dot) {
            barrier_no += 1;
            __syncthreads();
            if (tid == 0) {
                int ok = 1;
                __threadfence();
                const unsigned arrived = atomicAdd(ctl + kLbArrive, 1u);
                if (arrived == (unsigned)G - 1u) {
                    ctl[kLbArrive] = 0u;
                    __threadfence();
                    st_release(ctl + kLbGo, plan.epoch_base + barrier_no);
                } else if (!bounded_wait_for(ctl + kLbGo, plan.epoch_base + barrier_no, plan.barrier_budget)) {
                    atomicExch(ctl + kLbError, 1u);
                    ok = 0;
                }
                s_ok = ok;
            }
            __syncthreads();
            if (!s_ok) return;
            float acc = 0.0f;
            if (tid < kDotThreads)
                for (int c = tid; c < tb.num_chunks; c += kDotThreads) acc = add(acc, __ldcg(psum + c));
            dot = coop_sum_first256(acc, s_red, &s_result);
        }
        if (tid == 0) {
            float r = 0.0f;
            switch (ps.epilogue) {
                case 1: r = want_dot ? mul(dot, rho_dot) : 0.0f; break;
                case 2: r = want_dot ? sub(s_alpha[ps.alpha_in], mul(dot, rho_dot)) : 0.0f; break;
                default: r = (plan.have_pair && fabs((double)dot) > 1e-10) ? dvd(1.0f, dot) : 0.0f; break;
            }
            if (ps.epilogue == 1) { s_alpha[ps.out_alpha] = r; if (blockIdx.x == 0) plan.alpha[ps.out_alpha] = r; }
            else if (ps.epilogue == 2) s_coef = r;
            else if (blockIdx.x == 0) *plan.rho_prev = r;
        }
        __syncthreads();
    }
}

// ---- the step as one launch with the direction left in L2 ("lbfgs_coop" = 2) ----
// The same passes as the multi-launch step, by the same chunk walk (axpy_dot_walk) with the
// direction read and written through L2 under the evict_last policy, but inside ONE
// cooperative launch.  A CTA walks the same chunks in every pass, so it only ever reads
// direction values it wrote itself; the only thing that crosses CTAs is the dot product, and
// that travels as tagged 64-bit words (see the pass loop), collected by every CTA under the
// first loads of its next pass.  The idea: trade the fixed cost of a pass (launch, table
// warm-up, finisher, drain) for that exchange.  MEASURED per step at n = 10^7, m = 10, same
// box: 0.561 ms with a counter barrier (fence, atomic arrival, go word) waited for before the
// next pass's loads; 0.537 ms with the wait moved under those loads; 0.510 ms with the tagged
// words (floor of a pass 6.3 -> 5.9 -> 4.4 us); against 0.477 ms for the multi-launch step,
// whose passes leave their final sum to the next launch in the same way.  What is left is the
// 126 registers the walk needs inside the pass loop: two CTAs per SM instead of three (at 80
// registers it spills in its inner loop: 0.775 ms), and the passes stream slower for it.  Not
// the default.
#ifndef GM_LBFGS_FUSED_MINB
#define GM_LBFGS_FUSED_MINB 2      // 128 registers: at 3 CTAs per SM (80 registers) the walk spills inside its loop
#endif
__global__ void __launch_bounds__(kDotThreads, GM_LBFGS_FUSED_MINB)
lbfgs_fused_kernel(const LbfgsTable tb, const CoopPlan plan, unsigned long long* __restrict__ tagged,
                   unsigned int* __restrict__ ctl, const int keep_dir) {
    __shared__ float warp_sum[kDotThreads / 32];
    __shared__ float s_alpha[kCoopMaxHistory];
    __shared__ float s_coef;
    __shared__ float s_dot;
    const int tid = threadIdx.x;
    const int G = gridDim.x;
    const unsigned long long pol = l2_policy(keep_dir != 0);
    if (tid < kCoopMaxHistory) s_alpha[tid] = 0.0f;
    if (tid == 0) s_coef = 0.0f;
    __syncthreads();

    // A pass's dot product is finished inside the NEXT pass.  The producer writes every chunk sum
    // as ONE 64-bit word {barrier epoch, sum} (a single relaxed store at GPU scope: the tag and
    // the value arrive together, so there is no fence, no arrival counter and no go word).  The
    // consumer first issues the loads of its first chunk -- the history columns are read-only
    // and a CTA only reads direction values it wrote itself, so they depend on nobody -- and
    // only then collects the sums: lane t spins, bounded, on the words of chunks t, t+256, ...
    // which are exactly the ones it adds up, in that order.  Two halves alternate with the
    // barriers, so a word is only overwritten after every CTA has read it.
    unsigned barrier_no = 0;
    bool pending = false;                 // chunk sums have been written and not yet collected
    int pend_epilogue = 0, pend_alpha_in = -1, pend_out_alpha = -1;
    float pend_rho = 0.0f;
    bool failed = false;
    auto publish = [&](const int epilogue, const bool have, const float dot, const float rho_dot, const int alpha_in,
                       const int out_alpha) {
        if (tid == 0) {
            float r = 0.0f;
            switch (epilogue) {
                case 1: r = have ? mul(dot, rho_dot) : 0.0f; break;
                case 2: r = have ? sub(s_alpha[alpha_in], mul(dot, rho_dot)) : 0.0f; break;
                default: r = (plan.have_pair && fabs((double)dot) > 1e-10) ? dvd(1.0f, dot) : 0.0f; break;
            }
            if (epilogue == 1) { s_alpha[out_alpha] = r; if (blockIdx.x == 0) plan.alpha[out_alpha] = r; }
            else if (epilogue == 2) s_coef = r;
            else if (blockIdx.x == 0) *plan.rho_prev = r;
        }
        __syncthreads();
    };
    auto slots_of = [&](const unsigned barrier) { return tagged + (size_t)(barrier & 1u) * (size_t)tb.num_chunks; };
    auto resolve = [&]() {
        if (!pending) return;
        pending = false;
        const unsigned epoch = plan.epoch_base + barrier_no;
        const unsigned long long* slots = slots_of(barrier_no);
        const long long t0 = clock64();
        float acc = 0.0f;
        int ok = 1;
        for (int c = tid; c < tb.num_chunks && ok; c += kDotThreads) {
            unsigned long long w = ld_relaxed_u64(slots + c);
            while ((unsigned)(w >> 32) != epoch) {
                if (clock64() - t0 > plan.barrier_budget) { ok = 0; break; }
                __nanosleep(32);
                w = ld_relaxed_u64(slots + c);
            }
            if (ok) acc = add(acc, __uint_as_float((unsigned)w));
        }
        if (!__syncthreads_and(ok)) {
            if (tid == 0) atomicExch(ctl + kLbError, 1u);
            failed = true;
            return;
        }
        const float total = cta_reduce_256(acc, warp_sum);
        if (tid == 0) s_dot = total;
        __syncthreads();
        publish(pend_epilogue, true, s_dot, pend_rho, pend_alpha_in, pend_out_alpha);
    };

    for (int pi = 0; pi < plan.num_passes; ++pi) {
        const CoopPass& ps = plan.pass[pi];
        const bool final_pass = ps.kind == 3;
        // the half no CTA can still be reading: it alternates with the barriers, not with the passes
        unsigned long long* slots_out = slots_of(barrier_no + 1u);
        const unsigned long long tag_out = (unsigned long long)(plan.epoch_base + barrier_no + 1u) << 32;
        auto store = [&](int c, float v) { st_relaxed_u64(slots_out + c, tag_out | (unsigned long long)__float_as_uint(v)); };
        bool want_dot = false;
        float rho_dot = 0.0f;
        if (!final_pass) {
            const bool skip_axpy = ps.kind != 0 && rho_skips(plan.rho[ps.rho_axpy]);
            want_dot = ps.col_dot >= 0 && !(ps.rho_dot >= 0 && rho_skips(plan.rho[ps.rho_dot]));
            const bool has_vec = ps.kind != 0 && !skip_axpy;
            const bool writes = ps.kind == 0 || !skip_axpy;
            if (ps.rho_dot >= 0) rho_dot = *plan.rho[ps.rho_dot];
            axpy_dot_walk(tb, ps.kind, plan.descent, ps.col_axpy, ps.col_dot, 1, pol, store, warp_sum, blockIdx.x, G,
                          []() {},
                          [&]() -> WalkArgs {
                              resolve();
                              float coef = 0.0f;
                              if (ps.kind != 0) coef = ps.coef_alpha >= 0 ? s_alpha[ps.coef_alpha] : s_coef;
                              // after a wait that ran out the pass is skipped and the kernel returns below
                              return WalkArgs{coef, has_vec && !failed, want_dot && !failed, writes && !failed};
                          });
            if (failed) return;
        } else {
            resolve();
            if (failed) return;
            want_dot = plan.have_pair != 0;
            for (int c = blockIdx.x; c < tb.num_chunks; c += G) {
                const CoopChunk ck = coop_locate(tb, c);
                const float* dirg = reinterpret_cast<const float*>(__ldg(tb.ptrs + (size_t)COL_DIR * tb.T + ck.t));
                float4 d[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const long long e0 = ck.base + ((long long)i * kDotThreads + tid) * 4;
                    if (ck.fast) {
                        d[i] = ld_l2(dirg + e0, pol);
                    } else {
                        d[i] = make_float4(e0 < ck.n ? dirg[e0] : 0.f, e0 + 1 < ck.n ? dirg[e0 + 1] : 0.f,
                                           e0 + 2 < ck.n ? dirg[e0 + 2] : 0.f, e0 + 3 < ck.n ? dirg[e0 + 3] : 0.f);
                    }
                }
                const float acc = coop_final_chunk(tb, ck, plan, tid, d);
                if (want_dot) {
                    const float total = cta_reduce_256(acc, warp_sum);
                    if (tid == 0) store(c, total);
                }
            }
        }
        if (ps.epilogue == 0) continue;
        if (!want_dot) {
            publish(ps.epilogue, false, 0.0f, rho_dot, ps.alpha_in, ps.out_alpha);     // the scalar is zero
            continue;
        }
        barrier_no += 1;
        pending = true;
        pend_epilogue = ps.epilogue; pend_alpha_in = ps.alpha_in; pend_out_alpha = ps.out_alpha;
        pend_rho = rho_dot;
    }
    resolve();                                            // the final pass's s.y -> rho
}

}  // namespace gm

// gm_lbfgs.cu -- L-BFGS two-loop recursion with fixed-order dot products.
//
// Replaces execute_lbfgs_step_mpsgraph (cgo_bridge/bridge_optimizer.m:980-1321),
// whose body is scalar CPU loops over buffer contents.  The statement order of
// that function is kept (q=-g, first loop newest->oldest, identity initial
// Hessian, second loop oldest->newest, p=-r, fixed step, x+=step*p, old_g<-g,
// s[hi]=step*p, y[prev]=g-old_g, rho[prev]=1/(s.y) if |s.y|>1e-10 else 0;
// pairs with |rho|<1e-10 are skipped).  What changes is how it runs:
//
//  * every pass over the vectors is one multi-tensor launch; the axpy of one
//    history pair is fused with the dot product the next pair needs, so a
//    pair costs 16 B/element instead of 20;
//  * all scalars (rho, alpha, beta, the skip decisions) stay on the device;
//  * dot products use one fixed summation order, independent of the grid:
//    4096-element chunks, inside a chunk lane t of 256 adds the products of
//    elements (i*256+t)*4+k (i=0..3, k=0..3) in that order, the 32 lanes of a
//    warp combine with an xor tree (16,8,4,2,1), the 8 warp sums are added in
//    ascending order; the CTA that finishes last adds the chunk sums (lane t
//    takes chunks t, t+256, ... then the same tree).  Products are rounded to
//    fp32 before every add (no fused multiply-add, no float atomics).
//
// The mode is a bit set.  Bit 0: y[prev] is formed from the previous gradient
// before old_g is overwritten (the reference overwrites first, :1232-1239, so
// its y is always zero and every curvature pair is rejected).  Bit 1: the
// recursion starts from q = +g, so p = -H*g descends (the reference starts
// from q = -g, :1026-1038, and negates again at :1204-1213, which moves along
// +H*g).  Mode 0 is the reference's statement order; mode 3, the default, is a
// working L-BFGS.
#include <math.h>
#include <string.h>

#include <map>

#include "gm_apply.cuh"

namespace gm {

constexpr int kDotChunk = 4096;
constexpr int kDotThreads = 256;
#ifndef GM_LBFGS_MINB
#define GM_LBFGS_MINB 3          // resident CTAs per SM the axpy+dot kernel is compiled for (4 would spill)
#endif
#ifndef GM_LBFGS_PASS_MINB
#define GM_LBFGS_PASS_MINB 4     // the final-update / plain-dot kernel needs fewer registers
#endif

struct LbfgsTable {
    const unsigned long long* ptrs;   // [ncols][T]
    const long long* numel;           // [T]
    const int* chunk_prefix;          // [T+1]
    const int* aligned;               // [T] every column of the tensor is 16-byte aligned
    int T, num_chunks, ncols;
};

// column layout of the pointer table
constexpr int COL_W = 0, COL_G = 1, COL_OLDG = 2, COL_DIR = 3, COL_HIST = 4;   // then s[0..m), y[0..m)

struct LbfgsOp {
    int kind;                 // 0 init (dir=-g), 1 dir-=c*vec, 2 dir+=c*vec, 3 final update, 4 plain dot(colA,colB)
    int col_axpy;             // kinds 1,2: vector column; kind 4: first operand
    int col_dot;              // column dotted with the new direction (-1 none); kind 4: second operand
    const float* rho_axpy;    // kinds 1,2: the pair is skipped when |rho| < 1e-10
    const float* rho_dot;     // the dot is skipped when |rho| < 1e-10 (nullptr: never skipped)
    const float* coef;        // kinds 1,2: coefficient, read on the device
    int epilogue;             // 0 none, 1 out=dot*rho_dot, 2 out=alpha_in-dot*rho_dot, 3 out=1/dot if |dot|>1e-10 else 0, 4 out=dot
    float* out;
    const float* alpha_in;
    // kind 3
    int col_s_new, col_y_prev, col_s_prev, have_pair, corrected;
    int descent;              // kind 0: dir = +g instead of -g
    int keep_dir;             // kinds 0..2: the direction's lines get the evict_last L2 policy
    int early_trigger;        // kinds 0..2: dependents may launch from the start of this grid (else from its end)
    // The scalar a pass with epilogue 1 or 2 produces is only ever read by the pass launched right
    // after it.  With `defer` set the producer stops after writing its chunk sums (no ticket, no
    // finishing CTA) and the consumer, told by pro_epilogue, starts by adding them up itself, every
    // CTA for itself in the fixed order, while its first direction loads are already in flight.
    int defer;                // kinds 0..2: the epilogue is left to the next pass
    int pro_epilogue;         // kinds 1,2: epilogue of the previous pass to perform first (0: read *coef instead)
    const float* pro_rho_dot; // the previous pass's rho_dot
    const float* pro_alpha_in;
    float* pro_out;           // where CTA 0 stores the scalar for later passes and for the caller
    int part_in, part_out;    // which half of the chunk-sum buffer is read by the prologue / written by this pass
    int prewait;              // kinds 1,2: history loads issued before the wait for the previous pass (0 none, 1 first chunk, 2 + L2 prefetch of the second)
    float step;
};

__device__ __forceinline__ bool rho_skips(const float* rho) {
    // bridge_optimizer.m:1066: fabs(rho_j) < 1e-10, evaluated in double
    return rho != nullptr && fabs((double)(*rho)) < 1e-10;
}

// Sum of the 256 lane values of a CTA in the documented order; result valid in thread 0.
__device__ __forceinline__ float cta_reduce_256(float acc, float* warp_sum) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = add(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.0f;
    if (threadIdx.x == 0) {
        total = warp_sum[0];
#pragma unroll
        for (int w = 1; w < kDotThreads / 32; ++w) total = add(total, warp_sum[w]);
    }
    __syncthreads();
    return total;
}

// The CTA that takes the last ticket sees every chunk sum, finishes the
// reduction in the fixed order and applies the epilogue to the scalar.
__device__ __forceinline__ void finish_pass(const LbfgsTable& tb, const LbfgsOp& op, const bool have_dot,
                                            float* partials, unsigned int* ticket, float* warp_sum, int* is_last) {
    if (op.epilogue == 0) return;
    const int tid = threadIdx.x;
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned my = atomicAdd(ticket, 1u);
        *is_last = (my == gridDim.x - 1);
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();

    float dot = 0.0f;
    if (have_dot) {
        float acc = 0.0f;
        const volatile float* pv = partials;
        for (int c = tid; c < tb.num_chunks; c += kDotThreads) acc = add(acc, pv[c]);
        dot = cta_reduce_256(acc, warp_sum);
    }
    if (tid == 0) {
        float r = 0.0f;
        switch (op.epilogue) {
            case 1: r = have_dot ? mul(dot, *op.rho_dot) : 0.0f; break;                         // alpha_j
            case 2: r = have_dot ? sub(*op.alpha_in, mul(dot, *op.rho_dot)) : 0.0f; break;      // alpha_j - beta
            case 3: r = (op.have_pair && fabs((double)dot) > 1e-10) ? dvd(1.0f, dot) : 0.0f; break;
            default: r = dot; break;
        }
        *op.out = r;
        *ticket = 0u;
        __threadfence();
    }
}

__global__ void __launch_bounds__(kDotThreads, GM_LBFGS_PASS_MINB)
lbfgs_pass_kernel(const LbfgsTable tb, const LbfgsOp op, float* __restrict__ partials,
                  unsigned int* __restrict__ ticket) {
    __shared__ float warp_sum[kDotThreads / 32];
    __shared__ int is_last;
    const int tid = threadIdx.x;
    const int T = tb.T;

    // kinds 3 (final update) and 4 (plain dot); kinds 0..2 run in lbfgs_axpy_dot_kernel
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");          // no effect after an ordinary launch
    const bool want_dot = op.col_dot >= 0 && !rho_skips(op.rho_dot) && (op.kind != 3 || op.have_pair);

    {
        for (int c = blockIdx.x; c < tb.num_chunks; c += gridDim.x) {
            const int t = find_tensor(tb.chunk_prefix, T, c);
            const long long n = __ldg(tb.numel + t);
            const long long base = (long long)(c - __ldg(tb.chunk_prefix + t)) * kDotChunk;
            const bool vec_ok = __ldg(tb.aligned + t) != 0;
            auto col = [&](int cidx) -> float* {
                return reinterpret_cast<float*>(__ldg(tb.ptrs + (size_t)cidx * T + t));
            };
            float* dir = op.kind == 4 ? nullptr : col(COL_DIR);
            float acc = 0.0f;

            if (op.kind == 4) {
                const float* a = col(op.col_axpy);
                const float* b = col(op.col_dot);
#pragma unroll
                for (int i = 0; i < kDotChunk / (kDotThreads * 4); ++i) {
                    const long long e0 = base + ((long long)i * kDotThreads + tid) * 4;
                    if (vec_ok && e0 + 3 < n) {
                        const float4 av = *reinterpret_cast<const float4*>(a + e0);
                        const float4 bv = *reinterpret_cast<const float4*>(b + e0);
                        acc = add(acc, mul(av.x, bv.x)); acc = add(acc, mul(av.y, bv.y));
                        acc = add(acc, mul(av.z, bv.z)); acc = add(acc, mul(av.w, bv.w));
                    } else {
                        for (int k = 0; k < 4; ++k) if (e0 + k < n) acc = add(acc, mul(a[e0 + k], b[e0 + k]));
                    }
                }
            } else {
                float* x = col(COL_W);
                const float* g = col(COL_G);
                float* og = col(COL_OLDG);
                float* s_new = col(op.col_s_new);
                float* y_prev = op.have_pair ? col(op.col_y_prev) : nullptr;
                const float* s_prev = op.have_pair ? col(op.col_s_prev) : nullptr;
                const bool same_slot = op.col_s_prev == op.col_s_new;
                auto one = [&](long long e) {
                    const float p = -dir[e];
                    dir[e] = p;
                    const float sv = mul(op.step, p);
                    x[e] = add(x[e], sv);
                    const float gv = g[e];
                    if (op.have_pair) {
                        const float sp = same_slot ? sv : s_prev[e];
                        float yv;
                        if (op.corrected) yv = sub(gv, og[e]);        // previous gradient still in old_g
                        else yv = sub(gv, gv);                        // reference order: old_g already equals g
                        y_prev[e] = yv;
                        acc = add(acc, mul(sp, yv));
                    }
                    og[e] = gv;
                    s_new[e] = sv;
                };
#pragma unroll
                for (int i = 0; i < kDotChunk / (kDotThreads * 4); ++i) {
                    const long long e0 = base + ((long long)i * kDotThreads + tid) * 4;
                    if (vec_ok && e0 + 3 < n) {
                        float4 dv = *reinterpret_cast<float4*>(dir + e0);
                        float4 xv = *reinterpret_cast<float4*>(x + e0);
                        const float4 gv = *reinterpret_cast<const float4*>(g + e0);
                        dv.x = -dv.x; dv.y = -dv.y; dv.z = -dv.z; dv.w = -dv.w;
                        const float4 sv = make_float4(mul(op.step, dv.x), mul(op.step, dv.y), mul(op.step, dv.z), mul(op.step, dv.w));
                        xv.x = add(xv.x, sv.x); xv.y = add(xv.y, sv.y); xv.z = add(xv.z, sv.z); xv.w = add(xv.w, sv.w);
                        if (op.have_pair) {
                            float4 yv;
                            if (op.corrected) {
                                const float4 ov = *reinterpret_cast<const float4*>(og + e0);
                                yv = make_float4(sub(gv.x, ov.x), sub(gv.y, ov.y), sub(gv.z, ov.z), sub(gv.w, ov.w));
                            } else {
                                yv = make_float4(sub(gv.x, gv.x), sub(gv.y, gv.y), sub(gv.z, gv.z), sub(gv.w, gv.w));
                            }
                            const float4 sp = same_slot ? sv : __ldcs(reinterpret_cast<const float4*>(s_prev + e0));
                            acc = add(acc, mul(sp.x, yv.x)); acc = add(acc, mul(sp.y, yv.y));
                            acc = add(acc, mul(sp.z, yv.z)); acc = add(acc, mul(sp.w, yv.w));
                            *reinterpret_cast<float4*>(y_prev + e0) = yv;
                        }
                        *reinterpret_cast<float4*>(dir + e0) = dv;
                        *reinterpret_cast<float4*>(x + e0) = xv;
                        *reinterpret_cast<float4*>(og + e0) = gv;
                        *reinterpret_cast<float4*>(s_new + e0) = sv;
                    } else {
                        for (int k = 0; k < 4; ++k) if (e0 + k < n) one(e0 + k);
                    }
                }
            }

            if (want_dot || op.kind == 4) {
                const float total = cta_reduce_256(acc, warp_sum);
                if (tid == 0) partials[c] = total;
            }
        }
    }

    finish_pass(tb, op, want_dot || op.kind == 4, partials, ticket, warp_sum, &is_last);
}

// Kinds 0, 1 and 2: dir = -g | dir -= c*vec | dir += c*vec, fused with the dot
// product of the new direction and a second column.  Each CTA walks chunks
// blockIdx.x, blockIdx.x + gridDim.x, ...; the loads of its next chunk are issued
// before the current chunk's sum is reduced, so the shuffles, barriers and the
// table lookups run with a full set of loads in flight.  The chunk sums land in
// partials[chunk], so the summation order does not depend on the grid.
struct AxpyRef {
    float* dir;
    const float* src;        // kind 0: g; else dir
    const float* vec;
    const float* dv;
    long long base, n;
    bool fast;               // a whole chunk, 16-byte aligned in every column
};

// What a pass knows only once its predecessor has finished: the coefficient and which of its
// two halves the curvature test leaves standing.
struct WalkArgs {
    float coef;
    bool has_vec, want_dot, writes;
};

// The chunk walk shared by the multi-launch pass kernel and the single-launch step: kinds 0, 1
// and 2 over chunks first, first + stride, ...; the loads of the next chunk are issued before the
// current chunk's sum is reduced; thread 0 hands every chunk sum to store(chunk, sum).
//
// The history columns are read-only for the whole step, so the walk loads its first chunk of
// them (prewait >= 1) and asks L2 for its second (prewait >= 2) BEFORE it calls gate(), which
// in the multi-launch step is where the grid waits for its predecessor: while that grid's last
// CTA adds up the chunk sums, DRAM already works for this one.  Only the direction, the
// coefficient and the curvature test wait for the gate.
template <class Store, class Sync, class Gate>
__device__ __forceinline__ void axpy_dot_walk(const LbfgsTable& tb, const int kind, const int descent, const int col_axpy,
                                              const int col_dot, const int prewait, const unsigned long long pol,
                                              Store store, float* warp_sum, const int first,
                                              const int stride, Sync sync, Gate gate) {
    constexpr int PASSES = kDotChunk / (kDotThreads * 4);
    const int tid = threadIdx.x;
    const int T = tb.T;
    const bool may_vec = kind != 0 && col_axpy >= 0;
    const bool may_dot = col_dot >= 0;
    auto lookup = [&](int c) -> AxpyRef {
        AxpyRef r;
        const int t = find_tensor(tb.chunk_prefix, T, c);
        r.n = __ldg(tb.numel + t);
        r.base = (long long)(c - __ldg(tb.chunk_prefix + t)) * kDotChunk;
        r.fast = __ldg(tb.aligned + t) != 0 && r.base + kDotChunk <= r.n;
        auto col = [&](int cidx) -> float* { return reinterpret_cast<float*>(__ldg(tb.ptrs + (size_t)cidx * T + t)); };
        r.dir = col(COL_DIR);
        r.src = kind == 0 ? col(COL_G) : r.dir;
        r.vec = may_vec ? col(col_axpy) : nullptr;
        r.dv = may_dot ? col(col_dot) : nullptr;
        return r;
    };

    float4 d4[PASSES], v4[PASSES], o4[PASSES];
    // g and the history columns are read once per pass: streamed, so that dir stays in L2
    auto issue_hist = [&](const AxpyRef& r, const bool vec, const bool dot) {
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const long long e0 = r.base + ((long long)i * kDotThreads + tid) * 4;
            if (vec) v4[i] = __ldcs(reinterpret_cast<const float4*>(r.vec + e0));
            if (dot) o4[i] = __ldcs(reinterpret_cast<const float4*>(r.dv + e0));
        }
    };
    auto issue_dir = [&](const AxpyRef& r, const unsigned long long pol) {
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const long long e0 = r.base + ((long long)i * kDotThreads + tid) * 4;
            if (kind == 0) d4[i] = __ldcs(reinterpret_cast<const float4*>(r.src + e0));
            else d4[i] = ld_l2(r.src + e0, pol);
        }
    };

    int c = first;
    AxpyRef cur{}, nxt{};
    const bool any = c < tb.num_chunks;
    const bool early = prewait >= 1 && any;
    if (any) {
        cur = lookup(c);
        if (early && cur.fast) issue_hist(cur, may_vec, may_dot);
        if (c + stride < tb.num_chunks) {
            nxt = lookup(c + stride);
            if (prewait >= 2 && nxt.fast) {
                // one 64-byte piece of the chunk per thread and column
                if (may_vec) asm volatile("prefetch.global.L2 [%0];" :: "l"(nxt.vec + nxt.base + tid * 16LL));
                if (may_dot) asm volatile("prefetch.global.L2 [%0];" :: "l"(nxt.dv + nxt.base + tid * 16LL));
            }
        }
    }

    // sync(): the predecessor has finished.  The direction is loaded next, and gate() -- which may
    // have to add up the predecessor's chunk sums to know the coefficient -- runs under those loads.
    sync();
    if (any && cur.fast) issue_dir(cur, pol);
    const WalkArgs a = gate();
    if (!(a.writes || a.want_dot) || !any) return;
    auto new_dir = [&](float d_old, float v) -> float {
        return kind == 1 ? sub(d_old, mul(a.coef, v)) : add(d_old, mul(a.coef, v));
    };
    if (cur.fast && !early) issue_hist(cur, a.has_vec, a.want_dot);
    while (c < tb.num_chunks) {
        const int cn = c + stride;
        float acc = 0.0f;
        if (cur.fast) {
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
                const long long e0 = cur.base + ((long long)i * kDotThreads + tid) * 4;
                if (kind == 0) {
                    if (!descent) d4[i] = make_float4(-d4[i].x, -d4[i].y, -d4[i].z, -d4[i].w);
                } else if (a.has_vec) {
                    d4[i] = make_float4(new_dir(d4[i].x, v4[i].x), new_dir(d4[i].y, v4[i].y),
                                        new_dir(d4[i].z, v4[i].z), new_dir(d4[i].w, v4[i].w));
                }
                if (a.writes) st_l2(cur.dir + e0, d4[i], pol);
                if (a.want_dot) {
                    acc = add(acc, mul(o4[i].x, d4[i].x)); acc = add(acc, mul(o4[i].y, d4[i].y));
                    acc = add(acc, mul(o4[i].z, d4[i].z)); acc = add(acc, mul(o4[i].w, d4[i].w));
                }
            }
        } else {
            // ragged end of a tensor, or columns off a 16-byte boundary: element by
            // element, lane t still owning elements (i*256+t)*4+k in that order
            for (int i = 0; i < PASSES; ++i) {
                const long long e0 = cur.base + ((long long)i * kDotThreads + tid) * 4;
                for (int k = 0; k < 4; ++k) {
                    const long long e = e0 + k;
                    if (e < cur.n) {
                        float dn;
                        if (kind == 0) dn = descent ? cur.src[e] : -cur.src[e];
                        else dn = a.has_vec ? new_dir(cur.dir[e], cur.vec[e]) : cur.dir[e];
                        if (a.writes) cur.dir[e] = dn;
                        if (a.want_dot) acc = add(acc, mul(cur.dv[e], dn));
                    }
                }
            }
        }
        if (cn < tb.num_chunks && nxt.fast) {                   // in flight during the reduction below
            issue_hist(nxt, a.has_vec, a.want_dot);
            issue_dir(nxt, pol);
        }
        if (a.want_dot) {
            const float total = cta_reduce_256(acc, warp_sum);
            if (tid == 0) store(c, total);
        }
        c = cn;
        cur = nxt;
        if (c + stride < tb.num_chunks) nxt = lookup(c + stride);   // resolves while this chunk's loads arrive
    }
}


__global__ void __launch_bounds__(kDotThreads, GM_LBFGS_MINB)
lbfgs_axpy_dot_kernel(const LbfgsTable tb, const LbfgsOp op, float* __restrict__ partials,
                      unsigned int* __restrict__ ticket) {
    __shared__ float warp_sum[kDotThreads / 32];
    __shared__ float s_dot;
    __shared__ int is_last;
    const int kind = op.kind;
    const int tid = threadIdx.x;
    float* part_out = partials + (size_t)op.part_out * tb.num_chunks;
    const float* part_in = partials + (size_t)op.part_in * tb.num_chunks;

    // Launched with programmatic stream serialization (every pass of a step but the
    // first), this grid may become resident while the previous pass drains.  Only the
    // pointer table and the history columns, which no pass writes, are touched before
    // the wait; the scalars, the direction and the chunk sums are the previous pass's
    // to finish first.
    if (op.early_trigger) asm volatile("griddepcontrol.launch_dependents;");
    bool want_dot = false;
    auto sync = [&]() { asm volatile("griddepcontrol.wait;" ::: "memory"); };   // no effect after an ordinary launch
    auto gate = [&]() -> WalkArgs {
        const bool skip_axpy = kind != 0 && rho_skips(op.rho_axpy);
        WalkArgs a;
        a.want_dot = want_dot = op.col_dot >= 0 && !rho_skips(op.rho_dot);
        a.has_vec = kind != 0 && !skip_axpy;
        a.writes = kind == 0 || !skip_axpy;
        if (op.pro_epilogue != 0) {
            // the previous pass left its epilogue to this one: same order as finish_pass
            const bool have = !rho_skips(op.pro_rho_dot);
            float dot = 0.0f;
            if (have) {
                float acc = 0.0f;
                for (int c = tid; c < tb.num_chunks; c += kDotThreads) acc = add(acc, __ldcg(part_in + c));
                const float total = cta_reduce_256(acc, warp_sum);
                if (tid == 0) s_dot = total;
                __syncthreads();
                dot = s_dot;
            }
            float r = 0.0f;
            if (have) r = op.pro_epilogue == 1 ? mul(dot, *op.pro_rho_dot) : sub(*op.pro_alpha_in, mul(dot, *op.pro_rho_dot));
            if (blockIdx.x == 0 && tid == 0) *op.pro_out = r;
            a.coef = r;
        } else {
            a.coef = kind != 0 ? *op.coef : 0.0f;
        }
        return a;
    };
    axpy_dot_walk(tb, kind, op.descent, op.col_axpy, op.col_dot, kind == 0 ? 0 : op.prewait, l2_policy(op.keep_dir != 0),
                  [&](int c, float v) { part_out[c] = v; }, warp_sum, blockIdx.x, gridDim.x, sync, gate);
    if (!op.early_trigger) asm volatile("griddepcontrol.launch_dependents;");
    if (!op.defer) finish_pass(tb, op, want_dot, part_out, ticket, warp_sum, &is_last);
}

}  // namespace gm
#include "gm_lbfgs_coop.cuh"
namespace gm {

// ---- host side ----
struct LbfgsCtx {
    void* blob = nullptr;
    LbfgsTable tb{};
    std::vector<uintptr_t> key;      // every pointer + size, for exact comparison
    int history = 0;
    uint64_t validated_gen = 0;      // registry generation under which the buffer sizes were last checked
};

static std::mutex g_lb_mu;
static std::map<Device*, std::vector<LbfgsCtx*>> g_lb;
static std::map<Device*, LbfgsCtx*> g_lb_parked;   // the table evicted last, per device

static int get_ctx(Device* d, int T, int m, uintptr_t* const* cols4, uintptr_t* s_flat, uintptr_t* y_flat,
                   const int64_t* numel, LbfgsCtx** out) {
    const int ncols = COL_HIST + 2 * m;
    std::vector<uintptr_t> key;
    key.reserve((size_t)ncols * T + T + 2);
    key.push_back((uintptr_t)T); key.push_back((uintptr_t)m);
    for (int c = 0; c < 4; ++c) for (int t = 0; t < T; ++t) key.push_back(cols4[c][t]);
    for (int k = 0; k < m * T; ++k) key.push_back(s_flat[k]);
    for (int k = 0; k < m * T; ++k) key.push_back(y_flat[k]);
    for (int t = 0; t < T; ++t) key.push_back((uintptr_t)numel[t]);
    {
        std::lock_guard<std::mutex> lk(g_lb_mu);
        for (LbfgsCtx* c : g_lb[d]) if (c->key == key) { *out = c; return GM_OK; }
    }
    std::vector<unsigned long long> ptrs((size_t)ncols * T);
    std::vector<long long> n64(T);
    std::vector<int> prefix(T + 1), aligned(T);
    prefix[0] = 0;
    for (int t = 0; t < T; ++t) {
        bool al = true;
        for (int c = 0; c < 4; ++c) { ptrs[(size_t)c * T + t] = cols4[c][t]; al = al && cols4[c][t] % 16 == 0; }
        for (int k = 0; k < m; ++k) {
            ptrs[(size_t)(COL_HIST + k) * T + t] = s_flat[(size_t)k * T + t];
            ptrs[(size_t)(COL_HIST + m + k) * T + t] = y_flat[(size_t)k * T + t];
            al = al && s_flat[(size_t)k * T + t] % 16 == 0 && y_flat[(size_t)k * T + t] % 16 == 0;
        }
        aligned[t] = al ? 1 : 0;
        n64[t] = numel[t];
        int64_t nc = (numel[t] + kDotChunk - 1) / kDotChunk;
        if (prefix[t] + nc > 0x7fffffff) { set_error("L-BFGS problem too large"); return GM_ERR_BAD_SIZE; }
        prefix[t + 1] = prefix[t] + (int)nc;
    }
    size_t off_n = sizeof(unsigned long long) * ptrs.size();
    size_t off_p = off_n + sizeof(long long) * T;
    size_t off_a = off_p + sizeof(int) * (T + 1);
    size_t bytes = off_a + sizeof(int) * T;
    std::vector<unsigned char> host(bytes);
    memcpy(host.data(), ptrs.data(), off_n);
    memcpy(host.data() + off_n, n64.data(), sizeof(long long) * T);
    memcpy(host.data() + off_p, prefix.data(), sizeof(int) * (T + 1));
    memcpy(host.data() + off_a, aligned.data(), sizeof(int) * T);
    LbfgsCtx* c = new LbfgsCtx();
    DeviceGuard g(d);
    cudaError_t e = cudaMalloc(&c->blob, (bytes + 255) / 256 * 256);
    if (e == cudaSuccess) e = cudaMemcpy(c->blob, host.data(), bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { if (c->blob) cudaFree(c->blob); delete c; cudaGetLastError(); return cuda_fail(e, "L-BFGS table upload"); }
    unsigned char* b = (unsigned char*)c->blob;
    c->tb.ptrs = (const unsigned long long*)b;
    c->tb.numel = (const long long*)(b + off_n);
    c->tb.chunk_prefix = (const int*)(b + off_p);
    c->tb.aligned = (const int*)(b + off_a);
    c->tb.T = T; c->tb.num_chunks = prefix[T]; c->tb.ncols = ncols;
    c->key = std::move(key);
    c->history = m;
    int rc = ensure_partials(d, 2LL * c->tb.num_chunks);          // two halves: consecutive passes alternate
    if (rc != GM_OK) { cudaFree(c->blob); delete c; return rc; }
    std::lock_guard<std::mutex> lk(g_lb_mu);
    auto& v = g_lb[d];
    if (v.size() >= 8) {
        // Bounded: forget the oldest table.  It is parked until the next eviction rather than
        // freed at once, because a caller may hold it between its lookup and its launches.
        cudaStreamSynchronize(d->stream);
        LbfgsCtx*& parked = g_lb_parked[d];
        if (parked) { cudaFree(parked->blob); delete parked; }
        parked = v.front();
        v.erase(v.begin());
    }
    v.push_back(c);
    *out = c;
    return GM_OK;
}

// Grid of the pipelined kernel: the CTAs resident at once, trimmed so that every
// CTA walks the same number of chunks (no short last round).
static int axpy_grid(Device* d, int num_chunks) {
    static thread_local int per_sm = 0;
    if (per_sm == 0) {
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lbfgs_axpy_dot_kernel, kDotThreads, 0);
        if (per_sm < 1) per_sm = 1;
    }
    int waves = d->lbfgs_waves > 0 ? d->lbfgs_waves : 1;
    const long long resident = (long long)per_sm * d->sm_count * waves;
    if (num_chunks <= resident) return num_chunks;
    const long long rounds = (num_chunks + resident - 1) / resident;
    return (int)((num_chunks + rounds - 1) / rounds);
}

// Called when a device handle is destroyed: its pointer tables go with it.
void lbfgs_release_device(Device* d) {
    std::lock_guard<std::mutex> lk(g_lb_mu);
    auto pk = g_lb_parked.find(d);
    if (pk != g_lb_parked.end()) {
        if (pk->second) { cudaFree(pk->second->blob); delete pk->second; }
        g_lb_parked.erase(pk);
    }
    auto it = g_lb.find(d);
    if (it == g_lb.end()) return;
    for (LbfgsCtx* c : it->second) { cudaFree(c->blob); delete c; }
    g_lb.erase(it);
}

// Grid of the single-launch step (one CTA per SM), or 0 when it cannot serve this problem:
// too many chunks for the on-chip storage, too long a history, or no cooperative launch.
static int coop_grid(Device* d, int num_chunks, int m) {
    if (m > kCoopMaxHistory) return 0;
    static thread_local int prepared = 0;      // 1 ready, -1 unavailable
    if (prepared == 0) {
        int coop = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, d->ordinal);
        cudaError_t e = cudaFuncSetAttribute((const void*)lbfgs_coop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kCoopSmemBytes);
        int per_sm = 0;
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)lbfgs_coop_kernel, kCoopThreads, kCoopSmemBytes);
        if (e != cudaSuccess) cudaGetLastError();
        prepared = (coop && e == cudaSuccess && per_sm >= 1) ? 1 : -1;
    }
    if (prepared < 0) return 0;
    const int grid = d->sm_count < num_chunks ? d->sm_count : num_chunks;
    if ((long long)grid * kCoopMaxChunksPerCta < num_chunks) return 0;
    return grid;
}

// Grid of the single-launch step that leaves the direction in L2: the resident CTAs, trimmed so
// that every CTA walks the same number of chunks; 0 when it cannot serve this problem.
static int fused_grid(Device* d, int num_chunks, int m) {
    if (m > kCoopMaxHistory) return 0;
    static thread_local int per_sm = 0;          // -1 unavailable
    if (per_sm == 0) {
        int coop = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, d->ordinal);
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)lbfgs_fused_kernel, kDotThreads, 0);
        if (e != cudaSuccess) cudaGetLastError();
        if (!coop || e != cudaSuccess || per_sm < 1) per_sm = -1;
    }
    if (per_sm < 0) return 0;
    const long long resident = (long long)per_sm * d->sm_count;
    if (num_chunks <= resident) return num_chunks;
    const long long rounds = (num_chunks + resident - 1) / resident;
    return (int)((num_chunks + rounds - 1) / rounds);
}

static void launch_pass(Device* d, const LbfgsCtx* c, const LbfgsOp& op_in, const bool overlap = true) {
    LbfgsOp op = op_in;
    // Every pass after the first of a step is launched so that it may start while its
    // predecessor drains; each waits for that predecessor before touching its data.
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(kDotThreads); cfg.dynamicSmemBytes = 0; cfg.stream = d->stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (overlap && d->lbfgs_overlap) { cfg.attrs = &attr; cfg.numAttrs = 1; }
    if (op.kind <= 2) {
        op.keep_dir = d->lbfgs_keep_dir;
        op.early_trigger = d->lbfgs_overlap == 1;
        op.prewait = d->lbfgs_prewait;
        cfg.gridDim = dim3(axpy_grid(d, c->tb.num_chunks));
        cudaLaunchKernelEx(&cfg, lbfgs_axpy_dot_kernel, c->tb, op, d->partials, d->ticket);
    } else {
        cfg.gridDim = dim3(launch_grid(d, (const void*)lbfgs_pass_kernel, kDotThreads, c->tb.num_chunks));
        cudaLaunchKernelEx(&cfg, lbfgs_pass_kernel, c->tb, op, d->partials, d->ticket);
    }
    d->launches++;
}

static int lbfgs_step(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* old_g, uintptr_t* dir,
                      uintptr_t* s_flat, uintptr_t* y_flat, uintptr_t* rho_bufs, uintptr_t alpha_buf, int T,
                      int* buffer_sizes, int m, int hc, int hi, float initial_step, float* step_size) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (T <= 0 || m <= 0 || hc < 0 || hc > m || hi < 0 || hi >= m) {
        set_error("bad L-BFGS shape: tensors %d history %d count %d index %d", T, m, hc, hi);
        return GM_ERR_BAD_ARG;
    }
    if (!w || !g || !old_g || !dir || !s_flat || !y_flat || !rho_bufs || !alpha_buf || !buffer_sizes) {
        set_error("a buffer array is nil");
        return GM_ERR_NIL_BUFFER;
    }
    std::vector<int64_t> numel(T);
    for (int t = 0; t < T; ++t) {
        if (buffer_sizes[t] <= 0 || buffer_sizes[t] % 4) { set_error("buffer_sizes[%d]=%d is not a positive multiple of 4", t, buffer_sizes[t]); return GM_ERR_BAD_SIZE; }
        numel[t] = buffer_sizes[t] / 4;
        if (!w[t] || !g[t] || !old_g[t] || !dir[t]) { set_error("tensor %d has a nil buffer", t); return GM_ERR_NIL_BUFFER; }
    }
    for (int k = 0; k < m * T; ++k) if (!s_flat[k] || !y_flat[k]) { set_error("history buffer %d is nil", k); return GM_ERR_NIL_BUFFER; }
    for (int k = 0; k < m; ++k) if (!rho_bufs[k]) { set_error("rho buffer %d is nil", k); return GM_ERR_NIL_BUFFER; }

    uintptr_t* cols4[4] = {w, g, old_g, dir};
    LbfgsCtx* c = nullptr;
    int rc = get_ctx(d, T, m, cols4, s_flat, y_flat, numel.data(), &c);
    if (rc != GM_OK) return rc;
    // Buffers this library allocated are checked against their sizes, once per table and again
    // only after something was allocated or released.
    const uint64_t gen = registry_generation();
    if (c->validated_gen != gen) {
        for (int t = 0; t < T; ++t)
            for (uintptr_t p : {w[t], g[t], old_g[t], dir[t]})
                if (!buffer_holds(p, buffer_sizes[t], "L-BFGS vector")) return GM_ERR_BAD_SIZE;
        for (int k = 0; k < m * T; ++k)
            if (!buffer_holds(s_flat[k], buffer_sizes[k % T], "L-BFGS history") ||
                !buffer_holds(y_flat[k], buffer_sizes[k % T], "L-BFGS history")) return GM_ERR_BAD_SIZE;
        if (!buffer_holds(alpha_buf, 4LL * m, "L-BFGS alpha")) return GM_ERR_BAD_SIZE;
        c->validated_gen = gen;
    }

    DeviceGuard guard(d);
    float* alpha = (float*)alpha_buf;
    float* coeff = d->scalars;                 // alpha_j - beta_j of the pair being applied
    auto slot = [&](int j) { return (hi - hc + j + m) % m; };        // bridge_optimizer.m:1050
    auto rho_of = [&](int idx) { return (const float*)rho_bufs[idx]; };
    auto col_s = [&](int idx) { return COL_HIST + idx; };
    auto col_y = [&](int idx) { return COL_HIST + m + idx; };

    if (d->lbfgs_coop) {
        const bool on_chip = d->lbfgs_coop == 1;
        const int grid = on_chip ? coop_grid(d, c->tb.num_chunks, m) : fused_grid(d, c->tb.num_chunks, m);
        if (grid > 0) {
            CoopPlan plan{};
            int np = 0;
            {
                CoopPass& p0 = plan.pass[np++];
                p0 = CoopPass{0, -1, -1, -1, -1, -1, 0, -1, -1};
                if (hc > 0) { const int idx = slot(hc - 1); p0.col_dot = col_s(idx); p0.rho_dot = idx; p0.epilogue = 1; p0.out_alpha = hc - 1; }
            }
            for (int j = hc - 1; j >= 0; --j) {
                const int idx = slot(j);
                CoopPass& ps = plan.pass[np++];
                ps = CoopPass{1, col_y(idx), -1, idx, -1, j, 0, -1, -1};
                if (j > 0) { const int nx = slot(j - 1); ps.col_dot = col_s(nx); ps.rho_dot = nx; ps.epilogue = 1; ps.out_alpha = j - 1; }
                else { const int nx = slot(0); ps.col_dot = col_y(nx); ps.rho_dot = nx; ps.epilogue = 2; ps.alpha_in = 0; }
            }
            for (int j = 0; j < hc; ++j) {
                const int idx = slot(j);
                CoopPass& ps = plan.pass[np++];
                ps = CoopPass{2, col_s(idx), -1, idx, -1, -1, 0, -1, -1};
                if (j + 1 < hc) { const int nx = slot(j + 1); ps.col_dot = col_y(nx); ps.rho_dot = nx; ps.epilogue = 2; ps.alpha_in = j + 1; }
            }
            const int prev = (hi - 1 + m) % m;
            plan.pass[np++] = CoopPass{3, -1, -1, -1, -1, -1, hc > 0 ? 3 : 0, -1, -1};
            plan.num_passes = np;
            plan.history = m;
            plan.descent = (d->lbfgs_mode & 2) ? 1 : 0;
            plan.corrected = (d->lbfgs_mode & 1) ? 1 : 0;
            plan.have_pair = hc > 0 ? 1 : 0;
            plan.col_s_new = col_s(hi); plan.col_y_prev = col_y(prev); plan.col_s_prev = col_s(prev);
            plan.step = initial_step;
            plan.epoch_base = d->lbfgs_epoch;
            d->lbfgs_epoch += (unsigned)np + 1u;
            for (int k = 0; k < m; ++k) plan.rho[k] = (const float*)rho_bufs[k];
            plan.alpha = alpha;
            plan.rho_prev = (float*)rho_bufs[prev];
            plan.barrier_budget = d->barrier_budget_cycles;
            rc = ensure_partials(d, 2LL * c->tb.num_chunks);
            if (rc != GM_OK) return rc;
            LbfgsTable tbv = c->tb;
            float* partials = d->partials;
            unsigned int* ctl = d->ticket;
            int keep_dir = d->lbfgs_keep_dir;
            void* args[] = {&tbv, &plan, &partials, &ctl, &keep_dir};
            if (on_chip) {
                GM_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)lbfgs_coop_kernel, dim3(grid), dim3(kCoopThreads), args,
                                                          kCoopSmemBytes, d->stream));
            } else {
                rc = ensure_tagged(d, 2LL * c->tb.num_chunks);
                if (rc != GM_OK) return rc;
                unsigned long long* tagged = d->tagged;
                void* fargs[] = {&tbv, &plan, &tagged, &ctl, &keep_dir};
                GM_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)lbfgs_fused_kernel, dim3(grid), dim3(kDotThreads), fargs, 0,
                                                          d->stream));
            }
            d->launches++;
            if (step_size) *step_size = initial_step;
            GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
            unsigned int failed = 0;
            GM_CUDA_CHECK(cudaMemcpy(&failed, d->ticket + kLbError, sizeof(failed), cudaMemcpyDeviceToHost));
            if (failed) {
                GM_CUDA_CHECK(cudaMemset(d->ticket + kLbArrive, 0, 3 * sizeof(unsigned int)));
                set_error("a grid-barrier wait of the single-launch L-BFGS step ran out; the step is incomplete");
                return GM_ERR_TIMEOUT;
            }
            return GM_OK;
        }
    }

    rc = ensure_partials(d, 2LL * c->tb.num_chunks);
    if (rc != GM_OK) return rc;
    // Consecutive loop passes write their chunk sums to alternating halves of the buffer.  A pass whose
    // scalar only the next pass reads leaves its epilogue to that pass ("lbfgs_defer").
    LbfgsOp prev_op{};
    int half = 0;
    auto emit = [&](LbfgsOp o, const bool overlap) {
        o.part_out = half;
        o.part_in = prev_op.part_out;
        if (prev_op.defer) {
            o.pro_epilogue = prev_op.epilogue; o.pro_rho_dot = prev_op.rho_dot;
            o.pro_alpha_in = prev_op.alpha_in; o.pro_out = prev_op.out;
        }
        o.defer = d->lbfgs_defer && o.kind <= 2 && (o.epilogue == 1 || o.epilogue == 2) ? 1 : 0;
        launch_pass(d, c, o, overlap);
        prev_op = o;
        half ^= 1;
    };

    LbfgsOp op{};
    // q = -g, fused with the dot the newest pair needs
    op.kind = 0; op.col_dot = -1; op.epilogue = 0; op.descent = (d->lbfgs_mode & 2) ? 1 : 0;
    if (hc > 0) {
        const int idx = slot(hc - 1);
        op.col_dot = col_s(idx); op.rho_dot = rho_of(idx); op.epilogue = 1; op.out = alpha + (hc - 1);
    }
    emit(op, false);

    // first loop, newest to oldest: q -= alpha_j * y_j, fused with the next dot
    for (int j = hc - 1; j >= 0; --j) {
        const int idx = slot(j);
        LbfgsOp o{};
        o.kind = 1; o.col_axpy = col_y(idx); o.rho_axpy = rho_of(idx); o.coef = alpha + j;
        if (j > 0) {
            const int nx = slot(j - 1);
            o.col_dot = col_s(nx); o.rho_dot = rho_of(nx); o.epilogue = 1; o.out = alpha + (j - 1);
        } else {
            const int nx = slot(0);                                  // second loop starts with beta_0 = rho_0 * y_0.r
            o.col_dot = col_y(nx); o.rho_dot = rho_of(nx); o.epilogue = 2; o.out = coeff; o.alpha_in = alpha + 0;
        }
        emit(o, true);
    }

    // second loop, oldest to newest: r += (alpha_j - beta_j) * s_j, fused with the next dot
    for (int j = 0; j < hc; ++j) {
        const int idx = slot(j);
        LbfgsOp o{};
        o.kind = 2; o.col_axpy = col_s(idx); o.rho_axpy = rho_of(idx); o.coef = coeff;
        o.col_dot = -1; o.epilogue = 0;
        if (j + 1 < hc) {
            const int nx = slot(j + 1);
            o.col_dot = col_y(nx); o.rho_dot = rho_of(nx); o.epilogue = 2; o.out = coeff; o.alpha_in = alpha + (j + 1);
        }
        emit(o, true);
    }

    // p = -r ; x += step*p ; old_g <- g ; s[hi] = step*p ; y[prev], rho[prev]
    {
        const int prev = (hi - 1 + m) % m;
        LbfgsOp o{};
        o.kind = 3; o.step = initial_step; o.corrected = (d->lbfgs_mode & 1) ? 1 : 0;
        o.col_s_new = col_s(hi); o.have_pair = hc > 0 ? 1 : 0;
        o.col_y_prev = col_y(prev); o.col_s_prev = col_s(prev);
        o.col_dot = hc > 0 ? col_s(prev) : -1;
        o.epilogue = hc > 0 ? 3 : 0; o.out = (float*)rho_bufs[prev];
        o.part_in = 0; o.part_out = 0;
        launch_pass(d, c, o);
    }
    GM_CUDA_CHECK(cudaGetLastError());
    if (step_size) *step_size = initial_step;       // no line search (bridge_optimizer.m:1216-1217)
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return GM_OK;
}

}  // namespace gm

using namespace gm;

extern "C" {

int execute_lbfgs_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* old_g, uintptr_t* dir,
                            uintptr_t* s_flat, uintptr_t* y_flat, uintptr_t* rho_bufs, uintptr_t alpha_buf,
                            int num_weights, int* buffer_sizes, int history_size, int history_count,
                            int history_index, float initial_step, float c1, float c2, int max_line_search,
                            float current_loss, float prev_loss, float* step_size) {
    // c1, c2, max_line_search and the losses are accepted and unused, as in the
    // reference (bridge_optimizer.m:1216-1217).
    (void)c1; (void)c2; (void)max_line_search; (void)current_loss; (void)prev_loss;
    return lbfgs_step(device_ptr, w, g, old_g, dir, s_flat, y_flat, rho_bufs, alpha_buf, num_weights,
                      buffer_sizes, history_size, history_count, history_index, initial_step, step_size);
}

int execute_lbfgs_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* old_g,
                                   uintptr_t* dir, uintptr_t* s_flat, uintptr_t* y_flat, uintptr_t* rho_bufs,
                                   uintptr_t alpha_buf, int num_weights, int* buffer_sizes, int history_size,
                                   int history_count, int history_index, float initial_step, float c1, float c2,
                                   int max_line_search, float current_loss, float prev_loss,
                                   uintptr_t command_pool, float* step_size) {
    (void)command_pool;                       // bridge_optimizer.m:1324-1393 forwards to the plain entry
    return execute_lbfgs_step_cuda(device_ptr, w, g, old_g, dir, s_flat, y_flat, rho_bufs, alpha_buf, num_weights,
                                   buffer_sizes, history_size, history_count, history_index, initial_step, c1, c2,
                                   max_line_search, current_loss, prev_loss, step_size);
}

int gm_lbfgs_set_mode(uintptr_t device_ptr, int mode) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (mode < 0 || mode > 3) { set_error("L-BFGS mode must be in 0..3"); return GM_ERR_BAD_ARG; }
    d->lbfgs_mode = mode;
    return GM_OK;
}

int gm_dot_canonical(uintptr_t device_ptr, uintptr_t a, uintptr_t b, int64_t n, float* out) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!a || !b || !out) { set_error("nil argument"); return GM_ERR_NIL_BUFFER; }
    if (n <= 0) { set_error("length %lld is not positive", (long long)n); return GM_ERR_BAD_SIZE; }
    if (!buffer_holds(a, 4 * n, "dot operand") || !buffer_holds(b, 4 * n, "dot operand")) return GM_ERR_BAD_SIZE;
    // A one-tensor table with the two operands in columns 0 and 1.
    const int64_t nc = (n + kDotChunk - 1) / kDotChunk;
    if (nc > 0x7fffffff) { set_error("vector too long"); return GM_ERR_BAD_SIZE; }
    int rc = ensure_partials(d, nc);
    if (rc != GM_OK) return rc;
    DeviceGuard guard(d);
    struct { unsigned long long ptrs[2]; long long numel; int prefix[2]; int aligned; } host;
    host.ptrs[0] = a; host.ptrs[1] = b; host.numel = n; host.prefix[0] = 0; host.prefix[1] = (int)nc;
    host.aligned = (a % 16 == 0 && b % 16 == 0) ? 1 : 0;
    unsigned char* blob = nullptr;
    GM_CUDA_CHECK(cudaMalloc((void**)&blob, 256));
    cudaError_t e = cudaMemcpy(blob, &host, sizeof(host), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(blob); return cuda_fail(e, "dot table upload"); }
    LbfgsTable tb;
    tb.ptrs = (const unsigned long long*)blob;
    tb.numel = (const long long*)(blob + offsetof(decltype(host), numel));
    tb.chunk_prefix = (const int*)(blob + offsetof(decltype(host), prefix));
    tb.aligned = (const int*)(blob + offsetof(decltype(host), aligned));
    tb.T = 1; tb.num_chunks = (int)nc; tb.ncols = 2;
    LbfgsOp op{};
    op.kind = 4; op.col_axpy = 0; op.col_dot = 1; op.epilogue = 4; op.out = d->scalars + 1;
    int grid = launch_grid(d, (const void*)lbfgs_pass_kernel, kDotThreads, tb.num_chunks);
    lbfgs_pass_kernel<<<grid, kDotThreads, 0, d->stream>>>(tb, op, d->partials, d->ticket);
    d->launches++;
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
    if (e == cudaSuccess) e = cudaMemcpy(out, d->scalars + 1, sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(blob);
    if (e != cudaSuccess) return cuda_fail(e, "canonical dot");
    return GM_OK;
}

}  // extern "C"

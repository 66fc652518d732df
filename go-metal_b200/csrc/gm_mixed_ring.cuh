// gm_mixed_ring.cuh -- the mixed-precision step as ONE cooperative launch of
// resident CTAs that feed themselves through an asynchronous shared-memory ring.
// Included by gm_mixed.cu after StepPrep, MixedScalars and mixed_elem.
//
// MEASURED SLOWER than the two-launch step and therefore not the default (25.2 M
// parameters in 48 ragged tensors on B200: 135.5 us for the check kernel followed by the
// one-CTA-per-chunk update; 167 us for the check kernel followed by this ring update; 189 us
// for this kernel doing the whole step).  It stays selectable ("mixed_ring" of
// gm_device_set_tuning) because it is the only strategy that needs no second launch, and
// it carries the bounded grid barrier.  The idea it tests: the two-launch step spends a
// sixth of its time outside the update's steady state (a 50 MB check pass that is all ramp
// and tail, and the ramp and tail of a 5-wave update grid), so keep every CTA resident for
// the whole step (cooperative launch, so that is guaranteed, not assumed):
//
//   prologue  the loads of the CTA's first tiles of master/m/v/g16 are started
//             (cp.async into the ring; they need no decision yet);
//   check     the CTA reads the fp16 gradients of all ITS tiles once, marking the
//             lines evict_last in L2, and ORs its overflow vote into the flag;
//   barrier   one grid-wide barrier; the CTA that arrives last publishes the
//             step's scalars (overflow, 1/scale, bias corrections);
//   update    unless the step overflowed, the CTA walks its tiles: while tile q is
//             computed from shared memory, tiles q+1 .. q+S-1 are in flight.  A
//             thread only ever reads the ring slots it filled itself, so the ring
//             needs no barrier, only cp.async.wait_group;
//   finish    the CTA that takes the last ticket runs the loss-scale state machine.
//
// A tile is 1,024 consecutive elements of one chunk (4 per thread, so that four CTAs
// of 256 threads with a three-stage ring fit one SM: the arithmetic needs that many
// warps to hide its own latency); tiles are dealt round-robin to the CTAs, so all
// CTAs carry the same load to within one tile.  The check walks the gradients in
// units of 2,048 elements (16 bytes per thread), dealt the same way.  The arithmetic is
// mixed_elem, the same statements in the same order as the two-launch kernels: the
// results are bit-identical.  What it loses to: the per-tile table lookups (two per four
// elements per thread, against one per thirty-two in the chunk kernel) and the trip
// through shared memory cost more issue slots than the deeper pipeline wins back.
//
// The barrier wait is bounded (kBarrierBudgetCycles): a CTA whose wait runs out
// records the fact in the control block, skips its tiles and returns, and the
// loss-scale state is left alone, so a fault elsewhere can never turn into a hang
// here; the host reports GM_ERR_TIMEOUT on its next query (the buffers of that step
// are then partly updated and must be restored by the caller).
#pragma once

namespace gm {

constexpr int kRingStages = 3;
constexpr int kRingV = 4;                           // elements per thread and tile
constexpr int kTileElems = kApplyThreads * kRingV;  // 1,024
constexpr int kCheckElems = kApplyThreads * 8;      // 2,048: unit of the fused check
constexpr int kRingWide = 3;                        // 16-byte slots per thread and stage: master, m, v
constexpr size_t kRingStageBytes = (size_t)kApplyThreads * (kRingWide * 16 + 8);   // + 8 bytes of fp16 gradients
constexpr size_t kRingBytes = kRingStages * kRingStageBytes;
constexpr long long kBarrierBudgetCycles = 1LL << 31;   // about a second

// words of the control block (the 64-word flag buffer of a Mixed state)
constexpr int kCtlArrive = 32;     // CTAs that have reached the barrier
constexpr int kCtlGo = 33;         // epoch of the last barrier that was released
constexpr int kCtlError = 34;      // 1: a barrier wait ran out

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// Where global tile qg lies: tensor, chunk bounds and this thread's vector in it.
struct TileRef {
    int t, k, j, h;              // tensor, chunk inside the tensor, tile inside the chunk, head of the tensor
    long long n, b, e;           // tensor length, chunk bounds [b, e)
    long long off;               // element offset of this thread's 8 elements
    bool valid;                  // this thread has a whole vector in the tile
};

// V: elements per thread (the tile holds 256 * V elements)
template <int V>
__device__ __forceinline__ TileRef locate_tile(const DevList& L, const int tiles_per_chunk, const int qg, const int tid) {
    TileRef r;
    const int c = qg / tiles_per_chunk;
    r.j = qg - c * tiles_per_chunk;
    const int2 rec = __ldg(L.chunk_rec + c);
    r.t = rec.x; r.k = rec.y;
    r.n = __ldg(L.numel + r.t);
    r.h = __ldg(L.head + r.t);
    const long long chunk = L.chunk_elems;
    r.b = (long long)(r.h > 0 ? r.h : 0) + (long long)r.k * chunk;
    r.e = (r.b + chunk < r.n) ? r.b + chunk : r.n;
    const long long nvec = r.h < 0 ? 0 : ((r.e - r.b) / V);
    const long long i = (long long)r.j * kApplyThreads + tid;
    r.valid = i < nvec;
    r.off = r.b + V * i;
    return r;
}

// FUSED: the overflow check and the grid barrier run inside this kernel (cooperative launch);
// otherwise the check kernel has run before and this kernel starts from its published scalars.
template <bool FUSED, bool FAST>
__global__ void __launch_bounds__(kApplyThreads, 4)
mixed_ring_kernel(const DevList L, gm_loss_scale_t* __restrict__ state, unsigned int* __restrict__ flag,
                  StepPrep* __restrict__ prep, const MixedScalars sc, const float2* __restrict__ table,
                  const int table_len, const unsigned epoch, const int keep_g, const long long barrier_budget) {
    extern __shared__ uint4 ring[];                  // per stage: [3][256] x 16 bytes, then [256] x 8 bytes
    __shared__ int s_decision;
    constexpr int NT = kApplyThreads;
    const int tid = threadIdx.x;
    const int T = L.num_tensors;
    const int tpc = L.chunk_elems / kTileElems;
    const int total_tiles = L.num_chunks * tpc;
    const int G = gridDim.x;
    const int mine = (int)blockIdx.x < total_tiles ? (total_tiles - (int)blockIdx.x + G - 1) / G : 0;

    auto wide = [&](int stage, int s) -> uint4* {
        return reinterpret_cast<uint4*>(reinterpret_cast<char*>(ring) + stage * kRingStageBytes) + s * NT + tid;
    };
    auto narrow = [&](int stage) -> uint2* {
        return reinterpret_cast<uint2*>(reinterpret_cast<char*>(ring) + stage * kRingStageBytes + (size_t)kRingWide * NT * 16) + tid;
    };
    auto stream_ptr = [&](int s, int t) -> unsigned long long { return __ldg(L.ptrs + (size_t)s * T + t); };

    // starts the loads of this CTA's k-th tile; always closes a group so that the counting is uniform
    auto issue = [&](int k) {
        if (k < mine) {
            const TileRef r = locate_tile<kRingV>(L, tpc, blockIdx.x + k * G, tid);
            if (r.valid) {
                const int st = k % kRingStages;
                cp_async16(wide(st, 0), reinterpret_cast<const float*>(stream_ptr(1, r.t)) + r.off);
                cp_async16(wide(st, 1), reinterpret_cast<const float*>(stream_ptr(2, r.t)) + r.off);
                cp_async16(wide(st, 2), reinterpret_cast<const float*>(stream_ptr(3, r.t)) + r.off);
                cp_async8(narrow(st), reinterpret_cast<const unsigned short*>(stream_ptr(0, r.t)) + r.off);
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int k = 0; k < kRingStages - 1; ++k) issue(k);

    int decision = 0;                                // 0 update, 1 overflow: skip, 2 the barrier wait ran out
    if (FUSED) {
        const unsigned long long pol = l2_policy((keep_g & 1) != 0);
        const int upc = L.chunk_elems / kCheckElems;
        const int total_units = L.num_chunks * upc;
        const int units = (int)blockIdx.x < total_units ? (total_units - (int)blockIdx.x + G - 1) / G : 0;
        constexpr int U = 8;                         // 16-byte loads in flight per thread
        unsigned bad = 0;
        for (int k0 = 0; k0 < units; k0 += U) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                v[u] = make_uint4(0u, 0u, 0u, 0u);
                if (k0 + u < units) {
                    const TileRef r = locate_tile<8>(L, upc, blockIdx.x + (k0 + u) * G, tid);
                    const unsigned short* g = reinterpret_cast<const unsigned short*>(stream_ptr(0, r.t));
                    if (r.valid) v[u] = ld_l2(reinterpret_cast<const uint4*>(g + r.off), pol);
                    if (r.j == 0) {                  // the chunk's scalar pieces go with its first unit
                        if (r.h < 0) {
                            for (long long i = r.b + tid; i < r.e; i += NT) bad |= ((g[i] & 0x7c00u) == 0x7c00u);
                        } else {
                            if (r.k == 0 && tid < r.h) bad |= ((g[tid] & 0x7c00u) == 0x7c00u);
                            const long long tb = r.b + (((r.e - r.b) >> 3) << 3);
                            if (tb + tid < r.e) bad |= ((g[tb + tid] & 0x7c00u) == 0x7c00u);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                bad |= nonfinite_mask(v[u].x) | nonfinite_mask(v[u].y) | nonfinite_mask(v[u].z) | nonfinite_mask(v[u].w);
        }
        const int any_bad = __syncthreads_or(bad != 0);
        if (tid == 0) {
            int d = 0;
            if (any_bad) atomicOr(flag, 1u);
            __threadfence();
            const unsigned arrived = atomicAdd(flag + kCtlArrive, 1u);
            if (arrived == (unsigned)G - 1u) {
                // every vote is in: publish the step's scalars and release the others
                __threadfence();
                const unsigned overflow = *reinterpret_cast<volatile unsigned int*>(flag);
                const int tstep = state->adam_t + 1;
                const float2 bc = table[tstep < table_len ? tstep : table_len];
                publish_prep(prep, overflow, state->scale, bc, 1.0f);
                flag[kCtlArrive] = 0u;
                __threadfence();
                st_release(flag + kCtlGo, epoch);
            } else if (!bounded_wait_for(flag + kCtlGo, epoch, barrier_budget)) {
                atomicExch(flag + kCtlError, 1u);
                d = 2;
            }
            s_decision = d;
        }
        __syncthreads();
        decision = s_decision;
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }

    // the scalars were written by another CTA (or the check kernel): read them past L1
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(prep));
    const uint4 raw2 = __ldcg(reinterpret_cast<const uint4*>(prep) + 1);
    const unsigned overflow = raw.x;
    if (decision == 0 && overflow) decision = 1;

    if (decision == 0) {
        AdamRule::P p;
        p.lr = sc.lr; p.beta1 = sc.beta1; p.beta2 = sc.beta2; p.omb1 = sc.omb1; p.omb2 = sc.omb2;
        p.bc1 = __uint_as_float(raw.z); p.bc2 = __uint_as_float(raw.w);
        p.rbc1 = __uint_as_float(raw2.x); p.rbc2 = __uint_as_float(raw2.y);
        p.eps = sc.eps; p.wd = sc.wd; p.use_wd = sc.use_wd;
        const float inv_scale = __uint_as_float(raw.y);
        const bool fast = FAST && raw2.w != 0u;

        for (int k = 0; k < mine; ++k) {
            issue(k + kRingStages - 1);
            const TileRef r = locate_tile<kRingV>(L, tpc, blockIdx.x + k * G, tid);
            float* w = reinterpret_cast<float*>(stream_ptr(1, r.t));
            float* m = reinterpret_cast<float*>(stream_ptr(2, r.t));
            float* v = reinterpret_cast<float*>(stream_ptr(3, r.t));
            unsigned short* o = reinterpret_cast<unsigned short*>(stream_ptr(4, r.t));
            cp_async_wait<kRingStages - 1>();                 // this tile's group has landed
            if (r.valid) {
                const int st = k % kRingStages;
                const uint2 gc = *narrow(st);
                const float4 w0 = *reinterpret_cast<const float4*>(wide(st, 0));
                const float4 m0 = *reinterpret_cast<const float4*>(wide(st, 1));
                const float4 v0 = *reinterpret_cast<const float4*>(wide(st, 2));
                float W[4] = {w0.x, w0.y, w0.z, w0.w};
                float M[4] = {m0.x, m0.y, m0.z, m0.w};
                float V[4] = {v0.x, v0.y, v0.z, v0.w};
                const unsigned gw[2] = {gc.x, gc.y};
                unsigned ow[2];
                if (fast) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        unsigned short lo, hi;
                        mixed_elem<true, false>(half_bits_to_float((unsigned short)(gw[j] & 0xffffu)), inv_scale, 1.0f, W[2 * j], M[2 * j], V[2 * j], lo, p);
                        mixed_elem<true, false>(half_bits_to_float((unsigned short)(gw[j] >> 16)), inv_scale, 1.0f, W[2 * j + 1], M[2 * j + 1], V[2 * j + 1], hi, p);
                        ow[j] = (unsigned)lo | ((unsigned)hi << 16);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        unsigned short lo, hi;
                        mixed_elem<false, false>(half_bits_to_float((unsigned short)(gw[j] & 0xffffu)), inv_scale, 1.0f, W[2 * j], M[2 * j], V[2 * j], lo, p);
                        mixed_elem<false, false>(half_bits_to_float((unsigned short)(gw[j] >> 16)), inv_scale, 1.0f, W[2 * j + 1], M[2 * j + 1], V[2 * j + 1], hi, p);
                        ow[j] = (unsigned)lo | ((unsigned)hi << 16);
                    }
                }
                __stcs(reinterpret_cast<float4*>(w + r.off), make_float4(W[0], W[1], W[2], W[3]));
                __stcs(reinterpret_cast<float4*>(m + r.off), make_float4(M[0], M[1], M[2], M[3]));
                __stcs(reinterpret_cast<float4*>(v + r.off), make_float4(V[0], V[1], V[2], V[3]));
                __stcs(reinterpret_cast<uint2*>(o + r.off), make_uint2(ow[0], ow[1]));
            }
            if (r.j == 0) {
                // the chunk's scalar pieces: elements in front of the tensor's 16-byte boundary, the
                // fewer-than-four behind the last whole vector, or the whole chunk of a tensor whose
                // streams share no boundary
                const unsigned short* g = reinterpret_cast<const unsigned short*>(stream_ptr(0, r.t));
                auto scalar_at = [&](long long i) {
                    float wi = w[i], mi = m[i], vi = v[i];
                    unsigned short pi;
                    mixed_elem<false, false>(half_bits_to_float(g[i]), inv_scale, 1.0f, wi, mi, vi, pi, p);
                    w[i] = wi; m[i] = mi; v[i] = vi; o[i] = pi;
                };
                if (r.h < 0) {
                    for (long long i = r.b + tid; i < r.e; i += NT) scalar_at(i);
                } else {
                    if (r.k == 0 && tid < r.h) scalar_at(tid);
                    const long long tb = r.b + (((r.e - r.b) / kRingV) * kRingV);
                    if (tb + tid < r.e) scalar_at(tb + tid);
                }
            }
        }
    }
    cp_async_wait<0>();                              // nothing of this CTA is in flight when it leaves

    // the CTA that takes the last ticket runs the loss-scale state machine
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned ticket = atomicAdd(flag + 1, 1u);
        if (ticket == (unsigned)G - 1u) {
            const unsigned failed = *reinterpret_cast<volatile unsigned int*>(flag + kCtlError);
            if (!failed) {
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
            }
            flag[0] = 0u;
            flag[1] = 0u;
            __threadfence();
        }
    }
}

// A wait that nothing releases, with a short budget: the bounded wait must give up and say so.
__global__ void barrier_timeout_selftest_kernel(const unsigned* word, const long long budget, int* status) {
    if (threadIdx.x == 0 && blockIdx.x == 0) *status = bounded_wait_for(word, 0x5eedu, budget) ? 0 : 1;
}

}  // namespace gm

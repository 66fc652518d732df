/*
 * gm_oracle.c -- scalar CPU restatement of the go-metal optimizer-step rules.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT (see gm_oracle.h).  PARITY UNPINNED: the
 * reference has no golden vector for any optimizer step; this file follows the
 * operation order of cgo_bridge/bridge_optimizer.m, cited at each function.
 *
 * Every element operation is a single IEEE binary32 operation whose result is
 * rounded before the next one starts; compile with -ffp-contract=off so the
 * compiler cannot fuse a multiply with an add.
 */
#include "gm_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* threads                                                             */
/* ------------------------------------------------------------------ */

/* The elementwise loops and the per-chunk partial sums below are independent
 * per element / per chunk, so splitting an index range over threads changes no
 * bit of any result; it only makes the full-size parity cases affordable.  The
 * default is one thread (the loop then runs in the caller). */
static int g_threads = 1;

void gmo_set_threads(int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    g_threads = threads;
}

int gmo_get_threads(void) { return g_threads; }

typedef void (*range_fn)(size_t lo, size_t hi, void* ctx);
typedef struct { range_fn fn; void* ctx; size_t lo, hi; } range_job_t;

static void* range_worker(void* p) {
    range_job_t* j = (range_job_t*)p;
    j->fn(j->lo, j->hi, j->ctx);
    return NULL;
}

/* Runs fn over [0, n) split into contiguous slices, one per thread; no thread
 * gets fewer than `grain` indices. */
static void parallel_for_grain(size_t n, size_t grain, range_fn fn, void* ctx) {
    int threads = g_threads;
    if (grain < 1) grain = 1;
    if ((size_t)threads > n / grain) threads = (int)(n / grain);
    if (threads <= 1) { fn(0, n, ctx); return; }
    pthread_t tid[256];
    range_job_t job[256];
    size_t per = (n + (size_t)threads - 1) / (size_t)threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        size_t lo = (size_t)t * per;
        if (lo >= n) break;
        size_t hi = lo + per < n ? lo + per : n;
        range_job_t jb = { fn, ctx, lo, hi };
        job[t] = jb;
        if (pthread_create(&tid[t], NULL, range_worker, &job[t]) != 0) { fn(lo, n, ctx); break; }
        started++;
    }
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}

static void parallel_for(size_t n, range_fn fn, void* ctx) { parallel_for_grain(n, 32768, fn, ctx); }

/* ------------------------------------------------------------------ */
/* host scalars                                                        */
/* ------------------------------------------------------------------ */

/* bridge_optimizer.m:398-399 (bias corrections), :469-472 (1-beta). */
void gmo_adam_scalars(float beta1, float beta2, int step,
                      float* bc1, float* bc2, float* omb1, float* omb2) {
    *bc1 = 1.0f - powf(beta1, (float)step);
    *bc2 = 1.0f - powf(beta2, (float)step);
    *omb1 = 1.0f - beta1;
    *omb2 = 1.0f - beta2;
}

/* bridge_optimizer.m:2066 -- the "next" momentum-schedule value is the only
 * one the graph consumes. */
float gmo_nadam_mu_next(float beta1, int step) {
    return beta1 * (1.0f - 0.5f * powf(0.96f, (float)(step + 1) * 0.004f));
}

/* ------------------------------------------------------------------ */
/* elementwise rules                                                   */
/* ------------------------------------------------------------------ */

/* bridge_optimizer.m:484-550 */
void gmo_adam_step(float* w, const float* g, float* m, float* v, size_t n,
                   float lr, float beta1, float beta2, float eps, float wd, int step) {
    float bc1, bc2, omb1, omb2;
    gmo_adam_scalars(beta1, beta2, step, &bc1, &bc2, &omb1, &omb2);
    for (size_t i = 0; i < n; ++i) {
        float gi = g[i];
        float m_scaled = m[i] * beta1;
        float g_scaled = gi * omb1;
        float m_new = m_scaled + g_scaled;
        float g_sq = gi * gi;
        float v_scaled = v[i] * beta2;
        float gsq_scaled = g_sq * omb2;
        float v_new = v_scaled + gsq_scaled;
        float m_hat = m_new / bc1;
        float v_hat = v_new / bc2;
        float denom = sqrtf(v_hat) + eps;
        float upd = m_hat / denom;
        if (wd > 0.0f) {
            float decay = w[i] * wd;
            upd = upd + decay;
        }
        float scaled = upd * lr;
        w[i] = w[i] - scaled;
        m[i] = m_new;
        v[i] = v_new;
    }
}

/* bridge_optimizer.m:219-228 (decay), :244-278 (momentum), :315-322 (plain) */
void gmo_sgd_step(float* w, const float* g, float* mom, size_t n,
                  float lr, float momentum, float wd, int nesterov) {
    int use_mom = (momentum > 0.0f) && (mom != NULL);
    for (size_t i = 0; i < n; ++i) {
        float gf = g[i];
        if (wd > 0.0f) {
            float decay = w[i] * wd;
            gf = g[i] + decay;
        }
        if (use_mom) {
            float scaled_m = mom[i] * momentum;
            float m_new = scaled_m + gf;
            float stepv;
            if (nesterov != 0) {
                float t1 = momentum * m_new;
                float t2 = t1 + gf;
                stepv = lr * t2;
            } else {
                stepv = lr * m_new;
            }
            w[i] = w[i] - stepv;
            mom[i] = m_new;
        } else {
            float stepv = lr * gf;
            w[i] = w[i] - stepv;
        }
    }
}

/* bridge_optimizer.m:782-876; write-back :915-937 */
void gmo_rmsprop_step(float* w, const float* g, float* sq, float* mom, float* gavg, size_t n,
                      float lr, float alpha, float eps, float wd, float momentum,
                      int centered, int persist_aux) {
    float oma = 1.0f - alpha;
    for (size_t i = 0; i < n; ++i) {
        float gi = g[i];
        float g_sq = gi * gi;
        float old_scaled = sq[i] * alpha;
        float new_term = g_sq * oma;
        float sq_new = old_scaled + new_term;
        float denom;
        float gavg_new = 0.0f;
        if (centered) {
            float a_scaled = gavg[i] * alpha;
            float a_term = gi * oma;
            gavg_new = a_scaled + a_term;
            float a_sq = gavg_new * gavg_new;
            float var = sq_new - a_sq;
            float var_eps = var + eps;
            denom = sqrtf(var_eps);
        } else {
            float with_eps = sq_new + eps;
            denom = sqrtf(with_eps);
        }
        float upd = gi / denom;
        float mom_new = 0.0f;
        if (momentum > 0.0f) {
            float m_scaled = mom[i] * momentum;
            mom_new = m_scaled + upd;
            upd = mom_new;
        }
        if (wd > 0.0f) {
            float decay = w[i] * wd;
            upd = upd + decay;
        }
        float scaled = upd * lr;
        w[i] = w[i] - scaled;
        sq[i] = sq_new;
        if (persist_aux) {
            if (momentum > 0.0f) mom[i] = mom_new;
            if (centered) gavg[i] = gavg_new;
        }
    }
}

/* bridge_optimizer.m:1480-1517 */
void gmo_adagrad_step(float* w, const float* g, float* sq, size_t n,
                      float lr, float eps, float wd) {
    for (size_t i = 0; i < n; ++i) {
        float gf = g[i];
        if (wd > 0.0f) {
            float decay = w[i] * wd;
            gf = g[i] + decay;
        }
        float g_sq = gf * gf;
        float acc = sq[i] + g_sq;
        float denom = sqrtf(acc) + eps;
        float adj = lr / denom;
        float upd = adj * gf;
        w[i] = w[i] - upd;
        sq[i] = acc;
    }
}

/* bridge_optimizer.m:1773-1843 */
void gmo_adadelta_step(float* w, const float* g, float* sq, float* upd, size_t n,
                       float rho, float eps, float wd) {
    float omr = 1.0f - rho;
    for (size_t i = 0; i < n; ++i) {
        float gf = g[i];
        if (wd > 0.0f) {
            float decay = w[i] * wd;
            gf = g[i] + decay;
        }
        float g_sq = gf * gf;
        float e_scaled = sq[i] * rho;
        float e_term = g_sq * omr;
        float e_new = e_scaled + e_term;
        float rms_g = sqrtf(e_new + eps);
        float rms_u = sqrtf(upd[i] + eps);
        float ratio = rms_u / rms_g;
        float delta = ratio * gf;
        float neg = -delta;
        float w_new = w[i] + neg;
        float n_sq = neg * neg;
        float d_scaled = upd[i] * rho;
        float d_term = n_sq * omr;
        w[i] = w_new;
        sq[i] = e_new;
        upd[i] = d_scaled + d_term;
    }
}

/* bridge_optimizer.m:2061-2066 (host scalars), :2114-2200 (graph) */
void gmo_nadam_step(float* w, const float* g, float* m, float* v, size_t n,
                    float lr, float beta1, float beta2, float eps, float wd, int step) {
    float bc1, bc2, omb1, omb2;
    gmo_adam_scalars(beta1, beta2, step, &bc1, &bc2, &omb1, &omb2);
    float mu_next = gmo_nadam_mu_next(beta1, step);
    float om_mu = 1.0f - mu_next;
    for (size_t i = 0; i < n; ++i) {
        float gi = g[i];
        float m_scaled = m[i] * beta1;
        float g_scaled = gi * omb1;
        float m_new = m_scaled + g_scaled;
        float g_sq = gi * gi;
        float v_scaled = v[i] * beta2;
        float gsq_scaled = g_sq * omb2;
        float v_new = v_scaled + gsq_scaled;
        float v_hat = v_new / bc2;
        float m_hat = m_new / bc1;
        float g_hat = gi / bc1;
        float m_term = m_hat * mu_next;
        float g_term = g_hat * om_mu;
        float m_bar = m_term + g_term;
        float denom = sqrtf(v_hat) + eps;
        float upd = m_bar / denom;
        if (wd > 0.0f) {
            float decay = w[i] * wd;
            upd = upd + decay;
        }
        float scaled = upd * lr;
        w[i] = w[i] - scaled;
        m[i] = m_new;
        v[i] = v_new;
    }
}

/* ------------------------------------------------------------------ */
/* fp16                                                                */
/* ------------------------------------------------------------------ */

static uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* half(x) of the Metal conversion kernel (bridge_memory.m:362-368):
 * IEEE binary16, round-to-nearest-even, overflow to infinity. */
uint16_t gmo_f32_to_f16(float x) {
    uint32_t u = f32_bits(x);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t absu = u & 0x7fffffffu;
    if (absu >= 0x7f800000u) {                    /* inf / NaN */
        if (absu == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
        uint32_t payload = (absu >> 13) & 0x03ffu;
        return (uint16_t)(sign | 0x7c00u | 0x0200u | payload);   /* quiet NaN */
    }
    if (absu >= 0x477ff000u) {                    /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absu < 0x33000001u) {                     /* <= 2^-25 rounds to zero */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absu >> 23) - 127;
    uint32_t man = (absu & 0x007fffffu) | 0x00800000u;   /* 24-bit significand */
    uint32_t shift;
    uint32_t half_exp;
    if (exp < -14) {                              /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(exp + 15);
    }
    uint32_t kept = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (kept & 1u))) kept += 1;
    uint32_t out;
    if (half_exp == 0) {
        out = kept;                               /* carry into exponent is correct */
    } else {
        out = ((half_exp - 1) << 10) + kept;      /* kept carries the hidden bit */
    }
    return (uint16_t)(sign | out);
}

float gmo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x03ffu;
    if (exp == 0x1fu) return bits_f32(sign | 0x7f800000u | (man << 13));
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        float mag = (float)man * 5.9604644775390625e-08f;    /* man * 2^-24, exact */
        return sign ? -mag : mag;
    }
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

typedef struct { const float* f; uint16_t* h; const uint16_t* hc; float* fo; float factor; } cvt_ctx_t;

static void cvt_f32_to_f16_range(size_t lo, size_t hi, void* p) {
    cvt_ctx_t* c = (cvt_ctx_t*)p;
    for (size_t i = lo; i < hi; ++i) c->h[i] = gmo_f32_to_f16(c->f[i]);
}
static void cvt_f16_to_f32_range(size_t lo, size_t hi, void* p) {
    cvt_ctx_t* c = (cvt_ctx_t*)p;
    for (size_t i = lo; i < hi; ++i) c->fo[i] = gmo_f16_to_f32(c->hc[i]);
}
static void cvt_scale_range(size_t lo, size_t hi, void* p) {
    cvt_ctx_t* c = (cvt_ctx_t*)p;
    for (size_t i = lo; i < hi; ++i) {
        float scaled = c->f[i] * c->factor;
        c->h[i] = gmo_f32_to_f16(scaled);
    }
}

void gmo_convert_f32_to_f16(const float* src, uint16_t* dst, size_t n) {
    cvt_ctx_t c = { src, dst, NULL, NULL, 0.0f };
    parallel_for(n, cvt_f32_to_f16_range, &c);
}

void gmo_convert_f16_to_f32(const uint16_t* src, float* dst, size_t n) {
    cvt_ctx_t c = { NULL, NULL, src, dst, 0.0f };
    parallel_for(n, cvt_f16_to_f32_range, &c);
}

/* dst[i] = half(src[i] * factor): the product is rounded to binary32 first. */
void gmo_scale_to_f16(const float* src, float factor, uint16_t* dst, size_t n) {
    cvt_ctx_t c = { src, dst, NULL, NULL, factor };
    parallel_for(n, cvt_scale_range, &c);
}

/* ------------------------------------------------------------------ */
/* mixed-precision Adam                                                */
/* ------------------------------------------------------------------ */

/* training/model_trainer.go:258-270 */
void gmo_loss_scale_init(gmo_loss_scale_t* s) {
    s->scale = 65536.0f;
    s->growth = 2.0f;
    s->backoff = 0.5f;
    s->max_scale = 16777216.0f;
    s->interval = 2000;
    s->good_steps = 0;
    s->adam_t = 0;
    s->skipped = 0;
    s->last_overflow = 0;
}

typedef struct { const uint16_t* g; volatile int found; } nonfinite_ctx_t;

static void nonfinite_range(size_t lo, size_t hi, void* p) {
    nonfinite_ctx_t* c = (nonfinite_ctx_t*)p;
    for (size_t i = lo; i < hi; ++i) {
        if ((c->g[i] & 0x7c00u) == 0x7c00u) { c->found = 1; return; }   /* every writer stores 1 */
    }
}

int gmo_f16_has_nonfinite(const uint16_t* g16, size_t n) {
    nonfinite_ctx_t c = { g16, 0 };
    parallel_for(n, nonfinite_range, &c);
    return c.found;
}

/* docs/tutorials/mixed-precision.md:617-629: overflow => scale*backoff and
 * the update is skipped; `interval` clean steps => scale*growth (clamped).
 * The update itself is the Adam rule of bridge_optimizer.m:484-550 applied to
 * the fp32 master copy with g = float(g16) * (1/scale); the fp16 parameter
 * copy is half(master') (bridge_memory.m:362-368). */
typedef struct {
    const uint16_t* g; float* w; float* m; float* v; uint16_t* p;
    float inv_scale, beta1, beta2, omb1, omb2, bc1, bc2, eps, wd, lr, clip;
    int use_clip;
} mixed_ctx_t;

static void mixed_range(size_t lo, size_t hi, void* vp) {
    const mixed_ctx_t* c = (const mixed_ctx_t*)vp;
    for (size_t i = lo; i < hi; ++i) {
        float gi = gmo_f16_to_f32(c->g[i]) * c->inv_scale;
        if (c->use_clip) gi = gi * c->clip;
        float m_scaled = c->m[i] * c->beta1;
        float g_scaled = gi * c->omb1;
        float m_new = m_scaled + g_scaled;
        float g_sq = gi * gi;
        float v_scaled = c->v[i] * c->beta2;
        float gsq_scaled = g_sq * c->omb2;
        float v_new = v_scaled + gsq_scaled;
        float m_hat = m_new / c->bc1;
        float v_hat = v_new / c->bc2;
        float denom = sqrtf(v_hat) + c->eps;
        float upd = m_hat / denom;
        if (c->wd > 0.0f) {
            float decay = c->w[i] * c->wd;
            upd = upd + decay;
        }
        float scaled = upd * c->lr;
        float w_new = c->w[i] - scaled;
        c->w[i] = w_new;
        c->m[i] = m_new;
        c->v[i] = v_new;
        c->p[i] = gmo_f32_to_f16(w_new);
    }
}

static int mixed_adam_core(int num_tensors, const size_t* numel,
                           const uint16_t* const* g16, float* const* master,
                           float* const* m, float* const* v, uint16_t* const* p16,
                           float lr, float beta1, float beta2, float eps, float wd,
                           int use_clip, float clip, gmo_loss_scale_t* st) {
    int overflow = 0;
    for (int t = 0; t < num_tensors && !overflow; ++t) {
        overflow = gmo_f16_has_nonfinite(g16[t], numel[t]);
    }
    if (overflow) {
        st->scale = st->scale * st->backoff;
        st->good_steps = 0;
        st->skipped += 1;
        st->last_overflow = 1;
        return 1;
    }
    st->adam_t += 1;
    float bc1, bc2, omb1, omb2;
    gmo_adam_scalars(beta1, beta2, st->adam_t, &bc1, &bc2, &omb1, &omb2);
    mixed_ctx_t c;
    c.inv_scale = 1.0f / st->scale;
    c.beta1 = beta1; c.beta2 = beta2; c.omb1 = omb1; c.omb2 = omb2; c.bc1 = bc1; c.bc2 = bc2;
    c.eps = eps; c.wd = wd; c.lr = lr; c.use_clip = use_clip; c.clip = clip;
    for (int t = 0; t < num_tensors; ++t) {
        c.g = g16[t]; c.w = master[t]; c.m = m[t]; c.v = v[t]; c.p = p16[t];
        parallel_for(numel[t], mixed_range, &c);
    }
    st->last_overflow = 0;
    st->good_steps += 1;
    if (st->good_steps >= st->interval) {
        float grown = st->scale * st->growth;
        if (grown > st->max_scale) grown = st->max_scale;
        st->scale = grown;
        st->good_steps = 0;
    }
    return 0;
}

int gmo_mixed_adam_step(int num_tensors, const size_t* numel,
                        const uint16_t* const* g16, float* const* master,
                        float* const* m, float* const* v, uint16_t* const* p16,
                        float lr, float beta1, float beta2, float eps, float wd,
                        gmo_loss_scale_t* st) {
    return mixed_adam_core(num_tensors, numel, g16, master, m, v, p16, lr, beta1, beta2, eps, wd, 0, 1.0f, st);
}

/* ------------------------------------------------------------------ */
/* reductions                                                          */
/* ------------------------------------------------------------------ */

#define LANES 256
#define WARP 32

/* 256 lane values -> one float: xor tree inside each 32-lane group, then the
 * eight group sums added in ascending order. */
static float reduce_256(const float* lane) {
    float warp_sum[LANES / WARP];
    for (int wi = 0; wi < LANES / WARP; ++wi) {
        float cur[WARP], nxt[WARP];
        for (int l = 0; l < WARP; ++l) cur[l] = lane[wi * WARP + l];
        for (int off = 16; off >= 1; off >>= 1) {
            for (int l = 0; l < WARP; ++l) nxt[l] = cur[l] + cur[l ^ off];
            for (int l = 0; l < WARP; ++l) cur[l] = nxt[l];
        }
        warp_sum[wi] = cur[0];
    }
    float total = warp_sum[0];
    for (int wi = 1; wi < LANES / WARP; ++wi) total = total + warp_sum[wi];
    return total;
}

size_t gmo_dot_num_chunks(size_t n) {
    return (n + GMO_DOT_CHUNK - 1) / GMO_DOT_CHUNK;
}

typedef struct { const float* a; const float* b; size_t n; float* partials; } dotp_ctx_t;

static void dot_partials_range(size_t lo, size_t hi, void* vp) {
    const dotp_ctx_t* d = (const dotp_ctx_t*)vp;
    for (size_t c = lo; c < hi; ++c) {
        size_t base = c * GMO_DOT_CHUNK;
        float lane[LANES];
        for (int t = 0; t < LANES; ++t) {
            float acc = 0.0f;
            for (int i = 0; i < GMO_DOT_CHUNK / (LANES * 4); ++i) {
                for (int k = 0; k < 4; ++k) {
                    size_t e = base + ((size_t)i * LANES + (size_t)t) * 4 + (size_t)k;
                    if (e < d->n) {
                        float prod = d->a[e] * d->b[e];
                        acc = acc + prod;
                    }
                }
            }
            lane[t] = acc;
        }
        d->partials[c] = reduce_256(lane);
    }
}

void gmo_dot_chunk_partials(const float* a, const float* b, size_t n, float* partials) {
    dotp_ctx_t d = { a, b, n, partials };
    parallel_for_grain(gmo_dot_num_chunks(n), 8, dot_partials_range, &d);
}

float gmo_reduce_partials(const float* partials, size_t count) {
    float lane[LANES];
    for (int t = 0; t < LANES; ++t) {
        float acc = 0.0f;
        for (size_t c = (size_t)t; c < count; c += LANES) acc = acc + partials[c];
        lane[t] = acc;
    }
    return reduce_256(lane);
}

float gmo_dot_canonical(const float* a, const float* b, size_t n) {
    size_t nc = gmo_dot_num_chunks(n);
    float* p = (float*)malloc((nc ? nc : 1) * sizeof(float));
    gmo_dot_chunk_partials(a, b, n, p);
    float r = gmo_reduce_partials(p, nc);
    free(p);
    return r;
}

float gmo_dot_sequential(const float* a, const float* b, size_t n) {
    float acc = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float prod = a[i] * b[i];
        acc = acc + prod;
    }
    return acc;
}

double gmo_sumsq_f32(const float* g, size_t n) {
    double acc = 0.0;
    for (size_t i = 0; i < n; ++i) acc += (double)g[i] * (double)g[i];
    return acc;
}

double gmo_sumsq_f16(const uint16_t* g, size_t n, float inv_scale) {
    double acc = 0.0;
    for (size_t i = 0; i < n; ++i) {
        float x = gmo_f16_to_f32(g[i]) * inv_scale;
        acc += (double)x * (double)x;
    }
    return acc;
}

/* Sum of squares of a tensor list in the canonical dot order (the list dot
 * product of g with itself): chunk sums of every tensor concatenated in tensor
 * order and reduced once.  Independent of addresses and alignment. */
float gmo_sumsq_canonical(int nt, const size_t* numel, const float* const* g) {
    size_t total_chunks = 0;
    for (int t = 0; t < nt; ++t) total_chunks += gmo_dot_num_chunks(numel[t]);
    float* p = (float*)malloc((total_chunks ? total_chunks : 1) * sizeof(float));
    size_t at = 0;
    for (int t = 0; t < nt; ++t) {
        gmo_dot_chunk_partials(g[t], g[t], numel[t], p + at);
        at += gmo_dot_num_chunks(numel[t]);
    }
    float r = gmo_reduce_partials(p, total_chunks);
    free(p);
    return r;
}

/* Global-norm clipping coefficient, computed in binary32:
 * min(1, max_norm / (sqrt(sumsq) + 1e-6)).  The reference has no clipping code
 * (docs/guides/optimizers.md:568-569 names the concept only); the formula is
 * the usual one.  A NaN coefficient (NaN norm) is replaced by 1. */
float gmo_clip_coef(float sumsq, float max_norm) {
    float norm = sqrtf(sumsq);
    float denom = norm + 1e-6f;
    float coef = max_norm / denom;
    if (!(coef < 1.0f)) coef = 1.0f;
    return coef;
}

/* Sum of (half * inv_scale)^2 over a list of fp16 tensors, in the order the
 * overflow-check pass of the CUDA library walks them.  That order follows the
 * memory layout: head[t] is the number of elements of tensor t in front of the
 * first address at which every stream of the tensor is 16-byte aligned (-1:
 * no such address).  With head >= 0 the body [head, n) is cut into chunks of
 * `chunk` elements; in a chunk lane t of 256 adds the eight squares of vector
 * t, t+256, ... in memory order, then (first chunk only, t < head) element t
 * of the tensor, then element t of the fewer-than-eight after the last whole
 * vector.  With head < 0 the tensor is cut from element 0 and lane t adds
 * elements t, t+256, ... of the chunk.  Each square is rounded before it is
 * added; the 256 lane values and then the chunk sums are combined as in the
 * canonical dot product. */
typedef struct {
    const uint16_t* g; size_t n, h, chunk; int hd; float inv_scale; float* out;
} sumsq16_ctx_t;

static float sq_half(uint16_t hbits, float inv_scale) {
    float x = gmo_f16_to_f32(hbits) * inv_scale;
    return x * x;
}

static void sumsq16_range(size_t lo, size_t hi, void* vp) {
    const sumsq16_ctx_t* c = (const sumsq16_ctx_t*)vp;
    const uint16_t* g = c->g;
    const size_t n = c->n, h = c->h;
    for (size_t k = lo; k < hi; ++k) {
        float lane[LANES];
        size_t b = h + k * c->chunk;
        if (b > n) b = n;
        size_t e = b + c->chunk < n ? b + c->chunk : n;
        for (int tl = 0; tl < LANES; ++tl) {
            float acc = 0.0f;
            if (c->hd < 0) {
                for (size_t i = b + (size_t)tl; i < e; i += LANES) acc = acc + sq_half(g[i], c->inv_scale);
            } else {
                size_t nvec = (e - b) >> 3;
                for (size_t i = (size_t)tl; i < nvec; i += LANES)
                    for (int j = 0; j < 8; ++j) acc = acc + sq_half(g[b + 8 * i + (size_t)j], c->inv_scale);
                if (k == 0 && (size_t)tl < h) acc = acc + sq_half(g[tl], c->inv_scale);
                size_t tb = b + (nvec << 3);
                if (tb + (size_t)tl < e) acc = acc + sq_half(g[tb + (size_t)tl], c->inv_scale);
            }
            lane[tl] = acc;
        }
        c->out[k] = reduce_256(lane);
    }
}

float gmo_sumsq_f16_layout(int nt, const size_t* numel, const uint16_t* const* g16, const int* head,
                           size_t chunk, float inv_scale) {
    size_t total_chunks = 0;
    for (int t = 0; t < nt; ++t) {
        size_t h = head[t] > 0 ? (size_t)head[t] : 0;
        if (h > numel[t]) h = numel[t];
        size_t body = numel[t] - h;
        total_chunks += body > 0 ? (body + chunk - 1) / chunk : 1;
    }
    float* p = (float*)malloc((total_chunks ? total_chunks : 1) * sizeof(float));
    size_t at = 0;
    for (int t = 0; t < nt; ++t) {
        sumsq16_ctx_t c;
        c.g = g16[t]; c.n = numel[t]; c.hd = head[t]; c.chunk = chunk; c.inv_scale = inv_scale;
        c.h = head[t] > 0 ? (size_t)head[t] : 0;
        if (c.h > c.n) c.h = c.n;
        size_t body = c.n - c.h;
        size_t nchunks = body > 0 ? (body + chunk - 1) / chunk : 1;
        c.out = p + at;
        parallel_for_grain(nchunks, 4, sumsq16_range, &c);
        at += nchunks;
    }
    float r = gmo_reduce_partials(p, total_chunks);
    free(p);
    return r;
}

/* Mixed-precision step with global-norm clipping: the norm is that of the
 * unscaled gradients (gmo_sumsq_f16_layout with 1/scale), and every unscaled
 * gradient is multiplied by the coefficient before the Adam rule.  On an
 * overflow step the sum is not finite, the step is skipped and *coef is 1. */
int gmo_mixed_adam_step_clipped(int num_tensors, const size_t* numel,
                                const uint16_t* const* g16, float* const* master,
                                float* const* m, float* const* v, uint16_t* const* p16,
                                float lr, float beta1, float beta2, float eps, float wd,
                                float max_norm, const int* head, size_t chunk,
                                float* sumsq, float* coef, gmo_loss_scale_t* st) {
    float inv_scale = 1.0f / st->scale;
    float ss = gmo_sumsq_f16_layout(num_tensors, numel, g16, head, chunk, inv_scale);
    float c = gmo_clip_coef(ss, max_norm);
    if (sumsq) *sumsq = ss;
    if (coef) *coef = c;
    return mixed_adam_core(num_tensors, numel, g16, master, m, v, p16, lr, beta1, beta2, eps, wd, 1, c, st);
}

/* ------------------------------------------------------------------ */
/* L-BFGS                                                              */
/* ------------------------------------------------------------------ */

/* Dot over a tensor list.  Canonical order (0): chunk partials of every tensor
 * are concatenated in tensor order and reduced once.  Sequential order (1): one
 * accumulator per tensor, tensors added in order (bridge_optimizer.m:1073-1109).
 * Order 2: one accumulator across all tensors (the s.y sum, :1272-1297). */
static float list_dot(int nt, const size_t* numel, float* const* a, float* const* b, int order) {
    if (order == 1) {
        float total = 0.0f;
        for (int t = 0; t < nt; ++t) total = total + gmo_dot_sequential(a[t], b[t], numel[t]);
        return total;
    }
    if (order == 2) {
        /* one accumulator carried across the tensors: the shape of the s.y sum at
         * bridge_optimizer.m:1272-1297 */
        float acc = 0.0f;
        for (int t = 0; t < nt; ++t)
            for (size_t k = 0; k < numel[t]; ++k) {
                float prod = a[t][k] * b[t][k];
                acc = acc + prod;
            }
        return acc;
    }
    size_t total_chunks = 0;
    for (int t = 0; t < nt; ++t) total_chunks += gmo_dot_num_chunks(numel[t]);
    float* p = (float*)malloc((total_chunks ? total_chunks : 1) * sizeof(float));
    size_t at = 0;
    for (int t = 0; t < nt; ++t) {
        gmo_dot_chunk_partials(a[t], b[t], numel[t], p + at);
        at += gmo_dot_num_chunks(numel[t]);
    }
    float r = gmo_reduce_partials(p, total_chunks);
    free(p);
    return r;
}

/* The elementwise statements of the step, as index ranges (see parallel_for). */
typedef struct { float* dst; const float* a; const float* b; float c; int flag; } vec_ctx_t;

static void lb_init_range(size_t lo, size_t hi, void* vp) {          /* dst = flag ? a : -a */
    const vec_ctx_t* c = (const vec_ctx_t*)vp;
    for (size_t k = lo; k < hi; ++k) c->dst[k] = c->flag ? c->a[k] : -c->a[k];
}
static void lb_axpy_sub_range(size_t lo, size_t hi, void* vp) {      /* dst -= c*a */
    const vec_ctx_t* c = (const vec_ctx_t*)vp;
    for (size_t k = lo; k < hi; ++k) {
        float prod = c->c * c->a[k];
        c->dst[k] = c->dst[k] - prod;
    }
}
static void lb_axpy_add_range(size_t lo, size_t hi, void* vp) {      /* dst += c*a */
    const vec_ctx_t* c = (const vec_ctx_t*)vp;
    for (size_t k = lo; k < hi; ++k) {
        float prod = c->c * c->a[k];
        c->dst[k] = c->dst[k] + prod;
    }
}
static void lb_negate_range(size_t lo, size_t hi, void* vp) {        /* dst = -dst */
    const vec_ctx_t* c = (const vec_ctx_t*)vp;
    for (size_t k = lo; k < hi; ++k) c->dst[k] = -c->dst[k];
}
static void lb_diff_range(size_t lo, size_t hi, void* vp) {          /* dst = a - b */
    const vec_ctx_t* c = (const vec_ctx_t*)vp;
    for (size_t k = lo; k < hi; ++k) c->dst[k] = c->a[k] - c->b[k];
}
static void lb_scale_range(size_t lo, size_t hi, void* vp) {         /* dst = c*a */
    const vec_ctx_t* c = (const vec_ctx_t*)vp;
    for (size_t k = lo; k < hi; ++k) c->dst[k] = c->c * c->a[k];
}

static void vec_op(range_fn fn, size_t n, float* dst, const float* a, const float* b, float c, int flag) {
    vec_ctx_t ctx = { dst, a, b, c, flag };
    parallel_for(n, fn, &ctx);
}

int gmo_lbfgs_step(int nt, const size_t* numel,
                   float* const* w, const float* const* g, float* const* old_g,
                   float* const* dir, float* const* s, float* const* y,
                   float* rho, float* alpha,
                   int hs, int hc, int hi,
                   float initial_step, int mode, int order, float* step_size) {
    const int corrected = (mode & 1) != 0;   /* y formed before old_g is overwritten */
    const int descent = (mode & 2) != 0;     /* recursion starts from +g, so p = -H*g */

    /* q = -g  (:1026-1038).  With the final p = -r (:1204-1213) this makes the
     * reference move along +H*g; descent mode starts from q = +g instead. */
    for (int t = 0; t < nt; ++t) vec_op(lb_init_range, numel[t], dir[t], g[t], NULL, 0.0f, descent);

    /* first loop, newest to oldest (:1049-1126) */
    for (int j = hc - 1; j >= 0; --j) {
        int idx = (hi - hc + j + hs) % hs;
        float rho_j = rho[idx];
        if (fabs((double)rho_j) < 1e-10) { alpha[j] = 0.0f; continue; }
        float a = list_dot(nt, numel, s + (size_t)idx * nt, dir, order);
        a = a * rho_j;
        alpha[j] = a;
        for (int t = 0; t < nt; ++t)
            vec_op(lb_axpy_sub_range, numel[t], dir[t], y[(size_t)idx * nt + t], NULL, a, 0);
    }

    /* initial Hessian is the identity; second loop, oldest to newest (:1136-1200) */
    for (int j = 0; j < hc; ++j) {
        int idx = (hi - hc + j + hs) % hs;
        float rho_j = rho[idx];
        if (fabs((double)rho_j) < 1e-10) continue;
        float beta = list_dot(nt, numel, y + (size_t)idx * nt, dir, order);
        beta = beta * rho_j;
        float coeff = alpha[j] - beta;
        for (int t = 0; t < nt; ++t)
            vec_op(lb_axpy_add_range, numel[t], dir[t], s[(size_t)idx * nt + t], NULL, coeff, 0);
    }

    /* p = -r (:1204-1213) */
    for (int t = 0; t < nt; ++t) vec_op(lb_negate_range, numel[t], dir[t], NULL, NULL, 0.0f, 0);

    /* fixed step, no line search (:1216-1217) */
    float step = initial_step;
    if (step_size) *step_size = step;

    int prev = (hi - 1 + hs) % hs;

    /* corrected mode forms y from the previous gradient before it is lost */
    if (corrected && hc > 0) {
        for (int t = 0; t < nt; ++t)
            vec_op(lb_diff_range, numel[t], y[(size_t)prev * nt + t], g[t], old_g[t], 0.0f, 0);
    }

    /* x += step*p ; old_g <- g (:1232-1239) */
    for (int t = 0; t < nt; ++t) {
        vec_op(lb_axpy_add_range, numel[t], w[t], dir[t], NULL, step, 0);
        memcpy(old_g[t], g[t], numel[t] * sizeof(float));
    }

    /* s[hi] = step*p (:1246-1259) */
    for (int t = 0; t < nt; ++t) vec_op(lb_scale_range, numel[t], s[(size_t)hi * nt + t], dir[t], NULL, step, 0);

    /* curvature pair for the previous slot (:1262-1312) */
    if (hc > 0) {
        if (!corrected) {
            for (int t = 0; t < nt; ++t)
                vec_op(lb_diff_range, numel[t], y[(size_t)prev * nt + t], g[t], old_g[t], 0.0f, 0);
        }
        float sy = list_dot(nt, numel, s + (size_t)prev * nt, y + (size_t)prev * nt, order == 1 ? 2 : order);
        if (fabs((double)sy) > 1e-10) rho[prev] = 1.0f / sy;
        else rho[prev] = 0.0f;
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* generators                                                          */
/* ------------------------------------------------------------------ */

uint64_t gmo_hash64(uint64_t seed, uint64_t stream, uint64_t index) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (stream + 1) + 0xD1B54A32D192ED03ull * (index + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    /* second round so that neighbouring counters decorrelate */
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static double unit_open(uint64_t h) {            /* (0,1), 52 bits */
    return ((double)(h >> 12) + 0.5) * (1.0 / 4503599627370496.0);
}

/* Every value depends on (seed, stream, index) only, so the fills split over threads. */
typedef struct { float* dst; float a, b; uint64_t seed, stream; int per_mille; } fill_ctx_t;

static void fill_uniform_range(size_t lo_i, size_t hi_i, void* vp) {
    const fill_ctx_t* c = (const fill_ctx_t*)vp;
    for (size_t i = lo_i; i < hi_i; ++i) {
        double u = unit_open(gmo_hash64(c->seed, c->stream, i));
        c->dst[i] = (float)((double)c->a + u * ((double)c->b - (double)c->a));
    }
}
static void fill_normal_range(size_t lo_i, size_t hi_i, void* vp) {
    const fill_ctx_t* c = (const fill_ctx_t*)vp;
    const double two_pi = 6.283185307179586476925286766559;
    for (size_t i = lo_i; i < hi_i; ++i) {
        double u1 = unit_open(gmo_hash64(c->seed, c->stream * 2 + 0, i));
        double u2 = unit_open(gmo_hash64(c->seed, c->stream * 2 + 1, i));
        double z = sqrt(-2.0 * log(u1)) * cos(two_pi * u2);
        c->dst[i] = (float)((double)c->a + (double)c->b * z);
    }
}
static void scale_subset_range(size_t lo_i, size_t hi_i, void* vp) {
    const fill_ctx_t* c = (const fill_ctx_t*)vp;
    for (size_t i = lo_i; i < hi_i; ++i) {
        uint64_t h = gmo_hash64(c->seed ^ 0xA5A5A5A5A5A5A5A5ull, c->stream, i);
        if ((int)(h % 1000u) < c->per_mille) c->dst[i] = c->dst[i] * c->a;
    }
}
static void fill_loguniform_range(size_t lo_i, size_t hi_i, void* vp) {
    const fill_ctx_t* c = (const fill_ctx_t*)vp;
    for (size_t i = lo_i; i < hi_i; ++i) {
        double u = unit_open(gmo_hash64(c->seed, c->stream, i));
        double e = (double)c->a + u * ((double)c->b - (double)c->a);
        c->dst[i] = (float)pow(10.0, e);
    }
}

void gmo_fill_uniform(float* dst, size_t n, float lo, float hi, uint64_t seed, uint64_t stream) {
    fill_ctx_t c = { dst, lo, hi, seed, stream, 0 };
    parallel_for(n, fill_uniform_range, &c);
}

void gmo_fill_normal(float* dst, size_t n, float mean, float std, uint64_t seed, uint64_t stream) {
    fill_ctx_t c = { dst, mean, std, seed, stream, 0 };
    parallel_for(n, fill_normal_range, &c);
}

void gmo_scale_subset(float* dst, size_t n, int per_mille, float factor, uint64_t seed, uint64_t stream) {
    fill_ctx_t c = { dst, factor, 0.0f, seed, stream, per_mille };
    parallel_for(n, scale_subset_range, &c);
}

void gmo_fill_loguniform(float* dst, size_t n, float lo_exp10, float hi_exp10, uint64_t seed, uint64_t stream) {
    fill_ctx_t c = { dst, lo_exp10, hi_exp10, seed, stream, 0 };
    parallel_for(n, fill_loguniform_range, &c);
}

/* ------------------------------------------------------------------ */
/* threaded baseline                                                   */
/* ------------------------------------------------------------------ */

typedef struct {
    float* w; const float* g; float* m; float* v; size_t n;
    float lr, b1, b2, eps, wd; int step;
} adam_job_t;

static void* adam_worker(void* p) {
    adam_job_t* j = (adam_job_t*)p;
    gmo_adam_step(j->w, j->g, j->m, j->v, j->n, j->lr, j->b1, j->b2, j->eps, j->wd, j->step);
    return NULL;
}

void gmo_adam_step_mt(float* w, const float* g, float* m, float* v, size_t n,
                      float lr, float beta1, float beta2, float eps, float wd, int step,
                      int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    adam_job_t job[256];
    size_t per = (n + (size_t)threads - 1) / (size_t)threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        size_t lo = (size_t)t * per;
        if (lo >= n) break;
        size_t hi = lo + per < n ? lo + per : n;
        adam_job_t jb = { w + lo, g + lo, m + lo, v + lo, hi - lo, lr, beta1, beta2, eps, wd, step };
        job[t] = jb;
        pthread_create(&tid[t], NULL, adam_worker, &job[t]);
        started++;
    }
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}

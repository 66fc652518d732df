/*
 * gm_oracle.h -- CPU oracle for the go-metal optimizer-step path.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT.  Only the test-suite, the smoke check and
 * the benchmark's CPU-baseline leg and parity checks may link or call this code, and only as the
 * checker / the timed baseline.  The CUDA library never routes through it.
 *
 * PARITY UNPINNED: the reference computes every update rule inside Apple's
 * MPSGraph (closed source, needs Metal) and none of its tests reads back a
 * numeric result of an optimizer step, so there is no golden vector to pin
 * these restatements against.  What is restated here is the operation order
 * written in cgo_bridge/bridge_optimizer.m (cited per function) with IEEE-754
 * binary32 arithmetic, round-to-nearest-even, no fused multiply-add.
 *
 * Build with: gcc -O2 -ffp-contract=off -fno-fast-math (see Makefile).
 */
#ifndef GM_ORACLE_H
#define GM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- threads ----
 * Elementwise loops and per-chunk partial sums are independent per element or
 * chunk; running them on several threads (pthreads) changes no result bit.  The
 * default is 1.  Used by the full-size parity cases only. */
void gmo_set_threads(int threads);
int gmo_get_threads(void);

/* ---- elementwise rules (one flat tensor per call; in place) ---- */

/* cgo_bridge/bridge_optimizer.m:360-641 */
void gmo_adam_step(float* w, const float* g, float* m, float* v, size_t n,
                   float lr, float beta1, float beta2, float eps, float wd, int step);

/* cgo_bridge/bridge_optimizer.m:160-357; mom may be NULL (plain SGD). */
void gmo_sgd_step(float* w, const float* g, float* mom, size_t n,
                  float lr, float momentum, float wd, int nesterov);

/* cgo_bridge/bridge_optimizer.m:691-951.  persist_aux=0 reproduces the
 * reference's write-back (only w and sq are stored; mom/gavg stay untouched),
 * persist_aux=1 also stores the new momentum and gradient-average values. */
void gmo_rmsprop_step(float* w, const float* g, float* sq, float* mom, float* gavg, size_t n,
                      float lr, float alpha, float eps, float wd, float momentum,
                      int centered, int persist_aux);

/* cgo_bridge/bridge_optimizer.m:1421-1588 */
void gmo_adagrad_step(float* w, const float* g, float* sq, size_t n,
                      float lr, float eps, float wd);

/* cgo_bridge/bridge_optimizer.m:1708-1925 */
void gmo_adadelta_step(float* w, const float* g, float* sq, float* upd, size_t n,
                       float rho, float eps, float wd);

/* cgo_bridge/bridge_optimizer.m:2023-2280 */
void gmo_nadam_step(float* w, const float* g, float* m, float* v, size_t n,
                    float lr, float beta1, float beta2, float eps, float wd, int step);

/* Host-side scalars exactly as the reference forms them (powf from libm). */
void gmo_adam_scalars(float beta1, float beta2, int step,
                      float* bc1, float* bc2, float* omb1, float* omb2);
float gmo_nadam_mu_next(float beta1, int step);

/* ---- fp16 helpers (cgo_bridge/bridge_memory.m:362-376: half(x), float(h)) ---- */
uint16_t gmo_f32_to_f16(float x);   /* round-to-nearest-even */
float gmo_f16_to_f32(uint16_t h);   /* exact */
void gmo_convert_f32_to_f16(const float* src, uint16_t* dst, size_t n);
void gmo_convert_f16_to_f32(const uint16_t* src, float* dst, size_t n);
/* dst[i] = half(src[i] * factor), the product rounded to binary32 first. */
void gmo_scale_to_f16(const float* src, float factor, uint16_t* dst, size_t n);

/* ---- mixed-precision Adam with dynamic loss scaling ----
 * Policy: training/model_trainer.go:258-270 (defaults 65536, x2, x0.5, 2000)
 * and docs/tutorials/mixed-precision.md:617-629 (halve and skip on overflow,
 * grow after N clean steps, up to a maximum). */
typedef struct {
    float scale;          /* current loss scale */
    float growth;         /* multiply after `interval` clean steps */
    float backoff;        /* multiply on overflow */
    float max_scale;      /* growth is clamped here */
    int32_t interval;     /* clean steps between growths */
    int32_t good_steps;   /* consecutive clean steps since last change */
    int32_t adam_t;       /* Adam step counter: advances on clean steps only */
    int32_t skipped;      /* total skipped steps */
    int32_t last_overflow;/* 1 if the most recent step overflowed */
} gmo_loss_scale_t;

void gmo_loss_scale_init(gmo_loss_scale_t* s);

/* 1 if any of the n halves is inf or NaN. */
int gmo_f16_has_nonfinite(const uint16_t* g16, size_t n);

/* One optimizer step over a tensor list.  Returns 1 if the step was skipped. */
int gmo_mixed_adam_step(int num_tensors, const size_t* numel,
                        const uint16_t* const* g16, float* const* master,
                        float* const* m, float* const* v, uint16_t* const* p16,
                        float lr, float beta1, float beta2, float eps, float wd,
                        gmo_loss_scale_t* st);

/* Global-norm clipping (no code in the reference; docs/guides/optimizers.md:568-569
 * names the concept).  coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)) in binary32;
 * a NaN coefficient becomes 1.  Clipped steps multiply every gradient by coef
 * (one rounding) before the rule. */
float gmo_clip_coef(float sumsq, float max_norm);
/* Sum of squares of a list of fp32 tensors in the canonical dot order. */
float gmo_sumsq_canonical(int num_tensors, const size_t* numel, const float* const* g);
/* Sum of (half*inv_scale)^2 in the order of the CUDA overflow-check pass, which
 * follows the memory layout: head[t] = elements of tensor t before the first
 * address where all its streams are 16-byte aligned (-1 none), chunk = elements
 * per chunk of the list (8192 by default).  See the definition for the order. */
float gmo_sumsq_f16_layout(int num_tensors, const size_t* numel, const uint16_t* const* g16,
                           const int* head, size_t chunk, float inv_scale);
int gmo_mixed_adam_step_clipped(int num_tensors, const size_t* numel,
                                const uint16_t* const* g16, float* const* master,
                                float* const* m, float* const* v, uint16_t* const* p16,
                                float lr, float beta1, float beta2, float eps, float wd,
                                float max_norm, const int* head, size_t chunk,
                                float* sumsq, float* coef, gmo_loss_scale_t* st);

/* ---- reductions ---- */
/* Dot product in the canonical fixed order used by the CUDA kernels:
 * 4096-element chunks; inside a chunk lane t of 256 walks elements
 * (i*256+t)*4+k for i=0..3,k=0..3; 32-lane xor tree (16,8,4,2,1); 8 warp sums
 * added in order; chunk partials are then summed by 256 lanes with stride 256
 * and the same tree.  Products are rounded to fp32 before each add. */
#define GMO_DOT_CHUNK 4096
size_t gmo_dot_num_chunks(size_t n);
void gmo_dot_chunk_partials(const float* a, const float* b, size_t n, float* partials);
float gmo_reduce_partials(const float* partials, size_t count);
float gmo_dot_canonical(const float* a, const float* b, size_t n);
/* The reference's own order: one fp32 accumulator, left to right
 * (cgo_bridge/bridge_optimizer.m:1090-1095). */
float gmo_dot_sequential(const float* a, const float* b, size_t n);
/* Sum of squares in double, for grad-norm tolerance checks. */
double gmo_sumsq_f32(const float* g, size_t n);
double gmo_sumsq_f16(const uint16_t* g, size_t n, float inv_scale);

/* ---- L-BFGS (cgo_bridge/bridge_optimizer.m:980-1321) ----
 * s and y are arrays of history_size*num_tensors pointers, slot-major
 * ([slot*num_tensors + tensor], cgo_bridge/bridge.go:1987-1998).
 * mode is a bit set.  Bit 0 (1): y[prev] is formed from the previous gradient
 * before old_g is overwritten (the reference overwrites first, :1232-1239,
 * so its y is always zero and every pair is rejected).  Bit 1 (2): the
 * recursion starts from q = +g so that p = -H*g is a descent direction (the
 * reference starts from q = -g and negates again at the end, :1026-1038 and
 * :1204-1213, which moves along +H*g).  0 = the reference's statement order,
 * 3 = a working L-BFGS.
 * order 0 = canonical dot order, 1 = sequential (reference) order: one fp32
 * accumulator per tensor for the loop dots (:1073-1109) and one accumulator
 * carried across the tensors for s.y (:1272-1297). */
int gmo_lbfgs_step(int num_tensors, const size_t* numel,
                   float* const* w, const float* const* g, float* const* old_g,
                   float* const* dir, float* const* s, float* const* y,
                   float* rho, float* alpha,
                   int history_size, int history_count, int history_index,
                   float initial_step, int mode, int order, float* step_size);

/* ---- seeded input generators (counter based; host only) ---- */
uint64_t gmo_hash64(uint64_t seed, uint64_t stream, uint64_t index);
void gmo_fill_uniform(float* dst, size_t n, float lo, float hi, uint64_t seed, uint64_t stream);
void gmo_fill_normal(float* dst, size_t n, float mean, float std, uint64_t seed, uint64_t stream);
/* Multiply a seeded `per_mille`/1000 subset of entries by `factor`. */
void gmo_scale_subset(float* dst, size_t n, int per_mille, float factor, uint64_t seed, uint64_t stream);
void gmo_fill_loguniform(float* dst, size_t n, float lo_exp10, float hi_exp10, uint64_t seed, uint64_t stream);

/* ---- threaded wrapper for the timed CPU baseline ---- */
/* Adam over one flat array split into `threads` contiguous slices (pthread). */
void gmo_adam_step_mt(float* w, const float* g, float* m, float* v, size_t n,
                      float lr, float beta1, float beta2, float eps, float wd, int step,
                      int threads);

#ifdef __cplusplus
}
#endif
#endif /* GM_ORACLE_H */

/* Recording stand-in for libgometal_cuda.so used by the CPU tests of the host
 * mirror.  Buffers are host memory; the execute_* entries do NO arithmetic --
 * they only record that they were called and with which scalars, so host logic
 * (argument marshalling, step counters, state save/restore, pool tiers) can be
 * checked without a GPU.  Never loaded by product code. */
#include <stdbool.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static int g_calls[16];
static float g_last[16];
static int g_last_int[16];
static int g_allocs, g_frees, g_fail_after = -1, g_next_rc;
enum { SGD, ADAM, ADAM_POOLED, RMSPROP, ADAGRAD, ADADELTA, NADAM, LBFGS };

int fake_calls(int which) { return g_calls[which]; }
float fake_last_float(int i) { return g_last[i]; }
int fake_last_int(int i) { return g_last_int[i]; }
int fake_allocs(void) { return g_allocs; }
int fake_frees(void) { return g_frees; }
void fake_fail_alloc_after(int n) { g_fail_after = n; }
void fake_next_return(int rc) { g_next_rc = rc; }
void fake_reset(void) { memset(g_calls, 0, sizeof g_calls); g_allocs = g_frees = 0; g_fail_after = -1; g_next_rc = 0; }
static int take_rc(void) { int rc = g_next_rc; g_next_rc = 0; return rc; }

const char* gm_last_error(void) { return "fake backend"; }
uintptr_t create_cuda_device(void) { return 0x1000; }      /* memory/manager.go:322-333 uses the same mock value */
void destroy_cuda_device(uintptr_t d) { (void)d; }
uintptr_t allocate_cuda_buffer(uintptr_t dev, int size, int type) {
    (void)type;
    if (!dev || size <= 0) return 0;
    if (g_fail_after >= 0 && g_allocs >= g_fail_after) return 0;
    g_allocs++;
    return (uintptr_t)calloc(1, (size_t)size);
}
void deallocate_cuda_buffer(uintptr_t p) { if (p) { g_frees++; free((void*)p); } }
int zero_cuda_buffer(uintptr_t dev, uintptr_t p, int size) { if (!dev) return -1; if (!p) return -4; memset((void*)p, 0, (size_t)size); return 0; }
int copy_float32_array_to_cuda_buffer(uintptr_t p, float* data, int n) { if (!p) return -4; memcpy((void*)p, data, (size_t)n * 4); return 0; }
int copy_cuda_buffer_to_float32_array(uintptr_t p, float* data, int n) { if (!p) return -4; memcpy(data, (void*)p, (size_t)n * 4); return 0; }

int execute_sgd_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* m, int n, int* s, float lr, float mom, float wd, int nest, int step) {
    (void)d; (void)w; (void)g; (void)s; g_calls[SGD]++; g_last[0] = lr; g_last[1] = mom; g_last[2] = wd; g_last_int[0] = nest; g_last_int[1] = step; g_last_int[2] = n; g_last_int[3] = m != 0; return take_rc(); }
int execute_adam_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* m, uintptr_t* v, int n, int* s, float lr, float b1, float b2, float eps, float wd, int step) {
    (void)d; (void)w; (void)g; (void)m; (void)v; g_calls[ADAM]++; g_last[0] = lr; g_last[1] = b1; g_last[2] = b2; g_last[3] = eps; g_last[4] = wd; g_last_int[1] = step; g_last_int[2] = n; g_last_int[4] = s[0]; return take_rc(); }
int execute_adam_step_cuda_pooled(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* m, uintptr_t* v, int n, int* s, float lr, float b1, float b2, float eps, float wd, int step, uintptr_t pool) {
    (void)pool; g_calls[ADAM_POOLED]++; int rc = execute_adam_step_cuda(d, w, g, m, v, n, s, lr, b1, b2, eps, wd, step); g_calls[ADAM]--; return rc; }
int execute_rmsprop_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* sq, uintptr_t* m, uintptr_t* ga, int n, int* s, float lr, float a, float eps, float wd, float mom, bool cen, int step) {
    (void)d; (void)w; (void)g; (void)sq; (void)s; g_calls[RMSPROP]++; g_last[0] = lr; g_last[1] = a; g_last[2] = eps; g_last[3] = wd; g_last[4] = mom; g_last_int[0] = cen; g_last_int[1] = step; g_last_int[2] = n; g_last_int[3] = (m != 0) + 2 * (ga != 0); return take_rc(); }
int execute_adagrad_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* sq, int n, int* s, float lr, float eps, float wd) {
    (void)d; (void)w; (void)g; (void)sq; (void)s; g_calls[ADAGRAD]++; g_last[0] = lr; g_last[1] = eps; g_last[2] = wd; g_last_int[2] = n; return take_rc(); }
int execute_adadelta_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* sq, uintptr_t* u, int n, int* s, float rho, float eps, float wd) {
    (void)d; (void)w; (void)g; (void)sq; (void)u; (void)s; g_calls[ADADELTA]++; g_last[0] = rho; g_last[1] = eps; g_last[2] = wd; g_last_int[2] = n; return take_rc(); }
int execute_nadam_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* m, uintptr_t* v, int n, int* s, float lr, float b1, float b2, float eps, float wd, int step) {
    (void)d; (void)w; (void)g; (void)m; (void)v; (void)s; g_calls[NADAM]++; g_last[0] = lr; g_last[1] = b1; g_last[2] = b2; g_last[3] = eps; g_last[4] = wd; g_last_int[1] = step; g_last_int[2] = n; return take_rc(); }
int execute_lbfgs_step_cuda(uintptr_t d, uintptr_t* w, uintptr_t* g, uintptr_t* og, uintptr_t* dir, uintptr_t* s, uintptr_t* y, uintptr_t* rho, uintptr_t alpha,
                            int n, int* sizes, int m, int hc, int hi, float step0, float c1, float c2, int mls, float loss, float prev, float* out) {
    (void)d; (void)w; (void)g; (void)og; (void)dir; (void)s; (void)y; (void)rho; (void)alpha; (void)sizes; (void)c1; (void)c2; (void)mls;
    g_calls[LBFGS]++; g_last[0] = step0; g_last[1] = loss; g_last[2] = prev; g_last_int[0] = m; g_last_int[1] = hc; g_last_int[2] = n; g_last_int[3] = hi; if (out) *out = step0; return take_rc(); }

/* ---- mixed precision: the loss-scale state is kept on the host side of the fake so that
 * get/set round-trip; a step only counts the call and advances adam_t / good_steps. ---- */
typedef struct { float scale, growth, backoff, max_scale; int32_t interval, good_steps, adam_t, skipped, last_overflow; } fake_ls_t;
typedef struct { fake_ls_t ls; float beta1, beta2; } fake_mixed_t;
enum { MIXED_STEP = 8, LIST_CREATE = 9, LIST_DESTROY = 10, MIXED_CREATE = 11, MIXED_DESTROY = 12 };
static int g_list_streams, g_list_tensors, g_list_eb[8];
int fake_list_streams(void) { return g_list_streams; }
int fake_list_tensors(void) { return g_list_tensors; }
int fake_list_elem_bytes(int s) { return g_list_eb[s]; }

uintptr_t gm_mixed_create(uintptr_t dev, const fake_ls_t* init, float b1, float b2, int table_len) {
    (void)table_len;
    if (!dev) return 0;
    fake_mixed_t* m = (fake_mixed_t*)calloc(1, sizeof *m);
    if (init) m->ls = *init;
    m->beta1 = b1; m->beta2 = b2;
    g_calls[MIXED_CREATE]++; g_last[1] = b1; g_last[2] = b2;
    return (uintptr_t)m;
}
void gm_mixed_destroy(uintptr_t m) { if (m) { g_calls[MIXED_DESTROY]++; free((void*)m); } }
int gm_mixed_step_async(uintptr_t dev, uintptr_t mixed, uintptr_t list, float lr, float eps, float wd) {
    (void)dev; (void)list;
    fake_mixed_t* m = (fake_mixed_t*)mixed;
    g_calls[MIXED_STEP]++; g_last[0] = lr; g_last[3] = eps; g_last[4] = wd;
    int rc = take_rc();
    if (rc == 0) { m->ls.adam_t++; m->ls.good_steps++; }
    return rc;
}
int gm_mixed_get_state(uintptr_t dev, uintptr_t mixed, fake_ls_t* out) { (void)dev; *out = ((fake_mixed_t*)mixed)->ls; return 0; }
int gm_mixed_set_state(uintptr_t dev, uintptr_t mixed, const fake_ls_t* in) { (void)dev; ((fake_mixed_t*)mixed)->ls = *in; return 0; }
uintptr_t gm_tensor_list_create(uintptr_t dev, int ns, int nt, const uintptr_t* const* ptrs, const int64_t* numel, const int* eb) {
    (void)dev; (void)ptrs; (void)numel;
    g_calls[LIST_CREATE]++; g_list_streams = ns; g_list_tensors = nt;
    for (int s = 0; s < ns && s < 8; ++s) g_list_eb[s] = eb ? eb[s] : 4;
    return (uintptr_t)malloc(8);
}
void gm_tensor_list_destroy(uintptr_t l) { if (l) { g_calls[LIST_DESTROY]++; free((void*)l); } }
int gm_device_synchronize(uintptr_t dev) { (void)dev; return 0; }

/* ---- arenas: one malloc'd block, 256-byte granules ---- */
typedef struct { char* base; int64_t cap, used; } fake_arena_t;
static int g_arenas_live;
int fake_arenas_live(void) { return g_arenas_live; }
uintptr_t gm_arena_create(uintptr_t dev, int64_t bytes) {
    if (!dev || bytes <= 0) return 0;
    fake_arena_t* a = (fake_arena_t*)calloc(1, sizeof *a);
    a->base = (char*)aligned_alloc(256, (size_t)((bytes + 255) / 256 * 256));
    a->cap = bytes;
    g_arenas_live++;
    return (uintptr_t)a;
}
uintptr_t gm_arena_alloc(uintptr_t h, int64_t bytes) {
    fake_arena_t* a = (fake_arena_t*)h;
    int64_t need = (bytes + 255) / 256 * 256;
    if (!a || bytes <= 0 || a->used + need > a->cap) return 0;
    uintptr_t p = (uintptr_t)(a->base + a->used);
    a->used += need;
    return p;
}
void gm_arena_destroy(uintptr_t h) {
    fake_arena_t* a = (fake_arena_t*)h;
    if (!a) return;
    free(a->base); free(a); g_arenas_live--;
}

/*
 * gometal_cuda.h -- C ABI of libgometal_cuda.so, the CUDA (sm_100a) replacement
 * for go-metal's optimizer-step bridge.
 *
 * Part 1 mirrors, entry for entry, what the reference's cgo layer binds for
 * this path (cgo_bridge/bridge_optimizer.h, cgo_bridge/bridge_memory.h and the
 * device/queue calls of cgo_bridge/bridge.go).  Argument order, C types and the
 * int return convention (0 = ok, negative = failure class) are unchanged; only
 * the `_mpsgraph` / `metal` part of each name became `_cuda` / `cuda`, so a Go
 * wrapper changes its symbol and nothing else.  Every pointer is borrowed for
 * the duration of the call; host arrays are copied, never retained.  These
 * entries are synchronous: results are in the buffers when they return.
 *
 * Part 2 holds entries that have no counterpart in the reference (64-bit
 * sizes, persistent tensor lists, asynchronous steps, mixed precision with a
 * device-resident loss scale, grad-norm, ZeRO-1 sharding, timing).
 *
 * All buffers are device pointers (cudaMalloc or any CUDA allocation on the
 * device's ordinal).  No entry falls back to the CPU.
 */
#ifndef GOMETAL_CUDA_H
#define GOMETAL_CUDA_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes.  -1..-8 keep the reference's meaning where one exists
 * (cgo_bridge/bridge_optimizer.m:174-193, 377-394, 413, 630, 638). */
#define GM_OK                 0
#define GM_ERR_NIL_DEVICE    -1   /* device handle is 0 */
#define GM_ERR_NIL_BUFFER    -4   /* a required buffer pointer is 0 */
#define GM_ERR_AUX_BUFFER    -5   /* momentum>0 / centered without its buffer */
#define GM_ERR_CUDA          -8   /* a CUDA call failed; see gm_last_error() */
#define GM_ERR_BAD_SIZE      -9   /* size <= 0, not a multiple of the element, or too small */
#define GM_ERR_BAD_ARG      -10   /* any other invalid argument */
#define GM_ERR_UNSUPPORTED  -11   /* valid call that this build cannot serve (e.g. NCCL missing) */
#define GM_ERR_TIMEOUT      -12   /* a bounded wait ran out (gm_device_synchronize_timeout) */

/* ===================================================================== */
/* Part 1 -- drop-in entries                                              */
/* ===================================================================== */

/* ---- device and queue: cgo_bridge/bridge.go:632-645 (CreateMetalDevice,
 * DestroyMetalDevice), :1676-1695 (CreateCommandQueue, ReleaseCommandQueue) */
uintptr_t create_cuda_device(void);              /* ordinal from GOMETAL_CUDA_DEVICE or LOCAL_RANK, else 0 */
void destroy_cuda_device(uintptr_t device_ptr);
uintptr_t create_command_queue(uintptr_t device_ptr);   /* returns the device's stream handle */
void release_command_queue(uintptr_t command_queue);

/* ---- buffers: cgo_bridge/bridge_memory.h:6-26 ---- */
uintptr_t allocate_cuda_buffer(uintptr_t device_ptr, int size, int device_type);
void deallocate_cuda_buffer(uintptr_t buffer_ptr);
int zero_cuda_buffer(uintptr_t device_ptr, uintptr_t buffer_ptr, int size);
int copy_data_to_cuda_buffer(uintptr_t buffer_ptr, void* data, int size);
int copy_float32_array_to_cuda_buffer(uintptr_t buffer_ptr, float* data, int num_elements);
int copy_int32_array_to_cuda_buffer(uintptr_t buffer_ptr, int* data, int num_elements);
int copy_cuda_buffer_to_float32_array(uintptr_t buffer_ptr, float* data, int num_elements);
int copy_cuda_buffer_to_int32_array(uintptr_t buffer_ptr, int* data, int num_elements);
/* dtype codes follow memory/tensor.go:12-17: 0 Float32, 1 Int32, 2 Float16, 3 Int8.
 * Only Float32<->Float16 is implemented, as in bridge_memory.m:323-423. */
int convert_tensor_type_cuda(uintptr_t src_buffer_ptr, uintptr_t dst_buffer_ptr,
                             int* shape, int num_dims, int src_type, int dst_type,
                             uintptr_t device_ptr);

/* ---- SGD: cgo_bridge/bridge_optimizer.h:11-23 ---- */
int execute_sgd_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                          uintptr_t* gradient_buffers, uintptr_t* momentum_buffers,
                          int num_weights, int* buffer_sizes, float learning_rate,
                          float momentum, float weight_decay, int nesterov, int step_count);

/* ---- Adam: cgo_bridge/bridge_optimizer.h:26-40 and :58-73 (pooled) ---- */
int execute_adam_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                           uintptr_t* gradient_buffers, uintptr_t* momentum_buffers,
                           uintptr_t* variance_buffers, int num_weights, int* buffer_sizes,
                           float learning_rate, float beta1, float beta2, float epsilon,
                           float weight_decay, int step_count);
int execute_adam_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* weight_buffers,
                                  uintptr_t* gradient_buffers, uintptr_t* momentum_buffers,
                                  uintptr_t* variance_buffers, int num_weights, int* buffer_sizes,
                                  float learning_rate, float beta1, float beta2, float epsilon,
                                  float weight_decay, int step_count, uintptr_t command_pool);

/* ---- RMSProp: cgo_bridge/bridge_optimizer.h:76-92 ----
 * Unlike the reference (bridge_optimizer.m:915-937) the new momentum and
 * gradient-average values are stored, so momentum>0 and centered work. */
int execute_rmsprop_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                              uintptr_t* gradient_buffers, uintptr_t* squared_grad_avg_buffers,
                              uintptr_t* momentum_buffers, uintptr_t* gradient_avg_buffers,
                              int num_weights, int* buffer_sizes, float learning_rate,
                              float alpha, float epsilon, float weight_decay, float momentum,
                              bool centered, int step_count);

/* ---- AdaGrad: cgo_bridge/bridge_optimizer.h:97-120 ---- */
int execute_adagrad_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                              uintptr_t* gradient_buffers, uintptr_t* squared_grad_avg_buffers,
                              int num_weights, int* buffer_sizes, float learning_rate,
                              float epsilon, float weight_decay);
int execute_adagrad_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* weight_buffers,
                                     uintptr_t* gradient_buffers,
                                     uintptr_t* squared_grad_avg_buffers, int num_weights,
                                     int* buffer_sizes, float learning_rate, float epsilon,
                                     float weight_decay, uintptr_t command_pool);

/* ---- AdaDelta: cgo_bridge/bridge_optimizer.h:125-150 ---- */
int execute_adadelta_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                               uintptr_t* gradient_buffers, uintptr_t* squared_grad_avg_buffers,
                               uintptr_t* squared_update_avg_buffers, int num_weights,
                               int* buffer_sizes, float rho, float epsilon, float weight_decay);
int execute_adadelta_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* weight_buffers,
                                      uintptr_t* gradient_buffers,
                                      uintptr_t* squared_grad_avg_buffers,
                                      uintptr_t* squared_update_avg_buffers, int num_weights,
                                      int* buffer_sizes, float rho, float epsilon,
                                      float weight_decay, uintptr_t command_pool);

/* ---- NAdam: cgo_bridge/bridge_optimizer.h:207-221 ---- */
int execute_nadam_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                            uintptr_t* gradient_buffers, uintptr_t* momentum_buffers,
                            uintptr_t* variance_buffers, int num_weights, int* buffer_sizes,
                            float learning_rate, float beta1, float beta2, float epsilon,
                            float weight_decay, int step_count);

/* ---- L-BFGS: cgo_bridge/bridge_optimizer.h:155-202 ----
 * s_vectors_flat / y_vectors_flat are history_size*num_weights pointers laid
 * out [slot*num_weights + tensor] (cgo_bridge/bridge.go:1987-1998);
 * rho_buffers are history_size device buffers of one float; alpha_buffer holds
 * history_size floats.  Runs in mode 3 unless gm_lbfgs_set_mode() says otherwise. */
int execute_lbfgs_step_cuda(uintptr_t device_ptr, uintptr_t* weight_buffers,
                            uintptr_t* gradient_buffers, uintptr_t* old_gradient_buffers,
                            uintptr_t* search_dir_buffers, uintptr_t* s_vectors_flat,
                            uintptr_t* y_vectors_flat, uintptr_t* rho_buffers,
                            uintptr_t alpha_buffer, int num_weights, int* buffer_sizes,
                            int history_size, int history_count, int history_index,
                            float initial_step, float c1, float c2, int max_line_search,
                            float current_loss, float prev_loss, float* step_size);
int execute_lbfgs_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* weight_buffers,
                                   uintptr_t* gradient_buffers, uintptr_t* old_gradient_buffers,
                                   uintptr_t* search_dir_buffers, uintptr_t* s_vectors_flat,
                                   uintptr_t* y_vectors_flat, uintptr_t* rho_buffers,
                                   uintptr_t alpha_buffer, int num_weights, int* buffer_sizes,
                                   int history_size, int history_count, int history_index,
                                   float initial_step, float c1, float c2, int max_line_search,
                                   float current_loss, float prev_loss, uintptr_t command_pool,
                                   float* step_size);

/* ===================================================================== */
/* Part 2 -- entries with no counterpart in the reference                 */
/* ===================================================================== */

/* ---- diagnostics ---- */
const char* gm_last_error(void);                 /* thread-local text of the last failure */
const char* gm_version(void);
uintptr_t gm_device_create(int ordinal);         /* explicit ordinal */
int gm_device_ordinal(uintptr_t device_ptr);
int gm_device_sm_count(uintptr_t device_ptr);
uintptr_t gm_device_stream(uintptr_t device_ptr);/* cudaStream_t the device launches on */
int gm_device_synchronize(uintptr_t device_ptr);
/* The same wait with a deadline: polls the stream and returns GM_ERR_TIMEOUT when it has
 * not drained after timeout_ms.  Nothing is cancelled; the caller decides (wait again,
 * tear the group down).  Meant for sharded steps, where a peer that never enters its
 * collective would otherwise block this rank for ever. */
int gm_device_synchronize_timeout(uintptr_t device_ptr, int timeout_ms);
/* Launch-strategy switches of a handle; every setting computes the same bits.  Names:
 * "mixed_ring" (2: the mixed-precision step as one cooperative launch, 1: overflow check
 * followed by the shared-memory-ring update, 0: check followed by the one-CTA-per-chunk
 * update), "mixed_fastdiv", "mixed_pf", "mixed_variant", "lbfgs_coop", "lbfgs_prewait", "lbfgs_defer",
 * "barrier_budget_cycles" (bound of every device-side barrier wait). */
int gm_device_set_tuning(uintptr_t device_ptr, const char* name, long long value);
long long gm_device_get_tuning(uintptr_t device_ptr, const char* name);   /* -1: unknown name */
/* Number of kernels this library has launched on the device so far. */
int64_t gm_device_launch_count(uintptr_t device_ptr);

/* ---- 64-bit buffers and arenas (the reference's `int` sizes stop at 2 GiB) ----
 * An arena is one cudaMalloc carved into 256-byte-aligned sub-buffers. */
uintptr_t gm_buffer_alloc(uintptr_t device_ptr, int64_t bytes);
void gm_buffer_free(uintptr_t buffer_ptr);
int64_t gm_buffer_size(uintptr_t buffer_ptr);    /* bytes reserved, -1 if unknown to the library */
int gm_buffer_zero(uintptr_t device_ptr, uintptr_t buffer_ptr, int64_t bytes);
int gm_buffer_upload(uintptr_t device_ptr, uintptr_t buffer_ptr, const void* host, int64_t bytes);
int gm_buffer_download(uintptr_t device_ptr, uintptr_t buffer_ptr, void* host, int64_t bytes);
uintptr_t gm_arena_create(uintptr_t device_ptr, int64_t bytes);
uintptr_t gm_arena_alloc(uintptr_t arena, int64_t bytes);   /* 0 when the arena is full */
uintptr_t gm_arena_base(uintptr_t arena);
int64_t gm_arena_capacity(uintptr_t arena);
int64_t gm_arena_used(uintptr_t arena);
void gm_arena_reset(uintptr_t arena);
void gm_arena_destroy(uintptr_t arena);
/* Pinned host staging memory for callers that overlap copies with steps. */
void* gm_host_alloc_pinned(int64_t bytes);
void gm_host_free_pinned(void* p);
int gm_buffer_upload_async(uintptr_t device_ptr, uintptr_t buffer_ptr, const void* host, int64_t bytes);
int gm_buffer_download_async(uintptr_t device_ptr, uintptr_t buffer_ptr, void* host, int64_t bytes);

/* ---- persistent tensor lists ----
 * A tensor list is the device-resident descriptor one multi-tensor launch
 * walks: `num_streams` pointer arrays of `num_tensors` entries plus element
 * counts.  The drop-in entries build and cache one implicitly. */
uintptr_t gm_tensor_list_create(uintptr_t device_ptr, int num_streams, int num_tensors,
                                const uintptr_t* const* stream_ptrs, const int64_t* numel,
                                const int* elem_bytes /* per stream: 4 or 2 */);
void gm_tensor_list_destroy(uintptr_t list);
int64_t gm_tensor_list_total(uintptr_t list);
int gm_tensor_list_num_chunks(uintptr_t list);
int gm_tensor_list_chunk_elems(uintptr_t list);      /* elements per chunk of this list */
/* Elements of tensor `tensor` in front of the first address at which every stream of
 * the tensor is 16-byte aligned; -1 when the streams share no such address (that
 * tensor is then walked element by element); -2 on a bad handle or index. */
int gm_tensor_list_head(uintptr_t list, int tensor);

/* Optimizer rule selector for gm_step_async(). */
enum {
    GM_RULE_SGD = 0,        /* streams: w,g[,mom]            scalars: lr, momentum, wd, nesterov */
    GM_RULE_ADAM = 1,       /* streams: w,g,m,v              scalars: lr, beta1, beta2, eps, wd */
    GM_RULE_RMSPROP = 2,    /* streams: w,g,sq[,mom][,gavg]  scalars: lr, alpha, eps, wd, momentum, centered */
    GM_RULE_ADAGRAD = 3,    /* streams: w,g,sq               scalars: lr, eps, wd */
    GM_RULE_ADADELTA = 4,   /* streams: w,g,sq,upd           scalars: rho, eps, wd */
    GM_RULE_NADAM = 5       /* streams: w,g,m,v              scalars: lr, beta1, beta2, eps, wd */
};

typedef struct {
    float lr, beta1, beta2, eps, weight_decay;   /* beta1 doubles as momentum / alpha / rho */
    float momentum;                              /* RMSProp momentum */
    int nesterov, centered;
    int step;                                    /* 1-based, already incremented by the caller */
} gm_hyper_t;

/* Enqueue one step on the device's stream and return without waiting. */
int gm_step_async(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper);
/* Same, timed with CUDA events on the launching stream; waits for completion. */
int gm_step_timed(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper,
                  float* elapsed_ms);

/* One step for a caller whose gradients and parameters live in pinned HOST
 * memory: gradients are uploaded, the rule is applied and the new parameters
 * are downloaded slice by slice on three streams, so both PCIe directions and
 * the SMs are busy at once.  host_grads / host_params hold the tensors back to
 * back in list order; on the device stream 0 (parameters) and stream 1
 * (gradients) may be one flat run (one copy per slice and direction) or
 * separately allocated tensors (one copy each).  fp32 only.  Synchronous. */
int gm_step_host(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper,
                 const void* host_grads, void* host_params, int num_slices);

/* ---- mixed-precision Adam with a device-resident dynamic loss scale ---- */
typedef struct {
    float scale, growth, backoff, max_scale;
    int32_t interval, good_steps, adam_t, skipped, last_overflow;
} gm_loss_scale_t;

/* list streams: g16 (2 B), master, m, v (4 B), p16 (2 B). */
uintptr_t gm_mixed_create(uintptr_t device_ptr, const gm_loss_scale_t* initial,
                          float beta1, float beta2, int table_steps);
void gm_mixed_destroy(uintptr_t mixed);
int gm_mixed_step_async(uintptr_t device_ptr, uintptr_t mixed, uintptr_t list,
                        float lr, float eps, float weight_decay);
int gm_mixed_get_state(uintptr_t device_ptr, uintptr_t mixed, gm_loss_scale_t* out);   /* waits */
int gm_mixed_set_state(uintptr_t device_ptr, uintptr_t mixed, const gm_loss_scale_t* in);
uintptr_t gm_mixed_state_device_ptr(uintptr_t mixed);   /* device address of the gm_loss_scale_t */
/* Gradient norm from the overflow-check pass itself (no extra pass over the
 * gradients): when enabled, every step also leaves sum((g16 / scale)^2) over the
 * list (inf or NaN on an overflow step).  The sum is taken in a fixed order without
 * float atomics -- per chunk of the list a fixed lane walk and xor tree, chunk sums
 * added by the CTA that finishes last -- so a given memory layout (sizes and each
 * tensor's offset from a 16-byte boundary, see gm_tensor_list_head) always gives the
 * same bits.  gm_mixed_last_grad_sumsq waits for the stream and returns the last
 * step's value.  Under gm_zero1_mixed_step_async the value covers the rank's own
 * shard.  No counterpart in the reference, which has no clipping or norm.
 * gm_mixed_set_clip(max_norm > 0) turns on global-norm clipping: the same pass forms
 * coef = min(1, max_norm / (sqrt(sum) + 1e-6)) on the device and the update multiplies
 * every unscaled gradient by it (one rounding) before the Adam rule; 0 turns it off.
 * Not available in the sharded step.  gm_mixed_last_clip returns the last step's sum
 * and coefficient. */
int gm_mixed_enable_grad_norm(uintptr_t mixed, int enable);
int gm_mixed_last_grad_sumsq(uintptr_t device_ptr, uintptr_t mixed, float* out);
int gm_mixed_set_clip(uintptr_t mixed, float max_norm);
int gm_mixed_last_clip(uintptr_t device_ptr, uintptr_t mixed, float* out_sumsq, float* out_coef);

/* ---- gradient norm (sum of squares; one float atomic per CTA) ---- */
/* list stream 0 is the gradient (4 B or 2 B elements).  *out_sumsq is a
 * device float the kernel accumulates into after zeroing it. */
int gm_grad_sumsq_async(uintptr_t device_ptr, uintptr_t list, int elem_bytes, float inv_scale,
                        uintptr_t out_sumsq_device);

/* ---- deterministic gradient norm and global-norm clipping (fp32 rules) ----
 * No counterpart in the reference (docs/guides/optimizers.md:568-569 names the concept).
 * gm_grad_clip_coef_async leaves {sum g^2, coef, norm} (three floats) at out3_device, with
 * coef = min(1, max_norm / (sqrt(sum g^2) + 1e-6)) computed in binary32 on the device; the
 * gradients are stream 1 of the list.  The sum uses the library's fixed order (4096-element
 * chunks from element 0 of each tensor, fixed lane walk, xor tree, chunk sums added by the
 * CTA that finishes last), no float atomics: the same gradients give the same bits whatever
 * the grid or the addresses.  gm_step_clipped_async is gm_step_async with every gradient
 * multiplied by the float at coef_device first (one rounding).  gm_step_with_clip_async
 * chains the two on the device's stream; gm_last_clip waits and returns its three floats. */
int gm_grad_clip_coef_async(uintptr_t device_ptr, uintptr_t list, float max_norm, uintptr_t out3_device);
int gm_step_clipped_async(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper,
                          uintptr_t coef_device);
int gm_step_with_clip_async(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper,
                            float max_norm);
int gm_last_clip(uintptr_t device_ptr, float* out3);

/* ---- L-BFGS controls ---- */
/* mode is a bit set.  Bit 0: y[prev] = g - old_g is formed before old_g is
 * overwritten (the reference overwrites first, bridge_optimizer.m:1232-1239,
 * so its y is always zero and every curvature pair is rejected).  Bit 1: the
 * recursion starts from q = +g so the step descends (the reference starts from
 * q = -g, :1026-1038, negates again at :1204-1213 and so moves along +H*g).
 * 0 = the reference's statement order; 3 (default) = a working L-BFGS. */
int gm_lbfgs_set_mode(uintptr_t device_ptr, int mode);
int gm_dot_canonical(uintptr_t device_ptr, uintptr_t a, uintptr_t b, int64_t n, float* out);
/* No counterpart in the reference.  The same dot product for hosts that must
 * not allocate: a trainer whose own arenas already hold all of HBM, or a loop
 * that cannot take the device-wide synchronisation of cudaMalloc/cudaFree.
 * The chunk sums live in a ~64 KB array built into the library (one copy per
 * GPU that loads it, kept until exit), so n is limited to
 * GM_DOT_STATIC_MAX_ELEMENTS; longer vectors are rejected with GM_ERR_BAD_SIZE.
 * a, b, out (one float) are device pointers on the current device; stream is a
 * cudaStream_t (0 = default).  Asynchronous.  The first call on a device looks
 * up the array's address and should come before any stream capture; on that call
 * CUDA may also load the library's code onto the GPU (lazy module loading), which
 * is when the array takes its place in device memory.  The address is cached per
 * process and device and does not survive a cudaDeviceReset.  Calls on one device
 * share the array: calls that can overlap on the GPU race. */
#define GM_DOT_STATIC_MAX_ELEMENTS 67108864LL
int gm_dot_canonical_static(uintptr_t a, uintptr_t b, int64_t n, uintptr_t out_device, uintptr_t stream);

/* ---- ZeRO-1: sharded state + all-gather of updated parameters ---- */
#define GM_NCCL_UNIQUE_ID_BYTES 128
int gm_zero1_unique_id(void* out_id /* 128 bytes */);
uintptr_t gm_zero1_create(uintptr_t device_ptr, const void* unique_id, int rank, int world);
void gm_zero1_destroy(uintptr_t zero1);
/* In-place all-gather: every rank holds the whole arena; rank r has just
 * updated elements [r*count, (r+1)*count). */
int gm_zero1_allgather_async(uintptr_t zero1, uintptr_t arena_base, int64_t count_per_rank,
                             int elem_bytes);
/* Update of this rank's shard, then the all-gather, on one stream: any fp32 rule
 * (GM_RULE_*; stream 0 of the list is the parameters), or Adam by name. */
int gm_zero1_step_async(uintptr_t zero1, int rule, uintptr_t shard_list, const gm_hyper_t* hyper,
                        uintptr_t arena_base, int64_t count_per_rank);
int gm_zero1_adam_step_async(uintptr_t zero1, uintptr_t shard_list, const gm_hyper_t* hyper,
                             uintptr_t arena_base, int64_t count_per_rank);
int gm_zero1_rank(uintptr_t zero1);
int gm_zero1_world(uintptr_t zero1);
/* Fused update + exchange: one kernel updates the shard and stores every new
 * parameter to the same offset of each peer's arena through peer-mapped
 * pointers (plain stores over NVLink).  Setup: each rank exports its arena
 * with gm_zero1_ipc_handle (64 bytes), the caller exchanges the handles by
 * any host channel, and gm_zero1_open_peers maps them (rank order).  The
 * step ends with a one-word all-reduce that acts as the cross-rank barrier.
 * arena_base must be the first byte of its device allocation (an IPC handle
 * maps whole allocations); anything else is refused with -10. */
#define GM_IPC_HANDLE_BYTES 64
int gm_zero1_ipc_handle(uintptr_t zero1, uintptr_t arena_base, void* out_handle);
int gm_zero1_open_peers(uintptr_t zero1, const void* handles);
int gm_zero1_adam_push_step_async(uintptr_t zero1, uintptr_t shard_list, const gm_hyper_t* hyper);
/* The same step for a caller whose gradients and parameters live in pinned HOST memory:
 * the rank's gradient shard is uploaded, updated and pushed, and its new parameters are
 * downloaded, slice by slice on three streams as in gm_step_host.  host_grads /
 * host_params hold the shard's tensors back to back in list order.  Synchronous. */
int gm_zero1_adam_push_step_host(uintptr_t zero1, uintptr_t shard_list, const gm_hyper_t* hyper,
                                 const void* host_grads, void* host_params, int num_slices);
/* Update + exchange through the copy engines: the shard is updated in
 * `num_slices` groups of whole tensors and every finished slice is copied to
 * the same offset of each peer's arena (one cudaMemcpyAsync per peer and
 * slice, on per-peer streams) while the next slice is being updated.  Needs
 * the peer mapping of gm_zero1_open_peers and parameter tensors that lie back
 * to back in the arena.  Ends with the same one-word all-reduce barrier. */
int gm_zero1_adam_dma_step_async(uintptr_t zero1, uintptr_t shard_list, const gm_hyper_t* hyper, int num_slices);

/* Mixed-precision Adam over sharded fp16 gradients: the overflow flags of all
 * ranks are summed between the check and the update (one-word all-reduce on the
 * stream), so every rank takes the same skip/step decision and keeps the same
 * loss-scale state; then the fp16 parameter arena is all-gathered in place. */
int gm_zero1_mixed_step_async(uintptr_t zero1, uintptr_t mixed, uintptr_t shard_list, float lr, float eps,
                              float weight_decay, uintptr_t p16_arena_base, int64_t count_per_rank);

/* The same step with the exchange fused into the update kernel: every new fp16 parameter
 * vector is stored to the local fp16 arena and to the same offset of each peer's, by plain
 * stores over NVLink, and a one-word all-reduce closes the step.  The fp16 arena is a
 * second exported arena: slot 1 of gm_zero1_ipc_handle_slot / gm_zero1_open_peers_slot
 * (slot 0 is the fp32 arena of gm_zero1_ipc_handle / gm_zero1_open_peers). */
int gm_zero1_ipc_handle_slot(uintptr_t zero1, int slot, uintptr_t arena_base, void* out_handle);
int gm_zero1_open_peers_slot(uintptr_t zero1, int slot, const void* handles);
int gm_zero1_mixed_push_step_async(uintptr_t zero1, uintptr_t mixed, uintptr_t shard_list, float lr, float eps,
                                   float weight_decay);

/* Gradient hand-off of data-parallel training: in-place reduce-scatter (sum) of
 * the full gradient arena; afterwards rank r's shard holds the sum over ranks. */
int gm_zero1_reduce_scatter_async(uintptr_t zero1, uintptr_t grad_arena_base, int64_t count_per_rank, int elem_bytes);

/* ---- self-check ----
 * The mixed-precision update divides by the two Adam bias corrections, which are the
 * same for every element of a step, with a five-instruction sequence built on the
 * correctly rounded reciprocal instead of the general IEEE division; it must give the
 * same bits.  This entry compares the two on the GPU over all 2^32 values of the
 * dividend for one divisor c and reports how many differ (and the first such bit
 * pattern, 0xffffffff if none).  *fast_path_allowed is 0 when c lies outside the range
 * the library enables the sequence for (it then uses the IEEE division). */
int gm_selftest_const_div(uintptr_t device_ptr, float c, uint64_t* mismatches, uint32_t* first_bad_bits,
                          int* fast_path_allowed);
/* The single-launch steps synchronise their CTAs with a grid-wide barrier whose wait is
 * bounded.  This entry runs that wait on a word nothing sets, with a budget of
 * budget_cycles GPU clock cycles: it must return with *gave_up == 1 and leave the device
 * usable (a step whose barrier gives up reports GM_ERR_TIMEOUT). */
int gm_selftest_barrier_timeout(uintptr_t device_ptr, long long budget_cycles, int* gave_up);

/* ---- timing on the device's stream (CUDA events) ---- */
int gm_timer_start(uintptr_t device_ptr);                  /* records the start event */
int gm_timer_stop(uintptr_t device_ptr, float* elapsed_ms);/* records the stop event, waits, reports */

#ifdef __cplusplus
}
#endif
#endif /* GOMETAL_CUDA_H */

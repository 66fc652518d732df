// gm_rules.cu -- the six elementwise update rules as multi-tensor-apply
// kernels, and the drop-in C entries that replace
// execute_{sgd,adam,rmsprop,adagrad,adadelta,nadam}_step_mpsgraph of
// cgo_bridge/bridge_optimizer.m.  Each rule's operation order is the graph
// order of that file (line ranges at each rule); host-side scalars (1-beta,
// bias corrections, NAdam's schedule) are formed on the host with powf exactly
// as the reference forms them and reach the kernel as arguments.
#include <math.h>

#include "gm_apply.cuh"

namespace gm {

// ---- NAdam: bridge_optimizer.m:2061-2066 (host), :2114-2200 (graph) ----
struct NadamRule {
    static constexpr int NS = 4;
    static constexpr unsigned WMASK = 0b1101;
    struct P { float lr, beta1, beta2, omb1, omb2, bc1, bc2, eps, wd, mu_next, om_mu; int use_wd; };
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) {
        const float w = x[0], g = x[1];
        const float m_new = add(mul(x[2], p.beta1), mul(g, p.omb1));
        const float v_new = add(mul(x[3], p.beta2), mul(mul(g, g), p.omb2));
        const float v_hat = dvd0(v_new, p.bc2);
        const float m_hat = dvd0(m_new, p.bc1);
        const float g_hat = dvd0(g, p.bc1);
        const float m_bar = add(mul(m_hat, p.mu_next), mul(g_hat, p.om_mu));
        float upd = dvd0(m_bar, add(root0(v_hat), p.eps));
        if (p.use_wd) upd = add(upd, mul(w, p.wd));
        x[0] = sub(w, mul(upd, p.lr));
        x[2] = m_new;
        x[3] = v_new;
    }
};

// ---- SGD: bridge_optimizer.m:219-228 (decay), :244-278 (momentum), :315-322 (plain) ----
struct SgdScalars { float lr, momentum, wd; int use_wd, nesterov; };

struct SgdPlainRule {
    static constexpr int NS = 2;                 // w, g
    static constexpr unsigned WMASK = 0b01;
    using P = SgdScalars;
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) {
        const float w = x[0];
        float gf = x[1];
        if (p.use_wd) gf = add(x[1], mul(w, p.wd));
        x[0] = sub(w, mul(p.lr, gf));
    }
};

struct SgdMomentumRule {
    static constexpr int NS = 3;                 // w, g, momentum
    static constexpr unsigned WMASK = 0b101;
    using P = SgdScalars;
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) {
        const float w = x[0];
        float gf = x[1];
        if (p.use_wd) gf = add(x[1], mul(w, p.wd));
        const float m_new = add(mul(x[2], p.momentum), gf);
        float stepv;
        if (p.nesterov) stepv = mul(p.lr, add(mul(p.momentum, m_new), gf));
        else stepv = mul(p.lr, m_new);
        x[0] = sub(w, stepv);
        x[2] = m_new;
    }
};

// ---- RMSProp: bridge_optimizer.m:782-876.  The reference stores only w and
// the squared average (:915-937); here the momentum and gradient-average
// streams are stored too so those modes keep state between steps. ----
struct RmsScalars { float lr, alpha, oma, eps, wd, momentum; int use_wd; };

template <bool MOM, bool CEN>
struct RmsPropRule {
    static constexpr int NS = 3 + (MOM ? 1 : 0) + (CEN ? 1 : 0);   // w, g, sq, [mom], [gavg]
    static constexpr int MOM_S = 3;
    static constexpr int CEN_S = 3 + (MOM ? 1 : 0);
    static constexpr unsigned WMASK = 0b101u | (MOM ? (1u << MOM_S) : 0u) | (CEN ? (1u << CEN_S) : 0u);
    using P = RmsScalars;
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) {
        const float w = x[0], g = x[1];
        const float sq_new = add(mul(x[2], p.alpha), mul(mul(g, g), p.oma));
        float denom;
        if (CEN) {
            const float a_new = add(mul(x[CEN_S < NS ? CEN_S : 0], p.alpha), mul(g, p.oma));
            denom = root(add(sub(sq_new, mul(a_new, a_new)), p.eps));
            x[CEN_S < NS ? CEN_S : 0] = a_new;
        } else {
            denom = root(add(sq_new, p.eps));
        }
        float upd = dvd0(g, denom);
        if (MOM) {
            const float b_new = add(mul(x[MOM_S < NS ? MOM_S : 0], p.momentum), upd);
            x[MOM_S < NS ? MOM_S : 0] = b_new;
            upd = b_new;
        }
        if (p.use_wd) upd = add(upd, mul(w, p.wd));
        x[0] = sub(w, mul(upd, p.lr));
        x[2] = sq_new;
    }
};

// ---- AdaGrad: bridge_optimizer.m:1480-1517 ----
struct AdaGradRule {
    static constexpr int NS = 3;                 // w, g, sq
    static constexpr unsigned WMASK = 0b101;
    struct P { float lr, eps, wd; int use_wd; };
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) {
        const float w = x[0];
        float gf = x[1];
        if (p.use_wd) gf = add(x[1], mul(w, p.wd));
        const float acc = add(x[2], mul(gf, gf));
        const float adj = dvd(p.lr, add(root0(acc), p.eps));
        x[0] = sub(w, mul(adj, gf));
        x[2] = acc;
    }
};

// ---- AdaDelta: bridge_optimizer.m:1773-1843 ----
struct AdaDeltaRule {
    static constexpr int NS = 4;                 // w, g, sq, upd
    static constexpr unsigned WMASK = 0b1101;
    struct P { float rho, omr, eps, wd; int use_wd; };
    static __device__ __forceinline__ void elem(float (&x)[NS], const P& p) {
        const float w = x[0];
        float gf = x[1];
        if (p.use_wd) gf = add(x[1], mul(w, p.wd));
        const float e_new = add(mul(x[2], p.rho), mul(mul(gf, gf), p.omr));
        const float rms_g = root(add(e_new, p.eps));
        const float rms_u = root(add(x[3], p.eps));
        const float neg = -mul(dvd(rms_u, rms_g), gf);
        x[0] = add(w, neg);
        x[2] = e_new;
        x[3] = add(mul(x[3], p.rho), mul(mul(neg, neg), p.omr));
    }
};

int apply_window(const TensorList* l, Window win, DevList* out) {
    *out = l->dl;
    if (win.count < 0) return GM_OK;
    if (win.begin < 0 || win.begin + win.count > l->dl.num_chunks) { set_error("launch window outside the list"); return GM_ERR_BAD_ARG; }
    out->chunk_rec += win.begin;
    out->num_chunks = win.count;
    return GM_OK;
}

int launch_rule(Device* d, int rule, const TensorList* l, const gm_hyper_t& h, Window win, const float* clip) {
    DeviceGuard guard(d);
    const int use_wd = h.weight_decay > 0.0f ? 1 : 0;
    switch (rule) {
        case GM_RULE_ADAM: {
            if (h.step < 1) { set_error("Adam step count %d must be >= 1", h.step); return GM_ERR_BAD_ARG; }
            AdamRule::P p;
            p.lr = h.lr; p.beta1 = h.beta1; p.beta2 = h.beta2; p.eps = h.eps; p.wd = h.weight_decay; p.use_wd = use_wd;
            p.bc1 = 1.0f - powf(h.beta1, (float)h.step);
            p.bc2 = 1.0f - powf(h.beta2, (float)h.step);
            p.omb1 = 1.0f - h.beta1;
            p.omb2 = 1.0f - h.beta2;
            p.rbc1 = 0.0f; p.rbc2 = 0.0f;
            return launch_apply<AdamRule>(d, l, p, win, clip);
        }
        case GM_RULE_NADAM: {
            if (h.step < 1) { set_error("NAdam step count %d must be >= 1", h.step); return GM_ERR_BAD_ARG; }
            NadamRule::P p;
            p.lr = h.lr; p.beta1 = h.beta1; p.beta2 = h.beta2; p.eps = h.eps; p.wd = h.weight_decay; p.use_wd = use_wd;
            p.bc1 = 1.0f - powf(h.beta1, (float)h.step);
            p.bc2 = 1.0f - powf(h.beta2, (float)h.step);
            p.omb1 = 1.0f - h.beta1;
            p.omb2 = 1.0f - h.beta2;
            p.mu_next = h.beta1 * (1.0f - 0.5f * powf(0.96f, (float)(h.step + 1) * 0.004f));
            p.om_mu = 1.0f - p.mu_next;
            return launch_apply<NadamRule>(d, l, p, win, clip);
        }
        case GM_RULE_SGD: {
            SgdScalars p;
            p.lr = h.lr; p.momentum = h.beta1; p.wd = h.weight_decay; p.use_wd = use_wd; p.nesterov = h.nesterov ? 1 : 0;
            if (l->dl.num_streams == 3 && h.beta1 > 0.0f) return launch_apply<SgdMomentumRule>(d, l, p, win, clip);
            if (l->dl.num_streams == 2) return launch_apply<SgdPlainRule>(d, l, p, win, clip);
            set_error("SGD needs streams w,g (momentum==0) or w,g,mom (momentum>0); got %d streams, momentum %g",
                      l->dl.num_streams, (double)h.beta1);
            return GM_ERR_BAD_ARG;
        }
        case GM_RULE_RMSPROP: {
            RmsScalars p;
            p.lr = h.lr; p.alpha = h.beta1; p.oma = 1.0f - h.beta1; p.eps = h.eps; p.wd = h.weight_decay;
            p.momentum = h.momentum; p.use_wd = use_wd;
            const bool mom = h.momentum > 0.0f, cen = h.centered != 0;
            if (mom && cen) return launch_apply<RmsPropRule<true, true>>(d, l, p, win, clip);
            if (mom) return launch_apply<RmsPropRule<true, false>>(d, l, p, win, clip);
            if (cen) return launch_apply<RmsPropRule<false, true>>(d, l, p, win, clip);
            return launch_apply<RmsPropRule<false, false>>(d, l, p, win, clip);
        }
        case GM_RULE_ADAGRAD: {
            AdaGradRule::P p;
            p.lr = h.lr; p.eps = h.eps; p.wd = h.weight_decay; p.use_wd = use_wd;
            return launch_apply<AdaGradRule>(d, l, p, win, clip);
        }
        case GM_RULE_ADADELTA: {
            AdaDeltaRule::P p;
            p.rho = h.beta1; p.omr = 1.0f - h.beta1; p.eps = h.eps; p.wd = h.weight_decay; p.use_wd = use_wd;
            return launch_apply<AdaDeltaRule>(d, l, p, win, clip);
        }
        default:
            set_error("unknown rule %d", rule);
            return GM_ERR_BAD_ARG;
    }
}

// Shared body of the drop-in entries: validate, fetch the cached descriptor,
// launch, wait.
static int dropin_step(uintptr_t device_ptr, int rule, int num_streams, uintptr_t* const* streams,
                       int num_weights, const int* buffer_sizes, const gm_hyper_t& h) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (num_weights <= 0) { set_error("num_weights %d is not positive", num_weights); return GM_ERR_BAD_ARG; }
    if (!buffer_sizes) { set_error("buffer_sizes is nil"); return GM_ERR_BAD_ARG; }
    for (int s = 0; s < num_streams; ++s) {
        if (!streams[s]) { set_error("buffer array %d is nil", s); return GM_ERR_NIL_BUFFER; }
    }
    std::vector<int64_t> numel(num_weights);
    for (int i = 0; i < num_weights; ++i) {
        if (buffer_sizes[i] <= 0 || buffer_sizes[i] % 4 != 0) {
            set_error("buffer_sizes[%d]=%d is not a positive multiple of 4", i, buffer_sizes[i]);
            return GM_ERR_BAD_SIZE;
        }
        numel[i] = buffer_sizes[i] / 4;
    }
    int err = GM_OK;
    TensorList* l = build_list(d, num_streams, num_weights, streams, numel.data(), nullptr, true, &err);
    if (!l) return err;
    int rc = launch_rule(d, rule, l, h);
    if (rc != GM_OK) return rc;
    DeviceGuard guard(d);
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return GM_OK;
}

// The list is cut into `num_slices` groups of whole tensors and the three stages of each
// slice -- gradients host->device, `launch` over the slice's chunks, parameters
// device->host -- run on three streams, so the upload of slice s+1 and the download of
// slice s-1 overlap the kernel of slice s and both PCIe directions are busy at once.
// host_grads / host_params hold the tensors back to back in list order; the device
// gradient (stream 1) and parameter (stream 0) tensors may be one flat run (one copy per
// slice and direction) or separate allocations (one copy each).  `finish`, when given, is
// enqueued on the device stream after the last slice.  Waits for everything.
int host_pipelined_step(Device* d, const TensorList* l, const void* host_grads, void* host_params, int num_slices,
                        const std::function<int(Window)>& launch, const std::function<int()>& finish) {
    if (l->dl.num_streams < 2) { set_error("list needs at least the parameter and gradient streams"); return GM_ERR_BAD_ARG; }
    const int T = l->dl.num_tensors;
    if (l->elem_bytes[0] != 4 || l->elem_bytes[1] != 4) { set_error("the host-buffer step needs fp32 parameters and gradients"); return GM_ERR_BAD_ARG; }
    bool packed = true;
    for (int t = 0; t + 1 < T && packed; ++t)
        for (int s = 0; s < 2; ++s)
            if (l->ptrs[s][t] + (uintptr_t)l->numel[t] * 4 != l->ptrs[s][t + 1]) packed = false;
    if (num_slices < 1) num_slices = 1;
    if (num_slices > T) num_slices = T;
    DeviceGuard guard(d);
    if (!d->h2d_stream) GM_CUDA_CHECK(cudaStreamCreateWithFlags(&d->h2d_stream, cudaStreamNonBlocking));
    if (!d->d2h_stream) GM_CUDA_CHECK(cudaStreamCreateWithFlags(&d->d2h_stream, cudaStreamNonBlocking));
    while ((int)d->slice_events.size() < 2 * num_slices) {
        cudaEvent_t e;
        GM_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        d->slice_events.push_back(e);
    }
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));          // earlier work on the buffers is finished
    size_t host_off = 0;
    int rc = GM_OK;
    for (int s = 0; s < num_slices; ++s) {
        const int t0 = (int)((long long)T * s / num_slices), t1 = (int)((long long)T * (s + 1) / num_slices);
        if (t1 <= t0) continue;
        size_t bytes = 0;
        for (int t = t0; t < t1; ++t) bytes += (size_t)l->numel[t] * 4;
        cudaEvent_t in = d->slice_events[2 * s], done = d->slice_events[2 * s + 1];
        if (packed) {
            GM_CUDA_CHECK(cudaMemcpyAsync((void*)l->ptrs[1][t0], (const char*)host_grads + host_off, bytes, cudaMemcpyHostToDevice, d->h2d_stream));
        } else {
            size_t off = host_off;
            for (int t = t0; t < t1; ++t) {
                const size_t tb = (size_t)l->numel[t] * 4;
                GM_CUDA_CHECK(cudaMemcpyAsync((void*)l->ptrs[1][t], (const char*)host_grads + off, tb, cudaMemcpyHostToDevice, d->h2d_stream));
                off += tb;
            }
        }
        GM_CUDA_CHECK(cudaEventRecord(in, d->h2d_stream));
        GM_CUDA_CHECK(cudaStreamWaitEvent(d->stream, in, 0));
        Window win;
        win.begin = l->chunk_prefix[t0];
        win.count = l->chunk_prefix[t1] - l->chunk_prefix[t0];
        rc = launch(win);
        if (rc != GM_OK) break;
        GM_CUDA_CHECK(cudaEventRecord(done, d->stream));
        GM_CUDA_CHECK(cudaStreamWaitEvent(d->d2h_stream, done, 0));
        if (packed) {
            GM_CUDA_CHECK(cudaMemcpyAsync((char*)host_params + host_off, (const void*)l->ptrs[0][t0], bytes, cudaMemcpyDeviceToHost, d->d2h_stream));
        } else {
            size_t off = host_off;
            for (int t = t0; t < t1; ++t) {
                const size_t tb = (size_t)l->numel[t] * 4;
                GM_CUDA_CHECK(cudaMemcpyAsync((char*)host_params + off, (const void*)l->ptrs[0][t], tb, cudaMemcpyDeviceToHost, d->d2h_stream));
                off += tb;
            }
        }
        host_off += bytes;
    }
    if (rc == GM_OK && finish) rc = finish();
    cudaError_t e1 = cudaStreamSynchronize(d->h2d_stream);
    cudaError_t e2 = cudaStreamSynchronize(d->stream);
    cudaError_t e3 = cudaStreamSynchronize(d->d2h_stream);
    if (rc != GM_OK) return rc;
    if (e1 != cudaSuccess) return cuda_fail(e1, "host step (upload)");
    if (e2 != cudaSuccess) return cuda_fail(e2, "host step (update)");
    if (e3 != cudaSuccess) return cuda_fail(e3, "host step (download)");
    return GM_OK;
}

}  // namespace gm

using namespace gm;

extern "C" {

int gm_step_async(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    TensorList* l = as_list(list);
    if (!l) return GM_ERR_BAD_ARG;
    if (!hyper) { set_error("hyper-parameters are nil"); return GM_ERR_BAD_ARG; }
    if (l->dev != d) { set_error("tensor list belongs to another device"); return GM_ERR_BAD_ARG; }
    return launch_rule(d, rule, l, *hyper);
}

int gm_step_timed(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper, float* elapsed_ms) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    TensorList* l = as_list(list);
    if (!l) return GM_ERR_BAD_ARG;
    if (!hyper || !elapsed_ms) { set_error("nil argument"); return GM_ERR_BAD_ARG; }
    DeviceGuard guard(d);
    GM_CUDA_CHECK(cudaEventRecord(d->ev_start, d->stream));
    int rc = launch_rule(d, rule, l, *hyper);
    if (rc != GM_OK) return rc;
    GM_CUDA_CHECK(cudaEventRecord(d->ev_stop, d->stream));
    GM_CUDA_CHECK(cudaEventSynchronize(d->ev_stop));
    GM_CUDA_CHECK(cudaEventElapsedTime(elapsed_ms, d->ev_start, d->ev_stop));
    return GM_OK;
}

// One optimizer step for a caller whose gradients and parameters live in HOST
// memory (pinned): see host_pipelined_step.  Synchronous: host_params is complete on return.
int gm_step_host(uintptr_t device_ptr, int rule, uintptr_t list, const gm_hyper_t* hyper, const void* host_grads,
                 void* host_params, int num_slices) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    TensorList* l = as_list(list);
    if (!l) return GM_ERR_BAD_ARG;
    if (!hyper || !host_grads || !host_params) { set_error("nil argument"); return GM_ERR_BAD_ARG; }
    if (l->dev != d) { set_error("tensor list belongs to another device"); return GM_ERR_BAD_ARG; }
    const gm_hyper_t hy = *hyper;
    return host_pipelined_step(d, l, host_grads, host_params, num_slices,
                               [&](Window win) { return launch_rule(d, rule, l, hy, win); }, nullptr);
}

int execute_adam_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* m, uintptr_t* v,
                           int num_weights, int* buffer_sizes, float lr, float beta1, float beta2,
                           float epsilon, float weight_decay, int step_count) {
    uintptr_t* streams[4] = {w, g, m, v};
    gm_hyper_t h{};
    h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = epsilon; h.weight_decay = weight_decay; h.step = step_count;
    return dropin_step(device_ptr, GM_RULE_ADAM, 4, streams, num_weights, buffer_sizes, h);
}

// The reference's pooled variant is a stub that returns 0 without updating
// anything (bridge_optimizer.m:676-681); here it performs the step on the
// device's own stream and ignores the pool handle.
int execute_adam_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* m, uintptr_t* v,
                                  int num_weights, int* buffer_sizes, float lr, float beta1, float beta2,
                                  float epsilon, float weight_decay, int step_count, uintptr_t command_pool) {
    (void)command_pool;
    return execute_adam_step_cuda(device_ptr, w, g, m, v, num_weights, buffer_sizes, lr, beta1, beta2,
                                  epsilon, weight_decay, step_count);
}

int execute_nadam_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* m, uintptr_t* v,
                            int num_weights, int* buffer_sizes, float lr, float beta1, float beta2,
                            float epsilon, float weight_decay, int step_count) {
    uintptr_t* streams[4] = {w, g, m, v};
    gm_hyper_t h{};
    h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = epsilon; h.weight_decay = weight_decay; h.step = step_count;
    return dropin_step(device_ptr, GM_RULE_NADAM, 4, streams, num_weights, buffer_sizes, h);
}

int execute_sgd_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* mom, int num_weights,
                          int* buffer_sizes, float lr, float momentum, float weight_decay, int nesterov,
                          int step_count) {
    (void)step_count;
    gm_hyper_t h{};
    h.lr = lr; h.weight_decay = weight_decay; h.nesterov = nesterov;
    // bridge_optimizer.m:233: the momentum branch needs momentum > 0 and a buffer.
    bool use_mom = momentum > 0.0f && mom != nullptr;
    if (use_mom) {
        for (int i = 0; i < num_weights && use_mom; ++i) use_mom = mom[i] != 0;
    }
    if (use_mom) {
        uintptr_t* streams[3] = {w, g, mom};
        h.beta1 = momentum;
        return dropin_step(device_ptr, GM_RULE_SGD, 3, streams, num_weights, buffer_sizes, h);
    }
    uintptr_t* streams[2] = {w, g};
    h.beta1 = 0.0f;
    return dropin_step(device_ptr, GM_RULE_SGD, 2, streams, num_weights, buffer_sizes, h);
}

int execute_rmsprop_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* sq, uintptr_t* mom,
                              uintptr_t* gavg, int num_weights, int* buffer_sizes, float lr, float alpha,
                              float epsilon, float weight_decay, float momentum, bool centered, int step_count) {
    (void)step_count;
    // bridge_optimizer.m:745-752: momentum>0 / centered without the buffer is an error.
    if (momentum > 0.0f && !mom) { set_error("momentum > 0 without momentum buffers"); return GM_ERR_AUX_BUFFER; }
    if (centered && !gavg) { set_error("centered without gradient-average buffers"); return -6; }
    uintptr_t* streams[5] = {w, g, sq, nullptr, nullptr};
    int ns = 3;
    if (momentum > 0.0f) streams[ns++] = mom;
    if (centered) streams[ns++] = gavg;
    gm_hyper_t h{};
    h.lr = lr; h.beta1 = alpha; h.eps = epsilon; h.weight_decay = weight_decay; h.momentum = momentum;
    h.centered = centered ? 1 : 0;
    return dropin_step(device_ptr, GM_RULE_RMSPROP, ns, streams, num_weights, buffer_sizes, h);
}

int execute_adagrad_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* sq, int num_weights,
                              int* buffer_sizes, float lr, float epsilon, float weight_decay) {
    uintptr_t* streams[3] = {w, g, sq};
    gm_hyper_t h{};
    h.lr = lr; h.eps = epsilon; h.weight_decay = weight_decay;
    return dropin_step(device_ptr, GM_RULE_ADAGRAD, 3, streams, num_weights, buffer_sizes, h);
}

int execute_adagrad_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* sq,
                                     int num_weights, int* buffer_sizes, float lr, float epsilon,
                                     float weight_decay, uintptr_t command_pool) {
    (void)command_pool;
    return execute_adagrad_step_cuda(device_ptr, w, g, sq, num_weights, buffer_sizes, lr, epsilon, weight_decay);
}

int execute_adadelta_step_cuda(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* sq, uintptr_t* upd,
                               int num_weights, int* buffer_sizes, float rho, float epsilon, float weight_decay) {
    uintptr_t* streams[4] = {w, g, sq, upd};
    gm_hyper_t h{};
    h.beta1 = rho; h.eps = epsilon; h.weight_decay = weight_decay;
    return dropin_step(device_ptr, GM_RULE_ADADELTA, 4, streams, num_weights, buffer_sizes, h);
}

int execute_adadelta_step_cuda_pooled(uintptr_t device_ptr, uintptr_t* w, uintptr_t* g, uintptr_t* sq,
                                      uintptr_t* upd, int num_weights, int* buffer_sizes, float rho,
                                      float epsilon, float weight_decay, uintptr_t command_pool) {
    (void)command_pool;
    return execute_adadelta_step_cuda(device_ptr, w, g, sq, upd, num_weights, buffer_sizes, rho, epsilon,
                                      weight_decay);
}

}  // extern "C"

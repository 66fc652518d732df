// gm_host_capi.cpp -- flat C handle API over the C++ host mirror, so the host
// logic can be driven from pytest (ctypes).  Strings come back through a
// thread-local buffer; errors as a non-zero return plus gmh_last_error().
#include <string.h>

#include <set>

#include "gm_host.hpp"

using namespace gometal;

namespace {

thread_local std::string g_err;
thread_local std::string g_str;

int fail(const std::string& e) { g_err = e; return e.empty() ? 0 : -1; }

struct OptHandle {
    std::unique_ptr<optimizer::Optimizer> opt;
    std::unique_ptr<optimizer::LBFGSOptimizerState> lbfgs;
};

}  // namespace

#define GMH_API extern "C" __attribute__((visibility("default")))

GMH_API const char* gmh_last_error() { return g_err.c_str(); }
GMH_API int gmh_init(const char* backend_path) { return fail(backend().load(backend_path ? backend_path : "")); }
GMH_API uintptr_t gmh_device_create() { return backend().create_device ? backend().create_device() : 0; }
GMH_API void gmh_device_destroy(uintptr_t d) { if (backend().destroy_device) backend().destroy_device(d); }

// ---- memory manager ----
GMH_API void* gmh_mm_create(uintptr_t device) { return new memory::MemoryManager(device); }
GMH_API int gmh_mm_use_arena(void* mm, int64_t bytes) { return fail(static_cast<memory::MemoryManager*>(mm)->UseArena(bytes)); }
GMH_API void gmh_mm_destroy(void* mm) { delete static_cast<memory::MemoryManager*>(mm); }
GMH_API uintptr_t gmh_mm_allocate(void* mm, int size) { return static_cast<memory::MemoryManager*>(mm)->AllocateBuffer(size); }
GMH_API void gmh_mm_release(void* mm, uintptr_t p) { static_cast<memory::MemoryManager*>(mm)->ReleaseBuffer(p); }
GMH_API int gmh_mm_tracked_size(void* mm, uintptr_t p) { return static_cast<memory::MemoryManager*>(mm)->trackedSize(p); }
GMH_API int gmh_find_pool_size(int size) { return memory::findPoolSize(size); }
GMH_API int gmh_calculate_max_pool_size(int size) { return memory::calculateMaxPoolSize(size); }
GMH_API int gmh_mm_stats(void* mm, int tier, int* available, int* allocated, int* max_size) {
    auto st = static_cast<memory::MemoryManager*>(mm)->Stats();
    auto it = st.find(tier);
    if (it == st.end()) return -1;
    *available = it->second.available; *allocated = it->second.allocated; *max_size = it->second.maxSize;
    return 0;
}

// ---- helpers ----
GMH_API int gmh_extract_buffer_index(const char* name) { return optimizer::extractBufferIndex(name ? name : ""); }
GMH_API int gmh_calculate_tensor_size(const int* shape, int nd) {
    return optimizer::calculateTensorSize(std::vector<int>(shape, shape + nd));
}

// ---- state objects ----
GMH_API void* gmh_state_new(const char* type) { auto* s = new OptimizerState(); s->Type = type ? type : ""; return s; }
GMH_API void gmh_state_destroy(void* s) { delete static_cast<OptimizerState*>(s); }
GMH_API const char* gmh_state_type(void* s) { return static_cast<OptimizerState*>(s)->Type.c_str(); }
GMH_API void gmh_state_set_float64(void* s, const char* key, double v) { Param p; p.kind = Param::Float64; p.f = v; static_cast<OptimizerState*>(s)->Parameters[key] = p; }
GMH_API void gmh_state_set_bool(void* s, const char* key, int v) { Param p; p.kind = Param::Bool; p.b = v != 0; static_cast<OptimizerState*>(s)->Parameters[key] = p; }
GMH_API void gmh_state_set_uint64(void* s, const char* key, uint64_t v) { Param p; p.kind = Param::Uint64; p.u = v; static_cast<OptimizerState*>(s)->Parameters[key] = p; }
// kind: 0 float64, 1 bool, 2 uint64, 3 float32, -1 missing
GMH_API int gmh_state_get_param(void* s, const char* key, double* value) {
    auto& P = static_cast<OptimizerState*>(s)->Parameters;
    auto it = P.find(key);
    if (it == P.end()) return -1;
    switch (it->second.kind) {
        case Param::Float64: *value = it->second.f; return 0;
        case Param::Bool: *value = it->second.b ? 1.0 : 0.0; return 1;
        case Param::Uint64: *value = (double)it->second.u; return 2;
        default: *value = it->second.f; return 3;
    }
}
GMH_API float gmh_extract_float32_param(void* s, const char* key, float def) { return optimizer::extractFloat32Param(static_cast<OptimizerState*>(s)->Parameters, key, def); }
GMH_API int gmh_extract_bool_param(void* s, const char* key, int def) { return optimizer::extractBoolParam(static_cast<OptimizerState*>(s)->Parameters, key, def != 0) ? 1 : 0; }
GMH_API uint64_t gmh_extract_uint64_param(void* s, const char* key, uint64_t def) { return optimizer::extractUint64Param(static_cast<OptimizerState*>(s)->Parameters, key, def); }
GMH_API float gmh_pow(float x, float y) { return optimizer::pow(x, y); }
GMH_API int gmh_validate_state_type(const char* type, void* s) { return fail(optimizer::validateStateType(type, *static_cast<OptimizerState*>(s))); }
GMH_API void gmh_state_add_tensor(void* s, const char* name, const char* state_type, const float* data, int n) {
    OptimizerTensor t;
    t.Name = name; t.StateType = state_type; t.Shape = {n}; t.Data.assign(data, data + n);
    static_cast<OptimizerState*>(s)->StateData.push_back(std::move(t));
}
GMH_API int gmh_state_num_tensors(void* s) { return (int)static_cast<OptimizerState*>(s)->StateData.size(); }
GMH_API const char* gmh_state_tensor_name(void* s, int i) { return static_cast<OptimizerState*>(s)->StateData[i].Name.c_str(); }
GMH_API const char* gmh_state_tensor_type(void* s, int i) { return static_cast<OptimizerState*>(s)->StateData[i].StateType.c_str(); }
GMH_API int gmh_state_tensor_numel(void* s, int i) { return (int)static_cast<OptimizerState*>(s)->StateData[i].Data.size(); }
GMH_API int gmh_state_tensor_shape0(void* s, int i) { auto& sh = static_cast<OptimizerState*>(s)->StateData[i].Shape; return sh.size() == 1 ? sh[0] : -1; }
GMH_API void gmh_state_tensor_data(void* s, int i, float* out) {
    auto& d = static_cast<OptimizerState*>(s)->StateData[i].Data;
    memcpy(out, d.data(), d.size() * sizeof(float));
}

// JSON text of a state (thread-local buffer, valid until the next call) and back.
GMH_API const char* gmh_state_to_json(void* s) {
    std::string e = checkpoints::EncodeOptimizerState(*static_cast<OptimizerState*>(s), &g_str);
    if (!e.empty()) { g_err = e; return nullptr; }
    return g_str.c_str();
}
GMH_API void* gmh_state_from_json(const char* text) {
    auto* s = new OptimizerState();
    std::string e = checkpoints::DecodeOptimizerState(text ? text : "", s);
    if (!e.empty()) { g_err = e; delete s; return nullptr; }
    return s;
}

// ---- optimizers ----
// cfg layout per type (missing trailing values keep the reference defaults; pass ncfg = 0 for Default*Config()):
//   SGD      lr, momentum, weight_decay, nesterov
//   Adam     lr, beta1, beta2, epsilon, weight_decay
//   RMSProp  lr, alpha, epsilon, weight_decay, momentum, centered
//   AdaGrad  lr, epsilon, weight_decay
//   AdaDelta rho, epsilon, weight_decay
//   Nadam    lr, beta1, beta2, epsilon, weight_decay
//   LBFGS    history_size, line_search_tol, max_line_search, c1, c2, initial_step
//   MixedAdam lr, beta1, beta2, epsilon, weight_decay, initial_loss_scale, growth, backoff, growth_interval, max_loss_scale
GMH_API void* gmh_optimizer_create(const char* type, const double* cfg, int ncfg, const int* shape_flat, const int* shape_ndims,
                                   int num_weights, void* mm, uintptr_t device) {
    optimizer::Shapes shapes;
    int at = 0;
    for (int i = 0; i < num_weights; ++i) {
        shapes.emplace_back(shape_flat + at, shape_flat + at + shape_ndims[i]);
        at += shape_ndims[i];
    }
    auto get = [&](int i, double def) { return i < ncfg ? cfg[i] : def; };
    auto* M = static_cast<memory::MemoryManager*>(mm);
    std::string err;
    std::unique_ptr<OptHandle> h(new OptHandle());
    const std::string t = type ? type : "";
    if (t == "SGD") {
        optimizer::SGDConfig c; c.LearningRate = (float)get(0, c.LearningRate); c.Momentum = (float)get(1, c.Momentum);
        c.WeightDecay = (float)get(2, c.WeightDecay); c.Nesterov = get(3, c.Nesterov) != 0;
        h->opt = optimizer::NewSGDOptimizer(c, shapes, M, device, &err);
    } else if (t == "Adam") {
        optimizer::AdamConfig c; c.LearningRate = (float)get(0, c.LearningRate); c.Beta1 = (float)get(1, c.Beta1); c.Beta2 = (float)get(2, c.Beta2);
        c.Epsilon = (float)get(3, c.Epsilon); c.WeightDecay = (float)get(4, c.WeightDecay);
        h->opt = optimizer::NewAdamOptimizer(c, shapes, M, device, &err);
    } else if (t == "RMSProp") {
        optimizer::RMSPropConfig c; c.LearningRate = (float)get(0, c.LearningRate); c.Alpha = (float)get(1, c.Alpha); c.Epsilon = (float)get(2, c.Epsilon);
        c.WeightDecay = (float)get(3, c.WeightDecay); c.Momentum = (float)get(4, c.Momentum); c.Centered = get(5, c.Centered) != 0;
        h->opt = optimizer::NewRMSPropOptimizer(c, shapes, M, device, &err);
    } else if (t == "AdaGrad") {
        optimizer::AdaGradConfig c; c.LearningRate = (float)get(0, c.LearningRate); c.Epsilon = (float)get(1, c.Epsilon); c.WeightDecay = (float)get(2, c.WeightDecay);
        h->opt = optimizer::NewAdaGradOptimizer(c, shapes, M, device, &err);
    } else if (t == "AdaDelta") {
        optimizer::AdaDeltaConfig c; c.Rho = (float)get(0, c.Rho); c.Epsilon = (float)get(1, c.Epsilon); c.WeightDecay = (float)get(2, c.WeightDecay);
        h->opt = optimizer::NewAdaDeltaOptimizer(c, shapes, M, device, &err);
    } else if (t == "Nadam") {
        optimizer::NadamConfig c; c.LearningRate = (float)get(0, c.LearningRate); c.Beta1 = (float)get(1, c.Beta1); c.Beta2 = (float)get(2, c.Beta2);
        c.Epsilon = (float)get(3, c.Epsilon); c.WeightDecay = (float)get(4, c.WeightDecay);
        h->opt = optimizer::NewNadamOptimizer(c, shapes, M, device, &err);
    } else if (t == "LBFGS") {
        optimizer::LBFGSConfig c; c.HistorySize = (int)get(0, c.HistorySize); c.LineSearchTol = (float)get(1, c.LineSearchTol);
        c.MaxLineSearch = (int)get(2, c.MaxLineSearch); c.C1 = (float)get(3, c.C1); c.C2 = (float)get(4, c.C2); c.InitialStep = (float)get(5, c.InitialStep);
        h->lbfgs = optimizer::NewLBFGSOptimizer(c, shapes, M, device, &err);
    } else if (t == "MixedAdam") {
        optimizer::MixedAdamConfig c; c.LearningRate = (float)get(0, c.LearningRate); c.Beta1 = (float)get(1, c.Beta1); c.Beta2 = (float)get(2, c.Beta2);
        c.Epsilon = (float)get(3, c.Epsilon); c.WeightDecay = (float)get(4, c.WeightDecay); c.InitialLossScale = (float)get(5, c.InitialLossScale);
        c.GrowthFactor = (float)get(6, c.GrowthFactor); c.BackoffFactor = (float)get(7, c.BackoffFactor);
        c.GrowthInterval = (int)get(8, c.GrowthInterval); c.MaxLossScale = (float)get(9, c.MaxLossScale);
        h->opt = optimizer::NewMixedAdamOptimizer(c, shapes, M, device, &err);
    } else {
        err = "unknown optimizer type: " + t;
    }
    if (!h->opt && !h->lbfgs) { g_err = err; return nullptr; }
    return h.release();
}

GMH_API void gmh_optimizer_destroy(void* h) { delete static_cast<OptHandle*>(h); }

GMH_API int gmh_optimizer_set_weight_buffers(void* h, const uintptr_t* w, int n) {
    auto* o = static_cast<OptHandle*>(h);
    std::vector<uintptr_t> v(w, w + n);
    return fail(o->opt ? o->opt->SetWeightBuffers(v) : o->lbfgs->SetWeightBuffers(v));
}
GMH_API int gmh_optimizer_step(void* h, const uintptr_t* g, int n, float loss) {
    auto* o = static_cast<OptHandle*>(h);
    std::vector<uintptr_t> v(g, g + n);
    return fail(o->opt ? o->opt->Step(v) : o->lbfgs->Step(v, loss));
}
GMH_API uint64_t gmh_optimizer_step_count(void* h) { auto* o = static_cast<OptHandle*>(h); return o->opt ? o->opt->GetStepCount() : o->lbfgs->GetStep(); }
GMH_API int gmh_optimizer_update_lr(void* h, float lr) { auto* o = static_cast<OptHandle*>(h); return fail(o->opt ? o->opt->UpdateLearningRate(lr) : o->lbfgs->UpdateLearningRate(lr)); }
GMH_API float gmh_optimizer_lr(void* h) { auto* o = static_cast<OptHandle*>(h); return o->opt ? o->opt->LearningRate() : 0.0f; }
GMH_API const char* gmh_optimizer_type(void* h) { auto* o = static_cast<OptHandle*>(h); return o->opt ? o->opt->TypeName() : "LBFGS"; }
GMH_API void gmh_optimizer_set_command_pool(void* h, uintptr_t pool) { auto* o = static_cast<OptHandle*>(h); if (o->opt) o->opt->SetCommandPool(pool); }
GMH_API void gmh_optimizer_cleanup(void* h) { auto* o = static_cast<OptHandle*>(h); if (o->opt) o->opt->Cleanup(); else o->lbfgs->Cleanup(); }
GMH_API double gmh_optimizer_stat(void* h, const char* key) {
    auto* o = static_cast<OptHandle*>(h);
    auto m = o->opt ? o->opt->GetStats() : o->lbfgs->GetStats();
    auto it = m.find(key);
    return it == m.end() ? -1.0 : it->second;
}
GMH_API void* gmh_optimizer_get_state(void* h) {
    auto* o = static_cast<OptHandle*>(h);
    if (!o->opt) { g_err = "L-BFGS has no GetState"; return nullptr; }
    auto* s = new OptimizerState();
    std::string e = o->opt->GetState(s);
    if (!e.empty()) { g_err = e; delete s; return nullptr; }
    return s;
}
GMH_API int gmh_optimizer_load_state(void* h, void* s) {
    auto* o = static_cast<OptHandle*>(h);
    if (!o->opt) return fail("L-BFGS has no LoadState");
    return fail(o->opt->LoadState(*static_cast<OptimizerState*>(s)));
}
// ---- mixed-precision Adam extras ----
static optimizer::MixedAdamOptimizerState* as_mixed(void* h) {
    auto* o = static_cast<OptHandle*>(h);
    return o && o->opt ? dynamic_cast<optimizer::MixedAdamOptimizerState*>(o->opt.get()) : nullptr;
}
GMH_API int gmh_mixed_init_master(void* h, int index, const float* data, int n) {
    auto* m = as_mixed(h);
    return m ? fail(m->InitMaster(index, data, n)) : fail("not a MixedAdam optimizer");
}
GMH_API int gmh_mixed_read_master(void* h, int index, float* out, int n) {
    auto* m = as_mixed(h);
    return m ? fail(m->ReadMaster(index, out, n)) : fail("not a MixedAdam optimizer");
}
// out: scale, growth, backoff, max_scale as floats, then interval, good_steps, adam_t, skipped, last_overflow as int32
GMH_API int gmh_mixed_loss_scale(void* h, void* out) {
    auto* m = as_mixed(h);
    return m ? fail(m->LossScale(static_cast<Backend::LossScaleC*>(out))) : fail("not a MixedAdam optimizer");
}

GMH_API int gmh_mixed_set_clip(void* h, float max_norm) {
    auto* m = as_mixed(h);
    return m ? fail(m->SetGradClip(max_norm)) : fail("not a MixedAdam optimizer");
}
GMH_API int gmh_mixed_last_clip(void* h, float* sum_sq, float* coef) {
    auto* m = as_mixed(h);
    return m ? fail(m->LastClip(sum_sq, coef)) : fail("not a MixedAdam optimizer");
}

GMH_API int gmh_lbfgs_history(void* h, int* count, int* index) {
    auto* o = static_cast<OptHandle*>(h);
    if (!o->lbfgs) return -1;
    *count = o->lbfgs->historyCount(); *index = o->lbfgs->historyIndex();
    return 0;
}
GMH_API int gmh_lbfgs_read_rho(void* h, float* out, int n) {
    auto* o = static_cast<OptHandle*>(h);
    if (!o->lbfgs) return -1;
    auto r = o->lbfgs->readRho();
    for (int i = 0; i < n && i < (int)r.size(); ++i) out[i] = r[i];
    return (int)r.size();
}

// ---- schedulers ----
// kind: 0 StepLR(a=stepSize,b=gamma) 1 ExponentialLR(b=gamma) 2 Cosine(a=tMax,b=etaMin) 3 Plateau(b=factor,a=patience,c=threshold,mode) 4 NoOp
GMH_API void* gmh_sched_create(int kind, int a, double b, double c, const char* mode) {
    std::unique_ptr<training::LRScheduler> s;
    switch (kind) {
        case 0: s = training::NewStepLRScheduler(a, b); break;
        case 1: s = training::NewExponentialLRScheduler(b); break;
        case 2: s = training::NewCosineAnnealingLRScheduler(a, b); break;
        case 3: s = training::NewReduceLROnPlateauScheduler(b, a, c, mode ? mode : ""); break;
        default: s = training::NewNoOpScheduler(); break;
    }
    return s.release();
}
GMH_API void gmh_sched_destroy(void* s) { delete static_cast<training::LRScheduler*>(s); }
GMH_API double gmh_sched_get_lr(void* s, int epoch, int step, double base) { return static_cast<training::LRScheduler*>(s)->GetLR(epoch, step, base); }
GMH_API double gmh_sched_step(void* s, double metric, double lr) { return static_cast<training::LRScheduler*>(s)->Step(metric, lr); }
GMH_API const char* gmh_sched_name(void* s) { g_str = static_cast<training::LRScheduler*>(s)->GetName(); return g_str.c_str(); }
GMH_API int gmh_apply_scheduler(void* s, void* opt, int epoch, int step, double base) {
    auto* o = static_cast<OptHandle*>(opt);
    if (!o->opt) return fail(o->lbfgs->UpdateLearningRate(0));
    return fail(training::applyScheduler(*static_cast<training::LRScheduler*>(s), *o->opt, epoch, step, base));
}

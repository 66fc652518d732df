// gm_host_mixed.cpp -- mixed-precision Adam behind the Optimizer interface.
//
// The reference has the configuration of a dynamic loss scale
// (training/model_trainer.go:79-87, :258-270; training/simple_trainer.go:308-313)
// and the documented policy (docs/tutorials/mixed-precision.md:617-629) but no
// optimizer type that applies it.  This one owns the fp32 master weights and the
// two Adam moments (from the MemoryManager, like adam.go:95-133), drives the
// device-side step of include/gometal_cuda.h, and carries the loss-scale fields
// in the checkpoint payload next to the usual Adam ones.
#include <stdarg.h>
#include <stdio.h>

#include "gm_host.hpp"

namespace gometal {
namespace optimizer {

namespace {

std::string fmt(const char* f, ...) __attribute__((format(printf, 1, 2)));
std::string fmt(const char* f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof(buf), f, ap);
    va_end(ap);
    return buf;
}

const char* backend_error() {
    Backend& b = backend();
    return b.last_error ? b.last_error() : "";
}

}  // namespace

std::unique_ptr<MixedAdamOptimizerState> NewMixedAdamOptimizer(const MixedAdamConfig& c, const Shapes& shapes,
                                                               memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!mm) { *err = "memory manager cannot be nil"; return nullptr; }
    if (!device) { *err = "device cannot be nil"; return nullptr; }
    if (shapes.empty()) { *err = "no weight shapes provided"; return nullptr; }
    if (!(c.InitialLossScale > 0)) { *err = fmt("initial loss scale must be positive, got %f", c.InitialLossScale); return nullptr; }
    if (!(c.GrowthFactor >= 1)) { *err = fmt("loss scale growth factor must be at least 1, got %f", c.GrowthFactor); return nullptr; }
    if (!(c.BackoffFactor > 0 && c.BackoffFactor < 1)) { *err = fmt("loss scale backoff factor must be in (0, 1), got %f", c.BackoffFactor); return nullptr; }
    if (c.GrowthInterval < 1) { *err = fmt("loss scale growth interval must be positive, got %d", c.GrowthInterval); return nullptr; }
    Backend& b = backend();
    if (!b.has_mixed()) { *err = "the loaded backend has no mixed-precision entries"; return nullptr; }

    std::unique_ptr<MixedAdamOptimizerState> o(new MixedAdamOptimizerState());
    o->config_ = c; o->mm_ = mm; o->device_ = device;
    const size_t n = shapes.size();
    o->numel_.resize(n);
    o->weights16_.assign(n, 0);
    o->master_.assign(n, 0); o->momentum_.assign(n, 0); o->variance_.assign(n, 0);
    const char* names[3] = {"master weight", "momentum", "variance"};
    std::vector<uintptr_t>* slots[3] = {&o->master_, &o->momentum_, &o->variance_};
    for (size_t i = 0; i < n; ++i) {
        o->numel_[i] = calculateTensorSize(shapes[i]);
        for (int k = 0; k < 3; ++k) {
            uintptr_t p = mm->AllocateBuffer(o->numel_[i] * 4);
            if (!p) { *err = fmt("failed to allocate %s buffer for weight %zu", names[k], i); o->Cleanup(); return nullptr; }
            (*slots[k])[i] = p;
            int rc = b.zero(device, p, o->numel_[i] * 4);
            if (rc != 0) { *err = fmt("failed to zero %s buffer for weight %zu: error code %d", names[k], i, rc); o->Cleanup(); return nullptr; }
        }
    }
    Backend::LossScaleC ls{};
    ls.scale = c.InitialLossScale; ls.growth = c.GrowthFactor; ls.backoff = c.BackoffFactor; ls.max_scale = c.MaxLossScale;
    ls.interval = c.GrowthInterval;
    o->mixed_ = b.mixed_create(device, &ls, c.Beta1, c.Beta2, 0);
    if (!o->mixed_) { *err = fmt("failed to create the loss-scale state: %s", backend_error()); o->Cleanup(); return nullptr; }
    return o;
}

MixedAdamOptimizerState::~MixedAdamOptimizerState() { Cleanup(); }

void MixedAdamOptimizerState::Cleanup() {
    Backend& b = backend();
    if (list_ && b.list_destroy) { b.device_synchronize(device_); b.list_destroy(list_); }
    list_ = 0;
    if (mixed_ && b.mixed_destroy) b.mixed_destroy(mixed_);
    mixed_ = 0;
    if (!mm_) return;
    for (auto* v : {&master_, &momentum_, &variance_}) {
        for (auto& p : *v) { if (p) mm_->ReleaseBuffer(p); p = 0; }
    }
}

std::string MixedAdamOptimizerState::SetWeightBuffers(const std::vector<uintptr_t>& w) {
    if (w.size() != weights16_.size()) return fmt("expected %zu weight buffers, got %zu", weights16_.size(), w.size());
    weights16_ = w;
    return "";
}

// The device-resident descriptor is rebuilt only when a pointer changes.
std::string MixedAdamOptimizerState::ensureList(const std::vector<uintptr_t>& grads) {
    if (list_ && grads == listGrads_ && weights16_ == listWeights_) return "";
    Backend& b = backend();
    for (size_t i = 0; i < weights16_.size(); ++i) {
        if (!weights16_[i]) return fmt("weight buffer %zu is nil", i);
        if (!grads[i]) return fmt("gradient buffer %zu is nil", i);
    }
    if (list_) { b.device_synchronize(device_); b.list_destroy(list_); list_ = 0; }
    const uintptr_t* streams[5] = {grads.data(), master_.data(), momentum_.data(), variance_.data(), weights16_.data()};
    const int elem_bytes[5] = {2, 4, 4, 4, 2};
    std::vector<int64_t> n64(numel_.begin(), numel_.end());
    list_ = b.list_create(device_, 5, (int)numel_.size(), streams, n64.data(), elem_bytes);
    if (!list_) return fmt("failed to build the tensor list: %s", backend_error());
    listGrads_ = grads;
    listWeights_ = weights16_;
    return "";
}

std::string MixedAdamOptimizerState::Step(const std::vector<uintptr_t>& grads) {
    if (grads.size() != weights16_.size())
        return fmt("gradient buffers length (%zu) doesn't match weight buffers length (%zu)", grads.size(), weights16_.size());
    std::string e = ensureList(grads);
    if (!e.empty()) return e;
    stepCount_++;
    int rc = backend().mixed_step(device_, mixed_, list_, config_.LearningRate, config_.Epsilon, config_.WeightDecay);
    if (rc != 0) return fmt("MixedAdam step execution failed: MixedAdam step failed with error code: %d (%s)", rc, backend_error());
    return "";
}

std::string MixedAdamOptimizerState::SetGradClip(float maxNorm) {
    if (!backend().mixed_set_clip) return "the backend has no gradient clipping";
    int rc = backend().mixed_set_clip(mixed_, maxNorm);
    if (rc != 0) return fmt("failed to set the clipping norm: error code %d (%s)", rc, backend_error());
    return "";
}

std::string MixedAdamOptimizerState::LastClip(float* sumSq, float* coef) {
    if (!backend().mixed_last_clip) return "the backend has no gradient clipping";
    int rc = backend().mixed_last_clip(device_, mixed_, sumSq, coef);
    if (rc != 0) return fmt("failed to read the clipping result: error code %d (%s)", rc, backend_error());
    return "";
}

std::string MixedAdamOptimizerState::LossScale(Backend::LossScaleC* out) {
    int rc = backend().mixed_get_state(device_, mixed_, out);
    if (rc != 0) return fmt("failed to read the loss-scale state: error code %d (%s)", rc, backend_error());
    return "";
}

std::string MixedAdamOptimizerState::InitMaster(int index, const float* data, int numel) {
    if (index < 0 || index >= (int)master_.size()) return fmt("weight index %d out of range", index);
    if (numel != numel_[index]) return fmt("data size mismatch for master_%d: expected %d elements, got %d", index, numel_[index], numel);
    int rc = backend().copy_in(master_[index], const_cast<float*>(data), numel);
    if (rc != 0) return fmt("failed to write master buffer %d: error code %d", index, rc);
    return "";
}

std::string MixedAdamOptimizerState::ReadMaster(int index, float* out, int numel) {
    if (index < 0 || index >= (int)master_.size()) return fmt("weight index %d out of range", index);
    if (numel != numel_[index]) return fmt("data size mismatch for master_%d: expected %d elements, got %d", index, numel_[index], numel);
    Backend& b = backend();
    b.device_synchronize(device_);
    int rc = b.copy_out(master_[index], out, numel);
    if (rc != 0) return fmt("failed to read master buffer %d: error code %d", index, rc);
    return "";
}

std::string MixedAdamOptimizerState::GetState(OptimizerState* out) {
    Backend& b = backend();
    Backend::LossScaleC ls{};
    std::string e = LossScale(&ls);                      // waits for the stream: the tensors below are final
    if (!e.empty()) return e;
    out->Type = "MixedAdam";
    out->Parameters.clear();
    out->StateData.clear();
    auto putf = [&](const char* k, float v) { Param p; p.kind = Param::Float32; p.f = v; out->Parameters[k] = p; };
    auto putu = [&](const char* k, uint64_t v) { Param p; p.kind = Param::Uint64; p.u = v; out->Parameters[k] = p; };
    putf("learning_rate", config_.LearningRate); putf("beta1", config_.Beta1); putf("beta2", config_.Beta2);
    putf("epsilon", config_.Epsilon); putf("weight_decay", config_.WeightDecay);
    putu("step_count", stepCount_);
    putu("adam_step", (uint64_t)ls.adam_t);              // updates applied: skipped steps do not advance the bias correction
    putf("loss_scale", ls.scale); putf("growth_factor", ls.growth); putf("backoff_factor", ls.backoff);
    putf("max_loss_scale", ls.max_scale);
    putu("growth_interval", (uint64_t)ls.interval); putu("good_steps", (uint64_t)ls.good_steps);
    putu("skipped_steps", (uint64_t)ls.skipped);
    const char* names[3] = {"master", "momentum", "variance"};
    const std::vector<uintptr_t>* slots[3] = {&master_, &momentum_, &variance_};
    for (int k = 0; k < 3; ++k) {
        for (size_t i = 0; i < slots[k]->size(); ++i) {
            OptimizerTensor t;
            t.Name = std::string(names[k]) + "_" + std::to_string(i);
            t.StateType = names[k];
            t.Shape = {numel_[i]};
            t.Data.resize(numel_[i]);
            int rc = b.copy_out((*slots[k])[i], t.Data.data(), numel_[i]);
            if (rc != 0) return fmt("failed to read %s buffer %zu: error code %d", names[k], i, rc);
            out->StateData.push_back(std::move(t));
        }
    }
    return "";
}

std::string MixedAdamOptimizerState::LoadState(const OptimizerState& st) {
    std::string e = validateStateType("MixedAdam", st);
    if (!e.empty()) return e;
    Backend& b = backend();
    const auto& P = st.Parameters;
    // numbers arrive as float64 after a JSON round trip and as their own kinds straight from GetState
    auto num = [&](const char* key, double def) -> double {
        auto it = P.find(key);
        if (it == P.end()) return def;
        switch (it->second.kind) {
            case Param::Float64: case Param::Float32: return it->second.f;
            case Param::Uint64: return (double)it->second.u;
            default: return def;
        }
    };
    Backend::LossScaleC ls{};
    e = LossScale(&ls);
    if (!e.empty()) return e;
    config_.LearningRate = (float)num("learning_rate", config_.LearningRate);
    config_.Epsilon = (float)num("epsilon", config_.Epsilon);
    config_.WeightDecay = (float)num("weight_decay", config_.WeightDecay);
    const float b1 = (float)num("beta1", config_.Beta1), b2 = (float)num("beta2", config_.Beta2);
    if (b1 != config_.Beta1 || b2 != config_.Beta2)
        return fmt("beta1/beta2 of the saved state (%g, %g) differ from this optimizer's (%g, %g)", b1, b2, config_.Beta1, config_.Beta2);
    ls.scale = (float)num("loss_scale", ls.scale);
    ls.growth = (float)num("growth_factor", ls.growth);
    ls.backoff = (float)num("backoff_factor", ls.backoff);
    ls.max_scale = (float)num("max_loss_scale", ls.max_scale);
    ls.interval = (int32_t)num("growth_interval", ls.interval);
    ls.good_steps = (int32_t)num("good_steps", ls.good_steps);
    ls.skipped = (int32_t)num("skipped_steps", ls.skipped);
    ls.adam_t = (int32_t)num("adam_step", ls.adam_t);
    ls.last_overflow = 0;
    stepCount_ = (uint64_t)num("step_count", (double)stepCount_);
    for (const auto& t : st.StateData) {
        const int idx = extractBufferIndex(t.Name);
        if (idx < 0 || idx >= (int)master_.size()) return fmt("invalid buffer index in tensor name: %s", t.Name.c_str());
        if ((int)t.Data.size() != numel_[idx])
            return fmt("data size mismatch for %s: expected %d elements, got %zu", t.Name.c_str(), numel_[idx], t.Data.size());
        uintptr_t dst = 0;
        if (t.StateType == "master") dst = master_[idx];
        else if (t.StateType == "momentum") dst = momentum_[idx];
        else if (t.StateType == "variance") dst = variance_[idx];
        else return fmt("unknown state type: %s", t.StateType.c_str());
        int rc = b.copy_in(dst, const_cast<float*>(t.Data.data()), numel_[idx]);
        if (rc != 0) return fmt("failed to restore %s buffer %d: error code %d", t.StateType.c_str(), idx, rc);
    }
    int rc = b.mixed_set_state(device_, mixed_, &ls);
    if (rc != 0) return fmt("failed to restore the loss-scale state: error code %d (%s)", rc, backend_error());
    return "";
}

std::map<std::string, double> MixedAdamOptimizerState::GetStats() const {
    std::map<std::string, double> m;
    long total = 0;
    for (int n : numel_) total += 3L * n * 4;
    m["StepCount"] = (double)stepCount_;
    m["LearningRate"] = config_.LearningRate;
    m["NumWeights"] = (double)numel_.size();
    m["TotalBufferSize"] = (double)total;          // master + momentum + variance
    return m;
}

}  // namespace optimizer
}  // namespace gometal

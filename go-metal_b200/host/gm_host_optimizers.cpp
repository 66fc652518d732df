// gm_host_optimizers.cpp -- the six elementwise optimizer state types behind
// the Optimizer interface (optimizer/{sgd,adam,rmsprop,adagrad,adadelta,nadam}.go).
//
// The Go types differ only in their hyper-parameters, in which state buffers
// they own and in which bridge entry Step calls, so one class carries all six;
// the exported constructors keep the reference's names, defaults, validation
// order and messages.
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

enum class Kind { SGD, Adam, RMSProp, AdaGrad, AdaDelta, Nadam };

struct StateSlot {
    std::string name;        // "momentum", "variance", "squared_grad_avg", ...
    std::vector<uintptr_t> buffers;
};

class ElementwiseOptimizer : public Optimizer {
public:
    Kind kind;
    std::string type;
    float lr = 0, beta1 = 0, beta2 = 0, eps = 0, wd = 0, momentum = 0;
    bool nesterov = false, centered = false;
    uint64_t stepCount = 0;
    memory::MemoryManager* mm = nullptr;
    uintptr_t device = 0;
    uintptr_t commandPool = 0;
    bool usePooling = false;
    std::vector<int> bufferSizes;
    std::vector<uintptr_t> weights;
    std::vector<StateSlot> slots;

    ~ElementwiseOptimizer() override { Cleanup(); }
    const char* TypeName() const override { return type.c_str(); }
    float LearningRate() const override { return lr; }
    uint64_t GetStepCount() const override { return stepCount; }
    void SetCommandPool(uintptr_t pool) override { commandPool = pool; usePooling = pool != 0; }

    // adadelta.go:222-225: AdaDelta has no learning rate; the call is accepted and ignored
    std::string UpdateLearningRate(float newLR) override {
        if (kind != Kind::AdaDelta) lr = newLR;
        return "";
    }

    std::string SetWeightBuffers(const std::vector<uintptr_t>& w) override {
        if (w.size() != weights.size()) return fmt("expected %zu weight buffers, got %zu", weights.size(), w.size());
        weights = w;
        return "";
    }

    StateSlot* slot(const std::string& name) {
        for (auto& s : slots) if (s.name == name) return &s;
        return nullptr;
    }

    std::string Step(const std::vector<uintptr_t>& grads) override {
        if (grads.size() != weights.size())
            return fmt("gradient buffers length (%zu) doesn't match weight buffers length (%zu)", grads.size(), weights.size());
        Backend& b = backend();
        stepCount++;                                   // adam.go:183: incremented before the bridge call
        const int n = (int)weights.size();
        std::vector<uintptr_t> w = weights, g = grads;
        std::vector<int> sizes = bufferSizes;
        auto arr = [&](const char* name) -> uintptr_t* { StateSlot* s = slot(name); return s ? s->buffers.data() : nullptr; };
        int rc = 0;
        const int t = (int)stepCount;
        switch (kind) {
            case Kind::SGD:
                rc = b.sgd(device, w.data(), g.data(), arr("momentum"), n, sizes.data(), lr, momentum, wd, nesterov ? 1 : 0, t);
                break;
            case Kind::Adam:
                rc = usePooling
                    ? b.adam_pooled(device, w.data(), g.data(), arr("momentum"), arr("variance"), n, sizes.data(), lr, beta1, beta2, eps, wd, t, commandPool)
                    : b.adam(device, w.data(), g.data(), arr("momentum"), arr("variance"), n, sizes.data(), lr, beta1, beta2, eps, wd, t);
                break;
            case Kind::RMSProp:
                rc = b.rmsprop(device, w.data(), g.data(), arr("squared_grad_avg"), arr("momentum"), arr("gradient_avg"), n,
                               sizes.data(), lr, beta1, eps, wd, momentum, centered, t);
                break;
            case Kind::AdaGrad:
                rc = b.adagrad(device, w.data(), g.data(), arr("squared_grad_avg"), n, sizes.data(), lr, eps, wd);
                break;
            case Kind::AdaDelta:
                rc = b.adadelta(device, w.data(), g.data(), arr("squared_grad_avg"), arr("squared_update_avg"), n, sizes.data(), beta1, eps, wd);
                break;
            case Kind::Nadam:
                rc = b.nadam(device, w.data(), g.data(), arr("momentum"), arr("variance"), n, sizes.data(), lr, beta1, beta2, eps, wd, t);
                break;
        }
        if (rc != 0) {
            // bridge.go:1029-1031 wraps the code, adam.go:229-231 wraps again
            return fmt("%s step execution failed: %s step failed with error code: %d (%s)", type.c_str(), type.c_str(), rc,
                       b.last_error ? b.last_error() : "");
        }
        return "";
    }

    std::string GetState(OptimizerState* out) override {
        Backend& b = backend();
        out->Type = type;
        out->Parameters.clear();
        out->StateData.clear();
        auto putf = [&](const char* k, float v) { Param p; p.kind = Param::Float32; p.f = v; out->Parameters[k] = p; };
        switch (kind) {
            case Kind::SGD: putf("learning_rate", lr); putf("momentum", momentum); putf("weight_decay", wd);
                { Param p; p.kind = Param::Bool; p.b = nesterov; out->Parameters["nesterov"] = p; } break;
            case Kind::Adam: case Kind::Nadam:
                putf("learning_rate", lr); putf("beta1", beta1); putf("beta2", beta2); putf("epsilon", eps); putf("weight_decay", wd); break;
            case Kind::RMSProp: putf("learning_rate", lr); putf("alpha", beta1); putf("epsilon", eps); putf("weight_decay", wd);
                putf("momentum", momentum); { Param p; p.kind = Param::Bool; p.b = centered; out->Parameters["centered"] = p; } break;
            case Kind::AdaGrad: putf("learning_rate", lr); putf("epsilon", eps); putf("weight_decay", wd); break;
            case Kind::AdaDelta: putf("rho", beta1); putf("epsilon", eps); putf("weight_decay", wd); break;
        }
        { Param p; p.kind = Param::Uint64; p.u = stepCount; out->Parameters["step_count"] = p; }
        // adam.go:344-369: every momentum tensor, then every variance tensor
        for (auto& s : slots) {
            for (size_t i = 0; i < s.buffers.size(); ++i) {
                if (!s.buffers[i]) continue;
                OptimizerTensor t;
                t.Name = s.name + "_" + std::to_string(i);
                t.StateType = s.name;
                const int numel = bufferSizes[i] / 4;
                t.Data.resize(numel);
                int rc = b.copy_out(s.buffers[i], t.Data.data(), numel);
                if (rc != 0) return fmt("failed to read %s buffer %zu: error code %d", s.name.c_str(), i, rc);
                t.Shape = {numel};
                out->StateData.push_back(std::move(t));
            }
        }
        return "";
    }

    std::string LoadState(const OptimizerState& st) override {
        std::string e = validateStateType(type, st);
        if (!e.empty()) return e;
        Backend& b = backend();
        const auto& P = st.Parameters;
        switch (kind) {
            case Kind::SGD: lr = extractFloat32Param(P, "learning_rate", lr); momentum = extractFloat32Param(P, "momentum", momentum);
                wd = extractFloat32Param(P, "weight_decay", wd); nesterov = extractBoolParam(P, "nesterov", nesterov); break;
            case Kind::Adam: case Kind::Nadam:
                lr = extractFloat32Param(P, "learning_rate", lr); beta1 = extractFloat32Param(P, "beta1", beta1);
                beta2 = extractFloat32Param(P, "beta2", beta2); eps = extractFloat32Param(P, "epsilon", eps);
                wd = extractFloat32Param(P, "weight_decay", wd); break;
            case Kind::RMSProp: lr = extractFloat32Param(P, "learning_rate", lr); beta1 = extractFloat32Param(P, "alpha", beta1);
                eps = extractFloat32Param(P, "epsilon", eps); wd = extractFloat32Param(P, "weight_decay", wd);
                momentum = extractFloat32Param(P, "momentum", momentum); centered = extractBoolParam(P, "centered", centered); break;
            case Kind::AdaGrad: lr = extractFloat32Param(P, "learning_rate", lr); eps = extractFloat32Param(P, "epsilon", eps);
                wd = extractFloat32Param(P, "weight_decay", wd); break;
            case Kind::AdaDelta: beta1 = extractFloat32Param(P, "rho", beta1); eps = extractFloat32Param(P, "epsilon", eps);
                wd = extractFloat32Param(P, "weight_decay", wd); break;
        }
        // The reference's Adam/RMSProp/SGD read step_count only as float64 (adam.go:412-414)
        // while GetState stores a uint64; both kinds are accepted here, as nadam.go:361-365 does.
        auto it = P.find("step_count");
        if (it != P.end()) {
            if (it->second.kind == Param::Float64) stepCount = (uint64_t)it->second.f;
            else if (it->second.kind == Param::Uint64) stepCount = it->second.u;
        }
        for (const auto& t : st.StateData) {
            const int idx = extractBufferIndex(t.Name);
            if (idx < 0 || idx >= (int)weights.size()) return fmt("invalid buffer index in tensor name: %s", t.Name.c_str());
            const int expected = bufferSizes[idx] / 4;
            if ((int)t.Data.size() != expected)
                return fmt("data size mismatch for %s: expected %d elements, got %zu", t.Name.c_str(), expected, t.Data.size());
            StateSlot* s = slot(t.StateType);
            if (!s) return fmt("unknown state type: %s", t.StateType.c_str());
            if (!s->buffers[idx]) return fmt("%s buffer %d is nil", t.StateType.c_str(), idx);
            int rc = b.copy_in(s->buffers[idx], const_cast<float*>(t.Data.data()), expected);
            if (rc != 0) return fmt("failed to restore %s buffer %d: error code %d", t.StateType.c_str(), idx, rc);
        }
        return "";
    }

    void Cleanup() override {
        if (!mm) return;
        for (auto& s : slots) {
            for (auto& p : s.buffers) { if (p) mm->ReleaseBuffer(p); p = 0; }
        }
        slots.clear();
    }

    std::map<std::string, double> GetStats() const override {
        std::map<std::string, double> m;
        long total = 0;
        for (const auto& s : slots) for (size_t i = 0; i < s.buffers.size(); ++i) if (s.buffers[i]) total += bufferSizes[i];
        m["StepCount"] = (double)stepCount;
        m["LearningRate"] = lr;
        m["NumWeights"] = (double)weights.size();
        m["TotalBufferSize"] = (double)total;         // adam_test.go:248-251: state slots x sum of sizes
        return m;
    }
};

// Shared tail of every constructor: nil checks, shapes, buffer allocation and zeroing.
std::unique_ptr<Optimizer> finish(std::unique_ptr<ElementwiseOptimizer> o, const Shapes& shapes, memory::MemoryManager* mm,
                                  uintptr_t device, const std::vector<std::pair<std::string, std::string>>& stateNames,
                                  std::string* err) {
    Backend& b = backend();
    o->mm = mm; o->device = device;
    const size_t n = shapes.size();
    o->weights.assign(n, 0);
    o->bufferSizes.resize(n);
    for (size_t i = 0; i < n; ++i) o->bufferSizes[i] = calculateTensorSize(shapes[i]) * 4;
    for (const auto& sn : stateNames) {
        StateSlot s; s.name = sn.first; s.buffers.assign(n, 0);
        o->slots.push_back(std::move(s));
    }
    for (size_t i = 0; i < n; ++i) {
        for (size_t k = 0; k < o->slots.size(); ++k) {
            uintptr_t p = mm->AllocateBuffer(o->bufferSizes[i]);
            if (!p) { *err = fmt("failed to allocate %s buffer for weight %zu", stateNames[k].second.c_str(), i); o->Cleanup(); return nullptr; }
            o->slots[k].buffers[i] = p;
            int rc = b.zero(device, p, o->bufferSizes[i]);
            if (rc != 0) { *err = fmt("failed to zero %s buffer for weight %zu: error code %d", stateNames[k].second.c_str(), i, rc); o->Cleanup(); return nullptr; }
        }
    }
    return std::unique_ptr<Optimizer>(o.release());
}

bool common_checks(const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!mm) { *err = "memory manager cannot be nil"; return false; }
    if (!device) { *err = "device cannot be nil"; return false; }
    if (shapes.empty()) { *err = "no weight shapes provided"; return false; }
    return true;
}

}  // namespace

std::unique_ptr<Optimizer> NewSGDOptimizer(const SGDConfig& c, const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!common_checks(shapes, mm, device, err)) return nullptr;
    if (c.LearningRate < 0) { *err = fmt("learning rate cannot be negative: %f", c.LearningRate); return nullptr; }   // sgd.go:77-88
    if (c.Momentum < 0) { *err = fmt("momentum cannot be negative: %f", c.Momentum); return nullptr; }
    if (c.Momentum > 1.0f) { *err = fmt("momentum cannot be greater than 1.0: %f", c.Momentum); return nullptr; }
    if (c.WeightDecay < 0) { *err = fmt("weight decay cannot be negative: %f", c.WeightDecay); return nullptr; }
    std::unique_ptr<ElementwiseOptimizer> o(new ElementwiseOptimizer());
    o->kind = Kind::SGD; o->type = "SGD";
    o->lr = c.LearningRate; o->momentum = c.Momentum; o->wd = c.WeightDecay; o->nesterov = c.Nesterov;
    std::vector<std::pair<std::string, std::string>> st;
    if (c.Momentum > 0) st.push_back({"momentum", "momentum"});          // sgd.go:105-133: no buffers when momentum == 0
    return finish(std::move(o), shapes, mm, device, st, err);
}

std::unique_ptr<Optimizer> NewAdamOptimizer(const AdamConfig& c, const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!common_checks(shapes, mm, device, err)) return nullptr;
    std::unique_ptr<ElementwiseOptimizer> o(new ElementwiseOptimizer());
    o->kind = Kind::Adam; o->type = "Adam";
    o->lr = c.LearningRate; o->beta1 = c.Beta1; o->beta2 = c.Beta2; o->eps = c.Epsilon; o->wd = c.WeightDecay;
    return finish(std::move(o), shapes, mm, device, {{"momentum", "momentum"}, {"variance", "variance"}}, err);
}

std::unique_ptr<Optimizer> NewRMSPropOptimizer(const RMSPropConfig& c, const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!common_checks(shapes, mm, device, err)) return nullptr;
    std::unique_ptr<ElementwiseOptimizer> o(new ElementwiseOptimizer());
    o->kind = Kind::RMSProp; o->type = "RMSProp";
    o->lr = c.LearningRate; o->beta1 = c.Alpha; o->eps = c.Epsilon; o->wd = c.WeightDecay; o->momentum = c.Momentum; o->centered = c.Centered;
    std::vector<std::pair<std::string, std::string>> st = {{"squared_grad_avg", "squared gradient average"}};
    if (c.Momentum > 0) st.push_back({"momentum", "momentum"});           // rmsprop.go:117-146
    if (c.Centered) st.push_back({"gradient_avg", "gradient average"});
    return finish(std::move(o), shapes, mm, device, st, err);
}

std::unique_ptr<Optimizer> NewAdaGradOptimizer(const AdaGradConfig& c, const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!common_checks(shapes, mm, device, err)) return nullptr;
    std::unique_ptr<ElementwiseOptimizer> o(new ElementwiseOptimizer());
    o->kind = Kind::AdaGrad; o->type = "AdaGrad";
    o->lr = c.LearningRate; o->eps = c.Epsilon; o->wd = c.WeightDecay;
    return finish(std::move(o), shapes, mm, device, {{"squared_grad_avg", "squared gradient average"}}, err);
}

std::unique_ptr<Optimizer> NewAdaDeltaOptimizer(const AdaDeltaConfig& c, const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!common_checks(shapes, mm, device, err)) return nullptr;
    if (c.Rho <= 0 || c.Rho >= 1) { *err = fmt("rho must be in range (0, 1), got %f", c.Rho); return nullptr; }      // adadelta.go:70-72
    std::unique_ptr<ElementwiseOptimizer> o(new ElementwiseOptimizer());
    o->kind = Kind::AdaDelta; o->type = "AdaDelta";
    o->beta1 = c.Rho; o->eps = c.Epsilon; o->wd = c.WeightDecay;
    return finish(std::move(o), shapes, mm, device,
                  {{"squared_grad_avg", "squared gradient average"}, {"squared_update_avg", "squared update average"}}, err);
}

std::unique_ptr<Optimizer> NewNadamOptimizer(const NadamConfig& c, const Shapes& shapes, memory::MemoryManager* mm, uintptr_t device, std::string* err) {
    if (!common_checks(shapes, mm, device, err)) return nullptr;
    if (c.LearningRate <= 0) { *err = fmt("learning rate must be positive, got %f", c.LearningRate); return nullptr; }     // nadam.go:77-91
    if (c.Beta1 < 0 || c.Beta1 >= 1) { *err = fmt("beta1 must be in [0, 1), got %f", c.Beta1); return nullptr; }
    if (c.Beta2 < 0 || c.Beta2 >= 1) { *err = fmt("beta2 must be in [0, 1), got %f", c.Beta2); return nullptr; }
    if (c.Epsilon <= 0) { *err = fmt("epsilon must be positive, got %e", c.Epsilon); return nullptr; }
    if (c.WeightDecay < 0) { *err = fmt("weight decay must be non-negative, got %f", c.WeightDecay); return nullptr; }
    std::unique_ptr<ElementwiseOptimizer> o(new ElementwiseOptimizer());
    o->kind = Kind::Nadam; o->type = "Nadam";
    o->lr = c.LearningRate; o->beta1 = c.Beta1; o->beta2 = c.Beta2; o->eps = c.Epsilon; o->wd = c.WeightDecay;
    return finish(std::move(o), shapes, mm, device, {{"momentum", "momentum"}, {"variance", "variance"}}, err);
}

}  // namespace optimizer
}  // namespace gometal

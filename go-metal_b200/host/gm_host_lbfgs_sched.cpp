// gm_host_lbfgs_sched.cpp -- the L-BFGS optimizer state (optimizer/lbfgs.go) and
// the learning-rate schedulers (training/scheduler.go), host side only.
#include <stdarg.h>
#include <stdio.h>

#include <cmath>

#include "gm_host.hpp"

namespace gometal {
namespace optimizer {

static std::string lfmt(const char* f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof(buf), f, ap);
    va_end(ap);
    return buf;
}

// lbfgs.go:67-190: (2m+2) buffers per weight, m one-float rho buffers, one alpha buffer of m floats
std::unique_ptr<LBFGSOptimizerState> NewLBFGSOptimizer(const LBFGSConfig& c, const Shapes& shapes, memory::MemoryManager* mm,
                                                       uintptr_t device, std::string* err) {
    if (!mm) { *err = "memory manager cannot be nil"; return nullptr; }
    if (!device) { *err = "device cannot be nil"; return nullptr; }
    if (shapes.empty()) { *err = "no weight shapes provided"; return nullptr; }
    if (c.HistorySize <= 0) { *err = lfmt("history size must be positive, got %d", c.HistorySize); return nullptr; }
    Backend& b = backend();
    std::unique_ptr<LBFGSOptimizerState> o(new LBFGSOptimizerState());
    o->config_ = c; o->mm_ = mm; o->device_ = device;
    const size_t n = shapes.size();
    const int m = c.HistorySize;
    o->weights_.assign(n, 0);
    o->bufferSizes_.resize(n);
    for (size_t i = 0; i < n; ++i) o->bufferSizes_[i] = calculateTensorSize(shapes[i]) * 4;
    auto take = [&](int bytes, const std::string& what) -> uintptr_t {
        uintptr_t p = mm->AllocateBuffer(bytes);
        if (!p) { *err = "failed to allocate " + what; return 0; }
        if (b.zero(device, p, bytes) != 0) { *err = "failed to zero " + what; mm->ReleaseBuffer(p); return 0; }
        return p;
    };
    o->s_.assign(m, std::vector<uintptr_t>(n, 0));
    o->y_.assign(m, std::vector<uintptr_t>(n, 0));
    for (int h = 0; h < m; ++h) {
        for (size_t i = 0; i < n; ++i) {
            if (!(o->s_[h][i] = take(o->bufferSizes_[i], lfmt("s vector buffer for history %d, weight %zu", h, i)))) { o->Cleanup(); return nullptr; }
            if (!(o->y_[h][i] = take(o->bufferSizes_[i], lfmt("y vector buffer for history %d, weight %zu", h, i)))) { o->Cleanup(); return nullptr; }
        }
    }
    o->rho_.assign(m, 0);
    for (int h = 0; h < m; ++h)
        if (!(o->rho_[h] = take(4, lfmt("rho buffer for history %d", h)))) { o->Cleanup(); return nullptr; }
    if (!(o->alpha_ = take(4 * m, "alpha buffer"))) { o->Cleanup(); return nullptr; }
    o->oldGrad_.assign(n, 0);
    o->searchDir_.assign(n, 0);
    for (size_t i = 0; i < n; ++i) {
        if (!(o->oldGrad_[i] = take(o->bufferSizes_[i], lfmt("old gradient buffer for weight %zu", i)))) { o->Cleanup(); return nullptr; }
        if (!(o->searchDir_[i] = take(o->bufferSizes_[i], lfmt("search direction buffer for weight %zu", i)))) { o->Cleanup(); return nullptr; }
    }
    return o;
}

LBFGSOptimizerState::~LBFGSOptimizerState() { Cleanup(); }

void LBFGSOptimizerState::Cleanup() {
    if (!mm_) return;
    auto drop = [&](uintptr_t& p) { if (p) mm_->ReleaseBuffer(p); p = 0; };
    for (auto& v : s_) for (auto& p : v) drop(p);
    for (auto& v : y_) for (auto& p : v) drop(p);
    for (auto& p : rho_) drop(p);
    for (auto& p : oldGrad_) drop(p);
    for (auto& p : searchDir_) drop(p);
    drop(alpha_);
}

std::string LBFGSOptimizerState::SetWeightBuffers(const std::vector<uintptr_t>& w) {
    if (w.size() != weights_.size()) return lfmt("expected %zu weight buffers, got %zu", weights_.size(), w.size());
    weights_ = w;
    return "";
}

// lbfgs.go:245-301
std::string LBFGSOptimizerState::Step(const std::vector<uintptr_t>& grads, float currentLoss) {
    if (grads.size() != weights_.size())
        return lfmt("gradient buffers length (%zu) doesn't match weight buffers length (%zu)", grads.size(), weights_.size());
    Backend& b = backend();
    stepCount_++;
    const int n = (int)weights_.size();
    const int m = config_.HistorySize;
    std::vector<uintptr_t> sFlat((size_t)m * n), yFlat((size_t)m * n);     // bridge.go:1987-1998: [h*numWeights + w]
    for (int h = 0; h < m; ++h)
        for (int i = 0; i < n; ++i) { sFlat[(size_t)h * n + i] = s_[h][i]; yFlat[(size_t)h * n + i] = y_[h][i]; }
    std::vector<uintptr_t> w = weights_, g = grads;
    std::vector<int> sizes = bufferSizes_;
    float stepSize = 0.0f;
    int rc = b.lbfgs(device_, w.data(), g.data(), oldGrad_.data(), searchDir_.data(), sFlat.data(), yFlat.data(), rho_.data(),
                     alpha_, n, sizes.data(), m, historyCount_, historyIndex_, config_.InitialStep, config_.C1, config_.C2,
                     config_.MaxLineSearch, currentLoss, prevLoss_, &stepSize);
    if (rc != 0) return lfmt("L-BFGS step execution failed: L-BFGS step failed with error code: %d (%s)", rc, b.last_error ? b.last_error() : "");
    historyIndex_ = (historyIndex_ + 1) % m;                           // lbfgs.go:287-290
    if (historyCount_ < m) historyCount_++;
    prevLoss_ = currentLoss;
    return "";
}

std::string LBFGSOptimizerState::UpdateLearningRate(float) {
    return "L-BFGS does not use a fixed learning rate; it uses line search";     // lbfgs.go:330-332
}

std::map<std::string, double> LBFGSOptimizerState::GetStats() const {
    std::map<std::string, double> m;
    m["step_count"] = (double)stepCount_;
    m["history_count"] = historyCount_;
    m["history_index"] = historyIndex_;
    m["history_size"] = config_.HistorySize;
    m["prev_loss"] = prevLoss_;
    return m;
}

std::vector<float> LBFGSOptimizerState::readRho() {
    std::vector<float> out(rho_.size(), 0.0f);
    Backend& b = backend();
    for (size_t h = 0; h < rho_.size(); ++h) b.copy_out(rho_[h], &out[h], 1);
    return out;
}

}  // namespace optimizer

// ---------------------------------------------------------------------
// schedulers
// ---------------------------------------------------------------------
namespace training {

namespace {

struct StepLR : LRScheduler {
    int stepSize; double gamma;
    double GetLR(int epoch, int, double base) override { return base * std::pow(gamma, (double)(epoch / stepSize)); }
    std::string GetName() const override { return "StepLR"; }
};
struct ExponentialLR : LRScheduler {
    double gamma;
    double GetLR(int epoch, int, double base) override { return base * std::pow(gamma, (double)epoch); }
    std::string GetName() const override { return "ExponentialLR"; }
};
struct CosineLR : LRScheduler {
    int tMax; double etaMin;
    double GetLR(int epoch, int, double base) override {
        if (epoch >= tMax) return etaMin;
        return etaMin + (base - etaMin) * (1 + std::cos(M_PI * (double)epoch / (double)tMax)) / 2;
    }
    std::string GetName() const override { return "CosineAnnealingLR"; }
};
struct PlateauLR : LRScheduler {
    double factor; int patience; double threshold; std::string mode;
    double best = 0, current = 0; int bad = 0; bool initialized = false;
    double Step(double metric, double currentLR) override {
        if (!initialized) { best = metric; current = currentLR; initialized = true; return currentLR; }
        const bool improved = mode == "min" ? metric < best - threshold : metric > best + threshold;
        if (improved) { best = metric; bad = 0; }
        else if (++bad >= patience) { current *= factor; bad = 0; }
        return current;
    }
    double GetLR(int, int, double base) override { return initialized ? current : base; }
    std::string GetName() const override { return "ReduceLROnPlateau"; }
};
struct NoOp : LRScheduler {
    double GetLR(int, int, double base) override { return base; }
    std::string GetName() const override { return "ConstantLR"; }
};

}  // namespace

// Out-of-range arguments fall back to the reference's defaults (scheduler.go:27-36, 58-62, 84-93, 128-146).
std::unique_ptr<LRScheduler> NewStepLRScheduler(int stepSize, double gamma) {
    auto* s = new StepLR();
    s->stepSize = stepSize <= 0 ? 30 : stepSize;
    s->gamma = (gamma <= 0 || gamma >= 1) ? 0.1 : gamma;
    return std::unique_ptr<LRScheduler>(s);
}
std::unique_ptr<LRScheduler> NewExponentialLRScheduler(double gamma) {
    auto* s = new ExponentialLR();
    s->gamma = (gamma <= 0 || gamma >= 1) ? 0.95 : gamma;
    return std::unique_ptr<LRScheduler>(s);
}
std::unique_ptr<LRScheduler> NewCosineAnnealingLRScheduler(int tMax, double etaMin) {
    auto* s = new CosineLR();
    s->tMax = tMax <= 0 ? 100 : tMax;
    s->etaMin = etaMin < 0 ? 0 : etaMin;
    return std::unique_ptr<LRScheduler>(s);
}
std::unique_ptr<LRScheduler> NewReduceLROnPlateauScheduler(double factor, int patience, double threshold, const std::string& mode) {
    auto* s = new PlateauLR();
    s->factor = (factor <= 0 || factor >= 1) ? 0.1 : factor;
    s->patience = patience <= 0 ? 10 : patience;
    s->threshold = threshold < 0 ? 1e-4 : threshold;
    s->mode = (mode != "min" && mode != "max") ? "min" : mode;
    return std::unique_ptr<LRScheduler>(s);
}
std::unique_ptr<LRScheduler> NewNoOpScheduler() { return std::unique_ptr<LRScheduler>(new NoOp()); }

std::string applyScheduler(LRScheduler& s, optimizer::Optimizer& opt, int epoch, int step, double baseLR) {
    const double lr = s.GetLR(epoch, step, baseLR);
    return opt.UpdateLearningRate((float)lr);          // model_trainer.go:1490-1491: float64 -> float32
}

}  // namespace training
}  // namespace gometal

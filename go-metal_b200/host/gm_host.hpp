// gm_host.hpp -- C++ mirror of go-metal's host side of the optimizer step.
//
// The reference's host code is Go (optimizer/*.go, memory/manager.go,
// training/scheduler.go).  No Go toolchain exists where this repository is
// built, so the same types, method names, defaults, validation rules and error
// texts are restated here in C++ above the C ABI of include/gometal_cuda.h and
// tested from pytest through the small C handle API in gm_host_capi.cpp.  The
// Go sources that bind the same ABI live in go-metal_b200/go/.
//
// Every device operation goes through a Backend: a table of the drop-in C
// entries resolved from a shared library at run time (libgometal_cuda.so, or a
// recording fake in the CPU tests).  There is no arithmetic in this layer.
#pragma once

#include <stdint.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace gometal {

// ---------------------------------------------------------------------
// Backend: the C ABI, resolved with dlopen/dlsym
// ---------------------------------------------------------------------
struct Backend {
    void* handle = nullptr;
    uintptr_t (*create_device)() = nullptr;
    void (*destroy_device)(uintptr_t) = nullptr;
    uintptr_t (*allocate)(uintptr_t, int, int) = nullptr;
    void (*deallocate)(uintptr_t) = nullptr;
    int (*zero)(uintptr_t, uintptr_t, int) = nullptr;
    int (*copy_in)(uintptr_t, float*, int) = nullptr;
    int (*copy_out)(uintptr_t, float*, int) = nullptr;
    int (*sgd)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float, int, int) = nullptr;
    int (*adam)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float, float, float, int) = nullptr;
    int (*adam_pooled)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float, float, float, int, uintptr_t) = nullptr;
    int (*rmsprop)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float, float, float, bool, int) = nullptr;
    int (*adagrad)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float) = nullptr;
    int (*adadelta)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float) = nullptr;
    int (*nadam)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, int, int*, float, float, float, float, float, int) = nullptr;
    int (*lbfgs)(uintptr_t, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t*, uintptr_t,
                 int, int*, int, int, int, float, float, float, int, float, float, float*) = nullptr;
    const char* (*last_error)() = nullptr;

    // Mixed precision (include/gometal_cuda.h part 2).  Optional: a backend without
    // them still serves the seven reference optimizers.
    struct LossScaleC { float scale, growth, backoff, max_scale; int32_t interval, good_steps, adam_t, skipped, last_overflow; };
    uintptr_t (*mixed_create)(uintptr_t, const LossScaleC*, float, float, int) = nullptr;
    void (*mixed_destroy)(uintptr_t) = nullptr;
    int (*mixed_step)(uintptr_t, uintptr_t, uintptr_t, float, float, float) = nullptr;
    int (*mixed_get_state)(uintptr_t, uintptr_t, LossScaleC*) = nullptr;
    int (*mixed_set_state)(uintptr_t, uintptr_t, const LossScaleC*) = nullptr;
    int (*mixed_set_clip)(uintptr_t, float) = nullptr;
    int (*mixed_last_clip)(uintptr_t, uintptr_t, float*, float*) = nullptr;
    uintptr_t (*list_create)(uintptr_t, int, int, const uintptr_t* const*, const int64_t*, const int*) = nullptr;
    void (*list_destroy)(uintptr_t) = nullptr;
    int (*device_synchronize)(uintptr_t) = nullptr;
    // Flat arenas (optional as well)
    uintptr_t (*arena_create)(uintptr_t, int64_t) = nullptr;
    uintptr_t (*arena_alloc)(uintptr_t, int64_t) = nullptr;
    void (*arena_destroy)(uintptr_t) = nullptr;
    bool has_arena() const { return arena_create && arena_alloc && arena_destroy; }
    bool has_mixed() const {
        return mixed_create && mixed_destroy && mixed_step && mixed_get_state && mixed_set_state && list_create &&
               list_destroy && device_synchronize;
    }

    // Loads `path` and resolves every entry; returns an error text or "".
    std::string load(const std::string& path);
};

Backend& backend();                       // process-wide table

// ---------------------------------------------------------------------
// memory: mirrors memory/manager.go
// ---------------------------------------------------------------------
namespace memory {

// memory/manager.go:109-111
extern const std::vector<int> kDefaultPoolSizes;
int findPoolSize(int size);               // manager.go:172-180
int calculateMaxPoolSize(int bufferSize); // manager.go:210-224

struct PoolStats { int available = 0, allocated = 0, maxSize = 0; };

class MemoryManager {
public:
    explicit MemoryManager(uintptr_t device) : device_(device) {}
    ~MemoryManager();
    // manager.go:289-296: returns 0 when the tier is exhausted or the device allocation fails
    uintptr_t AllocateBuffer(int size);
    // manager.go:299-317: back to its tier, or freed when the tier's free list is full
    void ReleaseBuffer(uintptr_t buffer);
    std::map<int, PoolStats> Stats();
    uintptr_t device() const { return device_; }
    int trackedSize(uintptr_t buffer);    // -1 when unknown
    // Switches this manager to one flat, 256-byte-aligned arena of `bytes`: every later
    // buffer is carved from it (still rounded to its tier, still reused through the tier's
    // free list) and the per-tier caps of manager.go:210-224 no longer apply, only the
    // arena's size does.  The reference's caps cannot hold a large model (20 buffers of
    // 16 MB); this is the pool the large configurations use.  Call it before the first
    // allocation; returns "" or an error text.
    std::string UseArena(int64_t bytes);

private:
    struct Pool { int size = 0, maxSize = 0, allocated = 0; std::vector<uintptr_t> free; };
    std::mutex mu_;
    uintptr_t device_;
    std::map<int, Pool> pools_;
    std::map<uintptr_t, int> sizes_;
    uintptr_t arena_ = 0;
};

}  // namespace memory

// ---------------------------------------------------------------------
// checkpoints / optimizer state: checkpoints/checkpoint.go:74-86,
// optimizer/interface.go:47-51
// ---------------------------------------------------------------------
struct Param {
    enum Kind { Float64, Bool, Uint64, Float32 } kind = Float64;
    double f = 0;
    bool b = false;
    uint64_t u = 0;
};

struct OptimizerTensor {
    std::string Name;
    std::vector<int> Shape;
    std::vector<float> Data;
    std::string StateType;
};

struct OptimizerState {
    std::string Type;
    std::map<std::string, Param> Parameters;
    std::vector<OptimizerTensor> StateData;
};

namespace checkpoints {
// The optimizer part of a checkpoint as JSON text, field names of
// checkpoints/checkpoint.go:74-86.  Decode returns what a Go reader would pass to
// LoadState: every parameter number as Float64, tensors as float32 with the saved bits.
// Both return "" or an error text.
std::string EncodeOptimizerState(const OptimizerState& state, std::string* out);
std::string DecodeOptimizerState(const std::string& text, OptimizerState* out);
}  // namespace checkpoints

namespace optimizer {

// optimizer/interface.go:56-84, optimizer/state_helpers.go:52-74, adam.go (calculateTensorSize)
int extractBufferIndex(const std::string& name);
std::string validateStateType(const std::string& optimizerType, const OptimizerState& state);   // "" = ok
// adam.go:237-251: repeated multiplication, int(y) factors; 1 for y == 0, x for y == 1.
float pow(float x, float y);
float extractFloat32Param(const std::map<std::string, Param>& p, const std::string& key, float def);
bool extractBoolParam(const std::map<std::string, Param>& p, const std::string& key, bool def);
uint64_t extractUint64Param(const std::map<std::string, Param>& p, const std::string& key, uint64_t def);
int calculateTensorSize(const std::vector<int>& shape);

// optimizer/interface.go:13-43.  Errors are returned as text ("" = nil).
class Optimizer {
public:
    virtual ~Optimizer() {}
    virtual std::string Step(const std::vector<uintptr_t>& gradientBuffers) = 0;
    virtual std::string GetState(OptimizerState* out) = 0;
    virtual std::string LoadState(const OptimizerState& state) = 0;
    virtual uint64_t GetStepCount() const = 0;
    virtual std::string UpdateLearningRate(float lr) = 0;     // "" except where the reference refuses
    virtual std::string SetWeightBuffers(const std::vector<uintptr_t>& weightBuffers) = 0;
    virtual void SetCommandPool(uintptr_t commandPool) = 0;
    virtual void Cleanup() = 0;
    virtual std::map<std::string, double> GetStats() const = 0;
    virtual float LearningRate() const = 0;
    virtual const char* TypeName() const = 0;
};

// Configurations with the reference's defaults.
struct SGDConfig { float LearningRate = 0.01f, Momentum = 0.0f, WeightDecay = 0.0f; bool Nesterov = false; };            // sgd.go:48-55
struct AdamConfig { float LearningRate = 0.001f, Beta1 = 0.9f, Beta2 = 0.999f, Epsilon = 1e-8f, WeightDecay = 0.0f; };   // adam.go:51-59
struct RMSPropConfig { float LearningRate = 0.01f, Alpha = 0.99f, Epsilon = 1e-8f, WeightDecay = 0.0f, Momentum = 0.0f; bool Centered = false; };  // rmsprop.go:54-63
struct AdaGradConfig { float LearningRate = 0.01f, Epsilon = 1e-10f, WeightDecay = 0.0f; };                              // adagrad.go:42-48
struct AdaDeltaConfig { float Rho = 0.95f, Epsilon = 1e-6f, WeightDecay = 0.0f; };                                       // adadelta.go:43-49
struct NadamConfig { float LearningRate = 0.002f, Beta1 = 0.9f, Beta2 = 0.999f, Epsilon = 1e-8f, WeightDecay = 0.0f; };  // nadam.go:47-55
struct LBFGSConfig { int HistorySize = 10; float LineSearchTol = 1e-4f; int MaxLineSearch = 20; float C1 = 1e-4f, C2 = 0.9f, InitialStep = 1.0f; };  // lbfgs.go:55-64

using Shapes = std::vector<std::vector<int>>;

// Constructors: nullptr + *err on failure, with the reference's messages.
std::unique_ptr<Optimizer> NewSGDOptimizer(const SGDConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);
std::unique_ptr<Optimizer> NewAdamOptimizer(const AdamConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);
std::unique_ptr<Optimizer> NewRMSPropOptimizer(const RMSPropConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);
std::unique_ptr<Optimizer> NewAdaGradOptimizer(const AdaGradConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);
std::unique_ptr<Optimizer> NewAdaDeltaOptimizer(const AdaDeltaConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);
std::unique_ptr<Optimizer> NewNadamOptimizer(const NadamConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);

// Mixed-precision Adam: fp16 gradients and an fp16 parameter copy around fp32 master
// weights, with the dynamic loss scale of training/model_trainer.go:79-87 and
// :258-270 kept on the device.  No counterpart type exists in optimizer/*.go (the
// reference only carries the configuration fields); the interface is the same.
//   SetWeightBuffers: the fp16 parameter buffers the model reads (written every step)
//   Step:             one fp16 gradient buffer per weight; returns after the launch --
//                     overflow detection, the skipped update and the scale change happen
//                     on the device; GetState / LossScale wait for them
//   GetStepCount:     Step calls so far (a skipped step counts; "adam_step" in the state does not)
struct MixedAdamConfig {
    float LearningRate = 0.001f, Beta1 = 0.9f, Beta2 = 0.999f, Epsilon = 1e-8f, WeightDecay = 0.0f;   // adam.go:51-59
    float InitialLossScale = 65536.0f, GrowthFactor = 2.0f, BackoffFactor = 0.5f;                     // model_trainer.go:258-270
    int GrowthInterval = 2000;
    float MaxLossScale = 16777216.0f;
};
class MixedAdamOptimizerState : public Optimizer {
public:
    ~MixedAdamOptimizerState() override;
    std::string Step(const std::vector<uintptr_t>& gradientBuffers) override;
    std::string GetState(OptimizerState* out) override;
    std::string LoadState(const OptimizerState& state) override;
    uint64_t GetStepCount() const override { return stepCount_; }
    std::string UpdateLearningRate(float lr) override { config_.LearningRate = lr; return ""; }
    std::string SetWeightBuffers(const std::vector<uintptr_t>& weightBuffers) override;
    void SetCommandPool(uintptr_t) override {}
    void Cleanup() override;
    std::map<std::string, double> GetStats() const override;
    float LearningRate() const override { return config_.LearningRate; }
    const char* TypeName() const override { return "MixedAdam"; }
    // fp32 master weights of tensor `index` (a fresh run starts from these; a resumed one from LoadState)
    std::string InitMaster(int index, const float* data, int numel);
    std::string ReadMaster(int index, float* out, int numel);
    // waits for the stream; the device-resident loss-scale state
    std::string LossScale(Backend::LossScaleC* out);
    // global-norm gradient clipping: maxNorm > 0 turns it on, 0 off; LastClip waits for the stream and
    // returns the last step's sum of squared unscaled gradients and the coefficient applied
    std::string SetGradClip(float maxNorm);
    std::string LastClip(float* sumSq, float* coef);

private:
    friend std::unique_ptr<MixedAdamOptimizerState> NewMixedAdamOptimizer(const MixedAdamConfig&, const Shapes&, memory::MemoryManager*, uintptr_t, std::string*);
    std::string ensureList(const std::vector<uintptr_t>& grads);
    MixedAdamConfig config_;
    memory::MemoryManager* mm_ = nullptr;
    uintptr_t device_ = 0, mixed_ = 0, list_ = 0;
    std::vector<int> numel_;
    std::vector<uintptr_t> weights16_, master_, momentum_, variance_, listGrads_, listWeights_;
    uint64_t stepCount_ = 0;
};
std::unique_ptr<MixedAdamOptimizerState> NewMixedAdamOptimizer(const MixedAdamConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);

// L-BFGS keeps its own Step signature (lbfgs.go:245) and refuses a learning rate (lbfgs.go:330-332).
class LBFGSOptimizerState {
public:
    ~LBFGSOptimizerState();
    std::string SetWeightBuffers(const std::vector<uintptr_t>& weightBuffers);
    std::string Step(const std::vector<uintptr_t>& gradientBuffers, float currentLoss);
    std::string UpdateLearningRate(float lr);
    uint64_t GetStep() const { return stepCount_; }
    int historyCount() const { return historyCount_; }
    int historyIndex() const { return historyIndex_; }
    std::map<std::string, double> GetStats() const;
    void Cleanup();
    std::vector<float> readRho();          // one value per history slot (test hook)

private:
    friend std::unique_ptr<LBFGSOptimizerState> NewLBFGSOptimizer(const LBFGSConfig&, const Shapes&, memory::MemoryManager*, uintptr_t, std::string*);
    LBFGSConfig config_;
    memory::MemoryManager* mm_ = nullptr;
    uintptr_t device_ = 0;
    std::vector<int> bufferSizes_;
    std::vector<uintptr_t> weights_, oldGrad_, searchDir_, rho_;
    std::vector<std::vector<uintptr_t>> s_, y_;       // [history][weight]
    uintptr_t alpha_ = 0;
    int historyCount_ = 0, historyIndex_ = 0;
    uint64_t stepCount_ = 0;
    float prevLoss_ = 0.0f;
};
std::unique_ptr<LBFGSOptimizerState> NewLBFGSOptimizer(const LBFGSConfig&, const Shapes&, memory::MemoryManager*, uintptr_t device, std::string* err);

}  // namespace optimizer

// ---------------------------------------------------------------------
// training: learning-rate schedulers, training/scheduler.go:9-195
// ---------------------------------------------------------------------
namespace training {

class LRScheduler {
public:
    virtual ~LRScheduler() {}
    virtual double GetLR(int epoch, int step, double baseLR) = 0;
    virtual std::string GetName() const = 0;
    virtual double Step(double metric, double currentLR) { (void)metric; return currentLR; }
};

std::unique_ptr<LRScheduler> NewStepLRScheduler(int stepSize, double gamma);
std::unique_ptr<LRScheduler> NewExponentialLRScheduler(double gamma);
std::unique_ptr<LRScheduler> NewCosineAnnealingLRScheduler(int tMax, double etaMin);
std::unique_ptr<LRScheduler> NewReduceLROnPlateauScheduler(double factor, int patience, double threshold, const std::string& mode);
std::unique_ptr<LRScheduler> NewNoOpScheduler();

// model_trainer.go:1476-1582: the scheduler's float64 value becomes the
// optimizer's float32 learning rate for the next step.
std::string applyScheduler(LRScheduler& s, optimizer::Optimizer& opt, int epoch, int step, double baseLR);

}  // namespace training

}  // namespace gometal

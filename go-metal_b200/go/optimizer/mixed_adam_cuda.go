//go:build cuda

package optimizer

import (
	"fmt"
	"unsafe"

	"github.com/tsawler/go-metal/cgo_bridge"
	"github.com/tsawler/go-metal/checkpoints"
	"github.com/tsawler/go-metal/memory"
)

// MixedAdamConfig: Adam's hyper-parameters (adam.go:51-59) plus the dynamic loss
// scale whose defaults training/model_trainer.go:258-270 sets (65536, x2, x0.5,
// 2000 clean steps).
type MixedAdamConfig struct {
	LearningRate, Beta1, Beta2, Epsilon, WeightDecay float32
	InitialLossScale, GrowthFactor, BackoffFactor    float32
	GrowthInterval                                   int
	MaxLossScale                                     float32
}

func DefaultMixedAdamConfig() MixedAdamConfig {
	return MixedAdamConfig{LearningRate: 0.001, Beta1: 0.9, Beta2: 0.999, Epsilon: 1e-8,
		InitialLossScale: 65536, GrowthFactor: 2, BackoffFactor: 0.5, GrowthInterval: 2000, MaxLossScale: 16777216}
}

// MixedAdamOptimizerState keeps fp32 master weights and both Adam moments and
// steps them from fp16 gradients; the fp16 parameter buffers the model reads are
// rewritten every step.  Overflow detection, the skipped update and the change of
// the loss scale all happen on the device: Step returns after the launch, and
// GetState / LossScale wait for it.  The reference has the configuration fields
// only (training/model_trainer.go:79-87); the policy is that of
// docs/tutorials/mixed-precision.md:617-629.
type MixedAdamOptimizerState struct {
	Config MixedAdamConfig

	MasterBuffers   []unsafe.Pointer // fp32 master weights
	MomentumBuffers []unsafe.Pointer
	VarianceBuffers []unsafe.Pointer
	WeightBuffers   []unsafe.Pointer // fp16 parameters (set by the engine)

	StepCount uint64 // Step calls, skipped ones included

	memoryManager *memory.MemoryManager
	device        unsafe.Pointer
	numel         []int64
	mixed         *cgo_bridge.MixedAdam
	list          *cgo_bridge.TensorList
	listGrads     []unsafe.Pointer
	listWeights   []unsafe.Pointer
}

func NewMixedAdamOptimizer(config MixedAdamConfig, weightShapes [][]int, memoryManager *memory.MemoryManager,
	device unsafe.Pointer) (*MixedAdamOptimizerState, error) {
	if memoryManager == nil {
		return nil, fmt.Errorf("memory manager cannot be nil")
	}
	if device == nil {
		return nil, fmt.Errorf("device cannot be nil")
	}
	if len(weightShapes) == 0 {
		return nil, fmt.Errorf("no weight shapes provided")
	}
	if !(config.InitialLossScale > 0) {
		return nil, fmt.Errorf("initial loss scale must be positive, got %f", config.InitialLossScale)
	}
	if !(config.GrowthFactor >= 1) {
		return nil, fmt.Errorf("loss scale growth factor must be at least 1, got %f", config.GrowthFactor)
	}
	if !(config.BackoffFactor > 0 && config.BackoffFactor < 1) {
		return nil, fmt.Errorf("loss scale backoff factor must be in (0, 1), got %f", config.BackoffFactor)
	}
	if config.GrowthInterval < 1 {
		return nil, fmt.Errorf("loss scale growth interval must be positive, got %d", config.GrowthInterval)
	}
	n := len(weightShapes)
	o := &MixedAdamOptimizerState{Config: config, memoryManager: memoryManager, device: device,
		MasterBuffers: make([]unsafe.Pointer, n), MomentumBuffers: make([]unsafe.Pointer, n),
		VarianceBuffers: make([]unsafe.Pointer, n), WeightBuffers: make([]unsafe.Pointer, n), numel: make([]int64, n)}
	for i, shape := range weightShapes {
		o.numel[i] = int64(calculateTensorSize(shape))
		bytes := int(o.numel[i]) * 4
		for k, slot := range []*[]unsafe.Pointer{&o.MasterBuffers, &o.MomentumBuffers, &o.VarianceBuffers} {
			p := memoryManager.AllocateBuffer(bytes)
			if p == nil {
				o.Cleanup()
				return nil, fmt.Errorf("failed to allocate %s buffer for weight %d", []string{"master weight", "momentum", "variance"}[k], i)
			}
			(*slot)[i] = p
			if err := cgo_bridge.ZeroMetalBuffer(device, p, bytes); err != nil {
				o.Cleanup()
				return nil, fmt.Errorf("failed to zero buffer for weight %d: %v", i, err)
			}
		}
	}
	initial := cgo_bridge.LossScale{Scale: config.InitialLossScale, Growth: config.GrowthFactor, Backoff: config.BackoffFactor,
		MaxScale: config.MaxLossScale, Interval: int32(config.GrowthInterval)}
	mixed, err := cgo_bridge.NewMixedAdam(device, &initial, config.Beta1, config.Beta2)
	if err != nil {
		o.Cleanup()
		return nil, err
	}
	o.mixed = mixed
	return o, nil
}

func (o *MixedAdamOptimizerState) SetWeightBuffers(weightBuffers []unsafe.Pointer) error {
	if len(weightBuffers) != len(o.WeightBuffers) {
		return fmt.Errorf("expected %d weight buffers, got %d", len(o.WeightBuffers), len(weightBuffers))
	}
	copy(o.WeightBuffers, weightBuffers)
	return nil
}

// InitMaster sets the fp32 master weights of one tensor (a fresh run; a resumed one uses LoadState).
func (o *MixedAdamOptimizerState) InitMaster(index int, data []float32) error {
	if index < 0 || index >= len(o.MasterBuffers) {
		return fmt.Errorf("weight index %d out of range", index)
	}
	if int64(len(data)) != o.numel[index] {
		return fmt.Errorf("data size mismatch for master_%d: expected %d elements, got %d", index, o.numel[index], len(data))
	}
	return cgo_bridge.CopyFloat32ArrayToMetalBuffer(o.MasterBuffers[index], data)
}

func samePointers(a, b []unsafe.Pointer) bool {
	if len(a) != len(b) {
		return false
	}
	for i := range a {
		if a[i] != b[i] {
			return false
		}
	}
	return true
}

// The device-resident descriptor is rebuilt only when a pointer changes.
func (o *MixedAdamOptimizerState) ensureList(grads []unsafe.Pointer) error {
	if o.list != nil && samePointers(grads, o.listGrads) && samePointers(o.WeightBuffers, o.listWeights) {
		return nil
	}
	for i := range o.WeightBuffers {
		if o.WeightBuffers[i] == nil {
			return fmt.Errorf("weight buffer %d is nil", i)
		}
		if grads[i] == nil {
			return fmt.Errorf("gradient buffer %d is nil", i)
		}
	}
	if o.list != nil {
		if err := cgo_bridge.Synchronize(o.device); err != nil {
			return err
		}
		o.list.Destroy()
		o.list = nil
	}
	streams := [][]unsafe.Pointer{grads, o.MasterBuffers, o.MomentumBuffers, o.VarianceBuffers, o.WeightBuffers}
	list, err := cgo_bridge.NewTensorList(o.device, streams, o.numel, []int{2, 4, 4, 4, 2})
	if err != nil {
		return err
	}
	o.list = list
	o.listGrads = append([]unsafe.Pointer(nil), grads...)
	o.listWeights = append([]unsafe.Pointer(nil), o.WeightBuffers...)
	return nil
}

// Step takes one fp16 gradient buffer per weight.
func (o *MixedAdamOptimizerState) Step(gradientBuffers []unsafe.Pointer) error {
	if len(gradientBuffers) != len(o.WeightBuffers) {
		return fmt.Errorf("gradient buffers length (%d) doesn't match weight buffers length (%d)", len(gradientBuffers), len(o.WeightBuffers))
	}
	if err := o.ensureList(gradientBuffers); err != nil {
		return err
	}
	o.StepCount++
	if err := o.mixed.StepAsync(o.list, o.Config.LearningRate, o.Config.Epsilon, o.Config.WeightDecay); err != nil {
		return fmt.Errorf("MixedAdam step execution failed: %v", err)
	}
	return nil
}

// SetGradClip turns global-norm gradient clipping on (maxNorm > 0) or off (0); LastClip
// returns the last step's sum of squared unscaled gradients and clipping coefficient.
func (o *MixedAdamOptimizerState) SetGradClip(maxNorm float32) error { return o.mixed.SetClip(maxNorm) }

func (o *MixedAdamOptimizerState) LastClip() (float32, float32, error) { return o.mixed.LastClip() }

// LossScale waits for the stream and reads the device-resident loss-scale state.
func (o *MixedAdamOptimizerState) LossScale() (cgo_bridge.LossScale, error) { return o.mixed.State() }

func (o *MixedAdamOptimizerState) GetStepCount() uint64 { return o.StepCount }

func (o *MixedAdamOptimizerState) UpdateLearningRate(lr float32) { o.Config.LearningRate = lr }

func (o *MixedAdamOptimizerState) SetCommandPool(commandPool unsafe.Pointer) {}

func (o *MixedAdamOptimizerState) GetState() (*OptimizerState, error) {
	ls, err := o.mixed.State() // waits: the tensors read below are final
	if err != nil {
		return nil, err
	}
	state := &OptimizerState{Type: "MixedAdam", Parameters: map[string]interface{}{
		"learning_rate": o.Config.LearningRate, "beta1": o.Config.Beta1, "beta2": o.Config.Beta2,
		"epsilon": o.Config.Epsilon, "weight_decay": o.Config.WeightDecay,
		"step_count": o.StepCount, "adam_step": uint64(ls.AdamT),
		"loss_scale": ls.Scale, "growth_factor": ls.Growth, "backoff_factor": ls.Backoff, "max_loss_scale": ls.MaxScale,
		"growth_interval": uint64(ls.Interval), "good_steps": uint64(ls.GoodSteps), "skipped_steps": uint64(ls.Skipped),
	}}
	kinds := []string{"master", "momentum", "variance"}
	for k, slot := range [][]unsafe.Pointer{o.MasterBuffers, o.MomentumBuffers, o.VarianceBuffers} {
		for i, buffer := range slot {
			data, err := cgo_bridge.CopyMetalBufferToFloat32Array(buffer, int(o.numel[i]))
			if err != nil {
				return nil, fmt.Errorf("failed to read %s buffer %d: %v", kinds[k], i, err)
			}
			state.StateData = append(state.StateData, checkpoints.OptimizerTensor{
				Name: fmt.Sprintf("%s_%d", kinds[k], i), Shape: []int{len(data)}, Data: data, StateType: kinds[k]})
		}
	}
	return state, nil
}

// number reads a parameter that is float64 after a JSON round trip and its own kind straight from GetState.
func number(p map[string]interface{}, key string, def float64) float64 {
	switch v := p[key].(type) {
	case float64:
		return v
	case float32:
		return float64(v)
	case uint64:
		return float64(v)
	case int:
		return float64(v)
	}
	return def
}

func (o *MixedAdamOptimizerState) LoadState(state *OptimizerState) error {
	if err := validateStateType("MixedAdam", state); err != nil {
		return err
	}
	ls, err := o.mixed.State()
	if err != nil {
		return err
	}
	p := state.Parameters
	b1, b2 := float32(number(p, "beta1", float64(o.Config.Beta1))), float32(number(p, "beta2", float64(o.Config.Beta2)))
	if b1 != o.Config.Beta1 || b2 != o.Config.Beta2 {
		return fmt.Errorf("beta1/beta2 of the saved state (%g, %g) differ from this optimizer's (%g, %g)", b1, b2, o.Config.Beta1, o.Config.Beta2)
	}
	o.Config.LearningRate = float32(number(p, "learning_rate", float64(o.Config.LearningRate)))
	o.Config.Epsilon = float32(number(p, "epsilon", float64(o.Config.Epsilon)))
	o.Config.WeightDecay = float32(number(p, "weight_decay", float64(o.Config.WeightDecay)))
	o.StepCount = uint64(number(p, "step_count", float64(o.StepCount)))
	ls.Scale = float32(number(p, "loss_scale", float64(ls.Scale)))
	ls.Growth = float32(number(p, "growth_factor", float64(ls.Growth)))
	ls.Backoff = float32(number(p, "backoff_factor", float64(ls.Backoff)))
	ls.MaxScale = float32(number(p, "max_loss_scale", float64(ls.MaxScale)))
	ls.Interval = int32(number(p, "growth_interval", float64(ls.Interval)))
	ls.GoodSteps = int32(number(p, "good_steps", float64(ls.GoodSteps)))
	ls.Skipped = int32(number(p, "skipped_steps", float64(ls.Skipped)))
	ls.AdamT = int32(number(p, "adam_step", float64(ls.AdamT)))
	ls.LastOverflow = 0
	for _, t := range state.StateData {
		idx := extractBufferIndex(t.Name)
		if idx < 0 || idx >= len(o.MasterBuffers) {
			return fmt.Errorf("invalid buffer index in tensor name: %s", t.Name)
		}
		if int64(len(t.Data)) != o.numel[idx] {
			return fmt.Errorf("data size mismatch for %s: expected %d elements, got %d", t.Name, o.numel[idx], len(t.Data))
		}
		var dst unsafe.Pointer
		switch t.StateType {
		case "master":
			dst = o.MasterBuffers[idx]
		case "momentum":
			dst = o.MomentumBuffers[idx]
		case "variance":
			dst = o.VarianceBuffers[idx]
		default:
			return fmt.Errorf("unknown state type: %s", t.StateType)
		}
		if err := cgo_bridge.CopyFloat32ArrayToMetalBuffer(dst, t.Data); err != nil {
			return fmt.Errorf("failed to restore %s buffer %d: %v", t.StateType, idx, err)
		}
	}
	return o.mixed.SetState(ls)
}

func (o *MixedAdamOptimizerState) Cleanup() {
	if o.list != nil {
		_ = cgo_bridge.Synchronize(o.device)
		o.list.Destroy()
		o.list = nil
	}
	if o.mixed != nil {
		o.mixed.Destroy()
		o.mixed = nil
	}
	for _, slot := range [][]unsafe.Pointer{o.MasterBuffers, o.MomentumBuffers, o.VarianceBuffers} {
		for i, p := range slot {
			if p != nil {
				o.memoryManager.ReleaseBuffer(p)
				slot[i] = nil
			}
		}
	}
}

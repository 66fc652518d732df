//go:build cuda

// Additions to go-metal's optimizer package that ship with the CUDA bridge.
// These files sit beside the reference's optimizer/*.go, which compile unchanged
// against go-metal_b200/go/cgo_bridge.  No Go toolchain exists where this
// repository is built, so they have not been compiled there; the same logic is
// tested through the C++ mirror in go-metal_b200/host.
package optimizer

// GetStepCount completes the Optimizer interface (interface.go:13-43) on the two
// types that only offer GetStep in the reference (adam.go:266, rmsprop.go:261).
func (adam *AdamOptimizerState) GetStepCount() uint64 { return adam.StepCount }

func (rmsprop *RMSPropOptimizerState) GetStepCount() uint64 { return rmsprop.StepCount }

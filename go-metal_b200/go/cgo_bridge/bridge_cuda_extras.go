//go:build cuda

package cgo_bridge

/*
#include <stdlib.h>
#include "gometal_cuda.h"
*/
import "C"

import (
	"fmt"
	"unsafe"
)

// Entries with no counterpart in the Metal build: 64-bit buffers and arenas,
// persistent tensor lists with asynchronous steps, mixed-precision Adam with a
// device-resident loss scale, and ZeRO-1 sharding over the GPUs of one node.

// ---- arenas ----

type Arena struct{ h C.uintptr_t }

func NewArena(device unsafe.Pointer, bytes int64) (*Arena, error) {
	h := C.gm_arena_create(handle(device), C.int64_t(bytes))
	if h == 0 {
		return nil, fmt.Errorf("arena of %d bytes: %s", bytes, lastError())
	}
	return &Arena{h}, nil
}

// Alloc carves a 256-byte-aligned sub-buffer; nil when the arena is full.
func (a *Arena) Alloc(bytes int64) unsafe.Pointer {
	return unsafe.Pointer(uintptr(C.gm_arena_alloc(a.h, C.int64_t(bytes))))
}
func (a *Arena) Base() unsafe.Pointer { return unsafe.Pointer(uintptr(C.gm_arena_base(a.h))) }
func (a *Arena) Used() int64          { return int64(C.gm_arena_used(a.h)) }
func (a *Arena) Reset()               { C.gm_arena_reset(a.h) }
func (a *Arena) Destroy()             { C.gm_arena_destroy(a.h); a.h = 0 }

// ---- tensor lists and asynchronous steps ----

type Rule int

const (
	RuleSGD Rule = iota
	RuleAdam
	RuleRMSProp
	RuleAdaGrad
	RuleAdaDelta
	RuleNadam
)

// Hyper carries the scalars of one step (gm_hyper_t).  Beta1 doubles as the
// SGD momentum, RMSProp alpha and AdaDelta rho.
type Hyper struct {
	LR, Beta1, Beta2, Eps, WeightDecay, Momentum float32
	Nesterov, Centered                           bool
	Step                                         int
}

type TensorList struct{ h C.uintptr_t }

// NewTensorList builds the device-resident descriptor one multi-tensor launch
// walks.  streams[s][t] is the buffer of stream s (w, g, state...) for tensor t;
// elemBytes gives 4 or 2 per stream (nil: all fp32).
func NewTensorList(device unsafe.Pointer, streams [][]unsafe.Pointer, numel []int64, elemBytes []int) (*TensorList, error) {
	ns, nt := len(streams), len(numel)
	if ns == 0 || nt == 0 {
		return nil, fmt.Errorf("tensor list needs at least one stream and one tensor")
	}
	// The outer array holds C pointers, so it and the rows live in C memory for the call.
	outer := (*[1 << 20]*C.uintptr_t)(C.malloc(C.size_t(ns) * C.size_t(unsafe.Sizeof(uintptr(0)))))[:ns:ns]
	defer C.free(unsafe.Pointer(&outer[0]))
	for s := range streams {
		if len(streams[s]) != nt {
			return nil, fmt.Errorf("stream %d holds %d buffers, want %d", s, len(streams[s]), nt)
		}
		row := (*[1 << 28]C.uintptr_t)(C.malloc(C.size_t(nt) * C.size_t(unsafe.Sizeof(uintptr(0)))))[:nt:nt]
		defer C.free(unsafe.Pointer(&row[0]))
		for t, p := range streams[s] {
			row[t] = handle(p)
		}
		outer[s] = &row[0]
	}
	n64 := make([]C.int64_t, nt)
	for t, n := range numel {
		n64[t] = C.int64_t(n)
	}
	var eb *C.int
	if elemBytes != nil {
		if len(elemBytes) != ns {
			return nil, fmt.Errorf("elemBytes holds %d entries, want %d", len(elemBytes), ns)
		}
		e := cints(elemBytes)
		eb = &e[0]
	}
	h := C.gm_tensor_list_create(handle(device), C.int(ns), C.int(nt), &outer[0], &n64[0], eb)
	if h == 0 {
		return nil, fmt.Errorf("tensor list: %s", lastError())
	}
	return &TensorList{h}, nil
}

func (l *TensorList) Destroy() { C.gm_tensor_list_destroy(l.h); l.h = 0 }

func (h Hyper) c() C.gm_hyper_t {
	var out C.gm_hyper_t
	out.lr, out.beta1, out.beta2 = C.float(h.LR), C.float(h.Beta1), C.float(h.Beta2)
	out.eps, out.weight_decay, out.momentum = C.float(h.Eps), C.float(h.WeightDecay), C.float(h.Momentum)
	if h.Nesterov {
		out.nesterov = 1
	}
	if h.Centered {
		out.centered = 1
	}
	out.step = C.int(h.Step)
	return out
}

// StepAsync enqueues one step and returns; pair it with Synchronize.
func StepAsync(device unsafe.Pointer, rule Rule, list *TensorList, hyper Hyper) error {
	ch := hyper.c()
	return stepError("async", C.gm_step_async(handle(device), C.int(rule), list.h, &ch))
}

func Synchronize(device unsafe.Pointer) error {
	return stepError("synchronize", C.gm_device_synchronize(handle(device)))
}

// ---- mixed precision ----

// LossScale is the device-resident state of the dynamic loss scale
// (training/model_trainer.go:79-87 names the same fields on the host).
type LossScale struct {
	Scale, Growth, Backoff, MaxScale float32
	Interval, GoodSteps, AdamT       int32
	Skipped, LastOverflow            int32
}

type MixedAdam struct {
	h      C.uintptr_t
	device unsafe.Pointer
}

// NewMixedAdam uses the reference defaults (65536, x2, x0.5, 2000) when initial is nil.
func NewMixedAdam(device unsafe.Pointer, initial *LossScale, beta1, beta2 float32) (*MixedAdam, error) {
	var ci *C.gm_loss_scale_t
	if initial != nil {
		v := C.gm_loss_scale_t{scale: C.float(initial.Scale), growth: C.float(initial.Growth), backoff: C.float(initial.Backoff),
			max_scale: C.float(initial.MaxScale), interval: C.int32_t(initial.Interval), good_steps: C.int32_t(initial.GoodSteps),
			adam_t: C.int32_t(initial.AdamT), skipped: C.int32_t(initial.Skipped), last_overflow: C.int32_t(initial.LastOverflow)}
		ci = &v
	}
	h := C.gm_mixed_create(handle(device), ci, C.float(beta1), C.float(beta2), 0)
	if h == 0 {
		return nil, fmt.Errorf("mixed-precision state: %s", lastError())
	}
	return &MixedAdam{h, device}, nil
}

// StepAsync: list streams are g16, master, m, v, p16.  No host synchronisation;
// overflow detection, the skip decision and the scale update happen on the device.
func (m *MixedAdam) StepAsync(list *TensorList, lr, eps, weightDecay float32) error {
	return stepError("mixed Adam", C.gm_mixed_step_async(handle(m.device), m.h, list.h, C.float(lr), C.float(eps), C.float(weightDecay)))
}

// State waits for the stream and reads the loss-scale state (for checkpoints and logs).
func (m *MixedAdam) State() (LossScale, error) {
	var c C.gm_loss_scale_t
	if rc := C.gm_mixed_get_state(handle(m.device), m.h, &c); rc != 0 {
		return LossScale{}, stepError("mixed state", rc)
	}
	return LossScale{float32(c.scale), float32(c.growth), float32(c.backoff), float32(c.max_scale), int32(c.interval),
		int32(c.good_steps), int32(c.adam_t), int32(c.skipped), int32(c.last_overflow)}, nil
}

// SetState waits for the stream and overwrites the loss-scale state (checkpoint restore).
func (m *MixedAdam) SetState(s LossScale) error {
	c := C.gm_loss_scale_t{scale: C.float(s.Scale), growth: C.float(s.Growth), backoff: C.float(s.Backoff),
		max_scale: C.float(s.MaxScale), interval: C.int32_t(s.Interval), good_steps: C.int32_t(s.GoodSteps),
		adam_t: C.int32_t(s.AdamT), skipped: C.int32_t(s.Skipped), last_overflow: C.int32_t(s.LastOverflow)}
	return stepError("mixed state", C.gm_mixed_set_state(handle(m.device), m.h, &c))
}

// EnableGradNorm makes every following step also compute the sum of squares of the
// unscaled gradients inside the overflow-check pass; GradSumSq waits for the stream
// and returns the last step's value (inf or NaN on an overflow step).
func (m *MixedAdam) EnableGradNorm(on bool) error {
	v := C.int(0)
	if on {
		v = 1
	}
	return stepError("grad norm", C.gm_mixed_enable_grad_norm(m.h, v))
}

func (m *MixedAdam) GradSumSq() (float32, error) {
	var out C.float
	rc := C.gm_mixed_last_grad_sumsq(handle(m.device), m.h, &out)
	return float32(out), stepError("grad norm", rc)
}

// SetClip turns global-norm gradient clipping on (maxNorm > 0) or off (0): the overflow-check
// pass forms the norm of the unscaled gradients in a fixed order and the update multiplies
// every gradient by min(1, maxNorm/(norm+1e-6)) before the Adam rule.  LastClip waits for the
// stream and returns the last step's sum of squares and coefficient.
func (m *MixedAdam) SetClip(maxNorm float32) error {
	return stepError("clip", C.gm_mixed_set_clip(m.h, C.float(maxNorm)))
}

func (m *MixedAdam) LastClip() (sumSq, coef float32, err error) {
	var s, c C.float
	rc := C.gm_mixed_last_clip(handle(m.device), m.h, &s, &c)
	return float32(s), float32(c), stepError("clip", rc)
}

func (m *MixedAdam) Destroy() { C.gm_mixed_destroy(m.h); m.h = 0 }

// StepHost runs one step with the gradients in (pinned) host memory and the new
// parameters returned to host memory; upload, update and download are pipelined
// over `slices` groups of tensors.  Parameter and gradient tensors that lie back to back
// on the device move with one copy per slice, separately allocated ones one by one.
func StepHost(device unsafe.Pointer, rule Rule, list *TensorList, hyper Hyper, hostGrads, hostParams unsafe.Pointer, slices int) error {
	ch := hyper.c()
	return stepError("host-buffer step", C.gm_step_host(handle(device), C.int(rule), list.h, &ch, hostGrads, hostParams, C.int(slices)))
}

// ---- ZeRO-1 ----

const NCCLUniqueIDBytes = 128

// Zero1UniqueID is called on rank 0; the 128 bytes travel to the other ranks by any host channel.
func Zero1UniqueID() ([NCCLUniqueIDBytes]byte, error) {
	var id [NCCLUniqueIDBytes]byte
	if rc := C.gm_zero1_unique_id(unsafe.Pointer(&id[0])); rc != 0 {
		return id, stepError("nccl unique id", rc)
	}
	return id, nil
}

type Zero1 struct{ h C.uintptr_t }

func NewZero1(device unsafe.Pointer, id [NCCLUniqueIDBytes]byte, rank, world int) (*Zero1, error) {
	h := C.gm_zero1_create(handle(device), unsafe.Pointer(&id[0]), C.int(rank), C.int(world))
	if h == 0 {
		return nil, fmt.Errorf("ZeRO-1 group: %s", lastError())
	}
	return &Zero1{h}, nil
}

// AdamStepAsync updates this rank's shard and all-gathers the parameter arena in place.
func (z *Zero1) AdamStepAsync(shard *TensorList, hyper Hyper, arenaBase unsafe.Pointer, countPerRank int64) error {
	ch := hyper.c()
	return stepError("ZeRO-1 Adam", C.gm_zero1_adam_step_async(z.h, shard.h, &ch, handle(arenaBase), C.int64_t(countPerRank)))
}

// StepAsync is AdamStepAsync for any fp32 rule: the shard's update, then the in-place all-gather.
func (z *Zero1) StepAsync(rule Rule, shard *TensorList, hyper Hyper, arenaBase unsafe.Pointer, countPerRank int64) error {
	ch := hyper.c()
	return stepError("ZeRO-1 step", C.gm_zero1_step_async(z.h, C.int(rule), shard.h, &ch, handle(arenaBase), C.int64_t(countPerRank)))
}

// IPCHandle exports this rank's arena; OpenPeers maps every rank's handle (rank order, 64 bytes each).
func (z *Zero1) IPCHandle(arenaBase unsafe.Pointer) ([64]byte, error) {
	var hnd [64]byte
	rc := C.gm_zero1_ipc_handle(z.h, handle(arenaBase), unsafe.Pointer(&hnd[0]))
	return hnd, stepError("ipc handle", rc)
}

func (z *Zero1) OpenPeers(handles []byte) error {
	if len(handles) == 0 {
		return fmt.Errorf("no handles")
	}
	return stepError("open peers", C.gm_zero1_open_peers(z.h, unsafe.Pointer(&handles[0])))
}

// AdamPushStepAsync is the fused update + exchange: new parameters are stored to every peer's arena by the update kernel itself.
func (z *Zero1) AdamPushStepAsync(shard *TensorList, hyper Hyper) error {
	ch := hyper.c()
	return stepError("ZeRO-1 Adam push", C.gm_zero1_adam_push_step_async(z.h, shard.h, &ch))
}

// AdamDMAStepAsync updates the shard in slices and lets the copy engines carry each finished slice to the peers.
func (z *Zero1) AdamDMAStepAsync(shard *TensorList, hyper Hyper, slices int) error {
	ch := hyper.c()
	return stepError("ZeRO-1 Adam dma", C.gm_zero1_adam_dma_step_async(z.h, shard.h, &ch, C.int(slices)))
}

// MixedStepAsync is the mixed-precision step on a sharded list: the overflow flag is
// summed across ranks before the update, then the fp16 parameter arena is all-gathered.
func (z *Zero1) MixedStepAsync(m *MixedAdam, shard *TensorList, lr, eps, weightDecay float32, p16ArenaBase unsafe.Pointer, countPerRank int64) error {
	return stepError("ZeRO-1 mixed Adam", C.gm_zero1_mixed_step_async(z.h, m.h, shard.h, C.float(lr), C.float(eps), C.float(weightDecay),
		handle(p16ArenaBase), C.int64_t(countPerRank)))
}

// ReduceScatterAsync sums the ranks' gradient arenas; each rank keeps the sum of its own shard, in place.
func (z *Zero1) ReduceScatterAsync(gradArenaBase unsafe.Pointer, countPerRank int64, elemBytes int) error {
	return stepError("reduce-scatter", C.gm_zero1_reduce_scatter_async(z.h, handle(gradArenaBase), C.int64_t(countPerRank), C.int(elemBytes)))
}

func (z *Zero1) Destroy() { C.gm_zero1_destroy(z.h); z.h = 0 }

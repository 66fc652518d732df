//go:build cuda

// Package cgo_bridge, CUDA build.
//
// This file gives go-metal's cgo_bridge package a CUDA (B200, sm_100a) body
// for the optimizer-step path.  It exports the same Go functions, with the
// same signatures, that optimizer/*.go and memory/manager.go call in the Metal
// build (cgo_bridge/bridge.go:623-645, 729-760, 892-1196, 1676-1695,
// 1791-2354), so those packages compile unchanged; only the C symbol behind
// each wrapper differs (libgometal_cuda.so, include/gometal_cuda.h).
//
// Build:  go build -tags cuda ./...   with the Objective-C files of the
// package guarded by `//go:build !cuda`.
//
// No Go toolchain exists where this repository is built, so this file has not
// been compiled there; the same marshalling is exercised through the C++
// mirror in go-metal_b200/host and its tests.
package cgo_bridge

/*
#cgo CFLAGS: -I${SRCDIR}/../../../include
#cgo LDFLAGS: -L${SRCDIR}/../../lib -lgometal_cuda -Wl,-rpath,${SRCDIR}/../../lib
#include <stdlib.h>
#include <stdbool.h>
#include "gometal_cuda.h"
*/
import "C"

import (
	"fmt"
	"unsafe"
)

// DeviceType mirrors cgo_bridge/bridge.go:623-629; every kind maps to device memory.
type DeviceType int

const (
	CPU DeviceType = iota
	GPU
	PersistentGPU
)

func lastError() string { return C.GoString(C.gm_last_error()) }

func handle(p unsafe.Pointer) C.uintptr_t { return C.uintptr_t(uintptr(p)) }

// addrs copies a slice of device pointers into C-typed storage that lives for
// the duration of one call; the library copies what it needs and keeps nothing.
func addrs(ptrs []unsafe.Pointer) []C.uintptr_t {
	out := make([]C.uintptr_t, len(ptrs))
	for i, p := range ptrs {
		out[i] = handle(p)
	}
	return out
}

func first(a []C.uintptr_t) *C.uintptr_t {
	if len(a) == 0 {
		return nil
	}
	return &a[0]
}

func cints(v []int) []C.int {
	out := make([]C.int, len(v))
	for i, x := range v {
		out[i] = C.int(x)
	}
	return out
}

func sameLength(what string, n int, lists ...[]unsafe.Pointer) error {
	for _, l := range lists {
		if l != nil && len(l) != n {
			return fmt.Errorf("%s: buffer lists must all hold %d entries, got %d", what, n, len(l))
		}
	}
	return nil
}

func stepError(name string, rc C.int) error {
	if rc == 0 {
		return nil
	}
	return fmt.Errorf("%s step failed with error code: %d (%s)", name, int(rc), lastError())
}

// ---- device and queue ----

func CreateMetalDevice() (unsafe.Pointer, error) {
	d := C.create_cuda_device()
	if d == 0 {
		return nil, fmt.Errorf("failed to create CUDA device: %s", lastError())
	}
	return unsafe.Pointer(uintptr(d)), nil
}

func DestroyMetalDevice(device unsafe.Pointer) {
	if device != nil {
		C.destroy_cuda_device(handle(device))
	}
}

func CreateCommandQueue(device unsafe.Pointer) (unsafe.Pointer, error) {
	if device == nil {
		return nil, fmt.Errorf("device cannot be nil")
	}
	q := C.create_command_queue(handle(device))
	if q == 0 {
		return nil, fmt.Errorf("failed to create command queue: %s", lastError())
	}
	return unsafe.Pointer(uintptr(q)), nil
}

func ReleaseCommandQueue(commandQueue unsafe.Pointer) {
	if commandQueue != nil {
		C.release_command_queue(handle(commandQueue))
	}
}

// ---- buffers ----

func AllocateMetalBuffer(device unsafe.Pointer, size int, deviceType DeviceType) (unsafe.Pointer, error) {
	b := C.allocate_cuda_buffer(handle(device), C.int(size), C.int(deviceType))
	if b == 0 {
		return nil, fmt.Errorf("failed to allocate CUDA buffer of size %d: %s", size, lastError())
	}
	return unsafe.Pointer(uintptr(b)), nil
}

func DeallocateMetalBuffer(buffer unsafe.Pointer) {
	if buffer != nil {
		C.deallocate_cuda_buffer(handle(buffer))
	}
}

func ZeroMetalBuffer(device unsafe.Pointer, buffer unsafe.Pointer, size int) error {
	if rc := C.zero_cuda_buffer(handle(device), handle(buffer), C.int(size)); rc != 0 {
		return fmt.Errorf("failed to zero buffer with error code: %d (%s)", int(rc), lastError())
	}
	return nil
}

// ZeroMetalBufferMPSGraph is kept for callers of the Metal build; it is the same memset here.
func ZeroMetalBufferMPSGraph(device unsafe.Pointer, buffer unsafe.Pointer, size int) error {
	return ZeroMetalBuffer(device, buffer, size)
}

func CopyFloat32ArrayToMetalBuffer(buffer unsafe.Pointer, data []float32) error {
	if buffer == nil {
		return fmt.Errorf("buffer cannot be nil")
	}
	if len(data) == 0 {
		return fmt.Errorf("data cannot be empty")
	}
	rc := C.copy_float32_array_to_cuda_buffer(handle(buffer), (*C.float)(unsafe.Pointer(&data[0])), C.int(len(data)))
	if rc != 0 {
		return fmt.Errorf("failed to copy float32 data to buffer with error code: %d (%s)", int(rc), lastError())
	}
	return nil
}

func CopyMetalBufferToFloat32Array(buffer unsafe.Pointer, numElements int) ([]float32, error) {
	if buffer == nil {
		return nil, fmt.Errorf("buffer cannot be nil")
	}
	if numElements <= 0 {
		return nil, fmt.Errorf("number of elements must be positive")
	}
	out := make([]float32, numElements)
	rc := C.copy_cuda_buffer_to_float32_array(handle(buffer), (*C.float)(unsafe.Pointer(&out[0])), C.int(numElements))
	if rc != 0 {
		return nil, fmt.Errorf("failed to copy buffer to float32 array with error code: %d (%s)", int(rc), lastError())
	}
	return out, nil
}

func ConvertTensorType(srcBuffer, dstBuffer unsafe.Pointer, shape []int, srcType, dstType int, device unsafe.Pointer) error {
	if len(shape) == 0 {
		return fmt.Errorf("shape cannot be empty")
	}
	cs := cints(shape)
	rc := C.convert_tensor_type_cuda(handle(srcBuffer), handle(dstBuffer), &cs[0], C.int(len(cs)), C.int(srcType), C.int(dstType), handle(device))
	if rc != 0 {
		return fmt.Errorf("tensor type conversion failed with error code: %d (%s)", int(rc), lastError())
	}
	return nil
}

//go:build cuda

package cgo_bridge

/*
#include <stdbool.h>
#include "gometal_cuda.h"
*/
import "C"

import (
	"fmt"
	"unsafe"
)

// The optimizer-step wrappers.  Names and signatures are those of the Metal
// build (cgo_bridge/bridge.go:892-1034, 1791-2354); each marshals its Go slices
// into C arrays that live for the call only and maps the int return code to an
// error.  A non-zero code carries the library's text (gm_last_error).

func ExecuteSGDStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, momentumBuffers []unsafe.Pointer,
	bufferSizes []int, learningRate, momentum, weightDecay float32, nesterov bool, stepCount int) error {
	n := len(weightBuffers)
	if n == 0 || len(bufferSizes) != n {
		return fmt.Errorf("SGD: %d weight buffers but %d sizes", n, len(bufferSizes))
	}
	if err := sameLength("SGD", n, gradientBuffers, momentumBuffers); err != nil {
		return err
	}
	w, g, m, s := addrs(weightBuffers), addrs(gradientBuffers), addrs(momentumBuffers), cints(bufferSizes)
	nest := C.int(0)
	if nesterov {
		nest = 1
	}
	rc := C.execute_sgd_step_cuda(handle(device), first(w), first(g), first(m), C.int(n), &s[0],
		C.float(learningRate), C.float(momentum), C.float(weightDecay), nest, C.int(stepCount))
	return stepError("SGD", rc)
}

func adamLike(name string, pooled bool, device unsafe.Pointer, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers []unsafe.Pointer,
	bufferSizes []int, lr, beta1, beta2, eps, wd float32, stepCount int, commandPool unsafe.Pointer) error {
	n := len(weightBuffers)
	if n == 0 || len(bufferSizes) != n {
		return fmt.Errorf("%s: %d weight buffers but %d sizes", name, n, len(bufferSizes))
	}
	if err := sameLength(name, n, gradientBuffers, momentumBuffers, varianceBuffers); err != nil {
		return err
	}
	w, g, m, v, s := addrs(weightBuffers), addrs(gradientBuffers), addrs(momentumBuffers), addrs(varianceBuffers), cints(bufferSizes)
	var rc C.int
	switch {
	case name == "Nadam":
		rc = C.execute_nadam_step_cuda(handle(device), first(w), first(g), first(m), first(v), C.int(n), &s[0],
			C.float(lr), C.float(beta1), C.float(beta2), C.float(eps), C.float(wd), C.int(stepCount))
	case pooled:
		rc = C.execute_adam_step_cuda_pooled(handle(device), first(w), first(g), first(m), first(v), C.int(n), &s[0],
			C.float(lr), C.float(beta1), C.float(beta2), C.float(eps), C.float(wd), C.int(stepCount), handle(commandPool))
	default:
		rc = C.execute_adam_step_cuda(handle(device), first(w), first(g), first(m), first(v), C.int(n), &s[0],
			C.float(lr), C.float(beta1), C.float(beta2), C.float(eps), C.float(wd), C.int(stepCount))
	}
	return stepError(name, rc)
}

func ExecuteAdamStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers []unsafe.Pointer,
	bufferSizes []int, learningRate, beta1, beta2, epsilon, weightDecay float32, stepCount int) error {
	return adamLike("Adam", false, device, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers, bufferSizes,
		learningRate, beta1, beta2, epsilon, weightDecay, stepCount, nil)
}

func ExecuteAdamStepMPSGraphPooled(device unsafe.Pointer, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers []unsafe.Pointer,
	bufferSizes []int, learningRate, beta1, beta2, epsilon, weightDecay float32, stepCount int, commandPool unsafe.Pointer) error {
	return adamLike("Adam", true, device, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers, bufferSizes,
		learningRate, beta1, beta2, epsilon, weightDecay, stepCount, commandPool)
}

func ExecuteNadamStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers []unsafe.Pointer,
	bufferSizes []int, learningRate, beta1, beta2, epsilon, weightDecay float32, stepCount int) error {
	return adamLike("Nadam", false, device, weightBuffers, gradientBuffers, momentumBuffers, varianceBuffers, bufferSizes,
		learningRate, beta1, beta2, epsilon, weightDecay, stepCount, nil)
}

func ExecuteRMSPropStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, squaredGradAvgBuffers, momentumBuffers, gradientAvgBuffers []unsafe.Pointer,
	bufferSizes []int, learningRate, alpha, epsilon, weightDecay, momentum float32, centered bool, stepCount int) error {
	n := len(weightBuffers)
	if n == 0 || len(bufferSizes) != n {
		return fmt.Errorf("RMSProp: %d weight buffers but %d sizes", n, len(bufferSizes))
	}
	if err := sameLength("RMSProp", n, gradientBuffers, squaredGradAvgBuffers); err != nil {
		return err
	}
	w, g, q, s := addrs(weightBuffers), addrs(gradientBuffers), addrs(squaredGradAvgBuffers), cints(bufferSizes)
	// the optional buffers are passed only when the mode uses them
	var m, a []C.uintptr_t
	if momentum > 0 {
		m = addrs(momentumBuffers)
	}
	if centered {
		a = addrs(gradientAvgBuffers)
	}
	rc := C.execute_rmsprop_step_cuda(handle(device), first(w), first(g), first(q), first(m), first(a), C.int(n), &s[0],
		C.float(learningRate), C.float(alpha), C.float(epsilon), C.float(weightDecay), C.float(momentum), C.bool(centered), C.int(stepCount))
	return stepError("RMSProp", rc)
}

func ExecuteAdaGradStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, squaredGradAvgBuffers []unsafe.Pointer,
	numWeights int, bufferSizes []int, learningRate, epsilon, weightDecay float32) error {
	if numWeights <= 0 || len(weightBuffers) != numWeights || len(bufferSizes) != numWeights {
		return fmt.Errorf("AdaGrad: numWeights %d does not match %d buffers / %d sizes", numWeights, len(weightBuffers), len(bufferSizes))
	}
	if err := sameLength("AdaGrad", numWeights, gradientBuffers, squaredGradAvgBuffers); err != nil {
		return err
	}
	w, g, q, s := addrs(weightBuffers), addrs(gradientBuffers), addrs(squaredGradAvgBuffers), cints(bufferSizes)
	rc := C.execute_adagrad_step_cuda(handle(device), first(w), first(g), first(q), C.int(numWeights), &s[0],
		C.float(learningRate), C.float(epsilon), C.float(weightDecay))
	return stepError("AdaGrad", rc)
}

// The pooled variants run on the device's own stream; the pool handle is accepted and unused.
func ExecuteAdaGradStepMPSGraphPooled(device unsafe.Pointer, weightBuffers, gradientBuffers, squaredGradAvgBuffers []unsafe.Pointer,
	numWeights int, bufferSizes []int, learningRate, epsilon, weightDecay float32, commandPool unsafe.Pointer) error {
	_ = commandPool
	return ExecuteAdaGradStepMPSGraph(device, weightBuffers, gradientBuffers, squaredGradAvgBuffers, numWeights, bufferSizes, learningRate, epsilon, weightDecay)
}

func ExecuteAdaDeltaStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, squaredGradAvgBuffers, squaredUpdateAvgBuffers []unsafe.Pointer,
	numWeights int, bufferSizes []int, rho, epsilon, weightDecay float32) error {
	if numWeights <= 0 || len(weightBuffers) != numWeights || len(bufferSizes) != numWeights {
		return fmt.Errorf("AdaDelta: numWeights %d does not match %d buffers / %d sizes", numWeights, len(weightBuffers), len(bufferSizes))
	}
	if err := sameLength("AdaDelta", numWeights, gradientBuffers, squaredGradAvgBuffers, squaredUpdateAvgBuffers); err != nil {
		return err
	}
	w, g, q, u, s := addrs(weightBuffers), addrs(gradientBuffers), addrs(squaredGradAvgBuffers), addrs(squaredUpdateAvgBuffers), cints(bufferSizes)
	rc := C.execute_adadelta_step_cuda(handle(device), first(w), first(g), first(q), first(u), C.int(numWeights), &s[0],
		C.float(rho), C.float(epsilon), C.float(weightDecay))
	return stepError("AdaDelta", rc)
}

func ExecuteAdaDeltaStepMPSGraphPooled(device unsafe.Pointer, weightBuffers, gradientBuffers, squaredGradAvgBuffers, squaredUpdateAvgBuffers []unsafe.Pointer,
	numWeights int, bufferSizes []int, rho, epsilon, weightDecay float32, commandPool unsafe.Pointer) error {
	_ = commandPool
	return ExecuteAdaDeltaStepMPSGraph(device, weightBuffers, gradientBuffers, squaredGradAvgBuffers, squaredUpdateAvgBuffers, numWeights, bufferSizes, rho, epsilon, weightDecay)
}

// ExecuteLBFGSStepMPSGraph flattens the [history][weight] vectors slot-major
// ([h*numWeights + w], cgo_bridge/bridge.go:1987-1998) and returns the step size.
func ExecuteLBFGSStepMPSGraph(device unsafe.Pointer, weightBuffers, gradientBuffers, oldGradientBuffers, searchDirBuffers []unsafe.Pointer,
	sVectors, yVectors [][]unsafe.Pointer, rhoBuffers []unsafe.Pointer, alphaBuffer unsafe.Pointer, numWeights int, bufferSizes []int,
	historySize, historyCount, historyIndex int, initialStep, c1, c2 float32, maxLineSearch int, currentLoss, prevLoss float32,
	commandPool unsafe.Pointer, usePooling bool) (float32, error) {
	if numWeights <= 0 || len(weightBuffers) != numWeights || len(bufferSizes) != numWeights {
		return 0, fmt.Errorf("L-BFGS: numWeights %d does not match %d buffers / %d sizes", numWeights, len(weightBuffers), len(bufferSizes))
	}
	if len(sVectors) != historySize || len(yVectors) != historySize || len(rhoBuffers) != historySize {
		return 0, fmt.Errorf("L-BFGS: history size %d does not match the vector lists", historySize)
	}
	flat := func(v [][]unsafe.Pointer) ([]C.uintptr_t, error) {
		out := make([]C.uintptr_t, 0, historySize*numWeights)
		for h := range v {
			if len(v[h]) != numWeights {
				return nil, fmt.Errorf("L-BFGS: history slot %d holds %d vectors, want %d", h, len(v[h]), numWeights)
			}
			out = append(out, addrs(v[h])...)
		}
		return out, nil
	}
	sf, err := flat(sVectors)
	if err != nil {
		return 0, err
	}
	yf, err := flat(yVectors)
	if err != nil {
		return 0, err
	}
	w, g, og, d, r, s := addrs(weightBuffers), addrs(gradientBuffers), addrs(oldGradientBuffers), addrs(searchDirBuffers), addrs(rhoBuffers), cints(bufferSizes)
	var step C.float
	var rc C.int
	if usePooling {
		rc = C.execute_lbfgs_step_cuda_pooled(handle(device), first(w), first(g), first(og), first(d), first(sf), first(yf), first(r),
			handle(alphaBuffer), C.int(numWeights), &s[0], C.int(historySize), C.int(historyCount), C.int(historyIndex),
			C.float(initialStep), C.float(c1), C.float(c2), C.int(maxLineSearch), C.float(currentLoss), C.float(prevLoss), handle(commandPool), &step)
	} else {
		rc = C.execute_lbfgs_step_cuda(handle(device), first(w), first(g), first(og), first(d), first(sf), first(yf), first(r),
			handle(alphaBuffer), C.int(numWeights), &s[0], C.int(historySize), C.int(historyCount), C.int(historyIndex),
			C.float(initialStep), C.float(c1), C.float(c2), C.int(maxLineSearch), C.float(currentLoss), C.float(prevLoss), &step)
	}
	if rc != 0 {
		return 0, stepError("L-BFGS", rc)
	}
	return float32(step), nil
}

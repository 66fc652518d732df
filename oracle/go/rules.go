// Package gmoracle is the Go twin of oracle/gm_oracle.c: a scalar transcription
// of the update equations of go-metal's optimizer step, in the operation order
// of cgo_bridge/bridge_optimizer.m (line ranges at each function).
//
// TEST INFRASTRUCTURE, NOT PRODUCT.  PARITY UNPINNED: the reference holds no
// golden vector for any optimizer step.  This source is shipped uncompiled where
// no Go toolchain exists; bench.py times it only when `go` is on PATH.
//
// Every product is wrapped in an explicit float32 conversion: the Go
// specification lets a compiler fuse x*y + z unless the product is converted,
// and the rules here are defined with one rounding per operation.  The host
// scalars use math.Pow in float64 rounded once to float32, which can differ
// from C powf in the last bit for some (base, step) pairs; the C oracle, which
// calls powf like the reference does, is the one the kernels are tested against.
package gmoracle

import "math"

func sqrt32(x float32) float32 { return float32(math.Sqrt(float64(x))) }

func pow32(b, e float32) float32 { return float32(math.Pow(float64(b), float64(e))) }

// AdamScalars follows bridge_optimizer.m:398-399 and :469-472.
func AdamScalars(beta1, beta2 float32, step int) (bc1, bc2, omb1, omb2 float32) {
	bc1 = 1.0 - pow32(beta1, float32(step))
	bc2 = 1.0 - pow32(beta2, float32(step))
	omb1 = 1.0 - beta1
	omb2 = 1.0 - beta2
	return
}

// NadamMuNext follows bridge_optimizer.m:2066.
func NadamMuNext(beta1 float32, step int) float32 {
	e := float32(float32(step+1) * 0.004)
	return float32(beta1 * float32(1.0-float32(0.5*pow32(0.96, e))))
}

// AdamStep follows bridge_optimizer.m:484-550.
func AdamStep(w, g, m, v []float32, lr, beta1, beta2, eps, wd float32, step int) {
	bc1, bc2, omb1, omb2 := AdamScalars(beta1, beta2, step)
	for i := range w {
		gi := g[i]
		mNew := float32(m[i]*beta1) + float32(gi*omb1)
		gSq := float32(gi * gi)
		vNew := float32(v[i]*beta2) + float32(gSq*omb2)
		mHat := mNew / bc1
		vHat := vNew / bc2
		denom := sqrt32(vHat) + eps
		upd := mHat / denom
		if wd > 0 {
			upd = upd + float32(w[i]*wd)
		}
		w[i] = w[i] - float32(upd*lr)
		m[i] = mNew
		v[i] = vNew
	}
}

// SGDStep follows bridge_optimizer.m:219-228 (decay), :244-278 (momentum),
// :315-322 (plain).  mom may be nil.
func SGDStep(w, g, mom []float32, lr, momentum, wd float32, nesterov bool) {
	useMom := momentum > 0 && mom != nil
	for i := range w {
		gf := g[i]
		if wd > 0 {
			gf = g[i] + float32(w[i]*wd)
		}
		if useMom {
			mNew := float32(mom[i]*momentum) + gf
			var s float32
			if nesterov {
				s = float32(lr * (float32(momentum*mNew) + gf))
			} else {
				s = float32(lr * mNew)
			}
			w[i] = w[i] - s
			mom[i] = mNew
		} else {
			w[i] = w[i] - float32(lr*gf)
		}
	}
}

// RMSPropStep follows bridge_optimizer.m:782-876.  mom and gavg may be nil.
// persistAux=false reproduces the reference, which computes the new momentum
// and gradient average but never stores them (:915, :928-937).
func RMSPropStep(w, g, sq, mom, gavg []float32, lr, alpha, eps, wd, momentum float32, centered, persistAux bool) {
	oma := float32(1.0 - alpha)
	for i := range w {
		gi := g[i]
		vNew := float32(sq[i]*alpha) + float32(float32(gi*gi)*oma)
		var d float32
		var aNew float32
		if centered {
			aNew = float32(gavg[i]*alpha) + float32(gi*oma)
			d = sqrt32((vNew - float32(aNew*aNew)) + eps)
		} else {
			d = sqrt32(vNew + eps)
		}
		u := gi / d
		var bNew float32
		if momentum > 0 {
			bNew = float32(mom[i]*momentum) + u
			u = bNew
		}
		if wd > 0 {
			u = u + float32(w[i]*wd)
		}
		w[i] = w[i] - float32(u*lr)
		sq[i] = vNew
		if persistAux {
			if centered {
				gavg[i] = aNew
			}
			if momentum > 0 {
				mom[i] = bNew
			}
		}
	}
}

// AdaGradStep follows bridge_optimizer.m:1480-1517 (epsilon outside the root).
func AdaGradStep(w, g, sq []float32, lr, eps, wd float32) {
	for i := range w {
		gf := g[i]
		if wd > 0 {
			gf = g[i] + float32(w[i]*wd)
		}
		acc := sq[i] + float32(gf*gf)
		d := sqrt32(acc) + eps
		r := lr / d
		w[i] = w[i] - float32(r*gf)
		sq[i] = acc
	}
}

// AdaDeltaStep follows bridge_optimizer.m:1773-1843.
func AdaDeltaStep(w, g, sq, upd []float32, rho, eps, wd float32) {
	omr := float32(1.0 - rho)
	for i := range w {
		gf := g[i]
		if wd > 0 {
			gf = g[i] + float32(w[i]*wd)
		}
		eNew := float32(sq[i]*rho) + float32(float32(gf*gf)*omr)
		rg := sqrt32(eNew + eps)
		ru := sqrt32(upd[i] + eps)
		u := float32(float32(ru/rg) * gf)
		n := -u
		w[i] = w[i] + n
		upd[i] = float32(upd[i]*rho) + float32(float32(n*n)*omr)
		sq[i] = eNew
	}
}

// NadamStep follows bridge_optimizer.m:2114-2200.
func NadamStep(w, g, m, v []float32, lr, beta1, beta2, eps, wd float32, step int) {
	bc1, bc2, omb1, omb2 := AdamScalars(beta1, beta2, step)
	mu := NadamMuNext(beta1, step)
	om := float32(1.0 - mu)
	for i := range w {
		gi := g[i]
		mNew := float32(m[i]*beta1) + float32(gi*omb1)
		vNew := float32(v[i]*beta2) + float32(float32(gi*gi)*omb2)
		vHat := vNew / bc2
		mHat := mNew / bc1
		gHat := gi / bc1
		mb := float32(mHat*mu) + float32(gHat*om)
		d := sqrt32(vHat) + eps
		u := mb / d
		if wd > 0 {
			u = u + float32(w[i]*wd)
		}
		w[i] = w[i] - float32(u*lr)
		m[i] = mNew
		v[i] = vNew
	}
}

// DotSequential is the reference's own order: one fp32 accumulator, left to
// right (bridge_optimizer.m:1073-1109).
func DotSequential(a, b []float32) float32 {
	var acc float32
	for i := range a {
		acc = acc + float32(a[i]*b[i])
	}
	return acc
}

const (
	dotChunk = 4096
	dotLanes = 256
)

func tree256(lane *[dotLanes]float32) float32 {
	// 32 lanes of a warp combine by xor tree (16, 8, 4, 2, 1); the 8 warp sums add in ascending order
	var warp [dotLanes / 32]float32
	for w := 0; w < dotLanes/32; w++ {
		var x [32]float32
		copy(x[:], lane[w*32:(w+1)*32])
		for off := 16; off >= 1; off >>= 1 {
			var y [32]float32
			for l := 0; l < 32; l++ {
				y[l] = x[l] + x[l^off]
			}
			x = y
		}
		warp[w] = x[0]
	}
	total := warp[0]
	for w := 1; w < dotLanes/32; w++ {
		total = total + warp[w]
	}
	return total
}

// DotCanonical is the fixed summation order shared by the C oracle and the
// L-BFGS kernels: 4096-element chunks; inside a chunk lane t of 256 adds the
// products of elements (i*256+t)*4+k (i = 0..3, k = 0..3) in that order; then
// the tree above; the chunk sums are combined the same way (lane t takes
// chunks t, t+256, ...).
func DotCanonical(a, b []float32) float32 {
	n := len(a)
	chunks := (n + dotChunk - 1) / dotChunk
	partials := make([]float32, chunks)
	for c := 0; c < chunks; c++ {
		var lane [dotLanes]float32
		for t := 0; t < dotLanes; t++ {
			var acc float32
			for i := 0; i < dotChunk/(dotLanes*4); i++ {
				for k := 0; k < 4; k++ {
					e := c*dotChunk + (i*dotLanes+t)*4 + k
					if e < n {
						acc = acc + float32(a[e]*b[e])
					}
				}
			}
			lane[t] = acc
		}
		partials[c] = tree256(&lane)
	}
	var lane [dotLanes]float32
	for t := 0; t < dotLanes; t++ {
		var acc float32
		for c := t; c < chunks; c += dotLanes {
			acc = acc + partials[c]
		}
		lane[t] = acc
	}
	return tree256(&lane)
}

// gmoracle_bench times the Go transcription of the fp32 Adam step on the host
// cores and prints one JSON line: {"gparams_per_s": ..., "threads": ..., "n": ..., "steps": ...}.
package main

import (
	"flag"
	"fmt"
	"runtime"
	"sync"
	"time"

	"gmoracle"
)

func main() {
	n := flag.Int("n", 1<<26, "parameters")
	steps := flag.Int("steps", 5, "timed steps")
	threads := flag.Int("threads", runtime.NumCPU(), "goroutines, one contiguous slice each")
	flag.Parse()

	w := make([]float32, *n)
	g := make([]float32, *n)
	m := make([]float32, *n)
	v := make([]float32, *n)
	state := uint64(0x5EED601D)
	for i := range w {
		state = state*6364136223846793005 + 1442695040888963407
		w[i] = (float32(state>>40)/float32(1<<24) - 0.5) * 0.08
		state = state*6364136223846793005 + 1442695040888963407
		g[i] = (float32(state>>40)/float32(1<<24) - 0.5) * 0.02
	}
	per := (*n + *threads - 1) / *threads
	run := func(step int) {
		var wg sync.WaitGroup
		for t := 0; t < *threads; t++ {
			lo := t * per
			if lo >= *n {
				break
			}
			hi := lo + per
			if hi > *n {
				hi = *n
			}
			wg.Add(1)
			go func(lo, hi int) {
				defer wg.Done()
				gmoracle.AdamStep(w[lo:hi], g[lo:hi], m[lo:hi], v[lo:hi], 1e-3, 0.9, 0.999, 1e-8, 0, step)
			}(lo, hi)
		}
		wg.Wait()
	}
	run(1) // warm-up, also touches every page
	t0 := time.Now()
	for s := 0; s < *steps; s++ {
		run(2 + s)
	}
	dt := time.Since(t0).Seconds()
	fmt.Printf("{\"gparams_per_s\": %.4f, \"threads\": %d, \"n\": %d, \"steps\": %d}\n",
		float64(*n)*float64(*steps)/dt/1e9, *threads, *n, *steps)
}

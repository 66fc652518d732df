// gm_selftest.cu -- exhaustive self-check of the constant-divisor division.
//
// div_const (gm_apply.cuh) replaces __fdiv_rn(a, c) for a divisor c that is the
// same for a whole launch.  It must return the same bits for every a.  This
// entry runs both over all 2^32 bit patterns of a for one c and counts the
// patterns on which they differ (two NaN results count as equal).
#include "gm_apply.cuh"

namespace gm {

__global__ void __launch_bounds__(256)
const_div_selftest_kernel(const float c, const float r, unsigned long long* __restrict__ mismatches,
                          unsigned int* __restrict__ first_bad) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long bad = 0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < (1ull << 32); i += stride) {
        const float a = __uint_as_float((unsigned)i);
        const float want = __fdiv_rn(a, c);
        const float got = div_const(a, c, r);
        const bool same = (__float_as_uint(want) == __float_as_uint(got)) || (want != want && got != got);
        if (!same) { bad++; atomicMin(first_bad, (unsigned)i); }
    }
    if (bad) atomicAdd(mismatches, bad);
}

}  // namespace gm

using namespace gm;

extern "C" int gm_selftest_const_div(uintptr_t device_ptr, float c, uint64_t* mismatches, uint32_t* first_bad_bits,
                                     int* fast_path_allowed) {
    Device* d = as_device(device_ptr);
    if (!d) return GM_ERR_NIL_DEVICE;
    if (!mismatches) { set_error("output is nil"); return GM_ERR_BAD_ARG; }
    if (fast_path_allowed) *fast_path_allowed = const_div_ok(c) ? 1 : 0;
    if (!const_div_ok(c)) {                        // the kernels then use the IEEE division itself
        *mismatches = 0;
        if (first_bad_bits) *first_bad_bits = 0xffffffffu;
        return GM_OK;
    }
    DeviceGuard g(d);
    unsigned long long* d_count = reinterpret_cast<unsigned long long*>(d->scalars + 32);
    unsigned int* d_first = reinterpret_cast<unsigned int*>(d->scalars + 34);
    const unsigned long long zero = 0;
    const unsigned int ones = 0xffffffffu;
    GM_CUDA_CHECK(cudaMemcpyAsync(d_count, &zero, sizeof(zero), cudaMemcpyHostToDevice, d->stream));
    GM_CUDA_CHECK(cudaMemcpyAsync(d_first, &ones, sizeof(ones), cudaMemcpyHostToDevice, d->stream));
    const float r = 1.0f / c;                      // IEEE division on the host: the correctly rounded reciprocal
    const_div_selftest_kernel<<<d->sm_count * 16, 256, 0, d->stream>>>(c, r, d_count, d_first);
    d->launches++;
    GM_CUDA_CHECK(cudaGetLastError());
    GM_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    unsigned long long count = 0;
    unsigned int first = 0;
    GM_CUDA_CHECK(cudaMemcpy(&count, d_count, sizeof(count), cudaMemcpyDeviceToHost));
    GM_CUDA_CHECK(cudaMemcpy(&first, d_first, sizeof(first), cudaMemcpyDeviceToHost));
    *mismatches = count;
    if (first_bad_bits) *first_bad_bits = first;
    return GM_OK;
}

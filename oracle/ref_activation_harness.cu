// Builds the reference's OWN activation kernel for B200, for the tests only.
// TEST INFRASTRUCTURE: nothing in the product links or loads the result.
//
// The reference's sm120_activation_kernel<T>
// (src/cuda_kernels/sm120_pure_kernels.cu:128-176) is a template without an
// instantiation; its launcher (src/cuda_kernels/sm120_c_interface.cu:139-164)
// sits in a file that does not compile (:178).  This harness includes the
// reference source where it lies (the Makefile passes its directory with -I;
// no reference code is copied into this repository), instantiates that one
// kernel for float and half, and launches it the way the reference launcher
// does: 1024 threads per block, one element per thread.
// Nothing else of that file is instantiated: its matmul kernel reads B with
// 16-byte loads at addresses that are misaligned for most shapes (:41-47), and
// its attention kernel writes seq_len scores into a 256-entry shared array
// (:371,381-392); neither is ever launched here.
//
// Built without --use_fast_math (the reference's own build turns it on,
// CMakeLists.txt:43,47), so the formulas are compared at full accuracy.
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include "sm120_pure_kernels.cu"

extern "C" int sm120_reference_activation(const void* input, void* output, int size, int activation_type, int is_half) {
    if (size <= 0) return 0;
    const dim3 block(1024);
    const dim3 grid((size + 1023) / 1024);
    if (is_half)
        sm120_activation_kernel<half><<<grid, block>>>(static_cast<const half*>(input), static_cast<half*>(output), size, activation_type);
    else
        sm120_activation_kernel<float><<<grid, block>>>(static_cast<const float*>(input), static_cast<float*>(output), size, activation_type);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    return static_cast<int>(cudaDeviceSynchronize());
}

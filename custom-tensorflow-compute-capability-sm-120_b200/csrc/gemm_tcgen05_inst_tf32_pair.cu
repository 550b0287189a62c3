// Instantiates tensor-core GEMM variants (see gemm_tcgen05_kernel.cuh); one of several files so that
// the variants compile in parallel.
#include "gemm_tcgen05_kernel.cuh"

namespace sm120 {
template cudaError_t launch_variant<KIND_TF32, 128, 4, 2>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const DestMaps&,
                                                        const TcParams&, int, int, cudaStream_t, bool);
}  // namespace sm120

// Interface between the C-ABI translation unit and the kernels compiled in other units.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

namespace fk_w4a16 {

struct GemvParams;

struct UmmaLaunch {
  int group_size;   // 32, 64 or 128
  int rows;         // rows per pass: 1, 2, 4, 8 or 16
  bool bf16;
  int grid_x;       // CTAs = runs of the packet stream
  int row_tiles;
  size_t smem_bytes;
  int max_smem;     // opt-in limit of the device
  bool programmatic;  // launch with programmatic stream serialisation
  cudaStream_t stream;
};

// The pipelined tcgen05 / tensor-memory kernel (w4a16_gemm_umma.cuh).
cudaError_t launch_umma_kernel(const GemvParams& params, const UmmaLaunch& launch);

}  // namespace fk_w4a16

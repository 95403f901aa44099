// Host-side face of the kernel instantiations: one translation unit per (head_dim, page format)
// holds the 8 kernels of that pair (keys rotated or not x 4 head tiles), so that the build
// compiles them in parallel.
#pragma once

#include <cuda_runtime.h>

#include "page_decode_kernel.cuh"

namespace fk_page_decode {

struct Variant {
  int head_dim;
  int kv_format;
  bool keys_are_rotated;
  int group_tile;
  bool tensor_cores = false;  // the mma.sync form: rotated keys, tiles of 8 only
};

// Dynamic shared memory of a launch, or -1 for an unknown variant.
int variant_shared_bytes(const Variant& v, int warps, int stages);
cudaError_t launch_variant(const Variant& v, const DecodeParams& params, int blocks, int warps, int stages,
                           cudaStream_t stream);

#define FK_PAGE_DECODE_DECLARE_SHAPE(NAME)                                                              \
  int shared_bytes_##NAME(bool rotated, int group_tile, int warps, int stages);                        \
  cudaError_t launch_##NAME(bool rotated, int group_tile, const DecodeParams& params, int blocks,      \
                            int warps, int stages, cudaStream_t stream);
FK_PAGE_DECODE_DECLARE_SHAPE(d64_bf16)
FK_PAGE_DECODE_DECLARE_SHAPE(d64_fp8)
FK_PAGE_DECODE_DECLARE_SHAPE(d64_int8)
FK_PAGE_DECODE_DECLARE_SHAPE(d128_bf16)
FK_PAGE_DECODE_DECLARE_SHAPE(d128_fp8)
FK_PAGE_DECODE_DECLARE_SHAPE(d128_int8)
#undef FK_PAGE_DECODE_DECLARE_SHAPE
#define FK_PAGE_DECODE_DECLARE_MMA(NAME)                            \
  int shared_bytes_mma_##NAME(int warps, int stages);               \
  cudaError_t launch_mma_##NAME(const DecodeParams& params, int blocks, int warps, int stages, cudaStream_t stream);
FK_PAGE_DECODE_DECLARE_MMA(d64_bf16)
FK_PAGE_DECODE_DECLARE_MMA(d64_fp8)
FK_PAGE_DECODE_DECLARE_MMA(d64_int8)
FK_PAGE_DECODE_DECLARE_MMA(d128_bf16)
FK_PAGE_DECODE_DECLARE_MMA(d128_fp8)
FK_PAGE_DECODE_DECLARE_MMA(d128_int8)
#undef FK_PAGE_DECODE_DECLARE_MMA

}  // namespace fk_page_decode

// Host-side face of the kernel instantiations: one translation unit per (head_dim, page_size)
// holds the 24 kernels of that shape (3 page formats x keys rotated or not x 4 head tiles), so
// that the build compiles them in parallel.
#pragma once

#include <cuda_runtime.h>

#include "page_decode_kernel.cuh"

namespace fk_page_decode {

struct Variant {
  int head_dim;
  int page_size;
  int kv_format;
  bool keys_are_rotated;
  int group_tile;
};

// Dynamic shared memory of a launch, or -1 for an unknown variant.
int variant_shared_bytes(const Variant& v, int warps, int stages);
// Bytes one ring stage holds (keys + values + value scales of one page and kv head).
int variant_stage_bytes(const Variant& v);
cudaError_t launch_variant(const Variant& v, const DecodeParams& params, int blocks, int warps, int stages,
                           cudaStream_t stream);

#define FK_PAGE_DECODE_DECLARE_SHAPE(NAME)                                                                   \
  int shared_bytes_##NAME(int kv_format, bool rotated, int group_tile, int warps, int stages);              \
  int stage_bytes_##NAME(int kv_format);                                                                    \
  cudaError_t launch_##NAME(int kv_format, bool rotated, int group_tile, const DecodeParams& params,        \
                            int blocks, int warps, int stages, cudaStream_t stream);
FK_PAGE_DECODE_DECLARE_SHAPE(d64_p16)
FK_PAGE_DECODE_DECLARE_SHAPE(d64_p32)
FK_PAGE_DECODE_DECLARE_SHAPE(d128_p16)
FK_PAGE_DECODE_DECLARE_SHAPE(d128_p32)
#undef FK_PAGE_DECODE_DECLARE_SHAPE

}  // namespace fk_page_decode

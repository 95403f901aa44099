// Launches of the pipelined tcgen05 kernel, in a translation unit of their own so that the
// library's parts compile in parallel.
#include <cuda_runtime.h>

#include <mutex>
#include <type_traits>

#include "w4a16_gemm_umma.cuh"
#include "w4a16_launch.h"

namespace fk_w4a16 {
namespace {

constexpr int kMaxDevices = 64;

template <int G, int ROWS, class Mode>
cudaError_t launch_one(const GemvParams& params, const UmmaLaunch& launch) {
  auto kernel = w4a16_gemm_umma_kernel<G, ROWS, Mode>;
  static std::once_flag optin_flags[kMaxDevices];
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    return err;
  }
  if (device < 0 || device >= kMaxDevices) {
    return cudaErrorInvalidDevice;
  }
  std::call_once(optin_flags[device], [&] {
    cudaFuncAttributes attrs{};
    err = cudaFuncGetAttributes(&attrs, kernel);
    if (err == cudaSuccess) {
      err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 launch.max_smem - static_cast<int>(attrs.sharedSizeBytes));
    }
  });
  if (err != cudaSuccess) {
    return err;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(launch.grid_x), static_cast<unsigned>(launch.row_tiles), 1);
  config.blockDim = dim3(static_cast<unsigned>(kUmmaThreads));
  config.dynamicSmemBytes = launch.smem_bytes;
  config.stream = launch.stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = launch.programmatic ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, params);
}

template <int G, class Mode>
cudaError_t launch_rows(const GemvParams& params, const UmmaLaunch& launch) {
  switch (launch.rows) {
    case 1: return launch_one<G, 1, Mode>(params, launch);
    case 2: return launch_one<G, 2, Mode>(params, launch);
    case 4: return launch_one<G, 4, Mode>(params, launch);
    case 8: return launch_one<G, 8, Mode>(params, launch);
    default: return launch_one<G, 16, Mode>(params, launch);
  }
}

template <class Mode>
cudaError_t launch_group(const GemvParams& params, const UmmaLaunch& launch) {
  switch (launch.group_size) {
    case 32: return launch_rows<32, Mode>(params, launch);
    case 64: return launch_rows<64, Mode>(params, launch);
    default: return launch_rows<128, Mode>(params, launch);
  }
}

}  // namespace

cudaError_t launch_umma_kernel(const GemvParams& params, const UmmaLaunch& launch) {
  return launch.bf16 ? launch_group<UnpackBF16>(params, launch) : launch_group<UnpackF16>(params, launch);
}

#ifdef FK_W4A16_UMMA_TRACE
// Tuning builds only: copies CTA 0's per-packet timeline to a host buffer.
extern "C" __attribute__((visibility("default"))) int fk_w4a16_umma_trace_read(long long* host) {
  if (cudaDeviceSynchronize() != cudaSuccess) {
    return -2;
  }
  return cudaMemcpyFromSymbol(host, g_umma_trace, sizeof(long long) * kUmmaTracePackets * 8) == cudaSuccess ? 0 : -2;
}
#endif

}  // namespace fk_w4a16

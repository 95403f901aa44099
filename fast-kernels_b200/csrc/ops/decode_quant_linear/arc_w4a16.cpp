// C++ launchers: the reference's op names over the C ABI of libfk_w4a16.so.
#include "ops/decode_quant_linear/arc_w4a16.h"

#include <cuda_runtime_api.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

#include "fk_w4a16.h"

namespace fast_kernels::decode_quant_linear {
namespace {

void raise_if_failed(int code) {
  if (code == FK_W4A16_OK) {
    return;
  }
  const std::string message = fk_w4a16_last_error();
  if (code == FK_W4A16_ERR_INVALID_ARGUMENT) {
    throw std::invalid_argument(message);
  }
  throw std::runtime_error(message);
}

void* as_ptr(std::uintptr_t value) { return reinterpret_cast<void*>(value); }

// The reference's arc_w4a16_forward has no scratch parameter, so this layer keeps one workspace
// per (device, stream): calls on one stream are ordered and can share it, calls on different
// streams may overlap and must not. Buffers are allocated on first use (cudaMalloc: make that
// first call outside any stream capture), only ever grow, and live until the process ends.
struct OwnedWorkspace {
  void* ptr = nullptr;
  std::size_t bytes = 0;
};

OwnedWorkspace workspace_for(std::size_t need, cudaStream_t stream) {
  static std::mutex mutex;
  static std::map<std::pair<int, cudaStream_t>, OwnedWorkspace> table;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    throw std::runtime_error("cudaGetDevice failed");
  }
  std::lock_guard<std::mutex> lock(mutex);
  OwnedWorkspace& slot = table[{device, stream}];
  if (slot.bytes < need) {
    // Round up generously so shape changes rarely reallocate. The old buffer is left alive:
    // kernels already enqueued may still be using it.
    const std::size_t bytes = need < (std::size_t{4} << 20) ? (std::size_t{4} << 20) : need * 2;
    void* fresh = nullptr;
    cudaError_t err = cudaMalloc(&fresh, bytes);
    if (err == cudaSuccess) {
      err = cudaMemsetAsync(fresh, 0, bytes, stream);
    }
    if (err != cudaSuccess) {
      throw std::runtime_error(std::string("workspace allocation failed: ") +
                               cudaGetErrorString(err));
    }
    slot.ptr = fresh;
    slot.bytes = bytes;
  }
  return slot;
}

}  // namespace

void pack_arc_w4a16_packets(std::uintptr_t q_ptr, std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                            std::uintptr_t packets_ptr, int n, int k, int group_size,
                            int packet_stride_bytes, std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_pack_packets(as_ptr(q_ptr), as_ptr(alpha_ptr), as_ptr(beta_ptr),
                                        as_ptr(packets_ptr), n, k, group_size, packet_stride_bytes,
                                        as_ptr(stream_ptr)));
}

void compute_arc_w4a16_group_sums(std::uintptr_t activations_ptr, std::uintptr_t sums_ptr,
                                  int batch, int k, int group_size, std::uintptr_t stream_ptr) {
  compute_arc_w4a16_group_sums_typed(activations_ptr, sums_ptr, batch, k, group_size,
                                     kElementFloat16, stream_ptr);
}

void arc_w4a16_forward(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                       std::uintptr_t /*group_sums_ptr*/, std::uintptr_t output_ptr, int batch,
                       int n, int k, int group_size, int packet_stride_bytes,
                       std::uintptr_t stream_ptr) {
  const std::size_t need = fk_w4a16_workspace_bytes(batch, n, k, group_size);
  if (need == 0) {
    throw std::invalid_argument(fk_w4a16_last_error());  // the dimension rule that failed
  }
  const OwnedWorkspace ws = workspace_for(need, reinterpret_cast<cudaStream_t>(stream_ptr));
  raise_if_failed(fk_w4a16_gemv(as_ptr(activations_ptr), as_ptr(packets_ptr), as_ptr(output_ptr),
                                ws.ptr, ws.bytes, batch, n, k, group_size, packet_stride_bytes,
                                FK_W4A16_DTYPE_F16, as_ptr(stream_ptr)));
}

void arc_w4a16_forward_split_k(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                               std::uintptr_t /*group_sums_ptr*/, std::uintptr_t partials_ptr,
                               int batch, int n, int k, int group_size, int packet_stride_bytes,
                               int split_k_slices, std::uintptr_t stream_ptr) {
  arc_w4a16_forward_split_k_typed(activations_ptr, packets_ptr, partials_ptr, batch, n, k,
                                  group_size, packet_stride_bytes, split_k_slices, kElementFloat16,
                                  stream_ptr);
}

void reduce_arc_w4a16_split_k_partials(std::uintptr_t partials_ptr, std::uintptr_t output_ptr,
                                       int batch, int n, int split_k_slices,
                                       std::uintptr_t stream_ptr) {
  reduce_arc_w4a16_split_k_partials_typed(partials_ptr, output_ptr, batch, n, split_k_slices,
                                          kElementFloat16, stream_ptr);
}

void dequant_w4a16_to_fp16(std::uintptr_t q_ptr, std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                           std::uintptr_t output_ptr, int n, int k, int group_size,
                           std::uintptr_t stream_ptr) {
  dequant_w4a16_typed(q_ptr, alpha_ptr, beta_ptr, output_ptr, n, k, group_size, kElementFloat16,
                      stream_ptr);
}

void dequant_arc_w4a16_packets_to_fp16(std::uintptr_t packets_ptr, std::uintptr_t output_ptr, int n,
                                       int k, int group_size, int packet_stride_bytes,
                                       std::uintptr_t stream_ptr) {
  dequant_arc_w4a16_packets_typed(packets_ptr, output_ptr, n, k, group_size, packet_stride_bytes,
                                  kElementFloat16, stream_ptr);
}

void cublaslt_fp16_with_weight(std::uintptr_t activations_ptr, std::uintptr_t weight_ptr,
                               std::uintptr_t output_ptr, std::uintptr_t workspace_ptr,
                               std::size_t workspace_bytes, int batch, int n, int k,
                               std::uintptr_t stream_ptr) {
  cublaslt_with_weight_typed(activations_ptr, weight_ptr, output_ptr, workspace_ptr,
                             workspace_bytes, batch, n, k, kElementFloat16, stream_ptr);
}

void cublaslt_fp16_after_packet_dequant(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                                        std::uintptr_t output_ptr, std::uintptr_t weight_ptr,
                                        std::uintptr_t workspace_ptr, std::size_t workspace_bytes,
                                        int batch, int n, int k, int group_size,
                                        int packet_stride_bytes, std::uintptr_t stream_ptr) {
  if (batch <= 0) {
    throw std::invalid_argument("batch and k must be positive");
  }
  dequant_arc_w4a16_packets_to_fp16(packets_ptr, weight_ptr, n, k, group_size, packet_stride_bytes,
                                    stream_ptr);
  cublaslt_fp16_with_weight(activations_ptr, weight_ptr, output_ptr, workspace_ptr, workspace_bytes,
                            batch, n, k, stream_ptr);
}

void cublaslt_fp16_after_dequant(std::uintptr_t activations_ptr, std::uintptr_t q_ptr,
                                 std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                                 std::uintptr_t output_ptr, std::uintptr_t weight_ptr,
                                 std::uintptr_t workspace_ptr, std::size_t workspace_bytes,
                                 int batch, int n, int k, int group_size,
                                 std::uintptr_t stream_ptr) {
  if (batch <= 0) {
    throw std::invalid_argument("batch and k must be positive");
  }
  dequant_w4a16_to_fp16(q_ptr, alpha_ptr, beta_ptr, weight_ptr, n, k, group_size, stream_ptr);
  cublaslt_fp16_with_weight(activations_ptr, weight_ptr, output_ptr, workspace_ptr, workspace_bytes,
                            batch, n, k, stream_ptr);
}

// ---- additions ---------------------------------------------------------------------------------

std::size_t arc_w4a16_workspace_bytes(int batch, int n, int k, int group_size) {
  const std::size_t need = fk_w4a16_workspace_bytes(batch, n, k, group_size);
  if (need == 0) {
    throw std::invalid_argument(fk_w4a16_last_error());
  }
  return need;
}

void arc_w4a16_forward_fused(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                             std::uintptr_t output_ptr, std::uintptr_t workspace_ptr,
                             std::size_t workspace_bytes, int batch, int n, int k, int group_size,
                             int packet_stride_bytes, int element_type, std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_gemv(as_ptr(activations_ptr), as_ptr(packets_ptr), as_ptr(output_ptr),
                                as_ptr(workspace_ptr), workspace_bytes, batch, n, k, group_size,
                                packet_stride_bytes, element_type, as_ptr(stream_ptr)));
}

void compute_arc_w4a16_group_sums_typed(std::uintptr_t activations_ptr, std::uintptr_t sums_ptr,
                                        int batch, int k, int group_size, int element_type,
                                        std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_group_sums(as_ptr(activations_ptr), static_cast<float*>(as_ptr(sums_ptr)),
                                      batch, k, group_size, element_type, as_ptr(stream_ptr)));
}

void arc_w4a16_forward_split_k_typed(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                                     std::uintptr_t partials_ptr, int batch, int n, int k,
                                     int group_size, int packet_stride_bytes, int split_k_slices,
                                     int element_type, std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_gemv_split_k(as_ptr(activations_ptr), as_ptr(packets_ptr),
                                        static_cast<float*>(as_ptr(partials_ptr)), batch, n, k,
                                        group_size, packet_stride_bytes, split_k_slices,
                                        element_type, as_ptr(stream_ptr)));
}

void reduce_arc_w4a16_split_k_partials_typed(std::uintptr_t partials_ptr,
                                             std::uintptr_t output_ptr, int batch, int n,
                                             int split_k_slices, int element_type,
                                             std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_reduce_partials(static_cast<const float*>(as_ptr(partials_ptr)),
                                           as_ptr(output_ptr), batch, n, split_k_slices,
                                           element_type, as_ptr(stream_ptr)));
}

void dequant_w4a16_typed(std::uintptr_t q_ptr, std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                         std::uintptr_t output_ptr, int n, int k, int group_size, int element_type,
                         std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_dequant_rowmajor(as_ptr(q_ptr), as_ptr(alpha_ptr), as_ptr(beta_ptr),
                                            as_ptr(output_ptr), n, k, group_size, element_type,
                                            as_ptr(stream_ptr)));
}

void dequant_arc_w4a16_packets_typed(std::uintptr_t packets_ptr, std::uintptr_t output_ptr, int n,
                                     int k, int group_size, int packet_stride_bytes,
                                     int element_type, std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_dequant_packets(as_ptr(packets_ptr), as_ptr(output_ptr), n, k,
                                           group_size, packet_stride_bytes, element_type,
                                           as_ptr(stream_ptr)));
}

void cublaslt_with_weight_typed(std::uintptr_t activations_ptr, std::uintptr_t weight_ptr,
                                std::uintptr_t output_ptr, std::uintptr_t workspace_ptr,
                                std::size_t workspace_bytes, int batch, int n, int k,
                                int element_type, std::uintptr_t stream_ptr) {
  raise_if_failed(fk_w4a16_cublaslt_matmul(as_ptr(activations_ptr), as_ptr(weight_ptr),
                                           as_ptr(output_ptr), as_ptr(workspace_ptr),
                                           workspace_bytes, batch, n, k, element_type,
                                           as_ptr(stream_ptr)));
}

int arc_w4a16_device_status() {
  int status = 0;
  raise_if_failed(fk_w4a16_device_status(&status));
  return status;
}

}  // namespace fast_kernels::decode_quant_linear

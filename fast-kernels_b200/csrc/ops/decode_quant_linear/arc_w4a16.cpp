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
// streams may overlap and must not. The rule for callers:
//   * the FIRST call on a (device, stream) pair allocates the pair's workspace (cudaMalloc, one
//     buffer of kFixedWorkspaceBytes, enough for every layer shape at batches up to 16) -- make
//     that call outside stream capture; every later call allocates nothing and can be captured;
//   * a problem that needs more than that (batches far above 16) makes the buffer grow: the
//     stream is synchronised, the old buffer freed, a larger one allocated. Never under capture:
//     there the call fails with std::runtime_error instead.
// Buffers live until the process ends.
constexpr std::size_t kFixedWorkspaceBytes = std::size_t{16} << 20;

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
  if (slot.bytes >= need) {
    return slot;
  }
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) {
    (void)cudaGetLastError();
    capture = cudaStreamCaptureStatusNone;
  }
  if (capture != cudaStreamCaptureStatusNone) {
    throw std::runtime_error(
        "arc_w4a16_forward: this stream's workspace is not allocated yet (or too small) and the "
        "stream is being captured; make one call with this problem size outside capture first");
  }
  if (slot.ptr != nullptr) {
    // Kernels already enqueued on this stream may still use the old buffer.
    cudaError_t err = cudaStreamSynchronize(stream);
    if (err == cudaSuccess) {
      err = cudaFree(slot.ptr);
    }
    if (err != cudaSuccess) {
      throw std::runtime_error(std::string("workspace release failed: ") + cudaGetErrorString(err));
    }
    slot = OwnedWorkspace{};
  }
  const std::size_t bytes = need <= kFixedWorkspaceBytes ? kFixedWorkspaceBytes : need + (need / 2);
  void* fresh = nullptr;
  cudaError_t err = cudaMalloc(&fresh, bytes);
  if (err == cudaSuccess) {
    err = cudaMemsetAsync(fresh, 0, bytes, stream);
    if (err != cudaSuccess) {
      (void)cudaFree(fresh);
    }
  }
  if (err != cudaSuccess) {
    throw std::runtime_error(std::string("workspace allocation failed: ") + cudaGetErrorString(err));
  }
  slot.ptr = fresh;
  slot.bytes = bytes;
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

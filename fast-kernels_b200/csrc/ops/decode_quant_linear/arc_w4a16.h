// C++ op surface of the W4A16 decode path.
//
// The first ten functions keep the names, parameter order and meaning of the reference's
// csrc/ops/decode_quant_linear/arc_w4a16.h:8-52 (SamMausberg/fast-kernels), so code written
// against that header links against this library unchanged: every pointer is a device address
// passed as std::uintptr_t, `stream_ptr` is a cudaStream_t (0 = default stream), work is
// asynchronous on that stream, argument errors throw std::invalid_argument and CUDA / cuBLAS
// failures throw std::runtime_error("<call> failed: <reason>").
//
// Differences a caller can observe:
//   * fp16 entry points accept group_size 32 in addition to 64 and 128;
//   * arc_w4a16_forward ignores `group_sums_ptr` (the kernel derives the sums itself; the pointer
//     may be 0) and finishes split-K inside its single launch;
//   * the functions below the divider are additions (bf16, explicit workspace).
//
// Everything forwards to the C ABI in include/fk_w4a16.h; this layer only translates status codes
// into exceptions and owns the scratch that the reference signature has no parameter for.
#pragma once

#include <cstddef>
#include <cstdint>

namespace fast_kernels::decode_quant_linear {

// ---- reference-compatible surface (fp16) ---------------------------------------------------

// q_u8[n, k/2], alpha/beta[n, k/group_size] -> ARC packets [(n/128)*(k/group_size), stride].
void pack_arc_w4a16_packets(std::uintptr_t q_ptr, std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                            std::uintptr_t packets_ptr, int n, int k, int group_size,
                            int packet_stride_bytes, std::uintptr_t stream_ptr);

// sums[batch, k/group_size] = fp32 per-group sums of the activations.
void compute_arc_w4a16_group_sums(std::uintptr_t activations_ptr, std::uintptr_t sums_ptr,
                                  int batch, int k, int group_size, std::uintptr_t stream_ptr);

// output[batch, n] = activations[batch, k] . W^T, one launch.
void arc_w4a16_forward(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                       std::uintptr_t group_sums_ptr, std::uintptr_t output_ptr, int batch, int n,
                       int k, int group_size, int packet_stride_bytes, std::uintptr_t stream_ptr);

// partials[split_k_slices, batch, n] (fp32), slice s = groups [s * ceil(NG / S), ...).
void arc_w4a16_forward_split_k(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                               std::uintptr_t group_sums_ptr, std::uintptr_t partials_ptr,
                               int batch, int n, int k, int group_size, int packet_stride_bytes,
                               int split_k_slices, std::uintptr_t stream_ptr);

// output[batch, n] = fp16(sum of the slices, in slice order).
void reduce_arc_w4a16_split_k_partials(std::uintptr_t partials_ptr, std::uintptr_t output_ptr,
                                       int batch, int n, int split_k_slices,
                                       std::uintptr_t stream_ptr);

// output[n, k] = fp16(alpha * q + beta) from row-major nibbles / from packets.
void dequant_w4a16_to_fp16(std::uintptr_t q_ptr, std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                           std::uintptr_t output_ptr, int n, int k, int group_size,
                           std::uintptr_t stream_ptr);
void dequant_arc_w4a16_packets_to_fp16(std::uintptr_t packets_ptr, std::uintptr_t output_ptr, int n,
                                       int k, int group_size, int packet_stride_bytes,
                                       std::uintptr_t stream_ptr);

// Vendor baseline subjects: cuBLASLt fp16 GEMM with fp32 compute on a dequantised weight.
void cublaslt_fp16_with_weight(std::uintptr_t activations_ptr, std::uintptr_t weight_ptr,
                               std::uintptr_t output_ptr, std::uintptr_t workspace_ptr,
                               std::size_t workspace_bytes, int batch, int n, int k,
                               std::uintptr_t stream_ptr);
void cublaslt_fp16_after_packet_dequant(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                                        std::uintptr_t output_ptr, std::uintptr_t weight_ptr,
                                        std::uintptr_t workspace_ptr, std::size_t workspace_bytes,
                                        int batch, int n, int k, int group_size,
                                        int packet_stride_bytes, std::uintptr_t stream_ptr);
void cublaslt_fp16_after_dequant(std::uintptr_t activations_ptr, std::uintptr_t q_ptr,
                                 std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                                 std::uintptr_t output_ptr, std::uintptr_t weight_ptr,
                                 std::uintptr_t workspace_ptr, std::size_t workspace_bytes,
                                 int batch, int n, int k, int group_size,
                                 std::uintptr_t stream_ptr);

// ---- additions ---------------------------------------------------------------------------------

// element_type: 0 = fp16, 1 = bf16 (activations, scales, offsets and outputs share it).
constexpr int kElementFloat16 = 0;
constexpr int kElementBFloat16 = 1;

// Scratch bytes arc_w4a16_forward_fused needs for a problem on the current device.
std::size_t arc_w4a16_workspace_bytes(int batch, int n, int k, int group_size);

// arc_w4a16_forward with caller-owned scratch (zero-filled once, reusable; one per concurrently
// running call) and a selectable element type. Allocates nothing.
void arc_w4a16_forward_fused(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                             std::uintptr_t output_ptr, std::uintptr_t workspace_ptr,
                             std::size_t workspace_bytes, int batch, int n, int k, int group_size,
                             int packet_stride_bytes, int element_type, std::uintptr_t stream_ptr);

void compute_arc_w4a16_group_sums_typed(std::uintptr_t activations_ptr, std::uintptr_t sums_ptr,
                                        int batch, int k, int group_size, int element_type,
                                        std::uintptr_t stream_ptr);
void arc_w4a16_forward_split_k_typed(std::uintptr_t activations_ptr, std::uintptr_t packets_ptr,
                                     std::uintptr_t partials_ptr, int batch, int n, int k,
                                     int group_size, int packet_stride_bytes, int split_k_slices,
                                     int element_type, std::uintptr_t stream_ptr);
void reduce_arc_w4a16_split_k_partials_typed(std::uintptr_t partials_ptr,
                                             std::uintptr_t output_ptr, int batch, int n,
                                             int split_k_slices, int element_type,
                                             std::uintptr_t stream_ptr);
void dequant_w4a16_typed(std::uintptr_t q_ptr, std::uintptr_t alpha_ptr, std::uintptr_t beta_ptr,
                         std::uintptr_t output_ptr, int n, int k, int group_size, int element_type,
                         std::uintptr_t stream_ptr);
void dequant_arc_w4a16_packets_typed(std::uintptr_t packets_ptr, std::uintptr_t output_ptr, int n,
                                     int k, int group_size, int packet_stride_bytes,
                                     int element_type, std::uintptr_t stream_ptr);
void cublaslt_with_weight_typed(std::uintptr_t activations_ptr, std::uintptr_t weight_ptr,
                                std::uintptr_t output_ptr, std::uintptr_t workspace_ptr,
                                std::size_t workspace_bytes, int batch, int n, int k,
                                int element_type, std::uintptr_t stream_ptr);

// Device status word of the current device (0 = no bounded device-side wait ever gave up).
// Synchronises the device.
int arc_w4a16_device_status();

}  // namespace fast_kernels::decode_quant_linear

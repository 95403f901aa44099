// The reference's op declaration for the paged-KV decode attention, name for name and argument
// for argument (csrc/ops/clustered_page_decode/clustered_page_decode.h:8-25 there), so that the
// pybind11 module and any C++ caller of the reference link against this build unchanged.
//
// Differences in meaning, none in signature:
//  * `use_clustered_kernel` = 0 runs one thread block per (request, kv head, head tile) and needs
//    no scratch; != 0 lets the launcher cut a request's pages over as many blocks as fill the
//    device (the reference's cluster of `cluster_size` blocks). `cluster_size` is validated
//    ([1, 8]) and otherwise only a hint: 1 keeps one block per task.
//  * group sizes above 8 work in both modes (the reference's direct kernel refuses them).
//  * the scratch for the split form is one buffer per (device, stream), allocated by the first
//    call on that stream -- make that call outside stream capture.
#pragma once

#include <cstddef>
#include <cstdint>

namespace fast_kernels::clustered_page_decode {

enum class KvFormat : int {
  kBFloat16 = 0,
  kFp8E4M3 = 1,
  kInt8 = 2,
};

void clustered_page_decode_forward(
    std::uintptr_t query_ptr, std::uintptr_t key_ptr, std::uintptr_t value_ptr,
    std::uintptr_t key_scales_ptr, std::uintptr_t value_scales_ptr,
    std::uintptr_t run_base_pages_ptr, std::uintptr_t run_page_counts_ptr,
    std::uintptr_t run_logical_starts_ptr, std::uintptr_t run_last_page_lens_ptr,
    std::uintptr_t request_run_offsets_ptr, std::uintptr_t seq_lens_ptr, std::uintptr_t output_ptr,
    int batch, int num_runs, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
    int group_tile, int use_clustered_kernel, int cluster_size, int kv_format,
    int keys_are_rotated, float softmax_scale, float rope_theta, std::uintptr_t stream_ptr);

// Additions of this build: the same call with the longest request's page count as a hint (it
// keeps short requests from being cut into empty pieces) and with the caller's word that the
// kernel before this one in the stream does not write the descriptor arrays (they may then be
// read while that kernel drains); and the device status word.
void clustered_page_decode_forward_hinted(
    std::uintptr_t query_ptr, std::uintptr_t key_ptr, std::uintptr_t value_ptr,
    std::uintptr_t key_scales_ptr, std::uintptr_t value_scales_ptr,
    std::uintptr_t run_base_pages_ptr, std::uintptr_t run_page_counts_ptr,
    std::uintptr_t run_logical_starts_ptr, std::uintptr_t run_last_page_lens_ptr,
    std::uintptr_t request_run_offsets_ptr, std::uintptr_t seq_lens_ptr, std::uintptr_t output_ptr,
    int batch, int num_runs, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
    int group_tile, int use_clustered_kernel, int cluster_size, int kv_format,
    int keys_are_rotated, float softmax_scale, float rope_theta, int max_pages_hint,
    int early_descriptors, std::uintptr_t stream_ptr);
int page_decode_device_status();

}  // namespace fast_kernels::clustered_page_decode

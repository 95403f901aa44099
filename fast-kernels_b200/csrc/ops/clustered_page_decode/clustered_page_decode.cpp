// C++ launcher: the reference's op name over the C ABI of libfk_page_decode.so.
#include "ops/clustered_page_decode/clustered_page_decode.h"

#include <cuda_runtime_api.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

#include "fk_page_decode.h"

namespace fast_kernels::clustered_page_decode {
namespace {

void raise_if_failed(int code) {
  if (code == FK_PAGE_DECODE_OK) {
    return;
  }
  const std::string message = fk_page_decode_last_error();
  if (code == FK_PAGE_DECODE_ERR_INVALID_ARGUMENT) {
    throw std::invalid_argument(message);
  }
  throw std::runtime_error(message);
}

template <typename T>
T* as(std::uintptr_t value) {
  return reinterpret_cast<T*>(value);
}

// The reference's entry point has no scratch parameter, so this layer keeps one workspace per
// (device, stream): calls on one stream are ordered and share it, calls on different streams may
// overlap and must not. The first split call on a pair allocates it (cudaMalloc + memset on that
// stream) -- outside stream capture; under capture that first call fails with std::runtime_error
// instead of allocating. The size does not depend on the problem. Buffers live until the process
// ends.
void* workspace_for(std::size_t bytes, cudaStream_t stream) {
  static std::mutex mutex;
  static std::map<std::pair<int, cudaStream_t>, void*> table;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    throw std::runtime_error("cudaGetDevice failed");
  }
  std::lock_guard<std::mutex> lock(mutex);
  void*& slot = table[{device, stream}];
  if (slot != nullptr) {
    return slot;
  }
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) {
    (void)cudaGetLastError();
    capture = cudaStreamCaptureStatusNone;
  }
  if (capture != cudaStreamCaptureStatusNone) {
    throw std::runtime_error(
        "clustered_page_decode_forward: this stream's workspace is not allocated yet and the stream is "
        "being captured; make one call outside capture first");
  }
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
  slot = fresh;
  return slot;
}

}  // namespace

void clustered_page_decode_forward_hinted(
    std::uintptr_t query_ptr, std::uintptr_t key_ptr, std::uintptr_t value_ptr,
    std::uintptr_t key_scales_ptr, std::uintptr_t value_scales_ptr,
    std::uintptr_t run_base_pages_ptr, std::uintptr_t run_page_counts_ptr,
    std::uintptr_t run_logical_starts_ptr, std::uintptr_t run_last_page_lens_ptr,
    std::uintptr_t request_run_offsets_ptr, std::uintptr_t seq_lens_ptr, std::uintptr_t output_ptr,
    int batch, int num_runs, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
    int group_tile, int use_clustered_kernel, int cluster_size, int kv_format,
    int keys_are_rotated, float softmax_scale, float rope_theta, int max_pages_hint,
    int early_descriptors, std::uintptr_t stream_ptr) {
  // the argument rules of the reference's launcher that have no counterpart in the C ABI
  // (clustered_page_decode.cu:1110-1115 there)
  if (cluster_size < 1 || cluster_size > 8) {
    throw std::invalid_argument("cluster_size must be in [1, 8]");
  }
  if (group_tile != 1 && group_tile != 2 && group_tile != 4 && group_tile != 8) {
    throw std::invalid_argument("group_tile must be one of {1, 2, 4, 8}");
  }
  fk_page_decode_args args{};
  args.query = as<const void>(query_ptr);
  args.key_pages = as<const void>(key_ptr);
  args.value_pages = as<const void>(value_ptr);
  args.key_scales = as<const float>(key_scales_ptr);
  args.value_scales = as<const float>(value_scales_ptr);
  args.run_base_pages = as<const int32_t>(run_base_pages_ptr);
  args.run_page_counts = as<const int32_t>(run_page_counts_ptr);
  args.run_logical_starts = as<const int32_t>(run_logical_starts_ptr);
  args.run_last_page_lens = as<const int32_t>(run_last_page_lens_ptr);
  args.request_run_offsets = as<const int32_t>(request_run_offsets_ptr);
  args.seq_lens = as<const int32_t>(seq_lens_ptr);
  args.output = as<void>(output_ptr);
  args.batch = batch;
  args.num_runs = num_runs;
  args.num_q_heads = num_q_heads;
  args.num_kv_heads = num_kv_heads;
  args.head_dim = head_dim;
  args.page_size = page_size;
  args.group_tile = group_tile;
  args.kv_format = kv_format;
  args.keys_are_rotated = keys_are_rotated;
  args.splits = (use_clustered_kernel == 0 || cluster_size == 1) ? 1 : 0;
  args.max_pages_hint = max_pages_hint;
  args.softmax_scale = softmax_scale;
  args.rope_theta = rope_theta;
  args.stream = as<void>(stream_ptr);
  args.flags = early_descriptors != 0 ? FK_PAGE_DECODE_FLAG_EARLY_DESCRIPTORS : 0;
  if (args.splits != 1 && batch > 0 && num_q_heads > 0 && num_kv_heads > 0 && (head_dim == 64 || head_dim == 128)) {
    args.workspace_bytes = fk_page_decode_workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim);
    args.workspace = workspace_for(args.workspace_bytes, reinterpret_cast<cudaStream_t>(stream_ptr));
  }
  raise_if_failed(fk_page_decode_forward(&args));
}

void clustered_page_decode_forward(
    std::uintptr_t query_ptr, std::uintptr_t key_ptr, std::uintptr_t value_ptr,
    std::uintptr_t key_scales_ptr, std::uintptr_t value_scales_ptr,
    std::uintptr_t run_base_pages_ptr, std::uintptr_t run_page_counts_ptr,
    std::uintptr_t run_logical_starts_ptr, std::uintptr_t run_last_page_lens_ptr,
    std::uintptr_t request_run_offsets_ptr, std::uintptr_t seq_lens_ptr, std::uintptr_t output_ptr,
    int batch, int num_runs, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
    int group_tile, int use_clustered_kernel, int cluster_size, int kv_format,
    int keys_are_rotated, float softmax_scale, float rope_theta, std::uintptr_t stream_ptr) {
  clustered_page_decode_forward_hinted(query_ptr, key_ptr, value_ptr, key_scales_ptr, value_scales_ptr,
                                       run_base_pages_ptr, run_page_counts_ptr, run_logical_starts_ptr,
                                       run_last_page_lens_ptr, request_run_offsets_ptr, seq_lens_ptr, output_ptr,
                                       batch, num_runs, num_q_heads, num_kv_heads, head_dim, page_size, group_tile,
                                       use_clustered_kernel, cluster_size, kv_format, keys_are_rotated,
                                       softmax_scale, rope_theta, /*max_pages_hint=*/0, /*early_descriptors=*/0, stream_ptr);
}

int page_decode_device_status() {
  int status = 0;
  raise_if_failed(fk_page_decode_device_status(&status));
  return status;
}

}  // namespace fast_kernels::clustered_page_decode

// C entry point around the reference's OWN paged-KV decode launcher (namespace
// fast_kernels::clustered_page_decode, csrc/ops/clustered_page_decode/clustered_page_decode.h:16-25),
// so that tests and the bench can run the unmodified reference kernels on the same inputs as the
// new library. TEST INFRASTRUCTURE ONLY: built into oracle/_ref/ from the reference sources where
// they lie; the shipped library never links or loads it.
#include <cstdint>
#include <cstring>
#include <exception>

#include "ops/clustered_page_decode/clustered_page_decode.h"

namespace ref = fast_kernels::clustered_page_decode;

static thread_local char g_error[512];

extern "C" {

const char* fkref_page_decode_last_error() { return g_error; }

int fkref_page_decode_forward(std::uintptr_t query, std::uintptr_t keys, std::uintptr_t values,
                              std::uintptr_t key_scales, std::uintptr_t value_scales, std::uintptr_t run_base_pages,
                              std::uintptr_t run_page_counts, std::uintptr_t run_logical_starts,
                              std::uintptr_t run_last_page_lens, std::uintptr_t request_run_offsets,
                              std::uintptr_t seq_lens, std::uintptr_t output, int batch, int num_runs, int num_q_heads,
                              int num_kv_heads, int head_dim, int page_size, int group_tile, int use_clustered_kernel,
                              int cluster_size, int kv_format, int keys_are_rotated, float softmax_scale,
                              float rope_theta, std::uintptr_t stream) {
  try {
    ref::clustered_page_decode_forward(query, keys, values, key_scales, value_scales, run_base_pages, run_page_counts,
                                       run_logical_starts, run_last_page_lens, request_run_offsets, seq_lens, output,
                                       batch, num_runs, num_q_heads, num_kv_heads, head_dim, page_size, group_tile,
                                       use_clustered_kernel, cluster_size, kv_format, keys_are_rotated, softmax_scale,
                                       rope_theta, stream);
    g_error[0] = '\0';
    return 0;
  } catch (const std::exception& e) {
    std::strncpy(g_error, e.what(), sizeof(g_error) - 1);
    g_error[sizeof(g_error) - 1] = '\0';
    return -1;
  }
}

}  // extern "C"

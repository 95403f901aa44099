// The reference's op declaration for the shared-prefix paged decode, name for name and argument
// for argument (csrc/ops/prefix_union_decode/prefix_union_decode.h:8-17 there).
//
// No union kernel is built for sm_100a. The reference's own launcher refuses every device below
// compute capability 12 with std::invalid_argument
// (csrc/kernels/prefix_union_decode/prefix_union_decode.cu:843-846 there) and its Python op never
// reaches it on such a device: it computes the op with clustered_page_decode on the plan's
// fallback. This function keeps that contract -- nothing to do for zero tasks, std::invalid_argument
// otherwise -- so that the module exports the name and callers see the error they would see from
// the reference on a B200.
#pragma once

#include <cstddef>
#include <cstdint>

namespace fast_kernels::prefix_union_decode {

void prefix_union_decode_forward(
    std::uintptr_t query_ptr, std::uintptr_t key_ptr, std::uintptr_t value_ptr,
    std::uintptr_t key_scales_ptr, std::uintptr_t value_scales_ptr, std::uintptr_t tasks_ptr,
    std::uintptr_t shared_pages_ptr, std::uintptr_t tail_pages_ptr, std::uintptr_t consumers_ptr,
    std::uintptr_t scheduler_counter_ptr, std::uintptr_t output_ptr, int num_tasks, int num_pages,
    int num_q_heads, int num_kv_heads, int head_dim, int page_size, int cluster_size,
    int kv_format, int keys_are_rotated, float softmax_scale, float rope_theta,
    std::uintptr_t stream_ptr);

}  // namespace fast_kernels::prefix_union_decode

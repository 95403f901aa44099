// pybind11 module fast_kernels._native.
//
// Exposes the W4A16 ops under the names and keyword arguments of the reference's module
// (csrc/bindings/python_module.cpp:15-27 for build_info, :119-240 for the ops): each function
// takes raw device addresses and a stream handle, releases the GIL for the call, and maps
// std::invalid_argument to ValueError and std::runtime_error to RuntimeError (pybind11's default
// translation). Names below the divider are additions of this build.
#include <pybind11/pybind11.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "ops/clustered_page_decode/clustered_page_decode.h"
#include "ops/decode_quant_linear/arc_w4a16.h"
#include "ops/prefix_union_decode/prefix_union_decode.h"

#ifndef FK_COMPILED_WITH_CUDA
#define FK_COMPILED_WITH_CUDA 1
#endif
#if FK_COMPILED_WITH_CUDA
#include "fk_w4a16.h"
#endif

namespace py = pybind11;
namespace dql = fast_kernels::decode_quant_linear;
using ptr_t = std::uintptr_t;

#ifndef FK_PROJECT_VERSION
#define FK_PROJECT_VERSION "0.0.0"
#endif
#ifndef FK_CXX_COMPILER_ID
#define FK_CXX_COMPILER_ID "unknown"
#endif
#ifndef FK_CXX_COMPILER_VERSION
#define FK_CXX_COMPILER_VERSION "unknown"
#endif
#ifndef FK_CUDA_COMPILER_VERSION
#define FK_CUDA_COMPILER_VERSION "unknown"
#endif
#ifndef FK_CUDA_ARCHITECTURES
#define FK_CUDA_ARCHITECTURES "100a"
#endif

PYBIND11_MODULE(_native, m) {
  m.doc() = "fast-kernels native module: sm_100a W4A16 decode GEMV and paged-KV decode attention";

  m.def("build_info", []() {
    py::dict info;
    info["project_version"] = std::string(FK_PROJECT_VERSION);
    info["compiled_with_cuda"] = FK_COMPILED_WITH_CUDA != 0;
    info["cxx_compiler_id"] = std::string(FK_CXX_COMPILER_ID);
    info["cxx_compiler_version"] = std::string(FK_CXX_COMPILER_VERSION);
    info["cuda_compiler_version"] = std::string(FK_CUDA_COMPILER_VERSION);
    info["cuda_architectures"] = std::string(FK_CUDA_ARCHITECTURES);
#if FK_COMPILED_WITH_CUDA
    info["kernel_library_version"] = std::string(fk_w4a16_version());
#else
    info["kernel_library_version"] = std::string("none");
#endif
    return info;
  });

  // ---- the reference's names ---------------------------------------------------------------
  m.def(
      "compute_arc_w4a16_group_sums",
      [](ptr_t activations_ptr, ptr_t sums_ptr, int batch, int k, int group_size, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::compute_arc_w4a16_group_sums(activations_ptr, sums_ptr, batch, k, group_size, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("sums_ptr"), py::arg("batch"), py::arg("k"),
      py::arg("group_size"), py::arg("stream_ptr"));
  m.def(
      "pack_arc_w4a16_packets",
      [](ptr_t q_ptr, ptr_t alpha_ptr, ptr_t beta_ptr, ptr_t packets_ptr, int n, int k,
         int group_size, int packet_stride_bytes, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::pack_arc_w4a16_packets(q_ptr, alpha_ptr, beta_ptr, packets_ptr, n, k, group_size,
                                    packet_stride_bytes, stream_ptr);
      },
      py::arg("q_ptr"), py::arg("alpha_ptr"), py::arg("beta_ptr"), py::arg("packets_ptr"),
      py::arg("n"), py::arg("k"), py::arg("group_size"), py::arg("packet_stride_bytes"),
      py::arg("stream_ptr"));
  m.def(
      "arc_w4a16_forward",
      [](ptr_t activations_ptr, ptr_t packets_ptr, ptr_t group_sums_ptr, ptr_t output_ptr,
         int batch, int n, int k, int group_size, int packet_stride_bytes, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::arc_w4a16_forward(activations_ptr, packets_ptr, group_sums_ptr, output_ptr, batch, n, k,
                               group_size, packet_stride_bytes, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("packets_ptr"), py::arg("group_sums_ptr"),
      py::arg("output_ptr"), py::arg("batch"), py::arg("n"), py::arg("k"), py::arg("group_size"),
      py::arg("packet_stride_bytes"), py::arg("stream_ptr"));
  m.def(
      "arc_w4a16_forward_split_k",
      [](ptr_t activations_ptr, ptr_t packets_ptr, ptr_t group_sums_ptr, ptr_t partials_ptr,
         int batch, int n, int k, int group_size, int packet_stride_bytes, int split_k_slices,
         ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::arc_w4a16_forward_split_k(activations_ptr, packets_ptr, group_sums_ptr, partials_ptr,
                                       batch, n, k, group_size, packet_stride_bytes, split_k_slices,
                                       stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("packets_ptr"), py::arg("group_sums_ptr"),
      py::arg("partials_ptr"), py::arg("batch"), py::arg("n"), py::arg("k"), py::arg("group_size"),
      py::arg("packet_stride_bytes"), py::arg("split_k_slices"), py::arg("stream_ptr"));
  m.def(
      "reduce_arc_w4a16_split_k_partials",
      [](ptr_t partials_ptr, ptr_t output_ptr, int batch, int n, int split_k_slices,
         ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::reduce_arc_w4a16_split_k_partials(partials_ptr, output_ptr, batch, n, split_k_slices,
                                               stream_ptr);
      },
      py::arg("partials_ptr"), py::arg("output_ptr"), py::arg("batch"), py::arg("n"),
      py::arg("split_k_slices"), py::arg("stream_ptr"));
  m.def(
      "dequant_w4a16_to_fp16",
      [](ptr_t q_ptr, ptr_t alpha_ptr, ptr_t beta_ptr, ptr_t output_ptr, int n, int k,
         int group_size, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::dequant_w4a16_to_fp16(q_ptr, alpha_ptr, beta_ptr, output_ptr, n, k, group_size,
                                   stream_ptr);
      },
      py::arg("q_ptr"), py::arg("alpha_ptr"), py::arg("beta_ptr"), py::arg("output_ptr"),
      py::arg("n"), py::arg("k"), py::arg("group_size"), py::arg("stream_ptr"));
  m.def(
      "dequant_arc_w4a16_packets_to_fp16",
      [](ptr_t packets_ptr, ptr_t output_ptr, int n, int k, int group_size,
         int packet_stride_bytes, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::dequant_arc_w4a16_packets_to_fp16(packets_ptr, output_ptr, n, k, group_size,
                                               packet_stride_bytes, stream_ptr);
      },
      py::arg("packets_ptr"), py::arg("output_ptr"), py::arg("n"), py::arg("k"),
      py::arg("group_size"), py::arg("packet_stride_bytes"), py::arg("stream_ptr"));
  m.def(
      "cublaslt_fp16_with_weight",
      [](ptr_t activations_ptr, ptr_t weight_ptr, ptr_t output_ptr, ptr_t workspace_ptr,
         std::size_t workspace_bytes, int batch, int n, int k, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::cublaslt_fp16_with_weight(activations_ptr, weight_ptr, output_ptr, workspace_ptr,
                                       workspace_bytes, batch, n, k, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("weight_ptr"), py::arg("output_ptr"),
      py::arg("workspace_ptr"), py::arg("workspace_bytes"), py::arg("batch"), py::arg("n"),
      py::arg("k"), py::arg("stream_ptr"));
  m.def(
      "cublaslt_fp16_after_packet_dequant",
      [](ptr_t activations_ptr, ptr_t packets_ptr, ptr_t output_ptr, ptr_t weight_ptr,
         ptr_t workspace_ptr, std::size_t workspace_bytes, int batch, int n, int k, int group_size,
         int packet_stride_bytes, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::cublaslt_fp16_after_packet_dequant(activations_ptr, packets_ptr, output_ptr, weight_ptr,
                                                workspace_ptr, workspace_bytes, batch, n, k,
                                                group_size, packet_stride_bytes, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("packets_ptr"), py::arg("output_ptr"),
      py::arg("weight_ptr"), py::arg("workspace_ptr"), py::arg("workspace_bytes"), py::arg("batch"),
      py::arg("n"), py::arg("k"), py::arg("group_size"), py::arg("packet_stride_bytes"),
      py::arg("stream_ptr"));
  m.def(
      "cublaslt_fp16_after_dequant",
      [](ptr_t activations_ptr, ptr_t q_ptr, ptr_t alpha_ptr, ptr_t beta_ptr, ptr_t output_ptr,
         ptr_t weight_ptr, ptr_t workspace_ptr, std::size_t workspace_bytes, int batch, int n, int k,
         int group_size, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::cublaslt_fp16_after_dequant(activations_ptr, q_ptr, alpha_ptr, beta_ptr, output_ptr,
                                         weight_ptr, workspace_ptr, workspace_bytes, batch, n, k,
                                         group_size, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("q_ptr"), py::arg("alpha_ptr"), py::arg("beta_ptr"),
      py::arg("output_ptr"), py::arg("weight_ptr"), py::arg("workspace_ptr"),
      py::arg("workspace_bytes"), py::arg("batch"), py::arg("n"), py::arg("k"),
      py::arg("group_size"), py::arg("stream_ptr"));

  // ---- additions: element types and caller-owned scratch -------------------------------------
  m.attr("ELEMENT_FLOAT16") = dql::kElementFloat16;
  m.attr("ELEMENT_BFLOAT16") = dql::kElementBFloat16;
  m.def("arc_packet_stride_bytes", [](int group_size) {
#if FK_COMPILED_WITH_CUDA
    const int stride = fk_w4a16_packet_stride_bytes(group_size);
    if (stride < 0) {
      throw py::value_error(fk_w4a16_last_error());
    }
    return stride;
#else
    // pure arithmetic (reference: expected_packet_stride_bytes, arc_w4a16.cu:23-26)
    if (group_size != 32 && group_size != 64 && group_size != 128) {
      throw py::value_error("group_size must be 32, 64 or 128");
    }
    return (64 * group_size) + 512;
#endif
  }, py::arg("group_size"));
  m.def("arc_w4a16_workspace_bytes", &dql::arc_w4a16_workspace_bytes, py::arg("batch"),
        py::arg("n"), py::arg("k"), py::arg("group_size"));
  m.def(
      "arc_w4a16_forward_fused",
      [](ptr_t activations_ptr, ptr_t packets_ptr, ptr_t output_ptr, ptr_t workspace_ptr,
         std::size_t workspace_bytes, int batch, int n, int k, int group_size,
         int packet_stride_bytes, int element_type, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::arc_w4a16_forward_fused(activations_ptr, packets_ptr, output_ptr, workspace_ptr,
                                     workspace_bytes, batch, n, k, group_size, packet_stride_bytes,
                                     element_type, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("packets_ptr"), py::arg("output_ptr"),
      py::arg("workspace_ptr"), py::arg("workspace_bytes"), py::arg("batch"), py::arg("n"),
      py::arg("k"), py::arg("group_size"), py::arg("packet_stride_bytes"), py::arg("element_type"),
      py::arg("stream_ptr"));
  m.def(
      "compute_arc_w4a16_group_sums_typed",
      [](ptr_t activations_ptr, ptr_t sums_ptr, int batch, int k, int group_size, int element_type,
         ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::compute_arc_w4a16_group_sums_typed(activations_ptr, sums_ptr, batch, k, group_size,
                                                element_type, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("sums_ptr"), py::arg("batch"), py::arg("k"),
      py::arg("group_size"), py::arg("element_type"), py::arg("stream_ptr"));
  m.def(
      "arc_w4a16_forward_split_k_typed",
      [](ptr_t activations_ptr, ptr_t packets_ptr, ptr_t partials_ptr, int batch, int n, int k,
         int group_size, int packet_stride_bytes, int split_k_slices, int element_type,
         ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::arc_w4a16_forward_split_k_typed(activations_ptr, packets_ptr, partials_ptr, batch, n, k,
                                             group_size, packet_stride_bytes, split_k_slices,
                                             element_type, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("packets_ptr"), py::arg("partials_ptr"), py::arg("batch"),
      py::arg("n"), py::arg("k"), py::arg("group_size"), py::arg("packet_stride_bytes"),
      py::arg("split_k_slices"), py::arg("element_type"), py::arg("stream_ptr"));
  m.def(
      "reduce_arc_w4a16_split_k_partials_typed",
      [](ptr_t partials_ptr, ptr_t output_ptr, int batch, int n, int split_k_slices,
         int element_type, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::reduce_arc_w4a16_split_k_partials_typed(partials_ptr, output_ptr, batch, n,
                                                     split_k_slices, element_type, stream_ptr);
      },
      py::arg("partials_ptr"), py::arg("output_ptr"), py::arg("batch"), py::arg("n"),
      py::arg("split_k_slices"), py::arg("element_type"), py::arg("stream_ptr"));
  m.def(
      "dequant_w4a16_typed",
      [](ptr_t q_ptr, ptr_t alpha_ptr, ptr_t beta_ptr, ptr_t output_ptr, int n, int k,
         int group_size, int element_type, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::dequant_w4a16_typed(q_ptr, alpha_ptr, beta_ptr, output_ptr, n, k, group_size,
                                 element_type, stream_ptr);
      },
      py::arg("q_ptr"), py::arg("alpha_ptr"), py::arg("beta_ptr"), py::arg("output_ptr"),
      py::arg("n"), py::arg("k"), py::arg("group_size"), py::arg("element_type"),
      py::arg("stream_ptr"));
  m.def(
      "dequant_arc_w4a16_packets_typed",
      [](ptr_t packets_ptr, ptr_t output_ptr, int n, int k, int group_size,
         int packet_stride_bytes, int element_type, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::dequant_arc_w4a16_packets_typed(packets_ptr, output_ptr, n, k, group_size,
                                             packet_stride_bytes, element_type, stream_ptr);
      },
      py::arg("packets_ptr"), py::arg("output_ptr"), py::arg("n"), py::arg("k"),
      py::arg("group_size"), py::arg("packet_stride_bytes"), py::arg("element_type"),
      py::arg("stream_ptr"));
  m.def(
      "cublaslt_with_weight_typed",
      [](ptr_t activations_ptr, ptr_t weight_ptr, ptr_t output_ptr, ptr_t workspace_ptr,
         std::size_t workspace_bytes, int batch, int n, int k, int element_type,
         ptr_t stream_ptr) {
        py::gil_scoped_release release;
        dql::cublaslt_with_weight_typed(activations_ptr, weight_ptr, output_ptr, workspace_ptr,
                                        workspace_bytes, batch, n, k, element_type, stream_ptr);
      },
      py::arg("activations_ptr"), py::arg("weight_ptr"), py::arg("output_ptr"),
      py::arg("workspace_ptr"), py::arg("workspace_bytes"), py::arg("batch"), py::arg("n"),
      py::arg("k"), py::arg("element_type"), py::arg("stream_ptr"));
  m.def("arc_w4a16_device_status", []() {
    py::gil_scoped_release release;
    return dql::arc_w4a16_device_status();
  });

  // ---- paged-KV decode attention: the reference's name and keyword arguments, plus two
  // optional ones at the end ------------------------------------------------------------------
  m.def(
      "clustered_page_decode_forward",
      [](ptr_t query_ptr, ptr_t key_ptr, ptr_t value_ptr, ptr_t key_scales_ptr, ptr_t value_scales_ptr,
         ptr_t run_base_pages_ptr, ptr_t run_page_counts_ptr, ptr_t run_logical_starts_ptr,
         ptr_t run_last_page_lens_ptr, ptr_t request_run_offsets_ptr, ptr_t seq_lens_ptr, ptr_t output_ptr,
         int batch, int num_runs, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
         int group_tile, int use_clustered_kernel, int cluster_size, int kv_format, int keys_are_rotated,
         float softmax_scale, float rope_theta, ptr_t stream_ptr, int max_pages_hint, int early_descriptors) {
        py::gil_scoped_release release;
        fast_kernels::clustered_page_decode::clustered_page_decode_forward_hinted(
            query_ptr, key_ptr, value_ptr, key_scales_ptr, value_scales_ptr, run_base_pages_ptr,
            run_page_counts_ptr, run_logical_starts_ptr, run_last_page_lens_ptr, request_run_offsets_ptr,
            seq_lens_ptr, output_ptr, batch, num_runs, num_q_heads, num_kv_heads, head_dim, page_size,
            group_tile, use_clustered_kernel, cluster_size, kv_format, keys_are_rotated, softmax_scale,
            rope_theta, max_pages_hint, early_descriptors, stream_ptr);
      },
      py::arg("query_ptr"), py::arg("key_ptr"), py::arg("value_ptr"), py::arg("key_scales_ptr"),
      py::arg("value_scales_ptr"), py::arg("run_base_pages_ptr"), py::arg("run_page_counts_ptr"),
      py::arg("run_logical_starts_ptr"), py::arg("run_last_page_lens_ptr"),
      py::arg("request_run_offsets_ptr"), py::arg("seq_lens_ptr"), py::arg("output_ptr"), py::arg("batch"),
      py::arg("num_runs"), py::arg("num_q_heads"), py::arg("num_kv_heads"), py::arg("head_dim"),
      py::arg("page_size"), py::arg("group_tile"), py::arg("use_clustered_kernel"), py::arg("cluster_size"),
      py::arg("kv_format"), py::arg("keys_are_rotated"), py::arg("softmax_scale"), py::arg("rope_theta"),
      py::arg("stream_ptr"), py::arg("max_pages_hint") = 0, py::arg("early_descriptors") = 0);
  m.def(
      "prefix_union_decode_forward",
      [](ptr_t query_ptr, ptr_t key_ptr, ptr_t value_ptr, ptr_t key_scales_ptr, ptr_t value_scales_ptr,
         ptr_t tasks_ptr, ptr_t shared_pages_ptr, ptr_t tail_pages_ptr, ptr_t consumers_ptr,
         ptr_t scheduler_counter_ptr, ptr_t output_ptr, int num_tasks, int num_pages, int num_q_heads,
         int num_kv_heads, int head_dim, int page_size, int cluster_size, int kv_format, int keys_are_rotated,
         float softmax_scale, float rope_theta, ptr_t stream_ptr) {
        py::gil_scoped_release release;
        fast_kernels::prefix_union_decode::prefix_union_decode_forward(
            query_ptr, key_ptr, value_ptr, key_scales_ptr, value_scales_ptr, tasks_ptr, shared_pages_ptr,
            tail_pages_ptr, consumers_ptr, scheduler_counter_ptr, output_ptr, num_tasks, num_pages, num_q_heads,
            num_kv_heads, head_dim, page_size, cluster_size, kv_format, keys_are_rotated, softmax_scale, rope_theta,
            stream_ptr);
      },
      py::arg("query_ptr"), py::arg("key_ptr"), py::arg("value_ptr"), py::arg("key_scales_ptr"),
      py::arg("value_scales_ptr"), py::arg("tasks_ptr"), py::arg("shared_pages_ptr"), py::arg("tail_pages_ptr"),
      py::arg("consumers_ptr"), py::arg("scheduler_counter_ptr"), py::arg("output_ptr"), py::arg("num_tasks"),
      py::arg("num_pages"), py::arg("num_q_heads"), py::arg("num_kv_heads"), py::arg("head_dim"),
      py::arg("page_size"), py::arg("cluster_size"), py::arg("kv_format"), py::arg("keys_are_rotated"),
      py::arg("softmax_scale"), py::arg("rope_theta"), py::arg("stream_ptr"));
  m.def("page_decode_device_status", []() {
    py::gil_scoped_release release;
    return fast_kernels::clustered_page_decode::page_decode_device_status();
  });
}

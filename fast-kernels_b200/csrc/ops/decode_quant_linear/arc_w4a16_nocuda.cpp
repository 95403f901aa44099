// The op surface of a build WITHOUT CUDA: every launcher exists under the same name and throws
// std::runtime_error("fast-kernels was built without CUDA support"), which pybind11 turns into
// RuntimeError -- the contract of the reference's CPU-only module
// (csrc/bindings/python_module.cpp:241-287 there). There is deliberately no arithmetic here: the
// W4A16 path has no CPU fallback. Linked instead of arc_w4a16.cpp by `build.py --no-cuda`.
#include <stdexcept>

#include "ops/decode_quant_linear/arc_w4a16.h"

namespace fast_kernels::decode_quant_linear {
namespace {
[[noreturn]] void unavailable() {
  throw std::runtime_error("fast-kernels was built without CUDA support");
}
}  // namespace

using ptr = std::uintptr_t;

void pack_arc_w4a16_packets(ptr, ptr, ptr, ptr, int, int, int, int, ptr) { unavailable(); }
void compute_arc_w4a16_group_sums(ptr, ptr, int, int, int, ptr) { unavailable(); }
void arc_w4a16_forward(ptr, ptr, ptr, ptr, int, int, int, int, int, ptr) { unavailable(); }
void arc_w4a16_forward_split_k(ptr, ptr, ptr, ptr, int, int, int, int, int, int, ptr) { unavailable(); }
void reduce_arc_w4a16_split_k_partials(ptr, ptr, int, int, int, ptr) { unavailable(); }
void dequant_w4a16_to_fp16(ptr, ptr, ptr, ptr, int, int, int, ptr) { unavailable(); }
void dequant_arc_w4a16_packets_to_fp16(ptr, ptr, int, int, int, int, ptr) { unavailable(); }
void cublaslt_fp16_with_weight(ptr, ptr, ptr, ptr, std::size_t, int, int, int, ptr) { unavailable(); }
void cublaslt_fp16_after_packet_dequant(ptr, ptr, ptr, ptr, ptr, std::size_t, int, int, int, int, int, ptr) {
  unavailable();
}
void cublaslt_fp16_after_dequant(ptr, ptr, ptr, ptr, ptr, ptr, ptr, std::size_t, int, int, int, int, ptr) {
  unavailable();
}
std::size_t arc_w4a16_workspace_bytes(int, int, int, int) { unavailable(); }
void arc_w4a16_forward_fused(ptr, ptr, ptr, ptr, std::size_t, int, int, int, int, int, int, ptr) { unavailable(); }
void compute_arc_w4a16_group_sums_typed(ptr, ptr, int, int, int, int, ptr) { unavailable(); }
void arc_w4a16_forward_split_k_typed(ptr, ptr, ptr, int, int, int, int, int, int, int, ptr) { unavailable(); }
void reduce_arc_w4a16_split_k_partials_typed(ptr, ptr, int, int, int, int, ptr) { unavailable(); }
void dequant_w4a16_typed(ptr, ptr, ptr, ptr, int, int, int, int, ptr) { unavailable(); }
void dequant_arc_w4a16_packets_typed(ptr, ptr, int, int, int, int, int, ptr) { unavailable(); }
void cublaslt_with_weight_typed(ptr, ptr, ptr, ptr, std::size_t, int, int, int, int, ptr) { unavailable(); }
int arc_w4a16_device_status() { unavailable(); }

}  // namespace fast_kernels::decode_quant_linear

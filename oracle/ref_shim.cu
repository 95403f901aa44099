// C entry points around the reference's OWN W4A16 launchers (namespace
// fast_kernels::decode_quant_linear, csrc/ops/decode_quant_linear/arc_w4a16.h:8-52), so that the
// tests and the bench can run the unmodified reference kernels on the same inputs as the new
// library. TEST INFRASTRUCTURE ONLY: built into oracle/_ref/ from the reference sources where they
// lie; the shipped library never links or loads it.
#include <cstdint>
#include <cstring>
#include <exception>

#include "ops/decode_quant_linear/arc_w4a16.h"

namespace ref = fast_kernels::decode_quant_linear;

static thread_local char g_error[512];

template <class Fn>
static int guarded(Fn&& fn) {
  try {
    fn();
    g_error[0] = '\0';
    return 0;
  } catch (const std::exception& e) {
    std::strncpy(g_error, e.what(), sizeof(g_error) - 1);
    g_error[sizeof(g_error) - 1] = '\0';
    return -1;
  }
}

extern "C" {

const char* fkref_last_error() { return g_error; }

int fkref_pack(std::uintptr_t q, std::uintptr_t alpha, std::uintptr_t beta, std::uintptr_t packets,
               int n, int k, int group, int stride, std::uintptr_t stream) {
  return guarded([&] { ref::pack_arc_w4a16_packets(q, alpha, beta, packets, n, k, group, stride, stream); });
}

int fkref_group_sums(std::uintptr_t act, std::uintptr_t sums, int batch, int k, int group,
                     std::uintptr_t stream) {
  return guarded([&] { ref::compute_arc_w4a16_group_sums(act, sums, batch, k, group, stream); });
}

int fkref_forward(std::uintptr_t act, std::uintptr_t packets, std::uintptr_t sums,
                  std::uintptr_t out, int batch, int n, int k, int group, int stride,
                  std::uintptr_t stream) {
  return guarded([&] { ref::arc_w4a16_forward(act, packets, sums, out, batch, n, k, group, stride, stream); });
}

int fkref_forward_split_k(std::uintptr_t act, std::uintptr_t packets, std::uintptr_t sums,
                          std::uintptr_t partials, int batch, int n, int k, int group, int stride,
                          int slices, std::uintptr_t stream) {
  return guarded([&] {
    ref::arc_w4a16_forward_split_k(act, packets, sums, partials, batch, n, k, group, stride, slices, stream);
  });
}

int fkref_reduce(std::uintptr_t partials, std::uintptr_t out, int batch, int n, int slices,
                 std::uintptr_t stream) {
  return guarded([&] { ref::reduce_arc_w4a16_split_k_partials(partials, out, batch, n, slices, stream); });
}

int fkref_dequant(std::uintptr_t q, std::uintptr_t alpha, std::uintptr_t beta, std::uintptr_t out,
                  int n, int k, int group, std::uintptr_t stream) {
  return guarded([&] { ref::dequant_w4a16_to_fp16(q, alpha, beta, out, n, k, group, stream); });
}

int fkref_dequant_packets(std::uintptr_t packets, std::uintptr_t out, int n, int k, int group,
                          int stride, std::uintptr_t stream) {
  return guarded([&] { ref::dequant_arc_w4a16_packets_to_fp16(packets, out, n, k, group, stride, stream); });
}

int fkref_cublaslt_after_dequant(std::uintptr_t act, std::uintptr_t q, std::uintptr_t alpha,
                                 std::uintptr_t beta, std::uintptr_t out, std::uintptr_t weight,
                                 std::uintptr_t workspace, std::size_t workspace_bytes, int batch,
                                 int n, int k, int group, std::uintptr_t stream) {
  return guarded([&] {
    ref::cublaslt_fp16_after_dequant(act, q, alpha, beta, out, weight, workspace, workspace_bytes,
                                     batch, n, k, group, stream);
  });
}

int fkref_cublaslt_after_packet_dequant(std::uintptr_t act, std::uintptr_t packets, std::uintptr_t out,
                                        std::uintptr_t weight, std::uintptr_t workspace,
                                        std::size_t workspace_bytes, int batch, int n, int k,
                                        int group, int stride, std::uintptr_t stream) {
  return guarded([&] {
    ref::cublaslt_fp16_after_packet_dequant(act, packets, out, weight, workspace, workspace_bytes, batch,
                                            n, k, group, stride, stream);
  });
}

}  // extern "C"

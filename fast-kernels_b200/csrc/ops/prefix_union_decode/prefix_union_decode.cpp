#include "ops/prefix_union_decode/prefix_union_decode.h"

#include <stdexcept>

namespace fast_kernels::prefix_union_decode {

void prefix_union_decode_forward(std::uintptr_t, std::uintptr_t, std::uintptr_t, std::uintptr_t, std::uintptr_t,
                                 std::uintptr_t, std::uintptr_t, std::uintptr_t, std::uintptr_t, std::uintptr_t,
                                 std::uintptr_t, int num_tasks, int, int, int, int, int, int, int, int, float, float,
                                 std::uintptr_t) {
  if (num_tasks == 0) {
    return;
  }
  throw std::invalid_argument(
      "prefix_union_decode_forward requires a Blackwell-class GPU (compute capability 12.x); on this build "
      "the op runs through clustered_page_decode (the plan's fallback), as the reference does on sm_100");
}

}  // namespace fast_kernels::prefix_union_decode

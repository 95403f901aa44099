// The op surface of a build WITHOUT CUDA: same names, every call throws
// std::runtime_error("fast-kernels was built without CUDA support") -- there is no CPU path.
#include <stdexcept>

#include "ops/clustered_page_decode/clustered_page_decode.h"

namespace fast_kernels::clustered_page_decode {
namespace {
[[noreturn]] void unavailable() { throw std::runtime_error("fast-kernels was built without CUDA support"); }
}  // namespace

using ptr = std::uintptr_t;

void clustered_page_decode_forward(ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, int, int, int, int, int,
                                   int, int, int, int, int, int, float, float, ptr) {
  unavailable();
}
void clustered_page_decode_forward_hinted(ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, int, int, int, int,
                                          int, int, int, int, int, int, int, float, float, int, int, ptr) {
  unavailable();
}
int page_decode_device_status() { unavailable(); }

}  // namespace fast_kernels::clustered_page_decode

// Kernels for head_dim 64, bf16 pages.
#define FK_PD_D 64
#define FK_PD_KV kKvBf16
#define FK_PD_NAME d64_bf16
#include "page_decode_shape.inc"

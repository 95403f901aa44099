// Kernels for head_dim 128, bf16 pages.
#define FK_PD_D 128
#define FK_PD_KV kKvBf16
#define FK_PD_NAME d128_bf16
#include "page_decode_shape.inc"

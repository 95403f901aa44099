// Kernels for head_dim 128, fp8 pages.
#define FK_PD_D 128
#define FK_PD_KV kKvFp8
#define FK_PD_NAME d128_fp8
#include "page_decode_shape.inc"

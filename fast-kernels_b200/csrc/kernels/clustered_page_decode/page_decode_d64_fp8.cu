// Kernels for head_dim 64, fp8 pages.
#define FK_PD_D 64
#define FK_PD_KV kKvFp8
#define FK_PD_NAME d64_fp8
#include "page_decode_shape.inc"

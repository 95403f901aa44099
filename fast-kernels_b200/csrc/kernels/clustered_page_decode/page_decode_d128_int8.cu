// Kernels for head_dim 128, int8 pages.
#define FK_PD_D 128
#define FK_PD_KV kKvInt8
#define FK_PD_NAME d128_int8
#include "page_decode_shape.inc"

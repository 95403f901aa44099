// Kernels for head_dim 64, int8 pages.
#define FK_PD_D 64
#define FK_PD_KV kKvInt8
#define FK_PD_NAME d64_int8
#include "page_decode_shape.inc"

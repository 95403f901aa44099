// Kernels for head_dim 128, page_size 32.
#define FK_PD_D 128
#define FK_PD_PS 32
#define FK_PD_NAME d128_p32
#include "page_decode_shape.inc"

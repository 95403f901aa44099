// Kernels for head_dim 128, page_size 16.
#define FK_PD_D 128
#define FK_PD_PS 16
#define FK_PD_NAME d128_p16
#include "page_decode_shape.inc"

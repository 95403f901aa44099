// Kernels for head_dim 64, page_size 32.
#define FK_PD_D 64
#define FK_PD_PS 32
#define FK_PD_NAME d64_p32
#include "page_decode_shape.inc"

// Kernels for head_dim 64, page_size 16.
#define FK_PD_D 64
#define FK_PD_PS 16
#define FK_PD_NAME d64_p16
#include "page_decode_shape.inc"

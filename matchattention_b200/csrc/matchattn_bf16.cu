#define MATCHATTN_T __nv_bfloat16
#define MATCHATTN_T_IS_16BIT 1
#include "matchattn_launch.inl"

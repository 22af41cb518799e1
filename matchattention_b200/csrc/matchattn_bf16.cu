#define MATCHATTN_T __nv_bfloat16
#include "matchattn_launch.inl"

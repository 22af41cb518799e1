#define MATCHATTN_T __half
#define MATCHATTN_T_IS_16BIT 1
#include "matchattn_launch.inl"

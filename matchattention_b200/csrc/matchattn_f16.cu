#define MATCHATTN_T __half
#include "matchattn_launch.inl"

#define MATCHATTN_T float
#include "matchattn_launch.inl"

// elementwise entry points of libcumo_b200 for Cumo::Int64.
#define CB_T int64
#define CB_C int64_t
#define CB_FLOAT 0
#include "abi_elementwise.cuh"

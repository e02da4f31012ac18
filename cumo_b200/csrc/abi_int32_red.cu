// reduction and mulsum entry points of libcumo_b200 for Cumo::Int32.
#define CB_T int32
#define CB_C int32_t
#define CB_FLOAT 0
#include "abi_reduce.cuh"

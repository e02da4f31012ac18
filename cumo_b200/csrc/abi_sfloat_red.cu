// reduction and mulsum entry points of libcumo_b200 for Cumo::SFloat.
#define CB_T sfloat
#define CB_C float
#define CB_FLOAT 1
#include "abi_reduce.cuh"

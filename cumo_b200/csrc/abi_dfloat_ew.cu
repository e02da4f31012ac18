// elementwise entry points of libcumo_b200 for Cumo::DFloat.
#define CB_T dfloat
#define CB_C double
#define CB_FLOAT 1
#define CB_DOUBLE 1
#include "abi_elementwise.cuh"

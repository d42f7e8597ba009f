// Single translation unit of libvolundr_b200.so (one device link unit: the status word is shared by every kernel).
#include "runtime.cu"
#include "w4_gemm.cu"
#include "w4_tile.cu"
#include "w4_t5.cu"
#include "elementwise.cu"
#include "allreduce.cu"
#include "kda.cu"
#include "attention.cu"

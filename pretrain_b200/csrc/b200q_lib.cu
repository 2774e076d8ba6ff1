// Single translation unit of libb200q.so: the kernels share one device status word and a few
// inline helpers, so the sources are compiled together instead of with relocatable device code.
#include "quantize.cu"
#include "gemm.cu"
#include "gemm_2cta.cu"
#include "gemm_bstat.cu"
#include "gemm_rowstat.cu"
#include "moe.cu"

// Single translation unit of libb200q.so: the C-ABI entry points and every kernel.
// Built as one unit so that the device-side error word and the helpers are shared
// without relocatable device code.
#include "status.cu"
#include "dynamic_quant.cu"
#include "dynamic_quant_ext.cu"
#include "swiglu_quant.cu"
#include "int4pack.cu"
#include "anti_quant.cu"
#include "w8a8_gemm.cu"
#include "w4a16_gemm.cu"
#include "peer_scatter.cu"

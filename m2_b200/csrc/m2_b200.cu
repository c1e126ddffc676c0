// Single translation unit of libm2b200.so: the parts share one device-side status word
// and are compiled together (no relocatable device code needed).
#include "abi.cu"
#include "filter.cu"
#include "longconv_simt.cu"
#include "longconv_tc.cu"
#include "longconv_tcl.cu"
#include "longconv_tz.cu"
#include "longconv.cu"
#include "gemm_tc.cu"
#include "linear_tc.cu"
#include "glu_pair.cu"
#include "gemm_simt.cu"
#include "selftest.cu"

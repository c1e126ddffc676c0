// placeholder until the tensor-core family lands
#include "common.cuh"
namespace m2 {
int longconv_tc_supported(int, m2_dtype) { return 0; }
size_t spectrum_kind1_floats(int, int) { return 0; }
int spectrum_kind1_launch(int, int, const float*, float*, cudaStream_t) { return m2_set_error(M2_ERR_UNSUPPORTED, "kind 1 not built"); }
int longconv_tc_launch(const m2_longconv_args*, cudaStream_t) { return m2_set_error(M2_ERR_UNSUPPORTED, "kind 1 not built"); }
}

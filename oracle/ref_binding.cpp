// Python binding for the QUIK reference's own quantize / dequantize CUDA kernels, compiled unmodified from
// the reference checkout (src/asymmetric/asymmetric.cu, src/symmetric/symmetric.cu) by oracle/build_ref.py.
// Test infrastructure only: tests/ use it on a GPU to pin this repository's kernels against the reference's
// outputs on the same inputs.  The reference's GEMM and fused-dequantize sources are left out: they need
// CUTLASS GEMM templates from a submodule that is not vendored in the reference checkout.
#include <torch/extension.h>

#include "asymmetric/asymmetric_internal.h"
#include "symmetric/symmetric_internal.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("asym_quantize", &QUIK::asymmetric::quantizeCUDA, "reference quik.asymmetric.quantize (asymmetric.cu:492-584)");
  m.def("asym_quantize_old", &QUIK::asymmetric::quantizeCUDAOld, "reference quik.asymmetric.quantizeOld");
  m.def("asym_dequantize", &QUIK::asymmetric::dequantizeCUDA, "reference quik.asymmetric.dequantize (asymmetric.cu:175-233)");
  m.def("asym_find_meta", &QUIK::asymmetric::findMaxMinMetaCUDA, "reference quik.asymmetric.find_meta");
  m.def("sym_quantize_int4", &QUIK::symmetric::int4QuantizationCUDA, "reference quik.symmetric.quantize, bits = 4");
  m.def("sym_quantize_int8", &QUIK::symmetric::int8QuantizationCUDA, "reference quik.symmetric.quantize, bits = 8");
  m.def("sym_dequantize_int8", &QUIK::symmetric::dequantizationCUDA<int8_t>, "reference quik.symmetric.dequantize, 8-bit x");
  m.def("sym_dequantize_half", &QUIK::symmetric::dequantizationCUDA<torch::Half>, "reference quik.symmetric.dequantize, fp16 x");
  m.def("sym_dequantize_int32", &QUIK::symmetric::dequantizationCUDA<int>, "reference quik.symmetric.dequantize, int32 x");
}

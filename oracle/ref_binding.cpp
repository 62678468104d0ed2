// Python binding for the QUIK reference's own CUDA kernels, compiled unmodified from the reference checkout
// (src/asymmetric/*.cu, src/symmetric/*.cu, src/matmul/matmul.cu) by oracle/build_ref.py: quantize, dequantize,
// the CUTLASS int4 / int8 GEMMs and the fused GEMM + dequantize ops.  Test infrastructure only: tests/ use it on a
// GPU to pin this repository's kernels against the reference's outputs on the same inputs and to time both.
// Left out: the 2:4-sparse and cuSPARSELt entry points (out of this repository's scope).
#include <torch/extension.h>

#include "asymmetric/asymmetric_internal.h"
#include "matmul/matmul_internal.h"
#include "symmetric/symmetric_internal.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("asym_quantize", &QUIK::asymmetric::quantizeCUDA, "reference quik.asymmetric.quantize (asymmetric.cu:492-584)");
  m.def("asym_quantize_old", &QUIK::asymmetric::quantizeCUDAOld, "reference quik.asymmetric.quantizeOld");
  m.def("asym_dequantize", &QUIK::asymmetric::dequantizeCUDA, "reference quik.asymmetric.dequantize (asymmetric.cu:175-233)");
  m.def("asym_find_meta", &QUIK::asymmetric::findMaxMinMetaCUDA, "reference quik.asymmetric.find_meta");
  m.def("int4_matmul", &QUIK::matmul::int4MatmulCUDA, "reference quik.matmul.int4Matmul (matmul.cu:17-55)");
  m.def("int8_matmul", &QUIK::matmul::int8MatmulCUDA, "reference quik.matmul.int8Matmul (matmul.cu:98-136)");
  m.def("asym_int4_fused_dequantize", &QUIK::asymmetric::int4FusedDequantizeCUDA, "reference quik.asymmetric.int4FusedDequantize");
  m.def("asym_int8_fused_dequantize", &QUIK::asymmetric::int8FusedDequantizeCUDA, "reference quik.asymmetric.int8FusedDequantize");
  m.def("sym_int4_fused_dequantize", &QUIK::symmetric::int4FusedDequantizeCUDA, "reference quik.symmetric.int4FusedDequantize");
  m.def("sym_int8_fused_dequantize", &QUIK::symmetric::int8FusedDequantizeCUDA, "reference quik.symmetric.int8FusedDequantize");
  m.def("sym_quantize_int4", &QUIK::symmetric::int4QuantizationCUDA, "reference quik.symmetric.quantize, bits = 4");
  m.def("sym_quantize_int8", &QUIK::symmetric::int8QuantizationCUDA, "reference quik.symmetric.quantize, bits = 8");
  m.def("sym_dequantize_int8", &QUIK::symmetric::dequantizationCUDA<int8_t>, "reference quik.symmetric.dequantize, 8-bit x");
  m.def("sym_dequantize_half", &QUIK::symmetric::dequantizationCUDA<torch::Half>, "reference quik.symmetric.dequantize, fp16 x");
  m.def("sym_dequantize_int32", &QUIK::symmetric::dequantizationCUDA<int>, "reference quik.symmetric.dequantize, int32 x");
}

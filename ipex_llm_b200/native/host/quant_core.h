// quant_core: host-side (CPU) low-bit block formats.
//
// This is the B200 build's stand-in for the closed `libllama-api.so` that the
// reference binds through ctypes (python/llm/src/ipex_llm/ggml/model/llama/llama_cpp.py:946-1185):
// quantizers / dequantizers for every block format, `ggml_qk_size` / `ggml_type_size`,
// the canonical(disk) <-> device layout transform, and a CPU low-bit matmul that is the
// numerical oracle for every GPU GEMV/GEMM test.
//
// All functions use a plain C ABI so that Python can call them through ctypes.
#pragma once
#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// qtype ids follow python/llm/src/ipex_llm/ggml/quantize.py:28-61 of the reference.
enum ipex_qtype {
  QT_SYM_INT4 = 2,
  QT_ASYM_INT4 = 3,
  QT_SYM_INT5 = 6,
  QT_ASYM_INT5 = 7,
  QT_SYM_INT8 = 8,
  QT_NF4 = 10,
  QT_NF3 = 11,
  QT_FP16 = 12,
  QT_FP8_E4M3 = 15,
  QT_FP4 = 16,
  QT_MIXED_FP4 = 17,
  QT_MIXED_FP8 = 18,
  QT_FP8_E5M2 = 19,
  QT_BF16 = 20,
  QT_IQ2_XXS = 21,
  QT_IQ2_XS = 22,
  QT_Q2_K = 23,
  QT_IQ1_S = 24,
  QT_IQ1_M = 25,
  QT_Q6_K = 26,
  QT_Q4_K = 27,
  QT_Q5_K = 28,
  QT_FP6 = 29,
  QT_FP6_K = 30,
  QT_SYM_INT4_RTN = 31,
  QT_SYM_INT8_RTN = 32,
  QT_ASYM_INT4_RTN = 33,
  QT_WOQ_INT4 = 34,
};

// Number of weights per block (0 when the qtype has no host implementation).
int ggml_qk_size(int qtype);
// Bytes per canonical (serialized) block.
int ggml_type_size(int qtype);
// 1 when quantize/dequantize are implemented for this qtype.
int ipex_qtype_supported(int qtype);

// Quantize n floats laid out as rows of k (k % qk == 0). Returns bytes written.
// `hist` may be NULL; when given, 16 bins of the 4-bit code histogram are accumulated.
size_t ggml_quantize_tensor(const float* src, void* dst, int qtype, size_t n, int k,
                            int64_t* hist, int scale_search);
// Importance-weighted variant: `imatrix` has n_per_row floats (may be NULL).
size_t ggml_quantize_tensor_with_weights(const float* src, void* dst, int qtype, int nrow,
                                         int n_per_row, int64_t* hist, const float* imatrix);
// Round-to-nearest per-output-channel formats: dst holds codes, scale holds one
// (sym) or two (asym: scale,min) floats per row.
size_t ggml_quantize_tensor_rtn(const float* src, void* dst, float* scale, int qtype, size_t n,
                                int k, int64_t* hist, int scale_search);

// Dequantize k weights (any whole number of blocks) to fp32.
void ggml_dequantize(const void* src, float* dst, size_t k, int qtype);
void ggml_dequantize_q4_0(const void* src, float* dst, size_t k);

// Canonical (interleaved blocks, what is serialized) -> device layout and back.
// rows x cols is the logical weight shape; both buffers have
// ipex_device_bytes(rows, cols, qtype) / rows*cols/qk*type_size bytes respectively.
size_t ipex_device_bytes(int64_t rows, int64_t cols, int qtype);
int ggml_q_format_convet_cpu2xpu(const void* src, void* dst, int64_t rows, int64_t cols, int qtype);
int ggml_q_format_convet_xpu2cpu(const void* src, void* dst, int64_t rows, int64_t cols, int qtype);

// result[M,N] = src1[M,K] * dequant(src0[N,K])^T, fp32 accumulate.
// src0_ne = {K, N}, src1_ne = {K, M} (ggml order: fastest dimension first).
void ggml_compute_forward_mul_mat_q_fp32(const int64_t* src0_ne, const void* src0, int qtype,
                                         const int64_t* src1_ne, const float* src1, float* result);

// Mean squared reconstruction error of quantizing src with qtype (used by the
// mixed_fp4 / mixed_fp8 selection, reference low_bit_linear.py:337-346).
double ipex_quantize_mse(const float* src, int qtype, size_t n, int k);

int ipex_quant_core_version(void);

#ifdef __cplusplus
}
#endif

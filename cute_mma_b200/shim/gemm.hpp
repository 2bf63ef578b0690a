// Drop-in for the launcher templates of the reference's gemm_sm80_tc.cu:95-228 and 393-418:
// gemm_nt / gemm_tn / gemm<TO, TR> with the reference's signatures, for <half, half> and <float, float>.
#pragma once
#include <type_traits>

#include "common.hpp"

template <typename TO, typename TR>
void gemm_nt(int m, int n, int k, TO const* A, int ldA, TO const* B, int ldB, TR* C, int ldC, cudaStream_t stream = 0) {
  static_assert(std::is_same<TO, TR>::value && (std::is_same<TO, half>::value || std::is_same<TO, float>::value),
                "gemm_nt exists for <half, half> and <float, float>");
  if (std::is_same<TO, half>::value) B200_CHECK(b200_gemm_nt_f16(m, n, k, A, ldA, B, ldB, C, ldC, stream));
  else B200_CHECK(b200_gemm_nt_tf32(m, n, k, A, ldA, B, ldB, C, ldC, stream));
}

template <typename TO, typename TR>
void gemm_tn(int m, int n, int k, TO const* A, int ldA, TO const* B, int ldB, TR* C, int ldC, cudaStream_t stream = 0) {
  static_assert(std::is_same<TO, TR>::value && (std::is_same<TO, half>::value || std::is_same<TO, float>::value),
                "gemm_tn exists for <half, half> and <float, float>");
  if (std::is_same<TO, half>::value) B200_CHECK(b200_gemm_tn_f16(m, n, k, A, ldA, B, ldB, C, ldC, stream));
  else B200_CHECK(b200_gemm_tn_tf32(m, n, k, A, ldA, B, ldB, C, ldC, stream));
}

// The reference's lower-case flags pick its alternative shared-memory->register path (gemm_*_test);
// there is a single kernel per layout here, so both cases reach it.
template <typename TO, typename TR>
void gemm(char transA, char transB, int m, int n, int k, TO const* A, int ldA, TO const* B, int ldB, TR* C, int ldC,
          cudaStream_t stream = 0) {
  B200_CHECK(b200_gemm(transA, transB, std::is_same<TO, float>::value ? 1 : 0, m, n, k, A, ldA, B, ldB, C, ldC, stream));
}

// Compile-time tile hyperparameters of the plain GEMM kernels, one specialisation per
// (operand type, result type, layout of A, layout of B), selected by include path like the
// reference's default_configs/gemm_config.hpp:9-57.  The autotune generator writes files of this
// shape, one directory per candidate.
//   bM  rows of C per CTA tile (tcgen05 M, fixed at 128 for the 1-CTA kernels)
//   bN  columns of C per CTA tile (tcgen05 N, multiple of 32, <= 256)
//   bK  K extent of one shared-memory stage: always one 128-byte swizzle row (64 fp16 / 32 fp32)
//   bP  depth of the TMA -> shared-memory ring
//   ctas  1: one CTA per 128 x bN tile (ring of up to 4 stages of 48 KB);  2: a pair of CTAs on neighbouring SMs
//         shares a 256 x bN tile (tcgen05 cta_group::2; each CTA loads its 128 rows of A and half of the B
//         tile: 32 KB per stage, ring of up to 6)
#pragma once
#include <cuda_fp16.h>

namespace b200 {

struct MMA_T {};  // operand stored with K contiguous ("transposed" in the reference's BLAS naming)
struct MMA_N {};  // operand stored with M (or N) contiguous

template <typename TO, typename TR, typename LayoutA, typename LayoutB>
struct Params;

template <> struct Params<float, float, MMA_T, MMA_N> {   // float TN (TF32)
  static const int bM = 128; static const int bN = 256; static const int bK = 32; static const int bP = 4; static const int ctas = 1;
};
template <> struct Params<float, float, MMA_N, MMA_T> {   // float NT (TF32)
  static const int bM = 128; static const int bN = 256; static const int bK = 32; static const int bP = 4; static const int ctas = 1;
};
template <> struct Params<half, half, MMA_T, MMA_N> {     // half TN
  static const int bM = 128; static const int bN = 256; static const int bK = 64; static const int bP = 4; static const int ctas = 1;
};
template <> struct Params<half, half, MMA_N, MMA_T> {     // half NT
  static const int bM = 128; static const int bN = 256; static const int bK = 64; static const int bP = 4; static const int ctas = 1;
};

}  // namespace b200

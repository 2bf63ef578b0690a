// Compile-time tile hyperparameters of the fused OFT kernel, selected by include path like the
// reference's default_configs/oft_config.hpp:4-12.
//   bM, bN  C tile per CTA (bM fixed at 128; bN multiple of 64, <= 256)
//   bK      K extent of one shared-memory stage (64 fp16 = one 128-byte swizzle row)
//   bP1     depth of the {A, R} ring feeding the rotation MMA   (the reference's producer ring)
//   bP2     depth of the {B} ring feeding the main contraction  (the reference's consumer ring)
//   ctas    1: one CTA per 128 x bN tile;  2: a pair of CTAs on neighbouring SMs shares a 256 x bN tile
//           (tcgen05 cta_group::2; each CTA loads its 128 rows of A and half of the R and B tiles)
// The reference's warp_layout1 / warp_layout2 have no counterpart: one thread issues each MMA.
#pragma once

struct CurrCompParams {
  static const unsigned int bM = 128;
  static const unsigned int bN = 256;
  static const unsigned int bK = 64;
  static const unsigned int bP1 = 4;
  static const unsigned int bP2 = 6;
  static const int ctas = 2;
};

// Drop-in for the reference's cute_oft_coop_pc.hpp:4-23: same CurrKernelParams, same oft_tn template,
// same argument order; the body forwards to the C ABI instead of instantiating a CuTe kernel.
#pragma once
#include "common.hpp"

#ifndef OFT_GROUP_SIZE
#define OFT_GROUP_SIZE 256
#endif
#ifndef OFT_RECONN_SIZE
#define OFT_RECONN_SIZE 8
#endif

struct CurrKernelParams {
  static const unsigned int group_size = OFT_GROUP_SIZE;
  static const unsigned int reconn_sz = OFT_RECONN_SIZE;
};

template <class KernelParams>
void oft_tn(int m, int n, int k, half const* A, int ldA, half const* B, int ldB, half const* R, int ldR, half* C, int ldC,
            cudaStream_t stream = 0) {
  B200_CHECK(b200_oft_tn_f16(m, n, k, static_cast<int>(KernelParams::group_size), static_cast<int>(KernelParams::reconn_sz),
                             A, ldA, B, ldB, R, ldR, C, ldC, stream));
}

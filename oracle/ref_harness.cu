// Thin C entry point around the reference's own cpu_oft_tn, compiled from where the reference lies
// (the header is included by path at build time and never copied).  TEST INFRASTRUCTURE ONLY.
// Build recipe: oracle/build_ref.sh; output oracle/_ref/libref_cpu_oft.so.
#include <cuda_fp16.h>
#include <thrust/host_vector.h>
#include <thrust/fill.h>
#include <cstring>
#include <cstdint>
#include "cpu_oft.hpp"   // resolved through -I<reference root>

extern "C" int ref_cpu_oft_tn(const uint16_t* A, const uint16_t* R, const uint16_t* B, uint16_t* C,
                              int m, int group_size, int n_groups, int k, int reconn_sz) {
    const size_t n = (size_t)group_size * n_groups;
    thrust::host_vector<half> hA((size_t)m * k), hR((size_t)n_groups * reconn_sz * k), hB(n * k), hC((size_t)m * n);
    std::memcpy(hA.data(), A, hA.size() * 2);
    std::memcpy(hR.data(), R, hR.size() * 2);
    std::memcpy(hB.data(), B, hB.size() * 2);
    cpu_oft_tn(hA, hR, hB, hC, m, group_size, n_groups, k, reconn_sz);
    std::memcpy(C, hC.data(), hC.size() * 2);
    return 0;
}

// Benchmark driver of the fused OFT operator with the command line and stdout contract of the
// reference's cute_oft_pc (cute_oft_pc.cu:79-383): flags -m -n -k -w -t --sparse_speedup -rs --01init
// --correctness, the "M = / N = / K = / Number of groups / Number of blocks" header, the
// Base/Total TFLOPS lines and the parsed line
//   TFLOPS/s (AR_W): [%.2f], (AR_W_sparse): %.2f, (A_RW): %.2f, Time: %.3f ms
// group_size / reconn_sz default to the compile-time CurrKernelParams and can be overridden with
// --group_size / --reconn_sz (0 = all of N in one group); --mode A_RW times the other algebraic order
// (weight transform + plain GEMM, what the reference's --cublas_mode A_RW runs through cuBLAS).  --correctness compares against a naive
// CUDA restatement of the same arithmetic (one thread per output element) with the reference's
// relative-error count (check_result, cute_oft_pc.cu:31-77).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <ctime>
#include <numeric>
#include <random>
#include <vector>

#include "../shim/cute_oft_coop_pc.hpp"
#include "flags.hpp"

__global__ void naive_xr(const half* A, const half* R, half* XR, int m, int k, int b, int g) {
  // XR[i][kk] for group g: kk = kb*b + q
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)m * k) return;
  int i = idx / k, kk = idx % k, kb = kk / b, q = kk % b;
  float acc = 0.f;
  for (int p = 0; p < b; ++p) acc += __half2float(A[(long long)i * k + kb * b + p]) * __half2float(R[(long long)(g * b + q) * k + kb * b + p]);
  XR[idx] = __float2half_rn(acc);
}
__global__ void naive_xw(const half* XR, const half* B, half* C, int m, int n, int k, int n0, int gs) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)m * gs) return;
  int i = idx / gs, j = n0 + idx % gs;
  float acc = 0.f;
  for (int kk = 0; kk < k; ++kk) acc += __half2float(XR[(long long)i * k + kk]) * __half2float(B[(long long)j * k + kk]);
  C[(long long)i * n + j] = __float2half_rn(acc);
}

int main(int argc, char** argv) {
  Flags f;
  f.add({"-m", "--m"}, "4096");
  f.add({"-n", "--n"}, "4096");
  f.add({"-k", "--k"}, "4096");
  f.add({"-w", "--warmup_iterations"}, "10");
  f.add({"-t", "--timing_iterations"}, "100");
  f.add({"--sparse_speedup"}, "2.0");
  f.add({"-rs", "--random_seed"}, std::to_string((long long)time(nullptr)));
  f.add({"--01init"}, "0", true);
  f.add({"--correctness"}, "0", true);
  f.add({"--group_size"}, std::to_string(CurrKernelParams::group_size));
  f.add({"--reconn_sz"}, std::to_string(CurrKernelParams::reconn_sz));
  f.add({"--mode"}, "AR_W");  // AR_W: the fused kernel; A_RW: weight transform + plain GEMM (the reference's --cublas_mode names)
  try { f.parse(argc, argv); } catch (const std::exception& e) { fprintf(stderr, "%s\n", e.what()); return 1; }
  const int m = f.geti("--m"), n = f.geti("--n"), k = f.geti("--k");
  int group_size = f.geti("--group_size");
  if (group_size <= 0) group_size = n;
  const int reconn_sz = f.geti("--reconn_sz");
  const int n_groups = n / group_size, n_blocks = k / reconn_sz;
  printf("M = %d\nN = %d\nK = %d\nNumber of groups: %d\nNumber of blocks: %d\n", m, n, k, n_groups, n_blocks);

  std::vector<half> hA((size_t)m * k), hB((size_t)n * k), hR((size_t)n_groups * reconn_sz * k, __float2half(0.f));
  std::mt19937 gen(f.geti("--random_seed"));
  std::uniform_real_distribution<double> dist(0.0, 1.0);
  const bool zo = f.getb("--01init");
  for (auto& v : hA) v = __float2half(zo ? (float)(int)(dist(gen) * 2) : (float)dist(gen));
  for (auto& v : hB) v = __float2half(zo ? (float)(int)(dist(gen) * 2) : (float)dist(gen));
  std::vector<int> perm(reconn_sz);
  for (int g = 0; g < n_groups; ++g)
    for (int kb = 0; kb < n_blocks; ++kb) {  // random permutation blocks, as the reference initialises R
      std::iota(perm.begin(), perm.end(), 0);
      std::shuffle(perm.begin(), perm.end(), gen);
      for (int j = 0; j < reconn_sz; ++j) hR[(size_t)(g * reconn_sz + j) * k + kb * reconn_sz + perm[j]] = __float2half(1.f);
    }
  half *dA, *dB, *dR, *dC;
  try {
    GEMM_CHECK_CUDA(cudaMalloc(&dA, hA.size() * 2));
    GEMM_CHECK_CUDA(cudaMalloc(&dB, hB.size() * 2));
    GEMM_CHECK_CUDA(cudaMalloc(&dR, hR.size() * 2));
    GEMM_CHECK_CUDA(cudaMalloc(&dC, (size_t)m * n * 2));
    GEMM_CHECK_CUDA(cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice));
    GEMM_CHECK_CUDA(cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice));
    GEMM_CHECK_CUDA(cudaMemcpy(dR, hR.data(), hR.size() * 2, cudaMemcpyHostToDevice));
    const bool a_rw = f.gets("--mode") == "A_RW";
    auto run = [&]() {
      if (a_rw) B200_CHECK(b200_oft_tn_f16_a_rw(m, n, k, group_size, reconn_sz, dA, k, dB, k, dR, k, dC, n, nullptr));
      else B200_CHECK(b200_oft_tn_f16(m, n, k, group_size, reconn_sz, dA, k, dB, k, dR, k, dC, n, nullptr));
    };
    if (f.getb("--correctness")) {
      run();
      int st[4];
      B200_CHECK(b200_device_status(st));
      std::vector<half> got((size_t)m * n), ref((size_t)m * n);
      GEMM_CHECK_CUDA(cudaMemcpy(got.data(), dC, got.size() * 2, cudaMemcpyDeviceToHost));
      half *dXR, *dRef;
      GEMM_CHECK_CUDA(cudaMalloc(&dXR, (size_t)m * k * 2));
      GEMM_CHECK_CUDA(cudaMalloc(&dRef, (size_t)m * n * 2));
      for (int g = 0; g < n_groups; ++g) {
        naive_xr<<<(unsigned)(((long long)m * k + 255) / 256), 256>>>(dA, dR, dXR, m, k, reconn_sz, g);
        naive_xw<<<(unsigned)(((long long)m * group_size + 255) / 256), 256>>>(dXR, dB, dRef, m, n, k, g * group_size, group_size);
      }
      GEMM_CHECK_CUDA(cudaDeviceSynchronize());
      GEMM_CHECK_CUDA(cudaMemcpy(ref.data(), dRef, ref.size() * 2, cudaMemcpyDeviceToHost));
      unsigned long long errors = 0;
      float max_err = 0.f;
      for (size_t i = 0; i < ref.size(); ++i) {
        float r = __half2float(ref[i]), x = __half2float(got[i]);
        float e = fabsf((r - x) / r);
        if (e > max_err) max_err = e;
        if (e > 5e-3f) ++errors;
      }
      printf("Checking against naive AR_W reference result...\nerror count: %llu, max error: %e\n", errors, max_err);
      cudaFree(dXR);
      cudaFree(dRef);
    }
    for (int i = 0; i < f.geti("--warmup_iterations"); ++i) run();
    GEMM_CHECK_CUDA(cudaDeviceSynchronize());
    const int iters = f.geti("--timing_iterations");
    if (iters <= 0) return 0;
    const double base = (double)m * n * k * 2e-12;
    const double add_arw = (double)n_groups * m * k * reconn_sz * 2e-12, add_a_rw = (double)n * k * reconn_sz * 2e-12;
    const double t_arw = base + add_arw, t_a_rw = base + add_a_rw, t_sparse = base * f.getd("--sparse_speedup") + add_arw;
    printf("Base TFLOPS: %.5f\n", base);
    printf("Total TFLOPS (AR_W): %.5f, (AR_W_sparse): %.5f, (A_RW): %.5f\n", t_arw, t_sparse, t_a_rw);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0);
    for (int i = 0; i < iters; ++i) run();  // no per-iteration synchronisation
    cudaEventRecord(e1);
    GEMM_CHECK_CUDA(cudaEventSynchronize(e1));
    int st[4];
    B200_CHECK(b200_device_status(st));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    const double time = ms * 1e-3 / iters;
    printf("Theoretical speedup: %.2f\n", t_sparse / t_arw);
    printf("TFLOPS/s (AR_W): [%.2f], (AR_W_sparse): %.2f, (A_RW): %.2f, Time: %.3f ms\n", t_arw / time, t_sparse / time,
           t_a_rw / time, time * 1000.0);
  } catch (const std::exception& e) {
    fprintf(stderr, "%s\n", e.what());
    return 1;
  }
  return 0;
}

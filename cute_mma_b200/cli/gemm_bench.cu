// Benchmark driver of the plain GEMM operators with the command line and stdout contract of the
// reference's gemm_<TO>_<TR> executables (gemm_sm80_tc.cu:421-592): -m -n -k --transA --transB -t,
// ldC = m (C column-major), and the parsed line  CUTE_GEMM:     [%6.1f]GFlop/s  (%6.4f)ms.
// --correctness adds the check of the reference's DEBUG build (fp64 sums, gemm_sm80_tc.cu:552-575) on 512 sampled
// elements of C and prints  error count: N, max error: E  (relative error above 5e-3 counts; inputs are positive).
// The element type is a compile-time choice like the reference's CUTE_MMA_DTYPE_O/R:
//   -DGEMM_FLOAT builds gemm_float_float, otherwise gemm_half_half.
#include <cmath>
#include <cstdio>
#include <cctype>
#include <cstdlib>
#include <vector>

#include "../shim/gemm.hpp"
#include "flags.hpp"

#ifdef GEMM_FLOAT
using TO = float;
static float to_elem(double v) { return (float)v; }
#else
using TO = half;
static half to_elem(double v) { return __float2half((float)v); }
#endif

int main(int argc, char** argv) {
  Flags f;
  f.add({"-m", "--m"}, "8192");
  f.add({"-n", "--n"}, "8192");
  f.add({"-k", "--k"}, "4096");
  f.add({"--transA"}, "T");
  f.add({"--transB"}, "N");
  f.add({"-t", "--timing_iterations"}, "100");
  f.add({"--correctness"}, "0", true);
  try { f.parse(argc, argv); } catch (const std::exception& e) { fprintf(stderr, "%s\n", e.what()); return 1; }
  const int m = f.geti("--m"), n = f.geti("--n"), k = f.geti("--k");
  const char transA = f.gets("--transA")[0], transB = f.gets("--transB")[0];
  printf("M = %d\nN = %d\nK = %d\nC = A^%c B^%c\n", m, n, k, transA, transB);
  std::vector<TO> hA((size_t)m * k), hB((size_t)n * k);
  srand(1);  // positive values, as the reference initialises them, but from a fixed seed
  for (auto& v : hA) v = to_elem(rand() / double(RAND_MAX));
  for (auto& v : hB) v = to_elem(rand() / double(RAND_MAX));
  const int ldA = (toupper(transA) == 'N') ? m : k, ldB = (toupper(transB) == 'N') ? k : n, ldC = m;
  TO *dA, *dB, *dC;
  try {
    GEMM_CHECK_CUDA(cudaMalloc(&dA, hA.size() * sizeof(TO)));
    GEMM_CHECK_CUDA(cudaMalloc(&dB, hB.size() * sizeof(TO)));
    GEMM_CHECK_CUDA(cudaMalloc(&dC, (size_t)m * n * sizeof(TO)));
    GEMM_CHECK_CUDA(cudaMemcpy(dA, hA.data(), hA.size() * sizeof(TO), cudaMemcpyHostToDevice));
    GEMM_CHECK_CUDA(cudaMemcpy(dB, hB.data(), hB.size() * sizeof(TO), cudaMemcpyHostToDevice));
    auto run = [&]() { gemm<TO, TO>(transA, transB, m, n, k, dA, ldA, dB, ldB, dC, ldC); };
    for (int i = 0; i < 3; ++i) run();
    GEMM_CHECK_CUDA(cudaDeviceSynchronize());
    if (f.getb("--correctness")) {
      std::vector<TO> hC((size_t)m * n);
      GEMM_CHECK_CUDA(cudaMemcpy(hC.data(), dC, hC.size() * sizeof(TO), cudaMemcpyDeviceToHost));
      const bool a_n = toupper(transA) == 'N', b_n = toupper(transB) == 'N';
      unsigned long long errors = 0;
      double max_err = 0.0;
      srand(2);
      for (int t = 0; t < 512; ++t) {
        const int i = (t == 0) ? m - 1 : rand() % m, j = (t == 0) ? n - 1 : rand() % n;
        double ref = 0.0;
        for (int l = 0; l < k; ++l) {
          const double a = (double)(float)hA[a_n ? (size_t)i + (size_t)l * ldA : (size_t)i * ldA + l];
          const double b = (double)(float)hB[b_n ? (size_t)j * ldB + l : (size_t)j + (size_t)l * ldB];
          ref += a * b;
        }
        const double e = fabs(((double)(float)hC[(size_t)i + (size_t)j * ldC] - ref) / ref);
        if (e > max_err) max_err = e;
        if (e > 5e-3) ++errors;
      }
      printf("Checking 512 sampled elements against fp64 sums...\nerror count: %llu, max error: %e\n", errors, max_err);
    }
    const int iters = f.geti("--timing_iterations");
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0);
    for (int i = 0; i < iters; ++i) run();
    cudaEventRecord(e1);
    GEMM_CHECK_CUDA(cudaEventSynchronize(e1));
    int st[4];
    B200_CHECK(b200_device_status(st));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    const double t = ms * 1e-3 / iters, gflops = 2.0 * m * n * k * 1e-9;
    printf("CUTE_GEMM:     [%6.1f]GFlop/s  (%6.4f)ms\n", gflops / t, t * 1000);
  } catch (const std::exception& e) {
    fprintf(stderr, "%s\n", e.what());
    return 1;
  }
  return 0;
}

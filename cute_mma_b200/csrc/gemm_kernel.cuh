// Plain GEMM C(i,j) = sum_l A(i,l) * B(j,l) on the 5th-generation tensor cores.
//
// Replaces the reference's gemm_device (gemm_tc.hpp:4-242: cp.async ring -> registers -> mma.sync)
// with a persistent, warp-specialised kernel:
//   warp 0      TMA producer: A and B tiles -> 128B-swizzled shared-memory ring (kStages deep)
//   warp 1      allocates tensor memory, issues tcgen05.mma (fp32 accumulators in TMEM, two
//               accumulator buffers so the epilogue of tile t overlaps the main loop of tile t+1)
//   warps 2..5  epilogue: tcgen05.ld -> convert -> coalesced stores to column-major C
// Layouts follow gemm_sm80_tc.cu:95-228: TN = A,B K-major; NT = A M-major, B N-major; C(i,j) at
// C[i + j*ldC] always.  Ragged M, N, K are handled by TMA zero fill and predicated stores.
#pragma once
#include "ptx.cuh"

namespace b200 {

template <typename TIn_, typename TOut_, bool kAMn_, bool kBMn_, int kBN_, int kStages_>
struct GemmTraits {
  using TIn = TIn_;
  using TOut = TOut_;
  static constexpr bool kAMn = kAMn_, kBMn = kBMn_;
  static constexpr int kBM = 128;
  static constexpr int kBN = kBN_;
  static constexpr int kElem = sizeof(TIn);
  static constexpr int kBK = 128 / kElem;          // one 128-byte swizzle row of K per stage
  static constexpr int kUmmaK = 32 / kElem;        // 16 (fp16) or 8 (tf32)
  static constexpr int kChunk = 128 / kElem;       // MN elements per 128-byte row of an MN-major tile
  static constexpr int kStages = kStages_;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = kBN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kAccBufs = 2;
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 192;
  static constexpr int kNumBars = 2 * kStages + 2 * kAccBufs;
  static constexpr int kSmemBytes = kStages * kStageBytes + kNumBars * 8 + 64 + 1024;  // + alignment slack
  static constexpr int kFmt = (kElem == 2) ? kFmtF16 : kFmtTF32;
  // 32-bit MN-major operands must use the 32-byte-atom flavour of the 128-byte swizzle (4-row groups)
  static constexpr bool kA32Atom = kAMn && kElem == 4, kB32Atom = kBMn && kElem == 4;
  static_assert(kBN % 32 == 0 && kBN >= 32 && kBN <= 256, "bN must be a multiple of 32 up to 256");
  static_assert(kAccBufs * kBN <= kTmemCols, "accumulators exceed tensor memory");
  static_assert(kSmemBytes <= 232448, "shared memory ring too large");
};

struct GemmArgs {
  int m, n, k;
  void* C;
  long long ldC;
  int* status;
  int raster;  // 0: z-curve tile order; g > 0: bands of g tile rows
  int tile_sync;  // pair kernel: producers of all CTAs start each tile round together
  int* rounds;    // 4 zeroed counters of this launch's tile rounds (tile_sync only)
  int a3d, b3d;  // MN-major operand described by a 3-D map (chunk, K, chunk index): one copy per tile instead of one per chunk
  unsigned long long hint_a, hint_b;  // L2 eviction priority of the K-major tile loads of A and B (pair kernel)
  int k2;  // pair kernel, K-major operands: columns of a second operand pair (A2, B2) accumulated into the same C; 0 = none
  // pair kernel, split instance: tiles from split_first on are cut into split_parts pieces along K; every piece
  // leaves its fp32 partial tile in split_scratch and the last piece of a tile to finish (split_count) sums them
  unsigned split_first;
  int split_parts;
  float* split_scratch;
  int* split_count;
  float alpha = 1.f, beta = 0.f;  // C = alpha * A.B^T + beta * C; (1, 0) takes the plain store
};

template <class T>
__global__ void __launch_bounds__(T::kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs args) {
  using TOut = typename T::TOut;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // layout: [stages x (A tile, B tile)] [barriers] [tmem base] [abort flag]
  const uint32_t bars = smem_base + T::kStages * T::kStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (T::kStages + s); };
  auto accfull_bar = [&](int a) { return bars + 8u * (2 * T::kStages + a); };
  auto accempty_bar = [&](int a) { return bars + 8u * (2 * T::kStages + T::kAccBufs + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + T::kStages * T::kStageBytes + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};
#ifdef B200_PROFILE_WAITS
  const long long kernel_c0 = clock64();
#endif

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles_m = (args.m + T::kBM - 1) / T::kBM, tiles_n = (args.n + T::kBN - 1) / T::kBN;
  const unsigned num_tiles = tiles_m * tiles_n;
  const int k_steps = (args.k + T::kBK - 1) / T::kBK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < T::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < T::kAccBufs; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 128); }
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        unsigned tm, tn;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
        const int m0 = tm * T::kBM, n0 = tn * T::kBN;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % T::kStages;
          if (!(ok = mbar_wait(empty_bar(s), ((it / T::kStages) & 1) ^ 1, ctx, 1))) break;
          mbar_expect_tx(full_bar(s), T::kStageBytes);
          const uint32_t a_dst = smem_base + s * T::kStageBytes, b_dst = a_dst + T::kABytes;
          const int k0 = ks * T::kBK;
          if constexpr (!T::kAMn) {
            tma_load_2d(a_dst, &tmap_a, full_bar(s), k0, m0);
          } else {
            if (args.a3d) {
              tma_load_3d(a_dst, &tmap_a, full_bar(s), 0, k0, m0 / T::kChunk);
            } else {
#pragma unroll
              for (int c = 0; c < T::kBM / T::kChunk; ++c)
                tma_load_2d(a_dst + c * (T::kBK * 128), &tmap_a, full_bar(s), m0 + c * T::kChunk, k0);
            }
          }
          if constexpr (!T::kBMn) {
            tma_load_2d(b_dst, &tmap_b, full_bar(s), k0, n0);
          } else {
            if (args.b3d) {
              tma_load_3d(b_dst, &tmap_b, full_bar(s), 0, k0, n0 / T::kChunk);
            } else {
#pragma unroll
              for (int c = 0; c < T::kBN / T::kChunk; ++c)
                tma_load_2d(b_dst + c * (T::kBK * 128), &tmap_b, full_bar(s), n0 + c * T::kChunk, k0);
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(T::kFmt, T::kAMn, T::kBMn, T::kBM, T::kBN);
      // K-major: advance 32 bytes inside the swizzled row per UMMA-K; MN-major: UMMA-K rows of 128 bytes.
      constexpr uint32_t a_adv = T::kAMn ? T::kUmmaK * 128 : 32, b_adv = T::kBMn ? T::kUmmaK * 128 : 32;
      constexpr uint32_t a_lbo = T::kAMn ? T::kBK * 128 : 16, b_lbo = T::kBMn ? T::kBK * 128 : 16;
      // The tensor pipe queues only a couple of MMAs per issuing thread; to keep it fed, each stage
      // looks at the next stage's barrier (non-blocking) once its first MMAs are queued, and the
      // next stage only waits if that look did not find the data landed.
      uint32_t it = 0, tcount = 0;
      bool ok = true, have_full = false;
      const uint64_t a_desc0 = umma_desc_sw128(smem_base, a_lbo, T::kA32Atom ? 512 : 1024, T::kA32Atom ? 1 : 2);
      const uint64_t b_desc0 = umma_desc_sw128(smem_base + T::kABytes, b_lbo, T::kB32Atom ? 512 : 1024, T::kB32Atom ? 1 : 2);
      for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++tcount) {
        const int a = tcount % T::kAccBufs;
        if (!(ok = mbar_wait(accempty_bar(a), ((tcount / T::kAccBufs) & 1) ^ 1, ctx, 2))) break;
        const uint32_t d_tmem = tmem_base + a * T::kBN;
        const bool last_tile = tile + gridDim.x >= num_tiles;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % T::kStages;
          if (!have_full && !(ok = mbar_wait(full_bar(s), (it / T::kStages) & 1, ctx, 3))) break;
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (T::kStageBytes >> 4));
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(s * (T::kStageBytes >> 4));
#pragma unroll
          for (int kk = 0; kk < T::kBK / T::kUmmaK; ++kk) {
            if (kk == (T::kBK / T::kUmmaK) / 2) {
              const bool more = !(last_tile && ks + 1 == k_steps);
              have_full = more && mbar_test_wait(full_bar((it + 1) % T::kStages), ((it + 1) / T::kStages) & 1);
            }
            const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
            if constexpr (T::kFmt == kFmtF16)
              umma_f16_ss(d_tmem, a_desc + ((kk * a_adv) >> 4), b_desc + ((kk * b_adv) >> 4), idesc, acc);
            else
              umma_tf32_ss(d_tmem, a_desc + ((kk * a_adv) >> 4), b_desc + ((kk * b_adv) >> 4), idesc, acc);
          }
          umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(accfull_bar(a));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    uint32_t tcount = 0;
    bool ok = true;
    TOut* C = reinterpret_cast<TOut*>(args.C);
    const bool scaled = args.alpha != 1.f || args.beta != 0.f;
    for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++tcount) {
      unsigned tm, tn;
      tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
      const int a = tcount % T::kAccBufs;
      if (!(ok = mbar_wait_warp(accfull_bar(a), (tcount / T::kAccBufs) & 1, ctx, 4))) break;
      tc_fence_after();
      const int row = tm * T::kBM + quad * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + a * T::kBN;
#pragma unroll 1
      for (int c = 0; c < T::kBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_x32(t_row + c * 32, v);
        tmem_wait_ld();
        const int col0 = tn * T::kBN + c * 32;
        if (row < args.m) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + j < args.n) {
              float f = __uint_as_float(v[j]);
              TOut* dst = C + row + static_cast<long long>(col0 + j) * args.ldC;
              if (scaled) {  // C = alpha * A.B^T + beta * C (the epilogue the reference leaves as a stub, gemm_tc.hpp:241)
                f *= args.alpha;
                if (args.beta != 0.f) f += args.beta * static_cast<float>(*dst);
              }
              if constexpr (sizeof(TOut) == 2) *dst = __float2half_rn(f);
              else *dst = f;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(accempty_bar(a));
    }
  }

  // ---------------------------------------------------------------------- teardown
#ifdef B200_PROFILE_WAITS
  if (threadIdx.x == 0) {  // site 63: cycles this CTA ran
    ctx.prof_cycles[7] += static_cast<unsigned long long>(clock64() - kernel_c0);
    ctx.prof_count[7] += 1u;
    ctx.prof_site[7] = 63;
  }
#endif
  wait_profile_flush(ctx);
  __syncthreads();
  if (*abort_flag) {
    // Give copies and MMAs that were already issued time to land before shared and tensor memory go away.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

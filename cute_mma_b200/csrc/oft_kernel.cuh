// Fused OFT product  C[M,N] = sum_kb  half(A_kb . Rblk(g,kb)^T) . B_kb^T   (fp16 in, fp32 accumulate,
// fp16 out), the operator of the reference's oft_device / oft_ar / oft_arb
// (cute_oft_coop_pc.cu:363-479, 19-186, 188-361) re-designed for sm_100a.
//
// The reference hands one b-wide slice of A.R from producer warps to consumer warps through shared
// memory and named barriers, once per b (= 8) columns of K.  Here the rotated slice never leaves the
// SM's tensor memory:
//   MMA1   XRacc[128 x U] (fp32, TMEM)  = A_tile[128 x U] . Rblk^T           (tcgen05.mma, N = b)
//   cvt    XR16 [128 x U] (fp16, TMEM)  = round-to-nearest-even(XRacc)         (tcgen05.ld / st)
//   MMA2   acc  [128 x bN] (fp32, TMEM) += XR16 . B_tile[bN x U]^T             (A operand from TMEM)
// with U = max(b, 64) columns of K per "unit".  Warp roles:
//   warp 0      TMA producer of the {A, R} ring        warp 1      TMA producer of the {B} ring
//   warp 2      issues both MMAs                       warp 3      allocates / frees tensor memory
//   warps 4..7  fp32 -> fp16 conversion of XR          warps 8..11 epilogue (TMEM -> fp16 -> C)
// MMA1 of unit u+L is issued ahead of MMA2 of unit u, so the conversion of unit u+1.. overlaps the
// main contraction.  All hand-offs are mbarriers with bounded waits.
#pragma once
#include "ptx.cuh"

namespace b200 {

template <int kB_, int kBN_, int kS1_, int kS2_>
struct OftTraits {
  static constexpr int kB = kB_;                       // reconn_sz: edge of one orthogonal block
  static constexpr int kBM = 128;
  static constexpr int kBN = kBN_;
  static constexpr int kBK = 64;                       // fp16 columns of K per shared-memory stage (128 bytes)
  static constexpr int kUnitK = kB > 64 ? kB : 64;     // K columns per XR hand-off
  static constexpr int kStagesPerUnit = kUnitK / kBK;  // 1, or 2 for b = 128
  static constexpr int kS1 = kS1_;                     // {A, R} ring depth
  static constexpr int kS2 = kS2_;                     // {B} ring depth
  static constexpr int kABytes = kBM * 128;
  static constexpr int kRBytes = kB * 128;             // R tile: b rows (q) x 64 columns of K
  static constexpr int kS1Bytes = kABytes + kRBytes;
  static constexpr int kS2Bytes = kBN * 128;
  // tensor-memory budget (512 columns of 32 bits per SM)
  static constexpr int kXrAccBufs = (kBN + 2 * kUnitK + 2 * (kUnitK / 2) <= 512) ? 2 : 1;
  static constexpr int kXrHBufs = (kBN + kXrAccBufs * kUnitK + 3 * (kUnitK / 2) <= 512) ? 3 : 2;
  static constexpr int kLookahead = kXrAccBufs;        // MMA1 runs this many units ahead of MMA2
  static constexpr int kColAcc = 0;
  static constexpr int kColXrAcc = kBN;
  static constexpr int kColXrH = kBN + kXrAccBufs * kUnitK;
  static constexpr int kTmemUsed = kColXrH + kXrHBufs * (kUnitK / 2);
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 384;
  static constexpr int kNumBars = 2 * kS1 + 2 * kS2 + 2 * kXrAccBufs + 2 * kXrHBufs + 2;
  static constexpr int kSmemBytes = kS1 * kS1Bytes + kS2 * kS2Bytes + kNumBars * 8 + 64 + 1024;
  static_assert(kB == 16 || kB == 32 || kB == 64 || kB == 128, "block edge must be 16, 32, 64 or 128");
  static_assert(kBN % 32 == 0 && kBN >= 32 && kBN <= 256, "bN must be a multiple of 32 up to 256");
  static_assert(kTmemUsed <= kTmemCols, "tensor memory budget exceeded");
  static_assert(kSmemBytes <= 232448, "shared memory rings too large");
  static_assert(kRBytes % 1024 == 0, "R tile must keep the next tile 1024-byte aligned");
};

struct OftArgs {
  int m, n, k;
  int group_size;  // columns of N that share one block-diagonal R; a multiple of bN
  __half* C;
  long long ldC;
  int* status;
};

template <class T>
__global__ void __launch_bounds__(T::kThreads, 1)
oft_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_r,
           const __grid_constant__ CUtensorMap tmap_b, const OftArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t ring1 = smem_base, ring2 = smem_base + T::kS1 * T::kS1Bytes;
  const uint32_t bars = ring2 + T::kS2 * T::kS2Bytes;
  int bi = 0;
  const uint32_t full1 = bars + 8u * bi;  bi += T::kS1;        // {A,R} stage filled       (tx bytes)
  const uint32_t empty1 = bars + 8u * bi; bi += T::kS1;        // {A,R} stage read by MMA1 (commit)
  const uint32_t full2 = bars + 8u * bi;  bi += T::kS2;        // {B} stage filled
  const uint32_t empty2 = bars + 8u * bi; bi += T::kS2;        // {B} stage read by MMA2
  const uint32_t xa_full = bars + 8u * bi;  bi += T::kXrAccBufs;   // XRacc written by MMA1
  const uint32_t xa_empty = bars + 8u * bi; bi += T::kXrAccBufs;   // XRacc read by the converters
  const uint32_t xh_full = bars + 8u * bi;  bi += T::kXrHBufs;     // XR16 written by the converters
  const uint32_t xh_empty = bars + 8u * bi; bi += T::kXrHBufs;     // XR16 read by MMA2
  const uint32_t acc_full = bars + 8u * bi;  bi += 1;
  const uint32_t acc_empty = bars + 8u * bi; bi += 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + (bars - smem_base) + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles_m = (args.m + T::kBM - 1) / T::kBM, tiles_n = (args.n + T::kBN - 1) / T::kBN;
  const unsigned num_tiles = tiles_m * tiles_n;
  const int units = (args.k + T::kUnitK - 1) / T::kUnitK;  // K is a multiple of b; a ragged last 64-wide stage is zero filled
  unsigned my_tiles = 0;
  if (blockIdx.x < num_tiles) my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
  const unsigned total_units = my_tiles * units;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < T::kS1; ++s) { mbar_init(full1 + 8 * s, 1); mbar_init(empty1 + 8 * s, 1); }
    for (int s = 0; s < T::kS2; ++s) { mbar_init(full2 + 8 * s, 1); mbar_init(empty2 + 8 * s, 1); }
    for (int i = 0; i < T::kXrAccBufs; ++i) { mbar_init(xa_full + 8 * i, 1); mbar_init(xa_empty + 8 * i, 128); }
    for (int i = 0; i < T::kXrHBufs; ++i) { mbar_init(xh_full + 8 * i, 128); mbar_init(xh_empty + 8 * i, 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 128);
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_r);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 3) {
    tmem_alloc(smem_u32(tmem_slot), T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // -------------------------------------------------------------- producer of the {A, R} ring
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        unsigned tm, tn;
        tile_coord(tiles_m, tiles_n, tile, tm, tn);
        const int m0 = tm * T::kBM;
        const int r_row0 = ((tn * T::kBN) / args.group_size) * T::kB;  // first stored R row of this tile's group
        for (int st = 0; st < units * T::kStagesPerUnit; ++st, ++it) {
          const int s = it % T::kS1;
          if (!(ok = mbar_wait(empty1 + 8 * s, ((it / T::kS1) & 1) ^ 1, ctx, 10))) break;
          mbar_expect_tx(full1 + 8 * s, T::kS1Bytes);
          const uint32_t a_dst = ring1 + s * T::kS1Bytes;
          tma_load_2d(a_dst, &tmap_a, full1 + 8 * s, st * T::kBK, m0);
          tma_load_2d(a_dst + T::kABytes, &tmap_r, full1 + 8 * s, st * T::kBK, r_row0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- producer of the {B} ring
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        unsigned tm, tn;
        tile_coord(tiles_m, tiles_n, tile, tm, tn);
        const int n0 = tn * T::kBN;
        for (int st = 0; st < units * T::kStagesPerUnit; ++st, ++it) {
          const int s = it % T::kS2;
          if (!(ok = mbar_wait(empty2 + 8 * s, ((it / T::kS2) & 1) ^ 1, ctx, 11))) break;
          mbar_expect_tx(full2 + 8 * s, T::kS2Bytes);
          tma_load_2d(ring2 + s * T::kS2Bytes, &tmap_b, full2 + 8 * s, st * T::kBK, n0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc1 = umma_idesc(kFmtF16, 0, 0, T::kBM, T::kB);
      constexpr uint32_t idesc2 = umma_idesc(kFmtF16, 0, 0, T::kBM, T::kBN);
      uint32_t it1 = 0, it2 = 0;  // stage counters of the two rings as consumed by MMA1 / MMA2
      bool ok = true;
      // g enumerates this CTA's units over all of its tiles; MMA1 leads MMA2 by kLookahead units.
      for (unsigned g = 0; ok && g < total_units + T::kLookahead; ++g) {
        if (g < total_units) {
          // ---- MMA1(g): XRacc = A_tile . Rblk^T
          const int xa = g % T::kXrAccBufs;
          if (!(ok = mbar_wait(xa_empty + 8 * xa, ((g / T::kXrAccBufs) & 1) ^ 1, ctx, 20))) break;
          const uint32_t d1 = tmem_base + T::kColXrAcc + xa * T::kUnitK;
#pragma unroll
          for (int su = 0; su < T::kStagesPerUnit; ++su, ++it1) {
            const int s = it1 % T::kS1;
            if (!(ok = mbar_wait(full1 + 8 * s, (it1 / T::kS1) & 1, ctx, 21))) break;
            tc_fence_after();
            const uint32_t a_src = ring1 + s * T::kS1Bytes;
            const uint64_t a_desc = umma_desc_sw128(a_src, 16, 1024), r_desc = umma_desc_sw128(a_src + T::kABytes, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              // b < 64: the stage holds 64/b diagonal blocks; slice kk belongs to block (kk*16)/b and
              // lands in XRacc columns [blk*b, blk*b+b).  b >= 64: one block, accumulated over the unit.
              const int blk = (T::kB < 64) ? (kk * 16) / T::kB : 0;
              const uint32_t accum = (T::kB < 64) ? (((kk * 16) % T::kB) != 0) : ((su > 0 || kk > 0) ? 1u : 0u);
              umma_f16_ss(d1 + blk * T::kB, umma_desc_advance(a_desc, kk * 32), umma_desc_advance(r_desc, kk * 32), idesc1, accum);
            }
            umma_commit(empty1 + 8 * s);
          }
          if (!ok) break;
          umma_commit(xa_full + 8 * xa);
        }
        if (g >= static_cast<unsigned>(T::kLookahead)) {
          // ---- MMA2(u): acc += XR16 . B_tile^T
          const unsigned u = g - T::kLookahead;
          const int ku = u % units;  // unit index inside its tile
          const int xh = u % T::kXrHBufs;
          if (ku == 0) {
            const unsigned t = u / units;
            if (!(ok = mbar_wait(acc_empty, (t & 1) ^ 1, ctx, 22))) break;
          }
          if (!(ok = mbar_wait(xh_full + 8 * xh, (u / T::kXrHBufs) & 1, ctx, 23))) break;
          tc_fence_after();
          const uint32_t a_tmem = tmem_base + T::kColXrH + xh * (T::kUnitK / 2);
#pragma unroll
          for (int su = 0; su < T::kStagesPerUnit; ++su, ++it2) {
            const int s = it2 % T::kS2;
            if (!(ok = mbar_wait(full2 + 8 * s, (it2 / T::kS2) & 1, ctx, 24))) break;
            tc_fence_after();
            const uint64_t b_desc = umma_desc_sw128(ring2 + s * T::kS2Bytes, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              const uint32_t accum = (ku > 0 || su > 0 || kk > 0) ? 1u : 0u;
              umma_f16_ts(tmem_base + T::kColAcc, a_tmem + su * (T::kBK / 2) + kk * 8, umma_desc_advance(b_desc, kk * 32), idesc2, accum);
            }
            umma_commit(empty2 + 8 * s);
          }
          if (!ok) break;
          umma_commit(xh_empty + 8 * xh);
          if (ku == units - 1) umma_commit(acc_full);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // -------------------------------------------------------------- converters: XRacc (fp32) -> XR16 (fp16)
    const int quad = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (unsigned g = 0; ok && g < total_units; ++g) {
      const int xa = g % T::kXrAccBufs, xh = g % T::kXrHBufs;
      if (!(ok = mbar_wait_warp(xa_full + 8 * xa, (g / T::kXrAccBufs) & 1, ctx, 30))) break;
      tc_fence_after();
      const uint32_t src = tmem_base + lane_off + T::kColXrAcc + xa * T::kUnitK;
      const uint32_t dst = tmem_base + lane_off + T::kColXrH + xh * (T::kUnitK / 2);
#pragma unroll
      for (int h = 0; h < T::kUnitK / 64; ++h) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(src + h * 64, v0);
        tmem_ld_x32(src + h * 64 + 32, v1);
        tmem_wait_ld();
        if (h == T::kUnitK / 64 - 1) {
          // XRacc is free again as soon as its last columns sit in registers
          tc_fence_before();
          mbar_arrive(xa_empty + 8 * xa);
        }
        uint32_t p0[16], p1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 a = __floats2half2_rn(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
          __half2 b = __floats2half2_rn(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
          p0[j] = *reinterpret_cast<uint32_t*>(&a);
          p1[j] = *reinterpret_cast<uint32_t*>(&b);
        }
        if (h == 0) {
          if (!(ok = mbar_wait_warp(xh_empty + 8 * xh, ((g / T::kXrHBufs) & 1) ^ 1, ctx, 31))) break;
          tc_fence_after();
        }
        tmem_st_x16(dst + h * 32, p0);
        tmem_st_x16(dst + h * 32 + 16, p1);
      }
      if (!ok) break;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(xh_full + 8 * xh);
    }
  } else if (warp >= 8) {
    // -------------------------------------------------------------- epilogue: acc -> fp16 -> row-major C
    const int quad = warp & 3;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + T::kColAcc;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(args.C) & 15) == 0) && ((args.ldC & 7) == 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++tcount) {
      unsigned tm, tn;
      tile_coord(tiles_m, tiles_n, tile, tm, tn);
      if (!(ok = mbar_wait_warp(acc_full, tcount & 1, ctx, 40))) break;
      tc_fence_after();
      const int row = tm * T::kBM + quad * 32 + lane;
      __half* c_row = args.C + static_cast<long long>(row) * args.ldC;
#pragma unroll 1
      for (int c = 0; c < T::kBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_x32(t_row + c * 32, v);
        tmem_wait_ld();
        const int col0 = tn * T::kBN + c * 32;
        if (row < args.m) {
          uint32_t p[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __half2 h2 = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            p[j] = *reinterpret_cast<uint32_t*>(&h2);
          }
          if (vec_ok && col0 + 32 <= args.n) {
            uint4* dst = reinterpret_cast<uint4*>(c_row + col0);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_uint4(p[4 * q], p[4 * q + 1], p[4 * q + 2], p[4 * q + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < args.n) c_row[col0 + j] = reinterpret_cast<const __half*>(p)[j];
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty);
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

// Fused OFT product  C[M,N] = sum_kb  half(A_kb . Rblk(g,kb)^T) . B_kb^T   (fp16 in, fp32 accumulate,
// fp16 out), the operator of the reference's oft_device / oft_ar / oft_arb
// (cute_oft_coop_pc.cu:363-479, 19-186, 188-361) re-designed for sm_100a.
//
// The reference hands one b-wide slice of A.R from producer warps to consumer warps through shared
// memory and named barriers, once per b (= 8) columns of K.  Here the rotated slice never leaves the
// SM's tensor memory:
//   MMA1   XR[128 x U] (fp32, TMEM)     = A_tile[128 x U] . Rblk^T           (tcgen05.mma, N = b)
//   cvt    XR[128 x U] (fp16, TMEM)     = round-to-nearest-even(XR), in place  (tcgen05.ld / st)
//   MMA2   acc[128 x bN] (fp32, TMEM)  += XR . B_tile[bN x U]^T                (A operand from TMEM)
// with U = max(b, 64) columns of K per "unit".  Warp roles:
//   warp 0      TMA producer of the {A, R} ring        warp 1      TMA producer of the {B} ring
//   warp 2      issues MMA1                            warp 3      owns tensor memory, issues MMA2
//   warps 4..7  fp32 -> fp16 conversion of XR          warps 8..11 epilogue (TMEM -> fp16 -> C)
// MMA1 runs ahead of MMA2 by as many units as there are XR buffers in tensor memory, so the conversion of
// the next units overlaps the main contraction.  All hand-offs are mbarriers with bounded waits.
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
  // tensor-memory budget (512 columns of 32 bits per SM): the accumulator plus as many XR buffers
  // as fit.  One XR buffer holds a unit twice in turn: first the fp32 result of MMA1 (kUnitK columns),
  // then, converted in place, its fp16 image in the first kUnitK/2 columns, which MMA2 reads as A.
  static constexpr int kXrBufs = (512 - kBN) / kUnitK;
  static constexpr int kColAcc = 0;
  static constexpr int kColXr = kBN;
  static constexpr int kTmemUsed = kBN + kXrBufs * kUnitK;
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 384;
  static constexpr int kNumBars = 2 * kS1 + 2 * kS2 + (2 + kStagesPerUnit) * kXrBufs + 2;
  static constexpr int kSmemBytes = kS1 * kS1Bytes + kS2 * kS2Bytes + kNumBars * 8 + 64 + 1024;
  static_assert(kB == 16 || kB == 32 || kB == 64 || kB == 128, "block edge must be 16, 32, 64 or 128");
  static_assert(kBN % 32 == 0 && kBN >= 32 && kBN <= 256, "bN must be a multiple of 32 up to 256");
  static_assert(kTmemUsed <= kTmemCols && kXrBufs >= 2, "tensor memory budget exceeded");
  // A tile configuration may fit some block edges and not others (the R tile grows with b); the
  // launcher reports an unsupported shape for the ones that do not fit instead of failing the build.
  static constexpr bool kFits = kSmemBytes <= 232448;
  static_assert(kRBytes % 1024 == 0, "R tile must keep the next tile 1024-byte aligned");
};

struct OftArgs {
  int m, n, k;
  int group_size;  // columns of N that share one block-diagonal R; a multiple of bN
  __half* C;
  long long ldC;
  int* status;
  int raster;  // 0: z-curve tile order; g > 0: bands of g tile rows
  unsigned long long hint_a, hint_b;  // L2 eviction priority of the A and B tile loads (pair kernel)
  int tile_sync;  // pair kernel: producers of all CTAs start each tile round together
  int* rounds;    // 4 zeroed counters of this launch's tile rounds (tile_sync only)
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
  const uint32_t x_acc = bars + 8u * bi;   bi += T::kXrBufs;   // XR buffer holds the fp32 result of MMA1 (commit)
  const uint32_t x_half = bars + 8u * bi;  bi += T::kXrBufs * T::kStagesPerUnit;  // fp16 image of one 64-column slice ready (converters)
  const uint32_t x_empty = bars + 8u * bi; bi += T::kXrBufs;   // XR buffer read by MMA2 (commit)
  const uint32_t acc_full = bars + 8u * bi;  bi += 1;
  const uint32_t acc_empty = bars + 8u * bi; bi += 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + (bars - smem_base) + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};
#ifdef B200_PROFILE_WAITS
  const long long kernel_c0 = clock64();
#endif

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
    for (int i = 0; i < T::kXrBufs; ++i) { mbar_init(x_acc + 8 * i, 1); mbar_init(x_empty + 8 * i, 1); }
    for (int i = 0; i < T::kXrBufs * T::kStagesPerUnit; ++i) mbar_init(x_half + 8 * i, 128);
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

  // The epilogue keeps a whole accumulator row (bN/2 packed registers) per thread; the copy / issue
  // warps need few registers and the converters a moderate number, so the warpgroups trade registers.
  // (each role issues its own setmaxnreg at the top of its branch: warps 0..3 give registers up,
  // warps 4..7 keep a moderate number, warps 8..11 take the rest)

  if (warp == 0) {
    // -------------------------------------------------------------- producer of the {A, R} ring
    setmaxnreg_dec<96>();
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        unsigned tm, tn;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
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
    setmaxnreg_dec<96>();
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        unsigned tm, tn;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
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
    // -------------------------------------------------------------- issuer of MMA1: XRacc = A_tile . Rblk^T
    // The two MMAs have their own issuing threads: one thread cannot issue both at the rate the
    // tensor pipe retires them, and the mbarriers already carry every ordering between the two.
    setmaxnreg_dec<96>();
    if (lane == 0) {
      // The tensor pipe queues only a couple of MMAs per issuing thread, so whatever this thread does
      // between two stages (barrier waits, commits) is time the pipe may sit idle.  Each stage
      // therefore looks at the next stage's barriers (test_wait, non-blocking) after its first two
      // MMAs are queued, and the next stage only waits for what that look did not find complete.
      constexpr uint32_t idesc1 = umma_idesc(kFmtF16, 0, 0, T::kBM, T::kB);
      const uint64_t a_desc0 = umma_desc_sw128(ring1, 16, 1024), r_desc0 = umma_desc_sw128(ring1 + T::kABytes, 16, 1024);
      const unsigned total_stages = total_units * T::kStagesPerUnit;
      int s = 0, xb = 0, su = 0;
      uint32_t ph_s = 0, ph_xb = 0;
      unsigned g = 0;
      bool have_full = false, have_buf = false, ok = true;
      for (unsigned j = 0; ok && j < total_stages; ++j) {
        if (su == 0) {
          if (!have_buf && !(ok = mbar_wait(x_empty + 8 * xb, ph_xb ^ 1, ctx, 20))) break;  // MMA2 is done with this buffer
          trace_stamp(ctx, g, 0);
        }
        if (!have_full && !(ok = mbar_wait(full1 + 8 * s, ph_s, ctx, 21))) break;
        tc_fence_after();
        const uint32_t d1 = tmem_base + T::kColXr + xb * T::kUnitK;
        const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (T::kS1Bytes >> 4));
        const uint64_t r_desc = r_desc0 + static_cast<uint64_t>(s * (T::kS1Bytes >> 4));
        const bool unit_ends = (su == T::kStagesPerUnit - 1);
        int s_n = s + 1, xb_n = xb;
        uint32_t ph_s_n = ph_s, ph_xb_n = ph_xb;
        if (s_n == T::kS1) { s_n = 0; ph_s_n ^= 1; }
        if (unit_ends && ++xb_n == T::kXrBufs) { xb_n = 0; ph_xb_n ^= 1; }
#pragma unroll
        for (int kk = 0; kk < T::kBK / 16; ++kk) {
          if (kk == 2) {
            const bool more = j + 1 < total_stages;
            have_full = more && mbar_test_wait(full1 + 8 * s_n, ph_s_n);
            have_buf = more && unit_ends && mbar_test_wait(x_empty + 8 * xb_n, ph_xb_n ^ 1);
          }
          // b < 64: the stage holds 64/b diagonal blocks; slice kk belongs to block (kk*16)/b and
          // lands in XR columns [blk*b, blk*b+b).  b >= 64: one block, accumulated over the unit.
          constexpr bool small = T::kB < 64;
          const int blk = small ? (kk * 16) / T::kB : 0;
          const uint32_t accum = small ? ((((kk * 16) % T::kB) != 0) ? 1u : 0u) : ((su > 0 || kk > 0) ? 1u : 0u);
          umma_f16_ss(d1 + blk * T::kB, a_desc + kk * 2, r_desc + kk * 2, idesc1, accum);
        }
        umma_commit(empty1 + 8 * s);
        s = s_n;
        ph_s = ph_s_n;
        if (unit_ends) {
          umma_commit(x_acc + 8 * xb);
          trace_stamp(ctx, g, 1);
          xb = xb_n;
          ph_xb = ph_xb_n;
          su = 0;
          ++g;
        } else {
          ++su;
        }
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    // -------------------------------------------------------------- issuer of MMA2: acc += XR16 . B_tile^T
    setmaxnreg_dec<96>();
    if (lane == 0) {
      constexpr uint32_t idesc2 = umma_idesc(kFmtF16, 0, 0, T::kBM, T::kBN);
      const uint64_t b_desc0 = umma_desc_sw128(ring2, 16, 1024);
      const unsigned total_stages = total_units * T::kStagesPerUnit;
      int s = 0, xb = 0, ku = 0, su = 0;
      uint32_t ph_s = 0, ph_xb = 0, ph_acc = 0;
      unsigned u = 0;
      bool have_full = false, have_half = false, ok = true;
      for (unsigned j = 0; ok && j < total_stages; ++j) {
        // first stage of a tile: the epilogue must have drained the accumulator (never looked at
        // early: the epilogue of this tile cannot start before this thread commits the tile)
        if (su == 0 && ku == 0 && !(ok = mbar_wait(acc_empty, ph_acc ^ 1, ctx, 22))) break;
        if (!have_half && !(ok = mbar_wait(x_half + 8 * (xb * T::kStagesPerUnit + su), ph_xb, ctx, 23))) break;
        if (su == 0) trace_stamp(ctx, u, 4);
        if (!have_full && !(ok = mbar_wait(full2 + 8 * s, ph_s, ctx, 24))) break;
        tc_fence_after();
        const uint32_t a_tmem = tmem_base + T::kColXr + xb * T::kUnitK + su * (T::kBK / 2);
        const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(s * (T::kS2Bytes >> 4));
        const bool unit_ends = (su == T::kStagesPerUnit - 1);
        int s_n = s + 1, xb_n = xb;
        uint32_t ph_s_n = ph_s, ph_xb_n = ph_xb;
        if (s_n == T::kS2) { s_n = 0; ph_s_n ^= 1; }
        if (unit_ends && ++xb_n == T::kXrBufs) { xb_n = 0; ph_xb_n ^= 1; }
        const int su_n = unit_ends ? 0 : su + 1;
#pragma unroll
        for (int kk = 0; kk < T::kBK / 16; ++kk) {
          if (kk == 2) {
            const bool more = j + 1 < total_stages;
            have_full = more && mbar_test_wait(full2 + 8 * s_n, ph_s_n);
            have_half = more && mbar_test_wait(x_half + 8 * (xb_n * T::kStagesPerUnit + su_n), ph_xb_n);
          }
          const uint32_t accum = (su > 0 || kk > 0) ? 1u : (ku > 0 ? 1u : 0u);
          umma_f16_ts(tmem_base + T::kColAcc, a_tmem + kk * 8, b_desc + kk * 2, idesc2, accum);
        }
        // (committing a stage only after the next stage's first MMAs are queued was tried and cost
        // 15-20 % in cycles: the release has to follow its MMAs directly)
        umma_commit(empty2 + 8 * s);
        if (unit_ends) {
          umma_commit(x_empty + 8 * xb);
          if (ku + 1 == units) umma_commit(acc_full);
        }
        s = s_n;
        ph_s = ph_s_n;
        if (unit_ends) {
          trace_stamp(ctx, u, 5);
          xb = xb_n;
          ph_xb = ph_xb_n;
          su = 0;
          ++u;
          if (++ku == units) {
            ku = 0;
            ph_acc ^= 1;
          }
        } else {
          ++su;
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // -------------------------------------------------------------- converters: fp32 -> fp16, in place
    // Each warp owns its 32 lanes.  Columns are converted in 64-wide groups in ascending order, so the
    // fp16 words written to columns [32h, 32h+32) only ever land on fp32 columns already in registers.
    setmaxnreg_dec<152>();
    const int quad = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    int xb = 0;
    uint32_t ph_xb = 0;
    for (unsigned g = 0; ok && g < total_units; ++g) {
      if (!(ok = mbar_wait_warp(x_acc + 8 * xb, ph_xb, ctx, 30))) break;
      tc_fence_after();
      if (threadIdx.x == 128) trace_stamp(ctx, g, 2);
#ifdef B200_PROFILE_WAITS
      const long long cv0 = clock64();
#endif
      const uint32_t buf = tmem_base + lane_off + T::kColXr + xb * T::kUnitK;
#pragma unroll
      for (int h = 0; h < T::kUnitK / 64; ++h) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(buf + h * 64, v0);
        tmem_ld_x32(buf + h * 64 + 32, v1);
        tmem_wait_ld();
        uint32_t p0[16], p1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 a = __floats2half2_rn(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
          __half2 b = __floats2half2_rn(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
          p0[j] = *reinterpret_cast<uint32_t*>(&a);
          p1[j] = *reinterpret_cast<uint32_t*>(&b);
        }
        tmem_st_x16(buf + h * 32, p0);
        tmem_st_x16(buf + h * 32 + 16, p1);
        // each 64-column slice is handed to MMA2 as soon as it is written (b = 128 has two per unit)
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(x_half + 8 * (xb * T::kStagesPerUnit + h));
      }
      if (threadIdx.x == 128) trace_stamp(ctx, g, 3);
#ifdef B200_PROFILE_WAITS
      if (threadIdx.x == 128) { ctx.prof_cycles[3] += clock64() - cv0; ctx.prof_count[3] += 1; ctx.prof_site[3] = 51; }  // unit converted
#endif
      if (++xb == T::kXrBufs) { xb = 0; ph_xb ^= 1; }
    }
  } else if (warp >= 8) {
    // -------------------------------------------------------------- epilogue: acc -> fp16 -> row-major C
    setmaxnreg_inc<248>();
    const int quad = warp & 3;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + T::kColAcc;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(args.C) & 15) == 0) && ((args.ldC & 7) == 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (unsigned tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++tcount) {
      unsigned tm, tn;
      tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
      if (!(ok = mbar_wait_warp(acc_full, tcount & 1, ctx, 40))) break;
      tc_fence_after();
      const int row = tm * T::kBM + quad * 32 + lane;
      __half* c_row = args.C + static_cast<long long>(row) * args.ldC;
      // Drain the whole accumulator row into registers as packed fp16 first and hand the
      // accumulator back to MMA2 before any global store is issued: the stores (one row per lane,
      // 16 bytes per instruction) are slow and would otherwise sit on the tile-to-tile critical path.
      uint32_t p[T::kBN / 2];
#pragma unroll
      for (int c = 0; c < T::kBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_x32(t_row + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 h2 = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          p[c * 16 + j] = *reinterpret_cast<uint32_t*>(&h2);
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty);
      if (row < args.m) {
#pragma unroll
        for (int c = 0; c < T::kBN / 32; ++c) {
          const int col0 = tn * T::kBN + c * 32;
          if (vec_ok && col0 + 32 <= args.n) {
            uint4* dst = reinterpret_cast<uint4*>(c_row + col0);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              dst[q] = make_uint4(p[c * 16 + 4 * q], p[c * 16 + 4 * q + 1], p[c * 16 + 4 * q + 2], p[c * 16 + 4 * q + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < args.n) {
                const uint32_t w = p[c * 16 + j / 2];
                c_row[col0 + j] = __ushort_as_half(static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xFFFFu)));
              }
          }
        }
      }
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
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

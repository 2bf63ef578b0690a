// Fused OFT product on CTA pairs (tcgen05 cta_group::2): same operator, layouts and numerics as
// oft_kernel.cuh (reference: oft_device / oft_ar / oft_arb, cute_oft_coop_pc.cu:363-479), with a
// 256 x bN tile of C shared by two CTAs on neighbouring SMs.
//
// Each CTA loads its own 128 rows of A, its own half of the R tile (b/2 rows of q) and its own half of
// the B tile (bN/2 rows of N): 36 KB instead of 56 KB per 64 columns of K at b = 64.  The even
// ("leader") CTA issues both MMAs for the pair; each CTA converts and stores its own 128 rows.
//   MMA1  XR [256 x U] fp32 = A[256 x U] . Rblk^T     (B operand N = b split over the two CTAs)
//   cvt   in place, per CTA, fp32 -> fp16 (RNE)
//   MMA2  acc[256 x bN] += XR . B[bN x U]^T           (A operand from each CTA's tensor memory)
// Barriers: full1/full2, x_half and acc_empty are used in the leader only and collect both CTAs
// (TMA bytes through the pair form of the copy, 128 + 128 converter / epilogue threads through cluster
// arrives); empty1/empty2, x_acc and acc_full are signalled in both CTAs by multicast tcgen05.commit;
// x_empty stays inside the leader.  No load carries a multicast qualifier.
#pragma once
#include "oft_kernel.cuh"

namespace b200 {

constexpr int oft_gcd(int a, int b) { return b == 0 ? a : oft_gcd(b, a % b); }
constexpr int oft_lcm(int a, int b) { return a / oft_gcd(a, b) * b; }

template <int kB_, int kBN_, int kS1_, int kS2_, int kGT_ = 1>
struct Oft2Traits {
  static constexpr int kB = kB_;
  static constexpr int kBM = 128;                      // rows per CTA; the pair covers 256
  static constexpr int kBN = kBN_;
  static constexpr int kBNHalf = kBN / 2;
  static constexpr int kGT = kGT_;                     // N-groups per tile (group_size = bN / kGT): one R and one XR per group
  static constexpr int kGS = kBN / kGT;                // columns of one group inside the tile (tcgen05 N of MMA2)
  static constexpr int kGSHalf = kGS / 2;              // rows of a group's B sub-tile held by each CTA
  static constexpr int kBK = 64;
  static constexpr int kUnitK = kB > 64 ? kB : 64;
  static constexpr int kStagesPerUnit = kUnitK / kBK;
  static constexpr int kS1 = kS1_;
  static constexpr int kS2 = kS2_;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kRHalfBytes = (kB / 2) * 128;   // this CTA's half of one group's R tile: b/2 rows (q) x 64 columns of K
  static constexpr int kRBytes = kGT * kRHalfBytes;
  static constexpr int kS1Bytes = kABytes + kRBytes;
  static constexpr int kS2Bytes = kBNHalf * 128;
  static constexpr int kXrBufs = (512 - kBN) / kUnitK;
  static constexpr int kColAcc = 0;
  static constexpr int kColXr = kBN;
  static constexpr int kTmemUsed = kBN + kXrBufs * kUnitK;
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 384;
  static constexpr int kNumBars = 2 * kS1 + 2 * kS2 + (2 + kStagesPerUnit) * kXrBufs + 2;
  static constexpr int kSmemBytes = kS1 * kS1Bytes + kS2 * kS2Bytes + kNumBars * 8 + 64 + 1024;
  static_assert(kB == 16 || kB == 32 || kB == 64 || kB == 128, "block edge must be 16, 32, 64 or 128");
  static_assert(kBN % 64 == 0 && kBN >= 64 && kBN <= 256, "bN must be a multiple of 64 up to 256");
  static_assert(kTmemUsed <= kTmemCols && kXrBufs >= 2, "tensor memory budget exceeded");
  static_assert(kRHalfBytes % 1024 == 0, "R half-tile must keep the next tile 1024-byte aligned");
  static_assert(kGT == 1 || (kStagesPerUnit == 1 && kGS % 16 == 0 && (kGSHalf * 128) % 1024 == 0), "several groups per tile need b <= 64 and group_size >= 16");
  static constexpr bool kFits = kSmemBytes <= 232448;
  // Issue loops unrolled over a whole period of (ring slot, XR buffer): every barrier address, parity and
  // descriptor offset in them is a constant plus a base register.  Used when the tile holds one N-group and
  // the period is short; otherwise the loops that track slot and phase at run time.  Measured (cycles per 64
  // columns of K at M 16384, K = N 4096): b 128 926 -> 883, b 32 715 -> 704, but b 64 714 -> 726 (the hand-off
  // chain MMA1 -> conversion -> MMA2, not the issuing threads' integer work, bounds this kernel), so 64 x 64
  // blocks keep the run-time loops.
  static constexpr int kPeriod1 = oft_lcm(kS1, kXrBufs * kStagesPerUnit);
  static constexpr int kPeriod2 = oft_lcm(kS2, kXrBufs * kStagesPerUnit);
  static constexpr bool kUnrolledIssue = kGT == 1 && kB != 64 && kPeriod1 <= 24 && kPeriod2 <= 24;
};

template <class T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T::kThreads, 1)
oft2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_r,
            const __grid_constant__ CUtensorMap tmap_b, const OftArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t ring1 = smem_base, ring2 = smem_base + T::kS1 * T::kS1Bytes;
  const uint32_t bars = ring2 + T::kS2 * T::kS2Bytes;
  int bi = 0;
  const uint32_t full1 = bars + 8u * bi;  bi += T::kS1;
  const uint32_t empty1 = bars + 8u * bi; bi += T::kS1;
  const uint32_t full2 = bars + 8u * bi;  bi += T::kS2;
  const uint32_t empty2 = bars + 8u * bi; bi += T::kS2;
  const uint32_t x_acc = bars + 8u * bi;   bi += T::kXrBufs;
  const uint32_t x_half = bars + 8u * bi;  bi += T::kXrBufs * T::kStagesPerUnit;
  const uint32_t x_empty = bars + 8u * bi; bi += T::kXrBufs;
  const uint32_t acc_full = bars + 8u * bi;  bi += 1;
  const uint32_t acc_empty = bars + 8u * bi; bi += 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + (bars - smem_base) + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};
#ifdef B200_PROFILE_WAITS
  const long long kernel_c0 = clock64();
#endif

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const unsigned pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const unsigned tiles_m = (args.m + 2 * T::kBM - 1) / (2 * T::kBM), tiles_n = (args.n + T::kBN - 1) / T::kBN;
  const unsigned num_tiles = tiles_m * tiles_n;
  const int units = (args.k + T::kUnitK - 1) / T::kUnitK;
  unsigned my_tiles = 0;
  if (pair < num_tiles) my_tiles = (num_tiles - pair + num_pairs - 1) / num_pairs;
  const unsigned total_units = my_tiles * units * T::kGT;  // XR hand-offs of this CTA: one per unit and per N-group of the tile

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < T::kS1; ++s) { mbar_init(full1 + 8 * s, 1); mbar_init(empty1 + 8 * s, 1); }
    for (int s = 0; s < T::kS2; ++s) { mbar_init(full2 + 8 * s, 1); mbar_init(empty2 + 8 * s, 1); }
    for (int i = 0; i < T::kXrBufs; ++i) { mbar_init(x_acc + 8 * i, 1); mbar_init(x_empty + 8 * i, 1); }
    for (int i = 0; i < T::kXrBufs * T::kStagesPerUnit; ++i) mbar_init(x_half + 8 * i, 256);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 256);
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_r);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 3) {
    tmem_alloc_pair(smem_u32(tmem_slot), T::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // -------------------------------------------------------------- producer of the {A, R} ring (both CTAs)
    setmaxnreg_dec<96>();
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      unsigned done_rounds = 0, sync_target = 0;
      for (unsigned tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        if (args.tile_sync && done_rounds > 0) {
          if (!(ok = tile_round_sync(args.rounds + rank, sync_target, ctx, 12))) break;
        }
        {  // every pair that had a tile in this round takes part in the next rendezvous
          const unsigned first = tile - pair, left = num_tiles - first;
          sync_target += left < num_pairs ? left : num_pairs;
          ++done_rounds;
        }
        unsigned tm, tn;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
        const int m0 = tm * 2 * T::kBM + rank * T::kBM;
        const int r_row0 = ((tn * T::kBN) / args.group_size) * T::kB + rank * (T::kB / 2);  // this CTA's half of the first group's block rows
        for (int st = 0; st < units * T::kStagesPerUnit; ++st, ++it) {
          const int s = it % T::kS1;
          if (!(ok = mbar_wait(empty1 + 8 * s, ((it / T::kS1) & 1) ^ 1, ctx, 10))) break;
          if (rank == 0) mbar_expect_tx(full1 + 8 * s, 2 * T::kS1Bytes);
          const uint32_t a_dst = ring1 + s * T::kS1Bytes;
          tma_load_2d_pair_hint(a_dst, &tmap_a, full1 + 8 * s, st * T::kBK, m0, args.hint_a);
#pragma unroll
          for (int gl = 0; gl < T::kGT; ++gl)
            tma_load_2d_pair_hint(a_dst + T::kABytes + gl * T::kRHalfBytes, &tmap_r, full1 + 8 * s, st * T::kBK, r_row0 + gl * T::kB, kL2EvictLast);
        }
      }
      // leaving after its last round, this thread still counts for the rendezvous the others make
      if (ok && args.tile_sync && done_rounds > 0) atomicAdd(args.rounds + rank, 1);
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- producer of the {B} ring (both CTAs)
    setmaxnreg_dec<96>();
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      unsigned done_rounds = 0, sync_target = 0;
      for (unsigned tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        if (args.tile_sync && done_rounds > 0) {
          if (!(ok = tile_round_sync(args.rounds + 2 + rank, sync_target, ctx, 13))) break;
        }
        {
          const unsigned first = tile - pair, left = num_tiles - first;
          sync_target += left < num_pairs ? left : num_pairs;
          ++done_rounds;
        }
        unsigned tm, tn;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
        const int n0 = tn * T::kBN + rank * T::kGSHalf;  // this CTA's half of each group's columns
        for (int st = 0; st < units * T::kStagesPerUnit; ++st, ++it) {
          const int s = it % T::kS2;
          if (!(ok = mbar_wait(empty2 + 8 * s, ((it / T::kS2) & 1) ^ 1, ctx, 11))) break;
          if (rank == 0) mbar_expect_tx(full2 + 8 * s, 2 * T::kS2Bytes);
#pragma unroll
          for (int gl = 0; gl < T::kGT; ++gl)
            tma_load_2d_pair_hint(ring2 + s * T::kS2Bytes + gl * T::kGSHalf * 128, &tmap_b, full2 + 8 * s, st * T::kBK, n0 + gl * T::kGS, args.hint_b);
        }
      }
      if (ok && args.tile_sync && done_rounds > 0) atomicAdd(args.rounds + 2 + rank, 1);
    }
    __syncwarp();
  } else if (warp == 2) {
    // -------------------------------------------------------------- issuer of MMA1 (leader CTA only)
    setmaxnreg_dec<96>();
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc1 = umma_idesc(kFmtF16, 0, 0, 2 * T::kBM, T::kB);
      const uint64_t a_desc0 = umma_desc_sw128(ring1, 16, 1024), r_desc0 = umma_desc_sw128(ring1 + T::kABytes, 16, 1024);
      const unsigned total_stages = my_tiles * units * T::kStagesPerUnit;
      if constexpr (T::kUnrolledIssue) {
        constexpr int P = T::kPeriod1, SPU = T::kStagesPerUnit, XB = T::kXrBufs;
        uint32_t par_s = 0, par_x = 0;  // parities of ring slot 0 / XR buffer 0 at the start of the period
        bool have_full = false, have_buf = false, ok = true;
        for (unsigned base = 0; ok && base < total_stages; base += P) {
#pragma unroll
          for (int j = 0; j < P; ++j) {
            if (base + j >= total_stages) break;
            const int sl = j % T::kS1, su = j % SPU, xb = (j / SPU) % XB;
            const uint32_t p_full = par_s ^ ((j / T::kS1) & 1), p_x = par_x ^ (((j / SPU) / XB) & 1);
            if (su == 0 && !have_buf && !(ok = mbar_wait(x_empty + 8 * xb, p_x ^ 1, ctx, 20))) break;
            if (!have_full && !(ok = mbar_wait(full1 + 8 * sl, p_full, ctx, 21))) break;
            tc_fence_after();
            const uint32_t d1 = tmem_base + T::kColXr + xb * T::kUnitK;
            const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(sl * (T::kS1Bytes >> 4));
            const uint64_t r_desc = r_desc0 + static_cast<uint64_t>(sl * (T::kS1Bytes >> 4));
            const bool unit_ends = (su == SPU - 1);
            const int jn = j + 1;  // the next stage (jn == P: slot 0 of the next period, whose base parities have flipped)
#pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              if (kk == 2) {
                have_full = mbar_test_wait(full1 + 8 * (jn % T::kS1), par_s ^ ((jn / T::kS1) & 1));
                have_buf = unit_ends && mbar_test_wait(x_empty + 8 * ((jn / SPU) % XB), par_x ^ (((jn / SPU) / XB) & 1) ^ 1);
              }
              constexpr bool small = T::kB < 64;
              const int blk = small ? (kk * 16) / T::kB : 0;
              const uint32_t accum = small ? ((((kk * 16) % T::kB) != 0) ? 1u : 0u) : ((su > 0 || kk > 0) ? 1u : 0u);
              umma_f16_ss_pair(d1 + blk * T::kB, a_desc + kk * 2, r_desc + kk * 2, idesc1, accum);
            }
            umma_commit_pair(empty1 + 8 * sl, 3);
            if (unit_ends) umma_commit_pair(x_acc + 8 * xb, 3);  // the converters of both CTAs start on their halves
          }
          par_s ^= (P / T::kS1) & 1;
          par_x ^= ((P / SPU) / XB) & 1;
        }
      } else {
        int s = 0, xb = 0, su = 0;
        uint32_t ph_s = 0, ph_xb = 0;
        bool have_full = false, have_buf = false, ok = true;
        for (unsigned j = 0; ok && j < total_stages; ++j) {
          if (!have_full && !(ok = mbar_wait(full1 + 8 * s, ph_s, ctx, 21))) break;
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (T::kS1Bytes >> 4));
          const bool unit_ends = (su == T::kStagesPerUnit - 1);
          int s_n = s + 1;
          uint32_t ph_s_n = ph_s;
          if (s_n == T::kS1) { s_n = 0; ph_s_n ^= 1; }
  #pragma unroll
          for (int gl = 0; gl < T::kGT; ++gl) {  // one XR per N-group of the tile, all from the same stage of A
            if (su == 0 && !have_buf && !(ok = mbar_wait(x_empty + 8 * xb, ph_xb ^ 1, ctx, 20))) break;
            tc_fence_after();
            const uint32_t d1 = tmem_base + T::kColXr + xb * T::kUnitK;
            const uint64_t r_desc = r_desc0 + static_cast<uint64_t>((s * T::kS1Bytes + gl * T::kRHalfBytes) >> 4);
            int xb_n = xb;
            uint32_t ph_xb_n = ph_xb;
            if (unit_ends && ++xb_n == T::kXrBufs) { xb_n = 0; ph_xb_n ^= 1; }
  #pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              if (kk == 2) {
                const bool more = (j + 1 < total_stages) || (gl + 1 < T::kGT);
                if (gl == T::kGT - 1) have_full = (j + 1 < total_stages) && mbar_test_wait(full1 + 8 * s_n, ph_s_n);
                have_buf = more && unit_ends && mbar_test_wait(x_empty + 8 * xb_n, ph_xb_n ^ 1);
              }
              constexpr bool small = T::kB < 64;
              const int blk = small ? (kk * 16) / T::kB : 0;
              const uint32_t accum = small ? ((((kk * 16) % T::kB) != 0) ? 1u : 0u) : ((su > 0 || kk > 0) ? 1u : 0u);
              umma_f16_ss_pair(d1 + blk * T::kB, a_desc + kk * 2, r_desc + kk * 2, idesc1, accum);
            }
            if (unit_ends) {
              umma_commit_pair(x_acc + 8 * xb, 3);  // the converters of both CTAs start on their halves
              xb = xb_n;
              ph_xb = ph_xb_n;
            }
          }
          if (!ok) break;
          umma_commit_pair(empty1 + 8 * s, 3);
          s = s_n;
          ph_s = ph_s_n;
          su = unit_ends ? 0 : su + 1;
        }
          }
}
    __syncwarp();
  } else if (warp == 3) {
    // -------------------------------------------------------------- issuer of MMA2 (leader CTA only)
    setmaxnreg_dec<96>();
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc2 = umma_idesc(kFmtF16, 0, 0, 2 * T::kBM, T::kGS);
      const uint64_t b_desc0 = umma_desc_sw128(ring2, 16, 1024);
      const unsigned total_stages = my_tiles * units * T::kStagesPerUnit;
      if constexpr (T::kUnrolledIssue) {
        constexpr int P = T::kPeriod2, SPU = T::kStagesPerUnit, XB = T::kXrBufs;
        uint32_t par_s = 0, par_x = 0, ph_acc = 0;  // parities of ring slot 0 / XR buffer 0 at the start of the period
        int ku = 0;
        bool have_full = false, have_half = false, ok = true;
        for (unsigned base = 0; ok && base < total_stages; base += P) {
#pragma unroll
          for (int j = 0; j < P; ++j) {
            if (base + j >= total_stages) break;
            const int sl = j % T::kS2, su = j % SPU, xb = (j / SPU) % XB;
            const uint32_t p_full = par_s ^ ((j / T::kS2) & 1), p_x = par_x ^ (((j / SPU) / XB) & 1);
            // first stage of a tile: the epilogue must have drained the accumulator
            if (su == 0 && ku == 0 && !(ok = mbar_wait(acc_empty, ph_acc ^ 1, ctx, 22))) break;
            if (!have_half && !(ok = mbar_wait(x_half + 8 * (xb * SPU + su), p_x, ctx, 23))) break;
            if (!have_full && !(ok = mbar_wait(full2 + 8 * sl, p_full, ctx, 24))) break;
            tc_fence_after();
            const uint32_t a_tmem = tmem_base + T::kColXr + xb * T::kUnitK + su * (T::kBK / 2);
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(sl * (T::kS2Bytes >> 4));
            const bool unit_ends = (su == SPU - 1);
            const int jn = j + 1;  // the next stage (jn == P: the next period, whose base parities have flipped)
#pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              if (kk == 2) {
                have_full = mbar_test_wait(full2 + 8 * (jn % T::kS2), par_s ^ ((jn / T::kS2) & 1));
                have_half = mbar_test_wait(x_half + 8 * (((jn / SPU) % XB) * SPU + jn % SPU), par_x ^ (((jn / SPU) / XB) & 1));
              }
              const uint32_t accum = (su > 0 || kk > 0) ? 1u : (ku > 0 ? 1u : 0u);
              umma_f16_ts_pair(tmem_base + T::kColAcc, a_tmem + kk * 8, b_desc + kk * 2, idesc2, accum);
            }
            umma_commit_pair(empty2 + 8 * sl, 3);
            if (unit_ends) {
              umma_commit_pair(x_empty + 8 * xb, 1);  // only the leader's MMA1 issuer waits for this
              if (++ku == units) {
                umma_commit_pair(acc_full, 3);
                ku = 0;
                ph_acc ^= 1;
              }
            }
          }
          par_s ^= (P / T::kS2) & 1;
          par_x ^= ((P / SPU) / XB) & 1;
        }
      } else {
        int s = 0, xb = 0, ku = 0, su = 0;
        uint32_t ph_s = 0, ph_xb = 0, ph_acc = 0;
        bool have_full = false, have_half = false, ok = true;
        for (unsigned j = 0; ok && j < total_stages; ++j) {
          if (su == 0 && ku == 0 && !(ok = mbar_wait(acc_empty, ph_acc ^ 1, ctx, 22))) break;
          if (!have_full && !(ok = mbar_wait(full2 + 8 * s, ph_s, ctx, 24))) break;
          const bool unit_ends = (su == T::kStagesPerUnit - 1);
          int s_n = s + 1;
          uint32_t ph_s_n = ph_s;
          if (s_n == T::kS2) { s_n = 0; ph_s_n ^= 1; }
          const int su_n = unit_ends ? 0 : su + 1;
  #pragma unroll
          for (int gl = 0; gl < T::kGT; ++gl) {  // each N-group multiplies its own XR into its own columns of the accumulator
            if (!have_half && !(ok = mbar_wait(x_half + 8 * (xb * T::kStagesPerUnit + su), ph_xb, ctx, 23))) break;
            tc_fence_after();
            const uint32_t a_tmem = tmem_base + T::kColXr + xb * T::kUnitK + su * (T::kBK / 2);
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((s * T::kS2Bytes + gl * T::kGSHalf * 128) >> 4);
            int xb_n = xb;
            uint32_t ph_xb_n = ph_xb;
            if (unit_ends && ++xb_n == T::kXrBufs) { xb_n = 0; ph_xb_n ^= 1; }
  #pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              if (kk == 2) {
                const bool more = (j + 1 < total_stages) || (gl + 1 < T::kGT);
                if (gl == T::kGT - 1) have_full = (j + 1 < total_stages) && mbar_test_wait(full2 + 8 * s_n, ph_s_n);
                have_half = more && mbar_test_wait(x_half + 8 * (xb_n * T::kStagesPerUnit + (T::kGT > 1 ? 0 : su_n)), ph_xb_n);
              }
              const uint32_t accum = (su > 0 || kk > 0) ? 1u : (ku > 0 ? 1u : 0u);
              umma_f16_ts_pair(tmem_base + T::kColAcc + gl * T::kGS, a_tmem + kk * 8, b_desc + kk * 2, idesc2, accum);
            }
            if (unit_ends) {
              umma_commit_pair(x_empty + 8 * xb, 1);  // only the leader's MMA1 issuer waits for this
              xb = xb_n;
              ph_xb = ph_xb_n;
            }
          }
          if (!ok) break;
          umma_commit_pair(empty2 + 8 * s, 3);
          if (unit_ends && ku + 1 == units) umma_commit_pair(acc_full, 3);
          s = s_n;
          ph_s = ph_s_n;
          if (unit_ends) {
            su = 0;
            if (++ku == units) {
              ku = 0;
              ph_acc ^= 1;
            }
          } else {
            ++su;
          }
        }
          }
}
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // -------------------------------------------------------------- converters (both CTAs, own 128 rows)
    setmaxnreg_dec<152>();
    const int quad = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    int xb = 0;
    uint32_t ph_xb = 0;
    for (unsigned g = 0; ok && g < total_units; ++g) {
      if (!(ok = mbar_wait_warp(x_acc + 8 * xb, ph_xb, ctx, 30))) break;
      tc_fence_after();
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
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_cluster(mapa_shared(x_half + 8 * (xb * T::kStagesPerUnit + h), 0));  // leader collects both CTAs
      }
      if (++xb == T::kXrBufs) { xb = 0; ph_xb ^= 1; }
    }
  } else if (warp >= 8) {
    // -------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    setmaxnreg_inc<248>();
    const int quad = warp & 3;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + T::kColAcc;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(args.C) & 15) == 0) && ((args.ldC & 7) == 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (unsigned tile = pair; ok && tile < num_tiles; tile += num_pairs, ++tcount) {
      unsigned tm, tn;
      tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
      if (!(ok = mbar_wait_warp(acc_full, tcount & 1, ctx, 40))) break;
      tc_fence_after();
      const int row = tm * 2 * T::kBM + rank * T::kBM + quad * 32 + lane;
      __half* c_row = args.C + static_cast<long long>(row) * args.ldC;
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
      mbar_arrive_cluster(mapa_shared(acc_empty, 0));
      if (threadIdx.x == 256) skew_stamp(ctx, tcount);
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
  if (threadIdx.x == 0) {
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
  tc_fence_before();
  cluster_sync_all();
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

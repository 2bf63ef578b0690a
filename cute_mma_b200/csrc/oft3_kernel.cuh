// Fused OFT product in which one X.R serves every N tile of a row block (CTA pairs, tcgen05 cta_group::2).
// Same operator, layouts and numerics as oft2_kernel.cuh (reference: oft_device / oft_ar / oft_arb,
// cute_oft_coop_pc.cu:363-479; the producer -> consumer hand-off of cute_oft_coop_pc.cu:164-179, 337-351).
//
// oft2_kernel keeps X.R in tensor memory and therefore forms it again for every N tile (b / bN extra tensor
// work: +25 % at b = 64, +50 % at b = 128).  Here the rotation is a second, much smaller job of the same
// persistent kernel.  The pairs split the (256 rows x U columns) units of X.R among themselves, band by band, each
// pair a contiguous share of every band:
//   rotation  XR unit [256 x U] fp32 (TMEM) = X[256 x U] . Rblk^T        tcgen05.mma, N = b
//             -> fp16 (RNE) -> 128-byte-swizzled staging in shared memory -> TMA tile store into a ring of
//             row blocks in global memory that is sized to stay in L2 (2 bands of row blocks)
//   product   acc[256 x 256] fp32 (TMEM) += XR[256 x 64] . W[256 x 64]^T   both operands by TMA from L2 / HBM
// Tiles are visited band by band (bands of `raster` row blocks, all N tiles of a band before the next band), so
// a row block of X.R is written once, read by all its N tiles while it sits in L2, and its ring slot is reused
// two bands later.  Cross-CTA ordering goes through counters in global memory:
//   ready[2 * tm + rank]  += units stored by a CTA of that rank        (a tile waits for all units of its rows)
//   done[tm]              += 1 per finished tile of row block tm        (a slot is rewritten after all its tiles)
// Every CTA is resident (grid <= SM count, cooperative launch) and the rotation roles never wait for the
// product roles of their own CTA, so the oldest unfinished tile can always complete.  All waits are bounded.
//
// Roles (both CTAs of a pair unless noted):
//   warp 0      TMA producer of the {XR, W} ring           warp 1      TMA producer of the {X, R} ring
//   warp 2      issues the rotation MMAs (leader only)     warp 3      owns tensor memory, issues the product MMAs (leader only)
//   warps 4..7  rotation epilogue (TMEM -> fp16 -> ring)   warps 8..11 product epilogue (TMEM -> fp16 -> C)
// No load carries a multicast qualifier.
#pragma once
#include "oft2_kernel.cuh"

namespace b200 {

template <int kB_, int kS1_, int kS2_>
struct Oft3Traits {
  static constexpr int kB = kB_;
  static constexpr int kBM = 128;                      // rows per CTA; the pair covers 256
  static constexpr int kBN = 256;
  static constexpr int kBNHalf = kBN / 2;
  static constexpr int kBK = 64;
  static constexpr int kUnitK = kB > 64 ? kB : 64;     // K columns of one rotation unit
  static constexpr int kStagesPerUnit = kUnitK / kBK;
  static constexpr int kS1 = kS1_;                     // {X, R} ring depth
  static constexpr int kS2 = kS2_;                     // {XR, W} ring depth
  static constexpr int kXBytes = kBM * 128;
  static constexpr int kRHalfBytes = (kB / 2) * 128;   // this CTA's half of the R tile: b/2 rows (q) x 64 columns of K
  static constexpr int kS1Bytes = kXBytes + kRHalfBytes;
  static constexpr int kABytes = kBM * 128;            // this CTA's 128 rows of X.R
  static constexpr int kS2Bytes = kABytes + kBNHalf * 128;
  static constexpr int kOutBytes = kBM * 128;          // staging of one (128 x 64) fp16 slice of X.R
  static constexpr int kXrBufs = (512 - kBN) / kUnitK; // fp32 rotation results in flight in tensor memory
  static constexpr int kColAcc = 0;
  static constexpr int kColXr = kBN;
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 384;
  static constexpr int kNumBars = 2 * kS1 + 2 * kS2 + 2 * kXrBufs + 2;
  static constexpr int kSmemBytes = kS1 * kS1Bytes + kS2 * kS2Bytes + kOutBytes + kNumBars * 8 + 64 + 1024;
  static_assert(kB == 16 || kB == 32 || kB == 64 || kB == 128, "block edge must be 16, 32, 64 or 128");
  static_assert(kRHalfBytes % 1024 == 0, "R half-tile must keep the next tile 1024-byte aligned");
  static_assert(kXrBufs >= 2 && kS1 >= kStagesPerUnit, "rotation pipeline too shallow");
  static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

struct Oft3Args {
  int m, n, k;
  __half* C;
  long long ldC;
  int* status;
  int raster;                      // tiles are visited in bands of `raster` (> 0) row blocks
  unsigned long long hint_x, hint_a, hint_b;  // L2 eviction priority of the X, X.R and W tile loads
  int tile_sync;                   // producers of all CTAs start each tile round together
  int* rounds;                     // 4 zeroed counters of this launch's tile rounds (tile_sync only)
  int prefetch_w;                  // > 0: W tiles are asked into L2 this many K steps ahead of their load (W streams from DRAM)
  int slots;                       // row blocks the X.R ring holds (all of them, or 2 * raster)
  int* ready;                      // [2 * row blocks] zeroed
  int* done;                       // [row blocks] zeroed
  int n_more;                      // the result is also stored to this many further buffers of the same shape and ldC,
  __half* C_more[7];               // e.g. this rank's columns of Y on every other GPU of the node (plain stores over NVLink)
};

// A pair's rotation units: band after band (the order the tiles consume them), and inside each band a
// contiguous share of the band's units in (row block, unit) order.  Consecutive units of a pair therefore lie
// in the same row block, so one publication covers several of them.
struct RotationShare {
  unsigned raster, tiles_m, upb, pair, num_pairs;
  unsigned band = 0, j = 0, j_end = 0;
  bool started = false;
  __device__ RotationShare(unsigned raster_, unsigned tiles_m_, unsigned upb_, unsigned pair_, unsigned num_pairs_)
      : raster(raster_), tiles_m(tiles_m_), upb(upb_), pair(pair_), num_pairs(num_pairs_) {}
  __device__ unsigned band_units(unsigned b) const {
    const unsigned rows = (tiles_m - b * raster) < raster ? (tiles_m - b * raster) : raster;
    return rows * upb;
  }
  __device__ unsigned total() const {  // all full bands give this pair the same share
    const unsigned full = tiles_m / raster, u = raster * upb, rest = (tiles_m % raster) * upb;
    return full * ((pair + 1) * u / num_pairs - pair * u / num_pairs) + ((pair + 1) * rest / num_pairs - pair * rest / num_pairs);
  }
  // next unit of this pair: row block tm, unit ku inside it; false when there is none left
  __device__ bool next(unsigned& tm, unsigned& ku) {
    while (true) {
      if (!started) {
        if (band * raster >= tiles_m) return false;
        const unsigned u = band_units(band);
        j = pair * u / num_pairs;
        j_end = (pair + 1) * u / num_pairs;
        started = true;
      }
      if (j < j_end) {
        tm = band * raster + j / upb;
        ku = j % upb;
        ++j;
        return true;
      }
      ++band;
      started = false;
    }
  }
};

template <class T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T::kThreads, 1)
oft3_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_r,
            const __grid_constant__ CUtensorMap tmap_xr, const __grid_constant__ CUtensorMap tmap_b, const Oft3Args args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t ring1 = smem_base, ring2 = ring1 + T::kS1 * T::kS1Bytes;
  const uint32_t out_stage = ring2 + T::kS2 * T::kS2Bytes;
  const uint32_t bars = out_stage + T::kOutBytes;
  int bi = 0;
  const uint32_t full1 = bars + 8u * bi;  bi += T::kS1;
  const uint32_t empty1 = bars + 8u * bi; bi += T::kS1;
  const uint32_t full2 = bars + 8u * bi;  bi += T::kS2;
  const uint32_t empty2 = bars + 8u * bi; bi += T::kS2;
  const uint32_t x_acc = bars + 8u * bi;   bi += T::kXrBufs;
  const uint32_t x_empty = bars + 8u * bi; bi += T::kXrBufs;
  const uint32_t acc_full = bars + 8u * bi;  bi += 1;
  const uint32_t acc_empty = bars + 8u * bi; bi += 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + (bars - smem_base) + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* conv_abort = reinterpret_cast<volatile int*>(tmem_slot + 2);  // rotation epilogue: one of its warps gave up
  volatile unsigned* seen_tile = reinterpret_cast<volatile unsigned*>(tmem_slot + 3);  // tile whose X.R rows the epilogue saw ready
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};
#ifdef B200_PROFILE_WAITS
  const long long kernel_c0 = clock64();
  if (threadIdx.x == 0) skew_stamp(ctx, kSkewTiles - 2);  // when this CTA started
#endif

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const unsigned pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const unsigned tiles_m = (args.m + 2 * T::kBM - 1) / (2 * T::kBM), tiles_n = (args.n + T::kBN - 1) / T::kBN;
  const unsigned num_tiles = tiles_m * tiles_n;
  const int k_steps = (args.k + T::kBK - 1) / T::kBK;
  const unsigned upb = (args.k + T::kUnitK - 1) / T::kUnitK;  // rotation units per row block
  unsigned my_tiles = 0;
  if (pair < num_tiles) my_tiles = (num_tiles - pair + num_pairs - 1) / num_pairs;
  const unsigned my_units = RotationShare(args.raster, tiles_m, upb, pair, num_pairs).total();

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *conv_abort = 0;
    *seen_tile = ~0u;
    for (int s = 0; s < T::kS1; ++s) { mbar_init(full1 + 8 * s, 1); mbar_init(empty1 + 8 * s, 1); }
    for (int s = 0; s < T::kS2; ++s) { mbar_init(full2 + 8 * s, 1); mbar_init(empty2 + 8 * s, 1); }
    for (int i = 0; i < T::kXrBufs; ++i) { mbar_init(x_acc + 8 * i, 1); mbar_init(x_empty + 8 * i, 256); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 256);
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_r);
    prefetch_tmap(&tmap_xr);
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

  // Registers per thread by role: 112 for the four single-thread roles, 136 for the rotation epilogue, 248 for the
  // product epilogue (it holds a whole accumulator row).  The three sum to 496 of the 512 the register file gives a
  // thread of each kind: setmaxnreg.inc waits until registers are free, and a split of exactly 512 never got them.
  // With 96 / 152 / 248 the kernel needed 9 % more cycles (in-kernel counters, M 65536, K 8192, N 3584).
  if (warp == 0) {
    // -------------------------------------------------------------- producer of the {XR, W} ring (both CTAs)
    setmaxnreg_dec<112>();
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      unsigned done_rounds = 0, sync_target = 0, next_tm = 0;
      int next_n0 = -1;
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
        // This CTA's 128 rows of the row block: every unit of them has been stored and is visible.  Usually the
        // epilogue has seen that already while this thread was feeding the previous tile (the fences behind the
        // counter take 1 to 2 us, during which this thread could issue no load and the MMAs would run dry).
        if (*seen_tile == tile) {
          __threadfence_block();
        } else if (!(ok = flag_wait_ge(args.ready + 2 * tm + rank, static_cast<int>(upb), ctx, 14))) {
          break;
        }
        if (tile == pair) skew_stamp(ctx, kSkewTiles - 1);  // profiling build: when the first tile's rows were ready
        const int xr_row0 = static_cast<int>(tm % static_cast<unsigned>(args.slots)) * 2 * T::kBM + rank * T::kBM;
        const int n0 = tn * T::kBN + rank * T::kBNHalf;  // this CTA's half of the W tile
        next_n0 = -1;
        if (tile + num_pairs < num_tiles) {
          unsigned tn_next;
          tile_coord_r(args.raster, tiles_m, tiles_n, tile + num_pairs, next_tm, tn_next);
          next_n0 = tn_next * T::kBN + rank * T::kBNHalf;
        }
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % T::kS2;
          if (!(ok = mbar_wait(empty2 + 8 * s, ((it / T::kS2) & 1) ^ 1, ctx, 11))) break;
          if (rank == 0) mbar_expect_tx(full2 + 8 * s, 2 * T::kS2Bytes);  // both CTAs' bytes land on the leader's barrier
          const uint32_t a_dst = ring2 + s * T::kS2Bytes;
          tma_load_2d_pair_hint(a_dst, &tmap_xr, full2 + 8 * s, ks * T::kBK, xr_row0, args.hint_a);
          tma_load_2d_pair_hint(a_dst + T::kABytes, &tmap_b, full2 + 8 * s, ks * T::kBK, n0, args.hint_b);
          if (args.prefetch_w > 0) {  // W comes from DRAM: the ring alone (5 stages) does not cover that latency
            const int q = ks + args.prefetch_w;
            if (q < k_steps) tma_prefetch_2d(&tmap_b, q * T::kBK, n0);
            else if (next_n0 >= 0 && q - k_steps < k_steps) tma_prefetch_2d(&tmap_b, (q - k_steps) * T::kBK, next_n0);
          }

        }
      }
      // leaving after its last round, this thread still counts for the rendezvous the others make
      if (ok && args.tile_sync && done_rounds > 0) atomicAdd(args.rounds + rank, 1);
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- producer of the {X, R} ring (both CTAs)
    setmaxnreg_dec<112>();
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      unsigned last_tm = ~0u, tm = 0, ku = 0, unit_no = 0;
      RotationShare share(args.raster, tiles_m, upb, pair, num_pairs);
      for (; ok && share.next(tm, ku); ++unit_no) {
        if (tm != last_tm) {
          // the ring slot of this row block still belongs to row block tm - slots until all its tiles are finished
          if (tm >= static_cast<unsigned>(args.slots))
            if (!(ok = flag_wait_ge(args.done + (tm - args.slots), static_cast<int>(tiles_n), ctx, 15))) break;
          last_tm = tm;
        }
        const int m0 = tm * 2 * T::kBM + rank * T::kBM, k0 = ku * T::kUnitK;
        for (int su = 0; su < T::kStagesPerUnit; ++su, ++it) {
          const int s = it % T::kS1;
          if (!(ok = mbar_wait_parked(empty1 + 8 * s, ((it / T::kS1) & 1) ^ 1, ctx, 10))) break;
          if (su == 0) early_stamp(ctx, unit_no, 0);
          if (rank == 0) mbar_expect_tx(full1 + 8 * s, 2 * T::kS1Bytes);
          const uint32_t x_dst = ring1 + s * T::kS1Bytes;
          tma_load_2d_pair_hint(x_dst, &tmap_x, full1 + 8 * s, k0 + su * T::kBK, m0, args.hint_x);
          tma_load_2d_pair_hint(x_dst + T::kXBytes, &tmap_r, full1 + 8 * s, k0 + su * T::kBK, rank * (T::kB / 2), kL2EvictLast);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // -------------------------------------------------------------- issuer of the rotation MMAs (leader CTA only)
    setmaxnreg_dec<112>();
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc1 = umma_idesc(kFmtF16, 0, 0, 2 * T::kBM, T::kB);
      const uint64_t x_desc0 = umma_desc_sw128(ring1, 16, 1024), r_desc0 = umma_desc_sw128(ring1 + T::kXBytes, 16, 1024);
      uint32_t it = 0;
      bool ok = true;
      for (unsigned i = 0; ok && i < my_units; ++i) {
        const int xb = i % T::kXrBufs;
        if (!(ok = mbar_wait_parked(x_empty + 8 * xb, ((i / T::kXrBufs) & 1) ^ 1, ctx, 20))) break;
        const uint32_t d1 = tmem_base + T::kColXr + xb * T::kUnitK;
        for (int su = 0; su < T::kStagesPerUnit; ++su, ++it) {
          const int s = it % T::kS1;
          if (!(ok = mbar_wait_parked(full1 + 8 * s, (it / T::kS1) & 1, ctx, 21))) break;
          tc_fence_after();
          const uint64_t x_desc = x_desc0 + static_cast<uint64_t>(s * (T::kS1Bytes >> 4));
          const uint64_t r_desc = r_desc0 + static_cast<uint64_t>(s * (T::kS1Bytes >> 4));
#pragma unroll
          for (int kk = 0; kk < T::kBK / 16; ++kk) {
            // b < 64: the stage holds 64/b diagonal blocks; slice kk belongs to block (kk*16)/b and lands in
            // columns [blk*b, blk*b+b).  b >= 64: one block, accumulated over the unit.
            constexpr bool small = T::kB < 64;
            const int blk = small ? (kk * 16) / T::kB : 0;
            const uint32_t accum = small ? ((((kk * 16) % T::kB) != 0) ? 1u : 0u) : ((su > 0 || kk > 0) ? 1u : 0u);
            umma_f16_ss_pair(d1 + blk * T::kB, x_desc + kk * 2, r_desc + kk * 2, idesc1, accum);
          }
          umma_commit_pair(empty1 + 8 * s, 3);
        }
        if (!ok) break;
        early_stamp(ctx, i, 1);
        umma_commit_pair(x_acc + 8 * xb, 3);  // the rotation epilogues of both CTAs start on their halves
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    // -------------------------------------------------------------- issuer of the product MMAs (leader CTA only)
    setmaxnreg_dec<112>();
    if (lane == 0 && rank == 0) {
      // Unrolled over the ring's stages with the tiles flattened into one stream of K steps (every barrier
      // address, parity and descriptor offset is a constant plus a base register), like the plain pair GEMM.
      constexpr uint32_t idesc2 = umma_idesc(kFmtF16, 0, 0, 2 * T::kBM, T::kBN);
      const uint64_t a_desc0 = umma_desc_sw128(ring2, 16, 1024), b_desc0 = umma_desc_sw128(ring2 + T::kABytes, 16, 1024);
      const uint32_t total = my_tiles * static_cast<uint32_t>(k_steps);
      const uint32_t d_tmem = tmem_base + T::kColAcc;
      uint32_t phase = 0, tcount = 0;
      int ks = 0;
      bool ok = true, have_full = false;
      for (uint32_t base = 0; ok && base < total; base += T::kS2) {
#pragma unroll
        for (int s = 0; s < T::kS2; ++s) {
          if (base + s >= total) break;
          if (ks == 0) {  // first K step of a tile: the epilogue must have drained the accumulator
            if (!(ok = mbar_wait(acc_empty, (tcount & 1) ^ 1, ctx, 22))) break;
          }
          if (!have_full && !(ok = mbar_wait(full2 + 8 * s, phase, ctx, 24))) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < T::kBK / 16; ++kk) {
            if (kk == 2)  // is the next stage there already?  (never waits)
              have_full = mbar_test_wait(full2 + 8 * ((s + 1) % T::kS2), s + 1 == T::kS2 ? (phase ^ 1) : phase);
            const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
            const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * T::kS2Bytes + kk * 32) >> 4);
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((s * T::kS2Bytes + kk * 32) >> 4);
            umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc2, acc);
          }
          umma_commit_pair(empty2 + 8 * s, 3);  // frees the stage in both CTAs
          if (++ks == k_steps) {
            umma_commit_pair(acc_full, 3);
            ks = 0;
            ++tcount;
          }
        }
        phase ^= 1;
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // -------------------------------------------------------------- rotation epilogue (both CTAs, own 128 rows)
    setmaxnreg_dec<136>();
    const int quad = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int r = quad * 32 + lane;  // row of the unit this thread converts
    const uint32_t my_row = out_stage + r * 128;
    const bool issuer = (warp == 4 && lane == 0);
    // The issuer publishes units once their tile stores are complete (bulk_wait_group), several units of one row
    // block with one add: the publication (proxy fence + release) takes about 2 us, measured with in-kernel
    // timers, so it happens when the row block changes, when the next unit is not there yet (the thread would
    // idle anyway), and at the end.
    constexpr int kGroupsPerUnit = T::kUnitK / 64;
    int* pending = nullptr;
    int pending_n = 0;
    bool ok = true;
    unsigned tm = 0, ku = 0;
    RotationShare share(args.raster, tiles_m, upb, pair, num_pairs);
    for (unsigned i = 0; ok && share.next(tm, ku); ++i) {
      const int xb = i % T::kXrBufs;
      const int xr_row0 = static_cast<int>(tm % static_cast<unsigned>(args.slots)) * 2 * T::kBM + rank * T::kBM;
      const int k0 = ku * T::kUnitK;
      int* const counter = args.ready + 2 * tm + rank;
      if (issuer && pending && (pending != counter || !mbar_test_wait(x_acc + 8 * xb, (i / T::kXrBufs) & 1))) {
        bulk_wait_group<0>();
        early_stamp(ctx, i, 4);
        flag_signal(pending, pending_n);
        early_stamp(ctx, i, 5);
        pending = nullptr;
        pending_n = 0;
      }
      // The four warps meet at named barriers below, so they must leave together: a warp whose wait gave up says
      // so in shared memory and all of them read the word after a barrier that every one of them reaches.
      if (!mbar_wait_warp(x_acc + 8 * xb, (i / T::kXrBufs) & 1, ctx, 30)) *conv_abort = 1;
      named_barrier_sync(2, 128);
      if (*conv_abort) { ok = false; break; }
      tc_fence_after();
      if (issuer) early_stamp(ctx, i, 2);
      const uint32_t buf = tmem_base + lane_off + T::kColXr + xb * T::kUnitK;
#pragma unroll
      for (int h = 0; h < kGroupsPerUnit; ++h) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(buf + h * 64, v0);
        tmem_ld_x32(buf + h * 64 + 32, v1);
        tmem_wait_ld();
        if (h == kGroupsPerUnit - 1) {  // everything of this buffer is in registers: hand it back before storing
          tc_fence_before();
          mbar_arrive_cluster(mapa_shared(x_empty + 8 * xb, 0));  // the leader's barrier collects both CTAs
        }
        uint32_t p[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 a = __floats2half2_rn(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
          __half2 b = __floats2half2_rn(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
          p[j] = *reinterpret_cast<uint32_t*>(&a);
          p[16 + j] = *reinterpret_cast<uint32_t*>(&b);
        }
        if (issuer) bulk_wait_group_read<0>();  // the previous store has read the staging buffer
        named_barrier_sync(1, 128);
#pragma unroll
        for (int c = 0; c < 8; ++c)  // 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r mod 8)
          st_shared_v4(my_row + ((c ^ (r & 7)) << 4), p[4 * c], p[4 * c + 1], p[4 * c + 2], p[4 * c + 3]);
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (issuer) {
          tma_store_2d(&tmap_xr, out_stage, k0 + h * 64, xr_row0);
          bulk_commit_group();
        }
      }
      if (issuer) {
        early_stamp(ctx, i, 3);
        pending = counter;
        ++pending_n;
      }
    }
    if (issuer) {
      bulk_wait_group<0>();
      if (ok && pending) flag_signal(pending, pending_n);
    }
  } else if (warp >= 8) {
    // -------------------------------------------------------------- product epilogue (both CTAs, own 128 rows)
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
      if (threadIdx.x == 256 && tcount < kSkewTiles - 2) skew_stamp(ctx, tcount);  // profiling build: end of each tile's MMAs
      const int row = tm * 2 * T::kBM + rank * T::kBM + quad * 32 + lane;
      uint32_t p[T::kBN / 2];
#pragma unroll
      for (int c = 0; c < T::kBN / 32; c += 2) {  // two loads in flight per wait
        uint32_t v[32], w[32];
        tmem_ld_x32(t_row + c * 32, v);
        tmem_ld_x32(t_row + c * 32 + 32, w);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 h2 = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          __half2 g2 = __floats2half2_rn(__uint_as_float(w[2 * j]), __uint_as_float(w[2 * j + 1]));
          p[c * 16 + j] = *reinterpret_cast<uint32_t*>(&h2);
          p[c * 16 + 16 + j] = *reinterpret_cast<uint32_t*>(&g2);
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(mapa_shared(acc_empty, 0));
      if (row < args.m) {  // the caller's C: a lane owns a row and writes 64 contiguous bytes of it per 32 columns
        __half* out_row = args.C + static_cast<long long>(row) * args.ldC;
#pragma unroll
        for (int c = 0; c < T::kBN / 32; ++c) {
          const int col0 = tn * T::kBN + c * 32;
          if (vec_ok && col0 + 32 <= args.n) {
            uint4* dst = reinterpret_cast<uint4*>(out_row + col0);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              dst[q] = make_uint4(p[c * 16 + 4 * q], p[c * 16 + 4 * q + 1], p[c * 16 + 4 * q + 2], p[c * 16 + 4 * q + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < args.n) {
                const uint32_t w = p[c * 16 + j / 2];
                out_row[col0 + j] = __ushort_as_half(static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xFFFFu)));
              }
          }
        }
      }
      if (args.n_more > 0) {
        // Further destinations (other GPUs' memory): a write of 16 bytes per lane, each to another row, crosses
        // NVLink as 32 small packets.  The warp's 32 rows x 128 bytes are therefore transposed in registers first
        // (butterfly of lane exchanges, 32 x 32 words at a time), after which the 32 lanes write the 128 contiguous
        // bytes of one row with one instruction.  Needs 4-byte aligned rows; else the row-per-lane stores.
        bool words = (args.ldC & 1) == 0;
        for (int d = 0; d < args.n_more; ++d) words = words && (reinterpret_cast<uintptr_t>(args.C_more[d]) & 3) == 0;
        if (words) {
#pragma unroll
          for (int blk = 0; blk < T::kBN / 64; ++blk) {
#pragma unroll
            for (int sft = 16; sft >= 1; sft >>= 1) {
              const bool upper = (lane & sft) != 0;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (j & sft) continue;
                uint32_t& lo = p[blk * 32 + j];
                uint32_t& hi = p[blk * 32 + j + sft];
                const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, upper ? lo : hi, sft);
                if (upper) lo = got; else hi = got;
              }
            }
          }
          // now p[blk * 32 + i] of lane L is word (blk * 32 + L) of row i of this warp
          const int row0 = tm * 2 * T::kBM + rank * T::kBM + quad * 32;
          for (int d = 0; d < args.n_more; ++d) {
            __half* base = args.C_more[d] + static_cast<long long>(row0) * args.ldC + tn * T::kBN + 2 * lane;
#pragma unroll
            for (int blk = 0; blk < T::kBN / 64; ++blk) {
              const int col = tn * T::kBN + blk * 64 + 2 * lane;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (row0 + i >= args.m) continue;
                __half* dst = base + static_cast<long long>(i) * args.ldC + blk * 64;
                const uint32_t w = p[blk * 32 + i];
                if (col + 1 < args.n) *reinterpret_cast<uint32_t*>(dst) = w;
                else if (col < args.n) *dst = __ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu));
              }
            }
          }
        } else if (row < args.m) {
          for (int d = 0; d < args.n_more; ++d) {
            __half* out_row = args.C_more[d] + static_cast<long long>(row) * args.ldC;
#pragma unroll
            for (int c = 0; c < T::kBN / 32; ++c) {
              const int col0 = tn * T::kBN + c * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < args.n) {
                  const uint32_t w = p[c * 16 + j / 2];
                  out_row[col0 + j] = __ushort_as_half(static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xFFFFu)));
                }
            }
          }
        }
      }
      // Every MMA of the tile was done when acc_full completed, so every load of its X.R rows (both CTAs') has
      // landed: one count per tile.  Last in the tile's epilogue: the publication takes about 2 us, which must not
      // delay the hand-back of the accumulator.
      if (threadIdx.x == 256 && rank == 0) flag_signal(args.done + tm, 1);
      // ... and a look ahead for the producer of the {XR, W} ring: are the rows of this pair's tile after next there?
      // (The next tile is already being fed.)  One look; if not, the producer waits for them itself.
      if (threadIdx.x == 256 && tile + 2 * num_pairs < num_tiles) {
        unsigned tm2, tn2;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile + 2 * num_pairs, tm2, tn2);
        if (flag_test_ge(args.ready + 2 * tm2 + rank, static_cast<int>(upb))) {
          __threadfence_block();
          *seen_tile = tile + 2 * num_pairs;
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
  if (*abort_flag) {  // a wait ran out: let the copies in flight land before shared and tensor memory go away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while its pair may still use it
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

// Fused OFT product with the rotation on SM pairs of its own (CTA pairs, tcgen05 cta_group::2).
// Same operator, layouts, numerics and cross-CTA protocol as oft3_kernel.cuh (reference: oft_device / oft_ar /
// oft_arb, cute_oft_coop_pc.cu:363-479; its producer and consumer warps share one thread block, cute_oft_coop_pc.cu:
// 164-179, 337-351).  In oft3_kernel every pair does both jobs, which costs the product its second accumulator, a
// stage of its operand ring and a share of its issue slots.  Here the pairs of one cooperative launch are split:
//   product pairs   the loop of the plain pair GEMM (gemm2_kernel.cuh) unchanged: six 32 KB stages, two accumulators
//                   in tensor memory, A operand = 256 rows of W (the output columns), B operand = 256 rows of X.R
//                   read from the ring; a tile waits until its row block of X.R is published (`ready`), and counts
//                   itself in `done` when its MMAs are through
//   rotation pairs  X[256 x U] . Rblk^T (tcgen05.mma, N = b) -> fp16 (RNE) -> swizzled staging -> TMA tile stores into
//                   the ring (one per warp of 32 rows), unit after unit in band order, a contiguous share of every
//                   band per rotation pair; a deep {X, R} ring, since these SMs do nothing else
// The first bands are rotated by all pairs together before they split up, so the first wave of tiles starts after a
// few microseconds.  The ring of row blocks lives in global memory and is sized to stay in L2; `ready` / `done`
// counters as in oft3_kernel.  All CTAs are resident (cooperative launch); rotation pairs never wait for anything a
// product pair of a younger band has to do first, so the oldest unfinished tile can always complete.  All waits are
// bounded.
// 192 threads: product pairs  warp 0 TMA producer, warp 1 MMA issuer (leader), warps 2..5 epilogue;
//              rotation pairs warp 0 TMA producer, warp 1 MMA issuer (leader), warps 2..5 rotation epilogue.
// No load carries a multicast qualifier.
#pragma once
#include "oft3_kernel.cuh"

namespace b200 {

template <int kB_>
struct Oft4Traits {
  static constexpr int kB = kB_;
  static constexpr int kBM = 128;                      // rows of an operand tile per CTA; the pair covers 256
  static constexpr int kBN = 256;
  static constexpr int kBK = 64;
  static constexpr int kUnitK = kB > 64 ? kB : 64;     // K columns of one rotation unit
  static constexpr int kStagesPerUnit = kUnitK / kBK;
  // product pairs
  static constexpr int kStages = 6;
  static constexpr int kABytes = kBM * 128;            // this CTA's 128 rows of W
  static constexpr int kStageBytes = kABytes + kBM * 128;  // + this CTA's 128 rows of X.R
  static constexpr int kAccBufs = 2;
  // rotation pairs
  static constexpr int kXBytes = kBM * 128;
  static constexpr int kRHalfBytes = (kB / 2) * 128;
  static constexpr int kS1Bytes = kXBytes + kRHalfBytes;
  static constexpr int kS1 = kB > 64 ? 6 : 8;          // {X, R} stages: three units of 128 columns, or eight of 64
  static constexpr int kOutWarpBytes = 32 * 128;       // staging of one (32 x 64) fp16 slice; two per rotation-epilogue warp
  static constexpr int kXrBufs = 4;                    // fp32 rotation results in flight in tensor memory
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 192;
  static constexpr int kProductBytes = kStages * kStageBytes;
  static constexpr int kRotationBytes = kS1 * kS1Bytes + 8 * kOutWarpBytes;
  static constexpr int kDataBytes = kProductBytes > kRotationBytes ? kProductBytes : kRotationBytes;
  static constexpr int kNumBars = 2 * kStages + 2 * kAccBufs + 2 * kS1 + 2 * kXrBufs;
  static constexpr int kSmemBytes = kDataBytes + kNumBars * 8 + 64 + 1024;
  static_assert(kB == 16 || kB == 32 || kB == 64 || kB == 128, "block edge must be 16, 32, 64 or 128");
  static_assert(kRHalfBytes % 1024 == 0 && kXrBufs * kUnitK <= kTmemCols, "rotation layout");
  static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

struct Oft4Args {
  int m, n, k;
  __half* C;
  long long ldC;
  int* status;
  int raster;                      // tiles are visited in bands of `raster` (> 0) row blocks of X.R
  unsigned long long hint_x, hint_a, hint_b;  // L2 eviction priority of the X, X.R and W tile loads
  int tile_sync;                   // producers of all product pairs start each tile round together
  int* rounds;                     // 4 zeroed counters of this launch's tile rounds (tile_sync only)
  int slots;                       // row blocks the X.R ring holds
  int* ready;                      // [2 * row blocks] zeroed
  int* done;                       // [row blocks] zeroed
  int rot_pairs;                   // the last rot_pairs pairs of the grid rotate, the others multiply
  int prologue_bands;              // bands every pair helps to rotate before the pairs split up (<= bands the ring holds)
};

// Tile idx -> (row block of X.R, tile of W): bands of `raster` row blocks, inside a band one W tile after the other
// with the row blocks of the band running fastest (pairs next to each other share the W tile).
__device__ __forceinline__ void oft4_tile(int raster, unsigned tiles_x, unsigned tiles_w, unsigned idx, unsigned& xb, unsigned& wt) {
  const unsigned g = static_cast<unsigned>(raster);
  const unsigned band = idx / (g * tiles_w), r = idx % (g * tiles_w);
  const unsigned rows = (tiles_x - band * g) < g ? (tiles_x - band * g) : g;
  wt = r / rows;
  xb = band * g + r % rows;
}

// The rotation units of bands [band, band_end) that fall to share `idx` of `cnt`: band after band (the order the
// tiles consume them), and inside each band a contiguous run in (row block, unit) order, so that consecutive units
// of one share lie in the same row block and one publication covers several of them.
struct BandShare {
  unsigned raster, tiles_x, upb, idx, cnt, band, band_end;
  unsigned j = 0, j_end = 0;
  bool started = false;
  __device__ BandShare(unsigned raster_, unsigned tiles_x_, unsigned upb_, unsigned idx_, unsigned cnt_, unsigned band_, unsigned band_end_)
      : raster(raster_), tiles_x(tiles_x_), upb(upb_), idx(idx_), cnt(cnt_), band(band_), band_end(band_end_) {}
  // next unit of this share: row block xb, unit ku inside it; false when there is none left
  __device__ bool next(unsigned& xb, unsigned& ku) {
    while (true) {
      if (!started) {
        if (band >= band_end || band * raster >= tiles_x) return false;
        const unsigned rows = (tiles_x - band * raster) < raster ? (tiles_x - band * raster) : raster;
        const unsigned u = rows * upb;
        j = idx * u / cnt;
        j_end = (idx + 1) * u / cnt;
        started = true;
      }
      if (j < j_end) {
        xb = band * raster + j / upb;
        ku = j % upb;
        ++j;
        return true;
      }
      ++band;
      started = false;
    }
  }
};

// What a rotation role carries from one call of oft4_rotate to the next: positions in the {X, R} ring, in the
// tensor-memory buffers and in a warp's two staging buffers.
struct Oft4RotState {
  uint32_t it = 0;
  unsigned i = 0, slice = 0;
};

struct Oft4RotSmem {
  uint32_t ring1, out_stage, full1, empty1, x_acc, x_empty, tmem_base;
  volatile int* conv_abort;
};

// One warp's part of the rotation of the units in `share` (warp 0 loads, warp 1 issues the MMAs, warps 2..5 convert
// and store).  Returns false if a wait ran out.  On return every store of this CTA has completed and is published.
template <class T>
__device__ __forceinline__ bool oft4_rotate(int warp, int lane, uint32_t rank, BandShare share, Oft4RotState& st, const Oft4RotSmem& sm,
                                            const CUtensorMap* tmap_x, const CUtensorMap* tmap_r, const CUtensorMap* tmap_xr_st,
                                            const Oft4Args& args, unsigned tiles_w, const WaitCtx& ctx) {
  bool ok = true;
  unsigned xb = 0, ku = 0;
  if (warp == 0) {
    // -------------------------------------------------------------- producer of the {X, R} ring (both CTAs)
    if (lane == 0) {
      unsigned last_xb = ~0u;
      while (ok && share.next(xb, ku)) {
        if (xb != last_xb) {
          // the ring slot of this row block still belongs to row block xb - slots until all its tiles are finished
          if (xb >= static_cast<unsigned>(args.slots))
            if (!(ok = flag_wait_ge(args.done + (xb - args.slots), static_cast<int>(tiles_w), ctx, 15))) break;
          last_xb = xb;
        }
        const int m0 = xb * 2 * T::kBM + rank * T::kBM, k0 = ku * T::kUnitK;
        for (int su = 0; su < T::kStagesPerUnit; ++su, ++st.it) {
          const int s = st.it % T::kS1;
          if (!(ok = mbar_wait(sm.empty1 + 8 * s, ((st.it / T::kS1) & 1) ^ 1, ctx, 10))) break;
          if (rank == 0) mbar_expect_tx(sm.full1 + 8 * s, 2 * T::kS1Bytes);
          const uint32_t x_dst = sm.ring1 + s * T::kS1Bytes;
          tma_load_2d_pair_hint(x_dst, tmap_x, sm.full1 + 8 * s, k0 + su * T::kBK, m0, args.hint_x);
          tma_load_2d_pair_hint(x_dst + T::kXBytes, tmap_r, sm.full1 + 8 * s, k0 + su * T::kBK, rank * (T::kB / 2), kL2EvictLast);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- issuer of the rotation MMAs (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc1 = umma_idesc(kFmtF16, 0, 0, 2 * T::kBM, T::kB);
      const uint64_t x_desc0 = umma_desc_sw128(sm.ring1, 16, 1024), r_desc0 = umma_desc_sw128(sm.ring1 + T::kXBytes, 16, 1024);
      for (; ok && share.next(xb, ku); ++st.i) {
        const int buf = st.i % T::kXrBufs;
        if (!(ok = mbar_wait(sm.x_empty + 8 * buf, ((st.i / T::kXrBufs) & 1) ^ 1, ctx, 20))) break;
        const uint32_t d1 = sm.tmem_base + buf * T::kUnitK;
        for (int su = 0; su < T::kStagesPerUnit; ++su, ++st.it) {
          const int s = st.it % T::kS1;
          if (!(ok = mbar_wait(sm.full1 + 8 * s, (st.it / T::kS1) & 1, ctx, 21))) break;
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
          umma_commit_pair(sm.empty1 + 8 * s, 3);
        }
        if (!ok) break;
        umma_commit_pair(sm.x_acc + 8 * buf, 3);  // the rotation epilogues of both CTAs start on their halves
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------- rotation epilogue (warps 2..5, both CTAs, own 128 rows)
    // A warp owns 32 rows of the unit and works on its own: 64 fp32 columns per row from tensor memory -> fp16 (RNE)
    // -> its own 128-byte-swizzled staging (two buffers of 32 rows) -> its own TMA tile store into the ring.  The four
    // warps meet only where units are published: units of one row block together, with one add, when the share
    // moves on to the next row block and at the end.  A warp whose wait ran out keeps walking its share without
    // touching anything, so that all four warps reach the same publication barriers.
    const int quad = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t stage0 = sm.out_stage + quad * (2 * T::kOutWarpBytes);
    const bool issuer = (warp == 2 && lane == 0);
    constexpr int kGroupsPerUnit = T::kUnitK / 64;
    int* pending = nullptr;
    int pending_n = 0;
    auto publish = [&]() {
      if (lane == 0) bulk_wait_group<0>();  // this warp's tile stores are complete
      named_barrier_sync(1, 128);
      if (issuer && !*sm.conv_abort) flag_signal(pending, pending_n);
      pending = nullptr;
      pending_n = 0;
    };
    for (; share.next(xb, ku); ++st.i) {
      int* const counter = args.ready + 2 * xb + rank;
      if (pending && pending != counter) publish();
      pending = counter;
      ++pending_n;
      if (!ok) continue;
      const int buf = st.i % T::kXrBufs;
      if (!(ok = mbar_wait_warp(sm.x_acc + 8 * buf, (st.i / T::kXrBufs) & 1, ctx, 30))) {
        *sm.conv_abort = 1;
        continue;
      }
      tc_fence_after();
      const int xr_row = static_cast<int>(xb % static_cast<unsigned>(args.slots)) * 2 * T::kBM + rank * T::kBM + quad * 32;
      const int k0 = ku * T::kUnitK;
      const uint32_t src = sm.tmem_base + lane_off + buf * T::kUnitK;
#pragma unroll
      for (int h = 0; h < kGroupsPerUnit; ++h, ++st.slice) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(src + h * 64, v0);
        tmem_ld_x32(src + h * 64 + 32, v1);
        tmem_wait_ld();
        if (h == kGroupsPerUnit - 1) {  // everything of this buffer is in registers: hand it back before storing
          tc_fence_before();
          mbar_arrive_cluster(mapa_shared(sm.x_empty + 8 * buf, 0));  // the leader's barrier collects both CTAs
        }
        uint32_t p[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 a = __floats2half2_rn(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
          __half2 b = __floats2half2_rn(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
          p[j] = *reinterpret_cast<uint32_t*>(&a);
          p[16 + j] = *reinterpret_cast<uint32_t*>(&b);
        }
        const uint32_t stage = stage0 + (st.slice & 1u) * T::kOutWarpBytes;
        if (lane == 0) bulk_wait_group_read<1>();  // the store before the previous one has read this buffer
        __syncwarp();
        const uint32_t my_row = stage + lane * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)  // 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r mod 8)
          st_shared_v4(my_row + ((c ^ (lane & 7)) << 4), p[4 * c], p[4 * c + 1], p[4 * c + 2], p[4 * c + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(tmap_xr_st, stage, k0 + h * 64, xr_row);
          bulk_commit_group();
        }
      }
    }
    if (pending) publish();
    ok = ok && !*sm.conv_abort;
  }
  return ok;
}

template <class T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T::kThreads, 1)
oft4_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_r,
            const __grid_constant__ CUtensorMap tmap_xr, const __grid_constant__ CUtensorMap tmap_xr_st,
            const __grid_constant__ CUtensorMap tmap_w, const Oft4Args args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + T::kDataBytes;
  int bi = 0;
  const uint32_t full = bars + 8u * bi;      bi += T::kStages;   // product pairs
  const uint32_t empty = bars + 8u * bi;     bi += T::kStages;
  const uint32_t accfull = bars + 8u * bi;   bi += T::kAccBufs;
  const uint32_t accempty = bars + 8u * bi;  bi += T::kAccBufs;
  const uint32_t full1 = bars + 8u * bi;     bi += T::kS1;       // rotation pairs
  const uint32_t empty1 = bars + 8u * bi;    bi += T::kS1;
  const uint32_t x_acc = bars + 8u * bi;     bi += T::kXrBufs;
  const uint32_t x_empty = bars + 8u * bi;   bi += T::kXrBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + T::kDataBytes + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* conv_abort = reinterpret_cast<volatile int*>(tmem_slot + 2);     // rotation epilogue: one of its warps gave up
  volatile unsigned* seen_tile = reinterpret_cast<volatile unsigned*>(tmem_slot + 3);  // tile whose X.R rows the epilogue saw ready
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const unsigned pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const unsigned rot_pairs = static_cast<unsigned>(args.rot_pairs), prod_pairs = num_pairs - rot_pairs;
  const bool rotates = pair >= prod_pairs;
  const unsigned tiles_x = (args.m + 2 * T::kBM - 1) / (2 * T::kBM), tiles_w = (args.n + T::kBN - 1) / T::kBN;
  const unsigned num_tiles = tiles_x * tiles_w;
  const int k_steps = (args.k + T::kBK - 1) / T::kBK;
  const unsigned upb = (args.k + T::kUnitK - 1) / T::kUnitK;  // rotation units per row block

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *conv_abort = 0;
    *seen_tile = ~0u;
    for (int s = 0; s < T::kStages; ++s) { mbar_init(full + 8 * s, 1); mbar_init(empty + 8 * s, 1); }
    for (int a = 0; a < T::kAccBufs; ++a) { mbar_init(accfull + 8 * a, 1); mbar_init(accempty + 8 * a, 256); }
    for (int s = 0; s < T::kS1; ++s) { mbar_init(full1 + 8 * s, 1); mbar_init(empty1 + 8 * s, 1); }
    for (int i = 0; i < T::kXrBufs; ++i) { mbar_init(x_acc + 8 * i, 1); mbar_init(x_empty + 8 * i, 256); }
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_r);
    prefetch_tmap(&tmap_xr);
    prefetch_tmap(&tmap_xr_st);
    prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), T::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Phase 1: every pair rotates its share of the first bands, so the first wave of tiles finds its rows soon.
  // Phase 2: the rotation pairs go on with the remaining bands, the others multiply.
  const unsigned bands_total = (tiles_x + args.raster - 1) / args.raster;
  const unsigned pro_bands = (rot_pairs == 0 || static_cast<unsigned>(args.prologue_bands) > bands_total) ? bands_total : args.prologue_bands;
  Oft4RotState rot_state;
  const Oft4RotSmem rot_smem{smem_base, smem_base + T::kS1 * T::kS1Bytes, full1, empty1, x_acc, x_empty, tmem_base, conv_abort};
  oft4_rotate<T>(warp, lane, rank, BandShare(args.raster, tiles_x, upb, pair, num_pairs, 0, pro_bands), rot_state, rot_smem, &tmap_x,
                 &tmap_r, &tmap_xr_st, args, tiles_w, ctx);
  if (rotates) {
    oft4_rotate<T>(warp, lane, rank, BandShare(args.raster, tiles_x, upb, pair - prod_pairs, rot_pairs, pro_bands, bands_total), rot_state,
                   rot_smem, &tmap_x, &tmap_r, &tmap_xr_st, args, tiles_w, ctx);
  } else {
    // the product stages and accumulators take over the shared and tensor memory the rotation used
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    if (warp == 0) {
      // ------------------------------------------------------------ product pair: TMA producer (both CTAs)
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        unsigned done_rounds = 0, sync_target = 0;
        for (unsigned tile = pair; ok && tile < num_tiles; tile += prod_pairs) {
          if (args.tile_sync && done_rounds > 0) {
            if (!(ok = tile_round_sync(args.rounds + rank, sync_target, ctx, 12))) break;
          }
          {  // every product pair that had a tile in this round takes part in the next rendezvous
            const unsigned first = tile - pair, left = num_tiles - first;
            sync_target += left < prod_pairs ? left : prod_pairs;
            ++done_rounds;
          }
          unsigned xb, wt;
          oft4_tile(args.raster, tiles_x, tiles_w, tile, xb, wt);
          // This CTA's 128 rows of the row block: every unit of them has been stored and is visible.  Usually the
          // epilogue has seen that already while this thread was feeding the previous tile.
          if (*seen_tile == tile) {
            __threadfence_block();
          } else if (!(ok = flag_wait_ge(args.ready + 2 * xb + rank, static_cast<int>(upb), ctx, 14))) {
            break;
          }
          const int xr_row0 = static_cast<int>(xb % static_cast<unsigned>(args.slots)) * 2 * T::kBM + rank * T::kBM;
          const int w_row0 = wt * T::kBN + rank * T::kBM;  // this CTA's 128 rows of the W tile
          for (int ks = 0; ks < k_steps; ++ks, ++it) {
            const int s = it % T::kStages;
            if (!(ok = mbar_wait(empty + 8 * s, ((it / T::kStages) & 1) ^ 1, ctx, 11))) break;
            if (rank == 0) mbar_expect_tx(full + 8 * s, 2 * T::kStageBytes);  // both CTAs' bytes land on the leader's barrier
            const uint32_t a_dst = smem_base + s * T::kStageBytes;
            tma_load_2d_pair_hint(a_dst, &tmap_w, full + 8 * s, ks * T::kBK, w_row0, args.hint_b);
            tma_load_2d_pair_hint(a_dst + T::kABytes, &tmap_xr, full + 8 * s, ks * T::kBK, xr_row0, args.hint_a);
          }
        }
        // leaving after its last round, this thread still counts for the rendezvous the others make
        if (ok && args.tile_sync && done_rounds > 0) atomicAdd(args.rounds + rank, 1);
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------ product pair: MMA issuer (leader CTA only)
      if (lane == 0 && rank == 0) {
        // The ring is walked in a loop unrolled over its stages with the tiles flattened into one stream of K
        // steps: every barrier address, parity and descriptor offset is a constant plus a base register.
        constexpr uint32_t idesc = umma_idesc(kFmtF16, 0, 0, 2 * T::kBM, T::kBN);
        const uint64_t a_desc0 = umma_desc_sw128(smem_base, 16, 1024), b_desc0 = umma_desc_sw128(smem_base + T::kABytes, 16, 1024);
        unsigned my_tiles = 0;
        if (pair < num_tiles) my_tiles = (num_tiles - pair + prod_pairs - 1) / prod_pairs;
        const uint32_t total = my_tiles * static_cast<uint32_t>(k_steps);
        uint32_t phase = 0, tcount = 0, d_tmem = tmem_base;
        int ks = 0;
        bool ok = true, have_full = false;
        for (uint32_t base = 0; ok && base < total; base += T::kStages) {
#pragma unroll
          for (int s = 0; s < T::kStages; ++s) {
            if (base + s >= total) break;
            if (ks == 0) {  // first K step of a tile: its accumulator must have been drained by the epilogue
              const int a = tcount % T::kAccBufs;
              if (!(ok = mbar_wait(accempty + 8 * a, ((tcount / T::kAccBufs) & 1) ^ 1, ctx, 22))) break;
              d_tmem = tmem_base + a * T::kBN;
            }
            if (!have_full && !(ok = mbar_wait(full + 8 * s, phase, ctx, 24))) break;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < T::kBK / 16; ++kk) {
              if (kk == 2)  // is the next stage there already?  (never waits)
                have_full = mbar_test_wait(full + 8 * ((s + 1) % T::kStages), s + 1 == T::kStages ? (phase ^ 1) : phase);
              const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
              const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * T::kStageBytes + kk * 32) >> 4);
              const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((s * T::kStageBytes + kk * 32) >> 4);
              umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, acc);
            }
            umma_commit_pair(empty + 8 * s, 3);  // frees the stage in both CTAs
            if (++ks == k_steps) {
              umma_commit_pair(accfull + 8 * (tcount % T::kAccBufs), 3);
              ks = 0;
              ++tcount;
            }
          }
          phase ^= 1;
        }
      }
      __syncwarp();
    } else {
      // ------------------------------------------------------------ product pair: epilogue (warps 2..5, both CTAs)
      // The accumulator's lanes are rows of W, i.e. columns of Y; its columns are rows of X.  For one row of X the
      // 32 lanes of a warp write 32 neighbouring columns of Y (64 contiguous bytes).
      const int quad = warp & 3;
      uint32_t tcount = 0;
      bool ok = true;
      for (unsigned tile = pair; ok && tile < num_tiles; tile += prod_pairs, ++tcount) {
        unsigned xb, wt;
        oft4_tile(args.raster, tiles_x, tiles_w, tile, xb, wt);
        const int a = tcount % T::kAccBufs;
        if (!(ok = mbar_wait_warp(accfull + 8 * a, (tcount / T::kAccBufs) & 1, ctx, 40))) break;
        tc_fence_after();
        // Every MMA of the tile is done, so every load of its X.R rows (both CTAs') has landed: one count per tile.
        if (threadIdx.x == 64 && rank == 0) flag_signal(args.done + xb, 1);
        const int ycol = wt * T::kBN + rank * T::kBM + quad * 32 + lane;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + a * T::kBN;
        __half* out = args.C + ycol;
#pragma unroll 1
        for (int c = 0; c < T::kBN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_x32(t_row + c * 32, v);
          tmem_wait_ld();
          const int xrow0 = xb * 2 * T::kBM + c * 32;
          if (ycol < args.n) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (xrow0 + j < args.m) out[static_cast<long long>(xrow0 + j) * args.ldC] = __float2half_rn(__uint_as_float(v[j]));
          }
        }
        tc_fence_before();
        mbar_arrive_cluster(mapa_shared(accempty + 8 * a, 0));  // the leader's barrier collects both CTAs
        // A look ahead for the producer: are the rows of this pair's tile after next there?  (The next tile is
        // already being fed.)  One look; if not, the producer waits for them itself.
        if (threadIdx.x == 64 && tile + 2 * prod_pairs < num_tiles) {
          unsigned xb2, wt2;
          oft4_tile(args.raster, tiles_x, tiles_w, tile + 2 * prod_pairs, xb2, wt2);
          if (flag_test_ge(args.ready + 2 * xb2 + rank, static_cast<int>(upb))) {
            __threadfence_block();
            *seen_tile = tile + 2 * prod_pairs;
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  wait_profile_flush(ctx);
  __syncthreads();
  if (*abort_flag) {  // a wait ran out: let the copies in flight land before shared and tensor memory go away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while its pair may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

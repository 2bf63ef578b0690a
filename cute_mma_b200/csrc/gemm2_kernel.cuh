// Plain GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs on neighbouring SMs share one
// 256 x bN tile of C.  Each CTA loads its own 128 rows of A and its own half of the B tile (bN/2
// rows of N), so an SM pulls 32 KB per K stage from L2 instead of 48 KB and the ring is 6 deep; one
// thread of the even ("leader") CTA issues MMAs that read both CTAs' shared memory and write both
// CTAs' tensor memory.  Same operator and layouts as gemm_kernel.cuh (gemm_sm80_tc.cu:95-228).
//
// Protocol (per CTA, identical shared-memory layout in both):
//   full[s]     leader's barrier only: 1 arrival (leader's expect_tx) + the bytes of BOTH CTAs' copies;
//               the peer's TMA copies name the leader's barrier (pair form of cp.async.bulk.tensor)
//   empty[s]    one arrival per use from the leader's multicast tcgen05.commit (mask 0b11)
//   accfull[a]  one arrival per tile from the leader's multicast commit
//   accempty[a] leader's barrier only: 256 arrivals = the epilogue threads of both CTAs (the peer's
//               arrive through the cluster address of the leader's barrier)
// No load carries a multicast qualifier.  Both CTAs reach a cluster barrier before tensor memory is
// freed and before either exits, so no CTA leaves while its pair may still touch its memory.
#pragma once
#include "gemm_kernel.cuh"

namespace b200 {

template <typename TIn_, typename TOut_, bool kAMn_, bool kBMn_, int kBN_, int kStages_>
struct Gemm2Traits {
  using TIn = TIn_;
  using TOut = TOut_;
  static constexpr bool kAMn = kAMn_, kBMn = kBMn_;
  static constexpr int kBM = 128;                  // rows of C per CTA; the pair covers 256
  static constexpr int kBN = kBN_;                 // columns of C per pair (tcgen05 N)
  static constexpr int kBNHalf = kBN / 2;          // rows of the B tile each CTA loads
  static constexpr int kElem = sizeof(TIn);
  static constexpr int kBK = 128 / kElem;
  static constexpr int kUmmaK = 32 / kElem;
  static constexpr int kChunk = 128 / kElem;
  static constexpr int kStages = kStages_;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = kBNHalf * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kAccBufs = 2;
  static constexpr int kTmemCols = 512;
  static constexpr int kThreads = 192;
  static constexpr int kNumBars = 2 * kStages + 2 * kAccBufs;
  static constexpr int kSmemBytes = kStages * kStageBytes + kNumBars * 8 + 64 + 1024;
  static constexpr int kFmt = (kElem == 2) ? kFmtF16 : kFmtTF32;
  static constexpr bool kA32Atom = kAMn && kElem == 4, kB32Atom = kBMn && kElem == 4;
  static_assert(kBN % 64 == 0 && kBN >= 64 && kBN <= 256, "bN must be a multiple of 64 up to 256");
  static_assert(kBNHalf % kChunk == 0, "each CTA's half of the B tile must be whole 128-byte chunks");
  static_assert(kAccBufs * kBN <= kTmemCols, "accumulators exceed tensor memory");
  static_assert(kSmemBytes <= 232448, "shared memory ring too large");
};

template <class T, bool kSplit = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T::kThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const __grid_constant__ CUtensorMap tmap_a2, const __grid_constant__ CUtensorMap tmap_b2, const GemmArgs args) {
  using TOut = typename T::TOut;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
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
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs), 1 = peer
  const unsigned pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const unsigned tiles_m = (args.m + 2 * T::kBM - 1) / (2 * T::kBM), tiles_n = (args.n + T::kBN - 1) / T::kBN;
  const unsigned num_tiles = tiles_m * tiles_n;
  // C = A.B^T + A2.B2^T: the K steps of the second pair simply follow those of the first in every tile's stream
  const int k_steps1 = (args.k + T::kBK - 1) / T::kBK;
  const int k_steps = k_steps1 + (args.k2 + T::kBK - 1) / T::kBK;
  // Work items.  Without the split an item is a tile over all K steps.  With it, the tiles from args.split_first
  // on (all of them for a problem smaller than half a wave) are cut into args.split_parts pieces along K so that
  // idle SM pairs share them; the pieces meet in the epilogue (no CTA ever waits for another one).
  const unsigned num_items = kSplit ? args.split_first + (num_tiles - args.split_first) * args.split_parts : num_tiles;
  auto item_tile = [&](unsigned item) -> unsigned {
    if (!kSplit || item < args.split_first) return item;
    return args.split_first + (item - args.split_first) / args.split_parts;
  };
  auto item_part = [&](unsigned item) -> int { return (!kSplit || item < args.split_first) ? 0 : static_cast<int>((item - args.split_first) % args.split_parts); };
  auto item_ks0 = [&](unsigned item) -> int { return (!kSplit || item < args.split_first) ? 0 : item_part(item) * k_steps / args.split_parts; };
  auto item_ks1 = [&](unsigned item) -> int { return (!kSplit || item < args.split_first) ? k_steps : (item_part(item) + 1) * k_steps / args.split_parts; };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < T::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < T::kAccBufs; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 256); }
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    if (args.k2 > 0) { prefetch_tmap(&tmap_a2); prefetch_tmap(&tmap_b2); }
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), T::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the pair's barriers exist before anything arrives on them from the other CTA
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      unsigned done_rounds = 0, sync_target = 0;
      for (unsigned item = pair; ok && item < num_items; item += num_pairs) {
        const unsigned tile = item_tile(item);
        if (args.tile_sync && done_rounds > 0) {
          if (!(ok = tile_round_sync(args.rounds + rank, sync_target, ctx, 5))) break;
        }
        {
          const unsigned first = tile - pair, left = num_tiles - first;
          sync_target += left < num_pairs ? left : num_pairs;
          ++done_rounds;
        }
        unsigned tm, tn;
        tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
        const int m0 = tm * 2 * T::kBM + rank * T::kBM;      // this CTA's rows of A and C
        const int n0 = tn * T::kBN + rank * T::kBNHalf;      // this CTA's half of the B tile
        for (int ks = item_ks0(item), ks_end = item_ks1(item); ks < ks_end; ++ks, ++it) {
          const int s = it % T::kStages;
          if (!(ok = mbar_wait(empty_bar(s), ((it / T::kStages) & 1) ^ 1, ctx, 1))) break;
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * T::kStageBytes);  // both CTAs' bytes land on this barrier
          const uint32_t a_dst = smem_base + s * T::kStageBytes, b_dst = a_dst + T::kABytes;
          const bool second = ks >= k_steps1;
          const int k0 = (second ? ks - k_steps1 : ks) * T::kBK;
          if constexpr (!T::kAMn) {
            tma_load_2d_pair_hint(a_dst, second ? &tmap_a2 : &tmap_a, full_bar(s), k0, m0, args.hint_a);
          } else {
            if (args.a3d) {
              tma_load_3d_pair(a_dst, &tmap_a, full_bar(s), 0, k0, m0 / T::kChunk);
            } else {
#pragma unroll
              for (int c = 0; c < T::kBM / T::kChunk; ++c)
                tma_load_2d_pair(a_dst + c * (T::kBK * 128), &tmap_a, full_bar(s), m0 + c * T::kChunk, k0);
            }
          }
          if constexpr (!T::kBMn) {
            tma_load_2d_pair_hint(b_dst, second ? &tmap_b2 : &tmap_b, full_bar(s), k0, n0, args.hint_b);
          } else {
            if (args.b3d) {
              tma_load_3d_pair(b_dst, &tmap_b, full_bar(s), 0, k0, n0 / T::kChunk);
            } else {
#pragma unroll
              for (int c = 0; c < T::kBNHalf / T::kChunk; ++c)
                tma_load_2d_pair(b_dst + c * (T::kBK * 128), &tmap_b, full_bar(s), n0 + c * T::kChunk, k0);
            }
          }
        }
      }
      if (ok && args.tile_sync && done_rounds > 0) atomicAdd(args.rounds + rank, 1);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      // The issuing thread is on the critical path: measured with in-kernel cycle counters, every instruction
      // it executes between two MMAs shows up as idle time of the tensor pipe (a look at the next stage's
      // barrier whose address had to be computed: 512 -> 552 cycles per stage).  The ring is therefore walked
      // in a loop unrolled over its stages, so that every barrier address, parity and descriptor offset is a
      // constant plus a base register, and the tiles are flattened into one stream of K steps.
      constexpr uint32_t idesc = umma_idesc(T::kFmt, T::kAMn, T::kBMn, 2 * T::kBM, T::kBN);
      constexpr uint32_t a_adv = T::kAMn ? T::kUmmaK * 128 : 32, b_adv = T::kBMn ? T::kUmmaK * 128 : 32;
      constexpr uint32_t a_lbo = T::kAMn ? T::kBK * 128 : 16, b_lbo = T::kBMn ? T::kBK * 128 : 16;
      const uint64_t a_desc0 = umma_desc_sw128(smem_base, a_lbo, T::kA32Atom ? 512 : 1024, T::kA32Atom ? 1 : 2);
      const uint64_t b_desc0 = umma_desc_sw128(smem_base + T::kABytes, b_lbo, T::kB32Atom ? 512 : 1024, T::kB32Atom ? 1 : 2);
      unsigned my_tiles = 0;
      if (pair < num_items) my_tiles = (num_items - pair + num_pairs - 1) / num_pairs;
      uint32_t total = my_tiles * static_cast<uint32_t>(k_steps);
      int steps_this = k_steps;  // K steps of the item being multiplied
      if constexpr (kSplit) {
        total = 0;
        for (unsigned item = pair; item < num_items; item += num_pairs) total += static_cast<uint32_t>(item_ks1(item) - item_ks0(item));
      }
      const uint32_t full0 = full_bar(0), empty0 = empty_bar(0);
      uint32_t phase = 0, tcount = 0, d_tmem = tmem_base;
      int ks = 0;
      bool ok = true, have_full = false;
#ifdef B200_PROFILE_WAITS
      const long long issue_c0 = clock64();
#endif
      for (uint32_t base = 0; ok && base < total; base += T::kStages) {
#pragma unroll
        for (int s = 0; s < T::kStages; ++s) {
          if (base + s >= total) break;
          if (ks == 0) {  // first K step of a tile: its accumulator must have been drained by the epilogue
            const int a = tcount % T::kAccBufs;
            if (!(ok = mbar_wait(accempty_bar(a), ((tcount / T::kAccBufs) & 1) ^ 1, ctx, 2))) break;
            d_tmem = tmem_base + a * T::kBN;
            if constexpr (kSplit) {
              const unsigned item = pair + tcount * num_pairs;
              steps_this = item_ks1(item) - item_ks0(item);
            }
          }
          if (!have_full && !(ok = mbar_wait(full0 + 8 * s, phase, ctx, 3))) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < T::kBK / T::kUmmaK; ++kk) {
            if (kk == (T::kBK / T::kUmmaK) / 2)  // is the next stage there already?  (never waits; past the end it looks at a barrier nobody completes)
              have_full = mbar_test_wait(full0 + 8 * ((s + 1) % T::kStages), s + 1 == T::kStages ? (phase ^ 1) : phase);
            const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
            const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * T::kStageBytes + kk * a_adv) >> 4);
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((s * T::kStageBytes + kk * b_adv) >> 4);
            if constexpr (T::kFmt == kFmtF16) umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, acc);
            else umma_tf32_ss_pair(d_tmem, a_desc, b_desc, idesc, acc);
          }
          umma_commit_pair(empty0 + 8 * s, 3);  // frees the stage in both CTAs
          if (++ks == (kSplit ? steps_this : k_steps)) {
            umma_commit_pair(accfull_bar(tcount % T::kAccBufs), 3);
            ks = 0;
            ++tcount;
          }
        }
        phase ^= 1;
      }
#ifdef B200_PROFILE_WAITS  // site 62: cycles the issuing thread spent from its first MMA to its last commit
      ctx.prof_cycles[6] += static_cast<unsigned long long>(clock64() - issue_c0);
      ctx.prof_count[6] += 1u;
      ctx.prof_site[6] = 62;
#endif
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    uint32_t tcount = 0;
    bool ok = true;
    TOut* C = reinterpret_cast<TOut*>(args.C);
    const bool scaled = args.alpha != 1.f || args.beta != 0.f;
    for (unsigned item = pair; ok && item < num_items; item += num_pairs, ++tcount) {
      const unsigned tile = item_tile(item);
      unsigned tm, tn;
      tile_coord_r(args.raster, tiles_m, tiles_n, tile, tm, tn);
      const int a = tcount % T::kAccBufs;
      if (!(ok = mbar_wait_warp(accfull_bar(a), (tcount / T::kAccBufs) & 1, ctx, 4))) break;
      tc_fence_after();
      const int row = tm * 2 * T::kBM + rank * T::kBM + quad * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + a * T::kBN;
      if constexpr (kSplit) {
        if (item >= args.split_first) {
          // A piece of a split tile: park the fp32 partial tile (groups of four columns per row, so a thread moves
          // 16 bytes and a warp 512 contiguous bytes), count this CTA's arrival, and if it is the last of the tile's
          // pieces add all of them up in piece order (every run gives the same bits whoever comes last) and write C.
          const unsigned sidx = tile - args.split_first;
          const int part = item_part(item), parts = args.split_parts;  // parts <= 4
          const int r_in_cta = quad * 32 + lane;
          constexpr size_t kTileFloats = static_cast<size_t>(T::kBM) * T::kBN;
          float4* mine = reinterpret_cast<float4*>(args.split_scratch + ((static_cast<size_t>(sidx) * parts + part) * 2 + rank) * kTileFloats);
#pragma unroll 1
          for (int c = 0; c < T::kBN / 32; ++c) {
            uint32_t v[32];
            tmem_ld_x32(t_row + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < 8; ++g)
              mine[(c * 8 + g) * T::kBM + r_in_cta] = make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]),
                                                                  __uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3]));
          }
          tc_fence_before();
          mbar_arrive_cluster(mapa_shared(accempty_bar(a), 0));  // the accumulator is free again
          __threadfence();
          named_barrier_sync(1, 128);
          volatile int* arrivals = reinterpret_cast<volatile int*>(tmem_slot + 2);
          if (warp == 2 && lane == 0) *arrivals = atomicAdd(args.split_count + sidx * 2 + rank, 1);
          named_barrier_sync(1, 128);
          const bool last = (*arrivals == parts - 1);
          named_barrier_sync(1, 128);  // everyone has read the count before the next item may overwrite it
          if (last) {
            __threadfence();
            const float4* base = reinterpret_cast<const float4*>(args.split_scratch + (static_cast<size_t>(sidx) * parts * 2 + rank) * kTileFloats);
            constexpr size_t kPartStride = 2 * kTileFloats / 4;  // float4s between two pieces of one CTA's half tile
            if (row < args.m) {
#pragma unroll 1
              for (int g0 = 0; g0 < T::kBN / 4; g0 += 8) {  // 8 column groups x up to 4 pieces: 32 independent 16-byte loads
                float4 x[4][8];
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                  for (int g = 0; g < 8; ++g)
                    x[q][g] = (q < parts) ? __ldcg(base + q * kPartStride + (g0 + g) * T::kBM + r_in_cta) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                  float4 sum = x[0][g];
#pragma unroll
                  for (int q = 1; q < 4; ++q) { sum.x += x[q][g].x; sum.y += x[q][g].y; sum.z += x[q][g].z; sum.w += x[q][g].w; }
                  const float o[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int gcol = tn * T::kBN + (g0 + g) * 4 + e;
                    if (gcol < args.n) {
                      if constexpr (sizeof(TOut) == 2) C[row + static_cast<long long>(gcol) * args.ldC] = __float2half_rn(o[e]);
                      else C[row + static_cast<long long>(gcol) * args.ldC] = o[e];
                    }
                  }
                }
              }
            }
          }
          continue;
        }
      }
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
      mbar_arrive_cluster(mapa_shared(accempty_bar(a), 0));  // the leader's barrier collects both CTAs
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
  cluster_sync_all();  // neither CTA frees tensor memory or exits while its pair may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

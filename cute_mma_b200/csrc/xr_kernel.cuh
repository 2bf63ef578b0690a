// Rotation pass of the two-pass OFT product:  XR[M,K] = half(A . blockdiag(Rblk(g,kb)^T))  for one N-group g,
// i.e. per b-wide block of K columns  XR[:, kb*b .. kb*b+b) = half(A[:, kb*b .. kb*b+b) . Rblk(g,kb)^T)
// (fp16 in, fp32 accumulate, one round-to-nearest-even to fp16: the same X.R the fused kernel keeps in
// tensor memory, cute_oft_coop_pc.cu:19-186 in the reference).  The fused kernel recomputes X.R for every
// N tile of a group; when a group spans many N tiles it is cheaper to write X.R to memory once with this
// kernel and run the plain GEMM on it.  The pass is bound by memory traffic (2 bytes read + 2 bytes written
// per element of A, b/2 FLOPs per byte), so one CTA per SM streams (128 rows x U columns) units, U = max(b, 64):
//   warp 0      TMA producer of the {A, R} ring        warp 1      owns tensor memory, issues the MMAs
//   warps 2..5  epilogue of even units                 warps 6..9  epilogue of odd units
// An epilogue warpgroup reads the fp32 result from tensor memory, rounds it once to fp16, lays the (128 x 64)
// slice out in shared memory in the 128-byte swizzle and one of its threads stores it with a TMA tile store
// (whole 128-byte lines; the copy engine clips ragged edges).  Per-lane 16-byte stores straight to global
// memory, one row per lane, made the load/store unit the limit of this kernel (1740 cycles per unit, 0.59 of
// the copy bandwidth).  All hand-offs are mbarriers with bounded waits.
#pragma once
#include "ptx.cuh"

namespace b200 {

template <int kB_, int kS_>
struct XrTraits {
  static constexpr int kB = kB_;
  static constexpr int kBM = 128;
  static constexpr int kBK = 64;                       // fp16 columns of K per shared-memory stage (128 bytes)
  static constexpr int kUnitK = kB > 64 ? kB : 64;     // K columns per unit
  static constexpr int kStagesPerUnit = kUnitK / kBK;
  static constexpr int kS = kS_;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kRBytes = kB * 128;             // R tile: b rows (q) x 64 columns of K
  static constexpr int kSBytes = kABytes + kRBytes;
  static constexpr int kBufs = 4;                      // fp32 results in flight in tensor memory
  static constexpr int kTmemCols = kBufs * kUnitK;     // 256 or 512
  static constexpr int kThreads = 320;
  static constexpr int kNumBars = 2 * kS + 2 * kBufs;
  static constexpr int kOutBytes = kBM * 128;          // staging of one (128 x 64) fp16 slice, one per epilogue warpgroup
  static constexpr int kSmemBytes = kS * kSBytes + 2 * kOutBytes + kNumBars * 8 + 64 + 1024;
  static_assert(kB == 16 || kB == 32 || kB == 64 || kB == 128, "block edge must be 16, 32, 64 or 128");
  static_assert(kRBytes % 1024 == 0 && kSmemBytes <= 232448, "stage layout");
};

struct XrArgs {
  int m, k;
  int* status;
};

template <class T>
__global__ void __launch_bounds__(T::kThreads, 1)
xr_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_r,
          const __grid_constant__ CUtensorMap tmap_x, const XrArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t ring = smem_base;
  const uint32_t out_stage = ring + T::kS * T::kSBytes;
  const uint32_t bars = out_stage + 2 * T::kOutBytes;
  const uint32_t full = bars, empty = bars + 8u * T::kS;
  const uint32_t x_full = bars + 16u * T::kS, x_empty = x_full + 8u * T::kBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + (bars - smem_base) + T::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx ctx{abort_flag, args.status, kWaitLimitNs};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles_m = (args.m + T::kBM - 1) / T::kBM;
  const unsigned units = (args.k + T::kUnitK - 1) / T::kUnitK;
  const unsigned num_units = tiles_m * units;
  unsigned my_units = 0;
  if (blockIdx.x < num_units) my_units = (num_units - blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < T::kS; ++s) { mbar_init(full + 8 * s, 1); mbar_init(empty + 8 * s, 1); }
    for (int i = 0; i < T::kBufs; ++i) { mbar_init(x_full + 8 * i, 1); mbar_init(x_empty + 8 * i, 128); }
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_r);
    prefetch_tmap(&tmap_x);
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
    // -------------------------------------------------------------- producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (unsigned u = blockIdx.x; ok && u < num_units; u += gridDim.x) {
        const int m0 = (u / units) * T::kBM, k0 = (u % units) * T::kUnitK;
        for (int su = 0; su < T::kStagesPerUnit; ++su, ++it) {
          const int s = it % T::kS;
          if (!(ok = mbar_wait(empty + 8 * s, ((it / T::kS) & 1) ^ 1, ctx, 12))) break;
          mbar_expect_tx(full + 8 * s, T::kSBytes);
          const uint32_t dst = ring + s * T::kSBytes;
          tma_load_2d(dst, &tmap_a, full + 8 * s, k0 + su * T::kBK, m0);
          tma_load_2d(dst + T::kABytes, &tmap_r, full + 8 * s, k0 + su * T::kBK, 0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kFmtF16, 0, 0, T::kBM, T::kB);
      const uint64_t a_desc0 = umma_desc_sw128(ring, 16, 1024), r_desc0 = umma_desc_sw128(ring + T::kABytes, 16, 1024);
      uint32_t it = 0;
      bool ok = true;
      for (unsigned g = 0; ok && g < my_units; ++g) {
        const int buf = g % T::kBufs;
        if (!(ok = mbar_wait(x_empty + 8 * buf, ((g / T::kBufs) & 1) ^ 1, ctx, 25))) break;
        const uint32_t d = tmem_base + buf * T::kUnitK;
        for (int su = 0; su < T::kStagesPerUnit; ++su, ++it) {
          const int s = it % T::kS;
          if (!(ok = mbar_wait(full + 8 * s, (it / T::kS) & 1, ctx, 26))) break;
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (T::kSBytes >> 4));
          const uint64_t r_desc = r_desc0 + static_cast<uint64_t>(s * (T::kSBytes >> 4));
#pragma unroll
          for (int kk = 0; kk < T::kBK / 16; ++kk) {
            // b < 64: the stage holds 64/b diagonal blocks; slice kk belongs to block (kk*16)/b and lands in
            // columns [blk*b, blk*b+b).  b >= 64: one block, accumulated over the unit.
            constexpr bool small = T::kB < 64;
            const int blk = small ? (kk * 16) / T::kB : 0;
            const uint32_t accum = small ? ((((kk * 16) % T::kB) != 0) ? 1u : 0u) : ((su > 0 || kk > 0) ? 1u : 0u);
            umma_f16_ss(d + blk * T::kB, a_desc + kk * 2, r_desc + kk * 2, idesc, accum);
          }
          umma_commit(empty + 8 * s);
        }
        if (!ok) break;
        umma_commit(x_full + 8 * buf);
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------- epilogue: fp32 -> fp16 -> staging -> TMA store
    const int eg = (warp - 2) >> 2;  // this warpgroup takes the units of its parity
    const int quad = warp & 3;       // tensor-memory lanes a warp may read: 32 * (warp id mod 4)
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int r = quad * 32 + lane;  // row of the tile this thread converts
    const uint32_t stage = out_stage + eg * T::kOutBytes;
    const uint32_t my_row = stage + r * 128;
    const bool issuer = ((warp - 2) & 3) == 0 && lane == 0;
    bool ok = true;
    for (unsigned g = eg; ok && g < my_units; g += 2) {
      const unsigned u = blockIdx.x + g * gridDim.x;
      const int buf = g % T::kBufs;
      const int m0 = (u / units) * T::kBM, k0 = (u % units) * T::kUnitK;
      if (!(ok = mbar_wait_warp(x_full + 8 * buf, (g / T::kBufs) & 1, ctx, 41))) break;
      tc_fence_after();
      const uint32_t t = tmem_base + lane_off + buf * T::kUnitK;
#pragma unroll
      for (int h = 0; h < T::kUnitK / 64; ++h) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(t + h * 64, v0);
        tmem_ld_x32(t + h * 64 + 32, v1);
        tmem_wait_ld();
        if (h == T::kUnitK / 64 - 1) {  // everything of this buffer is in registers: hand it back before storing
          tc_fence_before();
          mbar_arrive(x_empty + 8 * buf);
        }
        uint32_t p[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __half2 a = __floats2half2_rn(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
          __half2 b = __floats2half2_rn(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
          p[j] = *reinterpret_cast<uint32_t*>(&a);
          p[16 + j] = *reinterpret_cast<uint32_t*>(&b);
        }
        if (issuer) bulk_wait_group_read<0>();  // the previous store of this warpgroup has read the staging buffer
        named_barrier_sync(1 + eg, 128);
#pragma unroll
        for (int c = 0; c < 8; ++c)  // 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r mod 8)
          st_shared_v4(my_row + ((c ^ (r & 7)) << 4), p[4 * c], p[4 * c + 1], p[4 * c + 2], p[4 * c + 3]);
        fence_proxy_async_smem();
        named_barrier_sync(1 + eg, 128);
        if (issuer) {
          tma_store_2d(&tmap_x, stage, k0 + h * 64, m0);
          bulk_commit_group();
        }
      }
    }
    if (issuer) bulk_wait_group<0>();  // every store of this thread is written before the CTA may exit
  }

  // ---------------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {  // a wait ran out: let the copies in flight land before shared and tensor memory go away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace b200

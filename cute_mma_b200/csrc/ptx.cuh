// Inline-PTX wrappers for the sm_100a building blocks used by the GEMM and OFT kernels:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld / st / fences) and the
// bounded-wait protocol that keeps a protocol bug from hanging the GPU.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace b200 {

// ---- device status record (global memory, owned by the library's per-device workspace) ----------
// status[0] = code (0 ok), [1] = blockIdx.x, [2] = wait site id, [3] = parity waited for.
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1 };
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // every mbarrier wait gives up after 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking look at a barrier phase (try_wait may suspend the thread; this never does).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Shared by every role of a CTA: where to raise the abort flag and where to record the failure.
struct WaitCtx {
  volatile int* abort_flag;  // shared memory, one per CTA
  int* status;               // global memory: 4 status ints, then (16-byte aligned) kWaitSites cycle counters
  unsigned long long limit_ns;
#ifdef B200_PROFILE_WAITS
  mutable unsigned long long prof_cycles[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  mutable unsigned prof_count[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  mutable int prof_site[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
};
// In-kernel stage timers: when the library is built with -DB200_PROFILE_WAITS every wait that
// has to spin adds its cycles to a per-site counter (and site+64 counts those waits), read back by b200_wait_profile.
constexpr int kWaitSites = 64;
constexpr int kStatusInts = 8;   // 4 status words, then 4 tile-round counters of the cross-CTA phase lock
constexpr int kTraceUnits = 32, kTraceEvents = 8;  // profiling build: clock64 stamps of CTA 0, units [kTraceFirst, +32)
constexpr int kTraceFirst = 70;
constexpr int kSkewCtas = 160, kSkewTiles = 24;  // profiling build: globaltimer at the end of each CTA's first tiles

__device__ __noinline__ void report_timeout(const WaitCtx& ctx, int site, uint32_t parity) {
  *ctx.abort_flag = 1;
  if (atomicCAS(ctx.status, kStatusOk, kStatusWaitTimeout) == kStatusOk) {
    ctx.status[1] = static_cast<int>(blockIdx.x);
    ctx.status[2] = site;
    ctx.status[3] = static_cast<int>(parity);
    __threadfence();
  }
}

// Bounded wait.  Returns false when this CTA is aborting (this wait or another one ran out); the
// caller then leaves its role loop and falls through to the common teardown.
__device__ __forceinline__ bool mbar_wait_impl(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  int it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63) == 0) {
      if (*ctx.abort_flag) return false;
      if (globaltimer_ns() - t0 > ctx.limit_ns) {
        report_timeout(ctx, site, parity);
        return false;
      }
    }
  }
}

// Profiling build: every wait adds its cycles to a per-thread slot (site % 8: the sites of one role map to distinct slots), flushed to the
// global counters once at the end of the kernel by wait_profile_flush().
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int site) {
#if defined(B200_PROFILE_WAITS) && !defined(B200_PROFILE_CYCLES_ONLY)
  // (try_wait may itself suspend the thread for a while, so every wait is timed, not only the spins)
  const long long c0 = clock64();
  const bool ok = mbar_wait_impl(bar, parity, ctx, site);
  ctx.prof_cycles[site & 7] += static_cast<unsigned long long>(clock64() - c0);
  ctx.prof_count[site & 7] += 1u;
  ctx.prof_site[site & 7] = site;
  return ok;
#else
  return mbar_wait_impl(bar, parity, ctx, site);
#endif
}
__device__ __forceinline__ void trace_stamp(const WaitCtx& ctx, unsigned unit, int event) {
#ifdef B200_PROFILE_WAITS
  if (blockIdx.x == 0 && unit >= kTraceFirst && unit < kTraceFirst + kTraceUnits) {
    unsigned long long* tr = reinterpret_cast<unsigned long long*>(ctx.status + kStatusInts) + 2 * kWaitSites;
    tr[(unit - kTraceFirst) * kTraceEvents + event] = static_cast<unsigned long long>(clock64());
  }
#endif
}
// Profiling build: globaltimer stamps of CTA 0 for its first kTraceUnits work items (same area as trace_stamp).
__device__ __forceinline__ void early_stamp(const WaitCtx& ctx, unsigned item, int event) {
#ifdef B200_PROFILE_WAITS
  if (blockIdx.x == 0 && item < kTraceUnits) {
    unsigned long long* tr = reinterpret_cast<unsigned long long*>(ctx.status + kStatusInts) + 2 * kWaitSites;
    tr[item * kTraceEvents + event] = globaltimer_ns();
  }
#endif
}
__device__ __forceinline__ void skew_stamp(const WaitCtx& ctx, unsigned tile_round) {
#ifdef B200_PROFILE_WAITS
  if (blockIdx.x < kSkewCtas && tile_round < kSkewTiles) {
    unsigned long long* sk = reinterpret_cast<unsigned long long*>(ctx.status + kStatusInts) + 2 * kWaitSites + kTraceUnits * kTraceEvents;
    sk[blockIdx.x * kSkewTiles + tile_round] = globaltimer_ns();
  }
#endif
}
__device__ __forceinline__ void wait_profile_flush(const WaitCtx& ctx) {
#ifdef B200_PROFILE_WAITS
  unsigned long long* prof = reinterpret_cast<unsigned long long*>(ctx.status + kStatusInts);
  for (int i = 0; i < 8; ++i)
    if (ctx.prof_count[i]) {
      atomicAdd(prof + ctx.prof_site[i], ctx.prof_cycles[i]);
      atomicAdd(prof + kWaitSites + ctx.prof_site[i], static_cast<unsigned long long>(ctx.prof_count[i]));
    }
#endif
}

// Cross-CTA phase lock for persistent kernels whose CTAs all are co-resident (grid <= SM count): the
// calling thread announces that it finished tile round `round` and waits, bounded, until `target` threads
// of its kind have done so.  Keeps concurrently running tiles within a few microseconds of each other so
// that the operand panels they share are still in L2 when the second reader arrives.
__device__ __forceinline__ bool tile_round_sync(int* counter, unsigned target, const WaitCtx& ctx, int site) {
  __threadfence();
  atomicAdd(counter, 1);
  const unsigned long long t0 = globaltimer_ns();
  int it = 0;
  while (static_cast<unsigned>(*reinterpret_cast<volatile int*>(counter)) < target) {
    if ((++it & 15) == 0) {
      if (*ctx.abort_flag) return false;
      if (globaltimer_ns() - t0 > ctx.limit_ns) {
        report_timeout(ctx, site, target);
        return false;
      }
    }
    __nanosleep(64);
  }
  return true;
}

// Counters in global memory that CTAs of one co-resident persistent kernel publish progress through.
// The data they guard moves through the async proxy (TMA stores and loads), so both sides put a proxy fence
// between the copies and the counter access.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Publishes whatever the calling thread wrote (or saw complete) before: one add with release semantics.
__device__ __forceinline__ void flag_signal(int* counter, int n) {
  fence_proxy_async_all();
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(counter), "r"(n) : "memory");
}
// Bounded wait until *counter >= target.  False when this CTA is aborting (this wait or another one ran out).
__device__ __forceinline__ bool flag_wait_ge_impl(const int* counter, int target, const WaitCtx& ctx, int site) {
  // polls with plain (volatile) loads; the acquire that orders the data behind the counter comes once, at the end
  if (*reinterpret_cast<const volatile int*>(counter) < target) {
    const unsigned long long t0 = globaltimer_ns();
    int it = 0;
    while (*reinterpret_cast<const volatile int*>(counter) < target) {
      if ((++it & 15) == 0) {
        if (*ctx.abort_flag) return false;
        if (globaltimer_ns() - t0 > ctx.limit_ns) {
          report_timeout(ctx, site, static_cast<uint32_t>(target));
          return false;
        }
      }
      __nanosleep(32);
    }
  }
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  fence_proxy_async_all();
  return true;
}

// One look, no waiting: true (with the same fences as a completed wait) when the counter has reached target.
__device__ __forceinline__ bool flag_test_ge(const int* counter, int target) {
  if (*reinterpret_cast<const volatile int*>(counter) < target) return false;
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  fence_proxy_async_all();
  return true;
}
__device__ __forceinline__ bool flag_wait_ge(const int* counter, int target, const WaitCtx& ctx, int site) {
#if defined(B200_PROFILE_WAITS) && !defined(B200_PROFILE_CYCLES_ONLY)
  const long long c0 = clock64();
  const bool ok = flag_wait_ge_impl(counter, target, ctx, site);
  ctx.prof_cycles[site & 7] += static_cast<unsigned long long>(clock64() - c0);
  ctx.prof_count[site & 7] += 1u;
  ctx.prof_site[site & 7] = site;
  return ok;
#else
  return flag_wait_ge_impl(counter, target, ctx, site);
#endif
}

// Waits that may take long and are not on the critical path of the tensor pipe (an epilogue waiting a whole tile
// for its accumulator, the rotation roles waiting for work): try_wait with a suspend-time hint, so that the
// hardware parks the thread until the phase completes instead of the thread polling.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_parked_impl(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  int it = 0;
  while (true) {
    if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
    if ((++it & 3) == 0) {
      if (*ctx.abort_flag) return false;
      if (globaltimer_ns() - t0 > ctx.limit_ns) {
        report_timeout(ctx, site, parity);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int site) {
#if defined(B200_PROFILE_WAITS) && !defined(B200_PROFILE_CYCLES_ONLY)
  const long long c0 = clock64();
  const bool ok = mbar_wait_parked_impl(bar, parity, ctx, site);
  ctx.prof_cycles[site & 7] += static_cast<unsigned long long>(clock64() - c0);
  ctx.prof_count[site & 7] += 1u;
  ctx.prof_site[site & 7] = site;
  return ok;
#else
  return mbar_wait_parked_impl(bar, parity, ctx, site);
#endif
}

// Whole-warp form for roles whose next instruction is warp-collective (tcgen05.ld / st / wait): every lane gets
// the same answer, so the warp stays converged when a wait gives up.  One lane waits (parked); the others then
// look at the completed phase once, which gives each of them the barrier's acquire.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int site) {
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_parked(bar, parity, ctx, site);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (ok)
    while (!mbar_try_wait(bar, parity)) {
    }
  return ok;
}

// Register re-balancing between warpgroups (all four warps of a warpgroup execute the same one).
template <int kRegs> __device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs> __device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---- TMA ----------------------------------------------------------------------------------------
// Tile store, shared memory (laid out as the tensor map's swizzle says) -> global; rows and columns past the
// tensor's extent are clipped by the copy engine.  The issuing thread groups its stores with commit_group and
// waits with wait_group: the .read form returns when the sources may be overwritten, the plain form when the
// data is written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending> __device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
template <int kPending> __device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}
// Barrier among `threads` threads (a multiple of 32) of the CTA that name the same id (1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load, completion counted in bytes on an mbarrier of this CTA.  x is the innermost
// coordinate: x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// 3-D tiled load (x innermost); used to fetch all 128-byte column chunks of an MN-major tile with one copy.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// ---- tcgen05: tensor memory ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One arrival on an mbarrier of this CTA once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] . B[smem]^T, fp16 inputs, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with A read from tensor memory (lane = row, two fp16 per 32-bit column along K).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp32 containers consumed as TF32, fp32 accumulate.
__device__ __forceinline__ void umma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// A warp reads its 32 lanes x 32 consecutive 32-bit columns (thread t <-> lane base+t).
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// A warp writes its 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---- CTA pairs (cta_group::2): one thread of the even CTA issues an MMA that spans both SMs ----------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of every CTA of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// In a CTA pair the shared-window address carries the CTA's rank in bit 24; clearing it names the
// same location in the even (leader) CTA.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
// Pair load: data lands in this CTA's shared memory, the bytes are counted on the leader's mbarrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Same with an L2 eviction-priority hint (one of the kL2* policy words below).
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y, uint64_t hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(x), "r"(y), "l"(hint)
      : "memory");
}
// Asks the copy engine to bring a tile into L2 ahead of the load that will use it (no shared memory, no barrier).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y)
               : "memory");
}
// Pre-encoded L2 cache policies (what createpolicy.fractional.L2::evict_* with fraction 1.0 returns).
constexpr uint64_t kL2EvictNormal = 0x1000000000000000ull;
constexpr uint64_t kL2EvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kL2EvictLast = 0x14F0000000000000ull;

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {  // same warp id in both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One arrival on the same mbarrier of every CTA in cta_mask once the issuing thread's MMAs are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- UMMA descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, tile rows of exactly 128 bytes.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
// K-major operand  (rows = M or N, 128 bytes of K per row): 8-row groups are 1024 bytes apart (SBO);
//                   the leading offset is not used by the hardware for swizzled K-major tiles.
// MN-major operand (rows = K, 128 bytes of M or N per row, tile = several such column chunks):
//                   8-row K groups are 1024 bytes apart (SBO), chunks are chunk_bytes apart (LBO).
// fp32 (TF32) MN-major operands have a single legal layout: layout type 1, the 128-byte swizzle whose
// unit is a 32-byte chunk (TMA mode 128B_ATOM_32B); its pattern repeats every 4 rows, so K groups
// are 4 rows = 512 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type = 2) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(layout_type) << 61;
  return d;
}
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t desc, uint32_t bytes) {
  return desc + static_cast<uint64_t>(bytes >> 4);
}

// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation.
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format (0 = f16, 2 = tf32)
//   [15] A major, [16] B major (0 = K-major, 1 = MN-major)   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc(int fmt, int a_mn_major, int b_mn_major, int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
constexpr int kFmtF16 = 0;
constexpr int kFmtTF32 = 2;

// ---- tile rasteriser -------------------------------------------------------------------------------
// Linear tile id -> (m, n) tile coordinate.  Same visiting order as the reference's z_curve
// (z_curve.hpp:4-49): the grid is factored level by level by the smallest prime factor of what is
// left of each dimension; inside a level m runs fastest.  For power-of-two grids this is Morton order.
__host__ __device__ inline unsigned smallest_prime_factor_of(unsigned n) {
  if (n <= 1u) return 1u;
  if (n % 2u == 0u) return 2u;
  for (unsigned d = 3u; d * d <= n; d += 2u)
    if (n % d == 0u) return d;
  return n;
}
__host__ __device__ inline void tile_coord(unsigned tiles_m, unsigned tiles_n, unsigned idx, unsigned& tm, unsigned& tn) {
  unsigned rem_m = tiles_m, rem_n = tiles_n, scale_m = 1u, scale_n = 1u;
  tm = 0u;
  tn = 0u;
  while (rem_m > 1u || rem_n > 1u) {
    const unsigned pm = smallest_prime_factor_of(rem_m), pn = smallest_prime_factor_of(rem_n);
    const unsigned level = idx % (pm * pn);
    idx /= pm * pn;
    tm += (level % pm) * scale_m;
    tn += (level / pm) * scale_n;
    scale_m *= pm;
    scale_n *= pn;
    rem_m /= pm;
    rem_n /= pn;
  }
}

// Tile order selected at launch: raster <= 0 is the z-curve above; raster = g > 0 walks bands of g tile
// rows, inside a band tile-column by tile-column (m fastest), so the g row panels of A stay in L2 while
// the band sweeps once over all of B.  Better than the z-curve when B is much larger than L2.
__host__ __device__ inline void tile_coord_r(int raster, unsigned tiles_m, unsigned tiles_n, unsigned idx, unsigned& tm, unsigned& tn) {
  if (raster <= 0) {
    tile_coord(tiles_m, tiles_n, idx, tm, tn);
    return;
  }
  const unsigned g = static_cast<unsigned>(raster);
  const unsigned band = idx / (g * tiles_n), r = idx % (g * tiles_n);
  const unsigned rows = (tiles_m - band * g) < g ? (tiles_m - band * g) : g;
  tn = r / rows;
  tm = band * g + r % rows;
}

}  // namespace b200

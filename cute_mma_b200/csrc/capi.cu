// Host side of the C ABI declared in include/cute_mma_b200.h: argument validation, TMA descriptor
// construction, launch of the sm_100a kernels, the per-device workspace (status record, staging
// buffers of the host-buffer entry point).  Takes over the role of the reference's host launchers
// oft_tn (cute_oft_coop_pc.cu:505-577) and gemm_tn / gemm_nt / gemm (gemm_sm80_tc.cu:95-228, 393-418),
// with the checks the reference leaves out (shape, alignment, shared-memory opt-in).
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>
#include <unordered_map>

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/cute_mma_b200.h"
#include "gemm_config.hpp"   // resolved through -I<config dir>
#include "oft_config.hpp"
#include "gemm_kernel.cuh"
#include "gemm2_kernel.cuh"
#include "oft_kernel.cuh"
#include "oft2_kernel.cuh"
#include "xr_kernel.cuh"
#include "oft3_kernel.cuh"
#include "oft4_kernel.cuh"

namespace {

using namespace b200;

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

// ---- launch options ----------------------------------------------------------------------------------
// Overrides of the launch heuristics, for experiments and tests.  -1 (or 0 for the route) means "let the
// library choose".  The B200_* environment variables of the same meaning are read ONCE, at the first use
// of any option in the process, as initial values; after that only b200_set_option changes them, so
// nothing on the launch path reads the environment.
enum OptionId { kOptOftRoute, kOptRaster, kOptTileSync, kOptL2Hints, kOptGemmTileSync, kOptGemmL2Hints, kOptGemmSplit, kOptMaps3d, kOptRingBands, kOptPrefetch, kOptRotPairs, kOptCount };
struct OptionDef { const char* name; const char* env; int initial; };
constexpr OptionDef kOptionDefs[kOptCount] = {
    {"oft_route", "B200_OFT_PATH", 0},            // 0 choose, 1 X.R in tensor memory per tile, 2 two passes, 3 / 4 X.R shared through the L2 ring
    {"raster", "B200_RASTER", -1},                // tile order: 0 z-curve, g > 0 bands of g tile rows
    {"tile_sync", "B200_TILE_SYNC", -1},          // cross-CTA phase lock of the fused kernels
    {"l2_hints", "B200_L2_HINTS", -1},            // 10 * a + b, a / b = 0 normal, 1 evict-first, 2 evict-last for the A / B loads
    {"gemm_tile_sync", "B200_GEMM_TILE_SYNC", -1},
    {"gemm_l2_hints", "B200_GEMM_L2_HINTS", -1},
    {"gemm_split", "B200_GEMM_SPLIT", -1},        // 0: never split small problems along K
    {"maps_3d", "B200_MAPS_3D", -1},              // 0: one 2-D copy per 128-byte chunk of an MN-major tile
    {"ring_bands", "B200_RING_BANDS", -1},        // bands of row blocks the X.R ring of route 3 holds (>= 2)
    {"prefetch", "B200_PREFETCH", -1},            // route 3: K steps by which W tiles are asked into L2 ahead of their load (0 off)
    {"rot_pairs", "B200_ROT_PAIRS", -1},          // route 4: SM pairs that only rotate (>= 1)
};
std::atomic<int> g_opt[kOptCount];
std::once_flag g_opt_once;
void options_init() {
  std::call_once(g_opt_once, [] {
    for (int i = 0; i < kOptCount; ++i) {
      int v = kOptionDefs[i].initial;
      if (const char* e = std::getenv(kOptionDefs[i].env)) v = std::atoi(e);
      g_opt[i].store(v);
    }
  });
}
int opt(OptionId id) {
  options_init();
  return g_opt[id].load(std::memory_order_relaxed);
}
unsigned long long hint_word(int code) { return code == 1 ? b200::kL2EvictFirst : (code == 2 ? b200::kL2EvictLast : b200::kL2EvictNormal); }

#define CUDA_TRY(call)                                                                       \
  do {                                                                                       \
    cudaError_t e_ = (call);                                                                 \
    if (e_ != cudaSuccess) return fail(B200_ECUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

// ---- per-device state ------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  long long l2_bytes = 126ll << 20;
  int* status = nullptr;            // 4 ints, zeroed; kernels record a timed-out wait here
  void* stage[4] = {nullptr, nullptr, nullptr, nullptr};  // staging of the host-buffer entry point
  size_t stage_bytes[4] = {0, 0, 0, 0};
  cudaStream_t host_stream = nullptr;  // compute stream of the host-buffer entry point
  cudaStream_t in_stream = nullptr, out_stream = nullptr;  // its host-to-device and device-to-host copy streams
  cudaMemPool_t pool = nullptr;     // stream-ordered scratch (expanded R, transformed weight); keeps its memory between calls
};
// workspace layout: kStatusInts ints of status, then 2 * kWaitSites 64-bit wait-profile counters
constexpr int kProfileWords = 2 * kWaitSites + kTraceUnits * kTraceEvents + kSkewCtas * kSkewTiles;  // counters, unit trace, tile-end times
constexpr size_t kWorkspaceBytes = kStatusInts * sizeof(int) + kProfileWords * sizeof(unsigned long long);
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;        // guards g_dev initialisation
std::mutex g_host_mu;   // serialises the host-buffer entry point (it owns the staging buffers)

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::mutex g_encode_mu;  // the allocating and the non-allocating set-up paths both look the entry point up

int resolve_encode() {
  std::lock_guard<std::mutex> lock(g_encode_mu);
  if (g_encode) return B200_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q)) {
    g_err = std::string("cudaGetDriverEntryPoint failed: ") + cudaGetErrorString(e);
    return B200_ECUDA;
  }
  if (q != cudaDriverEntryPointSuccess || !fn) {
    g_err = "cuTensorMapEncodeTiled not available from the driver";
    return B200_ECUDA;
  }
  g_encode = reinterpret_cast<EncodeFn>(fn);
  return B200_OK;
}

int device_state(DeviceState** out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(B200_EINVAL, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return fail(B200_EUNSUPPORTED, "device %d is sm_%d%d; this library contains sm_100a code only", dev, prop.major, prop.minor);
    st.sm_count = prop.multiProcessorCount;
    st.l2_bytes = prop.l2CacheSize > 0 ? prop.l2CacheSize : (126ll << 20);
    CUDA_TRY(cudaMalloc(&st.status, kWorkspaceBytes));
    CUDA_TRY(cudaMemset(st.status, 0, kWorkspaceBytes));
    // A pool of the library's own: the default pool hands unused memory back to the driver at every
    // synchronisation (release threshold 0), so a caller that synchronises between calls would pay a fresh
    // allocation on the next one (measured: 0.95 -> 1.6 ms per call at M = N = K = 8192, 8 x 8 blocks).
    cudaMemPoolProps props{};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    CUDA_TRY(cudaMemPoolCreate(&st.pool, &props));
    unsigned long long keep = ~0ull;
    CUDA_TRY(cudaMemPoolSetAttribute(st.pool, cudaMemPoolAttrReleaseThreshold, &keep));
    if (int rc = resolve_encode()) return rc;
    st.ready = true;
  }
  *out = &st;
  return B200_OK;
}

// 2-D tensor map over a matrix whose contiguous dimension has `inner` elements and whose other
// dimension has `outer` rows `ld` elements apart; boxes of box_inner x box_outer, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int elem_bytes, long long inner, long long outer, long long ld,
             int box_inner, int box_outer, const char* what, bool atom32 = false) {
  if (reinterpret_cast<uintptr_t>(base) & 15) return fail(B200_EINVAL, "%s: base pointer must be 16-byte aligned", what);
  if ((ld * elem_bytes) % 16 != 0) return fail(B200_EINVAL, "%s: leading dimension %lld x %d bytes must be a multiple of 16 bytes", what, ld, elem_bytes);
  if (ld < inner) return fail(B200_EINVAL, "%s: leading dimension %lld smaller than the contiguous extent %lld", what, ld, inner);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_ECUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, static_cast<int>(r));
  return B200_OK;
}

// Tile order of a launch.  The "raster" option overrides it for experiments.
int raster_for(long long operand_bytes, bool oft) {
  if (opt(kOptRaster) >= 0) return opt(kOptRaster);
  // Bands of 8 tile rows for the fused kernel once the operands no longer sit in L2 beside each other (see
  // launch_oft_gt); the plain GEMM chooses its order in launch_gemm_bn.
  return (oft && operand_bytes > (40ll << 20)) ? 8 : 0;
}

// 3-D map over an MN-major matrix [outer = K rows][inner = MN contiguous], inner a multiple of `chunk`:
// dimensions (chunk, K, inner / chunk) with strides (ld, chunk) elements, boxes of chunk x box_k x
// box_chunks.  One copy then brings box_chunks 128-byte column chunks, laid out chunk after chunk in
// shared memory exactly as the per-chunk 2-D copies would.  Returns B200_EUNSUPPORTED if the driver
// refuses the descriptor (the caller falls back to the 2-D map).
int make_map_chunks(CUtensorMap* map, const void* base, int elem_bytes, long long inner, long long outer, long long ld,
                    int chunk, int box_k, int box_chunks, bool atom32) {
  if (inner % chunk != 0 || (reinterpret_cast<uintptr_t>(base) & 15) || (ld * elem_bytes) % 16 != 0 || ld < inner) return B200_EUNSUPPORTED;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(chunk), static_cast<cuuint64_t>(outer), static_cast<cuuint64_t>(inner / chunk)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * elem_bytes, static_cast<cuuint64_t>(chunk) * elem_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(chunk), static_cast<cuuint32_t>(box_k), static_cast<cuuint32_t>(box_chunks)};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = g_encode(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_EUNSUPPORTED;
}

std::mutex g_optin_mu;
std::unordered_map<const void*, unsigned long long> g_optin;  // kernel -> bit per device ordinal that has opted in (cleared by b200_shutdown)

template <class Kernel>
int opt_in_smem(Kernel kernel, int bytes) {
  // The reference never raises the dynamic shared-memory limit and so cannot launch any tile
  // configuration above 48 KB; every kernel here needs the opt-in.
  // (once per kernel and device: the attribute belongs to the device's context)
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  const void* key = reinterpret_cast<const void*>(kernel);
  std::lock_guard<std::mutex> lock(g_optin_mu);
  unsigned long long& bits = g_optin[key];
  if (dev >= 0 && dev < 64 && ((bits >> dev) & 1ull)) return B200_OK;
  CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (dev >= 0 && dev < 64) bits |= 1ull << dev;
  return B200_OK;
}

int common_dims(int m, int n, int k, const void* A, const void* B, void* C) {
  if (m < 0 || n < 0 || k < 0) return fail(B200_EINVAL, "negative dimension (m=%d n=%d k=%d)", m, n, k);
  if (m > 0 && n > 0 && !C) return fail(B200_EINVAL, "C is null");
  if (m > 0 && n > 0 && k > 0 && (!A || !B)) return fail(B200_EINVAL, "A or B is null");
  return B200_OK;
}

// ---- plain GEMM --------------------------------------------------------------------------------------
// ctas = 2 in gemm_config.hpp selects the CTA-pair kernel (256 x bN tile per pair of SMs).
template <class P, class = void> struct CtasOf { static constexpr int value = 1; };
template <class P> struct CtasOf<P, decltype((void)P::ctas)> { static constexpr int value = P::ctas; };

// Launch of a phase-locked persistent kernel.  Its CTAs wait for one another between tile rounds, which is only
// safe when all of them are resident at once; a cooperative launch makes the device start them together (or not
// at all) even when other work holds some SMs.  If the cooperative launch is refused the caller launches again
// without the phase lock.
template <class Kernel, class... Args>
cudaError_t launch_cooperative(Kernel kernel, int grid, int threads, int smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Counters of the cross-CTA phase lock.  Each launch gets its own four, stream-ordered from the library's pool, so
// that launches on different streams never share them; the entry point that must not allocate uses the four
// that follow the status record in its static scratch (its calls may not overlap anyway).
int round_counters(DeviceState* st, cudaStream_t stream, int** out) {
  if (st->pool) {
    CUDA_TRY(cudaMallocFromPoolAsync(reinterpret_cast<void**>(out), 4 * sizeof(int), st->pool, stream));
  } else {
    *out = st->status + 4;
  }
  CUDA_TRY(cudaMemsetAsync(*out, 0, 4 * sizeof(int), stream));
  return B200_OK;
}
void release_round_counters(DeviceState* st, cudaStream_t stream, int* p) {
  if (st->pool && p) cudaFreeAsync(p, stream);
}

template <typename TIn, typename TOut, bool kNT, class P, int kBN>
int launch_gemm_bn(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream_v,
                   int k2, const void* A2, int ldA2, const void* B2, int ldB2, float alpha, float beta);

// (A pair kernel with half the N extent was tried for evening out the last wave of tiles and for small problems:
// a half-width tile takes 0.8 of the time of a full one, M = N = K = 4096 TF32 0.286 ms against 0.203 ms, so it
// never pays; the tiles of a short last wave are split along K instead, see below.)
template <typename TIn, typename TOut, bool kNT, class P>
int launch_gemm(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream_v,
                int k2 = 0, const void* A2 = nullptr, int ldA2 = 0, const void* B2 = nullptr, int ldB2 = 0, float alpha = 1.f, float beta = 0.f) {
  return launch_gemm_bn<TIn, TOut, kNT, P, P::bN>(m, n, k, A, ldA, B, ldB, C, ldC, stream_v, k2, A2, ldA2, B2, ldB2, alpha, beta);
}

template <typename TIn, typename TOut, bool kNT, class P, int kBN>
int launch_gemm_bn(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream_v,
                   int k2, const void* A2, int ldA2, const void* B2, int ldB2, float alpha, float beta) {
  constexpr bool kPair = CtasOf<P>::value == 2;
  using T1 = GemmTraits<TIn, TOut, kNT, kNT, kBN, kPair ? 4 : P::bP>;
  using T2 = Gemm2Traits<TIn, TOut, kNT, kNT, kBN, kPair ? P::bP : 6>;
  static_assert(P::bM == T1::kBM && P::bK == T1::kBK, "gemm_config.hpp: bM must be 128 and bK one 128-byte row");
  g_err.clear();
  if (int rc = common_dims(m, n, k, A, B, C)) return rc;
  if (ldC < m) return fail(B200_EINVAL, "ldC=%d smaller than m=%d (C is column-major)", ldC, m);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (m == 0 || n == 0) return B200_OK;
  if (k2 < 0 || (k2 > 0 && (!A2 || !B2))) return fail(B200_EINVAL, "bad second operand pair (k2=%d)", k2);
  if (k2 > 0 && (kNT || !kPair)) return fail(B200_EUNSUPPORTED, "a second operand pair needs K-contiguous operands and the CTA-pair kernel (ctas = 2)");
  if (k == 0 && k2 > 0) return launch_gemm_bn<TIn, TOut, kNT, P, kBN>(m, n, k2, A2, ldA2, B2, ldB2, C, ldC, stream_v, 0, nullptr, 0, nullptr, 0, alpha, beta);
  if (k == 0 && beta != 0.f) return fail(B200_EUNSUPPORTED, "k = 0 with beta != 0 (C = beta * C) is not a product; scale C yourself");
  if (k == 0) {
    CUDA_TRY(cudaMemset2DAsync(C, static_cast<size_t>(ldC) * sizeof(TOut), 0, static_cast<size_t>(m) * sizeof(TOut), n, stream));
    return B200_OK;
  }
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  constexpr int kBoxN = kPair ? T2::kBNHalf : T1::kBN;
  CUtensorMap ma, mb;
  int a3d = 0, b3d = 0;
  if (!kNT) {  // K contiguous
    if (int rc = make_map(&ma, A, sizeof(TIn), k, m, ldA, T1::kBK, T1::kBM, "A")) return rc;
    if (int rc = make_map(&mb, B, sizeof(TIn), k, n, ldB, T1::kBK, kBoxN, "B")) return rc;
  } else {     // M / N contiguous: all 128-byte column chunks of a tile with one 3-D copy when the extent is
               // a whole number of chunks (option maps_3d = 0 keeps the per-chunk 2-D copies), else one copy per chunk
    const bool try3d = opt(kOptMaps3d) != 0;
    if (try3d && make_map_chunks(&ma, A, sizeof(TIn), m, k, ldA, T1::kChunk, T1::kBK, T1::kBM / T1::kChunk, T1::kA32Atom) == B200_OK) a3d = 1;
    else if (int rc = make_map(&ma, A, sizeof(TIn), m, k, ldA, T1::kChunk, T1::kBK, "A", T1::kA32Atom)) return rc;
    if (try3d && make_map_chunks(&mb, B, sizeof(TIn), n, k, ldB, T1::kChunk, T1::kBK, kBoxN / T1::kChunk, T1::kB32Atom) == B200_OK) b3d = 1;
    else if (int rc = make_map(&mb, B, sizeof(TIn), n, k, ldB, T1::kChunk, T1::kBK, "B", T1::kB32Atom)) return rc;
  }
  // Cross-CTA phase lock of the tile rounds and banded tile order (see launch_oft) when the operand that spans
  // N is far larger than L2.  Measured at M 28672, N 65536, K 8192 (fp16): 34.2 ms with neither, 30.0 ms with
  // bands of 8 tile rows, 25.7 ms with both (before the L2 eviction priorities below were added).
  // The same three measures already pay when the two operands together exceed one and a half times L2 (one-pass
  // ncu counters, unthrottled launches): 8192^3 fp16 721 -> 689 us and 1.37 -> 0.85 GB of DRAM reads; M 8192,
  // N 4096, K 8192 354 -> 346 us; 4096 x 16384 x 4096 and below: no difference, so they stay on the z-curve.
  const bool big = kPair && (static_cast<long long>(m) + n) * k * static_cast<long long>(sizeof(TIn)) > 3ll * st->l2_bytes / 2;
  int tile_sync = big ? 1 : 0;
  if (opt(kOptGemmTileSync) >= 0) tile_sync = kPair ? opt(kOptGemmTileSync) : 0;
  int* rounds = nullptr;
  if (tile_sync)
    if (int rc = round_counters(st, stream, &rounds)) return rc;
  int raster = raster_for(static_cast<long long>(n) * k * sizeof(TIn), false);
  if (big && opt(kOptRaster) < 0) raster = 8;
  // With the bands, the band's panel of A is what later waves read again and B streams past once per band:
  // A is loaded evict-last, B evict-first.  Same shape: DRAM reads 26.2 -> 17.6 GB per launch, 23.9 -> 22.4 ms.
  unsigned long long hint_a = big ? kL2EvictLast : kL2EvictNormal, hint_b = big ? kL2EvictFirst : kL2EvictNormal;
  if (const int h = opt(kOptGemmL2Hints); h >= 0) { hint_a = hint_word(h / 10); hint_b = hint_word(h % 10); }
  GemmArgs args{m, n, k, C, ldC, st->status, raster, tile_sync, rounds, a3d, b3d, hint_a, hint_b, k2, 0u, 1, nullptr, nullptr, alpha, beta};
  if constexpr (kPair) {
    CUtensorMap ma2 = ma, mb2 = mb;  // never read when k2 == 0
    if (k2 > 0) {
      int rc = make_map(&ma2, A2, sizeof(TIn), k2, m, ldA2, T1::kBK, T1::kBM, "A2");
      if (rc == B200_OK) rc = make_map(&mb2, B2, sizeof(TIn), k2, n, ldB2, T1::kBK, kBoxN, "B2");
      if (rc != B200_OK) {
        release_round_counters(st, stream, rounds);
        return rc;
      }
    }
    const long long tiles = static_cast<long long>((m + 2 * T2::kBM - 1) / (2 * T2::kBM)) * ((n + T2::kBN - 1) / T2::kBN);
    // Split along K for problems of at most half a wave of tiles.  With P SM pairs and T <= P / 2 tiles, every
    // tile is cut into s = P / T pieces along K (at most 4, at least 8 K steps each) that run on otherwise idle
    // pairs and are summed by whichever piece of a tile finishes last (fp32 partial tiles in pool scratch, summed
    // in piece order: deterministic; no CTA waits for another).  Measured: M = N = 1024, K = 8192 fp16 49 -> 37 us.
    // Evening out the last wave of a larger problem the same way gained nothing (M = N = K = 4096 TF32: 0.2020
    // against 0.2031 ms; the reduction and the shorter K pipelines eat the saved half wave), so only problems
    // without a full wave are split.  Option gemm_split = 0 disables it.
    const long long all_pairs = st->sm_count / 2;
    const long long full_waves = tiles / all_pairs, rest = tiles % all_pairs;
    const long long k_steps_all = (k + T2::kBK - 1) / T2::kBK + (k2 + T2::kBK - 1) / T2::kBK;
    long long parts = (rest > 0 && rest * 2 <= all_pairs && full_waves == 0 && !big && st->pool) ? all_pairs / rest : 1;
    if (parts > 4) parts = 4;
    if (parts > k_steps_all / 8) parts = k_steps_all / 8;
    if (opt(kOptGemmSplit) == 0 || alpha != 1.f || beta != 0.f) parts = 1;  // the split instance sums pieces, it does not scale
    if (parts >= 2) {
      void* scratch = nullptr;
      const size_t tile_floats = static_cast<size_t>(T2::kBM) * T2::kBN;
      const size_t count_bytes = (static_cast<size_t>(rest) * 2 * sizeof(int) + 255) & ~static_cast<size_t>(255);
      const size_t bytes = count_bytes + static_cast<size_t>(rest) * parts * 2 * tile_floats * sizeof(float);
      if (cudaMallocFromPoolAsync(&scratch, bytes, st->pool, stream) == cudaSuccess) {
        CUDA_TRY(cudaMemsetAsync(scratch, 0, count_bytes, stream));
        args.split_first = static_cast<unsigned>(tiles - rest);
        args.split_parts = static_cast<int>(parts);
        args.split_count = static_cast<int*>(scratch);
        args.split_scratch = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + count_bytes);
        auto kernel = gemm2_kernel<T2, true>;
        if (int rc = opt_in_smem(kernel, T2::kSmemBytes)) {
          cudaFreeAsync(scratch, stream);
          release_round_counters(st, stream, rounds);
          return rc;
        }
        const long long items = tiles - rest + rest * parts;
        const int pairs = static_cast<int>(items < all_pairs ? items : all_pairs);
        kernel<<<2 * pairs, T2::kThreads, T2::kSmemBytes, stream>>>(ma, mb, ma2, mb2, args);
        const cudaError_t launched = cudaGetLastError();
        cudaFreeAsync(scratch, stream);
        release_round_counters(st, stream, rounds);
        CUDA_TRY(launched);
        return B200_OK;
      }
      cudaGetLastError();  // no scratch: the plain schedule
    }
    auto kernel = gemm2_kernel<T2>;
    if (int rc = opt_in_smem(kernel, T2::kSmemBytes)) return rc;
    const int pairs = static_cast<int>(tiles < st->sm_count / 2 ? tiles : st->sm_count / 2);
    bool launched_coop = false;
    if (args.tile_sync) {
      launched_coop = launch_cooperative(kernel, 2 * pairs, T2::kThreads, T2::kSmemBytes, stream, ma, mb, ma2, mb2, args) == cudaSuccess;
      if (!launched_coop) {
        cudaGetLastError();
        args.tile_sync = 0;
      }
    }
    if (!launched_coop) kernel<<<2 * pairs, T2::kThreads, T2::kSmemBytes, stream>>>(ma, mb, ma2, mb2, args);  // cluster dimension (2,1,1) is part of the kernel
  } else {
    auto kernel = gemm_kernel<T1>;
    if (int rc = opt_in_smem(kernel, T1::kSmemBytes)) return rc;
    const long long tiles = static_cast<long long>((m + T1::kBM - 1) / T1::kBM) * ((n + T1::kBN - 1) / T1::kBN);
    const int grid = static_cast<int>(tiles < st->sm_count ? tiles : st->sm_count);
    kernel<<<grid, T1::kThreads, T1::kSmemBytes, stream>>>(ma, mb, args);
  }
  const cudaError_t launched = cudaGetLastError();
  release_round_counters(st, stream, rounds);
  CUDA_TRY(launched);
  return B200_OK;
}

// ---- fused OFT ---------------------------------------------------------------------------------------
// ctas = 2 in oft_config.hpp selects the CTA-pair kernel (256 x bN tile per pair of SMs).
constexpr bool kOftPair = CtasOf<CurrCompParams>::value == 2;
// kGT > 1 (pair kernel only): group_size = bN / kGT, several N-groups (each with its own R) inside one tile.
// The R tiles of all groups travel with every stage of A, so the first ring gets shallower as they grow.
constexpr int oft_stages1(int b, int gt) {
  const int r_bytes = gt * (b / 2) * 128;
  return r_bytes <= 8 * 1024 ? CurrCompParams::bP1 : (r_bytes <= 16 * 1024 ? 3 : 2);
}
template <int kB, int kGT>
using OftT = std::conditional_t<kOftPair, Oft2Traits<kB, CurrCompParams::bN, oft_stages1(kB, kGT), CurrCompParams::bP2, kGT>,
                                OftTraits<kB, CurrCompParams::bN, CurrCompParams::bP1, CurrCompParams::bP2>>;

template <int kB, int kGT>
int launch_oft_gt(int m, int n, int k, int group_size, const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                  void* C, int ldC, cudaStream_t stream, DeviceState* st) {
  using T = OftT<kB, kGT>;
  static_assert(CurrCompParams::bM == T::kBM && CurrCompParams::bK == T::kBK, "oft_config.hpp: bM must be 128 and bK 64");
  if constexpr (!T::kFits) {
    return fail(B200_EUNSUPPORTED, "reconn_sz=%d with group_size=%d needs %d bytes of shared memory with this tile configuration (limit 232448)", kB,
                group_size, T::kSmemBytes);
  } else {
  const int n_groups = n / group_size;
  constexpr int kRowsPerCta = kOftPair ? 2 : 1;  // a pair splits the R tile and the B tile between its CTAs
  CUtensorMap ma, mr, mb;
  if (int rc = make_map(&ma, A, 2, k, m, ldA, T::kBK, T::kBM, "A")) return rc;
  if (int rc = make_map(&mr, R, 2, k, static_cast<long long>(n_groups) * kB, ldR, T::kBK, kB / kRowsPerCta, "R")) return rc;
  if (int rc = make_map(&mb, B, 2, k, n, ldB, T::kBK, T::kBN / kRowsPerCta / kGT, "B")) return rc;  // one copy per N-group of the tile
  // Tile order, L2 eviction priorities and the cross-CTA phase lock (pair kernel), chosen by the size of the two
  // operands together, (M + N) K fp16:
  //  * above 40 MB: bands of 8 tile rows instead of the z-curve (unthrottled launches under ncu, projection shape
  //    M 16384, K = N 4096, b 64: 438 -> 427 us, DRAM reads 372 -> 344 MB);
  //  * above 1.5 x L2 also the phase lock (without it the CTAs drift apart by up to a tile time, the panels that
  //    concurrently running tiles share fall out of L2 before the second reader arrives, and DRAM traffic grew
  //    to 17x the algorithmic bytes at M 65536, N 28672, K 8192: 650-730 -> 795-820 TFLOP/s with the lock) and
  //    evict-last for the band's rows of A, evict-first for B, which streams past it.  M = N = K = 8192, group
  //    256, b 8: 847 us with the bands alone, 835 with the lock, 828 with lock and priorities (DRAM reads
  //    1.26 -> 1.00 GB); priorities without the lock double the traffic (2.5 GB).  The priorities only when B
  //    itself exceeds L2: M 65536, N 28672, K 8192, b 128 27.85 -> 27.45 ms and 29.2 -> 22.5 GB of reads, but with
  //    N 3584 (B 59 MB, resident in L2 anyway) 3.551 -> 3.583 ms.
  // The options raster, tile_sync and l2_hints override each of them.
  const long long operand_bytes = (static_cast<long long>(m) + n) * k * 2;
  const bool big = kOftPair && operand_bytes > 3ll * st->l2_bytes / 2;
  const int raster = raster_for(operand_bytes, true);
  const bool streams = big && static_cast<long long>(n) * k * 2 > st->l2_bytes;  // B does not fit L2: it streams past the band
  unsigned long long hint_a = streams ? kL2EvictLast : kL2EvictNormal, hint_b = streams ? kL2EvictFirst : kL2EvictNormal;
  if (const int h = opt(kOptL2Hints); h >= 0) { hint_a = hint_word(h / 10); hint_b = hint_word(h % 10); }
  int tile_sync = big ? 1 : 0;
  if (opt(kOptTileSync) >= 0) tile_sync = kOftPair ? opt(kOptTileSync) : 0;
  int* rounds = nullptr;
  if (tile_sync)
    if (int rc = round_counters(st, stream, &rounds)) return rc;  // this launch's own counters, zeroed in stream order
  OftArgs args{m, n, k, group_size, static_cast<__half*>(C), ldC, st->status, raster, hint_a, hint_b, tile_sync, rounds};
  const long long tiles = static_cast<long long>((m + kRowsPerCta * T::kBM - 1) / (kRowsPerCta * T::kBM)) * ((n + T::kBN - 1) / T::kBN);
  if constexpr (kOftPair) {
    auto kernel = oft2_kernel<T>;
    if (int rc = opt_in_smem(kernel, T::kSmemBytes)) return rc;
    const int pairs = static_cast<int>(tiles < st->sm_count / 2 ? tiles : st->sm_count / 2);
    bool launched_coop = false;
    if (args.tile_sync) {
      launched_coop = launch_cooperative(kernel, 2 * pairs, T::kThreads, T::kSmemBytes, stream, ma, mr, mb, args) == cudaSuccess;
      if (!launched_coop) {
        cudaGetLastError();
        args.tile_sync = 0;
      }
    }
    if (!launched_coop) kernel<<<2 * pairs, T::kThreads, T::kSmemBytes, stream>>>(ma, mr, mb, args);  // cluster dimension (2,1,1) is part of the kernel
  } else {
    auto kernel = oft_kernel<T>;
    if (int rc = opt_in_smem(kernel, T::kSmemBytes)) return rc;
    const int grid = static_cast<int>(tiles < st->sm_count ? tiles : st->sm_count);
    kernel<<<grid, T::kThreads, T::kSmemBytes, stream>>>(ma, mr, mb, args);
  }
  const cudaError_t launched = cudaGetLastError();
  release_round_counters(st, stream, rounds);
  CUDA_TRY(launched);
  return B200_OK;
  }
}

// ---- two-pass OFT: rotation pass + plain GEMM ---------------------------------------------------------------
// The fused kernel recomputes X.R for every N tile of a group: per 64 columns of K a pair of SMs spends 726
// cycles (b <= 64) or 880-960 cycles (b = 128) where the plain GEMM spends 530-570.  Writing X.R to memory once
// (xr_kernel, bound by 4 bytes of traffic per element of X) and running the plain GEMM on it is cheaper as
// soon as a group spans enough N tiles: measured at M 65536, K 8192, N 28672, b 128: 38.2 ms fused, 26 ms in
// two passes.  Same arithmetic as the fused kernel: X.R rounded once to fp16, fp32 accumulation of the product.
template <int kB>
int launch_xr(int m, int k, const void* A, int ldA, const void* Rg, int ldR, void* XR, long long ldX, cudaStream_t stream, DeviceState* st) {
  using T = XrTraits<kB, 6>;
  CUtensorMap ma, mr, mx;
  if (int rc = make_map(&ma, A, 2, k, m, ldA, T::kBK, T::kBM, "A")) return rc;
  if (int rc = make_map(&mr, Rg, 2, k, kB, ldR, T::kBK, kB, "R")) return rc;
  if (int rc = make_map(&mx, XR, 2, k, m, ldX, T::kBK, T::kBM, "XR")) return rc;  // tile stores of (128 x 64) slices
  XrArgs args{m, k, st->status};
  const long long units = static_cast<long long>((m + T::kBM - 1) / T::kBM) * ((k + T::kUnitK - 1) / T::kUnitK);
  auto kernel = xr_kernel<T>;
  if (int rc = opt_in_smem(kernel, T::kSmemBytes)) return rc;
  kernel<<<static_cast<int>(units < st->sm_count ? units : st->sm_count), T::kThreads, T::kSmemBytes, stream>>>(ma, mr, mx, args);
  CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

constexpr int kNoScratch = -1000;  // internal: no device memory for X.R

template <int kB>
int oft_two_pass(int m, int n, int k, int group_size, const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                 void* C, int ldC, cudaStream_t stream, DeviceState* st) {
  if (!st->pool) return fail(B200_EUNSUPPORTED, "the two-pass path needs the library's scratch pool");
  const long long ldx = (k + 7) & ~7;
  void* xr = nullptr;
  if (cudaError_t e = cudaMallocFromPoolAsync(&xr, static_cast<size_t>(m) * ldx * 2, st->pool, stream)) {  // stays in the pool until b200_shutdown
    cudaGetLastError();
    if (e == cudaErrorMemoryAllocation) return kNoScratch;  // the caller decides: fused kernel, or an error for the explicit entry point
    return fail(B200_ECUDA, "cudaMallocFromPoolAsync: %s", cudaGetErrorString(e));
  }
  int rc = B200_OK;
  for (int g = 0; rc == B200_OK && g < n / group_size; ++g) {  // stream order serialises the groups on the one XR buffer
    rc = launch_xr<kB>(m, k, A, ldA, static_cast<const __half*>(R) + static_cast<long long>(g) * kB * ldR, ldR, xr, ldx, stream, st);
    // row-major C[m][n] is the column-major (n x m, ld = ldC) result of  W_g . XR^T:  gemm_tn with the operands swapped
    if (rc == B200_OK)
      rc = b200_gemm_tn_f16(group_size, m, k, static_cast<const __half*>(B) + static_cast<long long>(g) * group_size * ldB, ldB, xr,
                            static_cast<int>(ldx), static_cast<__half*>(C) + static_cast<long long>(g) * group_size, ldC, stream);
  }
  const std::string keep = g_err;
  cudaFreeAsync(xr, stream);
  g_err = keep;
  return rc;
}

// ---- fused OFT with X.R shared through an L2-resident ring (oft3_kernel, oft4_kernel) -----------------------
// One launch per N-group (each group has its own R, so its own X.R).  Scratch, stream-ordered from the library's
// pool: the ring of row blocks of X.R (at least 2 bands of row blocks of 256 rows, or all row blocks if fewer) and
// the zeroed ready / done / round counters of this launch.  The kernels' CTAs wait for one another, so they are only
// ever launched cooperatively (all CTAs resident); kNoRing tells the caller to take another route.
constexpr int kNoRing = -1001;

// Geometry and launch policy shared by the two kernels that keep X.R in the ring.
//   Tile order and ring size: a band of row blocks sweeps once over all of W.  When W stays in L2 beside the ring
//   the sweeps cost no DRAM traffic, so bands are short (4 row blocks): the tiles in flight then touch few row
//   blocks and the rotation can run further ahead in a ring of the same size.  When W streams from DRAM once per
//   band, bands of 8 halve that traffic.  The ring takes what L2 has left beside W (32 to 64 MB), at least two
//   bands, in whole bands.  The options raster and ring_bands override both.
//   Eviction priorities as for the plain pair GEMM (launch_gemm_bn): the band's rows of X.R are what the tiles of
//   a band share, W streams past them once per band, X is read once.
//   Phase lock of the tile rounds only when W streams from DRAM: the pairs that share a W tile then fetch it
//   together (one-pass ncu counters at M 16384, K 8192, N 28672: DRAM reads 19.1 -> 5.8 GB per launch, 6.13 -> 5.53 ms).
//   With W resident in L2 the ready / done counters keep the pairs close enough and the lock only costs time
//   (interleaved runs at M 65536, K 8192, N 3584: 17 % slower with it).
//   Rotation pairs (oft4_kernel only): measured under load, a pair of SMs that only rotates needs about 1.6 times
//   as long for 64 columns of a row block (256 x 64 of X, 0.7 to 0.8 us: shared-memory bandwidth) as a product pair
//   for one K step (0.5 us at the sustained clock), and a row block feeds tiles_w tiles; 25 % on top.
struct RingPlan {
  int tiles_x, tiles_w, raster, bands, bands_total, slots, tile_sync, rot_pairs;
  long long ldx;
  size_t counter_bytes, ring_bytes;
  unsigned long long hint_x, hint_a, hint_b;
};
RingPlan ring_plan(int m, int n, int k, const DeviceState* st) {
  RingPlan p;
  p.tiles_x = (m + 255) / 256;
  p.tiles_w = (n + 255) / 256;
  const long long w_bytes = static_cast<long long>(n) * k * 2, mib = 1ll << 20;
  const bool w_resident = w_bytes <= 64 * mib;
  p.raster = opt(kOptRaster) > 0 ? opt(kOptRaster) : (w_resident ? 4 : 8);
  p.ldx = (static_cast<long long>(k) + 63) & ~63ll;
  const long long block_bytes = 256 * p.ldx * 2;
  long long budget = 64 * mib;
  if (w_resident) {
    budget = st->l2_bytes - w_bytes - 16 * mib;
    budget = budget < 32 * mib ? 32 * mib : (budget > 64 * mib ? 64 * mib : budget);
  }
  p.bands = static_cast<int>(budget / (block_bytes * p.raster));
  if (p.bands < 2) p.bands = 2;
  if (opt(kOptRingBands) >= 2) p.bands = opt(kOptRingBands);
  p.bands_total = (p.tiles_x + p.raster - 1) / p.raster;
  p.slots = p.tiles_x <= p.bands * p.raster ? p.tiles_x : p.bands * p.raster;
  p.counter_bytes = ((static_cast<size_t>(3) * p.tiles_x + 4) * sizeof(int) + 1023) & ~static_cast<size_t>(1023);
  p.ring_bytes = static_cast<size_t>(p.slots) * 256 * p.ldx * 2;
  const long long operand_bytes = (static_cast<long long>(m) + n) * k * 2;
  const bool big = operand_bytes > 3ll * st->l2_bytes / 2;
  const bool streams = big && !w_resident;  // W cannot stay in L2 beside the ring: it streams from DRAM once per band
  p.hint_x = big ? kL2EvictFirst : kL2EvictNormal;
  p.hint_a = streams ? kL2EvictLast : kL2EvictNormal;
  p.hint_b = streams ? kL2EvictFirst : kL2EvictNormal;
  if (const int h = opt(kOptL2Hints); h >= 0) { p.hint_a = hint_word(h / 10); p.hint_b = hint_word(h % 10); }
  p.tile_sync = opt(kOptTileSync) >= 0 ? opt(kOptTileSync) : (streams ? 1 : 0);
  const double x = 1.6 / p.tiles_w;
  p.rot_pairs = static_cast<int>(1.25 * (st->sm_count / 2) * x / (1.0 + x) + 0.999);
  if (opt(kOptRotPairs) >= 1) p.rot_pairs = opt(kOptRotPairs);
  if (p.rot_pairs < 1) p.rot_pairs = 1;
  if (p.rot_pairs > st->sm_count / 4) p.rot_pairs = st->sm_count / 4;
  if (p.bands_total <= p.bands) p.rot_pairs = 0;  // the ring holds every row block: all pairs rotate, then all multiply
  return p;
}

// Further destinations of the result, set by b200_oft_tn_f16_gather for its own call: the shared-X.R kernel stores
// every tile to each of them from its epilogue (plain stores; the buffers may be another GPU's memory mapped into
// this process).  `stored` tells the entry point whether a launch took them; otherwise it copies.
struct MoreDst {
  int n = 0;
  __half* p[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  bool stored = false;
};
thread_local MoreDst g_more;

// Scratch of one ring launch, stream-ordered from the library's pool: zeroed counters, then the ring.
struct RingScratch {
  unsigned char* base = nullptr;
  cudaStream_t stream = nullptr;
  int* counters() const { return reinterpret_cast<int*>(base); }
  void* ring(const RingPlan& p) const { return base + p.counter_bytes; }
  ~RingScratch() {
    if (!base) return;
    const std::string keep = g_err;
    cudaFreeAsync(base, stream);
    g_err = keep;
  }
};
int ring_scratch(RingScratch* sc, const RingPlan& p, cudaStream_t stream, DeviceState* st) {
  if (cudaError_t e = cudaMallocFromPoolAsync(reinterpret_cast<void**>(&sc->base), p.counter_bytes + p.ring_bytes, st->pool, stream)) {
    cudaGetLastError();
    sc->base = nullptr;
    if (e == cudaErrorMemoryAllocation) return kNoRing;
    return fail(B200_ECUDA, "cudaMallocFromPoolAsync: %s", cudaGetErrorString(e));
  }
  sc->stream = stream;
  if (cudaError_t e = cudaMemsetAsync(sc->base, 0, p.counter_bytes, stream)) return fail(B200_ECUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  return B200_OK;
}

// oft3_kernel: every pair rotates and multiplies.
template <int kB>
int launch_oft3(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, const void* Rg, int ldR, void* C, int ldC,
                cudaStream_t stream, DeviceState* st, long long more_offset) {
  using T = Oft3Traits<kB, 2, 5>;
  if (!st->pool) return kNoRing;
  const RingPlan p = ring_plan(m, n, k, st);
  RingScratch sc;
  if (int rc = ring_scratch(&sc, p, stream, st)) return rc;
  int* counters = sc.counters();
  CUtensorMap mx, mr, mxr, mb;
  if (int rc = make_map(&mx, A, 2, k, m, ldA, T::kBK, T::kBM, "A")) return rc;
  if (int rc = make_map(&mr, Rg, 2, k, kB, ldR, T::kBK, kB / 2, "R")) return rc;
  if (int rc = make_map(&mxr, sc.ring(p), 2, p.ldx, static_cast<long long>(p.slots) * 2 * T::kBM, p.ldx, T::kBK, T::kBM, "XR ring")) return rc;
  if (int rc = make_map(&mb, B, 2, k, n, ldB, T::kBK, T::kBNHalf, "B")) return rc;
  // (asking W tiles into L2 a few K steps ahead of their loads was measured too: with the phase lock it added
  // 1.2 GB of DRAM reads and 5 % of time at M 16384, K 8192, N 28672, so it stays off unless the option asks for it)
  const int prefetch_w = opt(kOptPrefetch) >= 0 ? opt(kOptPrefetch) : 0;
  Oft3Args args{m, n, k, static_cast<__half*>(C), ldC, st->status, p.raster, p.hint_x, p.hint_a, p.hint_b,
                p.tile_sync, counters + 3 * p.tiles_x, prefetch_w, p.slots, counters, counters + 2 * p.tiles_x, g_more.n, {}};
  for (int d = 0; d < g_more.n; ++d) args.C_more[d] = g_more.p[d] + more_offset;
  auto kernel = oft3_kernel<T>;
  if (int rc = opt_in_smem(kernel, T::kSmemBytes)) return rc;
  const long long tiles = static_cast<long long>(p.tiles_x) * p.tiles_w;
  const int pairs = static_cast<int>(tiles < st->sm_count / 2 ? tiles : st->sm_count / 2);
  if (launch_cooperative(kernel, 2 * pairs, T::kThreads, T::kSmemBytes, stream, mx, mr, mxr, mb, args) != cudaSuccess) {
    cudaGetLastError();
    return kNoRing;
  }
  return B200_OK;
}

// oft4_kernel: the last rot_pairs pairs only rotate, the others only multiply (after all of them have rotated the
// first bands together).
template <int kB>
int launch_oft4(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, const void* Rg, int ldR, void* C, int ldC,
                cudaStream_t stream, DeviceState* st) {
  using T = Oft4Traits<kB>;
  if (!st->pool) return kNoRing;
  const RingPlan p = ring_plan(m, n, k, st);
  const long long tiles = static_cast<long long>(p.tiles_x) * p.tiles_w;
  const int all_pairs = st->sm_count / 2;
  const int prod_pairs = static_cast<int>(tiles < all_pairs - p.rot_pairs ? tiles : all_pairs - p.rot_pairs);
  // the first phase covers the first wave of tiles and one band more, as far as the ring goes
  int prologue = (prod_pairs + p.raster * p.tiles_w - 1) / (p.raster * p.tiles_w) + 1;
  if (prologue > p.bands) prologue = p.bands;
  if (p.rot_pairs == 0) prologue = p.bands_total;
  RingScratch sc;
  if (int rc = ring_scratch(&sc, p, stream, st)) return rc;
  int* counters = sc.counters();
  const long long ring_rows = static_cast<long long>(p.slots) * 2 * T::kBM;
  CUtensorMap mx, mr, mxr, mxs, mw;
  if (int rc = make_map(&mx, A, 2, k, m, ldA, T::kBK, T::kBM, "A")) return rc;
  if (int rc = make_map(&mr, Rg, 2, k, kB, ldR, T::kBK, kB / 2, "R")) return rc;
  if (int rc = make_map(&mxr, sc.ring(p), 2, p.ldx, ring_rows, p.ldx, T::kBK, T::kBM, "XR ring")) return rc;
  if (int rc = make_map(&mxs, sc.ring(p), 2, p.ldx, ring_rows, p.ldx, T::kBK, 32, "XR ring (stores)")) return rc;
  if (int rc = make_map(&mw, B, 2, k, n, ldB, T::kBK, T::kBM, "B")) return rc;
  Oft4Args args{m, n, k, static_cast<__half*>(C), ldC, st->status, p.raster, p.hint_x, p.hint_a, p.hint_b,
                p.tile_sync, counters + 3 * p.tiles_x, p.slots, counters, counters + 2 * p.tiles_x, p.rot_pairs, prologue};
  auto kernel = oft4_kernel<T>;
  if (int rc = opt_in_smem(kernel, T::kSmemBytes)) return rc;
  if (launch_cooperative(kernel, 2 * (prod_pairs + p.rot_pairs), T::kThreads, T::kSmemBytes, stream, mx, mr, mxr, mxs, mw, args) != cudaSuccess) {
    cudaGetLastError();
    return kNoRing;
  }
  return B200_OK;
}

template <int kB>
int oft_ring(int m, int n, int k, int group_size, const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
             void* C, int ldC, cudaStream_t stream, DeviceState* st, bool split_pairs) {
  int rc = B200_OK;
  for (int g = 0; rc == B200_OK && g < n / group_size; ++g) {  // stream order serialises the groups
    const __half* Bg = static_cast<const __half*>(B) + static_cast<long long>(g) * group_size * ldB;
    const __half* Rg = static_cast<const __half*>(R) + static_cast<long long>(g) * kB * ldR;
    __half* Cg = static_cast<__half*>(C) + static_cast<long long>(g) * group_size;
    if (split_pairs) rc = launch_oft4<kB>(m, group_size, k, A, ldA, Bg, ldB, Rg, ldR, Cg, ldC, stream, st);
    else rc = launch_oft3<kB>(m, group_size, k, A, ldA, Bg, ldB, Rg, ldR, Cg, ldC, stream, st, static_cast<long long>(g) * group_size);
  }
  if (rc == B200_OK && !split_pairs) g_more.stored = true;
  return rc;
}

// Routes of the AR_W product.  1: oft2_kernel, X.R kept in tensor memory and formed again for every N tile (no
// scratch; the only route for groups narrower than the N tile).  2: rotation pass + plain GEMM.  3: oft3_kernel,
// one X.R per row block shared by all N tiles of the group through the L2 ring, every SM pair rotating and
// multiplying.  4: oft4_kernel, the same ring with the rotation on a few SM pairs of its own, so that the others
// run the plain GEMM's loop (two accumulators, six stages).  0 = choose: a ring kernel when a group spans enough N
// tiles (its rotation work is 1 / tiles_n of route 1's, and unlike route 2 it neither writes X.R to HBM nor
// serialises the rotation in front of the product), else route 1.  Crossover measured at M 16384, K 4096
// (interleaved runs, route 3 / route 1 time): b 64: 4 tiles 1.13, 6 tiles 1.00, 8 tiles 0.98, 12 tiles 0.92,
// 16 tiles 0.95; b 128: 2 tiles 1.43, 4 tiles 0.95, 6 tiles 0.84, 8 tiles 0.82; b 32: 8 tiles 1.00; b 16: 16 tiles 0.89.
// Route 4 instead of 3 when three rotation pairs or fewer keep up with the product (wide groups: a rotation pair
// is bound by shared-memory bandwidth, and every pair that rotates is one that does not multiply).  Interleaved
// sustained runs, M 65536, K 8192, b 128, route 4 / route 3 time: N 28672 (2 pairs) 0.94, N 14336 (3 pairs) 0.93,
// N 7168 (6 pairs) 0.98 to 1.02, N 3584 (7 pairs) 1.02; M 16384, K = N 4096, b 64 (6 pairs) 1.25.
// Set by b200_oft_tn_f16_two_pass for its own call and by the option "oft_route".
thread_local int g_oft_path = 0;

int choose_route(int m, int group_size, int k, int b, const DeviceState* st) {
  int path = g_oft_path != 0 ? g_oft_path : opt(kOptOftRoute);
  const bool can_share = kOftPair && st->pool != nullptr;  // routes 2, 3 and 4 need scratch from the pool
  if (path == 2 || path == 3 || path == 4) return can_share ? path : 1;
  if (path == 1) return 1;
  const int min_tiles = b >= 128 ? 4 : 8;
  if (!can_share || group_size < min_tiles * static_cast<int>(CurrCompParams::bN)) return 1;
  if (g_more.n > 0) return 3;  // only oft3_kernel stores to further destinations
  // Route 4 also wants long tiles: its product pairs write C with the plain GEMM's epilogue (one 2-byte store per
  // element), which must fit beside a tile's MMAs.  Interleaved runs, route 4 / route 3 time: M 32768, N 28672, K 1024,
  // b 64: 1.61; M 262144, N 12288, K 2048, b 64 (3 pairs): 1.05; M 65536, N 28672, b 128 (2 pairs), K 2048: 0.86,
  // K 4096: 0.88.
  const RingPlan p = ring_plan(m, group_size, k, st);
  const int k_steps = (k + 63) / 64;
  const bool split = p.rot_pairs >= 1 && p.rot_pairs <= 3 && k_steps >= 32 && (p.rot_pairs <= 2 || k_steps >= 64);
  return split ? 4 : 3;
}

// group_size == n or a multiple of the N tile: one R per tile.  group_size a divisor of the N tile (the
// reference's bN % group_size == 0 case, cute_oft_coop_pc.cu:383): bN / group_size groups per tile, pair kernel.
template <int kB>
int launch_oft(int m, int n, int k, int group_size, const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
               void* C, int ldC, cudaStream_t stream, DeviceState* st) {
  constexpr int kBN = CurrCompParams::bN;
  const int route = choose_route(m, group_size, k, kB, st);
  if (route == 2) {
    const int rc = oft_two_pass<kB>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
    if (rc != kNoScratch) return rc;
    if (g_oft_path == 2) return fail(B200_ECUDA, "no device memory for the %lld bytes of X.R scratch", static_cast<long long>(m) * ((k + 7) & ~7) * 2);
    // out of memory for X.R: the kernel that keeps X.R in tensor memory needs no scratch
  }
  if constexpr (kOftPair) {
    if ((route == 3 || route == 4) && (group_size == n || group_size % kBN == 0)) {
      const int rc = oft_ring<kB>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st, route == 4);
      if (rc != kNoRing) return rc;
      // no scratch, or the cooperative launch was refused: fall through to the kernel that needs neither
    }
  }
  if (group_size == n || group_size % kBN == 0) return launch_oft_gt<kB, 1>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
  if constexpr (kOftPair && kB <= 64) {
    if (kBN % group_size == 0) {
      switch (kBN / group_size) {
        case 2: return launch_oft_gt<kB, 2>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
        case 4: return launch_oft_gt<kB, 4>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
        case 8: return launch_oft_gt<kB, 8>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
        default: break;
      }
    }
    return fail(B200_EUNSUPPORTED, "group_size=%d must equal n, be a multiple of the N tile %d, or be %d, %d or %d", group_size, kBN, kBN / 2, kBN / 4,
                kBN / 8);
  } else {
    return fail(B200_EUNSUPPORTED, "group_size=%d must equal n or be a multiple of the N tile %d (smaller groups need ctas = 2 and reconn_sz <= 64)",
                group_size, kBN);
  }
}

// ---- A_RW algebra: pre-transformed weight ----------------------------------------------------------------
// Y = X . (R . W): the rotation is folded into the weight once (cublas_oft.hpp:20-43 does this with batched
// cuBLAS calls), after which every product is a plain GEMM.  In the stored layouts
//   Bt[g*gs + j][kb*b + p] = half( sum_q R[g*b + q][kb*b + p] * B[g*gs + j][kb*b + q] )      fp32 accumulate
// One CTA transforms 64 rows of one N-group against one b x b block; 2*N*K*b FLOPs in all, on the CUDA cores
// (it runs once per weight update, not once per product).
__global__ void __launch_bounds__(256) transform_weight_kernel(const __half* __restrict__ B, long long ldB, const __half* __restrict__ R,
                                                               long long ldR, __half* __restrict__ Bt, long long ldBt, int group_size, int b,
                                                               int chunks_per_group) {
  extern __shared__ __half tw_smem[];
  __half* sR = tw_smem;            // [b][b]   sR[q][p]
  __half* sB = tw_smem + b * b;    // [64][b]  sB[r][q]
  const int kb = blockIdx.x, g = blockIdx.y / chunks_per_group, c = blockIdx.y % chunks_per_group;
  const int rows = min(64, group_size - c * 64);
  const long long row0 = static_cast<long long>(g) * group_size + c * 64, col0 = static_cast<long long>(kb) * b;
  for (int i = threadIdx.x; i < b * b; i += blockDim.x) sR[i] = R[(static_cast<long long>(g) * b + i / b) * ldR + col0 + i % b];
  for (int i = threadIdx.x; i < rows * b; i += blockDim.x) sB[i] = B[(row0 + i / b) * ldB + col0 + i % b];
  __syncthreads();
  for (int i = threadIdx.x; i < rows * b; i += blockDim.x) {
    const int r = i / b, p = i % b;
    float acc = 0.f;
    for (int q = 0; q < b; ++q) acc += __half2float(sB[r * b + q]) * __half2float(sR[q * b + p]);
    Bt[(row0 + r) * ldBt + col0 + p] = __float2half_rn(acc);
  }
}

// Tensor-core form of the same transform.  Per block, Bt_blk = B_blk . (R_blk^T)^T: the rotation pass of the two-pass
// route (xr_kernel) with the weight in X's place and every b x b block of R transposed, which a small kernel
// writes to scratch first (R is tiny beside B).  The reference does this step with batched tensor-core GEMMs
// through cuBLAS (cublas_oft.hpp:20-43).
__global__ void transpose_r_blocks_kernel(const __half* __restrict__ R, long long ldR, __half* __restrict__ Rt, long long ldt, int b, long long total) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / ldt, col = idx % ldt;  // row = g*b + p, col = kb*b + q  <-  R[g*b + q][kb*b + p]
    const long long g = row / b, p = row % b, kb = col / b, q = col % b;
    Rt[idx] = R[(g * b + q) * ldR + kb * b + p];
  }
}

template <int kB>
int launch_xr(int m, int k, const void* A, int ldA, const void* Rg, int ldR, void* XR, long long ldX, cudaStream_t stream, DeviceState* st);
int expand_r8(const void* R, int ldR, void* Rx, int n_groups, int k, cudaStream_t stream);
inline long long r8_ld(int k);
inline size_t r8_bytes(int n_groups, int k);

int transform_weight_tc(int n, int k, int group_size, int b, const void* B, int ldB, const void* R, int ldR, void* Bt, int ldBt, cudaStream_t stream,
                        DeviceState* st) {
  const int n_groups = n / group_size;
  const long long ldt = k;  // k is a multiple of b >= 8, so rows of the scratch stay 16-byte aligned
  __half* rt = nullptr;
  CUDA_TRY(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&rt), static_cast<size_t>(n_groups) * b * ldt * 2, st->pool, stream));
  const long long total = static_cast<long long>(n_groups) * b * ldt;
  transpose_r_blocks_kernel<<<static_cast<int>(total / 256 + 1 < 2048 ? total / 256 + 1 : 2048), 256, 0, stream>>>(static_cast<const __half*>(R), ldR, rt, ldt, b, total);
  int rc = cudaGetLastError() == cudaSuccess ? B200_OK : fail(B200_ECUDA, "launch of the block transpose failed");
  void* rx = nullptr;
  if (rc == B200_OK && b == 8) {  // 8 x 8 blocks: pairs of them embedded in 16 x 16 blocks, as for the product itself
    if (cudaMallocFromPoolAsync(&rx, r8_bytes(n_groups, k), st->pool, stream) != cudaSuccess) rc = fail(B200_ECUDA, "no scratch for the expanded R");
    if (rc == B200_OK) rc = expand_r8(rt, static_cast<int>(ldt), rx, n_groups, k, stream);
  }
  for (int g = 0; rc == B200_OK && g < n_groups; ++g) {
    const __half* Bg = static_cast<const __half*>(B) + static_cast<long long>(g) * group_size * ldB;
    __half* Btg = static_cast<__half*>(Bt) + static_cast<long long>(g) * group_size * ldBt;
    const __half* Rg = rt + static_cast<long long>(g) * b * ldt;
    switch (b) {
      case 8: rc = launch_xr<16>(group_size, k, Bg, ldB, static_cast<const __half*>(rx) + static_cast<long long>(g) * 16 * r8_ld(k), static_cast<int>(r8_ld(k)), Btg, ldBt, stream, st); break;
      case 16: rc = launch_xr<16>(group_size, k, Bg, ldB, Rg, static_cast<int>(ldt), Btg, ldBt, stream, st); break;
      case 32: rc = launch_xr<32>(group_size, k, Bg, ldB, Rg, static_cast<int>(ldt), Btg, ldBt, stream, st); break;
      case 64: rc = launch_xr<64>(group_size, k, Bg, ldB, Rg, static_cast<int>(ldt), Btg, ldBt, stream, st); break;
      case 128: rc = launch_xr<128>(group_size, k, Bg, ldB, Rg, static_cast<int>(ldt), Btg, ldBt, stream, st); break;
      default: rc = fail(B200_EUNSUPPORTED, "reconn_sz=%d", b);
    }
  }
  const std::string keep = g_err;
  if (rx) cudaFreeAsync(rx, stream);
  cudaFreeAsync(rt, stream);
  g_err = keep;
  return rc;
}

int transform_weight(int n, int k, int group_size, int b, const void* B, int ldB, const void* R, int ldR, void* Bt, int ldBt, cudaStream_t stream) {
  if (n < 0 || k < 0 || b <= 0 || group_size <= 0) return fail(B200_EINVAL, "bad transform_weight sizes (n=%d k=%d group_size=%d reconn_sz=%d)", n, k, group_size, b);
  if (b > 128) return fail(B200_EUNSUPPORTED, "reconn_sz=%d: the weight transform handles block edges up to 128", b);
  if (k % b != 0) return fail(B200_EINVAL, "k=%d is not a multiple of reconn_sz=%d", k, b);
  if (n % group_size != 0) return fail(B200_EINVAL, "n=%d is not a multiple of group_size=%d", n, group_size);
  if (ldB < k || ldR < k || ldBt < k) return fail(B200_EINVAL, "leading dimension smaller than k=%d", k);
  if (n == 0 || k == 0) return B200_OK;
  if (!B || !R || !Bt) return fail(B200_EINVAL, "B, R or the output is null");
  // Tensor cores when the block edge is one the rotation kernel is built for and the operands can be moved by TMA
  // (16-byte aligned bases, leading dimensions multiples of 8 elements); else the CUDA-core kernel below.
  const bool tma_ok = ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(Bt)) & 15) == 0 && ldB % 8 == 0 && ldBt % 8 == 0;
  if (tma_ok && (b == 8 || b == 16 || b == 32 || b == 64 || b == 128)) {
    DeviceState* st;
    if (int rc = device_state(&st)) return rc;
    if (st->pool) return transform_weight_tc(n, k, group_size, b, B, ldB, R, ldR, Bt, ldBt, stream, st);
  }
  const int chunks = (group_size + 63) / 64, n_groups = n / group_size;
  const size_t smem = (static_cast<size_t>(b) * b + 64 * b) * sizeof(__half);
  CUDA_TRY(cudaFuncSetAttribute(transform_weight_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  if (static_cast<long long>(n_groups) * chunks > 65535) return fail(B200_EUNSUPPORTED, "too many row chunks for one launch");
  transform_weight_kernel<<<dim3(k / b, n_groups * chunks), 256, smem, stream>>>(static_cast<const __half*>(B), ldB, static_cast<const __half*>(R), ldR,
                                                                             static_cast<__half*>(Bt), ldBt, group_size, b, chunks);
  CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// ---- self-test of the bounded-wait path ---------------------------------------------------------------
// One thread waits on an mbarrier that nothing ever arrives on, with a short limit: the wait gives up,
// records {code, CTA, site 99, parity} and the kernel returns normally.  Nothing faults or hangs.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    const WaitCtx ctx{&abort_flag, status, limit_ns};
    (void)mbar_wait(smem_u32(&bar), 0, ctx, 99);
  }
}

// ---- reconn_sz = 8 -----------------------------------------------------------------------------------
// tcgen05.mma needs N >= 16 and K = 16, so 8 x 8 blocks cannot be multiplied one by one.  Two
// neighbouring blocks (kb = 2j, 2j+1) of a group are embedded in one 16 x 16 block that is zero outside
// its two 8 x 8 diagonal corners, which leaves every sum unchanged (the added products are exact zeros):
//   Rx[g*16 + q'][16j + p'] = R[g*8 + (q' & 7)][16j + p']  if (q' >= 8) == (p' >= 8),  else 0
// and the product then runs as reconn_sz = 16 on Rx.  Rx is device scratch of 2x the size of R.
__global__ void expand_r8_kernel(const __half* __restrict__ R, long long ldR, __half* __restrict__ Rx, long long ldx,
                                 int n_groups, int k) {
  const long long chunks_per_row = ldx / 8;  // 8 halves = 16 bytes = one 8-wide block column
  const long long total = static_cast<long long>(n_groups) * 16 * chunks_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / chunks_per_row, c8 = idx % chunks_per_row;
    const int q = static_cast<int>(row % 16);
    const long long g = row / 16;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (((q >= 8) == ((c8 & 1) != 0)) && 8 * c8 < k)
      v = *reinterpret_cast<const uint4*>(R + (g * 8 + (q & 7)) * ldR + 8 * c8);
    *reinterpret_cast<uint4*>(Rx + row * ldx + 8 * c8) = v;
  }
}

inline long long r8_ld(int k) { return (static_cast<long long>(k) + 15) / 16 * 16; }
inline size_t r8_bytes(int n_groups, int k) { return static_cast<size_t>(n_groups) * 16 * r8_ld(k) * 2; }

int expand_r8(const void* R, int ldR, void* Rx, int n_groups, int k, cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(R) & 15) return fail(B200_EINVAL, "R: base pointer must be 16-byte aligned");
  if ((static_cast<long long>(ldR) * 2) % 16 != 0 || ldR < k) return fail(B200_EINVAL, "R: leading dimension %d must be >= k and a multiple of 8 elements", ldR);
  const long long total = static_cast<long long>(n_groups) * 16 * (r8_ld(k) / 8);
  const int blocks = static_cast<int>(total / 256 + 1 < 4096 ? total / 256 + 1 : 4096);
  expand_r8_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __half*>(R), ldR, static_cast<__half*>(Rx), r8_ld(k), n_groups, k);
  CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

int oft_dispatch(int m, int n, int k, int group_size, int b, const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                 void* C, int ldC, cudaStream_t stream) {
  g_err.clear();
  if (int rc = common_dims(m, n, k, A, B, C)) return rc;
  if (b <= 0 || group_size <= 0) return fail(B200_EINVAL, "group_size=%d and reconn_sz=%d must be positive", group_size, b);
  if (k % b != 0) return fail(B200_EINVAL, "k=%d is not a multiple of reconn_sz=%d", k, b);
  if (n % group_size != 0) return fail(B200_EINVAL, "n=%d is not a multiple of group_size=%d", n, group_size);
  if (ldC < n) return fail(B200_EINVAL, "ldC=%d smaller than n=%d (C is row-major)", ldC, n);
  if (m > 0 && n > 0 && k > 0 && !R) return fail(B200_EINVAL, "R is null");
  if (m == 0 || n == 0) return B200_OK;
  if (k == 0) {  // cpu_oft_tn zero-fills C and has no K block to add (cpu_oft.hpp:31,101-102)
    CUDA_TRY(cudaMemset2DAsync(C, static_cast<size_t>(ldC) * 2, 0, static_cast<size_t>(n) * 2, m, stream));
    return B200_OK;
  }
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  if (b == 8) {  // scratch from the stream-ordered allocator: no device-wide synchronisation, no sharing between calls
    const int n_groups = n / group_size;
    void* rx = nullptr;
    CUDA_TRY(cudaMallocFromPoolAsync(&rx, r8_bytes(n_groups, k), st->pool, stream));
    int rc = expand_r8(R, ldR, rx, n_groups, k, stream);
    if (rc == B200_OK) rc = launch_oft<16>(m, n, k, group_size, A, ldA, B, ldB, rx, static_cast<int>(r8_ld(k)), C, ldC, stream, st);
    cudaFreeAsync(rx, stream);
    return rc;
  }
  switch (b) {
    case 16: return launch_oft<16>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
    case 32: return launch_oft<32>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
    case 64: return launch_oft<64>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
    case 128: return launch_oft<128>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, st);
    default: return fail(B200_EUNSUPPORTED, "reconn_sz=%d not compiled in (8, 16, 32, 64, 128)", b);
  }
}

int stage_reserve(DeviceState* st, int slot, size_t bytes) {
  if (st->stage_bytes[slot] >= bytes) return B200_OK;
  if (st->stage[slot]) CUDA_TRY(cudaFree(st->stage[slot]));
  st->stage[slot] = nullptr;
  st->stage_bytes[slot] = 0;
  CUDA_TRY(cudaMalloc(&st->stage[slot], bytes));
  st->stage_bytes[slot] = bytes;
  return B200_OK;
}

// ---- scratch of the entry point that allocates nothing ------------------------------------------------
// Lives in the library image: every GPU that loads the library holds these bytes until the process
// exits.  In host code the name below is only a host-side stand-in for the symbol, never a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, per device.
constexpr size_t kStaticScratchBytes = 64 * 1024;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticScratchState {
  bool ready = false;
  int sm_count = 0;
  long long l2_bytes = 126ll << 20;
  void* scratch = nullptr;  // device address of g_static_scratch on this device
};
StaticScratchState g_static[kMaxDevices];
std::mutex g_static_mu;

// Device scratch one fused-OFT launch needs beyond its inputs and outputs: the status record of the
// bounded waits followed by the wait-profile words (the same layout the allocated workspace has).
// reconn_sz = 8 adds the expanded copy of R (see expand_r8_kernel) at kStaticRxOffset.
#ifdef B200_PROFILE_WAITS
constexpr size_t kStaticRecordBytes = kWorkspaceBytes;  // the kernels of this build also write their wait-profile words
constexpr size_t kStaticRxOffset = 36 * 1024;
#else
constexpr size_t kStaticRecordBytes = 256;              // status record (4 ints) and round counters (4 ints)
constexpr size_t kStaticRxOffset = 256;
#endif
static_assert(kStaticRecordBytes <= kStaticRxOffset && kStatusInts * sizeof(int) <= kStaticRecordBytes, "the record must fit below the expanded R");
size_t oft_scratch_bytes(int n_groups, int k, int reconn_sz) {
  return reconn_sz == 8 ? kStaticRxOffset + r8_bytes(n_groups, k) : kStaticRecordBytes;
}

// Once per device, with that device current.  Calls nothing that allocates device memory.
int static_scratch_state(StaticScratchState** out, cudaStream_t stream) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(B200_EINVAL, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticScratchState& st = g_static[dev];
  if (!st.ready) {
    int major = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(B200_EUNSUPPORTED, "device %d is not sm_100; this library contains sm_100a code only", dev);
    CUDA_TRY(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
    void* ptr = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (!ptr) return fail(B200_ECUDA, "cudaGetSymbolAddress returned a null address for the static scratch");
    int l2 = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev));
    st.l2_bytes = l2 > 0 ? l2 : (126ll << 20);
    // the status record must start at zero: cleared on the first caller's stream, ahead of its kernel; later
    // calls on other streams are ordered after this one by the rule that calls may not overlap
    CUDA_TRY(cudaMemsetAsync(ptr, 0, kStaticRecordBytes, stream));
    if (int rc = resolve_encode()) return rc;
    st.scratch = ptr;
    st.ready = true;
  }
  *out = &st;
  return B200_OK;
}

}  // namespace

extern "C" {

int b200_oft_tn_f16(int m, int n, int k, int group_size, int reconn_sz, const void* A, int ldA, const void* B, int ldB,
                    const void* R, int ldR, void* C, int ldC, void* stream) {
  return oft_dispatch(m, n, k, group_size, reconn_sz, A, ldA, B, ldB, R, ldR, C, ldC, static_cast<cudaStream_t>(stream));
}

int b200_rotate_f16(int m, int k, int reconn_sz, const void* A, int ldA, const void* R, int ldR, void* XR, int ldX, void* stream_v) {
  g_err.clear();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (m < 0 || k < 0 || reconn_sz <= 0) return fail(B200_EINVAL, "bad rotate sizes (m=%d k=%d reconn_sz=%d)", m, k, reconn_sz);
  if (k % reconn_sz != 0) return fail(B200_EINVAL, "k=%d is not a multiple of reconn_sz=%d", k, reconn_sz);
  if (m > 0 && k > 0 && (!A || !R || !XR)) return fail(B200_EINVAL, "A, R or XR is null");
  if (ldX < k) return fail(B200_EINVAL, "ldX=%d smaller than k=%d (XR is row-major)", ldX, k);
  if (m == 0 || k == 0) return B200_OK;
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  switch (reconn_sz) {
    case 8: {
      void* rx = nullptr;
      CUDA_TRY(cudaMallocFromPoolAsync(&rx, r8_bytes(1, k), st->pool, stream));
      int rc = expand_r8(R, ldR, rx, 1, k, stream);
      if (rc == B200_OK) rc = launch_xr<16>(m, k, A, ldA, rx, static_cast<int>(r8_ld(k)), XR, ldX, stream, st);
      cudaFreeAsync(rx, stream);
      return rc;
    }
    case 16: return launch_xr<16>(m, k, A, ldA, R, ldR, XR, ldX, stream, st);
    case 32: return launch_xr<32>(m, k, A, ldA, R, ldR, XR, ldX, stream, st);
    case 64: return launch_xr<64>(m, k, A, ldA, R, ldR, XR, ldX, stream, st);
    case 128: return launch_xr<128>(m, k, A, ldA, R, ldR, XR, ldX, stream, st);
    default: return fail(B200_EUNSUPPORTED, "reconn_sz=%d not compiled in (8, 16, 32, 64, 128)", reconn_sz);
  }
}

int b200_oft_plan(int m, int n, int k, int group_size, int reconn_sz, int* path, int* kernel_launches) {
  g_err.clear();
  if (m <= 0 || n <= 0 || k <= 0 || group_size <= 0 || reconn_sz <= 0 || n % group_size != 0 || k % reconn_sz != 0)
    return fail(B200_EINVAL, "bad plan arguments (m=%d n=%d k=%d group_size=%d reconn_sz=%d)", m, n, k, group_size, reconn_sz);
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  const int route = choose_route(m, group_size, k, reconn_sz == 8 ? 16 : reconn_sz, st);
  if (path) *path = route;
  const int groups = n / group_size;
  if (kernel_launches) *kernel_launches = (route == 2 ? 2 * groups : ((route == 3 || route == 4) ? groups : 1)) + (reconn_sz == 8 ? 1 : 0);
  return B200_OK;
}

int b200_oft_tn_f16_two_pass(int m, int n, int k, int group_size, int reconn_sz, const void* A, int ldA, const void* B, int ldB,
                             const void* R, int ldR, void* C, int ldC, void* stream) {
  g_oft_path = 2;
  const int rc = oft_dispatch(m, n, k, group_size, reconn_sz, A, ldA, B, ldB, R, ldR, C, ldC, static_cast<cudaStream_t>(stream));
  g_oft_path = 0;
  return rc;
}

int b200_oft_tn_f16_host(int m, int n, int k, int group_size, int reconn_sz, const void* A, int ldA, const void* B, int ldB,
                         const void* R, int ldR, void* C, int ldC) {
  g_err.clear();
  if (int rc = common_dims(m, n, k, A, B, C)) return rc;
  if (reconn_sz <= 0 || group_size <= 0 || n % group_size != 0) return fail(B200_EINVAL, "bad group_size / reconn_sz");
  if (ldA < k || ldB < k || ldR < k || ldC < n) return fail(B200_EINVAL, "leading dimension smaller than the row length");
  if (m == 0 || n == 0) return B200_OK;
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  std::lock_guard<std::mutex> lock(g_host_mu);
  if (!st->host_stream) CUDA_TRY(cudaStreamCreateWithFlags(&st->host_stream, cudaStreamNonBlocking));
  if (!st->in_stream) CUDA_TRY(cudaStreamCreateWithFlags(&st->in_stream, cudaStreamNonBlocking));
  if (!st->out_stream) CUDA_TRY(cudaStreamCreateWithFlags(&st->out_stream, cudaStreamNonBlocking));
  cudaStream_t s = st->host_stream, s_in = st->in_stream, s_out = st->out_stream;
  const int r_rows = (n / group_size) * reconn_sz;
  const int kp = (k + 7) & ~7, np = (n + 7) & ~7;  // device copies are packed with 16-byte aligned rows
  if (int rc = stage_reserve(st, 0, static_cast<size_t>(m) * kp * 2 + 16)) return rc;
  if (int rc = stage_reserve(st, 1, static_cast<size_t>(n) * kp * 2 + 16)) return rc;
  if (int rc = stage_reserve(st, 2, static_cast<size_t>(r_rows) * kp * 2 + 16)) return rc;
  if (int rc = stage_reserve(st, 3, static_cast<size_t>(m) * np * 2 + 16)) return rc;
  // Rows of X go up, are multiplied and come back chunk by chunk on three streams, so that the upload of chunk
  // i + 1, the product of chunk i and the download of chunk i - 1 overlap (the link is full duplex and the
  // download of Y is the longest leg: 3.76 GB against 1.55 GB up at M 65536, K 8192, N 28672).  Results do not
  // depend on the chunking: an element of Y only ever sees its own row of X and its own column of W.
  constexpr int kMaxChunks = 16;
  int chunk_rows = ((m + kMaxChunks - 1) / kMaxChunks + 255) & ~255;
  if (chunk_rows < 2048) chunk_rows = 2048;
  const int chunks = (m + chunk_rows - 1) / chunk_rows;
  cudaEvent_t up[kMaxChunks + 1] = {}, done[kMaxChunks] = {};
  int rc = B200_OK;
  auto check = [&](cudaError_t e, const char* what) {
    if (e != cudaSuccess && rc == B200_OK) rc = fail(B200_ECUDA, "%s: %s", what, cudaGetErrorString(e));
    return e == cudaSuccess;
  };
  for (int i = 0; i <= chunks && rc == B200_OK; ++i) check(cudaEventCreateWithFlags(&up[i], cudaEventDisableTiming), "cudaEventCreate");
  for (int i = 0; i < chunks && rc == B200_OK; ++i) check(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming), "cudaEventCreate");
  // The first row chunk does not wait for all of W: with one N-group, W goes up in kPieces column pieces behind
  // the first rows of X, and that chunk's product and download run piece by piece, so the download of Y (the
  // longest leg) starts after a quarter of W instead of all of it.
  constexpr int kPieces = 4;
  const bool piecewise = chunks > 1 && k > 0 && group_size == n && n % (kPieces * 256) == 0;
  cudaEvent_t w_up[kPieces] = {}, w_done[kPieces] = {};
  if (piecewise)
    for (int j = 0; j < kPieces && rc == B200_OK; ++j) {
      check(cudaEventCreateWithFlags(&w_up[j], cudaEventDisableTiming), "cudaEventCreate");
      if (rc == B200_OK) check(cudaEventCreateWithFlags(&w_done[j], cudaEventDisableTiming), "cudaEventCreate");
    }
  auto upload_rows = [&](int i) {
    const int r0 = i * chunk_rows, rows = (m - r0) < chunk_rows ? (m - r0) : chunk_rows;
    if (k > 0)
      check(cudaMemcpy2DAsync(static_cast<__half*>(st->stage[0]) + static_cast<size_t>(r0) * kp, kp * 2,
                              static_cast<const __half*>(A) + static_cast<size_t>(r0) * ldA, static_cast<size_t>(ldA) * 2,
                              static_cast<size_t>(k) * 2, rows, cudaMemcpyHostToDevice, s_in), "copy of A");
    if (rc == B200_OK) check(cudaEventRecord(up[i], s_in), "cudaEventRecord");
  };
  if (rc == B200_OK && k > 0)
    check(cudaMemcpy2DAsync(st->stage[2], kp * 2, R, static_cast<size_t>(ldR) * 2, static_cast<size_t>(k) * 2, r_rows, cudaMemcpyHostToDevice, s_in), "copy of R");
  if (piecewise && rc == B200_OK) upload_rows(0);
  if (rc == B200_OK && k > 0) {
    const int pieces = piecewise ? kPieces : 1, n_piece = n / pieces;
    for (int j = 0; j < pieces && rc == B200_OK; ++j) {
      check(cudaMemcpy2DAsync(static_cast<__half*>(st->stage[1]) + static_cast<size_t>(j) * n_piece * kp, kp * 2,
                              static_cast<const __half*>(B) + static_cast<size_t>(j) * n_piece * ldB, static_cast<size_t>(ldB) * 2,
                              static_cast<size_t>(k) * 2, n_piece, cudaMemcpyHostToDevice, s_in), "copy of B");
      if (piecewise && rc == B200_OK) check(cudaEventRecord(w_up[j], s_in), "cudaEventRecord");
    }
  }
  if (rc == B200_OK) check(cudaEventRecord(up[chunks], s_in), "cudaEventRecord");
  for (int i = 0; i < chunks && rc == B200_OK; ++i) {
    const int r0 = i * chunk_rows, rows = (m - r0) < chunk_rows ? (m - r0) : chunk_rows;
    __half* dA = static_cast<__half*>(st->stage[0]) + static_cast<size_t>(r0) * kp;
    __half* dC = static_cast<__half*>(st->stage[3]) + static_cast<size_t>(r0) * np;
    if (!(piecewise && i == 0)) upload_rows(i);
    if (rc == B200_OK) check(cudaStreamWaitEvent(s, up[i], 0), "cudaStreamWaitEvent");
    if (piecewise && i == 0) {
      const int n_piece = n / kPieces;
      for (int j = 0; j < kPieces && rc == B200_OK; ++j) {
        check(cudaStreamWaitEvent(s, w_up[j], 0), "cudaStreamWaitEvent");
        if (rc == B200_OK)
          rc = oft_dispatch(rows, n_piece, k, n_piece, reconn_sz, dA, kp, static_cast<__half*>(st->stage[1]) + static_cast<size_t>(j) * n_piece * kp, kp,
                            st->stage[2], kp, dC + static_cast<size_t>(j) * n_piece, np, s);
        if (rc == B200_OK) check(cudaEventRecord(w_done[j], s), "cudaEventRecord");
        if (rc == B200_OK) check(cudaStreamWaitEvent(s_out, w_done[j], 0), "cudaStreamWaitEvent");
        if (rc == B200_OK)
          check(cudaMemcpy2DAsync(static_cast<__half*>(C) + static_cast<size_t>(r0) * ldC + static_cast<size_t>(j) * n_piece, static_cast<size_t>(ldC) * 2,
                                  dC + static_cast<size_t>(j) * n_piece, np * 2, static_cast<size_t>(n_piece) * 2, rows, cudaMemcpyDeviceToHost, s_out),
                "copy of C");
      }
      continue;
    }
    if (rc == B200_OK) check(cudaStreamWaitEvent(s, up[chunks], 0), "cudaStreamWaitEvent");  // all of W and R
    if (rc == B200_OK) rc = oft_dispatch(rows, n, k, group_size, reconn_sz, dA, kp, st->stage[1], kp, st->stage[2], kp, dC, np, s);
    if (rc == B200_OK) check(cudaEventRecord(done[i], s), "cudaEventRecord");
    if (rc == B200_OK) check(cudaStreamWaitEvent(s_out, done[i], 0), "cudaStreamWaitEvent");
    if (rc == B200_OK)
      check(cudaMemcpy2DAsync(static_cast<__half*>(C) + static_cast<size_t>(r0) * ldC, static_cast<size_t>(ldC) * 2, dC, np * 2,
                              static_cast<size_t>(n) * 2, rows, cudaMemcpyDeviceToHost, s_out), "copy of C");
  }
  // everything queued is drained before the staging buffers may be reused, also after an error
  const std::string keep = g_err;
  cudaError_t e1 = cudaStreamSynchronize(s_in), e2 = cudaStreamSynchronize(s), e3 = cudaStreamSynchronize(s_out);
  for (int i = 0; i <= chunks; ++i) if (up[i]) cudaEventDestroy(up[i]);
  for (int i = 0; i < chunks; ++i) if (done[i]) cudaEventDestroy(done[i]);
  for (int j = 0; j < kPieces; ++j) { if (w_up[j]) cudaEventDestroy(w_up[j]); if (w_done[j]) cudaEventDestroy(w_done[j]); }
  if (rc != B200_OK) { g_err = keep; return rc; }
  if (!check(e1, "host-to-device stream") || !check(e2, "compute stream") || !check(e3, "device-to-host stream")) return rc;
  return B200_OK;
}

int b200_gemm_tn_f16(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream) {
  return launch_gemm<__half, __half, false, Params<half, half, MMA_T, MMA_N>>(m, n, k, A, ldA, B, ldB, C, ldC, stream);
}
int b200_gemm_tn_f16_acc2(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, int k2, const void* A2, int ldA2,
                          const void* B2, int ldB2, void* C, int ldC, void* stream) {
  return launch_gemm<__half, __half, false, Params<half, half, MMA_T, MMA_N>>(m, n, k, A, ldA, B, ldB, C, ldC, stream, k2, A2, ldA2, B2, ldB2);
}

int b200_lora_tn_f16(int m, int n, int k, int r, const void* X, int ldX, const void* W, int ldW, const void* L1, int ldL1,
                     const void* L2, int ldL2, void* C, int ldC, void* stream_v) {
  g_err.clear();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = common_dims(m, n, k, X, W, C)) return rc;
  if (r < 0 || (r > 0 && m > 0 && n > 0 && k > 0 && (!L1 || !L2))) return fail(B200_EINVAL, "bad low-rank factors (r=%d)", r);
  if (ldC < n) return fail(B200_EINVAL, "ldC=%d smaller than n=%d (C is row-major)", ldC, n);
  if (m == 0 || n == 0) return B200_OK;
  if (r == 0 || k == 0) return b200_gemm_tn_f16(n, m, k, W, ldW, X, ldX, C, ldC, stream_v);  // no adapter: the plain product, row-major
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  const int ldt = (r + 7) & ~7;
  void* t = nullptr;
  CUDA_TRY(cudaMallocFromPoolAsync(&t, static_cast<size_t>(m) * ldt * 2, st->pool, stream));
  // T[m][r] (row-major) = X . L1^T: the column-major r x m result of gemm_tn(L1, X); rounded to fp16 like the
  // reference's intermediate (playgrounds/lora.cu:44-49)
  int rc = b200_gemm_tn_f16(r, m, k, L1, ldL1, X, ldX, t, ldt, stream_v);
  // C[m][n] (row-major) = column-major n x m result of  W . X^T + L2 . T^T  in one pass over both operand pairs
  if (rc == B200_OK) rc = b200_gemm_tn_f16_acc2(n, m, k, W, ldW, X, ldX, r, L2, ldL2, t, ldt, C, ldC, stream_v);
  const std::string keep = g_err;
  cudaFreeAsync(t, stream);
  g_err = keep;
  return rc;
}

int b200_gemm_nt_f16(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream) {
  return launch_gemm<__half, __half, true, Params<half, half, MMA_N, MMA_T>>(m, n, k, A, ldA, B, ldB, C, ldC, stream);
}
int b200_gemm_tn_tf32(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream) {
  return launch_gemm<float, float, false, Params<float, float, MMA_T, MMA_N>>(m, n, k, A, ldA, B, ldB, C, ldC, stream);
}
int b200_gemm_nt_tf32(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream) {
  return launch_gemm<float, float, true, Params<float, float, MMA_N, MMA_T>>(m, n, k, A, ldA, B, ldB, C, ldC, stream);
}

int b200_gemm(char transA, char transB, int is_float, int m, int n, int k, const void* A, int ldA, const void* B, int ldB,
              void* C, int ldC, void* stream) {
  const bool tn = (transA == 'T' || transA == 't') && (transB == 'N' || transB == 'n');
  const bool nt = (transA == 'N' || transA == 'n') && (transB == 'T' || transB == 't');
  if (tn) return is_float ? b200_gemm_tn_tf32(m, n, k, A, ldA, B, ldB, C, ldC, stream) : b200_gemm_tn_f16(m, n, k, A, ldA, B, ldB, C, ldC, stream);
  if (nt) return is_float ? b200_gemm_nt_tf32(m, n, k, A, ldA, B, ldB, C, ldC, stream) : b200_gemm_nt_f16(m, n, k, A, ldA, B, ldB, C, ldC, stream);
  return fail(B200_EUNSUPPORTED, "gemm('%c','%c'): only ('T','N') and ('N','T') exist, as in the reference", transA, transB);
}

int b200_gemm_ex(char transA, char transB, int in_type, int out_type, int m, int n, int k, float alpha, const void* A, int ldA,
                 const void* B, int ldB, float beta, void* C, int ldC, void* stream) {
  const bool tn = (transA == 'T' || transA == 't') && (transB == 'N' || transB == 'n');
  const bool nt = (transA == 'N' || transA == 'n') && (transB == 'T' || transB == 't');
  g_err.clear();
  if (!tn && !nt) return fail(B200_EUNSUPPORTED, "gemm('%c','%c'): only ('T','N') and ('N','T') exist, as in the reference", transA, transB);
  using PH_TN = Params<half, half, MMA_T, MMA_N>;
  using PH_NT = Params<half, half, MMA_N, MMA_T>;
  using PF_TN = Params<float, float, MMA_T, MMA_N>;
  using PF_NT = Params<float, float, MMA_N, MMA_T>;
  if (in_type == B200_F16 && out_type == B200_F16)
    return tn ? launch_gemm<__half, __half, false, PH_TN>(m, n, k, A, ldA, B, ldB, C, ldC, stream, 0, nullptr, 0, nullptr, 0, alpha, beta)
              : launch_gemm<__half, __half, true, PH_NT>(m, n, k, A, ldA, B, ldB, C, ldC, stream, 0, nullptr, 0, nullptr, 0, alpha, beta);
  if (in_type == B200_F16 && out_type == B200_F32)
    return tn ? launch_gemm<__half, float, false, PH_TN>(m, n, k, A, ldA, B, ldB, C, ldC, stream, 0, nullptr, 0, nullptr, 0, alpha, beta)
              : launch_gemm<__half, float, true, PH_NT>(m, n, k, A, ldA, B, ldB, C, ldC, stream, 0, nullptr, 0, nullptr, 0, alpha, beta);
  if (in_type == B200_TF32 && out_type == B200_F32)
    return tn ? launch_gemm<float, float, false, PF_TN>(m, n, k, A, ldA, B, ldB, C, ldC, stream, 0, nullptr, 0, nullptr, 0, alpha, beta)
              : launch_gemm<float, float, true, PF_NT>(m, n, k, A, ldA, B, ldB, C, ldC, stream, 0, nullptr, 0, nullptr, 0, alpha, beta);
  return fail(B200_EUNSUPPORTED, "operand / result types %d / %d: f16 -> f16, f16 -> f32 and tf32 -> f32 exist", in_type, out_type);
}

int b200_gemm_rowmajor(char transA, char transB, int is_float, int m, int n, int k, const void* A, int ldA, const void* B, int ldB,
                       void* C, int ldC, void* stream) {
  // Row-major C (m x n, rows ldC apart) is the column-major n x m result of the same product with the operands
  // exchanged; both layouts keep their meaning under the exchange (K-contiguous stays K-contiguous).
  if (m > 0 && n > 0 && ldC < n) {
    g_err.clear();
    return fail(B200_EINVAL, "ldC=%d smaller than n=%d (C is row-major)", ldC, n);
  }
  return b200_gemm(transA, transB, is_float, n, m, k, B, ldB, A, ldA, C, ldC, stream);
}

int b200_peer_copy_async(void* dst, int dst_device, const void* src, int src_device, size_t bytes, void* stream) {
  g_err.clear();
  if (bytes == 0) return B200_OK;
  if (!dst || !src) return fail(B200_EINVAL, "null pointer in peer copy");
  if (dst_device != src_device) {  // direct copies over NVLink need peer access from the device that issues them
    int cur = 0, can = 0;
    CUDA_TRY(cudaGetDevice(&cur));
    CUDA_TRY(cudaDeviceCanAccessPeer(&can, src_device, dst_device));
    if (can) {
      if (cur != src_device) CUDA_TRY(cudaSetDevice(src_device));
      const cudaError_t e = cudaDeviceEnablePeerAccess(dst_device, 0);
      if (cur != src_device) cudaSetDevice(cur);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail(B200_ECUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
      cudaGetLastError();
    }
  }
  CUDA_TRY(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, static_cast<cudaStream_t>(stream)));
  return B200_OK;
}

int b200_shard_range(int n, int group_size, int world, int rank, int* n_begin, int* n_end) {
  g_err.clear();
  if (n < 0 || group_size <= 0 || world <= 0 || rank < 0 || rank >= world || !n_begin || !n_end)
    return fail(B200_EINVAL, "bad shard arguments (n=%d group_size=%d world=%d rank=%d)", n, group_size, world, rank);
  // Slabs are cut on multiples of `unit` columns: whole N-groups when R differs per group, otherwise
  // whole 256-column tiles so that every rank keeps full tiles; the remainder goes to the low ranks.
  const int unit = (group_size < n) ? group_size : 256;
  const int units = (n + unit - 1) / unit;
  const int base = units / world, extra = units % world;
  const long long u0 = static_cast<long long>(rank) * base + (rank < extra ? rank : extra);
  const long long u1 = u0 + base + (rank < extra ? 1 : 0);
  long long b0 = u0 * unit, b1 = u1 * unit;
  if (b0 > n) b0 = n;
  if (b1 > n) b1 = n;
  *n_begin = static_cast<int>(b0);
  *n_end = static_cast<int>(b1);
  return B200_OK;
}

int b200_oft_tn_f16_sharded(int m, int n, int k, int group_size, int reconn_sz, int world, const int* devices, const void* const* A, int ldA,
                            const void* const* B_slab, int ldB, const void* const* R_slab, int ldR, void* const* C_slab, int ldC,
                            void* const* streams) {
  g_err.clear();
  if (world <= 0 || !devices || !A || !B_slab || !R_slab || !C_slab) return fail(B200_EINVAL, "bad sharded arguments (world=%d)", world);
  if (group_size <= 0 || n < 0 || n % group_size != 0) return fail(B200_EINVAL, "n=%d is not a multiple of group_size=%d", n, group_size);
  int cur = 0;
  CUDA_TRY(cudaGetDevice(&cur));
  int rc = B200_OK;
  for (int r = 0; rc == B200_OK && r < world; ++r) {
    int n0 = 0, n1 = 0;
    rc = b200_shard_range(n, group_size, world, r, &n0, &n1);
    if (rc != B200_OK || n1 <= n0) continue;
    const int n_loc = n1 - n0;
    const int gs_loc = group_size >= n ? n_loc : group_size;  // one group over all of N: the slab is one group of its own width
    if (cudaError_t e = cudaSetDevice(devices[r])) {
      rc = fail(B200_ECUDA, "cudaSetDevice(%d): %s", devices[r], cudaGetErrorString(e));
      break;
    }
    rc = oft_dispatch(m, n_loc, k, gs_loc, reconn_sz, A[r], ldA, B_slab[r], ldB, R_slab[r], ldR, C_slab[r], ldC,
                      static_cast<cudaStream_t>(streams ? streams[r] : nullptr));
  }
  const std::string keep = g_err;
  cudaSetDevice(cur);
  g_err = keep;
  return rc;
}

int b200_oft_tn_f16_gather(int m, int n, int k, int group_size, int reconn_sz, const void* A, int ldA, const void* B, int ldB,
                           const void* R, int ldR, int n_dst, void* const* C_dst, int ldC, void* stream_v) {
  g_err.clear();
  if (n_dst < 1 || n_dst > 8 || !C_dst) return fail(B200_EINVAL, "n_dst=%d: between 1 and 8 destinations", n_dst);
  for (int d = 0; d < n_dst; ++d)
    if (!C_dst[d] && m > 0 && n > 0) return fail(B200_EINVAL, "destination %d is null", d);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  g_more = MoreDst{};
  g_more.n = n_dst - 1;
  for (int d = 1; d < n_dst; ++d) g_more.p[d - 1] = static_cast<__half*>(C_dst[d]);
  int rc = oft_dispatch(m, n, k, group_size, reconn_sz, A, ldA, B, ldB, R, ldR, C_dst[0], ldC, stream);
  const bool stored = g_more.stored;
  g_more = MoreDst{};
  if (rc != B200_OK || stored || m == 0 || n == 0) return rc;
  // a route without the multi-destination epilogue (few N tiles per group, k = 0, no scratch): copy the result
  for (int d = 1; d < n_dst; ++d)
    CUDA_TRY(cudaMemcpy2DAsync(C_dst[d], static_cast<size_t>(ldC) * 2, C_dst[0], static_cast<size_t>(ldC) * 2, static_cast<size_t>(n) * 2, m,
                               cudaMemcpyDeviceToDevice, stream));
  return B200_OK;
}

int b200_tile_coord(unsigned tiles_m, unsigned tiles_n, unsigned idx, unsigned* tile_m, unsigned* tile_n) {
  g_err.clear();
  if (!tile_m || !tile_n || tiles_m == 0 || tiles_n == 0 || idx >= tiles_m * tiles_n) return fail(B200_EINVAL, "tile index out of range");
  b200::tile_coord(tiles_m, tiles_n, idx, *tile_m, *tile_n);
  return B200_OK;
}

int b200_device_status(int out[4]) {
  g_err.clear();
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  CUDA_TRY(cudaDeviceSynchronize());
  int host[4] = {0, 0, 0, 0};
  CUDA_TRY(cudaMemcpy(host, st->status, sizeof host, cudaMemcpyDeviceToHost));
  if (out) std::memcpy(out, host, sizeof host);
  if (host[0] != 0) {
    CUDA_TRY(cudaMemset(st->status, 0, sizeof host));
    return fail(B200_EDEVICE, "a bounded wait ran out in CTA %d at wait site %d (parity %d)", host[1], host[2], host[3]);
  }
  return B200_OK;
}

int b200_static_status(int out[4]) {
  g_err.clear();
  StaticScratchState* ss;
  if (int rc = static_scratch_state(&ss, nullptr)) return rc;
  CUDA_TRY(cudaDeviceSynchronize());
  int host[4] = {0, 0, 0, 0};
  CUDA_TRY(cudaMemcpy(host, ss->scratch, sizeof host, cudaMemcpyDeviceToHost));
  if (out) std::memcpy(out, host, sizeof host);
  if (host[0] != 0) {
    CUDA_TRY(cudaMemset(ss->scratch, 0, sizeof host));
    return fail(B200_EDEVICE, "a bounded wait ran out in CTA %d at wait site %d (parity %d)", host[1], host[2], host[3]);
  }
  return B200_OK;
}

int b200_transform_weight_f16(int n, int k, int group_size, int reconn_sz, const void* B, int ldB, const void* R, int ldR,
                              void* Bt, int ldBt, void* stream) {
  g_err.clear();
  return transform_weight(n, k, group_size, reconn_sz, B, ldB, R, ldR, Bt, ldBt, static_cast<cudaStream_t>(stream));
}

int b200_oft_tn_f16_a_rw(int m, int n, int k, int group_size, int reconn_sz, const void* A, int ldA, const void* B, int ldB,
                         const void* R, int ldR, void* C, int ldC, void* stream_v) {
  g_err.clear();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = common_dims(m, n, k, A, B, C)) return rc;
  if (ldC < n) return fail(B200_EINVAL, "ldC=%d smaller than n=%d (C is row-major)", ldC, n);
  if (m == 0 || n == 0) return B200_OK;
  if (k == 0) {
    CUDA_TRY(cudaMemset2DAsync(C, static_cast<size_t>(ldC) * 2, 0, static_cast<size_t>(n) * 2, m, stream));
    return B200_OK;
  }
  const int ldt = (k + 7) & ~7;
  void* bt = nullptr;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  CUDA_TRY(cudaMallocFromPoolAsync(&bt, static_cast<size_t>(n) * ldt * 2, st->pool, stream));  // stays in the library's pool until b200_shutdown
  int rc = transform_weight(n, k, group_size, reconn_sz, B, ldB, R, ldR, bt, ldt, stream);
  // row-major C[m][n] is the column-major (n x m, ld = ldC) result of  Bt . A^T:  gemm_tn with the operands swapped
  if (rc == B200_OK) rc = b200_gemm_tn_f16(n, m, k, bt, ldt, A, ldA, C, ldC, stream);
  const std::string keep = g_err;
  cudaFreeAsync(bt, stream);
  g_err = keep;
  return rc;
}

int b200_selftest_wait_timeout(unsigned limit_us, int out[4]) {
  g_err.clear();
  if (limit_us == 0 || limit_us > 100000) return fail(B200_EINVAL, "limit_us must be in 1..100000");
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  wait_timeout_selftest_kernel<<<1, 32>>>(st->status, static_cast<unsigned long long>(limit_us) * 1000ull);
  CUDA_TRY(cudaGetLastError());
  const int rc = b200_device_status(out);  // synchronises, reads and clears the record
  if (rc != B200_EDEVICE) return fail(B200_ECUDA, "the wait did not report a timeout (status call returned %d)", rc);
  g_err.clear();
  return B200_OK;
}

int b200_wait_profile(unsigned long long* out, int n) {
  g_err.clear();
#ifdef B200_PROFILE_WAITS
  DeviceState* st;
  if (int rc = device_state(&st)) return rc;
  if (!out || n < 0 || n > kProfileWords) return fail(B200_EINVAL, "out must hold at most %d counters", kProfileWords);
  CUDA_TRY(cudaDeviceSynchronize());
  CUDA_TRY(cudaMemcpy(out, st->status + kStatusInts, static_cast<size_t>(n) * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaMemset(st->status + kStatusInts, 0, kProfileWords * sizeof(unsigned long long)));
  return B200_OK;
#else
  (void)out;
  (void)n;
  return fail(B200_EUNSUPPORTED, "this build has no wait profiling (compile with -DB200_PROFILE_WAITS)");
#endif
}

const char* b200_kernel_info(void) {
  static char buf[1536];
  using PH = Params<half, half, MMA_T, MMA_N>;
  using PF = Params<float, float, MMA_N, MMA_T>;
  using O64 = OftT<64, 1>;
  using O128 = OftT<128, 1>;
  using R64 = Oft3Traits<64, 2, 5>;
  using R128 = Oft3Traits<128, 2, 5>;
  using S64 = Oft4Traits<64>;
  using S128 = Oft4Traits<128>;
  snprintf(buf, sizeof buf,
           "{\"arch\": \"sm_100a\", \"gemm_half_tn\": {\"bM\": %d, \"bN\": %d, \"bK\": %d, \"bP\": %d}, "
           "\"gemm_float_nt\": {\"bM\": %d, \"bN\": %d, \"bK\": %d, \"bP\": %d}, "
           "\"oft\": {\"ctas\": %d, \"bM\": %d, \"bN\": %d, \"bK\": %d, \"bP1\": %d, \"bP2\": %d, \"threads\": %d, "
           "\"b64\": {\"smem\": %d, \"tmem_cols\": %d, \"xr_bufs\": %d}, "
           "\"b128\": {\"smem\": %d, \"tmem_cols\": %d, \"xr_bufs\": %d}}, "
           "\"oft_ring\": {\"ctas\": 2, \"bM\": 128, \"bN\": 256, \"bK\": 64, \"stages_x_r\": %d, \"stages_xr_w\": %d, \"threads\": %d, "
           "\"accumulators\": 1, \"b64\": {\"smem\": %d, \"rotation_bufs\": %d}, \"b128\": {\"smem\": %d, \"rotation_bufs\": %d}}, "
           "\"oft_ring_split\": {\"ctas\": 2, \"bM\": 128, \"bN\": 256, \"bK\": 64, \"stages_xr_w\": %d, \"threads\": %d, \"accumulators\": %d, "
           "\"rotation_bufs\": %d, \"b64\": {\"smem\": %d, \"stages_x_r\": %d}, \"b128\": {\"smem\": %d, \"stages_x_r\": %d}}}",
           PH::bM, PH::bN, PH::bK, PH::bP, PF::bM, PF::bN, PF::bK, PF::bP, kOftPair ? 2 : 1, (int)CurrCompParams::bM, (int)CurrCompParams::bN,
           (int)CurrCompParams::bK, (int)CurrCompParams::bP1, (int)CurrCompParams::bP2, O64::kThreads, O64::kSmemBytes,
           O64::kTmemUsed, O64::kXrBufs, O128::kSmemBytes, O128::kTmemUsed, O128::kXrBufs, R64::kS1, R64::kS2, R64::kThreads, R64::kSmemBytes,
           R64::kXrBufs, R128::kSmemBytes, R128::kXrBufs, S64::kStages, S64::kThreads, S64::kAccBufs, S64::kXrBufs, S64::kSmemBytes, S64::kS1,
           S128::kSmemBytes, S128::kS1);
  return buf;
}

const char* b200_last_error(void) { return g_err.c_str(); }

int b200_set_option(const char* name, int value) {
  g_err.clear();
  options_init();
  for (int i = 0; name && i < kOptCount; ++i)
    if (std::strcmp(name, kOptionDefs[i].name) == 0) {
      g_opt[i].store(value);
      return B200_OK;
    }
  return fail(B200_EINVAL, "unknown option '%s'", name ? name : "(null)");
}

int b200_get_option(const char* name, int* value) {
  g_err.clear();
  options_init();
  for (int i = 0; name && value && i < kOptCount; ++i)
    if (std::strcmp(name, kOptionDefs[i].name) == 0) {
      *value = g_opt[i].load();
      return B200_OK;
    }
  return fail(B200_EINVAL, "unknown option '%s'", name ? name : "(null)");
}

int b200_shutdown(void) {
  g_err.clear();
  {
    std::lock_guard<std::mutex> lock(g_optin_mu);
    g_optin.clear();
  }
  std::lock_guard<std::mutex> lock(g_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  for (int d = 0; d < kMaxDevices; ++d) {
    DeviceState& st = g_dev[d];
    if (!st.ready) continue;
    cudaSetDevice(d);
    cudaFree(st.status);
    for (int i = 0; i < 4; ++i) cudaFree(st.stage[i]);
    if (st.host_stream) cudaStreamDestroy(st.host_stream);
    if (st.in_stream) cudaStreamDestroy(st.in_stream);
    if (st.out_stream) cudaStreamDestroy(st.out_stream);
    if (st.pool) cudaMemPoolDestroy(st.pool);
    st = DeviceState{};
  }
  cudaSetDevice(cur);
  return B200_OK;
}

int b200_oft_tn_f16_static(int m, int n, int k, int group_size, int reconn_sz, const void* A, int ldA, const void* B, int ldB,
                           const void* R, int ldR, void* C, int ldC, void* stream_v) {
  g_err.clear();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = common_dims(m, n, k, A, B, C)) return rc;
  if (reconn_sz <= 0 || group_size <= 0) return fail(B200_EINVAL, "group_size=%d and reconn_sz=%d must be positive", group_size, reconn_sz);
  if (k % reconn_sz != 0) return fail(B200_EINVAL, "k=%d is not a multiple of reconn_sz=%d", k, reconn_sz);
  if (n % group_size != 0) return fail(B200_EINVAL, "n=%d is not a multiple of group_size=%d", n, group_size);
  if (ldC < n) return fail(B200_EINVAL, "ldC=%d smaller than n=%d (C is row-major)", ldC, n);
  if (m > 0 && n > 0 && k > 0 && !R) return fail(B200_EINVAL, "R is null");
  const size_t need = oft_scratch_bytes(n / group_size, k, reconn_sz);
  if (need > kStaticScratchBytes)
    return fail(B200_EUNSUPPORTED, "this problem needs %zu bytes of device scratch; the static scratch of b200_oft_tn_f16_static holds %zu",
                need, kStaticScratchBytes);
  if (m == 0 || n == 0) return B200_OK;
  if (k == 0) {
    CUDA_TRY(cudaMemset2DAsync(C, static_cast<size_t>(ldC) * 2, 0, static_cast<size_t>(n) * 2, m, stream));
    return B200_OK;
  }
  StaticScratchState* ss;
  if (int rc = static_scratch_state(&ss, stream)) return rc;
  // Every call shares the one array, which still holds what the last call left there.  The record of a
  // bounded wait that ran out (words 0..3) stays until b200_static_status reads it; the round counters
  // that follow are zeroed by the launcher when a launch uses them.
  DeviceState view;  // what the launcher reads: SM count, L2 size and where the kernel's scratch is
  view.sm_count = ss->sm_count;
  view.l2_bytes = ss->l2_bytes;
  view.status = static_cast<int*>(ss->scratch);
  if (reconn_sz == 8) {
    void* rx = static_cast<unsigned char*>(ss->scratch) + kStaticRxOffset;
    if (int rc = expand_r8(R, ldR, rx, n / group_size, k, stream)) return rc;
    return launch_oft<16>(m, n, k, group_size, A, ldA, B, ldB, rx, static_cast<int>(r8_ld(k)), C, ldC, stream, &view);
  }
  switch (reconn_sz) {
    case 16: return launch_oft<16>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, &view);
    case 32: return launch_oft<32>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, &view);
    case 64: return launch_oft<64>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, &view);
    case 128: return launch_oft<128>(m, n, k, group_size, A, ldA, B, ldB, R, ldR, C, ldC, stream, &view);
    default: return fail(B200_EUNSUPPORTED, "reconn_sz=%d not compiled in (8, 16, 32, 64, 128)", reconn_sz);
  }
}

}  // extern "C"

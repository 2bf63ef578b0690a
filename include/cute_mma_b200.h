/*
 * C ABI of the B200 (sm_100a) GEMM / OFT library.  Plain pointers and sizes only.
 *
 * Every entry point returns 0 on success or one of the B200_E* codes; b200_last_error() then
 * describes the failure of the calling thread's last call.  Unless stated otherwise all matrix
 * pointers are caller-owned DEVICE memory, calls are asynchronous on `stream` (a cudaStream_t passed
 * as void*, NULL = default stream) and the library keeps no reference to the buffers after return.
 * Requirements common to all compute calls: base pointers of A, B, R aligned to 16 bytes and
 * leading dimensions whose byte size is a multiple of 16 (they are read through TMA descriptors);
 * C needs only natural alignment.  M, N, K need not be multiples of the tile.
 */
#ifndef CUTE_MMA_B200_H_
#define CUTE_MMA_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200_OK = 0,
  B200_EINVAL = 1,        /* bad pointer, size, alignment or leading dimension */
  B200_EUNSUPPORTED = 2,  /* shape class not compiled into this build (e.g. block edge) */
  B200_ECUDA = 3,         /* a CUDA runtime / driver call failed */
  B200_EDEVICE = 4        /* a kernel reported a bounded wait that ran out (see b200_device_status) */
};

/* Fused OFT product  C[m,n] = (A[m,k] . R) . B^T  with block-diagonal R.
 * Replaces oft_tn<KernelParams> (cute_oft_coop_pc.hpp:17-23, cute_oft_coop_pc.cu:505-577); the
 * reference's compile-time KernelParams::group_size / reconn_sz are the run-time arguments
 * group_size / reconn_sz here (the C++ shim cute_mma_b200/shim/cute_oft_coop_pc.hpp restores the template form).
 *   A [m][k] ldA, B [n][k] ldB (= W^T), R [(n/group_size)*reconn_sz][k] ldR, C [m][n] ldC, all fp16,
 *   all row-major; stored R block (g,kb) = rows g*b.., cols kb*b.. holds the TRANSPOSE of the
 *   mathematical rotation.  fp32 accumulation, X.R rounded to fp16 (RNE) before the main product.
 * reconn_sz in {8, 16, 32, 64, 128}; k % reconn_sz == 0; n % group_size == 0; group_size == n or a
 * multiple of the kernel's N tile (256), or, with reconn_sz <= 64, one half, quarter or eighth of it
 * (the reference's bN % group_size == 0 case, cute_oft_coop_pc.cu:383).  reconn_sz = 8 (the reference's
 * default) first expands R into pairs of 8 x 8 blocks embedded in zero-padded 16 x 16 blocks (device
 * scratch of twice the size of R, stream-ordered on `stream` from a memory pool the library keeps until
 * b200_shutdown) and then runs as 16.
 * The product is fused in one of two ways (b200_oft_plan tells which, the option "oft_route" overrides): a group of
 * fewer than 8 N tiles of 256 columns (4 for reconn_sz = 128) keeps X.R in tensor memory and forms it per N tile, as
 * the reference's kernel forms it per thread block (cute_oft_coop_pc.cu:19-186); a wider group forms one X.R per block
 * of 256 rows and shares it among all its N tiles through a ring of row blocks in device scratch that is sized to
 * stay in L2 (32 to 64 MB and a few counters per call in flight, from the same pool, one launch per N-group).  In the
 * ring kernel every SM pair rotates and multiplies; for very wide groups (three rotating pairs or fewer keep up) a
 * variant gives the rotation to a few SM pairs of its own and runs the plain GEMM's loop on the others.  All give the
 * same numbers; the ring kernels also the same bits as b200_oft_tn_f16_two_pass. */
int b200_oft_tn_f16(int m, int n, int k, int group_size, int reconn_sz,
                    const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                    void* C, int ldC, void* stream);

/* Rotation alone: XR[m][k] (row-major, ld = ldX, fp16) = half(A . blockdiag(R_kb^T)), R = the reconn_sz stored
 * rows of ONE N-group (see b200_oft_tn_f16 for the stored layout), fp32 accumulation, one rounding to fp16.
 * A, R and XR: 16-byte aligned, leading dimensions multiples of 8 elements (TMA tile loads and stores).
 * The first pass of b200_oft_tn_f16_two_pass; replaces the batched cublasHgemmStridedBatched that forms d_AR
 * in the reference's cuBLAS comparator (cublas_oft.hpp:69-81). */
int b200_rotate_f16(int m, int k, int reconn_sz, const void* A, int ldA, const void* R, int ldR,
                    void* XR, int ldX, void* stream);

/* Which route b200_oft_tn_f16 takes for this problem on the current device and how many of the library's
 * kernels one call launches.  *path: 1 fused kernel that keeps X.R in tensor memory and forms it per N tile
 * (narrow groups), 2 rotation pass + GEMM (only when asked for), 3 fused kernel in which one X.R per row block
 * serves all N tiles of its group through a ring of row blocks that stays in L2 (groups of 8 N tiles or more, 4 for
 * reconn_sz = 128), 4 the same ring with the rotation on SM pairs of its own (when at most three such pairs keep
 * up with the product: groups of about 40 N tiles or more, K of 2048 or more).  No counterpart in the reference. */
int b200_oft_plan(int m, int n, int k, int group_size, int reconn_sz, int* path, int* kernel_launches);

/* The same product in two passes: X.R (rounded to fp16, as above) is written once to device scratch of
 * m * k * 2 bytes (stream-ordered on `stream`, from the pool the library keeps until b200_shutdown) and
 * the plain fp16 GEMM runs on it, group by group.  b200_oft_tn_f16 takes this path only when the
 * option "oft_route" is 2 (see b200_set_option); this entry point always does.  Counterpart in the reference: cublas_oft(..., RW_mode = false), the AR_W
 * order with a batched cuBLAS GEMM for X.R and one cublasHgemm per group (cublas_oft.hpp:66-91); its own
 * kernel never lets X.R leave the thread block (cute_oft_coop_pc.cu:19-186). */
int b200_oft_tn_f16_two_pass(int m, int n, int k, int group_size, int reconn_sz,
                             const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                             void* C, int ldC, void* stream);

/* Same product with HOST buffers: copies B and R to the device, then A up, the product and C back in up to
 * 16 row chunks on three streams (upload, product and download of successive chunks overlap), and
 * synchronises before returning.  Pinned host memory is needed for the overlap (pageable memory works, the
 * copies then serialise).  Device staging buffers and streams are owned and reused by the library; calls
 * are serialised.  This is the call the end-to-end figure of bench.py times. */
int b200_oft_tn_f16_host(int m, int n, int k, int group_size, int reconn_sz,
                         const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                         void* C, int ldC);

/* The same fused product for callers that must not allocate device memory.  It has no counterpart in
 * the reference.  Some programs hand all of a GPU's memory to their own pool when they start, so a later
 * cudaMalloc fails; others run this call on a path where the device-wide synchronisation that cudaMalloc
 * implies is not acceptable.  b200_oft_tn_f16 creates a small per-device workspace with cudaMalloc the
 * first time it runs on a device; this entry point calls no cudaMalloc, no cudaFree and no allocating
 * library routine, ever.  The device scratch its kernel needs beyond A, B, R and C lives in a 64 KB array
 * inside the library image, which every GPU that loads the library keeps until the process exits: the first
 * 256 bytes hold the record in which a kernel reports a bounded wait that ran out and the counters of the
 * tile-round lock (36 KB in -DB200_PROFILE_WAITS builds, which add their profiling words); for
 * reconn_sz = 8 the expanded copy of R follows, 32 * (n / group_size) * k bytes, so 8 x 8 blocks are served
 * up to (n / group_size) * k <= 2040.  A problem whose scratch need exceeds the 64 KB is refused with
 * B200_EUNSUPPORTED and a message naming both sizes.
 *   - Arguments, layouts and result are exactly those of b200_oft_tn_f16 on its route 1 (the kernel that
 *     keeps X.R in tensor memory, which needs no scratch for X.R): same bits as b200_oft_tn_f16 with the
 *     option "oft_route" set to 1.
 *   - The first call on each device looks up the array's device address, reads three device attributes
 *     and zeroes the record with a cudaMemsetAsync on the caller's stream; make that first call, with the
 *     device current, before any stream capture begins.  Later calls only enqueue work on `stream`.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left in it.
 *     Two calls whose kernels overlap on the GPU (different streams, no dependency) race on it.
 *     Serialise them.
 *   - A bounded wait that ran out is reported by b200_static_status (below), which reads this array;
 *     b200_device_status reports the allocated workspace, not this array.  The record stays until read. */
int b200_oft_tn_f16_static(int m, int n, int k, int group_size, int reconn_sz,
                           const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                           void* C, int ldC, void* stream);

/* The other algebraic order of the same product, Y = X . (R . W)  ("A_RW", cublas_oft.hpp:20-65).
 * b200_transform_weight_f16 replaces transform_weight (cublas_oft.hpp:20-43): it folds the rotation into the
 * weight,  Bt[g*gs+j][kb*b+p] = half(sum_q R[g*b+q][kb*b+p] * B[g*gs+j][kb*b+q])  (fp32 accumulate), Bt [n][k]
 * ldBt, any reconn_sz <= 128 that divides k.  b200_oft_tn_f16_a_rw does the transform into stream-ordered
 * scratch and then one plain GEMM (cublas_oft.hpp:58-65); callers that reuse a weight transform it once and
 * call b200_gemm_tn_f16(n, m, k, Bt, ldBt, A, ldA, C, ldC) themselves.  The result differs from
 * b200_oft_tn_f16 only by rounding (R.W is rounded to fp16 instead of X.R). */
int b200_transform_weight_f16(int n, int k, int group_size, int reconn_sz, const void* B, int ldB,
                              const void* R, int ldR, void* Bt, int ldBt, void* stream);
int b200_oft_tn_f16_a_rw(int m, int n, int k, int group_size, int reconn_sz,
                         const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                         void* C, int ldC, void* stream);

/* Plain GEMM  C(i,j) = sum_l A(i,l) B(j,l),  C column-major: C(i,j) at C[i + j*ldC].
 * Replace gemm_tn / gemm_nt<TO,TR> (gemm_sm80_tc.cu:163-228 / 95-160).
 *   tn: A(i,l) at A[i*ldA + l], B(j,l) at B[j*ldB + l]   (both K-contiguous)
 *   nt: A(i,l) at A[i + l*ldA], B(j,l) at B[j + l*ldB]   (M- / N-contiguous)
 * f16: fp16 in, fp32 accumulate, fp16 out.  tf32: fp32 in consumed as TF32 by the tensor cores
 * (low 13 mantissa bits ignored), fp32 accumulate and out. */
int b200_gemm_tn_f16(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream);
int b200_gemm_nt_f16(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream);
int b200_gemm_tn_tf32(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream);
int b200_gemm_nt_tf32(int m, int n, int k, const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream);

/* C = A . B^T + A2 . B2^T in one pass (tn layouts, fp16, C column-major): the K steps of the second operand pair
 * (k2 columns) follow those of the first in every tile's accumulation.  CTA-pair build only.  No counterpart
 * in the reference, whose accumulate-into-C epilogue is stubbed out (axpby, gemm_tc.hpp:241). */
int b200_gemm_tn_f16_acc2(int m, int n, int k, const void* A, int ldA, const void* B, int ldB,
                          int k2, const void* A2, int ldA2, const void* B2, int ldB2, void* C, int ldC, void* stream);

/* LoRA-equivalent product, the comparator of playgrounds/lora.cu:33-64 (three cublasHgemm calls there):
 *   C[m][n] (row-major, ldC) = X . W^T + (X . L1^T) . L2^T,   X [m][k], W [n][k], L1 [r][k], L2 [n][r], all fp16,
 * as one small GEMM for T = X . L1^T (rounded to fp16, m * r * 2 bytes of stream-ordered scratch from the
 * library's pool) and one b200_gemm_tn_f16_acc2 over (W, X) and (L2, T) with fp32 accumulation of both terms. */
int b200_lora_tn_f16(int m, int n, int k, int r, const void* X, int ldX, const void* W, int ldW,
                     const void* L1, int ldL1, const void* L2, int ldL2, void* C, int ldC, void* stream);

/* Dispatcher of gemm(char transA, char transB, ...) (gemm_sm80_tc.cu:393-418): ('T','N') -> tn,
 * ('N','T') -> nt; lower-case letters select the same kernels (the reference's *_test variants are
 * an alternative shared-memory path of the same operator).  is_float: 0 = half/half, 1 = float/float. */
int b200_gemm(char transA, char transB, int is_float, int m, int n, int k,
              const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream);

/* The epilogue variants the reference leaves out: C = alpha * A.B^T + beta * C (its axpby is a commented-out stub,
 * gemm_tc.hpp:241; its kernels store the bare product), and a float result from half operands (the fp32
 * accumulator stored unrounded).  in_type / out_type: B200_F16 -> B200_F16, B200_F16 -> B200_F32,
 * B200_TF32 -> B200_F32 (float operands multiplied as TF32).  Layouts and transA / transB as in b200_gemm,
 * C column-major.  beta != 0 reads C, which then must hold valid numbers; (alpha, beta) = (1, 0) returns the bits
 * of b200_gemm.  Products scaled this way are never split along K. */
#define B200_F16 0
#define B200_F32 1
#define B200_TF32 2
int b200_gemm_ex(char transA, char transB, int in_type, int out_type, int m, int n, int k, float alpha,
                 const void* A, int ldA, const void* B, int ldB, float beta, void* C, int ldC, void* stream);

/* The same products with C row-major: C(i,j) at C[i*ldC + j], ldC >= n.  The reference's kernels only write
 * column-major C (gemm_tc.hpp:12-14); the rotation + GEMM route of the OFT product uses this form internally. */
int b200_gemm_rowmajor(char transA, char transB, int is_float, int m, int n, int k,
                       const void* A, int ldA, const void* B, int ldB, void* C, int ldC, void* stream);

/* Device-to-device copy between two GPUs of this process' view (dst may be memory of another process mapped
 * through CUDA IPC), asynchronous on `stream` of the current device: a copy-engine transfer over NVLink, with
 * peer access enabled on first use.  Used by the overlapped all-gather of Y; no counterpart in the reference. */
int b200_peer_copy_async(void* dst, int dst_device, const void* src, int src_device, size_t bytes, void* stream);

/* Column range [n_begin, n_end) of B (rows of the stored [n][k] matrix) and of C owned by `rank` when
 * the product is sharded along N over `world` GPUs, A and R replicated.  The reference has no
 * multi-GPU path; the partition follows its group structure (cpu_oft.hpp:52-93: columns of one
 * N-group share an R, so slabs never split a group; with a single group they are cut on 256-column
 * tiles).  Pure host arithmetic, no CUDA call. */
int b200_shard_range(int n, int group_size, int world, int rank, int* n_begin, int* n_end);

/* The N-sharded product on `world` GPUs of this process, one call: for r = 0 .. world-1 the slab of
 * b200_shard_range(n, group_size, world, r) is launched on device devices[r] (asynchronously, on streams[r] or
 * that device's default stream when streams is NULL) through b200_oft_tn_f16, and the calling thread's current
 * device is restored.  Per device r the caller supplies, in that device's memory: A[r] = all of X (replicated),
 * B_slab[r] = rows [n0, n1) of the stored B, R_slab[r] = the stored R rows of the slab's groups (all of R when
 * group_size == n), C_slab[r] = where column n0 of C goes (a private [m][n1-n0] buffer with ldC = n1 - n0, or
 * column n0 of a full C with ldC = n).  No collective and no peer access are involved: the product shards with no
 * exchange; gathering C is left to the caller (NCCL, or b200_peer_copy_async).  The same device may appear more
 * than once (its slabs then run one after the other).  The reference is single-GPU (cute_oft_pc.cu:257-264). */
int b200_oft_tn_f16_sharded(int m, int n, int k, int group_size, int reconn_sz, int world, const int* devices,
                            const void* const* A, int ldA, const void* const* B_slab, int ldB,
                            const void* const* R_slab, int ldR, void* const* C_slab, int ldC, void* const* streams);

/* The product with its result stored to n_dst (1..8) buffers at once: C_dst[d][i*ldC + j] for every d, all with the
 * same ldC.  On the route that shares X.R through L2 the epilogue of the kernel writes every tile to each destination
 * with ordinary global stores, so a destination may be another GPU's memory mapped into this process (peer access or
 * a shared allocation): with C_dst[d] = column n0 of GPU d's full Y[m][N] and ldC = N, every GPU of a node ends up
 * with all of Y without a separate all-gather (the direct peer-store epilogue; no TMA and no multicast touch peer
 * memory; with an even ldC the further destinations are written in whole 128-byte lines).  Other routes compute into C_dst[0] and copy.  The caller synchronises the GPUs before reading (the
 * stores of a peer are complete when that peer's stream is).  No counterpart in the reference, which is single-GPU. */
int b200_oft_tn_f16_gather(int m, int n, int k, int group_size, int reconn_sz,
                           const void* A, int ldA, const void* B, int ldB, const void* R, int ldR,
                           int n_dst, void* const* C_dst, int ldC, void* stream);

/* Tile visiting order of the persistent kernels; same order as z_curve(grid, idx) (z_curve.hpp:28-49). */
int b200_tile_coord(unsigned tiles_m, unsigned tiles_n, unsigned idx, unsigned* tile_m, unsigned* tile_n);

/* Synchronises the current device and reads the kernels' status record:
 * out[0] = 0 ok / 1 a bounded wait ran out, out[1] = CTA, out[2] = wait site, out[3] = parity.
 * Clears the record.  Returns B200_EDEVICE when out[0] != 0. */
int b200_device_status(int out[4]);

/* The same for the array of b200_oft_tn_f16_static: synchronises the current device, copies the four
 * words out of the array with cudaMemcpy and clears them if set.  Allocates nothing.  No counterpart in
 * the reference. */
int b200_static_status(int out[4]);

/* Exercises the kernels' failure path without any fault: a one-thread kernel waits, with a limit of
 * limit_us microseconds (1..100000), on a barrier nothing arrives on; the wait gives up, records
 * {1, CTA 0, site 99, parity 0} and the kernel returns.  Returns B200_OK when exactly that was
 * observed (out receives the record) and leaves the status record cleared.  The reference has no
 * failure detection (errors surface as cudaErrors at the next synchronisation). */
int b200_selftest_wait_timeout(unsigned limit_us, int out[4]);

/* In-kernel stage timers (the reference has no tracing beyond cudaEvent timing, cute_oft_pc.cu:372-377).
 * A library built with -DB200_PROFILE_WAITS adds, per wait site of the kernels' mbarrier protocol,
 * the cycles spent waiting (out[site]) and the number of waits (out[64 + site]); this call
 * synchronises the device, copies up to n counters and clears them (n <= 128; larger n also
 * returns a 32-unit x 8-event clock trace of CTA 0 and tile-end times of the first CTAs, used when
 * tuning the OFT hand-off and the tile order).  Ordinary builds return
 * B200_EUNSUPPORTED. */
int b200_wait_profile(unsigned long long* out, int n);

/* Compile-time configuration of this build as a short JSON string (tile sizes, ring depths). */
const char* b200_kernel_info(void);

/* Overrides of the launch heuristics, for experiments and tests (the reference fixes such choices at compile
 * time).  Names: "oft_route" (0 choose, 1 / 2 / 3 / 4 as in b200_oft_plan), "raster" (0 z-curve, g > 0 bands of g
 * tile rows), "tile_sync", "gemm_tile_sync" (cross-CTA phase lock off / on), "l2_hints", "gemm_l2_hints"
 * (10 * a + b with 0 normal, 1 evict-first, 2 evict-last for the A / B tile loads), "gemm_split" (0: never
 * split small problems along K), "maps_3d" (0: per-chunk 2-D copies of MN-major tiles), "ring_bands" (bands of row
 * blocks the X.R ring of routes 3 and 4 holds, >= 2), "prefetch" (route 3: K steps by which W tiles are asked into
 * L2 ahead of their load), "rot_pairs" (route 4: SM pairs that only rotate, >= 1).  -1 (0 for the route)
 * hands the choice back to the library.  Process-wide; the B200_* environment variables of the same meaning
 * (B200_OFT_PATH, B200_RASTER, B200_TILE_SYNC, B200_L2_HINTS, B200_GEMM_TILE_SYNC, B200_GEMM_L2_HINTS,
 * B200_GEMM_SPLIT, B200_MAPS_3D, B200_RING_BANDS, B200_PREFETCH, B200_ROT_PAIRS) are read once, at the first use of
 * any option, as initial values. */
int b200_set_option(const char* name, int value);
int b200_get_option(const char* name, int* value);

/* Text of the calling thread's last error ("" if none). */
const char* b200_last_error(void);

/* Frees the per-device workspaces and staging buffers. */
int b200_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* CUTE_MMA_B200_H_ */

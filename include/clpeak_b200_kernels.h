/* clpeak_b200 kernel shim -- the C ABI between clpeak's C++ host code and the
 * sm_100a kernels.
 *
 * In the reference project the CUDA backend reaches its kernels through three
 * pieces: fatbin blobs embedded in the binary (cuda_kernels::Blob,
 * include/cuda/cuda_peak.h:214-248), CudaDevice::getKernel, which loads a blob
 * with cuModuleLoadData (src/cuda/cuda_device.cpp:140-173), and
 * cuLaunchKernel inside CudaPeak::runKernel (src/cuda/cuda_peak.cpp:64-107).
 * This header replaces that trio: one plain C function per kernel, POD
 * arguments and a stream, an int status back.  Each entry point names the
 * reference kernel or host routine whose job it takes over.
 *
 * Conventions
 *  - Every function returns CLPK_OK (0) or a CLPK_ERR_* code; clpk_last_error()
 *    gives a thread-local human-readable detail string.  No C++ exceptions
 *    cross this boundary.
 *  - Pointers named d_* are device pointers of the current device, h_* are
 *    host pointers.  Buffers are allocated and freed by the caller
 *    (clpk_malloc/clpk_free or any other CUDA allocator in the same context).
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *    stream).  Calls are asynchronous unless stated otherwise.
 *  - Callable from any host thread that has made the target device current
 *    (clpk_set_device).  No global state except per-device lazily created
 *    handles.
 *  - There is no CPU fallback: on a machine without an sm_100 GPU every
 *    compute entry point fails with CLPK_ERR_NO_DEVICE / CLPK_ERR_UNSUPPORTED.
 */
#ifndef CLPEAK_B200_KERNELS_H
#define CLPEAK_B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32)
#define CLPK_API __declspec(dllexport)
#else
#define CLPK_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define CLPK_OK               0
#define CLPK_ERR_CUDA         1   /* a CUDA runtime/driver call failed            */
#define CLPK_ERR_BAD_ARG      2   /* size/alignment/enum rejected before launch   */
#define CLPK_ERR_TIMEOUT      3   /* a bounded device-side wait expired           */
#define CLPK_ERR_UNSUPPORTED  4   /* device is not compute capability 10.x        */
#define CLPK_ERR_NO_DEVICE    5   /* no CUDA device / driver                      */
#define CLPK_ERR_TOO_LARGE    6   /* request exceeds a documented fixed capacity  */

CLPK_API const char *clpk_last_error(void);
CLPK_API const char *clpk_version(void);

/* ---- device / memory / stream plumbing ------------------------------------
 * Replaces CudaDevice::init and the cuMemAlloc / cuMemcpy / cuEvent calls
 * scattered through src/cuda/ (cuda_device.cpp:40-120, cuda_peak.cpp:69-83). */
typedef struct clpk_device_info {
    char     name[256];
    int      cc_major, cc_minor;
    int      num_sms;
    uint64_t total_mem_bytes;
    int      driver_version;      /* e.g. 12090 */
    int      runtime_version;
    int      sm_clock_khz;        /* max */
    int      mem_clock_khz;       /* max */
    int      mem_bus_bits;
    int      l2_bytes;
    int      smem_optin_bytes;    /* max dynamic shared memory per block */
} clpk_device_info_t;

CLPK_API int clpk_device_count(int *count);
CLPK_API int clpk_device_info(int device, clpk_device_info_t *out);
CLPK_API int clpk_set_device(int device);
CLPK_API int clpk_malloc(void **d_ptr, size_t bytes);
CLPK_API int clpk_free(void *d_ptr);
CLPK_API int clpk_malloc_host(void **h_ptr, size_t bytes);      /* pinned */
CLPK_API int clpk_free_host(void *h_ptr);
CLPK_API int clpk_memset(void *d_ptr, int byte, size_t bytes, void *stream);
CLPK_API int clpk_memcpy_h2d(void *d_dst, const void *h_src, size_t bytes, void *stream);
CLPK_API int clpk_memcpy_d2h(void *h_dst, const void *d_src, size_t bytes, void *stream);
CLPK_API int clpk_memcpy_d2d(void *d_dst, const void *d_src, size_t bytes, void *stream);
CLPK_API int clpk_stream_create(void **stream);                 /* non-blocking */
CLPK_API int clpk_stream_destroy(void *stream);
CLPK_API int clpk_stream_sync(void *stream);
CLPK_API int clpk_event_create(void **event);
CLPK_API int clpk_event_destroy(void *event);
CLPK_API int clpk_event_record(void *event, void *stream);
CLPK_API int clpk_event_sync(void *event);
CLPK_API int clpk_event_elapsed_ms(void *start, void *stop, float *ms);
/* Writes `bytes` (rounded down to 16) of a throw-away buffer so that the L2
 * holds none of the previous kernel's data.  d_scratch must hold `bytes`. */
CLPK_API int clpk_flush_l2(void *d_scratch, size_t bytes, void *stream);

/* ---- tuning knobs ---------------------------------------------------------------------------
 * Scheduling choices that do not change any result.  Each knob's default is what measured
 * fastest; the environment variable of the same name (CLPK_GEMM_NO_ALIGN, ...) is read ONCE,
 * at the first use of any knob in the process, and replaces the default; clpk_set_tuning
 * replaces both from then on (value < 0: back to "not set").  clpk_get_tuning returns -1 for
 * a knob that is not set.  No reference counterpart (cuBLASLt picks its own schedule).
 *   GEMM_NO_ALIGN  1 = the producers of the persistent GEMM do not meet once per wave
 *   GEMM_ALIGN_AT  k block at which they meet (default 2)
 *   GEMM_GROUP     raster group width in tile columns (default 12 dense, 8 block-scaled)
 *   MMA_PAIR       peak probes as CTA pairs (1) or lone CTAs (0); default per kind
 *   GEMM_FP4_TILE  block-scaled GEMM tile: 0 = by size, 1 = 256x256 one accumulator,
 *                  2 = 256x128 two accumulators (the epilogue overlaps the next tile)
 *   MMA_LONE_LANE  1 = the peak probes issue from one thread instead of an elected lane of a whole warp
 *   GEMM_NO_PDL    1 = GEMMs too small for the per-wave alignment are launched plainly; by default they carry
 *                  the programmatic-serialisation attribute, so that a launch's set-up overlaps the tail of
 *                  the kernel before it in the stream (it waits for that kernel before touching memory) */
#define CLPK_TUNE_GEMM_NO_ALIGN 0
#define CLPK_TUNE_GEMM_ALIGN_AT 1
#define CLPK_TUNE_GEMM_GROUP    2
#define CLPK_TUNE_MMA_PAIR      3
#define CLPK_TUNE_GEMM_FP4_TILE 4
#define CLPK_TUNE_MMA_LONE_LANE 5   /* 1 = the peak probes issue from one thread instead of an elected lane of a whole warp */
#define CLPK_TUNE_GEMM_NO_PDL   6   /* 1 = small GEMMs are launched without programmatic stream serialisation */
#define CLPK_TUNE_COUNT         7
CLPK_API int clpk_set_tuning(int knob, int value);
CLPK_API int clpk_get_tuning(int knob, int *value);

/* ---- seeded operand generation ----------------------------------------------
 * Replaces populate() (src/common/common.cpp:76-95, a sequential xorshift32
 * fill on the host) with counter-based device fills: element i of stream
 * `seed` is a pure function of (seed, i); see clpk_rng.h for the definition. */
#define CLPK_DIST_UNIFORM01   0   /* [0,1)               */
#define CLPK_DIST_UNIFORM_PM1 1   /* [-1,1)              */
#define CLPK_DIST_NORMAL      2   /* mean + std * N(0,1) */
CLPK_API int clpk_fill_f32(float *d_dst, uint64_t n, uint64_t seed, int dist,
                           float mean, float std, void *stream);
/* int8 uniform in [-8,7]. */
CLPK_API int clpk_fill_i8(int8_t *d_dst, uint64_t n, uint64_t seed, void *stream);

/* Element formats for conversion, tensor-core peak tests and GEMM. */
#define CLPK_DT_F32   0
#define CLPK_DT_F16   1
#define CLPK_DT_BF16  2
#define CLPK_DT_E4M3  3
#define CLPK_DT_E5M2  4
#define CLPK_DT_I8    5
#define CLPK_DT_MXF4  6   /* e2m1 pairs + one ue8m0 scale per 32 elements            */
#define CLPK_DT_NVF4  7   /* e2m1 pairs + one ue4m3 scale per 16 elements + fp32 scale */
#define CLPK_DT_MXF4_B64 8   /* as MXF4 with one ue8m0 scale per 64: the dense B operand of MXF4_SP */
#define CLPK_DT_NVF4_B32 9   /* as NVF4 with one ue4m3 scale per 32: the dense B operand of NVF4_SP */
#define CLPK_DT_TF32  10  /* fp32 word rounded (nearest even) to 10 mantissa bits, low 13 bits clear       */
#define CLPK_DT_E2M1  11  /* plain e2m1, two per byte (element 2i in the low nibble), saturating at +-6   */
#define CLPK_DT_F64   12  /* double; clpk_convert_f32 widens exactly                                      */

/* Round-to-nearest-even conversion of n floats to a plain (unscaled) format:
 * F16, BF16, E4M3 / E5M2 (saturating to the largest finite value), I8
 * (round-to-nearest-even, saturating), TF32 (a 4-byte word per element) and E2M1
 * (two per byte; n must be even). */
CLPK_API int clpk_convert_f32(void *d_dst, const float *d_src, uint64_t n, int dtype, void *stream);

/* max |x| over n floats -> *d_absmax (a float the call overwrites). */
CLPK_API int clpk_absmax_f32(float *d_absmax, const float *d_src, uint64_t n, void *stream);

/* Block-scaled FP4 quantisation of a row-major [rows][cols] float matrix
 * (cols a multiple of 64; blocks run along a row).
 *   d_packed : rows*cols/2 bytes, element 2j in the low nibble of byte j
 *   d_scales : one byte per block, row-major [rows][cols/block]
 *              (block = 32, ue8m0 for MXF4; block = 16, ue4m3 for NVF4; the _B64 / _B32
 *              variants use the doubled block of the sparse kinds' dense operand)
 *   tensor_scale : NVF4 kinds only; values are divided by it before the block scale
 *              is chosen.  Pass absmax/(6*448) for the usual recipe, 1.0f for MXF4. */
CLPK_API int clpk_quantize_fp4(uint8_t *d_packed, uint8_t *d_scales, const float *d_src,
                               uint64_t rows, uint64_t cols, int dtype, float tensor_scale,
                               void *stream);

/* ---- global-memory bandwidth ------------------------------------------------------
 * clpk_global_bandwidth: the reference's read-and-sum test, same per-thread
 * order (global_bandwidth_v{1,2,4}, src/cuda/cuda_kernels/global_bandwidth.cu:14-71;
 * host side src/cuda/global_bandwidth.cpp:6-92) with 64-bit indexing.
 * `width` is 1, 2 or 4 floats per fetch; n_floats must be a multiple of
 * 256*16*width.  d_out receives n_floats/(16*width) sums. */
CLPK_API int clpk_global_bandwidth(int width, const float *d_in, float *d_out,
                                   uint64_t n_floats, void *stream);

/* STREAM-style kernels over large buffers; definitions follow the reference's
 * CPU backend (read / copy / triad with s = 1.5f, src/cpu/bandwidth.cpp:325-352)
 * -- its CUDA backend has read only.  `variant`:
 *   CLPK_STREAM_LDG : 128-bit loads/stores from registers
 *   CLPK_STREAM_TMA : cp.async.bulk global->shared->global staging
 *   CLPK_STREAM_WIDE: 256-bit loads/stores, one 8 KiB tile per CTA (pointers 32-byte
 *                     aligned); the read flavour XORs into 4096 partial words
 * n_bytes must be a multiple of 16.
 * read  : d_partials[grid] receives per-CTA XOR of all 32-bit words read
 *         (clpk_stream_read_grid() gives the grid size to allocate for).
 * copy  : dst = src.           triad : a = b + s*c (no FMA contraction). */
#define CLPK_STREAM_LDG 0
#define CLPK_STREAM_TMA 1
#define CLPK_STREAM_WIDE 2
CLPK_API int clpk_stream_read_grid(int variant, int *grid);
CLPK_API int clpk_stream_read(int variant, const void *d_src, uint64_t n_bytes,
                              uint32_t *d_partials, void *stream);
CLPK_API int clpk_stream_copy(int variant, void *d_dst, const void *d_src, uint64_t n_bytes,
                              void *stream);
CLPK_API int clpk_stream_triad(int variant, float *d_a, const float *d_b, const float *d_c,
                               float s, uint64_t n_floats, void *stream);
/* The TMA variants bound every device-side wait; a wait that expired is
 * recorded in a per-device status word.  This call synchronises the stream,
 * returns CLPK_ERR_TIMEOUT (and clears the word) if one did, and stores the
 * raw code in *h_status. */
CLPK_API int clpk_stream_status(uint32_t *h_status, void *stream);

/* clpk_stream_checksum_static: no counterpart in the reference.  The same
 * streaming read as clpk_stream_read(CLPK_STREAM_LDG), for callers that must
 * not allocate device memory when they need the checksum (inside a region where
 * cudaMalloc's implicit synchronisation is unacceptable, in a host that forbids
 * allocator calls after start-up, or with the memory pool fully handed out):
 * the per-CTA partials live in a fixed array inside the library's device image
 * instead of a caller buffer, and *d_xor_out (one device word supplied by the
 * caller) receives the XOR of every 32-bit word of the source.
 *  - Capacity: partials for at most 4096 CTAs (16.25 KiB held on every GPU that
 *    loads the library, until the process exits).  grid_ctas = 0 picks
 *    4 x SM count; a larger request fails with CLPK_ERR_TOO_LARGE.
 *  - Calls no cudaMalloc / cudaFree and no allocating library routine.  The first
 *    call on a device resolves the array's device address
 *    (cudaGetSymbolAddress); make that first call before any stream capture.
 *  - All calls on one device share the array: calls that overlap on the GPU
 *    race; serialise them. */
CLPK_API int clpk_stream_checksum_static(const void *d_src, uint64_t n_bytes, uint32_t grid_ctas,
                                         uint32_t *d_xor_out, void *stream);

/* ---- fp32 multiply-add chains ----------------------------------------------------------
 * clpk_compute_sp: the reference chain x = fma(x,x,c), c = threadIdx.x,
 * 128 x 16 FMAs (compute_sp, src/cuda/cuda_kernels/compute_sp.cu:12-24).
 * grid blocks of 256 threads; d_out holds grid*256 floats. */
CLPK_API int clpk_compute_sp(float *d_out, float a, uint32_t grid, void *stream);
/* clpk_mad_chain: work-item i holds a float4 seeded uniform[-1,1) from
 * (seed, 4i..4i+3) and runs `iters` steps of x = fma(x, y, x) per lane;
 * d_out[i] = ((x0 + x1) + x2) + x3.  n_items must be a multiple of 256. */
CLPK_API int clpk_mad_chain(float *d_out, uint64_t n_items, uint64_t seed, float y,
                            uint32_t iters, void *stream);

/* clpk_compute_chain: the shader-core chains of the other element types, with the
 * arithmetic of the reference kernels compute_hp / compute_hp2 / compute_dp /
 * compute_mp / compute_bf16 / compute_int32 / compute_int8_dp{,2,4,8}
 * (src/cuda/cuda_kernels/compute_*.cu): recurrence x = x*x + c with c = threadIdx.x,
 * started from `a` (1.3 for the floating chains, 3 for int32, 4 for the dot
 * products in the reference's host code, src/cuda/compute_float.cpp:30-125,
 * src/cuda/compute_int.cpp:10-64).  grid blocks of 256 threads; d_out holds
 * grid*256 elements of clpk_compute_chain_info()'s size (float for the floating
 * chains except DOUBLE, int32 for the integer ones). */
#define CLPK_CHAIN_HALF       0   /* two scalar fp16 chains of 1024 FMAs, out = float(x0 + x1)       */
#define CLPK_CHAIN_HALF2      1   /* 1024 packed half2 FMAs, out = float(lo) + float(hi)            */
#define CLPK_CHAIN_DOUBLE     2   /* 2048 fp64 FMAs                                                 */
#define CLPK_CHAIN_MIXED      3   /* 2048 fp32 FMAs, value rounded through fp16 every 16            */
#define CLPK_CHAIN_BF16       4   /* 2048 fp32 FMAs, value rounded through bf16 every 128           */
#define CLPK_CHAIN_INT32      5   /* 2048 wrapping 32-bit multiply-adds                             */
#define CLPK_CHAIN_INT8_DOT1  6   /* 1024 dp4a steps (a = dp4a(x, y, a); y ^= a) in 1 chain         */
#define CLPK_CHAIN_INT8_DOT2  7   /* ... split over 2 independent chains                            */
#define CLPK_CHAIN_INT8_DOT4  8   /* ... 4 chains                                                   */
#define CLPK_CHAIN_INT8_DOT8  9   /* ... 8 chains                                                   */
#define CLPK_CHAIN_COUNT      10
CLPK_API int clpk_compute_chain(int chain, void *d_out, double a, uint32_t grid, void *stream);
/* Operations counted per thread (4096; 8192 for the dot products: COMPUTE_FP_WORK_PER_WI,
 * COMPUTE_INT8_DP_WORK_PER_WI, include/common/common.h:100,114) and bytes per output element. */
CLPK_API int clpk_compute_chain_info(int chain, uint32_t *ops_per_thread, uint32_t *out_elem_bytes);

/* ---- shared-memory and texture bandwidth ---------------------------------------------------
 * clpk_local_bandwidth: 64 rounds of "store my value to shared memory, barrier, load
 * my neighbour's, barrier" on `width` (1, 2, 4) floats per thread
 * (local_bandwidth_v1/v2/v4, src/cuda/cuda_kernels/local_bandwidth.cu).  grid blocks
 * of 256 threads; d_out[gid] = sum of the lanes the thread ends with, which are
 * (float)(g + l), l < width, for g = block*256 + (thread + 64) % 256.
 * Bytes per launch: 64 * 2 * width * 4 * grid * 256 (src/cuda/local_bandwidth.cpp). */
CLPK_API int clpk_local_bandwidth(int width, float *d_out, uint32_t grid, void *stream);
/* A width x height image of float4 texels in a CUDA array behind a point-sampled texture
 * object (src/cuda/image_bandwidth.cpp builds the same from populate()); texel (x, y)
 * channel ch = clpk uniform[0,1) number 4*(y*width + x) + ch of `seed`.  Allocates; the
 * call synchronises the stream. */
CLPK_API int clpk_image_create(void **image, uint32_t width, uint32_t height, uint64_t seed, void *stream);
/* 16 float4 fetches per thread, fetch i at texel (gid + i*grid*256) mod (width*height),
 * channel-wise running sums then x+y+z+w (image_bandwidth,
 * src/cuda/cuda_kernels/image_bandwidth.cu).  d_out holds grid*256 floats.  Bytes per
 * launch: 16 * 16 * grid * 256. */
CLPK_API int clpk_image_bandwidth(void *image, float *d_out, uint32_t grid, void *stream);
/* The same work in an order that suits the texture path: a warp reads a 4 x 8 patch of
 * texels, a block an 8 x 32 tile, and fetch i of block b is tile (16 b + i) mod tiles, tiles
 * numbered along x.  Thread t of the block sits at (x, y) = (4 (w % 2) + l % 4, 8 (w / 2) + l / 4)
 * inside the tile, w = t / 32, l = t % 32.  Same per-thread sum as clpk_image_bandwidth.  The
 * image's width must be a multiple of 8 and its height a multiple of 32.  (Additive row: the
 * reference has only the strided order, src/cuda/cuda_kernels/image_bandwidth.cu:9-25.) */
CLPK_API int clpk_image_bandwidth_tiled(void *image, float *d_out, uint32_t grid, void *stream);
CLPK_API int clpk_image_destroy(void *image);

/* ---- latency -------------------------------------------------------------------------------
 * clpk_pointer_chase: one thread follows next[] for `hops` dependent loads
 * starting at `start` (the CUDA backend has no such test; the model is
 * chaseLatencyNs, src/cpu/latency.cpp:42-87).  d_result[0] = final index,
 * d_result[1] = XOR of all indices visited, d_result[2..3] = elapsed
 * %globaltimer nanoseconds (low, high word). */
CLPK_API int clpk_pointer_chase(const uint32_t *d_next, uint32_t start, uint64_t hops,
                                uint32_t *d_result, void *stream);
/* Host-side construction of the chase cycle (Sattolo shuffle of 0..n-1 with a
 * seeded generator, then next[order[i]] = order[i+1]); h_next holds n entries. */
CLPK_API int clpk_build_chase_cycle(uint32_t *h_next, uint64_t n, uint64_t seed);
/* clpk_launch_noop: one empty 1x1 kernel (kernel_latency_noop,
 * src/cuda/cuda_kernels/kernel_latency.cu:5-7).
 * clpk_launch_latency: `iters` x (launch + stream synchronise), each timed on
 * the host clock, after `warmup` untimed rounds; *mean_us is the mean
 * (src/cuda/kernel_latency.cpp:44-75).  Synchronous. */
CLPK_API int clpk_launch_noop(void *stream);
CLPK_API int clpk_launch_latency(uint32_t iters, uint32_t warmup, double *mean_us, void *stream);
/* `nodes` empty kernels captured once as a CUDA graph, replayed `iters` times (launch +
 * synchronise each); the mean per kernel node.  A NULL stream gets a stream of the call's own. */
CLPK_API int clpk_graph_launch_latency(uint32_t nodes, uint32_t iters, uint32_t warmup, double *mean_us_per_node,
                                       void *stream);

/* ---- tensor-core peak (tcgen05.mma, accumulator in tensor memory) ------------------------------
 * Takes over the sixteen wmma / mma.sync probes filled in by CudaPeak::runWmma
 * (src/cuda/wmma.cpp:10-425, kernels src/cuda/cuda_kernels/wmma_*.cu).  Each
 * CTA stages one A tile [128][K] and one B tile [256][K] (both K-contiguous,
 * row-major in global memory) in shared memory and issues `n_mma`
 * tcgen05.mma instructions of shape 128x256xK that accumulate into one
 * 128x256 tile in tensor memory.
 *   kind   K    A/B element        D
 *   F16    16   fp16               f32      BF16  16  bf16  f32
 *   E4M3   32   fp8 e4m3           f32      E5M2  32  e5m2  f32
 *   I8     32   int8               s32
 *   TF32    8   fp32 word, 10-bit mantissa   f32
 *   F16_F16 16  fp16               f16 (one half per 32-bit output word, bits 0..15)
 *   E2M1   32   e2m1 x2 per byte   f32   unscaled 4-bit operands of kind::f8f6f4; 16 bytes per row
 *   MXF4   64   e2m1 x2 per byte   f32   + ue8m0 scale per 32 (d_sfa [128][2], d_sfb [256][2])
 *   NVF4   64   e2m1 x2 per byte   f32   + ue4m3 scale per 16 (d_sfa [128][4], d_sfb [256][4])
 *   E4M3_SP / I8_SP   K = 64 logical, 2:4 sparse A: d_a is the compressed tile
 *          [128][32] (the two kept elements of every group of four, in K order),
 *          d_b the dense tile [256][64], d_meta [128][8] bytes: one byte per eight
 *          logical K positions, low nibble = first group, each nibble =
 *          position of 1st kept element | position of 2nd kept element << 2.
 *   MXF4_SP / NVF4_SP K = 128 logical.  4-bit operands are pruned in pairs: of every
 *          four pairs (eight positions) along K two are kept.  d_a is the compressed
 *          tile [128][64 e2m1] = 32 bytes per row, d_b the dense tile [256][128 e2m1],
 *          d_meta [128][8] bytes: one nibble per eight logical positions (low nibble
 *          first) = index of 1st kept pair | index of 2nd kept pair << 2.  Scale
 *          factors: d_sfa [128][n], d_sfb [256][n] with n = 2 (MXF4_SP, ue8m0) or 4
 *          (NVF4_SP, ue4m3); factor j covers logical K positions [j*128/n, (j+1)*128/n),
 *          i.e. 32 / 16 compressed elements of A (CLPK_DT_MXF4 / NVF4 on the compressed
 *          tile) and 64 / 32 elements of B (CLPK_DT_MXF4_B64 / NVF4_B32).
 * d_out receives the first `n_out_tiles` CTAs' accumulator tiles, row-major
 * [128][256] 32-bit words; d_checksum[grid] the XOR of every CTA's accumulator
 * bits; *d_status is set non-zero if a device-side wait timed out. */
#define CLPK_MMA_F16      0
#define CLPK_MMA_BF16     1
#define CLPK_MMA_E4M3     2
#define CLPK_MMA_E5M2     3
#define CLPK_MMA_I8       4
#define CLPK_MMA_MXF4     5
#define CLPK_MMA_NVF4     6
#define CLPK_MMA_E4M3_SP  7
#define CLPK_MMA_MXF4_SP  8
#define CLPK_MMA_NVF4_SP  9
#define CLPK_MMA_I8_SP    10
#define CLPK_MMA_TF32     11  /* K = 8: fp32 words with the low 13 mantissa bits clear (CLPK_DT_TF32), f32 accumulate  */
#define CLPK_MMA_F16_F16  12  /* K = 16: fp16 operands, fp16 accumulate; output words hold the half in bits 0..15   */
#define CLPK_MMA_E2M1     13  /* K = 32: unscaled e2m1 through kind::f8f6f4; tiles [rows][16 bytes], two per byte    */
#define CLPK_MMA_KIND_COUNT 14

typedef struct clpk_mma_peak_args {
    int         kind;
    const void *d_a;          /* [128][K] (dense) or [128][K/2] (sparse), element type of kind */
    const void *d_b;          /* [256][K]                                                     */
    const void *d_sfa;        /* block-scaled kinds only                                      */
    const void *d_sfb;
    const void *d_meta;       /* sparse kinds only: [128][K/8] bytes, see mma_peak.cu         */
    uint32_t    n_mma;        /* instructions per CTA (>= 1)                                  */
    uint32_t    grid;         /* CTAs                                                         */
    uint32_t    n_out_tiles;  /* how many CTAs store their tile to d_out (<= grid)            */
    void       *d_out;        /* n_out_tiles * 128*256 * 4 bytes                              */
    uint32_t   *d_checksum;   /* grid words, may be NULL                                      */
    uint32_t   *d_status;     /* one word, zeroed by the call                                 */
    unsigned long long *d_clock; /* optional, two words: CTA 0 stores the SM cycles (clock64) and the
                                  * nanoseconds (%globaltimer) between its first issue and the retirement
                                  * of its last instruction; cycles / ns is the SM clock the run really had */
} clpk_mma_peak_args_t;

CLPK_API int clpk_mma_peak(const clpk_mma_peak_args_t *args, void *stream);
/* K (logical, per instruction) and flop count per instruction for a kind
 * (2*128*256*K, counted at the logical K for sparse kinds, the reference's
 * convention: src/cuda/cuda_kernels/wmma_int8_sparse.cu:29-34). */
CLPK_API int clpk_mma_kind_k(int kind);
CLPK_API double clpk_mma_flops_per_instr(int kind);

/* fp64 tensor-core peak.  Takes the place of wmma_fp64
 * (src/cuda/cuda_kernels/wmma_fp64.cu:15-46; row at src/cuda/wmma.cpp:131-138).  tcgen05 has
 * no fp64 kind, so this is the warp-level mma.sync.m8n8k4.f64 path: CLPK_DMMA_WARPS warps
 * per CTA, CLPK_DMMA_CHAINS independent accumulator tiles per warp, n_mma dependent
 * instructions D = A*B + D per chain.  d_a is A [8][4] row-major, d_b is B as [8][4]: row n
 * holds column n of B.  Chain j of warp w starts at w*CLPK_DMMA_CHAINS + j in every element.
 * d_out receives, for each of the first n_out_tiles CTAs and each of its warps, the
 * element-wise sum of that warp's chains: [n_out_tiles][CLPK_DMMA_WARPS][8][8] doubles.
 * d_checksum[grid] (may be NULL) is a hash of each CTA's tiles; all CTAs must agree.
 * Work: 8*8*4*2 = 512 flop per instruction per warp, the reference's count. */
#define CLPK_DMMA_WARPS   8
#define CLPK_DMMA_CHAINS  8
CLPK_API int clpk_dmma_peak(const double *d_a, const double *d_b, uint32_t n_mma, uint32_t grid,
                            uint32_t n_out_tiles, double *d_out, uint32_t *d_checksum, void *stream);

/* ---- GEMM (takes the place of cuBLASLt in CudaPeak::runCublas) -----------------------------------
 * C[M][N] = A[M][K] * B[N][K]^T: A row-major, B "column-major K x N" = N rows
 * of K contiguous elements -- the reference's TN layout
 * (src/cuda/cuda_blas.cpp:275-287).  Accumulation in tensor memory, no epilogue
 * beyond the multiplication by `alpha` (the product of the NVF4 tensor scales).
 *   dtype            A / B elements                  accumulate   C element
 *   CLPK_DT_F32      fp32, CUDA cores (FFMA)         fp32         fp32   the reference's "fp32" row
 *   CLPK_DT_F64      fp64, mma.sync.m8n8k4 (DMMA)    fp64         fp64   the reference's "fp64" row
 *                    (src/cuda/cuda_blas.cpp:567-581); any M, N > 0, K a multiple of 4 (fp32) or 2 (fp64)
 *   CLPK_DT_BF16     bf16                            fp32         bf16
 *   CLPK_DT_F16      fp16                            fp32         bf16
 *   CLPK_DT_TF32     fp32 words (19 bits read)       fp32         fp32
 *   CLPK_DT_E4M3     e4m3                            fp32         bf16
 *   CLPK_DT_E5M2     A e5m2, B e4m3 (the pairing of the reference's fp8_e5m2 row,
 *                    src/cuda/cuda_blas.cpp:632-638)  fp32         bf16
 *   CLPK_DT_I8       int8                            int32        int32 (alpha ignored)
 *   CLPK_DT_MXF4     e2m1 + ue8m0 per 32             fp32         bf16
 *   CLPK_DT_NVF4     e2m1 + ue4m3 per 16             fp32         bf16
 * tcgen05 kinds: any M, N, K > 0 such that a row of A / B and a row of C are multiples of 16
 * bytes (partial tiles are computed whole and clipped; whole 512 x 256 tiles and K a multiple
 * of 128 bytes waste nothing).  FP4 kinds: K a multiple of 256; the workspace holds scale
 * blocks for M and N rounded up to multiples of 256.
 * FP4 kinds: d_a/d_b are packed e2m1 (K/2 bytes per row); d_sfa/d_sfb are the
 * scale bytes row-major [rows][K/16] (NVF4) or [rows][K/32] (MXF4) as written by
 * clpk_quantize_fp4; the call repacks them into the tensor-core tile order in
 * d_workspace (clpk_gemm_workspace_bytes) before the main kernel.  Operands that
 * are multiplied more than once can be repacked once: clpk_gemm_pack_scales does
 * only the repack (same arguments; d_a, d_b, d_c, d_status unused), and a
 * clpk_gemm call with d_sfa = d_sfb = NULL takes the workspace as already packed
 * -- the position cuBLASLt puts its caller in, whose scale arrays must arrive
 * in tile order (src/cuda/cuda_blas.cpp:456-491 fills them once, before timing). */
typedef struct clpk_gemm_args {
    int         dtype;
    uint32_t    m, n, k;
    const void *d_a;
    const void *d_b;
    void       *d_c;          /* [M][N] row-major, element type by dtype (table above) */
    const void *d_sfa;
    const void *d_sfb;
    float       alpha;        /* applied in the epilogue; pass 1.0f when unused */
    void       *d_workspace;
    size_t      workspace_bytes;
    uint32_t   *d_status;     /* one word, zeroed by the call */
} clpk_gemm_args_t;

CLPK_API int clpk_gemm_workspace_bytes(int dtype, uint32_t m, uint32_t n, uint32_t k, size_t *bytes);
CLPK_API int clpk_gemm_pack_scales(const clpk_gemm_args_t *args, void *stream);
CLPK_API int clpk_gemm(const clpk_gemm_args_t *args, void *stream);
/* 1 if the calling thread's last clpk_gemm launch ran with the per-wave producer meeting (a
 * cooperative launch), 0 if it ran without (small problem, knob, or the cooperative launch did
 * not fit), -1 before any launch.  Lets a benchmark record which schedule it timed. */
CLPK_API int clpk_gemm_last_launch_aligned(void);
/* SM cycles (clock64) and nanoseconds (%globaltimer) that CTA 0 of the last tensor-core GEMM
 * launched on the current device ran for; cycles / ns is the SM clock the kernel really had, which
 * under the power cap is well below the nominal one.  Waits for `stream`.  The fp32 / fp64 kernels
 * do not write it. */
CLPK_API int clpk_gemm_last_clock(unsigned long long *h_cycles, unsigned long long *h_ns, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* CLPEAK_B200_KERNELS_H */

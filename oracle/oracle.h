/* CPU oracle for the clpeak_b200 kernels -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of what every kernel behind
 * include/clpeak_b200_kernels.h must compute.  Only tests/, the smoke check and
 * the cpu_baseline / reference legs of bench.py may load this library; the
 * product never does.
 *
 * Parity status: the reference project (clpeak) never reads a kernel's output
 * back and holds no numeric golden vectors for this path, so kernel VALUES are
 * "parity unpinned" by the reference.  What the reference does pin, and what
 * this oracle is checked against, are: the per-thread access order of its
 * read-and-sum kernel, the chain shapes, the Sattolo cycle construction, the
 * op/byte accounting formulas, and the three format constants it hard-codes
 * (0x7F = 1.0 ue8m0, 0x38 = 1.0 ue4m3, src/cuda/cuda_blas.cpp:655-660).
 * Each function names the reference lines it follows.
 */
#ifndef CLPEAK_B200_ORACLE_H
#define CLPEAK_B200_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- seeded generators (the build's own counter-based streams) ---------- */
uint64_t orc_rand64(uint64_t seed, uint64_t idx);
float    orc_uniform01(uint64_t seed, uint64_t idx);
float    orc_uniform_pm1(uint64_t seed, uint64_t idx);
int      orc_uniform_i4(uint64_t seed, uint64_t idx);
float    orc_normal01(uint64_t seed, uint64_t idx);
/* dist: 0 uniform[0,1), 1 uniform[-1,1), 2 mean + std*N(0,1) */
void     orc_fill_f32(float *dst, uint64_t first, uint64_t n, uint64_t seed, int dist, float mean, float std);
void     orc_fill_i8(int8_t *dst, uint64_t first, uint64_t n, uint64_t seed);
/* The reference's own buffer fill (xorshift32 from 0xDEADBEEF, finite floats). */
void     orc_populate_reference(float *dst, uint64_t n);

/* ---- format codecs --------------------------------------------------------- */
uint16_t orc_f32_to_bf16(float x);
uint16_t orc_f32_to_f16(float x);
uint8_t  orc_f32_to_e4m3(float x);      /* RNE, saturate to +-448, NaN -> 0x7F */
uint8_t  orc_f32_to_e5m2(float x);      /* RNE, saturate to +-57344, NaN -> 0x7F */
uint8_t  orc_f32_to_e2m1(float x);      /* RNE, saturate to +-6 */
int8_t   orc_f32_to_i8(float x);
float    orc_bf16_to_f32(uint16_t h);
float    orc_f16_to_f32(uint16_t h);
float    orc_e4m3_to_f32(uint8_t b);
float    orc_e5m2_to_f32(uint8_t b);
float    orc_e2m1_to_f32(uint8_t nibble);
float    orc_ue8m0_to_f32(uint8_t b);
uint8_t  orc_ue8m0_for_absmax(float amax);
/* dtype numbering of include/clpeak_b200_kernels.h (CLPK_DT_*). */
void     orc_convert_f32(void *dst, const float *src, uint64_t n, int dtype);
float    orc_absmax_f32(const float *src, uint64_t n);
void     orc_quantize_fp4(uint8_t *packed, uint8_t *scales, const float *src, uint64_t rows,
                          uint64_t cols, int dtype, float tensor_scale);
/* Dequantise one element of a block-scaled FP4 matrix (without the tensor scale). */
double   orc_fp4_element(const uint8_t *packed, const uint8_t *scales, uint64_t cols, int dtype,
                         uint64_t row, uint64_t col);

/* 2:4 structured sparsity along K: keep the two largest magnitudes of every
 * group of four (ties: lower index), write them in index order to
 * `compressed` ([rows][k/2]) and their 2-bit positions to `meta`
 * ([rows][k/4] bytes: low nibble = idx0 | idx1 << 2).  `pruned` (optional)
 * receives the dense tile with the dropped elements zeroed. */
void     orc_prune_2to4(float *compressed, uint8_t *meta, float *pruned, const float *dense,
                        uint64_t rows, uint64_t k);

/* ---- bandwidth kernels -------------------------------------------------------- */
/* Reference order: src/cuda/cuda_kernels/global_bandwidth.cu:14-71. */
void     orc_global_bandwidth(int width, const float *in, float *out, uint64_t n_floats);
uint32_t orc_xor_words(const void *src, uint64_t n_bytes);
/* a = b + s*c, two roundings; src/cpu/bandwidth.cpp:339-346. */
void     orc_triad(float *a, const float *b, const float *c, float s, uint64_t n);
/* Multi-threaded STREAM passes used as the CPU baseline of bench.py.
 * kind: 0 read (returns XOR), 1 copy, 2 triad.  Returns seconds per pass. */
double   orc_stream_pass_mt(int kind, float *a, const float *b, const float *c, uint64_t n,
                            int threads, int passes, uint32_t *xor_out);

/* ---- chains -------------------------------------------------------------------------- */
/* src/cuda/cuda_kernels/compute_sp.cu:12-24: x = fma(x,x,c), c = thread index in block. */
void     orc_compute_sp(float *out, float a, uint64_t n_threads);
/* chain = CLPK_CHAIN_* (half, half2, double, mixed, bf16, int32, int8 dot x1/2/4/8):
 * src/cuda/cuda_kernels/compute_{hp,dp,mp,bf16,int32,int8_dp}.cu. */
void     orc_compute_chain(int chain, void *out, double a, uint64_t n_threads);
/* src/cuda/cuda_kernels/local_bandwidth.cu, image_bandwidth.cu. */
void     orc_local_bandwidth(int width, float *out, uint64_t n_threads);
/* threads [first, first + count) of a launch of n_threads */
void     orc_image_bandwidth(float *out, uint64_t first, uint64_t count, uint64_t n_threads, uint64_t texels, uint64_t seed);
void     orc_image_bandwidth_tiled(float *out, uint64_t first, uint64_t count, uint32_t width, uint32_t height, uint64_t seed);
void     orc_mad_chain(float *out, uint64_t first, uint64_t n_items, uint64_t seed, float y, uint32_t iters);

/* ---- pointer chase ---------------------------------------------------------------------- */
/* Sattolo single cycle as in src/cpu/latency.cpp:50-60 (seeded by orc_rand64). */
void     orc_chase_cycle(uint32_t *next, uint64_t n, uint64_t seed);
int      orc_is_single_cycle(const uint32_t *next, uint64_t n);
void     orc_chase(const uint32_t *next, uint32_t start, uint64_t hops, uint32_t *final_idx, uint32_t *xor_idx);

/* ---- tensor tiles ------------------------------------------------------------------------- */
/* One instruction's exact product tile P[128][256] = A[128][K] * B[256][K]^T in
 * double, and S = sum |a||b| (for tolerances).  kind = CLPK_MMA_* (dense kinds
 * 0..6).  Operands in the kernel's input encoding. */
void     orc_mma_tile(int kind, const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb,
                      double *p_out, double *s_out);
/* int8: n_mma accumulations, wrapped to int32 exactly like the hardware adder. */
void     orc_mma_tile_i8(const int8_t *a, const int8_t *b, uint32_t n_mma, int32_t *out);

/* Pair-granular 2:4 pruning for 4-bit operands and the exact product tile of one
 * sparse instruction (kinds CLPK_MMA_E4M3_SP / I8_SP: logical K = 64;
 * MXF4_SP / NVF4_SP: logical K = 128, 2 / 4 scale factors per row). */
void     orc_prune_pairs_2to4(float *compressed, uint8_t *meta, float *pruned, const float *dense,
                              uint64_t rows, uint64_t k);
void     orc_mma_tile_sp(int kind, const void *a_comp, const uint8_t *meta, const void *b, const uint8_t *sfa,
                         const uint8_t *sfb, double *p_out, double *s_out);

/* One element of C = A * B^T in double from the quantised operands.
 * dtype = CLPK_DT_BF16 / F16 / E4M3 / E5M2 (e5m2 A x e4m3 B) / I8 / TF32 / MXF4 / NVF4
 * (sfa/sfb used for the block-scaled kinds). */
double   orc_gemm_element(int dtype, const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb,
                          uint64_t k, uint64_t i, uint64_t j, double *abs_sum);

/* fp64 tensor probe: expected [warps][8][8] chain sums of clpk_dmma_peak (successor of
 * src/cuda/cuda_kernels/wmma_fp64.cu:15-46). */
void     orc_dmma_tiles(const double *a, const double *b, uint32_t n_mma, int warps, int chains, double *out);

/* pickIters, src/common/common.cpp:35-45. */
unsigned orc_pick_iters(double per_iter_us, unsigned target_us, unsigned forced, unsigned max_iters);

#ifdef __cplusplus
}
#endif
#endif

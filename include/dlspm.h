/*
 * dlspm.h — C ABI of the B200 (sm_100a) sparse-kernel library: CSR SpMM, SDDMM and the
 * fused SDDMM->SpMM chain in fp32.
 *
 * The reference project (zubair23517/dlspm-esimd) has no library boundary; its de-facto
 * interfaces are kernel templates that take raw device pointers, host loops with the same
 * argument order, and command-line drivers.  Every entry point below names the reference
 * interface it replaces (file:line inside that project).
 *
 * Conventions
 *   - CSR layout is the reference's: int32 row_offsets[M+1], int32 column_indices[nnz],
 *     fp32 values[nnz]; dense operands are row-major fp32.
 *   - Pointers are DEVICE pointers unless the function name ends in _host.
 *   - The caller owns every buffer it passes (as in the reference, where main() allocates
 *     and frees everything: SPMM/spmm-esimd-fromfile.cpp:172-180,294-304).
 *   - Every function returns a dlspm_status; nothing throws across the boundary.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 *   - Differences from the reference kernels, on purpose: arrays are exact-size (no 2*VLC
 *     padding, SPMM/spmm-esimd-fromfile2.cpp:174-176); outputs are fully written, so no
 *     memset before a launch is needed (the reference relies on a pre-zeroed output for
 *     empty rows, SPMM/spmmesimd2.hpp:90-91); any N >= 1 is accepted (the reference needs
 *     N % 16 == 0, SPMM/spmm-esimd-fromfile2.cpp:230-231); addressing is 64-bit; results
 *     are deterministic (no atomics, unlike SDDMM/sddmm-esimd-fromfile_v4.hpp:161).
 *   - There is no CPU fallback: without a usable CUDA device dlspm_create fails.
 */
#ifndef DLSPM_H
#define DLSPM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dlspm_status {
    DLSPM_OK = 0,
    DLSPM_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, bad enum            */
    DLSPM_ERR_CUDA = 2,             /* a CUDA runtime call failed (see dlspm_last_error) */
    DLSPM_ERR_IO = 3,               /* file could not be opened                          */
    DLSPM_ERR_FORMAT = 4,           /* .smtx text did not parse                          */
    DLSPM_ERR_CSR = 5,              /* CSR structure failed the sanity check             */
    DLSPM_ERR_NOMEM = 6,            /* host or device allocation failed                  */
    DLSPM_ERR_UNSUPPORTED = 7,      /* size beyond a documented limit                    */
    DLSPM_ERR_NO_DEVICE = 8,        /* no CUDA device / not an sm_100 device             */
    DLSPM_ERR_TIMEOUT = 9           /* a bounded wait inside a kernel ran out            */
} dlspm_status;

typedef struct dlspm_ctx dlspm_ctx;   /* one per device; not shared between host threads */
typedef struct dlspm_plan dlspm_plan; /* reusable row binning of one CSR pattern         */
typedef struct dlspm_mg dlspm_mg;     /* a set of devices driven by one host process     */

/* ---- library / context ------------------------------------------------------------ */

/* Replaces the reference's queue construction (SPMM/spmm-esimd-fromfile.cpp:98). */
int dlspm_create(dlspm_ctx **ctx, int device);
int dlspm_destroy(dlspm_ctx *ctx);
/* Human-readable text for a status code. */
const char *dlspm_strerror(int status);
/* Text of the last CUDA error seen by this context ("" if none). */
const char *dlspm_last_error(const dlspm_ctx *ctx);
/* Device facts the drivers print (the reference prints the device name, :101-103). */
int dlspm_device_info(const dlspm_ctx *ctx, char *name, size_t name_len, int *sm_count,
                      size_t *global_mem_bytes);

typedef enum dlspm_option {
    /* 1: SpMM multiplies and adds with separate roundings in CSR order, which reproduces the
     * reference CPU loop (SPMM/spmm-esimd-fromfile.cpp:63-83, built without FMA contraction)
     * bit for bit.  0 (default): fused multiply-add. */
    DLSPM_OPT_STRICT_FP32 = 0,
    /* SpMM kernel choice in prepared batches: 0 = automatic (density threshold below), 1 = row-gather
     * kernel only, 2 and 3 = shared-memory tiled kernel wherever it applies (N % 4 == 0, aligned dense
     * operands, strictly ascending columns in every row; restricted by the threshold below only if
     * the caller has set one).  3 is the form the automatic choice uses: absent entries are
     * multiplied as zeros, except in chunks of B that hold an infinity or a NaN, which run under the
     * presence masks, so that a non-finite value of B reaches exactly the rows that reference it, as
     * in the reference loop.  2 runs every chunk under the masks (slower; kept for tests).  All
     * choices give the same bits on the same input (apart from the sign of a zero sum, see the
     * kernel). */
    DLSPM_OPT_SPMM_KERNEL = 1,
    /* Threshold of the automatic choice, in thousandths: the tiled kernel is taken for problems
     * whose fraction of nonzeros is at least value/1000.  Default 450: on B200 the tiled kernel
     * reaches 22.5 TFLOP/s on half-full problems against 15.8 for the row-gather kernel, and loses
     * at 30 % nonzeros (13.9 against 17).  1001 = never; -1 = back to the default, as if never set. */
    DLSPM_OPT_TILE_MIN_DENSITY = 2,
    /* 1: every entry point that takes a CSR pattern validates it before it launches anything
     * (row offsets start at 0, end at nnz, never decrease, no row longer than K, every column index
     * in [0, K)) and returns DLSPM_ERR_CSR with the reason in dlspm_last_error otherwise: device
     * arrays through the kernel of dlspm_sanity_check_csr, host arrays (the *_host entry points)
     * through dlspm_sanity_check_csr_host.  The kernels trust their input as the reference's do
     * (a column index beyond K reads outside B), so this is the mode to run untrusted or freshly
     * assembled patterns under; it stands in for a memory checker.  A debugging mode: every check
     * of a device pattern allocates a status word and synchronises the stream, grouped calls check
     * their problems one by one; not for calls on a capturing stream (the check would end the
     * capture with an error).  dlspm_spmm_batched_f32_static, which must not allocate, ignores
     * it.  0 (default): no checks. */
    DLSPM_OPT_CHECK_INPUT = 3
} dlspm_option;
int dlspm_set_option(dlspm_ctx *ctx, int option, int value);
int dlspm_get_option(const dlspm_ctx *ctx, int option, int *value);

/* ---- the three kernels ------------------------------------------------------------ */

/* C[M x N] = A_csr[M x K] * B[K x N].  Replaces SpmmEsimd<CHUNK>(a_values, a_row_offsets,
 * a_column_indices, b, c, item, MSZ, KSZ, NSZ) (SPMM/spmmesimd2.hpp:63-67) together with its
 * launch geometry (SPMM/spmm-esimd-fromfile2.cpp:188-231); same result as the host loop Spmm
 * (SPMM/spmm-esimd-fromfile.cpp:63-83).  Empty rows produce zeros. */
int dlspm_spmm_csr_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                       const int *row_offsets, const int *column_indices, const float *B,
                       float *C, void *stream);

/* Same with a plan (row-length binning computed once per sparsity pattern). */
int dlspm_spmm_csr_f32_planned(dlspm_ctx *ctx, const dlspm_plan *plan, int N,
                               const float *values, const int *row_offsets,
                               const int *column_indices, const float *B, float *C,
                               void *stream);

/* out_values[p] = dot(lhs[i, 0:N], rhs[column_indices[p], 0:N]) for every nonzero p of row i.
 * N is the inner (dot) dimension, as NSZ is in the reference.  Replaces smallK::Launcher(
 * row_offsets, column_indices, lhs, rhs, out, NSZ, NT, nh_threads, NSZC, queue)
 * (SDDMM/sddmm-esimd-fromfile_v4.hpp:255-262); same result as the host loop Sddmm
 * (SDDMM/sddmm-esimd-fromfile_v4.cpp:18-36).  Mask values are never read (treated as 1).
 * lhs is M x N, rhs is K x N. */
int dlspm_sddmm_csr_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                        const int *column_indices, const float *lhs, const float *rhs,
                        float *out_values, void *stream);

/* The same with the stored values of the mask as factors: out_values[p] = mask_values[p] * dot
 * (the S_ij * (A_i . B_j) form).  mask_values may be NULL, which means 1.0 and is the reference's
 * behaviour (its kernels never read the mask's values, SDDMM/sddmm-esimd-fromfile_v4.hpp:102-177).
 * mask_values and out_values must not overlap. */
int dlspm_sddmm_csr_masked_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                               const int *column_indices, const float *mask_values,
                               const float *lhs, const float *rhs, float *out_values, void *stream);

/* E[M x N] = (pattern(A) .* (C * B^T)) * D without writing the sampled products to memory.
 * C is M x N, B and D are K x N.  Replaces FusedEsimd(a_row_offsets, a_column_indices, c, b,
 * d, e, item) (FUSED/fused-esimd_cb.cpp:100-105); same result as Sddmm followed by Spmm
 * (FUSED/fused.cpp:47-89). */
int dlspm_fused_sddmm_spmm_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                               const int *row_offsets, const int *column_indices,
                               const float *C, const float *B, const float *D, float *E,
                               void *stream);

/* Sparse attention around the fused kernel: O[i, :] = sum_p w_p * V[column_indices[p], :] over the
 * stored entries p of row i, with s_p = scale * dot(Q[i, :], Kmat[column_indices[p], :]) and
 *   flags = 0:                   w_p = s_p              (the fused chain with a scale factor)
 *   flags = DLSPM_ATTN_SOFTMAX:  w_p = exp(s_p - max_p s_p) / sum_p exp(s_p - max_p s_p)
 * The weights never reach memory; rows without stored entries give zeros.  Q and O are M x N,
 * Kmat and V are K x N; scale must be finite.  The reference has no counterpart of the two extra
 * steps (its fused chain is FUSED/fused-esimd_cb.cpp:100-189, which this call reproduces for
 * flags = 0, scale = 1); the checker for them is a double-precision restatement of the formulas
 * above, so their parity is not pinned to reference code. */
#define DLSPM_ATTN_SOFTMAX 1u
int dlspm_fused_attention_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                              const int *row_offsets, const int *column_indices,
                              const float *Q, const float *Kmat, const float *V, float *O,
                              float scale, unsigned flags, void *stream);

/* ---- plans ------------------------------------------------------------------------ */

/* Bins the rows of one pattern by length so that warps of one thread block get rows of similar
 * length and long rows start first.  The reference has a single launch geometry per matrix
 * (ComputeNT, SPMM/spmmesimd2.hpp:30-60); this is the equivalent set-up step.  row_offsets is a
 * device pointer; the plan keeps its own device copy of the row order. */
int dlspm_plan_create(dlspm_ctx *ctx, int M, int K, int nnz, const int *row_offsets,
                      const int *column_indices, void *stream, dlspm_plan **plan);
int dlspm_plan_destroy(dlspm_plan *plan);
/* Copies the plan's row order (M ints) to HOST memory `order` and synchronises `stream`: rows in
 * bins by length (bin b: 2^(b-1) <= length < 2^b, empty rows last) from the longest bin to the
 * shortest, by ascending row number inside a bin.  The order is a function of the pattern alone,
 * so the kernels that walk it do the same work in the same order in every run.  For inspection
 * and tests; the SpMM entry points read the plan on the device. */
int dlspm_plan_row_order(const dlspm_plan *plan, int *order, void *stream);

/* ---- grouped launch over many independent SpMMs ------------------------------------- */

typedef struct dlspm_problem {
    int M, K, N, nnz;
    const float *values;       /* device */
    const int *row_offsets;    /* device */
    const int *column_indices; /* device */
    const float *B;            /* device, K x N */
    float *C;                  /* device, M x N */
} dlspm_problem;

/* Runs `count` independent SpMMs in one launch.  Replaces the per-matrix process launches of
 * the batch drivers (SPMM/batch-run-spmm_fromfile:29-47).  `problems` is a HOST array; the
 * table is copied to device scratch owned by the context, so calls on one context must be ordered
 * on one stream (two calls whose work overlaps on the GPU would share that scratch).  The table
 * copies read host memory that dies with the call, so the call cannot be recorded into a CUDA
 * graph: on a capturing stream it returns DLSPM_ERR_UNSUPPORTED before anything is enqueued (use
 * dlspm_batch_create + dlspm_batch_launch there). */
int dlspm_spmm_batched_f32(dlspm_ctx *ctx, int count, const dlspm_problem *problems,
                           void *stream);

/* The same grouped launch for callers that must not allocate device memory (a plug-in whose host
 * owns the device heap, a loop that may not take the allocator's lock).  This entry point has no
 * counterpart in the reference.  It never calls cudaMalloc/cudaFree or any allocating routine: its
 * problem table, tile index and work counter live in a fixed __device__ array inside the library
 * (90 624 bytes = 88.5 KiB per GPU, held until the process exits).  Limit: count <= 1024 problems,
 * otherwise DLSPM_ERR_UNSUPPORTED.  Host side: no heap either, and about 5 KiB of stack (the table is
 * built and sent in chunks of 32 problems), so it fits the small stacks of plug-in threads.  The
 * first call on a device looks up the array's device address; make that call before any stream
 * capture starts in the process.  Like the allocating one-shot call it copies its table from host
 * memory and therefore refuses a capturing stream with DLSPM_ERR_UNSUPPORTED.  All calls on a device
 * share the one array, so two calls whose work overlaps on the GPU (different streams, no ordering)
 * race; calls on one stream are safe.  Results are identical to dlspm_spmm_batched_f32. */
int dlspm_spmm_batched_f32_static(dlspm_ctx *ctx, int count, const dlspm_problem *problems,
                                  void *stream);

/* ---- grouped launches over many independent SDDMMs / fused chains --------------------------- */

typedef struct dlspm_sddmm_problem {
    int M, K, N, nnz;          /* N = inner (dot) dimension                                   */
    const int *row_offsets;    /* device */
    const int *column_indices; /* device */
    const float *mask_values;  /* device, nnz factors, or NULL = 1.0 (the reference's behaviour) */
    const float *lhs;          /* device, M x N */
    const float *rhs;          /* device, K x N */
    float *out_values;         /* device, nnz   */
} dlspm_sddmm_problem;

typedef struct dlspm_fused_problem {
    int M, K, N, nnz;
    const int *row_offsets;    /* device */
    const int *column_indices; /* device */
    const float *C;            /* device, M x N */
    const float *B;            /* device, K x N */
    const float *D;            /* device, K x N */
    float *E;                  /* device, M x N */
} dlspm_fused_problem;

/* Runs `count` independent SDDMMs (each as dlspm_sddmm_csr_masked_f32 would) in one persistent
 * launch per register layout present in the batch (the layout follows from N: at most twelve, one for
 * a batch with a single inner dimension).  Replaces the per-matrix process launches of
 * SDDMM/batch-run-sddmm_fromfile:31-47, where every layer-sized pattern is launch-bound on its own.
 * `problems` is a HOST array; the tables go to the context's scratch, so the same rules as for
 * dlspm_spmm_batched_f32 hold: calls on one context ordered on one stream, not on a capturing
 * stream.  Problems whose N or pointers rule out 128-bit loads (for the fused chain also those with
 * N > 1024) are run one by one with the single-matrix kernels inside the same call. */
int dlspm_sddmm_batched_f32(dlspm_ctx *ctx, int count, const dlspm_sddmm_problem *problems, void *stream);
/* The same for the fused SDDMM -> SpMM chain (each problem as dlspm_fused_sddmm_spmm_f32 would);
 * replaces the per-matrix runs of FUSED/batch-run-fused:22-34. */
int dlspm_fused_batched_f32(dlspm_ctx *ctx, int count, const dlspm_fused_problem *problems, void *stream);
/* Host-pointer forms: every array of every problem is copied in, the grouped launch runs, results
 * are copied back; returns when they are on the host. */
int dlspm_sddmm_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_sddmm_problem *problems);
int dlspm_fused_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_fused_problem *problems);

/* A prepared batch: the problem table and its tile index live on the device, so repeated
 * launches cost no host work.  Creating it also analyses the patterns on the device: rows are
 * ordered by length inside every problem (so that the warps of a tile finish together), and
 * problems that are dense enough and have ascending columns are routed to the tiled kernel. */
typedef struct dlspm_batch dlspm_batch;
int dlspm_batch_create(dlspm_ctx *ctx, int count, const dlspm_problem *problems,
                       dlspm_batch **batch);
int dlspm_batch_launch(dlspm_ctx *ctx, const dlspm_batch *batch, void *stream);
/* Launches one part of a prepared batch only: 0 = everything (same as dlspm_batch_launch),
 * 1 = the problems served by the row-gather kernel, 2 = those served by the tiled kernel.  Lets a
 * benchmark time the two kernels separately. */
int dlspm_batch_launch_part(dlspm_ctx *ctx, const dlspm_batch *batch, int part, void *stream);
/* How many problems of the batch run on the row-gather and on the tiled kernel; (if device_error
 * is not NULL: synchronises the device) whether a kernel of this batch gave up a bounded wait
 * (0 = no); stats4 = {2*nnz*N, algorithmic bytes} of the row-gather part, then of the tiled part.
 * Any pointer may be NULL. */
int dlspm_batch_info(dlspm_ctx *ctx, const dlspm_batch *batch, int *gather_problems,
                     int *tiled_problems, int *device_error, double *stats4);
int dlspm_batch_destroy(dlspm_batch *batch);

/* ---- host-buffer entry points (copies in and out included) ----------------------------- */

/* Same operations with HOST pointers: inputs are copied to the device, the kernel runs, the
 * result is copied back, all on the context's stream; returns after the result is on the host.
 * These are what a caller that keeps its data in host memory (as the reference drivers do
 * before their explicit memcpy, SPMM/spmm-esimd-fromfile.cpp:172-180) binds to. */
int dlspm_spmm_csr_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                            const int *row_offsets, const int *column_indices, const float *B,
                            float *C);
int dlspm_sddmm_csr_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                             const int *row_offsets, const int *column_indices,
                             const float *lhs, const float *rhs, float *out_values);
int dlspm_fused_sddmm_spmm_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                                    const int *row_offsets, const int *column_indices,
                                    const float *C, const float *B, const float *D, float *E);
/* Batched SpMM with host pointers inside every dlspm_problem: pieces of up to 128 MiB are copied in,
 * run as one grouped launch and copied out on three streams, so the two copy directions and the
 * kernels overlap.  Arrays are copied one by one unless they are neighbours in ONE pinned host
 * allocation in the order and spacing of the staging layout (per problem row_offsets,
 * column_indices, values, B, each padded to a multiple of 256 bytes, problems one after the other;
 * the C buffers likewise in problem order): such a run goes as a single copy, one per piece and
 * direction for a batch kept in two pinned arenas.  Results are the same either way. */
int dlspm_spmm_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_problem *problems);
/* Number of cudaMemcpyAsync calls the pipelined host-buffer batch has issued on this context so far
 * (lets a caller see whether its buffer layout was merged into few copies). */
int dlspm_host_copy_count(const dlspm_ctx *ctx, long long *copies);

/* ---- .smtx reader and CSR validation (host) -------------------------------------------- */

/* Reads "M, K, nnz" / M+1 row offsets / nnz column indices.  Replaces the fscanf reader in
 * every *fromfile* driver (SPMM/spmm-esimd-fromfile.cpp:105-137).  The arrays are malloc'ed
 * here; release them with dlspm_free_host. */
int dlspm_read_smtx_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                         int **column_indices);
/* Writes the same text format (used by tests and by the drivers' --dump option). */
int dlspm_write_smtx_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                          const int *column_indices);
/* The text format with values: a fourth block of nnz decimal floats ("%.9g", exact for fp32)
 * after the column indices.  The reference's format carries no values (its drivers fill them with
 * rand(), SPMM/spmm-esimd-fromfile.cpp:140-149) and its reader stops after the indices, so such a
 * file is still a valid pattern file for it.  On reading, *values is NULL when the file has no
 * fourth block. */
int dlspm_read_smtx_values_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                                int **column_indices, float **values);
int dlspm_write_smtx_values_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                                 const int *column_indices, const float *values);
/* Binary cache of a parsed matrix, so that large inputs are not re-parsed from text: 48-byte
 * little-endian header (magic "DLSPMCSR", version, flags, M, K, nnz, checksum, payload size),
 * then row_offsets, column_indices and, if values != NULL, values, each padded to 8 bytes.
 * Reading verifies magic, version, sizes against the file length and the checksum
 * (DLSPM_ERR_FORMAT otherwise); *values is NULL when the file carries none.  No reference
 * counterpart. */
int dlspm_write_csr_cache_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                               const int *column_indices, const float *values);
int dlspm_read_csr_cache_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                              int **column_indices, float **values);
void dlspm_free_host(void *p);

/* The reference's SanityCheck (SPMM/spmm-esimd-fromfile.cpp:36-61): nnz <= M*K,
 * row_offsets[M] == nnz, monotone offsets, row length <= K, column < K; plus the checks the
 * reference omits (row_offsets[0] == 0, column >= 0).  Returns DLSPM_ERR_CSR on failure and, if
 * `why` is not NULL, copies a one-line reason (the reference's exception text where it has
 * one). */
int dlspm_sanity_check_csr_host(int M, int K, int N, int nnz, const int *row_offsets,
                                const int *column_indices, char *why, size_t why_len);

/* The same validation for CSR arrays in DEVICE memory (patterns generated or assembled on the device
 * never pass the host check): one kernel over the offsets and the column indices, then the answer is
 * read back (the call synchronises `stream`).  The kernels of this library trust their CSR arrays as
 * the reference's do: a column index beyond K reads outside B.  Run this first on input that is not
 * trusted; DLSPM_ERR_CSR and a one-line reason as above. */
int dlspm_sanity_check_csr(dlspm_ctx *ctx, int M, int K, int nnz, const int *row_offsets,
                           const int *column_indices, char *why, size_t why_len, void *stream);

/* ---- seeded synthetic inputs (host and device) ------------------------------------------ */
/* One counter-based generator (splitmix64 of seed, stream and element index) defines every
 * synthetic input, so host and device produce identical bits.  These stand in for the
 * reference's rand()-based generators (SPMM/spmm-esimd-allbenchs2.cpp:58-77). */

uint64_t dlspm_rand_u64(uint64_t seed, uint64_t stream, uint64_t index);
/* out[i] = U(-1,1) (kind 0), U[0,1) (kind 1) or N(0,1) (kind 2, Box-Muller) of element
 * first_index + i of (seed, stream). */
int dlspm_gen_dense_host(float *out, size_t n, uint64_t seed, uint64_t stream,
                         uint64_t first_index, int kind);
int dlspm_gen_dense(dlspm_ctx *ctx, float *out, size_t n, uint64_t seed, uint64_t stream,
                    uint64_t first_index, int kind, void *stream_);
/* Bernoulli-per-entry pattern: entry (i,j) is present iff its 24-bit uniform is below
 * density*2^24.  Same construction as the reference sweep generator.  column_indices has room
 * for `capacity` entries; *nnz receives the count (DLSPM_ERR_NOMEM if it does not fit). */
int dlspm_gen_bernoulli_csr_host(int M, int K, double density, uint64_t seed, int *row_offsets,
                                 int *column_indices, size_t capacity, int *nnz);
/* Row lengths clip(round(Normal(mu, cov*mu)), 0, K) with mu = K*(1-sparsity); writes the
 * prefix sum into row_offsets[M+1]. */
int dlspm_gen_rowlen_normal_host(int M, int K, double sparsity, double cov, uint64_t seed,
                                 int *row_offsets);
/* For given row_offsets, fills each row with a sorted uniform sample (without replacement) of
 * row-length columns out of K. */
int dlspm_gen_sample_columns_host(int M, int K, const int *row_offsets, uint64_t seed,
                                  int *column_indices);
int dlspm_gen_sample_columns(dlspm_ctx *ctx, int M, int K, const int *row_offsets,
                             uint64_t seed, int *column_indices, void *stream);
/* Banded mask: row i holds every j with |i-j| <= half_band plus Bernoulli(extra_density)
 * extras, sorted and without duplicates. */
int dlspm_gen_band_csr_host(int M, int K, int half_band, double extra_density, uint64_t seed,
                            int *row_offsets, int *column_indices, size_t capacity, int *nnz);
/* Device Bernoulli pattern in two steps: counts per row -> caller prefix-sums -> fill.  The M rows
 * generated are rows first_row .. first_row+M-1 of the K-column pattern of `seed`, so a row block
 * of a large matrix can be produced on its own; row_offsets/row_counts are local to the block. */
int dlspm_gen_bernoulli_count(dlspm_ctx *ctx, int M, int K, int first_row, double density,
                              uint64_t seed, int *row_counts, void *stream);
int dlspm_gen_bernoulli_fill(dlspm_ctx *ctx, int M, int K, int first_row, double density,
                             uint64_t seed, const int *row_offsets, int *column_indices,
                             void *stream);

/* ---- partitioning for several GPUs (host, no CUDA) --------------------------------------- */

/* Longest-processing-time assignment of `count` weighted items to `parts` parts: items in
 * decreasing weight (ties: lower index first) go to the least-loaded part (ties: lower part).
 * owner[i] receives the part of item i. */
int dlspm_partition_lpt_host(int count, const double *weights, int parts, int *owner);
/* Row boundaries so that each of `parts` contiguous row blocks holds about nnz/parts nonzeros:
 * bounds[parts+1], bounds[0] = 0, bounds[parts] = M. */
int dlspm_partition_rows_by_nnz_host(int M, const int *row_offsets, int parts, int *bounds);

/* ---- one process, several devices ------------------------------------------------------- */

int dlspm_mg_create(dlspm_mg **mg, int ndev, const int *devices);
int dlspm_mg_destroy(dlspm_mg *mg);
int dlspm_mg_device_count(const dlspm_mg *mg);
/* Batch of independent SpMMs with HOST pointers, partitioned by nnz*N across the devices, one
 * grouped launch per device, no exchange between devices. */
int dlspm_mg_spmm_batched_f32_host(dlspm_mg *mg, int count, const dlspm_problem *problems);
/* One large SpMM with HOST pointers: rows are sharded by nonzero count, B is replicated, every
 * device computes its row block of C, and the blocks are gathered into C on the host. */
int dlspm_mg_spmm_rowshard_f32_host(dlspm_mg *mg, int M, int K, int N, int nnz,
                                    const float *values, const int *row_offsets,
                                    const int *column_indices, const float *B, float *C);

/* ---- fused SpMM + gather over peer memory ------------------------------------------------------- */

/* Row-sharded SpMM whose epilogue is the gather: computes the M local rows (global rows first_row ..
 * first_row+M-1) and stores each of them into all `ndst` (<= 8) destination matrices C_dsts[d]
 * (full-size row-major C buffers: the local one and the peers', reached through peer mappings), so
 * no collective follows.  C_dsts is a HOST array of device pointers.  After every participating GPU
 * has finished its launch (stream synchronise + a host-side barrier between the processes or
 * threads), every destination holds the complete C.  The reference has no multi-GPU path
 * (SPMM/batch-run-spmm_fromfile:45 pins one device). */
int dlspm_spmm_csr_f32_scatter(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                               const int *row_offsets, const int *column_indices, const float *B,
                               int ndst, float *const *C_dsts, long long first_row, void *stream);
/* Same process, several devices: lets kernels of this context's device store into memory of
 * peer_device (cudaDeviceEnablePeerAccess). */
int dlspm_enable_peer_access(dlspm_ctx *ctx, int peer_device);
/* Other processes: allocate a device buffer and get the 64-byte handle a peer process turns into a
 * pointer with dlspm_peer_open (CUDA IPC); close / free when done. */
int dlspm_peer_alloc(dlspm_ctx *ctx, size_t bytes, void **ptr, unsigned char handle[64]);
int dlspm_peer_open(dlspm_ctx *ctx, const unsigned char handle[64], void **ptr);
int dlspm_peer_close(dlspm_ctx *ctx, void *ptr);
int dlspm_peer_free(dlspm_ctx *ctx, void *ptr);

/* ---- failure reporting ---------------------------------------------------------------------------- */

/* No kernel of the library waits without a limit: a wait that runs out sets a status word and the
 * kernel returns (DLSPM_ERR_TIMEOUT through dlspm_batch_info).  This self-test exercises exactly that
 * path with no fault involved: one thread polls, at most `polls` (<= 2^20) times, an mbarrier that
 * nothing completes.  Returns DLSPM_ERR_TIMEOUT with *timed_out = 1, and the context stays usable. */
int dlspm_selftest_bounded_wait(dlspm_ctx *ctx, unsigned polls, int *timed_out);

/* ---- measurement helpers ------------------------------------------------------------------ */

/* Sustained fp32 FMA rate of the device in TFLOP/s (a register-only FMA loop over all SMs); the
 * denominator of the compute term of the roofline. */
int dlspm_measure_fp32_peak(dlspm_ctx *ctx, double *tflops);
/* The same figure twice: with one multiply-add per instruction (as above) and with the packed form
 * (two per instruction, fma.rn.f32x2).  Both run on the same fp32 lanes; the pair shows whether the
 * packed form changes the arithmetic peak or only the number of issue slots it needs. */
int dlspm_measure_fp32_peaks(dlspm_ctx *ctx, double *scalar_tflops, double *packed_tflops);

#ifdef __cplusplus
}
#endif
#endif /* DLSPM_H */

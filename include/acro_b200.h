/*
 * acro_b200.h — C ABI of the B200 (sm_100a) contraction library.
 *
 * Plain C: pointers, sizes and integer status codes only.  Two layers:
 *
 *  1. KERNEL LAYER (acro_b200_*): one launcher per hand-written kernel family.
 *     This is the boundary the C++ back end (acro::B200Executor) binds; it
 *     stands where LLNL/acrotensor's "Cuda" policy calls its run-time generated
 *     kernel: CudaExecutor::ExecuteSingle / ExecuteMulti
 *     (exec/CudaExecutor.cpp:36-102) -> CudaKernel::Launch -> cuLaunchKernel
 *     (util/CudaUtil.cpp:95-103).  All pointers are DEVICE pointers of the
 *     current device; launches are asynchronous on `stream` (a cudaStream_t
 *     passed as void*, NULL = legacy default stream).
 *
 *  2. ENGINE LAYER (acro_tensor_*, acro_engine_*): handle-based mirror of the
 *     reference's user API (acro::Tensor, tensor/Tensor.hpp:15-127;
 *     acro::TensorEngine, kernel/TensorEngine.hpp:26-86) for hosts that cannot
 *     include C++ headers (ctypes, cgo, JNI ...).  Each function states the
 *     reference member it corresponds to.
 *
 * Every function returns ACRO_B200_OK or a negative status; the text of the
 * last failure on the calling thread is available from acro_b200_last_error().
 * Nothing here runs on the CPU: when no CUDA device is usable the compute
 * entry points fail with ACRO_B200_ECUDA.
 */
#ifndef ACRO_B200_H
#define ACRO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ACRO_B200_OK 0
#define ACRO_B200_EINVAL (-1)       /* bad argument / failed precondition (an exception in the C++ API) */
#define ACRO_B200_EUNSUPPORTED (-2) /* the family has no instantiation for these sizes */
#define ACRO_B200_ECUDA (-3)        /* CUDA runtime failure, or no device */
#define ACRO_B200_ETIMEOUT (-4)     /* a bounded device-side wait gave up */

#define ACRO_B200_MAX_PEERS 16
#define ACRO_B200_IPC_HANDLE_BYTES 64
#define ACRO_B200_MAX_LOOPS 24
#define ACRO_B200_MAX_INPUTS 12

/* assignment operators of a contraction string (kernel/TensorKernel.cpp:120-139) */
#define ACRO_B200_OP_ASSIGN 0 /* "="  */
#define ACRO_B200_OP_ADD 1    /* "+=" */
#define ACRO_B200_OP_SUB 2    /* "-=" */
/* May be or-ed into the `op` of the reduce_batch entry points that take caller-provided scratch: the
 * caller zeroed the first 256 bytes of that scratch buffer once (cudaMemset) and nothing but
 * reduce_batch calls has written to it since, so the clear in front of every launch is skipped. */
#define ACRO_B200_SCRATCH_READY 0x100

const char *acro_b200_last_error(void);

/* Number of usable CUDA devices (0 when there is none).  Replaces acro::isCudaReady(),
 * util/CudaUtil.hpp:175-184. */
int acro_b200_device_count(void);

/* Waits for the current device to go idle and reports ACRO_B200_ETIMEOUT if, since the last
 * call, a kernel's bounded wait on an asynchronous copy gave up (its results are invalid),
 * ACRO_B200_ECUDA on a CUDA failure, else ACRO_B200_OK.  Plays the role of the reference's
 * acroCudaErrorCheck after a launch (util/CudaUtil.hpp:59-89). */
int acro_b200_device_status(void);

/* Makes an externally created driver context (a CUcontext passed as void*) current for the
 * calling thread, as acro::setCudaContext does (util/CudaUtil.hpp:93-98); later calls of this
 * thread run in it.  Device addresses the library looked up in the previous context are
 * forgotten.  Device memory, tensors and engines created in one context must not be used in
 * another. */
int acro_b200_set_context(void *cuda_context);

/* ---------------------------------------------------------------- kernel layer */

/* Aout[i] = val / Aout[i] *= c.  Replace CudaSet / CudaMult, util/CudaUtil.cpp:123-140. */
int acro_b200_fill(double *data, int64_t n, double val, void *stream);
int acro_b200_scale(double *data, int64_t n, double c, void *stream);

/*
 * Generic contraction: any string the parser accepts.
 * Loops 0..n_outer-1 are the non-contracted loops (ordered so that the last
 * one is the output's fastest dimension), the remaining loops are the
 * contracted ones in the reference's summation order.  `*_step[l]` is the
 * element stride of that variable when loop l advances by one (0 when the
 * variable does not carry the loop; the sum of both strides for B_i_i).
 * One thread per output entry; terms are multiplied left to right and added
 * one by one without fused multiply-add, exactly as
 * exec/CPUInterpretedExecutor.hpp:58-77 does, so "=" results are bit-identical
 * to the reference's CPU executor.  Replaces the generated kernel of
 * exec/CudaExecutor.cpp:111-190 for shapes no specialised family covers.
 */
typedef struct acro_b200_generic_desc
{
    int32_t n_loops;
    int32_t n_outer;
    int32_t n_inputs;
    int32_t op;
    int64_t extent[ACRO_B200_MAX_LOOPS];
    int64_t out_step[ACRO_B200_MAX_LOOPS];
    int64_t in_step[ACRO_B200_MAX_INPUTS][ACRO_B200_MAX_LOOPS];
} acro_b200_generic_desc;

int acro_b200_generic_launch(const acro_b200_generic_desc *desc, double *out,
                             const double *const *inputs, double *scratch, size_t scratch_bytes,
                             void *stream);
/* Shapes with at most 2048 output entries and at least 16384 terms each (for example
 * "S_a = X_n_a Y_n_a") use a second variant, because one thread per entry would idle the GPU:
 * the terms of an entry are cut into ranges, one CTA per range, combined in a fixed order
 * (equal to the reference up to rounding, reproducible run to run).  It needs
 * acro_b200_generic_scratch_bytes(desc) bytes of 256-byte aligned device scratch (0 for the
 * one-thread-per-entry variant, which accepts scratch = NULL); calls sharing one scratch
 * buffer must not overlap on the device. */
int acro_b200_generic_uses_wide_kernel(const acro_b200_generic_desc *desc);
size_t acro_b200_generic_scratch_bytes(const acro_b200_generic_desc *desc);
/* Other shapes with 2..5 inputs whose offsets fit 31 bits run a register-blocked variant when
 * some outer loop is not carried by every input: a thread owns 2..5 output entries along that
 * loop, loads the inputs without it once for all of them, and multiplies the leading inputs
 * without the innermost contracted index once per pass of that index (what the reference's
 * generator gets from its shared-memory preloads and hoisted loops,
 * exec/CudaExecutor.cpp:193-375).  Operation order per entry is unchanged: bit-identical
 * results.  Returns the entries per thread (1 = not blocked) and, in *loop, the blocked loop. */
int acro_b200_generic_blocking(const acro_b200_generic_desc *desc, int *loop);

/*
 * permute: out (op)= the single input with its indices in another order ("A_i_j = B_j_i").  The descriptor is
 * the generic one with no contracted loop (n_outer = n_loops, n_inputs = 1, every loop carried by both
 * tensors).  Used when the fastest index of the input is not the fastest index of the output: 64 x 64 tiles
 * over those two indices go through shared memory, so that loads and stores are both contiguous.  The
 * reference's generator copies entry by entry (exec/CudaExecutor.cpp:520-604), strided on one side.
 */
int acro_b200_permute_supported(const acro_b200_generic_desc *desc);
int acro_b200_permute(const acro_b200_generic_desc *desc, double *out, const double *in, void *stream);

/*
 * reduce_batch:  out[f] (op)= sum_{n<rows} A[n*F + f] * (w ? w[n] : 1),  f < F.
 * The contracted batch index is the slowest dimension of A (README kernel
 * "S_i_j = A_n_i_j B_n").  Streams A once (8*F + 8 bytes per row), keeps
 * per-thread partial sums, and combines them in a fixed order, so results are
 * reproducible run to run.  `scratch` is device memory of at least
 * acro_b200_reduce_batch_scratch_bytes(F) bytes that the call may overwrite;
 * calls sharing one scratch buffer must not overlap on the device.
 * Replaces the generated kernel (one 64-thread block for this shape,
 * exec/CudaExecutor.cpp:193-204).
 */
size_t acro_b200_reduce_batch_scratch_bytes(int F);
int acro_b200_reduce_batch_supported(int64_t rows, int F);
int acro_b200_reduce_batch(const double *A, const double *w, double *out, int64_t rows, int F,
                           int op, double *scratch, size_t scratch_bytes, void *stream);

/*
 * Peer groups: the ranks (one process per GPU of one node) that hold slabs of a contracted
 * batch index.  No counterpart in the reference, which is single-GPU (it is hard-wired to
 * device 0, exec/CudaExecutor.cpp:21, util/CudaUtil.hpp:105).
 *   create   allocates this rank's mailbox on the current device and returns its CUDA IPC handle
 *            (ACRO_B200_IPC_HANDLE_BYTES bytes) to be exchanged by the host program
 *            (MPI, torch.distributed ...);
 *   connect  takes the world * ACRO_B200_IPC_HANDLE_BYTES handle bytes of all ranks, in rank order,
 *            and maps the peers' mailboxes (NVLink peer access); world = 1 needs no connect.
 * acro_b200_reduce_batch_allreduce is reduce_batch over this rank's rows followed, in the same
 * kernel, by the sum over all ranks: each rank stores its F totals into every rank's mailbox and
 * waits (bounded, on its own memory) for the others; every rank gets bit-identical results.
 * All ranks must issue the same sequence of calls.
 */
typedef struct acro_b200_peer_group acro_b200_peer_group;
int acro_b200_peer_group_create(int world, int rank, acro_b200_peer_group **out, unsigned char *handle_out);
int acro_b200_peer_group_connect(acro_b200_peer_group *group, const unsigned char *all_handles);
int acro_b200_peer_group_destroy(acro_b200_peer_group *group);
int acro_b200_peer_group_world(const acro_b200_peer_group *group);
int acro_b200_peer_group_is_connected(const acro_b200_peer_group *group);
int acro_b200_reduce_batch_allreduce(const double *A, const double *w, double *out, int64_t rows, int F, int op,
                                     double *scratch, size_t scratch_bytes, acro_b200_peer_group *group,
                                     void *stream);
/* The all-reduce on its own, for results any other kernel family left on each rank:
 * dst[i] (op)= sum over the ranks of src[i], i < n (src == dst allowed).  One small kernel; the entries
 * travel through the mailboxes in exchanges of at most 4096 (results of up to 256 entries in the form
 * the fused exchange of acro_b200_reduce_batch_allreduce uses, so a rank may make either call for the
 * same result), summed in rank order (bit-identical on every rank).  Every wait is bounded (about half
 * a second): an absent rank shows as ACRO_B200_ETIMEOUT in
 * acro_b200_device_status() and the result is then invalid.  All ranks must make the same sequence of
 * calls, with the same n, on this group. */
int acro_b200_peer_allreduce(double *dst, const double *src, int64_t n, int op, acro_b200_peer_group *group,
                             void *stream);

/*
 * reduce_batch without any allocation.  No counterpart in the reference.
 * Some callers cannot obtain device memory at the point where they need this reduction:
 * a plug-in inside an application that owns the whole device memory pool and forbids
 * allocations in its time-step loop, an in-situ component whose memory budget was fixed at
 * start-up, or a host library that is handed device pointers but must not call cudaMalloc
 * itself (an allocation can synchronise the whole device).  For them the partial sums and the ticket
 * counter live in a static device array inside the library (524,544 bytes per GPU, kept
 * until the process exits) instead of a caller-provided scratch buffer; inputs and the
 * output are still the caller's.  Limits and rules:
 *   - rows of at most acro_b200_reduce_batch_noalloc_max_f() = 32 entries, otherwise
 *     ACRO_B200_EUNSUPPORTED (use acro_b200_reduce_batch with your own scratch);
 *   - the first call on each device looks up the array's device address (a one-time
 *     set-up, done with that device current); make that call before any stream capture.
 *     The address belongs to the CUDA context that was current then: after
 *     acro_b200_set_context the next call on each device is a first call again;
 *   - every call on a GPU shares the one array, so calls that overlap on that GPU race:
 *     keep them on one stream or order them yourself.
 * Results are identical to acro_b200_reduce_batch's.
 */
int acro_b200_reduce_batch_noalloc_max_f(void);
int acro_b200_reduce_batch_noalloc(const double *A, const double *w, double *out, int64_t rows, int F,
                                   int op, void *stream);

/*
 * pointwise_sym:  D[p,m,n] (op)= s[p] * sum_{l<dim} X[p,m,l] * Y[p,n,l],   m,n,l < dim,
 * where s[p] is the left-to-right product of n_scalars point-wise factors
 * (diffusion geometric factors "D_e_k_m_n = W_k DetJ_e_k Jinv_e_k_m_l Jinv_e_k_n_l").
 * A point p is a tuple over n_point_loops leading loops with extents
 * point_extent[]; scalar factor i sits at sum_j idx[j]*scalar_step[i][j].
 * X, Y and D hold dim*dim contiguous doubles per point.  Arithmetic follows the
 * reference order term by term, without fused multiply-add (bit-identical for "=").
 */
#define ACRO_B200_MAX_POINT_LOOPS 6
#define ACRO_B200_MAX_SCALARS 6
typedef struct acro_b200_pointwise_desc
{
    int32_t dim;
    int32_t op;
    int32_t n_point_loops;
    int32_t n_scalars;
    int64_t point_extent[ACRO_B200_MAX_POINT_LOOPS];
    int64_t scalar_step[ACRO_B200_MAX_SCALARS][ACRO_B200_MAX_POINT_LOOPS];
    /* Output layout.  cell_points = 1: D holds the dim*dim block of each point contiguously
     * (D_e_k_m_n).  cell_points = K > 1: the last point loops (K points, a "cell") come AFTER
     * the block indices, D[cell][m][n][k] (D_e_m_n_k1_k2_k3, the layout of the reference's own
     * partial-assembly tests, unittest/kernel/test_TensorEngine.cpp:498-590); the point
     * count must be a multiple of K.  X and Y are point-major in both cases. */
    int64_t cell_points;
    /* 0: D[m][n] = sum_l (s X[m][l]) Y[n][l];  1: the string lists the n-operand first,
     * D[m][n] = sum_l (s X[n][l]) Y[m][l] (same values up to rounding, different term order). */
    int32_t swapped;
    int32_t reserved;
} acro_b200_pointwise_desc;

int acro_b200_pointwise_sym_supported(const acro_b200_pointwise_desc *desc);
int acro_b200_pointwise_sym(const acro_b200_pointwise_desc *desc, const double *const *scalars,
                            const double *X, const double *Y, double *D, void *stream);

/*
 * rank1_gemm:  M[e,i,j] (op)= sum_{q<Q} W[e,q] * B1[q,i] * B2[q,j]   (batched element mass matrices,
 * "M_e_i_j = W_e_q B_q_i B_q_j").  One GEMM  [elements x Q] * [Q x ni*nj]  whose right operand
 * B1[q,i]*B2[q,j] is formed on the fly; fp64 tensor cores (mma.sync m8n8k4).  Instantiated
 * for Q up to 64 (processed in steps of four, zero-padded on chip) and ni, nj <= 32.  HBM traffic 8*(Q + ni*nj) bytes per element, 2*Q*ni*nj flops.
 * Replaces the generated kernel (one block per element, serial 64-term sums per thread,
 * exec/CudaExecutor.cpp:193-204,520-523).
 */
int acro_b200_rank1_gemm_supported(int q, int ni, int nj);
int acro_b200_rank1_gemm(const double *W, const double *B1, const double *B2, double *M, int64_t elements,
                         int q, int ni, int nj, int op, void *stream);

/*
 * batched_gemm:  C[e,i,j] (op)= sum_{k} A[e,i,k] * B[e,k,j]  for a batch of dense row-major
 * matrices ("C_e_i_j = A_e_i_k B_e_k_j"), any m, n, k (above 64: acro_b200_gemm_batched).  64^3 and 32^3: persistent CTAs,
 * three-stage asynchronous copy ring for A_e and B_e, fp64 tensor cores; other sizes above 16 use
 * the same kernel with the matrices zero-padded on chip to 32 or 64.  Every m, n, k <= 16 is
 * HBM-bound: tiles of matrices streamed through shared memory by bulk copies, separate multiply
 * and add in ascending k, bit-identical to the reference's CPU executor.  n = 1 or m = 1 (an element
 * matrix applied to an element vector, "Y_e_i = M_e_i_j X_e_j") takes a streaming matrix-vector kernel
 * whose lanes walk the rows in a rotated order (bank conflicts): within tolerance, not bit-identical.
 * HBM traffic 8*(mk + kn + mn) bytes and 2mnk flops per element.  Replaces the generated kernel
 * (scalar DFMA from global memory, no tiling, exec/CudaExecutor.cpp:520-604).
 */
int acro_b200_batched_gemm_supported(int m, int n, int k);
int acro_b200_batched_gemm(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k,
                           int op, void *stream);
/* The same with either operand stored transposed: trans_a != 0 means A_e is stored k x m
 * ("C_e_i_j = A_e_k_i B_e_k_j"), trans_b != 0 means B_e is stored n x k ("C_e_i_j = A_e_i_k B_e_j_k",
 * e.g. the metric "G_e_m_n = J_e_m_l J_e_n_l").  A transposed operand needs m, n, k <= 64 (the kernels
 * that stage whole matrices in shared memory; only the strides of their shared-memory reads change);
 * the same bit-identity up to 16 and tolerance above as the plain form. */
int acro_b200_batched_gemm_t_supported(int m, int n, int k, int trans_a, int trans_b);
/* 1 when products of this shape travel as PAIRS of elements by bulk copy (sizes 17 .. 32 whose stored rows have an odd
 * length, operands on 16-byte boundaries) instead of through the zero-padded ring; for plan descriptions. */
int acro_b200_batched_gemm_by_pairs(int m, int n, int k, int trans_a, int trans_b);
int acro_b200_batched_gemm_t(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k,
                             int trans_a, int trans_b, int op, void *stream);

/*
 * gram:  S[a,b] (op)= sum_{n} X[n,a] * Y[n,b]  ("S_a_b = X_n_a Y_n_b": normal equations, Gram matrices,
 * moments), a, b <= 64, any number of rows.  X and Y are read once.  a, b <= 16 (bound by HBM): tiles of
 * rows arrive by bulk copies, a thread keeps a 4 x 4 block of S in registers over its share of the rows.
 * Larger: slabs of 32 (64 when a or b exceeds 32) rows go through the batched_gemm ring as products
 * X_slab^T * Y_slab on the fp64 tensor cores and every CTA keeps summing into its accumulators.  Either
 * way a CTA writes one a x b tile of partial sums to `scratch` (acro_b200_gram_scratch_bytes) and a
 * second kernel adds the tiles in ascending order: the same bits on every run on the same device,
 * within tolerance of the reference's sequential sum.
 * HBM traffic 8*(a + b) bytes and 2ab flops per row.  The generated kernel of the reference runs one
 * thread per entry of S over all rows (exec/CudaExecutor.cpp:520-604).
 */
int acro_b200_gram_supported(int a, int b);
size_t acro_b200_gram_scratch_bytes(int a, int b);
int acro_b200_gram(const double *X, const double *Y, double *S, int64_t rows, int a, int b, int op,
                   double *scratch, size_t scratch_bytes, void *stream);

/*
 * gemm:  C[M x N] (op)= A[M x K] * P[K x N], row-major fp64 with leading dimensions lda, ldp, ldc (in
 * doubles), on the fp64 tensor cores: 64 x 64 tiles, K walked in slabs of 64 through a three-slot
 * asynchronous copy ring.  The engine uses it for contractions in which exactly one input carries the
 * batch index and all its other indices are contracted (assembly strings such as
 * "M_e_i1_i2_j1_j2 = B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2"): the batch-invariant inputs are first
 * multiplied out into P by acro_b200_generic_launch.  The reference's generator runs these as scalar
 * loops per output entry (exec/CudaExecutor.cpp:520-604).
 */
int acro_b200_gemm(const double *A, const double *P, double *C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldp,
                   int64_t ldc, int op, void *stream);
/* `batch` independent products of that kind in one launch: element e uses A + e*stride_a, P + e*stride_p and
 * C + e*stride_c (strides in doubles; 0 shares the operand between the elements). */
int acro_b200_gemm_batched(const double *A, const double *P, double *C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                           int64_t ldp, int64_t ldc, int64_t stride_a, int64_t stride_p, int64_t stride_c, int op, void *stream);

/*
 * sumfact_mass: the six-stage sum-factorised 3D mass operator as ONE kernel,
 *   V_e_i1_i2_i3 = sum B_k3_i3 B_k2_i2 B_k1_i1 W_e_k1_k2_k3 (sum B_k1_j1 B_k2_j2 B_k3_j3 U_e_j1_j2_j3),
 * evaluated stage by stage (contract i3, i2, i1, scale by W, contract k1, k2, k3) with every
 * intermediate kept in registers / shared memory.  B is [q][p], U and V are [elements][p][p][p],
 * W is [elements][q][q][q]; instantiated for (p, q) = (2,3), (2,4), (3,4), (3,5), (4,5), (4,6), (5,6).  HBM traffic:
 * 8*(2p^3 + q^3) bytes per element.  Replaces the
 * reference's fused multi-kernel launch (exec/CudaExecutor.cpp:69-102,286-323), which still
 * writes every intermediate tensor to global memory (:536).
 */
int acro_b200_sumfact_mass_supported(int p, int q);
int acro_b200_sumfact_mass(const double *B, const double *U, const double *W, double *V,
                           int64_t elements, int p, int q, void *stream);

/*
 * Batched inverse and/or determinant of `count` dense dim x dim matrices (dim = 1, 2, 3), each
 * dim*dim contiguous doubles.  Ainv or Adet may be NULL (not both); Ainv may alias A.  Same
 * formulas, operation by operation, as the reference's CPU ops (ops/NativeCPUOps.hpp:38-86):
 * bit-identical results, including its 3x3 convention of storing entry (r,c) of the inverse
 * at position (c,r).  Replaces the CudaInv.., CudaDet.. and CudaInvDet.. kernels (ops/CudaGPUOps.cpp:108-275).
 */
int acro_b200_batch_inv_det(const double *A, double *Ainv, double *Adet, int64_t count, int dim, void *stream);

/* Aout[i] = Ain[map[i]], i < range_size.  Replaces CudaScatter (ops/CudaGPUOps.cpp:278-285). */
int acro_b200_flat_scatter(double *Aout, const double *Ain, const int *map, int64_t range_size, void *stream);

/* Aout[d] = sum over k in [inv_offsets[d], inv_offsets[d+1]) of Ain[inv_map[k]], d < domain_size:
 * the inverse map in CSR form, summed in ascending position (the reference CPU order), no
 * atomics.  Replaces CudaSumGather (ops/CudaGPUOps.cpp:288-302). */
int acro_b200_flat_sum_gather(double *Aout, const double *Ain, const int *inv_map, const int *inv_offsets,
                              int64_t domain_size, void *stream);

/*
 * Shared-entry exchange for a sharded FlatIndexedSumGather.  No counterpart in the reference,
 * which is single-GPU.  The range of an IndexMapping (element-local entries) is cut into one
 * slab per rank (one process per GPU of one node); after acro_b200_flat_sum_gather over its own
 * slab a rank holds partial sums, and the domain entries reached from several ranks' slabs must
 * be summed over those ranks.
 *   mark_touched  host helper: bitmap ((domain_size + 7) / 8 bytes, bit d = some map value equals d)
 *   create        takes the world bitmaps in rank order (exchanged by the host program), derives which
 *                 entries this rank shares with which ranks and every rank's inbox layout; with
 *                 on_device = 1 it also allocates this rank's inbox on the current device and returns
 *                 its CUDA IPC handle.  on_device = 0 makes a host-side plan only (no CUDA call) whose
 *                 arrays copy_plan returns: for shared entry k (domain position shared_idx[k], ascending),
 *                 pairs entry_off[k] .. entry_off[k+1]-1 name the other ranks reaching it (entry_peer,
 *                 ascending), the slot this rank writes in that rank's inbox (entry_send) and the slot of
 *                 its own inbox where that rank's value arrives (entry_recv).
 *   connect       maps the other ranks' inboxes from their IPC handles (world * ACRO_B200_IPC_HANDLE_BYTES
 *                 bytes, rank order); connect_pointers does the same from device pointers for ranks that
 *                 live in one process (acro_b200_halo_inbox gives a rank's own pointer).
 *   send          stores this rank's value of every shared entry into the inboxes of the ranks sharing it
 *                 (remote stores over NVLink peer mappings) and publishes the call's sequence number;
 *   combine       waits (bounded; a wait that gives up shows in acro_b200_device_status) for the ranks it
 *                 shares entries with and replaces every shared entry of `values` by the sum over all
 *                 sharing ranks in ascending rank order, so every rank holds identical bits.
 *   exchange_sum  = send, then combine, on the same stream.
 * All ranks must issue the same sequence of send/combine calls; ranks of ONE process sharing a GPU must
 * launch every send before the first combine on one stream, so that no kernel waits for a later one.
 */
typedef struct acro_b200_halo acro_b200_halo;
int acro_b200_halo_mark_touched(const int *map, int64_t range_size, int64_t domain_size, unsigned char *bitmap);
int acro_b200_halo_create(int world, int rank, int64_t domain_size, const unsigned char *all_bitmaps, int on_device,
                          acro_b200_halo **out, unsigned char *handle_out);
int acro_b200_halo_counts(const acro_b200_halo *halo, int64_t *shared_entries, int64_t *sharing_pairs, int64_t *inbox_doubles);
int acro_b200_halo_copy_plan(const acro_b200_halo *halo, int *shared_idx, int *entry_off, int *entry_peer, int *entry_send,
                             int *entry_recv);
int acro_b200_halo_connect(acro_b200_halo *halo, const unsigned char *all_handles);
void *acro_b200_halo_inbox(const acro_b200_halo *halo);
int acro_b200_halo_connect_pointers(acro_b200_halo *halo, void *const *inboxes);
int acro_b200_halo_send(acro_b200_halo *halo, const double *values, void *stream);
int acro_b200_halo_combine(acro_b200_halo *halo, double *values, void *stream);
int acro_b200_halo_exchange_sum(acro_b200_halo *halo, double *values, void *stream);
int acro_b200_halo_destroy(acro_b200_halo *halo);

/* ---------------------------------------------------------------- engine layer */

typedef struct acro_tensor acro_tensor;   /* an acro::Tensor */
typedef struct acro_engine acro_engine;   /* an acro::TensorEngine */
typedef struct acro_index_mapping acro_index_mapping;   /* an acro::IndexMapping */

/* Tensor(dims, hdata, ddata, ongpu), tensor/Tensor.hpp:19-42.  hdata NULL = library-owned host buffer. */
int acro_tensor_create(int rank, const int *dims, double *hdata, double *ddata, int ongpu, acro_tensor **out);
/* SliceTensor(parent, i0, ...), tensor/SliceTensor.hpp:14-57.  The parent must outlive the slice. */
int acro_tensor_slice(acro_tensor *parent, int n_indices, const int *indices, acro_tensor **out);
int acro_tensor_destroy(acro_tensor *t);
int acro_tensor_rank(const acro_tensor *t);
int64_t acro_tensor_size(const acro_tensor *t);
int acro_tensor_dim(const acro_tensor *t, int d);
double *acro_tensor_data(const acro_tensor *t);         /* GetData */
double *acro_tensor_device_data(const acro_tensor *t);  /* GetDeviceData */
int acro_tensor_is_on_gpu(const acro_tensor *t);
int acro_tensor_is_mapped_to_gpu(const acro_tensor *t);
int acro_tensor_map_to_gpu(acro_tensor *t);
int acro_tensor_move_to_gpu(acro_tensor *t);
int acro_tensor_switch_to_gpu(acro_tensor *t);
int acro_tensor_unmap_from_gpu(acro_tensor *t);
int acro_tensor_move_from_gpu(acro_tensor *t);
int acro_tensor_switch_from_gpu(acro_tensor *t);
int acro_tensor_set(acro_tensor *t, double val);
int acro_tensor_mult(acro_tensor *t, double c);
int acro_tensor_reshape(acro_tensor *t, int rank, const int *dims);
int acro_tensor_retarget(acro_tensor *t, double *hdata, double *ddata);
int acro_tensor_set_transient(acro_tensor *t, int transient);

/* Multi-GPU, one process per GPU (no counterpart in the reference, which is single-device,
 * exec/CudaExecutor.cpp:21).  acro_b200_batch_slab: the range [*begin, *end) of a batch index of
 * extent `batch` that rank `rank` of `world` owns (contiguous, rank order, sizes differing by at most
 * one; host arithmetic only, acro::SlabOf).  acro_tensor_slab: rows [begin, end) of the leading
 * dimension of `parent` as a tensor that shares the parent's host buffer, owns a device mirror of the
 * slab only and is flagged sharded (acro::SlabTensor; offset arithmetic as tensor/SliceTensor.cpp:142-168).
 * acro_tensor_set_sharded: flags a tensor the caller built per rank as such a slab (Tensor::SetSharded). */
int acro_b200_batch_slab(int64_t batch, int rank, int world, int64_t *begin, int64_t *end);
int acro_tensor_slab(acro_tensor *parent, int64_t begin, int64_t end, acro_tensor **out);
int acro_tensor_set_sharded(acro_tensor *t, int sharded);
int acro_tensor_is_sharded(const acro_tensor *t);

/* TensorEngine(exec_type), kernel/TensorEngine.cpp:27-48. */
int acro_engine_create(const char *exec_type, acro_engine **out);
int acro_engine_destroy(acro_engine *e);
int acro_engine_set_executor_type(acro_engine *e, const char *exec_type);
int acro_engine_exec_type(acro_engine *e, char *buf, size_t buf_len);
/* TE(kernel, out, inputs), kernel/TensorEngine.cpp:290-315. */
int acro_engine_contract(acro_engine *e, const char *kernel, acro_tensor *out, int n_inputs,
                         acro_tensor *const *inputs);
/* GetImplementation(kernel, out, inputs); the text is truncated to buf_len-1 characters. */
int acro_engine_implementation(acro_engine *e, const char *kernel, acro_tensor *out, int n_inputs,
                               acro_tensor *const *inputs, char *buf, size_t buf_len);
/* BeginMultiKernelLaunch / EndMultiKernelLaunch, kernel/TensorEngine.cpp:318-336. */
int acro_engine_begin_multi(acro_engine *e);
int acro_engine_end_multi(acro_engine *e);
/* Ends the recording and returns the description of the fused plan instead of running it. */
int acro_engine_end_multi_describe(acro_engine *e, char *buf, size_t buf_len);
int acro_engine_clear(acro_engine *e);
/* Attach (or detach with NULL) a peer group: from then on a contraction that sums over the leading
 * index of an input flagged sharded (acro_tensor_slab, acro_tensor_set_sharded) returns, on every
 * rank, the sum over all ranks' slabs: inside the kernel for the reduce_batch family, through
 * acro_b200_peer_allreduce after the step for every other family.  Every rank of the group must
 * make the same sequence of such calls.  The engine does not own the group. */
int acro_engine_set_peer_group(acro_engine *e, acro_b200_peer_group *group);
/* cudaStream_t as void*; applies to later launches of this engine. */
int acro_engine_set_stream(acro_engine *e, void *stream);
/* IndexMapping(domain_size, range_size), tensor/IndexMapping.hpp:14-48.  acro_index_mapping_data
 * returns the host array of range_size ints to fill with M[i] in [0, domain_size). */
int acro_index_mapping_create(int domain_size, int range_size, acro_index_mapping **out);
int acro_index_mapping_destroy(acro_index_mapping *m);
int *acro_index_mapping_data(acro_index_mapping *m);
int acro_index_mapping_compute_inverse(acro_index_mapping *m);
/* Host arrays of the inverse (range_size and domain_size+1 ints); NULL before it is computed. */
const int *acro_index_mapping_inverse(acro_index_mapping *m);
const int *acro_index_mapping_inverse_offsets(acro_index_mapping *m);

/* BatchMatrixInverse / BatchMatrixDet / BatchMatrixInvDet, kernel/TensorEngine.cpp:627-690: the
 * last two dimensions of A are the (square, <= 3) matrix, the leading ones the batch. */
int acro_engine_batch_matrix_inverse(acro_engine *e, acro_tensor *Ainv, acro_tensor *A);
int acro_engine_batch_matrix_det(acro_engine *e, acro_tensor *Adet, acro_tensor *A);
int acro_engine_batch_matrix_inv_det(acro_engine *e, acro_tensor *Ainv, acro_tensor *Adet, acro_tensor *A);
/* FlatIndexedScatter / FlatIndexedSumGather, kernel/TensorEngine.cpp:693-716. */
int acro_engine_flat_indexed_scatter(acro_engine *e, acro_tensor *Aout, acro_tensor *Ain, acro_index_mapping *m);
int acro_engine_flat_indexed_sum_gather(acro_engine *e, acro_tensor *Aout, acro_tensor *Ain, acro_index_mapping *m);
/* The same over this rank's slab of the range, followed by the sum of the shared domain entries over the
 * ranks (acro_b200_halo_exchange_sum); `halo` was created from the touched-entry bitmaps of all ranks. */
int acro_engine_flat_indexed_sum_gather_shared(acro_engine *e, acro_tensor *Aout, acro_tensor *Ain, acro_index_mapping *m,
                                               acro_b200_halo *halo);

/* Stream used by the calling host thread's tensor copies / fills and by engines without their
 * own stream (per thread; NULL = legacy default stream). */
int acro_b200_set_stream(void *stream);

/* Host-only introspection (no device needed): a text dump of the parser's view of a
 * kernel string — variables, AllIndexNames, ContractionIndexNames
 * (kernel/TensorKernel.cpp:28-67).  Fails with ACRO_B200_EINVAL on a grammar error. */
int acro_b200_describe_kernel(const char *kernel, char *buf, size_t buf_len);
/* Host-only: bind a group of kernels to extents (no data needed) and describe the plan the
 * "Cuda" back end would run: loop order, shared-outer loops, unique variables, chosen
 * family per step.  dims_flat holds, per kernel, the output dims then each input's dims. */
int acro_b200_describe_plan(int n_kernels, const char *const *kernels, const int *dims_flat,
                            int transient_intermediates, char *buf, size_t buf_len);

#ifdef __cplusplus
}
#endif

#endif /* ACRO_B200_H */

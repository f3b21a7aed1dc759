/* tpb200 -- C ABI of the sm_100a reduction and top-k kernels.
 *
 * This is the boundary a TensorPlay build binds to replace the CUDA kernels that
 * p10/src/backend/cuda/ReductionKernels.cu registers for DispatchKey::CUDA (registration block
 * at ReductionKernels.cu:385-418).  Plain pointers and sizes only; no TensorPlay, PyTorch or C++
 * types cross it.  The C++ adapter that wraps these calls into kernels with the exact
 * signatures TensorPlay's DispatchStub expects lives in tensorplay_b200/csrc/adapter/.
 *
 * Conventions
 *   - All data pointers are device pointers on the CUDA device that is current at the call.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, which is
 *     where the reference launches everything: ReductionKernels.cu:86-95).
 *   - Calls only enqueue work; they never synchronise and never allocate device memory.
 *     Scratch memory is the caller's: ask tpb200_*_workspace_bytes(), pass a buffer of at
 *     least that size (256-byte aligned).  Its contents need no initialisation.
 *   - sizes/strides are in ELEMENTS, as in TensorImpl (p10/include/TensorImpl.h:87-98);
 *     `in` points at the first element (storage offset already applied).  Any strided view
 *     is accepted; no copy is made.
 *   - Outputs are written contiguously over the kept dims in their original order
 *     (keepdim only changes the shape the caller reports, not the layout).
 *   - Every function returns TPB200_OK or an error code, never throws, never aborts;
 *     tpb200_last_error() gives the message of the calling thread's last failure.
 *   - Supported element type: float32 (TPB200_F32).  Other dtypes return
 *     TPB200_ERR_UNSUPPORTED so that an adapter can fall through to the kernel registered
 *     before it.
 */
#ifndef TPB200_H_
#define TPB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TPB200_VERSION 100

/* error codes */
#define TPB200_OK 0
#define TPB200_ERR_INVALID 1      /* bad argument: message says which                          */
#define TPB200_ERR_UNSUPPORTED 2  /* dtype / rank not handled by these kernels                 */
#define TPB200_ERR_DIM_RANGE 3    /* "Dimension out of range" (ReductionKernels.cpp:55-57)     */
#define TPB200_ERR_EMPTY 4        /* "max(): Expected reduction dim to be non-empty" (:240)    */
#define TPB200_ERR_WORKSPACE 5    /* workspace missing or too small                            */
#define TPB200_ERR_CUDA 6         /* a CUDA runtime call failed: "CUDA Error: ..."             */

/* dtypes */
#define TPB200_F32 0

/* reduction operators.  The first eight replace, one to one, the kernels registered at
 * ReductionKernels.cu:386-391 and :410-417; the two fused forms serve callers that want
 * torch-style (values, indices) from one pass (the reference needs max.dim + argmax). */
#define TPB200_OP_SUM 0        /* sum, sum.dim_IntList        ReductionKernels.cu:227-238 */
#define TPB200_OP_MEAN 1       /* mean, mean.dim              ReductionKernels.cu:241-253 */
#define TPB200_OP_VAR 2        /* var, var.dim                ReductionKernels.cu:358-374 */
#define TPB200_OP_STD 3        /* std, std.dim                ReductionKernels.cu:376-382 */
#define TPB200_OP_MAX 4        /* max, max.dim (values only)  ReductionKernels.cu:270-281 */
#define TPB200_OP_MIN 5        /* min, min.dim (values only)  ReductionKernels.cu:284-293 */
#define TPB200_OP_ARGMAX 6     /* argmax                      ReductionKernels.cu:31-117  */
#define TPB200_OP_ARGMIN 7     /* argmin                      ReductionKernels.cu:119-121 */
#define TPB200_OP_MAX_ARGMAX 8 /* values + indices in one pass */
#define TPB200_OP_MIN_ARGMIN 9
/* The other operators of the same registration block (ReductionKernels.cu:256-267, 296-345,
 * 392-408).  tpb200_reduce only; float32 in.  PROD and the norms write float32; ALL and ANY write
 * one byte per output element (the reference's Bool tensor: 1 = true). */
#define TPB200_OP_PROD 10         /* prod, prod.dim_IntList                                   */
#define TPB200_OP_NORM1 11        /* norm(p = 1): sum |x|                                     */
#define TPB200_OP_NORM2 12        /* norm(p = 2): sqrt(sum x^2)  (the one p the reference's CUDA path has) */
#define TPB200_OP_NORM_INF 13     /* norm(p = +inf): max |x|                                  */
#define TPB200_OP_NORM_NEG_INF 14 /* norm(p = -inf): min |x|                                  */
#define TPB200_OP_ALL 15          /* all, all.dim: every element != 0 (NaN counts as true)    */
#define TPB200_OP_ANY 16          /* any, any.dim                                             */

#define TPB200_MAX_DIMS 8

/* Size of one packed partial record (see tpb200_reduce_partial). */
#define TPB200_PARTIAL_BYTES 40

const char* tpb200_last_error(void);
int tpb200_version(void);

/* ---- reductions over a dim, several dims, or the whole tensor ---------------------------------
 * Replaces cuda::{sum,mean,max,min,var,std}[_dim]_kernel and arg_reduce_kernel
 * (ReductionKernels.cu:54-121, 128-293, 348-382).
 *
 *   reduce_mask   bit d set = dim d is reduced; 0 = reduce every dim (the overloads without a
 *                 dim argument, and an empty dim list)
 *   index_dim     for ARGMAX/ARGMIN/fused: -1 = position in the flattened (row-major) tensor,
 *                 as argmax(dim=None) returns; otherwise reduce_mask must be exactly that one
 *                 dim and the position along it is returned
 *   correction    var/std: divisor is max(0, n - correction) (ReductionKernels.cu:364-365)
 *   out_val       float32 results (NULL for ARGMAX/ARGMIN)
 *   out_idx       int64 results (NULL unless the op returns indices)
 *
 * Semantics follow the reference's CPU kernels (p10/src/backend/cpu/ReductionKernels.cpp):
 * first occurrence wins ties, NaN is never selected by max/min/argmax/argmin, sums are
 * accumulated in float64 and rounded once.
 */
int tpb200_reduce(int op, const void* in, int dtype, int ndim, const int64_t* sizes,
                  const int64_t* strides, uint64_t reduce_mask, int index_dim, int64_t correction,
                  void* out_val, int64_t* out_idx, void* workspace, size_t workspace_bytes,
                  void* stream);

size_t tpb200_reduce_workspace_bytes(int op, int dtype, int ndim, const int64_t* sizes,
                                     const int64_t* strides, uint64_t reduce_mask);

/* ---- top-k along one dim ----------------------------------------------------------------------
 * New operator (the reference declares none): schema
 *   topk(Tensor self, int64_t k, int64_t dim=-1, bool largest=true, bool sorted=true)
 *        -> (Tensor values, Tensor indices)
 * Contract: the first k entries of each row stably sorted by value (descending if largest,
 * else ascending), ties in ascending index -- the tie rule of the reference's argmax/argmin
 * scan (ReductionKernels.cpp:727-735, 793-801), so k = 1 equals argmax/argmin.  -0.0 ties with
 * +0.0; NaN ranks after every number in both directions; values are returned bit-exact.
 * sorted = 0 may return the same k entries in any order (this implementation returns them sorted).
 * out_val / out_idx are written contiguously as [non-selected dims in their original order..., k]:
 * for dim = last that is the input's shape with dim replaced by k; for another dim the caller
 * reports the result as a permuted view.  The non-selected dims must collapse to at most two
 * strided dims; k <= 2048, or any k on rows of at most 16384 elements; rows * slices per row must
 * stay below 2^31 (rows ride on grid.x).
 * Long rows (32 K elements and more) go through a kernel that fixes its threshold from a sample of
 * the row and verifies it afterwards; rows that fail the check (sorted rows, rows of equal values,
 * rows with fewer than k numbers) are redone by a second launch that needs no assumption.  The
 * result is exact either way; only the time depends on the data.
 */
int tpb200_topk(const void* in, int dtype, int ndim, const int64_t* sizes, const int64_t* strides,
                int dim, int64_t k, int largest, int sorted, void* out_val, int64_t* out_idx,
                void* workspace, size_t workspace_bytes, void* stream);

size_t tpb200_topk_workspace_bytes(int dtype, int ndim, const int64_t* sizes, const int64_t* strides,
                                   int dim, int64_t k);

/* What the planner chose for a top-k call (no launch, no GPU needed); for benchmarks and tests.
 * No reference counterpart.  info[0..n_info) receives, in this order:
 *   0 scanning kernel (0 none, 1 whole-row sort, 2 rendezvous kernel, 3 ring kernel, 4 warp per row)
 *   1 its slices per row            2 its warps per CTA
 *   3 1 if the sampled-threshold kernel runs first    4 its CTAs per row (cluster size)
 *   5 its warps per CTA             6 rank of the threshold key in the sample
 *   7 candidate words per row       8 sample tiles per warp
 *   9 kernel launches of one call   10 workspace bytes
 */
#define TPB200_PLAN_INFO_FIELDS 11
int tpb200_topk_plan_info(int dtype, int ndim, const int64_t* sizes, const int64_t* strides, int dim,
                          int64_t k, int64_t* info, int n_info);

/* ---- softmax / log_softmax along one dim --------------------------------------------------------
 * Replaces softmax_kernel_cudnn / log_softmax_kernel_cudnn (p10/src/backend/cuda/ActivationKernels.cu:
 * 136-181: cudnnSoftmaxForward on a 4-D padded descriptor with int dims); schema
 *   softmax(Tensor self, int64_t dim, DType dtype=Undefined) -> Tensor      (native_functions.yaml:587-597)
 * Arithmetic as the reference's CPU kernels (p10/src/backend/cpu/PointwiseKernels.cpp:519-546):
 * m = max over dim (NaN never the maximum), e = exp(x - m), s = sum e; softmax = e / s,
 * log_softmax = (x - m) - log s; no special cases, so NaN, +inf and all -inf rows give NaN where that
 * chain of float operations does.  `out` is contiguous, same shape as the input.
 * dim = last with unit stride: any strided view whose other dims collapse to at most two; any other
 * dim: the tensor must be contiguous.  Other layouts return TPB200_ERR_UNSUPPORTED.  No workspace.
 */
int tpb200_softmax(int log, const void* in, int dtype, int ndim, const int64_t* sizes,
                   const int64_t* strides, int dim, void* out, void* stream);

/* ---- median of the whole tensor ---------------------------------------------------------------
 * The reference has a CPU kernel only (p10/src/backend/cpu/ReductionKernels.cpp:874-901; schema
 * median(Tensor self) -> Tensor, native_functions.yaml:796-799): element (n - 1) / 2 of the sorted
 * values, i.e. the lower middle one for even n; NaN for an empty tensor.  Here NaNs rank after all
 * numbers (the reference's std::nth_element leaves their place undefined); -0.0 and +0.0 are one
 * value and +0.0 is returned for it.  `out` receives one float32.  Any strided view; the workspace
 * (tpb200_median_workspace_bytes(), about 4 MB: the selection state and a buffer for the elements
 * around the median; 8-byte aligned) needs no initialisation.
 */
int tpb200_median(const void* in, int dtype, int ndim, const int64_t* sizes, const int64_t* strides,
                  void* out, void* workspace, size_t workspace_bytes, void* stream);
size_t tpb200_median_workspace_bytes(void);

/* ---- strided copy ------------------------------------------------------------------------------
 * dst[i0, i1, ...] = src[i0, i1, ...] for two views of the same shape (sizes) with their own strides,
 * 4-byte elements (TPB200_F32; the bits are copied, so int32 data works as well).  Replaces
 * copy_cast_kernel_impl (p10/src/backend/cuda/CopyKernels.cu:42-53, launched at :105-156: one element
 * per thread, a div/mod chain over every dim on both sides) for what callers do around reductions:
 * permute().contiguous(), transposes, slices (ReductionKernels.cu:67-75, 143).  Coalesced on both sides
 * whenever each view has a unit stride somewhere (shared-memory tiles when those are different dims).
 * The views must not overlap each other; dst must not overlap itself (no zero strides in dst).
 */
int tpb200_strided_copy(void* dst, const int64_t* dst_strides, const void* src, const int64_t* src_strides,
                        int dtype, int ndim, const int64_t* sizes, void* stream);

/* ---- sharded whole-tensor reductions: per-GPU partial, then a rank-ordered combine ------------
 * No reference counterpart (the reference is single-GPU: p10/src/backend/cuda/CUDAAllocator.cpp:87-88).
 *
 * tpb200_reduce_partial reduces `n` contiguous floats -- this GPU's flat partition, which starts
 * at element `global_offset` of the whole tensor -- to ONE packed record of TPB200_PARTIAL_BYTES
 * written at `partial_out` (device memory; typically the slot of this rank in the all-gather
 * buffer, so the kernel's output is the collective's input with no copy between).
 *   family:  TPB200_OP_SUM (also serves MEAN), TPB200_OP_VAR (also STD),
 *            TPB200_OP_MAX_ARGMAX (also MAX, ARGMAX), TPB200_OP_MIN_ARGMIN (also MIN, ARGMIN)
 * Record layout (little endian): double d0, d1, d2; int64 i0; float f0; uint32 pad
 *   sum: d0 = sum | var: d0 = count, d1 = mean, d2 = M2 | extremum: f0 = value, i0 = GLOBAL position
 *
 * tpb200_reduce_combine merges `n_parts` records in index order (deterministic, independent of
 * which rank runs it) and writes the result of `op` (any of the ten operators) for a tensor of
 * `total_count` elements.
 */
int tpb200_reduce_partial(int family, const void* in, int dtype, int64_t n, int64_t global_offset,
                          void* partial_out, void* workspace, size_t workspace_bytes, void* stream);

size_t tpb200_reduce_partial_workspace_bytes(int family, int dtype, int64_t n);

int tpb200_reduce_combine(int op, const void* partials, int n_parts, int64_t total_count,
                          int64_t correction, void* out_val, int64_t* out_idx, void* stream);

/* ---- fused partial + exchange over peer memory (NVLink) ----------------------------------------
 * No reference counterpart.  The same result as tpb200_reduce_partial -> all-gather ->
 * tpb200_reduce_combine without a library collective: after the slice kernel, a one-warp kernel
 * merges the slices and writes this rank's record straight into the exchange buffer of every rank
 * (peer-to-peer stores; no multicast), raises an epoch flag and waits -- bounded -- for the flags
 * of all ranks before merging the `world` records in rank order.
 *   peer_buffers  host array of `world` device pointers: the exchange buffer of every rank as
 *                 mapped on THIS GPU (peer_buffers[rank] is this rank's own); each buffer has
 *                 tpb200_exchange_buffer_bytes() bytes and is zero-filled once before the first call
 *   n / global_offset / total_count   this rank's flat partition and the size of the whole tensor
 * All ranks must issue the same sequence of calls (one process per GPU, one kernel in flight per
 * rank).  A rank whose peers do not arrive gives up after a bounded wait (about half a second by
 * default; launch skew between ranks must stay below it): its outputs are set to NaN / -1, so that the
 * previous call's answer cannot pass for this one's, and tpb200_device_status() reports 5.  The caller
 * reads the status wherever it synchronises anyway.  world <= 16.
 * tpb200_set_exchange_wait_polls sets the bound for the calls that follow, in polls of at least
 * 100 ns each (1 .. 2^25, a few seconds; default 2^22).
 */
size_t tpb200_exchange_buffer_bytes(void);
int tpb200_set_exchange_wait_polls(int polls);
int tpb200_reduce_fused_exchange(int op, const void* in, int dtype, int64_t n, int64_t global_offset,
                                 int64_t total_count, int64_t correction, int rank, int world,
                                 void* const* peer_buffers, void* out_val, int64_t* out_idx,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* ---- single-process multi-GPU host -------------------------------------------------------------
 * No reference counterpart (the reference is single-GPU: p10/src/backend/cuda/CUDAAllocator.cpp:87-88).
 * For a host that drives several GPUs of one box from one process (a C++ TensorPlay program; no
 * Python, no PyTorch, no NCCL needed): a comm owns a stream, the exchange buffer, scratch and gather
 * buffers on each of its GPUs -- all allocated by tpb200_comm_create -- and the two calls below run a
 * whole-tensor reduction or a global top-k over a flat tensor whose partition g (counts[g] contiguous
 * float32 elements at parts[g]) lives on GPU g of the comm.  Partition g starts at element
 * counts[0] + ... + counts[g-1] of the whole tensor; indices in the results are global.
 *   - Distinct GPUs with peer access: reductions use tpb200_reduce_fused_exchange on every GPU (records
 *     cross NVLink by peer stores inside the kernels).  Otherwise -- e.g. one device listed several times,
 *     which is how the tests emulate ranks on a single GPU -- records and candidates are copied between
 *     the gather buffers and merged in rank order; no kernel then waits for another.
 *   - The calls enqueue on the comm's streams and return; out_val[g] / out_idx[g] (device pointers on
 *     GPU g, or NULL to use the comm's own result buffers, tpb200_comm_result_values / _indices) hold the
 *     result -- identical on every GPU -- after tpb200_comm_synchronize (or a wait on
 *     tpb200_comm_stream(comm, g)).  Inputs must be ready when the call is made.
 *   - tpb200_topk_sharded: every GPU must hold at least k elements; k <= 2048 and GPUs * k <= 8192.
 */
typedef struct tpb200_comm tpb200_comm;
int tpb200_comm_create(int n_gpus, const int* devices, tpb200_comm** out);
int tpb200_comm_destroy(tpb200_comm* comm);
int tpb200_comm_size(const tpb200_comm* comm);
int tpb200_comm_fused(const tpb200_comm* comm);          /* 1: reductions exchange by peer stores */
void* tpb200_comm_stream(const tpb200_comm* comm, int g);  /* cudaStream_t of GPU g */
int tpb200_comm_synchronize(tpb200_comm* comm);
void* tpb200_comm_result_values(const tpb200_comm* comm, int g);
int64_t* tpb200_comm_result_indices(const tpb200_comm* comm, int g);
int tpb200_reduce_sharded(tpb200_comm* comm, int op, const void* const* parts, const int64_t* counts, int dtype,
                          int64_t correction, void* const* out_val, int64_t* const* out_idx);
int tpb200_topk_sharded(tpb200_comm* comm, const void* const* parts, const int64_t* counts, int dtype, int64_t k,
                        int largest, float* const* out_val, int64_t* const* out_idx);

/* ---- global top-k over candidate lists --------------------------------------------------------
 * Final step of a sharded top-k: `n_cand` candidates (value, int64 GLOBAL index), e.g. the
 * all-gathered local top-k lists of every GPU, are reduced to the best k under the same order
 * (value, then ascending index).  n_cand <= 8192.
 * If list_offsets is not NULL the candidates are `n_cand / list_len` lists of list_len entries
 * holding list-LOCAL indices, and list_offsets[j] is added to every index of list j (the start of
 * rank j's partition); with NULL the indices are taken as global already.
 */
int tpb200_topk_merge(const float* cand_val, const int64_t* cand_idx, int64_t n_cand, int64_t k,
                      int largest, const int64_t* list_offsets, int64_t list_len, float* out_val,
                      int64_t* out_idx, void* stream);

/* ---- whole-tensor reduction that allocates nothing and needs no workspace ----------------------
 * No counterpart in the reference.  For callers that cannot allocate device memory and have no
 * scratch buffer to pass: a host whose own pool already owns the whole device, or a loop that must
 * not pay the device-wide synchronisation hidden in cudaMalloc / cudaFree.  Same operators, same
 * kernels and bit-identical results as tpb200_reduce with reduce_mask = 0 on a contiguous 1-D
 * tensor of n float32 elements; the partial records live in a TPB200_NOALLOC_SCRATCH_BYTES array
 * built into the library (each GPU that loads the library holds it until the process exits).
 *   - n must not exceed TPB200_NOALLOC_MAX_ELEMENTS; larger sizes are refused with
 *     TPB200_ERR_UNSUPPORTED before anything is launched.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before any stream capture is begun.
 *   - The call uses no cudaMalloc, cudaFree or other allocating routine, and never synchronises.
 *   - All calls on one device share the array.  Nothing in it has to be cleared between calls (the
 *     first pass overwrites every record the second pass reads), but two calls whose kernels
 *     overlap on the GPU -- different streams, no ordering between them -- race on it: order them.
 */
#define TPB200_NOALLOC_SCRATCH_BYTES (128 * 1024)
#define TPB200_NOALLOC_MAX_ELEMENTS (1ull << 33)
int tpb200_reduce_all_noalloc(int op, const void* in, int dtype, int64_t n, int64_t correction,
                              void* out_val, int64_t* out_idx, void* stream);

/* ---- diagnostics ------------------------------------------------------------------------------
 * Every device-side wait in these kernels is bounded: the ring and rendezvous waits between the
 * warps of a top-k CTA, and the wait of the fused exchange for the records of the other ranks.  A
 * kernel whose wait gave up sets a per-device status word; a top-k kernel then leaves its outputs
 * unwritten, the fused exchange writes NaN / -1 so that a timed-out call cannot pass for a result.
 * Status values: 0 no wait ever gave up; 1..4, 6..8 a top-k wait (which one is in the low byte);
 * 5 the peer exchange; 0x40000000 a range violation in a checked build (below).  This call
 * SYNCHRONISES with the device, returns the word in *status_out and clears it.  No reference
 * counterpart.
 */
int tpb200_device_status(int* status_out);

/* ---- checked build ----------------------------------------------------------------------------
 * libtpb200_checked.so is the same library compiled with -DTPB200_CHECKED: every entry point first
 * registers the address ranges its kernels may touch (the input view, the outputs, the workspace,
 * exchange buffers), and every access of a kernel to global memory is compared with them.  An
 * access outside the ranges is not made (it is turned to a sink buffer), the first one is recorded
 * and all are counted; nothing traps and the context stays usable.  It is the stand-in for a memory
 * checker, several times slower than the ordinary build, one call at a time per device.
 *
 * tpb200_check_report fills info[0..5] = {1 in a checked build else 0, violations since the last
 * report, source file id of the first (1 reduce, 2 top-k, 3 top-k select, 4 softmax, 5 median,
 * 6 copy, 0 shared header), its line, its address, its size in bytes}, SYNCHRONISES and clears the
 * record.  tpb200_check_trim_next(bytes) is the checker's own test: the next entry point registers
 * every range `bytes` shorter at its end, so that correct kernels are seen to be caught and skipped;
 * TPB200_ERR_UNSUPPORTED in the ordinary build.  No reference counterpart.
 */
#define TPB200_CHECK_INFO_FIELDS 6
int tpb200_check_report(int64_t* info, int n_info);
int tpb200_check_trim_next(int64_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* TPB200_H_ */

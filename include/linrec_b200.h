/*
 * linrec_b200 -- C ABI of the B200 (sm_100a) linear-recurrence scan library.
 *
 *     y[i] = y[i-1] * c[i] + x[i]        along the last dimension, forward or reversed,
 *     and its backward:  dx = scan of dy in the opposite direction with the coefficients
 *     shifted by one, dc[i] = dx[i] * y[i-+1].
 *
 * This is the drop-in boundary: plain pointers and sizes, no torch types.  Every function works
 * on device memory laid out as `numseq` rows of `seqlen` elements, element (r, i) at
 * r*row_stride + i (row_stride >= seqlen, in elements), launches on the caller's stream
 * (passed as a void* holding a cudaStream_t) and returns immediately; the return value is
 * LINREC_OK or a negative LINREC_ERR_* code.  The library keeps no global mutable state except
 * a launch counter; calls are re-entrant across host threads as long as each concurrent call has
 * its own workspace.
 *
 * Each entry point names the interface of the reference (safelix/linrec, paths relative to that
 * project) that it stands in for.
 */
#ifndef LINREC_B200_H
#define LINREC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define LINREC_API
#else
#define LINREC_API __attribute__((visibility("default")))
#endif

/* ---- status codes ------------------------------------------------------------------------- */
#define LINREC_OK                   0
#define LINREC_ERR_INVALID_ARG     (-1)  /* null pointer, negative size, stride < seqlen, ...  */
#define LINREC_ERR_WORKSPACE       (-2)  /* workspace missing, misaligned or too small          */
#define LINREC_ERR_NOT_IMPLEMENTED (-3)  /* option name or value that no compiled variant has   */
#define LINREC_ERR_CUDA            (-4)  /* a CUDA runtime/driver call failed                   */
#define LINREC_ERR_TIMEOUT         (-5)  /* a bounded device-side wait gave up (see _status)    */
#define LINREC_ERR_TOO_LONG        (-6)  /* tile-only call and the row does not fit one tile    */
#define LINREC_ERR_UNALIGNED       (-7)  /* bulk-copy path forced on pointers/strides it cannot take */
#define LINREC_ERR_SCRATCH_LIMIT   (-8)  /* problem needs more scratch than the built-in buffer has  */

/* ---- element storage types (arithmetic is fp32, except for LINREC_DTYPE_F64) ----------------- */
#define LINREC_DTYPE_F32   0
#define LINREC_DTYPE_BF16  1
#define LINREC_DTYPE_F16   2
#define LINREC_DTYPE_F64   3   /* fp64 storage AND arithmetic (the type dispatch the reference leaves open,
                                  linrec/impl/cuda/linrec_pipe.cu:22): LINREC_KIND_REF one thread per row,
                                  the other kinds one CTA per row (no variants to pin: pinning options answer
                                  LINREC_ERR_NOT_IMPLEMENTED, as do the middle-axis, static-buffer and
                                  sharding entry points) */

/* ---- which family of kernels a call may use --------------------------------------------------
 * The reference exposes three operator families with one signature
 * (linrec/impl/cuda/linrec.h:17-57); the same three are kept:
 *   REF   one thread walks one row sequentially     (linrec_ref_fwd/bwd,  linrec_ref.cu:11-95)
 *   TILE  the whole row must fit one tile           (linrec_tile_fwd/bwd, linrec_tile.cu:17-177)
 *   PIPE  any length; rows longer than a tile are chained with look-back carries
 *                                                   (linrec_pipe_fwd/bwd, linrec_pipe.cu:16-174) */
#define LINREC_KIND_REF   0
#define LINREC_KIND_TILE  1
#define LINREC_KIND_PIPE  2

/* Options are passed the way the reference passes its **kwargs -> std::map<std::string,int>
 * (linrec/impl/cuda/extension.cpp:20-31): parallel arrays of names and integer values.  Known
 * names are listed by linrec_b200_config_names(); an unknown name or a value without a compiled
 * variant gives LINREC_ERR_NOT_IMPLEMENTED (the reference raises NotImplementedError from
 * dispatch.h:70-71).  n_opts may be 0, in which case the regime selector chooses.
 * `memcode` names the way rows are brought in: 0 plain loads, 1 bulk-tensor copies (rows of whole
 * 128-byte lines), 2 / 3 16-byte / 4-byte asynchronous copies, 4 one CTA per row with aligned 16-byte
 * accesses (any row length and start; all tensors of the call must start equally far from a 16-byte
 * boundary, else LINREC_ERR_UNALIGNED; it has no variants, so it cannot be combined with the other
 * selectors).
 *
 * Besides the variant selectors there is one option that changes what is computed:
 *   logCoeffs = 1   the coefficient tensor holds logarithms (the `logc` argument of the reference's
 *                   Python operator, linrec/impl/python/ops.py:8-14): the kernels use exp(c), and
 *                   the backward entry points return the gradient with respect to the logarithm
 *                   (d_c * exp(c)) in `dc`.  Accepted by linrec_b200_fwd/bwd (all kinds) and
 *                   linrec_b200_fwd_dim/bwd_dim; the sequence-sharding entry points answer
 *                   LINREC_ERR_NOT_IMPLEMENTED. */
typedef struct linrec_opts {
    int n_opts;
    const char* const* names;
    const int* values;
} linrec_opts;

/* Bytes of scratch a call on this shape may need (look-back descriptors, ticket counter, epoch and
 * the status word).  Always > 0 and a multiple of 256; the buffer must be 256-byte aligned device
 * memory that its owner ZEROES ONCE before the first call (cudaMemset).  After that no call needs
 * any preparation: each launch leaves the workspace ready for the next one, whatever its shape.
 * Replaces nothing in the reference (its kernels never leave one CTA per row). */
LINREC_API size_t linrec_b200_workspace_size(int64_t numseq, int64_t seqlen, int dtype);

/* Forward scan.  Replaces linrec_{ref,tile,pipe}_fwd (linrec/impl/cuda/linrec.h:17-19,28-31,44-47).
 * `kind` is one of LINREC_KIND_*; `reverse` scans from the last element down. */
LINREC_API int linrec_b200_fwd(int kind, const void* x, const void* c, void* y,
                               int64_t numseq, int64_t seqlen, int64_t row_stride,
                               int reverse, int dtype, const linrec_opts* opts,
                               void* workspace, size_t workspace_bytes, void* stream);

/* Backward.  Replaces linrec_{ref,tile,pipe}_bwd (linrec/impl/cuda/linrec.h:21-25,33-38,49-54).
 * `reverse` is the flag the forward pass was run with. */
LINREC_API int linrec_b200_bwd(int kind, const void* dy, const void* c, const void* y,
                               void* dx, void* dc,
                               int64_t numseq, int64_t seqlen, int64_t row_stride,
                               int reverse, int dtype, const linrec_opts* opts,
                               void* workspace, size_t workspace_bytes, void* stream);

/* Device-side status word of the calls that used `workspace` since it was last read: synchronises
 * `stream`, reads the word, clears it, and returns LINREC_OK or LINREC_ERR_TIMEOUT.  A NULL
 * `workspace` stands for the built-in buffer of the current device (linrec_b200_fwd_static).
 * The bounded waits inside the kernels
 * (look-back on a predecessor tile, arrival of a bulk copy) never trap and never spin forever;
 * when one gives up the kernel finishes with wrong numbers and sets this word.
 * No counterpart in the reference (its kernels contain no inter-CTA wait). */
LINREC_API int linrec_b200_status(const void* workspace, void* stream);

/* Kernel attributes of the variant that the options select, as parallel name/value arrays
 * written into caller storage (at most `cap` entries; returns the number written or a negative
 * error).  Replaces linrec_{tile,pipe}_attrs (linrec/impl/cuda/linrec_pipe.cu:177-212) together
 * with cudaFuncAttributesAsMap (linrec/impl/cuda/cuhelpers.cuh:36-55). */
LINREC_API int linrec_b200_attrs(int kind, int fwd, int dtype, const linrec_opts* opts,
                                 const char** names, int* values, int cap);

/* Introspection of the compiled variants.  Replaces CONFIG_NAMES / CONFIG_LIST
 * (linrec/impl/cuda/linrec.h:8-13) as exported through extension.cpp:46-47.
 * config_names: returns the number of option names, writes up to `cap` pointers.
 * config_list : returns the number of variants; writes up to cap_rows rows of n_names ints. */
LINREC_API int linrec_b200_config_names(const char** names, int cap);
LINREC_API int linrec_b200_config_list(int* values, int cap_rows);

/* Sequence sharding: one row split over `nshards` GPUs, shard s owning the columns
 * [s*seqlen, (s+1)*seqlen) of every row (`seqlen` is the SHARD's length here).  No counterpart in
 * the reference, which is single-device.  Per rank:
 *   1. *_carry   local scan of the shard with zero carry-in; also writes one fp32 record per row:
 *                forward  records[2r+{0,1}]   = (P, Y): product of c over the shard, last local y;
 *                backward records[4r+{0..3}]  = (P, Y, c at the shard's scan-last element,
 *                                                y at the shard's scan-first element).
 *   2. the caller gathers the records of all shards in shard order into
 *      gathered[(s*numseq + r)*rec + k]   (one all-gather; rec = 2 forward, 4 backward);
 *   3. *_fixup   folds the records of the shards that come earlier in scan order into the carry that
 *                enters this shard and computes the head of the shard AGAIN from its operands and that
 *                carry (x, c -> y; dy, c, y -> dx, dc), as far along each row as the carry can still
 *                change a result: until carry * running product of the coefficients is exactly zero or
 *                less than a quarter ulp (2^-26) of the true value at that element.
 *                Recomputing instead of adding a correction rounds each result to the storage type
 *                once, as the unsharded scan does.
 * `reverse` is the flag of the forward pass in all four. */
LINREC_API int linrec_b200_fwd_carry(const void* x, const void* c, void* y, float* records,
                                     int64_t numseq, int64_t seqlen, int64_t row_stride,
                                     int reverse, int dtype, int shard, int nshards,
                                     const linrec_opts* opts,
                                     void* workspace, size_t workspace_bytes, void* stream);
LINREC_API int linrec_b200_fwd_fixup(const void* x, void* y, const void* c, const float* gathered,
                                     int64_t numseq, int64_t seqlen, int64_t row_stride,
                                     int reverse, int dtype, int shard, int nshards, void* stream);
LINREC_API int linrec_b200_bwd_carry(const void* dy, const void* c, const void* y, void* dx, void* dc,
                                     float* records,
                                     int64_t numseq, int64_t seqlen, int64_t row_stride,
                                     int reverse, int dtype, int shard, int nshards,
                                     const linrec_opts* opts,
                                     void* workspace, size_t workspace_bytes, void* stream);
LINREC_API int linrec_b200_bwd_fixup(const void* dy, void* dx, void* dc, const void* c, const void* y,
                                     const float* gathered,
                                     int64_t numseq, int64_t seqlen, int64_t row_stride,
                                     int reverse, int dtype, int shard, int nshards, void* stream);

/* Sequence sharding without a collective call.  Each rank owns an "exchange buffer" of
 * linrec_b200_exchange_size(max_rows, nranks) bytes, 256-byte aligned, that every rank of the node can
 * address (peer-mapped / symmetric memory).  linrec_b200_exchange_init zeroes the local buffer and
 * stores in it the addresses of all ranks' buffers as mapped in the calling process
 * (peer_bufs[rank] must be the local buffer); the ranks must synchronise once after it (a barrier)
 * before the first exchange.  One *_seq_p2p call = local scan whose kernel leaves each row's record
 * in the rank's own buffer and, when the launch is complete, releases one flag in every rank's
 * buffer, followed by the fix-up kernel, which waits (bounded) for the flags it needs in its own
 * buffer and reads the records from their owners' buffers.  No NCCL kernel, no host
 * synchronisation.  `epoch` must be 1 for the first exchange on these buffers and grow by one with
 * every call, identically on all ranks (the calls are collective: every rank makes the same sequence
 * of them, with numseq <= max_rows).  Slots are double-buffered by epoch parity and released by
 * acknowledgements, so ranks may run ahead of each other by at most one exchange.  A wait that runs
 * out of its budget sets the status word of `workspace` (linrec_b200_status).
 * No counterpart in the reference. */
LINREC_API size_t linrec_b200_exchange_size(int64_t max_rows, int nranks);
LINREC_API int linrec_b200_exchange_init(void* local_buf, void* const* peer_bufs, int rank, int nranks,
                                         int64_t max_rows, void* stream);
LINREC_API int linrec_b200_fwd_seq_p2p(const void* x, const void* c, void* y,
                                       int64_t numseq, int64_t seqlen, int64_t row_stride,
                                       int reverse, int dtype, int shard, int nshards,
                                       void* exchange, uint32_t epoch, const linrec_opts* opts,
                                       void* workspace, size_t workspace_bytes, void* stream);
LINREC_API int linrec_b200_bwd_seq_p2p(const void* dy, const void* c, const void* y, void* dx, void* dc,
                                       int64_t numseq, int64_t seqlen, int64_t row_stride,
                                       int reverse, int dtype, int shard, int nshards,
                                       void* exchange, uint32_t epoch, const linrec_opts* opts,
                                       void* workspace, size_t workspace_bytes, void* stream);

/* Forward scan for callers that cannot give the library any scratch memory.
 *
 * linrec_b200_fwd needs a caller-provided workspace, which normally means the caller allocates
 * device memory.  Some hosts cannot: a program that binds only this C function from another
 * runtime and owns no device allocator to get a workspace from; a service whose device memory is
 * handed out in full to another pool at start-up; a latency-critical loop in which cudaMalloc's
 * device-wide synchronisation is not acceptable.  For them this entry point does the same forward
 * scan (LINREC_KIND_PIPE, selector defaults, same arguments otherwise) but keeps its ticket counter,
 * status word and look-back descriptors in a buffer that is compiled into the library:
 * LINREC_STATIC_SCRATCH_BYTES (1 MiB) of device memory per GPU that loads the library, held until
 * the process exits.  It calls no cudaMalloc, no cudaFree and no other allocating routine (the CUDA
 * calls it makes are cudaGetDevice/cudaSetDevice on the current device, attribute and occupancy
 * queries, cudaGetSymbolAddress, two 4-byte cudaMemsetAsync on `stream`, and the kernel launch).
 *
 * Limit: the scratch a problem needs must fit the built-in buffer.  Rows that fit one tile need
 * 256 bytes whatever their number; rows longer than a tile need 16 more bytes per tile.  A tile is
 * 8192 elements for fp32 rows that are 16-byte aligned and a multiple of 128 bytes long, and 2048
 * to 8192 otherwise (alignment, storage type and row count decide).  So at most 65,520 tiles of
 * long rows (about 5.3e8 fp32 elements in the aligned case) can be scanned by one call; larger
 * problems return LINREC_ERR_SCRATCH_LIMIT and launch nothing.
 *
 * The first call on each device looks up the buffer's device address (once per device, with that
 * device current); make that first call outside any stream capture.  All calls on a device share
 * the one buffer, which keeps what the previous call left in it.  What has to start from zero is
 * cleared by every call on `stream` before its kernel: the ticket counter and the count of finished
 * CTAs (the kernels normally leave both at zero themselves, but a launch that failed, or two launches
 * that raced, may not have).  The look-back descriptors need no clearing: each is tagged with the
 * launch epoch kept in the buffer, which every launch advances, and a descriptor of another epoch
 * reads as empty.  Two calls that overlap on the GPU (different streams, different host threads) race
 * on the buffer -- serialise them, or use linrec_b200_fwd with separate workspaces.
 *
 * The bounded waits of a call through this entry point report to the status word inside the built-in
 * buffer: read (and clear) it with linrec_b200_status(NULL, stream) on the same device.
 * This function has no counterpart in the reference. */
#define LINREC_STATIC_SCRATCH_BYTES (1u << 20)
LINREC_API int linrec_b200_fwd_static(const void* x, const void* c, void* y,
                                      int64_t numseq, int64_t seqlen, int64_t row_stride,
                                      int reverse, int dtype, void* stream);

/* The built-in buffer of the current device as a workspace for the other entry points: writes its
 * device address and size (LINREC_STATIC_SCRATCH_BYTES).  For callers that cannot allocate but want
 * what linrec_b200_fwd_static does not offer (options, the backward pass, the middle-axis scan);
 * the same sharing rule applies -- one call at a time per device on this buffer -- and the caller
 * checks the size against linrec_b200_workspace_size itself.  The first call on a device resolves the
 * address (outside any stream capture).  No counterpart in the reference. */
LINREC_API int linrec_b200_static_workspace(void** workspace, size_t* bytes);

/* ---- scan along a dimension other than the last ------------------------------------------------------
 * The `dim` argument of the reference's Python operator (linrec/impl/python/ops.py:8-14,43-61); the
 * reference's CUDA operators scan the last dimension only (linrec/impl/cuda/linrec_pipe.cu:17-35), so
 * its callers transpose in and out.  Here the tensor is taken as contiguous (nb, seqlen, nchan) and
 * the recurrence runs along the MIDDLE axis in place of those copies: element (b, l, d) follows
 * (b, l-1, d).  Arguments and error codes as linrec_b200_fwd / linrec_b200_bwd; all tensors have the
 * same (nb, seqlen, nchan) shape and are dense.  Requirements: 16-byte aligned pointers and
 * nchan * element size a multiple of 16 bytes (else LINREC_ERR_UNALIGNED: transpose and use the
 * last-axis operators).  The workspace must be zeroed once by its owner, like the other workspaces
 * (they are interchangeable), and hold linrec_b200_dim_workspace_size(...) bytes for the same
 * arguments and options; that size query returns 0 for options no compiled variant matches.
 * Options: kThreadsPerBlock, kRowsPerChunk, kStages pin a variant; kChunksPerJob (0 = a whole column
 * per job) sets how finely a column is cut into jobs that are linked by look-back carries.
 * Performance note: the kernel gets its parallelism from the columns (one column = 32 channel words of
 * one batch entry).  With fewer than 64 columns the sequence axis has to supply it through per-thread
 * look-back, which is latency-bound (0.7-1.5 TB/s on B200 against 6.5 TB/s with many columns); a caller
 * that can afford transposed copies is better off with the last-axis entry points there (the Python
 * wrapper linrec_general does that below 128 columns). */
LINREC_API size_t linrec_b200_dim_workspace_size(int bwd, int64_t nb, int64_t seqlen, int64_t nchan,
                                                 int dtype, const linrec_opts* opts);
LINREC_API int linrec_b200_fwd_dim(const void* x, const void* c, void* y,
                                   int64_t nb, int64_t seqlen, int64_t nchan, int reverse, int dtype,
                                   const linrec_opts* opts, void* workspace, size_t workspace_bytes,
                                   void* stream);
LINREC_API int linrec_b200_bwd_dim(const void* dy, const void* c, const void* y, void* dx, void* dc,
                                   int64_t nb, int64_t seqlen, int64_t nchan, int reverse, int dtype,
                                   const linrec_opts* opts, void* workspace, size_t workspace_bytes,
                                   void* stream);

/* Number of kernels this library has launched in this process (all threads). */
LINREC_API uint64_t linrec_b200_launch_count(void);

/* What LINREC_ERR_CUDA stood for in the last call of the calling thread that returned it: the name of
 * the failing CUDA call and the runtime's error text ("" if there was none).  The reference reports
 * such failures through C10_CUDA_KERNEL_LAUNCH_CHECK (linrec/impl/cuda/linrec_pipe.cu:88). */
LINREC_API const char* linrec_b200_last_cuda_error(void);

/* Text for a status code. */
LINREC_API const char* linrec_b200_strerror(int code);

/* Library version, e.g. 200 for 0.2.0 (0.2.0 changed the fix-up entry points: they take the operands x / dy). */
LINREC_API int linrec_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* LINREC_B200_H */

/*
 * gqa_decode_b200.h -- C ABI of the B200 (sm_100a) paged grouped-query decode library.
 *
 * Every entry point takes plain pointers and sizes, never allocates or frees
 * device memory, never throws, and returns an int status: 0 = ok, < 0 = invalid
 * argument (see gqa_b200_strerror), > 0 = a cudaError_t raised by a launch.  No
 * entry point synchronises the device, with two exceptions that say so below:
 * the debug getters gqa_b200_prefill_tc_status and mla_b200_tc_status, which
 * copy a status word back with a blocking cudaMemcpy.  All device pointers must belong to the
 * device that is current in the calling thread; work is enqueued on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *
 * Tensor layouts are those of the reference library's operator
 * (csrc/cuda/dense/gqa_decode.cu:109-113), all contiguous:
 *   q, out        [batch, q_heads, head_dim]
 *   k/v_cache     [num_blocks, block_size, kv_heads, head_dim]
 *   block_table   [batch, max_pages] int32; slots past a sequence's used pages
 *                 are never read and may hold -1
 *   context_lens  [batch] int32
 */
#ifndef GQA_DECODE_B200_H
#define GQA_DECODE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GQA_B200_API __attribute__((visibility("default")))

#define GQA_B200_ABI_VERSION 2

/* element types of q / k_cache / v_cache / out */
#define GQA_B200_F32 0
#define GQA_B200_F16 1
#define GQA_B200_BF16 2

/* kernel selection for gqa_b200_decode_ex */
#define GQA_B200_KERNEL_AUTO 0 /* tensor-core kernel when eligible, else SIMT   */
#define GQA_B200_KERNEL_SIMT 1 /* warp dot products + shuffle reductions, any D */
#define GQA_B200_KERNEL_MMA 2  /* mma.sync m16n8k16; fp16/bf16, D in {64,128,256},
                                  16-byte aligned tensors                        */

#define GQA_B200_KERNEL_TCGEN05 4 /* prefill only: warp-specialised tcgen05.mma kernel
                                  (persistent CTAs, two query tiles per CTA, scores,
                                  P and accumulators in tensor memory); same shapes
                                  as GQA_B200_KERNEL_MMA                            */

/* status codes (negative = invalid argument) */
#define GQA_B200_OK 0
#define GQA_B200_ERR_NULL_POINTER (-1)
#define GQA_B200_ERR_DTYPE (-2)       /* q/k/v must be float32/float16/bfloat16 */
#define GQA_B200_ERR_HEADS (-3)       /* Hq must be divisible by Hkv            */
#define GQA_B200_ERR_HEAD_DIM (-4)    /* supported head_dim is [1, 256]         */
#define GQA_B200_ERR_CACHE_SHAPE (-5) /* cache must have positive blocks and block_size */
#define GQA_B200_ERR_MAX_PAGES (-6)   /* block_table must have at least one page */
#define GQA_B200_ERR_SCALE (-7)       /* scale must be positive and finite      */
#define GQA_B200_ERR_BATCH (-8)       /* negative batch                         */
#define GQA_B200_ERR_WORKSPACE (-9)   /* workspace missing, misaligned or too small */
#define GQA_B200_ERR_SPLITS (-10)     /* splits must be in [1, 65535]           */
#define GQA_B200_ERR_KERNEL (-11)     /* requested kernel cannot run these arguments */
#define GQA_B200_ERR_CHUNK (-12)      /* chunk_tokens out of range              */
#define GQA_B200_ERR_INT32_RANGE (-13)/* tensor sizes exceed int32 launch limits */
#define GQA_B200_ERR_STATIC_LIMIT (-14) /* shape needs more than GQA_B200_STATIC_SCRATCH_BYTES */

/* Workspace header: the first int32 words of the workspace, readable by the
 * host after a stream synchronise when debugging.
 *   word 0  work-item counter (zero between calls)
 *   word 1  number of (sequence, chunk) pairs the last plan produced
 *   word 2  device status: 0 ok, 1 = plan overflowed the workspace (cannot
 *           happen when it is sized by gqa_b200_workspace_bytes)
 *   word 3  base chunk length the last plan used                            */
#define GQA_B200_HDR_COUNTER 0
#define GQA_B200_HDR_TOTAL_CHUNKS 1
#define GQA_B200_HDR_STATUS 2
#define GQA_B200_HDR_CHUNK_BASE 3

GQA_B200_API int gqa_b200_abi_version(void);

/* Text for a status code returned by any entry point (static storage). */
GQA_B200_API const char* gqa_b200_strerror(int code);

/* chunk_tokens = 0 leaves the base KV-chunk length to the plan kernel, which
 * picks it ON THE DEVICE from the batch's actual context_lens (never read by
 * the host): the largest of 1024, 512, 256, 128, 64 that still yields about one
 * work item per resident decode CTA, so a small batch is cut finely enough to
 * occupy every SM, a large one pays little per-chunk overhead, and a block
 * table much wider than the sequences in it costs nothing.  The choice is
 * stored in workspace header word GQA_B200_HDR_CHUNK_BASE.  This function
 * previews the rule on the host for sequences that fill their table. */
GQA_B200_API int gqa_b200_auto_chunk_tokens(int batch, int q_heads, int kv_heads, int block_size,
                                            int max_pages);

/* KV-chunk length, in tokens, that a sequence of `context_len` tokens is cut
 * into for a given base `chunk_tokens` (16 .. 65536).  A function of the
 * sequence's own length only, so with one base a sequence is cut, and its
 * partials merged, the same way whichever batch or GPU it lands on.  Sequences
 * longer than 32x / 128x the base use 2x / 4x the base. */
GQA_B200_API int gqa_b200_chunk_tokens(int context_len, int chunk_tokens);

/* Upper bound on chunks per sequence for a table of max_pages*block_size tokens. */
GQA_B200_API int gqa_b200_max_chunks_per_seq(int max_pages, int block_size, int chunk_tokens);

/* Bytes of device scratch gqa_b200_decode / _decode_ex need for this static
 * shape (worst case over context_lens).  The buffer must be 256-byte aligned.
 * Its control words -- the first gqa_b200_workspace_control_bytes() bytes,
 * whatever the shape: a header and the arrival counters of the one-launch
 * path -- must be ZERO before the first call that uses it: cudaMemset the
 * buffer once after allocating it, or call gqa_b200_workspace_init.  Every
 * call leaves those words at zero again, so a workspace is initialised once,
 * not per call, and may be reused by calls of other shapes that fit in it.
 * Nothing else carries over between calls.  Two calls that may overlap on the
 * device need two workspaces. */
GQA_B200_API size_t gqa_b200_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim,
                                             int block_size, int max_pages, int chunk_tokens);

/* Size of the control region at the start of every workspace (about 64 KB). */
GQA_B200_API size_t gqa_b200_workspace_control_bytes(void);

/* Zero the control words of a workspace (one cudaMemsetAsync on `stream`; no
 * allocation, no synchronisation).  Needed once per workspace, and again only
 * if something else wrote into the buffer or a call was torn down by a CUDA
 * error. */
GQA_B200_API int gqa_b200_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Paged single-token MHA/MQA/GQA decode.
 * Replaces gqa_decode_cuda (csrc/binding/torch_ops.cpp:5-11,
 * csrc/cuda/dense/gqa_decode.cu:186-188) and, through it, gqa_decode_impl
 * (gqa_decode.cu:96-183) with its two kernels (gqa_decode.cu:18-87).
 * No plan launch for batches of up to 2048 sequences: every persistent decode
 * CTA cuts the sequences into KV chunks itself from context_lens (never read by
 * the host) and pulls (sequence, chunk, kv head) items from a counter -- every
 * K/V row is read once for all query heads of its group.  Sequences of several
 * chunks leave fp32 partials; the merge kernel (a second launch) folds them,
 * log-sum-exp, in slot order.  When the static shape is small enough for every
 * work item to get a CTA of its own (small batches of short tables), there is
 * ONE launch: the CTA that takes the last ticket of a sequence merges it.
 * Batches above 2048 sequences take three launches: plan, decode, merge.  All
 * three paths cut a sequence the same way and give the same bits for the same
 * chunk_tokens.  Empty sequences get zero rows.
 * batch == 0 returns OK without launching (gqa_decode.cu:142). */
GQA_B200_API int gqa_b200_decode(const void* q, const void* k_cache, const void* v_cache,
                                 const int32_t* block_table, const int32_t* context_lens,
                                 void* out, int dtype, int batch, int q_heads, int kv_heads,
                                 int head_dim, int64_t num_blocks, int block_size, int max_pages,
                                 float scale, void* workspace, size_t workspace_bytes,
                                 void* stream);

/* phases of gqa_b200_decode_ex: 0 = the default path, chosen from the static
 * shape (see gqa_b200_decode); bits 1, 2, 4 select launches of the three-launch
 * path (7 = all three); 8 or 16 alone force the one- or the two-launch path; 32 then
 * 4 are the two launches of the two-launch path, one per call */
#define GQA_B200_PHASE_PLAN 1
#define GQA_B200_PHASE_DECODE 2
#define GQA_B200_PHASE_MERGE 4
#define GQA_B200_PHASE_ONE_LAUNCH 8  /* alone: self-planning decode kernel that also merges   */
#define GQA_B200_PHASE_TWO_LAUNCH 16 /* alone: self-planning decode kernel, then merge kernel */
#define GQA_B200_PHASE_SELF_DECODE 32 /* alone: the self-planning decode kernel only; a call
                                         with GQA_B200_PHASE_MERGE must follow (timing aid) */

/* Same operator with explicit tuning knobs (tests, benchmarks):
 *   chunk_tokens  base KV-chunk length (0 = built-in; otherwise 16..65536)
 *   kernel        GQA_B200_KERNEL_*
 *   max_ctas      cap on the persistent grid (0 = SM count x resident CTAs)
 *   phases        0 = default; GQA_B200_PHASE_* otherwise.  A benchmark uses the
 *                 bits 1, 2, 4 to put its own events around the decode kernel;
 *                 the phases of one call must still run in order plan, decode,
 *                 merge on the same workspace.                                 */
GQA_B200_API int gqa_b200_decode_ex(const void* q, const void* k_cache, const void* v_cache,
                                    const int32_t* block_table, const int32_t* context_lens,
                                    void* out, int dtype, int batch, int q_heads, int kv_heads,
                                    int head_dim, int64_t num_blocks, int block_size,
                                    int max_pages, float scale, void* workspace,
                                    size_t workspace_bytes, void* stream, int chunk_tokens,
                                    int kernel, int max_ctas, int phases);

/* Size of the scratch array built into the library for gqa_b200_decode_static. */
#define GQA_B200_STATIC_SCRATCH_BYTES (8u << 20)

/* gqa_b200_decode for callers that can hand over no scratch at all.  It has no
 * counterpart in the reference library.
 *
 * Who needs it: a serving engine that has already given all free HBM to its KV
 * page pool, where a later cudaMalloc can fail or fragment; a decode loop that
 * must not stall, since cudaMalloc / cudaFree synchronise the whole device; a
 * plug-in hosted by a runtime that owns device memory and forbids allocations
 * behind its back.  Such a caller still passes its inputs and `out`; the chunk
 * list and the split partials go to a fixed array of
 * GQA_B200_STATIC_SCRATCH_BYTES (8 MiB) that is part of the library image, so
 * every GPU that loads the library holds that much until the process exits.
 *
 * The call allocates and frees nothing (no cudaMalloc/cudaFree, no allocating
 * library routine) and runs the same kernel as gqa_b200_decode, so the
 * result is identical.  Limits and rules:
 *   - a shape whose gqa_b200_workspace_bytes(..., chunk_tokens = 0) exceeds
 *     GQA_B200_STATIC_SCRATCH_BYTES is refused with GQA_B200_ERR_STATIC_LIMIT
 *     and nothing is launched (for scale: batch 64, 32 query heads, head_dim
 *     128, tables of 4096 tokens need about 4.3 MB);
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     outside any stream capture;
 *   - all calls on a device share the one array, which keeps whatever the last
 *     call left in it.  Nothing in it has to be cleared by the caller (the array
 *     is zero when the library is loaded and every call puts its control words
 *     back to zero), but two
 *     calls that may run at the same time on the GPU -- different streams, or
 *     different host threads -- race on it: serialise them, or give the
 *     concurrent ones gqa_b200_decode with workspaces of their own. */
GQA_B200_API int gqa_b200_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                        const int32_t* block_table, const int32_t* context_lens,
                                        void* out, int dtype, int batch, int q_heads,
                                        int kv_heads, int head_dim, int64_t num_blocks,
                                        int block_size, int max_pages, float scale, void* stream);

/* Decode with a caller-chosen number of KV partitions and the reference's
 * partial layout.  Replaces gqa_decode_split_cuda and
 * gqa_decode_split_workspace_cuda (csrc/cuda/dense/gqa_decode.cu:189-195):
 * partition z of a sequence of length L covers tokens [L*z/splits, L*(z+1)/splits)
 * (gqa_decode.cu:40-41); `partials` is float32 [batch, q_heads, splits, head_dim+2]
 * holding [max, sum, acc...] per partition (gqa_decode.cu:67-69) and is
 * overwritten; it is required when splits > 1 and ignored when splits == 1. */
GQA_B200_API int gqa_b200_decode_split(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* block_table, const int32_t* context_lens,
                                       void* out, int dtype, int batch, int q_heads, int kv_heads,
                                       int head_dim, int64_t num_blocks, int block_size,
                                       int max_pages, float scale, int splits, float* partials,
                                       void* stream);

/* Dense (non-paged) GQA prefill.  Replaces gqa_prefill_cuda
 * (csrc/cuda/dense/gqa_prefill.cu:104-141, kernels :19-100) and the reference's
 * Triton "tensorcore" backend (attention/triton_prefill.py): q/out are
 * [batch, tq, q_heads, head_dim], k/v [batch, tk, kv_heads, head_dim], q_lens /
 * kv_lens int32 [batch].  Query row i of a sequence attends to keys
 * 0 .. kv_len - q_len + i when `causal` (right-aligned causal mask,
 * csrc/cuda/common/tile_utils.cuh:6-9), else to all kv_len keys; rows at or past
 * q_len, and rows that see no key, are written as zeros.  One kernel launch, no
 * scratch.  `kernel`: GQA_B200_KERNEL_AUTO / _SIMT / _MMA / _TCGEN05 (the last two:
 * fp16/bf16, head_dim 64 or 128, 16-byte aligned tensors). */
GQA_B200_API int gqa_b200_prefill(const void* q, const void* k, const void* v,
                                  const int32_t* q_lens, const int32_t* kv_lens, void* out,
                                  int dtype, int batch, int tq, int tk, int q_heads, int kv_heads,
                                  int head_dim, float scale, int causal, int kernel, void* stream);

/* Debug aid for the tcgen05 prefill kernel: synchronises, returns its device status word
 * (0 ok, 2 = a bounded mbarrier wait ran out, 3 = misaligned shared memory; negative = a
 * cudaError_t) and clears it when `reset` is non-zero.  Not for a hot path. */
GQA_B200_API int gqa_b200_prefill_tc_status(int reset);

/* Write one new token per sequence into its page.  Replaces kv_append_cuda
 * (csrc/cuda/cache/kv_append.cu:29-56): key/value are [batch, kv_heads,
 * head_dim]; the row goes to block_table[b, positions[b] / block_size], slot
 * positions[b] % block_size.  The caller owns distinct, valid destinations.
 * A position outside [0, max_pages*block_size) or a page id outside
 * [0, num_blocks) is skipped (the reference reads out of bounds there). */
GQA_B200_API int gqa_b200_kv_append(const void* key, const void* value, void* k_cache,
                                    void* v_cache, const int32_t* block_table,
                                    const int32_t* positions, int dtype, int batch, int kv_heads,
                                    int head_dim, int64_t num_blocks, int block_size,
                                    int max_pages, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GQA_DECODE_B200_H */

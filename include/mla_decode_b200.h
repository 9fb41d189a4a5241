/*
 * mla_decode_b200.h -- C ABI of the B200 (sm_100a) paged latent-attention (MLA) decode path.
 *
 * Exported by the same shared library as gqa_decode_b200.h and under the same
 * rules: plain pointers and sizes, no allocation, no device synchronisation
 * (except the debug getter mla_b200_tc_status), no exceptions; every function
 * returns an int status (0 = ok, < 0 = one of the
 * GQA_B200_ERR_* codes of gqa_decode_b200.h or an MLA_B200_ERR_* code below,
 * > 0 = a cudaError_t); gqa_b200_strerror() gives the text for all of them.
 * Work is enqueued on `stream` (a cudaStream_t passed as void*).
 *
 * Tensor layouts are those of the reference library's MLA operators
 * (attention/mla.py:1-6, csrc/cuda/mla/mla.cu:161-167), all contiguous and of
 * one element type (GQA_B200_F32 / _F16 / _BF16):
 *   q_nope        [batch, tq, heads, dn]       un-rotated query part
 *   q_absorbed    [batch, tq, heads, dc]       q_nope . W_uk
 *   q_rope        [batch, tq, heads, dr]       rotated query part
 *   cache         [num_blocks, page, dc + dr]  latent row ++ rotated key row
 *   block_table   [batch, max_pages] int32     slots past the used pages are never read
 *   lengths       [batch] int32
 *   positions     [batch, tq] int32            absolute position of each query token
 *   indices       [batch, tq, nk] int32 or NULL; logical token ids, -1 = ignored
 *   w_uk          [heads, dn, dc]
 *   w_uv          [heads, dv, dc]
 * A query row attends to logical tokens s < end, end = min(len, max(0, pos + 1))
 * when `causal` and end = len otherwise; with `indices` only listed tokens with
 * 0 <= s < end count.  Rows that see no token are zero.  Scores and sums are
 * fp32; every tensor written is rounded once to the element type.
 */
#ifndef MLA_DECODE_B200_H
#define MLA_DECODE_B200_H

#include "gqa_decode_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MLA_B200_ERR_SHAPE (-32)     /* a width, head count, tq or nk is not positive      */
#define MLA_B200_ERR_LATENT_DIM (-33)/* supported latent width dc is [1, 512]              */

/* kernel selection for mla_b200_attend_ex */
#define MLA_B200_KERNEL_AUTO 0    /* tensor-core kernel when eligible, else SIMT           */
#define MLA_B200_KERNEL_SIMT 1    /* any shape and element type, dense or index-selected   */
#define MLA_B200_KERNEL_TCGEN05 4 /* tcgen05.mma over a CTA pair; fp16/bf16, dc = 512,
                                     dr = 64, dense (indices == NULL), 16-byte aligned rows */

/*
 * Per-head projection.  Replaces mla_project_cuda (csrc/cuda/mla/mla.cu:138-150).
 *   absorb != 0 : x [rows, heads, d_in] . w [heads, d_in, d_out]   (query absorption, W_uk)
 *   absorb == 0 : x [rows, heads, d_in] . w [heads, d_out, d_in]^T (value projection, W_uv)
 * out is [rows, heads, d_out]; rows = batch * tq.  fp32 accumulation.
 */
GQA_B200_API int mla_b200_project(const void* x, const void* w, void* out, int dtype, int64_t rows,
                                  int heads, int d_in, int d_out, int absorb, void* stream);

/*
 * Scatter n tokens into the paged cache: row slots[i] of cache viewed as
 * [cache_rows, dc + dr] becomes latent[i] ++ rope[i].  slots are int64, unique
 * and caller-checked.  Replaces latent_kv_write_cuda (csrc/cuda/mla/mla.cu:151-160).
 */
GQA_B200_API int mla_b200_latent_kv_write(const void* latent, const void* rope, void* cache,
                                          const int64_t* slots, int64_t n, int dc, int dr,
                                          int dtype, void* stream);

/* Bytes of scratch mla_b200_attend needs for this shape (256-byte aligned base).
 * nk = 0 for dense attention; with nk > 0 the answer covers a call with and without
 * `indices`.  Returns 0 for an invalid shape. */
GQA_B200_API size_t mla_b200_attend_workspace_bytes(int batch, int tq, int heads, int dc, int dr,
                                                    int page, int max_pages, int nk);

/*
 * Paged latent attention: out [batch, tq, heads, dc].  Replaces mla_attend_cuda
 * (csrc/cuda/mla/mla.cu:161-181); the split count is chosen inside from the
 * static shape only, so no length is read on the host.
 */
GQA_B200_API int mla_b200_attend(const void* q_absorbed, const void* q_rope, const void* cache,
                                 const int32_t* block_table, const int32_t* lengths,
                                 const int32_t* positions, const int32_t* indices, void* out,
                                 int dtype, int batch, int tq, int heads, int dc, int dr,
                                 int64_t num_blocks, int page, int max_pages, int nk, float scale,
                                 int causal, void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of scratch mla_b200_attend_ex needs for this shape and split count (0 =
 * automatic), whichever kernel it takes and whether or not `indices` is passed. */
GQA_B200_API size_t mla_b200_attend_ex_workspace_bytes(int batch, int tq, int heads, int dc, int dr,
                                                       int page, int max_pages, int nk, int splits);

/* Same with an explicit kernel (MLA_B200_KERNEL_*) and split count (0 = automatic). */
GQA_B200_API int mla_b200_attend_ex(const void* q_absorbed, const void* q_rope, const void* cache,
                                    const int32_t* block_table, const int32_t* lengths,
                                    const int32_t* positions, const int32_t* indices, void* out,
                                    int dtype, int batch, int tq, int heads, int dc, int dr,
                                    int64_t num_blocks, int page, int max_pages, int nk,
                                    float scale, int causal, void* workspace,
                                    size_t workspace_bytes, void* stream, int kernel, int splits);

/* Bytes of scratch mla_b200_decode needs: the absorbed queries, the latent
 * output and the attention scratch. */
GQA_B200_API size_t mla_b200_decode_workspace_bytes(int batch, int tq, int heads, int dc, int dr,
                                                    int page, int max_pages, int nk);

/*
 * Absorbed MLA decode: out [batch, tq, heads, dv] = ((q_nope . W_uk) attends the cache) . W_uv^T.
 * Replaces mla_decode_fused_cuda (csrc/cuda/mla/mla.cu:184-198) and the
 * three-operator path of attention/mla.py:50-52; like both, the absorbed query
 * and the latent output are rounded to the element type between the stages.
 */
GQA_B200_API int mla_b200_decode(const void* q_nope, const void* q_rope, const void* cache,
                                 const int32_t* block_table, const int32_t* lengths,
                                 const int32_t* positions, const void* w_uk, const void* w_uv,
                                 const int32_t* indices, void* out, int dtype, int batch, int tq,
                                 int heads, int dn, int dr, int dc, int dv, int64_t num_blocks,
                                 int page, int max_pages, int nk, float scale, int causal,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* Status word of the tensor-core attention kernel's bounded waits: 0 = never
 * timed out.  `reset` != 0 clears it.  Synchronises the device. */
GQA_B200_API int mla_b200_tc_status(int reset);

#ifdef __cplusplus
}
#endif
#endif /* MLA_DECODE_B200_H */

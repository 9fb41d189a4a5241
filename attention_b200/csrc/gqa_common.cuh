// Shared definitions of the paged GQA decode kernels: launch parameters, the
// KV-chunk policy, the work-item decoding used by both decode kernels, and the
// in-CTA combine of per-warp softmax states.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gqa_b200 {

constexpr int kDefaultChunkTokens = 512;
constexpr int kMinChunkTokens = 16;
constexpr int kMaxChunkTokens = 65536;
constexpr int kHdrWords = 64;           // int32 words reserved at the head of the workspace
constexpr int kHdrCounter = 0;
constexpr int kHdrTotalChunks = 1;
constexpr int kHdrStatus = 2;
constexpr int kHdrChunkBase = 3;
constexpr int kHdrDone = 4;             // CTAs that have left the decode kernel (self-cleaning)
constexpr int kFusedMaxBatch = 2048;    // one-launch mode keeps a [batch + 1] prefix array in shared memory
constexpr int kFusedMaxTickets = 16384; // arrival counters at a FIXED place and size in every workspace, so
                                        // that a call of one shape cannot scribble partials over what a
                                        // later call of another shape takes for its (zero) tickets
constexpr int kNumAutoBases = 5;        // adaptive base candidates: 1024 >> i, i = 0..4
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------
// KV-chunk policy.  A function of the sequence's own length only, so a sequence
// is cut (and its partials merged) identically whatever batch or GPU holds it.
// ---------------------------------------------------------------------------
__host__ __device__ inline int chunk_tokens_for(int len, int base) {
    if (len <= 32 * base) return base;
    if ((long long)len <= 128ll * base) return 2 * base;
    return 4 * base;
}

__host__ __device__ inline int chunks_for(int len, int base) {
    if (len <= 0) return 0;
    const int ct = chunk_tokens_for(len, base);
    return (int)(((long long)len + ct - 1) / ct);
}

// Largest chunks_for(len) over 0 <= len <= cap (not monotone at the policy steps).
inline int max_chunks_for_capacity(long long cap, int base) {
    auto at = [&](long long len) {
        if (len > 0x7fffffffll) len = 0x7fffffffll;
        return chunks_for((int)len, base);
    };
    int m = at(cap);
    if (cap > 32ll * base) m = m > at(32ll * base) ? m : at(32ll * base);
    if (cap > 128ll * base) m = m > at(128ll * base) ? m : at(128ll * base);
    return m < 1 ? 1 : m;
}

// ---------------------------------------------------------------------------
// Launch parameters shared by the plan, decode and merge kernels.
// ---------------------------------------------------------------------------
// kModePlanned   plan kernel -> decode kernel -> merge kernel (three launches)
// kModeRefSplits caller-chosen split count, the reference's partial layout
// kModeFused     no plan launch: every decode CTA derives the chunk list from context_lens
//                itself.  With fused_merge the decode kernel also merges (one launch in all):
//                the CTA that takes the last ticket of a (sequence, kv head, head group)
//                folds that group's partials into `out`; without it the merge kernel
//                follows as a second launch.
enum : int { kModePlanned = 0, kModeRefSplits = 1, kModeFused = 2 };

struct DecodeParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    const int32_t* table;   // [batch, max_pages]
    const int32_t* lens;    // [batch]
    // planned mode (workspace sections)
    int32_t* hdr;           // kHdrWords int32
    int32_t* chunk_off;     // [batch + 1] exclusive prefix of chunks per sequence
    int4* items;            // [cap_chunks] (sequence, partial slot | single<<30, t0, t1)
    float2* part_ml;        // [cap_chunks * q_heads] (max in log2 units, sum)
    float* part_acc;        // [cap_chunks * q_heads * head_dim]
    int32_t* tickets;       // fused mode: [batch * kv_heads * head_groups] arrival counts, zero between calls
    int cap_chunks;
    int item_target;        // adaptive base: smallest chunk total that fills the resident CTAs
    // reference-split mode
    float* ref_partials;    // [batch, q_heads, splits, head_dim + 2]
    int splits;
    int mode;
    int fused_merge;        // kModeFused: 1 = tickets and merge inside the decode kernel
    // shapes
    int batch, q_heads, kv_heads, group, head_dim;
    int heads_per_item;     // query heads of one kv head handled by one work item
    int head_groups;        // ceil(group / heads_per_item)
    int block_size, bs_shift, max_pages;
    long long num_blocks;
    int cap_tokens;         // min(max_pages * block_size, INT_MAX)
    int chunk_base;         // base chunk length; 0 = the plan kernel picks it from the lengths
    int seg_tokens;         // tokens whose page ids are staged in shared memory at once
    int table_smem_entries; // seg_tokens / block_size + 2
    float scale_log2;       // scale * log2(e)
};

// One unit of work of a decode CTA.
struct WorkItem {
    int b, kvh, hg;         // sequence, kv head, head group
    int t0, t1;             // token range [t0, t1)
    int n_parts;            // partitions of this sequence (1 => write `out` directly)
    int part;               // partition index (chunk or split)
    long long part_slot;    // planned: global chunk id; ref splits: unused
};

__device__ __forceinline__ int clamp_len(const DecodeParams& p, int b) {
    int len = __ldg(p.lens + b);
    len = len < 0 ? 0 : len;
    return len > p.cap_tokens ? p.cap_tokens : len;
}

// (planned and reference-split modes; the fused mode counts its items in fused_plan)
__device__ __forceinline__ int total_items(const DecodeParams& p) {
    const int per = p.kv_heads * p.head_groups;
    if (p.mode == kModePlanned) {
        int chunks = p.hdr[kHdrTotalChunks];
        chunks = chunks > p.cap_chunks ? p.cap_chunks : chunks;
        return chunks * per;
    }
    return p.batch * p.splits * per;
}

constexpr int kSingleFlag = 1 << 30;   // item record .y: the sequence has one chunk only

// Items are numbered with the kv head fastest, so CTAs that run side by side
// read neighbouring 2*D-byte rows of the same pages.  An item's record is
// (sequence, partial slot or split index [| kSingleFlag], first token, end token): written by the
// plan kernel in planned mode (one 16-byte load, no dependent reads), computed
// from context_lens in reference-split mode.
__device__ __forceinline__ int4 load_item_record(const DecodeParams& p, int item) {
    const int per = p.kv_heads * p.head_groups;
    const int cg = item / per;
    if (p.mode == kModePlanned) return __ldg(p.items + cg);
    const int b = cg / p.splits;
    const int z = cg - b * p.splits;
    const int len = clamp_len(p, b);
    return make_int4(b, z, (int)(((long long)len * z) / p.splits),
                     (int)(((long long)len * (z + 1)) / p.splits));
}

__device__ __forceinline__ WorkItem item_from_record(const DecodeParams& p, int item, int4 rec) {
    WorkItem w;
    const int per = p.kv_heads * p.head_groups;
    const int cg = item / per;
    const int r = item - cg * per;
    w.kvh = r / p.head_groups;
    w.hg = r - w.kvh * p.head_groups;
    w.b = rec.x;
    w.part = rec.y & ~kSingleFlag;
    w.t0 = rec.z;
    w.t1 = rec.w;
    if (p.mode == kModePlanned) {
        w.n_parts = (rec.y & kSingleFlag) ? 1 : 2;   // only "one" vs "several" matters here
        w.part_slot = w.part;                         // chunk_off[b] + chunk index
    } else {
        w.n_parts = p.splits;
        w.part_slot = 0;
    }
    return w;
}

__device__ __forceinline__ WorkItem decode_item(const DecodeParams& p, int item) {
    return item_from_record(p, item, load_item_record(p, item));
}

// Programmatic dependent launch.  Every kernel of this library lets the next
// kernel in the stream start launching at once and then waits, in every thread
// and before its first global access, until the kernels before it have
// completed and flushed.  Because every CTA waits before it can exit, the chain
// plan -> decode -> merge -> (next call's) plan stays ordered end to end.  When
// a kernel is launched without the programmatic attribute both are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
    return __bfloat162float(x);
}
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Page id of token t of the staged segment, and its slot in the page.
__device__ __forceinline__ void token_page_slot(const DecodeParams& p, int t, int& page, int& slot) {
    if (p.bs_shift >= 0) {
        page = t >> p.bs_shift;
        slot = t & (p.block_size - 1);
    } else {
        page = t / p.block_size;
        slot = t - page * p.block_size;
    }
}

// Copy the page ids covering tokens [s0, s1) of sequence b into shared memory.
// Returns (via first_page) the table column of entry 0.  All threads call it.
__device__ __forceinline__ void stage_table(const DecodeParams& p, int b, int s0, int s1,
                                            int* s_table, int& first_page) {
    int pg0, pg1, slot;
    token_page_slot(p, s0, pg0, slot);
    token_page_slot(p, s1 - 1, pg1, slot);
    first_page = pg0;
    const int n = pg1 - pg0 + 1;
    const int32_t* row = p.table + (long long)b * p.max_pages + pg0;
    // A page id outside the pool (a caller error the reference leaves undefined)
    // is clamped so that it reads some valid page instead of faulting the device.
    const int last = (int)(p.num_blocks - 1);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        int pg = __ldg(row + i);
        pg = pg < 0 ? 0 : pg;
        s_table[i] = pg > last ? last : pg;
    }
}

// ---------------------------------------------------------------------------
// Combine the softmax states of the CTA's warps for one work item and store the
// result: to `out` when the sequence has a single partition, else as a partial.
//   s_o   warp wp's row r starts at s_o + wp*o_warp_stride + r*o_stride (fp32
//         words): un-normalised accumulators
//   s_m   [NWARPS][rows_alloc]            running max (log2 units), -inf if idle
//   s_l   [NWARPS][rows_alloc]            running sum
// Row r of the item is query head  kvh*group + hg*heads_per_item + r.
// VEC4: head_dim % 4 == 0 and out / partial rows are 16-byte (fp32) or 8-byte
// (16-bit) aligned.
// ---------------------------------------------------------------------------
template <typename T, int NWARPS, bool VEC4>
__device__ __forceinline__ void combine_and_store(const DecodeParams& p, const WorkItem& w,
                                                  const float* s_o, int o_warp_stride,
                                                  int o_stride, const float* s_m,
                                                  const float* s_l, int rows_alloc,
                                                  int rows_valid) {
    const int D = p.head_dim;
    const int head0 = w.kvh * p.group + w.hg * p.heads_per_item;
    const int per_row = VEC4 ? (D >> 2) : D;
    const int total = rows_valid * per_row;
    T* out = reinterpret_cast<T*>(p.out);
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int row = idx / per_row;
        const int col = (idx - row * per_row) * (VEC4 ? 4 : 1);
        float mx = -INFINITY;
#pragma unroll
        for (int wp = 0; wp < NWARPS; ++wp) mx = fmaxf(mx, s_m[wp * rows_alloc + row]);
        float sum = 0.f;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int wp = 0; wp < NWARPS; ++wp) {
            const float lw = s_l[wp * rows_alloc + row];
            if (lw > 0.f) {
                const float wgt = fast_exp2(s_m[wp * rows_alloc + row] - mx);
                sum += wgt * lw;
                const float* o = s_o + (size_t)wp * o_warp_stride + row * o_stride + col;
                if (VEC4) {
                    const float4 x = *reinterpret_cast<const float4*>(o);
                    a0 += wgt * x.x; a1 += wgt * x.y; a2 += wgt * x.z; a3 += wgt * x.w;
                } else {
                    a0 += wgt * o[0];
                }
            }
        }
        const int hq = head0 + row;
        if (w.n_parts == 1) {
            const float inv = sum > 0.f ? 1.f / sum : 0.f;
            T* dst = out + ((size_t)w.b * p.q_heads + hq) * D + col;
            if (VEC4) {
                if (sizeof(T) == 4) {
                    *reinterpret_cast<float4*>(dst) = make_float4(a0 * inv, a1 * inv, a2 * inv, a3 * inv);
                } else {
                    T tmp[4] = {from_f32<T>(a0 * inv), from_f32<T>(a1 * inv),
                                from_f32<T>(a2 * inv), from_f32<T>(a3 * inv)};
                    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(tmp);
                }
            } else {
                dst[0] = from_f32<T>(a0 * inv);
            }
        } else if (p.mode != kModeRefSplits) {
            const size_t slot = (size_t)w.part_slot * p.q_heads + hq;
            float* dst = p.part_acc + slot * D + col;
            if (VEC4) *reinterpret_cast<float4*>(dst) = make_float4(a0, a1, a2, a3);
            else dst[0] = a0;
            if (col == 0) p.part_ml[slot] = make_float2(mx, sum);
        } else {
            // reference layout [B, Hq, S, D + 2] = [max (natural units), sum, acc...]
            float* dst = p.ref_partials +
                         (((size_t)w.b * p.q_heads + hq) * p.splits + w.part) * (D + 2);
            if (VEC4) {
                dst[2 + col] = a0; dst[3 + col] = a1; dst[4 + col] = a2; dst[5 + col] = a3;
            } else {
                dst[2 + col] = a0;
            }
            if (col == 0) { dst[0] = mx * kLn2; dst[1] = sum; }
        }
    }
}

// An item with an empty token range (reference-split mode only: a sequence with
// fewer tokens than splits, or of length 0).  Its partial must still be defined
// because the caller's buffer is uninitialised; with a single partition the
// output row itself is zero (csrc/cuda/dense/gqa_decode.cu:65).
template <typename T>
__device__ __forceinline__ void store_empty(const DecodeParams& p, const WorkItem& w,
                                            int rows_valid) {
    const int D = p.head_dim;
    const int head0 = w.kvh * p.group + w.hg * p.heads_per_item;
    if (w.n_parts == 1) {
        T* out = reinterpret_cast<T*>(p.out);
        for (int idx = threadIdx.x; idx < rows_valid * D; idx += blockDim.x) {
            const int row = idx / D, col = idx - row * D;
            out[((size_t)w.b * p.q_heads + head0 + row) * D + col] = from_f32<T>(0.f);
        }
        return;
    }
    if (p.mode != kModeRefSplits) return;
    for (int idx = threadIdx.x; idx < rows_valid * (D + 2); idx += blockDim.x) {
        const int row = idx / (D + 2), col = idx - row * (D + 2);
        float* dst = p.ref_partials +
                     (((size_t)w.b * p.q_heads + head0 + row) * p.splits + w.part) * (D + 2);
        dst[col] = col == 0 ? -INFINITY : 0.f;
    }
}

}  // namespace gqa_b200

// One-launch ("fused") mode of the paged GQA decode kernels.
//
// The three-launch path spends a plan kernel before and a merge kernel after the
// decode kernel; on small batches and on the shards of a batch split over several
// GPUs those two launches are a large part of the call.  In fused mode there is one
// launch:
//   * every decode CTA derives the chunk list from context_lens itself (a block scan
//     over at most kFusedMaxBatch sequences into shared memory) and turns an item
//     number into (sequence, chunk) with a binary search;
//   * the partial of a chunk goes to its slot as before; when a CTA has run out of work it
//     takes a ticket of the (sequence, kv head, head group) of every multi-chunk item it
//     processed, and the CTA that draws a group's last ticket folds that group's partials
//     IN SLOT ORDER, so the bits do not depend on which CTA came last.  Nobody waits for
//     anybody: there is no spin anywhere;
//   * the work counter, the exit counter and the tickets are left at zero by the kernel
//     itself (the last arriver clears its ticket, the last CTA to leave clears the
//     counters), so the control words of a workspace are zeroed once, before its first use.
// The merge arithmetic repeats gqa_merge_kernel / gqa_merge_warp_kernel operation for
// operation (four interleaved running sums, added 0+1+2+3), so both paths give the same bits.
#pragma once

#include "gqa_common.cuh"

namespace gqa_b200 {

// Release / acquire fence at device scope (__threadfence() is the sequentially consistent one).
__device__ __forceinline__ void fence_acq_rel_gpu() {
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

struct FusedPlan {
    int base;           // base chunk length in tokens
    int total_chunks;   // chunks of the whole batch (an empty sequence counts one, empty, chunk)
};

// An empty sequence still gets one chunk, so that some CTA writes its zero row
// (csrc/cuda/dense/gqa_decode.cu:65).
__device__ __forceinline__ int fused_chunks_for(int len, int base) {
    const int n = chunks_for(len, base);
    return n < 1 ? 1 : n;
}

// Estimated cost, in token-times of one CTA, of cutting the batch at base 1024 >> i:
//   (items per resident CTA) x (per-item overhead: pipeline fill and drain, the combine,
//   the partial written and read back)  +  the expected idle tail at the end of the kernel,
//   about half of the longest item when CTAs pull items from a counter.
// The base with the lowest estimate wins; a base whose chunk total does not fit the
// workspace is not considered.  The two constants were fitted to measured call times at
// explicit bases 1024 .. 64 of the benchmark workloads (group 4 to 8, bf16 / fp16 / fp32, D 128)
// and of the quarter and the eighth of the skewed batch that one GPU of four or eight decodes:
// with 96 tokens per item every one of them gets its fastest base (with 64 the eighth, 2 - 6
// items per CTA, was cut at 256 and ran 66.8 us instead of 57.4).
constexpr float kFusedItemOverheadTokens = 96.f;
constexpr float kFusedTailFraction = 0.5f;

__device__ __forceinline__ int fused_pick_base(const int (&cnt)[kNumAutoBases], const int (&longest)[kNumAutoBases],
                                               int per, int slots, int cap_chunks) {
    int pick = 1024;
    float best = 3.0e38f;
#pragma unroll
    for (int i = 0; i < kNumAutoBases; ++i) {
        if (i > 0 && cnt[i] > cap_chunks) continue;
        const float items = (float)cnt[i] * (float)per;
        const float cost = items / (float)slots * kFusedItemOverheadTokens + kFusedTailFraction * (float)longest[i];
        if (cost < best) { best = cost; pick = 1024 >> i; }
    }
    return pick;
}

// All THREADS threads of the CTA.  Fills s_off[0 .. batch] with the exclusive prefix of
// chunks per sequence and s_off[batch + 1 + b] with the clamped length of sequence b (an item
// is then set up from shared memory alone), and returns the plan.
// s_red: scratch of 2 * kNumAutoBases * 32 + 32 ints.
template <int THREADS>
__device__ __forceinline__ FusedPlan fused_plan(const DecodeParams& p, int* s_off, int* s_red) {
    int* s_len = s_off + p.batch + 1;
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int base = p.chunk_base;
    int cnt[kNumAutoBases], longest[kNumAutoBases];
#pragma unroll
    for (int i = 0; i < kNumAutoBases; ++i) { cnt[i] = 0; longest[i] = 0; }
    for (int b = tid; b < p.batch; b += THREADS) {
        const int len = clamp_len(p, b);
        s_len[b] = len;
        if (base == 0) {
#pragma unroll
            for (int i = 0; i < kNumAutoBases; ++i) {
                cnt[i] += fused_chunks_for(len, 1024 >> i);
                const int ct = chunk_tokens_for(len, 1024 >> i);
                longest[i] = max(longest[i], min(len, ct));
            }
        }
    }
    if (base == 0) {
#pragma unroll
        for (int i = 0; i < kNumAutoBases; ++i) {
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) {
                cnt[i] += __shfl_xor_sync(0xffffffffu, cnt[i], d);
                longest[i] = max(longest[i], __shfl_xor_sync(0xffffffffu, longest[i], d));
            }
            if (lane == 0) {
                s_red[i * 32 + warp] = cnt[i];
                s_red[(kNumAutoBases + i) * 32 + warp] = longest[i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kNumAutoBases; ++i) {
            int c = 0, m = 0;
#pragma unroll
            for (int wp = 0; wp < NW; ++wp) {
                c += s_red[i * 32 + wp];
                m = max(m, s_red[(kNumAutoBases + i) * 32 + wp]);
            }
            cnt[i] = c;
            longest[i] = m;
        }
        base = fused_pick_base(cnt, longest, p.kv_heads * p.head_groups, (int)gridDim.x, p.cap_chunks);
    }
    __syncthreads();   // every length is in s_len; s_red is free again

    // exclusive prefix of chunks: each thread owns a contiguous run of sequences
    const int run = (p.batch + THREADS - 1) / THREADS;
    const int b0 = min(p.batch, tid * run), b1 = min(p.batch, b0 + run);
    int mine = 0;
    for (int b = b0; b < b1; ++b) mine += fused_chunks_for(s_len[b], base);
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += y;
    }
    int* s_warp = s_red + 2 * kNumAutoBases * 32;
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int wp = 0; wp < NW; ++wp) {
        const int x = s_warp[wp];
        if (wp < warp) before += x;
        total += x;
    }
    int at = before + incl - mine;
    for (int b = b0; b < b1; ++b) {
        s_off[b] = at;
        at += fused_chunks_for(s_len[b], base);
    }
    if (tid == 0) s_off[p.batch] = total;
    __syncthreads();
    if (blockIdx.x == 0) {
        // one CTA publishes the plan for the merge kernel that may follow (and for debugging);
        // every CTA computes the same one
        for (int b = tid; b <= p.batch; b += THREADS) p.chunk_off[b] = s_off[b];
        if (tid == 0) {
            p.hdr[kHdrTotalChunks] = total;
            p.hdr[kHdrChunkBase] = base;
            p.hdr[kHdrStatus] = total > p.cap_chunks ? 1 : 0;
        }
    }
    FusedPlan plan;
    plan.base = base;
    plan.total_chunks = total > p.cap_chunks ? p.cap_chunks : total;
    return plan;
}

// Item number -> work item.  Items are numbered chunk-major with the kv head fastest, as in
// the planned mode; the chunk's sequence is found by binary search in the prefix array.
__device__ __forceinline__ WorkItem fused_item(const DecodeParams& p, int item, const int* s_off, int base) {
    WorkItem w;
    const int per = p.kv_heads * p.head_groups;
    const int cg = item / per;
    const int r = item - cg * per;
    w.kvh = r / p.head_groups;
    w.hg = r - w.kvh * p.head_groups;
    int lo = 0, hi = p.batch;            // s_off[lo] <= cg < s_off[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= cg) lo = mid; else hi = mid;
    }
    w.b = lo;
    const int len = s_off[p.batch + 1 + lo];
    const int ct = chunk_tokens_for(len, base);
    w.part = cg - s_off[lo];
    const long long t0 = (long long)w.part * ct;
    w.t0 = (int)(t0 < len ? t0 : len);
    w.t1 = (int)(t0 + ct < len ? t0 + ct : len);
    w.n_parts = s_off[lo + 1] - s_off[lo];
    w.part_slot = cg;
    return w;
}

// Fold the partials of (sequence w.b, the rows of this item) into `out`.  Slot order, four
// interleaved running sums added 0+1+2+3: the arithmetic of gqa_merge_kernel.
template <typename T, bool VEC4>
__device__ __forceinline__ void fused_merge_rows(const DecodeParams& p, const WorkItem& w, int rows_valid) {
    constexpr int W = VEC4 ? 4 : 1;
    const int D = p.head_dim;
    const int head0 = w.kvh * p.group + w.hg * p.heads_per_item;
    const int per_row = VEC4 ? (D >> 2) : D;
    const int total = rows_valid * per_row;
    const int n = w.n_parts;
    const size_t first = (size_t)(w.part_slot - w.part);
    const size_t ml_step = p.q_heads, acc_step = (size_t)p.q_heads * D;
    T* out = reinterpret_cast<T*>(p.out);
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int row = idx / per_row;
        const int col = (idx - row * per_row) * W;
        const int hq = head0 + row;
        const float2* ml = p.part_ml + first * p.q_heads + hq;
        const float* acc = p.part_acc + (first * p.q_heads + hq) * D + col;
        // (loads are issued in batches of eight chunks: a long sequence has up to 64 partials,
        // and the merge of the last sequence to finish is on the kernel's critical path)
        float mx = -INFINITY;
#pragma unroll 8
        for (int c = 0; c < n; ++c) {
            const float2 u = __ldcg(ml + c * ml_step);
            if (u.y > 0.f) mx = fmaxf(mx, u.x);
        }
        float a[4][W], sum[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sum[j] = 0.f;
#pragma unroll
            for (int k = 0; k < W; ++k) a[j][k] = 0.f;
        }
        for (int cb = 0; cb < n; cb += 8) {
            float2 u[8];
            float x[8][W];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool live = cb + j < n;
                u[j] = live ? __ldcg(ml + (cb + j) * ml_step) : make_float2(-INFINITY, 0.f);
                const float* src = acc + (cb + j) * acc_step;
                if constexpr (VEC4) {
                    const float4 v = live ? __ldcg(reinterpret_cast<const float4*>(src))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                    x[j][0] = v.x; x[j][1] = v.y; x[j][2] = v.z; x[j][3] = v.w;
                } else {
                    x[j][0] = live ? __ldcg(src) : 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {      // chunk cb + j goes to running sum (cb + j) mod 4 = j mod 4
                if (u[j].y > 0.f) {
                    const float wgt = fast_exp2(u[j].x - mx);
                    sum[j & 3] += wgt * u[j].y;
#pragma unroll
                    for (int k = 0; k < W; ++k) a[j & 3][k] += wgt * x[j][k];
                }
            }
        }
        auto fold = [](float s0, float s1, float s2, float s3) { return ((0.f + s0) + s1 + s2) + s3; };
        const float tot = fold(sum[0], sum[1], sum[2], sum[3]);
        const float inv = tot > 0.f ? 1.f / tot : 0.f;
        float r[W];
#pragma unroll
        for (int k = 0; k < W; ++k) r[k] = fold(a[0][k], a[1][k], a[2][k], a[3][k]) * inv;
        T* dst = out + ((size_t)w.b * p.q_heads + hq) * D + col;
        if constexpr (VEC4) {
            if (sizeof(T) == 4) {
                *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
            } else {
                T tmp[4] = {from_f32<T>(r[0]), from_f32<T>(r[1]), from_f32<T>(r[2]), from_f32<T>(r[3])};
                *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(tmp);
            }
        } else {
            dst[0] = from_f32<T>(r[0]);
        }
    }
}

// The same fold with the partials staged through shared memory: the rows of one item are
// adjacent query heads, so their accumulators in one partial slot are one contiguous run of
// rows_valid x D floats, fetched with 16-byte cp.async copies that bypass L1.  A round brings
// as many slots as fit (tens of KB in flight per CTA instead of a few loads per thread); a
// long sequence has up to 64 partials of 4 KB, and the merge of the last sequence to finish
// is on the kernel's critical path.  `smem`: free shared memory, 16-byte aligned; the caller
// checks fused_merge_fits_smem.  All threads of the CTA; head_dim % 4 == 0.
__device__ __forceinline__ bool fused_merge_fits_smem(const DecodeParams& p, int n_parts, int rows_valid,
                                                      int threads, int smem_bytes) {
    const int d4 = p.head_dim >> 2;
    const int rb = threads / d4 > 0 ? threads / d4 : 1;
    const long long ml_bytes = (((long long)rows_valid * n_parts * 8) + 15) & ~15ll;
    return threads % d4 == 0 && ml_bytes + 4ll * rb * p.head_dim * 4 <= smem_bytes;
}

template <typename T>
__device__ __forceinline__ void fused_merge_rows_staged(const DecodeParams& p, const WorkItem& w, int rows_valid,
                                                        unsigned char* smem, int smem_bytes) {
    const int D = p.head_dim, D4 = D >> 2, n = w.n_parts;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int head0 = w.kvh * p.group + w.hg * p.heads_per_item;
    const size_t first = (size_t)(w.part_slot - w.part);
    float2* s_ml = reinterpret_cast<float2*>(smem);                    // [rows_valid][n]
    const int ml_bytes = ((rows_valid * n * 8) + 15) & ~15;
    float4* s_acc = reinterpret_cast<float4*>(smem + ml_bytes);       // [slots of a round][RB][D4]
    const int RB = nthr / D4;                                          // rows per batch
    const int per_round = ((smem_bytes - ml_bytes) / (RB * D * 4)) & ~3;   // slots per round, multiple of 4
    T* out = reinterpret_cast<T*>(p.out);

    for (int i = tid; i < rows_valid * n; i += nthr) {
        const int row = i / n, c = i - row * n;
        s_ml[i] = __ldcg(p.part_ml + (first + c) * p.q_heads + head0 + row);
    }
    __syncthreads();
    for (int rb = 0; rb < rows_valid; rb += RB) {
        const int nrows = min(RB, rows_valid - rb);
        const int row = rb + tid / D4, col = (tid % D4) * 4;
        const bool act = tid < nrows * D4;
        const float2* my_ml = s_ml + (act ? row : 0) * n;
        float mx = -INFINITY;
        if (act) {
            for (int c = 0; c < n; ++c) {
                const float2 u = my_ml[c];
                if (u.y > 0.f) mx = fmaxf(mx, u.x);
            }
        }
        float a[4][4], sum[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { sum[j] = 0.f; a[j][0] = a[j][1] = a[j][2] = a[j][3] = 0.f; }
        const int ppc = nrows * D4;                                    // 16-byte pieces per slot
        for (int r0 = 0; r0 < n; r0 += per_round) {
            const int cnt = min(per_round, n - r0);
            for (int i = tid; i < cnt * ppc; i += nthr) {
                const int c = i / ppc, rem = i - c * ppc;
                const float* src = p.part_acc + ((first + r0 + c) * p.q_heads + head0 + rb) * D + rem * 4;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_acc + c * (RB * D4) + rem);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            __syncthreads();
            if (act) {
                for (int cb = 0; cb < cnt; cb += 4) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {      // slot r0 + cb + j goes to running sum j (r0, cb multiples of 4)
                        if (cb + j < cnt) {
                            const float2 u = my_ml[r0 + cb + j];
                            if (u.y > 0.f) {
                                const float wgt = fast_exp2(u.x - mx);
                                const float4 x = s_acc[(cb + j) * (RB * D4) + tid];
                                sum[j] += wgt * u.y;
                                a[j][0] += wgt * x.x; a[j][1] += wgt * x.y;
                                a[j][2] += wgt * x.z; a[j][3] += wgt * x.w;
                            }
                        }
                    }
                }
            }
            __syncthreads();                           // the round's slots may be overwritten
        }
        if (act) {
            auto fold = [](float s0, float s1, float s2, float s3) { return ((0.f + s0) + s1 + s2) + s3; };
            const float tot = fold(sum[0], sum[1], sum[2], sum[3]);
            const float inv = tot > 0.f ? 1.f / tot : 0.f;
            float r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) r[k] = fold(a[0][k], a[1][k], a[2][k], a[3][k]) * inv;
            T* dst = out + ((size_t)w.b * p.q_heads + head0 + row) * D + col;
            if (sizeof(T) == 4) {
                *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
            } else {
                T tmp[4] = {from_f32<T>(r[0]), from_f32<T>(r[1]), from_f32<T>(r[2]), from_f32<T>(r[3])};
                *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(tmp);
            }
        }
    }
}

// The ticket protocol.  A release fence followed by an atomic costs its thread, and through
// the next CTA barrier the whole CTA, one to two microseconds: measured per multi-chunk item,
// that was 5 % of a long-context call.  So tickets are not taken item by item.  A CTA keeps a
// list (shared memory) of the multi-chunk items whose partial it has stored, and takes all
// their tickets together when it has run out of work (or when the list is full): one barrier,
// then one thread per list entry fences and takes that entry's ticket, in parallel.  For
// every entry that turned out to be the last arrival the CTA then merges the sequence.
// All CTAs run out of work at about the same time, so the merges of a call run side by side
// on as many CTAs as there are (sequence, kv head) groups, after the streaming.
constexpr int kFusedMaxPending = 32;

struct FusedPending {
    int4 rec[kFusedMaxPending];    // (sequence, kv head * head_groups + head group, partials, first slot)
    int last[kFusedMaxPending];
};

// thread 0, after the item's closing barrier was passed by everyone
__device__ __forceinline__ void fused_note_item(FusedPending& pd, int n, const DecodeParams& p, const WorkItem& w) {
    pd.rec[n] = make_int4(w.b, w.kvh * p.head_groups + w.hg, w.n_parts, (int)(w.part_slot - w.part));
}

// All threads of the CTA.  STAGED: merge through `smem` (free shared memory, 16-byte aligned).
template <typename T, bool VEC4, bool STAGED>
__device__ __forceinline__ void fused_flush_tickets(const DecodeParams& p, FusedPending& pd, int n_pend,
                                                    unsigned char* smem, int smem_bytes) {
    if (n_pend == 0) return;
    __syncthreads();                    // the list is written; every partial of its items was stored
                                        // before an earlier barrier
    if ((int)threadIdx.x < n_pend) {
        const int4 r = pd.rec[threadIdx.x];
        int32_t* t = p.tickets + ((size_t)r.x * p.kv_heads * p.head_groups + r.y);
        fence_acq_rel_gpu();            // release: cumulative over what the barriers showed this thread
        const int old = atomicAdd(t, 1);
        const int last = old == r.z - 1;
        if (last) *t = 0;               // nobody else comes to this ticket in this call
        pd.last[threadIdx.x] = last;
    }
    __syncthreads();
    for (int i = 0; i < n_pend; ++i) {
        if (!pd.last[i]) continue;      // (uniform: shared memory)
        const int4 r = pd.rec[i];
        WorkItem w;
        w.b = r.x;
        w.kvh = r.y / p.head_groups;
        w.hg = r.y - w.kvh * p.head_groups;
        w.n_parts = r.z;
        w.part = 0;
        w.part_slot = r.w;
        w.t0 = w.t1 = 0;
        const int rows_valid = min(p.heads_per_item, p.group - w.hg * p.heads_per_item);
        fence_acq_rel_gpu();            // acquire: the other CTAs' partials, published before their tickets
        if constexpr (STAGED) {
            if (fused_merge_fits_smem(p, w.n_parts, rows_valid, (int)blockDim.x, smem_bytes)) {
                fused_merge_rows_staged<T>(p, w, rows_valid, smem, smem_bytes);
                continue;
            }
        }
        fused_merge_rows<T, VEC4>(p, w, rows_valid);
    }
    __syncthreads();                    // the list and the staging memory are free again
}

// Last statement of a decode kernel that pulled items from the work counter: the CTA that
// leaves last puts the counters back to zero.
__device__ __forceinline__ void decode_counters_release(const DecodeParams& p) {
    if (threadIdx.x != 0) return;
    fence_acq_rel_gpu();
    const int old = atomicAdd(p.hdr + kHdrDone, 1);
    if (old == (int)gridDim.x - 1) {
        p.hdr[kHdrCounter] = 0;
        p.hdr[kHdrDone] = 0;
    }
}

}  // namespace gqa_b200

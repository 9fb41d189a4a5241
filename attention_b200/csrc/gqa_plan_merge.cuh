// Plan kernel (cuts sequences into KV chunks on the device) and the
// log-sum-exp merge kernel that folds chunk partials into the output.
#pragma once

#include "gqa_common.cuh"

namespace gqa_b200 {

constexpr int kPlanThreads = 1024;

// Block-wide inclusive scan of one int per thread (kPlanThreads threads).
__device__ __forceinline__ int plan_block_scan(int x, int* s_warp, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
    }
    __syncthreads();                 // s_warp free from the previous use
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    if (warp == 0) {
        int t = s_warp[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, t, d);
            if (lane >= d) t += y;
        }
        s_warp[lane] = t;
    }
    __syncthreads();
    total = s_warp[kPlanThreads / 32 - 1];
    return x + (warp ? s_warp[warp - 1] : 0);
}

// One CTA.  Reads context_lens and writes, without any host read of the lengths:
//   the base chunk length, when the caller left it open (chunk_base == 0): the
//                 largest of 1024, 512, ... 64 for which the batch's ACTUAL
//                 lengths give at least item_target chunks, i.e. enough work items
//                 to occupy every resident decode CTA; a block table much wider
//                 than the sequences in it therefore costs nothing
//   chunk_off[b]  exclusive prefix of chunks per sequence = first partial slot of b
//   items[]       one record per chunk, in sequence order.  (Putting all short
//                 last chunks at the end of the list was measured slower: equal
//                 items make every CTA start and drain its copy pipeline at the
//                 same moments.)
//   hdr           chunk total, status, chosen base, and the zeroed work counter
__global__ void __launch_bounds__(kPlanThreads) gqa_plan_kernel(const DecodeParams p) {
    __shared__ int s_warp[kPlanThreads / 32];
    __shared__ int s_cand[kNumAutoBases][kPlanThreads / 32];
    __shared__ int s_base;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int base_tokens = p.chunk_base;
    if (base_tokens == 0) {
        int cnt[kNumAutoBases];
#pragma unroll
        for (int i = 0; i < kNumAutoBases; ++i) cnt[i] = 0;
        for (int b = tid; b < p.batch; b += kPlanThreads) {
            const int len = clamp_len(p, b);
#pragma unroll
            for (int i = 0; i < kNumAutoBases; ++i) cnt[i] += chunks_for(len, 1024 >> i);
        }
#pragma unroll
        for (int i = 0; i < kNumAutoBases; ++i) {
            int x = cnt[i];
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
            if (lane == 0) s_cand[i][warp] = x;
        }
        __syncthreads();
        if (warp == 0) {
            int pick = 1024 >> (kNumAutoBases - 1);
            bool found = false;
#pragma unroll
            for (int i = 0; i < kNumAutoBases; ++i) {
                int x = s_cand[i][lane];
#pragma unroll
                for (int d = 16; d >= 1; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
                if (!found && x >= p.item_target) { pick = 1024 >> i; found = true; }
            }
            if (lane == 0) s_base = pick;
        }
        __syncthreads();
        base_tokens = s_base;
    }
    int run_n = 0;
    for (int base = 0; base < p.batch; base += kPlanThreads) {
        const int b = base + tid;
        const int len = b < p.batch ? clamp_len(p, b) : 0;
        const int n = chunks_for(len, base_tokens);
        int tot_n;
        const int incl_n = plan_block_scan(n, s_warp, tot_n);
        if (b < p.batch) {
            const int co = run_n + incl_n - n;
            p.chunk_off[b] = co;
            const int ct = chunk_tokens_for(len, base_tokens);
            const int flag = n == 1 ? kSingleFlag : 0;
            for (int c = 0; c < n; ++c) {
                const long long t0 = (long long)c * ct;
                const int t1 = (int)(t0 + ct < len ? t0 + ct : len);
                if (co + c < p.cap_chunks)
                    p.items[co + c] = make_int4(b, (co + c) | flag, (int)t0, t1);
            }
        }
        run_n += tot_n;
    }
    if (tid == 0) {
        p.chunk_off[p.batch] = run_n;
        p.hdr[kHdrTotalChunks] = run_n;
        p.hdr[kHdrCounter] = 0;
        p.hdr[kHdrDone] = 0;
        p.hdr[kHdrStatus] = run_n > p.cap_chunks ? 1 : 0;
        p.hdr[kHdrChunkBase] = base_tokens;
    }
}

constexpr int kMergeWarps = 4;

// One CTA per (sequence, query head).  Sequences with one chunk were written by
// the decode kernel; empty sequences get their zero row here
// (csrc/cuda/dense/gqa_decode.cu:65,86); the rest fold their partials:
//   out = sum_c 2^(m_c - M) acc_c / sum_c 2^(m_c - M) l_c,  M = max_c m_c,
// which equals the reference's left-to-right SoftmaxState::merge
// (csrc/cuda/common/online_softmax.cuh:17-24) up to fp32 rounding.
// In reference-split mode the partials are read from the caller's
// [B, Hq, S, D+2] buffer with max in natural units.
template <typename T, bool VEC4>
__global__ void __launch_bounds__(kMergeWarps * 32) gqa_merge_kernel(const DecodeParams p) {
    pdl_launch_dependents();
    pdl_wait();
    // 1-D grid of batch * q_heads CTAs (no 65535 limit on the batch)
    const int b = blockIdx.x / p.q_heads, hq = blockIdx.x - b * p.q_heads;
    const int D = p.head_dim;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    T* out = reinterpret_cast<T*>(p.out) + ((size_t)b * p.q_heads + hq) * D;

    int n_parts;
    size_t first_slot = 0;
    if (p.mode == kModePlanned) {
        const int c0 = p.chunk_off[b];
        n_parts = p.chunk_off[b + 1] - c0;
        if (c0 + n_parts > p.cap_chunks) n_parts = p.cap_chunks > c0 ? p.cap_chunks - c0 : 0;
        first_slot = (size_t)c0;
        if (n_parts == 1) return;
    } else {
        n_parts = p.splits;
    }
    if (n_parts == 0) {
        for (int c = tid; c < D; c += blockDim.x) out[c] = from_f32<T>(0.f);
        return;
    }
    auto part_m = [&](int c) -> float {
        if (p.mode == kModePlanned) return p.part_ml[(first_slot + c) * p.q_heads + hq].x;
        return p.ref_partials[(((size_t)b * p.q_heads + hq) * p.splits + c) * (D + 2)] * kLog2e;
    };
    auto part_l = [&](int c) -> float {
        if (p.mode == kModePlanned) return p.part_ml[(first_slot + c) * p.q_heads + hq].y;
        return p.ref_partials[(((size_t)b * p.q_heads + hq) * p.splits + c) * (D + 2) + 1];
    };
    auto part_acc = [&](int c) -> const float* {
        if (p.mode == kModePlanned) return p.part_acc + ((first_slot + c) * p.q_heads + hq) * D;
        return p.ref_partials + (((size_t)b * p.q_heads + hq) * p.splits + c) * (D + 2) + 2;
    };

    __shared__ float s_red[kMergeWarps];
    __shared__ float s_acc[kMergeWarps][256 + 4];
    __shared__ float s_sum[kMergeWarps];

    // global max over partitions that hold tokens
    float mx = -INFINITY;
    for (int c = tid; c < n_parts; c += blockDim.x)
        if (part_l(c) > 0.f) mx = fmaxf(mx, part_m(c));
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
#pragma unroll
    for (int wp = 1; wp < kMergeWarps; ++wp) mx = fmaxf(mx, s_red[wp]);

    // each warp folds partitions warp, warp + kMergeWarps, ...; lanes own columns
    constexpr int kCols = VEC4 ? 2 : 8;   // VEC4: float4 x 2 x 32 lanes = 256 columns
    float acc[kCols][VEC4 ? 4 : 1];
#pragma unroll
    for (int i = 0; i < kCols; ++i)
#pragma unroll
        for (int j = 0; j < (VEC4 ? 4 : 1); ++j) acc[i][j] = 0.f;
    float sum = 0.f;
    // The warp's partitions are fetched four at a time: all loads of a batch are issued before
    // the first is used (a long sequence has up to 64 partitions; one dependent round trip per
    // partition is what the kernel's duration used to consist of).  The additions stay in
    // partition order.
    constexpr int kBatch = 4;
    for (int cb = warp; cb < n_parts; cb += kMergeWarps * kBatch) {
        float lw[kBatch], mw[kBatch];
        float x[kBatch][kCols][VEC4 ? 4 : 1];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int c = cb + u * kMergeWarps;
            const bool live = c < n_parts;
            lw[u] = live ? part_l(c) : 0.f;
            mw[u] = live ? part_m(c) : -INFINITY;
            const float* src = part_acc(live ? c : 0);
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
                if constexpr (VEC4) {
                    const int col = (i * 32 + lane) * 4;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (live && col < D) v = *reinterpret_cast<const float4*>(src + col);
                    x[u][i][0] = v.x; x[u][i][1] = v.y; x[u][i][2] = v.z; x[u][i][3] = v.w;
                } else {
                    const int col = i * 32 + lane;
                    x[u][i][0] = (live && col < D) ? src[col] : 0.f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            if (!(lw[u] > 0.f)) continue;
            const float wgt = fast_exp2(mw[u] - mx);
            sum += wgt * lw[u];
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
#pragma unroll
                for (int j = 0; j < (VEC4 ? 4 : 1); ++j) acc[i][j] += wgt * x[u][i][j];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kCols; ++i) {
#pragma unroll
        for (int j = 0; j < (VEC4 ? 4 : 1); ++j) {
            const int col = VEC4 ? (i * 32 + lane) * 4 + j : i * 32 + lane;
            if (col < D) s_acc[warp][col] = acc[i][j];
        }
    }
    if (lane == 0) s_sum[warp] = sum;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int wp = 0; wp < kMergeWarps; ++wp) tot += s_sum[wp];
    const float inv = tot > 0.f ? 1.f / tot : 0.f;
    for (int col = tid; col < D; col += blockDim.x) {
        float x = 0.f;
#pragma unroll
        for (int wp = 0; wp < kMergeWarps; ++wp) x += s_acc[wp][col];
        out[col] = from_f32<T>(x * inv);
    }
}

// Planned-mode merge for short sequences (few chunks each): one WARP per
// (sequence, query head), four pairs per CTA; lanes own float4 columns.  The
// chunk count and first partial slot come from chunk_off (one round trip) and
// four partial rows are fetched at a time, so a sequence of up to four chunks
// costs two dependent memory round trips.  head_dim % 4 == 0.
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32) gqa_merge_warp_kernel(const DecodeParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long pair = (long long)blockIdx.x * kMergeWarps + warp;
    if (pair >= (long long)p.batch * p.q_heads) return;
    const int b = (int)(pair / p.q_heads), hq = (int)(pair - (long long)b * p.q_heads);
    const int D = p.head_dim;
    const int c0 = p.chunk_off[b];
    int n = p.chunk_off[b + 1] - c0;
    if (c0 + n > p.cap_chunks) n = p.cap_chunks > c0 ? p.cap_chunks - c0 : 0;
    if (n == 1) return;
    T* out = reinterpret_cast<T*>(p.out) + ((size_t)b * p.q_heads + hq) * D;
    const int col0 = lane * 4, col1 = (32 + lane) * 4;
    const bool use0 = col0 < D, use1 = col1 < D;
    auto store4 = [&](int col, float x0, float x1, float x2, float x3) {
        if (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(out + col) = make_float4(x0, x1, x2, x3);
        } else {
            T tmp[4] = {from_f32<T>(x0), from_f32<T>(x1), from_f32<T>(x2), from_f32<T>(x3)};
            *reinterpret_cast<uint2*>(out + col) = *reinterpret_cast<const uint2*>(tmp);
        }
    };
    if (n == 0) {
        if (use0) store4(col0, 0.f, 0.f, 0.f, 0.f);
        if (use1) store4(col1, 0.f, 0.f, 0.f, 0.f);
        return;
    }
    const size_t slot0 = (size_t)c0;
    const float2* ml = p.part_ml + slot0 * p.q_heads + hq;
    const float* acc = p.part_acc + (slot0 * p.q_heads + hq) * D;
    const size_t ml_step = p.q_heads, acc_step = (size_t)p.q_heads * D;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    // first four partial rows in flight before anything depends on them
    float2 v[4];
    float4 x0[4], x1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const bool live = j < n;
        v[j] = live ? ml[j * ml_step] : make_float2(-INFINITY, 0.f);
        const float* src = acc + j * acc_step;
        x0[j] = live && use0 ? *reinterpret_cast<const float4*>(src + col0) : zero4;
        x1[j] = live && use1 ? *reinterpret_cast<const float4*>(src + col1) : zero4;
    }
    // global max over chunks that hold tokens (chunks 4.. only exist for longer sequences)
    float mx = -INFINITY;
    for (int c = 4 + lane; c < n; c += 32) {
        const float2 u = ml[c * ml_step];
        if (u.y > 0.f) mx = fmaxf(mx, u.x);
    }
    if (n > 4) {
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (v[j].y > 0.f) mx = fmaxf(mx, v[j].x);
    // Four interleaved running sums (chunks c = j mod 4), added 0+1+2+3 at the end: the
    // same order of additions as the CTA-per-pair kernel, whose warp j folds those chunks,
    // so the two merge kernels give identical bits.
    float4 a0[4], a1[4];
    float sum[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { a0[j] = zero4; a1[j] = zero4; sum[j] = 0.f; }
    for (int cb = 0; cb < n; cb += 4) {
        if (cb > 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool live = cb + j < n;
                v[j] = live ? ml[(cb + j) * ml_step] : make_float2(-INFINITY, 0.f);
                const float* src = acc + (cb + j) * acc_step;
                x0[j] = live && use0 ? *reinterpret_cast<const float4*>(src + col0) : zero4;
                x1[j] = live && use1 ? *reinterpret_cast<const float4*>(src + col1) : zero4;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (v[j].y > 0.f) {
                const float wgt = fast_exp2(v[j].x - mx);
                sum[j] += wgt * v[j].y;
                a0[j].x += wgt * x0[j].x; a0[j].y += wgt * x0[j].y;
                a0[j].z += wgt * x0[j].z; a0[j].w += wgt * x0[j].w;
                a1[j].x += wgt * x1[j].x; a1[j].y += wgt * x1[j].y;
                a1[j].z += wgt * x1[j].z; a1[j].w += wgt * x1[j].w;
            }
        }
    }
    auto fold = [](float s0, float s1, float s2, float s3) { return ((0.f + s0) + s1 + s2) + s3; };
    const float tot = fold(sum[0], sum[1], sum[2], sum[3]);
    const float inv = tot > 0.f ? 1.f / tot : 0.f;
    if (use0)
        store4(col0, fold(a0[0].x, a0[1].x, a0[2].x, a0[3].x) * inv,
               fold(a0[0].y, a0[1].y, a0[2].y, a0[3].y) * inv,
               fold(a0[0].z, a0[1].z, a0[2].z, a0[3].z) * inv,
               fold(a0[0].w, a0[1].w, a0[2].w, a0[3].w) * inv);
    if (use1)
        store4(col1, fold(a1[0].x, a1[1].x, a1[2].x, a1[3].x) * inv,
               fold(a1[0].y, a1[1].y, a1[2].y, a1[3].y) * inv,
               fold(a1[0].z, a1[1].z, a1[2].z, a1[3].z) * inv,
               fold(a1[0].w, a1[1].w, a1[2].w, a1[3].w) * inv);
}

}  // namespace gqa_b200

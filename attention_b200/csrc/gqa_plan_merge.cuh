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
//   chunk_off[b]  exclusive prefix of chunks per sequence (position of the
//                 sequence's records in the item list)
//   items[]       one record per chunk, in sequence order.  (Putting all short
//                 last chunks at the end of the list was measured slower: equal
//                 items make every CTA start and drain its copy pipeline at the
//                 same moments.)
//   hdr           chunk total, status, and the zeroed work counter
__global__ void __launch_bounds__(kPlanThreads) gqa_plan_kernel(const DecodeParams p) {
    __shared__ int s_warp[kPlanThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    int run_n = 0;
    for (int base = 0; base < p.batch; base += kPlanThreads) {
        const int b = base + tid;
        const int len = b < p.batch ? clamp_len(p, b) : 0;
        const int n = chunks_for(len, p.chunk_base);
        int tot_n;
        const int incl_n = plan_block_scan(n, s_warp, tot_n);
        if (b < p.batch) {
            const int co = run_n + incl_n - n;
            p.chunk_off[b] = co;
            const int ct = chunk_tokens_for(len, p.chunk_base);
            const int flag = n == 1 ? kSingleFlag : 0;
            const int slot0 = b * p.slots_per_seq;
            for (int c = 0; c < n && c < p.slots_per_seq; ++c) {
                const long long t0 = (long long)c * ct;
                const int t1 = (int)(t0 + ct < len ? t0 + ct : len);
                if (co + c < p.cap_chunks)
                    p.items[co + c] = make_int4(b, (slot0 + c) | flag, (int)t0, t1);
            }
        }
        run_n += tot_n;
    }
    if (tid == 0) {
        p.chunk_off[p.batch] = run_n;
        p.hdr[kHdrTotalChunks] = run_n;
        p.hdr[kHdrCounter] = 0;
        p.hdr[kHdrStatus] = run_n > p.cap_chunks ? 1 : 0;
    }
}

constexpr int kMergeWarps = 4;

// One CTA per (query head, sequence).  Sequences with one chunk were written by
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
    const int hq = blockIdx.x, b = blockIdx.y;
    const int D = p.head_dim;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    T* out = reinterpret_cast<T*>(p.out) + ((size_t)b * p.q_heads + hq) * D;

    int n_parts;
    size_t first_slot = 0;
    if (p.mode == kModePlanned) {
        n_parts = chunks_for(clamp_len(p, b), p.chunk_base);
        if (n_parts > p.slots_per_seq) n_parts = p.slots_per_seq;
        first_slot = (size_t)b * p.slots_per_seq;
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
    for (int c = warp; c < n_parts; c += kMergeWarps) {
        const float lw = part_l(c);
        if (!(lw > 0.f)) continue;
        const float wgt = fast_exp2(part_m(c) - mx);
        sum += wgt * lw;
        const float* src = part_acc(c);
#pragma unroll
        for (int i = 0; i < kCols; ++i) {
            if (VEC4) {
                const int col = (i * 32 + lane) * 4;
                if (col < D) {
                    const float4 x = *reinterpret_cast<const float4*>(src + col);
                    acc[i][0] += wgt * x.x; acc[i][1] += wgt * x.y;
                    acc[i][2] += wgt * x.z; acc[i][3] += wgt * x.w;
                }
            } else {
                const int col = i * 32 + lane;
                if (col < D) acc[i][0] += wgt * src[col];
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
// chunk count comes from the sequence's own length (one load), the partial
// slots are at a fixed place per sequence, and four partial rows are fetched at
// a time, so a sequence of up to four chunks costs two dependent memory round
// trips.  Batches are folded with a running max.  head_dim % 4 == 0.
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32) gqa_merge_warp_kernel(const DecodeParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long pair = (long long)blockIdx.x * kMergeWarps + warp;
    if (pair >= (long long)p.batch * p.q_heads) return;
    const int b = (int)(pair / p.q_heads), hq = (int)(pair - (long long)b * p.q_heads);
    const int D = p.head_dim;
    int n = chunks_for(clamp_len(p, b), p.chunk_base);
    if (n > p.slots_per_seq) n = p.slots_per_seq;
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
    const size_t slot0 = (size_t)b * p.slots_per_seq;
    const float2* ml = p.part_ml + slot0 * p.q_heads + hq;
    const float* acc = p.part_acc + (slot0 * p.q_heads + hq) * D;
    const size_t ml_step = p.q_heads, acc_step = (size_t)p.q_heads * D;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 a0 = zero4, a1 = zero4;
    float mx = -INFINITY, sum = 0.f;
    for (int c0 = 0; c0 < n; c0 += 4) {
        float2 v[4];
        float4 x0[4], x1[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const bool live = c0 + j < n;
            v[j] = live ? ml[(c0 + j) * ml_step] : make_float2(-INFINITY, 0.f);
            const float* src = acc + (c0 + j) * acc_step;
            x0[j] = live && use0 ? *reinterpret_cast<const float4*>(src + col0) : zero4;
            x1[j] = live && use1 ? *reinterpret_cast<const float4*>(src + col1) : zero4;
        }
        float bm = mx;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (v[j].y > 0.f) bm = fmaxf(bm, v[j].x);
        const float r = sum > 0.f ? fast_exp2(mx - bm) : 0.f;
        sum *= r;
        a0.x *= r; a0.y *= r; a0.z *= r; a0.w *= r;
        a1.x *= r; a1.y *= r; a1.z *= r; a1.w *= r;
        mx = bm;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float wgt = v[j].y > 0.f ? fast_exp2(v[j].x - mx) : 0.f;
            sum += wgt * v[j].y;
            a0.x += wgt * x0[j].x; a0.y += wgt * x0[j].y; a0.z += wgt * x0[j].z; a0.w += wgt * x0[j].w;
            a1.x += wgt * x1[j].x; a1.y += wgt * x1[j].y; a1.z += wgt * x1[j].z; a1.w += wgt * x1[j].w;
        }
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    if (use0) store4(col0, a0.x * inv, a0.y * inv, a0.z * inv, a0.w * inv);
    if (use1) store4(col1, a1.x * inv, a1.y * inv, a1.z * inv, a1.w * inv);
}

}  // namespace gqa_b200

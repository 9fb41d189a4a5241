// Plan kernel (cuts sequences into KV chunks on the device) and the
// log-sum-exp merge kernel that folds chunk partials into the output.
#pragma once

#include "gqa_common.cuh"

namespace gqa_b200 {

constexpr int kPlanThreads = 1024;

// One CTA.  Reads context_lens, writes the exclusive prefix of chunks per
// sequence, the (sequence, chunk) item list, the total, and zeroes the decode
// kernel's work counter.  No host read of the lengths is ever needed.
__global__ void __launch_bounds__(kPlanThreads) gqa_plan_kernel(const DecodeParams p) {
    __shared__ int s_warp[kPlanThreads / 32];
    __shared__ int s_running;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_running = 0;
    __syncthreads();
    for (int base = 0; base < p.batch; base += kPlanThreads) {
        const int b = base + tid;
        const int n = b < p.batch ? chunks_for(clamp_len(p, b), p.chunk_base) : 0;
        int incl = n;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += y;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int x = s_warp[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, x, d);
                if (lane >= d) x += y;
            }
            s_warp[lane] = x;   // inclusive prefix of warp totals
        }
        __syncthreads();
        const int running = s_running;
        const int off = running + (warp ? s_warp[warp - 1] : 0) + incl - n;
        if (b < p.batch) {
            p.chunk_off[b] = off;
            for (int c = 0; c < n; ++c)
                if (off + c < p.cap_chunks) p.items[off + c] = make_int2(b, c);
        }
        __syncthreads();
        if (tid == 0) s_running = running + s_warp[kPlanThreads / 32 - 1];
        __syncthreads();
    }
    if (tid == 0) {
        const int total = s_running;
        p.chunk_off[p.batch] = total;
        p.hdr[kHdrTotalChunks] = total;
        p.hdr[kHdrCounter] = 0;
        p.hdr[kHdrStatus] = total > p.cap_chunks ? 1 : 0;
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
    const int hq = blockIdx.x, b = blockIdx.y;
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

}  // namespace gqa_b200

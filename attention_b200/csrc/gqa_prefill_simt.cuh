// Dense (non-paged) GQA prefill, SIMT kernel: q [B,Tq,Hq,D], k/v [B,Tk,Hkv,D],
// per-sequence q_lens / kv_lens, right-aligned causal mask (query row i of a
// sequence sees keys 0 .. kv_len - q_len + i).  Handles every dtype, head_dim in
// [1,256] and any alignment; it is the only prefill kernel for float32 and for
// shapes the tensor-core kernels reject.
//
// A warp owns kPrefillRows consecutive query rows of one head: every K/V row it
// loads is used for all of them (fp32 online softmax per row, warp-shuffle dot
// products), kSimtTok keys per iteration.
#pragma once

#include "gqa_common.cuh"
#include "gqa_decode_simt.cuh"

namespace gqa_b200 {

constexpr int kPrefillRows = 4;
constexpr int kPrefillWarps = 4;

struct PrefillParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    const int32_t* q_lens;
    const int32_t* kv_lens;
    int batch, tq, tk, q_heads, kv_heads, group, head_dim;
    int causal;
    float scale_log2;
};

// Keys visible to query row `row` of a sequence (attention/reference/gqa.py:57,
// csrc/cuda/common/tile_utils.cuh:6-9).
__device__ __forceinline__ int prefill_row_end(int row, int q_len, int kv_len, int causal) {
    if (!causal) return kv_len;
    const int end = kv_len - q_len + row + 1;
    return end < 0 ? 0 : (end > kv_len ? kv_len : end);
}

__device__ __forceinline__ void prefill_lengths(const PrefillParams& p, int b, int& q_len,
                                                int& kv_len) {
    q_len = __ldg(p.q_lens + b);
    kv_len = __ldg(p.kv_lens + b);
    q_len = q_len < 0 ? 0 : (q_len > p.tq ? p.tq : q_len);
    kv_len = kv_len < 0 ? 0 : (kv_len > p.tk ? p.tk : kv_len);
}

template <typename T, int EPL, bool CONTIG>
__global__ void __launch_bounds__(kPrefillWarps * 32)
gqa_prefill_simt_kernel(const PrefillParams p) {
    constexpr int RB = kPrefillRows;
    constexpr int TOK = kSimtTok;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, b = blockIdx.z;
    const int row0 = (blockIdx.x * kPrefillWarps + warp) * RB;
    if (row0 >= p.tq) return;
    const int D = p.head_dim;
    const int kvh = h / p.group;
    const T* qp = reinterpret_cast<const T*>(p.q);
    const T* kp = reinterpret_cast<const T*>(p.k);
    const T* vp = reinterpret_cast<const T*>(p.v);
    T* op = reinterpret_cast<T*>(p.out);
    int q_len, kv_len;
    prefill_lengths(p, b, q_len, kv_len);

    float qf[RB][EPL], acc[RB][EPL], m[RB], l[RB];
    int end[RB];
    int max_end = 0;
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const int row = row0 + r;
        const bool live = row < q_len;
        end[r] = live ? prefill_row_end(row, q_len, kv_len, p.causal) : 0;
        max_end = max(max_end, end[r]);
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) { acc[r][j] = 0.f; qf[r][j] = 0.f; }
        if (live && row < p.tq)
            load_row<T, EPL, CONTIG>(qp + (((size_t)b * p.tq + row) * p.q_heads + h) * D, lane, D, qf[r]);
    }

    for (int t0 = 0; t0 < max_end; t0 += TOK) {
        float kx[TOK][EPL], vx[TOK][EPL];
#pragma unroll
        for (int tk = 0; tk < TOK; ++tk) {
            const int t = t0 + tk;
            if (t < max_end) {
                const size_t off = (((size_t)b * p.tk + t) * p.kv_heads + kvh) * D;
                load_row<T, EPL, CONTIG>(kp + off, lane, D, kx[tk]);
                load_row<T, EPL, CONTIG>(vp + off, lane, D, vx[tk]);
            } else {
#pragma unroll
                for (int j = 0; j < EPL; ++j) { kx[tk][j] = 0.f; vx[tk][j] = 0.f; }
            }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            if (t0 >= end[r]) continue;       // warp-uniform: this row sees none of these keys
            float s[TOK];
#pragma unroll
            for (int tk = 0; tk < TOK; ++tk) {
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < EPL; ++j) d = fmaf(qf[r][j], kx[tk][j], d);
#pragma unroll
                for (int sh = 16; sh >= 1; sh >>= 1) d += __shfl_xor_sync(0xffffffffu, d, sh);
                s[tk] = t0 + tk < end[r] ? d * p.scale_log2 : -INFINITY;
            }
            float mt = s[0];
#pragma unroll
            for (int tk = 1; tk < TOK; ++tk) mt = fmaxf(mt, s[tk]);
            const float m_new = fmaxf(m[r], mt);   // finite: key t0 is visible to this row
            const float alpha = fast_exp2(m[r] - m_new);
            float pw[TOK], psum = 0.f;
#pragma unroll
            for (int tk = 0; tk < TOK; ++tk) {
                pw[tk] = fast_exp2(s[tk] - m_new);
                psum += pw[tk];
            }
            l[r] = l[r] * alpha + psum;
            m[r] = m_new;
#pragma unroll
            for (int j = 0; j < EPL; ++j) {
                float a = acc[r][j] * alpha;
#pragma unroll
                for (int tk = 0; tk < TOK; ++tk) a = fmaf(pw[tk], vx[tk][j], a);
                acc[r][j] = a;
            }
        }
    }
    // rows past q_len (and rows that see no key) are zero (reference/gqa.py:53,58-59)
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const int row = row0 + r;
        if (row >= p.tq) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        T* dst = op + (((size_t)b * p.tq + row) * p.q_heads + h) * D;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = CONTIG ? lane * EPL + j : lane + 32 * j;
            if (e < D) dst[e] = from_f32<T>(acc[r][j] * inv);
        }
    }
}

}  // namespace gqa_b200

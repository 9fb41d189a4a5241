// Dense GQA prefill, tensor-core kernel for fp16 / bf16 and head_dim 64 / 128.
//
// One CTA = one query head x kPfBM query rows of one sequence; its four warps own
// 16 rows each.  K/V tiles of kPfBN keys are double-buffered in shared memory by
// all threads (16-byte cp.async, XOR-swizzled rows, zero-filled past kv_len);
// Q.K^T and P.V are mma.sync.m16n8k16 with ldmatrix operands, the softmax is the
// fp32 online (max, sum) form with lazy rescaling, and the right-aligned causal
// mask is applied only to the tiles that straddle a row's last visible key.
// Query tiles are launched last-rows-first so the longest causal rows start first.
#pragma once

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"
#include "gqa_prefill_simt.cuh"

namespace gqa_b200 {

constexpr int kPfBM = 64;
constexpr int kPfBN = 64;
constexpr int kPfWarps = 4;

template <int D> struct PrefillGeom {
    static constexpr int kRowBytes = D * 2;
    static constexpr int kChunksPerRow = kRowBytes / 16;
    static constexpr int kQBytes = kPfBM * kRowBytes;
    static constexpr int kTileBytes = kPfBN * kRowBytes;
    static constexpr int kSmemBytes = kQBytes + 2 * 2 * kTileBytes;   // Q + 2 stages of (K, V)
};

template <typename T, int D>
__global__ void __launch_bounds__(kPfWarps * 32, 2) gqa_prefill_mma_kernel(const PrefillParams p) {
    using G = PrefillGeom<D>;
    using Ops = MmaOps<T>;
    constexpr int ROWB = G::kRowBytes;
    constexpr int CPR = G::kChunksPerRow;
    constexpr int BM = kPfBM, BN = kPfBN, NT = kPfWarps * 32;
    constexpr int NB = BN / 8, KS = D / 16, ND = D / 8, KK = BN / 16;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* s_q = smem_raw;
    unsigned char* s_kv = smem_raw + G::kQBytes;       // [2 stages][K tile | V tile]
    const uint32_t sq_u32 = (uint32_t)__cvta_generic_to_shared(s_q);
    const uint32_t skv_u32 = (uint32_t)__cvta_generic_to_shared(s_kv);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = lane >> 2, cq = (lane & 3) * 2;
    const int qt = gridDim.x - 1 - blockIdx.x;        // heavy (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / p.group;
    const int m0 = qt * BM;
    int q_len, kv_len;
    prefill_lengths(p, b, q_len, kv_len);
    const T* qp = reinterpret_cast<const T*>(p.q);
    const char* kp = reinterpret_cast<const char*>(p.k);
    const char* vp = reinterpret_cast<const char*>(p.v);
    T* op = reinterpret_cast<T*>(p.out);

    // keys this CTA has to look at: up to the last visible key of its last live row
    int tile_end = 0;
    if (m0 < q_len) tile_end = prefill_row_end(min(m0 + BM, q_len) - 1, q_len, kv_len, p.causal);
    const int n_tiles = (tile_end + BN - 1) / BN;

    // ---- asynchronous copies -------------------------------------------------
    auto load_q_tile = [&]() {
        for (int i = tid; i < BM * CPR; i += NT) {
            const int row = i / CPR, cc = i % CPR;
            const int qrow = m0 + row;
            const bool valid = qrow < q_len;
            const T* src = qp + (((size_t)b * p.tq + (valid ? qrow : 0)) * p.q_heads + h) * D + cc * 8;
            cp_async16<0>(sq_u32 + row * ROWB + ((cc ^ (row & 7)) << 4), src, valid ? 16 : 0, 0);
        }
    };
    auto load_kv_tile = [&](int j) {
        const uint32_t sk = skv_u32 + (j & 1) * 2 * G::kTileBytes;
        const uint32_t sv = sk + G::kTileBytes;
        for (int i = tid; i < BN * CPR; i += NT) {
            const int row = i / CPR, cc = i % CPR;
            const int t = j * BN + row;
            const bool valid = t < kv_len;
            const size_t off = ((((size_t)b * p.tk + (valid ? t : 0)) * p.kv_heads + kvh) * D) * 2 + cc * 16;
            const uint32_t dst = row * ROWB + ((cc ^ (row & 7)) << 4);
            cp_async16<0>(sk + dst, kp + off, valid ? 16 : 0, 0);
            cp_async16<0>(sv + dst, vp + off, valid ? 16 : 0, 0);
        }
    };

    load_q_tile();
    if (n_tiles > 0) load_kv_tile(0);
    cp_async_commit();

    // per-row visibility of this thread's two fragment rows
    const int row_a = m0 + warp * 16 + r0, row_b = row_a + 8;
    const int end_a = row_a < q_len ? prefill_row_end(row_a, q_len, kv_len, p.causal) : 0;
    const int end_b = row_b < q_len ? prefill_row_end(row_b, q_len, kv_len, p.causal) : 0;
    // smallest / largest number of visible keys among the warp's 16 rows
    const int wrow0 = m0 + warp * 16;
    const int warp_min_end = wrow0 < q_len ? prefill_row_end(wrow0, q_len, kv_len, p.causal) : 0;
    const int warp_full_rows = wrow0 + 16 <= q_len;   // no dead rows in this warp's slice
    const int warp_max_end =
        wrow0 < q_len ? prefill_row_end(min(wrow0 + 16, q_len) - 1, q_len, kv_len, p.causal) : 0;

    float o[ND][4];
#pragma unroll
    for (int nd = 0; nd < ND; ++nd) { o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    uint32_t qa[KS][4];

    const uint32_t k_lane_off = (lane & 7) * ROWB;
    const uint32_t k_lane_x = (lane >> 3) ^ (lane & 7);
    const uint32_t v_lane_off = (((lane >> 3) & 1) * 8 + (lane & 7)) * ROWB;
    const uint32_t v_lane_x = (lane >> 4) ^ (lane & 7);

    for (int j = 0; j < n_tiles; ++j) {
        if (j + 1 < n_tiles) load_kv_tile(j + 1);
        cp_async_commit();
        cp_async_wait<1>();      // tile j (and Q) have landed for this thread
        __syncthreads();         // ... and for every thread
        if (j == 0) {
            // query fragments of this warp's 16 rows
            const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int cc = 2 * ks + (lane >> 4);
                ldmatrix_x4(sq_u32 + row * ROWB + ((cc ^ (row & 7)) << 4), qa[ks][0], qa[ks][1],
                            qa[ks][2], qa[ks][3]);
            }
        }
        const int t_base = j * BN;
        if (t_base < warp_max_end) {     // warp-uniform: some row of this warp sees this tile
            const uint32_t sk = skv_u32 + (j & 1) * 2 * G::kTileBytes;
            const uint32_t sv = sk + G::kTileBytes;
            float s[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
            for (int kp2 = 0; kp2 < KS / 2; ++kp2) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(sk + nb * 8 * ROWB + k_lane_off + ((k_lane_x ^ (4 * kp2)) << 4), b0, b1,
                                b2, b3);
                    Ops::mma(s[nb], qa[2 * kp2], b0, b1);
                    Ops::mma(s[nb], qa[2 * kp2 + 1], b2, b3);
                }
            }
            // mask only where a row's last visible key falls inside (or before) this tile
            if (!warp_full_rows || t_base + BN > warp_min_end) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int t = t_base + nb * 8 + cq;
                    if (t >= end_a) s[nb][0] = -INFINITY;
                    if (t + 1 >= end_a) s[nb][1] = -INFINITY;
                    if (t >= end_b) s[nb][2] = -INFINITY;
                    if (t + 1 >= end_b) s[nb][3] = -INFINITY;
                }
            }
            float mx_a = fmaxf(s[0][0], s[0][1]), mx_b = fmaxf(s[0][2], s[0][3]);
#pragma unroll
            for (int nb = 1; nb < NB; ++nb) {
                mx_a = fmaxf(mx_a, fmaxf(s[nb][0], s[nb][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[nb][2], s[nb][3]));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            mx_a *= p.scale_log2;      // -inf stays -inf (scale > 0): a row that sees nothing here
            mx_b *= p.scale_log2;
            if (__any_sync(0xffffffffu, mx_a > m_a + kRescaleSlack || mx_b > m_b + kRescaleSlack)) {
                const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
                // a row with no visible key so far keeps m = -inf and l = 0, o = 0
                const float al_a = mn_a == -INFINITY ? 1.f : fast_exp2(m_a - mn_a);
                const float al_b = mn_b == -INFINITY ? 1.f : fast_exp2(m_b - mn_b);
                m_a = mn_a;
                m_b = mn_b;
                l_a *= al_a;
                l_b *= al_b;
#pragma unroll
                for (int nd = 0; nd < ND; ++nd) {
                    o[nd][0] *= al_a; o[nd][1] *= al_a;
                    o[nd][2] *= al_b; o[nd][3] *= al_b;
                }
            }
            const float ref_a = m_a == -INFINITY ? 0.f : m_a;   // exp2(-inf - 0) = 0, never NaN
            const float ref_b = m_b == -INFINITY ? 0.f : m_b;
            uint32_t pa[KK][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const float p0 = fast_exp2(fmaf(s[nb][0], p.scale_log2, -ref_a));
                const float p1 = fast_exp2(fmaf(s[nb][1], p.scale_log2, -ref_a));
                const float p2 = fast_exp2(fmaf(s[nb][2], p.scale_log2, -ref_b));
                const float p3 = fast_exp2(fmaf(s[nb][3], p.scale_log2, -ref_b));
                l_a += p0 + p1;
                l_b += p2 + p3;
                pa[nb >> 1][(nb & 1) * 2 + 0] = Ops::pack(p0, p1);
                pa[nb >> 1][(nb & 1) * 2 + 1] = Ops::pack(p2, p3);
            }
#pragma unroll
            for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
                for (int np = 0; np < ND / 2; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(sv + kk * 16 * ROWB + v_lane_off + ((v_lane_x ^ (2 * np)) << 4),
                                      b0, b1, b2, b3);
                    Ops::mma(o[2 * np], pa[kk], b0, b1);
                    Ops::mma(o[2 * np + 1], pa[kk], b2, b3);
                }
            }
        }
        __syncthreads();         // stage j&1 may be refilled by the next iteration's copy
    }
    cp_async_wait<0>();
    if (n_tiles == 0) __syncthreads();   // the Q copies of other threads (zero rows) have landed

    // ---- normalise, stage this warp's 16 rows in its own slice of the Q buffer, store ----
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f;
    const float inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
    __syncwarp();
    unsigned char* s_out = s_q + warp * 16 * ROWB;     // only this warp ever read these rows
#pragma unroll
    for (int nd = 0; nd < ND; ++nd) {
        const int cc = nd;                             // 8 columns = one 16-byte chunk
        *reinterpret_cast<uint32_t*>(s_out + r0 * ROWB + ((cc ^ (r0 & 7)) << 4) + cq * 2) =
            Ops::pack(o[nd][0] * inv_a, o[nd][1] * inv_a);
        *reinterpret_cast<uint32_t*>(s_out + (r0 + 8) * ROWB + ((cc ^ ((r0 + 8) & 7)) << 4) + cq * 2) =
            Ops::pack(o[nd][2] * inv_b, o[nd][3] * inv_b);
    }
    __syncwarp();
    for (int i = lane; i < 16 * CPR; i += 32) {
        const int row = i / CPR, cc = i % CPR;
        const int qrow = m0 + warp * 16 + row;
        if (qrow < p.tq) {
            const uint4 val = *reinterpret_cast<const uint4*>(s_out + row * ROWB + ((cc ^ (row & 7)) << 4));
            *reinterpret_cast<uint4*>(op + (((size_t)b * p.tq + qrow) * p.q_heads + h) * D + cc * 8) = val;
        }
    }
}

}  // namespace gqa_b200

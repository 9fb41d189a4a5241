// Dense GQA prefill on the 5th-generation tensor cores (tcgen05 + TMEM), fp16 / bf16,
// head_dim 64 / 128.
//
// One CTA = one query head x 128 query rows.  Both contractions are single-thread-issued
// tcgen05.mma (cta_group::1, kind::f16) with operands in shared memory as K-major
// 128-byte-swizzled tiles and fp32 accumulators in TMEM:
//   S[128 x 64]  = Q[128 x D] . K_tile[64 x D]^T          (TMEM columns 0..63)
//   O[128 x D]  += P[128 x 64] . Vt_tile[D x 64]^T        (TMEM columns 64..64+D)
// K/V tiles arrive with 16-byte cp.async; V ([key][d] in memory) is transposed into the
// K-major tile Vt with ldmatrix.trans + stmatrix.  The softmax is thread-per-row: thread r
// reads row r of S from TMEM (no shuffles), keeps the fp32 running (max, sum), writes its
// row of P as a swizzled 128-byte row, and rescales its row of O in TMEM only when the
// row maximum moved by more than 2^8 (lazy rescaling).  Two CTAs fit per SM (112 KB of
// shared memory, 256 TMEM columns each), so one CTA's softmax overlaps the other's MMAs.
//
// Every mbarrier wait is bounded; a wait that runs out marks the CTA dead (later waits
// give up at once), raises the status word and the kernel still frees its TMEM.
#pragma once

#include <type_traits>

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"
#include "gqa_prefill_simt.cuh"
#include "tcgen05_util.cuh"

namespace gqa_b200 {

constexpr int kTcBM = 128;
constexpr int kTcBN = 64;
constexpr int kTcThreads = 128;
constexpr int kTcTmemCols = 256;

template <int D> struct PrefillTcGeom {
    static constexpr int kKB = D / 64;                        // 128-byte K blocks of Q / K rows
    static constexpr int kQBytes = kKB * kTcBM * 128;
    static constexpr int kKTileBytes = kKB * kTcBN * 128;
    static constexpr int kVRawBytes = kTcBN * D * 2;
    static constexpr int kVtBytes = D * 128;                  // [D rows][64 keys x 2 B]
    static constexpr int kPBytes = kTcBM * 128;
    static constexpr int kOffK = kQBytes;
    static constexpr int kOffVRaw = kOffK + 2 * kKTileBytes;
    static constexpr int kOffVt = kOffVRaw + kVRawBytes;
    static constexpr int kOffP = kOffVt + kVtBytes;
    static constexpr int kSmemBytes = kOffP + kPBytes;
};

template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 2)
gqa_prefill_tc_kernel(const PrefillParams p, int* status) {
    using G = PrefillTcGeom<D>;
    using Ops = MmaOps<T>;
    constexpr int BM = kTcBM, BN = kTcBN, NT = kTcThreads;
    constexpr int KB = G::kKB;
    constexpr int AB_TYPE = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr int VROWB = D * 2, VCPR = VROWB / 16;

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t s_bar[2];     // [0] S ready, [1] P.V done
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int qt = gridDim.x - 1 - blockIdx.x;     // heavy (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / p.group;
    const int m0 = qt * BM;
    int q_len, kv_len;
    prefill_lengths(p, b, q_len, kv_len);
    const T* qp = reinterpret_cast<const T*>(p.q);
    const char* kp = reinterpret_cast<const char*>(p.k);
    const char* vp = reinterpret_cast<const char*>(p.v);
    T* op = reinterpret_cast<T*>(p.out);
    const int my_row = m0 + tid;                   // thread-per-row

    int tile_end = 0;
    if (m0 < q_len) tile_end = prefill_row_end(min(m0 + BM, q_len) - 1, q_len, kv_len, p.causal);
    const int n_tiles = (tile_end + BN - 1) / BN;
    if (n_tiles == 0) {                            // nothing visible: zero rows, no TMEM needed
        if (my_row < p.tq) {
            uint4* dst = reinterpret_cast<uint4*>(op + (((size_t)b * p.tq + my_row) * p.q_heads + h) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        return;
    }

    const uint32_t s_base = tc::smem_u32(smem);
    if (s_base & 1023u) {                          // the swizzled tiles need a 1024-byte aligned base
        if (tid == 0 && status) atomicExch(status, 3);
        return;
    }
    const uint32_t sq = s_base, sk = s_base + G::kOffK, svraw = s_base + G::kOffVRaw;
    const uint32_t svt = s_base + G::kOffVt, sp = s_base + G::kOffP;
    const uint32_t bar_s = tc::smem_u32(&s_bar[0]), bar_pv = tc::smem_u32(&s_bar[1]);

    if (warp == 0) { tc::tmem_alloc(tc::smem_u32(&s_tmem), kTcTmemCols); tc::tmem_relinquish(); }
    if (tid == 0) {
        tc::mbar_init(bar_s, 1);
        tc::mbar_init(bar_pv, 1);
        tc::fence_mbar_init();
        s_dead = 0;
    }

    // ---- asynchronous copies into swizzled tiles ----
    auto load_q = [&]() {
        for (int i = tid; i < BM * D / 8; i += NT) {
            const int row = i / (D / 8), c = i % (D / 8);
            const int kb = c >> 3, cc = c & 7;
            const int qrow = m0 + row;
            const bool valid = qrow < q_len;
            const T* src = qp + (((size_t)b * p.tq + (valid ? qrow : 0)) * p.q_heads + h) * D + c * 8;
            cp_async16<0>(sq + kb * (BM * 128) + row * 128 + ((cc ^ (row & 7)) << 4), src, valid ? 16 : 0, 0);
        }
    };
    auto load_k = [&](int j) {
        const uint32_t dst0 = sk + (j & 1) * G::kKTileBytes;
        for (int i = tid; i < BN * D / 8; i += NT) {
            const int row = i / (D / 8), c = i % (D / 8);
            const int kb = c >> 3, cc = c & 7;
            const int t = j * BN + row;
            const bool valid = t < kv_len;
            const size_t off = ((((size_t)b * p.tk + (valid ? t : 0)) * p.kv_heads + kvh) * D) * 2 + c * 16;
            cp_async16<0>(dst0 + kb * (BN * 128) + row * 128 + ((cc ^ (row & 7)) << 4), kp + off,
                          valid ? 16 : 0, 0);
        }
    };
    auto load_v = [&](int j) {
        for (int i = tid; i < BN * VCPR; i += NT) {
            const int row = i / VCPR, cc = i % VCPR;
            const int t = j * BN + row;
            const bool valid = t < kv_len;
            const size_t off = ((((size_t)b * p.tk + (valid ? t : 0)) * p.kv_heads + kvh) * D) * 2 + cc * 16;
            cp_async16<0>(svraw + row * VROWB + ((cc ^ (row & 7)) << 4), vp + off, valid ? 16 : 0, 0);
        }
    };

    load_q();
    load_k(0);
    load_v(0);
    cp_async_commit();

    const int my_end = my_row < q_len ? prefill_row_end(my_row, q_len, kv_len, p.causal) : 0;
    float m_run = -INFINITY, l_run = 0.f;
    const uint32_t idesc_s = tc::idesc_f16(BM, BN, AB_TYPE);
    const uint32_t idesc_o = tc::idesc_f16(BM, D, AB_TYPE);
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;      // this warp's TMEM lanes
    bool alive = true;

    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        const bool ok = tc::mbar_wait(bar, parity, s_dead ? 16u : (1u << 22));
        if (!ok) {
            s_dead = 1;
            alive = false;
            if (status) atomicExch(status, 2);
        }
    };

    __syncthreads();                               // s_tmem, barriers, s_dead visible
    tc::tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_s = tmem, tmem_o = tmem + BN;

    for (int j = 0; j < n_tiles; ++j) {
        // ---- tile j has landed; the P.V of tile j-1 no longer reads Vt / P ----
        cp_async_wait<0>();
        tc::fence_async_smem();
        if (j > 0) wait_bar(bar_pv, (j - 1) & 1);
        __syncthreads();

        // ---- V [key][d]  ->  Vt [d][key], K-major swizzled (8 x4 ops per warp for D = 128) ----
        for (int x = warp; x < (D / 8) * (BN / 8) / 4; x += NT / 32) {
            // four 8x8 blocks: key blocks kb0..kb0+3 of one d block
            const int db = x / (BN / 32), kb0 = (x % (BN / 32)) * 4;
            const int blk = lane >> 3, i = lane & 7;
            const int key_row = (kb0 + blk) * 8 + i;
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4_trans(svraw + key_row * VROWB + ((db ^ (key_row & 7)) << 4), r0, r1, r2, r3);
            const int d_row = db * 8 + i;
            tc::stmatrix_x4(svt + d_row * 128 + (((kb0 + blk) ^ (d_row & 7)) << 4), r0, r1, r2, r3);
        }
        tc::fence_async_smem();
        tc::tc_fence_before();
        __syncthreads();                           // Vt complete; raw V stage free again

        if (j + 1 < n_tiles) { load_k(j + 1); load_v(j + 1); }
        cp_async_commit();

        // ---- S = Q K^T ----
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t kt = sk + (j & 1) * G::kKTileBytes;
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t da = tc::smem_desc_sw128_kmajor(sq + kb * (BM * 128) + k * 32);
                    const uint64_t db = tc::smem_desc_sw128_kmajor(kt + kb * (BN * 128) + k * 32);
                    tc::mma_f16_ss(tmem_s, da, db, idesc_s, (kb | k) ? 1u : 0u);
                }
            }
            tc::mma_commit(bar_s);
        }
        wait_bar(bar_s, j & 1);
        tc::tc_fence_after();

        // ---- softmax of this thread's row ----
        float s[BN];
        {
            uint32_t r[32];
            tc::tmem_ld32(tmem_s + lane_sel, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) s[c] = __uint_as_float(r[c]);
            tc::tmem_ld32(tmem_s + lane_sel + 32, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) s[32 + c] = __uint_as_float(r[c]);
        }
        const int t_base = j * BN;
        if (t_base + BN > my_end) {
#pragma unroll
            for (int c = 0; c < BN; ++c)
                if (t_base + c >= my_end) s[c] = -INFINITY;
        }
        float mx = s[0];
#pragma unroll
        for (int c = 1; c < BN; ++c) mx = fmaxf(mx, s[c]);
        mx *= p.scale_log2;
        const bool need = mx > m_run + kRescaleSlack;
        if (__any_sync(0xffffffffu, need)) {        // warp-uniform: TMEM ld/st are warp-collective
            float alpha = 1.f;
            if (need) {
                const float mn = fmaxf(m_run, mx);
                alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - mn);
                m_run = mn;
                l_run *= alpha;
            }
            if (j > 0) {                           // O holds nothing before the first P.V
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t r[32];
                    tc::tmem_ld32(tmem_o + lane_sel + c0, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                    tc::tmem_st32(tmem_o + lane_sel + c0, r);
                }
                tc::tmem_st_wait();
            }
        }
        const float ref = m_run == -INFINITY ? 0.f : m_run;
        {
            float psum = 0.f;
#pragma unroll
            for (int c8 = 0; c8 < BN / 8; ++c8) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p0 = fast_exp2(fmaf(s[c8 * 8 + 2 * e], p.scale_log2, -ref));
                    const float p1 = fast_exp2(fmaf(s[c8 * 8 + 2 * e + 1], p.scale_log2, -ref));
                    psum += p0 + p1;
                    w[e] = Ops::pack(p0, p1);
                }
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(sp + tid * 128 + ((c8 ^ (tid & 7)) << 4)),
                             "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
            l_run += psum;
        }
        tc::fence_async_smem();
        tc::tc_fence_before();
        __syncthreads();                           // P complete; all reads of S and O rescales done

        // ---- O += P V ----
        if (tid == 0) {
            tc::tc_fence_after();
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
                const uint64_t da = tc::smem_desc_sw128_kmajor(sp + k * 32);
                const uint64_t db = tc::smem_desc_sw128_kmajor(svt + k * 32);
                tc::mma_f16_ss(tmem_o, da, db, idesc_o, (j | k) ? 1u : 0u);
            }
            tc::mma_commit(bar_pv);
        }
    }
    wait_bar(bar_pv, (n_tiles - 1) & 1);
    tc::tc_fence_after();

    // ---- normalise and store this thread's row ----
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tc::tmem_ld32(tmem_o + lane_sel + c0, r);
        tc::tmem_ld_wait();
        if (my_row < p.tq && alive) {
            uint4* dst = reinterpret_cast<uint4*>(op + (((size_t)b * p.tq + my_row) * p.q_heads + h) * D + c0);
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
                uint4 v;
                v.x = Ops::pack(__uint_as_float(r[c8 * 8 + 0]) * inv, __uint_as_float(r[c8 * 8 + 1]) * inv);
                v.y = Ops::pack(__uint_as_float(r[c8 * 8 + 2]) * inv, __uint_as_float(r[c8 * 8 + 3]) * inv);
                v.z = Ops::pack(__uint_as_float(r[c8 * 8 + 4]) * inv, __uint_as_float(r[c8 * 8 + 5]) * inv);
                v.w = Ops::pack(__uint_as_float(r[c8 * 8 + 6]) * inv, __uint_as_float(r[c8 * 8 + 7]) * inv);
                dst[c8] = v;
            }
        }
    }
    cp_async_wait<0>();
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, kTcTmemCols);
}

}  // namespace gqa_b200

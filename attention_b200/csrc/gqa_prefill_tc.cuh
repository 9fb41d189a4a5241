// Dense GQA prefill on the 5th-generation tensor cores (tcgen05 + TMEM), fp16 / bf16,
// head_dim 64 / 128.
//
// One CTA = one query head x 128 query rows.  Both contractions are single-thread-issued
// tcgen05.mma (cta_group::1, kind::f16) with operands in shared memory as 128-byte-swizzled
// tiles and fp32 accumulators in TMEM:
//   S[128 x 64]  = Q[128 x D] . K_tile[64 x D]^T     Q, K: K-major tiles    (TMEM: two S buffers)
//   O[128 x D]  += P[128 x 64] . V_tile[64 x D]      V: used as it lies in memory ([key][d]),
//                                                    as an MN-major B operand    (TMEM: D columns)
// K and V tiles arrive with 16-byte cp.async into two-stage rings.  The softmax uses two
// threads per row (warps w and w + 4 own the same 32 TMEM lanes): both read row r of S from
// TMEM and take its maximum (so they agree on the running max without talking to each
// other), each exponentiates and sums its own half, writes its half of P as part of a
// swizzled 128-byte row, and rescales its half of row r of O in TMEM only when the row
// maximum moved by more than 2^8 (lazy rescaling).  The two half sums meet once, at the end.
//
// Software pipeline (iteration j = softmax of tile j): S(j+1) = Q.K(j+1)^T is issued before
// the softmax of tile j starts, so the tensor cores work on the next scores (and on the
// previous P.V) while the threads exponentiate; P.V(j) is issued as soon as P(j) is in
// shared memory.  Two CTAs fit per SM (112 KB of shared memory, 256 TMEM columns each).
//
// Every mbarrier wait is bounded (one second); a wait that runs out marks the CTA dead (later
// waits give up at once), raises the status word and the kernel still frees its TMEM.
#pragma once

#include <type_traits>

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"
#include "gqa_prefill_simt.cuh"
#include "tcgen05_util.cuh"

namespace gqa_b200 {

constexpr int kTcBM = 128;
constexpr int kTcBN = 64;
constexpr int kTcThreads = 256;
constexpr int kTcTmemCols = 256;

template <int D> struct PrefillTcGeom {
    static constexpr int kKB = D / 64;                        // 128-byte blocks of a Q/K/V row
    static constexpr int kQBytes = kKB * kTcBM * 128;
    static constexpr int kTileBytes = kKB * kTcBN * 128;      // one K or V tile
    static constexpr int kPBytes = kTcBM * 128;
    static constexpr int kOffK = kQBytes;
    static constexpr int kOffV = kOffK + 2 * kTileBytes;
    static constexpr int kOffP = kOffV + 2 * kTileBytes;
    static constexpr int kSmemBytes = kOffP + kPBytes;
};

template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 2)
gqa_prefill_tc_kernel(const PrefillParams p, int* status) {
    using G = PrefillTcGeom<D>;
    using Ops = MmaOps<T>;
    constexpr int BM = kTcBM, BN = kTcBN, NT = kTcThreads;
    constexpr int KB = G::kKB;
    constexpr int AB_TYPE = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t s_bar[3];     // [0], [1]: S buffer ready; [2]: P.V done
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hf = warp >> 2;     // TMEM lane quadrant, column half
    const int row_l = quad * 32 + lane;            // this thread's row of the 128-row tile
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
    const int my_row = m0 + row_l;

    int tile_end = 0;
    if (m0 < q_len) tile_end = prefill_row_end(min(m0 + BM, q_len) - 1, q_len, kv_len, p.causal);
    const int n_tiles = (tile_end + BN - 1) / BN;
    if (n_tiles == 0) {                            // nothing visible: zero rows, no TMEM needed
        if (my_row < p.tq) {
            uint4* dst = reinterpret_cast<uint4*>(op + (((size_t)b * p.tq + my_row) * p.q_heads + h) * D) +
                         hf * (D / 16);
#pragma unroll
            for (int c = 0; c < D / 16; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        return;
    }

    const uint32_t s_base = tc::smem_u32(smem);
    if (s_base & 1023u) {                          // the swizzled tiles need a 1024-byte aligned base
        if (tid == 0 && status) atomicExch(status, 3);
        return;
    }
    const uint32_t sq = s_base, sk = s_base + G::kOffK, sv = s_base + G::kOffV, sp = s_base + G::kOffP;
    const uint32_t bar_s0 = tc::smem_u32(&s_bar[0]), bar_pv = tc::smem_u32(&s_bar[2]);

    if (warp == 0) { tc::tmem_alloc(tc::smem_u32(&s_tmem), kTcTmemCols); tc::tmem_relinquish(); }
    if (tid == 0) {
        tc::mbar_init(bar_s0, 1);
        tc::mbar_init(bar_s0 + 8, 1);
        tc::mbar_init(bar_pv, 1);
        tc::fence_mbar_init();
        s_dead = 0;
    }

    // ---- asynchronous copies into swizzled tiles: [64-element block][row][128 B] ----
    auto load_q = [&]() {
        for (int i = tid; i < BM * D / 8; i += NT) {
            const int row = i / (D / 8), c = i % (D / 8);
            const int qrow = m0 + row;
            const bool valid = qrow < q_len;
            const T* src = qp + (((size_t)b * p.tq + (valid ? qrow : 0)) * p.q_heads + h) * D + c * 8;
            cp_async16<0>(sq + (c >> 3) * (BM * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4), src,
                          valid ? 16 : 0, 0);
        }
    };
    // K or V tile j (keys are rows).  Each thread always copies the same 16-byte chunk of
    // rows row0, row0 + RPI, ...: since RPI is a multiple of 8 the swizzle term is constant,
    // so source and destination advance by fixed steps (no per-copy address arithmetic).
    constexpr int CPRW = D / 8;                    // 16-byte chunks per row
    constexpr int RPI = NT / CPRW;                 // rows covered by one pass of the CTA
    static_assert(RPI % 8 == 0 && BN % RPI == 0, "copy pattern");
    const int ld_c = tid % CPRW, ld_row0 = tid / CPRW;
    const size_t row_stride = (size_t)p.kv_heads * D * 2;
    const size_t thr_src = (size_t)ld_row0 * row_stride + (size_t)kvh * D * 2 + ld_c * 16;
    const uint32_t thr_dst = (ld_c >> 3) * (BN * 128) + ld_row0 * 128 + (((ld_c & 7) ^ (ld_row0 & 7)) << 4);
    auto load_tile = [&](const char* base, uint32_t dst0, int j) {
        const char* src = base + ((size_t)b * p.tk + (size_t)j * BN) * row_stride + thr_src;
        uint32_t dst = dst0 + thr_dst;
        const int t0 = j * BN + ld_row0;
#pragma unroll
        for (int it = 0; it < BN / RPI; ++it) {
            const bool valid = t0 + it * RPI < kv_len;
            cp_async16<0>(dst, valid ? src : base, valid ? 16 : 0, 0);
            src += (size_t)RPI * row_stride;
            dst += RPI * 128;
        }
    };

    load_q();
    load_tile(kp, sk, 0);
    load_tile(vp, sv, 0);
    if (n_tiles > 1) load_tile(kp, sk + G::kTileBytes, 1);
    cp_async_commit();

    const int my_end = my_row < q_len ? prefill_row_end(my_row, q_len, kv_len, p.causal) : 0;
    float m_run = -INFINITY, l_run = 0.f;
    const uint32_t idesc_s = tc::idesc_f16(BM, BN, AB_TYPE);
    const uint32_t idesc_o = tc::idesc_f16(BM, D, AB_TYPE) | tc::kIdescBMnMajor;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;      // this warp's TMEM lanes
    bool alive = true;

    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        const bool ok = tc::mbar_wait(bar, parity, s_dead ? 1000ull : 1000000000ull);
        if (!ok) {
            s_dead = 1;
            alive = false;
            if (status) atomicExch(status, 2);
        }
    };
    // S(j) = Q K(j)^T into S buffer j & 1 (one thread)
    auto issue_qk = [&](int j, uint32_t tmem) {
        const uint32_t kt = sk + (j & 1) * G::kTileBytes;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t da = tc::smem_desc_sw128_kmajor(sq + kb * (BM * 128) + k * 32);
                const uint64_t db = tc::smem_desc_sw128_kmajor(kt + kb * (BN * 128) + k * 32);
                tc::mma_f16_ss(tmem + (j & 1) * BN, da, db, idesc_s, (kb | k) ? 1u : 0u);
            }
        }
        tc::mma_commit(bar_s0 + (j & 1) * 8);
    };

    cp_async_wait<0>();
    tc::fence_async_smem();
    tc::tc_fence_before();
    __syncthreads();                               // Q, K(0..1), V(0) in place; s_tmem, barriers visible
    tc::tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_o = tmem + 2 * BN;
    if (tid == 0) issue_qk(0, tmem);

    for (int j = 0; j < n_tiles; ++j) {
        // ---- S(j) is ready, so K stage j&1 is free: fetch K(j+2) into it ----
        wait_bar(bar_s0 + (j & 1) * 8, (j >> 1) & 1);
        tc::tc_fence_after();
        if (j + 2 < n_tiles) load_tile(kp, sk + (j & 1) * G::kTileBytes, j + 2);
        cp_async_commit();

        // ---- start S(j+1) on the tensor cores before exponentiating tile j ----
        if (j + 1 < n_tiles && tid == 0) issue_qk(j + 1, tmem);

        // ---- scores of this thread's row: own half kept, the other half only for the maximum ----
        constexpr int HC = BN / 2;                 // columns per thread
        float s[HC];
        float mx;
        {
            uint32_t r[32], ro[32];
            tc::tmem_ld32(tmem + (j & 1) * BN + lane_sel + hf * HC, r);          // this thread's half
            tc::tmem_ld32(tmem + (j & 1) * BN + lane_sel + (hf ^ 1) * HC, ro);   // the other half
            tc::tmem_ld_wait();                                                   // both in flight together
            const int t_other = j * BN + (hf ^ 1) * HC;
            float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
            if (t_other + HC > my_end) {
#pragma unroll
                for (int c = 0; c < HC; ++c)
                    if (t_other + c >= my_end) ro[c] = 0xff800000u;   // -inf
            }
#pragma unroll
            for (int c = 0; c < HC; c += 4) {
                a0 = fmaxf(a0, __uint_as_float(ro[c])); a1 = fmaxf(a1, __uint_as_float(ro[c + 1]));
                a2 = fmaxf(a2, __uint_as_float(ro[c + 2])); a3 = fmaxf(a3, __uint_as_float(ro[c + 3]));
            }
#pragma unroll
            for (int c = 0; c < HC; ++c) s[c] = __uint_as_float(r[c]);
            const int t_base = j * BN + hf * HC;
            if (t_base + HC > my_end) {
#pragma unroll
                for (int c = 0; c < HC; ++c)
                    if (t_base + c >= my_end) s[c] = -INFINITY;
            }
#pragma unroll
            for (int c = 0; c < HC; c += 4) {
                a0 = fmaxf(a0, s[c]); a1 = fmaxf(a1, s[c + 1]);
                a2 = fmaxf(a2, s[c + 2]); a3 = fmaxf(a3, s[c + 3]);
            }
            mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) * p.scale_log2;
        }
        const bool need = mx > m_run + kRescaleSlack;
        float alpha = 1.f;
        if (need) {
            const float mn = fmaxf(m_run, mx);
            alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - mn);
            m_run = mn;
            l_run *= alpha;
        }
        const float ref = m_run == -INFINITY ? 0.f : m_run;
        uint32_t pw[HC / 2];
        {
            float ps0 = 0.f, ps1 = 0.f, ps2 = 0.f, ps3 = 0.f;   // independent partial sums
#pragma unroll
            for (int c2 = 0; c2 < HC / 2; c2 += 2) {
                const float p0 = fast_exp2(fmaf(s[2 * c2], p.scale_log2, -ref));
                const float p1 = fast_exp2(fmaf(s[2 * c2 + 1], p.scale_log2, -ref));
                const float p2 = fast_exp2(fmaf(s[2 * c2 + 2], p.scale_log2, -ref));
                const float p3 = fast_exp2(fmaf(s[2 * c2 + 3], p.scale_log2, -ref));
                ps0 += p0; ps1 += p1; ps2 += p2; ps3 += p3;
                pw[c2] = Ops::pack(p0, p1);
                pw[c2 + 1] = Ops::pack(p2, p3);
            }
            l_run += (ps0 + ps1) + (ps2 + ps3);     // this thread's half of the row sum
        }

        // ---- P.V(j-1) is done: V stage (j+1)&1, the P tile and O may be touched ----
        if (j > 0) wait_bar(bar_pv, (j - 1) & 1);
        tc::tc_fence_after();
        if (j + 1 < n_tiles) load_tile(vp, sv + ((j + 1) & 1) * G::kTileBytes, j + 1);
        cp_async_commit();
        if (j > 0 && __any_sync(0xffffffffu, need)) {   // warp-uniform: TMEM ld/st are collective
#pragma unroll
            for (int c0 = hf * (D / 2); c0 < (hf + 1) * (D / 2); c0 += 32) {
                uint32_t r[32];
                tc::tmem_ld32(tmem_o + lane_sel + c0, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                tc::tmem_st32(tmem_o + lane_sel + c0, r);
            }
            tc::tmem_st_wait();
        }
#pragma unroll
        for (int c8 = 0; c8 < HC / 8; ++c8) {
            const int chunk = hf * (HC / 8) + c8;
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(sp + row_l * 128 + ((chunk ^ (row_l & 7)) << 4)),
                         "r"(pw[c8 * 4 + 0]), "r"(pw[c8 * 4 + 1]), "r"(pw[c8 * 4 + 2]), "r"(pw[c8 * 4 + 3])
                         : "memory");
        }
        // V(j) (issued one iteration ago) and K(j+1) must have landed for everyone
        cp_async_wait<1>();
        tc::fence_async_smem();
        tc::tc_fence_before();
        __syncthreads();                           // P complete, S(j) consumed, O rescaled, V(j) in place

        // ---- O += P V(j)  (issued by another warp than Q.K^T, to share the issue work) ----
        if (tid == NT / 2) {
            tc::tc_fence_after();
            const uint32_t vt = sv + (j & 1) * G::kTileBytes;
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
                const uint64_t da = tc::smem_desc_sw128_kmajor(sp + k * 32);
                const uint64_t db = tc::smem_desc_sw128_mnmajor(vt + k * 2048, BN * 128);
                tc::mma_f16_ss(tmem_o, da, db, idesc_o, (j | k) ? 1u : 0u);
            }
            tc::mma_commit(bar_pv);
        }
    }
    wait_bar(bar_pv, (n_tiles - 1) & 1);
    tc::tc_fence_after();

    // ---- row sum = sum of the two halves (exchanged through the idle P tile); normalise and
    //      store this thread's half row ----
    float* s_half = reinterpret_cast<float*>(smem + G::kOffP);          // [2][128]
    s_half[hf * BM + row_l] = l_run;
    __syncthreads();
    const float l_tot = l_run + s_half[(hf ^ 1) * BM + row_l];
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
#pragma unroll
    for (int c0 = hf * (D / 2); c0 < (hf + 1) * (D / 2); c0 += 32) {
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

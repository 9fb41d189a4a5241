// Dense GQA prefill on the 5th-generation tensor cores: fp16 / bf16, head_dim 64 / 128.
// Persistent CTAs (one per SM) walk the work items (batch, query head, 256 query rows),
// heaviest first, in alternating CTA order from round to round.  An item is two tiles of 128 query rows, A and B, that share every K and V
// tile; a K/V tile of 128 keys is worked on in two halves of 64 keys (h = 0, 1):
//
//   S_X(j,h)[128 x 64] = Q_X[128 x D] . K(j)[64 h .. 64 h + 63][D]^T   A = Q_X from shared memory, B = K rows (K-major)
//   O_X[128 x D]      += P_X(j,h)[128 x 64] . V(j)[64 h ..][D]         A = P_X from TENSOR MEMORY, B = V rows as they
//                                                                      lie in memory ([key][d], an MN-major operand)
//
// Why this shape.  Per 128 x 128 scores the tensor pipe needs 1024 clocks and the special-
// function unit (16 exponentials per clock and SM) needs 1024 clocks as well, so neither may
// wait for the other:
//   * two query tiles give two independent chains  scores -> softmax -> P.V : the softmax
//     warps of A work while the tensor pipe computes for B and the other way round, and a K or
//     V tile fetched once serves 256 query rows;
//   * within a chain the two key halves have their own score columns and hand-offs, so the
//     scores of half h of the NEXT tile are issued right after P.V of half h of this one and
//     are ready while the softmax warps are still busy with the other half: a softmax thread
//     goes from half to half without waiting for the tensor pipe, and holds only 64 scores in
//     registers (one pass, no exchange: a thread owns a whole query row);
//   * each query tile has its own MMA-issuing warp (a warp issues about one tcgen05.mma per 60
//     clocks, and every hand-off wait costs it ~150 clocks; one warp for both chains was the
//     bottleneck), and every lane of such a warp runs the issue loop, with one elected lane
//     executing the instruction, so that descriptors stay in uniform registers;
//   * the exponentials of the two softmax groups take turns (a token passed through two named
//     barriers): a group that has the special-function unit to itself is done in half the
//     time, and the other group loads, reduces, converts and stores meanwhile.
//
// TMEM (512 columns): S_A, S_B (2 x 64 columns each; P_X(j,h), 32 columns of packed 16-bit
// pairs, overwrites the first half of S_X(j,h)), O_A, O_B (D columns each).
// Shared memory: both Q tiles, a ring of K tiles and a ring of V tiles (32 KB per tile at D 128).
//
// Warp roles (384 threads):
//   warps 0-3   softmax of tile A: one thread per query row (TMEM lane = row)
//   warps 4-7   the same for tile B
//   warp 8      loader of Q and K (16-byte cp.async, completion by cp.async.mbarrier.arrive)
//   warp 9      loader of V
//   warp 10/11  issue every tcgen05.mma of tile A / tile B
// No CTA-wide barrier in the loop and none between items: the mbarriers are initialised once
// and their phases run on across the items of a CTA (running tile numbers give every hand-off
// its stage and parity).  The MMA warps need nothing from the softmax warps to start the next
// item (Q comes from the loader), so they issue the next item's first scores while the
// softmax warps still store the rows of the current one.
//   q_full  / k_full[] / v_full[]   32 loader arrivals (when their copies land)            -> MMA warps
//   q_empty / k_empty[] / v_empty[] one arrival per MMA warp (tcgen05.commit after its last
//                                   product on the tile, or a plain arrival if it has none) -> loaders
//   bar_s[X][h]                     tcgen05.commit: S_X(j,h) is in TMEM                     -> softmax X
//   bar_p[X][h]                     4 warp arrivals: P_X(j,h) is in TMEM, O_X rescaled      -> MMA warp X
//   bar_o[X][h]                     tcgen05.commit: P.V of (j,h) is done                    -> softmax X
// Every wait is bounded (one second); a wait that runs out marks the CTA dead (later waits
// give up at once), raises the status word, and the CTA still walks its protocol and frees
// its tensor memory.
#pragma once

#include <type_traits>

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"
#include "gqa_prefill_simt.cuh"
#include "tcgen05_util.cuh"

namespace gqa_b200 {

constexpr int kPpBM = 128;                           // rows of one query tile; an item has two
constexpr int kPpBN = 128;
constexpr int kPpThreads = 384;
constexpr int kPpTmemCols = 512;

template <int D> struct PrefillPpGeom {
    static constexpr int kKB = D / 64;                           // 128-byte blocks of a row
    static constexpr int kTileBytes = kKB * 128 * 128;           // a Q, K or V tile: [block][row][128 B]
    static constexpr int kStagesK = 3;
    static constexpr int kStagesV = D == 128 ? 2 : 3;
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = 2 * kTileBytes;
    static constexpr int kOffV = kOffK + kStagesK * kTileBytes;
    static constexpr int kTileSmem = (2 + kStagesK + kStagesV) * kTileBytes;   // 224 KB at D 128, 128 KB at D 64
    // a floor above half an SM's shared memory: a second resident CTA could never get tensor memory
    static constexpr int kSmemBytes = kTileSmem < 120 * 1024 ? 120 * 1024 : kTileSmem;
    static constexpr int kColS = 0;                              // 2 x 128
    static constexpr int kColO = 2 * kPpBN;                      // 2 x D
    static_assert(kColO + 2 * D <= kPpTmemCols, "TMEM budget");
};

template <typename T, int D>
__global__ void __launch_bounds__(kPpThreads, 1)
gqa_prefill_pp_kernel(const PrefillParams p, int* status) {
    using G = PrefillPpGeom<D>;
    using Ops = MmaOps<T>;
    constexpr int BM = kPpBM, BN = kPpBN, NSK = G::kStagesK, NSV = G::kStagesV;
    constexpr int KB = G::kKB;
    constexpr int HN = BN / 2;                       // keys of a half tile
    constexpr int AB_TYPE = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    static_assert(D % 32 == 0, "output rows are moved 32 columns at a time");

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t s_bar[2 + 2 * NSK + 2 * NSV + 12];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_softmax = warp < 8, is_kload = warp == 8, is_vload = warp == 9, is_mma = warp >= 10;
    const int X = (warp >> 2) & 1;                   // softmax warps: query tile A (0) or B (1)
    const int quad = warp & 3;                       // softmax warps: TMEM lane quadrant
    const int row_l = quad * 32 + lane;              // softmax thread's row of its tile
    const T* qp = reinterpret_cast<const T*>(p.q);
    const char* kp = reinterpret_cast<const char*>(p.k);
    const char* vp = reinterpret_cast<const char*>(p.v);
    T* op = reinterpret_cast<T*>(p.out);

    const uint32_t s_base = tc::smem_u32(smem);
    if (s_base & 1023u) {                            // the swizzled tiles need a 1024-byte aligned base
        if (tid == 0 && status) atomicExch(status, 3);
        return;
    }
    const uint32_t sq = s_base + G::kOffQ, sk = s_base + G::kOffK, sv = s_base + G::kOffV;
    const uint32_t q_full = tc::smem_u32(&s_bar[0]);
    const uint32_t q_empty = tc::smem_u32(&s_bar[1]);
    const uint32_t k_full = tc::smem_u32(&s_bar[2]);
    const uint32_t k_empty = tc::smem_u32(&s_bar[2 + NSK]);
    const uint32_t v_full = tc::smem_u32(&s_bar[2 + 2 * NSK]);
    const uint32_t v_empty = tc::smem_u32(&s_bar[2 + 2 * NSK + NSV]);
    const uint32_t bar_s = tc::smem_u32(&s_bar[2 + 2 * NSK + 2 * NSV]);       // [4]: query tile x 2 + key half
    const uint32_t bar_p = bar_s + 32;                                         // [4]
    const uint32_t bar_o = bar_s + 64;                                         // [4]

    if (warp == 0) { tc::tmem_alloc(tc::smem_u32(&s_tmem), kPpTmemCols); tc::tmem_relinquish(); }
    if (tid == 0) {
        tc::mbar_init(q_full, 32);
        tc::mbar_init(q_empty, 2);             // one arrival per MMA warp
#pragma unroll
        for (int i = 0; i < NSK; ++i) { tc::mbar_init(k_full + i * 8, 32); tc::mbar_init(k_empty + i * 8, 2); }
#pragma unroll
        for (int i = 0; i < NSV; ++i) { tc::mbar_init(v_full + i * 8, 32); tc::mbar_init(v_empty + i * 8, 2); }
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            tc::mbar_init(bar_s + x * 8, 1);
            // (a softmax warp cannot run a tile ahead of the other warps of its group: the scores
            // of the group's next tile are only issued once all four arrivals of this one are in)
            tc::mbar_init(bar_p + x * 8, 4);
            tc::mbar_init(bar_o + x * 8, 1);
        }
        tc::fence_mbar_init();
        s_dead = 0;
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    // The exponentials of the two softmax groups take turns (named barriers 2 and 3 as a token
    // that goes back and forth): the special-function unit is what both contend for, and a
    // group that has it to itself is done in half the time, while the other group loads,
    // reduces and stores.  Group B hands the first turn to group A here.
    if (is_softmax && X == 1) asm volatile("bar.arrive 2, 256;" ::: "memory");

    bool alive = true;
    auto timed_out = [&]() {
        s_dead = 1;
        alive = false;
        if (status) atomicExch(status, 2);
    };
    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        if (tc::mbar_test(bar, parity)) return;      // already there: no look at the dead flag, no timer
        if (!tc::mbar_wait(bar, parity, s_dead ? 1000ull : 1000000000ull)) timed_out();
    };

    // copy `rows` rows of D elements (row r from src + r * row_stride, rows >= valid_rows as zeros)
    // into a [block][row][128 B] tile with the 128-byte swizzle; one warp, 16 bytes per copy
    constexpr int CPRW = D / 8;                      // 16-byte chunks per row
    constexpr int RPI = 32 / CPRW;                   // rows covered by one pass of the warp
    const int ld_c = lane % CPRW, ld_row0 = lane / CPRW;
    auto load_tile = [&](const char* src0, size_t row_stride, int valid_rows, uint32_t dst0) {
        const char* src = src0 + (size_t)ld_row0 * row_stride + ld_c * 16;
        const uint32_t dblk = dst0 + (ld_c >> 3) * (128 * 128);
#pragma unroll 8
        for (int it = 0; it < 128 / RPI; ++it) {
            const int row = ld_row0 + it * RPI;
            const bool valid = row < valid_rows;
            cp_async16<0>(dblk + row * 128 + (((ld_c & 7) ^ (row & 7)) << 4), valid ? src : src0, valid ? 16 : 0, 0);
            src += (size_t)RPI * row_stride;
        }
    };

    // ---- work items: (256 query rows, head, sequence), late (heavy) query rows first ----
    const int n_qt = (p.tq + 2 * BM - 1) / (2 * BM);
    const int per_qt = p.q_heads * p.batch;
    const int n_items = n_qt * per_qt;
    int J0 = 0;                                      // running number of the item's first K/V tile
    int JX0 = 0;                                     // softmax warps: running tile number of their query tile
    int JA0 = 0, JB0 = 0;                            // MMA lane: the same for A and B
    int item_no = 0;                                 // items with tiles this CTA has started
    // Round k hands items k * grid .. (k + 1) * grid - 1 to the CTAs, in CTA order in even rounds
    // and in reverse order in odd ones: the items get lighter with their number, and a CTA that
    // always took the i-th of a round would end 6 - 7 % (T 4096 .. 16384) above the mean.
    for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
        const int item = round * (int)gridDim.x +
                         ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (item >= n_items) continue;
        const int qt = n_qt - 1 - item / per_qt;
        const int rem = item - (item / per_qt) * per_qt;
        const int b = rem / p.q_heads, h = rem - b * p.q_heads;
        const int kvh = h / p.group;
        const int m0 = qt * 2 * BM;
        int q_len, kv_len;
        prefill_lengths(p, b, q_len, kv_len);
        auto tiles_of = [&](int m) {                 // K/V tiles the query tile starting at row m needs
            if (m >= q_len) return 0;
            const int end = prefill_row_end(min(m + BM, q_len) - 1, q_len, kv_len, p.causal);
            return (end + BN - 1) / BN;
        };
        const int nA = tiles_of(m0), nB = tiles_of(m0 + BM);
        const int n = max(nA, nB);
        const int my_row = m0 + X * BM + row_l;      // (softmax threads)
        const int nX = X ? nB : nA;
        const long long out_off = (((long long)b * p.tq + my_row) * p.q_heads + h) * D;
        if (is_softmax && nX == 0 && my_row < p.tq) {   // nothing visible: zero rows
            uint4* dst = reinterpret_cast<uint4*>(op + out_off);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (n == 0) continue;                        // no role does anything else

        if (is_kload) {
            // =============================== loader of Q and K ===============================
            if (item_no >= 1) wait_bar(q_empty, (item_no - 1) & 1);
            const size_t q_stride = (size_t)p.q_heads * D * 2;
            const char* qsrc = reinterpret_cast<const char*>(qp) + (((size_t)b * p.tq + m0) * p.q_heads + h) * D * 2;
            if (nA) load_tile(qsrc, q_stride, q_len - m0, sq);
            if (nB) load_tile(qsrc + (size_t)BM * q_stride, q_stride, q_len - m0 - BM, sq + G::kTileBytes);
            tc::cp_async_arrive(q_full);
            const size_t row_stride = (size_t)p.kv_heads * D * 2;
            const char* ksrc = kp + (size_t)b * p.tk * row_stride + (size_t)kvh * D * 2;
            for (int j = 0; j < n; ++j) {
                const int J = J0 + j, stage = J % NSK;
                if (J >= NSK) wait_bar(k_empty + stage * 8, ((J / NSK) - 1) & 1);
                load_tile(ksrc + (size_t)j * BN * row_stride, row_stride, kv_len - j * BN, sk + stage * G::kTileBytes);
                tc::cp_async_arrive(k_full + stage * 8);
            }
        } else if (is_vload) {
            // =============================== loader of V ===============================
            const size_t row_stride = (size_t)p.kv_heads * D * 2;
            const char* vsrc = vp + (size_t)b * p.tk * row_stride + (size_t)kvh * D * 2;
            for (int j = 0; j < n; ++j) {
                const int J = J0 + j, stage = J % NSV;
                if (J >= NSV) wait_bar(v_empty + stage * 8, ((J / NSV) - 1) & 1);
                load_tile(vsrc + (size_t)j * BN * row_stride, row_stride, kv_len - j * BN, sv + stage * G::kTileBytes);
                tc::cp_async_arrive(v_full + stage * 8);
            }
        } else if (is_mma) {
            // =============================== MMA warp of query tile x ===============================
            {
                const uint32_t elected = tc::elect_one();
                const int x = warp - 10;             // this warp's query tile
                const int nx = x ? nB : nA;
                const int Jx0 = x ? JB0 : JA0;
                const uint32_t idesc_s = tc::idesc_f16(BM, HN, AB_TYPE);
                const uint32_t idesc_o = tc::idesc_f16(BM, D, AB_TYPE) | tc::kIdescBMnMajor;
                const uint64_t dq = tc::smem_desc_sw128_kmajor(sq + x * G::kTileBytes);
                const uint64_t dk0 = tc::smem_desc_sw128_kmajor(sk);
                const uint64_t dv0 = tc::smem_desc_sw128_mnmajor(sv, BN * 128);
                const uint32_t s_col = tmem + G::kColS + x * BN;
                const uint32_t o_col = tmem + G::kColO + x * D;
                // S_x(j, h) = Q_x . K(j)[keys 64 h .. 64 h + 63]^T; the first half waits for K(j)
                auto scores_of = [&](int j, int h) {
                    const int J = J0 + j, stage = J % NSK;
                    if (h == 0) {
                        wait_bar(k_full + stage * 8, (J / NSK) & 1);
                        tc::fence_async_smem();
                        tc::tc_fence_after();
                    }
                    const uint64_t dk = dk0 + (uint64_t)((stage * G::kTileBytes + h * HN * 128) >> 4);
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc::mma_f16_ss_w(elected, s_col + h * HN, dq + (uint64_t)((kb * (BM * 128) + k * 32) >> 4),
                                             dk + (uint64_t)((kb * (BN * 128) + k * 32) >> 4), idesc_s,
                                             (kb | k) ? 1u : 0u);
                    }
                    tc::mma_commit_w(elected, bar_s + (x * 2 + h) * 8);
                    if (h == 1) {
                        tc::mma_commit_w(elected, k_empty + stage * 8);       // this warp is done with K(j)
                        if (j == nx - 1) tc::mma_commit_w(elected, q_empty);  // ... and with Q_x
                    }
                };
                // O_x += P_x(j, h) . V(j)[keys 64 h .. 64 h + 63]; the first half waits for V(j)
                auto pv_of = [&](int j, int h) {
                    wait_bar(bar_p + (x * 2 + h) * 8, (Jx0 + j) & 1);
                    const int J = J0 + j, stage = J % NSV;
                    if (h == 0) { wait_bar(v_full + stage * 8, (J / NSV) & 1); tc::fence_async_smem(); }
                    tc::tc_fence_after();
                    const uint64_t dv = dv0 + (uint64_t)((stage * G::kTileBytes + h * (HN / 16) * 2048) >> 4);
#pragma unroll
                    for (int k = 0; k < HN / 16; ++k)
                        tc::mma_f16_ts_w(elected, o_col, s_col + h * HN + k * 8, dv + (uint64_t)((k * 2048) >> 4), idesc_o, (j | h | k) ? 1u : 0u);
                    tc::mma_commit_w(elected, bar_o + (x * 2 + h) * 8);
                    if (h == 1) tc::mma_commit_w(elected, v_empty + stage * 8);   // this warp is done with V(j)
                };
                // A K or V tile this warp has no use for (the other query tile reaches further) is
                // released by a plain arrival, but only once the tile has landed: an arrival for the
                // stage's next use could otherwise be counted towards this one
                auto pass_k = [&](int j) {
                    const int J = J0 + j, stage = J % NSK;
                    wait_bar(k_full + stage * 8, (J / NSK) & 1);
                    if (elected) tc::mbar_arrive(k_empty + stage * 8);
                };
                auto pass_v = [&](int j) {
                    const int J = J0 + j, stage = J % NSV;
                    wait_bar(v_full + stage * 8, (J / NSV) & 1);
                    if (elected) tc::mbar_arrive(v_empty + stage * 8);
                };
                wait_bar(q_full, item_no & 1);
                if (nx) { scores_of(0, 0); scores_of(0, 1); }
                else { if (elected) tc::mbar_arrive(q_empty); pass_k(0); }
                for (int j = 0; j < n; ++j) {
                    if (j < nx) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            // S_x(j+1, h) reuses the columns of S_x(j, h) / P_x(j, h): P.V(j, h) is queued
                            // ahead of it and the tensor pipe runs this warp's products in order
                            pv_of(j, h);
                            if (j + 1 < nx) scores_of(j + 1, h);
                        }
                        if (j + 1 >= nx && j + 1 < n) pass_k(j + 1);
                    } else {
                        pass_v(j);
                        if (j + 1 < n) pass_k(j + 1);
                    }
                }
            }
            __syncwarp();
        } else if (nX > 0) {
            // =============================== softmax warps of query tile X ===============================
            const int my_end = my_row < q_len ? prefill_row_end(my_row, q_len, kv_len, p.causal) : 0;
            const uint32_t s_addr = tmem + G::kColS + X * BN + lane_sel;
            const uint32_t o_addr = tmem + G::kColO + X * D + lane_sel;
            float m_run = -INFINITY, l_run = 0.f;
            const int turns = 2 * min(nA, nB);      // half tiles both groups have

            for (int j = 0; j < nX; ++j) {
                const int Jx = JX0 + j;
#pragma unroll
                for (int h = 0; h < 2; ++h) {        // the tile's keys in two halves of 64
                    wait_bar(bar_s + (X * 2 + h) * 8, Jx & 1);
                    tc::tc_fence_after();
                    const int t_base = j * BN + h * HN;
                    // ---- this row's 64 scores ----
                    float sc[HN];
#pragma unroll
                    for (int q = 0; q < HN / 32; ++q) {
                        uint32_t r[32];
                        tc::tmem_ld32(s_addr + h * HN + q * 32, r);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 32; ++c) sc[q * 32 + c] = __uint_as_float(r[c]);
                    }
                    if (t_base + HN > my_end) {      // some of these positions are masked
#pragma unroll
                        for (int c = 0; c < HN; ++c)
                            if (t_base + c >= my_end) sc[c] = -INFINITY;
                    }
                    float mx;
                    {
                        float a0 = sc[0], a1 = sc[1], a2 = sc[2], a3 = sc[3];
#pragma unroll
                        for (int c = 4; c < HN - 4; c += 8) {
                            a0 = tc::max3(a0, sc[c], sc[c + 1]); a1 = tc::max3(a1, sc[c + 2], sc[c + 3]);
                            a2 = tc::max3(a2, sc[c + 4], sc[c + 5]); a3 = tc::max3(a3, sc[c + 6], sc[c + 7]);
                        }
                        a0 = tc::max3(a0, sc[HN - 4], sc[HN - 3]);
                        a1 = tc::max3(a1, sc[HN - 2], sc[HN - 1]);
                        mx = fmaxf(tc::max3(a0, a1, a2), a3) * p.scale_log2;
                    }
                    const bool need = mx > m_run + kRescaleSlack;
                    float alpha = 1.f;
                    if (need) {
                        const float mn = fmaxf(m_run, mx);
                        alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - mn);
                        m_run = mn;
                        l_run *= alpha;
                    }
                    const float nref = m_run == -INFINITY ? 0.f : -m_run;
                    // exponents first, then the exponentials alone inside this group's turn (volatile,
                    // so that they stay between the two barriers), sums and conversions after it
#pragma unroll
                    for (int c = 0; c < HN; c += 2) tc::fma2(sc[c], sc[c + 1], sc[c], sc[c + 1], p.scale_log2, nref);
                    const bool turn = 2 * j + h < turns;   // both groups still have half tiles: take turns
                    if (turn) {
                        if (X == 0) asm volatile("bar.sync 2, 256;" ::: "memory");
                        else asm volatile("bar.sync 3, 256;" ::: "memory");
                    }
#pragma unroll
                    for (int c = 0; c < HN; ++c) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(sc[c]));
                    if (turn) {
                        if (X == 0) asm volatile("bar.arrive 3, 256;" ::: "memory");
                        else asm volatile("bar.arrive 2, 256;" ::: "memory");
                    }
                    uint32_t pw[HN / 2];
                    {
                        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                        for (int c = 0; c < HN; c += 2) {
                            tc::add2(ps0, ps1, sc[c], sc[c + 1]);
                            pw[c / 2] = Ops::pack(sc[c], sc[c + 1]);
                        }
                        l_run += ps0 + ps1;
                    }
                    // ---- O_X may be rescaled once P.V of the half tile before is done ----
                    if ((j > 0 || h > 0) && __any_sync(0xffffffffu, need)) {   // warp-uniform: TMEM ld/st are collective
                        wait_bar(bar_o + (X * 2 + (h ^ 1)) * 8, (h ? Jx : Jx - 1) & 1);
                        tc::tc_fence_after();
#pragma unroll
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            uint32_t o[32];
                            tc::tmem_ld32(o_addr + c0, o);
                            tc::tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                            tc::tmem_st32(o_addr + c0, o);
                        }
                    }
                    // ---- P(j, h) goes over the first 32 columns of S(j, h) ----
                    tc::tmem_st32(s_addr + h * HN, pw);
                    tc::tmem_st_wait();
                    tc::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(bar_p + (X * 2 + h) * 8);
                }
            }

            // ---- the finished rows: wait for the last P.V, normalise, store ----
            wait_bar(bar_o + (X * 2 + 1) * 8, (JX0 + nX - 1) & 1);
            tc::tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const bool write = my_row < p.tq && alive;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                tc::tmem_ld32(o_addr + c0, o);
                tc::tmem_ld_wait();
                if (write) {
                    uint4* dst = reinterpret_cast<uint4*>(op + out_off + c0);
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        uint4 v;
                        v.x = Ops::pack(__uint_as_float(o[c8 * 8 + 0]) * inv, __uint_as_float(o[c8 * 8 + 1]) * inv);
                        v.y = Ops::pack(__uint_as_float(o[c8 * 8 + 2]) * inv, __uint_as_float(o[c8 * 8 + 3]) * inv);
                        v.z = Ops::pack(__uint_as_float(o[c8 * 8 + 4]) * inv, __uint_as_float(o[c8 * 8 + 5]) * inv);
                        v.w = Ops::pack(__uint_as_float(o[c8 * 8 + 6]) * inv, __uint_as_float(o[c8 * 8 + 7]) * inv);
                        dst[c8] = v;
                    }
                }
            }
            tc::tc_fence_before();                   // the loads of O_X are done before this warp's next arrival
        }
        J0 += n;
        JX0 += nX;
        JA0 += nA;
        JB0 += nB;
        ++item_no;
    }
    if (is_kload || is_vload) cp_async_wait<0>();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    if (warp == 0) tc::tmem_dealloc(tmem, kPpTmemCols);
}

}  // namespace gqa_b200

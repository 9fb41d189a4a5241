// Dense GQA prefill on the 5th-generation tensor cores, warp-specialised: fp16 / bf16,
// head_dim 64 / 128.  Persistent CTAs (one per SM) walk the work items (batch, query head,
// 128 query rows), heaviest first.
//
//   S[128 x 128] = Q[128 x D] . K_tile[128 x D]^T      A = Q from TENSOR MEMORY, B = K tile (K-major)
//   O[128 x D]  += P[128 x 128] . V_tile[128 x D]      A = P from TENSOR MEMORY, B = V tile as it
//                                                      lies in memory ([key][d], an MN-major operand)
// Both A operands live in tensor memory: Q is written there once per item (tcgen05.st from
// registers) and P is written over the scores it was computed from, so an MMA reads only its
// B tile from shared memory (with A in shared memory a 128-row operand is another 4 KB per
// MMA, which is what the barrier-per-tile predecessor of this kernel spent its shared-memory
// bandwidth on).  Tiles of 128 keys make every MMA 128 x 128 x 16: the tensor pipe is then
// busy for about as long as one MMA takes its lane to issue.
//
// TMEM (512 columns): two score buffers of 128 columns (P(j), 64 columns of packed 16-bit
// pairs, overwrites the first half of S(j)), D columns of output, D / 2 columns of Q.
// Shared memory: a three-stage ring of K tiles and one of V tiles (32 KB per tile at D 128).
//
// Warp roles (352 threads):
//   warps 0-7   softmax: two threads per query row (64 score columns each); they also move Q
//               into tensor memory and the finished rows out
//   warps 8-9   loaders: 16-byte cp.async of K and V tiles, completion by
//               cp.async.mbarrier.arrive
//   warp 10     one lane issues every tcgen05.mma
// No CTA-wide barrier in the loop and none between items: the mbarriers are initialised once
// and their phases run on across the items of a CTA (every tile has a running number J; stage,
// buffer and parity of each hand-off derive from it), so the loaders run ahead into the next
// item, and an item's rows leave tensor memory only after the next item's Q went in (the
// tensor cores compute that item's first scores meanwhile).
//   k_full[3] / v_full[3]    64 loader arrivals (when their copies land)      -> MMA lane
//   k_empty[3]               tcgen05.commit: Q.K^T of the stage's tile done   -> loaders
//   v_empty[3]               tcgen05.commit: P.V of the stage's tile done     -> loaders, softmax (O may be touched)
//   bar_s[2]                 tcgen05.commit: scores of a tile are in TMEM     -> softmax
//   bar_p[2]                 8 warp arrivals: P is in TMEM, O rescaled        -> MMA lane
//   bar_q                    8 warp arrivals: the item's Q is in TMEM         -> MMA lane
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

constexpr int kWsBM = 128;
constexpr int kWsBN = 128;
constexpr int kWsSoftmaxThreads = 256;
constexpr int kWsLoadThreads = 64;
constexpr int kWsThreads = kWsSoftmaxThreads + kWsLoadThreads + 32;
constexpr int kWsStages = 3;
constexpr int kWsTmemCols = 512;

template <int D> struct PrefillWsGeom {
    static constexpr int kKB = D / 64;                           // 128-byte blocks of a K/V row
    static constexpr int kTileBytes = kKB * kWsBN * 128;         // one K or V tile: [block][key][128 B]
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kWsStages * kTileBytes;
    static constexpr int kTileSmem = 2 * kWsStages * kTileBytes; // 192 KB at D 128, 96 KB at D 64
    // a floor above half an SM's shared memory: a second resident CTA could never get tensor memory
    static constexpr int kSmemBytes = kTileSmem < 120 * 1024 ? 120 * 1024 : kTileSmem;
    static constexpr int kColS = 0;                              // 2 x 128
    static constexpr int kColO = 2 * kWsBN;                      // D columns
    static constexpr int kColQ = kColO + D;                      // D / 2 columns
    static_assert(kColQ + D / 2 <= kWsTmemCols, "TMEM budget");
};

template <typename T, int D>
__global__ void __launch_bounds__(kWsThreads, 1)
gqa_prefill_ws_kernel(const PrefillParams p, int* status) {
    using G = PrefillWsGeom<D>;
    using Ops = MmaOps<T>;
    constexpr int BM = kWsBM, BN = kWsBN, NT = kWsSoftmaxThreads, NL = kWsLoadThreads, NS = kWsStages;
    constexpr int KB = G::kKB;
    constexpr int AB_TYPE = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr int HC = BN / 2;                       // score columns per softmax thread
    constexpr int OC = D / 2;                        // output columns per softmax thread
    static_assert(OC % 32 == 0, "output half rows are moved 32 columns at a time");

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t s_bar[4 * NS + 5];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    __shared__ float s_max[2][2][kWsBM];             // [tile parity][column half][row]: half-row maxima
    __shared__ float s_half[2][kWsBM];               // [column half][row]: half-row sums at the end of an item

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_loader = tid >= NT && tid < NT + NL, is_mma = tid >= NT + NL;
    const int quad = warp & 3, hf = (warp >> 2) & 1; // softmax warps: TMEM lane quadrant, column half
    const int row_l = quad * 32 + lane;              // softmax thread's row of the 128-row tile
    const T* qp = reinterpret_cast<const T*>(p.q);
    const char* kp = reinterpret_cast<const char*>(p.k);
    const char* vp = reinterpret_cast<const char*>(p.v);
    T* op = reinterpret_cast<T*>(p.out);

    const uint32_t s_base = tc::smem_u32(smem);
    if (s_base & 1023u) {                            // the swizzled tiles need a 1024-byte aligned base
        if (tid == 0 && status) atomicExch(status, 3);
        return;
    }
    const uint32_t sk = s_base + G::kOffK, sv = s_base + G::kOffV;
    const uint32_t k_full = tc::smem_u32(&s_bar[0]);
    const uint32_t k_empty = tc::smem_u32(&s_bar[NS]);
    const uint32_t v_full = tc::smem_u32(&s_bar[2 * NS]);
    const uint32_t v_empty = tc::smem_u32(&s_bar[3 * NS]);
    const uint32_t bar_s0 = tc::smem_u32(&s_bar[4 * NS]);          // [2]
    const uint32_t bar_p = tc::smem_u32(&s_bar[4 * NS + 2]);       // [2], by tile parity
    const uint32_t bar_q = tc::smem_u32(&s_bar[4 * NS + 4]);

    if (warp == 0) { tc::tmem_alloc(tc::smem_u32(&s_tmem), kWsTmemCols); tc::tmem_relinquish(); }
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            tc::mbar_init(k_full + i * 8, NL); tc::mbar_init(k_empty + i * 8, 1);
            tc::mbar_init(v_full + i * 8, NL); tc::mbar_init(v_empty + i * 8, 1);
        }
        tc::mbar_init(bar_s0, 1);
        tc::mbar_init(bar_s0 + 8, 1);
        // (bar_p: two barriers used alternately.  A warp can be one tile ahead of another warp,
        // and its next arrival must not count towards the phase the other is still in; it cannot
        // be two ahead, because the scores of tile J + 2 are only issued once every warp's P(J)
        // has arrived.)
        tc::mbar_init(bar_p, NT / 32);               // one arrival per softmax warp
        tc::mbar_init(bar_p + 8, NT / 32);
        tc::mbar_init(bar_q, NT / 32);
        tc::fence_mbar_init();
        s_dead = 0;
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_o = tmem + G::kColO, tmem_q = tmem + G::kColQ;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;

    bool alive = true;
    auto timed_out = [&]() {
        s_dead = 1;
        alive = false;
        if (status) atomicExch(status, 2);
    };
    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        if (!tc::mbar_wait(bar, parity, s_dead ? 1000ull : 1000000000ull)) timed_out();
    };

    // The rows of an item are stored at the start of the next item, after its Q went to tensor
    // memory (nothing writes O before P.V of the next item's first tile, which waits for every
    // softmax warp's P, i.e. until after its store).
    bool st_pending = false, st_write = false;
    long long st_row = 0;                            // element offset of this thread's output half row
    float st_inv = 0.f;
    auto store_rows = [&]() {
#pragma unroll
        for (int c0 = 0; c0 < OC; c0 += 32) {
            uint32_t o[32];
            tc::tmem_ld32(tmem_o + lane_sel + hf * OC + c0, o);
            tc::tmem_ld_wait();
            if (st_write) {
                uint4* dst = reinterpret_cast<uint4*>(op + st_row + c0);
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    uint4 v;
                    v.x = Ops::pack(__uint_as_float(o[c8 * 8 + 0]) * st_inv, __uint_as_float(o[c8 * 8 + 1]) * st_inv);
                    v.y = Ops::pack(__uint_as_float(o[c8 * 8 + 2]) * st_inv, __uint_as_float(o[c8 * 8 + 3]) * st_inv);
                    v.z = Ops::pack(__uint_as_float(o[c8 * 8 + 4]) * st_inv, __uint_as_float(o[c8 * 8 + 5]) * st_inv);
                    v.w = Ops::pack(__uint_as_float(o[c8 * 8 + 6]) * st_inv, __uint_as_float(o[c8 * 8 + 7]) * st_inv);
                    dst[c8] = v;
                }
            }
        }
        tc::tc_fence_before();                       // the loads of O are done before the barrier arrivals that follow
        st_pending = false;
    };

    // ---- work items: (query tile, head, sequence), late (heavy) query tiles first ----
    const int n_qt = (p.tq + BM - 1) / BM;
    const int per_qt = p.q_heads * p.batch;
    const int n_items = n_qt * per_qt;
    int J0 = 0;                                      // running number of the item's first tile
    int item_no = 0;                                 // items with tiles this CTA has started
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int qt = n_qt - 1 - item / per_qt;
        const int rem = item - (item / per_qt) * per_qt;
        const int b = rem / p.q_heads, h = rem - b * p.q_heads;
        const int kvh = h / p.group;
        const int m0 = qt * BM;
        int q_len, kv_len;
        prefill_lengths(p, b, q_len, kv_len);
        const int my_row = m0 + row_l;               // (softmax threads)
        int tile_end = 0;
        if (m0 < q_len) tile_end = prefill_row_end(min(m0 + BM, q_len) - 1, q_len, kv_len, p.causal);
        const int n_tiles = (tile_end + BN - 1) / BN;
        const long long out_off = (((long long)b * p.tq + my_row) * p.q_heads + h) * D + hf * OC;
        if (n_tiles == 0) {                          // nothing visible: zero rows; no role does anything else
            if (!is_loader && !is_mma && my_row < p.tq) {
                uint4* dst = reinterpret_cast<uint4*>(op + out_off);
#pragma unroll
                for (int c = 0; c < OC / 8; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
            }
            continue;
        }

        if (is_loader) {
            // =============================== loader warps ===============================
            const int lt = tid - NT;
            constexpr int CPRW = D / 8;              // 16-byte chunks per row
            constexpr int RPI = NL / CPRW;           // rows covered by one pass of the loader threads
            static_assert(NL % CPRW == 0 && BN % RPI == 0, "copy pattern");
            const int ld_c = lt % CPRW, ld_row0 = lt / CPRW;
            const size_t row_stride = (size_t)p.kv_heads * D * 2;
            const size_t seq_off = (size_t)b * p.tk * row_stride + (size_t)kvh * D * 2 + ld_c * 16;
            auto load_tile = [&](const char* base, uint32_t dst0, int j) {
                const char* src = base + seq_off + ((size_t)j * BN + ld_row0) * row_stride;
                const uint32_t dblk = dst0 + (ld_c >> 3) * (BN * 128);
#pragma unroll 8
                for (int it = 0; it < BN / RPI; ++it) {
                    const int row = ld_row0 + it * RPI;
                    const bool valid = j * BN + row < kv_len;
                    cp_async16<0>(dblk + row * 128 + (((ld_c & 7) ^ (row & 7)) << 4), valid ? src : base,
                                  valid ? 16 : 0, 0);
                    src += (size_t)RPI * row_stride;
                }
            };
            // K runs two tiles ahead of V (the scores of tile j + 2 are issued before P.V of tile j)
            for (int step = 0; step < n_tiles + 2; ++step) {
                if (step < n_tiles) {
                    const int J = J0 + step, stage = J % NS;
                    if (J >= NS) wait_bar(k_empty + stage * 8, ((J / NS) - 1) & 1);
                    load_tile(kp, sk + stage * G::kTileBytes, step);
                    tc::cp_async_arrive(k_full + stage * 8);
                }
                if (step >= 2) {
                    const int J = J0 + step - 2, stage = J % NS;
                    if (J >= NS) wait_bar(v_empty + stage * 8, ((J / NS) - 1) & 1);
                    load_tile(vp, sv + stage * G::kTileBytes, step - 2);
                    tc::cp_async_arrive(v_full + stage * 8);
                }
            }
        } else if (is_mma) {
            // =============================== MMA warp: one lane issues everything ===============================
            if (lane == 0) {
                const uint32_t idesc_s = tc::idesc_f16(BM, BN, AB_TYPE);
                const uint32_t idesc_o = tc::idesc_f16(BM, D, AB_TYPE) | tc::kIdescBMnMajor;
                const uint64_t dk0 = tc::smem_desc_sw128_kmajor(sk);
                const uint64_t dv0 = tc::smem_desc_sw128_mnmajor(sv, BN * 128);
                auto scores_of = [&](int j) {        // wait for K(j), then S(j) = Q K(j)^T into buffer J & 1
                    const int J = J0 + j, stage = J % NS;
                    wait_bar(k_full + stage * 8, (J / NS) & 1);
                    tc::fence_async_smem();
                    tc::tc_fence_after();
                    const uint64_t dk = dk0 + (uint64_t)((stage * G::kTileBytes) >> 4);
                    const uint32_t d = tmem + (J & 1) * BN;
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc::mma_f16_ts(d, tmem_q + kb * 32 + k * 8,
                                           dk + (uint64_t)((kb * (BN * 128) + k * 32) >> 4), idesc_s,
                                           (kb | k) ? 1u : 0u);
                    }
                    tc::mma_commit(bar_s0 + (J & 1) * 8);
                    tc::mma_commit(k_empty + stage * 8);
                };
                wait_bar(bar_q, item_no & 1);        // this item's Q is in tensor memory
                tc::tc_fence_after();
                scores_of(0);
                if (n_tiles > 1) scores_of(1);
                for (int j = 0; j < n_tiles; ++j) {
                    const int J = J0 + j, stage = J % NS;
                    wait_bar(bar_p + (J & 1) * 8, (J >> 1) & 1);   // P(j) is in tensor memory, O rescaled
                    wait_bar(v_full + stage * 8, (J / NS) & 1);
                    tc::fence_async_smem();
                    tc::tc_fence_after();
                    const uint64_t dv = dv0 + (uint64_t)((stage * G::kTileBytes) >> 4);
                    const uint32_t pa = tmem + (J & 1) * BN;
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k)
                        tc::mma_f16_ts(tmem_o, pa + k * 8, dv + (uint64_t)((k * 2048) >> 4), idesc_o, (j | k) ? 1u : 0u);
                    tc::mma_commit(v_empty + stage * 8);
                    // S(j+2) reuses the buffer of S(j) / P(j): P.V(j) is queued ahead of it and the
                    // tensor pipe runs in order
                    if (j + 2 < n_tiles) scores_of(j + 2);
                }
            }
            __syncwarp();
        } else {
            // =============================== softmax warps ===============================
            const int my_end = my_row < q_len ? prefill_row_end(my_row, q_len, kv_len, p.causal) : 0;
            float m_run = -INFINITY, l_run = 0.f;

            // ---- Q: global -> registers -> tensor memory; this thread writes half of its row
            //      (D / 2 elements = D / 4 columns); rows past the last query row are zero ----
            {
                const T* qrow = qp + (((long long)b * p.tq + (my_row < q_len ? my_row : 0)) * p.q_heads + h) * D + hf * OC;
                constexpr int QW = D / 4;            // 32-bit words of this thread's half row
                uint32_t w[QW];
#pragma unroll
                for (int i = 0; i < QW / 4; ++i) {
                    const uint4 v = my_row < q_len ? __ldg(reinterpret_cast<const uint4*>(qrow) + i)
                                                   : make_uint4(0u, 0u, 0u, 0u);
                    w[i * 4] = v.x; w[i * 4 + 1] = v.y; w[i * 4 + 2] = v.z; w[i * 4 + 3] = v.w;
                }
                if constexpr (QW == 32) {
                    tc::tmem_st32(tmem_q + lane_sel + hf * QW, w);
                } else {
                    tc::tmem_st16(tmem_q + lane_sel + hf * QW, w);
                }
                tc::tmem_st_wait();
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(bar_q);
            }
            if (st_pending) store_rows();            // the previous item's rows (see above)

            for (int j = 0; j < n_tiles; ++j) {
                const int J = J0 + j;
                wait_bar(bar_s0 + (J & 1) * 8, (J >> 1) & 1);
                tc::tc_fence_after();
                // ---- this thread's 64 scores; the two threads of a row swap their maxima through
                //      shared memory when the two warps of the lane quadrant meet.  After that meeting
                //      both have read S(j), so P(j) may overwrite it ----
                float s[HC];
#pragma unroll
                for (int q = 0; q < HC / 32; ++q) {
                    uint32_t r[32];
                    tc::tmem_ld32(tmem + (J & 1) * BN + lane_sel + hf * HC + q * 32, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) s[q * 32 + c] = __uint_as_float(r[c]);
                }
                const int t_base = j * BN + hf * HC;
                if (t_base + HC > my_end) {
#pragma unroll
                    for (int c = 0; c < HC; ++c)
                        if (t_base + c >= my_end) s[c] = -INFINITY;
                }
                float mx;
                {
                    float a0 = s[0], a1 = s[1], a2 = s[2], a3 = s[3];
#pragma unroll
                    for (int c = 4; c < HC - 4; c += 8) {
                        a0 = tc::max3(a0, s[c], s[c + 1]); a1 = tc::max3(a1, s[c + 2], s[c + 3]);
                        a2 = tc::max3(a2, s[c + 4], s[c + 5]); a3 = tc::max3(a3, s[c + 6], s[c + 7]);
                    }
                    a0 = tc::max3(a0, s[HC - 4], s[HC - 3]);
                    a1 = tc::max3(a1, s[HC - 2], s[HC - 1]);
                    mx = fmaxf(tc::max3(a0, a1, a2), a3);
                }
                s_max[J & 1][hf][row_l] = mx;
                asm volatile("bar.sync %0, 64;" ::"r"(2 + quad) : "memory");
                mx = fmaxf(mx, s_max[J & 1][hf ^ 1][row_l]) * p.scale_log2;
                const bool need = mx > m_run + kRescaleSlack;
                float alpha = 1.f;
                if (need) {
                    const float mn = fmaxf(m_run, mx);
                    alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - mn);
                    m_run = mn;
                    l_run *= alpha;
                }
                const float nref = m_run == -INFINITY ? 0.f : -m_run;
                uint32_t pw[HC / 2];
                {
                    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                    for (int c = 0; c < HC; c += 2) {
                        float e0, e1;
                        tc::fma2(e0, e1, s[c], s[c + 1], p.scale_log2, nref);
                        const float p0 = fast_exp2(e0), p1 = fast_exp2(e1);
                        tc::add2(ps0, ps1, p0, p1);
                        pw[c / 2] = Ops::pack(p0, p1);
                    }
                    l_run += ps0 + ps1;              // this thread's half of the row sum
                }
                // ---- O may be rescaled once P.V(j-1) is done ----
                if (j > 0 && __any_sync(0xffffffffu, need)) {   // warp-uniform: TMEM ld/st are collective
                    wait_bar(v_empty + ((J - 1) % NS) * 8, ((J - 1) / NS) & 1);
                    tc::tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < OC; c0 += 32) {
                        uint32_t o[32];
                        tc::tmem_ld32(tmem_o + lane_sel + hf * OC + c0, o);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                        tc::tmem_st32(tmem_o + lane_sel + hf * OC + c0, o);
                    }
                }
                // ---- P(j) goes over the first 64 columns of S(j) ----
                tc::tmem_st32(tmem + (J & 1) * BN + lane_sel + hf * (HC / 2), pw);
                tc::tmem_st_wait();
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(bar_p + (J & 1) * 8);
            }
            wait_bar(v_empty + ((J0 + n_tiles - 1) % NS) * 8, ((J0 + n_tiles - 1) / NS) & 1);
            tc::tc_fence_after();

            // ---- row sum = the two halves, exchanged through shared memory; the rows themselves
            //      are stored at the start of the next item (or after the last one) ----
            s_half[hf][row_l] = l_run;
            asm volatile("bar.sync 1, %0;" ::"n"(kWsSoftmaxThreads) : "memory");
            const float l_tot = l_run + s_half[hf ^ 1][row_l];
            st_inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            st_row = out_off;
            st_write = my_row < p.tq && alive;
            st_pending = true;
        }
        J0 += n_tiles;
        ++item_no;
    }
    if (st_pending) store_rows();                    // the last item's rows
    if (is_loader) cp_async_wait<0>();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    if (warp == 0) tc::tmem_dealloc(tmem, kWsTmemCols);
}

}  // namespace gqa_b200

// Paged latent attention (MLA decode) on the 5th-generation tensor cores: tcgen05.mma with
// TMEM accumulators, run by a pair of CTAs (a cluster of two) that split the 576-wide cache
// row between them.  fp16 / bf16, dc = 512, dr = 64, dense attention.
//
// Why a pair.  With 128 query rows (heads x query tokens of one sequence) the output
// accumulator is 128 x 512 fp32 = all 512 TMEM columns of an SM, leaving no room for scores.
// So the row is cut at column 256:
//   rank 0 : latent columns   0..255                    (4 blocks of 64 columns = 128 bytes)
//   rank 1 : latent columns 256..511 + the 64 rotated   (5 blocks)
// Each CTA loads only its own blocks of every cache row (so every byte is read once by the
// pair), and those same blocks serve both contractions:
//   S_r[128 x 64]  = Q_r[128 x 64 nb] . C_r[64 x 64 nb]^T     partial scores over its columns
//   O_r[128 x 256] += P[128 x 64] . C_r[64 x 256]             its half of the latent output
// The full scores are S_0 + S_1: every thread sends its partial scores to the peer CTA through
// distributed shared memory (st.async, completing a transaction barrier there) and adds what it
// receives, so both CTAs hold the same scores bit for bit (a + b == b + a) and take the same
// softmax decisions without further talk.  (A thread only needs the peer's partials for its
// own 32 columns; the two threads of a row swap their half-row maxima.)
//
// Both A operands live in tensor memory, not in shared memory: the latent part of Q_r is
// written there once per work item (tcgen05.st from registers), and P is written over the score
// buffer it was computed from.  An MMA with 128 rows of A in shared memory re-reads 4 KB of A
// for every tile of B; that made the first version of this kernel shared-memory-bandwidth
// bound.  With A in TMEM an MMA reads only its B tile (the cache rows) from shared memory.  An
// MMA also costs its issuing lane about 70 cycles whatever its width, and every tile costs the
// softmax warps a fixed round of waits, TMEM round trips and fences: hence 64-token tiles.
//
// TMEM (512 columns): two score buffers of 64 columns (P(j) overwrites the first 32 columns of
// S(j)), 256 columns of output, 128 columns for the latent part of Q_r.  Shared memory: a
// three-stage ring of 64-token tiles (40 KB each), the rotated block of Q_r (16 KB, rank 1) and
// two 32 KB landing buffers: 200 KB, one CTA per SM.
//
// Warp roles (352 threads):
//   warps 0-7    softmax: two threads per query row (32 score columns each)
//   warps 8-9    loaders: 16-byte cp.async of this CTA's blocks of each cache row, one page lookup
//                per 32 tokens when the page size is a multiple of 32 tokens, else one per row
//   warp 10      one lane issues every tcgen05.mma
// There is no CTA-wide barrier in the token loop, and none between work items either: the
// mbarriers are initialised once per kernel and their phases run on across the items of a CTA
// pair (every tile the pair processes has a running number J, and stage, buffer and parity of
// every hand-off derive from J), so the loader warps run ahead into the next item's tiles while
// the softmax warps still store the current item's rows.  The hand-offs are mbarriers (and one
// 64-thread named barrier between the two warps that share a TMEM lane quadrant).  Every mbarrier wait is
// time-bounded: a wait that runs out marks the CTA dead and raises the status word, and the CTA
// still walks the protocol to the end, so its peer is never left waiting and no CTA exits
// while the other may still write into its memory.
//   full[3]    64 loader arrivals (when their copies land)   tile is in its stage   -> MMA lane
//   empty[3]   tcgen05.commit   P.C of the stage's tile is done: stage and O are free
//   bar_s[2]   tcgen05.commit   partial scores of a tile are in TMEM                -> softmax
//   bar_p[2]   8 warp arrivals  P is in TMEM, O rescaled (even / odd tiles)         -> MMA lane
//   bar_x[2]   transaction barriers: the peer's st.async stores complete 32 KB per tile
//   bar_free[2] 8 remote warp arrivals   the peer has consumed a landing buffer of its own
#pragma once

#include <type_traits>

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"
#include "mla_simt.cuh"
#include "tcgen05_util.cuh"

namespace gqa_b200 {

constexpr int kMlaTcRows = 128;        // query rows (token x head) per CTA pair
constexpr int kMlaTcBN = 64;           // tokens per tile
constexpr int kMlaTcSoftmaxThreads = 256;
constexpr int kMlaTcLoadThreads = 64;
constexpr int kMlaTcThreads = kMlaTcSoftmaxThreads + kMlaTcLoadThreads + 32;
constexpr int kMlaTcStages = 3;
constexpr int kMlaTcSBufs = 2;
constexpr int kMlaTcTmemCols = 512;
constexpr int kMlaTcDc = 512;
constexpr int kMlaTcDr = 64;
constexpr int kMlaTcWidth = kMlaTcDc + kMlaTcDr;

struct MlaTcGeom {
    static constexpr int kBlocks = 5;                                   // 128-byte column blocks (rank 1)
    static constexpr int kTileBlockBytes = kMlaTcBN * 128;              // 8 KB: one tile's rows of one block
    static constexpr int kStageBytes = kBlocks * kTileBlockBytes;       // 40 KB: [block][64 rows][128 B]
    static constexpr int kQRopeBytes = kMlaTcRows * 128;                // 16 KB: rotated query block (rank 1),
                                                                        // two of them (work items alternate)
    static constexpr int kXBytes = kMlaTcRows * kMlaTcBN * 4;           // 32 KB, two of them
    static constexpr int kOffK = 0;
    static constexpr int kOffQr = kOffK + kMlaTcStages * kStageBytes;
    static constexpr int kOffX = kOffQr + 2 * kQRopeBytes;
    static constexpr int kSmemBytes = kOffX + 2 * kXBytes;              // 221184
    // tensor memory columns
    static constexpr int kColS = 0;                                     // kMlaTcSBufs x 64
    static constexpr int kColO = kMlaTcSBufs * kMlaTcBN;                // 256
    static constexpr int kColQ = kColO + 256;                           // 128: the latent part of Q_r
    static_assert(kColQ + 4 * 32 <= kMlaTcTmemCols, "TMEM budget");
};

namespace tc {
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 16-byte store into another CTA's shared memory that, when it lands, completes 16 bytes of the
// transaction count of an mbarrier in that CTA: data and signal travel together, no fence.
__device__ __forceinline__ void st_async_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                            uint32_t cluster_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1,%2,%3,%4}, [%5];"
                 ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(cluster_bar) : "memory");
}
// the single arrival of a phase of a transaction barrier, announcing the bytes that will land
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// mbar_wait with cluster-scope acquire: orders the peer CTA's stores before the reads that follow.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, uint64_t max_ns) {
    uint64_t start = 0;
    for (uint32_t i = 0;; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 63u) == 63u) {
            const uint64_t now = global_timer_ns();
            if (start == 0) start = now;
            else if (now - start > max_ns) return false;
        }
    }
}
}  // namespace tc

// Schedule of the tensor-core kernel, computed on the device from the lengths (the host never
// reads them): tiles per unit, their exclusive prefix sum, and the number of consecutive tiles
// each range gets so that `pairs` CTA pairs share the tiles evenly.  One CTA.
constexpr int kMlaTcPlanThreads = 256;
constexpr int kMlaTcMinRange = 4;       // a range is at least 4 tiles (256 tokens)
__global__ void __launch_bounds__(kMlaTcPlanThreads)
mla_tc_plan_kernel(const MlaParams p, int pairs) {
    __shared__ int s_sum[kMlaTcPlanThreads];
    pdl_launch_dependents();
    pdl_wait();                                      // the previous call's kernels still read the schedule
    const int tid = threadIdx.x, U = p.tc_units, R = p.tq * p.heads;
    const int per = (U + kMlaTcPlanThreads - 1) / kMlaTcPlanThreads;
    const int lo = min(U, tid * per), hi = min(U, lo + per);
    int* prefix = p.tc_sched + 4;
    auto tiles_of = [&](int u) {
        const int b = u / p.tc_row_tiles, g0 = (u - b * p.tc_row_tiles) * kMlaTcRows;
        int end_max = 0;
        for (int t = g0 / p.heads; t <= (min(R, g0 + kMlaTcRows) - 1) / p.heads; ++t)
            end_max = max(end_max, mla_row_end(p, b, t));
        end_max = min(end_max, p.page * p.max_pages);    // a length past the table is clamped
        return (end_max + kMlaTcBN - 1) / kMlaTcBN;
    };
    int sum = 0;
    for (int u = lo; u < hi; ++u) sum += tiles_of(u);
    s_sum[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < kMlaTcPlanThreads; ++i) { const int x = s_sum[i]; s_sum[i] = run; run += x; }
        const int per_range = p.tc_force_range > 0 ? p.tc_force_range
                                                   : max(kMlaTcMinRange, (run + pairs - 1) / pairs);
        p.tc_sched[0] = run;
        p.tc_sched[1] = per_range;
        p.tc_sched[2] = (run + per_range - 1) / per_range;
        prefix[U] = run;
    }
    __syncthreads();
    int run = s_sum[tid];
    for (int u = lo; u < hi; ++u) { prefix[u] = run; run += tiles_of(u); }
}

// One warp per query row: fold the partial slots of the row's unit (slot = range + unit, for
// the ranges that overlap the unit), or nothing when one item covered the whole unit and wrote
// the final rows itself; rows of units without any visible token are zeroed here.
template <typename T>
__global__ void __launch_bounds__(kMlaMergeWarps * 32)
mla_tc_merge_kernel(const MlaParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * kMlaMergeWarps + (threadIdx.x >> 5);
    const int u = (int)(wid / kMlaTcRows), r = (int)(wid - (long long)u * kMlaTcRows);
    if (u >= p.tc_units) return;
    const int R = p.tq * p.heads;
    const int b = u / p.tc_row_tiles, g = (u - b * p.tc_row_tiles) * kMlaTcRows + r;
    if (g >= R) return;
    const int* prefix = p.tc_sched + 4;
    const int per_range = p.tc_sched[1];
    const int first = prefix[u], tiles = prefix[u + 1] - first;
    T* op = reinterpret_cast<T*>(p.out) + ((long long)b * R + g) * kMlaTcDc;
    if (tiles == 0) {
        for (int d = lane * 4; d < kMlaTcDc; d += 128) {
            op[d] = from_f32<T>(0.f); op[d + 1] = from_f32<T>(0.f);
            op[d + 2] = from_f32<T>(0.f); op[d + 3] = from_f32<T>(0.f);
        }
        return;
    }
    const int r0 = first / per_range, r1 = (first + tiles - 1) / per_range;
    if (r0 == r1) return;                            // one item covered the unit
    const float* ml = p.part_ml + ((long long)(r0 + u) * kMlaTcRows + r) * 2;         // slot stride below
    const float* acc = p.part_acc + ((long long)(r0 + u) * kMlaTcRows + r) * kMlaTcDc;
    const long long ml_stride = (long long)kMlaTcRows * 2, acc_stride = (long long)kMlaTcRows * kMlaTcDc;
    const int n = r1 - r0 + 1;
    // Slots are fetched four at a time and all of a batch's loads are issued before the first
    // use (a slot-by-slot loop is one L2 round trip after the other: 12 us for this kernel on
    // 64 x 128 rows); the additions keep the slot order, so the bits are those of that loop.
    float mx = -INFINITY;
    for (int s0 = 0; s0 < n; s0 += 4) {
        float2 e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            e[i] = s0 + i < n ? *reinterpret_cast<const float2*>(ml + (s0 + i) * ml_stride) : make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (e[i].y > 0.f) mx = fmaxf(mx, e[i].x);
    }
    float sum = 0.f;
    float4 a[kMlaTcDc / 128];
#pragma unroll
    for (int k = 0; k < kMlaTcDc / 128; ++k) a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < n; s0 += 4) {
        float2 e[4];
        float4 x[4][kMlaTcDc / 128];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool in = s0 + i < n;
            e[i] = in ? *reinterpret_cast<const float2*>(ml + (s0 + i) * ml_stride) : make_float2(0.f, 0.f);
#pragma unroll
            for (int k = 0; k < kMlaTcDc / 128; ++k)
                x[i][k] = in ? *reinterpret_cast<const float4*>(acc + (s0 + i) * acc_stride + lane * 4 + k * 128)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (e[i].y > 0.f) {
                const float w = fast_exp2(e[i].x - mx);
                sum += w * e[i].y;
#pragma unroll
                for (int k = 0; k < kMlaTcDc / 128; ++k) {
                    a[k].x += w * x[i][k].x; a[k].y += w * x[i][k].y;
                    a[k].z += w * x[i][k].z; a[k].w += w * x[i][k].w;
                }
            }
        }
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
    for (int k = 0; k < kMlaTcDc / 128; ++k) {
        const int d = lane * 4 + k * 128;
        op[d] = from_f32<T>(a[k].x * inv); op[d + 1] = from_f32<T>(a[k].y * inv);
        op[d + 2] = from_f32<T>(a[k].z * inv); op[d + 3] = from_f32<T>(a[k].w * inv);
    }
}

// grid (2 * pairs), cluster (2, 1, 1): persistent pairs that walk the schedule written by
// mla_tc_plan_kernel (p.tc_sched).  p.page_shift = log2(page) or -1.
template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMlaTcThreads, 1)
mla_attend_tc_kernel(const MlaParams p, int* status) {
    using G = MlaTcGeom;
    using Ops = MmaOps<T>;
    constexpr int BM = kMlaTcRows, BN = kMlaTcBN, NT = kMlaTcSoftmaxThreads, NL = kMlaTcLoadThreads;
    constexpr int NS = kMlaTcStages, NSB = kMlaTcSBufs;
    constexpr int AB_TYPE = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr int HC = BN / 2;                       // score columns per softmax thread

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t s_bar[2 * NS + NSB + 7];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    __shared__ float s_max[2][2][kMlaTcRows];        // [tile parity][column half][row]: half-row maxima
    __shared__ float s_half[2][kMlaTcRows];          // [column half][row]: half-row sums at the end of an item

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_loader = tid >= NT && tid < NT + NL, is_mma = tid >= NT + NL;
    const int quad = warp & 3, hf = (warp >> 2) & 1; // softmax warps: TMEM lane quadrant, column half
    const int row_l = quad * 32 + lane;              // softmax thread's row of the 128-row tile
    const uint32_t rank = tc::cluster_ctarank(), peer = rank ^ 1u;
    const int R = p.tq * p.heads;                    // query rows of one sequence
    const int nb = rank ? 5 : 4;                     // 128-byte blocks this CTA owns
    const int col0 = rank ? 256 : 0;                 // first cache column this CTA owns
    T* op = reinterpret_cast<T*>(p.out);

    pdl_launch_dependents();
    pdl_wait();                                      // the schedule and the queries come from earlier kernels
    const uint32_t s_base = tc::smem_u32(smem);
    if (s_base & 1023u) {                            // the swizzled tiles need a 1024-byte aligned base
        if (tid == 0 && status) atomicExch(status, 3);
        return;
    }
    const uint32_t sk = s_base + G::kOffK, sqr = s_base + G::kOffQr, sx = s_base + G::kOffX;
    const uint32_t bar_full = tc::smem_u32(&s_bar[0]);
    const uint32_t bar_empty = tc::smem_u32(&s_bar[NS]);
    const uint32_t bar_s0 = tc::smem_u32(&s_bar[2 * NS]);
    const uint32_t bar_p = tc::smem_u32(&s_bar[2 * NS + NSB]);
    const uint32_t bar_x = tc::smem_u32(&s_bar[2 * NS + NSB + 1]);      // [2], one per landing buffer
    const uint32_t bar_free = tc::smem_u32(&s_bar[2 * NS + NSB + 3]);   // [2]
    const uint32_t bar_q = tc::smem_u32(&s_bar[2 * NS + NSB + 5]);
    const uint32_t bar_p1 = tc::smem_u32(&s_bar[2 * NS + NSB + 6]);     // bar_p of the odd tiles

    if (warp == 0) { tc::tmem_alloc(tc::smem_u32(&s_tmem), kMlaTcTmemCols); tc::tmem_relinquish(); }
    if (tid == 0) s_dead = 0;
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_o = tmem + G::kColO, tmem_q = tmem + G::kColQ;

    // ---- this pair's share of the work: ranges of `per_range` consecutive tiles of the global
    //      tile sequence (all tiles of unit 0, then unit 1, ...; a unit = 128 query rows of one
    //      sequence).  A range may end inside a unit and start the next one: every (range, unit)
    //      overlap is one work item, and range + unit is a distinct partial slot for each. ----
    const int* sched = p.tc_sched;
    const int total_tiles = sched[0], per_range = sched[1], n_ranges = sched[2];
    const int* prefix = sched + 4;                   // prefix[u] = tiles before unit u, [units + 1]
    // tiles this pair will process over all of its ranges: they are numbered J = 0, 1, ... in the
    // order they are processed, across work items
    int pair_tiles = 0;
    for (int range = blockIdx.x >> 1; range < n_ranges; range += gridDim.x >> 1)
        pair_tiles += min(total_tiles, (range + 1) * per_range) - range * per_range;
    // With few heads most of the 128 rows are padding.  A softmax warp whose 32 rows hold no
    // query row in ANY unit of this launch takes no part at all (its rows of Q, S, P and O are
    // never read by anyone); the barrier counts and the bytes expected from the peer cover the
    // live warps only.  (The host passes 4 when units differ in their number of rows.)
    const int live_quads = p.tc_live_quads;
    const int live_warps = 2 * live_quads;
    const uint32_t x_bytes = (uint32_t)live_warps * 32u * (uint32_t)(kMlaTcBN / 2) * 4u;
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NS; ++i) { tc::mbar_init(bar_full + i * 8, NL); tc::mbar_init(bar_empty + i * 8, 1); }
#pragma unroll
        for (int i = 0; i < NSB; ++i) tc::mbar_init(bar_s0 + i * 8, 1);
        // (two barriers used alternately: a warp can be one tile ahead of another warp, and its
        // next arrival must not count towards the phase the other is still in; it cannot be two
        // ahead, because the scores of tile J + 2 are only issued once every warp's P(J) has arrived)
        tc::mbar_init(bar_p, live_warps);            // one arrival per live softmax warp
        tc::mbar_init(bar_p1, live_warps);
        tc::mbar_init(bar_q, live_warps);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(bar_x + i * 8, 1);         // one local arrival announcing the bytes per tile
            tc::mbar_init(bar_free + i * 8, live_warps);   // one arrival per live softmax warp of the peer
        }
        tc::fence_mbar_init();
        if (pair_tiles > 0) tc::mbar_arrive_expect_tx(bar_x, x_bytes);         // tile 0
        if (pair_tiles > 1) tc::mbar_arrive_expect_tx(bar_x + 8, x_bytes);     // tile 1
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();                          // both CTAs' barriers exist before any remote arrival
    tc::tc_fence_after();
    bool alive = true;
    int J0 = 0;                                      // running number of the item's first tile
    int item_no = 0;                                 // items of this pair so far
    // The rows of an item are not stored when its last tile is done but at the start of the next
    // item, after that item's queries have gone to tensor memory: the tensor cores then compute the
    // next item's first scores while the softmax threads move the finished accumulators out.
    // (Nothing writes O before P.C of the next item's first tile, which waits for every softmax
    // warp's P, i.e. until after its store.)
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    bool st_pending = false, st_final = false, st_write = false;
    int st_slot = 0;
    long long st_grow = 0;
    float st_inv = 1.f, st_m = 0.f, st_l = 0.f;
    auto store_rows = [&]() {
        float* pacc = p.part_acc + ((long long)st_slot * BM + row_l) * kMlaTcDc + col0;
#pragma unroll
        for (int c0 = hf * 128; c0 < (hf + 1) * 128; c0 += 32) {
            uint32_t o[32];
            tc::tmem_ld32(tmem_o + lane_sel + c0, o);
            tc::tmem_ld_wait();
            if (st_write) {
                if (st_final) {
                    uint4* dst = reinterpret_cast<uint4*>(op + st_grow * kMlaTcDc + col0 + c0);
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        uint4 v;
                        v.x = Ops::pack(__uint_as_float(o[c8 * 8 + 0]) * st_inv, __uint_as_float(o[c8 * 8 + 1]) * st_inv);
                        v.y = Ops::pack(__uint_as_float(o[c8 * 8 + 2]) * st_inv, __uint_as_float(o[c8 * 8 + 3]) * st_inv);
                        v.z = Ops::pack(__uint_as_float(o[c8 * 8 + 4]) * st_inv, __uint_as_float(o[c8 * 8 + 5]) * st_inv);
                        v.w = Ops::pack(__uint_as_float(o[c8 * 8 + 6]) * st_inv, __uint_as_float(o[c8 * 8 + 7]) * st_inv);
                        dst[c8] = v;
                    }
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(pacc + c0);
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4)
                        dst[c4] = make_uint4(o[c4 * 4], o[c4 * 4 + 1], o[c4 * 4 + 2], o[c4 * 4 + 3]);
                }
            }
        }
        if (!st_final && st_write && rank == 0 && hf == 0) {
            p.part_ml[((long long)st_slot * BM + row_l) * 2] = st_m;
            p.part_ml[((long long)st_slot * BM + row_l) * 2 + 1] = st_l;
        }
        tc::tc_fence_before();                       // the loads of O are done before the barrier arrivals below
        st_pending = false;
    };
    for (int range = blockIdx.x >> 1; range < n_ranges; range += gridDim.x >> 1) {
    int pos = range * per_range;
    const int range_end = min(total_tiles, pos + per_range);
    int u = 0;
    {   // last unit whose first tile is at or before pos
        int lo = 0, hi = p.tc_units;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= pos) lo = mid; else hi = mid;
        }
        u = lo;
    }
    while (pos < range_end) {
    while (prefix[u + 1] <= pos) ++u;                // units without tiles, or already done
    const int u_lo = prefix[u], u_tiles = prefix[u + 1] - u_lo;
    const int seg_lo = pos - u_lo, seg_hi = min(u_tiles, range_end - u_lo);
    pos = u_lo + seg_hi;
    const int slot = range + u;
    const bool final_out = seg_lo == 0 && seg_hi == u_tiles;   // the item is the whole unit: no partial

    // =============================== one work item ===============================
    const int b = u / p.tc_row_tiles;
    const int g0 = (u - b * p.tc_row_tiles) * BM, g = g0 + row_l;
    int end_max = 0;
    for (int t = g0 / p.heads; t <= (min(R, g0 + BM) - 1) / p.heads; ++t) end_max = max(end_max, mla_row_end(p, b, t));
    end_max = min(end_max, p.page * p.max_pages);    // a length past the table is clamped (as in the plan)
    const int t0 = seg_lo * BN;
    const int t1 = min(end_max, seg_hi * BN);
    const int n_tiles = seg_hi - seg_lo;
    const long long grow = (long long)b * R + g;     // global query row (softmax threads)
    const uint32_t sqr_i = sqr + (uint32_t)(item_no & 1) * G::kQRopeBytes;   // this item's rotated block of Q_r

    auto timed_out = [&]() {
        s_dead = 1;
        alive = false;
        if (status) atomicExch(status, 2);
    };
    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        if (tc::mbar_test(bar, parity)) return;      // already there: no look at the dead flag, no timer
        if (!tc::mbar_wait(bar, parity, s_dead ? 1000ull : 1000000000ull)) timed_out();
    };
    auto wait_bar_cluster = [&](uint32_t bar, uint32_t parity) {
        if (!tc::mbar_wait_cluster(bar, parity, s_dead ? 1000ull : 1000000000ull)) timed_out();
    };

    if (is_loader) {
        // =============================== loader warps ===============================
        const int lt = tid - NT;
        const int cpr = nb * 8;                      // 16-byte chunks of a row that this CTA owns
        if (rank) {   // the rotated block of Q_r stays in shared memory: [128 rows][128 B]; it rides
                      // on the full barrier of the item's first tile
            // The buffer was last used by the item before the previous one, whose tiles are all
            // numbered J0 - 2 or lower: once the scores of tile J0 - 2 are done (the tensor pipe
            // runs in order), nothing reads it any more.  That phase of bar_s cannot be
            // overtaken: its successor needs tile J0, which is loaded below.
            if (item_no >= 2) wait_bar(bar_s0 + ((J0 - 2) % NSB) * 8, ((J0 - 2) / NSB) & 1);
            const T* qr = reinterpret_cast<const T*>(p.qr);
            for (int i = lt; i < BM * 8; i += NL) {
                const int row = i >> 3, c = i & 7;
                const bool valid = g0 + row < R;
                const T* src = qr + ((long long)b * R + (valid ? g0 + row : 0)) * kMlaTcDr + c * 8;
                cp_async16<0>(sqr_i + row * 128 + ((c ^ (row & 7)) << 4), src, valid ? 16 : 0, 0);
            }
        }
        // this thread's chunks of a 32-row half tile: the same (row, 16-byte column) for every
        // half (the second half of a tile is 32 rows further in both the cache page and the stage)
        constexpr int HR = 32;                       // rows per half
        constexpr int MAXC = HR * 40 / NL;           // 20 chunks per thread for rank 1, 16 for rank 0
        const int nchunk = HR * cpr / NL;
        uint32_t soff[MAXC], doff[MAXC];             // byte offsets in the cache page run / in the stage
#pragma unroll
        for (int k = 0; k < MAXC; ++k) {
            const int i = lt + k * NL;
            const int row = i / cpr, c = i - row * cpr;
            soff[k] = (uint32_t)(row * kMlaTcWidth + col0 + c * 8) * 2u;
            doff[k] = (uint32_t)((c >> 3) * G::kTileBlockBytes + row * 128 + (((c & 7) ^ (row & 7)) << 4));
        }
        const char* cache = reinterpret_cast<const char*>(p.cache);
        const int32_t* trow = p.table + (long long)b * p.max_pages;
        const int last_block = (int)(p.num_blocks - 1);
        const bool page_run = p.page_shift >= 5;     // a 32-token half never straddles a page
        for (int j = 0; j < n_tiles; ++j) {
            const int J = J0 + j;
            const int stage = J % NS;
            if (J >= NS) wait_bar(bar_empty + stage * 8, ((J / NS) - 1) & 1);
#pragma unroll
            for (int half = 0; half < BN / HR; ++half) {
                const uint32_t st = sk + stage * G::kStageBytes + half * (HR * 128);
                const int tok0 = t0 + j * BN + half * HR;
                if (page_run) {
                    const int pg = min(tok0 >> p.page_shift, p.max_pages - 1);
                    // a page id outside the pool (a caller error) is clamped instead of faulting
                    const long long phys = min(max(__ldg(trow + pg), 0), last_block);
                    const char* base = cache + (phys * p.page + (tok0 & (p.page - 1))) * (kMlaTcWidth * 2);
                    const int rows_ok = t1 - tok0;   // rows below this are inside the chunk
#pragma unroll
                    for (int k = 0; k < MAXC; ++k) {
                        if (k < nchunk) {
                            const bool valid = (int)((doff[k] >> 7) & 31u) < rows_ok;
                            cp_async16<0>(st + doff[k], valid ? base + soff[k] : cache, valid ? 16 : 0, 0);
                        }
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < MAXC; ++k) {
                        if (k < nchunk) {
                            const int row = (int)((doff[k] >> 7) & 31u);
                            const int tok = tok0 + row;
                            const bool valid = tok < t1;
                            const char* src = cache;
                            if (valid) {
                                const int pg = p.page_shift >= 0 ? tok >> p.page_shift : tok / p.page;
                                const long long phys = min(max(__ldg(trow + pg), 0), last_block);
                                src = cache + (phys * p.page + (tok - pg * p.page)) * (kMlaTcWidth * 2) +
                                      (soff[k] - (uint32_t)row * (kMlaTcWidth * 2));
                            }
                            cp_async16<0>(st + doff[k], src, valid ? 16 : 0, 0);
                        }
                    }
                }
            }
            tc::cp_async_arrive(bar_full + stage * 8);
        }
    } else if (is_mma) {
        // =============================== MMA warp: one lane issues everything ===============================
        if (lane == 0) {
            const uint32_t idesc_s = tc::idesc_f16(BM, BN, AB_TYPE);
            const uint32_t idesc_o = tc::idesc_f16(BM, 256, AB_TYPE) | tc::kIdescBMnMajor;
            // Descriptors differ only in their start-address field ((address >> 4) in the low bits,
            // no carry out of it below 256 KB), so each one is a base plus a small offset: the
            // issuing lane's instruction stream per MMA stays a handful of instructions.
            const uint64_t dk0 = tc::smem_desc_sw128_kmajor(sk);
            const uint64_t dqr0 = tc::smem_desc_sw128_kmajor(sqr_i);
            const uint64_t dv0 = tc::smem_desc_sw128_mnmajor(sk, G::kTileBlockBytes);
            // S_r(j) = Q_r C_r(j)^T into score buffer j & 1.  A = the latent part of Q_r from tensor
            // memory (8 columns = 16 elements per step) and, on rank 1, its rotated block from
            // shared memory.  (An MMA costs the issuing lane about 70 cycles whatever its width,
            // which is why the tile is 64 tokens wide and not 32.)
            auto issue_qk = [&](int j) {
                const int J = J0 + j;
                const uint64_t dk = dk0 + (uint64_t)(((J % NS) * G::kStageBytes) >> 4);
                const uint32_t d = tmem + (J % NSB) * BN;
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_f16_ts(d, tmem_q + blk * 32 + k * 8,
                                       dk + (uint64_t)((blk * G::kTileBlockBytes + k * 32) >> 4), idesc_s,
                                       (blk | k) ? 1u : 0u);
                }
                if (rank) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_f16_ss(d, dqr0 + (uint64_t)((k * 32) >> 4),
                                       dk + (uint64_t)((4 * G::kTileBlockBytes + k * 32) >> 4), idesc_s, 1u);
                }
                tc::mma_commit(bar_s0 + (J % NSB) * 8);
            };
            // O_r += P C_r(j): A = P(j) from the first 32 columns of score buffer j & 1, B = the first
            // four blocks of the stage as an MN-major operand
            auto issue_pv = [&](int j) {
                const int J = J0 + j;
                const uint64_t dv = dv0 + (uint64_t)(((J % NS) * G::kStageBytes) >> 4);
                const uint32_t pa = tmem + (J % NSB) * BN;
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    tc::mma_f16_ts(tmem_o, pa + k * 8, dv + (uint64_t)((k * 2048) >> 4), idesc_o, (j | k) ? 1u : 0u);
                tc::mma_commit(bar_empty + (J % NS) * 8);
            };
            auto scores_of = [&](int j) {             // wait for tile j to land, then issue its scores
                wait_bar(bar_full + ((J0 + j) % NS) * 8, ((J0 + j) / NS) & 1);
                tc::fence_async_smem();
                tc::tc_fence_after();
                issue_qk(j);
            };
            wait_bar(bar_q, item_no & 1);            // this item's Q_r is in tensor memory
            tc::tc_fence_after();
            scores_of(0);                            // (the rotated block of Q_r rides on the first tile's barrier)
            if (n_tiles > 1) scores_of(1);
            for (int j = 0; j < n_tiles; ++j) {
                wait_bar(((J0 + j) & 1) ? bar_p1 : bar_p, ((J0 + j) >> 1) & 1);   // P(j) is in tensor memory, O rescaled
                tc::tc_fence_after();
                issue_pv(j);
                // S(j+2) reuses the buffer of S(j) / P(j): P.C(j) is queued ahead of it and the tensor
                // pipe runs in order
                if (j + 2 < n_tiles) scores_of(j + 2);
            }
        }
        __syncwarp();
    } else {
        // =============================== softmax warps ===============================
        const uint32_t peer_sx = tc::map_to_cta(sx, peer);
        const uint32_t peer_bar_x = tc::map_to_cta(bar_x, peer);
        const uint32_t peer_bar_free = tc::map_to_cta(bar_free, peer);
        const int my_end = g < R ? mla_row_end(p, b, g / p.heads) : 0;
        const int my_stop = min(my_end, t1);         // this row sees tokens [t0, my_stop) of the chunk
        float m_run = -INFINITY, l_run = 0.f;
        const bool warp_live = quad < live_quads;

        if (warp_live) {
        // ---- latent part of Q_r: global -> registers -> tensor memory.  This thread writes half of
        //      its row (16 columns = 32 elements per step); rows past the last query row are zero ----
        {
            const T* qa = reinterpret_cast<const T*>(p.q) + grow * kMlaTcDc + col0 + hf * 128;
            // two batches of eight 16-byte loads, each batch issued before its first use (one
            // memory round trip per batch instead of one per step)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    v[i] = g < R ? __ldg(reinterpret_cast<const uint4*>(qa + half * 64) + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int st = 0; st < 2; ++st) {
                    uint32_t w[16];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        w[q4 * 4] = v[st * 4 + q4].x; w[q4 * 4 + 1] = v[st * 4 + q4].y;
                        w[q4 * 4 + 2] = v[st * 4 + q4].z; w[q4 * 4 + 3] = v[st * 4 + q4].w;
                    }
                    tc::tmem_st16(tmem_q + lane_sel + hf * 64 + (half * 2 + st) * 16, w);
                }
            }
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar_q);
        }
        if (st_pending) store_rows();                // the previous item's rows (see above)

        // this thread's 32 columns of the partial scores of tile t: TMEM -> registers -> landing
        // buffer t & 1 of the peer (once the peer has consumed tile t - 2 from it)
        auto send_partial = [&](int t) {             // t: running tile number
            wait_bar(bar_s0 + (t % NSB) * 8, (t / NSB) & 1);
            tc::tc_fence_after();
            uint32_t r[32];
            tc::tmem_ld32(tmem + (t % NSB) * BN + lane_sel + hf * HC, r);
            tc::tmem_ld_wait();
            // (no data is read after this wait, so it needs no cluster-scope acquire)
            if (t >= 2) wait_bar(bar_free + (t & 1) * 8, ((t >> 1) - 1) & 1);
            const uint32_t dst = peer_sx + (t & 1) * G::kXBytes + (hf * (HC / 4) * BM + row_l) * 16;
            const uint32_t dbar = peer_bar_x + (t & 1) * 8;
#pragma unroll
            for (int q4 = 0; q4 < HC / 4; ++q4)
                tc::st_async_v4(dst + q4 * (BM * 16), r[q4 * 4], r[q4 * 4 + 1], r[q4 * 4 + 2], r[q4 * 4 + 3], dbar);
        };
        // full scores of 32 columns starting at column c0 of tile j: partial (TMEM) + the peer's
        auto full_scores = [&](int j, int c0, float (&s)[32]) {
            const int J = J0 + j;
            uint32_t r[32];
            tc::tmem_ld32(tmem + (J % NSB) * BN + lane_sel + c0, r);
            tc::tmem_ld_wait();
            const uint32_t xb = sx + (J & 1) * G::kXBytes + ((c0 / 4) * BM + row_l) * 16;
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
                uint32_t x0, x1, x2, x3;
                asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                             : "r"(xb + c4 * (BM * 16)) : "memory");
                s[c4 * 4 + 0] = __uint_as_float(r[c4 * 4 + 0]); s[c4 * 4 + 1] = __uint_as_float(r[c4 * 4 + 1]);
                s[c4 * 4 + 2] = __uint_as_float(r[c4 * 4 + 2]); s[c4 * 4 + 3] = __uint_as_float(r[c4 * 4 + 3]);
                tc::add2(s[c4 * 4 + 0], s[c4 * 4 + 1], __uint_as_float(x0), __uint_as_float(x1));
                tc::add2(s[c4 * 4 + 2], s[c4 * 4 + 3], __uint_as_float(x2), __uint_as_float(x3));
            }
            const int tok0 = t0 + j * BN + c0;
            if (tok0 + 32 > my_stop) {
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (tok0 + c >= my_stop) s[c] = -INFINITY;
            }
        };
        auto max_of = [&](const float (&s)[32]) {
            float a0 = s[0], a1 = s[1], a2 = s[2], a3 = s[3];
#pragma unroll
            for (int c = 4; c < 28; c += 8) {
                a0 = tc::max3(a0, s[c], s[c + 1]); a1 = tc::max3(a1, s[c + 2], s[c + 3]);
                a2 = tc::max3(a2, s[c + 4], s[c + 5]); a3 = tc::max3(a3, s[c + 6], s[c + 7]);
            }
            a0 = tc::max3(a0, s[28], s[29]);
            a1 = tc::max3(a1, s[30], s[31]);
            return fmaxf(tc::max3(a0, a1, a2), a3);
        };

        send_partial(J0);
        for (int j = 0; j < n_tiles; ++j) {
            const int J = J0 + j;
            // ---- full scores = mine + the peer's; the other half of the row only for the maximum ----
            wait_bar(bar_x + (J & 1) * 8, (J >> 1) & 1);
            // announce the bytes of tile j + 2 on the same barrier; they cannot land before every
            // warp here has passed the wait above, because the peer sends them only after all
            // warps have released the buffer below
            if (tid == 0 && J + 2 < pair_tiles) tc::mbar_arrive_expect_tx(bar_x + (J & 1) * 8, x_bytes);
            // this thread's half of the row; the two threads of a row swap their maxima through
            // shared memory when the two warps of the lane quadrant meet.  After that meeting both
            // have read S(j) and the landing buffer: the buffer goes back to the peer, and P(j) may
            // overwrite S(j).
            float s[32];
            full_scores(j, hf * HC, s);
            float mx = max_of(s);
            s_max[J & 1][hf][row_l] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(2 + quad) : "memory");
            mx = fmaxf(mx, s_max[J & 1][hf ^ 1][row_l]) * p.scale_log2;
            if (lane == 0) tc::mbar_arrive_remote_relaxed(peer_bar_free + (J & 1) * 8);
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
                l_run += ps0 + ps1;                  // this thread's half of the row sum
            }
            // ---- O may be rescaled once P.C(j-1) is done ----
            if (j > 0 && __any_sync(0xffffffffu, need)) {   // warp-uniform: TMEM ld/st are collective
                wait_bar(bar_empty + ((J - 1) % NS) * 8, ((J - 1) / NS) & 1);
                tc::tc_fence_after();
#pragma unroll
                for (int c0 = hf * 128; c0 < (hf + 1) * 128; c0 += 32) {
                    uint32_t o[32];
                    tc::tmem_ld32(tmem_o + lane_sel + c0, o);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                    tc::tmem_st32(tmem_o + lane_sel + c0, o);
                }
            }
            // ---- P(j) goes over the first 32 columns of S(j) ----
            tc::tmem_st16(tmem + (J % NSB) * BN + lane_sel + hf * (HC / 2), pw);
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive((J & 1) ? bar_p1 : bar_p);
            // ---- the next tile's partial scores travel while the tensor cores take P(j) ----
            if (j + 1 < n_tiles) send_partial(J + 1);
        }
        wait_bar(bar_empty + ((J0 + n_tiles - 1) % NS) * 8, ((J0 + n_tiles - 1) / NS) & 1);
        tc::tc_fence_after();

        // ---- row sum = the two halves, exchanged through shared memory by the live softmax warps
        //      (the landing buffers are not idle here: the peer may already send the next item's
        //      first tile); store ----
        s_half[hf][row_l] = l_run;
        asm volatile("bar.sync 1, %0;" ::"r"(live_warps * 32) : "memory");
        const float l_tot = l_run + s_half[hf ^ 1][row_l];
        st_final = final_out;
        st_inv = final_out ? (l_tot > 0.f ? 1.f / l_tot : 0.f) : 1.f;
        st_slot = slot;
        st_grow = grow;
        st_write = g < R && alive;
        st_m = m_run;
        st_l = l_tot;
        st_pending = true;
        }   // live warps
    }
    J0 += n_tiles;
    ++item_no;
    }   // items of a range
    }   // ranges of this pair
    if (st_pending) store_rows();                    // the last item's rows
    // ---- nobody leaves while the peer may still signal this CTA or write into it ----
    if (is_loader) cp_async_wait<0>();
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();
    tc::tc_fence_after();
    if (warp == 0) tc::tmem_dealloc(tmem, kMlaTcTmemCols);
}

}  // namespace gqa_b200

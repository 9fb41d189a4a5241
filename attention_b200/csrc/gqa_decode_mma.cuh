// Tensor-core paged GQA decode kernel for fp16 / bf16 caches, head_dim 64/128/256.
//
// Why tensor cores on a bandwidth-bound operator: every K/V byte feeds
// `group` FMAs (one per query head sharing the kv head).  At B200's HBM rate
// that is more fp32 FMA issue than the CUDA cores have left after the 16-bit to
// fp32 converts once group >= 4, so the SIMT kernel stops being bandwidth bound.
// Here the query heads of a group are the M rows (padded to 16) of
// mma.sync.m16n8k16, tokens are the N columns of Q.K^T and the K dimension of
// P.V; the issue cost per byte no longer depends on the group size.
//
// Structure: persistent CTAs pull items = (sequence, KV chunk, kv head, group of
// <= 16 query heads).  Each warp owns a private cp.async ring of NSTAGES tiles
// (TILE_N tokens of K and of V, rows gathered through the page table with
// 16-byte copies that bypass L1, zero-filled past the end) and walks the tiles
// warp, warp + NWARPS, ... of the chunk with its own fp32 online-softmax state;
// there is no CTA-wide barrier inside the token loop.  At the end of the item
// the warp states are combined in shared memory.
#pragma once

#include "gqa_common.cuh"
#include "gqa_fused.cuh"

namespace gqa_b200 {

template <typename T> struct MmaOps;

template <> struct MmaOps<__half> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
};

template <> struct MmaOps<__nv_bfloat16> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
};

// 16-byte asynchronous global->shared copy that bypasses L1; bytes beyond
// src_bytes are zero-filled.  CP_MODE selects an L2 hint: 0 none, 1 prefetch the
// 128-byte line, 2 prefetch 256 bytes, 3 = 2 plus an evict-first policy, 4 =
// evict-first only.  K/V rows are read exactly once per call, so keeping them
// out of L2's retained set leaves it to the partials, tables and queries
// (measured: 2-4 % faster calls than no hint; the prefetch sizes alone: no change).
template <int CP_MODE>
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes,
                                           uint64_t policy) {
    if (CP_MODE == 1) {
        asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;\n" ::"r"(dst),
                     "l"(src), "r"(src_bytes) : "memory");
    } else if (CP_MODE == 2) {
        asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;\n" ::"r"(dst),
                     "l"(src), "r"(src_bytes) : "memory");
    } else if (CP_MODE == 3) {
        asm volatile("cp.async.cg.shared.global.L2::cache_hint.L2::256B [%0], [%1], 16, %2, %3;\n"
                     ::"r"(dst), "l"(src), "r"(src_bytes), "l"(policy) : "memory");
    } else if (CP_MODE == 4) {
        asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n"
                     ::"r"(dst), "l"(src), "r"(src_bytes), "l"(policy) : "memory");
    } else {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
                     "r"(src_bytes) : "memory");
    }
}
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                            uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr)
                 : "memory");
}

// Compile-time geometry of one instantiation (shared with the host launcher).
template <int D, int TILE_N, int NSTAGES, int NWARPS> struct MmaGeom {
    static constexpr int kRowBytes = D * 2;
    static constexpr int kChunksPerRow = kRowBytes / 16;
    static constexpr int kTileBytes = TILE_N * kRowBytes;
    static constexpr int kStageBytes = 2 * kTileBytes;            // K tile then V tile
    static constexpr int kWarpBytes = NSTAGES * kStageBytes;
    static constexpr int kOStride = D + 8;                         // fp32 words, padded
    static constexpr int kQBytes = (D > 128) ? 16 * kRowBytes : 0; // Q staged in smem for D=256
    static constexpr int kFixedBytes = NWARPS * kWarpBytes + kQBytes + 2 * NWARPS * 16 * 4;
    static_assert(kChunksPerRow <= 32 && 32 % kChunksPerRow == 0, "row must fit a warp pass");
    static_assert(16 * kOStride * 4 <= kWarpBytes, "combine scratch must fit the warp's ring");
    // the tile fetched ahead for the next item lives in the last stage while the combine of
    // the current item uses the first bytes of the ring
    static_assert(16 * kOStride * 4 <= (NSTAGES - 1) * kStageBytes, "combine scratch overlaps the prefetch stage");
    static_assert(TILE_N % 16 == 0, "tile is a multiple of the mma K step");
};

// Lazy rescaling: the running maximum used as the exponent reference is only
// moved when a tile's maximum exceeds it by more than kRescaleSlack (log2
// units), so the O accumulators are rescaled a few times per item instead of
// once per tile.  Probabilities then lie in (0, 2^kRescaleSlack], exact in
// fp32 and well inside fp16/bf16 range; (m, l, O) stay mutually consistent, so
// the normalised result is unchanged.
constexpr float kRescaleSlack = 8.f;

template <typename T, int D, int TILE_N, int NSTAGES, int NWARPS, int MIN_CTAS, int CP_MODE = 3>
__global__ void __launch_bounds__(NWARPS * 32, MIN_CTAS)
gqa_decode_mma_kernel(const DecodeParams p) {
    using G = MmaGeom<D, TILE_N, NSTAGES, NWARPS>;
    using Ops = MmaOps<T>;
    constexpr int ROWB = G::kRowBytes;
    constexpr int CPR = G::kChunksPerRow;
    constexpr int ROWS_PER_IT = 32 / CPR;
    constexpr int LD_ITERS = TILE_N / ROWS_PER_IT;
    constexpr int SUB_ITERS = 16 / ROWS_PER_IT;   // copy passes per 16-token sub-tile
    constexpr int NB = TILE_N / 8;    // n-blocks of S
    constexpr int KS = D / 16;        // k-steps of Q.K^T
    constexpr int ND = D / 8;         // n-blocks of O
    constexpr int KK = TILE_N / 16;   // k-steps of P.V
    constexpr bool Q_IN_REGS = (D <= 128);
    constexpr int QREGS = Q_IN_REGS ? KS : 1;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* s_ring = smem_raw;                                   // [NWARPS][kWarpBytes]
    unsigned char* s_q = s_ring + NWARPS * G::kWarpBytes;               // [16][ROWB] swizzled
    float* s_m = reinterpret_cast<float*>(s_q + G::kQBytes);            // [NWARPS][16]
    float* s_l = s_m + NWARPS * 16;                                     // [NWARPS][16]
    int* s_table = reinterpret_cast<int*>(s_l + NWARPS * 16);           // [table_smem_entries]
    int* s_off = s_table + p.table_smem_entries;                         // fused mode: [batch + 1]
    __shared__ int s_item;
    __shared__ unsigned long long s_ahead;   // (sequence number of the current item << 32) | next item
    __shared__ FusedPending s_pending;
    __shared__ int s_red[2 * kNumAutoBases * 32 + 32];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = lane >> 2;            // fragment row (and row + 8)
    const int cq = (lane & 3) * 2;       // fragment column pair
    const uint32_t ring_u32 =
        (uint32_t)__cvta_generic_to_shared(s_ring + (size_t)warp * G::kWarpBytes);
    const uint32_t sq_u32 = (uint32_t)__cvta_generic_to_shared(s_q);
    const char* kc = reinterpret_cast<const char*>(p.k);
    const char* vc = reinterpret_cast<const char*>(p.v);
    const T* qp = reinterpret_cast<const T*>(p.q);
    const long long row_bytes_all = (long long)p.kv_heads * ROWB;   // one token, all kv heads
    const uint64_t policy = CP_MODE >= 3 ? evict_first_policy() : 0;
    pdl_launch_dependents();
    pdl_wait();   // the plan kernel wrote hdr / items; the call before left the counters at zero
    const bool fused = p.mode == kModeFused;
    const bool tickets = fused && p.fused_merge;   // merge inside this kernel
    const bool counted = p.mode != kModeRefSplits;      // items are pulled from the work counter
    FusedPlan plan;
    plan.base = p.chunk_base;
    plan.total_chunks = 0;
    // the first item number is asked for before the plan, so the counter's answer travels
    // while the plan is computed
    int first_item = 0;
    if (counted && tid == 0) first_item = atomicAdd(p.hdr + kHdrCounter, 1);
    int n_items;
    if (fused) {
        plan = fused_plan<NWARPS * 32>(p, s_off, s_red);
        n_items = plan.total_chunks * p.kv_heads * p.head_groups;
    } else {
        n_items = total_items(p);
    }

    // per-lane constants of the tile copy: row within a pass and 16-byte chunk
    const int ld_row = lane / CPR;
    const int ld_cc = lane % CPR;
    // per-lane constants of the ldmatrix addresses (swizzle: chunk ^ (row & 7))
    const uint32_t k_lane_off = (lane & 7) * ROWB;                    // K: token row within an n-block
    const uint32_t k_lane_x = (lane >> 3) ^ (lane & 7);               // chunk 4kp + (lane>>3)
    const uint32_t v_lane_off = (((lane >> 3) & 1) * 8 + (lane & 7)) * ROWB;   // V: token row in a k-step
    const uint32_t v_lane_x = (lane >> 4) ^ (lane & 7);               // chunk 2np + (lane>>4)
    // 16-token sub-tiles sit inside one page when the page size is a power of two >= 16
    const bool pages_hold_subtiles = p.bs_shift >= 4;

    int item;
    if (counted) {
        if (tid == 0) s_item = first_item;
        __syncthreads();
        item = s_item;
    } else {
        item = blockIdx.x;
    }
    int4 rec = make_int4(0, 0, 0, 0);
    if (!fused && item < n_items) rec = load_item_record(p, item);
    int n_pend = 0;     // one-launch mode: multi-chunk items whose tickets are still to be taken
    // Cross-item prefetch (self-planning mode): when a warp has finished its tiles of an item it
    // already requests its first tile of the CTA's NEXT item, into the ring stage the combine does
    // not use, so the data travels during the combine, the partial store and the next item's
    // set-up (measured before this: 2 - 3 us from the start of an item to its first tile, 15 -
    // 30 % of an item of a few hundred tokens).  Tile k of every item lives in stage
    // (k + NSTAGES - 1) % NSTAGES, so tile 0 is in the last stage.
    unsigned int seq = 0;          // items this CTA has started
    int pf_item = -1;              // item whose tile 0 this warp has already requested
    if (tid == 0) s_ahead = ~0ull;

    while (item < n_items) {
        int next = 0;
        if (counted) {
            if (tid == 0) next = atomicAdd(p.hdr + kHdrCounter, 1);
        } else {
            next = item + gridDim.x;
        }
        const WorkItem w = fused ? fused_item(p, item, s_off, plan.base) : item_from_record(p, item, rec);
        const int rows_valid = min(16, p.group - w.hg * 16);
        const bool nonempty = w.t1 > w.t0;

        if (nonempty) {
            // ---- Q fragments (A operand: rows = query heads, padded with zeros) ----
            uint32_t qa[QREGS][4];
            const int head0 = w.kvh * p.group + w.hg * 16;
            if (Q_IN_REGS) {
                const T* q0 = qp + ((size_t)w.b * p.q_heads + head0 + r0) * D;
                const T* q1 = q0 + (size_t)8 * D;
                const bool v0 = r0 < rows_valid, v1 = r0 + 8 < rows_valid;
#pragma unroll
                for (int ks = 0; ks < QREGS; ++ks) {
                    const int c = ks * 16 + cq;
                    qa[ks][0] = v0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c)) : 0u;
                    qa[ks][1] = v1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c)) : 0u;
                    qa[ks][2] = v0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c + 8)) : 0u;
                    qa[ks][3] = v1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c + 8)) : 0u;
                }
            } else {
                for (int i = tid; i < 16 * CPR; i += NWARPS * 32) {
                    const int row = i / CPR, cc = i % CPR;
                    uint4 val = make_uint4(0u, 0u, 0u, 0u);
                    if (row < rows_valid)
                        val = __ldg(reinterpret_cast<const uint4*>(
                            qp + ((size_t)w.b * p.q_heads + head0 + row) * D + cc * 8));
                    *reinterpret_cast<uint4*>(s_q + row * ROWB + ((cc ^ (row & 7)) << 4)) = val;
                }
            }

            float o[ND][4];
#pragma unroll
            for (int nd = 0; nd < ND; ++nd) { o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f; }
            float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

            for (int s0 = w.t0; s0 < w.t1; s0 += p.seg_tokens) {
                const int s1 = min(w.t1, s0 + p.seg_tokens);
                int first_page;
                if (s0 != w.t0) __syncthreads();   // previous segment's table no longer read
                stage_table(p, w.b, s0, s1, s_table, first_page);
                __syncthreads();

                const int n_tiles = (s1 - s0 + TILE_N - 1) / TILE_N;
                const int my_tiles = n_tiles > warp ? (n_tiles - warp + NWARPS - 1) / NWARPS : 0;
                const bool fast_segment = pages_hold_subtiles && (s0 & 15) == 0;
                const bool pf_here = pf_item == item && s0 == w.t0;   // this warp's tile 0 is on its way

                // issue the copies of this warp's k-th tile (and always commit a group)
                auto issue = [&](int k) {
                    if (k < my_tiles) {
                        const int tile_t0 = s0 + (warp + k * NWARPS) * TILE_N;
                        const uint32_t sk = ring_u32 + ((k + NSTAGES - 1) % NSTAGES) * G::kStageBytes;
                        const uint32_t sv = sk + G::kTileBytes;
                        if (k == 0 && pf_here) {
                            // requested at the end of the previous item
                        } else if (fast_segment && tile_t0 + TILE_N <= s1) {
                            // whole tile valid, each 16-token sub-tile inside one page: one
                            // table lookup per sub-tile, then a constant source stride
#pragma unroll
                            for (int sub = 0; sub < TILE_N / 16; ++sub) {
                                const int t = tile_t0 + sub * 16;
                                const long long phys = s_table[(t >> p.bs_shift) - first_page];
                                const int slot = (t & (p.block_size - 1)) + ld_row;
                                const long long off = (phys * p.block_size + slot) * row_bytes_all +
                                                      (long long)w.kvh * ROWB + ld_cc * 16;
                                const char* ks = kc + off;
                                const char* vs = vc + off;
#pragma unroll
                                for (int it = 0; it < SUB_ITERS; ++it) {
                                    const int row = sub * 16 + it * ROWS_PER_IT + ld_row;
                                    const uint32_t dst = row * ROWB + ((ld_cc ^ (row & 7)) << 4);
                                    cp_async16<CP_MODE>(sk + dst, ks, 16, policy);
                                    cp_async16<CP_MODE>(sv + dst, vs, 16, policy);
                                    ks += ROWS_PER_IT * row_bytes_all;
                                    vs += ROWS_PER_IT * row_bytes_all;
                                }
                            }
                        } else if (p.bs_shift >= 0 && tile_t0 + TILE_N <= s1) {
                            // whole tile valid, power-of-two pages of any size (or an
                            // unaligned start): one table lookup per row, no predicates
#pragma unroll 2
                            for (int it = 0; it < LD_ITERS; ++it) {
                                const int row = it * ROWS_PER_IT + ld_row;
                                const int t = tile_t0 + row;
                                const long long phys = s_table[(t >> p.bs_shift) - first_page];
                                const int slot = t & (p.block_size - 1);
                                const long long off = (phys * p.block_size + slot) * row_bytes_all +
                                                      (long long)w.kvh * ROWB + ld_cc * 16;
                                const uint32_t dst = row * ROWB + ((ld_cc ^ (row & 7)) << 4);
                                cp_async16<CP_MODE>(sk + dst, kc + off, 16, policy);
                                cp_async16<CP_MODE>(sv + dst, vc + off, 16, policy);
                            }
                        } else {
#pragma unroll 1
                            for (int it = 0; it < LD_ITERS; ++it) {
                                const int row = it * ROWS_PER_IT + ld_row;
                                const int t = tile_t0 + row;
                                const bool valid = t < s1;
                                long long off = 0;
                                if (valid) {
                                    int pg, slot;
                                    token_page_slot(p, t, pg, slot);
                                    const long long phys = s_table[pg - first_page];
                                    off = (phys * p.block_size + slot) * row_bytes_all +
                                          (long long)w.kvh * ROWB + ld_cc * 16;
                                }
                                const uint32_t dst = row * ROWB + ((ld_cc ^ (row & 7)) << 4);
                                cp_async16<CP_MODE>(sk + dst, kc + off, valid ? 16 : 0, policy);
                                cp_async16<CP_MODE>(sv + dst, vc + off, valid ? 16 : 0, policy);
                            }
                        }
                    }
                    cp_async_commit();
                };

#pragma unroll
                for (int k = 0; k < NSTAGES - 1; ++k) issue(k);

                for (int k = 0; k < my_tiles; ++k) {
                    cp_async_wait<NSTAGES - 2>();   // this lane's copies of tile k have landed
                    __syncwarp();                   // ... and every lane's; tile k-1 fully consumed
                    // (by now the work counter has answered: every warp may learn the next item)
                    if (counted && tid == 0 && k == 0 && s0 == w.t0)
                        *reinterpret_cast<volatile unsigned long long*>(&s_ahead) =
                            ((unsigned long long)seq << 32) | (unsigned int)next;
                    issue(k + NSTAGES - 1);         // refill the stage tile k-1 used

                    const int tile_t0 = s0 + (warp + k * NWARPS) * TILE_N;
                    const uint32_t sk = ring_u32 + ((k + NSTAGES - 1) % NSTAGES) * G::kStageBytes;
                    const uint32_t sv = sk + G::kTileBytes;

                    // ---- S = Q K^T : [16 heads] x [TILE_N tokens] ----
                    float s[NB][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
                    for (int kp = 0; kp < KS / 2; ++kp) {
                        uint32_t a0[4], a1[4];
                        if (Q_IN_REGS) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                a0[i] = qa[Q_IN_REGS ? 2 * kp : 0][i];
                                a1[i] = qa[Q_IN_REGS ? 2 * kp + 1 : 0][i];
                            }
                        } else {
                            const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
                            const int cc0 = 4 * kp + (lane >> 4);
                            ldmatrix_x4(sq_u32 + row * ROWB + ((cc0 ^ (row & 7)) << 4), a0[0], a0[1],
                                        a0[2], a0[3]);
                            ldmatrix_x4(sq_u32 + row * ROWB + (((cc0 + 2) ^ (row & 7)) << 4), a1[0],
                                        a1[1], a1[2], a1[3]);
                        }
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            // matrices: (tokens nb*8..+7) x 16-byte chunks 4kp .. 4kp+3
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4(sk + nb * 8 * ROWB + k_lane_off + ((k_lane_x ^ (4 * kp)) << 4),
                                        b0, b1, b2, b3);
                            Ops::mma(s[nb], a0, b0, b1);
                            Ops::mma(s[nb], a1, b2, b3);
                        }
                    }

                    // ---- mask the tail, online softmax in fp32 (log2 units) ----
                    if (tile_t0 + TILE_N > s1) {
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const int t = tile_t0 + nb * 8 + cq;
                            if (t >= s1) { s[nb][0] = -INFINITY; s[nb][2] = -INFINITY; }
                            if (t + 1 >= s1) { s[nb][1] = -INFINITY; s[nb][3] = -INFINITY; }
                        }
                    }
                    float mx0 = fmaxf(s[0][0], s[0][1]), mx1 = fmaxf(s[0][2], s[0][3]);
#pragma unroll
                    for (int nb = 1; nb < NB; ++nb) {
                        mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
                        mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
                    }
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                    // the first token of a tile is always valid, so the tile maxima are finite
                    mx0 *= p.scale_log2;
                    mx1 *= p.scale_log2;
                    if (__any_sync(0xffffffffu, mx0 > m0 + kRescaleSlack || mx1 > m1 + kRescaleSlack)) {
                        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                        const float alpha0 = fast_exp2(m0 - mn0), alpha1 = fast_exp2(m1 - mn1);
                        m0 = mn0;
                        m1 = mn1;
                        l0 *= alpha0;
                        l1 *= alpha1;
#pragma unroll
                        for (int nd = 0; nd < ND; ++nd) {
                            o[nd][0] *= alpha0; o[nd][1] *= alpha0;
                            o[nd][2] *= alpha1; o[nd][3] *= alpha1;
                        }
                    }
                    uint32_t pa[KK][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const float p0 = fast_exp2(fmaf(s[nb][0], p.scale_log2, -m0));
                        const float p1 = fast_exp2(fmaf(s[nb][1], p.scale_log2, -m0));
                        const float p2 = fast_exp2(fmaf(s[nb][2], p.scale_log2, -m1));
                        const float p3 = fast_exp2(fmaf(s[nb][3], p.scale_log2, -m1));
                        l0 += p0 + p1;
                        l1 += p2 + p3;
                        pa[nb >> 1][(nb & 1) * 2 + 0] = Ops::pack(p0, p1);
                        pa[nb >> 1][(nb & 1) * 2 + 1] = Ops::pack(p2, p3);
                    }

                    // ---- O += P V : [16 heads] x [D] ----
#pragma unroll
                    for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
                        for (int np = 0; np < ND / 2; ++np) {
                            // matrices: tokens kk*16 + {0..7, 8..15} x chunks 2np, 2np+1
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4_trans(sv + kk * 16 * ROWB + v_lane_off +
                                                  ((v_lane_x ^ (2 * np)) << 4),
                                              b0, b1, b2, b3);
                            Ops::mma(o[2 * np], pa[kk], b0, b1);
                            Ops::mma(o[2 * np + 1], pa[kk], b2, b3);
                        }
                    }
                }
                cp_async_wait<0>();
            }

            // ---- this warp's first tile of the CTA's next item (see pf_item above) ----
            // (not in the one-launch mode: its merges stage partials through the whole ring)
            if (fused && !tickets && pages_hold_subtiles) {
                const unsigned long long ahead = *reinterpret_cast<volatile unsigned long long*>(&s_ahead);
                const int cand = (int)(unsigned int)ahead;
                if ((unsigned int)(ahead >> 32) == seq && cand < n_items) {
                    const WorkItem wn = fused_item(p, cand, s_off, plan.base);
                    const int tile_t0 = wn.t0 + warp * TILE_N;
                    if ((wn.t0 & 15) == 0 && wn.t1 - wn.t0 <= p.seg_tokens && tile_t0 + TILE_N <= wn.t1) {
                        const uint32_t sk = ring_u32 + (NSTAGES - 1) * G::kStageBytes;
                        const uint32_t sv = sk + G::kTileBytes;
                        const int32_t* trow = p.table + (long long)wn.b * p.max_pages;
                        const int last_block = (int)(p.num_blocks - 1);
#pragma unroll
                        for (int sub = 0; sub < TILE_N / 16; ++sub) {
                            const int t = tile_t0 + sub * 16;
                            int pg = __ldg(trow + (t >> p.bs_shift));
                            pg = pg < 0 ? 0 : (pg > last_block ? last_block : pg);   // as stage_table
                            const int slot = (t & (p.block_size - 1)) + ld_row;
                            const long long off = ((long long)pg * p.block_size + slot) * row_bytes_all +
                                                  (long long)wn.kvh * ROWB + ld_cc * 16;
                            const char* ks = kc + off;
                            const char* vs = vc + off;
#pragma unroll
                            for (int it = 0; it < SUB_ITERS; ++it) {
                                const int row = sub * 16 + it * ROWS_PER_IT + ld_row;
                                const uint32_t dst = row * ROWB + ((ld_cc ^ (row & 7)) << 4);
                                cp_async16<CP_MODE>(sk + dst, ks, 16, policy);
                                cp_async16<CP_MODE>(sv + dst, vs, 16, policy);
                                ks += ROWS_PER_IT * row_bytes_all;
                                vs += ROWS_PER_IT * row_bytes_all;
                            }
                        }
                        cp_async_commit();
                        pf_item = cand;
                    }
                }
            }

            // ---- publish this warp's state ----
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            __syncwarp();
            float* s_o = reinterpret_cast<float*>(s_ring + (size_t)warp * G::kWarpBytes);
#pragma unroll
            for (int nd = 0; nd < ND; ++nd) {
                *reinterpret_cast<float2*>(s_o + r0 * G::kOStride + nd * 8 + cq) =
                    make_float2(o[nd][0], o[nd][1]);
                *reinterpret_cast<float2*>(s_o + (r0 + 8) * G::kOStride + nd * 8 + cq) =
                    make_float2(o[nd][2], o[nd][3]);
            }
            if ((lane & 3) == 0) {
                s_m[warp * 16 + r0] = m0;
                s_m[warp * 16 + r0 + 8] = m1;
                s_l[warp * 16 + r0] = l0;
                s_l[warp * 16 + r0 + 8] = l1;
            }
        }
        if (tid == 0) s_item = next;
        __syncthreads();
        // fetch the next item's record now; its latency hides behind the combine
        const int nxt = s_item;
        int4 rec_next = make_int4(0, 0, 0, 0);
        if (!fused && nxt < n_items) rec_next = load_item_record(p, nxt);
        if (nonempty) {
            combine_and_store<T, NWARPS, true>(p, w, reinterpret_cast<const float*>(s_ring),
                                               G::kWarpBytes / 4, G::kOStride, s_m, s_l, 16,
                                               rows_valid);
        } else {
            store_empty<T>(p, w, rows_valid);
        }
        __syncthreads();   // rings, Q tile, table and s_item are free again
        if (tickets && nonempty && w.n_parts > 1) {
            if (tid == 0) fused_note_item(s_pending, n_pend, p, w);
            if (++n_pend == kFusedMaxPending) {
                fused_flush_tickets<T, true, true>(p, s_pending, n_pend, s_ring, NWARPS * G::kWarpBytes);
                n_pend = 0;
            }
        }
        item = nxt;
        rec = rec_next;
        ++seq;
    }
    if (tickets) fused_flush_tickets<T, true, true>(p, s_pending, n_pend, s_ring, NWARPS * G::kWarpBytes);
    if (counted) decode_counters_release(p);
}

}  // namespace gqa_b200

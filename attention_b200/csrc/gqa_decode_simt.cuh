// SIMT paged GQA decode kernel: warp-level dot products with shuffle
// reductions and an fp32 online (max, sum) softmax.  Handles every dtype, every
// head_dim in [1, 256], every block size and every group size; it is the only
// kernel for float32 tensors and for shapes the tensor-core kernel rejects.
//
// One CTA works on one item = (sequence, KV chunk, kv head, group of up to GB
// query heads).  Its warps take interleaved runs of TOK tokens; every K/V row a
// warp loads is used for all GB query heads held in registers, so a row is read
// once per item.  Per-warp states are combined in shared memory at the end of
// the item.
#pragma once

#include "gqa_common.cuh"
#include "gqa_fused.cuh"

namespace gqa_b200 {

constexpr int kSimtWarps = 4;
constexpr int kSimtTok = 4;   // tokens per warp iteration (independent row loads in flight)

// Load the EPL elements of one row that belong to this lane, as fp32.
//   CONTIG: head_dim == 32 * EPL, the lane owns elements [lane*EPL, lane*EPL+EPL)
//           and the row is (EPL * sizeof(T))-byte aligned -> one vector load.
//   else  : the lane owns elements lane, lane+32, ... (< head_dim), scalar loads.
template <typename T, int EPL, bool CONTIG>
__device__ __forceinline__ void load_row(const T* row, int lane, int D, float (&x)[EPL]) {
    if (CONTIG) {
        constexpr int BYTES = EPL * (int)sizeof(T);
        const char* src = reinterpret_cast<const char*>(row + lane * EPL);
        T tmp[EPL];
        if (BYTES == 32) {
            reinterpret_cast<uint4*>(tmp)[0] = __ldg(reinterpret_cast<const uint4*>(src));
            reinterpret_cast<uint4*>(tmp)[1] = __ldg(reinterpret_cast<const uint4*>(src) + 1);
        } else if (BYTES == 16) {
            reinterpret_cast<uint4*>(tmp)[0] = __ldg(reinterpret_cast<const uint4*>(src));
        } else if (BYTES == 8) {
            reinterpret_cast<uint2*>(tmp)[0] = __ldg(reinterpret_cast<const uint2*>(src));
        } else if (BYTES == 4) {
            reinterpret_cast<uint32_t*>(tmp)[0] = __ldg(reinterpret_cast<const uint32_t*>(src));
        } else {
            reinterpret_cast<uint16_t*>(tmp)[0] = __ldg(reinterpret_cast<const uint16_t*>(src));
        }
#pragma unroll
        for (int j = 0; j < EPL; ++j) x[j] = to_f32<T>(tmp[j]);
    } else {
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = lane + 32 * j;
            x[j] = e < D ? to_f32<T>(row[e]) : 0.f;
        }
    }
}

template <typename T, int EPL, bool CONTIG, int GB>
__global__ void __launch_bounds__(kSimtWarps * 32)
gqa_decode_simt_kernel(const DecodeParams p) {
    constexpr int NW = kSimtWarps;
    constexpr int TOK = kSimtTok;
    constexpr bool VEC4 = CONTIG;   // head_dim is then a multiple of 32 and rows are aligned
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int D = p.head_dim;
    const int o_stride = ((D + 3) & ~3) + 4;
    float* s_o = reinterpret_cast<float*>(smem_raw);            // [NW][GB][o_stride]
    float* s_m = s_o + NW * GB * o_stride;                       // [NW][GB]
    float* s_l = s_m + NW * GB;                                  // [NW][GB]
    int* s_table = reinterpret_cast<int*>(s_l + NW * GB);        // [table_smem_entries]
    int* s_off = s_table + p.table_smem_entries;                 // fused mode: [batch + 1]
    __shared__ int s_item;
    __shared__ FusedPending s_pending;
    __shared__ int s_red[2 * kNumAutoBases * 32 + 32];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* kc = reinterpret_cast<const T*>(p.k);
    const T* vc = reinterpret_cast<const T*>(p.v);
    const T* qp = reinterpret_cast<const T*>(p.q);
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
        plan = fused_plan<NW * 32>(p, s_off, s_red);
        n_items = plan.total_chunks * p.kv_heads * p.head_groups;
    } else {
        n_items = total_items(p);
    }
    const long long row_elems = (long long)p.kv_heads * D;

    int n_pend = 0;     // one-launch mode: multi-chunk items whose tickets are still to be taken
    int item;
    if (counted) {
        if (tid == 0) s_item = first_item;
        __syncthreads();
        item = s_item;
    } else {
        item = blockIdx.x;
    }
    while (item < n_items) {
        int next = 0;
        if (counted) {
            if (tid == 0) next = atomicAdd(p.hdr + kHdrCounter, 1);
        } else {
            next = item + gridDim.x;
        }
        const WorkItem w = fused ? fused_item(p, item, s_off, plan.base) : decode_item(p, item);
        const int rows_valid = min(GB, p.group - w.hg * GB);

        if (w.t1 <= w.t0) {
            store_empty<T>(p, w, rows_valid);
        } else {
            // query rows of this item, fp32, this lane's elements
            float qf[GB][EPL];
#pragma unroll
            for (int g = 0; g < GB; ++g) {
                if (g < rows_valid) {
                    const T* qrow = qp + ((size_t)w.b * p.q_heads + w.kvh * p.group + w.hg * GB + g) * D;
                    load_row<T, EPL, CONTIG>(qrow, lane, D, qf[g]);
                } else {
#pragma unroll
                    for (int j = 0; j < EPL; ++j) qf[g][j] = 0.f;
                }
            }
            float m[GB], l[GB], acc[GB][EPL];
#pragma unroll
            for (int g = 0; g < GB; ++g) {
                m[g] = -INFINITY;
                l[g] = 0.f;
#pragma unroll
                for (int j = 0; j < EPL; ++j) acc[g][j] = 0.f;
            }

            for (int s0 = w.t0; s0 < w.t1; s0 += p.seg_tokens) {
                const int s1 = min(w.t1, s0 + p.seg_tokens);
                int first_page;
                __syncthreads();   // previous segment's table no longer in use
                stage_table(p, w.b, s0, s1, s_table, first_page);
                __syncthreads();
                auto load_tokens = [&](int tb, float (&kx)[TOK][EPL], float (&vx)[TOK][EPL], bool (&valid)[TOK]) {
#pragma unroll
                    for (int tk = 0; tk < TOK; ++tk) {
                        const int t = tb + tk;
                        valid[tk] = t < s1;
                        if (valid[tk]) {
                            int pg, slot;
                            token_page_slot(p, t, pg, slot);
                            const long long phys = s_table[pg - first_page];
                            const long long off = (phys * p.block_size + slot) * row_elems +
                                                  (long long)w.kvh * D;
                            load_row<T, EPL, CONTIG>(kc + off, lane, D, kx[tk]);
                            load_row<T, EPL, CONTIG>(vc + off, lane, D, vx[tk]);
                        } else {
#pragma unroll
                            for (int j = 0; j < EPL; ++j) { kx[tk][j] = 0.f; vx[tk][j] = 0.f; }
                        }
                    }
                };
                // (requesting the next TOK rows ahead of use, a register double buffer, was tried for
                // the few-iteration items of small batches: no gain there, and its registers cost a
                // resident CTA per SM on large ones: 779 against 620 us on batch 64 x 1-4 k tokens)
                for (int tb = s0 + warp * TOK; tb < s1; tb += NW * TOK) {
                    float kx[TOK][EPL], vx[TOK][EPL];
                    bool valid[TOK];
                    load_tokens(tb, kx, vx, valid);
#pragma unroll
                    for (int g = 0; g < GB; ++g) {
                        if (g >= rows_valid) continue;
                        float s[TOK];
#pragma unroll
                        for (int tk = 0; tk < TOK; ++tk) {
                            float d = 0.f;
#pragma unroll
                            for (int j = 0; j < EPL; ++j) d = fmaf(qf[g][j], kx[tk][j], d);
#pragma unroll
                            for (int sh = 16; sh >= 1; sh >>= 1)
                                d += __shfl_xor_sync(0xffffffffu, d, sh);
                            s[tk] = valid[tk] ? d * p.scale_log2 : -INFINITY;
                        }
                        float mt = s[0];
#pragma unroll
                        for (int tk = 1; tk < TOK; ++tk) mt = fmaxf(mt, s[tk]);
                        const float m_new = fmaxf(m[g], mt);   // finite: token tb is valid
                        const float alpha = fast_exp2(m[g] - m_new);
                        float pw[TOK], psum = 0.f;
#pragma unroll
                        for (int tk = 0; tk < TOK; ++tk) {
                            pw[tk] = fast_exp2(s[tk] - m_new);
                            psum += pw[tk];
                        }
                        l[g] = l[g] * alpha + psum;
                        m[g] = m_new;
#pragma unroll
                        for (int j = 0; j < EPL; ++j) {
                            float a = acc[g][j] * alpha;
#pragma unroll
                            for (int tk = 0; tk < TOK; ++tk) a = fmaf(pw[tk], vx[tk][j], a);
                            acc[g][j] = a;
                        }
                    }
                }
            }
            // publish this warp's state
#pragma unroll
            for (int g = 0; g < GB; ++g) {
                float* dst = s_o + ((size_t)warp * GB + g) * o_stride;
#pragma unroll
                for (int j = 0; j < EPL; ++j) {
                    const int e = CONTIG ? lane * EPL + j : lane + 32 * j;
                    if (e < D) dst[e] = acc[g][j];
                }
                if (lane == 0) { s_m[warp * GB + g] = m[g]; s_l[warp * GB + g] = l[g]; }
            }
            __syncthreads();
            combine_and_store<T, NW, VEC4>(p, w, s_o, GB * o_stride, o_stride, s_m, s_l, GB,
                                           rows_valid);
        }
        __syncthreads();
        if (tickets && w.t1 > w.t0 && w.n_parts > 1) {
            if (tid == 0) fused_note_item(s_pending, n_pend, p, w);
            if (++n_pend == kFusedMaxPending) {
                fused_flush_tickets<T, VEC4, false>(p, s_pending, n_pend, nullptr, 0);
                n_pend = 0;
            }
        }
        if (counted) {
            if (tid == 0) s_item = next;
            __syncthreads();
            item = s_item;
        } else {
            item = next;
        }
    }
    if (tickets) fused_flush_tickets<T, VEC4, false>(p, s_pending, n_pend, nullptr, 0);
    if (counted) decode_counters_release(p);
}

}  // namespace gqa_b200

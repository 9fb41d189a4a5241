// SIMT kernels of the paged latent-attention (MLA) decode path: the general
// attention kernel (any widths, any element type, dense or index-selected), the
// split merge, the per-head projections and the cache writer.
#pragma once

#include "gqa_common.cuh"

namespace gqa_b200 {

struct MlaParams {
    const void* q;             // absorbed queries [rows, heads, dc], rows = batch * tq
    const void* qr;            // rotated queries  [rows, heads, dr]
    const void* cache;         // [num_blocks, page, dc + dr]
    const int32_t* table;      // [batch, max_pages]
    const int32_t* lens;       // [batch]
    const int32_t* pos;        // [batch, tq]
    const int32_t* indices;    // [batch, tq, nk] or nullptr
    void* out;                 // [rows, heads, dc]
    float* part_ml;            // [rows * heads][splits][2]   (max in log2 units, sum)
    float* part_acc;           // [rows * heads][splits][dc]  unnormalised
    long long num_blocks;
    int batch, tq, heads, dc, dr, page, max_pages, nk, splits, causal;
    int* tc_sched;             // tensor-core kernel: [0] total tiles, [1] tiles per range, [2] ranges,
                               //   [4 ...] prefix[u] = tiles before unit u (units + 1 entries)
    int tc_units;              // units = batch * tc_row_tiles; a unit = 128 query rows of one sequence
    int tc_row_tiles;          // ceil(tq * heads / 128)
    int tc_force_range;        // > 0: tiles per range (else total / pairs)
    int tc_live_quads;         // 32-row groups of a unit that hold query rows in every unit (1..4)
    int page_shift;            // log2(page) when page is a power of two, else -1
    float scale_log2;          // scale * log2(e)
};

// Tokens a query row may attend to: [0, end).
__device__ __forceinline__ int mla_row_end(const MlaParams& p, int b, int t) {
    const int len = max(0, __ldg(p.lens + b));
    if (!p.causal) return len;
    return min(len, max(0, __ldg(p.pos + (long long)b * p.tq + t) + 1));
}

constexpr int kMlaSimtWarps = 4;
constexpr int kMlaSimtHeads = 4;      // heads per CTA

// One CTA = (query row, head group of HB heads, split).  Each warp walks every
// NW-th token of the split's range; lane l holds columns l, l+32, ... of the row.
// DCN = ceil(dc / 32) columns of the latent part stay in registers for the
// weighted sum.  Shared memory: the HB scaled query rows in fp32, then (after
// the loop) every warp's running state for the in-CTA combine.
template <typename T, int DCN>
__global__ void __launch_bounds__(kMlaSimtWarps * 32)
mla_attend_simt_kernel(const MlaParams p) {
    constexpr int NW = kMlaSimtWarps, HB = kMlaSimtHeads;
    extern __shared__ __align__(16) float s_mem[];
    const int width = p.dc + p.dr;
    float* s_q = s_mem;                               // [HB][width]
    float* s_acc = s_mem + HB * width;                // [NW][HB][dc]
    __shared__ float s_m[NW][HB], s_l[NW][HB];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = blockIdx.x;                       // b * tq + t
    const int h0 = blockIdx.y * HB;
    const int part = blockIdx.z;
    const int b = row / p.tq, t = row - b * p.tq;
    const int nh = min(HB, p.heads - h0);
    const T* qp = reinterpret_cast<const T*>(p.q);
    const T* qrp = reinterpret_cast<const T*>(p.qr);
    const T* cp = reinterpret_cast<const T*>(p.cache);

    pdl_launch_dependents();
    pdl_wait();

    for (int i = tid; i < HB * width; i += NW * 32) {
        const int hh = i / width, d = i - hh * width;
        float x = 0.f;
        if (hh < nh) {
            const long long rh = (long long)row * p.heads + h0 + hh;
            x = d < p.dc ? to_f32(qp[rh * p.dc + d]) : to_f32(qrp[rh * p.dr + d - p.dc]);
        }
        s_q[i] = x * p.scale_log2;
    }
    __syncthreads();

    const int end = mla_row_end(p, b, t);
    const int count = p.indices ? p.nk : end;
    const int begin = (int)((long long)count * part / p.splits);
    const int stop = (int)((long long)count * (part + 1) / p.splits);
    const int32_t* sel = p.indices ? p.indices + (long long)row * p.nk : nullptr;
    const int32_t* trow = p.table + (long long)b * p.max_pages;
    const int last_block = (int)(p.num_blocks - 1);

    float m[HB], l[HB], acc[HB][DCN];
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) {
        m[hh] = -INFINITY;
        l[hh] = 0.f;
#pragma unroll
        for (int k = 0; k < DCN; ++k) acc[hh][k] = 0.f;
    }

    for (int i = begin + warp; i < stop; i += NW) {
        const int s = sel ? __ldg(sel + i) : i;
        if (s < 0 || s >= end) continue;              // warp-uniform
        const int pg = s / p.page;
        // a page id outside the pool (a caller error) is clamped instead of faulting
        const int phys = min(max(__ldg(trow + pg), 0), last_block);
        const T* r = cp + ((long long)phys * p.page + (s - pg * p.page)) * width;
        float v[DCN], dot[HB];
#pragma unroll
        for (int hh = 0; hh < HB; ++hh) dot[hh] = 0.f;
#pragma unroll
        for (int k = 0; k < DCN; ++k) {
            const int d = lane + 32 * k;
            v[k] = d < p.dc ? to_f32(r[d]) : 0.f;
            if (d < p.dc) {
#pragma unroll
                for (int hh = 0; hh < HB; ++hh) dot[hh] += s_q[hh * width + d] * v[k];
            }
        }
        for (int d = p.dc + lane; d < width; d += 32) {
            const float x = to_f32(r[d]);
#pragma unroll
            for (int hh = 0; hh < HB; ++hh) dot[hh] += s_q[hh * width + d] * x;
        }
#pragma unroll
        for (int hh = 0; hh < HB; ++hh) {
            float sc = dot[hh];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
            const float mn = fmaxf(m[hh], sc);
            const float a = m[hh] == -INFINITY ? 0.f : fast_exp2(m[hh] - mn);
            const float w = fast_exp2(sc - mn);
            m[hh] = mn;
            l[hh] = l[hh] * a + w;
#pragma unroll
            for (int k = 0; k < DCN; ++k) acc[hh][k] = acc[hh][k] * a + w * v[k];
        }
    }

    // ---- combine the NW warps of this CTA (fixed order: deterministic) ----
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) {
        if (lane == 0) { s_m[warp][hh] = m[hh]; s_l[warp][hh] = l[hh]; }
#pragma unroll
        for (int k = 0; k < DCN; ++k) {
            const int d = lane + 32 * k;
            if (d < p.dc) s_acc[((size_t)warp * HB + hh) * p.dc + d] = acc[hh][k];
        }
    }
    __syncthreads();
    T* op = reinterpret_cast<T*>(p.out);
    for (int i = tid; i < nh * p.dc; i += NW * 32) {
        const int hh = i / p.dc, d = i - hh * p.dc;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) mx = fmaxf(mx, s_m[w][hh]);
        float sum = 0.f, a = 0.f;
        if (mx != -INFINITY) {
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float wgt = s_m[w][hh] == -INFINITY ? 0.f : fast_exp2(s_m[w][hh] - mx);
                sum += wgt * s_l[w][hh];
                a += wgt * s_acc[((size_t)w * HB + hh) * p.dc + d];
            }
        }
        const long long rh = (long long)row * p.heads + h0 + hh;
        if (p.splits == 1) {
            op[rh * p.dc + d] = from_f32<T>(sum > 0.f ? a / sum : 0.f);
        } else {
            const long long slot = rh * p.splits + part;
            p.part_acc[slot * p.dc + d] = a;
            if (d == 0) { p.part_ml[slot * 2] = mx; p.part_ml[slot * 2 + 1] = sum; }
        }
    }
}

// One warp per (row, head): fold the splits against their global maximum.  Lanes read the
// partial sums as float4 (dc a multiple of 4) or scalars; the order of the sum over splits is
// fixed, so the result does not depend on the launch shape.
constexpr int kMlaMergeWarps = 4;
template <typename T>
__global__ void __launch_bounds__(kMlaMergeWarps * 32)
mla_merge_kernel(const MlaParams p, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long rh = (long long)blockIdx.x * kMlaMergeWarps + (threadIdx.x >> 5);
    if (rh >= total) return;
    const float* ml = p.part_ml + rh * p.splits * 2;
    float mx = -INFINITY;
    for (int s = 0; s < p.splits; ++s)
        if (ml[2 * s + 1] > 0.f) mx = fmaxf(mx, ml[2 * s]);
    float sum = 0.f;
    for (int s = 0; s < p.splits; ++s)
        if (ml[2 * s + 1] > 0.f) sum += fast_exp2(ml[2 * s] - mx) * ml[2 * s + 1];
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    T* op = reinterpret_cast<T*>(p.out) + rh * p.dc;
    const float* acc = p.part_acc + rh * p.splits * p.dc;
    if ((p.dc & 3) == 0) {
        for (int d = lane * 4; d < p.dc; d += 128) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < p.splits; ++s) {
                if (ml[2 * s + 1] > 0.f) {
                    const float w = fast_exp2(ml[2 * s] - mx);
                    const float4 x = *reinterpret_cast<const float4*>(acc + (long long)s * p.dc + d);
                    a.x += w * x.x; a.y += w * x.y; a.z += w * x.z; a.w += w * x.w;
                }
            }
            op[d] = from_f32<T>(a.x * inv); op[d + 1] = from_f32<T>(a.y * inv);
            op[d + 2] = from_f32<T>(a.z * inv); op[d + 3] = from_f32<T>(a.w * inv);
        }
    } else {
        for (int d = lane; d < p.dc; d += 32) {
            float a = 0.f;
            for (int s = 0; s < p.splits; ++s)
                if (ml[2 * s + 1] > 0.f) a += fast_exp2(ml[2 * s] - mx) * acc[(long long)s * p.dc + d];
            op[d] = from_f32<T>(a * inv);
        }
    }
}

// ---------------------------------------------------------------------------
// per-head projections
// ---------------------------------------------------------------------------
constexpr int kProjRows = 16;         // rows of x per CTA
constexpr int kProjThreads = 128;

// x rows of one head into shared memory as [d_in][kProjRows] fp32 (rows innermost, so that a
// thread reads all rows of one contraction index with four 16-byte loads)
template <typename T>
__device__ __forceinline__ void proj_stage_x(float* s_x, const T* __restrict__ x, long long r0, int nr, int heads,
                                             int h, int d_in) {
    for (int i = threadIdx.x; i < kProjRows * d_in; i += kProjThreads) {
        const int rr = i / d_in, j = i - rr * d_in;       // coalesced along j
        s_x[j * kProjRows + rr] = rr < nr ? to_f32(x[((r0 + rr) * heads + h) * d_in + j]) : 0.f;
    }
}
__device__ __forceinline__ void proj_fma_rows(float (&acc)[kProjRows], const float* s_xj, float wv) {
#pragma unroll
    for (int q = 0; q < kProjRows / 4; ++q) {
        const float4 xv = *reinterpret_cast<const float4*>(s_xj + q * 4);
        acc[q * 4 + 0] += xv.x * wv; acc[q * 4 + 1] += xv.y * wv;
        acc[q * 4 + 2] += xv.z * wv; acc[q * 4 + 3] += xv.w * wv;
    }
}

// out[r, h, c] = sum_j x[r, h, j] * w[h, j, c]: one thread per output column,
// weights read coalesced along c.  grid (row chunks, column tiles, heads).
template <typename T>
__global__ void __launch_bounds__(kProjThreads)
mla_absorb_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out,
                  long long rows, int heads, int d_in, int d_out) {
    extern __shared__ __align__(16) float s_x[];      // [d_in][kProjRows]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z;
    const long long r0 = (long long)blockIdx.x * kProjRows;
    const int nr = (int)min((long long)kProjRows, rows - r0);
    proj_stage_x(s_x, x, r0, nr, heads, h, d_in);
    __syncthreads();
    const int c = blockIdx.y * kProjThreads + threadIdx.x;
    if (c >= d_out) return;
    float acc[kProjRows];
#pragma unroll
    for (int rr = 0; rr < kProjRows; ++rr) acc[rr] = 0.f;
    const T* wp = w + (long long)h * d_in * d_out + c;
#pragma unroll 4
    for (int j = 0; j < d_in; ++j) proj_fma_rows(acc, s_x + j * kProjRows, to_f32(wp[(long long)j * d_out]));
#pragma unroll
    for (int rr = 0; rr < kProjRows; ++rr)
        if (rr < nr) out[((r0 + rr) * heads + h) * d_out + c] = from_f32<T>(acc[rr]);
}

// out[r, h, v] = sum_c x[r, h, c] * w[h, v, c]: one thread per output column v; it walks its
// weight row with 16-byte loads (the other half of each 32-byte sector is the same thread's
// next load) and reads x as shared-memory broadcasts.  No reductions across threads.
template <typename T>
__global__ void __launch_bounds__(kProjThreads)
mla_value_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out,
                 long long rows, int heads, int d_in, int d_out) {
    extern __shared__ __align__(16) float s_x[];      // [d_in][kProjRows]
    pdl_launch_dependents();
    pdl_wait();
    constexpr int VEC = 16 / (int)sizeof(T);          // elements per 16-byte load
    const int h = blockIdx.z;
    const long long r0 = (long long)blockIdx.x * kProjRows;
    const int nr = (int)min((long long)kProjRows, rows - r0);
    proj_stage_x(s_x, x, r0, nr, heads, h, d_in);
    __syncthreads();
    const int v = blockIdx.y * kProjThreads + threadIdx.x;
    if (v >= d_out) return;
    float acc[kProjRows];
#pragma unroll
    for (int rr = 0; rr < kProjRows; ++rr) acc[rr] = 0.f;
    const T* wp = w + ((long long)h * d_out + v) * d_in;
    int c = 0;
    if ((d_in % VEC) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        for (; c < d_in; c += VEC) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(wp + c));
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) proj_fma_rows(acc, s_x + (c + i) * kProjRows, to_f32(e[i]));
        }
    }
    for (; c < d_in; ++c) proj_fma_rows(acc, s_x + c * kProjRows, to_f32(wp[c]));
#pragma unroll
    for (int rr = 0; rr < kProjRows; ++rr)
        if (rr < nr) out[((r0 + rr) * heads + h) * d_out + v] = from_f32<T>(acc[rr]);
}

// Row slots[i] of the cache (viewed as [rows, dc + dr]) = latent[i] ++ rope[i].
template <typename T>
__global__ void __launch_bounds__(128)
mla_cache_write_kernel(const T* __restrict__ latent, const T* __restrict__ rope, T* __restrict__ cache,
                       const int64_t* __restrict__ slots, int dc, int dr) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = blockIdx.x;
    T* dst = cache + slots[i] * (long long)(dc + dr);
    for (int d = threadIdx.x; d < dc + dr; d += blockDim.x)
        dst[d] = d < dc ? latent[i * dc + d] : rope[i * dr + d - dc];
}

}  // namespace gqa_b200

// Per-head MLA projections on the tensor cores (mma.sync m16n8k16, fp16 / bf16): the two
// small batched GEMMs either side of the latent attention,
//   absorb : out[r, h, c] = sum_j x[r, h, j] * w[h, j, c]     (W_uk, [heads, d_in, d_out])
//   value  : out[r, h, v] = sum_c x[r, h, c] * w[h, v, c]     (W_uv, [heads, d_out, d_in])
// One CTA = one head x 64 rows x 64 output columns; x and the weight tile are staged once in
// shared memory (16-byte cp.async, 16-byte chunks XOR-swizzled by the row) and read with
// ldmatrix: the weight tile as it lies in memory, transposed by ldmatrix.trans for W_uk.
// These GEMMs are tiny (1 GFLOP at 64 rows x 128 heads) and weight-bandwidth bound, so the
// legacy tensor path is enough; d_in and d_out must be multiples of 64.
#pragma once

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"

namespace gqa_b200 {

constexpr int kProjMmaRows = 64;
constexpr int kProjMmaCols = 64;
constexpr int kProjMmaThreads = 128;

inline size_t proj_mma_smem_bytes(int d_in) { return (size_t)2 * kProjMmaRows * d_in * 2; }

template <typename T, bool ABSORB>
__global__ void __launch_bounds__(kProjMmaThreads)
mla_project_mma_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out,
                       long long rows, int heads, int d_in, int d_out) {
    using Ops = MmaOps<T>;
    extern __shared__ __align__(128) unsigned char s_proj[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.z, n0 = blockIdx.y * kProjMmaCols;
    const long long r0 = (long long)blockIdx.x * kProjMmaRows;
    const int rb_a = d_in * 2;                                   // bytes per staged x row
    const int rb_b = ABSORB ? kProjMmaCols * 2 : d_in * 2;       // bytes per staged weight row
    const int rows_b = ABSORB ? d_in : kProjMmaCols;             // staged weight rows
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(s_proj);
    const uint32_t sb = sa + kProjMmaRows * rb_a;

    pdl_launch_dependents();
    pdl_wait();

    // ---- stage x rows of this head and the weight tile; chunk c of row r goes to chunk
    //      (c & ~7) | ((c ^ r) & 7) ----
    const int cpr_a = rb_a >> 4;
    for (int i = tid; i < kProjMmaRows * cpr_a; i += kProjMmaThreads) {
        const int row = i / cpr_a, c = i - row * cpr_a;
        const bool valid = r0 + row < rows;
        const T* src = x + ((valid ? r0 + row : 0) * heads + h) * d_in + c * 8;
        cp_async16<0>(sa + row * rb_a + (((c & ~7) | ((c ^ row) & 7)) << 4), src, valid ? 16 : 0, 0);
    }
    const int cpr_b = rb_b >> 4;
    for (int i = tid; i < rows_b * cpr_b; i += kProjMmaThreads) {
        const int row = i / cpr_b, c = i - row * cpr_b;
        const T* src = ABSORB ? w + ((long long)h * d_in + row) * d_out + n0 + c * 8
                              : w + ((long long)h * d_out + n0 + row) * d_in + c * 8;
        cp_async16<0>(sb + row * rb_b + (((c & ~7) | ((c ^ row) & 7)) << 4), src, 16, 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    float acc[kProjMmaCols / 8][4];
#pragma unroll
    for (int nt = 0; nt < kProjMmaCols / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    const int a_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    for (int ks = 0; ks < d_in / 16; ++ks) {
        uint32_t a[4];
        {
            const int c = 2 * ks + (lane >> 4);
            ldmatrix_x4(sa + a_row * rb_a + (((c & ~7) | ((c ^ a_row) & 7)) << 4), a[0], a[1], a[2], a[3]);
        }
        if (ABSORB) {
            // weight tile rows are the contraction index: transpose on load
            const int k_row = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
            for (int np = 0; np < kProjMmaCols / 16; ++np) {
                const int c = 2 * np + (lane >> 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(sb + k_row * rb_b + (((c ^ k_row) & 7) << 4), b0, b1, b2, b3);
                Ops::mma(acc[2 * np], a, b0, b1);
                Ops::mma(acc[2 * np + 1], a, b2, b3);
            }
        } else {
            // weight tile rows are output columns, the contraction index runs along the row
#pragma unroll
            for (int np = 0; np < kProjMmaCols / 16; ++np) {
                const int n_row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int c = 2 * ks + ((lane >> 3) & 1);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(sb + n_row * rb_b + (((c & ~7) | ((c ^ n_row) & 7)) << 4), b0, b1, b2, b3);
                Ops::mma(acc[2 * np], a, b0, b1);
                Ops::mma(acc[2 * np + 1], a, b2, b3);
            }
        }
    }

    // ---- fragments to global: thread holds rows (lane >> 2) and +8, columns 2 * (lane & 3), +1 ----
    const long long row_lo = r0 + warp * 16 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < kProjMmaCols / 8; ++nt) {
        const int col = n0 + nt * 8 + (lane & 3) * 2;
        if (row_lo < rows)
            *reinterpret_cast<uint32_t*>(out + (row_lo * heads + h) * d_out + col) = Ops::pack(acc[nt][0], acc[nt][1]);
        if (row_lo + 8 < rows)
            *reinterpret_cast<uint32_t*>(out + ((row_lo + 8) * heads + h) * d_out + col) =
                Ops::pack(acc[nt][2], acc[nt][3]);
    }
}

}  // namespace gqa_b200

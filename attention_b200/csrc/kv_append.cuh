// One-token-per-sequence KV cache append: the writer of the pages the decode
// kernels read.  One CTA per sequence copies the [kv_heads * head_dim] row of
// key and of value into slot positions[b] % block_size of page
// block_table[b, positions[b] / block_size].
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gqa_b200 {

constexpr int kAppendThreads = 256;

struct AppendParams {
    const void* key;
    const void* value;
    void* k_cache;
    void* v_cache;
    const int32_t* table;
    const int32_t* positions;
    long long row_bytes;     // kv_heads * head_dim * sizeof(element)
    long long num_blocks;
    int block_size, max_pages, cap_tokens;
};

// UNIT is the copy granule: uint4 when rows and bases are 16-byte aligned, else
// the element size.  Out-of-range positions or page ids are skipped.
template <typename UNIT>
__global__ void __launch_bounds__(kAppendThreads) kv_append_kernel(const AppendParams a) {
    const int b = blockIdx.x;
    const int t = __ldg(a.positions + b);
    if (t < 0 || t >= a.cap_tokens) return;
    const int page = t / a.block_size;
    const int slot = t - page * a.block_size;
    const long long phys = __ldg(a.table + (long long)b * a.max_pages + page);
    if (phys < 0 || phys >= a.num_blocks) return;
    const long long units = a.row_bytes / (long long)sizeof(UNIT);
    const UNIT* ks = reinterpret_cast<const UNIT*>(static_cast<const char*>(a.key) + b * a.row_bytes);
    const UNIT* vs = reinterpret_cast<const UNIT*>(static_cast<const char*>(a.value) + b * a.row_bytes);
    const long long dst_off = (phys * a.block_size + slot) * a.row_bytes;
    UNIT* kd = reinterpret_cast<UNIT*>(static_cast<char*>(a.k_cache) + dst_off);
    UNIT* vd = reinterpret_cast<UNIT*>(static_cast<char*>(a.v_cache) + dst_off);
    for (long long i = threadIdx.x; i < units; i += kAppendThreads) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
}

}  // namespace gqa_b200

// Host side of the paged latent-attention (MLA) decode entry points declared in
// include/mla_decode_b200.h: argument checks, the static split policy, the
// workspace layout and the kernel launches.  No allocation, no synchronisation.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "../../include/mla_decode_b200.h"
#include "mla_attend_tc.cuh"
#include "mla_project_mma.cuh"
#include "mla_simt.cuh"

namespace gqa_b200 {
namespace {

constexpr int kMaxDevices = 64;
constexpr int kMlaMaxSplits = 32;
constexpr int kMlaMinTokensPerSplit = 64;

int g_sm_count[kMaxDevices];
std::mutex g_mla_cache_mutex;   // guards the per-device caches of this file

cudaError_t sm_count(int* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mla_cache_mutex);
    if (g_sm_count[dev] == 0) {
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        g_sm_count[dev] = n;
    }
    *out = g_sm_count[dev];
    return cudaSuccess;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Launch with programmatic stream serialization: the kernel may start while its predecessor
// in the stream drains; every kernel of this file executes griddepcontrol.wait before its first
// global access, so the order of the data is kept and only launch latency overlaps.
// GQA_B200_NO_PDL=1 in the environment turns it off.
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    static const bool no_pdl = [] {
        const char* e = std::getenv("GQA_B200_NO_PDL");
        return e && e[0] == '1';
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = no_pdl ? 0 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Status word of the tensor-core attention kernel: 0 ok, 2 = a bounded wait ran out, 3 = the
// dynamic shared memory base was not 1024-byte aligned.  Read with mla_b200_tc_status.
__device__ int g_mla_tc_status;
int* g_mla_tc_status_ptr[kMaxDevices];
bool g_mla_tc_ready[kMaxDevices][2];

cudaError_t mla_tc_status_address(int** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mla_cache_mutex);
    if (!g_mla_tc_status_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_mla_tc_status);
        if (e != cudaSuccess) return e;
        g_mla_tc_status_ptr[dev] = static_cast<int*>(ptr);
    }
    *out = g_mla_tc_status_ptr[dev];
    return cudaSuccess;
}

// Scratch of the tensor-core kernel: the schedule (4 ints + units + 1 prefix entries), then one
// partial slot (128 rows x (2 + 512) floats) per (range, unit) overlap; range + unit is the slot,
// so ranges + units slots suffice.  With the automatic schedule there are at most `pairs` ranges;
// with a forced range length, one range per `force_range` tiles of the capacity.
struct TcScratch {
    size_t sched_bytes, ml_bytes, acc_bytes;
    size_t total() const { return sched_bytes + ml_bytes + acc_bytes; }
};
TcScratch tc_scratch(long long units, int capacity, int pairs, int force_range) {
    const long long cap_tiles = units * ((capacity + kMlaTcBN - 1) / kMlaTcBN);
    const long long ranges = force_range > 0 ? (cap_tiles + force_range - 1) / force_range : pairs;
    const long long slots = ranges + units;
    TcScratch t;
    t.sched_bytes = align_up((size_t)(units + 5) * sizeof(int), 256);
    t.ml_bytes = align_up((size_t)slots * kMlaTcRows * 2 * sizeof(float), 256);
    t.acc_bytes = align_up((size_t)slots * kMlaTcRows * kMlaTcDc * sizeof(float), 256);
    return t;
}
int tc_force_range(int capacity, int splits) {       // an explicit split count: that many ranges per unit
    if (splits <= 0) return 0;
    const int cap_tiles = (capacity + kMlaTcBN - 1) / kMlaTcBN;
    const int fr = (cap_tiles + splits - 1) / splits;
    return fr < 1 ? 1 : fr;
}

bool tc_eligible(int dtype, int dc, int dr, const void* indices) {
    return (dtype == GQA_B200_F16 || dtype == GQA_B200_BF16) && dc == kMlaTcDc && dr == kMlaTcDr && !indices;
}

// Split count of the SIMT attention kernel: a function of the static shape only
// (token capacity and CTA count), so that the host never reads a length.  148
// SMs x 4 resident CTAs is the target; a split never gets fewer than 64 tokens
// of capacity.
int simt_auto_splits(long long rows, int heads, int capacity) {
    const long long base = rows * ((heads + kMlaSimtHeads - 1) / kMlaSimtHeads);
    const long long target = 148LL * 4;
    long long s = base > 0 ? (target + base - 1) / base : 1;
    const long long by_cap = capacity / kMlaMinTokensPerSplit;
    if (s > by_cap) s = by_cap;
    if (s > kMlaMaxSplits) s = kMlaMaxSplits;
    return s < 1 ? 1 : (int)s;
}

size_t partial_bytes(long long rows, int heads, int dc, int splits) {
    if (splits <= 1) return 0;
    const size_t n = (size_t)rows * heads * splits;
    return align_up(n * 2 * sizeof(float), 256) + align_up(n * dc * sizeof(float), 256);
}

// Scratch the two attention paths need; the size queries and mla_b200_attend_ex both use these.
size_t simt_scratch_bytes(int batch, int tq, int heads, int dc, int capacity, int splits) {
    const long long rows = (long long)batch * tq;
    return partial_bytes(rows, heads, dc, splits > 0 ? splits : simt_auto_splits(rows, heads, capacity));
}
long long tc_unit_count(int batch, int tq, int heads) {
    return (long long)batch * (((long long)tq * heads + kMlaTcRows - 1) / kMlaTcRows);
}
size_t tc_scratch_bytes(int batch, int tq, int heads, int capacity, int sms, int splits) {
    return tc_scratch(tc_unit_count(batch, tq, heads), capacity, sms / 2 > 0 ? sms / 2 : 1,
                      tc_force_range(capacity, splits)).total();
}

int check_attend_shape(int dtype, int batch, int tq, int heads, int dc, int dr, long long num_blocks,
                       int page, int max_pages, int nk) {
    if (dtype != GQA_B200_F32 && dtype != GQA_B200_F16 && dtype != GQA_B200_BF16) return GQA_B200_ERR_DTYPE;
    if (batch < 0) return GQA_B200_ERR_BATCH;
    if (tq < 0 || heads <= 0 || dr <= 0 || nk < 0) return MLA_B200_ERR_SHAPE;
    if (dc <= 0 || dc > 512) return MLA_B200_ERR_LATENT_DIM;
    if (num_blocks <= 0 || page <= 0) return GQA_B200_ERR_CACHE_SHAPE;
    if (max_pages <= 0) return GQA_B200_ERR_MAX_PAGES;
    if ((long long)batch * tq > 2147483647LL || (long long)page * max_pages > 2147483647LL ||
        num_blocks > 2147483647LL || (heads + kMlaSimtHeads - 1) / kMlaSimtHeads > 65535)
        return GQA_B200_ERR_INT32_RANGE;
    return GQA_B200_OK;
}

template <typename T>
int launch_attend_simt(const MlaParams& p, cudaStream_t stream) {
    const long long rows = (long long)p.batch * p.tq;
    const size_t smem = ((size_t)kMlaSimtHeads * (p.dc + p.dr) +
                         (size_t)kMlaSimtWarps * kMlaSimtHeads * p.dc) * sizeof(float);
    const dim3 grid((unsigned)rows, (unsigned)((p.heads + kMlaSimtHeads - 1) / kMlaSimtHeads),
                    (unsigned)p.splits);
    const int dcn = (p.dc + 31) / 32;
    auto go = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            if (smem > 200 * 1024) return GQA_B200_ERR_KERNEL;
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        kernel<<<grid, kMlaSimtWarps * 32, smem, stream>>>(p);
        return (int)cudaGetLastError();
    };
    int rc;
    if (dcn <= 2) rc = go(mla_attend_simt_kernel<T, 2>);
    else if (dcn <= 4) rc = go(mla_attend_simt_kernel<T, 4>);
    else if (dcn <= 8) rc = go(mla_attend_simt_kernel<T, 8>);
    else rc = go(mla_attend_simt_kernel<T, 16>);
    if (rc != 0) return rc;
    if (p.splits > 1) {
        const long long total = rows * p.heads;
        rc = launch_pdl(mla_merge_kernel<T>, dim3((unsigned)((total + kMlaMergeWarps - 1) / kMlaMergeWarps)),
                        dim3(kMlaMergeWarps * 32), 0, stream, p, total);
    }
    return rc;
}

template <typename T>
int launch_attend_tc(const MlaParams& p, cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    constexpr int slot = std::is_same<T, __half>::value ? 0 : 1;
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(g_mla_cache_mutex);
        if (!g_mla_tc_ready[dev][slot]) {
            e = cudaFuncSetAttribute(mla_attend_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     MlaTcGeom::kSmemBytes);
            if (e != cudaSuccess) return (int)e;
            g_mla_tc_ready[dev][slot] = true;
        }
    }
    int* status = nullptr;
    e = mla_tc_status_address(&status);
    if (e != cudaSuccess) return (int)e;
    int sms = 0;
    e = sm_count(&sms);
    if (e != cudaSuccess) return (int)e;
    const int pairs = sms / 2 > 0 ? sms / 2 : 1;
    int rc = launch_pdl(mla_tc_plan_kernel, dim3(1), dim3(kMlaTcPlanThreads), 0, stream, p, pairs);
    if (rc != 0) return rc;
    rc = launch_pdl(mla_attend_tc_kernel<T>, dim3(2 * pairs), dim3(kMlaTcThreads), MlaTcGeom::kSmemBytes, stream, p,
                    status);
    if (rc != 0) return rc;
    const long long warps = (long long)p.tc_units * kMlaTcRows;
    return launch_pdl(mla_tc_merge_kernel<T>, dim3((unsigned)((warps + kMlaMergeWarps - 1) / kMlaMergeWarps)),
                      dim3(kMlaMergeWarps * 32), 0, stream, p);
}

// fp16 / bf16 with both widths multiples of 64 and 16-byte aligned tensors: tensor-core kernel
template <typename T, bool ABSORB>
int launch_project_mma(const void* x, const void* w, void* out, long long rows, int heads, int d_in, int d_out,
                       cudaStream_t stream) {
    static bool ready[kMaxDevices];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    const size_t smem = proj_mma_smem_bytes(d_in);
    {
        std::lock_guard<std::mutex> lock(g_mla_cache_mutex);
        if (!ready[dev]) {
            e = cudaFuncSetAttribute(mla_project_mma_kernel<T, ABSORB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     160 * 1024);
            if (e != cudaSuccess) return (int)e;
            ready[dev] = true;
        }
    }
    const dim3 grid((unsigned)((rows + kProjMmaRows - 1) / kProjMmaRows), (unsigned)(d_out / kProjMmaCols),
                    (unsigned)heads);
    return launch_pdl(mla_project_mma_kernel<T, ABSORB>, grid, dim3(kProjMmaThreads), smem, stream,
                      static_cast<const T*>(x), static_cast<const T*>(w), static_cast<T*>(out), rows, heads, d_in,
                      d_out);
}

template <typename T>
int launch_project(const void* x, const void* w, void* out, long long rows, int heads, int d_in,
                   int d_out, int absorb, cudaStream_t stream) {
    if constexpr (!std::is_same<T, float>::value) {
        const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
                               reinterpret_cast<uintptr_t>(out)) & 15) == 0;
        if (aligned && d_in % 64 == 0 && d_out % 64 == 0 && proj_mma_smem_bytes(d_in) <= 160 * 1024)
            return absorb ? launch_project_mma<T, true>(x, w, out, rows, heads, d_in, d_out, stream)
                          : launch_project_mma<T, false>(x, w, out, rows, heads, d_in, d_out, stream);
    }
    const size_t smem = (size_t)kProjRows * d_in * sizeof(float);
    if (smem > 48 * 1024) return GQA_B200_ERR_KERNEL;
    const unsigned chunks = (unsigned)((rows + kProjRows - 1) / kProjRows);
    if (absorb) {
        const dim3 grid(chunks, (unsigned)((d_out + kProjThreads - 1) / kProjThreads), (unsigned)heads);
        // (plain launches: with an early-launched successor holding shared memory on every SM
        // these full-grid kernels ran slower)
        mla_absorb_kernel<T><<<grid, kProjThreads, smem, stream>>>(
            static_cast<const T*>(x), static_cast<const T*>(w), static_cast<T*>(out), rows, heads, d_in, d_out);
    } else {
        const dim3 grid(chunks, (unsigned)((d_out + kProjThreads - 1) / kProjThreads), (unsigned)heads);
        mla_value_kernel<T><<<grid, kProjThreads, smem, stream>>>(
            static_cast<const T*>(x), static_cast<const T*>(w), static_cast<T*>(out), rows, heads, d_in, d_out);
    }
    return (int)cudaGetLastError();
}

template <typename F>
int by_dtype(int dtype, F&& f) {
    switch (dtype) {
        case GQA_B200_F32: return f(float{});
        case GQA_B200_F16: return f(__half{});
        case GQA_B200_BF16: return f(__nv_bfloat16{});
        default: return GQA_B200_ERR_DTYPE;
    }
}

}  // namespace
}  // namespace gqa_b200

using namespace gqa_b200;

extern "C" {

int mla_b200_project(const void* x, const void* w, void* out, int dtype, int64_t rows, int heads,
                     int d_in, int d_out, int absorb, void* stream) {
    if (dtype != GQA_B200_F32 && dtype != GQA_B200_F16 && dtype != GQA_B200_BF16) return GQA_B200_ERR_DTYPE;
    if (rows < 0 || heads <= 0 || d_in <= 0 || d_out <= 0) return MLA_B200_ERR_SHAPE;
    if (heads > 65535 || (rows + kProjRows - 1) / kProjRows > 2147483647LL) return GQA_B200_ERR_INT32_RANGE;
    if (rows == 0) return GQA_B200_OK;
    if (!x || !w || !out) return GQA_B200_ERR_NULL_POINTER;
    return by_dtype(dtype, [&](auto tag) {
        return launch_project<decltype(tag)>(x, w, out, rows, heads, d_in, d_out, absorb,
                                             static_cast<cudaStream_t>(stream));
    });
}

int mla_b200_latent_kv_write(const void* latent, const void* rope, void* cache, const int64_t* slots,
                             int64_t n, int dc, int dr, int dtype, void* stream) {
    if (dtype != GQA_B200_F32 && dtype != GQA_B200_F16 && dtype != GQA_B200_BF16) return GQA_B200_ERR_DTYPE;
    if (n < 0 || dc <= 0 || dr <= 0) return MLA_B200_ERR_SHAPE;
    if (n > 2147483647LL) return GQA_B200_ERR_INT32_RANGE;
    if (n == 0) return GQA_B200_OK;
    if (!latent || !rope || !cache || !slots) return GQA_B200_ERR_NULL_POINTER;
    return by_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        return launch_pdl(mla_cache_write_kernel<T>, dim3((unsigned)n), dim3(128), 0, static_cast<cudaStream_t>(stream),
                          static_cast<const T*>(latent), static_cast<const T*>(rope), static_cast<T*>(cache), slots,
                          dc, dr);
    });
}

size_t mla_b200_attend_ex_workspace_bytes(int batch, int tq, int heads, int dc, int dr, int page,
                                          int max_pages, int nk, int splits) {
    if (check_attend_shape(GQA_B200_F32, batch, tq, heads, dc, dr, 1, page, max_pages, nk) != 0) return 0;
    if (splits < 0 || splits > 65535) return 0;
    // Whether `indices` will be passed is not known here, so the answer covers both kernels
    // mla_b200_attend_ex may take for this shape: the SIMT kernel (dense, or index-selected
    // over nk entries) and, for the tensor-core shape, the dense tensor-core kernel.
    size_t need = simt_scratch_bytes(batch, tq, heads, dc, page * max_pages, splits);
    if (nk > 0) {
        const size_t sel = simt_scratch_bytes(batch, tq, heads, dc, nk, splits);
        if (sel > need) need = sel;
    }
    if (dc == kMlaTcDc && dr == kMlaTcDr && splits <= 32767) {
        int sms = 0;
        if (sm_count(&sms) != cudaSuccess) sms = 148;
        const size_t tc = tc_scratch_bytes(batch, tq, heads, page * max_pages, sms, splits);
        if (tc > need) need = tc;
    }
    return need > 256 ? need : 256;
}

size_t mla_b200_attend_workspace_bytes(int batch, int tq, int heads, int dc, int dr, int page,
                                       int max_pages, int nk) {
    return mla_b200_attend_ex_workspace_bytes(batch, tq, heads, dc, dr, page, max_pages, nk, 0);
}

int mla_b200_attend_ex(const void* q_absorbed, const void* q_rope, const void* cache,
                       const int32_t* block_table, const int32_t* lengths, const int32_t* positions,
                       const int32_t* indices, void* out, int dtype, int batch, int tq, int heads,
                       int dc, int dr, int64_t num_blocks, int page, int max_pages, int nk,
                       float scale, int causal, void* workspace, size_t workspace_bytes, void* stream,
                       int kernel, int splits) {
    int rc = check_attend_shape(dtype, batch, tq, heads, dc, dr, num_blocks, page, max_pages, nk);
    if (rc != 0) return rc;
    if (!(scale > 0.f) || !std::isfinite(scale)) return GQA_B200_ERR_SCALE;
    if (splits < 0 || splits > 65535) return GQA_B200_ERR_SPLITS;
    if (batch == 0 || tq == 0) return GQA_B200_OK;
    if (!q_absorbed || !q_rope || !cache || !block_table || !lengths || !positions || !out)
        return GQA_B200_ERR_NULL_POINTER;
    if (indices && nk <= 0) return MLA_B200_ERR_SHAPE;
    if (kernel != MLA_B200_KERNEL_AUTO && kernel != MLA_B200_KERNEL_SIMT && kernel != MLA_B200_KERNEL_TCGEN05)
        return GQA_B200_ERR_KERNEL;
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    const bool tc_ok = tc_eligible(dtype, dc, dr, indices) && aligned16(q_absorbed) && aligned16(q_rope) &&
                       aligned16(cache) && aligned16(out) && (long long)tq * heads <= 65535LL * kMlaTcRows &&
                       batch <= 65535;
    if (kernel == MLA_B200_KERNEL_TCGEN05 && !tc_ok) return GQA_B200_ERR_KERNEL;
    const bool use_tc = tc_ok && kernel != MLA_B200_KERNEL_SIMT;

    const long long rows = (long long)batch * tq;
    const int capacity = indices ? nk : page * max_pages;
    MlaParams p{};
    p.q = q_absorbed; p.qr = q_rope; p.cache = cache; p.table = block_table; p.lens = lengths;
    p.pos = positions; p.indices = indices; p.out = out;
    p.num_blocks = num_blocks;
    p.batch = batch; p.tq = tq; p.heads = heads; p.dc = dc; p.dr = dr; p.page = page;
    p.max_pages = max_pages; p.nk = indices ? nk : 0; p.causal = causal ? 1 : 0;
    p.scale_log2 = scale * kLog2e;
    p.page_shift = (page & (page - 1)) == 0 ? __builtin_ctz((unsigned)page) : -1;
    if (use_tc) {
        int sms = 0;
        cudaError_t e = sm_count(&sms);
        if (e != cudaSuccess) return (int)e;
        if (splits > 32767) return GQA_B200_ERR_SPLITS;
        const long long units = tc_unit_count(batch, tq, heads);
        if (units > 2147483647LL / kMlaTcRows) return GQA_B200_ERR_INT32_RANGE;
        p.tc_units = (int)units;
        p.tc_row_tiles = (int)(((long long)tq * heads + kMlaTcRows - 1) / kMlaTcRows);
        p.tc_force_range = tc_force_range(capacity, splits);
        {   // softmax warps whose rows are padding in EVERY unit stay out of the kernel's protocol;
            // when units differ in their row count (rows per sequence above 128 and not a multiple
            // of it) all four row groups take part
            const long long rows_per_seq = (long long)tq * heads;
            p.tc_live_quads = rows_per_seq <= kMlaTcRows ? (int)((rows_per_seq + 31) / 32) : 4;
        }
        const TcScratch t = tc_scratch(units, capacity, sms / 2 > 0 ? sms / 2 : 1, p.tc_force_range);
        if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < t.total())
            return GQA_B200_ERR_WORKSPACE;
        char* ws = static_cast<char*>(workspace);
        p.tc_sched = reinterpret_cast<int*>(ws);
        p.part_ml = reinterpret_cast<float*>(ws + t.sched_bytes);
        p.part_acc = reinterpret_cast<float*>(ws + t.sched_bytes + t.ml_bytes);
        p.splits = 1;
    } else {
        p.splits = splits > 0 ? splits : simt_auto_splits(rows, heads, capacity);
    }
    if (!use_tc && p.splits > 1) {
        const size_t need = simt_scratch_bytes(batch, tq, heads, dc, capacity, p.splits);
        if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < need)
            return GQA_B200_ERR_WORKSPACE;
        const size_t n = (size_t)rows * heads * p.splits;
        p.part_ml = static_cast<float*>(workspace);
        p.part_acc = reinterpret_cast<float*>(static_cast<char*>(workspace) + align_up(n * 2 * sizeof(float), 256));
    }
    if (use_tc) {
        if (dtype == GQA_B200_F16) return launch_attend_tc<__half>(p, static_cast<cudaStream_t>(stream));
        return launch_attend_tc<__nv_bfloat16>(p, static_cast<cudaStream_t>(stream));
    }
    return by_dtype(dtype, [&](auto tag) {
        return launch_attend_simt<decltype(tag)>(p, static_cast<cudaStream_t>(stream));
    });
}

int mla_b200_attend(const void* q_absorbed, const void* q_rope, const void* cache,
                    const int32_t* block_table, const int32_t* lengths, const int32_t* positions,
                    const int32_t* indices, void* out, int dtype, int batch, int tq, int heads, int dc,
                    int dr, int64_t num_blocks, int page, int max_pages, int nk, float scale,
                    int causal, void* workspace, size_t workspace_bytes, void* stream) {
    return mla_b200_attend_ex(q_absorbed, q_rope, cache, block_table, lengths, positions, indices, out,
                              dtype, batch, tq, heads, dc, dr, num_blocks, page, max_pages, nk, scale,
                              causal, workspace, workspace_bytes, stream, MLA_B200_KERNEL_AUTO, 0);
}

static size_t stage_bytes(int batch, int tq, int heads, int dc) {
    return align_up((size_t)batch * tq * heads * dc * 4, 256);   // sized for fp32 elements
}

size_t mla_b200_decode_workspace_bytes(int batch, int tq, int heads, int dc, int dr, int page,
                                       int max_pages, int nk) {
    const size_t attend = mla_b200_attend_workspace_bytes(batch, tq, heads, dc, dr, page, max_pages, nk);
    if (attend == 0) return 0;
    return 2 * stage_bytes(batch, tq, heads, dc) + attend;
}

int mla_b200_decode(const void* q_nope, const void* q_rope, const void* cache,
                    const int32_t* block_table, const int32_t* lengths, const int32_t* positions,
                    const void* w_uk, const void* w_uv, const int32_t* indices, void* out, int dtype,
                    int batch, int tq, int heads, int dn, int dr, int dc, int dv, int64_t num_blocks,
                    int page, int max_pages, int nk, float scale, int causal, void* workspace,
                    size_t workspace_bytes, void* stream) {
    int rc = check_attend_shape(dtype, batch, tq, heads, dc, dr, num_blocks, page, max_pages, nk);
    if (rc != 0) return rc;
    if (dn <= 0 || dv <= 0) return MLA_B200_ERR_SHAPE;
    if (!(scale > 0.f) || !std::isfinite(scale)) return GQA_B200_ERR_SCALE;
    if (batch == 0 || tq == 0) return GQA_B200_OK;
    if (!q_nope || !w_uk || !w_uv || !out) return GQA_B200_ERR_NULL_POINTER;
    const size_t stage = stage_bytes(batch, tq, heads, dc);
    const size_t need = mla_b200_decode_workspace_bytes(batch, tq, heads, dc, dr, page, max_pages, nk);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < need)
        return GQA_B200_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    void* q_abs = ws;
    void* latent = ws + stage;
    const int64_t rows = (int64_t)batch * tq;
    rc = mla_b200_project(q_nope, w_uk, q_abs, dtype, rows, heads, dn, dc, 1, stream);
    if (rc != 0) return rc;
    rc = mla_b200_attend(q_abs, q_rope, cache, block_table, lengths, positions, indices, latent, dtype,
                         batch, tq, heads, dc, dr, num_blocks, page, max_pages, nk, scale, causal,
                         ws + 2 * stage, workspace_bytes - 2 * stage, stream);
    if (rc != 0) return rc;
    return mla_b200_project(latent, w_uv, out, dtype, rows, heads, dc, dv, 0, stream);
}

int mla_b200_tc_status(int reset) {
    int* status = nullptr;
    cudaError_t e = mla_tc_status_address(&status);
    if (e != cudaSuccess) return -(int)e;
    int host = 0;
    e = cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return -(int)e;
    if (reset) {
        const int zero = 0;
        e = cudaMemcpy(status, &zero, sizeof(int), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return -(int)e;
    }
    return host;
}

}  // extern "C"

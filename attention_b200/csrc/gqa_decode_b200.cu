// C ABI of the B200 paged GQA decode library: argument checks, workspace
// carving, kernel selection and launches.  No allocation, no synchronisation,
// no exceptions cross this boundary.
#include "../../include/gqa_decode_b200.h"
#include "../../include/mla_decode_b200.h"

#include <cmath>
#include <cstdlib>
#include <cstdint>
#include <limits>
#include <mutex>

#include "gqa_common.cuh"
#include "gqa_decode_mma.cuh"
#include "gqa_decode_simt.cuh"
#include "gqa_plan_merge.cuh"
#include "gqa_prefill_mma.cuh"
#include "gqa_prefill_simt.cuh"
#include "gqa_prefill_pp.cuh"
#include "kv_append.cuh"

using namespace gqa_b200;

namespace {

constexpr int kTableEntriesBudget = 2048;   // page ids staged in shared memory per segment
constexpr int kMaxDevices = 64;
constexpr bool kPrefillAutoPicksTcgen05 = true;    // KERNEL_AUTO prefers the tcgen05 prefill kernel
constexpr int kWarpMergeMinPairs = 1024;    // fewer (sequence, head) pairs: CTA-per-pair merge

struct DeviceInfo {
    int sm_count = 0;
    int max_smem_optin = 0;
    bool ready = false;
};
DeviceInfo g_dev[kMaxDevices];
std::mutex g_dev_mutex;

// Device properties are read once per device (two cudaDeviceGetAttribute calls).
cudaError_t device_info(DeviceInfo** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return e;
        d.ready = true;
    }
    *out = &d;
    return cudaSuccess;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int elem_size(int dtype) { return dtype == GQA_B200_F32 ? 4 : 2; }

struct WorkspaceLayout {
    size_t hdr, tickets, chunk_off, items, part_ml, part_acc, total;
    size_t control_bytes;   // header + tickets: the part that must be zero before the first call
    int cap_chunks;
};

constexpr int kAssumedCtaSlots = 2 * 148;   // B200: 148 SMs x 2 resident decode CTAs

// Chunk total at which the work items (chunks x kv heads x head groups) number about
// three quarters of the resident decode CTAs: enough to occupy every SM in one wave.
int item_target_chunks(int q_heads, int kv_heads) {
    const int group = q_heads / kv_heads;
    const long long per_chunk = (long long)kv_heads * ((group + 15) / 16);
    const long long t = (3ll * kAssumedCtaSlots + 4 * per_chunk - 1) / (4 * per_chunk);
    return (int)(t < 1 ? 1 : t);
}

// chunk_base == 0 (the plan kernel picks the base from the actual lengths): the chunk
// total is at most that of base 1024 when 1024 is picked, and below twice the item
// target otherwise (halving the base at most doubles a sequence's chunk count, and a
// smaller base is only taken while the next larger one stays below the target).
WorkspaceLayout workspace_layout(int batch, int q_heads, int kv_heads, int head_dim,
                                 int block_size, int max_pages, int chunk_base) {
    WorkspaceLayout w{};
    const long long cap_tokens = (long long)max_pages * block_size;
    const long long nb = batch > 0 ? batch : 0;
    long long cap;
    if (chunk_base == 0) {
        cap = nb * max_chunks_for_capacity(cap_tokens, 1024);
        // room for the finer bases the device may pick: eight waves of items over the resident
        // CTAs (the one-launch kernel only considers bases whose chunk total fits), never less
        // than the plan kernel's own bound of twice its item target
        const long long per = (long long)kv_heads * (((q_heads / kv_heads) + 15) / 16);
        long long dyn = (8ll * kAssumedCtaSlots + per - 1) / per + nb;
        const long long plan_bound = 2ll * item_target_chunks(q_heads, kv_heads) + nb;
        if (plan_bound > dyn) dyn = plan_bound;
        const long long finest = nb * max_chunks_for_capacity(cap_tokens, 1024 >> (kNumAutoBases - 1));
        const long long other = dyn < finest ? dyn : finest;
        if (other > cap) cap = other;
    } else {
        cap = nb * max_chunks_for_capacity(cap_tokens, chunk_base);
    }
    if (cap > 0x3fffffffll) cap = 0x3fffffffll;   // bit 30 of a slot is the single-chunk flag
                                                  // (decode_ex refuses shapes that hit this)
    w.cap_chunks = (int)cap;
    size_t at = 0;
    w.hdr = at;        at = align_up(at + kHdrWords * sizeof(int32_t), 256);
    // one ticket per (sequence, kv head, head group); a fixed region whatever the shape
    w.tickets = at;    at = align_up(at + (size_t)kFusedMaxTickets * sizeof(int32_t), 256);
    w.control_bytes = at;
    w.chunk_off = at;  at = align_up(at + ((size_t)batch + 1) * sizeof(int32_t), 256);
    w.items = at;      at = align_up(at + (size_t)cap * sizeof(int4), 256);
    w.part_ml = at;    at = align_up(at + (size_t)cap * q_heads * sizeof(float2), 256);
    w.part_acc = at;   at = align_up(at + (size_t)cap * q_heads * head_dim * sizeof(float), 256);
    w.total = at;
    return w;
}

// What the plan kernel would pick if every sequence filled its table: a host-side
// preview of the adaptive rule (the device applies it to the real lengths).
int auto_chunk_base(int batch, int q_heads, int kv_heads, int block_size, int max_pages) {
    const long long cap_tokens = (long long)max_pages * block_size;
    const int target = item_target_chunks(q_heads, kv_heads);
    for (int i = 0; i < kNumAutoBases; ++i) {
        const int base = 1024 >> i;
        const int len = cap_tokens > 0x7fffffffll ? 0x7fffffff : (int)cap_tokens;
        if ((long long)batch * chunks_for(len, base) >= target) return base;
    }
    return 1024 >> (kNumAutoBases - 1);
}

// 0 stays 0 (= adaptive, decided on the device); anything else must be in range.
int resolve_chunk_base(int chunk_tokens) {
    if (chunk_tokens == 0) return 0;
    if (chunk_tokens < kMinChunkTokens || chunk_tokens > kMaxChunkTokens) return -1;
    return chunk_tokens;
}

// The reference's argument checks (csrc/cuda/dense/gqa_decode.cu:103-138) that
// can be made on sizes alone; dtype/device/contiguity of the tensors themselves
// are the caller's (the Python wrapper's) to check.
int check_common(const void* q, const void* k, const void* v, const int32_t* table,
                 const int32_t* lens, const void* out, int dtype, int batch, int q_heads,
                 int kv_heads, int head_dim, int64_t num_blocks, int block_size, int max_pages,
                 float scale) {
    if (dtype != GQA_B200_F32 && dtype != GQA_B200_F16 && dtype != GQA_B200_BF16)
        return GQA_B200_ERR_DTYPE;
    if (batch < 0) return GQA_B200_ERR_BATCH;
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return GQA_B200_ERR_HEADS;
    if (head_dim <= 0 || head_dim > 256) return GQA_B200_ERR_HEAD_DIM;
    if (num_blocks <= 0 || block_size <= 0) return GQA_B200_ERR_CACHE_SHAPE;
    if (max_pages <= 0) return GQA_B200_ERR_MAX_PAGES;
    if (!(std::isfinite(scale) && scale > 0.f)) return GQA_B200_ERR_SCALE;
    if (num_blocks > std::numeric_limits<int>::max()) return GQA_B200_ERR_INT32_RANGE;
    if ((long long)batch * q_heads > std::numeric_limits<int>::max())
        return GQA_B200_ERR_INT32_RANGE;
    if (batch > 0 && (!q || !k || !v || !table || !lens || !out)) return GQA_B200_ERR_NULL_POINTER;
    return GQA_B200_OK;
}

void fill_shape(DecodeParams& p, const void* q, const void* k, const void* v,
                const int32_t* table, const int32_t* lens, void* out, int batch, int q_heads,
                int kv_heads, int head_dim, int64_t num_blocks, int block_size, int max_pages,
                float scale) {
    p.q = q; p.k = k; p.v = v; p.out = out; p.table = table; p.lens = lens;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = q_heads / kv_heads;
    p.head_dim = head_dim;
    p.block_size = block_size;
    p.bs_shift = -1;
    if ((block_size & (block_size - 1)) == 0) {
        int s = 0;
        while ((1 << s) < block_size) ++s;
        p.bs_shift = s;
    }
    p.max_pages = max_pages;
    p.num_blocks = num_blocks;
    const long long cap = (long long)max_pages * block_size;
    p.cap_tokens = cap > 0x7fffffffll ? 0x7fffffff : (int)cap;
    p.scale_log2 = scale * kLog2e;
}

void set_segment(DecodeParams& p, long long max_part_tokens) {
    long long seg = (long long)kTableEntriesBudget * p.block_size;
    if (seg > max_part_tokens) seg = max_part_tokens;
    if (seg < 1) seg = 1;
    if (seg > 0x40000000ll) seg = 0x40000000ll;
    p.seg_tokens = (int)seg;
    p.table_smem_entries = (int)(seg / p.block_size) + 2;
}

bool mma_eligible(const DecodeParams& p, int dtype) {
    if (dtype == GQA_B200_F32) return false;
    if (p.head_dim != 64 && p.head_dim != 128 && p.head_dim != 256) return false;
    return aligned16(p.q) && aligned16(p.k) && aligned16(p.v) && aligned16(p.out);
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
// Resident CTAs per SM of a (kernel, dynamic shared memory) pair on a device.
// Looked up on every call, computed once: the first use also raises the
// kernel's dynamic shared-memory limit.
struct OccEntry {
    const void* kernel;
    int dev;
    size_t smem;
    int per_sm;
};
constexpr int kOccEntries = 256;
OccEntry g_occ[kOccEntries];
int g_occ_count = 0;
std::mutex g_occ_mutex;

template <typename KernelT>
cudaError_t resident_ctas(KernelT kernel, int threads, size_t smem, int smem_limit, int* per_sm) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const void* key = reinterpret_cast<const void*>(kernel);
    std::lock_guard<std::mutex> lock(g_occ_mutex);
    for (int i = 0; i < g_occ_count; ++i) {
        if (g_occ[i].kernel == key && g_occ[i].dev == dev && g_occ[i].smem == smem) {
            *per_sm = g_occ[i].per_sm;
            return cudaSuccess;
        }
    }
    // raise the dynamic limit to the device maximum (less the kernel's static
    // shared memory) once, so later calls with another table size never lower it
    cudaFuncAttributes fa{};
    e = cudaFuncGetAttributes(&fa, kernel);
    if (e != cudaSuccess) return e;
    const int dyn_limit = smem_limit - (int)fa.sharedSizeBytes;
    if ((long long)smem > dyn_limit) return cudaErrorInvalidValue;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_limit);
    if (e != cudaSuccess) return e;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, kernel, threads, smem);
    if (e != cudaSuccess) return e;
    if (g_occ_count < kOccEntries) g_occ[g_occ_count++] = OccEntry{key, dev, smem, *per_sm};
    return cudaSuccess;
}

// Launch with the programmatic-stream-serialization attribute, so the kernel may
// begin launching while the kernel before it in the stream drains (each kernel
// waits on-device before touching memory; see pdl_wait).  GQA_B200_NO_PDL=1 in the
// environment falls back to plain stream order.
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = getenv("GQA_B200_NO_PDL");
        return !(v && v[0] == '1');
    }();
    return on;
}

template <typename KernelT>
cudaError_t launch_kernel(KernelT kernel, dim3 grid, int threads, size_t smem, cudaStream_t stream,
                          const DecodeParams& p) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

// Shared memory of the one-launch mode's chunk prefix and length arrays, in steps of 1 KB so that
// the occupancy cache sees few distinct sizes.
inline size_t fused_prefix_bytes(const DecodeParams& p) {
    if (p.mode != kModeFused) return 0;
    return align_up((2 * (size_t)p.batch + 1) * sizeof(int), 1024);   // chunk prefix + lengths
}

template <typename KernelT>
cudaError_t launch_persistent(KernelT kernel, const DecodeParams& p, int threads, size_t smem,
                              int max_ctas, long long item_bound, cudaStream_t stream) {
    DeviceInfo* dev = nullptr;
    cudaError_t e = device_info(&dev);
    if (e != cudaSuccess) return e;
    if (smem > (size_t)dev->max_smem_optin) return cudaErrorInvalidValue;
    int per_sm = 0;
    e = resident_ctas(kernel, threads, smem, dev->max_smem_optin, &per_sm);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    long long grid = (long long)per_sm * dev->sm_count;
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    if (grid > item_bound) grid = item_bound;
    if (grid < 1) grid = 1;
    return launch_kernel(kernel, dim3((unsigned)grid), threads, smem, stream, p);
}

template <typename T, int D, int TILE_N, int NSTAGES, int MIN_CTAS, int NWARPS = 4, int CP_MODE = 3>
cudaError_t launch_mma(const DecodeParams& p, int max_ctas, long long item_bound,
                       cudaStream_t stream) {
    using G = MmaGeom<D, TILE_N, NSTAGES, NWARPS>;
    const size_t smem = G::kFixedBytes + (size_t)p.table_smem_entries * sizeof(int) + fused_prefix_bytes(p);
    return launch_persistent(gqa_decode_mma_kernel<T, D, TILE_N, NSTAGES, NWARPS, MIN_CTAS, CP_MODE>, p,
                             NWARPS * 32, smem, max_ctas, item_bound, stream);
}

template <typename T>
cudaError_t launch_mma_for_dim(const DecodeParams& p, int max_ctas, long long item_bound,
                               cudaStream_t stream) {
    switch (p.head_dim) {
        case 64:  return launch_mma<T, 64, 32, 3, 2>(p, max_ctas, item_bound, stream);
        case 128:
            return launch_mma<T, 128, 16, 3, 2>(p, max_ctas, item_bound, stream);
        case 256: return launch_mma<T, 256, 16, 3, 1>(p, max_ctas, item_bound, stream);
        default:  return cudaErrorInvalidValue;
    }
}

template <typename T, int EPL, bool CONTIG, int GB>
cudaError_t launch_simt(const DecodeParams& p, int max_ctas, long long item_bound,
                        cudaStream_t stream) {
    const int o_stride = ((p.head_dim + 3) & ~3) + 4;
    const size_t smem = ((size_t)kSimtWarps * GB * o_stride + 2 * kSimtWarps * GB) * sizeof(float) +
                        (size_t)p.table_smem_entries * sizeof(int) + fused_prefix_bytes(p);
    return launch_persistent(gqa_decode_simt_kernel<T, EPL, CONTIG, GB>, p, kSimtWarps * 32, smem,
                             max_ctas, item_bound, stream);
}

// Query heads handled per SIMT item (registers: GB * EPL fp32 for q and for acc).
inline int simt_heads_per_item(int head_dim, int group) {
    const int epl = (head_dim + 31) / 32;
    if (epl > 4) return 4;
    return group > 4 ? 8 : 4;
}

template <typename T, int EPL, bool CONTIG>
cudaError_t launch_simt_gb(const DecodeParams& p, int max_ctas, long long item_bound,
                           cudaStream_t stream) {
    if constexpr (EPL <= 4) {
        if (p.heads_per_item == 8)
            return launch_simt<T, EPL, CONTIG, 8>(p, max_ctas, item_bound, stream);
    }
    return launch_simt<T, EPL, CONTIG, 4>(p, max_ctas, item_bound, stream);
}

template <typename T>
cudaError_t launch_simt_for_dim(const DecodeParams& p, int max_ctas, long long item_bound,
                                cudaStream_t stream) {
    const int D = p.head_dim;
    const bool contig = (D % 32 == 0) && aligned16(p.q) && aligned16(p.k) && aligned16(p.v) &&
                        aligned16(p.out);
    const int epl = (D + 31) / 32;
    if (contig) {
        switch (epl) {
            case 1: return launch_simt_gb<T, 1, true>(p, max_ctas, item_bound, stream);
            case 2: return launch_simt_gb<T, 2, true>(p, max_ctas, item_bound, stream);
            case 4: return launch_simt_gb<T, 4, true>(p, max_ctas, item_bound, stream);
            case 8: return launch_simt_gb<T, 8, true>(p, max_ctas, item_bound, stream);
            default: break;   // 96, 160, 192, 224: strided path below
        }
    }
    if (epl <= 1) return launch_simt_gb<T, 1, false>(p, max_ctas, item_bound, stream);
    if (epl <= 2) return launch_simt_gb<T, 2, false>(p, max_ctas, item_bound, stream);
    if (epl <= 4) return launch_simt_gb<T, 4, false>(p, max_ctas, item_bound, stream);
    return launch_simt_gb<T, 8, false>(p, max_ctas, item_bound, stream);
}

template <typename T>
cudaError_t launch_decode_t(DecodeParams& p, bool use_mma, int max_ctas, cudaStream_t stream) {
    if (use_mma) {
        p.heads_per_item = 16;
    } else {
        p.heads_per_item = simt_heads_per_item(p.head_dim, p.group);
    }
    p.head_groups = (p.group + p.heads_per_item - 1) / p.heads_per_item;
    long long parts = p.mode == kModeRefSplits ? (long long)p.batch * p.splits
                                               : (long long)p.cap_chunks;
    long long item_bound = parts * p.kv_heads * p.head_groups;
    if (item_bound > 0x7fffffffll) return cudaErrorInvalidValue;
    if (use_mma) {
        if constexpr (sizeof(T) == 2) {
            return launch_mma_for_dim<T>(p, max_ctas, item_bound, stream);
        } else {
            return cudaErrorInvalidValue;
        }
    }
    return launch_simt_for_dim<T>(p, max_ctas, item_bound, stream);
}

cudaError_t launch_decode(DecodeParams& p, int dtype, bool use_mma, int max_ctas,
                          cudaStream_t stream) {
    switch (dtype) {
        case GQA_B200_F32:  return launch_decode_t<float>(p, use_mma, max_ctas, stream);
        case GQA_B200_F16:  return launch_decode_t<__half>(p, use_mma, max_ctas, stream);
        default:            return launch_decode_t<__nv_bfloat16>(p, use_mma, max_ctas, stream);
    }
}

// Planned mode with head_dim % 4 == 0: one warp per (sequence, head) when there are
// enough pairs to fill the GPU that way, else one CTA per pair (its four warps share a
// long sequence's partials).
template <typename T>
cudaError_t launch_merge_t(const DecodeParams& p, cudaStream_t stream) {
    const bool vec4 = p.mode == kModePlanned && p.head_dim % 4 == 0;
    if (vec4 && (long long)p.batch * p.q_heads >= kWarpMergeMinPairs) {
        const long long pairs = (long long)p.batch * p.q_heads;
        const unsigned grid = (unsigned)((pairs + kMergeWarps - 1) / kMergeWarps);
        return launch_kernel(gqa_merge_warp_kernel<T>, dim3(grid), kMergeWarps * 32, 0, stream, p);
    }
    const dim3 grid((unsigned)((long long)p.batch * p.q_heads));   // <= INT_MAX by check_common
    if (vec4) return launch_kernel(gqa_merge_kernel<T, true>, grid, kMergeWarps * 32, 0, stream, p);
    return launch_kernel(gqa_merge_kernel<T, false>, grid, kMergeWarps * 32, 0, stream, p);
}

cudaError_t launch_merge(const DecodeParams& p, int dtype, cudaStream_t stream) {
    switch (dtype) {
        case GQA_B200_F32:  return launch_merge_t<float>(p, stream);
        case GQA_B200_F16:  return launch_merge_t<__half>(p, stream);
        default:            return launch_merge_t<__nv_bfloat16>(p, stream);
    }
}

}  // namespace

// ---------------------------------------------------------------------------
// exported entry points
// ---------------------------------------------------------------------------
extern "C" {

int gqa_b200_abi_version(void) { return GQA_B200_ABI_VERSION; }

const char* gqa_b200_strerror(int code) {
    switch (code) {
        case GQA_B200_OK: return "ok";
        case GQA_B200_ERR_NULL_POINTER: return "a required pointer is null";
        case GQA_B200_ERR_DTYPE: return "q/k/v must be float32/float16/bfloat16";
        case GQA_B200_ERR_HEADS: return "Hq must be divisible by Hkv";
        case GQA_B200_ERR_HEAD_DIM: return "supported head_dim is [1, 256]";
        case GQA_B200_ERR_CACHE_SHAPE: return "cache must have positive blocks and block_size";
        case GQA_B200_ERR_MAX_PAGES: return "block_table must have at least one page";
        case GQA_B200_ERR_SCALE: return "scale must be positive and finite";
        case GQA_B200_ERR_BATCH: return "batch must be non-negative";
        case GQA_B200_ERR_WORKSPACE: return "workspace is missing, not 256-byte aligned, or too small";
        case GQA_B200_ERR_SPLITS: return "splits must be in [1, 65535]";
        case GQA_B200_ERR_KERNEL: return "the requested kernel cannot run these arguments";
        case GQA_B200_ERR_CHUNK: return "chunk_tokens must be 0 or in [16, 65536]";
        case GQA_B200_ERR_INT32_RANGE: return "tensor sizes exceed int32 CUDA launch limits";
        case GQA_B200_ERR_STATIC_LIMIT:
            return "shape needs more scratch than gqa_b200_decode_static's built-in "
                   "GQA_B200_STATIC_SCRATCH_BYTES; use gqa_b200_decode with a caller workspace";
        case MLA_B200_ERR_SHAPE: return "MLA: a width, head count, tq or nk is not positive";
        case MLA_B200_ERR_LATENT_DIM: return "MLA: supported latent width dc is [1, 512]";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown gqa_b200 status";
}

int gqa_b200_auto_chunk_tokens(int batch, int q_heads, int kv_heads, int block_size,
                               int max_pages) {
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || block_size <= 0 ||
        max_pages <= 0)
        return GQA_B200_ERR_HEADS;
    return auto_chunk_base(batch, q_heads, kv_heads, block_size, max_pages);
}

int gqa_b200_chunk_tokens(int context_len, int chunk_tokens) {
    if (chunk_tokens < kMinChunkTokens || chunk_tokens > kMaxChunkTokens) return GQA_B200_ERR_CHUNK;
    return chunk_tokens_for(context_len < 0 ? 0 : context_len, chunk_tokens);
}

int gqa_b200_max_chunks_per_seq(int max_pages, int block_size, int chunk_tokens) {
    if (chunk_tokens < kMinChunkTokens || chunk_tokens > kMaxChunkTokens) return GQA_B200_ERR_CHUNK;
    if (max_pages <= 0 || block_size <= 0) return 0;
    return max_chunks_for_capacity((long long)max_pages * block_size, chunk_tokens);
}

size_t gqa_b200_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim, int block_size,
                                int max_pages, int chunk_tokens) {
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || head_dim <= 0 ||
        block_size <= 0 || max_pages <= 0)
        return 0;
    const int base = resolve_chunk_base(chunk_tokens);
    if (base < 0) return 0;
    return workspace_layout(batch, q_heads, kv_heads, head_dim, block_size, max_pages, base).total;
}

size_t gqa_b200_workspace_control_bytes(void) {
    return workspace_layout(1, 1, 1, 1, 1, 1, 0).control_bytes;
}

int gqa_b200_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
    const size_t control = gqa_b200_workspace_control_bytes();
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < control)
        return GQA_B200_ERR_WORKSPACE;
    return (int)cudaMemsetAsync(workspace, 0, control, static_cast<cudaStream_t>(stream));
}

int gqa_b200_decode_ex(const void* q, const void* k_cache, const void* v_cache,
                       const int32_t* block_table, const int32_t* context_lens, void* out,
                       int dtype, int batch, int q_heads, int kv_heads, int head_dim,
                       int64_t num_blocks, int block_size, int max_pages, float scale,
                       void* workspace, size_t workspace_bytes, void* stream, int chunk_tokens,
                       int kernel, int max_ctas, int phases) {
    int rc = check_common(q, k_cache, v_cache, block_table, context_lens, out, dtype, batch,
                          q_heads, kv_heads, head_dim, num_blocks, block_size, max_pages, scale);
    if (rc != GQA_B200_OK) return rc;
    const int base = resolve_chunk_base(chunk_tokens);
    if (base < 0) return GQA_B200_ERR_CHUNK;
    if (kernel != GQA_B200_KERNEL_AUTO && kernel != GQA_B200_KERNEL_SIMT &&
        kernel != GQA_B200_KERNEL_MMA)
        return GQA_B200_ERR_KERNEL;
    if (batch == 0) return GQA_B200_OK;

    const WorkspaceLayout lay =
        workspace_layout(batch, q_heads, kv_heads, head_dim, block_size, max_pages, base);
    if (lay.cap_chunks >= 0x3fffffff) return GQA_B200_ERR_INT32_RANGE;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < lay.total)
        return GQA_B200_ERR_WORKSPACE;

    DecodeParams p{};
    fill_shape(p, q, k_cache, v_cache, block_table, context_lens, out, batch, q_heads, kv_heads,
               head_dim, num_blocks, block_size, max_pages, scale);
    char* ws = static_cast<char*>(workspace);
    p.hdr = reinterpret_cast<int32_t*>(ws + lay.hdr);
    p.tickets = reinterpret_cast<int32_t*>(ws + lay.tickets);
    p.chunk_off = reinterpret_cast<int32_t*>(ws + lay.chunk_off);
    p.items = reinterpret_cast<int4*>(ws + lay.items);
    p.part_ml = reinterpret_cast<float2*>(ws + lay.part_ml);
    p.part_acc = reinterpret_cast<float*>(ws + lay.part_acc);
    p.cap_chunks = lay.cap_chunks;
    p.item_target = item_target_chunks(q_heads, kv_heads);
    p.mode = kModePlanned;
    p.splits = 1;
    p.chunk_base = base;
    set_segment(p, 4ll * (base ? base : 1024));

    bool use_mma = mma_eligible(p, dtype);
    if (kernel == GQA_B200_KERNEL_MMA && !use_mma) return GQA_B200_ERR_KERNEL;
    if (kernel == GQA_B200_KERNEL_SIMT) use_mma = false;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    constexpr int kSelfPlanPhases = GQA_B200_PHASE_ONE_LAUNCH | GQA_B200_PHASE_TWO_LAUNCH | GQA_B200_PHASE_SELF_DECODE;
    if ((phases & kSelfPlanPhases) && phases != GQA_B200_PHASE_ONE_LAUNCH &&
        phases != GQA_B200_PHASE_TWO_LAUNCH && phases != GQA_B200_PHASE_SELF_DECODE)
        return GQA_B200_ERR_KERNEL;
    // (the SIMT kernel's groups of four query heads are the finest grouping any kernel uses)
    const long long ticket_count = (long long)batch * kv_heads * ((q_heads / kv_heads + 3) / 4);
    const bool can_self_plan = batch <= kFusedMaxBatch;
    const bool can_ticket = can_self_plan && ticket_count <= kFusedMaxTickets;
    if ((phases == GQA_B200_PHASE_ONE_LAUNCH && !can_ticket) ||
        ((phases == GQA_B200_PHASE_TWO_LAUNCH || phases == GQA_B200_PHASE_SELF_DECODE) && !can_self_plan))
        return GQA_B200_ERR_KERNEL;
    if ((phases == 0 && can_self_plan) || (phases & kSelfPlanPhases)) {
        // No plan launch: the decode kernel cuts the sequences itself.  Whether it also merges is
        // decided from the static shape: tickets cost a CTA a fence and an atomic round trip per
        // item and put the merge of the last sequences behind the streaming, which only pays
        // when every work item can have a CTA of its own even at the finest chunk length, i.e.
        // on small batches of short tables.  Otherwise the merge kernel follows.
        const int hpi = use_mma ? 16 : simt_heads_per_item(head_dim, q_heads / kv_heads);
        const long long head_groups = (q_heads / kv_heads + hpi - 1) / hpi;
        const long long finest_items = (long long)batch *
            max_chunks_for_capacity((long long)max_pages * block_size, base ? base : 1024 >> (kNumAutoBases - 1)) *
            kv_heads * head_groups;
        const bool one_launch = phases == GQA_B200_PHASE_ONE_LAUNCH ||
                                (phases == 0 && can_ticket && finest_items <= kAssumedCtaSlots);
        p.mode = kModeFused;
        p.fused_merge = one_launch ? 1 : 0;
        cudaError_t e = launch_decode(p, dtype, use_mma, max_ctas, s);
        if (e != cudaSuccess || one_launch || phases == GQA_B200_PHASE_SELF_DECODE) return (int)e;
        DecodeParams pm = p;            // the merge kernels read the plan the decode kernel published
        pm.mode = kModePlanned;
        return (int)launch_merge(pm, dtype, s);
    }
    if (phases == 0) phases = GQA_B200_PHASE_PLAN | GQA_B200_PHASE_DECODE | GQA_B200_PHASE_MERGE;
    cudaError_t e = cudaSuccess;
    if (phases & GQA_B200_PHASE_PLAN) {
        e = launch_kernel(gqa_plan_kernel, dim3(1), kPlanThreads, 0, s, p);
        if (e != cudaSuccess) return (int)e;
    }
    if (phases & GQA_B200_PHASE_DECODE) {
        e = launch_decode(p, dtype, use_mma, max_ctas, s);
        if (e != cudaSuccess) return (int)e;
    }
    if (phases & GQA_B200_PHASE_MERGE) e = launch_merge(p, dtype, s);
    return (int)e;
}

int gqa_b200_decode(const void* q, const void* k_cache, const void* v_cache,
                    const int32_t* block_table, const int32_t* context_lens, void* out, int dtype,
                    int batch, int q_heads, int kv_heads, int head_dim, int64_t num_blocks,
                    int block_size, int max_pages, float scale, void* workspace,
                    size_t workspace_bytes, void* stream) {
    return gqa_b200_decode_ex(q, k_cache, v_cache, block_table, context_lens, out, dtype, batch,
                              q_heads, kv_heads, head_dim, num_blocks, block_size, max_pages, scale,
                              workspace, workspace_bytes, stream, 0, GQA_B200_KERNEL_AUTO, 0, 0);
}

// ---------------------------------------------------------------------------
// Decode without any caller- or library-side allocation.
// ---------------------------------------------------------------------------
// Scratch of gqa_b200_decode_static: one fixed array in the module image, so it
// exists on every GPU that loads this library from load until process exit.
constexpr size_t kStaticScratchBytes = (size_t)GQA_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device.  In host code the array's name
// is only a handle for the runtime, not a device pointer; the address each GPU
// gave its copy is asked for once, with that GPU current.
static void* g_static_scratch_ptr[kMaxDevices];
static std::mutex g_static_scratch_mutex;

static cudaError_t static_scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return e;
        if (!ptr) return cudaErrorInvalidSymbol;
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return cudaSuccess;
}

int gqa_b200_decode_static(const void* q, const void* k_cache, const void* v_cache,
                           const int32_t* block_table, const int32_t* context_lens, void* out,
                           int dtype, int batch, int q_heads, int kv_heads, int head_dim,
                           int64_t num_blocks, int block_size, int max_pages, float scale,
                           void* stream) {
    int rc = check_common(q, k_cache, v_cache, block_table, context_lens, out, dtype, batch,
                          q_heads, kv_heads, head_dim, num_blocks, block_size, max_pages, scale);
    if (rc != GQA_B200_OK) return rc;
    if (batch == 0) return GQA_B200_OK;
    const size_t need = gqa_b200_workspace_bytes(batch, q_heads, kv_heads, head_dim, block_size,
                                                 max_pages, 0);
    if (need == 0 || need > kStaticScratchBytes) return GQA_B200_ERR_STATIC_LIMIT;
    void* scratch = nullptr;
    const cudaError_t e = static_scratch_address(&scratch);
    if (e != cudaSuccess) return (int)e;
    // The control words (work counter, tickets) must be zero when a call starts: the
    // array is zero when the module is loaded, and every call leaves them at zero.
    // Partial slots are written before they are read.
    return gqa_b200_decode_ex(q, k_cache, v_cache, block_table, context_lens, out, dtype, batch,
                              q_heads, kv_heads, head_dim, num_blocks, block_size, max_pages, scale,
                              scratch, kStaticScratchBytes, stream, 0, GQA_B200_KERNEL_AUTO, 0, 0);
}

int gqa_b200_decode_split(const void* q, const void* k_cache, const void* v_cache,
                          const int32_t* block_table, const int32_t* context_lens, void* out,
                          int dtype, int batch, int q_heads, int kv_heads, int head_dim,
                          int64_t num_blocks, int block_size, int max_pages, float scale,
                          int splits, float* partials, void* stream) {
    if (splits < 1 || splits > 65535) return GQA_B200_ERR_SPLITS;
    int rc = check_common(q, k_cache, v_cache, block_table, context_lens, out, dtype, batch,
                          q_heads, kv_heads, head_dim, num_blocks, block_size, max_pages, scale);
    if (rc != GQA_B200_OK) return rc;
    if (batch == 0) return GQA_B200_OK;
    if (splits > 1 && !partials) return GQA_B200_ERR_WORKSPACE;

    DecodeParams p{};
    fill_shape(p, q, k_cache, v_cache, block_table, context_lens, out, batch, q_heads, kv_heads,
               head_dim, num_blocks, block_size, max_pages, scale);
    p.mode = kModeRefSplits;
    p.splits = splits;
    p.ref_partials = partials;
    p.chunk_base = kDefaultChunkTokens;
    p.cap_chunks = 0;
    set_segment(p, p.cap_tokens);

    const bool use_mma = mma_eligible(p, dtype);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = launch_decode(p, dtype, use_mma, 0, s);
    if (e != cudaSuccess) return (int)e;
    if (splits > 1) e = launch_merge(p, dtype, s);
    return (int)e;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// dense prefill
// ---------------------------------------------------------------------------
namespace {

template <typename T, int EPL, bool CONTIG>
cudaError_t launch_prefill_simt(const PrefillParams& p, cudaStream_t stream) {
    const int rows_per_cta = kPrefillRows * kPrefillWarps;
    const dim3 grid((unsigned)((p.tq + rows_per_cta - 1) / rows_per_cta), (unsigned)p.q_heads,
                    (unsigned)p.batch);
    gqa_prefill_simt_kernel<T, EPL, CONTIG><<<grid, kPrefillWarps * 32, 0, stream>>>(p);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_prefill_simt_for_dim(const PrefillParams& p, cudaStream_t stream) {
    const int D = p.head_dim;
    const bool contig = (D % 32 == 0) && aligned16(p.q) && aligned16(p.k) && aligned16(p.v) &&
                        aligned16(p.out);
    const int epl = (D + 31) / 32;
    if (contig) {
        switch (epl) {
            case 1: return launch_prefill_simt<T, 1, true>(p, stream);
            case 2: return launch_prefill_simt<T, 2, true>(p, stream);
            case 4: return launch_prefill_simt<T, 4, true>(p, stream);
            case 8: return launch_prefill_simt<T, 8, true>(p, stream);
            default: break;
        }
    }
    if (epl <= 1) return launch_prefill_simt<T, 1, false>(p, stream);
    if (epl <= 2) return launch_prefill_simt<T, 2, false>(p, stream);
    if (epl <= 4) return launch_prefill_simt<T, 4, false>(p, stream);
    return launch_prefill_simt<T, 8, false>(p, stream);
}

template <typename T, int D>
cudaError_t launch_prefill_mma(const PrefillParams& p, cudaStream_t stream) {
    DeviceInfo* dev = nullptr;
    cudaError_t e = device_info(&dev);
    if (e != cudaSuccess) return e;
    const size_t smem = PrefillGeom<D>::kSmemBytes;
    int per_sm = 0;   // the first call also raises the kernel's dynamic shared-memory limit
    e = resident_ctas(gqa_prefill_mma_kernel<T, D>, kPfWarps * 32, smem, dev->max_smem_optin, &per_sm);
    if (e != cudaSuccess) return e;
    const dim3 grid((unsigned)((p.tq + kPfBM - 1) / kPfBM), (unsigned)p.q_heads, (unsigned)p.batch);
    gqa_prefill_mma_kernel<T, D><<<grid, kPfWarps * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

// Status word of the tcgen05 prefill kernel: 0 ok, 2 = an mbarrier wait ran out, 3 = the
// dynamic shared memory base was not 1024-byte aligned.  Read with gqa_b200_prefill_tc_status.
static __device__ int g_prefill_tc_status;
static int* g_prefill_tc_status_ptr[kMaxDevices];
static std::mutex g_prefill_tc_status_mutex;

cudaError_t prefill_tc_status_address(int** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_prefill_tc_status_mutex);
    if (!g_prefill_tc_status_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_prefill_tc_status);
        if (e != cudaSuccess) return e;
        g_prefill_tc_status_ptr[dev] = static_cast<int*>(ptr);
    }
    *out = g_prefill_tc_status_ptr[dev];
    return cudaSuccess;
}

template <typename T, int D>
cudaError_t launch_prefill_pp(const PrefillParams& p, cudaStream_t stream) {
    DeviceInfo* dev = nullptr;
    cudaError_t e = device_info(&dev);
    if (e != cudaSuccess) return e;
    const size_t smem = PrefillPpGeom<D>::kSmemBytes;
    int per_sm = 0;   // the first call also raises the kernel's dynamic shared-memory limit
    e = resident_ctas(gqa_prefill_pp_kernel<T, D>, kPpThreads, smem, dev->max_smem_optin, &per_sm);
    if (e != cudaSuccess) return e;
    int* status = nullptr;
    e = prefill_tc_status_address(&status);
    if (e != cudaSuccess) return e;
    const long long items = (long long)((p.tq + 2 * kPpBM - 1) / (2 * kPpBM)) * p.q_heads * p.batch;
    const unsigned grid = (unsigned)(items < dev->sm_count ? items : dev->sm_count);   // persistent: one CTA per SM
    gqa_prefill_pp_kernel<T, D><<<grid, kPpThreads, smem, stream>>>(p, status);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_prefill_t(const PrefillParams& p, bool use_mma, bool use_tc, cudaStream_t stream) {
    if (use_tc) {
        if constexpr (sizeof(T) == 2) {
            if (p.head_dim == 64) return launch_prefill_pp<T, 64>(p, stream);
            return launch_prefill_pp<T, 128>(p, stream);
        } else {
            return cudaErrorInvalidValue;
        }
    }
    if (use_mma) {
        if constexpr (sizeof(T) == 2) {
            if (p.head_dim == 64) return launch_prefill_mma<T, 64>(p, stream);
            return launch_prefill_mma<T, 128>(p, stream);
        } else {
            return cudaErrorInvalidValue;
        }
    }
    return launch_prefill_simt_for_dim<T>(p, stream);
}

}  // namespace

extern "C" {

int gqa_b200_prefill(const void* q, const void* k, const void* v, const int32_t* q_lens,
                     const int32_t* kv_lens, void* out, int dtype, int batch, int tq, int tk,
                     int q_heads, int kv_heads, int head_dim, float scale, int causal, int kernel,
                     void* stream) {
    if (dtype != GQA_B200_F32 && dtype != GQA_B200_F16 && dtype != GQA_B200_BF16)
        return GQA_B200_ERR_DTYPE;
    if (batch < 0 || tq < 0 || tk < 0) return GQA_B200_ERR_BATCH;
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return GQA_B200_ERR_HEADS;
    if (head_dim <= 0 || head_dim > 256) return GQA_B200_ERR_HEAD_DIM;
    if (!(std::isfinite(scale) && scale > 0.f)) return GQA_B200_ERR_SCALE;
    if (batch > 65535 || q_heads > 65535) return GQA_B200_ERR_INT32_RANGE;
    if (kernel != GQA_B200_KERNEL_AUTO && kernel != GQA_B200_KERNEL_SIMT &&
        kernel != GQA_B200_KERNEL_MMA && kernel != GQA_B200_KERNEL_TCGEN05)
        return GQA_B200_ERR_KERNEL;
    if (batch == 0 || tq == 0) return GQA_B200_OK;
    if (!q || !out || !q_lens || !kv_lens || (tk > 0 && (!k || !v))) return GQA_B200_ERR_NULL_POINTER;
    PrefillParams p{};
    p.q = q; p.k = k; p.v = v; p.out = out; p.q_lens = q_lens; p.kv_lens = kv_lens;
    p.batch = batch; p.tq = tq; p.tk = tk; p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.group = q_heads / kv_heads; p.head_dim = head_dim; p.causal = causal ? 1 : 0;
    p.scale_log2 = scale * kLog2e;
    bool use_mma = dtype != GQA_B200_F32 && (head_dim == 64 || head_dim == 128) && aligned16(q) &&
                   aligned16(k) && aligned16(v) && aligned16(out);
    if ((kernel == GQA_B200_KERNEL_MMA || kernel == GQA_B200_KERNEL_TCGEN05) && !use_mma)
        return GQA_B200_ERR_KERNEL;
    if (kernel == GQA_B200_KERNEL_SIMT) use_mma = false;
    // the tcgen05 kernel covers the same shapes as the mma.sync one
    const bool use_tc = use_mma && (kernel == GQA_B200_KERNEL_TCGEN05 ||
                                    (kernel == GQA_B200_KERNEL_AUTO && kPrefillAutoPicksTcgen05));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (dtype) {
        case GQA_B200_F32:  e = launch_prefill_t<float>(p, use_mma, use_tc, s); break;
        case GQA_B200_F16:  e = launch_prefill_t<__half>(p, use_mma, use_tc, s); break;
        default:            e = launch_prefill_t<__nv_bfloat16>(p, use_mma, use_tc, s); break;
    }
    return (int)e;
}

int gqa_b200_prefill_tc_status(int reset) {
    int* status = nullptr;
    cudaError_t e = prefill_tc_status_address(&status);
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

int gqa_b200_kv_append(const void* key, const void* value, void* k_cache, void* v_cache,
                       const int32_t* block_table, const int32_t* positions, int dtype, int batch,
                       int kv_heads, int head_dim, int64_t num_blocks, int block_size,
                       int max_pages, void* stream) {
    if (dtype != GQA_B200_F32 && dtype != GQA_B200_F16 && dtype != GQA_B200_BF16)
        return GQA_B200_ERR_DTYPE;
    if (batch < 0) return GQA_B200_ERR_BATCH;
    if (kv_heads <= 0) return GQA_B200_ERR_HEADS;
    if (head_dim <= 0) return GQA_B200_ERR_HEAD_DIM;
    if (num_blocks <= 0 || block_size <= 0) return GQA_B200_ERR_CACHE_SHAPE;
    if (max_pages <= 0) return GQA_B200_ERR_MAX_PAGES;
    if (num_blocks > std::numeric_limits<int>::max()) return GQA_B200_ERR_INT32_RANGE;
    if (batch == 0) return GQA_B200_OK;
    if (!key || !value || !k_cache || !v_cache || !block_table || !positions)
        return GQA_B200_ERR_NULL_POINTER;
    AppendParams a{};
    a.key = key; a.value = value; a.k_cache = k_cache; a.v_cache = v_cache;
    a.table = block_table; a.positions = positions;
    a.row_bytes = (long long)kv_heads * head_dim * elem_size(dtype);
    a.block_size = block_size; a.max_pages = max_pages; a.num_blocks = num_blocks;
    const long long cap = (long long)max_pages * block_size;
    a.cap_tokens = cap > 0x7fffffffll ? 0x7fffffff : (int)cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = a.row_bytes % 16 == 0 && aligned16(key) && aligned16(value) &&
                     aligned16(k_cache) && aligned16(v_cache);
    if (vec) kv_append_kernel<uint4><<<batch, kAppendThreads, 0, s>>>(a);
    else if (elem_size(dtype) == 4) kv_append_kernel<uint32_t><<<batch, kAppendThreads, 0, s>>>(a);
    else kv_append_kernel<uint16_t><<<batch, kAppendThreads, 0, s>>>(a);
    return (int)cudaGetLastError();
}

}  // extern "C"

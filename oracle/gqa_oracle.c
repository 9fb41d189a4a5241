/*
 * CPU oracle for paged grouped-query decode attention -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain C / OpenMP restatement of the reference library's slow oracle
 * (attention/reference/gqa.py:21-44): for every sequence b and query head h
 *   1. gather the first context_lens[b] tokens of kv head h / (Hq/Hkv) through
 *      block_table[b, :]                          (gqa.py:34-39)
 *   2. scores = <q, k_t> * scale in fp32          (gqa.py:40)
 *   3. weights = softmax(scores) (dense, not streaming: max, exp, sum, divide)
 *                                                 (gqa.py:41)
 *   4. out = sum_t weights[t] * v_t, rounded once to the input dtype
 *                                                 (gqa.py:42-43)
 * A sequence of length 0 produces zeros (gqa.py:31-33).  Table slots past the
 * used pages are never read (they may hold -1).
 *
 * The shipped library never links or calls this file.  It is the checker for
 * the tests and the smoke run, and the timed CPU baseline of the benchmark.
 * Its outputs are pinned against outputs of the reference itself (fixtures
 * under tests/golden/).
 *
 * dtype codes: 0 = float32, 1 = float16, 2 = bfloat16 (raw 16-bit storage).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) { /* round to nearest even */
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline void row_to_f32(const void* base, int64_t elem_off, int dtype, int d, float* dst) {
    if (dtype == 0) {
        memcpy(dst, (const float*)base + elem_off, (size_t)d * sizeof(float));
    } else if (dtype == 1) {
        const _Float16* p = (const _Float16*)base + elem_off;
        for (int i = 0; i < d; ++i) dst[i] = (float)p[i];
    } else {
        const uint16_t* p = (const uint16_t*)base + elem_off;
        for (int i = 0; i < d; ++i) dst[i] = bf16_to_f32(p[i]);
    }
}

static inline void store_row(void* base, int64_t elem_off, int dtype, int d, const float* src) {
    if (dtype == 0) {
        memcpy((float*)base + elem_off, src, (size_t)d * sizeof(float));
    } else if (dtype == 1) {
        _Float16* p = (_Float16*)base + elem_off;
        for (int i = 0; i < d; ++i) p[i] = (_Float16)src[i];
    } else {
        uint16_t* p = (uint16_t*)base + elem_off;
        for (int i = 0; i < d; ++i) p[i] = f32_to_bf16(src[i]);
    }
}

int gqa_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Returns 0 on success, 1 on bad arguments, 2 on allocation failure. */
int gqa_oracle_decode(const void* q, const void* k_cache, const void* v_cache,
                      const int32_t* block_table, const int32_t* context_lens, void* out,
                      int dtype, int batch, int q_heads, int kv_heads, int head_dim,
                      int64_t num_blocks, int block_size, int max_pages, float scale,
                      int threads) {
    if (dtype < 0 || dtype > 2 || batch < 0 || q_heads <= 0 || kv_heads <= 0 ||
        q_heads % kv_heads || head_dim <= 0 || head_dim > 4096 || block_size <= 0 ||
        max_pages <= 0 || num_blocks <= 0)
        return 1;
    const int group = q_heads / kv_heads;
    int max_len = 0;
    for (int b = 0; b < batch; ++b)
        if (context_lens[b] > max_len) max_len = context_lens[b];
    if ((int64_t)max_len > (int64_t)max_pages * block_size) return 1;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    threads = 1;
#endif
    int failed = 0;
    const int64_t tasks = (int64_t)batch * q_heads;
#pragma omp parallel num_threads(threads)
    {
        float* scores = (float*)malloc(((size_t)max_len + 1) * sizeof(float));
        float* qf = (float*)malloc((size_t)head_dim * sizeof(float));
        float* row = (float*)malloc((size_t)head_dim * sizeof(float));
        float* acc = (float*)malloc((size_t)head_dim * sizeof(float));
        if (!scores || !qf || !row || !acc) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp barrier
        if (!failed) {
#pragma omp for schedule(dynamic, 1)
            for (int64_t task = 0; task < tasks; ++task) {
                const int b = (int)(task / q_heads);
                const int h = (int)(task % q_heads);
                const int kvh = h / group;
                const int len = context_lens[b];
                const int64_t q_off = ((int64_t)b * q_heads + h) * head_dim;
                for (int i = 0; i < head_dim; ++i) acc[i] = 0.f;
                if (len > 0) {
                    row_to_f32(q, q_off, dtype, head_dim, qf);
                    const int32_t* pages = block_table + (int64_t)b * max_pages;
                    float mx = -INFINITY;
                    for (int t = 0; t < len; ++t) {
                        const int64_t phys = pages[t / block_size];
                        const int64_t off =
                            ((phys * block_size + t % block_size) * kv_heads + kvh) * head_dim;
                        row_to_f32(k_cache, off, dtype, head_dim, row);
                        float dot = 0.f;
                        for (int i = 0; i < head_dim; ++i) dot += qf[i] * row[i];
                        dot *= scale;
                        scores[t] = dot;
                        if (dot > mx) mx = dot;
                    }
                    float sum = 0.f;
                    for (int t = 0; t < len; ++t) {
                        scores[t] = expf(scores[t] - mx);
                        sum += scores[t];
                    }
                    const float inv = 1.f / sum;
                    for (int t = 0; t < len; ++t) {
                        const int64_t phys = pages[t / block_size];
                        const int64_t off =
                            ((phys * block_size + t % block_size) * kv_heads + kvh) * head_dim;
                        row_to_f32(v_cache, off, dtype, head_dim, row);
                        const float w = scores[t] * inv;
                        for (int i = 0; i < head_dim; ++i) acc[i] += w * row[i];
                    }
                }
                store_row(out, q_off, dtype, head_dim, acc);
            }
        }
        free(scores);
        free(qf);
        free(row);
        free(acc);
    }
    return failed ? 2 : 0;
}

/*
 * CPU oracle for the vkop post-processing path (Softmax + TopK, NMS).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker: the parity tests, the
 * smoke check and the CPU-baseline leg of the benchmark call it.  Nothing in
 * the shipped library links it or falls back to it.
 *
 * It is a plain-C restatement of the arithmetic the reference performs on
 * this path (reference paths are relative to the junka/vkop tree):
 *   - core/function.cpp:150-183  Function::get_top_k_predictions
 *                                (max -> exp(x-max) -> sequential sum ->
 *                                 divide -> sort by probability, truncate to k)
 *   - tests/SoftmaxTest.cpp:34-97 softmax_nd (max from -INFINITY, sequential sum)
 *   - shaders/softmax2.comp:50-117 row softmax: exp(x-max)/sum with a true division
 *   - shaders/topk.comp:110-175   value-descending selection of k (value,index) pairs
 *   - shaders/nms.comp:47-68      to_corners / compute_iou (operand order, early-out,
 *                                 union > 0, true division)
 *   - shaders/nms.comp:85-195     score filter (strict >), score-descending greedy sweep,
 *                                 max_output_boxes_per_class cut-off, (batch,class,box) rows
 *   - tests/NmsTest.cpp:66-176    the reference's in-test greedy NMS (second statement of
 *                                 the same sweep)
 *
 * Where the reference leaves the order of equal values unspecified (std::sort
 * with a value-only comparator, the bitonic network of topk.comp, the
 * selection sort of nms.comp) the oracle fixes the ONNX rule: value
 * descending, then index ascending.  -0.0 and +0.0 compare equal; NaN sorts
 * above +inf (torch ordering).
 *
 * Parity pin: the reference ships no golden vectors for this path.  Its tests
 * compute expectations with libtorch at run time (tests/TopkTest.cpp:71-75,
 * tests/SoftmaxTest.cpp:118-138).  This oracle is pinned against torch-CPU
 * outputs generated with the reference's own seeds and shapes and committed as
 * fixtures (tests/golden), and against the reference's in-test NMS algorithm.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/build.py).
 * -ffp-contract=off keeps every multiply and add separately rounded, as the
 * restated formulas are written.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_BF16 = 2 };
enum { ORACLE_SUM_F32_SEQUENTIAL = 0, ORACLE_SUM_F64 = 1 };
enum { ORACLE_VALUE_PROBABILITY = 0, ORACLE_VALUE_RAW = 1 };

/* ---- storage formats -> fp32 (exact) ---- */

static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static float bf16_bits_to_float(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline float load_elem(const void *base, int dtype, int64_t i) {
    switch (dtype) {
    case ORACLE_F16:
        return half_bits_to_float(((const uint16_t *)base)[i]);
    case ORACLE_BF16:
        return bf16_bits_to_float(((const uint16_t *)base)[i]);
    default:
        return ((const float *)base)[i];
    }
}

/* Order-preserving map float -> uint32: a > b  <=>  key(a) > key(b), with
 * -0 == +0 and every NaN mapped to the single largest key. */
static inline uint32_t order_key(float x) {
    if (x != x)
        return 0xFFFFFFFFu;
    if (x == 0.0f)
        return 0x80000000u;
    uint32_t u;
    memcpy(&u, &x, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

typedef struct {
    uint32_t key;
    uint32_t idx;
} cand_t;

/* value descending, index ascending (ONNX TopK) */
static int cand_cmp_desc(const void *a, const void *b) {
    const cand_t *x = (const cand_t *)a, *y = (const cand_t *)b;
    if (x->key != y->key)
        return x->key > y->key ? -1 : 1;
    if (x->idx != y->idx)
        return x->idx < y->idx ? -1 : 1;
    return 0;
}

/* value ascending, index ascending (ONNX TopK, largest = 0) */
static int cand_cmp_asc(const void *a, const void *b) {
    const cand_t *x = (const cand_t *)a, *y = (const cand_t *)b;
    if (x->key != y->key)
        return x->key < y->key ? -1 : 1;
    if (x->idx != y->idx)
        return x->idx < y->idx ? -1 : 1;
    return 0;
}

static inline int cand_before(cand_t a, cand_t b) { /* a ranks ahead of b (descending) */
    return a.key > b.key || (a.key == b.key && a.idx < b.idx);
}

/* Select the k best of n candidates, sorted.  full_sort = 1 sorts everything
 * the way core/function.cpp:173-181 does; full_sort = 0 keeps a k-sized
 * min-heap (same result, used where the tests need speed). */
static void select_topk_desc(cand_t *c, int64_t n, int k, int full_sort, cand_t *out) {
    if (full_sort || n <= 4 * (int64_t)k) {
        qsort(c, (size_t)n, sizeof(cand_t), cand_cmp_desc);
        memcpy(out, c, (size_t)k * sizeof(cand_t));
        return;
    }
    /* heap[0] is the worst of the current best k */
    cand_t *h = out;
    int hn = 0;
    for (int64_t i = 0; i < n; i++) {
        cand_t v = c[i];
        if (hn < k) {
            int j = hn++;
            h[j] = v;
            while (j > 0) {
                int p = (j - 1) / 2;
                if (cand_before(h[p], h[j])) {
                    cand_t t = h[p];
                    h[p] = h[j];
                    h[j] = t;
                    j = p;
                } else
                    break;
            }
        } else if (cand_before(v, h[0])) {
            int j = 0;
            h[0] = v;
            for (;;) {
                int l = 2 * j + 1, r = l + 1, w = j;
                if (l < hn && cand_before(h[w], h[l]))
                    w = l;
                if (r < hn && cand_before(h[w], h[r]))
                    w = r;
                if (w == j)
                    break;
                cand_t t = h[w];
                h[w] = h[j];
                h[j] = t;
                j = w;
            }
        }
    }
    qsort(h, (size_t)k, sizeof(cand_t), cand_cmp_desc);
}

/* ------------------------------------------------------------------------- */
/* Softmax statistics of one row: m = max z, sum = sum exp(z - m), z = x*invT.
 * core/function.cpp:154-160 (max_element, then exp and a running float sum);
 * sum_mode F64 is the tolerance referee (same terms, double accumulation). */
static void row_softmax_stats(const void *row, int dtype, int64_t cols, float inv_t, int sum_mode,
                              float *m_out, double *sum_out) {
    float m = -INFINITY;
    for (int64_t i = 0; i < cols; i++) {
        float z = load_elem(row, dtype, i) * inv_t;
        if (z > m)
            m = z;
    }
    if (sum_mode == ORACLE_SUM_F64) {
        double s = 0.0;
        for (int64_t i = 0; i < cols; i++) {
            float z = load_elem(row, dtype, i) * inv_t;
            s += exp((double)z - (double)m);
        }
        *sum_out = s;
    } else {
        float s = 0.0f;
        for (int64_t i = 0; i < cols; i++) {
            float z = load_elem(row, dtype, i) * inv_t;
            s += expf(z - m);
        }
        *sum_out = (double)s;
    }
    *m_out = m;
}

static inline float prob_of(float x, float inv_t, float m, double sum, int sum_mode) {
    float z = x * inv_t;
    if (sum_mode == ORACLE_SUM_F64)
        return (float)(exp((double)z - (double)m) / sum);
    return expf(z - m) / (float)sum; /* core/function.cpp:162-164, softmax2.comp:115 */
}

/* Fused Softmax + TopK over [rows, cols] (row stride in elements).
 * Selection is on the stored logit (value descending, index ascending);
 * values are softmax probabilities of z = x * inv_temperature, or the raw
 * logit.  out_values: float [rows,k]; out_indices: int64 [rows,k].
 * Returns 0, or -1 on a bad argument. */
int oracle_softmax_topk(const void *logits, int dtype, int64_t rows, int64_t cols, int64_t row_stride,
                        int k, float inv_temperature, int value_kind, int sum_mode, int full_sort,
                        float *out_values, int64_t *out_indices) {
    if (!logits || rows < 0 || cols <= 0 || k <= 0 || k > cols || row_stride < cols)
        return -1;
    size_t esz = dtype == ORACLE_F32 ? 4 : 2;
    int status = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t r = 0; r < rows; r++) {
        const void *row = (const char *)logits + (size_t)r * (size_t)row_stride * esz;
        cand_t *c = (cand_t *)malloc((size_t)cols * sizeof(cand_t));
        cand_t *best = (cand_t *)malloc((size_t)k * sizeof(cand_t));
        if (!c || !best) {
            status = -1;
            free(c);
            free(best);
            continue;
        }
        for (int64_t i = 0; i < cols; i++) {
            c[i].key = order_key(load_elem(row, dtype, i));
            c[i].idx = (uint32_t)i;
        }
        select_topk_desc(c, cols, k, full_sort, best);
        float m = 0.0f;
        double sum = 1.0;
        if (value_kind == ORACLE_VALUE_PROBABILITY)
            row_softmax_stats(row, dtype, cols, inv_temperature, sum_mode, &m, &sum);
        for (int j = 0; j < k; j++) {
            float x = load_elem(row, dtype, best[j].idx);
            out_indices[r * k + j] = best[j].idx;
            out_values[r * k + j] =
                value_kind == ORACLE_VALUE_PROBABILITY ? prob_of(x, inv_temperature, m, sum, sum_mode) : x;
        }
        free(c);
        free(best);
    }
    return status;
}

/* Full softmax along the middle axis of a row-major [outer, axis_len, inner]
 * view (inner = 1 for the 2-D post-processing case; the 4-D cases of
 * tests/SoftmaxTest.cpp:195-201 map to outer/axis/inner products).
 * out: float, same shape. */
int oracle_softmax(const void *x, int dtype, int64_t outer, int64_t axis_len, int64_t inner,
                   float inv_temperature, int sum_mode, float *out) {
    if (!x || !out || outer < 0 || axis_len <= 0 || inner <= 0)
        return -1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t o = 0; o < outer; o++) {
        for (int64_t in = 0; in < inner; in++) {
            int64_t base = o * axis_len * inner + in;
            float m = -INFINITY;
            for (int64_t a = 0; a < axis_len; a++) {
                float z = load_elem(x, dtype, base + a * inner) * inv_temperature;
                if (z > m)
                    m = z;
            }
            if (sum_mode == ORACLE_SUM_F64) {
                double s = 0.0;
                for (int64_t a = 0; a < axis_len; a++)
                    s += exp((double)(load_elem(x, dtype, base + a * inner) * inv_temperature) - (double)m);
                for (int64_t a = 0; a < axis_len; a++)
                    out[base + a * inner] =
                        (float)(exp((double)(load_elem(x, dtype, base + a * inner) * inv_temperature) - (double)m) / s);
            } else {
                float s = 0.0f;
                for (int64_t a = 0; a < axis_len; a++)
                    s += expf(load_elem(x, dtype, base + a * inner) * inv_temperature - m);
                for (int64_t a = 0; a < axis_len; a++)
                    out[base + a * inner] = expf(load_elem(x, dtype, base + a * inner) * inv_temperature - m) / s;
            }
        }
    }
    return 0;
}

/* Standalone TopK along the middle axis of [outer, axis_len, inner]
 * (ops/Topk.hpp:62-79 attributes k / largest / sorted / axis).  Values are
 * copies of the input (as float).  Unsorted output (sorted = 0) is returned in
 * ascending index order.  out_*: [outer, k, inner]. */
int oracle_topk(const void *x, int dtype, int64_t outer, int64_t axis_len, int64_t inner, int k, int largest,
                int sorted, float *out_values, int64_t *out_indices) {
    if (!x || outer < 0 || axis_len <= 0 || inner <= 0 || k <= 0 || k > axis_len)
        return -1;
    int status = 0;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t o = 0; o < outer; o++) {
        for (int64_t in = 0; in < inner; in++) {
            cand_t *c = (cand_t *)malloc((size_t)axis_len * sizeof(cand_t));
            if (!c) {
                status = -1;
                continue;
            }
            int64_t base = o * axis_len * inner + in;
            for (int64_t a = 0; a < axis_len; a++) {
                c[a].key = order_key(load_elem(x, dtype, base + a * inner));
                c[a].idx = (uint32_t)a;
            }
            qsort(c, (size_t)axis_len, sizeof(cand_t), largest ? cand_cmp_desc : cand_cmp_asc);
            if (!sorted) { /* index order among the selected k */
                for (int i = 1; i < k; i++) {
                    cand_t v = c[i];
                    int j = i - 1;
                    while (j >= 0 && c[j].idx > v.idx) {
                        c[j + 1] = c[j];
                        j--;
                    }
                    c[j + 1] = v;
                }
            }
            for (int j = 0; j < k; j++) {
                int64_t o_idx = (o * k + j) * inner + in;
                out_indices[o_idx] = c[j].idx;
                out_values[o_idx] = load_elem(x, dtype, base + (int64_t)c[j].idx * inner);
            }
            free(c);
        }
    }
    return status;
}

/* ---- vocab-sharded form: per-shard packet, then merge ------------------- */

/* Per-shard partial of one row: m = max z over the shard, s = sum exp(z - m)
 * (float, pairwise-free sequential sum in double to serve as referee), and the
 * shard's k best (key, global index).  Used to check the multi-GPU exchange:
 * merging the packets of all shards must reproduce oracle_softmax_topk. */
int oracle_shard_packet(const void *shard_logits, int dtype, int64_t rows, int64_t shard_cols, int64_t row_stride,
                        int64_t index_offset, int k, float inv_temperature, float *out_m, double *out_s,
                        uint32_t *out_keys, int64_t *out_idx, int32_t *out_count) {
    if (!shard_logits || rows < 0 || shard_cols <= 0 || k <= 0)
        return -1;
    size_t esz = dtype == ORACLE_F32 ? 4 : 2;
    for (int64_t r = 0; r < rows; r++) {
        const void *row = (const char *)shard_logits + (size_t)r * (size_t)row_stride * esz;
        cand_t *c = (cand_t *)malloc((size_t)shard_cols * sizeof(cand_t));
        if (!c)
            return -1;
        for (int64_t i = 0; i < shard_cols; i++) {
            c[i].key = order_key(load_elem(row, dtype, i));
            c[i].idx = (uint32_t)i;
        }
        qsort(c, (size_t)shard_cols, sizeof(cand_t), cand_cmp_desc);
        int cnt = k < shard_cols ? k : (int)shard_cols;
        for (int j = 0; j < k; j++) {
            out_keys[r * k + j] = j < cnt ? c[j].key : 0u;
            out_idx[r * k + j] = j < cnt ? index_offset + c[j].idx : -1;
        }
        out_count[r] = cnt;
        row_softmax_stats(row, dtype, shard_cols, inv_temperature, ORACLE_SUM_F64, &out_m[r], &out_s[r]);
        free(c);
    }
    return 0;
}

/* Merge of G shard statistics: M = max m_g, S = sum s_g * exp(m_g - M). */
void oracle_merge_stats(const float *m, const double *s, int g, float *m_out, double *s_out) {
    float M = -INFINITY;
    for (int i = 0; i < g; i++)
        if (m[i] > M)
            M = m[i];
    double S = 0.0;
    for (int i = 0; i < g; i++)
        if (s[i] > 0.0)
            S += s[i] * exp((double)m[i] - (double)M);
    *m_out = M;
    *s_out = S;
}

/* ------------------------------------------------------------------------- */
/* NMS */

typedef struct {
    float x1, y1, x2, y2;
} box_t;

/* shaders/nms.comp:47-55.  w*0.5 is exact in binary floating point. */
static box_t to_corners(const float *b, int center_point_box) {
    box_t r;
    if (!center_point_box) {
        r.x1 = b[0];
        r.y1 = b[1];
        r.x2 = b[2];
        r.y2 = b[3];
    } else {
        float xc = b[0], yc = b[1], w = b[2], h = b[3];
        r.x1 = xc - w * 0.5f;
        r.y1 = yc - h * 0.5f;
        r.x2 = xc + w * 0.5f;
        r.y2 = yc + h * 0.5f;
    }
    return r;
}

/* shaders/nms.comp:57-68: a = the later (lower-score) box, b = the kept box. */
static float compute_iou(box_t a, box_t b) {
    float x1 = a.x1 > b.x1 ? a.x1 : b.x1;
    float y1 = a.y1 > b.y1 ? a.y1 : b.y1;
    float x2 = a.x2 < b.x2 ? a.x2 : b.x2;
    float y2 = a.y2 < b.y2 ? a.y2 : b.y2;
    if (x2 <= x1 || y2 <= y1)
        return 0.0f;
    float inter = (x2 - x1) * (y2 - y1);
    float area_a = (a.x2 - a.x1) * (a.y2 - a.y1);
    float area_b = (b.x2 - b.x1) * (b.y2 - b.y1);
    float union_area = area_a + area_b - inter;
    return union_area > 0.0f ? inter / union_area : 0.0f;
}

/* Per-(batch, class) greedy NMS, ONNX NonMaxSuppression semantics with the
 * reference shader's arithmetic.
 *   boxes  [B, N, 4] float, scores [B, C, N] float (ops/Nms.hpp:69-75)
 *   candidates: score > score_threshold (strict; shaders/nms.comp:89)
 *   order: score descending, index ascending
 *   pre_topk > 0: only the best pre_topk candidates enter the sweep
 *   sweep: shaders/nms.comp:153-185; stops at max_output_boxes_per_class (> 0)
 * Output rows (batch, class, box) in (batch, class, rank) order, at most
 * capacity_rows written; *out_count = rows produced (may exceed capacity).
 * per_problem_count (nullable): kept boxes of each (b,c). */
int oracle_nms(const float *boxes, const float *scores, int B, int C, int N, int center_point_box,
               int max_output_boxes_per_class, float iou_threshold, float score_threshold, int pre_topk,
               int32_t *out_rows, int64_t capacity_rows, int64_t *out_count, int32_t *per_problem_count) {
    if (!boxes || !scores || B < 0 || C < 0 || N < 0)
        return -1;
    int64_t problems = (int64_t)B * C;
    int32_t *kept = (int32_t *)malloc((size_t)(problems * (N > 0 ? N : 1)) * sizeof(int32_t));
    int32_t *cnt = (int32_t *)calloc((size_t)(problems > 0 ? problems : 1), sizeof(int32_t));
    if (!kept || !cnt) {
        free(kept);
        free(cnt);
        return -1;
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t p = 0; p < problems; p++) {
        int b = (int)(p / C);
        const float *s = scores + p * N;
        const float *bx = boxes + (int64_t)b * N * 4;
        cand_t *c = (cand_t *)malloc((size_t)(N > 0 ? N : 1) * sizeof(cand_t));
        int n = 0;
        for (int i = 0; i < N; i++) {
            if (s[i] > score_threshold) {
                c[n].key = order_key(s[i]);
                c[n].idx = (uint32_t)i;
                n++;
            }
        }
        qsort(c, (size_t)n, sizeof(cand_t), cand_cmp_desc);
        if (pre_topk > 0 && n > pre_topk)
            n = pre_topk;
        box_t *cb = (box_t *)malloc((size_t)(n > 0 ? n : 1) * sizeof(box_t));
        unsigned char *dead = (unsigned char *)calloc((size_t)(n > 0 ? n : 1), 1);
        for (int i = 0; i < n; i++)
            cb[i] = to_corners(bx + (int64_t)c[i].idx * 4, center_point_box);
        int max_out = n;
        if (max_output_boxes_per_class > 0 && max_output_boxes_per_class < n)
            max_out = max_output_boxes_per_class;
        int sel = 0;
        for (int i = 0; i < n && sel < max_out; i++) {
            if (dead[i])
                continue;
            kept[p * N + sel++] = (int32_t)c[i].idx;
            for (int j = i + 1; j < n; j++)
                if (!dead[j] && compute_iou(cb[j], cb[i]) > iou_threshold)
                    dead[j] = 1;
        }
        cnt[p] = sel;
        free(c);
        free(cb);
        free(dead);
    }
    int64_t total = 0;
    for (int64_t p = 0; p < problems; p++) {
        for (int j = 0; j < cnt[p]; j++) {
            if (out_rows && total < capacity_rows) {
                out_rows[total * 3 + 0] = (int32_t)(p / C);
                out_rows[total * 3 + 1] = (int32_t)(p % C);
                out_rows[total * 3 + 2] = kept[p * N + j];
            }
            total++;
        }
        if (per_problem_count)
            per_problem_count[p] = cnt[p];
    }
    if (out_count)
        *out_count = total;
    free(kept);
    free(cnt);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Reference-emulation variants: they restate what the shaders do, including
 * behaviour the canonical contract above deliberately does not follow, so the
 * tests can list where the two differ. */

/* shaders/topk.comp:46-78,110-175 with the host loop of ops/Topk.hpp:179-217:
 * repeated passes over 256-wide blocks, each block bitonic-sorted descending
 * on the value alone (strict compare, so equal values keep network order),
 * padded with (-3.4e38, -1), the first min(k, block_count) pairs of each block
 * feeding the next pass.  One fp32 row.  Slots the shader leaves unwritten
 * when a trailing block holds fewer than k elements are filled here with the
 * padding pair (the shader leaves them uninitialised). */
int oracle_ref_topk_bitonic(const float *row, int n, int k, float *out_values, int32_t *out_indices) {
    if (!row || n <= 0 || k <= 0 || k >= 256)
        return -1;
    int cap = n > 256 ? n : 256;
    float *v0 = (float *)malloc((size_t)cap * sizeof(float)), *v1 = (float *)malloc((size_t)cap * sizeof(float));
    int32_t *i0 = (int32_t *)malloc((size_t)cap * sizeof(int32_t)), *i1 = (int32_t *)malloc((size_t)cap * sizeof(int32_t));
    if (!v0 || !v1 || !i0 || !i1)
        return -1;
    for (int i = 0; i < n; i++) {
        v0[i] = row[i];
        i0[i] = i;
    }
    int width = n;
    for (;;) {
        int blocks = (width + 255) / 256;
        for (int g = 0; g < blocks; g++) {
            float sv[256];
            int32_t si[256];
            int local = width - g * 256 < 256 ? width - g * 256 : 256;
            for (int t = 0; t < 256; t++) {
                if (t < local) {
                    sv[t] = v0[g * 256 + t];
                    si[t] = i0[g * 256 + t];
                } else {
                    sv[t] = -3.4e38f;
                    si[t] = -1;
                }
            }
            int pow2 = 1; /* topk.comp:47-50: the network spans the next power of two >= count */
            while (pow2 < local && pow2 < 512)
                pow2 <<= 1;
            for (int size = 2; size <= pow2; size <<= 1) {
                for (int stride = size >> 1; stride > 0; stride >>= 1) {
                    for (int t = 0; t < pow2; t++) {
                        int partner = t ^ stride;
                        if (partner > t) {
                            int descending = (t & size) == 0;
                            int swap = descending ? (sv[t] < sv[partner]) : (sv[t] > sv[partner]);
                            if (swap) {
                                float tv = sv[t];
                                sv[t] = sv[partner];
                                sv[partner] = tv;
                                int32_t ti = si[t];
                                si[t] = si[partner];
                                si[partner] = ti;
                            }
                        }
                    }
                }
            }
            for (int j = 0; j < k; j++) {
                if (j < local) {
                    v1[g * k + j] = sv[j];
                    i1[g * k + j] = si[j];
                } else {
                    v1[g * k + j] = -3.4e38f;
                    i1[g * k + j] = -1;
                }
            }
        }
        float *tv = v0;
        v0 = v1;
        v1 = tv;
        int32_t *ti = i0;
        i0 = i1;
        i1 = ti;
        if (width <= 256)
            break;
        width = k * blocks;
    }
    for (int j = 0; j < k; j++) {
        out_values[j] = v0[j];
        out_indices[j] = i0[j];
    }
    free(v0);
    free(v1);
    free(i0);
    free(i1);
    return 0;
}

/* shaders/softmax2.comp:50-117 summation shape for one fp32 row: 256 strided
 * per-thread partials, each group of 32 lanes added together, then the 8
 * group sums added serially.  The order inside a subgroup add is
 * implementation-defined; a sequential lane order is used here, so this is
 * indicative and compared under tolerance only.  Running max starts at -1e9
 * as the shader does. */
int oracle_ref_softmax2_row(const float *row, int n, float *out) {
    if (!row || !out || n <= 0)
        return -1;
    float m = -1e9f;
    for (int i = 0; i < n; i++)
        if (row[i] > m)
            m = row[i];
    float part[256];
    for (int t = 0; t < 256; t++) {
        float s = 0.0f;
        for (int c = t; c < n; c += 256)
            s += expf(row[c] - m);
        part[t] = s;
    }
    float total = 0.0f;
    for (int g = 0; g < 8; g++) {
        float sg = 0.0f;
        for (int l = 0; l < 32; l++)
            sg += part[g * 32 + l];
        total += sg;
    }
    for (int i = 0; i < n; i++)
        out[i] = expf(row[i] - m) / total;
    return 0;
}

/* shaders/nms.comp:85-195 for one (batch, class): the first <= 1024 boxes in
 * index order with score > threshold, selection-sorted descending with a
 * strict compare, then the same greedy sweep.  Returns the kept count. */
int oracle_ref_nms_problem(const float *boxes_n4, const float *scores_n, int N, int center_point_box,
                           int max_output_boxes_per_class, float iou_threshold, float score_threshold,
                           int32_t *kept_out) {
    enum { MAXC = 1024 };
    static __thread box_t sb[MAXC];
    static __thread float ss[MAXC];
    static __thread int32_t si[MAXC];
    static __thread unsigned char act[MAXC];
    int count = 0;
    for (int i = 0; i < N && count < MAXC; i++) {
        if (scores_n[i] > score_threshold) {
            sb[count] = to_corners(boxes_n4 + (int64_t)i * 4, center_point_box);
            ss[count] = scores_n[i];
            si[count] = i;
            count++;
        }
    }
    for (int i = 0; i < count; i++) {
        int best = i;
        for (int j = i + 1; j < count; j++)
            if (ss[j] > ss[best])
                best = j;
        if (best != i) {
            float ts = ss[i];
            ss[i] = ss[best];
            ss[best] = ts;
            box_t tb = sb[i];
            sb[i] = sb[best];
            sb[best] = tb;
            int32_t ti = si[i];
            si[i] = si[best];
            si[best] = ti;
        }
    }
    for (int i = 0; i < count; i++)
        act[i] = 1;
    int max_out = count;
    if (max_output_boxes_per_class > 0 && max_output_boxes_per_class < count)
        max_out = max_output_boxes_per_class;
    int sel = 0;
    for (int i = 0; i < count && sel < max_out; i++) {
        if (!act[i])
            continue;
        kept_out[sel++] = si[i];
        for (int j = i + 1; j < count; j++)
            if (act[j] && compute_iou(sb[j], sb[i]) > iou_threshold)
                act[j] = 0;
    }
    return sel;
}

/* Sampling tail over the k survivors of one fused Softmax + TopK call (no counterpart in the
 * reference; it is the step that follows top-k in a vocabulary-selection path).  Per row, with the
 * probabilities p_0 >= p_1 >= ... as the operator emits them and all sums sequential in fp32:
 *   total = sum of all k;  n = the smallest count whose prefix sum reaches top_p * total (n = k when
 *   top_p >= 1);  mass = prefix sum of those n;  the choice is the first j < n whose prefix sum
 *   exceeds u * mass (j = n - 1 if none does).
 * out_choice[r] = j; out_token[r] = indices[r][j]. */
int oracle_sample_topk(const void *values, int dtype, const int64_t *indices, int64_t rows, int k, float top_p,
                       const float *u, int32_t *out_choice, int64_t *out_token) {
    if (!values || !indices || !u || !out_choice || !out_token || rows < 0 || k < 1 || !(top_p > 0.0f))
        return -1;
    for (int64_t r = 0; r < rows; r++) {
        float total = 0.0f;
        for (int j = 0; j < k; j++)
            total += load_elem(values, dtype, r * k + j);
        int n = k;
        if (top_p < 1.0f) {
            const float want = top_p * total;
            float acc = 0.0f;
            for (int j = 0; j < k; j++) {
                acc += load_elem(values, dtype, r * k + j);
                if (acc >= want) {
                    n = j + 1;
                    break;
                }
            }
        }
        float mass = 0.0f;
        for (int j = 0; j < n; j++)
            mass += load_elem(values, dtype, r * k + j);
        const float target = u[r] * mass;
        int pick = n - 1;
        float acc = 0.0f;
        for (int j = 0; j < n; j++) {
            acc += load_elem(values, dtype, r * k + j);
            if (acc > target) {
                pick = j;
                break;
            }
        }
        out_choice[r] = pick;
        out_token[r] = indices[r * k + pick];
    }
    return 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}

uint32_t oracle_order_key(float x) { return order_key(x); }

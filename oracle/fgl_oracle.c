/*
 * CPU oracle (plain C) for the FastGL per-mini-batch hot path.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA kernels are
 * compared with and the timed CPU baseline.  The shipped library never
 * links, loads or calls it.
 *
 * PARITY UNPINNED: the reference has no tests, golden vectors or CPU code
 * path; every function below restates the reference's CUDA kernels as a
 * sequential (thread 0, 1, 2 ... in order) execution, citing the lines it
 * follows.  It is cross-checked against the independent numpy restatement
 * in oracle_np.py and against the published Philox4x32-10 known answers.
 *
 *   fglo_sample          cuda_operators/sample.cu:17-38, 82-95
 *   fglo_map             cuda_operators/id_map.cu:179-255, 259-383
 *   fglo_cal_deg         cuda_operators/utilis.cu:43-79
 *   fglo_exclusive_sum   cuda_operators/utilis.cu:17-41
 *   fglo_agg_fwd         cuda_operators/aggregate_acc_kernel.cu:271-331, 376-427
 *   fglo_agg_bwd         cuda_operators/aggregate_acc_kernel.cu:468-517, 555-596
 *   fglo_agg_edge_fwd/bwd cuda_operators/aggregate_acc_kernel.cu:836-885, 925-979
 *
 * Loops over independent seeds / rows carry an OpenMP pragma so that the
 * CPU baseline can use all host cores; results do not depend on the thread
 * count (the id-mapping pass, whose result is order dependent, is serial).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FGLO_MODE_SUM 0
#define FGLO_MODE_MEAN 1
#define FGLO_MODE_SYMNORM 2

int fglo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void fglo_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---- Philox4x32-10 (Salmon, Moraes, Dror, Shaw; SC'11) ------------------ */
void fglo_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

static inline uint32_t fglo_draw(uint64_t rng_seed, uint64_t rng_ctr, uint32_t seed_slot, uint32_t pick_slot) {
    /* one block serves four picks: counter word 0 = pick_slot / 4, output word pick_slot % 4 */
    uint32_t ctr[4] = {pick_slot >> 2, seed_slot, (uint32_t)rng_ctr, (uint32_t)(rng_ctr >> 32)};
    uint32_t key[2] = {(uint32_t)rng_seed, (uint32_t)(rng_seed >> 32)};
    uint32_t out[4];
    fglo_philox4x32_10(ctr, key, out);
    return out[pick_slot & 3];
}

static inline uint32_t fglo_bounded(uint32_t r, uint32_t n) {
    return (uint32_t)(((uint64_t)r * n) >> 32);
}

/* ---- a1: sampling (sample.cu:17-38 counts + scan, :82-95 copy / random) -- */
int64_t fglo_sample(const int64_t* indptr, const int32_t* indices, const int32_t* seeds, int32_t n_seeds,
                    int32_t fanout, int replace, uint64_t rng_seed, uint64_t rng_ctr,
                    int32_t* out_indptr, int32_t* out_src, int32_t* out_dst) {
    out_indptr[0] = 0;
    for (int32_t s = 0; s < n_seeds; ++s) { /* sample.cu:17-38 and the scan at :155-159 */
        int64_t deg = indptr[seeds[s] + 1] - indptr[seeds[s]];
        out_indptr[s + 1] = out_indptr[s] + (int32_t)(deg < fanout ? deg : fanout);
    }
#pragma omp parallel for schedule(dynamic, 256)
    for (int32_t s = 0; s < n_seeds; ++s) {
        const int32_t v = seeds[s];
        const int64_t start = indptr[v];
        const int64_t deg = indptr[v + 1] - start;
        const int32_t off = out_indptr[s];
        if (deg <= fanout) { /* sample.cu:82-87 */
            for (int64_t i = 0; i < deg; ++i) {
                out_src[off + i] = indices[start + i];
                if (out_dst) out_dst[off + i] = v;
            }
        } else if (replace) { /* sample.cu:88-94 */
            for (int32_t i = 0; i < fanout; ++i) {
                uint32_t p = fglo_bounded(fglo_draw(rng_seed, rng_ctr, (uint32_t)s, (uint32_t)i), (uint32_t)deg);
                out_src[off + i] = indices[start + p];
                if (out_dst) out_dst[off + i] = v;
            }
        } else { /* uniform k-subset, Floyd's algorithm; picks kept in the output slots' order */
            uint32_t picks[1024];
            uint32_t* pk = fanout <= 1024 ? picks : (uint32_t*)malloc(sizeof(uint32_t) * (size_t)fanout);
            for (int32_t i = 0; i < fanout; ++i) {
                uint32_t j = (uint32_t)(deg - fanout + i);
                uint32_t t = fglo_bounded(fglo_draw(rng_seed, rng_ctr, (uint32_t)s, (uint32_t)i), j + 1u);
                int hit = 0;
                for (int32_t q = 0; q < i; ++q) hit |= (pk[q] == t);
                pk[i] = hit ? j : t;
                out_src[off + i] = indices[start + pk[i]];
                if (out_dst) out_dst[off + i] = v;
            }
            if (pk != picks) free(pk);
        }
    }
    return out_indptr[n_seeds];
}

/* ---- a2: id mapping (id_map.cu) ----------------------------------------- */
typedef struct { int32_t key; int32_t local; } fglo_slot;

static inline uint64_t fglo_pow2_at_least(uint64_t n) { uint64_t p = 16; while (p < n) p <<= 1; return p; }

static inline uint64_t fglo_find(fglo_slot* t, uint64_t mask, int32_t key) {
    uint64_t pos = ((uint64_t)(uint32_t)key * 0x9E3779B97F4A7C15ull >> 20) & mask;
    while (t[pos].key != -1 && t[pos].key != key) pos = (pos + 1) & mask;
    return pos;
}

/* src/dst are rewritten in place with local ids (id_map.cu:351-383); unique[] needs n_seeds + n_edges
 * entries.  Returns the number of unique nodes (seeds first, then new sources in first-occurrence order:
 * a sequential run of id_map.cu:290-322). */
int64_t fglo_map(int32_t* src, int32_t* dst, const int32_t* seeds, int32_t n_seeds, int64_t n_edges, int32_t* unique) {
    uint64_t size = fglo_pow2_at_least(2 * ((uint64_t)n_seeds + (uint64_t)n_edges) + 16);
    uint64_t mask = size - 1;
    fglo_slot* t = (fglo_slot*)malloc(size * sizeof(fglo_slot));
    memset(t, 0xFF, size * sizeof(fglo_slot));
    int64_t n_unique = 0;
    for (int32_t i = 0; i < n_seeds; ++i) { /* id_map.cu:259-287 */
        uint64_t pos = fglo_find(t, mask, seeds[i]);
        t[pos].key = seeds[i];
        t[pos].local = i;
        unique[n_unique++] = seeds[i];
    }
    for (int64_t e = 0; e < n_edges; ++e) { /* id_map.cu:290-349 */
        uint64_t pos = fglo_find(t, mask, src[e]);
        if (t[pos].key == -1) {
            t[pos].key = src[e];
            t[pos].local = (int32_t)n_unique;
            unique[n_unique++] = src[e];
        }
    }
    for (int64_t e = 0; e < n_edges; ++e) { /* id_map.cu:351-383 */
        src[e] = t[fglo_find(t, mask, src[e])].local;
        if (dst) dst[e] = t[fglo_find(t, mask, dst[e])].local;
    }
    free(t);
    return n_unique;
}

/* ---- a3: block CSR helpers (utilis.cu) ----------------------------------- */
void fglo_cal_deg(const int32_t* ids, int64_t n_ids, int32_t n_nodes, int32_t* deg) {
    memset(deg, 0, sizeof(int32_t) * (size_t)n_nodes);
    for (int64_t e = 0; e < n_ids; ++e) deg[ids[e]] += 1; /* utilis.cu:43-58 */
}

void fglo_exclusive_sum(const int32_t* in, int64_t n, int32_t* out) {
    int32_t acc = 0; /* utilis.cu:17-41: scan of [in, 0] */
    for (int64_t i = 0; i < n; ++i) { out[i] = acc; acc += in[i]; }
    out[n] = acc;
}

/* ---- a4-a7: aggregation (aggregate_acc_kernel.cu) ------------------------ */
static inline double fglo_weight(int mode, int32_t d, int32_t s, const int32_t* indptr,
                                 const int32_t* src_deg, const int32_t* dst_deg) {
    if (mode == FGLO_MODE_SUM) return 1.0;
    if (mode == FGLO_MODE_MEAN) return 1.0 / (double)(indptr[d + 1] - indptr[d]);
    float a = 1.0f / sqrtf((float)dst_deg[d]); /* aggregate_acc_kernel.cu:300 */
    float b = 1.0f / sqrtf((float)src_deg[s]); /* aggregate_acc_kernel.cu:321 */
    return (double)(a * b);
}

/* out[d,:] = sum_e w * x[row(src[e]),:], accumulated in double and rounded once to float.
 * row_map (may be NULL) turns a block-local id into a row of x. */
void fglo_agg_fwd(int mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                  const int32_t* dst_deg, const int32_t* row_map, const float* x, int64_t ldx, int32_t dim,
                  int32_t n_dst, int zero_deg_passthrough, float* out, int64_t ldo) {
#pragma omp parallel
    {
        double* acc = (double*)malloc(sizeof(double) * (size_t)dim);
#pragma omp for schedule(dynamic, 64)
        for (int32_t d = 0; d < n_dst; ++d) {
            float* o = out + (int64_t)d * ldo;
            if (indptr[d] == indptr[d + 1]) { /* aggregate_acc_kernel.cu:307-308, 405-406 */
                const float* r = x + (int64_t)(row_map ? row_map[d] : d) * ldx;
                for (int32_t f = 0; f < dim; ++f) o[f] = zero_deg_passthrough ? r[f] : 0.0f;
                continue;
            }
            for (int32_t f = 0; f < dim; ++f) acc[f] = 0.0;
            for (int32_t e = indptr[d]; e < indptr[d + 1]; ++e) {
                const int32_t s = src[e];
                const double w = fglo_weight(mode, d, s, indptr, src_deg, dst_deg);
                const float* r = x + (int64_t)(row_map ? row_map[s] : s) * ldx;
                for (int32_t f = 0; f < dim; ++f) acc[f] += w * (double)r[f];
            }
            for (int32_t f = 0; f < dim; ++f) o[f] = (float)acc[f];
        }
        free(acc);
    }
}

/* dx[s,:] += w * dy[d,:] per edge; double accumulation in a scratch matrix, serial over edges so the
 * result does not depend on threads (aggregate_acc_kernel.cu:494-513, 579-594; rows without in-edges
 * contribute nothing, :498-500, :580-582). */
void fglo_agg_bwd(int mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                  const int32_t* dst_deg, const float* dy, int64_t ldy, int32_t dim, int32_t n_dst,
                  int32_t n_src, float* dx, int64_t ldx) {
    double* acc = (double*)calloc((size_t)n_src * (size_t)dim, sizeof(double));
    for (int32_t d = 0; d < n_dst; ++d) {
        const float* g = dy + (int64_t)d * ldy;
        for (int32_t e = indptr[d]; e < indptr[d + 1]; ++e) {
            const int32_t s = src[e];
            const double w = fglo_weight(mode, d, s, indptr, src_deg, dst_deg);
            double* a = acc + (size_t)s * (size_t)dim;
            for (int32_t f = 0; f < dim; ++f) a[f] += w * (double)g[f];
        }
    }
#pragma omp parallel for
    for (int32_t s = 0; s < n_src; ++s)
        for (int32_t f = 0; f < dim; ++f) dx[(int64_t)s * ldx + f] = (float)acc[(size_t)s * (size_t)dim + f];
    free(acc);
}

/* ---- edge-weighted multi-head aggregation (GAT; aggregate_acc_kernel.cu:836-885, 925-979) --------------- */
void fglo_agg_edge_fwd(const int32_t* indptr, const int32_t* src, const float* edge_w, int32_t n_heads, const float* x,
                       int64_t ldx, int32_t dim, int32_t n_dst, int zero_deg_passthrough, float* out, int64_t ldo) {
    const int32_t unit = dim / n_heads;
#pragma omp parallel
    {
        double* acc = (double*)malloc(sizeof(double) * (size_t)dim);
#pragma omp for schedule(dynamic, 64)
        for (int32_t d = 0; d < n_dst; ++d) {
            float* o = out + (int64_t)d * ldo;
            if (indptr[d] == indptr[d + 1]) { /* aggregate_acc_kernel.cu:870-872 */
                for (int32_t f = 0; f < dim; ++f) o[f] = zero_deg_passthrough ? x[(int64_t)d * ldx + f] : 0.0f;
                continue;
            }
            for (int32_t f = 0; f < dim; ++f) acc[f] = 0.0;
            for (int32_t e = indptr[d]; e < indptr[d + 1]; ++e) {
                const float* r = x + (int64_t)src[e] * ldx;
                const float* w = edge_w + (int64_t)e * n_heads;
                for (int32_t f = 0; f < dim; ++f) acc[f] += (double)w[f / unit] * (double)r[f];
            }
            for (int32_t f = 0; f < dim; ++f) o[f] = (float)acc[f];
        }
        free(acc);
    }
}

void fglo_agg_edge_bwd(const int32_t* indptr, const int32_t* src, const float* edge_w, int32_t n_heads, const float* dy,
                       int64_t ldy, int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx) {
    const int32_t unit = dim / n_heads;
    double* acc = (double*)calloc((size_t)n_src * (size_t)dim, sizeof(double));
    for (int32_t d = 0; d < n_dst; ++d) {
        const float* g = dy + (int64_t)d * ldy;
        for (int32_t e = indptr[d]; e < indptr[d + 1]; ++e) {
            const float* w = edge_w + (int64_t)e * n_heads;
            double* a = acc + (size_t)src[e] * (size_t)dim;
            for (int32_t f = 0; f < dim; ++f) a[f] += (double)w[f / unit] * (double)g[f];
        }
    }
    for (int32_t s = 0; s < n_src; ++s)
        for (int32_t f = 0; f < dim; ++f) dx[(int64_t)s * ldx + f] = (float)acc[(size_t)s * (size_t)dim + f];
    free(acc);
}

/*
 * CPU restatement of the permutohedral-lattice hash encoding of
 * RaduAlexandru/permutohedral_encoding, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared with
 * (tests, the smoke check and the benchmark's CPU-baseline leg).  The product package never
 * links, imports or calls it and has no CPU fallback.
 *
 * Parity status: pinned against fixtures produced by the reference's own CUDA extension
 * (rebuilt unmodified for sm_100, see build_ref.py) run on a B200: tests/golden/ and
 * tests/golden/make_golden.py.  The reference ships no tests or golden vectors of its own.
 *
 * Every function cites the reference lines it follows; paths are relative to the
 * reference project root.  All per-point arithmetic is IEEE binary32 in the operation
 * order of the reference kernels; compile with -ffp-contract=off so the only fused
 * multiply-adds are the explicit fmaf() calls that restate what nvcc's default -fmad=true
 * does to the reference source.  Sums over points (table gradient) and over levels
 * (position gradient) are accumulated in binary64 because the reference accumulates them
 * with fp32 atomics in a nondeterministic order: the binary64 sum is the value every
 * ordering approximates.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PERMUTO_MAX_DIM 7
#define MAX_FEAT 8
/* Features per level.  2 is the only width the reference implements (Encoding.cuh:140-143);
 * 4 and 8 follow the same arithmetic with wider table entries and are pinned by the identities
 * in the tests only (the reference cannot produce fixtures for them).  Set per call by the
 * Python front end from the table's last dimension. */
static int g_nfeat = 2;
#define NFEAT g_nfeat
void permuto_oracle_set_nfeat(int nfeat) { g_nfeat = nfeat; }

/* How nvcc's default -fmad=true contracts the reference's elevate loop
 * (EncodingGPU.cuh:130-138; cf_i = t_i*scale_i with t_i = pos_i + shift_i).  Determined by
 * exhaustive search over the legal contractions against the reference's outputs on a B200
 * (tests/golden/, every pos_dim 2..7 reproduces with zero mismatches under exactly this rule):
 *   i = d      : elevated[d] = -(d*cf_d), sm = cf_d                      (sm starts at 0)
 *   2 <= i < d : elevated[i] = fma(-i, cf_i, sm), sm = sm + cf_i         (cf_i stays a rounded product:
 *                                                                          it feeds i*cf_i)
 *   i = 1      : elevated[1] = fma(-t_1, scale_1, sm), elevated[0] = fma(t_1, scale_1, sm)
 *                                                                         (1*cf folds away, so both uses
 *                                                                          of the product fuse)
 * 1 = that rule (default), 0 = no contraction anywhere (kept to show the fixtures tell them apart). */
static int g_fma_elevate = 1;
/* 1 = scale = fl(base) * fl(1/sigma) (ATen tensor/scalar division multiplies by the
 * reciprocal), 0 = fl(base) / sigma. */
static int g_scale_by_reciprocal = 1;

void permuto_oracle_set_modes(int fma_elevate, int scale_by_reciprocal) {
    g_fma_elevate = fma_elevate;
    g_scale_by_reciprocal = scale_by_reciprocal;
}

int permuto_oracle_extra_levels(int pos_dim, int concat_points) {
    /* src/Encoding.cu:71-74: ceil(pos_dim / val_dim) extra output levels hold the raw points */
    return concat_points ? (pos_dim + NFEAT - 1) / NFEAT : 0;
}

/* include/permutohedral_encoding/Encoding.cuh:55-69.
 * base = 1/sqrt((i+1)(i+2)) is computed in binary64 and stored into a binary32 tensor
 * element; the element is then divided by sigma (binary32) through ATen's tensor-by-scalar
 * division, which for a host scalar divisor multiplies by the binary32 reciprocal. */
void permuto_oracle_scale_factor(const double *sigmas, int nr_levels, int pos_dim, float *out) {
    for (int l = 0; l < nr_levels; l++) {
        float sigma = (float)sigmas[l]; /* pybind converts the float64 list to std::vector<float> */
        for (int i = 0; i < pos_dim; i++) {
            float base = (float)(1.0 / sqrt((double)((i + 1) * (i + 2))) * 1.0);
            if (g_scale_by_reciprocal) {
                float inv = 1.0f / sigma;
                out[l * pos_dim + i] = base * inv;
            } else {
                out[l * pos_dim + i] = base / sigma;
            }
        }
    }
}

/* kernels/permutohedral_encoding/EncodingGPU.cuh:22-45: base-conversion hash, uint32 wrap,
 * unsigned modulo by the capacity (any capacity, not only powers of two). */
static inline int hash_slot(const int *key, int pos_dim, int capacity) {
    uint32_t k = 0;
    for (int i = 0; i < pos_dim; i++) {
        k += (uint32_t)key[i];
        k *= 2531011u;
    }
    return (int)(k % (uint32_t)capacity);
}

typedef struct {
    float elevated[PERMUTO_MAX_DIM + 1];
    int rem0[PERMUTO_MAX_DIM + 1];
    int rank[PERMUTO_MAX_DIM + 1];
    float bary[PERMUTO_MAX_DIM + 2];
} simplex_t;

/* EncodingGPU.cuh:130-199 (the same block is repeated at :311-382, :577-635, :1061-1132,
 * :1304-1375): elevate, round to the nearest remainder-0 point, rank the residuals, wrap
 * ranks back onto the plane, barycentric weights. */
static void locate_simplex(int d, const float *pos, const float *shift, const float *scale,
                           simplex_t *s) {
    const float inv = 1.0f / (float)(d + 1);
    float sm = 0.0f;
    for (int i = d; i > 0; i--) {
        float t = pos[i - 1] + shift[i - 1];
        float sc = scale[i - 1];
        float cf = t * sc;
        if (!g_fma_elevate) {
            float icf = (float)i * cf;
            s->elevated[i] = sm - icf;
            sm = sm + cf;
        } else if (i == 1) {
            s->elevated[i] = fmaf(-t, sc, sm);
            sm = fmaf(t, sc, sm);
        } else if (i == d) {
            float icf = (float)i * cf;
            s->elevated[i] = -icf;
            sm = cf;
        } else {
            s->elevated[i] = fmaf(-(float)i, cf, sm);
            sm = sm + cf;
        }
    }
    s->elevated[0] = sm;

    int sum = 0;
    for (int i = 0; i <= d; i++) {
        float v = s->elevated[i] * inv;
        float up = ceilf(v) * (float)(d + 1);
        float down = floorf(v) * (float)(d + 1);
        float du = up - s->elevated[i];
        float dd = s->elevated[i] - down;
        s->rem0[i] = (du < dd) ? (int)up : (int)down; /* ties go down */
        sum += s->rem0[i];
        s->rank[i] = 0;
    }
    sum /= d + 1; /* exact: every rem0 is a multiple of d+1 */

    for (int i = 0; i < d; i++) {
        float di = s->elevated[i] - (float)s->rem0[i];
        for (int j = i + 1; j <= d; j++) {
            float dj = s->elevated[j] - (float)s->rem0[j];
            if (di < dj)
                s->rank[i]++;
            else
                s->rank[j]++; /* ties raise the later index */
        }
    }
    for (int i = 0; i <= d; i++) {
        s->rank[i] += sum;
        if (s->rank[i] < 0) {
            s->rank[i] += d + 1;
            s->rem0[i] += d + 1;
        } else if (s->rank[i] > d) {
            s->rank[i] -= d + 1;
            s->rem0[i] -= d + 1;
        }
    }
    for (int i = 0; i <= d + 1; i++) s->bary[i] = 0.0f;
    for (int i = 0; i <= d; i++) {
        float delta = (s->elevated[i] - (float)s->rem0[i]) * inv;
        s->bary[d - s->rank[i]] += delta;
        s->bary[d + 1 - s->rank[i]] -= delta;
    }
    s->bary[0] += 1.0f + s->bary[d + 1];
}

/* EncodingGPU.cuh:212-223: key of the vertex with remainder r (first d coordinates). */
static inline void vertex_key(int d, const simplex_t *s, int r, int *key) {
    for (int i = 0; i < d; i++) {
        key[i] = s->rem0[i] + r;
        if (s->rank[i] > d - r) key[i] -= d + 1;
    }
}

static inline const float *row(const float *p, int64_t n, int64_t stride) { return p + n * stride; }

/* Debug view of the geometry: keys [N,L,d+1,d], slots [N,L,d+1], barycentric [N,L,d+1],
 * rank [N,L,d+1].  Any output pointer may be NULL. */
void permuto_oracle_lattice(int pos_dim, int nr_levels, int capacity, int64_t n_pos,
                            const float *positions, const float *scale, const float *shift,
                            int32_t *keys, int32_t *slots, float *bary, int32_t *rank) {
    const int d = pos_dim, V = d + 1;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < n_pos; n++) {
        simplex_t s;
        int key[PERMUTO_MAX_DIM];
        for (int l = 0; l < nr_levels; l++) {
            locate_simplex(d, row(positions, n, d), shift + l * d, scale + l * d, &s);
            int64_t base = (n * nr_levels + l) * V;
            for (int r = 0; r < V; r++) {
                vertex_key(d, &s, r, key);
                if (keys)
                    for (int i = 0; i < d; i++) keys[(base + r) * d + i] = key[i];
                if (slots) slots[base + r] = hash_slot(key, d, capacity);
                if (bary) bary[base + r] = s.bary[r];
                if (rank) rank[base + r] = s.rank[r];
            }
        }
    }
}

/* Forward: EncodingGPU.cuh:88-254 plus the output ordering of
 * src/pytorch_modules/modules.py:87 ([L,F,N] -> [N, L*F], level-major, feature inside).
 * table [L,C,2]; out [N,(L+extra)*2]. */
void permuto_oracle_forward(int pos_dim, int nr_levels, int capacity, int64_t n_pos,
                            const float *positions, const float *table, const float *scale,
                            const float *shift, const float *anneal, int concat_points,
                            float points_scaling, float *out) {
    const int d = pos_dim, V = d + 1;
    const int extra = permuto_oracle_extra_levels(d, concat_points);
    const int width = (nr_levels + extra) * NFEAT;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < n_pos; n++) {
        simplex_t s;
        int key[PERMUTO_MAX_DIM];
        const float *pos = row(positions, n, d);
        float *o = out + n * width;
        for (int l = 0; l < nr_levels; l++) {
            locate_simplex(d, pos, shift + l * d, scale + l * d, &s);
            const float *tl = table + (int64_t)l * capacity * NFEAT;
            float w_lvl = anneal[l];
            float acc_f[MAX_FEAT] = {0};
            for (int r = 0; r < V; r++) {
                vertex_key(d, &s, r, key);
                int slot = hash_slot(key, d, capacity);
                float w = s.bary[r] * w_lvl;
                for (int f = 0; f < NFEAT; f++) /* :246-247, contracted by -fmad */
                    acc_f[f] = fmaf(tl[slot * NFEAT + f], w, acc_f[f]);
            }
            for (int f = 0; f < NFEAT; f++) o[l * NFEAT + f] = acc_f[f];
        }
        /* :105-121 concat rows */
        for (int e = 0; e < extra; e++)
            for (int f = 0; f < NFEAT; f++) {
                int src = f + e * NFEAT;
                o[(nr_levels + e) * NFEAT + f] = (src < d) ? pos[src] * points_scaling : 0.0f;
            }
    }
}

/* First-order backward.
 * Table gradient: EncodingGPU.cuh:389-414 (addend = grad*w, w = bary*anneal), returned in the
 * parameter's own [L,C,2] layout (the reference returns a permuted view of [L,2,C],
 * src/Encoding.cu:141,204).  Position gradient: EncodingGPU.cuh:660-749, [N,d].
 * grad_out is [N,(L+extra)*2]; the extra rows receive no gradient path
 * (src/Encoding.cu:129-134,161).  table_grad / table_abs (sum of |addend|, for tolerances) /
 * pos_grad may be NULL. */
void permuto_oracle_backward(int pos_dim, int nr_levels, int capacity, int64_t n_pos,
                             const float *positions, const float *table, const float *scale,
                             const float *shift, const float *anneal, int concat_points,
                             const float *grad_out, float *table_grad, float *table_abs,
                             float *pos_grad) {
    const int d = pos_dim, V = d + 1;
    const int extra = permuto_oracle_extra_levels(d, concat_points);
    const int width = (nr_levels + extra) * NFEAT;
    const float inv = 1.0f / (float)(d + 1);
    const int64_t slice = (int64_t)capacity * NFEAT;

    if (table_grad) {
        /* one level per task: a level's slice is written by exactly one thread */
#pragma omp parallel for schedule(dynamic, 1)
        for (int l = 0; l < nr_levels; l++) {
            double *acc = (double *)calloc((size_t)slice, sizeof(double));
            double *aabs = table_abs ? (double *)calloc((size_t)slice, sizeof(double)) : NULL;
            simplex_t s;
            int key[PERMUTO_MAX_DIM];
            float w_lvl = anneal[l];
            for (int64_t n = 0; n < n_pos; n++) {
                locate_simplex(d, row(positions, n, d), shift + l * d, scale + l * d, &s);
                const float *gl = grad_out + n * width + l * NFEAT;
                for (int r = 0; r < V; r++) {
                    vertex_key(d, &s, r, key);
                    int slot = hash_slot(key, d, capacity);
                    float w = s.bary[r] * w_lvl;
                    for (int f = 0; f < NFEAT; f++) {
                        float af = gl[f] * w;
                        acc[slot * NFEAT + f] += (double)af;
                        if (aabs) aabs[slot * NFEAT + f] += fabs((double)af);
                    }
                }
            }
            for (int64_t i = 0; i < slice; i++) table_grad[l * slice + i] = (float)acc[i];
            if (aabs)
                for (int64_t i = 0; i < slice; i++) table_abs[l * slice + i] = (float)aabs[i];
            free(acc);
            free(aabs);
        }
    }

    if (pos_grad) {
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < n_pos; n++) {
            simplex_t s;
            int key[PERMUTO_MAX_DIM];
            double total[PERMUTO_MAX_DIM] = {0};
            for (int l = 0; l < nr_levels; l++) {
                const float *sc = scale + l * d;
                locate_simplex(d, row(positions, n, d), shift + l * d, sc, &s);
                const float *tl = table + (int64_t)l * slice;
                float w_lvl = anneal[l];
                const float *gl = grad_out + n * width + l * NFEAT;
                float dB[PERMUTO_MAX_DIM + 2];
                for (int r = 0; r <= d + 1; r++) dB[r] = 0.0f;
                for (int r = 0; r < V; r++) {
                    vertex_key(d, &s, r, key);
                    int slot = hash_slot(key, d, capacity);
                    for (int f = 0; f < NFEAT; f++) dB[r] += tl[slot * NFEAT + f] * w_lvl * gl[f]; /* :688-689 */
                }
                dB[d + 1] += dB[0]; /* :698 */
                float dE[PERMUTO_MAX_DIM + 1];
                for (int i = 0; i <= d; i++) { /* :703-706 */
                    dE[i] = 0.0f;
                    dE[i] += dB[d - s.rank[i]] * inv;
                    dE[i] -= dB[d + 1 - s.rank[i]] * inv;
                }
                for (int i = 0; i < d; i++) { /* :729-740 */
                    float dp = 0.0f;
                    for (int j = 0; j <= i; j++) dp += dE[j] * sc[i];
                    dp -= dE[i + 1] * sc[i] * (float)(i + 1);
                    total[i] += (double)dp; /* :748 atomicAdd across levels */
                }
            }
            for (int i = 0; i < d; i++) pos_grad[n * d + i] = (float)total[i];
        }
    }
}

/* Double backward of the position gradient: EncodingGPU.cuh:1187-1245 (table part, kernel 1)
 * and :1424-1491 (upstream-gradient part, kernel 2).  dpg = d loss / d positions_grad [N,d];
 * grad_out = the upstream gradient the first backward received [N,(L+extra)*2].
 * Outputs: table_grad [L,C,2] (+ optional table_abs), grad_grad_out [N,(L+extra)*2] with the
 * extra rows zero (:1290-1295).  Either output may be NULL. */
void permuto_oracle_double_backward(int pos_dim, int nr_levels, int capacity, int64_t n_pos,
                                    const float *positions, const float *table,
                                    const float *scale, const float *shift, const float *anneal,
                                    int concat_points, const float *dpg, const float *grad_out,
                                    float *table_grad, float *table_abs, float *grad_grad_out) {
    const int d = pos_dim, V = d + 1;
    const int extra = permuto_oracle_extra_levels(d, concat_points);
    const int width = (nr_levels + extra) * NFEAT;
    const float inv = 1.0f / (float)(d + 1);
    const int64_t slice = (int64_t)capacity * NFEAT;

    /* dB for one (point, level): :1187-1218 */
#define DOUBLE_BACK_DB(dB, s, sc, gp)                                       \
    do {                                                                    \
        float dE_[PERMUTO_MAX_DIM + 1];                                     \
        for (int i_ = 0; i_ <= d; i_++) dE_[i_] = 0.0f;                     \
        for (int i_ = 0; i_ < d; i_++) {                                    \
            float g_ = (gp)[i_] * (sc)[i_];                                 \
            for (int j_ = 0; j_ <= i_; j_++) dE_[j_] += g_;                 \
        }                                                                   \
        for (int i_ = 0; i_ < d; i_++)                                      \
            dE_[i_ + 1] -= (gp)[i_] * (sc)[i_] * (float)(i_ + 1);           \
        for (int r_ = 0; r_ <= d + 1; r_++) (dB)[r_] = 0.0f;                \
        for (int i_ = 0; i_ <= d; i_++) {                                   \
            (dB)[d - (s).rank[i_]] += dE_[i_] * inv;                        \
            (dB)[d + 1 - (s).rank[i_]] -= dE_[i_] * inv;                    \
        }                                                                   \
        (dB)[0] += (dB)[d + 1];                                             \
    } while (0)

    if (table_grad) {
#pragma omp parallel for schedule(dynamic, 1)
        for (int l = 0; l < nr_levels; l++) {
            double *acc = (double *)calloc((size_t)slice, sizeof(double));
            double *aabs = table_abs ? (double *)calloc((size_t)slice, sizeof(double)) : NULL;
            simplex_t s;
            int key[PERMUTO_MAX_DIM];
            const float *sc = scale + l * d;
            float w_lvl = anneal[l];
            for (int64_t n = 0; n < n_pos; n++) {
                locate_simplex(d, row(positions, n, d), shift + l * d, sc, &s);
                float dB[PERMUTO_MAX_DIM + 2];
                DOUBLE_BACK_DB(dB, s, sc, dpg + n * d);
                const float *gl = grad_out + n * width + l * NFEAT;
                for (int r = 0; r < V; r++) {
                    vertex_key(d, &s, r, key);
                    int slot = hash_slot(key, d, capacity);
                    for (int f = 0; f < NFEAT; f++) {
                        float af = dB[r] * w_lvl * gl[f]; /* :1244-1245 */
                        acc[slot * NFEAT + f] += (double)af;
                        if (aabs) aabs[slot * NFEAT + f] += fabs((double)af);
                    }
                }
            }
            for (int64_t i = 0; i < slice; i++) table_grad[l * slice + i] = (float)acc[i];
            if (aabs)
                for (int64_t i = 0; i < slice; i++) table_abs[l * slice + i] = (float)aabs[i];
            free(acc);
            free(aabs);
        }
    }

    if (grad_grad_out) {
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < n_pos; n++) {
            simplex_t s;
            int key[PERMUTO_MAX_DIM];
            float *o = grad_grad_out + n * width;
            for (int l = 0; l < nr_levels; l++) {
                const float *sc = scale + l * d;
                locate_simplex(d, row(positions, n, d), shift + l * d, sc, &s);
                const float *tl = table + (int64_t)l * slice;
                float w_lvl = anneal[l];
                float dB[PERMUTO_MAX_DIM + 2];
                DOUBLE_BACK_DB(dB, s, sc, dpg + n * d);
                float acc_f[MAX_FEAT] = {0};
                for (int r = 0; r < V; r++) {
                    vertex_key(d, &s, r, key);
                    int slot = hash_slot(key, d, capacity);
                    for (int f = 0; f < NFEAT; f++) acc_f[f] += dB[r] * w_lvl * tl[slot * NFEAT + f]; /* :1484-1485 */
                }
                for (int f = 0; f < NFEAT; f++) o[l * NFEAT + f] = acc_f[f];
            }
            for (int e = 0; e < extra * NFEAT; e++) o[nr_levels * NFEAT + e] = 0.0f;
        }
    }
#undef DOUBLE_BACK_DB
}

int permuto_oracle_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void permuto_oracle_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference neighbor-list
 * algorithm (vesin's CPU cell list), in plain C, single threaded.
 *
 * This file is the checker the GPU engine is compared against. It is never
 * linked into, called from, or shipped with the product library: only the
 * tests, the smoke check and the CPU-baseline leg of the benchmark load it.
 *
 * Parity pin: the restatement is checked (tests/test_oracle.py) against
 *   - the known answers of the reference's own C++/Fortran tests
 *     (vesin/tests/neighbors.cpp, vesin/tests/memory.cpp, vesin/tests/cuda.cpp,
 *     fortran/tests/tests.f90), and
 *   - outputs of the unmodified reference CPU sources compiled as
 *     oracle/_ref/libvesin_ref.so, stored as fixtures under tests/golden/.
 * With one thread the reference visits cells, stencil offsets and atoms in the
 * same order as this file does, so even the unsorted output order is the same.
 *
 * Each function cites the reference file:line it follows (paths relative to
 * the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

typedef struct {
    size_t length;
    size_t capacity;
    size_t* pairs;     /* [length][2] */
    int32_t* shifts;   /* [length][3] or NULL */
    double* distances; /* [length]    or NULL */
    double* vectors;   /* [length][3] or NULL */
} OracleList;

/* ---- 3-vector helpers: same association as vesin/src/math.hpp:14-36 ---- */
typedef struct {
    double v[3];
} vec3;

static double dot3(vec3 a, vec3 b) {
    /* math.hpp:14-16: (a0*b0 + a1*b1) + a2*b2 */
    return a.v[0] * b.v[0] + a.v[1] * b.v[1] + a.v[2] * b.v[2];
}

static vec3 scale3(vec3 a, double s) {
    vec3 r = {{s * a.v[0], s * a.v[1], s * a.v[2]}};
    return r;
}

static vec3 normalize3(vec3 a) {
    /* math.hpp:18-24: multiply by (1 / norm) */
    return scale3(a, 1.0 / sqrt(dot3(a, a)));
}

static vec3 cross3(vec3 a, vec3 b) {
    /* math.hpp:26-32 */
    vec3 r = {{
        a.v[1] * b.v[2] - a.v[2] * b.v[1],
        a.v[2] * b.v[0] - a.v[0] * b.v[2],
        a.v[0] * b.v[1] - a.v[1] * b.v[0],
    }};
    return r;
}

static double det3(const double m[3][3]) {
    /* math.hpp:72-78 */
    return m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) -
           m[0][1] * (m[1][0] * m[2][2] - m[1][2] * m[2][0]) +
           m[0][2] * (m[1][0] * m[2][1] - m[1][1] * m[2][0]);
}

static void inverse3(const double m[3][3], double det, double inv[3][3]) {
    /* math.hpp:80-98 */
    inv[0][0] = (m[1][1] * m[2][2] - m[2][1] * m[1][2]) / det;
    inv[0][1] = (m[0][2] * m[2][1] - m[0][1] * m[2][2]) / det;
    inv[0][2] = (m[0][1] * m[1][2] - m[0][2] * m[1][1]) / det;
    inv[1][0] = (m[1][2] * m[2][0] - m[1][0] * m[2][2]) / det;
    inv[1][1] = (m[0][0] * m[2][2] - m[0][2] * m[2][0]) / det;
    inv[1][2] = (m[1][0] * m[0][2] - m[0][0] * m[1][2]) / det;
    inv[2][0] = (m[1][0] * m[2][1] - m[2][0] * m[1][1]) / det;
    inv[2][1] = (m[2][0] * m[0][1] - m[0][0] * m[2][1]) / det;
    inv[2][2] = (m[0][0] * m[1][1] - m[1][0] * m[0][1]) / det;
}

/* ---- bounding box: vesin/src/types.hpp:12-210 ---- */
typedef struct {
    double matrix[3][3];
    double inverse[3][3];
    int periodic[3];
    double min_pos[3];
    double max_pos[3];
    double face_dist[3];
} OracleBox;

static vec3 row3(const double m[3][3], int i) {
    vec3 r = {{m[i][0], m[i][1], m[i][2]}};
    return r;
}

static void set_row3(double m[3][3], int i, vec3 a) {
    m[i][0] = a.v[0];
    m[i][1] = a.v[1];
    m[i][2] = a.v[2];
}

/* types.hpp:20-97. Returns 0, or 1 with `err` filled. */
static int box_init(OracleBox* b, const double* box9, const unsigned char* periodic, char* err, size_t errlen) {
    int n_periodic = 0, p1 = -1, p2 = -1;
    for (int i = 0; i < 3; i++) {
        for (int j = 0; j < 3; j++) {
            b->matrix[i][j] = box9[3 * i + j];
        }
        b->periodic[i] = periodic[i] != 0;
        b->max_pos[i] = -1e300;
        b->min_pos[i] = 1e300;
        if (b->periodic[i]) {
            n_periodic++;
            if (p1 == -1) {
                p1 = i;
            } else if (p2 == -1) {
                p2 = i;
            }
        }
    }

    /* types.hpp:41-72: non-periodic rows are replaced by unit vectors
       orthogonal to the periodic ones */
    if (n_periodic == 0) {
        for (int i = 0; i < 3; i++) {
            for (int j = 0; j < 3; j++) {
                b->matrix[i][j] = (i == j) ? 1.0 : 0.0;
            }
        }
    } else if (n_periodic == 1) {
        vec3 a = row3(b->matrix, p1);
        vec3 bb = {{0, 1, 0}};
        if (fabs(dot3(normalize3(a), bb)) > 0.9) {
            vec3 z = {{0, 0, 1}};
            bb = z;
        }
        vec3 c = normalize3(cross3(a, bb));
        bb = normalize3(cross3(c, a));
        set_row3(b->matrix, (p1 + 1) % 3, bb);
        set_row3(b->matrix, (p1 + 2) % 3, c);
    } else if (n_periodic == 2) {
        vec3 a = row3(b->matrix, p1);
        vec3 bb = row3(b->matrix, p2);
        vec3 c = normalize3(cross3(a, bb));
        set_row3(b->matrix, 3 - p1 - p2, c);
    }

    /* types.hpp:74-80 */
    double det = det3(b->matrix);
    if (fabs(det) < 1e-30) {
        snprintf(err, errlen, "the box matrix is not invertible");
        return 1;
    }
    inverse3(b->matrix, det, b->inverse);

    /* types.hpp:82-96: distances between opposite faces */
    vec3 a = row3(b->matrix, 0), bb = row3(b->matrix, 1), c = row3(b->matrix, 2);
    vec3 na = normalize3(cross3(bb, c));
    vec3 nb = normalize3(cross3(c, a));
    vec3 nc = normalize3(cross3(a, bb));
    b->face_dist[0] = b->periodic[0] ? fabs(dot3(na, a)) : b->max_pos[0] - b->min_pos[0];
    b->face_dist[1] = b->periodic[1] ? fabs(dot3(nb, bb)) : b->max_pos[1] - b->min_pos[1];
    b->face_dist[2] = b->periodic[2] ? fabs(dot3(nc, c)) : b->max_pos[2] - b->min_pos[2];
    return 0;
}

/* types.hpp:159-200 */
static int box_make_bounding_for(OracleBox* b, const double* points, size_t n, char* err, size_t errlen) {
    for (size_t i = 0; i < n; i++) {
        for (int s = 0; s < 3; s++) {
            double x = points[3 * i + s];
            if (!isfinite(x)) {
                /* types.hpp:163-169; std::to_string(double) prints "%f" */
                snprintf(err, errlen, "point %zu has non-finite coordinate along axis %d: %f", i, s, x);
                return 1;
            }
            if (x < b->min_pos[s]) {
                b->min_pos[s] = x;
            }
            if (x > b->max_pos[s]) {
                b->max_pos[s] = x;
            }
        }
    }
    for (int d = 0; d < 3; d++) {
        if (b->max_pos[d] - b->min_pos[d] < 1e-6) {
            b->max_pos[d] = b->min_pos[d] + 1;
        }
        if (!b->periodic[d]) {
            b->face_dist[d] = (b->max_pos[d] - b->min_pos[d]) * 1.01;
            if (b->face_dist[d] < 1.0) {
                b->face_dist[d] = 1.0;
            }
        }
    }
    return 0;
}

/* types.hpp:107-126: row-vector times inverse, then the non-periodic
   components are replaced by (x - min) / extent along the Cartesian axis */
static void box_cartesian_to_fractional(const OracleBox* b, const double* r, double f[3]) {
    for (int k = 0; k < 3; k++) {
        /* math.hpp:111-117 */
        f[k] = r[0] * b->inverse[0][k] + r[1] * b->inverse[1][k] + r[2] * b->inverse[2][k];
    }
    for (int k = 0; k < 3; k++) {
        if (!b->periodic[k]) {
            f[k] = (r[k] - b->min_pos[k]) / b->face_dist[k];
        }
    }
}

/* cpu_cell_list.cpp:253-263: Python-style divmod */
static void divmod_i32(int32_t a, int32_t b, int32_t* q, int32_t* r) {
    int32_t quotient = a / b;
    int32_t remainder = a % b;
    if (remainder < 0) {
        remainder += b;
        quotient -= 1;
    }
    *q = quotient;
    *r = remainder;
}

static double clamp_min1(double x) {
    /* std::clamp(x, 1.0, HUGE_VAL) */
    return x < 1.0 ? 1.0 : x;
}

static int list_reserve(OracleList* l, size_t want, int S, int d, int D) {
    if (want <= l->capacity) {
        return 0;
    }
    size_t cap = l->capacity ? l->capacity : 1024;
    while (cap < want) {
        cap *= 2;
    }
    size_t* p = realloc(l->pairs, cap * 2 * sizeof(size_t));
    if (!p) {
        return 1;
    }
    l->pairs = p;
    if (S) {
        int32_t* s = realloc(l->shifts, cap * 3 * sizeof(int32_t));
        if (!s) {
            return 1;
        }
        l->shifts = s;
    }
    if (d) {
        double* x = realloc(l->distances, cap * sizeof(double));
        if (!x) {
            return 1;
        }
        l->distances = x;
    }
    if (D) {
        double* x = realloc(l->vectors, cap * 3 * sizeof(double));
        if (!x) {
            return 1;
        }
        l->vectors = x;
    }
    l->capacity = cap;
    return 0;
}

ORACLE_API void vesin_oracle_free(OracleList* l) {
    if (!l) {
        return;
    }
    free(l->pairs);
    free(l->shifts);
    free(l->distances);
    free(l->vectors);
    memset(l, 0, sizeof(*l));
}

/*
 * Whole CPU path for one system: vesin.cpp:109-125 (box, bounding extent),
 * cpu_cell_list.cpp:61-163 (cell list, half-list filter, distance predicate).
 * `out` must be zero-initialised on first use; it can be re-used across calls.
 * Returns 0 on success, 1 on failure with a message in `err`.
 */
ORACLE_API int vesin_oracle_neighbors(
    const double* points,
    size_t n_points,
    const double* box9,
    const unsigned char* periodic,
    double cutoff,
    int full,
    int return_shifts,
    int return_distances,
    int return_vectors,
    OracleList* out,
    char* err,
    size_t errlen
) {
    OracleBox box;
    if (box_init(&box, box9, periodic, err, errlen)) {
        return 1;
    }
    if (box_make_bounding_for(&box, points, n_points, err, errlen)) {
        return 1;
    }

    /* ---- CellList::CellList, cpu_cell_list.cpp:277-351 ---- */
    double n_cells[3];
    for (int k = 0; k < 3; k++) {
        n_cells[k] = clamp_min1(trunc(box.face_dist[k] / cutoff));
    }
    double n_total = n_cells[0] * n_cells[1] * n_cells[2];
    if (n_total > 1e5) {
        /* :293-303 */
        double ratio_x_y = n_cells[0] / n_cells[1];
        double ratio_y_z = n_cells[1] / n_cells[2];
        n_cells[2] = trunc(cbrt(1e5 / (ratio_x_y * ratio_y_z * ratio_y_z)));
        n_cells[1] = trunc(ratio_y_z * n_cells[2]);
        n_cells[0] = trunc(ratio_x_y * n_cells[1]);
    }
    int32_t n_search[3];
    int32_t shape[3];
    for (int k = 0; k < 3; k++) {
        n_search[k] = (int32_t)ceil(cutoff * n_cells[k] / box.face_dist[k]);
        shape[k] = (int32_t)(size_t)n_cells[k];
        if (n_search[k] < 1) {
            n_search[k] = 1;
        }
    }
    int has_periodic = box.periodic[0] || box.periodic[1] || box.periodic[2];
    int has_non_periodic = !box.periodic[0] || !box.periodic[1] || !box.periodic[2];
    if (has_periodic && has_non_periodic) {
        /* :325-348 */
        for (int k = 0; k < 3; k++) {
            if (!box.periodic[k] && n_search[k] < shape[k] - 1) {
                n_search[k] = shape[k] - 1;
            }
        }
    }
    size_t total_cells = (size_t)shape[0] * (size_t)shape[1] * (size_t)shape[2];

    /* ---- CellList::add_point, :353-374. The per-cell vectors of the
       reference are stored here as a stable counting sort (same order). ---- */
    int32_t* atom_cell = malloc((n_points ? n_points : 1) * sizeof(int32_t));
    int32_t* atom_shift = malloc((n_points ? n_points : 1) * 3 * sizeof(int32_t));
    size_t* cell_start = calloc(total_cells + 1, sizeof(size_t));
    size_t* sorted = malloc((n_points ? n_points : 1) * sizeof(size_t));
    if (!atom_cell || !atom_shift || !cell_start || !sorted) {
        free(atom_cell);
        free(atom_shift);
        free(cell_start);
        free(sorted);
        snprintf(err, errlen, "failed to allocate memory");
        return 1;
    }
    for (size_t i = 0; i < n_points; i++) {
        double f[3];
        box_cartesian_to_fractional(&box, points + 3 * i, f);
        int32_t c[3];
        for (int k = 0; k < 3; k++) {
            int32_t ci = (int32_t)floor(f[k] * (double)shape[k]);
            divmod_i32(ci, shape[k], &atom_shift[3 * i + k], &c[k]);
        }
        /* get_cell, :453-461: x fastest */
        size_t lin = ((size_t)shape[0] * (size_t)shape[1] * (size_t)c[2]) + ((size_t)shape[0] * (size_t)c[1]) + (size_t)c[0];
        atom_cell[i] = (int32_t)lin;
        cell_start[lin + 1]++;
    }
    for (size_t c = 0; c < total_cells; c++) {
        cell_start[c + 1] += cell_start[c];
    }
    {
        size_t* cursor = malloc((total_cells ? total_cells : 1) * sizeof(size_t));
        memcpy(cursor, cell_start, total_cells * sizeof(size_t));
        for (size_t i = 0; i < n_points; i++) {
            sorted[cursor[atom_cell[i]]++] = i;
        }
        free(cursor);
    }

    double cutoff2 = cutoff * cutoff; /* cpu_cell_list.cpp:77 */
    out->length = 0;
    if ((return_shifts && !out->shifts) || (return_distances && !out->distances) || (return_vectors && !out->vectors)) {
        /* a re-used list that lacks a requested array starts over */
        vesin_oracle_free(out);
    }
    int status = 0;

    /* ---- CellList::foreach_pair, :376-451 (one thread: cells in order) ---- */
    for (size_t lin_i = 0; lin_i < total_cells && !status; lin_i++) {
        if (cell_start[lin_i] == cell_start[lin_i + 1]) {
            continue;
        }
        int32_t cx = (int32_t)(lin_i % (size_t)shape[0]);
        int32_t cy = (int32_t)((lin_i / (size_t)shape[0]) % (size_t)shape[1]);
        int32_t cz = (int32_t)(lin_i / ((size_t)shape[0] * (size_t)shape[1]));

        for (int32_t dx = -n_search[0]; dx <= n_search[0] && !status; dx++) {
            for (int32_t dy = -n_search[1]; dy <= n_search[1] && !status; dy++) {
                for (int32_t dz = -n_search[2]; dz <= n_search[2] && !status; dz++) {
                    int32_t cell_shift[3] = {0, 0, 0};
                    int32_t nb[3] = {cx + dx, cy + dy, cz + dz};
                    int valid = 1;
                    for (int k = 0; k < 3; k++) {
                        if (box.periodic[k]) {
                            divmod_i32(nb[k], shape[k], &cell_shift[k], &nb[k]);
                        } else if (nb[k] < 0 || nb[k] >= shape[k]) {
                            valid = 0;
                            break;
                        }
                    }
                    if (!valid) {
                        continue;
                    }
                    size_t lin_j = ((size_t)shape[0] * (size_t)shape[1] * (size_t)nb[2]) + ((size_t)shape[0] * (size_t)nb[1]) + (size_t)nb[0];

                    for (size_t a = cell_start[lin_i]; a < cell_start[lin_i + 1] && !status; a++) {
                        size_t i = sorted[a];
                        for (size_t bidx = cell_start[lin_j]; bidx < cell_start[lin_j + 1]; bidx++) {
                            size_t j = sorted[bidx];
                            int32_t S[3];
                            for (int k = 0; k < 3; k++) {
                                S[k] = cell_shift[k] + atom_shift[3 * i + k] - atom_shift[3 * j + k]; /* :423 */
                            }
                            int shift_is_zero = S[0] == 0 && S[1] == 0 && S[2] == 0;
                            if ((S[0] != 0 && !box.periodic[0]) || (S[1] != 0 && !box.periodic[1]) || (S[2] != 0 && !box.periodic[2])) {
                                continue; /* :426-432 */
                            }
                            if (i == j && shift_is_zero) {
                                continue; /* :434-438 */
                            }

                            /* half-list filter, :101-133 */
                            if (!full) {
                                if (i > j) {
                                    continue;
                                }
                                if (i == j) {
                                    int32_t sum = S[0] + S[1] + S[2];
                                    if (sum < 0) {
                                        continue;
                                    }
                                    if (sum == 0 && (S[2] < 0 || (S[2] == 0 && S[1] < 0))) {
                                        continue;
                                    }
                                }
                            }

                            /* :135-138 with types.hpp:232-243, math.hpp:111-117:
                               v = (r_j - r_i) + ((S0*H0 + S1*H1) + S2*H2) */
                            double sf[3] = {(double)S[0], (double)S[1], (double)S[2]};
                            double v[3];
                            for (int k = 0; k < 3; k++) {
                                double sh = sf[0] * box.matrix[0][k] + sf[1] * box.matrix[1][k] + sf[2] * box.matrix[2][k];
                                v[k] = (points[3 * j + k] - points[3 * i + k]) + sh;
                            }
                            double d2 = v[0] * v[0] + v[1] * v[1] + v[2] * v[2];
                            if (d2 < cutoff2) {
                                size_t idx = out->length;
                                if (list_reserve(out, idx + 1, return_shifts, return_distances, return_vectors)) {
                                    snprintf(err, errlen, "failed to allocate memory");
                                    status = 1;
                                    break;
                                }
                                out->pairs[2 * idx] = i;
                                out->pairs[2 * idx + 1] = j;
                                if (return_shifts) {
                                    memcpy(out->shifts + 3 * idx, S, sizeof(S));
                                }
                                if (return_distances) {
                                    out->distances[idx] = sqrt(d2);
                                }
                                if (return_vectors) {
                                    memcpy(out->vectors + 3 * idx, v, sizeof(v));
                                }
                                out->length = idx + 1;
                            }
                        }
                    }
                }
            }
        }
    }

    free(atom_cell);
    free(atom_shift);
    free(cell_start);
    free(sorted);
    return status;
}

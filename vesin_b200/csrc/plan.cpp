#include "plan.hpp"

#include <algorithm>
#include <cmath>
#include <limits>
#include <stdexcept>

namespace vb200 {

namespace {

struct V3 {
    double x, y, z;
};

V3 row(const double m[3][3], int i) {
    return {m[i][0], m[i][1], m[i][2]};
}

void set_row(double m[3][3], int i, V3 v) {
    m[i][0] = v.x;
    m[i][1] = v.y;
    m[i][2] = v.z;
}

double dot(V3 a, V3 b) {
    return a.x * b.x + a.y * b.y + a.z * b.z;
}

V3 cross(V3 a, V3 b) {
    return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x};
}

V3 unit(V3 a) {
    double inv = 1.0 / std::sqrt(dot(a, a));
    return {a.x * inv, a.y * inv, a.z * inv};
}

double determinant(const double m[3][3]) {
    return m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) -
           m[0][1] * (m[1][0] * m[2][2] - m[1][2] * m[2][0]) +
           m[0][2] * (m[1][0] * m[2][1] - m[1][1] * m[2][0]);
}

void invert(const double m[3][3], double det, double inv[3][3]) {
    // adjugate / determinant
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

} // namespace

/// fp32 screen of the pair passes. Local coordinates (relative to the centre
/// of the unit) of a point and of its candidates are bounded by M; each carries
/// a rounding error of at most eps * M, a difference eps * (2 M + d), and the
/// squared distance of a candidate near the cutoff is then off by at most
///   eps * (2 sqrt(3) c (2 M + c) + 3 c^2).
/// Four times that, plus the rounding of the expanded form used by the fused
/// pass, is the half-width of the band inside which the fp64 predicate decides.
static void update_screen(GridPlan& plan, double cutoff) {
    double reach = 0.0;
    for (int k = 0; k < 3; k++) {
        double len = std::sqrt(
            plan.cell_vec[k][0] * plan.cell_vec[k][0] + plan.cell_vec[k][1] * plan.cell_vec[k][1] +
            plan.cell_vec[k][2] * plan.cell_vec[k][2]
        );
        double cells = plan.n_search[k] + 1.0;
        if (k == 0) {
            cells += 0.5 * plan.pencil; // the frame is centred on the pencil
        }
        reach += cells * len;
    }
    for (int c = 0; c < 3; c++) {
        volatile double zero = 0.0; // keeps the three products and two sums as written
        plan.zero_shift[c] = (zero * plan.H[0][c] + zero * plan.H[1][c]) + zero * plan.H[2][c];
    }
    const double eps = 5.9604644775390625e-08; // 2^-24
    double c = cutoff * 1.01;
    double band = 4.0 * eps * (2.0 * std::sqrt(3.0) * c * (2.0 * reach + c) + 3.0 * c * c);
    // The fused pass evaluates d2 as |c|^2 + |i|^2 - 2 c.i: seven roundings on
    // terms bounded by (2 M)^2.
    band += 40.0 * eps * reach * reach;
    band += 4.0 * eps * plan.cutoff2; // rounding of the bounds themselves
    double lo = plan.cutoff2 - band;
    double hi = plan.cutoff2 + band;
    // "surely inside" only exists when the band is narrower than the cutoff;
    // the expanded form of d2 can come out negative, so 0 is not a safe floor
    plan.cutoff2_lo = (lo > 0.0) ? std::nextafter(static_cast<float>(lo), 0.0f) : -std::numeric_limits<float>::infinity();
    float hi_f = static_cast<float>(hi);
    plan.cutoff2_hi = std::isfinite(hi_f) ? std::nextafter(hi_f, std::numeric_limits<float>::infinity())
                                          : std::numeric_limits<float>::max();
}

GridPlan make_plan(
    const double box[9],
    const bool periodic[3],
    const PointBounds& bounds,
    size_t n_points,
    double cutoff,
    bool full,
    bool sorted,
    size_t max_cells
) {
    GridPlan plan{};
    int n_periodic = 0;
    int first = -1;
    int second = -1;
    for (int i = 0; i < 3; i++) {
        for (int j = 0; j < 3; j++) {
            plan.H[i][j] = box[3 * i + j];
        }
        plan.periodic[i] = periodic[i] ? 1 : 0;
        if (periodic[i]) {
            n_periodic++;
            if (first < 0) {
                first = i;
            } else if (second < 0) {
                second = i;
            }
        }
    }

    // Rows of non-periodic directions never enter a pair vector (their shift
    // is always zero); they are replaced by unit vectors orthogonal to the
    // periodic rows so that H stays invertible whatever the caller left there.
    // Same construction as the reference CPU path (vesin/src/types.hpp:41-72),
    // so that "not invertible" is raised for the same inputs.
    if (n_periodic == 0) {
        for (int i = 0; i < 3; i++) {
            for (int j = 0; j < 3; j++) {
                plan.H[i][j] = (i == j) ? 1.0 : 0.0;
            }
        }
    } else if (n_periodic == 1) {
        V3 a = row(plan.H, first);
        V3 helper{0, 1, 0};
        if (std::abs(dot(unit(a), helper)) > 0.9) {
            helper = V3{0, 0, 1};
        }
        V3 c = unit(cross(a, helper));
        V3 b = unit(cross(c, a));
        set_row(plan.H, (first + 1) % 3, b);
        set_row(plan.H, (first + 2) % 3, c);
    } else if (n_periodic == 2) {
        V3 a = row(plan.H, first);
        V3 b = row(plan.H, second);
        set_row(plan.H, 3 - first - second, unit(cross(a, b)));
    }

    double det = determinant(plan.H);
    if (!(std::abs(det) >= 1e-30)) {
        throw std::runtime_error("the box matrix is not invertible");
    }
    invert(plan.H, det, plan.Hinv);

    // A cutoff inflated by 2^-30 absorbs the rounding of the binning
    // arithmetic: two points closer than the cutoff are then never further
    // apart than n_search cells, even when the box is an exact multiple of
    // the cutoff.
    const double safe_cutoff = cutoff * (1.0 + 9.5e-10);

    double n_wanted[3];
    double width_nonperiodic[3] = {0, 0, 0};
    for (int k = 0; k < 3; k++) {
        if (plan.periodic[k]) {
            // distance between the two faces spanned by the other two rows:
            // 1 / |column k of the inverse|
            double norm = std::sqrt(
                plan.Hinv[0][k] * plan.Hinv[0][k] + plan.Hinv[1][k] * plan.Hinv[1][k] + plan.Hinv[2][k] * plan.Hinv[2][k]
            );
            plan.face_dist[k] = 1.0 / norm;
            plan.t0[k] = 0.0;
        } else {
            // Extent of the projections on the unit vector u_k = column k of
            // the inverse (u_k is orthogonal to every other row of H and has
            // unit length, so H^-1's column k is u_k itself). The projections
            // of all points lie inside the projection of their bounding box.
            double lo = 0.0;
            double hi = 0.0;
            for (int c = 0; c < 3; c++) {
                double u = plan.Hinv[c][k];
                double a = u * bounds.min[c];
                double b = u * bounds.max[c];
                lo += std::min(a, b);
                hi += std::max(a, b);
            }
            if (n_points == 0 || !(hi >= lo)) {
                lo = 0.0;
                hi = 1.0;
            }
            double extent = (hi - lo) * 1.01;
            if (!(extent >= 1.0)) {
                extent = 1.0;
            }
            plan.t0[k] = lo - 0.5 * (extent - (hi - lo));
            plan.face_dist[k] = extent;
            width_nonperiodic[k] = extent;
        }
        n_wanted[k] = std::max(1.0, std::floor(plan.face_dist[k] / safe_cutoff));
    }

    // Bound the number of cells by the number of points (and by what fits the
    // scratch arrays): a huge, almost empty box must not allocate by volume.
    double cap = static_cast<double>(std::max<size_t>(1, std::min<size_t>(max_cells, std::max<size_t>(n_points, 1))));
    for (int iter = 0; iter < 64 && n_wanted[0] * n_wanted[1] * n_wanted[2] > cap; iter++) {
        double factor = std::cbrt(cap / (n_wanted[0] * n_wanted[1] * n_wanted[2]));
        factor = std::min(factor, 0.98);
        for (int k = 0; k < 3; k++) {
            n_wanted[k] = std::max(1.0, std::floor(n_wanted[k] * factor));
        }
    }

    plan.n_stencil = 1;
    for (int k = 0; k < 3; k++) {
        plan.n_cells[k] = static_cast<int32_t>(n_wanted[k]);
        double cells_per_cutoff = safe_cutoff * n_wanted[k] / plan.face_dist[k];
        plan.n_search[k] = std::max<int32_t>(1, static_cast<int32_t>(std::ceil(cells_per_cutoff)));
        if (!plan.periodic[k]) {
            // no images: never look further than the grid itself
            plan.n_search[k] = std::min(plan.n_search[k], std::max(1, plan.n_cells[k] - 1));
            if (plan.n_cells[k] == 1) {
                plan.n_search[k] = 0;
            }
            plan.scale[k] = n_wanted[k] / width_nonperiodic[k];
        } else {
            plan.scale[k] = n_wanted[k];
        }
        for (int c = 0; c < 3; c++) {
            double step = plan.periodic[k] ? 1.0 / n_wanted[k] : width_nonperiodic[k] / n_wanted[k];
            plan.cell_vec[k][c] = plan.H[k][c] * step;
        }
        plan.n_stencil *= 2 * plan.n_search[k] + 1;
    }
    {
        // a cutoff many times the box (a collapsed box, a wrong unit) would mean a stencil of
        // billions of cells: an error, not a kernel that never ends
        double stencil = 1.0;
        for (int k = 0; k < 3; k++) {
            stencil *= 2.0 * plan.n_search[k] + 1.0;
        }
        if (stencil > static_cast<double>(MAX_STENCIL_CELLS)) {
            throw std::runtime_error(
                "the cutoff is too large for this box: every point would be compared with more than " + std::to_string(MAX_STENCIL_CELLS) +
                " periodic images of the cells around it"
            );
        }
    }
    plan.n_cells_total = plan.n_cells[0] * plan.n_cells[1] * plan.n_cells[2];
    for (int c = 0; c < 3; c++) {
        plan.origin[c] = 0.0;
        for (int k = 0; k < 3; k++) {
            if (!plan.periodic[k]) {
                plan.origin[c] += plan.t0[k] * plan.H[k][c];
            }
        }
    }

    plan.cutoff2 = cutoff * cutoff;
    plan.full = full ? 1 : 0;
    plan.by_index = sorted ? 1 : 0;
    plan.window_axis = -1;
    plan.n_owned = 0;

    // Pencil length: the pair passes give one lane to every home point, so a
    // work unit should hold about one warp of points.
    double per_cell = static_cast<double>(n_points) / static_cast<double>(plan.n_cells_total);
    int pencil = 1;
    if (per_cell > 0.0) {
        pencil = static_cast<int>(std::floor(30.0 / per_cell));
    }
    pencil = std::max(1, std::min({pencil, 8, plan.n_cells[0]}));
    plan.pencil = pencil;
    plan.n_units = ((plan.n_cells[0] + pencil - 1) / pencil) * plan.n_cells[1] * plan.n_cells[2];

    update_screen(plan, cutoff);
    return plan;
}

void make_slab_window(GridPlan& plan, int axis, double lower, double upper, size_t n_points, size_t n_owned, double cutoff) {
    if (axis < 0 || axis > 2 || !plan.periodic[axis]) {
        throw std::runtime_error("the slab direction must be a periodic direction of the box");
    }
    if (!(upper > lower)) {
        throw std::runtime_error("the slab must have a positive thickness");
    }
    const double safe_cutoff = cutoff * (1.0 + 9.5e-10);
    const double thickness = (upper - lower) * plan.face_dist[axis];
    const double layers = std::floor(thickness / safe_cutoff);
    if (layers < 1.0) {
        throw std::runtime_error("the slab of a rank is thinner than the cutoff: use fewer ranks for this system");
    }
    const double width = (upper - lower) / layers; // fractional width of one layer
    if ((upper - lower) + 2.0 * width > 1.0) {
        throw std::runtime_error("slab plus halo is longer than the box: the box must span at least two slabs plus two cutoffs");
    }
    // install the window: one halo layer, the owned layers, one halo layer
    plan.n_cells[axis] = static_cast<int32_t>(layers) + 2;
    plan.n_search[axis] = 1;
    plan.t0[axis] = lower - width;
    plan.scale[axis] = 1.0 / width;
    for (int c = 0; c < 3; c++) {
        plan.cell_vec[axis][c] = plan.H[axis][c] * width;
        plan.origin[c] += plan.t0[axis] * plan.H[axis][c];
    }
    plan.window_axis = axis;
    plan.n_owned = static_cast<int32_t>(n_owned);
    plan.n_cells_total = plan.n_cells[0] * plan.n_cells[1] * plan.n_cells[2];
    plan.n_stencil = (2 * plan.n_search[0] + 1) * (2 * plan.n_search[1] + 1) * (2 * plan.n_search[2] + 1);

    // pencils run along the first direction; they must not mix layers
    double per_cell = static_cast<double>(n_points) / static_cast<double>(plan.n_cells_total);
    int pencil = per_cell > 0.0 ? static_cast<int>(std::floor(30.0 / per_cell)) : 1;
    pencil = std::max(1, std::min({pencil, 8, plan.n_cells[0]}));
    if (axis == 0) {
        pencil = 1;
    }
    plan.pencil = pencil;
    plan.n_units = ((plan.n_cells[0] + pencil - 1) / pencil) * plan.n_cells[1] * plan.n_cells[2];
    update_screen(plan, cutoff);
}

double min_periodic_face_distance(const GridPlan& plan) {
    double result = std::numeric_limits<double>::infinity();
    for (int k = 0; k < 3; k++) {
        if (plan.periodic[k]) {
            result = std::min(result, plan.face_dist[k]);
        }
    }
    return result;
}

} // namespace vb200

// Test helper: the host-side planning code of the engine (vesin_b200/csrc/plan.cpp,
// plain C++) behind a C interface that tests/test_plan_cpu.py calls through ctypes.
#include <cstring>
#include <exception>

#include "plan.hpp"

extern "C" {

struct PlanSummary {
    double H[9];
    double Hinv[9];
    double t0[3];
    double scale[3];
    double cell_vec[9];
    double face_dist[3];
    double origin[3];
    double zero_shift[3];
    double cutoff2;
    double cutoff2_lo;
    double cutoff2_hi;
    int periodic[3];
    int n_cells[3];
    int n_search[3];
    int n_cells_total;
    int pencil;
    int n_units;
    int window_axis;
    int n_owned;
};

static void summarise(const vb200::GridPlan& plan, PlanSummary* out) {
    std::memcpy(out->H, plan.H, sizeof(out->H));
    std::memcpy(out->Hinv, plan.Hinv, sizeof(out->Hinv));
    std::memcpy(out->t0, plan.t0, sizeof(out->t0));
    std::memcpy(out->scale, plan.scale, sizeof(out->scale));
    std::memcpy(out->cell_vec, plan.cell_vec, sizeof(out->cell_vec));
    std::memcpy(out->face_dist, plan.face_dist, sizeof(out->face_dist));
    std::memcpy(out->origin, plan.origin, sizeof(out->origin));
    std::memcpy(out->zero_shift, plan.zero_shift, sizeof(out->zero_shift));
    out->cutoff2 = plan.cutoff2;
    out->cutoff2_lo = plan.cutoff2_lo;
    out->cutoff2_hi = plan.cutoff2_hi;
    for (int k = 0; k < 3; k++) {
        out->periodic[k] = plan.periodic[k];
        out->n_cells[k] = plan.n_cells[k];
        out->n_search[k] = plan.n_search[k];
    }
    out->n_cells_total = plan.n_cells_total;
    out->pencil = plan.pencil;
    out->n_units = plan.n_units;
    out->window_axis = plan.window_axis;
    out->n_owned = plan.n_owned;
}

/// Returns 0, or 1 with the exception's text in `error`.
int plan_check_make(
    const double box[9], const bool periodic[3], const double lower[3], const double upper[3], size_t n_points, double cutoff,
    int full, int sorted, size_t max_cells, int slab_axis, double slab_lower, double slab_upper, size_t n_owned, PlanSummary* out,
    char* error, size_t error_size
) {
    try {
        vb200::PointBounds bounds{};
        for (int c = 0; c < 3; c++) {
            bounds.min[c] = lower[c];
            bounds.max[c] = upper[c];
        }
        vb200::GridPlan plan = vb200::make_plan(box, periodic, bounds, n_points, cutoff, full != 0, sorted != 0, max_cells);
        if (slab_axis >= 0) {
            vb200::make_slab_window(plan, slab_axis, slab_lower, slab_upper, n_points, n_owned, cutoff);
        }
        summarise(plan, out);
        return 0;
    } catch (const std::exception& e) {
        std::strncpy(error, e.what(), error_size - 1);
        error[error_size - 1] = '\0';
        return 1;
    }
}
}

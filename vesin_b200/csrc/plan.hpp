// Host-side geometry of one neighbor-list build: the normalised box, the
// binning frame, the cell grid and the stencil. All of it is a few dozen fp64
// operations on 9 + 6 numbers, so it runs on the host between two launches
// instead of in one-thread kernels.
#ifndef VESIN_B200_PLAN_HPP
#define VESIN_B200_PLAN_HPP

#include <cstddef>
#include <cstdint>
#include <string>

namespace vb200 {

/// Everything the kernels need to know about the box and the cell grid.
/// Passed to kernels by value (fits the parameter space).
struct GridPlan {
    /// Box with the rows of non-periodic directions replaced by unit vectors
    /// orthogonal to the periodic rows. Rows of periodic directions are the
    /// caller's values, bit for bit: they enter the distance predicate.
    double H[3][3];
    /// Inverse of H; t = r . Hinv gives fractional coordinates along periodic
    /// directions and a length along the unit vector of non-periodic ones.
    double Hinv[3][3];
    /// For direction k: cell = floor((t_k - t0[k]) * scale[k]).
    /// periodic: t0 = 0, scale = n_cells; non-periodic: t0 = lower bound of the
    /// projections, scale = 1 / cell width.
    double t0[3];
    double scale[3];
    /// Cartesian step from one cell to the next along each direction
    double cell_vec[3][3];
    /// Distance between opposite faces of H along each direction (periodic
    /// directions), or the extent covered by the cells (non-periodic ones)
    double face_dist[3];
    /// Cartesian position of the corner of cell (0, 0, 0)
    double origin[3];
    int32_t periodic[3];
    int32_t n_cells[3];
    int32_t n_search[3];
    int32_t n_cells_total;
    int32_t n_stencil; // product of (2 * n_search + 1)
    /// Work units of the pair passes: pencils of `pencil` consecutive cells
    /// along the first direction, n_units of them.
    int32_t pencil;
    int32_t n_units;
    /// Output order: 0 = unit after unit (any order is allowed for unsorted
    /// lists), 1 = one row per point in index order (sorted lists).
    int32_t by_index;
    /// Slab decomposition: direction cut into slabs (-1: none). Along it the
    /// cells cover only the window of this rank: layer 0 and the last layer
    /// hold halo points, the layers between hold the owned points; there is
    /// no wrap of the cell index, the image shift of a point is whatever
    /// brings it into the window. Points with local index < n_owned are owned.
    int32_t window_axis;
    int32_t n_owned;

    /// (0 * H[0][c] + 0 * H[1][c]) + 0 * H[2][c]: the signed zero the reference's
    /// shift arithmetic adds to r_j - r_i when S = 0
    double zero_shift[3];
    double cutoff2;   // cutoff * cutoff in fp64: the exact predicate's bound
    float cutoff2_lo; // fp32 screen: below this a candidate is surely inside
    float cutoff2_hi; // fp32 screen: above this a candidate is surely outside
    int32_t full;     // full list (1) or half list (0)
};

/// Largest stencil (product of 2 * n_search + 1 over the directions; for a
/// batch system: of 2 * reach + 1) a build accepts. A larger one means the
/// cutoff is hundreds of box lengths: refused with an error.
constexpr long long MAX_STENCIL_CELLS = 1 << 20;

/// Bounds of the input points, as found by the reduction kernel
struct PointBounds {
    double min[3];
    double max[3];
};

/// Build the plan. Throws std::runtime_error("the box matrix is not
/// invertible") for singular boxes, the message of the reference CPU path
/// (vesin/src/types.hpp:75-78).
GridPlan make_plan(
    const double box[9],
    const bool periodic[3],
    const PointBounds& bounds,
    size_t n_points,
    double cutoff,
    bool full,
    bool sorted,
    size_t max_cells
);

/// Turn a plan of the whole box into the plan of one slab: direction `axis`
/// (periodic) is cut, this rank owns fractional coordinates [lower, upper).
/// Throws when the slab is thinner than the cutoff or the window (slab plus
/// one halo layer on each side) is longer than the box.
void make_slab_window(GridPlan& plan, int axis, double lower, double upper, size_t n_points, size_t n_owned, double cutoff);

/// Smallest distance between opposite faces among periodic directions, or
/// +inf when no direction is periodic (used for the brute-force legality
/// check, vesin/src/vesin_cuda.cpp:404-409).
double min_periodic_face_distance(const GridPlan& plan);

} // namespace vb200

#endif

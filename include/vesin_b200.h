/*
 * Additive entry points of the B200 engine. Nothing here exists in the
 * reference's C API (vesin/include/vesin.h); callers that only know the
 * reference header never need this one.
 */
#ifndef VESIN_B200_H
#define VESIN_B200_H

#include "vesin.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Stages of one build, in launch order (index into the timing array). */
enum VesinB200Stage {
    VesinB200StageBounds = 0,  /* header + min/max + finite check, incl. its read-back */
    VesinB200StageBin = 1,     /* wrap + bin + histogram */
    VesinB200StageScanCells = 2,
    VesinB200StageScatter = 3,
    VesinB200StageCount = 4,   /* pass 1: hit masks + pairs per point */
    VesinB200StageScanRows = 5,
    VesinB200StageEmit = 6,    /* pass 2: writes i, j, S, d, D */
    VesinB200StageCount_ = 7,
};

/* No counterpart in the reference. Switches per-stage device timing (CUDA
 * events on the engine's own stream) on or off for all later calls of
 * vesin_neighbors in this process. Off by default: recording costs a few
 * microseconds per call. */
VESIN_API void vesin_b200_set_profiling(int enabled);

/* No counterpart in the reference. Copies the device time, in milliseconds,
 * of every stage of the LAST build made with `neighbors` into `stage_ms`
 * (VesinB200StageCount_ doubles). Returns 0, or 1 when no timed build was
 * made with this list. */
VESIN_API int vesin_b200_stage_times(const struct VesinNeighborList* neighbors, double* stage_ms);

/* No counterpart in the reference. Version string of this library. */
VESIN_API const char* vesin_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif

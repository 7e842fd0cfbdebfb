// Instantiations of the segment SpMM kernel for vector width 2 (floats per lane per load).
// Kept in a translation unit of its own so the widths compile in parallel.
#include "spmm_kernel.cuh"

#define CFS_ALL(LPR_, V_) \
    CASE(LPR_, 1, 2, V_) CASE(LPR_, 2, 2, V_) CASE(LPR_, 3, 2, V_) \
    CASE(LPR_, 4, 2, V_) CASE(LPR_, 6, 2, V_) CASE(LPR_, 8, 2, V_)
#define CFS_4(LPR_, V_) \
    CASE(LPR_, 1, 2, V_) CASE(LPR_, 2, 2, V_) CASE(LPR_, 3, 2, V_) CASE(LPR_, 4, 2, V_)
#define CFS_2(LPR_, V_) CASE(LPR_, 1, 2, V_) CASE(LPR_, 2, 2, V_)
#define CASE PSPMM_SPMM_CASE

bool pspmm_launch_spmm_vw2(const LaunchShape &s, int V, const SpmmArgs &a, dim3 grid, cudaStream_t st)
{
    if (V == 1) {
        CFS_ALL(8, 1)
        CFS_ALL(16, 1)
        CFS_ALL(32, 1)
    } else if (V == 2) {
        CFS_ALL(16, 2)
        CFS_ALL(32, 2)
    } else if (V == 3) {
        CFS_4(32, 3)
    }
    return false;
}

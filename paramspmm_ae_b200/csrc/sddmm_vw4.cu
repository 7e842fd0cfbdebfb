// Instantiations of the segment SDDMM kernel for vector width 4 (floats per lane per load).
// Kept in a translation unit of its own so the widths compile in parallel.
#include "sddmm_kernel.cuh"

#define CFS_ALL(LPR_, V_) \
    CASE(LPR_, 1, 4, V_) CASE(LPR_, 2, 4, V_) CASE(LPR_, 3, 4, V_) \
    CASE(LPR_, 4, 4, V_) CASE(LPR_, 6, 4, V_) CASE(LPR_, 8, 4, V_)
#define CFS_4(LPR_, V_) \
    CASE(LPR_, 1, 4, V_) CASE(LPR_, 2, 4, V_) CASE(LPR_, 3, 4, V_) CASE(LPR_, 4, 4, V_)
#define CFS_2(LPR_, V_) CASE(LPR_, 1, 4, V_) CASE(LPR_, 2, 4, V_)
#define CASE PSPMM_SDDMM_CASE

bool pspmm_launch_sddmm_vw4(const LaunchShape &s, int V, const SddmmArgs &a, dim3 grid, cudaStream_t st)
{
    if (V == 1) {
        CFS_ALL(2, 1)
        CFS_ALL(4, 1)
        CFS_ALL(8, 1)
        CFS_ALL(16, 1)
        CFS_ALL(32, 1)
    } else if (V == 2) {
        CFS_4(4, 2)
        CFS_4(8, 2)
        CFS_4(16, 2)
        CFS_4(32, 2)
    } else if (V == 3) {
        CFS_2(16, 3)
        CFS_2(32, 3)
    }
    return false;
}

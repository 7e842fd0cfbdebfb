// Instantiations of the segment SpMM kernel for vector width 4 (floats per lane per load).
// Kept in a translation unit of its own so the widths compile in parallel.
#include "spmm_kernel.cuh"

#define CFS_ALL(LPR_, V_) \
    CASE(LPR_, 1, 4, V_) CASE(LPR_, 2, 4, V_) CASE(LPR_, 3, 4, V_) \
    CASE(LPR_, 4, 4, V_) CASE(LPR_, 6, 4, V_) CASE(LPR_, 8, 4, V_)
#define CFS_4(LPR_, V_) \
    CASE(LPR_, 1, 4, V_) CASE(LPR_, 2, 4, V_) CASE(LPR_, 3, 4, V_) CASE(LPR_, 4, 4, V_)
#define CFS_2(LPR_, V_) CASE(LPR_, 1, 4, V_) CASE(LPR_, 2, 4, V_)
#define CASE PSPMM_SPMM_CASE
#define CFS_ALL_MLP(LPR_) \
    PSPMM_SPMM_CASE_MLP(LPR_, 1, 4, 1) PSPMM_SPMM_CASE_MLP(LPR_, 2, 4, 1) PSPMM_SPMM_CASE_MLP(LPR_, 3, 4, 1) \
    PSPMM_SPMM_CASE_MLP(LPR_, 4, 4, 1) PSPMM_SPMM_CASE_MLP(LPR_, 6, 4, 1) PSPMM_SPMM_CASE_MLP(LPR_, 8, 4, 1)

bool pspmm_launch_spmm_vw4(const LaunchShape &s, int V, const SpmmArgs &a, dim3 grid, cudaStream_t st)
{
    if (V == 1) {
        CFS_ALL(2, 1)
        CFS_ALL_MLP(4)
        CFS_ALL_MLP(8)
        CFS_ALL_MLP(16)
        CFS_ALL_MLP(32)
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

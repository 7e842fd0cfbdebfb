// Instantiations of the segment SpMM kernel that add into C (C += A B): vector width 4, CSR and
// split CSR, gather-batch depth 8.  A translation unit of its own so it compiles in parallel.
#include "spmm_kernel.cuh"

#define CFS_ACC(LPR_) \
    PSPMM_SPMM_CASE_ACC(LPR_, 1) PSPMM_SPMM_CASE_ACC(LPR_, 2) PSPMM_SPMM_CASE_ACC(LPR_, 3) \
    PSPMM_SPMM_CASE_ACC(LPR_, 4) PSPMM_SPMM_CASE_ACC(LPR_, 6) PSPMM_SPMM_CASE_ACC(LPR_, 8)

bool pspmm_launch_spmm_vw4_acc(const LaunchShape &s, const SpmmArgs &a, dim3 grid, cudaStream_t st)
{
    CFS_ACC(4)
    CFS_ACC(8)
    CFS_ACC(16)
    CFS_ACC(32)
    return false;
}

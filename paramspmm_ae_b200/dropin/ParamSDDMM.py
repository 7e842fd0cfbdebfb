"""Drop-in module with the function names and positional signatures of the reference's
``ParamSDDMM`` extension (SDDMM/sddmm.cpp:675-701), backed by libpspmm."""
from paramspmm_ae_b200.ops import (  # noqa: F401
    csr_sddmm, csr_split_sddmm, bcsr_sddmm, bcsr_split_sddmm, vec_sddmm, vec_split_sddmm,
    csr_sddmm_profile, csr_split_sddmm_profile, bcsr_sddmm_profile, bcsr_split_sddmm_profile,
    vec_sddmm_profile, vec_split_sddmm_profile, genmask,
)
from paramspmm_ae_b200.baselines import cusparse_sddmm_compute, cusparse_sddmm_profile  # noqa: F401

"""Drop-in module with the function names and positional signatures of the reference's
``ParamSpMM`` extension (SpMM/SpMM.cpp:891-926), backed by libpspmm."""
from paramspmm_ae_b200.ops import (  # noqa: F401
    split_csr, split_csr_par,
    csr_spmm, csr_split_spmm, bcsr_spmm, bcsr_split_spmm, vec_spmm, vec_split_spmm,
    csr_spmm_profile, csr_split_spmm_profile, bcsr_spmm_profile, bcsr_split_spmm_profile,
    vec_spmm_profile, vec_split_spmm_profile,
)
from paramspmm_ae_b200.baselines import (  # noqa: F401
    cusparse_compute, cusparse_profile, cusparse_compute_csr_alg2, cusparse_profile_csr_alg2,
    cusparse_compute_coo_alg4, cusparse_profile_coo_alg4, cusparse_compute_csc, cusparse_profile_csc,
    gespmm_compute, gespmm_profile,
)

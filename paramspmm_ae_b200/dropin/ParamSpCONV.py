"""Drop-in module with the function names and positional signatures of the reference's
``ParamSpCONV`` extension (SpCONV/SpCONV.cpp:496-512), backed by libpspmm (SpMM) and
torch.mm (the dense GEMMs, cuBLAS in the reference too)."""
from paramspmm_ae_b200.ops import (  # noqa: F401
    split_csr, split_csr_par,
    csr_spmm_forward, csr_spmm_backward, csr_split_spmm_forward, csr_split_spmm_backward,
    bcsr_spmm_forward, bcsr_spmm_backward, bcsr_split_spmm_forward, bcsr_split_spmm_backward,
)

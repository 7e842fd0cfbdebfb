"""B200 (sm_100a) implementation of the ParamSpMM sparse hot path: CSR/PCSR x dense SpMM,
pattern-masked SDDMM and the PCSR index builders, behind the reference's extension-module
call surface.

``install_dropin()`` makes ``import ParamSpMM``, ``import ParamSDDMM`` and
``import ParamSpCONV`` resolve to this package, so the reference's Python layers
(PCSR.py, graph_input.py, gnn_conv.py, decider.py) run on it unchanged.
"""
import os
import sys

__version__ = "0.1.0"

_DROPIN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dropin")


def install_dropin():
    """Put the drop-in extension modules on sys.path (idempotent)."""
    if _DROPIN_DIR not in sys.path:
        sys.path.insert(0, _DROPIN_DIR)
    return _DROPIN_DIR

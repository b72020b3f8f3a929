"""naju_b200 — the Naju gated state-space scan as hand-written sm_100a CUDA behind a C ABI.

Same public names as the scan part of the reference package (naju/__init__.py:11):
`naju_scan`, `resolve_backend`; plus the decode step, the multi-GPU helpers and the pipeline for
host-resident tensors.
"""
from .scan import naju_scan, naju_b200_scan, naju_scan_step, resolve_backend  # noqa: F401
from .host import scan_fwd_bwd_host  # noqa: F401

__all__ = ["naju_scan", "naju_b200_scan", "naju_scan_step", "resolve_backend", "scan_fwd_bwd_host"]

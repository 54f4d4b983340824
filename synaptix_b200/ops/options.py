"""Choices between kernels that exist for measurement: which of two ways an operation runs.

Every default is the side that measured faster on a B200.  The switches are values of this
process, set from Python (``set_options(pdl=False)``, or ``with options(attn_tc=False): ...``
in a test or a benchmark); nothing here reads the environment.  The reference keeps such
switches in its runtime options (crates/synaptix-config/src/runtime.rs, ``AttnBackend`` and
``graph`` among them), not in the environment either.

``attn_tc``         prompt attention at head size 128 on tcgen05 (else ``mma.sync``)
``attn_prep``       single-token steps: the attention kernel norms, rotates and stores the new
                    heads itself (else a separate head-preparation launch)
``attn_tma``        single-token steps at head size 64 / 128: pages by TMA, a warp per page (else the
                    cp.async kernel, four warps a page)
``gemm_cut``        the persistent tcgen05 product cuts tiles over K where whole tiles would
                    leave SMs idle
``gemm_cut_few``    a few hundred rows: tiles fewer than the SMs are cut over K too, where an estimate
                    from measured times says that beats whole tiles
``gemm_ws``         2 to 160 rows: the product with the weights as the tensor cores' M side, K shared by
                    the blocks of a cluster (else the tcgen05 product of prompt steps, split over K)
``qkv_epilogue``    prompt steps at head size 128: the q/k/v product prepares the heads in its epilogue (norm,
                    rotation, cache write; else a head-preparation launch)
``fused_residual``  2 to 160 rows: the o / down product adds itself into the residual stream and
                    prepares the next norm
``pdl``             kernels are launched with programmatic dependent launch
"""
from __future__ import annotations

import contextlib
import dataclasses


@dataclasses.dataclass
class KernelOptions:
    attn_tc: bool = True
    attn_prep: bool = True
    attn_tma: bool = True
    gemm_cut: bool = True
    gemm_cut_few: bool = True
    gemm_ws: bool = True
    qkv_epilogue: bool = True
    fused_residual: bool = True
    pdl: bool = True


OPTIONS = KernelOptions()
_NAMES = tuple(f.name for f in dataclasses.fields(KernelOptions))


def set_options(**kw) -> None:
    for k, v in kw.items():
        if k not in _NAMES:
            raise ValueError(f"unknown kernel option {k!r}; there are {', '.join(_NAMES)}")
        setattr(OPTIONS, k, bool(v))
    if "pdl" in kw:
        from ._lib import apply_pdl
        apply_pdl()


@contextlib.contextmanager
def options(**kw):
    """Set options for the length of a ``with`` block.  Steps captured as CUDA graphs keep the
    choice they were recorded with."""
    old = {k: getattr(OPTIONS, k) for k in kw}
    set_options(**kw)
    try:
        yield OPTIONS
    finally:
        set_options(**old)

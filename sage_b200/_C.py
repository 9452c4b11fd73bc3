"""Same public signatures as the reference's compiled extension
(weight_vq/inference/_C.pyi there; bindings at csrc/bindings.cpp:85-87), so
`from sage_b200 import _C` can stand in for `from weight_vq.inference import _C` inside the
reference's `wvq::sage` and `wvq::sphquant` ops."""

from .ops import sage_forward as sage_gemv_forward_cuda  # noqa: F401
from .sphquant import sph_gemv_forward as sph_gemv_forward_cuda  # noqa: F401


def _set_sage_tuning(value: int) -> None:
    """The reference's debug sweep knob (csrc/bindings.cpp:81-84).  Negative restores the
    production dispatch, as there; the sweep values 0-7 have no meaning for these kernels
    and also select the built-in heuristic."""
    from . import _lib

    _lib.check(_lib.load().sageb200_set_tuning(0, 0, 0, 0))

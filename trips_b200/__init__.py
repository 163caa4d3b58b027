"""trips_b200: B200 (sm_100a) implementation of TRIPS's differentiable trilinear point-splatting rasterizer,
its point-parameter store and the fused Adam, behind the reference's operator interface.

The compute lives in libtrips_b200.so (hand-written CUDA, C ABI in include/trips_b200.h); this package is the
host-side mirror of the reference's C++ interface.  Importing the package does not load the library; the first
renderer / optimizer call does, and fails loudly if it was not built (python -m trips_b200.build).
"""
from . import scenes  # noqa: F401
from ._lib import TripsError  # noqa: F401

__all__ = ["scenes", "TripsError"]

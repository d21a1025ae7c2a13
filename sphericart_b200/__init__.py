"""B200 (sm_100a) implementation of sphericart's CUDA hot path: real spherical and solid
harmonics with gradients, Hessians and a fused VJP, behind sphericart's own CUDA interfaces."""

from .spherical_harmonics import SolidHarmonics, SphericalHarmonics  # noqa: F401

__all__ = ["SphericalHarmonics", "SolidHarmonics"]

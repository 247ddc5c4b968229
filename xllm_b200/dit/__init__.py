"""Diffusion-transformer support: step caches and a small DiT used to exercise them."""
from .cache import FBCache, ResidualCache, TaylorSeer, make_cache  # noqa: F401

"""DP-fleet reverse proxy in front of N serving backends (single GPUs or the leaders of tensor-parallel groups)."""
from .keying import affinity_key, fnv64, mix64, rendezvous  # noqa: F401
from .core import AffinityMap, Backend, Fleet  # noqa: F401

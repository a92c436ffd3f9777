"""Group operations from one cluster file: validate, launch plan, group-aware supervisor."""
from .schema import ClusterError, load_cluster, validate  # noqa: F401
from .supervise import Attempt, Policy, classify, supervise  # noqa: F401

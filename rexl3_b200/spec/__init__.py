from .core import AcceptStats, CopyDrafter, NgramDrafter, SpecMode, accept, draft_pick  # noqa: F401
from .arbiter import Arbiter, Choice, DepthCurve  # noqa: F401
from .tree import DraftTree, Lattice, Policy, accept_tree, best_first, with_copy  # noqa: F401
from .stats import MarginBins, PositionStats, mode_of  # noqa: F401
from .selector import SelectorError, SelectorInputs, selector_lattice, selector_walk  # noqa: F401

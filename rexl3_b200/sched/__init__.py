"""Scheduling primitives (no GPU): admission, block pool, prefix index, round planner."""
from .memory import AdmitError, Admission, BlockPool, KvLayout, KvPlane, ModelMemory, MemoryError_  # noqa: F401
from .planner import (CostModel, Demand, DraftCost, Plan, RoundCost, RoundShape, StepCost, TreeDemand, adaptive_block, allocate,  # noqa: F401
                      allocation_order, choose_budget, expected_tokens, plan_round, plan_trees)
from .prefix import BLOCK_TOKENS, CacheBudget, CutPolicy, PrefixIndex, chain_hashes, image_token, plan_cuts  # noqa: F401

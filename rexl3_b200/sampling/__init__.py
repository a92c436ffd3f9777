from .keyed import (GREEDY, MARGIN, Sampling, SamplingError, choose, choose_rows, gumbel, pairwise_sum,  # noqa: F401
                    seed_for, top_candidates, uniform, unit_open)

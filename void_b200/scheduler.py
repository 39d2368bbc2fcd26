"""Row-length analysis that decides whether the Stream-K splitter is worth using.

The reference's scheduler (void/scheduler.py) never launches anything: analyze_workload (:63-147)
turns row-length statistics into a regularity score = max(0, 1 - CoV / 2) (:94-101) and
recommendation strings about CUDA cores versus tensor cores.  On B200 every product runs on the
tensor cores, so what survives is the statistic and one decision: split heavy rows or not.
"""
from dataclasses import dataclass

from .stream_k import analyze_workload_balance


@dataclass
class WorkloadProfile:
    regularity_score: float
    mean_blocks_per_row: float
    imbalance_ratio: float
    coefficient_of_variation: float
    use_stream_k: bool


def analyze_workload(void_tensor, b_shape=None) -> WorkloadProfile:
    """Regularity of the tile-row lengths (void/scheduler.py:90-101, :114-116)."""
    bal = analyze_workload_balance(void_tensor)
    nbr = void_tensor.block_grid[0]
    mean_blocks = void_tensor.n_blocks / max(nbr, 1)
    if bal.get("empty", False):
        return WorkloadProfile(1.0, mean_blocks, 1.0, 0.0, False)
    cov = bal.get("coefficient_of_variation", 0.0)
    cov = 0.0 if cov != cov else cov  # NaN for a single row
    regularity = max(0.0, 1.0 - cov / 2.0)
    # rows several times heavier than the mean cannot be balanced by whole-row assignment
    return WorkloadProfile(regularity, mean_blocks, bal["imbalance_ratio"], cov,
                           use_stream_k=bal["imbalance_ratio"] > 2.0)


__all__ = ["WorkloadProfile", "analyze_workload"]

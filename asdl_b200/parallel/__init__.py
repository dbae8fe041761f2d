"""Data-parallel machinery: owner assignment, process-group helpers, symmetric-memory buffers and
the fused compute+collective kernels' host wrappers."""
from .partition import assign_owners, curvature_cost, shampoo_cost, balance_report

__all__ = ['assign_owners', 'curvature_cost', 'shampoo_cost', 'balance_report']

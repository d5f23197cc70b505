"""Fused CAM read (reference: gdnet/kernel/fused_mem_read/function.py:59-81)."""

from ...ops.functional import fused_mem_read


class FusedMemReadFunction:
    @staticmethod
    def apply(q, gamma, e, buffer_tags, buffer_vals, alpha):
        return fused_mem_read(q, gamma, e, buffer_tags, buffer_vals, alpha)


__all__ = ["fused_mem_read", "FusedMemReadFunction"]

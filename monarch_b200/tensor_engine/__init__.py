"""Distributed tensors and one-sided buffers.

Parity: python/monarch/tensor_engine/__init__.py (RDMABuffer, is_available)."""
from .rdma import RDMABuffer, RDMAError, is_available

__all__ = ["RDMABuffer", "RDMAError", "is_available"]

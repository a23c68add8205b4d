"""One-sided buffers (monarch_rdma; monarch_extension rdma module).
"""
from ..tensor_engine.rdma import RDMABuffer as _RdmaBuffer  # noqa: F401
from ..tensor_engine.rdma import _Manager as _RdmaManager  # noqa: F401

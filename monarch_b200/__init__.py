"""monarch_b200: a B200-native actor-mesh execution engine for PyTorch.

Sub-packages: ``actor`` (actor meshes, endpoints, supervision), ``ops`` (sm_100a
kernels), ``models``, ``parallel`` (DDP/FSDP/TP/PP/EP over NVLink), ``tensor_engine``
(distributed tensors, RDMABuffer), ``utils``.
"""
__version__ = "0.1.0"

"""Message serialisation: cloudpickle with large tensors carried out of band.

Parity: python/monarch/_src/actor/pickle.py (flatten/unflatten; tensors are loaded on the
CPU).  The pickled body travels as the envelope's data, tensor payloads as separate
frame parts that the channel writes with scatter-gather IO (no copy into the body).
"""
from __future__ import annotations

import io
import pickle
import sys
from typing import Any, Callable, List, Optional, Tuple

import cloudpickle

_PLAIN_TYPES = frozenset({str, int, float, bool, type(None), tuple, list, dict, set, frozenset,
                          complex, range, slice})
_OOB_MIN_BYTES = 4096
_OOB_MIN_RAW_BYTES = 65536   # bytes / bytearray payloads of this size travel as parts too


def _torch():
    return sys.modules.get("torch")


class _Pickler(cloudpickle.Pickler):
    def __init__(self, f, parts: List[bytes], extra_pid: Optional[Callable[[Any], Any]]):
        super().__init__(f, protocol=pickle.HIGHEST_PROTOCOL)
        self._parts = parts
        self._extra = extra_pid

    def persistent_id(self, obj):
        # called for every object of the message: the common plain types leave at once
        tp = type(obj)
        if tp in _PLAIN_TYPES:
            return None
        if self._extra is not None:
            r = self._extra(obj)
            if r is not None:
                return ("x", r)
        torch = _torch()
        if torch is not None and type(obj) is torch.Tensor and obj.layout == torch.strided \
                and not getattr(obj, "is_meta", False):
            t = obj.detach()
            if t.device.type != "cpu":
                t = t.cpu()
            t = t.contiguous()
            nbytes = t.numel() * t.element_size()
            if nbytes >= _OOB_MIN_BYTES:
                # a view of the tensor's memory: the native send copies it once, straight
                # into the buffer that goes on the wire
                self._parts.append(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
                return ("t", len(self._parts) - 1, str(t.dtype).split(".")[-1], tuple(t.shape),
                        bool(obj.requires_grad))
        tp = type(obj)
        if (tp is bytes or tp is bytearray) and len(obj) >= _OOB_MIN_RAW_BYTES:
            self._parts.append(obj)
            return ("b" if tp is bytes else "ba", len(self._parts) - 1)
        return None


class _Unpickler(pickle.Unpickler):
    def __init__(self, f, parts: List[bytes], extra_load: Optional[Callable[[Any], Any]]):
        super().__init__(f)
        self._parts = parts
        self._extra = extra_load

    def persistent_load(self, pid):
        if pid[0] == "x":
            if self._extra is None:
                raise pickle.UnpicklingError("message carries references this context cannot resolve")
            return self._extra(pid[1])
        if pid[0] == "t":
            import torch
            _, idx, dtype, shape, req = pid
            raw = self._parts[idx]
            if type(raw) is not bytes:
                raw = bytes(raw)      # same-process delivery hands the sender's view over
            dt = getattr(torch, dtype)
            # a plain local tensor, whatever dispatch mode is active where the message is
            # opened (e.g. a reply read inside ``with mesh.activate():``)
            from torch.utils._python_dispatch import _disable_current_modes
            with _disable_current_modes():
                if len(raw) == 0:
                    t = torch.empty(shape, dtype=dt)
                else:
                    # one copy into storage that torch owns (no Python buffer kept alive by
                    # a tensor that may outlive this interpreter thread)
                    t = torch.empty(len(raw), dtype=torch.uint8)
                    import ctypes
                    ctypes.memmove(t.data_ptr(), raw, len(raw))
                    t = t.view(dt).reshape(shape)
                return t.requires_grad_(req) if req else t
        if pid[0] == "b":
            raw = self._parts[pid[1]]
            return raw if type(raw) is bytes else bytes(raw)
        if pid[0] == "ba":
            return bytearray(self._parts[pid[1]])
        raise pickle.UnpicklingError(f"unknown persistent id {pid!r}")


def flatten(obj: Any, extra_pid: Optional[Callable[[Any], Any]] = None) -> Tuple[bytes, List[bytes]]:
    """Serialise ``obj``; returns (body, out-of-band parts)."""
    parts: List[bytes] = []
    f = io.BytesIO()
    _Pickler(f, parts, extra_pid).dump(obj)
    return f.getvalue(), parts


def unflatten(body: bytes, parts: List[bytes],
              extra_load: Optional[Callable[[Any], Any]] = None) -> Any:
    torch = _torch()
    if torch is not None and torch._C._len_torch_dispatch_stack() > 0:
        # tensors inside the message become plain local tensors, whatever dispatch mode is
        # active where the message is opened (e.g. a reply read under ``mesh.activate()``)
        from torch.utils._python_dispatch import _disable_current_modes
        with _disable_current_modes():
            return _Unpickler(io.BytesIO(body), list(parts), extra_load).load()
    return _Unpickler(io.BytesIO(body), list(parts), extra_load).load()

"""The tensor worker's message set (monarch_messages/src/worker.rs; monarch_extension/src/
tensor_worker.rs).  Messages travel as tuples ``(kind, *fields)``; these constructors build
them with the reference's names and field order checks.
"""
from ...tensor_engine.worker import Ref, TensorWorker  # noqa: F401


def _msg(kind, *names):
    def make(*args, **kwargs):
        vals = list(args)
        for n in names[len(args):]:
            if n not in kwargs:
                raise TypeError(f"{kind}: missing field {n!r}")
            vals.append(kwargs[n])
        if len(vals) != len(names):
            raise TypeError(f"{kind} takes {len(names)} fields {names}, got {len(vals)}")
        return (kind, *vals)
    make.__name__ = kind
    make.fields = names
    return make


StreamRef = int
CallFunction = _msg("call", "seq", "results", "mutates", "function", "args", "kwargs", "stream")
CreateStream = _msg("create_stream", "id", "default")
BorrowCreate = _msg("borrow_create", "borrow", "tensor", "from_stream", "to_stream", "result")
BorrowDrop = _msg("borrow_drop", "borrow")
DeleteRefs = _msg("delete", "refs")
Reduce = _msg("reduce", "seq", "result", "tensor", "comm", "reduction", "scatter", "in_place",
              "out", "stream", "in_meta")
SendTensor = _msg("send_tensor", "seq", "result", "tensor", "from_ranks", "to_ranks", "from_stream",
                  "to_stream")
SplitComm = _msg("split_comm", "key", "groups")
BackendNetworkInit = _msg("init_pg", "addr", "port", "ranks")
CreatePipe = _msg("create_pipe", "pipe", "function", "max_messages", "args", "kwargs", "labels",
                  "offset", "sizes", "strides")
PipeRecv = _msg("pipe_recv", "seq", "results", "pipe", "stream")
SendValue = _msg("pipe_send", "seq", "pipe", "value", "stream")
DefineRecording = _msg("define_recording", "recording", "commands", "temps")
CallRecording = _msg("call_recording", "recording", "bind")


class ReductionType:
    Stack, Sum, Prod, Max, Min, Avg = "stack", "sum", "product", "max", "min", "avg"

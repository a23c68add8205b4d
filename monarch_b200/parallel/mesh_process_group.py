"""A ``torch.distributed`` process group whose collectives are this package's NVLink
kernels (:class:`~monarch_b200.parallel.meshcomm.MeshComm`) instead of NCCL.

The tensor worker hands one to a remote function wherever the controller passed a
``RemoteProcessGroup``: user code written against ``torch.distributed``
(``dist.all_reduce(t, group=pg)``, ``dist.all_gather_into_tensor``, ...) then runs on the
hand-written collectives without ``init_process_group`` ever being called.  Operations are
enqueued on the current CUDA stream and the returned work objects are already complete,
which is the contract NCCL groups give as well (``wait()`` only orders streams).

Parity: the reference wraps its NCCL communicator the same way for user-defined functions
(torch-sys/src/backend.rs:139-360 ``BoxedBackend`` / ``Backend`` over
monarch_tensor_worker/src/comm.rs:466).  Point-to-point ``send``/``recv`` are not offered:
pipeline transfers go through ``to_mesh`` / NCCL p2p.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from .meshcomm import MeshComm

_OPS = {dist.ReduceOp.SUM: "sum", dist.ReduceOp.AVG: "avg", dist.ReduceOp.PRODUCT: "product",
        dist.ReduceOp.MIN: "min", dist.ReduceOp.MAX: "max", dist.ReduceOp.BAND: "band",
        dist.ReduceOp.BOR: "bor", dist.ReduceOp.BXOR: "bxor"}


def _op_name(op) -> str:
    for k, v in _OPS.items():
        if op == k:
            return v
    raise NotImplementedError(f"reduce op {op} is not offered by the NVLink collectives")


def _done(result=None):
    fut = torch.futures.Future()
    fut.set_result(result)
    return torch._C._distributed_c10d._create_work_from_future(fut)


class MeshProcessGroup(dist.ProcessGroup):
    def __init__(self, comm: MeshComm):
        super().__init__(comm.rank, comm.world)
        self.comm = comm
        # torch.distributed looks groups up in its registry (rank translation for
        # broadcast / reduce roots, get_world_size ...): enter this one, with the ranks of the
        # group as the "global" ranks user code names (src=0 is the group's first member)
        from torch.distributed import distributed_c10d as c10d
        c10d._world.pg_map[self] = ("mb200", None)
        c10d._world.pg_names[self] = f"mb200_{id(self):x}"
        c10d._world.pg_group_ranks[self] = {r: r for r in range(comm.world)}

    def getBackendName(self) -> str:
        return "mb200"

    # --------------------------------------------------------------------- reductions
    def allreduce(self, tensors: List[torch.Tensor], opts=None):
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for t in tensors:
            self.comm.all_reduce(t, op, out=t)
        return _done(tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        return self.allreduce(tensors, opts)

    def reduce(self, tensors, opts=None):
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        root = opts.rootRank if opts is not None else 0
        for t in tensors:
            r = self.comm.reduce(t, root, op)
            if r is not None:
                t.copy_(r)
        return _done(tensors)

    def _reduce_scatter_base(self, output, input, opts=None):
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        output.copy_(self.comm.reduce_scatter(input.reshape(self.comm.world, -1), op)
                     .view_as(output))
        return _done(output)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None):
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for out, ins in zip(output_tensors, input_tensors):
            out.copy_(self.comm.reduce_scatter(torch.stack([i.contiguous() for i in ins]), op))
        return _done(output_tensors)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._reduce_scatter_base(o, i, opts)
        return _done(outputs)

    # ------------------------------------------------------------------------- copies
    def broadcast(self, tensors, opts=None):
        root = opts.rootRank if opts is not None else 0
        for t in tensors:
            t.copy_(self.comm.broadcast(t, root))
        return _done(tensors)

    def _allgather_base(self, output, input, opts=None):
        output.copy_(self.comm.all_gather(input).view_as(output))
        return _done(output)

    def allgather(self, output_tensors, input_tensors, opts=None):
        for outs, t in zip(output_tensors, input_tensors):
            g = self.comm.all_gather(t)
            for p, o in enumerate(outs):
                o.copy_(g[p])
        return _done(output_tensors)

    def allgather_coalesced(self, output_lists, input_list, opts=None):
        return self.allgather(output_lists, input_list, opts)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._allgather_base(o, i, opts)
        return _done(outputs)

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=None):
        if output_split_sizes or input_split_sizes:
            raise NotImplementedError("the NVLink all-to-all moves equal splits only")
        W = self.comm.world
        output.copy_(self.comm.all_to_all(input.reshape(W, -1)).view_as(output))
        return _done(output)

    def alltoall(self, output_tensors, input_tensors, opts=None):
        got = self.comm.all_to_all(torch.stack([t.contiguous() for t in input_tensors]))
        for p, o in enumerate(output_tensors):
            o.copy_(got[p])
        return _done(output_tensors)

    def barrier(self, opts=None):
        self.comm.barrier()
        return _done(None)

    # ------------------------------------------------------------------- not offered
    def send(self, tensors, dst, tag=0):
        raise NotImplementedError("point-to-point transfers use to_mesh / NCCL p2p")

    def recv(self, tensors, src, tag=0):
        raise NotImplementedError("point-to-point transfers use to_mesh / NCCL p2p")

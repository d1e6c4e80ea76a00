"""Inter-domain transports: how rows travel between ranks that do NOT share an NVSwitch.

Inside one NVLink domain every byte moves by the hand-written peer-memory kernels of this library. Between
domains the two-level path of :mod:`deepep_efa_b200.parallel.internode` needs exactly one primitive: a
variable-size all-to-all of row blocks among the ranks of a "rail" (the ranks with the same local index in
every domain). :class:`CollectiveTransport` provides it on top of ``torch.distributed`` (NCCL on GPUs, which
reaches InfiniBand / RoCE / EFA through NCCL's own network plugins; gloo on CPUs for the tests).

The reference talks to AWS EFA directly: ``EfaTransport`` / ``EfaEndpoint`` (csrc/transport/efa_transport.cpp:83-472)
open one libfabric RDM endpoint per NIC, register the RDMA buffer via DMA-BUF and post ``fi_writemsg`` with
immediate data; ``EfaWorkerManager`` / ``LLPipelineWorker`` (efa_worker.cpp, ll_pipeline.cpp) drive them from
host threads and ``ImmCounterMap`` (imm_counter.cpp) counts completions per (tag, source). This machine class has
neither libfabric nor GDRCopy nor an EFA NIC, so :class:`EfaTransport` here is a declared stub that fails at
construction with that explanation; the protocol ideas that matter on NVLink (arrival counters that tolerate
early arrival, a slot per source in the receive layout, tags per phase) live in the device kernels instead.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class Transport:
    """Variable-size all-to-all of row blocks among the ranks of one group."""

    name = "abstract"

    def size(self) -> int:
        raise NotImplementedError

    def rank(self) -> int:
        raise NotImplementedError

    def all_to_all_rows(self, rows: torch.Tensor, send_splits: Sequence[int], recv_splits: Sequence[int]) -> torch.Tensor:
        """``rows`` is ``[sum(send_splits), ...]`` ordered by destination; returns ``[sum(recv_splits), ...]`` ordered by source."""
        raise NotImplementedError

    def all_to_all_equal(self, t: torch.Tensor) -> torch.Tensor:
        """``t`` is ``[size * n, ...]``: block i goes to rank i; returns the blocks received, ordered by source."""
        raise NotImplementedError


def group_moves_cuda_tensors(group: dist.ProcessGroup) -> bool:
    """True when the group's backend list has an entry for CUDA tensors (``nccl`` or ``cpu:gloo,cuda:nccl``)."""
    name = str(dist.get_backend(group)).lower()
    try:
        name += "," + str(dist.get_backend_config(group)).lower()
    except Exception:  # older torch: the plain name is all there is
        pass
    return "nccl" in name


class CollectiveTransport(Transport):
    """``torch.distributed.all_to_all_single`` over a process group (NCCL or gloo).

    A caller may hand the library a gloo group (it is all the bootstrap needs: ``all_gather_object`` and barriers). CUDA
    tensors cannot travel over it, so the first CUDA tensor makes every member create, once, an NCCL group over the same
    global ranks and use that from then on; the caller's group keeps serving CPU tensors. Same behaviour as the reference's
    ``Buffer._get_gpu_group`` (deep_ep/buffer.py:228-265).
    """

    name = "torch.distributed"

    def __init__(self, group: Optional[dist.ProcessGroup]) -> None:
        self.group = group
        self._gpu_group: Optional[dist.ProcessGroup] = None
        self._size = group.size() if group is not None else 1
        self._rank = group.rank() if group is not None else 0

    def group_for(self, t: torch.Tensor) -> Optional[dist.ProcessGroup]:
        """The group that can move ``t``: the caller's, or the lazily created NCCL twin for CUDA tensors on a gloo group.
        Collective over the group the first time a CUDA tensor arrives (every member moves the same kind of tensor)."""
        if self.group is None or not t.is_cuda:
            return self.group
        if self._gpu_group is None:
            if group_moves_cuda_tensors(self.group):
                self._gpu_group = self.group
            else:
                ranks = dist.get_process_group_ranks(self.group)
                self._gpu_group = dist.new_group(ranks=ranks, backend="nccl", use_local_synchronization=True)
        return self._gpu_group

    def size(self) -> int:
        return self._size

    def rank(self) -> int:
        return self._rank

    def all_to_all_rows(self, rows, send_splits, recv_splits):
        if rows.element_size() == 1 and rows.dtype != torch.uint8:
            # 8-bit float types travel as bytes: not every collective backend knows them
            return self.all_to_all_rows(rows.view(torch.uint8), send_splits, recv_splits).view(rows.dtype)
        send_splits, recv_splits = [int(s) for s in send_splits], [int(r) for r in recv_splits]
        assert len(send_splits) == self._size and len(recv_splits) == self._size and rows.size(0) == sum(send_splits)
        out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
        if self._size == 1:
            out.copy_(rows)
            return out
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=self.group_for(rows))
        return out

    def all_to_all_equal(self, t):
        out = torch.empty_like(t)
        if self._size == 1:
            out.copy_(t)
            return out
        dist.all_to_all_single(out, t.contiguous(), group=self.group_for(t))
        return out


class EfaTransport(Transport):
    """Placeholder of the reference's libfabric/EFA transport (csrc/transport/efa_transport.h:144-184)."""

    name = "efa"

    def __init__(self, *args, **kwargs) -> None:
        raise NotImplementedError(
            "the EFA transport needs libfabric (rdma/fabric.h), GDRCopy and an EFA NIC, none of which exist on this class "
            "of machine; use CollectiveTransport (NCCL reaches EFA through its aws-ofi-nccl plugin where one is installed)")


def make_subgroups(group: dist.ProcessGroup, ranks_per_node: int):
    """Split ``group`` into NVLink domains of ``ranks_per_node`` consecutive ranks and into rails (same local index
    in every domain). Returns ``(node_group, rail_group)`` of the calling rank. Collective over ``group``."""
    W, r = group.size(), group.rank()
    P = ranks_per_node
    assert W % P == 0, "the group must consist of whole NVLink domains"
    nodes = W // P
    members: List[int] = dist.get_process_group_ranks(group)
    backend = dist.get_backend(group)
    node_group = rail_group = None
    whole_world = W == dist.get_world_size()
    node, local = divmod(r, P)
    # new_group is collective over the default group unless local synchronisation is requested; when `group` is a
    # strict subset of the world only its members are here, so they create just their own two subgroups.
    for n in range(nodes):
        if whole_world or n == node:
            g = dist.new_group([members[n * P + j] for j in range(P)], backend=backend, use_local_synchronization=not whole_world)
            if n == node:
                node_group = g
    for j in range(P):
        if whole_world or j == local:
            g = dist.new_group([members[n * P + j] for n in range(nodes)], backend=backend, use_local_synchronization=not whole_world)
            if j == local:
                rail_group = g
    return node_group, rail_group

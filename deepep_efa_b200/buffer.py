"""``Buffer``: the public expert-parallel communication API (normal and low-latency mode).

The class keeps the names, arguments and return tuples of the reference's ``deep_ep.Buffer``
(deep_ep/buffer.py:80-2852) so that model code written against it runs unchanged, on top of a
different machine model:

* one process per GPU, all GPUs in one NVSwitch domain; peers map each other's symmetric buffer
  with CUDA IPC at construction (reference: deep_ep/buffer.py:146-187, csrc/deep_ep.cpp:419-445);
* normal-mode outputs are carved out of the symmetric arena and written in place by the senders;
  combine pulls expert outputs straight from the peers' symmetric memory;
* low-latency outputs ARE the symmetric landing zone (two parities), so a result stays valid until
  the second next ``low_latency_dispatch`` on this buffer;
* every routing fact a later call needs lives in the returned handle (the reference keeps hidden
  per-buffer state, deep_ep/buffer.py:839-848, 2433-2446);
* a process group whose ranks have no GPU (gloo) selects a pure-PyTorch backend with identical
  results, used for tests and as the semantic reference.

All collectives of one ``Buffer`` must be called by every rank of the group in the same order.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from . import _ext
from .config import Config
from .utils.event import EventHandle, EventOverlap
from .utils.logging import log as _log
from .utils.profiler import PROFILE_ENABLED, PhaseProfiler, nvtx_range
import logging as _logging

topk_idx_t = torch.int64

_NUM_SM_B200 = 148


class EPTimeoutError(RuntimeError):
    """A bounded device-side wait ran out (a peer never arrived). The Buffer must be ``recover()``-ed."""


def _env_timeout_ms() -> float:
    return float(os.environ.get("DEEPEP_TIMEOUT_MS", "10000"))


class Buffer:
    """Expert-parallel communication buffer for one rank.

    Attributes:
        num_sms: default number of CTAs of the normal-mode dispatch/combine kernels (class-wide,
            see :meth:`set_num_sms`).
        rank, group_size, group: position in the communication group.
        num_nvl_bytes: bytes of symmetric memory for normal mode (control block + output arena).
        num_rdma_bytes: bytes of symmetric memory for the low-latency region (the name is kept from
            the reference, where this region is the RDMA buffer).
        runtime: the native per-rank runtime.
    """

    num_sms: int = 32
    # CTAs of the low-latency kernels; None = one CTA per token (+1) for dispatch and every SM for combine
    ll_num_sms: Optional[int] = None

    # ------------------------------------------------------------------------------------------
    # construction / teardown
    # ------------------------------------------------------------------------------------------
    def __init__(self, group: Optional[dist.ProcessGroup], num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 low_latency_mode: bool = False, num_qps_per_rank: int = 24,
                 allow_nvlink_for_low_latency_mode: bool = True, allow_mnnvl: bool = False, use_fabric: bool = False,
                 explicitly_destroy: bool = False, enable_shrink: bool = False, comm=None, *,
                 timeout_ms: Optional[float] = None, num_nvl_ranks: Optional[int] = None,
                 _virtual: Optional[Tuple[int, int]] = None) -> None:
        """Create the buffer and exchange peer mappings (collective over ``group``).

        Arguments follow the reference (deep_ep/buffer.py:99-131). ``num_qps_per_rank``,
        ``allow_nvlink_for_low_latency_mode``, ``allow_mnnvl`` and ``use_fabric`` describe the RDMA /
        fabric transports of the reference and are accepted and ignored on a single NVSwitch box.
        ``timeout_ms`` bounds every device-side wait (default: env ``DEEPEP_TIMEOUT_MS`` or 10 s).
        ``enable_shrink`` makes low-latency waits mask a silent rank instead of failing the call.
        ``num_nvl_ranks`` (default: env ``DEEPEP_NVL_DOMAIN_SIZE`` or 8) is the size of one NVLink domain; a larger
        group runs the two-level path of :mod:`deepep_efa_b200.parallel.internode` (NVLink kernels inside every
        domain, collectives between them), where the reference uses NCCL + libfabric/EFA
        (deep_ep/buffer.py:193-226, 582-1560).
        """
        self.num_nvl_bytes = int(num_nvl_bytes)
        self.num_rdma_bytes = int(num_rdma_bytes)
        self.low_latency_mode = low_latency_mode
        self.explicitly_destroy = explicitly_destroy
        self.enable_shrink = enable_shrink
        self._destroyed = False
        self._cpu = None
        self._ll_cache = {}
        self._ll_parity = 0
        self._virtual_peers: Optional[List["Buffer"]] = None
        self._hier = None
        self._ll_mask_local = None
        if allow_mnnvl or use_fabric:
            # fabric / multi-node NVLink handles are not built: peers are mapped with plain CUDA IPC, which covers one box
            _log(_logging.WARNING, group.rank() if group is not None else 0,
                 "allow_mnnvl / use_fabric are ignored: this library maps peers with CUDA IPC inside one NVSwitch domain")

        if _virtual is not None:
            self.rank, self.group_size = _virtual
            self.group = None
            all_gather_object = None
        elif group is not None:
            self.rank, self.group_size, self.group = group.rank(), group.size(), group

            def all_gather_object(obj):
                out = [None] * self.group_size
                dist.all_gather_object(out, obj, group)
                return out
        elif comm is not None:
            self.rank, self.group_size, self.group = comm.Get_rank(), comm.Get_size(), comm

            def all_gather_object(obj):
                return comm.allgather(obj)
        else:
            raise ValueError("Either 'group' or 'comm' must be provided.")

        nvl = int(num_nvl_ranks if num_nvl_ranks is not None else os.environ.get("DEEPEP_NVL_DOMAIN_SIZE", "8"))
        assert 1 <= nvl <= 8, "an NVLink domain of this library has at most 8 ranks"
        if _virtual is None and self.group_size > nvl:
            if group is None:
                raise NotImplementedError("groups larger than one NVLink domain need a torch.distributed process group")
            from .parallel.internode import HierarchicalEP
            self.runtime = None
            self._hier = HierarchicalEP(group, nvl, lambda g: Buffer(
                g, num_nvl_bytes, num_rdma_bytes, low_latency_mode, num_qps_per_rank, allow_nvlink_for_low_latency_mode, allow_mnnvl,
                use_fabric, True, enable_shrink, timeout_ms=timeout_ms, num_nvl_ranks=nvl))
            nb = self._hier.node_buf
            if nb._cpu is None:
                self._C, self.device, self.comm_stream = nb._C, nb.device, nb.comm_stream
            return

        if not torch.cuda.is_available():
            # CPU ranks (gloo): pure-PyTorch backend with the same semantics.
            from .parallel.gloo_backend import GlooBackend
            self._cpu = GlooBackend(self.rank, self.group_size, group)
            self.runtime = None
            return

        self._C = _ext.load()
        device = torch.cuda.current_device()
        self.device = torch.device("cuda", device)
        self.runtime = self._C.Runtime(self.rank, self.group_size, self.num_nvl_bytes, self.num_rdma_bytes, device,
                                       timeout_ms if timeout_ms is not None else _env_timeout_ms(), bool(enable_shrink))
        self.comm_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.runtime.set_comm_stream(self.comm_stream.cuda_stream)
        if _virtual is None:
            from .utils.nvlink import check_nvlink_connections
            check_nvlink_connections(group)
            device_ids = all_gather_object(device)
            handles = all_gather_object(bytes(self.runtime.ipc_handle()))
            assert len(set(device_ids)) == len(device_ids) or self.group_size == 1, \
                "every rank of the group must own a different GPU"
            self.runtime.open_peers(handles)
            torch.cuda.synchronize()
            if group is not None and self.group_size > 1:
                dist.barrier(group)
            assert self.runtime.is_available()

    def destroy(self) -> None:
        """Release the symmetric buffer (collective: every rank must call it)."""
        if self._destroyed:
            return
        self._destroyed = True
        if self._hier is not None:
            self._hier.destroy()
            return
        if self._cpu is not None or self.runtime is None:
            return
        torch.cuda.synchronize()
        if self.group is not None and self.group_size > 1 and isinstance(self.group, dist.ProcessGroup):
            dist.barrier(self.group)
        self._ll_cache.clear()
        self.runtime.release()

    def __del__(self):
        try:
            if not getattr(self, "explicitly_destroy", True) and not getattr(self, "_destroyed", True):
                if self.runtime is not None:
                    self._ll_cache.clear()
                    self.runtime.release()
        except Exception:
            pass

    # ------------------------------------------------------------------------------------------
    # housekeeping API
    # ------------------------------------------------------------------------------------------
    @staticmethod
    def is_sm90_compiled() -> bool:
        """Kept for API compatibility: the kernels here are sm_100a-only, which includes every
        sm_90-era feature the reference tests for (csrc/deep_ep.cpp is_sm90_compiled)."""
        return True

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        """Set the default CTA count of the normal-mode kernels. The reference requires an even number
        (sender/receiver CTA pairs, deep_ep/buffer.py:282-292); any positive number works here."""
        assert new_num_sms > 0
        Buffer.num_sms = int(new_num_sms)

    @staticmethod
    def set_low_latency_num_sms(new_num_sms: Optional[int]) -> None:
        """Bound the grid of the low-latency kernels (``None`` restores the default: one CTA per token for dispatch,
        every SM for combine). With the receive hook this leaves the remaining SMs to a GEMM that runs between the two
        halves; the kernels stride over tokens, so any value >= 2 is valid."""
        assert new_num_sms is None or new_num_sms >= 2
        Buffer.ll_num_sms = None if new_num_sms is None else int(new_num_sms)

    @staticmethod
    def capture() -> EventOverlap:
        """An event recorded on the current stream (deep_ep/buffer.py:294-302)."""
        return EventOverlap(EventHandle())

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int,
                                       num_experts: int) -> int:
        """Bytes of ``num_rdma_bytes`` the low-latency mode needs for this shape."""
        from .config import get_low_latency_rdma_size_hint
        return get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks, num_experts)

    # Accessors of the reference's runtime object (csrc/deep_ep.cpp:308-358), answered for one NVSwitch domain.
    def is_available(self) -> bool:
        if self._hier is not None:
            return self._hier.node_buf.is_available()
        return self._cpu is not None or (self.runtime is not None and self.runtime.is_available())

    def get_num_rdma_ranks(self) -> int:
        """Number of NVLink domains of the group (the reference's ``num_rdma_ranks``, csrc/deep_ep.cpp:243-244)."""
        return self._hier.num_nodes if self._hier is not None else 1

    def get_rdma_rank(self) -> int:
        return self._hier.node if self._hier is not None else 0

    def get_root_rdma_rank(self, global_: bool = True) -> int:
        if self._hier is None:
            return 0
        return self._hier.node * self._hier.P if global_ else 0

    def get_local_device_id(self) -> int:
        if self._hier is not None:
            return self._hier.node_buf.get_local_device_id()
        return self.device.index if self._cpu is None else -1

    def get_local_ipc_handle(self) -> bytes:
        if self._hier is not None:
            return self._hier.node_buf.get_local_ipc_handle()
        return bytes(self.runtime.ipc_handle())

    def get_comm_stream(self) -> "torch.cuda.Stream":
        return self.comm_stream

    def get_local_buffer_tensor(self, dtype: torch.dtype, size: Optional[torch.Size] = None, offset: int = 0,
                                use_rdma_buffer: bool = False) -> torch.Tensor:
        """A view of this rank's symmetric memory: the arena part (default) or the low-latency region."""
        if self._hier is not None:
            return self._hier.node_buf.get_local_buffer_tensor(dtype, size, offset, use_rdma_buffer)
        ctrl = self._C.CONTROL_BYTES
        base = ctrl if use_rdma_buffer else ctrl + self.runtime.ll_bytes()
        total = self.runtime.ll_bytes() if use_rdma_buffer else self.runtime.total_bytes() - base
        esz = torch.empty((), dtype=dtype).element_size()
        numel = (total - offset) // esz
        t = self.runtime.view(base + offset, [numel], dtype)
        return t if size is None else t[:size.numel()].view(size)

    def empty_symmetric(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Allocate a tensor inside this rank's peer-mapped arena. A combine whose input lives there is
        zero-copy; anything else is staged through one local copy first."""
        if self._hier is not None:
            return self._hier.node_buf.empty_symmetric(shape, dtype)
        if self._cpu is not None or self.runtime is None:
            return torch.empty(list(shape), dtype=dtype)  # CPU backend: there is no peer-mapped memory, an ordinary tensor serves
        return self.runtime.alloc_symmetric(list(shape), dtype)

    @staticmethod
    def _unpack_bias(bias):
        b0, b1 = None, None
        if isinstance(bias, torch.Tensor):
            b0 = bias
        elif isinstance(bias, tuple):
            assert len(bias) == 2
            b0, b1 = bias
        return b0, b1

    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        """Recommended dispatch config per group size (re-tuned for B200; the reference's table is at
        deep_ep/buffer.py:361-389)."""
        from .config import DISPATCH_CONFIGS
        assert num_ranks in DISPATCH_CONFIGS, f"Unsupported number of EP ranks: {num_ranks}"
        return Config(*DISPATCH_CONFIGS[num_ranks])

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        from .config import COMBINE_CONFIGS
        assert num_ranks in COMBINE_CONFIGS, f"Unsupported number of EP ranks: {num_ranks}"
        return Config(*COMBINE_CONFIGS[num_ranks])

    # ------------------------------------------------------------------------------------------
    # status / recovery
    # ------------------------------------------------------------------------------------------
    def check_status(self, sync: bool = False) -> None:
        """Raise :class:`EPTimeoutError` if a kernel of this buffer reported a timed-out wait."""
        if self._hier is not None:
            return self._hier.node_buf.check_status(sync)
        if self.runtime is None:
            return
        if sync:
            torch.cuda.synchronize()
        if self.runtime.status_code() != 0:
            raise EPTimeoutError(self.runtime.status_string())
        if sync:
            # the grouped GEMM reports through a per-device word (1 = a bounded pipeline wait ran out, 2 = a group of the
            # natively block-scaled kernel does not start on a 128-row boundary); reading it synchronises, so it is only
            # looked at here
            err = self._C.gemm_error(self.device.index)
            if err != 0:
                self._C.gemm_clear_error(self.device.index)
                raise EPTimeoutError(f"grouped GEMM reported error {err} " +
                                     ("(pipeline wait timed out)" if err == 1 else "(group start not on a 128-row boundary)"))

    def recover(self) -> None:
        """Collective reset after an error: zero the control block and all sequence state."""
        if self._hier is not None:
            return self._hier.node_buf.recover()
        if self.runtime is None:
            return
        _log(_logging.WARNING, self.rank, f"recovering buffer after: {self.runtime.status_string()}")
        torch.cuda.synchronize()
        if self.group is not None and self.group_size > 1:
            dist.barrier(self.group)
        self.runtime.reset_control()
        self._ll_parity = 0
        for views in self._ll_cache.values():  # sequences restart: no row-number word may keep a tag of the old numbering
            for v in views:
                v["send_row"].zero_()
        torch.cuda.synchronize()
        if self.group is not None and self.group_size > 1:
            dist.barrier(self.group)

    # ------------------------------------------------------------------------------------------
    # normal mode
    # ------------------------------------------------------------------------------------------
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventOverlap] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """Count tokens per rank / expert and build the membership matrix.

        Returns ``(num_tokens_per_rank[R] i32, None, num_tokens_per_expert[E] i32, is_token_in_rank[T,R] bool,
        event)``; the second entry (tokens per RDMA rank = per NVLink domain, i32 ``[domains]``) is ``None`` when the
        group is a single NVLink domain (deep_ep/buffer.py:422-448).
        """
        topk_idx = _as_topk_idx(topk_idx)
        if self._hier is not None:
            _wait_previous(previous_event)
            return self._hier.get_dispatch_layout(topk_idx, num_experts)
        if self._cpu is not None:
            a, b, c = self._cpu.get_dispatch_layout(topk_idx, num_experts)
            return a, None, b, c, EventOverlap()
        with _CommScope(self, previous_event, async_finish, allocate_on_comm_stream, (topk_idx,)) as scope:
            per_rank, per_expert, in_rank = self._C.get_dispatch_layout(self.runtime, topk_idx, num_experts)
            scope.outputs(per_rank, per_expert, in_rank)
        return per_rank, None, per_expert, in_rank, scope.event

    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], handle: Optional[Tuple] = None,
                 num_tokens_per_rank: Optional[torch.Tensor] = None, num_tokens_per_rdma_rank: Optional[torch.Tensor] = None,
                 is_token_in_rank: Optional[torch.Tensor] = None, num_tokens_per_expert: Optional[torch.Tensor] = None,
                 topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                 expert_alignment: int = 1, num_worst_tokens: int = 0, config: Optional[Config] = None,
                 previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                 allocate_on_comm_stream: bool = False, *, quantize_fp8: bool = False, round_scale: bool = False):
        """Send every token to the ranks that own its selected experts.

        Same arguments and return tuple as the reference (deep_ep/buffer.py:451-531):
        ``(recv_x, recv_topk_idx, recv_topk_weights, num_recv_tokens_per_expert_list, handle, event)``.
        ``x`` is bf16 ``[T, hidden]`` or an ``(e4m3 [T, hidden], f32 scales [T, hidden/128])`` pair and
        ``recv_x`` has the same form. With a ``handle`` from an earlier dispatch the layout is reused
        (only ``x`` travels, four ``None`` placeholders are returned). ``num_worst_tokens > 0`` sizes the
        outputs for that many rows and skips the host synchronisation (CUDA-graph friendly).

        Extension: ``quantize_fp8=True`` takes bf16 ``x`` and casts rows to e4m3 with one fp32 scale per
        128 channels inside the dispatch kernel, returning an ``(e4m3, scales)`` pair.

        Rows of ``recv_x`` are ordered by source rank, then by token order at the source. The returned
        tensors live in this rank's symmetric arena; their memory returns to the arena when they die.
        """
        topk_idx = _as_topk_idx(topk_idx)
        if self._hier is not None:
            return self.internode_dispatch(x, handle, num_tokens_per_rank, num_tokens_per_rdma_rank, is_token_in_rank,
                                           num_tokens_per_expert, topk_idx, topk_weights, expert_alignment, num_worst_tokens, config,
                                           previous_event, async_finish, allocate_on_comm_stream, quantize_fp8=quantize_fp8,
                                           round_scale=round_scale)
        if self._cpu is not None:
            return self._cpu.dispatch(x, handle, num_tokens_per_rank, is_token_in_rank, num_tokens_per_expert, topk_idx,
                                      topk_weights, expert_alignment, num_worst_tokens)
        req = _DispatchReq(x, handle, num_tokens_per_rank, is_token_in_rank, num_tokens_per_expert, topk_idx, topk_weights,
                           expert_alignment, num_worst_tokens, quantize_fp8, round_scale)
        config = self.get_dispatch_config(self.group_size) if config is None else config
        return _dispatch_many([self], [req], config, previous_event, async_finish, allocate_on_comm_stream)[0]

    def combine(self, x: torch.Tensor, handle: Tuple, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor], None] = None, config: Optional[Config] = None,
                previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                allocate_on_comm_stream: bool = False):
        """Reduce expert outputs back to the tokens' home ranks (un-weighted fp32 sum + optional biases, bf16 out).

        Returns ``(combined_x [T, hidden], combined_topk_weights or None, event)`` (deep_ep/buffer.py:534-579).
        If ``x`` already lives in the symmetric arena (a dispatch result, or a tensor from
        :meth:`empty_symmetric`) it is read in place by the peers; otherwise it is staged with one local copy.
        """
        if self._hier is not None:
            return self.internode_combine(x, handle, topk_weights, bias, config, previous_event, async_finish, allocate_on_comm_stream)
        if self._cpu is not None:
            return self._cpu.combine(x, handle, topk_weights, bias)
        config = self.get_combine_config(self.group_size) if config is None else config
        return _combine_many([self], [(x, handle, topk_weights, bias)], config, previous_event, async_finish,
                             allocate_on_comm_stream)[0]

    # Groups that span several NVLink domains (the reference's "internode" paths).
    def internode_dispatch(self, x, handle: Optional[Tuple] = None, num_tokens_per_rank: Optional[torch.Tensor] = None,
                           num_tokens_per_rdma_rank: Optional[torch.Tensor] = None, is_token_in_rank: Optional[torch.Tensor] = None,
                           num_tokens_per_expert: Optional[torch.Tensor] = None, topk_idx: Optional[torch.Tensor] = None,
                           topk_weights: Optional[torch.Tensor] = None, expert_alignment: int = 1, num_worst_tokens: int = 0,
                           config: Optional[Config] = None, previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                           allocate_on_comm_stream: bool = False, *, quantize_fp8: bool = False, round_scale: bool = False):
        """Dispatch across NVLink domains: one rail hop per destination domain, then the NVLink dispatch kernel inside the
        domain (see :mod:`deepep_efa_b200.parallel.internode`). Same arguments and return tuple as the reference
        (deep_ep/buffer.py:582-861); the handle is a self-contained 10-tuple. ``dispatch`` routes here automatically when
        the group is larger than one NVLink domain. Work is issued on the current stream; ``event`` marks its end."""
        if self._hier is None:
            raise NotImplementedError("this group is a single NVLink domain: use dispatch()")
        _wait_previous(previous_event)
        config = self.get_dispatch_config(self._hier.P) if config is None else config
        out = self._hier.dispatch(x, handle, num_tokens_per_rank, num_tokens_per_rdma_rank, is_token_in_rank, num_tokens_per_expert,
                                  _as_topk_idx(topk_idx), topk_weights, expert_alignment, num_worst_tokens, config, quantize_fp8, round_scale)
        return out[:5] + (_end_event(self),)

    def internode_combine(self, x: torch.Tensor, handle: Tuple, topk_weights: Optional[torch.Tensor] = None,
                          bias: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor], None] = None, config: Optional[Config] = None,
                          previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                          allocate_on_comm_stream: bool = False):
        """Combine across NVLink domains: NVLink reduction per domain, one partial per domain back over the rail, fp32 sum
        at the home rank (reference: deep_ep/buffer.py:1437-1560)."""
        if self._hier is None:
            raise NotImplementedError("this group is a single NVLink domain: use combine()")
        _wait_previous(previous_event)
        config = self.get_combine_config(self._hier.P) if config is None else config
        out, out_w, _ = self._hier.combine(x, handle, topk_weights, bias, config)
        return out, out_w, _end_event(self)

    # ------------------------------------------------------------------------------------------
    # low-latency mode
    # ------------------------------------------------------------------------------------------
    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int = 0, hidden: int = 0, num_experts: int = 0) -> None:
        """Collective reset of all signalling state. Sequence numbers are monotonic, so this is only
        needed after an error or a shrink event (reference: deep_ep/buffer.py:1562-1584)."""
        if self._cpu is not None or self._hier is not None:
            return
        self.recover()

    def _ll_views(self, num_max_tokens: int, hidden: int, num_experts: int):
        key = (num_max_tokens, hidden, num_experts)
        v = self._ll_cache.get(key)
        if v is not None:
            return v
        lay = self._C.ll_layout(self.runtime, num_max_tokens, hidden, num_experts)
        if lay["total_bytes"] > lay["available_bytes"]:
            raise RuntimeError(
                f"low-latency region too small: need {lay['total_bytes']} B, have {lay['available_bytes']} B; create the "
                f"Buffer with num_rdma_bytes=Buffer.get_low_latency_rdma_size_hint(...)")
        R = self.group_size
        L, N = num_experts // R, R * num_max_tokens
        rt = self.runtime
        v = []
        for p in range(2):
            d = dict(
                x_fp8=rt.view(lay["recv_x"][p], [L, N, hidden], torch.float8_e4m3fn),
                x_bf16=rt.view(lay["recv_x"][p], [L, N, hidden], torch.bfloat16),
                scales=rt.view(lay["recv_scales"][p], [L, N, hidden // 128], torch.float32),
                scales_ue8m0=rt.view(lay["recv_scales"][p], [L, N, max(hidden // 512, 1)], torch.int32),
                src_info=rt.view(lay["recv_src_info"][p], [L, N], torch.int32),
                combine_src=rt.view(lay["combine_src"][p], [L, N, hidden], torch.bfloat16),
                count=torch.zeros(L, dtype=torch.int32, device=self.device),
                layout_range=torch.zeros(L, R, dtype=torch.int64, device=self.device),
                # row of every (token, k) selection at its expert's rank, written by dispatch and read by the pull form of
                # combine; lives as long as the handle's tensors (until the second next dispatch)
                # (words are (call tag << 16) | (row + 1); zero = never written)
                send_row=torch.zeros(num_max_tokens * 32, dtype=torch.int32, device=self.device),
            )
            v.append(d)
        self._ll_cache[key] = v
        return v

    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int,
                             num_experts: int, cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                             dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, async_finish: bool = False,
                             return_recv_hook: bool = False, topk_weights: Optional[torch.Tensor] = None):
        """Low-latency dispatch (one kernel, no host synchronisation, CUDA-graph friendly).

        Returns ``(packed_recv_x, packed_recv_count, handle, event, hook)`` as the reference
        (deep_ep/buffer.py:1816-2457): ``packed_recv_x`` is ``[L, N, hidden]`` e4m3 plus scales
        ``[L, N, hidden/128]`` f32 (``[L, N, hidden/512]`` int32 with ``use_ue8m0``) when ``use_fp8``, else bf16;
        only the first ``packed_recv_count[e]`` rows of expert ``e`` are valid. ``handle`` is
        ``(src_info [L,N] i32, layout_range [L,R] i64 = begin<<32|count, num_max_dispatch_tokens_per_rank, hidden,
        num_experts)``. The returned tensors are views of the symmetric landing zone and stay valid until the
        second next low-latency dispatch. ``topk_weights`` is accepted for signature parity and unused.
        With ``return_recv_hook`` only the send half runs now and ``hook()`` launches the receive half.
        """
        topk_idx = _as_topk_idx(topk_idx)
        if self._hier is not None:
            # across NVLink domains: the collective fallback (count exchange, packed rows, one all-to-all, scatter)
            rx, cnt, h, _, _ = self._hier.low_latency_dispatch(x, topk_idx, num_max_dispatch_tokens_per_rank, num_experts, use_fp8,
                                                               round_scale, use_ue8m0, cumulative_local_expert_recv_stats)
            return rx, cnt, h, _end_event(self), ((lambda: None) if return_recv_hook else None)
        if self._cpu is not None:
            return self._cpu.low_latency_dispatch(x, topk_idx, num_max_dispatch_tokens_per_rank, num_experts, use_fp8,
                                                  round_scale, use_ue8m0, cumulative_local_expert_recv_stats, return_recv_hook)
        assert not (async_finish and return_recv_hook)
        if PROFILE_ENABLED:
            prof = self.__dict__.setdefault("_ll_dispatch_profiler", PhaseProfiler("LL-DISPATCH", self.rank))
            prof.mark("start")
            res = _ll_dispatch_many([self], [(x, topk_idx, cumulative_local_expert_recv_stats, dispatch_wait_recv_cost_stats)],
                                    num_max_dispatch_tokens_per_rank, num_experts, use_fp8, round_scale, use_ue8m0, async_finish,
                                    return_recv_hook)[0]
            prof.mark("kernel")
            prof.finish_iter()
            return res
        return _ll_dispatch_many([self], [(x, topk_idx, cumulative_local_expert_recv_stats, dispatch_wait_recv_cost_stats)],
                                 num_max_dispatch_tokens_per_rank, num_experts, use_fp8, round_scale, use_ue8m0, async_finish,
                                 return_recv_hook)[0]

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            use_logfmt: bool = False, zero_copy: bool = False, async_finish: bool = False,
                            return_recv_hook: bool = False, out: Optional[torch.Tensor] = None,
                            combine_wait_recv_cost_stats: Optional[torch.Tensor] = None):
        """Low-latency combine: ``out[t] = sum_k topk_weights[t,k] * x[expert k, slot of t]`` in fp32, bf16 out.

        Returns ``(combined_x [T, hidden], event, hook)`` (deep_ep/buffer.py:2460-2803). With ``zero_copy`` the
        input is read from the buffer returned by :meth:`get_next_low_latency_combine_buffer` and ``x`` is ignored.
        ``use_logfmt`` (a 10-bit wire format of upstream DeepEP) is accepted and ignored: rows travel as bf16.
        """
        topk_idx = _as_topk_idx(topk_idx)
        if self._hier is not None:
            if zero_copy:
                x = self.get_next_low_latency_combine_buffer(handle)
            res, _, _ = self._hier.low_latency_combine(x, topk_idx, topk_weights, handle, out)
            return res, _end_event(self), ((lambda: None) if return_recv_hook else None)
        if self._cpu is not None:
            return self._cpu.low_latency_combine(x, topk_idx, topk_weights, handle, out, return_recv_hook)
        assert not (async_finish and return_recv_hook)
        if PROFILE_ENABLED:
            prof = self.__dict__.setdefault("_ll_combine_profiler", PhaseProfiler("LL-COMBINE", self.rank))
            prof.mark("start")
            res = _ll_combine_many([self], [(x, topk_idx, topk_weights, handle, out, combine_wait_recv_cost_stats)], zero_copy,
                                   async_finish, return_recv_hook)[0]
            prof.mark("kernel")
            prof.finish_iter()
            return res
        return _ll_combine_many([self], [(x, topk_idx, topk_weights, handle, out, combine_wait_recv_cost_stats)], zero_copy,
                                async_finish, return_recv_hook)[0]

    def get_next_low_latency_combine_buffer(self, handle: tuple) -> torch.Tensor:
        """The symmetric ``[L, N, hidden]`` bf16 buffer the next ``low_latency_combine(..., zero_copy=True)`` with
        this handle reads; let the expert GEMM write its output here (deep_ep/buffer.py:2831-2852)."""
        src_info, _, num_max_tokens, hidden, num_experts = handle[:5]
        if self._hier is not None:
            key = ("hier_combine_src", num_max_tokens, hidden, num_experts)
            if key not in self._ll_cache:
                self._ll_cache[key] = torch.empty(num_experts // self.group_size, self.group_size * num_max_tokens, hidden,
                                                  dtype=torch.bfloat16, device=src_info.device)
            return self._ll_cache[key]
        if self._cpu is not None:
            return self._cpu.get_next_low_latency_combine_buffer(handle)
        views = self._ll_views(num_max_tokens, hidden, num_experts)
        return views[_parity_of(views, src_info)]["combine_src"]

    def low_latency_update_mask_buffer(self, rank_to_mask: int, mask: bool = False) -> None:
        """Mask (or unmask) a rank: low-latency kernels stop sending to it and stop waiting for it. The mask is
        device memory the kernels read (the reference keeps a Python-side tensor no kernel consults,
        deep_ep/buffer.py:2805-2829)."""
        if self._hier is not None:
            # across NVLink domains the collective fallback has no waits to shorten: the mask is recorded and reported only
            self._hier_mask()[rank_to_mask] = 1 if mask else 0
            return
        if self._cpu is not None:
            return self._cpu.update_mask(rank_to_mask, mask)
        self.runtime.set_mask(rank_to_mask, mask)

    def _hier_mask(self) -> torch.Tensor:
        if self._ll_mask_local is None:
            self._ll_mask_local = torch.zeros(self.group_size, dtype=torch.int32)
        return self._ll_mask_local

    def low_latency_query_mask_buffer(self, mask_status: torch.Tensor) -> None:
        if self._hier is not None:
            mask_status.copy_(self._hier_mask())
            return
        if self._cpu is not None:
            return self._cpu.query_mask(mask_status)
        self.runtime.query_mask(mask_status)

    def low_latency_clean_mask_buffer(self) -> None:
        if self._hier is not None:
            self._hier_mask().zero_()
            return
        if self._cpu is not None:
            return self._cpu.clean_mask()
        self.runtime.clean_mask()

    # test hook: a wait that nothing satisfies must come back as a status, not as a hang
    def _timeout_probe(self) -> None:
        self._C.timeout_probe(self.runtime)


# ================================================================================================
# helpers shared by the single-rank API above and the single-GPU multi-rank emulation
# ================================================================================================
def _wait_previous(previous_event) -> None:
    if previous_event is not None:
        previous_event.current_stream_wait()


def _end_event(buf) -> EventOverlap:
    return EventOverlap(EventHandle()) if torch.cuda.is_available() else EventOverlap()


def _as_topk_idx(topk_idx):
    """The kernels take int64 expert ids (``topk_idx_t``); int32 ids (the reference's TOPK_IDX_BITS=32 build,
    csrc/kernels/configs.cuh:66-72) are widened."""
    if topk_idx is not None and topk_idx.dtype != torch.int64:
        return topk_idx.to(torch.int64)
    return topk_idx


class _DispatchReq:
    __slots__ = ("x", "handle", "num_tokens_per_rank", "is_token_in_rank", "num_tokens_per_expert", "topk_idx",
                 "topk_weights", "expert_alignment", "num_worst_tokens", "quantize_fp8", "round_scale")

    def __init__(self, x, handle, num_tokens_per_rank, is_token_in_rank, num_tokens_per_expert, topk_idx, topk_weights,
                 expert_alignment, num_worst_tokens, quantize_fp8=False, round_scale=False):
        self.x, self.handle = x, handle
        self.num_tokens_per_rank, self.is_token_in_rank = num_tokens_per_rank, is_token_in_rank
        self.num_tokens_per_expert, self.topk_idx, self.topk_weights = num_tokens_per_expert, topk_idx, topk_weights
        self.expert_alignment, self.num_worst_tokens = expert_alignment, num_worst_tokens
        self.quantize_fp8, self.round_scale = quantize_fp8, round_scale


class _CommScope:
    """Stream choreography of one collective call (reference contract: csrc/deep_ep.cpp:526-578, 845-876).

    On entry the communication stream waits for ``previous_event`` (or for the caller's stream). Inside the block the
    communication stream is current. On exit either an event is returned (``async_finish``) and the inputs are kept
    safe with ``record_stream``, or the caller's stream waits for the communication stream."""

    def __init__(self, buf: Buffer, previous_event, async_finish, allocate_on_comm_stream, inputs=()):
        if allocate_on_comm_stream:
            assert previous_event is not None and async_finish, \
                "allocate_on_comm_stream requires previous_event and async_finish"
        self.buf, self.prev, self.async_finish = buf, previous_event, async_finish
        self.inputs = [t for t in inputs if isinstance(t, torch.Tensor)]
        self._outputs: List[torch.Tensor] = []
        self._early_outputs: List[torch.Tensor] = []
        self.event = EventOverlap()

    def outputs(self, *tensors):
        self._outputs.extend(t for t in tensors if isinstance(t, torch.Tensor))

    def outputs_from_caller_stream(self, *tensors):
        """Outputs that were allocated BEFORE the block, on the caller's stream. Without ``async_finish`` the caller's stream
        waits for the communication stream on exit, so such a block needs no ``record_stream`` at all: freed on the caller's
        stream it is reusable at once. (A block allocated under the communication stream and recorded on the caller's stream is
        reusable only after an event, and a host that runs ahead of the GPU then makes the caching allocator ``cudaMalloc`` a
        fresh block on every call: a combine of 4096 x 7168 was measured at 1.4 ms instead of 0.28 ms that way.)"""
        self._early_outputs.extend(t for t in tensors if isinstance(t, torch.Tensor))

    def __enter__(self):
        self.compute = torch.cuda.current_stream()
        comm = self.buf.comm_stream
        if self.prev is not None and self.prev.event is not None and self.prev.event.event is not None:
            comm.wait_event(self.prev.event.event)
        else:
            comm.wait_stream(self.compute)
        self._ctx = torch.cuda.stream(comm)
        self._ctx.__enter__()
        return self

    def __exit__(self, et, ev, tb):
        comm = self.buf.comm_stream
        self._ctx.__exit__(et, ev, tb)
        if et is not None:
            return False
        # outputs were allocated while the communication stream was current; they will be used on the caller's stream
        for t in self._outputs:
            if t.is_cuda and self.buf.runtime.symmetric_offset(t) < 0:
                t.record_stream(self.compute)
        if self.async_finish:
            for t in self.inputs + self._early_outputs:
                if t.is_cuda:
                    t.record_stream(comm)
            self.event = EventOverlap(EventHandle(comm), tuple(self.inputs))
        else:
            self.compute.wait_stream(comm)
        return False


_DEBUG_CHECKS = os.environ.get("DEEPEP_DEBUG_CHECKS", "0") == "1"


def validate_handle(handle: Tuple, rank: int, num_ranks: int) -> None:
    """Debug aid (``DEEPEP_DEBUG_CHECKS=1`` runs it before every cached dispatch and every combine; it synchronises):
    checks that a normal-mode handle is self-consistent, so that a corrupted or foreign handle is reported on the host
    instead of making a kernel write outside a peer's tensors. compute-sanitizer is not available on every
    machine; these checks cover the addresses the kernels derive from the handle."""
    rpm, cpm, rcpm, recv_src_idx, in_rank, send_head = handle
    assert rpm.shape == (num_ranks, num_ranks) and send_head.shape[1] == num_ranks and in_rank.shape == send_head.shape
    r = rpm.cpu().long()
    assert (r[1:] >= r[:-1]).all() and (r >= 0).all(), "rank_prefix_matrix must be a non-decreasing inclusive prefix"
    assert int(r[-1, rank]) == recv_src_idx.numel(), "handle does not belong to this rank (receive count mismatch)"
    sh = send_head.cpu().long()
    sent = r[rank] - (r[rank - 1] if rank > 0 else 0)
    for d in range(num_ranks):
        col = sh[:, d]
        pos = col[col >= 0]
        assert pos.numel() == int(sent[d]), f"send_head column {d} disagrees with the prefix matrix"
        if pos.numel():
            assert torch.equal(pos, torch.arange(pos.numel())), f"send_head column {d} is not a dense 0..n-1 sequence"
    assert torch.equal(in_rank.cpu(), sh >= 0), "is_token_in_rank disagrees with send_head"


def _clamp_sms(num_sms: int, num_virtual: int) -> int:
    # all CTAs of all emulated ranks must be co-resident (cooperative launch)
    return num_sms if num_virtual == 1 else max(1, min(num_sms, _NUM_SM_B200 // num_virtual - 1))


def _dispatch_many(bufs: List[Buffer], reqs: List[_DispatchReq], config: Config, previous_event, async_finish,
                   allocate_on_comm_stream):
    C = bufs[0]._C
    rts = [b.runtime for b in bufs]
    V = len(bufs)
    R = bufs[0].group_size
    for b in bufs:
        b.check_status()
    inputs = []
    for q in reqs:
        inputs += list(q.x) if isinstance(q.x, tuple) else [q.x]
        inputs += [q.topk_idx, q.topk_weights, q.is_token_in_rank, q.num_tokens_per_rank, q.num_tokens_per_expert]
    num_sms = _clamp_sms(config.num_sms if config.num_sms > 0 else Buffer.num_sms, V)
    num_channels = max(1, min(config.num_sms // 2 if config.num_sms >= 2 else 1, 128))
    cached = reqs[0].handle is not None
    worst = reqs[0].num_worst_tokens
    results = []
    with _CommScope(bufs[0], previous_event, async_finish, allocate_on_comm_stream, inputs) as scope, nvtx_range("ep.dispatch"):
        if cached:
            metas = []
            for q in reqs:
                assert q.topk_idx is None and q.topk_weights is None, "cached dispatch carries no top-k data"
                rpm, cpm, rcpm, recv_src_idx, itir, send_head = q.handle
                if _DEBUG_CHECKS:
                    validate_handle(q.handle, bufs[len(metas)].rank, R)
                metas.append((rpm, cpm, rcpm, send_head, itir, recv_src_idx.size(0), []))
        else:
            for q in reqs:
                assert q.num_tokens_per_rank is not None and q.is_token_in_rank is not None and q.num_tokens_per_expert is not None
            num_experts = reqs[0].num_tokens_per_expert.numel()
            outs = C.notify(rts, [q.num_tokens_per_rank for q in reqs], [q.num_tokens_per_expert for q in reqs],
                            [q.is_token_in_rank for q in reqs], num_channels, reqs[0].expert_alignment)
            metas = []
            for b, q, (rpm, cpm, rcpm, send_head) in zip(bufs, reqs, outs):
                if worst > 0:
                    n_recv, per_expert = worst, []
                else:
                    n_recv, per_expert = b.runtime.wait_recv_counts(num_experts // R)
                metas.append((rpm, cpm, rcpm, send_head, q.is_token_in_rank, n_recv, per_expert))
        num_experts = reqs[0].num_tokens_per_expert.numel() if not cached else R  # only used for local-id remap
        per_rank, outs_all = [], []
        for b, q, (rpm, cpm, rcpm, send_head, itir, n_recv, per_expert) in zip(bufs, reqs, metas):
            x, x_scales = q.x if isinstance(q.x, tuple) else (q.x, None)
            x = x.contiguous()
            if x_scales is not None:
                x_scales = x_scales.contiguous()  # the reference's tests pass column-major scales (tests/test_intranode.py:29)
            H = x.size(1)
            rt = b.runtime
            quant = q.quantize_fp8
            out_dtype = torch.float8_e4m3fn if quant else x.dtype
            recv_x = rt.alloc_symmetric([n_recv, H], out_dtype)
            recv_scales = rt.alloc_symmetric([n_recv, H // 128], torch.float32) if (quant or x_scales is not None) else None
            K = q.topk_idx.size(1) if q.topk_idx is not None else 0
            recv_topk_idx = rt.alloc_symmetric([n_recv, K], torch.int64) if q.topk_idx is not None else None
            recv_topk_w = rt.alloc_symmetric([n_recv, K], torch.float32) if q.topk_weights is not None else None
            if cached:
                recv_src_idx = rt.alloc_symmetric([n_recv], torch.int32)  # rewritten with identical content
            else:
                recv_src_idx = rt.alloc_symmetric([n_recv], torch.int32)
            per_rank.append((x, x_scales, q.topk_idx, q.topk_weights, send_head, rpm, recv_x, recv_scales, recv_topk_idx,
                             recv_topk_w, recv_src_idx))
            outs_all.append((recv_x, recv_scales, recv_topk_idx, recv_topk_w, recv_src_idx, rpm, cpm, rcpm, send_head, itir,
                             per_expert))
            scope.outputs(rpm, cpm, rcpm, send_head)
        C.dispatch(rts, per_rank, num_experts, reqs[0].quantize_fp8, reqs[0].round_scale, worst, num_sms)
    for q, o in zip(reqs, outs_all):
        recv_x, recv_scales, recv_topk_idx, recv_topk_w, recv_src_idx, rpm, cpm, rcpm, send_head, itir, per_expert = o
        rx = (recv_x, recv_scales) if recv_scales is not None else recv_x
        if cached:
            results.append((rx, None, None, None, None, scope.event))
        else:
            handle = (rpm, cpm, rcpm, recv_src_idx, itir, send_head)
            results.append((rx, recv_topk_idx, recv_topk_w, per_expert, handle, scope.event))
    return results


def _combine_many(bufs: List[Buffer], calls, config: Config, previous_event, async_finish, allocate_on_comm_stream):
    C = bufs[0]._C
    rts = [b.runtime for b in bufs]
    V = len(bufs)
    for b in bufs:
        b.check_status()
    num_sms = _clamp_sms(config.num_sms if config.num_sms > 0 else Buffer.num_sms, V)
    inputs = []
    for x, handle, w, bias in calls:
        inputs += [x, w] + list(Buffer._unpack_bias(bias))
    results, per_rank, keep = [], [], []
    # results are allocated here, on the caller's stream (see _CommScope.outputs_from_caller_stream)
    early = []
    if not allocate_on_comm_stream:
        for x, handle, w, bias in calls:
            T = handle[5].size(0)
            early.append((torch.empty((T, x.size(1)), dtype=torch.bfloat16, device=x.device),
                          torch.empty((T, w.size(1)), dtype=torch.float32, device=x.device) if w is not None else None))
    with _CommScope(bufs[0], previous_event, async_finish, allocate_on_comm_stream, inputs) as scope, nvtx_range("ep.combine"):
        for ci, (b, (x, handle, w, bias)) in enumerate(zip(bufs, calls)):
            rpm, _, _, src_idx, _, send_head = handle
            if _DEBUG_CHECKS:
                validate_handle(handle, b.rank, b.group_size)
            rt = b.runtime
            assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.size(0) == src_idx.size(0)
            if rt.symmetric_offset(x) < 0:
                xs = rt.alloc_symmetric(list(x.shape), x.dtype)
                xs.copy_(x)
                x = xs
            if w is not None and rt.symmetric_offset(w) < 0:
                ws = rt.alloc_symmetric(list(w.shape), torch.float32)
                ws.copy_(w)
                w = ws
            keep += [x, w]
            b0, b1 = Buffer._unpack_bias(bias)
            T = send_head.size(0)
            if early:
                out, out_w = early[ci]
                scope.outputs_from_caller_stream(out, out_w)
            else:
                out = torch.empty((T, x.size(1)), dtype=torch.bfloat16, device=x.device)
                out_w = torch.empty((T, w.size(1)), dtype=torch.float32, device=x.device) if w is not None else None
                scope.outputs(out, out_w)
            per_rank.append((x, w, send_head, rpm, b0, b1, out, out_w))
            results.append([out, out_w])
        C.combine(rts, per_rank, num_sms)
    del keep
    return [(o, ow, scope.event) for o, ow in results]


def _parity_of(views, src_info: torch.Tensor) -> int:
    return 0 if src_info.data_ptr() == views[0]["src_info"].data_ptr() else 1


def _ll_stream_enter(buf: Buffer, async_finish: bool):
    """Low-latency kernels run on the caller's stream unless the caller asked for an event."""
    if not async_finish:
        return None, None
    compute = torch.cuda.current_stream()
    buf.comm_stream.wait_stream(compute)
    ctx = torch.cuda.stream(buf.comm_stream)
    ctx.__enter__()
    return ctx, compute


def _ll_stream_exit(buf: Buffer, ctx, tensors) -> EventOverlap:
    if ctx is None:
        return EventOverlap()
    ctx.__exit__(None, None, None)
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.is_cuda and buf.runtime.symmetric_offset(t) < 0:
            t.record_stream(buf.comm_stream)
    return EventOverlap(EventHandle(buf.comm_stream))


def _ll_num_sms(num_tokens: int, num_virtual: int) -> int:
    cap = _NUM_SM_B200 if num_virtual == 1 else _NUM_SM_B200 // num_virtual
    if Buffer.ll_num_sms is not None:
        cap = min(cap, Buffer.ll_num_sms)
    return max(2, min(num_tokens + 1, cap))


def _ll_dispatch_many(bufs: List[Buffer], calls, num_max_tokens: int, num_experts: int, use_fp8: bool, round_scale: bool,
                      use_ue8m0: bool, async_finish: bool, return_recv_hook: bool):
    C = bufs[0]._C
    rts = [b.runtime for b in bufs]
    V = len(bufs)
    parity = bufs[0]._ll_parity
    for b in bufs:
        b._ll_parity ^= 1
    per_rank, results = [], []
    hidden = calls[0][0].size(1)
    for b, (x, topk_idx, cum, wait) in zip(bufs, calls):
        v = b._ll_views(num_max_tokens, hidden, num_experts)[parity]
        per_rank.append((x, topk_idx, v["count"], v["layout_range"], cum, wait, v["send_row"]))
        if use_fp8:
            rx = (v["x_fp8"], v["scales_ue8m0"] if use_ue8m0 else v["scales"])
        else:
            rx = v["x_bf16"]
        results.append((rx, v["count"], (v["src_info"], v["layout_range"], num_max_tokens, hidden, num_experts)))
    num_sms = _ll_num_sms(max(c[0].size(0) for c in calls), V)

    def launch(phases: int):
        C.ll_dispatch(rts, per_rank, num_max_tokens, num_experts, use_fp8, round_scale, use_ue8m0, parity, phases, num_sms)

    ctx, _ = _ll_stream_enter(bufs[0], async_finish)
    with nvtx_range("ep.ll_dispatch"):
        launch(1 if return_recv_hook else 3)
    event = _ll_stream_exit(bufs[0], ctx, [c[0] for c in calls] + [c[1] for c in calls])
    hook = (lambda: launch(2)) if return_recv_hook else None
    return [(rx, cnt, handle, event, hook) for rx, cnt, handle in results]


def _ll_combine_many(bufs: List[Buffer], calls, zero_copy: bool, async_finish: bool, return_recv_hook: bool):
    C = bufs[0]._C
    rts = [b.runtime for b in bufs]
    V = len(bufs)
    per_rank, outs = [], []
    parity = None
    pull, close_barrier = True, False
    for b, (x, topk_idx, topk_w, handle, out, wait) in zip(bufs, calls):
        src_info, layout_range, num_max_tokens, hidden, num_experts = handle
        views = b._ll_views(num_max_tokens, hidden, num_experts)
        parity = _parity_of(views, src_info)
        if zero_copy:
            x = views[parity]["combine_src"]
        # Expert outputs that already sit in symmetric memory (the zero-copy buffer, or a tensor from empty_symmetric)
        # are read in place by the home ranks; anything else is pushed through the stage. Every rank of the group must
        # pass the same kind of tensor: the two forms are different protocols.
        off = b.runtime.symmetric_offset(x)
        if off < 0:
            pull = False
        elif x.data_ptr() != views[parity]["combine_src"].data_ptr():
            close_barrier = True  # a caller-owned tensor: its owner may rewrite it as soon as the call returns
        if out is None:
            out = torch.empty((topk_idx.size(0), hidden), dtype=torch.bfloat16, device=topk_idx.device)
        per_rank.append((x, topk_idx, topk_w, src_info, layout_range, out, wait, views[parity]["send_row"]))
        outs.append(out)
    _, _, num_max_tokens, hidden, num_experts = calls[0][3]
    num_sms = _ll_num_sms(_NUM_SM_B200, V)

    def launch(phases: int):
        C.ll_combine(rts, per_rank, num_max_tokens, num_experts, parity, phases, num_sms, pull, close_barrier)

    ctx, _ = _ll_stream_enter(bufs[0], async_finish)
    with nvtx_range("ep.ll_combine"):
        launch(1 if return_recv_hook else 3)
    event = _ll_stream_exit(bufs[0], ctx, [c[0] for c in calls] + [o for o in outs if o.is_cuda])
    hook = (lambda: launch(2)) if return_recv_hook else None
    return [(o, event, hook) for o in outs]

"""Expert-parallel dispatch / combine: host logic around the pack, permute and reduce kernels.

Experts are sharded in contiguous blocks (expert e lives on rank e // (E / R)); tokens stay data-parallel.
One exchange each way: dispatch sends int8 rows plus fp32 scales to the experts' owners, combine sends the
bf16 expert outputs back (reference converters moe_distribute_dispatch.py:4-45 and
moe_distribute_combine.py:4-60 under python/torchair/_ge_concrete_graph/ge_converter/custom).  The
collectives are torch.distributed all_to_all_single calls (NCCL over NVLink on GPUs); with one rank there is
no collective at all.

The device work is reached through a small "kernels" provider so that the same host logic can be driven by
CPU stand-ins in multi-process gloo tests; the shipped provider is CudaKernels and nothing else is ever
selected implicitly.

`group_ep` is a string in the reference (an HCCL communicator name from get_hccl_comm_name,
python/torchair/_ge_concrete_graph/hcom_utils.py:13-15).  Here it names a process group registered with
register_ep_group().
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .watchdog import EpGroupFailed, EpWatchdog, backend_abort

_ST_INV = {torch.int8: 1, torch.int32: 3, torch.float16: 5, torch.float32: 6, torch.bfloat16: 15}

_groups: Dict[str, object] = {}
# host-side split sizes remembered between a dispatch and its combine, keyed by the handshake tensors
_splits: Dict[Tuple[int, int], Tuple[List[int], List[int]]] = {}
_SPLITS_MAX = 64

counters = {"dispatch_calls": 0, "combine_calls": 0, "wire_bytes_sent": 0}


_transport: Dict[str, str] = {}
_peer: Dict[tuple, "PeerExchange"] = {}
_last_dispatch: Dict[tuple, "PeerExchange"] = {}
_watchdogs: Dict[str, "EpWatchdog"] = {}


def register_ep_group(name: str, process_group, transport: str = "auto", watchdog=None) -> None:
    """Associates a group_ep name with a torch.distributed process group.

    transport: "peer" = rows are stored straight into the owner's receive buffer over NVLink peer memory by this
    library's kernels (one node, CUDA-graph capturable, no host read); "nccl" = all_to_all_single with exact split
    sizes (one host read per dispatch; also the path used for CPU tensors in tests); "auto" = peer for CUDA tensors
    when symmetric memory can be set up, else nccl.  Every rank of the group must pass the same value.

    watchdog: None (off), True, or a dict with any of interval_s, timeout_s, store, device: starts a host thread that
    exchanges heartbeats with the other ranks through the rendezvous store and follows the events of the exchanges
    (torchair_b200/watchdog.py).  With it a dispatch / combine raises EpGroupFailed before launching anything once a
    rank has been silent for timeout_s, and an 'nccl' exchange that does not finish within timeout_s gets its
    communicator aborted.
    """
    if not isinstance(name, str) or not name:
        raise ValueError("group name must be a non-empty string")
    if transport not in ("auto", "peer", "nccl"):
        raise ValueError("transport must be 'auto', 'peer' or 'nccl'")
    _groups[name] = process_group
    _transport[name] = transport
    old = _watchdogs.pop(name, None)
    if old is not None:
        old.stop()
    if watchdog:
        opts = dict(watchdog) if isinstance(watchdog, dict) else {}
        store = opts.pop("store", None) or dist.distributed_c10d._get_default_store()
        device = opts.pop("device", None)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        _watchdogs[name] = EpWatchdog(name, store, dist.get_rank(process_group), dist.get_world_size(process_group),
                                      abort=backend_abort(process_group, device), **opts).start()


def watchdog_of(name: str):
    """The running watchdog of a registered group, or None."""
    return _watchdogs.get(name)


def _watch(group_ep, tensor, what):
    """Hands the watchdog an event recorded after the collectives that were just enqueued (eager CUDA work only)."""
    wd = _watchdogs.get(group_ep)
    if wd is None or not tensor.is_cuda or torch.cuda.is_current_stream_capturing():
        return
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(tensor.device))
    wd.watch(ev, what)


def transport_of(name: str, is_cuda: bool) -> str:
    t = _transport.get(name, "auto")
    if t == "auto":
        t = "peer" if is_cuda and os.environ.get("TORCHAIR_B200_EP_TRANSPORT", "peer") == "peer" else "nccl"
    if t == "peer" and not is_cuda:
        raise RuntimeError("the peer-memory transport needs CUDA tensors")
    return t


def get_ep_group(name: str):
    if name in _groups:
        return _groups[name]
    raise RuntimeError(f"expert-parallel group {name!r} is not registered; call "
                       "torchair_b200.register_ep_group(name, process_group) first")


def slot_tokens(T: int, R: int, global_bs: int) -> int:
    """Tokens a rank may hold: T when global_bs == 0 (every rank holds the same number), else global_bs / R (decision:
    global_bs is R times the largest per-rank batch, so that ranks may hold different numbers of tokens up to that)."""
    return T if not global_bs else global_bs // R


def dispatch_rows(T: int, R: int, E: int, K: int, global_bs: int = 0) -> int:
    """Static row count of expand_x: every rank may send min(E/R, K) copies of each of its (at most) slot_tokens tokens."""
    return slot_tokens(T, R, global_bs) * R * min(E // R, K)


def check_dispatch_args(x, expert_ids, R, rank, E, scales, x_active_mask, tp_world_size, expert_shard_type,
                        shared_expert_rank_num, quant_mode, global_bs, nums_type):
    op = "npu_moe_distribute_dispatch"
    if x.dim() != 2 or expert_ids.dim() != 2 or x.shape[0] != expert_ids.shape[0]:
        raise RuntimeError(f"{op}: x must be [T, H] and expert_ids [T, K]")
    if R < 1 or E < 1 or E % R != 0 or not (0 <= rank < R):
        raise RuntimeError(f"{op}: ep_world_size={R}, ep_rank_id={rank}, moe_expert_num={E} are inconsistent")
    if scales is not None:
        if quant_mode != 2:
            raise RuntimeError(f"{op}: `scales` (smooth scales) need quant_mode 2")
        if scales.dtype != torch.float32 or scales.dim() != 2 or scales.shape[1] != x.shape[1] or scales.shape[0] not in (1, E):
            raise RuntimeError(f"{op}: scales must be float32 [{E}, {x.shape[1]}] (one row per expert) or [1, {x.shape[1]}]")
    if x_active_mask is not None and (x_active_mask.dtype != torch.bool or x_active_mask.shape != (x.shape[0],)):
        raise RuntimeError(f"{op}: x_active_mask must be bool [T]")
    if global_bs < 0 or (global_bs and (global_bs % R != 0 or global_bs // R < x.shape[0])):
        raise RuntimeError(f"{op}: global_bs={global_bs} must be a multiple of ep_world_size and at least ep_world_size * T")
    if tp_world_size not in (0, 1):
        raise NotImplementedError(f"{op}: tensor parallelism inside an expert (tp_world_size={tp_world_size}) is not sharded here")
    if expert_shard_type != 0 or shared_expert_rank_num != 0:
        raise NotImplementedError(f"{op}: shared-expert ranks / expert_shard_type != 0 are not sharded here")
    if quant_mode not in (0, 2):
        raise NotImplementedError(f"{op}: quant_mode must be 0 (none) or 2 (per-token dynamic int8)")
    if nums_type not in (0, 1):
        raise RuntimeError(f"{op}: expert_token_nums_type must be 0 (cumsum) or 1 (counts)")


def check_combine_args(expand_x, expert_ids, expert_scales, R, rank, E, x_active_mask, activation_scale, weight_scale,
                       group_list, tp_world_size, expert_shard_type, shared_expert_rank_num, global_bs, out_dtype,
                       comm_quant_mode):
    op = "npu_moe_distribute_combine"
    if expand_x.dim() != 2 or expert_ids.dim() != 2 or expert_scales.shape != expert_ids.shape:
        raise RuntimeError(f"{op}: expand_x must be [A, H]; expert_ids and expert_scales [T, K]")
    if R < 1 or E < 1 or E % R != 0 or not (0 <= rank < R):
        raise RuntimeError(f"{op}: ep_world_size={R}, ep_rank_id={rank}, moe_expert_num={E} are inconsistent")
    if activation_scale is not None or weight_scale is not None or group_list is not None:
        raise NotImplementedError(f"{op}: the dequant-in-combine arguments (int32 expand_x) are outside the W8A8 MoE path")
    if x_active_mask is not None and (x_active_mask.dtype != torch.bool or x_active_mask.shape != (expert_ids.shape[0],)):
        raise RuntimeError(f"{op}: x_active_mask must be bool [T]")
    if tp_world_size not in (0, 1) or expert_shard_type != 0 or shared_expert_rank_num != 0:
        raise NotImplementedError(f"{op}: tensor-parallel / shared-expert-rank sharding is not supported")
    if global_bs < 0 or (global_bs and (global_bs % R != 0 or global_bs // R < expert_ids.shape[0])):
        raise RuntimeError(f"{op}: global_bs={global_bs} must be a multiple of ep_world_size and at least ep_world_size * T")
    if comm_quant_mode != 0 or out_dtype != 0:
        raise NotImplementedError(f"{op}: comm_quant_mode and out_dtype must be 0")


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class CudaKernels:
    """The shipped provider: every step is one or more sm_100a kernels behind the C ABI."""

    @staticmethod
    def dispatch_pack(x, expert_ids, E, quant_mode, nums_type=None, mask=None, scales=None, special=0):
        """Sort + quantise + scatter of this rank's copies.  mask: bool [T] (False = the token sends nothing); scales: fp32
        smooth scales [E, H] or [1, H]; special > 0: expert ids >= E are special experts that are not sent."""
        if not x.is_cuda:
            raise RuntimeError("torchair_b200 kernels need CUDA tensors; there is no CPU implementation")
        if expert_ids.dtype != torch.int32:
            raise RuntimeError("npu_moe_distribute_dispatch: expert_ids must be int32")
        if x.dtype not in (torch.bfloat16, torch.float16):
            raise NotImplementedError("npu_moe_distribute_dispatch: x must be bfloat16 or float16")
        x, expert_ids = x.contiguous(), expert_ids.contiguous()
        T, K = expert_ids.shape
        H = x.shape[1]
        dev = x.device
        rows = torch.empty((T * K, H), dtype=torch.int8 if quant_mode == 2 else x.dtype, device=dev)
        out_scales = torch.empty((T * K,), dtype=torch.float32, device=dev)
        expand_idx = torch.empty((T * K,), dtype=torch.int32, device=dev)
        counts = torch.empty((E,), dtype=torch.int32, device=dev)
        nums = None if nums_type is None else torch.empty((E,), dtype=torch.int64, device=dev)   # counts / running total
        nbytes = _lib.workspace_bytes("tab_moe_dispatch_pack_workspace_bytes", T, K, E)
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        mask = None if mask is None else mask.contiguous()
        scales = None if scales is None else scales.contiguous()
        _lib.call("tab_moe_dispatch_pack_ex", _ptr(x), _ST_INV[x.dtype], _ptr(expert_ids), T, K, H, 0, E, int(special > 0), _ptr(mask),
                  _ptr(scales), 0 if scales is None else scales.shape[0], None, 0, quant_mode, _ptr(rows), _ptr(out_scales),
                  _ptr(expand_idx), _ptr(counts), _ptr(nums), int(nums_type or 0), _ptr(ws), ws.numel(), _stream(x))
        return rows, out_scales, expand_idx, counts, nums

    @staticmethod
    def exchange_plan(recv_counts, R, E_l, slot_rows, nums_type):
        dev = recv_counts.device
        plan = torch.empty((2 * R * E_l + 1,), dtype=torch.int32, device=dev)
        nums = torch.empty((E_l,), dtype=torch.int64, device=dev)
        ep_recv = torch.empty((E_l * R,), dtype=torch.int32, device=dev)
        _lib.call("tab_moe_exchange_plan", _ptr(recv_counts.contiguous()), R, E_l, slot_rows, nums_type, _ptr(plan), _ptr(nums),
                  _ptr(ep_recv), _stream(recv_counts))
        return plan, nums, ep_recv

    @staticmethod
    def exchange_rows(src, src_scales, plan, R, E_l, slot_rows, direction, dst_rows, zero_fill):
        dst = torch.empty((dst_rows, src.shape[1]), dtype=src.dtype, device=src.device)
        dst_scales = None if src_scales is None else torch.empty((dst_rows,), dtype=torch.float32, device=src.device)
        if src.shape[0] == 0:  # nothing arrived: no row of dst is defined, and the kernel would have no source to read
            return dst, dst_scales
        _lib.call("tab_moe_exchange_rows", _ptr(src), _ptr(src_scales), _ptr(plan), R, E_l, slot_rows, direction,
                  src.shape[1] * src.element_size(), dst_rows, int(zero_fill), _ptr(dst), _ptr(dst_scales), _stream(src))
        return dst, dst_scales

    @staticmethod
    def combine(rows, expand_idx, expert_scales, shared, T, K, mask=None, special=None, ack=None):
        """special: None, or a dict with expert_ids [T, K], E, zero, copy, const, ori_x, alpha_1, alpha_2, const_v."""
        if rows.dtype not in (torch.bfloat16, torch.float16):
            raise NotImplementedError("npu_moe_distribute_combine: expand_x must be bfloat16 or float16")
        rows = rows.contiguous()
        out = torch.empty((T, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        if expand_idx.dtype != torch.int32 or expert_scales.dtype != torch.float32:
            raise RuntimeError("npu_moe_distribute_combine: expand_idx must be int32 and expert_scales float32")
        if shared is not None:
            if shared.dtype != rows.dtype or shared.shape != out.shape:
                raise RuntimeError("npu_moe_distribute_combine: shared_expert_x must match the output")
            shared = shared.contiguous()
        if mask is None and special is None and ack is None:
            _lib.call("tab_moe_combine", _ptr(rows), _ST_INV[rows.dtype], _ptr(expand_idx.contiguous()),
                      _ptr(expert_scales.contiguous()), _ptr(shared), T, K, rows.shape[1], _ptr(out), _stream(rows))
            return out
        sp = special or {}
        c = lambda t: None if t is None else t.to(rows.dtype).contiguous()
        ids = sp.get("expert_ids")
        args = (_ptr(rows), _ST_INV[rows.dtype], _ptr(expand_idx.contiguous()), _ptr(expert_scales.contiguous()),
                _ptr(shared), T, K, rows.shape[1], _ptr(out), _ptr(None if mask is None else mask.contiguous()),
                _ptr(None if ids is None else ids.contiguous()), int(sp.get("E", 0)), int(sp.get("zero", 0)), int(sp.get("copy", 0)),
                int(sp.get("const", 0)), _ptr(c(sp.get("ori_x"))), _ptr(c(sp.get("alpha_1"))), _ptr(c(sp.get("alpha_2"))),
                _ptr(c(sp.get("const_v"))))
        if ack is None:
            _lib.call("tab_moe_combine_ex", *args, _stream(rows))
        else:   # (device table of the peers' flag slots, signal counter, arrival counter, ranks): the last CTA acknowledges
            _lib.call("tab_moe_combine_ack", *args, _ptr(ack[0]), ctypes.c_void_p(ack[1]), ctypes.c_void_p(ack[2]), int(ack[3]),
                      _stream(rows))
        return out


class PeerExchange:
    """Peer-mapped buffers, flags and counters of one exchange configuration (see csrc/ep_peer.cu for the layout).

    Built collectively (every rank of the group at the same call) on first use of a (group, T, K, H, E) combination.
    """

    KIND_DATA_D, KIND_ACK_D, KIND_DATA_C, KIND_ACK_C = 0, 1, 2, 3

    def __init__(self, pg, R, rank, T, K, H, E, disp_row_bytes, device):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
        import torch.distributed._symmetric_memory as symm
        self.R, self.rank, self.E_l = R, rank, E // R
        self.C = T * min(self.E_l, K)
        self.H = H
        self.disp_row_bytes = disp_row_bytes
        self.ret_row_bytes = H * 2
        al = lambda n: (n + 255) // 256 * 256
        self.off_recv = 0
        self.off_counts = al(R * self.C * (disp_row_bytes + 16))
        self.off_ret = self.off_counts + al(R * self.E_l * 4)
        self.off_ctrl = self.off_ret + al(R * self.C * self.ret_row_bytes)
        ctrl_bytes = al(4 * R * 8) + 256
        total = self.off_ctrl + ctrl_bytes
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.hdl = symm.rendezvous(self.buf, pg)
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        dev_ptrs = lambda offs: torch.tensor(offs, dtype=torch.int64, device=device)
        self.peer_recv = dev_ptrs([p + self.off_recv for p in ptrs])
        self.peer_counts = dev_ptrs([p + self.off_counts for p in ptrs])
        self.peer_ret = dev_ptrs([p + self.off_ret for p in ptrs])
        # flag array k of a rank lives at off_ctrl + k*R*8; this rank's slot in it is entry `rank`
        self.peer_flags = [dev_ptrs([p + self.off_ctrl + k * R * 8 + rank * 8 for p in ptrs]) for k in range(4)]
        base = self.buf.data_ptr()
        self.flags_local = [base + self.off_ctrl + k * R * 8 for k in range(4)]
        cbase = base + self.off_ctrl + al(4 * R * 8)
        self.sig_counter = [cbase + k * 8 for k in range(4)]
        self.wait_counter = [cbase + 32 + k * 8 for k in range(4)]
        self.status_ptr = cbase + 64
        self.done_ptr = cbase + 72          # arrival counter of the unpack kernel's CTAs (wraps to zero by itself)
        self.recv_local = self.buf[self.off_recv:self.off_counts]
        self.counts_local = self.buf[self.off_counts:self.off_counts + R * self.E_l * 4].view(torch.int32)
        self.ret_local = self.buf[self.off_ret:self.off_ret + R * self.C * self.ret_row_bytes]
        dist.barrier(pg)     # nobody signals into a buffer that is not zeroed and mapped yet

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.buf.device).cuda_stream)

    def enter(self):
        """Buffers and flag counters of one exchange are used in call order, which only one stream at a time can give.
        Outside CUDA-graph capture this is checked: a call from another stream while the previous call's work is still
        pending raises (use a second group name for the second stream).  Inside a capture the graph's own edges order
        the work, and nothing is checked."""
        dev = self.buf.device
        if torch.cuda.is_current_stream_capturing():
            return
        sid = torch.cuda.current_stream(dev).cuda_stream
        last = getattr(self, "_last", None)
        if last is not None and last[0] != sid and not last[1].query():
            raise RuntimeError("expert-parallel exchange over peer memory: this (group, shape) is still busy on another stream; "
                               "exchanges that overlap on two streams need two group names (register_ep_group twice)")

    def leave(self):
        if torch.cuda.is_current_stream_capturing():
            return
        st = torch.cuda.current_stream(self.buf.device)
        ev = torch.cuda.Event()
        ev.record(st)
        self._last = (st.cuda_stream, ev)

    def signal(self, kind):
        _lib.call("tab_ep_signal", _ptr(self.peer_flags[kind]), ctypes.c_void_p(self.sig_counter[kind]), self.R, self._stream())

    def wait(self, kind, pre_increment):
        _lib.call("tab_ep_wait", ctypes.c_void_p(self.flags_local[kind]), ctypes.c_void_p(self.wait_counter[kind]), self.R,
                  int(pre_increment), ctypes.c_void_p(self.status_ptr), 100 + kind, self._stream())

    def signal_wait(self, kind, bump_kind=None):
        """signal(kind) followed by wait(kind, pre_increment=1) as one launch; bump_kind: an acknowledgement counter that the
        preceding data kernel only read and that advances here."""
        bump = None if bump_kind is None else ctypes.c_void_p(self.wait_counter[bump_kind])
        _lib.call("tab_ep_signal_wait", _ptr(self.peer_flags[kind]), ctypes.c_void_p(self.sig_counter[kind]),
                  ctypes.c_void_p(self.flags_local[kind]), ctypes.c_void_p(self.wait_counter[kind]), self.R,
                  ctypes.c_void_p(self.status_ptr), 100 + kind, bump, self._stream())

    def combine_and_acknowledge(self, kern, back, expand_idx, expert_scales, shared, T, K, mask, special):
        """The weighted sum over the returned rows; its last CTA tells the peers that this rank's return buffer is free
        again (a separate one-CTA launch when the kernels provider has no such form or the rank holds no token)."""
        if T > 0 and kern is CudaKernels:
            ack = (self.peer_flags[self.KIND_ACK_C], self.sig_counter[self.KIND_ACK_C], self.done_ptr, self.R)
            return kern.combine(back, expand_idx, expert_scales, shared, T, K, mask, special, ack)
        out = kern.combine(back, expand_idx, expert_scales, shared, T, K, mask, special)
        self.signal(self.KIND_ACK_C)
        return out

    def status(self) -> int:
        """Synchronises and returns 0, 100 + kind of the first flag wait that ran out of time, or 110 when a sender held
        more rows for one destination than its slot takes (those rows were not sent)."""
        torch.cuda.synchronize(self.buf.device)
        off = self.status_ptr - self.buf.data_ptr()
        return int(self.buf[off:off + 4].view(torch.int32).item())


def peer_exchange(group_ep, pg, R, rank, T, K, H, E, disp_row_bytes, device) -> PeerExchange:
    key = (group_ep, R, rank, T, K, H, E, disp_row_bytes, device.index)
    px = _peer.get(key)
    if px is None:
        px = PeerExchange(pg, R, rank, T, K, H, E, disp_row_bytes, device)
        _peer[key] = px
    return px


def peer_status() -> int:
    """0 if no peer-memory wait ever timed out on this rank (synchronises the device)."""
    for px in _peer.values():
        st = px.status()
        if st:
            return st
    return 0


def _dispatch_peer(kern, x, expert_ids, group_ep, pg, R, rank, E, quant_mode, nums_type, send, tp_recv, expand_scales, t_slot):
    send_rows, send_scales, expand_idx, counts = send[:4]
    T, K = expert_ids.shape
    H = x.shape[1]
    E_l = E // R
    dev = x.device
    row_bytes = H * send_rows.element_size()
    px = peer_exchange(group_ep, pg, R, rank, t_slot, K, H, E, row_bytes, dev)
    _last_dispatch[(group_ep, R, rank, T, K, H, E, dev.index)] = px     # the matching combine returns through the same buffers
    px.enter()
    A = R * px.C
    st = px._stream()
    slot_idx = torch.empty_like(expand_idx)
    # four launches: send (checks the peers' acknowledgement of the previous exchange itself), hand-over (signal + wait),
    # unpack (derives the row offsets from the delivered counts itself; its last CTA acknowledges)
    _lib.call("tab_ep_send_rows", _ptr(send_rows), _ptr(send_scales), _ptr(counts), _ptr(expand_idx), R, E_l, px.C, row_bytes,
              T * K, rank, _ptr(px.peer_recv), _ptr(px.peer_counts), _ptr(slot_idx), ctypes.c_void_p(px.status_ptr), 110,
              ctypes.c_void_p(px.flags_local[px.KIND_ACK_D]), ctypes.c_void_p(px.wait_counter[px.KIND_ACK_D]), 100 + px.KIND_ACK_D, st)
    px.signal_wait(px.KIND_DATA_D, bump_kind=px.KIND_ACK_D)    # every source's rows and counts have landed here
    expand_x = torch.empty((A, H), dtype=send_rows.dtype, device=dev)
    dyn = torch.empty((A,), dtype=torch.float32, device=dev)
    nums = torch.empty((E_l,), dtype=torch.int64, device=dev)
    ep_recv = torch.empty((E_l * R,), dtype=torch.int32, device=dev)
    _lib.call("tab_ep_unpack_rows_fused", _ptr(px.recv_local), _ptr(px.counts_local), R, E_l, px.C, row_bytes, A, nums_type,
              _ptr(expand_x), _ptr(dyn), _ptr(nums), _ptr(ep_recv), _ptr(px.peer_flags[px.KIND_ACK_D]),
              ctypes.c_void_p(px.sig_counter[px.KIND_ACK_D]), ctypes.c_void_p(px.done_ptr), st)
    counters["wire_bytes_sent"] += T * K * (row_bytes + 16)
    px.leave()
    return expand_x, dyn, slot_idx, nums, ep_recv, tp_recv, expand_scales


def _combine_peer(kern, expand_x, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep, pg, R, rank, E, shared,
                  mask=None, special=None):
    T, K = expert_ids.shape
    H = expand_x.shape[1]
    E_l = E // R
    if expand_x.element_size() != 2:
        raise NotImplementedError("npu_moe_distribute_combine over peer memory: expand_x must be bfloat16 or float16")
    px = _last_dispatch.get((group_ep, R, rank, T, K, H, E, expand_x.device.index))
    if px is None:
        raise RuntimeError("npu_moe_distribute_combine: no matching npu_moe_distribute_dispatch ran on this group")
    px.enter()
    st = px._stream()
    y = expand_x.contiguous()
    recv_counts = ep_send_counts.view(E_l, R).t().contiguous()
    plan, _, _ = kern.exchange_plan(recv_counts, R, E_l, px.C, 1)
    px.wait(px.KIND_ACK_C, 0)                     # the sources have reduced the rows of the previous combine
    _lib.call("tab_ep_return_rows", _ptr(y), _ptr(plan), R, E_l, px.C, H * 2, y.shape[0], rank, _ptr(px.peer_ret), st)
    px.signal(px.KIND_DATA_C)
    px.wait(px.KIND_DATA_C, 1)
    back = px.ret_local.view(expand_x.dtype).view(R * px.C, H)
    out = px.combine_and_acknowledge(kern, back, expand_idx, expert_scales, shared, T, K, mask, special)
    counters["wire_bytes_sent"] += T * K * H * 2
    px.leave()
    return out


def combine_from_producer(kern, produce_rows, rows, H, dtype, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep,
                          R, rank, E, shared=None, mask=None, special=None):
    """Combine whose expert-output rows are stored into the source ranks' return buffers by their producer.

    Peer transport only.  ``produce_rows(row_dst)`` must enqueue, on the current stream, work that stores output row i
    (``H`` elements of ``dtype``, i < rows) at the address ``row_dst[i]`` (an int64 device tensor; 0 = row not in any
    group); with the grouped GEMM's scatter epilogue the rows cross NVLink tile by tile while the GEMM runs, and
    neither a local [rows, H] tensor nor a copy kernel exists.  Everything else is _combine_peer.
    """
    counters["combine_calls"] += 1
    T, K = expert_ids.shape
    E_l = E // R
    if dtype not in (torch.bfloat16, torch.float16):
        raise NotImplementedError("npu_moe_distribute_combine over peer memory: rows must be bfloat16 or float16")
    px = _last_dispatch.get((group_ep, R, rank, T, K, H, E, expand_idx.device.index))
    if px is None:
        raise RuntimeError("npu_moe_distribute_combine: no matching npu_moe_distribute_dispatch ran on this group")
    wd = _watchdogs.get(group_ep)
    if wd is not None:
        wd.check()
    px.enter()
    st = px._stream()
    row_dst = torch.empty((rows,), dtype=torch.int64, device=expand_idx.device)
    # address table from ep_send_counts in one launch; its first CTA also waits until the sources have reduced the rows of
    # the previous combine
    _lib.call("tab_ep_return_plan_fused", _ptr(ep_send_counts.contiguous()), R, E_l, px.C, H * 2, rows, rank, _ptr(px.peer_ret),
              _ptr(row_dst), ctypes.c_void_p(px.flags_local[px.KIND_ACK_C]), ctypes.c_void_p(px.wait_counter[px.KIND_ACK_C]),
              ctypes.c_void_p(px.status_ptr), 100 + px.KIND_ACK_C, st)
    produce_rows(row_dst)
    px.signal_wait(px.KIND_DATA_C)
    back = px.ret_local.view(dtype).view(R * px.C, H)
    out = px.combine_and_acknowledge(kern, back, expand_idx, expert_scales, shared, T, K, mask, special)
    counters["wire_bytes_sent"] += T * K * H * 2
    px.leave()
    return out


def _remember(key, value):
    if len(_splits) >= _SPLITS_MAX:
        _splits.pop(next(iter(_splits)))
    _splits[key] = value


_zero_cache: Dict[tuple, torch.Tensor] = {}


def _zeros(shape, dtype, device) -> torch.Tensor:
    """The all-zero handshake outputs (tp_recv_count, expand_scales).  Nothing in this library writes them, so on a GPU
    one tensor per shape is filled once and handed out again: no fill launch per call.  Callers must not write into them."""
    if device.type != "cuda":
        return torch.zeros(shape, dtype=dtype, device=device)
    key = (tuple(shape), dtype, device.index)
    t = _zero_cache.get(key)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            return torch.zeros(shape, dtype=dtype, device=device)    # a capture's pool must not own the shared tensor
        t = _zero_cache[key] = torch.zeros(shape, dtype=dtype, device=device)
    return t


def dispatch(kern, x, expert_ids, group_ep, R, rank, E, quant_mode, nums_type, tp_slots=1, mask=None, scales=None, special=0,
             global_bs=0):
    """Returns the seven outputs of npu_moe_distribute_dispatch.

    Rows of expand_x / dynamic_scales past the received total (sum of expert_token_nums) are not written: expand_x is
    sized for the worst case, and nothing downstream reads that tail.
    Handshake tensors (consumed only by combine): expand_idx[t*K+k] = position of that copy in this rank's
    send order (sorted by global expert id, stable), -1 for a copy that is not sent; ep_recv_count[e*R+s] = rows received
    for local expert e from rank s; tp_recv_count and expand_scales are zero.
    mask (x_active_mask): tokens marked False send nothing; scales: smooth scales before the quantisation of each copy;
    special > 0: ids >= E are special experts of the second-generation operator, evaluated by the combine, not sent;
    global_bs: R times the largest per-rank batch when the ranks hold different numbers of tokens.
    """
    counters["dispatch_calls"] += 1
    T, K = expert_ids.shape
    H = x.shape[1]
    E_l = E // R
    t_slot = slot_tokens(T, R, global_bs)
    A = dispatch_rows(T, R, E, K, global_bs)
    dev = x.device
    send_rows, send_scales, expand_idx, counts, nums = kern.dispatch_pack(x, expert_ids, E, quant_mode, nums_type if R == 1 else None,
                                                                          mask, scales, special)
    tp_recv = _zeros((tp_slots,), torch.int32, dev)
    expand_scales = _zeros((A,), torch.float32, dev)
    if R == 1:
        if A != T * K:  # K > E or a larger slot: the static shape is padded
            pad_rows = torch.zeros((A, H), dtype=send_rows.dtype, device=dev)
            pad_rows[:T * K] = send_rows
            pad_scales = torch.zeros((A,), dtype=torch.float32, device=dev)
            pad_scales[:T * K] = send_scales
            send_rows, send_scales = pad_rows, pad_scales
        return send_rows, send_scales, expand_idx, nums, counts, tp_recv, expand_scales

    pg = get_ep_group(group_ep)
    wd = _watchdogs.get(group_ep)
    if wd is not None:
        wd.check()                      # a rank that is gone: raise before enqueueing work that would wait for it
    if dist.get_world_size(pg) != R or dist.get_rank(pg) != rank:
        raise RuntimeError(f"npu_moe_distribute_dispatch: group {group_ep!r} has size/rank "
                           f"{dist.get_world_size(pg)}/{dist.get_rank(pg)}, arguments say {R}/{rank}")
    if transport_of(group_ep, x.is_cuda) == "peer":
        return _dispatch_peer(kern, x, expert_ids, group_ep, pg, R, rank, E, quant_mode, nums_type,
                              (send_rows, send_scales, expand_idx, counts), tp_recv, expand_scales, t_slot)
    recv_counts = torch.empty_like(counts)                       # [R, E_l]: rows from rank s for my expert e
    dist.all_to_all_single(recv_counts, counts, group=pg)
    sums = torch.stack([counts.view(R, E_l).sum(1), recv_counts.view(R, E_l).sum(1)]).cpu()   # the one host read
    send_splits = [int(v) for v in sums[0]]
    recv_splits = [int(v) for v in sums[1]]
    total = sum(recv_splits)
    if total > A:
        raise RuntimeError(f"npu_moe_distribute_dispatch: received {total} rows but expand_x holds {A}; "
                           "every rank must pass the same number of tokens when global_bs == 0")
    wire_rows = torch.empty((total, H), dtype=send_rows.dtype, device=dev)
    wire_scales = torch.empty((total,), dtype=torch.float32, device=dev)
    sent = sum(send_splits)                                      # copies that were dropped have no row
    dist.all_to_all_single(wire_rows, send_rows[:sent], recv_splits, send_splits, group=pg)
    dist.all_to_all_single(wire_scales, send_scales[:sent], recv_splits, send_splits, group=pg)
    counters["wire_bytes_sent"] += (sum(send_splits) - send_splits[rank]) * (H * send_rows.element_size() + 4)
    plan, nums, ep_recv = kern.exchange_plan(recv_counts.view(R, E_l), R, E_l, 0, nums_type)
    expand_x, dyn_scales = kern.exchange_rows(wire_rows, wire_scales, plan, R, E_l, 0, 0, A, False)
    _remember((ep_recv.data_ptr(), expand_idx.data_ptr()), (send_splits, recv_splits))
    _watch(group_ep, expand_x, "the dispatch exchange")
    return expand_x, dyn_scales, expand_idx, nums, ep_recv, tp_recv, expand_scales


def combine(kern, expand_x, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep, R, rank, E, shared=None, mask=None,
            special=None):
    """out[t] = sum_k expert_scales[t,k] * (expert output of copy (t,k)), after returning rows to their senders.
    mask (x_active_mask): tokens marked False get an all-zero row; special: the special experts of the second-generation
    operator (see CudaKernels.combine)."""
    counters["combine_calls"] += 1
    T, K = expert_ids.shape
    H = expand_x.shape[1]
    if R == 1:
        return kern.combine(expand_x, expand_idx, expert_scales, shared, T, K, mask, special)
    pg = get_ep_group(group_ep)
    wd = _watchdogs.get(group_ep)
    if wd is not None:
        wd.check()
    E_l = E // R
    if transport_of(group_ep, expand_x.is_cuda) == "peer":
        return _combine_peer(kern, expand_x, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep, pg, R, rank, E, shared,
                             mask, special)
    remembered = _splits.get((ep_send_counts.data_ptr(), expand_idx.data_ptr()))
    if remembered is not None:
        send_splits, recv_splits = remembered
    else:  # handshake tensors were copied: rebuild the split sizes (one host read)
        got = ep_send_counts.view(E_l, R).sum(0)
        sent_to = (expert_ids.reshape(-1) // E_l).to(torch.int64)
        sent_ok = (expand_idx.reshape(-1) >= 0) & (sent_to < R)
        sent = torch.bincount(sent_to[sent_ok], minlength=R).to(got.dtype)
        sums = torch.stack([sent, got]).cpu()
        send_splits = [int(v) for v in sums[0]]
        recv_splits = [int(v) for v in sums[1]]
    recv_counts = ep_send_counts.view(E_l, R).t().contiguous()
    plan, _, _ = kern.exchange_plan(recv_counts, R, E_l, 0, 1)
    total = sum(recv_splits)
    wire, _ = kern.exchange_rows(expand_x.contiguous(), None, plan, R, E_l, 0, 1, total, False)
    back = torch.empty((T * K, H), dtype=expand_x.dtype, device=expand_x.device)
    dist.all_to_all_single(back[:sum(send_splits)], wire, send_splits, recv_splits, group=pg)
    counters["wire_bytes_sent"] += (total - recv_splits[rank]) * H * expand_x.element_size()
    out = kern.combine(back, expand_idx, expert_scales, shared, T, K, mask, special)
    _watch(group_ep, out, "the combine exchange")
    return out

"""Expert parallelism over 2, 4 or 8 GPUs of one box, one process per GPU.  Two forms of the exchange:
``PeerExpertParallelLayer`` stores rows straight into the peers' buffers over NVLink (CUDA IPC mappings, flags polled
on the device, no collective and no host synchronisation per layer - the one the benchmark runs);
``ExpertParallelLayer`` uses ``torch.distributed`` all-to-all calls (NCCL on GPUs, gloo in the CPU tests of the
exchange logic).  The library's kernels do everything else.

Experts are block-sharded - rank g owns experts [g*E/G, (g+1)*E/G) and only their slice of the pool - tokens stay
data-parallel, the router weights and the shared expert are replicated.  Per layer:

    norm + router (local) -> plan send order (by destination rank) -> pack rows -> all-to-all (counts, expert ids, rows)
    -> grouped expert FFN on the received rows (sorted by expert; tensor-core path for 4-bit shapes)
    -> all-to-all of the fp32 result rows back -> weighted rank-ordered reduce + shared expert + residual (one kernel)

The result is bit-identical to the single-GPU prefill layer: the same per-row arithmetic, the same summation order.
The reference (single device) has no counterpart; what is preserved is the order of prefill_moe_reduce_token_major
(Sources/Mference/Metal/Prefill/prefill.metal:631-652).

The exchange logic (`exchange_plan`, `ExpertParallelLayer.forward`) only needs an object with the five compute
methods of `DeviceOps`; the product always uses `DeviceOps` (CUDA, fails loudly without the library).
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch
import torch.distributed as dist

from . import _lib as L


def exchange_plan(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """recv_counts[g] = number of pairs rank g sends to this rank (an all-to-all of one int32 per peer)."""
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    return recv_counts


def exchange_rows(rows: torch.Tensor, send_counts: List[int], recv_counts: List[int], group=None) -> torch.Tensor:
    """All-to-all-v of rows: send_counts[g] consecutive rows go to rank g; returns the rows received, by source rank."""
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out


class DeviceOps:
    """The compute steps of an expert-parallel layer on the GPU, through the C ABI."""

    def __init__(self, d, f, num_experts, top_k, world, max_tokens, max_recv_rows, *, bits=4, shared_bits=4, x_dtype=L.DT_BF16,
                 tensor_core=True, **kw):
        from .moe import MoE
        self.lib = L.load()
        self.d, self.f, self.E, self.K, self.world, self.x_dtype = d, f, num_experts, top_k, world, x_dtype
        self.local_E = num_experts // world
        # home side: norm + router over all experts; expert side: the local experts with one "rank slot" per received row
        self.home = MoE(d, f, num_experts, top_k, bits=bits, shared_bits=shared_bits, x_dtype=x_dtype, max_tokens=max_tokens, **kw)
        self.expert = MoE(d, f, self.local_E, 1, bits=bits, shared_bits=0, x_dtype=x_dtype, max_tokens=max_recv_rows,
                          tensor_core_prefill=tensor_core, **kw)
        self.shared = MoE(d, f, 1, 1, bits=shared_bits or bits, shared_bits=0, x_dtype=x_dtype, max_tokens=max_tokens,
                          tensor_core_prefill=tensor_core and (shared_bits or bits) == 4, **kw)
        self.tdt = torch.bfloat16 if x_dtype == L.DT_BF16 else torch.float16

    @staticmethod
    def _s():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def ones_for(self, n, device):
        """fp16 ones [n, 1]: the routing weight of a received row on the expert side (cached)."""
        cur = getattr(self, "_ones", None)
        if cur is None or cur.shape[0] < n or cur.device != device:
            self._ones = torch.ones((n, 1), dtype=torch.float16, device=device)
        return self._ones[:n]

    def norm(self, weights, h):
        xn = torch.empty_like(h)
        self.home.encode_rmsnorm(h, xn, weights.norm_w)
        return xn

    def router(self, weights, xn):
        T = xn.shape[0]
        idx = torch.empty((T, self.K), dtype=torch.int32, device=xn.device)
        w = torch.empty((T, self.K), dtype=torch.float16, device=xn.device)
        self.home.encode_router(xn, weights, idx, w)
        return idx, w

    def route(self, weights, h):
        """RMSNorm + router top-k of the local rows: (xn, idx int32 [T,K], w fp16 [T,K])."""
        xn = self.norm(weights, h)
        idx, w = self.router(weights, xn)
        return xn, idx, w

    def plan(self, idx):
        T, K = idx.shape
        n = T * K
        perm = torch.empty(n, dtype=torch.int32, device=idx.device)
        inv = torch.empty(n, dtype=torch.int32, device=idx.device)
        counts = torch.empty(self.world, dtype=torch.int32, device=idx.device)
        local_expert = torch.empty(n, dtype=torch.int32, device=idx.device)
        L.check(self.lib.mfb_ep_plan(self._s(), idx.data_ptr(), T, K, self.E, self.world, perm.data_ptr(), inv.data_ptr(),
                                     counts.data_ptr(), local_expert.data_ptr()))
        return perm, inv, counts, local_expert

    def pack(self, xn, perm):
        n = perm.numel()
        rows = torch.empty((n, self.d), dtype=xn.dtype, device=xn.device)
        L.check(self.lib.mfb_ep_pack(self._s(), xn.data_ptr(), xn.stride(0), self.d, perm.data_ptr(), n, self.K, rows.data_ptr()))
        return rows

    def expert_ffn(self, local_weights, rows, local_expert):
        """fp32 [R, d] down-projection rows of the received rows through this rank's experts."""
        R = rows.shape[0]
        out = torch.empty((R, self.d), dtype=torch.float32, device=rows.device)
        if R == 0:
            return out
        idx = local_expert.view(R, 1)
        ones = torch.ones((R, 1), dtype=torch.float16, device=rows.device)
        sp, _, _, groups, n_groups = self.expert.encode_group(idx, ones)
        self.expert.encode_prefill_grouped(local_weights, rows, sp, groups, n_groups, out)
        return out

    def shared_ffn(self, shared_weights, xn):
        T = xn.shape[0]
        out = torch.empty((T, self.d), dtype=torch.float32, device=xn.device)
        idx = torch.zeros((T, 1), dtype=torch.int32, device=xn.device)
        ones = torch.ones((T, 1), dtype=torch.float16, device=xn.device)
        sp, _, _, groups, n_groups = self.shared.encode_group(idx, ones)
        self.shared.encode_prefill_grouped(shared_weights, xn, sp, groups, n_groups, out)
        return out

    def combine(self, recv, inv, w, shared_partial, residual, y):
        T = w.shape[0]
        L.check(self.lib.mfb_ep_combine(self._s(), recv.data_ptr(), inv.data_ptr(), w.data_ptr(),
                                        None if shared_partial is None else shared_partial.data_ptr(),
                                        None if residual is None else residual.data_ptr(), y.data_ptr(), T, self.K, self.d,
                                        self.x_dtype))


class ExpertParallelLayer:
    """One MoE layer over `world` ranks.  `weights`: the replicated part (router, norm, shared expert); `local_weights`:
    this rank's slice of the pool as a layer with E/world experts; `shared_weights`: the shared expert as a one-expert
    layer (or None)."""

    def __init__(self, ops, world: int, group=None):
        self.ops, self.world, self.group = ops, world, group
        self.last_send_counts: List[int] = []
        self.last_recv_counts: List[int] = []

    def forward(self, weights, local_weights, shared_weights, h_in, h_out):
        ops = self.ops
        xn, idx, w = ops.route(weights, h_in)
        perm, inv, counts, local_expert = ops.plan(idx)
        recv_counts_t = exchange_plan(counts, self.group)
        send_counts = counts.cpu().tolist()          # the one host synchronisation of a layer: split sizes for NCCL
        recv_counts = recv_counts_t.cpu().tolist()
        self.last_send_counts, self.last_recv_counts = send_counts, recv_counts
        rows = ops.pack(xn, perm)
        got_rows = exchange_rows(rows, send_counts, recv_counts, self.group)
        got_expert = exchange_rows(local_expert, send_counts, recv_counts, self.group)
        partial = ops.expert_ffn(local_weights, got_rows, got_expert)
        back = exchange_rows(partial, recv_counts, send_counts, self.group)     # reversed split sizes
        shared_partial = ops.shared_ffn(shared_weights, xn) if shared_weights is not None else None
        ops.combine(back, inv, w, shared_partial, h_in, h_out)
        return h_out


class PeerExchange:
    """mfb_ep_*: the one-sided exchange over peer memory.  Buffers are created and their CUDA IPC handles swapped once;
    after that a layer needs no collective call and no host synchronisation."""

    def __init__(self, rank: int, world: int, d: int, max_pairs: int, group=None):
        self.lib = L.load()
        self.rank, self.world, self.d, self.cap = rank, world, d, max_pairs
        self.handle = C.c_void_p()
        L.check(self.lib.mfb_ep_create(rank, world, d, max_pairs, C.byref(self.handle)))
        mine = (C.c_uint8 * 256)()
        L.check(self.lib.mfb_ep_export(self.handle, mine))
        if world > 1:
            gathered: List[bytes] = [b""] * world
            dist.all_gather_object(gathered, bytes(mine), group=group)
        else:
            gathered = [bytes(mine)]
        blob = b"".join(gathered)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        L.check(self.lib.mfb_ep_import(self.handle, buf))
        if world > 1:
            dist.barrier(group=group)   # every rank has mapped every buffer before anyone stores into one

    def close(self):
        if getattr(self, "handle", None) and self.handle.value:
            self.lib.mfb_ep_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _s():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def dispatch(self, xn, idx, num_experts):
        T, K = idx.shape
        inv = torch.empty(T * K, dtype=torch.int32, device=idx.device)
        L.check(self.lib.mfb_ep_dispatch(self.handle, self._s(), xn.data_ptr(), xn.stride(0), idx.data_ptr(), T, K, num_experts,
                                         inv.data_ptr()))
        return inv

    def receive(self):
        rows, row_expert, row_dest, n = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_uint32()
        L.check(self.lib.mfb_ep_receive(self.handle, self._s(), C.byref(rows), C.byref(row_expert), C.byref(row_dest), C.byref(n)))
        return rows.value, row_expert.value, row_dest.value, n.value

    def send_back(self):
        L.check(self.lib.mfb_ep_return(self.handle, self._s()))

    def results(self) -> int:
        ret = C.c_void_p()
        L.check(self.lib.mfb_ep_results(self.handle, self._s(), C.byref(ret)))
        return ret.value

    def status(self, with_counts: bool = False):
        st = C.c_uint32()
        counts = (C.c_int32 * self.world)() if with_counts else None
        rc = self.lib.mfb_ep_status(self.handle, self._s(), C.byref(st), counts)
        if rc not in (L.OK, L.ERR_DEVICE_STATUS):
            L.check(rc)
        return (st.value, list(counts)) if with_counts else st.value


def _view(ptr: int, shape, typestr: str):
    """A CUDA tensor over library-owned device memory (no copy, no ownership)."""
    class _Ptr:
        pass
    holder = _Ptr()
    holder.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}
    return torch.as_tensor(holder, device="cuda")


class PeerExpertParallelLayer:
    """One MoE layer over `world` ranks with the one-sided exchange: route locally, store the packed rows into the
    owners' receive buffers, run the grouped expert FFN on what arrived with every result row written straight into
    its home rank's buffer, reduce at home in rank order.  Same arguments and same result, bit for bit, as
    `ExpertParallelLayer` (and as the single-GPU prefill layer); nothing in `forward` synchronises the host."""

    def __init__(self, ops: DeviceOps, rank: int, world: int, tokens_per_rank: int, group=None):
        self.ops, self.rank, self.world = ops, rank, world
        self.cap = tokens_per_rank * ops.K
        assert ops.expert.cfg.max_tokens >= world * self.cap, "the expert-side handle must hold world * tokens * top_k rows"
        self.ex = PeerExchange(rank, world, ops.d, self.cap, group)
        # the shared expert needs only the normalised rows: it runs on a stream of its own beside the router and the
        # dispatch (few CTAs each), and is joined before the combine
        self.side = torch.cuda.Stream()

    def forward(self, weights, local_weights, shared_weights, h_in, h_out, marks=None):
        """marks: optional list that receives (name, CUDA event) at the stage boundaries (for the benchmark's breakdown)."""
        ops, ex = self.ops, self.ex

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        xn = ops.norm(weights, h_in)
        shared_partial = None
        if shared_weights is not None:
            main = torch.cuda.current_stream()
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                shared_partial = ops.shared_ffn(shared_weights, xn)
        idx, w = ops.router(weights, xn)
        mark("routed")
        inv = ex.dispatch(xn, idx, ops.E)
        mark("dispatched")
        rows_p, expert_p, dest_p, n_rows = ex.receive()
        mark("received")
        rows = _view(rows_p, (n_rows, ops.d), "<i2").view(ops.tdt)
        row_expert = _view(expert_p, (n_rows, 1), "<i4")
        ones = ops.ones_for(n_rows, rows.device)
        sp, _, _, groups, n_groups = ops.expert.encode_group(row_expert, ones)
        w_c = local_weights.c_struct()
        L.check(ops.lib.mfb_moe_prefill_grouped_rows(ops.expert.handle, ex._s(), C.byref(w_c), rows.data_ptr(), rows.stride(0), n_rows,
                                                     sp.data_ptr(), groups.data_ptr(), n_groups.data_ptr(), C.c_void_p(dest_p)))
        ex.send_back()
        mark("experts")
        ret_p = ex.results()
        mark("returned")
        if shared_partial is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        L.check(ops.lib.mfb_ep_combine(ex._s(), C.c_void_p(ret_p), inv.data_ptr(), w.data_ptr(),
                                       None if shared_partial is None else shared_partial.data_ptr(), h_in.data_ptr(),
                                       h_out.data_ptr(), h_in.shape[0], ops.K, ops.d, ops.x_dtype))
        mark("combined")
        return h_out

    def capture(self, weights, local_weights, shared_weights, h_in, h_out):
        """Records one `forward` over these (fixed) tensors into a CUDA graph.  A layer is some twenty-five small
        launches with no host synchronisation between them; issued one by one from the host they leave the GPU idle for
        a third of a short step, replayed as a graph they run back to back.  The exchange epoch lives in device memory
        and is advanced by the first kernel of the dispatch, so every replay is a new epoch on every rank.  Call
        `forward` at least once before (caches, lazily created buffers), and `replay()` on every rank the same number
        of times."""
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self.forward(weights, local_weights, shared_weights, h_in, h_out)
        self.graph = graph
        return graph

    def replay(self):
        self.graph.replay()

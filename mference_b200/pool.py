"""Expert-slot cache over an HBM-resident pool: Python mirror of the reference's ``PreadExpertStreamer`` surface
(Sources/Mference/Infrastructure/Streaming/PreadExpertStreamer.swift), over ``mfb_pool_*`` of the C ABI."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _lib as L

LFU, LRU = 0, 1


@dataclass
class ExpertCachePlan:
    """ExpertCachePlan (PreadExpertStreamer.swift): experts, the slot each one gets, which have to be filled."""
    experts: List[int]
    assigned_slots: List[int]
    misses: List[int]          # indices into ``experts``
    hits: int


class ExpertPool:
    def __init__(self, num_experts: int, slot_bytes: int, slot_count: int, policy: int = LFU, host_only: bool = False):
        self.lib = L.load()
        self.num_experts, self.slot_bytes, self.slot_count = num_experts, slot_bytes, slot_count
        self.handle = C.c_void_p()
        L.check(self.lib.mfb_pool_create(num_experts, slot_bytes, slot_count, policy, 1 if host_only else 0,
                                         C.byref(self.handle)))
        slab, stride, table = C.c_void_p(), C.c_uint64(), C.c_void_p()
        L.check(self.lib.mfb_pool_info(self.handle, C.byref(slab), C.byref(stride), C.byref(table)))
        self.slab_ptr, self.slot_stride, self.slot_of_ptr = slab.value, stride.value, table.value

    def close(self):
        if getattr(self, "handle", None) and self.handle.value:
            self.lib.mfb_pool_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # planExpertsCachedIfPossible: None when the misses cannot be placed
    def plan_experts_cached_if_possible(self, experts: Sequence[int], avoiding_slots: Sequence[int] = ()) -> Optional[ExpertCachePlan]:
        n = len(experts)
        ex = (C.c_int32 * max(n, 1))(*experts)
        av = (C.c_int32 * max(len(avoiding_slots), 1))(*avoiding_slots)
        slots = (C.c_int32 * max(n, 1))()
        miss = (C.c_uint8 * max(n, 1))()
        hits = C.c_uint32()
        rc = self.lib.mfb_pool_plan(self.handle, ex, n, av, len(avoiding_slots), slots, miss, C.byref(hits))
        if rc == L.ERR_NO_SLOT:
            return None
        L.check(rc)
        return ExpertCachePlan(list(experts), [slots[i] for i in range(n)], [i for i in range(n) if miss[i]], hits.value)

    def plan_experts_cached(self, experts: Sequence[int], avoiding_slots: Sequence[int] = ()) -> ExpertCachePlan:
        plan = self.plan_experts_cached_if_possible(experts, avoiding_slots)
        if plan is None:
            raise L.MfbError(L.ERR_NO_SLOT, "expert cache cannot place requested misses")
        return plan

    def _arrays(self, plan: ExpertCachePlan):
        n = len(plan.experts)
        ex = (C.c_int32 * max(n, 1))(*plan.experts)
        sl = (C.c_int32 * max(n, 1))(*plan.assigned_slots)
        missing = set(plan.misses)
        ms = (C.c_uint8 * max(n, 1))(*[1 if i in missing else 0 for i in range(n)])
        return n, ex, sl, ms

    def fill_async(self, plan: ExpertCachePlan, host_blobs, stream: int = 0):
        """beginAsyncFill: copy the plan's misses from pinned host tensors (host_blobs[expert] -> uint8 tensor) into
        their slots on ``stream``.  The device slot table is untouched until ``publish``."""
        if not plan.misses:
            return
        n, ex, sl, ms = self._arrays(plan)
        ptrs = (C.c_void_p * max(n, 1))()
        blob_bytes = None
        for i in plan.misses:
            t = host_blobs[plan.experts[i]]
            ptrs[i] = t.data_ptr()
            size = t.numel() * t.element_size()
            if blob_bytes is not None and size != blob_bytes:   # one byte count serves every copy of the call
                raise L.MfbError(L.ERR_IO, f"expert blobs of different sizes in one fill ({blob_bytes} and {size} bytes)")
            blob_bytes = size
        L.check(self.lib.mfb_pool_fill_async(self.handle, C.c_void_p(stream), ex, sl, ms, n, ptrs, blob_bytes))

    def publish(self, plan: ExpertCachePlan, stream: int = 0):
        """Makes the plan's slot assignment visible to kernels launched on ``stream`` after this call."""
        n, ex, sl, ms = self._arrays(plan)
        L.check(self.lib.mfb_pool_publish(self.handle, C.c_void_p(stream), ex, sl, ms, n))

    def execute_expert_cache_plan(self, plan: ExpertCachePlan, host_blobs, stream: int = 0):
        """Fill the misses from pinned host tensors and publish them, all on ``stream``.  Returns the byte offset of
        every expert's slot in the slab."""
        self.fill_async(plan, host_blobs, stream)
        self.publish(plan, stream)
        return [s * self.slot_stride for s in plan.assigned_slots]

    # ---- speculative / eager staging (PreadExpertStreamer.swift:330-469) ----------------------------------------------
    def non_resident_experts(self, experts: Sequence[int]) -> List[int]:
        """The experts of a prediction that no slot holds (what is worth reading ahead), in order, without duplicates."""
        table = self.slot_of_host()
        out: List[int] = []
        for e in experts:
            if 0 <= e < self.num_experts and table[e] < 0 and e not in out:
                out.append(e)
        return out

    def reserve_speculative_slots(self, experts: Sequence[int], keep_evictable: int) -> List[tuple]:
        """reserveSpeculativeSlots: [(expert, slot)] for as many of `experts` as fit while `keep_evictable` evictable slots
        stay untouched; the reserved slots are in flight (never victims, reading -1) until the reservation is executed."""
        n = len(experts)
        if n == 0:
            return []
        ex = (C.c_int32 * n)(*experts)
        out_e, out_s, out_n = (C.c_int32 * n)(), (C.c_int32 * n)(), C.c_uint32()
        L.check(self.lib.mfb_pool_reserve_speculative(self.handle, ex, n, max(0, keep_evictable), out_e, out_s, C.byref(out_n)))
        return [(out_e[i], out_s[i]) for i in range(out_n.value)]

    def execute_speculative_reservation(self, reservation: Sequence[tuple], host_blobs, stream: int = 0) -> int:
        """executeSpeculativeReservation: copies every reserved expert that `host_blobs` can supply into its slot on
        `stream`, then publishes exactly those (an expert without a source - the failed read of the reference - leaves
        its slot empty) and clears every in-flight mark.  Returns the bytes queued."""
        n = len(reservation)
        if n == 0:
            return 0
        ex = (C.c_int32 * n)(*[e for e, _ in reservation])
        sl = (C.c_int32 * n)(*[s for _, s in reservation])
        loaded = (C.c_uint8 * n)(*[1 if host_blobs.get(e) is not None else 0 for e, _ in reservation])
        ptrs = (C.c_void_p * n)()
        blob_bytes = None
        for i, (e, _) in enumerate(reservation):
            if loaded[i]:
                t = host_blobs[e]
                ptrs[i] = t.data_ptr()
                size = t.numel() * t.element_size()
                if blob_bytes is not None and size != blob_bytes:
                    raise L.MfbError(L.ERR_IO, f"expert blobs of different sizes in one fill ({blob_bytes} and {size} bytes)")
                blob_bytes = size
        if blob_bytes is not None:
            L.check(self.lib.mfb_pool_fill_async(self.handle, C.c_void_p(stream), ex, sl, loaded, n, ptrs, blob_bytes))
        L.check(self.lib.mfb_pool_finish_speculative(self.handle, C.c_void_p(stream), ex, sl, loaded, n))
        return sum(loaded) * (blob_bytes or 0)

    def begin_async_fill(self, plan: ExpertCachePlan, host_blobs, stream: int = 0) -> bool:
        """beginAsyncFill: the plan's miss slots are marked in flight (concurrent plans keep away from them), their copies
        are queued on `stream` and published behind them in stream order; GPU work the caller queues on the same stream
        afterwards sees the filled slots.  False = at least one source was missing: that slot stays unpublished and the
        caller must not use the layer's result (the reference's completion(false))."""
        pairs = [(plan.experts[i], plan.assigned_slots[i]) for i in plan.misses]
        if not pairs:
            return True
        sl = (C.c_int32 * len(pairs))(*[s for _, s in pairs])
        L.check(self.lib.mfb_pool_mark_in_flight(self.handle, sl, len(pairs)))
        sizes = {host_blobs[e].numel() * host_blobs[e].element_size() for e, _ in pairs if host_blobs.get(e) is not None}
        queued = self.execute_speculative_reservation(pairs, host_blobs, stream)
        return len(sizes) == 1 and queued == len(pairs) * next(iter(sizes))

    def note_all_hit_use(self, experts: Sequence[int]):
        ex = (C.c_int32 * max(len(experts), 1))(*experts)
        L.check(self.lib.mfb_pool_note_all_hit(self.handle, ex, len(experts)))

    def slot_of_host(self) -> np.ndarray:
        out = np.empty(self.num_experts, dtype=np.int16)
        L.check(self.lib.mfb_pool_slot_of_host(self.handle, out.ctypes.data_as(C.c_void_p)))
        return out

    def slab_tensor(self):
        """The slab as a uint8 CUDA tensor view (no copy; the pool keeps ownership)."""
        import torch

        class _Ptr:
            pass
        holder = _Ptr()
        holder.__cuda_array_interface__ = {"shape": (self.slot_count * self.slot_stride,), "typestr": "|u1",
                                           "data": (self.slab_ptr, False), "version": 2}
        return torch.as_tensor(holder, device="cuda")

    def slot_of_tensor(self):
        import torch

        class _Ptr:
            pass
        holder = _Ptr()
        holder.__cuda_array_interface__ = {"shape": (self.num_experts,), "typestr": "<i2",
                                           "data": (self.slot_of_ptr, False), "version": 2}
        return torch.as_tensor(holder, device="cuda")

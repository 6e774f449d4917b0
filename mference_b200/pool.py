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

"""Streamed grouped prefill through a pool that holds fewer slots than the layer has experts.

Host logic of the reference's tile pipeline, with the same names and decisions:

* ``PrefillRoutedTileScheduler`` (Sources/Mference/Kernels/Prefill/MoE/PrefillRoutedTileScheduler.swift:1-67):
  issue / prefetch the next tile around the pending tile's slots / drain first, and the slot budget rule
  ``(max_pending_depth + 1) * tile_experts + reserved_hits <= slot_count``.
* ``PrefillStreamedTileSlotLifetime`` (Sources/Mference/Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:66-102):
  a slot may not be handed to a tile while another tile that uses it is still in flight.
* ``StreamedGroupedPrefill.encode`` plays ``PrefillGroupedRoutedMoE.encodeStreamedBatched`` (:391-466): the sorted
  pair list is cut into tiles of at most ``tile_experts`` expert groups; while the kernels of tile t run on the
  compute stream, the missing experts of tile t+1 are copied from pinned host memory into slots that tile t does
  not use, on a copy stream.  Events order the two streams; nothing here blocks the host except a drain.

The compute of a tile is the library's grouped FFN (``mfb_moe_prefill_grouped``) on that tile's groups, so the
result is the same bits as with every expert resident.
"""
from __future__ import annotations

import ctypes as C
import enum
from collections import deque
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from . import _lib as L


class DrainReason(enum.Enum):
    PENDING_TILE_HAS_NO_ASSIGNED_SLOTS = "pendingTileHasNoAssignedSlots"
    AVOIDING_SLOT_PLAN_UNAVAILABLE = "avoidingSlotPlanUnavailable"
    MAX_PENDING_DEPTH_REACHED = "maxPendingDepthReached"


@dataclass(frozen=True)
class Decision:
    """One of ``issue_without_pending``, ``prefetch_next`` (with the slots to keep away from, in the order given)
    and ``drain_before_issue`` (with the reason)."""
    kind: str
    avoiding_slots: Tuple[int, ...] = ()
    reason: Optional[DrainReason] = None

    @staticmethod
    def issue_without_pending() -> "Decision":
        return Decision("issue_without_pending")

    @staticmethod
    def prefetch_next(avoiding_slots: Sequence[int]) -> "Decision":
        return Decision("prefetch_next", tuple(avoiding_slots))

    @staticmethod
    def drain_before_issue(reason: DrainReason) -> "Decision":
        return Decision("drain_before_issue", (), reason)


class PrefillRoutedTileSchedulerInput:
    def __init__(self, has_pending_tile: bool, pending_assigned_slots: Sequence[int], avoiding_slot_plan_available: bool,
                 pending_depth: Optional[int] = None):
        self.has_pending_tile = bool(has_pending_tile)
        depth = pending_depth if pending_depth is not None else (1 if has_pending_tile else 0)
        self.pending_depth = max(0, int(depth))
        self.pending_assigned_slots = list(pending_assigned_slots)
        self.avoiding_slot_plan_available = bool(avoiding_slot_plan_available)


class PrefillRoutedTileSchedulerConfig:
    def __init__(self, max_pending_depth: int = 1, tile_experts: int = 8):
        self.max_pending_depth = max(1, int(max_pending_depth))
        self.tile_experts = max(1, min(16, int(tile_experts)))

    def fits_slot_budget(self, slot_count: int, reserved_hits: int = 0) -> bool:
        if slot_count <= 0 or reserved_hits < 0:
            return False
        return (self.max_pending_depth + 1) * self.tile_experts + reserved_hits <= slot_count


class PrefillRoutedTileScheduler:
    def __init__(self, config: Optional[PrefillRoutedTileSchedulerConfig] = None):
        self.config = config or PrefillRoutedTileSchedulerConfig()

    def decide(self, inp: PrefillRoutedTileSchedulerInput) -> Decision:
        if not inp.has_pending_tile:
            return Decision.issue_without_pending()
        if inp.pending_depth > self.config.max_pending_depth:
            return Decision.drain_before_issue(DrainReason.MAX_PENDING_DEPTH_REACHED)
        if not inp.pending_assigned_slots:
            return Decision.drain_before_issue(DrainReason.PENDING_TILE_HAS_NO_ASSIGNED_SLOTS)
        if not inp.avoiding_slot_plan_available:
            return Decision.drain_before_issue(DrainReason.AVOIDING_SLOT_PLAN_UNAVAILABLE)
        return Decision.prefetch_next(inp.pending_assigned_slots)


class PrefillStreamedTileLifetimeError(RuntimeError):
    """``case`` is one of duplicateSlots, slotReuseBeforeCompletion, completeWithoutInFlightTile."""

    def __init__(self, case: str, tile_index: int, slots: Sequence[int] = (), conflicting_tile_index: Optional[int] = None):
        self.case, self.tile_index, self.slots = case, tile_index, list(slots)
        self.conflicting_tile_index = conflicting_tile_index
        if case == "duplicateSlots":
            msg = f"prefill streamed tile {tile_index} plans duplicate slots {self.slots}"
        elif case == "slotReuseBeforeCompletion":
            msg = (f"prefill streamed tile {tile_index} reuses slots {self.slots} before tile "
                   f"{conflicting_tile_index} completed")
        else:
            msg = f"prefill streamed tile {tile_index} completed without a matching in-flight tile"
        super().__init__(msg)


class PrefillStreamedTileSlotLifetime:
    def __init__(self):
        self._in_flight: Dict[int, frozenset] = {}

    def begin(self, tile_index: int, planned_slots: Sequence[int]) -> None:
        slots = set()
        for s in planned_slots:
            if s in slots:
                raise PrefillStreamedTileLifetimeError("duplicateSlots", tile_index, sorted(planned_slots))
            slots.add(s)
        for other, other_slots in self._in_flight.items():
            overlap = slots & other_slots
            if overlap:
                raise PrefillStreamedTileLifetimeError("slotReuseBeforeCompletion", tile_index, sorted(overlap), other)
        self._in_flight[tile_index] = frozenset(slots)

    def complete(self, tile_index: int) -> None:
        if self._in_flight.pop(tile_index, None) is None:
            raise PrefillStreamedTileLifetimeError("completeWithoutInFlightTile", tile_index)

    @property
    def in_flight_tiles(self) -> List[int]:
        return sorted(self._in_flight)


class StreamedGroupedPrefill:
    """Grouped routed FFN of a prefill chunk with the experts staged tile by tile through ``pool``.

    ``host_blobs[e]`` is expert e's blob as a pinned uint8 tensor.  ``encode`` returns without waiting for the GPU;
    tiles still in flight are kept (and their slots kept away from) until ``drain`` or a later ``encode`` retires them.
    ``decisions`` logs (tile index, Decision) for every tile issued.
    """

    def __init__(self, moe, pool, host_blobs, config: Optional[PrefillRoutedTileSchedulerConfig] = None):
        import torch
        self.moe, self.pool, self.host_blobs = moe, pool, host_blobs
        self.lib = L.load()
        self.scheduler = PrefillRoutedTileScheduler(config)
        cfg = self.scheduler.config
        if not cfg.fits_slot_budget(pool.slot_count):
            raise ValueError(f"streamed prefill: ({cfg.max_pending_depth} + 1) x {cfg.tile_experts} experts do not fit "
                             f"{pool.slot_count} slots")
        self.copy_stream = torch.cuda.Stream()
        self.lifetime = PrefillStreamedTileSlotLifetime()
        self.decisions: List[Tuple[int, Decision]] = []
        self._pending = deque()      # (tile serial, slots, event recorded after the tile's kernels)
        self._serial = 0
        self.filled_experts = 0      # blobs copied host -> HBM so far

    # -- in-flight bookkeeping -------------------------------------------------------------------------------
    def _retire_finished(self) -> None:
        while self._pending and self._pending[0][2].query():
            serial, _, _ = self._pending.popleft()
            self.lifetime.complete(serial)

    def drain(self) -> None:
        """Blocks until every issued tile has finished and releases their slots."""
        while self._pending:
            serial, _, done = self._pending.popleft()
            done.synchronize()
            self.lifetime.complete(serial)

    # -- one chunk ---------------------------------------------------------------------------------------------
    def encode(self, weights, x, sorted_pairs, groups, n_groups, partial) -> None:
        """``weights``: the layer's replicated part (offsets, shared expert ...); its pool fields are replaced by this
        object's pool.  ``sorted_pairs``, ``groups``, ``n_groups``: device output of the grouping.  ``partial``:
        f32 [tokens * top_k, d]."""
        import copy
        import torch
        cfg = self.scheduler.config
        n = int(n_groups.item())     # the one host read of a chunk (the reference groups on the CPU)
        if n == 0:
            return
        host_groups = groups[:n].cpu().numpy()
        tiles = [(s, min(cfg.tile_experts, n - s)) for s in range(0, n, cfg.tile_experts)]
        counts = torch.tensor([c for _, c in tiles], dtype=torch.int32, device=x.device)
        compute = torch.cuda.current_stream()
        staged = copy.copy(weights)
        staged.pool, staged.slot_stride, staged.slot_of = self.pool.slab_tensor(), self.pool.slot_stride, self.pool.slot_of_tensor()
        w = staged.c_struct()
        group_bytes = groups.element_size() * groups.shape[1]
        for t, (start, count) in enumerate(tiles):
            experts = [int(e) for e in host_groups[start:start + count, 0] if int(e) < self.pool.num_experts]
            self._retire_finished()
            avoid = [s for (_, slots, _) in self._pending for s in slots]
            plan = self.pool.plan_experts_cached_if_possible(experts, avoid) if self._pending else None
            decision = self.scheduler.decide(PrefillRoutedTileSchedulerInput(
                bool(self._pending), avoid, plan is not None, pending_depth=len(self._pending)))
            if decision.kind == "drain_before_issue":
                self.drain()
            if plan is None:
                plan = self.pool.plan_experts_cached(experts)
            serial = self._serial
            self._serial += 1
            self.decisions.append((serial, decision))
            self.lifetime.begin(serial, plan.assigned_slots)
            # copies of the misses on the copy stream; the table and the kernels follow on the compute stream
            self.pool.fill_async(plan, self.host_blobs, self.copy_stream.cuda_stream)
            self.filled_experts += len(plan.misses)
            filled = torch.cuda.Event()
            filled.record(self.copy_stream)
            compute.wait_event(filled)
            self.pool.publish(plan, compute.cuda_stream)
            L.check(self.lib.mfb_moe_prefill_grouped(
                self.moe.handle, C.c_void_p(compute.cuda_stream), C.byref(w), C.c_void_p(x.data_ptr()), x.stride(0), x.shape[0],
                C.c_void_p(sorted_pairs.data_ptr()), C.c_void_p(groups.data_ptr() + start * group_bytes),
                C.c_void_p(counts.data_ptr() + 4 * t), C.c_void_p(partial.data_ptr())))
            done = torch.cuda.Event()
            done.record(compute)
            # a later tile's copies may only overwrite these slots once this event has completed (see _retire_finished)
            self._pending.append((serial, list(plan.assigned_slots), done))

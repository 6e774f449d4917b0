"""Expert-slot cache: planning rules restated from the reference's own cache-planning tests
(Tests/Mference/Core/Infrastructure/Streaming/PreadExpertStreamerTests+CachePlanning.swift), on the host-only pool
(no GPU), and the fill / publish path with tagged blobs on the GPU."""
import numpy as np
import pytest

from mference_b200 import _lib as L
from mference_b200.pool import LFU, LRU, ExpertPool


def _warm(pool, experts):
    plan = pool.plan_experts_cached(experts)
    n, ex, sl, ms = pool._arrays(plan)
    L.check(pool.lib.mfb_pool_publish(pool.handle, None, ex, sl, ms, n))   # host-only: bookkeeping only
    return plan


def test_plan_reports_hits_and_misses_in_request_order():
    pool = ExpertPool(8, 1024, 4, host_only=True)
    _warm(pool, [0])
    plan = pool.plan_experts_cached([0, 1, 2])
    assert plan.hits == 1
    assert [plan.experts[i] for i in plan.misses] == [1, 2]
    assert plan.assigned_slots[0] == 0 and sorted(plan.assigned_slots) == [0, 1, 2]


def test_plan_avoids_in_flight_slots_for_hits_and_misses():
    pool = ExpertPool(8, 1024, 4, host_only=True)
    _warm(pool, [0, 1])
    plan = pool.plan_experts_cached([0, 2], avoiding_slots=[0, 1])
    assert plan.assigned_slots == [0, 2]
    assert plan.hits == 1
    assert plan.misses == [1]


def test_plan_is_refused_when_misses_cannot_avoid_in_flight_slots():
    pool = ExpertPool(8, 1024, 4, host_only=True)
    _warm(pool, [0, 1])
    before = pool.slot_of_host().copy()
    assert pool.plan_experts_cached_if_possible([0, 2, 3, 4], avoiding_slots=[0, 1]) is None
    assert np.array_equal(pool.slot_of_host(), before)      # a refused plan changes nothing
    with pytest.raises(L.MfbError):
        pool.plan_experts_cached([0, 2, 3, 4], avoiding_slots=[0, 1])


def test_lfu_evicts_the_least_used_expert_and_lru_the_oldest():
    for policy, expect_victim in ((LFU, 1), (LRU, 0)):
        pool = ExpertPool(8, 1024, 2, policy=policy, host_only=True)
        _warm(pool, [0, 1])
        _warm(pool, [0])          # expert 0: used twice
        _warm(pool, [0])
        pool.note_all_hit_use([1])   # expert 1: used twice too, but more recently; expert 0 used three times
        plan = pool.plan_experts_cached([5])
        table = pool.slot_of_host()
        assert table[expect_victim] == -1, policy
        assert plan.misses == [0]


def test_victim_slot_reads_minus_one_until_published():
    pool = ExpertPool(8, 1024, 2, host_only=True)
    _warm(pool, [0, 1])
    plan = pool.plan_experts_cached([2])
    table = pool.slot_of_host()
    assert table[2] == -1 and (table[0] == -1) != (table[1] == -1)
    n, ex, sl, ms = pool._arrays(plan)
    L.check(pool.lib.mfb_pool_publish(pool.handle, None, ex, sl, ms, n))
    assert pool.slot_of_host()[2] == plan.assigned_slots[0]


def test_too_many_experts_for_the_slot_count_is_a_contract_violation():
    pool = ExpertPool(8, 1024, 2, host_only=True)
    with pytest.raises(L.MfbError) as err:
        pool.plan_experts_cached([0, 1, 2])
    assert err.value.code == L.ERR_INVALID_ARGUMENT


@pytest.mark.gpu
def test_fill_and_publish_move_tagged_blobs_and_update_the_device_table():
    import torch
    E, stride, slots = 6, 4096, 4
    pool = ExpertPool(E, stride, slots)
    host = {e: torch.full((stride,), 16 + e, dtype=torch.uint8).pin_memory() for e in range(E)}
    s = torch.cuda.current_stream().cuda_stream
    offs = pool.execute_expert_cache_plan(pool.plan_experts_cached([0]), host, s)
    plan = pool.plan_experts_cached([0, 1, 2])
    assert plan.hits == 1 and [plan.experts[i] for i in plan.misses] == [1, 2]
    offs = pool.execute_expert_cache_plan(plan, host, s)
    torch.cuda.synchronize()
    slab = pool.slab_tensor()
    for e, off in zip(plan.experts, offs):
        assert bool((slab[off:off + stride] == 16 + e).all())
    table = pool.slot_of_tensor().cpu().numpy()
    assert np.array_equal(table, pool.slot_of_host())
    assert [int(table[e]) for e in (0, 1, 2)] == plan.assigned_slots and table[3] == -1
    # eviction under pressure: four more experts through a four-slot pool
    plan2 = pool.plan_experts_cached([3, 4, 5, 0])
    offs2 = pool.execute_expert_cache_plan(plan2, host, s)
    torch.cuda.synchronize()
    for e, off in zip(plan2.experts, offs2):
        assert bool((slab[off:off + stride] == 16 + e).all())
    assert np.array_equal(pool.slot_of_tensor().cpu().numpy(), pool.slot_of_host())


@pytest.mark.gpu
def test_decode_through_a_partially_resident_pool_matches_full_residency():
    """Experts staged through the cache give the same layer output as the fully resident slab; an expert that is
    not resident contributes nothing (the guarded kernels of the reference, moe.metal:586-708)."""
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    d, f, E, K, T = 512, 256, 16, 4, 5
    layer = synth_layer(0xB2000001, 0, d, f, E)
    moe = MoE(d, f, E, K, max_tokens=T)
    x = synth_normal(0xB2000001, "x.pool", T * d, dtype=L.DT_BF16).view(T, d)
    y_full = torch.empty_like(x)
    moe.encode_layer(layer, x, y_full)
    # stage exactly the experts this batch routes to into an 8-slot pool
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float16, device="cuda")
    xn = torch.empty_like(x)
    moe.encode_rmsnorm(x, xn, layer.norm_w)
    moe.encode_router(xn, layer, idx, w)
    need = sorted(set(idx.cpu().numpy().reshape(-1).tolist()))
    blob = layer.slot_stride
    pool = ExpertPool(E, blob, max(len(need), 8))
    host = {e: layer.pool[e * blob:(e + 1) * blob].cpu().pin_memory() for e in need}
    s = torch.cuda.current_stream().cuda_stream
    pool.execute_expert_cache_plan(pool.plan_experts_cached(need), host, s)
    import copy
    staged = copy.copy(layer)
    staged.pool, staged.slot_stride, staged.slot_of = pool.slab_tensor(), pool.slot_stride, pool.slot_of_tensor()
    y_pool = torch.empty_like(x)
    moe.encode_layer(staged, x, y_pool)
    torch.cuda.synchronize()
    assert torch.equal(y_pool, y_full)


# ---- speculative / eager staging (PreadExpertStreamer.swift:330-469) -------------------------------------------------

class _FakeBlob:
    """Stands in for a pinned host tensor on the host-only pool (nothing is copied there)."""

    def __init__(self, n):
        self.n = n

    def data_ptr(self):
        return 0

    def numel(self):
        return self.n

    def element_size(self):
        return 1


def test_speculative_reservation_protects_predicted_and_in_flight_slots_and_keeps_room():
    pool = ExpertPool(16, 1024, 6, host_only=True)
    _warm(pool, [0, 1, 2, 3])                 # slots 0-3 hold experts 0-3, slots 4 and 5 are empty
    assert pool.non_resident_experts([2, 9, 9, 3, 10, 99]) == [9, 10]
    # predicted expert 2 is resident: its slot may not be taken; two evictable slots must stay for the real plan
    res = pool.reserve_speculative_slots([9, 10, 11, 12], keep_evictable=2)
    # evictable = 6 slots - none in flight - the slot of ... (no predicted expert is among the wanted ids 9-12) = 6,
    # budget = min(4, 6 - 2) = 4, empty slots go first
    assert [e for e, _ in res] == [9, 10, 11, 12]
    assert {s for _, s in res[:2]} == {4, 5}
    table = pool.slot_of_host()
    assert all(table[e] == -1 for e in (9, 10, 11, 12))          # nothing is published yet
    evicted = [e for e in (0, 1, 2, 3) if table[e] == -1]
    assert len(evicted) == 2                                      # two resident experts gave up their slots
    # a second prediction while the first is in flight: its slots are never victims, and with keep_evictable = 2 the two
    # slots left are out of reach
    assert pool.reserve_speculative_slots([13], keep_evictable=2) == []
    # a real plan in between keeps away from the in-flight slots too
    plan = pool.plan_experts_cached([14])
    assert plan.assigned_slots[0] not in {s for _, s in res}
    # one read fails (no source for expert 11): its slot stays empty, the others become hits, marks are cleared
    blobs = {9: _FakeBlob(1024), 10: _FakeBlob(1024), 12: _FakeBlob(1024)}
    with pytest.raises(L.MfbError):                               # host-only pool: copies are refused, bookkeeping is not
        pool.execute_speculative_reservation(res, blobs)
    ex = [e for e, _ in res]
    sl = [s for _, s in res]
    import ctypes as C
    L.check(pool.lib.mfb_pool_finish_speculative(pool.handle, None, (C.c_int32 * 4)(*ex), (C.c_int32 * 4)(*sl),
                                                 (C.c_uint8 * 4)(1, 1, 0, 1), 4))
    table = pool.slot_of_host()
    assert [table[e] for e in (9, 10, 12)] == [sl[0], sl[1], sl[3]] and table[11] == -1
    assert len(pool.reserve_speculative_slots([13], keep_evictable=0)) == 1     # the marks are gone


def test_speculative_reservation_writes_no_policy_bookkeeping():
    # LFU: expert 0 used three times, expert 1 once.  A speculative guess of expert 1's neighbours must not change which
    # expert the next real plan evicts.
    a = ExpertPool(8, 1024, 2, policy=LFU, host_only=True)
    b = ExpertPool(8, 1024, 2, policy=LFU, host_only=True)
    for pool in (a, b):
        _warm(pool, [0, 1])
        _warm(pool, [0])
        _warm(pool, [0])
    assert b.reserve_speculative_slots([5, 6], keep_evictable=2) == []          # no room beyond what must stay evictable
    for pool in (a, b):
        plan = pool.plan_experts_cached([7])
        assert pool.slot_of_host()[1] == -1 and pool.slot_of_host()[0] >= 0     # the less used expert 1 went, in both


@pytest.mark.gpu
def test_speculative_and_eager_fills_move_blobs_and_respect_failures():
    import torch
    E, n_bytes = 8, 4096
    pool = ExpertPool(E, n_bytes, 4)
    blobs = {e: torch.full((n_bytes,), e + 1, dtype=torch.uint8).pin_memory() for e in range(E)}
    stream = torch.cuda.current_stream().cuda_stream
    res = pool.reserve_speculative_slots(pool.non_resident_experts([2, 5]), keep_evictable=2)
    assert [e for e, _ in res] == [2, 5]
    assert pool.execute_speculative_reservation(res, blobs, stream) == 2 * n_bytes
    torch.cuda.synchronize()
    slab, table = pool.slab_tensor(), pool.slot_of_tensor().cpu().numpy()
    for e, s in res:
        assert table[e] == s and bool((slab[s * pool.slot_stride: s * pool.slot_stride + n_bytes] == e + 1).all())
    # eager fill of a real plan: expert 2 hits, 6 and 7 miss; the source of 7 is missing -> reported, slot unpublished
    plan = pool.plan_experts_cached([2, 6, 7])
    assert plan.hits == 1
    partial = {k: v for k, v in blobs.items() if k != 7}
    assert pool.begin_async_fill(plan, partial, stream) is False
    torch.cuda.synchronize()
    table = pool.slot_of_tensor().cpu().numpy()
    assert table[6] == plan.assigned_slots[1] and table[7] == -1 and table[2] == plan.assigned_slots[0]
    plan2 = pool.plan_experts_cached([7])
    assert pool.begin_async_fill(plan2, blobs, stream) is True
    torch.cuda.synchronize()
    assert pool.slot_of_tensor().cpu().numpy()[7] == plan2.assigned_slots[0]

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

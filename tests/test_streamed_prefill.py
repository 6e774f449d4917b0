"""Tile scheduler and slot lifetime of the streamed prefill (host logic), and the streamed grouped FFN on the GPU.

The decision cases are the ones the reference checks in
Tests/Mference/Core/Kernels/Prefill/PrefillRoutedTileSchedulerTests.swift; the lifetime cases follow
PrefillStreamedTileSlotLifetime (PrefillGroupedRoutedMoE.swift:66-102)."""
import pytest

from mference_b200 import _lib as L
from mference_b200.streamed_prefill import (Decision, DrainReason, PrefillRoutedTileScheduler,
                                            PrefillRoutedTileSchedulerConfig as Config,
                                            PrefillRoutedTileSchedulerInput as Input,
                                            PrefillStreamedTileLifetimeError, PrefillStreamedTileSlotLifetime)


def test_first_tile_is_issued_without_pending_work():
    d = PrefillRoutedTileScheduler().decide(Input(False, [], False))
    assert d == Decision.issue_without_pending()


def test_next_tile_is_prefetched_around_the_pending_tiles_slots():
    d = PrefillRoutedTileScheduler().decide(Input(True, [3, 7, 8], True))
    assert d == Decision.prefetch_next([3, 7, 8])
    # the order (and repeats) of the pending slots is passed through untouched
    d = PrefillRoutedTileScheduler().decide(Input(True, [9, 1, 9, 3], True))
    assert d.kind == "prefetch_next" and d.avoiding_slots == (9, 1, 9, 3)


def test_drain_reasons_in_order_of_precedence():
    s = PrefillRoutedTileScheduler()
    assert s.decide(Input(True, [], True)) == Decision.drain_before_issue(DrainReason.PENDING_TILE_HAS_NO_ASSIGNED_SLOTS)
    assert s.decide(Input(True, [1, 2], False)) == Decision.drain_before_issue(DrainReason.AVOIDING_SLOT_PLAN_UNAVAILABLE)
    # depth is checked before anything else
    assert s.decide(Input(True, [], False, pending_depth=2)) == Decision.drain_before_issue(DrainReason.MAX_PENDING_DEPTH_REACHED)


def test_pending_depth_budget():
    s = PrefillRoutedTileScheduler(Config(max_pending_depth=2, tile_experts=4))
    slots = [1, 2, 3, 4, 5, 6, 7, 8]
    assert s.decide(Input(True, slots, True, pending_depth=2)) == Decision.prefetch_next(slots)
    assert s.decide(Input(True, [1, 2], True, pending_depth=3)) == Decision.drain_before_issue(DrainReason.MAX_PENDING_DEPTH_REACHED)
    # default depth: 1 with a pending tile, 0 without; negative depths clamp to 0
    assert Input(True, [1], True).pending_depth == 1 and Input(False, [], True).pending_depth == 0
    assert Input(True, [1], True, pending_depth=-4).pending_depth == 0


def test_config_clamps_and_slot_budget():
    assert Config(0, 0).max_pending_depth == 1 and Config(0, 0).tile_experts == 1 and Config(1, 99).tile_experts == 16
    assert Config().fits_slot_budget(16)                       # (1 + 1) * 8 = 16
    assert Config(2, 4).fits_slot_budget(16)                   # 3 * 4 = 12
    assert not Config(2, 8).fits_slot_budget(16)               # 3 * 8 = 24
    assert not Config().fits_slot_budget(16, reserved_hits=1)
    assert not Config().fits_slot_budget(0) and not Config().fits_slot_budget(64, reserved_hits=-1)


def test_slot_lifetime_rejects_reuse_before_completion():
    life = PrefillStreamedTileSlotLifetime()
    life.begin(0, [4, 5, 6])
    life.begin(1, [7, 8])
    with pytest.raises(PrefillStreamedTileLifetimeError) as e:
        life.begin(2, [9, 5, 4])
    assert e.value.case == "slotReuseBeforeCompletion" and e.value.slots == [4, 5] and e.value.conflicting_tile_index == 0
    assert life.in_flight_tiles == [0, 1]                      # a refused tile leaves nothing behind
    life.complete(0)
    life.begin(2, [9, 5, 4])
    with pytest.raises(PrefillStreamedTileLifetimeError) as e:
        life.begin(3, [1, 2, 1])
    assert e.value.case == "duplicateSlots" and e.value.slots == [1, 1, 2]
    with pytest.raises(PrefillStreamedTileLifetimeError) as e:
        life.complete(0)
    assert e.value.case == "completeWithoutInFlightTile"
    life.complete(1)
    life.complete(2)
    assert life.in_flight_tiles == []


def _layer_and_grouping(d, f, E, K, T):
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    layer = synth_layer(0xB2000001, 0, d, f, E)
    moe = MoE(d, f, E, K, max_tokens=T, shared_bits=0)
    x = synth_normal(0xB2000001, "x.streamed", T * d, dtype=L.DT_BF16).view(T, d)
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float16, device="cuda")
    moe.encode_router(x, layer, idx, w)
    sp, _, _, groups, n_groups = moe.encode_group(idx, w)
    return layer, moe, x, sp, groups, n_groups


@pytest.mark.gpu
@pytest.mark.parametrize("tile_experts,slots,depth", [(4, 8, 1), (4, 16, 2), (8, 16, 1), (3, 9, 2)])
def test_streamed_grouped_ffn_matches_full_residency(tile_experts, slots, depth):
    """Experts staged tile by tile through a pool much smaller than the layer give the same partial rows, bit for
    bit, as the fully resident slab; the second chunk reuses what the first left in the pool."""
    import copy
    import torch
    from mference_b200.pool import ExpertPool
    from mference_b200.streamed_prefill import StreamedGroupedPrefill
    d, f, E, K, T = 512, 512, 32, 4, 192
    layer, moe, x, sp, groups, n_groups = _layer_and_grouping(d, f, E, K, T)
    routed = copy.copy(layer)
    routed.shared_blob = None
    want = torch.zeros((T * K, d), dtype=torch.float32, device="cuda")
    moe.encode_prefill_grouped(routed, x, sp, groups, n_groups, want)
    blob = layer.slot_stride
    host = {e: layer.pool[e * blob:(e + 1) * blob].cpu().pin_memory() for e in range(E)}
    pool = ExpertPool(E, blob, slots)
    streamed = StreamedGroupedPrefill(moe, pool, host, Config(max_pending_depth=depth, tile_experts=tile_experts))
    for chunk in range(2):
        got = torch.full((T * K, d), float("nan"), dtype=torch.float32, device="cuda")
        streamed.encode(routed, x, sp, groups, n_groups, got)
        streamed.drain()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    n_tiles = -(-int(n_groups.item()) // tile_experts)
    kinds = [dec.kind for _, dec in streamed.decisions]
    assert len(kinds) == 2 * n_tiles and kinds[0] == "issue_without_pending"
    assert streamed.lifetime.in_flight_tiles == []
    assert streamed.filled_experts >= int(n_groups.item())     # every expert crossed PCIe at least once
    for _, dec in streamed.decisions:
        if dec.kind == "prefetch_next":
            assert len(dec.avoiding_slots) <= depth * tile_experts


@pytest.mark.gpu
def test_streamed_prefill_refuses_a_pool_below_the_slot_budget():
    from mference_b200.moe import MoE
    from mference_b200.pool import ExpertPool
    from mference_b200.streamed_prefill import StreamedGroupedPrefill
    moe = MoE(512, 512, 32, 4, max_tokens=8, shared_bits=0)
    pool = ExpertPool(32, 4096, 15)
    with pytest.raises(ValueError):
        StreamedGroupedPrefill(moe, pool, {}, Config(max_pending_depth=1, tile_experts=8))

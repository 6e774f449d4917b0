"""CPU tests of the C ABI boundary: the library loads, exports every symbol the header declares, keeps the
struct layouts the reference pins, and its host-side grouping reproduces the reference's fixtures."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from helpers import golden
from mference_b200 import _lib as L
from mference_b200.moe import PAIR_DTYPE, PrefillMoEGroupingError, group_token_expert_pairs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(mfb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
    assert set(L.SIGNATURES) >= set(names), sorted(set(names) - set(L.SIGNATURES))


def test_struct_layouts():
    # MoEExpertOffsets is nine u32 (MoE.swift:4-15); PrefillTokenExpertPair is 16 bytes with the documented field
    # offsets (PrefillRouterTests.swift:12-19)
    assert C.sizeof(L.ExpertOffsets) == 36
    assert C.sizeof(L.Pair) == 16
    assert [getattr(L.Pair, n).offset for n in ("token", "expert", "rank", "weight_bits")] == [0, 4, 8, 12]
    assert C.sizeof(L.Group) == 12 and C.sizeof(L.Tile) == 16
    assert PAIR_DTYPE.itemsize == 16


def test_expert_layout_matches_reference_blob_size():
    lib = L.load()
    off, total = L.ExpertOffsets(), C.c_uint64()
    assert lib.mfb_expert_layout(4, 2048, 512, C.byref(off), C.byref(total)) == 0
    assert total.value == 1769472            # Qwen 3.6 expert blob (SupportedModelSource.swift:72-75)
    assert (off.gate_w, off.gate_s, off.gate_b, off.up_w) == (0, 524288, 557056, 589824)
    assert lib.mfb_expert_layout(2, 4096, 2048, C.byref(off), C.byref(total)) == 0
    assert total.value == 7864320
    assert lib.mfb_expert_layout(3, 64, 64, C.byref(off), C.byref(total)) == L.ERR_INVALID_ARGUMENT
    assert b"bits" in lib.mfb_last_error()


@pytest.mark.parametrize("case", golden("grouping_cases.json")["cases"], ids=lambda c: c["name"])
def test_host_grouping_golden(case):
    pairs = np.array([tuple(p) for p in case["pairs"]], dtype=PAIR_DTYPE)
    g = group_token_expert_pairs(pairs, case["query_count"], case["top_k"], case["num_experts"],
                                 case["tile_expert_count"], case["sort_keys"])
    sp = g["sorted_pairs"]
    if "sorted_experts" in case:
        assert sp["expert"].tolist() == case["sorted_experts"]
    if "sorted_token_rank" in case:
        assert [[int(t), int(r)] for t, r in zip(sp["token"], sp["rank"])] == case["sorted_token_rank"]
    if "sorted_weight_bits" in case:
        assert sp["weight_bits"].tolist() == case["sorted_weight_bits"]
    if "offsets" in case:
        assert g["per_expert_offsets"].tolist() == case["offsets"]
    if "counts" in case:
        assert g["per_expert_counts"].tolist() == case["counts"]
    if "groups" in case:
        assert [list(map(int, x)) for x in g["groups"].tolist()] == case["groups"]
    if "group_experts" in case:
        assert g["groups"]["expert"].tolist() == case["group_experts"]
    if "tiles" in case:
        assert [list(map(int, x)) for x in g["tiles"].tolist()] == case["tiles"]
    for key in ("max_pairs_per_expert", "max_pairs_per_tile", "max_live_experts_per_tile"):
        if key in case:
            assert g[key] == case[key]


@pytest.mark.parametrize("case", golden("grouping_cases.json")["errors"], ids=lambda c: c["case"])
def test_host_grouping_errors(case):
    pairs = np.array([tuple(p) for p in case["pairs"]], dtype=PAIR_DTYPE)
    with pytest.raises(PrefillMoEGroupingError) as ei:
        group_token_expert_pairs(pairs, case["query_count"], case["top_k"], case["num_experts"],
                                 case["tile_expert_count"], case["sort_keys"])
    assert ei.value.case == case["case"] and ei.value.a == case["a"] and ei.value.b == case.get("b", 0)


def test_host_grouping_matches_oracle_on_random_tables():
    from oracle import oracle as O
    rng = np.random.default_rng(5)
    for T, K, E, tile in [(1, 8, 256, 16), (37, 6, 64, 8), (300, 8, 256, 16), (0, 2, 4, 1)]:
        experts = np.array([rng.choice(E, K, replace=False) for _ in range(T)], dtype=np.uint32).reshape(T, K)
        pairs = np.array([(t, experts[t, r], r, 1000 + t * K + r) for t in range(T) for r in range(K)], dtype=PAIR_DTYPE)
        pairs = pairs[rng.permutation(pairs.size)] if pairs.size else pairs
        keys = rng.integers(0, 1 << 40, E).astype(np.uint64)
        for sk in (None, keys):
            a = group_token_expert_pairs(pairs, T, K, E, tile, sk)
            b = O.group_pairs(pairs.astype(O.PAIR_DTYPE), T, K, E, tile, sk)
            assert (a["sorted_pairs"] == b["sorted_pairs"].astype(PAIR_DTYPE)).all()
            assert (a["per_expert_offsets"] == b["offsets"]).all() and (a["per_expert_counts"] == b["counts"]).all()
            assert a["groups"].tolist() == b["groups"].tolist() and a["tiles"].tolist() == b["tiles"].tolist()


def test_no_device_means_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    cfg = L.MoEConfig(2048, 512, 256, 8, 4, 4, 64, L.DT_F16, L.DT_BF16, 0, 0, 0.0, 1.0, 1e-6, 1, 0)
    h = C.c_void_p()
    rc = L.load().mfb_moe_create(C.byref(cfg), C.byref(h))
    assert rc == L.ERR_CUDA and not h.value
    assert b"CUDA" in L.load().mfb_last_error()


def test_create_rejects_bad_shapes_before_touching_the_device():
    lib = L.load()
    h = C.c_void_p()
    bad = [dict(d=100), dict(bits=3), dict(num_experts=0), dict(num_experts=513), dict(top_k=17), dict(group_size=32),
           dict(x_dtype=L.DT_F32), dict(max_tokens=0), dict(d=192)]
    base = dict(d=2048, f=512, num_experts=256, top_k=8, bits=4, shared_bits=4, group_size=64, scale_dtype=L.DT_F16,
                x_dtype=L.DT_BF16, activation=0, router_mode=0, swiglu_limit=0.0, route_scale=1.0, rms_eps=1e-6,
                max_tokens=1, flags=0)
    for b in bad:
        kw = dict(base); kw.update(b)
        cfg = L.MoEConfig(**kw)
        rc = lib.mfb_moe_create(C.byref(cfg), C.byref(h))
        assert rc in (L.ERR_INVALID_ARGUMENT, L.ERR_UNSUPPORTED_SHAPE), (b, rc)
        assert not h.value

"""CPU tests of the oracle itself: known-answer vectors for the PRNG, the structural fixtures the reference's
own tests pin (nibble order, constant groups, grouping order, tie-breaks), and self-consistency of its two
arithmetic flavours."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import golden, make_x
from router_fixtures import EXPERT_COUNTS, ROUTE_SCALE, k6_inputs, k8_inputs


def test_splitmix64_known_answers():
    # published SplitMix64 test vector for seed 0
    assert [O.splitmix_at(0, i) for i in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    # sequential == counter form
    seed = 0x1234567
    raw = O.fill_raw(seed, 64)
    assert all(int(raw[i]) == O.splitmix_at(seed, i) for i in range(64))


def test_seedtree_fnv1a_known_answers():
    # FNV-1a 64 reference values
    assert O.seed_for_label(0, "") == 0xCBF29CE484222325
    assert O.seed_for_label(0, "a") == 0xAF63DC4C8601EC8C
    assert O.seed_for_label(0, "foobar") == 0x85944171F73967E8
    assert O.seed_for_label(0xFF, "a") == 0xAF63DC4C8601EC8C ^ 0xFF


def test_uniform_is_24_bit():
    for i in range(100):
        u = O.uniform_at(7, i, 0.0, 1.0)
        assert 0.0 <= u < 1.0 and float(u) * (1 << 24) == int(float(u) * (1 << 24))


def test_normal_moments_and_dtypes():
    z = O.fill_normal(O.seed_for_label(1, "x"), 200000, dtype=O.DT_F32)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    s = O.f16_to_f32(O.fill_normal(3, 50000, std=0.02, absolute=True, dtype=O.DT_F16))
    assert (s >= 0).all() and abs(s.mean() - 0.02 * np.sqrt(2 / np.pi)) < 5e-4
    # value i does not depend on where the fill starts
    a = O.fill_normal(9, 100, dtype=O.DT_BF16)
    b = O.fill_normal(9, 40, dtype=O.DT_BF16, first=60)
    assert (a[60:] == b).all()


def test_bf16_round_half_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38], dtype=np.float32)
    assert (O.f32_to_bf16(x) == np.array([O.lib().mfbo_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)).all()
    assert O.lib().mfbo_f32_to_bf16(1.00390625) == 0x3F80   # tie -> even
    assert O.lib().mfbo_f32_to_bf16(1.01171875) == 0x3F82   # tie -> even (up)


def test_int4_nibble_layout_low_even_high_odd():
    # QuantizationTests.nibbleLayoutIsLowEvenHighOdd
    row = np.arange(64, dtype=np.float32) - 31.5
    packed, s, b = O.quantize_int4_row(row)
    scale, bias = O.bf16_to_f32(s)[0], O.bf16_to_f32(b)[0]
    lo, hi = packed[0] & 0xF, packed[0] >> 4
    assert abs(lo * scale + bias - row[0]) <= scale + 1e-3
    assert abs(hi * scale + bias - row[1]) <= scale + 1e-3
    deq = O.dequant_rows(packed, s, b, 4, 1, 64, scale_dtype=O.DT_BF16)[0]
    assert abs(deq[0] - (lo * scale + bias)) < 1e-6 and abs(deq[1] - (hi * scale + bias)) < 1e-6


def test_int4_constant_group_roundtrips():
    # QuantizationAffineTests.quantizeInt4Affine_constantGroupRoundtripsExact
    row = np.full(64, 0.42, dtype=np.float32)
    packed, s, b = O.quantize_int4_row(row)
    deq = O.dequant_rows(packed, s, b, 4, 1, 64, scale_dtype=O.DT_BF16)[0]
    ref = O.bf16_to_f32(O.f32_to_bf16(np.array([0.42], dtype=np.float32)))[0]
    assert np.abs(deq - ref).max() < 1e-6


def test_int4_roundtrip_error_bounded_by_scale():
    # DequantInt4GEMVReferenceTests: |w - deq| <= scale + 1e-4 per group
    rng = np.random.default_rng(0)
    row = rng.normal(0, 0.05, 256).astype(np.float32)
    packed, s, b = O.quantize_int4_row(row)
    deq = O.dequant_rows(packed, s, b, 4, 1, 256, scale_dtype=O.DT_BF16)[0]
    scale = np.repeat(O.bf16_to_f32(s), 64)
    assert (np.abs(deq - row) <= scale + 1e-4).all()


def test_int2_element_order():
    # moe.metal:948-950: byte k holds elements 4k..4k+3, element j at bit 2*(j%4)
    codes = np.array([0b11100100] * 16, dtype=np.uint8)      # elements 0,1,2,3 -> 0,1,2,3
    s = O.f32_to_f16(np.array([1.0], dtype=np.float32))
    b = O.f32_to_f16(np.array([0.0], dtype=np.float32))
    deq = O.dequant_rows(codes, s, b, 2, 1, 64)[0]
    assert (deq == np.tile(np.array([0, 1, 2, 3], dtype=np.float32), 16)).all()


@pytest.mark.parametrize("case", golden("grouping_cases.json")["cases"], ids=lambda c: c["name"])
def test_grouping_golden(case):
    pairs = np.array([tuple(p) for p in case["pairs"]], dtype=O.PAIR_DTYPE)
    g = O.group_pairs(pairs, case["query_count"], case["top_k"], case["num_experts"], case["tile_expert_count"],
                      case["sort_keys"])
    sp = g["sorted_pairs"]
    if "sorted_experts" in case:
        assert sp["expert"].tolist() == case["sorted_experts"]
    if "sorted_token_rank" in case:
        assert [[int(t), int(r)] for t, r in zip(sp["token"], sp["rank"])] == case["sorted_token_rank"]
    if "sorted_weight_bits" in case:
        assert sp["weight_bits"].tolist() == case["sorted_weight_bits"]
    if "offsets" in case:
        assert g["offsets"].tolist() == case["offsets"]
    if "counts" in case:
        assert g["counts"].tolist() == case["counts"]
    if "groups" in case:
        assert [list(map(int, x)) for x in g["groups"].tolist()] == case["groups"]
    if "group_experts" in case:
        assert g["groups"]["expert"].tolist() == case["group_experts"]
    if "tiles" in case:
        assert [list(map(int, x)) for x in g["tiles"].tolist()] == case["tiles"]


@pytest.mark.parametrize("case", golden("grouping_cases.json")["errors"], ids=lambda c: c["case"])
def test_grouping_errors(case):
    pairs = np.array([tuple(p) for p in case["pairs"]], dtype=O.PAIR_DTYPE)
    with pytest.raises(O.GroupingError) as ei:
        O.group_pairs(pairs, case["query_count"], case["top_k"], case["num_experts"], case["tile_expert_count"],
                      case["sort_keys"])
    assert ei.value.case == case["case"] and ei.value.a == case["a"] and ei.value.b == case.get("b", 0)


def test_grouping_trace_pressure_t32():
    # PrefillMoEGroupingTests.groupingToleratesRealTracePairPressureAtT32
    pairs = np.array([(t, (t + r * 7) % 74, r, t * 8 + r) for t in range(32) for r in range(8)], dtype=O.PAIR_DTYPE)
    g = O.group_pairs(pairs, 32, 8, 128, 16)
    assert g["sorted_pairs"].size == 256 and g["groups"].size <= 74
    assert (g["tiles"]["group_count"] <= 16).all() and (g["tiles"]["pair_count"] > 0).all()


def test_topk_selectors_match_golden():
    cases = {(c["mode"], c["num_experts"], c["trial"]): c for c in golden("router_topk_cases.json")["cases"]}
    for ne in EXPERT_COUNTS:
        for trial, lg, scale in k8_inputs(ne):
            idx, w = O.topk_softmax(lg[None, :], 8, O.f32_to_bf16(scale))
            c = cases[("softmax_k8", ne, trial)]
            assert idx[0].tolist() == c["indices"], (ne, trial)
            assert np.abs(O.f16_to_f32(w[0]) - np.array(c["weights"])).max() < 1e-3
        for trial, lg, bias in k6_inputs(ne):
            idx, w = O.topk_sqrtsoftplus(lg[None, :], 6, bias, ROUTE_SCALE)
            c = cases[("sqrtsoftplus_k6", ne, trial)]
            assert idx[0].tolist() == c["indices"], (ne, trial)
            assert np.abs(O.f16_to_f32(w[0]) - np.array(c["weights"])).max() < 2e-3


def test_topk_fewer_experts_than_k_leaves_index_zero():
    idx, w = O.topk_softmax(np.array([[0.5, 1.5, 1.0]], dtype=np.float32), 8)
    assert idx[0].tolist() == [1, 2, 0, 0, 0, 0, 0, 0]
    assert O.f16_to_f32(w[0])[3:].max() == 0.0


def test_router_logits_fixed_order_close_to_exact():
    W = O.LayerWeights(256, 64, 40, 4, experts=[])
    x = make_x("x", 5, 256)
    a = O.router_logits(x, O.DT_BF16, W.router)
    b = O.router_logits(x, O.DT_BF16, W.router, exact_f64=True)
    assert np.abs(a - b).max() < 1e-5
    bias = np.linspace(-1, 1, 40).astype(np.float32)
    c = O.router_logits(x, O.DT_BF16, W.router, logit_bias=bias)
    assert (c == a + bias[None, :]).all()


@pytest.mark.parametrize("bits", [4, 2])
def test_fp32_scalar_path_agrees_with_double_oracle(bits):
    # the timed CPU baseline (reference-style factored fp32) against the grading oracle (double accumulation)
    W = O.LayerWeights(256, 128, 12, 3, bits=bits, shared_bits=4)
    x = make_x("x", 4, 256)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, 3)
    res = O.bf16_to_f32(make_x("res", 4, 256))
    y = O.moe_layer(W, x, O.DT_BF16, idx, w, res)
    y2 = O.ref_moe_layer_f32(W, O.bf16_to_f32(x), idx, w, res)
    assert O.rel_l2(y2, y) < 1e-4


def test_pair_partials_and_reduce_equal_layer():
    W = O.LayerWeights(128, 64, 6, 2, shared=False)
    x = make_x("x", 5, 128)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, 2)
    pairs = np.array([(t, idx[t, r], r, w[t, r]) for t in range(5) for r in range(2)], dtype=O.PAIR_DTYPE)
    g = O.group_pairs(pairs, 5, 2, 6)
    part_sorted = O.pair_partials(W, x, O.DT_BF16, g["sorted_pairs"])
    part = np.zeros((5, 2, 128), dtype=np.float32)
    for p, row in zip(g["sorted_pairs"], part_sorted):
        part[p["token"], p["rank"]] = row
    h2 = O.reduce_token_major(part, w, 5, 2, 128)
    y = O.moe_layer(W, x, O.DT_BF16, idx, w)
    assert O.rel_l2(h2, y) < 1e-6


def test_gate_group_32_layout_and_dequant():
    # DeepSeek V4's gate_proj: one scale and bias per 32 elements (routedGateGroupSize, ModelExpertIO.swift:118-135); only
    # the gate's scale and bias arrays grow, the codes and the other two matrices keep their sizes
    d, f = 128, 64
    o64, b64 = O.make_offsets(2, d, f, 64)
    o32, b32 = O.make_offsets(2, d, f, 32)
    assert o32.gate_w == o64.gate_w and o32.gate_s == o64.gate_s
    assert o32.gate_b - o32.gate_s == 2 * (o64.gate_b - o64.gate_s)
    assert b32 - b64 == 2 * (d * f // 64 * 2)
    blob = O.synth_expert(0xB2000001, 0, 3, 2, O.DT_BF16, d, f, 32)
    codes = blob[o32.gate_w:o32.gate_s]
    sc = blob[o32.gate_s:o32.gate_b].view(np.uint16)
    bi = blob[o32.gate_b:o32.up_w].view(np.uint16)
    w32 = O.dequant_rows(codes, sc, bi, 2, f, d, scale_dtype=O.DT_BF16, group_size=32)
    # element (r, c) = code * scale[r, c // 32] + bias[r, c // 32], 2-bit codes LSB first
    r, c = 5, 77
    byte = codes[r * d // 4 + c // 4]
    q = (int(byte) >> (2 * (c % 4))) & 3
    g = r * (d // 32) + c // 32
    want = np.float32(np.float32(q) * O.bf16_to_f32(sc[g:g + 1])[0]) + O.bf16_to_f32(bi[g:g + 1])[0]
    assert w32[r, c] == np.float32(want)
    # the layer function reads a pool of such blobs with the gate group taken from the layer
    W = O.LayerWeights(d, f, 6, 2, bits=2, shared_bits=4, scale_dtype=O.DT_BF16, gate_group_size=32)
    x = make_x("x.g32", 3, d)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, 2)
    y = O.moe_layer(W, x, O.DT_BF16, idx, w)
    assert np.isfinite(y).all() and y.shape == (3, d)


def test_int8_shared_expert_rows_are_plain_bytes():
    # SharedExpertInt8: unsigned byte codes, one scale and bias per 64 elements
    d, f = 128, 64
    off, total = O.make_offsets(8, d, f)
    assert off.gate_s - off.gate_w == d * f
    blob = O.synth_expert(0xB2000001, 0, -1, 8, O.DT_BF16, d, f)
    codes = blob[off.down_w:off.down_s]
    sc = blob[off.down_s:off.down_b].view(np.uint16)
    bi = blob[off.down_b:total].view(np.uint16)
    w8 = O.dequant_rows(codes, sc, bi, 8, d, f, scale_dtype=O.DT_BF16)
    r, c = 17, 33
    g = r * (f // 64) + c // 64
    want = np.float32(np.float32(codes[r * f + c]) * O.bf16_to_f32(sc[g:g + 1])[0]) + O.bf16_to_f32(bi[g:g + 1])[0]
    assert w8[r, c] == np.float32(want)


def test_inkling_accumulate_is_expert_ordered():
    # inkling_prefill_expert_down_accum: experts in ascending order, fp32 accumulator and weights; with weights whose
    # ranks are not in expert order the result differs from the rank-ordered reduce only by rounding
    W = O.LayerWeights(128, 64, 6, 3, shared=False)
    x = make_x("x.ink", 4, 128)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, 3)
    w32 = O.f16_to_f32(w).reshape(4, 3).astype(np.float32)
    acc = O.inkling_accumulate(W, x, O.DT_BF16, idx.reshape(4, 3), w32)
    y = O.moe_layer(W, x, O.DT_BF16, idx, w)          # rank order, no residual, no shared expert
    assert O.rel_l2(acc, y) < 1e-5
    acc2 = O.inkling_accumulate(W, x, O.DT_BF16, idx.reshape(4, 3), w32, acc0=np.ones((4, 128), dtype=np.float32))
    assert np.abs((acc2 - acc) - 1.0).max() < 1e-3


def test_rmsnorm_definition():
    x = O.bf16_to_f32(make_x("h", 3, 128))
    out = O.rmsnorm(x, None, 1e-6)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-6)
    assert np.abs(out - ref).max() < 1e-6

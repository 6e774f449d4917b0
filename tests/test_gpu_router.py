"""GPU parity tests of the router through the C ABI: logits bit for bit against the oracle's fixed-order fp32
definition, selections exact (ties to the lower index), routing weights within 1e-3."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import TOL_ROUTE_WEIGHT, golden, make_x, to_dev16
from router_fixtures import EXPERT_COUNTS, ROUTE_SCALE, k6_inputs, k8_inputs

pytestmark = pytest.mark.gpu


def _moe(**kw):
    from mference_b200.moe import MoE
    base = dict(d=256, f=64, num_experts=16, top_k=4, max_tokens=64)
    base.update(kw)
    return MoE(**base)


@pytest.mark.parametrize("T,E,D", [(1, 256, 2048), (2, 256, 2048), (8, 256, 2048), (64, 256, 2048), (300, 256, 2048),
                                   (5, 40, 256), (3, 33, 64), (17, 100, 4096),
                                   # above 64 rows: the lane-major fp32 kernel (d a multiple of 128; ragged row and expert
                                   # counts, fewer chunks than ring stages) and the self-contained tile kernel (d = 64)
                                   (130, 100, 1536), (1025, 256, 2048), (97, 33, 256), (70, 20, 64), (65, 1, 128)])
def test_logits_bit_exact(T, E, D):
    import torch
    W = O.LayerWeights(D, 64, E, 4, experts=[], shared=False)
    x = make_x(f"x.{T}.{E}.{D}", T, D)
    bias = np.linspace(-2, 2, E).astype(np.float32)
    moe = _moe(d=D, num_experts=E, max_tokens=T)
    xd = to_dev16(x, O.DT_BF16)
    wd = to_dev16(W.router, O.DT_BF16)
    out = torch.empty((T, E), dtype=torch.float32, device="cuda")
    for lb in (None, bias):
        moe.encode_router_logits(xd, wd, out, None if lb is None else torch.from_numpy(lb).cuda())
        ref = O.router_logits(x, O.DT_BF16, W.router, logit_bias=lb)
        got = out.cpu().numpy()
        assert (got.view(np.uint32) == ref.view(np.uint32)).all(), np.abs(got - ref).max()


def test_logits_fp16_activations_and_row_stride():
    import torch
    T, E, D = 6, 24, 128
    W = O.LayerWeights(D, 64, E, 4, experts=[], shared=False)
    x = make_x("x16", T, D, dtype=O.DT_F16)
    from mference_b200 import DT_F16
    moe = _moe(d=D, num_experts=E, max_tokens=T, x_dtype=DT_F16)
    wide = torch.zeros((T, D + 64), dtype=torch.float16, device="cuda")
    wide[:, :D] = to_dev16(x, O.DT_F16)
    out = torch.empty((T, E), dtype=torch.float32, device="cuda")
    moe.encode_router_logits(wide[:, :D], to_dev16(W.router, O.DT_BF16), out)
    ref = O.router_logits(x, O.DT_F16, W.router)
    assert (out.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()


def test_logits_many_rows_fp16_activations_and_row_stride():
    import torch
    T, E, D = 97, 48, 512
    W = O.LayerWeights(D, 64, E, 4, experts=[], shared=False)
    x = make_x("x16.many", T, D, dtype=O.DT_F16)
    from mference_b200 import DT_F16
    moe = _moe(d=D, num_experts=E, max_tokens=T, x_dtype=DT_F16)
    wide = torch.zeros((T, D + 72), dtype=torch.float16, device="cuda")
    wide[:, :D] = to_dev16(x, O.DT_F16)
    out = torch.empty((T, E), dtype=torch.float32, device="cuda")
    moe.encode_router_logits(wide[:, :D], to_dev16(W.router, O.DT_BF16), out)
    ref = O.router_logits(x, O.DT_F16, W.router)
    assert (out.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()


def test_block_of_rows_equals_single_rows_bit_for_bit():
    # PrefillRouterTests: the block router equals the repeated single-row router
    import torch
    T, E, D, K = 19, 256, 2048, 8
    W = O.LayerWeights(D, 64, E, K, experts=[], shared=False)
    x = to_dev16(make_x("xb", T, D), O.DT_BF16)
    wd = to_dev16(W.router, O.DT_BF16)
    moe = _moe(d=D, num_experts=E, top_k=K, max_tokens=T)
    block = torch.empty((T, E), dtype=torch.float32, device="cuda")
    moe.encode_router_logits(x, wd, block)
    single = torch.empty((T, E), dtype=torch.float32, device="cuda")
    for t in range(T):
        moe.encode_router_logits(x[t:t + 1], wd, single[t:t + 1])
    assert torch.equal(block.view(torch.int32), single.view(torch.int32))


def test_select_golden_tie_fixtures():
    import torch
    from mference_b200 import ROUTER_SQRTSOFTPLUS
    cases = {(c["mode"], c["num_experts"], c["trial"]): c for c in golden("router_topk_cases.json")["cases"]}
    for ne in EXPERT_COUNTS:
        moe8 = _moe(num_experts=ne, top_k=8, max_tokens=16)
        lgs, scales = zip(*[(lg, sc) for _, lg, sc in k8_inputs(ne)])
        idx = torch.empty((len(lgs), 8), dtype=torch.int32, device="cuda")
        w = torch.empty((len(lgs), 8), dtype=torch.float16, device="cuda")
        for trial, (lg, sc) in enumerate(zip(lgs, scales)):
            moe8.encode_router_select(torch.from_numpy(lg[None]).cuda(), idx[trial:trial + 1], w[trial:trial + 1],
                                      per_expert_scale=to_dev16(O.f32_to_bf16(sc), O.DT_BF16))
        for trial in range(len(lgs)):
            c = cases[("softmax_k8", ne, trial)]
            assert idx[trial].tolist() == c["indices"], (ne, trial)
            assert np.abs(w[trial].float().cpu().numpy() - np.array(c["weights"])).max() < TOL_ROUTE_WEIGHT
            oi, ow = O.topk_softmax(lgs[trial][None], 8, O.f32_to_bf16(scales[trial]))
            assert idx[trial].tolist() == oi[0].tolist()
        moe6 = _moe(num_experts=ne, top_k=6, max_tokens=16, router_mode=ROUTER_SQRTSOFTPLUS, route_scale=ROUTE_SCALE)
        for trial, lg, bias in k6_inputs(ne):
            i6 = torch.empty((1, 6), dtype=torch.int32, device="cuda")
            w6 = torch.empty((1, 6), dtype=torch.float16, device="cuda")
            moe6.encode_router_select(torch.from_numpy(lg[None]).cuda(), i6, w6, correction_bias=torch.from_numpy(bias).cuda())
            c = cases[("sqrtsoftplus_k6", ne, trial)]
            assert i6[0].tolist() == c["indices"], (ne, trial)
            assert np.abs(w6[0].float().cpu().numpy() - np.array(c["weights"])).max() < 2e-3


def test_select_fewer_experts_than_k():
    import torch
    moe = _moe(num_experts=3, top_k=8, max_tokens=1)
    lg = torch.tensor([[0.5, 1.5, 1.0]], dtype=torch.float32, device="cuda")
    idx = torch.empty((1, 8), dtype=torch.int32, device="cuda")
    w = torch.empty((1, 8), dtype=torch.float16, device="cuda")
    moe.encode_router_select(lg, idx, w)
    assert idx[0].tolist() == [1, 2, 0, 0, 0, 0, 0, 0]
    assert float(w[0, 3:].float().abs().max()) == 0.0


@pytest.mark.parametrize("T", [1, 8, 64, 4096])
def test_router_topk_exact_at_qwen_shape(T):
    import torch
    E, D, K = 256, 2048, 8
    W = O.LayerWeights(D, 64, E, K, experts=[], shared=False)
    x = make_x(f"xq{T}", T, D)
    from mference_b200.moe import MoELayerWeights, expert_layout
    moe = _moe(d=D, f=512, num_experts=E, top_k=K, max_tokens=T)
    off, _ = expert_layout(4, D, 512)
    lw = MoELayerWeights(router_w=to_dev16(W.router, O.DT_BF16), pool=torch.zeros(16, dtype=torch.uint8, device="cuda"),
                         slot_stride=16, routed_off=off)
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float16, device="cuda")
    moe.encode_router(to_dev16(x, O.DT_BF16), lw, idx, w)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    oi, ow = O.topk_softmax(lg, K)
    assert (idx.cpu().numpy().astype(np.uint32) == oi).all()
    assert np.abs(w.float().cpu().numpy() - O.f16_to_f32(ow)).max() < TOL_ROUTE_WEIGHT
    # the fixed summation order does not hide a wrong answer: wherever the exact (double) logits separate the
    # candidates by more than fp32 noise, the selection is the same
    lg64 = O.router_logits(x, O.DT_BF16, W.router, exact_f64=True)
    clear = O.topk_margin(lg64, K) > 1e-4
    oi64, _ = O.topk_softmax(lg64, K)
    assert (idx.cpu().numpy().astype(np.uint32)[clear] == oi64[clear]).all()
    assert clear.mean() > 0.95


def test_slot_lookup():
    import torch
    moe = _moe(num_experts=16, top_k=4, max_tokens=8)
    table = torch.full((16,), -1, dtype=torch.int16, device="cuda")
    table[3], table[5], table[7], table[9] = 0, 2, 1, 3
    idx = torch.tensor([[3, 5, 7, 9], [3, 4, 7, 9], [99, 3, 5, 7]], dtype=torch.int32, device="cuda")
    offs = torch.empty((3, 4), dtype=torch.int64, device="cuda")
    hit = torch.empty(3, dtype=torch.int32, device="cuda")
    moe.encode_slot_lookup(idx, table, 1000, offs, hit)
    assert hit.tolist() == [1, 0, 0]        # row 2: index clamped to the last expert, which is not resident
    assert offs[0].tolist() == [0, 2000, 1000, 3000] and offs[1].tolist() == [0, 0, 1000, 3000]

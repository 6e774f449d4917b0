"""The allocation-free router entry point (mfb_router_topk_static) against mfb_router_topk, through the C ABI.

Collected last (file name) so that it also runs after every other GPU test has used the library; it passes alone
as well.  Two calls in a row check that nothing left in the fixed scratch by one call leaks into the next."""
import ctypes as C

import pytest
import torch

from mference_b200 import _lib as L
from mference_b200.moe import MoE, encode_router_static, synth_layer, synth_normal

pytestmark = pytest.mark.gpu

ROOT = 0xB2000001


def _route_with_handle(moe, x, layer):
    idx = torch.empty((x.shape[0], moe.cfg.top_k), dtype=torch.int32, device="cuda")
    w = torch.empty((x.shape[0], moe.cfg.top_k), dtype=torch.float16, device="cuda")
    moe.encode_router(x, layer, idx, w)
    return idx, w


@pytest.mark.parametrize("d,num_experts,top_k", [(2048, 256, 8), (512, 64, 6)])
def test_static_router_matches_handle_router_twice(d, num_experts, top_k):
    layer = synth_layer(ROOT, 0, d, 256, num_experts)
    moe = MoE(d, 256, num_experts, top_k, max_tokens=64)
    # first call: 64 rows fill the whole scratch; second call: 5 different rows must not see leftovers
    for call, rows in enumerate((64, 5)):
        x = synth_normal(ROOT, f"x.static.{call}", rows * d, dtype=L.DT_BF16).view(rows, d)
        ref_idx, ref_w = _route_with_handle(moe, x, layer)
        idx = torch.full((rows, top_k), -1, dtype=torch.int32, device="cuda")
        w = torch.zeros((rows, top_k), dtype=torch.float16, device="cuda")
        before = torch.cuda.memory_allocated()
        encode_router_static(x, layer.router_w, idx, w, top_k=top_k)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx)
        assert torch.equal(w.view(torch.int16), ref_w.view(torch.int16))
        # and directly against the CPU oracle: same experts in the same rank order
        import numpy as np
        from oracle import oracle as O
        x_bits = x.view(torch.int16).cpu().numpy().view(np.uint16)
        rw_bits = layer.router_w.view(torch.int16).cpu().numpy().view(np.uint16)
        o_idx, o_w = O.topk_softmax(O.router_logits(x_bits, O.DT_BF16, rw_bits), top_k)
        assert np.array_equal(idx.cpu().numpy().view(np.uint32), o_idx)
        got_w = w.float().cpu().numpy()
        assert np.abs(got_w - O.f16_to_f32(o_w)).max() <= 1e-3


def test_static_router_rejects_more_rows_than_the_scratch_holds():
    d, num_experts, top_k = 512, 64, 6
    layer = synth_layer(ROOT, 0, d, 256, num_experts)
    x = synth_normal(ROOT, "x.static.big", 65 * d, dtype=L.DT_BF16).view(65, d)
    idx = torch.empty((65, top_k), dtype=torch.int32, device="cuda")
    w = torch.empty((65, top_k), dtype=torch.float16, device="cuda")
    with pytest.raises(L.MfbError) as err:
        encode_router_static(x, layer.router_w, idx, w, top_k=top_k)
    assert err.value.code == L.ERR_CAPACITY
    assert "64" in str(err.value)

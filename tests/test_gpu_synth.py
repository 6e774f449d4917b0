"""The device-side generator of synthetic weights produces the same bytes as the oracle's host generator."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import ROOT_SEED

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,scale_dtype,d,f", [(4, O.DT_F16, 256, 128), (2, O.DT_BF16, 128, 256), (4, O.DT_F16, 2048, 512)])
def test_device_layer_equals_host_layer(bits, scale_dtype, d, f):
    from mference_b200.moe import synth_layer
    E = 5
    lw = synth_layer(ROOT_SEED, 3, d, f, E, bits=bits, shared_bits=4, scale_dtype=scale_dtype)
    W = O.LayerWeights(d, f, E, 2, bits=bits, shared_bits=4, scale_dtype=scale_dtype, root=ROOT_SEED, layer=3)
    assert lw.slot_stride == W.expert_stride
    pool = lw.pool.cpu().numpy()
    for e in range(E):
        a = pool[e * W.expert_stride: e * W.expert_stride + W.blob_bytes]
        b = W.pool[e * W.expert_stride: e * W.expert_stride + W.blob_bytes]
        assert (a == b).all(), (e, int((a != b).sum()))
    assert (lw.shared_blob.cpu().numpy() == W.shared_blob).all()
    import torch
    assert (lw.router_w.view(torch.int16).cpu().numpy().view(np.uint16) == W.router).all()


def test_device_normal_equals_host_normal():
    from mference_b200.moe import synth_normal
    from mference_b200 import DT_BF16, DT_F32
    import torch
    a = synth_normal(ROOT_SEED, "x", 10000, dtype=DT_BF16).view(torch.int16).cpu().numpy().view(np.uint16)
    b = O.fill_normal(O.seed_for_label(ROOT_SEED, "x"), 10000, dtype=O.DT_BF16)
    assert (a == b).all()
    c = synth_normal(ROOT_SEED, "y", 1000, mean=0.5, std=2.0, absolute=True, dtype=DT_F32).cpu().numpy()
    d = O.fill_normal(O.seed_for_label(ROOT_SEED, "y"), 1000, mean=0.5, std=2.0, absolute=True, dtype=O.DT_F32)
    assert np.abs(c - d).max() <= 1e-6

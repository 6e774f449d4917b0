"""Shared test helpers: seeded layers built on the host by the oracle's generator and uploaded to the GPU."""
import json
import os

import numpy as np

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROOT_SEED = 0xB2000001
TOL_REL_L2 = 2e-3          # north-star bar: relative L2 against the fp32-dequantised oracle
TOL_ROUTE_WEIGHT = 1e-3    # absolute, routing weights (fp16)


def golden(name):
    with open(os.path.join(GOLDEN, name)) as fh:
        return json.load(fh)


def make_x(label, n_tokens, d, dtype=O.DT_BF16, root=ROOT_SEED, std=1.0):
    return O.fill_normal(O.seed_for_label(root, label), n_tokens * d, std=std, dtype=dtype).reshape(n_tokens, d)


def upload_layer(W: "O.LayerWeights", device="cuda", slot_of=None, norm=True):
    """Oracle-side host layer -> device MoELayerWeights (same bytes)."""
    import torch
    from mference_b200 import _lib as L
    from mference_b200.moe import MoELayerWeights

    def offs(o):
        r = L.ExpertOffsets()
        for n, _ in r._fields_:
            setattr(r, n, getattr(o, n))
        return r

    pool = torch.from_numpy(W.pool).to(device)
    shared = None if W.shared_blob is None else torch.from_numpy(W.shared_blob).to(device)
    router = torch.from_numpy(W.router.view(np.int16)).to(device).view(torch.bfloat16)
    return MoELayerWeights(
        router_w=router, pool=pool, slot_stride=W.expert_stride, routed_off=offs(W.routed_off), shared_blob=shared,
        shared_off=None if shared is None else offs(W.shared_off),
        norm_w=torch.ones(W.d, dtype=torch.bfloat16, device=device) if norm else None,
        slot_of=None if slot_of is None else torch.tensor(slot_of, dtype=torch.int16, device=device),
        gate_group_size=getattr(W, "gate_group_size", 64))


def to_dev16(bits: np.ndarray, dtype, device="cuda"):
    """uint16 bit patterns -> torch bf16/fp16 tensor on the device."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device)
    return t.view(torch.bfloat16 if dtype == O.DT_BF16 else torch.float16)


def from_dev16(t) -> np.ndarray:
    """torch bf16/fp16 tensor -> fp32 numpy."""
    return t.float().cpu().numpy()

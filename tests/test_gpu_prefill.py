"""GPU parity tests of the prefill / ragged-batch path: grouped routed FFN over sorted pairs and the
token-major weighted reduce."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import TOL_REL_L2, make_x, to_dev16, upload_layer

pytestmark = pytest.mark.gpu


def _grouped(W, x, idx, w, tensor_core):
    import torch
    from mference_b200.moe import MoE
    T = x.shape[0]
    moe = MoE(W.d, W.f, W.num_experts, W.top_k, bits=W.bits, shared_bits=0, max_tokens=T, tensor_core_prefill=tensor_core)
    lw = upload_layer(W)
    xd = to_dev16(x, O.DT_BF16)
    idxd = torch.from_numpy(idx.view(np.int32)).cuda()
    wd = torch.from_numpy(w.view(np.int16)).cuda().view(torch.float16)
    sp, offsets, counts, groups, n_groups = moe.encode_group(idxd, wd)
    partial = torch.full((T * W.top_k, W.d), float("nan"), dtype=torch.float32, device="cuda")
    moe.encode_prefill_grouped(lw, xd, sp, groups, n_groups, partial)
    y = torch.empty_like(xd)
    moe.encode_reduce_token_major(partial, wd, y)
    torch.cuda.synchronize()
    return partial.cpu().numpy(), y.float().cpu().numpy(), sp.cpu().numpy().view(np.uint32), moe


@pytest.mark.parametrize("d,f,E,K,bits,T", [(256, 128, 8, 2, 4, 40), (128, 64, 6, 3, 2, 33), (512, 256, 16, 4, 4, 96)])
def test_grouped_ffn_and_reduce_match_oracle(d, f, E, K, bits, T):
    W = O.LayerWeights(d, f, E, K, bits=bits, shared=False)
    x = make_x("x", T, d)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, K)
    partial, y, sp, _ = _grouped(W, x, idx, w, tensor_core=False)
    pairs = np.array([tuple(r) for r in sp], dtype=O.PAIR_DTYPE)
    ref_sorted = O.pair_partials(W, x, O.DT_BF16, pairs)
    ref = np.zeros((T * K, d), dtype=np.float32)
    ref[pairs["token"] * K + pairs["rank"]] = ref_sorted
    assert np.isfinite(partial).all()
    assert O.rel_l2(partial, ref) <= TOL_REL_L2
    h2 = O.reduce_token_major(ref.reshape(T, K, d), w, T, K, d)
    assert O.rel_l2(y, h2) <= TOL_REL_L2

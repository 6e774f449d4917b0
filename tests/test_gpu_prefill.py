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


@pytest.mark.parametrize("d,f,E,K,bits,T", [(256, 128, 8, 2, 4, 40), (512, 256, 16, 4, 2, 33)])
def test_expert_order_fp32_accumulate_matches_oracle(d, f, E, K, bits, T):
    # the Inkling batched expert application: fp32 accumulator, fp32 pair weights, experts in ascending order
    import torch
    from mference_b200.moe import MoE
    W = O.LayerWeights(d, f, E, K, bits=bits, shared=False)
    x = make_x("x.ink", T, d)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, K)
    w32 = (O.f16_to_f32(w).reshape(T, K) * np.float32(1.5)).astype(np.float32)    # fp32 weights the fp16 path could not hold exactly
    acc0 = np.linspace(-1.0, 1.0, T * d, dtype=np.float32).reshape(T, d)          # e.g. the shared expert's contribution
    moe = MoE(d, f, E, K, bits=bits, shared_bits=0, max_tokens=T)
    lw = upload_layer(W)
    xd = to_dev16(x, O.DT_BF16)
    idxd = torch.from_numpy(idx.view(np.int32)).cuda()
    wd = torch.from_numpy(w.view(np.int16)).cuda().view(torch.float16)
    sp, _, _, groups, n_groups = moe.encode_group(idxd, wd)
    acc = torch.from_numpy(acc0.copy()).cuda()
    moe.encode_prefill_accumulate_f32(lw, xd, sp, groups, n_groups, torch.from_numpy(w32).cuda(), acc)
    torch.cuda.synchronize()
    ref = O.inkling_accumulate(W, x, O.DT_BF16, idx.reshape(T, K), w32, acc0)
    got = acc.cpu().numpy()
    assert np.isfinite(got).all()
    assert O.rel_l2(got, ref) <= TOL_REL_L2, O.rel_l2(got, ref)
    assert O.rel_l2(got - acc0, ref - acc0) <= TOL_REL_L2


# ---- tensor-core (tcgen05 / TMEM) grouped GEMM ---------------------------------------------------------------
# d and f multiples of 512; token counts chosen to give groups below 16 rows, around a TMA box, and above one
# 256-row MMA tile (several passes per expert).
TC_CASES = [(512, 512, 8, 2, 40, 4), (1024, 512, 16, 4, 300, 4), (512, 512, 4, 2, 700, 4), (2048, 512, 16, 8, 128, 4),
            (512, 512, 8, 2, 150, 2), (1024, 1024, 8, 3, 90, 2)]


@pytest.mark.parametrize("d,f,E,K,T,bits", TC_CASES)
def test_tensor_core_grouped_ffn_matches_oracle(d, f, E, K, T, bits):
    W = O.LayerWeights(d, f, E, K, bits=bits, shared=False)
    x = make_x("x.tc", T, d)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, K)
    partial, y, sp, moe = _grouped(W, x, idx, w, tensor_core=True)
    assert moe.device_status() == 0
    pairs = np.array([tuple(r) for r in sp], dtype=O.PAIR_DTYPE)
    ref_sorted = O.pair_partials(W, x, O.DT_BF16, pairs)
    ref = np.zeros((T * K, d), dtype=np.float32)
    ref[pairs["token"] * K + pairs["rank"]] = ref_sorted
    assert np.isfinite(partial).all()
    assert O.rel_l2(partial, ref) <= TOL_REL_L2
    # per pair row as well: a wrong tile would hide in the aggregate
    rows = pairs["token"] * K + pairs["rank"]
    err = np.linalg.norm(partial[rows] - ref[rows], axis=1) / np.maximum(np.linalg.norm(ref[rows], axis=1), 1e-20)
    assert err.max() <= 2 * TOL_REL_L2
    h2 = O.reduce_token_major(ref.reshape(T, K, d), w, T, K, d)
    assert O.rel_l2(y, h2) <= TOL_REL_L2


def test_tensor_core_matches_generic_kernels():
    d, f, E, K, T = 1024, 512, 16, 4, 200
    W = O.LayerWeights(d, f, E, K, bits=4, shared=False)
    x = make_x("x.tc2", T, d)
    lg = O.router_logits(x, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, K)
    p_tc, y_tc, _, _ = _grouped(W, x, idx, w, tensor_core=True)
    p_gen, y_gen, _, _ = _grouped(W, x, idx, w, tensor_core=False)
    assert O.rel_l2(p_tc, p_gen) <= TOL_REL_L2


def test_tensor_core_prefill_layer_with_2bit_experts_and_4bit_shared_expert():
    """The V-shape combination (2-bit routed experts, 4-bit shared expert) through the whole prefill layer."""
    import torch
    from mference_b200.moe import MoE
    d, f, E, K, T = 512, 512, 8, 3, 140
    W = O.LayerWeights(d, f, E, K, bits=2, shared=True, shared_bits=4)
    lw = upload_layer(W)
    x = to_dev16(make_x("x.tc4", T, d), O.DT_BF16)
    moe_tc = MoE(d, f, E, K, bits=2, shared_bits=4, max_tokens=T, tensor_core_prefill=True)
    moe_ref = MoE(d, f, E, K, bits=2, shared_bits=4, max_tokens=T)
    moe_ref.set_generic(True)
    y_tc, y_ref = torch.empty_like(x), torch.empty_like(x)
    moe_tc.encode_layer_prefill(lw, x, y_tc)
    moe_ref.encode_layer(lw, x, y_ref)
    torch.cuda.synchronize()
    assert moe_tc.device_status() == 0
    assert O.rel_l2(y_tc.float().cpu().numpy(), y_ref.float().cpu().numpy()) <= TOL_REL_L2


def test_tensor_core_prefill_layer_matches_decode_layer():
    """The whole prefill layer (RMSNorm, router, sort, grouped GEMM incl. the shared expert, reduce + residual) on the
    tensor-core path against the decode-path layer on the same rows."""
    import torch
    from mference_b200.moe import MoE
    d, f, E, K, T = 1024, 512, 16, 4, 150
    W = O.LayerWeights(d, f, E, K, bits=4, shared=True)
    lw = upload_layer(W)
    x = to_dev16(make_x("x.tc3", T, d), O.DT_BF16)
    moe_tc = MoE(d, f, E, K, max_tokens=T, tensor_core_prefill=True)
    moe_ref = MoE(d, f, E, K, max_tokens=T)
    y_tc, y_ref = torch.empty_like(x), torch.empty_like(x)
    moe_tc.encode_layer_prefill(lw, x, y_tc)
    moe_ref.encode_layer(lw, x, y_ref)
    torch.cuda.synchronize()
    assert moe_tc.device_status() == 0
    assert O.rel_l2(y_tc.float().cpu().numpy(), y_ref.float().cpu().numpy()) <= TOL_REL_L2


# ---- full-size configurations, through properties that need no CPU evaluation --------------------------------

def _prefill_layer(d, f, E, K, T, bits, shared_bits, tensor_core, x, layer, generic=False):
    import torch
    from mference_b200.moe import MoE
    moe = MoE(d, f, E, K, bits=bits, shared_bits=shared_bits, max_tokens=T, tensor_core_prefill=tensor_core)
    if generic:
        moe.set_generic(True)
    y = torch.empty_like(x)
    (moe.encode_layer_prefill if tensor_core else moe.encode_layer)(layer, x, y)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    return y


@pytest.mark.parametrize("name,d,f,E,K,T,bits,shared_bits", [
    ("qwen-a3b prefill, 4096 tokens", 2048, 512, 256, 8, 4096, 4, 4),
    ("dsv4-flash shape, 2-bit experts + 4-bit shared, 2048 tokens", 4096, 2048, 256, 6, 2048, 2, 4),
])
def test_full_size_prefill_tensor_core_agrees_with_generic_kernels_and_is_row_independent(name, d, f, E, K, T, bits, shared_bits):
    """At the full sizes of the benchmark configurations: (1) the tensor-core layer agrees with the generic SIMT
    kernels on a sample of rows (those kernels are the ones checked against the oracle at small sizes); (2) a
    token's output does not depend on which other tokens share its batch: permuting the rows permutes the outputs
    bit for bit."""
    import torch
    from mference_b200 import _lib as L
    from mference_b200.moe import synth_layer, synth_normal
    layer = synth_layer(0xB2000001, 0, d, f, E, bits=bits, shared_bits=shared_bits)
    x = synth_normal(0xB2000001, "x.full", T * d, dtype=L.DT_BF16).view(T, d)
    y = _prefill_layer(d, f, E, K, T, bits, shared_bits, True, x, layer)
    assert bool(torch.isfinite(y.float()).all())
    sample = torch.arange(0, T, max(T // 64, 1), device="cuda")[:64]
    xs = x[sample].contiguous()
    y_gen = _prefill_layer(d, f, E, K, xs.shape[0], bits, shared_bits, False, xs, layer, generic=True)
    err = float((y[sample].float() - y_gen.float()).norm() / y_gen.float().norm())
    assert err <= TOL_REL_L2, (name, err)
    perm = torch.randperm(T, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
    y_perm = _prefill_layer(d, f, E, K, T, bits, shared_bits, True, x[perm].contiguous(), layer)
    assert torch.equal(y_perm, y[perm]), name


def test_ragged_continuous_batch_mix_full_size():
    """The ragged mix of the benchmark configurations at full size: 48 sequences, each one decode row and prefill
    chunks of 256, 512 and 1024 rows, packed into one batch of 86,064 rows (688,512 token-expert pairs).  The layer
    works row by row, so packing must not matter: segments of every kind run on their own give the same rows bit
    for bit, and a sample of rows agrees with the generic kernels."""
    import numpy as np
    import torch
    from mference_b200 import _lib as L
    from mference_b200.moe import synth_layer, synth_normal
    d, f, E, K = 2048, 512, 256, 8
    sizes = np.tile(np.asarray([1, 256, 512, 1024], dtype=np.int64), 48)
    offsets = np.concatenate([[0], np.cumsum(sizes)])
    T = int(offsets[-1])
    assert T == 86064
    layer = synth_layer(0xB2000001, 0, d, f, E)
    x = synth_normal(0xB2000001, "x.ragged", T * d, dtype=L.DT_BF16).view(T, d)
    y = _prefill_layer(d, f, E, K, T, 4, 4, True, x, layer)
    assert bool(torch.isfinite(y.float()).all())
    for seg in (0, 1, 2, 3, 4, len(sizes) - 1):          # a decode row, one chunk of each length, the next decode row, the last chunk
        a, b = int(offsets[seg]), int(offsets[seg + 1])
        y_seg = _prefill_layer(d, f, E, K, b - a, 4, 4, True, x[a:b].contiguous(), layer)
        assert torch.equal(y_seg, y[a:b]), (seg, a, b)
    sample = torch.arange(0, T, T // 48, device="cuda")[:48]
    xs = x[sample].contiguous()
    y_gen = _prefill_layer(d, f, E, K, xs.shape[0], 4, 4, False, xs, layer, generic=True)
    err = float((y[sample].float() - y_gen.float()).norm() / y_gen.float().norm())
    assert err <= TOL_REL_L2, err


def test_tensor_core_layer_prefill_without_a_shared_expert():
    """A layer with no shared expert through the tensor-core layer call: no rows are gathered behind the routed pairs
    (the grouping does not append any), and the result equals the generic kernels'."""
    import torch
    from mference_b200.moe import MoE
    d, f, E, K, T = 512, 512, 8, 2, 70
    W = O.LayerWeights(d, f, E, K, shared=False)
    h = make_x("h.noshared", T, d, std=2.0)
    lw = upload_layer(W)
    assert lw.shared_blob is None
    hd = to_dev16(h, O.DT_BF16)
    tc = MoE(d, f, E, K, shared_bits=0, max_tokens=T, tensor_core_prefill=True)
    # poison the tail of the arena's sort scratch: stale entries there must never be dereferenced
    tc.encode_layer_prefill(upload_layer(O.LayerWeights(d, f, E, K, shared=False, layer=1)), hd, torch.empty_like(hd))
    out_tc = torch.empty_like(hd)
    tc.encode_layer_prefill(lw, hd, out_tc)
    assert tc.device_status() == 0
    gen = MoE(d, f, E, K, shared_bits=0, max_tokens=T)
    out_gen = torch.empty_like(hd)
    gen.encode_layer(lw, hd, out_gen)
    a, b = out_tc.float().cpu().numpy(), out_gen.float().cpu().numpy()
    assert np.isfinite(a).all()
    assert O.rel_l2(a, b) <= TOL_REL_L2
    # and against the oracle, teacher-forced on the kernel's normalised rows
    xn = torch.empty_like(hd)
    tc.encode_rmsnorm(hd, xn, lw.norm_w)
    xn_bits = xn.view(torch.int16).cpu().numpy().view(np.uint16)
    lg = O.router_logits(xn_bits, O.DT_BF16, W.router)
    idx, w = O.topk_softmax(lg, K)
    ref = O.moe_layer(W, xn_bits, O.DT_BF16, idx, w, O.bf16_to_f32(h))
    assert O.rel_l2(a, ref) <= TOL_REL_L2

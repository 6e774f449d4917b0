"""GPU parity tests of the decode-time expert FFN, the weighted combine and the layer/stack calls, through the
C ABI, against the fp32-dequantised oracle (relative L2 <= 2e-3, the bar the task states)."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import TOL_REL_L2, make_x, to_dev16, upload_layer

pytestmark = pytest.mark.gpu

ROOT = 0xB2000001


def _route(W, x, dtype=O.DT_BF16):
    lg = O.router_logits(x, dtype, W.router)
    return O.topk_softmax(lg, W.top_k)


def _run_decode(W, x, idx, w, residual_bits=None, dtype=O.DT_BF16, **moe_kw):
    import torch
    from mference_b200.moe import MoE
    T = x.shape[0]
    moe = MoE(W.d, W.f, W.num_experts, W.top_k, bits=W.bits, shared_bits=W.shared_bits if W.shared_blob is not None else 0,
              scale_dtype=W.scale_dtype, x_dtype=dtype, activation=W.activation, swiglu_limit=W.swiglu_limit,
              max_tokens=max(T, 1), **moe_kw)
    lw = upload_layer(W)
    xd = to_dev16(x, dtype)
    idxd = torch.from_numpy(idx.view(np.int32)).cuda()
    wd = torch.from_numpy(w.view(np.int16)).cuda().view(torch.float16)
    res = None if residual_bits is None else to_dev16(residual_bits, dtype)
    y = torch.empty_like(xd)
    moe.encode_decode(lw, xd, idxd, wd, y, residual=res)
    torch.cuda.synchronize()
    return y.float().cpu().numpy(), moe, lw, (xd, idxd, wd, res)


SHAPES = [
    # d, f, E, K, bits, shared_bits, T
    (256, 128, 16, 4, 4, 4, 1),
    (256, 128, 16, 4, 4, 4, 5),
    (64, 64, 8, 2, 4, 4, 3),
    (128, 64, 8, 2, 2, 4, 4),
    (512, 256, 12, 3, 2, 2, 7),
    (1024, 256, 10, 6, 4, 0, 2),
    (4096, 256, 8, 2, 4, 4, 2),
    (2048, 512, 24, 8, 4, 4, 1),
    (2048, 512, 24, 8, 4, 4, 8),
    # shapes the tensor-core-fragment fast path takes (d a multiple of 512, f <= 512), both code widths,
    # token counts that leave partial and multiple 8-column tiles
    (2048, 512, 12, 4, 2, 4, 3),
    (2048, 512, 6, 3, 4, 4, 19),
    (512, 128, 8, 2, 4, 4, 5),
    (1024, 256, 8, 3, 2, 2, 11),
    (4096, 512, 6, 2, 4, 2, 2),
    # 8-bit shared expert (SharedExpertInt8): generic kernels
    (256, 128, 16, 4, 4, 8, 5),
    (128, 64, 8, 2, 2, 8, 1),
    (512, 256, 8, 2, 4, 8, 19),
]


@pytest.mark.parametrize("d,f,E,K,bits,sbits,T", SHAPES)
def test_decode_matches_oracle(d, f, E, K, bits, sbits, T):
    W = O.LayerWeights(d, f, E, K, bits=bits, shared_bits=sbits or 4, shared=bool(sbits))
    x = make_x("x", T, d)
    idx, w = _route(W, x)
    res = make_x("res", T, d)
    y, *_ = _run_decode(W, x, idx, w, residual_bits=res)
    ref = O.moe_layer(W, x, O.DT_BF16, idx, w, O.bf16_to_f32(res))
    for t in range(T):
        assert O.rel_l2(y[t], ref[t]) <= TOL_REL_L2, (t, O.rel_l2(y[t], ref[t]))
    assert O.rel_l2(y, ref) <= TOL_REL_L2


@pytest.mark.parametrize("d,f,E,K,bits,T", [(256, 128, 16, 4, 2, 5), (512, 256, 8, 2, 2, 1), (256, 128, 8, 3, 4, 7),
                                            (2048, 512, 12, 4, 2, 3)])
def test_decode_with_32_element_gate_groups_matches_oracle(d, f, E, K, bits, T):
    # DeepSeek V4's conversion: gate_proj of the routed experts with one scale and bias per 32 elements
    # (routedGateGroupSize, ModelExpertIO.swift:118-135); up, down and the shared expert keep 64
    W = O.LayerWeights(d, f, E, K, bits=bits, shared_bits=4, gate_group_size=32)
    x = make_x("x.g32", T, d)
    idx, w = _route(W, x)
    res = make_x("res.g32", T, d)
    y, *_ = _run_decode(W, x, idx, w, residual_bits=res)
    ref = O.moe_layer(W, x, O.DT_BF16, idx, w, O.bf16_to_f32(res))
    assert O.rel_l2(y, ref) <= TOL_REL_L2, O.rel_l2(y, ref)
    # and it is not the 64-element reading of the same bytes
    W64 = O.LayerWeights(d, f, E, K, bits=bits, shared_bits=4, gate_group_size=64)
    assert W.blob_bytes > W64.blob_bytes


def test_decode_config0_qwen_layer_single_token():
    # BASELINE configs[0]: hidden 2048, 256 experts top-8 + 1 shared, intermediate 512, 4-bit group-64
    K = 8
    W0 = O.LayerWeights(2048, 512, 256, K, experts=[])
    x = make_x("x", 1, 2048)
    idx, w = _route(W0, x)
    W = O.LayerWeights(2048, 512, 256, K, experts=sorted(set(idx[0].tolist())))
    y, *_ = _run_decode(W, x, idx, w)
    ref = O.moe_layer(W, x, O.DT_BF16, idx, w)
    assert O.rel_l2(y, ref) <= TOL_REL_L2, O.rel_l2(y, ref)


def test_decode_fp16_activations_bf16_scales_gelu_and_clamp():
    from mference_b200 import DT_F16
    W = O.LayerWeights(256, 128, 8, 2, scale_dtype=O.DT_BF16, activation=O.ACT_GELU_TANH, swiglu_limit=0.75)
    x = make_x("x", 3, 256, dtype=O.DT_F16, std=0.25)
    idx, w = _route(W, x, O.DT_F16)
    y, *_ = _run_decode(W, x, idx, w, dtype=DT_F16)
    ref = O.moe_layer(W, x, O.DT_F16, idx, w)
    assert O.rel_l2(y, ref) <= TOL_REL_L2, O.rel_l2(y, ref)


def test_hit_miss_split_is_bit_identical_to_full():
    # MoEFusedFFNTests: full == hit/miss split exactly
    import torch
    W = O.LayerWeights(256, 128, 16, 8)
    x = make_x("x", 3, 256)
    idx, w = _route(W, x)
    y_full, moe, lw, (xd, idxd, wd, _) = _run_decode(W, x, idx, w)
    y2 = torch.empty_like(xd)
    moe.encode_experts(lw, xd, idxd, wd, active_slots=[0, 2, 5], with_shared=True)
    moe.encode_experts(lw, xd, idxd, wd, active_slots=[1, 3, 4, 6, 7], with_shared=False)
    moe.encode_combine(wd, y2)
    assert np.array_equal(y2.float().cpu().numpy(), y_full)


def test_slot_map_equals_identity_and_missing_expert_is_a_no_op():
    # slot-map path == argument-buffer path bit for bit (MoEFusedFFNTests.swift:195-316)
    import torch
    from mference_b200.moe import MoE
    W = O.LayerWeights(256, 128, 8, 2)
    x = make_x("x", 4, 256)
    idx, w = _route(W, x)
    y_id, *_ = _run_decode(W, x, idx, w)
    perm = np.random.default_rng(1).permutation(8)
    Wp = O.LayerWeights(256, 128, 8, 2)
    Wp.pool = W.pool.reshape(8, -1)[np.argsort(perm)].reshape(-1).copy()   # expert e now lives in slot perm[e]
    moe = MoE(256, 128, 8, 2, max_tokens=4)
    lw = upload_layer(Wp, slot_of=perm.tolist())
    xd = to_dev16(x, O.DT_BF16)
    y = torch.empty_like(xd)
    idxd = torch.from_numpy(idx.view(np.int32)).cuda()
    wd = torch.from_numpy(w.view(np.int16)).cuda().view(torch.float16)
    moe.encode_decode(lw, xd, idxd, wd, y)
    assert np.array_equal(y.float().cpu().numpy(), y_id)


def test_batch_equals_single_rows_bit_for_bit():
    # MultiXKernelParityTests: multi-row == per-row bit for bit
    import torch
    W = O.LayerWeights(256, 128, 6, 3)
    x = make_x("x", 9, 256)
    idx, w = _route(W, x)
    y_batch, moe, lw, (xd, idxd, wd, _) = _run_decode(W, x, idx, w)
    from mference_b200.moe import MoE
    one = MoE(256, 128, 6, 3, max_tokens=1)
    for t in range(9):
        yt = torch.empty_like(xd[t:t + 1])
        one.encode_decode(lw, xd[t:t + 1], idxd[t:t + 1], wd[t:t + 1], yt)
        assert np.array_equal(yt.float().cpu().numpy()[0], y_batch[t]), t


def test_token_permutation_permutes_outputs_exactly_at_batch_64():
    # size-independent property at the full decode batch: per-row arithmetic does not depend on the grouping
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    from mference_b200 import DT_BF16
    d, f, E, K, T = 2048, 512, 256, 8, 64
    lw = synth_layer(0xB2000001, 0, d, f, E)
    moe = MoE(d, f, E, K, max_tokens=T)
    h = synth_normal(0xB2000001, "x", T * d, dtype=DT_BF16).view(T, d)
    out = torch.empty_like(h)
    moe.encode_layer(lw, h, out)
    perm = torch.randperm(T, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    out_p = torch.empty_like(h)
    moe.encode_layer(lw, h[perm].contiguous(), out_p)
    assert torch.equal(out_p.view(torch.int16), out[perm].view(torch.int16))
    assert torch.isfinite(out.float()).all()


def test_layer_matches_oracle_with_its_own_router():
    import torch
    from mference_b200.moe import MoE
    d, f, E, K, T = 512, 128, 32, 4, 6
    W = O.LayerWeights(d, f, E, K)
    h = make_x("h", T, d, std=3.0)
    moe = MoE(d, f, E, K, max_tokens=T)
    lw = upload_layer(W)
    hd = to_dev16(h, O.DT_BF16)
    xn = torch.empty_like(hd)
    moe.encode_rmsnorm(hd, xn, lw.norm_w)
    out = torch.empty_like(hd)
    moe.encode_layer(lw, hd, out)
    # norm: against the oracle, then teacher-force the layer on the kernel's own normalised rows
    hf = O.bf16_to_f32(h)
    xn_ref = O.rmsnorm(hf, None, 1e-6)
    xn_np = xn.float().cpu().numpy()
    assert np.abs(xn_np - xn_ref).max() <= 2.0 ** -8 * np.abs(xn_ref).max()
    xn_bits = xn.view(torch.int16).cpu().numpy().view(np.uint16)
    idx, w = _route(W, xn_bits)
    ref = O.moe_layer(W, xn_bits, O.DT_BF16, idx, w, hf)
    assert O.rel_l2(out.float().cpu().numpy(), ref) <= TOL_REL_L2


def test_stack_equals_layer_by_layer():
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    from mference_b200 import DT_BF16
    d, f, E, K, T, NL = 256, 128, 16, 4, 5, 6
    layers = [synth_layer(0xB2000001, l, d, f, E) for l in range(NL)]
    moe = MoE(d, f, E, K, max_tokens=T)
    h0 = synth_normal(0xB2000001, "x", T * d, dtype=DT_BF16).view(T, d)
    a = h0.clone()
    moe.encode_stack(moe.make_stack(layers), a)
    b = h0.clone()
    for lw in layers:
        nxt = torch.empty_like(b)
        moe.encode_layer(lw, b, nxt)
        b = nxt
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert torch.isfinite(a.float()).all()


def test_capacity_and_argument_errors():
    import torch
    from mference_b200 import MfbError, _lib as L
    from mference_b200.moe import MoE
    W = O.LayerWeights(64, 64, 4, 2)
    moe = MoE(64, 64, 4, 2, max_tokens=2)
    lw = upload_layer(W)
    x = torch.zeros((3, 64), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((3, 2), dtype=torch.int32, device="cuda")
    w = torch.zeros((3, 2), dtype=torch.float16, device="cuda")
    with pytest.raises(MfbError) as ei:
        moe.encode_decode(lw, x, idx, w, torch.empty_like(x))
    assert ei.value.code == L.ERR_CAPACITY
    with pytest.raises(MfbError) as ei:
        moe.encode_experts(lw, x[:2], idx[:2], w[:2], active_slots=[5])
    assert ei.value.code == L.ERR_INVALID_ARGUMENT
    assert moe.device_status() == 0


@pytest.mark.parametrize("T", [1, 3, 8, 9, 64])
def test_fast_path_agrees_with_generic_path(T):
    import torch
    from mference_b200.moe import MoE
    d, f, E, K = 2048, 512, 32, 8
    W = O.LayerWeights(d, f, E, K)
    h = make_x("h", T, d, std=2.0)
    moe = MoE(d, f, E, K, max_tokens=T)
    lw = upload_layer(W)
    hd = to_dev16(h, O.DT_BF16)
    fast = torch.empty_like(hd)
    moe.encode_layer(lw, hd, fast)
    moe.set_generic(True)
    slow = torch.empty_like(hd)
    moe.encode_layer(lw, hd, slow)
    assert moe.device_status() == 0
    a, b = fast.float().cpu().numpy(), slow.float().cpu().numpy()
    assert np.isfinite(a).all()
    # both sit within the tolerance of the oracle; against each other they differ by output rounding at most
    assert O.rel_l2(a, b) <= TOL_REL_L2


@pytest.mark.parametrize("T", [1, 5, 64])
def test_fused_stack_kernel_equals_layer_by_layer(T):
    # one cooperative launch for all layers against the per-layer launch sequence: bit for bit
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    from mference_b200 import DT_BF16
    d, f, E, K, NL = 2048, 512, 32, 8, 5
    layers = [synth_layer(0xB2000001, l, d, f, E) for l in range(NL)]
    moe = MoE(d, f, E, K, max_tokens=T)
    stack = moe.make_stack(layers)
    h0 = synth_normal(0xB2000001, "x", T * d, dtype=DT_BF16).view(T, d)
    a = h0.clone()
    moe.encode_stack(stack, a)
    b = h0.clone()
    for lw in layers:
        nxt = torch.empty_like(b)
        moe.encode_layer(lw, b, nxt)
        b = nxt
    assert moe.device_status() == 0
    assert torch.isfinite(a.float()).all()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # separate row blocks per layer, layers in order
    rows = synth_normal(0xB2000001, "rows", NL * T * d, dtype=DT_BF16).view(NL, T, d)
    c = rows.clone()
    moe.encode_stack_rows(stack, c)
    for l, lw in enumerate(layers):
        ref = torch.empty_like(rows[l])
        moe.encode_layer(lw, rows[l], ref)
        assert torch.equal(c[l].view(torch.int16), ref.view(torch.int16)), l
    assert moe.device_status() == 0


def test_phase_trace_of_the_fused_stack_kernel():
    """mfb_moe_set_trace: per-layer phase stamps are increasing global-timer values and the output is unchanged."""
    import torch
    from mference_b200 import _lib as L
    from mference_b200.moe import MoE, synth_layer, synth_normal
    d, f, E, K, T, NL = 2048, 512, 16, 8, 8, 3
    layers = [synth_layer(0xB2000001, l, d, f, E) for l in range(NL)]
    moe = MoE(d, f, E, K, max_tokens=T)
    stack = moe.make_stack(layers)
    h0 = synth_normal(0xB2000001, "x.trace", T * d, dtype=L.DT_BF16).view(T, d)
    ref = h0.clone()
    moe.encode_stack(stack, ref)
    trace = torch.zeros((NL + 17, 8), dtype=torch.int64, device="cuda")
    moe.set_trace(trace)
    h = h0.clone()
    moe.encode_stack(stack, h)
    moe.set_trace(None)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    assert torch.equal(h, ref)
    stamps = trace[:NL].cpu().numpy()
    assert (stamps > 0).all()
    flat = stamps.reshape(-1)
    assert (flat[1:] >= flat[:-1]).all()          # phases within a layer and layers in order
    clocks = trace[NL + 16].cpu().numpy()
    assert clocks[5] > clocks[4] and clocks[7] > clocks[6]   # SM clock and global timer advanced over the launch


def test_fast_shape_capacity_is_checked_on_the_host():
    """A handle created for two rows refuses three rows of a fast-path shape with ERR_CAPACITY and launches nothing."""
    import torch
    from mference_b200 import MfbError, _lib as L
    from mference_b200.moe import MoE
    d, f, E, K = 512, 256, 4, 2
    W = O.LayerWeights(d, f, E, K)
    moe = MoE(d, f, E, K, max_tokens=2)
    lw = upload_layer(W)
    x = torch.zeros((3, d), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((3, K), dtype=torch.int32, device="cuda")
    w = torch.zeros((3, K), dtype=torch.float16, device="cuda")
    before = moe.lib.mfb_launch_count()
    with pytest.raises(MfbError) as ei:
        moe.encode_decode(lw, x, idx, w, torch.empty_like(x))
    assert ei.value.code == L.ERR_CAPACITY
    with pytest.raises(MfbError) as ei:
        moe.encode_layer(lw, x, torch.empty_like(x))
    assert ei.value.code == L.ERR_CAPACITY
    assert moe.lib.mfb_launch_count() == before
    assert moe.device_status() == 0


@pytest.mark.parametrize("T", [1, 8, 19, 64])
def test_fp32_partial_rows_of_the_fast_path_match_the_oracle(T):
    """The decode fast path judged below the output rounding: its fp32 down-projection rows per (token, rank slot)
    against the oracle's per-pair rows.  What remains is the fp16 rounding of the hidden activations (the reference
    stores them as fp16 too, half an ulp is 4.9e-4 relative): bound 8e-4, well under the layer tolerance."""
    import torch
    from mference_b200.moe import MoE
    d, f, E, K = 2048, 512, 24, 8
    W = O.LayerWeights(d, f, E, K)
    x = make_x("x.partial", T, d)
    idx, w = _route(W, x)
    y, moe, lw, _ = _run_decode(W, x, idx, w)
    part = moe.partial_rows(T).cpu().numpy()            # [T, K + 1, d]
    pairs = np.zeros(T * K, dtype=O.PAIR_DTYPE)
    for t in range(T):
        for r in range(K):
            pairs[t * K + r] = (t, idx[t, r], r, 0)
    ref = O.pair_partials(W, x, O.DT_BF16, pairs).reshape(T, K, d)   # the routed slots; slot K is the shared expert's
    assert moe.device_status() == 0
    worst = max(O.rel_l2(part[t, r], ref[t, r]) for t in range(T) for r in range(K))
    assert worst <= 8e-4, worst


@pytest.mark.parametrize("T", [1, 8, 64])
def test_fused_stack_kernel_on_the_headline_shape(T):
    """256 experts, top-8 + shared, hidden 2048 / intermediate 512 - the benchmark's layer shape and work split (about
    9 / 58 / 223 expert groups per layer): the fused kernel against the layer-by-layer launches bit for bit, chained
    and with separate rows per layer, and sampled rows against the oracle."""
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    from mference_b200 import DT_BF16
    d, f, E, K, NL = 2048, 512, 256, 8, 4
    layers = [synth_layer(ROOT, l, d, f, E) for l in range(NL)]
    moe = MoE(d, f, E, K, max_tokens=T)
    stack = moe.make_stack(layers)
    h0 = synth_normal(ROOT, "x.headline", T * d, dtype=DT_BF16).view(T, d)
    a = h0.clone()
    moe.encode_stack(stack, a)
    b = h0.clone()
    for lw in layers:
        nxt = torch.empty_like(b)
        moe.encode_layer(lw, b, nxt)
        b = nxt
    assert moe.device_status() == 0
    assert torch.isfinite(a.float()).all()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    rows = synth_normal(ROOT, "rows.headline", NL * T * d, dtype=DT_BF16).view(NL, T, d)
    c = rows.clone()
    moe.encode_stack_rows(stack, c)
    assert moe.device_status() == 0
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float16, device="cuda")
    for l, lw in enumerate(layers):
        ref = torch.empty_like(rows[l])
        moe.encode_layer(lw, rows[l], ref)
        assert torch.equal(c[l].view(torch.int16), ref.view(torch.int16)), l
        # oracle on up to eight rows of this layer, teacher-forced on the kernel's own normalised rows and routes
        xn = torch.empty_like(rows[l])
        moe.encode_rmsnorm(rows[l], xn, lw.norm_w)
        moe.encode_router(xn, lw, idx, w)
        sample = sorted(set(np.linspace(0, T - 1, num=min(T, 8)).astype(int).tolist()))
        xn_bits = xn.view(torch.int16).cpu().numpy().view(np.uint16)[sample]
        idx_h = idx.cpu().numpy().view(np.uint32)[sample]
        w_h = w.view(torch.int16).cpu().numpy().view(np.uint16)[sample]
        W = O.LayerWeights(d, f, E, K, layer=l, experts=sorted(set(idx_h.reshape(-1).tolist())))
        lg = O.router_logits(xn_bits, O.DT_BF16, W.router)
        idx_o, w_o = O.topk_softmax(lg, K)
        assert np.array_equal(idx_o, idx_h)
        res = rows[l].float().cpu().numpy()[sample]
        want = O.moe_layer(W, xn_bits, O.DT_BF16, idx_h, w_h, res)
        got = c[l].float().cpu().numpy()[sample]
        for i in range(len(sample)):
            assert O.rel_l2(got[i], want[i]) <= TOL_REL_L2, (l, sample[i], O.rel_l2(got[i], want[i]))
    assert moe.device_status() == 0


def test_a_bounded_wait_that_runs_out_is_reported_and_the_handle_stays_usable():
    """One CTA waits about a millisecond on a barrier nothing arrives at: the kernel returns, the status word carries
    the time-out, reading it clears it, and the next decode call on the same handle is exact again."""
    import torch
    from mference_b200 import _lib as L
    W = O.LayerWeights(512, 256, 8, 2)
    x = make_x("x.wait", 3, 512)
    idx, w = _route(W, x)
    y0, moe, lw, (xd, idxd, wd, _) = _run_decode(W, x, idx, w)
    assert moe.device_status() == 0
    moe.selftest_wait(2_000_000)
    torch.cuda.synchronize()
    assert moe.device_status() == 1          # STATUS_MBAR_TIMEOUT, through MFB_ERR_DEVICE_STATUS
    assert moe.device_status() == 0          # cleared by the read
    y1 = torch.empty_like(xd)
    moe.encode_decode(lw, xd, idxd, wd, y1)
    torch.cuda.synchronize()
    assert np.array_equal(y1.float().cpu().numpy(), y0)
    assert moe.device_status() == 0

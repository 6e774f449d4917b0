"""GPU parity of the quantised gates and resident projections: hash-routed weights and the INT8 gate GEMV bit for bit
against the oracle's restatement of the reference kernels, the INT4 GEMV within 1e-5 of the fp32 reference, the Qwen
layer switches (INT8 router, shared-expert scalar gate) against the oracle, and a toy model directory read from disk."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import TOL_REL_L2, make_x, to_dev16, upload_layer

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def _int8_tensor(rng, rows, cols, scale=0.004):
    import torch
    W = rng.integers(0, 256, (rows, cols), dtype=np.uint8)
    s = O.f32_to_bf16(np.abs(rng.standard_normal((rows, cols // 64)).astype(np.float32)) * scale)
    b = O.f32_to_bf16(rng.standard_normal((rows, cols // 64)).astype(np.float32) * scale * 100)
    return W, s, b


def test_hash_weights_are_bit_exact():
    import ctypes as C
    import torch
    from mference_b200 import _lib as L
    rng = np.random.default_rng(11)
    T, E, K = 37, 256, 6
    logits = rng.standard_normal((T, E)).astype(np.float32) * 3
    idx = np.stack([rng.choice(E, K, replace=False) for _ in range(T)]).astype(np.uint32)
    want = O.hash_weights(logits, idx, 1.5)
    out = torch.zeros((T, K), dtype=torch.float16, device="cuda")
    lg_d, idx_d = _dev(logits), _dev(idx.view(np.int32))     # held in variables: the call only sees raw pointers
    L.check(L.load().mfb_router_hash_weights(None, lg_d.data_ptr(), idx_d.data_ptr(), T, E, K, 1.5, out.data_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)


@pytest.mark.parametrize("M,N,T,eff", [(256, 2048, 3, False), (1, 2048, 5, False), (64, 512, 9, True), (7, 128, 1, True)])
def test_int8_gate_gemv_is_bit_exact(M, N, T, eff):
    import torch
    from mference_b200 import _lib as L
    rng = np.random.default_rng(M * 7 + N)
    W, s, b = _int8_tensor(rng, M, N)
    x = make_x(f"x.int8.{M}", T, N)
    es = O.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(N).astype(np.float32)) if eff else None
    want = O.gemv_int8(W, s, b, x, O.DT_BF16, es)
    y = torch.zeros((T, M), dtype=torch.float32, device="cuda")
    xd = to_dev16(x, O.DT_BF16)
    W_d, s_d, b_d = _dev(W), _dev(s.view(np.int16)), _dev(b.view(np.int16))
    es_d = None if es is None else _dev(es.view(np.int16))
    L.check(L.load().mfb_gemv_int8(None, W_d.data_ptr(), s_d.data_ptr(), b_d.data_ptr(), xd.data_ptr(), L.DT_BF16, N, T,
                                   None if es_d is None else es_d.data_ptr(), M, N, y.data_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("M,N,T,sdt", [(512, 2048, 1, O.DT_BF16), (300, 2048, 8, O.DT_BF16), (64, 512, 3, O.DT_F16), (2048, 4096, 5, O.DT_BF16)])
def test_int4_gemv_matches_the_fp32_reference(M, N, T, sdt):
    import torch
    from mference_b200 import MfbError, _lib as L
    rng = np.random.default_rng(M + N + T)
    W = rng.integers(0, 256, (M, N // 2), dtype=np.uint8)
    conv = O.f32_to_bf16 if sdt == O.DT_BF16 else O.f32_to_f16
    s = conv(np.abs(rng.standard_normal((M, N // 64)).astype(np.float32)) * 0.02)
    b = conv(rng.standard_normal((M, N // 64)).astype(np.float32) * 0.01)
    x = make_x(f"x.int4.{M}", T, N)
    want = O.gemv_int4(W, s, b, sdt, x, O.DT_BF16)
    y = torch.zeros((T, M), dtype=torch.float32, device="cuda")
    xd = to_dev16(x, O.DT_BF16)
    lib = L.load()
    W_d, s_d, b_d = _dev(W), _dev(s.view(np.int16)), _dev(b.view(np.int16))
    L.check(lib.mfb_gemv_int4(None, W_d.data_ptr(), s_d.data_ptr(), b_d.data_ptr(), sdt, xd.data_ptr(), L.DT_BF16, N, T, M, N, y.data_ptr()))
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    for t in range(T):
        assert O.rel_l2(got[t], want[t]) <= 1e-5, (t, O.rel_l2(got[t], want[t]))
    with pytest.raises(MfbError) as err:   # nine rows: over the limit of one call
        L.check(lib.mfb_gemv_int4(None, W_d.data_ptr(), s_d.data_ptr(), b_d.data_ptr(), sdt, xd.data_ptr(), L.DT_BF16, N, 9, M, N, y.data_ptr()))
    assert err.value.code == L.ERR_CAPACITY


def _gated_reference(W, Wq, x_bits, res_f32, gate, K):
    """Oracle composition of a Qwen layer: INT8 router logits -> top-k softmax -> experts; the shared expert's row
    (layer with shared minus layer without) times sigmoid(fp16(gate logit))."""
    rw, rs, rb = Wq
    lg = O.gemv_int8(rw, rs, rb, x_bits, O.DT_BF16)
    idx, w = O.topk_softmax(lg, K)
    with_shared = O.moe_layer(W, x_bits, O.DT_BF16, idx, w, res_f32)
    blob, W.shared_blob = W.shared_blob, None
    without = O.moe_layer(W, x_bits, O.DT_BF16, idx, w, res_f32)
    W.shared_blob = blob
    gw, gs, gb = gate
    g = O.gemv_int8(gw, gs, gb, x_bits, O.DT_BF16)[:, 0]
    m = 1.0 / (1.0 + np.exp(-O.f16_to_f32(O.f32_to_f16(g)).astype(np.float64)))
    return without + (with_shared - without) * m[:, None].astype(np.float32), idx, w


@pytest.mark.parametrize("d,f,E,K,T", [(512, 256, 16, 4, 5), (2048, 512, 32, 8, 3), (2048, 512, 32, 8, 24)])
def test_layer_with_int8_router_and_shared_scalar_gate(d, f, E, K, T):
    import torch
    from mference_b200.moe import MoE
    rng = np.random.default_rng(d + T)
    W = O.LayerWeights(d, f, E, K, scale_dtype=O.DT_BF16)
    router = _int8_tensor(rng, E, d)
    gate = _int8_tensor(rng, 1, d, scale=0.0005)
    h = make_x("h.qwen", T, d, std=2.0)
    lw = upload_layer(W)
    lw.router_w = _dev(router[0])
    lw.router_scales, lw.router_biases = _dev(router[1].view(np.int16), torch.bfloat16), _dev(router[2].view(np.int16), torch.bfloat16)
    lw.shared_gate_w = _dev(gate[0].reshape(-1))
    lw.shared_gate_s, lw.shared_gate_b = _dev(gate[1].view(np.int16), torch.bfloat16), _dev(gate[2].view(np.int16), torch.bfloat16)
    moe = MoE(d, f, E, K, scale_dtype=O.DT_BF16, max_tokens=T)
    hd = to_dev16(h, O.DT_BF16)
    out = torch.empty_like(hd)
    moe.encode_layer(lw, hd, out)
    xn = torch.empty_like(hd)
    moe.encode_rmsnorm(hd, xn, lw.norm_w)
    idx_d = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w_d = torch.empty((T, K), dtype=torch.float16, device="cuda")
    moe.encode_router(xn, lw, idx_d, w_d)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    xn_bits = xn.view(torch.int16).cpu().numpy().view(np.uint16)
    ref, idx, w = _gated_reference(W, router, xn_bits, O.bf16_to_f32(h), gate, K)
    assert np.array_equal(idx_d.cpu().numpy().view(np.uint32), idx)
    assert O.rel_l2(out.float().cpu().numpy(), ref) <= TOL_REL_L2
    # a stack call with such layers takes the layer-by-layer route and gives the same rows
    again = hd.clone()
    moe.encode_stack(moe.make_stack([lw]), again)
    assert torch.equal(again, out)
    # the generic kernels agree
    moe.set_generic(True)
    slow = torch.empty_like(hd)
    moe.encode_layer(lw, hd, slow)
    assert O.rel_l2(slow.float().cpu().numpy(), ref) <= TOL_REL_L2


def test_toy_model_directory_drives_the_layer(tmp_path):
    """A one-layer Qwen-shaped toy directory written to disk the way the reference's toy fixture lays it out
    (model_weights.bin with INT8 router, scalar gate, shared expert and norm; packed_experts/ with the routed experts),
    read back by the two readers, and run: equal to the layer built from the in-memory tensors, and to the oracle."""
    import torch
    from mference_b200.moe import MoE
    from mference_b200.packed_experts import layer_weights_from_packed, write_packed_experts
    from mference_b200.resident_index import DTYPE_AFFINE, DTYPE_BF16, ResidentIndex, layer_resident_weights, qwen_moe_tensor_names, write_resident_file
    d, f, E, K, T = 512, 256, 8, 2, 7
    rng = np.random.default_rng(99)
    W = O.LayerWeights(d, f, E, K, scale_dtype=O.DT_BF16)
    router = _int8_tensor(rng, E, d)
    gate = _int8_tensor(rng, 1, d, scale=0.0005)
    norm = O.f32_to_bf16(1.0 + 0.05 * rng.standard_normal(d).astype(np.float32))
    names = qwen_moe_tensor_names(0)
    so = W.shared_off
    sb = W.shared_blob

    def part(a, n):
        return sb[a:a + n]

    tensors = [(names["norm"], DTYPE_BF16, (d,), norm, None, None),
               (names["router"], DTYPE_AFFINE, (E, d), router[0], router[1], router[2]),
               (names["shared_gate"], DTYPE_AFFINE, (1, d), gate[0], gate[1], gate[2]),
               (names["shared_gate_proj"], DTYPE_AFFINE, (f, d), part(so.gate_w, f * d // 2), part(so.gate_s, f * d // 32).view(np.uint16),
                part(so.gate_b, f * d // 32).view(np.uint16)),
               (names["shared_up_proj"], DTYPE_AFFINE, (f, d), part(so.up_w, f * d // 2), part(so.up_s, f * d // 32).view(np.uint16),
                part(so.up_b, f * d // 32).view(np.uint16)),
               (names["shared_down_proj"], DTYPE_AFFINE, (d, f), part(so.down_w, f * d // 2), part(so.down_s, f * d // 32).view(np.uint16),
                part(so.down_b, f * d // 32).view(np.uint16))]
    write_resident_file(str(tmp_path / "model_weights.bin"), tensors)
    mem = upload_layer(W)
    layout = write_packed_experts(str(tmp_path), [dict(pool=mem.pool, slot_stride=mem.slot_stride, offsets=mem.routed_off, d=d, f=f,
                                                       bits=4, scale_dtype="BF16")])
    index = ResidentIndex(str(tmp_path / "model_weights.bin"))
    resident = layer_resident_weights(index, 0, d, f, E)
    router_w = resident.pop("router_w")
    lw = layer_weights_from_packed(str(tmp_path), layout, 0, router_w, **resident)
    moe = MoE(d, f, E, K, scale_dtype=O.DT_BF16, max_tokens=T)
    h = make_x("h.toy", T, d, std=1.5)
    hd = to_dev16(h, O.DT_BF16)
    out = torch.empty_like(hd)
    moe.encode_layer(lw, hd, out)
    xn = torch.empty_like(hd)
    moe.encode_rmsnorm(hd, xn, lw.norm_w)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    xn_bits = xn.view(torch.int16).cpu().numpy().view(np.uint16)
    ref, _, _ = _gated_reference(W, router, xn_bits, O.bf16_to_f32(h), gate, K)
    assert O.rel_l2(out.float().cpu().numpy(), ref) <= TOL_REL_L2
    # the norm weight from the file was used: against the oracle's RMSNorm with it
    xn_ref = O.rmsnorm(O.bf16_to_f32(h), norm, 1e-6)
    assert np.abs(xn.float().cpu().numpy() - xn_ref).max() <= 2.0 ** -7 * np.abs(xn_ref).max()

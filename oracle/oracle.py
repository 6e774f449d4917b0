"""ctypes front end of the CPU oracle (oracle/mfb_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU-baseline
leg.  The shipped package never imports this module.  Each wrapper takes and returns numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libmfb_oracle.so")

DT_BF16, DT_F16, DT_F32 = 0, 1, 2
ACT_SILU, ACT_GELU_TANH = 0, 1

GROUP_ERRORS = {
    0: "ok", 1: "invalidQueryCount", 2: "invalidTopK", 3: "invalidNumExperts", 4: "invalidTileExpertCount",
    5: "pairCountMismatch", 6: "tokenOutOfRange", 7: "rankOutOfRange", 8: "expertOutOfRange",
    9: "duplicateTokenRank", 10: "expertSortKeyCountMismatch",
}


class ExpertOffsets(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b", "down_w", "down_s", "down_b")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


class Layer(C.Structure):
    _fields_ = [("d", C.c_uint32), ("f", C.c_uint32), ("num_experts", C.c_uint32), ("top_k", C.c_uint32),
                ("bits", C.c_uint32), ("shared_bits", C.c_uint32), ("group_size", C.c_uint32),
                ("scale_dtype", C.c_uint32), ("activation", C.c_uint32), ("swiglu_limit", C.c_float),
                ("pool", C.c_void_p), ("expert_stride", C.c_uint64), ("shared_blob", C.c_void_p),
                ("routed_off", ExpertOffsets), ("shared_off", ExpertOffsets), ("gate_group_size", C.c_uint32)]


PAIR_DTYPE = np.dtype([("token", "<u4"), ("expert", "<u4"), ("rank", "<u4"), ("weight_bits", "<u4")])
GROUP_DTYPE = np.dtype([("expert", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])
TILE_DTYPE = np.dtype([("group_start", "<u4"), ("group_count", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])


def build(force: bool = False) -> str:
    """Compile the oracle with the system gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "mfb_oracle.c")
    hdr = os.path.join(_HERE, "mfb_oracle.h")
    stale = (not os.path.exists(_SO)) or any(os.path.getmtime(p) > os.path.getmtime(_SO) for p in (src, hdr))
    if force or stale:
        env = dict(os.environ)
        env["PATH"] = "/usr/bin:" + env.get("PATH", "")
        env.pop("CC", None)
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, env=env, stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.mfbo_splitmix_at.restype = C.c_uint64
        _lib.mfbo_splitmix_at.argtypes = [C.c_uint64, C.c_uint64]
        _lib.mfbo_seed_for_label.restype = C.c_uint64
        _lib.mfbo_seed_for_label.argtypes = [C.c_uint64, C.c_char_p]
        _lib.mfbo_uniform_at.restype = C.c_float
        _lib.mfbo_uniform_at.argtypes = [C.c_uint64, C.c_uint64, C.c_float, C.c_float]
        _lib.mfbo_f32_to_bf16.restype = C.c_uint16
        _lib.mfbo_f32_to_bf16.argtypes = [C.c_float]
        _lib.mfbo_f32_to_f16.restype = C.c_uint16
        _lib.mfbo_f32_to_f16.argtypes = [C.c_float]
        _lib.mfbo_num_threads.restype = C.c_int
        _lib.mfbo_group_pairs.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


# ----------------------------------------------------------------------------- PRNG / synthesis

def seed_for_label(root: int, label: str) -> int:
    return lib().mfbo_seed_for_label(C.c_uint64(root), label.encode())


def splitmix_at(seed: int, index: int) -> int:
    return lib().mfbo_splitmix_at(C.c_uint64(seed), C.c_uint64(index))


def uniform_at(seed: int, index: int, lo: float, hi: float) -> float:
    return lib().mfbo_uniform_at(C.c_uint64(seed), C.c_uint64(index), lo, hi)


def fill_raw(seed: int, n_draws: int, first: int = 0) -> np.ndarray:
    out = np.empty(n_draws, dtype=np.uint64)
    lib().mfbo_fill_raw(C.c_uint64(seed), C.c_uint64(first), C.c_uint64(n_draws), _p(out))
    return out


def fill_normal(seed: int, n: int, mean=0.0, std=1.0, absolute=False, dtype=DT_BF16, first: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32 if dtype == DT_F32 else np.uint16)
    lib().mfbo_fill_normal(C.c_uint64(seed), C.c_uint64(first), C.c_uint64(n), C.c_double(mean), C.c_double(std),
                           C.c_int(1 if absolute else 0), C.c_int(dtype), _p(out))
    return out


def make_offsets(bits: int, d: int, f: int, gate_group_size: int = 64):
    off = ExpertOffsets()
    total = C.c_uint64()
    lib().mfbo_make_offsets_gate(C.c_int(bits), C.c_uint32(d), C.c_uint32(f), C.c_uint32(gate_group_size), C.byref(off),
                                 C.byref(total))
    return off, total.value


def synth_expert(root: int, layer: int, expert: int, bits: int, scale_dtype: int, d: int, f: int,
                 gate_group_size: int = 64) -> np.ndarray:
    _, total = make_offsets(bits, d, f, gate_group_size)
    blob = np.empty(total, dtype=np.uint8)
    lib().mfbo_synth_expert_gate(C.c_uint64(root), C.c_uint32(layer), C.c_int32(expert), C.c_int(bits),
                                 C.c_int(scale_dtype), C.c_uint32(d), C.c_uint32(f), C.c_uint32(gate_group_size), _p(blob))
    return blob


def synth_router(root: int, layer: int, num_experts: int, d: int) -> np.ndarray:
    out = np.empty((num_experts, d), dtype=np.uint16)
    lib().mfbo_synth_router(C.c_uint64(root), C.c_uint32(layer), C.c_uint32(num_experts), C.c_uint32(d), _p(out))
    return out


# ----------------------------------------------------------------------------- conversions

def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def widen(bits: np.ndarray, dtype: int) -> np.ndarray:
    return bf16_to_f32(bits) if dtype == DT_BF16 else f16_to_f32(bits)


def narrow(x: np.ndarray, dtype: int) -> np.ndarray:
    return f32_to_bf16(x) if dtype == DT_BF16 else f32_to_f16(x)


# ----------------------------------------------------------------------------- quantisation

def dequant_rows(codes, scales, biases, bits, rows, cols, scale_dtype=DT_F16, group_size=64) -> np.ndarray:
    codes = _c(codes, np.uint8); scales = _c(scales, np.uint16); biases = _c(biases, np.uint16)
    out = np.empty((rows, cols), dtype=np.float32)
    lib().mfbo_dequant_rows(_p(codes), _p(scales), _p(biases), C.c_int(bits), C.c_int(group_size),
                            C.c_int(scale_dtype), C.c_uint32(rows), C.c_uint32(cols), _p(out))
    return out


def quantize_int4_row(row):
    row = _c(row, np.float32)
    n = row.size
    packed = np.empty(n // 2, dtype=np.uint8)
    s = np.empty(n // 64, dtype=np.uint16)
    b = np.empty(n // 64, dtype=np.uint16)
    lib().mfbo_quantize_int4_row(_p(row), C.c_uint32(n), _p(packed), _p(s), _p(b))
    return packed, s, b


# ----------------------------------------------------------------------------- router

def router_logits(x, x_dtype, w_bf16, logit_bias=None, exact_f64=False) -> np.ndarray:
    x = _c(x, np.uint16); w = _c(w_bf16, np.uint16)
    T, d = x.shape
    E = w.shape[0]
    lb = None if logit_bias is None else _c(logit_bias, np.float32)
    out = np.empty((T, E), dtype=np.float32)
    lib().mfbo_router_logits(_p(x), C.c_int(x_dtype), C.c_uint32(d), C.c_uint32(T), _p(w), C.c_uint32(E),
                             C.c_uint32(d), _p(lb), C.c_int(1 if exact_f64 else 0), _p(out))
    return out


def topk_softmax(logits, top_k, per_expert_scale_bf16=None):
    lg = _c(logits, np.float32)
    T, E = lg.shape
    pes = None if per_expert_scale_bf16 is None else _c(per_expert_scale_bf16, np.uint16)
    idx = np.empty((T, top_k), dtype=np.uint32)
    w = np.empty((T, top_k), dtype=np.uint16)
    lib().mfbo_topk_softmax(_p(lg), C.c_uint32(T), C.c_uint32(E), C.c_uint32(top_k), _p(pes), _p(idx), _p(w))
    return idx, w


def topk_sqrtsoftplus(logits, top_k, correction_bias=None, route_scale=1.0):
    lg = _c(logits, np.float32)
    T, E = lg.shape
    cb = None if correction_bias is None else _c(correction_bias, np.float32)
    idx = np.empty((T, top_k), dtype=np.uint32)
    w = np.empty((T, top_k), dtype=np.uint16)
    lib().mfbo_topk_sqrtsoftplus(_p(lg), C.c_uint32(T), C.c_uint32(E), C.c_uint32(top_k), _p(cb),
                                 C.c_float(route_scale), _p(idx), _p(w))
    return idx, w


def topk_margin(scores, top_k) -> np.ndarray:
    sc = _c(scores, np.float32)
    T, E = sc.shape
    out = np.empty(T, dtype=np.float32)
    lib().mfbo_topk_margin(_p(sc), C.c_uint32(T), C.c_uint32(E), C.c_uint32(top_k), _p(out))
    return out


# ----------------------------------------------------------------------------- layer

class LayerWeights:
    """Host copy of one synthetic MoE layer: a pool of expert blobs, a shared blob and the router."""

    def __init__(self, d, f, num_experts, top_k, bits=4, shared_bits=4, scale_dtype=DT_F16,
                 activation=ACT_SILU, swiglu_limit=0.0, root=0xB2000001, layer=0, experts=None, shared=True,
                 gate_group_size=64):
        self.d, self.f, self.num_experts, self.top_k = d, f, num_experts, top_k
        self.bits, self.shared_bits, self.scale_dtype = bits, shared_bits, scale_dtype
        self.activation, self.swiglu_limit = activation, swiglu_limit
        self.gate_group_size = gate_group_size   # routed experts' gate_proj only (DeepSeek V4: 32 on most layers)
        self.routed_off, self.blob_bytes = make_offsets(bits, d, f, gate_group_size)
        self.shared_off, self.shared_bytes = make_offsets(shared_bits, d, f)
        self.expert_stride = (self.blob_bytes + 255) // 256 * 256
        self.pool = np.zeros(num_experts * self.expert_stride, dtype=np.uint8)
        which = range(num_experts) if experts is None else experts
        for e in which:
            self.pool[e * self.expert_stride: e * self.expert_stride + self.blob_bytes] = \
                synth_expert(root, layer, e, bits, scale_dtype, d, f, gate_group_size)
        self.shared_blob = synth_expert(root, layer, -1, shared_bits, scale_dtype, d, f) if shared else None
        self.router = synth_router(root, layer, num_experts, d)

    def c_layer(self) -> Layer:
        L = Layer()
        L.d, L.f, L.num_experts, L.top_k = self.d, self.f, self.num_experts, self.top_k
        L.bits, L.shared_bits, L.group_size, L.scale_dtype = self.bits, self.shared_bits, 64, self.scale_dtype
        L.activation, L.swiglu_limit = self.activation, self.swiglu_limit
        L.pool = self.pool.ctypes.data
        L.expert_stride = self.expert_stride
        L.shared_blob = None if self.shared_blob is None else self.shared_blob.ctypes.data
        L.routed_off, L.shared_off = self.routed_off, self.shared_off
        L.gate_group_size = self.gate_group_size
        return L


def moe_layer(W: LayerWeights, x, x_dtype, idx, w_f16, residual=None) -> np.ndarray:
    x = _c(x, np.uint16); idx = _c(idx, np.uint32); w = _c(w_f16, np.uint16)
    T, d = x.shape
    res = None if residual is None else _c(residual, np.float32)
    y = np.empty((T, d), dtype=np.float32)
    L = W.c_layer()
    lib().mfbo_moe_layer(C.byref(L), _p(x), C.c_int(x_dtype), C.c_uint32(d), C.c_uint32(T), _p(idx), _p(w),
                         _p(res), _p(y))
    return y


def pair_partials(W: LayerWeights, x, x_dtype, pairs) -> np.ndarray:
    x = _c(x, np.uint16)
    pairs = np.ascontiguousarray(pairs, dtype=PAIR_DTYPE)
    out = np.empty((pairs.size, W.d), dtype=np.float32)
    L = W.c_layer()
    lib().mfbo_pair_partials(C.byref(L), _p(x), C.c_int(x_dtype), C.c_uint32(x.shape[1]), _p(pairs),
                             C.c_uint32(pairs.size), _p(out))
    return out


def inkling_accumulate(W: LayerWeights, x, x_dtype, idx, w_f32, acc0=None) -> np.ndarray:
    """inkling_prefill_expert_act + inkling_prefill_expert_down_accum (Sources/Mference/Metal/Prefill/prefill.metal:
    654-746): expert by expert in ascending expert id, acc[t] = fma(w[t, r], down_row(t, r), acc[t]) in fp32; idx is
    [T, K] expert ids, w_f32 [T, K].  The rows come from the float64 definition (`pair_partials`); the reference's
    fp16 roundings of gate, up and their product are below the parity tolerance and are not modelled."""
    idx = np.asarray(idx)
    T, K = idx.shape
    pairs = np.zeros(T * K, dtype=PAIR_DTYPE)
    pairs["token"] = np.repeat(np.arange(T, dtype=np.uint32), K)
    pairs["expert"] = idx.reshape(-1)
    pairs["rank"] = np.tile(np.arange(K, dtype=np.uint32), T)
    rows = pair_partials(W, x, x_dtype, pairs).reshape(T, K, W.d).astype(np.float32)
    acc = np.zeros((T, W.d), dtype=np.float32) if acc0 is None else np.array(acc0, dtype=np.float32, copy=True)
    for t in range(T):
        for r in np.argsort(idx[t], kind="stable"):
            acc[t] = np.float32(w_f32[t, r]) * rows[t, r] + acc[t]
    return acc


def ref_moe_layer_f32(W: LayerWeights, x_f32, idx, w_f16, residual=None) -> np.ndarray:
    x = _c(x_f32, np.float32); idx = _c(idx, np.uint32); w = _c(w_f16, np.uint16)
    T, d = x.shape
    res = None if residual is None else _c(residual, np.float32)
    y = np.empty((T, d), dtype=np.float32)
    L = W.c_layer()
    lib().mfbo_ref_moe_layer_f32(C.byref(L), _p(x), C.c_uint32(T), _p(idx), _p(w), _p(res), _p(y))
    return y


def hash_weights(logits, idx, route_scale=1.0) -> np.ndarray:
    logits = _c(logits, np.float32); idx = _c(idx, np.uint32)
    T, E = logits.shape
    K = idx.shape[1]
    out = np.empty((T, K), dtype=np.uint16)
    lib().mfbo_hash_weights(_p(logits), _p(idx), C.c_uint32(T), C.c_uint32(E), C.c_uint32(K), C.c_float(route_scale), _p(out))
    return out


def gemv_int8(W, scales_bf16, biases_bf16, x, x_dtype, effective_scale_bf16=None) -> np.ndarray:
    """y[t, r] of the INT8 affine group-64 GEMV in the reference kernels' summation order; W uint8 [M, N]."""
    W = _c(W, np.uint8); s = _c(scales_bf16, np.uint16); b = _c(biases_bf16, np.uint16); x = _c(x, np.uint16)
    M, N = W.shape
    T = x.shape[0]
    es = None if effective_scale_bf16 is None else _c(effective_scale_bf16, np.uint16)
    y = np.empty((T, M), dtype=np.float32)
    lib().mfbo_gemv_int8(_p(W), _p(s), _p(b), _p(x), C.c_int(x_dtype), C.c_uint32(x.shape[1]), C.c_uint32(T), _p(es),
                         C.c_uint32(M), C.c_uint32(N), _p(y))
    return y


def gemv_int4(W, scales, biases, scale_dtype, x, x_dtype) -> np.ndarray:
    """fp32 reference of the INT4 affine group-64 GEMV; W uint8 [M, N/2] (low nibble = even element)."""
    W = _c(W, np.uint8); s = _c(scales, np.uint16); b = _c(biases, np.uint16); x = _c(x, np.uint16)
    M, N = W.shape[0], W.shape[1] * 2
    T = x.shape[0]
    y = np.empty((T, M), dtype=np.float32)
    lib().mfbo_gemv_int4(_p(W), _p(s), _p(b), C.c_int(scale_dtype), _p(x), C.c_int(x_dtype), C.c_uint32(x.shape[1]),
                         C.c_uint32(T), C.c_uint32(M), C.c_uint32(N), _p(y))
    return y


def num_threads() -> int:
    return lib().mfbo_num_threads()


def set_num_threads(n: int) -> None:
    lib().mfbo_set_num_threads(C.c_int(int(n)))


# ----------------------------------------------------------------------------- grouping / reduce / norm

class GroupingError(ValueError):
    def __init__(self, code, a, b):
        super().__init__(f"{GROUP_ERRORS[code]}({a}, {b})")
        self.code, self.case, self.a, self.b = code, GROUP_ERRORS[code], a, b


def group_pairs(pairs, query_count, top_k, num_experts, tile_expert_count=16, sort_keys=None):
    pairs = np.ascontiguousarray(pairs, dtype=PAIR_DTYPE)
    n = pairs.size
    keys = None if sort_keys is None else _c(sort_keys, np.uint64)
    ne = max(num_experts, 1)
    sorted_pairs = np.empty(max(n, 1), dtype=PAIR_DTYPE)
    offsets = np.empty(ne, dtype=np.uint32)
    counts = np.empty(ne, dtype=np.uint32)
    groups = np.empty(ne, dtype=GROUP_DTYPE)
    tiles = np.empty(ne, dtype=TILE_DTYPE)
    ng, nt, ea, eb = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
    rc = lib().mfbo_group_pairs(_p(pairs), C.c_int64(n), C.c_int64(query_count), C.c_int64(top_k),
                                C.c_int64(num_experts), C.c_int64(tile_expert_count), _p(keys),
                                C.c_int64(0 if keys is None else keys.size), _p(sorted_pairs), _p(offsets),
                                _p(counts), _p(groups), C.byref(ng), _p(tiles), C.byref(nt), C.byref(ea),
                                C.byref(eb))
    if rc != 0:
        raise GroupingError(rc, ea.value, eb.value)
    return dict(sorted_pairs=sorted_pairs[:n], offsets=offsets, counts=counts, groups=groups[:ng.value],
                tiles=tiles[:nt.value])


def reduce_token_major(partial, w_f16, n_tokens, top_k, d) -> np.ndarray:
    partial = _c(partial, np.float32); w = _c(w_f16, np.uint16)
    out = np.empty((n_tokens, d), dtype=np.float32)
    lib().mfbo_reduce_token_major(_p(partial), _p(w), C.c_uint32(n_tokens), C.c_uint32(top_k), C.c_uint32(d), _p(out))
    return out


def rmsnorm(x_f32, w_bf16, eps=1e-6) -> np.ndarray:
    x = _c(x_f32, np.float32)
    rows, d = x.shape
    w = None if w_bf16 is None else _c(w_bf16, np.uint16)
    out = np.empty_like(x)
    lib().mfbo_rmsnorm(_p(x), _p(w), C.c_uint32(rows), C.c_uint32(d), C.c_float(eps), _p(out))
    return out


def rel_l2(actual, reference) -> float:
    a = np.asarray(actual, dtype=np.float64); r = np.asarray(reference, dtype=np.float64)
    return float(np.linalg.norm(a - r) / max(np.linalg.norm(r), 1e-30))

"""Host-side mirror of the reference's MoE kernel-call surface over the C ABI.

The reference keeps this path behind Swift wrapper classes whose ``encode…`` methods put GPU work on a
caller-owned command buffer (Sources/Mference/Kernels/MoE/MoE.swift, Kernels/Prefill/MoE/*.swift).  The
classes here keep those names and argument meanings; a command buffer becomes the current CUDA stream and
an MTLBuffer a torch CUDA tensor (torch is used for device memory and streams only).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib as L


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def expert_layout(bits: int, d: int, f: int, gate_group_size: int = 64):
    """Canonical blob layout: (ExpertOffsets, blob_bytes); gate_group_size 32 gives gate_proj one scale and bias per 32
    elements (DeepSeek V4's conversion, ModelExpertIO.swift:118-135)."""
    off = L.ExpertOffsets()
    total = C.c_uint64()
    L.check(L.load().mfb_expert_layout_gate(bits, d, f, gate_group_size, C.byref(off), C.byref(total)))
    return off, total.value


@dataclass
class MoELayerWeights:
    """Device-resident weights of one layer (MoEExpertOffsets + the slab the streamer owns)."""
    router_w: torch.Tensor                     # bf16 [E, d]
    pool: torch.Tensor                         # uint8 slab of expert slots
    slot_stride: int
    routed_off: L.ExpertOffsets
    shared_blob: Optional[torch.Tensor] = None
    shared_off: Optional[L.ExpertOffsets] = None
    norm_w: Optional[torch.Tensor] = None      # bf16 [d]
    slot_of: Optional[torch.Tensor] = None     # int16 [E]
    logit_bias: Optional[torch.Tensor] = None  # f32 [E]
    per_expert_scale: Optional[torch.Tensor] = None
    correction_bias: Optional[torch.Tensor] = None
    # INT8 gate (router_w then holds uint8 codes [E, d]) and the Qwen shared-expert scalar gate
    router_scales: Optional[torch.Tensor] = None            # bf16 [E, d/64]
    router_biases: Optional[torch.Tensor] = None
    router_effective_scale: Optional[torch.Tensor] = None   # bf16 [d]
    shared_gate_w: Optional[torch.Tensor] = None            # uint8 [d]
    shared_gate_s: Optional[torch.Tensor] = None            # bf16 [d/64]
    shared_gate_b: Optional[torch.Tensor] = None
    gate_group_size: int = 0                                # routed gate_proj scale group: 0 / 64, or 32

    def c_struct(self) -> L.LayerWeightsC:
        w = L.LayerWeightsC()
        w.router_w = self.router_w.data_ptr()
        w.logit_bias = None if self.logit_bias is None else self.logit_bias.data_ptr()
        w.per_expert_scale = None if self.per_expert_scale is None else self.per_expert_scale.data_ptr()
        w.correction_bias = None if self.correction_bias is None else self.correction_bias.data_ptr()
        w.norm_w = None if self.norm_w is None else self.norm_w.data_ptr()
        w.pool = self.pool.data_ptr()
        w.slot_stride = self.slot_stride
        w.slot_of = None if self.slot_of is None else self.slot_of.data_ptr()
        w.shared_blob = None if self.shared_blob is None else self.shared_blob.data_ptr()
        w.routed_off = self.routed_off
        w.shared_off = self.shared_off if self.shared_off is not None else L.ExpertOffsets()
        for name in ("router_scales", "router_biases", "router_effective_scale", "shared_gate_w", "shared_gate_s", "shared_gate_b"):
            t = getattr(self, name)
            setattr(w, name, None if t is None else t.data_ptr())
        w.gate_group_size = self.gate_group_size
        return w


class PrefillMoEGroupingError(ValueError):
    """PrefillMoEGroupingError (PrefillMoEGrouping.swift:52-88): ``case`` names the reference's enum case."""

    def __init__(self, code: int, a: int, b: int):
        self.code, self.case, self.a, self.b = code, L.GROUP_ERROR_NAMES.get(code, str(code)), a, b
        super().__init__(f"{self.case}({a}, {b})")


PAIR_DTYPE = np.dtype([("token", "<u4"), ("expert", "<u4"), ("rank", "<u4"), ("weight_bits", "<u4")])
GROUP_DTYPE = np.dtype([("expert", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])
TILE_DTYPE = np.dtype([("group_start", "<u4"), ("group_count", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])


def group_token_expert_pairs(pairs, query_count: int, top_k: int, num_experts: int, tile_expert_count: int = 16,
                             expert_sort_keys=None) -> dict:
    """PrefillMoEGrouping.groupTokenExpertPairs (PrefillMoEGrouping.swift:90-192) on host arrays."""
    pairs = np.ascontiguousarray(pairs, dtype=PAIR_DTYPE)
    n = pairs.size
    ne = max(int(num_experts), 1)
    keys = None if expert_sort_keys is None else np.ascontiguousarray(expert_sort_keys, dtype=np.uint64)
    sorted_pairs = np.empty(max(n, 1), dtype=PAIR_DTYPE)
    offsets = np.empty(ne, dtype=np.uint32)
    counts = np.empty(ne, dtype=np.uint32)
    groups = np.empty(ne, dtype=GROUP_DTYPE)
    tiles = np.empty(ne, dtype=TILE_DTYPE)
    ng, nt, ea, eb = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
    vp = lambda a: None if a is None else C.c_void_p(a.ctypes.data)
    rc = L.load().mfb_moe_group_host(vp(pairs), n, query_count, top_k, num_experts, tile_expert_count, vp(keys),
                                     0 if keys is None else keys.size, vp(sorted_pairs), vp(offsets), vp(counts),
                                     vp(groups), C.byref(ng), vp(tiles), C.byref(nt), C.byref(ea), C.byref(eb))
    if rc >= L.ERR_GROUP_BASE:
        raise PrefillMoEGroupingError(rc, ea.value, eb.value)
    L.check(rc)
    groups, tiles = groups[:ng.value], tiles[:nt.value]
    return dict(sorted_pairs=sorted_pairs[:n], per_expert_offsets=offsets, per_expert_counts=counts, groups=groups,
                tiles=tiles, query_count=query_count,
                max_pairs_per_expert=int(groups["pair_count"].max()) if groups.size else 0,
                max_pairs_per_tile=int(tiles["pair_count"].max()) if tiles.size else 0,
                max_live_experts_per_tile=int(tiles["group_count"].max()) if tiles.size else 0)


class MoE:
    """The reference's ``MoE`` / ``PrefillRouter`` / ``PrefillGroupedRoutedMoE`` / ``PrefillMoE`` wrappers in one
    handle: shape-specialised at construction (MoE.init, MoE.swift:65-70), owns only its scratch arena."""

    def __init__(self, d: int, f: int, num_experts: int, top_k: int, *, bits: int = 4, shared_bits: int = 4,
                 scale_dtype: int = L.DT_F16, x_dtype: int = L.DT_BF16, activation: int = L.ACT_SILU,
                 router_mode: int = L.ROUTER_SOFTMAX_TOPK, swiglu_limit: float = 0.0, route_scale: float = 1.0,
                 rms_eps: float = 1e-6, max_tokens: int = 1, tensor_core_prefill: bool = False, max_layers: int = 0):
        self.lib = L.load()
        cfg = L.MoEConfig(d, f, num_experts, top_k, bits, shared_bits, 64, scale_dtype, x_dtype, activation,
                          router_mode, swiglu_limit, route_scale, rms_eps, max_tokens,
                          L.FLAG_PREFILL_TENSOR_CORE if tensor_core_prefill else 0, max_layers)
        self.cfg = cfg
        self.handle = C.c_void_p()
        L.check(self.lib.mfb_moe_create(C.byref(cfg), C.byref(self.handle)))
        self.torch_dtype = torch.bfloat16 if x_dtype == L.DT_BF16 else torch.float16

    def close(self):
        if getattr(self, "handle", None) and self.handle.value:
            self.lib.mfb_moe_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- router ------------------------------------------------------------------------------------------
    def encode_router_logits(self, x, router_w, logits, logit_bias=None):
        L.check(self.lib.mfb_router_logits(self.handle, _stream(), _ptr(x), x.stride(0), x.shape[0], _ptr(router_w),
                                           _ptr(logit_bias), _ptr(logits)))

    def encode_router_select(self, logits, out_indices, out_weights, per_expert_scale=None, correction_bias=None):
        L.check(self.lib.mfb_router_select(self.handle, _stream(), _ptr(logits), logits.shape[0],
                                           _ptr(per_expert_scale), _ptr(correction_bias), _ptr(out_indices),
                                           _ptr(out_weights)))

    def encode_router(self, x, weights: MoELayerWeights, out_indices, out_weights):
        """MoE.encodeRouterGemma4 (one row) / PrefillRouter.encodeGemma4Block (a block of rows)."""
        w = weights.c_struct()
        L.check(self.lib.mfb_router_topk(self.handle, _stream(), _ptr(x), x.stride(0), x.shape[0], C.byref(w),
                                         _ptr(out_indices), _ptr(out_weights)))

    def encode_slot_lookup(self, indices, table, slot_stride, slot_offsets, all_hit):
        """MoE.encodeSlotLookup."""
        L.check(self.lib.mfb_slot_lookup(self.handle, _stream(), _ptr(indices), indices.shape[0], _ptr(table),
                                         slot_stride, _ptr(slot_offsets), _ptr(all_hit)))

    # ---- decode ------------------------------------------------------------------------------------------
    def encode_experts(self, weights, x, indices, routing_weights, active_slots: Optional[Sequence[int]] = None,
                       with_shared: bool = True):
        """encodeRoutedPersistentPhase1(Subset)U16Load + the down projections of the chosen rank slots."""
        w = weights.c_struct()
        arr = None
        n = 0
        if active_slots is not None:
            n = len(active_slots)
            arr = (C.c_uint32 * max(n, 1))(*active_slots)
        L.check(self.lib.mfb_moe_experts(self.handle, _stream(), C.byref(w), _ptr(x), x.stride(0), x.shape[0],
                                         _ptr(indices), _ptr(routing_weights), arr, n, 1 if with_shared else 0))

    def encode_combine(self, routing_weights, y, residual=None, with_shared: bool = True):
        """encodeRoutedPersistentPhase2Reduce's weighted reduce: residual first, rank order."""
        L.check(self.lib.mfb_moe_combine(self.handle, _stream(), y.shape[0], _ptr(routing_weights),
                                         1 if with_shared else 0, _ptr(residual), _ptr(y)))

    def encode_decode(self, weights, x, indices, routing_weights, y, residual=None):
        w = weights.c_struct()
        L.check(self.lib.mfb_moe_decode(self.handle, _stream(), C.byref(w), _ptr(x), x.stride(0), x.shape[0],
                                        _ptr(indices), _ptr(routing_weights), _ptr(residual), _ptr(y)))

    def encode_layer(self, weights, h_in, h_out):
        w = weights.c_struct()
        L.check(self.lib.mfb_moe_layer(self.handle, _stream(), C.byref(w), _ptr(h_in), _ptr(h_out), h_in.shape[0]))

    def make_stack(self, layers: Sequence[MoELayerWeights]):
        arr = (L.LayerWeightsC * len(layers))(*[lw.c_struct() for lw in layers])
        return arr

    def encode_stack(self, stack, hidden):
        L.check(self.lib.mfb_moe_stack(self.handle, _stream(), stack, len(stack), _ptr(hidden), hidden.shape[0]))

    def encode_stack_rows(self, stack, rows):
        """rows: [n_layers, n_tokens, d]; layer l transforms rows[l] in place, layers run one after the other."""
        L.check(self.lib.mfb_moe_stack_rows(self.handle, _stream(), stack, len(stack), _ptr(rows), rows.stride(0),
                                            rows.shape[1]))

    # ---- prefill -----------------------------------------------------------------------------------------
    def encode_group(self, indices, routing_weights):
        """Device-side PrefillMoEGrouping: returns (sorted_pairs[int32 P,4], offsets, counts, groups[int32 E,3], n_groups)."""
        T, K = indices.shape
        E = self.cfg.num_experts
        dev = indices.device
        sorted_pairs = torch.empty((max(T * K, 1), 4), dtype=torch.int32, device=dev)
        offsets = torch.empty(E, dtype=torch.int32, device=dev)
        counts = torch.empty(E, dtype=torch.int32, device=dev)
        groups = torch.empty((E + 1, 3), dtype=torch.int32, device=dev)
        n_groups = torch.zeros(1, dtype=torch.int32, device=dev)
        L.check(self.lib.mfb_moe_group(self.handle, _stream(), _ptr(indices), _ptr(routing_weights), T,
                                       _ptr(sorted_pairs), _ptr(offsets), _ptr(counts), _ptr(groups), _ptr(n_groups)))
        return sorted_pairs[:T * K], offsets, counts, groups, n_groups

    def encode_prefill_grouped(self, weights, x, sorted_pairs, groups, n_groups, partial):
        """PrefillGroupedRoutedMoE.encodeStreamedBatched over all groups; partial is f32 [T*top_k, d]."""
        w = weights.c_struct()
        L.check(self.lib.mfb_moe_prefill_grouped(self.handle, _stream(), C.byref(w), _ptr(x), x.stride(0), x.shape[0],
                                                 _ptr(sorted_pairs), _ptr(groups), _ptr(n_groups), _ptr(partial)))

    def encode_prefill_accumulate_f32(self, weights, x, sorted_pairs, groups, n_groups, pair_weights, acc):
        """The Inkling batched expert application (inkling_prefill_expert_act / _down_accum, prefill.metal:654-746):
        acc (f32 [T, d], read and written) += the routed experts' rows, expert by expert, with f32 pair weights [T, top_k]."""
        w = weights.c_struct()
        L.check(self.lib.mfb_moe_prefill_accumulate_f32(self.handle, _stream(), C.byref(w), _ptr(x), x.stride(0), x.shape[0],
                                                        _ptr(sorted_pairs), _ptr(groups), _ptr(n_groups), _ptr(pair_weights),
                                                        _ptr(acc)))

    def encode_reduce_token_major(self, partial, routing_weights, y, residual=None):
        """PrefillMoE.encodeReduceTokenMajor."""
        L.check(self.lib.mfb_moe_reduce(self.handle, _stream(), _ptr(partial), _ptr(routing_weights), y.shape[0],
                                        _ptr(residual), _ptr(y)))

    def encode_layer_prefill(self, weights, h_in, h_out):
        w = weights.c_struct()
        L.check(self.lib.mfb_moe_layer_prefill(self.handle, _stream(), C.byref(w), _ptr(h_in), _ptr(h_out), h_in.shape[0]))

    # ---- glue --------------------------------------------------------------------------------------------
    def encode_rmsnorm(self, x, out, weight=None):
        L.check(self.lib.mfb_rmsnorm(self.handle, _stream(), _ptr(x), _ptr(weight), x.shape[0], _ptr(out)))

    def encode_residual_add(self, a, b, out):
        L.check(self.lib.mfb_residual_add(self.handle, _stream(), _ptr(a), _ptr(b), a.numel(), _ptr(out)))

    def set_generic(self, on):
        """True / 1: route every call through the generic kernels instead of the shape-specialised fast ones.
        2: fast kernels, but a stack runs layer by layer and phase by phase instead of as one fused launch."""
        L.check(self.lib.mfb_moe_set_generic(self.handle, int(on)))

    def set_trace(self, stamps):
        """Attach (or detach with None) a zeroed uint64 [n_layers + 17, 8] CUDA tensor: per-phase global-timer stamps
        of every layer, then 17 rows of cycle counters of CTA 0 (see mfb_moe_set_trace in the header)."""
        L.check(self.lib.mfb_moe_set_trace(self.handle, _ptr(stamps)))

    def partial_rows(self, n_tokens: int) -> torch.Tensor:
        """fp32 [n_tokens, top_k + 1, d] view of the handle's down-projection rows (slot top_k = shared expert) as the
        last decode / layer / stack call left them (mfb_moe_partial_rows)."""
        p = C.c_void_p()
        L.check(self.lib.mfb_moe_partial_rows(self.handle, C.byref(p)))
        shape = (n_tokens, self.cfg.top_k + 1, self.cfg.d)

        class _Ptr:
            pass
        holder = _Ptr()
        holder.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (p.value, False), "version": 2}
        return torch.as_tensor(holder, device="cuda")

    def selftest_wait(self, limit_cycles: int = 2_000_000):
        """Launches the bounded-wait self-test: device_status() reports the timeout bit afterwards."""
        L.check(self.lib.mfb_moe_selftest_wait(self.handle, _stream(), limit_cycles))

    def device_status(self) -> int:
        st = C.c_uint32()
        rc = self.lib.mfb_moe_device_status(self.handle, _stream(), C.byref(st))
        if rc not in (L.OK, L.ERR_DEVICE_STATUS):
            L.check(rc)
        return st.value


def encode_router_static(x, router_w, out_indices, out_weights, *, top_k: int, x_dtype: int = L.DT_BF16,
                         router_mode: int = L.ROUTER_SOFTMAX_TOPK, logit_bias=None, per_expert_scale=None,
                         correction_bias=None, route_scale: float = 1.0):
    """Router top-k for at most 64 rows without a handle and without allocating (mfb_router_topk_static): the
    logits scratch is a fixed device array inside the library.  Calls that may overlap in time race on it."""
    L.check(L.load().mfb_router_topk_static(_stream(), _ptr(x), x_dtype, x.stride(0), x.shape[0], x.shape[1], _ptr(router_w),
                                            _ptr(logit_bias), router_w.shape[0], top_k, router_mode,
                                            _ptr(per_expert_scale), _ptr(correction_bias), route_scale,
                                            _ptr(out_indices), _ptr(out_weights)))


# --------------------------------------------------------------------------------------------- synthetic layers

def synth_normal(root: int, label: str, n: int, *, mean=0.0, std=1.0, absolute=False, dtype=L.DT_BF16,
                 device="cuda") -> torch.Tensor:
    tdt = {L.DT_BF16: torch.bfloat16, L.DT_F16: torch.float16, L.DT_F32: torch.float32}[dtype]
    out = torch.empty(n, dtype=tdt, device=device)
    L.check(L.load().mfb_synth_normal(_stream(), root, label.encode(), n, mean, std, 1 if absolute else 0, dtype,
                                      _ptr(out)))
    return out


def synth_layer(root: int, layer: int, d: int, f: int, num_experts: int, *, bits=4, shared_bits=4,
                scale_dtype=L.DT_F16, device="cuda", with_norm=True) -> MoELayerWeights:
    """One layer of seeded synthetic weights generated on the device (uniform codes, |N(0,0.02)| scales,
    N(0,0.01) biases, N(0,0.02) bf16 router, RMSNorm weight 1)."""
    lib = L.load()
    off, blob = expert_layout(bits, d, f)
    stride = (blob + 255) // 256 * 256
    pool = torch.empty(num_experts * stride, dtype=torch.uint8, device=device)
    L.check(lib.mfb_synth_expert_pool(_stream(), root, layer, 0, num_experts, 0, bits, scale_dtype, d, f, _ptr(pool), stride))
    shared_blob = shared_off = None
    if shared_bits:
        shared_off, sblob = expert_layout(shared_bits, d, f)
        shared_blob = torch.empty(sblob, dtype=torch.uint8, device=device)
        L.check(lib.mfb_synth_expert_pool(_stream(), root, layer, 0, 1, 1, shared_bits, scale_dtype, d, f, _ptr(shared_blob), 0))
    router = synth_normal(root, f"L{layer}.router", num_experts * d, std=0.02, dtype=L.DT_BF16, device=device).view(num_experts, d)
    norm_w = torch.ones(d, dtype=torch.bfloat16, device=device) if with_norm else None
    return MoELayerWeights(router_w=router, pool=pool, slot_stride=stride, routed_off=off, shared_blob=shared_blob,
                           shared_off=shared_off, norm_w=norm_w)

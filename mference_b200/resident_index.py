"""Reader (and a writer for synthetic models) of a model directory's ``model_weights.bin``: a 24-byte header, a table of
72-byte tensor entries, a string table with the tensor names, padding, then the tensor bytes.

The layout is that of the reference's resident index (Sources/Mference/Infrastructure/ModelIO/ResidentIndex.swift:1-160):
header = (index_size, resident_size, entry_count) as little-endian u64, index_size counting everything in front of the
tensor region; an entry = name offset u32 (absolute in the file), name length u16, dtype u8, one reserved byte, file
offset u64, size u64, four u32 of logical shape, then offset and size of the scales and of the biases (0 = none).
dtype 0 marks an affine group-quantised tensor (packed codes + bf16 scales + bf16 biases per 64 elements), 1 a bf16
tensor.  What this path needs from the file are the MoE tensors of a layer under the reference's Qwen 3.6 names
(Tests/Mference/Core/Runtime/QwenToySynthetic.swift:64-90): ``mlp.gate`` (INT8 router), ``mlp.shared_expert_gate``
(INT8 scalar gate), the shared expert's three projections, and ``post_attention_layernorm`` (the norm in front of the
MoE block).
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from .packed_experts import IndexCorrupt, MissingFile

HEADER_BYTES = 24
ENTRY_BYTES = 72
DTYPE_AFFINE, DTYPE_BF16 = 0, 1
_ENTRY = struct.Struct("<IHBBQQIIIIQQQQ")
assert _ENTRY.size == ENTRY_BYTES


@dataclass(frozen=True)
class ResidentIndexEntry:
    name: str
    dtype: int
    file_offset: int
    size_bytes: int
    shape: Tuple[int, int, int, int]
    scale_offset: int
    scale_size: int
    bias_offset: int
    bias_size: int


class ResidentIndex:
    """The parsed index of one ``model_weights.bin`` plus positional reads of tensor bytes."""

    def __init__(self, path: str):
        if not os.path.exists(path):
            raise MissingFile(os.path.basename(path))
        self.path = path
        with open(path, "rb") as fh:
            head = fh.read(HEADER_BYTES)
            if len(head) != HEADER_BYTES:
                raise IndexCorrupt(f"short read for IndexHeader ({len(head)}/{HEADER_BYTES})")
            self.index_size, self.resident_size, self.entry_count = struct.unpack("<QQQ", head)
            if self.index_size < HEADER_BYTES:
                raise IndexCorrupt(f"indexSize {self.index_size} < header size {HEADER_BYTES}")
            table_end = HEADER_BYTES + self.entry_count * ENTRY_BYTES
            if table_end > self.index_size:
                raise IndexCorrupt(f"header+entries ({table_end}) > indexSize {self.index_size}")
            fh.seek(0)
            region = fh.read(self.index_size)
            if len(region) != self.index_size:
                raise IndexCorrupt(f"short read for index region ({len(region)}/{self.index_size})")
        self.entries: Dict[str, ResidentIndexEntry] = {}
        for i in range(self.entry_count):
            (name_off, name_len, dtype, _reserved, file_off, size, s0, s1, s2, s3, sc_off, sc_size, b_off,
             b_size) = _ENTRY.unpack_from(region, HEADER_BYTES + i * ENTRY_BYTES)
            if name_off < HEADER_BYTES or name_off + name_len > self.index_size:
                raise IndexCorrupt(f"entry {i} name range [{name_off}, {name_off + name_len}) out of index region "
                                   f"[{HEADER_BYTES}, {self.index_size})")
            name = region[name_off:name_off + name_len].decode("utf-8", errors="replace")
            if name in self.entries:
                raise IndexCorrupt(f"duplicate tensor name {name}")
            self.entries[name] = ResidentIndexEntry(name, dtype, file_off, size, (s0, s1, s2, s3), sc_off, sc_size, b_off, b_size)
        file_size = os.path.getsize(path)
        if file_size != self.index_size + self.resident_size:
            raise IndexCorrupt(f"model_weights.bin size {file_size} != indexSize {self.index_size} + residentSize {self.resident_size}")

    def entry(self, name: str) -> ResidentIndexEntry:
        if name not in self.entries:
            raise IndexCorrupt(f"no IndexEntry named {name} in model_weights.bin")
        return self.entries[name]

    def _pread(self, offset: int, size: int) -> np.ndarray:
        if offset < self.index_size or offset + size > self.index_size + self.resident_size:
            raise IndexCorrupt(f"tensor bytes [{offset}, {offset + size}) outside the resident region")
        with open(self.path, "rb") as fh:
            fh.seek(offset)
            data = fh.read(size)
        if len(data) != size:
            raise IndexCorrupt(f"short read of {size} bytes at {offset}")
        return np.frombuffer(data, dtype=np.uint8)

    def tensor(self, name: str):
        """(codes or bf16 bits as uint8, scales bits uint16 or None, biases bits uint16 or None, entry)."""
        e = self.entry(name)
        w = self._pread(e.file_offset, e.size_bytes)
        s = self._pread(e.scale_offset, e.scale_size).view(np.uint16) if e.scale_size else None
        b = self._pread(e.bias_offset, e.bias_size).view(np.uint16) if e.bias_size else None
        return w, s, b, e


def write_resident_file(path: str, tensors: Sequence[Tuple[str, int, Tuple[int, ...], np.ndarray, Optional[np.ndarray],
                                                           Optional[np.ndarray]]], page: int = 16384) -> None:
    """Writes a ``model_weights.bin`` holding `tensors` = (name, dtype, shape, weight bytes, scales bits, biases bits) in
    the order given: index (padded to `page` bytes), then for each tensor its weight bytes, scales, biases."""
    names = [t[0].encode("utf-8") for t in tensors]
    table_base = HEADER_BYTES + len(tensors) * ENTRY_BYTES
    index_size = table_base + sum(len(n) for n in names)
    index_size = (index_size + page - 1) // page * page
    entries, payload, cursor, name_cursor = [], [], index_size, table_base
    for (name, dtype, shape, w, s, b), raw in zip(tensors, names):
        w = np.ascontiguousarray(w).view(np.uint8).reshape(-1)
        sb = None if s is None else np.ascontiguousarray(s).view(np.uint8).reshape(-1)
        bb = None if b is None else np.ascontiguousarray(b).view(np.uint8).reshape(-1)
        w_off = cursor
        s_off = w_off + w.size if sb is not None else 0
        b_off = (s_off + sb.size) if bb is not None else 0
        shape4 = tuple(list(shape) + [0] * (4 - len(shape)))
        entries.append(_ENTRY.pack(name_cursor, len(raw), dtype, 0, w_off, w.size, *shape4, s_off, 0 if sb is None else sb.size,
                                   b_off, 0 if bb is None else bb.size))
        payload += [w] + ([sb] if sb is not None else []) + ([bb] if bb is not None else [])
        cursor += w.size + (0 if sb is None else sb.size) + (0 if bb is None else bb.size)
        name_cursor += len(raw)
    resident_size = cursor - index_size
    with open(path, "wb") as fh:
        fh.write(struct.pack("<QQQ", index_size, resident_size, len(tensors)))
        fh.write(b"".join(entries))
        fh.write(b"".join(names))
        fh.write(b"\0" * (index_size - fh.tell()))
        for p in payload:
            fh.write(p.tobytes())


def qwen_moe_tensor_names(layer: int) -> Dict[str, str]:
    """The reference's tensor names of the MoE block of one Qwen 3.6 layer."""
    p = f"language_model.model.layers.{layer}"
    return {"norm": f"{p}.post_attention_layernorm.weight", "router": f"{p}.mlp.gate.weight",
            "shared_gate": f"{p}.mlp.shared_expert_gate.weight", "shared_gate_proj": f"{p}.mlp.shared_expert.gate_proj.weight",
            "shared_up_proj": f"{p}.mlp.shared_expert.up_proj.weight", "shared_down_proj": f"{p}.mlp.shared_expert.down_proj.weight"}


def layer_resident_weights(index: ResidentIndex, layer: int, d: int, f: int, num_experts: int, device="cuda"):
    """The resident MoE tensors of `layer` on the device, as the keyword arguments ``MoELayerWeights`` takes beside the
    expert pool: the INT8 router with its scales and biases, the RMSNorm weight, the shared expert's scalar gate, and the
    shared expert as one blob in the expert layout (gate W,S,B, up W,S,B, down W,S,B).  The shared expert must be stored
    as 4-bit codes (rows of d/2 and f/2 bytes); other widths are rejected."""
    import torch
    from .moe import expert_layout
    names = qwen_moe_tensor_names(layer)

    def dev(a, dtype=None):
        t = torch.from_numpy(np.array(a, copy=True)).to(device)   # file reads come back read-only
        return t if dtype is None else t.view(dtype)

    rw, rs, rb, re_ = index.tensor(names["router"])
    if re_.dtype != DTYPE_AFFINE or rw.size != num_experts * d:
        raise IndexCorrupt(f"{names['router']}: expected an INT8 affine tensor of {num_experts} x {d} codes, got {rw.size} bytes")
    gw, gs, gb, _ = index.tensor(names["shared_gate"])
    if gw.size != d:
        raise IndexCorrupt(f"{names['shared_gate']}: expected {d} INT8 codes, got {gw.size} bytes")
    nw, _, _, ne = index.tensor(names["norm"])
    if ne.dtype != DTYPE_BF16 or nw.size != d * 2:
        raise IndexCorrupt(f"{names['norm']}: expected {d} bf16 values")
    off, blob_bytes = expert_layout(4, d, f)
    blob = np.zeros(blob_bytes, dtype=np.uint8)
    fields = [int(getattr(off, n)) for n, _ in off._fields_]
    for i, key in enumerate(("shared_gate_proj", "shared_up_proj", "shared_down_proj")):
        w, s, b, e = index.tensor(names[key])
        rows, cols = (f, d) if i < 2 else (d, f)
        if w.size != rows * cols // 2 or s is None or b is None:
            raise IndexCorrupt(f"{names[key]}: expected 4-bit codes of {rows} x {cols} with scales and biases, got {w.size} bytes")
        for part, o in ((w, fields[3 * i]), (s.view(np.uint8), fields[3 * i + 1]), (b.view(np.uint8), fields[3 * i + 2])):
            blob[o:o + part.size] = part
    return dict(router_w=dev(rw).view(num_experts, d), router_scales=dev(rs, torch.bfloat16), router_biases=dev(rb, torch.bfloat16),
                norm_w=dev(nw.view(np.int16), torch.bfloat16), shared_gate_w=dev(gw), shared_gate_s=dev(gs, torch.bfloat16),
                shared_gate_b=dev(gb, torch.bfloat16), shared_blob=dev(blob), shared_off=off)

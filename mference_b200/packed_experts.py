"""Reader (and a writer for synthetic layers) of a model directory's ``packed_experts/``: ``layout.json`` plus one
``layer_XX.bin`` per MoE layer, each a sequence of fixed-stride expert blobs (gate W,S,B, up W,S,B, down W,S,B).

Follows the reference's ``PackedExpertsLayoutReader.load`` (Sources/Mference/Infrastructure/ModelIO/
PackedExpertsLayout.swift:48-148): the same keys, defaults and rejections; ``routed_expert_offsets`` is
``Model.routedExpertOffsets`` (Sources/Mference/Runtime/Inference/ModelExpertIO.swift:20-35).  What the reference
hands to its pread streamer goes here into pinned host tensors for ``ExpertPool`` (partial residency) or in one piece
into HBM (full residency, the normal case with 180 GB).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from . import _lib as L

DEFAULT_MAX_BYTES = 64 * 1024 * 1024      # cap on layout.json (a 40-layer, 256-expert layout is about 22 MB)
ROLES = ("gate", "gate_scales", "gate_biases", "up", "up_scales", "up_biases", "down", "down_scales", "down_biases")


class ModelError(Exception):
    pass


class MissingFile(ModelError):
    def __init__(self, name: str):
        self.name = name
        super().__init__(f"missing file: {name}")


class IndexCorrupt(ModelError):
    def __init__(self, detail: str):
        self.detail = detail
        super().__init__(f"index corrupt: {detail}")


@dataclass(frozen=True)
class SubTensorEntry:
    offset: int      # relative to the start of the expert blob
    size: int        # bytes


@dataclass(frozen=True)
class ExpertEntry:
    expert: int      # logical routed-expert id (what the router emits)
    offset: int      # byte offset of the blob inside its layer file
    size: int        # bytes of the blob (== expert_stride)
    sub_tensors: Dict[str, SubTensorEntry] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerLayout:
    layer: int
    file: str        # basename, e.g. "layer_00.bin"
    experts: List[ExpertEntry]


@dataclass(frozen=True)
class PackedExpertsLayout:
    expert_stride: int
    num_layers: int
    experts_per_layer: int
    layers: List[LayerLayout]

    def expert(self, layer: int, expert: int) -> ExpertEntry:
        return self.layers[layer].experts[expert]

    def routed_expert_offsets(self, layer: int) -> L.ExpertOffsets:
        """The nine byte offsets common to all experts of a layer, taken from expert 0; an absent role reads 0."""
        sub = self.expert(layer, 0).sub_tensors
        return L.ExpertOffsets(*[sub[r].offset if r in sub else 0 for r in ROLES])

    def routed_expert_physical_offsets(self, layer: int) -> List[int]:
        return [e.offset for e in self.layers[layer].experts]


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _u64(v) -> Optional[int]:
    # the reference accepts any JSON number here and takes its unsigned 64-bit value
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        return None
    return int(v)


class PackedExpertsLayoutReader:
    @staticmethod
    def load(directory: str, max_bytes: int = DEFAULT_MAX_BYTES) -> PackedExpertsLayout:
        path = os.path.join(directory, "packed_experts", "layout.json")
        if not os.path.isfile(path):
            raise MissingFile("packed_experts/layout.json")
        size = os.path.getsize(path)
        if size > max_bytes:
            raise IndexCorrupt(f"layout.json size {size} exceeds metadata cap {max_bytes}")
        try:
            with open(path, "rb") as fh:
                root = json.loads(fh.read())
        except (ValueError, UnicodeDecodeError) as e:
            raise IndexCorrupt(f"layout.json: {e}") from None
        if not isinstance(root, dict):
            root = {}
        stride, n_layers = _u64(root.get("expertStride")), root.get("numLayers")
        per_layer, layers_arr = root.get("expertsPerLayer"), root.get("layers")
        if stride is None or not _is_int(n_layers) or not _is_int(per_layer) or not isinstance(layers_arr, list) \
                or not all(isinstance(x, dict) for x in layers_arr):
            raise IndexCorrupt("layout.json: missing top-level keys")
        layers: List[LayerLayout] = []
        for obj in layers_arr:
            idx, file, experts_arr = obj.get("layer"), obj.get("file"), obj.get("experts")
            if not _is_int(idx) or not isinstance(file, str) or not isinstance(experts_arr, list) \
                    or not all(isinstance(x, dict) for x in experts_arr):
                raise IndexCorrupt("layout.json: malformed layer entry")
            if not experts_arr:      # a leading dense layer: listed, no experts, no blob file
                layers.append(LayerLayout(idx, file, []))
                continue
            experts: List[Optional[ExpertEntry]] = [None] * per_layer
            for eobj in experts_arr:
                off, sz, tensors = _u64(eobj.get("offset")), _u64(eobj.get("size")), eobj.get("tensors")
                if off is None or sz is None or not isinstance(tensors, dict) \
                        or not all(isinstance(t, dict) for t in tensors.values()):
                    raise IndexCorrupt("layout.json: malformed expert entry")
                subs: Dict[str, SubTensorEntry] = {}
                for role, t in tensors.items():
                    toff, tsz, shape = _u64(t.get("offset")), _u64(t.get("size")), t.get("shape")
                    if toff is None or tsz is None or not isinstance(t.get("dtype"), str) \
                            or not isinstance(shape, list) or not all(_is_int(x) for x in shape):
                        raise IndexCorrupt(f"layout.json: malformed tensor {role}")
                    if "bits" in t and not _is_int(t["bits"]):
                        raise IndexCorrupt(f"layout.json: malformed tensor bits {role}")
                    subs[role] = SubTensorEntry(toff, tsz)
                eid = eobj.get("expert")
                if not _is_int(eid):
                    eid = sum(1 for x in experts if x is not None)      # no id given: the next one in file order
                if not 0 <= eid < per_layer:
                    raise IndexCorrupt("layout.json: expert id out of range")
                rank = eobj.get("physicalRank")
                if _is_int(rank) and not 0 <= rank < per_layer:
                    raise IndexCorrupt("layout.json: physicalRank out of range")
                experts[eid] = ExpertEntry(eid, off, sz, subs)
            if any(x is None for x in experts):
                raise IndexCorrupt("layout.json: missing expert entries")
            layers.append(LayerLayout(idx, file, experts))      # type: ignore[arg-type]
        return PackedExpertsLayout(stride, n_layers, per_layer, layers)


class PackedLayerFile:
    """One ``layer_XX.bin`` opened for positional reads (the reference's pread streamer reads the same ranges)."""

    def __init__(self, directory: str, layout: PackedExpertsLayout, layer: int):
        self.layout, self.layer = layout, layer
        entry = layout.layers[layer]
        self.experts = entry.experts
        self.path = os.path.join(directory, "packed_experts", entry.file)
        if not os.path.isfile(self.path):
            raise MissingFile(f"packed_experts/{entry.file}")
        self.fd = os.open(self.path, os.O_RDONLY)
        size = os.fstat(self.fd).st_size
        for e in self.experts:
            if e.size != layout.expert_stride or e.offset + e.size > size:
                self.close()
                raise IndexCorrupt(f"{entry.file}: expert {e.expert} at {e.offset}+{e.size} does not fit the file ({size} bytes, "
                                   f"stride {layout.expert_stride})")

    def close(self) -> None:
        if getattr(self, "fd", None) is not None:
            os.close(self.fd)
            self.fd = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def read_expert_into(self, expert: int, out) -> None:
        """Reads the blob of logical expert ``expert`` into ``out``, a host uint8 tensor of at least expert_stride bytes."""
        e = self.experts[expert]
        view = memoryview(out.numpy()).cast("B")[:e.size]
        done = 0
        while done < e.size:
            n = os.preadv(self.fd, [view[done:]], e.offset + done)
            if n <= 0:
                raise IndexCorrupt(f"short read of expert {expert} in {self.path}")
            done += n

    def host_blob(self, expert: int):
        """The expert's blob as a pinned uint8 tensor (a source for ``ExpertPool`` fills)."""
        import torch
        t = torch.empty(self.layout.expert_stride, dtype=torch.uint8).pin_memory()
        self.read_expert_into(expert, t)
        return t

    def host_blobs(self, experts: Optional[Sequence[int]] = None) -> dict:
        return {e: self.host_blob(e) for e in (range(len(self.experts)) if experts is None else experts)}

    def load_resident(self, device="cuda"):
        """The whole layer in HBM, experts in logical order at ``expert_stride`` (whatever their order in the file):
        two pinned staging buffers, reads overlapping the copies."""
        import torch
        stride, n = self.layout.expert_stride, len(self.experts)
        slab = torch.empty(n * stride, dtype=torch.uint8, device=device)
        stage = [torch.empty(stride, dtype=torch.uint8).pin_memory() for _ in range(2)]
        free = [torch.cuda.Event(), torch.cuda.Event()]
        used = [False, False]
        for e in range(n):
            b = e & 1
            if used[b]:
                free[b].synchronize()      # the copy out of this buffer has finished
            self.read_expert_into(e, stage[b])
            slab[e * stride:(e + 1) * stride].copy_(stage[b], non_blocking=True)
            free[b].record()
            used[b] = True
        torch.cuda.current_stream().synchronize()
        return slab


def layer_weights_from_packed(directory: str, layout: PackedExpertsLayout, layer: int, router_w, **replicated):
    """A fully resident ``MoELayerWeights`` for ``layer``: the expert slab from its layer file; router, norm and
    shared-expert tensors (which live in the model's other files) are passed through."""
    from .moe import MoELayerWeights
    with PackedLayerFile(directory, layout, layer) as fh:
        slab = fh.load_resident(router_w.device)
    return MoELayerWeights(router_w=router_w, pool=slab, slot_stride=layout.expert_stride,
                           routed_off=layout.routed_expert_offsets(layer), **replicated)


def write_packed_experts(directory: str, layers: Sequence[dict], expert_stride: Optional[int] = None) -> PackedExpertsLayout:
    """Writes ``packed_experts/`` for synthetic layers (tests, exporting seeded weights).  Each layer is a dict with
    ``pool`` (uint8 tensor, experts at ``slot_stride``), ``slot_stride``, ``offsets`` (ExpertOffsets), ``d``, ``f``,
    ``bits``, optional ``scale_dtype`` name ("F16" / "BF16") and ``physical_order`` (logical ids in file order)."""
    out_dir = os.path.join(directory, "packed_experts")
    os.makedirs(out_dir, exist_ok=True)
    blob_max = 0
    for ly in layers:
        d, f, bits = ly["d"], ly["f"], ly["bits"]
        blob_max = max(blob_max, ly["offsets"].down_b + d * (f // 64) * 2)
    stride = expert_stride or (blob_max + 4095) // 4096 * 4096
    if stride < blob_max:
        raise ValueError(f"expert_stride {stride} is smaller than a blob ({blob_max} bytes)")
    root = {"expertStride": stride, "numLayers": len(layers), "expertsPerLayer": 0, "layers": []}
    for li, ly in enumerate(layers):
        d, f, bits, off = ly["d"], ly["f"], ly["bits"], ly["offsets"]
        sdt = ly.get("scale_dtype", "F16")
        pool = ly["pool"].cpu().numpy()
        n = pool.size // ly["slot_stride"]
        root["expertsPerLayer"] = max(root["expertsPerLayer"], n)
        order = list(ly.get("physical_order") or range(n))
        name = f"layer_{li:02d}.bin"

        def tensors():
            t = {}
            for role, rows, k, base in (("gate", f, d, (off.gate_w, off.gate_s, off.gate_b)),
                                        ("up", f, d, (off.up_w, off.up_s, off.up_b)),
                                        ("down", d, f, (off.down_w, off.down_s, off.down_b))):
                t[role] = {"offset": base[0], "size": rows * k * bits // 8, "dtype": "U32", "shape": [rows, k * bits // 32], "bits": bits}
                t[role + "_scales"] = {"offset": base[1], "size": rows * (k // 64) * 2, "dtype": sdt, "shape": [rows, k // 64]}
                t[role + "_biases"] = {"offset": base[2], "size": rows * (k // 64) * 2, "dtype": sdt, "shape": [rows, k // 64]}
            return t

        entries = [None] * n
        with open(os.path.join(out_dir, name), "wb") as fh:
            for rank, e in enumerate(order):
                blob = pool[e * ly["slot_stride"]:e * ly["slot_stride"] + off.down_b + d * (f // 64) * 2].tobytes()
                fh.write(blob + b"\0" * (stride - len(blob)))
                entries[e] = {"expert": e, "physicalRank": rank, "offset": rank * stride, "size": stride, "tensors": tensors()}
        root["layers"].append({"layer": li, "file": name, "experts": entries})
    with open(os.path.join(out_dir, "layout.json"), "w") as fh:
        json.dump(root, fh, sort_keys=True)
    return PackedExpertsLayoutReader.load(directory)

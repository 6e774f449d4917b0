"""packed_experts/ reader: the cases of the reference's Tests/Mference/Core/Infrastructure/ModelIO/
PackedExpertsLayoutTests.swift (toy layout, missing file, metadata cap) plus the malformed-entry rejections of
PackedExpertsLayoutReader.load, and on the GPU a synthetic layer written to disk, read back and run."""
import json
import os

import numpy as np
import pytest

from mference_b200 import _lib as L
from mference_b200.packed_experts import (IndexCorrupt, MissingFile, PackedExpertsLayoutReader, PackedLayerFile,
                                          layer_weights_from_packed, write_packed_experts)


def _tensor(offset, size, dtype, shape, **kw):
    return dict(offset=offset, size=size, dtype=dtype, shape=shape, **kw)


def toy_root():
    tensors = {"gate": _tensor(0, 4096, "U32", [64, 64], bits=4), "gate_scales": _tensor(4096, 256, "BF16", [64, 1])}
    return {"expertStride": 16384, "numLayers": 1, "expertsPerLayer": 2,
            "layers": [{"layer": 0, "file": "layer_00.bin",
                        "experts": [{"expert": 0, "offset": 0, "size": 16384, "tensors": tensors},
                                    {"expert": 1, "physicalRank": 1, "offset": 16384, "size": 16384, "tensors": tensors}]}]}


def write_root(tmp_path, root):
    os.makedirs(tmp_path / "packed_experts", exist_ok=True)
    (tmp_path / "packed_experts" / "layout.json").write_text(json.dumps(root, sort_keys=True))
    return str(tmp_path)


def test_toy_layout_decodes(tmp_path):
    layout = PackedExpertsLayoutReader.load(write_root(tmp_path, toy_root()))
    assert (layout.expert_stride, layout.num_layers, layout.experts_per_layer, len(layout.layers)) == (16384, 1, 2, 1)
    e0, e1 = layout.expert(0, 0), layout.expert(0, 1)
    assert (e0.offset, e0.size, e0.sub_tensors["gate"].offset, e0.sub_tensors["gate_scales"].offset) == (0, 16384, 0, 4096)
    assert (e1.offset, e1.expert) == (16384, 1)
    off = layout.routed_expert_offsets(0)
    assert (off.gate_w, off.gate_s, off.gate_b, off.down_w) == (0, 4096, 0, 0)      # absent roles read 0
    assert layout.routed_expert_physical_offsets(0) == [0, 16384]


def test_missing_layout_and_metadata_cap(tmp_path):
    os.makedirs(tmp_path / "packed_experts")
    with pytest.raises(MissingFile):
        PackedExpertsLayoutReader.load(str(tmp_path))
    (tmp_path / "packed_experts" / "layout.json").write_bytes(b" " * 64)
    with pytest.raises(IndexCorrupt) as e:
        PackedExpertsLayoutReader.load(str(tmp_path), max_bytes=16)
    assert "metadata cap" in e.value.detail
    with pytest.raises(IndexCorrupt):                                      # blank file: not JSON
        PackedExpertsLayoutReader.load(str(tmp_path))


@pytest.mark.parametrize("mutate,needle", [
    (lambda r: r.pop("expertStride"), "missing top-level keys"),
    (lambda r: r.__setitem__("numLayers", "1"), "missing top-level keys"),
    (lambda r: r["layers"][0].pop("file"), "malformed layer entry"),
    (lambda r: r["layers"][0]["experts"][0].pop("size"), "malformed expert entry"),
    (lambda r: r["layers"][0]["experts"][0]["tensors"]["gate"].pop("dtype"), "malformed tensor gate"),
    (lambda r: r["layers"][0]["experts"][0]["tensors"]["gate"].__setitem__("shape", [64, "x"]), "malformed tensor gate"),
    (lambda r: r["layers"][0]["experts"][0]["tensors"]["gate"].__setitem__("bits", "4"), "malformed tensor bits gate"),
    (lambda r: r["layers"][0]["experts"][1].__setitem__("expert", 2), "expert id out of range"),
    (lambda r: r["layers"][0]["experts"][1].__setitem__("physicalRank", 2), "physicalRank out of range"),
    (lambda r: r["layers"][0]["experts"][1].__setitem__("expert", 0), "missing expert entries"),
    (lambda r: r["layers"][0]["experts"].pop(), "missing expert entries"),
])
def test_malformed_layouts_are_rejected(tmp_path, mutate, needle):
    root = toy_root()
    mutate(root)
    with pytest.raises(IndexCorrupt) as e:
        PackedExpertsLayoutReader.load(write_root(tmp_path, root))
    assert needle in e.value.detail


def test_defaults_of_optional_keys(tmp_path):
    root = toy_root()
    for ex in root["layers"][0]["experts"]:
        ex.pop("expert")                                   # ids default to the position in the file
        ex.pop("physicalRank", None)
    root["layers"].insert(0, {"layer": 0, "file": "layer_00.bin", "experts": []})      # a dense layer: no experts, no file
    root["layers"][1]["layer"] = 1
    layout = PackedExpertsLayoutReader.load(write_root(tmp_path, root))
    assert layout.layers[0].experts == [] and [e.expert for e in layout.layers[1].experts] == [0, 1]


def test_layer_file_is_checked_against_the_layout(tmp_path):
    d = write_root(tmp_path, toy_root())
    layout = PackedExpertsLayoutReader.load(d)
    with pytest.raises(MissingFile):
        PackedLayerFile(d, layout, 0)
    (tmp_path / "packed_experts" / "layer_00.bin").write_bytes(b"\x07" * 20000)       # second blob does not fit
    with pytest.raises(IndexCorrupt):
        PackedLayerFile(d, layout, 0)
    (tmp_path / "packed_experts" / "layer_00.bin").write_bytes(b"\x07" * 16384 + b"\x09" * 16384)
    import torch
    with PackedLayerFile(d, layout, 0) as fh:
        buf = torch.zeros(16384, dtype=torch.uint8)
        fh.read_expert_into(1, buf)
        assert bool((buf == 9).all())
        fh.read_expert_into(0, buf)
        assert bool((buf == 7).all())


@pytest.mark.gpu
def test_synthetic_layer_round_trips_through_packed_experts_and_runs(tmp_path):
    """A seeded layer written as packed_experts/ (blobs shuffled in the file), read back (a) whole into HBM and
    (b) expert by expert through a 6-slot pool: both give the output of the original layer, bit for bit."""
    import copy
    import torch
    from mference_b200.moe import MoE, synth_layer, synth_normal
    from mference_b200.pool import ExpertPool
    d, f, E, K, T = 512, 256, 16, 4, 6
    layer = synth_layer(0xB2000001, 3, d, f, E)
    order = list(np.random.default_rng(5).permutation(E))
    layout = write_packed_experts(str(tmp_path), [dict(pool=layer.pool, slot_stride=layer.slot_stride, offsets=layer.routed_off,
                                                       d=d, f=f, bits=4, physical_order=[int(x) for x in order])])
    assert layout.experts_per_layer == E and layout.expert_stride % 4096 == 0
    assert sorted(layout.routed_expert_physical_offsets(0)) == [i * layout.expert_stride for i in range(E)]
    off = layout.routed_expert_offsets(0)
    assert bytes(off) == bytes(layer.routed_off)
    moe = MoE(d, f, E, K, max_tokens=T)
    x = synth_normal(0xB2000001, "x.packed", T * d, dtype=L.DT_BF16).view(T, d)
    want = torch.empty_like(x)
    moe.encode_layer(layer, x, want)
    loaded = layer_weights_from_packed(str(tmp_path), layout, 0, layer.router_w, norm_w=layer.norm_w,
                                       shared_blob=layer.shared_blob, shared_off=layer.shared_off)
    got = torch.empty_like(x)
    moe.encode_layer(loaded, x, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # partial residency: stage what this batch routes to from the file through a small pool
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float16, device="cuda")
    xn = torch.empty_like(x)
    moe.encode_rmsnorm(x, xn, layer.norm_w)
    moe.encode_router(xn, layer, idx, w)
    need = sorted(set(idx.cpu().numpy().reshape(-1).tolist()))
    pool = ExpertPool(E, layout.expert_stride, max(len(need), 6))
    with PackedLayerFile(str(tmp_path), layout, 0) as fh:
        host = fh.host_blobs(need)
    pool.execute_expert_cache_plan(pool.plan_experts_cached(need), host, torch.cuda.current_stream().cuda_stream)
    staged = copy.copy(loaded)
    staged.pool, staged.slot_stride, staged.slot_of = pool.slab_tensor(), pool.slot_stride, pool.slot_of_tensor()
    got2 = torch.empty_like(x)
    moe.encode_layer(staged, x, got2)
    torch.cuda.synchronize()
    assert torch.equal(got2, want)

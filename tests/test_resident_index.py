"""model_weights.bin reader: header / entry / string-table layout of the reference's resident index
(Sources/Mference/Infrastructure/ModelIO/ResidentIndex.swift) - a file written entry by entry is read back, and the
reader's rejections (short header, entry table past the index region, name outside the region, duplicate name, size
mismatch) fire as the reference's do."""
import os
import struct

import numpy as np
import pytest

from mference_b200.packed_experts import IndexCorrupt, MissingFile
from mference_b200.resident_index import (DTYPE_AFFINE, DTYPE_BF16, ENTRY_BYTES, HEADER_BYTES, ResidentIndex, qwen_moe_tensor_names,
                                          write_resident_file)


def _toy(path):
    rng = np.random.default_rng(2)
    gate_w = rng.integers(0, 256, (4, 128), dtype=np.uint8)
    gate_s = rng.integers(0, 65536, (4, 2), dtype=np.uint16)
    gate_b = rng.integers(0, 65536, (4, 2), dtype=np.uint16)
    norm = rng.integers(0, 65536, 128, dtype=np.uint16)
    names = qwen_moe_tensor_names(0)
    write_resident_file(path, [(names["router"], DTYPE_AFFINE, (4, 128), gate_w, gate_s, gate_b),
                               (names["norm"], DTYPE_BF16, (128,), norm, None, None)])
    return names, gate_w, gate_s, gate_b, norm


def test_written_file_reads_back(tmp_path):
    path = str(tmp_path / "model_weights.bin")
    names, gate_w, gate_s, gate_b, norm = _toy(path)
    idx = ResidentIndex(path)
    assert idx.entry_count == 2 and idx.index_size % 16384 == 0
    assert os.path.getsize(path) == idx.index_size + idx.resident_size
    e = idx.entry(names["router"])
    assert (e.dtype, e.shape, e.size_bytes, e.scale_size, e.bias_size) == (DTYPE_AFFINE, (4, 128, 0, 0), 512, 16, 16)
    assert e.file_offset == idx.index_size and e.scale_offset == e.file_offset + 512 and e.bias_offset == e.scale_offset + 16
    w, s, b, _ = idx.tensor(names["router"])
    assert np.array_equal(w.reshape(4, 128), gate_w) and np.array_equal(s.reshape(4, 2), gate_s) and np.array_equal(b.reshape(4, 2), gate_b)
    w, s, b, e = idx.tensor(names["norm"])
    assert s is None and b is None and e.dtype == DTYPE_BF16 and np.array_equal(w.view(np.uint16), norm)
    with pytest.raises(IndexCorrupt) as err:
        idx.entry("language_model.model.layers.0.mlp.nothing")
    assert "no IndexEntry named" in err.value.detail


def test_rejections(tmp_path):
    with pytest.raises(MissingFile):
        ResidentIndex(str(tmp_path / "absent.bin"))
    path = str(tmp_path / "model_weights.bin")
    _toy(path)
    good = open(path, "rb").read()

    def variant(data):
        p = str(tmp_path / "bad.bin")
        open(p, "wb").write(data)
        return p

    with pytest.raises(IndexCorrupt) as err:                       # short header
        ResidentIndex(variant(good[:10]))
    assert "short read for IndexHeader" in err.value.detail
    bad = bytearray(good)
    bad[0:8] = struct.pack("<Q", 8)                                 # indexSize below the header
    with pytest.raises(IndexCorrupt) as err:
        ResidentIndex(variant(bytes(bad)))
    assert "< header size" in err.value.detail
    bad = bytearray(good)
    bad[16:24] = struct.pack("<Q", 10 ** 6)                         # entry table past the index region
    with pytest.raises(IndexCorrupt) as err:
        ResidentIndex(variant(bytes(bad)))
    assert "header+entries" in err.value.detail
    bad = bytearray(good)
    bad[HEADER_BYTES:HEADER_BYTES + 4] = struct.pack("<I", 3)       # name offset inside the header
    with pytest.raises(IndexCorrupt) as err:
        ResidentIndex(variant(bytes(bad)))
    assert "out of index region" in err.value.detail
    bad = bytearray(good)                                           # second entry renamed to the first one's name
    bad[HEADER_BYTES + ENTRY_BYTES:HEADER_BYTES + ENTRY_BYTES + 6] = good[HEADER_BYTES:HEADER_BYTES + 6]
    with pytest.raises(IndexCorrupt) as err:
        ResidentIndex(variant(bytes(bad)))
    assert "duplicate tensor name" in err.value.detail
    with pytest.raises(IndexCorrupt) as err:                        # truncated tensor region
        ResidentIndex(variant(good[:-4]))
    assert "size" in err.value.detail

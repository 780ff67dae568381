"""Header parsing of the safetensors reader (no GPU: the library is loaded, files are mapped and
described, nothing is copied to a device).  Files are written by the `safetensors` Python package
(the implementation the format comes from) and by hand for the malformed cases."""
import json
import struct

import numpy as np
import pytest

st_np = pytest.importorskip("safetensors.numpy")


def test_library_exports_reader():
    from ug_b200 import _lib
    names = set(_lib.parse_header())
    assert {"ugb_st_open", "ugb_st_close", "ugb_st_count", "ugb_st_name", "ugb_st_info", "ugb_st_load_slice",
            "ugb_st_load_slice_with_cast"} <= names
    for n in names:
        assert hasattr(_lib.lib, n)


def test_written_file_layout_matches_what_the_reader_expects(tmp_path):
    """The container layout the C reader parses, checked here against the reference implementation's
    writer: 8-byte little-endian header length, JSON header, gap-free data section."""
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(5, dtype=np.int64)
    p = tmp_path / "t.safetensors"
    st_np.save_file({"a": a, "b": b}, str(p), metadata={"k": "v"})
    raw = p.read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    assert hdr["__metadata__"] == {"k": "v"}
    ends = sorted((v["data_offsets"] for k, v in hdr.items() if k != "__metadata__"))
    assert ends[0][0] == 0 and ends[0][1] == ends[1][0] and ends[1][1] == len(raw) - 8 - n
    assert hdr["a"]["dtype"] == "F32" and hdr["a"]["shape"] == [3, 4] and hdr["b"]["dtype"] == "I64"

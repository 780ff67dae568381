"""safetensors reader through the C ABI: files written by the `safetensors` Python package are read
back bit for bit, casts follow the reference's host conversions, malformed files are rejected, and a
model built from a file equals the model built from the same arrays."""
import json
import struct

import numpy as np
import pytest

from ug_b200 import DType, UgError, synth
from ug_b200.llama import Config, Model, weight_names
from ug_b200.safetensors import MmapedSafetensors

st_np = pytest.importorskip("safetensors.numpy")
pytestmark = pytest.mark.gpu


def bf16_bits(x):
    return synth.to_bf16_bits(np.asarray(x, np.float32))


def write_raw(path, header, data=b""):
    h = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(h)) + h + data)


def test_round_trip_all_dtypes(dev, tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"f32": rng.standard_normal((3, 5)).astype(np.float32),
               "f16": rng.standard_normal((7,)).astype(np.float16),
               "i32": rng.integers(-1000, 1000, (2, 2, 3)).astype(np.int32),
               "i64": rng.integers(-2**40, 2**40, (4,)).astype(np.int64),
               "empty": np.zeros((0, 4), np.float32),
               "u8": np.arange(6, dtype=np.uint8)}
    p = tmp_path / "a.safetensors"
    st_np.save_file(tensors, str(p))
    # bf16 has no numpy dtype: a second file written by hand
    bits = bf16_bits(rng.standard_normal((4, 8)))
    q = tmp_path / "b.safetensors"
    write_raw(q, {"bf": {"dtype": "BF16", "shape": [4, 8], "data_offsets": [0, 64]}, "__metadata__": {"format": "pt"}},
              bits.tobytes())
    st = MmapedSafetensors.multi([p, q], dev)
    assert sorted(st.names()) == sorted(list(tensors) + ["bf"])
    assert st.get("f32") == (DType.F32, (3, 5)) and st.get("u8") == (None, (6,)) and st.get("bf") == (DType.BF16, (4, 8))
    for name in ("f32", "f16", "i32", "i64", "empty"):
        shape, s = st.load_slice(name)
        assert shape == tensors[name].shape and len(s) == tensors[name].size
        got = s.to_vec()
        want = tensors[name].reshape(-1)
        assert np.array_equal(got.view(want.dtype) if got.dtype != want.dtype else got, want)
    shape, s = st.load_slice("bf")
    assert np.array_equal(s.to_vec(), bits.reshape(-1))
    with pytest.raises(UgError) as e:
        st.load_slice("u8")
    assert e.value.code == 2 and "unsupported dtype" in e.value.msg
    with pytest.raises(UgError) as e:
        st.load_slice("missing")
    assert "cannot find tensor" in e.value.msg
    st.close()


def test_casts_follow_the_reference(dev, tmp_path):
    f = np.array([0.0, -1.5, 3.1415927, 1e10, -1e10, 65504.0, 1e-8, np.nan], np.float32)
    i = np.array([0, -7, 2**31 - 1, 16777217], np.int32)
    l = np.array([5, -2**33, 2**40 + 3], np.int64)
    p = tmp_path / "c.safetensors"
    st_np.save_file({"f": f, "i": i, "l": l, "h": f[:3].astype(np.float16)}, str(p))
    st = MmapedSafetensors(p, dev)
    # f32 -> bf16 / f16: round to nearest even; -> i32 / i64: saturating, NaN -> 0
    assert np.array_equal(st.load_slice_with_cast("f", DType.BF16)[1].to_vec(), bf16_bits(f))
    with np.errstate(over="ignore"):
        assert np.array_equal(st.load_slice_with_cast("f", DType.F16)[1].to_vec().view(np.float16), f.astype(np.float16), equal_nan=True)
    assert np.array_equal(st.load_slice_with_cast("f", DType.I32)[1].to_vec(),
                          np.array([0, -1, 3, 2**31 - 1, -2**31, 65504, 0, 0], np.int32))
    assert np.array_equal(st.load_slice_with_cast("f", DType.I64)[1].to_vec(),
                          np.array([0, -1, 3, 10**10, -10**10, 65504, 0, 0], np.int64))
    # ints -> f32 (nearest), i64 -> i32 wraps like `as i32`
    assert np.array_equal(st.load_slice_with_cast("i", DType.F32)[1].to_vec(), i.astype(np.float32))
    assert np.array_equal(st.load_slice_with_cast("i", DType.I64)[1].to_vec(), i.astype(np.int64))
    assert np.array_equal(st.load_slice_with_cast("l", DType.I32)[1].to_vec(), l.astype(np.int32))
    assert np.array_equal(st.load_slice_with_cast("l", DType.F32)[1].to_vec(), l.astype(np.float32))
    # f16 -> f32 exact, f16 -> bf16 through f32; f16 -> i64 is the reference's own dtype mismatch
    assert np.array_equal(st.load_slice_with_cast("h", DType.F32)[1].to_vec(), f[:3].astype(np.float16).astype(np.float32))
    assert np.array_equal(st.load_slice_with_cast("h", DType.BF16)[1].to_vec(), bf16_bits(f[:3].astype(np.float16).astype(np.float32)))
    with pytest.raises(UgError) as e:
        st.load_slice_with_cast("h", DType.I64)
    assert e.value.code == 2
    st.close()


def test_malformed_files_are_rejected(dev, tmp_path):
    ok = {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    cases = {
        "short": b"\x01\x02",
        "huge_header": struct.pack("<Q", 2**40) + b"{}",
        "not_json": struct.pack("<Q", 4) + b"abcd",
        "bad_len": None, "gap": None, "overlap": None, "trailing": None, "unknown_dtype": None,
    }
    for name, raw in cases.items():
        p = tmp_path / f"{name}.safetensors"
        if raw is not None:
            p.write_bytes(raw)
        elif name == "bad_len":
            write_raw(p, {"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
        elif name == "gap":
            write_raw(p, {"t": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
        elif name == "overlap":
            write_raw(p, {"t": ok["t"], "u": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
        elif name == "trailing":
            write_raw(p, ok, b"\0" * 16)
        elif name == "unknown_dtype":
            write_raw(p, {"t": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
        with pytest.raises(UgError) as e:
            MmapedSafetensors(p, dev)
        assert e.value.code == 1 and str(p) in e.value.msg, name
    with pytest.raises(UgError):
        MmapedSafetensors(tmp_path / "nope.safetensors", dev)
    p = tmp_path / "fine.safetensors"
    write_raw(p, ok, np.array([1.5, -2.0], np.float32).tobytes())
    st = MmapedSafetensors(p, dev)
    assert np.array_equal(st.load_slice("t")[1].to_vec(), np.array([1.5, -2.0], np.float32))
    dev.synchronize()


def test_model_from_safetensors_equals_model_from_arrays(dev, tmp_path):
    cfg = Config(hidden_size=128, intermediate_size=256, max_position_embeddings=256, num_attention_heads=2,
                 num_key_value_heads=1, num_hidden_layers=2, vocab_size=512)
    w = synth.llama_weights(cfg, 5)
    # the file holds f32 matrices (rounded to bf16 on load, as the arrays path does with these bit patterns)
    # and f32 norm weights; the config goes through config.json
    tensors = {n: (synth.bf16_bits_to_f32(a) if a.dtype == np.uint16 else a) for n, a in w.items()}
    p = tmp_path / "model.safetensors"
    st_np.save_file(tensors, str(p))
    (tmp_path / "config.json").write_text(json.dumps(dict(cfg.__dict__, architectures=["LlamaForCausalLM"])))
    cfg2 = Config.from_json(tmp_path / "config.json")
    assert cfg2 == cfg
    st = MmapedSafetensors(p, dev)
    assert set(weight_names(cfg2)) <= set(st.names())
    a = Model.new(cfg, w, dev, 4, 64)
    b = Model.from_safetensors(cfg2, st, dev, 4, 64)
    prompts = synth.tokens(3, (4, 20), cfg.vocab_size)
    for m in (a, b):
        m.prefill(prompts)
        m.decode(3)
    assert np.array_equal(a.logits(), b.logits()) and np.array_equal(a.next_tokens(), b.next_tokens())
    a.close()
    b.close()
    st.close()

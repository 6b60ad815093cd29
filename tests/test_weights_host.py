"""The checkpoint reader (ampstein_b200/weights.py) on the host: the safetensors layout, single-file
and sharded directories, zero-copy views, and the errors a damaged file must raise. No GPU."""
import json
import os
import struct

import numpy as np
import pytest

torch = pytest.importorskip("torch")


def _tensors(seed):
    g = torch.Generator().manual_seed(seed)
    return {
        "model.layers.0.q_proj.trellis": torch.randint(-32768, 32768, (8, 16, 64), dtype=torch.int16, generator=g),
        "model.layers.0.q_proj.suh": torch.randn(128, generator=g).to(torch.float16),
        "model.layers.0.q_proj.svh": torch.randn(256, generator=g).to(torch.float16),
        "model.layers.0.q_proj.mul1": torch.zeros(1, dtype=torch.int32),
        "model.norm.weight": torch.randn(128, generator=g).to(torch.bfloat16),
        "scalar": torch.tensor(3.5),
        "empty": torch.zeros((0, 4), dtype=torch.float32),
    }


def test_single_file_round_trip(tmp_path):
    from ampstein_b200 import weights
    want = _tensors(1)
    weights.save_file(want, str(tmp_path / "model.safetensors"), metadata={"format": "pt"})
    ws = weights.open(str(tmp_path))
    assert ws.keys() == sorted(want)
    for k, t in want.items():
        assert ws.has(k) and ws.info(k) == {"shape": list(t.shape), "dtype": {torch.int16: "I16", torch.float16: "F16",
                                            torch.int32: "I32", torch.bfloat16: "BF16", torch.float32: "F32"}[t.dtype]}
        got = ws.tensor(k)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
    assert not ws.has("nope")
    with pytest.raises(KeyError):
        ws.info("nope")
    assert ws.fp16("model.norm.weight").dtype == torch.float16
    # the header is the public layout: 8-byte length, JSON, then the buffer
    raw = (tmp_path / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + n])
    b, e = head["model.layers.0.q_proj.suh"]["data_offsets"]
    assert np.array_equal(np.frombuffer(raw[8 + n + b:8 + n + e], np.float16), want["model.layers.0.q_proj.suh"].numpy())
    with pytest.raises(RuntimeError):
        ws.upload(0) if not torch.cuda.is_available() else (_ for _ in ()).throw(RuntimeError("skip"))


def test_sharded_directory_and_only_file(tmp_path):
    from ampstein_b200 import weights
    want = _tensors(2)
    keys = sorted(want)
    a, b = {k: want[k] for k in keys[:3]}, {k: want[k] for k in keys[3:]}
    weights.save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    weights.save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    with open(tmp_path / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in a},
                                  **{k: "model-00002-of-00002.safetensors" for k in b}}}, f)
    ws = weights.open(str(tmp_path))
    assert ws.keys() == keys
    for k in keys:
        assert torch.equal(ws.tensor(k), want[k])
    assert len(ws._files) == 2                                   # shards are opened on first use
    one = weights.open(str(tmp_path), "model-00002-of-00002.safetensors")
    assert one.keys() == sorted(b) and not one.has(keys[0])


def test_damaged_files_are_rejected(tmp_path):
    from ampstein_b200 import weights
    with pytest.raises(FileNotFoundError):
        weights.open(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\\x01\\x02")
    with pytest.raises(ValueError):
        weights.open(str(tmp_path)).keys()
    head = json.dumps({"w": {"dtype": "F16", "shape": [4], "data_offsets": [0, 6]}}).encode()      # 4 halves are 8 bytes
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\\0" * 8)
    with pytest.raises(ValueError):
        weights.open(str(tmp_path)).keys()
    head = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\\0" * 4)
    with pytest.raises(ValueError):
        weights.open(str(tmp_path)).keys()
    (tmp_path / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(ValueError):
        weights.open(str(tmp_path))

"""GGUF container reader: header, metadata and tensor directory round trips, the error cases the
reference's reader reports (crates/gguf/src/lib.rs:199-300, 806-871), and the dense-Qwen3 config keys."""
import struct

import numpy as np
import pytest

from ribn_b200 import gguf
from tests import helpers as H

META = {"general.architecture": "qwen3", "general.name": "tiny", "qwen3.block_count": 2, "qwen3.embedding_length": 256,
        "qwen3.feed_forward_length": 512, "qwen3.attention.head_count": 4, "qwen3.attention.head_count_kv": 2,
        "qwen3.attention.key_length": 64, "qwen3.rope.freq_base": 1.0e6,
        "qwen3.attention.layer_norm_rms_epsilon": 1.0e-6, "tokenizer.ggml.tokens": ["a", "b", "c"], "flag": True}
CFG = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512, rope_base=1.0e6, rms_eps=1.0e-6)


def test_write_then_read_round_trips(tmp_path):
    tensors = H.make_model(CFG, seed=5)
    path = str(tmp_path / "tiny.gguf")
    gguf.write_gguf(path, META, tensors)
    f = gguf.GgufFile(path)
    assert f.metadata["general.architecture"] == "qwen3" and f.metadata["flag"] is True
    assert f.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
    assert set(f.tensors) == set(tensors)
    assert f.data_offset % 32 == 0
    for name, (kind, rows, cols, data) in tensors.items():
        t = f.tensors[name]
        assert (t.ggml_type, t.rows, t.cols) == (kind, rows, cols)
        assert (f.data_offset + t.offset) % 32 == 0
        assert np.array_equal(f.tensor_bytes(name), np.ascontiguousarray(data).view(np.uint8).reshape(-1))
    got = gguf.qwen3_config(f)
    assert got == {**CFG, "rope_base": pytest.approx(1.0e6), "rms_eps": pytest.approx(1.0e-6)}
    f.close()


def test_reader_rejects_malformed_files(tmp_path):
    tensors = {"token_embd.weight": H.make_model(CFG, seed=5)["token_embd.weight"]}
    good = str(tmp_path / "good.gguf")
    gguf.write_gguf(good, META, tensors)
    raw = bytearray(open(good, "rb").read())

    def variant(name, mutate):
        data = bytearray(raw)
        mutate(data)
        p = str(tmp_path / name)
        open(p, "wb").write(data)
        return p

    with pytest.raises(gguf.GgufError, match="magic"):
        gguf.GgufFile(variant("magic.gguf", lambda d: d.__setitem__(slice(0, 4), b"GGML")))
    with pytest.raises(gguf.GgufError, match="version"):
        gguf.GgufFile(variant("version.gguf", lambda d: d.__setitem__(slice(4, 8), struct.pack("<I", 2))))
    with pytest.raises(gguf.GgufError, match="truncated|out-of-bounds"):
        gguf.GgufFile(variant("short.gguf", lambda d: d.__delitem__(slice(len(d) - 64, len(d)))))
    with pytest.raises(gguf.GgufError, match="truncated|exceeds the parser bound"):
        gguf.GgufFile(variant("header.gguf", lambda d: d.__delitem__(slice(40, len(d)))))
    bad_meta = dict(META); bad_meta["general.architecture"] = "llama"
    other = str(tmp_path / "llama.gguf")
    gguf.write_gguf(other, bad_meta, tensors)
    f = gguf.GgufFile(other)
    with pytest.raises(gguf.GgufError, match="architecture"):
        gguf.qwen3_config(f)
    f.close()
    missing = {k: v for k, v in META.items() if k != "qwen3.block_count"}
    gguf.write_gguf(other, missing, tensors)
    f = gguf.GgufFile(other)
    with pytest.raises(gguf.GgufError, match="qwen3.block_count"):
        gguf.qwen3_config(f)
    with pytest.raises(gguf.GgufError, match="not found"):
        f.tensor_bytes("output.weight")
    f.close()

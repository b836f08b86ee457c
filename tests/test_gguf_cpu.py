"""The GGUF reader of the upload path: directory and metadata of a generated file, zero-copy tensor views, and the
malformed inputs the reference's own parser tests reject (tests/fuzz_gguf.cpp, tests/qwen_invalid_model.py)."""
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_llama_golden import SEED, TINY, WEIGHT_STD, write_gguf  # noqa: E402

from zeninfer_b200 import gguf
from zeninfer_b200.llama import synthetic_tensors, tensor_plan


@pytest.fixture(scope="module")
def model_path(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    write_gguf(path, TINY, synthetic_tensors(TINY, SEED, WEIGHT_STD))
    return path


def test_directory_metadata_and_views(model_path):
    with gguf.GgufFile(model_path) as g:
        cfg = gguf.llama_config(g)
        assert abs(cfg.rms_eps - TINY.rms_eps) < 1e-12 and cfg.rms_eps == float(np.float32(TINY.rms_eps))   # stored as fp32
        assert {k: v for k, v in cfg.__dict__.items() if k != "rms_eps"} == {k: v for k, v in TINY.__dict__.items() if k != "rms_eps"}
        assert g.metadata["general.architecture"] == "llama" and len(g.metadata["tokenizer.ggml.tokens"]) == TINY.vocab
        assert set(g.tensors) == {n for n, _, _ in tensor_plan(TINY)}
        ref = {n: a for n, a, _ in synthetic_tensors(TINY, SEED, WEIGHT_STD)}
        for name, arr, is_matrix in gguf.llama_tensors(g, cfg):
            assert g.tensors[name].offset % 32 == 0
            assert not arr.flags["OWNDATA"] and arr.flags["C_CONTIGUOUS"]     # a view of the mapping, not a copy
            assert np.array_equal(arr, ref[name]), name
            assert arr.dtype == (np.uint8 if is_matrix else np.float32)


def test_malformed_files_are_rejected(model_path, tmp_path):
    data = open(model_path, "rb").read()

    def rejects(blob: bytes):
        p = str(tmp_path / "bad.gguf")
        with open(p, "wb") as f:
            f.write(blob)
        with pytest.raises(gguf.GgufError):
            gguf.GgufFile(p).close()

    rejects(b"GGML" + data[4:])                                   # wrong magic
    rejects(data[:4] + struct.pack("<I", 1) + data[8:])            # unsupported version
    rejects(data[: len(data) // 2])                                # tensor data cut off
    rejects(data[:200])                                            # metadata cut off
    rejects(data[:8] + struct.pack("<Q", 1 << 40) + data[16:])     # absurd tensor count


def test_wrong_architecture_or_type_is_refused(model_path, tmp_path):
    data = bytearray(open(model_path, "rb").read())
    i = data.find(b"llama", data.find(b"general.architecture"))
    data[i:i + 5] = b"qwen2"
    p = str(tmp_path / "other.gguf")
    with open(p, "wb") as f:
        f.write(data)
    with gguf.GgufFile(p) as g, pytest.raises(gguf.GgufError):
        gguf.llama_config(g)


def test_k_quant_tensors_are_sized_and_readable(tmp_path):
    """Q4_K (type 12) and Q5_K (type 13) tensors: the directory sizes them by their super-blocks and hands out their raw
    bytes; an unknown type is listed but not readable; a Q4_K tensor whose columns are not whole super-blocks is refused."""
    from zeninfer_b200 import blocks

    def s(text: str) -> bytes:
        b = text.encode()
        return struct.pack("<Q", len(b)) + b

    def build(entries) -> bytes:
        out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(entries), 0))
        off, datas = 0, []
        for name, dims, ggml_type, data in entries:
            off = (off + 31) & ~31
            out += s(name) + struct.pack("<I", len(dims)) + struct.pack("<" + "Q" * len(dims), *dims) + struct.pack("<IQ", ggml_type, off)
            datas.append((off, data))
            off += len(data)
        out += bytes((-len(out)) % 32)
        start = len(out)
        for o, data in datas:
            out += bytes(start + o - len(out)) + data
        return bytes(out)

    w4 = blocks.random_k_blocks(blocks.Q4_K, 4, 512, 1)
    w5 = blocks.random_k_blocks(blocks.Q5_K, 3, 256, 2)
    p = str(tmp_path / "k.gguf")
    with open(p, "wb") as f:
        f.write(build([("a.weight", [512, 4], 12, w4.tobytes()), ("b.weight", [256, 3], 13, w5.tobytes()), ("c.weight", [32, 2], 99, bytes(64))]))
    with gguf.GgufFile(p) as g:
        assert g.tensors["a.weight"].shape == (4, 512) and g.tensors["a.weight"].nbytes == 4 * 2 * 144
        assert g.tensors["b.weight"].nbytes == 3 * 176
        assert np.array_equal(g.array("a.weight"), w4) and np.array_equal(g.array("b.weight"), w5)
        assert np.array_equal(blocks.dequantize(blocks.Q5_K, np.array(g.array("b.weight")), 3, 256), blocks.dequantize(blocks.Q5_K, w5, 3, 256))
        with pytest.raises(gguf.GgufError):
            g.array("c.weight")
    bad = str(tmp_path / "bad.gguf")
    with open(bad, "wb") as f:
        f.write(build([("a.weight", [128, 4], 12, bytes(4 * 72))]))
    with pytest.raises(gguf.GgufError):
        gguf.GgufFile(bad)

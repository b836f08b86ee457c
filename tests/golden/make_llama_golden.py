#!/usr/bin/env python
"""Generates tests/golden/llama_tiny.npz: token ids and final logits the UNMODIFIED reference produces for a small
generated Llama-layout GGUF model (Q8_0 matrices, fp32 norms).

    make -C oracle runtime            # builds oracle/_ref/libzenrt.so from the reference's own sources
    python tests/golden/make_llama_golden.py

The model is zeninfer_b200.llama.synthetic_tensors(TINY, seed) written as a GGUF v3 file; the reference loads it
with load_model_runtime and generates greedily (ModelRuntime::generate, include/zen/model_runtime.h:26-28).  The GPU
test rebuilds the same tensors from the same seed and must reproduce the ids exactly and the logits within 1e-3.
A second generation comes from a child process with ZEN_CPU_Q8_ACT=1 (the reference latches that switch on its first
Q8_0 call, so it needs a process of its own): there the reference quantises the activations of every single-token
product to int8 (src/quant.cpp:1088-1123) while the prompt block still goes through its fp32-activation GEMM
(src/quant.cpp:1667-1680, tokens >= 2).  Stored as ids_int8 / last_logits_int8.
Needs the reference tree; the committed .npz is what travels.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from zeninfer_b200.llama import LlamaConfig, synthetic_tensors, tensor_plan  # noqa: E402

TINY = LlamaConfig(embedding=256, layers=2, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512, rope_base=500000.0, rms_eps=1e-5, context=128)
SEED, WEIGHT_STD = 6, 0.06
PROMPT_LEN, MAX_NEW = 12, 16

U32, F32, BOOL, STRING, ARRAY, I32 = 4, 6, 7, 8, 9, 5
GGML_F32, GGML_Q8_0 = 0, 8


def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _value(kind: int, v) -> bytes:
    if kind == STRING:
        return _s(v)
    if kind == U32:
        return struct.pack("<I", v)
    if kind == I32:
        return struct.pack("<i", v)
    if kind == F32:
        return struct.pack("<f", v)
    if kind == BOOL:
        return struct.pack("<B", v)
    sub, items = v
    return struct.pack("<IQ", sub, len(items)) + b"".join(_value(sub, x) for x in items)


def write_gguf(path: str, cfg: LlamaConfig, tensors) -> None:
    """GGUF v3: header, metadata, tensor directory (dims innermost first), 32-byte aligned tensor data."""
    tokens = ["<unk>", "<s>", "</s>"] + [f"<t{i}>" for i in range(3, cfg.vocab)]
    meta = [("general.architecture", STRING, "llama"), ("general.name", STRING, "synthetic-llama-q8_0"),
            ("llama.embedding_length", U32, cfg.embedding), ("llama.block_count", U32, cfg.layers),
            ("llama.attention.head_count", U32, cfg.heads), ("llama.attention.head_count_kv", U32, cfg.kv_heads),
            ("llama.feed_forward_length", U32, cfg.ffn), ("llama.context_length", U32, cfg.context),
            ("llama.rope.dimension_count", U32, cfg.head_dim), ("llama.rope.freq_base", F32, cfg.rope_base),
            ("llama.attention.layer_norm_rms_epsilon", F32, cfg.rms_eps), ("llama.vocab_size", U32, cfg.vocab),
            ("tokenizer.ggml.model", STRING, "llama"), ("tokenizer.ggml.tokens", ARRAY, (STRING, tokens)),
            ("tokenizer.ggml.token_type", ARRAY, (I32, [2, 3, 3] + [1] * (cfg.vocab - 3))),
            ("tokenizer.ggml.bos_token_id", U32, 1), ("tokenizer.ggml.eos_token_id", U32, 2), ("tokenizer.ggml.unknown_token_id", U32, 0),
            ("tokenizer.ggml.add_bos_token", BOOL, 0)]
    shapes = {name: shape for name, shape, _ in tensor_plan(cfg)}
    entries, offset = [], 0
    for name, arr, is_matrix in tensors:
        data = np.ascontiguousarray(arr).tobytes()
        offset = (offset + 31) & ~31
        dims = list(reversed(shapes[name]))  # GGUF lists the innermost dimension first
        entries.append((name, dims, GGML_Q8_0 if is_matrix else GGML_F32, offset, data))
        offset += len(data)
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(entries), len(meta)))
    for key, kind, v in meta:
        out += _s(key) + struct.pack("<I", kind) + _value(kind, v)
    for name, dims, ggml_type, off, _ in entries:
        out += _s(name) + struct.pack("<I", len(dims)) + struct.pack("<" + "Q" * len(dims), *dims) + struct.pack("<IQ", ggml_type, off)
    out += bytes((-len(out)) % 32)
    start = len(out)
    for _, _, _, off, data in entries:
        out += bytes(start + off - len(out))
        out += data
    with open(path, "wb") as f:
        f.write(out)


def reference_generate(gguf_path: str, prompt: np.ndarray, max_new: int, vocab: int):
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libzenrt.so"))
    ids = np.zeros(max_new, np.uint32)
    logits = np.zeros(vocab, np.float32)
    err = C.create_string_buffer(512)
    p = np.ascontiguousarray(prompt, np.uint32)
    n = lib.zrt_generate(gguf_path.encode(), p.ctypes.data_as(C.c_void_p), C.c_uint(len(p)), C.c_uint(max_new), ids.ctypes.data_as(C.c_void_p),
                         logits.ctypes.data_as(C.c_void_p), C.c_uint(vocab), err, C.c_uint(512))
    if n < 0:
        raise RuntimeError(f"reference generate failed ({n}): {err.value.decode()}")
    return ids[:n], logits


def child(gguf_path: str, out_path: str) -> None:
    """Runs in a process whose environment already carries ZEN_CPU_Q8_ACT=1."""
    prompt = np.random.default_rng([SEED, 1]).integers(3, TINY.vocab, size=PROMPT_LEN, dtype=np.int64)
    ids, logits = reference_generate(gguf_path, prompt, MAX_NEW, TINY.vocab)
    np.savez(out_path, ids=ids.astype(np.int64), last_logits=logits)


def main() -> None:
    os.environ["ZEN_BACKEND"] = "cpu"
    if len(sys.argv) == 4 and sys.argv[1] == "--child":
        child(sys.argv[2], sys.argv[3])
        return
    prompt = np.random.default_rng([SEED, 1]).integers(3, TINY.vocab, size=PROMPT_LEN, dtype=np.int64)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "llama_tiny.gguf")
        write_gguf(path, TINY, synthetic_tensors(TINY, SEED, WEIGHT_STD))
        ids, logits = reference_generate(path, prompt, MAX_NEW, TINY.vocab)
        side = os.path.join(tmp, "int8.npz")
        subprocess.run([sys.executable, os.path.abspath(__file__), "--child", path, side], check=True,
                       env={**os.environ, "ZEN_CPU_Q8_ACT": "1", "ZEN_BACKEND": "cpu"})
        with np.load(side) as g:
            ids_int8, logits_int8 = g["ids"].copy(), g["last_logits"].copy()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "llama_tiny.npz")
    print("int8-activation ids:", ids_int8.tolist(), "max |logit diff| to the fp32 run:", float(np.abs(logits_int8 - logits).max()))
    np.savez_compressed(out, prompt=prompt, ids=ids.astype(np.int64), last_logits=logits, ids_int8=ids_int8, last_logits_int8=logits_int8,
                        meta=json.dumps({"config": TINY.__dict__, "seed": SEED, "weight_std": WEIGHT_STD, "max_new": MAX_NEW}))
    print("reference ids:", ids.tolist())
    print("logits: max", float(logits.max()), "top-2 gap", float(np.sort(logits)[-1] - np.sort(logits)[-2]))
    print("wrote", out)


if __name__ == "__main__":
    main()

"""The drop-in, dropped in: the reference's own model runtime, built with the CUDA backend hooked into its dispatch
(tests/integration/Makefile compiles a patched copy of its src/quant.cpp, made at build time, against include/zen/cuda_backend.h
and links libzen_cuda.so), loads the small generated GGUF model and generates greedily.  Every projection and the lm_head
of prefill and decode then go through zen::cuda::* -> the C-ABI -> the kernels, and the token ids must be the ones the
unmodified CPU build produced (tests/golden/llama_tiny.npz).

Runs the generation in a child process: the backend reads ZEN_BACKEND / ZEN_CUDA_Q8_ACT once, at start-up."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import assert_parity

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "integration", "_build", "libzenrt_cuda.so")
GOLDEN = os.path.join(HERE, "golden", "llama_tiny.npz")

CHILD = r"""
import ctypes as C, json, os, sys, tempfile
import numpy as np
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests", "golden"))
import make_llama_golden as mk
from zeninfer_b200.llama import LlamaConfig, synthetic_tensors
with np.load(sys.argv[3]) as g:
    meta = json.loads(str(g["meta"])); prompt = g["prompt"].copy()
cfg = LlamaConfig(**meta["config"])
lib = C.CDLL(sys.argv[2])
with tempfile.TemporaryDirectory() as tmp:
    path = os.path.join(tmp, "llama_tiny.gguf")
    mk.write_gguf(path, cfg, synthetic_tensors(cfg, meta["seed"], meta["weight_std"]))
    ids = np.zeros(meta["max_new"], np.uint32); logits = np.zeros(cfg.vocab, np.float32)
    stats = (C.c_ulonglong * 4)(); err = C.create_string_buffer(512)
    p = np.ascontiguousarray(prompt, np.uint32)
    n = lib.zrt_cuda_generate(path.encode(), p.ctypes.data_as(C.c_void_p), C.c_uint(len(p)), C.c_uint(meta["max_new"]), ids.ctypes.data_as(C.c_void_p),
                              logits.ctypes.data_as(C.c_void_p), C.c_uint(cfg.vocab), stats, err, C.c_uint(512))
print("RESULT " + json.dumps({"n": n, "err": err.value.decode(), "ids": ids[:max(n, 0)].tolist(), "logits": logits.tolist(), "stats": list(stats)}))
"""


def run_child(q8_act: str):
    env = {**os.environ, "ZEN_BACKEND": "cuda", "ZEN_CUDA_Q8_ACT": q8_act}
    out = subprocess.run([sys.executable, "-c", CHILD, os.path.dirname(HERE), LIB, GOLDEN], env=env, capture_output=True, text=True, timeout=600)
    lines = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, f"child failed: {out.stdout[-2000:]}\n{out.stderr[-2000:]}"
    return json.loads(lines[-1][7:])


@pytest.mark.skipif(not os.path.exists(LIB), reason="tests/integration/_build/libzenrt_cuda.so not built (needs the reference tree: make -C tests/integration)")
def test_reference_runtime_generates_the_golden_ids_through_the_cuda_backend():
    with np.load(GOLDEN) as g:
        ids, logits = g["ids"].tolist(), g["last_logits"].copy()
    got = run_child("fp32")     # the activation arithmetic of the reference's default CPU route, which produced the golden vectors
    assert got["n"] == len(ids), got["err"]
    assert got["ids"] == ids
    assert_parity(np.asarray(got["logits"], np.float32), logits, 1e-3, "last logits, reference runtime on the CUDA backend")
    submits, dispatches, fallbacks, upload_bytes = got["stats"]
    assert fallbacks == 0 and submits > 0 and dispatches >= submits
    # every Q8_0 matrix but the embedding table (decoded row by row on the host) crossed to the device exactly once:
    # q, k, v, o, gate, up, down of two layers and the lm_head
    cfg = json.loads(str(np.load(GOLDEN)["meta"]))["config"]
    E, F, V, KW = cfg["embedding"], cfg["ffn"], cfg["vocab"], cfg["kv_heads"] * cfg["head_dim"]
    per_layer = (2 * E * E + 2 * KW * E + 3 * F * E) // 32 * 34
    assert upload_bytes == cfg["layers"] * per_layer + V * E // 32 * 34
    # decode steps alone are 15 tokens x (2 layers x 3 submissions + lm_head): q|k|v, o and the fused gate|up|silu|down
    # (quant::ffn_gemv -> zen::cuda::gemv_q8_0_ffn); the prompt block adds its own
    # (8 tokens, 25 submissions here); with the three FFN products submitted separately the decode steps alone would be 135
    assert 15 * (cfg["layers"] * 3 + 1) <= submits < 15 * (cfg["layers"] * 4 + 1), submits


@pytest.mark.skipif(not os.path.exists(LIB), reason="tests/integration/_build/libzenrt_cuda.so not built")
def test_reference_runtime_int8_activation_mode_through_the_cuda_backend():
    """ZEN_CUDA_Q8_ACT=int8: the prompt block goes through the tensor-core product with int8 activations as well (the CPU
    reference keeps its prompt in fp32), so only the arithmetic class is checked: same first ids, finite logits."""
    with np.load(GOLDEN) as g:
        ids8 = g["ids_int8"].tolist()
    got = run_child("int8")
    assert got["n"] == len(ids8), got["err"]
    assert got["ids"][:4] == ids8[:4]
    assert np.all(np.isfinite(np.asarray(got["logits"], np.float32)))
    assert got["stats"][2] == 0

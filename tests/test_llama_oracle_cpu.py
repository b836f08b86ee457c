"""The numpy restatement of the reference's Llama decode step (oracle/llama.py) against the golden vectors the
unmodified reference produced for a generated GGUF model (tests/golden/make_llama_golden.py)."""
import json
import os

import numpy as np

from zeninfer_b200.llama import LlamaConfig, rope_tables, synthetic_tensors, tensor_plan

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "llama_tiny.npz")


def load_golden():
    with np.load(GOLDEN) as g:
        meta = json.loads(str(g["meta"]))
        return LlamaConfig(**meta["config"]), meta, g["prompt"].copy(), g["ids"].copy(), g["last_logits"].copy()


def test_numpy_decode_reproduces_the_reference():
    from oracle import llama as ol
    cfg, meta, prompt, ids, logits = load_golden()
    tensors = {n: a for n, a, _ in synthetic_tensors(cfg, meta["seed"], meta["weight_std"])}
    shapes = {n: s for n, s, _ in tensor_plan(cfg)}
    got_ids, got_logits = ol.generate(cfg, tensors, shapes, prompt, meta["max_new"])
    assert got_ids == ids.tolist()
    assert np.abs(got_logits - logits).max() <= 1e-4 * np.abs(logits).max()


def test_tensor_plan_and_tables():
    cfg = LlamaConfig()
    plan = tensor_plan(cfg)
    assert len(plan) == 3 + 9 * cfg.layers
    assert dict((n, s) for n, s, _ in plan)["blk.31.ffn_down.weight"] == (4096, 14336)
    cos, sin = rope_tables(LlamaConfig(head_dim=64, rope_base=10000.0), 4)
    assert cos.shape == (4, 32) and np.all(cos[0] == 1) and np.all(sin[0] == 0)
    assert abs(float(cos[1, 0]) - np.cos(1.0)) < 1e-6 and abs(float(sin[3, 0]) - np.sin(3.0)) < 1e-6

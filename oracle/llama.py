"""CPU restatement (numpy) of the reference's dense Llama decode step, for checking the device decoder.

TEST INFRASTRUCTURE ONLY: tests/ import this; the product (zeninfer_b200/) never does.

Follows DenseTransformerRuntime::forward for `general.architecture = llama`
(src/adapters/dense_transformer_runtime.cpp): embedding row decode :3692, rms_norm :117-125 (sum of squares in
double, inv = 1/sqrt(float(ss/n) + eps)), projections as fp32-activation products over the decoded Q8_0 weights
(the reference's default CPU route, kernels/avx2.cpp:587-641), adjacent-pair rope :300-329, attention :4284-4337
(scores / sqrt(D), exp(score - max), double denominator, a = score * (1/denominator)), silu_mul :193-199, greedy
pick :391-418.  Pinned by tests/golden/llama_tiny.npz, which the unmodified reference produced.
"""
from __future__ import annotations

import numpy as np


def _dequant_q8_0(packed: np.ndarray, rows: int, cols: int) -> np.ndarray:
    b = np.ascontiguousarray(packed, np.uint8).reshape(rows, cols // 32, 34)
    d = b[..., :2].copy().view(np.float16).astype(np.float32)          # [rows, nb, 1]
    q = b[..., 2:].view(np.int8).astype(np.float32)                      # [rows, nb, 32]
    return (q * d).reshape(rows, cols)


def _rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    ss = float(np.sum(x.astype(np.float64) ** 2))
    inv = np.float32(1.0) / np.sqrt(np.float32(ss / x.size) + np.float32(eps), dtype=np.float32)
    return (x * inv * w).astype(np.float32)


def generate(cfg, tensors: dict, shapes: dict, prompt, max_new: int, rank: int = 0, world: int = 1, gather=None, cut: str = "rows"):
    """tensors: name -> array (Q8_0 raw blocks for matrices, fp32 for norms); shapes: name -> (rows, cols).
    Returns (ids, last_logits).

    world > 1 restates the row-sharded decoder: every matrix but the embedding table keeps rows
    [rank * rows / world, (rank + 1) * rows / world), attention runs on the rank's heads, and `gather(piece)` returns the
    concatenation of all ranks' pieces in rank order (four per layer: attention output, o projection, SwiGLU activation,
    down projection; one for the logits).  Rows are independent, so the result equals the unsharded one.
    cut = "rows+cols": the o and down projections keep columns [rank * cols / world, ...) instead, multiply the rank's own
    attention output / SwiGLU activation, and the ranks' partial products are added in rank order (two exchanges per
    layer); equal to the unsharded result up to fp32 rounding."""
    if gather is None:
        if world != 1:
            raise ValueError("a sharded run needs a gather")
        gather = lambda piece: piece
    W = {n: _dequant_q8_0(a, *shapes[n]) for n, a in tensors.items() if len(shapes[n]) == 2}
    if world > 1:
        for n in W:
            if cut == "rows+cols" and n.endswith(("attn_output.weight", "ffn_down.weight")):
                per = W[n].shape[1] // world
                W[n] = W[n][:, rank * per:(rank + 1) * per]
            elif n != "token_embd.weight":
                per = W[n].shape[0] // world
                W[n] = W[n][rank * per:(rank + 1) * per]
    N = {n: np.asarray(a, np.float32) for n, a in tensors.items() if len(shapes[n]) == 1}

    def add_partials(x: np.ndarray, partial: np.ndarray) -> np.ndarray:
        for piece in gather(partial).reshape(world, -1):     # x + p0 + p1 + ..., the same order on every rank
            x = x + piece
        return x

    E, H, KH, D = cfg.embedding, cfg.heads // world, cfg.kv_heads // world, cfg.head_dim      # H, KH: this rank's heads
    half = D // 2
    kc = [np.zeros((0, KH * D), np.float32) for _ in range(cfg.layers)]
    vc = [np.zeros((0, KH * D), np.float32) for _ in range(cfg.layers)]

    def rope(v: np.ndarray, heads: int, pos: int) -> np.ndarray:
        i = np.arange(half, dtype=np.float32)
        freq = np.power(np.float32(cfg.rope_base), (np.float32(-2.0) * i / np.float32(D)).astype(np.float32)).astype(np.float32)
        ang = (np.float32(pos) * freq).astype(np.float32)
        c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        v = v.reshape(heads, half, 2).copy()
        a, b = v[..., 0].copy(), v[..., 1].copy()
        v[..., 0] = a * c - b * s
        v[..., 1] = a * s + b * c
        return v.reshape(-1)

    def forward(token: int, pos: int) -> np.ndarray:
        x = W["token_embd.weight"][token].copy()
        for l in range(cfg.layers):
            p = f"blk.{l}."
            xn = _rms_norm(x, N[p + "attn_norm.weight"], cfg.rms_eps)
            q, k, v = W[p + "attn_q.weight"] @ xn, W[p + "attn_k.weight"] @ xn, W[p + "attn_v.weight"] @ xn
            q, k = rope(q, H, pos), rope(k, KH, pos)
            kc[l] = np.concatenate([kc[l], k[None]], 0)
            vc[l] = np.concatenate([vc[l], v[None]], 0)
            att = np.zeros(H * D, np.float32)
            for h in range(H):
                kh = h // (H // KH)
                sc = (kc[l][:, kh * D:(kh + 1) * D] @ q[h * D:(h + 1) * D]) * np.float32(1.0 / np.sqrt(np.float32(D)))
                e = np.exp(sc - sc.max()).astype(np.float32)
                a = e * np.float32(1.0 / float(e.astype(np.float64).sum()))
                att[h * D:(h + 1) * D] = a @ vc[l][:, kh * D:(kh + 1) * D]
            x = add_partials(x, W[p + "attn_output.weight"] @ att) if cut == "rows+cols" else x + gather(W[p + "attn_output.weight"] @ gather(att))
            xn = _rms_norm(x, N[p + "ffn_norm.weight"], cfg.rms_eps)
            g, u = W[p + "ffn_gate.weight"] @ xn, W[p + "ffn_up.weight"] @ xn
            hid = ((g / (np.float32(1.0) + np.exp(-g))) * u).astype(np.float32)
            x = add_partials(x, W[p + "ffn_down.weight"] @ hid) if cut == "rows+cols" else x + gather(W[p + "ffn_down.weight"] @ gather(hid))
        return gather(W["output.weight"] @ _rms_norm(x, N["output_norm.weight"], cfg.rms_eps))

    def pick(logits: np.ndarray) -> int:
        finite = np.isfinite(logits)
        return int(np.argmax(np.where(finite, logits, -np.inf))) if finite.any() else -1   # argmax returns the first maximum

    logits, pos = None, 0
    for t in prompt:
        logits = forward(int(t), pos)
        pos += 1
    ids = []
    for n in range(max_new):
        ids.append(pick(logits))
        if n + 1 < max_new:
            logits = forward(ids[-1], pos)
            pos += 1
    return ids, logits

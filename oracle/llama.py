"""CPU restatement (numpy) of the reference's dense Llama decode step, for checking the device decoder.

TEST INFRASTRUCTURE ONLY: tests/ import this; the product (zeninfer_b200/) never does.

Follows DenseTransformerRuntime::forward for `general.architecture = llama`
(src/adapters/dense_transformer_runtime.cpp): embedding row decode :3692, rms_norm :117-125 (sum of squares in
double, inv = 1/sqrt(float(ss/n) + eps)), projections as fp32-activation products over the decoded Q8_0 weights
(the reference's default CPU route, kernels/avx2.cpp:587-641), adjacent-pair rope :300-329, attention :4284-4337
(scores / sqrt(D), exp(score - max), double denominator, a = score * (1/denominator)), silu_mul :193-199, greedy
pick :391-418.  Pinned by tests/golden/llama_tiny.npz, which the unmodified reference produced.

int8_single_token=True restates the reference run with ZEN_CPU_Q8_ACT=1: every single-token product (all of a decode
step, and the lm_head after the prompt) quantises its input to int8 per 32-element block (src/quant.cpp:1094-1113) and
sums exact int32 block dot products scaled by d_w * d_x (kernels/avx2.cpp:562-585), while the prompt block's layer
products stay fp32-activation (the reference routes tokens >= 2 to its fp32 GEMM, src/quant.cpp:1667-1680).  Pinned by
ids_int8 / last_logits_int8 of the same file.
"""
from __future__ import annotations

import numpy as np


def _dequant_q8_0(packed: np.ndarray, rows: int, cols: int) -> np.ndarray:
    b = np.ascontiguousarray(packed, np.uint8).reshape(rows, cols // 32, 34)
    d = b[..., :2].copy().view(np.float16).astype(np.float32)          # [rows, nb, 1]
    q = b[..., 2:].view(np.int8).astype(np.float32)                      # [rows, nb, 32]
    return (q * d).reshape(rows, cols)


def _split_q8_0(packed: np.ndarray, rows: int, cols: int):
    b = np.ascontiguousarray(packed, np.uint8).reshape(rows, cols // 32, 34)
    return b[..., 2:].view(np.int8).astype(np.int32), b[..., :2].copy().view(np.float16).astype(np.float32)[..., 0]


def _quantise_acts(x: np.ndarray):
    """quantise_acts_q8_0 (kernels/avx2.cpp:502-524): d = amax / 127, inv = 1 / d, q = lround(clamp(x * inv, +-127))."""
    xb = np.asarray(x, np.float32).reshape(-1, 32)
    amax = np.abs(xb).max(axis=1)
    d = np.where(amax > 0, amax / np.float32(127.0), np.float32(0.0)).astype(np.float32)
    inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    v = np.clip((xb * inv[:, None]).astype(np.float32), np.float32(-127.0), np.float32(127.0))
    q = (np.trunc(v) + np.where(np.abs(v - np.trunc(v)) >= 0.5, np.sign(v), 0)).astype(np.int32)   # round half away from zero
    return q, d


def _matvec_int8(qw: np.ndarray, dw: np.ndarray, x: np.ndarray) -> np.ndarray:
    qx, dx = _quantise_acts(x)
    isum = np.einsum("rbk,bk->rb", qw, qx)                       # exact int32 block dot products
    return ((dw * dx[None, :]) * isum.astype(np.float32)).astype(np.float32).sum(axis=1, dtype=np.float32)


def _rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    ss = float(np.sum(x.astype(np.float64) ** 2))
    inv = np.float32(1.0) / np.sqrt(np.float32(ss / x.size) + np.float32(eps), dtype=np.float32)
    return (x * inv * w).astype(np.float32)


def generate(cfg, tensors: dict, shapes: dict, prompt, max_new: int, rank: int = 0, world: int = 1, gather=None, cut: str = "rows",
             int8_single_token: bool = False):
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
    if int8_single_token and world != 1:
        raise ValueError("the int8 restatement is unsharded")
    Q = {n: _split_q8_0(a, *shapes[n]) for n, a in tensors.items() if len(shapes[n]) == 2} if int8_single_token else {}
    int8_now = [False]

    def mv(name: str, x: np.ndarray) -> np.ndarray:
        return _matvec_int8(*Q[name], x) if int8_now[0] else W[name] @ x

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
            q, k, v = mv(p + "attn_q.weight", xn), mv(p + "attn_k.weight", xn), mv(p + "attn_v.weight", xn)
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
            x = add_partials(x, mv(p + "attn_output.weight", att)) if cut == "rows+cols" else x + gather(mv(p + "attn_output.weight", gather(att)))
            xn = _rms_norm(x, N[p + "ffn_norm.weight"], cfg.rms_eps)
            g, u = mv(p + "ffn_gate.weight", xn), mv(p + "ffn_up.weight", xn)
            hid = ((g / (np.float32(1.0) + np.exp(-g))) * u).astype(np.float32)
            x = add_partials(x, mv(p + "ffn_down.weight", hid)) if cut == "rows+cols" else x + gather(mv(p + "ffn_down.weight", gather(hid)))
        return x

    def head(x: np.ndarray) -> np.ndarray:
        return gather(mv("output.weight", _rms_norm(x, N["output_norm.weight"], cfg.rms_eps)))

    def pick(logits: np.ndarray) -> int:
        finite = np.isfinite(logits)
        return int(np.argmax(np.where(finite, logits, -np.inf))) if finite.any() else -1   # argmax returns the first maximum

    x, pos = None, 0
    for t in prompt:                      # the prompt block: fp32-activation products in every layer
        x = forward(int(t), pos)
        pos += 1
    int8_now[0] = int8_single_token       # from the prompt's lm_head on, every product is a single-token product
    logits = head(x)
    ids = []
    for n in range(max_new):
        ids.append(pick(logits))
        if n + 1 < max_new:
            logits = head(forward(ids[-1], pos))
            pos += 1
    return ids, logits

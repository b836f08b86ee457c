"""Small, self-contained launches of the hot kernels for a profiler capture: a few launches of one kernel, a few hundred
megabytes on the device at most, inputs larger than L2 where DRAM figures matter.

    python -m zeninfer_b200.profile_cases gemm                       # Q8_0 prefill product 512 x 14336 x 4096, four launches
    python -m zeninfer_b200.profile_cases gemv Q6_K 14336 4096 [T]   # decode product of one format, six launches over three copies
    python -m zeninfer_b200.profile_cases attention_prefill          # causal block attention, 512 tokens, 32/8 heads of 128, three launches

Run the same command once without the profiler first; then, for instance,
    ncu --set full --clock-control none -k regex:gemm_q8_0_i8 -s 2 -c 1 -o out python -m zeninfer_b200.profile_cases gemm
"""
from __future__ import annotations

import sys

import numpy as np


def case_gemm() -> None:
    import torch
    from . import Backend, blocks
    tokens, rows, cols = 512, 14336, 4096
    be = Backend()
    w = np.random.default_rng(3).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
    packed = np.ascontiguousarray(blocks.quantize_q8_0(w))
    handles = [be.dev_upload("Q8_0", packed, rows, cols) for _ in range(2)]
    x = torch.randn(tokens, cols, device="cuda")
    outs = [torch.zeros(tokens, rows, device="cuda") for _ in range(2)]
    nbytes = be.gemm_workspace_bytes(tokens, cols)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    st = torch.cuda.Stream()
    for _ in range(2):
        for h, o in zip(handles, outs):
            be.dev_gemm_q8_0([h], [o.data_ptr()], x.data_ptr(), tokens, ws.data_ptr(), nbytes, st.cuda_stream)
    st.synchronize()
    be.dev_check(st.cuda_stream)
    print("ok", float(outs[0].abs().sum()))


def case_gemv(fmt: str, rows: int, cols: int, tokens: int = 1) -> None:
    import torch
    from . import Backend, blocks
    from .backend import ACT_FP32, FORMAT_IDS
    be = Backend()
    if fmt in ("Q4_K", "Q5_K"):
        packed = blocks.random_k_blocks(FORMAT_IDS[fmt], rows, cols, 4)
    else:
        w = np.random.default_rng(4).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
        packed = np.ascontiguousarray(blocks.quantize(FORMAT_IDS[fmt], w))
    handles = [be.dev_upload(fmt, packed, rows, cols) for _ in range(3)]
    x = torch.randn(tokens, cols, device="cuda")
    y = torch.zeros(tokens, rows, device="cuda")
    st = torch.cuda.Stream()
    for _ in range(2):
        for h in handles:
            be.dev_gemv([h], [y.data_ptr()], x.data_ptr(), tokens, ACT_FP32, st.cuda_stream)
    st.synchronize()
    be.dev_check(st.cuda_stream)
    print("ok", float(y.abs().sum()))


def case_attention_prefill() -> None:
    import torch
    from . import Backend
    be = Backend()
    dev = torch.device("cuda")
    st = torch.cuda.Stream()
    q_width, kv_width, heads, kv_heads, head_dim, positions, tokens = 4096, 1024, 32, 8, 128, 1024, 512
    q, att = torch.randn(tokens, q_width, device=dev), torch.zeros(tokens, q_width, device=dev)
    kc, vc = torch.randn(positions, kv_width, device=dev), torch.randn(positions, kv_width, device=dev)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    for _ in range(3):
        be.dev_attention_prefill(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), att.data_ptr(), tokens, heads, kv_heads, head_dim,
                                 positions, 0.0, 0, st.cuda_stream)
    st.synchronize()
    be.dev_check(st.cuda_stream)
    print("ok", float(att.abs().sum()))


def main(argv: list[str]) -> int:
    if len(argv) >= 1 and argv[0] == "gemm":
        case_gemm()
    elif len(argv) >= 4 and argv[0] == "gemv":
        case_gemv(argv[1], int(argv[2]), int(argv[3]), int(argv[4]) if len(argv) > 4 else 1)
    elif len(argv) >= 1 and argv[0] == "attention_prefill":
        case_attention_prefill()
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))

#!/usr/bin/env python
"""Writes a copy of the reference's src/quant.cpp with the CUDA backend hooked in, for the drop-in test.

    python tests/integration/apply_cuda_hooks.py <reference>/src/quant.cpp <out>/quant_cuda.cpp

The copy is made at build time and never committed: the reference's source stays where it is.  The hooks are the ones a
maintainer would add, placed beside the reference's own `#ifdef ZEN_HAS_HIP` blocks (src/quant.cpp:1007-1012 gemv,
:1457-1468 gemv_batch, :1528-1543 gemm_batch, :1656-1659 gemm, :1553-1580 ffn_gemv), and they count their attempts on the reference's own route
counters (g_gemv_routes / g_gemm_routes, :48-75).  The product hooks `return` their result: this backend has no CPU route
behind it, so a failed call is the caller's error, not a fall-through.  The ffn_gemv hook keeps the reference's own
contract for that function (false = "no backend took the fused FFN", after which the runtime issues the three products
separately).  Each anchor must match exactly once, or the script stops.
"""
import sys

INCLUDE = '''#ifdef ZEN_HAS_CUDA
#include "zen/cuda_backend.h"
#endif
'''

GEMV = '''#ifdef ZEN_HAS_CUDA
    if(scale==1.0f&&(f.encoding==Encoding::q8_0||f.encoding==Encoding::q6_k||f.encoding==Encoding::q4_0||f.encoding==Encoding::q4_k||f.encoding==Encoding::q5_k)&&zen::cuda::enabled()){
        g_gemv_routes.gpu_try.fetch_add(1,std::memory_order_relaxed);
        const bool ok=f.encoding==Encoding::q8_0?zen::cuda::gemv_q8_0(w,x,y,rows,cols):
                      f.encoding==Encoding::q6_k?zen::cuda::gemm_q6_k(w,x,y,1,rows,cols):
                      f.encoding==Encoding::q4_0?zen::cuda::gemm_q4_0(w,x,y,1,rows,cols):
                      zen::cuda::gemm_kquant(w,x,y,1,rows,cols,f.encoding==Encoding::q5_k);
        if(ok)g_gemv_routes.gpu_ok.fetch_add(1,std::memory_order_relaxed);
        return ok;
    }
#endif
'''

GEMV_BATCH = '''#ifdef ZEN_HAS_CUDA
    if(format.encoding==Encoding::q8_0&&scale==1.0f&&count>1&&count<=zen::cuda::kMaxBatch&&zen::cuda::enabled()){
        zen::cuda::GemvTask tasks[zen::cuda::kMaxBatch];
        for(std::size_t i=0;i<count;++i){
            if(!weights[i])return false;
            tasks[i]={weights[i],outputs[i],rows[i],columns};
        }
        g_gemv_routes.gpu_try.fetch_add(count,std::memory_order_relaxed);
        const bool ok=zen::cuda::gemv_q8_0_batch(input,tasks,count);
        if(ok)g_gemv_routes.gpu_ok.fetch_add(count,std::memory_order_relaxed);
        return ok;
    }
#endif
'''

GEMM_BATCH = '''    #ifdef ZEN_HAS_CUDA
    if(format.encoding==Encoding::q8_0&&scale==1.0f&&count>1&&count<=zen::cuda::kMaxBatch&&zen::cuda::enabled()){
        zen::cuda::GemmTask tasks[zen::cuda::kMaxBatch];
        for(std::size_t i=0;i<count;++i){
            if(!weights[i]||!outputs[i]||!rows[i])return false;
            tasks[i]={weights[i],outputs[i],rows[i]};
        }
        g_gemm_routes.gpu_try.fetch_add(count,std::memory_order_relaxed);
        const bool ok=zen::cuda::gemm_q8_0_batch(input,tasks,count,tokens,columns);
        if(ok)g_gemm_routes.gpu_ok.fetch_add(count,std::memory_order_relaxed);
        return ok;
    }
    #endif
'''

GEMM = '''#ifdef ZEN_HAS_CUDA
    if(scale==1.0f&&(f.encoding==Encoding::q8_0||f.encoding==Encoding::q6_k||f.encoding==Encoding::q4_0||f.encoding==Encoding::q4_k||f.encoding==Encoding::q5_k)&&zen::cuda::enabled()){
        g_gemm_routes.gpu_try.fetch_add(1,std::memory_order_relaxed);
        const bool ok=f.encoding==Encoding::q8_0?zen::cuda::gemm_q8_0(w,input,output,tokens,rows,cols):
                      f.encoding==Encoding::q6_k?zen::cuda::gemm_q6_k(w,input,output,tokens,rows,cols):
                      f.encoding==Encoding::q4_0?zen::cuda::gemm_q4_0(w,input,output,tokens,rows,cols):
                      zen::cuda::gemm_kquant(w,input,output,tokens,rows,cols,f.encoding==Encoding::q5_k);
        if(ok)g_gemm_routes.gpu_ok.fetch_add(1,std::memory_order_relaxed);
        return ok;
    }
#endif
'''

FFN = '''#ifdef ZEN_HAS_CUDA
    if(gate_format.encoding==Encoding::q8_0&&up_format.encoding==Encoding::q8_0&&
       down_format.encoding==Encoding::q8_0&&zen::cuda::enabled()&&
       zen::cuda::gemv_q8_0_ffn(gate_weights,up_weights,down_weights,input,output,
                                ffn_rows,columns,output_rows))return true;
#endif
'''

# (anchor text that starts the line group the block goes BEFORE, block)
HOOKS = [
    ('#include "zen/compute_pool.h"\n', INCLUDE),
    ('#ifdef ZEN_HAS_HIP\n    // GPU residency is keyed by the weight pointer', GEMV),
    ('#ifdef ZEN_HAS_HIP\n    if(format.encoding==Encoding::q8_0&&scale==1.0f&&count>1&&count<=zen::hip::kMaxBatch', GEMV_BATCH),
    ('    // No GPU batch (gate off, HIP-only build', GEMM_BATCH),
    ('#ifdef ZEN_HAS_HIP\n    if(f.encoding==Encoding::q8_0&&scale==1.0f&&zen::hip::enabled()&&\n       zen::hip::gemm_q8_0(', GEMM),
    ('#ifdef ZEN_HAS_D3D12\n    if(gate_format.encoding==Encoding::q8_0&&up_format.encoding==Encoding::q8_0&&\n'
     '       down_format.encoding==Encoding::q8_0&&zen::d3d12::enabled()&&\n       zen::d3d12::gemv_q8_0_ffn(', FFN),
]


def main() -> None:
    src, dst = sys.argv[1], sys.argv[2]
    text = open(src, encoding="utf-8").read()
    for anchor, block in HOOKS:
        if text.count(anchor) != 1:
            raise SystemExit(f"anchor matched {text.count(anchor)} times, expected once: {anchor[:60]!r}")
        text = text.replace(anchor, block + anchor)
    with open(dst, "w", encoding="utf-8") as f:
        f.write(text)
    print("wrote", dst, "with", len(HOOKS), "hook blocks")


if __name__ == "__main__":
    main()

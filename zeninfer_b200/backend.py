"""ctypes binding of include/zen_cuda.h, shaped like the reference's dispatch layer.

``Backend.gemv / gemm / gemv_batch / gemm_batch`` take the same arguments, in the same order and with
the same meaning, as ``zen::quant::gemv / gemm / gemv_batch / gemm_batch`` (include/zen/quant.h:28-91):
a format name, host pointers to raw GGUF blocks, fp32 activations, token-major fp32 outputs.  Where
the reference returns ``false`` and lets the caller try its next route, this raises ``BackendError``:
the CUDA build has no other route.

NumPy arrays stand in for the reference's raw pointers.  A weight array must stay alive (and keep its
address) while it is resident, exactly as the reference requires of the loader's file mapping
(include/zen/hip_backend.h:52-58); call ``release_weights`` before dropping it.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import numpy as np

from . import blocks

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_PKG, "lib", "libzen_cuda.so")

ACT_INT8, ACT_FP32 = 1, 2
FORMAT_IDS = {"Q8_0": blocks.Q8_0, "Q4_0": blocks.Q4_0, "Q6_K": blocks.Q6_K, "Q4_K": blocks.Q4_K, "Q5_K": blocks.Q5_K}

# every symbol include/zen_cuda.h declares; the CPU test-suite checks the library exports them all
ABI_SYMBOLS = (
    "zen_cuda_enabled", "zen_cuda_init", "zen_cuda_shutdown", "zen_cuda_info", "zen_cuda_get_stats",
    "zen_cuda_last_error", "zen_cuda_set_q8_act_mode", "zen_cuda_get_q8_act_mode",
    "zen_cuda_gemv_q8_0", "zen_cuda_gemm_q8_0", "zen_cuda_gemv_q8_0_batch", "zen_cuda_gemm_q8_0_batch",
    "zen_cuda_gemm_q6_k", "zen_cuda_gemm_q4_0", "zen_cuda_gemm_kquant", "zen_cuda_release_weights", "zen_cuda_quantize_acts",
    "zen_cuda_rms_norm", "zen_cuda_gemv_q8_0_ffn", "zen_cuda_set_vram_budget", "zen_cuda_residency", "zen_cuda_set_q6k_codes", "zen_cuda_set_gemm_groups",
    "zen_cuda_dev_upload", "zen_cuda_dev_free", "zen_cuda_dev_weight_bytes", "zen_cuda_dev_gemv",
    "zen_cuda_dev_quantize_acts", "zen_cuda_dev_check", "zen_cuda_error_name", "zen_cuda_set_wait_budget_ms",
    "zen_cuda_gemv_list_create", "zen_cuda_gemv_list_destroy", "zen_cuda_gemv_list_bytes", "zen_cuda_dev_gemv_list",
    "zen_cuda_gemm_workspace_bytes", "zen_cuda_dev_gemm_q8_0", "zen_cuda_gemm_workspace_bytes_act", "zen_cuda_dev_gemm_q8_0_act",
    "zen_cuda_gemm_q6_k_workspace_bytes", "zen_cuda_dev_gemm_q6_k", "zen_cuda_gemm_q4_0_workspace_bytes", "zen_cuda_dev_gemm_q4_0",
    "zen_cuda_gemm_kquant_workspace_bytes", "zen_cuda_dev_gemm_kquant",
    "zen_cuda_dev_gemm_q8_0_noalloc",
    "zen_cuda_gather_region_bytes", "zen_cuda_ipc_alloc", "zen_cuda_ipc_open", "zen_cuda_ipc_close", "zen_cuda_ipc_free",
    "zen_cuda_gather_create", "zen_cuda_gather_destroy", "zen_cuda_dev_gemv_gather", "zen_cuda_dev_gather_fetch", "zen_cuda_dev_allgather", "zen_cuda_dev_allreduce_add",
    "zen_cuda_dev_greedy_pick", "zen_cuda_dev_sample",
    "zen_cuda_dev_embed_q8_0", "zen_cuda_dev_rms_norm", "zen_cuda_dev_rope_kv_append", "zen_cuda_dev_attention", "zen_cuda_dev_silu_mul",
    "zen_cuda_dev_advance_position", "zen_cuda_dev_gemv_swiglu", "zen_cuda_dev_attention_block", "zen_cuda_dev_gemv_fused",
    "zen_cuda_dev_embed_rows_q8_0", "zen_cuda_dev_rope_kv_append_rows", "zen_cuda_dev_attention_prefill",
)


class BackendError(RuntimeError):
    pass


class AdapterInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("dedicated_vram", C.c_uint64), ("shared_memory", C.c_uint64),
                ("sm_count", C.c_int), ("warp_size", C.c_int), ("arch", C.c_char * 64)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "dispatches", "submits", "batches", "upload_bytes", "weight_bytes", "upload_us", "alloc_us", "stage_us",
        "repack_us", "transfer_us", "wait_us", "launch_us", "readback_us", "gpu_us", "fallbacks")]

    def as_dict(self) -> dict:
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class GemvTask(C.Structure):
    _fields_ = [("weights", C.c_void_p), ("y", C.c_void_p), ("rows", C.c_size_t), ("columns", C.c_size_t)]


class GemmTask(C.Structure):
    _fields_ = [("weights", C.c_void_p), ("y", C.c_void_p), ("rows", C.c_size_t)]


class GemvFusion(C.Structure):
    _fields_ = [("norm_weight", C.c_void_p), ("norm_eps", C.c_float), ("accumulate", C.c_int), ("gate", C.c_void_p), ("warm_next", C.c_void_p), ("swiglu_pair", C.c_int)]


class GemvListItem(C.Structure):
    _fields_ = [("w", C.POINTER(C.c_void_p)), ("d_y", C.POINTER(C.c_void_p)), ("count", C.c_size_t), ("d_x", C.c_void_p),
                ("fusion", GemvFusion), ("depends_on_earlier_items", C.c_int)]


class PickSegment(C.Structure):
    _fields_ = [("base", C.c_void_p), ("len", C.c_uint32), ("first_index", C.c_uint32), ("token_stride", C.c_uint32), ("reserved", C.c_uint32)]


def load_library(path: str | None = None) -> C.CDLL:
    """dlopen the backend.  Raises BackendError when it has not been built: there is no fallback."""
    path = path or os.environ.get("ZEN_CUDA_LIB") or _LIB_PATH   # ZEN_CUDA_LIB: an alternative build of the library
    if not os.path.exists(path):
        raise BackendError(f"{path} is missing: build it with `python -m zeninfer_b200.build` (needs nvcc)")
    lib = C.CDLL(path)
    vp, sz, i = C.c_void_p, C.c_size_t, C.c_int
    lib.zen_cuda_enabled.restype = i
    lib.zen_cuda_init.restype = i
    lib.zen_cuda_shutdown.restype = None
    lib.zen_cuda_info.argtypes = [C.POINTER(AdapterInfo)]
    lib.zen_cuda_get_stats.argtypes = [C.POINTER(Stats)]
    lib.zen_cuda_get_stats.restype = None
    lib.zen_cuda_last_error.restype = C.c_char_p
    lib.zen_cuda_set_q8_act_mode.argtypes = [i]
    lib.zen_cuda_gemv_q8_0.argtypes = [vp, vp, vp, sz, sz]
    lib.zen_cuda_gemm_q8_0.argtypes = [vp, vp, vp, sz, sz, sz]
    lib.zen_cuda_gemv_q8_0_batch.argtypes = [vp, C.POINTER(GemvTask), sz]
    lib.zen_cuda_gemm_q8_0_batch.argtypes = [vp, C.POINTER(GemmTask), sz, sz, sz]
    lib.zen_cuda_gemm_q6_k.argtypes = [vp, vp, vp, sz, sz, sz]
    lib.zen_cuda_gemm_q4_0.argtypes = [vp, vp, vp, sz, sz, sz]
    lib.zen_cuda_gemm_kquant.argtypes = [vp, vp, vp, sz, sz, sz, C.c_int]
    lib.zen_cuda_release_weights.argtypes = [vp]
    lib.zen_cuda_rms_norm.argtypes = [vp, vp, vp, sz, sz, C.c_float]
    lib.zen_cuda_gemv_q8_0_ffn.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz]
    lib.zen_cuda_set_vram_budget.argtypes = [C.c_uint64]
    lib.zen_cuda_residency.argtypes = [C.POINTER(C.c_uint64)] * 4
    lib.zen_cuda_release_weights.restype = None
    lib.zen_cuda_quantize_acts.argtypes = [vp, vp, vp, sz, sz]
    lib.zen_cuda_dev_upload.argtypes = [i, vp, sz, sz, sz, sz]
    lib.zen_cuda_dev_upload.restype = vp
    lib.zen_cuda_dev_free.argtypes = [vp]
    lib.zen_cuda_dev_free.restype = None
    lib.zen_cuda_dev_weight_bytes.argtypes = [vp]
    lib.zen_cuda_dev_weight_bytes.restype = sz
    lib.zen_cuda_dev_gemv.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, vp, sz, i, vp]
    lib.zen_cuda_dev_quantize_acts.argtypes = [vp, vp, vp, sz, sz, vp]
    lib.zen_cuda_dev_gemv_swiglu.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, vp, vp, sz, i, vp]
    lib.zen_cuda_dev_gemv_fused.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, vp, sz, i, C.POINTER(GemvFusion), vp]
    lib.zen_cuda_gemv_list_create.argtypes = [C.POINTER(GemvListItem), sz, i]
    lib.zen_cuda_gemv_list_create.restype = vp
    lib.zen_cuda_gemv_list_destroy.argtypes = [vp]
    lib.zen_cuda_gemv_list_destroy.restype = None
    lib.zen_cuda_gemv_list_bytes.argtypes = [vp]
    lib.zen_cuda_gemv_list_bytes.restype = C.c_uint64
    lib.zen_cuda_dev_gemv_list.argtypes = [vp, vp]
    lib.zen_cuda_dev_check.argtypes = [vp]
    lib.zen_cuda_error_name.argtypes = [i]
    lib.zen_cuda_error_name.restype = C.c_char_p
    lib.zen_cuda_set_wait_budget_ms.argtypes = [C.c_uint]
    lib.zen_cuda_gemm_workspace_bytes.argtypes = [sz, sz]
    lib.zen_cuda_gemm_workspace_bytes.restype = sz
    lib.zen_cuda_dev_gemm_q8_0.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, vp, sz, vp, sz, vp]
    lib.zen_cuda_gemm_workspace_bytes_act.argtypes = [sz, sz, i]
    lib.zen_cuda_gemm_workspace_bytes_act.restype = sz
    lib.zen_cuda_dev_gemm_q8_0_act.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, vp, sz, i, vp, sz, vp]
    lib.zen_cuda_gemm_q6_k_workspace_bytes.argtypes = [sz, sz]
    lib.zen_cuda_gemm_q6_k_workspace_bytes.restype = sz
    lib.zen_cuda_dev_gemm_q6_k.argtypes = [vp, vp, vp, sz, vp, sz, vp]
    lib.zen_cuda_gemm_q4_0_workspace_bytes.argtypes = [sz, sz, sz]
    lib.zen_cuda_gemm_q4_0_workspace_bytes.restype = sz
    lib.zen_cuda_dev_gemm_q4_0.argtypes = [vp, vp, vp, sz, vp, sz, vp]
    lib.zen_cuda_gemm_kquant_workspace_bytes.argtypes = [sz, sz, sz]
    lib.zen_cuda_gemm_kquant_workspace_bytes.restype = sz
    lib.zen_cuda_dev_gemm_kquant.argtypes = [vp, vp, vp, sz, vp, sz, vp]
    lib.zen_cuda_dev_gemm_q8_0_noalloc.argtypes = [vp, vp, vp, sz, vp]
    lib.zen_cuda_gather_region_bytes.argtypes = [sz, sz]
    lib.zen_cuda_gather_region_bytes.restype = sz
    lib.zen_cuda_ipc_alloc.argtypes = [sz, vp]
    lib.zen_cuda_ipc_alloc.restype = vp
    lib.zen_cuda_ipc_open.argtypes = [vp]
    lib.zen_cuda_ipc_open.restype = vp
    lib.zen_cuda_ipc_close.argtypes = [vp]
    lib.zen_cuda_ipc_close.restype = None
    lib.zen_cuda_ipc_free.argtypes = [vp]
    lib.zen_cuda_ipc_free.restype = None
    lib.zen_cuda_gather_create.argtypes = [sz, sz, sz, C.POINTER(vp)]
    lib.zen_cuda_gather_create.restype = vp
    lib.zen_cuda_gather_destroy.argtypes = [vp]
    lib.zen_cuda_gather_destroy.restype = None
    lib.zen_cuda_dev_gemv_gather.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), sz, vp, sz, i, vp]
    lib.zen_cuda_dev_gather_fetch.argtypes = [vp, vp, vp]
    lib.zen_cuda_dev_allgather.argtypes = [vp, vp, sz, vp, vp]
    lib.zen_cuda_dev_allreduce_add.argtypes = [vp, vp, sz, vp, vp]
    lib.zen_cuda_dev_greedy_pick.argtypes = [C.POINTER(PickSegment), sz, sz, vp, vp]
    lib.zen_cuda_dev_sample.argtypes = [vp, sz, C.c_float, C.c_uint32, C.c_float, C.c_double, vp, vp, vp, vp, vp, vp]
    lib.zen_cuda_dev_embed_q8_0.argtypes = [vp, vp, vp, vp]
    lib.zen_cuda_dev_rms_norm.argtypes = [vp, vp, vp, vp, sz, sz, C.c_float, vp]
    lib.zen_cuda_dev_rope_kv_append.argtypes = [vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, i, vp, vp, sz, vp]
    lib.zen_cuda_dev_attention.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, C.c_float, sz, sz, vp]
    lib.zen_cuda_dev_silu_mul.argtypes = [vp, vp, vp, sz, vp]
    lib.zen_cuda_dev_embed_rows_q8_0.argtypes = [vp, vp, sz, vp, vp]
    lib.zen_cuda_dev_rope_kv_append_rows.argtypes = [vp, vp, vp, sz, vp, vp, vp, sz, sz, sz, sz, i, vp, vp, sz, vp]
    lib.zen_cuda_dev_attention_prefill.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz, C.c_float, sz, sz, vp]
    lib.zen_cuda_dev_attention_block.argtypes = [vp, vp, vp, vp, vp, sz, vp, vp, vp, vp, sz, sz, sz, C.c_float, sz, sz, vp]
    lib.zen_cuda_dev_advance_position.argtypes = [vp, i, vp]
    return lib


def _addr(a: np.ndarray) -> int:
    return a.ctypes.data


class Backend:
    """One process, one GPU (the device is LOCAL_RANK when launched under torchrun)."""

    def __init__(self, lib_path: str | None = None) -> None:
        self.lib = load_library(lib_path)
        if not self.lib.zen_cuda_init():
            raise BackendError("zen_cuda_init failed: " + self.last_error())

    # ---- lifecycle (zen::hip::enabled/info/stats/shutdown) ----
    def enabled(self) -> bool:
        return bool(self.lib.zen_cuda_enabled())

    def last_error(self) -> str:
        return (self.lib.zen_cuda_last_error() or b"").decode()

    def info(self) -> dict:
        a = AdapterInfo()
        if not self.lib.zen_cuda_info(C.byref(a)):
            raise BackendError("backend not initialised")
        return {"name": a.name.decode(), "dedicated_vram": int(a.dedicated_vram), "shared_memory": int(a.shared_memory),
                "sm_count": a.sm_count, "warp_size": a.warp_size, "arch": a.arch.decode()}

    def stats(self) -> dict:
        s = Stats()
        self.lib.zen_cuda_get_stats(C.byref(s))
        return s.as_dict()

    def shutdown(self) -> None:
        self.lib.zen_cuda_shutdown()

    def set_q8_act_mode(self, mode: int) -> None:
        if not self.lib.zen_cuda_set_q8_act_mode(mode):
            raise BackendError("bad activation mode")

    def _fail(self, what: str):
        raise BackendError(f"{what}: {self.last_error()}")

    @staticmethod
    def _weights(w) -> np.ndarray:
        if not (isinstance(w, np.ndarray) and w.dtype == np.uint8 and w.flags["C_CONTIGUOUS"]):
            raise TypeError("weights must be a C-contiguous uint8 ndarray that outlives its residency")
        return w

    # ---- zen::quant::gemv / gemm / gemv_batch / gemm_batch ----
    def gemv(self, fmt: str, weights: np.ndarray, x, rows: int, columns: int) -> np.ndarray:
        return self.gemm(fmt, weights, np.asarray(x, np.float32).reshape(1, columns), 1, rows, columns)[0]

    def gemm(self, fmt: str, weights: np.ndarray, x, tokens: int, rows: int, columns: int) -> np.ndarray:
        w = self._weights(weights)
        x = np.ascontiguousarray(x, np.float32).reshape(tokens, columns)
        out = np.empty((tokens, rows), np.float32)
        if fmt == "Q8_0":
            ok = (self.lib.zen_cuda_gemv_q8_0(_addr(w), _addr(x), _addr(out), rows, columns) if tokens == 1
                  else self.lib.zen_cuda_gemm_q8_0(_addr(w), _addr(x), _addr(out), tokens, rows, columns))
        elif fmt == "Q6_K":
            ok = self.lib.zen_cuda_gemm_q6_k(_addr(w), _addr(x), _addr(out), tokens, rows, columns)
        elif fmt == "Q4_0":
            ok = self.lib.zen_cuda_gemm_q4_0(_addr(w), _addr(x), _addr(out), tokens, rows, columns)
        elif fmt in ("Q4_K", "Q5_K"):
            ok = self.lib.zen_cuda_gemm_kquant(_addr(w), _addr(x), _addr(out), tokens, rows, columns, int(fmt == "Q5_K"))
        else:
            raise BackendError(f"format {fmt} is not on this path")
        if not ok:
            self._fail(f"{fmt} product {tokens}x{rows}x{columns}")
        return out

    def gemv_batch(self, fmt: str, weights: Sequence[np.ndarray], x, rows: Sequence[int], columns: int) -> list[np.ndarray]:
        return [o[0] for o in self.gemm_batch(fmt, weights, np.asarray(x, np.float32).reshape(1, columns), rows, 1, columns)]

    def gemm_batch(self, fmt: str, weights: Sequence[np.ndarray], x, rows: Sequence[int], tokens: int, columns: int) -> list[np.ndarray]:
        if fmt != "Q8_0":  # the reference batches Q8_0 only and loops otherwise (src/quant.cpp:1499-1501)
            return [self.gemm(fmt, w, x, tokens, r, columns) for w, r in zip(weights, rows)]
        x = np.ascontiguousarray(x, np.float32).reshape(tokens, columns)
        outs = [np.empty((tokens, r), np.float32) for r in rows]
        n = len(outs)
        if tokens == 1:
            tasks = (GemvTask * n)(*[GemvTask(_addr(self._weights(w)), _addr(o), r, columns) for w, o, r in zip(weights, outs, rows)])
            ok = self.lib.zen_cuda_gemv_q8_0_batch(_addr(x), tasks, n)
        else:
            tasks = (GemmTask * n)(*[GemmTask(_addr(self._weights(w)), _addr(o), r) for w, o, r in zip(weights, outs, rows)])
            ok = self.lib.zen_cuda_gemm_q8_0_batch(_addr(x), tasks, n, tokens, columns)
        if not ok:
            self._fail("Q8_0 batched product")
        return outs

    def release_weights(self, weights: np.ndarray) -> None:
        self.lib.zen_cuda_release_weights(_addr(weights))

    def rms_norm(self, x, weight, epsilon: float) -> np.ndarray:
        """zen::hip::rms_norm (include/zen/hip_backend.h:74-76): x [rows, columns] normalised row by row, times weight."""
        x = np.ascontiguousarray(x, np.float32)
        weight = np.ascontiguousarray(weight, np.float32)
        rows, columns = x.reshape(-1, x.shape[-1]).shape
        y = np.empty_like(x)
        if not self.lib.zen_cuda_rms_norm(_addr(x), _addr(weight), _addr(y), rows, columns, epsilon):
            self._fail(f"rms_norm {rows}x{columns}")
        return y

    def gemv_ffn(self, gate: np.ndarray, up: np.ndarray, down: np.ndarray, x, ffn_rows: int, columns: int, out_rows: int) -> np.ndarray:
        """zen::hip::gemv_q8_0_ffn (include/zen/hip_backend.h:78-83): down * (silu(gate * x) * (up * x)), raw Q8_0 tensors."""
        x = np.ascontiguousarray(x, np.float32).reshape(columns)
        y = np.empty(out_rows, np.float32)
        if not self.lib.zen_cuda_gemv_q8_0_ffn(_addr(self._weights(gate)), _addr(self._weights(up)), _addr(self._weights(down)), _addr(x), _addr(y),
                                               ffn_rows, columns, out_rows):
            self._fail(f"gemv_q8_0_ffn {ffn_rows}x{columns} -> {out_rows}")
        return y

    def set_q6k_codes(self, on: bool) -> bool:
        """Device layout of Q6_K tensors uploaded from now on: unpacked int8 codes (True, the default) or the file's
        ql | qh planes.  Returns the previous setting."""
        before = self.lib.zen_cuda_set_q6k_codes(int(bool(on)))
        if before < 0:
            self._fail("set_q6k_codes")
        return bool(before)

    def set_gemm_groups(self, on: bool) -> bool:
        """Q8_0 many-row products through the group-scale kernel (True, the default) or the per-block kernel.  Returns the
        previous setting."""
        before = self.lib.zen_cuda_set_gemm_groups(int(bool(on)))
        if before < 0:
            self._fail("set_gemm_groups")
        return bool(before)

    def set_vram_budget(self, nbytes: int) -> None:
        """Residency budget of the pointer-keyed weights in bytes; 0 restores 80 % of the device's memory."""
        if not self.lib.zen_cuda_set_vram_budget(int(nbytes)):
            self._fail("set_vram_budget")

    def residency(self) -> dict:
        v = [C.c_uint64() for _ in range(4)]
        if not self.lib.zen_cuda_residency(*[C.byref(c) for c in v]):
            self._fail("residency")
        return dict(zip(("budget_bytes", "held_bytes", "tensors", "evictions"), (int(c.value) for c in v)))

    def quantize_acts(self, x) -> tuple[np.ndarray, np.ndarray]:
        """fp32 [tokens, K] -> (int8 codes [tokens, K], fp32 scales [tokens, K/32]); quantise_acts_q8_0 on the device."""
        x = np.ascontiguousarray(x, np.float32)
        tokens, k = x.reshape(-1, x.shape[-1]).shape
        q = np.empty((tokens, k), np.int8)
        sc = np.empty((tokens, k // 32), np.float32)
        if not self.lib.zen_cuda_quantize_acts(_addr(x), _addr(q), _addr(sc), tokens, k):
            self._fail("quantize_acts")
        return q.reshape(x.shape), sc.reshape(x.shape[:-1] + (k // 32,))

    # ---- device-pointer calls (addresses are plain ints, e.g. torch.Tensor.data_ptr()) ----
    def dev_upload(self, fmt: str, weights: np.ndarray, rows_total: int, columns: int, first_row: int = 0, nrows: int | None = None) -> int:
        nrows = rows_total - first_row if nrows is None else nrows
        h = self.lib.zen_cuda_dev_upload(FORMAT_IDS[fmt], _addr(self._weights(weights)), rows_total, columns, first_row, nrows)
        if not h:
            self._fail(f"upload {fmt} {nrows}x{columns}")
        return h

    def dev_free(self, handle: int) -> None:
        self.lib.zen_cuda_dev_free(handle)

    def dev_weight_bytes(self, handle: int) -> int:
        return int(self.lib.zen_cuda_dev_weight_bytes(handle))

    def dev_gemv(self, handles: Sequence[int], d_y: Sequence[int], d_x: int, tokens: int, act_mode: int, stream: int = 0) -> None:
        n = len(handles)
        hs = (C.c_void_p * n)(*handles)
        ys = (C.c_void_p * n)(*d_y)
        if not self.lib.zen_cuda_dev_gemv(hs, ys, n, d_x, tokens, act_mode, stream):
            self._fail("dev_gemv")

    def dev_gemv_swiglu(self, handles: Sequence[int], d_y: Sequence[int], d_gate: int, d_up: int, tokens: int, act_mode: int, stream: int = 0) -> None:
        """dev_gemv whose input is silu(gate) * up, formed inside the product kernel (Q8_0 only)."""
        n = len(handles)
        hs = (C.c_void_p * n)(*handles)
        ys = (C.c_void_p * n)(*d_y)
        if not self.lib.zen_cuda_dev_gemv_swiglu(hs, ys, n, d_gate, d_up, tokens, act_mode, stream):
            self._fail("dev_gemv_swiglu")

    def dev_gemv_fused(self, handles: Sequence[int], d_y: Sequence[int], d_x: int, tokens: int, act_mode: int, stream: int = 0, *,
                       norm_weight: int | None = None, norm_eps: float = 0.0, gate: int | None = None, accumulate: bool = False,
                       warm_next: int | None = None, swiglu_pair: bool = False) -> None:
        """dev_gemv (Q8_0) with RMSNorm or SwiGLU applied to the input inside the launch and/or y += W x; warm_next
        names the tensor the stream's next product reads, whose start this launch pulls into L2; swiglu_pair: the two
        tensors are gate and up, and d_y[0] receives silu(gate . x) * (up . x)."""
        n = len(handles)
        hs = (C.c_void_p * n)(*handles)
        ys = (C.c_void_p * n)(*d_y)
        f = GemvFusion(norm_weight, norm_eps, int(accumulate), gate, warm_next, int(swiglu_pair))
        if not self.lib.zen_cuda_dev_gemv_fused(hs, ys, n, d_x, tokens, act_mode, C.byref(f), stream):
            self._fail("dev_gemv_fused")

    def gemv_list_create(self, items: Sequence[dict], act_mode: int) -> int:
        """Builds a list of batch-1 Q8_0 products for one persistent launch (zen_cuda_gemv_list_create).  An item is a dict:
        handles, d_y (device addresses), d_x, and optionally norm_weight, norm_eps, gate, accumulate (as dev_gemv_fused) and
        depends (True when the item reads or accumulates into what earlier items of the list write)."""
        n = len(items)
        arr = (GemvListItem * n)()
        keep = []
        for dst, it in zip(arr, items):
            k = len(it["handles"])
            hs, ys = (C.c_void_p * k)(*it["handles"]), (C.c_void_p * k)(*it["d_y"])
            keep.append((hs, ys))
            dst.w, dst.d_y, dst.count, dst.d_x = hs, ys, k, it["d_x"]
            dst.fusion = GemvFusion(it.get("norm_weight"), it.get("norm_eps", 0.0), int(bool(it.get("accumulate"))), it.get("gate"), None, 0)
            dst.depends_on_earlier_items = int(bool(it.get("depends")))
        h = self.lib.zen_cuda_gemv_list_create(arr, n, act_mode)
        if not h:
            self._fail("gemv_list_create")
        return int(h)

    def gemv_list_destroy(self, handle: int) -> None:
        self.lib.zen_cuda_gemv_list_destroy(handle)

    def gemv_list_bytes(self, handle: int) -> int:
        return int(self.lib.zen_cuda_gemv_list_bytes(handle))

    def dev_gemv_list(self, handle: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_gemv_list(handle, stream):
            self._fail("dev_gemv_list")

    def gemm_workspace_bytes(self, tokens: int, columns: int, act_mode: int = ACT_INT8) -> int:
        return int(self.lib.zen_cuda_gemm_workspace_bytes_act(tokens, columns, act_mode))

    def dev_gemm_q8_0(self, handles: Sequence[int], d_out: Sequence[int], d_x: int, tokens: int, workspace: int, workspace_bytes: int, stream: int = 0,
                      act_mode: int = ACT_INT8) -> None:
        """The tensor-core prefill product; act_mode ACT_FP32 takes two activation digits (fp32-equivalent results)."""
        n = len(handles)
        hs = (C.c_void_p * n)(*handles)
        outs = (C.c_void_p * n)(*d_out)
        if not self.lib.zen_cuda_dev_gemm_q8_0_act(hs, outs, n, d_x, tokens, act_mode, workspace, workspace_bytes, stream):
            self._fail("dev_gemm_q8_0")

    def gemm_q6_k_workspace_bytes(self, tokens: int, columns: int) -> int:
        return int(self.lib.zen_cuda_gemm_q6_k_workspace_bytes(tokens, columns))

    def dev_gemm_q6_k(self, handle: int, d_out: int, d_x: int, tokens: int, workspace: int, workspace_bytes: int, stream: int = 0) -> None:
        """Q6_K (codes unpacked on upload) times two or more activation rows on the tensor cores; out [tokens][rows]."""
        if not self.lib.zen_cuda_dev_gemm_q6_k(handle, d_out, d_x, tokens, workspace, workspace_bytes, stream):
            self._fail("dev_gemm_q6_k")

    def gemm_q4_0_workspace_bytes(self, tokens: int, rows: int, columns: int) -> int:
        return int(self.lib.zen_cuda_gemm_q4_0_workspace_bytes(tokens, rows, columns))

    def dev_gemm_q4_0(self, handle: int, d_out: int, d_x: int, tokens: int, workspace: int, workspace_bytes: int, stream: int = 0) -> None:
        """Q4_0 times many activation rows: nibbles widened to int8 codes in the workspace, then the Q8_0 tensor-core GEMM."""
        if not self.lib.zen_cuda_dev_gemm_q4_0(handle, d_out, d_x, tokens, workspace, workspace_bytes, stream):
            self._fail("dev_gemm_q4_0")

    def gemm_kquant_workspace_bytes(self, tokens: int, rows: int, columns: int) -> int:
        return int(self.lib.zen_cuda_gemm_kquant_workspace_bytes(tokens, rows, columns))

    def dev_gemm_kquant(self, handle: int, d_out: int, d_x: int, tokens: int, workspace: int, workspace_bytes: int, stream: int = 0) -> None:
        """Q4_K / Q5_K times many activation rows: codes widened to int8 in the workspace, then the tensor-core GEMM with
        fp32 sub-block scales and the minimum term in its epilogue."""
        if not self.lib.zen_cuda_dev_gemm_kquant(handle, d_out, d_x, tokens, workspace, workspace_bytes, stream):
            self._fail("dev_gemm_kquant")

    def dev_gemm_q8_0_noalloc(self, handle: int, d_out: int, d_x: int, tokens: int, stream: int = 0) -> None:
        """The prefill product for one resident tensor without any device allocation: the quantised activations live in a
        scratch array built into the library (see zen_cuda_dev_gemm_q8_0_noalloc in include/zen_cuda.h for the limits)."""
        if not self.lib.zen_cuda_dev_gemm_q8_0_noalloc(handle, d_out, d_x, tokens, stream):
            self._fail("dev_gemm_q8_0_noalloc")

    # ---- row-sharded products with the output all-gather fused into the kernel (one process per GPU) ----
    IPC_HANDLE_BYTES = 64

    def gather_region_bytes(self, world: int, slot_floats: int) -> int:
        return int(self.lib.zen_cuda_gather_region_bytes(world, slot_floats))

    def ipc_alloc(self, nbytes: int) -> tuple[int, bytes]:
        """Zero-filled device memory other processes can map: (device pointer, 64-byte handle to send them)."""
        handle = (C.c_ubyte * self.IPC_HANDLE_BYTES)()
        p = self.lib.zen_cuda_ipc_alloc(nbytes, handle)
        if not p:
            self._fail("ipc_alloc")
        return int(p), bytes(handle)

    def ipc_open(self, handle: bytes) -> int:
        buf = (C.c_ubyte * self.IPC_HANDLE_BYTES).from_buffer_copy(handle)
        p = self.lib.zen_cuda_ipc_open(buf)
        if not p:
            self._fail("ipc_open")
        return int(p)

    def ipc_close(self, peer_region: int) -> None:
        self.lib.zen_cuda_ipc_close(peer_region)

    def ipc_free(self, own_region: int) -> None:
        self.lib.zen_cuda_ipc_free(own_region)

    def gather_create(self, world: int, rank: int, slot_floats: int, regions: Sequence[int]) -> int:
        arr = (C.c_void_p * world)(*regions)
        g = self.lib.zen_cuda_gather_create(world, rank, slot_floats, arr)
        if not g:
            self._fail("gather_create")
        return int(g)

    def gather_destroy(self, gather: int) -> None:
        self.lib.zen_cuda_gather_destroy(gather)

    def dev_gemv_gather(self, gather: int, handles: Sequence[int], d_y: Sequence[int] | None, d_x: int | None, tokens: int,
                        act_mode: int, stream: int = 0) -> None:
        """The shard product with every output also stored into each rank's gather region by the kernel itself.
        d_x None: the input is what the previous launch on this gather object gathered."""
        n = len(handles)
        hs = (C.c_void_p * n)(*handles)
        ys = (C.c_void_p * n)(*d_y) if d_y is not None else None
        if not self.lib.zen_cuda_dev_gemv_gather(gather, hs, ys, n, d_x, tokens, act_mode, stream):
            self._fail("dev_gemv_gather")

    def dev_gather_fetch(self, gather: int, d_out: int | None, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_gather_fetch(gather, d_out, stream):
            self._fail("dev_gather_fetch")

    def dev_allgather(self, gather: int, d_piece: int, count: int, d_whole: int, stream: int = 0) -> None:
        """Every rank's d_piece (count floats) into every rank's d_whole, by peer stores and a bounded device wait."""
        if not self.lib.zen_cuda_dev_allgather(gather, d_piece, count, d_whole, stream):
            self._fail("dev_allgather")

    def dev_allreduce_add(self, gather: int, d_partial: int, count: int, d_inout: int, stream: int = 0) -> None:
        """d_inout += the ranks' d_partial vectors, added in rank order on every rank."""
        if not self.lib.zen_cuda_dev_allreduce_add(gather, d_partial, count, d_inout, stream):
            self._fail("dev_allreduce_add")

    def dev_quantize_acts(self, d_x: int, d_codes: int, d_scales: int, tokens: int, columns: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_quantize_acts(d_x, d_codes, d_scales, tokens, columns, stream):
            self._fail("dev_quantize_acts")

    def dev_greedy_pick(self, segments: Sequence[tuple[int, int, int, int]], tokens: int, d_pick: int, stream: int = 0) -> None:
        """Greedy token pick (first maximum among finite logits, -1 if none) into device int64 [tokens].  A segment is
        (device address of token 0's first entry, entries per token, index of the first entry, floats between tokens)."""
        n = len(segments)
        segs = (PickSegment * n)(*[PickSegment(b, ln, first, stride, 0) for b, ln, first, stride in segments])
        if not self.lib.zen_cuda_dev_greedy_pick(segs, n, tokens, d_pick, stream):
            self._fail("dev_greedy_pick")

    SAMPLE_MAX_CANDIDATES = 1024

    def dev_sample(self, d_logits: int, n: int, temperature: float, top_k: int, top_p: float, u: float, d_pick: int, stream: int = 0, *,
                   d_kept_ids: int | None = None, d_kept_probs: int | None = None, d_kept_count: int | None = None, d_truncated: int | None = None) -> None:
        """Temperature / top-k / top-p sampling of one token on the device (the non-greedy branch of the reference's sampler);
        u is a uniform number in [0, 1) from the caller's generator."""
        if not self.lib.zen_cuda_dev_sample(d_logits, n, temperature, top_k, top_p, u, d_pick, d_kept_ids, d_kept_probs, d_kept_count, d_truncated, stream):
            self._fail("dev_sample")

    # ---- decode-step operators between the projections ----
    def dev_embed_q8_0(self, handle: int, d_token: int, d_out: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_embed_q8_0(handle, d_token, d_out, stream):
            self._fail("dev_embed_q8_0")

    def dev_rms_norm(self, d_x: int, d_delta: int | None, d_weight: int | None, d_y: int | None, n: int, rows: int, eps: float, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_rms_norm(d_x, d_delta, d_weight, d_y, n, rows, eps, stream):
            self._fail("dev_rms_norm")

    def dev_rope_kv_append(self, d_q: int, d_k: int, d_v: int, d_cos: int, d_sin: int, d_pos: int, heads: int, kv_heads: int, head_dim: int,
                           pairs: int, adjacent: bool, d_k_cache: int, d_v_cache: int, max_positions: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_rope_kv_append(d_q, d_k, d_v, d_cos, d_sin, d_pos, heads, kv_heads, head_dim, pairs, int(adjacent), d_k_cache,
                                                    d_v_cache, max_positions, stream):
            self._fail("dev_rope_kv_append")

    def dev_attention(self, d_q: int, d_k_cache: int, d_v_cache: int, d_pos: int, d_out: int, heads: int, kv_heads: int, head_dim: int,
                      max_positions: int, scale: float = 0.0, window: int = 0, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_attention(d_q, d_k_cache, d_v_cache, d_pos, d_out, heads, kv_heads, head_dim, scale, window, max_positions, stream):
            self._fail("dev_attention")

    def dev_attention_block(self, d_q: int, d_k: int, d_v: int, d_cos: int, d_sin: int, pairs: int, d_pos: int, d_k_cache: int, d_v_cache: int,
                            d_out: int, heads: int, kv_heads: int, head_dim: int, max_positions: int, scale: float = 0.0, window: int = 0,
                            stream: int = 0) -> None:
        """Adjacent-pair RoPE + KV append + attention of one new token in one launch."""
        if not self.lib.zen_cuda_dev_attention_block(d_q, d_k, d_v, d_cos, d_sin, pairs, d_pos, d_k_cache, d_v_cache, d_out, heads, kv_heads, head_dim,
                                                     scale, window, max_positions, stream):
            self._fail("dev_attention_block")

    # ---- the block (prefill) forms ----
    def dev_embed_rows_q8_0(self, handle: int, d_tokens: int, tokens: int, d_out: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_embed_rows_q8_0(handle, d_tokens, tokens, d_out, stream):
            self._fail("dev_embed_rows_q8_0")

    def dev_rope_kv_append_rows(self, d_q: int, d_k: int, d_v: int, tokens: int, d_cos: int, d_sin: int, d_pos: int, heads: int, kv_heads: int,
                                head_dim: int, pairs: int, adjacent: bool, d_k_cache: int, d_v_cache: int, max_positions: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_rope_kv_append_rows(d_q, d_k, d_v, tokens, d_cos, d_sin, d_pos, heads, kv_heads, head_dim, pairs, int(adjacent),
                                                         d_k_cache, d_v_cache, max_positions, stream):
            self._fail("dev_rope_kv_append_rows")

    def dev_attention_prefill(self, d_q: int, d_k_cache: int, d_v_cache: int, d_pos: int, d_out: int, tokens: int, heads: int, kv_heads: int,
                              head_dim: int, max_positions: int, scale: float = 0.0, window: int = 0, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_attention_prefill(d_q, d_k_cache, d_v_cache, d_pos, d_out, tokens, heads, kv_heads, head_dim, scale, window,
                                                       max_positions, stream):
            self._fail("dev_attention_prefill")

    def dev_silu_mul(self, d_gate: int, d_up: int, d_out: int, count: int, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_silu_mul(d_gate, d_up, d_out, count, stream):
            self._fail("dev_silu_mul")

    def dev_advance_position(self, d_pos: int, delta: int = 1, stream: int = 0) -> None:
        if not self.lib.zen_cuda_dev_advance_position(d_pos, delta, stream):
            self._fail("dev_advance_position")

    def dev_check(self, stream: int = 0) -> None:
        """Synchronises `stream` and raises if a kernel reported through the device-side error word (a bounded wait that
        gave up, a bad token or position, a non-finite value) or the CUDA runtime reported a failure; .code holds
        zen_cuda_dev_check's value."""
        code = self.lib.zen_cuda_dev_check(stream)
        if code:
            what = (self.lib.zen_cuda_error_name(code) or b"").decode()
            err = BackendError(f"device-side error {code}: {what}" + (f" [{self.last_error()}]" if code < 0 else ""))
            err.code = code
            raise err

    def set_wait_budget_ms(self, milliseconds: int) -> None:
        """How long a bounded device-side wait may last before its kernel gives up (0: the default, about a second)."""
        if not self.lib.zen_cuda_set_wait_budget_ms(int(milliseconds)):
            self._fail("set_wait_budget_ms")

"""GGUF file -> resident device tensors, straight from the file mapping.

The reference maps the whole model file and hands the backend raw pointers into the mapping
(DenseTransformerRuntime::load, src/adapters/dense_transformer_runtime.cpp:934, :993-1004, over the tensor directory of
gguf::inspect, src/gguf.cpp:281-292: each tensor's bytes start at tensor_data_offset + offset, 32-byte aligned).  This
module does the same for the formats on the path: it parses the header, metadata and tensor directory of a GGUF v2/v3
file, maps the file read-only, and yields every tensor as a zero-copy view of the mapping, so that
Backend.dev_upload streams the bytes from the page cache through the pinned bounce buffers to the GPU without an
intermediate copy of the model in host memory.

Only what the decode path needs is understood: scalar and string metadata, arrays (skipped or kept as lists), and the
tensor types F32, Q4_0, Q8_0 and Q6_K, plus Q4_K and Q5_K by size (their bytes can be read; the device library does not
take them yet).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

from . import blocks

GGML_F32, GGML_Q4_0, GGML_Q8_0, GGML_Q6_K = 0, 2, 8, 14
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9
_MAX_DIMS, _MAX_STRING = 4, 1 << 24


class GgufError(ValueError):
    pass


@dataclass(frozen=True)
class GgufTensor:
    name: str
    shape: tuple[int, ...]      # outermost first (rows, columns for a matrix); GGUF stores the innermost first
    ggml_type: int
    offset: int                 # from the start of the file
    nbytes: int


class GgufFile:
    """A parsed, memory-mapped GGUF file.  `metadata` maps keys to Python values; `tensors` maps names to GgufTensor."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        try:
            self._parse()
        except (struct.error, IndexError) as e:
            self.close()
            raise GgufError(f"{path}: truncated or malformed GGUF ({e})") from None
        except GgufError:
            self.close()
            raise

    # ---- parsing ----
    def _take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self._pos + size > len(self._map):
            raise GgufError("unexpected end of file")
        v = struct.unpack_from(fmt, self._map, self._pos)[0]
        self._pos += size
        return v

    def _string(self) -> str:
        n = self._take("<Q")
        if n > _MAX_STRING or self._pos + n > len(self._map):
            raise GgufError("string length out of range")
        s = self._map[self._pos:self._pos + n].decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _value(self, kind: int):
        if kind in _SCALAR:
            return self._take(_SCALAR[kind])
        if kind == _STRING:
            return self._string()
        if kind == _ARRAY:
            sub, count = self._take("<I"), self._take("<Q")
            if sub == _ARRAY or count > (1 << 28):
                raise GgufError("unsupported array")
            return [self._value(sub) for _ in range(count)]
        raise GgufError(f"unknown metadata type {kind}")

    def _parse(self) -> None:
        if self._map[:4] != b"GGUF":
            raise GgufError("not a GGUF file")
        self._pos = 4
        version = self._take("<I")
        if version not in (2, 3):
            raise GgufError(f"GGUF version {version} is not supported")
        n_tensors, n_kv = self._take("<Q"), self._take("<Q")
        if n_tensors > (1 << 20) or n_kv > (1 << 20):
            raise GgufError("implausible tensor or metadata count")
        self.metadata: dict[str, object] = {}
        for _ in range(n_kv):
            key = self._string()
            self.metadata[key] = self._value(self._take("<I"))
        raw = []
        for _ in range(n_tensors):
            name = self._string()
            ndim = self._take("<I")
            if not 1 <= ndim <= _MAX_DIMS:
                raise GgufError(f"{name}: {ndim} dimensions")
            dims = [self._take("<Q") for _ in range(ndim)]
            raw.append((name, dims, self._take("<I"), self._take("<Q")))
        align = int(self.metadata.get("general.alignment", 32))
        if align <= 0 or align & (align - 1):
            raise GgufError("alignment is not a power of two")
        data_start = (self._pos + align - 1) & ~(align - 1)
        self.tensors: dict[str, GgufTensor] = {}
        for name, dims, ggml_type, offset in raw:
            shape = tuple(reversed(dims))
            cols = dims[0]
            count = int(np.prod(dims, dtype=np.uint64))
            if ggml_type == GGML_F32:
                nbytes = 4 * count
            elif ggml_type in blocks.BLOCK_BYTES:
                rb = blocks.row_bytes(ggml_type, cols)
                if rb == 0:
                    raise GgufError(f"{name}: {cols} columns are not a multiple of the block size")
                nbytes = rb * (count // cols)
            else:
                nbytes = -1   # a type this path does not decode: listed, but not readable
            if offset % align or (nbytes >= 0 and data_start + offset + nbytes > len(self._map)):
                raise GgufError(f"{name}: data lies outside the file or is misaligned")
            self.tensors[name] = GgufTensor(name, shape, ggml_type, data_start + offset, nbytes)

    # ---- access ----
    def array(self, name: str) -> np.ndarray:
        """A zero-copy view of the tensor in the mapping: fp32 in its own shape, quantised tensors as uint8 [rows, row_bytes]."""
        t = self.tensors[name]
        if t.nbytes < 0:
            raise GgufError(f"{name}: tensor type {t.ggml_type} is not on this path")
        buf = np.frombuffer(self._map, dtype=np.uint8, count=t.nbytes, offset=t.offset)
        if t.ggml_type == GGML_F32:
            return buf.view(np.float32).reshape(t.shape)
        rows = int(np.prod(t.shape[:-1], dtype=np.uint64)) if len(t.shape) > 1 else 1
        return buf.reshape(rows, -1)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:
            pass      # tensor views are still alive: the mapping goes away with the last of them
        finally:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def llama_config(g: GgufFile):
    """The LlamaConfig a `general.architecture = llama` file describes (the keys the reference reads,
    src/adapters/dense_transformer_runtime.cpp:700-770)."""
    from .llama import LlamaConfig
    md = g.metadata
    arch = md.get("general.architecture")
    if arch != "llama":
        raise GgufError(f"architecture {arch!r} is not served by this decoder")
    heads = int(md["llama.attention.head_count"])
    emb = int(md["llama.embedding_length"])
    head_dim = int(md.get("llama.attention.key_length", emb // heads))
    vocab = int(md.get("llama.vocab_size", 0)) or g.tensors["token_embd.weight"].shape[0]
    return LlamaConfig(embedding=emb, layers=int(md["llama.block_count"]), heads=heads,
                       kv_heads=int(md.get("llama.attention.head_count_kv", heads)), head_dim=head_dim,
                       ffn=int(md["llama.feed_forward_length"]), vocab=vocab, rope_base=float(md.get("llama.rope.freq_base", 10000.0)),
                       rms_eps=float(md.get("llama.attention.layer_norm_rms_epsilon", 1e-5)), context=int(md.get("llama.context_length", 2048)))


def llama_tensors(g: GgufFile, cfg):
    """(name, array view, is_matrix) for every tensor of the decoder's plan, matrices as raw Q8_0 blocks in the mapping."""
    from .llama import tensor_plan
    for name, shape, is_matrix in tensor_plan(cfg):
        if name == "output.weight" and name not in g.tensors:
            name_in_file = "token_embd.weight"   # tied lm_head
        else:
            name_in_file = name
        if name_in_file not in g.tensors:
            raise GgufError(f"missing tensor {name}")
        t = g.tensors[name_in_file]
        if tuple(t.shape) != tuple(shape):
            raise GgufError(f"{name}: shape {t.shape}, expected {shape}")
        if is_matrix and t.ggml_type != GGML_Q8_0:
            raise GgufError(f"{name}: the decoder takes Q8_0 matrices, the file has type {t.ggml_type}")
        if not is_matrix and t.ggml_type != GGML_F32:
            raise GgufError(f"{name}: norm weights must be F32")
        yield name, g.array(name_in_file), is_matrix

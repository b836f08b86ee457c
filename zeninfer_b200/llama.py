"""A dense Llama-style decoder whose every token step runs on the device through the C-ABI.

Host-side mirror of the reference's ModelRuntime::generate for a `general.architecture = llama` model
(src/adapters/dense_transformer_runtime.cpp:4660-4820 over forward() :3670-4600): embedding fetch, per layer
RMSNorm -> q|k|v -> adjacent-pair RoPE + KV append -> grouped-query attention -> o -> residual -> RMSNorm ->
gate|up -> SwiGLU -> down -> residual, final RMSNorm, lm_head, greedy pick.  All projections and the lm_head go
through the quantised product kernels (zen_cuda_dev_gemv); the operators between them are the decode-step entry
points of include/zen_cuda.h.  Nothing here computes on the host: Python only orders launches and builds the RoPE
cos/sin tables (the reference's table contract, rope_table :264-276).

A step is captured once into two CUDA graphs (layers; lm_head + pick), because the position and the token are read
from device memory.  The prompt goes through prefill() in blocks (tensor-core products) or token by token.

Several GPUs (one process per GPU, `rank` of `world`): every matrix but the embedding table is cut by output rows, a
rank uploads only its rows, and the vector a row-cut product leaves in pieces is put together by an all-gather before
the next operator needs it whole: the attention output (heads are cut with the q|k|v rows, so attention and the KV
cache are rank-local), the o projection's residual stream, the SwiGLU activation, the down projection's residual
stream, and the logits.  Four gathers per layer and one for the lm_head, each one launch of the peer-store all-gather
kernel (zen_cuda_dev_allgather; default) or an NCCL collective on the decoder's stream; either way they are captured
into the step graphs.  With cut="rows+cols" the o and down projections are cut by columns instead (a rank multiplies
its own heads' attention output, or its own slice of the SwiGLU activation, by the matching columns): their partial
products are summed into the residual stream by one all-reduce each (zen_cuda_dev_allreduce_add, rank order, identical
on every rank), which leaves two exchanges per layer instead of four; the sums then differ from the unsharded
decoder's by fp32 rounding (the order of the block sums changes), not by more.  Rows are independent, so every rank holds the same residual stream bit for
bit and picks the same token.  The reference drives one device; the row cut is its worker cut (ComputePool::parallel_for,
src/compute_pool.cpp:104-106).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import blocks
from .backend import ACT_FP32, ACT_INT8, Backend


@dataclass(frozen=True)
class LlamaConfig:
    embedding: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_base: float = 500000.0
    rms_eps: float = 1e-5
    context: int = 1024

    @property
    def q_width(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.kv_heads * self.head_dim


MATRIX_SHAPES = {  # GGUF tensor name suffix -> (rows, columns) as functions of the config
    "attn_q.weight": lambda c: (c.q_width, c.embedding), "attn_k.weight": lambda c: (c.kv_width, c.embedding),
    "attn_v.weight": lambda c: (c.kv_width, c.embedding), "attn_output.weight": lambda c: (c.embedding, c.q_width),
    "ffn_gate.weight": lambda c: (c.ffn, c.embedding), "ffn_up.weight": lambda c: (c.ffn, c.embedding),
    "ffn_down.weight": lambda c: (c.embedding, c.ffn),
}


def tensor_plan(cfg: LlamaConfig) -> list[tuple[str, tuple[int, ...], bool]]:
    """(name, shape, is_matrix) in file order; matrices are [rows, columns] and stored quantised."""
    plan = [("token_embd.weight", (cfg.vocab, cfg.embedding), True), ("output_norm.weight", (cfg.embedding,), False),
            ("output.weight", (cfg.vocab, cfg.embedding), True)]
    for layer in range(cfg.layers):
        p = f"blk.{layer}."
        plan.append((p + "attn_norm.weight", (cfg.embedding,), False))
        for suffix in ("attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight"):
            plan.append((p + suffix, MATRIX_SHAPES[suffix](cfg), True))
        plan.append((p + "ffn_norm.weight", (cfg.embedding,), False))
        for suffix in ("ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"):
            plan.append((p + suffix, MATRIX_SHAPES[suffix](cfg), True))
    return plan


def synthetic_tensors(cfg: LlamaConfig, seed: int, weight_std: float = 0.02):
    """Random-init model, one generator: matrices N(0, weight_std) packed to Q8_0 (raw GGUF blocks), norm weights
    1 + N(0, weight_std) in fp32.  Yields (name, array, is_matrix) in tensor_plan order, one tensor at a time."""
    rng = np.random.default_rng(seed)
    for name, shape, is_matrix in tensor_plan(cfg):
        if is_matrix:
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(weight_std)
            yield name, np.ascontiguousarray(blocks.quantize_q8_0(w)), True
        else:
            yield name, (np.float32(1.0) + rng.standard_normal(shape, dtype=np.float32) * np.float32(weight_std)).astype(np.float32), False


def rope_tables(cfg: LlamaConfig, positions: int) -> tuple[np.ndarray, np.ndarray]:
    """cos/sin [positions][head_dim / 2] in fp32, the arithmetic of rope_table (no scaling):
    freq_i = base^(-2 i / rotary_dim), angle = float(pos) * freq_i, all in single precision."""
    half = cfg.head_dim // 2
    i = np.arange(half, dtype=np.float32)
    freq = np.power(np.float32(cfg.rope_base), (np.float32(-2.0) * i / np.float32(cfg.head_dim)).astype(np.float32)).astype(np.float32)
    angle = (np.arange(positions, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    return np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)


class LlamaDecoder:
    """Holds the resident model and the step's device buffers.  `tensors` yields (name, array, is_matrix) as
    synthetic_tensors does; matrices must be Q8_0 raw blocks [rows, row_bytes]."""

    def __init__(self, backend: Backend, cfg: LlamaConfig, tensors, act_mode: int = ACT_INT8, max_positions: int | None = None, device=None,
                 fused: bool | str = "nrp", rank: int = 0, world: int = 1, group=None, gather: str = "peer", cut: str = "rows+cols",
                 prompt_act_mode: int | None = None):
        """fused: which of the layer's small operators are folded into the projection launches, as a string of letters:
        'n' RMSNorm into the q|k|v, gate|up and lm_head prologues, 's' SwiGLU into the down projection's prologue,
        'r' the residual adds into the o and down projections' stores, 'p' SwiGLU into the gate|up launch's store (the two
        halves of a CTA compute row r of gate and of up together and store silu(g) * u; not together with 's').  True =
        "nsr", False = none (8 launches per layer); the default folds what pays: the norm costs a CTA one extra pass over a
        16 KB row, 's' would cost every CTA 14336 exponentials, 'p' costs a barrier per row group.  Same arithmetic either way.
        rank, world, group: this process's share of a row-sharded model and the torch.distributed group of the ranks; world
        must divide the KV heads, the embedding, the ffn width and the vocabulary, and fused must be "nr" or "nrp".
        gather: "peer" = the library's own all-gather kernel over NVLink peer memory (the group only carries the IPC
        handles and host barriers, any backend), "nccl" = all_gather_into_tensor (the group must be NCCL).
        cut: "rows" = every matrix by output rows (four gathers per layer); "rows+cols" (default) = o and down by columns,
        summed by an all-reduce (two exchanges per layer; with gather="nccl" the row cut is used).
        prompt_act_mode: activation mode of the layer products while the prompt is consumed, when it differs from act_mode.
        The reference with ZEN_CPU_Q8_ACT=1 is such a mix: its prompt block goes through the fp32-activation GEMM
        (src/quant.cpp:1667-1680) and only single-token products quantise their input to int8 (:1088-1123); ACT_FP32 here
        with act_mode=ACT_INT8 reproduces it (prompt blocks go through the two-digit tensor-core product, leftover prompt
        tokens one by one outside the step graphs)."""
        import torch
        self.torch, self.be, self.cfg, self.act_mode = torch, backend, cfg, act_mode
        self.prompt_act_mode = prompt_act_mode if prompt_act_mode not in (None, act_mode) else None
        self.fuse = "nsr" if fused is True else "" if fused is False else str(fused)
        if "p" in self.fuse and "s" in self.fuse:
            raise ValueError("SwiGLU is folded into the gate|up store ('p') or into the down prologue ('s'), not both")
        self.rank, self.world, self.group = int(rank), int(world), group
        if not 0 <= self.rank < self.world:
            raise ValueError(f"rank {rank} of {world}")
        if self.world > 1:
            for what, n in (("kv_heads", cfg.kv_heads), ("embedding", cfg.embedding), ("ffn", cfg.ffn), ("vocab", cfg.vocab)):
                if n % self.world:
                    raise ValueError(f"{what} = {n} does not split over {self.world} ranks")
            if set(self.fuse) - {"p"} != set("nr"):
                raise ValueError('a row-sharded decoder runs with fused="nr" or "nrp"')
            import torch.distributed  # noqa: F401  (the collectives of _gather, handle exchange, host barriers)
            if gather not in ("peer", "nccl"):
                raise ValueError(f"gather = {gather!r}")
            if gather == "nccl" and cut == "rows+cols":
                cut = "rows"                               # the all-reduce in rank order is the peer kernel's
            if cut not in ("rows", "rows+cols"):
                raise ValueError(f"cut = {cut!r}")
        self.col_cut = self.world > 1 and cut == "rows+cols"
        self.gather_kind, self.peer = gather if self.world > 1 else "none", None
        self.dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.max_positions = max_positions or cfg.context
        self.stream = torch.cuda.Stream(device=self.dev)
        self.h: dict[str, int] = {}        # matrix name -> resident handle
        self.norm: dict[str, "torch.Tensor"] = {}
        shapes = {name: shape for name, shape, _ in tensor_plan(cfg)}
        for name, arr, is_matrix in tensors:
            if is_matrix:
                rows, cols = shapes[name]
                if self.col_cut and name.endswith(("attn_output.weight", "ffn_down.weight")):
                    # this rank's columns: whole 34-byte blocks of every row, copied out of the source
                    from . import shard
                    part, kept = shard.column_shard(arr, blocks.Q8_0, rows, cols, self.world, self.rank)
                    self.h[name] = backend.dev_upload("Q8_0", part, rows, kept)
                elif self.world > 1 and name != "token_embd.weight":   # this rank's rows only; every rank fetches embeddings itself
                    per = rows // self.world
                    self.h[name] = backend.dev_upload("Q8_0", arr, rows, cols, self.rank * per, per)
                else:
                    self.h[name] = backend.dev_upload("Q8_0", arr, rows, cols)
            else:
                self.norm[name] = torch.from_numpy(np.array(arr, np.float32)).to(self.dev)   # a copy: the source may be a read-only file mapping
        missing = [n for n, _, m in tensor_plan(cfg) if (m and n not in self.h) or (not m and n not in self.norm)]
        if missing:
            raise ValueError(f"model is missing tensors: {missing[:4]}...")
        f32 = dict(dtype=torch.float32, device=self.dev)
        E, QW, KW, F, V, w = cfg.embedding, cfg.q_width, cfg.kv_width, cfg.ffn, cfg.vocab, self.world
        # whole vectors (x, att, hid, logits: every rank holds all of them) and rank-local ones (q, k, v, gate, up, the caches)
        self.x, self.xn, self.tmp = torch.zeros(E, **f32), torch.zeros(E, **f32), torch.zeros(E, **f32)
        self.q, self.k, self.v, self.att = torch.zeros(QW // w, **f32), torch.zeros(KW // w, **f32), torch.zeros(KW // w, **f32), torch.zeros(QW, **f32)
        self.gate, self.up, self.hid = torch.zeros(F // w, **f32), torch.zeros(F // w, **f32), torch.zeros(F, **f32)
        self.logits = torch.zeros(V, **f32)
        self.k_cache = torch.zeros((cfg.layers, self.max_positions, KW // w), **f32)
        self.v_cache = torch.zeros((cfg.layers, self.max_positions, KW // w), **f32)
        mine = lambda t: t[self.rank * (t.numel() // w):(self.rank + 1) * (t.numel() // w)]     # the piece this rank's rows produce
        self.x_mine, self.att_mine, self.hid_mine, self.logits_mine = mine(self.x), mine(self.att), mine(self.hid), mine(self.logits)
        if self.gather_kind == "peer":
            from . import shard
            slot = max(E, QW, F, V) // w
            self.peer = shard.PeerGather(backend, w, self.rank, (slot + 3) & ~3, group=group)     # collective: handles travel through the group
        cos, sin = rope_tables(cfg, self.max_positions)
        self.cos, self.sin = torch.from_numpy(cos).to(self.dev), torch.from_numpy(sin).to(self.dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.token = torch.zeros(1, dtype=torch.int64, device=self.dev)
        self.host_token = torch.zeros(1, dtype=torch.int64).pin_memory()   # generate() feeds every step from the host, as the reference does
        self.graph_layers = self.graph_head = None

    @classmethod
    def from_gguf(cls, backend: Backend, path: str, **kwargs) -> "LlamaDecoder":
        """Loads a `general.architecture = llama` GGUF file with Q8_0 matrices: the tensors are uploaded straight from
        the file mapping (no host copy of the model), as the reference's loader hands its backends pointers into the
        mapping (src/adapters/dense_transformer_runtime.cpp:993-1004)."""
        from . import gguf
        with gguf.GgufFile(path) as g:
            cfg = gguf.llama_config(g)
            return cls(backend, cfg, gguf.llama_tensors(g, cfg), **kwargs)   # uploads complete before the mapping closes

    # ---- one token step, as launches on self.stream ----
    def _gemv(self, handles, outs, x, *, norm=None, gate=None, acc=False, warm=None, pair=False) -> None:
        """One product launch on the decoder's stream; `warm` is the tensor the next product launch will read."""
        self.be.dev_gemv_fused(handles, outs, x, 1, self.act_mode, self.stream.cuda_stream, norm_weight=norm, norm_eps=self.cfg.rms_eps if norm else 0.0,
                               gate=gate, accumulate=acc, warm_next=warm, swiglu_pair=pair)

    def _gather(self, whole, piece) -> None:
        """Every rank's piece into every rank's whole vector, in place (piece is this rank's slice of whole), ordered on
        the decoder's stream: the caller is inside `with torch.cuda.stream(self.stream)`."""
        if self.peer is not None:
            self.peer.allgather(piece.data_ptr(), piece.numel(), whole.data_ptr(), self.stream.cuda_stream)
        elif self.world > 1:
            self.torch.distributed.all_gather_into_tensor(whole, piece, group=self.group)

    def sync_ranks(self) -> None:
        """Host barrier after draining the own stream: the peer all-gather waits about a second for the other ranks on
        the device, so the ranks begin a sequence of steps together."""
        if self.world > 1:
            self.stream.synchronize()
            self.torch.distributed.barrier(group=self.group)

    def _enqueue_layers(self) -> None:
        be, cfg, st = self.be, self.cfg, self.stream.cuda_stream
        P = lambda t: t.data_ptr()
        E, eps = cfg.embedding, cfg.rms_eps
        fn, fs, fr, fp = "n" in self.fuse, "s" in self.fuse, "r" in self.fuse, "p" in self.fuse
        # the residual stream is self.x; a projection's input is x itself (norm folded in) or its normalised copy self.xn
        be.dev_embed_q8_0(self.h["token_embd.weight"], P(self.token), P(self.x), st)
        if not fn:
            be.dev_rms_norm(P(self.x), None, P(self.norm["blk.0.attn_norm.weight"]), P(self.xn), E, 1, eps, st)
        for layer in range(cfg.layers):
            p = f"blk.{layer}."
            nxt_q = self.h[f"blk.{layer + 1}.attn_q.weight"] if layer + 1 < cfg.layers else self.h["output.weight"]
            qkv = [self.h[p + "attn_q.weight"], self.h[p + "attn_k.weight"], self.h[p + "attn_v.weight"]]
            self._gemv(qkv, [P(self.q), P(self.k), P(self.v)], P(self.x) if fn else P(self.xn),
                       norm=P(self.norm[p + "attn_norm.weight"]) if fn else None, warm=self.h[p + "attn_output.weight"])
            be.dev_attention_block(P(self.q), P(self.k), P(self.v), P(self.cos), P(self.sin), cfg.head_dim // 2, P(self.pos), P(self.k_cache[layer]),
                                   P(self.v_cache[layer]), P(self.att_mine), cfg.heads // self.world, cfg.kv_heads // self.world, cfg.head_dim,
                                   self.max_positions, 0.0, 0, st)
            # attention output projection and its residual add (x += o(att))
            if self.col_cut:      # this rank's heads times their columns of o: a partial product of every output, summed over the ranks into x
                self._gemv([self.h[p + "attn_output.weight"]], [P(self.tmp)], P(self.att_mine), warm=self.h[p + "ffn_gate.weight"])
                self.peer.allreduce_add(P(self.tmp), E, P(self.x), st)
            else:
                self._gather(self.att, self.att_mine)
                self._gemv([self.h[p + "attn_output.weight"]], [P(self.x_mine) if fr else P(self.tmp)], P(self.att), acc=fr, warm=self.h[p + "ffn_gate.weight"])
                self._gather(self.x, self.x_mine)
            # ffn norm (with the residual add when it was not folded into the store)
            if not fn:
                be.dev_rms_norm(P(self.x), None if fr else P(self.tmp), P(self.norm[p + "ffn_norm.weight"]), P(self.xn), E, 1, eps, st)
            elif not fr:
                be.dev_rms_norm(P(self.x), P(self.tmp), None, None, E, 1, eps, st)                                 # x += tmp only
            self._gemv([self.h[p + "ffn_gate.weight"], self.h[p + "ffn_up.weight"]], [P(self.hid_mine), None] if fp else [P(self.gate), P(self.up)],
                       P(self.x) if fn else P(self.xn), norm=P(self.norm[p + "ffn_norm.weight"]) if fn else None, warm=self.h[p + "ffn_down.weight"], pair=fp)
            if not fs and not fp:
                be.dev_silu_mul(P(self.gate), P(self.up), P(self.hid_mine), cfg.ffn // self.world, st)
            if self.col_cut:
                self._gemv([self.h[p + "ffn_down.weight"]], [P(self.tmp)], P(self.hid_mine), warm=nxt_q)
                self.peer.allreduce_add(P(self.tmp), E, P(self.x), st)
            else:
                if not fs:
                    self._gather(self.hid, self.hid_mine)
                self._gemv([self.h[p + "ffn_down.weight"]], [P(self.x_mine) if fr else P(self.tmp)], P(self.up) if fs else P(self.hid),
                           gate=P(self.gate) if fs else None, acc=fr, warm=nxt_q)                                  # (x +=) down(silu(gate) * up)
                self._gather(self.x, self.x_mine)
            # the next norm: the next layer's attention norm, or the output norm
            nxt = self.norm[f"blk.{layer + 1}.attn_norm.weight"] if layer + 1 < cfg.layers else self.norm["output_norm.weight"]
            if not fn:
                be.dev_rms_norm(P(self.x), None if fr else P(self.tmp), P(nxt), P(self.xn), E, 1, eps, st)
            elif not fr:
                be.dev_rms_norm(P(self.x), P(self.tmp), None, None, E, 1, eps, st)
        be.dev_advance_position(P(self.pos), 1, st)

    def _enqueue_head(self) -> None:
        fn = "n" in self.fuse
        self._gemv([self.h["output.weight"]], [self.logits_mine.data_ptr()], self.x.data_ptr() if fn else self.xn.data_ptr(),
                   norm=self.norm["output_norm.weight"].data_ptr() if fn else None, warm=self.h["blk.0.attn_q.weight"])
        self._gather(self.logits, self.logits_mine)
        self.be.dev_greedy_pick([(self.logits.data_ptr(), self.cfg.vocab, 0, self.cfg.vocab)], 1, self.token.data_ptr(), self.stream.cuda_stream)

    def capture(self) -> None:
        """Runs one throw-away step (kernel attributes are set on first launch), then captures the two graphs."""
        torch = self.torch
        self.sync_ranks()
        with torch.cuda.stream(self.stream):
            self.reset()
            self._enqueue_layers()
            self._enqueue_head()
            self.stream.synchronize()
            self.graph_layers, self.graph_head = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            # with collectives in the graph, other threads of the process (the collective library's watchdog) may call
            # the runtime during the capture: only this thread's calls belong to it
            mode = dict(capture_error_mode="thread_local") if self.world > 1 else {}
            with torch.cuda.graph(self.graph_layers, stream=self.stream, **mode):
                self._enqueue_layers()
            with torch.cuda.graph(self.graph_head, stream=self.stream, **mode):
                self._enqueue_head()
            self.stream.synchronize()
        self.reset()

    def reset(self) -> None:
        with self.torch.cuda.stream(self.stream):
            self.pos.zero_()
            self.token.zero_()
        self.stream.synchronize()

    def step(self, want_token: bool) -> None:
        """Consumes the token in self.token at position self.pos; with want_token the pick replaces self.token."""
        with self.torch.cuda.stream(self.stream):
            if self.graph_layers is not None:
                self.graph_layers.replay()
                if want_token:
                    self.graph_head.replay()
            else:
                self._enqueue_layers()
                if want_token:
                    self._enqueue_head()

    # ---- prefill: a block of prompt tokens through the tensor-core products ----
    PREFILL_CHUNK = 512     # tokens per block (buffers are sized for it)
    PREFILL_MIN = 16        # shorter blocks go token by token

    def _prefill_buffers(self):
        if getattr(self, "_pf", None) is None:
            torch, cfg, T, w = self.torch, self.cfg, self.PREFILL_CHUNK, self.world
            f32 = dict(dtype=torch.float32, device=self.dev)
            mode = self._prefill_mode()
            ws_bytes = max(self.be.gemm_workspace_bytes(T, n, mode) for n in (cfg.embedding, cfg.ffn // w, cfg.q_width // w))
            # x, xn, tmp are whole on every rank; q, k, v, att, gate, up, hid hold this rank's heads / ffn rows
            self._pf = dict(x=torch.zeros((T, cfg.embedding), **f32), xn=torch.zeros((T, cfg.embedding), **f32), tmp=torch.zeros((T, cfg.embedding), **f32),
                            q=torch.zeros((T, cfg.q_width // w), **f32), k=torch.zeros((T, cfg.kv_width // w), **f32), v=torch.zeros((T, cfg.kv_width // w), **f32),
                            att=torch.zeros((T, cfg.q_width // w), **f32), gate=torch.zeros((T, cfg.ffn // w), **f32), up=torch.zeros((T, cfg.ffn // w), **f32),
                            hid=torch.zeros((T, cfg.ffn // w), **f32), ws=torch.zeros(ws_bytes, dtype=torch.uint8, device=self.dev), ws_bytes=ws_bytes)
        return self._pf

    def _prefill_mode(self) -> int:
        """Activation mode of the prompt block's products: prompt_act_mode when one was given, else the decode mode."""
        return self.prompt_act_mode if self.prompt_act_mode is not None else self.act_mode

    def can_prefill_blocks(self) -> bool:
        """One GPU, or a sharded decoder whose o and down projections are cut by columns and whose group is NCCL: the
        block's two exchanges per layer are then all-reduces of [tokens, embedding] partial products."""
        if self.world == 1:
            return True
        return self.col_cut and self.torch.distributed.get_backend(self.group) == "nccl"

    def prefill(self, d_tokens, count: int) -> None:
        """Consumes `count` tokens (device int64) at positions pos .. pos + count - 1 as one block: the projections run
        as tcgen05 GEMMs (int8 activations, or two int8 digits per activation in the fp32-equivalent mode), the attention
        as the causal block kernel; afterwards the residual stream and its normalised copy of the LAST token are in
        self.x / self.xn, ready for the lm_head, and pos has advanced.
        Sharded (can_prefill_blocks): q|k|v, gate and up are this rank's rows (its heads, its slice of the ffn), attention
        and the KV cache are rank-local, o and down multiply this rank's columns and the ranks' partial products of the
        whole block are summed by one NCCL all-reduce each (two per layer, [tokens, embedding] fp32), after which every
        rank adds the same sum to its copy of the residual stream."""
        if not self.can_prefill_blocks():
            raise ValueError("the block prefill needs one GPU, or the column cut with an NCCL group; this decoder takes its prompt token by token")
        be, cfg, st, w = self.be, self.cfg, self.stream.cuda_stream, self.world
        b = self._prefill_buffers()
        P = lambda t: t.data_ptr()
        T, E, eps = count, cfg.embedding, cfg.rms_eps
        mode = self._prefill_mode()
        gemm = lambda hs, outs, x: be.dev_gemm_q8_0(hs, [P(o) for o in outs], P(x), T, P(b["ws"]), b["ws_bytes"], st, act_mode=mode)

        def reduce_partials():
            if w > 1:   # tmp[:T] holds this rank's partial product of every output
                self.torch.distributed.all_reduce(b["tmp"][:T], group=self.group)

        be.dev_embed_rows_q8_0(self.h["token_embd.weight"], P(d_tokens), T, P(b["x"]), st)
        be.dev_rms_norm(P(b["x"]), None, P(self.norm["blk.0.attn_norm.weight"]), P(b["xn"]), E, T, eps, st)
        for layer in range(cfg.layers):
            p = f"blk.{layer}."
            gemm([self.h[p + "attn_q.weight"], self.h[p + "attn_k.weight"], self.h[p + "attn_v.weight"]], [b["q"], b["k"], b["v"]], b["xn"])
            be.dev_rope_kv_append_rows(P(b["q"]), P(b["k"]), P(b["v"]), T, P(self.cos), P(self.sin), P(self.pos), cfg.heads // w, cfg.kv_heads // w, cfg.head_dim,
                                       cfg.head_dim // 2, True, P(self.k_cache[layer]), P(self.v_cache[layer]), self.max_positions, st)
            be.dev_attention_prefill(P(b["q"]), P(self.k_cache[layer]), P(self.v_cache[layer]), P(self.pos), P(b["att"]), T, cfg.heads // w, cfg.kv_heads // w,
                                     cfg.head_dim, self.max_positions, 0.0, 0, st)
            gemm([self.h[p + "attn_output.weight"]], [b["tmp"]], b["att"])
            reduce_partials()
            be.dev_rms_norm(P(b["x"]), P(b["tmp"]), P(self.norm[p + "ffn_norm.weight"]), P(b["xn"]), E, T, eps, st)          # x += o; xn = norm(x)
            gemm([self.h[p + "ffn_gate.weight"], self.h[p + "ffn_up.weight"]], [b["gate"], b["up"]], b["xn"])
            be.dev_silu_mul(P(b["gate"]), P(b["up"]), P(b["hid"]), T * (cfg.ffn // w), st)
            gemm([self.h[p + "ffn_down.weight"]], [b["tmp"]], b["hid"])
            reduce_partials()
            nxt = self.norm[f"blk.{layer + 1}.attn_norm.weight"] if layer + 1 < cfg.layers else self.norm["output_norm.weight"]
            be.dev_rms_norm(P(b["x"]), P(b["tmp"]), P(nxt), P(b["xn"]), E, T, eps, st)                                       # x += down; xn = next norm
        be.dev_advance_position(P(self.pos), T, st)
        with self.torch.cuda.stream(self.stream):
            self.x.copy_(b["x"][T - 1])
            self.xn.copy_(b["xn"][T - 1])

    def forward_block(self, tokens: list[int], start_pos: int | None = None, tail_count: int = 1):
        """DenseTransformerRuntime::forward_batch (src/adapters/dense_transformer_runtime.cpp:2298): consumes `tokens` as one
        block at positions start_pos .. (default: the current position) and returns the logits of the last `tail_count` of
        them, [tail_count][vocab] fp32 on the device, with the greedy pick of every row in self.block_picks[:tail_count].
        Speculative verification is this call with tail_count = len(proposals) (:4874): row i is the target model's
        distribution after proposal i.  Afterwards the position is start_pos + len(tokens); a caller that rejects proposals
        passes the position after the last accepted token as the next start_pos (the cache rows past it are overwritten,
        as in the reference, whose caches are indexed by the position it is given).
        The layers run through prefill() (tcgen05 GEMMs, causal block attention); the lm_head takes the tail rows through
        the decode kernel (up to eight, in the decode activation mode) or the GEMM (more, in the block's mode).  One GPU only."""
        if self.world != 1:
            raise ValueError("forward_block: the sharded decoder keeps only its shard of the logits; use one GPU")
        T = len(tokens)
        if not 1 <= tail_count <= T or T > self.PREFILL_CHUNK:
            raise ValueError("forward_block: 1 <= tail_count <= len(tokens) <= PREFILL_CHUNK")
        torch, be, cfg, st = self.torch, self.be, self.cfg, self.stream.cuda_stream
        if start_pos is None:
            self.stream.synchronize()
            start_pos = int(self.pos.item())
        if start_pos + T > self.max_positions:
            raise ValueError("forward_block: the block does not fit the configured positions")
        with torch.cuda.stream(self.stream):
            self.pos.fill_(start_pos)
            d_ids = torch.tensor(tokens, dtype=torch.int64).pin_memory().to(self.dev, non_blocking=True)
            self.prefill(d_ids, T)
            b = self._prefill_buffers()
            if getattr(self, "block_logits", None) is None or self.block_logits.shape[0] < tail_count:
                self.block_logits = torch.zeros((max(tail_count, 8), cfg.vocab), dtype=torch.float32, device=self.dev)
                self.block_picks = torch.zeros((max(tail_count, 8),), dtype=torch.int64, device=self.dev)
            xn_tail = b["xn"][T - tail_count:T]       # normalised with the output norm by the block's last step
            head, out = self.h["output.weight"], self.block_logits
            if tail_count <= 8:
                be.dev_gemv([head], [out.data_ptr()], xn_tail.data_ptr(), tail_count, self.act_mode, st)
            else:
                be.dev_gemm_q8_0([head], [out.data_ptr()], xn_tail.data_ptr(), tail_count, b["ws"].data_ptr(), b["ws_bytes"], st, act_mode=self._prefill_mode())
            be.dev_greedy_pick([(out.data_ptr(), cfg.vocab, 0, cfg.vocab)], tail_count, self.block_picks.data_ptr(), st)
            self.logits.copy_(out[tail_count - 1])     # what a following single step or last_logits() sees
            self.token.copy_(self.block_picks[tail_count - 1:tail_count])
        return self.block_logits[:tail_count]

    def feed_prompt(self, prompt: list[int], batched_prefill: bool | None = None) -> None:
        """Enqueues the whole prompt from position self.pos on, ending with the first pick (left in self.token).  Blocks of
        at least PREFILL_MIN tokens go through prefill() when batched_prefill (default: wherever can_prefill_blocks()), the
        rest token by token."""
        torch = self.torch
        ids = torch.tensor(prompt, dtype=torch.int64).pin_memory()
        if batched_prefill is None:
            batched_prefill = self.can_prefill_blocks()
        with torch.cuda.stream(self.stream):
            done = 0
            if batched_prefill and len(prompt) >= self.PREFILL_MIN:
                d_ids = ids.to(self.dev, non_blocking=True)
                while len(prompt) - done >= self.PREFILL_MIN:
                    n = min(self.PREFILL_CHUNK, len(prompt) - done)
                    self.prefill(d_ids[done:done + n], n)
                    done += n
                if done == len(prompt):
                    self._enqueue_head()      # the first pick, from the last prompt token's hidden state
            for i in range(done, len(prompt)):
                self.token.copy_(ids[i:i + 1], non_blocking=True)
                last = i + 1 == len(prompt)
                if self.prompt_act_mode is None:
                    self.step(want_token=last)
                    continue
                decode_mode, self.act_mode = self.act_mode, self.prompt_act_mode
                try:
                    self._enqueue_layers()            # eager: the captured graphs hold the decode mode
                finally:
                    self.act_mode = decode_mode
                if last:
                    self._enqueue_head()              # a single-token product: the decode mode

    def _sample(self, temperature: float, top_k: int, top_p: float, u: float) -> None:
        """Replaces the greedy pick in self.token by a draw from the filtered distribution of self.logits."""
        self.be.dev_sample(self.logits.data_ptr(), self.cfg.vocab, temperature, top_k, top_p, u, self.token.data_ptr(), self.stream.cuda_stream)

    def generate(self, prompt: list[int], max_new: int, on_token=None, batched_prefill: bool | None = None, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> list[int]:
        """Generation: the prompt, then max_new picks (each read back, as the reference's per-token callback does).  With
        temperature <= 0 the picks are greedy; otherwise every token is drawn on the device from the temperature / top-k /
        top-p distribution of the step's logits (GenerationOptions, sample_logits :391-418), with one uniform number per
        token from a host generator seeded with `seed` (the generator stays on the host, as the reference's does).  The
        prompt goes through prefill() in blocks (in the prompt's activation mode) on one GPU and on a column-cut sharded
        decoder with an NCCL group, token by token otherwise; batched_prefill overrides the choice.
        Raises when the context would overflow."""
        torch = self.torch
        if not prompt or len(prompt) + max_new > self.max_positions:
            raise ValueError("prompt + max_new exceeds the configured positions")
        self.reset()
        self.sync_ranks()
        out: list[int] = []
        rng = np.random.default_rng(seed) if temperature > 0.0 else None
        with torch.cuda.stream(self.stream):
            self.feed_prompt(prompt, batched_prefill)
            for n in range(max_new):
                if rng is not None:               # the step left the greedy pick in self.token: draw instead
                    self._sample(temperature, top_k, top_p, float(rng.random()))
                tok = int(self.token.item())      # device -> host read of the step's result
                out.append(tok)
                if on_token:
                    on_token(tok)
                if n + 1 < max_new:
                    self.host_token[0] = tok      # host -> device: the next step's input comes from the caller's side
                    self.token.copy_(self.host_token, non_blocking=True)
                    self.step(want_token=True)
        self.be.dev_check(self.stream.cuda_stream)
        return out

    def last_logits(self) -> np.ndarray:
        self.stream.synchronize()
        return self.logits.cpu().numpy()

    def close(self) -> None:
        self.stream.synchronize()
        self.graph_layers = self.graph_head = None     # captured collectives hold on to the communicator: release them before the group goes
        if self.peer is not None:
            self.peer.close()                          # collective: every rank closes its decoder
            self.peer = None
        for h in self.h.values():
            self.be.dev_free(h)
        self.h.clear()


__all__ = ["LlamaConfig", "LlamaDecoder", "synthetic_tensors", "tensor_plan", "rope_tables", "ACT_FP32", "ACT_INT8"]

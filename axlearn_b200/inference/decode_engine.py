"""Decode engine for Fuji-style decoders: paged KV cache, tensor parallelism, CUDA-graph steps.

What the reference does for generation is a jitted ``while_loop`` over ``Decoder.extend_step``
(axlearn/common/decoder.py:286-448, axlearn/common/decoding.py:978-1150) with a functional KV
cache that is rebuilt every step.  On a B200 the step is a fixed, short list of kernels on
persistent buffers, so the engine:

* keeps per-layer K/V page pools ``[num_pages, page_size, Nkv_local, H]`` resident and appends in
  place (``rope_append_paged`` writes the rotated key / value of the new token straight into
  its page slot while producing the rotated query);
* runs attention over the pages with the split-KV decode kernel (``paged_decode_attention``);
* packs the projections so that a layer is four GEMMs on the tcgen05 kernel (QKV, output,
  gate|up, down); the residual adds are the GEMMs' accumulate epilogues on one GPU;
* under tensor parallelism (heads and FFN columns split over the ``model`` group) fuses the two
  all-reduces per layer with the GEMMs that feed them: the row-parallel GEMM's epilogue stores
  its rows straight into every peer's staging slot and raises the flags
  (``OneShotAllReduce.gemm_push``), and one finish kernel per all-reduce sums the slots and adds
  the residual;
* captures one decode step (all layers, head, greedy pick, length bump) in a CUDA graph and
  replays it per token.

Prefill runs the same weights over whole prompts with the flash-attention forward kernel and
writes K/V into the pages.  Sequences own a contiguous run of pages (sequence ``b`` owns pages
``[b * max_pages, (b + 1) * max_pages)``), which keeps the page table trivial without making
the kernels depend on it.
"""

from __future__ import annotations

import dataclasses
import math
import os
from typing import Any, Optional

import torch

from axlearn_b200.ops import attention_ops, cuda_ops, decode_ops

Tensor = torch.Tensor


@dataclasses.dataclass
class FujiDims:
    num_layers: int
    hidden_dim: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn_dim: int
    vocab_size: int
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5


@dataclasses.dataclass
class LayerWeights:
    attn_norm: Tensor   # [D]
    wqkv: Tensor        # [D, (Nq_l + 2 Nkv_l) * H]
    wo: Tensor          # [Nq_l * H, D]
    ffn_norm: Tensor    # [D]
    wgu: Tensor         # [D, 2 F_l]  (gate | up)
    wdown: Tensor       # [F_l, D]


def _get(tree: dict, path: str):
    node = tree
    for part in path.split("/"):
        node = node[part]
    return node


def weights_from_fuji_state(model_state: dict, dims: FujiDims, *, rank: int = 0, world: int = 1,
                            dtype=torch.bfloat16, device=None) -> dict:
    """Slices a (full, unsharded) Fuji parameter tree for tensor-parallel rank ``rank``.

    Heads and FFN columns are split contiguously over ranks; embeddings, norms and the output
    head are replicated.  Layout of the tree: see ``experiments/text/gpt/fuji.py``.
    """
    d, n, nkv, h, f = dims.hidden_dim, dims.num_heads, dims.num_kv_heads, dims.head_dim, dims.ffn_dim
    assert n % world == 0 and nkv % world == 0 and f % world == 0, (n, nkv, f, world)
    nl, nkvl, fl = n // world, nkv // world, f // world
    layer = _get(model_state, "decoder/transformer/repeat/layer")
    qkv = _get(layer, "self_attention/attention/i_proj/i_proj/qkv_proj/weight")
    wo_all = _get(layer, "self_attention/attention/o_proj/weight")            # [L, D, N, H]
    w_gate = _get(layer, "feed_forward/linear1_0/weight")                     # [L, D, F]
    w_up = _get(layer, "feed_forward/linear1_1/weight")
    w_down = _get(layer, "feed_forward/linear2/weight")                       # [L, F, D]
    attn_norm = _get(layer, "self_attention/norm/scale")
    ffn_norm = _get(layer, "feed_forward/norm/scale")

    def put(t):
        return t.to(device=device, dtype=dtype).contiguous()

    layers = []
    for i in range(dims.num_layers):
        if qkv.dim() == 5:   # [L, 3, D, N, H]: separate q / k / v stacks (MHA)
            q = qkv[i, 0][:, rank * nl:(rank + 1) * nl]
            k = qkv[i, 1][:, rank * nkvl:(rank + 1) * nkvl]
            v = qkv[i, 2][:, rank * nkvl:(rank + 1) * nkvl]
        else:                # [L, D, N + 2 Nkv, H]: grouped-query layout
            q = qkv[i][:, rank * nl:(rank + 1) * nl]
            k = qkv[i][:, n + rank * nkvl:n + (rank + 1) * nkvl]
            v = qkv[i][:, n + nkv + rank * nkvl:n + nkv + (rank + 1) * nkvl]
        wqkv = torch.cat([q.reshape(d, -1), k.reshape(d, -1), v.reshape(d, -1)], dim=1)
        wo = wo_all[i][:, rank * nl:(rank + 1) * nl].reshape(d, nl * h).t()
        wgu = torch.cat([w_gate[i][:, rank * fl:(rank + 1) * fl], w_up[i][:, rank * fl:(rank + 1) * fl]], dim=1)
        layers.append(LayerWeights(
            attn_norm=put(attn_norm[i]), wqkv=put(wqkv), wo=put(wo), ffn_norm=put(ffn_norm[i]),
            wgu=put(wgu), wdown=put(w_down[i][rank * fl:(rank + 1) * fl])))
    dec = model_state["decoder"]
    emb = put(_get(dec, "emb/token_emb/weight"))
    head = put(_get(dec, "lm_head/weight")) if "lm_head" in dec else emb
    return {"layers": layers, "emb": emb, "head": head, "final_norm": put(_get(dec, "output_norm/scale"))}


class DecodeEngine:
    """Greedy generation for ``batch`` sequences of up to ``max_len`` tokens on one GPU of a
    tensor-parallel group (``group=None``: single GPU)."""

    def __init__(self, weights: dict, dims: FujiDims, *, batch: int, max_len: int, page_size: int = 16,
                 group=None, device=None, use_graph: bool = True, prefill_chunk_tokens: int = 16384):
        self.w, self.dims = weights, dims
        self.batch, self.page_size = batch, page_size
        self.device = device if device is not None else weights["emb"].device
        self.group = group
        if group is not None:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        d = dims
        assert d.head_dim == 128, "the decode kernels are specialised for head_dim 128"
        self.nq_l, self.nkv_l = d.num_heads // self.world, d.num_kv_heads // self.world
        self.max_pages = (max_len + page_size - 1) // page_size
        self.max_len = self.max_pages * page_size
        pool = (batch * self.max_pages, page_size, self.nkv_l, d.head_dim)
        self.k_pools = [torch.zeros(pool, dtype=torch.bfloat16, device=self.device) for _ in range(d.num_layers)]
        self.v_pools = [torch.zeros(pool, dtype=torch.bfloat16, device=self.device) for _ in range(d.num_layers)]
        self.page_table = torch.arange(batch * self.max_pages, dtype=torch.int32, device=self.device).reshape(
            batch, self.max_pages)
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=self.device)
        # Logits of the latest position (a fixed buffer: the captured step writes into it, and a
        # sampler outside the graph reads it).
        self.logits = torch.zeros(batch, dims.vocab_size, dtype=torch.float32, device=self.device)
        self.splits = decode_ops.default_splits(batch, self.nkv_l, self.nq_l // self.nkv_l, self.max_len, page_size)
        self._scratch = torch.empty(
            max(1, decode_ops._lib().axb_decode_attn_scratch_floats(batch, self.nq_l, self.splits)),  # pylint: disable=protected-access
            dtype=torch.float32, device=self.device)
        self._softmax_scale = 1.0 / math.sqrt(d.head_dim)
        self._allreduce: Optional[decode_ops.OneShotAllReduce] = None
        if self.world > 1:
            self._allreduce = decode_ops.OneShotAllReduce(
                batch * d.hidden_dim, 2 * d.num_layers, group=group, device=self.device)
        self._use_graph = use_graph
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._prefill_chunk_tokens = prefill_chunk_tokens
        self.launches_per_step = 0

    # ------------------------------------------------------------------ shared pieces
    def _gemm_reduce(self, a: Tensor, w: Tensor, residual: Tensor, site: int) -> Tensor:
        """``residual + sum over ranks of (a @ w)``; the finish kernel sums the peers' slots.

        With two ranks the GEMM's epilogue stores its rows into the peer's staging slot and raises
        the flags itself (one launch less per all-reduce; measured 5.63 vs 5.89 ms per token on two
        GPUs).  With more ranks the epilogue's row-per-lane 16-byte stores to seven peers are a
        poor fit for NVLink (8 GPUs, batch 64: 7.55 ms per token against 6.72 ms with the separate
        push kernel, whose stores are coalesced), so the push stays a kernel of its own there;
        ``AXB_DECODE_FUSED_PUSH=0/1`` overrides the choice."""
        fused = os.environ.get("AXB_DECODE_FUSED_PUSH")
        use_fused = (self._allreduce.world <= 2) if fused is None else fused == "1"
        if use_fused and w.shape[1] % 32 == 0:
            self._allreduce.gemm_push(a, w, site)
        else:
            self._allreduce.push(cuda_ops.gemm(a, w).reshape(-1), site)
        return self._allreduce.finish(site, residual=residual.reshape(-1)).reshape(residual.shape)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, prompt_ids: Tensor, lengths: Optional[Tensor] = None) -> Tensor:
        """Runs the prompts ``[batch, T]``, fills the caches and returns the greedy first token of
        every sequence ``[batch]`` (its logits stay in ``self.logits``).  ``lengths [batch]``:
        right-padded prompts of different lengths (the padding's cache entries are overwritten
        as decoding proceeds); None = all of length T."""
        d = self.dims
        b, t = prompt_ids.shape
        assert b == self.batch and t <= self.max_len
        h = d.head_dim
        per_chunk = max(1, self._prefill_chunk_tokens // t)
        positions = torch.arange(t, device=self.device)
        last_hidden = torch.empty((b, d.hidden_dim), dtype=torch.bfloat16, device=self.device)
        for b0 in range(0, b, per_chunk):
            b1 = min(b, b0 + per_chunk)
            x = self.w["emb"][prompt_ids[b0:b1]]                              # [bs, T, D]
            for li, lw in enumerate(self.w["layers"]):
                hn = cuda_ops.rms_norm(x, lw.attn_norm, d.norm_eps)
                qkv = cuda_ops.linear(hn, lw.wqkv).reshape(b1 - b0, t, self.nq_l + 2 * self.nkv_l, h)
                q = cuda_ops.rope(qkv[:, :, :self.nq_l], positions, d.rope_theta)
                k = cuda_ops.rope(qkv[:, :, self.nq_l:self.nq_l + self.nkv_l], positions, d.rope_theta)
                v = qkv[:, :, self.nq_l + self.nkv_l:].contiguous()
                kp = self.k_pools[li].view(b, self.max_len, self.nkv_l, h)
                vp = self.v_pools[li].view(b, self.max_len, self.nkv_l, h)
                kp[b0:b1, :t] = k
                vp[b0:b1, :t] = v
                attn = attention_ops.flash_attention(q, k, v, causal=True, softmax_scale=self._softmax_scale)
                o = cuda_ops.linear(attn.reshape(b1 - b0, t, self.nq_l * h), lw.wo)
                if self.world > 1:
                    import torch.distributed as dist

                    dist.all_reduce(o, group=self.group)
                x = x + o
                hn = cuda_ops.rms_norm(x, lw.ffn_norm, d.norm_eps)
                gu = cuda_ops.linear(hn, lw.wgu)
                act = decode_ops.swiglu_packed(gu.reshape(-1, gu.shape[-1]))
                dn = cuda_ops.linear(act, lw.wdown).reshape(x.shape)
                if self.world > 1:
                    dist.all_reduce(dn, group=self.group)
                x = x + dn
            if lengths is None:
                last_hidden[b0:b1] = x[:, -1]
            else:
                idx = (lengths[b0:b1].long() - 1).clamp(min=0)
                last_hidden[b0:b1] = x[torch.arange(b1 - b0, device=self.device), idx]
        if lengths is None:
            self.lengths.fill_(t)
        else:
            self.lengths.copy_(lengths.to(self.lengths.dtype))
        self.logits.copy_(self._logits(last_hidden))
        self.tokens.copy_(self.logits.argmax(dim=-1))
        if self.device.type == "cuda":
            cuda_ops.check_status(self.device)
        return self.tokens.clone()

    def _logits(self, hidden: Tensor) -> Tensor:
        hn = cuda_ops.rms_norm(hidden, self.w["final_norm"], self.dims.norm_eps)
        return cuda_ops.gemm(hn, self.w["head"].t(), out_dtype=torch.float32)

    # ------------------------------------------------------------------ decode
    def _step(self) -> None:
        """One token for every sequence: consumes ``self.tokens`` (the latest token), appends
        its K/V, and leaves the next token in ``self.tokens``."""
        d = self.dims
        before = cuda_ops.launch_count
        self.lengths.add_(1).clamp_(max=self.max_len)   # rows that ran out of room rewrite their last slot
        if self._allreduce is not None:
            self._allreduce.begin_step()
        x = self.w["emb"][self.tokens]                                        # [B, D]
        for li, lw in enumerate(self.w["layers"]):
            hn = cuda_ops.rms_norm(x, lw.attn_norm, d.norm_eps)
            qkv = cuda_ops.gemm(hn, lw.wqkv)
            q = decode_ops.rope_append_paged(
                qkv, self.k_pools[li], self.v_pools[li], self.page_table, self.lengths,
                num_q_heads=self.nq_l, theta=d.rope_theta)
            attn = decode_ops.paged_decode_attention(
                q, self.k_pools[li], self.v_pools[li], self.page_table, self.lengths,
                softmax_scale=self._softmax_scale, splits=self.splits, scratch=self._scratch)
            attn2 = attn.reshape(self.batch, self.nq_l * d.head_dim)
            if self.world > 1:
                x = self._gemm_reduce(attn2, lw.wo, x, 2 * li)
            else:
                cuda_ops.gemm(attn2, lw.wo, out=x, accumulate=True)           # x += attn @ Wo
            hn = cuda_ops.rms_norm(x, lw.ffn_norm, d.norm_eps)
            act = decode_ops.swiglu_packed(cuda_ops.gemm(hn, lw.wgu))
            if self.world > 1:
                x = self._gemm_reduce(act, lw.wdown, x, 2 * li + 1)
            else:
                cuda_ops.gemm(act, lw.wdown, out=x, accumulate=True)
        self.logits.copy_(self._logits(x))
        self.tokens.copy_(self.logits.argmax(dim=-1))
        self.launches_per_step = cuda_ops.launch_count - before

    @torch.no_grad()
    def decode(self, steps: int) -> Tensor:
        """Generates ``steps`` further tokens per sequence (after ``prefill``); returns them
        ``[batch, steps]``.  The first call captures the step in a CUDA graph."""
        out = torch.empty((self.batch, steps), dtype=torch.int64, device=self.device)
        self._ensure_graph()
        for i in range(steps):
            if self._graph is not None:
                self._graph.replay()
            else:
                self._step()
            out[:, i] = self.tokens
        cuda_ops.check_status(self.device)
        return out

    def _ensure_graph(self) -> None:
        if self._use_graph and self._graph is None:
            # Warm up on a side stream (lazy module loading, tensor-map encoding), restoring
            # the state the warm-up steps consumed, then capture.
            saved = (self.lengths.clone(), self.tokens.clone())
            epoch = None if self._allreduce is None else self._allreduce.epoch.clone()
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                self._step()
            torch.cuda.current_stream(self.device).wait_stream(s)
            self.lengths.copy_(saved[0])
            self.tokens.copy_(saved[1])
            del epoch  # The epoch keeps counting: peers warmed up the same number of steps.
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._step()
            self.lengths.copy_(saved[0])
            self.tokens.copy_(saved[1])

    @torch.no_grad()
    def step_logits(self, tokens: Tensor) -> Tensor:
        """Feeds one token per sequence (``[batch]``: the token at each sequence's current end),
        appends its K/V and returns the fp32 logits of the next position ``[batch, vocab]`` -- the
        engine as a ``tokens -> scores`` function for samplers and searches that live outside."""
        self._ensure_graph()
        self.tokens.copy_(tokens.reshape(-1))
        if self._graph is not None:
            self._graph.replay()
        else:
            self._step()
        return self.logits

    @torch.no_grad()
    def generate(self, prompt_ids: Tensor, max_new_tokens: int) -> Tensor:
        first = self.prefill(prompt_ids)
        rest = self.decode(max_new_tokens - 1) if max_new_tokens > 1 else first[:, :0]
        return torch.cat([first[:, None], rest], dim=1)


# ------------------------------------------------------------------------------------------
# The engine behind the framework's decoding API.
# ------------------------------------------------------------------------------------------

_ENGINES: dict = {}


def dims_from_decoder(decoder) -> Optional[FujiDims]:
    """``FujiDims`` of a ``Decoder`` whose stack is the Fuji / Llama shape this engine implements
    (repeated pre-norm layers, RMSNorm, RoPE on q / k, fused QKV, SwiGLU, no biases); None for
    anything else."""
    try:
        cfg = decoder.config
        stack = cfg.transformer
        layer = stack.layer
        attn = layer.self_attention.attention
        ff = layer.feed_forward
        qkv = attn.input_linear
        rope = qkv.rope_pos_emb_layer
        inner = qkv.input_linear
        if layer.self_attention.structure != "prenorm" or ff.structure != "prenorm":
            return None
        if tuple(ff.activation) != ("nn.silu", "linear") or getattr(layer, "cross_attention", None) is not None:
            return None
        if "RMSNorm" not in layer.self_attention.norm.klass.__name__ or cfg.output_norm is None:
            return None
        num_heads = attn.num_heads
        num_kv = getattr(inner, "num_kv_heads", None) or num_heads
        state = decoder.parameter_tree()
        w_gate = _get(state, "transformer/repeat/layer/feed_forward/linear1_0/weight")
        return FujiDims(num_layers=stack.num_layers, hidden_dim=cfg.dim, num_heads=num_heads, num_kv_heads=num_kv,
                        head_dim=cfg.dim // num_heads, ffn_dim=w_gate.shape[-1], vocab_size=cfg.vocab_size,
                        rope_theta=float(rope.theta), norm_eps=float(layer.self_attention.norm.eps))
    except (AttributeError, KeyError, TypeError):
        return None


def engine_for_decoder(decoder, *, batch: int, max_len: int) -> Optional["DecodeEngine"]:
    """A (cached) engine over the decoder's current parameters, or None when the decoder, its
    placement or its shapes are outside what the engine implements."""
    from axlearn_b200.parallel.mesh import current_mesh

    if os.environ.get("AXB200_DECODE_ENGINE", "1") == "0":
        return None
    mesh = current_mesh()
    if mesh is not None and mesh.size > 1:
        return None
    dims = dims_from_decoder(decoder)
    if dims is None or dims.head_dim != 128:
        return None
    state = decoder.parameter_tree()
    emb = _get(state, "emb/token_emb/weight")
    if not emb.is_cuda or emb.dtype != torch.bfloat16:
        return None
    key = (id(decoder), batch, max_len, emb.data_ptr())
    engine = _ENGINES.get(key)
    if engine is None:
        _ENGINES.clear()          # one resident engine: its caches and weight copies are large
        weights = weights_from_fuji_state({"decoder": state}, dims, device=emb.device)
        engine = DecodeEngine(weights, dims, batch=batch, max_len=max_len, device=emb.device)
        _ENGINES[key] = engine
    return engine

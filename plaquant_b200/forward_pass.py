"""Llama-architecture forward with the mixed NVFP4 / MXFP8 linears, in the shape of the reference's
`IndependentResQForward` (inference/forward_pass.py:118-319 in the reference): norm -> q,k,v ->
RoPE -> attention -> o_proj -> norm -> gate, up -> silu * up -> down_proj, LM head unquantised.

What runs where.  The hot path of this repository - RMSNorm + rotation + quantise-and-pack and the
quantised linears - runs on the CUDA library (fused: the two RMSNorms of a layer never produce a
bf16 tensor, they feed the pack kernel, which also absorbs the residual add in front of each norm and
SiLU(gate) * up in front of the down projection).  Everything else the reference leaves to PyTorch
stays in PyTorch: embedding, RoPE, scaled-dot-product attention (forward_pass.py:249 there), the final
norm and the LM head (forward_pass.py:178-181 there).

Tensor parallelism (Megatron): QKV and gate_up are column-parallel (N sharded by heads / by FFN
columns, no exchange), O and down are row-parallel (K sharded, one all-reduce each), see tp.py.  With
`fused_reduce_rows` > 0, decode batches of up to that many rows do not call NCCL for those all-reduces:
the row-parallel GEMV writes its partial output into a peer-visible buffer and the following
RMSNorm-quant kernel sums the ranks' buffers over NVLink itself (ops.allreduce_add_rmsnorm_pack).
Weights are random-initialised per layer from a seed (no checkpoints are available offline).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import kv_cache, ops, tp
from .quantize import QuantizedLinear
from .rotation import get_hadamard_matrix  # noqa: F401  (re-exported, as the reference module does)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """Stand-alone RMSNorm with the reference's arithmetic (forward_pass.py:33-39): float32, one cast.
    Only used off the hot path (final norm before the unquantised LM head)."""
    dtype = x.dtype
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.float() * xf).to(dtype)


def rms_norm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, k_hi: int, hadamard: bool = True,
                   sf_layout: str = "tiled") -> ops.PackedMatrix:
    """Fused RMSNorm -> block-Hadamard(128) -> NVFP4 | MXFP8 pack: what a quantised linear consumes."""
    return ops.pack(x, k_hi, hadamard=hadamard, sf_layout=sf_layout, gamma=weight, eps=eps)


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-6
    high_fraction: float = 1.0 / 32

    @classmethod
    def llama3_70b(cls):
        return cls(8192, 28672, 80, 64, 8, 128, 128256)

    @classmethod
    def llama3_8b(cls):
        return cls()


_IN_PEER_BUFFER = object()      # marker: a layer's MLP output is waiting, unreduced, in the peer buffer


class _Layer:
    __slots__ = ("ln1", "ln2", "qkv", "o", "gate_up", "down")


class ResQForwardB200:
    """Decoder stack with packed weights resident on one GPU (one tensor-parallel rank)."""

    def __init__(self, cfg: LlamaConfig, device, ctx: Optional[tp.TPContext] = None, seed: int = 0,
                 num_layers: Optional[int] = None, fused_reduce_rows: int = 0, kv_quant: bool = False):
        self.cfg, self.device, self.ctx = cfg, torch.device(device), ctx or tp.TPContext()
        c, r, s = cfg, self.ctx.rank, self.ctx.size
        assert c.num_heads % s == 0 and c.num_kv_heads % s == 0 and c.intermediate_size % (s * 128) == 0
        self.heads, self.kv_heads = c.num_heads // s, c.num_kv_heads // s
        self.ffn = c.intermediate_size // s
        self.k_hi_hidden = tp.outlier_count(c.hidden_size, c.high_fraction)
        self.k_hi_attn = tp.outlier_count(self.heads * c.head_dim, c.high_fraction)     # rank-local K of o_proj
        self.k_hi_ffn = tp.outlier_count(self.ffn, c.high_fraction)                     # rank-local K of down_proj
        self.layers: List[_Layer] = []
        n_layers = c.num_layers if num_layers is None else num_layers
        for li in range(n_layers):
            g = torch.Generator(device=self.device).manual_seed(seed * 100003 + li * 16 + r)
            L = _Layer()
            L.ln1 = (torch.rand(c.hidden_size, generator=g, device=self.device) + 0.5).to(torch.bfloat16)
            L.ln2 = (torch.rand(c.hidden_size, generator=g, device=self.device) + 0.5).to(torch.bfloat16)
            L.qkv = self._linear((self.heads + 2 * self.kv_heads) * c.head_dim, c.hidden_size, self.k_hi_hidden, g)
            L.o = self._linear(c.hidden_size, self.heads * c.head_dim, self.k_hi_attn, g)
            L.gate_up = self._linear(2 * self.ffn, c.hidden_size, self.k_hi_hidden, g)
            L.down = self._linear(c.hidden_size, self.ffn, self.k_hi_ffn, g)
            self.layers.append(L)
        g = torch.Generator(device=self.device).manual_seed(seed * 100003 + 999983)      # replicated on every rank
        self.embed = (torch.randn(c.vocab_size, c.hidden_size, generator=g, device=self.device) * 0.02).to(torch.bfloat16)
        self.final_norm = (torch.rand(c.hidden_size, generator=g, device=self.device) + 0.5).to(torch.bfloat16)
        self.lm_head = (torch.randn(c.vocab_size, c.hidden_size, generator=g, device=self.device) * 0.02).to(torch.bfloat16)
        self.kv: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.pos = 0
        # keys go into the cache as NVFP4 (Hadamard over the head dimension, per-head rows), queries get the same
        # rotation: the reference's QKRotationWrapper with k_had (promix/quantize/kv_quant.py:244-279)
        self.kv_quant = kv_quant
        if kv_quant and c.head_dim != 128:
            raise ValueError("kv_quant needs head_dim = 128 (one Hadamard block per head)")
        # decode batches of up to `fused_reduce_rows` rows reduce over peer memory inside the RMSNorm-quant kernel
        self.peer = (tp.PeerReduce(fused_reduce_rows, c.hidden_size, self.device, self.ctx.group)
                     if fused_reduce_rows > 0 and self.ctx.size > 1 else None)

    def _linear(self, n: int, k: int, k_hi: int, g: torch.Generator) -> QuantizedLinear:
        """Random N(0, 0.02) weight [n, k], rotated and packed on the device; only the packed form is kept."""
        w = (torch.randn(n, k, generator=g, device=self.device) * 0.02).to(torch.bfloat16)
        p = ops.pack(w, k_hi, hadamard=True, sf_layout="rowmajor")
        del w
        return QuantizedLinear(p.lo_codes, p.lo_sf, p.hi_codes, p.hi_sf, online_had=True)

    # ---- pieces ----------------------------------------------------------------------------------
    def _quantized_linear(self, x, lin: QuantizedLinear, norm_weight=None):
        """[RMSNorm] -> Hadamard -> quantise -> packed GEMM / GEMV (reference: forward_pass.py:278-319)."""
        return lin(x, norm_weight=norm_weight, eps=self.cfg.rms_eps)

    def _rope_angles(self, pos: torch.Tensor):
        """cos / sin tables [1, T, 1, head_dim] for float32 positions `pos` [T] (a device tensor, so that a decode
        step captured in a CUDA graph reads its position from memory)."""
        c = self.cfg
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=pos.device, dtype=torch.float32) / c.head_dim))
        ang = torch.outer(pos, inv)
        return (torch.cat([ang.cos(), ang.cos()], -1)[None, :, None, :],
                torch.cat([ang.sin(), ang.sin()], -1)[None, :, None, :])

    def _rope(self, q, k, cos_sin):
        c = self.cfg
        cos, sin = cos_sin

        def rot(v):
            v1, v2 = v[..., : c.head_dim // 2], v[..., c.head_dim // 2:]
            return (v.float() * cos + torch.cat([-v2, v1], -1).float() * sin).to(v.dtype)
        return rot(q), rot(k)

    def _forward_layer(self, li: int, h: torch.Tensor, delta: Optional[torch.Tensor], pos0: int, cos_sin,
                       static: Optional[dict] = None):
        """One decoder layer.  `h` is the residual stream and `delta` the previous layer's MLP output that has
        not been added to it yet (None for the first layer): the add is fused into this layer's first
        RMSNorm-quant kernel, and the layer returns its own (h, delta) in the same form.

        Without `static`, keys and values are kept in a growing Python-side cache (prefill, and decode steps of
        arbitrary length).  With `static` (a dict holding preallocated caches [B, T_max, ...], the device tensors
        `pos` [1] int64 and `mask` [1, 1, 1, T_max] bool) every shape is fixed and the position is data, which
        is what CUDA-graph capture of a decode step needs."""
        c, L = self.cfg, self.layers[li]
        b, t, _ = h.shape
        fused = self.peer is not None and b * t <= self.peer.rows      # all-reduce inside the RMSNorm-quant kernel
        if delta is None:
            qkv = self._quantized_linear(h, L.qkv, norm_weight=L.ln1)
        elif delta is _IN_PEER_BUFFER:   # h += sum over ranks of the previous down_proj; RMSNorm(ln1); quantise
            h, pa = ops.allreduce_add_rmsnorm_pack(self.peer, b * t, h, L.ln1, c.rms_eps, self.k_hi_hidden)
            qkv = L.qkv(pa).view(b, t, -1)
        else:   # h += delta; RMSNorm(ln1); rotate; quantise: one kernel
            h, pa = ops.add_rmsnorm_pack(delta, h, L.ln1, c.rms_eps, self.k_hi_hidden)
            qkv = L.qkv(pa).view(b, t, -1)
        q, k, v = qkv.split([self.heads * c.head_dim, self.kv_heads * c.head_dim, self.kv_heads * c.head_dim], -1)
        q, k, v = q.view(b, t, self.heads, c.head_dim), k.view(b, t, self.kv_heads, c.head_dim), v.view(b, t, self.kv_heads, c.head_dim)
        q, k = self._rope(q, k, cos_sin)
        if self.kv_quant:
            q = kv_cache.rotate_heads(q)
            k = kv_cache.dequantize_heads(kv_cache.quantize_heads(k.contiguous()), k.shape)   # what the packed cache holds
        if static is None:
            if pos0 == 0:
                self.kv[li] = (k, v)
            else:
                self.kv[li] = (torch.cat([self.kv[li][0], k], 1), torch.cat([self.kv[li][1], v], 1))
            kk, vv = self.kv[li]
            attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                  is_causal=(t > 1), enable_gqa=True)
        else:
            kk, vv = static["k"][li], static["v"][li]
            kk.index_copy_(1, static["pos"], k)
            vv.index_copy_(1, static["pos"], v)
            attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                  attn_mask=static["mask"], enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(b, t, self.heads * c.head_dim)
        if fused:
            L.o(attn.reshape(b * t, -1), out=self.peer.buffer(b * t))                   # partial sums stay in the peer buffer
            h, pa = ops.allreduce_add_rmsnorm_pack(self.peer, b * t, h, L.ln2, c.rms_eps, self.k_hi_hidden)
        else:
            o = self.ctx.all_reduce(self._quantized_linear(attn, L.o))
            h, pa = ops.add_rmsnorm_pack(o, h, L.ln2, c.rms_eps, self.k_hi_hidden)      # h += o; RMSNorm(ln2); quantise
        gu = L.gate_up(pa)                                                              # [b*t, 2*ffn] = [gate | up]
        pa = ops.silu_mul_pack(gu, self.k_hi_ffn)                                       # SiLU(gate)*up; rotate; quantise
        if fused:
            L.down(pa, out=self.peer.buffer(b * t))       # reduced by the next layer's first kernel (or _finish)
            return h, _IN_PEER_BUFFER
        return h, self.ctx.all_reduce(L.down(pa)).view(b, t, -1)

    def _finish(self, h: torch.Tensor, delta) -> torch.Tensor:
        """Residual stream after the last layer: h + delta.  When the last MLP output is still waiting in the peer
        buffers it is reduced by the same fused kernel as everywhere else (its packed output is not needed), which
        also makes the number of fused calls per pass even: 2 per layer."""
        if delta is _IN_PEER_BUFFER:
            b, t, _ = h.shape
            h, _ = ops.allreduce_add_rmsnorm_pack(self.peer, b * t, h, self.final_norm, self.cfg.rms_eps, self.k_hi_hidden)
            return h
        return h + delta

    # ---- public ----------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, pos0: int = 0) -> torch.Tensor:
        """input_ids [B, T] -> logits of the last position [B, vocab] (float32)."""
        if pos0 == 0:
            self.kv = [None] * len(self.layers)
        h = F.embedding(input_ids, self.embed)
        t = input_ids.shape[1]
        cos_sin = self._rope_angles(torch.arange(pos0, pos0 + t, device=h.device, dtype=torch.float32))   # once per pass
        delta = None
        for li in range(len(self.layers)):
            h, delta = self._forward_layer(li, h, delta, pos0, cos_sin)
        self.pos = pos0 + input_ids.shape[1]
        return self._logits(self._finish(h, delta)[:, -1])

    def _logits(self, h_last: torch.Tensor) -> torch.Tensor:
        """Final norm + unquantised LM head in the model dtype (inference/forward_pass.py:178-181 in the reference)."""
        last = rms_norm(h_last, self.final_norm, self.cfg.rms_eps)
        return F.linear(last, self.lm_head).float()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, steps: int, use_graph: bool = True) -> torch.Tensor:
        """Prefill + `steps` greedy decode steps; returns the generated ids [B, steps].

        With `use_graph` the decode step (fixed shapes: caches preallocated for prefill + steps positions, the
        position and the attention mask held in device memory) is captured once in a CUDA graph and replayed, so
        a step costs its kernels and not ~2000 Python-side launches."""
        if not use_graph or steps < 2:
            out = []
            nxt = self.forward(input_ids).argmax(-1, keepdim=True)
            for _ in range(steps):
                out.append(nxt)
                nxt = self.forward(nxt, pos0=self.pos).argmax(-1, keepdim=True)
            return torch.cat(out, 1)

        c, dev = self.cfg, self.device
        b, t0 = input_ids.shape
        t_max = t0 + steps
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        nxt = self.forward(input_ids).argmax(-1, keepdim=True)              # eager prefill fills self.kv
        ev[1].record()
        st = {"k": [], "v": [], "pos": torch.full((1,), t0, dtype=torch.int64, device=dev),
              "mask": torch.zeros(1, 1, 1, t_max, dtype=torch.bool, device=dev)}
        for li in range(len(self.layers)):
            for name, src in (("k", self.kv[li][0]), ("v", self.kv[li][1])):
                buf = torch.zeros(b, t_max, self.kv_heads, c.head_dim, dtype=src.dtype, device=dev)
                buf[:, :t0] = src
                st[name].append(buf)
        self.kv = [None] * len(self.layers)
        tok = nxt.clone()                                                    # [B, 1] current token, updated in place
        out = torch.zeros(b, steps, dtype=nxt.dtype, device=dev)
        step_idx = torch.zeros(1, dtype=torch.int64, device=dev)
        arange = torch.arange(t_max, device=dev)

        def decode_step():
            out.index_copy_(1, step_idx, tok)
            st["mask"].copy_((arange <= st["pos"]).view(1, 1, 1, t_max))
            h = F.embedding(tok, self.embed)
            cos_sin = self._rope_angles(st["pos"].to(torch.float32))
            delta = None
            for li in range(len(self.layers)):
                h, delta = self._forward_layer(li, h, delta, 0, cos_sin, static=st)
            tok.copy_(self._logits(self._finish(h, delta)[:, -1]).argmax(-1, keepdim=True))
            st["pos"].add_(1)
            step_idx.add_(1)

        decode_step()                                                        # warm-up (also step 0 of the output)
        if steps > 1:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                decode_step()                                                # step 1, eager on the capture stream
                side.synchronize()
                if steps > 2:
                    calls_before = self.peer.calls if self.peer is not None else 0
                    with torch.cuda.graph(graph, stream=side):
                        decode_step()
            torch.cuda.current_stream(dev).wait_stream(side)
            if self.peer is not None and steps > 2:
                # a replayed step keeps the buffer set of each call site: sets alternate across replays only if the
                # step holds an even number of fused reductions (two per layer)
                assert (self.peer.calls - calls_before) % 2 == 0, "odd number of fused reductions in the decode step"
                # ranks reach this point at different times (capture is ~2000 host launches): line them up so the
                # bounded cross-rank wait of the first replay measures the peers, not the host skew
                import torch.distributed as dist
                dist.barrier(self.ctx.group)
            for _ in range(steps - 2):                                       # capture does not execute: steps 2 .. steps-1
                graph.replay()
        ev[2].record()
        ops.check_device_status(dev)                                         # a missing rank or a protocol error is loud
        self.timing_events = ev      # prefill = ev[0] -> ev[1], decode (incl. capture) = ev[1] -> ev[2], once synchronised
        self.pos = t_max
        return out

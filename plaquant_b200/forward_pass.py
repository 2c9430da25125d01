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
import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

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


class _DecodeState:
    """What generate() keeps per (batch, prompt length, steps): static caches, position / mask / token buffers and
    the captured CUDA graph of one decode step."""
    __slots__ = ("st", "tok", "out", "step_idx", "arange", "graph", "first_set")


class _Layer:
    __slots__ = ("ln1", "ln2", "qkv", "o", "gate_up", "down")


class ResQForwardB200:
    """Decoder stack with packed weights resident on one GPU (one tensor-parallel rank)."""

    def __init__(self, cfg: LlamaConfig, device, ctx: Optional[tp.TPContext] = None, seed: int = 0,
                 num_layers: Optional[int] = None, fused_reduce_rows: int = 0, kv_quant: bool = False,
                 weights: Optional[Dict[str, torch.Tensor]] = None, packed: Optional[dict] = None,
                 scatter_prefill_rows: int = 0):
        """Weights come from one of three places: `packed` (the state a packed-weight container holds, see
        weight_packer.py), `weights` (a dict of full bf16 tensors under the reference's names, `l{i}.q_proj.weight`
        ... as `IndependentResQForward` takes them; every rank picks its own shard), or, with neither, a random
        initialisation per layer from `seed` (no checkpoints are available offline)."""
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
        if packed is not None:
            self._load_packed(packed, n_layers)
        else:
            for li in range(n_layers):
                t = self._shard_of(weights, li) if weights is not None else self._random_layer(li, seed)
                L = _Layer()
                L.ln1, L.ln2 = t["ln1"], t["ln2"]
                L.qkv = self._linear(t.pop("qkv"), self.k_hi_hidden)
                L.o = self._linear(t.pop("o"), self.k_hi_attn)
                L.gate_up = self._linear(t.pop("gate_up"), self.k_hi_hidden)
                L.down = self._linear(t.pop("down"), self.k_hi_ffn)
                self.layers.append(L)
            if weights is not None:
                to = dict(device=self.device, dtype=torch.bfloat16)
                self.embed, self.final_norm = weights["embed"].to(**to), weights["final_norm"].to(**to)
                self.lm_head = weights["lm_head"].to(**to)
            else:
                g = torch.Generator(device=self.device).manual_seed(seed * 100003 + 999983)      # replicated on every rank
                self.embed = (torch.randn(c.vocab_size, c.hidden_size, generator=g, device=self.device) * 0.02).to(torch.bfloat16)
                self.final_norm = (torch.rand(c.hidden_size, generator=g, device=self.device) + 0.5).to(torch.bfloat16)
                self.lm_head = (torch.randn(c.vocab_size, c.hidden_size, generator=g, device=self.device) * 0.02).to(torch.bfloat16)
        self.kv: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.pos = 0
        self._decode_states: Dict[tuple, _DecodeState] = {}
        # keys go into the cache as NVFP4 (Hadamard over the head dimension, per-head rows), queries get the same
        # rotation: the reference's QKRotationWrapper with k_had (promix/quantize/kv_quant.py:244-279)
        self.kv_quant = kv_quant                     # False | True (packed NVFP4 rows in the cache) | "fake" (their bf16 values)
        if kv_quant and c.head_dim != 128:
            raise ValueError("kv_quant needs head_dim = 128 (one Hadamard block per head)")
        # decode batches of up to `fused_reduce_rows` rows reduce over peer memory inside the RMSNorm-quant kernel
        self.peer = (tp.PeerReduce(fused_reduce_rows, c.hidden_size, self.device, self.ctx.group)
                     if fused_reduce_rows > 0 and self.ctx.size > 1 else None)
        # prefill batches of up to `scatter_prefill_rows` rows (B * T, a multiple of the number of ranks) keep the
        # residual stream sharded by rows between the linears: reduce-scatter + norm + quantise + all-gather of the
        # packed rows in one kernel over peer memory instead of an NCCL all-reduce of bf16
        self.scatter = (tp.ScatterReduce(scatter_prefill_rows, c.hidden_size, self.k_hi_hidden, self.device, self.ctx.group)
                        if scatter_prefill_rows > 0 and self.ctx.size > 1 else None)

    # ---- where the weights come from ---------------------------------------------------------------
    def _random_layer(self, li: int, seed: int) -> Dict[str, torch.Tensor]:
        """This rank's bf16 tensors of layer `li`: norm weights ~ U(0.5, 1.5) (replicated: the same on every rank,
        from a stream of their own), linears ~ N(0, 0.02) (this rank's shards)."""
        c, r = self.cfg, self.ctx.rank
        g = torch.Generator(device=self.device).manual_seed(seed * 100003 + li * 16 + r)
        gn = torch.Generator(device=self.device).manual_seed(seed * 100003 + li * 16 + 15)

        def lin(n, k):
            return (torch.randn(n, k, generator=g, device=self.device) * 0.02).to(torch.bfloat16)
        t = {"ln1": (torch.rand(c.hidden_size, generator=gn, device=self.device) + 0.5).to(torch.bfloat16),
             "ln2": (torch.rand(c.hidden_size, generator=gn, device=self.device) + 0.5).to(torch.bfloat16)}
        t["qkv"] = lin((self.heads + 2 * self.kv_heads) * c.head_dim, c.hidden_size)
        t["o"] = lin(c.hidden_size, self.heads * c.head_dim)
        t["gate_up"] = lin(2 * self.ffn, c.hidden_size)
        t["down"] = lin(c.hidden_size, self.ffn)
        return t

    def _shard_of(self, weights: Dict[str, torch.Tensor], li: int) -> Dict[str, torch.Tensor]:
        """This rank's tensors of layer `li` cut out of full weights under the reference's names
        (inference/forward_pass.py:185-276 there): column-parallel q/k/v (by heads) and gate/up (by FFN columns),
        fused into one [q | k | v] and one [gate | up] matrix; row-parallel o_proj (input columns of this rank's
        heads) and down_proj (input columns of this rank's FFN slice)."""
        c, r, s, p = self.cfg, self.ctx.rank, self.ctx.size, f"l{li}"
        to = dict(device=self.device, dtype=torch.bfloat16)
        hd = c.head_dim
        qs = tp.column_parallel_rows(c.num_heads * hd, r, s)
        ks = tp.column_parallel_rows(c.num_kv_heads * hd, r, s)
        fs = tp.column_parallel_rows(c.intermediate_size, r, s)
        oc = tp.row_parallel_cols(c.num_heads * hd, r, s)
        dc = tp.row_parallel_cols(c.intermediate_size, r, s)
        w = lambda name: weights[f"{p}.{name}.weight"]
        return {
            "ln1": weights[f"{p}.ln1"].to(**to), "ln2": weights[f"{p}.ln2"].to(**to),
            "qkv": torch.cat([w("q_proj")[qs], w("k_proj")[ks], w("v_proj")[ks]], 0).to(**to),
            "o": w("o_proj")[:, oc].to(**to).contiguous(),
            "gate_up": torch.cat([w("mlp.gate_proj")[fs], w("mlp.up_proj")[fs]], 0).to(**to),
            "down": w("mlp.down_proj")[:, dc].to(**to).contiguous(),
        }

    def _linear(self, w: torch.Tensor, k_hi: int) -> QuantizedLinear:
        """bf16 weight [n, k] -> rotated and packed on the device; only the packed form is kept."""
        p = ops.pack(w, k_hi, hadamard=True, sf_layout="rowmajor")
        return QuantizedLinear(p.lo_codes, p.lo_sf, p.hi_codes, p.hi_sf, online_had=True)

    def packed_state(self) -> dict:
        """Everything needed to rebuild this rank's model without the bf16 weights: per linear the packed codes
        and row-major scale bytes, the norm weights, embedding and LM head (see weight_packer.save_packed)."""
        c = self.cfg
        tensors, linears = {"embed": self.embed, "final_norm": self.final_norm, "lm_head": self.lm_head}, {}
        for li, L in enumerate(self.layers):
            tensors[f"l{li}.ln1"], tensors[f"l{li}.ln2"] = L.ln1, L.ln2
            for name in ("qkv", "o", "gate_up", "down"):
                q: QuantizedLinear = getattr(L, name)
                key = f"l{li}.{name}"
                tensors[key + ".lo_codes"], tensors[key + ".lo_sf"] = q.w_main_int, q.w_main_scale
                tensors[key + ".hi_codes"], tensors[key + ".hi_sf"] = q.w_high_int, q.w_high_scale
                linears[key] = {"n": q.out_features, "k_lo": q.w_main_int.shape[1] * 2, "k_hi": q.high_bits_length,
                                "rotated": True, "sf_layout": "rowmajor"}
        return {"config": dict(vars(c)), "num_layers": len(self.layers), "tp": {"rank": self.ctx.rank, "size": self.ctx.size},
                "tensors": tensors, "linears": linears}

    def _load_packed(self, state: dict, n_layers: int) -> None:
        if (state["tp"]["rank"], state["tp"]["size"]) != (self.ctx.rank, self.ctx.size):
            raise ValueError(f"packed weights were written for rank {state['tp']['rank']} of {state['tp']['size']}, "
                             f"this is rank {self.ctx.rank} of {self.ctx.size}: the K split of the row-parallel linears "
                             "(each rank's own MXFP8 columns) depends on the tensor-parallel degree")
        if n_layers > state["num_layers"]:
            raise ValueError(f"the container holds {state['num_layers']} layers, {n_layers} were asked for")
        def wanted(name: str) -> bool:               # "l{i}.*" of the layers kept, and the tensors outside the layers
            m = re.match(r"l(\d+)\.", name)
            return m is None or int(m.group(1)) < n_layers
        t = {k: v.to(self.device) for k, v in state["tensors"].items() if wanted(k)}
        for li in range(n_layers):
            L = _Layer()
            L.ln1, L.ln2 = t[f"l{li}.ln1"], t[f"l{li}.ln2"]
            for name in ("qkv", "o", "gate_up", "down"):
                key = f"l{li}.{name}"
                meta = state["linears"][key]
                if not meta["rotated"] or meta["sf_layout"] != "rowmajor":
                    raise ValueError(f"{key}: unsupported container entry {meta}")
                q = QuantizedLinear(t[key + ".lo_codes"], t[key + ".lo_sf"], t[key + ".hi_codes"], t[key + ".hi_sf"],
                                    online_had=True)
                if (q.out_features, q.in_features - q.high_bits_length, q.high_bits_length) != (meta["n"], meta["k_lo"], meta["k_hi"]):
                    raise ValueError(f"{key}: tensor shapes do not match the recorded {meta}")
                setattr(L, name, q)
            self.layers.append(L)
        self.embed, self.final_norm, self.lm_head = t["embed"], t["final_norm"], t["lm_head"]

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

    def _attention(self, li: int, qkv: torch.Tensor, pos0: int, cos_sin, static: Optional[dict]) -> torch.Tensor:
        """[B, T, (heads + 2 kv_heads) * head_dim] fused projections -> RoPE -> cache update -> attention over the
        cache -> [B, T, heads * head_dim] (this rank's heads)."""
        c = self.cfg
        b, t, _ = qkv.shape
        if not self.kv_quant and c.head_dim == 128:
            # RoPE on q and k and the cache append in one kernel (same float32 arithmetic as _rope, bit for bit)
            cos, sin = cos_sin[0].reshape(t, c.head_dim), cos_sin[1].reshape(t, c.head_dim)
            if static is None:
                k = torch.empty(b, t, self.kv_heads, c.head_dim, dtype=qkv.dtype, device=qkv.device)
                v = torch.empty_like(k)
                q = ops.rope_kv_append(qkv, cos, sin, self.heads, self.kv_heads, k, v, 0)
                if pos0 == 0:
                    self.kv[li] = (k, v)
                else:
                    self.kv[li] = (torch.cat([self.kv[li][0], k], 1), torch.cat([self.kv[li][1], v], 1))
                kk, vv = self.kv[li]
                attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                      is_causal=(t > 1), enable_gqa=True)
            else:
                kk, vv = static["k"][li], static["v"][li]
                q = ops.rope_kv_append(qkv, cos, sin, self.heads, self.kv_heads, kk, vv, static["pos"])
                attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                      attn_mask=static["mask"], enable_gqa=True)
            return attn.transpose(1, 2).reshape(b, t, self.heads * c.head_dim)
        q, k, v = qkv.split([self.heads * c.head_dim, self.kv_heads * c.head_dim, self.kv_heads * c.head_dim], -1)
        q, k, v = q.view(b, t, self.heads, c.head_dim), k.view(b, t, self.kv_heads, c.head_dim), v.view(b, t, self.kv_heads, c.head_dim)
        q, k = self._rope(q, k, cos_sin)
        if self.kv_quant:
            # NVFP4 cache: keys rotated over the head dimension (queries get the same rotation), values as they are
            # (the reference's k_bits / v_bits "nvfp4", promix/configs/llama-3-8b-mxfp8-nvfp4-kv4.yaml:20-25).  The
            # cache holds the packed rows: 64 code bytes + 8 scale bytes per (token, head) instead of 256 bytes.
            q = kv_cache.rotate_heads(q)
            k = kv_cache.pack_head_rows(k, hadamard=True)
            v = kv_cache.pack_head_rows(v, hadamard=False)
            if self.kv_quant == "fake":            # keep, in bf16, exactly what the packed cache gives back
                k, v = kv_cache.unpack_head_rows(k), kv_cache.unpack_head_rows(v)
        packed_cache = bool(self.kv_quant) and self.kv_quant != "fake"
        if static is None:
            if pos0 == 0:
                self.kv[li] = (k, v)
            else:
                self.kv[li] = (torch.cat([self.kv[li][0], k], 1), torch.cat([self.kv[li][1], v], 1))
            kk, vv = self.kv[li]
            if packed_cache:                       # dequantise on read (no attention kernel reads the codes yet)
                kk, vv = kv_cache.unpack_head_rows(kk), kv_cache.unpack_head_rows(vv)
            attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                  is_causal=(t > 1), enable_gqa=True)
        else:
            kk, vv = static["k"][li], static["v"][li]
            kk.index_copy_(1, static["pos"], k)
            vv.index_copy_(1, static["pos"], v)
            if packed_cache:
                kk, vv = kv_cache.unpack_head_rows(kk), kv_cache.unpack_head_rows(vv)
            attn = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                  attn_mask=static["mask"], enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(b, t, self.heads * c.head_dim)
        return attn

    def _forward_layer(self, li: int, h: torch.Tensor, delta: Optional[torch.Tensor], pos0: int, cos_sin,
                       static: Optional[dict] = None):
        """One decoder layer.  `h` is the residual stream and `delta` the previous layer's MLP output that has
        not been added to it yet (None for the first layer): the add is fused into this layer's first
        RMSNorm-quant kernel, and the layer returns its own (h, delta) in the same form.

        Without `static`, keys and values are kept in a growing Python-side cache (prefill, and decode steps of
        arbitrary length).  With `static` (a dict holding preallocated caches [B, T_max, ...], the device tensors
        `pos` [1] int64 and the additive `mask` [1, 1, 1, T_max]) every shape is fixed and the position is data, which
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
        attn = self._attention(li, qkv, pos0, cos_sin, static)
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
    def forward(self, input_ids: torch.Tensor, pos0: int = 0, all_positions: bool = False) -> torch.Tensor:
        """input_ids [B, T] -> logits of the last position [B, vocab] (float32), or of every position
        [B, T, vocab] with `all_positions` (what the reference's forward returns, forward_pass.py:178-183)."""
        rows = input_ids.shape[0] * input_ids.shape[1]
        if (self.scatter is not None and pos0 == 0 and rows <= self.scatter.rows and rows % self.ctx.size == 0
                and rows > (self.peer.rows if self.peer is not None else 16)):
            return self._prefill_scattered(input_ids, all_positions)
        if pos0 == 0:
            self.kv = [None] * len(self.layers)
        h = F.embedding(input_ids, self.embed)
        t = input_ids.shape[1]
        cos_sin = self._rope_angles(torch.arange(pos0, pos0 + t, device=h.device, dtype=torch.float32))   # once per pass
        delta = None
        for li in range(len(self.layers)):
            h, delta = self._forward_layer(li, h, delta, pos0, cos_sin)
        self.pos = pos0 + input_ids.shape[1]
        h = self._finish(h, delta)
        return self._logits(h if all_positions else h[:, -1])

    def _prefill_scattered(self, input_ids: torch.Tensor, all_positions: bool) -> torch.Tensor:
        """Prefill with the residual stream sharded by rows (sequence-parallel between the linears).  Rank r keeps
        rows [r * R / world, (r + 1) * R / world) of h; every row-parallel linear writes its partial output for all
        R rows into the peer-visible buffer, and one kernel per norm reduces this rank's rows over NVLink, adds,
        normalises, quantises, and stores the packed rows into every rank's packed buffer, which the next
        column-parallel linear then reads whole.  Same arithmetic per row as the all-reduce path: the logits are
        bit-identical."""
        c, sr = self.cfg, self.scatter
        b, t = input_ids.shape
        R = b * t
        per = R // self.ctx.size
        self.kv = [None] * len(self.layers)
        h_full = F.embedding(input_ids, self.embed).view(R, -1)
        h = h_full[self.ctx.rank * per:(self.ctx.rank + 1) * per].contiguous()
        cos_sin = self._rope_angles(torch.arange(0, t, device=h.device, dtype=torch.float32))
        pa = ops.pack(h_full, self.k_hi_hidden, hadamard=True, gamma=self.layers[0].ln1, eps=c.rms_eps)
        del h_full
        for li, L in enumerate(self.layers):
            if li > 0:      # h += previous down_proj (reduced over the ranks); RMSNorm(ln1); quantise; gather
                h, pa = ops.reduce_scatter_add_rmsnorm_pack(sr, R, h, L.ln1, c.rms_eps)
            attn = self._attention(li, L.qkv(pa).view(b, t, -1), 0, cos_sin, None)
            L.o(attn.reshape(R, -1), out=sr.buffer(R))
            h, pa = ops.reduce_scatter_add_rmsnorm_pack(sr, R, h, L.ln2, c.rms_eps)
            pa = ops.silu_mul_pack(L.gate_up(pa), self.k_hi_ffn)
            L.down(pa, out=sr.buffer(R))
        h, _ = ops.reduce_scatter_add_rmsnorm_pack(sr, R, h, self.final_norm, c.rms_eps)     # last add; packed rows unused
        self.pos = t
        import torch.distributed as dist
        if all_positions:
            full = torch.empty(R, c.hidden_size, dtype=h.dtype, device=h.device)
            dist.all_gather_into_tensor(full, h, group=self.ctx.group)
            return self._logits(full.view(b, t, -1))
        return self._logits(gather_last_positions(h, b, t, self.ctx.rank, self.ctx.size, self.ctx.group))

    def _logits(self, h_last: torch.Tensor) -> torch.Tensor:
        """Final norm + unquantised LM head in the model dtype, for rows [..., hidden] (inference/forward_pass.py:178-181 in the reference)."""
        last = rms_norm(h_last, self.final_norm, self.cfg.rms_eps)
        return F.linear(last, self.lm_head).float()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, steps: int, use_graph: bool = True) -> torch.Tensor:
        """Prefill + `steps` greedy decode steps; returns the generated ids [B, steps].

        With `use_graph` the decode step (fixed shapes: caches preallocated for prefill + steps positions, the
        position and the attention mask held in device memory) is captured once in a CUDA graph and replayed, so
        a step costs its kernels and not ~2000 Python-side launches.  The graph and its buffers are kept: the next
        call with the same batch, prompt length and step count reloads the caches and replays every step."""
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
        # the decode state of this shape - caches, position, mask, token buffers and, once captured, the graph - is
        # kept: a later call with the same (batch, prompt length, steps) reloads the caches and only replays
        S = self._decode_states.get((b, t0, steps))
        nxt_dtype = self.embed.dtype       # the attention mask is additive, in the model dtype, built once per step
        if S is None:
            S = _DecodeState()
            S.st = {"k": [], "v": [], "pos": torch.zeros(1, dtype=torch.int64, device=dev),
                    "mask": torch.zeros(1, 1, 1, t_max, dtype=nxt_dtype, device=dev)}      # additive: 0 / -inf
            for li in range(len(self.layers)):
                for name, src in (("k", self.kv[li][0]), ("v", self.kv[li][1])):    # bf16 rows or packed rows
                    S.st[name].append(torch.zeros(b, t_max, self.kv_heads, src.shape[-1], dtype=src.dtype, device=dev))
            S.tok = torch.zeros_like(nxt)                                    # [B, 1] current token, updated in place
            S.out = torch.zeros(b, steps, dtype=nxt.dtype, device=dev)
            S.step_idx = torch.zeros(1, dtype=torch.int64, device=dev)
            S.arange = torch.arange(t_max, device=dev)
            S.graph, S.first_set = None, None
            self._decode_states.clear()                                      # one shape at a time: the caches are large
            self._decode_states[(b, t0, steps)] = S
        st, tok, out, step_idx = S.st, S.tok, S.out, S.step_idx
        for li in range(len(self.layers)):
            st["k"][li][:, :t0].copy_(self.kv[li][0])
            st["v"][li][:, :t0].copy_(self.kv[li][1])
        self.kv = [None] * len(self.layers)
        st["pos"].fill_(t0)
        step_idx.zero_()
        tok.copy_(nxt)

        def decode_step():
            out.index_copy_(1, step_idx, tok)
            st["mask"].copy_(torch.where(S.arange <= st["pos"], 0.0, float("-inf")).view(1, 1, 1, t_max))
            h = F.embedding(tok, self.embed)
            cos_sin = self._rope_angles(st["pos"].to(torch.float32))
            delta = None
            for li in range(len(self.layers)):
                h, delta = self._forward_layer(li, h, delta, 0, cos_sin, static=st)
            tok.copy_(self._logits(self._finish(h, delta)[:, -1]).argmax(-1, keepdim=True))
            st["pos"].add_(1)
            step_idx.add_(1)

        if S.graph is not None and (self.peer is None or self.peer.next == S.first_set):
            for _ in range(steps):                                           # every step from the kept graph
                S.graph.replay()
        else:
            decode_step()                                                    # warm-up (also step 0 of the output)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                decode_step()                                                # step 1, eager on the capture stream
                side.synchronize()
                if steps > 2:
                    calls_before = self.peer.calls if self.peer is not None else 0
                    S.first_set = self.peer.next if self.peer is not None else None
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
            if steps > 2:
                S.graph = graph
        ev[2].record()
        ops.check_device_status(dev)                                         # a missing rank or a protocol error is loud
        self.timing_events = ev      # prefill = ev[0] -> ev[1], decode (incl. a capture, if any) = ev[1] -> ev[2], once synchronised
        self.pos = t_max
        return out.clone()           # the buffer belongs to the kept decode state


def gather_last_positions(h_slice: torch.Tensor, batch: int, seq: int, rank: int, world: int, group=None) -> torch.Tensor:
    """Row-sharded residual stream -> the last position of every sequence, on every rank.  `h_slice` holds rows
    [rank * R / world, (rank + 1) * R / world) of the flattened [batch * seq, hidden] stream; row b * seq + seq - 1
    is contributed by the rank that owns it and as zeros by the others, and one all-reduce (exact: a single
    non-zero term per row) hands it to everybody.  Returns [batch, hidden] in the dtype of `h_slice`."""
    import torch.distributed as dist
    per = batch * seq // world
    rows = torch.arange(batch, device=h_slice.device) * seq + (seq - 1) - rank * per
    own = (rows >= 0) & (rows < per)
    last = torch.where(own[:, None], h_slice[rows.clamp(0, per - 1)].float(), torch.zeros((), device=h_slice.device))
    dist.all_reduce(last, group=group)
    return last.to(h_slice.dtype)


class IndependentResQForward:
    """The reference's forward object by name (inference/forward_pass.py:118-183 there): built from a dict of
    weights and a config dict, moved to the GPU with `.to()`, `forward(input_ids)` returns the logits of every
    position.  Here the linears run on the packed NVFP4 / MXFP8 kernels; the object is a thin shell around
    `ResQForwardB200`.

    weights  {"embed", "final_norm", "lm_head", "l{i}.ln1", "l{i}.ln2", "l{i}.q_proj.weight", "l{i}.k_proj.weight",
             "l{i}.v_proj.weight", "l{i}.o_proj.weight", "l{i}.mlp.gate_proj.weight", "l{i}.mlp.up_proj.weight",
             "l{i}.mlp.down_proj.weight"}: full (unsharded) tensors, any float dtype; quantised on the device when
             the object is moved there (round to nearest; last 1/32 of the input channels in MXFP8).
    config   {"num_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "intermediate_size",
             "rope_theta", optional "vocab_size", "rms_eps", "high_fraction"}

    Differences from the reference that follow from the formats: every linear rotates its input by the
    block-Hadamard(128) (the weights carry the same rotation, applied once at packing time), so `online_had` of
    `_quantized_linear` has nothing left to switch; q/k/v and gate/up are stored fused."""

    def __init__(self, weights: Dict[str, torch.Tensor], config: dict, ctx: Optional[tp.TPContext] = None, **model_kw):
        self.weights, self.config, self.ctx, self._model_kw = weights, config, ctx, model_kw
        self.num_layers = config["num_layers"]
        self.hidden_size = config["hidden_size"]
        self.num_heads = config["num_attention_heads"]
        self.num_kv_heads = config["num_key_value_heads"]
        self.head_dim = self.hidden_size // self.num_heads
        self.intermediate_size = config["intermediate_size"]
        self.rope_theta = config.get("rope_theta", 500000.0)
        self.device = "cpu"
        self.model: Optional[ResQForwardB200] = None

    def _llama_config(self) -> LlamaConfig:
        c = self.config
        return LlamaConfig(self.hidden_size, self.intermediate_size, self.num_layers, self.num_heads, self.num_kv_heads,
                           self.head_dim, c.get("vocab_size", self.weights["embed"].shape[0]), self.rope_theta,
                           c.get("rms_eps", 1e-5), c.get("high_fraction", 1.0 / 32))

    def to(self, device):
        """Moves to `device` (a CUDA device: there is no CPU path) and packs the weights there."""
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("IndependentResQForward runs on a CUDA device only: plaquant_b200 has no CPU path")
        self.device = device
        self.model = ResQForwardB200(self._llama_config(), dev, self.ctx, weights=self.weights, **self._model_kw)
        return self

    def _require_model(self) -> ResQForwardB200:
        if self.model is None:
            raise RuntimeError("call .to('cuda') first: the weights are packed on the device")
        return self.model

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Full forward pass; logits [B, T, vocab] (float32)."""
        return self._require_model().forward(input_ids, all_positions=True)

    __call__ = forward

    def generate(self, input_ids: torch.Tensor, steps: int, **kw) -> torch.Tensor:
        return self._require_model().generate(input_ids, steps, **kw)

    _SLICES = {"q_proj": ("qkv", 0), "k_proj": ("qkv", 1), "v_proj": ("qkv", 2), "o_proj": ("o", None),
               "mlp.gate_proj": ("gate_up", 0), "mlp.up_proj": ("gate_up", 1), "mlp.down_proj": ("down", None)}

    def _quantized_linear(self, x: torch.Tensor, prefix: str, online_had: bool = False) -> torch.Tensor:
        """x[..., K] through the quantised linear named `prefix` ("l3.q_proj", "l0.mlp.down_proj", ...), as
        forward_pass.py:278-319 of the reference: rotation, activation quantiser, packed product (this rank's
        shard under tensor parallelism).  q/k/v and gate/up are slices of their fused linears."""
        m = self._require_model()
        layer, name = prefix.split(".", 1)
        fused, part = self._SLICES[name]
        y = m._quantized_linear(x, getattr(m.layers[int(layer[1:])], fused))
        if part is None:
            return y
        hd = m.cfg.head_dim
        sizes = [m.heads * hd, m.kv_heads * hd, m.kv_heads * hd] if fused == "qkv" else [m.ffn, m.ffn]
        return y.split(sizes, -1)[part]


def synthetic_weights(cfg: LlamaConfig, seed: int = 0, num_layers: Optional[int] = None, device="cuda") -> Dict[str, torch.Tensor]:
    """The weights `ResQForwardB200(cfg, device, seed=seed)` draws on one rank, as a dict under the reference's
    names (the form `IndependentResQForward` takes).  Only sensible for small configurations: the dict holds
    every bf16 tensor at once."""
    probe = ResQForwardB200.__new__(ResQForwardB200)
    probe.cfg, probe.device, probe.ctx = cfg, torch.device(device), tp.TPContext()
    probe.heads, probe.kv_heads, probe.ffn = cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size
    hd = cfg.head_dim
    out: Dict[str, torch.Tensor] = {}
    for li in range(cfg.num_layers if num_layers is None else num_layers):
        t = probe._random_layer(li, seed)
        q, k, v = t["qkv"].split([cfg.num_heads * hd, cfg.num_kv_heads * hd, cfg.num_kv_heads * hd], 0)
        gate, up = t["gate_up"].split([cfg.intermediate_size, cfg.intermediate_size], 0)
        p = f"l{li}"
        out.update({f"{p}.ln1": t["ln1"], f"{p}.ln2": t["ln2"], f"{p}.q_proj.weight": q, f"{p}.k_proj.weight": k,
                    f"{p}.v_proj.weight": v, f"{p}.o_proj.weight": t["o"], f"{p}.mlp.gate_proj.weight": gate,
                    f"{p}.mlp.up_proj.weight": up, f"{p}.mlp.down_proj.weight": t["down"]})
    g = torch.Generator(device=probe.device).manual_seed(seed * 100003 + 999983)
    out["embed"] = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g, device=probe.device) * 0.02).to(torch.bfloat16)
    out["final_norm"] = (torch.rand(cfg.hidden_size, generator=g, device=probe.device) + 0.5).to(torch.bfloat16)
    out["lm_head"] = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g, device=probe.device) * 0.02).to(torch.bfloat16)
    return out

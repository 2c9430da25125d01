"""Packed-weight container: the on-disk form of a model whose linears are already NVFP4 / MXFP8.

The reference packs INT weights only (`pack_model_weights`, promix/inference/weight_packer.py:17-77, skips the FP
layers) and exports checkpoints for another runtime with scripts/convert_resq_to_sglang.py:27-242; for the FP
formats its spec fixes the byte layout (docs/specs/spec-mxfp8-nvfp4.md:150-176) but nothing writes it.  This
module writes and reads it.

One file per tensor-parallel rank (`torch.save` of plain CPU tensors and python scalars):

    format, version      "plaquant_b200.packed", 1
    config               the LlamaConfig fields
    num_layers           layers held
    tp                   {"rank", "size"}: the shard this file is
    linears[name]        {"n", "k_lo", "k_hi", "rotated", "sf_layout"} for name = "l{i}.qkv" | ".o" | ".gate_up" | ".down"
    tensors[name + ...]  ".lo_codes" u8 [n, k_lo/2] (E2M1, low nibble = lower K), ".lo_sf" u8 [n, k_lo/16] (E4M3),
                         ".hi_codes" u8 [n, k_hi] (E4M3), ".hi_sf" u8 [n, k_hi/32] (E8M0), row-major: the spec's
                         layout and what `QuantizedLinear` is constructed from; plus "l{i}.ln1", "l{i}.ln2", "embed",
                         "final_norm", "lm_head" in bf16

Files are per tensor-parallel degree: a row-parallel linear's K shard designates its own last columns as the
MXFP8 subspace (tp.outlier_count), so a shard cannot be cut out of codes packed for another degree.  Loading
copies bytes; nothing is re-quantised, so logits after save -> load are bit-identical.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import tp
from .real_forward import pack_model_weights  # noqa: F401  (the reference keeps it in this module)

FORMAT, VERSION = "plaquant_b200.packed", 1


def shard_path(path: str, rank: int, size: int) -> str:
    """`path` for a single rank; `stem.tp{size}-rank{rank}.ext` otherwise."""
    if size == 1:
        return path
    stem, ext = os.path.splitext(path)
    return f"{stem}.tp{size}-rank{rank}{ext}"


def save_packed(model, path: str) -> str:
    """Writes this rank's shard of `model` (a forward_pass.ResQForwardB200); returns the file written."""
    state = model.packed_state()
    state["tensors"] = {k: (v.detach().cpu() if v is not None else None) for k, v in state["tensors"].items()}
    state["format"], state["version"] = FORMAT, VERSION
    out = shard_path(path, model.ctx.rank, model.ctx.size)
    torch.save(state, out)
    return out


def read_packed(path: str, tp_rank: int = 0, tp_size: int = 1) -> dict:
    """The container of rank `tp_rank` of `tp_size`, validated, tensors still on the CPU."""
    state = torch.load(shard_path(path, tp_rank, tp_size), map_location="cpu", weights_only=True)
    if state.get("format") != FORMAT or state.get("version") != VERSION:
        raise ValueError(f"{path}: not a {FORMAT} v{VERSION} container")
    for name, meta in state["linears"].items():
        t = state["tensors"]
        n, k_lo, k_hi = meta["n"], meta["k_lo"], meta["k_hi"]
        want = {".lo_codes": (n, k_lo // 2), ".lo_sf": (n, k_lo // 16), ".hi_codes": (n, k_hi), ".hi_sf": (n, k_hi // 32)}
        for suffix, shape in want.items():
            got = t.get(name + suffix)
            if got is None or got.dtype != torch.uint8 or tuple(got.shape) != shape:
                raise ValueError(f"{path}: {name}{suffix} should be uint8 {shape}")
    return state


def load_packed(path: str, device, tp_rank: int = 0, tp_size: int = 1, ctx: Optional[tp.TPContext] = None,
                num_layers: Optional[int] = None, **model_kw):
    """Rebuilds the decoder of rank `tp_rank` of `tp_size` on `device` from its container."""
    from .forward_pass import LlamaConfig, ResQForwardB200
    state = read_packed(path, tp_rank, tp_size)
    ctx = ctx or tp.TPContext(tp_rank, tp_size, None)
    cfg = LlamaConfig(**state["config"])
    return ResQForwardB200(cfg, device, ctx, num_layers=num_layers if num_layers is not None else state["num_layers"],
                           packed=state, **model_kw)

"""Model-level installers with the reference's names (promix/inference/real_forward.py:34-164 and
promix/inference/weight_packer.py:17-77 in the reference), for the FP formats the reference skips.

    init_kernel()            load (and if needed build) the CUDA library
    pack_model_weights(m)    quantise every nn.Linear of a module tree on the GPU -> QuantizedLinear
    install_real_forward(m)  make those linears run the packed kernels

Unlike the reference there is no PyTorch fallback when the library is missing
(real_forward.py:122-129 there): loading fails loudly.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn as nn

from . import _lib, build
from .quantize import QuantizedLinear

_kernel_loaded = False


def init_kernel(path: Optional[str] = None, build_if_missing: bool = True):
    """Loads libplq_b200.so (optionally from `path`); returns the ctypes handle."""
    global _kernel_loaded
    if path is not None:
        _lib.LIB_PATH = path
    elif build_if_missing and build.needs_build():
        build.build_library()
    handle = _lib.lib()
    _kernel_loaded = True
    return handle


def pack_model_weights(model: nn.Module, high_fraction: float = 1.0 / 32, rotate: bool = True,
                       skip: Callable[[str], bool] = lambda name: "lm_head" in name) -> Dict[str, QuantizedLinear]:
    """name -> QuantizedLinear for every nn.Linear under `model` (bf16 weights on a CUDA device).
    The LM head stays unquantised, as in the reference (inference/forward_pass.py:180-181)."""
    packed = {}
    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear) and not skip(name):
            if mod.bias is not None:
                raise ValueError(f"{name}: bias is not supported (Llama linears have none)")
            packed[name] = QuantizedLinear.from_weight(mod.weight.detach().to(torch.bfloat16), high_fraction, rotate,
                                                       online_had=rotate)
    return packed


class _PackedLinear(nn.Module):
    def __init__(self, q: QuantizedLinear):
        super().__init__()
        self.q = q

    def forward(self, x):
        return self.q(x.to(torch.bfloat16)).to(x.dtype)


def install_real_forward(model: nn.Module, packed: Optional[Dict[str, QuantizedLinear]] = None, **pack_kw) -> int:
    """Replaces the packed linears inside `model` by modules that call the kernels; returns how many."""
    if not _kernel_loaded:
        init_kernel()
    if packed is None:
        packed = pack_model_weights(model, **pack_kw)
    n = 0
    for name, q in packed.items():
        parent = model
        *path, leaf = name.split(".")
        for part in path:
            parent = getattr(parent, part)
        setattr(parent, leaf, _PackedLinear(q))
        n += 1
    return n

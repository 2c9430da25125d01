"""Helpers shared by the GPU parity tests: seeded synthetic inputs (the shapes, sizes and value
distributions of the benchmark configurations) and numpy <-> torch bf16 conversion."""
import numpy as np
import torch

from oracle import formats as F


def synth_activation(rows, k, seed, outlier_frac=0.01, outlier_gain=20.0):
    """bf16 N(0,1) with a seeded 1% of the channels multiplied by 20 (generated on the CPU so the
    CPU oracle and the GPU see identical bits)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g, dtype=torch.float32)
    idx = torch.randperm(k, generator=g)[: int(outlier_frac * k)]
    x[:, idx] *= outlier_gain
    return x.to(torch.bfloat16)


def synth_weight(n, k, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)


def synth_gamma(k, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f32_of(t: torch.Tensor) -> np.ndarray:
    return F.bf16_bits_to_f32(bits_of(t))


def from_bits(bits: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16).to(device)


def packed_to_numpy(p) -> dict:
    """plaquant_b200.PackedMatrix -> the oracle's dict form with row-major scale buffers."""
    lo_sf, hi_sf = p.lo_sf.cpu().numpy(), p.hi_sf.cpu().numpy()
    if p.sf_layout == 1:
        lo_sf = F.untile_sf(lo_sf, p.rows, p.k_lo // 16) if p.k_lo else np.zeros((p.rows, 0), np.uint8)
        hi_sf = F.untile_sf(hi_sf, p.rows, p.k_hi // 32) if p.k_hi else np.zeros((p.rows, 0), np.uint8)
    return {"rows": p.rows, "k_lo": p.k_lo, "k_hi": p.k_hi, "lo_codes": p.lo_codes.cpu().numpy(),
            "lo_sf": lo_sf.reshape(p.rows, -1), "hi_codes": p.hi_codes.cpu().numpy(), "hi_sf": hi_sf.reshape(p.rows, -1)}


def assert_packed_equal(got: dict, want: dict):
    for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"):
        a, b = got[key], want[key]
        assert a.shape == b.shape, (key, a.shape, b.shape)
        bad = int((a != b).sum())
        assert bad == 0, f"{key}: {bad} of {a.size} bytes differ"


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64); b = b.astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))

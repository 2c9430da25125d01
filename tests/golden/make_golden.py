"""Generate the golden fixtures in this directory by running the REFERENCE's own code.

Run once, on a machine that has the reference checkout (it is not needed at test time):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

What is stored (all small, deterministic, seeded):
  pack_small.npz ......... bf16 inputs with outlier channels -> codes and scale bytes derived
                           from the reference's own intermediates (select_block_scales_*,
                           _round_to_nearest_value), after checking that re-multiplying them
                           reproduces fake_quantize_nvfp4 / fake_quantize_mxfp8 bit for bit,
                           plus the ActQuantizer [main | high] routed fake-quant output.
  scales_exhaustive.npz .. scale bytes for every finite non-negative bf16 block maximum.
  kats.npz ............... tie / midpoint / zero / saturation known answers.
  norm_rot.npz ........... rms_norm -> (x.float() @ H).to(bf16) from the reference functions,
                           used to bound the deterministic restatement's distance from torch.
  rope.npz ............... apply_rotary_pos_emb of the reference on bf16-valued float32 heads.
  linear_cfg0.npz ........ the single-linear config: Y = F.linear(fq(rot(X)), fq(rot(W))) in
                           bf16 and the same product in float32, with input checksums.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(ref_root):
    # fast_hadamard_transform is imported (never called) on the FP fake-quant path.
    stub = types.ModuleType("fast_hadamard_transform")
    stub.hadamard_transform = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("stub"))
    sys.modules["fast_hadamard_transform"] = stub
    sys.path.insert(0, ref_root)
    import promix.quantize.quant_utils as qu  # noqa
    import inference.rotation as rot  # noqa
    import inference.forward_pass as fp  # noqa
    return qu, rot, fp


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def synth_activation(rows, k, seed, outlier_frac=0.01, outlier_gain=20.0):
    """N(0,1) with a seeded 1% of channels multiplied by 20, cast to bf16."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g, dtype=torch.float32)
    idx = torch.randperm(k, generator=g)[: int(outlier_frac * k)]
    x[:, idx] *= outlier_gain
    return x.to(torch.bfloat16)


def ref_codes_nvfp4(qu, x):
    """Codes/scales from the reference's intermediates; asserts they rebuild its output."""
    xf = x.float()
    s = qu.select_block_scales_nvfp4(xf)                                 # [.., K/16] fp32
    grid = torch.tensor(qu.FP4_E2M1_POS, dtype=torch.float32)
    xb = xf.view(*xf.shape[:-1], -1, 16)
    q = qu._round_to_nearest_value((xb / s.unsqueeze(-1)).clamp(-6.0, 6.0), grid)
    deq = (q * s.unsqueeze(-1)).view(xf.shape).to(x.dtype)
    assert torch.equal(deq.view(torch.int16), qu.fake_quantize_nvfp4(x).view(torch.int16))
    idx = torch.searchsorted(grid, q.abs().contiguous())
    assert torch.equal(grid[idx], q.abs())
    codes = (idx | (torch.signbit(q).long() << 3)).to(torch.uint8).view(xf.shape)
    sbytes = s.to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(s.to(torch.float8_e4m3fn).float(), s)
    return codes.numpy(), sbytes.numpy(), deq


def ref_codes_mxfp8(qu, x):
    xf = x.float()
    s = qu.select_block_scales_mxfp8(xf)
    grid = torch.tensor(qu._FP8_E4M3_POS, dtype=torch.float32)
    xb = xf.view(*xf.shape[:-1], -1, 32)
    q = qu._round_to_nearest_value((xb / s.unsqueeze(-1)).clamp(-448.0, 448.0), grid)
    deq = (q * s.unsqueeze(-1)).view(xf.shape).to(x.dtype)
    assert torch.equal(deq.view(torch.int16), qu.fake_quantize_mxfp8(x).view(torch.int16))
    idx = torch.searchsorted(grid, q.abs().contiguous())
    assert torch.equal(grid[idx], q.abs())
    codes = (idx | (torch.signbit(q).long() << 7)).to(torch.uint8).view(xf.shape)
    e = torch.log2(s)
    assert torch.equal(e, e.round())
    sbytes = (e + 127).to(torch.uint8)
    return codes.numpy(), sbytes.numpy(), deq


def main(ref_root):
    qu, rot, fp = _import_reference(ref_root)
    torch.set_num_threads(os.cpu_count())

    # ---------------- pack_small -------------------------------------------------------
    out = {}
    cases = {"a": (8, 512, 64, 11), "b": (5, 4096, 128, 12), "c": (3, 1024, 0, 13), "d": (4, 256, 256, 14)}
    for name, (rows, k, k_hi, seed) in cases.items():
        x = synth_activation(rows, k, seed)
        if name == "a":          # edge content: zero blocks, -0.0, tiny, huge, exact ties
            x[0, :32] = 0.0
            x[1, :16] = -0.0
            x[2, :16] = torch.tensor([6.0, 5.0, 2.5, 1.75, 1.25, 0.75, 0.25, -0.25, -0.75, -1.25,
                                      -1.75, -2.5, -5.0, -6.0, 3.5, -3.5]).to(torch.bfloat16)
            x[3, 16:32] = 3.0e38
            x[3, 32:48] = 1.0e-38
            x[4, 448:480] = torch.linspace(-1e-3, 1e-3, 32).to(torch.bfloat16)
            x[5, 448:512] = 5.0e4
            x[6, 448:480] = 0.0
        k_lo = k - k_hi
        out[f"{name}_x"] = bf16_bits(x)
        out[f"{name}_khi"] = np.int64(k_hi)
        parts = []
        if k_lo:
            c, s, deq = ref_codes_nvfp4(qu, x[:, :k_lo])
            out[f"{name}_lo_codes"], out[f"{name}_lo_sf"] = c, s
            parts.append(deq)
        if k_hi:
            c, s, deq = ref_codes_mxfp8(qu, x[:, k_lo:])
            out[f"{name}_hi_codes"], out[f"{name}_hi_sf"] = c, s
            parts.append(deq)
        # the routed fake quantiser (quant_utils.py:182-224) must equal the per-segment calls
        aq = qu.ActQuantizer()
        if k_lo and k_hi:
            aq.configure(bits="nvfp4", high_bits="mxfp8", high_bits_length=k_hi)
        else:
            aq.configure(bits="nvfp4" if k_lo else "mxfp8")
        routed = aq(x)
        assert torch.equal(routed.view(torch.int16), torch.cat(parts, -1).view(torch.int16))
        out[f"{name}_fq"] = bf16_bits(routed)
    np.savez_compressed(os.path.join(HERE, "pack_small.npz"), **out)

    # ---------------- scales_exhaustive ------------------------------------------------
    bits = np.arange(0, 0x7F80, dtype=np.uint16)          # every finite non-negative bf16
    v = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
    blk16 = torch.zeros(bits.size, 16, dtype=torch.bfloat16); blk16[:, 3] = v
    blk32 = torch.zeros(bits.size, 32, dtype=torch.bfloat16); blk32[:, 5] = v
    s4 = torch.cat([qu.select_block_scales_nvfp4(blk16[i:i + 4096].float()) for i in range(0, bits.size, 4096)])
    s8 = qu.select_block_scales_mxfp8(blk32.float())
    e = torch.log2(s8); assert torch.equal(e, e.round())
    np.savez_compressed(os.path.join(HERE, "scales_exhaustive.npz"),
                        nvfp4=s4.to(torch.float8_e4m3fn).view(torch.uint8).numpy().reshape(-1),
                        mxfp8=(e + 127).to(torch.uint8).numpy().reshape(-1))

    # ---------------- kats --------------------------------------------------------------
    g4 = torch.tensor(qu.FP4_E2M1_POS, dtype=torch.float32)
    g8 = torch.tensor(qu._FP8_E4M3_POS, dtype=torch.float32)
    x4 = torch.tensor([1.25, -1.25, 1.75, 2.5, 5.0, 1.1, 1.4, 0.25, 0.75, 3.5, -0.0, 0.0, 6.0, -6.0,
                       0.2499, 0.2501] + list(qu.FP4_E2M1_POS), dtype=torch.float32)
    a, b = 2.0 ** -6, 1.125 * 2.0 ** -6
    x8 = torch.tensor([0.5 * (a + b), -0.5 * (a + b), 2.0 ** -10, 3 * 2.0 ** -10, 448.0, -448.0, 440.0,
                       432.0, 2.0 ** -11, -2.0 ** -11, 0.0, 17.0, 19.0], dtype=torch.float32)
    np.savez_compressed(os.path.join(HERE, "kats.npz"),
                        x4=x4.numpy(), y4=qu._round_to_nearest_value(x4, g4).numpy(),
                        x8=x8.numpy(), y8=qu._round_to_nearest_value(x8, g8).numpy(),
                        e2m1_grid=g4.numpy(), e4m3_grid=g8.numpy())

    # ---------------- norm_rot -----------------------------------------------------------
    x = synth_activation(16, 4096, 21)
    g = torch.Generator().manual_seed(22)
    gamma = (torch.rand(4096, generator=g) + 0.5).to(torch.bfloat16)
    y = fp.rms_norm(x, gamma, eps=1e-6)
    H = rot.get_hadamard_matrix(128)
    z = (y.float().view(16, 32, 128) @ H).view(16, 4096).to(torch.bfloat16)
    zh = (x.float().view(16, 32, 128) @ H).view(16, 4096).to(torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "norm_rot.npz"), x=bf16_bits(x), gamma=bf16_bits(gamma),
                        norm=bf16_bits(y), norm_rot=bf16_bits(z), rot_only=bf16_bits(zh),
                        h128_row1=H[1].numpy())

    # ---------------- linear_cfg0 ---------------------------------------------------------
    X = synth_activation(16, 4096, 0)
    g = torch.Generator().manual_seed(1)
    W = (torch.randn(4096, 4096, generator=g) * 0.02).to(torch.bfloat16)
    Xr = (X.float().view(16, 32, 128) @ H).view(16, 4096).to(torch.bfloat16)
    Wr = (W.float().view(4096, 32, 128) @ H).view(4096, 4096).to(torch.bfloat16)
    aq = qu.ActQuantizer(); aq.configure(bits="nvfp4", high_bits="mxfp8", high_bits_length=128)
    Xq = aq(Xr)
    Wq = torch.cat([aq(Wr[i:i + 512]) for i in range(0, 4096, 512)])
    Y_bf16 = torch.nn.functional.linear(Xq, Wq)
    Y_f32 = Xq.float() @ Wq.float().T
    np.savez_compressed(os.path.join(HERE, "linear_cfg0.npz"), x=bf16_bits(X),
                        w_checksum=np.uint64(int(bf16_bits(W).astype(np.uint64).sum())),
                        xr=bf16_bits(Xr), wr_rows=bf16_bits(Wr[:4]), wq_rows=bf16_bits(Wq[:4]),
                        y_bf16=bf16_bits(Y_bf16), y_f32=Y_f32.numpy())
    # ---------------- gptq_frozen ---------------------------------------------------------
    # The reference's own GPTQ class on a seeded single-block problem (K = blocksize = 128, so the comparison
    # involves no cross-block matmul, whose float32 summation order is unspecified): 96 output rows, NVFP4 for the
    # first 64 input columns and MXFP8 for the last 64, Hessian from 512 synthetic calibration rows.  The factor
    # of the inverse Hessian that the loop consumes is recomputed here exactly as gptq.py:125-141 does and stored,
    # since LAPACK results are not portable bit for bit.
    from promix.quantize.gptq import GPTQ
    from promix.quantize.kv_quant import WeightQuantizer
    g = torch.Generator().manual_seed(11)
    n_out, k, k_hi = 96, 128, 64
    Wg = (torch.randn(n_out, k, generator=g) * 0.02).to(torch.bfloat16)
    Xc = torch.randn(512, k, generator=g) * (1.0 + 3.0 * torch.rand(k, generator=g))
    layer = torch.nn.Linear(k, n_out, bias=False)
    layer.weight.data = Wg.float().clone()
    gq = GPTQ(layer, mixed_precision=True, high_bits_length=k_hi, low_bits_length=0)
    gq.quantizer = WeightQuantizer(); gq.quantizer.configure("nvfp4", perchannel=True, sym=True, mse=False)
    gq.high_quantizer = WeightQuantizer(); gq.high_quantizer.configure("mxfp8", perchannel=True, sym=True, mse=False)
    gq.add_batch(Xc, None)
    Hm = gq.H.clone()
    Hd = Hm.clone()
    Hd[torch.arange(k), torch.arange(k)] += 0.01 * torch.mean(torch.diag(Hd))
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(Hd)), upper=True)
    gq.fasterquant(blocksize=128, percdamp=0.01, groupsize=-1, actorder=False)
    Qg = layer.weight.data.float()
    np.savez_compressed(os.path.join(HERE, "gptq_frozen.npz"), w=bf16_bits(Wg), hinv=Hinv.numpy(), q=Qg.numpy(),
                        k_hi=np.int64(k_hi))
    # ---------------- rope -------------------------------------------------------------------
    # The reference's apply_rotary_pos_emb (inference/forward_pass.py:82-116) on bf16-valued float32 heads with
    # float32 tables (the reference's decoder feeds it the model dtype; the formula is the same): the product of
    # this repository's kernel is its result rounded to bf16.
    g = torch.Generator().manual_seed(13)
    t, hq, hk = 9, 3, 2
    qf = (torch.randn(2, t, hq, 128, generator=g) * 3).to(torch.bfloat16)
    kf = (torch.randn(2, t, hk, 128, generator=g) * 0.3).to(torch.bfloat16)
    inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    emb = torch.outer(torch.arange(37, 37 + t, dtype=torch.float32), inv)
    emb = torch.cat((emb, emb), dim=-1)
    cos, sin = emb.cos(), emb.sin()
    q_out, k_out = fp.apply_rotary_pos_emb(qf.float(), kf.float(), cos, sin)
    np.savez_compressed(os.path.join(HERE, "rope.npz"), q=bf16_bits(qf), k=bf16_bits(kf), cos=cos.numpy(), sin=sin.numpy(),
                        q_out=q_out.numpy(), k_out=k_out.numpy())
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])

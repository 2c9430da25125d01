"""RoPE + key/value cache append kernel (through the C ABI) against the CPU oracle and against the PyTorch
formulation it replaces, bit for bit; positions from the host and from device memory; a full cache is reported
through the status word, not by a fault."""
import numpy as np
import pytest
import torch

from oracle import formats as F
from tests._util import f32_of

pytestmark = pytest.mark.gpu
plq = pytest.importorskip("plaquant_b200")


def _tables(pos0, t, theta=500000.0):
    inv = 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    ang = torch.outer(torch.arange(pos0, pos0 + t, dtype=torch.float32), inv)
    return torch.cat([ang.cos(), ang.cos()], -1).contiguous(), torch.cat([ang.sin(), ang.sin()], -1).contiguous()


def _torch_rope(v, cos, sin):
    v1, v2 = v[..., :64], v[..., 64:]
    return (v.float() * cos[None, :, None, :] + torch.cat([-v2, v1], -1).float() * sin[None, :, None, :]).to(v.dtype)


@pytest.mark.parametrize("b,t,heads,kv,pos0,t_max", [(2, 5, 4, 2, 0, 5), (3, 1, 8, 1, 7, 16), (1, 33, 2, 2, 100, 160),
                                                    (16, 1, 64, 8, 2048, 2176)])
def test_rope_kv_append_bit_exact(b, t, heads, kv, pos0, t_max):
    from plaquant_b200 import ops
    g = torch.Generator().manual_seed(b * 100 + t)
    qkv = (torch.randn(b, t, (heads + 2 * kv) * 128, generator=g) * 2).to(torch.bfloat16)
    cos, sin = _tables(pos0, t)
    kc = torch.full((b, t_max, kv, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full((b, t_max, kv, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    q = ops.rope_kv_append(qkv.cuda(), cos.cuda(), sin.cuda(), heads, kv, kc, vc, pos0)
    plq.check_device_status()
    qs, ks, vs = qkv.split([heads * 128, kv * 128, kv * 128], -1)
    qs, ks, vs = qs.reshape(b, t, heads, 128), ks.reshape(b, t, kv, 128), vs.reshape(b, t, kv, 128)
    want_q = F.rope_bf16(f32_of(qs), cos.numpy(), sin.numpy())
    want_k = F.rope_bf16(f32_of(ks), cos.numpy(), sin.numpy())
    assert np.array_equal(f32_of(q), want_q)
    assert np.array_equal(f32_of(kc[:, pos0:pos0 + t]), want_k)
    assert np.array_equal(f32_of(vc[:, pos0:pos0 + t]), f32_of(vs))
    assert torch.equal(q.cpu(), _torch_rope(qs, cos, sin)) and torch.equal(kc[:, pos0:pos0 + t].cpu(), _torch_rope(ks, cos, sin))
    untouched = torch.ones(t_max, dtype=torch.bool)
    untouched[pos0:pos0 + t] = False
    assert bool((kc[:, untouched.cuda()] == 7.0).all()) and bool((vc[:, untouched.cuda()] == 7.0).all())
    # the same call with the position in device memory
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    pos = torch.tensor([pos0], dtype=torch.int64, device="cuda")
    q2 = ops.rope_kv_append(qkv.cuda(), cos.cuda(), sin.cuda(), heads, kv, kc2, vc2, pos)
    plq.check_device_status()
    assert torch.equal(q2, q) and torch.equal(kc2[:, pos0:pos0 + t], kc[:, pos0:pos0 + t])
    assert torch.equal(vc2[:, pos0:pos0 + t], vc[:, pos0:pos0 + t])


def test_full_cache_is_reported_not_overrun():
    from plaquant_b200 import ops
    b, t, heads, kv, t_max = 2, 1, 2, 1, 4
    qkv = torch.randn(b, t, (heads + 2 * kv) * 128).to(torch.bfloat16).cuda()
    cos, sin = (x.cuda() for x in _tables(0, t))
    guard = torch.full((b * t_max * kv * 128 + 4096,), 3.0, dtype=torch.bfloat16, device="cuda")
    kc = guard[:b * t_max * kv * 128].view(b, t_max, kv, 128)
    vc = torch.zeros(b, t_max, kv, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(plq.PlqError) as e:                      # host-side position: refused before the launch
        ops.rope_kv_append(qkv, cos, sin, heads, kv, kc, vc, t_max)
    assert e.value.status == -2
    pos = torch.tensor([t_max], dtype=torch.int64, device="cuda")
    ops.rope_kv_append(qkv, cos, sin, heads, kv, kc, vc, pos)   # device-side position: the kernel skips the store
    with pytest.raises(plq.PlqError) as e:
        plq.check_device_status()
    assert e.value.status == 3
    assert bool((guard == 3.0).all()) and bool((vc == 0).all())
    pos.fill_(t_max - 1)
    ops.rope_kv_append(qkv, cos, sin, heads, kv, kc, vc, pos)
    plq.check_device_status()
    assert bool((guard[b * t_max * kv * 128:] == 3.0).all())


def test_decoder_logits_do_not_depend_on_the_rope_path():
    """The decoder with the fused RoPE / append kernel against the same decoder on the PyTorch formulation
    (kv_quant="fake" keeps the old path but changes the cache values, so the old path is forced by hand)."""
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=2048, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=128,
                      vocab_size=512)
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(3)).cuda()
    m = ResQForwardB200(cfg, "cuda", seed=9)
    a = m.forward(ids)
    toks = m.generate(ids, 6)
    import plaquant_b200.ops as ops
    saved = ops.rope_kv_append

    def torch_path(qkv, cos, sin, heads, kv, kc, vc, pos):
        b, t, _ = qkv.shape
        q, k, v = qkv.split([heads * 128, kv * 128, kv * 128], -1)
        q, k, v = q.reshape(b, t, heads, 128), k.reshape(b, t, kv, 128), v.reshape(b, t, kv, 128)
        idx = (pos if isinstance(pos, torch.Tensor) else torch.tensor([pos], device=qkv.device)) + torch.arange(t, device=qkv.device)
        kc.index_copy_(1, idx, _torch_rope(k, cos, sin))
        vc.index_copy_(1, idx, v)
        return _torch_rope(q, cos, sin)
    ops.rope_kv_append = torch_path
    try:
        m2 = ResQForwardB200(cfg, "cuda", seed=9)
        assert torch.equal(m2.forward(ids), a)
        assert torch.equal(m2.generate(ids, 6), toks)
    finally:
        ops.rope_kv_append = saved
    plq.check_device_status()

"""The reference-shaped Python API (QuantizedLinear, fused_mixed_gemm, installers, the decoder
forward) on top of the C ABI, checked against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import formats as F
from tests._util import f32_of, rel_l2, synth_activation, synth_gamma, synth_weight

pytestmark = pytest.mark.gpu
plq = pytest.importorskip("plaquant_b200")


def _oracle_linear(x, w, k_hi, gamma=None):
    px = F.prepare_activation(f32_of(x), k_hi, gamma=None if gamma is None else f32_of(gamma), eps=1e-6, hadamard=True)
    pw = F.prepare_activation(f32_of(w), k_hi, hadamard=True)
    return F.round_to_bf16(F.linear(px, pw))


@pytest.mark.parametrize("rows", [4, 200])
@pytest.mark.parametrize("norm", [False, True])
def test_quantized_linear_matches_oracle(rows, norm):
    from plaquant_b200.quantize import QuantizedLinear
    k, n = 1024, 384
    x, w = synth_activation(rows, k, seed=rows), synth_weight(n, k, seed=9)
    gamma = synth_gamma(k, seed=3) if norm else None
    lin = QuantizedLinear.from_weight(w.cuda(), high_fraction=1 / 32)
    assert (lin.in_features, lin.out_features, lin.high_bits_length, lin.gemm_impl) == (k, n, 64, "b200")
    y = lin(x.cuda().view(2, rows // 2, k), norm_weight=None if gamma is None else gamma.cuda())
    assert y.shape == (2, rows // 2, n) and y.dtype == torch.bfloat16
    plq.check_device_status()
    assert rel_l2(f32_of(y).reshape(rows, n), _oracle_linear(x, w, 64, gamma)) <= 1e-3
    with pytest.raises(NotImplementedError):
        lin.set_kernel("pytorch")              # the reference's fallback does not exist here
    cpu = QuantizedLinear(lin.w_main_int.cpu(), lin.w_main_scale.cpu(), lin.w_high_int.cpu(), lin.w_high_scale.cpu(),
                          online_had=True)
    with pytest.raises(RuntimeError):
        cpu(x)                                 # weights not on a GPU: loud error, no CPU path
    y2 = cpu.to("cuda")(x.cuda(), norm_weight=None if gamma is None else gamma.cuda())
    assert torch.equal(y2, y.view(rows, n))


def test_fused_mixed_gemm_call_shape():
    from plaquant_b200.mixed_gemm import fused_mixed_gemm
    x, w = synth_activation(130, 512, seed=1), synth_weight(264, 512, seed=2)
    pa = plq.pack(x.cuda(), 64, hadamard=True, sf_layout="tiled")
    pb = plq.pack(w.cuda(), 64, hadamard=True, sf_layout="tiled")
    y = fused_mixed_gemm(pa.lo_codes.view(2, 65, -1), pb.lo_codes, pa.hi_codes, pb.hi_codes, pa.lo_sf, pb.lo_sf,
                         None, None, pa.hi_sf, pb.hi_sf, None, None)
    assert y.shape == (2, 65, 264)
    assert torch.equal(y.view(130, 264), plq.mixed_gemm(pa, pb))
    with pytest.raises(ValueError):
        fused_mixed_gemm(pa.lo_codes, pb.lo_codes, pa.hi_codes, pb.hi_codes, pa.lo_sf, pb.lo_sf, torch.zeros(1), None,
                         pa.hi_sf, pb.hi_sf)


def test_install_real_forward_on_a_module_tree():
    from plaquant_b200 import real_forward
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512, bias=False), torch.nn.SiLU(),
                                torch.nn.Linear(512, 128, bias=False)).cuda().to(torch.bfloat16)
    x = synth_activation(32, 256, seed=4).cuda()
    ref = model(x).float()
    real_forward.init_kernel()
    assert real_forward.install_real_forward(model, high_fraction=1 / 8) == 2
    y = model(x).float()
    cos = torch.nn.functional.cosine_similarity(y.flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.97, cos                     # 4-bit weights and activations against the bf16 model


def test_hadamard_matrix_and_decoder_forward():
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200, rms_norm_quant
    from plaquant_b200.rotation import get_hadamard_matrix, is_block_hadamard
    h = get_hadamard_matrix(128)
    assert torch.allclose(h @ h.T, torch.eye(128), atol=1e-5) and is_block_hadamard(h)
    assert torch.equal(torch.sign(h[1]), torch.tensor([1.0, -1.0] * 64))           # Sylvester order
    x = synth_activation(16, 256, seed=8)
    rot = (x.float().view(16, 2, 128) @ h).view(16, 256)
    assert rel_l2(F.block_hadamard_det(f32_of(x)), F.round_to_bf16(rot.numpy())) < 2e-3
    gamma = synth_gamma(256, 2)
    p = rms_norm_quant(x.cuda(), gamma.cuda(), 1e-6, 64, sf_layout="rowmajor")
    want = F.prepare_activation(f32_of(x), 64, gamma=f32_of(gamma), eps=1e-6)
    assert np.array_equal(p.lo_codes.cpu().numpy(), want["lo_codes"])
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                      vocab_size=1000)
    model = ResQForwardB200(cfg, "cuda", seed=1)
    ids = torch.randint(0, 1000, (3, 40), generator=torch.Generator().manual_seed(0)).cuda()
    logits = model.forward(ids)
    assert logits.shape == (3, 1000) and torch.isfinite(logits).all()
    assert torch.equal(logits, model.forward(ids))
    gen = model.generate(ids, 5)
    assert gen.shape == (3, 5)
    # the CUDA-graph decode (static caches, position as data) and the eager growing-cache decode agree
    assert torch.equal(gen, model.generate(ids, 5, use_graph=False))
    # incremental decoding reproduces a full forward over the extended sequence
    full = model.forward(torch.cat([ids, gen[:, :1]], 1))
    model.forward(ids)
    step = model.forward(gen[:, :1], pos0=40)
    assert rel_l2(step.cpu().numpy(), full.cpu().numpy()) < 0.05
    plq.check_device_status()


def test_device_reported_timeout_surfaces_as_an_error():
    """Failure detection without faulting a GPU: a kernel whose bounded wait runs out writes
    PLQ_DEV_TIMEOUT into the status word; here the word is set from the host and the front end
    must raise, name the cause and clear the word."""
    from plaquant_b200 import ops
    w = ops.status_word("cuda")
    w.fill_(1)
    with pytest.raises(plq.PlqError) as e:
        plq.check_device_status()
    assert e.value.status == 1 and "bounded wait" in str(e.value)
    plq.check_device_status()          # cleared


def test_outputs_with_a_row_stride_leave_the_other_columns_alone():
    """y may be a column block of a wider tensor (ldy > n): GEMM, both GEMVs."""
    k, k_hi, n = 1024, 64, 384
    w = synth_weight(n, k, seed=5).cuda()
    for m, op, layout in ((200, plq.mixed_gemm, "tiled"), (16, plq.gemv_tc, "tiled"), (8, plq.gemv, "rowmajor")):
        x = synth_activation(m, k, seed=m).cuda()
        pa = plq.pack(x, k_hi, hadamard=True, sf_layout=layout)
        pb = plq.pack(w, k_hi, hadamard=True, sf_layout=layout)
        want = op(pa, pb)
        wide = torch.full((m, n + 128), 7.0, dtype=torch.bfloat16, device="cuda")
        got = op(pa, pb, out=wide[:, 64:64 + n])
        plq.check_device_status()
        assert got.data_ptr() == wide[:, 64:].data_ptr()
        assert torch.equal(wide[:, 64:64 + n], want)
        assert bool((wide[:, :64] == 7.0).all()) and bool((wide[:, 64 + n:] == 7.0).all())


@pytest.mark.parametrize("k_hi", [0, 64])
def test_kv_cache_quantisation_per_head(k_hi):
    """Keys [batch, tokens, kv_heads, 128] -> packed per-head rows: codes equal the oracle's on the rotated rows,
    the dequantised cache equals the oracle's fake-quantised values, and q . k survives the common rotation."""
    from plaquant_b200 import kv_cache
    k = synth_activation(2 * 9 * 4, 128, seed=21).view(2, 9, 4, 128).cuda()
    q = synth_activation(2 * 9 * 4, 128, seed=22).view(2, 9, 4, 128).cuda()
    p = kv_cache.quantize_heads(k, k_hi=k_hi)
    want = F.prepare_activation(f32_of(k.view(-1, 128)), k_hi, hadamard=True)
    assert np.array_equal(p.lo_codes.cpu().numpy(), want["lo_codes"]) and np.array_equal(p.lo_sf.cpu().numpy(), want["lo_sf"])
    if k_hi:
        assert np.array_equal(p.hi_codes.cpu().numpy(), want["hi_codes"]) and np.array_equal(p.hi_sf.cpu().numpy(), want["hi_sf"])
    kd = kv_cache.dequantize_heads(p, k.shape)
    assert np.array_equal(f32_of(kd.view(-1, 128)), F.round_to_bf16(F.dequant_mixed(want)))
    s_ref = torch.einsum("bthd,bshd->bhts", q.float(), k.float())
    s_q = torch.einsum("bthd,bshd->bhts", kv_cache.rotate_heads(q).float(), kd.float())
    s_rot = torch.einsum("bthd,bshd->bhts", kv_cache.rotate_heads(q).float(), kv_cache.rotate_heads(k).float())
    assert rel_l2(s_rot.cpu().numpy(), s_ref.cpu().numpy()) < 1e-2     # the common rotation leaves the scores alone
    assert rel_l2(s_q.cpu().numpy(), s_ref.cpu().numpy()) < 0.35       # 4-bit keys with x20 outlier channels


def test_decoder_with_packed_nvfp4_key_value_cache():
    """kv_quant: the cache holds packed NVFP4 rows (keys rotated, values plain).  The stored bytes equal the
    oracle's for the same keys / values; logits and generated tokens equal, bit for bit, those of the run that
    stores the dequantised bf16 values instead ("fake": the reference's semantics); both stay close to the run with
    a bf16 cache; eager and graph decode agree."""
    from plaquant_b200 import kv_cache
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
    kv = synth_activation(2 * 5 * 3, 128, seed=31).view(2, 5, 3, 128)
    for had in (True, False):
        rows = kv_cache.pack_head_rows(kv.cuda(), hadamard=had)
        want = F.prepare_activation(f32_of(kv.view(-1, 128)), 0, hadamard=had)
        assert rows.shape == (2, 5, 3, 72) and rows.dtype == torch.uint8
        got = rows.view(-1, 72).cpu().numpy()
        assert np.array_equal(got[:, :64], want["lo_codes"]) and np.array_equal(got[:, 64:], want["lo_sf"])
        back = kv_cache.unpack_head_rows(rows)
        assert np.array_equal(f32_of(back.view(-1, 128)), F.round_to_bf16(F.dequant_mixed(want)))
    assert not kv_cache.unpack_head_rows(torch.zeros(1, 2, 1, 72, dtype=torch.uint8, device="cuda")).any()
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=128,
                      vocab_size=500)
    ids = torch.randint(0, 500, (2, 24), generator=torch.Generator().manual_seed(3)).cuda()
    ref = ResQForwardB200(cfg, "cuda", seed=2).forward(ids)
    fake = ResQForwardB200(cfg, "cuda", seed=2, kv_quant="fake")
    model = ResQForwardB200(cfg, "cuda", seed=2, kv_quant=True)
    got = model.forward(ids)
    assert model.kv[0][0].dtype == torch.uint8 and model.kv[0][0].shape == (2, 24, 1, 72)     # the cache is packed
    assert torch.equal(got, fake.forward(ids))
    assert torch.isfinite(got).all() and rel_l2(got.cpu().numpy(), ref.cpu().numpy()) < 0.3
    gen = model.generate(ids, 4)
    assert torch.equal(gen, model.generate(ids, 4, use_graph=False)) and torch.equal(gen, fake.generate(ids, 4))
    plq.check_device_status()


def test_independent_resq_forward_from_a_weights_dict_matches_the_seeded_decoder(tmp_path):
    """The reference-named forward object: built from {name: bf16 tensor} + a config dict, `.to("cuda")`, logits
    for every position - bit-identical to ResQForwardB200 drawing the same weights from its seed; per-linear
    access by the reference's prefixes; and the packed-weight container: save -> load gives identical logits."""
    from plaquant_b200 import tp, weight_packer
    from plaquant_b200.forward_pass import IndependentResQForward, LlamaConfig, ResQForwardB200, synthetic_weights
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                      vocab_size=1000)
    ids = torch.randint(0, 1000, (3, 24), generator=torch.Generator().manual_seed(0)).cuda()
    seeded = ResQForwardB200(cfg, "cuda", seed=5)
    want_last = seeded.forward(ids)
    weights = {k: v.cpu() for k, v in synthetic_weights(cfg, seed=5).items()}
    config = {"num_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
              "intermediate_size": 512, "rope_theta": cfg.rope_theta, "rms_eps": cfg.rms_eps}
    fwd = IndependentResQForward(weights, config)
    with pytest.raises(RuntimeError):
        fwd.forward(ids)                                    # still on the CPU: there is no CPU path
    fwd = fwd.to("cuda")
    logits = fwd.forward(ids)
    assert logits.shape == (3, 24, 1000) and logits.dtype == torch.float32
    assert torch.equal(logits[:, -1], want_last)
    assert torch.equal(seeded.forward(ids, all_positions=True), logits)
    # per-linear entry point under the reference's prefixes: slices of the fused linears
    x = synth_activation(5, 256, seed=9).cuda()
    q = fwd._quantized_linear(x, "l1.q_proj")
    k = fwd._quantized_linear(x, "l1.k_proj")
    assert q.shape == (5, 256) and k.shape == (5, 128)
    want_q = _oracle_linear(x, weights["l1.q_proj.weight"], fwd.model.k_hi_hidden)
    assert rel_l2(f32_of(q), want_q) <= 1e-3
    # container round trip
    path = weight_packer.save_packed(seeded, str(tmp_path / "model.plq"))
    loaded = weight_packer.load_packed(path, "cuda")
    assert torch.equal(loaded.forward(ids), want_last)
    assert torch.equal(loaded.generate(ids, 4), seeded.generate(ids, 4))
    with pytest.raises(ValueError):
        weight_packer.load_packed(path, "cuda", ctx=tp.TPContext(1, 2, None))   # written for one rank, not for rank 1 of 2
    plq.check_device_status()


def test_generate_keeps_its_decode_graph_between_calls():
    """The second generate() with the same batch, prompt length and step count replays the kept graph for every
    step: same tokens as the first call and as the eager loop, also for a different prompt of that shape; another
    shape builds a new state."""
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=2048, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=128,
                      vocab_size=512)
    g = torch.Generator().manual_seed(21)
    ids_a = torch.randint(0, cfg.vocab_size, (3, 20), generator=g).cuda()
    ids_b = torch.randint(0, cfg.vocab_size, (3, 20), generator=g).cuda()
    m = ResQForwardB200(cfg, "cuda", seed=2)
    eager_a = m.generate(ids_a, 7, use_graph=False)
    eager_b = m.generate(ids_b, 7, use_graph=False)
    first = m.generate(ids_a, 7)
    state = m._decode_states[(3, 20, 7)]
    assert state.graph is not None
    assert torch.equal(first, eager_a)
    assert torch.equal(m.generate(ids_a, 7), eager_a) and m._decode_states[(3, 20, 7)] is state
    assert torch.equal(m.generate(ids_b, 7), eager_b)
    assert torch.equal(m.generate(ids_a, 7), eager_a)
    shorter = m.generate(ids_a[:, :12], 7)
    assert (3, 12, 7) in m._decode_states and (3, 20, 7) not in m._decode_states
    assert torch.equal(shorter, m.generate(ids_a[:, :12], 7, use_graph=False))
    plq.check_device_status()

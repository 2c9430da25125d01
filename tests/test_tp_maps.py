"""Tensor-parallel partition maps and the reduce algebra, on CPU ranks (gloo, world size 2),
with the CPU oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import formats as F
from plaquant_b200 import tp
from tests._util import bits_of, synth_activation, synth_gamma, synth_weight


def test_outlier_count_respects_kernel_granularity():
    for k, want in ((4096, 128), (14336, 448), (8192, 256), (28672, 896), (1024, 64), (3584, 128), (128, 64)):
        k_hi = tp.outlier_count(k)
        assert k_hi == want, (k, k_hi)
        assert k_hi % 32 == 0 and (k - k_hi) % 64 == 0 and k_hi >= k / 32
    # the 70B shapes at every tensor-parallel degree
    for size in (1, 2, 4, 8):
        for k in (8192, 28672):
            for r in range(size):
                s = tp.row_parallel_cols(k, r, size)
                assert (s.stop - s.start) % 128 == 0
                tp.outlier_count(s.stop - s.start)
        for n in (10240, 57344):
            assert sum(tp.column_parallel_rows(n, r, size).stop - tp.column_parallel_rows(n, r, size).start
                       for r in range(size)) == n
    with pytest.raises(ValueError):
        tp.row_parallel_cols(4096 + 128, 0, 8)


def _f32(t):
    return F.bf16_bits_to_f32(bits_of(t))


def _partial(x, w, ks: slice):
    xs, ws = _f32(x)[:, ks], _f32(w)[:, ks]
    k_hi = tp.outlier_count(ks.stop - ks.start)
    return F.linear(F.prepare_activation(xs, k_hi, hadamard=True), F.prepare_activation(ws, k_hi, hadamard=True))


def _worker(rank, size, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        ctx = tp.TPContext.from_env()
        x, w = synth_activation(4, 512, seed=5), synth_weight(48, 512, seed=6)
        # row-parallel: own K shard, partial product, one all-reduce
        y = torch.from_numpy(_partial(x, w, tp.row_parallel_cols(512, rank, size)))
        ctx.all_reduce(y)
        # column-parallel: own N shard, no exchange (gathered here only to check it)
        rows = tp.column_parallel_rows(48, rank, size)
        k_hi = tp.outlier_count(512)
        yc = torch.from_numpy(F.linear(F.prepare_activation(_f32(x), k_hi, hadamard=True),
                                       F.prepare_activation(_f32(w)[rows], k_hi, hadamard=True)))
        parts = [torch.empty_like(yc) for _ in range(size)]
        dist.all_gather(parts, yc)
        if rank == 0:
            out.put((y.numpy(), torch.cat(parts, 1).numpy()))
    finally:
        dist.destroy_process_group()


def test_row_and_column_parallel_on_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    y_row, y_col = out.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    x, w = synth_activation(4, 512, seed=5), synth_weight(48, 512, seed=6)
    want_row = _partial(x, w, slice(0, 256)) + _partial(x, w, slice(256, 512))
    assert np.array_equal(y_row, want_row)                      # same partials, same sum
    k_hi = tp.outlier_count(512)
    want_col = F.linear(F.prepare_activation(_f32(x), k_hi, hadamard=True), F.prepare_activation(_f32(w), k_hi, hadamard=True))
    assert np.array_equal(y_col, want_col)                      # N shards are independent rows of W
    # the sharded product is a different (rank-local) quantisation of the same linear map
    full = _f32(x) @ _f32(w).T
    assert np.linalg.norm(want_row - full) / np.linalg.norm(full) < 0.2


def test_rank_that_fails_before_the_collective_is_reported():
    """Host-side failure injection: a rank that raises never joins; the other must not hang forever."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_failing_pair, args=(q,))
    p.start()
    p.join(90)
    assert p.exitcode == 0
    assert q.get(timeout=5) == "timeout-detected"


def _failing_pair(q):
    import datetime
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # world of 2 in which rank 1 never shows up: initialisation must time out, not hang
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=5))
        q.put("unexpected-success")
    except Exception:
        q.put("timeout-detected")


def test_shards_of_a_weights_dict_partition_the_model():
    """`ResQForwardB200._shard_of` (what every rank cuts out of a dict of full weights under the reference's
    names): the column-parallel shards tile the output rows, the row-parallel shards tile the input columns, and
    the row-parallel partial products add up to the full product.  CPU tensors, two ranks."""
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_layers=1, num_heads=4, num_kv_heads=2, head_dim=64,
                      vocab_size=100)
    g = torch.Generator().manual_seed(3)
    full = {"l0.ln1": torch.rand(256, generator=g), "l0.ln2": torch.rand(256, generator=g)}
    for name, (n, k) in {"q_proj": (256, 256), "k_proj": (128, 256), "v_proj": (128, 256), "o_proj": (256, 256),
                         "mlp.gate_proj": (512, 256), "mlp.up_proj": (512, 256), "mlp.down_proj": (256, 512)}.items():
        full[f"l0.{name}.weight"] = torch.randn(n, k, generator=g)
    shards = []
    for rank in range(2):
        m = ResQForwardB200.__new__(ResQForwardB200)
        m.cfg, m.device, m.ctx = cfg, torch.device("cpu"), tp.TPContext(rank, 2, None)
        shards.append(m._shard_of(full, 0))
    f = lambda t: t.float()
    q = torch.cat([f(s["qkv"][:128]) for s in shards]); k = torch.cat([f(s["qkv"][128:192]) for s in shards])
    v = torch.cat([f(s["qkv"][192:]) for s in shards])
    bf = lambda t: t.to(torch.bfloat16).float()
    assert torch.equal(q, bf(full["l0.q_proj.weight"])) and torch.equal(k, bf(full["l0.k_proj.weight"]))
    assert torch.equal(v, bf(full["l0.v_proj.weight"]))
    assert torch.equal(torch.cat([f(s["gate_up"][:256]) for s in shards]), bf(full["l0.mlp.gate_proj.weight"]))
    assert torch.equal(torch.cat([f(s["gate_up"][256:]) for s in shards]), bf(full["l0.mlp.up_proj.weight"]))
    assert torch.equal(torch.cat([f(s["o"]) for s in shards], 1), bf(full["l0.o_proj.weight"]))
    assert torch.equal(torch.cat([f(s["down"]) for s in shards], 1), bf(full["l0.mlp.down_proj.weight"]))
    x = torch.randn(5, 512, generator=g)
    part = sum(x[:, tp.row_parallel_cols(512, r, 2)] @ f(shards[r]["down"]).T for r in range(2))
    assert torch.allclose(part, x @ bf(full["l0.mlp.down_proj.weight"]).T, atol=1e-4)


def _scatter_worker(rank, size, port, out):
    """The scattered reduction's data flow with gloo standing for the peer loads and stores: every rank sums ITS
    rows of the partial outputs (float32, rank order, one rounding), adds its slice of the residual stream,
    normalises / rotates / quantises them with the oracle, and the packed rows are all-gathered."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        from plaquant_b200.forward_pass import gather_last_positions
        batch, seq, k, k_hi = 3, 4, 256, 32
        total = batch * seq
        per = total // size
        mine = slice(rank * per, (rank + 1) * per)
        parts = [synth_activation(total, k, seed=70 + r) for r in range(size)]      # every rank's partial output
        res = synth_activation(total, k, seed=80)
        gamma = synth_gamma(k, 81)
        got = [torch.empty_like(parts[rank]) for _ in range(size)]
        dist.all_gather(got, parts[rank])                                           # stands for the peer loads
        acc = np.zeros((per, k), np.float32)
        for g_ in got:
            acc = acc + _f32(g_)[mine]
        h = F.add_bf16(_f32(res)[mine], F.round_to_bf16(acc))
        p = F.prepare_activation(h, k_hi, gamma=_f32(gamma), eps=1e-6, hadamard=True)
        gathered = {}
        for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"):                      # stands for the peer stores
            t = torch.from_numpy(np.ascontiguousarray(p[key]))
            parts_k = [torch.empty_like(t) for _ in range(size)]
            dist.all_gather(parts_k, t)
            gathered[key] = torch.cat(parts_k, 0).numpy()
        last = gather_last_positions(torch.from_numpy(h).to(torch.bfloat16), batch, seq, rank, size)
        hs = [torch.empty(per, k) for _ in range(size)]
        dist.all_gather(hs, torch.from_numpy(h))
        if rank == size - 1:
            out.put((gathered, torch.cat(hs, 0).numpy(), last.float().numpy()))
    finally:
        dist.destroy_process_group()


def test_scattered_reduction_on_two_gloo_ranks_equals_the_all_reduce_path():
    """Reduce-scatter + add + norm + quantise per row slice + all-gather of the packed rows gives the bytes of
    all-reduce + add + norm + quantise of all rows; the last-position gather returns the right rows."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_scatter_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    gathered, h_all, last = out.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    batch, seq, k, k_hi = 3, 4, 256, 32
    parts = [synth_activation(batch * seq, k, seed=70 + r) for r in range(2)]
    acc = _f32(parts[0]) + _f32(parts[1])
    want_h = F.add_bf16(_f32(synth_activation(batch * seq, k, seed=80)), F.round_to_bf16(acc))
    want = F.prepare_activation(want_h, k_hi, gamma=_f32(synth_gamma(k, 81)), eps=1e-6, hadamard=True)
    assert np.array_equal(h_all, want_h)
    for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"):
        assert np.array_equal(gathered[key], want[key]), key
    assert np.array_equal(last, want_h.reshape(batch, seq, k)[:, -1])

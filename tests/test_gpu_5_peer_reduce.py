"""Fused all-reduce + residual add + RMSNorm-quant over peer memory (two or more GPUs of one node): every rank's
result must equal the CPU restatement bit for bit, call after call, eager and replayed from a CUDA graph."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
plq = pytest.importorskip("plaquant_b200")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, k, k_hi, calls, q):
    try:
        import torch.distributed as dist
        from oracle import formats as F
        from plaquant_b200 import ops, tp
        from tests._util import f32_of, packed_to_numpy
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        peer = tp.PeerReduce(16, k, dev)
        g = torch.Generator().manual_seed(7)                   # same stream on every rank: all partials known to all
        gamma = (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16)
        ok = True
        for c in range(calls):
            parts = [torch.randn(rows, k, generator=g).to(torch.bfloat16) for _ in range(world)]
            res = torch.randn(rows, k, generator=g).to(torch.bfloat16)
            peer.buffer(rows).copy_(parts[rank].to(dev))       # stands for the row-parallel linear's output
            h, p = ops.allreduce_add_rmsnorm_pack(peer, rows, res.to(dev), gamma.to(dev), 1e-6, k_hi)
            plq.check_device_status(dev)
            acc = np.zeros((rows, k), dtype=np.float32)
            for part in parts:                                  # float32, rank order
                acc = acc + f32_of(part)
            want_h = F.add_bf16(f32_of(res), F.round_to_bf16(acc))
            want = F.prepare_activation(want_h, k_hi, gamma=f32_of(gamma), eps=1e-6, hadamard=True)
            got = packed_to_numpy(p)
            ok = ok and np.array_equal(f32_of(h), want_h)
            ok = ok and all(np.array_equal(got[key], want[key]) for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, bool(ok), ""))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, False, repr(exc)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("rows,k,k_hi", [(16, 8192, 256), (3, 1024, 64)])
def test_fused_allreduce_add_rmsnorm_pack_bit_exact(rows, k, k_hi):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, rows, k, k_hi, 5, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in results), results


def test_a_rank_that_never_announces_itself_gives_a_timeout_status_not_a_hang():
    """Failure detection without faulting a GPU: rank 1 of a two-rank job is emulated by buffers on this GPU whose
    flag nothing ever sets.  The bounded wait (about two seconds of SM clock) runs out, the kernel stores
    PLQ_DEV_TIMEOUT and finishes, the front end raises, and the context stays usable."""
    from plaquant_b200 import _lib, ops
    from tests._util import synth_activation, synth_gamma
    dev = torch.device("cuda", 0)
    rows, k, k_hi = 4, 1024, 64
    x = torch.zeros(2, rows, k, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    peer_x = torch.tensor([x[0].data_ptr(), x[1].data_ptr()], dtype=torch.int64, device=dev)
    peer_flags = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64, device=dev)
    res = synth_activation(rows, k, seed=1).cuda()
    gamma = synth_gamma(k, 2).cuda()
    h = torch.empty_like(res)
    p = ops.alloc_packed(rows, k, k_hi, "tiled", dev)
    st = _lib.lib().plq_allreduce_add_rmsnorm_pack(
        peer_x.data_ptr(), peer_flags.data_ptr(), flags.data_ptr(), sync.data_ptr(), 2, 0, 0, res.data_ptr(), h.data_ptr(),
        gamma.data_ptr(), 1e-6, rows, k, k_hi, 1, p.lo_codes.data_ptr(), p.lo_sf.data_ptr(), p.hi_codes.data_ptr(),
        p.hi_sf.data_ptr(), p.sf_layout, ops.status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    assert st == 0
    with pytest.raises(plq.PlqError) as e:
        plq.check_device_status(dev)
    assert e.value.status == 1
    assert int(sync[0].item()) == 1 and int(flags[0].item()) == 1 and int(flags[1].item()) == 0
    q = plq.pack(res, k_hi, hadamard=True)                       # the context is intact
    plq.check_device_status(dev)
    assert q.rows == rows


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sum_over_emulated_ranks_on_one_gpu(world):
    """The arithmetic and the handshake for `world` ranks with one GPU: the other ranks' buffers live on this GPU
    and their announcements are written from the host before each call (call numbers 1, 2, 3)."""
    from oracle import formats as F
    from plaquant_b200 import _lib, ops
    from tests._util import f32_of, packed_to_numpy, synth_activation, synth_gamma
    dev = torch.device("cuda", 0)
    rows, k, k_hi = 5, 2048, 64
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    peer_flags = torch.tensor([flags.data_ptr()] * world, dtype=torch.int64, device=dev)
    gamma = synth_gamma(k, 2)
    gamma_d = gamma.cuda()
    for call in (1, 2, 3):
        parts = [synth_activation(rows, k, seed=100 * call + r).cuda() for r in range(world)]
        res = synth_activation(rows, k, seed=100 * call + 50)
        res_d = res.cuda()                                       # named: a temporary would be freed before the kernel runs
        peer_x = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=dev)
        flags[1:world] = call                                   # "ranks 1.. have announced this call"
        h = torch.empty(rows, k, dtype=torch.bfloat16, device=dev)
        p = ops.alloc_packed(rows, k, k_hi, "rowmajor", dev)
        st = _lib.lib().plq_allreduce_add_rmsnorm_pack(
            peer_x.data_ptr(), peer_flags.data_ptr(), flags.data_ptr(), sync.data_ptr(), world, 0, -1, res_d.data_ptr(),
            h.data_ptr(), gamma_d.data_ptr(), 1e-6, rows, k, k_hi, 1, p.lo_codes.data_ptr(), p.lo_sf.data_ptr(),
            p.hi_codes.data_ptr(), p.hi_sf.data_ptr(), p.sf_layout, ops.status_word(dev).data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream)
        assert st == 0
        plq.check_device_status(dev)
        assert int(sync[0].item()) == call and int(flags[0].item()) == call
        acc = np.zeros((rows, k), dtype=np.float32)
        for part in parts:
            acc = acc + f32_of(part)
        want_h = F.add_bf16(f32_of(res), F.round_to_bf16(acc))
        assert np.array_equal(f32_of(h), want_h)
        want = F.prepare_activation(want_h, k_hi, gamma=f32_of(gamma), eps=1e-6, hadamard=True)
        got = packed_to_numpy(p)
        for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"):
            assert np.array_equal(got[key], want[key]), key


def test_replayed_graph_alternates_buffer_sets_and_an_odd_call_count_is_reported():
    """A decode step replayed from a CUDA graph freezes which buffer set each call site reads.  With an even number
    of fused reductions per graph the sets keep alternating across replays and every replay is bit-exact; a graph
    with an odd number reuses the set of the call just before it on its second replay, which the kernel reports as
    PLQ_DEV_PROTOCOL.  Two ranks emulated on one GPU: rank 1's buffers are local and its announcements are written
    from the host before each replay."""
    from oracle import formats as F
    from plaquant_b200 import _lib, ops
    from tests._util import f32_of, packed_to_numpy, synth_activation, synth_gamma
    dev = torch.device("cuda", 0)
    rows, k, k_hi, world = 4, 1024, 64, 2
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    peer_flags = torch.tensor([flags.data_ptr()] * world, dtype=torch.int64, device=dev)
    bufs = torch.zeros(2, world, rows, k, dtype=torch.bfloat16, device=dev)          # [set][rank]
    peer_x = [torch.tensor([bufs[s, r].data_ptr() for r in range(world)], dtype=torch.int64, device=dev) for s in range(2)]
    gamma = synth_gamma(k, 2)
    gamma_d = gamma.cuda()
    res = [synth_activation(rows, k, seed=900 + s) for s in range(2)]
    res_d = [r.cuda() for r in res]
    h = [torch.empty(rows, k, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    p = [ops.alloc_packed(rows, k, k_hi, "rowmajor", dev) for _ in range(2)]
    status = ops.status_word(dev)
    status.zero_()

    def call(s, stream):
        st = _lib.lib().plq_allreduce_add_rmsnorm_pack(
            peer_x[s].data_ptr(), peer_flags.data_ptr(), flags.data_ptr(), sync.data_ptr(), world, 0, s,
            res_d[s].data_ptr(), h[s].data_ptr(), gamma_d.data_ptr(), 1e-6, rows, k, k_hi, 1, p[s].lo_codes.data_ptr(),
            p[s].lo_sf.data_ptr(), p[s].hi_codes.data_ptr(), p[s].hi_sf.data_ptr(), p[s].sf_layout, status.data_ptr(),
            stream.cuda_stream)
        assert st == 0

    def check(s, parts):
        acc = np.zeros((rows, k), dtype=np.float32)
        for part in parts:
            acc = acc + f32_of(part)
        want_h = F.add_bf16(f32_of(res[s]), F.round_to_bf16(acc))
        assert np.array_equal(f32_of(h[s]), want_h)
        want = F.prepare_activation(want_h, k_hi, gamma=f32_of(gamma), eps=1e-6, hadamard=True)
        got = packed_to_numpy(p[s])
        for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"):
            assert np.array_equal(got[key], want[key]), key

    side = torch.cuda.Stream(device=dev)
    even = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(even, stream=side):
            call(0, side)
            call(1, side)
    torch.cuda.synchronize()
    for replay in range(1, 4):
        parts = [[synth_activation(rows, k, seed=1000 * replay + 10 * s + r) for r in range(world)] for s in range(2)]
        for s in range(2):
            for r in range(world):
                bufs[s, r].copy_(parts[s][r])
        flags[1] = 2 * replay                                  # "rank 1 has announced both calls of this replay"
        torch.cuda.synchronize()
        even.replay()
        plq.check_device_status(dev)
        assert int(sync[0].item()) == 2 * replay
        check(0, parts[0])
        check(1, parts[1])

    odd = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(odd, stream=side):
            call(0, side)                                       # call 7 reads set 0: right the first time
    torch.cuda.synchronize()
    flags[1] = 8
    odd.replay()
    plq.check_device_status(dev)
    odd.replay()                                                # call 8 must read set 1 but the graph names set 0
    with pytest.raises(plq.PlqError) as e:
        plq.check_device_status(dev)
    assert e.value.status == 2


def _oracle_scatter(parts, res_full, gamma, k_hi):
    """h = res + bf16(sum of parts in rank order), then RMSNorm + rotation + pack, for all rows."""
    from oracle import formats as F
    from tests._util import f32_of
    acc = np.zeros(tuple(parts[0].shape), dtype=np.float32)
    for part in parts:
        acc = acc + f32_of(part)
    want_h = F.add_bf16(f32_of(res_full), F.round_to_bf16(acc))
    return want_h, F.prepare_activation(want_h, k_hi, gamma=f32_of(gamma), eps=1e-6, hadamard=True)


@pytest.mark.parametrize("world,total,k,k_hi", [(2, 6, 1024, 64), (4, 264, 4096, 128), (8, 16, 2048, 64)])
def test_scattered_form_with_emulated_ranks_on_one_gpu(world, total, k, k_hi):
    """Reduce-scatter + add + RMSNorm-quant + all-gather of the packed rows, `world` ranks emulated on one GPU one
    after the other: every rank has its own flag array and its own packed output buffers on this GPU, the other
    ranks' announcements (start and completion words) are written from the host before a rank runs.  After all
    ranks have run, EVERY rank's packed buffer must hold all rows, bit-exact against the CPU restatement, and the
    residual slices must tile the full residual stream."""
    from oracle import formats as F
    from plaquant_b200 import _lib, ops
    from tests._util import f32_of, packed_to_numpy, synth_activation, synth_gamma
    dev = torch.device("cuda", 0)
    per = total // world
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
    sync = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(world)]
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    outs = [ops.alloc_packed(total, k, k_hi, "tiled", dev) for _ in range(world)]       # codes + the tiled scales
    stage = [ops.alloc_packed(total, k, k_hi, "rowmajor", dev) for _ in range(world)]   # gathered row-major scales
    tbl = [0] * 32
    for r in range(world):
        for i, t in enumerate((outs[r].lo_codes, stage[r].lo_sf, outs[r].hi_codes, stage[r].hi_sf)):
            tbl[8 * i + r] = t.data_ptr()
    tbl_d = torch.tensor(tbl, dtype=torch.int64, device=dev)
    gamma = synth_gamma(k, 3)
    gamma_d = gamma.cuda()
    for call in (1, 2):
        parts = [synth_activation(total, k, seed=50 * call + r) for r in range(world)]
        parts_d = [p.cuda() for p in parts]
        res = synth_activation(total, k, seed=50 * call + 40)
        res_d = res.cuda()
        peer_x = torch.tensor([p.data_ptr() for p in parts_d], dtype=torch.int64, device=dev)
        h = torch.zeros(total, k, dtype=torch.bfloat16, device=dev)
        for r in range(world):
            for j in range(world):
                if j != r:                      # "rank j has announced this call and its completion" (kept if already ahead)
                    flags[r][j] = call
                    flags[r][32 + j] = call
            st = _lib.lib().plq_reduce_scatter_add_rmsnorm_pack(
                peer_x.data_ptr(), peer_flags.data_ptr(), flags[r].data_ptr(), sync[r].data_ptr(), world, r, -1,
                tbl_d.data_ptr(), r * per, total, res_d[r * per:].data_ptr(), h[r * per:].data_ptr(), gamma_d.data_ptr(),
                1e-6, per, k, k_hi, 1, outs[r].lo_codes.data_ptr(), stage[r].lo_sf.data_ptr(), outs[r].hi_codes.data_ptr(),
                stage[r].hi_sf.data_ptr(), outs[r].lo_sf.data_ptr(), outs[r].hi_sf.data_ptr(),
                ops.status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
            assert st == 0
            plq.check_device_status(dev)
            assert int(sync[r][0].item()) == call
        for r in range(world):                  # every rank told every other one, start and completion
            f = flags[r].cpu().numpy()
            assert (f[:world] == call).all() and (f[32:32 + world] == call).all()
        want_h, want = _oracle_scatter(parts, res, gamma, k_hi)
        assert np.array_equal(f32_of(h), want_h)
        # rank r re-tiled the scales at the end of ITS call, when only ranks <= r had run: the last rank's tiled
        # copy is whole, and so is every rank's gathered row-major form; the codes are whole everywhere
        for r, o in enumerate(outs):
            got = packed_to_numpy(o)
            for key in ("lo_codes", "hi_codes"):
                assert np.array_equal(got[key], want[key]), key
            assert np.array_equal(stage[r].lo_sf.cpu().numpy(), want["lo_sf"])
            assert np.array_equal(stage[r].hi_sf.cpu().numpy(), want["hi_sf"])
        # the tiled copy byte for byte, padding (rows and scales beyond the matrix) included
        assert np.array_equal(outs[world - 1].lo_sf.cpu().numpy(), F.tile_sf(want["lo_sf"]))
        assert np.array_equal(outs[world - 1].hi_sf.cpu().numpy(), F.tile_sf(want["hi_sf"]))


def test_scattered_form_times_out_when_a_peer_never_completes():
    """Rank 1 announces the call but never its completion: the closing wait is bounded, the kernel stores
    PLQ_DEV_TIMEOUT and ends, and the context stays usable."""
    from plaquant_b200 import _lib, ops
    from tests._util import synth_activation, synth_gamma
    dev = torch.device("cuda", 0)
    total, k, k_hi, world = 4, 1024, 64, 2
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    other = torch.zeros(64, dtype=torch.int32, device=dev)
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    flags[1] = 1                                   # started, but flags[33] stays 0
    peer_flags = torch.tensor([flags.data_ptr(), other.data_ptr()], dtype=torch.int64, device=dev)
    x = synth_activation(total, k, seed=5).cuda()
    peer_x = torch.tensor([x.data_ptr()] * 2, dtype=torch.int64, device=dev)
    outs = [ops.alloc_packed(total, k, k_hi, "rowmajor", dev) for _ in range(2)]
    tbl = [0] * 32
    for r, o in enumerate(outs):
        for i, t in enumerate((o.lo_codes, o.lo_sf, o.hi_codes, o.hi_sf)):
            tbl[8 * i + r] = t.data_ptr()
    tbl_d = torch.tensor(tbl, dtype=torch.int64, device=dev)
    gamma = synth_gamma(k, 2).cuda()
    h = torch.empty(2, k, dtype=torch.bfloat16, device=dev)
    st = _lib.lib().plq_reduce_scatter_add_rmsnorm_pack(
        peer_x.data_ptr(), peer_flags.data_ptr(), flags.data_ptr(), sync.data_ptr(), world, 0, 0, tbl_d.data_ptr(), 0,
        total, x.data_ptr(), h.data_ptr(), gamma.data_ptr(), 1e-6, 2, k, k_hi, 1, outs[0].lo_codes.data_ptr(),
        outs[0].lo_sf.data_ptr(), outs[0].hi_codes.data_ptr(), outs[0].hi_sf.data_ptr(), None, None,
        ops.status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    assert st == 0
    with pytest.raises(plq.PlqError) as e:
        plq.check_device_status(dev)
    assert e.value.status == 1
    assert int(sync[0].item()) == 1 and int(other[32].item()) == 1
    plq.pack(x, k_hi, hadamard=True)
    plq.check_device_status(dev)


def _scatter_worker(rank, world, port, total, k, k_hi, calls, q):
    try:
        import torch.distributed as dist
        from plaquant_b200 import ops, tp
        from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
        from tests._util import f32_of, packed_to_numpy
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        sr = tp.ScatterReduce(total, k, k_hi, dev)
        per = total // world
        g = torch.Generator().manual_seed(11)
        gamma = (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16)
        ok = True
        for c in range(calls):
            parts = [torch.randn(total, k, generator=g).to(torch.bfloat16) for _ in range(world)]
            res = torch.randn(total, k, generator=g).to(torch.bfloat16)
            sr.buffer(total).copy_(parts[rank].to(dev))
            h, p = ops.reduce_scatter_add_rmsnorm_pack(sr, total, res[rank * per:(rank + 1) * per].to(dev), gamma.to(dev), 1e-6)
            plq.check_device_status(dev)
            want_h, want = _oracle_scatter(parts, res, gamma, k_hi)
            got = packed_to_numpy(p)
            ok = ok and np.array_equal(f32_of(h), want_h[rank * per:(rank + 1) * per])
            ok = ok and all(np.array_equal(got[key], want[key]) for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"))
        # the decoder: prefill with the row-sharded residual stream gives, bit for bit, the logits of the path whose
        # all-reduces run in the all-reduce form of the same kernel (float32 sum in rank order, one rounding; NCCL
        # rounds its partial sums to bf16 between the ranks, which differs from three ranks on)
        cfg = LlamaConfig(hidden_size=1024, intermediate_size=1024 * world, num_layers=2, num_heads=8 * world,
                          num_kv_heads=world, head_dim=128, vocab_size=512)
        ctx = tp.TPContext(rank, world, None)
        ids = torch.randint(0, cfg.vocab_size, (2, 16 * world), generator=torch.Generator().manual_seed(3)).to(dev)
        plain = ResQForwardB200(cfg, dev, ctx, seed=5, fused_reduce_rows=ids.numel())
        a = plain.forward(ids)
        a_all = plain.forward(ids, all_positions=True)
        sharded = ResQForwardB200(cfg, dev, ctx, seed=5, scatter_prefill_rows=ids.numel())
        b = sharded.forward(ids)
        b_all = sharded.forward(ids, all_positions=True)
        plq.check_device_status(dev)
        checks = {"calls": sharded.scatter.calls == 4 * len(sharded.layers), "last": torch.equal(a, b),
                  "all": torch.equal(a_all, b_all),
                  "kv": all(torch.equal(x, y) for kv0, kv1 in zip(plain.kv, sharded.kv) for x, y in zip(kv0, kv1))}
        ok_model = all(checks.values())
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, bool(ok and ok_model), "" if ok_model else f"model mismatch: {checks}"))
    except Exception as exc:  # noqa: BLE001
        import traceback
        q.put((rank, False, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("total,k,k_hi", [(256, 4096, 128), (8, 1024, 64)])
def test_scattered_form_across_gpus_bit_exact(total, k, k_hi):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_scatter_worker, args=(r, world, port, total, k, k_hi, 4, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in results), results

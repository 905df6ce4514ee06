"""Multi-process path on CPU: two gloo ranks shard whole sequences, run the encoder layer on
their own shard (here with the CPU oracle standing in for the GPU kernels: the sharding logic
under test is host code), and the gathered result must equal the unsharded evaluation bit for
bit.  Also covers the timing protocol (max over ranks, whole-job throughput)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def test_shard_range_covers_every_unit_once():
    et = entry.load_package()
    for n in (0, 1, 5, 16, 17, 1000):
        for world in (1, 2, 3, 8):
            got = []
            for r in range(world):
                a, b = et.sharding.shard_range(n, world, r)
                assert 0 <= a <= b <= n
                got += list(range(a, b))
            assert got == list(range(n))
            sizes = [np.diff(et.sharding.shard_range(n, world, r))[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        et.sharding.shard_range(4, 2, 2)
    assert et.sharding.shard_rows(5, 128, 2, 1) == (3 * 128, 5 * 128)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n_seq: int, seq: int, out_q):
    try:
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        et = entry.load_package()
        orc = entry.load_oracle()
        orc.build()
        hidden, nhead, ff = 64, 4, 128
        w = et.synth.encoder_layer_weights(11, 0, hidden, ff, std=0.05, bias_std=0.02, ln_noise=0.1)
        x = et.synth.normal(11, 5, (n_seq * seq, hidden), 1.0)
        vl = np.array([(7 * i) % seq + 1 for i in range(n_seq)], dtype=np.int32)
        job = et.sharding.Job(rank=rank, world=world, device=torch.device("cpu"))
        a, b = et.sharding.shard_range(n_seq, world, rank)
        ra, rb = et.sharding.shard_rows(n_seq, seq, world, rank)
        local = orc.encoder_layer(x[ra:rb], w, b - a, seq, nhead, et.ACT_GELU, 2, None, vl[a:b]) \
            if b > a else np.zeros((0, hidden), np.float32)
        full = job.gather_rows(torch.from_numpy(np.ascontiguousarray(local)), n_seq, seq).numpy()
        job.barrier()
        slow = job.max_over_ranks(1.0 + rank)          # rank r "took" 1 + r seconds
        thr = job.throughput(b - a, 1.0 + rank)
        if rank == 0:
            ref = orc.encoder_layer(x, w, n_seq, seq, nhead, et.ACT_GELU, 2, None, vl)
            out_q.put(("ok", bool(np.array_equal(full, ref)), slow, thr))
        dist.destroy_process_group()
    except Exception as e:  # surfaced by the parent
        out_q.put(("error", repr(e), 0.0, 0.0))
        raise


@pytest.mark.parametrize("n_seq", [4, 5])
def test_two_gloo_ranks_shard_sequences_exactly(n_seq):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_seq, 32, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a gloo rank did not finish")
        assert p.exitcode == 0
    kind, same, slow, thr = q.get(timeout=10)
    assert kind == "ok", same
    assert same, "sharded and unsharded results differ"
    assert slow == 2.0
    assert thr == n_seq / 2.0


def _hp_worker(rank: int, world: int, port: int, out_q):
    """Head-parallel attention block with the oracle standing in for the kernels: the partial
    sums of the ranks, all-reduced, must equal the unsharded block."""
    try:
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        et = entry.load_package()
        orc = entry.load_oracle()
        orc.build()
        hidden, nhead, ff, seq = 96, 6, 128, 80
        kdim, vdim = 6 * 16, 6 * 32          # dh_qk 16, dh_v 32: Q/K narrower than V
        w = et.synth.encoder_layer_weights(5, 0, hidden, ff, kdim=kdim, vdim=vdim, std=0.1,
                                           bias_std=0.05)
        x = et.synth.normal(5, 9, (seq, hidden), 1.0).astype(np.float32)
        sl = et.sharding.head_shard_weights(w, nhead, world, rank)
        nh, dqk, dv = sl["nhead_local"], sl["dh_qk"], sl["dh_v"]
        qkv = orc.linear_dense(x, sl["wqkv"], sl["bqkv"], 0)
        z = orc.attention(qkv[:, :nh * dqk], qkv[:, nh * dqk:2 * nh * dqk], qkv[:, 2 * nh * dqk:],
                          1, seq, nh, dqk, dv, 1)
        part = torch.from_numpy(orc.linear_dense(z, sl["wo"], sl["bo"], 0))
        dist.all_reduce(part)
        if rank == 0:
            fq = orc.linear_dense(x, w["wqkv"], w["bqkv"], 0)
            fz = orc.attention(fq[:, :kdim], fq[:, kdim:2 * kdim], fq[:, 2 * kdim:], 1, seq, nhead,
                               kdim // nhead, vdim // nhead, 1)
            full = orc.linear_dense(fz, w["wo"], w["bo"], 0)
            err = float(np.abs(part.numpy() - full).max())
            out_q.put(("ok", err))
        dist.destroy_process_group()
    except Exception as e:
        out_q.put(("error", repr(e)))
        raise


def test_head_shards_cover_every_head_and_bias_once():
    et = entry.load_package()
    w = et.synth.encoder_layer_weights(5, 0, 64, 128, kdim=48, vdim=64)
    for world in (1, 2, 3, 4, 8):
        rows, cols, bias = [], [], np.zeros(64, np.float32)
        for r in range(world):
            sl = et.sharding.head_shard_weights(w, 4, world, r)
            assert sl["wqkv"].shape[0] == sl["nhead_local"] * (2 * 12 + 16)
            rows.append(sl["wqkv"].shape[0])
            cols.append(sl["wo"].shape[1])
            bias += sl["bo"].astype(np.float32)
        assert sum(rows) == w["wqkv"].shape[0] and sum(cols) == w["wo"].shape[1]
        assert np.array_equal(bias, w["bo"].astype(np.float32))


def test_two_gloo_ranks_head_parallel_attention_block():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_hp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a gloo rank did not finish")
        assert p.exitcode == 0
    kind, err = q.get(timeout=10)
    assert kind == "ok", err
    assert err < 1e-4, f"head-parallel partial sums differ from the full block by {err}"


def test_work_units_cover_every_head_and_query_block_once():
    """12 heads on 8 ranks: 24 (head, query half) units, 3 per rank, every (head, query block)
    pair owned by exactly one rank and every rank with the same amount of attention work."""
    et = entry.load_package()
    for nhead, world, seq in ((12, 8, 4096), (12, 2, 1024), (16, 8, 4096), (12, 3, 384), (4, 8, 512)):
        qsplit, per_rank, bpu = et.sharding.head_parallel_plan(nhead, world, seq)
        nblocks = -(-seq // 128)
        owner = np.full((nhead, nblocks), -1)
        for r in range(world):
            units = et.sharding.units_of_rank(nhead, world, r, seq)
            assert len(units) == per_rank
            for h, first in units:
                assert (owner[h, first:first + bpu] == -1).all()
                owner[h, first:first + bpu] = r
        assert (owner >= 0).all()
    assert et.sharding.head_parallel_plan(12, 8, 4096) == (2, 3, 16)
    with pytest.raises(ValueError):
        et.sharding.head_parallel_plan(12, 8, 128)  # one query block cannot be halved


def _hp_units_worker(rank: int, world: int, port: int, out_q):
    """Work-unit form on `world` gloo ranks with the oracle standing in for the kernels: each
    rank attends over its (head, query range) units only; the all-reduced partial sums must
    equal the unsharded attention block."""
    try:
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        et = entry.load_package()
        orc = entry.load_oracle()
        orc.build()
        orc.set_num_threads(1)
        hidden, nhead, ff, seq = 96, 12, 128, 256   # 2 query blocks: 24 half-head units on 8 ranks
        w = et.synth.encoder_layer_weights(5, 0, hidden, ff, std=0.1, bias_std=0.05)
        x = et.synth.normal(5, 9, (seq, hidden), 1.0).astype(np.float32)
        _, _, bpu = et.sharding.head_parallel_plan(nhead, world, seq)
        units = et.sharding.units_of_rank(nhead, world, rank, seq)
        heads = sorted({h for h, _ in units})
        sl = et.sharding.head_rows(w, nhead, heads)
        nh, dqk, dv = sl["nhead_local"], sl["dh_qk"], sl["dh_v"]
        qkv = orc.linear_dense(x, sl["wqkv"], sl["bqkv"], 0)
        zfull = orc.attention(qkv[:, :nh * dqk], qkv[:, nh * dqk:2 * nh * dqk], qkv[:, 2 * nh * dqk:],
                              1, seq, nh, dqk, dv, 0)
        z = np.zeros_like(zfull)
        for h, first in units:  # query rows are independent: keep the unit's rows of its head
            lh = heads.index(h)
            r0, r1 = first * 128, min(seq, (first + bpu) * 128)
            z[r0:r1, lh * dv:(lh + 1) * dv] = zfull[r0:r1, lh * dv:(lh + 1) * dv]
        part = torch.from_numpy(orc.linear_dense(z, sl["wo"], w["bo"] if rank == 0 else None, 0))
        dist.all_reduce(part)
        if rank == 0:
            fq = orc.linear_dense(x, w["wqkv"], w["bqkv"], 0)
            fz = orc.attention(fq[:, :hidden], fq[:, hidden:2 * hidden], fq[:, 2 * hidden:], 1, seq,
                               nhead, hidden // nhead, hidden // nhead, 0)
            full = orc.linear_dense(fz, w["wo"], w["bo"], 0)
            out_q.put(("ok", float(np.abs(part.numpy() - full).max())))
        dist.destroy_process_group()
    except Exception as e:
        out_q.put(("error", repr(e)))
        raise


def test_eight_gloo_ranks_head_parallel_work_units():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, port = 8, _free_port()
    procs = [ctx.Process(target=_hp_units_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a gloo rank did not finish")
        assert p.exitcode == 0
    kind, err = q.get(timeout=10)
    assert kind == "ok", err
    assert err < 1e-4, f"work-unit partial sums differ from the full block by {err}"

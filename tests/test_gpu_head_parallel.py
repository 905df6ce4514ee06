"""Head-parallel encoder layer (one long sequence, one all-reduce per layer) against the
unsharded oracle layer: the ranks' shares computed one after another on ONE GPU and added there
(the product's two entry points, every rank's work units, no collective), and the real thing on
two GPUs over NCCL (skipped with fewer than two visible GPUs)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,reduce_dtype,mask_kind", [(8, "fp16", 0), (8, "fp32", 1), (3, "fp16", 0)])
def test_head_parallel_ranks_emulated_on_one_gpu(world, reduce_dtype, mask_kind):
    """12 heads on 8 ranks = 24 (head, query half) units, 3 per rank; on 3 ranks 4 heads each."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from conftest import assert_close
    et = entry.load_package()
    orc = entry.load_oracle()
    orc.build()
    dev = torch.device("cuda:0")
    hidden, nhead, ff, seq = 768, 12, 3072, 1024
    w = et.synth.encoder_layer_weights(41, 0, hidden, ff, std=0.03, bias_std=0.02, ln_noise=0.1)
    x = et.synth.normal(41, 3, (seq, hidden), 1.0)
    xd = torch.from_numpy(x).to(dev)
    total, layer0 = None, None
    for rank in range(world):
        layer = et.HeadParallelLayer(w, nhead, et.sharding.Job(rank=rank, world=world, device=dev),
                                     et.ACT_GELU, device=dev, reduce_dtype=reduce_dtype)
        part = layer.partial_sum(xd, 1, seq, mask_kind)
        total = part.float() if total is None else total + part.float()
        layer0 = layer0 or layer
    total = total if reduce_dtype == "fp32" else total.half()
    y = layer0.finish(total.contiguous(), xd, 1, seq)
    torch.cuda.synchronize()
    assert et.device_error() == 0
    ref = orc.encoder_layer(x, w, 1, seq, nhead, 2, mask_kind)
    assert_close(y.float().cpu().numpy(), ref, f"head-parallel layer, {world} emulated ranks")


@pytest.mark.parametrize("world,seq", [(8, 1024), (3, 1000)])
def test_peer_exchange_ranks_emulated_on_one_gpu(world, seq):
    """The exchange over peer memory (signal -> reduce + LayerNorm + gather -> wait) with every
    rank's buffer on ONE GPU: all ranks' partials and signals run first, then all reductions, then the waits,
    so no kernel ever waits for a later one.  Every rank must end up with the same y and the
    same layer output as the all-reduce form; two layers in a row exercise buffer reuse."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from conftest import assert_close
    et = entry.load_package()
    orc = entry.load_oracle()
    orc.build()
    dev = torch.device("cuda:0")
    hidden, nhead, ff = 768, 12, 3072
    w = et.synth.encoder_layer_weights(43, 0, hidden, ff, std=0.03, bias_std=0.02, ln_noise=0.1)
    x = et.synth.normal(43, 3, (seq, hidden), 1.0)
    layers = [et.HeadParallelLayer(w, nhead, et.sharding.Job(rank=r, world=world, device=dev),
                                   et.ACT_GELU, device=dev) for r in range(world)]
    exs = et.PeerExchange.local(world, seq, hidden)
    d = layers[0].full.desc
    import ctypes
    g, b = ctypes.c_void_p(d.ln1_gamma), ctypes.c_void_p(d.ln1_beta)
    cur = x
    try:
        for _ in range(2):
            xd = torch.from_numpy(np.ascontiguousarray(cur)).to(dev)
            for r in range(world):
                layers[r].partial_sum(xd, 1, seq, out_ptr=exs[r].partial())
                exs[r].epoch += 1
                exs[r].signal()
            for r in range(world):
                exs[r].reduce_layernorm(xd, None, g, b)
            outs = []
            for r in range(world):
                exs[r].wait()
                outs.append(layers[r].ffn(exs[r].y(), xd, 1, seq))
            torch.cuda.synchronize()
            assert et.device_error() == 0
            for r in range(1, world):
                assert torch.equal(outs[r], outs[0]), f"rank {r} differs from rank 0"
            ref = orc.encoder_layer(cur, w, 1, seq, nhead, 2, 0)
            assert_close(outs[0].float().cpu().numpy(), ref, f"peer exchange, {world} emulated ranks")
            cur = outs[0].cpu().numpy()
    finally:
        for ex in exs:
            ex.close()


@pytest.mark.parametrize("world,seq", [(8, 1024), (3, 1000)])
def test_token_sharded_ffn_ranks_emulated_on_one_gpu(world, seq):
    """The token-sharded form (reduce-scatter after the output projection, feed-forward block on
    the rank's own rows, all-gather of the finished rows), every rank's buffer on ONE GPU and
    every rank's step run before the next step of any rank.  Two layers chained through the
    exchange buffers' alternating out slots; all ranks must hold the same output."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from conftest import assert_close
    et = entry.load_package()
    orc = entry.load_oracle()
    orc.build()
    dev = torch.device("cuda:0")
    hidden, nhead, ff = 768, 12, 3072
    w = et.synth.encoder_layer_weights(47, 0, hidden, ff, std=0.03, bias_std=0.02, ln_noise=0.1)
    x = et.synth.normal(47, 3, (seq, hidden), 1.0)
    layers = [et.HeadParallelLayer(w, nhead, et.sharding.Job(rank=r, world=world, device=dev),
                                   et.ACT_GELU, device=dev) for r in range(world)]
    exs = et.PeerExchange.local(world, seq, hidden)
    try:
        xs = [torch.from_numpy(x).to(dev) for _ in range(world)]
        ref = x
        for _ in range(2):
            for phase in ("partial", "reduce", "ffn", "wait"):
                outs = [layers[r].forward_peer_sharded(xs[r], 1, seq, exs[r], phase=phase) for r in range(world)]
            torch.cuda.synchronize()
            assert et.device_error() == 0
            for r in range(1, world):
                assert torch.equal(outs[r], outs[0]), f"rank {r} differs from rank 0"
            ref = orc.encoder_layer(ref, w, 1, seq, nhead, 2, 0)
            assert_close(outs[0].float().cpu().numpy(), ref, f"token-sharded form, {world} emulated ranks")
            ref = outs[0].cpu().numpy()
            xs = outs
    finally:
        for ex in exs:
            ex.close()


def _worker(rank: int, world: int, port: int, out_q, peer=False):
    try:
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        et = entry.load_package()
        hidden, nhead, ff, seq = 768, 12, 3072, 1024
        w = et.synth.encoder_layer_weights(41, 0, hidden, ff, std=0.03, bias_std=0.02, ln_noise=0.1)
        x = et.synth.normal(41, 3, (seq, hidden), 1.0)
        job = et.sharding.Job(rank=rank, world=world, device=dev)
        layer = et.HeadParallelLayer(w, nhead, job, et.ACT_GELU, device=dev)
        xd = torch.from_numpy(x).to(dev)
        if peer:
            ex = et.PeerExchange(job, seq, hidden)
            dist.barrier()
            fwd = layer.forward_peer_sharded if peer == "sharded" else layer.forward_peer
            y = fwd(xd, 1, seq, ex)
            y = fwd(y, 1, seq, ex).clone()  # a second layer call reuses the buffers
        else:
            y = layer.forward(xd, 1, seq)
        torch.cuda.synchronize()
        err = et.device_error()
        if peer:
            dist.barrier()
            ex.close()
        if rank == 0:
            out_q.put(("ok", y.float().cpu().numpy(), err))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        out_q.put(("error", repr(e), -1))
        raise


@pytest.mark.parametrize("peer", [False, True, "sharded"])
def test_head_parallel_layer_two_gpus(peer):
    """peer=False: one NCCL all-reduce per layer; peer=True: the exchange by this library's
    kernels over peer memory (CUDA IPC mappings), two layer calls in a row; "sharded": the same
    with the feed-forward block on each rank's own token rows."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    et = entry.load_package()
    orc = entry.load_oracle()
    orc.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, peer)) for r in range(world)]
    for p in procs:
        p.start()
    kind, y, err = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert kind == "ok", y
    assert err == 0
    hidden, nhead, ff, seq = 768, 12, 3072, 1024
    w = et.synth.encoder_layer_weights(41, 0, hidden, ff, std=0.03, bias_std=0.02, ln_noise=0.1)
    x = et.synth.normal(41, 3, (seq, hidden), 1.0)
    ref = orc.encoder_layer(x, w, 1, seq, nhead, 2, 0)
    if peer:
        ref = orc.encoder_layer(np.asarray(ref, dtype=np.float32).astype(np.float16).astype(np.float32), w,
                                1, seq, nhead, 2, 0)
    from conftest import assert_close
    assert_close(y, ref, "head-parallel layer on 2 GPUs" + (" over peer memory" if peer else ""))

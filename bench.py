#!/usr/bin/env python
"""Throughput benchmark of the encoder hot path: BERT-base, seq 128, sequences/s.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # CPU evaluation of the same math

A step is one forward pass of the 12-layer BERT-base encoder stack (hidden 768, 12 heads,
FFN 3072, GELU, post-LN) over one batch of 16 sequences of 128 tokens per GPU, fp16 storage
with fp32 accumulation, all-ones attention mask, seeded synthetic weights ~N(0, 0.02) and
inputs ~N(0, 1).  With N > 1 (launched by torch.distributed.run, one process per GPU) every
rank runs its own batch with replicated weights and no data-path collective (weak scaling).
Prints ONE JSON line on rank 0.

The timed region of K steps is repeated (`--repeats`, default 9) and the line reports the
median repeat, with the spread and the repeats binned by the SM clock sampled during them.
Beside the headline the line carries, under `configs`, the other benchmark configurations
(batch 64; tile-pruned with pruned Q/K features; BERT-large with mixed pruning formats;
seq 512 at a global batch of 256; one 4096-token sequence head-parallel when N > 1), each with
its own step time, sequences/s, TFLOP/s and fraction of its tensor-core roofline.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "BERT-base seq128 sequences/s"
UNIT = "sequences/s"
WORKLOAD = ("BERT-base 12L h768 12 heads FFN3072 GELU, batch 16 per GPU, seq 128, dense weights, "
            "all-ones mask")
HIDDEN, NHEAD, FF, LAYERS, SEQ, BATCH = 768, 12, 3072, 12, 128, 16
LONG_BATCH, LONG_SEQ = 2, 4096  # secondary per-kernel entry: attention on long sequences
SEED = 2021
# The four kernels of one layer at this batch: measured DRAM bytes of one launch ("traffic") and
# the operands read / written once in fp16 ("algorithmic_bytes").
_T = BATCH * SEQ
STACK_KERNELS = {
    "qkv_attention_fused": {
        "label": "qkv_attention_kernel (Q/K/V projection + attention)",
        "traffic": 6727424, "algorithmic_bytes": 2 * (2 * _T * HIDDEN + 3 * HIDDEN * HIDDEN)},
    "o_layernorm_fused": {
        "label": "gemm_ln_kernel (O projection + residual + LayerNorm)",
        "traffic": 7507712, "algorithmic_bytes": 2 * (3 * _T * HIDDEN + HIDDEN * HIDDEN)},
    "ffn1_gelu": {
        "label": f"gemm_f16_kernel (FFN1 + GELU, [{_T}x768]x[3072x768]^T)",
        "traffic": 7931392, "algorithmic_bytes": 2 * (_T * HIDDEN + FF * HIDDEN + _T * FF)},
    "ffn2_layernorm_fused": {
        "label": f"gemm_ln_kernel (FFN2 + residual + LayerNorm, [{_T}x3072]x[768x3072]^T)",
        "traffic": 20484096, "algorithmic_bytes": 2 * (_T * FF + FF * HIDDEN + 2 * _T * HIDDEN)},
}


def config_dict(world: int) -> dict:
    """Identical in both arms (notes live outside `config`)."""
    return {"workload": WORKLOAD, "global_batch": BATCH * world, "seq_len": SEQ,
            "parallelism": f"dp{world}"}


def flops_per_sequence(seq=SEQ, hidden=HIDDEN, ff=FF, layers=LAYERS, kdim=None, vdim=None,
                       lin_flops_per_token=None) -> float:
    """GEMM-like contractions only: per layer per sequence seq * 2 * (weights kept) +
    2 * seq^2 * kdim + 2 * seq^2 * vdim.  `lin_flops_per_token` overrides the dense count of the
    four Linear layers (2 * stored weights, e.g. 512 per stored 16 x 16 tile)."""
    kdim = hidden if kdim is None else kdim
    vdim = hidden if vdim is None else vdim
    if lin_flops_per_token is None:
        lin_flops_per_token = 2 * ((2 * kdim + vdim) * hidden + hidden * vdim + 2 * hidden * ff)
    return layers * (seq * lin_flops_per_token + 2 * seq * seq * (kdim + vdim))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0,
            "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.active = False

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            }
            while not self._stop_evt.is_set():
                if self.active:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                time.sleep(0.002)
        except Exception as e:  # NVML missing: report what we know
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._stop_evt.set()

    def mark(self) -> int:
        return len(self.samples)

    def median_since(self, mark: int):
        s = self.samples[mark:]
        return statistics.median(s) if s else None

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def build_weights(et, tile_sparsity: float = 0.0, base=None):
    """The headline stack's weights (counter-based generator); `base` re-uses a dense set and
    only re-prunes it."""
    ws = []
    for layer in range(LAYERS):
        w = dict(base[layer]) if base is not None else \
            et.synth.encoder_layer_weights(SEED, layer, HIDDEN, FF)
        if tile_sparsity > 0:
            for i, name in enumerate(("wqkv", "wo", "w1", "w2")):
                w[name] = et.synth.prune_tiles(w[name], SEED, 100 * (layer + 1) + 50 + i,
                                               tile_sparsity)
        ws.append(w)
    return ws


def stored_tiles(ws) -> int:
    n = 0
    for w in ws:
        for name in ("wqkv", "wo", "w1", "w2"):
            m = w[name]
            n += int((m.reshape(m.shape[0] // 16, 16, -1, 16) != 0).any(axis=(1, 3)).sum())
    return n


def run_reference(args, rank: int, world: int):
    """CPU arm: the reference has no CPU implementation; the oracle (a C++/OpenMP port of the same
    math) is timed on the host cores.  A step is the whole 12-layer stack over one batch of 16
    sequences, the same unit of work as a step of the GPU arm."""
    if rank != 0:
        return
    import numpy as np
    et = entry.load_package()
    orc = entry.load_oracle()
    orc.build()
    # process launchers export OMP_NUM_THREADS=1: use every core this process may run on
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    ws = [et.synth.encoder_layer_weights(SEED, l, HIDDEN, FF, fast=True) for l in range(LAYERS)]
    x = et.synth.normal(SEED, 7000, (BATCH * SEQ, HIDDEN), 1.0).astype(np.float32)

    def step():
        cur = x
        for w in ws:
            cur = orc.encoder_layer(cur, w, BATCH, SEQ, NHEAD, 2, 0)
        return cur

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = BATCH / dt
    sample = (f"{args.steps} steps, each the full {LAYERS}-layer stack over {BATCH} sequences of "
              f"{SEQ} tokens (fp32, OpenMP)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_dict(world),
        "notes": {"what": "CPU evaluation (oracle port, OpenMP, fp32) of the same encoder math on "
                          "rank 0's host cores; one batch of 16 sequences per step whatever N"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def time_kernel(fns, rounds: int = 6, warm: int = 3):
    """Seconds per call.  `fns` is a list of closures over DISTINCT buffer sets whose total size
    exceeds L2; one CUDA graph launches them round-robin `rounds` times, so every call finds its
    operands evicted, and no host launch gap is timed."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for fn in fns:
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(rounds):
            for fn in fns:
                fn()
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (rounds * len(fns))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=9, help="timed regions of --steps steps each")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch kernels directly")
    ap.add_argument("--lanes", type=int, default=1,
                    help="groups of sequences that run through the stack on their own streams")
    ap.add_argument("--skip-extras", action="store_true",
                    help="skip the other configurations / per-kernel / CPU legs (used under profilers)")
    ap.add_argument("--attention-only", action="store_true",
                    help="launch the attention kernel alone (2 sequences of 4096 tokens, three "
                         "times) and exit: the small case profilers capture")
    ap.add_argument("--tile-only", action="store_true",
                    help="launch the tile-pruned Linear alone (2048 x 768 -> 3072, 80 %% of the "
                         "tiles pruned, three times) and exit: the small case profilers capture")
    ap.add_argument("--only", default="", choices=["", "vo", "pair", "layernorm", "1x16", "col", "row", "tile_qkv", "fuse_o", "hp_reduce", "layer"],
                    help="launch one more small case three times and exit (for profilers): fused V.O "
                         "attention, the CTA-pair GEMM at 8192^3, skip-LayerNorm, the 1x16 vector "
                         "kernel, the column-pruned Linear (gather + GEMM), a tile-pruned Q/K/V projection "
                         "(on the persistent tile kernel when ET_B200_TEST_HOOKS=1 selects the hooks "
                         "library), one dense encoder layer")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    et = entry.load_package()
    et.lib()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # the job's stdout carries exactly one JSON line: NCCL's own messages (the version
        # banner it prints at the WARN and VERSION levels included) go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    if args.attention_only:
        qkv = torch.from_numpy(et.synth.normal(1, 70, (LONG_BATCH * LONG_SEQ, 3 * HIDDEN), 1.0)).to(dev)
        z = torch.empty((LONG_BATCH * LONG_SEQ, HIDDEN), dtype=torch.float16, device=dev)
        for _ in range(3):
            et.attention(qkv[:, :HIDDEN], qkv[:, HIDDEN:2 * HIDDEN], qkv[:, 2 * HIDDEN:],
                         LONG_BATCH, LONG_SEQ, NHEAD, 64, 64, out=z)
        torch.cuda.synchronize()
        print(json.dumps({"attention_only": True, "batch": LONG_BATCH, "seq": LONG_SEQ,
                          "device_error": et.device_error()}))
        return
    if args.tile_only:
        W = et.synth.prune_tiles(et.synth.normal_fast(1, 40, (FF, HIDDEN), 0.02), 1, 41, 0.8)
        pk = et.PackedTiles(*et.synth.dense_to_tile(W), HIDDEN, FF, dev)
        x = torch.from_numpy(et.synth.normal_fast(1, 42, (_T, HIDDEN), 1.0)).to(dev)
        for _ in range(3):
            et.linear_tile_packed(x, pk, None, et.ACT_GELU)
        torch.cuda.synchronize()
        print(json.dumps({"tile_only": True, "tokens": _T, "in": HIDDEN, "out": FF,
                          "stored_tiles": pk.nnz, "device_error": et.device_error()}))
        return

    if args.only:
        rnd = lambda tid, shape, std=1.0: torch.from_numpy(et.synth.normal_fast(1, tid, shape, std)).to(dev)
        T = _T
        if args.only == "vo":      # 16 sequences x 128 tokens, 12 heads
            q, k = rnd(1, (T, HIDDEN)), rnd(2, (T, HIDDEN))
            vo = rnd(3, (BATCH * NHEAD * SEQ, HIDDEN))
            fn = lambda: et.fused_vo_attention(q, k, vo, None, BATCH, SEQ, NHEAD, 64, HIDDEN)
        elif args.only == "pair":  # 8192^3 on CTA pairs
            a, w = rnd(1, (8192, 8192)), rnd(2, (8192, 8192), 0.02)
            y = torch.empty((8192, 8192), dtype=torch.float16, device=dev)
            fn = lambda: et.linear_dense(a, w, None, 0, out=y)
        elif args.only == "layernorm":  # 64 x 2048 rows of 768: 600 MB of traffic, beyond L2
            a, s2 = rnd(1, (64 * T, HIDDEN)), rnd(2, (64 * T, HIDDEN))
            g = torch.ones(HIDDEN, dtype=torch.float16, device=dev)
            o = torch.empty_like(a)
            fn = lambda: et.skip_layernorm(a, s2, g, g, out=o)
        elif args.only == "1x16":  # 2048 x 768 -> 3072, 90 % of the vectors pruned
            W = et.synth.prune_1x16(et.synth.normal_fast(1, 2, (FF, HIDDEN), 0.02), 1, 3, 0.9)
            ti, ri, da = (torch.from_numpy(v).to(dev) for v in et.synth.dense_to_1x16(W))
            x = rnd(1, (T, HIDDEN))
            fn = lambda: et.linear_1x16(x, ti, ri, da, FF)
        elif args.only == "tile_qkv":  # 2048 x 768 -> 2304, 80 % of the tiles pruned
            # (with ET_B200_TEST_HOOKS=1 in the environment: on the persistent tile kernel)
            if hasattr(et.lib(), "et_debug_set_tile_persist"):
                et.lib().et_debug_set_tile_persist(1)
            W = et.synth.prune_tiles(et.synth.normal_fast(1, 40, (3 * HIDDEN, HIDDEN), 0.02), 1, 41, 0.8)
            pk = et.PackedTiles(*et.synth.dense_to_tile(W), HIDDEN, 3 * HIDDEN, dev)
            x = rnd(1, (T, HIDDEN))
            fn = lambda: et.linear_tile_packed(x, pk, None, et.ACT_NONE)
        elif args.only == "row":   # 8192 x 768 -> 3072, half of the output rows kept, full-width output
            W = et.synth.normal_fast(1, 2, (FF, HIDDEN), 0.02)
            ids = et.synth.choose_ids(1, 3, FF, 0.5)
            rid, rows = (torch.from_numpy(v).to(dev) for v in et.synth.dense_to_row(W, ids))
            x = rnd(1, (4 * T, HIDDEN))
            fn = lambda: et.linear_row(x, rid, rows, FF, None, et.ACT_GELU)
        elif args.only == "hp_reduce":  # head-parallel exchange, 8 ranks emulated on this GPU
            # one 4096-token sequence: every rank publishes its partial, then rank 0 pulls its
            # 512 rows of all eight partials, adds the residual, normalises and stores the rows
            # into every rank's buffer (all buffers live on this GPU: local HBM, not NVLink)
            exs = et.PeerExchange.local(8, 4096, HIDDEN)
            x = rnd(1, (4096, HIDDEN))
            gma = torch.ones(HIDDEN, dtype=torch.float16, device=dev)
            for r, ex in enumerate(exs):
                part = et.device_view(ex.partial(), (4096, HIDDEN), dev)
                part.copy_(rnd(10 + r, (4096, HIDDEN), 0.3))

            def fn():
                for ex in exs:
                    ex.epoch += 1
                    ex.signal()
                for ex in exs:
                    ex.reduce_layernorm(x, None, gma, gma)
        elif args.only == "fuse_o":  # attention + 80 %-pruned O projection in one kernel
            qkv = rnd(1, (T, 3 * HIDDEN))
            Wo = et.synth.prune_tiles(et.synth.normal_fast(1, 45, (HIDDEN, HIDDEN), 0.02), 1, 46, 0.8)
            rp_o, ro_o, tl_o = (torch.from_numpy(v).to(dev) for v in et.synth.dense_to_tile(Wo))
            fn = lambda: et.attention_fuse_o(qkv[:, :HIDDEN], qkv[:, HIDDEN:2 * HIDDEN],
                                             qkv[:, 2 * HIDDEN:], rp_o, ro_o, tl_o, None, BATCH, SEQ,
                                             NHEAD, 64, 64, HIDDEN, single_launch=True)
        elif args.only == "col":   # 8192 x 3072 -> 768, half of the input columns kept
            W = et.synth.normal_fast(1, 2, (HIDDEN, FF), 0.02)
            ids = et.synth.choose_ids(1, 3, FF, 0.5)
            cid, cols = (torch.from_numpy(v).to(dev) for v in et.synth.dense_to_col(W, ids))
            x = rnd(1, (4 * T, FF))
            fn = lambda: et.linear_col(x, cid, cols)
        else:                      # one dense BERT-base layer, 16 x 128 tokens
            lw = et.synth.encoder_layer_weights(SEED, 0, HIDDEN, FF, fast=True)
            st1 = et.EncoderStack([et.EncoderLayer(lw, NHEAD, et.ACT_GELU, device=dev)], BATCH, SEQ, dev)
            x = rnd(1, (T, HIDDEN))
            fn = lambda: st1.forward(x)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        print(json.dumps({"only": args.only, "device_error": et.device_error()}))
        return

    def launch_count():
        return int(et.lib().et_launch_count())

    job = et.sharding.Job(rank=rank, world=world, device=dev)

    def barrier():
        job.barrier()
        torch.cuda.synchronize()

    max_over_ranks = job.max_over_ranks
    peaks = measured_peaks()
    stream = torch.cuda.Stream(device=dev)
    sampler = ClockSampler(local_rank)
    sampler.start()

    def make_step(st, x):
        """Returns (callable, launches per step): one forward of the whole stack on `stream`,
        replayed from a CUDA graph unless --no-graph."""
        with torch.cuda.stream(stream):
            n0 = launch_count()
            st.forward(x)  # warm: sets kernel attributes before capture
            launches = launch_count() - n0  # the library's own host-side count
            stream.synchronize()
            if args.no_graph:
                return (lambda: st.forward(x)), launches
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                st.forward(x)
            return g.replay, launches

    def timed(step_fn, steps, repeats=1, before=None, after=None, sample_clock=False):
        """`repeats` timed regions of `steps` steps, each bracketed by barrier + synchronize and
        timed with CUDA events on the launching stream; returns [(seconds, median SM MHz)] with
        the seconds already the maximum over ranks."""
        out = []
        with torch.cuda.stream(stream):
            for _ in range(args.warmup):
                if before:
                    before()
                step_fn()
                if after:
                    after()
            for _ in range(repeats):
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                mark = sampler.mark()
                sampler.active = sample_clock
                e0.record(stream)
                for _ in range(steps):
                    if before:
                        before()
                    step_fn()
                    if after:
                        after()
                e1.record(stream)
                barrier()
                sampler.active = False
                out.append((max_over_ranks(e0.elapsed_time(e1) * 1e-3), sampler.median_since(mark)))
        return out

    def med(regions):
        return statistics.median(t for t, _ in regions)

    # ---------------------------------------------------------------- headline: C2, batch 16
    ws = build_weights(et)
    layers = [et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev) for w in ws]
    stack = et.EncoderStack(layers, BATCH, SEQ, device=dev, lanes=args.lanes)
    x_host = torch.from_numpy(et.synth.normal(SEED, 7000 + rank, (BATCH * SEQ, HIDDEN), 1.0))
    x_pinned = x_host.pin_memory()
    y_pinned = torch.empty_like(x_pinned).pin_memory()
    x_dev = x_pinned.to(dev)
    final_out = stack.buf[(LAYERS - 1) & 1]
    step_fn, kernels_per_step = make_step(stack, x_dev)  # BERT-base b16: 4 kernels per layer

    regions = timed(step_fn, args.steps, args.repeats, sample_clock=True)
    dt = med(regions)
    serial = timed(step_fn, args.steps, 3, sample_clock=True,
                   before=lambda: x_dev.copy_(x_pinned, non_blocking=True),
                   after=lambda: y_pinned.copy_(final_out, non_blocking=True))
    dt_e2e_serial = med(serial)

    # End to end through the package's serving loop: every step copies its input batch from
    # pinned host memory and its result back; copies of neighbouring steps overlap the compute.
    pipe = et.HostPipeline(stack, depth=2, use_graph=not args.no_graph)
    x_pin = [x_pinned, x_host.clone().pin_memory()]
    y_pin = [y_pinned, torch.empty_like(x_pinned).pin_memory()]

    def timed_pipeline(steps, repeats):
        out = []
        for i in range(args.warmup):
            pipe.submit(x_pin[i & 1], y_pin[i & 1])
        pipe.drain()
        for _ in range(repeats):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sampler.active = True
            e0.record(pipe.s_in)
            for i in range(steps):
                pipe.submit(x_pin[i & 1], y_pin[i & 1])
            e1.record(pipe.s_out)
            pipe.drain()
            barrier()
            sampler.active = False
            out.append(max_over_ranks(e0.elapsed_time(e1) * 1e-3))
        return out

    e2e_regions = timed_pipeline(args.steps, min(args.repeats, 5))
    dt_e2e = statistics.median(e2e_regions)
    with torch.cuda.stream(stream):
        step_fn()
        stream.synchronize()
    if not torch.equal(y_pin[0], final_out.cpu()) or not torch.equal(y_pin[1], y_pin[0]):
        raise SystemExit("serving loop and resident forward disagree")
    code = et.device_error()
    if code != 0:
        raise SystemExit(f"device error word = {code}")

    value = world * BATCH * args.steps / dt
    e2e_value = world * BATCH * args.steps / dt_e2e
    ms = [t / args.steps * 1e3 for t, _ in regions]
    bins = {}
    for t, mhz in regions:
        bins.setdefault(str(int(mhz)) if mhz else "unsampled", []).append(t / args.steps * 1e3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (f32 accumulate)",
        "data": "synthetic", "config": config_dict(world),
        "notes": {"l2": "weights (170 MB fp16) exceed the 126 MB L2 and are streamed every step",
                  "cuda_graph": not args.no_graph,
                  "value": "median of the repeated timed regions of `steps` steps each"},
        "repeats": {"n": len(regions), "ms_per_step_median": statistics.median(ms),
                    "ms_per_step_min": min(ms), "ms_per_step_max": max(ms),
                    "ms_per_step_by_sm_mhz": {k: statistics.median(v) for k, v in bins.items()}},
        "e2e_serial": {"value": world * BATCH * args.steps / dt_e2e_serial, "unit": UNIT,
                       "note": "copy in, stack, copy out on one stream (no overlap)"},
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": x_pinned.numel() * 2, "d2h_bytes_per_step": y_pinned.numel() * 2,
                "repeats": len(e2e_regions)},
        "gpu_launches": world * args.steps * kernels_per_step,
        "kernels_per_step": kernels_per_step,
        "stack_tflops": value / world * flops_per_sequence() * 1e-12,
        "stack_frac_of_peak": value / world * flops_per_sequence() * 1e-12 / peaks["bf16_tflops_sustained"],
        "stack_frac_of_burst_roofline": value / world * flops_per_sequence() * 1e-12 / peaks["bf16_tflops"],
    }

    if not args.skip_extras:
        # ---- the layer's kernels in isolation ----
        T = BATCH * SEQ
        with torch.cuda.stream(stream):
            per_kernel = {}
            shapes = {"qkv": (HIDDEN, 3 * HIDDEN, 0), "o": (HIDDEN, HIDDEN, 0),
                      "ffn1_gelu": (HIDDEN, FF, 2), "ffn2": (FF, HIDDEN, 0)}
            NSETS = 10  # x 20 MB per set: beyond the 126 MB L2

            def rnd(tid, shape, std):
                return torch.from_numpy(et.synth.normal_fast(1, tid, shape, std)).to(dev)

            for name, (inn, out, act) in shapes.items():
                a = [rnd(10 + i, (T, inn), 1.0) for i in range(NSETS)]
                w = [rnd(40 + i, (out, inn), 0.02) for i in range(NSETS)]
                y = [torch.empty((T, out), dtype=torch.float16, device=dev) for _ in range(NSETS)]
                b = torch.zeros(out, dtype=torch.float16, device=dev)
                sec = time_kernel([lambda i=i: et.linear_dense(a[i], w[i], b, act, out=y[i])
                                   for i in range(NSETS)])
                per_kernel[name] = {"us": sec * 1e6, "tflops": 2.0 * T * inn * out / sec * 1e-12}
                if out == HIDDEN:
                    # the same product with residual + LayerNorm in its epilogue (what the
                    # stack runs at this batch for the O projection and FFN2)
                    res = [rnd(60 + i, (T, out), 1.0) for i in range(NSETS)]
                    gm = torch.ones(out, dtype=torch.float16, device=dev)
                    sec = time_kernel([lambda i=i: et.linear_skip_layernorm(a[i], w[i], b, res[i],
                                                                            gm, b, out=y[i])
                                       for i in range(NSETS)])
                    per_kernel[name + "_layernorm_fused"] = {
                        "us": sec * 1e6, "tflops": 2.0 * T * inn * out / sec * 1e-12}
                    del res
                if name == "ffn1_gelu":
                    # the tile-pruned Linear on the same shape, 80 % of the tiles pruned
                    pks = []
                    for i in range(NSETS):
                        Wp = et.synth.prune_tiles(w[i].cpu().numpy(), 1, 80 + i, 0.8)
                        pks.append(et.PackedTiles(*et.synth.dense_to_tile(Wp), inn, out, dev))
                    sec = time_kernel([lambda i=i: et.linear_tile_packed(a[i], pks[i], b, act)
                                       for i in range(NSETS)])
                    per_kernel["ffn1_gelu_tile80"] = {
                        "us": sec * 1e6, "stored_tiles": pks[0].nnz,
                        "tflops_surviving": 512.0 * pks[0].nnz * T / sec * 1e-12,
                        "speedup_vs_dense": per_kernel[name]["us"] / (sec * 1e6)}
                    del pks
            qkv = [rnd(70 + i, (T, 3 * HIDDEN), 1.0) for i in range(NSETS)]
            z = [torch.empty((T, HIDDEN), dtype=torch.float16, device=dev) for _ in range(NSETS)]
            sec = time_kernel([lambda i=i: et.attention(qkv[i][:, :HIDDEN],
                                                        qkv[i][:, HIDDEN:2 * HIDDEN],
                                                        qkv[i][:, 2 * HIDDEN:], BATCH, SEQ, NHEAD,
                                                        64, 64, out=z[i]) for i in range(NSETS)])
            per_kernel["attention"] = {"us": sec * 1e6,
                                       "tflops": 4.0 * BATCH * SEQ * SEQ * HIDDEN / sec * 1e-12}
            xs = [rnd(10 + i, (T, HIDDEN), 1.0) for i in range(NSETS)]
            wq = [rnd(40 + i, (3 * HIDDEN, HIDDEN), 0.02) for i in range(NSETS)]
            bqz = torch.zeros(3 * HIDDEN, dtype=torch.float16, device=dev)
            sec = time_kernel([lambda i=i: et.qkv_attention(xs[i], wq[i], bqz, BATCH, SEQ, NHEAD,
                                                            HIDDEN, HIDDEN) for i in range(NSETS)])
            per_kernel["qkv_attention_fused"] = {
                "us": sec * 1e6,
                "tflops": (2.0 * T * HIDDEN * 3 * HIDDEN + 4.0 * BATCH * SEQ * SEQ * HIDDEN) / sec * 1e-12}
            del xs, wq, qkv, z
            # the on-the-fly attention kernel where it dominates: long sequences (not part of
            # the headline workload, whose 128-token sequences take the fused kernel above)
            TL = LONG_BATCH * LONG_SEQ
            qkv = [rnd(70 + i, (TL, 3 * HIDDEN), 1.0) for i in range(4)]
            z = [torch.empty((TL, HIDDEN), dtype=torch.float16, device=dev) for _ in range(4)]
            sec = time_kernel([lambda i=i: et.attention(qkv[i][:, :HIDDEN],
                                                        qkv[i][:, HIDDEN:2 * HIDDEN],
                                                        qkv[i][:, 2 * HIDDEN:], LONG_BATCH,
                                                        LONG_SEQ, NHEAD, 64, 64, out=z[i])
                               for i in range(4)], rounds=3)
            per_kernel[f"attention_b{LONG_BATCH}_seq{LONG_SEQ}"] = {
                "us": sec * 1e6,
                "tflops": 4.0 * LONG_BATCH * LONG_SEQ * LONG_SEQ * HIDDEN / sec * 1e-12}
            a = [rnd(90 + i, (T, HIDDEN), 1.0) for i in range(4 * NSETS)]
            o = [torch.empty((T, HIDDEN), dtype=torch.float16, device=dev) for _ in range(4 * NSETS)]
            g = torch.ones(HIDDEN, dtype=torch.float16, device=dev)
            sec = time_kernel([lambda i=i: et.skip_layernorm(a[i], a[i], g, g, out=o[i])
                               for i in range(4 * NSETS)], rounds=2)
            per_kernel["skip_layernorm"] = {"us": sec * 1e6, "gbs": 6.0 * T * HIDDEN / sec * 1e-9}
            # attention + tile-pruned output projection (80 % of W_O's tiles pruned): one
            # kernel (work tickets and completion counters) against the two kernels chained by
            # dependent launch
            qkv = [rnd(70 + i, (T, 3 * HIDDEN), 1.0) for i in range(NSETS)]
            Wo = et.synth.prune_tiles(et.synth.normal_fast(1, 45, (HIDDEN, HIDDEN), 0.02), 1, 46, 0.8)
            rp_o, ro_o, tl_o = (torch.from_numpy(v).to(dev) for v in et.synth.dense_to_tile(Wo))
            fo = {}
            for single in (True, False):
                fo[single] = time_kernel([lambda i=i: et.attention_fuse_o(
                    qkv[i][:, :HIDDEN], qkv[i][:, HIDDEN:2 * HIDDEN], qkv[i][:, 2 * HIDDEN:], rp_o, ro_o,
                    tl_o, bqz[:HIDDEN], BATCH, SEQ, NHEAD, 64, 64, HIDDEN, single_launch=single)
                    for i in range(NSETS)]) * 1e6
            per_kernel["attention_fuse_o_tile80"] = {
                "single_launch_us": fo[True], "two_chained_kernels_us": fo[False],
                "product_path": "two chained kernels"}
            # row-pruned Linear at the FFN1 shape, half of the output features kept: full-width
            # output (compressed GEMM + in-place expand) and compressed output
            ids_r = et.synth.choose_ids(1, 47, FF, 0.5)
            Wr = et.synth.normal_fast(1, 48, (FF, HIDDEN), 0.02)
            rid_r, rows_r = (torch.from_numpy(v).to(dev) for v in et.synth.dense_to_row(Wr, ids_r))
            xr = [rnd(10 + i, (T, HIDDEN), 1.0) for i in range(NSETS)]
            b_ff = torch.zeros(FF, dtype=torch.float16, device=dev)
            t_full = time_kernel([lambda i=i: et.linear_row(xr[i], rid_r, rows_r, FF, b_ff, et.ACT_GELU)
                                  for i in range(NSETS)]) * 1e6
            t_comp = time_kernel([lambda i=i: et.linear_row_compressed(xr[i], rid_r, rows_r, b_ff)
                                  for i in range(NSETS)]) * 1e6
            per_kernel["ffn1_row_pruned_half"] = {
                "full_width_output_us": t_full, "compressed_output_us": t_comp,
                "dense_us": per_kernel["ffn1_gelu"]["us"], "kept_features": int(len(ids_r))}
            del xr
            per_kernel["note"] = ("each kernel timed inside one CUDA graph that rotates over buffer "
                                  "sets larger than L2")
            del a, w, y, qkv, z, o
        # the dominant kernel = the longest of the four that make up a layer at this batch
        dom = max(STACK_KERNELS, key=lambda n: per_kernel[n]["us"])
        k = per_kernel[dom]
        line["roofline"] = {"bound": "tensor", "kernel": STACK_KERNELS[dom]["label"],
                            "achieved": k["tflops"], "peak": peaks["bf16_tflops"],
                            "unit": "TFLOP/s", "frac": k["tflops"] / peaks["bf16_tflops"],
                            "us_per_launch": k["us"],
                            "traffic": STACK_KERNELS[dom]["traffic"],
                            "algorithmic_bytes": STACK_KERNELS[dom]["algorithmic_bytes"],
                            "peak_source": peaks["source"] + " (burst, kernel timed alone)"}
        line["kernels"] = per_kernel

        # ---- the other configurations, each through the same stack object and CUDA graph ----
        def run_config(layer_list, batch, seq, flops_seq, dense_equiv_flops_seq=None,
                       mask_kind=0, valid_len=None, repeats=3):
            hidden = layer_list[0].hidden
            st = et.EncoderStack(layer_list, batch, seq, device=dev)
            xc = torch.from_numpy(et.synth.normal_fast(SEED, 7100 + rank, (batch * seq, hidden), 1.0)).to(dev)
            vl = None if valid_len is None else torch.from_numpy(valid_len).to(dev)
            fwd = lambda: st.forward(xc, mask_kind, None, vl)
            with torch.cuda.stream(stream):
                n0 = launch_count()
                fwd()
                launches = launch_count() - n0
                stream.synchronize()
                if args.no_graph:
                    fn = fwd
                else:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        fwd()
                    fn = g.replay
            steps = max(3, min(args.steps, 20))
            sec = med(timed(fn, steps, repeats)) / steps
            if et.device_error() != 0:
                raise SystemExit("device error in a configuration run")
            tfl = batch / sec * flops_seq * 1e-12
            r = {"batch_per_gpu": batch, "seq_len": seq, "ms_per_step": sec * 1e3,
                 "value": world * batch / sec, "unit": UNIT, "tflops_per_gpu": tfl,
                 "frac_of_burst_roofline": tfl / peaks["bf16_tflops"],
                 "gflop_per_sequence": flops_seq * 1e-9, "kernels_per_step": launches}
            if dense_equiv_flops_seq:
                r["dense_equivalent_tflops_per_gpu"] = batch / sec * dense_equiv_flops_seq * 1e-12
            del st, xc
            return r

        configs = {}
        configs["c2_b64"] = run_config(layers, 64, SEQ, flops_per_sequence())
        # the reference's own operating point: one sequence, causal mask (latency of the stack)
        configs["c2_b1_causal"] = run_config(layers, 1, SEQ, flops_per_sequence(),
                                             mask_kind=et.MASK_CAUSAL)
        configs["c2_b1_causal"]["us_per_stack_forward"] = configs["c2_b1_causal"]["ms_per_step"] * 1e3

        # C3: every Linear tile-pruned at 80 %, a quarter of each head's Q/K features removed
        kq = NHEAD * 48
        base3 = [et.synth.encoder_layer_weights(SEED, l, HIDDEN, FF, kdim=kq, vdim=HIDDEN, fast=True)
                 for l in range(LAYERS)]
        c3w = []
        for l, w in enumerate(base3):
            w = dict(w)
            for i, name in enumerate(("wqkv", "wo", "w1", "w2")):
                w[name] = et.synth.prune_tiles(w[name], SEED, 100 * (l + 1) + 50 + i, 0.8)
            c3w.append(w)
        stored = stored_tiles(c3w)
        f3 = flops_per_sequence(kdim=kq, lin_flops_per_token=512.0 * stored / LAYERS)
        f3_dense = flops_per_sequence(kdim=kq)
        c3 = {}
        for key, mode in (("tile_kernel", True), ("plan_time_choice", "auto")):
            ls = [et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev, tile_sparse=mode) for w in c3w]
            c3[key] = run_config(ls, 64, SEQ, f3, f3_dense)
            del ls
        ls = [et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev) for w in base3]
        c3["dense_same_shapes"] = run_config(ls, 64, SEQ, f3_dense)
        del ls
        for key in ("tile_kernel", "plan_time_choice"):
            c3[key]["speedup_vs_dense_same_shapes"] = \
                c3["dense_same_shapes"]["ms_per_step"] / c3[key]["ms_per_step"]
            c3[key]["speedup_vs_c2_b64"] = configs["c2_b64"]["ms_per_step"] / c3[key]["ms_per_step"]
        c3["stored_tiles_per_layer"] = stored / LAYERS
        # the same shapes at higher tile sparsity: how the tile kernels' time falls with the tiles
        sweep = {"80": {"ms_per_step": c3["tile_kernel"]["ms_per_step"],
                        "speedup_vs_dense_same_shapes": c3["tile_kernel"]["speedup_vs_dense_same_shapes"]}}
        for pct, sp in ((90, 0.9), (95, 0.95)):
            wsp = []
            for l, w in enumerate(base3):
                w = dict(w)
                for i, name in enumerate(("wqkv", "wo", "w1", "w2")):
                    w[name] = et.synth.prune_tiles(w[name], SEED, 100 * (l + 1) + 50 + i, sp)
                wsp.append(w)
            ls = [et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev, tile_sparse=True) for w in wsp]
            r = run_config(ls, 64, SEQ, flops_per_sequence(kdim=kq, lin_flops_per_token=512.0 * stored_tiles(wsp) / LAYERS),
                           f3_dense)
            sweep[str(pct)] = {"ms_per_step": r["ms_per_step"],
                               "speedup_vs_dense_same_shapes": c3["dense_same_shapes"]["ms_per_step"] / r["ms_per_step"]}
            del ls, wsp
        c3["tile_kernel_by_sparsity_pct"] = sweep
        configs["c3_b64_tile80_qk25"] = c3
        del base3, c3w

        # C5 (batch-sharded part): seq 512, global batch 256 split over the ranks
        b5 = max(1, 256 // world)
        c5 = {"global_batch": b5 * world}
        c5["dense"] = run_config(layers, b5, 512, flops_per_sequence(seq=512))
        w80 = build_weights(et, 0.8, base=ws)
        st80 = stored_tiles(w80)
        ls = [et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev, tile_sparse=True) for w in w80]
        c5["tile80_tile_kernel"] = run_config(
            ls, b5, 512, flops_per_sequence(seq=512, lin_flops_per_token=512.0 * st80 / LAYERS),
            flops_per_sequence(seq=512))
        c5["tile80_tile_kernel"]["speedup_vs_dense"] = \
            c5["dense"]["ms_per_step"] / c5["tile80_tile_kernel"]["ms_per_step"]
        del ls
        configs["c5_seq512_gb256"] = c5

        # ---- the tile-pruned stack at the headline batch: the tile kernel on packed weights, and
        # the plan-time choice between it and dense math on the expanded weights ----
        def pruned(sparsity, mode, wsp=None):
            wsp = wsp if wsp is not None else build_weights(et, sparsity, base=ws)
            stack_p = et.EncoderStack([et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev,
                                                       tile_sparse=mode) for w in wsp],
                                      BATCH, SEQ, dev)
            step_p, _ = make_step(stack_p, x_dev)
            dt_p = med(timed(step_p, args.steps, 3))
            return {"value": world * BATCH * args.steps / dt_p, "unit": UNIT,
                    "ms_per_step": dt_p / args.steps * 1e3, "speedup_vs_dense": dt / dt_p}

        line["tile_pruned_80"] = pruned(0.8, "auto", w80)
        line["tile_pruned_80"]["tile_kernel_only"] = pruned(0.8, True, w80)
        del w80
        for pct, sp in ((90, 0.9), (95, 0.95)):
            wsp = build_weights(et, sp, base=ws)
            line[f"tile_pruned_{pct}"] = pruned(sp, "auto", wsp)
            line[f"tile_pruned_{pct}"]["tile_kernel_only"] = pruned(sp, True, wsp)
            del wsp

        # C4: BERT-large, seq 384, batch 32, padding mask; dense and the mixed pruning formats
        LH, LNH, LFF, LL, LS, LB = 1024, 16, 4096, 24, 384, 32
        del layers, stack, pipe, step_fn
        torch.cuda.empty_cache()
        vl = (128 + (et.synth.uniform(SEED, 7003, LB) * 257).astype(np.int64)).clip(128, 384).astype(np.int32)
        c4 = {}
        lsd, lsf, stored_w = [], [], 0
        for l in range(LL):
            wd = et.synth.encoder_layer_weights(SEED, l, LH, LFF, fast=True)
            lsd.append(et.EncoderLayer(wd, LNH, et.ACT_GELU, device=dev))
            wf, fm = et.synth.mixed_format_layer(SEED, l, LH, LFF, fast=True)
            stored_w += sum(int(np.count_nonzero(wf[n])) for n in ("wqkv", "wo", "w1", "w2"))
            lsf.append(et.EncoderLayer(wf, LNH, et.ACT_GELU, device=dev, formats=fm))
            del wd, wf
        f4d = flops_per_sequence(seq=LS, hidden=LH, ff=LFF, layers=LL)
        f4f = flops_per_sequence(seq=LS, hidden=LH, ff=LFF, layers=LL,
                                 lin_flops_per_token=2.0 * stored_w / LL)
        c4["dense"] = run_config(lsd, LB, LS, f4d, mask_kind=et.MASK_PADDING, valid_len=vl)
        del lsd
        c4["mixed_formats"] = run_config(lsf, LB, LS, f4f, f4d, mask_kind=et.MASK_PADDING, valid_len=vl)
        c4["mixed_formats"]["speedup_vs_dense"] = c4["dense"]["ms_per_step"] / c4["mixed_formats"]["ms_per_step"]
        c4["mixed_formats"]["note"] = ("1x16 projections run as dense GEMMs on the expanded weights "
                                       "(plan-time choice); the FFN runs at the kept width")
        del lsf
        configs["c4_bert_large_b32_s384"] = c4
        torch.cuda.empty_cache()

        # C5 (head-parallel part): one 4096-token sequence over all ranks, one all-reduce per layer
        if world > 1 and hasattr(et.HeadParallelLayer, "units_of"):
            w0 = et.synth.encoder_layer_weights(SEED, 0, HIDDEN, FF, fast=True)
            hp = et.HeadParallelLayer(w0, NHEAD, job, et.ACT_GELU, device=dev)
            xl = torch.from_numpy(et.synth.normal_fast(SEED, 7200, (4096, HIDDEN), 1.0)).to(dev)
            with torch.cuda.stream(stream):
                hp.forward(xl, 1, 4096)
                stream.synchronize()
            t_layer = med(timed(lambda: hp.forward(xl, 1, 4096), 10, 3)) / 10
            t_local = med(timed(lambda: hp.forward(xl, 1, 4096, skip_allreduce=True), 10, 3)) / 10
            # the same layer with the exchange done by the library's kernels over peer memory
            # (collective set-up: fails on every rank or on none)
            t_peer, t_sp, peer_note, ex = None, None, None, None
            try:
                ex = et.PeerExchange(job, 4096, HIDDEN)
            except et.EtError as e:
                peer_note = str(e)
            if ex is not None:
                job.barrier()
                with torch.cuda.stream(stream):
                    hp.forward_peer(xl, 1, 4096, ex)
                    stream.synchronize()
                t_peer = med(timed(lambda: hp.forward_peer(xl, 1, 4096, ex), 10, 3)) / 10
                job.barrier()
                # ... and with the feed-forward block on each rank's own token rows (reduce-scatter
                # after the output projection, all-gather after the layer: one all-reduce's bytes)
                with torch.cuda.stream(stream):
                    hp.forward_peer_sharded(xl, 1, 4096, ex)
                    stream.synchronize()
                t_sp = med(timed(lambda: hp.forward_peer_sharded(xl, 1, 4096, ex), 10, 3)) / 10
                job.barrier()
            f_layer = flops_per_sequence(seq=4096, layers=1)
            best = min(t for t in (t_layer, t_peer, t_sp) if t is not None)
            configs["c5_head_parallel_b1_s4096"] = {
                "ranks": world, "work_units_per_rank": hp.units_per_rank,
                "ms_per_layer_nccl_allreduce": t_layer * 1e3,
                "ms_per_layer_peer_memory_exchange": None if t_peer is None else t_peer * 1e3,
                "ms_per_layer_peer_memory_token_sharded_ffn": None if t_sp is None else t_sp * 1e3,
                "peer_memory_exchange_note": peer_note,
                "ms_per_layer_without_exchange": t_local * 1e3,
                "exchange_share_nccl": max(0.0, 1.0 - t_local / t_layer),
                "exchange_share_peer_memory": None if t_peer is None else max(0.0, 1.0 - t_local / t_peer),
                "tflops_all_ranks": f_layer / best * 1e-12,
                "frac_of_burst_roofline": f_layer / best * 1e-12 / (world * peaks["bf16_tflops"]),
                "sequences_per_s_12_layers": 1.0 / (best * LAYERS),
                "device_error": et.device_error()}
            if ex is not None:
                ex.close()
        line["configs"] = configs

        # ---- CPU baseline and parity of the benchmarked stack (rank 0, N = 1 only) ----
        if world == 1:
            orc = entry.load_oracle()
            orc.build()
            orc.set_num_threads(len(os.sched_getaffinity(0)))
            cx = x_host.numpy().astype(np.float32)
            best, cur = float("inf"), None
            for _ in range(2):
                t0 = time.perf_counter()
                cur = cx
                for w in ws:
                    cur = orc.encoder_layer(cur, w, BATCH, SEQ, NHEAD, 2, 0)
                best = min(best, time.perf_counter() - t0)
            # the oracle as checker: the whole benchmarked stack, at the benchmarked shape
            layers = [et.EncoderLayer(w, NHEAD, et.ACT_GELU, device=dev) for w in ws]
            one = et.EncoderStack(layers, BATCH, SEQ, device=dev)
            with torch.cuda.stream(stream):
                gy = one.forward(x_dev).float()
                stream.synchronize()
            gy = gy.cpu().numpy()
            ref = np.asarray(cur, dtype=np.float32)
            rel = float(np.linalg.norm(gy - ref) / np.linalg.norm(ref))
            mx = float(np.abs(gy - ref).max())
            line["parity"] = {"rel_l2": rel, "max_abs": mx, "tolerance": [5e-3, 2e-2],
                              "what": f"output of the benchmarked {LAYERS}-layer stack on {BATCH} "
                                      "sequences against the CPU oracle (fp32)"}
            if not (rel <= 5e-3 and mx <= 2e-2) or et.device_error() != 0:
                raise SystemExit(f"parity check failed: rel-L2 {rel:.3e}, max-abs {mx:.3e}")
            line["cpu_baseline"] = {"value": BATCH / best, "unit": UNIT, "cores": orc.num_threads(),
                                    "kind": "port",
                                    "sample": f"best of 2 runs of the full {LAYERS}-layer stack over "
                                              f"{BATCH} sequences ({best:.2f} s each)"}

    # ---- the reference's own CUDA build (recompiled for sm_100a), reported alongside: its
    # paper-table driver at batch 1, seq 128, 12 layers.  Run last, in a process of its own.
    if not args.skip_extras and world == 1:
        import subprocess
        ref_bin = os.path.join(ROOT, "oracle", "_ref", "ref_table2")
        if os.path.exists(ref_bin):
            try:
                r = subprocess.run([ref_bin, str(LAYERS), "0.8"], capture_output=True, text=True,
                                   timeout=180)
                last = [l for l in r.stdout.splitlines() if l.startswith("{")]
                rec = json.loads(last[-1]) if last else {"unavailable": f"no result line (exit {r.returncode})"}
                rec["exit_code"] = r.returncode
            except Exception as e:  # timeout, missing libraries ...
                rec = {"unavailable": f"{type(e).__name__}: {e}"}
        else:
            rec = {"unavailable": "oracle/_ref/ref_table2 not built (needs the reference checkout at build time)"}
        rec["note"] = ("the reference's kernels, cuBLAS calls and host classes compiled unmodified; "
                       "constant weights, causal mask, batch 1; outputs not validated")
        if "configs" in line and "c2_b1_causal" in line["configs"]:
            rec["this_library_us_same_shape"] = line["configs"]["c2_b1_causal"]["us_per_stack_forward"]
        line["reference_cuda"] = rec

    sampler.stop()
    line["clocks"] = sampler.summary()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

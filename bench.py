#!/usr/bin/env python
"""Decoder-layer benchmark (one JSON line on stdout).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload prefill|decode]

Workload (default): the Llama-3-8B-shaped dense decoder layer in bf16, prefill batch 4 x
sequence 2048 (8192 tokens per step), tensor parallel over the N GPUs of one node with an NCCL
all-reduce after the O and Down projections.  A "step" is one pass of the layer.

  value   whole-job tokens/s with the layer input already resident in HBM (kernels + collectives)
  e2e     the same metric through the host-buffer plan call (sfb_decoder_execute): pinned host
          input -> device, layer, device -> pinned host output, every step
  roofline   the dominant kernel (fused gate/up tcgen05 GEMM) timed live with CUDA events
  cpu_baseline  the reference's own native CPU path (or the oracle port when the reference build
          is absent) on a bounded sample of the same layer, rank 0, N == 1 only

`--impl reference` times the reference's CPU implementation instead (rank 0 only).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA = dict(hidden=4096, intermediate=14336, query_heads=32, kv_heads=8, head_dim=128, rms_epsilon=1e-5,
             rope_theta=500000.0)
PREFILL = dict(batch=4, sequence=2048)
DECODE = dict(batch=128, sequence=1, context_sequence=2048)
CPU_SAMPLE = dict(batch=1, sequence=384)  # bounded sample of the prefill workload for the CPU arms


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def make_weights(seed, cfg, with_cache=False):
    """Synthetic weights ~N(0, 0.02), RMSNorm weights 1, cached K/V ~N(0,1); seeded, on the host."""
    import torch
    g = torch.Generator().manual_seed(seed)
    h, i = cfg["hidden"], cfg["intermediate"]
    kv = cfg["kv_heads"] * cfg["head_dim"]
    shapes = dict(query_weight=(h, h), key_weight=(h, kv), value_weight=(h, kv), output_weight=(h, h),
                  gate_weight=(h, i), up_weight=(h, i), down_weight=(i, h))
    data = {k: (torch.randn(s, generator=g) * 0.02).numpy() for k, s in shapes.items()}
    data["rms1_weight"] = np.ones(h, np.float32)
    data["rms2_weight"] = np.ones(h, np.float32)
    if with_cache:
        n = (cfg["batch"], cfg["kv_heads"], cfg["context_sequence"], cfg["head_dim"])
        data["cached_key"] = torch.randn(n, generator=g).numpy()
        data["cached_value"] = torch.randn(n, generator=g).numpy()
    return data


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = sorted(sm)[len(sm) // 2:]  # upper half of the samples = the ones taken under load
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_arm(steps, warmup, cfg_sample):
    """The reference's own CPU implementation (oracle/_ref) or the oracle port on a bounded sample."""
    from oracle import binding as ob
    cfg = dict(LLAMA, **cfg_sample)
    oc = ob.decoder_config(**cfg)
    data = make_weights(0, cfg)
    import torch
    t = cfg["batch"] * cfg["sequence"]
    x = torch.randn((t, cfg["hidden"]), generator=torch.Generator().manual_seed(1)).numpy()
    port = ob.Port()
    for k in data:
        data[k] = port.round_bf16(data[k])
    data["input"] = port.round_bf16(x)
    times = []
    if ob.Ref.available():
        ref = ob.Ref()
        cores = ref.hardware_threads()
        dec = ref.decoder_create(oc, data, threads=cores)
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            dec.execute_once()
            if i >= warmup:
                times.append(time.perf_counter() - t0)
        dec.close()
        kind = "reference"
    else:
        cores = port.hardware_threads()
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            port.decoder_layer(oc, data, native=True, threads=cores)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
        kind = "port"
    ms = 1000.0 * float(np.mean(times))
    return {"value": t * 1000.0 / ms, "unit": "tokens/s", "cores": cores, "kind": kind, "ms_per_step": ms,
            "sample": f"same layer, bf16-rounded weights, fp32 CPU arithmetic, B{cfg['batch']}xS{cfg['sequence']} "
                      f"= {t} tokens per step ({steps} timed step(s) after {warmup} warm-up)"}


def kernel_case(args):
    """One kernel of the hot path, timed with CUDA events on its launching stream.

    gemm       the fused gate/up projection (tcgen05, SwiGLU epilogue), Llama-3-8B shape
               (--small: M=4096, N=16384, K=4096, 224 MB of operands, larger than L2)
    gemm_decode  the same projection for the 128 rows of a decode step: blocked weights, streamed
               once (--small: N=8192; three weight copies are rotated so that L2 does not help)
    attention  headline attention case: causal GQA prefill B4 Hq32 Hkv8 S4096 D128 (--small: B1; --head-dim 64)
    decode     headline decode case: paged split-KV decode, batch 64, context ~U[512, 8192], 16-token
               blocks, permuted block table (--small: batch 16)
    """
    import torch
    from schedforge_b200 import lib as L
    lib = L.load()
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(0)
    cur = torch.cuda.current_stream()
    sp = C.c_void_p(cur.cuda_stream)
    keep = []
    if args.kernel == "gemm":
        m, n, k = (4096, 16384, 4096) if args.small else (8192, 28672, 4096)
        a = (torch.randn((m, k), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        bt = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
        o = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        g = L.GemmArgs()
        g.a, g.bt, g.out, g.m, g.n, g.k = a.data_ptr(), bt.data_ptr(), o.data_ptr(), m, n, k
        g.epilogue, g.backend, g.swiglu_block = L.EPI_SWIGLU, L.GEMM_TCGEN05, 128
        launch = lambda: L.check(lib.sfb_k_gemm_bf16(C.byref(g), sp))
        work, unit, peak, bound = 2.0 * m * n * k, "TFLOP/s", peaks["bf16_tflops"], "tensor"
        name, shape = "gemm_tcgen05_kernel<256>", {"m": m, "n": n, "k": k, "epilogue": "swiglu"}
    elif args.kernel == "gemm_decode":
        # gate/up projection of the decode step: 128 rows, every weight byte read once (HBM-bound)
        m, n, k = 128, (8192 if args.small else 28672), 4096
        a = (torch.randn((m, k), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        copies = 3  # rotate over weight copies larger than L2 together
        o = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        nbytes = lib.sfb_gemm_stream_workspace_bytes(n)
        scratch = torch.zeros((nbytes // 4,), dtype=torch.float32, device="cuda")
        gs = []
        for _ in range(copies):
            bt = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
            tiled = torch.empty((lib.sfb_tiled_weight_elems(n, k),), dtype=torch.bfloat16, device="cuda")
            L.check(lib.sfb_k_tile_weight_bf16(C.c_void_p(bt.data_ptr()), C.c_void_p(tiled.data_ptr()), n, k, sp))
            torch.cuda.synchronize()
            g = L.GemmArgs()
            g.a, g.bt, g.out, g.m, g.n, g.k = a.data_ptr(), tiled.data_ptr(), o.data_ptr(), m, n, k
            g.epilogue, g.backend, g.swiglu_block, g.bt_tiled = L.EPI_SWIGLU, L.GEMM_TCGEN05, 64, 1
            g.split_workspace, g.split_workspace_bytes = scratch.data_ptr(), nbytes
            gs.append(g)
            keep.append(tiled)
        keep.append(scratch)
        turn = [0]

        def launch():
            L.check(lib.sfb_k_gemm_bf16(C.byref(gs[turn[0] % copies]), sp))
            turn[0] += 1
        work = float(n * k * 2 + m * k * 2 + m * (n // 2) * 2)
        unit, peak, bound = "GB/s", peaks["hbm_gbs"], "hbm"
        name, shape = "gemm_tcgen05_kernel<128, true>", {"m": m, "n": n, "k": k, "epilogue": "swiglu", "weights": "64x64 blocks"}
    elif args.kernel == "attention":
        b, hq, hkv, s, d = (1 if args.small else 4), 32, 8, 4096, args.head_dim
        q = torch.randn((b, hq, s, d), generator=gen, device="cuda").to(torch.bfloat16)
        kk = torch.randn((b, hkv, s, d), generator=gen, device="cuda").to(torch.bfloat16)
        v = torch.randn((b, hkv, s, d), generator=gen, device="cuda").to(torch.bfloat16)
        o = torch.empty((b, hq, s, d), dtype=torch.bfloat16, device="cuda")
        a = L.AttentionArgs(q.data_ptr(), kk.data_ptr(), v.data_ptr(), o.data_ptr(), b, hq, hkv, s, s, d, d, 1,
                            0.0, 0, L.BF16, 2)
        launch = lambda: L.check(lib.sfb_k_attention_prefill(C.byref(a), sp))
        pairs = b * hq * s * (s + 1) / 2
        work, unit, peak, bound = 2.0 * pairs * 2 * d, "TFLOP/s", peaks["bf16_tflops"], "tensor"
        name, shape = f"attention_prefill_tcgen05_kernel<{d}>", {"batch": b, "q_heads": hq, "kv_heads": hkv, "seq": s, "head_dim": d, "causal": True}
    else:
        batch, hq, hkv, d, block = (16 if args.small else 64), 32, 8, 128, 16
        ctx = torch.randint(512, 8193, (batch,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
        blocks_per = (ctx + block - 1) // block
        max_blocks = 8192 // block
        num_blocks = int(blocks_per.sum()) + 8
        perm = torch.randperm(num_blocks, generator=torch.Generator().manual_seed(1), dtype=torch.int32)
        table = torch.zeros((batch, max_blocks), dtype=torch.int32)
        cursor = 0
        for i in range(batch):
            nb = int(blocks_per[i])
            table[i, :nb] = perm[cursor:cursor + nb]
            cursor += nb
        k_pool = torch.randn((num_blocks, hkv, block, d), generator=gen, device="cuda").to(torch.bfloat16)
        v_pool = torch.randn((num_blocks, hkv, block, d), generator=gen, device="cuda").to(torch.bfloat16)
        q = torch.randn((batch, hq, d), generator=gen, device="cuda").to(torch.bfloat16)
        o = torch.empty((batch, hq, d), dtype=torch.bfloat16, device="cuda")
        dtab, dctx = table.cuda(), ctx.cuda()
        splits = lib.sfb_attention_decode_default_splits(batch, hkv, 8192)
        part = torch.empty((lib.sfb_attention_decode_workspace(batch, hq, d, splits) // 4,), dtype=torch.float32, device="cuda")
        a = L.DecodeArgs(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), dtab.data_ptr(), dctx.data_ptr(), o.data_ptr(),
                         part.data_ptr(), batch, hq, hkv, d, d, block, max_blocks, num_blocks, 8192, splits, 0.0, L.BF16)
        keep += [dtab, dctx, part]
        launch = lambda: L.check(lib.sfb_k_attention_decode_paged(C.byref(a), sp))
        total_ctx = int(ctx.sum())
        work = total_ctx * hkv * (2 * d) * 2 + 2 * batch * hq * d * 2 + int(blocks_per.sum()) * 4
        unit, peak, bound = "GB/s", peaks["hbm_gbs"], "hbm"
        name = "decode_paged_mma_kernel<4> + decode_combine_kernel"
        shape = {"batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d, "block_tokens": block,
                 "total_context": total_ctx, "splits": splits}
    for _ in range(args.warmup):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(cur)
    for _ in range(args.steps):
        launch()
    e1.record(cur)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    achieved = work / (ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)
    print(json.dumps({"kernel": name, "shape": shape, "steps": args.steps, "warmup": args.warmup, "kernel_ms": ms,
                      "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                                   "peak_source": peaks["source"], "algorithmic_work_per_launch": work}}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode", "moe"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "int8"],
                    help="int8: per-output-channel weight-only INT8 (the reference's quantized layer); not the default")
    ap.add_argument("--collective", default="auto", choices=["auto", "nccl", "peer"],
                    help="N > 1: all-reduce after the O and Down projections through NCCL, or fused into the GEMM "
                         "epilogues over NVLink peer memory")
    ap.add_argument("--kernel", default="", choices=["", "gemm", "gemm_decode", "attention", "decode"],
                    help="time ONE kernel through the kernel ABI instead of the layer (also the ncu target)")
    ap.add_argument("--head-dim", type=int, default=128, choices=[128, 64], help="--kernel attention: head dimension")
    ap.add_argument("--small", action="store_true", help="--kernel: a case small enough for an ncu --set full capture")
    args = ap.parse_args()
    if args.kernel:
        return kernel_case(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    shape = DECODE if args.workload == "decode" else PREFILL
    cfg = dict(LLAMA, **shape)
    if args.workload == "moe":  # Mixtral-shaped layer: 8 experts, top-2, expert FFN 14336, 8192 tokens
        cfg.update(moe=True, experts=8, top_k=2)
    tokens = cfg["batch"] * cfg["sequence"]
    workload = {"prefill": "llama3_8b_decoder_layer_prefill_b4_s2048",
                "decode": "llama3_8b_decoder_layer_decode_b128_ctx2048",
                "moe": "mixtral_moe_decoder_layer_8x_top2_t8192"}[args.workload]
    config = {"workload": workload, "hidden": 4096, "intermediate": 14336, "q_heads": 32, "kv_heads": 8,
              "head_dim": 128, "tokens_per_step": tokens, "parallelism": f"tp{world}", "collective": "none",
              "l2": "weights + activations (>0.9 GB per step) exceed the 126 MB L2; no flush between steps"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        base = cpu_arm(max(1, min(args.steps, 3)), min(args.warmup, 1), CPU_SAMPLE)
        line = {"impl": "reference", "metric": "decoder_layer_tokens_per_s", "value": base["value"], "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist
    from schedforge_b200 import api, lib as L

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = L.load()

    data = make_weights(0, cfg, with_cache=args.workload == "decode")
    if args.workload == "moe":
        g = torch.Generator().manual_seed(7)
        h, i, e = cfg["hidden"], cfg["intermediate"], cfg["experts"]
        for key in ("gate_weight", "up_weight", "down_weight"):
            data.pop(key)
        data["router_weight"] = (torch.randn((h, e), generator=g) * 0.02).numpy()
        data["router_bias"] = torch.randn(e, generator=g).numpy()  # per-expert bias: skewed expert loads
        for key, shape_ in (("w1", (e, h, i)), ("w3", (e, h, i)), ("w2", (e, i, h))):
            data[key] = torch.empty(shape_).normal_(0.0, 0.02, generator=g).numpy()
    x_host = torch.randn((tokens, cfg["hidden"]), generator=torch.Generator().manual_seed(1)).pin_memory()
    out_host = torch.empty((tokens, cfg["hidden"]), dtype=torch.float32).pin_memory()
    c = api.decoder_config(**cfg)
    plan = api.DecoderCompiler.compile(c, data, "", api.compile_options(tp_rank=rank, tp_size=world,
                                                                         seed_block_table=1 if args.workload == "decode" else 0,
                                                                         weight_int8=args.weights == "int8"))
    config["weights"] = args.weights
    del data
    stream = torch.cuda.ExternalStream(plan.stream)
    views = {}

    def allreduce(buf, count, dtype, stream_ptr):
        key = (buf, count)
        if key not in views:
            class Raw:  # CUDA array interface over the plan's workspace (int16 view of the bf16 data)
                __cuda_array_interface__ = {"shape": (count,), "typestr": "<i2", "data": (buf, False), "version": 3}
            views[key] = torch.as_tensor(Raw(), device="cuda").view(torch.bfloat16)
        with torch.cuda.stream(stream):
            dist.all_reduce(views[key])

    collective = "none"
    if world > 1:
        plan.set_allreduce(allreduce)
        collective = args.collective
        if collective == "auto":  # one-shot pushes cost (N-1) x bytes per rank: two ranks, or the small decode outputs
            collective = "peer" if (world == 2 or args.workload == "decode") and args.workload != "moe" else "nccl"
        if collective == "peer":
            def exchange(handle):
                handles = [None] * world
                dist.all_gather_object(handles, handle)
                return handles
            plan.enable_peer_allreduce(rank, world, exchange)
            dist.barrier()
    config["collective"] = {"none": "none", "nccl": "nccl all-reduce after O and Down",
                            "peer": "all-reduce fused into the O and Down GEMM epilogues over NVLink peer memory"}[collective]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: input resident, kernels (+ collectives) only ------------------------------------
    plan.upload_input(x_host.numpy())
    for _ in range(args.warmup):
        plan.execute_resident()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.sfb_launch_count()
    start.record(stream)
    for _ in range(args.steps):
        plan.execute_resident()
    stop.record(stream)
    barrier()
    launches = lib.sfb_launch_count() - launches0
    ms = start.elapsed_time(stop) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # ---- e2e: host buffers through the plan call ------------------------------------------------
    # With several ranks every rank brings and takes its own rows (sfb_decoder_execute_rows): the whole job
    # still moves the full input and output between host and device each step, 1/N of it per PCIe link.
    sharded_io = world > 1 and tokens % world == 0
    if sharded_io:
        rows = tokens // world
        row0 = rank * rows
        x_rows, out_rows = x_host[row0:row0 + rows], out_host[row0:row0 + rows]

        def e2e_step(result=None):
            plan.execute_rows_ptr(x_rows.data_ptr(), out_rows.data_ptr(), row0, rows, result)
    else:
        def e2e_step(result=None):
            plan.execute_ptr(x_host.data_ptr(), out_host.data_ptr(), result)
    config["e2e_io"] = "each rank copies its 1/N of the rows; all-reduce hook gathers the input" if sharded_io \
        else "whole input and output on every rank"
    for _ in range(min(args.warmup, 3)):
        e2e_step()
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = 1000.0 * (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    result = L.DecoderResult()
    e2e_step(result)
    clocks = sampler.stop() if rank == 0 else None
    finite = bool(torch.isfinite(out_rows if sharded_io else out_host).all())

    # ---- roofline of the dominant kernel, timed live on its launching stream --------------------
    peaks = measured_peaks()
    roofline = None
    if args.workload == "prefill":
        m, k, n = tokens, cfg["hidden"], 2 * cfg["intermediate"] // world
        a = (torch.randn((m, k), device="cuda") * 0.5).to(torch.bfloat16)
        bt = (torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16)
        o = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        g = L.GemmArgs()
        g.a, g.bt, g.out, g.m, g.n, g.k = a.data_ptr(), bt.data_ptr(), o.data_ptr(), m, n, k
        g.epilogue, g.backend, g.swiglu_block = L.EPI_SWIGLU, L.GEMM_TCGEN05, 128
        cur = torch.cuda.current_stream()
        for _ in range(3):
            L.check(lib.sfb_k_gemm_bf16(C.byref(g), C.c_void_p(cur.cuda_stream)))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(cur)
        for _ in range(reps):
            L.check(lib.sfb_k_gemm_bf16(C.byref(g), C.c_void_p(cur.cuda_stream)))
        e1.record(cur)
        torch.cuda.synchronize()
        kernel_ms = e0.elapsed_time(e1) / reps
        flops = 2.0 * m * n * k
        achieved = flops / (kernel_ms * 1e-3) / 1e12
        roofline = {"kernel": "gemm_tcgen05_kernel<256, false> (gate/up projection, SwiGLU epilogue)", "bound": "tensor",
                    "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst: kernel timed alone)",
                    "kernel_ms": kernel_ms, "algorithmic_flops_per_launch": flops,
                    # dram read + write of one launch: 359.4 MB measured by ncu on the M4096 N16384 case (2048 output
                    # tiles), scaled by the tile count of this launch; B is re-read once per band of 16 M-tiles
                    "traffic": 359.4e6 * ((m + 127) // 128) * ((n + 255) // 256) / 2048.0,
                    "traffic_source": "ncu dram__bytes_read+write of the --kernel gemm --small capture, scaled by output tiles"}
    elif args.workload == "moe":
        flops = 6.0 * tokens * cfg["top_k"] * cfg["hidden"] * cfg["intermediate"] / world
        achieved = flops / (result.ffn_milliseconds * 1e-3) / 1e12 if result.ffn_milliseconds > 0 else None
        roofline = {"kernel": "gemm_tcgen05_kernel<256> grouped mode (experts W3|W1 + SwiGLU, then W2), timed with the "
                              "routing chain around it (router, dispatch, combine)", "bound": "tensor",
                    "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops_sustained"] if achieved else None,
                    "peak_source": peaks["source"] + " (sustained: timed inside the layer step)",
                    "kernel_ms": result.ffn_milliseconds, "algorithmic_flops_per_launch": flops, "traffic": None}
    else:
        kv_bytes = cfg["batch"] * cfg["context_sequence"] * (cfg["kv_heads"] // world) * cfg["head_dim"] * 2 * 2
        roofline = {"kernel": "decode_paged_mma_kernel<4> + combine (inside the layer)", "bound": "hbm", "achieved": kv_bytes / (result.attention_milliseconds * 1e-3) / 1e9
                    if result.attention_milliseconds > 0 else None, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": (kv_bytes / (result.attention_milliseconds * 1e-3) / 1e9 / peaks["hbm_gbs"])
                    if result.attention_milliseconds > 0 else None, "peak_source": peaks["source"],
                    "kernel_ms": result.attention_milliseconds, "algorithmic_bytes_per_launch": kv_bytes,
                    # ncu on the batch-16 case: 307.0 MB of dram traffic for 301.2 MB of K/V pages (every byte once)
                    "traffic": kv_bytes * 307.0 / 301.2,
                    "traffic_source": "ncu dram__bytes_read+write of the --kernel decode --small capture, scaled by K/V bytes"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload == "prefill":
        base = cpu_arm(1, 1, CPU_SAMPLE)
        cpu = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if world > 1:
        dist.barrier()
    if rank == 0:
        line = {"metric": "decoder_layer_tokens_per_s", "value": tokens * 1000.0 / ms, "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": config,
                "e2e": {"value": tokens * 1000.0 / e2e_ms, "unit": "tokens/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": tokens * cfg["hidden"] * 4, "d2h_bytes_per_step": tokens * cfg["hidden"] * 4},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
                "stages_ms": {"attention": result.attention_milliseconds, "projection": result.projection_milliseconds,
                              "norm": result.norm_rope_milliseconds, "ffn": result.ffn_milliseconds,
                              "h2d": result.h2d_milliseconds, "d2h": result.d2h_milliseconds},
                "output_finite": finite}
        print(json.dumps(line))
    plan.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

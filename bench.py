#!/usr/bin/env python
"""Decoder-layer benchmark (one JSON line on stdout).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload prefill|decode|moe]

Headline workload (default): the Llama-3-8B-shaped dense decoder layer in bf16, prefill batch 4 x
sequence 2048 (8192 tokens per step), tensor parallel over the N GPUs of one node.  A "step" is one pass
of the layer.

  value   whole-job tokens/s with the layer input already resident in HBM (kernels + collectives)
  e2e     the same metric through the host-buffer plan call (sfb_decoder_execute): pinned host
          input -> device, layer, device -> pinned host output, every step
  roofline   the dominant kernel (fused gate/up tcgen05 GEMM) timed live with CUDA events
  cpu_baseline  the reference's own native CPU path (or the oracle port when the reference build
          is absent) on a bounded sample of the same layer, rank 0, N == 1 only
  parity  the device plan (sharded like the run) on that same bounded sample against the CPU output
  decode / moe / kernels   sub-records of the same line: the decode half of the metric (batch 128 over
          2048 cached tokens), the Mixtral-shaped MoE layer (8192 tokens), and the two stand-alone kernel
          cases (causal GQA prefill attention B4 S4096; paged split-KV decode, batch 64), each with its own
          timing, roofline and clocks

`--impl reference` times the reference's CPU implementation instead (rank 0 only).
`--workload decode|moe` makes that workload the headline and prints no sub-records.
`--kernel ...` times ONE kernel through the kernel ABI (also the command ncu captures).
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
SHAPES = {"prefill": dict(batch=4, sequence=2048),
          "decode": dict(batch=128, sequence=1, context_sequence=2048),
          "moe": dict(batch=4, sequence=2048, moe=True, experts=8, top_k=2)}
NAMES = {"prefill": "llama3_8b_decoder_layer_prefill_b4_s2048",
         "decode": "llama3_8b_decoder_layer_decode_b128_ctx2048",
         "moe": "mixtral_moe_decoder_layer_8x_top2_t8192"}
CPU_SAMPLE = dict(batch=1, sequence=384)  # bounded sample of the prefill workload for the CPU arms
CPU_WALL_BUDGET_S = 150.0                 # the reference arm stops adding timed steps beyond this


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def make_weights(seed, cfg, with_cache=False):
    """Synthetic dense-layer weights ~N(0, 0.02), RMSNorm weights 1, cached K/V ~N(0,1); seeded, on the host."""
    import torch
    g = torch.Generator().manual_seed(seed)
    h, i = cfg["hidden"], cfg["intermediate"]
    kv = cfg["kv_heads"] * cfg["head_dim"]
    shapes = dict(query_weight=(h, h), key_weight=(h, kv), value_weight=(h, kv), output_weight=(h, h))
    if not cfg.get("moe"):
        shapes.update(gate_weight=(h, i), up_weight=(h, i), down_weight=(i, h))
    data = {k: (torch.randn(s, generator=g) * 0.02).numpy() for k, s in shapes.items()}
    data["rms1_weight"] = np.ones(h, np.float32)
    data["rms2_weight"] = np.ones(h, np.float32)
    if with_cache:
        n = (cfg["batch"], cfg["kv_heads"], cfg["context_sequence"], cfg["head_dim"])
        data["cached_key"] = torch.randn(n, generator=g).numpy()
        data["cached_value"] = torch.randn(n, generator=g).numpy()
    return data


def add_expert_weights(data, cfg, rank, world):
    """Router ~N(0, 0.02) with a per-expert bias ~N(0, 1) (skewed loads) and THIS rank's experts ~N(0, 0.02),
    one seed per expert so that every rank count sees the same layer."""
    import torch
    h, i, e = cfg["hidden"], cfg["intermediate"], cfg["experts"]
    g = torch.Generator().manual_seed(7)
    data["router_weight"] = (torch.randn((h, e), generator=g) * 0.02).numpy()
    data["router_bias"] = torch.randn(e, generator=g).numpy()
    local = e // world
    for key, shape in (("w1", (h, i)), ("w3", (h, i)), ("w2", (i, h))):
        block = torch.empty((local,) + shape)
        for j in range(local):
            ge = torch.Generator().manual_seed(1000 + 10 * (rank * local + j) + len(key) + ord(key[1]))
            block[j].normal_(0.0, 0.02, generator=ge)
        data[key] = block.numpy()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run.  Every sample is
    stamped on arrival; the summary is the median over ALL samples that fall inside the marked regions."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.samples = []   # (arrival time, fields)
        self.regions = []   # (begin, end) of timed regions, host clock

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def mark(self, begin, end):
        self.regions.append((begin, end))

    def summary(self, regions=None):
        regions = self.regions if regions is None else regions
        inside, everything, reasons_inside, reasons_all = [], [], set(), set()
        smax = []
        for stamp, line in list(self.samples):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm = float(f[1])
                smax.append(float(f[2]))
            except ValueError:
                continue
            active = {name for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9])
                      if val.lower().startswith("active")}
            everything.append(sm)
            reasons_all |= active
            if any(b <= stamp <= e + 0.03 for b, e in regions):  # a sample describes the ~20 ms before it arrives
                inside.append(sm)
                reasons_inside |= active
        if not everything:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if len(inside) >= 3:
            return {"sm_mhz": float(np.median(inside)), "sm_min_mhz": float(min(inside)), "sm_max_mhz": max(smax),
                    "reasons": sorted(reasons_inside), "samples": len(inside), "window": "timed regions"}
        return {"sm_mhz": float(np.median(everything)), "sm_min_mhz": float(min(everything)), "sm_max_mhz": max(smax),
                "reasons": sorted(reasons_all), "samples": len(everything),
                "window": "whole run (fewer than 3 samples fell inside the timed regions)"}

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return self.summary()


def cpu_arm(steps, warmup, cfg_sample, wall_budget=None, want_output=False):
    """The reference's own CPU implementation (oracle/_ref) or the oracle port on a bounded sample."""
    from oracle import binding as ob
    import torch
    cfg = dict(LLAMA, **cfg_sample)
    oc = ob.decoder_config(**cfg)
    data = make_weights(0, cfg)
    t = cfg["batch"] * cfg["sequence"]
    x = torch.randn((t, cfg["hidden"]), generator=torch.Generator().manual_seed(1)).numpy()
    port = ob.Port()
    for k in data:
        data[k] = port.round_bf16(data[k])
    data["input"] = port.round_bf16(x)
    times, out = [], None
    begin = time.perf_counter()
    if ob.Ref.available():
        ref = ob.Ref()
        cores = ref.hardware_threads()
        dec = ref.decoder_create(oc, data, threads=cores)
        run = lambda: dec.execute_once()[0]
        kind = "reference"
    else:
        dec = None
        cores = port.hardware_threads()
        run = lambda: port.decoder_layer(oc, data, native=True, threads=cores)
        kind = "port"
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out = run()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
            if wall_budget is not None and time.perf_counter() - begin > wall_budget:
                break
    if dec is not None:
        dec.close()
    ms = 1000.0 * float(np.mean(times))
    record = {"value": t * 1000.0 / ms, "unit": "tokens/s", "cores": cores, "kind": kind, "ms_per_step": ms,
              "steps_timed": len(times), "warmup": warmup, "tokens_per_step": t,
              "sample": f"same layer, bf16-rounded weights, fp32 CPU arithmetic, B{cfg['batch']}xS{cfg['sequence']} "
                        f"= {t} tokens per step ({len(times)} timed step(s) after {warmup} warm-up)"}
    if want_output:
        record["_output"], record["_data"] = out, data
    return record


def time_kernel(kernel, small, head_dim, steps, warmup):
    """One kernel of the hot path, timed with CUDA events on its launching stream.

    gemm       the fused gate/up projection (tcgen05, SwiGLU epilogue), Llama-3-8B shape
               (small: M=4096, N=16384, K=4096, 224 MB of operands, larger than L2)
    gemm_shard the O projection of one shard of an 8-way tensor-parallel plan: M=8192, N=4096, K=512, plain store of
               the partial sums (three rotated outputs of 67 MB; the short K loop leaves the epilogue in charge)
    gemm_decode  the same projection for the 128 rows of a decode step: blocked weights, streamed
               once (small: N=8192; three weight copies are rotated so that L2 does not help)
    attention  headline attention case: causal GQA prefill B4 Hq32 Hkv8 S4096 D128 (small: B1; head_dim 64)
    decode     headline decode case: paged split-KV decode, batch 64, context ~U[512, 8192], 16-token
               blocks, permuted block table (small: batch 16)
    """
    import torch
    from schedforge_b200 import lib as L
    lib = L.load()
    peaks = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(0)
    cur = torch.cuda.current_stream()
    sp = C.c_void_p(cur.cuda_stream)
    keep = []
    if kernel == "gemm":
        m, n, k = (4096, 16384, 4096) if small else (8192, 28672, 4096)
        a = (torch.randn((m, k), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        bt = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
        o = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        g = L.GemmArgs()
        g.a, g.bt, g.out, g.m, g.n, g.k = a.data_ptr(), bt.data_ptr(), o.data_ptr(), m, n, k
        g.epilogue, g.backend, g.swiglu_block = L.EPI_SWIGLU, L.GEMM_TCGEN05, 128
        launch = lambda: L.check(lib.sfb_k_gemm_bf16(C.byref(g), sp))
        work, unit, peak, bound = 2.0 * m * n * k, "TFLOP/s", peaks["bf16_tflops"], "tensor"
        name, shape = "gemm_tcgen05_kernel<256>", {"m": m, "n": n, "k": k, "epilogue": "swiglu"}
        l2 = "operands (0.3 GB) exceed the 126 MB L2"
    elif kernel == "gemm_shard":
        m, n, k = 8192, 4096, 512
        a = (torch.randn((m, k), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        bt = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
        outs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        gs = []
        for o in outs:
            g = L.GemmArgs()
            g.a, g.bt, g.out, g.m, g.n, g.k = a.data_ptr(), bt.data_ptr(), o.data_ptr(), m, n, k
            g.epilogue, g.backend = L.EPI_STORE, L.GEMM_TCGEN05
            gs.append(g)
        keep += outs
        turn = [0]

        def launch():
            turn[0] += 1
            L.check(lib.sfb_k_gemm_bf16(C.byref(gs[turn[0] % 3]), sp))
        # memory-bound by its output: A and B once, the bf16 result once
        work, unit, peak, bound = (m * k + n * k + m * n) * 2, "GB/s", peaks["hbm_gbs"], "hbm"
        name, shape = "gemm_tcgen05_kernel<256>", {"m": m, "n": n, "k": k, "epilogue": "store"}
        l2 = "three outputs of 67 MB are rotated (201 MB, larger than L2)"
    elif kernel == "gemm_decode":
        # gate/up projection of the decode step: 128 rows, every weight byte read once (HBM-bound)
        m, n, k = 128, (8192 if small else 28672), 4096
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
        l2 = "three weight copies rotated (larger than L2 together)"
    elif kernel == "attention":
        b, hq, hkv, s, d = (1 if small else 4), 32, 8, 4096, head_dim
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
        l2 = "Q, K, V, O of one launch are 0.34 GB (B4), larger than L2"
    else:
        batch, hq, hkv, d, block = (16 if small else 64), 32, 8, 128, 16
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
        name = "decode_paged_mma_kernel<4> + decode_combine_warp_kernel"
        shape = {"batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d, "block_tokens": block,
                 "total_context": total_ctx, "splits": splits}
        l2 = "K/V pages of one launch (1.1 GB at batch 64) exceed L2"
    for _ in range(warmup):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(cur)
    for _ in range(steps):
        launch()
    e1.record(cur)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1) / steps
    achieved = work / (ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)
    return {"kernel": name, "shape": shape, "steps": steps, "warmup": warmup, "kernel_ms": ms, "l2": l2,
            "roofline": {"kernel": name, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                         "frac": achieved / peak, "peak_source": peaks["source"] + " (burst: kernel timed alone)",
                         "algorithmic_work_per_launch": work},
            "_region": (t0, t1)}


class Layer:
    """One workload as a (possibly sharded) device plan with its pinned host buffers and collective."""

    def __init__(self, workload, args, rank, world, cfg_override=None, data=None, x=None):
        import torch
        import torch.distributed as dist
        from schedforge_b200 import api
        self.workload, self.rank, self.world = workload, rank, world
        cfg = dict(LLAMA, **SHAPES[workload])
        if cfg_override:
            cfg.update(cfg_override)
        self.cfg = cfg
        self.tokens = cfg["batch"] * cfg["sequence"]
        if data is None:
            data = make_weights(0, cfg, with_cache=workload == "decode")
            if workload == "moe":
                add_expert_weights(data, cfg, rank, world)
        if x is None:
            x = torch.randn((self.tokens, cfg["hidden"]), generator=torch.Generator().manual_seed(1))
        self.x_host = x.pin_memory()
        self.out_host = torch.empty((self.tokens, cfg["hidden"]), dtype=torch.float32).pin_memory()
        c = api.decoder_config(**cfg)
        self.plan = api.DecoderCompiler.compile(c, data, "", api.compile_options(
            tp_rank=rank, tp_size=world, seed_block_table=1 if workload == "decode" else 0,
            weight_int8=args.weights == "int8", local_expert_weights=workload == "moe",
            norm_fusion=True if args.norm_fusion else None))
        self.stream = torch.cuda.ExternalStream(self.plan.stream)
        self.collective = "none"
        self.form = "none"
        views = {}
        stream = self.stream

        def allreduce(buf, count, dtype, stream_ptr):
            key = (buf, count)
            if key not in views:
                class Raw:  # CUDA array interface over the plan's workspace (int16 view of the bf16 data)
                    __cuda_array_interface__ = {"shape": (count,), "typestr": "<i2", "data": (buf, False), "version": 3}
                views[key] = torch.as_tensor(Raw(), device="cuda").view(torch.bfloat16)
            with torch.cuda.stream(stream):
                dist.all_reduce(views[key])

        if world > 1:
            self.plan.set_allreduce(allreduce)
            collective = args.collective
            if collective == "auto":
                # one-shot pushes cost (N-1) x bytes per rank: two ranks, or the small decode outputs; more ranks with
                # large outputs scatter the rows to their owners and gather the sums (two-shot)
                if workload == "moe":
                    collective = "two-shot"   # token-sharded expert parallelism needs the row ownership of this form
                elif world == 2 or workload == "decode":
                    collective = "peer"
                else:
                    collective = "two-shot"
            if collective in ("peer", "two-shot", "two-shot-sm", "two-shot-ce"):
                def exchange(handle):
                    handles = [None] * world
                    dist.all_gather_object(handles, handle)
                    return handles
                self.plan.enable_peer_allreduce(rank, world, exchange, {"peer": 1, "two-shot": 0, "two-shot-sm": 2, "two-shot-ce": 3}[collective])
                dist.barrier()
            self.collective = collective
            for line in self.plan.dump().splitlines():
                if line.startswith("decoder.shard"):
                    self.form = line.split("collective=")[-1]

    def collective_text(self):
        return {"none": "none", "nccl": "nccl all-reduce after O and Down",
                "peer": "all-reduce fused into the O and Down GEMM epilogues over NVLink peer memory",
                "two-shot": "row owners pull their rows of the O / Down partial sums over NVLink peer memory, add the residual and "
                            "sum; dense layers all-gather the rows with copy engines under the next GEMM, MoE layers run "
                            "token-sharded expert parallelism (all-to-all over peer stores)",
                "two-shot-sm": "row owners pull, sum and all-gather with peer stores from one kernel",
                "two-shot-ce": "row owners pull and sum; all-gather on copy engines under the next GEMM"}[self.collective]

    def close(self):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
            if self.collective in ("peer", "two-shot", "two-shot-sm", "two-shot-ce"):
                self.plan.disable_peer_allreduce()
        self.plan.close()


def barrier(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return value
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_layer(layer, args, sampler):
    """value (input resident) and e2e (host buffers) of one workload; --steps timed steps each."""
    import torch
    from schedforge_b200 import lib as L
    lib = L.load()
    plan, world, rank, tokens, cfg = layer.plan, layer.world, layer.rank, layer.tokens, layer.cfg
    regions = []
    plan.upload_input(layer.x_host.numpy())
    for _ in range(args.warmup):
        plan.execute_resident()
    barrier(world)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.sfb_launch_count()
    t0 = time.perf_counter()
    start.record(layer.stream)
    for _ in range(args.steps):
        plan.execute_resident()
    stop.record(layer.stream)
    barrier(world)
    regions.append((t0, time.perf_counter()))
    launches = lib.sfb_launch_count() - launches0
    ms = max_over_ranks(start.elapsed_time(stop) / args.steps, world)

    # e2e: host buffers through the plan call.  With several ranks every rank brings and takes its own rows
    # (sfb_decoder_execute_rows): the whole job still moves the full input and output between host and device
    # each step, 1/N of it per PCIe link.
    sharded_io = world > 1 and tokens % world == 0 and (layer.workload != "moe" or layer.collective in ("two-shot", "two-shot-sm", "two-shot-ce"))
    if sharded_io:
        rows = tokens // world
        row0 = rank * rows
        x_rows, out_rows = layer.x_host[row0:row0 + rows], layer.out_host[row0:row0 + rows]

        def e2e_step(result=None):
            plan.execute_rows_ptr(x_rows.data_ptr(), out_rows.data_ptr(), row0, rows, result)
    else:
        out_rows = layer.out_host

        def e2e_step(result=None):
            plan.execute_ptr(layer.x_host.data_ptr(), layer.out_host.data_ptr(), result)
    for _ in range(args.warmup):
        e2e_step()
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier(world)
    t1 = time.perf_counter()
    regions.append((t0, t1))
    e2e_ms = max_over_ranks(1000.0 * (t1 - t0) / args.steps, world)
    result = L.DecoderResult()
    e2e_step(result)
    finite = bool(torch.isfinite(out_rows).all())
    for region in regions:
        if sampler:
            sampler.mark(*region)
    io_bytes = tokens * cfg["hidden"] * 4
    record = {"workload": NAMES[layer.workload], "tokens_per_step": tokens, "steps": args.steps, "warmup": args.warmup,
              "ms_per_step": ms, "tokens_per_s": tokens * 1000.0 / ms,
              "e2e": {"value": tokens * 1000.0 / e2e_ms, "unit": "tokens/s", "ms_per_step": e2e_ms, "steps": args.steps,
                      "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                      "io": ("each rank copies its 1/N of the rows; " + ("peer stores gather the input" if layer.collective in ("two-shot", "two-shot-sm", "two-shot-ce")
                                                                            else "the all-reduce hook gathers the input")) if sharded_io
                      else "whole input and output on every rank"},
              "gpu_launches": int(launches), "collective": layer.collective_text(), "collective_form": layer.form,
              "stages_ms": {"attention": result.attention_milliseconds, "projection": result.projection_milliseconds,
                            "norm": result.norm_rope_milliseconds, "ffn": result.ffn_milliseconds,
                            "h2d": result.h2d_milliseconds, "d2h": result.d2h_milliseconds},
              "output_finite": finite,
              "clocks": sampler.summary(regions) if sampler else None}
    return record, result


def layer_roofline(workload, cfg, world, result, ms):
    """Roofline record of the dominant kernel of a workload (timed inside the layer step for decode / moe)."""
    peaks = measured_peaks()
    tokens = cfg["batch"] * cfg["sequence"]
    if workload == "moe":
        flops = 6.0 * tokens * cfg["top_k"] * cfg["hidden"] * cfg["intermediate"] / world
        t = result.ffn_milliseconds
        achieved = flops / (t * 1e-3) / 1e12 if t > 0 else None
        return {"kernel": "gemm_tcgen05_kernel<256> grouped mode (experts W3|W1 + SwiGLU, then W2), timed with the "
                          "routing chain around it (router, dispatch, combine)", "bound": "tensor",
                "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops_sustained"] if achieved else None,
                "peak_source": peaks["source"] + " (sustained: timed inside the layer step)",
                "kernel_ms": t, "algorithmic_flops_per_launch": flops, "traffic": None}
    h, i, kvw = cfg["hidden"], cfg["intermediate"], cfg["kv_heads"] * cfg["head_dim"]
    kv_bytes = cfg["batch"] * cfg["context_sequence"] * (cfg["kv_heads"] // world) * cfg["head_dim"] * 2 * 2
    weight_bytes = 2 * (h * (h + 2 * kvw) + h * h + 3 * h * i) // world
    t = result.attention_milliseconds
    achieved = kv_bytes / (t * 1e-3) / 1e9 if t > 0 else None
    step_bytes = kv_bytes + weight_bytes
    return {"kernel": "decode_paged_mma_kernel<4> + combine (inside the layer)", "bound": "hbm", "achieved": achieved,
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"] if achieved else None,
            "peak_source": peaks["source"], "kernel_ms": t, "algorithmic_bytes_per_launch": kv_bytes,
            # ncu on the batch-16 case: 307.0 MB of dram traffic for 301.2 MB of K/V pages (every byte once)
            "traffic": kv_bytes * 307.0 / 301.2,
            "traffic_source": "ncu dram__bytes_read+write of the --kernel decode --small capture, scaled by K/V bytes",
            "whole_step": {"algorithmic_bytes": step_bytes, "achieved": step_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
                           "frac": step_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                           "note": "every layer weight once + every cached K/V byte once, over the whole step time"}}


def gate_up_roofline(tokens, cfg, world):
    """The gate/up tcgen05 GEMM of the prefill step timed alone on the current stream."""
    import torch
    from schedforge_b200 import lib as L
    lib = L.load()
    peaks = measured_peaks()
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
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(cur)
    for _ in range(reps):
        L.check(lib.sfb_k_gemm_bf16(C.byref(g), C.c_void_p(cur.cuda_stream)))
    e1.record(cur)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    kernel_ms = e0.elapsed_time(e1) / reps
    flops = 2.0 * m * n * k
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    return {"kernel": "gemm_tcgen05_kernel<256, false> (gate/up projection, SwiGLU epilogue)", "bound": "tensor",
            "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst: kernel timed alone)",
            "kernel_ms": kernel_ms, "algorithmic_flops_per_launch": flops,
            # dram read + write of one launch: 359.4 MB measured by ncu on the M4096 N16384 case (2048 output
            # tiles), scaled by the tile count of this launch; B is re-read once per band of 16 M-tiles
            "traffic": 359.4e6 * ((m + 127) // 128) * ((n + 255) // 256) / 2048.0,
            "traffic_source": "ncu dram__bytes_read+write of the --kernel gemm --small capture, scaled by output tiles"}, (t0, t1)


def sample_parity(args, rank, world, base):
    """The device plan, sharded like the run, on the bounded CPU sample: max-abs relative error against the
    CPU arm's output (outside every timed region).  `base` is the CPU arm's record on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist
    data, want = (base["_data"], base["_output"]) if base is not None else (None, None)
    cfg = dict(LLAMA, **CPU_SAMPLE)
    if world > 1:  # rank 0 ran the CPU layer; every rank rebuilds the same seeded tensors for its shard
        from oracle import binding as ob
        port = ob.Port()
        data = make_weights(0, cfg)
        for k in data:
            data[k] = port.round_bf16(data[k])
        t = cfg["batch"] * cfg["sequence"]
        data["input"] = port.round_bf16(torch.randn((t, cfg["hidden"]), generator=torch.Generator().manual_seed(1)).numpy())
    x = torch.from_numpy(np.asarray(data["input"], np.float32).reshape(-1, cfg["hidden"]))
    weights = {k: v for k, v in data.items() if k != "input"}
    layer = Layer("prefill", args, rank, world, cfg_override=CPU_SAMPLE, data=weights, x=x)
    layer.plan.execute_ptr(layer.x_host.data_ptr(), layer.out_host.data_ptr(), None)
    got = layer.out_host.numpy().copy()
    layer.close()
    if rank != 0:
        return None
    err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
    return {"rel_err": err, "bar": 2e-2, "ok": bool(err < 2e-2), "n_gpus": world,
            "sample": f"B{cfg['batch']}xS{cfg['sequence']} of the same layer against the CPU arm's output "
                      f"({base['kind']}), max|got - want| / max|want|"}


def strip(record):
    return {k: v for k, v in record.items() if not k.startswith("_")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode", "moe"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="headline only: skip the decode / moe / kernel sub-records")
    ap.add_argument("--norm-fusion", action="store_true",
                    help="fold the RMSNorms into the QKV and gate/up GEMMs instead of stand-alone norm kernels (for A/B runs)")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "int8"],
                    help="int8: per-output-channel weight-only INT8 (the reference's quantized layer); not the default")
    ap.add_argument("--collective", default="auto", choices=["auto", "nccl", "peer", "two-shot", "two-shot-sm", "two-shot-ce"],
                    help="N > 1: all-reduce after the O and Down projections through NCCL, or fused into the GEMM "
                         "epilogues over NVLink peer memory")
    ap.add_argument("--kernel", default="", choices=["", "gemm", "gemm_shard", "gemm_decode", "attention", "decode"],
                    help="time ONE kernel through the kernel ABI instead of the layer (also the ncu target)")
    ap.add_argument("--head-dim", type=int, default=128, choices=[128, 64], help="--kernel attention: head dimension")
    ap.add_argument("--small", action="store_true", help="--kernel: a case small enough for an ncu --set full capture")
    args = ap.parse_args()
    if args.kernel:
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(strip(time_kernel(args.kernel, args.small, args.head_dim, args.steps, args.warmup))))
        return 0

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = dict(LLAMA, **SHAPES[args.workload])
    tokens = cfg["batch"] * cfg["sequence"]
    config = {"workload": NAMES[args.workload], "hidden": 4096, "intermediate": 14336, "q_heads": 32, "kv_heads": 8,
              "head_dim": 128, "tokens_per_step": tokens, "parallelism": f"tp{world}", "collective": "none",
              "l2": "weights + activations (>0.9 GB per step) exceed the 126 MB L2; no flush between steps"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        # The CPU layer takes ~35 s for the 8192-token step, so every step of this arm is a bounded sample of
        # it (one 384-token sequence): exactly --steps timed steps after --warmup, cut short only by a wall budget.
        base = cpu_arm(max(1, args.steps), max(0, args.warmup), CPU_SAMPLE, wall_budget=CPU_WALL_BUDGET_S)
        sample_tokens = base["tokens_per_step"]
        config.update(workload=NAMES["prefill"] + f"_cpu_sample_b{CPU_SAMPLE['batch']}_s{CPU_SAMPLE['sequence']}",
                      sample_of=NAMES["prefill"], tokens_per_step=sample_tokens, parallelism=f"{base['cores']} host threads",
                      same_config=False, l2="n/a (CPU)")
        line = {"impl": "reference", "metric": "decoder_layer_tokens_per_s", "value": base["value"], "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": base["steps_timed"], "warmup": base["warmup"], "steps_requested": args.steps,
                "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    # ---- headline workload ----------------------------------------------------------------------
    layer = Layer(args.workload, args, rank, world)
    config["weights"] = args.weights
    config["collective"] = layer.collective_text()
    head, result = time_layer(layer, args, sampler)
    config["e2e_io"] = head["e2e"]["io"]
    config["collective_form"] = head["collective_form"]
    layer.close()
    if args.workload == "prefill":
        roofline, region = gate_up_roofline(tokens, cfg, world)
        if sampler:
            sampler.mark(*region)
    else:
        roofline = layer_roofline(args.workload, cfg, world, result, head["ms_per_step"])

    subs = {}
    full = args.workload == "prefill" and not args.no_sub
    if full:
        for name in ("decode", "moe"):
            sub_layer = Layer(name, args, rank, world)
            record, sub_result = time_layer(sub_layer, args, sampler)
            sub_layer.close()
            record["roofline"] = layer_roofline(name, sub_layer.cfg, world, sub_result, record["ms_per_step"])
            record["parallelism"] = (f"tp{world}" if name == "decode" else
                                     f"attention tp{world}; FFN token-sharded expert parallel ep{world}: local route + dispatch, "
                                     f"all-to-all dispatch and combine over NVLink peer stores" if sub_layer.collective in ("two-shot", "two-shot-sm", "two-shot-ce")
                                     else f"attention tp{world}, experts sharded {world} ways on replicated tokens")
            subs[name] = record
        if world == 1:
            kernels = {}
            for key, kernel in (("attention_cfg1", "attention"), ("paged_decode_cfg2", "decode")):
                record = time_kernel(kernel, False, 128, args.steps, args.warmup)
                if sampler:
                    record["clocks"] = sampler.summary([record["_region"]])
                    sampler.mark(*record["_region"])
                kernels[key] = strip(record)
            subs["kernels"] = kernels

    # ---- CPU baseline and parity on the bounded sample (outside every timed region) -------------------
    cpu, parity = None, None
    if args.workload == "prefill" and not args.no_cpu_baseline:
        base = None
        if rank == 0:
            base = cpu_arm(1, 1, CPU_SAMPLE, want_output=True)
            if world == 1:
                cpu = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        parity = sample_parity(args, rank, world, base)

    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
    if rank == 0:
        line = {"metric": "decoder_layer_tokens_per_s", "value": head["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": config,
                "e2e": {k: head["e2e"][k] for k in ("value", "unit", "ms_per_step", "steps", "h2d_bytes_per_step", "d2h_bytes_per_step")},
                "gpu_launches": head["gpu_launches"], "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
                "stages_ms": head["stages_ms"], "output_finite": head["output_finite"], "parity": parity}
        line.update(subs)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

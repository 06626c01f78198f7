"""Decoder layer parity through the plan ABI (sfb_decoder_compile / sfb_decoder_execute):
the reference's own test shapes and seeds from the golden fixtures, the tiny fp32 benchmark configuration, and
bf16 tensor-core plans against the oracle on bf16-rounded data."""
import os
import sys

import numpy as np
import pytest

from conftest import rel_err
from oracle import binding as ob
from schedforge_b200 import api, lib as L

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
from stablehlo_texts import DECODER_TEXT, MOE_TEXT, dense_decoder_text  # noqa: E402

F32_TOL = 1e-4   # max-abs relative, fp32 plan
BF16_TOL = 2e-2  # max-abs relative, bf16 plan


def fixture(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    oc = ob.DecoderConfig()
    for (field, _), value in zip(oc._fields_, z["config"]):
        setattr(oc, field, float(value) if field in ("rms_epsilon", "rope_theta") else int(value))
    c = L.DecoderConfig(*[getattr(oc, f) for f, _ in oc._fields_])
    data = {k[3:]: z[k] for k in z.files if k.startswith("in_")}
    return c, oc, data, z


def weights_of(data):
    return {k: v for k, v in data.items() if k != "input"}


@pytest.mark.parametrize("name,text", [("decoder_dense", DECODER_TEXT), ("decoder_moe", DECODER_TEXT),
                                       ("decoder_moe", MOE_TEXT), ("decoder_decode", DECODER_TEXT),
                                       ("decoder_cfg1_shape", ""), ("decoder_batched", ""),
                                       ("decoder_moe_medium", "")])
def test_fp32_plan_matches_reference_fixtures(name, text):
    c, _, data, z = fixture(name)
    plan = api.DecoderCompiler.compile(c, weights_of(data), text, api.compile_options(dtype=L.F32))
    out, result = plan.execute(data["input"])
    assert out.shape == z["out_reference"].shape
    assert np.max(np.abs(out - z["out_reference"])) < 1e-3          # the reference's own bar
    assert rel_err(out, z["out_reference"]) < F32_TOL
    assert rel_err(out, z["out_native"]) < 1e-5                     # same FMA-chain GEMM arithmetic
    assert result.tokens_per_second > 0 and result.kernel_launches > 0
    dump = plan.dump()
    assert "sfe.decoder_executable" in dump and "tensor.fused_qkv" in dump and "attention.online_softmax" in dump
    if c.ffn_moe:
        assert "moe.histogram" in dump
    else:
        assert "tensor.fused_gate_up" in dump
    if c.context_sequence > 0:
        assert "split_kv_decode" in dump
    plan.close()


def baseline_config1():
    """The tiny fp32 benchmark configuration: dense prefill, weights ~N(0,0.02), activations ~N(0,1), seed 0."""
    kw = dict(batch=1, sequence=128, hidden=256, intermediate=688, query_heads=4, kv_heads=2, head_dim=64,
              rms_epsilon=1e-5, rope_theta=10000.0)
    rng = np.random.default_rng(0)
    h, i, kv = 256, 688, 128
    data = {"input": rng.standard_normal((128, h)).astype(np.float32),
            "rms1_weight": np.ones(h, np.float32), "rms2_weight": np.ones(h, np.float32)}
    for key, shape in (("query_weight", (h, h)), ("key_weight", (h, kv)), ("value_weight", (h, kv)),
                       ("output_weight", (h, h)), ("gate_weight", (h, i)), ("up_weight", (h, i)),
                       ("down_weight", (i, h))):
        data[key] = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    return kw, data


def test_baseline_config1_fp32(port):
    kw, data = baseline_config1()
    want = port.decoder_layer(ob.decoder_config(**kw), data, native=False)
    plan = api.DecoderCompiler.compile(api.decoder_config(**kw), weights_of(data), dense_decoder_text(128, 256, 128, 688),
                                       api.compile_options(dtype=L.F32))
    out, _ = plan.execute(data["input"])
    assert rel_err(out, want) < F32_TOL
    # the plan can be re-run with the input resident, and gives the same bits
    plan.execute_resident()
    assert np.array_equal(plan.download_output(), out)
    plan.close()


def bf16_case(port, seed, moe=False, **kw):
    oc = ob.decoder_config(moe=moe, **kw)
    rng = np.random.default_rng(seed)
    shapes = ob.decoder_shapes(oc)
    data = {}
    for key, n in shapes.items():
        scale = 1.0 if key in ("input", "cached_key", "cached_value") else 0.05
        data[key] = port.round_bf16((rng.standard_normal(n) * scale).astype(np.float32))
    data["rms1_weight"] = (1.0 + 0.1 * rng.standard_normal(oc.hidden)).astype(np.float32)
    data["rms2_weight"] = (1.0 + 0.1 * rng.standard_normal(oc.hidden)).astype(np.float32)
    return oc, api.decoder_config(moe=moe, **kw), data


@pytest.mark.parametrize("fuse,backend", [(True, L.GEMM_AUTO), (True, L.GEMM_SIMT), (False, L.GEMM_AUTO)])
def test_bf16_dense_prefill(port, fuse, backend):
    kw = dict(batch=2, sequence=192, hidden=512, intermediate=1024, query_heads=8, kv_heads=2, head_dim=64,
              rope_theta=500000.0)
    oc, c, data = bf16_case(port, 1, **kw)
    want = port.decoder_layer(oc, data, native=True)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(fuse_epilogues=fuse, gemm_backend=backend))
    out, result = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert result.kernel_launches >= 6
    plan.close()


@pytest.mark.parametrize("intermediate", [688, 1376])   # 2*I a multiple of 64 or not: blocked or row-major gate/up
def test_bf16_cfg1_shape_with_ragged_ffn_width(port, intermediate):
    kw, _ = baseline_config1()
    kw = dict(kw, intermediate=intermediate)
    oc, c, data = bf16_case(port, 2, **kw)
    want = port.decoder_layer(oc, data, native=True)
    plan = api.DecoderCompiler.compile(c, weights_of(data))
    out, _ = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    plan.close()


@pytest.mark.parametrize("head_dim,seed_table", [(128, 7), (64, 0)])
def test_bf16_decode_over_paged_cache(port, head_dim, seed_table):
    kw = dict(batch=5, sequence=1, hidden=8 * head_dim, intermediate=512, query_heads=8, kv_heads=2,
              head_dim=head_dim, context_sequence=300)
    oc, c, data = bf16_case(port, 3, **kw)
    want = port.decoder_layer(oc, data, native=True)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(seed_block_table=seed_table))
    out, _ = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert "paged_kv page_tokens=16" in plan.dump()
    plan.close()


def test_bf16_moe_layer_and_bit_exact_routing(port):
    kw = dict(batch=2, sequence=128, hidden=256, intermediate=256, query_heads=4, kv_heads=2, head_dim=64,
              experts=8, top_k=2)
    oc, c, data = bf16_case(port, 4, moe=True, **kw)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(no_workspace_reuse=True))
    out, _ = plan.execute(data["input"])
    T = 256
    # routing chain on the very tensor the GPU routed: integer outputs must be identical
    n2 = plan.read_tensor("normalized2").reshape(T, 256)
    mc = ob.MoeConfig(T, 256, 256, 8, 2)
    ids, weights, counts = port.route_topk(mc, n2, data["router_weight"].reshape(256, 8))
    got_ids = plan.read_tensor("expert_ids", np.int32).reshape(T, 2)
    got_counts = plan.read_tensor("counts", np.int32)
    assert port.last_tie_tokens == 0
    assert np.array_equal(got_ids, ids) and np.array_equal(got_counts, counts)
    assert np.allclose(plan.read_tensor("expert_weights").reshape(T, 2), weights, rtol=1e-5, atol=1e-6)
    _, offsets, token_ids, slots, _ = port.dispatch_tokens(mc, n2, ids, weights, counts, copy_values=False)
    assert np.array_equal(plan.read_tensor("offsets", np.int32), offsets)
    assert np.array_equal(plan.read_tensor("token_ids", np.int32), token_ids)
    assert np.array_equal(plan.read_tensor("route_slots", np.int32), slots)
    # layer output against the oracle with the same routing injected as a trace
    want = port.decoder_layer(oc, data, native=True, trace=(ids, weights, counts))
    assert rel_err(out, want) < BF16_TOL
    # and the plan honours an injected trace like DecoderData::routing_trace
    out2, _ = plan.execute(data["input"], trace=(ids, weights, counts))
    assert rel_err(out2, want) < BF16_TOL
    plan.close()


@pytest.mark.parametrize("shards,decode", [(2, False), (4, False), (8, False), (8, True)])
def test_tensor_parallel_shards_reproduce_the_full_layer(port, shards, decode):
    """Tensor-parallel shards on ONE GPU with the all-reduce emulated through the plan's hook:
    pass 1 captures each shard's O-projection partial, pass 2 adds the peers' partials where the
    collective would run and captures the down-projection partials, whose sum is the layer output.
    Eight shards of eight KV heads is the one-KV-head-per-rank case of an 8-GPU node."""
    import ctypes as C
    import torch
    kw = dict(batch=2, sequence=64, hidden=512, intermediate=1024, query_heads=16, kv_heads=8, head_dim=32)
    if decode:
        kw.update(sequence=1, batch=4, context_sequence=100)
    oc, c, data = bf16_case(port, 6, **kw)
    want = port.decoder_layer(oc, data, native=True)
    lib = L.load()
    rows = kw["batch"] * kw["sequence"]
    count = rows * kw["hidden"]
    # (one-shot execute: the hook then sees the whole [T, H] partial sums in one call)
    plans = [api.DecoderCompiler.compile(c, weights_of(data), "",
                                         api.compile_options(tp_rank=r, tp_size=shards, no_pipeline=True))
             for r in range(shards)]
    first = [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(shards)]
    second = [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(shards)]

    def copy_out(buf, dst, stream):
        L.check(lib.sfb_k_convert(C.c_void_p(buf), L.BF16, C.c_void_p(dst.data_ptr()), L.BF16, C.c_int64(count),
                                  C.c_void_p(stream)))

    for rank, plan in enumerate(plans):  # pass 1: capture the first partial of every shard
        calls = []

        def hook(buf, n, dtype, stream, rank=rank, calls=calls):
            assert n == count and dtype == L.BF16
            if not calls:
                copy_out(buf, first[rank], stream)
            calls.append(buf)
        plan.set_allreduce(hook)
        plan.execute(data["input"])
        assert len(calls) == 2
    for rank, plan in enumerate(plans):  # pass 2: sum the peers' partials, capture the second one
        calls = []

        def hook(buf, n, dtype, stream, rank=rank, calls=calls):
            if not calls:
                for peer in range(shards):
                    if peer != rank:
                        L.check(lib.sfb_k_add(C.c_void_p(buf), C.c_void_p(first[peer].data_ptr()), C.c_void_p(buf),
                                              C.c_int64(count), L.BF16, C.c_void_p(stream)))
            else:
                copy_out(buf, second[rank], stream)
            calls.append(buf)
        plan.set_allreduce(hook)
        plan.execute(data["input"])
    torch.cuda.synchronize()
    out = sum(t.float() for t in second).cpu().numpy().reshape(rows, kw["hidden"])
    assert rel_err(out, want) < BF16_TOL
    for p in plans:
        p.close()


@pytest.mark.parametrize("dtype,head_dim,ctx", [(L.F32, 64, 37), (L.BF16, 64, 37), (L.BF16, 128, 48)])
def test_autoregressive_step_equals_last_token_of_the_prefill(port, dtype, head_dim, ctx):
    """append_new_token: the decode step over a cache of `ctx` tokens must give what a causal
    prefill over ctx + 1 tokens gives for its last token.  The prefill side is the oracle's layer
    (bit-identical to the reference build); the cache holds the rotated K and the V of the first
    ctx tokens, computed with the oracle's own norm / GEMM / split+RoPE."""
    batch, hq, hkv = 3, 4, 2
    kw = dict(batch=batch, sequence=ctx + 1, hidden=hq * head_dim, intermediate=384, query_heads=hq, kv_heads=hkv,
              head_dim=head_dim, rope_theta=10000.0)
    oc, _, data = bf16_case(port, 21, **kw)
    hidden = oc.hidden
    want = port.decoder_layer(oc, data, native=True).reshape(batch, ctx + 1, hidden)[:, ctx, :]
    x = data["input"].reshape(batch * (ctx + 1), hidden)
    normalized = port.rms_norm(x, data["rms1_weight"], oc.rms_epsilon)
    kvw = hkv * head_dim
    wqkv = np.concatenate([data["query_weight"].reshape(hidden, hidden), data["key_weight"].reshape(hidden, kvw),
                           data["value_weight"].reshape(hidden, kvw)], axis=1)
    _, keys, values = port.split_qkv_rope(oc, port.matmul(normalized, wqkv, fma=True))  # [B, Hkv, ctx + 1, D]
    step = dict(weights_of(data))
    step["cached_key"] = np.ascontiguousarray(keys[:, :, :ctx, :])
    step["cached_value"] = np.ascontiguousarray(values[:, :, :ctx, :])
    if dtype == L.BF16:  # the plan stores the cache in bf16
        step["cached_key"] = port.round_bf16(step["cached_key"])
        step["cached_value"] = port.round_bf16(step["cached_value"])
    c = api.decoder_config(**dict(kw, sequence=1, context_sequence=ctx))
    plan = api.DecoderCompiler.compile(c, step, "", api.compile_options(dtype=dtype, append_new_token=True,
                                                                        seed_block_table=5))
    last = np.ascontiguousarray(data["input"].reshape(batch, ctx + 1, hidden)[:, ctx, :])
    out, _ = plan.execute(last)
    assert rel_err(out, want) < (F32_TOL if dtype == L.F32 else BF16_TOL)
    again, _ = plan.execute(last)  # the append overwrites the same position: the plan can be run again
    # (bf16 plans sum the partial tiles of their few-row GEMMs with fp32 reductions at L2, whose order is not fixed:
    # a last-bit difference in a sum can move a bf16 intermediate by one step, which the fp32 output then shows)
    assert rel_err(again, out) < (1e-5 if dtype == L.F32 else BF16_TOL / 4)
    # without the flag the same plan input gives the reference's decode semantics, which differ
    legacy = api.DecoderCompiler.compile(c, step, "", api.compile_options(dtype=dtype))
    out_legacy, _ = legacy.execute(last)
    assert rel_err(out_legacy, want) > 2 * BF16_TOL
    plan.close()
    legacy.close()


def test_plan_optimizer_measures_ranks_and_confirms(port):
    """The reference's own bar for its optimizer (tests/test_schedforge.cpp:916-921): at least 16
    candidates, at least 5 hardware measurements with a budget of 4, a measured winner, a positive
    speedup and a usable plan; plus: the winner is never slower than the confirmed baseline."""
    kw = dict(batch=2, sequence=128, hidden=512, intermediate=1024, query_heads=8, kv_heads=2, head_dim=64)
    oc, c, data = bf16_case(port, 31, **kw)
    base = api.compile_options(fuse_epilogues=False)  # a deliberately weak baseline: materialised intermediates
    plan, result, candidates = api.ExecutablePlanOptimizer.optimize(c, weights_of(data), data["input"], "", base,
                                                                    measurement_budget=4, repetitions=3)
    assert result.candidates >= 16 and len(candidates) >= 16
    assert result.hardware_measurements >= 5
    assert result.winner.measured and result.speedup > 0.0
    assert result.winner.measured_milliseconds <= result.baseline.measured_milliseconds
    assert result.winner.workspace_bytes > 0
    scores = [cand.cost.analytical_score for cand in candidates[1:]]
    assert scores == sorted(scores)                       # ranked by the analytic score
    assert sum(cand.cost.measured for cand in candidates[1:]) == 4  # exactly the budget was measured
    assert candidates[1].options.fuse_epilogues == 1      # fused tensor-core plans rank first
    out, _ = plan.execute(data["input"])
    assert rel_err(out, port.decoder_layer(oc, data, native=True)) < BF16_TOL
    plan.close()


def test_pipelined_execute_in_row_chunks_equals_the_one_shot_plan(port):
    """Two sequences of 1024 tokens, head_dim 128: sfb_decoder_execute overlaps its host copies with compute in
    four chunks of 512 rows (half sequences; attention runs on row slices).  Same numbers as the one-shot form."""
    kw = dict(batch=2, sequence=1024, hidden=512, intermediate=1024, query_heads=4, kv_heads=2, head_dim=128,
              rope_theta=500000.0)
    oc, c, data = bf16_case(port, 41, **kw)
    piped = api.DecoderCompiler.compile(c, weights_of(data))
    one_shot = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(no_pipeline=True))
    out_piped, _ = piped.execute(data["input"])
    out_one, _ = one_shot.execute(data["input"])
    assert np.array_equal(out_piped, out_one)
    assert rel_err(out_piped, port.decoder_layer(oc, data, native=True)) < BF16_TOL
    assert np.array_equal(piped.execute(data["input"])[0], out_piped)  # and again on the used workspace
    piped.close()
    one_shot.close()


def test_pipelined_execute_in_chunks_that_span_sequences_equals_the_one_shot_plan(port):
    """Three sequences of 1280 tokens at hidden 1792: the chunks are sized in row blocks that fill whole rounds of
    the SMs (4, 21 and 5 blocks of 128 rows on 148 SMs), so the middle chunk holds the tail of the first sequence,
    the whole second one and the head of the third: three attention launches.  Same numbers as the one-shot form
    (below 2048 columns the RMSNorm kernel is the same one for every row count)."""
    kw = dict(batch=3, sequence=1280, hidden=1792, intermediate=1024, query_heads=14, kv_heads=2, head_dim=128,
              rope_theta=500000.0)
    oc, c, data = bf16_case(port, 43, **kw)
    piped = api.DecoderCompiler.compile(c, weights_of(data))
    one_shot = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(no_pipeline=True))
    out_piped, result = piped.execute(data["input"])
    out_one, one_result = one_shot.execute(data["input"])
    assert result.kernel_launches > one_result.kernel_launches + 8    # it did run in several chunks
    assert np.array_equal(out_piped, out_one)
    assert rel_err(out_piped, port.decoder_layer(oc, data, native=True)) < BF16_TOL
    assert np.array_equal(piped.execute(data["input"])[0], out_piped)  # and again on the used workspace
    piped.close()
    one_shot.close()


def test_fixed_order_decode_plan_is_bitwise_reproducible(port):
    """fixed_order: the few-row GEMMs of a decode plan compute every output tile in one CTA (no fp32 partial sums
    meeting at L2 in arrival order), so repeated runs give the same bits; the default plan of the same layer only
    promises the bf16 tolerance."""
    kw = dict(batch=5, sequence=1, hidden=1024, intermediate=1536, query_heads=8, kv_heads=2, head_dim=128,
              context_sequence=300)
    oc, c, data = bf16_case(port, 53, **kw)
    want = port.decoder_layer(oc, data, native=True)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(fixed_order=True))
    outs = [plan.execute(data["input"])[0] for _ in range(8)]
    assert all(np.array_equal(o, outs[0]) for o in outs[1:])
    assert rel_err(outs[0], want) < BF16_TOL
    plan.close()
    shared = api.DecoderCompiler.compile(c, weights_of(data))
    assert rel_err(shared.execute(data["input"])[0], outs[0]) < BF16_TOL / 4
    shared.close()


@pytest.mark.parametrize("kw", [
    dict(batch=5, sequence=1, hidden=1024, intermediate=512, query_heads=8, kv_heads=2, head_dim=128, context_sequence=300),
    dict(batch=1, sequence=96, hidden=512, intermediate=1024, query_heads=8, kv_heads=2, head_dim=64),   # few rows: int8 kept
    dict(batch=2, sequence=192, hidden=512, intermediate=1024, query_heads=8, kv_heads=2, head_dim=64),  # many rows: q * scale in bf16
])
def test_weight_only_int8_plan_matches_the_quantized_oracle(port, kw):
    """weight_int8: the oracle layer on q * scale weights is what the reference's INT8 layer computes
    (pinned on the CPU against the reference build); the bf16 activations add the usual tolerance."""
    oc, c, data = bf16_case(port, 51, **kw)
    want = port.decoder_layer(oc, ob.int8_weight_data(oc, data), native=True)
    plain = port.decoder_layer(oc, data, native=True)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(weight_int8=True))
    out, _ = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert rel_err(out, plain) > rel_err(out, want)   # it is the quantized layer, not the plain one
    assert "_int8" in plan.dump()
    plan.close()
    with pytest.raises(L.SfbError):
        api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(weight_int8=True, dtype=L.F32))


def test_benchmark_profile_matrix_measures_on_the_device(port, tmp_path):
    """benchmark_decoder_profile on the device plan: a prefill, a decode and a skewed MoE profile of the reference's
    matrix, one of them through the plan optimizer, and one profile above the budget; both CSV files carry one
    row per record / candidate."""
    profiles = {p.name.decode(): p for p in api.realistic_decoder_profiles()}
    records = [api.benchmark_decoder_profile(profiles["tiny-prefill-s128"], optimize_plan=True, repetitions=2),
               api.benchmark_decoder_profile(profiles["tiny-decode-kv512"], repetitions=2),
               api.benchmark_decoder_profile(profiles["tiny-moe-heavy-skew"], repetitions=2),
               api.benchmark_decoder_profile(profiles["large-prefill-s2048"], max_real_flops=1 << 30)]
    for r in records[:3]:
        assert r.evidence == L.EVIDENCE_MEASURED and r.measured.milliseconds > 0 and r.measured.tokens_per_second > 0
        assert r.plan_cost.workspace_bytes > 0 and r.compile_milliseconds > 0
        assert r.selected_policy.decode().startswith("decoder.policy layout=")
    assert records[0].candidate_count == 17 and records[0].hardware_measurements >= 5 and records[0].optimizer_speedup > 0
    assert "attention=split-kv-decode" in records[1].selected_policy.decode()
    assert records[3].evidence == L.EVIDENCE_COMPILE_ONLY and records[3].measured.milliseconds == 0.0
    api.write_decoder_benchmark_csv(tmp_path / "decoder.csv", records)
    lines = (tmp_path / "decoder.csv").read_text().splitlines()
    header = lines[0].split(",")
    assert len(lines) == 5 and all(len(l.split(",")) == len(header) for l in lines[1:])
    row = dict(zip(header, lines[3].split(",")))
    assert row["profile"] == "tiny-moe-heavy-skew" and row["ffn"] == "moe" and row["experts"] == "16"
    assert row["routing"] == "heavy-skew" and float(row["latency_ms"]) > 0 and row["evidence"] == "measured"
    api.write_decoder_plan_candidates_csv(tmp_path / "candidates.csv", records)
    cand = (tmp_path / "candidates.csv").read_text().splitlines()
    assert len(cand) == 1 + 17 and sum(l.split(",")[2] == "1" for l in cand[1:]) >= 1
    assert sum(l.split(",")[3] == "1" for l in cand[1:]) >= 5                    # measured candidates


def test_execute_rows_whole_range_and_guards(port):
    # 256 rows: above the few-row GEMMs, whose partial sums meet in L2 in an order that differs from run to run
    kw = dict(batch=2, sequence=128, hidden=256, intermediate=512, query_heads=4, kv_heads=2, head_dim=64)
    oc, c, data = bf16_case(port, 3, **kw)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(no_pipeline=True))
    want, _ = plan.execute(data["input"])
    x = np.asarray(data["input"], np.float32).reshape(256, 256)
    got, result = plan.execute_rows(x, 0)
    assert np.array_equal(got.ravel(), want.ravel()) and result.milliseconds > 0
    with pytest.raises(L.InvalidArgument, match="all-reduce hook"):
        plan.execute_rows(x[:64], 0)          # a part of the rows needs the other ranks
    with pytest.raises(L.InvalidArgument, match="outside the plan"):
        plan.execute_rows(x, 64)
    plan.close()


def test_device_wait_that_runs_out_surfaces_as_device_timeout(port, dev):
    """Failure detection at the plan level without a fault: shard 0 of a two-shard plan is given a peer
    buffer whose flags nothing ever sets (ordinary memory of this GPU stands in for the absent rank), so
    the bounded wait of the fused all-reduce gives up.  sfb_decoder_execute must then return
    SFB_DEVICE_TIMEOUT instead of SFB_OK with unsummed partials, clear the status word, and the same plan
    must run normally afterwards."""
    import ctypes as C
    kw = dict(batch=1, sequence=160, hidden=256, intermediate=512, query_heads=4, kv_heads=2, head_dim=64)
    oc, c, data = bf16_case(port, 61, **kw)
    plan = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(tp_rank=0, tp_size=2, no_pipeline=True))
    lib = L.load()
    nbytes = lib.sfb_decoder_peer_bytes(plan._h)
    local = dev.zeros((nbytes,), dev.torch.uint8)
    absent = dev.zeros((nbytes,), dev.torch.uint8)
    bases = (C.c_void_p * 2)(None, absent.data_ptr())
    L.check(lib.sfb_decoder_set_peer_allreduce(plan._h, C.c_void_p(local.data_ptr()), bases))
    with pytest.raises(L.SfbError) as failure:
        plan.execute(data["input"])
    assert failure.value.status == L.SFB_DEVICE_TIMEOUT and "wait gave up" in failure.value.message
    word = C.c_uint32(7)
    L.check(lib.sfb_device_status(C.byref(word)))
    assert word.value == 0                      # reported once, then cleared
    # back to the hook form with a hook that adds nothing: shard 0 alone runs to completion
    L.check(lib.sfb_decoder_set_peer_allreduce(plan._h, None, None))
    plan.set_allreduce(lambda buf, count, dtype, stream: None)
    out, _ = plan.execute(data["input"])
    assert np.all(np.isfinite(out))
    plan.close()


@pytest.mark.parametrize("dtype,head_dim", [(L.BF16, 128), (L.BF16, 64), (L.F32, 64)])
def test_decode_loop_steps_across_a_page_boundary(port, dtype, head_dim):
    """sfb_decoder_step: five successive steps from a cache of 13 tokens (16-token pages, so the fourth step
    opens the second page) must reproduce the last five tokens of the oracle's causal prefill over 18 tokens,
    and the page accounting after every step must equal the reference's PagedKVCache fed the same appends;
    then truncate / release behave like truncate_paged_kv / release_paged_kv_pages."""
    batch, hq, hkv, ctx, steps = 3, 4, 2, 13, 5
    total = ctx + steps
    kw = dict(batch=batch, sequence=total, hidden=hq * head_dim, intermediate=384, query_heads=hq, kv_heads=hkv,
              head_dim=head_dim, rope_theta=10000.0)
    oc, _, data = bf16_case(port, 71, **kw)
    hidden, kvw = oc.hidden, hkv * head_dim
    want = port.decoder_layer(oc, data, native=True).reshape(batch, total, hidden)
    x = data["input"].reshape(batch * total, hidden)
    normalized = port.rms_norm(x, data["rms1_weight"], oc.rms_epsilon)
    wqkv = np.concatenate([data["query_weight"].reshape(hidden, hidden), data["key_weight"].reshape(hidden, kvw),
                           data["value_weight"].reshape(hidden, kvw)], axis=1)
    _, keys, values = port.split_qkv_rope(oc, port.matmul(normalized, wqkv, fma=True))
    start = dict(weights_of(data))
    start["cached_key"] = np.ascontiguousarray(keys[:, :, :ctx, :])
    start["cached_value"] = np.ascontiguousarray(values[:, :, :ctx, :])
    if dtype == L.BF16:
        start["cached_key"], start["cached_value"] = port.round_bf16(start["cached_key"]), port.round_bf16(start["cached_value"])
    capacity = 40                                    # three pages
    c = api.decoder_config(**dict(kw, sequence=1, context_sequence=ctx))
    plan = api.DecoderCompiler.compile(c, start, "", api.compile_options(dtype=dtype, append_new_token=True,
                                                                         seed_block_table=9, kv_capacity=capacity,
                                                                         norm_fusion=head_dim == 128))
    if dtype == L.BF16:
        assert "kv_append=paged_cache" in plan.dump()
        assert ("prologue=rms_norm_folded" in plan.dump()) == (head_dim == 128)
    mirror = port.paged_create(batch, hkv, head_dim, head_dim, 16, capacity)   # the reference's accounting
    mirror.append(start["cached_key"], start["cached_value"], ctx)
    tokens = data["input"].reshape(batch, total, hidden)
    tol = F32_TOL if dtype == L.F32 else BF16_TOL
    one = np.zeros((batch, hkv, 1, head_dim), np.float32)
    for i in range(steps):
        out, _ = plan.step(np.ascontiguousarray(tokens[:, ctx + i, :]))
        assert rel_err(out, want[:, ctx + i, :]) < tol, i
        mirror.append(one, one, 1)
        got, ref_info = plan.kv_info(), mirror.info()
        assert got["length"] == ref_info["length"] == ctx + i + 1
        assert np.array_equal(got["page_table"], ref_info["page_table"])
        assert np.array_equal(got["free_pages"], ref_info["free_pages"]) and got["pages"] == ref_info["pages"] == 3
    assert len(plan.kv_info()["page_table"]) == 2
    # execute() on the same plan runs the pass at the current length without advancing it
    before = plan.kv_info()["length"]
    plan.execute(np.ascontiguousarray(tokens[:, total - 1, :]))
    assert plan.kv_info()["length"] == before
    # truncate back into the first page: the second page returns to the free list; stepping again from there
    # reproduces the prefill's token 15 and 16 (the page is handed out again at the boundary)
    plan.kv_truncate(ctx + 2)
    mirror.truncate(ctx + 2)
    assert np.array_equal(plan.kv_info()["page_table"], mirror.info()["page_table"])
    assert np.array_equal(plan.kv_info()["free_pages"], mirror.info()["free_pages"])
    for i in (2, 3):
        out, _ = plan.step(np.ascontiguousarray(tokens[:, ctx + i, :]))
        assert rel_err(out, want[:, ctx + i, :]) < tol, i
    with pytest.raises(L.InvalidArgument, match="cannot release an active paged KV page"):
        plan.kv_release([int(plan.kv_info()["page_table"][0])])
    with pytest.raises(L.InvalidArgument, match="invalid physical KV page"):
        plan.kv_release([99])
    with pytest.raises(L.InvalidArgument, match="invalid paged KV truncation length"):
        plan.kv_truncate(100)
    # fill the cache: the step after the last slot is refused
    while plan.kv_info()["length"] < capacity:
        plan.step(np.ascontiguousarray(tokens[:, total - 1, :]))
    with pytest.raises(L.InvalidArgument, match="paged KV capacity exceeded"):
        plan.step(np.ascontiguousarray(tokens[:, total - 1, :]))
    mirror.close()
    plan.close()
    # a plan without the flag has no loop
    legacy = api.DecoderCompiler.compile(c, start, "", api.compile_options(dtype=dtype))
    with pytest.raises(L.InvalidArgument, match="append_new_token"):
        legacy.step(np.ascontiguousarray(tokens[:, ctx, :]))
    legacy.close()


@pytest.mark.parametrize("kw", [
    dict(batch=2, sequence=192, hidden=512, intermediate=1024, query_heads=8, kv_heads=2, head_dim=64, rope_theta=500000.0),
    dict(batch=1, sequence=300, hidden=1024, intermediate=2752, query_heads=8, kv_heads=8, head_dim=128),
    dict(batch=5, sequence=1, hidden=1024, intermediate=512, query_heads=8, kv_heads=2, head_dim=128, context_sequence=300),
])
def test_rms_norm_folded_into_the_gemms(port, kw):
    """norm_fusion: both RMSNorms disappear as kernels; the norm weights are multiplied into the packed QKV and
    gate/up weights, the QKV / gate-up epilogues scale their accumulator rows by 1/rms (sums of squares from the
    input conversion and from the O projection's epilogue).  Same oracle, same bar; fewer launches."""
    oc, c, data = bf16_case(port, 81, **kw)
    want = port.decoder_layer(oc, data, native=True)
    plain = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(no_pipeline=True))
    folded = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(no_pipeline=True, norm_fusion=True))
    out_plain, r_plain = plain.execute(data["input"])
    out, r = folded.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL and rel_err(out_plain, want) < BF16_TOL
    assert r.kernel_launches == r_plain.kernel_launches - 2
    dump = folded.dump()
    assert dump.count("prologue=rms_norm_folded") == 2 and "_rms_folded" in dump
    assert "rms_norm_folded" not in plain.dump()
    if kw["batch"] == 2:   # the row-chunk pipeline takes the sums of squares per chunk
        piped = api.DecoderCompiler.compile(c, weights_of(data), "", api.compile_options(norm_fusion=True))
        assert rel_err(piped.execute(data["input"])[0], want) < BF16_TOL
        piped.close()
    plain.close()
    folded.close()

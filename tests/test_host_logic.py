"""Host-side logic that needs no GPU: StableHLO import + fusion check, configuration
validation and compile-time guards, MoE task table, RoPE table, weight shards."""
import ctypes as C
import json
import os
import sys

import numpy as np
import pytest

from schedforge_b200 import api, lib as L

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
from stablehlo_texts import DECODER_TEXT, MOE_TEXT, NO_QKV_TEXT  # noqa: E402


def golden_import():
    return json.load(open(os.path.join(GOLDEN, "importer.json")))


@pytest.mark.parametrize("key,text", [("decoder", DECODER_TEXT), ("moe", MOE_TEXT), ("no_qkv", NO_QKV_TEXT)])
def test_importer_matches_reference_fixture(key, text):
    got = api.StableHLOImporter.import_text(text)
    want = golden_import()[key]
    for field in ("operations", "values", "inputs", "matmuls", "fused_qkv", "fused_gate_up", "fused_rope"):
        assert got[field] == want[field], field


def test_importer_matches_reference_build(ref):
    for text in (DECODER_TEXT, MOE_TEXT, NO_QKV_TEXT):
        got, want = api.StableHLOImporter.import_text(text), ref.import_stablehlo(text)
        assert {k: got[k] for k in want} == want


def test_importer_dump_and_errors():
    dump = api.StableHLOImporter.dump(DECODER_TEXT)
    assert dump.startswith("graph @model {") and "tensor.rms_norm" in dump and "tensor.rope" in dump
    assert "tensor.swiglu" in dump and "func.return" in dump
    assert "moe.combine" in api.StableHLOImporter.dump(MOE_TEXT)
    with pytest.raises(L.InvalidArgument, match="unsupported StableHLO operation: sine"):
        api.StableHLOImporter.import_text("%a = stablehlo.sine %x : tensor<4xf32>")
    with pytest.raises(L.InvalidArgument, match="matmul reduction dimensions do not match"):
        api.StableHLOImporter.import_text(
            "func.func @f(%x: tensor<4x16xf32>, %w: tensor<8x16xf32>)\n %y = stablehlo.dot_general %x, %w : tensor<4x16xf32>\n")
    # symbolic and dynamic extents are accepted
    summary = api.StableHLOImporter.import_text(
        "func.func @f(%x: tensor<?x16xf32>, %w: tensor<16xf32>)\n %y = stablehlo.custom_call @RmsNorm(%x, %w) : tensor<?x16xf32>\n return %y")
    assert summary["operations"] == 4


def _weights(c, rng):
    h, i, kv = c.hidden, c.intermediate, c.kv_heads * c.head_dim
    shapes = dict(rms1_weight=h, query_weight=h * h, key_weight=h * kv, value_weight=h * kv, output_weight=h * h,
                  rms2_weight=h, gate_weight=h * i, up_weight=h * i, down_weight=i * h)
    return {k: rng.standard_normal(n).astype(np.float32) for k, n in shapes.items()}


def test_compile_rejects_invalid_configuration_before_touching_the_device():
    rng = np.random.default_rng(0)
    bad = api.decoder_config(hidden=60)  # hidden != query_heads * head_dim
    with pytest.raises(L.InvalidArgument, match="invalid decoder configuration"):
        api.DecoderCompiler.compile(bad, _weights(api.decoder_config(), rng))
    bad_moe = api.decoder_config(moe=True, experts=2, top_k=3)
    with pytest.raises(L.InvalidArgument, match="invalid decoder MoE configuration"):
        api.DecoderCompiler.compile(bad_moe, {})
    with pytest.raises(L.InvalidArgument, match="invalid decoder context sequence"):
        api.DecoderCompiler.compile(api.decoder_config(context_sequence=-1), {})


def test_compile_requires_fusion_patterns():
    c = api.decoder_config(1, 4, 16, 32, 4, 2, 4)
    with pytest.raises(L.InvalidArgument, match="decoder graph is missing required fusion patterns"):
        api.DecoderCompiler.compile(c, _weights(c, np.random.default_rng(0)), stablehlo_text=NO_QKV_TEXT)
    # a MoE text lacks the gate/up pattern, which a dense plan requires
    with pytest.raises(L.InvalidArgument, match="missing required fusion patterns"):
        api.DecoderCompiler.compile(c, _weights(c, np.random.default_rng(0)), stablehlo_text=MOE_TEXT)


def test_compile_rejects_bad_shard():
    c = api.decoder_config(1, 4, 16, 32, 4, 2, 4)
    with pytest.raises(L.InvalidArgument, match="tensor-parallel size does not divide"):
        api.DecoderCompiler.compile(c, _weights(c, np.random.default_rng(0)), options=api.compile_options(tp_size=3))


@pytest.mark.parametrize("name", ["moe_small", "moe_medium"])
def test_plan_moe_tasks_matches_fixture(name, port):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    c = api.moe_config(*[int(v) for v in z["config"]])
    tasks = api.plan_moe_tasks(c, z["counts"])
    assert np.array_equal(tasks, z["tasks"])
    # load-aware split: no task longer than the threshold, rows covered exactly once
    split = api.plan_moe_tasks(c, z["counts"], split_threshold=2)
    assert np.all(split[:, 2] - split[:, 1] <= 2) and np.all(split[:, 2] > split[:, 1])
    assert (split[:, 2] - split[:, 1]).sum() == z["counts"].sum()
    from oracle import binding as ob
    assert np.array_equal(split, port.plan_moe_tasks(ob.MoeConfig(*[int(v) for v in z["config"]]), z["counts"], 2))


def test_rope_table_matches_reference_formula(port):
    from oracle import binding as ob
    seq, dim, theta = 6, 8, 500000.0
    cos, sin = np.zeros((seq, dim // 2), np.float32), np.zeros((seq, dim // 2), np.float32)
    L.check(L.load().sfb_rope_table(seq, dim, C.c_float(theta), cos.ctypes.data_as(L.f32p), sin.ctypes.data_as(L.f32p)))
    # rotate (1, 0) pairs with the oracle: the result is (cos, sin) of the table entry
    c = ob.decoder_config(1, seq, dim, 8, 1, 1, dim, rope_theta=theta)
    fused = np.zeros((seq, 3 * dim), np.float32)
    fused[:, 0:dim:2] = 1.0
    q, _, _ = port.split_qkv_rope(c, fused)
    assert np.array_equal(q[0, 0, :, 0::2], cos) and np.array_equal(q[0, 0, :, 1::2], sin)


def test_weight_shards():
    a = np.arange(6 * 8, dtype=np.float32).reshape(6, 8)
    assert np.array_equal(api.shard_columns(a, 1, 4), a[:, 2:4])
    assert np.array_equal(api.shard_rows(a, 2, 3), a[4:6])
    with pytest.raises(L.InvalidArgument):
        api.shard_columns(a, 0, 3)


# ---- decoder benchmark matrix (realistic_decoder_profiles / CSV writers) ---------------------------
def golden_profiles():
    lines = open(os.path.join(GOLDEN, "decoder_profiles.txt")).read().splitlines()
    rows = [l.split("|") for l in lines if not l.startswith("#")]
    tagged = {l.split(" ", 1)[0]: l.split(" ", 1)[1] for l in lines if l.startswith("#")}
    return rows, tagged


def test_profile_matrix_matches_reference_fixture():
    rows, _ = golden_profiles()
    profiles = api.realistic_decoder_profiles()
    assert len(profiles) == len(rows) == 24
    names = {0: "uniform", 1: "moderate-skew", 2: "heavy-skew"}
    for p, row in zip(profiles, rows):
        c = p.config
        got = [p.name.decode(), c.batch, c.sequence, c.context_sequence, c.hidden, c.intermediate, c.query_heads,
               c.kv_heads, c.head_dim, c.ffn_moe, c.experts, c.top_k, names[p.routing], p.estimated_flops,
               p.estimated_weight_bytes, p.estimated_activation_bytes]
        assert [str(v) for v in got] == row
    assert profiles[0].config.hidden == 512 and profiles[14].config.hidden == 4096   # the reference's own checks


def test_benchmark_csv_schemas_and_compile_only_row_match_reference(tmp_path):
    _, tagged = golden_profiles()
    profile = api.realistic_decoder_profiles()[14]
    record = api.benchmark_decoder_profile(profile, max_real_flops=1, max_real_weight_bytes=1)   # no device work
    assert record.evidence == L.EVIDENCE_COMPILE_ONLY and record.measured.milliseconds == 0.0
    assert record.profile.estimated_weight_bytes > 0
    path = tmp_path / "out" / "decoder.csv"
    api.write_decoder_benchmark_csv(path, [record])
    header, row = path.read_text().splitlines()
    assert header == tagged["#benchmark_header"]
    assert "profile,evidence" in header and "tokens_per_second" in header and "compile-only" in row
    want = tagged["#compile_only_row"].split(",")
    got = row.split(",")
    assert len(got) == len(want) == len(header.split(","))
    # all columns but the reference's host plan figures (workspace, compile and memory planning times)
    skip = {header.split(",").index(n) for n in ("workspace_bytes", "compile_ms", "memory_planning_ms", "memory_planning_pct")}
    assert [g for i, g in enumerate(got) if i not in skip] == [w for i, w in enumerate(want) if i not in skip]
    api.write_decoder_plan_candidates_csv(tmp_path / "candidates.csv", [record])
    assert (tmp_path / "candidates.csv").read_text().splitlines() == [tagged["#candidates_header"]]
    api.write_decoder_benchmark_csv(tmp_path / "empty.csv", [])
    assert (tmp_path / "empty.csv").read_text().splitlines() == [tagged["#benchmark_header"]]


def test_seeded_generators_match_reference_fixtures():
    z = np.load(os.path.join(GOLDEN, "routing_traces.npz"))
    for distribution, experts in ((0, 8), (1, 8), (2, 16)):
        ids, weights, counts = api.make_routing_trace(api.moe_config(32, 512, 1376, experts, 2), distribution, 103)
        assert np.array_equal(ids, z[f"ids{distribution}"]) and np.array_equal(counts, z[f"counts{distribution}"])
        assert np.array_equal(weights, z[f"weights{distribution}"])
    dense = np.load(os.path.join(GOLDEN, "decoder_dense.npz"))     # make_decoder_data(config, 81)
    c = api.decoder_config(batch=1, sequence=4, hidden=16, intermediate=32, query_heads=4, kv_heads=2, head_dim=4)
    assert np.array_equal(api.make_decoder_input(c, 81).ravel(), dense["in_input"].ravel())
    with pytest.raises(L.InvalidArgument):
        api.make_routing_trace(api.moe_config(4, 8, 8, 2, 3), 0, 1)


def test_malformed_routing_trace_is_rejected_on_the_host(sfb):
    """A caller's routing trace indexes device memory by expert id and places rows by its counts, so it is
    checked on the host before anything is copied or launched: an id outside [0, experts), counts that are
    not the histogram of the ids, or a missing array give the reference's invalid_argument ("routing trace
    does not match MoE configuration", src/moe_compiler.cpp:498-501).  No device is needed to be refused."""
    import ctypes as C
    from schedforge_b200 import api
    config = api.moe_config(4, 8, 16, 4, 2)
    x = np.zeros((4, 8), np.float32)
    weights = np.full((4, 2), 0.5, np.float32)
    good = np.array([[0, 1], [2, 3], [0, 2], [1, 3]], np.int32)
    counts = np.array([2, 2, 2, 2], np.int32)
    outside = good.copy()
    outside[2, 1] = 4
    negative = good.copy()
    negative[0, 0] = -1
    for ids, cnt in ((outside, counts), (negative, counts), (good, np.array([3, 1, 2, 2], np.int32))):
        with pytest.raises(sfb.InvalidArgument, match="routing trace does not match MoE configuration"):
            api.dispatch_tokens(config, x, ids, weights, cnt)
        w = np.zeros((4, 8, 16), np.float32)
        with pytest.raises(sfb.InvalidArgument, match="routing trace does not match MoE configuration"):
            api.execute_moe(config, x, w, w, w.reshape(4, 16, 8), ids, weights, cnt)
    lib = sfb.load()
    offsets, tokens = np.zeros(5, np.int32), np.zeros(8, np.int32)
    ip, fp = C.POINTER(C.c_int), C.POINTER(C.c_float)
    status = lib.sfb_moe_dispatch_tokens(C.byref(config), x.ctypes.data_as(fp), 4, good.ctypes.data_as(ip), None,
                                         counts.ctypes.data_as(ip), 0, None, offsets.ctypes.data_as(ip),
                                         tokens.ctypes.data_as(ip), tokens.ctypes.data_as(ip), weights.ctypes.data_as(fp))
    assert status == sfb.SFB_INVALID_ARGUMENT


@pytest.mark.parametrize("name", ["decoder_dense", "decoder_moe", "decoder_decode", "decoder_moe_medium"])
def test_make_decoder_data_equals_the_reference_generator(sfb, name):
    """sfb_make_decoder_data against the tensors the reference's make_decoder_data produced for the same
    configuration and seed (stored in the golden fixtures as in_*): every weight stream bit for bit."""
    from schedforge_b200 import api
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    fields = [f for f, _ in sfb.DecoderConfig._fields_]
    values = [float(v) if f in ("rms_epsilon", "rope_theta") else int(v) for f, v in zip(fields, z["config"])]
    config = sfb.DecoderConfig(*values)
    data = api.make_decoder_data(config, int(z["seed"]))
    compared = 0
    for key in z.files:
        if not key.startswith("in_"):
            continue
        got = data[key[3:]]
        assert got.shape == z[key].reshape(-1).shape and np.array_equal(got, z[key].reshape(-1)), key
        compared += 1
    assert compared >= 10


def test_row_chunks_of_the_pipelined_execute_fill_whole_rounds_of_tiles(sfb):
    """sfb_decoder_row_chunks: the chunk plan of the host-buffer prefill pass is host arithmetic.  The headline shape
    (8192 rows, 4096 columns, 148 SMs) runs as 4 9 18 18 9 6 blocks of 128 rows: 9 blocks x 16 tiles = 144 tiles of
    the O / Down GEMMs per round of 148 SMs, short chunks where nothing overlaps the copies."""
    lib = sfb.load()

    def chunks(rows, hidden, sms):
        out = (C.c_int * 64)()
        n = lib.sfb_decoder_row_chunks(rows, hidden, sms, out, 64)
        assert lib.sfb_decoder_row_chunks(rows, hidden, sms, None, 0) == n     # the count alone
        return list(out[:n])

    assert chunks(8192, 4096, 148) == [4, 9, 18, 18, 9, 6]
    assert chunks(4096, 4096, 148) == [4, 9, 9, 10]          # two sequences of 2048: the third chunk spans both
    assert chunks(3840, 1792, 148) == [4, 21, 5]             # tests/test_decoder.py: three sequences of 1280
    assert chunks(2048, 4096, 148) == []                     # too few rows for a middle chunk: whole sequences instead
    assert chunks(8192, 4100, 148) == [] and chunks(8200, 4096, 148) == [] and chunks(8192, 4096, 0) == []
    for rows, hidden, sms in [(8192, 4096, 148), (65536, 4096, 148), (16384, 8192, 132), (12288, 2048, 148), (5120, 5120, 148)]:
        got = chunks(rows, hidden, sms)
        unit = sms // (hidden // 256)
        assert sum(got) == rows // 128 and got[0] == 4 and 4 <= got[-1] < 4 + unit and len(got) <= 12
        assert all(size % unit == 0 for size in got[1:-1])

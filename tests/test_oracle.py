"""Pins the oracle.  The C++ restatement (oracle/port.cpp) must reproduce

  * the committed golden vectors under tests/golden/ (generated from the reference itself
    by tests/golden/make_golden.py), and
  * the reference build oracle/_ref/libsfref.so directly, when it is present,

bit for bit for integers and for every float path (the port follows the reference's
operation order and both are compiled with -ffp-contract=off)."""
import json
import os

import numpy as np
import pytest

from oracle import binding as ob

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def decoder_case(name):
    z = load(name)
    c = ob.DecoderConfig()
    for (field, ctype), value in zip(c._fields_, z["config"]):
        setattr(c, field, float(value) if field in ("rms_epsilon", "rope_theta") else int(value))
    data = {k[3:]: z[k] for k in z.files if k.startswith("in_")}
    return c, data, z


DECODER_CASES = ["decoder_dense", "decoder_moe", "decoder_decode", "decoder_cfg1_shape", "decoder_batched",
                 "decoder_moe_medium"]


@pytest.mark.parametrize("name", DECODER_CASES)
def test_port_decoder_layer_matches_golden(port, name):
    c, data, z = decoder_case(name)
    assert np.array_equal(port.decoder_layer(c, data, native=False), z["out_reference"])
    assert np.array_equal(port.decoder_layer(c, data, native=True, threads=2), z["out_native"])
    # the reference's own acceptance bar between its native path and its scalar reference
    assert np.max(np.abs(z["out_native"] - z["out_reference"])) < 1e-3


@pytest.mark.parametrize("name", DECODER_CASES[:3])
def test_port_decoder_layer_matches_reference_build(port, ref, name):
    c, data, _ = decoder_case(name)
    for seed in (1, 2):
        fresh = ref.make_decoder_data(c, seed)
        assert np.array_equal(port.decoder_layer(c, fresh, native=False), ref.decoder_layer(c, fresh, native=False))
        assert np.array_equal(port.decoder_layer(c, fresh, native=True, threads=2),
                              ref.decoder_layer(c, fresh, native=True, threads=2))


def attention_case(name):
    z = load(name)
    c = ob.AttentionConfig(*[int(v) for v in z["config"][:8]], float(z["config"][8]))
    return c, z


@pytest.mark.parametrize("name", ["attention_causal_gqa", "attention_dynamic", "attention_noncausal", "attention_d64"])
def test_port_attention_prefill_matches_golden(port, name):
    c, z = attention_case(name)
    assert np.array_equal(port.attention_reference(c, z["q"], z["k"], z["v"]), z["out_reference"])
    assert np.array_equal(port.attention_io_aware(c, z["q"], z["k"], z["v"], 4, 3), z["out_io_aware"])
    assert np.array_equal(port.attention_materialized(c, z["q"], z["k"], z["v"]), z["out_materialized"])
    assert np.max(np.abs(z["out_io_aware"] - z["out_reference"])) < 1e-4  # the reference's bar


@pytest.mark.parametrize("name", ["attention_decode_gqa", "attention_decode_mqa"])
def test_port_split_kv_decode_matches_golden(port, name):
    c, z = attention_case(name)
    # the reference ran with 4 threads: split_kv = clamp(max(2, 11/128), 2, 4) = 2, kv_tile = 11
    got = port.attention_split_kv(c, z["q"], z["k"], z["v"], splits=2, kv_tile=11)
    assert np.array_equal(got, z["out_decode"])
    assert np.max(np.abs(got - z["out_reference"])) < 1e-4


def test_port_paged_kv_matches_golden(port):
    z = load("paged_kv")
    cache = port.paged_create(1, 2, 4, 4, 4, 12)
    cache.append(z["keys"], z["values"], 7)
    info = cache.info()
    assert info["length"] == 7 and len(info["page_table"]) == 2
    assert np.array_equal(info["page_table"], z["page_table"])       # pages come from the back: [2, 1]
    assert np.array_equal(info["free_pages"], z["free_pages"])
    gk, gv = cache.gather()
    assert np.array_equal(gk, z["keys"]) and np.array_equal(gv, z["values"])   # gather == input, exactly
    sk, sv = cache.storage()
    assert np.array_equal(sk, z["storage_keys"]) and np.array_equal(sv, z["storage_values"])
    c = ob.AttentionConfig(1, 4, 2, 1, 7, 4, 4, 1, 0.0)
    assert np.array_equal(cache.decode(c, z["query"]), z["decode_out"])
    assert np.max(np.abs(cache.decode(c, z["query"], two_pass=True) - z["decode_out"])) < 1e-5
    with pytest.raises(ob.OracleError):
        cache.release([int(info["page_table"][0])])                   # active page guard
    cache.truncate(3)
    info = cache.info()
    assert info["length"] == 3
    assert np.array_equal(info["page_table"], z["truncated_page_table"])
    assert np.array_equal(info["free_pages"], z["truncated_free_pages"])
    with pytest.raises(ob.OracleError):
        cache.append(z["keys"], z["values"], 10)                      # capacity exceeded
    cache.close()


@pytest.mark.parametrize("name", ["moe_small", "moe_medium"])
def test_port_moe_matches_golden(port, name):
    z = load(name)
    c = ob.MoeConfig(*[int(v) for v in z["config"]])
    ids, weights, counts = port.route_topk(c, z["in_input"], z["in_router_weight"])
    assert np.array_equal(ids, z["expert_ids"]) and np.array_equal(counts, z["counts"])
    assert np.array_equal(weights, z["expert_weights"])
    assert counts.sum() == c.tokens * c.top_k
    assert np.allclose(weights.sum(axis=1), 1.0, atol=1e-5)
    values, offsets, token_ids, slots, rw = port.dispatch_tokens(c, z["in_input"], ids, weights, counts)
    assert np.array_equal(offsets, z["offsets"]) and offsets[-1] == c.tokens * c.top_k
    assert np.array_equal(token_ids, z["token_ids"]) and np.array_equal(slots, z["route_slots"])
    assert np.array_equal(values, z["dispatched"]) and np.array_equal(rw, z["routing_weights"])
    assert np.array_equal(port.plan_moe_tasks(c, counts), z["tasks"])
    assert np.array_equal(port.moe_reference(c, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], ids, weights),
                          z["out_reference"])
    assert np.array_equal(port.moe_grouped(c, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], ids, weights, counts),
                          z["out_native"])


def test_port_pieces_match_reference_build(port, ref):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((9, 40)).astype(np.float32)
    w = rng.standard_normal(40).astype(np.float32)
    assert np.array_equal(port.rms_norm(x, w, 1e-5), ref.rms_norm(x, w, 1e-5))
    a = rng.standard_normal((13, 70)).astype(np.float32)
    b = rng.standard_normal((70, 37)).astype(np.float32)
    assert np.array_equal(port.matmul(a, b, fma=False), ref.matmul(a, b, fma=False))
    assert np.array_equal(port.matmul(a, b, fma=True), ref.matmul(a, b, fma=True, threads=2))
    c = ob.decoder_config(2, 5, 24, 16, 4, 2, 6, rope_theta=500000.0)
    fused = rng.standard_normal((10, 24 + 2 * 12)).astype(np.float32)
    for got, want in zip(port.split_qkv_rope(c, fused), ref.split_qkv_rope(c, fused)):
        assert np.array_equal(got, want)
    gu = rng.standard_normal((6, 14)).astype(np.float32)
    assert np.array_equal(port.swiglu(gu, 7), ref.swiglu(gu, 7))
    assert np.array_equal(port.round_bf16(x), ref.round_bf16(x))


def test_bf16_rounding_known_answers(port):
    z = np.load(os.path.join(GOLDEN, "bf16_round.npz"))
    assert np.array_equal(port.round_bf16(z["x"]), z["y"])
    assert port.round_bf16(np.array([1.00390625], np.float32))[0] == 1.0          # tie -> even
    assert port.round_bf16(np.array([1.01171875], np.float32))[0] == 1.015625     # tie -> even (up)


def test_port_router_bias_is_one_added_term(port):
    """The bias variant (no counterpart in the reference) equals routing on logits+bias."""
    rng = np.random.default_rng(3)
    c = ob.MoeConfig(50, 32, 8, 8, 2)
    x = rng.standard_normal((50, 32)).astype(np.float32)
    w = (rng.standard_normal((32, 8)) * 0.1).astype(np.float32)
    ids0, _, counts0 = port.route_topk(c, x, w, bias=np.zeros(8, np.float32))
    ids1, _, counts1 = port.route_topk(c, x, w)
    assert np.array_equal(ids0, ids1) and np.array_equal(counts0, counts1)
    bias = np.array([5, 0, 0, 0, 0, 0, 0, -5], np.float32)
    ids2, _, counts2 = port.route_topk(c, x, w, bias=bias)
    assert counts2[0] == 50 and counts2[7] == 0 and counts2.sum() == 100


def test_importer_fixture_is_consistent(ref):
    import sys
    sys.path.insert(0, GOLDEN)
    from stablehlo_texts import DECODER_TEXT, MOE_TEXT, NO_QKV_TEXT
    want = json.load(open(os.path.join(GOLDEN, "importer.json")))
    assert ref.import_stablehlo(DECODER_TEXT) == want["decoder"]
    assert ref.import_stablehlo(MOE_TEXT, moe=True) == want["moe"]
    assert ref.import_stablehlo(NO_QKV_TEXT) == want["no_qkv"]
    assert want["decoder"]["operations"] == 25 and want["decoder"]["fused_qkv"] and want["decoder"]["fused_gate_up"]


@pytest.mark.parametrize("name", ["moe_small", "moe_medium", "reference_test_shape"])
def test_int8_expert_round_trip_reproduces_the_reference_quantized_moe(port, ref, name):
    """quantize_moe_weights + execute_quantized_moe of the reference build against the oracle's MoE run on
    q * scale expert weights; on the shape of the reference's own INT8 MoE test its bar (0.2) holds too."""
    if name == "reference_test_shape":  # tests/test_schedforge.cpp:902-914 of the reference
        c = ob.MoeConfig(8, 16, 24, 4, 2)
        d = ref.make_moe_data(c, 91)
        x, w1, w3, w2 = d["input"], d["w1"], d["w3"], d["w2"]
        ids, weights, counts = ref.route_topk(c, x, d["router_weight"])
    else:
        z = load(name)
        c = ob.MoeConfig(*[int(v) for v in z["config"]])
        x, w1, w3, w2 = z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"]
        ids, weights, counts = z["expert_ids"], z["expert_weights"], z["counts"]
    want, max_error = ref.moe_quantized(c, x, w1, w3, w2, ids, weights, counts)
    if name == "reference_test_shape":
        assert max_error < 0.2
    q1 = ob.int8_expert_weights(w1, c.experts, c.hidden, c.intermediate)
    q3 = ob.int8_expert_weights(w3, c.experts, c.hidden, c.intermediate)
    q2 = ob.int8_expert_weights(w2, c.experts, c.intermediate, c.hidden)
    got = port.moe_reference(c, x, q1, q3, q2, ids, weights)
    assert np.max(np.abs(got - want)) <= 2e-5 * max(1.0, np.max(np.abs(want)))
    assert np.max(np.abs(got - port.moe_reference(c, x, w1, w3, w2, ids, weights))) > 1e-6   # the weights did change


@pytest.mark.parametrize("name", ["decoder_dense", "decoder_decode", "decoder_batched", "decoder_cfg1_shape"])
def test_int8_weight_round_trip_reproduces_the_reference_quantized_layer(port, ref, name):
    """The reference's weight-only INT8 layer (quantize_decoder_weights + execute_quantized_decoder_layer)
    against the oracle layer run on q * scale weights: equal up to the association of `x * q * scale`,
    and, on the reference's own test shapes, inside its bar (0.15 absolute against its unquantized scalar layer)."""
    c, data, _ = decoder_case(name)
    dec = ref.decoder_create(c, data)
    try:
        want, max_error = dec.quantized(per_channel=True)
    finally:
        dec.close()
    if name in ("decoder_dense", "decoder_decode"):  # the shapes of the reference's own INT8 test
        assert max_error < 0.15
    got = port.decoder_layer(c, ob.int8_weight_data(c, data), native=False)
    assert np.max(np.abs(got - want)) <= 2e-5 * max(1.0, np.max(np.abs(want)))
    # the round trip really changes the weights, and a second round trip changes nothing
    assert np.max(np.abs(got - port.decoder_layer(c, data, native=False))) > 1e-5
    again = ob.int8_weight_data(c, ob.int8_weight_data(c, data))
    assert np.array_equal(again["down_weight"], ob.int8_weight_data(c, data)["down_weight"])

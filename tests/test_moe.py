"""MoE routing chain parity: bit-exact integers (top-k ids, histogram, prefix sums, dispatch
permutation) against the oracle, expert FFN and weighted combine within tolerance."""
import os

import numpy as np
import pytest

from conftest import rel_err
from oracle import binding as ob
from schedforge_b200 import api, lib as L

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def moe_fixture(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    vals = [int(v) for v in z["config"]]
    return api.moe_config(*vals), ob.MoeConfig(*vals), z


@pytest.mark.parametrize("name", ["moe_small", "moe_medium"])
def test_routing_chain_matches_reference_fixture(name):
    c, _, z = moe_fixture(name)
    ids, weights, counts = api.route_topk(c, z["in_input"], z["in_router_weight"], dtype=L.F32)
    assert np.array_equal(ids, z["expert_ids"]) and np.array_equal(counts, z["counts"])     # bit-exact integers
    assert counts.sum() == c.tokens * c.top_k
    assert np.allclose(weights, z["expert_weights"], rtol=1e-5, atol=1e-7)
    assert np.allclose(weights.sum(axis=1), 1.0, atol=1e-5)
    values, offsets, token_ids, slots, rw = api.dispatch_tokens(c, z["in_input"], z["expert_ids"],
                                                                z["expert_weights"], z["counts"], dtype=L.F32)
    assert np.array_equal(offsets, z["offsets"]) and offsets.size == c.experts + 1
    assert offsets[-1] == c.tokens * c.top_k
    assert np.array_equal(token_ids, z["token_ids"]) and np.array_equal(slots, z["route_slots"])
    assert np.array_equal(values, z["dispatched"]) and np.array_equal(rw, z["routing_weights"])


@pytest.mark.parametrize("name", ["moe_small", "moe_medium"])
def test_expert_ffn_fp32_matches_reference_fixture(name):
    c, _, z = moe_fixture(name)
    out, ms = api.execute_moe(c, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], z["expert_ids"],
                              z["expert_weights"], z["counts"], dtype=L.F32)
    assert np.max(np.abs(out - z["out_reference"])) < 1e-3        # the reference's bar
    assert rel_err(out, z["out_reference"]) < 1e-4
    assert rel_err(out, z["out_native"]) < 1e-5
    with pytest.raises(L.InvalidArgument, match="runtime token count exceeds compiled MoE guard"):
        small = api.moe_config(c.tokens - 1, c.hidden, c.intermediate, c.experts, c.top_k)
        api.execute_moe(small, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], z["expert_ids"],
                        z["expert_weights"], z["counts"])


@pytest.mark.parametrize("name", ["moe_small", "moe_medium"])
def test_int8_experts_match_oracle_on_round_tripped_weights(port, name):
    """execute_quantized_moe: bf16 arithmetic on q * scale expert weights against the oracle's fp32 MoE on the
    same weights (2e-2 of the largest output), and inside the reference's own bar (0.2 absolute) against the
    unquantized fixture output."""
    c, oc, z = moe_fixture(name)
    args = (z["expert_ids"], z["expert_weights"], z["counts"])
    out, ms = api.execute_quantized_moe(c, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], *args)
    bf = lambda a: port.round_bf16(np.asarray(a, np.float32))
    q1 = ob.int8_expert_weights(bf(z["in_w1"]), oc.experts, oc.hidden, oc.intermediate)
    q3 = ob.int8_expert_weights(bf(z["in_w3"]), oc.experts, oc.hidden, oc.intermediate)
    q2 = ob.int8_expert_weights(bf(z["in_w2"]), oc.experts, oc.intermediate, oc.hidden)
    want = port.moe_reference(oc, bf(z["in_input"]), q1, q3, q2, z["expert_ids"], z["expert_weights"])
    assert rel_err(out, want) < 2e-2
    assert np.max(np.abs(out - z["out_reference"])) < 0.2
    plain, _ = api.execute_moe(c, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], *args, dtype=L.BF16)
    assert not np.array_equal(plain, out)
    with pytest.raises(L.InvalidArgument, match="per-output-channel"):
        api.execute_quantized_moe(c, z["in_input"], z["in_w1"], z["in_w3"], z["in_w2"], *args, per_channel=False)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("tokens,hidden,experts,top_k,bias", [(1000, 512, 8, 2, False), (333, 260, 16, 4, True),
                                                              (4096, 1024, 8, 2, True)])
def test_router_bit_exact_against_oracle(port, dtype, tokens, hidden, experts, top_k, bias):
    rng = np.random.default_rng(tokens)
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    w = (rng.standard_normal((hidden, experts)) * 0.02).astype(np.float32)
    b = rng.standard_normal(experts).astype(np.float32) if bias else None   # skewed loads
    if dtype == L.BF16:
        x, w = port.round_bf16(x), port.round_bf16(w)
    c, oc = api.moe_config(tokens, hidden, 64, experts, top_k), ob.MoeConfig(tokens, hidden, 64, experts, top_k)
    want_ids, want_w, want_counts = port.route_topk(oc, x, w, bias=b)
    ids, weights, counts = api.route_topk(c, x, w, router_bias=b, dtype=dtype)
    if port.last_tie_tokens == 0:
        assert np.array_equal(ids, want_ids) and np.array_equal(counts, want_counts)
    else:  # exact ties in exp space make the reference's order history-dependent: compare as sets
        assert np.array_equal(np.sort(ids, axis=1), np.sort(want_ids, axis=1))
    assert np.allclose(weights, want_w, rtol=2e-5, atol=1e-7)
    # dispatch permutation on the same routing: bit-exact
    _, offsets, token_ids, slots, rw = api.dispatch_tokens(c, None, want_ids, want_w, want_counts, copy_values=False)
    _, o_off, o_tok, o_slot, o_rw = port.dispatch_tokens(oc, x, want_ids, want_w, want_counts, copy_values=False)
    assert np.array_equal(offsets, o_off) and np.array_equal(token_ids, o_tok) and np.array_equal(slots, o_slot)
    assert np.array_equal(rw, o_rw)


@pytest.mark.parametrize("backend", [L.GEMM_SIMT, L.GEMM_TCGEN05])
def test_expert_ffn_bf16_grouped_gemm(port, backend):
    tokens, hidden, inter, experts, top_k = 512, 256, 384, 8, 2
    rng = np.random.default_rng(2)
    x = port.round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32))
    w1 = port.round_bf16((rng.standard_normal((experts, hidden, inter)) * 0.05).astype(np.float32))
    w3 = port.round_bf16((rng.standard_normal((experts, hidden, inter)) * 0.05).astype(np.float32))
    w2 = port.round_bf16((rng.standard_normal((experts, inter, hidden)) * 0.05).astype(np.float32))
    router = (rng.standard_normal((hidden, experts)) * 0.05).astype(np.float32)
    bias = np.array([2.0, 1.0, 0, 0, 0, -1.0, -2.0, -9.0], np.float32)  # skew incl. a (nearly) empty expert
    oc = ob.MoeConfig(tokens, hidden, inter, experts, top_k)
    ids, weights, counts = port.route_topk(oc, x, router, bias=bias)
    want = port.moe_grouped(oc, x, w1, w3, w2, ids, weights, counts)
    out, _ = api.execute_moe(api.moe_config(tokens, hidden, inter, experts, top_k), x, w1, w3, w2, ids, weights,
                             counts, dtype=L.BF16, gemm_backend=backend)
    assert rel_err(out, want) < 2e-2


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
def test_compiled_moe_plan_keeps_its_weights_and_runs_repeatedly(port, dtype):
    """sfb_moe_compile / sfb_moe_plan_execute: the expert weights are packed and uploaded once; passes with a
    routing trace, passes that route themselves (router bias included), a shorter token count and the reference's
    guard for a longer one.  Results equal the one-call form and the oracle."""
    rng = np.random.default_rng(12)
    t, h, i, e, k = 192, 128, 256, 8, 2
    c, oc = api.moe_config(t, h, i, e, k), ob.MoeConfig(t, h, i, e, k)
    x = port.round_bf16(rng.standard_normal((t, h)).astype(np.float32))
    w1 = port.round_bf16((rng.standard_normal((e, h, i)) * 0.05).astype(np.float32))
    w3 = port.round_bf16((rng.standard_normal((e, h, i)) * 0.05).astype(np.float32))
    w2 = port.round_bf16((rng.standard_normal((e, i, h)) * 0.05).astype(np.float32))
    router = port.round_bf16((rng.standard_normal((h, e)) * 0.1).astype(np.float32))
    bias = rng.standard_normal(e).astype(np.float32)
    tol = 1e-4 if dtype == L.F32 else 2e-2
    plan = api.MoeExecutablePlan(c, w1, w3, w2, router, bias, dtype=dtype)
    ids, weights, counts = port.route_topk(oc, x, router, bias)
    want = port.moe_grouped(oc, x, w1, w3, w2, ids, weights, counts)
    routed, ms = plan.execute(x)                                  # the plan routes itself
    assert rel_err(routed, want) < tol and ms > 0
    traced, _ = plan.execute(x, trace=(ids, weights, counts))     # DecoderData::routing_trace style
    assert rel_err(traced, want) < tol
    one_call, _ = api.execute_moe(c, x, w1, w3, w2, ids, weights, counts, dtype=dtype)
    assert np.array_equal(traced, one_call)
    # fewer tokens than compiled: allowed; more: the reference's guard
    half = t // 2
    ids_h, weights_h, counts_h = port.route_topk(ob.MoeConfig(half, h, i, e, k), x[:half], router, bias)
    short, _ = plan.execute(x[:half], trace=(ids_h, weights_h, counts_h))
    assert rel_err(short, port.moe_grouped(ob.MoeConfig(half, h, i, e, k), x[:half], w1, w3, w2, ids_h, weights_h, counts_h)) < tol
    again, _ = plan.execute(x)
    assert np.array_equal(again, routed)
    with pytest.raises(L.InvalidArgument, match="runtime token count exceeds compiled MoE guard"):
        plan.execute(np.concatenate([x, x]))
    plan.close()
    unrouted = api.MoeExecutablePlan(c, w1, w3, w2, dtype=dtype)
    with pytest.raises(L.InvalidArgument, match="no router weights"):
        unrouted.execute(x)
    unrouted.close()

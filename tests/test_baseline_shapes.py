"""Parity at the shapes the headline numbers are quoted on.

The Llama-3-8B-shaped dense layer (hidden 4096, 32 query / 8 KV heads of 128, SwiGLU FFN 14336, RoPE theta
500000), the Mixtral-shaped MoE layer (8 experts, top-2, expert FFN 14336, router bias) and the paged decode
case (batch 64, contexts uniform in [512, 8192], 16-token blocks, permuted block table) run on the device at
their real widths and are compared with the CPU oracle on bf16-rounded data.  Only the token counts are cut
down to what the oracle finishes in seconds.  Bars: 2e-2 max-abs relative for bf16 layer outputs, bit-exact
for expert ids, histograms, prefix sums and the dispatch permutation."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err
from oracle import binding as ob
from schedforge_b200 import api, lib as L

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2
LLAMA = dict(hidden=4096, intermediate=14336, query_heads=32, kv_heads=8, head_dim=128, rms_epsilon=1e-5,
             rope_theta=500000.0)


def _normal(shape, std, seed):
    """~N(0, std) rounded to bf16 (round to nearest even, as convert_to_bf16 of the reference), float32 on the host."""
    import torch
    g = torch.Generator().manual_seed(seed)
    t = torch.empty(shape, dtype=torch.float32).normal_(0.0, std, generator=g)
    return t.bfloat16().float().numpy()


@pytest.fixture(scope="module")
def llama_weights():
    h, i, kv = LLAMA["hidden"], LLAMA["intermediate"], LLAMA["kv_heads"] * LLAMA["head_dim"]
    shapes = dict(query_weight=(h, h), key_weight=(h, kv), value_weight=(h, kv), output_weight=(h, h),
                  gate_weight=(h, i), up_weight=(h, i), down_weight=(i, h))
    data = {k: _normal(s, 0.02, 100 + n) for n, (k, s) in enumerate(shapes.items())}
    rng = np.random.default_rng(5)
    data["rms1_weight"] = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
    data["rms2_weight"] = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
    return data


@pytest.fixture(scope="module")
def llama_prefill_b2_s1024(port, llama_weights):
    """Input and oracle output of the dense layer on two sequences of 1024 tokens (shared by two tests)."""
    kw = dict(LLAMA, batch=2, sequence=1024)
    data = dict(llama_weights, input=_normal((2048, 4096), 1.0, 1))
    want = port.decoder_layer(ob.decoder_config(**kw), data, native=True)
    return kw, data, want


def test_llama_layer_prefill_pipelined_row_chunks(llama_prefill_b2_s1024, llama_weights):
    """Two sequences of 1024 tokens: sfb_decoder_execute runs four row chunks of 512 (copies overlapped,
    attention on row slices of a sequence), each GEMM at N = 6144 / 4096 / 28672 and K = 4096 / 14336."""
    kw, data, want = llama_prefill_b2_s1024
    plan = api.DecoderCompiler.compile(api.decoder_config(**kw), llama_weights)
    out, result = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert result.kernel_launches >= 4 * 6   # four chunks went through the layer
    plan.close()


def test_llama_layer_prefill_pipelined_chunks_across_sequences(port, llama_weights):
    """Two sequences of 2048 tokens (half the headline batch): sfb_decoder_execute runs chunks of 4, 9, 9 and 10
    row blocks (9 x 128 rows = 144 output tiles of the O and Down GEMMs on 148 SMs); the third chunk holds the
    end of the first sequence and the start of the second."""
    kw = dict(LLAMA, batch=2, sequence=2048)
    data = dict(llama_weights, input=_normal((4096, 4096), 1.0, 3))
    want = port.decoder_layer(ob.decoder_config(**kw), data, native=True)
    plan = api.DecoderCompiler.compile(api.decoder_config(**kw), llama_weights)
    out, result = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert result.kernel_launches >= 4 * 6 + 1   # four chunks went through the layer, one of them with two attention launches
    plan.close()


@pytest.mark.parametrize("norm_fusion", [False, True])
def test_llama_layer_prefill_one_shot(port, llama_weights, norm_fusion):
    """One sequence of 384 tokens through the unchunked path (the sample the CPU baseline of bench.py times), with
    stand-alone RMSNorm kernels and with both norms folded into the QKV and gate/up GEMMs."""
    kw = dict(LLAMA, batch=1, sequence=384)
    data = dict(llama_weights, input=_normal((384, 4096), 1.0, 2))
    want = port.decoder_layer(ob.decoder_config(**kw), data, native=True)
    plan = api.DecoderCompiler.compile(api.decoder_config(**kw), llama_weights, "", api.compile_options(norm_fusion=norm_fusion))
    out, _ = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert ("prologue=rms_norm_folded" in plan.dump()) == norm_fusion
    plan.close()


def test_llama_layer_decode_over_2048_cached_tokens(port, llama_weights):
    """Decode plan (few-row weight-streaming GEMMs on blocked weights, paged split-KV attention, permuted
    block table) with the reference's decode semantics: batch 8, 2048 cached tokens per sequence."""
    kw = dict(LLAMA, batch=8, sequence=1, context_sequence=2048)
    cache = (8, 8, 2048, 128)
    data = dict(llama_weights, input=_normal((8, 4096), 1.0, 3), cached_key=_normal(cache, 1.0, 4),
                cached_value=_normal(cache, 1.0, 5))
    want = port.decoder_layer(ob.decoder_config(**kw), data, native=True)
    weights = {k: v for k, v in data.items() if k != "input"}
    plan = api.DecoderCompiler.compile(api.decoder_config(**kw), weights, "", api.compile_options(seed_block_table=3))
    out, _ = plan.execute(data["input"])
    assert rel_err(out, want) < BF16_TOL
    assert "split_kv_decode" in plan.dump()
    plan.close()


def test_llama_layer_autoregressive_step_equals_last_prefill_token(port, llama_prefill_b2_s1024, llama_weights):
    """append_new_token at the Llama shape: the step over 1023 cached tokens (rotated keys of the prefill) must
    give the prefill's output for token 1023; RoPE at theta 500000 runs at position 1023."""
    kw, data, want_all = llama_prefill_b2_s1024
    ctx, hidden, kvw = 1023, 4096, 1024
    oc = ob.decoder_config(**kw)
    x = data["input"].reshape(2048, hidden)
    normalized = port.rms_norm(x, data["rms1_weight"], oc.rms_epsilon)
    wqkv = np.concatenate([data["query_weight"].reshape(hidden, hidden), data["key_weight"].reshape(hidden, kvw),
                           data["value_weight"].reshape(hidden, kvw)], axis=1)
    _, keys, values = port.split_qkv_rope(oc, port.matmul(normalized, wqkv, fma=True))  # [2, 8, 1024, 128]
    step = dict(llama_weights)
    step["cached_key"] = port.round_bf16(np.ascontiguousarray(keys[:, :, :ctx, :]))
    step["cached_value"] = port.round_bf16(np.ascontiguousarray(values[:, :, :ctx, :]))
    c = api.decoder_config(**dict(kw, sequence=1, context_sequence=ctx))
    plan = api.DecoderCompiler.compile(c, step, "", api.compile_options(append_new_token=True, seed_block_table=5,
                                                                        norm_fusion=True))
    last = np.ascontiguousarray(x.reshape(2, ctx + 1, hidden)[:, ctx, :])
    out, _ = plan.execute(last)
    want = want_all.reshape(2, ctx + 1, hidden)[:, ctx, :]
    assert rel_err(out, want) < BF16_TOL
    plan.close()


def test_mixtral_layer_with_router_bias(port):
    """Mixtral-shaped MoE layer at full width (8 experts of 4096 x 14336, top-2) on 256 tokens, with the
    per-expert router bias that skews the loads.  The routing chain is compared bit for bit on the very
    tensor the device routed; the layer output is compared with the oracle given the same routes."""
    h, i, e, k, t = 4096, 14336, 8, 2, 256
    kw = dict(LLAMA, batch=1, sequence=t, experts=e, top_k=k)
    kv = 1024
    data = {"input": _normal((t, h), 1.0, 11),
            "query_weight": _normal((h, h), 0.02, 12), "key_weight": _normal((h, kv), 0.02, 13),
            "value_weight": _normal((h, kv), 0.02, 14), "output_weight": _normal((h, h), 0.02, 15),
            "router_weight": _normal((h, e), 0.02, 16),
            "w1": _normal((e, h, i), 0.02, 17), "w3": _normal((e, h, i), 0.02, 18), "w2": _normal((e, i, h), 0.02, 19),
            "rms1_weight": np.ones(h, np.float32), "rms2_weight": np.ones(h, np.float32)}
    bias = np.random.default_rng(20).standard_normal(e).astype(np.float32)
    weights = {key: v for key, v in data.items() if key != "input"}
    weights["router_bias"] = bias
    plan = api.DecoderCompiler.compile(api.decoder_config(moe=True, **kw), weights, "",
                                       api.compile_options(no_workspace_reuse=True))
    out, _ = plan.execute(data["input"])
    n2 = plan.read_tensor("normalized2").reshape(t, h)
    mc = ob.MoeConfig(t, h, i, e, k)
    ids, wts, counts = port.route_topk(mc, n2, data["router_weight"], bias)
    assert port.last_tie_tokens == 0
    assert np.array_equal(plan.read_tensor("expert_ids", np.int32).reshape(t, k), ids)
    assert np.array_equal(plan.read_tensor("counts", np.int32), counts)
    assert counts.max() > 2 * counts.min()        # the bias does skew the loads
    assert np.allclose(plan.read_tensor("expert_weights").reshape(t, k), wts, rtol=1e-5, atol=1e-6)
    _, offsets, token_ids, slots, _ = port.dispatch_tokens(mc, n2, ids, wts, counts, copy_values=False)
    assert np.array_equal(plan.read_tensor("offsets", np.int32), offsets)
    assert np.array_equal(plan.read_tensor("token_ids", np.int32), token_ids)
    assert np.array_equal(plan.read_tensor("route_slots", np.int32), slots)
    plan.close()
    want = port.decoder_layer(ob.decoder_config(moe=True, **kw), data, native=True, trace=(ids, wts, counts))
    assert rel_err(out, want) < BF16_TOL


def test_routing_chain_bit_exact_at_8192_tokens_hidden_4096(port):
    """Router (4096 rounded multiply-adds per logit, with bias), top-2, histogram, prefix sum and the stable
    dispatch permutation at the Mixtral token count: every integer output equals the oracle's."""
    t, h, e, k = 8192, 4096, 8, 2
    x = _normal((t, h), 1.0, 31)
    wr = _normal((h, e), 0.02, 32)
    bias = np.random.default_rng(33).standard_normal(e).astype(np.float32)
    mc, oc = api.moe_config(t, h, 14336, e, k), ob.MoeConfig(t, h, 14336, e, k)
    ids, wts, counts = api.route_topk(mc, x, wr, bias, dtype=L.BF16)
    want_ids, want_wts, want_counts = port.route_topk(oc, x, wr, bias)
    ties = port.last_tie_tokens
    if ties == 0:
        assert np.array_equal(ids, want_ids)
    else:  # bit-equal exponentials may be ordered differently by the reference's carried index vector
        assert np.array_equal(np.sort(ids, axis=1), np.sort(want_ids, axis=1))
    assert np.array_equal(counts, want_counts) and int(counts.sum()) == t * k
    assert np.allclose(wts, want_wts, rtol=1e-5, atol=1e-6)
    _, offsets, token_ids, slots, rw = api.dispatch_tokens(mc, None, want_ids, want_wts, want_counts, dtype=L.BF16,
                                                           copy_values=False)
    _, want_offsets, want_tokens, want_slots, want_rw = port.dispatch_tokens(oc, x, want_ids, want_wts, want_counts,
                                                                             copy_values=False)
    assert np.array_equal(offsets, want_offsets) and offsets[-1] == t * k
    assert np.array_equal(token_ids, want_tokens) and np.array_equal(slots, want_slots)
    assert np.array_equal(rw, want_rw)


def test_paged_decode_batch64_contexts_512_to_8192(dev, port):
    """The paged split-KV decode kernel at its headline shape: 64 sequences, contexts uniform in [512, 8192]
    (seed 0), 32 query / 8 KV heads of 128, 16-token blocks scattered over the pool by a random permutation.
    Ten sequences (the longest, the shortest and eight others) are compared with the oracle's paged cache
    (one cache per sequence, pages handed out in the device table's order) decoding key by key."""
    rng = np.random.default_rng(0)
    batch, hq, hkv, d, block = 64, 32, 8, 128, 16
    ctx = rng.integers(512, 8193, size=batch).astype(np.int32)
    max_blocks = 8192 // block
    needed = (ctx + block - 1) // block
    num_blocks = int(needed.sum()) + 8
    perm = rng.permutation(num_blocks).astype(np.int32)
    table = np.zeros((batch, max_blocks), np.int32)
    cursor = 0
    for b in range(batch):
        table[b, :needed[b]] = perm[cursor:cursor + needed[b]]
        cursor += int(needed[b])
    torch = dev.torch
    gen = torch.Generator(device="cuda").manual_seed(1)
    k_pool = torch.randn((num_blocks, hkv, block, d), generator=gen, device="cuda").to(torch.bfloat16)
    v_pool = torch.randn((num_blocks, hkv, block, d), generator=gen, device="cuda").to(torch.bfloat16)
    q = torch.randn((batch, hq, d), generator=gen, device="cuda").to(torch.bfloat16)
    out = dev.zeros((batch, hq, d), torch.bfloat16)
    dtab, dctx = dev.i32(table), dev.i32(ctx)
    lib = L.load()
    splits = lib.sfb_attention_decode_default_splits(batch, hkv, 8192)
    part = dev.zeros((lib.sfb_attention_decode_workspace(batch, hq, d, splits) // 4,), torch.float32)
    a = L.DecodeArgs(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), dtab.data_ptr(), dctx.data_ptr(), out.data_ptr(),
                     part.data_ptr(), batch, hq, hkv, d, d, block, max_blocks, num_blocks, 8192, splits, 0.0, L.BF16)
    L.check(lib.sfb_k_attention_decode_paged(C.byref(a), C.c_void_p(dev.stream())))
    got = dev.np(out)
    word = C.c_uint32(0)
    L.check(lib.sfb_device_status(C.byref(word)))
    assert word.value == 0
    order = np.argsort(ctx)
    chosen = sorted({int(order[0]), int(order[-1]), *[int(s) for s in order[3:-1:8]]})
    assert len(chosen) >= 10 and ctx[chosen].max() > 8000 and ctx[chosen].min() < 640
    qh = dev.np(q)
    for b in chosen:
        n, pages = int(ctx[b]), table[b, :needed[b]]
        idx = torch.from_numpy(pages.astype(np.int64)).cuda()
        keys = dev.np(k_pool[idx]).transpose(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n]     # logical order
        values = dev.np(v_pool[idx]).transpose(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n]
        cache = port.paged_create(1, hkv, d, d, block, int(needed[b]) * block)
        # the oracle hands pages out from the back of its free list: reverse a permutation of its own pages
        local = np.random.default_rng(b).permutation(int(needed[b])).astype(np.int32)
        cache.set_free_pages(local[::-1].copy())
        cache.append(keys[None], values[None], n)
        assert np.array_equal(cache.info()["page_table"], local)
        oc = ob.AttentionConfig(1, hq, hkv, 1, n, d, d, 1, 0.0)
        want = cache.decode(oc, qh[b][None, :, None, :])[0, :, 0, :]
        two_pass = cache.decode(oc, qh[b][None, :, None, :], two_pass=True)[0, :, 0, :]
        cache.close()
        assert rel_err(want, two_pass) < 1e-5
        assert rel_err(got[b], want) < BF16_TOL, (b, n)

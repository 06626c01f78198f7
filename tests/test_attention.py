"""Attention parity: prefill (sfb_attention_execute / sfb_k_attention_prefill), contiguous and
paged decode (sfb_attention_decode, sfb_paged_*), and the split-KV kernel ABI with ragged
context lengths over a permuted block table."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import rel_err
from oracle import binding as ob
from schedforge_b200 import api, lib as L

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def attention_fixture(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    vals = [int(v) for v in z["config"][:8]]
    return api.attention_config(*vals[:7], causal=bool(vals[7]), scale=float(z["config"][8])), z


@pytest.mark.parametrize("name", ["attention_causal_gqa", "attention_dynamic", "attention_noncausal", "attention_d64"])
def test_prefill_fp32_matches_reference_fixture(name):
    c, z = attention_fixture(name)
    out, ms = api.execute_attention(c, z["q"], z["k"], z["v"], dtype=L.F32)
    assert np.max(np.abs(out - z["out_reference"])) < 1e-4      # the reference's bar
    assert np.max(np.abs(out - z["out_io_aware"])) < 1e-4
    assert rel_err(out, z["out_reference"]) < 1e-4
    assert ms >= 0.0


def test_prefill_bf16_matches_oracle(port):
    c, z = attention_fixture("attention_d64")
    q, k, v = (port.round_bf16(z[n]) for n in "qkv")
    oc = ob.AttentionConfig(2, 8, 2, 70, 70, 64, 64, 1, 0.0)
    want = port.attention_reference(oc, q, k, v)
    out, _ = api.execute_attention(c, q, k, v, dtype=L.BF16)
    assert rel_err(out, want) < 2e-2


def test_prefill_token_major_layout_and_value_dim(dev, port):
    """head_dim_value != head_dim, Sq < Sk causal offset, token-major output."""
    oc = ob.AttentionConfig(2, 4, 2, 37, 50, 16, 24, 1, 0.0)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((2, 4, 37, 16)).astype(np.float32)
    k = rng.standard_normal((2, 2, 50, 16)).astype(np.float32)
    v = rng.standard_normal((2, 2, 50, 24)).astype(np.float32)
    want = port.attention_reference(oc, q, k, v)
    dq, dk, dv = dev.f32(q), dev.f32(k), dev.f32(v)
    out = dev.zeros((2 * 37, 4 * 24), dev.torch.float32)
    a = L.AttentionArgs(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), out.data_ptr(), 2, 4, 2, 37, 50, 16, 24, 1,
                        0.0, 1, L.F32, 1)
    L.check(L.load().sfb_k_attention_prefill(C.byref(a), C.c_void_p(dev.stream())))
    got = dev.np(out).reshape(2, 37, 4, 24).transpose(0, 2, 1, 3)
    assert rel_err(got, want) < 1e-4


def test_attention_guards():
    bad = api.attention_config(1, 4, 3, 8, 8, 8)
    z = np.zeros(1, np.float32)
    with pytest.raises(L.InvalidArgument, match="invalid attention configuration"):
        api.execute_attention(bad, z, z, z)
    c = api.attention_config(1, 4, 2, 1, 11, 8, causal=True)
    q, kv = np.zeros((1, 4, 1, 8), np.float32), np.zeros((1, 2, 12, 8), np.float32)
    with pytest.raises(L.InvalidArgument, match="KV cache length violates compiled guard"):
        api.execute_decode_attention(c, q, kv, kv, 12)


@pytest.mark.parametrize("name", ["attention_decode_gqa", "attention_decode_mqa"])
def test_contiguous_decode_matches_reference_fixture(name):
    c, z = attention_fixture(name)
    out, _ = api.execute_decode_attention(c, z["q"], z["k"], z["v"], c.sequence_kv, dtype=L.F32)
    assert np.max(np.abs(out - z["out_decode"])) < 1e-4
    assert np.max(np.abs(out - z["out_reference"])) < 1e-4


def test_paged_kv_cache_matches_reference_fixture():
    z = np.load(os.path.join(GOLDEN, "paged_kv.npz"))
    cache = api.PagedKVCache(1, 2, 4, 4, 4, 12, dtype=L.F32)
    cache.append(z["keys"], z["values"], 7)
    info = cache.info()
    assert info["length"] == 7 and len(info["page_table"]) == 2
    assert np.array_equal(info["page_table"], z["page_table"]) and np.array_equal(info["free_pages"], z["free_pages"])
    gk, gv = cache.gather()
    assert np.array_equal(gk, z["keys"]) and np.array_equal(gv, z["values"])  # gather == input exactly
    c = api.attention_config(1, 4, 2, 1, 7, 4, causal=True)
    out, _ = cache.decode(c, z["query"])
    assert np.max(np.abs(out - z["decode_out"])) < 1e-5
    with pytest.raises(L.InvalidArgument, match="cannot release an active paged KV page"):
        cache.release([int(info["page_table"][0])])
    with pytest.raises(L.InvalidArgument, match="invalid physical KV page"):
        cache.release([99])
    cache.truncate(3)
    info = cache.info()
    assert info["length"] == 3
    assert np.array_equal(info["page_table"], z["truncated_page_table"])
    assert np.array_equal(info["free_pages"], z["truncated_free_pages"])
    with pytest.raises(L.InvalidArgument, match="paged KV capacity exceeded"):
        cache.append(z["keys"], z["values"], 10)
    with pytest.raises(L.InvalidArgument, match="invalid paged KV truncation length"):
        cache.truncate(5)
    with pytest.raises(L.InvalidArgument, match="paged KV length violates compiled guard"):
        cache.decode(api.attention_config(1, 4, 2, 1, 2, 4, causal=True), z["query"])
    # two appends, a shuffled free list and a batch of 2: logical order survives
    rng = np.random.default_rng(1)
    cache2 = api.PagedKVCache(2, 2, 8, 8, 4, 24, dtype=L.F32)
    cache2.set_free_pages([3, 0, 5, 1, 4, 2])
    k1, v1 = rng.standard_normal((2, 2, 5, 8)).astype(np.float32), rng.standard_normal((2, 2, 5, 8)).astype(np.float32)
    k2, v2 = rng.standard_normal((2, 2, 6, 8)).astype(np.float32), rng.standard_normal((2, 2, 6, 8)).astype(np.float32)
    cache2.append(k1, v1, 5)
    cache2.append(k2, v2, 6)
    assert list(cache2.info()["page_table"]) == [2, 4, 1]
    gk, gv = cache2.gather()
    assert np.array_equal(gk, np.concatenate([k1, k2], axis=2)) and np.array_equal(gv, np.concatenate([v1, v2], axis=2))
    with pytest.raises(L.InvalidArgument, match="invalid paged KV configuration"):
        api.PagedKVCache(1, 2, 4, 4, 0, 12)
    with pytest.raises(L.InvalidArgument, match="cannot gather empty paged KV cache"):
        api.PagedKVCache(1, 2, 4, 4, 4, 12).gather()


def paged_problem(rng, batch, hq, hkv, d, block, max_ctx, min_ctx, port, bf16):
    ctx = rng.integers(min_ctx, max_ctx + 1, size=batch).astype(np.int32)
    max_blocks = (max_ctx + block - 1) // block
    needed = [(int(n) + block - 1) // block for n in ctx]
    num_blocks = sum(needed) + 3
    perm = rng.permutation(num_blocks).astype(np.int32)
    table = np.zeros((batch, max_blocks), np.int32)
    k_pool = np.zeros((num_blocks, hkv, block, d), np.float32)
    v_pool = np.zeros((num_blocks, hkv, block, d), np.float32)
    keys, values, cursor = [], [], 0
    for b in range(batch):
        k = rng.standard_normal((hkv, int(ctx[b]), d)).astype(np.float32)
        v = rng.standard_normal((hkv, int(ctx[b]), d)).astype(np.float32)
        if bf16:
            k, v = port.round_bf16(k), port.round_bf16(v)
        keys.append(k)
        values.append(v)
        for i in range(needed[b]):
            page = perm[cursor]
            cursor += 1
            table[b, i] = page
            n = min(block, int(ctx[b]) - i * block)
            k_pool[page, :, :n] = k[:, i * block:i * block + n]
            v_pool[page, :, :n] = v[:, i * block:i * block + n]
    q = rng.standard_normal((batch, hq, d)).astype(np.float32)
    if bf16:
        q = port.round_bf16(q)
    return ctx, table, k_pool, v_pool, keys, values, q, num_blocks, max_blocks


@pytest.mark.parametrize("bf16,hq,hkv,d,splits", [(True, 32, 8, 128, 0), (True, 8, 2, 128, 5), (True, 4, 4, 128, 1),
                                                  (False, 4, 2, 32, 3), (True, 6, 2, 64, 2)])
def test_split_kv_decode_kernel_ragged_contexts(dev, port, bf16, hq, hkv, d, splits):
    rng = np.random.default_rng(5)
    batch, block = 6, 16
    ctx, table, k_pool, v_pool, keys, values, q, num_blocks, max_blocks = paged_problem(
        rng, batch, hq, hkv, d, block, 700, 1, port, bf16)
    to_dev = dev.bf16 if bf16 else dev.f32
    tdt = dev.torch.bfloat16 if bf16 else dev.torch.float32
    dq, dk, dv = to_dev(q), to_dev(k_pool), to_dev(v_pool)
    dtab, dctx = dev.i32(table), dev.i32(ctx)
    out = dev.zeros((batch, hq, d), tdt)
    lib = L.load()
    use_splits = splits if splits > 0 else lib.sfb_attention_decode_default_splits(batch, hkv, 700)
    part = dev.zeros((lib.sfb_attention_decode_workspace(batch, hq, d, use_splits) // 4,), dev.torch.float32)
    a = L.DecodeArgs(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dtab.data_ptr(), dctx.data_ptr(), out.data_ptr(),
                     part.data_ptr(), batch, hq, hkv, d, d, block, max_blocks, num_blocks, 700, splits, 0.0,
                     L.BF16 if bf16 else L.F32)
    L.check(lib.sfb_k_attention_decode_paged(C.byref(a), C.c_void_p(dev.stream())))
    got = dev.np(out)
    for b in range(batch):
        oc = ob.AttentionConfig(1, hq, hkv, 1, int(ctx[b]), d, d, 1, 0.0)
        want = port.attention_reference(oc, q[b][None, :, None, :], keys[b][None], values[b][None])[0, :, 0, :]
        assert rel_err(got[b], want) < (2e-2 if bf16 else 1e-4), (b, int(ctx[b]))


def test_paged_kernels_skip_positions_and_blocks_outside_the_cache(dev, port):
    """A length past the block table or a block id outside the pool (as a faulty producer kernel could
    write them) must not be followed: the append skips the token, the decode cuts the context to what the
    table covers, and both report through the device status word (bit 0x200)."""
    rng = np.random.default_rng(9)
    batch, hq, hkv, d, block, max_blocks = 2, 8, 2, 128, 16, 4
    num_blocks = batch * max_blocks
    torch = dev.torch
    lib, s = L.load(), C.c_void_p(dev.stream())
    word = C.c_uint32(0)
    L.check(lib.sfb_device_status(C.byref(word)))  # start from a clear word
    k_pool = dev.zeros((num_blocks, hkv, block, d), torch.bfloat16)
    v_pool = dev.zeros((num_blocks, hkv, block, d), torch.bfloat16)
    table = np.arange(num_blocks, dtype=np.int32).reshape(batch, max_blocks)
    table[1, 0] = num_blocks + 5                      # sequence 1: first block id lies outside the pool
    dtab = dev.i32(table)
    k = dev.bf16(np.ones((batch, hkv, 1, d), np.float32))
    # sequence 0 appends at position 64 = one past the table (4 blocks x 16 tokens), sequence 1 into the bad block
    start = dev.i32(np.array([max_blocks * block, 3]))
    L.check(lib.sfb_k_paged_kv_append(C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), C.c_void_p(k_pool.data_ptr()),
                                      C.c_void_p(v_pool.data_ptr()), C.c_void_p(dtab.data_ptr()), C.c_void_p(start.data_ptr()),
                                      batch, hkv, 1, d, d, block, max_blocks, num_blocks, L.BF16, s))
    L.check(lib.sfb_device_status(C.byref(word)))
    assert word.value & 0x200
    assert float(dev.np(k_pool).sum()) == 0.0 and float(dev.np(v_pool).sum()) == 0.0   # nothing was written
    # decode: a context of 1000 tokens against a table that covers 64 is cut to 64 keys
    kp = port.round_bf16(rng.standard_normal((num_blocks, hkv, block, d)).astype(np.float32))
    vp = port.round_bf16(rng.standard_normal((num_blocks, hkv, block, d)).astype(np.float32))
    q = port.round_bf16(rng.standard_normal((batch, hq, d)).astype(np.float32))
    good = np.arange(num_blocks, dtype=np.int32).reshape(batch, max_blocks)
    dk, dv, dq, dgood = dev.bf16(kp), dev.bf16(vp), dev.bf16(q), dev.i32(good)
    outs = []
    for lens in ([1000, 64], [64, 64]):
        dctx = dev.i32(np.array(lens))
        out = dev.zeros((batch, hq, d), torch.bfloat16)
        splits = 2
        part = dev.zeros((lib.sfb_attention_decode_workspace(batch, hq, d, splits) // 4,), torch.float32)
        a = L.DecodeArgs(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dgood.data_ptr(), dctx.data_ptr(), out.data_ptr(),
                         part.data_ptr(), batch, hq, hkv, d, d, block, max_blocks, num_blocks, 64, splits, 0.0, L.BF16)
        L.check(lib.sfb_k_attention_decode_paged(C.byref(a), s))
        L.check(lib.sfb_device_status(C.byref(word)))
        outs.append((dev.np(out), word.value))
    assert outs[0][1] & 0x200 and outs[1][1] == 0
    assert np.array_equal(outs[0][0], outs[1][0])


def test_paged_append_kernel_then_decode_roundtrip(dev, port):
    """append kernel writes exactly what gather kernel reads back (bf16, permuted table)."""
    rng = np.random.default_rng(8)
    batch, hkv, d, block, tokens = 3, 2, 64, 16, 40
    max_blocks = 4
    table = rng.permutation(batch * max_blocks).astype(np.int32).reshape(batch, max_blocks)
    k = port.round_bf16(rng.standard_normal((batch, hkv, tokens, d)).astype(np.float32))
    v = port.round_bf16(rng.standard_normal((batch, hkv, tokens, d)).astype(np.float32))
    torch = dev.torch
    k_pool = dev.zeros((batch * max_blocks, hkv, block, d), torch.bfloat16)
    v_pool = dev.zeros((batch * max_blocks, hkv, block, d), torch.bfloat16)
    dk, dv, dtab = dev.bf16(k), dev.bf16(v), dev.i32(table)
    lib, s = L.load(), C.c_void_p(dev.stream())
    first, rest = 25, tokens - 25
    start0, start1 = dev.i32(np.zeros(batch)), dev.i32(np.full(batch, first))
    k1, v1 = dk[:, :, :first].contiguous(), dv[:, :, :first].contiguous()
    k2, v2 = dk[:, :, first:].contiguous(), dv[:, :, first:].contiguous()
    for kk, vv, st, n in ((k1, v1, start0, first), (k2, v2, start1, rest)):
        L.check(lib.sfb_k_paged_kv_append(C.c_void_p(kk.data_ptr()), C.c_void_p(vv.data_ptr()), C.c_void_p(k_pool.data_ptr()),
                                          C.c_void_p(v_pool.data_ptr()), C.c_void_p(dtab.data_ptr()), C.c_void_p(st.data_ptr()),
                                          batch, hkv, n, d, d, block, max_blocks, int(k_pool.shape[0]), L.BF16, s))
    gk, gv = dev.zeros((batch, hkv, tokens, d), torch.bfloat16), dev.zeros((batch, hkv, tokens, d), torch.bfloat16)
    L.check(lib.sfb_k_paged_kv_gather(C.c_void_p(k_pool.data_ptr()), C.c_void_p(v_pool.data_ptr()), C.c_void_p(gk.data_ptr()),
                                      C.c_void_p(gv.data_ptr()), C.c_void_p(dtab.data_ptr()), batch, hkv, tokens, d, d,
                                      block, max_blocks, L.BF16, s))
    assert np.array_equal(dev.np(gk), k) and np.array_equal(dev.np(gv), v)


@pytest.mark.parametrize("backend", [1, 2])  # CUDA-core kernel, tcgen05 kernel
@pytest.mark.parametrize("batch,hq,hkv,sq,sk,causal,qscale,token_major", [
    (2, 8, 2, 300, 300, True, 1.0, False),     # ragged tiles, causal
    (1, 4, 4, 256, 256, False, 1.0, True),     # exact tiles, non-causal, token-major output
    (1, 4, 1, 200, 333, True, 1.0, False),     # Sq < Sk: causal frontier offset
    (1, 8, 2, 1000, 1000, True, 6.0, True),    # long rows with large scores: running-max growth
    (3, 2, 2, 70, 70, True, 1.0, False),       # less than one Q tile
])
@pytest.mark.parametrize("d", [128, 64])
def test_prefill_bf16_head_dim_128_and_64(dev, port, backend, batch, hq, hkv, sq, sk, causal, qscale, token_major, d):
    rng = np.random.default_rng(sq + sk)
    q = port.round_bf16((rng.standard_normal((batch, hq, sq, d)) * qscale).astype(np.float32))
    k = port.round_bf16(rng.standard_normal((batch, hkv, sk, d)).astype(np.float32))
    v = port.round_bf16(rng.standard_normal((batch, hkv, sk, d)).astype(np.float32))
    oc = ob.AttentionConfig(batch, hq, hkv, sq, sk, d, d, int(causal), 0.0)
    want = port.attention_reference(oc, q, k, v)
    dq, dk, dv = dev.bf16(q), dev.bf16(k), dev.bf16(v)
    out = dev.zeros((batch * sq * hq * d,), dev.torch.bfloat16)
    a = L.AttentionArgs(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), out.data_ptr(), batch, hq, hkv, sq, sk, d, d,
                        int(causal), 0.0, int(token_major), L.BF16, backend)
    L.check(L.load().sfb_k_attention_prefill(C.byref(a), C.c_void_p(dev.stream())))
    dev.torch.cuda.synchronize()
    word = C.c_uint32(0)
    L.check(L.load().sfb_device_status(C.byref(word)))
    assert word.value == 0, f"device wait timed out, status word {word.value:#x}"
    got = dev.np(out)
    got = got.reshape(batch, sq, hq, d).transpose(0, 2, 1, 3) if token_major else got.reshape(batch, hq, sq, d)
    assert rel_err(got, want) < 2e-2


def test_prefill_tcgen05_baseline_config2_slices(dev, port):
    """Headline attention shape (B4, Hq32, Hkv8, S4096, D128, causal): full run on the GPU, the
    oracle on sampled (batch, head) slices and query rows (materialised softmax(QK^T)V)."""
    torch = dev.torch
    batch, hq, hkv, s = 4, 32, 8, 4096
    gen = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn((batch, hq, s, 128), generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn((batch, hkv, s, 128), generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn((batch, hkv, s, 128), generator=gen, device="cuda").to(torch.bfloat16)
    out = torch.zeros((batch, hq, s, 128), dtype=torch.bfloat16, device="cuda")
    a = L.AttentionArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), batch, hq, hkv, s, s, 128, 128, 1,
                        0.0, 0, L.BF16, 2)
    L.check(L.load().sfb_k_attention_prefill(C.byref(a), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    rng = np.random.default_rng(0)
    for b, h in ((0, 0), (3, 31), (1, 13)):
        rows = np.sort(rng.choice(s, 48, replace=False))
        rows[-1] = s - 1
        kvh = h * hkv // hq
        kk, vv = k[b, kvh].float().cpu().numpy(), v[b, kvh].float().cpu().numpy()
        for row in rows:
            # one query row against its visible prefix = a non-causal problem of length row+1
            oc = ob.AttentionConfig(1, 1, 1, 1, int(row) + 1, 128, 128, 0, 0.0)
            want = port.attention_reference(oc, q[b, h, row].float().cpu().numpy()[None, None, None, :],
                                            kk[None, None, :row + 1], vv[None, None, :row + 1])[0, 0, 0]
            got = out[b, h, row].float().cpu().numpy()
            assert np.max(np.abs(got - want)) < 2e-2 * max(np.max(np.abs(want)), 0.05), (b, h, int(row))


def test_prefill_tcgen05_row_slices_equal_the_whole_sequence(dev, port):
    """A causal prefill run as row chunks (queries [r0, r1) against keys [0, r1), head strides of
    the whole sequence) must give exactly the rows of the one-shot run: this is what the pipelined
    plan execute relies on."""
    torch = dev.torch
    hq, hkv, s, chunk = 4, 2, 1024, 256
    gen = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn((1, hq, s, 128), generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn((1, hkv, s, 128), generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, hkv, s, 128), generator=gen, device="cuda").to(torch.bfloat16)
    whole = torch.zeros((s, hq * 128), dtype=torch.bfloat16, device="cuda")   # token-major
    sliced = torch.zeros_like(whole)
    lib = L.load()
    a = L.AttentionArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), whole.data_ptr(), 1, hq, hkv, s, s, 128, 128, 1, 0.0, 1,
                        L.BF16, 2)
    L.check(lib.sfb_k_attention_prefill(C.byref(a), C.c_void_p(dev.stream())))
    for r0 in range(0, s, chunk):
        a = L.AttentionArgs(q.data_ptr() + r0 * 128 * 2, k.data_ptr(), v.data_ptr(), sliced.data_ptr() + r0 * hq * 128 * 2,
                            1, hq, hkv, chunk, r0 + chunk, 128, 128, 1, 0.0, 1, L.BF16, 2, s, s)
        L.check(lib.sfb_k_attention_prefill(C.byref(a), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    assert torch.equal(whole, sliced)
    oc = ob.AttentionConfig(1, hq, hkv, s, s, 128, 128, 1, 0.0)
    want = port.attention_reference(oc, q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
    got = whole.float().cpu().numpy().reshape(1, s, hq, 128).transpose(0, 2, 1, 3)
    assert rel_err(got, want) < 2e-2
    # the CUDA-core kernel does not take slices and says so
    a = L.AttentionArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), sliced.data_ptr(), 1, hq, hkv, chunk, chunk, 128, 128, 1,
                        0.0, 1, L.BF16, 1, s, s)
    with pytest.raises(L.SfbError):
        L.check(lib.sfb_k_attention_prefill(C.byref(a), C.c_void_p(dev.stream())))

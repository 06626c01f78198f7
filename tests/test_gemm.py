"""GEMM parity: the fp32 exact-order kernel, the CUDA-core bf16 kernel and the tcgen05
tensor-core kernel against the oracle, through sfb_k_gemm_f32 / sfb_k_gemm_bf16."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2  # max-abs relative, bf16 outputs with fp32 accumulation


def gemm_bf16(sfb, dev, a, bt, epilogue=0, backend=0, out_f32=False, residual=None, swiglu_block=0,
              rope=None, offsets=None, groups=0, n=None, scratch=None, blocked=False, int8_scales=None):
    torch = dev.torch
    m, k = a.shape
    n = n if n is not None else bt.shape[-2]
    assert int8_scales is None or not blocked
    g = sfb.GemmArgs()
    g.a, g.bt = a.data_ptr(), bt.data_ptr()
    g.m, g.n, g.k = m, n, k
    keep = []
    if blocked:  # re-lay the [n,k] weight in 64x64 blocks first
        lib = sfb.load()
        tiled = dev.zeros((lib.sfb_tiled_weight_elems(n, k),), torch.bfloat16)
        sfb.check(lib.sfb_k_tile_weight_bf16(C.c_void_p(bt.data_ptr()), C.c_void_p(tiled.data_ptr()), n, k,
                                             C.c_void_p(dev.stream())))
        keep.append(tiled)
        g.bt, g.bt_tiled = tiled.data_ptr(), 1
    g.epilogue, g.backend, g.out_f32 = epilogue, backend, int(out_f32)
    out = None
    if epilogue == sfb.EPI_ROPE_SPLIT:
        batch, seq, hq, hkv, d, cos, sin = rope
        q = dev.zeros((batch, hq, seq, d), torch.bfloat16)
        key = dev.zeros((batch, hkv, seq, d), torch.bfloat16)
        val = dev.zeros((batch, hkv, seq, d), torch.bfloat16)
        g.q, g.key, g.value = q.data_ptr(), key.data_ptr(), val.data_ptr()
        g.rope_cos, g.rope_sin = cos.data_ptr(), sin.data_ptr()
        g.batch, g.seq, g.q_heads, g.kv_heads, g.head_dim = batch, seq, hq, hkv, d
        out = (q, key, val)
    else:
        width = n // 2 if epilogue == sfb.EPI_SWIGLU else n
        out = dev.zeros((m, width), torch.float32 if out_f32 else torch.bfloat16)
        g.out = out.data_ptr()
    if residual is not None:
        g.residual = residual.data_ptr()
    g.swiglu_block = swiglu_block
    if offsets is not None:
        g.group_offsets, g.groups = offsets.data_ptr(), groups
        table = dev.zeros((4 * (m // 128 + groups + 2),), torch.int32)
        keep.append(table)
        g.tile_table = table.data_ptr()
    if scratch is not None:
        g.split_workspace, g.split_workspace_bytes = scratch[0].data_ptr(), scratch[1]
    if int8_scales is not None:
        g.bt_scales = int8_scales.data_ptr()
    sfb.check(sfb.load().sfb_k_gemm_bf16(C.byref(g), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    word = C.c_uint32(0)
    sfb.check(sfb.load().sfb_device_status(C.byref(word)))
    assert word.value == 0, f"device wait timed out, status word {word.value:#x}"
    return out


@pytest.mark.parametrize("m,n,k", [(128, 384, 256), (7, 33, 19), (130, 70, 1000)])
def test_gemm_f32_bit_exact(sfb, dev, port, m, n, k):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    da, db = dev.f32(a), dev.f32(b)
    dc = dev.zeros((m, n), dev.torch.float32)
    sfb.check(sfb.load().sfb_k_gemm_f32(C.c_void_p(da.data_ptr()), C.c_void_p(db.data_ptr()),
                                        C.c_void_p(dc.data_ptr()), m, n, k, C.c_void_p(dev.stream())))
    want = port.matmul(a, b, fma=True)  # FMA chain of the reference's native GEMM
    assert np.array_equal(dev.np(dc), want)
    # and within fp32 round-off of the scalar (multiply-then-add) layer reference
    assert rel_err(dev.np(dc), port.matmul(a, b, fma=False)) < 1e-5


def _inputs(port, m, n, k, seed=0, scale=0.05):
    rng = np.random.default_rng(seed)
    a = port.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = port.round_bf16((rng.standard_normal((k, n)) * scale).astype(np.float32))  # [k, n], y = x.W
    return a, w


BACKENDS = [1, 2]  # SIMT, tcgen05


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 512, 256), (300, 264, 136), (1, 256, 128),
                                   (520, 1024, 320)])
def test_gemm_bf16_store(sfb, dev, port, backend, m, n, k):
    a, w = _inputs(port, m, n, k)
    want = port.matmul(a, w, fma=True)
    got = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), backend=backend)
    assert rel_err(dev.np(got), want) < BF16_TOL
    got32 = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), backend=backend, out_f32=True)
    assert rel_err(dev.np(got32), want) < 1e-4  # fp32 accumulation of exact bf16 products


@pytest.mark.parametrize("backend", BACKENDS)
def test_gemm_bf16_residual(sfb, dev, port, backend):
    m, n, k = 260, 384, 192
    a, w = _inputs(port, m, n, k, seed=2)
    res = port.round_bf16(np.random.default_rng(3).standard_normal((m, n)).astype(np.float32))
    want = port.matmul(a, w, fma=True) + res
    got = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), epilogue=sfb.EPI_RESIDUAL,
                    backend=backend, residual=dev.bf16(res))
    assert rel_err(dev.np(got), want) < BF16_TOL


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("block", [64, 128])
def test_gemm_bf16_swiglu(sfb, dev, port, backend, block):
    m, inter, k = 200, 384, 128
    rng = np.random.default_rng(4)
    a = port.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    wg = port.round_bf16((rng.standard_normal((k, inter)) * 0.1).astype(np.float32))
    wu = port.round_bf16((rng.standard_normal((k, inter)) * 0.1).astype(np.float32))
    gate_up = port.matmul(a, np.concatenate([wg, wu], axis=1), fma=True)
    want = port.swiglu(gate_up, inter)
    # weight rows: blocks of `block` gate rows followed by `block` up rows
    bt = np.concatenate([np.concatenate([wg.T[i:i + block], wu.T[i:i + block]]) for i in range(0, inter, block)])
    got = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(bt), epilogue=sfb.EPI_SWIGLU, backend=backend,
                    swiglu_block=block)
    assert rel_err(dev.np(got), want) < BF16_TOL


@pytest.mark.parametrize("backend", BACKENDS)
def test_gemm_bf16_rope_split(sfb, dev, port, backend):
    from oracle import binding as ob
    batch, seq, hq, hkv, d = 2, 96, 4, 2, 64
    hidden = hq * d
    c = ob.decoder_config(batch, seq, hidden, 64, hq, hkv, d, rope_theta=10000.0)
    n, k, m = hidden + 2 * hkv * d, hidden, batch * seq
    a, w = _inputs(port, m, n, k, seed=5)
    fused = port.matmul(a, w, fma=True)
    wq, wk, wv = port.split_qkv_rope(c, fused)
    cos = np.zeros((seq, d // 2), np.float32)
    sin = np.zeros((seq, d // 2), np.float32)
    sfb.check(sfb.load().sfb_rope_table(seq, d, C.c_float(10000.0), cos.ctypes.data_as(sfb.f32p),
                                        sin.ctypes.data_as(sfb.f32p)))
    q, key, val = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), epilogue=sfb.EPI_ROPE_SPLIT,
                            backend=backend, rope=(batch, seq, hq, hkv, d, dev.f32(cos), dev.f32(sin)))
    assert rel_err(dev.np(q), wq) < BF16_TOL
    assert rel_err(dev.np(key), wk) < BF16_TOL
    assert rel_err(dev.np(val), wv) < BF16_TOL


# Few rows (decode).  Given zeroed scratch the tcgen05 kernel cuts the (tile, K block) sequence
# into one equal range per SM, sums partial tiles in the scratch and leaves it zeroed again.
def _scratch(sfb, dev, n):
    nbytes = sfb.load().sfb_gemm_stream_workspace_bytes(n)
    return dev.zeros((nbytes // 4,), dev.torch.float32), nbytes


@pytest.mark.parametrize("blocked", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 256, 4096), (17, 200, 2048), (1, 512, 8200), (64, 320, 1000),
                                   (128, 128, 512), (100, 6144, 1024)])
def test_gemm_tcgen05_few_rows_equal_ranges(sfb, dev, port, m, n, k, blocked):
    a, w = _inputs(port, m, n, k, seed=11, scale=0.02)
    res = port.round_bf16(np.random.default_rng(12).standard_normal((m, n)).astype(np.float32))
    want = port.matmul(a, w, fma=True)
    da, dw = dev.bf16(a), dev.bf16(w.T.copy())
    scratch = _scratch(sfb, dev, n)
    got32 = gemm_bf16(sfb, dev, da, dw, backend=2, out_f32=True, scratch=scratch, blocked=blocked)
    assert rel_err(dev.np(got32), want) < 1e-4
    assert not dev.np(scratch[0]).any()  # the kernel put the zeros back
    got = gemm_bf16(sfb, dev, da, dw, backend=0, epilogue=sfb.EPI_RESIDUAL, residual=dev.bf16(res),
                    scratch=scratch, blocked=blocked)
    assert rel_err(dev.np(got), want + res) < BF16_TOL
    assert not dev.np(scratch[0]).any()


def test_gemm_tcgen05_few_rows_rope_split(sfb, dev, port):
    from oracle import binding as ob
    batch, seq, hq, hkv, d = 24, 1, 8, 2, 64
    hidden = hq * d
    c = ob.decoder_config(batch, seq, hidden, 64, hq, hkv, d, rope_theta=10000.0)
    n, k, m = hidden + 2 * hkv * d, 2048, batch * seq
    a, w = _inputs(port, m, n, k, seed=13, scale=0.02)
    wq, wk, wv = port.split_qkv_rope(c, port.matmul(a, w, fma=True))
    cos = np.zeros((seq, d // 2), np.float32)
    sin = np.zeros((seq, d // 2), np.float32)
    sfb.check(sfb.load().sfb_rope_table(seq, d, C.c_float(10000.0), cos.ctypes.data_as(sfb.f32p),
                                        sin.ctypes.data_as(sfb.f32p)))
    scratch = _scratch(sfb, dev, n)
    for _ in range(2):  # the second call runs on the scratch the first one left behind
        q, key, val = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), epilogue=sfb.EPI_ROPE_SPLIT,
                                backend=2, rope=(batch, seq, hq, hkv, d, dev.f32(cos), dev.f32(sin)),
                                scratch=scratch, blocked=True)
        assert rel_err(dev.np(q), wq) < BF16_TOL
        assert rel_err(dev.np(key), wk) < BF16_TOL
        assert rel_err(dev.np(val), wv) < BF16_TOL


def test_gemm_blocked_weight_many_rows(sfb, dev, port):
    m, n, k = 300, 384, 512
    a, w = _inputs(port, m, n, k, seed=15, scale=0.02)
    got32 = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), backend=2, out_f32=True, blocked=True)
    assert rel_err(dev.np(got32), port.matmul(a, w, fma=True)) < 1e-4


def test_gemm_blocked_weight_rejected_by_simt(sfb, dev, port):
    a, w = _inputs(port, 8, 64, 64)
    with pytest.raises(sfb.SfbError):
        gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(w.T.copy()), backend=1, blocked=True)


@pytest.mark.parametrize("blocked", [False, True])
@pytest.mark.parametrize("m", [1, 100, 128])
def test_gemm_tcgen05_swiglu_few_rows(sfb, dev, port, m, blocked):
    inter, k, block = 320, 1024, 64
    rng = np.random.default_rng(14)
    a = port.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    wg = port.round_bf16((rng.standard_normal((k, inter)) * 0.1).astype(np.float32))
    wu = port.round_bf16((rng.standard_normal((k, inter)) * 0.1).astype(np.float32))
    want = port.swiglu(port.matmul(a, np.concatenate([wg, wu], axis=1), fma=True), inter)
    bt = np.concatenate([np.concatenate([wg.T[i:i + block], wu.T[i:i + block]]) for i in range(0, inter, block)])
    scratch = _scratch(sfb, dev, 2 * inter)
    for _ in range(2):
        got = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(bt), epilogue=sfb.EPI_SWIGLU, backend=2,
                        swiglu_block=block, scratch=scratch, blocked=blocked)
        assert rel_err(dev.np(got), want) < BF16_TOL
    assert not dev.np(scratch[0]).any()


@pytest.mark.parametrize("backend", BACKENDS)
def test_gemm_bf16_grouped(sfb, dev, port, backend):
    """Variable-M expert GEMM: empty, tiny, ragged and >128-row segments."""
    groups, n, k = 5, 256, 128
    offsets = np.array([0, 5, 5, 200, 456, 460], np.int32)
    m = int(offsets[-1])
    rng = np.random.default_rng(6)
    a = port.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = port.round_bf16((rng.standard_normal((groups, k, n)) * 0.1).astype(np.float32))
    want = np.zeros((m, n), np.float32)
    for g in range(groups):
        lo, hi = offsets[g], offsets[g + 1]
        if hi > lo:
            want[lo:hi] = port.matmul(a[lo:hi], w[g], fma=True)
    bt = np.ascontiguousarray(w.transpose(0, 2, 1))
    got = gemm_bf16(sfb, dev, dev.bf16(a), dev.bf16(bt), backend=backend, offsets=dev.i32(offsets),
                    groups=groups, n=n)
    assert rel_err(dev.np(got), want) < BF16_TOL


def test_gemm_tcgen05_llama_shape_sampled_rows(sfb, dev, port):
    """Full-size projection (T=8192, 4096x4096): oracle on 24 sampled rows."""
    m, n, k = 8192, 4096, 4096
    torch = dev.torch
    gen = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    bt = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    got = gemm_bf16(sfb, dev, a, bt, backend=2)
    rows = np.random.default_rng(0).choice(m, 24, replace=False)
    a_rows = a[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    want = port.matmul(a_rows, bt.float().cpu().numpy().T.copy(), fma=True)
    assert rel_err(dev.np(got)[rows], want) < BF16_TOL


# ---- weight-only INT8 (few rows) ----------------------------------------------------------------------

def _quantize_like_the_reference(w_nk):
    """quantize_matmul_weights, src/next_milestones.cpp:611-637, per output channel."""
    maximum = np.max(np.abs(w_nk), axis=1)
    scale = np.where(maximum > 0, (maximum / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    value = (w_nk / scale[:, None]).astype(np.float32)
    rounded = np.sign(value) * np.floor(np.abs(value) + np.float32(0.5))  # std::round: halves away from zero
    return np.clip(rounded, -127, 127).astype(np.int8), scale


def _blocked(q_nk):
    n, k = q_nk.shape
    nb, kb = (n + 63) // 64, (k + 63) // 64
    padded = np.zeros((nb * 64, kb * 64), q_nk.dtype)
    padded[:n, :k] = q_nk
    return padded.reshape(nb, 64, kb, 64).transpose(0, 2, 1, 3).copy()


def _quantize_on_device(sfb, dev, w_nk):
    torch = dev.torch
    n, k = w_nk.shape
    lib = sfb.load()
    q = torch.zeros((lib.sfb_tiled_weight_elems(n, k),), dtype=torch.int8, device="cuda")
    scales = torch.zeros(((n + 127) // 128 * 128,), dtype=torch.float32, device="cuda")
    dw = dev.bf16(w_nk)
    sfb.check(lib.sfb_k_quantize_weight_int8(C.c_void_p(dw.data_ptr()), C.c_void_p(q.data_ptr()),
                                             C.c_void_p(scales.data_ptr()), n, k, C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    return q, scales


@pytest.mark.parametrize("n,k", [(128, 64), (200, 1000), (512, 4096)])
def test_int8_weight_quantization_is_the_reference_formula(sfb, dev, port, n, k):
    rng = np.random.default_rng(n + k)
    w = port.round_bf16((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    w[3] = 0.0  # an all-zero output channel keeps scale 1
    q, scales = _quantize_on_device(sfb, dev, w)
    want_q, want_scale = _quantize_like_the_reference(w)
    assert np.array_equal(scales.cpu().numpy()[:n], want_scale)
    assert np.array_equal(q.cpu().numpy().reshape(_blocked(want_q).shape), _blocked(want_q))
    back = dev.zeros((n, k), dev.torch.bfloat16)
    sfb.check(sfb.load().sfb_k_dequantize_weight_int8(C.c_void_p(q.data_ptr()), C.c_void_p(scales.data_ptr()),
                                                      C.c_void_p(back.data_ptr()), n, k, C.c_void_p(dev.stream())))
    assert np.array_equal(dev.np(back), port.round_bf16(want_q.astype(np.float32) * want_scale[:, None]))


@pytest.mark.parametrize("m,n,k", [(128, 256, 4096), (17, 200, 2048), (1, 512, 8200), (100, 6144, 1024)])
def test_gemm_int8_weights_few_rows(sfb, dev, port, m, n, k):
    """y = (x . q^T) * scale with q, scale from the reference's quantizer (quantized_invoke,
    src/next_milestones.cpp:50-69), bf16 activations, fp32 sums; plain, residual and fp32 outputs."""
    a, w = _inputs(port, m, n, k, seed=21, scale=0.02)
    w_nk = np.ascontiguousarray(w.T)
    q, scales = _quantize_on_device(sfb, dev, w_nk)
    want_q, want_scale = _quantize_like_the_reference(w_nk)
    want = (a.astype(np.float64) @ want_q.astype(np.float64).T * want_scale[None, :]).astype(np.float32)
    res = port.round_bf16(np.random.default_rng(22).standard_normal((m, n)).astype(np.float32))
    scratch = _scratch(sfb, dev, n)
    for _ in range(2):
        got32 = gemm_bf16(sfb, dev, dev.bf16(a), q, backend=2, out_f32=True, scratch=scratch, n=n, int8_scales=scales)
        assert rel_err(dev.np(got32), want) < 1e-4
        got = gemm_bf16(sfb, dev, dev.bf16(a), q, epilogue=sfb.EPI_RESIDUAL, residual=dev.bf16(res), scratch=scratch, n=n,
                        int8_scales=scales)
        assert rel_err(dev.np(got), want + res) < BF16_TOL
    assert not dev.np(scratch[0]).any()


def test_gemm_int8_weights_swiglu(sfb, dev, port):
    m, inter, k, block = 100, 320, 1024, 64
    rng = np.random.default_rng(23)
    a = port.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    wg = port.round_bf16((rng.standard_normal((inter, k)) * 0.1).astype(np.float32))
    wu = port.round_bf16((rng.standard_normal((inter, k)) * 0.1).astype(np.float32))
    bt = np.concatenate([np.concatenate([wg[i:i + block], wu[i:i + block]]) for i in range(0, inter, block)])
    q, scales = _quantize_on_device(sfb, dev, bt)
    qg, sg = _quantize_like_the_reference(wg)
    qu, su = _quantize_like_the_reference(wu)
    gate = (a.astype(np.float64) @ qg.astype(np.float64).T * sg[None, :]).astype(np.float32)
    up = (a.astype(np.float64) @ qu.astype(np.float64).T * su[None, :]).astype(np.float32)
    want = port.swiglu(np.concatenate([gate, up], axis=1), inter)
    got = gemm_bf16(sfb, dev, dev.bf16(a), q, epilogue=sfb.EPI_SWIGLU, backend=2, swiglu_block=block,
                    scratch=_scratch(sfb, dev, 2 * inter), n=2 * inter, int8_scales=scales)
    assert rel_err(dev.np(got), want) < BF16_TOL


def test_gemm_scatters_rows_to_their_owners(sfb, dev, port):
    """Two-shot form, producer side: with scatter_rows the tcgen05 epilogue stores row r only into the buffer of
    rank r / scatter_rows at row r % scatter_rows (here four buffers of one GPU stand in for four ranks)."""
    rng = np.random.default_rng(17)
    m, n, k, owners = 512, 384, 256, 4
    a = port.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = port.round_bf16((rng.standard_normal((k, n)) * 0.05).astype(np.float32))
    da, dbt = dev.bf16(a), dev.bf16(np.ascontiguousarray(w.T))
    plain = dev.zeros((m, n), dev.torch.bfloat16)
    slots = [dev.zeros((m // owners, n), dev.torch.bfloat16) for _ in range(owners)]
    L = sfb
    lib, s = L.load(), C.c_void_p(dev.stream())
    g = L.GemmArgs()
    g.a, g.bt, g.out, g.m, g.n, g.k = da.data_ptr(), dbt.data_ptr(), plain.data_ptr(), m, n, k
    g.epilogue, g.backend = L.EPI_STORE, L.GEMM_TCGEN05
    L.check(lib.sfb_k_gemm_bf16(C.byref(g), s))
    want = dev.np(plain)
    unused = dev.zeros((m, n), dev.torch.bfloat16)
    g.out, g.scatter_rows = unused.data_ptr(), m // owners
    for r in range(owners):
        g.scatter_out[r] = slots[r].data_ptr()
    L.check(lib.sfb_k_gemm_bf16(C.byref(g), s))
    for r in range(owners):
        assert np.array_equal(dev.np(slots[r]), want[r * (m // owners):(r + 1) * (m // owners)])
    assert float(np.abs(dev.np(unused)).sum()) == 0.0
    assert rel_err(want, a @ w) < 2e-2

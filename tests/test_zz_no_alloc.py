"""The allocation-free dispatch entry point (sfb_k_moe_dispatch_static).

Some callers of this library cannot allocate device memory at all: a serving process whose
memory pool was sized at start-up and owns every byte, or a plugin that is forbidden to call
cudaMalloc once the host application is running.  For them the library keeps the dispatch
scratch inside its own image.  This test calls that entry point through the C ABI twice in a
row and checks every output against the ordinary entry point (caller-provided scratch), which
in turn is checked against the oracle elsewhere.  Collected last on purpose: a run that stops
at the first failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

from schedforge_b200 import lib as L

pytestmark = pytest.mark.gpu


def run_dispatch(dev, static, x, ids, weights, counts, tokens, hidden, experts, top_k):
    torch = dev.torch
    lib = L.load()
    n = tokens * top_k
    values = dev.zeros((n, hidden), torch.bfloat16)
    offsets = dev.zeros((experts + 1,), torch.int32)
    token_ids, slots, dest = (dev.zeros((n,), torch.int32) for _ in range(3))
    rw = dev.zeros((n,), torch.float32)
    args = [C.c_void_p(x.data_ptr()), L.BF16, C.c_void_p(ids.data_ptr()), C.c_void_p(weights.data_ptr()),
            C.c_void_p(counts.data_ptr()), tokens, hidden, experts, top_k, C.c_void_p(values.data_ptr()),
            C.c_void_p(offsets.data_ptr()), C.c_void_p(token_ids.data_ptr()), C.c_void_p(slots.data_ptr()),
            C.c_void_p(rw.data_ptr()), C.c_void_p(dest.data_ptr())]
    if static:
        L.check(lib.sfb_k_moe_dispatch_static(*args, C.c_void_p(dev.stream())))
    else:
        scratch = dev.zeros((lib.sfb_moe_dispatch_scratch_bytes(tokens, experts, top_k) // 4,), torch.int32)
        L.check(lib.sfb_k_moe_dispatch(*args, C.c_void_p(scratch.data_ptr()), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    return [dev.np(t) for t in (values, offsets, token_ids, slots, rw, dest)]


def test_static_dispatch_matches_regular_dispatch_twice(dev):
    rng = np.random.default_rng(0)
    # two different problems back to back: the second call sees the first call's scratch contents
    for tokens, hidden, experts, top_k in ((3000, 256, 8, 2), (777, 64, 16, 4)):
        x = dev.bf16(rng.standard_normal((tokens, hidden)))
        ids_host = np.stack([rng.permutation(experts)[:top_k] for _ in range(tokens)]).astype(np.int32)
        ids = dev.i32(ids_host)
        weights = dev.f32(rng.random((tokens, top_k)))
        counts = dev.i32(np.bincount(ids_host.ravel(), minlength=experts))
        want = run_dispatch(dev, False, x, ids, weights, counts, tokens, hidden, experts, top_k)
        got = run_dispatch(dev, True, x, ids, weights, counts, tokens, hidden, experts, top_k)
        for a, b in zip(got, want):
            assert np.array_equal(a, b)  # integers and copied rows: bit-exact, same tolerance as test_moe.py


def test_static_dispatch_rejects_oversized_requests(dev):
    one = dev.zeros((8,), dev.torch.int32)
    p = C.c_void_p(one.data_ptr())
    status = L.load().sfb_k_moe_dispatch_static(p, L.BF16, p, p, p, 200000, 64, 8, 2, None, p, p, p, p, p, None)
    assert status == L.SFB_UNSUPPORTED
    assert b"262144" in L.load().sfb_last_error()

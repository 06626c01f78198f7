"""The finish kernel of the fused all-reduce on ONE GPU: the peers' slots and flags are filled by
the test, so nothing waits on another kernel.  The sum must be taken in rank order with fp32
accumulation; a flag that nothing sets must end the bounded wait with a status bit and leave the
data alone (failure detection without a fault)."""
import ctypes as C

import numpy as np
import pytest

from schedforge_b200 import lib as L

pytestmark = pytest.mark.gpu


class PeerArgs(C.Structure):
    _fields_ = [("data", C.c_void_p), ("recv", C.c_void_p), ("local_flags", C.c_void_p),
                ("peer_flags", C.c_void_p * 8), ("rank", C.c_int), ("size", C.c_int), ("epoch", C.c_uint32),
                ("count", C.c_int64), ("slot_elems", C.c_int64)]


def _run(dev, port, size, rank, count, flag_value, epoch):
    torch = dev.torch
    rng = np.random.default_rng(size * 100 + rank)
    slot = (count + 7) // 8 * 8
    partials = [port.round_bf16(rng.standard_normal(count).astype(np.float32)) for _ in range(size)]
    data = dev.bf16(partials[rank])
    recv_host = np.zeros((size, slot), np.float32)
    for s in range(size):
        if s != rank:
            recv_host[s, :count] = partials[s]
    recv = dev.bf16(recv_host)
    local_flags = torch.full((8,), flag_value, dtype=torch.int32, device="cuda")
    sink = torch.zeros((8,), dtype=torch.int32, device="cuda")  # stands in for the peers' flag arrays
    a = PeerArgs()
    a.data, a.recv, a.local_flags = data.data_ptr(), recv.data_ptr(), local_flags.data_ptr()
    for s in range(size):
        a.peer_flags[s] = sink.data_ptr() + 4 * s
    a.rank, a.size, a.epoch, a.count, a.slot_elems = rank, size, epoch, count, slot
    lib = L.load()
    L.check(lib.sfb_k_peer_allreduce_finish(C.byref(a), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    word = C.c_uint32(0)
    L.check(lib.sfb_device_status(C.byref(word)))
    return partials, dev.np(data), dev.np(sink.float()), word.value


@pytest.mark.parametrize("size,rank,count", [(2, 0, 4096), (2, 1, 1000), (4, 2, 8 * 1024 + 3), (8, 7, 70000)])
def test_finish_sums_the_slots_in_rank_order(dev, port, size, rank, count):
    partials, got, sink, status = _run(dev, port, size, rank, count, flag_value=5, epoch=5)
    assert status == 0
    acc = np.zeros(count, np.float32)
    for s in range(size):       # rank order, fp32 accumulation, one rounding to bf16 at the end
        acc = (acc + partials[s]).astype(np.float32)
    assert np.array_equal(got, port.round_bf16(acc))
    for s in range(size):       # the epoch was published to every peer (and to nobody else)
        assert sink[s] == (0 if s == rank else 5)


def test_wait_that_runs_out_sets_the_status_bit_and_keeps_the_partial_sums(dev, port):
    partials, got, _, status = _run(dev, port, 2, 0, 2048, flag_value=0, epoch=1)  # the peer never signals
    assert status & 0x100
    assert np.array_equal(got, partials[0])
    # the device stays usable and the status word was cleared by the read
    _, got2, _, status2 = _run(dev, port, 2, 0, 2048, flag_value=1, epoch=1)
    assert status2 == 0 and not np.array_equal(got2, partials[0])


def test_finish_rejects_bad_groups(dev, port):
    a = PeerArgs()
    a.rank, a.size, a.count, a.slot_elems = 0, 1, 8, 8
    with pytest.raises(L.SfbError):
        L.check(L.load().sfb_k_peer_allreduce_finish(C.byref(a), C.c_void_p(dev.stream())))

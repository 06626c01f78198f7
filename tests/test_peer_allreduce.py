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


class GatherArgs(C.Structure):
    _fields_ = [("recv", C.c_void_p), ("slot_elems", C.c_int64), ("slots", C.c_int), ("pull", C.c_void_p * 8),
                ("source", C.c_void_p),
                ("source_ss", C.c_void_p), ("residual", C.c_void_p), ("gathered", C.c_void_p * 8), ("ss", C.c_void_p * 8),
                ("local_flags", C.c_void_p), ("peer_flags", C.c_void_p * 8), ("done_counter", C.c_void_p),
                ("rank", C.c_int), ("size", C.c_int), ("epoch", C.c_uint32), ("rows_own", C.c_int), ("width", C.c_int),
                ("gather", C.c_int), ("epoch_out", C.c_void_p)]


def _run_gather(dev, port, size, rank, rows_own, width, flag_a, flag_b, epoch, slots=None, with_residual=True, pull=False):
    """The owner's kernel of the two-shot form on ONE GPU: the slots the peers' GEMMs would have filled, the peers'
    copies of the gathered tensor and both flag sets are plain tensors of this GPU prepared by the test."""
    torch = dev.torch
    rng = np.random.default_rng(size * 1000 + rank * 10 + rows_own)
    slots = size if slots is None else slots
    total = size * rows_own
    parts = [port.round_bf16(rng.standard_normal((rows_own, width)).astype(np.float32)) for _ in range(max(slots, 1))]
    residual = port.round_bf16(rng.standard_normal((rows_own, width)).astype(np.float32))
    recv = dev.bf16(np.stack(parts))
    res = dev.bf16(residual)
    copies = [dev.zeros((total, width), torch.bfloat16) for _ in range(size)]      # every rank's full tensor
    sums = [dev.zeros((total,), torch.float32) for _ in range(size)]
    flags = torch.zeros((16,), dtype=torch.int32, device="cuda")
    flags[:8] = flag_a
    flags[8:] = flag_b
    sink = torch.zeros((8, 16), dtype=torch.int32, device="cuda")                   # peers' flag arrays
    counter = torch.zeros((1,), dtype=torch.int32, device="cuda")
    a = GatherArgs()
    if slots > 0 and pull:   # every rank's partial rows sit in a tensor of their own (here: of this GPU)
        a.slots = slots
        singles = [recv[s].clone() for s in range(slots)]
        for s in range(slots):
            a.pull[s] = singles[s].data_ptr()
    elif slots > 0:
        a.recv, a.slot_elems, a.slots = recv.data_ptr(), rows_own * width, slots
    else:
        a.source = recv.data_ptr()
    a.residual = res.data_ptr() if with_residual else None
    for s in range(size):
        a.gathered[s] = copies[s].data_ptr()
        a.ss[s] = sums[s].data_ptr()
        a.peer_flags[s] = sink[s].data_ptr() + 4 * rank
    a.local_flags, a.done_counter = flags.data_ptr(), counter.data_ptr()
    a.rank, a.size, a.epoch, a.rows_own, a.width, a.gather = rank, size, epoch, rows_own, width, 1
    lib = L.load()
    L.check(lib.sfb_k_peer_reduce_gather(C.byref(a), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    word = C.c_uint32(0)
    L.check(lib.sfb_device_status(C.byref(word)))
    acc = np.zeros((rows_own, width), np.float32)
    for part in parts[:max(slots, 1)]:
        acc = (acc + part).astype(np.float32)
    if with_residual:
        acc = (acc + residual).astype(np.float32)
    want = port.round_bf16(acc)
    return want, [dev.np(t) for t in copies], [dev.np(t) for t in sums], dev.np(sink.float()), int(counter.item()), word.value


@pytest.mark.parametrize("pull", [False, True])
@pytest.mark.parametrize("size,rank,rows_own,width", [(2, 1, 64, 256), (4, 2, 37, 512), (8, 5, 128, 4096)])
def test_two_shot_owner_sums_its_rows_and_hands_them_to_every_rank(dev, port, size, rank, rows_own, width, pull):
    want, copies, sums, sink, counter, status = _run_gather(dev, port, size, rank, rows_own, width, 3, 3, 3, pull=pull)
    assert status == 0 and counter == 0
    lo, hi = rank * rows_own, (rank + 1) * rows_own
    for s in range(size):       # the finished rows and their sums of squares landed in every rank's copy, nowhere else
        assert np.array_equal(copies[s][lo:hi], want)
        assert float(np.abs(copies[s][:lo]).sum()) == 0.0 and float(np.abs(copies[s][hi:]).sum()) == 0.0
        assert np.allclose(sums[s][lo:hi], (want.astype(np.float64) ** 2).sum(1), rtol=1e-5)
    for s in range(size):       # both announcements reached every peer's flag array at this rank's entry
        expect = 0 if s == rank else 3
        assert sink[s][rank] == expect and sink[s][8 + rank] == expect


def test_two_shot_all_gather_of_rows_a_rank_already_holds(dev, port):
    want, copies, _, _, _, status = _run_gather(dev, port, 4, 1, 48, 256, 1, 1, 1, slots=0, with_residual=False)
    assert status == 0
    for s in range(4):
        assert np.array_equal(copies[s][48:96], want)


def test_two_shot_wait_that_runs_out_reports_and_leaves_the_rows_alone(dev, port):
    # partial sums never announced: nothing is summed; rows announced late: the sum is done, the wait reports
    _, copies, _, _, _, status = _run_gather(dev, port, 2, 0, 16, 256, 0, 0, 1)
    assert status & 0x100 and float(np.abs(copies[0]).sum()) == 0.0
    want, copies, _, _, counter, status = _run_gather(dev, port, 2, 0, 16, 256, 1, 0, 1)
    assert status & 0x100 and np.array_equal(copies[1][:16], want) and counter == 0


def test_flag_wait_returns_for_a_word_a_copy_wrote_and_reports_one_that_nothing_writes(dev):
    """sfb_k_flag_wait: the kernel stream of sfb_decoder_execute waits with it for "chunk landed" words that the
    copy stream writes behind each upload.  A word at or past the epoch (wrap-around compare) lets it through; a
    word that nothing writes ends the bounded wait with status bit 0x100 and the device stays usable."""
    torch = dev.torch
    lib = L.load()
    flags = torch.tensor([7, 0, 0xFFFFFFF0 - (1 << 32)], dtype=torch.int32, device="cuda")
    word = C.c_uint32(0)
    L.check(lib.sfb_device_status(C.byref(word)))
    for index, epoch in ((0, 7), (0, 5), (2, 0xFFFFFFF0), (0, 0xFFFFFFF8)):   # the last one: 7 is past a wrapped epoch
        L.check(lib.sfb_k_flag_wait(C.c_void_p(flags.data_ptr() + 4 * index), C.c_uint32(epoch), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    L.check(lib.sfb_device_status(C.byref(word)))
    assert word.value == 0
    L.check(lib.sfb_k_flag_wait(C.c_void_p(flags.data_ptr() + 4), C.c_uint32(1), C.c_void_p(dev.stream())))
    torch.cuda.synchronize()
    L.check(lib.sfb_device_status(C.byref(word)))
    assert word.value & 0x100
    assert lib.sfb_k_flag_wait(None, C.c_uint32(1), C.c_void_p(dev.stream())) != 0

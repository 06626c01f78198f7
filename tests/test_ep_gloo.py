"""World-size-2 and -4 checks (gloo, CPU) of the multi-rank index arithmetic:

* token-sharded expert parallelism: every rank routes and dispatches its own contiguous token range with the
  oracle, the histograms are all-gathered, the library's own table function (sfb_moe_ep_tables, the host form of
  what sfb_k_moe_ep_plan computes on the device) gives each rank its send positions, receive segments and return
  table, the rows travel with all-to-all exchanges, and the global dispatch order rebuilt from the ranks must be
  bit-equal to the oracle's single-process dispatch_tokens; the rows must also come back to the positions the
  source's local combine expects;
* the row ownership of the two-shot collective: reduce-scatter by owner, sum in rank order, all-gather."""
import ctypes as C
import os
import pickle
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import binding as ob
from schedforge_b200 import lib as L

TOKENS, HIDDEN, EXPERTS, TOP_K = 96, 32, 8, 2


def problem():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((TOKENS, HIDDEN)).astype(np.float32)
    router = (rng.standard_normal((HIDDEN, EXPERTS)) * 0.3).astype(np.float32)
    bias = np.array([2.0, -1.0, 0.5, 0.0, -3.0, 1.0, 0.0, -0.5], np.float32)   # skewed loads, one nearly empty expert
    return x, router, bias


def ep_tables(counts_all, world, rank):
    lib = L.load()
    local = EXPERTS // world
    send_base, recv_offsets = np.zeros(EXPERTS, np.int32), np.zeros(local + 1, np.int32)
    table = np.zeros((local * world, 4), np.int32)
    ip = C.POINTER(C.c_int)
    flat = np.ascontiguousarray(counts_all, np.int32)
    L.check(lib.sfb_moe_ep_tables(flat.ctypes.data_as(ip), world, EXPERTS, rank, send_base.ctypes.data_as(ip),
                                  recv_offsets.ctypes.data_as(ip), table.ctypes.data_as(ip)))
    return send_base, recv_offsets, table


def exchange(objects, world):
    """all-to-all of python objects: objects[d] goes to rank d; returns what every rank sent to this one."""
    gathered = [None] * world
    dist.all_gather_object(gathered, objects)
    return [gathered[s][dist.get_rank()] for s in range(world)]


def ep_worker(rank, world, port_number, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_number)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    port = ob.Port()
    x, router, bias = problem()
    rows, local = TOKENS // world, EXPERTS // world
    mine = x[rank * rows:(rank + 1) * rows]
    mc = ob.MoeConfig(rows, HIDDEN, 16, EXPERTS, TOP_K)
    ids, weights, counts = port.route_topk(mc, mine, router, bias)
    _, offsets, token_ids, slots, _ = port.dispatch_tokens(mc, mine, ids, weights, counts, copy_values=False)
    counts_all = [None] * world
    dist.all_gather_object(counts_all, counts)
    counts_all = np.stack(counts_all)
    send_base, recv_offsets, table = ep_tables(counts_all, world, rank)
    # send: every locally dispatched row a goes to the owner of its expert at send_base[e] + (a - offsets[e])
    outgoing = [[] for _ in range(world)]
    for e in range(EXPERTS):
        for a in range(offsets[e], offsets[e + 1]):
            outgoing[e // local].append((int(send_base[e] + a - offsets[e]), rank * rows + int(token_ids[a]), int(slots[a]),
                                         mine[token_ids[a]].copy()))
    received = int(recv_offsets[-1])
    recv_tokens, recv_slots = np.full(received, -1, np.int32), np.full(received, -1, np.int32)
    recv_rows = np.zeros((received, HIDDEN), np.float32)
    for batch in exchange(outgoing, world):
        for dest, token, slot, row in batch:
            assert recv_tokens[dest] == -1          # every receive position is written exactly once
            recv_tokens[dest], recv_slots[dest], recv_rows[dest] = token, slot, row
    assert (recv_tokens >= 0).all()
    # return: received row j goes back to its source at (first row of the expert's segment there) + (j - run start)
    back = [[] for _ in range(world)]
    for start, count, source, at_source in table:
        for j in range(start, start + count):
            back[source].append((int(at_source + j - start), recv_rows[j] * 2.0))   # "expert" = times two
    returned = np.zeros((rows * TOP_K, HIDDEN), np.float32)
    hits = np.zeros(rows * TOP_K, np.int32)
    for batch in exchange(back, world):
        for at, row in batch:
            returned[at] = row
            hits[at] += 1
    assert (hits == 1).all()
    # every returned row sits where the local dispatched order has it: row a belongs to token_ids[a]
    assert np.array_equal(returned, 2.0 * mine[token_ids])
    with open(os.path.join(out_dir, f"rank{rank}.pkl"), "wb") as f:
        pickle.dump({"ids": ids, "weights": weights, "recv_offsets": recv_offsets, "recv_tokens": recv_tokens,
                     "recv_slots": recv_slots}, f)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_order_equals_single_process_dispatch(tmp_path, world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port_number = s.getsockname()[1]
    mp.spawn(ep_worker, args=(world, port_number, str(tmp_path)), nprocs=world, join=True)
    parts = [pickle.load(open(tmp_path / f"rank{r}.pkl", "rb")) for r in range(world)]
    port = ob.Port()
    x, router, bias = problem()
    mc = ob.MoeConfig(TOKENS, HIDDEN, 16, EXPERTS, TOP_K)
    ids, weights, counts = port.route_topk(mc, x, router, bias)
    _, offsets, token_ids, slots, _ = port.dispatch_tokens(mc, x, ids, weights, counts, copy_values=False)
    assert counts.min() <= 2 and counts.max() >= 40           # the bias does skew the loads
    assert np.array_equal(np.concatenate([p["ids"] for p in parts]), ids)
    got_offsets, base = [0], 0
    for p in parts:
        got_offsets += [base + int(v) for v in p["recv_offsets"][1:]]
        base += int(p["recv_offsets"][-1])
    assert np.array_equal(np.array(got_offsets, np.int32), offsets)
    assert np.array_equal(np.concatenate([p["recv_tokens"] for p in parts]), token_ids)
    assert np.array_equal(np.concatenate([p["recv_slots"] for p in parts]), slots)


def two_shot_worker(rank, world, port_number, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_number)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows_total, width = 24, 16
    rows_own = rows_total // world
    rng = np.random.default_rng(100 + rank)
    partial = rng.standard_normal((rows_total, width)).astype(np.float32)       # this rank's partial sums
    residual = np.random.default_rng(7).standard_normal((rows_total, width)).astype(np.float32)
    # reduce-scatter: the owner of rows [r * rows_own, ...) fetches those rows of every rank's partial tensor
    everything = [None] * world
    dist.all_gather_object(everything, partial)
    lo, hi = rank * rows_own, (rank + 1) * rows_own
    acc = np.zeros((rows_own, width), np.float32)
    for s in range(world):                      # rank order: the same arithmetic wherever it is done
        acc = (acc + everything[s][lo:hi]).astype(np.float32)
    acc = (acc + residual[lo:hi]).astype(np.float32)
    # all-gather: every owner hands its finished rows (and their sums of squares) to every rank
    finished = [None] * world
    dist.all_gather_object(finished, (acc, (acc.astype(np.float64) ** 2).sum(1)))
    full = np.concatenate([f[0] for f in finished])
    np.save(os.path.join(out_dir, f"full{rank}.npy"), full)
    dist.destroy_process_group()


def test_two_shot_ownership_gives_every_rank_the_same_sum(tmp_path):
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port_number = s.getsockname()[1]
    mp.spawn(two_shot_worker, args=(world, port_number, str(tmp_path)), nprocs=world, join=True)
    partials = [np.random.default_rng(100 + r).standard_normal((24, 16)).astype(np.float32) for r in range(world)]
    residual = np.random.default_rng(7).standard_normal((24, 16)).astype(np.float32)
    want = (partials[0] + partials[1]).astype(np.float32) + residual
    full = [np.load(tmp_path / f"full{r}.npy") for r in range(world)]
    assert np.array_equal(full[0], full[1]) and np.array_equal(full[0], want.astype(np.float32))

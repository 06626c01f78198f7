"""World-size-2 check (gloo, CPU) of the tensor-parallel partition the plan build uses:
rank r owns Q heads [r*Hq/G, ...), KV heads [r*Hkv/G, ...), the matching rows of Wo, columns
r of Wgate/Wup and rows r of Wdown; the partial O-projection and down-projection outputs are
summed with an all-reduce and the residual enters the sum once.  The arithmetic of each
shard is done by the CPU oracle; the shards are cut with the library's own shard functions."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import binding as ob
from schedforge_b200 import api

KW = dict(batch=2, sequence=12, hidden=64, intermediate=96, query_heads=8, kv_heads=4, head_dim=8, rope_theta=10000.0)


def make_data():
    rng = np.random.default_rng(0)
    oc = ob.decoder_config(**KW)
    data = {k: (rng.standard_normal(n) * (1.0 if k == "input" else 0.1)).astype(np.float32)
            for k, n in ob.decoder_shapes(oc).items()}
    return oc, data


def shard_layer(rank, world, oc, data):
    """Weights of one shard, cut with sfb_shard_columns / sfb_shard_rows."""
    h, i, kv = oc.hidden, oc.intermediate, oc.kv_heads * oc.head_dim
    m = lambda name, r, c: data[name].reshape(r, c)
    return {"wq": api.shard_columns(m("query_weight", h, h), rank, world),
            "wk": api.shard_columns(m("key_weight", h, kv), rank, world),
            "wv": api.shard_columns(m("value_weight", h, kv), rank, world),
            "wo": api.shard_rows(m("output_weight", h, h), rank, world),
            "wg": api.shard_columns(m("gate_weight", h, i), rank, world),
            "wu": api.shard_columns(m("up_weight", h, i), rank, world),
            "wd": api.shard_rows(m("down_weight", i, h), rank, world)}


def worker(rank, world, port_number, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_number)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    port = ob.Port()
    oc, data = make_data()
    w = shard_layer(rank, world, oc, data)
    t, h = oc.batch * oc.sequence, oc.hidden
    x = data["input"].reshape(t, h)
    local = ob.decoder_config(**dict(KW, hidden=h // world, query_heads=oc.query_heads // world,
                                     kv_heads=oc.kv_heads // world))
    n1 = port.rms_norm(x, data["rms1_weight"], oc.rms_epsilon)
    fused = port.matmul(n1, np.concatenate([w["wq"], w["wk"], w["wv"]], axis=1), fma=True)
    q, k, v = port.split_qkv_rope(local, fused)
    ac = ob.AttentionConfig(oc.batch, local.query_heads, local.kv_heads, oc.sequence, oc.sequence, oc.head_dim,
                            oc.head_dim, 1, 0.0)
    attn = port.attention_reference(ac, q, k, v)                          # [B, hq_l, S, D]
    merged = np.ascontiguousarray(attn.transpose(0, 2, 1, 3)).reshape(t, -1)
    partial = torch.from_numpy(port.matmul(merged, w["wo"], fma=True))
    if rank == 0:
        partial += torch.from_numpy(x)                                    # residual enters once
    dist.all_reduce(partial)
    r1 = partial.numpy()
    n2 = port.rms_norm(r1, data["rms2_weight"], oc.rms_epsilon)
    act = port.swiglu(port.matmul(n2, np.concatenate([w["wg"], w["wu"]], axis=1), fma=True), oc.intermediate // world)
    down = torch.from_numpy(port.matmul(act, w["wd"], fma=True))
    if rank == 0:
        down += torch.from_numpy(r1)
    dist.all_reduce(down)
    if rank == 0:
        np.save(out_path, down.numpy())
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_layer_matches_unsharded(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port_number = s.getsockname()[1]
    out_path = str(tmp_path / "tp_out.npy")
    mp.spawn(worker, args=(2, port_number, out_path), nprocs=2, join=True)
    oc, data = make_data()
    want = ob.Port().decoder_layer(oc, data, native=True)
    got = np.load(out_path)
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 1e-5   # only the summation order differs

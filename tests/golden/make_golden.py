"""Generates tests/golden/*.npz from the reference itself (oracle/_ref/libsfref.so, built
from the unmodified reference sources by oracle/Makefile).  Run where the reference
sources exist:

    make -C oracle ref && python tests/golden/make_golden.py

Each fixture holds the inputs the reference's own seeded generators produced (the same
shapes and seeds as its unit tests, tests/test_schedforge.cpp) together with the outputs
of its scalar reference and of its native execution path.  The fixtures pin the oracle
port (oracle/port.cpp) and the CUDA path on machines where the reference is absent.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import binding as ob  # noqa: E402

from stablehlo_texts import DECODER_TEXT, MOE_TEXT, NO_QKV_TEXT  # noqa: E402

DECODER_CASES = {
    # name: (config kwargs, seed)  -- shapes/seeds of test_decoder_compiler (tests/test_schedforge.cpp:822-893)
    "decoder_dense": (dict(batch=1, sequence=4, hidden=16, intermediate=32, query_heads=4, kv_heads=2, head_dim=4), 81),
    "decoder_moe": (dict(batch=1, sequence=4, hidden=16, intermediate=32, query_heads=4, kv_heads=2, head_dim=4,
                         moe=True, experts=4, top_k=2), 83),
    "decoder_decode": (dict(batch=1, sequence=1, hidden=16, intermediate=32, query_heads=4, kv_heads=2, head_dim=4,
                            context_sequence=16), 87),
    # the tiny fp32 benchmark shape with the reference's generator
    "decoder_cfg1_shape": (dict(batch=1, sequence=128, hidden=256, intermediate=688, query_heads=4, kv_heads=2,
                                head_dim=64), 0),
    "decoder_batched": (dict(batch=2, sequence=24, hidden=64, intermediate=96, query_heads=4, kv_heads=2, head_dim=16), 5),
    "decoder_moe_medium": (dict(batch=2, sequence=16, hidden=64, intermediate=48, query_heads=4, kv_heads=1, head_dim=16,
                                moe=True, experts=8, top_k=2), 9),
}


def main():
    ref = ob.Ref()
    out = {}
    for name, (kw, seed) in DECODER_CASES.items():
        c = ob.decoder_config(**kw)
        data = ref.make_decoder_data(c, seed)
        dec = ref.decoder_create(c, data, threads=2)
        fixture = {"config": np.array([getattr(c, f) for f, _ in c._fields_], np.float64), "seed": seed}
        fixture.update({"in_" + k: v for k, v in data.items()})
        fixture["out_reference"] = dec.reference()
        fixture["out_native"] = dec.execute_once()[0]
        info = dec.plan_info()
        fixture["attention_strategy"] = info["attention_strategy"]
        dec.close()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **fixture)
        out[name] = fixture["out_reference"].shape

    # attention: causal GQA S9 D8 (test_attention_compiler :689-717), non-causal, decode Sk=11
    for name, (cfg, seed) in {
        "attention_causal_gqa": (ob.AttentionConfig(1, 4, 2, 9, 9, 8, 8, 1, 0.0), 43),
        "attention_dynamic": (ob.AttentionConfig(1, 4, 2, 5, 7, 8, 8, 1, 0.0), 45),
        "attention_noncausal": (ob.AttentionConfig(1, 4, 2, 8, 8, 8, 8, 0, 0.0), 46),
        "attention_decode_gqa": (ob.AttentionConfig(1, 4, 2, 1, 11, 8, 8, 1, 0.0), 47),
        "attention_decode_mqa": (ob.AttentionConfig(1, 4, 1, 1, 11, 8, 8, 1, 0.0), 49),
        "attention_d64": (ob.AttentionConfig(2, 8, 2, 70, 70, 64, 64, 1, 0.0), 3),
    }.items():
        q, k, v = ref.make_attention_data(cfg, seed)
        fixture = {"config": np.array([getattr(cfg, f) for f, _ in cfg._fields_], np.float64), "q": q, "k": k, "v": v,
                   "out_reference": ref.attention_reference(cfg, q, k, v)}
        if cfg.sequence_query > 1:
            fixture["out_io_aware"] = ref.attention_io_aware(cfg, q, k, v, 4, 3, threads=2)
            fixture["out_materialized"] = ref.attention_materialized(cfg, q, k, v)
        else:
            fixture["out_decode"] = ref.decode_attention(cfg, q, k, v, cfg.sequence_kv, threads=4)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **fixture)

    # paged KV (test_next_milestones :369-409): keys = iota, 7 tokens, page 4, capacity 12
    keys = np.arange(2 * 7 * 4, dtype=np.float32).reshape(1, 2, 7, 4)
    values = keys + 1.0
    cache = ref.paged_create(1, 2, 4, 4, 4, 12)
    cache.append(keys, values, 7)
    info = cache.info()
    gk, gv = cache.gather()
    acfg = ob.AttentionConfig(1, 4, 2, 1, 7, 4, 4, 1, 0.0)
    query = np.full((1, 4, 1, 4), 0.125, np.float32)
    paged_out = cache.decode(acfg, query)
    sk, sv = cache.storage()
    cache.truncate(3)
    info_t = cache.info()
    np.savez_compressed(os.path.join(HERE, "paged_kv.npz"), keys=keys, values=values, page_table=info["page_table"],
                        free_pages=info["free_pages"], gathered_keys=gk, gathered_values=gv, query=query,
                        decode_out=paged_out, storage_keys=sk, storage_values=sv,
                        truncated_page_table=info_t["page_table"], truncated_free_pages=info_t["free_pages"])
    cache.close()

    # MoE (test_moe_compiler :616-686): T7 H8 I12 E4 k2 seed 41, plus a larger skewed case
    for name, (cfg, seed) in {"moe_small": (ob.MoeConfig(7, 8, 12, 4, 2), 41),
                              "moe_medium": (ob.MoeConfig(96, 64, 48, 8, 2), 11)}.items():
        d = ref.make_moe_data(cfg, seed)
        ids, weights, counts = ref.route_topk(cfg, d["input"], d["router_weight"])
        values, offsets, token_ids, slots, rw = ref.dispatch_tokens(cfg, d["input"], ids, weights, counts)
        tasks = ref.plan_moe_tasks(cfg, ids, weights, counts)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), config=np.array([getattr(cfg, f) for f, _ in cfg._fields_], np.int32),
            expert_ids=ids, expert_weights=weights, counts=counts, dispatched=values, offsets=offsets,
            token_ids=token_ids, route_slots=slots, routing_weights=rw, tasks=tasks,
            out_reference=ref.moe_reference(cfg, d["input"], d["w1"], d["w3"], d["w2"], ids, weights, counts),
            out_native=ref.moe_grouped(cfg, d["input"], d["w1"], d["w3"], d["w2"], ids, weights, counts, threads=3),
            **{"in_" + k: v for k, v in d.items()})

    # importer + fusion pass on three texts
    import json
    summary = {"decoder": ref.import_stablehlo(DECODER_TEXT), "moe": ref.import_stablehlo(MOE_TEXT, moe=True),
               "no_qkv": ref.import_stablehlo(NO_QKV_TEXT),
               "canonical_dense": ref.canonical_graph_names(ob.decoder_config()),
               "canonical_moe": ref.canonical_graph_names(ob.decoder_config(moe=True))}
    with open(os.path.join(HERE, "importer.json"), "w") as f:
        json.dump(summary, f, indent=1, sort_keys=True)
    # the benchmark matrix: 24 profiles with their estimates, both CSV headers, one compile-only row
    with open(os.path.join(HERE, "decoder_profiles.txt"), "w") as f:
        f.write(ref.decoder_profiles())
    # make_routing_trace for the three distributions (benchmark_decoder_profile uses seed 103)
    traces = {}
    for distribution, experts in ((0, 8), (1, 8), (2, 16)):
        cfg = ob.MoeConfig(32, 512, 1376, experts, 2)
        ids, weights, counts = ref.make_routing_trace(cfg, distribution, 103)
        traces.update({f"ids{distribution}": ids, f"weights{distribution}": weights, f"counts{distribution}": counts})
    np.savez(os.path.join(HERE, "routing_traces.npz"), **traces)
    # bf16 rounding known answers
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5e-3, 3.1415927, 65504.0, 1e-30, 0.1], np.float32)
    np.savez(os.path.join(HERE, "bf16_round.npz"), x=x, y=ref.round_bf16(x))
    print("wrote fixtures:", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()

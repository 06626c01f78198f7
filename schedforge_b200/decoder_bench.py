"""Runs the reference's decoder benchmark matrix on the device plan and writes its two CSV files.

    python -m schedforge_b200.decoder_bench [--suite realistic|optimizer] [--output decoder_realistic.csv]
        [--repetitions 3] [--max-real-gflop 1e9] [--max-weight-mib 1e9] [--filter tiny-decode] [--optimize]

The counterpart of tools/schedforge-decoder-bench.cpp of the reference (same suites, filter and budget
switches; the budgets default to "everything fits", because a 708 MB layer is small for this device).
A profile above a budget is recorded as compile-only, like there.  `<output>` receives the benchmark
rows and `<output minus .csv>_candidates.csv` the optimizer's candidates.
"""
import argparse
import sys

from . import api, lib as L


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--suite", choices=("realistic", "optimizer"), default="realistic")
    ap.add_argument("--output", default="decoder_realistic.csv")
    ap.add_argument("--repetitions", type=int, default=3)
    ap.add_argument("--max-real-gflop", type=float, default=1.0e9)
    ap.add_argument("--max-weight-mib", type=float, default=1.0e9)
    ap.add_argument("--filter", default="")
    ap.add_argument("--optimize", action="store_true")
    args = ap.parse_args(argv)
    optimize = args.optimize or args.suite == "optimizer"
    profiles = [p for p in api.realistic_decoder_profiles() if args.filter in p.name.decode()]
    if args.suite == "optimizer":  # the two dense profiles the reference's optimizer suite keeps
        profiles = [p for p in profiles if p.name.decode() in ("tiny-prefill-s128", "tiny-decode-kv512")]
    records = []
    for p in profiles:
        print(f"[Profile] {p.name.decode()} ... ", end="", flush=True)
        r = api.benchmark_decoder_profile(p, max_real_flops=int(args.max_real_gflop * 1.0e9),
                                          max_real_weight_bytes=int(args.max_weight_mib * 1024 * 1024),
                                          optimize_plan=optimize, repetitions=args.repetitions)
        text = {L.EVIDENCE_MEASURED: "measured", L.EVIDENCE_COMPILE_ONLY: "compile-only"}.get(r.evidence, "skipped")
        if r.evidence == L.EVIDENCE_MEASURED:
            text += f" {r.measured.milliseconds:.4f} ms, {r.measured.tokens_per_second:.1f} tokens/s"
            if optimize:
                text += f", optimizer speedup {r.optimizer_speedup:.3f}"
        print(text, flush=True)
        records.append(r)
    api.write_decoder_benchmark_csv(args.output, records)
    stem = args.output[:-4] if args.output.endswith(".csv") else args.output
    api.write_decoder_plan_candidates_csv(stem + "_candidates.csv", records)
    print(f"wrote {args.output} ({len(records)} rows)")
    return 0


if __name__ == "__main__":
    sys.exit(main())

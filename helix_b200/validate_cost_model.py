"""Check the profiled cost model against measurement on the benchmark shapes.

  python -m helix_b200.validate_cost_model [--exhaustive]

Profiles the fp16 dictionary (as `profile_template.py -b Ampere_FP16` does), then for every shape prints
the configuration the model picks, its predicted and measured time, and -- with --exhaustive -- the
best measured time over the whole search space.  The reference compares its model's pick with the
exhaustive optimum the same way ("Oracle" vs "Default",
scripts/Ampere_FP16/benchmark_Ampere_FP16_performance_comparison.py:44-93).
"""
import argparse
import sys

from . import costmodel, datagen, harness, workloads


def shapes():
    out = [(M, N, K, None) for (M, N, K) in datagen.C3_SHAPES]
    seen = set()
    for u in workloads.model_level_sweep():
        if u["kind"] != "gemm":
            continue
        s = tuple(u["shape"])
        if s in seen:
            continue
        seen.add(s)
        out.append((s[0], s[1], s[2], s[3] if len(s) > 3 else None))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--exhaustive", action="store_true", help="also time every applicable configuration")
    args = ap.parse_args(argv)
    d = harness.profile_fp16()
    print("profiled:", {k: (round(v, 3) if isinstance(v, float) else v) for k, v in d.items() if len(k) == 1})
    print("%-28s %-28s %10s %10s %6s %10s" % ("shape (M,N,K,batch)", "model's pick", "pred us", "meas us", "ratio", "best us"))
    worst = 0.0
    for (M, N, K, b) in shapes():
        key = harness.cost_model(d, M, N, K, b)
        pred = harness.predicted_time(d, key, M, N, K, b)
        meas = harness.time_gemm_f16(M, N, K, harness.key_to_cfg(key), b)
        best = float("nan")
        if args.exhaustive:
            best = min(harness.time_gemm_f16(M, N, K, harness.key_to_cfg(k), b) for k in costmodel.gemm_keys()
                       if costmodel.gemm_time(d, k, M, N, K, b or 1) < float("inf"))
            worst = max(worst, meas / best)
        print("%-28s %-28s %10.1f %10.1f %6.2f %10.1f" % ((M, N, K, b), key, pred * 1e6, meas * 1e6, pred / meas,
                                                          best * 1e6), flush=True)
    if args.exhaustive:
        print("worst pick / exhaustive best: %.2f" % worst)
    # the same model asked about ONE launch (no overlap with neighbours), for the memory-bound shapes
    print("lone launches:")
    for (M, N, K, b) in [s for s in shapes() if harness.overlaps(*s)]:
        key = costmodel.cost_model(d, M, N, K, b or 1)
        pred = costmodel.predicted_time(d, key, M, N, K, b or 1)
        meas = harness.time_gemm_f16(M, N, K, harness.key_to_cfg(key, prof_dict=d), b, lone=True)
        lib = harness.time_gemm_f16(M, N, K, None, b, lone=True)
        print("%-28s %-28s %10.1f %10.1f %6.2f   library default %.1f" % ((M, N, K, b), key, pred * 1e6, meas * 1e6,
                                                                         pred / meas, lib * 1e6), flush=True)
    # convolutions (the five ResNet-style layers): the model's pick against the library's default
    print("convolutions:")
    for layer in datagen.C4_LAYERS:
        B, C, H, W, OC, kh, kw, stride, pad = layer
        cost_ms, _ = harness.conv_f16_result(d, *layer)
        lib = harness.time_conv_f16(*layer)
        print("%-40s model's pick %8.1f us   library default %8.1f us" % (layer, cost_ms * 1e3, lib * 1e6), flush=True)
    print("searched fields:", {k: v for k, v in d.items() if k[0] in ("load_group", "load_group_probe", "stages_probe",
                                                                     "splitk_overhead", "conv_slab", "conv_slab_swap")})
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Profiling tool, not part of the operator path: run one operator a few times on seeded data -- the target of
the `ncu` captures whose summaries are kept under profiles/ (their command lines name this module).

  python -m helix_b200.profile_case gemm M N K [--batch B] [--bn 256] [--pair] [--stream-k] [--swap] [--reps 3]
  python -m helix_b200.profile_case conv B IC H W OC kH kW stride pad [--bn 128] [--reps 3]
  python -m helix_b200.profile_case gemv ROWS K [--m 1] [--reps 3]
  python -m helix_b200.profile_case sgemm M N K [--reps 3]
  python -m helix_b200.profile_case gemv32 ROWS K [--m 1] [--reps 3]
  ... [--probe P] [--time]   leave out the MMAs or an operand's loads (helix_cfg_t.probe) and print the time

Keeps device memory small and launches few kernels, so that a full-metric capture of one launch
(`ncu --set full --clock-control none -k regex:<kernel> -s 1 -c 1 ...`) ends by itself quickly.
"""
import argparse
import sys

import torch

from . import datagen, ops
from ._lib import OP_CONV_F16, OP_GEMM_F16


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "conv", "gemv", "sgemm", "gemv32"])
    ap.add_argument("dims", type=int, nargs="+")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--stream-k", action="store_true")
    ap.add_argument("--swap", action="store_true")
    ap.add_argument("--pair", action="store_true", help="CTA-pair kernel (cta_group 2) with the --bn tile width")
    ap.add_argument("--gather", action="store_true", help="conv: gathering producer warps even where a tensor map applies")
    ap.add_argument("--probe", type=int, default=0,
                    help="helix_cfg_t.probe: 1 = no MMAs, 2 = no A loads, 4 = no B loads, 16*g = g stages per arrival barrier")
    ap.add_argument("--split-k", type=int, default=1)
    ap.add_argument("--time", action="store_true", help="also print microseconds per launch (CUDA-graph replay, events)")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args(argv)
    dev = "cuda"
    if args.op == "gemm":
        M, N, K = args.dims
        a, b = datagen.c3_gemm(M, N, K, seed=2, batch=args.batch)
        a, b = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        cfg = None
        if args.bn and args.pair:
            cfg = ops.make_cfg(OP_GEMM_F16, 128, args.bn, 64, cta_group=2, probe=args.probe)
        elif args.bn:
            cfg = ops.make_cfg(OP_GEMM_F16, 128, args.bn, 64, stream_k=int(args.stream_k), swap_ab=int(args.swap),
                               load_group=0, probe=args.probe, split_k=args.split_k)
        for _ in range(args.reps):
            out = ops.gemm_f16(a, b, cfg=cfg)
        if args.time:
            l = ops.launch_gemm_f16(a, b, out, cfg)
            print("us per launch: %.2f" % (ops.time_launches([l] * 4, warmup=3, iters=20, use_graph=True)[0] * 1e6))
    elif args.op == "conv":
        geom = tuple(args.dims)
        x, w = datagen.c4_conv(*geom, seed=3)
        x, w = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
        cfg = None
        if args.bn:
            cfg = ops.make_cfg(OP_CONV_F16, 128, args.bn, 64, stream_k=int(args.stream_k), swap_ab=int(args.swap),
                               conv_gather=int(args.gather), probe=args.probe, split_k=args.split_k)
        for _ in range(args.reps):
            out = ops.conv2d_f16_nhwc(x, w, geom[7], geom[8], cfg=cfg)
        if args.time:
            l = ops.launch_conv2d_f16(x, w, out, geom[7], geom[8], cfg)
            print("us per launch: %.2f" % (ops.time_launches([l] * 4, warmup=3, iters=20, use_graph=True)[0] * 1e6))
    elif args.op == "gemv":
        rows, K = args.dims
        w, x = datagen.c2_gemv(rows, K, args.m, seed=1)
        w, x = torch.from_numpy(w).to(dev), torch.from_numpy(x).to(dev)
        for _ in range(args.reps):
            out = ops.gemv_f16(w, x)
    elif args.op == "gemv32":
        rows, K = args.dims
        w = (torch.rand(rows, K, device=dev) * 2 - 1)
        x = (torch.rand(args.m, K, device=dev) * 2 - 1)
        for _ in range(args.reps):
            out = ops.gemv_f32(w, x)
    else:
        M, N, K = args.dims
        a, b = datagen.c1_fp32_gemm(M, N, K, seed=0)
        a, b = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        for _ in range(args.reps):
            out = ops.gemm_f32(a, b)
    torch.cuda.synchronize()
    ops.check_status()
    print("ok", tuple(out.shape), float(out.float().abs().mean()))
    return 0


if __name__ == "__main__":
    sys.exit(main())

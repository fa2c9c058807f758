"""One oversized fp16 GEMM over the GPUs of one box, split along N, with no collective in the data path.

The reference runs every GEMM on GPU 0 (src_template/Ampere_FP16/gemm.cu:585-660 never selects a
device).  C = A x B^T with B stored [N, K] (gemm.cu:597-601) splits naturally by rows of B: rank r
keeps the contiguous slab B[n0:n1, :], a replica of A, and writes the column slab C[:, n0:n1] into a
buffer of its own.  Nothing is reduced and nothing is exchanged in the timed region; an all-gather
of the slabs exists only for verification.

Operands are drawn block by block (256 rows per block, one generator per block seeded with the
matrix seed and the block index), so a rank draws exactly its rows and the bytes of a row do not
depend on how many ranks share the matrix.

Under `python -m torch.distributed.run --nproc-per-node G -m helix_b200.nsplit M N K` every rank times
its own slab with CUDA events; the job's time is the slowest rank's.
"""
import argparse
import json
import os

import numpy as np

ROW_BLOCK = 256          # rows per seeded block; slab boundaries fall on multiples of it


def slab_bounds(N, world, rank, align=ROW_BLOCK):
    """[n0, n1) of rank `rank`: blocks of `align` rows of B dealt contiguously and as evenly as possible.

    The slabs of ranks 0..world-1 tile [0, N) exactly; a rank may get an empty slab when there are
    fewer blocks than ranks.
    """
    if world < 1 or not (0 <= rank < world) or N < 0 or align < 1:
        raise ValueError("slab_bounds: bad arguments")
    blocks = (N + align - 1) // align
    b0 = blocks * rank // world
    b1 = blocks * (rank + 1) // world
    return min(b0 * align, N), min(b1 * align, N)


def seeded_rows(seed, r0, r1, K, scale):
    """Rows [r0, r1) of the fp16 matrix with `K` columns whose 256-row blocks are drawn from
    default_rng([seed, block]) as N(0,1)*scale; r0 must be a multiple of the block size."""
    if r0 % ROW_BLOCK:
        raise ValueError("seeded_rows: r0 must be a multiple of %d" % ROW_BLOCK)
    out = np.empty((max(r1 - r0, 0), K), dtype=np.float16)
    for b0 in range(r0, r1, ROW_BLOCK):
        n = min(ROW_BLOCK, r1 - b0)
        rng = np.random.default_rng([int(seed), b0 // ROW_BLOCK])
        blk = rng.standard_normal((ROW_BLOCK, K), dtype=np.float32) * np.float32(scale)
        out[b0 - r0:b0 - r0 + n] = blk[:n].astype(np.float16)
    return out


def operands(M, N, K, seed, world, rank):
    """(A[M,K], B[n0:n1,K], (n0, n1)) as numpy fp16; A is the same on every rank."""
    s = 1.0 / np.sqrt(K)
    n0, n1 = slab_bounds(N, world, rank)
    a = seeded_rows(2 * int(seed), 0, M, K, s)
    b = seeded_rows(2 * int(seed) + 1, n0, n1, K, s)
    return a, b, (n0, n1)


def assemble(slabs, bounds, M, N):
    """Full C[M,N] from per-rank column slabs (verification only)."""
    c = np.empty((M, N), dtype=slabs[0].dtype)
    seen = 0
    for s, (n0, n1) in zip(slabs, bounds):
        if s.shape != (M, n1 - n0):
            raise ValueError("assemble: slab shape does not match its bounds")
        c[:, n0:n1] = s
        seen += n1 - n0
    if seen != N:
        raise ValueError("assemble: slabs do not tile N")
    return c


class NSplitGemm:
    """This rank's share of C[M,N] = A[M,K] x B[N,K]^T on the current CUDA device."""

    def __init__(self, M, N, K, seed, world, rank, device="cuda", cfg=None):
        import torch
        from . import ops
        self.M, self.N, self.K, self.world, self.rank = M, N, K, world, rank
        a, b, (self.n0, self.n1) = operands(M, N, K, seed, world, rank)
        self.a = torch.from_numpy(a).to(device)
        self.b = torch.from_numpy(b).to(device)
        self.c = torch.empty(M, self.n1 - self.n0, dtype=torch.float16, device=device)
        self.launch = ops.launch_gemm_f16(self.a, self.b, self.c, cfg=cfg) if self.n1 > self.n0 else None
        self.flops = 2.0 * M * (self.n1 - self.n0) * K

    def step(self):
        from . import ops
        if self.launch is not None:
            ops.run(self.launch)
        return 1 if self.launch is not None else 0

    def gather(self, dist=None):
        """Full C on every rank (numpy fp16): slabs padded to the widest one, all-gathered, trimmed."""
        import torch
        if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
            return assemble([self.c.cpu().numpy()], [(self.n0, self.n1)], self.M, self.N)
        bounds = [slab_bounds(self.N, self.world, r) for r in range(self.world)]
        widest = max(n1 - n0 for n0, n1 in bounds)
        mine = torch.zeros(self.M, widest, dtype=torch.float16, device=self.c.device)
        mine[:, :self.n1 - self.n0] = self.c
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine)
        return assemble([p[:, :n1 - n0].cpu().numpy() for p, (n0, n1) in zip(parts, bounds)], bounds, self.M, self.N)


def main(argv=None):
    ap = argparse.ArgumentParser(description="one fp16 GEMM split along N over the ranks of a torchrun job")
    # positional M N K, as the reference's kernel executables take them (gemm.cu:669)
    ap.add_argument("m", type=int, nargs="?", default=8192)
    ap.add_argument("n", type=int, nargs="?", default=65536)
    ap.add_argument("k", type=int, nargs="?", default=8192)
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--verify", action="store_true", help="all-gather C (untimed) and compare ranks' checksums")
    args = ap.parse_args(argv)
    import torch
    from . import dist_util, ops
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g = NSplitGemm(args.m, args.n, args.k, args.seed, world, rank)
    for _ in range(max(args.warmup, 1)):
        g.step()
    torch.cuda.synchronize()
    ops.check_status()
    dist_util.barrier(dist)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        g.step()
    e1.record()
    torch.cuda.synchronize()
    dist_util.barrier(dist)
    own_ms = e0.elapsed_time(e1) / args.steps
    ms = dist_util.max_over_ranks(own_ms, dist, "cuda")
    ops.check_status()
    line = {"metric": "fp16 GEMM split along N", "M": args.m, "N": args.n, "K": args.k, "n_gpus": world,
            "ms_per_step": ms, "value": 2.0 * args.m * args.n * args.k / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "scaling": "strong", "slab": [g.n0, g.n1], "rank0_ms": own_ms,
            "collectives_in_timed_region": 0}
    if args.verify:
        c = g.gather(dist)
        digest = float(np.abs(c.astype(np.float32)).sum())
        line["checksum_abs_sum"] = digest
        line["checksum_spread_over_ranks"] = dist_util.max_over_ranks(digest, dist, "cuda") - \
            (-dist_util.max_over_ranks(-digest, dist, "cuda"))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

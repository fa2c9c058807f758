"""Run a list of independent GEMM / convolution units on one GPU.

This is the in-process form of the reference's sweep loops, which call one
executable per shape (scripts/Ampere_FP16/benchmark_Ampere_FP16_gemm.py:9-17,
benchmark_Ampere_FP16_model_level_LLM.py:9-27, ..._CNN.py:9-27): every unit gets
its own operand buffers in HBM and one prepared launch; ``step()`` queues all of
them on the current stream.  ``HostSweep`` is the host-buffer variant (pinned
host operands copied in, results copied out, copies overlapped with compute).
"""
import math

import torch

from . import ops, workloads
from ._lib import LAUNCH_INDEPENDENT

def unit_operand_shapes(unit):
    """Shapes (a, b, out) of a unit's device tensors in the layouts the kernels take."""
    s = unit["shape"]
    if unit["kind"] == "gemm":
        M, N, K = s[:3]
        if len(s) > 3:
            return (s[3], M, K), (s[3], N, K), (s[3], M, N)
        return (M, K), (N, K), (M, N)
    B, IC, H, W, OC, kh, kw, stride, pad = s
    C = ops.conv_stored_channels(IC, H, W, OC, kh, kw, stride, pad)   # C = 3 is stored as 4 (first layer) or 8
    Ho, Wo = ops.conv_out_hw(H, W, kh, kw, stride, pad)
    return (B, H, W, C), (OC, kh, kw, C), (B, Ho, Wo, OC)


def _fill(shape, scale, gen, device, valid_channels=None):
    t = torch.empty(shape, dtype=torch.float16, device=device)
    t.normal_(0.0, 1.0, generator=gen)
    t.mul_(scale)
    if valid_channels is not None and valid_channels < shape[-1]:
        t[..., valid_channels:] = 0
    return t


class Sweep:
    """Device-resident sweep: distinct operand buffers per unit, one prepared launch each."""

    def __init__(self, units, seed=4, device=None, cfg_for=None, lanes=1, seeds=None):
        """lanes > 1: the units are dealt to that many streams (balanced by estimated time) and every launch is limited to
        1/lanes of the SMs, so independent shapes run side by side with longer-lived CTAs (the set-up and
        drain of one launch hide behind the steady state of its neighbour).
        seeds: one integer per unit that replaces its position in the data seed, so that a unit of a
        partitioned list gets the same bytes whichever GPU it lands on."""
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.lanes = max(1, int(lanes))
        self.units = list(units)
        self.tensors = []
        self.launches = []
        # lanes: longest-processing-time-first on a roofline estimate of each unit, so that the chains end a
        # step together (round-robin puts all the heavy GEMMs of a repeated layer pattern into one chain)
        est = [max(workloads.unit_flops(u) / 1.0e15, workloads.unit_bytes(u) / 5.0e12) + 4e-6 for u in self.units]
        self.lane_of = [0] * len(self.units)
        if self.lanes > 1:
            for lane, idxs in enumerate(workloads.lpt_partition(est, self.lanes)):
                for i in idxs:
                    self.lane_of[i] = lane
        # odd lanes walk their units backwards: while one chain is in the memory-bound part of the list
        # (batched attention GEMMs, 1x1 convolutions) its neighbour is in a tensor-bound part
        per_lane = [[i for i in range(len(self.units)) if self.lane_of[i] == lane] for lane in range(self.lanes)]
        for lane in range(1, self.lanes, 2):
            per_lane[lane].reverse()
        self.issue_order = [lst[j] for j in range(max(map(len, per_lane))) for lst in per_lane if j < len(lst)]
        gen = torch.Generator(device=self.device)
        for i, u in enumerate(self.units):
            gen.manual_seed(int(seed) * 1000003 + (int(seeds[i]) if seeds is not None else i))
            sa, sb, so = unit_operand_shapes(u)
            if u["kind"] == "gemm":
                K = u["shape"][2]
                scale = 1.0 / math.sqrt(K)
                a = _fill(sa, scale, gen, self.device)
                b = _fill(sb, scale, gen, self.device)
            else:
                B, IC, H, W, OC, kh, kw, stride, pad = u["shape"]
                scale = 1.0 / math.sqrt(IC * kh * kw)
                a = _fill(sa, scale, gen, self.device, valid_channels=IC)
                b = _fill(sb, scale, gen, self.device, valid_channels=IC)
            out = torch.empty(so, dtype=torch.float16, device=self.device)
            self.tensors.append((a, b, out))
            cfg = cfg_for(u) if cfg_for is not None else None
            l = self._prepare(u, a, b, out, cfg)
            # units of a sweep share no buffers, so a launch need not wait for its predecessor
            l.flags = LAUNCH_INDEPENDENT
            if self.lanes > 1:
                ops.limit_ctas(l, self.lane_sms()[self.lane_of[i]], lane=self.lane_of[i])
            self.launches.append(l)
        self.flops = sum(workloads.unit_flops(u) for u in self.units)
        self.bytes = sum(workloads.unit_bytes(u) for u in self.units)

    def lane_sms(self):
        """SMs each lane's launches may spread over: even shares (CTA pairs), the SMs left over handed out two at a
        time to the first lanes (148 SMs on four lanes: 38, 38, 36, 36)."""
        sms = ops.device_info().sm_count
        base = (sms // self.lanes) & ~1
        extra = (sms - base * self.lanes) // 2
        return [base + (2 if lane < extra else 0) for lane in range(self.lanes)]

    @staticmethod
    def _prepare(u, a, b, out, cfg):
        if u["kind"] == "gemm":
            return ops.launch_gemm_f16(a, b, out, cfg)
        stride, pad = u["shape"][7], u["shape"][8]
        return ops.launch_conv2d_f16(a, b, out, stride, pad, cfg)

    def step(self):
        """Queue every unit once (on the current stream, or dealt to the lanes' streams, which fork from
        and join back into the current stream); returns the number of library launches."""
        before = ops.launch_count()
        if self.lanes == 1:
            for l in self.launches:
                ops.run(l)
            return ops.launch_count() - before
        main = torch.cuda.current_stream()
        if getattr(self, "_streams", None) is None:
            self._streams = [torch.cuda.Stream(device=self.device) for _ in range(self.lanes)]
        fork = torch.cuda.Event()
        fork.record(main)
        for s in self._streams:
            s.wait_event(fork)
        for i in self.issue_order:
            with torch.cuda.stream(self._streams[self.lane_of[i]]):
                ops.run(self.launches[i])
        for s in self._streams:
            done = torch.cuda.Event()
            done.record(s)
            main.wait_event(done)
        return ops.launch_count() - before


class HostSweep:
    """Host-buffer sweep: per step every operand travels host -> device and every result back.

    Pinned host buffers are shared between units of identical shape (the twelve BERT layers
    reuse one set), device buffers are the sweep's own.  Copies run on two side streams and
    overlap the kernels; a unit's kernel waits for its operands, its download for the kernel.
    """

    def __init__(self, sweep):
        self.sweep = sweep
        self.host = {}
        for u, (a, b, out) in zip(sweep.units, sweep.tensors):
            key = (u["kind"], tuple(u["shape"]))
            if key not in self.host:
                ha = torch.empty(a.shape, dtype=a.dtype, pin_memory=True)
                hb = torch.empty(b.shape, dtype=b.dtype, pin_memory=True)
                ho = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
                ha.copy_(a)
                hb.copy_(b)
                self.host[key] = (ha, hb, ho)
        self.h2d = torch.cuda.Stream()
        self.d2h = torch.cuda.Stream()
        self.h2d_bytes = sum(a.numel() * 2 + b.numel() * 2 for a, b, _ in sweep.tensors)
        self.d2h_bytes = sum(o.numel() * 2 for _, _, o in sweep.tensors)
        self._done = [None] * len(sweep.units)
        self._drained = [None] * len(sweep.units)

    def step(self):
        compute = torch.cuda.current_stream()
        for i, (u, (a, b, out), l) in enumerate(zip(self.sweep.units, self.sweep.tensors, self.sweep.launches)):
            ha, hb, ho = self.host[(u["kind"], tuple(u["shape"]))]
            with torch.cuda.stream(self.h2d):
                if self._done[i] is not None:
                    self.h2d.wait_event(self._done[i])   # previous step's kernel still reads a, b
                a.copy_(ha, non_blocking=True)
                b.copy_(hb, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.h2d)
            compute.wait_event(ready)
            if self._drained[i] is not None:
                compute.wait_event(self._drained[i])     # previous step's download still reads out
            ops.run(l)
            done = torch.cuda.Event()
            done.record(compute)
            self._done[i] = done
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(done)
                ho.copy_(out, non_blocking=True)
                drained = torch.cuda.Event()
                drained.record(self.d2h)
            self._drained[i] = drained

    def finish(self):
        self.h2d.synchronize()
        self.d2h.synchronize()
        torch.cuda.current_stream().synchronize()

"""Operator front-end over the C ABI.  torch supplies device memory and streams only.

These calls replace what the reference does by spawning a per-configuration
executable and parsing its stdout (scripts/Ampere_FP16/Ampere_FP16_gemm.py
:432-441, scripts/Ampere_FP16/Ampere_FP16_conv.py:431-446,
scripts/Ampere_FP32/Ampere_FP32_gemm.py:101-107).  Layouts follow the reference
kernels: fp16 GEMM takes A[M,K] and B stored [N,K]; fp32 GEMM takes A[M,K] (or
K x M with ``trans_a``) and B[K,N].
"""
import ctypes

import torch

from . import _lib
from ._lib import Cfg, DevInfo, Launch, OP_CONV_F16, OP_GEMM_F16, OP_GEMM_F32, OP_GEMV_F16, check

_status_words = {}
_workspaces = {}


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("helix_b200 operators take CUDA tensors only (there is no CPU path)")


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device=None):
    """Per-device int32 the kernels write HELIX_ERR_TIMEOUT into when a bounded wait runs out."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev not in _status_words:
        _status_words[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _status_words[dev]


def check_status(device=None):
    """Synchronising read of the status word; raises HelixError if a kernel reported a failure."""
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise _lib.HelixError(v, "device status word")


def workspace(nbytes, device=None, lane=0):
    """Grow-only scratch buffer per device (and per lane of concurrent launch chains), reused across
    calls that are ordered on one stream."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    cur = _workspaces.get((dev, lane))
    if cur is None or cur.numel() < nbytes:
        cur = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=f"cuda:{dev}")
        _workspaces[(dev, lane)] = cur
    return cur


def limit_ctas(launch, max_ctas, lane=0):
    """Let `launch` spread over at most `max_ctas` SMs (so that independent launches on other streams can
    run beside it) and give it the scratch buffer of its lane; the library re-chooses its configuration
    for the smaller machine when cfg is left to it."""
    lib = _lib.load()
    launch.cfg.max_ctas = int(max_ctas)
    need = lib.helix_workspace_bytes(ctypes.byref(launch))
    if need:
        buf = workspace(need, lane=lane)
        launch.ws = buf.data_ptr()
        launch.ws_bytes = buf.numel() * buf.element_size()
        launch._ws_ref = buf
    else:
        launch.ws, launch.ws_bytes = None, 0
    return launch


def device_info(dev=-1):
    info = DevInfo()
    check(_lib.load().helix_device_info(dev, ctypes.byref(info)), "helix_device_info")
    return info


def configs(op):
    lib = _lib.load()
    out = []
    for i in range(lib.helix_num_configs(op)):
        c = Cfg()
        if lib.helix_get_config(op, i, ctypes.byref(c)) == 0:
            out.append(c)
    return out


def default_config(launch):
    """The configuration the library picks for `launch` when its cfg is left zero (helix_default_config)."""
    c = Cfg()
    check(_lib.load().helix_default_config(ctypes.byref(launch), ctypes.byref(c)), "helix_default_config")
    return c


def kernel_name(launch):
    """Name of the main kernel `launch` resolves to, as a profiler lists it."""
    c = launch.cfg if launch.cfg.tile_n or launch.cfg.tile_m else default_config(launch)
    if launch.op == _lib.OP_GEMV_F16:
        return "gemv_f16_kernel"
    if launch.op == _lib.OP_GEMV_F32:
        return "gemv_f32_kernel"
    if launch.op == _lib.OP_GEMM_F32:
        return "sgemm_f32_kernel<%d,%d>" % (c.tile_m, c.tile_n)
    if c.cta_group == 2:
        return "gemm_f16_tc2_kernel<%d>" % c.tile_n
    gathers = False
    if launch.op == OP_CONV_F16:
        n, h, w, ch, ko, r, s, stride, pad = list(launch.conv)
        if ch == 4:
            return "conv_f16_stem_kernel<%d>" % (4 if ko <= 64 else 2)
        rows_geom = ch == 64 and ko == 64 and r == 3 and s == 3 and stride == 1 and pad == 1 and w + 2 <= 64
        if rows_geom and c.conv_gather == 4:    # explicit, or the library's default for this geometry
            return "conv_f16_rows_kernel"
        as_gemm = r == 1 and s == 1 and stride == 1 and pad == 0
        im2col = ch % 64 == 0 and n * h * w * ch * 2 >= 131072 and stride <= 8 and not c.conv_gather
        gathers = not as_gemm and not im2col
    return "gemm_f16_tc_kernel<%d,%d>" % (c.tile_n, 1 if gathers else 0)


def make_cfg(op, tile_m=128, tile_n=128, tile_k=64, stages=0, cta_group=1, split_k=1, swap_ab=0, raster=8,
             thread_m=0, thread_n=0, load_group=0, stream_k=0, conv_gather=0, probe=0):
    c = Cfg()
    c.op, c.tile_m, c.tile_n, c.tile_k, c.stages = op, tile_m, tile_n, tile_k, stages
    c.cta_group, c.split_k, c.swap_ab, c.raster, c.thread_m, c.thread_n = cta_group, split_k, swap_ab, raster, thread_m, thread_n
    c.load_group = load_group
    c.stream_k = stream_k
    c.conv_gather = conv_gather
    c.probe = probe
    return c


# ----------------------------------------------------------------------------- launch builders
def _finish(launch, cfg, ws):
    lib = _lib.load()
    if cfg is not None:
        launch.cfg = cfg
    need = lib.helix_workspace_bytes(ctypes.byref(launch))
    if need:
        buf = ws if ws is not None else workspace(need)
        if buf.numel() * buf.element_size() < need:
            raise ValueError(f"workspace too small: need {need} bytes")
        launch.ws = buf.data_ptr()
        launch.ws_bytes = buf.numel() * buf.element_size()
        launch._ws_ref = buf
    return launch


def launch_gemm_f16(a, b_nk, out, cfg=None, ws=None):
    """A[M,K] (or [B,M,K]) x B[N,K] (or [B,N,K]) -> out[M,N] (or [B,M,N]), fp16."""
    _require_cuda(a, b_nk, out)
    assert a.dtype == b_nk.dtype == out.dtype == torch.float16
    l = Launch()
    l.op = OP_GEMM_F16
    if a.dim() == 3:
        assert a.stride(2) == 1 and b_nk.stride(2) == 1 and out.stride(2) == 1
        l.batch, l.M, l.K = a.shape
        l.N = b_nk.shape[1]
        l.lda, l.ldb, l.ldc = a.stride(1), b_nk.stride(1), out.stride(1)
        l.stride_a, l.stride_b, l.stride_c = a.stride(0), b_nk.stride(0), out.stride(0)
    else:
        assert a.stride(1) == 1 and b_nk.stride(1) == 1 and out.stride(1) == 1
        l.batch = 1
        l.M, l.K = a.shape
        l.N = b_nk.shape[0]
        l.lda, l.ldb, l.ldc = a.stride(0), b_nk.stride(0), out.stride(0)
    assert b_nk.shape[-1] == l.K and tuple(out.shape[-2:]) == (l.M, l.N)
    l.a, l.b, l.c = a.data_ptr(), b_nk.data_ptr(), out.data_ptr()
    l._refs = (a, b_nk, out)
    return _finish(l, cfg, ws)


def launch_gemv_f16(w, x, out, cfg=None, ws=None, out_transposed=False):
    """W[rows,K], X[m,K] (m <= 8) -> out[m,rows]; or out[rows,m] when ``out_transposed``."""
    _require_cuda(w, x, out)
    assert w.dtype == x.dtype == out.dtype == torch.float16
    assert w.stride(1) == 1 and x.stride(1) == 1
    l = Launch()
    l.op = OP_GEMV_F16
    l.N, l.K = w.shape
    l.M = x.shape[0]
    assert x.shape[1] == l.K
    l.lda, l.ldb = w.stride(0), x.stride(0)
    if out_transposed:
        assert tuple(out.shape) == (l.N, l.M)
        l.ldc, l.ldc_inner = out.stride(1), out.stride(0)
    else:
        assert tuple(out.shape) == (l.M, l.N)
        l.ldc, l.ldc_inner = out.stride(0), out.stride(1)
    l.a, l.b, l.c = w.data_ptr(), x.data_ptr(), out.data_ptr()
    l._refs = (w, x, out)
    return _finish(l, cfg, ws)


def launch_gemv_f32(w, x, out, cfg=None, ws=None, out_transposed=False):
    """W[rows,K], X[m,K] (m <= 8), fp32 -> out[m,rows]; or out[rows,m] when ``out_transposed``."""
    _require_cuda(w, x, out)
    assert w.dtype == x.dtype == out.dtype == torch.float32
    assert w.stride(1) == 1 and x.stride(1) == 1
    l = Launch()
    l.op = _lib.OP_GEMV_F32
    l.N, l.K = w.shape
    l.M = x.shape[0]
    assert x.shape[1] == l.K
    l.lda, l.ldb = w.stride(0), x.stride(0)
    if out_transposed:
        assert tuple(out.shape) == (l.N, l.M)
        l.ldc, l.ldc_inner = out.stride(1), out.stride(0)
    else:
        assert tuple(out.shape) == (l.M, l.N)
        l.ldc, l.ldc_inner = out.stride(0), out.stride(1)
    l.a, l.b, l.c = w.data_ptr(), x.data_ptr(), out.data_ptr()
    l._refs = (w, x, out)
    return _finish(l, cfg, ws)


def gemv_f32(w, x, out=None, cfg=None):
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=w.device)
    run(launch_gemv_f32(w, x, out, cfg))
    return out


def conv_out_hw(H, W, R, S, stride, pad):
    return (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1


def conv_stored_channels(IC, H, W, OC, kh, kw, stride, pad):
    """Channels an NHWC fp16 activation of IC logical channels is stored with (the rest are zeros).  Pixels are
    16 bytes or more (C a multiple of 8) for the tensor-map kernels; an input of up to 4 channels is stored as 4
    where the first-layer kernel covers the geometry (stride 2, filter up to 8 x 7, output rows of up to 128 pixels,
    64 or 128 output channels -- the conditions of conv_f16_stem_eligible in csrc/conv_f16_stem.cu)."""
    if IC <= 4 and stride == 2 and 2 <= kh <= 8 and pad < kh and W % 2 == 0 and OC in (64, 128):
        P = (pad + 1) & ~1
        Wo = (W + 2 * pad - kw) // 2 + 1
        Ho = (H + 2 * pad - kh) // 2 + 1
        if P - pad + kw <= 8 and 1 <= Wo <= 128 and Ho >= 1 and (P + W) * 8 <= 2176:
            return 4
    return (IC + 7) // 8 * 8


def conv_has_fixed_kernel(N, C, H, W, KO, R, S, stride, pad):
    """True where the library runs a convolution through a kernel without a tunable configuration (the 4-channel
    first-layer kernel, the 64 -> 64 channel row-pair kernel): nothing for a cost model to pick there."""
    if C == 4:
        return True
    l = Launch()
    l.op = OP_CONV_F16
    for i, v in enumerate((N, H, W, C, KO, R, S, stride, pad)):
        l.conv[i] = v
    return default_config(l).conv_gather == 4


def launch_conv2d_f16(x, w, out, stride, pad, cfg=None, ws=None):
    """x[N,H,W,C], w[KO,R,S,C] -> out[N,Ho,Wo,KO], all contiguous fp16."""
    _require_cuda(x, w, out)
    assert x.dtype == w.dtype == out.dtype == torch.float16
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    N, H, W, C = x.shape
    KO, R, S, C2 = w.shape
    assert C == C2
    Ho, Wo = conv_out_hw(H, W, R, S, stride, pad)
    assert tuple(out.shape) == (N, Ho, Wo, KO)
    l = Launch()
    l.op = OP_CONV_F16
    l.a, l.b, l.c = x.data_ptr(), w.data_ptr(), out.data_ptr()
    for i, v in enumerate((N, H, W, C, KO, R, S, stride, pad)):
        l.conv[i] = v
    l._refs = (x, w, out)
    return _finish(l, cfg, ws)


def launch_conv2d_f32(x, w, out, stride, pad, cfg=None, ws=None):
    """x[N,H,W,C], w[KO,R,S,C] -> out[N,Ho,Wo,KO], true fp32 (column matrix + FFMA GEMM in the workspace)."""
    _require_cuda(x, w, out)
    assert x.dtype == w.dtype == out.dtype == torch.float32
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    N, H, W, C = x.shape
    KO, R, S, C2 = w.shape
    assert C2 == C
    Ho, Wo = conv_out_hw(H, W, R, S, stride, pad)
    assert tuple(out.shape) == (N, Ho, Wo, KO)
    l = Launch()
    l.op = _lib.OP_CONV_F32
    for i, v in enumerate((N, H, W, C, KO, R, S, stride, pad)):
        l.conv[i] = v
    l.a, l.b, l.c = x.data_ptr(), w.data_ptr(), out.data_ptr()
    l._refs = (x, w, out)
    return _finish(l, cfg, ws)


def conv2d_f32_nhwc(x, w, stride=1, pad=0, out=None, cfg=None):
    N, H, W, _ = x.shape
    KO, R, S, _ = w.shape
    Ho, Wo = conv_out_hw(H, W, R, S, stride, pad)
    if out is None:
        out = torch.empty((N, Ho, Wo, KO), dtype=torch.float32, device=x.device)
    run(launch_conv2d_f32(x, w, out, stride, pad, cfg))
    return out


def launch_gemm_f32(a, b, out, trans_a=False, cfg=None):
    """A[M,K] (or [K,M] with trans_a) x B[K,N] -> out[M,N], fp32 FFMA."""
    _require_cuda(a, b, out)
    assert a.dtype == b.dtype == out.dtype == torch.float32
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    l = Launch()
    l.op = OP_GEMM_F32
    if trans_a:
        l.K, l.M = a.shape
    else:
        l.M, l.K = a.shape
    assert b.shape[0] == l.K
    l.N = b.shape[1]
    assert tuple(out.shape) == (l.M, l.N)
    l.lda, l.ldb, l.ldc = a.stride(0), b.stride(0), out.stride(0)
    l.trans_a = int(trans_a)
    l.a, l.b, l.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    l._refs = (a, b, out)
    return _finish(l, cfg, None)


def run(launch):
    """Queue a prepared launch on torch's current stream."""
    check(_lib.load().helix_launch(ctypes.byref(launch), ctypes.c_void_p(status_word().data_ptr()), _stream()),
          "helix_launch")


# ----------------------------------------------------------------------------- eager operators
def gemm_f16(a, b_nk, out=None, cfg=None):
    shape = (*a.shape[:-1], b_nk.shape[-2])
    if out is None:
        out = torch.empty(shape, dtype=torch.float16, device=a.device)
    run(launch_gemm_f16(a, b_nk, out, cfg))
    return out


def gemv_f16(w, x, out=None, cfg=None):
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float16, device=w.device)
    run(launch_gemv_f16(w, x, out, cfg))
    return out


def conv2d_f16_nhwc(x, w, stride=1, pad=0, out=None, cfg=None):
    if out is None:
        Ho, Wo = conv_out_hw(x.shape[1], x.shape[2], w.shape[1], w.shape[2], stride, pad)
        out = torch.empty((x.shape[0], Ho, Wo, w.shape[0]), dtype=torch.float16, device=x.device)
    run(launch_conv2d_f16(x, w, out, stride, pad, cfg))
    return out


def gemm_f32(a, b, trans_a=False, out=None, cfg=None):
    M = a.shape[1] if trans_a else a.shape[0]
    if out is None:
        out = torch.empty((M, b.shape[1]), dtype=torch.float32, device=a.device)
    run(launch_gemm_f32(a, b, out, trans_a, cfg))
    return out


# ----------------------------------------------------------------------------- timing
def time_launches(launches, warmup=3, iters=20, use_graph=False):
    """Seconds per launch (average), plus (min, max) seconds per round over the list.

    The list is walked round-robin, so passing launches over distinct operand
    buffers whose total footprint exceeds the L2 gives HBM-resident timings.
    """
    arr = (Launch * len(launches))()
    for i, l in enumerate(launches):
        ctypes.memmove(ctypes.byref(arr[i]), ctypes.byref(l), ctypes.sizeof(Launch))
    avg, mn, mx = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
    torch.cuda.synchronize()
    check(_lib.load().helix_time_launches(arr, len(launches), warmup, iters, int(use_graph),
                                          ctypes.byref(avg), ctypes.byref(mn), ctypes.byref(mx)),
          "helix_time_launches")
    return avg.value, mn.value, mx.value


def capture_timeline(launch, warm=2):
    """Run `launch` (a one-CTA fp16 GEMM / convolution) with timeline capture on and return an int64
    array [CTAs, words] of the stamps described at helix_trace_buffer; rows of CTAs that did not run
    stay zero."""
    lib = _lib.load()
    words = lib.helix_trace_words_per_cta()
    ctas = device_info().sm_count
    buf = torch.zeros((ctas, words), dtype=torch.int64, device="cuda")
    for _ in range(warm):
        run(launch)
    torch.cuda.synchronize()
    check(lib.helix_trace_buffer(buf.data_ptr(), buf.numel() * 8), "helix_trace_buffer")
    try:
        run(launch)
        torch.cuda.synchronize()
    finally:
        lib.helix_trace_buffer(None, 0)
    check_status()
    return buf.cpu().numpy()


def selftest_bounded_wait(limit_ns=2_000_000):
    """Launch the library's wait self-test on the current stream: a wait nothing satisfies gives up after
    `limit_ns` and leaves HELIX_ERR_TIMEOUT in the status word (read it with check_status)."""
    check(_lib.load().helix_selftest_bounded_wait(int(limit_ns), ctypes.c_void_p(status_word().data_ptr()), _stream()),
          "helix_selftest_bounded_wait")


def launch_count():
    return int(_lib.load().helix_launch_count())

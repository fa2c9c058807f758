// extern "C" layer of libhelix_b200.so: argument checking, per-device facts, dispatch to the
// kernel launchers, event timing and the host-buffer convenience entry points.
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace {

// One thread waits, with the bounded wait every kernel of the library uses, on a barrier that nothing will
// ever arrive at.  The wait gives up after `limit_ns`, records HELIX_ERR_TIMEOUT in the status word and the
// kernel returns normally: the path a stalled pipeline takes, exercised without stalling one.
__global__ void selftest_wait_kernel(unsigned long long limit_ns, int* status_dev) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    helix::mbar_init(&bar, 1);
    abort_flag = 0;
    helix::mbar_fence_init();
    (void)helix::mbar_wait_limit(&bar, 0, &abort_flag, status_dev, limit_ns);
  }
}

std::atomic<int64_t> g_launches{0};

struct DevCache {
  std::mutex mu;
  std::vector<helix_devinfo_t> info;
  std::vector<char> valid;
};
DevCache& dev_cache() {
  static DevCache c;
  return c;
}

int query_device(int dev, helix_devinfo_t* out) {
  DevCache& c = dev_cache();
  std::lock_guard<std::mutex> lock(c.mu);
  if (dev < 0) {
    if (cudaGetDevice(&dev) != cudaSuccess) return HELIX_ERR_NODEVICE;
  }
  if ((size_t)dev >= c.info.size()) {
    c.info.resize(dev + 1);
    c.valid.resize(dev + 1, 0);
  }
  if (!c.valid[dev]) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return HELIX_ERR_NODEVICE;
    helix_devinfo_t& d = c.info[dev];
    std::memset(&d, 0, sizeof(d));
    d.sm_count = prop.multiProcessorCount;
    d.cc_major = prop.major;
    d.cc_minor = prop.minor;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) == cudaSuccess) d.clock_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, dev) == cudaSuccess) d.mem_clock_khz = v;
    d.l2_bytes = prop.l2CacheSize;
    d.smem_per_sm = (int64_t)prop.sharedMemPerMultiprocessor;
    d.smem_per_block_optin = (int64_t)prop.sharedMemPerBlockOptin;
    d.total_mem = (int64_t)prop.totalGlobalMem;
    std::strncpy(d.name, prop.name, sizeof(d.name) - 1);
    c.valid[dev] = 1;
  }
  *out = c.info[dev];
  return HELIX_OK;
}

// Facts of the current device; tensor-core paths require compute capability 10.x.
int current_device(helix_devinfo_t* info, bool need_sm100) {
  const int rc = query_device(-1, info);
  if (rc != HELIX_OK) return rc;
  if (need_sm100 && info->cc_major != 10) return HELIX_ERR_NODEVICE;
  return HELIX_OK;
}

helix::ConvGeom conv_geom(const int* c) {
  helix::ConvGeom g;
  g.NB = c[0]; g.H = c[1]; g.W = c[2]; g.C = c[3]; g.KO = c[4]; g.R = c[5]; g.S = c[6]; g.stride = c[7]; g.pad = c[8];
  // a filter larger than the padded image has no valid window (C division would truncate towards zero
  // and report one)
  if (g.stride > 0 && g.H + 2 * g.pad >= g.R && g.W + 2 * g.pad >= g.S) {
    g.Ho = (g.H + 2 * g.pad - g.R) / g.stride + 1;
    g.Wo = (g.W + 2 * g.pad - g.S) / g.stride + 1;
  } else {
    g.Ho = g.Wo = 0;
  }
  return g;
}

int dispatch(const helix_launch_t* l, void* status_dev, cudaStream_t stream) {
  if (!l) return HELIX_ERR_INVALID;
  helix_devinfo_t info;
  int64_t n = 0;
  int rc;
  const helix_cfg_t* cfg = l->cfg.tile_m != 0 ? &l->cfg : nullptr;
  // max_ctas (read even from an otherwise zeroed cfg) limits the SMs a launch may spread over
  auto sms_of = [&](const helix_devinfo_t& di) {
    int s = di.sm_count;
    if (l->cfg.max_ctas > 0) s = std::max(2, std::min(s, l->cfg.max_ctas));
    return s;
  };
  switch (l->op) {
    case HELIX_OP_GEMM_F16:
      if ((rc = current_device(&info, true)) != HELIX_OK) return rc;
      rc = helix::gemm_f16_launch(cfg, l->a, l->lda, l->b, l->ldb, l->c, l->ldc, l->M, l->N, l->K, l->batch,
                                  l->stride_a, l->stride_b, l->stride_c, l->ws, l->ws_bytes,
                                  static_cast<int*>(status_dev), sms_of(info),
                                  (l->flags & HELIX_LAUNCH_INDEPENDENT) != 0, stream, &n);
      break;
    case HELIX_OP_GEMV_F16:
      if ((rc = current_device(&info, false)) != HELIX_OK) return rc;
      // Three or more right-hand sides: the SIMT kernel becomes issue bound (measured 11.7 us at
      // m = 4 and 22 us at m = 8 on 4096 x 4096) while the tcgen05 kernel streams the same weights
      // in 6.4 us with X as a 128-row A box of which only m rows are fetched.  Taken only for the
      // library's own configuration, the plain output layout and TMA-compatible operands.
      if (!cfg && l->M >= 3 && l->M <= 8 && info.cc_major == 10 && l->N >= 1024 && l->K >= 512 &&
          (l->ldc_inner == 0 || l->ldc_inner == 1) && (l->K % 8) == 0 &&
          ((l->lda == 0 ? l->K : l->lda) % 8) == 0 && ((l->ldb == 0 ? l->K : l->ldb) % 8) == 0 &&
          (reinterpret_cast<uintptr_t>(l->a) & 15) == 0 && (reinterpret_cast<uintptr_t>(l->b) & 15) == 0) {
        rc = helix::gemm_f16_launch(nullptr, l->b, l->ldb, l->a, l->lda, l->c, l->ldc == 0 ? l->N : l->ldc, l->M,
                                    l->N, l->K, 1, 0, 0, 0, nullptr, 0, static_cast<int*>(status_dev),
                                    sms_of(info), (l->flags & HELIX_LAUNCH_INDEPENDENT) != 0, stream, &n);
        break;
      }
      rc = helix::gemv_f16_launch(cfg, l->a, l->lda, l->b, l->ldb, l->c, l->ldc, l->ldc_inner, l->N, l->K, l->M,
                                  l->ws, l->ws_bytes, sms_of(info),
                                  (l->flags & HELIX_LAUNCH_INDEPENDENT) ? 2 : (l->flags & HELIX_LAUNCH_STATIC_A) ? 1 : 0,
                                  stream, &n);
      break;
    case HELIX_OP_CONV_F16: {
      if ((rc = current_device(&info, true)) != HELIX_OK) return rc;
      const helix::ConvGeom g = conv_geom(l->conv);
      rc = helix::conv_f16_launch(cfg, l->a, l->b, l->c, g, l->ws, l->ws_bytes, static_cast<int*>(status_dev),
                                  sms_of(info), (l->flags & HELIX_LAUNCH_INDEPENDENT) != 0, stream, &n);
      break;
    }
    case HELIX_OP_GEMM_F32:
      if ((rc = current_device(&info, false)) != HELIX_OK) return rc;
      rc = helix::sgemm_f32_launch(cfg, static_cast<const float*>(l->a), l->lda, l->trans_a,
                                   static_cast<const float*>(l->b), l->ldb, static_cast<float*>(l->c), l->ldc, l->M,
                                   l->N, l->K, sms_of(info), stream, &n);
      break;
    case HELIX_OP_GEMV_F32:
      if ((rc = current_device(&info, false)) != HELIX_OK) return rc;
      rc = helix::gemv_f32_launch(cfg, static_cast<const float*>(l->a), l->lda, static_cast<const float*>(l->b), l->ldb,
                                  static_cast<float*>(l->c), l->ldc, l->ldc_inner, l->N, l->K, l->M, l->ws,
                                  l->ws_bytes, sms_of(info), stream, &n);
      break;
    case HELIX_OP_CONV_F32: {
      if ((rc = current_device(&info, false)) != HELIX_OK) return rc;
      const helix::ConvGeom g = conv_geom(l->conv);
      rc = helix::conv_f32_launch(cfg, static_cast<const float*>(l->a), static_cast<const float*>(l->b),
                                  static_cast<float*>(l->c), g, l->ws, l->ws_bytes, sms_of(info), stream, &n);
      break;
    }
    default:
      return HELIX_ERR_INVALID;
  }
  g_launches += n;
  return rc;
}

struct DeviceBuffer {
  void* p = nullptr;
  ~DeviceBuffer() {
    if (p) cudaFree(p);
  }
  int alloc(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 1) == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA; }
};

}  // namespace

extern "C" {

int helix_version(void) { return 100; }

const char* helix_status_string(int status) {
  switch (status) {
    case HELIX_OK: return "ok";
    case HELIX_ERR_INVALID: return "invalid argument";
    case HELIX_ERR_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case HELIX_ERR_WORKSPACE: return "workspace missing or too small";
    case HELIX_ERR_CUDA: return "CUDA call failed";
    case HELIX_ERR_TIMEOUT: return "bounded device-side wait ran out";
    case HELIX_ERR_UNSUPPORTED: return "configuration not built into the library";
    case HELIX_ERR_NODEVICE: return "no sm_100 device is current";
    case HELIX_ERR_CAPACITY: return "problem exceeds the capacity of a fixed built-in buffer";
    default: return "unknown status";
  }
}

int helix_device_info(int dev, helix_devinfo_t* out) {
  if (!out) return HELIX_ERR_INVALID;
  return query_device(dev, out);
}

int helix_num_configs(int op) {
  switch (op) {
    case HELIX_OP_GEMM_F16:
    case HELIX_OP_CONV_F16: return helix::gemm_f16_num_configs();
    case HELIX_OP_GEMV_F16:
    case HELIX_OP_GEMV_F32: return 5;  // split-K 1, 2, 4, 8, 16
    case HELIX_OP_GEMM_F32:
    case HELIX_OP_CONV_F32: return helix::sgemm_f32_num_configs();
    default: return HELIX_ERR_INVALID;
  }
}

int helix_get_config(int op, int idx, helix_cfg_t* out) {
  if (!out) return HELIX_ERR_INVALID;
  const int n = helix_num_configs(op);
  if (n < 0) return n;
  if (idx < 0 || idx >= n) return HELIX_ERR_INVALID;
  std::memset(out, 0, sizeof(*out));
  switch (op) {
    case HELIX_OP_GEMM_F16:
      helix::gemm_f16_get_config(idx, out);
      break;
    case HELIX_OP_CONV_F16:
      helix::gemm_f16_get_config(idx, out);
      out->op = HELIX_OP_CONV_F16;
      if (out->swap_ab || out->cta_group != 1) return HELIX_ERR_UNSUPPORTED;
      break;
    case HELIX_OP_GEMV_F16:
    case HELIX_OP_GEMV_F32:
      out->op = op;
      out->tile_m = 1;
      out->tile_n = 2;
      out->tile_k = op == HELIX_OP_GEMV_F16 ? 256 : 128;
      out->split_k = 1 << idx;
      out->cta_group = 1;
      break;
    case HELIX_OP_GEMM_F32:
    case HELIX_OP_CONV_F32:
      helix::sgemm_f32_get_config(idx, out);     // a convolution runs the GEMM's configurations
      out->op = op;
      break;
  }
  return HELIX_OK;
}

int helix_default_config(const helix_launch_t* l, helix_cfg_t* out) {
  if (!l || !out) return HELIX_ERR_INVALID;
  helix_devinfo_t info;
  int sms = (query_device(-1, &info) == HELIX_OK) ? info.sm_count : 148;
  if (l->cfg.max_ctas > 0) sms = std::max(2, std::min(sms, l->cfg.max_ctas));
  std::memset(out, 0, sizeof(*out));
  switch (l->op) {
    case HELIX_OP_GEMM_F16:
      helix::gemm_f16_default_config(l->M, l->N, l->K, l->batch > 0 ? l->batch : 1, sms, false, out);
      return HELIX_OK;
    case HELIX_OP_CONV_F16: {
      const helix::ConvGeom g = conv_geom(l->conv);
      const int64_t M = (int64_t)g.NB * g.Ho * g.Wo, K = (int64_t)g.R * g.S * g.C;
      if (M <= 0 || M > 0x7fffffff || K <= 0 || K > 0x7fffffff) return HELIX_ERR_INVALID;
      helix::conv_f16_default_config(g, sms, out);
      return HELIX_OK;
    }
    case HELIX_OP_GEMV_F16:
      out->op = HELIX_OP_GEMV_F16;
      out->tile_m = 1; out->tile_n = 2; out->tile_k = 256; out->cta_group = 1;
      out->split_k = helix::gemv_f16_default_split(l->N, l->K, sms);
      return HELIX_OK;
    case HELIX_OP_GEMV_F32:
      out->op = HELIX_OP_GEMV_F32;
      out->tile_m = 1; out->tile_n = l->M <= 2 ? 2 : 1; out->tile_k = 128; out->cta_group = 1;
      out->load_group = l->M <= 4 ? 4 : 2;
      out->split_k = helix::gemv_f32_default_split(l->N, l->K, sms);
      return HELIX_OK;
    case HELIX_OP_GEMM_F32:
      helix::sgemm_f32_default_config(l->M, l->N, sms, out);
      return HELIX_OK;
    case HELIX_OP_CONV_F32: {
      const helix::ConvGeom g = conv_geom(l->conv);
      const int64_t M = (int64_t)g.NB * g.Ho * g.Wo;
      if (M <= 0 || M > 0x7fffffff || g.KO <= 0) return HELIX_ERR_INVALID;
      helix::sgemm_f32_default_config((int)M, g.KO, sms, out);
      out->op = HELIX_OP_CONV_F32;
      return HELIX_OK;
    }
    default:
      return HELIX_ERR_INVALID;
  }
}

size_t helix_workspace_bytes(const helix_launch_t* l) {
  if (!l) return 0;
  helix_devinfo_t info;
  int sms = (query_device(-1, &info) == HELIX_OK) ? info.sm_count : 148;
  if (l->cfg.max_ctas > 0) sms = std::max(2, std::min(sms, l->cfg.max_ctas));
  const bool have_cfg = l->cfg.tile_m != 0;
  switch (l->op) {
    case HELIX_OP_GEMM_F16: {
      helix_cfg_t cfg = l->cfg;
      if (!have_cfg) helix::gemm_f16_default_config(l->M, l->N, l->K, l->batch > 0 ? l->batch : 1, sms, false, &cfg);
      return helix::gemm_f16_workspace_bytes(&cfg, l->M, l->N, l->K, l->batch > 0 ? l->batch : 1, sms);
    }
    case HELIX_OP_CONV_F16: {
      const helix::ConvGeom g = conv_geom(l->conv);
      const int64_t M = (int64_t)g.NB * g.Ho * g.Wo, K = (int64_t)g.R * g.S * g.C;
      if (M <= 0 || M > 0x7fffffff || K > 0x7fffffff) return 0;
      if (g.C == 4) return 0;   // the four-channel first-layer kernel keeps everything on chip
      helix_cfg_t cfg = l->cfg;
      if (!have_cfg) helix::conv_f16_default_config(g, sms, &cfg);
      return helix::gemm_f16_workspace_bytes(&cfg, (int)M, g.KO, (int)K, 1, sms);
    }
    case HELIX_OP_GEMV_F16: {
      const int split = have_cfg && l->cfg.split_k > 0 ? l->cfg.split_k : helix::gemv_f16_default_split(l->N, l->K, sms);
      return helix::gemv_f16_workspace_bytes(l->N, l->M, split);
    }
    case HELIX_OP_GEMV_F32: {
      const int split = have_cfg && l->cfg.split_k > 0 ? l->cfg.split_k : helix::gemv_f32_default_split(l->N, l->K, sms);
      return helix::gemv_f32_workspace_bytes(l->N, l->M, split);
    }
    case HELIX_OP_CONV_F32:
      return helix::conv_f32_workspace_bytes(conv_geom(l->conv));
    default:
      return 0;
  }
}

int helix_launch(const helix_launch_t* launch, void* status_dev, void* stream) {
  return dispatch(launch, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_gemm_f16(const helix_cfg_t* cfg, const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                   int64_t ldc, int M, int N, int K, int batch, int64_t stride_a, int64_t stride_b,
                   int64_t stride_c, void* ws, size_t ws_bytes, void* status_dev, void* stream) {
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_GEMM_F16;
  if (cfg) l.cfg = *cfg;
  l.a = A; l.b = B; l.c = C;
  l.lda = lda; l.ldb = ldb; l.ldc = ldc;
  l.M = M; l.N = N; l.K = K;
  l.batch = batch;
  l.stride_a = stride_a; l.stride_b = stride_b; l.stride_c = stride_c;
  l.ws = ws; l.ws_bytes = ws_bytes;
  return dispatch(&l, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_gemv_f16(const helix_cfg_t* cfg, const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y,
                   int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes,
                   void* status_dev, void* stream) {
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_GEMV_F16;
  if (cfg) l.cfg = *cfg;
  l.a = W; l.b = X; l.c = Y;
  l.lda = ldw; l.ldb = ldx; l.ldc = ldy; l.ldc_inner = ldy_inner;
  l.M = m; l.N = rows; l.K = K;
  l.ws = ws; l.ws_bytes = ws_bytes;
  return dispatch(&l, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_gemv_f32(const helix_cfg_t* cfg, const float* W, int64_t ldw, const float* X, int64_t ldx, float* Y,
                   int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes,
                   void* status_dev, void* stream) {
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_GEMV_F32;
  if (cfg) l.cfg = *cfg;
  l.a = W; l.b = X; l.c = Y;
  l.lda = ldw; l.ldb = ldx; l.ldc = ldy; l.ldc_inner = ldy_inner;
  l.M = m; l.N = rows; l.K = K;
  l.ws = ws; l.ws_bytes = ws_bytes;
  return dispatch(&l, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_conv2d_f16_nhwc(const helix_cfg_t* cfg, const void* x, const void* w, void* y, int N, int H, int W, int C,
                          int KO, int R, int S, int stride, int pad, void* ws, size_t ws_bytes, void* status_dev,
                          void* stream) {
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_CONV_F16;
  if (cfg) l.cfg = *cfg;
  l.a = x; l.b = w; l.c = y;
  const int c9[9] = {N, H, W, C, KO, R, S, stride, pad};
  std::memcpy(l.conv, c9, sizeof(c9));
  l.ws = ws; l.ws_bytes = ws_bytes;
  return dispatch(&l, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_gemm_f32(const helix_cfg_t* cfg, const float* A, int64_t lda, int trans_a, const float* B, int64_t ldb,
                   float* C, int64_t ldc, int M, int N, int K, void* status_dev, void* stream) {
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_GEMM_F32;
  if (cfg) l.cfg = *cfg;
  l.a = A; l.b = B; l.c = C;
  l.lda = lda; l.ldb = ldb; l.ldc = ldc;
  l.M = M; l.N = N; l.K = K;
  l.trans_a = trans_a;
  return dispatch(&l, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_conv2d_f32_nhwc(const helix_cfg_t* cfg, const float* x, const float* w, float* y, int N, int H, int W, int C,
                          int KO, int R, int S, int stride, int pad, void* ws, size_t ws_bytes, void* status_dev,
                          void* stream) {
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_CONV_F32;
  if (cfg) l.cfg = *cfg;
  l.a = x; l.b = w; l.c = y;
  const int geom[9] = {N, H, W, C, KO, R, S, stride, pad};
  std::memcpy(l.conv, geom, sizeof(geom));
  l.ws = ws;
  l.ws_bytes = ws_bytes;
  return dispatch(&l, status_dev, static_cast<cudaStream_t>(stream));
}

int helix_time_launches(const helix_launch_t* list, int count, int warmup, int iters, int use_graph, double* avg_s,
                        double* min_round_s, double* max_round_s) {
  if (!list || count <= 0 || iters <= 0 || warmup < 0) return HELIX_ERR_INVALID;
  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int rc = HELIX_OK;
  int* status_dev = nullptr;
  auto round = [&]() -> int {
    for (int i = 0; i < count; ++i) {
      const int r = dispatch(&list[i], status_dev, stream);
      if (r != HELIX_OK) return r;
    }
    return HELIX_OK;
  };
  do {
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    if (cudaMalloc(&status_dev, sizeof(int)) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    cudaMemsetAsync(status_dev, 0, sizeof(int), stream);
    if ((rc = round()) != HELIX_OK) break;  // first round outside any capture: sets function attributes
    if (cudaStreamSynchronize(stream) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    if (use_graph) {
      if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
      const int r = round();
      const cudaError_t ce = cudaStreamEndCapture(stream, &graph);
      if (r != HELIX_OK) { rc = r; break; }
      if (ce != cudaSuccess || !graph) { rc = HELIX_ERR_CUDA; break; }
      if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    }
    auto run_round = [&]() -> int {
      if (exec) return cudaGraphLaunch(exec, stream) == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
      return round();
    };
    for (int w = 0; w < warmup && rc == HELIX_OK; ++w) rc = run_round();
    if (rc != HELIX_OK) break;
    if (cudaStreamSynchronize(stream) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    // whole timed region between one pair of events; per-round extremes from a second pass
    cudaEventRecord(e0, stream);
    for (int it = 0; it < iters && rc == HELIX_OK; ++it) rc = run_round();
    cudaEventRecord(e1, stream);
    if (rc != HELIX_OK) break;
    if (cudaEventSynchronize(e1) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (avg_s) *avg_s = (double)ms * 1e-3 / ((double)iters * count);
    if (min_round_s || max_round_s) {
      double mn = 1e30, mx = 0.0;
      const int reps = iters < 5 ? iters : 5;
      for (int it = 0; it < reps && rc == HELIX_OK; ++it) {
        cudaEventRecord(e0, stream);
        rc = run_round();
        cudaEventRecord(e1, stream);
        if (cudaEventSynchronize(e1) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
        cudaEventElapsedTime(&ms, e0, e1);
        const double s = (double)ms * 1e-3;
        if (s < mn) mn = s;
        if (s > mx) mx = s;
      }
      if (min_round_s) *min_round_s = mn;
      if (max_round_s) *max_round_s = mx;
    }
    int st = 0;
    if (cudaMemcpy(&st, status_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) { rc = HELIX_ERR_CUDA; break; }
    if (st != 0) rc = st;
  } while (false);
  if (exec) cudaGraphExecDestroy(exec);
  if (graph) cudaGraphDestroy(graph);
  if (status_dev) cudaFree(status_dev);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (stream) cudaStreamDestroy(stream);
  return rc;
}

// ---------------------------------------------------------------- host-buffer wrappers
static int finish_host(int rc, int* status_dev) {
  if (rc != HELIX_OK) return rc;
  if (cudaDeviceSynchronize() != cudaSuccess) return HELIX_ERR_CUDA;
  int st = 0;
  if (cudaMemcpy(&st, status_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return HELIX_ERR_CUDA;
  return st;
}

int helix_gemm_f16_host(const void* A, const void* B, void* C, int M, int N, int K) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return HELIX_ERR_INVALID;
  // leading dimensions padded to 8 halves so any K is accepted
  const int64_t ldk = ((int64_t)K + 7) / 8 * 8;
  DeviceBuffer dA, dB, dC, dS, dW;
  if (dA.alloc((size_t)M * ldk * 2) || dB.alloc((size_t)N * ldk * 2) || dC.alloc((size_t)M * N * 2) || dS.alloc(4))
    return HELIX_ERR_CUDA;
  cudaMemset(dS.p, 0, 4);
  if (ldk != K) { cudaMemset(dA.p, 0, (size_t)M * ldk * 2); cudaMemset(dB.p, 0, (size_t)N * ldk * 2); }
  if (cudaMemcpy2D(dA.p, ldk * 2, A, (size_t)K * 2, (size_t)K * 2, M, cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy2D(dB.p, ldk * 2, B, (size_t)K * 2, (size_t)K * 2, N, cudaMemcpyHostToDevice) != cudaSuccess)
    return HELIX_ERR_CUDA;
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_GEMM_F16;
  l.a = dA.p; l.b = dB.p; l.c = dC.p;
  l.lda = ldk; l.ldb = ldk; l.ldc = N;
  l.M = M; l.N = N; l.K = (int)ldk; l.batch = 1;
  const size_t ws = helix_workspace_bytes(&l);
  if (ws) { if (dW.alloc(ws)) return HELIX_ERR_CUDA; l.ws = dW.p; l.ws_bytes = ws; }
  int rc = finish_host(dispatch(&l, dS.p, nullptr), static_cast<int*>(dS.p));
  if (rc != HELIX_OK) return rc;
  return cudaMemcpy(C, dC.p, (size_t)M * N * 2, cudaMemcpyDeviceToHost) == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

int helix_gemv_f16_host(const void* W, const void* X, void* Y, int rows, int K, int m) {
  if (!W || !X || !Y || rows <= 0 || K <= 0 || m <= 0 || m > 8) return HELIX_ERR_INVALID;
  const int64_t ldk = ((int64_t)K + 7) / 8 * 8;
  DeviceBuffer dW, dX, dY, dS, dWs;
  if (dW.alloc((size_t)rows * ldk * 2) || dX.alloc((size_t)m * ldk * 2) || dY.alloc((size_t)m * rows * 2) || dS.alloc(4))
    return HELIX_ERR_CUDA;
  cudaMemset(dS.p, 0, 4);
  if (ldk != K) { cudaMemset(dW.p, 0, (size_t)rows * ldk * 2); cudaMemset(dX.p, 0, (size_t)m * ldk * 2); }
  if (cudaMemcpy2D(dW.p, ldk * 2, W, (size_t)K * 2, (size_t)K * 2, rows, cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy2D(dX.p, ldk * 2, X, (size_t)K * 2, (size_t)K * 2, m, cudaMemcpyHostToDevice) != cudaSuccess)
    return HELIX_ERR_CUDA;
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_GEMV_F16;
  l.a = dW.p; l.b = dX.p; l.c = dY.p;
  l.lda = ldk; l.ldb = ldk; l.ldc = rows; l.ldc_inner = 1;
  l.M = m; l.N = rows; l.K = (int)ldk;
  const size_t ws = helix_workspace_bytes(&l);
  if (ws) { if (dWs.alloc(ws)) return HELIX_ERR_CUDA; l.ws = dWs.p; l.ws_bytes = ws; }
  int rc = finish_host(dispatch(&l, dS.p, nullptr), static_cast<int*>(dS.p));
  if (rc != HELIX_OK) return rc;
  return cudaMemcpy(Y, dY.p, (size_t)m * rows * 2, cudaMemcpyDeviceToHost) == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

int helix_gemm_f32_host(const float* A, const float* B, float* C, int M, int N, int K) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K < 0) return HELIX_ERR_INVALID;
  DeviceBuffer dA, dB, dC, dS;
  if (dA.alloc((size_t)M * K * 4) || dB.alloc((size_t)K * N * 4) || dC.alloc((size_t)M * N * 4) || dS.alloc(4))
    return HELIX_ERR_CUDA;
  cudaMemset(dS.p, 0, 4);
  if (cudaMemcpy(dA.p, A, (size_t)M * K * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(dB.p, B, (size_t)K * N * 4, cudaMemcpyHostToDevice) != cudaSuccess)
    return HELIX_ERR_CUDA;
  int rc = helix_gemm_f32(nullptr, static_cast<float*>(dA.p), K, 0, static_cast<float*>(dB.p), N,
                          static_cast<float*>(dC.p), N, M, N, K, dS.p, nullptr);
  rc = finish_host(rc, static_cast<int*>(dS.p));
  if (rc != HELIX_OK) return rc;
  return cudaMemcpy(C, dC.p, (size_t)M * N * 4, cudaMemcpyDeviceToHost) == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

int helix_conv2d_f16_nhwc_host(const void* x, const void* w, void* y, int N, int H, int W, int C, int KO, int R,
                               int S, int stride, int pad) {
  if (!x || !w || !y || stride <= 0) return HELIX_ERR_INVALID;
  const int c9[9] = {N, H, W, C, KO, R, S, stride, pad};
  const helix::ConvGeom g = conv_geom(c9);
  if (g.Ho <= 0 || g.Wo <= 0) return HELIX_ERR_INVALID;
  const size_t xb = (size_t)N * H * W * C * 2, wb = (size_t)KO * R * S * C * 2, yb = (size_t)N * g.Ho * g.Wo * KO * 2;
  DeviceBuffer dx, dw, dy, dS, dWs;
  if (dx.alloc(xb) || dw.alloc(wb) || dy.alloc(yb) || dS.alloc(4)) return HELIX_ERR_CUDA;
  cudaMemset(dS.p, 0, 4);
  if (cudaMemcpy(dx.p, x, xb, cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(dw.p, w, wb, cudaMemcpyHostToDevice) != cudaSuccess)
    return HELIX_ERR_CUDA;
  helix_launch_t l;
  std::memset(&l, 0, sizeof(l));
  l.op = HELIX_OP_CONV_F16;
  l.a = dx.p; l.b = dw.p; l.c = dy.p;
  std::memcpy(l.conv, c9, sizeof(c9));
  const size_t ws = helix_workspace_bytes(&l);
  if (ws) { if (dWs.alloc(ws)) return HELIX_ERR_CUDA; l.ws = dWs.p; l.ws_bytes = ws; }
  int rc = finish_host(dispatch(&l, dS.p, nullptr), static_cast<int*>(dS.p));
  if (rc != HELIX_OK) return rc;
  return cudaMemcpy(y, dy.p, yb, cudaMemcpyDeviceToHost) == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

int helix_gemv_f16_static(const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y, int64_t ldy,
                          int64_t ldy_inner, int rows, int K, int m, int split_k, void* stream) {
  helix_devinfo_t info;
  const int rc = current_device(&info, false);
  if (rc != HELIX_OK) return rc;
  int64_t n = 0;
  const int st = helix::gemv_f16_static_launch(W, ldw, X, ldx, Y, ldy, ldy_inner, rows, K, m, split_k,
                                               info.sm_count, static_cast<cudaStream_t>(stream), &n);
  g_launches += n;
  return st;
}

int helix_selftest_bounded_wait(uint64_t limit_ns, void* status_dev, void* stream) {
  if (!status_dev || limit_ns == 0 || limit_ns > 1000000000ull) return HELIX_ERR_INVALID;
  helix_devinfo_t info;
  const int rc = current_device(&info, false);
  if (rc != HELIX_OK) return rc;
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, static_cast<int*>(status_dev));
  g_launches += 1;
  return cudaGetLastError() == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

int64_t helix_launch_count(void) { return g_launches.load(); }

int helix_trace_buffer(void* device_buf, size_t bytes) {
  helix::gemm_f16_set_trace(device_buf, bytes);
  return HELIX_OK;
}

int helix_trace_words_per_cta(void) { return helix::gemm_f16_trace_words_per_cta(); }

}  // extern "C"

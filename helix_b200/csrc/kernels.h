// Internal launch interfaces between the kernel translation units and the C ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/helix_b200.h"

namespace helix {

// ---- gemv_f16.cu
size_t gemv_f16_workspace_bytes(int rows, int m, int split_k);
int gemv_f16_default_split(int rows, int K, int sm_count);
int gemv_f16_launch(const helix_cfg_t* cfg, const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y,
                    int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes,
                    int sm_count, int order_mode, cudaStream_t stream, int64_t* launches);

// Variant with the split-K partials in an array that is part of the library image.
size_t gemv_f16_static_capacity_floats();
int gemv_f16_static_launch(const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y, int64_t ldy,
                           int64_t ldy_inner, int rows, int K, int m, int split_k, int sm_count,
                           cudaStream_t stream, int64_t* launches);

// ---- gemv_f32.cu (true-fp32 GEMV)
size_t gemv_f32_workspace_bytes(int rows, int m, int split_k);
int gemv_f32_default_split(int rows, int K, int sm_count);
int gemv_f32_launch(const helix_cfg_t* cfg, const float* W, int64_t ldw, const float* X, int64_t ldx, float* Y,
                    int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes, int sm_count,
                    cudaStream_t stream, int64_t* launches);


// ---- sgemm_f32.cu
int sgemm_f32_num_configs();
void sgemm_f32_get_config(int idx, helix_cfg_t* out);
void sgemm_f32_default_config(int M, int N, int sm_count, helix_cfg_t* out);
int sgemm_f32_launch(const helix_cfg_t* cfg, const float* A, int64_t lda, int trans_a, const float* B, int64_t ldb,
                     float* C, int64_t ldc, int M, int N, int K, int sm_count, cudaStream_t stream,
                     int64_t* launches);

// ---- gemm_f16_tc.cu (tcgen05 GEMM and implicit-GEMM convolution)
struct ConvGeom {
  int NB, H, W, C, KO, R, S, stride, pad, Ho, Wo;
};
int gemm_f16_num_configs();
void gemm_f16_get_config(int idx, helix_cfg_t* out);
// Fills *out with the library's default choice for the problem.
void gemm_f16_default_config(int M, int N, int K, int batch, int sm_count, bool conv, helix_cfg_t* out);
void conv_f16_default_config(const ConvGeom& g, int sm_count, helix_cfg_t* out);
// ---- conv_f32.cu (column matrix + FFMA GEMM)
size_t conv_f32_workspace_bytes(const ConvGeom& g);
int conv_f32_launch(const helix_cfg_t* cfg, const float* x, const float* w, float* y, const ConvGeom& g, void* ws,
                    size_t ws_bytes, int sm_count, cudaStream_t stream, int64_t* launches);
// Per-CTA timeline capture shared by the one-CTA and the CTA-pair kernel (layout: helix_b200.h).
constexpr int kTraceTiles = 20;   // work items with six stamps each
constexpr int kTraceSlabs = 32;   // first K slabs of the CTA: request issued, data consumed
constexpr int kTraceWords = 8 + 6 * kTraceTiles + 2 * kTraceSlabs;
void gemm_f16_set_trace(void* device_buf, size_t bytes);
int gemm_f16_trace_words_per_cta();
unsigned long long* gemm_f16_trace_for_grid(int grid);   // the capture buffer if one is set and large enough
size_t gemm_f16_workspace_bytes(const helix_cfg_t* cfg, int M, int N, int K, int batch, int sm_count);
int gemm_f16_launch(const helix_cfg_t* cfg, const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                    int64_t ldc, int M, int N, int K, int batch, int64_t sa, int64_t sb, int64_t sc, void* ws,
                    size_t ws_bytes, int* status_dev, int sm_count, bool independent, cudaStream_t stream,
                    int64_t* launches);
// ---- gemm_f16_tc2.cu (CTA pairs, tcgen05.mma.cta_group::2)
int gemm_f16_pair_max_stages(int bn);
size_t gemm_f16_pair_workspace_bytes(const helix_cfg_t& cfg, int M, int N, int K, int batch, int sm_count);
int gemm_f16_pair_launch(const helix_cfg_t& cfg, const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                         int64_t ldc, int M, int N, int K, int batch, int64_t sa, int64_t sb, int64_t sc, void* ws,
                         size_t ws_bytes, int* status_dev, int sm_count, bool independent, cudaStream_t stream,
                         int64_t* launches);
// ---- conv_f16_halo.cu (stride-1 convolution with the input window resident in shared memory)
bool conv_f16_halo_eligible(const ConvGeom& g, const helix_cfg_t* cfg);
double conv_f16_halo_estimate_us(const ConvGeom& g, int sm_count);   // < 0: geometry not covered
int conv_f16_halo_launch(const helix_cfg_t* cfg, const void* x, const void* w, void* y, const ConvGeom& g,
                         int* status_dev, int sm_count, bool independent, cudaStream_t stream, int64_t* launches);
// ---- conv_f16_stem.cu (stride-2 convolution over 4 stored channels, input rows resident in shared memory)
bool conv_f16_stem_eligible(const ConvGeom& g);
int conv_f16_stem_launch(const void* x, const void* w, void* y, const ConvGeom& g, int probe, int* status_dev,
                         int sm_count, bool independent, cudaStream_t stream, int64_t* launches);
// ---- conv_f16_rows.cu (3 x 3 / 1, 64 -> 64 channels: pixels on the accumulator rows, window and weights resident)
bool conv_f16_rows_eligible(const ConvGeom& g, int sm_count, bool worth_it);
int conv_f16_rows_launch(const void* x, const void* w, void* y, const ConvGeom& g, int probe, int* status_dev,
                         int sm_count, bool independent, cudaStream_t stream, int64_t* launches);
int conv_f16_launch(const helix_cfg_t* cfg, const void* x, const void* w, void* y, const ConvGeom& g, void* ws,
                    size_t ws_bytes, int* status_dev, int sm_count, bool independent, cudaStream_t stream,
                    int64_t* launches);

}  // namespace helix

// Internal launch functions shared by the translation units of libsq_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/sq_b200.h"

namespace sq {

// Optional work fused in front of the quantizer: normalisation over the row, AdaLN modulation, rounding.
struct PrepassFusion {
  int input_activation = SQ_ACT_FN_NONE;  // applied to x first, result rounded to x's dtype (a module boundary)
  int norm_kind = SQ_NORM_NONE;      // SQ_NORM_NONE / SQ_NORM_LAYER (no affine) / SQ_NORM_RMS
  float norm_eps = 0.0f;
  const void* norm_weight = nullptr; // [K] in x's dtype, or null (RMS only)
  const void* mod_scale = nullptr;   // AdaLN: y = (1 + scale) * y + shift; rows of K in x's dtype
  const void* mod_shift = nullptr;
  int64_t mod_span = 1;              // input rows per modulation row
  int64_t mod_row_stride = 0;        // elements between modulation rows
  int round_after = 0;               // round the result to x's dtype before rotation / quantization
  // static mode: read the schedule entry from device memory; act_scale / gains passed to launch_prepass are
  // then the bases of the [calls] and [calls, streams] tables
  const int32_t* call_index = nullptr;
  int64_t calls = 0;
  // 256 ints (1024 bytes) thread block 0 clears before anything else: the K-split counters of the GEMM behind it
  int* clear_words = nullptr;
  // composite rotation: K = mix_order x (power of two); replaces the block rotation, excludes the fusions above
  const float* mix = nullptr;        // [mix_order, mix_order] of +-1
  int mix_order = 0;
};

int launch_prepass(const void* x, int x_dtype, int64_t rows, int64_t K, int abits, int mode, const float* inv_d,
                   const float* signs, int rht_block, const float* act_scale, const float* gains, int64_t span,
                   int64_t streams, int64_t seq_tokens, int codes_layout, int pack_int4, void* codes,
                   float* row_scales, cudaStream_t stream, const PrepassFusion* fusion = nullptr);

struct GemmArgs {
  const int8_t* codes;
  int codes_layout;
  const uint8_t* w_packed;
  const void* w_scales;
  int wscale_mode;
  const float* row_scales;
  const void* bias;
  void* out;
  int out_dtype;
  int64_t M, N, K;
  int32_t* acc_dump;
  bool after_prepass = false;  // launched right behind the pre-pass that writes codes / row_scales: overlap the prologue
  bool weights_prepacked = false;  // SQ_WEIGHTS_PREPACKED: w_packed is int8 [N, K] from sq_prepack_weights
  bool codes_int4_range = false;  // SQ_CODES_INT4_RANGE was set: every code lies in [-8, 7]
  // fused epilogue: out = residual + gate * act(acc * scales + bias)
  int activation = SQ_ACT_FN_NONE;
  const void* gate = nullptr;      // rows of N in out's dtype, one per gate_span output rows
  int64_t gate_span = 1;
  int64_t gate_row_stride = 0;     // elements between gate rows
  const void* residual = nullptr;  // [M, N] in out's dtype
  // scratch for tiles that are split along K (see sq_gemm_ts.cu); null: whole tiles only
  void* split_workspace = nullptr;
  size_t split_workspace_bytes = 0;
  bool split_counters_cleared = false;  // the caller already put a memset of the first 1024 bytes on the stream
  // Channel-split form (sq_gemm_scatter): this GPU holds N of the layer's output channels and writes its [M, N]
  // block into columns [out_col0, out_col0 + N) of row-major [M, out_ld] matrices, `out` and up to 7 more - the
  // same matrix on the other GPUs of the split, reached through peer pointers: the all-gather is the epilogue's
  // own stores over NVLink.  out_ld == 0: a plain [M, N] output.
  int64_t out_ld = 0;
  int64_t out_col0 = 0;
  int n_more_outs = 0;
  void* more_outs[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};

int validate_gemm(const GemmArgs& a);
int launch_prepack_weights(const uint8_t* w_packed, int64_t N, int64_t K, int8_t* w_tiled, cudaStream_t stream);
int launch_gemm_tc(const GemmArgs& a, cudaStream_t stream);
// Second-generation kernel (weights in tensor memory, K-split scheduling); packed int4 weights only.
int launch_gemm_ts(const GemmArgs& a, cudaStream_t stream);
int launch_gemm_ts_timeline(const GemmArgs& a, long long* timeline, cudaStream_t stream);
size_t gemm_split_workspace_bytes(int64_t M);
// Picks the kernel: sq_gemm_tc.cu unless SQ_GEMM_KERNEL=ts is set (and the weights are not prepacked).
int launch_gemm(const GemmArgs& a, cudaStream_t stream);
bool gemm_takes_split_workspace(const GemmArgs& a);
int launch_gemm_check(const GemmArgs& a, cudaStream_t stream);
// Group-scale bf16 GEMM with M > 128 only: same result, plus clock stamps of CTA 0's pipeline roles.
int launch_gemm_timeline(const GemmArgs& a, long long* timeline, cudaStream_t stream);

// Tensor-pipe rate probe: n_cols in {64, 128, 256}; cycles is a device int64.
int launch_mma_rate(int n_cols, int iters, long long* cycles, cudaStream_t stream);

// One CTA waits `limit_us` for a barrier nobody arrives at, then reports status 9190 (see sq_wait_probe).
int launch_wait_probe(int64_t limit_us, long long* waited_ns, cudaStream_t stream);

// Device-side status word (0 = fine).  Written by kernels that gave up a bounded wait.
int* device_status_word();

}  // namespace sq

// extern "C" surface of libsq_b200.so, argument validation, the device status word and the
// CUDA-core cross-check GEMM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "sq_internal.h"

namespace sq {

// ------------------------------------------------------------------ device status word
__device__ int g_device_status = 0;

int* device_status_word() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;  // callers treat null as a driver error
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) == cudaSuccess) cached[dev] = static_cast<int*>(ptr);
  }
  return cached[dev];
}

// ------------------------------------------------------------------ validation
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate_gemm(const GemmArgs& a) {
  if (a.codes == nullptr || a.w_packed == nullptr || a.w_scales == nullptr || a.row_scales == nullptr || a.out == nullptr)
    return SQ_ERR_NULL;
  if (a.codes_layout != SQ_CODES_NATURAL && a.codes_layout != SQ_CODES_EVEN_ODD) return SQ_ERR_ENUM;
  if (a.wscale_mode != SQ_WSCALE_CHANNEL_F32 && a.wscale_mode != SQ_WSCALE_GROUP_F16) return SQ_ERR_ENUM;
  if (a.out_dtype != SQ_BF16 && a.out_dtype != SQ_FP16) return SQ_ERR_ENUM;
  if (a.activation != SQ_ACT_FN_NONE) return SQ_ERR_ENUM;  // activations are fused on the input side only
  if (a.gate != nullptr && (a.gate_span <= 0 || a.gate_row_stride < a.N)) return SQ_ERR_SHAPE;
  if (a.M < 0 || a.N <= 0 || a.K <= 0) return SQ_ERR_SHAPE;
  if (a.K % 32 != 0 || a.N % 8 != 0 || a.K < 128) return SQ_ERR_SHAPE;
  if (a.wscale_mode == SQ_WSCALE_GROUP_F16 && a.K % 128 != 0) return SQ_ERR_SHAPE;
  if (a.M > (int64_t{1} << 30) || a.N > (int64_t{1} << 30) || a.K > 131072) return SQ_ERR_SHAPE;
  if (!aligned16(a.codes) || !aligned16(a.w_packed) || !aligned16(a.out)) return SQ_ERR_SHAPE;
  // the drain reads row scales four at a time; scales, bias, gate, residual and the dump are read or written
  // element by element in their own types
  if (!aligned16(a.row_scales)) return SQ_ERR_SHAPE;
  const uintptr_t scale_align = a.wscale_mode == SQ_WSCALE_GROUP_F16 ? 2u : 4u;
  if ((reinterpret_cast<uintptr_t>(a.w_scales) & (scale_align - 1)) != 0) return SQ_ERR_SHAPE;
  if (((reinterpret_cast<uintptr_t>(a.bias) | reinterpret_cast<uintptr_t>(a.gate) |
        reinterpret_cast<uintptr_t>(a.residual)) & 1u) != 0)
    return SQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a.acc_dump) & 3u) != 0) return SQ_ERR_SHAPE;
  // unpacked weights are stored in the even-odd k order
  if (a.weights_prepacked && a.codes_layout != SQ_CODES_EVEN_ODD) return SQ_ERR_ENUM;
  return SQ_OK;
}

// ------------------------------------------------------------------ kernel choice
// Two GEMM kernels share the interface.  sq_gemm_tc.cu (operands in shared memory, whole tiles only) is the
// faster one at every size measured so far and is the default; SQ_GEMM_KERNEL=ts in the environment (read once)
// selects sq_gemm_ts.cu (weights in tensor memory, tiles split along K) for comparisons.
static bool second_generation_requested() {
  static const bool requested = [] {
    const char* value = std::getenv("SQ_GEMM_KERNEL");
    return value != nullptr && std::strcmp(value, "ts") == 0;
  }();
  return requested;
}

bool gemm_takes_split_workspace(const GemmArgs&) { return true; }  // both kernels split K when tiles are few

int launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.weights_prepacked || !second_generation_requested()) return launch_gemm_tc(a, stream);
  return launch_gemm_ts(a, stream);
}

// ------------------------------------------------------------------ weight prepack
// One thread per packed 32-bit word (8 consecutive k of one channel): the unpack the GEMM's converter warps do
// per tile, done once.  Output bytes: 16 w of k0 k2 k4 k6, then of k1 k3 k5 k7.
__global__ void sq_prepack_kernel(const uint32_t* __restrict__ packed, uint2* __restrict__ tiled, int64_t words) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= words) return;
  const uint32_t w = __ldg(packed + i);
  tiled[i] = make_uint2((w << 4) & 0xF0F0F0F0u, w & 0xF0F0F0F0u);
}

int launch_prepack_weights(const uint8_t* w_packed, int64_t N, int64_t K, int8_t* w_tiled, cudaStream_t stream) {
  if (w_packed == nullptr || w_tiled == nullptr) return SQ_ERR_NULL;
  if (N <= 0 || K <= 0 || K % 32 != 0 || N > (int64_t{1} << 30) || K > 131072) return SQ_ERR_SHAPE;
  if (!aligned16(w_packed) || !aligned16(w_tiled)) return SQ_ERR_SHAPE;
  const int64_t words = N * (K / 8);
  const int threads = 256;
  const int64_t blocks = (words + threads - 1) / threads;
  sq_prepack_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
      reinterpret_cast<const uint32_t*>(w_packed), reinterpret_cast<uint2*>(w_tiled), words);
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? SQ_OK : static_cast<int>(err);
}

// ------------------------------------------------------------------ cross-check GEMM (CUDA cores)
// One thread per output element.  fp32 steps are separate multiplies and adds in the oracle's order,
// so this kernel matches the CPU oracle bit for bit.
template <typename OutT>
__global__ void sq_gemm_check_kernel(const int8_t* __restrict__ codes, int even_odd, const uint8_t* __restrict__ packed,
                                     const void* __restrict__ w_scales, int group_mode, const float* __restrict__ row_scales,
                                     const OutT* __restrict__ bias, OutT* __restrict__ out, int64_t M, int64_t N, int64_t K,
                                     int32_t* __restrict__ acc_dump) {
  const int64_t n = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t m = blockIdx.y;
  if (n >= N || m >= M) return;
  const int8_t* a = codes + m * K;
  const uint8_t* w = packed + n * (K / 2);
  const int groups = group_mode ? static_cast<int>(K / 128) : 1;
  const int64_t group_len = group_mode ? 128 : K;
  float total = 0.0f;
  int32_t acc_all = 0;
  for (int g = 0; g < groups; ++g) {
    int32_t acc = 0;
    for (int64_t k8 = g * group_len; k8 < (g + 1) * group_len; k8 += 8) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint8_t byte = w[(k8 >> 1) + j];
        const int lo = (static_cast<int>(byte & 0xF) ^ 8) - 8;  // k8 + 2j
        const int hi = (static_cast<int>(byte >> 4) ^ 8) - 8;   // k8 + 2j + 1
        const int a_lo = even_odd ? a[k8 + j] : a[k8 + 2 * j];
        const int a_hi = even_odd ? a[k8 + 4 + j] : a[k8 + 2 * j + 1];
        acc += a_lo * lo + a_hi * hi;
      }
    }
    if (acc_dump != nullptr) acc_dump[(m * N + n) * groups + g] = acc;
    if (group_mode) {
      const float s = __half2float(static_cast<const __half*>(w_scales)[n * groups + g]);
      total = __fadd_rn(total, __fmul_rn(static_cast<float>(acc), s));
    } else {
      acc_all = acc;
    }
  }
  float y;
  if (group_mode) {
    y = __fmul_rn(total, row_scales[m]);
  } else {
    y = __fmul_rn(__fmul_rn(static_cast<float>(acc_all), row_scales[m]), static_cast<const float*>(w_scales)[n]);
  }
  if (bias != nullptr) {
    float b;
    if constexpr (std::is_same<OutT, __half>::value) b = __half2float(bias[n]);
    else b = __bfloat162float(bias[n]);
    y = __fadd_rn(y, b);
  }
  if constexpr (std::is_same<OutT, __half>::value) out[m * N + n] = __float2half_rn(y);
  else out[m * N + n] = __float2bfloat16_rn(y);
}

int launch_gemm_check(const GemmArgs& a, cudaStream_t stream) {
  int v = validate_gemm(a);
  if (v != SQ_OK) return v;
  if (a.weights_prepacked) return SQ_ERR_ENUM;  // the cross-check reads the packed int4 form only
  if (a.M == 0) return SQ_OK;
  if (a.M > 65535) return SQ_ERR_SHAPE;
  const dim3 block(128);
  const dim3 grid(static_cast<unsigned>((a.N + 127) / 128), static_cast<unsigned>(a.M));
  const int eo = a.codes_layout == SQ_CODES_EVEN_ODD;
  const int gm = a.wscale_mode == SQ_WSCALE_GROUP_F16;
  if (a.out_dtype == SQ_BF16) {
    sq_gemm_check_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        a.codes, eo, a.w_packed, a.w_scales, gm, a.row_scales, static_cast<const __nv_bfloat16*>(a.bias),
        static_cast<__nv_bfloat16*>(a.out), a.M, a.N, a.K, a.acc_dump);
  } else {
    sq_gemm_check_kernel<__half><<<grid, block, 0, stream>>>(
        a.codes, eo, a.w_packed, a.w_scales, gm, a.row_scales, static_cast<const __half*>(a.bias),
        static_cast<__half*>(a.out), a.M, a.N, a.K, a.acc_dump);
  }
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? SQ_OK : static_cast<int>(err);
}

static size_t round256(size_t v) { return (v + 255u) & ~static_cast<size_t>(255u); }

// sq_linear*: a workspace that is larger than codes + row scales by sq_split_workspace_bytes() lends the GEMM its
// tail for tiles split along K; the pre-pass in front clears the counters at the head of that area.
static void attach_split_area(GemmArgs& a, void* workspace, size_t workspace_bytes, int64_t rows, int64_t K,
                              PrepassFusion* prepass) {
  if (rows <= 0 || !gemm_takes_split_workspace(a)) return;
  const size_t basic = round256(static_cast<size_t>(rows) * static_cast<size_t>(K)) + round256(static_cast<size_t>(rows) * 4u);
  const size_t extra = gemm_split_workspace_bytes(rows);
  if (workspace_bytes < basic + extra) return;
  a.split_workspace = static_cast<uint8_t*>(workspace) + basic;
  a.split_workspace_bytes = extra;
  a.split_counters_cleared = true;
  prepass->clear_words = static_cast<int*>(a.split_workspace);
}

// ------------------------------------------------------------------ library-owned scratch (sq_linear_noalloc)
// Scratch for callers that cannot allocate: a fixed array in the library's own device image.  Every GPU that
// loads the library carries it until the process exits.  In host code the name below is only a handle for
// the runtime, not a device address; the address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SQ_NOALLOC_SCRATCH_BYTES];

// Device address of the scratch array on the current device (looked up on first use), or null with *err set.
static void* noalloc_scratch_ptr(cudaError_t* err) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    *err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (*err != cudaSuccess) return nullptr;
    cached[dev] = ptr;
  }
  return cached[dev];
}

}  // namespace sq

// ====================================================================== C ABI
extern "C" {
#pragma GCC visibility push(default)

int sq_prepass(const void* x, int x_dtype, int64_t rows, int64_t K, int abits, int mode, const float* inv_d,
               const float* signs, int rht_block, const float* act_scale, const float* gains, int64_t span,
               int64_t streams, int64_t seq_tokens, int codes_layout, int pack_int4, void* codes, float* row_scales,
               void* stream) {
  return sq::launch_prepass(x, x_dtype, rows, K, abits, mode, inv_d, signs, rht_block, act_scale, gains, span, streams,
                            seq_tokens, codes_layout, pack_int4, codes, row_scales, static_cast<cudaStream_t>(stream));
}

static sq::GemmArgs make_args(const void* codes, int codes_layout, const void* w_packed, const void* w_scales,
                              int wscale_mode, const float* row_scales, const void* bias, void* out, int out_dtype,
                              int64_t M, int64_t N, int64_t K, int32_t* acc_dump) {
  sq::GemmArgs a;
  a.codes = static_cast<const int8_t*>(codes);
  a.codes_layout = codes_layout & ~SQ_CODES_INT4_RANGE;
  a.codes_int4_range = (codes_layout & SQ_CODES_INT4_RANGE) != 0;
  a.w_packed = static_cast<const uint8_t*>(w_packed);
  a.w_scales = w_scales;
  a.wscale_mode = wscale_mode & ~SQ_WEIGHTS_PREPACKED;
  a.weights_prepacked = (wscale_mode & SQ_WEIGHTS_PREPACKED) != 0;
  a.row_scales = row_scales;
  a.bias = bias;
  a.out = out;
  a.out_dtype = out_dtype;
  a.M = M; a.N = N; a.K = K;
  a.acc_dump = acc_dump;
  a.activation = SQ_ACT_FN_NONE;
  a.gate = nullptr; a.gate_span = 1; a.gate_row_stride = 0; a.residual = nullptr;
  return a;
}

int sq_gemm(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
            const float* row_scales, const void* bias, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
            int32_t* acc_dump, void* stream) {
  return sq::launch_gemm(make_args(codes, codes_layout, w_packed, w_scales, wscale_mode, row_scales, bias, out,
                                   out_dtype, M, N, K, acc_dump),
                         static_cast<cudaStream_t>(stream));
}

int sq_gemm_split(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
                  const float* row_scales, const void* bias, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                  int32_t* acc_dump, void* split_workspace, size_t split_workspace_bytes, void* stream) {
  sq::GemmArgs a = make_args(codes, codes_layout, w_packed, w_scales, wscale_mode, row_scales, bias, out, out_dtype, M,
                             N, K, acc_dump);
  if (split_workspace != nullptr && (reinterpret_cast<uintptr_t>(split_workspace) & 15u) != 0) return SQ_ERR_SHAPE;
  if (sq::gemm_takes_split_workspace(a)) {
    a.split_workspace = split_workspace;
    a.split_workspace_bytes = split_workspace_bytes;
  }
  return sq::launch_gemm(a, static_cast<cudaStream_t>(stream));
}

size_t sq_split_workspace_bytes(int64_t M) { return sq::gemm_split_workspace_bytes(M); }

int sq_gemm_scatter(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
                    const float* row_scales, const void* bias, void* const* outs, int n_outs, int64_t out_ld,
                    int64_t out_col0, int out_dtype, int64_t M, int64_t N, int64_t K, void* stream) {
  if (outs == nullptr) return SQ_ERR_NULL;
  if (n_outs < 1 || n_outs > 8) return SQ_ERR_SHAPE;
  if (out_col0 < 0 || out_ld < out_col0 + N) return SQ_ERR_SHAPE;
  for (int d = 0; d < n_outs; ++d) {
    if (outs[d] == nullptr) return SQ_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(outs[d]) & 1u) != 0) return SQ_ERR_SHAPE;  // 2-byte elements
  }
  sq::GemmArgs a = make_args(codes, codes_layout, w_packed, w_scales, wscale_mode, row_scales, bias, outs[0], out_dtype,
                             M, N, K, nullptr);
  a.out_ld = out_ld;
  a.out_col0 = out_col0;
  a.n_more_outs = n_outs - 1;
  for (int d = 1; d < n_outs; ++d) a.more_outs[d - 1] = outs[d];
  if (M > 0 && M < 128) return SQ_ERR_SHAPE;  // the channel-split form is built for many tokens (128-token tiles)
  return sq::launch_gemm_tc(a, static_cast<cudaStream_t>(stream));
}

int sq_gemm_check(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
                  const float* row_scales, const void* bias, void* out, int out_dtype, int64_t M, int64_t N,
                  int64_t K, int32_t* acc_dump, void* stream) {
  return sq::launch_gemm_check(make_args(codes, codes_layout, w_packed, w_scales, wscale_mode, row_scales, bias, out,
                                         out_dtype, M, N, K, acc_dump),
                               static_cast<cudaStream_t>(stream));
}

int sq_gemm_timeline(const void* codes, const void* w_packed, const void* w_scales, const float* row_scales,
                     const void* bias, void* out, int64_t M, int64_t N, int64_t K, long long* timeline, void* stream) {
  const sq::GemmArgs a = make_args(codes, SQ_CODES_EVEN_ODD | SQ_CODES_INT4_RANGE, w_packed, w_scales,
                                   SQ_WSCALE_GROUP_F16, row_scales, bias, out, SQ_BF16, M, N, K, nullptr);
  if (sq::second_generation_requested()) return sq::launch_gemm_ts_timeline(a, timeline, static_cast<cudaStream_t>(stream));
  return sq::launch_gemm_timeline(a, timeline, static_cast<cudaStream_t>(stream));
}

int sq_prepack_weights(const void* w_packed, int64_t N, int64_t K, void* w_tiled, void* stream) {
  return sq::launch_prepack_weights(static_cast<const uint8_t*>(w_packed), N, K, static_cast<int8_t*>(w_tiled),
                                    static_cast<cudaStream_t>(stream));
}

int sq_mma_rate(int n_cols, int iterations, long long* cycles, void* stream) {
  return sq::launch_mma_rate(n_cols, iterations, cycles, static_cast<cudaStream_t>(stream));
}

int sq_wait_probe(int64_t limit_us, long long* waited_ns, void* stream) {
  return sq::launch_wait_probe(limit_us, waited_ns, static_cast<cudaStream_t>(stream));
}

size_t sq_workspace_bytes(int64_t M, int64_t K) {
  if (M < 0 || K < 0) return 0;
  return sq::round256(static_cast<size_t>(M) * static_cast<size_t>(K)) + sq::round256(static_cast<size_t>(M) * 4u);
}

int sq_linear(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode, const float* inv_d,
              const float* signs, int rht_block, const float* act_scales, const float* gains, int64_t calls,
              int64_t call, int64_t span, int64_t streams, int64_t seq_tokens, const void* w_packed,
              const void* w_scales, int wscale_mode, const void* bias, void* out, void* workspace,
              size_t workspace_bytes, void* stream) {
  return sq_linear_fused(x, x_dtype, rows, K, N, abits, mode, inv_d, signs, rht_block, act_scales, gains, calls, call,
                         span, streams, seq_tokens, w_packed, w_scales, wscale_mode, bias, SQ_ACT_FN_NONE, SQ_NORM_NONE, 0.0f,
                         nullptr, nullptr, nullptr, 1, 0, 0, SQ_ACT_FN_NONE, nullptr, 1, 0, nullptr, out, workspace,
                         workspace_bytes, stream);
}

int sq_linear_fused(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                    const float* inv_d, const float* signs, int rht_block, const float* act_scales,
                    const float* gains, int64_t calls, int64_t call, int64_t span, int64_t streams,
                    int64_t seq_tokens, const void* w_packed, const void* w_scales, int wscale_mode,
                    const void* bias, int input_activation, int norm_kind, float norm_eps, const void* norm_weight,
                    const void* mod_scale,
                    const void* mod_shift, int64_t mod_span, int64_t mod_row_stride, int round_after_norm,
                    int activation, const void* gate, int64_t gate_span, int64_t gate_row_stride,
                    const void* residual, void* out, void* workspace, size_t workspace_bytes, void* stream) {
  return sq_linear_scheduled(x, x_dtype, rows, K, N, abits, mode, inv_d, signs, rht_block, act_scales, gains, calls,
                             call, nullptr, span, streams, seq_tokens, w_packed, w_scales, wscale_mode, bias,
                             input_activation, norm_kind, norm_eps, norm_weight, mod_scale, mod_shift, mod_span,
                             mod_row_stride, round_after_norm, activation, gate, gate_span, gate_row_stride, residual,
                             out, workspace, workspace_bytes, stream);
}

int sq_linear_scheduled(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                        const float* inv_d, const float* signs, int rht_block, const float* act_scales,
                        const float* gains, int64_t calls, int64_t call, const int32_t* call_index, int64_t span,
                        int64_t streams, int64_t seq_tokens, const void* w_packed, const void* w_scales,
                        int wscale_mode, const void* bias, int input_activation, int norm_kind, float norm_eps,
                        const void* norm_weight, const void* mod_scale, const void* mod_shift, int64_t mod_span,
                        int64_t mod_row_stride, int round_after_norm, int activation, const void* gate,
                        int64_t gate_span, int64_t gate_row_stride, const void* residual, void* out,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (workspace == nullptr && rows > 0) return SQ_ERR_NULL;
  if (workspace_bytes < sq_workspace_bytes(rows, K)) return SQ_ERR_WORKSPACE;
  const float* act_scale = nullptr;
  const float* gain_row = nullptr;
  if (mode == SQ_ACT_STATIC) {
    if (act_scales == nullptr || gains == nullptr) return SQ_ERR_NULL;
    if (streams <= 0) return SQ_ERR_SHAPE;
    if (call_index != nullptr) {
      // the entry is read (and clamped to the table) on the device: the tables are passed whole
      if (calls <= 0) return SQ_ERR_INDEX;
      act_scale = act_scales;
      gain_row = gains;
    } else {
      if (calls <= 0 || call < 0 || call >= calls) return SQ_ERR_INDEX;
      act_scale = act_scales + call;
      gain_row = gains + call * streams;
    }
  }
  int8_t* codes = static_cast<int8_t*>(workspace);
  float* row_scales = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                               sq::round256(static_cast<size_t>(rows) * static_cast<size_t>(K)));
  // validate the GEMM half before launching anything, so a rejected call leaves no work on the stream
  // the pre-pass clamps 4-bit codes to +-7, so the GEMM may use its small accumulator offset
  sq::GemmArgs a = make_args(codes, SQ_CODES_EVEN_ODD | (abits == 4 ? SQ_CODES_INT4_RANGE : 0), w_packed, w_scales, wscale_mode, row_scales, bias, out, x_dtype,
                             rows, N, K, nullptr);
  a.activation = activation;
  a.gate = gate; a.gate_span = gate_span; a.gate_row_stride = gate_row_stride; a.residual = residual;
  sq::PrepassFusion fusion;
  fusion.input_activation = input_activation;
  fusion.norm_kind = norm_kind; fusion.norm_eps = norm_eps; fusion.norm_weight = norm_weight;
  fusion.mod_scale = mod_scale; fusion.mod_shift = mod_shift; fusion.mod_span = mod_span;
  fusion.mod_row_stride = mod_row_stride; fusion.round_after = round_after_norm;
  if (mode == SQ_ACT_STATIC && call_index != nullptr) {
    fusion.call_index = call_index;
    fusion.calls = calls;
  }
  if (rows > 0) {
    int v = sq::validate_gemm(a);
    if (v != SQ_OK) return v;
  }
  sq::attach_split_area(a, workspace, workspace_bytes, rows, K, &fusion);
  int status = sq::launch_prepass(x, x_dtype, rows, K, abits, mode, inv_d, signs, rht_block, act_scale, gain_row, span,
                                  streams, seq_tokens, SQ_CODES_EVEN_ODD, 0, codes, row_scales,
                                  static_cast<cudaStream_t>(stream), &fusion);
  if (status != SQ_OK) return status;
  a.after_prepass = true;
  return sq::launch_gemm(a, static_cast<cudaStream_t>(stream));
}

int sq_prepass_composite(const void* x, int x_dtype, int64_t rows, int64_t K, int abits, int mode, const float* inv_d,
                         const float* signs, const float* mix, int mix_order, const float* act_scale,
                         const float* gains, int64_t span, int64_t streams, int64_t seq_tokens, int codes_layout,
                         int pack_int4, void* codes, float* row_scales, void* stream) {
  if (mix == nullptr) return SQ_ERR_NULL;
  sq::PrepassFusion rotation;
  rotation.mix = mix;
  rotation.mix_order = mix_order;
  return sq::launch_prepass(x, x_dtype, rows, K, abits, mode, inv_d, signs, 0, act_scale, gains, span, streams,
                            seq_tokens, codes_layout, pack_int4, codes, row_scales, static_cast<cudaStream_t>(stream),
                            &rotation);
}

int sq_linear_composite(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                        const float* inv_d, const float* signs, const float* mix, int mix_order,
                        const float* act_scales, const float* gains, int64_t calls, int64_t call,
                        const int32_t* call_index, int64_t span, int64_t streams, int64_t seq_tokens,
                        const void* w_packed, const void* w_scales, int wscale_mode, const void* bias, void* out,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (mix == nullptr || (workspace == nullptr && rows > 0)) return SQ_ERR_NULL;
  if (workspace_bytes < sq_workspace_bytes(rows, K)) return SQ_ERR_WORKSPACE;
  const float* act_scale = nullptr;
  const float* gain_row = nullptr;
  if (mode == SQ_ACT_STATIC) {
    if (act_scales == nullptr || gains == nullptr) return SQ_ERR_NULL;
    if (streams <= 0) return SQ_ERR_SHAPE;
    if (call_index != nullptr) {
      if (calls <= 0) return SQ_ERR_INDEX;
      act_scale = act_scales;
      gain_row = gains;
    } else {
      if (calls <= 0 || call < 0 || call >= calls) return SQ_ERR_INDEX;
      act_scale = act_scales + call;
      gain_row = gains + call * streams;
    }
  }
  int8_t* codes = static_cast<int8_t*>(workspace);
  float* row_scales = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                               sq::round256(static_cast<size_t>(rows) * static_cast<size_t>(K)));
  sq::GemmArgs a = make_args(codes, SQ_CODES_EVEN_ODD | (abits == 4 ? SQ_CODES_INT4_RANGE : 0), w_packed, w_scales,
                             wscale_mode, row_scales, bias, out, x_dtype, rows, N, K, nullptr);
  if (rows > 0) {
    const int v = sq::validate_gemm(a);
    if (v != SQ_OK) return v;
  }
  sq::PrepassFusion rotation;
  rotation.mix = mix;
  rotation.mix_order = mix_order;
  if (mode == SQ_ACT_STATIC && call_index != nullptr) {
    rotation.call_index = call_index;
    rotation.calls = calls;
  }
  sq::attach_split_area(a, workspace, workspace_bytes, rows, K, &rotation);
  const int status = sq::launch_prepass(x, x_dtype, rows, K, abits, mode, inv_d, signs, 0, act_scale, gain_row, span,
                                        streams, seq_tokens, SQ_CODES_EVEN_ODD, 0, codes, row_scales,
                                        static_cast<cudaStream_t>(stream), &rotation);
  if (status != SQ_OK) return status;
  a.after_prepass = true;
  return sq::launch_gemm(a, static_cast<cudaStream_t>(stream));
}

int sq_linear_noalloc(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                      const float* inv_d, const float* signs, int rht_block, const float* act_scales,
                      const float* gains, int64_t calls, int64_t call, int64_t span, int64_t streams,
                      int64_t seq_tokens, const void* w_packed, const void* w_scales, int wscale_mode,
                      const void* bias, void* out, void* stream) {
  if (rows < 0 || K <= 0) return SQ_ERR_SHAPE;
  const size_t need = sq_workspace_bytes(rows, K);
  if (need > static_cast<size_t>(SQ_NOALLOC_SCRATCH_BYTES)) return SQ_ERR_SCRATCH_LIMIT;
  cudaError_t err = cudaSuccess;
  void* scratch = sq::noalloc_scratch_ptr(&err);
  if (scratch == nullptr) return err != cudaSuccess ? static_cast<int>(err) : SQ_ERR_DRIVER;
  // Nothing in the scratch has to start at zero: the pre-pass writes every code and row scale the GEMM reads.
  return sq_linear(x, x_dtype, rows, K, N, abits, mode, inv_d, signs, rht_block, act_scales, gains, calls, call, span,
                   streams, seq_tokens, w_packed, w_scales, wscale_mode, bias, out, scratch, need, stream);
}

int sq_device_status(void) {
  int* word = sq::device_status_word();
  if (word == nullptr) return SQ_ERR_DRIVER;
  int value = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return SQ_ERR_DRIVER;
  if (cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return SQ_ERR_DRIVER;
  if (value != 0) {
    int zero = 0;
    cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return value;
}

const char* sq_status_string(int status) {
  switch (status) {
    case SQ_OK: return "ok";
    case SQ_ERR_NULL: return "a required pointer is null";
    case SQ_ERR_SHAPE: return "unsupported shape or alignment";
    case SQ_ERR_ENUM: return "enum argument out of range";
    case SQ_ERR_INDEX: return "schedule index out of range";
    case SQ_ERR_DRIVER: return "CUDA driver call failed";
    case SQ_ERR_WORKSPACE: return "workspace too small";
    case SQ_ERR_DEVICE_WAIT: return "a kernel gave up a bounded wait";
    case SQ_ERR_SCRATCH_LIMIT: return "rows * K is beyond the library-owned scratch of sq_linear_noalloc";
    case 9006: return "device: the MMA rate probe timed out waiting for its MMAs";
    case 9007: return "device: drain warp timed out waiting for its partner at a block of group scales";
    case 9101: return "device: TMA producer timed out waiting for a free stage";
    case 9102: return "device: MMA warp timed out waiting for a free accumulator";
    case 9103: return "device: MMA warp timed out waiting for operands";
    case 9104: return "device: unpack warp timed out waiting for packed weights or a free weight stage";
    case 9105: return "device: drain warp timed out waiting for an accumulator";
    case 9107: return "device: TMA producer timed out waiting for a free row-scale slot";
    case 9108: return "device: drain warps timed out meeting around a split tile";
    case 9109: return "device: drain warp timed out waiting for row scales";
    case 9190: return "device: the wait probe gave up, as it is meant to";
    case 9001: return "device: TMA producer timed out waiting for a free stage";
    case 9002: return "device: MMA warp timed out waiting for a free accumulator";
    case 9003: return "device: MMA warp timed out waiting for operands";
    case 9004: return "device: converter warp timed out waiting for packed weights";
    case 9005: return "device: drain warp timed out waiting for an accumulator";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown status";
}

const char* sq_version(void) { return "sq_b200 sm_100a"; }

#pragma GCC visibility pop
}  // extern "C"

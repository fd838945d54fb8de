// Fused activation pre-pass: bf16/fp16 rows -> [sign flip + block Hadamard, rounded to the
// input type] -> [1/D] -> per-token or scheduled scale -> int8 (or packed int4) codes + fp32
// row scales.  One pass over global memory: each row lives in registers between the 128-bit
// loads and the 64-bit code stores.
//
// Thread layout.  A row is covered by TPR threads (a power of two, 32..512); thread t of the
// row owns the 8-element vectors t, t + TPR, t + 2 TPR, ... (VPT of them), so a warp reads 512
// contiguous bytes per load.  A rotation block of B elements is B/8 consecutive vectors, i.e.
// B/8 consecutive lanes of one warp: three butterfly stages run inside the thread (strides 1,
// 2, 4) and log2(B/8) stages run as __shfl_xor_sync exchanges (strides 8, 16, ...), which is the
// stage order of the reference's CPU transform (rht.py:104-111), so the fp32 sums are the same.
//
// Arithmetic contract (what the CPU oracle does):
//   token mode : s = max(amax / qmax, 1e-8);  code = clamp(rint(v / s))   (IEEE division, rint = half to even)
//   static mode: f = gain / scale;            code = clamp(rint((v * inv_d) * f)),  row_scale = scale / gain
// How it is computed without the slow paths:
//   * v / s with one correctly rounded reciprocal r = RN(1/s) per row and two residual corrections per
//     element, q0 = v r; q1 = q0 + (v - q0 s) r; q2 = q1 + (v - q1 s) r, each residual one exact FMA.  q1 is
//     within one ulp of v / s, so q2 is the correctly rounded quotient (Markstein's theorem), i.e. the
//     same float an IEEE division returns.
//   * rint + clamp as clamp-then-add-1.5*2^23: the fp32 addition rounds to the nearest integer, ties to
//     even, and leaves the code in the low byte of the sum's bit pattern.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "sq_internal.h"

namespace sq {

template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  // round two floats to bf16 and back with one packed conversion
  static __device__ __forceinline__ void round_trip2(float& a, float& b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const uint32_t bits = *reinterpret_cast<const uint32_t*>(&h);
    a = __uint_as_float(bits << 16);
    b = __uint_as_float(bits & 0xFFFF0000u);
  }
};
template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void unpack(const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 f = __half22float2(h);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void round_trip2(float& a, float& b) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x;
    b = f.y;
  }
};

struct PrepassParams {
  const void* x;
  const float* inv_d;
  const float* signs;
  const float* act_scale;
  const float* gains;
  void* codes;
  float* row_scales;
  int64_t rows, K;
  int64_t span, streams, seq_tokens;
  int tpr_log2;        // threads per row = 1 << tpr_log2
  int rht_lanes_log2;  // log2(block / 8): number of shuffle stages
  float rht_norm;      // float(1 / sqrt(block))
  int qmax;            // 127 or 7
  int mode, codes_layout, pack_int4;
  // fused front end
  int input_activation;
  int norm_kind;
  float norm_eps;
  const void* norm_weight;
  const void* mod_scale;
  const void* mod_shift;
  int64_t mod_span, mod_row_stride;
  int round_after;
  // static mode with the schedule entry chosen on the device: act_scale / gains are then the table bases
  const int32_t* call_index;
  int64_t calls;
  int* clear_words;      // 256 ints thread block 0 sets to zero (the GEMM's K-split counters), or null
  // composite rotation (kMix): K = mix_order x part, part a power of two in [8, 512]
  const float* mix;      // [mix_order, mix_order] entries +-1, row-major
  int mix_order;
  int mix_part_log2;
  float mix_part_norm;   // float(1 / sqrt(part))
  float mix_order_root;  // float(sqrt(mix_order))
};

constexpr float kRoundMagic = 12582912.0f;  // 1.5 * 2^23

// Packed single-precision arithmetic (two IEEE operations per instruction, each rounded to nearest even exactly
// like its scalar form): the pre-pass is bound by the instructions it issues, and most of its arithmetic applies
// the same operation to neighbouring elements.
#define SQ_PACK2(dst, lo, hi) "mov.b64 " dst ", {" lo ", " hi "};\n\t"
// (a0, a1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void mul2(float& a0, float& a1, float b0, float b1) {
  asm("{\n\t.reg .b64 a, b;\n\t" SQ_PACK2("a", "%0", "%1") SQ_PACK2("b", "%2", "%3")
      "mul.rn.f32x2 a, a, b;\n\tmov.b64 {%0, %1}, a;\n\t}\n"
      : "+f"(a0), "+f"(a1) : "f"(b0), "f"(b1));
}
// (a0, a1) = (a0, a1) + (b0, b1)
__device__ __forceinline__ void add2(float& a0, float& a1, float b0, float b1) {
  asm("{\n\t.reg .b64 a, b;\n\t" SQ_PACK2("a", "%0", "%1") SQ_PACK2("b", "%2", "%3")
      "add.rn.f32x2 a, a, b;\n\tmov.b64 {%0, %1}, a;\n\t}\n"
      : "+f"(a0), "+f"(a1) : "f"(b0), "f"(b1));
}
// butterfly on two pairs: (a, b) -> (a + b, a - b)
__device__ __forceinline__ void butterfly2(float& a0, float& a1, float& b0, float& b1) {
  asm("{\n\t.reg .b64 a, b, s, d;\n\t" SQ_PACK2("a", "%0", "%1") SQ_PACK2("b", "%2", "%3")
      "add.rn.f32x2 s, a, b;\n\tsub.rn.f32x2 d, a, b;\n\t"
      "mov.b64 {%0, %1}, s;\n\tmov.b64 {%2, %3}, d;\n\t}\n"
      : "+f"(a0), "+f"(a1), "+f"(b0), "+f"(b1));
}
// (a0, a1) = (a0, a1) * (m, m) + (c0, c1)
__device__ __forceinline__ void fma2s(float& a0, float& a1, float m, float c0, float c1) {
  asm("{\n\t.reg .b64 a, b, c;\n\t" SQ_PACK2("a", "%0", "%1") SQ_PACK2("b", "%2", "%2") SQ_PACK2("c", "%3", "%4")
      "fma.rn.f32x2 a, a, b, c;\n\tmov.b64 {%0, %1}, a;\n\t}\n"
      : "+f"(a0), "+f"(a1) : "f"(m), "f"(c0), "f"(c1));
}
// correctly rounded (x0, x1) / divisor from reciprocal = RN(1 / divisor): q0 = x r, two residual corrections
__device__ __forceinline__ void divide2(float& x0, float& x1, float divisor, float reciprocal) {
  asm("{\n\t.reg .b64 x, r, nd, q, t;\n\t.reg .f32 negd;\n\t"
      SQ_PACK2("x", "%0", "%1") SQ_PACK2("r", "%3", "%3")
      "neg.f32 negd, %2;\n\t" SQ_PACK2("nd", "negd", "negd")
      "mul.rn.f32x2 q, x, r;\n\t"
      "fma.rn.f32x2 t, q, nd, x;\n\tfma.rn.f32x2 q, t, r, q;\n\t"
      "fma.rn.f32x2 t, q, nd, x;\n\tfma.rn.f32x2 q, t, r, q;\n\t"
      "mov.b64 {%0, %1}, q;\n\t}\n"
      : "+f"(x0), "+f"(x1) : "f"(divisor), "f"(reciprocal));
}

// clamp to [-qmax, qmax], round to nearest even; the code is the low byte of the result
__device__ __forceinline__ uint32_t round_code(float q, float qmax) {
  return __float_as_uint(__fadd_rn(fminf(fmaxf(q, -qmax), qmax), kRoundMagic));
}

// kFused compiles the normalisation / modulation front end in; the plain pre-pass keeps its register count.
// The plain kernel with up to three vectors per thread fits 48 registers without spills: five 256-thread blocks
// per SM instead of four.  Every variant stays within 128 registers, so the 512-thread launches fit an SM.
// kMix compiles the composite rotation in (a sign matrix across power-of-two parts of the row, through
// dynamic shared memory: one fp32 row per row of the CTA, then the matrix).
template <typename T, int VPT, bool kFused, bool kMix = false>
__global__ void __maxnreg__((VPT <= 3 && !kFused && !kMix) ? 48 : 128) sq_prepass_kernel(const PrepassParams p) {
  // lets a GEMM launched as this grid's programmatic dependent set itself up while this grid still runs
  asm volatile("griddepcontrol.launch_dependents;");
  if (p.clear_words != nullptr && blockIdx.x == 0 && threadIdx.x < 256) p.clear_words[threadIdx.x] = 0;
  const int tpr = 1 << p.tpr_log2;
  const int t = threadIdx.x & (tpr - 1);
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> p.tpr_log2) + (threadIdx.x >> p.tpr_log2);
  const bool row_ok = row < p.rows;
  const int vectors = static_cast<int>(p.K >> 3);
  const uint4* xrow = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + (row_ok ? row : 0) * p.K);

  float v[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int vec = j * tpr + t;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (row_ok && vec < vectors) raw = __ldg(xrow + vec);
    Vec8<T>::unpack(raw, v[j]);
  }

  // sum over the threads of one row (warp shuffle, then one shared-memory hop when a row spans warps)
  __shared__ float row_partial[32];
  auto row_sum = [&](float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    if (tpr > 32) {
      const int warp = threadIdx.x >> 5;
      __syncthreads();  // the previous use of row_partial is over
      if ((threadIdx.x & 31) == 0) row_partial[warp] = value;
      __syncthreads();
      const int warps_per_row = tpr >> 5;
      const int first = (warp / warps_per_row) * warps_per_row;
      value = 0.0f;
      for (int w = 0; w < warps_per_row; ++w) value += row_partial[first + w];
    }
    return value;
  };

  if (kFused && p.input_activation == SQ_ACT_FN_GELU) {
    // exact (erf) GELU of the input, rounded to the input type as the output of a separate module would be
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        v[j][i] = 0.5f * v[j][i] * (1.0f + erff(v[j][i] * 0.70710678118654752440f));
        v[j][i + 1] = 0.5f * v[j][i + 1] * (1.0f + erff(v[j][i + 1] * 0.70710678118654752440f));
        Vec8<T>::round_trip2(v[j][i], v[j][i + 1]);
      }
    }
  }

  if (kFused && p.norm_kind != SQ_NORM_NONE) {
    const float inv_k = 1.0f / static_cast<float>(p.K);
    float mean = 0.0f;
    if (p.norm_kind == SQ_NORM_LAYER) {
      float total = 0.0f;
#pragma unroll
      for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) total += v[j][i];  // masked vectors hold zeros
      mean = row_sum(total) * inv_k;
    }
    float squares = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      if (j * tpr + t < vectors) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = v[j][i] - mean;
          squares = fmaf(d, d, squares);
        }
      }
    }
    const float rstd = rsqrtf(row_sum(squares) * inv_k + p.norm_eps);
    const int64_t mod_row = (row_ok ? row : 0) / p.mod_span;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vec = j * tpr + t;
      if (vec < vectors) {
        float w[8], sc[8], sh[8];
        if (p.norm_weight != nullptr) Vec8<T>::unpack(__ldg(reinterpret_cast<const uint4*>(p.norm_weight) + vec), w);
        if (p.mod_scale != nullptr) {
          const T* srow = static_cast<const T*>(p.mod_scale) + mod_row * p.mod_row_stride;
          const T* hrow = static_cast<const T*>(p.mod_shift) + mod_row * p.mod_row_stride;
          Vec8<T>::unpack(__ldg(reinterpret_cast<const uint4*>(srow) + vec), sc);
          Vec8<T>::unpack(__ldg(reinterpret_cast<const uint4*>(hrow) + vec), sh);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float y = (v[j][i] - mean) * rstd;
          if (p.norm_weight != nullptr) y *= w[i];
          if (p.mod_scale != nullptr) y = fmaf(y, 1.0f + sc[i], sh[i]);
          v[j][i] = y;
        }
        if (p.round_after) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) Vec8<T>::round_trip2(v[j][i], v[j][i + 1]);
        }
      }
    }
  }

  if (p.signs != nullptr) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vec = j * tpr + t;
      if (vec < vectors) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.signs) + 2 * vec);
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.signs) + 2 * vec + 1);
        mul2(v[j][0], v[j][1], s0.x, s0.y); mul2(v[j][2], v[j][3], s0.z, s0.w);
        mul2(v[j][4], v[j][5], s1.x, s1.y); mul2(v[j][6], v[j][7], s1.z, s1.w);
      }
      // stride 1 inside the thread (the two halves of a pair meet: scalar)
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const float left = v[j][i], right = v[j][i + 1];
        v[j][i] = left + right;
        v[j][i + 1] = left - right;
      }
      // strides 2 and 4 inside the thread: whole pairs meet
      butterfly2(v[j][0], v[j][1], v[j][2], v[j][3]);
      butterfly2(v[j][4], v[j][5], v[j][6], v[j][7]);
      butterfly2(v[j][0], v[j][1], v[j][4], v[j][5]);
      butterfly2(v[j][2], v[j][3], v[j][6], v[j][7]);
      // strides 8, 16, ... across lanes: the lane whose bit is clear holds "left"
#pragma unroll
      for (int stage = 0; stage < 5; ++stage) {  // blocks of up to 256 = 32 lanes x 8
        if (stage < p.rht_lanes_log2) {
          constexpr int kOne = 1;
          const int lane_bit = kOne << stage;
          const float mine = (threadIdx.x & lane_bit) != 0 ? -1.0f : 1.0f;  // right: other - v, left: v + other
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const float other0 = __shfl_xor_sync(0xffffffffu, v[j][i], lane_bit);
            const float other1 = __shfl_xor_sync(0xffffffffu, v[j][i + 1], lane_bit);
            fma2s(v[j][i], v[j][i + 1], mine, other0, other1);
          }
        }
      }
      if (!kMix) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          mul2(v[j][i], v[j][i + 1], p.rht_norm, p.rht_norm);
          Vec8<T>::round_trip2(v[j][i], v[j][i + 1]);
        }
      }
    }
  }

  if (kMix) {
    // Composite rotation, the reference's order of operations (rht.py:27-39): normalised FWHT of every part
    // (the stages up to 256 are done above; a 512-long part needs one more, across warps), then the sign
    // matrix across the parts, then one division by sqrt(order); rounded to the input type at the end.
    extern __shared__ __align__(16) float mix_smem[];
    const int order = p.mix_order;
    float* matrix = mix_smem;                                   // [order * order], padded to 1024 floats
    float* buf = mix_smem + 1024 + (threadIdx.x >> p.tpr_log2) * p.K;  // this row, fp32
    for (int i = threadIdx.x; i < order * order; i += blockDim.x) matrix[i] = __ldg(p.mix + i);
    const int part = 1 << p.mix_part_log2;
    if (part == 512) {
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int vec = j * tpr + t;
        if (vec < vectors) {
          *reinterpret_cast<float4*>(buf + 8 * vec) = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
          *reinterpret_cast<float4*>(buf + 8 * vec + 4) = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
        }
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int vec = j * tpr + t;
        if (vec < vectors) {
          const int pos = 8 * vec;
          const float4 o0 = *reinterpret_cast<const float4*>(buf + (pos ^ 256));
          const float4 o1 = *reinterpret_cast<const float4*>(buf + (pos ^ 256) + 4);
          const float other[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
          const float mine = (pos & 256) != 0 ? -1.0f : 1.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i) v[j][i] = fmaf(v[j][i], mine, other[i]);
        }
      }
      __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vec = j * tpr + t;
      if (vec < vectors) {
        float h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(v[j][i], p.mix_part_norm);
        *reinterpret_cast<float4*>(buf + 8 * vec) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(buf + 8 * vec + 4) = make_float4(h[4], h[5], h[6], h[7]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vec = j * tpr + t;
      if (vec < vectors) {
        const int pos = 8 * vec;
        const int out_part = pos >> p.mix_part_log2;
        const int column = pos & (part - 1);
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        for (int src = 0; src < order; ++src) {
          const float m = matrix[out_part * order + src];
          const float4 h0 = *reinterpret_cast<const float4*>(buf + (src << p.mix_part_log2) + column);
          const float4 h1 = *reinterpret_cast<const float4*>(buf + (src << p.mix_part_log2) + column + 4);
          acc[0] = fmaf(m, h0.x, acc[0]); acc[1] = fmaf(m, h0.y, acc[1]);
          acc[2] = fmaf(m, h0.z, acc[2]); acc[3] = fmaf(m, h0.w, acc[3]);
          acc[4] = fmaf(m, h1.x, acc[4]); acc[5] = fmaf(m, h1.y, acc[5]);
          acc[6] = fmaf(m, h1.z, acc[6]); acc[7] = fmaf(m, h1.w, acc[7]);
        }
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          v[j][i] = __fdiv_rn(acc[i], p.mix_order_root);
          v[j][i + 1] = __fdiv_rn(acc[i + 1], p.mix_order_root);
          Vec8<T>::round_trip2(v[j][i], v[j][i + 1]);
        }
      }
    }
  }

  if (p.inv_d != nullptr) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vec = j * tpr + t;
      if (vec < vectors) {
        const float4 d0 = __ldg(reinterpret_cast<const float4*>(p.inv_d) + 2 * vec);
        const float4 d1 = __ldg(reinterpret_cast<const float4*>(p.inv_d) + 2 * vec + 1);
        mul2(v[j][0], v[j][1], d0.x, d0.y); mul2(v[j][2], v[j][3], d0.z, d0.w);
        mul2(v[j][4], v[j][5], d1.x, d1.y); mul2(v[j][6], v[j][7], d1.z, d1.w);
      }
    }
  }

  // scale: one number per row
  float divisor = 1.0f;     // token mode: codes = v / divisor
  float reciprocal = 1.0f;  // RN(1 / divisor)
  float multiplier = 1.0f;  // static mode: codes = v * multiplier
  const float qmax = static_cast<float>(p.qmax);
  if (p.mode == SQ_ACT_TOKEN) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
    if (tpr > 32) {
      __shared__ float warp_max[32];
      const int warp = threadIdx.x >> 5;
      if ((threadIdx.x & 31) == 0) warp_max[warp] = amax;
      __syncthreads();
      const int warps_per_row = tpr >> 5;
      const int first = (warp / warps_per_row) * warps_per_row;
      amax = 0.0f;
      for (int w = 0; w < warps_per_row; ++w) amax = fmaxf(amax, warp_max[first + w]);
    }
    divisor = fmaxf(__fdiv_rn(amax, static_cast<float>(p.qmax)), 1e-8f);
    reciprocal = __frcp_rn(divisor);
    if (row_ok && t == 0) p.row_scales[row] = divisor;
  } else {
    int64_t stream;
    if (p.span > 0) {
      stream = (row / p.span) % p.streams;
    } else {
      stream = ((row % p.seq_tokens) < p.seq_tokens + p.span) ? 0 : 1;
    }
    int64_t entry = 0;
    if (p.call_index != nullptr) {
      // clamped: a stale or wild index must not read outside the tables
      const int64_t wanted = __ldg(p.call_index);
      entry = wanted < 0 ? 0 : (wanted >= p.calls ? p.calls - 1 : wanted);
    }
    const float scale = __ldg(p.act_scale + entry);
    const float gain = __ldg(p.gains + entry * p.streams + (row_ok ? stream : 0));
    multiplier = __fdiv_rn(gain, scale);
    if (row_ok && t == 0) p.row_scales[row] = __fdiv_rn(scale, gain);
  }

  if (!row_ok) return;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int vec = j * tpr + t;
    if (vec >= vectors) continue;
    uint32_t q[8];  // code in the low byte
    if (p.mode == SQ_ACT_TOKEN) {
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        float q0 = v[j][i], q1 = v[j][i + 1];
        divide2(q0, q1, divisor, reciprocal);
        // no clamp: |x| <= amax and divisor >= RN(amax / qmax) give |q| <= qmax (1 + 2^-23), which rounds to qmax
        add2(q0, q1, kRoundMagic, kRoundMagic);
        q[i] = __float_as_uint(q0);
        q[i + 1] = __float_as_uint(q1);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = round_code(__fmul_rn(v[j][i], multiplier), qmax);
    }
    if (p.pack_int4) {
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) word |= (q[i] & 0xFu) << (4 * i);
      reinterpret_cast<uint32_t*>(p.codes)[row * vectors + vec] = word;
    } else {
      uint32_t lo, hi;
      // low bytes of four words -> one word: two byte-permutes per pair, one to join
      if (p.codes_layout == SQ_CODES_EVEN_ODD) {
        lo = __byte_perm(__byte_perm(q[0], q[2], 0x0040), __byte_perm(q[4], q[6], 0x0040), 0x5410);
        hi = __byte_perm(__byte_perm(q[1], q[3], 0x0040), __byte_perm(q[5], q[7], 0x0040), 0x5410);
      } else {
        lo = __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
        hi = __byte_perm(__byte_perm(q[4], q[5], 0x0040), __byte_perm(q[6], q[7], 0x0040), 0x5410);
      }
      reinterpret_cast<uint2*>(p.codes)[row * vectors + vec] = make_uint2(lo, hi);
    }
  }
}

template <typename T, bool kFused>
static cudaError_t launch_for_type(const PrepassParams& p, int vpt, dim3 grid, dim3 block, cudaStream_t stream) {
  switch (vpt) {
    case 1: sq_prepass_kernel<T, 1, kFused><<<grid, block, 0, stream>>>(p); break;
    case 2: sq_prepass_kernel<T, 2, kFused><<<grid, block, 0, stream>>>(p); break;
    case 3: sq_prepass_kernel<T, 3, kFused><<<grid, block, 0, stream>>>(p); break;
    case 4: sq_prepass_kernel<T, 4, kFused><<<grid, block, 0, stream>>>(p); break;
    case 5: sq_prepass_kernel<T, 5, kFused><<<grid, block, 0, stream>>>(p); break;
    case 6: sq_prepass_kernel<T, 6, kFused><<<grid, block, 0, stream>>>(p); break;
    case 7: sq_prepass_kernel<T, 7, kFused><<<grid, block, 0, stream>>>(p); break;
    default: sq_prepass_kernel<T, 8, kFused><<<grid, block, 0, stream>>>(p); break;
  }
  return cudaGetLastError();
}

// Composite-rotation instantiations need dynamic shared memory, above the default limit for wide rows.
template <typename T, int VPT>
static cudaError_t launch_mix_one(const PrepassParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
  auto kernel = sq_prepass_kernel<T, VPT, false, true>;
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return err;
  }
  kernel<<<grid, block, smem, stream>>>(p);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_mix(const PrepassParams& p, int vpt, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
  switch (vpt) {
    case 1: return launch_mix_one<T, 1>(p, grid, block, smem, stream);
    case 2: return launch_mix_one<T, 2>(p, grid, block, smem, stream);
    case 3: return launch_mix_one<T, 3>(p, grid, block, smem, stream);
    case 4: return launch_mix_one<T, 4>(p, grid, block, smem, stream);
    default: return cudaErrorInvalidValue;  // rows wider than 16384 are rejected before the launch
  }
}

int launch_prepass(const void* x, int x_dtype, int64_t rows, int64_t K, int abits, int mode, const float* inv_d,
                   const float* signs, int rht_block, const float* act_scale, const float* gains, int64_t span,
                   int64_t streams, int64_t seq_tokens, int codes_layout, int pack_int4, void* codes,
                   float* row_scales, cudaStream_t stream, const PrepassFusion* fusion) {
  if (rows == 0) return SQ_OK;  // nothing to do; an empty tensor may come with a null pointer
  if (x == nullptr || codes == nullptr || row_scales == nullptr) return SQ_ERR_NULL;
  PrepassFusion none;
  const PrepassFusion& f = fusion != nullptr ? *fusion : none;
  if (f.norm_kind != SQ_NORM_NONE && f.norm_kind != SQ_NORM_LAYER && f.norm_kind != SQ_NORM_RMS) return SQ_ERR_ENUM;
  if ((f.mod_scale == nullptr) != (f.mod_shift == nullptr)) return SQ_ERR_NULL;
  if (f.norm_kind == SQ_NORM_NONE && (f.mod_scale != nullptr || f.norm_weight != nullptr)) return SQ_ERR_ENUM;
  if (f.input_activation != SQ_ACT_FN_NONE && f.input_activation != SQ_ACT_FN_GELU) return SQ_ERR_ENUM;
  if (f.mod_scale != nullptr && (f.mod_span <= 0 || f.mod_row_stride < K || (f.mod_row_stride & 7) != 0)) return SQ_ERR_SHAPE;
  if (x_dtype != SQ_BF16 && x_dtype != SQ_FP16) return SQ_ERR_ENUM;
  if (abits != 8 && abits != 4) return SQ_ERR_ENUM;
  if (mode != SQ_ACT_STATIC && mode != SQ_ACT_TOKEN) return SQ_ERR_ENUM;
  if (codes_layout != SQ_CODES_NATURAL && codes_layout != SQ_CODES_EVEN_ODD) return SQ_ERR_ENUM;
  if (pack_int4 != 0 && (pack_int4 != 1 || abits != 4 || codes_layout != SQ_CODES_NATURAL)) return SQ_ERR_ENUM;
  if (rows < 0 || K <= 0 || (K & 7) != 0 || K > 32768) return SQ_ERR_SHAPE;
  if (rows == 0) return SQ_OK;
  {
    // everything the kernel reads or writes as 8- or 16-byte vectors; a misaligned pointer is refused here, on
    // the host, instead of becoming a misaligned-address fault on the device
    auto aligned = [](const void* ptr, uintptr_t bytes) { return (reinterpret_cast<uintptr_t>(ptr) & (bytes - 1)) == 0; };
    if (!aligned(x, 16) || !aligned(codes, 16) || !aligned(row_scales, 4)) return SQ_ERR_SHAPE;
    if (!aligned(signs, 16) || !aligned(inv_d, 16)) return SQ_ERR_SHAPE;
    if (!aligned(f.norm_weight, 16) || !aligned(f.mod_scale, 16) || !aligned(f.mod_shift, 16)) return SQ_ERR_SHAPE;
    if (!aligned(f.mix, 4) || !aligned(act_scale, 4) || !aligned(gains, 4) || !aligned(f.call_index, 4)) return SQ_ERR_SHAPE;
  }
  if (rows > (int64_t{1} << 31) - 1) return SQ_ERR_SHAPE;
  int lanes_log2 = 0;
  float norm = 1.0f;
  int part_log2 = 0;
  if (f.mix != nullptr) {
    // K = order x part: FWHT of length part (in-warp stages up to 256, one shared-memory stage for 512), then the matrix
    if (signs == nullptr) return SQ_ERR_NULL;
    if (f.norm_kind != SQ_NORM_NONE || f.input_activation != SQ_ACT_FN_NONE) return SQ_ERR_ENUM;
    if (f.mix_order < 2 || f.mix_order > 32 || K % f.mix_order != 0 || K > 16384) return SQ_ERR_SHAPE;
    const int64_t part = K / f.mix_order;
    if (part < 8 || part > 512 || (part & (part - 1)) != 0) return SQ_ERR_SHAPE;
    while ((int64_t{1} << part_log2) < part) ++part_log2;
    const int64_t in_warp = part < 256 ? part : 256;
    while ((8 << lanes_log2) < in_warp) ++lanes_log2;
  } else if (signs != nullptr) {
    if (rht_block < 8 || rht_block > 256 || (rht_block & (rht_block - 1)) != 0 || K % rht_block != 0) return SQ_ERR_SHAPE;
    while ((8 << lanes_log2) < rht_block) ++lanes_log2;
    norm = static_cast<float>(1.0 / std::sqrt(static_cast<double>(rht_block)));
  }
  if (mode == SQ_ACT_STATIC) {
    if (act_scale == nullptr || gains == nullptr) return SQ_ERR_NULL;
    if (streams <= 0 || span == 0) return SQ_ERR_SHAPE;
    if (f.call_index != nullptr && f.calls <= 0) return SQ_ERR_INDEX;
    if (span < 0 && (seq_tokens <= 0 || -span >= seq_tokens || streams != 2)) return SQ_ERR_SHAPE;
  }
  // threads per row: smallest power of two in [32, 512] that leaves at most 4 vectors per thread
  // (up to 8 vectors per thread beyond K = 16384)
  const int64_t vectors = K >> 3;
  int tpr_log2 = 5;
  while (tpr_log2 < 9 && ((vectors + (int64_t{1} << tpr_log2) - 1) >> tpr_log2) > 4) ++tpr_log2;
  const int tpr = 1 << tpr_log2;
  const int vpt = static_cast<int>((vectors + tpr - 1) / tpr);
  const int threads = tpr > 256 ? tpr : 256;
  const int rows_per_cta = threads / tpr;

  PrepassParams p;
  p.x = x; p.inv_d = inv_d; p.signs = signs; p.act_scale = act_scale; p.gains = gains;
  p.codes = codes; p.row_scales = row_scales; p.rows = rows; p.K = K;
  p.span = span; p.streams = streams; p.seq_tokens = seq_tokens;
  p.tpr_log2 = tpr_log2; p.rht_lanes_log2 = lanes_log2; p.rht_norm = norm;
  p.qmax = abits == 8 ? 127 : 7; p.mode = mode; p.codes_layout = codes_layout; p.pack_int4 = pack_int4;
  p.input_activation = f.input_activation;
  p.norm_kind = f.norm_kind; p.norm_eps = f.norm_eps; p.norm_weight = f.norm_weight;
  p.mod_scale = f.mod_scale; p.mod_shift = f.mod_shift;
  p.mod_span = f.mod_span > 0 ? f.mod_span : 1; p.mod_row_stride = f.mod_row_stride; p.round_after = f.round_after;
  p.call_index = f.call_index; p.calls = f.calls;
  p.clear_words = f.clear_words;
  p.mix = f.mix; p.mix_order = f.mix_order; p.mix_part_log2 = part_log2;
  p.mix_part_norm = static_cast<float>(1.0 / std::sqrt(static_cast<double>(int64_t{1} << part_log2)));
  p.mix_order_root = static_cast<float>(std::sqrt(static_cast<double>(f.mix_order > 0 ? f.mix_order : 1)));

  const dim3 grid(static_cast<unsigned>((rows + rows_per_cta - 1) / rows_per_cta));
  const dim3 block(threads);
  cudaError_t err;
  if (f.mix != nullptr) {
    const size_t smem = (1024 + static_cast<size_t>(rows_per_cta) * static_cast<size_t>(K)) * sizeof(float);
    err = x_dtype == SQ_BF16 ? launch_mix<__nv_bfloat16>(p, vpt, grid, block, smem, stream)
                             : launch_mix<__half>(p, vpt, grid, block, smem, stream);
  } else if (f.norm_kind != SQ_NORM_NONE || f.input_activation != SQ_ACT_FN_NONE) {
    err = x_dtype == SQ_BF16 ? launch_for_type<__nv_bfloat16, true>(p, vpt, grid, block, stream)
                             : launch_for_type<__half, true>(p, vpt, grid, block, stream);
  } else {
    err = x_dtype == SQ_BF16 ? launch_for_type<__nv_bfloat16, false>(p, vpt, grid, block, stream)
                             : launch_for_type<__half, false>(p, vpt, grid, block, stream);
  }
  return err == cudaSuccess ? SQ_OK : static_cast<int>(err);
}

}  // namespace sq

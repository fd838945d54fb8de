// W4A8 / W4A4 GEMM on the 5th-generation tensor cores: out[m, n] = sum_k a[m, k] * w[n, k].
//
// The MMA runs "weights as rows": the UMMA M dimension (TMEM lanes) is 128 output channels,
// the UMMA N dimension (TMEM columns) is up to 128 tokens.  A TMEM lane therefore belongs to ONE
// output channel, so the per-group weight scale is a per-thread scalar when the accumulator is
// drained, and small token counts map to a small UMMA N instead of a wasted 128-row tile.
//
// Per CTA (persistent over tiles; 768 threads, or 512 in the two-warp drain):
//   warp 0        TMA producer: per 128-K block one box of packed int4 weights [128 ch x 64 B] and one
//                 box of int8 activation codes [tokens x 128 B, 128-byte swizzle]
//   warps 1-3     issue tcgen05.mma.kind::i8 (4 x K=32 per block) and commit to mbarriers; in the group form
//                 they take the groups round-robin, in the channel form warps 1 and 2 take alternate K blocks
//                 into private accumulators that the drain adds.  Warp 1 owns TMEM.
//   warps 4-7     unpack int4 -> int8 from the packed stage into the canonical K-major 128B-swizzled
//                 operand tile (nibble v becomes the int8 value 16 v; the factor 1/16 is exact and is
//                 folded into the scale).  With prepacked weights (kPre) the producer loads that tile itself
//                 and these warps have nothing to do.
//   warps 8-      drain, four warps per TMEM lane quarter (32 token columns each) or two (64 columns each):
//                 tcgen05.ld the int32 accumulator of one weight group, hand the accumulator back, fold it
//                 into fp32 sums in registers with the group scale; after the last group apply the row
//                 scale, bias, gate and residual and store bf16/fp16
// The drain loop comes in several forms (generic; ring and scale position unrolled, kStatic; two wide warps per lane
// quarter with the stores of a tile deferred into the next, kDW = 2), each in a template instantiation of its own
// that the launcher picks: two forms of the loop inside one kernel function made the compiler spill the accumulator
// registers, which cost more than either form gains.
// TMEM holds a ring of four accumulators, so the MMA warps run ahead of the drain.
//
// The group form is bound by the instructions the drain issues per accumulator element, so the integer to float
// conversion is done by the tensor core itself: see the note at kConstTileBytes.
//
// Every mbarrier wait is time-bounded (see sq_ptx.cuh); a wait that gives up sets the CTA's abort
// flag and the device status word, all roles leave their loops, TMEM is released, the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "sq_internal.h"
#include "sq_ptx.cuh"

namespace sq {

namespace {

constexpr int kBlockCh = 128;  // output channels per tile = UMMA M = TMEM lanes
constexpr int kBlockK = 128;   // int8 K elements per stage = one swizzle row = one weight group
constexpr int kUmmaK = 32;     // K of one kind::i8 instruction
// Registers per thread after the roles re-partition the CTA's allocation (setmaxnreg).  setmaxnreg.inc only hands out
// registers the CTA was launched with and waits for ever when the targets add up to more, so the launcher checks this
// sum against (registers per thread at launch) x (threads) before every launch.  Control and unpack warps at 24 / 40
// instead of 32 / 48 registers measured 8 % slower in the two-warp drain.  `wide_drain`: the variant of
// the 128-token kernel that can split K keeps a few more values live in its drain loop and takes the registers for
// them from the other roles.
// `dw`: drain warps per TMEM lane quarter.  Four warps of 32 token columns each (768 threads, 80 registers per thread
// at launch), or two of 64 columns (512 threads, 128 registers at launch: a drain warp then holds 64 sums and the 64
// accumulator words of a group).
__host__ __device__ constexpr int regs_control(bool wide_drain, int dw = 4) { return dw == 2 ? 32 : wide_drain ? 24 : 32; }
__host__ __device__ constexpr int regs_unpack(bool wide_drain, int dw = 4) { return dw == 2 ? 48 : wide_drain ? 40 : 48; }
__host__ __device__ constexpr int regs_drain(bool wide_drain, int dw = 4) { return dw == 2 ? 216 : wide_drain ? 104 : 96; }
__host__ __device__ constexpr int register_pool_needed(bool wide_drain, int dw = 4) {
  return 4 * 32 * regs_control(wide_drain, dw) + 4 * 32 * regs_unpack(wide_drain, dw) + 4 * dw * 32 * regs_drain(wide_drain, dw);
}
__host__ __device__ constexpr int threads_for(int dw) { return 256 + 128 * dw; }  // 4 control + 4 unpack + 4 dw drain warps
constexpr uint32_t kPackedBytes = kBlockCh * kBlockK / 2;  // 8 KiB
constexpr uint32_t kWBytes = kBlockCh * kBlockK;           // 16 KiB
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait

// Timeline capture (debug entry point sq_gemm_timeline): CTA 0 stamps clock64() per K block.
constexpr int kTraceSlots = 512;
enum TraceRole { kTrTmaIssue = 0, kTrConvStart, kTrConvDone, kTrMmaAccFree, kTrMmaIssue, kTrDrainStart,
                 kTrDrainRelease, kTrDrainDone, kTrMmaCommitted, kTrIssuerWaits, kTrDrainWaits, kTrTileEnds, kTraceRoles };

// Group mode keeps every accumulator positive: before the real MMAs of a group, MMAs of a constant tile (both
// operands the same bytes c) put 32 c^2 per MMA into each element.  A positive int32 below 2^23 read as a float
// is the denormal acc * 2^-149, so the conversion to float costs no instruction at all: the drain is one packed
// FFMA per two elements with the scale pre-multiplied by 2^96.
//   any int8 codes:      16 |sum w a| over one 128-K group is at most 16 * 8 * 128 * 128 = 2^21, reached only by
//                        w = a = minimum, which is positive; c = -128, four MMAs: offset 2^21, sums below 2^22 + 1
//   codes within [-8, 7]: 16 |sum w a| <= 16 * 8 * 8 * 128 = 2^17, the negative side stays above -2^17;
//                        c = 64, one MMA: offset 2^17 (a smaller offset also costs less fp32 precision)
constexpr uint32_t kConstTileBytes = kBlockCh * kBlockK;  // 16 KiB
constexpr float kScaleUp = 7.922816251426434e28f;    // 2^96: keeps acc * 2^-149 * scale a normal float
constexpr float kScaleDown = 562949953421312.0f;     // 2^49 = 2^149 / 2^96 / 16 (the unpacked weights are 16 w)

constexpr int kNumConverterWarps = 4;

#ifndef SQ_TC_STAGES128
#define SQ_TC_STAGES128 5
#endif
// Four stages measured 3-7 % slower than five; a three-stage build ended in a launch failure in the per-channel
// prepacked form and is refused here (the cause was not found by reading the code, and it was not run again).
static_assert(SQ_TC_STAGES128 >= 4 && SQ_TC_STAGES128 <= 5, "load stages of the 128-token kernel");
#ifndef SQ_TC_EARLY_PROBE
#define SQ_TC_EARLY_PROBE 1
#endif
__host__ __device__ constexpr int stages_for(int tok) {
  // shared memory per stage: unpacked weights + codes + packed weights
  return tok == 128 ? SQ_TC_STAGES128 : tok == 64 ? 6 : 7;
}
__host__ __device__ constexpr uint32_t stage_bytes(int tok) { return kWBytes + tok * kBlockK + kPackedBytes; }
__host__ __device__ constexpr uint32_t smem_bytes_for(int tok) {
  return stages_for(tok) * stage_bytes(tok) + kConstTileBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ +
         2048 /*row-scale tables of the two-warp drain*/;
}

struct TcParams {
  const void* w_scales;
  const float* row_scales;
  const void* bias;
  void* out;
  int32_t* acc_dump;
  long long* timeline;  // kTrace only: [kTraceRoles][kTraceSlots] SM clock stamps written by CTA 0
  int* status;
  int64_t M, N, K;
  int ch_tiles, tok_tiles, k_blocks;
  int tok_tile;   // tokens per tile at run time: a multiple of 16, <= TOK
  int slice_cols;  // token columns per drain warp: drain warp j of a lane quarter owns [j, j + 1) * slice_cols
  int mma_split;        // channel form: 2 when both issuers have K blocks to take (k_blocks >= 2), else 1
  // K split (few tiles, many K blocks): a work item is one of `splits` parts of a tile's K blocks; every part leaves
  // its sums in `partials` ([item][token column][128 channels], fp32 or int32 bits) and the part whose drain warp
  // arrives last at the tile's counter (one 4-bit field per drain warp) adds them in part order and finalizes
  int splits;
  float* partials;
  unsigned long long* counters;
  // output matrix: row stride and first column (a plain [M, N] output: N and 0); kScatter: the same block also
  // goes to n_more matrices at these distances (in elements) from `out`
  int64_t out_ld, out_col0;
  int n_more;
  int64_t more_delta[7];
  int offset_steps;     // group mode: constant-tile MMAs in front of every group (1 or 4)
  uint32_t offset_word;  // four copies of the constant tile's byte
  uint32_t offset_bits;  // what those MMAs add to every accumulator element
  uint32_t offset_unsigned;  // the offset MMA multiplies unsigned bytes
  int out_dtype;
  // fused epilogue: out = residual + gate * act(linear)
  int activation;
  const void* gate;
  int64_t gate_span, gate_row_stride;
  const void* residual;
};

template <typename T>
__device__ __forceinline__ T from_float(float f);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }
template <>
__device__ __forceinline__ __half from_float<__half>(float f) { return __float2half_rn(f); }
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <int kRegs>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs)); }
template <int kRegs>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs)); }

// Packed single-precision pairs live in 64-bit registers, so the compiler keeps them in aligned register pairs
// and the packed FMA needs no moves around it.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ float2 unpack2(uint64_t v) {
  float2 f;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(f.x), "=f"(f.y) : "l"(v));
  return f;
}
// c += (a0, a1) * b as one packed FMA; a0 / a1 are raw bit patterns of two adjacent registers
__device__ __forceinline__ void ffma2(uint64_t& c, uint32_t a0, uint32_t a1, uint64_t b) {
  asm("{\n\t"
      ".reg .b64 a;\n\t"
      "mov.b64 a, {%1, %2};\n\t"
      "fma.rn.f32x2 %0, a, %3, %0;\n\t"
      "}\n"
      : "+l"(c)
      : "r"(a0), "r"(a1), "l"(b));
}

__device__ __forceinline__ void report_timeout(int* status, volatile int* abort_flag, int code) {
  *abort_flag = 1;
  atomicCAS(status, 0, code);
}

// Timeline capture inside the static drain: thread 256 (lane 0 of the first drain warp) of thread block 0 stamps the SM clock;
// `tl` is null in every launch but sq_gemm_timeline's.
__device__ __forceinline__ void stamp_drain(long long* tl, int role, uint32_t slot) {
  if (tl != nullptr && threadIdx.x == 256 && slot < 512u) tl[role * 512 + slot] = clock64();
}

// One group of the drain (group form, chunked scales, no K split) with its place E in the chunk of eight group
// scales - and with it its place E mod 4 in the accumulator ring - a compile-time constant: barrier addresses, TMEM
// columns, the ring's phase and the position of the scale inside the chunk then cost no instructions.  `g` is the
// group index of place 0 of the round (a multiple of eight), `phase` the ring's parity at place 0 (the same at place
// 4: two ring rounds per chunk, so it flips there).  Returns false when the wait gave up.
template <uint32_t E, int kCols>
__device__ __forceinline__ bool drain_group_static(uint32_t bar_acc_full, uint32_t bar_acc_empty, uint32_t tmem_slice,
                                                   uint32_t phase, volatile int* abort_flag, int lane,
                                                   bool& acc_ready, uint4& chunk, uint4& chunk_next,
                                                   const unsigned short* my_scales, int groups, int g,
                                                   float offset_float, float& offset_sum, uint64_t (&sums2)[kCols / 2],
                                                   long long* tl = nullptr, uint32_t slot0 = 0) {
  constexpr uint32_t POS = E & 3u;
  const uint32_t my_phase = E < 4u ? phase : phase ^ 1u;
  stamp_drain(tl, 10, slot0 + E);
  if (!acc_ready && !mbar_wait_bounded(bar_acc_full + 8 * POS, my_phase, abort_flag, 1000ull * 1000ull * 1000ull)) return false;
  tc_fence_after_sync();
  stamp_drain(tl, 5, slot0 + E);
  uint32_t r[kCols];
  tmem_ld_chunk(tmem_slice + POS * 128u, r);
  // the next group's barrier is probed under the load (a probe takes over a hundred cycles to answer)
  acc_ready = mbar_test_wait(bar_acc_full + 8 * ((POS + 1u) & 3u), POS == 3u ? my_phase ^ 1u : my_phase);
  const uint32_t word = E < 2u ? chunk.x : E < 4u ? chunk.y : E < 6u ? chunk.z : chunk.w;
  const __half2 pair = *reinterpret_cast<const __half2*>(&word);
  const float scale = ((E & 1u) != 0u ? __high2float(pair) : __low2float(pair)) * 7.922816251426434e28f;  // 2^96 (kScaleUp)
  offset_sum = fmaf(offset_float, scale, offset_sum);
  tmem_wait_ld();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar_acc_empty + 8 * POS);
  // (after the hand-back: the arrive is a release, and a global load or store issued before it would make it wait)
  if (E == 7u) {  // the chunk is used up: the next one takes its place, the one after that is requested
    chunk = chunk_next;
    const int c2 = (g >> 3) + 2;
    if (8 * c2 < groups) chunk_next = __ldg(reinterpret_cast<const uint4*>(my_scales) + c2);
  }
  stamp_drain(tl, 6, slot0 + E);
  const uint64_t scale2 = pack2(scale, scale);
#pragma unroll
  for (int i = 0; i < kCols; i += 2) ffma2(sums2[i / 2], r[i], r[i + 1], scale2);
  stamp_drain(tl, 7, slot0 + E);
  return true;
}

// Two-warp drain: the results of a tile that wait to be stored.  When a tile's last group is done its 64 sums per
// lane get their row scale, bias and cast at once (packed arithmetic, the row scales read four at a time from a
// table the warp keeps in shared memory) and are kept as 32 words of two 16-bit results; the stores - a 64-byte run
// per column and warp - then go out eight columns at a time under the accumulator loads of the next tile's first
// eight groups, instead of holding up the accumulator ring between the tiles.
// `cols`: how many of the warp's columns are real tokens (0: nothing is pending, or this lane's channel does not exist).
template <typename OutT>
struct PendingTile {
  uint32_t pairs[32];  // columns 2i (low half) and 2i + 1 (high half)
  OutT* out;           // row of the slice's first token, this lane's channel
  int cols;
};
template <typename OutT>
__device__ __forceinline__ uint32_t pack_out2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_out2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack_out2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t c;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(c) : "l"(a), "l"(b));
  return c;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t c;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(c) : "l"(a), "l"(b));
  return c;
}
// (sum - offset_sum) * row scale (+ bias), each operation rounded as in the four-warp drain's finalize; rs_table: this
// warp's 64 row scales in shared memory (byte address), written by the warp itself just before
template <typename OutT>
__device__ __forceinline__ void finish_tile(PendingTile<OutT>& t, const uint64_t (&sums2)[32], float offset_sum, float bias,
                                            bool has_bias, uint32_t rs_table) {
  const uint64_t minus_offset = pack2(-offset_sum, -offset_sum);
  const uint64_t bias2 = pack2(bias, bias);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float r0, r1, r2, r3;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r0), "=f"(r1), "=f"(r2), "=f"(r3) : "r"(rs_table + 16 * j));
    uint64_t a = mul2(add2(sums2[2 * j], minus_offset), pack2(r0, r1));
    uint64_t b = mul2(add2(sums2[2 * j + 1], minus_offset), pack2(r2, r3));
    if (has_bias) {
      a = add2(a, bias2);
      b = add2(b, bias2);
    }
    const float2 fa = unpack2(a), fb = unpack2(b);
    t.pairs[2 * j] = pack_out2<OutT>(fa.x, fa.y);
    t.pairs[2 * j + 1] = pack_out2<OutT>(fb.x, fb.y);
  }
}
// the stores of columns [kFirst, kFirst + kCount) of the pending tile
template <int kFirst, int kCount, typename OutT>
__device__ __forceinline__ void store_pending(const PendingTile<OutT>& t, int64_t out_ld) {
  unsigned short* out = reinterpret_cast<unsigned short*>(t.out);
#pragma unroll
  for (int i = kFirst; i < kFirst + kCount; ++i) {
    const uint32_t word = t.pairs[i / 2];
    if (i < t.cols) out[i * out_ld] = static_cast<unsigned short>((i & 1) != 0 ? word >> 16 : word & 0xFFFFu);
  }
}

// A group of a tile's first round in the two-warp drain: drain_group_static with the stores of eight columns of the
// pending tile issued after the accumulator's hand-back, in front of the arithmetic.
template <uint32_t E, typename OutT>
__device__ __forceinline__ bool drain_group_first(uint32_t bar_acc_full, uint32_t bar_acc_empty, uint32_t tmem_slice,
                                                  uint32_t phase, volatile int* abort_flag, int lane, bool& acc_ready,
                                                  uint4& chunk, uint4& chunk_next, const unsigned short* my_scales,
                                                  int groups, int g, float offset_float, float& offset_sum,
                                                  uint64_t (&sums2)[32], const PendingTile<OutT>& pending, int64_t out_ld,
                                                  long long* tl = nullptr, uint32_t slot0 = 0) {
  constexpr uint32_t POS = E & 3u;
  const uint32_t my_phase = E < 4u ? phase : phase ^ 1u;
  stamp_drain(tl, 10, slot0 + E);
  if (!acc_ready && !mbar_wait_bounded(bar_acc_full + 8 * POS, my_phase, abort_flag, 1000ull * 1000ull * 1000ull)) return false;
  tc_fence_after_sync();
  stamp_drain(tl, 5, slot0 + E);
  uint32_t r[64];
  tmem_ld_chunk(tmem_slice + POS * 128u, r);
  acc_ready = mbar_test_wait(bar_acc_full + 8 * ((POS + 1u) & 3u), POS == 3u ? my_phase ^ 1u : my_phase);
  const uint32_t word = E < 2u ? chunk.x : E < 4u ? chunk.y : E < 6u ? chunk.z : chunk.w;
  const __half2 pair = *reinterpret_cast<const __half2*>(&word);
  const float scale = ((E & 1u) != 0u ? __high2float(pair) : __low2float(pair)) * 7.922816251426434e28f;  // 2^96 (kScaleUp)
  offset_sum = fmaf(offset_float, scale, offset_sum);
  tmem_wait_ld();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar_acc_empty + 8 * POS);
  // (after the hand-back: the arrive is a release, and a global load or store issued before it would make it wait)
  if (E == 7u) {
    chunk = chunk_next;
    const int c2 = (g >> 3) + 2;
    if (8 * c2 < groups) chunk_next = __ldg(reinterpret_cast<const uint4*>(my_scales) + c2);
  }
  store_pending<8 * E, 8, OutT>(pending, out_ld);
  stamp_drain(tl, 6, slot0 + E);
  const uint64_t scale2 = pack2(scale, scale);
#pragma unroll
  for (int i = 0; i < 64; i += 2) ffma2(sums2[i / 2], r[i], r[i + 1], scale2);
  stamp_drain(tl, 7, slot0 + E);
  return true;
}

// TOK    capacity in tokens of one tile (TMEM columns per accumulator, rows of a codes stage); the
//        tile actually used, p.tok_tile <= TOK, is chosen per call so the tiles fill the SMs evenly
// kGroup one accumulator per 128-K weight group (fp16 scales [N, K/128]); otherwise one per tile (fp32 [N])
// kEvenOdd codes are stored even-k-first inside each run of 8 (no byte interleave needed when unpacking)
// kDump  also write the exact integer accumulators
// kPre   the weights arrive already unpacked (int8 = 16 w, even-odd k order, from sq_prepack_weights): TMA puts
//        them straight into the operand tile and the unpack warps have nothing to do
template <int TOK, bool kGroup, bool kEvenOdd, bool kDump, typename OutT, bool kTrace = false, bool kPre = false,
          bool kScatter = false, bool kSplit = (TOK <= 64), bool kStatic = false, int kDW = 4>
__global__ void __launch_bounds__(threads_for(kDW), 1)
sq_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_codes, const __grid_constant__ CUtensorMap tmap_packed,
                  const TcParams p) {
  constexpr int S = stages_for(TOK);
  constexpr uint32_t kXBytes = TOK * kBlockK;
  // Each of the four drain warps of a lane quarter owns up to kCols token columns of an accumulator and
  // reads them with ONE tcgen05.ld (a TMEM load costs a few hundred cycles whatever its width, and the
  // loads of one warp do not overlap each other).  While some warps of a scheduler wait for their load,
  // the others convert and accumulate: four warps per scheduler hide the TMEM and barrier round trips.
  constexpr int kCols = TOK / kDW < 16 ? 16 : TOK / kDW;  // 64, 32 or 16 columns per drain warp
  static_assert(kDW == 4 || (kDW == 2 && TOK == 128 && kStatic && !kSplit && !kScatter), "the two-warp drain serves the static form only");
  // TMEM holds a ring of four accumulators so the MMA warp can run ahead of the drain by three groups
  constexpr uint32_t kAccBufs = 4;
  // Channel form: two issuers take alternate K blocks into private accumulators (buffers 2j, 2j + 1 of tile
  // parity j) that the drain adds; one warp's wait / fence / commit round trips per K block (about 570 cycles
  // against 256 of tensor-pipe time) would otherwise bound the kernel.
  constexpr int kMmaWarps = kGroup ? 3 : 2;
  constexpr uint32_t kBufStride = 128;  // TMEM columns between accumulators
  constexpr uint32_t kTmemCols = 512;
  // Two-warp drain: the unpack warps work in pairs on alternate K blocks (each pair the whole block) instead of all
  // four on every block: a warp's chain per block (barrier, loads, unpack, stores, proxy fence, arrive) then has two
  // block times to finish in.
  constexpr bool kUnpackPairs = kDW == 2 && !kPre;
  static_assert(TOK == 128 || TOK == 64 || TOK == 32, "tile capacities");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_ring = smem_base;                  // S x 16 KiB, unpacked weights (UMMA A)
  const uint32_t x_ring = w_ring + S * kWBytes;       // S x TOK*128, codes (UMMA B)
  const uint32_t p_ring = x_ring + S * kXBytes;       // S x 8 KiB, packed weights
  const uint32_t c_tile = p_ring + S * kPackedBytes;  // 16 KiB of 0x80: both operands of the offset MMAs
  const uint32_t bars = c_tile + kConstTileBytes;     // mbarriers, 8 B each
  const uint32_t bar_full = bars;                     // [S] TMA landed (tx bytes)
  const uint32_t bar_wfull = bars + 8 * S;            // [S] converters wrote W[s]
  const uint32_t bar_empty = bars + 16 * S;           // [S] MMAs reading stage s retired
  const uint32_t bar_acc_full = bars + 24 * S;        // [kAccBufs]
  const uint32_t bar_acc_empty = bars + 24 * S + 32;  // [kAccBufs]
  const uint32_t tmem_slot = bars + 24 * S + 64;
  const uint32_t abort_slot = tmem_slot + 4;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_wfull + 8 * s, kPre ? 1 : kUnpackPairs ? kNumConverterWarps / 2 : kNumConverterWarps);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < static_cast<int>(kAccBufs); ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4 * kDW);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_codes);
    tma_prefetch_desc(&tmap_packed);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (kGroup) {
    uint32_t* c_words = reinterpret_cast<uint32_t*>(smem_gen + (c_tile - smem_base));
    for (uint32_t i = threadIdx.x; i < kConstTileBytes / 4; i += blockDim.x) c_words[i] = p.offset_word;
    fence_proxy_async_smem();  // the tensor core reads this tile through the async proxy
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Launched as a programmatic dependent of the pre-pass (sq_linear*), this kernel may become resident while the
  // pre-pass still runs: everything above touches only this CTA's shared and tensor memory.  From here on the
  // codes and row scales are read, so wait for the pre-pass grid (a no-op for an ordinary launch).
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int num_tiles = p.ch_tiles * p.tok_tiles;
  // K is split by the small-tile kernels (few tokens: few tiles) and by a variant of the 128-token kernel built for
  // it; the 128-token kernel that large problems run carries none of that code
  constexpr bool kSplitK = kSplit;
  constexpr bool kWideDrain = kSplit && TOK == 128;
  const int splits = kSplitK ? p.splits : 1;
  const int num_items = num_tiles * splits;
  // a work item is a tile, or one part of a tile's K blocks: [kb0, kb1)
  auto item_range = [&](int item, int& tile, int& kb0, int& kb1) {
    if (kSplitK) {
      tile = item / splits;
      const int part = item - tile * splits;
      kb0 = static_cast<int>(static_cast<int64_t>(part) * p.k_blocks / splits);
      kb1 = static_cast<int>(static_cast<int64_t>(part + 1) * p.k_blocks / splits);
    } else {
      tile = item;
      kb0 = 0;
      kb1 = p.k_blocks;
    }
  };
  const bool tracing = kTrace && blockIdx.x == 0 && p.timeline != nullptr;
  auto stamp = [&](int role, uint32_t slot) {
    if (kTrace && tracing && slot < kTraceSlots) p.timeline[role * kTraceSlots + slot] = clock64();
  };
  const int groups = kGroup ? p.k_blocks : 1;  // of a whole tile: what scale rows and accumulator dumps are indexed by

  if (warp < 4) {
    // ------------------------------------------------------------------ control warpgroup
    reg_dec<regs_control(kWideDrain, kDW)>();
    // Both roles keep the whole warp in the loop and pick the issuing thread with elect.sync: TMA and
    // tcgen05 instructions take warp-uniform operands, and only an elected region lets the compiler keep
    // them in uniform registers (a plain `lane == 0` branch costs about a hundred cycles per instruction).
    if (warp == 0) {
      // TMA producer
      uint32_t it = 0;
      uint32_t s = 0, phase = 0;  // stage of the ring and its phase, as running values
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int tile, kb0, kb1;
        item_range(item, tile, kb0, kb1);
        const int ch0 = (tile % p.ch_tiles) * kBlockCh;
        const int tok0 = (tile / p.ch_tiles) * p.tok_tile;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (!mbar_wait_bounded(bar_empty + 8 * s, phase ^ 1u, abort_flag, kWaitLimitNs)) {
            if (lane == 0) report_timeout(p.status, abort_flag, 9001);
            ok = false;
            break;
          }
          if (elect_one()) {
            stamp(kTrTmaIssue, it);
            // The codes land on the barrier the MMA warps wait on (together with the unpack warps'
            // arrivals), the packed weights on the barrier the unpack warps wait on.  The expect_tx on
            // bar_wfull is issued before the packed load, so no unpack warp can arrive for this phase first.
            if (kPre) {
              // both operand tiles land on the barrier the MMA warps wait on
              mbar_arrive_expect_tx(bar_wfull + 8 * s, static_cast<uint32_t>(p.tok_tile) * kBlockK + kWBytes);
              tma_load_2d(x_ring + s * kXBytes, &tmap_codes, kb * kBlockK, tok0, bar_wfull + 8 * s);
              tma_load_2d(w_ring + s * kWBytes, &tmap_packed, kb * kBlockK, ch0, bar_wfull + 8 * s);
            } else {
              mbar_expect_tx(bar_wfull + 8 * s, static_cast<uint32_t>(p.tok_tile) * kBlockK);
              mbar_arrive_expect_tx(bar_full + 8 * s, kPackedBytes);
              tma_load_2d(x_ring + s * kXBytes, &tmap_codes, kb * kBlockK, tok0, bar_wfull + 8 * s);
              tma_load_2d(p_ring + s * kPackedBytes, &tmap_packed, kb * (kBlockK / 2), ch0, bar_full + 8 * s);
            }
          }
          __syncwarp();
          if (++s == S) {
            s = 0;
            phase ^= 1u;
          }
        }
      }
    } else if (warp <= kMmaWarps) {
      // MMA issuers.  Group mode: warps 1..3 take the groups round-robin (a group is one K block with its
      // own accumulator), so the barrier round trips of one group overlap the issue of the next two.
      // Channel mode: warp 1 alone, because all K blocks of a tile add into one accumulator in order.
      const uint32_t mine = static_cast<uint32_t>(warp - 1);
      if constexpr (kGroup) {
        // Group form.  An issuer's own chain per group - two barrier round trips, the issue, the loop around it - has
        // three group times to finish in, and on a scheduler it shares with drain warps in long runs of arithmetic
        // every instruction of it waits its turn: the loop steps from one of its groups straight to the next, with
        // the group's stage and accumulator (and their barrier phases) as running values, and issues the offset MMA,
        // the four MMAs and both commits in one elected region.
        uint32_t git = mine;                 // this issuer's next group, counted over all work items of the thread block
        uint32_t s = mine, phase = 0;        // its stage of the load ring (mine < 3 <= S)
        uint32_t buf = mine, aphase = 0;     // its accumulator of the ring of four
        uint32_t base = 0;                   // groups of the items before this one
        bool ok = true;
        const uint64_t desc_c = umma_desc_k128(c_tile);
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
          int tile, kb0, kb1;
          item_range(item, tile, kb0, kb1);
          const uint32_t end = base + static_cast<uint32_t>(kb1 - kb0);
          if (git < end) {
            const int tok0 = (tile / p.ch_tiles) * p.tok_tile;
            const int64_t left = p.M - tok0;
            const int tok_count = left < p.tok_tile ? static_cast<int>(left) : p.tok_tile;
            const uint32_t umma_n = static_cast<uint32_t>((tok_count + 15) & ~15);
            const uint32_t idesc = umma_idesc_i8(kBlockCh, umma_n);
            // codes of any int8 value: ONE unsigned x unsigned MMA of 0xFF bytes adds 32 * 255 * 255, which covers
            // the most negative group sum (16 * 8 * 127 * 128); codes within [-8, 7]: one signed MMA of 0x40 bytes
            const uint32_t idesc_offset = p.offset_unsigned != 0 ? umma_idesc_u8(kBlockCh, umma_n) : idesc;
            for (; git < end; git += 3) {
              if (lane == 0) stamp(kTrIssuerWaits, git);
              if (!mbar_wait_bounded(bar_acc_empty + 8 * buf, aphase, abort_flag, kWaitLimitNs)) {
                if (lane == 0) report_timeout(p.status, abort_flag, 9002);
                ok = false;
                break;
              }
              if (lane == 0) stamp(kTrMmaAccFree, git);
              if (!mbar_wait_bounded(bar_wfull + 8 * s, phase, abort_flag, kWaitLimitNs)) {
                if (lane == 0) report_timeout(p.status, abort_flag, 9003);
                ok = false;
                break;
              }
              tc_fence_after_sync();
              if (lane == 0) stamp(kTrMmaIssue, git);
              if (elect_one()) {
                const uint32_t tmem_d = tmem_base + buf * kBufStride;
                // the offset MMA starts the accumulator at a positive value (no operand from the pipeline)
                umma_i8(tmem_d, desc_c, desc_c, idesc_offset, 0u);
                const uint64_t desc_a = umma_desc_k128(w_ring + s * kWBytes);
                const uint64_t desc_b = umma_desc_k128(x_ring + s * kXBytes);
#pragma unroll
                for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                  // advancing K by 32 bytes inside the 128-byte swizzle row: +2 in the (address >> 4) field
                  umma_i8(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, 1u);
                }
                umma_commit(bar_empty + 8 * s);        // frees the stage when these MMAs retire
                umma_commit(bar_acc_full + 8 * buf);   // and hands the accumulator to the drain
              }
              __syncwarp();
              if (lane == 0) stamp(kTrMmaCommitted, git);
              s += 3;
              if (s >= static_cast<uint32_t>(S)) {
                s -= S;
                phase ^= 1u;
              }
              if (buf == 0) {
                buf = 3;
              } else {
                buf -= 1;
                aphase ^= 1u;
              }
            }
          }
          base = end;
        }
      } else {
      uint32_t it = 0, git = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int tile, kb0, kb1;
        item_range(item, tile, kb0, kb1);
        const int groups = kGroup ? kb1 - kb0 : 1;
        const int blocks_per_group = kGroup ? 1 : kb1 - kb0;
        const int tok0 = (tile / p.ch_tiles) * p.tok_tile;
        const int64_t left = p.M - tok0;
        const int tok_count = left < p.tok_tile ? static_cast<int>(left) : p.tok_tile;
        const uint32_t umma_n = static_cast<uint32_t>((tok_count + 15) & ~15);
        const uint32_t idesc = umma_idesc_i8(kBlockCh, umma_n);
        for (int g = 0; g < groups && ok; ++g, ++git) {
          if (kGroup && git % kMmaWarps != mine) {
            it += blocks_per_group;
            continue;
          }
          const uint32_t split = (kGroup || blocks_per_group < 2) ? 1u : static_cast<uint32_t>(p.mma_split);
          if (!kGroup && mine >= split) {
            it += blocks_per_group;
            continue;
          }
          // channel form: tile parity picks the buffer pair, the issuer its half of it
          const uint32_t buf = kGroup ? git % kAccBufs : (git & 1u) * 2u + mine;
          const uint32_t aphase = kGroup ? (git / kAccBufs) & 1u : (git >> 1) & 1u;
          if (lane == 0) stamp(kTrIssuerWaits, git);
          if (!mbar_wait_bounded(bar_acc_empty + 8 * buf, aphase, abort_flag, kWaitLimitNs)) {
            if (lane == 0) report_timeout(p.status, abort_flag, 9002);
            ok = false;
            break;
          }
          if (lane == 0) stamp(kTrMmaAccFree, git);
          const uint32_t tmem_d = tmem_base + buf * kBufStride;
#ifdef SQ_TC_NO_OFFSET
          if (false) {
#else
          if (kGroup) {
#endif
            // the offset MMAs need no operand from the pipeline: they start the accumulator at a positive value
            tc_fence_after_sync();
            if (elect_one()) {
              const uint64_t desc_c = umma_desc_k128(c_tile);
              // codes of any int8 value: ONE unsigned x unsigned MMA of 0xFF bytes adds 32 * 255 * 255, which covers
              // the most negative group sum (16 * 8 * 127 * 128); codes within [-8, 7]: one signed MMA of 0x40 bytes
              umma_i8(tmem_d, desc_c, desc_c, p.offset_unsigned != 0 ? umma_idesc_u8(kBlockCh, umma_n) : idesc, 0u);
            }
            __syncwarp();
          }
          for (int kb = 0; kb < blocks_per_group; ++kb, ++it) {
            if (!kGroup && static_cast<uint32_t>(kb) % split != mine) continue;  // the other issuer's block
            const uint32_t s = it % S, phase = (it / S) & 1u;
            if (!mbar_wait_bounded(bar_wfull + 8 * s, phase, abort_flag, kWaitLimitNs)) {
              if (lane == 0) report_timeout(p.status, abort_flag, 9003);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (lane == 0) stamp(kTrMmaIssue, it);
            if (elect_one()) {
              const uint64_t desc_a = umma_desc_k128(w_ring + s * kWBytes);
              const uint64_t desc_b = umma_desc_k128(x_ring + s * kXBytes);
#pragma unroll
              for (int k = 0; k < kBlockK / kUmmaK; ++k) {
#ifdef SQ_TC_NO_OFFSET
                const uint32_t accumulate = k > 0 ? 1u : 0u;
#else
                const uint32_t accumulate = (kGroup || static_cast<uint32_t>(kb) >= split || k > 0) ? 1u : 0u;
#endif
                // advancing K by 32 bytes inside the 128-byte swizzle row: +2 in the (address >> 4) field
                umma_i8(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, accumulate);
              }
              umma_commit(bar_empty + 8 * s);  // frees the stage when these MMAs retire
              // after this issuer's last block of the accumulator
              if (static_cast<uint32_t>(kb) + split >= static_cast<uint32_t>(blocks_per_group))
                umma_commit(bar_acc_full + 8 * buf);
            }
            __syncwarp();
          }
          if (lane == 0) stamp(kTrMmaCommitted, git);
        }
      }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ converter warpgroup
    reg_dec<regs_unpack(kWideDrain, kDW)>();
    // kUnpackPairs: 64 threads per K block, eight 16-byte units each; otherwise 128 threads, four units each
    constexpr int kUnits = kUnpackPairs ? 8 : 4;
    constexpr uint32_t kStep = kUnpackPairs ? 2u : 1u;           // K blocks between two blocks of this warp
    const int ctid = kUnpackPairs ? (threadIdx.x - 128) & 63 : threadIdx.x - 128;
    const uint32_t pair = kUnpackPairs ? static_cast<uint32_t>(threadIdx.x - 128) >> 6 : 0u;
    uint32_t it = 0;
    // stage of the ring and its phase, kept as running values (a division by the stage count per block is a
    // dozen instructions on a warp whose time per block bounds the packed form)
    uint32_t s = pair, phase = 0;
    bool ok = true;
    bool stage_ready = false;  // an early probe saw the coming stage's packed weights landed
    // what does not change from block to block: this thread's 16-byte units of the packed tile and where their
    // unpacked halves go inside the swizzled operand tile (the swizzle only looks at the row's low bits)
    const uint32_t src_off = static_cast<uint32_t>(ctid) * 16u;
    const uint32_t row0 = static_cast<uint32_t>(ctid >> 2), c0 = static_cast<uint32_t>(ctid & 3);
    const uint32_t dst_off_a = row0 * 128u + (((2u * c0) ^ (row0 & 7u)) << 4);
    const uint32_t dst_off_b = row0 * 128u + (((2u * c0 + 1u) ^ (row0 & 7u)) << 4);
    constexpr uint32_t kSrcStride = kUnpackPairs ? 1024u : 2048u;  // between a thread's units: 64 or 128 units on
    constexpr uint32_t kDstStride = kUnpackPairs ? 2048u : 4096u;  // 16 or 32 rows on
    for (int item = blockIdx.x; !kPre && item < num_items && ok; item += gridDim.x) {
      int tile, kb0, kb1;
      item_range(item, tile, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        if (kUnpackPairs && (it & 1u) != pair) continue;  // the other pair's block
        if (!(SQ_TC_EARLY_PROBE && stage_ready) && !mbar_wait_bounded(bar_full + 8 * s, phase, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9004);
          ok = false;
          break;
        }
        if (ctid == 0) stamp(kTrConvStart, it);
        const uint32_t src = p_ring + s * kPackedBytes;
        const uint32_t dst = w_ring + s * kWBytes;
        const uint32_t s_next = s + kStep >= S ? s + kStep - S : s + kStep, phase_next = s + kStep >= S ? phase ^ 1u : phase;
#pragma unroll
        for (int half = 0; half < kUnits / 4; ++half) {
          // four 16-byte loads first, then the unpack and the eight stores: the loads overlap
          uint32_t win[4][4];
#pragma unroll
          for (int u4 = 0; u4 < 4; ++u4) {
            // unit (4 half + u4) * threads + ctid: 16 packed bytes = 32 k of one channel row
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(win[u4][0]), "=r"(win[u4][1]), "=r"(win[u4][2]), "=r"(win[u4][3])
                         : "r"(src + src_off + (4 * half + u4) * kSrcStride));
          }
          // the next stage's barrier is probed under this stage's work (a probe takes over a hundred cycles)
          if (SQ_TC_EARLY_PROBE && half == 0) stage_ready = mbar_test_wait(bar_full + 8 * s_next, phase_next);
#pragma unroll
          for (int u4 = 0; u4 < 4; ++u4) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t lo = (win[u4][i] << 4) & 0xF0F0F0F0u;  // 16 * nibble of even k, as int8
              const uint32_t hi = win[u4][i] & 0xF0F0F0F0u;         // 16 * nibble of odd k
              if (kEvenOdd) {
                o[2 * i] = lo;
                o[2 * i + 1] = hi;
              } else {
                o[2 * i] = __byte_perm(lo, hi, 0x5140);      // k0 k1 k2 k3
                o[2 * i + 1] = __byte_perm(lo, hi, 0x7362);  // k4 k5 k6 k7
              }
            }
            // the same place inside the swizzle atom, kDstStride further on per unit
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + dst_off_a + (4 * half + u4) * kDstStride),
                         "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]));
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + dst_off_b + (4 * half + u4) * kDstStride),
                         "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]));
          }
        }
        fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_wfull + 8 * s);
        if (ctid == 0) stamp(kTrConvDone, it);
        s = s_next;
        phase = phase_next;
      }
    }
  } else {
    // ------------------------------------------------------------------ drain warpgroups
    reg_inc<regs_drain(kWideDrain, kDW)>();
    const int dwarp = warp - 8;           // 0..4 kDW - 1
    const int quarter = warp & 3;         // TMEM lane quarter this warp may address
    const int slice = dwarp >> 2;         // which slice of the token columns (kDW warps per lane quarter)
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int ch_in_tile = quarter * 32 + lane;

    // hand every accumulator of the ring to the MMA warp
    const int my_col0 = slice * p.slice_cols;  // first token column of this warp inside a tile
#pragma unroll
    for (int b = 0; b < static_cast<int>(kAccBufs); ++b) {
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * b);
    }
    const __half* scale_row = static_cast<const __half*>(p.w_scales);
    const uint32_t offset_bits = kGroup ? p.offset_bits : 0u;
    const float offset_float = __uint_as_float(offset_bits);

    uint32_t git = 0;
    bool ok = true;
    bool acc_ready = false;  // an early probe saw the coming group's accumulator complete
    // two-warp drain: the sums of the tile before, finalized under the first groups of the tile in hand
    PendingTile<OutT> pending;
    pending.cols = 0;
    pending.out = static_cast<OutT*>(p.out);
#pragma unroll
    for (int i = 0; i < 32; ++i) pending.pairs[i] = 0u;
    const uint32_t rs_table = bars + 256 + static_cast<uint32_t>(dwarp & 7) * 256u;  // this warp's 64 row scales
    // the first two chunks of group scales of the coming tile, requested a tile ahead (a global load in front of a
    // tile's first group would hold up every role of the pipeline)
    uint4 ahead_chunk = make_uint4(0u, 0u, 0u, 0u), ahead_chunk_next = make_uint4(0u, 0u, 0u, 0u);
    // without a K split a work item is a tile and the next one lies gridDim.x tiles on: channel tile and token tile
    // as running values (two integer divisions per tile sit in front of the tile's first group otherwise)
    int ch_idx = static_cast<int>(blockIdx.x) % p.ch_tiles, tok_idx = static_cast<int>(blockIdx.x) / p.ch_tiles;
    const int step_ch = static_cast<int>(gridDim.x) % p.ch_tiles, step_tok = static_cast<int>(gridDim.x) / p.ch_tiles;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      int tile, kb0, kb1;
      item_range(item, tile, kb0, kb1);
      const int g0 = kGroup ? kb0 : 0, g1 = kGroup ? kb1 : 1;  // this item's groups
      const int ch0 = (kSplitK ? tile % p.ch_tiles : ch_idx) * kBlockCh;
      const int tok0 = (kSplitK ? tile / p.ch_tiles : tok_idx) * p.tok_tile;
      // the coming tile's coordinates
      const int ch_ahead = ch_idx + step_ch >= p.ch_tiles ? ch_idx + step_ch - p.ch_tiles : ch_idx + step_ch;
      tok_idx += step_tok + (ch_idx + step_ch >= p.ch_tiles ? 1 : 0);
      ch_idx = ch_ahead;
      const int64_t left = p.M - tok0;
      const int tok_count = left < p.tok_tile ? static_cast<int>(left) : p.tok_tile;
      const int my_cols = min(max(tok_count - my_col0, 0), p.slice_cols);  // real tokens in my slice
      const int64_t n = ch0 + ch_in_tile;
      const bool n_ok = n < p.N;
      // what the finalize needs from global memory is requested now, a whole tile ahead of its use: lane i keeps the
      // row scale of column i of this warp's slice (group form: times 2^-49, see kScaleDown), every lane its bias
      const int64_t m0 = tok0 + my_col0;
      float* part_out = kSplitK && splits > 1
                            ? p.partials + (static_cast<int64_t>(item) * p.tok_tile + my_col0) * kBlockCh + ch_in_tile
                            : nullptr;
      float my_rs[kCols > 32 ? 2 : 1];
#pragma unroll
      for (int h = 0; h < (kCols > 32 ? 2 : 1); ++h) {
        my_rs[h] = 32 * h + lane < my_cols ? __ldg(p.row_scales + m0 + 32 * h + lane) : 0.0f;
        if (kGroup) my_rs[h] = __fmul_rn(my_rs[h], kScaleDown);
      }
      const bool has_bias = p.bias != nullptr;
      const float bias = has_bias && n_ok ? to_float<OutT>(__ldg(static_cast<const OutT*>(p.bias) + n)) : 0.0f;
      const float wscale = !kGroup && n_ok ? __ldg(static_cast<const float*>(p.w_scales) + n) : 1.0f;

      // group form: packed pairs (columns 2i, 2i + 1); channel form: plain floats.  (A packed f32x2 FMA issues at
      // half the rate of a scalar one, so it buys no arithmetic throughput, only fewer instructions: measured 4 %
      // faster than 32 scalar FFMAs.)
      uint64_t sums2[kGroup ? kCols / 2 : 1];
      float sums[kGroup ? 1 : kCols];
#pragma unroll
      for (int i = 0; i < (kGroup ? kCols / 2 : 1); ++i) sums2[i] = 0ull;
#pragma unroll
      for (int i = 0; i < (kGroup ? 1 : kCols); ++i) sums[i] = 0.0f;
      float offset_sum = 0.0f;  // what the constant offsets added to every sum of this channel

      // Group scales: chunks of eight (one 16-byte load), the next chunk requested a whole chunk ahead, so no global
      // load latency sits on the per-group path; other group counts use scalar loads two groups ahead.
      const unsigned short* my_scales = reinterpret_cast<const unsigned short*>(scale_row) + (n_ok ? n : 0) * groups;
      const bool scale_vectors = kGroup && (groups & 7) == 0 && (reinterpret_cast<uintptr_t>(p.w_scales) & 15u) == 0;
      uint4 chunk = make_uint4(0u, 0u, 0u, 0u), chunk_next = make_uint4(0u, 0u, 0u, 0u);
      unsigned short raw_a = 0, raw_b = 0;
      if (kGroup) {
        if (kStatic && kDW == 2 && item != static_cast<int>(blockIdx.x)) {
          chunk = ahead_chunk;
          chunk_next = ahead_chunk_next;
        } else if (scale_vectors) {
          chunk = __ldg(reinterpret_cast<const uint4*>(my_scales) + (g0 >> 3));
          if (8 * ((g0 >> 3) + 1) < groups) chunk_next = __ldg(reinterpret_cast<const uint4*>(my_scales) + (g0 >> 3) + 1);
          {
            // the scale in use is always the lowest half of `chunk`: drop the halves in front of group g0
            for (int skip = 0; skip < (g0 & 7); ++skip) {
              chunk.x = __funnelshift_r(chunk.x, chunk.y, 16);
              chunk.y = __funnelshift_r(chunk.y, chunk.z, 16);
              chunk.z = __funnelshift_r(chunk.z, chunk.w, 16);
              chunk.w >>= 16;
            }
          }
        } else {
          // raw_a holds the scale of the next even group, raw_b of the next odd one
          const unsigned short first = __ldg(my_scales + g0);
          const unsigned short second = g0 + 1 < groups ? __ldg(my_scales + g0 + 1) : static_cast<unsigned short>(0);
          raw_a = (g0 & 1) == 0 ? first : second;
          raw_b = (g0 & 1) == 0 ? second : first;
        }
      }

      if constexpr (kStatic && kDW == 2) {
        long long* trace_to = kTrace && tracing ? p.timeline : nullptr;
        {
          // (past the last tile this reads some tile's scales again: always a valid address, never used)
          const int64_t n_ahead = ch_ahead * kBlockCh + ch_in_tile;
          const uint4* scales_ahead = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(scale_row) +
                                                                     (n_ahead < p.N ? n_ahead : 0) * groups);
          ahead_chunk = __ldg(scales_ahead);
          ahead_chunk_next = __ldg(scales_ahead + (groups > 8 ? 1 : 0));
        }
        stamp_drain(trace_to, kTrTileEnds, 4 * (git / groups) + 2);  // the tile's head is done
        if (my_cols > 0) {
          const uint32_t phase = (git >> 2) & 1u;
          const uint32_t tmem_slice = tmem_base + lane_addr + my_col0;
          int g = g0;
#define SQ_DRAIN_FIRST(E)                                                                                               \
  drain_group_first<E, OutT>(bar_acc_full, bar_acc_empty, tmem_slice, phase, abort_flag, lane, acc_ready, chunk, chunk_next, \
                             my_scales, groups, g, offset_float, offset_sum, sums2, pending, p.out_ld, trace_to, git)
#define SQ_DRAIN_AT(E)                                                                                                   \
  drain_group_static<E, kCols>(bar_acc_full, bar_acc_empty, tmem_slice, phase, abort_flag, lane, acc_ready, chunk, chunk_next, \
                               my_scales, groups, g, offset_float, offset_sum, sums2, trace_to, git)
          ok = SQ_DRAIN_FIRST(0u) && SQ_DRAIN_FIRST(1u) && SQ_DRAIN_FIRST(2u) && SQ_DRAIN_FIRST(3u) && SQ_DRAIN_FIRST(4u) &&
               SQ_DRAIN_FIRST(5u) && SQ_DRAIN_FIRST(6u) && SQ_DRAIN_FIRST(7u);
          git += 8;
          for (g = g0 + 8; g < g1 && ok; g += 8, git += 8) {
            ok = SQ_DRAIN_AT(0u) && SQ_DRAIN_AT(1u) && SQ_DRAIN_AT(2u) && SQ_DRAIN_AT(3u) && SQ_DRAIN_AT(4u) &&
                 SQ_DRAIN_AT(5u) && SQ_DRAIN_AT(6u) && SQ_DRAIN_AT(7u);
          }
#undef SQ_DRAIN_AT
#undef SQ_DRAIN_FIRST
        } else {
          // no columns of this tile (past the last token): store what is pending, keep the hand-over going
          store_pending<0, 64, OutT>(pending, p.out_ld);
          for (int g = g0; g < g1 && ok; ++g, ++git) {
            const uint32_t buf = git & 3u;
            ok = mbar_wait_bounded(bar_acc_full + 8 * buf, (git >> 2) & 1u, abort_flag, kWaitLimitNs);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
          }
          acc_ready = false;
        }
        if (!ok) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9005);
          break;
        }
        // this tile's results: scaled and cast now, stored under the next tile's first groups
        stamp_drain(trace_to, kTrTileEnds, 4 * (git / groups) - 4);  // the last group is done
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(rs_table + 4 * lane), "f"(my_rs[0]) : "memory");
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(rs_table + 128 + 4 * lane), "f"(my_rs[kCols > 32 ? 1 : 0]) : "memory");
        __syncwarp();
        finish_tile<OutT>(pending, sums2, offset_sum, bias, p.bias != nullptr, rs_table);
        __syncwarp();
        pending.out = static_cast<OutT*>(p.out) + m0 * p.out_ld + p.out_col0 + (n_ok ? n : 0);
        pending.cols = n_ok ? my_cols : 0;
        stamp_drain(trace_to, kTrTileEnds, 4 * (git / groups) - 3);  // scaled and cast
        continue;
      } else if constexpr (kStatic) {
        // The launcher picks this variant when every tile has a multiple of eight groups in chunked scales and K is
        // not split: eight groups (one chunk of scales) per round, each with its place in the chunk and in the
        // accumulator ring a compile-time constant.
        // The instructions a drain warp spends per group are what bounds this kernel.
        if (my_cols > 0) {
          const uint32_t phase = (git >> 2) & 1u;  // git is a multiple of eight at every round: the same parity each time
          const uint32_t tmem_slice = tmem_base + lane_addr + my_col0;
#define SQ_DRAIN_AT(E)                                                                                                   \
  drain_group_static<E, kCols>(bar_acc_full, bar_acc_empty, tmem_slice, phase, abort_flag, lane, acc_ready, chunk, chunk_next, \
                               my_scales, groups, g, offset_float, offset_sum, sums2)
          for (int g = g0; g < g1 && ok; g += 8, git += 8) {
            ok = SQ_DRAIN_AT(0u) && SQ_DRAIN_AT(1u) && SQ_DRAIN_AT(2u) && SQ_DRAIN_AT(3u) && SQ_DRAIN_AT(4u) &&
                 SQ_DRAIN_AT(5u) && SQ_DRAIN_AT(6u) && SQ_DRAIN_AT(7u);
          }
#undef SQ_DRAIN_AT
        } else {
          // a warp whose columns lie beyond the tile's tokens only keeps the accumulator hand-over going
          for (int g = g0; g < g1 && ok; ++g, ++git) {
            const uint32_t buf = git & 3u;
            ok = mbar_wait_bounded(bar_acc_full + 8 * buf, (git >> 2) & 1u, abort_flag, kWaitLimitNs);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
          }
          acc_ready = false;
        }
        if (!ok && lane == 0) report_timeout(p.status, abort_flag, 9005);
      }
      if constexpr (!kStatic)
      for (int g = g0; g < g1 && ok; ++g, ++git) {
        // channel form: the tile's accumulator pair (2j, 2j + 1), the second in use when the issuers split K
        const uint32_t buf = kGroup ? git % kAccBufs : (git & 1u) * 2u;
        const uint32_t aphase = kGroup ? (git / kAccBufs) & 1u : (git >> 1) & 1u;
        const bool split = !kGroup && p.mma_split == 2 && kb1 - kb0 >= 2;
        float scale = 0.0625f;  // the unpacked weights are 16 x the int4 value
        if (threadIdx.x == 256) stamp(kTrDrainWaits, git);
        // (group form: usually the probe made during the previous group already saw this barrier complete)
        if (!(kGroup && SQ_TC_EARLY_PROBE && acc_ready) &&
            !mbar_wait_bounded(bar_acc_full + 8 * buf, aphase, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9005);
          ok = false;
          break;
        }
        if (split && !mbar_wait_bounded(bar_acc_full + 8 * (buf + 1), aphase, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9005);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (threadIdx.x == 256) stamp(kTrDrainStart, git);
        uint32_t r[kCols];
        const uint32_t taddr = tmem_base + lane_addr + buf * kBufStride + my_col0;
        if (my_cols > 0) {
          tmem_ld_chunk(taddr, r);
          if (!kGroup) {
            if (split) {
              uint32_t other[kCols];
              tmem_ld_chunk(taddr + kBufStride, other);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < kCols; ++i) r[i] += other[i];  // exact: int32 partial sums of disjoint K blocks
            } else {
              tmem_wait_ld();
            }
          }
        }
        // A probe of an mbarrier takes over a hundred cycles to answer even when the phase is long complete: the
        // next group's barrier is probed now, under the load, instead of in front of the next load.
        if (kGroup && SQ_TC_EARLY_PROBE)
          acc_ready = mbar_test_wait(bar_acc_full + 8 * ((git + 1) % kAccBufs), ((git + 1) / kAccBufs) & 1u);
        // the scale of this group is picked while the load is in flight
        if (kGroup) {
          unsigned short raw;
          if (scale_vectors) {
            // the lowest half of the chunk is this group's scale; the chunk then moves down by one half (four
            // funnel shifts instead of picking a half out of four registers by the group index)
            raw = static_cast<unsigned short>(chunk.x & 0xFFFFu);
            if ((g & 7) == 7) {
              chunk = chunk_next;  // (the chunk after that is requested below, after the hand-back)
            } else {
              chunk.x = __funnelshift_r(chunk.x, chunk.y, 16);
              chunk.y = __funnelshift_r(chunk.y, chunk.z, 16);
              chunk.z = __funnelshift_r(chunk.z, chunk.w, 16);
              chunk.w >>= 16;
            }
          } else {
            raw = (g & 1) == 0 ? raw_a : raw_b;
          }
          scale = __half2float(__ushort_as_half(raw)) * kScaleUp;
          offset_sum = fmaf(offset_float, scale, offset_sum);
        }
        if (kGroup && my_cols > 0) tmem_wait_ld();
        // the accumulator is in registers: give it back before doing the arithmetic
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar_acc_empty + 8 * buf);
          if (!kGroup) mbar_arrive(bar_acc_empty + 8 * (buf + 1));  // kept in step even when unused
        }
        if (threadIdx.x == 256) stamp(kTrDrainRelease, git);
        if (kGroup) {
          // the coming scales are requested after the hand-back: the arrive is a release, and a global load issued
          // before it would make it wait for the load
          if (scale_vectors) {
            const int c2 = (g >> 3) + 2;
            if ((g & 7) == 7 && 8 * c2 < groups) chunk_next = __ldg(reinterpret_cast<const uint4*>(my_scales) + c2);
          } else if (g + 2 < groups) {
            const unsigned short ahead = __ldg(my_scales + g + 2);
            if ((g & 1) == 0) raw_a = ahead; else raw_b = ahead;
          }
        }
        if (my_cols > 0) {
          const uint64_t scale2 = pack2(scale, scale);
#pragma unroll
          for (int i = 0; i < kCols; i += 2) {
            // group mode: the accumulator is positive and below 2^23, so its bit pattern read as a float is the
            // denormal acc * 2^-149 and the FFMA takes it as it is (a conversion instruction runs at a sixteenth
            // of the rate); two columns go through one packed FFMA
            if (kGroup) {
              ffma2(sums2[kGroup ? i / 2 : 0], r[i], r[i + 1], scale2);
            } else {
              sums[kGroup ? 0 : i] = fmaf(static_cast<float>(static_cast<int32_t>(r[i])), scale, sums[kGroup ? 0 : i]);
              sums[kGroup ? 0 : i + 1] =
                  fmaf(static_cast<float>(static_cast<int32_t>(r[i + 1])), scale, sums[kGroup ? 0 : i + 1]);
            }
          }
          if (kDump) {
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
              if (n_ok && i < my_cols) {
                const int64_t m = tok0 + my_col0 + i;
                p.acc_dump[(m * p.N + n) * groups + g] = static_cast<int32_t>(r[i] - offset_bits) >> 4;
              }
            }
          }
          if (kSplitK && !kGroup && splits > 1) {
            // channel form under a K split: the parts exchange the exact int32 accumulators
#pragma unroll
            for (int i = 0; i < kCols; ++i)
              if (i < my_cols) part_out[i * kBlockCh] = __uint_as_float(r[i]);
          }
        }
        if (threadIdx.x == 256) stamp(kTrDrainDone, git);
      }
      if (!ok) break;

      if (kSplitK && splits > 1) {
        // K split: leave this part's sums, take a ticket at the tile's counter; the last of the `splits` parts adds
        // all of them in part order (so the result does not depend on which part came last) and goes on to finalize.
        // Nobody waits for anybody.  Warps without columns of this tile (my_cols == 0) have nothing to do in any part.
        if (my_cols == 0) continue;
        if (kGroup) {
#pragma unroll
          for (int i = 0; i < kCols; ++i) {
            const float2 pair = unpack2(sums2[kGroup ? i / 2 : 0]);
            if (i < my_cols) part_out[i * kBlockCh] = __fsub_rn((i & 1) != 0 ? pair.y : pair.x, offset_sum);
          }
        }
        __threadfence();
        __syncwarp();
        unsigned long long before = 0ull;
        if (lane == 0) before = atomicAdd(p.counters + tile, 1ull << (4 * dwarp));
        before = __shfl_sync(0xffffffffu, before, 0);
        if (static_cast<int>((before >> (4 * dwarp)) & 15ull) != splits - 1) continue;  // another part finalizes
        __threadfence();
        if (lane == 0) atomicAdd(p.counters + tile, ~(static_cast<unsigned long long>(splits) << (4 * dwarp)) + 1ull);
        const float* part_in = p.partials + (static_cast<int64_t>(tile) * splits * p.tok_tile + my_col0) * kBlockCh + ch_in_tile;
        if (kGroup) {
          if constexpr (kCols > 16) {
            // wide slices: no room for a second set of loads in flight; the 32 loads of one part still overlap
            float total[kCols];
#pragma unroll
            for (int i = 0; i < kCols; ++i) total[i] = 0.0f;
            for (int part = 0; part < splits; ++part) {
#pragma unroll
              for (int i = 0; i < kCols; ++i)
                if (i < my_cols)
                  total[i] = __fadd_rn(total[i], __ldcg(part_in + (static_cast<int64_t>(part) * p.tok_tile + i) * kBlockCh));
            }
#pragma unroll
            for (int i = 0; i < kCols; i += 2) sums2[kGroup ? i / 2 : 0] = pack2(total[i], total[i + 1]);
            offset_sum = 0.0f;
          } else {
          // the loads of the next part are in flight while this part is added (parts are added in part order)
          float total[kCols], ahead[kCols];
#pragma unroll
          for (int i = 0; i < kCols; ++i) {
            total[i] = 0.0f;
            ahead[i] = i < my_cols ? __ldcg(part_in + static_cast<int64_t>(i) * kBlockCh) : 0.0f;
          }
          for (int part = 0; part < splits; ++part) {
            float now[kCols];
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
              now[i] = ahead[i];
              if (part + 1 < splits && i < my_cols)
                ahead[i] = __ldcg(part_in + (static_cast<int64_t>(part + 1) * p.tok_tile + i) * kBlockCh);
            }
#pragma unroll
            for (int i = 0; i < kCols; ++i) total[i] = __fadd_rn(total[i], now[i]);
          }
#pragma unroll
          for (int i = 0; i < kCols; i += 2) sums2[kGroup ? i / 2 : 0] = pack2(total[i], total[i + 1]);
          offset_sum = 0.0f;
          }
        } else if constexpr (kCols > 16) {
          int32_t total[kCols];
#pragma unroll
          for (int i = 0; i < kCols; ++i) total[i] = 0;
          for (int part = 0; part < splits; ++part) {
#pragma unroll
            for (int i = 0; i < kCols; ++i)
              if (i < my_cols)
                total[i] += static_cast<int32_t>(__float_as_uint(__ldcg(part_in + (static_cast<int64_t>(part) * p.tok_tile + i) * kBlockCh)));
          }
#pragma unroll
          for (int i = 0; i < kCols; ++i) sums[kGroup ? 0 : i] = static_cast<float>(total[i]) * 0.0625f;
        } else {
          int32_t total[kCols];
          float ahead[kCols];
#pragma unroll
          for (int i = 0; i < kCols; ++i) {
            total[i] = 0;
            ahead[i] = i < my_cols ? __ldcg(part_in + static_cast<int64_t>(i) * kBlockCh) : 0.0f;
          }
          for (int part = 0; part < splits; ++part) {
            float now[kCols];
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
              now[i] = ahead[i];
              if (part + 1 < splits && i < my_cols)
                ahead[i] = __ldcg(part_in + (static_cast<int64_t>(part + 1) * p.tok_tile + i) * kBlockCh);
            }
#pragma unroll
            for (int i = 0; i < kCols; ++i) total[i] += static_cast<int32_t>(__float_as_uint(now[i]));
          }
#pragma unroll
          for (int i = 0; i < kCols; ++i) sums[kGroup ? 0 : i] = static_cast<float>(total[i]) * 0.0625f;
        }
      }

      // finalize: row scale, bias, gate, residual, cast, store.  Lanes hold consecutive channels -> 64 B per
      // warp store.  (A version that transposed the block through shared memory to store 16-byte vectors along
      // the channel axis measured 30 % slower end to end and was dropped.)  The row scale of column i was loaded by
      // lane i when the tile began and comes over by shuffle, so no global load sits in front of the stores; the
      // shuffles run in every lane, whether or not its channel exists.
      const bool plain = p.gate == nullptr && p.residual == nullptr;
      const bool store_ok = n_ok;
      OutT* out = static_cast<OutT*>(p.out) + m0 * p.out_ld + p.out_col0 + (n_ok ? n : 0);
      if (threadIdx.x == 256) stamp(kTrTileEnds, 2 * (git / groups) - 2);  // finalize begins / has ended
      if (plain) {
        // the common case is kept apart from the fused forms: a short straight run of instructions per column
#pragma unroll
        for (int i = 0; i < kCols; ++i) {
          const float rs = __shfl_sync(0xffffffffu, my_rs[i >> 5], i & 31);
          float y;
          if (kGroup) {
            const float2 pair = unpack2(sums2[kGroup ? i / 2 : 0]);
            y = __fmul_rn(__fsub_rn((i & 1) != 0 ? pair.y : pair.x, offset_sum), rs);
          } else {
            y = __fmul_rn(__fmul_rn(sums[kGroup ? 0 : i], rs), wscale);
          }
          if (has_bias) y = __fadd_rn(y, bias);
          if (store_ok && i < my_cols) {
            const OutT value = from_float<OutT>(y);
            *out = value;
            if (kScatter) {
              // the same 64 bytes per warp to the other GPUs' matrices: plain stores through peer pointers
              for (int d = 0; d < p.n_more; ++d) out[p.more_delta[d]] = value;
            }
          }
          out += p.out_ld;
        }
      } else {
        // gate rows change every gate_span tokens: one division for the first column, then a running remainder
        int64_t gate_row = m0 / p.gate_span;
        int64_t gate_left = p.gate_span - m0 % p.gate_span;  // columns before the next gate row
        const OutT* gate = p.gate != nullptr ? static_cast<const OutT*>(p.gate) + gate_row * p.gate_row_stride + (n_ok ? n : 0) : nullptr;
        const OutT* residual = p.residual != nullptr ? static_cast<const OutT*>(p.residual) + m0 * p.N + (n_ok ? n : 0) : nullptr;
#pragma unroll
        for (int i = 0; i < kCols; ++i) {
          const float rs = __shfl_sync(0xffffffffu, my_rs[i >> 5], i & 31);
          float y;
          if (kGroup) {
            const float2 pair = unpack2(sums2[kGroup ? i / 2 : 0]);
            y = __fmul_rn(__fsub_rn((i & 1) != 0 ? pair.y : pair.x, offset_sum), rs);
          } else {
            y = __fmul_rn(__fmul_rn(sums[kGroup ? 0 : i], rs), wscale);
          }
          if (has_bias) y = __fadd_rn(y, bias);
          if (store_ok && i < my_cols) {
            // gate and residual: a separate multiply and add, each rounded, as an unfused epilogue would
            if (gate != nullptr) y = __fmul_rn(y, to_float<OutT>(__ldg(gate)));
            if (residual != nullptr) y = __fadd_rn(y, to_float<OutT>(__ldg(residual)));
            *out = from_float<OutT>(y);
          }
          out += p.out_ld;
          if (residual != nullptr) residual += p.N;
          if (gate != nullptr && --gate_left == 0) {
            gate_left = p.gate_span;
            gate += p.gate_row_stride;
          }
        }
      }
      if (threadIdx.x == 256) stamp(kTrTileEnds, 2 * (git / groups) - 1);
    }
    if constexpr (kStatic && kDW == 2) {
      if (ok) store_pending<0, 64, OutT>(pending, p.out_ld);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// uint8 matrix [rows, row_bytes] -> box [box_rows, box_bytes]
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
              uint32_t box_bytes, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
  return cached[dev] > 0 ? cached[dev] : 148;
}

// Cost of one 128-K block of a tile of t tokens, and what a tile and a K split add, in the same "column units"
// (measured on B200: a block costs a fixed part - barrier and TMEM round trips, int4 unpack - plus a part
// proportional to the tile width; set-up and finalize of a tile about 20 narrow blocks; the exchange of partial sums
// through memory about twice that: at K = 3072 a split gains nothing, at K = 12288 it halves the time).
constexpr double kTileCost = 3000.0, kSplitCost = 6000.0;
inline double block_cost(int t) { return t + 150.0; }

// How many parts the K blocks of a tile are split into: only when the tiles leave at least half of the SMs idle, the
// blocks saved outweigh the exchange, and within the scratch given.
int pick_splits(int tok_tile, int64_t tiles, int k_blocks, int sms, size_t split_bytes) {
  if (tiles * 2 > sms || tiles > 128 || k_blocks < 4) return 1;
  int splits = static_cast<int>(sms / tiles);
  if (splits > k_blocks / 2) splits = k_blocks / 2;
  if (splits > 15) splits = 15;  // a drain warp's field of the tile counter has four bits
  if (splits < 2) return 1;
  const size_t need = 1024 + static_cast<size_t>(tiles) * splits * tok_tile * kBlockCh * sizeof(float);
  if (split_bytes < need) return 1;
  const double saved = (k_blocks - (k_blocks + splits - 1) / splits) * block_cost(tok_tile);
  return saved > kSplitCost ? splits : 1;
}

// Tokens per tile: a multiple of 16 up to 128 (four drain warps x 32 columns per TMEM lane quarter); the kernel runs
// ceil(items / SMs) waves of items (tiles, or parts of tiles split along K).
int pick_tok_tile(int64_t M, int ch_tiles, int k_blocks, int sms, size_t split_bytes) {
  int best = 16;
  double best_cost = 1e30;
  for (int t = 16; t <= 128; t += 16) {
    const int64_t tiles = static_cast<int64_t>(ch_tiles) * ((M + t - 1) / t);
    const int splits = pick_splits(t, tiles, k_blocks, sms, split_bytes);
    const int64_t waves = (tiles * splits + sms - 1) / sms;
    const double blocks = static_cast<double>((k_blocks + splits - 1) / splits);
    const double cost = static_cast<double>(waves) * (blocks * block_cost(t) + kTileCost + (splits > 1 ? kSplitCost : 0.0));
    if (cost <= best_cost) {  // ties go to the wider tile
      best_cost = cost;
      best = t;
    }
    if (t >= M) break;
  }
  return best;
}

template <int TOK, bool kGroup, bool kEvenOdd, bool kDump, typename OutT, bool kTrace = false, bool kPre = false,
          bool kScatter = false, bool kSplit = (TOK <= 64), bool kStatic = false, int kDW = 4>
int launch_variant(const GemmArgs& a, int tok_tile, cudaStream_t stream, long long* timeline = nullptr) {
  auto kernel = sq_gemm_tc_kernel<TOK, kGroup, kEvenOdd, kDump, OutT, kTrace, kPre, kScatter, kSplit, kStatic, kDW>;
  constexpr int kThreads = threads_for(kDW);
  constexpr uint32_t smem = smem_bytes_for(TOK);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  CUtensorMap tmap_codes, tmap_packed;
  if (!make_map(&tmap_codes, a.codes, static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.K),
                static_cast<uint32_t>(tok_tile), kBlockK, CU_TENSOR_MAP_SWIZZLE_128B))
    return SQ_ERR_DRIVER;
  if (kPre) {
    if (!make_map(&tmap_packed, a.w_packed, static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K), kBlockCh, kBlockK,
                  CU_TENSOR_MAP_SWIZZLE_128B))
      return SQ_ERR_DRIVER;
  } else if (!make_map(&tmap_packed, a.w_packed, static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 2), kBlockCh,
                       kBlockK / 2, CU_TENSOR_MAP_SWIZZLE_NONE)) {
    return SQ_ERR_DRIVER;
  }
  TcParams p;
  p.w_scales = a.w_scales; p.row_scales = a.row_scales; p.bias = a.bias; p.out = a.out;
  p.acc_dump = a.acc_dump; p.timeline = timeline; p.status = device_status_word();
  if (p.status == nullptr) return SQ_ERR_DRIVER;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.ch_tiles = static_cast<int>((a.N + kBlockCh - 1) / kBlockCh);
  p.tok_tile = tok_tile;
  {  // the tile's share of one drain warp rounded up to 16 columns, at most a drain warp's register capacity
    const int cap = TOK / kDW < 16 ? 16 : TOK / kDW;
    const int want = ((tok_tile + 16 * kDW - 1) / (16 * kDW)) * 16;
    p.slice_cols = want < cap ? want : cap;
    p.mma_split = (a.K + kBlockK - 1) / kBlockK >= 2 ? 2 : 1;
    if (a.codes_int4_range) {
      p.offset_steps = 1; p.offset_word = 0x40404040u; p.offset_bits = 1u << 17; p.offset_unsigned = 0u;
    } else {
      p.offset_steps = 1; p.offset_word = 0xFFFFFFFFu; p.offset_bits = 32u * 255u * 255u; p.offset_unsigned = 1u;
    }
  }
  p.tok_tiles = static_cast<int>((a.M + tok_tile - 1) / tok_tile);
  p.k_blocks = static_cast<int>((a.K + kBlockK - 1) / kBlockK);
  p.out_dtype = a.out_dtype;
  p.out_ld = a.out_ld > 0 ? a.out_ld : a.N;
  p.out_col0 = a.out_ld > 0 ? a.out_col0 : 0;
  p.n_more = kScatter ? a.n_more_outs : 0;
  for (int d = 0; d < 7; ++d) {
    // distance in elements between the matrices (any two addresses of the unified address space)
    p.more_delta[d] = d < p.n_more ? (reinterpret_cast<intptr_t>(a.more_outs[d]) - reinterpret_cast<intptr_t>(a.out)) /
                                         static_cast<intptr_t>(sizeof(OutT))
                                   : 0;
  }
  p.activation = a.activation; p.gate = a.gate; p.gate_span = a.gate_span > 0 ? a.gate_span : 1;
  p.gate_row_stride = a.gate_row_stride; p.residual = a.residual;
  const int tiles = p.ch_tiles * p.tok_tiles;
  // K split: when the tiles leave at least half of the SMs idle and a tile has K blocks to share out (not with an
  // accumulator dump, whose per-tile sums the parts would have to add up)
  p.splits = 1; p.partials = nullptr; p.counters = nullptr;
  if (kSplit && a.split_workspace != nullptr && a.acc_dump == nullptr) {
    const int splits = pick_splits(tok_tile, tiles, p.k_blocks, sm_count(), a.split_workspace_bytes);
    if (splits >= 2) {
      p.splits = splits;
      p.counters = static_cast<unsigned long long*>(a.split_workspace);
      p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a.split_workspace) + 1024);
      if (!a.split_counters_cleared) {
        const cudaError_t e = cudaMemsetAsync(p.counters, 0, 1024, stream);
        if (e != cudaSuccess) return static_cast<int>(e);
      }
    }
  }
  const int items = tiles * p.splits;
  const int grid = items < sm_count() ? items : sm_count();
  {  // never launch a register split the CTA cannot satisfy
    static int launch_regs[64] = {0};
    if (dev >= 0 && dev < 64 && launch_regs[dev] == 0) {
      cudaFuncAttributes attr;
      const cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
      if (e != cudaSuccess) return static_cast<int>(e);
      launch_regs[dev] = attr.numRegs;
    }
    const int regs = (dev >= 0 && dev < 64) ? launch_regs[dev] : 0;
    if (regs * kThreads < register_pool_needed(kSplit && TOK == 128, kDW)) return SQ_ERR_DRIVER;
  }
  cudaError_t err;
  if (a.after_prepass) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(grid));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    err = cudaLaunchKernelEx(&config, kernel, tmap_codes, tmap_packed, p);
  } else {
    kernel<<<grid, kThreads, smem, stream>>>(tmap_codes, tmap_packed, p);
    err = cudaGetLastError();
  }
  return err == cudaSuccess ? SQ_OK : static_cast<int>(err);
}

template <int TOK, bool kGroup>
int launch_tok(const GemmArgs& a, int tok_tile, cudaStream_t stream) {
  const bool eo = a.codes_layout == SQ_CODES_EVEN_ODD;
  const bool dump = a.acc_dump != nullptr;
  const bool bf16 = a.out_dtype == SQ_BF16;
#define SQ_LAUNCH(EO, DUMP)                                                                          \
  (bf16 ? launch_variant<TOK, kGroup, EO, DUMP, __nv_bfloat16>(a, tok_tile, stream)          \
        : launch_variant<TOK, kGroup, EO, DUMP, __half>(a, tok_tile, stream))
  const bool whole_chunks = TOK == 128 && kGroup && eo && !dump && ((a.K / kBlockK) & 7) == 0 && (a.K % kBlockK) == 0 &&
                            (reinterpret_cast<uintptr_t>(a.w_scales) & 15u) == 0;
  if (a.n_more_outs > 0) {
    // channel-split form: the 128-token kernel only (a split over GPUs is for many tokens), even-odd codes, packed weights
    if (TOK != 128 || !eo || dump || a.weights_prepacked) return SQ_ERR_ENUM;
    if (whole_chunks)  // the drain with the ring position unrolled (four warps per lane quarter: its finalize has the peer stores)
      return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, false, true, false, kGroup>(a, tok_tile, stream)
                  : launch_variant<128, kGroup, true, false, __half, false, false, true, false, kGroup>(a, tok_tile, stream);
    return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, false, true>(a, tok_tile, stream)
                : launch_variant<128, kGroup, true, false, __half, false, false, true>(a, tok_tile, stream);
  }
  static const int drain_warps_env = [] { const char* e = getenv("SQ_TC_DW"); return e != nullptr ? atoi(e) : 2; }();
  const int drain_warps = a.gate == nullptr && a.residual == nullptr ? drain_warps_env : 4;  // the deferred finalize has no fused forms
  if (a.weights_prepacked && whole_chunks && drain_warps == 2) {
    return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, true, false, false, kGroup, kGroup ? 2 : 4>(a, tok_tile, stream)
                : launch_variant<128, kGroup, true, false, __half, false, true, false, false, kGroup, kGroup ? 2 : 4>(a, tok_tile, stream);
  }
  if (a.weights_prepacked && whole_chunks) {
    return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, true, false, false, kGroup>(a, tok_tile, stream)
                : launch_variant<128, kGroup, true, false, __half, false, true, false, false, kGroup>(a, tok_tile, stream);
  }
  if (a.weights_prepacked) {  // validated: even-odd codes, no accumulator dump
    return bf16 ? launch_variant<TOK, kGroup, true, false, __nv_bfloat16, false, true>(a, tok_tile, stream)
                : launch_variant<TOK, kGroup, true, false, __half, false, true>(a, tok_tile, stream);
  }
  if (TOK == 128 && eo && !dump && a.split_workspace != nullptr) {
    // few tiles of many K blocks (a few hundred tokens into a narrow layer): the variant of the 128-token kernel
    // that can split K
    const int64_t tiles = static_cast<int64_t>((a.N + kBlockCh - 1) / kBlockCh) * ((a.M + tok_tile - 1) / tok_tile);
    if (pick_splits(tok_tile, tiles, static_cast<int>((a.K + kBlockK - 1) / kBlockK), sm_count(), a.split_workspace_bytes) >= 2)
      return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, false, false, true>(a, tok_tile, stream)
                  : launch_variant<128, kGroup, true, false, __half, false, false, false, true>(a, tok_tile, stream);
  }
  if (whole_chunks && drain_warps == 2) {
    return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, false, false, false, kGroup, kGroup ? 2 : 4>(a, tok_tile, stream)
                : launch_variant<128, kGroup, true, false, __half, false, false, false, false, kGroup, kGroup ? 2 : 4>(a, tok_tile, stream);
  }
  if (whole_chunks) {
    // whole chunks of eight group scales per tile, no K split: the variant with the ring position unrolled
    return bf16 ? launch_variant<128, kGroup, true, false, __nv_bfloat16, false, false, false, false, kGroup>(a, tok_tile, stream)
                : launch_variant<128, kGroup, true, false, __half, false, false, false, false, kGroup>(a, tok_tile, stream);
  }
  if (eo) return dump ? SQ_LAUNCH(true, true) : SQ_LAUNCH(true, false);
  return dump ? SQ_LAUNCH(false, true) : SQ_LAUNCH(false, false);
#undef SQ_LAUNCH
}

template <bool kGroup>
int launch_mode(const GemmArgs& a, cudaStream_t stream) {
  const int ch_tiles = static_cast<int>((a.N + kBlockCh - 1) / kBlockCh);
  const int k_blocks = static_cast<int>((a.K + kBlockK - 1) / kBlockK);
  const size_t split_bytes = (a.split_workspace != nullptr && a.acc_dump == nullptr) ? a.split_workspace_bytes : 0;
  int t = pick_tok_tile(a.M, ch_tiles, k_blocks, sm_count(), split_bytes);
  if (a.n_more_outs > 0 && t <= 64) t = 128;  // the channel-split form exists in the 128-token kernel only
  if (t <= 32) return launch_tok<32, kGroup>(a, t, stream);
  if (t <= 64) return launch_tok<64, kGroup>(a, t, stream);
  return launch_tok<128, kGroup>(a, t, stream);
}

// ---------------------------------------------------------------------------------- tensor-pipe rate probe
// One warp per SM issues `iters` x 4 kind::i8 MMAs (M = 128, N = kN, K = 32) back to back on fixed shared-memory
// tiles, commits once and waits (bounded); thread block 0 reports the SM cycles from first issue to completion.
template <int kN, bool kTs = false>
__global__ void __launch_bounds__(128, 1) sq_mma_rate_kernel(long long* cycles, int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_tile = base;                   // 128 rows x 128 B
  const uint32_t b_tile = base + kWBytes;         // kN rows x 128 B
  const uint32_t bar = b_tile + kN * kBlockK;
  const uint32_t slot = bar + 16;
  const uint32_t abort_slot = slot + 4;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + (abort_slot - base));
  for (uint32_t i = threadIdx.x; i < (kWBytes + kN * kBlockK) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(gen)[i] = 0x01010101u;
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(gen + (slot - base));
  if (warp == 0) {
    const uint32_t idesc = umma_idesc_i8(kBlockCh, kN);
    const uint64_t desc_a = umma_desc_k128(a_tile), desc_b = umma_desc_k128(b_tile);
    const long long t0 = clock64();
    if (elect_one()) {
      for (int it = 0; it < iters; ++it) {
        const uint32_t d = tmem + (it & 1) * 256;
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          // kTs: operand A from tensor memory (whatever columns 384.. hold; only the rate matters)
          if (kTs) umma_i8_ts(d, tmem + 384 + 8 * k, desc_b + 2 * k, idesc, k > 0 ? 1u : 0u);
          else umma_i8(d, desc_a + 2 * k, desc_b + 2 * k, idesc, k > 0 ? 1u : 0u);
        }
      }
      umma_commit(bar);
    }
    __syncwarp();
    if (!mbar_wait_bounded(bar, 0, abort_flag, kWaitLimitNs) && threadIdx.x == 0) report_timeout(status, abort_flag, 9006);
    const long long t1 = clock64();
    if (threadIdx.x == 0 && blockIdx.x == 0) cycles[0] = t1 - t0;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

template <int kN, bool kTs = false>
int launch_mma_rate_n(long long* cycles, int iters, cudaStream_t stream) {
  const int smem = static_cast<int>(kWBytes) + kN * kBlockK + 2048;
  cudaError_t err = cudaFuncSetAttribute(sq_mma_rate_kernel<kN, kTs>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return static_cast<int>(err);
  int* status = device_status_word();
  if (status == nullptr) return SQ_ERR_DRIVER;
  sq_mma_rate_kernel<kN, kTs><<<sm_count(), 128, smem, stream>>>(cycles, iters, status);
  err = cudaGetLastError();
  return err == cudaSuccess ? SQ_OK : static_cast<int>(err);
}

}  // namespace

int launch_mma_rate(int n_cols, int iters, long long* cycles, cudaStream_t stream) {
  if (cycles == nullptr) return SQ_ERR_NULL;
  if (iters <= 0 || iters > 100000) return SQ_ERR_SHAPE;
  switch (n_cols) {
    case 64: return launch_mma_rate_n<64>(cycles, iters, stream);
    case 128: return launch_mma_rate_n<128>(cycles, iters, stream);
    case 256: return launch_mma_rate_n<256>(cycles, iters, stream);
    case 0x1000 + 128: return launch_mma_rate_n<128, true>(cycles, iters, stream);  // weights from tensor memory
    default: return SQ_ERR_ENUM;
  }
}

int launch_gemm_timeline(const GemmArgs& a, long long* timeline, cudaStream_t stream) {
  int v = validate_gemm(a);
  if (v != SQ_OK) return v;
  if (timeline == nullptr) return SQ_ERR_NULL;
  if (a.wscale_mode != SQ_WSCALE_GROUP_F16 || a.codes_layout != SQ_CODES_EVEN_ODD || a.out_dtype != SQ_BF16 || a.M <= 128)
    return SQ_ERR_ENUM;
  const int ch_tiles = static_cast<int>((a.N + kBlockCh - 1) / kBlockCh);
  int t = pick_tok_tile(a.M, ch_tiles, static_cast<int>((a.K + kBlockK - 1) / kBlockK), sm_count(), 0);
  if (t <= 64) t = 128;
  if (((a.K / kBlockK) & 7) == 0 && (a.K % kBlockK) == 0 && (reinterpret_cast<uintptr_t>(a.w_scales) & 15u) == 0 &&
      a.gate == nullptr && a.residual == nullptr)  // the form large problems run: two-warp drain, static ring
    return launch_variant<128, true, true, false, __nv_bfloat16, true, false, false, false, true, 2>(a, t, stream, timeline);
  return launch_variant<128, true, true, false, __nv_bfloat16, true>(a, t, stream, timeline);
}

int launch_gemm_tc(const GemmArgs& a, cudaStream_t stream) {
  if (a.M == 0) return SQ_OK;  // nothing to do; an empty tensor may come with a null pointer
  int v = validate_gemm(a);
  if (v != SQ_OK) return v;
  if (a.weights_prepacked && a.acc_dump != nullptr) return SQ_ERR_ENUM;  // the prepacked variants carry no dump path
  if (a.wscale_mode == SQ_WSCALE_GROUP_F16) return launch_mode<true>(a, stream);
  return launch_mode<false>(a, stream);
}

}  // namespace sq

// W4A8 / W4A4 GEMM, second generation: the weight operand lives in TENSOR memory.
//
//   out[m, n] = sum_k a[m, k] * w[n, k]        a: int8 codes [M, K], w: packed int4 [N, K/2]
//
// "Weights as rows": UMMA M (TMEM lanes) = 128 output channels, UMMA N (TMEM columns) = up to 128 tokens, so a
// weight-group scale is a per-thread scalar in the drain.  What is new against sq_gemm_tc.cu:
//
//   * The unpack warps write the int4 -> int8 expanded weights straight into tensor memory (tcgen05.st) and the
//     MMAs take operand A from there.  Shared memory then carries, per 128-K block, only the packed weights
//     (8 KiB in, 8 KiB read once) and the codes (16 KiB in, 16 KiB read by the tensor core) instead of also a
//     16 KiB unpacked tile written and read: a 128 x 128 x 32 MMA with both operands in shared memory needs
//     the full 128 B/clk of the shared-memory port for itself.
//   * Eight "fat" drain warps (two per TMEM lane quarter, 64 token columns each, 200 registers) keep TWO
//     accumulators in flight: the tcgen05.ld of group g + 1 is issued before the FFMAs of group g, so the
//     barrier / TMEM round trips of one group hide behind the arithmetic of the previous one.
//   * Work is cut into (tile, K-range) items.  Whole tiles go round-robin over the persistent CTAs; what is
//     left of the last wave - or everything, when there are fewer tiles than SMs (small M) - is split along K
//     so every CTA gets the same number of 128-K blocks.  Partial sums go through a caller-provided scratch
//     area; the CTA that arrives last at a tile adds the partials in K order (deterministic) and finalizes.
//     No CTA ever waits for another one.
//   * Codes of any int8 value get their positive accumulator offset from ONE unsigned MMA (32 * 255 * 255).
//
// Per CTA (persistent, 512 threads):
//   warp 0        TMA producer (packed weights, 64-byte swizzle; codes, 128-byte swizzle) + row-scale staging
//   warps 1-3     MMA issuers (group form: groups round-robin; channel form: warp 1 alone)
//   warps 4-7     unpack: one channel row per thread, 64 packed bytes -> 32 TMEM columns
//   warps 8-15    drain
// Tensor memory: columns [0, 384) three accumulators, [384, 512) four stages of unpacked weights.
// Every mbarrier wait is time-bounded; a wait that gives up sets the CTA's abort flag and the device status word.
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
constexpr int kThreads = 768;
constexpr int kUnpackWarps = 4;
constexpr int kDrainWarps = 16;
constexpr int kRegsControl = 32, kRegsUnpack = 32, kRegsDrain = 104;
// setmaxnreg.inc only hands out registers the CTA was launched with: the launcher checks this sum against
// (registers per thread at launch) x kThreads before every launch.
constexpr int kRegisterPoolNeeded = 128 * kRegsControl + 128 * kRegsUnpack + 512 * kRegsDrain;
constexpr uint32_t kPackedBytes = kBlockCh * kBlockK / 2;  // 8 KiB
constexpr uint32_t kConstTileBytes = kBlockCh * kBlockK;   // 16 KiB: both operands of the offset MMA
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait

constexpr uint32_t kAccBufs = 3;       // accumulator ring
constexpr uint32_t kAccStride = 128;   // TMEM columns between accumulators
constexpr uint32_t kAStages = 4;       // unpacked-weight ring in TMEM
constexpr uint32_t kAStageCols = 32;   // 128 K bytes per lane
constexpr uint32_t kAColBase = kAccBufs * kAccStride;  // 384
constexpr uint32_t kTmemCols = 512;
constexpr int kRowScaleSlots = 2;
// shared-memory ring (packed weights + codes): what is left next to the constant tile and the output staging
__host__ __device__ constexpr int stages_for(int tok) { return tok == 128 ? 8 : 10; }


// Group mode keeps every accumulator positive (see sq_gemm_tc.cu): a positive int32 below 2^23 read as a float is
// the denormal acc * 2^-149, so the drain is one packed FFMA per two elements with the scale pre-multiplied.
constexpr float kScaleUp = 7.922816251426434e28f;  // 2^96
constexpr float kScaleDown = 562949953421312.0f;   // 2^49 = 2^149 / 2^96 / 16 (the unpacked weights are 16 w)

constexpr int kTraceSlots = 512;
enum TraceRole { kTrTmaIssue = 0, kTrConvStart, kTrConvDone, kTrMmaAccFree, kTrMmaIssue, kTrDrainStart,
                 kTrDrainRelease, kTrDrainDone, kTrMmaCommitted, kTrDrainTop, kTrDrainLoaded, kTrItemEnd, kTraceRoles };

__host__ __device__ constexpr uint32_t stage_bytes(int tok) { return tok * kBlockK + kPackedBytes; }
__host__ __device__ constexpr uint32_t smem_bytes_for(int tok) {
  return stages_for(tok) * stage_bytes(tok) + kConstTileBytes + kRowScaleSlots * 512 +
         1024 /*alignment slack*/ + 512 /*barriers*/;
}

// How the tiles are dealt to the CTAs.  Tiles [0, tail_first) are whole items: tile = round * grid + cta.
// Tiles [tail_first, tail_first + tail_tiles) are cut into tail_tiles * groups units of one 128-K block; CTA c
// (c < tail_ctas) takes units [c W / tail_ctas, (c + 1) W / tail_ctas).
struct Plan {
  int ch_tiles, tok_tiles, tiles, groups;
  int full_rounds, tail_first, tail_tiles, tail_ctas;
};

struct Item {
  int tile, g0, g1, slot;
};

__host__ __device__ inline int unit_start(int c, int total_units, int ctas) {
  return static_cast<int>((static_cast<long long>(c) * total_units) / ctas);
}

struct ItemIter {
  int round, u, u_end, emitted;
  __device__ void init(const Plan& pl, int cta) {
    round = 0;
    emitted = 0;
    u = u_end = 0;
    if (cta < pl.tail_ctas) {
      const int total = pl.tail_tiles * pl.groups;
      u = unit_start(cta, total, pl.tail_ctas);
      u_end = unit_start(cta + 1, total, pl.tail_ctas);
    }
  }
  __device__ bool next(const Plan& pl, int cta, int grid, Item& item) {
    while (round < pl.full_rounds) {
      const int t = round * grid + cta;
      ++round;
      if (t < pl.tail_first) {
        item.tile = t; item.g0 = 0; item.g1 = pl.groups; item.slot = 0;
        return true;
      }
    }
    if (u < u_end) {
      const int t = u / pl.groups;
      const int gs = u - t * pl.groups;
      const int len = min(pl.groups - gs, u_end - u);
      item.tile = pl.tail_first + t; item.g0 = gs; item.g1 = gs + len; item.slot = emitted == 0 ? 0 : 1;
      ++emitted;
      u += len;
      return true;
    }
    return false;
  }
};

struct TsParams {
  const void* w_scales;
  const float* row_scales;
  const void* bias;
  void* out;
  int32_t* acc_dump;
  long long* timeline;
  int* status;
  float* partials;   // [grid][2][tok_tile][128] fp32, or null when no tile is split
  int* counters;     // [tail_tiles], zero at launch
  int64_t M, N, K;
  Plan plan;
  int tok_tile;
  uint32_t offset_word;  // four copies of the constant tile's byte
  uint32_t offset_bits;  // what the offset MMA adds to every accumulator element
  uint32_t offset_unsigned;  // the offset MMA multiplies unsigned bytes
  int out_dtype;
  uint32_t flags;  // experiment switches (SQ_TS_FLAGS in the environment; 0 in production)
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
// c += (a0, a1) * b as one packed FMA; a0 / a1 are raw bit patterns of two adjacent registers.  Volatile: the
// accumulator registers become valid only at the tcgen05.wait::ld in front, which is a volatile asm too, and
// volatile asms keep their order.
__device__ __forceinline__ void ffma2(uint64_t& c, uint32_t a0, uint32_t a1, uint64_t b) {
  asm volatile("{\n\t"
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

// TOK    capacity in tokens of one tile (TMEM columns per accumulator, rows of a codes stage)
// kGroup one accumulator per 128-K weight group (fp16 scales [N, K/128]); otherwise one per item (fp32 [N])
// kEvenOdd codes are stored even-k-first inside each run of 8
// kDump  also write the exact integer accumulators
template <int TOK, bool kGroup, bool kEvenOdd, bool kDump, typename OutT, bool kTrace = false>
__global__ void __launch_bounds__(kThreads, 1)
sq_gemm_ts_kernel(const __grid_constant__ CUtensorMap tmap_codes, const __grid_constant__ CUtensorMap tmap_packed,
                  const TsParams p) {
  constexpr int S = stages_for(TOK);
  constexpr uint32_t kXBytes = TOK * kBlockK;
  constexpr int kCols = TOK / 4 < 16 ? 16 : TOK / 4;  // token columns per drain warp: 32 or 16
  static_assert(TOK == 128 || TOK == 64 || TOK == 32, "tile capacities");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t x_ring = smem_base;                   // S x TOK*128, codes (UMMA B)
  const uint32_t p_ring = x_ring + S * kXBytes;        // S x 8 KiB, packed weights (64-byte swizzle)
  const uint32_t c_tile = p_ring + S * kPackedBytes;   // 16 KiB of one byte value: operands of the offset MMA
  const uint32_t rs_base = c_tile + kConstTileBytes;   // kRowScaleSlots x 128 floats
  const uint32_t bars = rs_base + kRowScaleSlots * 512;
  const uint32_t bar_full_p = bars;                    // [S] packed weights landed
  const uint32_t bar_full_x = bars + 8 * S;            // [S] codes landed
  const uint32_t bar_x_empty = bars + 16 * S;          // [S] the MMAs of this stage retired
  const uint32_t bar_a_full = bars + 24 * S;           // [kAStages] unpacked weights are in tensor memory
  const uint32_t bar_acc_full = bar_a_full + 8 * kAStages;
  const uint32_t bar_acc_empty = bar_acc_full + 8 * kAccBufs;
  const uint32_t bar_rs_full = bar_acc_empty + 8 * kAccBufs;
  const uint32_t bar_rs_empty = bar_rs_full + 8 * kRowScaleSlots;
  const uint32_t bar_meet = bar_rs_empty + 8 * kRowScaleSlots;  // drain warps' rendezvous around a split tile
  const uint32_t tmem_slot = bar_meet + 8;
  const uint32_t abort_slot = tmem_slot + 4;
  const uint32_t last_slot = abort_slot + 4;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));
  volatile int* last_flag = reinterpret_cast<volatile int*>(smem_gen + (last_slot - smem_base));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int grid = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full_p + 8 * s, 1);
      mbar_init(bar_full_x + 8 * s, 1);
      mbar_init(bar_x_empty + 8 * s, 1);
    }
    for (uint32_t a = 0; a < kAStages; ++a) mbar_init(bar_a_full + 8 * a, kUnpackWarps);
    for (uint32_t b = 0; b < kAccBufs; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, kDrainWarps);
    }
    for (int r = 0; r < kRowScaleSlots; ++r) {
      mbar_init(bar_rs_full + 8 * r, 1);
      mbar_init(bar_rs_empty + 8 * r, kDrainWarps);
    }
    mbar_init(bar_meet, kDrainWarps);
    *abort_flag = 0;
    *last_flag = 0;
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
    for (uint32_t i = threadIdx.x; i < kConstTileBytes / 4; i += kThreads) c_words[i] = p.offset_word;
    fence_proxy_async_smem();  // the tensor core reads this tile through the async proxy
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Launched as a programmatic dependent of the pre-pass, this kernel may become resident while the pre-pass
  // still runs: everything above touches only this CTA's shared and tensor memory.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const Plan& pl = p.plan;
  const uint32_t wait_kind = (p.flags >> 3) & 3u;  // experiment switch: how a role waits on a barrier
  auto wait_on = [&](uint32_t bar, uint32_t parity, volatile int* flag, uint64_t limit) {
    if (wait_kind == 1u) return mbar_wait_bounded(bar, parity, flag, limit);
    if (wait_kind == 2u) return mbar_wait_probe<32>(bar, parity, flag, limit);
    if (wait_kind == 3u) return mbar_wait_probe<0>(bar, parity, flag, limit);
    return mbar_wait_light(bar, parity, flag, limit);
  };
  const bool tracing = kTrace && blockIdx.x == 0 && p.timeline != nullptr;
  auto stamp = [&](int role, uint32_t slot) {
    if (kTrace && tracing && slot < kTraceSlots) p.timeline[role * kTraceSlots + slot] = clock64();
  };

  if (warp < 4) {
    // ------------------------------------------------------------------ control warpgroup
    reg_dec<kRegsControl>();
    if (warp == 0) {
      // TMA producer; after the loads of an item it also stages the item's row scales in shared memory
      ItemIter iter;
      iter.init(pl, cta);
      Item item;
      uint32_t it = 0, item_idx = 0;
      bool ok = true;
      while (ok && iter.next(pl, cta, grid, item)) {
        const int ch0 = (item.tile % pl.ch_tiles) * kBlockCh;
        const int tok0 = (item.tile / pl.ch_tiles) * p.tok_tile;
        for (int g = item.g0; g < item.g1; ++g, ++it) {
          const uint32_t s = it % S, phase = (it / S) & 1u;
          if (!wait_on(bar_x_empty + 8 * s, phase ^ 1u, abort_flag, kWaitLimitNs)) {
            if (lane == 0) report_timeout(p.status, abort_flag, 9101);
            ok = false;
            break;
          }
          if (elect_one()) {
            stamp(kTrTmaIssue, it);
            mbar_arrive_expect_tx(bar_full_x + 8 * s, static_cast<uint32_t>(p.tok_tile) * kBlockK);
            tma_load_2d(x_ring + s * kXBytes, &tmap_codes, g * kBlockK, tok0, bar_full_x + 8 * s);
            mbar_arrive_expect_tx(bar_full_p + 8 * s, kPackedBytes);
            tma_load_2d(p_ring + s * kPackedBytes, &tmap_packed, g * (kBlockK / 2), ch0, bar_full_p + 8 * s);
          }
          __syncwarp();
        }
        if (!ok) break;
        const uint32_t slot = item_idx % kRowScaleSlots, rphase = (item_idx / kRowScaleSlots) & 1u;
        if (!wait_on(bar_rs_empty + 8 * slot, rphase ^ 1u, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9107);
          break;
        }
        float4 rs = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const int64_t m = static_cast<int64_t>(tok0) + 4 * lane;
        if (m + 4 <= p.M) {
          rs = __ldg(reinterpret_cast<const float4*>(p.row_scales + m));
        } else {
          if (m < p.M) rs.x = __ldg(p.row_scales + m);
          if (m + 1 < p.M) rs.y = __ldg(p.row_scales + m + 1);
          if (m + 2 < p.M) rs.z = __ldg(p.row_scales + m + 2);
        }
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(rs_base + slot * 512 + lane * 16), "f"(rs.x),
                     "f"(rs.y), "f"(rs.z), "f"(rs.w)
                     : "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rs_full + 8 * slot);
        ++item_idx;
      }
    } else {
      // MMA issuers.  Group form: a group is one K block with its own accumulator; warps 1..3 take the groups
      // round-robin (group it uses accumulator it % 3, which is also its issuer), so the barrier round trips of
      // one group overlap the issue of the next two.  Channel form: warp 1 alone, one accumulator per item.
      const uint32_t mine = static_cast<uint32_t>(warp - 1);
      ItemIter iter;
      iter.init(pl, cta);
      Item item;
      uint32_t it = 0, item_idx = 0;
      bool ok = kGroup || mine == 0;
      const uint32_t idesc_bits = p.offset_unsigned;
      while (ok && iter.next(pl, cta, grid, item)) {
        const int tok0 = (item.tile / pl.ch_tiles) * p.tok_tile;
        const int64_t left = p.M - tok0;
        const int tok_count = left < p.tok_tile ? static_cast<int>(left) : p.tok_tile;
        const uint32_t umma_n = static_cast<uint32_t>((tok_count + 15) & ~15);
        const uint32_t idesc = umma_idesc_i8(kBlockCh, umma_n);
        const uint32_t idesc_off = idesc_bits != 0 ? umma_idesc_u8(kBlockCh, umma_n) : idesc;
        uint32_t buf = 0;
        if (!kGroup) {
          buf = item_idx % kAccBufs;
          const uint32_t aphase = (item_idx / kAccBufs) & 1u;
          if (!wait_on(bar_acc_empty + 8 * buf, aphase ^ 1u, abort_flag, kWaitLimitNs)) {
            if (lane == 0) report_timeout(p.status, abort_flag, 9102);
            break;
          }
        }
        for (int g = item.g0; g < item.g1 && ok; ++g, ++it) {
          if (kGroup) {
            if (it % kAccBufs != mine) continue;
            buf = mine;
            const uint32_t aphase = (it / kAccBufs) & 1u;
            if (!wait_on(bar_acc_empty + 8 * buf, aphase ^ 1u, abort_flag, kWaitLimitNs)) {
              if (lane == 0) report_timeout(p.status, abort_flag, 9102);
              ok = false;
              break;
            }
          }
          if (lane == 0) stamp(kTrMmaAccFree, it);
          const uint32_t tmem_d = tmem_base + buf * kAccStride;
          if (kGroup) {
            // the offset MMA needs no operand from the pipeline: it starts the accumulator at a positive value
            tc_fence_after_sync();
            if (elect_one()) {
              const uint64_t desc_c = umma_desc_k128(c_tile);
              umma_i8(tmem_d, desc_c, desc_c, idesc_off, 0u);
            }
            __syncwarp();
          }
          const uint32_t s = it % S, sphase = (it / S) & 1u;
          const uint32_t ta = it % kAStages, tphase = (it / kAStages) & 1u;
          if (!wait_on(bar_a_full + 8 * ta, tphase, abort_flag, kWaitLimitNs) ||
              !wait_on(bar_full_x + 8 * s, sphase, abort_flag, kWaitLimitNs)) {
            if (lane == 0) report_timeout(p.status, abort_flag, 9103);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (lane == 0) stamp(kTrMmaIssue, it);
          if (elect_one()) {
            const uint32_t tmem_a = tmem_base + kAColBase + ta * kAStageCols;
            const uint64_t desc_b = umma_desc_k128(x_ring + s * kXBytes);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              const uint32_t accumulate = (kGroup || g > item.g0 || k > 0) ? 1u : 0u;
              // operand A: eight TMEM columns per K = 32 step; operand B: +2 in the (address >> 4) field
              umma_i8_ts(tmem_d, tmem_a + 8 * k, desc_b + 2 * k, idesc, accumulate);
            }
            umma_commit(bar_x_empty + 8 * s);  // frees the stage and the TMEM weight stage when these MMAs retire
            if (kGroup || g + 1 == item.g1) umma_commit(bar_acc_full + 8 * buf);
          }
          __syncwarp();
          if (lane == 0) stamp(kTrMmaCommitted, it);
        }
        ++item_idx;
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ unpack warpgroup
    reg_dec<kRegsUnpack>();
    const int quarter = warp - 4;            // == warp % 4: the TMEM lane quarter this warp may address
    const int row = quarter * 32 + lane;     // channel row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t sw = static_cast<uint32_t>((row >> 1) & 3);  // 64-byte swizzle: chunk ^= (row / 2) % 4
    ItemIter iter;
    iter.init(pl, cta);
    Item item;
    uint32_t it = 0;
    bool ok = true;
    const bool defer = (p.flags & 1u) == 0u;
    bool pending = false;
    uint32_t pending_stage = 0;
    while (ok && iter.next(pl, cta, grid, item)) {
      for (int g = item.g0; g < item.g1; ++g, ++it) {
        const uint32_t s = it % S, phase = (it / S) & 1u;
        const uint32_t ta = it % kAStages;
        bool ready = wait_on(bar_full_p + 8 * s, phase, abort_flag, kWaitLimitNs);
        if (ready && it >= kAStages) {
          // the TMEM stage is free when the MMAs of iteration it - kAStages have retired
          const uint32_t j = it - kAStages;
          ready = wait_on(bar_x_empty + 8 * (j % S), (j / S) & 1u, abort_flag, kWaitLimitNs);
        }
        if (!ready) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9104);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (threadIdx.x == 128) stamp(kTrConvStart, it);
        const uint32_t src = p_ring + s * kPackedBytes + static_cast<uint32_t>(row) * 64u;
        const uint32_t dst = tmem_base + lane_addr + kAColBase + ta * kAStageCols;
        // a 16-byte chunk (32 k) at a time: 4 words in, 8 words = 8 TMEM columns out.  The stores of the previous
        // stage are waited for only after this stage's first chunk is unpacked, so their latency hides behind
        // this stage's barrier waits and shared-memory loads.
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t win[4];
          const uint32_t chunk = static_cast<uint32_t>(c) ^ sw;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(win[0]), "=r"(win[1]), "=r"(win[2]), "=r"(win[3])
                       : "r"(src + chunk * 16u));
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t lo = (win[i] << 4) & 0xF0F0F0F0u;  // 16 * nibble of even k, as int8
            const uint32_t hi = win[i] & 0xF0F0F0F0u;         // 16 * nibble of odd k
            if (kEvenOdd) {
              o[2 * i] = lo;
              o[2 * i + 1] = hi;
            } else {
              o[2 * i] = __byte_perm(lo, hi, 0x5140);      // k0 k1 k2 k3
              o[2 * i + 1] = __byte_perm(lo, hi, 0x7362);  // k4 k5 k6 k7
            }
          }
          if (c == 0 && pending) {
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_a_full + 8 * pending_stage);
            pending = false;
          }
          tmem_st_32x32b_x8(dst + 8 * c, o);
        }
        if (defer) {
          pending = true;
          pending_stage = ta;
        } else {
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_a_full + 8 * ta);
        }
        if (threadIdx.x == 128) stamp(kTrConvDone, it);
      }
    }
    if (pending) {  // the last stage's stores
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_a_full + 8 * pending_stage);
    }
  } else {
    // ------------------------------------------------------------------ drain warpgroups
    reg_inc<kRegsDrain>();
    const int dwarp = warp - 8;            // 0..15
    const int quarter = warp & 3;          // TMEM lane quarter this warp may address
    const int slice = dwarp >> 2;          // which slice of the token columns (four warps per lane quarter)
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int ch_in_tile = quarter * 32 + lane;
    const int my_col0 = slice * kCols;
    const unsigned short* scale_bits = static_cast<const unsigned short*>(p.w_scales);
    const uint32_t offset_bits = kGroup ? p.offset_bits : 0u;
    const float offset_float = __uint_as_float(offset_bits);
    const int groups = pl.groups;
    // eight group scales of a channel are one 16-byte load when the rows of the scale matrix allow it
    const bool scale_vectors = kGroup && (groups & 7) == 0 && (reinterpret_cast<uintptr_t>(p.w_scales) & 15u) == 0;
    ItemIter iter;
    iter.init(pl, cta);
    Item item;
    uint32_t it = 0, item_idx = 0, meets = 0;
    bool ok = true;
    while (ok && iter.next(pl, cta, grid, item)) {
      const int ch0 = (item.tile % pl.ch_tiles) * kBlockCh;
      const int tok0 = (item.tile / pl.ch_tiles) * p.tok_tile;
      const int64_t left = p.M - tok0;
      const int tok_count = left < p.tok_tile ? static_cast<int>(left) : p.tok_tile;
      const int my_cols = min(max(tok_count - my_col0, 0), kCols);  // real tokens in my slice
      const int64_t n = ch0 + ch_in_tile;
      const bool n_ok = n < p.N;
      const int n_groups = item.g1 - item.g0;

      uint64_t sums2[kCols / 2];  // packed pairs (columns 2i, 2i + 1)
#pragma unroll
      for (int i = 0; i < kCols / 2; ++i) sums2[i] = 0ull;
      float offset_sum = 0.0f;  // what the constant offsets added to every sum of this channel

      if (kGroup) {
        // Group scales: chunks of eight (one uint4), the next chunk requested a whole chunk ahead, so no global
        // load latency sits on the per-group path.  Scalar loads (other group counts) are requested two groups ahead.
        const unsigned short* my_scales = scale_bits + (n_ok ? n : 0) * groups;
        uint4 chunk = make_uint4(0u, 0u, 0u, 0u), chunk_next = make_uint4(0u, 0u, 0u, 0u);
        unsigned short raw_a = 0, raw_b = 0;
        if (scale_vectors) {
          const int c0 = item.g0 >> 3;
          chunk = __ldg(reinterpret_cast<const uint4*>(my_scales) + c0);
          if (8 * (c0 + 1) < groups) chunk_next = __ldg(reinterpret_cast<const uint4*>(my_scales) + c0 + 1);
        } else {
          raw_a = __ldg(my_scales + item.g0);
          if (n_groups > 1) raw_b = __ldg(my_scales + item.g0 + 1);
        }
        // per group: wait for the accumulator, one wide TMEM load, hand the accumulator back, then the arithmetic
        // (a load takes about a hundred cycles; the two drain warps of a scheduler overlap each other's loads
        // and FFMAs, keeping a second load in flight per warp measured no faster)
        for (int i = 0; i < n_groups; ++i) {
          const int g = item.g0 + i;
          if (threadIdx.x == 256) stamp(kTrDrainTop, it + static_cast<uint32_t>(i));
          unsigned short raw;
          if (scale_vectors) {
            const int e = g & 7;
            const uint32_t word = e < 4 ? (e < 2 ? chunk.x : chunk.y) : (e < 6 ? chunk.z : chunk.w);
            raw = static_cast<unsigned short>((e & 1) != 0 ? word >> 16 : word & 0xFFFFu);
            if (e == 7) {
              chunk = chunk_next;
              const int c2 = (g >> 3) + 2;
              if (8 * c2 < groups) chunk_next = __ldg(reinterpret_cast<const uint4*>(my_scales) + c2);
            }
          } else {
            raw = (i & 1) == 0 ? raw_a : raw_b;
            if (i + 2 < n_groups) {
              const unsigned short ahead = __ldg(my_scales + g + 2);
              if ((i & 1) == 0) raw_a = ahead; else raw_b = ahead;
            }
          }
          const float scale = __half2float(__ushort_as_half(raw)) * kScaleUp;
          offset_sum = fmaf(offset_float, scale, offset_sum);
          const uint32_t git = it + static_cast<uint32_t>(i);
          const uint32_t buf = git % kAccBufs, aphase = (git / kAccBufs) & 1u;
          if (!wait_on(bar_acc_full + 8 * buf, aphase, abort_flag, kWaitLimitNs)) {
            if (lane == 0) report_timeout(p.status, abort_flag, 9105);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (threadIdx.x == 256) stamp(kTrDrainStart, git);
          uint32_t r[kCols];
          if (my_cols > 0) {
            tmem_ld_chunk(tmem_base + lane_addr + buf * kAccStride + my_col0, r);
            tmem_wait_ld();
          }
          if (threadIdx.x == 256) stamp(kTrDrainLoaded, git);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
          if (threadIdx.x == 256) stamp(kTrDrainRelease, git);
          if (my_cols > 0) {
            const uint64_t scale2 = pack2(scale, scale);
#pragma unroll
            for (int c = 0; c < kCols; c += 2) ffma2(sums2[c / 2], r[c], r[c + 1], scale2);
            if (kDump) {
              for (int c = 0; c < my_cols; ++c) {
                uint32_t v = 0;
#pragma unroll
                for (int k = 0; k < kCols; ++k) v = k == c ? r[k] : v;
                const int64_t m = tok0 + my_col0 + c;
                if (n_ok) p.acc_dump[(m * p.N + n) * groups + g] = static_cast<int32_t>(v - offset_bits) >> 4;
              }
            }
          }
          if (threadIdx.x == 256) stamp(kTrDrainDone, git);
        }
        if (!ok) break;
        it += static_cast<uint32_t>(n_groups);
      } else {
        const uint32_t buf = item_idx % kAccBufs, aphase = (item_idx / kAccBufs) & 1u;
        if (!wait_on(bar_acc_full + 8 * buf, aphase, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9105);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t r[kCols];
        if (my_cols > 0) {
          tmem_ld_chunk(tmem_base + lane_addr + buf * kAccStride + my_col0, r);
          tmem_wait_ld();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
        if (my_cols > 0) {
#pragma unroll
          for (int c = 0; c < kCols; c += 2) {
            // the unpacked weights are 16 w: a multiple of 16 below 2^28 converts exactly, times 1/16 is exact
            sums2[c / 2] = pack2(static_cast<float>(static_cast<int32_t>(r[c])) * 0.0625f,
                                 static_cast<float>(static_cast<int32_t>(r[c + 1])) * 0.0625f);
          }
        }
      }

      // ---------------------------------------------------------------- end of the item
      // Straight-line code over this warp's (at most 32) columns: every column is independent, so the loads,
      // the arithmetic and the stores of different columns overlap.
      const bool whole = item.g0 == 0 && item.g1 == groups;
      const uint32_t rslot = item_idx % kRowScaleSlots, rphase = (item_idx / kRowScaleSlots) & 1u;
      if (!wait_on(bar_rs_full + 8 * rslot, rphase, abort_flag, kWaitLimitNs)) {
        if (lane == 0) report_timeout(p.status, abort_flag, 9109);
        ok = false;
        break;
      }
      if (threadIdx.x == 256) stamp(kTrItemEnd, 8 * item_idx);
      float wscale = 1.0f;
      if (!kGroup && n_ok) wscale = __ldg(static_cast<const float*>(p.w_scales) + n);
      const bool has_bias = p.bias != nullptr && n_ok;
      const float bias = has_bias ? to_float<OutT>(__ldg(static_cast<const OutT*>(p.bias) + n)) : 0.0f;
      const float* row_scale = reinterpret_cast<const float*>(smem_gen + (rs_base - smem_base)) + rslot * 128 + my_col0;
      // one output element: row scale, weight scale, bias, gate, residual, one rounding to the output type
      auto emit = [&](float v, float rs, int col) {
        float y = kGroup ? __fmul_rn(v, __fmul_rn(rs, kScaleDown)) : __fmul_rn(__fmul_rn(v, rs), wscale);
        if (has_bias) y = __fadd_rn(y, bias);
        const int64_t m = tok0 + my_col0 + col;
        if (n_ok) {
          // gate and residual: a separate multiply and add, each rounded, as an unfused epilogue would
          if (p.gate != nullptr)
            y = __fmul_rn(y, to_float<OutT>(__ldg(static_cast<const OutT*>(p.gate) + (m / p.gate_span) * p.gate_row_stride + n)));
          if (p.residual != nullptr)
            y = __fadd_rn(y, to_float<OutT>(__ldg(static_cast<const OutT*>(p.residual) + m * p.N + n)));
          static_cast<OutT*>(p.out)[m * p.N + n] = from_float<OutT>(y);
        }
      };
      if (whole) {
#pragma unroll
        for (int c = 0; c < kCols; c += 4) {
          if (c < my_cols) {
            const float4 rs = *reinterpret_cast<const float4*>(row_scale + c);
            const float2 lo = unpack2(sums2[c / 2]), hi = unpack2(sums2[c / 2 + 1]);
            emit(__fsub_rn(lo.x, offset_sum), rs.x, c);
            if (c + 1 < my_cols) emit(__fsub_rn(lo.y, offset_sum), rs.y, c + 1);
            if (c + 2 < my_cols) emit(__fsub_rn(hi.x, offset_sum), rs.z, c + 2);
            if (c + 3 < my_cols) emit(__fsub_rn(hi.y, offset_sum), rs.w, c + 3);
          }
        }
      }
      if (kDump && !kGroup && my_cols > 0) {  // channel form: the item's integer sum (exact in fp32: |sum| < 2^24)
        for (int c = 0; c < my_cols; ++c) {
          float v = 0.0f;
#pragma unroll
          for (int k = 0; k < kCols; ++k) {
            const float2 pair = unpack2(sums2[k / 2]);
            v = k == c ? ((k & 1) != 0 ? pair.y : pair.x) : v;
          }
          const int64_t m = tok0 + my_col0 + c;
          if (n_ok) {
            if (whole) p.acc_dump[m * p.N + n] = static_cast<int32_t>(v);
            else atomicAdd(p.acc_dump + m * p.N + n, static_cast<int32_t>(v));  // the launcher cleared the dump
          }
        }
      }
      if (!whole) {
        // split tile: park the partial sums (offset removed), count this CTA in.  The last CTA to arrive adds all
        // partials in K order (so the result does not depend on who was last) and does the epilogue.  Nobody waits
        // for anybody.
        const int t_rel = item.tile - pl.tail_first;
        const size_t slot_floats = static_cast<size_t>(p.tok_tile) * kBlockCh;
        float* mine = p.partials + (static_cast<size_t>(cta) * 2 + item.slot) * slot_floats +
                      static_cast<size_t>(my_col0) * kBlockCh + ch_in_tile;
#pragma unroll
        for (int c = 0; c < kCols; c += 2) {
          const float2 pair = unpack2(sums2[c / 2]);
          if (c < my_cols) __stcg(mine + c * kBlockCh, __fsub_rn(pair.x, offset_sum));
          if (c + 1 < my_cols) __stcg(mine + (c + 1) * kBlockCh, __fsub_rn(pair.y, offset_sum));
        }
        const int total = pl.tail_tiles * groups;
        const int lo_unit = t_rel * groups, hi_unit = lo_unit + groups;
        int c_lo = static_cast<int>((static_cast<long long>(lo_unit) * pl.tail_ctas) / total);
        while (c_lo + 1 < pl.tail_ctas && unit_start(c_lo + 1, total, pl.tail_ctas) <= lo_unit) ++c_lo;
        while (c_lo > 0 && unit_start(c_lo, total, pl.tail_ctas) > lo_unit) --c_lo;
        int c_hi = c_lo;
        while (c_hi + 1 < pl.tail_ctas && unit_start(c_hi + 1, total, pl.tail_ctas) < hi_unit) ++c_hi;
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_meet);
        if (!wait_on(bar_meet, meets & 1u, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9108);
          ok = false;
          break;
        }
        ++meets;
        if (threadIdx.x == 256) {
          const int before = atomicAdd(p.counters + t_rel, 1);
          *last_flag = before == (c_hi - c_lo) ? 1 : 0;
          __threadfence();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_meet);
        if (!wait_on(bar_meet, meets & 1u, abort_flag, kWaitLimitNs)) {
          if (lane == 0) report_timeout(p.status, abort_flag, 9108);
          ok = false;
          break;
        }
        ++meets;
        if (*last_flag != 0) {
          __threadfence();
          // eight columns at a time: the loads of one contributor are independent of each other
          for (int c0 = 0; c0 < my_cols; c0 += 8) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
            for (int c = c_lo; c <= c_hi; ++c) {
              const int first_tile = unit_start(c, total, pl.tail_ctas) / groups;
              const int slot = first_tile == t_rel ? 0 : 1;
              const float* theirs = p.partials + (static_cast<size_t>(c) * 2 + slot) * slot_floats +
                                    static_cast<size_t>(my_col0 + c0) * kBlockCh + ch_in_tile;
              float part[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) part[j] = c0 + j < my_cols ? __ldcg(theirs + j * kBlockCh) : 0.0f;
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], part[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c0 + j < my_cols) emit(acc[j], row_scale[c0 + j], c0 + j);
          }
        }
      }
      if (threadIdx.x == 256) stamp(kTrItemEnd, 8 * item_idx + 7);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_rs_empty + 8 * rslot);
      ++item_idx;
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

int round_up16(int64_t v) { return static_cast<int>((v + 15) & ~int64_t{15}); }

// Tokens per tile: the tiles of a token axis are equal, a multiple of 16, at most 128.
int pick_tok_tile(int64_t M) {
  const int64_t tok_tiles = (M + 127) / 128;
  const int t = round_up16((M + tok_tiles - 1) / tok_tiles);
  return t < 16 ? 16 : (t > 128 ? 128 : t);
}

constexpr int kSplitOverheadUnits = 3;  // what parking and adding the partials of a split tile costs, in 128-K blocks
constexpr int kMinUnitsPerCta = 2;

// Deal `tiles` tiles of `groups` K blocks to at most `sms` CTAs.  With `may_split` the remainder of the last wave
// is cut along K when that is cheaper than one more whole wave.
Plan make_plan(int ch_tiles, int tok_tiles, int groups, int sms, bool may_split, int* grid_out) {
  Plan pl;
  pl.ch_tiles = ch_tiles; pl.tok_tiles = tok_tiles; pl.tiles = ch_tiles * tok_tiles; pl.groups = groups;
  const int tiles = pl.tiles;
  const int rounds = tiles / sms, rest = tiles % sms;
  pl.full_rounds = rounds + (rest > 0 ? 1 : 0);
  pl.tail_first = tiles; pl.tail_tiles = 0; pl.tail_ctas = 0;
  int grid = tiles < sms ? tiles : sms;
  if (may_split && rest > 0 && groups >= 2 * kMinUnitsPerCta) {
    const int units = rest * groups;
    int ctas = units / kMinUnitsPerCta < sms ? units / kMinUnitsPerCta : sms;
    if (ctas > rest) {
      const int split_cost = (units + ctas - 1) / ctas + kSplitOverheadUnits;
      if (split_cost < groups) {
        pl.full_rounds = rounds;
        pl.tail_first = rounds * sms;
        pl.tail_tiles = rest;
        pl.tail_ctas = ctas;
        grid = rounds > 0 ? sms : ctas;
      }
    }
  }
  *grid_out = grid;
  return pl;
}

size_t split_bytes_for(int tok_tile, int sms) {
  return 1024 /*counters*/ + static_cast<size_t>(sms) * 2 * static_cast<size_t>(tok_tile) * kBlockCh * sizeof(float);
}

template <int TOK, bool kGroup, bool kEvenOdd, bool kDump, typename OutT, bool kTrace = false>
int launch_variant(const GemmArgs& a, int tok_tile, cudaStream_t stream, long long* timeline = nullptr) {
  auto kernel = sq_gemm_ts_kernel<TOK, kGroup, kEvenOdd, kDump, OutT, kTrace>;
  constexpr uint32_t smem = smem_bytes_for(TOK);
  static bool configured[64] = {false};
  static int launch_regs[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SQ_ERR_DRIVER;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess) return static_cast<int>(e);
    launch_regs[dev] = attr.numRegs;
    configured[dev] = true;
  }
  // never launch a register split the CTA cannot satisfy
  if (launch_regs[dev] * kThreads < kRegisterPoolNeeded) return SQ_ERR_DRIVER;
  CUtensorMap tmap_codes, tmap_packed;
  if (!make_map(&tmap_codes, a.codes, static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.K),
                static_cast<uint32_t>(tok_tile), kBlockK, CU_TENSOR_MAP_SWIZZLE_128B))
    return SQ_ERR_DRIVER;
  if (!make_map(&tmap_packed, a.w_packed, static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 2), kBlockCh,
                kBlockK / 2, CU_TENSOR_MAP_SWIZZLE_64B))
    return SQ_ERR_DRIVER;
  TsParams p;
  p.w_scales = a.w_scales; p.row_scales = a.row_scales; p.bias = a.bias; p.out = a.out;
  p.acc_dump = a.acc_dump; p.timeline = timeline; p.status = device_status_word();
  if (p.status == nullptr) return SQ_ERR_DRIVER;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tok_tile = tok_tile;
  if (a.codes_int4_range) {
    p.offset_word = 0x40404040u; p.offset_bits = 1u << 17; p.offset_unsigned = 0u;   // 32 * 64 * 64
  } else {
    p.offset_word = 0xFFFFFFFFu; p.offset_bits = 32u * 255u * 255u; p.offset_unsigned = 1u;
  }
  p.out_dtype = a.out_dtype;
  {
    static const uint32_t env_flags = [] {
      const char* value = std::getenv("SQ_TS_FLAGS");
      return value != nullptr ? static_cast<uint32_t>(std::strtoul(value, nullptr, 0)) : 0u;
    }();
    p.flags = env_flags;
  }
  p.gate = a.gate; p.gate_span = a.gate_span > 0 ? a.gate_span : 1;
  p.gate_row_stride = a.gate_row_stride; p.residual = a.residual;
  const int ch_tiles = static_cast<int>((a.N + kBlockCh - 1) / kBlockCh);
  const int tok_tiles = static_cast<int>((a.M + tok_tile - 1) / tok_tile);
  const int groups = static_cast<int>((a.K + kBlockK - 1) / kBlockK);
  const int sms = sm_count();
  const bool may_split = a.split_workspace != nullptr && a.split_workspace_bytes >= split_bytes_for(tok_tile, sms);
  int grid = 0;
  p.plan = make_plan(ch_tiles, tok_tiles, groups, sms, may_split, &grid);
  p.partials = nullptr; p.counters = nullptr;
  if (p.plan.tail_tiles > 0) {
    p.counters = static_cast<int*>(a.split_workspace);
    p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a.split_workspace) + 1024);
    if (!a.split_counters_cleared) {
      const cudaError_t e = cudaMemsetAsync(p.counters, 0, 1024, stream);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    if (kDump && !kGroup) {
      const cudaError_t e = cudaMemsetAsync(a.acc_dump, 0, static_cast<size_t>(a.M) * a.N * sizeof(int32_t), stream);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
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
#define SQ_LAUNCH(EO, DUMP)                                                                    \
  (bf16 ? launch_variant<TOK, kGroup, EO, DUMP, __nv_bfloat16>(a, tok_tile, stream)            \
        : launch_variant<TOK, kGroup, EO, DUMP, __half>(a, tok_tile, stream))
#ifdef SQ_TS_PROBE_BUILD  // compile-time probe of one instantiation (register allocation checks)
  return launch_variant<TOK, kGroup, true, false, __nv_bfloat16>(a, tok_tile, stream);
#else
  if (eo) return dump ? SQ_LAUNCH(true, true) : SQ_LAUNCH(true, false);
  return dump ? SQ_LAUNCH(false, true) : SQ_LAUNCH(false, false);
#endif
#undef SQ_LAUNCH
}

template <bool kGroup>
int launch_mode(const GemmArgs& a, cudaStream_t stream) {
  const int t = pick_tok_tile(a.M);
#ifndef SQ_TS_PROBE_BUILD
  if (t <= 32) return launch_tok<32, kGroup>(a, t, stream);
  if (t <= 64) return launch_tok<64, kGroup>(a, t, stream);
#endif
  return launch_tok<128, kGroup>(a, t, stream);
}

// ---------------------------------------------------------------------------------- bounded-wait probe
// One CTA goes through the motions of a pipeline role whose partner never shows up: it owns tensor memory, waits
// on a barrier nobody arrives at with the same bounded wait every role of the GEMM uses (only the limit is
// shorter), gives up, records its code, releases tensor memory and returns.  The context stays usable.
__global__ void __launch_bounds__(128, 1) sq_wait_probe_kernel(uint64_t limit_ns, int* status, long long* waited_ns) {
  __shared__ __align__(8) uint64_t barrier_word;
  __shared__ uint32_t tmem_slot_word;
  __shared__ int abort_word;
  const uint32_t bar = smem_u32(&barrier_word);
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot_word), 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&tmem_slot_word);
  if (warp == 1) {
    const uint64_t start = global_timer_ns();
    const bool arrived = mbar_wait_light(bar, 0, abort_flag, limit_ns);
    if (!arrived && (threadIdx.x & 31) == 0) {
      report_timeout(status, abort_flag, 9190);
      if (waited_ns != nullptr) *waited_ns = static_cast<long long>(global_timer_ns() - start);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 32);
  }
}

}  // namespace

int launch_wait_probe(int64_t limit_us, long long* waited_ns, cudaStream_t stream) {
  if (limit_us <= 0 || limit_us > 100000) return SQ_ERR_SHAPE;  // at most 0.1 s: this wait is meant to run out
  int* status = device_status_word();
  if (status == nullptr) return SQ_ERR_DRIVER;
  sq_wait_probe_kernel<<<1, 128, 0, stream>>>(static_cast<uint64_t>(limit_us) * 1000ull, status, waited_ns);
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? SQ_OK : static_cast<int>(err);
}

size_t gemm_split_workspace_bytes(int64_t M) {
  if (M <= 0) return 0;
  // enough for either kernel: this one's two partial tiles per thread block, or the first-generation kernel's one
  // part of a tile of up to 128 tokens per thread block
  const size_t here = split_bytes_for(pick_tok_tile(M), sm_count());
  const int64_t tokens = M < 128 ? ((M + 15) / 16) * 16 : 128;
  const size_t first = 1024 + static_cast<size_t>(sm_count()) * static_cast<size_t>(tokens) * kBlockCh * sizeof(float);
  return here > first ? here : first;
}

int launch_gemm_ts_timeline(const GemmArgs& a, long long* timeline, cudaStream_t stream) {
  int v = validate_gemm(a);
  if (v != SQ_OK) return v;
  if (timeline == nullptr) return SQ_ERR_NULL;
  if (a.wscale_mode != SQ_WSCALE_GROUP_F16 || a.codes_layout != SQ_CODES_EVEN_ODD || a.out_dtype != SQ_BF16 ||
      a.M <= 64 || a.weights_prepacked)
    return SQ_ERR_ENUM;
  return launch_variant<128, true, true, false, __nv_bfloat16, true>(a, pick_tok_tile(a.M), stream, timeline);
}

int launch_gemm_ts(const GemmArgs& a, cudaStream_t stream) {
  if (a.M == 0) return SQ_OK;  // nothing to do; an empty tensor may come with a null pointer
  int v = validate_gemm(a);
  if (v != SQ_OK) return v;
  if (a.weights_prepacked) return SQ_ERR_ENUM;
  if (a.wscale_mode == SQ_WSCALE_GROUP_F16) return launch_mode<true>(a, stream);
  return launch_mode<false>(a, stream);
}

}  // namespace sq

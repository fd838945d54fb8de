/* C ABI of libsq_b200.so: the SteerQuant quantized-linear path on NVIDIA B200 (sm_100a).
 *
 * One quantized linear is two launches on the caller's stream:
 *   sq_prepass  bf16/fp16 activations -> [randomized Hadamard] -> [1/D] -> int8 codes + fp32 row scales
 *   sq_gemm     codes x packed-int4 weights -> int32 (tcgen05 kind::i8, TMEM) -> scales, bias -> bf16/fp16
 *
 * All pointers are DEVICE pointers unless a name ends in _host.  Nothing here allocates,
 * synchronises the host or reads device memory on the host, so every call may be recorded into
 * a CUDA graph.  `stream` is a cudaStream_t passed as void*.  Every function returns 0 on
 * success, a negative SQ_ERR_* for a rejected argument (nothing was launched) or the positive
 * CUDA error of a failed launch.  sq_status_string() names any of them.
 *
 * Citations name the file and lines of the reference project (CathyyW/Fastwamjoint-quantization,
 * paths below src/fastwam_steerquant/) whose role each entry point takes over.
 */
#ifndef SQ_B200_H
#define SQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SQ_OK 0
#define SQ_ERR_NULL (-1)      /* a required pointer is null                            */
#define SQ_ERR_SHAPE (-2)     /* sizes violate the alignment rules stated per function */
#define SQ_ERR_ENUM (-3)      /* an enum-like int argument is out of range             */
#define SQ_ERR_INDEX (-4)     /* schedule index outside [0, calls)                     */
#define SQ_ERR_DRIVER (-5)    /* the CUDA driver refused a tensor-map encode           */
#define SQ_ERR_WORKSPACE (-6) /* workspace smaller than sq_workspace_bytes()           */
#define SQ_ERR_DEVICE_WAIT (-7) /* a kernel gave up a bounded wait (see sq_device_status) */
#define SQ_ERR_SCRATCH_LIMIT (-8) /* sq_linear_noalloc: the linear needs more scratch than the library owns */

/* element types of activations / outputs */
#define SQ_BF16 0
#define SQ_FP16 1

/* activation quantizer modes */
#define SQ_ACT_STATIC 0 /* per-call scale, per-stream gain: code = rn(x * inv_d * (gain / scale)) */
#define SQ_ACT_TOKEN 1  /* per-token dynamic:               code = rn(x * inv_d / (amax / qmax))  */

/* order of the codes along K inside each run of 8 */
#define SQ_CODES_NATURAL 0 /* k, k+1, ..., k+7                                                     */
#define SQ_CODES_EVEN_ODD 1 /* k, k+2, k+4, k+6, k+1, k+3, k+5, k+7 (what sq_gemm unpacks fastest) */
/* sq_gemm only, OR-ed onto the layout: a promise that every code lies in [-8, 7] (what sq_prepass writes for
 * abits = 4).  The group-scale kernel then starts each accumulator at 2^17 instead of 2^21, which is faster and
 * loses less fp32 precision; codes outside the range under this promise give wrong sums. */
#define SQ_CODES_INT4_RANGE 2

/* normalisation fused in front of the quantizer (sq_linear_fused) */
#define SQ_NORM_NONE 0
#define SQ_NORM_LAYER 1 /* (x - mean) * rsqrt(var + eps), no affine (the reference's fused AdaLN producer) */
#define SQ_NORM_RMS 2   /* x * rsqrt(mean(x^2) + eps) [* weight] */

/* activation fused in front of the quantizer or behind the GEMM (sq_linear_fused) */
#define SQ_ACT_FN_NONE 0
#define SQ_ACT_FN_GELU 1 /* exact (erf) GELU */

/* weight-scale forms */
#define SQ_WSCALE_CHANNEL_F32 0 /* float  [N]          (reference: checkpoint.py:49-50, runtime.py:89) */
#define SQ_WSCALE_GROUP_F16 1   /* __half [N, K / 128] (group-128 scheme of the benchmark)             */

/* OR-ed onto wscale_mode of sq_gemm / sq_linear*: `w_packed` is not the packed int4 matrix but the int8 [N, K]
 * matrix sq_prepack_weights made from it.  The GEMM then loads operand tiles directly and skips its unpack
 * stage (faster once the GEMM is compute-bound; twice the weight bytes, so not for small M).  Needs
 * SQ_CODES_EVEN_ODD codes; acc_dump must be null. */
#define SQ_WEIGHTS_PREPACKED 4

/* Fused activation pre-pass.
 * Replaces the producer kernels quantize_static_per_tensor_stream_kernel (kernels/w4a8/csrc/w4a8.cu:838-881),
 * quantize_dynamic_per_token_kernel (w4a8.cu:693-747), quantize_static_stream_s4_kernel and
 * quantize_per_token_s4_kernel (kernels/w4a4/csrc/w4a4.cu:1085-1124, 918-961) and the rotate-then-quantize
 * producer (kernels/w4a4/csrc/rht.cuh:8-61) for block-local power-of-two rotations.
 *
 *   x            [rows, K] bf16 or fp16 (x_dtype), row-major, 16-byte aligned
 *   abits        8 or 4: codes are clamped to +-127 or +-7 (symmetric, as the reference)
 *   mode         SQ_ACT_STATIC or SQ_ACT_TOKEN
 *   inv_d        [K] fp32 multiplier 1/D, or null
 *   signs        [K] fp32 +-1, or null for no rotation
 *   rht_block    rotation block length: a power of two in [8, 256] dividing K (ignored when signs is null).
 *                The rotated value is rounded to x_dtype before quantization (reference contract
 *                rht_install.py:46-49, rht.cuh:55-56).
 *   act_scale    static mode: pointer to THIS call's activation scale (one float)
 *   gains        static mode: pointer to THIS call's row of stream gains [streams]
 *   span         static mode: > 0: row r belongs to stream (r / span) % streams;
 *                < 0: rows with (r % seq_tokens) >= seq_tokens + span belong to stream 1, others to 0
 *                (w4a8.cu:857-861)
 *   codes_layout SQ_CODES_NATURAL or SQ_CODES_EVEN_ODD
 *   pack_int4    0: int8 codes [rows, K]; 1: two codes per byte [rows, K/2], low nibble = even k
 *                (only with abits == 4 and SQ_CODES_NATURAL; the reference's A4 storage, w4a4.cu:1119-1123)
 *   codes        out, 16-byte aligned
 *   row_scales   out fp32 [rows]: static: scale / gain; token: max(amax, tiny) / qmax
 * Alignment: K % 8 == 0 and K <= 32768.
 */
int sq_prepass(const void* x, int x_dtype, int64_t rows, int64_t K, int abits, int mode,
               const float* inv_d, const float* signs, int rht_block,
               const float* act_scale, const float* gains, int64_t span, int64_t streams, int64_t seq_tokens,
               int codes_layout, int pack_int4, void* codes, float* row_scales, void* stream);

/* Quantized GEMM with fused epilogue.
 * Replaces PlainFusedEpilogueGemm + launch_packed_w4a8_gemm (w4a8.cu:309-381, 891-922) and
 * FusedEpilogueGemm + launch_fused_w4a4_gemm (w4a4.cu:257-371, 1217-1249).
 *
 *   codes        int8 [M, K] from sq_prepass (codes_layout says in which order)
 *   w_packed     uint8 [N, K/2]: two's-complement nibbles, low nibble = even k (kernels/w4a8/ops.py:8-14)
 *   w_scales     float [N] (SQ_WSCALE_CHANNEL_F32) or __half [N, K/128] (SQ_WSCALE_GROUP_F16)
 *   row_scales   float [M]
 *   bias         [N] in out_dtype, or null
 *   out          [M, N] bf16/fp16 (out_dtype), row-major
 *   acc_dump     null, or int32 [M, N, G] (G = 1 or K/128): the exact integer accumulators, for parity checks
 * channel form:  out = dtype((float(acc) * row_scale[m]) * w_scale[n] + bias[n])      (w4a8.cu:324-360)
 * group form:    out = dtype((sum_g float(acc_g) * w_scale[n,g]) * row_scale[m] + bias[n]); the sum over groups
 *                is kept in fp32 in the kernel's own order, so outputs match sq_gemm_check to fp32 rounding
 *                (about 1e-4 relative before the cast) while the integer accumulators match bit for bit
 * Alignment: K % 32 == 0 (K % 128 == 0 in group form), N % 8 == 0, all pointers 16-byte aligned.
 */
int sq_gemm(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
            const float* row_scales, const void* bias, void* out, int out_dtype,
            int64_t M, int64_t N, int64_t K, int32_t* acc_dump, void* stream);

/* sq_gemm with scratch for tiles that are split along K.  Whole output tiles (128 channels x up to 128 tokens)
 * are dealt round-robin to one persistent thread block per SM.  With few tokens - the small-M regime of the
 * reference (M = 32 ... 360, w4a8.cu:1038-1076 picks its tile shapes for it) - there are fewer tiles than SMs; when
 * the tiles (of at most 64 tokens) leave at least half of the SMs idle and a tile has enough 128-K blocks for the
 * exchange to pay (K >= 6144 in practice), a tile's K blocks are cut into up to 15 parts, one thread block each.
 * Every part parks its partial sums in `split_workspace`; the one that arrives last at the tile's counter adds
 * them in part order (the result does not depend on the arrival order) and finishes the tile; nobody waits.
 * Integer accumulators are unchanged; group-form outputs differ from the unsplit kernel by fp32 rounding only,
 * channel-form outputs not at all (the partial sums are exact integers).  With acc_dump the kernel never splits.
 *   split_workspace        16-byte aligned, sq_split_workspace_bytes(M) bytes, or null (then this is sq_gemm).
 *                          Its first 1024 bytes are counters; this call puts a memset of them on `stream`.
 * The reference has no counterpart: its CUTLASS GEMMs never split K. */
int sq_gemm_split(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
                  const float* row_scales, const void* bias, void* out, int out_dtype,
                  int64_t M, int64_t N, int64_t K, int32_t* acc_dump,
                  void* split_workspace, size_t split_workspace_bytes, void* stream);
size_t sq_split_workspace_bytes(int64_t M);

/* sq_gemm for a layer whose output channels are split over GPUs (one process per GPU; this GPU holds rows
 * [out_col0, out_col0 + N) of the layer's weight matrix): the [M, N] block goes into columns
 * [out_col0, out_col0 + N) of row-major [M, out_ld] matrices, outs[0] on this GPU and outs[1 .. n_outs) the same
 * matrix on the other GPUs, given as peer pointers (CUDA IPC or any other peer mapping).  The epilogue stores every
 * 64-byte run of a row to all of them, so the all-gather that would follow the GEMM (ncclAllGather plus a local
 * permute into the [M, out_ld] layout) is the GEMM's own NVLink traffic and overlaps its tensor-core work tile by
 * tile.  Plain stores only: no TMA copy and no cluster-wide load touches peer memory.  The caller orders the GPUs around the call
 * (nobody may read a matrix before every GPU's kernel has finished; nobody may start the next call's stores
 * before every reader is done).  M >= 128; packed int4 weights; even-odd codes; bf16 or fp16 output.
 * The reference has no counterpart (it runs on one GPU). */
int sq_gemm_scatter(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
                    const float* row_scales, const void* bias, void* const* outs, int n_outs, int64_t out_ld,
                    int64_t out_col0, int out_dtype, int64_t M, int64_t N, int64_t K, void* stream);

/* Plain-CUDA-core version of sq_gemm with the same arguments (SQ_CODES_INT4_RANGE is accepted and ignored), the
 * same accumulators and, in the group form, the oracle's own fp32 summation order.  It exists so the
 * tensor-core kernel can be cross-checked on the device; it is not a fallback and nothing dispatches to it. */
int sq_gemm_check(const void* codes, int codes_layout, const void* w_packed, const void* w_scales, int wscale_mode,
                  const float* row_scales, const void* bias, void* out, int out_dtype,
                  int64_t M, int64_t N, int64_t K, int32_t* acc_dump, void* stream);

/* Profiling aid with no counterpart in the reference: sq_gemm for the group-scale bf16 case (even-odd codes,
 * M > 128) that also records, for the thread block with index 0, the SM clock at which each pipeline role
 * reached each 128-K block.  `timeline` is int64 [12][512]: rows are TMA issue, unpack start, unpack done,
 * accumulator free, MMA issue, drain start, accumulator released, drain done, MMAs committed, top of the drain loop,
 * accumulator loaded, and (eight slots per work item) the steps of the end-of-item code; unused slots keep their
 * value.  The first-generation kernel (SQ_GEMM_KERNEL=tc) fills the first nine rows only. */
#define SQ_TIMELINE_ROLES 12
#define SQ_TIMELINE_SLOTS 512
int sq_gemm_timeline(const void* codes, const void* w_packed, const void* w_scales, const float* row_scales,
                     const void* bias, void* out, int64_t M, int64_t N, int64_t K, long long* timeline, void* stream);

/* Kernel-native weight form, made once at load time from the on-disk / checkpoint format
 * (uint8 [N, K/2], kernels/w4a8/ops.py:8-14; the deployment loader deployment.py:180-226 keeps that format):
 * w_tiled is int8 [N, K], every byte 16 w, in the even-odd k order of SQ_CODES_EVEN_ODD
 * (k, k+2, k+4, k+6, k+1, k+3, k+5, k+7 within each run of 8).  K % 32 == 0, pointers 16-byte aligned. */
int sq_prepack_weights(const void* w_packed, int64_t N, int64_t K, void* w_tiled, void* stream);

/* Profiling aid with no counterpart in the reference: one warp per SM issues `iterations` x 4
 * tcgen05.mma.kind::i8 (M = 128, N = n_cols in {64, 128, 256}, K = 32) back to back on fixed shared-memory tiles
 * and waits for them; `cycles` (device int64) receives thread block 0's SM cycles from first issue to
 * completion, so cycles / (4 * iterations) is the tensor pipe's time per MMA of that shape.  n_cols = 0x1000 + 128
 * measures the N = 128 shape with operand A read from tensor memory instead of shared memory. */
int sq_mma_rate(int n_cols, int iterations, long long* cycles, void* stream);

/* Bytes of scratch one linear needs between sq_prepass and sq_gemm (codes + row scales), 256-byte rounded.
 * Takes the place of the per-call torch::empty of run_static_streams (w4a8.cu:1358-1360). */
size_t sq_workspace_bytes(int64_t M, int64_t K);

/* One whole linear: sq_prepass into `workspace`, then sq_gemm.  Same role as run_static_streams
 * (w4a8.cu:1337-1387, w4a4.cu:1517-1574) / symmetric_dynamic (w4a8.cu:1389-1452).
 * A workspace of at least sq_workspace_bytes(rows, K) + sq_split_workspace_bytes(rows) bytes also lets the GEMM
 * split tiles along K (see sq_gemm_split); the pre-pass clears the counters, so no memset is added.
 * `calls` and `call` select the schedule entry in static mode: act_scales [calls], gains [calls, streams];
 * an index outside [0, calls) is SQ_ERR_INDEX (w4a8.cu:1587-1628). */
int sq_linear(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
              const float* inv_d, const float* signs, int rht_block,
              const float* act_scales, const float* gains, int64_t calls, int64_t call,
              int64_t span, int64_t streams, int64_t seq_tokens,
              const void* w_packed, const void* w_scales, int wscale_mode, const void* bias,
              void* out, void* workspace, size_t workspace_bytes, void* stream);

/* The composite rotation of widths K = order x part with part a power of two in [8, 512]: the reference's
 * had12 x H256 at K = 3072 and had28 x H512 at K = 14336 (rht.py:27-39; device producer rht.cuh:8-100).
 * Per row: multiply by `signs`, normalised FWHT of every `part` consecutive elements, then
 * out[i * part + c] = (sum_j mix[i, j] * h[j * part + c]) / sqrt(order), rounded to x_dtype; the rest is
 * sq_prepass / sq_linear.  `mix` is float [order, order] with entries +-1 (the caller's Hadamard matrix of that
 * order, device memory), 2 <= order <= 32, K <= 16384.  The sum over j runs in ascending j in fp32, which is
 * not the reference's BLAS order: rotated values agree to fp32 rounding, codes to +-1 on a few in ten thousand.
 * `call_index` of sq_linear_composite: null, or a device int32 read when the kernel runs (see sq_linear_scheduled). */
int sq_prepass_composite(const void* x, int x_dtype, int64_t rows, int64_t K, int abits, int mode, const float* inv_d,
                         const float* signs, const float* mix, int mix_order, const float* act_scale,
                         const float* gains, int64_t span, int64_t streams, int64_t seq_tokens, int codes_layout,
                         int pack_int4, void* codes, float* row_scales, void* stream);
int sq_linear_composite(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                        const float* inv_d, const float* signs, const float* mix, int mix_order,
                        const float* act_scales, const float* gains, int64_t calls, int64_t call,
                        const int32_t* call_index, int64_t span, int64_t streams, int64_t seq_tokens,
                        const void* w_packed, const void* w_scales, int wscale_mode, const void* bias, void* out,
                        void* workspace, size_t workspace_bytes, void* stream);

/* sq_linear with work of the surrounding block folded into its two kernels.
 * Pre-pass side, replaces quantize_static_adaln_stream_kernel / quantize_dynamic_adaln_per_token_kernel
 * (w4a8.cu:519-691) and their int4 forms (w4a4.cu:963-1049, 1126-1211): optionally an activation of the input
 * (input_activation, SQ_ACT_FN_*, result rounded to x's dtype), then a normalisation of each row
 * (norm_kind, norm_eps, optional norm_weight [K] for RMS), then y = (1 + mod_scale) * y + mod_shift with one
 * modulation row per mod_span input rows (rows mod_row_stride elements apart; both null for none), optionally
 * rounded to x's dtype (round_after_norm, what an unfused module boundary would do), then the pre-pass proper.
 * GEMM side, replaces GatedResidualEpilogueGemm (w4a8.cu:383-479): out = residual + gate * linear, with gate rows
 * of N (one per gate_span output rows, gate_row_stride elements apart, null for none) and residual [rows, N]
 * (null for none), all in fp32 before the single rounding to out's dtype.  `activation` must be
 * SQ_ACT_FN_NONE: an activation is fused on the input side of the linear that consumes it (input_activation),
 * where it costs nothing; in the GEMM epilogue it measured slower than a separate kernel. */
int sq_linear_fused(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                    const float* inv_d, const float* signs, int rht_block,
                    const float* act_scales, const float* gains, int64_t calls, int64_t call,
                    int64_t span, int64_t streams, int64_t seq_tokens,
                    const void* w_packed, const void* w_scales, int wscale_mode, const void* bias,
                    int input_activation, int norm_kind, float norm_eps, const void* norm_weight,
                    const void* mod_scale, const void* mod_shift, int64_t mod_span, int64_t mod_row_stride,
                    int round_after_norm,
                    int activation, const void* gate, int64_t gate_span, int64_t gate_row_stride,
                    const void* residual,
                    void* out, void* workspace, size_t workspace_bytes, void* stream);

/* sq_linear_fused with the schedule entry chosen on the device: when `call_index` (device int32) is not null,
 * static mode reads act_scales[*call_index] and gains[*call_index, :] when the kernel runs (clamped to
 * [0, calls)); `call` is then ignored.  One captured CUDA graph serves every denoise call: the host changes the
 * integer between replays.  The reference bakes the entry into each capture (pointer arithmetic on the host,
 * w4a8.cu:1362-1363) and therefore keeps one graph per call (rollout_graph.py:111-155). */
int sq_linear_scheduled(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                        const float* inv_d, const float* signs, int rht_block,
                        const float* act_scales, const float* gains, int64_t calls, int64_t call,
                        const int32_t* call_index, int64_t span, int64_t streams, int64_t seq_tokens,
                        const void* w_packed, const void* w_scales, int wscale_mode, const void* bias,
                        int input_activation, int norm_kind, float norm_eps, const void* norm_weight,
                        const void* mod_scale, const void* mod_shift, int64_t mod_span, int64_t mod_row_stride,
                        int round_after_norm, int activation, const void* gate, int64_t gate_span,
                        int64_t gate_row_stride, const void* residual,
                        void* out, void* workspace, size_t workspace_bytes, void* stream);

/* sq_linear for callers that cannot allocate device memory.  It has no counterpart in the reference, whose
 * operators always allocate their scratch per call (torch::empty, w4a8.cu:1358-1360).
 *
 * Who needs it: code that runs after a point where allocation is off the table - a control loop that must
 * not hit the implicit device synchronisation of cudaMalloc, a host framework whose own pool already holds
 * all free device memory (so cudaMalloc would simply fail), or a plug-in that is handed device pointers but
 * no allocator.  Such a caller still passes its input, weights and output; the codes and row scales that
 * live between the pre-pass and the GEMM go into an array of SQ_NOALLOC_SCRATCH_BYTES that is part of the
 * library image on every GPU that loads it.  This function calls no cudaMalloc, cudaFree or other
 * allocating routine.
 *
 * Limit: sq_workspace_bytes(rows, K) <= SQ_NOALLOC_SCRATCH_BYTES, i.e. about rows * K <= 8 Mi elements
 * (2048 x 3072 fits, 4096 x 3072 does not); larger calls return SQ_ERR_SCRATCH_LIMIT and launch nothing.
 * The first call on a device looks the array's address up (cudaGetSymbolAddress, with that device current);
 * make that first call outside any stream capture.
 * All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it needs
 * clearing (each call overwrites what it reads), but two calls that overlap on the GPU - different streams
 * without an ordering between them - race on it; order them.
 * Arguments and results are those of sq_linear without `workspace` / `workspace_bytes`. */
#define SQ_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u + 65536u)
int sq_linear_noalloc(const void* x, int x_dtype, int64_t rows, int64_t K, int64_t N, int abits, int mode,
                      const float* inv_d, const float* signs, int rht_block,
                      const float* act_scales, const float* gains, int64_t calls, int64_t call,
                      int64_t span, int64_t streams, int64_t seq_tokens,
                      const void* w_packed, const void* w_scales, int wscale_mode, const void* bias,
                      void* out, void* stream);

/* Test aid with no counterpart in the reference: proves that a wait which runs out ends as a status, not as a hung
 * GPU.  One thread block allocates tensor memory, waits at most `limit_us` microseconds (1 ... 100000) on a barrier
 * nobody ever arrives at - through the same bounded wait every pipeline role of sq_gemm uses, whose own limit is
 * one second - then records status 9190, frees its tensor memory and returns; `waited_ns` (device int64, or
 * null) receives how long it waited.  sq_device_status() then returns 9190 once, and the context stays usable. */
int sq_wait_probe(int64_t limit_us, long long* waited_ns, void* stream);

/* Reads (and clears) the device-side status word of the current device.  Kernels never spin forever:
 * a wait that exceeds its time limit records a code here and the kernel returns.  0 = no kernel gave up.
 * Synchronises the device; not for use during stream capture. */
int sq_device_status(void);

const char* sq_status_string(int status);

/* Library build tag, e.g. "sq_b200 sm_100a". */
const char* sq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SQ_B200_H */

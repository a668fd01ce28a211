/* C ABI of the sm_100a kernel library ("ops/cuda", the sibling of the reference's empty
 * ops/cpu/ops.h).  One entry point per kernel family; each is the CUDA replacement for
 * the code the reference generates for the named LLH ops.  Pointers are device pointers,
 * extents and strides are in elements, `stream` is a cudaStream_t (NULL = legacy default
 * stream).  Every function returns 0 or an LlcStatus (llc_runtime.h) and records a message
 * readable with llc_last_error().  Nothing here allocates device memory.
 */
#ifndef LLC_CUDA_H_
#define LLC_CUDA_H_

#include <stdint.h>

#include "llc_runtime.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum LlcAct { LLC_ACT_NONE = 0, LLC_ACT_RELU = 1, LLC_ACT_GELU = 2 } LlcAct;
typedef enum LlcPrecision { LLC_PREC_FP32 = 0, LLC_PREC_TF32 = 1, LLC_PREC_TF32X3 = 2, LLC_PREC_BF16 = 3 } LlcPrecision;

/* out[b0,b1,m,n] = act(alpha * scale[n] * sum_k A[b0,b1,m,k] * B[b0,b1,k,n] + shift[n] + res[b0,b1,m,n])
 * Replaces llh.matmul / llh.batch_matmul (-> stablehlo.dot / dot_general,
 * src/Conversion/LLHToHLO/LLHToHLO.cpp:363-382, :485) together with the elementwise ops that
 * follow it in the graph (bias add, ReLU = max(x,0) LLHPreprocessingForHLO.cpp:76-101, residual).
 * A must have unit stride along k.  B has unit stride along k (b_sk == 1, weights stored [n][k])
 * or along n (b_sn == 1).  scale/shift/res may be NULL.  Accumulation is fp32. */
typedef struct LlcGemmParams {
  const void* a; const void* b; void* out;
  const float* scale; const float* shift; const void* res;
  int32_t in_dtype;    /* LLC_FLOAT32 or LLC_BFLOAT16, both operands */
  int32_t out_dtype;   /* LLC_FLOAT32 or LLC_BFLOAT16 */
  int32_t res_dtype;
  int32_t precision;   /* LlcPrecision; LLC_PREC_FP32 = FMA path */
  int64_t m, n, k, b0, b1;
  int64_t a_s0, a_s1, a_sm;            /* strides of A: batch0, batch1, row (k stride is 1) */
  int64_t b_s0, b_s1, b_sk, b_sn;
  int64_t o_s0, o_s1, o_sm;            /* n stride is 1 */
  int64_t r_s0, r_s1, r_sm, r_sn;
  float alpha;
  int32_t act;         /* LlcAct */
  /* Optional scratch for the split-K path (few output tiles, long K): device memory, 16-byte
   * aligned, whose first 4096 bytes are zero before the first use (the kernel leaves them zero).
   * NULL disables split-K.  Launches that share one workspace must not overlap on the GPU. */
  void* workspace;
  int64_t workspace_bytes;
  /* Optional, precision tf32x3 only: B - truncate_to_tf32(B), laid out exactly like b (same strides).  When given, the
   * kernel loads it instead of splitting every B tile itself; weights are split once at load time this way. */
  const void* b_lo;
} LlcGemmParams;
int llc_cuda_gemm(const LlcGemmParams* p, void* stream);

/* llc_cuda_gemm on the FMA path for callers that must not allocate device memory (a process whose
 * own pool already owns the GPU, a loop that cannot take the synchronisation an allocation
 * implies).  No counterpart in the reference.  The split-K scratch is a 1 MiB array built into the
 * library (each GPU that loads the library holds it until exit); `workspace` in the parameter block
 * is ignored.  A shape whose split needs more than 1 MiB is refused with LLC_ERR_ARGUMENT.  The
 * first call on a device looks up the array's device address (cudaGetSymbolAddress); make that
 * first call before starting any stream capture.  All calls share the one array: launches that
 * overlap on the GPU (different streams or threads of one process on one device) race.
 * Calls no cudaMalloc / cudaFree. */
int llc_cuda_gemm_static_scratch(const LlcGemmParams* p, void* stream);

/* out[b0,b1,m,:] = softmax_n(scale * sum_d Q[b0,b1,m,d] K[b0,b1,n,d] + mask[b0,b1,m,n]) V[b0,b1,n,:] in one kernel: the
 * scores stay in tensor memory, the probabilities in shared memory (keys in blocks of 128, running softmax).  Replaces the chain llh.batch_matmul -> llh.div /
 * llh.add (scale, mask) -> softmax (decomposed by llcompiler/compiler/torch_compile_config.py:24) -> llh.batch_matmul that
 * the reference lowers op by op (src/Conversion/LLHToHLO/LLHToHLO.cpp:363-382).  bf16 operands and output with unit
 * stride along d, d == 64, 1 <= n <= 512; every other stride a non-negative multiple of 8 elements (0 = broadcast for
 * batch strides), pointers 16-byte aligned.  mask may be NULL; it has unit stride along n and may broadcast over
 * b0, b1 and m (stride 0).  Anything else returns LLC_ERR_UNSUPPORTED. */
typedef struct LlcAttentionParams {
  const void* q; const void* k; const void* v; const void* mask; void* out;
  int32_t dtype;        /* LLC_BFLOAT16 */
  int32_t mask_dtype;   /* LLC_FLOAT32 or LLC_BFLOAT16 */
  int64_t b0, b1, m, n, d;
  int64_t q_s0, q_s1, q_sm;
  int64_t k_s0, k_s1, k_sn;
  int64_t v_s0, v_s1, v_sn;
  int64_t o_s0, o_s1, o_sm;
  int64_t mask_s0, mask_s1, mask_sm;
  float scale;
} LlcAttentionParams;
int llc_cuda_attention(const LlcAttentionParams* p, void* stream);

/* Health word of the tensor-core kernels.  Their waits on memory barriers are bounded; a wait that
 * gives up records 1 (producer), 2 (issuer), 3 (operand split), 4 (epilogue), 5 (gather), 6 or 7 (attention) and the launch's
 * result is then invalid.  Returns the recorded code (0 = healthy) and clears it; -1 if the device
 * cannot be read.  Synchronises the device.  No counterpart in the reference. */
int llc_cuda_status(void);

/* NHWC implicit-GEMM convolution with the same epilogue; replaces llh.conv
 * (-> stablehlo.convolution, LLHToHLO.cpp:214-270), the decomposed batch-norm inference that
 * follows it (src/Dialect/LLH/Transforms/DecomposeOps.cpp:125-144, folded to scale/shift),
 * the residual add and the ReLU.  x is [N,H,W,C], w is [F,KH,KW,C], out and res are [N,OH,OW,F]. */
typedef struct LlcConvParams {
  const void* x; const void* w; void* out;
  const float* scale; const float* shift; const void* res;
  int32_t in_dtype, out_dtype, res_dtype, precision;
  int64_t n, h, w_in, c, f, kh, kw, oh, ow;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  float alpha;
  int32_t act;
  const void* w_lo;   /* optional, precision tf32x3: w - truncate_to_tf32(w), same layout as w (see LlcGemmParams.b_lo) */
  /* Optional element strides of x along n, h and w (the channel stride is 1); all 0 = dense [N,H,W,C].  The strides may
   * describe an overlapping view: with x_sw < c every "pixel" is a window of c consecutive elements that advances by x_sw,
   * which turns a filter row of a narrow-channel convolution into the channels of a 1-wide kernel.  Tensor-core precisions
   * only (bf16, tf32, tf32x3); c * element size must then be a multiple of 16 bytes and so must the strides. */
  int64_t x_sn, x_sh, x_sw;
  /* Optional scratch for split-K (few output tiles, long K), as in LlcGemmParams: device memory, 16-byte aligned, first
   * 4096 bytes zero before the first use (left zero).  NULL disables split-K. */
  void* workspace;
  int64_t workspace_bytes;
} LlcConvParams;
int llc_cuda_conv2d(const LlcConvParams* p, void* stream);

/* NHWC max pooling; replaces llh.max_pool (-> stablehlo.reduce_window, LLHToHLO.cpp:295-339).
 * Padding taps are skipped (equivalent to a -inf initial value; the reference initialises
 * with 0, :313-314). */
typedef struct LlcPoolParams {
  const void* x; void* out;
  int32_t in_dtype, out_dtype;
  int64_t n, h, w, c, oh, ow;
  int32_t kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
} LlcPoolParams;
int llc_cuda_maxpool2d(const LlcPoolParams* p, void* stream);

/* out[o,i] = reduce_r x[o,r,i]; x dense [outer,R,inner].  op: 0 sum, 1 max, 2 min, 3 mean.
 * Replaces llh.reduce_sum/max/min (-> stablehlo.reduce, LLHToHLO.cpp:81-171) and the global
 * average pool (llh.adaptive_average_pool, declared without a lowering, LLHOps.td:337-339). */
int llc_cuda_reduce(const void* x, void* out, int32_t in_dtype, int32_t out_dtype, int64_t outer,
                    int64_t r, int64_t inner, int32_t op, void* stream);

/* Row softmax over dense [rows, len]; replaces the amax/sub/exp/sum/div chain of the
 * reference's decomposition (llcompiler/compiler/torch_compile_config.py:24). */
int llc_cuda_softmax(const void* x, void* out, int32_t in_dtype, int32_t out_dtype, int64_t rows,
                     int64_t len, void* stream);

/* Row LayerNorm over dense [rows, d] with fp32 statistics; llh.layer_norm is declared by the
 * reference (LLHOps.td:454-463) without a lowering. */
int llc_cuda_layernorm(const void* x, const void* gamma, const void* beta, void* out, int32_t in_dtype,
                       int32_t param_dtype, int32_t out_dtype, int64_t rows, int64_t d, float eps, void* stream);

/* out[r,:] = table[ids[r],:]; ids are int64.  Rows with an id outside [0, vocab) are written
 * as zeros and counted in *bad_ids when bad_ids is not NULL (a device int32). */
int llc_cuda_gather(const void* table, const int64_t* ids, void* out, int32_t table_dtype, int32_t out_dtype,
                    int64_t rows, int64_t d, int64_t vocab, int32_t* bad_ids, void* stream);

/* x [n, c, hw] (NCHW planes) -> out [n, hw, c_pad] (NHWC pixels), channels c..c_pad-1 written as
 * zeros.  The layout change the reference expresses as llh.transpose perms [0,2,3,1] around conv
 * (src/Dialect/LLH/Transforms/TransformLayout.cpp:141-198), with the channel padding the
 * tensor-core convolution wants for a 3-channel stem. */
int llc_cuda_nchw_to_nhwc(const void* x, void* out, int32_t dtype, int64_t n, int64_t c, int64_t hw, int64_t c_pad, void* stream);

/* The same re-layout into rows of w_total pixels: the image starts at column w_left, the columns left and right of it are
 * zeros.  out is [n, h, w_total, c_pad]; f32 with c_pad 4 or bf16 with c_pad 8 (16 bytes per pixel).  With the halo in
 * memory, eight neighbouring pixels of a narrow-channel input are one contiguous 128-byte run, which is what lets the stem
 * convolution read a whole filter row per K block (see LlcConvParams.x_sw). */
int llc_cuda_nchw_to_nhwc_wide(const void* x, void* out, int32_t dtype, int64_t n, int64_t c, int64_t h, int64_t w, int64_t c_pad, int64_t w_left,
                               int64_t w_total, void* stream);

/* Multi-destination copy: `bytes` bytes at `src` are stored at byte offset `dst_offset_bytes` of each of the `n_dst`
 * (at most 8) buffers in `dst` (a host array of device pointers); each source vector is read once.  The destinations may
 * be peer memory of other GPUs (plain stores over NVLink): this is the gather step of batch-sharded inference, every rank
 * pushing its slice of the output into every rank's copy of the full batch; the caller synchronises the ranks before
 * (the destinations are free) and after (every slice has arrived).  No counterpart in the reference, which runs on one
 * device; it stands where its Execution::run results (src/Compiler/Execution.cpp:21-66) of several GPUs are put together. */
int llc_cuda_push_rows(const void* src, void* const* dst, int32_t n_dst, int64_t dst_offset_bytes, int64_t bytes, void* stream);

/* Fused elementwise chain: one coalesced pass that evaluates a small register program per
 * output element.  Replaces chains of llh.add/sub/mul/div/max/min/abs/sqrt/exp/where/compare/
 * convert_to/broadcast_to (-> stablehlo elementwise ops, LLHToHLO.cpp:479-490) and strided
 * copies (llh.transpose -> stablehlo.transpose).  `prog` is ';'-separated instructions, the
 * i-th defines register i: "ld<k>" loads input k, "#<v>" is a constant, "<op>,<a>[,<b>[,<c>]]"
 * applies an op to earlier registers.  All arithmetic is fp32.  Up to 8 inputs, rank <= 6. */
typedef struct LlcEltwiseOperand { const void* data; int32_t dtype; int64_t strides[6]; } LlcEltwiseOperand;
typedef struct LlcEltwiseParams {
  void* out; int32_t out_dtype; int32_t rank;
  int64_t shape[6]; int64_t out_strides[6];
  int32_t n_in; LlcEltwiseOperand in[8];
  const char* prog;
} LlcEltwiseParams;
int llc_cuda_eltwise(const LlcEltwiseParams* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LLC_CUDA_H_ */

// Entry points of the contraction kernels: argument checks and the choice between the
// tensor-core path and the FMA path.
#include "common.cuh"

namespace llc {
int igemmSimtGemm(const LlcGemmParams* p, cudaStream_t st, void* workspace, long long workspaceBytes);
int igemmSimtConv(const LlcConvParams* p, cudaStream_t st);
bool tcGemmSupported(const LlcGemmParams* p);
int tcGemm(const LlcGemmParams* p, cudaStream_t st);
bool tcConvSupported(const LlcConvParams* p);
int tcConv(const LlcConvParams* p, cudaStream_t st);
int tcStatus();
int attnStatus();
}  // namespace llc

using namespace llc;

static bool floatIo(int32_t dt) { return dt == LLC_FLOAT32 || dt == LLC_BFLOAT16; }

extern "C" int llc_cuda_gemm(const LlcGemmParams* p, void* stream) {
  if (!p) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm null parameter block");
  if (p->m < 0 || p->n < 0 || p->k < 0 || p->b0 < 0 || p->b1 < 0) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm negative extent");
  if (p->m == 0 || p->n == 0 || p->b0 == 0 || p->b1 == 0) return LLC_OK;
  if (!p->a || !p->b || !p->out) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm null operand");
  if (!floatIo(p->in_dtype) || !floatIo(p->out_dtype) || (p->res && !floatIo(p->res_dtype)))
    return setError(LLC_ERR_UNSUPPORTED, "llc argument: gemm operands must be f32 or bf16");
  if (tcGemmSupported(p)) return tcGemm(p, (cudaStream_t)stream);
  return igemmSimtGemm(p, (cudaStream_t)stream, p->workspace, p->workspace_bytes);
}

extern "C" int llc_cuda_status(void) {
  const int a = tcStatus(), b = attnStatus();
  return a ? a : b;
}

extern "C" int llc_cuda_conv2d(const LlcConvParams* p, void* stream) {
  if (!p) return setError(LLC_ERR_ARGUMENT, "llc argument: conv null parameter block");
  if (p->n < 0 || p->oh < 0 || p->ow < 0 || p->f < 0) return setError(LLC_ERR_ARGUMENT, "llc argument: conv negative extent");
  if (p->n == 0 || p->oh == 0 || p->ow == 0 || p->f == 0) return LLC_OK;
  if (!p->x || !p->w || !p->out) return setError(LLC_ERR_ARGUMENT, "llc argument: conv null operand");
  if (p->stride_h <= 0 || p->stride_w <= 0 || p->dil_h <= 0 || p->dil_w <= 0 || p->kh <= 0 || p->kw <= 0 || p->c <= 0)
    return setError(LLC_ERR_ARGUMENT, "llc argument: conv stride, dilation, kernel and channel extents must be positive");
  if (!floatIo(p->in_dtype) || !floatIo(p->out_dtype) || (p->res && !floatIo(p->res_dtype)))
    return setError(LLC_ERR_UNSUPPORTED, "llc argument: conv operands must be f32 or bf16");
  if (p->h * p->w_in * p->c >= (1LL << 31) || p->kh * p->kw * p->c >= (1LL << 31)) return setError(LLC_ERR_UNSUPPORTED, "llc argument: conv image or filter too large");
  const bool strided = p->x_sn != 0 || p->x_sh != 0 || p->x_sw != 0;
  if (!strided && p->kh == 1 && p->kw == 1 && p->stride_h == 1 && p->stride_w == 1 && p->pad_h == 0 && p->pad_w == 0) {
    // a 1x1 stride-1 convolution over NHWC data is a plain GEMM: [N*H*W, C] x [F, C]^T
    LlcGemmParams g{};
    g.a = p->x; g.b = p->w; g.out = p->out; g.scale = p->scale; g.shift = p->shift; g.res = p->res;
    g.in_dtype = p->in_dtype; g.out_dtype = p->out_dtype; g.res_dtype = p->res_dtype; g.precision = p->precision;
    g.m = p->n * p->oh * p->ow; g.n = p->f; g.k = p->c; g.b0 = g.b1 = 1;
    g.a_sm = p->c; g.b_sk = 1; g.b_sn = p->c; g.o_sm = p->f; g.r_sm = p->f; g.r_sn = 1;
    g.alpha = p->alpha; g.act = p->act; g.b_lo = p->w_lo;
    if (tcGemmSupported(&g)) return tcGemm(&g, (cudaStream_t)stream);
  }
  if (tcConvSupported(p)) return tcConv(p, (cudaStream_t)stream);
  if (strided) return setError(LLC_ERR_UNSUPPORTED, "llc argument: conv with explicit activation strides needs a tensor-core precision and 16-byte aligned strides");
  return igemmSimtConv(p, (cudaStream_t)stream);
}

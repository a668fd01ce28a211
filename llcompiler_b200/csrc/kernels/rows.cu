// Row kernels: softmax, LayerNorm and reductions.  All are HBM-bound: each input element is
// read once and each output element written once (softmax: 2*rows*len elements, LayerNorm:
// 2*rows*d (+2d parameters), reduce: outer*R*inner + outer*inner).  One warp owns a row when it
// fits in registers (<= 1024 fp32 values per warp as 8 float4 per lane), with 128-bit loads;
// longer rows fall back to a block per row that re-reads the row from L2.
#include "common.cuh"

namespace llc {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxVecPerLane = 8;   // 8 x 4 x 32 = 1024 elements per row held in registers

template <typename T> __device__ __forceinline__ float4 ldg4(const T* p) { return Vec4<T>::load(p); }

// ---- softmax ---------------------------------------------------------------------------------
template <typename TI, typename TO, int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_warp_kernel(const TI* __restrict__ x, TO* __restrict__ out, long long rows, int len) {
  long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const TI* xr = x + row * len;
  TO* orow = out + row * len;
  float4 v[NV];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int c = (i * 32 + lane) * 4;
    if (c < len) { v[i] = ldg4(xr + c); mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w))); }
  }
  mx = warpMax(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int c = (i * 32 + lane) * 4;
    if (c < len) {
      v[i].x = expf(v[i].x - mx); v[i].y = expf(v[i].y - mx); v[i].z = expf(v[i].z - mx); v[i].w = expf(v[i].w - mx);
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  sum = warpSum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int c = (i * 32 + lane) * 4;
    if (c < len) Vec4<TO>::store(orow + c, make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv));
  }
}

// generic: block per row, any length / alignment / element type
__global__ void __launch_bounds__(256) softmax_block_kernel(const void* x, void* out, int idt, int odt, long long rows, long long len) {
  __shared__ float red[32];
  long long row = blockIdx.x;
  long long base = row * len;
  float mx = -INFINITY;
  for (long long c = threadIdx.x; c < len; c += blockDim.x) mx = fmaxf(mx, loadAs(x, base + c, idt));
  mx = warpMax(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (long long c = threadIdx.x; c < len; c += blockDim.x) sum += expf(loadAs(x, base + c, idt) - mx);
  sum = warpSum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sum += red[w];
  const float inv = 1.f / sum;
  for (long long c = threadIdx.x; c < len; c += blockDim.x) storeAs(out, base + c, odt, expf(loadAs(x, base + c, idt) - mx) * inv);
}

template <typename TI, typename TO>
int launchSoftmaxWarp(const void* x, void* out, long long rows, int len, cudaStream_t st) {
  unsigned blocks = (unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
  int nv = (len + 127) / 128;
  const TI* xi = reinterpret_cast<const TI*>(x); TO* oo = reinterpret_cast<TO*>(out);
  if (nv <= 1) softmax_warp_kernel<TI, TO, 1><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, oo, rows, len);
  else if (nv <= 2) softmax_warp_kernel<TI, TO, 2><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, oo, rows, len);
  else if (nv <= 4) softmax_warp_kernel<TI, TO, 4><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, oo, rows, len);
  else softmax_warp_kernel<TI, TO, 8><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, oo, rows, len);
  LLC_LAUNCH_CHECK("softmax_warp_kernel");
  return LLC_OK;
}

// ---- LayerNorm -------------------------------------------------------------------------------
// 16 bytes of a row per lane and load: E = 8 bf16 or 4 fp32 elements.
template <typename T, int E> __device__ __forceinline__ void unpackVec(const uint4& raw, float* v);
template <> __device__ __forceinline__ void unpackVec<float, 4>(const uint4& raw, float* v) {
  v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y); v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void unpackVec<__nv_bfloat16, 8>(const uint4& raw, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
}
// E consecutive elements of type T as floats (E * sizeof(T) is 8, 16 or 32 bytes, aligned to min(16, that))
template <typename T, int E> __device__ __forceinline__ void loadElems(const T* p, float* v) {
  if constexpr (sizeof(T) * E == 16) { const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p)); unpackVec<T, E>(raw, v); }
  else if constexpr (sizeof(T) == 4) { unpackVec<float, 4>(__ldg(reinterpret_cast<const uint4*>(p)), v); unpackVec<float, 4>(__ldg(reinterpret_cast<const uint4*>(p) + 1), v + 4); }
  else { const float4 f = Vec4<T>::load(p); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
}
template <typename T, int E> __device__ __forceinline__ void storeElems(T* p, const float* v) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(p + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  } else if constexpr (E == 8) {
    uint4 o; __nv_bfloat162 h;
    h = __floats2bfloat162_rn(v[0], v[1]); o.x = *reinterpret_cast<unsigned*>(&h); h = __floats2bfloat162_rn(v[2], v[3]); o.y = *reinterpret_cast<unsigned*>(&h);
    h = __floats2bfloat162_rn(v[4], v[5]); o.z = *reinterpret_cast<unsigned*>(&h); h = __floats2bfloat162_rn(v[6], v[7]); o.w = *reinterpret_cast<unsigned*>(&h);
    *reinterpret_cast<uint4*>(p) = o;
  } else {
    Vec4<T>::store(p, make_float4(v[0], v[1], v[2], v[3]));
  }
}

// One warp per row, rows taken grid-stride; a lane holds NV vectors of 16 bytes of the row.  The next row's loads are
// issued before the current row's two reductions, so that the statistics of one row hide the memory latency of the next.
template <typename TI, typename TP, typename TO, int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_warp_kernel(const TI* __restrict__ x, const TP* __restrict__ gamma, const TP* __restrict__ beta,
                                                                              TO* __restrict__ out, long long rows, int d, float eps) {
  constexpr int E = 16 / sizeof(TI);
  const int lane = threadIdx.x & 31;
  const long long warpsTotal = (long long)gridDim.x * kWarpsPerBlock;
  long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  uint4 nxt[NV];
  auto fetch = [&](long long r) {
    const TI* xr = x + r * d;
#pragma unroll
    for (int i = 0; i < NV; ++i) { const int c = (i * 32 + lane) * E; if (c < d) nxt[i] = __ldg(reinterpret_cast<const uint4*>(xr + c)); }
  };
  fetch(row);
  const float invD = 1.f / (float)d;
  for (; row < rows; row += warpsTotal) {
    float v[NV][E];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * E;
      if (c < d) {
        unpackVec<TI, E>(nxt[i], v[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) s += v[i][e];
      }
    }
    if (row + warpsTotal < rows) fetch(row + warpsTotal);
    const float mean = warpSum(s) * invD;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * E;
      if (c < d) {
#pragma unroll
        for (int e = 0; e < E; ++e) { const float a = v[i][e] - mean; q = fmaf(a, a, q); }
      }
    }
    const float rstd = rsqrtf(warpSum(q) * invD + eps);
    TO* orow = out + row * d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * E;
      if (c < d) {
        float g[E], b[E], o[E];
        loadElems<TP, E>(gamma + c, g); loadElems<TP, E>(beta + c, b);
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = fmaf((v[i][e] - mean) * rstd, g[e], b[e]);
        storeElems<TO, E>(orow + c, o);
      }
    }
  }
}

__global__ void __launch_bounds__(256) layernorm_block_kernel(const void* x, const void* gamma, const void* beta, void* out, int idt, int pdt, int odt,
                                                               long long rows, long long d, float eps) {
  __shared__ float red[32];
  long long base = (long long)blockIdx.x * d;
  float s = 0.f;
  for (long long c = threadIdx.x; c < d; c += blockDim.x) s += loadAs(x, base + c, idt);
  s = warpSum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
  const float mean = s / (float)d;
  __syncthreads();
  float q = 0.f;
  for (long long c = threadIdx.x; c < d; c += blockDim.x) { float a = loadAs(x, base + c, idt) - mean; q += a * a; }
  q = warpSum(q);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
  __syncthreads();
  q = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) q += red[w];
  const float rstd = rsqrtf(q / (float)d + eps);
  for (long long c = threadIdx.x; c < d; c += blockDim.x)
    storeAs(out, base + c, odt, (loadAs(x, base + c, idt) - mean) * rstd * loadAs(gamma, c, pdt) + loadAs(beta, c, pdt));
}

template <typename TI, typename TP, typename TO>
int launchLayerNormWarp(const void* x, const void* g, const void* b, void* out, long long rows, int d, float eps, cudaStream_t st) {
  constexpr int E = 16 / (int)sizeof(TI);
  // enough warps to keep every SM full (8 blocks of 8 warps each), each taking its rows grid-stride
  const long long wantBlocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock, cap = (long long)deviceSMs() * 8;
  const unsigned blocks = (unsigned)(wantBlocks < cap ? wantBlocks : cap);
  const int nv = (d + 32 * E - 1) / (32 * E);
  const TI* xi = reinterpret_cast<const TI*>(x); const TP* gi = reinterpret_cast<const TP*>(g); const TP* bi = reinterpret_cast<const TP*>(b);
  TO* oo = reinterpret_cast<TO*>(out);
  if (nv <= 1) layernorm_warp_kernel<TI, TP, TO, 1><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, gi, bi, oo, rows, d, eps);
  else if (nv <= 2) layernorm_warp_kernel<TI, TP, TO, 2><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, gi, bi, oo, rows, d, eps);
  else if (nv <= 3) layernorm_warp_kernel<TI, TP, TO, 3><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, gi, bi, oo, rows, d, eps);
  else if (nv <= 4) layernorm_warp_kernel<TI, TP, TO, 4><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, gi, bi, oo, rows, d, eps);
  else if (nv <= 6) layernorm_warp_kernel<TI, TP, TO, 6><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, gi, bi, oo, rows, d, eps);
  else layernorm_warp_kernel<TI, TP, TO, 8><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xi, gi, bi, oo, rows, d, eps);
  LLC_LAUNCH_CHECK("layernorm_warp_kernel");
  return LLC_OK;
}

// ---- reductions ------------------------------------------------------------------------------
__device__ __forceinline__ float redInit(int op) { return op == 1 ? -INFINITY : op == 2 ? INFINITY : 0.f; }
__device__ __forceinline__ float redOp(float a, float b, int op) { return op == 1 ? fmaxf(a, b) : op == 2 ? fminf(a, b) : a + b; }

// inner == 1: one warp per output element, lanes stride over R
__global__ void __launch_bounds__(256) reduce_rows_kernel(const void* x, void* out, int idt, int odt, long long outer, long long r, int op) {
  long long o = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (o >= outer) return;
  const int lane = threadIdx.x & 31;
  float acc = redInit(op);
  for (long long i = lane; i < r; i += 32) acc = redOp(acc, loadAs(x, o * r + i, idt), op);
  acc = op == 1 ? warpMax(acc) : op == 2 ? warpMin(acc) : warpSum(acc);
  if (lane == 0) storeAs(out, o, odt, op == 3 ? acc / (float)r : acc);
}
// inner > 1: one thread per (outer, inner) element, coalesced across inner
__global__ void __launch_bounds__(256) reduce_cols_kernel(const void* x, void* out, int idt, int odt, long long outer, long long r, long long inner, int op) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= outer * inner) return;
  long long o = idx / inner, i = idx - o * inner;
  float acc = redInit(op);
  long long base = o * r * inner + i;
  for (long long k = 0; k < r; ++k) acc = redOp(acc, loadAs(x, base + k * inner, idt), op);
  storeAs(out, idx, odt, op == 3 ? acc / (float)r : acc);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; }

}  // namespace
}  // namespace llc

using namespace llc;

extern "C" int llc_cuda_softmax(const void* x, void* out, int32_t idt, int32_t odt, int64_t rows, int64_t len, void* stream) {
  if (rows <= 0 || len <= 0) return LLC_OK;
  if (!x || !out) return setError(LLC_ERR_ARGUMENT, "llc argument: softmax null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  bool fast = len % 4 == 0 && len <= 1024 && aligned16(x) && aligned16(out);
  if (fast && idt == LLC_FLOAT32 && odt == LLC_FLOAT32) return launchSoftmaxWarp<float, float>(x, out, rows, (int)len, st);
  if (fast && idt == LLC_BFLOAT16 && odt == LLC_BFLOAT16) return launchSoftmaxWarp<__nv_bfloat16, __nv_bfloat16>(x, out, rows, (int)len, st);
  if (fast && idt == LLC_FLOAT32 && odt == LLC_BFLOAT16) return launchSoftmaxWarp<float, __nv_bfloat16>(x, out, rows, (int)len, st);
  if (fast && idt == LLC_BFLOAT16 && odt == LLC_FLOAT32) return launchSoftmaxWarp<__nv_bfloat16, float>(x, out, rows, (int)len, st);
  if (rows > 2147483647LL) return setError(LLC_ERR_ARGUMENT, "llc argument: softmax row count too large");
  softmax_block_kernel<<<(unsigned)rows, 256, 0, st>>>(x, out, idt, odt, rows, len);
  LLC_LAUNCH_CHECK("softmax_block_kernel");
  return LLC_OK;
}

extern "C" int llc_cuda_layernorm(const void* x, const void* gamma, const void* beta, void* out, int32_t idt, int32_t pdt, int32_t odt,
                                  int64_t rows, int64_t d, float eps, void* stream) {
  if (rows <= 0 || d <= 0) return LLC_OK;
  if (!x || !out || !gamma || !beta) return setError(LLC_ERR_ARGUMENT, "llc argument: layernorm null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  // rows of whole 16-byte vectors of the input type, at most 8 of them per lane
  const int e = idt == LLC_BFLOAT16 ? 8 : 4;
  bool fast = d % e == 0 && d <= 32 * e * 8 && aligned16(x) && aligned16(out) && aligned16(gamma) && aligned16(beta);
#define LN_CASE(I, P, O, TI, TP, TO) if (fast && idt == I && pdt == P && odt == O) return launchLayerNormWarp<TI, TP, TO>(x, gamma, beta, out, rows, (int)d, eps, st);
  LN_CASE(LLC_FLOAT32, LLC_FLOAT32, LLC_FLOAT32, float, float, float)
  LN_CASE(LLC_BFLOAT16, LLC_BFLOAT16, LLC_BFLOAT16, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16)
  LN_CASE(LLC_BFLOAT16, LLC_FLOAT32, LLC_BFLOAT16, __nv_bfloat16, float, __nv_bfloat16)
  LN_CASE(LLC_FLOAT32, LLC_BFLOAT16, LLC_BFLOAT16, float, __nv_bfloat16, __nv_bfloat16)
  LN_CASE(LLC_FLOAT32, LLC_FLOAT32, LLC_BFLOAT16, float, float, __nv_bfloat16)
  LN_CASE(LLC_BFLOAT16, LLC_BFLOAT16, LLC_FLOAT32, __nv_bfloat16, __nv_bfloat16, float)
  LN_CASE(LLC_BFLOAT16, LLC_FLOAT32, LLC_FLOAT32, __nv_bfloat16, float, float)
#undef LN_CASE
  if (rows > 2147483647LL) return setError(LLC_ERR_ARGUMENT, "llc argument: layernorm row count too large");
  layernorm_block_kernel<<<(unsigned)rows, 256, 0, st>>>(x, gamma, beta, out, idt, pdt, odt, rows, d, eps);
  LLC_LAUNCH_CHECK("layernorm_block_kernel");
  return LLC_OK;
}

extern "C" int llc_cuda_reduce(const void* x, void* out, int32_t idt, int32_t odt, int64_t outer, int64_t r, int64_t inner, int32_t op, void* stream) {
  if (outer <= 0 || inner <= 0) return LLC_OK;
  if (r <= 0) return setError(LLC_ERR_ARGUMENT, "llc argument: reduce over an empty extent");
  if (op < 0 || op > 3) return setError(LLC_ERR_ARGUMENT, "llc argument: unknown reduce op");
  cudaStream_t st = (cudaStream_t)stream;
  if (inner == 1) {
    reduce_rows_kernel<<<(unsigned)((outer + 7) / 8), 256, 0, st>>>(x, out, idt, odt, outer, r, op);
    LLC_LAUNCH_CHECK("reduce_rows_kernel");
  } else {
    long long total = outer * inner;
    reduce_cols_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, out, idt, odt, outer, r, inner, op);
    LLC_LAUNCH_CHECK("reduce_cols_kernel");
  }
  return LLC_OK;
}

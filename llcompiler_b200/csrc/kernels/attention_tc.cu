// Fused attention for sm_100a: out = softmax(scale * Q K^T + mask) V, bf16 operands, head size 64.  This file: the
// two-pass kernel for up to 384 keys (the whole score tile in tensor memory) and the entry point; 385 to 512 keys go
// to the blockwise kernel of attention_blocks_tc.cu.
// Persistent CTAs (one per SM) walk (batch, head, 128-query block) tiles; the score tile never leaves the SM:
//   last warp, lane 0  TMA loads of Q, K and V (128-byte swizzle) and the MMAs: S = Q K^T into tensor memory (128 lanes x
//                      up to 384 fp32 columns); once that MMA is complete the next tile's Q, K and this tile's V are
//                      requested, so their flight hides behind the softmax; O = P V into 64 further columns when P is
//                      written.
//   16 softmax warps   straight out of tensor memory: thread = one query row and every fourth 32-column chunk; pass 1 row
//                      maximum, pass 2 exp2 and row sum, P written as bf16 into shared memory in the K-major swizzled
//                      layout the second MMA reads; then the epilogue O / rowsum -> bf16 -> global.  A mask row that is
//                      all zeros (the usual full-length batch) takes a path without mask loads.
// Replaces batch_matmul -> (scale, mask add) -> softmax -> batch_matmul of the reference's decomposed attention
// (llcompiler/compiler/torch_compile_config.py:24 decomposes aten._softmax; the matmuls lower through
// src/Conversion/LLHToHLO/LLHToHLO.cpp:363-382).  Algorithmic HBM bytes: Q + K + V + out (+ mask); the S x S
// scores and probabilities of the unfused path (3 x b0*b1*M*N elements of traffic) never reach memory.
#include "common.cuh"
#include "tc_common.cuh"

namespace llc {
__device__ int g_attnStatus = 0;   // non-zero after a bounded wait gave up: 6 loader/issuer thread, 7 softmax warps

namespace {
using namespace tc;

constexpr int kD = 64;            // head size (one 128-byte swizzle atom of bf16)
constexpr int kBM = 128;          // query rows per CTA
constexpr int kMaxN = 384;        // keys: 384 score columns + 64 output columns of tensor memory
constexpr int kTile = kBM * 128;  // bytes of a 128-row x 128-byte tile
constexpr int kGroups = 4;              // softmax warps per lane quarter: group h takes every kGroups-th 32-column chunk
constexpr int kSoftmaxThreads = 4 * kGroups * 32;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnArgs {
  void* out; const void* mask; int mask_dtype;
  long long M, N;
  long long o_s0, o_s1, o_sm, m_s0, m_s1, m_sm;
  long long tiles;                   // (batch, head, query block) triples, walked by persistent CTAs
  int b1, mTiles, nBlocks, kAtoms;   // key blocks of 128 (first MMA), key atoms of 64 (second MMA)
  int qZ0, qZ1, kZ0, kZ1, vZ0, vZ1;  // 1: the operand has this batch dim, 0: broadcast
  float scaleLog2e;
};

constexpr int kSmemBytes = kTile /*Q*/ + 3 * kTile /*K*/ + 3 * kTile /*V*/ + 6 * kTile /*P*/ + 8192 /*barriers, row statistics, mask row*/ + 1024;

__device__ __forceinline__ float fastExp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void softmaxBarrier() { asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory"); }

__global__ void __launch_bounds__(kSoftmaxThreads + 32, 1)
attention_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                 const AttnArgs p) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;
  uint8_t* sV = sK + 3 * kTile;
  uint8_t* sP = sV + 3 * kTile;
  uint8_t* misc = sP + 6 * kTile;
  // One phase per tile on every barrier: [0] Q,K landed  [1] V landed  [2] S complete  [3] P written  [4] O complete  [5] O read
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc);
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(misc + 64);
  volatile int* abortWord = reinterpret_cast<volatile int*>(misc + 68);
  float* sMax = reinterpret_cast<float*>(misc + 128);           // [kGroups][128]
  float* sSum = sMax + kGroups * 128;                           // [kGroups][128]
  float* sMask = sSum + kGroups * 128;                          // [384] mask row * log2(e); -inf past the last key
  volatile int* sMaskSet = reinterpret_cast<volatile int*>(misc + 72);   // whether the current mask row has any non-zero entry

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kIssuerWarp = kSoftmaxThreads / 32;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 5; ++i) mbarInit(&bars[i], 1);
    mbarInit(&bars[5], kSoftmaxThreads / 32);
    *abortWord = 0;
    fenceBarrierInit();
  }
  if (warp == kIssuerWarp) tmemAlloc(tmemSlot, 512);
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const bool rowMask = p.mask == nullptr || p.m_sm == 0;        // the mask does not depend on the query row
  auto coords = [&](long long t, int& tileM, int& zb0, int& zb1) {
    const int z = (int)(t / p.mTiles); tileM = (int)(t - (long long)z * p.mTiles);
    zb0 = z / p.b1; zb1 = z - zb0 * p.b1;
  };

  if (warp == kIssuerWarp) {
    if (lane == 0) {
      // Loader and MMA issuer.  Per tile: S = Q K^T as soon as Q and K are there; once that MMA is complete (Q, K
      // and, from the previous tile, V and P are free again) the next tile's Q, K and this tile's V are requested,
      // so their flight time hides behind the softmax; O = P V when the softmax warps have written P.
      prefetchTensorMap(&mapQ); prefetchTensorMap(&mapK); prefetchTensorMap(&mapV);
      auto loadQK = [&](long long t) {
        int tileM, zb0, zb1; coords(t, tileM, zb0, zb1);
        mbarExpectTx(&bars[0], (1 + p.nBlocks) * kTile);
        tmaLoad4d(sQ, &mapQ, &bars[0], 0, tileM * kBM, zb1 * p.qZ1, zb0 * p.qZ0);
        for (int j = 0; j < p.nBlocks; ++j) tmaLoad4d(sK + j * kTile, &mapK, &bars[0], 0, j * 128, zb1 * p.kZ1, zb0 * p.kZ0);
      };
      constexpr uint32_t idescS = instrDesc(1, kBM, 128, 0, 0);
      constexpr uint32_t idescO = instrDesc(1, kBM, kD, 0, 1);
      const uint64_t dQ = smemDescKMajorSw128(smemAddr(sQ));
      if ((long long)blockIdx.x < p.tiles) loadQK(blockIdx.x);
      uint32_t it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it) {
        const uint32_t ph = it & 1;
        int tileM, zb0, zb1; coords(t, tileM, zb0, zb1);
        ok = mbarWait(&bars[0], ph, abortWord);
        tcFenceAfter();
        for (int j = 0; j < p.nBlocks; ++j) {           // one 128 x 128 block of scores per 128 keys, K = 64 in four steps of 16
          const uint64_t dK = smemDescKMajorSw128(smemAddr(sK + j * kTile));
#pragma unroll
          for (int k = 0; k < 4; ++k) mmaSS<false>(tmemBase + (uint32_t)(j * 128), dQ + 2 * k, dK + 2 * k, idescS, k > 0 ? 1u : 0u);
        }
        mmaCommit(&bars[2]);
        ok = ok && mbarWait(&bars[2], ph, abortWord);   // every MMA issued so far is complete
        if (t + gridDim.x < p.tiles) loadQK(t + gridDim.x);
        mbarExpectTx(&bars[1], p.nBlocks * kTile);
        for (int j = 0; j < p.nBlocks; ++j) tmaLoad4d(sV + j * kTile, &mapV, &bars[1], 0, j * 128, zb1 * p.vZ1, zb0 * p.vZ0);
        ok = ok && mbarWait(&bars[3], ph, abortWord) && mbarWait(&bars[1], ph, abortWord);
        if (it > 0) ok = ok && mbarWait(&bars[5], ph ^ 1, abortWord);   // the previous tile's O has been read
        tcFenceAfter();
        for (int a = 0; a < p.kAtoms; ++a) {            // P is K-major in atoms of 64 keys, V the MN-major operand (head dim contiguous)
          const uint64_t dP = smemDescKMajorSw128(smemAddr(sP + a * kTile));
          const uint64_t dV = smemDescMnMajorSw128(smemAddr(sV + a * 64 * 128), 64 * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) mmaSS<false>(tmemBase + kMaxN, dP + 2 * k, dV + (uint64_t)(k * ((16 * 128) >> 4)), idescO, (a > 0 || k > 0) ? 1u : 0u);
        }
        mmaCommit(&bars[4]);                            // also reached after a failed wait, so that the other warps do not spin out
        if (!ok) atomicExch(&g_attnStatus, 6);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax and epilogue
    const int q = warp & 3, h = warp >> 2;             // tensor-memory lane quarter (a hardware rule) and chunk group
    const int row = q * 32 + lane;
    const uint32_t trow = tmemBase + ((uint32_t)(q * 32) << 16);
    const int nChunks = p.nBlocks * 4;
    int maskZ = -1;
    bool plain = false;                                // the mask row is all zeros and covers every column: logits are scale * score
    uint32_t it = 0;
    bool ok = true;                                    // after a wait gave up the loop still runs (every thread must reach every barrier)
    for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it) {
      const uint32_t ph = it & 1;
      int tileM, zb0, zb1; coords(t, tileM, zb0, zb1);
      const long long gm = (long long)tileM * kBM + row;
      const int z = zb0 * p.b1 + zb1;
      if (rowMask && z != maskZ) {                     // mask row (times log2 e); columns past the last key get -inf
        if (threadIdx.x == 0) *sMaskSet = 0;
        softmaxBarrier();
        const long long mBase = zb0 * p.m_s0 + zb1 * p.m_s1;
        bool any = false;
        for (int c = threadIdx.x; c < kMaxN; c += kSoftmaxThreads) {
          const float mv = c < p.N ? (p.mask ? loadAs(p.mask, mBase + c, p.mask_dtype) * kLog2e : 0.f) : -INFINITY;
          sMask[c] = mv;
          any = any || (c < nChunks * 32 && mv != 0.f);
        }
        if (any) *sMaskSet = 1;
        maskZ = z;
        softmaxBarrier();
        plain = *sMaskSet == 0 && p.scaleLog2e > 0.f;
      }
      softmaxBarrier();
      const long long mRow = zb0 * p.m_s0 + zb1 * p.m_s1 + gm * p.m_sm;
      auto logit = [&](float s, int col) -> float {    // scaled score plus mask, in units of log2
        if (rowMask) return fmaf(s, p.scaleLog2e, sMask[col]);
        if (col >= p.N || gm >= p.M) return col < p.N ? s * p.scaleLog2e : -INFINITY;
        return fmaf(s, p.scaleLog2e, loadAs(p.mask, mRow + col, p.mask_dtype) * kLog2e);
      };
      if (ok && !mbarWait(&bars[2], ph, abortWord)) { atomicExch(&g_attnStatus, 7); ok = false; }
      tcFenceAfter();
      float mx = -INFINITY;
      for (int c = h; c < nChunks; c += kGroups) {
        float v[32];
        __syncwarp();
        tmemLoad32x32(trow + (uint32_t)(c * 32), v);
        if (plain) {                                     // no mask at all: the maximum of the raw scores, scaled afterwards
#pragma unroll
          for (int j = 0; j < 32; j += 2) mx = fmaxf(mx, fmaxf(v[j], v[j + 1]));
        } else if (rowMask) {                            // the mask row sits in shared memory, four columns per load
          const float4* m4 = reinterpret_cast<const float4*>(sMask + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 mk = m4[j];
            mx = fmaxf(fmaxf(mx, fmaf(v[4 * j], p.scaleLog2e, mk.x)), fmaxf(fmaf(v[4 * j + 1], p.scaleLog2e, mk.y), fmaxf(fmaf(v[4 * j + 2], p.scaleLog2e, mk.z), fmaf(v[4 * j + 3], p.scaleLog2e, mk.w))));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, logit(v[j], c * 32 + j));
        }
      }
      if (plain) mx *= p.scaleLog2e;
      sMax[h * 128 + row] = mx;
      softmaxBarrier();
#pragma unroll
      for (int g = 0; g < kGroups; ++g) mx = fmaxf(mx, sMax[g * 128 + row]);
      if (mx == -INFINITY) mx = 0.f;                   // a fully masked row: all probabilities become 0
      float sum = 0.f;
      for (int c = h; c < nChunks; c += kGroups) {
        float v[32];
        __syncwarp();
        tmemLoad32x32(trow + (uint32_t)(c * 32), v);
        const uint32_t rowAddr = smemAddr(sP + (c >> 1) * kTile) + (uint32_t)row * 128u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 pk[4];
          float e8[8];
          if (plain) {
#pragma unroll
            for (int e = 0; e < 8; ++e) e8[e] = v[j * 8 + e] * p.scaleLog2e;
          } else if (rowMask) {
            const float4 ma = reinterpret_cast<const float4*>(sMask + c * 32 + j * 8)[0], mb = reinterpret_cast<const float4*>(sMask + c * 32 + j * 8)[1];
            e8[0] = fmaf(v[j * 8], p.scaleLog2e, ma.x); e8[1] = fmaf(v[j * 8 + 1], p.scaleLog2e, ma.y); e8[2] = fmaf(v[j * 8 + 2], p.scaleLog2e, ma.z); e8[3] = fmaf(v[j * 8 + 3], p.scaleLog2e, ma.w);
            e8[4] = fmaf(v[j * 8 + 4], p.scaleLog2e, mb.x); e8[5] = fmaf(v[j * 8 + 5], p.scaleLog2e, mb.y); e8[6] = fmaf(v[j * 8 + 6], p.scaleLog2e, mb.z); e8[7] = fmaf(v[j * 8 + 7], p.scaleLog2e, mb.w);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) e8[e] = logit(v[j * 8 + e], c * 32 + j * 8 + e);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) { e8[e] = fastExp2(e8[e] - mx); sum += e8[e]; }
#pragma unroll
          for (int e = 0; e < 4; ++e) pk[e] = __floats2bfloat162_rn(e8[2 * e], e8[2 * e + 1]);
          const uint32_t chunk = (uint32_t)((c & 1) * 4 + j);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowAddr + ((chunk ^ (uint32_t)(row & 7)) << 4)), "r"(*reinterpret_cast<unsigned*>(&pk[0])),
                       "r"(*reinterpret_cast<unsigned*>(&pk[1])), "r"(*reinterpret_cast<unsigned*>(&pk[2])), "r"(*reinterpret_cast<unsigned*>(&pk[3])) : "memory");
        }
      }
      sSum[h * 128 + row] = sum;
      tcFenceBefore();                                 // this thread's reads of S are done before the next tile's MMA may overwrite it
      fenceProxyAsync();                               // P was written through the generic proxy, the MMA reads it through the async proxy
      softmaxBarrier();
      if (threadIdx.x == 0) mbarArrive(&bars[3]);
      float tot = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) tot += sSum[g * 128 + row];
      const float inv = 1.f / tot;
      if (ok && !mbarWait(&bars[4], ph, abortWord)) { atomicExch(&g_attnStatus, 7); ok = false; }
      tcFenceAfter();
      // epilogue: group h takes 64 / kGroups output columns of its rows
      constexpr int kCols = kD / kGroups;
      float o[kCols];
      __syncwarp();
      tmemLoadCols<kCols>(trow + (uint32_t)(kMaxN + h * kCols), o);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&bars[5]);             // O is in registers: the next tile's second MMA may overwrite it
      if (gm < p.M) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + zb0 * p.o_s0 + zb1 * p.o_s1 + gm * p.o_sm + h * kCols);
#pragma unroll
        for (int j = 0; j < kCols / 8; ++j) {
          __nv_bfloat162 a0 = __floats2bfloat162_rn(o[8 * j] * inv, o[8 * j + 1] * inv), a1 = __floats2bfloat162_rn(o[8 * j + 2] * inv, o[8 * j + 3] * inv);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(o[8 * j + 4] * inv, o[8 * j + 5] * inv), a3 = __floats2bfloat162_rn(o[8 * j + 6] * inv, o[8 * j + 7] * inv);
          uint4 pk; pk.x = *reinterpret_cast<unsigned*>(&a0); pk.y = *reinterpret_cast<unsigned*>(&a1); pk.z = *reinterpret_cast<unsigned*>(&a2); pk.w = *reinterpret_cast<unsigned*>(&a3);
          dst[j] = pk;
        }
      }
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == kIssuerWarp) { tcFenceAfter(); tmemDealloc(tmemBase, 512); }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 operand [b0, b1, rows, 64] with unit stride along the head dim -> 4-D tensor map, box = 64 elements x 128 rows.
bool makeHeadMap(CUtensorMap* map, const void* base, long long rows, long long b1, long long b0, long long sRow, long long s1, long long s0) {
  EncodeTiledFn enc = encodeTiled();
  if (!enc) return false;
  const bool has1 = b1 > 1 && s1 > 0, has0 = b0 > 1 && s0 > 0;
  const long long dense = sRow * rows;
  cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)rows, (cuuint64_t)(has1 ? b1 : 1), (cuuint64_t)(has0 ? b0 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)(sRow * 2), (cuuint64_t)((has1 ? s1 : dense) * 2), (cuuint64_t)((has0 ? s0 : dense) * 2)};
  cuuint32_t box[4] = {(cuuint32_t)kD, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int* attnStatusAddress() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_attnStatus) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}

int attentionBlocks(const LlcAttentionParams* p, cudaStream_t stream);   // attention_blocks_tc.cu: up to 512 keys
int attnBlocksStatus();
int* attnBlocksStatusAddress();

// Reads and clears the status words of the two attention kernels.
int attnStatus() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attnStatus, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attnStatus, &zero, sizeof(int));
  const int w = attnBlocksStatus();
  return v ? v : w;
}

}  // namespace llc

using namespace llc;

extern "C" int llc_cuda_attention(const LlcAttentionParams* p, void* stream) {
  if (!p) return setError(LLC_ERR_ARGUMENT, "llc_cuda_attention: null parameter block");
  if (p->m == 0 || p->b0 == 0 || p->b1 == 0) return LLC_OK;     // no queries: nothing to write
  if (!p->q || !p->k || !p->v || !p->out) return setError(LLC_ERR_ARGUMENT, "llc_cuda_attention: null operand");
  if (p->dtype != LLC_BFLOAT16) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: operands must be bf16");
  if (p->d != kD) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: head size must be 64");
  if (p->n < 1 || p->n > 512) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: 1 to 512 keys");
  if (p->m < 1 || p->b0 < 1 || p->b1 < 1) return setError(LLC_ERR_ARGUMENT, "llc_cuda_attention: empty problem");
  if (p->mask && p->mask_dtype != LLC_FLOAT32 && p->mask_dtype != LLC_BFLOAT16) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: mask must be f32 or bf16");
  auto ok8 = [](long long s) { return s >= 0 && s % 8 == 0; };    // 16-byte multiples of bf16
  if (!ok8(p->q_s0) || !ok8(p->q_s1) || !ok8(p->q_sm) || !ok8(p->k_s0) || !ok8(p->k_s1) || !ok8(p->k_sn) || !ok8(p->v_s0) || !ok8(p->v_s1) || !ok8(p->v_sn) ||
      !ok8(p->o_s0) || !ok8(p->o_s1) || !ok8(p->o_sm) || p->q_sm < kD || p->k_sn < kD || p->v_sn < kD || p->o_sm < kD)
    return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: strides must be non-negative multiples of 8 elements and rows must not overlap");
  if ((reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) | reinterpret_cast<uintptr_t>(p->v) | reinterpret_cast<uintptr_t>(p->out)) & 15)
    return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: operands must be 16-byte aligned");
  // more keys than the score tile of the two-pass kernel holds (384 columns of tensor memory): the blockwise kernel
  // (LLC_ATTENTION_BLOCKS=1 sends every shape there: the tests use it to run that kernel on the small shapes too)
  const char* forceBlocks = getenv("LLC_ATTENTION_BLOCKS");
  if (p->n > kMaxN || (forceBlocks && forceBlocks[0] == '1')) return attentionBlocks(p, static_cast<cudaStream_t>(stream));
  const long long batch = p->b0 * p->b1, mTiles = (p->m + kBM - 1) / kBM;
  if (batch * mTiles > 0x7FFFFFFFLL) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: too many tiles");
  CUtensorMap mq, mk, mv;
  if (!makeHeadMap(&mq, p->q, p->m, p->b1, p->b0, p->q_sm, p->q_s1, p->q_s0) || !makeHeadMap(&mk, p->k, p->n, p->b1, p->b0, p->k_sn, p->k_s1, p->k_s0) ||
      !makeHeadMap(&mv, p->v, p->n, p->b1, p->b0, p->v_sn, p->v_s1, p->v_s0))
    return setError(LLC_ERR_CUDA, "llc cuda: cuTensorMapEncodeTiled rejected the attention operands");
  AttnArgs a{};
  a.out = p->out; a.mask = p->mask; a.mask_dtype = p->mask_dtype;
  a.M = p->m; a.N = p->n;
  a.o_s0 = p->o_s0; a.o_s1 = p->o_s1; a.o_sm = p->o_sm; a.m_s0 = p->mask_s0; a.m_s1 = p->mask_s1; a.m_sm = p->mask_sm;
  a.b1 = (int)p->b1; a.mTiles = (int)mTiles; a.nBlocks = (int)((p->n + 127) / 128); a.kAtoms = (int)((p->n + 63) / 64);
  a.qZ0 = p->b0 > 1 && p->q_s0 > 0; a.qZ1 = p->b1 > 1 && p->q_s1 > 0; a.kZ0 = p->b0 > 1 && p->k_s0 > 0; a.kZ1 = p->b1 > 1 && p->k_s1 > 0;
  a.vZ0 = p->b0 > 1 && p->v_s0 > 0; a.vZ1 = p->b1 > 1 && p->v_s1 > 0;
  a.scaleLog2e = p->scale * kLog2e;
  static DeviceOnce configured;                          // the shared-memory opt-in is kept per device
  const int dev = currentDevice();
  if (!configured.test(dev)) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return cudaFail(e, "cudaFuncSetAttribute(attention_kernel)");
    configured.set(dev);
  }
  a.tiles = batch * mTiles;
  const int sms = deviceSMs();
  const unsigned grid = (unsigned)(a.tiles < sms ? a.tiles : sms);
  attention_kernel<<<grid, kSoftmaxThreads + 32, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, a);
  LLC_LAUNCH_CHECK("attention_kernel");
  return LLC_OK;
}

// Fused attention for sm_100a: out = softmax(scale * Q K^T + mask) V, bf16 operands, head size 64.  This file: the
// two-pass kernel for up to 384 keys (the whole score tile in tensor memory) and the entry point; 385 to 512 keys go
// to the blockwise kernel of attention_blocks_tc.cu.
// Persistent CTAs (one per SM) walk (batch, head, 128-query block) tiles; the score tile never leaves the SM:
//   last warp, lane 0  TMA loads of Q, K and V (128-byte swizzle) and the MMAs: S = Q K^T into tensor memory (128 lanes x
//                      up to 384 fp32 columns), one commit per 128-key block; once that MMA is complete the next tile's
//                      Q, K and this tile's V are requested, so their flight hides behind the softmax; O = P V into 64
//                      further columns, issued round by round as P is written (two 64-key atoms per round, last block first); then at
//                      once the NEXT tile's S = Q K^T (the score columns are free as soon as the last round of P is
//                      written), which so runs under this tile's second MMA and epilogue.
//   16 softmax warps   straight out of tensor memory: thread = one query row and every fourth 32-column chunk, so that
//                      round r of either pass touches key block r only; pass 1 row maximum (block r as soon as its
//                      MMAs are complete), pass 2 exp2 and row sum, P written as bf16 into shared memory in the K-major
//                      swizzled layout the second MMA reads and handed over after every round; then the epilogue
//                      O / rowsum -> bf16 -> shared memory.
//   mask-row warp      the tile's mask row (times log2 e) into shared memory, a tile ahead
//   store warp         one TMA store per output tile  A mask row that is all zeros (the usual full-length batch) takes a
//                      path without mask loads.
// Replaces batch_matmul -> (scale, mask add) -> softmax -> batch_matmul of the reference's decomposed attention
// (llcompiler/compiler/torch_compile_config.py:24 decomposes aten._softmax; the matmuls lower through
// src/Conversion/LLHToHLO/LLHToHLO.cpp:363-382).  Algorithmic HBM bytes: Q + K + V + out (+ mask); the S x S
// scores and probabilities of the unfused path (3 x b0*b1*M*N elements of traffic) never reach memory.
#include "common.cuh"
#include "tc_common.cuh"

namespace llc {
__device__ int g_attnStatus = 0;   // non-zero after a bounded wait gave up: 6 loader/issuer thread, 7 softmax warps, 8 mask-row warp, 9 store warp

namespace {
using namespace tc;

constexpr int kD = 64;            // head size (one 128-byte swizzle atom of bf16)
constexpr int kBM = 128;          // query rows per CTA
constexpr int kMaxN = 384;        // keys: 384 score columns + 64 output columns of tensor memory
constexpr int kTile = kBM * 128;  // bytes of a 128-row x 128-byte tile
constexpr int kGroups = 4;              // softmax warps per lane quarter: group h takes every kGroups-th 32-column chunk
constexpr int kSoftmaxThreads = 4 * kGroups * 32;
constexpr int kThreads = kSoftmaxThreads + 96;   // + the loader / MMA issuer warp, the mask-row warp and the store warp
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

// ROWMASK: the mask (if any) does not depend on the query row.  The per-row form is a kernel of its own because its
// per-element mask loads multiply the code size, and the common kernel is bound by instruction fetch as it is.
template <bool ROWMASK>
__global__ void __launch_bounds__(kThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                 const __grid_constant__ CUtensorMap mapO, const AttnArgs p) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;
  uint8_t* sV = sK + 3 * kTile;
  uint8_t* sP = sV + 3 * kTile;
  uint8_t* misc = sP + 6 * kTile;
  // One phase per tile on every barrier: [0] Q,K landed  [1] V landed  [2] O complete  [3] O read
  // barS[j] key block j of S complete   barP[r] round r of P (atoms 2r, 2r+1) written
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc);
  uint64_t* barS = bars + 4;
  uint64_t* barP = bars + 7;
  uint64_t* barMaskFull = bars + 10;   // [2] the mask row of a tile is in buffer (tile & 1)
  uint64_t* barMaskFree = bars + 12;   // [2] the softmax warps are done with that buffer
  uint64_t* barOut = bars + 14;        // the output tile is staged in shared memory
  uint64_t* barOutFree = bars + 15;    // ... and has left it again
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(misc + 128);
  volatile int* abortWord = reinterpret_cast<volatile int*>(misc + 132);
  float* sMax = reinterpret_cast<float*>(misc + 256);           // [kGroups][128]
  float* sSum = sMax + kGroups * 128;                           // [kGroups][128]
  float* sMask = sSum + kGroups * 128;                          // [2][384] mask row * log2(e); -inf past the last key
  volatile int* sMaskSet = reinterpret_cast<volatile int*>(misc + 136);   // [2] whether that mask row has any non-zero entry

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kIssuerWarp = kSoftmaxThreads / 32, kMaskWarp = kIssuerWarp + 1, kStoreWarp = kIssuerWarp + 2;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 16; ++i) mbarInit(&bars[i], (i == 3 || (i >= 7 && i <= 9) || i == 14) ? kSoftmaxThreads / 32 : 1);   // O read, P rounds, output staged: one arrival per softmax warp
    *abortWord = 0;
    fenceBarrierInit();
  }
  if (warp == kIssuerWarp) tmemAlloc(tmemSlot, 512);
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  constexpr bool rowMask = ROWMASK;
  // The CTA's tiles: blockIdx.x, + gridDim.x, ...; (query block, head, batch) are stepped without a division per tile.
  struct TileWalk {
    int tileM, zb1, zb0, dM, d1, d0, mTiles, b1;
    __device__ TileWalk(const AttnArgs& a, unsigned first, unsigned step) : mTiles(a.mTiles), b1(a.b1) {
      const int z = (int)(first / (unsigned)mTiles); tileM = (int)(first - (unsigned)z * (unsigned)mTiles);
      zb0 = z / b1; zb1 = z - zb0 * b1;
      const int gz = (int)(step / (unsigned)mTiles); dM = (int)(step - (unsigned)gz * (unsigned)mTiles);
      d0 = gz / b1; d1 = gz - d0 * b1;
    }
    __device__ void next() {
      tileM += dM; int c = tileM >= mTiles; tileM -= c * mTiles;
      zb1 += d1 + c; c = zb1 >= b1; zb1 -= c * b1;
      zb0 += d0 + c;
    }
  };

  if (warp == kIssuerWarp) {
    if (lane == 0) {
      // Loader and MMA issuer.  Per tile: once S = Q K^T is complete (Q, K and, from the previous tile, V and P are
      // free again: a commit covers every MMA issued before it) the next tile's Q, K and this tile's V are requested;
      // O = P V round by round as the softmax warps hand P over; then the next tile's S = Q K^T.
      prefetchTensorMap(&mapQ); prefetchTensorMap(&mapK); prefetchTensorMap(&mapV);
      auto loadQK = [&](const TileWalk& w) {
        const int tileM = w.tileM, zb0 = w.zb0, zb1 = w.zb1;
        mbarExpectTx(&bars[0], (1 + p.nBlocks) * kTile);
        tmaLoad4d(sQ, &mapQ, &bars[0], 0, tileM * kBM, zb1 * p.qZ1, zb0 * p.qZ0);
        for (int j = 0; j < p.nBlocks; ++j) tmaLoad4d(sK + j * kTile, &mapK, &bars[0], 0, j * 128, zb1 * p.kZ1, zb0 * p.kZ0);
      };
      constexpr uint32_t idescS = instrDesc(1, kBM, 128, 0, 0);
      constexpr uint32_t idescO = instrDesc(1, kBM, kD, 0, 1);
      const uint64_t dQ = smemDescKMajorSw128(smemAddr(sQ));
      auto issueS = [&]() {                             // one 128 x 128 block of scores per 128 keys, K = 64 in four steps of 16
        for (int j = 0; j < p.nBlocks; ++j) {
          const uint64_t dK = smemDescKMajorSw128(smemAddr(sK + j * kTile));
#pragma unroll
          for (int k = 0; k < 4; ++k) mmaSS<false>(tmemBase + (uint32_t)(j * 128), dQ + 2 * k, dK + 2 * k, idescS, k > 0 ? 1u : 0u);
          mmaCommit(&barS[j]);
        }
      };
      bool ok = true;
      TileWalk cur(p, blockIdx.x, gridDim.x), nxt = cur;
      nxt.next();
      if ((long long)blockIdx.x < p.tiles) {
        loadQK(cur);
        ok = mbarWait(&bars[0], 0, abortWord);
        tcFenceAfter();
        issueS();
      }
      uint32_t it = 0;
      for (long long t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it, cur.next(), nxt.next()) {
        const uint32_t ph = it & 1;
        const int zb0 = cur.zb0, zb1 = cur.zb1;
        const bool more = t + gridDim.x < p.tiles;
        ok = mbarWait(&barS[p.nBlocks - 1], ph, abortWord);   // every MMA issued so far is complete
        if (more) loadQK(nxt);
        mbarExpectTx(&bars[1], p.nBlocks * kTile);
        for (int j = 0; j < p.nBlocks; ++j) tmaLoad4d(sV + j * kTile, &mapV, &bars[1], 0, j * 128, zb1 * p.vZ1, zb0 * p.vZ0);
        ok = ok && mbarWait(&bars[1], ph, abortWord);
        if (it > 0) ok = ok && mbarWait(&bars[3], ph ^ 1, abortWord);   // the previous tile's O has been read
        uint32_t accumulate = 0;
        for (int r = p.nBlocks - 1; r >= 0; --r) {      // P is K-major in atoms of 64 keys, V the MN-major operand (head dim contiguous);
          ok = ok && mbarWait(&barP[r], ph, abortWord);  // the softmax warps hand the rounds over from the last key block to the first
          tcFenceAfter();
          for (int a = 2 * r; a < 2 * r + 2 && a < p.kAtoms; ++a) {
            const uint64_t dP = smemDescKMajorSw128(smemAddr(sP + a * kTile));
            const uint64_t dV = smemDescMnMajorSw128(smemAddr(sV + a * 64 * 128), 64 * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) { mmaSS<false>(tmemBase + kMaxN, dP + 2 * k, dV + (uint64_t)(k * ((16 * 128) >> 4)), idescO, accumulate); accumulate = 1; }
          }
        }
        mmaCommit(&bars[2]);                            // also reached after a failed wait, so that the other warps do not spin out
        if (more && ok) {                               // the score columns are free: every softmax thread has read them
          ok = mbarWait(&bars[0], ph ^ 1, abortWord);
          tcFenceAfter();
          issueS();
        }
        if (!ok) atomicExch(&g_attnStatus, 6);
      }
    }
  } else if (warp == kMaskWarp) {
    // ---------------------------------------------------------------- mask rows
    // One mask row (times log2 e; -inf past the last key) per tile, into one of two buffers, a tile ahead of the softmax
    // warps: a global load issued by them would stall them for as long as the TMA loads keep the memory system busy.
    if (rowMask) {
      const int usedCols = p.nBlocks * 128;
      uint32_t it = 0;
      bool ok = true;
      TileWalk w(p, blockIdx.x, gridDim.x);
      for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it, w.next()) {
        const int buf = (int)(it & 1);
        const uint32_t use = it >> 1;                  // how often this buffer has been filled before
        if (use > 0 && ok && !mbarWait(&barMaskFree[buf], (use - 1) & 1, abortWord)) { atomicExch(&g_attnStatus, 8); ok = false; }
        const long long mBase = w.zb0 * p.m_s0 + w.zb1 * p.m_s1;
        // every load of the row is issued before the first one is used (a branch per element would serialise them)
        constexpr int kPerLane = kMaxN / 32;
        float mv[kPerLane];
        const int last = (int)p.N - 1;
        if (p.mask == nullptr) {
#pragma unroll
          for (int i = 0; i < kPerLane; ++i) mv[i] = 0.f;
        } else if (p.mask_dtype == LLC_FLOAT32) {
          const float* m = static_cast<const float*>(p.mask) + mBase;
#pragma unroll
          for (int i = 0; i < kPerLane; ++i) mv[i] = __ldg(m + min(lane + 32 * i, last));
        } else {
          const __nv_bfloat16* m = static_cast<const __nv_bfloat16*>(p.mask) + mBase;
#pragma unroll
          for (int i = 0; i < kPerLane; ++i) mv[i] = __bfloat162float(m[min(lane + 32 * i, last)]);
        }
        bool any = false;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
          const int c = lane + 32 * i;
          const float v = c < p.N ? mv[i] * kLog2e : -INFINITY;
          sMask[buf * kMaxN + c] = v;
          any = any || (c < usedCols && v != 0.f);
        }
        any = __any_sync(0xffffffffu, any);
        if (lane == 0) { sMaskSet[buf] = any ? 1 : 0; mbarArrive(&barMaskFull[buf]); }   // the arrive releases the warp's writes (ordered by the vote)
      }
    }
  } else if (warp == kStoreWarp) {
    // ---------------------------------------------------------------- output tiles: shared memory -> one TMA store each
    if (lane == 0) {
      TileWalk w(p, blockIdx.x, gridDim.x);
      uint32_t it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it, w.next()) {
        if (ok && !mbarWait(barOut, it & 1, abortWord)) { atomicExch(&g_attnStatus, 9); ok = false; }
        tmaStore4d(&mapO, sP, 0, w.tileM * kBM, w.zb1, w.zb0);   // also clips the rows past the last query
        bulkCommit();
        bulkWaitRead();                                // the store has read the staging buffer: P may overwrite it
        mbarArrive(barOutFree);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax and epilogue
    const int q = warp & 3, h = warp >> 2;             // tensor-memory lane quarter (a hardware rule) and chunk group
    const int row = q * 32 + lane;
    const uint32_t trow = tmemBase + ((uint32_t)(q * 32) << 16);
    const int nB = p.nBlocks;                          // rounds: in round r group h owns chunk 4r + h, which lies in key block r
    uint32_t it = 0;
    bool ok = true;                                    // after a wait gave up the loop still runs (every thread must reach every barrier)
    TileWalk w(p, blockIdx.x, gridDim.x);
    for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it, w.next()) {
      const uint32_t ph = it & 1;
      const int tileM = w.tileM, zb0 = w.zb0, zb1 = w.zb1;
      const long long gm = (long long)tileM * kBM + row;
      float* sMaskCur = sMask + (it & 1) * kMaxN;
      if (rowMask && ok && !mbarWait(&barMaskFull[it & 1], (it >> 1) & 1, abortWord)) { atomicExch(&g_attnStatus, 7); ok = false; }
      // the mask row is all zeros and covers every column: logits are scale * score
      const bool plain = rowMask && sMaskSet[it & 1] == 0 && p.scaleLog2e > 0.f;
      // per-row mask: eight neighbouring mask values of this thread's query row (times log2 e; -inf past the last key;
      // rows past the last query read the last row's and are clipped by the store), the element type decided once
      const long long mRow = zb0 * p.m_s0 + zb1 * p.m_s1 + (gm < p.M ? gm : p.M - 1) * p.m_sm;
      auto mask8 = [&](int col0, float* mk) {
        const int last = (int)p.N - 1;
        if (p.mask_dtype == LLC_FLOAT32) {
          const float* m = static_cast<const float*>(p.mask) + mRow;
#pragma unroll
          for (int e = 0; e < 8; ++e) mk[e] = __ldg(m + min(col0 + e, last));
        } else {
          const __nv_bfloat16* m = static_cast<const __nv_bfloat16*>(p.mask) + mRow;
#pragma unroll
          for (int e = 0; e < 8; ++e) mk[e] = __bfloat162float(m[min(col0 + e, last)]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) mk[e] = col0 + e <= last ? mk[e] * kLog2e : -INFINITY;
      };
      // ---- pass 1: row maximum.  Chunk r of the thread lives in sc[r & 1]; the load of the next chunk is in flight while
      // this one is worked on.  Tensor memory delivers about 128 bytes per clock to the SM, which is what bounds this pass.
      uint32_t sc[2][32];
      auto chunkMax = [&](const uint32_t* v, int c, float mx) -> float {
        if (plain) {                                     // no mask at all: the maximum of the raw scores, scaled afterwards
#pragma unroll
          for (int j = 0; j < 32; j += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(v[j]), __uint_as_float(v[j + 1])));
        } else if (rowMask) {                            // the mask row sits in shared memory, four columns per load
          const float4* m4 = reinterpret_cast<const float4*>(sMaskCur + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 mk = m4[j];
            mx = fmaxf(fmaxf(mx, fmaf(__uint_as_float(v[4 * j]), p.scaleLog2e, mk.x)),
                       fmaxf(fmaf(__uint_as_float(v[4 * j + 1]), p.scaleLog2e, mk.y),
                             fmaxf(fmaf(__uint_as_float(v[4 * j + 2]), p.scaleLog2e, mk.z), fmaf(__uint_as_float(v[4 * j + 3]), p.scaleLog2e, mk.w))));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float mk[8];
            mask8(c * 32 + j * 8, mk);
#pragma unroll
            for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fmaf(__uint_as_float(v[j * 8 + e]), p.scaleLog2e, mk[e]));
          }
        }
        return mx;
      };
      auto waitS = [&](int r) {
        if (ok && !mbarWait(&barS[r], ph, abortWord)) { atomicExch(&g_attnStatus, 7); ok = false; }
        tcFenceAfter();
        __syncwarp();
      };
      float mx = -INFINITY;
      waitS(0);
      tmemIssue32(trow + (uint32_t)(h * 32), sc[0]);
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        if (r < nB) {
          tmemWait32(sc[r & 1]);
          if (r + 1 < nB) { waitS(r + 1); tmemIssue32(trow + (uint32_t)((4 * (r + 1) + h) * 32), sc[(r + 1) & 1]); }
          mx = chunkMax(sc[r & 1], 4 * r + h, mx);
        }
      }
      if (plain) mx *= p.scaleLog2e;
      sMax[h * 128 + row] = mx;
      softmaxBarrier();
#pragma unroll
      for (int g = 0; g < kGroups; ++g) mx = fmaxf(mx, sMax[g * 128 + row]);
      if (mx == -INFINITY) mx = 0.f;                   // a fully masked row: all probabilities become 0
      // ---- pass 2: exp2 and row sum, from the last chunk (still in registers) down to the first, each earlier chunk read
      // again while the one after it is worked on; P is handed to the second MMA after every round
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 2; r >= 0; --r) {
        if (r < nB) {
          const int c = 4 * r + h;
          const uint32_t* v = sc[r & 1];
          // the first atoms of P double as the staging buffer of the previous tile's output
          if (r == 0 && it > 0 && ok && !mbarWait(barOutFree, (it - 1) & 1, abortWord)) { atomicExch(&g_attnStatus, 7); ok = false; }
          if (r < nB - 1) tmemWait32(sc[r & 1]);
          if (r > 0) { __syncwarp(); tmemIssue32(trow + (uint32_t)((c - 4) * 32), sc[(r - 1) & 1]); }
          else tcFenceBefore();                          // this thread's reads of S come before the next tile's MMA, which may overwrite it
          const uint32_t rowAddr = smemAddr(sP + (c >> 1) * kTile) + (uint32_t)row * 128u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 pk[4];
            float e8[8];
            if (plain) {
#pragma unroll
              for (int e = 0; e < 8; ++e) e8[e] = fmaf(__uint_as_float(v[j * 8 + e]), p.scaleLog2e, -mx);
            } else if (rowMask) {
              const float4 ma = reinterpret_cast<const float4*>(sMaskCur + c * 32 + j * 8)[0], mb = reinterpret_cast<const float4*>(sMaskCur + c * 32 + j * 8)[1];
              const float mk[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
#pragma unroll
              for (int e = 0; e < 8; ++e) e8[e] = fmaf(__uint_as_float(v[j * 8 + e]), p.scaleLog2e, mk[e]) - mx;
            } else {
              float mk[8];
              mask8(c * 32 + j * 8, mk);
#pragma unroll
              for (int e = 0; e < 8; ++e) e8[e] = fmaf(__uint_as_float(v[j * 8 + e]), p.scaleLog2e, mk[e]) - mx;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) { e8[e] = fastExp2(e8[e]); sum4[e & 3] += e8[e]; }
#pragma unroll
            for (int e = 0; e < 4; ++e) pk[e] = __floats2bfloat162_rn(e8[2 * e], e8[2 * e + 1]);
            const uint32_t chunk = (uint32_t)((c & 1) * 4 + j);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowAddr + ((chunk ^ (uint32_t)(row & 7)) << 4)), "r"(*reinterpret_cast<unsigned*>(&pk[0])),
                         "r"(*reinterpret_cast<unsigned*>(&pk[1])), "r"(*reinterpret_cast<unsigned*>(&pk[2])), "r"(*reinterpret_cast<unsigned*>(&pk[3])) : "memory");
          }
          // Round done for this warp: atoms 2r and 2r+1 of P are whole once every warp has arrived (no CTA-wide barrier).
          fenceProxyAsync();                             // P was written through the generic proxy, the MMA reads it through the async proxy
          __syncwarp();
          if (lane == 0) mbarArrive(&barP[r]);
        }
      }
      sSum[h * 128 + row] = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      softmaxBarrier();
      if (rowMask && threadIdx.x == 0) mbarArrive(&barMaskFree[it & 1]);   // past the last barrier: nobody reads this tile's mask row any more
      float tot = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) tot += sSum[g * 128 + row];
      const float inv = 1.f / tot;
      if (ok && !mbarWait(&bars[2], ph, abortWord)) { atomicExch(&g_attnStatus, 7); ok = false; }
      tcFenceAfter();
      // ---- epilogue: group h takes 64 / kGroups output columns of its rows; the tile leaves through the first atom of the
      // P buffer (free once the second MMA is complete) and one TMA store, which also clips the rows past the last query
      constexpr int kCols = kD / kGroups;
      float o[kCols];
      __syncwarp();
      tmemLoadCols<kCols>(trow + (uint32_t)(kMaxN + h * kCols), o);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&bars[3]);             // O is in registers: the next tile's second MMA may overwrite it
      const uint32_t outRow = smemAddr(sP) + (uint32_t)row * 128u;
#pragma unroll
      for (int j = 0; j < kCols / 8; ++j) {
        __nv_bfloat162 a0 = __floats2bfloat162_rn(o[8 * j] * inv, o[8 * j + 1] * inv), a1 = __floats2bfloat162_rn(o[8 * j + 2] * inv, o[8 * j + 3] * inv);
        __nv_bfloat162 a2 = __floats2bfloat162_rn(o[8 * j + 4] * inv, o[8 * j + 5] * inv), a3 = __floats2bfloat162_rn(o[8 * j + 6] * inv, o[8 * j + 7] * inv);
        const uint32_t chunk = (uint32_t)(h * (kCols / 8) + j);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(outRow + ((chunk ^ (uint32_t)(row & 7)) << 4)), "r"(*reinterpret_cast<unsigned*>(&a0)),
                     "r"(*reinterpret_cast<unsigned*>(&a1)), "r"(*reinterpret_cast<unsigned*>(&a2)), "r"(*reinterpret_cast<unsigned*>(&a3)) : "memory");
      }
      fenceProxyAsync();
      __syncwarp();
      if (lane == 0) mbarArrive(barOut);               // the store warp sends the tile off
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
  CUtensorMap mq, mk, mv, mo;
  if (!makeHeadMap(&mq, p->q, p->m, p->b1, p->b0, p->q_sm, p->q_s1, p->q_s0) || !makeHeadMap(&mk, p->k, p->n, p->b1, p->b0, p->k_sn, p->k_s1, p->k_s0) ||
      !makeHeadMap(&mv, p->v, p->n, p->b1, p->b0, p->v_sn, p->v_s1, p->v_s0) || !makeHeadMap(&mo, p->out, p->m, p->b1, p->b0, p->o_sm, p->o_s1, p->o_s0))
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
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return cudaFail(e, "cudaFuncSetAttribute(attention_kernel)");
    configured.set(dev);
  }
  a.tiles = batch * mTiles;
  const int sms = deviceSMs();
  const unsigned grid = (unsigned)(a.tiles < sms ? a.tiles : sms);
  if (p->mask == nullptr || p->mask_sm == 0) attention_kernel<true><<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, mo, a);
  else attention_kernel<false><<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, mo, a);
  LLC_LAUNCH_CHECK("attention_kernel");
  return LLC_OK;
}

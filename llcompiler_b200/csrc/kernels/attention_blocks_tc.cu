// Fused attention for sm_100a, blockwise form: out = softmax(scale * Q K^T + mask) V, bf16 operands, head size 64, up to
// 512 keys.  llc_cuda_attention (attention_tc.cu) uses it for more keys than its two-pass kernel holds in tensor memory
// (384); at 384 keys and fewer the two-pass kernel measured faster (0.39 against 0.43 ms at batch 256, 12 heads), because
// this form pays one exchange of row maxima, two barrier waits and one release per 128 keys.
// Persistent CTAs (one per SM) walk (batch, head, 128-query block) tiles; the scores never leave the SM.  The keys are
// taken in blocks of 128 with a running ("online") softmax, so that the tensor core works on one block while the
// softmax warps work on another:
//   issuer warp        one lane issues the MMAs.  S_j = Q K_j^T goes into one of two 128-column score buffers in tensor
//                      memory, O += P_j V_j into 64 further columns.  Issue order per tile: S_0, S_1, then for every
//                      block j: O += P_j V_j as soon as P_j is written, S_{j+2} as soon as its score buffer has been read.
//   loader warp        one lane issues the TMA loads of Q, K and V (128-byte swizzle; K and V of a (batch, head) pair stay
//                      resident): the next tile's Q and K when the current tile's last score block is complete, block j
//                      of its V when the current O += P_j V_j is complete (commit barriers of the issuer, one phase
//                      per tile), so the issuer never waits for an MMA.
//   16 softmax warps   thread = one query row and one 32-column chunk of the block.  The chunk is read from tensor
//                      memory ONCE and stays in registers: chunk maximum -> exchanged between the row's four threads
//                      through shared memory -> running maximum -> exp2 -> P_j as bf16 into shared memory (the K-major
//                      swizzled layout the second MMA reads) and the thread's share of the row sum.  The running
//                      maximum only moves when the block's maximum exceeds it by more than 8 (in log2 units; the
//                      probabilities then stay below 2^8, far inside fp32 and bf16 range); when it does move, the
//                      warps rescale the O accumulator in tensor memory (load, multiply, store) before they release
//                      P_j.  After the last block: O / rowsum -> bf16 -> global.
//                      A mask row that is all zeros (the usual full-length batch) takes a path without mask loads.
// Replaces batch_matmul -> (scale, mask add) -> softmax -> batch_matmul of the reference's decomposed attention
// (llcompiler/compiler/torch_compile_config.py:24 decomposes aten._softmax; the matmuls lower through
// src/Conversion/LLHToHLO/LLHToHLO.cpp:363-382).  Algorithmic HBM bytes: Q + K + V + out (+ mask); the S x S
// scores and probabilities of the unfused path (3 x b0*b1*M*N elements of traffic) never reach memory.
#include "common.cuh"
#include "tc_common.cuh"

namespace llc {
__device__ int g_attnBlocksStatus = 0;   // non-zero after a bounded wait gave up: 6 loader/issuer thread, 7 softmax warps

namespace {
using namespace tc;

constexpr int kD = 64;            // head size (one 128-byte swizzle atom of bf16)
constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 128;          // keys per block
constexpr int kMaxBlocks = 4;
constexpr int kMaxN = kMaxBlocks * kBN;   // keys: K and V of a (batch, head) pair stay resident in shared memory
constexpr int kTile = kBM * 128;  // bytes of a 128-row x 128-byte tile
constexpr int kGroups = 4;        // softmax warps per lane quarter: group h takes the h-th 32-column chunk of a block
constexpr int kSoftmaxThreads = 4 * kGroups * 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.f;       // the running maximum follows the block maximum only in steps larger than this
constexpr uint32_t kColS = 0, kColO = 2 * kBN;   // tensor-memory columns: two score buffers, then the output accumulator

struct AttnArgs {
  void* out; const void* mask; int mask_dtype;
  long long M, N;
  long long o_s0, o_s1, o_sm, m_s0, m_s1, m_sm;
  long long tiles;                   // (batch, head, query block) triples, walked by persistent CTAs
  long long numZ; int zMajor;        // (batch, head) pairs; zMajor: a CTA takes whole pairs (all their query blocks in a row)
  int b1, mTiles, nBlocks, kAtoms;   // key blocks of 128 (first MMA), key atoms of 64 (second MMA)
  int qZ0, qZ1, kZ0, kZ1, vZ0, vZ1;  // 1: the operand has this batch dim, 0: broadcast
  float scaleLog2e;
};

constexpr int kSmemBytes = kTile /*Q*/ + kMaxBlocks * kTile /*K*/ + kMaxBlocks * kTile /*V*/ + 2 * 2 * kTile /*P, two blocks*/ +
                           12288 /*barriers, row statistics, mask row*/ + 1024;

__device__ __forceinline__ float fastExp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void softmaxBarrier() { asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory"); }
// the four warps that share a lane quarter (the four 32-column chunks of the same 32 rows)
__device__ __forceinline__ void quarterBarrier(int q) { asm volatile("bar.sync %0, %1;" ::"r"(2 + q), "n"(kGroups * 32) : "memory"); }
// 32 lanes x 16 fp32 columns back into tensor memory: thread i of the warp writes row (lane base + i)
__device__ __forceinline__ void tmemStore16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

constexpr int kThreads = kSoftmaxThreads + 64;   // + the MMA issuer warp and the loader warp
__global__ void __launch_bounds__(kThreads, 1)
attention_blocks_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                 const AttnArgs p) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;
  uint8_t* sV = sK + kMaxBlocks * kTile;
  uint8_t* sP = sV + kMaxBlocks * kTile;            // two blocks of probabilities, each two 64-key atoms
  uint8_t* misc = sP + 4 * kTile;
  // Barriers.  Per tile (one phase each): Q and K landed, block j of V landed, O complete, O read.  Per key block, two of
  // each, used in turn by a block counter that runs across tiles: S complete, S read, P written (and O rescaled), P consumed.
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc);
  // A parity wait only tells the current phase of a barrier from the one before it, so every waiter must be the one
  // whose own progress the barrier's next-but-one phase depends on.  The loader therefore has barriers of its own
  // (Q and K free, block j of V free: one phase per tile, the next phase needs the load it is about to issue)
  // instead of watching the two-buffer barriers, which can run two phases ahead of it.
  uint64_t* barQK = bars, *barOFull = bars + 1, *barOEmpty = bars + 2, *barQKFree = bars + 3;
  uint64_t* barSFull = bars + 4, *barSEmpty = bars + 6, *barPFull = bars + 8, *barPEmpty = bars + 10;
  uint64_t* barV = bars + 12;                                   // [kMaxBlocks] one per key block of V (a phase per tile)
  uint64_t* barVFree = bars + 16;                               // [kMaxBlocks] O += P_j V_j of this tile is complete
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(misc + 192);
  volatile int* abortWord = reinterpret_cast<volatile int*>(misc + 196);
  volatile int* sMaskSet = reinterpret_cast<volatile int*>(misc + 200);   // whether the current mask row has any non-zero entry
  float* sPart = reinterpret_cast<float*>(misc + 256);          // [2][kGroups][128] chunk maxima of a block (double-buffered)
  float* sSum = sPart + 2 * kGroups * 128;                      // [kGroups][128]
  float* sMask = sSum + kGroups * 128;                          // [kMaxN] mask row * log2(e); -inf past the last key

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kIssuerWarp = kSoftmaxThreads / 32, kLoaderWarp = kIssuerWarp + 1;
  constexpr int kWarps = kSoftmaxThreads / 32;

  if (threadIdx.x == 0) {
    mbarInit(barQK, 1); mbarInit(barOFull, 1); mbarInit(barOEmpty, kWarps); mbarInit(barQKFree, 1);
    for (int i = 0; i < kMaxBlocks; ++i) { mbarInit(&barV[i], 1); mbarInit(&barVFree[i], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&barSFull[i], 1); mbarInit(&barSEmpty[i], kWarps); mbarInit(&barPFull[i], kWarps); mbarInit(&barPEmpty[i], 1); }
    *abortWord = 0;
    fenceBarrierInit();
  }
  if (warp == kIssuerWarp) tmemAlloc(tmemSlot, 512);
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const bool rowMask = p.mask == nullptr || p.m_sm == 0;        // the mask does not depend on the query row
  const int nb = p.nBlocks;
  // The tiles of this CTA, in order.  With many (batch, head) pairs a CTA takes whole pairs, so that consecutive tiles
  // share their keys, values and mask row (L2-hot, and the mask row is staged once per pair); with few pairs the tiles
  // are dealt out one by one so that every SM has work.
  const long long nIter = p.zMajor ? (blockIdx.x < p.numZ ? (long long)p.mTiles * ((p.numZ - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0)
                                   : (blockIdx.x < p.tiles ? (p.tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0);
  auto coords = [&](long long it, int& tileM, int& zb0, int& zb1) {
    long long z;
    if (p.zMajor) { const long long k = it / p.mTiles; tileM = (int)(it - k * p.mTiles); z = blockIdx.x + k * gridDim.x; }
    else { const long long t = blockIdx.x + it * gridDim.x; z = t / p.mTiles; tileM = (int)(t - z * p.mTiles); }
    zb0 = (int)(z / p.b1); zb1 = (int)(z - (long long)zb0 * p.b1);
  };

  if (warp == kLoaderWarp) {
    if (lane == 0) {
      // ------------------------------------------------------------ loader
      // Q and K of the next tile come in as soon as the current tile's last score block is complete (nothing reads Q
      // and K after that), block j of V as soon as the current tile's O += P_j V_j is complete: commit barriers of
      // the issuer, watched here so that the issuer itself never waits for an MMA to finish.
      prefetchTensorMap(&mapQ); prefetchTensorMap(&mapK); prefetchTensorMap(&mapV);
      auto loadQK = [&](long long t) {
        int tileM, zb0, zb1; coords(t, tileM, zb0, zb1);
        mbarExpectTx(barQK, (1 + nb) * kTile);
        tmaLoad4d(sQ, &mapQ, barQK, 0, tileM * kBM, zb1 * p.qZ1, zb0 * p.qZ0);
        for (int j = 0; j < nb; ++j) tmaLoad4d(sK + j * kTile, &mapK, barQK, 0, j * kBN, zb1 * p.kZ1, zb0 * p.kZ0);
      };
      auto loadV = [&](long long t, int j) {
        int tileM, zb0, zb1; coords(t, tileM, zb0, zb1);
        mbarExpectTx(&barV[j], kTile);
        tmaLoad4d(sV + j * kTile, &mapV, &barV[j], 0, j * kBN, zb1 * p.vZ1, zb0 * p.vZ0);
      };
      bool ok = true;
      if (nIter > 0) { loadQK(0); for (int j = 0; j < nb; ++j) loadV(0, j); }
      for (long long it = 0; it + 1 < nIter && ok; ++it) {
        const uint32_t ph = (uint32_t)it & 1u;
        ok = mbarWait(barQKFree, ph, abortWord);          // every score block of this tile is complete
        if (ok) loadQK(it + 1);
        for (int j = 0; j < nb && ok; ++j) {
          ok = mbarWait(&barVFree[j], ph, abortWord);     // this tile's O += P_j V_j is complete
          if (ok) loadV(it + 1, j);
        }
      }
      if (!ok) atomicExch(&g_attnBlocksStatus, 6);
    }
  } else if (warp == kIssuerWarp) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idescS = instrDesc(1, kBM, kBN, 0, 0);
      constexpr uint32_t idescO = instrDesc(1, kBM, kD, 0, 1);
      const uint64_t dQ = smemDescKMajorSw128(smemAddr(sQ));
      bool ok = true;
      uint32_t g = 0;                                     // key blocks issued so far (over all tiles): buffer g & 1, phase (g >> 1) & 1
      auto issueS = [&](int j, uint32_t gj) {             // S_j = Q K_j^T into score buffer gj & 1, once that buffer has been read
        const uint32_t b = gj & 1u;
        ok = ok && mbarWait(&barSEmpty[b], ((gj >> 1) & 1u) ^ 1u, abortWord);
        tcFenceAfter();
        const uint64_t dK = smemDescKMajorSw128(smemAddr(sK + j * kTile));
#pragma unroll
        for (int k = 0; k < 4; ++k) mmaSS<false>(tmemBase + kColS + b * kBN, dQ + 2 * k, dK + 2 * k, idescS, k > 0 ? 1u : 0u);
        mmaCommit(&barSFull[b]);
      };
      for (long long it = 0; it < nIter && ok; ++it) {
        const uint32_t ph = (uint32_t)it & 1u;
        ok = mbarWait(barQK, ph, abortWord);
        tcFenceAfter();
        issueS(0, g);
        if (nb > 1) issueS(1, g + 1);
        if (nb <= 2) mmaCommit(barQKFree);                // the tile's last score block has been issued
        for (int j = 0; j < nb; ++j) {
          const uint32_t gj = g + (uint32_t)j, b = gj & 1u;
          ok = ok && mbarWait(&barPFull[b], (gj >> 1) & 1u, abortWord);      // P_j written, O rescaled if the maximum moved
          if (j == 0 && it > 0) ok = ok && mbarWait(barOEmpty, ph ^ 1, abortWord);   // the previous tile's O has been read
          ok = ok && mbarWait(&barV[j], ph, abortWord);
          tcFenceAfter();
          const int atoms = p.kAtoms - 2 * j < 2 ? p.kAtoms - 2 * j : 2;     // 64-key atoms of this block
          for (int a = 0; a < atoms; ++a) {               // P is K-major in atoms of 64 keys, V the MN-major operand (head dim contiguous)
            const uint64_t dP = smemDescKMajorSw128(smemAddr(sP + (b * 2 + a) * kTile));
            const uint64_t dV = smemDescMnMajorSw128(smemAddr(sV + (2 * j + a) * 64 * 128), 64 * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) mmaSS<false>(tmemBase + kColO, dP + 2 * k, dV + (uint64_t)(k * ((16 * 128) >> 4)), idescO, (j > 0 || a > 0 || k > 0) ? 1u : 0u);
          }
          mmaCommit(&barPEmpty[b]);
          mmaCommit(&barVFree[j]);
          if (j == nb - 1) mmaCommit(barOFull);           // also reached after a failed wait, so that the other warps do not spin out
          if (j + 2 < nb) { issueS(j + 2, gj + 2); if (j + 2 == nb - 1) mmaCommit(barQKFree); }
        }
        g += (uint32_t)nb;
      }
      if (!ok) atomicExch(&g_attnBlocksStatus, 6);
    }
  } else {
    // ---------------------------------------------------------------- softmax and epilogue
    const int q = warp & 3, h = warp >> 2;             // tensor-memory lane quarter (a hardware rule) and chunk of the block
    const int row = q * 32 + lane;
    const uint32_t trow = tmemBase + ((uint32_t)(q * 32) << 16);
    long long maskAt = -1;                             // offset of the mask row that is staged in shared memory
    bool plain = false;                                // the mask row is all zeros and covers every column: logits are scale * score
    uint32_t g = 0;
    bool ok = true;                                    // after a wait gave up the loop still runs (every thread must reach every barrier)
    for (long long it = 0; it < nIter; ++it) {
      const uint32_t ph = (uint32_t)it & 1u;
      int tileM, zb0, zb1; coords(it, tileM, zb0, zb1);
      const long long gm = (long long)tileM * kBM + row;
      const long long maskRow = zb0 * p.m_s0 + zb1 * p.m_s1;
      if (rowMask && maskRow != maskAt) {              // mask row (times log2 e); columns past the last key get -inf
        softmaxBarrier();                              // nobody still reads the previous row
        if (threadIdx.x == 0) *sMaskSet = 0;
        softmaxBarrier();
        const long long mBase = maskRow;
        bool any = false;
        for (int c = threadIdx.x; c < kMaxN; c += kSoftmaxThreads) {
          const float mv = c < p.N ? (p.mask ? loadAs(p.mask, mBase + c, p.mask_dtype) * kLog2e : 0.f) : -INFINITY;
          sMask[c] = mv;
          any = any || (c < nb * kBN && mv != 0.f);
        }
        if (any) *sMaskSet = 1;
        maskAt = maskRow;
        softmaxBarrier();
        plain = *sMaskSet == 0 && p.scaleLog2e > 0.f;
      }
      const long long mRow = zb0 * p.m_s0 + zb1 * p.m_s1 + gm * p.m_sm;
      float mRun = 0.f, sum = 0.f;                     // running maximum (log2 units) and this thread's share of the row sum
      bool have = false;                               // a finite maximum has been seen (until then every probability was 0)
      for (int j = 0; j < nb; ++j, ++g) {
        const uint32_t b = g & 1u, bph = (g >> 1) & 1u;
        if (ok && !mbarWait(&barSFull[b], bph, abortWord)) { atomicExch(&g_attnBlocksStatus, 7); ok = false; }
        tcFenceAfter();
        float v[32];
        __syncwarp();
        tmemLoad32x32(trow + kColS + b * kBN + (uint32_t)(h * 32), v);
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(&barSEmpty[b]);      // the chunk is in registers: the buffer may take the block after next
        // logits in log2 units
        const int col0 = j * kBN + h * 32;
        if (plain) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= p.scaleLog2e;
        } else if (rowMask) {
          const float4* m4 = reinterpret_cast<const float4*>(sMask + col0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 mk = m4[i];
            v[4 * i] = fmaf(v[4 * i], p.scaleLog2e, mk.x); v[4 * i + 1] = fmaf(v[4 * i + 1], p.scaleLog2e, mk.y);
            v[4 * i + 2] = fmaf(v[4 * i + 2], p.scaleLog2e, mk.z); v[4 * i + 3] = fmaf(v[4 * i + 3], p.scaleLog2e, mk.w);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = col0 + i;
            v[i] = (col >= p.N) ? -INFINITY : (gm >= p.M ? v[i] * p.scaleLog2e : fmaf(v[i], p.scaleLog2e, loadAs(p.mask, mRow + col, p.mask_dtype) * kLog2e));
          }
        }
        float mx = v[0];
#pragma unroll
        for (int i = 1; i < 32; ++i) mx = fmaxf(mx, v[i]);
        float* part = sPart + (j & 1) * kGroups * 128;
        part[h * 128 + row] = mx;
        quarterBarrier(q);
        mx = fmaxf(fmaxf(part[row], part[128 + row]), fmaxf(part[256 + row], part[384 + row]));
        // the running maximum follows in steps: the same decision in the row's four threads (they read the same values)
        float factor = 1.f;
        bool moved = false;
        if (!have) {                                   // nothing but masked columns so far: O and the sum are still 0, no rescaling
          if (mx != -INFINITY) { mRun = mx; have = true; }
        } else if (mx > mRun + kRescaleStep) { factor = fastExp2(mRun - mx); mRun = mx; moved = true; }
        const bool anyMoved = __any_sync(0xffffffffu, moved);
        sum *= factor;
        // P_j: its buffer was last read by the O += P V of two blocks ago
        if (ok && !mbarWait(&barPEmpty[b], bph ^ 1u, abortWord)) { atomicExch(&g_attnBlocksStatus, 7); ok = false; }
        const uint32_t rowAddr = smemAddr(sP + (b * 2 + (h >> 1)) * kTile) + (uint32_t)row * 128u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 pk[4];
          float e8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) { e8[e] = fastExp2(v[i * 8 + e] - mRun); sum += e8[e]; }
#pragma unroll
          for (int e = 0; e < 4; ++e) pk[e] = __floats2bfloat162_rn(e8[2 * e], e8[2 * e + 1]);
          const uint32_t chunk = (uint32_t)((h & 1) * 4 + i);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowAddr + ((chunk ^ (uint32_t)(row & 7)) << 4)), "r"(*reinterpret_cast<unsigned*>(&pk[0])),
                       "r"(*reinterpret_cast<unsigned*>(&pk[1])), "r"(*reinterpret_cast<unsigned*>(&pk[2])), "r"(*reinterpret_cast<unsigned*>(&pk[3])) : "memory");
        }
        if (anyMoved) {
          // some row of this warp moved its maximum: O so far refers to the old one.  Wait for the previous block's
          // O += P V, then scale this warp's 32 rows x 16 columns of O in place (rows that did not move scale by 1).
          const uint32_t gp = g - 1u;
          if (ok && !mbarWait(&barPEmpty[gp & 1u], (gp >> 1) & 1u, abortWord)) { atomicExch(&g_attnBlocksStatus, 7); ok = false; }
          tcFenceAfter();
          float o[16];
          __syncwarp();
          tmemLoadCols<16>(trow + kColO + (uint32_t)(h * 16), o);
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] *= factor;
          tmemStore16(trow + kColO + (uint32_t)(h * 16), o);
          tcFenceBefore();
        }
        fenceProxyAsync();                             // P was written through the generic proxy, the MMA reads it through the async proxy
        __syncwarp();
        if (lane == 0) mbarArrive(&barPFull[b]);
      }
      // row sum over the row's four threads, then the epilogue: group h takes 64 / kGroups output columns of its rows
      sSum[h * 128 + row] = sum;
      quarterBarrier(q);
      const float tot = (sSum[row] + sSum[128 + row]) + (sSum[256 + row] + sSum[384 + row]);
      const float inv = 1.f / tot;
      if (ok && !mbarWait(barOFull, ph, abortWord)) { atomicExch(&g_attnBlocksStatus, 7); ok = false; }
      tcFenceAfter();
      constexpr int kCols = kD / kGroups;
      float o[kCols];
      __syncwarp();
      tmemLoadCols<kCols>(trow + kColO + (uint32_t)(h * kCols), o);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(barOEmpty);            // O is in registers: the next tile's first O = P V may overwrite it
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
      quarterBarrier(q);                               // sSum and the maxima buffers are free for the next tile
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

int* attnBlocksStatusAddress() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_attnBlocksStatus) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}

// Reads and clears this kernel's status word.
int attnBlocksStatus() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attnBlocksStatus, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attnBlocksStatus, &zero, sizeof(int));
  return v;
}

// The blockwise kernel for a call that llc_cuda_attention has already checked (bf16, head size 64, aligned strides).
int attentionBlocks(const LlcAttentionParams* p, cudaStream_t stream) {
  if (p->n < 1 || p->n > kMaxN) return setError(LLC_ERR_UNSUPPORTED, "llc_cuda_attention: 1 to 512 keys");
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
    cudaError_t e = cudaFuncSetAttribute(attention_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return cudaFail(e, "cudaFuncSetAttribute(attention_blocks_kernel)");
    configured.set(dev);
  }
  a.tiles = batch * mTiles;
  const int sms = deviceSMs();
  a.numZ = batch; a.zMajor = batch >= 2LL * sms;         // enough (batch, head) pairs for every SM to take whole ones
  const long long work = a.zMajor ? a.numZ : a.tiles;
  const unsigned grid = (unsigned)(work < sms ? work : sms);
  attention_blocks_kernel<<<grid, kThreads, kSmemBytes, stream>>>(mq, mk, mv, a);
  LLC_LAUNCH_CHECK("attention_blocks_kernel");
  return LLC_OK;
}

}  // namespace llc

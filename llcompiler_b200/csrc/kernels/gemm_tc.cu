// Tensor-core GEMM and implicit-GEMM convolution for sm_100a: tcgen05.mma with accumulators in
// tensor memory, TMA-fed operands, persistent warp-specialised CTAs, fused epilogue.  Serves
// llc_cuda_gemm / llc_cuda_conv2d for bf16 operands and for fp32 operands at precision tf32 (one
// pass) or tf32x3 (three passes, fp32-grade accuracy).
//
// One CTA per SM loops over 128 x BN output tiles (BN = 64, 128 or 256).  Roles, by warp:
//   warp 0      TMA producer: per K block waits for a free stage, arms its mbarrier with the byte
//               count and issues the tile loads (B: BN rows x 128 bytes; dense GEMM also A: 128 rows
//               x 128 bytes; K-major, 128-byte swizzle; rows/columns past the edge are zero-filled
//               by TMA, which is how M, N and K tails are handled).
//   warp 1      MMA issuer: one lane waits for the stage, issues BK/UMMA_K tcgen05.mma (fp32
//               accumulation into one of two TMEM accumulators), commits the stage back to the
//               producer; after the last K block commits the accumulator to the epilogue.
//               Allocates and frees tensor memory.
//   warps 2-9   epilogue: tcgen05.ld (32 lanes x 32 columns per warp and step, the next step's load in
//               flight; a warp owns one lane quarter and one column half), alpha*scale[n]*acc + shift[n]
//               + res, activation, rows staged in one of two swizzled slots and written by TMA stores;
//               releases the accumulator as soon as it is in registers so that the next tile's MMAs
//               overlap the stores.
//   next 8      convolution only: im2col gather of the A tile (NHWC activations) with 16-byte
//               cp.async into the swizzled layout, zero-filling padding taps.
//   next 4      tf32x3 only: split each landed fp32 tile into its low-order part x - tf32(x)
//               (same swizzled position in a second buffer) and hand the stage to the issuer.
// tf32x3: acc = A_hi*B_hi + A_lo*B_hi + A_hi*B_lo.  The tensor core reads only the upper 19 bits
// of an fp32 operand, so A_hi is the raw tile and A_lo = A - truncate_to_tf32(A) is exact.
//
// Bound: tensor pipe.  Algorithmic FLOPs 2*M*N*K per batch entry; HBM bytes (M*K + N*K + M*N)
// elements; A is re-read once per column of tiles and B once per row of tiles (L2 hits).
#include "common.cuh"
#include "tc_common.cuh"

namespace llc {

__device__ int g_tcStatus = 0;   // non-zero after a bounded wait gave up: 1 producer, 2 issuer, 3 split, 4 epilogue, 5 gather

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int kTileKBytes = 128;          // one swizzle atom along K

struct TcArgs {
  void* out; const float* scale; const float* shift; const void* res;
  int out_dtype, res_dtype, act; float alpha;
  long long M, N, K;
  long long o_s0, o_s1, o_sm, r_s0, r_s1, r_sm, r_sn;
  int b1; int kBlocks; int vecOut;
  int resTile;              // the residual can be fetched as 32-row x 64-byte units with 16-byte loads
  int splits;               // K is cut into this many slices, each a work unit of its own; partial tiles meet in `ws`
  float* ws; int* counters; // split-K: [units][128][BN] partial accumulators; one arrival counter per tile (zero between launches)
  int hasBLo;               // tf32x3: the low-order part of B comes from memory (mapBLo) instead of the split warps
  int tmaOut;               // 0, or the bytes per row of the output box the epilogue stores through TMA (64)
  int aZ0, aZ1, bZ0, bZ1;   // 1: the operand has this batch dim, 0: it is broadcast (coordinate 0)
  int rZ0, rZ1;             // the same for the residual (RES kernels: it is loaded through a tensor map)
  int mTiles, nTiles; long long tiles;
  // convolution (A gathered from NHWC activations)
  const void* x; int H, W, C, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
  long long xs_n, xs_h, xs_w;   // element strides of x along image, row and pixel (dense NHWC: H*W*C, W*C, C)
};

// RES: the epilogue adds a residual tile that TMA loads fetch ahead of time into a ring of four units per epilogue warp
// (the ring also stages the output); without it a warp has two output slots.
template <int BN, bool X3, bool RES> struct Smem {
  static constexpr int kABytes = BM * kTileKBytes, kBBytes = BN * kTileKBytes;
  static constexpr int kStageBytes = (kABytes + kBBytes) * (X3 ? 2 : 1);
  static constexpr int kStagingPerWarp = RES ? 8192 : 4096;   // units of 32 rows x 64 bytes: a ring of four, or two output slots
  static constexpr int kStagingBytes = 8 * kStagingPerWarp;
  static constexpr int kStageBudget = 224 * 1024 - kStagingBytes;
  static constexpr int kStages = kStageBudget / kStageBytes > 8 ? 8 : kStageBudget / kStageBytes;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + kStagingBytes + 1024;   // + alignment slack
};

__device__ __forceinline__ void cpAsync16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // src-size 0: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cpAsyncWait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// The barrier receives one arrival (counted against its expected count) when every cp.async this
// thread has issued so far has landed: the thread itself never waits for its copies.
__device__ __forceinline__ void cpAsyncArriveOn(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smemAddr(bar)) : "memory");
}

// KIND: 0 bf16, 1 tf32, 2 tf32x3.  BMN: B is stored [k][n] (unit stride along n) instead of [n][k].
// Threads of a CTA: producer, issuer, 8 epilogue warps, 8 gather warps (MODE 1), 4 split warps (tf32x3).
__host__ __device__ constexpr int tcThreads(int kind, int mode) { return (2 + 8 + (mode == 1 ? 8 : 0) + (kind == 2 ? 4 : 0)) * 32; }

// MODE: 0 dense GEMM (A by tiled TMA), 1 convolution with A gathered by warps (any channel count that keeps a
// 16-byte chunk inside one filter tap), 2 convolution with A loaded by TMA in im2col mode (a K block of 128
// bytes lies inside one filter tap: channels * element size is a multiple of 128).  (A variant with sixteen epilogue
// warps and one pipeline stage less was measured 1.2 to 1.9 times slower on every shape tried and is not kept.)
template <int BN, int KIND, int MODE, bool BMN, bool RES>
__global__ void __launch_bounds__(tcThreads(KIND, MODE), 1)
tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapO,
          const __grid_constant__ CUtensorMap mapBLo, const __grid_constant__ CUtensorMap mapR, const TcArgs p) {
  constexpr bool X3 = KIND == 2;
  constexpr bool TF32 = KIND != 0;
  constexpr bool CONV = MODE == 1;      // the gather warps exist
  constexpr bool IM2COL = MODE == 2;
  using S = Smem<BN, X3, RES>;
  static_assert(!RES || (KIND != 2 && MODE != 1 && !BMN), "the residual ring exists for bf16 / tf32 kernels with TMA-fed operands");
  constexpr int kStages = S::kStages;
  constexpr int kElemBytes = TF32 ? 4 : 2;
  constexpr int BK = kTileKBytes / kElemBytes;          // 64 bf16 / 32 tf32
  constexpr int UMMA_K = 32 / kElemBytes;               // 16 bf16 / 8 tf32 (32 bytes of K per instruction)
  constexpr uint32_t kIdesc = instrDesc(TF32 ? 2 : 1, BM, BN, 0, BMN ? 1 : 0);
  // Two accumulator sets (double buffering).  tf32x3 splits the K loop over kChains independent
  // accumulators per set and adds them in the epilogue: the tensor core truncates when it adds into
  // its fp32 accumulator, so shorter chains mean a smaller (K-proportional) rounding bias.
  constexpr int kChains = X3 ? 256 / BN : 1;
  constexpr int kSetCols = X3 ? 256 : BN;
  constexpr int kAccCols = 2 * kSetCols;
  static_assert(!X3 || BN <= 128, "tf32x3 uses BN <= 128");
  constexpr int kAtomN = kTileKBytes / kElemBytes;      // BMN: elements of n per 128-byte slab row
  constexpr int kSlabBytes = BK * 128;                  // BMN: one slab = BK rows of k x 128 bytes of n
  constexpr int kEpiWarps = 8;
  constexpr int kGatherWarps = 8;
  constexpr int kGatherWarp0 = 2 + kEpiWarps, kSplitWarp0 = kGatherWarp0 + (CONV ? kGatherWarps : 0);
  constexpr int kFullCount = CONV ? kGatherWarps * 32 + 1 : 1;   // gather threads + the TMA arm

  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* full = bars;                    // [kStages] operands landed
  uint64_t* empty = bars + kStages;         // [kStages] MMAs that read the stage are done
  uint64_t* split = bars + 2 * kStages;     // [kStages] low-order tiles written (tf32x3)
  uint64_t* accFull = bars + 3 * kStages;   // [2] accumulator complete
  uint64_t* accEmpty = bars + 3 * kStages + 2;  // [2] accumulator drained by the epilogue
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 4);
  volatile int* abortWord = reinterpret_cast<volatile int*>(tmemSlot + 1);
  volatile int* lastFlag = abortWord + 1;       // split-K: whether this CTA's unit arrived last at its tile
  uint64_t* resFull = bars + 64;                // [8 epilogue warps][4]: a unit of the residual has landed (RES)
  uint8_t* staging = smem + kStages * S::kStageBytes + S::kBarrierBytes;   // 1024-byte aligned
  constexpr int kStagingPerWarp = S::kStagingPerWarp;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbarInit(&full[s], kFullCount); mbarInit(&empty[s], 1); mbarInit(&split[s], 4); }
    for (int a = 0; a < 2; ++a) { mbarInit(&accFull[a], 1); mbarInit(&accEmpty[a], kEpiWarps); }
    if (RES) for (int i = 0; i < kEpiWarps * 4; ++i) mbarInit(&resFull[i], 1);
    *abortWord = 0;
    fenceBarrierInit();
  }
  if (warp == 1) tmemAlloc(tmemSlot, kAccCols);
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  auto stageA = [&](int s) { return tiles + s * S::kStageBytes; };
  auto stageB = [&](int s) { return tiles + s * S::kStageBytes + S::kABytes; };
  auto stageALo = [&](int s) { return tiles + s * S::kStageBytes + S::kABytes + S::kBBytes; };
  auto stageBLo = [&](int s) { return tiles + s * S::kStageBytes + 2 * S::kABytes + S::kBBytes; };
  const long long tilesPerBatch = (long long)p.mTiles * p.nTiles;
  // Work units: (tile, K slice).  Without split-K a unit is a tile and its slice the whole K loop.
  const long long units = p.tiles * p.splits;
  const int kPer = (p.kBlocks + p.splits - 1) / p.splits;
  auto sliceOf = [&](long long u, long long& t, int& kb0, int& kb1) {
    t = u / p.splits; const int sidx = (int)(u - t * p.splits);
    kb0 = sidx * kPer; kb1 = kb0 + kPer < p.kBlocks ? kb0 + kPer : p.kBlocks;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      if (!CONV) prefetchTensorMap(&mapA);
      int ow0 = 0, oh0 = 0, img0 = 0;
      prefetchTensorMap(&mapB);
      uint32_t it = 0;
      bool ok = true;
      for (long long u = blockIdx.x; u < units && ok; u += gridDim.x) {
        long long t; int kb0, kb1; sliceOf(u, t, kb0, kb1);
        const int z = (int)(t / tilesPerBatch); const int rem = (int)(t - z * tilesPerBatch);
        const int tileM = rem / p.nTiles, tileN = rem - tileM * p.nTiles;
        const int zb0 = z / p.b1, zb1 = z - zb0 * p.b1;
        int tapR = 0, tapS = 0, cc = 0;                      // im2col: filter tap and first channel of the K block
        if (IM2COL && kb0 > 0) { const long long k0 = (long long)kb0 * BK; const int tap = (int)(k0 / p.C); cc = (int)(k0 - (long long)tap * p.C); tapR = tap / p.KW; tapS = tap - tapR * p.KW; }
        if (IM2COL) {
          const long long m0 = (long long)tileM * BM;          // first output pixel of the tile
          ow0 = (int)(m0 % p.OW); const long long t2 = m0 / p.OW; oh0 = (int)(t2 % p.OH); img0 = (int)(t2 / p.OH);
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
          if (!mbarWait(&empty[s], ph ^ 1, abortWord)) { atomicExch(&g_tcStatus, 1); ok = false; break; }
          mbarExpectTx(&full[s], (CONV ? S::kBBytes : S::kABytes + S::kBBytes) + ((X3 && p.hasBLo) ? S::kBBytes : 0));
          if (MODE == 0) tmaLoad4d(stageA(s), &mapA, &full[s], kb * BK, tileM * BM, zb1 * p.aZ1, zb0 * p.aZ0);
          if (IM2COL) {
            // 128 output pixels from (img0, oh0, ow0) on, in w -> h -> n order; the coordinates name the input pixel
            // under filter tap (0, 0), the offsets select the tap
            tmaLoadIm2col4d(stageA(s), &mapA, &full[s], cc, ow0 * p.sw - p.pw, oh0 * p.sh - p.ph, img0, (uint16_t)(tapS * p.dw), (uint16_t)(tapR * p.dh));
            cc += BK;
            if (cc >= p.C) { cc = 0; if (++tapS == p.KW) { tapS = 0; ++tapR; } }
          }
          if (BMN) {
#pragma unroll
            for (int a = 0; a < BN / kAtomN; ++a)
              tmaLoad4d(stageB(s) + a * kSlabBytes, &mapB, &full[s], tileN * BN + a * kAtomN, kb * BK, zb1 * p.bZ1, zb0 * p.bZ0);
          } else {
            tmaLoad4d(stageB(s), &mapB, &full[s], kb * BK, tileN * BN, zb1 * p.bZ1, zb0 * p.bZ0);
            if (X3 && p.hasBLo) tmaLoad4d(stageBLo(s), &mapBLo, &full[s], kb * BK, tileN * BN, zb1 * p.bZ1, zb0 * p.bZ0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (long long u = blockIdx.x; u < units && ok; u += gridDim.x, ++tcount) {
        long long t; int kb0, kb1; sliceOf(u, t, kb0, kb1);
        const int ab = tcount & 1; const uint32_t aph = (tcount >> 1) & 1;
        if (!mbarWait(&accEmpty[ab], aph ^ 1, abortWord)) { atomicExch(&g_tcStatus, 2); ok = false; break; }
        tcFenceAfter();
        const uint32_t accSet = tmemBase + (uint32_t)(ab * kSetCols);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
          if (!mbarWait(X3 ? &split[s] : &full[s], ph, abortWord)) { atomicExch(&g_tcStatus, 2); ok = false; break; }
          if (CONV && !X3) fenceProxyAsync();               // the gathered A tile was written through the generic proxy
          tcFenceAfter();
          const uint32_t acc = accSet + (uint32_t)(((kb - kb0) % kChains) * BN);
          const bool fresh = kb - kb0 < kChains;           // first K block of this chain: overwrite
          const uint64_t dA = smemDescKMajorSw128(smemAddr(stageA(s)));
          const uint64_t dB = BMN ? smemDescMnMajorSw128(smemAddr(stageB(s)), kSlabBytes) : smemDescKMajorSw128(smemAddr(stageB(s)));
          constexpr uint64_t kAdvA = (UMMA_K * kElemBytes) >> 4;                      // 32 bytes of K inside the swizzle atom
          constexpr uint64_t kAdvB = BMN ? (uint64_t)(UMMA_K * 128) >> 4 : kAdvA;     // BMN: UMMA_K rows of 128 bytes
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            mmaSS<TF32>(acc, dA + k * kAdvA, dB + k * kAdvB, kIdesc, (!fresh || k > 0) ? 1u : 0u);
          if (X3) {
            const uint64_t dAl = smemDescKMajorSw128(smemAddr(stageALo(s)));
            const uint64_t dBl = BMN ? smemDescMnMajorSw128(smemAddr(stageBLo(s)), kSlabBytes) : smemDescKMajorSw128(smemAddr(stageBLo(s)));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              mmaSS<TF32>(acc, dAl + k * kAdvA, dB + k * kAdvB, kIdesc, 1u);
              mmaSS<TF32>(acc, dA + k * kAdvA, dBl + k * kAdvB, kIdesc, 1u);
            }
          }
          mmaCommit(&empty[s]);
        }
        mmaCommit(&accFull[ab]);   // also reached after a failed wait so that the epilogue does not spin out
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ---------------------------------------------------------------- epilogue
    // Warp w reads TMEM lanes 32*(w%4)..+31 (a hardware rule) and the column share (w-2)/4 of the tile, in chunks of 32
    // columns; the accumulator load of chunk i+1 is in flight while chunk i is worked on.  Results leave as units of
    // 32 rows x 64 bytes (32 bf16 or 16 fp32 columns, 64-byte swizzle), each staged in shared memory and written by one
    // TMA store, so that the store of a unit overlaps the arithmetic of the next.
    //   RES kernels: a warp owns a ring of four unit buffers.  The residual of a unit is loaded into its buffer by TMA
    //   three units ahead (across tile boundaries: it depends on nothing the MMAs produce), the lane adds its row,
    //   writes the result back into the same buffer and the store takes it from there.
    //   Other kernels: two output slots used in turn; a residual, if any, comes through registers (below).
    const int q = warp & 3, half = (warp - 2) >> 2;
    constexpr int kColsPerWarp = BN / (kEpiWarps / 4);
    constexpr int kChunks = kColsPerWarp / 32;
    constexpr bool kPrefetch = kChains == 1 && !CONV;           // tf32x3 adds several accumulators per chunk, and the gather form has no registers to spare
    constexpr uint32_t kRing = RES ? 4u : 2u;
    char* outBase = reinterpret_cast<char*>(p.out);
    const bool outF32 = p.out_dtype == LLC_FLOAT32;
    const bool tma = RES || p.tmaOut != 0;
    const int esz = outF32 ? 4 : 2;
    const int unitCols = 64 / esz;                              // columns of one staged unit
    const int nUnits = kColsPerWarp / unitCols;                 // units of this warp per tile
    uint8_t* const warpStaging = staging + (warp - 2) * kStagingPerWarp;
    const uint32_t slotBase = smemAddr(warpStaging);
    uint64_t* const myResFull = resFull + (warp - 2) * 4;
    uint32_t slotIt = 0;                                        // units this warp has staged so far; the buffer in use is slotIt % kRing
    // 16-byte piece c of row r of a unit buffer (64-byte swizzle: the piece index is XORed with bits 1-2 of the row)
    auto pieceAddr = [&](uint32_t slot, uint32_t r, uint32_t c) { return slotBase + (slot << 11) + r * 64u + ((c ^ ((r >> 1) & 3u)) << 4); };
    auto acquireSlot = [&]() { if (lane == 0) bulkWaitRead1(); __syncwarp(); };   // the store before the last has read its slot
    // RES: starts the TMA load of the residual of this warp's unit number m (counted over all its tiles) into buffer m % 4
    auto loadResUnit = [&](uint32_t m) {
      const long long um = blockIdx.x + (long long)(m / (uint32_t)nUnits) * gridDim.x;
      if (um >= units) return;                                   // past this CTA's last tile: nobody will wait for it
      const int g = (int)(m % (uint32_t)nUnits);
      const int z = (int)(um / tilesPerBatch); const int rem = (int)(um - z * tilesPerBatch);
      const int tM = rem / p.nTiles, tN = rem - tM * p.nTiles;
      const int z0 = z / p.b1, z1 = z - z0 * p.b1;
      uint64_t* bar = &myResFull[m & 3u];
      mbarExpectTx(bar, 2048);
      tmaLoad4d(warpStaging + ((m & 3u) << 11), &mapR, bar, tN * BN + half * kColsPerWarp + g * unitCols, tM * BM + q * 32, z1 * p.rZ1, z0 * p.rZ0);
    };
    if (RES && lane == 0) { prefetchTensorMap(&mapR); loadResUnit(0); loadResUnit(1); loadResUnit(2); }
    if (tma && lane == 0) prefetchTensorMap(&mapO);
    uint32_t tcount = 0;
    for (long long u = blockIdx.x; u < units; u += gridDim.x, ++tcount) {
      long long t; int kb0, kb1; sliceOf(u, t, kb0, kb1);
      const int z = (int)(t / tilesPerBatch); const int rem = (int)(t - z * tilesPerBatch);
      const int tileM = rem / p.nTiles, tileN = rem - tileM * p.nTiles;
      const int zb0 = z / p.b1, zb1 = z - zb0 * p.b1;
      const int ab = tcount & 1; const uint32_t aph = (tcount >> 1) & 1;
      const long long gm = (long long)tileM * BM + q * 32 + lane;
      const bool rowOk = gm < p.M;
      const bool rowsInside = (long long)tileM * BM + q * 32 < p.M;          // this warp's 32 rows are not all past the edge
      const long long oRow = zb0 * p.o_s0 + zb1 * p.o_s1 + gm * p.o_sm;
      const long long rRow = zb0 * p.r_s0 + zb1 * p.r_s1 + gm * p.r_sm;
      // Residual through registers (kernels without the ring).  A unit of the residual (32 rows x 64 bytes, the box
      // the output store writes) is fetched with coalesced 16-byte loads (four lanes per row, eight rows per
      // instruction), passed through the staging slot and read back one row per lane: lane = row is how the
      // accumulator arrives, but loading global memory that way touches 32 lines per instruction.  The loads of unit
      // g + 1 are issued when unit g is taken over, those of unit 0 while the MMAs still run.
      const bool resTile = !RES && !CONV && p.resTile && tma;    // (the gather kernel has no registers to spare and its layers no residual)
      uint4 rA[4];
      auto issueRes = [&](int g) {
        const int piece = lane & 3, r0 = lane >> 2;
        const long long gcol = (long long)tileN * BN + half * kColsPerWarp + (long long)g * unitCols + piece * (16 / esz);
        const char* base = reinterpret_cast<const char*>(p.res) + (zb0 * p.r_s0 + zb1 * p.r_s1 + gcol) * esz;
        const bool colOk = gcol < p.N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long gr = (long long)tileM * BM + q * 32 + j * 8 + r0;
          rA[j] = (gr < p.M && colOk) ? __ldg(reinterpret_cast<const uint4*>(base + gr * p.r_sm * esz)) : make_uint4(0u, 0u, 0u, 0u);
        }
      };
      // The lane's own row of the residual of the unit in buffer `slot`, as four 16-byte pieces.
      auto ownRow = [&](uint32_t slot, uint4* own) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(own[c].x), "=r"(own[c].y), "=r"(own[c].z), "=r"(own[c].w)
                       : "r"(pieceAddr(slot, (uint32_t)lane, (uint32_t)c)) : "memory");
      };
      // Takes unit g over (register path): the residual rows go through the acquired slot, the next unit's loads start.
      auto residualRow = [&](int g, uint4* own) {
        const uint32_t slot = slotIt % kRing;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 r = rA[j];
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(pieceAddr(slot, (uint32_t)(j * 8 + (lane >> 2)), (uint32_t)(lane & 3))), "r"(r.x), "r"(r.y),
                       "r"(r.z), "r"(r.w) : "memory");
        }
        __syncwarp();                                            // from here on every lane touches only its own row
        if (g + 1 < nUnits) issueRes(g + 1);
        ownRow(slot, own);
      };
      // Ring path: waits for the residual of the current unit to land and reads the lane's row.
      auto ringRow = [&](uint4* own) {
        if (!mbarWait(&myResFull[slotIt & 3u], (slotIt >> 2) & 1u, abortWord)) atomicExch(&g_tcStatus, 4);
        ownRow(slotIt & 3u, own);
      };
      // Hands the staged unit to the TMA store (columns from x0 on; rows past M and columns past N are clipped by the
      // store).  A group is committed even when nothing is stored, so that "all but the latest group" always means
      // "every unit before this one".  RES: the buffer of the unit before this one is then free for the residual of
      // the unit three ahead.
      auto storeUnit = [&](long long x0) {
        fenceProxyAsync();
        __syncwarp();
        if (lane == 0) {
          if (rowsInside && x0 < p.N) tmaStore4d(&mapO, warpStaging + ((slotIt % kRing) << 11), (int)x0, tileM * BM + q * 32, zb1, zb0);
          bulkCommit();
          if (RES) { bulkWaitRead1(); loadResUnit(slotIt + 3u); }
        }
        ++slotIt;
      };
      auto stageF32 = [&](const float* w) {                      // 16 fp32 values -> the lane's row of the current buffer
        const uint32_t slot = slotIt % kRing;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(pieceAddr(slot, (uint32_t)lane, (uint32_t)c)), "f"(w[4 * c]), "f"(w[4 * c + 1]),
                       "f"(w[4 * c + 2]), "f"(w[4 * c + 3]) : "memory");
      };
      auto stageBf16 = [&](const float* w) {                     // 32 fp32 values, rounded to bf16
        const uint32_t slot = slotIt % kRing;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const __nv_bfloat162 a0 = __floats2bfloat162_rn(w[8 * c], w[8 * c + 1]), a1 = __floats2bfloat162_rn(w[8 * c + 2], w[8 * c + 3]);
          const __nv_bfloat162 a2 = __floats2bfloat162_rn(w[8 * c + 4], w[8 * c + 5]), a3 = __floats2bfloat162_rn(w[8 * c + 6], w[8 * c + 7]);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(pieceAddr(slot, (uint32_t)lane, (uint32_t)c)),
                       "r"(*reinterpret_cast<const unsigned*>(&a0)), "r"(*reinterpret_cast<const unsigned*>(&a1)), "r"(*reinterpret_cast<const unsigned*>(&a2)),
                       "r"(*reinterpret_cast<const unsigned*>(&a3)) : "memory");
        }
      };
      const bool splitK = !RES && p.splits > 1;
      if (resTile && !splitK) issueRes(0);
      if (!mbarWait(&accFull[ab], aph, abortWord)) atomicExch(&g_tcStatus, 4);   // carry on with whatever is there: every warp must still reach the barriers below
      tcFenceAfter();
      const uint32_t acc = tmemBase + (uint32_t)(ab * kSetCols) + ((uint32_t)(q * 32) << 16);
      const int usedChains = kb1 - kb0 < kChains ? kb1 - kb0 : kChains;
      // Split-K: every unit parks its partial tile (fp32, this lane's row) in the workspace; the unit that arrives last
      // at the tile's counter adds the slices up and runs the epilogue.  Units of one tile run on different CTAs at the
      // same time (the grid holds every unit), so nobody waits for anybody.
      const float4* wsRow = nullptr;
      if (splitK) {
        // Layout of a parked tile: [epilogue warp][32-column chunk][float4 of the chunk][lane], so that one store (and,
        // in the unit that adds up, one load) of a warp covers 512 contiguous bytes.  Writer and reader are the same
        // (warp, lane) position of their CTAs, so the layout needs to make sense to nobody else.
        float4* mine = reinterpret_cast<float4*>(p.ws + (size_t)u * BM * BN) + (size_t)((half * 4 + q) * (kColsPerWarp / 4)) * 32 + lane;
#pragma unroll 1
        for (int ci = 0; ci < kChunks; ++ci) {
          const int c0 = half * kColsPerWarp + ci * 32;
          float v[32];
          __syncwarp();
          tmemLoad32x32(acc + (uint32_t)c0, v);
          if (kChains > 1) {
            for (int ch = 1; ch < usedChains; ++ch) {
              float w[32];
              tmemLoad32x32(acc + (uint32_t)(ch * BN + c0), w);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += w[j];
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) __stcg(mine + (ci * 8 + j) * 32, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
        }
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(&accEmpty[ab]);
        __threadfence();                                 // the partial tile is visible before the arrival is counted
        asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * 32) : "memory");
        if (warp == 2 && lane == 0) {
          const int old = atomicAdd(&p.counters[t], 1);
          const int last = old == p.splits - 1;
          if (last) p.counters[t] = 0;                   // everyone has arrived: the counter is zero again for the next launch
          *lastFlag = last;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * 32) : "memory");
        if (!*lastFlag) continue;
        __threadfence();
        wsRow = reinterpret_cast<const float4*>(p.ws + (size_t)(t * p.splits) * BM * BN) + (size_t)((half * 4 + q) * (kColsPerWarp / 4)) * 32 + lane;
        if (resTile) issueRes(0);
      }
      const bool pipelined = kPrefetch && !splitK;
      uint32_t raw[32];
      if (pipelined) { __syncwarp(); tmemIssue32(acc + (uint32_t)(half * kColsPerWarp), raw); }
#pragma unroll 1
      for (int ci = 0; ci < kChunks; ++ci) {
        const int c0 = half * kColsPerWarp + ci * 32;
        float v[32];
        if (splitK) {                                   // the slices' partial sums, from the workspace (L2)
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float4 f = __ldcg(wsRow + (ci * 8 + j) * 32); v[4 * j] = f.x; v[4 * j + 1] = f.y; v[4 * j + 2] = f.z; v[4 * j + 3] = f.w; }
          for (int sl = 1; sl < p.splits; ++sl) {
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float4 f = __ldcg(wsRow + (size_t)sl * (BM * BN / 4) + (ci * 8 + j) * 32); v[4 * j] += f.x; v[4 * j + 1] += f.y; v[4 * j + 2] += f.z; v[4 * j + 3] += f.w; }
          }
        } else if (pipelined) {
          tmemWait32(raw);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          if (ci + 1 < kChunks) { __syncwarp(); tmemIssue32(acc + (uint32_t)(c0 + 32), raw); }
        } else {
          __syncwarp();                                 // the load is warp-collective
          tmemLoad32x32(acc + (uint32_t)c0, v);
          if (kChains > 1) {
            for (int ch = 1; ch < usedChains; ++ch) {
              float w[32];
              tmemLoad32x32(acc + (uint32_t)(ch * BN + c0), w);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += w[j];
            }
          }
        }
        if (!splitK && ci == kChunks - 1) {             // this warp's share is in registers: hand the accumulator back
          tcFenceBefore();
          __syncwarp();
          if (lane == 0) mbarArrive(&accEmpty[ab]);
        }
        const long long gn0 = (long long)tileN * BN + c0;
        const bool inside = gn0 < p.N;
        const bool whole = p.vecOut && gn0 + 32 <= p.N;
        const int g0 = (ci * 32) / unitCols;              // first unit of this chunk
        // v = alpha * scale[n] * v + shift[n]: one multiply-add per element with the folded per-column factors
        if (whole) {
          const float4* sc = p.scale ? reinterpret_cast<const float4*>(p.scale + gn0) : nullptr;
          const float4* sh = p.shift ? reinterpret_cast<const float4*>(p.shift + gn0) : nullptr;
          if (sc || sh || p.alpha != 1.f) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 s4 = sc ? __ldg(sc + j) : make_float4(1.f, 1.f, 1.f, 1.f);
              const float4 b4 = sh ? __ldg(sh + j) : make_float4(0.f, 0.f, 0.f, 0.f);
              s4.x *= p.alpha; s4.y *= p.alpha; s4.z *= p.alpha; s4.w *= p.alpha;
              v[4 * j] = fmaf(v[4 * j], s4.x, b4.x); v[4 * j + 1] = fmaf(v[4 * j + 1], s4.y, b4.y);
              v[4 * j + 2] = fmaf(v[4 * j + 2], s4.z, b4.z); v[4 * j + 3] = fmaf(v[4 * j + 3], s4.w, b4.w);
            }
          }
        } else if (inside) {
          // ragged edge (the last column tile, or vectors that are not 16-byte aligned): element by element
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const long long n = gn0 + j;
            if (n < p.N) {
              float x = v[j] * p.alpha;
              if (p.scale) x *= __ldg(p.scale + n);
              if (p.shift) x += __ldg(p.shift + n);
              v[j] = x;
            }
          }
        }
        auto activate = [&](float* w, int count) {
          if (p.act == LLC_ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < count) w[j] = fmaxf(w[j], 0.f);
          } else if (p.act == LLC_ACT_GELU) {
            if (outF32) {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < count) w[j] = geluFast(w[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < count) w[j] = geluTanhBf16(w[j]);
            }
          }
        };
        if constexpr (RES) {
          // every unit of every tile goes through the ring, inside the matrix or not (loads past the edge read zeros,
          // stores past the edge write nothing), so that buffers and barrier phases advance uniformly
          if (outF32) {
#pragma unroll
            for (int un = 0; un < 2; ++un) {
              uint4 own[4];
              ringRow(own);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                v[un * 16 + 4 * c] += __uint_as_float(own[c].x); v[un * 16 + 4 * c + 1] += __uint_as_float(own[c].y);
                v[un * 16 + 4 * c + 2] += __uint_as_float(own[c].z); v[un * 16 + 4 * c + 3] += __uint_as_float(own[c].w);
              }
              activate(v + un * 16, 16);
              stageF32(v + un * 16);
              storeUnit(gn0 + un * 16);
            }
          } else {
            uint4 own[4];
            ringRow(own);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&own[c]);
#pragma unroll
              for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[8 * c + 2 * e] += f.x; v[8 * c + 2 * e + 1] += f.y; }
            }
            activate(v, 32);
            stageBf16(v);
            storeUnit(gn0);
          }
        } else if (whole) {
          // residual, in fp32 (one rounding for the sum, whatever the storage type)
          bool slotHeld = false;                            // bf16: the unit's slot was acquired for the residual already
          if (resTile) {
            if (!outF32) {
              uint4 own[4];
              acquireSlot(); residualRow(g0, own); slotHeld = true;
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&own[c]);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[8 * c + 2 * e] += f.x; v[8 * c + 2 * e + 1] += f.y; }
              }
            }                                               // fp32: two units per chunk, each takes its residual below
          } else if (p.res && rowOk) {
            if (p.r_sn == 1 && p.res_dtype == LLC_BFLOAT16 && ((rRow + gn0) & 3) == 0) {
              const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(p.res) + rRow + gn0;
#pragma unroll
              for (int j = 0; j < 8; ++j) { float4 r4 = Vec4<__nv_bfloat16>::load(rp + 4 * j); v[4 * j] += r4.x; v[4 * j + 1] += r4.y; v[4 * j + 2] += r4.z; v[4 * j + 3] += r4.w; }
            } else if (p.r_sn == 1 && p.res_dtype == LLC_FLOAT32 && ((rRow + gn0) & 3) == 0) {
              const float* rp = reinterpret_cast<const float*>(p.res) + rRow + gn0;
#pragma unroll
              for (int j = 0; j < 8; ++j) { float4 r4 = Vec4<float>::load(rp + 4 * j); v[4 * j] += r4.x; v[4 * j + 1] += r4.y; v[4 * j + 2] += r4.z; v[4 * j + 3] += r4.w; }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += loadAs(p.res, rRow + (gn0 + j) * p.r_sn, p.res_dtype);
            }
          }
          // (with fp32 output and a residual tile the activation follows the residual, unit by unit, below)
          if (!(resTile && outF32)) activate(v, 32);
          if (tma) {
            if (outF32) {
#pragma unroll
              for (int un = 0; un < 2; ++un) {
                acquireSlot();
                if (resTile) {
                  uint4 own[4];
                  residualRow(g0 + un, own);
#pragma unroll
                  for (int c = 0; c < 4; ++c) {
                    v[un * 16 + 4 * c] += __uint_as_float(own[c].x); v[un * 16 + 4 * c + 1] += __uint_as_float(own[c].y);
                    v[un * 16 + 4 * c + 2] += __uint_as_float(own[c].z); v[un * 16 + 4 * c + 3] += __uint_as_float(own[c].w);
                  }
                  activate(v + un * 16, 16);
                }
                stageF32(v + un * 16);
                storeUnit(gn0 + un * 16);
              }
            } else {
              if (!slotHeld) acquireSlot();
              stageBf16(v);
              storeUnit(gn0);
            }
          } else if (rowOk) {
            if (outF32) {
              float* dst = reinterpret_cast<float*>(outBase) + oRow + gn0;
#pragma unroll
              for (int j = 0; j < 32; j += 4) Vec4<float>::store(dst + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
            } else {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(outBase) + oRow + gn0);
              const bool al16 = ((oRow + gn0) & 7) == 0;
              if (al16) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 a0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]), a1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                  __nv_bfloat162 a2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]), a3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                  uint4 pk; pk.x = *reinterpret_cast<unsigned*>(&a0); pk.y = *reinterpret_cast<unsigned*>(&a1); pk.z = *reinterpret_cast<unsigned*>(&a2); pk.w = *reinterpret_cast<unsigned*>(&a3);
                  dst[j] = pk;
                }
              } else {
                __nv_bfloat16* d2 = reinterpret_cast<__nv_bfloat16*>(outBase) + oRow + gn0;
#pragma unroll
                for (int j = 0; j < 32; j += 4) Vec4<__nv_bfloat16>::store(d2 + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
              }
            }
          }
        } else if (inside) {
          // ragged edge, continued: residual and activation element by element, then staged units or scalar stores
          if (rowOk) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const long long n = gn0 + j;
              if (n < p.N) {
                float x = v[j];
                if (p.res) x += loadAs(p.res, rRow + n * p.r_sn, p.res_dtype);
                v[j] = applyAct(x, p.act);
              }
            }
          }
          if (tma) {
            if (outF32) {
#pragma unroll
              for (int un = 0; un < 2; ++un) {
                if (gn0 + un * 16 < p.N) { acquireSlot(); stageF32(v + un * 16); storeUnit(gn0 + un * 16); }
              }
            } else {
              acquireSlot(); stageBf16(v); storeUnit(gn0);
            }
          } else if (rowOk) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (gn0 + j < p.N) storeAs(p.out, oRow + gn0 + j, p.out_dtype, v[j]);
          }
        }
      }
    }
    if (tma && lane == 0) bulkWaitRead();   // shared memory stays valid until the last store has read it
  } else if (CONV && warp < kGatherWarp0 + kGatherWarps) {
    // ---------------------------------------------------------------- im2col gather of A (convolution)
    // 256 threads; thread g owns 16-byte chunk (g & 7) of tile rows (g >> 3) + 32*j, j = 0..3, so that
    // eight neighbouring lanes fetch one row's 128 contiguous bytes.  A chunk never straddles a filter
    // tap (C * element size is a multiple of 16), so it is one load from x[n, ih, iw, c..] or zeros.
    // The tap of a chunk depends only on the K block, not on the row: it is tracked incrementally.
    constexpr int kChunkElems = 16 / kElemBytes;
    const int g = threadIdx.x - kGatherWarp0 * 32;
    const int chunk = g & 7, row0 = g >> 3;
    const char* X = reinterpret_cast<const char*>(p.x);
    const uint32_t dstOff = (uint32_t)(row0 * 128 + ((chunk ^ (row0 & 7)) << 4));   // (row0 + 32 j) & 7 == row0 & 7
    const int tapsPerBlock = (p.C <= BK && BK % p.C == 0) ? BK / p.C : 0;          // whole taps per K block
    uint32_t it = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < p.tiles && ok; t += gridDim.x) {      // (the gathered form is never split along K)
      const int rem = (int)(t % tilesPerBatch);
      const int tileM = rem / p.nTiles;
      long long rowBase[4]; int ih0[4], iw0[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long gm = (long long)tileM * BM + row0 + 32 * j;
        if (gm < p.M) {
          const int ow = (int)(gm % p.OW); const long long t2 = gm / p.OW; const int oh = (int)(t2 % p.OH); const long long img = t2 / p.OH;
          ih0[j] = oh * p.sh - p.ph; iw0[j] = ow * p.sw - p.pw;
          rowBase[j] = img * p.xs_n + (long long)ih0[j] * p.xs_h + (long long)iw0[j] * p.xs_w;
        } else { ih0[j] = -(1 << 28); iw0[j] = 0; rowBase[j] = 0; }   // never in range: the row is zero-filled
      }
      int tapR = 0, tapS = 0, cc = chunk * kChunkElems;       // filter tap and channel of this thread's chunk
      while (cc >= p.C) { cc -= p.C; if (++tapS == p.KW) { tapS = 0; ++tapR; } }
      for (int kb = 0; kb < p.kBlocks; ++kb, ++it) {
        const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
        if (!mbarWait(&empty[s], ph ^ 1, abortWord)) { atomicExch(&g_tcStatus, 5); ok = false; break; }
        const int dIh = tapR * p.dh, dIw = tapS * p.dw;
        const long long tapOff = (long long)dIh * p.xs_h + (long long)dIw * p.xs_w + cc;
        const bool tapOk = tapR < p.KH;                        // past the last tap: K tail, zero-filled
        const uint32_t dst = smemAddr(stageA(s)) + dstOff;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool valid = tapOk && (unsigned)(ih0[j] + dIh) < (unsigned)p.H && (unsigned)(iw0[j] + dIw) < (unsigned)p.W;
          cpAsync16(dst + j * 32 * 128, X + (valid ? (rowBase[j] + tapOff) * kElemBytes : 0), valid);
        }
        cpAsyncArriveOn(&full[s]);                           // arrives when the four copies above have landed
        // next K block: 128 bytes further along K.  Narrow channel counts (the padded stem) step over several taps at once.
        if (tapsPerBlock > 0) { tapS += tapsPerBlock; while (tapS >= p.KW) { tapS -= p.KW; ++tapR; } }
        else { cc += BK; while (cc >= p.C) { cc -= p.C; if (++tapS == p.KW) { tapS = 0; ++tapR; } } }
      }
    }
    cpAsyncCommit();
    cpAsyncWait<0>();                                          // nothing of this thread is in flight at exit
  } else if (X3 && warp >= kSplitWarp0) {
    // ---------------------------------------------------------------- low-order tiles (tf32x3)
    // elementwise, so every 16-byte chunk keeps its swizzled position
    const int et = threadIdx.x - kSplitWarp0 * 32;
    uint32_t it = 0;
    bool ok = true;
    for (long long u = blockIdx.x; u < units && ok; u += gridDim.x) {
      long long t; int kb0, kb1; sliceOf(u, t, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
        if (!mbarWait(&full[s], ph, abortWord)) { atomicExch(&g_tcStatus, 3); ok = false; break; }
        const float4* srcA = reinterpret_cast<const float4*>(stageA(s)); float4* dstA = reinterpret_cast<float4*>(stageALo(s));
        const float4* srcB = reinterpret_cast<const float4*>(stageB(s)); float4* dstB = reinterpret_cast<float4*>(stageBLo(s));
        auto lo = [](float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); };
#pragma unroll 4
        for (int i = et; i < S::kABytes / 16; i += 128) { float4 v = srcA[i]; dstA[i] = make_float4(lo(v.x), lo(v.y), lo(v.z), lo(v.w)); }
        if (!p.hasBLo) {
#pragma unroll 4
          for (int i = et; i < S::kBBytes / 16; i += 128) { float4 v = srcB[i]; dstB[i] = make_float4(lo(v.x), lo(v.y), lo(v.z), lo(v.w)); }
        }
        fenceProxyAsync();
        __syncwarp();
        if (lane == 0) mbarArrive(&split[s]);
      }
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) { tcFenceAfter(); tmemDealloc(tmemBase, kAccCols); }
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

// K-major operand [b0, b1, rows, K] with unit stride along K -> 4-D tensor map, box = 128 bytes of K x boxRows rows.
bool makeMap(CUtensorMap* map, const void* base, bool f32, long long K, long long rows, long long b1, long long b0, long long sRow, long long s1,
             long long s0, int boxRows) {
  EncodeTiledFn enc = encodeTiled();
  if (!enc) return false;
  const int eb = f32 ? 4 : 2;
  // a broadcast batch dim (stride 0) or a unit extent becomes extent 1 with any legal stride
  const bool has1 = b1 > 1 && s1 > 0, has0 = b0 > 1 && s0 > 0;
  const long long dense = sRow * rows;
  cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)(has1 ? b1 : 1), (cuuint64_t)(has0 ? b0 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)(sRow * eb), (cuuint64_t)((has1 ? s1 : dense) * eb), (cuuint64_t)((has0 ? s0 : dense) * eb)};
  cuuint32_t box[4] = {(cuuint32_t)(kTileKBytes / eb), (cuuint32_t)boxRows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeIm2colFn encodeIm2col() {
  static EncodeIm2colFn fn = []() -> EncodeIm2colFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeIm2colFn>(p);
  }();
  return fn;
}

// NHWC activations -> im2col tensor map: a load brings 128 output positions x 128 bytes of channels for one filter tap.
// The bounding box is the set of input pixels that sit under tap (0, 0) of some output position: it starts `pad` pixels
// before the image and ends (kernel extent - 1 - pad) pixels before its end; the traversal strides are the convolution's.
bool makeIm2colMap(CUtensorMap* map, const LlcConvParams* p, bool f32) {
  EncodeIm2colFn enc = encodeIm2col();
  if (!enc) return false;
  const int eb = f32 ? 4 : 2;
  cuuint64_t dims[4] = {(cuuint64_t)p->c, (cuuint64_t)p->w_in, (cuuint64_t)p->h, (cuuint64_t)p->n};
  const bool dense = p->x_sn == 0 && p->x_sh == 0 && p->x_sw == 0;
  cuuint64_t strides[3] = {(cuuint64_t)((dense ? p->c : p->x_sw) * eb), (cuuint64_t)((dense ? p->w_in * p->c : p->x_sh) * eb),
                           (cuuint64_t)((dense ? p->h * p->w_in * p->c : p->x_sn) * eb)};
  int lower[2] = {-p->pad_w, -p->pad_h};
  int upper[2] = {p->pad_w - (int)(p->kw - 1) * p->dil_w, p->pad_h - (int)(p->kh - 1) * p->dil_h};
  cuuint32_t estr[4] = {1, (cuuint32_t)p->stride_w, (cuuint32_t)p->stride_h, 1};
  CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(p->x), dims, strides, lower, upper,
                   (cuuint32_t)(kTileKBytes / eb), (cuuint32_t)BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
// Whether the im2col load can serve this convolution: a K block inside one tap, corners and tap offsets inside the
// ranges the 4-D descriptor and instruction encode, and the output extents exactly those the bounding box yields.
bool im2colEligible(const LlcConvParams* p, bool f32) {
  const int eb = f32 ? 4 : 2;
  static const bool off = []() { const char* e = getenv("LLC_TC_CONV_GATHER"); return e && e[0] == '1'; }();
  if (off || (p->c * eb) % kTileKBytes != 0) return false;
  const int lowW = -p->pad_w, lowH = -p->pad_h;
  const int upW = p->pad_w - (int)(p->kw - 1) * p->dil_w, upH = p->pad_h - (int)(p->kh - 1) * p->dil_h;
  auto in8 = [](int v) { return v >= -128 && v <= 127; };
  if (!in8(lowW) || !in8(lowH) || !in8(upW) || !in8(upH)) return false;
  if ((p->kw - 1) * p->dil_w > 255 || (p->kh - 1) * p->dil_h > 255) return false;
  if (p->stride_w < 1 || p->stride_w > 8 || p->stride_h < 1 || p->stride_h > 8) return false;
  const long long extW = p->w_in + upW - lowW, extH = p->h + upH - lowH;     // base positions per row / column
  if (extW < 1 || extH < 1) return false;
  if ((extW - 1) / p->stride_w + 1 != p->ow || (extH - 1) / p->stride_h + 1 != p->oh) return false;
  if (p->n * p->oh * p->ow > (1LL << 31)) return false;
  return encodeIm2col() != nullptr;
}

// MN-major operand [b0, b1, K, N] with unit stride along N -> 4-D tensor map, box = 128 bytes of N x boxK rows of K.
bool makeMapMn(CUtensorMap* map, const void* base, bool f32, long long N, long long K, long long b1, long long b0, long long sK, long long s1,
               long long s0, int boxK) {
  EncodeTiledFn enc = encodeTiled();
  if (!enc) return false;
  const int eb = f32 ? 4 : 2;
  const bool has1 = b1 > 1 && s1 > 0, has0 = b0 > 1 && s0 > 0;
  const long long dense = sK * K;
  cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)K, (cuuint64_t)(has1 ? b1 : 1), (cuuint64_t)(has0 ? b0 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)(sK * eb), (cuuint64_t)((has1 ? s1 : dense) * eb), (cuuint64_t)((has0 ? s0 : dense) * eb)};
  cuuint32_t box[4] = {(cuuint32_t)(kTileKBytes / eb), (cuuint32_t)boxK, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Output [b0, b1, M, N] with unit stride along N -> 4-D tensor map for the epilogue's stores; box = rowBytes of N x 32 rows,
// swizzle span = rowBytes (64 or 128).  Returns false when the layout cannot be described (the epilogue then stores directly).
bool makeOutMap(CUtensorMap* map, void* base, bool f32, long long N, long long M, long long b1, long long b0, long long sRow, long long s1,
                long long s0, int rowBytes) {
  EncodeTiledFn enc = encodeTiled();
  if (!enc) return false;
  const int eb = f32 ? 4 : 2;
  const bool has1 = b1 > 1, has0 = b0 > 1;
  auto ok16 = [&](long long s) { return s > 0 && (s * eb) % 16 == 0; };
  if ((reinterpret_cast<uintptr_t>(base) & 15) || !ok16(sRow) || sRow < N || (has1 && !ok16(s1)) || (has0 && !ok16(s0))) return false;
  if (N > (1LL << 31) || M > (1LL << 31)) return false;
  const long long dense = sRow * M;
  cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)(has1 ? b1 : 1), (cuuint64_t)(has0 ? b0 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)(sRow * eb), (cuuint64_t)((has1 ? s1 : dense) * eb), (cuuint64_t)((has0 ? s0 : dense) * eb)};
  cuuint32_t box[4] = {(cuuint32_t)(rowBytes / eb), 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, rowBytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
// Residual [b0, b1, M, N] (unit stride along N, batch dims possibly broadcast) -> the same 64-byte x 32-row boxes as the
// output map, for the ring of TMA loads in the RES kernels.  `has1` / `has0` tell whether the batch coordinates apply.
bool makeResMap(CUtensorMap* map, const void* base, bool f32, long long N, long long M, long long b1, long long b0, long long sRow, long long s1,
                long long s0, bool* has1Out, bool* has0Out) {
  EncodeTiledFn enc = encodeTiled();
  if (!enc) return false;
  const int eb = f32 ? 4 : 2;
  const bool has1 = b1 > 1 && s1 > 0, has0 = b0 > 1 && s0 > 0;
  auto ok16 = [&](long long s) { return s > 0 && (s * eb) % 16 == 0; };
  if ((reinterpret_cast<uintptr_t>(base) & 15) || !ok16(sRow) || sRow < N || (has1 && !ok16(s1)) || (has0 && !ok16(s0))) return false;
  if ((b1 > 1 && s1 < 0) || (b0 > 1 && s0 < 0) || N > (1LL << 31) || M > (1LL << 31)) return false;
  const long long dense = sRow * M;
  cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)(has1 ? b1 : 1), (cuuint64_t)(has0 ? b0 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)(sRow * eb), (cuuint64_t)((has1 ? s1 : dense) * eb), (cuuint64_t)((has0 ? s0 : dense) * eb)};
  cuuint32_t box[4] = {(cuuint32_t)(64 / eb), 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  *has1Out = has1; *has0Out = has0;
  return enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// LLC_TC_RES_RING=0 keeps residuals on the register path (used to compare the two).
bool resRingEnabled() {
  static const bool on = []() { const char* e = getenv("LLC_TC_RES_RING"); return !(e && e[0] == '0'); }();
  return on;
}
// Bytes per row of the output box the epilogue stages and stores: 32 bf16 or 16 fp32 columns.
constexpr int kOutBoxBytes = 64;

int numSMs() { return deviceSMs(); }

// LLC_TC_SPLITK=0 keeps every K loop in one piece (2 is accepted and means the default: split wherever SMs would idle).
int splitKMode() {
  const char* e = getenv("LLC_TC_SPLITK");
  return e && *e ? atoi(e) : 1;
}
bool splitKEnabled() { return splitKMode() != 0; }

// LLC_TC_DIRECT_STORES=1 keeps the epilogue on direct global stores (used to compare the two paths).
bool tmaEpilogueEnabled() {
  static const bool on = []() { const char* e = getenv("LLC_TC_DIRECT_STORES"); return !(e && e[0] == '1'); }();
  return on;
}

template <int BN, int KIND, int MODE, bool BMN, bool RES>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mbl, const CUtensorMap& mr, TcArgs a, long long batch, cudaStream_t st) {
  using S = Smem<BN, KIND == 2, RES>;
  static_assert(S::kStages >= 2, "at least two pipeline stages");
  static DeviceOnce configured;                          // the shared-memory opt-in is kept per device
  const int dev = currentDevice();
  if (!configured.test(dev)) {
    cudaError_t e = cudaFuncSetAttribute(tc_kernel<BN, KIND, MODE, BMN, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return cudaFail(e, "cudaFuncSetAttribute(tc_kernel)");
    configured.set(dev);
  }
  a.mTiles = (int)((a.M + BM - 1) / BM); a.nTiles = (int)((a.N + BN - 1) / BN);
  a.tiles = (long long)a.mTiles * a.nTiles * batch;
  if (a.splits < 1 || RES) a.splits = 1;
  const int threads = tcThreads(KIND, MODE);
  const long long units = a.tiles * a.splits;
  const unsigned grid = (unsigned)(units < numSMs() ? units : numSMs());
  tc_kernel<BN, KIND, MODE, BMN, RES><<<grid, threads, S::kTotal, st>>>(ma, mb, mo, mbl, mr, a);
  LLC_LAUNCH_CHECK("tc_kernel");
  return LLC_OK;
}

// `res`: the kernel variant whose epilogue fetches the residual through a ring of TMA loads (bf16 / tf32, TMA-fed operands).
template <int MODE, bool BMN>
int dispatch(int bn, int kind, bool res, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mbl, const CUtensorMap& mr,
             const TcArgs& a, long long batch, cudaStream_t st) {
#define TC_CASE(BN_, K_) if (bn == BN_ && kind == K_ && !res) return launch<BN_, K_, MODE, BMN, false>(ma, mb, mo, mbl, mr, a, batch, st);
#define TC_CASE_RES(BN_, K_) if (bn == BN_ && kind == K_ && res) return launch<BN_, K_, MODE, BMN, true>(ma, mb, mo, mbl, mr, a, batch, st);
  TC_CASE(64, 0) TC_CASE(128, 0)
  if constexpr (!BMN) { TC_CASE(64, 1) TC_CASE(64, 2) TC_CASE(128, 1) TC_CASE(128, 2) TC_CASE(256, 0) TC_CASE(256, 1) }
  if constexpr (!BMN && MODE != 1) { TC_CASE_RES(64, 0) TC_CASE_RES(128, 0) TC_CASE_RES(256, 0) TC_CASE_RES(64, 1) TC_CASE_RES(128, 1) TC_CASE_RES(256, 1) }
#undef TC_CASE
#undef TC_CASE_RES
  return setError(LLC_ERR_INTERNAL, "llc internal: no tensor-core kernel for this tile");
}

// Tile width by a cost model: a persistent CTA works through ceil(tiles / SMs) tiles, and a tile costs the longer of its
// main loop (K blocks x a per-block time that grows slowly with the width, because narrow tiles are bound by operand
// traffic and latency rather than by the tensor pipe) and its epilogue.  Times in microseconds, measured on B200.
struct TilePlan { int bn; int splits; };
// `wsBytes` > 0 allows split-K: when the tiles of a width leave at least half of the SMs idle and the K loop is long, K
// is cut into slices that run side by side (every unit resident at once) and meet in the workspace.
TilePlan chooseTile(long long M, long long N, long long batch, bool allow256, int kind, int kBlocks, long long wsBytes) {
  static const float kBlockUs[3][3] = {{0.22f, 0.25f, 0.40f}, {0.28f, 0.33f, 0.50f}, {0.60f, 0.75f, 0.f}};   // [kind][width]
  static const float epilogueUs[3] = {0.8f, 1.2f, 2.0f};
  const long long mT = (M + BM - 1) / BM;
  TilePlan best{64, 1}; float bestCost = 0.f;
  for (int i = 0; i < 3; ++i) {
    const int bn = 64 << i;
    if (bn == 256 && (!allow256 || kind == 2)) continue;
    if (i > 0 && N <= bn / 2) continue;                    // at least half of the tile's columns exist
    const long long tiles = mT * ((N + bn - 1) / bn) * batch;
    int splits = 1;
    if (wsBytes > 0 && tiles * 2 <= numSMs() && kBlocks >= 8) {
      splits = (int)(numSMs() / tiles);
      if (splits > 4) splits = 4;
      // a slice keeps at least four K blocks.  With the parked tiles laid out for 512-byte warp accesses, splitting
      // whenever half of the SMs would idle measured equal or faster on every workload (encoder 128: 0.153 against
      // 0.162 ms, ResNet-18 1.185 against 1.298 ms without split-K), so there is no minimum slice time any more.
      while (splits > 1 && (kBlocks / splits < 4 || 4096 + tiles * splits * (long long)BM * bn * 4 > wsBytes)) --splits;
    }
    const long long rounds = (tiles * splits + numSMs() - 1) / numSMs();
    const float loop = ((kBlocks + splits - 1) / splits) * kBlockUs[kind][i];
    const float cost = (float)rounds * ((loop > epilogueUs[i] ? loop : epilogueUs[i]) + 0.3f) + (splits > 1 ? 10.0f : 0.f);
    if (i == 0 || cost <= bestCost) { best = TilePlan{bn, splits}; bestCost = cost; }
  }
  return best;
}

}  // namespace

// Whether the tensor-core kernel takes this call (otherwise the FMA kernel does).
bool tcGemmSupported(const LlcGemmParams* p) {
  const bool f32 = p->in_dtype == LLC_FLOAT32;
  if (!f32 && p->in_dtype != LLC_BFLOAT16) return false;
  if (f32 && p->precision != LLC_PREC_TF32 && p->precision != LLC_PREC_TF32X3) return false;
  const bool bmn = p->b_sk != 1;                        // B stored [k][n]
  if (bmn && p->b_sn != 1) return false;
  if (bmn && f32) return false;                         // 32-bit operands are taken K-major only (an MN-major tf32 B produced zeros on B200)
  const int eb = f32 ? 4 : 2;
  auto ok16 = [&](long long s) { return (s * eb) % 16 == 0; };
  if (!ok16(p->a_sm) || !ok16(p->a_s0) || !ok16(p->a_s1) || !ok16(bmn ? p->b_sk : p->b_sn) || !ok16(p->b_s0) || !ok16(p->b_s1)) return false;
  if (p->a_sm < p->k || (bmn ? p->b_sk < p->n : p->b_sn < p->k)) return false;   // overlapping rows are not expressible as a tensor map
  if (p->a_s0 < 0 || p->a_s1 < 0 || p->b_s0 < 0 || p->b_s1 < 0) return false;
  if ((reinterpret_cast<uintptr_t>(p->a) | reinterpret_cast<uintptr_t>(p->b)) & 15) return false;
  if (p->m < 1 || p->n < 1 || p->k < 1) return false;
  if (p->b0 > (1 << 30) || p->b1 > (1 << 30) || p->m > (1LL << 31) * 64 || p->n > (1LL << 31)) return false;
  // tiny problems: the FMA kernel has less fixed cost.  For 32-bit operands the break-even measured near 2^25
  // multiply-adds (64x512x784 took 20 us on either kernel, 64x10x512 19 us against 27 us); LLC_TC_MIN_MACS_LOG2 moves it.
  const char* minEnv = getenv("LLC_TC_MIN_MACS_LOG2");
  int minLog2F32 = minEnv && *minEnv ? atoi(minEnv) : 25;
  minLog2F32 = minLog2F32 < 0 ? 0 : (minLog2F32 > 40 ? 40 : minLog2F32);
  const long long macs = p->m * p->n * p->k * (p->b0 > 0 ? p->b0 : 1) * (p->b1 > 0 ? p->b1 : 1);
  if (p->m * p->n * p->k < (1LL << 18) || (f32 && macs < (1LL << minLog2F32))) return false;
  return encodeTiled() != nullptr;
}

int tcGemm(const LlcGemmParams* p, cudaStream_t st) {
  const bool f32 = p->in_dtype == LLC_FLOAT32;
  const int eb = f32 ? 4 : 2;
  const int bk = kTileKBytes / eb;
  const long long batch = p->b0 * p->b1;
  const bool bmn = p->b_sk != 1;
  const int kind = !f32 ? 0 : (p->precision == LLC_PREC_TF32X3 ? 2 : 1);
  const bool wsOk = p->workspace && (reinterpret_cast<uintptr_t>(p->workspace) & 15) == 0 && !bmn && splitKEnabled();
  const TilePlan plan = chooseTile(p->m, p->n, batch, !bmn, kind, (int)((p->k + bk - 1) / bk), wsOk ? p->workspace_bytes : 0);
  const int bn = plan.bn;
  CUtensorMap ma, mb;
  bool okMaps = makeMap(&ma, p->a, f32, p->k, p->m, p->b1, p->b0, p->a_sm, p->a_s1, p->a_s0, BM);
  okMaps = okMaps && (bmn ? makeMapMn(&mb, p->b, f32, p->n, p->k, p->b1, p->b0, p->b_sk, p->b_s1, p->b_s0, bk)
                          : makeMap(&mb, p->b, f32, p->k, p->n, p->b1, p->b0, p->b_sn, p->b_s1, p->b_s0, bn));
  if (!okMaps) return setError(LLC_ERR_CUDA, "llc cuda: cuTensorMapEncodeTiled rejected the GEMM operands");
  TcArgs a{};
  a.out = p->out; a.scale = p->scale; a.shift = p->shift; a.res = p->res;
  a.out_dtype = p->out_dtype; a.res_dtype = p->res_dtype; a.act = p->act; a.alpha = p->alpha;
  a.M = p->m; a.N = p->n; a.K = p->k;
  a.o_s0 = p->o_s0; a.o_s1 = p->o_s1; a.o_sm = p->o_sm; a.r_s0 = p->r_s0; a.r_s1 = p->r_s1; a.r_sm = p->r_sm; a.r_sn = p->r_sn;
  a.b1 = (int)p->b1; a.kBlocks = (int)((p->k + bk - 1) / bk);
  a.splits = plan.splits; a.counters = reinterpret_cast<int*>(p->workspace); a.ws = reinterpret_cast<float*>(reinterpret_cast<char*>(p->workspace) + 4096);
  a.aZ0 = p->b0 > 1 && p->a_s0 > 0; a.aZ1 = p->b1 > 1 && p->a_s1 > 0; a.bZ0 = p->b0 > 1 && p->b_s0 > 0; a.bZ1 = p->b1 > 1 && p->b_s1 > 0;
  const int ob = p->out_dtype == LLC_FLOAT32 ? 4 : 2;
  a.vecOut = (reinterpret_cast<uintptr_t>(p->out) % (ob * 4)) == 0 && p->o_sm % 4 == 0 && p->o_s0 % 4 == 0 && p->o_s1 % 4 == 0 &&
             ((reinterpret_cast<uintptr_t>(p->scale) | reinterpret_cast<uintptr_t>(p->shift)) & 15) == 0;
  CUtensorMap mo = ma;   // a valid map even when unused
  if (tmaEpilogueEnabled() && makeOutMap(&mo, p->out, ob == 4, p->n, p->m, p->b1, p->b0, p->o_sm, p->o_s1, p->o_s0, kOutBoxBytes)) a.tmaOut = kOutBoxBytes;
  auto r16 = [&](long long st) { return st >= 0 && (st * ob) % 16 == 0; };
  a.resTile = p->res && p->r_sn == 1 && p->res_dtype == p->out_dtype && (reinterpret_cast<uintptr_t>(p->res) & 15) == 0 && r16(p->r_sm) && r16(p->r_s0) &&
              r16(p->r_s1) && p->n % (16 / ob) == 0;
  CUtensorMap mbl = mb;
  if (kind == 2 && !bmn && p->b_lo && (reinterpret_cast<uintptr_t>(p->b_lo) & 15) == 0 &&
      makeMap(&mbl, p->b_lo, f32, p->k, p->n, p->b1, p->b0, p->b_sn, p->b_s1, p->b_s0, bn))
    a.hasBLo = 1;
  // the residual through a ring of TMA loads: whole tiles only (no split-K), same element type as the output
  CUtensorMap mr = mo;
  bool resRing = false;
  if (a.resTile && a.tmaOut && plan.splits == 1 && kind != 2 && !bmn && resRingEnabled()) {
    bool h1 = false, h0 = false;
    if (makeResMap(&mr, p->res, ob == 4, p->n, p->m, p->b1, p->b0, p->r_sm, p->r_s1, p->r_s0, &h1, &h0)) { resRing = true; a.rZ1 = h1; a.rZ0 = h0; }
  }
  return bmn ? dispatch<0, true>(bn, kind, false, ma, mb, mo, mbl, mr, a, batch, st) : dispatch<0, false>(bn, kind, resRing, ma, mb, mo, mbl, mr, a, batch, st);
}

bool tcConvSupported(const LlcConvParams* p) {
  const bool f32 = p->in_dtype == LLC_FLOAT32;
  if (!f32 && p->in_dtype != LLC_BFLOAT16) return false;
  if (f32 && p->precision != LLC_PREC_TF32 && p->precision != LLC_PREC_TF32X3) return false;
  const int eb = f32 ? 4 : 2;
  if ((p->c * eb) % 16 != 0) return false;              // a 16-byte chunk must stay inside one filter tap
  if ((p->x_sn * eb) % 16 != 0 || (p->x_sh * eb) % 16 != 0 || (p->x_sw * eb) % 16 != 0 || p->x_sn < 0 || p->x_sh < 0 || p->x_sw < 0) return false;
  if ((reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->w)) & 15) return false;
  const long long M = p->n * p->oh * p->ow, K = p->kh * p->kw * p->c;
  if (M * p->f * K < (1LL << 18)) return false;
  return encodeTiled() != nullptr;
}

int tcConv(const LlcConvParams* p, cudaStream_t st) {
  const bool f32 = p->in_dtype == LLC_FLOAT32;
  const int eb = f32 ? 4 : 2;
  const int bk = kTileKBytes / eb;
  const long long M = p->n * p->oh * p->ow, K = p->kh * p->kw * p->c;
  const int kind = !f32 ? 0 : (p->precision == LLC_PREC_TF32X3 ? 2 : 1);
  const bool wsOk = p->workspace && (reinterpret_cast<uintptr_t>(p->workspace) & 15) == 0 && im2colEligible(p, f32) && splitKEnabled();
  const TilePlan plan = chooseTile(M, p->f, 1, true, kind, (int)((K + bk - 1) / bk), wsOk ? p->workspace_bytes : 0);
  const int bn = plan.bn;
  CUtensorMap mb;
  if (!makeMap(&mb, p->w, f32, K, p->f, 1, 1, K, 0, 0, bn))
    return setError(LLC_ERR_CUDA, "llc cuda: cuTensorMapEncodeTiled rejected the convolution weights");
  TcArgs a{};
  a.out = p->out; a.scale = p->scale; a.shift = p->shift; a.res = p->res;
  a.out_dtype = p->out_dtype; a.res_dtype = p->res_dtype; a.act = p->act; a.alpha = p->alpha;
  a.M = M; a.N = p->f; a.K = K; a.o_sm = p->f; a.r_sm = p->f; a.r_sn = 1; a.b1 = 1;
  a.kBlocks = (int)((K + bk - 1) / bk);
  a.splits = plan.splits; a.counters = reinterpret_cast<int*>(p->workspace); a.ws = reinterpret_cast<float*>(reinterpret_cast<char*>(p->workspace) + 4096);
  const int ob = p->out_dtype == LLC_FLOAT32 ? 4 : 2;
  a.vecOut = (reinterpret_cast<uintptr_t>(p->out) % (ob * 4)) == 0 && p->f % 4 == 0 &&
             ((reinterpret_cast<uintptr_t>(p->scale) | reinterpret_cast<uintptr_t>(p->shift)) & 15) == 0;
  a.x = p->x; a.H = (int)p->h; a.W = (int)p->w_in; a.C = (int)p->c; a.KH = (int)p->kh; a.KW = (int)p->kw; a.OH = (int)p->oh; a.OW = (int)p->ow;
  a.sh = p->stride_h; a.sw = p->stride_w; a.ph = p->pad_h; a.pw = p->pad_w; a.dh = p->dil_h; a.dw = p->dil_w;
  {
    const bool dense = p->x_sn == 0 && p->x_sh == 0 && p->x_sw == 0;
    a.xs_w = dense ? p->c : p->x_sw; a.xs_h = dense ? p->w_in * p->c : p->x_sh; a.xs_n = dense ? p->h * p->w_in * p->c : p->x_sn;
  }
  CUtensorMap mo = mb;
  if (tmaEpilogueEnabled() && makeOutMap(&mo, p->out, ob == 4, p->f, M, 1, 1, p->f, 0, 0, kOutBoxBytes)) a.tmaOut = kOutBoxBytes;
  a.resTile = p->res && p->res_dtype == p->out_dtype && (reinterpret_cast<uintptr_t>(p->res) & 15) == 0 && (p->f * ob) % 16 == 0;
  CUtensorMap mbl = mb;
  if (kind == 2 && p->w_lo && (reinterpret_cast<uintptr_t>(p->w_lo) & 15) == 0 && makeMap(&mbl, p->w_lo, f32, K, p->f, 1, 1, K, 0, 0, bn)) a.hasBLo = 1;
  if (im2colEligible(p, f32)) {
    CUtensorMap ma;
    if (makeIm2colMap(&ma, p, f32)) {
      CUtensorMap mr = mo;
      bool resRing = false;
      if (a.resTile && a.tmaOut && plan.splits == 1 && kind != 2 && resRingEnabled()) {
        bool h1 = false, h0 = false;
        if (makeResMap(&mr, p->res, ob == 4, p->f, M, 1, 1, p->f, 0, 0, &h1, &h0)) resRing = true;
      }
      return dispatch<2, false>(bn, kind, resRing, ma, mb, mo, mbl, mr, a, 1, st);
    }
  }
  a.splits = 1;                                          // the gathered form walks whole tiles
  return dispatch<1, false>(bn, kind, false, mb, mb, mo, mbl, mo, a, 1, st);
}

// Device address of the status word on the current device (for callers that copy it back on their own stream).
int* tcStatusAddress() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_tcStatus) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}

// Reads and clears the status word the bounded waits write (0 = no wait ever gave up).
int tcStatus() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tcStatus, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_tcStatus, &zero, sizeof(int));
  return v;
}

}  // namespace llc

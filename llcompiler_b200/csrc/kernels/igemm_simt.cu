// FMA (CUDA-core) implicit-GEMM kernel: dense / batched GEMM and NHWC convolution share one
// main loop and one fused epilogue.  This is the fp32-exact path (precision "fp32") and the
// fallback for shapes the tensor-core kernels do not take.
//
// Tiling: BM x BN output tile per 256-thread CTA, BK = 16, register tile (BM/16) x (BN/16)
// per thread, double-buffered shared memory filled through registers so that global loads of
// tile t+1 overlap the FMAs of tile t.  Operands are stored k-major in shared memory
// (As[k][m], Bs[k][n]) so that each thread reads its m/n fragments as float4.
// Bound: fp32 FMA throughput (148 SMs x 128 lanes x 2 flop x clock); HBM traffic is
// M*K + N*K + M*N elements per call plus re-reads of A across the N/BN column tiles (L2 hits).
#include <mutex>

#include "common.cuh"

namespace llc {
namespace {

struct IgemmArgs {
  const void* a; const void* b; void* out; const float* scale; const float* shift; const void* res;
  int out_dtype, res_dtype, act; float alpha;
  long long M, N, K;
  long long a_s0, a_s1, a_sm, b_s0, b_s1, b_sk, b_sn, o_s0, o_s1, o_sm, r_s0, r_s1, r_sm, r_sn;
  int b1; int vecOut;
  int H, W, C, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
  // split-K: grid.z = batch * splitK; CTA kz reduces K range [kz*kPer, (kz+1)*kPer) into `partial`,
  // the last CTA to arrive at a tile (counted in `counters`) sums the partials in kz order and
  // runs the epilogue, then puts the counter back to zero.
  int splitK; long long kPer; float* partial; unsigned* counters;
};

constexpr int BK = 16;

template <typename T, int BM, int BN, bool CONV, bool VEC>
__global__ void __launch_bounds__(256) igemm_simt_kernel(IgemmArgs p) {
  constexpr int TM = BM / 16, TN = BN / 16;
  constexpr int AV = BM / 64, BV = BN / 64;        // float4 loads per thread per tile (VEC)
  constexpr int AS = BM / 16, BS = BN / 16;        // scalar loads per thread per tile (!VEC)
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const long long m0 = (long long)blockIdx.x * BM, n0 = (long long)blockIdx.y * BN;
  const int kz = p.splitK > 1 ? (int)(blockIdx.z % p.splitK) : 0;
  const int z = p.splitK > 1 ? (int)(blockIdx.z / p.splitK) : (int)blockIdx.z, zb0 = z / p.b1, zb1 = z % p.b1;
  const long long kBeg = (long long)kz * p.kPer;
  const long long kEnd = p.splitK > 1 ? (kBeg + p.kPer < p.K ? kBeg + p.kPer : p.K) : p.K;
  const T* A = reinterpret_cast<const T*>(p.a) + (CONV ? 0 : zb0 * p.a_s0 + zb1 * p.a_s1);
  const T* B = reinterpret_cast<const T*>(p.b) + zb0 * p.b_s0 + zb1 * p.b_s1;
  const bool bKMajor = p.b_sk == 1;

  // per-thread row bookkeeping for the A loads
  constexpr int AR = VEC ? AV : AS;
  long long aBase[AR]; int aIh0[AR], aIw0[AR]; bool aOk[AR];
#pragma unroll
  for (int i = 0; i < AR; ++i) {
    int e = tid + i * 256;
    int row = VEC ? (e >> 2) : (e >> 4);
    long long gm = m0 + row;
    aOk[i] = gm < p.M;
    if (CONV) {
      long long mm = aOk[i] ? gm : 0;
      int ow = (int)(mm % p.OW); long long t = mm / p.OW; int oh = (int)(t % p.OH); long long img = t / p.OH;
      aIh0[i] = oh * p.sh - p.ph; aIw0[i] = ow * p.sw - p.pw;
      aBase[i] = img * p.H * p.W * p.C;
    } else {
      aBase[i] = gm * p.a_sm; aIh0[i] = aIw0[i] = 0;
    }
  }

  float4 ra4[VEC ? AV : 1], rb4[VEC ? BV : 1];
  float ras[VEC ? 1 : AS], rbs[VEC ? 1 : BS];

  auto loadTile = [&](long long k0) {
    if (VEC) {
#pragma unroll
      for (int i = 0; i < AV; ++i) {
        int e = tid + i * 256;
        long long kk = k0 + ((e & 3) << 2);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (aOk[i] && kk < kEnd) {
          if (CONV) {
            int tap = (int)(kk / p.C), c = (int)(kk - (long long)tap * p.C);
            int r = tap / p.KW, s = tap - r * p.KW;
            int ih = aIh0[i] + r * p.dh, iw = aIw0[i] + s * p.dw;
            if (ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) v = Vec4<T>::load(A + aBase[i] + ((long long)ih * p.W + iw) * p.C + c);
          } else v = Vec4<T>::load(A + aBase[i] + kk);
        }
        ra4[i] = v;
      }
      if (bKMajor) {
#pragma unroll
        for (int i = 0; i < BV; ++i) {
          int e = tid + i * 256;
          long long gn = n0 + (e >> 2), kk = k0 + ((e & 3) << 2);
          rb4[i] = (gn < p.N && kk < kEnd) ? Vec4<T>::load(B + gn * p.b_sn + kk) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      } else {
#pragma unroll
        for (int i = 0; i < BV; ++i) {
          int e = tid + i * 256;
          int kr = e / (BN / 4); long long gn = n0 + (e % (BN / 4)) * 4, kk = k0 + kr;
          rb4[i] = (gn < p.N && kk < kEnd) ? Vec4<T>::load(B + kk * p.b_sk + gn) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < AS; ++i) {
        int e = tid + i * 256;
        long long kk = k0 + (e & 15);
        float v = 0.f;
        if (aOk[i] && kk < kEnd) {
          if (CONV) {
            int tap = (int)(kk / p.C), c = (int)(kk - (long long)tap * p.C);
            int r = tap / p.KW, s = tap - r * p.KW;
            int ih = aIh0[i] + r * p.dh, iw = aIw0[i] + s * p.dw;
            if (ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) v = toFloat<T>(A[aBase[i] + ((long long)ih * p.W + iw) * p.C + c]);
          } else v = toFloat<T>(A[aBase[i] + kk]);
        }
        ras[i] = v;
      }
#pragma unroll
      for (int i = 0; i < BS; ++i) {
        int e = tid + i * 256;
        long long gn = n0 + (e >> 4), kk = k0 + (e & 15);
        rbs[i] = (gn < p.N && kk < kEnd) ? toFloat<T>(B[gn * p.b_sn + kk * p.b_sk]) : 0.f;
      }
    }
  };
  auto storeTile = [&](int buf) {
    if (VEC) {
#pragma unroll
      for (int i = 0; i < AV; ++i) {
        int e = tid + i * 256, row = e >> 2, kv = (e & 3) << 2;
        As[buf][kv + 0][row] = ra4[i].x; As[buf][kv + 1][row] = ra4[i].y; As[buf][kv + 2][row] = ra4[i].z; As[buf][kv + 3][row] = ra4[i].w;
      }
      if (bKMajor) {
#pragma unroll
        for (int i = 0; i < BV; ++i) {
          int e = tid + i * 256, row = e >> 2, kv = (e & 3) << 2;
          Bs[buf][kv + 0][row] = rb4[i].x; Bs[buf][kv + 1][row] = rb4[i].y; Bs[buf][kv + 2][row] = rb4[i].z; Bs[buf][kv + 3][row] = rb4[i].w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < BV; ++i) {
          int e = tid + i * 256, kr = e / (BN / 4), nv = (e % (BN / 4)) * 4;
          *reinterpret_cast<float4*>(&Bs[buf][kr][nv]) = rb4[i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < AS; ++i) { int e = tid + i * 256; As[buf][e & 15][e >> 4] = ras[i]; }
#pragma unroll
      for (int i = 0; i < BS; ++i) { int e = tid + i * 256; Bs[buf][e & 15][e >> 4] = rbs[i]; }
    }
  };

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const long long nk = (kEnd - kBeg + BK - 1) / BK;
  loadTile(kBeg);
  storeTile(0);
  __syncthreads();
  for (long long kt = 0; kt < nk; ++kt) {
    const int buf = (int)(kt & 1);
    if (kt + 1 < nk) loadTile(kBeg + (kt + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int g = 0; g < TM / 4; ++g) {
        float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][g * 64 + ty * 4]);
        a[g * 4 + 0] = v.x; a[g * 4 + 1] = v.y; a[g * 4 + 2] = v.z; a[g * 4 + 3] = v.w;
      }
#pragma unroll
      for (int g = 0; g < TN / 4; ++g) {
        float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][g * 64 + tx * 4]);
        b[g * 4 + 0] = v.x; b[g * 4 + 1] = v.y; b[g * 4 + 2] = v.z; b[g * 4 + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < nk) storeTile(buf ^ 1);
    __syncthreads();
  }

  if (p.splitK > 1) {
    __shared__ int isLast;
    const long long tileId = ((long long)z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    float* mine = p.partial + (tileId * p.splitK + kz) * (BM * BN);
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int g = 0; g < TN / 4; ++g)
        *reinterpret_cast<float4*>(mine + ((i >> 2) * 64 + ty * 4 + (i & 3)) * BN + g * 64 + tx * 4) =
            make_float4(acc[i][g * 4 + 0], acc[i][g * 4 + 1], acc[i][g * 4 + 2], acc[i][g * 4 + 3]);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      unsigned prev = atomicAdd(&p.counters[tileId], 1u);
      isLast = prev == (unsigned)(p.splitK - 1);
      if (isLast) p.counters[tileId] = 0;       // leave the counter at zero for the next launch
    }
    __syncthreads();
    if (!isLast) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    for (int q = 0; q < p.splitK; ++q) {
      const float* part = p.partial + (tileId * p.splitK + q) * (BM * BN);
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int g = 0; g < TN / 4; ++g) {
          float4 v = __ldcg(reinterpret_cast<const float4*>(part + ((i >> 2) * 64 + ty * 4 + (i & 3)) * BN + g * 64 + tx * 4));
          acc[i][g * 4 + 0] += v.x; acc[i][g * 4 + 1] += v.y; acc[i][g * 4 + 2] += v.z; acc[i][g * 4 + 3] += v.w;
        }
    }
  }

  // fused epilogue: alpha * scale[n] * acc + shift[n] + res, activation, store
  char* outBase = reinterpret_cast<char*>(p.out);
  const long long oOff = CONV ? 0 : zb0 * p.o_s0 + zb1 * p.o_s1;
  const long long rOff = CONV ? 0 : zb0 * p.r_s0 + zb1 * p.r_s1;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    long long gm = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (gm >= p.M) continue;
#pragma unroll
    for (int g = 0; g < TN / 4; ++g) {
      long long gn = n0 + g * 64 + tx * 4;
      if (gn >= p.N) continue;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        long long n = gn + j;
        float x = acc[i][g * 4 + j] * p.alpha;
        if (n < p.N) {
          if (p.scale) x *= p.scale[n];
          if (p.shift) x += p.shift[n];
          if (p.res) x += loadAs(p.res, rOff + gm * p.r_sm + n * p.r_sn, p.res_dtype);
        }
        v[j] = applyAct(x, p.act);
      }
      long long o = oOff + gm * p.o_sm + gn;
      if (p.vecOut && gn + 3 < p.N) {
        if (p.out_dtype == LLC_FLOAT32) Vec4<float>::store(reinterpret_cast<float*>(outBase) + o, make_float4(v[0], v[1], v[2], v[3]));
        else Vec4<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16*>(outBase) + o, make_float4(v[0], v[1], v[2], v[3]));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) if (gn + j < p.N) storeAs(p.out, o + j, p.out_dtype, v[j]);
      }
    }
  }
}

constexpr size_t kCounterBytes = 4096;   // head of the workspace: one counter per output tile

// The split-K decision, in one place for the launcher and for the entry point that has to refuse a shape whose
// split does not fit its fixed scratch.  Few 64 x 64 output tiles and a long reduction: K is cut over the idle SMs.
// `split` == 1 means no split; `need` is the scratch a split takes (tile counters + fp32 partial tiles).
struct SplitKChoice { long long split = 1, kPer = 0; size_t need = 0; };
SplitKChoice chooseSplitK(long long M, long long N, long long K, long long batch) {
  SplitKChoice c;
  const long long t64 = ((M + 63) / 64) * ((N + 63) / 64) * batch;
  if (t64 <= 0 || t64 * 2 > kNumSMs || K < 512 || t64 > (long long)(kCounterBytes / 4)) return c;
  long long want = kNumSMs / t64; if (want > 32) want = 32; if (want > K / 128) want = K / 128;
  if (want < 1) return c;
  const long long kPer = ((K + want - 1) / want + BK - 1) / BK * BK;
  const long long split = (K + kPer - 1) / kPer;
  if (split <= 1 || batch * split > 65535) return c;
  c.split = split; c.kPer = kPer;
  c.need = kCounterBytes + (size_t)t64 * split * 64 * 64 * sizeof(float);
  return c;
}

template <typename T, bool CONV, bool VEC>
int launchTiles(IgemmArgs a, long long batch, cudaStream_t st, void* workspace, long long workspaceBytes) {
  auto tiles = [&](long long bm, long long bn) { return ((a.M + bm - 1) / bm) * ((a.N + bn - 1) / bn) * batch; };
  if (a.M <= 0 || a.N <= 0 || batch <= 0) return LLC_OK;
  if (batch > 65535) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm batch count above 65535");
  a.splitK = 1;
  if (workspace) {                      // splitting needs caller scratch
    const SplitKChoice c = chooseSplitK(a.M, a.N, a.K, batch);
    if (c.split > 1 && c.need <= (size_t)workspaceBytes) {
      a.splitK = (int)c.split; a.kPer = c.kPer;
      a.counters = reinterpret_cast<unsigned*>(workspace);
      a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kCounterBytes);
      dim3 g((unsigned)((a.M + 63) / 64), (unsigned)((a.N + 63) / 64), (unsigned)(batch * c.split));
      igemm_simt_kernel<T, 64, 64, CONV, VEC><<<g, 256, 0, st>>>(a);
      LLC_LAUNCH_CHECK("igemm_simt_kernel(split-K)");
      return LLC_OK;
    }
  }
  // largest tile that still fills the 148 SMs at least ~once
  if (a.N > 64 && tiles(128, 128) >= kNumSMs) {
    dim3 g((unsigned)((a.M + 127) / 128), (unsigned)((a.N + 127) / 128), (unsigned)batch);
    igemm_simt_kernel<T, 128, 128, CONV, VEC><<<g, 256, 0, st>>>(a);
  } else if (tiles(128, 64) >= kNumSMs) {
    dim3 g((unsigned)((a.M + 127) / 128), (unsigned)((a.N + 63) / 64), (unsigned)batch);
    igemm_simt_kernel<T, 128, 64, CONV, VEC><<<g, 256, 0, st>>>(a);
  } else {
    dim3 g((unsigned)((a.M + 63) / 64), (unsigned)((a.N + 63) / 64), (unsigned)batch);
    igemm_simt_kernel<T, 64, 64, CONV, VEC><<<g, 256, 0, st>>>(a);
  }
  LLC_LAUNCH_CHECK("igemm_simt_kernel");
  return LLC_OK;
}

bool aligned(const void* p, int bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

}  // namespace

int igemmSimtGemm(const LlcGemmParams* p, cudaStream_t st, void* workspace, long long workspaceBytes) {
  IgemmArgs a{};
  a.a = p->a; a.b = p->b; a.out = p->out; a.scale = p->scale; a.shift = p->shift; a.res = p->res;
  a.out_dtype = p->out_dtype; a.res_dtype = p->res_dtype; a.act = p->act; a.alpha = p->alpha;
  a.M = p->m; a.N = p->n; a.K = p->k;
  a.a_s0 = p->a_s0; a.a_s1 = p->a_s1; a.a_sm = p->a_sm;
  a.b_s0 = p->b_s0; a.b_s1 = p->b_s1; a.b_sk = p->b_sk; a.b_sn = p->b_sn;
  a.o_s0 = p->o_s0; a.o_s1 = p->o_s1; a.o_sm = p->o_sm;
  a.r_s0 = p->r_s0; a.r_s1 = p->r_s1; a.r_sm = p->r_sm; a.r_sn = p->r_sn;
  a.b1 = (int)p->b1;
  if (p->b_sk != 1 && p->b_sn != 1) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm B needs unit stride along k or n");
  const int eb = p->in_dtype == LLC_FLOAT32 ? 4 : 2, ob = p->out_dtype == LLC_FLOAT32 ? 4 : 2;
  a.vecOut = aligned(p->out, ob * 4) && p->o_sm % 4 == 0 && p->o_s0 % 4 == 0 && p->o_s1 % 4 == 0;
  bool vec = p->k % 4 == 0 && p->a_sm % 4 == 0 && p->a_s0 % 4 == 0 && p->a_s1 % 4 == 0 && aligned(p->a, eb * 4) && aligned(p->b, eb * 4) &&
             p->b_s0 % 4 == 0 && p->b_s1 % 4 == 0 &&
             (p->b_sk == 1 ? p->b_sn % 4 == 0 : (p->n % 4 == 0 && p->b_sk % 4 == 0));
  long long batch = p->b0 * p->b1;
  void* ws = workspace; long long wsb = workspaceBytes;
  if (ws && (reinterpret_cast<uintptr_t>(ws) & 15)) ws = nullptr;
  if (p->in_dtype == LLC_FLOAT32) return vec ? launchTiles<float, false, true>(a, batch, st, ws, wsb) : launchTiles<float, false, false>(a, batch, st, ws, wsb);
  if (p->in_dtype == LLC_BFLOAT16) return vec ? launchTiles<__nv_bfloat16, false, true>(a, batch, st, ws, wsb) : launchTiles<__nv_bfloat16, false, false>(a, batch, st, ws, wsb);
  return setError(LLC_ERR_UNSUPPORTED, "llc argument: gemm input type must be f32 or bf16");
}

int igemmSimtConv(const LlcConvParams* p, cudaStream_t st) {
  IgemmArgs a{};
  a.a = p->x; a.b = p->w; a.out = p->out; a.scale = p->scale; a.shift = p->shift; a.res = p->res;
  a.out_dtype = p->out_dtype; a.res_dtype = p->res_dtype; a.act = p->act; a.alpha = p->alpha;
  a.M = p->n * p->oh * p->ow; a.N = p->f; a.K = p->kh * p->kw * p->c;
  a.b_sk = 1; a.b_sn = a.K; a.o_sm = p->f; a.r_sm = p->f; a.r_sn = 1; a.b1 = 1;
  a.H = (int)p->h; a.W = (int)p->w_in; a.C = (int)p->c; a.KH = (int)p->kh; a.KW = (int)p->kw; a.OH = (int)p->oh; a.OW = (int)p->ow;
  a.sh = p->stride_h; a.sw = p->stride_w; a.ph = p->pad_h; a.pw = p->pad_w; a.dh = p->dil_h; a.dw = p->dil_w;
  const int eb = p->in_dtype == LLC_FLOAT32 ? 4 : 2, ob = p->out_dtype == LLC_FLOAT32 ? 4 : 2;
  a.vecOut = aligned(p->out, ob * 4) && p->f % 4 == 0;
  bool vec = p->c % 4 == 0 && aligned(p->x, eb * 4) && aligned(p->w, eb * 4);
  if (p->in_dtype == LLC_FLOAT32) return vec ? launchTiles<float, true, true>(a, 1, st, nullptr, 0) : launchTiles<float, true, false>(a, 1, st, nullptr, 0);
  if (p->in_dtype == LLC_BFLOAT16) return vec ? launchTiles<__nv_bfloat16, true, true>(a, 1, st, nullptr, 0) : launchTiles<__nv_bfloat16, true, false>(a, 1, st, nullptr, 0);
  return setError(LLC_ERR_UNSUPPORTED, "llc argument: conv input type must be f32 or bf16");
}

}  // namespace llc

// ---- entry point that allocates nothing ----------------------------------------------------------
// Some hosts of this library cannot allocate device memory when they call it: a serving process
// that handed the whole GPU to its own pool at start-up (a cudaMalloc here would fail or eat into
// that pool), or a control loop that cannot afford the device-wide synchronisation and driver lock
// an allocation takes.  For them the split-K GEMM keeps its scratch (tile counters + fp32 partial
// tiles) in a fixed array that is part of the library image: every GPU that loads the library
// holds these kStaticScratchBytes until the process exits.
namespace llc {
namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;   // 1 MiB: 4096 bytes of counters + partial tiles
static __device__ __align__(256) unsigned char g_staticScratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_staticScratchPtr[kMaxDevices] = {nullptr};
std::mutex g_staticScratchMutex;

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, not something a kernel can dereference; the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int staticScratchAddress(void** out) {
  int dev = 0;
  LLC_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return setError(LLC_ERR_ARGUMENT, "llc argument: device ordinal above 63");
  std::lock_guard<std::mutex> lock(g_staticScratchMutex);
  if (!g_staticScratchPtr[dev]) {
    void* ptr = nullptr;
    LLC_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_staticScratch));
    if (!ptr) return setError(LLC_ERR_CUDA, "llc cuda: cudaGetSymbolAddress returned a null address");
    g_staticScratchPtr[dev] = ptr;
  }
  *out = g_staticScratchPtr[dev];
  return LLC_OK;
}

}  // namespace
}  // namespace llc

extern "C" int llc_cuda_gemm_static_scratch(const LlcGemmParams* p, void* stream) {
  using namespace llc;
  if (!p) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm null parameter block");
  if (p->m < 0 || p->n < 0 || p->k < 0 || p->b0 < 0 || p->b1 < 0) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm negative extent");
  if (p->m == 0 || p->n == 0 || p->b0 == 0 || p->b1 == 0) return LLC_OK;
  if (!p->a || !p->b || !p->out) return setError(LLC_ERR_ARGUMENT, "llc argument: gemm null operand");
  auto floatIo = [](int32_t dt) { return dt == LLC_FLOAT32 || dt == LLC_BFLOAT16; };
  if (!floatIo(p->in_dtype) || !floatIo(p->out_dtype) || (p->res && !floatIo(p->res_dtype)))
    return setError(LLC_ERR_UNSUPPORTED, "llc argument: gemm operands must be f32 or bf16");
  // the split the launcher would choose with scratch at hand; a shape whose split does not fit is refused
  const SplitKChoice c = chooseSplitK(p->m, p->n, p->k, p->b0 * p->b1);
  if (c.split > 1 && c.need > kStaticScratchBytes)
    return setError(LLC_ERR_ARGUMENT, "llc argument: this GEMM needs " + std::to_string(c.need) + " bytes of split-K scratch, the built-in array holds " +
                                          std::to_string(kStaticScratchBytes));
  void* scratch = nullptr;
  int rc = staticScratchAddress(&scratch);
  if (rc != LLC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps whatever the previous call left: the tile counters must start at zero
  LLC_CUDA_CHECK(cudaMemsetAsync(scratch, 0, kCounterBytes, st));
  return igemmSimtGemm(p, st, scratch, (long long)kStaticScratchBytes);
}

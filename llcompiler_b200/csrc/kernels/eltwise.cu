// Fused elementwise chains, strided copies, max pooling and embedding gather: the HBM-bound
// data-movement kernels.  Algorithmic bytes per call: every input element once + every output
// element once at storage width.
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <vector>

#include "common.cuh"

namespace llc {
namespace {

constexpr int kMaxInstr = 48;
constexpr int kMaxRank = 6;
constexpr int kMaxIn = 8;

enum EltOp : int {
  E_LD = 0, E_IMM, E_ADD, E_SUB, E_MUL, E_DIV, E_MAX, E_MIN, E_POW, E_RELU, E_ABS, E_SQRT, E_RSQRT, E_EXP, E_GELU, E_TANH,
  E_ERF, E_SIGMOID, E_NEG, E_CAST, E_TRUNC, E_TF32LO, E_WHERE, E_EQ, E_NE, E_GE, E_GT, E_LE, E_LT
};

struct EltProgram {
  int n;
  unsigned char op[kMaxInstr], a[kMaxInstr], b[kMaxInstr], c[kMaxInstr];
  float imm[kMaxInstr];
};

struct EltArgs {
  void* out; int odt; int rank; int nin;
  long long shape[kMaxRank], ostr[kMaxRank];
  const void* in[kMaxIn]; int idt[kMaxIn]; long long istr[kMaxIn][kMaxRank];
  long long total;      // number of output elements
  int innerVec;         // elements handled per thread along the innermost dim (1 or 4)
  EltProgram prog;
};

__device__ __forceinline__ float evalOp(int op, float x, float y, float z, float imm) {
  switch (op) {
    case E_IMM: return imm;
    case E_ADD: return x + y;
    case E_SUB: return x - y;
    case E_MUL: return x * y;
    case E_DIV: return x / y;
    case E_MAX: return fmaxf(x, y);
    case E_MIN: return fminf(x, y);
    case E_POW: return powf(x, y);
    case E_RELU: return fmaxf(x, 0.f);
    case E_ABS: return fabsf(x);
    case E_SQRT: return sqrtf(x);
    case E_RSQRT: return rsqrtf(x);
    case E_EXP: return expf(x);
    case E_GELU: return geluErf(x);
    case E_TANH: return tanhf(x);
    case E_ERF: return erff(x);
    case E_SIGMOID: return 1.f / (1.f + expf(-x));
    case E_NEG: return -x;
    case E_CAST: return x;
    case E_TRUNC: return truncf(x);
    case E_TF32LO: return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);   // what a tf32 operand read drops
    case E_WHERE: return x != 0.f ? y : z;
    case E_EQ: return x == y ? 1.f : 0.f;
    case E_NE: return x != y ? 1.f : 0.f;
    case E_GE: return x >= y ? 1.f : 0.f;
    case E_GT: return x > y ? 1.f : 0.f;
    case E_LE: return x <= y ? 1.f : 0.f;
    case E_LT: return x < y ? 1.f : 0.f;
  }
  return 0.f;
}

// One thread produces V consecutive elements of the innermost (unit output stride) dim.
template <int V>
__global__ void __launch_bounds__(256) eltwise_kernel(const __grid_constant__ EltArgs p) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long first = t * V;
  if (first >= p.total) return;
  // decompose the linear index over the (collapsed) shape, innermost last
  long long rem = first, oOff = 0, iOff[kMaxIn];
#pragma unroll
  for (int k = 0; k < kMaxIn; ++k) iOff[k] = 0;
  for (int d = p.rank - 1; d >= 0; --d) {
    long long c = rem % p.shape[d]; rem /= p.shape[d];
    oOff += c * p.ostr[d];
    for (int k = 0; k < p.nin; ++k) iOff[k] += c * p.istr[k][d];
  }
  const int last = p.rank - 1;
  float regs[kMaxInstr][V];
  for (int i = 0; i < p.prog.n; ++i) {
    const int op = p.prog.op[i];
    if (op == E_LD) {
      const int k = p.prog.a[i];
#pragma unroll
      for (int v = 0; v < V; ++v) regs[i][v] = loadAs(p.in[k], iOff[k] + v * p.istr[k][last], p.idt[k]);
    } else {
      const int a = p.prog.a[i], b = p.prog.b[i], c = p.prog.c[i];
#pragma unroll
      for (int v = 0; v < V; ++v) regs[i][v] = evalOp(op, regs[a][v], regs[b][v], regs[c][v], p.prog.imm[i]);
    }
  }
  const int r = p.prog.n - 1;
#pragma unroll
  for (int v = 0; v < V; ++v) storeAs(p.out, oOff + v * p.ostr[last], p.odt, regs[r][v]);
}

// Fast path: everything dense (or broadcast) along the innermost dim, f32/bf16 storage, 16-byte
// aligned: 128-bit loads and stores, four elements per thread.
struct VecIo {
  static __device__ __forceinline__ float4 load(const void* p, long long off, int dt, long long stride) {
    if (stride == 0) { float v = loadAs(p, off, dt); return make_float4(v, v, v, v); }
    if (dt == LLC_FLOAT32) return Vec4<float>::load(reinterpret_cast<const float*>(p) + off);
    return Vec4<__nv_bfloat16>::load(reinterpret_cast<const __nv_bfloat16*>(p) + off);
  }
  static __device__ __forceinline__ void store(void* p, long long off, int dt, float4 v) {
    if (dt == LLC_FLOAT32) Vec4<float>::store(reinterpret_cast<float*>(p) + off, v);
    else Vec4<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16*>(p) + off, v);
  }
};
__global__ void __launch_bounds__(256) eltwise_vec_kernel(const __grid_constant__ EltArgs p) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long first = t * 4;
  if (first >= p.total) return;
  long long rem = first, oOff = 0, iOff[kMaxIn];
#pragma unroll
  for (int k = 0; k < kMaxIn; ++k) iOff[k] = 0;
  for (int d = p.rank - 1; d >= 0; --d) {
    long long c = rem % p.shape[d]; rem /= p.shape[d];
    oOff += c * p.ostr[d];
    for (int k = 0; k < p.nin; ++k) iOff[k] += c * p.istr[k][d];
  }
  const int last = p.rank - 1;
  float regs[kMaxInstr][4];
  for (int i = 0; i < p.prog.n; ++i) {
    const int op = p.prog.op[i];
    if (op == E_LD) {
      const int k = p.prog.a[i];
      float4 v = VecIo::load(p.in[k], iOff[k], p.idt[k], p.istr[k][last]);
      regs[i][0] = v.x; regs[i][1] = v.y; regs[i][2] = v.z; regs[i][3] = v.w;
    } else {
      const int a = p.prog.a[i], b = p.prog.b[i], c = p.prog.c[i];
#pragma unroll
      for (int v = 0; v < 4; ++v) regs[i][v] = evalOp(op, regs[a][v], regs[b][v], regs[c][v], p.prog.imm[i]);
    }
  }
  const int r = p.prog.n - 1;
  VecIo::store(p.out, oOff, p.odt, make_float4(regs[r][0], regs[r][1], regs[r][2], regs[r][3]));
}

// Short programs (at most four instructions: a copy, a cast, one unary or binary op on loaded operands, ...) on rows that
// are dense or broadcast along the innermost dim: eight elements per thread with 16-byte accesses, the registers of the
// program in real registers (the general kernels above index their register file dynamically, which puts it in local
// memory).  This is the path of the big memory-bound steps: layout copies, embedding sums, residual adds, casts.
constexpr int kSmallProg = 4;
template <typename T> __device__ __forceinline__ void load8(const T* p, float* v);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* v) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
}
__device__ __forceinline__ float pick4(const float (*r)[8], int which, int v) {
  const float lo = which & 1 ? r[1][v] : r[0][v], hi = which & 1 ? r[3][v] : r[2][v];
  return which & 2 ? hi : lo;
}
// Eight neighbouring elements of the innermost dim: the operands' element offsets are given, the program is run on registers.
__device__ __forceinline__ void eltwiseSmallBody(const EltArgs& p, long long oOff, const long long* iOff) {
  const int last = p.rank - 1;
  auto loadOperand = [&](int k, float* dst) {
    const void* base = k == 0 ? p.in[0] : k == 1 ? p.in[1] : k == 2 ? p.in[2] : p.in[3];
    const int dt = k == 0 ? p.idt[0] : k == 1 ? p.idt[1] : k == 2 ? p.idt[2] : p.idt[3];
    const long long off = k == 0 ? iOff[0] : k == 1 ? iOff[1] : k == 2 ? iOff[2] : iOff[3];
    const long long str = k == 0 ? p.istr[0][last] : k == 1 ? p.istr[1][last] : k == 2 ? p.istr[2][last] : p.istr[3][last];
    if (str == 0) {
      const float x = loadAs(base, off, dt);
#pragma unroll
      for (int v = 0; v < 8; ++v) dst[v] = x;
    } else if (dt == LLC_FLOAT32) load8<float>(reinterpret_cast<const float*>(base) + off, dst);
    else load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(base) + off, dst);
  };
  float o[8];
  // the two shapes almost every large step has: one operand (a copy, a cast, one unary op) or two operands and one
  // binary op; the op is decoded once, outside the element loop
  const int n = p.prog.n;
  const bool unary = (n == 1 || (n == 2 && p.prog.op[1] != E_LD && p.prog.op[1] != E_IMM && p.prog.a[1] == 0)) && p.prog.op[0] == E_LD;
  const bool binary = n == 3 && p.prog.op[0] == E_LD && p.prog.op[1] == E_LD && p.prog.op[2] >= E_ADD && p.prog.op[2] <= E_MIN && p.prog.a[2] + p.prog.b[2] == 1;
  if (unary) {
    loadOperand(p.prog.a[0], o);
    if (n == 2) {
      const int op = p.prog.op[1];
      if (op == E_RELU) {
#pragma unroll
        for (int v = 0; v < 8; ++v) o[v] = fmaxf(o[v], 0.f);
      } else if (op != E_CAST) {
#pragma unroll
        for (int v = 0; v < 8; ++v) o[v] = evalOp(op, o[v], o[v], o[v], 0.f);
      }
    }
  } else if (binary) {
    float x[8], y[8];
    loadOperand(p.prog.a[p.prog.a[2]], x); loadOperand(p.prog.a[p.prog.b[2]], y);
    switch (p.prog.op[2]) {
#define LLC_BIN(OP, EXPR) case OP: _Pragma("unroll") for (int v = 0; v < 8; ++v) o[v] = EXPR; break;
      LLC_BIN(E_ADD, x[v] + y[v]) LLC_BIN(E_SUB, x[v] - y[v]) LLC_BIN(E_MUL, x[v] * y[v]) LLC_BIN(E_DIV, x[v] / y[v])
      LLC_BIN(E_MAX, fmaxf(x[v], y[v])) LLC_BIN(E_MIN, fminf(x[v], y[v]))
#undef LLC_BIN
    }
  } else {
  float r[kSmallProg][8];
#pragma unroll
  for (int i = 0; i < kSmallProg; ++i) {
    if (i < p.prog.n) {
      const int op = p.prog.op[i];
      if (op == E_LD) {
        loadOperand(p.prog.a[i], r[i]);
      } else {
        const int a = p.prog.a[i], b = p.prog.b[i], c = p.prog.c[i];
        const float imm = p.prog.imm[i];
#pragma unroll
        for (int v = 0; v < 8; ++v) r[i][v] = evalOp(op, pick4(r, a, v), pick4(r, b, v), pick4(r, c, v), imm);
      }
    } else {
#pragma unroll
      for (int v = 0; v < 8; ++v) r[i][v] = 0.f;
    }
  }
#pragma unroll
  for (int v = 0; v < 8; ++v) o[v] = pick4(r, p.prog.n - 1, v);
  }

  if (p.odt == LLC_FLOAT32) {
    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + oOff);
    dst[0] = make_float4(o[0], o[1], o[2], o[3]); dst[1] = make_float4(o[4], o[5], o[6], o[7]);
  } else {
    uint4 q; __nv_bfloat162 h;
    h = __floats2bfloat162_rn(o[0], o[1]); q.x = *reinterpret_cast<unsigned*>(&h); h = __floats2bfloat162_rn(o[2], o[3]); q.y = *reinterpret_cast<unsigned*>(&h);
    h = __floats2bfloat162_rn(o[4], o[5]); q.z = *reinterpret_cast<unsigned*>(&h); h = __floats2bfloat162_rn(o[6], o[7]); q.w = *reinterpret_cast<unsigned*>(&h);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + oOff) = q;
  }
}

template <typename IDX>
__global__ void __launch_bounds__(256) eltwise_small_kernel(const __grid_constant__ EltArgs p) {
  const IDX t = (IDX)blockIdx.x * blockDim.x + threadIdx.x;
  if ((long long)t * 8 >= p.total) return;
  IDX rem = t * 8;
  long long oOff = 0, iOff[kSmallProg] = {0, 0, 0, 0};
  for (int d = p.rank - 1; d >= 0; --d) {
    const IDX ext = (IDX)p.shape[d];
    const IDX c = rem % ext; rem /= ext;
    oOff += (long long)c * p.ostr[d];
#pragma unroll
    for (int k = 0; k < kSmallProg; ++k) if (k < p.nin) iOff[k] += (long long)c * p.istr[k][d];
  }
  eltwiseSmallBody(p, oOff, iOff);
}

// The same for at most two dims (rows x inner, which is what is left of most steps once dense dims are merged): a block
// is blockDim.y rows by blockDim.x eight-element pieces of one row part, so no thread divides.
__global__ void __launch_bounds__(256) eltwise_small_rows_kernel(const __grid_constant__ EltArgs p, int partsPerRow, long long rows, int pieces) {
  const long long rowBlock = blockIdx.x / partsPerRow;
  const int part = (int)(blockIdx.x - rowBlock * partsPerRow);
  const long long row = rowBlock * blockDim.y + threadIdx.y;
  const int piece = part * (int)blockDim.x + (int)threadIdx.x;
  if (row >= rows || piece >= pieces) return;
  const bool two = p.rank == 2;
  const int last = p.rank - 1;
  const long long col = (long long)piece * 8;
  long long oOff = col + (two ? row * p.ostr[0] : 0), iOff[kSmallProg] = {0, 0, 0, 0};
#pragma unroll
  for (int k = 0; k < kSmallProg; ++k) if (k < p.nin) iOff[k] = col * p.istr[k][last] + (two ? row * p.istr[k][0] : 0);
  eltwiseSmallBody(p, oOff, iOff);
}

int parseProgram(const char* text, EltProgram& prog, int nin) {
  static const struct { const char* name; int op; int arity; } table[] = {
      {"add", E_ADD, 2}, {"sub", E_SUB, 2}, {"mul", E_MUL, 2}, {"div", E_DIV, 2}, {"max", E_MAX, 2}, {"min", E_MIN, 2}, {"pow", E_POW, 2},
      {"relu", E_RELU, 1}, {"abs", E_ABS, 1}, {"sqrt", E_SQRT, 1}, {"rsqrt", E_RSQRT, 1}, {"exp", E_EXP, 1}, {"gelu", E_GELU, 1},
      {"tanh", E_TANH, 1}, {"erf", E_ERF, 1}, {"sigmoid", E_SIGMOID, 1}, {"neg", E_NEG, 1}, {"cast", E_CAST, 1}, {"trunc", E_TRUNC, 1}, {"tf32lo", E_TF32LO, 1},
      {"where", E_WHERE, 3}, {"eq", E_EQ, 2}, {"ne", E_NE, 2}, {"ge", E_GE, 2}, {"gt", E_GT, 2}, {"le", E_LE, 2}, {"lt", E_LT, 2}};
  prog.n = 0;
  std::string s = text ? text : "";
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t end = s.find(';', pos);
    if (end == std::string::npos) end = s.size();
    std::string ins = s.substr(pos, end - pos);
    pos = end + 1;
    if (ins.empty()) { if (end == s.size()) break; continue; }
    if (prog.n >= kMaxInstr) return setError(LLC_ERR_ARGUMENT, "llc argument: elementwise program longer than 48 instructions");
    int i = prog.n++;
    prog.a[i] = prog.b[i] = prog.c[i] = 0; prog.imm[i] = 0.f;
    if (ins.compare(0, 2, "ld") == 0) {
      int k = atoi(ins.c_str() + 2);
      if (k < 0 || k >= nin) return setError(LLC_ERR_ARGUMENT, "llc argument: elementwise program loads a missing input");
      prog.op[i] = E_LD; prog.a[i] = (unsigned char)k;
    } else if (ins[0] == '#') {
      prog.op[i] = E_IMM; prog.imm[i] = strtof(ins.c_str() + 1, nullptr);
    } else {
      std::vector<std::string> f; size_t q = 0;
      while (q <= ins.size()) { size_t e = ins.find(',', q); if (e == std::string::npos) e = ins.size(); f.push_back(ins.substr(q, e - q)); q = e + 1; }
      int found = -1;
      for (size_t k = 0; k < sizeof(table) / sizeof(table[0]); ++k) if (f[0] == table[k].name) found = (int)k;
      if (found < 0) return setError(LLC_ERR_ARGUMENT, "llc argument: unknown elementwise op '" + f[0] + "'");
      if ((int)f.size() - 1 != table[found].arity) return setError(LLC_ERR_ARGUMENT, "llc argument: wrong operand count for '" + f[0] + "'");
      prog.op[i] = (unsigned char)table[found].op;
      unsigned char* dst[3] = {&prog.a[i], &prog.b[i], &prog.c[i]};
      for (int k = 0; k < table[found].arity; ++k) {
        int r = atoi(f[k + 1].c_str());
        if (r < 0 || r >= i) return setError(LLC_ERR_ARGUMENT, "llc argument: elementwise program reads an undefined register");
        *dst[k] = (unsigned char)r;
      }
    }
  }
  if (prog.n == 0) return setError(LLC_ERR_ARGUMENT, "llc argument: empty elementwise program");
  return LLC_OK;
}

// ---- max pooling (NHWC) -------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(256) maxpool_nhwc_kernel(const T* __restrict__ x, T* __restrict__ out, LlcPoolParams p) {
  const long long cv = p.c / V;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = p.n * p.oh * p.ow * cv;
  if (idx >= total) return;
  int c = (int)(idx % cv) * V; long long t = idx / cv;
  int ow = (int)(t % p.ow); t /= p.ow; int oh = (int)(t % p.oh); long long n = t / p.oh;
  float m[V];
#pragma unroll
  for (int v = 0; v < V; ++v) m[v] = -INFINITY;
  for (int r = 0; r < p.kh; ++r) {
    int ih = oh * p.stride_h - p.pad_h + r * p.dil_h;
    if (ih < 0 || ih >= p.h) continue;
    for (int s = 0; s < p.kw; ++s) {
      int iw = ow * p.stride_w - p.pad_w + s * p.dil_w;
      if (iw < 0 || iw >= p.w) continue;
      const T* src = x + ((n * p.h + ih) * p.w + iw) * p.c + c;
      if (V == 4) { float4 q = Vec4<T>::load(src); m[0] = fmaxf(m[0], q.x); m[1] = fmaxf(m[1], q.y); m[2] = fmaxf(m[2], q.z); m[3] = fmaxf(m[3], q.w); }
      else m[0] = fmaxf(m[0], toFloat<T>(src[0]));
    }
  }
  T* dst = out + ((n * p.oh + oh) * p.ow + ow) * p.c + c;
  if (V == 4) Vec4<T>::store(dst, make_float4(m[0], m[1], m[2], m[3]));
  else storeAs(dst, 0, sizeof(T) == 4 ? LLC_FLOAT32 : LLC_BFLOAT16, m[0]);
}

// ---- gather --------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_rows_kernel(const void* table, const long long* ids, void* out, int tdt, int odt, long long rows, long long d,
                                                          long long vocab, int* bad, int fastCopy) {
  long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  long long id = ids[row];
  bool ok = id >= 0 && id < vocab;
  if (!ok && lane == 0 && bad) atomicAdd(bad, 1);
  if (ok && fastCopy) {
    // same storage type: copy 16 bytes at a time
    const int eb = tdt == LLC_FLOAT32 ? 4 : 2;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(table) + id * d * eb);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(out) + row * d * eb);
    long long n16 = d * eb / 16;
    for (long long i = lane; i < n16; i += 32) dst[i] = src[i];
    return;
  }
  for (long long c = lane; c < d; c += 32) storeAs(out, row * d + c, odt, ok ? loadAs(table, id * d + c, tdt) : 0.f);
}

// ---- NCHW -> NHWC re-layout with optional zero padding of the channel count --------------------
// Few channels (the image stem): one thread per pixel reads its C planes (coalesced across the
// warp) and writes the padded pixel with 16-byte stores.
template <typename T, int CP>
__global__ void __launch_bounds__(256) nchw_to_nhwc_small_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int c, long long hw) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * hw) return;
  long long img = idx / hw, px = idx - img * hw;
  __align__(16) T v[CP];
#pragma unroll
  for (int k = 0; k < CP; ++k) v[k] = k < c ? x[(img * c + k) * hw + px] : T(0.f);
  constexpr int kVec = CP * sizeof(T) / 16;
  uint4* dst = reinterpret_cast<uint4*>(out + idx * CP);
#pragma unroll
  for (int k = 0; k < kVec; ++k) dst[k] = reinterpret_cast<const uint4*>(v)[k];
}
// Many channels: 32 x 32 tiles of the [C, HW] plane of one image go through shared memory so that
// both the read (along HW) and the write (along C) are coalesced.
template <typename T>
__global__ void __launch_bounds__(256) nchw_to_nhwc_tiled_kernel(const T* __restrict__ x, T* __restrict__ out, int c, long long hw, int cp) {
  __shared__ T tile[32][33];
  const long long img = blockIdx.z;
  const long long p0 = (long long)blockIdx.x * 32; const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    int ch = c0 + r; long long px = p0 + tx;
    tile[r][tx] = (ch < c && px < hw) ? x[(img * c + ch) * hw + px] : T(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    long long px = p0 + r; int ch = c0 + tx;
    if (px < hw && ch < cp) out[(img * hw + px) * cp + ch] = tile[tx][r];
  }
}

}  // namespace
}  // namespace llc

using namespace llc;

// Same with the rows widened: output pixel (img, h, wq) of a [n, h, w_total, CP] buffer is input pixel wq - w_left, or
// zeros in the halo columns left and right of the image.
// A thread block takes kRows output rows; thread t takes the pixels t, t + 256, ... of each of them, so that kRows * c
// loads are in flight per thread, neighbouring threads read neighbouring elements, and no thread divides.
template <typename T, int CP, int kRows>
__global__ void __launch_bounds__(256) nchw_to_nhwc_wide_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int c, int h, int w, int w_left,
                                                                 int w_total) {
  const long long row0 = (long long)blockIdx.x * kRows, rows = n * h;
  const long long hw = (long long)h * w;
  const T* src[kRows];
  T* dst[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const long long r = min(row0 + i, rows - 1);
    const long long img = r / h;
    src[i] = x + img * c * hw + (r - img * h) * w;
    dst[i] = out + r * (long long)w_total * CP;
  }
  for (int wq = threadIdx.x; wq < w_total; wq += 256) {
    const int wi = wq - w_left;
    const bool inside = wi >= 0 && wi < w;
    __align__(16) T v[kRows][CP];
#pragma unroll
    for (int i = 0; i < kRows; ++i)
#pragma unroll
      for (int k = 0; k < CP; ++k) v[i][k] = (inside && k < c) ? src[i][k * hw + wi] : T(0.f);
    constexpr int kVec = CP * sizeof(T) / 16;
#pragma unroll
    for (int i = 0; i < kRows; ++i)
      if (row0 + i < rows) {
        uint4* d = reinterpret_cast<uint4*>(dst[i] + (long long)wq * CP);
#pragma unroll
        for (int k = 0; k < kVec; ++k) d[k] = reinterpret_cast<const uint4*>(v[i])[k];
      }
  }
}

// The same for image rows that start on a 4-element boundary: a thread reads four neighbouring pixels of every channel
// with one vector load each and writes their four padded pixels (64 contiguous bytes); the zero columns left and right of
// the image are written by a few extra threads per row.
template <typename T, int CP>
__global__ void __launch_bounds__(256) nchw_to_nhwc_wide_quad_kernel(const T* __restrict__ x, T* __restrict__ out, long long rows, int c, int h, int w,
                                                                      int w_left, int w_total) {
  struct alignas(4 * sizeof(T)) Quad { T v[4]; };
  const int quads = w / 4, halo = w_total - w, perRow = quads + (halo + 3) / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long r = idx / perRow;
  if (r >= rows) return;
  const int j = (int)(idx - r * perRow);
  T* dstRow = out + r * (long long)w_total * CP;
  constexpr int kVec = CP * sizeof(T) / 16;
  if (j < quads) {
    const long long img = r / h, hw = (long long)h * w;
    const T* src = x + img * c * hw + (r - img * h) * w + 4 * j;
    Quad q[CP];
#pragma unroll
    for (int k = 0; k < CP; ++k)
      if (k < c) q[k] = *reinterpret_cast<const Quad*>(src + k * hw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __align__(16) T v[CP];
#pragma unroll
      for (int k = 0; k < CP; ++k) v[k] = k < c ? q[k].v[i] : T(0.f);
      uint4* d = reinterpret_cast<uint4*>(dstRow + (long long)(w_left + 4 * j + i) * CP);
#pragma unroll
      for (int k = 0; k < kVec; ++k) d[k] = reinterpret_cast<const uint4*>(v)[k];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int hq = (j - quads) * 4 + i;
      if (hq < halo) {
        uint4* d = reinterpret_cast<uint4*>(dstRow + (long long)(hq < w_left ? hq : w + hq) * CP);
#pragma unroll
        for (int k = 0; k < kVec; ++k) d[k] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
}

extern "C" int llc_cuda_nchw_to_nhwc_wide(const void* x, void* out, int32_t dtype, int64_t n, int64_t c, int64_t h, int64_t w, int64_t c_pad, int64_t w_left,
                                          int64_t w_total, void* stream) {
  if (n <= 0 || h <= 0 || w <= 0 || c <= 0) return LLC_OK;
  if (!x || !out) return setError(LLC_ERR_ARGUMENT, "llc argument: nchw_to_nhwc_wide null pointer");
  if (c_pad < c || w_left < 0 || w_total < w_left + w) return setError(LLC_ERR_ARGUMENT, "llc argument: nchw_to_nhwc_wide padding smaller than the image");
  if (reinterpret_cast<uintptr_t>(out) % 16 != 0) return setError(LLC_ERR_ARGUMENT, "llc argument: nchw_to_nhwc_wide output must be 16-byte aligned");
  const bool f32 = dtype == LLC_FLOAT32;
  if (!((f32 && c_pad == 4) || (dtype == LLC_BFLOAT16 && c_pad == 8)))
    return setError(LLC_ERR_UNSUPPORTED, "llc argument: nchw_to_nhwc_wide takes f32 padded to 4 channels or bf16 padded to 8");
  if (n * h > 0x7FFFFFFFLL) return setError(LLC_ERR_UNSUPPORTED, "llc argument: nchw_to_nhwc_wide takes at most 2^31 - 1 image rows");
  constexpr int kRows = 4;
  const unsigned blocks = (unsigned)((n * h + kRows - 1) / kRows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t elt = f32 ? 4 : 2;
  if (w % 4 == 0 && reinterpret_cast<uintptr_t>(x) % (4 * elt) == 0) {       // every image row starts on a 4-element boundary
    const long long perRow = w / 4 + (w_total - w + 3) / 4, threads = n * h * perRow;
    const unsigned qb = (unsigned)((threads + 255) / 256);
    if (f32) nchw_to_nhwc_wide_quad_kernel<float, 4><<<qb, 256, 0, st>>>((const float*)x, (float*)out, n * h, (int)c, (int)h, (int)w, (int)w_left, (int)w_total);
    else nchw_to_nhwc_wide_quad_kernel<__nv_bfloat16, 8><<<qb, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n * h, (int)c, (int)h, (int)w, (int)w_left, (int)w_total);
    LLC_LAUNCH_CHECK("nchw_to_nhwc_wide_quad_kernel");
    return LLC_OK;
  }
  if (f32) nchw_to_nhwc_wide_kernel<float, 4, kRows><<<blocks, 256, 0, st>>>((const float*)x, (float*)out, n, (int)c, (int)h, (int)w, (int)w_left, (int)w_total);
  else nchw_to_nhwc_wide_kernel<__nv_bfloat16, 8, kRows><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, (int)c, (int)h, (int)w, (int)w_left, (int)w_total);
  LLC_LAUNCH_CHECK("nchw_to_nhwc_wide_kernel");
  return LLC_OK;
}

extern "C" int llc_cuda_nchw_to_nhwc(const void* x, void* out, int32_t dtype, int64_t n, int64_t c, int64_t hw, int64_t c_pad, void* stream) {
  if (n <= 0 || c <= 0 || hw <= 0) return LLC_OK;
  if (!x || !out) return setError(LLC_ERR_ARGUMENT, "llc argument: nchw_to_nhwc null pointer");
  if (c_pad < c) return setError(LLC_ERR_ARGUMENT, "llc argument: padded channel count below the channel count");
  if (dtype != LLC_FLOAT32 && dtype != LLC_BFLOAT16) return setError(LLC_ERR_UNSUPPORTED, "llc argument: nchw_to_nhwc type must be f32 or bf16");
  if (n > 65535) return setError(LLC_ERR_ARGUMENT, "llc argument: nchw_to_nhwc batch above 65535");
  cudaStream_t st = (cudaStream_t)stream;
  const bool f32 = dtype == LLC_FLOAT32;
  const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const unsigned blocks = (unsigned)((n * hw + 255) / 256);
  if (aligned && f32 && c_pad == 4) nchw_to_nhwc_small_kernel<float, 4><<<blocks, 256, 0, st>>>((const float*)x, (float*)out, n, (int)c, hw);
  else if (aligned && f32 && c_pad == 8) nchw_to_nhwc_small_kernel<float, 8><<<blocks, 256, 0, st>>>((const float*)x, (float*)out, n, (int)c, hw);
  else if (aligned && !f32 && c_pad == 8) nchw_to_nhwc_small_kernel<__nv_bfloat16, 8><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, (int)c, hw);
  else if (aligned && !f32 && c_pad == 16) nchw_to_nhwc_small_kernel<__nv_bfloat16, 16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, (int)c, hw);
  else {
    dim3 g((unsigned)((hw + 31) / 32), (unsigned)((c_pad + 31) / 32), (unsigned)n);
    if (f32) nchw_to_nhwc_tiled_kernel<float><<<g, 256, 0, st>>>((const float*)x, (float*)out, (int)c, hw, (int)c_pad);
    else nchw_to_nhwc_tiled_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, (int)c, hw, (int)c_pad);
  }
  LLC_LAUNCH_CHECK("nchw_to_nhwc_kernel");
  return LLC_OK;
}

extern "C" int llc_cuda_eltwise(const LlcEltwiseParams* q, void* stream) {
  if (!q) return setError(LLC_ERR_ARGUMENT, "llc argument: eltwise null pointer");
  if (q->rank >= 1 && q->rank <= kMaxRank) {             // an empty tensor: nothing to do, whatever the pointers are
    bool none = false;
    for (int d = 0; d < q->rank; ++d) none = none || q->shape[d] == 0;
    if (none) return LLC_OK;
  }
  if (!q->out) return setError(LLC_ERR_ARGUMENT, "llc argument: eltwise null pointer");
  if (q->rank < 1 || q->rank > kMaxRank) return setError(LLC_ERR_ARGUMENT, "llc argument: eltwise rank must be 1..6");
  if (q->n_in < 0 || q->n_in > kMaxIn) return setError(LLC_ERR_ARGUMENT, "llc argument: eltwise takes at most 8 inputs");
  EltArgs a{};
  int rc = parseProgram(q->prog, a.prog, q->n_in);
  if (rc) return rc;
  a.out = q->out; a.odt = q->out_dtype; a.nin = q->n_in;
  for (int k = 0; k < q->n_in; ++k) { a.in[k] = q->in[k].data; a.idt[k] = q->in[k].dtype; if (!a.in[k]) return setError(LLC_ERR_ARGUMENT, "llc argument: eltwise null input"); }
  // order dims by output stride (outermost first), drop unit dims, merge dims that are dense in every operand
  std::vector<int> dims;
  long long total = 1;
  for (int d = 0; d < q->rank; ++d) { if (q->shape[d] < 0) return setError(LLC_ERR_ARGUMENT, "llc argument: negative extent"); total *= q->shape[d]; if (q->shape[d] != 1) dims.push_back(d); }
  if (total == 0) return LLC_OK;
  std::stable_sort(dims.begin(), dims.end(), [&](int x, int y) { return q->out_strides[x] > q->out_strides[y]; });
  int r = 0;
  for (int d : dims) {
    bool merge = r > 0;
    if (merge) {
      if (a.ostr[r - 1] != q->shape[d] * q->out_strides[d]) merge = false;
      for (int k = 0; k < q->n_in && merge; ++k) if (a.istr[k][r - 1] != q->shape[d] * q->in[k].strides[d]) merge = false;
    }
    if (merge) {
      a.shape[r - 1] *= q->shape[d]; a.ostr[r - 1] = q->out_strides[d];
      for (int k = 0; k < q->n_in; ++k) a.istr[k][r - 1] = q->in[k].strides[d];
    } else {
      a.shape[r] = q->shape[d]; a.ostr[r] = q->out_strides[d];
      for (int k = 0; k < q->n_in; ++k) a.istr[k][r] = q->in[k].strides[d];
      ++r;
    }
  }
  if (r == 0) { a.shape[0] = 1; a.ostr[0] = 1; for (int k = 0; k < q->n_in; ++k) a.istr[k][0] = 0; r = 1; }
  a.rank = r; a.total = total;
  cudaStream_t st = (cudaStream_t)stream;
  const long long inner = a.shape[r - 1];
  auto isVecType = [](int dt) { return dt == LLC_FLOAT32 || dt == LLC_BFLOAT16; };
  auto alignedFor = [](const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) % (dt == LLC_FLOAT32 ? 16 : 8)) == 0; };
  bool vec = inner % 4 == 0 && a.ostr[r - 1] == 1 && isVecType(a.odt) && alignedFor(a.out, a.odt);
  for (int d = 0; d + 1 < r && vec; ++d) if (a.ostr[d] % 4) vec = false;
  for (int k = 0; k < a.nin && vec; ++k) {
    long long s = a.istr[k][r - 1];
    if (s == 0) continue;
    if (s != 1 || !isVecType(a.idt[k]) || !alignedFor(a.in[k], a.idt[k])) vec = false;
    for (int d = 0; d + 1 < r && vec; ++d) if (a.istr[k][d] % 4) vec = false;
  }
  // eight elements per thread: every access 16 bytes wide (fp32: two of them) and aligned, whatever the outer coordinates
  bool small = vec && a.prog.n <= kSmallProg && a.nin <= kSmallProg && inner % 8 == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
  for (int d = 0; d + 1 < r && small; ++d) if (a.ostr[d] % 8) small = false;
  for (int k = 0; k < a.nin && small; ++k) {
    if (a.istr[k][r - 1] == 0) continue;
    if (reinterpret_cast<uintptr_t>(a.in[k]) & 15) small = false;
    for (int d = 0; d + 1 < r && small; ++d) if (a.istr[k][d] % 8) small = false;
  }
  if (small && r <= 2) {
    const long long rows = r == 2 ? a.shape[0] : 1, pieces = inner / 8;
    // threads along a row: the row's pieces split into equal parts of at most 256, rounded up to whole warps
    const long long parts = (pieces + 255) / 256;
    const int tx = (int)((((pieces + parts - 1) / parts) + 31) / 32 * 32);
    const int ty = (int)std::max<long long>(1, std::min<long long>(256 / tx, rows));
    const long long blocks = ((rows + ty - 1) / ty) * parts;
    if (pieces <= 0x7FFFFFFFLL / 8 && blocks <= 0x7FFFFFFFLL) {
      eltwise_small_rows_kernel<<<(unsigned)blocks, dim3((unsigned)tx, (unsigned)ty), 0, st>>>(a, (int)parts, rows, (int)pieces);
      LLC_LAUNCH_CHECK("eltwise_small_rows_kernel");
      return LLC_OK;
    }
  }
  if (small) {
    const long long threads = total / 8;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    if (total < (1LL << 32)) eltwise_small_kernel<unsigned><<<blocks, 256, 0, st>>>(a);
    else eltwise_small_kernel<unsigned long long><<<blocks, 256, 0, st>>>(a);
    LLC_LAUNCH_CHECK("eltwise_small_kernel");
  } else if (vec) {
    long long threads = total / 4;
    eltwise_vec_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(a);
    LLC_LAUNCH_CHECK("eltwise_vec_kernel");
  } else if (inner % 4 == 0) {
    long long threads = total / 4;
    eltwise_kernel<4><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(a);
    LLC_LAUNCH_CHECK("eltwise_kernel<4>");
  } else {
    eltwise_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a);
    LLC_LAUNCH_CHECK("eltwise_kernel<1>");
  }
  return LLC_OK;
}

// bf16 with a channel count that is a multiple of 8: 16-byte loads, maxima taken on packed pairs (exact).
__global__ void __launch_bounds__(256) maxpool_nhwc_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, LlcPoolParams p) {
  const long long cv = p.c / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.n * p.oh * p.ow * cv) return;
  const int c = (int)(idx % cv) * 8; long long t = idx / cv;
  const int ow = (int)(t % p.ow); t /= p.ow; const int oh = (int)(t % p.oh); const long long n = t / p.oh;
  const __nv_bfloat162 lowest = __floats2bfloat162_rn(-INFINITY, -INFINITY);
  __nv_bfloat162 m[4] = {lowest, lowest, lowest, lowest};
  for (int r = 0; r < p.kh; ++r) {
    const int ih = oh * p.stride_h - p.pad_h + r * p.dil_h;
    if (ih < 0 || ih >= p.h) continue;
    for (int s = 0; s < p.kw; ++s) {
      const int iw = ow * p.stride_w - p.pad_w + s * p.dil_w;
      if (iw < 0 || iw >= p.w) continue;
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + ((n * p.h + ih) * p.w + iw) * p.c + c));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) m[e] = __hmax2(m[e], h[e]);
    }
  }
  uint4 o;
  o.x = *reinterpret_cast<unsigned*>(&m[0]); o.y = *reinterpret_cast<unsigned*>(&m[1]); o.z = *reinterpret_cast<unsigned*>(&m[2]); o.w = *reinterpret_cast<unsigned*>(&m[3]);
  *reinterpret_cast<uint4*>(out + ((n * p.oh + oh) * p.ow + ow) * p.c + c) = o;
}

// The same for a window and stride known at compile time (3x3 / stride 2 is what the ResNets use): every load of the window
// is issued before the first maximum is taken (out-of-range taps read a clamped address and are masked afterwards), so a
// thread has KH*KW 16-byte loads in flight instead of one.
template <int KH, int KW, int S>
__global__ void __launch_bounds__(256) maxpool_nhwc_bf16x8_window_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, LlcPoolParams p) {
  const int cv = (int)(p.c / 8);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.n * p.oh * p.ow * cv) return;
  const unsigned pix = (unsigned)(idx / cv);
  const int c = (int)(idx - (long long)pix * cv) * 8;
  const unsigned ohow = (unsigned)(p.oh * p.ow);
  const unsigned n = pix / ohow, rem = pix - n * ohow;
  const int oh = (int)(rem / (unsigned)p.ow), ow = (int)(rem - (unsigned)oh * (unsigned)p.ow);
  const int ih0 = oh * S - (int)p.pad_h, iw0 = ow * S - (int)p.pad_w;
  const __nv_bfloat16* img = x + (long long)n * p.h * p.w * p.c + c;
  uint4 q[KH * KW];
#pragma unroll
  for (int r = 0; r < KH; ++r)
#pragma unroll
    for (int t = 0; t < KW; ++t) {
      const int ih = min(max(ih0 + r, 0), (int)p.h - 1), iw = min(max(iw0 + t, 0), (int)p.w - 1);
      q[r * KW + t] = __ldg(reinterpret_cast<const uint4*>(img + ((long long)ih * p.w + iw) * p.c));
    }
  const __nv_bfloat162 lowest = __floats2bfloat162_rn(-INFINITY, -INFINITY);
  __nv_bfloat162 m[4] = {lowest, lowest, lowest, lowest};
#pragma unroll
  for (int r = 0; r < KH; ++r)
#pragma unroll
    for (int t = 0; t < KW; ++t) {
      const bool in = ih0 + r >= 0 && ih0 + r < p.h && iw0 + t >= 0 && iw0 + t < p.w;
      const __nv_bfloat162* hq = reinterpret_cast<const __nv_bfloat162*>(&q[r * KW + t]);
#pragma unroll
      for (int e = 0; e < 4; ++e) m[e] = in ? __hmax2(m[e], hq[e]) : m[e];
    }
  uint4 o;
  o.x = *reinterpret_cast<unsigned*>(&m[0]); o.y = *reinterpret_cast<unsigned*>(&m[1]); o.z = *reinterpret_cast<unsigned*>(&m[2]); o.w = *reinterpret_cast<unsigned*>(&m[3]);
  *reinterpret_cast<uint4*>(out + (long long)pix * p.c + c) = o;
}

extern "C" int llc_cuda_maxpool2d(const LlcPoolParams* p, void* stream) {
  if (!p) return setError(LLC_ERR_ARGUMENT, "llc argument: maxpool null parameter block");
  long long total = p->n * p->oh * p->ow * p->c;
  if (total <= 0) return LLC_OK;                        // an empty batch: nothing to do, whatever the pointers are
  if (!p->x || !p->out) return setError(LLC_ERR_ARGUMENT, "llc argument: maxpool null pointer");
  if (p->in_dtype != p->out_dtype) return setError(LLC_ERR_ARGUMENT, "llc argument: maxpool input and output types differ");
  cudaStream_t st = (cudaStream_t)stream;
  bool v4 = p->c % 4 == 0 && (reinterpret_cast<uintptr_t>(p->x) % 16) == 0 && (reinterpret_cast<uintptr_t>(p->out) % 16) == 0;
  long long threads = v4 ? total / 4 : total;
  unsigned blocks = (unsigned)((threads + 255) / 256);
  if (p->in_dtype == LLC_FLOAT32) {
    if (v4) maxpool_nhwc_kernel<float, 4><<<blocks, 256, 0, st>>>((const float*)p->x, (float*)p->out, *p);
    else maxpool_nhwc_kernel<float, 1><<<blocks, 256, 0, st>>>((const float*)p->x, (float*)p->out, *p);
  } else if (p->in_dtype == LLC_BFLOAT16) {
    if (p->c % 8 == 0 && ((reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->out)) & 15) == 0) {
      const long long total8 = p->n * p->oh * p->ow * (p->c / 8);
      if (p->kh == 3 && p->kw == 3 && p->stride_h == 2 && p->stride_w == 2 && p->dil_h == 1 && p->dil_w == 1 && p->n * p->oh * p->ow < (1LL << 31))
        maxpool_nhwc_bf16x8_window_kernel<3, 3, 2><<<(unsigned)((total8 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)p->x, (__nv_bfloat16*)p->out, *p);
      else maxpool_nhwc_bf16x8_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)p->x, (__nv_bfloat16*)p->out, *p);
    } else if (v4) maxpool_nhwc_kernel<__nv_bfloat16, 4><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)p->x, (__nv_bfloat16*)p->out, *p);
    else maxpool_nhwc_kernel<__nv_bfloat16, 1><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)p->x, (__nv_bfloat16*)p->out, *p);
  } else return setError(LLC_ERR_UNSUPPORTED, "llc argument: maxpool type must be f32 or bf16");
  LLC_LAUNCH_CHECK("maxpool_nhwc_kernel");
  return LLC_OK;
}

extern "C" int llc_cuda_gather(const void* table, const int64_t* ids, void* out, int32_t tdt, int32_t odt, int64_t rows, int64_t d, int64_t vocab,
                               int32_t* bad, void* stream) {
  if (rows <= 0 || d <= 0) return LLC_OK;
  if (!table || !ids || !out) return setError(LLC_ERR_ARGUMENT, "llc argument: gather null pointer");
  int fast = tdt == odt && d % 8 == 0 && (tdt == LLC_BFLOAT16 || tdt == LLC_FLOAT32) && (reinterpret_cast<uintptr_t>(table) % 16) == 0 &&
             (reinterpret_cast<uintptr_t>(out) % 16) == 0;
  gather_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(table, (const long long*)ids, out, tdt, odt, rows, d, vocab, bad, fast);
  LLC_LAUNCH_CHECK("gather_rows_kernel");
  return LLC_OK;
}

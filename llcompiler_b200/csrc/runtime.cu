// The executor: loads a kernel plan, owns weights and the activation arena, binds shape
// symbols per call and launches the plan's kernels on a CUDA stream.
//
// Stands in for llc::compiler::Execution (src/Compiler/Execution.cpp:10-66), which dlopens the
// compiled object and calls its main(void**).  The reference's generated code mallocs and frees
// every intermediate on every call (memref_include.mlir:4-23); here all intermediates live in one
// arena whose layout is computed once per symbol binding from the plan's symbolic sizes by
// lifetime-based first-fit packing, and reused by every later call with that binding.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <sys/stat.h>
#include <unistd.h>

#include "../../include/llc_cuda.h"
#include "../../include/llc_runtime.h"
#include "capi_common.h"
#include "plan.h"

namespace llc {

int* tcStatusAddress();     // device addresses of the status words the bounded waits of the tensor-core kernels write
int* attnStatusAddress();
int* attnBlocksStatusAddress();

namespace {

// Makes `device` current for the duration of a call and puts the caller's device back afterwards.
struct DeviceGuard {
  int prev = -1; bool switched = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != device) { if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("llc cuda: cudaSetDevice failed"); switched = true; }
  }
  ~DeviceGuard() { if (switched && prev >= 0) cudaSetDevice(prev); }
};

[[noreturn]] void failArg(const std::string& m) { throw std::runtime_error("llc argument: " + m); }
[[noreturn]] void failIo(const std::string& m) { throw std::runtime_error("llc io: " + m); }
void cudaOk(cudaError_t e, const char* what) { if (e != cudaSuccess) throw std::runtime_error(std::string("llc cuda: ") + what + ": " + cudaGetErrorString(e)); }

int toLlcDType(DType t) {
  switch (t) {
    case DType::F32: return LLC_FLOAT32; case DType::BF16: return LLC_BFLOAT16; case DType::F16: return LLC_FLOAT16;
    case DType::F64: return LLC_FLOAT64; case DType::I64: case DType::Index: return LLC_INT64; case DType::I32: return LLC_INT32;
    case DType::I16: return LLC_INT16; case DType::I8: return LLC_INT8; case DType::I1: return LLC_INT1; default: return -1;
  }
}
size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

uint16_t f32ToBf16(float f) { uint32_t u; memcpy(&u, &f, 4); if ((u & 0x7fffffff) > 0x7f800000) return 0x7fc0; u += 0x7fff + ((u >> 16) & 1); return (uint16_t)(u >> 16); }

// .npy reader for the files llh.weight names (format v1/v2, little endian, C order); the
// reference's reader is src/Dialect/LLH/Transforms/LoadWeight.cpp:58-103.
std::vector<char> readNpy(const std::string& path, DType want, size_t numel) {
  std::ifstream f(path, std::ios::binary);
  if (!f) failIo("cannot open weight file " + path);
  char magic[10];
  f.read(magic, 10);
  if (!f || memcmp(magic, "\x93NUMPY", 6) != 0) failIo(path + " is not an .npy file");
  size_t hlen = (unsigned char)magic[8] | ((unsigned char)magic[9] << 8);
  if (magic[6] >= 2) { char more[2]; f.read(more, 2); hlen |= ((size_t)(unsigned char)more[0] << 16) | ((size_t)(unsigned char)more[1] << 24); }
  std::string header(hlen, ' ');
  f.read(&header[0], (std::streamsize)hlen);
  auto field = [&](const std::string& key) { size_t p = header.find("'" + key + "'"); if (p == std::string::npos) failIo(path + ": header lacks " + key); return header.substr(header.find(':', p) + 1); };
  std::string descr = field("descr");
  size_t q1 = descr.find('\''), q2 = descr.find('\'', q1 + 1);
  descr = descr.substr(q1 + 1, q2 - q1 - 1);
  if (field("fortran_order").find("True") < 8) failIo(path + ": fortran_order arrays are not supported");
  if (descr[0] == '>') failIo(path + ": big-endian arrays are not supported");
  std::string code = descr.substr(1);
  size_t srcSize = std::stoul(code.substr(1));
  std::vector<char> raw(numel * srcSize);
  f.read(raw.data(), (std::streamsize)raw.size());
  if ((size_t)f.gcount() != raw.size()) failIo(path + ": holds fewer than " + std::to_string(numel) + " elements");
  size_t dstSize = (size_t)dtypeSize(want);
  auto same = [&](const char* c) { return code == c; };
  bool direct = (want == DType::F32 && same("f4")) || (want == DType::BF16 && (same("u2") || same("i2"))) || (want == DType::F16 && same("f2")) ||
                (want == DType::I64 && same("i8")) || (want == DType::I32 && same("i4")) || (want == DType::I1 && same("b1")) ||
                (want == DType::F64 && same("f8")) || (want == DType::I8 && (same("i1") || same("u1"))) || (want == DType::I16 && same("i2"));
  if (direct) return raw;
  std::vector<char> out(numel * dstSize);
  for (size_t i = 0; i < numel; ++i) {
    double v;
    if (same("f4")) { float x; memcpy(&x, &raw[i * 4], 4); v = x; }
    else if (same("f8")) { memcpy(&v, &raw[i * 8], 8); }
    else if (same("i8")) { int64_t x; memcpy(&x, &raw[i * 8], 8); v = (double)x; }
    else if (same("i4")) { int32_t x; memcpy(&x, &raw[i * 4], 4); v = x; }
    else failIo(path + ": cannot convert dtype " + descr + " to " + dtypeName(want));
    if (want == DType::F32) { float x = (float)v; memcpy(&out[i * 4], &x, 4); }
    else if (want == DType::BF16) { uint16_t x = f32ToBf16((float)v); memcpy(&out[i * 2], &x, 2); }
    else if (want == DType::I64) { int64_t x = (int64_t)v; memcpy(&out[i * 8], &x, 8); }
    else failIo(path + ": cannot convert dtype " + descr + " to " + dtypeName(want));
  }
  return out;
}

struct RView { int buf; long long off; int rank; long long shape[6], strides[6]; int dtype; };

// A plan step resolved for one symbol binding: the kernel's parameter block is filled once, only the
// pointers (which depend on where the caller's tensors and the arena are) are patched per call.
struct PtrPatch { void** slot; int buf; long long byteOff; };
enum StepKind { kGemm, kConv, kPool, kReduce, kSoftmax, kLayerNorm, kGather, kEltwise, kNchw2Nhwc, kAttention };
struct RStep {
  const Step* step;
  std::vector<std::pair<std::string, RView>> views;
  const RView* view(const char* n) const { for (auto& v : views) if (v.first == n) return &v.second; return nullptr; }
  int kind = -1;
  LlcGemmParams gemm{}; LlcConvParams conv{}; LlcPoolParams pool{}; LlcEltwiseParams elt{}; LlcAttentionParams attn{};
  std::string prog;
  void* sp[4] = {nullptr, nullptr, nullptr, nullptr};   // pointer operands of the row kernels
  int sdt[3] = {0, 0, 0}; long long sd[3] = {0, 0, 0}; int sop = 0; float seps = 0.f;
  long long wide[4] = {0, 0, 0, 0};             // nchw2nhwc with a halo: left columns, total columns, h, w
  std::vector<PtrPatch> patches;
  RStep() {}
  RStep(const RStep&) = delete;             // patches point into this object
  RStep& operator=(const RStep&) = delete;
};

struct Binding {
  std::map<std::string, int64_t> env;
  std::vector<size_t> bufBytes, arenaOffset;   // per buffer
  size_t arenaBytes = 0;
  std::vector<std::unique_ptr<RStep>> steps;
  std::vector<std::vector<int64_t>> inShapes, outShapes;
  // CUDA-graph replay of the step list for callers that come back with the same device pointers (a serving loop):
  // the second call with one set of pointers is captured, later ones are a single graph launch.
  struct GraphSlot { std::vector<const void*> key; cudaGraphExec_t exec = nullptr; int64_t launches = 0; };
  std::vector<GraphSlot> graphs;
  std::vector<std::pair<std::vector<const void*>, int>> seen;   // pointer sets met lately, with how often
  bool graphsBroken = false;
  int captures = 0;                         // bounded, so that a caller with ever-new addresses stops paying for captures
  ~Binding() { for (auto& g : graphs) if (g.exec) cudaGraphExecDestroy(g.exec); }
};

std::vector<int64_t> ints(const std::string& s) {
  std::vector<int64_t> o; std::stringstream ss(s); std::string t;
  while (std::getline(ss, t, ',')) o.push_back(std::stoll(t));
  return o;
}

}  // namespace
}  // namespace llc

using namespace llc;

struct LlcExec {
  Plan plan;
  int device = 0;
  char* staticPool = nullptr;                 // weights + load-time constants
  std::vector<size_t> staticOffset;           // per buffer (weights/consts)
  char* arena = nullptr; size_t arenaCap = 0;
  char* stageIn = nullptr; size_t stageInCap = 0;
  char* stageOut = nullptr; size_t stageOutCap = 0;
  int* badIds = nullptr;
  int* tcWord = nullptr; int* attnWord = nullptr; int* attnBlocksWord = nullptr;   // device addresses of the kernels' status words on `device`
  int* hostStatus = nullptr;                  // page-locked mirror: [tensor-core word, attention word, bad embedding ids, blockwise attention word]
  bool usesTc = false, usesGather = false;    // which of the words this plan's kernels can write
  std::mutex mutex;                           // one call at a time per executor (bindings, arena and staging are shared state)
  char* workspace = nullptr;                  // split-K scratch (counters at the head stay zero between launches)
  static constexpr size_t kWorkspaceBytes = 16u << 20;
  cudaStream_t capStream = nullptr;         // capture happens here, so that the legacy default stream can replay too
  std::map<std::vector<int64_t>, std::unique_ptr<Binding>> bindings;
  int64_t lastLaunches = 0;
  bool loadedFromPool = false;                // the static pool came from a saved file (no weight files read, no load-time kernels)
  std::vector<char*> base;                    // per-buffer device base pointers for the current call

  ~LlcExec() {
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    cudaSetDevice(device);
    if (staticPool) cudaFree(staticPool);
    if (arena) cudaFree(arena);
    if (stageIn) cudaFree(stageIn);
    if (stageOut) cudaFree(stageOut);
    if (badIds) cudaFree(badIds);
    if (hostStatus) cudaFreeHost(hostStatus);
    if (workspace) cudaFree(workspace);
    bindings.clear();                       // graph executables go before the stream they were captured on
    if (capStream) cudaStreamDestroy(capStream);
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
  }

  RView resolve(const View& v, const std::map<std::string, int64_t>& env) const {
    RView r{};
    r.buf = v.buf; r.off = EvalExpr::eval(v.offset.str(), env); r.rank = (int)v.rank(); r.dtype = toLlcDType(v.dtype);
    if (r.rank > 6) failArg("view rank above 6");
    for (int d = 0; d < r.rank; ++d) { r.shape[d] = EvalExpr::eval(v.shape[d].str(), env); r.strides[d] = EvalExpr::eval(v.strides[d].str(), env); }
    return r;
  }
  void* ptr(const RView& v) const { return base[v.buf] + v.off * dtypeSize(plan.buffers[v.buf].dtype); }

  void prepare(RStep& rs);
  int launch(RStep& rs, cudaStream_t st);
  Binding& bind(const int64_t* symbols, int nsym, const LlcTensor* in, int nin);
  void queueStatusRead(cudaStream_t st);
  void raiseOnStatus(cudaStream_t st);
  void runSteps(std::vector<std::unique_ptr<RStep>>& steps, cudaStream_t st);
};

// Fills the parameter block of one plan step (everything except the pointers).
void LlcExec::prepare(RStep& rs) {
  const Step& s = *rs.step;
  auto need = [&](const char* n) -> const RView& { const RView* v = rs.view(n); if (!v) throw std::runtime_error(std::string("llc internal: step '") + s.kernel + "' lacks operand " + n); return *v; };
  auto actOf = [&]() { std::string a = s.param("act", "none"); return a == "relu" ? LLC_ACT_RELU : a == "gelu" ? LLC_ACT_GELU : LLC_ACT_NONE; };
  auto precOf = [&]() { std::string p = s.param("prec", "fp32"); return p == "tf32" ? LLC_PREC_TF32 : p == "tf32x3" ? LLC_PREC_TF32X3 : p == "bf16" ? LLC_PREC_BF16 : LLC_PREC_FP32; };
  auto patch = [&](const void* slot, const RView& v) {
    rs.patches.push_back({reinterpret_cast<void**>(const_cast<void*>(slot)), v.buf, v.off * dtypeSize(plan.buffers[v.buf].dtype)});
  };
  if (s.kernel == "gemm") {
    rs.kind = kGemm;
    const RView &a = need("a"), &b = need("b"), &o = need("out");
    LlcGemmParams& p = rs.gemm;
    patch(&p.a, a); patch(&p.b, b); patch(&p.out, o);
    p.in_dtype = a.dtype; p.out_dtype = o.dtype; p.precision = precOf();
    p.b0 = o.shape[0]; p.b1 = o.shape[1]; p.m = o.shape[2]; p.n = o.shape[3]; p.k = a.shape[3];
    p.a_s0 = a.strides[0]; p.a_s1 = a.strides[1]; p.a_sm = a.strides[2];
    p.b_s0 = b.strides[0]; p.b_s1 = b.strides[1]; p.b_sk = b.strides[2]; p.b_sn = b.strides[3];
    if (b.shape[2] == 1 && p.b_sn != 1) p.b_sk = 1;   // k == 1: either operand order is unit-stride
    p.o_s0 = o.strides[0]; p.o_s1 = o.strides[1]; p.o_sm = o.strides[2];
    if (a.shape[3] != 1 && a.strides[3] != 1) failArg("gemm A operand must have unit stride along k");
    if (o.strides[3] != 1 && o.shape[3] != 1) failArg("gemm output must have unit stride along n");
    if (const RView* v = rs.view("scale")) patch(&p.scale, *v);
    if (const RView* v = rs.view("shift")) patch(&p.shift, *v);
    if (const RView* v = rs.view("res")) { patch(&p.res, *v); p.res_dtype = v->dtype; p.r_s0 = v->strides[0]; p.r_s1 = v->strides[1]; p.r_sm = v->strides[2]; p.r_sn = v->strides[3]; }
    p.alpha = std::stof(s.param("alpha", "1")); p.act = actOf();
    p.workspace = workspace; p.workspace_bytes = (int64_t)kWorkspaceBytes;
    if (const RView* v = rs.view("b_lo")) {
      if (v->strides[0] != b.strides[0] || v->strides[1] != b.strides[1] || v->strides[2] != b.strides[2] || v->strides[3] != b.strides[3]) failArg("gemm b_lo must be laid out like b");
      patch(&p.b_lo, *v);
    }
  } else if (s.kernel == "attention") {
    rs.kind = kAttention;
    const RView &q = need("q"), &k = need("k"), &v = need("v"), &o = need("out");   // q, out [b0,b1,M,D]; k [b0,b1,D,N]; v [b0,b1,N,D]
    LlcAttentionParams& p = rs.attn;
    patch(&p.q, q); patch(&p.k, k); patch(&p.v, v); patch(&p.out, o);
    if (q.dtype != k.dtype || q.dtype != v.dtype || q.dtype != o.dtype) failArg("attention operand types differ");
    p.dtype = q.dtype;
    p.b0 = o.shape[0]; p.b1 = o.shape[1]; p.m = o.shape[2]; p.d = o.shape[3]; p.n = k.shape[3];
    if (q.strides[3] != 1 || k.strides[2] != 1 || v.strides[3] != 1 || o.strides[3] != 1) failArg("attention operands must have unit stride along the head dim");
    auto bs = [](const RView& t, int d) { return t.shape[d] == 1 ? 0 : t.strides[d]; };
    p.q_s0 = bs(q, 0); p.q_s1 = bs(q, 1); p.q_sm = q.strides[2];
    p.k_s0 = bs(k, 0); p.k_s1 = bs(k, 1); p.k_sn = k.strides[3];
    p.v_s0 = bs(v, 0); p.v_s1 = bs(v, 1); p.v_sn = v.strides[2];
    p.o_s0 = o.strides[0]; p.o_s1 = o.strides[1]; p.o_sm = o.strides[2];
    if (const RView* mk = rs.view("mask")) {
      patch(&p.mask, *mk); p.mask_dtype = mk->dtype;
      if (mk->strides[3] != 1 && mk->shape[3] != 1) failArg("attention mask must have unit stride along the keys");
      p.mask_s0 = mk->strides[0]; p.mask_s1 = mk->strides[1]; p.mask_sm = mk->strides[2];
    }
    p.scale = std::stof(s.param("scale", "1"));
  } else if (s.kernel == "conv") {
    rs.kind = kConv;
    const RView &x = need("x"), &w = need("w"), &o = need("out");
    LlcConvParams& p = rs.conv;
    patch(&p.x, x); patch(&p.w, w); patch(&p.out, o);
    p.in_dtype = x.dtype; p.out_dtype = o.dtype; p.precision = precOf();
    p.n = x.shape[0]; p.c = x.shape[1]; p.h = x.shape[2]; p.w_in = x.shape[3];
    p.f = w.shape[0]; p.kh = w.shape[1]; p.kw = w.shape[2]; p.oh = o.shape[2]; p.ow = o.shape[3];
    auto st2 = ints(s.param("stride", "1,1")), pd = ints(s.param("pad", "0,0,0,0")), dl = ints(s.param("dil", "1,1"));
    p.stride_h = (int)st2[0]; p.stride_w = (int)st2[1]; p.pad_h = (int)pd[0]; p.pad_w = (int)pd[1]; p.dil_h = (int)dl[0]; p.dil_w = (int)dl[1];
    if (const RView* v = rs.view("scale")) patch(&p.scale, *v);
    if (const RView* v = rs.view("shift")) patch(&p.shift, *v);
    if (const RView* v = rs.view("res")) { patch(&p.res, *v); p.res_dtype = v->dtype; }
    if (const RView* v = rs.view("w_lo")) patch(&p.w_lo, *v);
    p.workspace = workspace; p.workspace_bytes = (int64_t)kWorkspaceBytes;
    // x is the logical [N, C, H, W] view of channel-last storage: anything but the dense strides is passed on
    if (x.strides[1] != 1 && x.shape[1] != 1) failArg("conv input must have unit stride along the channels");
    if (!(x.strides[3] == p.c && x.strides[2] == p.w_in * p.c && (x.strides[0] == p.h * p.w_in * p.c || p.n == 1))) {
      p.x_sn = x.strides[0]; p.x_sh = x.strides[2]; p.x_sw = x.strides[3];
    }
    p.alpha = std::stof(s.param("alpha", "1")); p.act = actOf();
  } else if (s.kernel == "maxpool") {
    rs.kind = kPool;
    const RView &x = need("x"), &o = need("out");
    LlcPoolParams& p = rs.pool;
    patch(&p.x, x); patch(&p.out, o); p.in_dtype = x.dtype; p.out_dtype = o.dtype;
    p.n = x.shape[0]; p.c = x.shape[1]; p.h = x.shape[2]; p.w = x.shape[3]; p.oh = o.shape[2]; p.ow = o.shape[3];
    auto k = ints(s.param("kernel")), st2 = ints(s.param("stride", "1,1")), pd = ints(s.param("pad", "0,0,0,0")), dl = ints(s.param("dil", "1,1"));
    p.kh = (int)k[0]; p.kw = (int)k[1]; p.stride_h = (int)st2[0]; p.stride_w = (int)st2[1]; p.pad_h = (int)pd[0]; p.pad_w = (int)pd[1]; p.dil_h = (int)dl[0]; p.dil_w = (int)dl[1];
  } else if (s.kernel == "reduce") {
    rs.kind = kReduce;
    const RView &x = need("x"), &o = need("out");
    std::string op = s.param("op", "sum");
    rs.sop = op == "max" ? 1 : op == "min" ? 2 : op == "mean" ? 3 : 0;
    patch(&rs.sp[0], x); patch(&rs.sp[1], o);
    rs.sdt[0] = x.dtype; rs.sdt[1] = o.dtype; rs.sd[0] = x.shape[0]; rs.sd[1] = x.shape[1]; rs.sd[2] = x.shape[2];
  } else if (s.kernel == "softmax") {
    rs.kind = kSoftmax;
    const RView &x = need("x"), &o = need("out");
    patch(&rs.sp[0], x); patch(&rs.sp[1], o);
    rs.sdt[0] = x.dtype; rs.sdt[1] = o.dtype; rs.sd[0] = x.shape[0]; rs.sd[1] = x.shape[1];
  } else if (s.kernel == "layernorm") {
    rs.kind = kLayerNorm;
    const RView &x = need("x"), &g = need("gamma"), &b = need("beta"), &o = need("out");
    if (g.dtype != b.dtype) failArg("layernorm scale and bias types differ");
    patch(&rs.sp[0], x); patch(&rs.sp[1], g); patch(&rs.sp[2], b); patch(&rs.sp[3], o);
    rs.sdt[0] = x.dtype; rs.sdt[1] = g.dtype; rs.sdt[2] = o.dtype; rs.sd[0] = x.shape[0]; rs.sd[1] = x.shape[1];
    rs.seps = std::stof(s.param("eps", "1e-5"));
  } else if (s.kernel == "gather") {
    rs.kind = kGather;
    const RView &t = need("table"), &ids = need("ids"), &o = need("out");
    if (ids.dtype != LLC_INT64) failArg("gather indices must be int64");
    patch(&rs.sp[0], t); patch(&rs.sp[1], ids); patch(&rs.sp[2], o);
    rs.sdt[0] = t.dtype; rs.sdt[1] = o.dtype; rs.sd[0] = o.shape[0]; rs.sd[1] = o.shape[1]; rs.sd[2] = t.shape[0];
  } else if (s.kernel == "nchw2nhwc") {
    rs.kind = kNchw2Nhwc;
    const RView &x = need("x"), &o = need("out");      // both logical [N, C, H, W]
    if (x.dtype != o.dtype) failArg("nchw2nhwc input and output types differ");
    patch(&rs.sp[0], x); patch(&rs.sp[1], o);
    rs.sdt[0] = x.dtype; rs.sd[0] = x.shape[0]; rs.sd[1] = x.shape[1]; rs.sd[2] = x.shape[2] * x.shape[3];
    rs.sop = (int)o.shape[1];
    // rows widened by a zero halo ("wide" = left columns, total columns): the out view is then the whole widened buffer
    rs.wide[0] = rs.wide[1] = 0;
    if (!s.param("wide", "").empty()) {
      auto wl = ints(s.param("wide"));
      rs.wide[0] = wl[0]; rs.wide[1] = wl[1]; rs.wide[2] = x.shape[2]; rs.wide[3] = x.shape[3];
    }
  } else if (s.kernel == "eltwise") {
    rs.kind = kEltwise;
    const RView& o = need("out");
    LlcEltwiseParams& p = rs.elt;
    patch(&p.out, o); p.out_dtype = o.dtype; p.rank = o.rank;
    for (int d = 0; d < o.rank; ++d) { p.shape[d] = o.shape[d]; p.out_strides[d] = o.strides[d]; }
    rs.prog = s.param("prog");
    p.prog = rs.prog.c_str();
    for (int k = 0; k < 8; ++k) {
      const RView* v = rs.view(("in" + std::to_string(k)).c_str());
      if (!v) break;
      patch(&p.in[k].data, *v); p.in[k].dtype = v->dtype;
      for (int d = 0; d < v->rank; ++d) p.in[k].strides[d] = v->strides[d];
      p.n_in = k + 1;
    }
  } else {
    throw std::runtime_error("llc internal: unknown kernel '" + s.kernel + "' in plan");
  }
}

// One kernel call of the plan: patch the pointers for this call, launch.
int LlcExec::launch(RStep& rs, cudaStream_t st) {
  if (rs.kind < 0) prepare(rs);
  for (auto& pp : rs.patches) *pp.slot = base[pp.buf] + pp.byteOff;
  switch (rs.kind) {
    case kGemm: return llc_cuda_gemm(&rs.gemm, st);
    case kConv: return llc_cuda_conv2d(&rs.conv, st);
    case kAttention: return llc_cuda_attention(&rs.attn, st);
    case kPool: return llc_cuda_maxpool2d(&rs.pool, st);
    case kReduce: return llc_cuda_reduce(rs.sp[0], rs.sp[1], rs.sdt[0], rs.sdt[1], rs.sd[0], rs.sd[1], rs.sd[2], rs.sop, st);
    case kSoftmax: return llc_cuda_softmax(rs.sp[0], rs.sp[1], rs.sdt[0], rs.sdt[1], rs.sd[0], rs.sd[1], st);
    case kLayerNorm: return llc_cuda_layernorm(rs.sp[0], rs.sp[1], rs.sp[2], rs.sp[3], rs.sdt[0], rs.sdt[1], rs.sdt[2], rs.sd[0], rs.sd[1], rs.seps, st);
    case kGather: return llc_cuda_gather(rs.sp[0], (const int64_t*)rs.sp[1], rs.sp[2], rs.sdt[0], rs.sdt[1], rs.sd[0], rs.sd[1], rs.sd[2], badIds, st);
    case kEltwise: return llc_cuda_eltwise(&rs.elt, st);
    case kNchw2Nhwc:
      if (rs.wide[1] > 0) return llc_cuda_nchw_to_nhwc_wide(rs.sp[0], rs.sp[1], rs.sdt[0], rs.sd[0], rs.sd[1], rs.wide[2], rs.wide[3], rs.sop, rs.wide[0], rs.wide[1], st);
      return llc_cuda_nchw_to_nhwc(rs.sp[0], rs.sp[1], rs.sdt[0], rs.sd[0], rs.sd[1], rs.sd[2], rs.sop, st);
  }
  throw std::runtime_error("llc internal: unprepared plan step");
}

void LlcExec::runSteps(std::vector<std::unique_ptr<RStep>>& steps, cudaStream_t st) {
  for (auto& rs : steps) {
    int rc = launch(*rs, st);
    if (rc != LLC_OK) throw std::runtime_error(std::string(llc_last_error()));
    ++lastLaunches;
  }
}

// The kernels report failures they cannot raise themselves through three device words: the tensor-core GEMM /
// convolution and the attention kernel record a bounded wait that gave up, the embedding gather counts ids outside
// its table (those rows are written as zeros).  queueStatusRead copies the words this plan can write into page-locked
// host memory behind the work already on `st`; raiseOnStatus, called once the stream has been synchronised, clears
// whatever is set and throws, so a broken launch or a bad id is an error of the call instead of a wrong result.
void LlcExec::queueStatusRead(cudaStream_t st) {
  hostStatus[0] = hostStatus[1] = hostStatus[2] = hostStatus[3] = 0;
  if (usesTc && attnBlocksWord) cudaOk(cudaMemcpyAsync(&hostStatus[3], attnBlocksWord, sizeof(int), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(status)");
  if (usesTc && tcWord) cudaOk(cudaMemcpyAsync(&hostStatus[0], tcWord, sizeof(int), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(status)");
  if (usesTc && attnWord) cudaOk(cudaMemcpyAsync(&hostStatus[1], attnWord, sizeof(int), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(status)");
  if (usesGather) cudaOk(cudaMemcpyAsync(&hostStatus[2], badIds, sizeof(int), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(status)");
}
void LlcExec::raiseOnStatus(cudaStream_t st) {
  const int tc = hostStatus[0], at = hostStatus[1] ? hostStatus[1] : hostStatus[3], bad = hostStatus[2];
  if (!tc && !at && !bad) return;
  if (tc) cudaMemsetAsync(tcWord, 0, sizeof(int), st);
  if (hostStatus[1]) cudaMemsetAsync(attnWord, 0, sizeof(int), st);
  if (hostStatus[3]) cudaMemsetAsync(attnBlocksWord, 0, sizeof(int), st);
  if (bad) cudaMemsetAsync(badIds, 0, sizeof(int), st);
  cudaStreamSynchronize(st);
  hostStatus[0] = hostStatus[1] = hostStatus[2] = hostStatus[3] = 0;
  if (bad) failArg(std::to_string(bad) + " embedding indices lie outside their table (those rows were written as zeros)");
  throw std::runtime_error("llc cuda: a tensor-core kernel gave up on a bounded wait (status " + std::to_string(tc ? tc : at) +
                           (tc ? ", GEMM / convolution" : ", attention") + "); the results of this call are invalid");
}

Binding& LlcExec::bind(const int64_t* symbols, int nsym, const LlcTensor* in, int nin) {
  if (nin != (int)plan.inputs.size()) failArg("expected " + std::to_string(plan.inputs.size()) + " input tensors, got " + std::to_string(nin));
  if (nsym != plan.numSymbolArgs && nsym != 0) failArg("expected " + std::to_string(plan.numSymbolArgs) + " symbol values, got " + std::to_string(nsym));
  std::map<std::string, int64_t> env;
  for (auto& sb : plan.symbols) {
    int64_t v;
    if (sb.symbolArg >= 0) { if (nsym == 0) continue; v = symbols[sb.symbolArg]; }
    else {
      if (sb.input >= nin || sb.dim >= in[sb.input].rank) failArg("input " + std::to_string(sb.input) + " has too few dims for symbol " + sb.name);
      v = in[sb.input].sizes[sb.dim];
    }
    auto it = env.find(sb.name);
    if (it == env.end()) env[sb.name] = v;
    else if (it->second != v) failArg("shape symbol " + sb.name + " bound to both " + std::to_string(it->second) + " and " + std::to_string(v));
  }
  std::vector<int64_t> key;
  for (auto& kv : env) key.push_back(kv.second);
  auto it = bindings.find(key);
  if (it != bindings.end()) return *it->second;

  std::unique_ptr<Binding> b(new Binding());
  b->env = env;
  size_t nb = plan.buffers.size();
  b->bufBytes.assign(nb, 0); b->arenaOffset.assign(nb, 0);
  for (size_t i = 0; i < nb; ++i) {
    int64_t n = EvalExpr::eval(plan.buffers[i].numel.str(), env);
    if (n < 0) failArg("negative buffer extent for the given symbols");
    b->bufBytes[i] = (size_t)n * dtypeSize(plan.buffers[i].dtype);
  }
  for (auto& io : plan.inputs) { std::vector<int64_t> s; for (auto& e : io.shape) s.push_back(EvalExpr::eval(e.str(), env)); b->inShapes.push_back(s); }
  for (auto& io : plan.outputs) { std::vector<int64_t> s; for (auto& e : io.shape) s.push_back(EvalExpr::eval(e.str(), env)); b->outShapes.push_back(s); }
  // resolve run steps and buffer lifetimes
  std::vector<int> firstUse(nb, -1), lastUse(nb, -1);
  for (auto& s : plan.steps) {
    if (s.init) continue;
    std::unique_ptr<RStep> rs(new RStep()); rs->step = &s;
    for (auto& v : s.views) {
      rs->views.emplace_back(v.first, resolve(v.second, env));
      int id = v.second.buf, idx = (int)b->steps.size();
      if (firstUse[id] < 0) firstUse[id] = idx;
      lastUse[id] = idx;
    }
    prepare(*rs);
    b->steps.push_back(std::move(rs));
  }
  // first-fit packing of temporaries by lifetime
  std::vector<int> temps;
  for (size_t i = 0; i < nb; ++i) if (plan.buffers[i].kind == BufferDecl::Temp && firstUse[i] >= 0) temps.push_back((int)i);
  std::sort(temps.begin(), temps.end(), [&](int x, int y) { return firstUse[x] != firstUse[y] ? firstUse[x] < firstUse[y] : b->bufBytes[x] > b->bufBytes[y]; });
  std::vector<int> placed;
  for (int t : temps) {
    size_t size = align256(std::max<size_t>(b->bufBytes[t], 1));
    std::vector<std::pair<size_t, size_t>> busy;
    for (int c : placed) if (!(lastUse[c] < firstUse[t] || lastUse[t] < firstUse[c])) busy.emplace_back(b->arenaOffset[c], align256(std::max<size_t>(b->bufBytes[c], 1)));
    std::sort(busy.begin(), busy.end());
    size_t off = 0;
    for (auto& iv : busy) { if (off + size <= iv.first) break; off = std::max(off, iv.first + iv.second); }
    b->arenaOffset[t] = off;
    b->arenaBytes = std::max(b->arenaBytes, off + size);
    placed.push_back(t);
  }
  Binding& ref = *b;
  bindings[key] = std::move(b);
  return ref;
}

static bool isDenseRowMajor(const LlcTensor& t) {
  int64_t acc = 1;
  for (int d = t.rank - 1; d >= 0; --d) { if (t.sizes[d] != 1 && t.strides && t.strides[d] != acc) return false; acc *= t.sizes[d]; }
  return true;
}

namespace {
// The static pool (weights as uploaded plus everything the load-time kernels derive from them: re-laid-out filters,
// folded batch-norm vectors, the low-order parts of tf32x3 weights) saved beside the weights, so that a later load of
// the same plan with the same weights is one file read and one copy.  The header ties the file to the plan text, the
// pool size and the library build.
struct PoolHeader { char magic[8]; uint64_t planHash, bytes, buildHash; };
const char kPoolMagic[8] = {'L', 'L', 'C', 'P', 'O', 'O', 'L', '1'};
uint64_t buildHash() { return std::hash<std::string>()(std::string(llc_version()) + __DATE__ + __TIME__); }
bool fileExists(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0; }
std::string baseName(const std::string& p) { size_t k = p.find_last_of('/'); return k == std::string::npos ? p : p.substr(k + 1); }
}  // namespace

extern "C" int llc_load(const char* path, int device, LlcExec** out) { return llc_load_from(path, nullptr, device, out); }

extern "C" int llc_load_from(const char* path, const char* weightDirC, int device, LlcExec** out) {
  const std::string weightDir = weightDirC ? weightDirC : "";
  if (!path || !out) return setError(LLC_ERR_ARGUMENT, "null argument");
  std::unique_ptr<LlcExec> ex(new LlcExec());
  try {
    std::ifstream f(path);
    if (!f) failIo(std::string("cannot open plan ") + path);
    std::stringstream ss; ss << f.rdbuf();
    const std::string planText = ss.str();
    ex->plan = parsePlan(planText);
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) throw std::runtime_error("llc cuda: no CUDA device is available (the B200 backend has no CPU fallback)");
    if (device < 0 || device >= count) failArg("device ordinal " + std::to_string(device) + " out of range");
    ex->device = device;
    DeviceGuard guard(device);
    size_t nb = ex->plan.buffers.size();
    ex->staticOffset.assign(nb, 0);
    ex->base.assign(nb, nullptr);
    size_t total = 0;
    std::map<std::string, int64_t> empty;
    std::vector<size_t> bytes(nb, 0);
    for (size_t i = 0; i < nb; ++i) {
      auto& b = ex->plan.buffers[i];
      if (b.kind != BufferDecl::Weight && b.kind != BufferDecl::Const) continue;
      bytes[i] = (size_t)EvalExpr::eval(b.numel.str(), empty) * dtypeSize(b.dtype);
      ex->staticOffset[i] = total; total += align256(std::max<size_t>(bytes[i], 1));
    }
    cudaOk(cudaMalloc(&ex->staticPool, std::max<size_t>(total, 256)), "cudaMalloc(weights)");
    cudaOk(cudaMalloc(&ex->badIds, sizeof(int)), "cudaMalloc(status)");
    cudaOk(cudaMemset(ex->badIds, 0, sizeof(int)), "cudaMemset(status)");
    cudaOk(cudaHostAlloc(reinterpret_cast<void**>(&ex->hostStatus), 4 * sizeof(int), cudaHostAllocDefault), "cudaHostAlloc(status)");
    ex->tcWord = tcStatusAddress(); ex->attnWord = attnStatusAddress(); ex->attnBlocksWord = attnBlocksStatusAddress();
    for (auto& s : ex->plan.steps) {
      if (s.kernel == "gemm" || s.kernel == "conv" || s.kernel == "attention") ex->usesTc = true;
      if (s.kernel == "gather") ex->usesGather = true;
    }
    cudaOk(cudaMalloc(&ex->workspace, LlcExec::kWorkspaceBytes), "cudaMalloc(workspace)");
    cudaOk(cudaMemset(ex->workspace, 0, 4096), "cudaMemset(workspace)");
    // a saved pool for this plan, these weights and this build: one read, one copy, no load-time kernels
    const std::string poolPath = weightDir.empty() ? "" : weightDir + "/pool.bin";
    const PoolHeader wantHeader = [&]() { PoolHeader h{}; memcpy(h.magic, kPoolMagic, 8); h.planHash = std::hash<std::string>()(planText); h.bytes = total; h.buildHash = buildHash(); return h; }();
    bool fromPool = false;
    if (!poolPath.empty() && total > 0) {
      std::ifstream pf(poolPath, std::ios::binary);
      PoolHeader got{};
      if (pf && pf.read(reinterpret_cast<char*>(&got), sizeof got) && memcmp(&got, &wantHeader, sizeof got) == 0) {
        std::vector<char> host(total);
        if (pf.read(host.data(), (std::streamsize)total)) {
          cudaOk(cudaMemcpy(ex->staticPool, host.data(), total, cudaMemcpyHostToDevice), "cudaMemcpy(pool)");
          fromPool = true;
        }
      }
    }
    for (size_t i = 0; i < nb; ++i) {
      auto& b = ex->plan.buffers[i];
      if (b.kind != BufferDecl::Weight && b.kind != BufferDecl::Const) continue;
      ex->base[i] = ex->staticPool + ex->staticOffset[i];
      if (fromPool) continue;
      size_t n = bytes[i] / dtypeSize(b.dtype);
      if (b.kind == BufferDecl::Weight) {
        // with a weight directory the files are looked up there by name (the plan records where the importer put them)
        std::string file = b.file;
        if (!weightDir.empty() && fileExists(weightDir + "/" + baseName(b.file))) file = weightDir + "/" + baseName(b.file);
        std::vector<char> host = readNpy(file, b.dtype, n);
        cudaOk(cudaMemcpy(ex->base[i], host.data(), bytes[i], cudaMemcpyHostToDevice), "cudaMemcpy(weight)");
      } else if (!b.values.empty()) {
        if (b.values.size() != n) failArg("constant buffer value count mismatch");
        std::vector<char> host(bytes[i]);
        for (size_t k = 0; k < n; ++k) {
          double v = b.values[k];
          switch (b.dtype) {
            case DType::F32: { float x = (float)v; memcpy(&host[k * 4], &x, 4); break; }
            case DType::BF16: { uint16_t x = f32ToBf16((float)v); memcpy(&host[k * 2], &x, 2); break; }
            case DType::I64: { int64_t x = (int64_t)v; memcpy(&host[k * 8], &x, 8); break; }
            case DType::I32: { int32_t x = (int32_t)v; memcpy(&host[k * 4], &x, 4); break; }
            case DType::I1: case DType::I8: { host[k] = (char)(int)v; break; }
            default: failArg("unsupported constant element type");
          }
        }
        cudaOk(cudaMemcpy(ex->base[i], host.data(), bytes[i], cudaMemcpyHostToDevice), "cudaMemcpy(constant)");
      }
    }
    // load-time kernels: weight re-layout, folded batch-norm vectors
    std::vector<std::unique_ptr<RStep>> init;
    for (auto& s : ex->plan.steps) {
      if (!s.init) continue;
      std::unique_ptr<RStep> rs(new RStep()); rs->step = &s;
      for (auto& v : s.views) rs->views.emplace_back(v.first, ex->resolve(v.second, empty));
      init.push_back(std::move(rs));
    }
    if (!fromPool) {
      ex->runSteps(init, 0);
      ex->queueStatusRead(0);
      cudaOk(cudaDeviceSynchronize(), "load-time kernels");
      ex->raiseOnStatus(0);
      if (!poolPath.empty() && total > 0) {            // save the pool for the next load (written whole, then renamed)
        std::vector<char> host(total);
        cudaOk(cudaMemcpy(host.data(), ex->staticPool, total, cudaMemcpyDeviceToHost), "cudaMemcpy(pool)");
        const std::string tmp = poolPath + ".tmp" + std::to_string((long long)getpid());
        std::ofstream pf(tmp, std::ios::binary);
        if (pf && pf.write(reinterpret_cast<const char*>(&wantHeader), sizeof wantHeader) && pf.write(host.data(), (std::streamsize)total)) {
          pf.close();
          if (::rename(tmp.c_str(), poolPath.c_str()) != 0) ::unlink(tmp.c_str());
        } else { pf.close(); ::unlink(tmp.c_str()); }
      }
    }
    ex->loadedFromPool = fromPool;
    ex->lastLaunches = 0;
    *out = ex.release();
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

extern "C" int llc_num_inputs(const LlcExec* e) { return e ? (int)e->plan.inputs.size() : -1; }
extern "C" int llc_num_outputs(const LlcExec* e) { return e ? (int)e->plan.outputs.size() : -1; }
extern "C" int llc_num_symbols(const LlcExec* e) { return e ? e->plan.numSymbolArgs : -1; }
extern "C" int64_t llc_last_launch_count(const LlcExec* e) { return e ? e->lastLaunches : -1; }
extern "C" int64_t llc_arena_bytes(const LlcExec* e) { return e ? (int64_t)e->arenaCap : -1; }
extern "C" int llc_loaded_from_pool(const LlcExec* e) { return e ? (e->loadedFromPool ? 1 : 0) : -1; }
extern "C" void llc_free(LlcExec* e) { delete e; }

extern "C" int llc_output_shape(LlcExec* ex, const int64_t* symbols, int nsym, const LlcTensor* in, int nin, int index, int64_t* sizes, int32_t* rank, int32_t* dtype) {
  if (!ex || !sizes || !rank) return setError(LLC_ERR_ARGUMENT, "null argument");
  try {
    std::lock_guard<std::mutex> lock(ex->mutex);
    Binding& b = ex->bind(symbols, nsym, in, nin);
    if (index < 0 || index >= (int)b.outShapes.size()) failArg("output index out of range");
    auto& s = b.outShapes[index];
    if (s.size() > 8) failArg("output rank above 8");
    *rank = (int32_t)s.size();
    for (size_t d = 0; d < s.size(); ++d) sizes[d] = s[d];
    if (dtype) *dtype = toLlcDType(ex->plan.outputs[index].dtype);
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

// Binds symbols, sizes the arena, points every input/output buffer at caller memory (staging host
// tensors through the device) and returns the binding to launch.
static Binding& prepareCall(LlcExec* ex, const int64_t* symbols, int nsym, const LlcTensor* in, int nin, LlcTensor* outs, int nout, cudaStream_t st, bool& anyHostOut) {
  Binding& b = ex->bind(symbols, nsym, in, nin);
  if (nout != (int)ex->plan.outputs.size()) failArg("expected " + std::to_string(ex->plan.outputs.size()) + " output tensors, got " + std::to_string(nout));
  if (b.arenaBytes > ex->arenaCap) {
    cudaOk(cudaStreamSynchronize(st), "cudaStreamSynchronize");
    if (ex->arena) cudaOk(cudaFree(ex->arena), "cudaFree(arena)");
    ex->arena = nullptr; ex->arenaCap = 0;
    cudaOk(cudaMalloc(&ex->arena, b.arenaBytes), "cudaMalloc(arena)");
    ex->arenaCap = b.arenaBytes;
  }
  size_t nb = ex->plan.buffers.size();
  for (size_t i = 0; i < nb; ++i) if (ex->plan.buffers[i].kind == BufferDecl::Temp) ex->base[i] = ex->arena + b.arenaOffset[i];
  // inputs: device tensors are used in place, host tensors are staged
  auto check = [&](const LlcTensor& t, const IoDecl& io, const std::vector<int64_t>& shape, const char* what, int k) {
    if (t.dtype != toLlcDType(io.dtype)) failArg(std::string(what) + " " + std::to_string(k) + " has element type code " + std::to_string(t.dtype) + ", the plan expects " + dtypeName(io.dtype));
    if (t.rank != (int)shape.size() && !(t.rank == 0 && shape.size() == 1 && shape[0] == 1)) failArg(std::string(what) + " " + std::to_string(k) + " has rank " + std::to_string(t.rank) + ", expected " + std::to_string(shape.size()));
    for (int d = 0; d < t.rank; ++d) if (t.sizes[d] != shape[d]) failArg(std::string(what) + " " + std::to_string(k) + " dim " + std::to_string(d) + " is " + std::to_string(t.sizes[d]) + ", expected " + std::to_string(shape[d]));
    if (!isDenseRowMajor(t)) failArg(std::string(what) + " " + std::to_string(k) + " must be contiguous");
    int64_t n = 1; for (auto s : shape) n *= s;
    if (!t.data && n) failArg(std::string(what) + " " + std::to_string(k) + " has a null data pointer");
    if (t.device >= 0 && t.device != ex->device) failArg(std::string(what) + " " + std::to_string(k) + " lives on device " + std::to_string(t.device) + ", the plan is loaded on " + std::to_string(ex->device));
  };
  size_t needIn = 0, needOut = 0;
  for (int k = 0; k < nin; ++k) { check(in[k], ex->plan.inputs[k], b.inShapes[k], "input", k); if (in[k].device < 0) needIn += align256(b.bufBytes[ex->plan.inputs[k].buf]); }
  for (int k = 0; k < nout; ++k) { check(outs[k], ex->plan.outputs[k], b.outShapes[k], "output", k); if (outs[k].device < 0) needOut += align256(b.bufBytes[ex->plan.outputs[k].buf]); }
  auto grow = [&](char*& p, size_t& cap, size_t need) {
    if (need <= cap) return;
    cudaOk(cudaStreamSynchronize(st), "cudaStreamSynchronize");
    if (p) cudaOk(cudaFree(p), "cudaFree(staging)");
    p = nullptr; cap = 0;
    cudaOk(cudaMalloc(&p, need), "cudaMalloc(staging)");
    cap = need;
  };
  grow(ex->stageIn, ex->stageInCap, needIn);
  grow(ex->stageOut, ex->stageOutCap, needOut);
  size_t offIn = 0, offOut = 0;
  for (int k = 0; k < nin; ++k) {
    int buf = ex->plan.inputs[k].buf;
    if (in[k].device >= 0) ex->base[buf] = (char*)in[k].data;
    else {
      ex->base[buf] = ex->stageIn + offIn;
      if (b.bufBytes[buf]) cudaOk(cudaMemcpyAsync(ex->base[buf], in[k].data, b.bufBytes[buf], cudaMemcpyHostToDevice, st), "cudaMemcpyAsync(H2D)");
      offIn += align256(b.bufBytes[buf]);
    }
  }
  anyHostOut = false;
  for (int k = 0; k < nout; ++k) {
    int buf = ex->plan.outputs[k].buf;
    if (outs[k].device >= 0) ex->base[buf] = (char*)outs[k].data;
    else { ex->base[buf] = ex->stageOut + offOut; offOut += align256(b.bufBytes[buf]); anyHostOut = true; }
  }
  return b;
}

static void finishCall(LlcExec* ex, Binding& b, LlcTensor* outs, int nout, cudaStream_t st, bool anyHostOut) {
  if (!anyHostOut) return;
  for (int k = 0; k < nout; ++k) {
    int buf = ex->plan.outputs[k].buf;
    if (outs[k].device < 0 && b.bufBytes[buf]) cudaOk(cudaMemcpyAsync(outs[k].data, ex->base[buf], b.bufBytes[buf], cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(D2H)");
  }
  ex->queueStatusRead(st);                    // the call waits for its results anyway: look at the failure words too
  cudaOk(cudaStreamSynchronize(st), "cudaStreamSynchronize");
  ex->raiseOnStatus(st);
}

// Replays (or, on the second call with the same pointers, captures) the binding's steps as one CUDA graph.  Only for calls whose
// tensors all live on the device, short plans (where launch gaps matter) and streams that are not being captured by the
// caller.  Returns false when the steps still have to be launched one by one.  LLC_CUDA_GRAPHS=0 switches it off.
static bool runThroughGraph(LlcExec* ex, Binding& b, const LlcTensor* in, int nin, LlcTensor* outs, int nout, cudaStream_t st) {
  static const bool enabled = []() { const char* e = getenv("LLC_CUDA_GRAPHS"); return !(e && e[0] == '0'); }();
  if (!enabled || b.graphsBroken || b.steps.size() < 2 || b.steps.size() > 256) return false;
  for (int k = 0; k < nin; ++k) if (in[k].device < 0) return false;
  for (int k = 0; k < nout; ++k) if (outs[k].device < 0) return false;
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) { cudaGetLastError(); return false; }
  std::vector<const void*> key;
  key.push_back(ex->arena); key.push_back(st);
  for (int k = 0; k < nin; ++k) key.push_back(in[k].data);
  for (int k = 0; k < nout; ++k) key.push_back(outs[k].data);
  for (auto& g : b.graphs)
    if (g.key == key) {
      if (cudaGraphLaunch(g.exec, st) != cudaSuccess) { cudaGetLastError(); b.graphsBroken = true; return false; }
      ex->lastLaunches = g.launches;
      return true;
    }
  // a caller that allocates its outputs per call still cycles through a few addresses: count each set on its own
  auto it = std::find_if(b.seen.begin(), b.seen.end(), [&](const std::pair<std::vector<const void*>, int>& e) { return e.first == key; });
  if (it == b.seen.end()) {
    if (b.seen.size() >= 8) b.seen.erase(b.seen.begin());
    b.seen.emplace_back(key, 1);
    return false;
  }
  if (++it->second < 2 || b.captures >= 16) return false;
  b.seen.erase(it);
  ++b.captures;
  // capture: every first-use initialisation (function attributes, driver entry points) happened in the earlier runs
  if (!ex->capStream && cudaStreamCreateWithFlags(&ex->capStream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); b.graphsBroken = true; return false; }
  cudaStream_t cap = ex->capStream;
  if (cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); b.graphsBroken = true; return false; }
  bool ok = true;
  try { ex->lastLaunches = 0; ex->runSteps(b.steps, cap); } catch (const std::exception&) { ok = false; }
  cudaGraph_t graph = nullptr;
  if (cudaStreamEndCapture(cap, &graph) != cudaSuccess || !graph) ok = false;
  cudaGraphExec_t exec = nullptr;
  if (ok && cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) ok = false;
  if (graph) cudaGraphDestroy(graph);
  if (!ok) { cudaGetLastError(); if (exec) cudaGraphExecDestroy(exec); b.graphsBroken = true; ex->lastLaunches = 0; return false; }
  if (b.graphs.size() >= 4) { cudaGraphExecDestroy(b.graphs.front().exec); b.graphs.erase(b.graphs.begin()); }
  Binding::GraphSlot slot; slot.key = key; slot.exec = exec; slot.launches = ex->lastLaunches;
  b.graphs.push_back(slot);
  if (cudaGraphLaunch(exec, st) != cudaSuccess) { cudaGetLastError(); b.graphsBroken = true; b.graphs.pop_back(); cudaGraphExecDestroy(exec); ex->lastLaunches = 0; return false; }
  return true;
}

extern "C" int llc_run(LlcExec* ex, const int64_t* symbols, int nsym, const LlcTensor* in, int nin, LlcTensor* outs, int nout, void* stream) {
  if (!ex || (nin > 0 && !in) || (nout > 0 && !outs)) return setError(LLC_ERR_ARGUMENT, "null argument");
  try {
    cudaStream_t st = (cudaStream_t)stream;
    bool anyHostOut = false;
    std::lock_guard<std::mutex> lock(ex->mutex);
    DeviceGuard guard(ex->device);
    Binding& b = prepareCall(ex, symbols, nsym, in, nin, outs, nout, st, anyHostOut);
    ex->lastLaunches = 0;
    if (!runThroughGraph(ex, b, in, nin, outs, nout, st)) ex->runSteps(b.steps, st);
    finishCall(ex, b, outs, nout, st, anyHostOut);
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

extern "C" int llc_status(LlcExec* ex, int32_t* words) {
  if (!ex) return setError(LLC_ERR_ARGUMENT, "null argument");
  try {
    std::lock_guard<std::mutex> lock(ex->mutex);
    DeviceGuard guard(ex->device);
    cudaOk(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    ex->queueStatusRead(0);
    cudaOk(cudaStreamSynchronize(0), "cudaStreamSynchronize");
    if (words) { words[0] = ex->hostStatus[0]; words[1] = ex->hostStatus[1] ? ex->hostStatus[1] : ex->hostStatus[3]; words[2] = ex->hostStatus[2]; }
    ex->raiseOnStatus(0);
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

// Algorithmic work of one step: FLOPs of the contraction, bytes = every operand element once.
static void stepWork(const RStep& rs, double& flops, double& bytes) {
  flops = 0; bytes = 0;
  for (auto& v : rs.views) {
    double n = 1;
    for (int d = 0; d < v.second.rank; ++d) if (v.second.strides[d] != 0 || v.second.shape[d] == 1) n *= (double)v.second.shape[d];
    int eb = v.second.dtype == LLC_FLOAT32 || v.second.dtype == LLC_INT32 ? 4 : v.second.dtype == LLC_BFLOAT16 || v.second.dtype == LLC_FLOAT16 || v.second.dtype == LLC_INT16 ? 2
           : v.second.dtype == LLC_INT64 || v.second.dtype == LLC_FLOAT64 ? 8 : 1;
    bytes += n * eb;
  }
  const std::string& k = rs.step->kernel;
  if (k == "gemm") { const RView* a = rs.view("a"); const RView* o = rs.view("out"); flops = 2.0 * o->shape[0] * o->shape[1] * o->shape[2] * o->shape[3] * a->shape[3]; }
  if (k == "attention") { const RView* kk = rs.view("k"); const RView* o = rs.view("out"); flops = 4.0 * o->shape[0] * o->shape[1] * o->shape[2] * o->shape[3] * kk->shape[3]; }
  if (k == "conv") {
    // the contraction length as the model wrote it ("kalg"), not the packed weight view, which may hold padded channels
    const RView* w = rs.view("w"); const RView* o = rs.view("out");
    const std::string kalg = rs.step->param("kalg", "");
    const double kLen = kalg.empty() ? (double)w->shape[1] * w->shape[2] * w->shape[3] : std::stod(kalg);
    flops = 2.0 * o->shape[0] * o->shape[2] * o->shape[3] * w->shape[0] * kLen;
  }
}

extern "C" int llc_profile(LlcExec* ex, const int64_t* symbols, int nsym, const LlcTensor* in, int nin, LlcTensor* outs, int nout, int reps, void* stream,
                           char* report, size_t reportLen) {
  if (!ex || !report || reps <= 0) return setError(LLC_ERR_ARGUMENT, "null argument");
  try {
    cudaStream_t st = (cudaStream_t)stream;
    bool anyHostOut = false;
    std::lock_guard<std::mutex> lock(ex->mutex);
    DeviceGuard guard(ex->device);
    Binding& b = prepareCall(ex, symbols, nsym, in, nin, outs, nout, st, anyHostOut);
    size_t n = b.steps.size();
    std::vector<cudaEvent_t> ev(2 * n);
    for (auto& e : ev) cudaOk(cudaEventCreate(&e), "cudaEventCreate");
    std::vector<double> ms(n, 0.0);
    for (int r = 0; r < reps + 1; ++r) {   // the first pass is a warm-up
      for (size_t i = 0; i < n; ++i) {
        cudaOk(cudaEventRecord(ev[2 * i], st), "cudaEventRecord");
        int rc = ex->launch(*b.steps[i], st);
        if (rc != LLC_OK) throw std::runtime_error(std::string(llc_last_error()));
        cudaOk(cudaEventRecord(ev[2 * i + 1], st), "cudaEventRecord");
      }
      cudaOk(cudaStreamSynchronize(st), "cudaStreamSynchronize");
      if (r == 0) continue;
      for (size_t i = 0; i < n; ++i) { float t = 0; cudaOk(cudaEventElapsedTime(&t, ev[2 * i], ev[2 * i + 1]), "cudaEventElapsedTime"); ms[i] += t; }
    }
    for (auto& e : ev) cudaEventDestroy(e);
    finishCall(ex, b, outs, nout, st, anyHostOut);
    if (!anyHostOut) { ex->queueStatusRead(st); cudaOk(cudaStreamSynchronize(st), "cudaStreamSynchronize"); ex->raiseOnStatus(st); }
    struct Agg { int launches = 0; double ms = 0, flops = 0, bytes = 0; };
    std::map<std::string, Agg> agg;
    std::ostringstream o;
    o.precision(9);
    for (size_t i = 0; i < n; ++i) {
      double f, by; stepWork(*b.steps[i], f, by);
      Agg& a = agg[b.steps[i]->step->kernel];
      a.launches += 1; a.ms += ms[i] / reps; a.flops += f; a.bytes += by;
      o << "step " << i << " " << b.steps[i]->step->kernel << " " << ms[i] / reps << " " << f << " " << by << "\n";
    }
    for (auto& kv : agg) o << "kernel " << kv.first << " " << kv.second.launches << " " << kv.second.ms << " " << kv.second.flops << " " << kv.second.bytes << "\n";
    std::string text = o.str();
    if (text.size() + 1 > reportLen) text.resize(reportLen ? reportLen - 1 : 0);
    memcpy(report, text.c_str(), text.size() + 1);
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

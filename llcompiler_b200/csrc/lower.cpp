// The GPU pipeline: LLH module -> kernel plan.
//
// This replaces everything the reference does below the LLH level
// (src/Pipeline/TransformPipeline.cpp:100-226: LLH -> StableHLO -> linalg ->
// affine -> LLVM).  Ops are visited in program order.  Every tensor value is
// one of: a strided view onto a buffer, a lazy elementwise expression tree, the
// not-yet-emitted result of a GEMM/conv call that can still absorb elementwise
// consumers into its epilogue, or a reshape that could not be expressed on
// strides.  Data movement ops (reshape, transpose, broadcast_to, slice,
// extract) only rewrite strides; layout changes (the reference's
// transform-layout pass, src/Dialect/LLH/Transforms/TransformLayout.cpp:141-198)
// fall out of the same mechanism because an NHWC buffer is an NCHW-shaped view
// with permuted strides.  Shapes are symbolic expressions following the
// reference's inference rules (src/Dialect/LLH/IR/LLHinfersymbolShape.cpp:
// 114-212 broadcast/reduce, :257-292 and :640-672 conv/pool, :531-585 matmul).
#include <cmath>
#include <cstring>
#include <functional>
#include <set>
#include <sstream>

#include "plan.h"

namespace llc {
namespace {

[[noreturn]] void fail(const std::string& m) { throw std::runtime_error("llc compile: " + m); }

struct ENode {
  enum Kind { Leaf, Const, Op } kind = Const;
  std::string op;
  int a = -1, b = -1, c = -1;
  View leaf;
  bool leafConst = false;
  double cst = 0;
};

struct TV {
  enum Kind { None, Scalar, ViewK, Lazy, Pending, Deferred, AttnProb } kind = None;
  Expr scalar;                 // Scalar (i64)
  double fscalar = 0; bool isFloatScalar = false;
  DType dtype = DType::F32;
  std::vector<Expr> shape;
  View view;                   // ViewK / Pending (logical view onto the result buffer) / Deferred (source)
  int root = -1;               // Lazy
  int pending = -1;            // Pending
  int attn = -1;               // AttnProb: softmax of a not-yet-emitted score GEMM (index into Lowering::attn); view = where the
                               // probabilities go if some consumer other than the second GEMM needs them
  bool isConst = false;        // computable at load time
};

// softmax(Q K^T) waiting for its consumer: a GEMM with V turns the three ops into one attention step, anything else
// materialises the scores and the probabilities the ordinary way.
struct AttnCand { int pending = -1; bool materialized = false; };

struct PendingK {
  Step step;
  int buf = -1;
  View nativeOut;
  int chanDim = -1;            // channel dim in nativeOut
  int stage = 0;               // 0 affine, 1 residual added, 2 activation applied
  int scaleRoot = -1, shiftRoot = -1;
  bool hasRes = false; View res;
  std::string act = "none";
  bool emitted = false;
};

std::vector<int64_t> intArray(const Op* op, const char* name, std::vector<int64_t> dflt = {}) {
  const Attr* a = op->attr(name);
  if (!a) return dflt;
  if (a->kind == Attr::IntArray) return a->ints;
  if (a->kind == Attr::Dense) return a->ints;
  if (a->kind == Attr::Array) { std::vector<int64_t> o; for (auto& e : a->elems) o.push_back(e.i); return o; }
  fail(std::string("attribute '") + name + "' of " + op->name + " is not an integer array");
}

Expr numelOf(const std::vector<Expr>& shape) { Expr n(1); for (auto& d : shape) n = n * d; return n; }

std::vector<Expr> rowMajor(const std::vector<Expr>& shape) {
  std::vector<Expr> st(shape.size());
  Expr acc(1);
  for (int i = (int)shape.size() - 1; i >= 0; --i) { st[i] = acc; acc = acc * shape[i]; }
  return st;
}

bool isContiguous(const View& v) {
  Expr acc(1);
  for (int i = (int)v.rank() - 1; i >= 0; --i) {
    if (v.shape[i].isConst(1)) continue;
    if (v.strides[i] != acc) return false;
    acc = acc * v.shape[i];
  }
  return true;
}

// Finds the dim order (outermost first) in which `v` is dense, if it is a permuted-contiguous view.
bool denseOrder(const View& v, std::vector<int>& order) {
  size_t r = v.rank();
  std::vector<bool> used(r, false);
  std::vector<int> inner;  // innermost first
  Expr acc(1);
  for (size_t n = 0; n < r; ++n) {
    int pick = -1;
    for (size_t d = 0; d < r; ++d) if (!used[d] && !v.shape[d].isConst(1) && v.strides[d] == acc) { pick = (int)d; break; }
    if (pick < 0) { for (size_t d = 0; d < r; ++d) if (!used[d] && v.shape[d].isConst(1)) { pick = (int)d; break; } }
    if (pick < 0) return false;
    used[pick] = true; inner.push_back(pick); acc = acc * v.shape[pick];
  }
  order.assign(inner.rbegin(), inner.rend());
  return true;
}

// Re-expresses `v` with a new shape without moving data, when the strides allow it.
bool reshapeView(const View& v, const std::vector<Expr>& newShape, View& out) {
  out = v; out.shape = newShape; out.strides.assign(newShape.size(), Expr(0));
  // maximal mergeable chunks of the old view (size-1 dims dropped)
  struct Chunk { Expr numel, base; };
  std::vector<Chunk> chunks;
  for (size_t d = 0; d < v.rank(); ++d) {
    if (v.shape[d].isConst(1)) continue;
    if (!chunks.empty() && chunks.back().base == v.strides[d] * v.shape[d]) { chunks.back().numel = chunks.back().numel * v.shape[d]; chunks.back().base = v.strides[d]; }
    else chunks.push_back({v.shape[d], v.strides[d]});
  }
  size_t c = 0; Expr acc(1); std::vector<size_t> group;
  auto flush = [&](const Chunk& ch) {
    Expr st = ch.base;
    for (int k = (int)group.size() - 1; k >= 0; --k) { out.strides[group[k]] = st; st = st * newShape[group[k]]; }
    group.clear(); acc = Expr(1);
  };
  for (size_t d = 0; d < newShape.size(); ++d) {
    if (newShape[d].isConst(1)) { out.strides[d] = Expr(0); continue; }
    if (c >= chunks.size()) return false;
    group.push_back(d); acc = acc * newShape[d];
    if (acc == chunks[c].numel) { flush(chunks[c]); ++c; }
  }
  if (!group.empty() || c != chunks.size()) return false;
  // size-1 dims get the stride a contiguous tensor would have (harmless, keeps isContiguous true)
  Expr run(1);
  for (int d = (int)newShape.size() - 1; d >= 0; --d) { if (newShape[d].isConst(1)) out.strides[d] = run; else run = out.strides[d] * newShape[d]; }
  return true;
}

View broadcastView(const View& v, const std::vector<Expr>& shape, const std::vector<int64_t>& castDims) {
  View o = v; o.shape = shape; o.strides.assign(shape.size(), Expr(0));
  for (size_t i = 0; i < v.rank(); ++i) {
    int64_t d = castDims[i];
    if (d < 0 || d >= (int64_t)shape.size()) fail("broadcast dim out of range");
    if (v.shape[i] == shape[d]) o.strides[d] = v.shape[i].isConst(1) ? Expr(0) : v.strides[i];
    else if (v.shape[i].isConst(1)) o.strides[d] = Expr(0);
    else fail("cannot broadcast extent " + v.shape[i].str() + " to " + shape[d].str());
  }
  return o;
}

std::string fmtDouble(double v) { char b[64]; snprintf(b, sizeof b, "%.9g", v); return b; }

// ---------------------------------------------------------------------------------------------
struct Lowering {
  Module& m;
  const CompileOptionsData& opts;
  Plan plan;
  std::vector<ENode> nodes;
  std::vector<PendingK> pend;
  std::vector<AttnCand> attn;
  bool shapesOnly = false;     // infer-symbol-shape: the plan is discarded, so results need not be materialised (scalars may be returned)
  // How a derived extent came about, keyed by its printed form: the affine map the reference attaches to the new symbol
  // (SymbolAnalysis::buildNewSymbol, LLHinfersymbolShape.cpp:277-292) and the extents it is a function of.
  struct RelInfo { std::string map; std::vector<Expr> operands; };
  std::map<std::string, RelInfo> relInfo;
  void noteRelation(const Expr& result, const std::string& map, const std::vector<Expr>& operands) {
    if (!result.isConst()) relInfo.emplace(result.str(), RelInfo{map, operands});
  }
  std::map<Value*, TV> tvs;
  std::map<std::string, int> constVecCache;

  Lowering(Module& mod, const CompileOptionsData& o) : m(mod), opts(o) {}

  // ---- buffers
  int newBuffer(DType dt, const Expr& numel, BufferDecl::Kind kind) {
    BufferDecl b; b.dtype = dt; b.numel = numel; b.kind = kind;
    plan.buffers.push_back(b);
    return (int)plan.buffers.size() - 1;
  }
  View freshView(DType dt, const std::vector<Expr>& shape, bool isConst, const std::vector<Expr>* strides = nullptr) {
    Expr n = numelOf(shape);
    View v; v.dtype = dt; v.shape = shape; v.strides = strides ? *strides : rowMajor(shape);
    v.buf = newBuffer(dt, n, (isConst && n.isConst()) ? BufferDecl::Const : BufferDecl::Temp);
    return v;
  }
  bool bufIsConst(int buf) const { auto k = plan.buffers[buf].kind; return k == BufferDecl::Weight || k == BufferDecl::Const; }

  // ---- lazy trees
  int leafNode(const View& v) { ENode n; n.kind = ENode::Leaf; n.leaf = v; n.leafConst = bufIsConst(v.buf); nodes.push_back(n); return (int)nodes.size() - 1; }
  int constNode(double c) { ENode n; n.kind = ENode::Const; n.cst = c; nodes.push_back(n); return (int)nodes.size() - 1; }
  int opNode(const std::string& op, int a, int b = -1, int c = -1) { ENode n; n.kind = ENode::Op; n.op = op; n.a = a; n.b = b; n.c = c; nodes.push_back(n); return (int)nodes.size() - 1; }
  bool treeIsConst(int root) {
    const ENode& n = nodes[root];
    if (n.kind == ENode::Leaf) return n.leafConst;
    if (n.kind == ENode::Const) return true;
    return treeIsConst(n.a) && (n.b < 0 || treeIsConst(n.b)) && (n.c < 0 || treeIsConst(n.c));
  }
  int mapLeaves(int root, const std::function<bool(const View&, View&)>& f, std::map<int, int>& memo, bool& ok) {
    auto it = memo.find(root);
    if (it != memo.end()) return it->second;
    ENode n = nodes[root];
    int res;
    if (n.kind == ENode::Leaf) { View nv; if (!f(n.leaf, nv)) { ok = false; nv = n.leaf; } ENode c = n; c.leaf = nv; nodes.push_back(c); res = (int)nodes.size() - 1; }
    else if (n.kind == ENode::Const) res = root;
    else {
      int a = mapLeaves(n.a, f, memo, ok), b = n.b >= 0 ? mapLeaves(n.b, f, memo, ok) : -1, c = n.c >= 0 ? mapLeaves(n.c, f, memo, ok) : -1;
      ENode o = n; o.a = a; o.b = b; o.c = c; nodes.push_back(o); res = (int)nodes.size() - 1;
    }
    memo[root] = res;
    return res;
  }
  bool splatValue(const TV& t, double& v) const {
    if (t.kind != TV::Lazy) return false;
    if (nodes[t.root].kind != ENode::Const) return false;
    v = nodes[t.root].cst; return true;
  }

  // ---- eltwise emission
  void emitEltwise(int root, const View& out, bool init) {
    Step s; s.kernel = "eltwise"; s.init = init;
    s.views.emplace_back("out", out);
    std::vector<std::string> leafKeys;
    std::map<int, int> reg;  // node -> register
    std::vector<std::string> prog;
    std::function<int(int)> walk = [&](int id) -> int {
      auto it = reg.find(id);
      if (it != reg.end()) return it->second;
      const ENode n = nodes[id];
      std::string ins;
      if (n.kind == ENode::Leaf) {
        std::string key = n.leaf.str();
        size_t k = 0;
        for (; k < leafKeys.size(); ++k) if (leafKeys[k] == key) break;
        if (k == leafKeys.size()) { leafKeys.push_back(key); s.views.emplace_back("in" + std::to_string(k), n.leaf); }
        ins = "ld" + std::to_string(k);
      } else if (n.kind == ENode::Const) {
        ins = "#" + fmtDouble(n.cst);
      } else {
        int a = walk(n.a), b = n.b >= 0 ? walk(n.b) : -1, c = n.c >= 0 ? walk(n.c) : -1;
        ins = n.op + "," + std::to_string(a);
        if (b >= 0) ins += "," + std::to_string(b);
        if (c >= 0) ins += "," + std::to_string(c);
      }
      prog.push_back(ins);
      reg[id] = (int)prog.size() - 1;
      return reg[id];
    };
    walk(root);
    std::string p;
    for (size_t i = 0; i < prog.size(); ++i) p += (i ? ";" : "") + prog[i];
    s.params.emplace_back("prog", p);
    if (leafKeys.size() > 8) fail("elementwise fusion produced more than 8 inputs");
    if (prog.size() > 48) fail("elementwise fusion produced more than 48 instructions");
    plan.steps.push_back(s);
  }

  // Materialises a lazy tree.  The result layout follows the first dense, non-broadcast leaf so that
  // NHWC data stays NHWC.
  std::string treeKey(int id) {
    const ENode& n = nodes[id];
    if (n.kind == ENode::Leaf) return "L(" + n.leaf.str() + ")";
    if (n.kind == ENode::Const) return "#" + fmtDouble(n.cst);
    return n.op + "(" + treeKey(n.a) + (n.b >= 0 ? "," + treeKey(n.b) : "") + (n.c >= 0 ? "," + treeKey(n.c) : "") + ")";
  }
  void countTree(int id, std::set<std::string>& leaves, std::set<int>& seen) {
    if (!seen.insert(id).second) return;
    const ENode& n = nodes[id];
    if (n.kind == ENode::Leaf) { leaves.insert(n.leaf.str()); return; }
    if (n.kind == ENode::Const) return;
    countTree(n.a, leaves, seen); if (n.b >= 0) countTree(n.b, leaves, seen); if (n.c >= 0) countTree(n.c, leaves, seen);
  }
  std::map<std::string, View> constTreeCache;
  View materializeTree(int root, DType dt, const std::vector<Expr>& shape, const std::vector<Expr>* wantStrides = nullptr, int intoBuf = -1) {
    bool isC = treeIsConst(root) && numelOf(shape).isConst();
    std::string ckey;
    if (isC && intoBuf < 0) {   // load-time values are computed once, however often the graph repeats them
      ckey = treeKey(root) + "|" + dtypeName(dt) + "|";
      for (auto& e : shape) ckey += e.str() + ",";
      if (wantStrides) for (auto& e : *wantStrides) ckey += e.str() + ";";
      auto it = constTreeCache.find(ckey);
      if (it != constTreeCache.end()) return it->second;
    }
    std::vector<Expr> strides = rowMajor(shape);
    if (wantStrides) strides = *wantStrides;
    else {
      std::function<bool(int)> findLeaf = [&](int id) -> bool {
        const ENode& n = nodes[id];
        if (n.kind == ENode::Leaf) {
          std::vector<int> order;
          bool nz = true; for (auto& st : n.leaf.strides) if (st.isConst(0)) nz = false;
          for (size_t d = 0; d < n.leaf.rank(); ++d) if (n.leaf.shape[d].isConst(1)) nz = nz;  // size-1 dims are fine
          if (n.leaf.shape == shape && denseOrder(n.leaf, order)) {
            bool bcast = false;
            for (size_t d = 0; d < shape.size(); ++d) if (!shape[d].isConst(1) && n.leaf.strides[d].isConst(0)) bcast = true;
            if (!bcast) { Expr acc(1); for (int k = (int)order.size() - 1; k >= 0; --k) { strides[order[k]] = acc; acc = acc * shape[order[k]]; } return true; }
          }
          return false;
        }
        if (n.kind == ENode::Const) return false;
        return findLeaf(n.a) || (n.b >= 0 && findLeaf(n.b)) || (n.c >= 0 && findLeaf(n.c));
      };
      if (intoBuf < 0) findLeaf(root);
    }
    View out;
    if (intoBuf >= 0) { out.buf = intoBuf; out.dtype = dt; out.shape = shape; out.strides = strides; }
    else out = freshView(dt, shape, isC, &strides);
    emitEltwise(root, out, isC && intoBuf < 0);
    if (!ckey.empty()) constTreeCache[ckey] = out;
    return out;
  }

  // ---- pending producers
  void emitPending(int id) {
    PendingK& p = pend[id];
    if (p.emitted) return;
    p.emitted = true;
    Step s = p.step;
    s.views.emplace_back("out", p.nativeOut);
    if (s.kernel == "attention") { plan.steps.push_back(s); return; }
    double alpha = 1.0;
    Expr C = p.nativeOut.shape[p.chanDim];
    auto vec = [&](int root, const char* name) {
      const ENode& rn = nodes[root];
      if (rn.kind == ENode::Leaf && rn.leaf.dtype == DType::F32 && rn.leaf.strides[0].isConst(1)) { s.views.emplace_back(name, rn.leaf); return; }
      View v = materializeTree(root, DType::F32, {C});
      s.views.emplace_back(name, v);
    };
    if (p.scaleRoot >= 0) {
      if (nodes[p.scaleRoot].kind == ENode::Const) alpha = nodes[p.scaleRoot].cst;
      else vec(p.scaleRoot, "scale");
    }
    if (p.shiftRoot >= 0) {
      if (!(nodes[p.shiftRoot].kind == ENode::Const && nodes[p.shiftRoot].cst == 0.0)) {
        int root = p.shiftRoot;
        vec(root, "shift");   // a constant shift still becomes a per-channel vector
      }
    }
    if (p.hasRes) s.views.emplace_back("res", p.res);
    s.params.emplace_back("alpha", fmtDouble(alpha));
    s.params.emplace_back("act", p.act);
    plan.steps.push_back(s);
  }

  // ---- TV access
  TV& raw(Value* v) {
    auto it = tvs.find(v);
    if (it == tvs.end()) fail("value " + v->name + " used before definition");
    return it->second;
  }
  void settle(TV& t) {
    if (t.kind == TV::Pending && pend[t.pending].emitted) { t.kind = TV::ViewK; }
    if (t.kind == TV::AttnProb && attn[t.attn].materialized) { t.kind = TV::ViewK; }
  }

  // Forces a value into a strided view (emitting whatever produces it).
  void toView(TV& t) {
    settle(t);
    if (t.kind == TV::ViewK) return;
    if (t.kind == TV::Pending) { emitPending(t.pending); t.kind = TV::ViewK; return; }
    if (t.kind == TV::AttnProb) {
      // not consumed by a GEMM with V after all: scores, then a row softmax into the buffer t.view lives in
      AttnCand& c = attn[t.attn];
      PendingK& P = pend[c.pending];
      emitPending(c.pending);
      const View& sc = P.nativeOut;
      Expr rows = sc.shape[0] * sc.shape[1] * sc.shape[2];
      View x2 = sc; x2.shape = {rows, sc.shape[3]}; x2.strides = {sc.shape[3], Expr(1)};
      View o2 = t.view; o2.offset = Expr(0); o2.shape = x2.shape; o2.strides = x2.strides;
      Step st; st.kernel = "softmax"; st.views.emplace_back("x", x2); st.views.emplace_back("out", o2);
      plan.steps.push_back(st);
      c.materialized = true; t.kind = TV::ViewK; return;
    }
    if (t.kind == TV::Lazy) {
      View v = materializeTree(t.root, t.dtype, t.shape);
      t.isConst = bufIsConst(v.buf);
      t.view = v; t.kind = TV::ViewK; return;
    }
    if (t.kind == TV::Deferred) {
      // copy the strided source into a dense row-major buffer, then the reshape is free
      std::vector<Expr> rm = rowMajor(t.view.shape);
      View dense = materializeTree(leafNode(t.view), t.dtype, t.view.shape, &rm);
      View r;
      if (!reshapeView(dense, t.shape, r)) { r = dense; r.shape = t.shape; r.strides = rowMajor(t.shape); }   // dense: any shape of the same count
      t.view = r; t.kind = TV::ViewK; t.isConst = bufIsConst(r.buf); return;
    }
    fail("expected a tensor value");
  }
  TV& get(Value* v) {
    TV& t = raw(v);
    settle(t);
    // a value with several consumers is computed once
    if (v->users.size() > 1 && (t.kind == TV::Pending || t.kind == TV::AttnProb || (t.kind == TV::Lazy && nodes[t.root].kind != ENode::Const && !isCheap(t.root))))
      toView(t);
    return t;
  }
  bool isCheap(int root) {  // leaf or constant: re-reading is free
    return nodes[root].kind != ENode::Op;
  }
  View viewOf(Value* v) { TV& t = get(v); toView(t); return t.view; }
  // A float->float convert_to is only a change of storage type: consumers that read any float
  // type take the view underneath it instead of a converted copy.
  bool isLeafOnly(const TV& t) const { return t.kind == TV::Lazy && nodes[t.root].kind == ENode::Leaf && isFloat(nodes[t.root].leaf.dtype) && isFloat(t.dtype); }
  View leafOrView(Value* v) {
    TV& t = get(v);
    if (isLeafOnly(t)) return nodes[t.root].leaf;
    toView(t); return t.view;
  }
  View contiguousLeafOrView(Value* v) {
    TV& t = get(v);
    if (isLeafOnly(t) && isContiguous(nodes[t.root].leaf)) return nodes[t.root].leaf;
    return contiguousViewOf(v);
  }
  // If the only consumer of `res` converts it to another float type, produce that type directly.
  DType resultDtype(Value* res) {
    DType dt = res->type.elt;
    if (res->users.size() == 1 && res->users[0]->name == "llh.convert_to" && isFloat(dt)) {
      DType to = res->users[0]->results[0]->type.elt;
      if (isFloat(to) && dtypeSize(to) < dtypeSize(dt)) return to;   // a narrowing convert is done by the producer; a widening one changes nothing (readers compute in fp32)
    }
    return dt;
  }
  View contiguousViewOf(Value* v) {
    TV& t = get(v); toView(t);
    if (isContiguous(t.view)) return t.view;
    std::vector<Expr> rm = rowMajor(t.shape);
    View d = materializeTree(leafNode(t.view), t.dtype, t.shape, &rm);
    t.view = d; t.isConst = bufIsConst(d.buf);
    return d;
  }
  View viewWithStrides(Value* v, const std::vector<Expr>& want) {
    TV& t = get(v);
    if (t.kind == TV::Lazy && nodes[t.root].kind == ENode::Op) {   // compute straight into the wanted layout
      View d = materializeTree(t.root, t.dtype, t.shape, &want);
      t.kind = TV::ViewK; t.view = d; t.isConst = bufIsConst(d.buf);
      return d;
    }
    toView(t);
    bool same = true;
    for (size_t d = 0; d < want.size(); ++d) if (!t.shape[d].isConst(1) && t.view.strides[d] != want[d]) same = false;
    if (same) return t.view;
    View d = materializeTree(leafNode(t.view), t.dtype, t.shape, &want);
    t.view = d; t.isConst = bufIsConst(d.buf);
    return d;
  }
  Expr scalarOf(Value* v) {
    TV& t = raw(v);
    if (t.kind != TV::Scalar || t.isFloatScalar) fail("expected an integer scalar for " + v->name);
    return t.scalar;
  }

  TV makeView(const View& v, bool isConst) { TV t; t.kind = TV::ViewK; t.view = v; t.shape = v.shape; t.dtype = v.dtype; t.isConst = isConst; return t; }
  TV makeLazy(int root, DType dt, const std::vector<Expr>& shape) { TV t; t.kind = TV::Lazy; t.root = root; t.dtype = dt; t.shape = shape; t.isConst = treeIsConst(root); return t; }

  // node for an operand inside an elementwise op, broadcast (numpy style) to `shape`
  int operandNode(TV& t, const std::vector<Expr>& shape) {
    if (t.kind == TV::Scalar) {
      if (t.isFloatScalar) return constNode(t.fscalar);
      if (t.scalar.isConst()) return constNode((double)t.scalar.constant());
      fail("symbolic scalar used as a tensor operand");
    }
    if (t.kind != TV::Lazy) toView(t);
    std::vector<int64_t> cast;
    size_t off = shape.size() - t.shape.size();
    for (size_t i = 0; i < t.shape.size(); ++i) cast.push_back((int64_t)(off + i));
    if (t.kind == TV::ViewK) return leafNode(broadcastView(t.view, shape, cast));
    if (t.shape == shape) return t.root;
    std::map<int, int> memo; bool ok = true;
    return mapLeaves(t.root, [&](const View& l, View& o) { o = broadcastView(l, shape, cast); return true; }, memo, ok);
  }

  std::vector<Expr> broadcastShapes(const std::vector<Expr>& a, const std::vector<Expr>& b) {
    size_t r = std::max(a.size(), b.size());
    std::vector<Expr> o(r);
    for (size_t i = 0; i < r; ++i) {
      const Expr* x = i + a.size() >= r ? &a[i + a.size() - r] : nullptr;
      const Expr* y = i + b.size() >= r ? &b[i + b.size() - r] : nullptr;
      if (!x) o[i] = *y; else if (!y) o[i] = *x;
      else if (x->isConst(1)) o[i] = *y; else if (y->isConst(1)) o[i] = *x;
      else if (*x == *y) o[i] = *x;
      else o[i] = *x;   // symbolically different names for the same extent: trust the producer
    }
    return o;
  }

  // ---- epilogue absorption
  // Restricts a tensor operand that only varies along `dim` of `shape` to a 1-D tree over that dim.
  bool channelTree(TV& x, const std::vector<Expr>& shape, int dim, int& rootOut) {
    if (x.kind == TV::Pending || x.kind == TV::Deferred || x.kind == TV::Scalar) return false;
    if (x.kind == TV::ViewK && !x.isConst) return false;
    if (x.kind == TV::Lazy && !treeIsConst(x.root)) return false;
    int root = operandNode(x, shape);
    std::map<int, int> memo; bool ok = true;
    rootOut = mapLeaves(root, [&](const View& l, View& o) {
      for (size_t d = 0; d < l.rank(); ++d) if ((int)d != dim && !l.strides[d].isConst(0) && !l.shape[d].isConst(1)) return false;
      o = l; o.shape = {shape[dim]}; o.strides = {l.strides[dim]};
      return true;
    }, memo, ok);
    return ok;
  }

  // Tries to fold `op(P, other)` into pending P's epilogue.  `pIsLhs` tells which side P is on.
  bool absorb(const std::string& op, Value* pv, Value* ov, bool pIsLhs, Value* result) {
    TV& pt = raw(pv);
    settle(pt);
    if (pt.kind != TV::Pending || pv->users.size() != 1) return false;
    PendingK& P = pend[pt.pending];
    if (P.step.kernel == "attention") return false;
    // channel dim of the current logical view: unit stride, extent = channel count
    Expr C = P.nativeOut.shape[P.chanDim];
    int cd = -1;
    for (size_t d = 0; d < pt.view.rank(); ++d) if (pt.view.strides[d].isConst(1) && pt.view.shape[d] == C) cd = (int)d;
    auto finish = [&]() {
      TV r = pt;
      DType to = result->type.elt;
      if (to != DType::None && isFloat(to) && to != r.dtype) { r.dtype = to; r.view.dtype = to; P.nativeOut.dtype = to; plan.buffers[P.buf].dtype = to; }
      tvs[result] = r; return true;
    };
    if (!ov) {  // unary activation
      if (P.stage == 2) return false;
      if (op == "relu" || op == "gelu") { P.act = op; P.stage = 2; return finish(); }
      return false;
    }
    TV& ot = get(ov);
    if (broadcastShapes(pt.shape, ot.shape) != pt.shape) return false;
    double sv;
    bool isSplat = splatValue(ot, sv);
    if (op == "max" && isSplat && sv == 0.0 && P.stage < 2) { P.act = "relu"; P.stage = 2; return finish(); }
    if (P.stage == 0 && cd >= 0) {
      int vroot = -1;
      bool isVec = isSplat ? (vroot = constNode(sv), true) : channelTree(ot, pt.shape, cd, vroot);
      if (isVec) {
        if (op == "mul" || (op == "div" && pIsLhs)) {
          P.scaleRoot = P.scaleRoot < 0 ? (op == "mul" ? vroot : opNode("div", constNode(1.0), vroot)) : opNode(op, P.scaleRoot, vroot);
          if (P.shiftRoot >= 0) P.shiftRoot = opNode(op, P.shiftRoot, vroot);
          foldConst(P.scaleRoot);
          return finish();
        }
        if (op == "add" || (op == "sub" && pIsLhs)) {
          P.shiftRoot = P.shiftRoot < 0 ? (op == "add" ? vroot : opNode("neg", vroot)) : opNode(op, P.shiftRoot, vroot);
          return finish();
        }
        return false;
      }
    }
    if (op == "add" && P.stage <= 0 + 0 && !P.hasRes) {
      // residual: another run-time tensor of the same shape
      if (ot.kind == TV::Lazy && nodes[ot.root].kind == ENode::Const) return false;
      if (ot.kind == TV::Pending && ot.pending == pt.pending) return false;
      View ov2;
      if (isLeafOnly(ot)) ov2 = nodes[ot.root].leaf; else { toView(ot); ov2 = ot.view; }
      std::vector<int64_t> cast; size_t off = pt.shape.size() - ot.shape.size();
      for (size_t i = 0; i < ot.shape.size(); ++i) cast.push_back((int64_t)(off + i));
      View r = broadcastView(ov2, pt.shape, cast);
      bool sameLayout = true;
      for (size_t d = 0; d < r.rank(); ++d) if (!r.shape[d].isConst(1) && r.strides[d] != pt.view.strides[d]) sameLayout = false;
      bool isNative = pt.view.shape == P.nativeOut.shape && pt.view.strides == P.nativeOut.strides;
      if (sameLayout) { View nr = P.nativeOut; nr.buf = r.buf; nr.offset = r.offset; nr.dtype = r.dtype; P.res = nr; }
      else if (isNative && P.step.kernel == "gemm") P.res = r;
      else return false;
      P.hasRes = true; P.stage = 1;
      return finish();
    }
    return false;
  }
  void foldConst(int& root) {
    ENode& n = nodes[root];
    if (n.kind == ENode::Op && n.b >= 0 && nodes[n.a].kind == ENode::Const && nodes[n.b].kind == ENode::Const) {
      double a = nodes[n.a].cst, b = nodes[n.b].cst, r;
      if (n.op == "mul") r = a * b; else if (n.op == "div") r = a / b; else if (n.op == "add") r = a + b; else if (n.op == "sub") r = a - b; else return;
      root = constNode(r);
    }
  }

  // ---- generic elementwise op
  void eltwise(Op* op, const std::string& name) {
    Value* res = op->results[0];
    size_t n = op->operands.size();
    DType outDt = res->type.elt;
    if (n == 1 && absorb(name, op->operands[0], nullptr, true, res)) return;
    if (n == 2) {
      if (absorb(name, op->operands[0], op->operands[1], true, res)) return;
      if ((name == "add" || name == "mul" || name == "max") && absorb(name, op->operands[1], op->operands[0], false, res)) return;
    }
    std::vector<TV*> ts;
    std::vector<Expr> shape;
    for (Value* v : op->operands) { TV& t = get(v); ts.push_back(&t); if (t.kind != TV::Scalar) shape = shape.empty() ? t.shape : broadcastShapes(shape, t.shape); }
    if (shape.empty()) fail("elementwise op without tensor operands: " + op->name);
    // identities: x*1, x/1, x+0, x-0
    if (n == 2) {
      double sv;
      if (splatValue(*ts[1], sv) && ts[0]->shape == shape && ((sv == 1.0 && (name == "mul" || name == "div")) || (sv == 0.0 && (name == "add" || name == "sub"))) && ts[0]->dtype == outDt) { TV c = *ts[0]; tvs[res] = c; return; }
      if (splatValue(*ts[0], sv) && ts[1]->shape == shape && ((sv == 1.0 && name == "mul") || (sv == 0.0 && name == "add")) && ts[1]->dtype == outDt) { TV c = *ts[1]; tvs[res] = c; return; }
    }
    std::vector<int> ids;
    for (TV* t : ts) ids.push_back(operandNode(*t, shape));
    int root = opNode(name, ids[0], n > 1 ? ids[1] : -1, n > 2 ? ids[2] : -1);
    {   // keep fused chains within the kernel's limits (8 inputs, 48 instructions)
      std::set<std::string> leaves; std::set<int> seen;
      countTree(root, leaves, seen);
      if (leaves.size() > 8 || seen.size() > 40) {
        ids.clear();
        for (TV* t : ts) { if (t->kind == TV::Lazy && nodes[t->root].kind == ENode::Op) toView(*t); ids.push_back(operandNode(*t, shape)); }
        root = opNode(name, ids[0], n > 1 ? ids[1] : -1, n > 2 ? ids[2] : -1);
      }
    }
    if (n == 2) foldConst(root);
    tvs[res] = makeLazy(root, outDt, shape);
  }

  // ---- GEMM
  View to4d(const View& v) {  // [.., M, K] -> [b0, b1, M, K]
    View o = v;
    while (o.rank() < 4) { o.shape.insert(o.shape.begin(), Expr(1)); o.strides.insert(o.strides.begin(), Expr(0)); }
    return o;
  }
  std::string gemmPrecision(DType dt) {
    if (dt == DType::BF16 || dt == DType::F16) return "bf16";
    if (opts.precision == "tf32" || opts.precision == "tf32x3" || opts.precision == "fp32") return opts.precision;
    return "fp32";
  }
  View gemmOperand(Value* v, bool isB, std::vector<Expr>* split) {
    TV& t = get(v);
    settle(t);
    // reshape(rank-4 strided) that only merges the two leading dims: use the rank-4 strides directly
    if (t.kind == TV::Deferred && t.view.rank() == 4 && t.shape.size() == 3 && t.shape[1] == t.view.shape[2] && t.shape[2] == t.view.shape[3]) {
      const View& s = t.view;
      bool unitInner = s.strides[3].isConst(1) || s.strides[2].isConst(1);
      if (unitInner && (isB || s.strides[3].isConst(1))) { if (split) *split = {s.shape[0], s.shape[1]}; return s; }
    }
    View x;
    if (isLeafOnly(t)) x = nodes[t.root].leaf; else { toView(t); x = t.view; }
    size_t r = x.rank();
    bool ok = isB ? (x.strides[r - 1].isConst(1) || x.strides[r - 2].isConst(1)) : x.strides[r - 1].isConst(1);
    if (x.shape[r - 1].isConst(1) && !isB) ok = true;
    if (!ok) { std::vector<Expr> rm = rowMajor(x.shape); x = materializeTree(leafNode(x), x.dtype, x.shape, &rm); }
    return x;
  }
  // Whether a pending GEMM is the score matrix the fused attention kernel can produce itself: bf16 Q and K with a
  // head size of 64 read along their unit-stride dim, at most 512 keys (a compile-time constant), nothing absorbed but
  // a constant scale and an additive mask with unit stride along the keys, and the logical view still the plain
  // [.., M, N] matrix.
  bool attentionScores(const TV& t) {
    if (opts.fuseAttention == false) return false;
    const PendingK& P = pend[t.pending];
    if (P.emitted || P.step.kernel != "gemm" || P.act != "none" || P.shiftRoot >= 0) return false;
    if (P.scaleRoot >= 0 && nodes[P.scaleRoot].kind != ENode::Const) return false;
    const View* a = nullptr; const View* b = nullptr;
    for (auto& v : P.step.views) { if (v.first == "a") a = &v.second; if (v.first == "b") b = &v.second; }
    if (!a || !b || a->dtype != DType::BF16 || b->dtype != DType::BF16) return false;
    if (!a->shape[3].isConst(64) || !a->strides[3].isConst(1) || !b->strides[2].isConst(1)) return false;
    const Expr& N = b->shape[3];
    if (!N.isConst() || N.constant() < 1 || N.constant() > 512) return false;
    auto mult8 = [](const Expr& e) { return e.isConst() && e.constant() >= 0 && e.constant() % 8 == 0; };
    if (!mult8(a->strides[0]) || !mult8(a->strides[1]) || !mult8(a->strides[2]) || !mult8(b->strides[0]) || !mult8(b->strides[1]) || !mult8(b->strides[3]) ||
        !mult8(a->offset) || !mult8(b->offset)) return false;
    if (P.hasRes && !(P.res.strides[3].isConst(1) || P.res.shape[3].isConst(1))) return false;
    if (t.view.shape.empty() || !(t.view.shape.back() == N) || t.view.strides != rowMajor(t.view.shape) || !t.view.offset.isConst(0)) return false;
    return true;
  }
  // probs x V where probs is the softmax of pending scores: one attention step instead of GEMM, softmax, GEMM.
  bool tryAttention(Op* op, TV& pt, bool batched) {
    PendingK& S = pend[attn[pt.attn].pending];
    if (S.emitted || attn[pt.attn].materialized) return false;
    if (pt.view.shape.empty() || pt.view.strides != rowMajor(pt.view.shape) || !(pt.view.shape.back() == S.nativeOut.shape[3])) return false;
    std::vector<Expr> splitB;
    View v = gemmOperand(op->operands[1], true, &splitB);
    const Expr b0 = S.nativeOut.shape[0], b1 = S.nativeOut.shape[1], M = S.nativeOut.shape[2], N = S.nativeOut.shape[3];
    View v4;
    if (v.rank() == 4) v4 = v;
    else if (v.rank() == 3) { v4 = v; v4.shape = {b0, b1, v.shape[1], v.shape[2]}; v4.strides = {v.strides[0] * b1, v.strides[0], v.strides[1], v.strides[2]}; }
    else if (v.rank() == 2) { v4 = v; v4.shape = {Expr(1), Expr(1), v.shape[0], v.shape[1]}; v4.strides = {Expr(0), Expr(0), v.strides[0], v.strides[1]}; }
    else return false;
    if (v.rank() == 3 && !(v.shape[0] == b0 * b1)) return false;
    if (v.rank() == 4 && (!(v4.shape[0] == b0) || !(v4.shape[1] == b1))) return false;
    auto mult8 = [](const Expr& e) { return e.isConst() && e.constant() >= 0 && e.constant() % 8 == 0; };
    if (v4.dtype != DType::BF16 || !v4.shape[3].isConst(64) || !v4.strides[3].isConst(1) || !(v4.shape[2] == N)) return false;
    if (!mult8(v4.strides[0]) || !mult8(v4.strides[1]) || !mult8(v4.strides[2]) || !mult8(v4.offset)) return false;
    DType dt = op->results[0]->type.elt;
    if (dt != DType::BF16) return false;
    PendingK P;
    P.step.kernel = "attention";
    for (auto& sv : S.step.views) { if (sv.first == "a") P.step.views.emplace_back("q", sv.second); if (sv.first == "b") P.step.views.emplace_back("k", sv.second); }
    P.step.views.emplace_back("v", v4);
    if (S.hasRes) P.step.views.emplace_back("mask", S.res);
    P.step.params.emplace_back("scale", fmtDouble(S.scaleRoot >= 0 ? nodes[S.scaleRoot].cst : 1.0));
    std::vector<Expr> nshape = {b0, b1, M, Expr(64)};
    P.nativeOut = freshView(dt, nshape, false);
    P.buf = P.nativeOut.buf;
    P.chanDim = 3;
    pend.push_back(P);
    S.emitted = true;                     // the scores are never written
    attn[pt.attn].materialized = false;
    TV t; t.kind = TV::Pending; t.pending = (int)pend.size() - 1; t.dtype = dt;
    t.shape = batched ? std::vector<Expr>{b0 * b1, M, Expr(64)} : std::vector<Expr>{M, Expr(64)};
    t.view = pend.back().nativeOut; t.view.shape = t.shape; t.view.strides = rowMajor(t.shape);
    tvs[op->results[0]] = t;
    return true;
  }
  void gemm(Op* op, bool batched) {
    {
      TV& a0 = raw(op->operands[0]);
      settle(a0);
      if (a0.kind == TV::AttnProb && op->operands[0]->users.size() == 1 && tryAttention(op, a0, batched)) return;
    }
    std::vector<Expr> splitA, splitB;
    View a = gemmOperand(op->operands[0], false, &splitA);
    View b = gemmOperand(op->operands[1], true, &splitB);
    std::vector<Expr> split = !splitA.empty() ? splitA : splitB;
    auto lift = [&](View v) -> View {
      if (v.rank() == 4) return v;
      if (v.rank() == 3 && !split.empty()) {   // [b, r, c] -> [b0, b1, r, c]
        View o = v; o.shape = {split[0], split[1], v.shape[1], v.shape[2]};
        o.strides = {v.strides[0] * split[1], v.strides[0], v.strides[1], v.strides[2]};
        return o;
      }
      return to4d(v);
    };
    if (a.dtype != b.dtype) {   // mixed storage types: bring both to the wider one
      DType wide = (a.dtype == DType::F32 || b.dtype == DType::F32) ? DType::F32 : a.dtype;
      auto conv = [&](View& v) { if (v.dtype != wide) { v = materializeTree(leafNode(v), wide, v.shape); } };
      conv(a); conv(b);
    }
    a = lift(a); b = lift(b);
    // fp32 operands reach the tensor cores only K-major (a 32-bit MN-major B tile produced zeros on B200): a run-time B
    // stored [k][n] (attention's V) is copied once into [n][k] order, which costs far less than the FMA kernel would
    {
      const std::string prec = gemmPrecision(a.dtype);
      if ((prec == "tf32" || prec == "tf32x3") && b.dtype == DType::F32 && !b.strides[2].isConst(1) && !b.shape[2].isConst(1)) {
        std::vector<Expr> st = {b.shape[1] * b.shape[2] * b.shape[3], b.shape[2] * b.shape[3], Expr(1), b.shape[2]};
        b = materializeTree(leafNode(b), DType::F32, b.shape, &st);
      }
    }
    Expr M = a.shape[2], K = a.shape[3], N = b.shape[3];
    DType dt = op->results[0]->type.elt;
    PendingK P;
    P.step.kernel = "gemm";
    P.step.views.emplace_back("a", a);
    P.step.views.emplace_back("b", b);
    // tf32x3 with a constant (weight) B: its low-order part is computed once at load time and handed to the kernel,
    // which otherwise derives it from every B tile it loads
    if (gemmPrecision(a.dtype) == "tf32x3" && b.dtype == DType::F32 && bufIsConst(b.buf) && b.strides[2].isConst(1)) {
      View lo = materializeTree(opNode("tf32lo", leafNode(b)), DType::F32, b.shape, &b.strides);
      if (lo.strides == b.strides) P.step.views.emplace_back("b_lo", lo);
    }
    P.step.params.emplace_back("prec", gemmPrecision(a.dtype));
    std::vector<Expr> nshape = {a.shape[0], a.shape[1], M, N};
    if (a.shape[0].isConst(1) && !b.shape[0].isConst(1)) nshape[0] = b.shape[0];
    if (a.shape[1].isConst(1) && !b.shape[1].isConst(1)) nshape[1] = b.shape[1];
    P.nativeOut = freshView(dt, nshape, false);
    P.buf = P.nativeOut.buf;
    P.chanDim = 3;
    pend.push_back(P);
    TV t; t.kind = TV::Pending; t.pending = (int)pend.size() - 1; t.dtype = dt;
    t.shape = batched ? std::vector<Expr>{nshape[0] * nshape[1], M, N} : std::vector<Expr>{M, N};
    t.view = P.nativeOut; t.view.shape = t.shape; t.view.strides = rowMajor(t.shape);
    (void)K;
    tvs[op->results[0]] = t;
  }

  // ---- conv / pool
  std::vector<Expr> nhwcStrides(const std::vector<Expr>& s) {  // logical [N,C,H,W] over an NHWC buffer
    return {s[2] * s[3] * s[1], Expr(1), s[3] * s[1], s[1]};
  }
  Expr windowOut(const Expr& in, int64_t padLo, int64_t padHi, int64_t dil, int64_t k, int64_t stride, bool ceil = false) {
    // LLHinfersymbolShape.cpp:257-292: (in + pad_l + pad_h - dil*(k-1) - 1) / stride + 1
    const int64_t c = padLo + padHi - dil * (k - 1) - 1;
    Expr num = in + Expr(c);
    Expr out = (ceil ? num.ceildiv(Expr(stride)) : num.floordiv(Expr(stride))) + Expr(1);
    if (!in.isConst()) {
      // the reference records the relation as the map (s0 + c) ceildiv stride + 1 (LLHinfersymbolShape.cpp:281-287), printed
      // the way MLIR prints affine expressions
      auto plus = [](const std::string& a, int64_t v) { return v == 0 ? a : a + (v < 0 ? " - " : " + ") + std::to_string(v < 0 ? -v : v); };
      std::string body = stride == 1 ? plus("s0", c + 1) : plus((c == 0 ? std::string("s0") : "(" + plus("s0", c) + ")") + " ceildiv " + std::to_string(stride), 1);
      noteRelation(out, "(d0)[s0] -> (" + body + ")", {in});
    }
    return out;
  }
  void conv(Op* op, bool hasBias) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    if (xt.shape.size() != 4) fail("llh.conv expects rank-4 input");
    auto stride = intArray(op, "stride", {1, 1}), pad = intArray(op, "pad", {0, 0, 0, 0}), dil = intArray(op, "dilation", {1, 1});
    const Attr* g = op->attr("group");
    if (g && g->i != 1) fail("grouped convolution is not supported by the CUDA pipeline");
    const Attr* lay = op->attr("layout");
    if (lay && lay->s != "NCHW") fail("llh.conv: only NCHW-typed modules are accepted (the NHWC layout is chosen internally)");
    TV& wt = get(op->operands[1]); toView(wt);
    if (wt.shape.size() != 4) fail("llh.conv expects rank-4 weight");
    // The tensor-core kernel gathers 16-byte chunks that must not straddle a filter tap: pad a small
    // channel count (the 3-channel stem) to the next multiple of 16 bytes with zeros, in both the
    // NHWC activation copy and the re-laid-out weight.
    Expr Cin = xt.shape[1];
    int64_t cPad = 0;
    {
      const int eb = dtypeSize(xt.dtype), mult = 16 / eb;
      if (gemmPrecision(xt.dtype) != "fp32" && Cin.isConst() && Cin.constant() % mult != 0 && xt.shape[1] == wt.shape[1])
        cPad = (Cin.constant() + mult - 1) / mult * mult;
    }
    View x;
    settle(xt);
    const bool denseNchw = xt.kind == TV::ViewK && isContiguous(xt.view) && isFloat(xt.dtype) && dtypeSize(xt.dtype) <= 4 && !xt.isConst;
    // A narrow-channel stem (16 bytes per padded pixel, kernel at most 8 wide): eight neighbouring pixels are one
    // contiguous 128-byte run of the channel-last copy, so a whole filter row becomes the "channels" of a kernel that is one
    // pixel wide over an overlapping view (pixel stride 16 bytes, 8 * cPad channels), provided the copy carries the zero
    // padding columns itself.  One K block of the tensor-core kernel is then one filter row, loaded by a single TMA
    // im2col box instead of being gathered tap by tap.  (The eighth pixel of a row meets zero weights.)
    bool rowMerge = false; int64_t wLeft = 0, wTotal = 0, mergedW = 0;
    if (cPad && denseNchw && cPad * dtypeSize(xt.dtype) == 16 && wt.shape[2].isConst() && wt.shape[3].isConst() && wt.shape[3].constant() <= 8 &&
        wt.shape[3].constant() > 1 && dil[1] == 1 && xt.shape[3].isConst() && opts.mergeStemRows) {
      const int64_t W = xt.shape[3].constant(), KW = wt.shape[3].constant();
      const int64_t OWc = (W + pad[1] + pad[3] - (KW - 1) - 1) / stride[1] + 1;
      if (OWc >= 1) { rowMerge = true; wLeft = pad[1]; wTotal = std::max(pad[1] + W, (OWc - 1) * stride[1] + 8); mergedW = (OWc - 1) * stride[1] + 1; }
    }
    if (cPad || (denseNchw && !xt.shape[1].isConst(1))) {
      // NCHW data entering a conv chain: one re-layout kernel (with the channel padding if any)
      std::vector<Expr> pshape = {xt.shape[0], cPad ? Expr(cPad) : xt.shape[1], xt.shape[2], rowMerge ? Expr(wTotal) : xt.shape[3]};
      std::vector<Expr> pst = nhwcStrides(pshape);
      if (denseNchw) {
        x = freshView(xt.dtype, pshape, false, &pst);
        Step st; st.kernel = "nchw2nhwc";
        st.views.emplace_back("x", xt.view); st.views.emplace_back("out", x);
        if (rowMerge) {
          st.params.emplace_back("wide", std::to_string(wLeft) + "," + std::to_string(wTotal));
          // the convolution's view: [N, 8 * cPad, H, mergedW], a window of eight pixels per position
          x.shape = {xt.shape[0], Expr(8 * cPad), xt.shape[2], Expr(mergedW)};
        }
        plan.steps.push_back(st);
      } else {
        toView(xt);
        x = freshView(xt.dtype, pshape, false, &pst);
        emitEltwise(constNode(0.0), x, false);                          // zero the padding channels
        View real = x; real.shape = xt.shape;                           // same strides, real channel extent
        emitEltwise(leafNode(xt.view), real, false);
      }
    } else {
      x = viewWithStrides(xv, nhwcStrides(xt.shape));
    }
    // weight [F,C,KH,KW] -> dense [F,KH,KW,C(padded)]
    View wperm = wt.view;
    wperm.shape = {wt.view.shape[0], wt.view.shape[2], wt.view.shape[3], wt.view.shape[1]};
    wperm.strides = {wt.view.strides[0], wt.view.strides[2], wt.view.strides[3], wt.view.strides[1]};
    std::string key = "wperm:" + wperm.str() + (cPad ? ":pad" + std::to_string(cPad) : "") + (rowMerge ? ":rows" : "");
    View w;
    std::vector<Expr> wshape = wperm.shape;
    if (cPad) wshape[3] = Expr(cPad);
    if (rowMerge) wshape[2] = Expr(8);
    if (constVecCache.count(key)) { w = wperm; w.shape = wshape; w.buf = constVecCache[key]; w.offset = Expr(0); w.strides = rowMajor(wshape); }
    else if (cPad) {
      std::vector<Expr> rm = rowMajor(wshape);
      w = freshView(wperm.dtype, wshape, true, &rm);
      emitEltwise(constNode(0.0), w, true);
      View real = w; real.shape = wperm.shape;
      emitEltwise(leafNode(wperm), real, true);
      constVecCache[key] = w.buf;
    }
    else { std::vector<Expr> rm = rowMajor(wperm.shape); w = materializeTree(leafNode(wperm), wperm.dtype, wperm.shape, &rm); constVecCache[key] = w.buf; }
    if (rowMerge) {                          // [F, KH, 8, cPad] read as [F, KH, 1, 8 * cPad]
      w.shape = {wshape[0], wshape[1], Expr(1), Expr(8 * cPad)};
      w.strides = rowMajor(w.shape);
    }
    Expr N = xt.shape[0], H = xt.shape[2], W = xt.shape[3], F = wt.shape[0];
    int64_t KH = wt.shape[2].constant(), KW = wt.shape[3].constant();
    if (!wt.shape[2].isConst() || !wt.shape[3].isConst()) fail("symbolic kernel extent");
    // pad attr order: (top, left, bottom, right) as written by the importer (fx_op_translate/conv.py:48-57)
    Expr OH = windowOut(H, pad[0], pad[2], dil[0], KH, stride[0]);
    Expr OW = windowOut(W, pad[1], pad[3], dil[1], KW, stride[1]);
    std::vector<Expr> oshape = {N, F, OH, OW};
    DType dt = op->results[0]->type.elt;
    PendingK P;
    P.step.kernel = "conv";
    P.step.views.emplace_back("x", x);
    P.step.views.emplace_back("w", w);
    if (gemmPrecision(x.dtype) == "tf32x3" && w.dtype == DType::F32 && bufIsConst(w.buf) && isContiguous(w)) {
      View lo = materializeTree(opNode("tf32lo", leafNode(w)), DType::F32, w.shape);
      P.step.views.emplace_back("w_lo", lo);
    }
    auto arr = [](const std::vector<int64_t>& v) { std::string o; for (size_t i = 0; i < v.size(); ++i) o += (i ? "," : "") + std::to_string(v[i]); return o; };
    P.step.params.emplace_back("stride", arr(stride));
    P.step.params.emplace_back("pad", rowMerge ? arr({pad[0], 0, pad[2], 0}) : arr(pad));   // the copy holds the left and right padding
    P.step.params.emplace_back("dil", arr(dil));
    P.step.params.emplace_back("prec", gemmPrecision(x.dtype));
    // the contraction length of the convolution as written (the views above may carry padded channels or a zero tap)
    if (Cin.isConst()) P.step.params.emplace_back("kalg", std::to_string(KH * KW * Cin.constant()));
    std::vector<Expr> ost = nhwcStrides(oshape);
    P.nativeOut = freshView(dt, oshape, false, &ost);
    P.buf = P.nativeOut.buf;
    P.chanDim = 1;
    if (hasBias) {
      TV& bt = get(op->operands[2]); toView(bt);
      P.shiftRoot = leafNode(bt.view);
    }
    pend.push_back(P);
    TV t; t.kind = TV::Pending; t.pending = (int)pend.size() - 1; t.dtype = dt; t.shape = oshape; t.view = P.nativeOut;
    tvs[op->results[0]] = t;
  }
  void maxPool(Op* op) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    if (xt.shape.size() != 4) fail("llh.max_pool expects rank-4 input");
    auto stride = intArray(op, "stride", {1, 1}), pad = intArray(op, "pad", {0, 0, 0, 0}), dil = intArray(op, "dilation", {1, 1}), k = intArray(op, "kernel_shape");
    const Attr* cm = op->attr("ceil_mode");
    bool ceil = cm && cm->i;
    View x = viewWithStrides(xv, nhwcStrides(xt.shape));
    std::vector<Expr> oshape = {xt.shape[0], xt.shape[1], windowOut(xt.shape[2], pad[0], pad[2], dil[0], k[0], stride[0], ceil),
                                windowOut(xt.shape[3], pad[1], pad[3], dil[1], k[1], stride[1], ceil)};
    std::vector<Expr> ost = nhwcStrides(oshape);
    DType odt = resultDtype(op->results[0]);
    View out = freshView(odt, oshape, false, &ost);
    Step s; s.kernel = "maxpool";
    s.views.emplace_back("x", x); s.views.emplace_back("out", out);
    auto arr = [](const std::vector<int64_t>& v) { std::string o; for (size_t i = 0; i < v.size(); ++i) o += (i ? "," : "") + std::to_string(v[i]); return o; };
    s.params.emplace_back("kernel", arr(k)); s.params.emplace_back("stride", arr(stride));
    s.params.emplace_back("pad", arr(pad)); s.params.emplace_back("dil", arr(dil));
    plan.steps.push_back(s);
    tvs[op->results[0]] = makeView(out, false);
  }

  // ---- reductions
  // x viewed as [outer, R, inner]; out [outer, inner]
  View emitReduce(const View& x3, const std::string& kind, DType dt, bool isConst) {
    View out = freshView(dt, {x3.shape[0], x3.shape[2]}, isConst);
    Step s; s.kernel = "reduce"; s.init = plan.buffers[out.buf].kind == BufferDecl::Const;
    s.views.emplace_back("x", x3); s.views.emplace_back("out", out);
    s.params.emplace_back("op", kind);
    plan.steps.push_back(s);
    return out;
  }
  void reduce(Op* op, const std::string& kind) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    size_t r = xt.shape.size();
    std::vector<int64_t> axes = intArray(op, "axis");
    if (axes.empty()) { const Attr* a = op->attr("axis"); if (a && a->kind == Attr::Int) axes = {a->i}; }
    for (auto& a : axes) if (a < 0) a += (int64_t)r;
    std::sort(axes.begin(), axes.end());
    std::set<int64_t> ax(axes.begin(), axes.end());
    std::vector<Expr> kept;
    for (size_t d = 0; d < r; ++d) if (!ax.count((int64_t)d)) kept.push_back(xt.shape[d]);
    if (kept.empty()) kept.push_back(Expr(1));
    toView(xt);
    View x = xt.view;
    // permute reduced axes to a block: (kept-before..., reduced..., kept-after...) when they are adjacent, else move them last
    bool adjacent = true;
    for (size_t i = 1; i < axes.size(); ++i) if (axes[i] != axes[i - 1] + 1) adjacent = false;
    View x3;
    bool done = false;
    if (adjacent) {
      Expr outer(1), R(1), inner(1);
      for (size_t d = 0; d < r; ++d) { if ((int64_t)d < axes.front()) outer = outer * xt.shape[d]; else if ((int64_t)d > axes.back()) inner = inner * xt.shape[d]; else R = R * xt.shape[d]; }
      done = reshapeView(x, {outer, R, inner}, x3);
      if (!done) {
        // NHWC-style views: try (kept..., reduced...) order on strides
        View perm = x; perm.shape.clear(); perm.strides.clear();
        for (size_t d = 0; d < r; ++d) if (!ax.count((int64_t)d)) { perm.shape.push_back(x.shape[d]); perm.strides.push_back(x.strides[d]); }
        size_t nk = perm.shape.size();
        for (auto a : axes) { perm.shape.push_back(x.shape[a]); perm.strides.push_back(x.strides[a]); }
        // find any dim order in which the view is dense with the reduced dims forming one block
        std::vector<int> order;
        if (denseOrder(perm, order)) {
          // positions of reduced dims in the dense order must be adjacent
          std::vector<int> pos;
          for (size_t k = 0; k < order.size(); ++k) if ((size_t)order[k] >= nk) pos.push_back((int)k);
          bool blk = true; for (size_t i = 1; i < pos.size(); ++i) if (pos[i] != pos[i - 1] + 1) blk = false;
          bool keptOrdered = true; int last = -1;
          for (size_t k = 0; k < order.size(); ++k) if ((size_t)order[k] < nk) { if (order[k] < last) keptOrdered = false; last = order[k]; }
          if (blk && keptOrdered && !pos.empty()) {
            Expr o2(1), R2(1), i2(1);
            for (size_t k = 0; k < order.size(); ++k) { const Expr& e = perm.shape[order[k]]; if ((int)k < pos.front()) o2 = o2 * e; else if ((int)k > pos.back()) i2 = i2 * e; else R2 = R2 * e; }
            x3 = x; x3.shape = {o2, R2, i2}; x3.strides = {R2 * i2, i2, Expr(1)};
            done = true;
          }
        }
      }
    }
    if (!done) {
      View perm = x; perm.shape.clear(); perm.strides.clear();
      for (size_t d = 0; d < r; ++d) if (!ax.count((int64_t)d)) { perm.shape.push_back(x.shape[d]); perm.strides.push_back(x.strides[d]); }
      Expr R(1);
      for (auto a : axes) { perm.shape.push_back(x.shape[a]); perm.strides.push_back(x.strides[a]); R = R * x.shape[a]; }
      std::vector<Expr> rm = rowMajor(perm.shape);
      View dense = materializeTree(leafNode(perm), x.dtype, perm.shape, &rm);
      if (!reshapeView(dense, {numelOf(kept), R, Expr(1)}, x3)) fail("internal: reduce reshape");
    }
    View out = emitReduce(x3, kind, op->results[0]->type.elt, xt.isConst);
    View o2;
    if (!reshapeView(out, kept, o2)) fail("internal: reduce result reshape");
    tvs[op->results[0]] = makeView(o2, bufIsConst(o2.buf));
  }
  void adaptiveAvgPool(Op* op) {
    auto os = intArray(op, "out_size");
    if (os.size() != 2 || os[0] != 1 || os[1] != 1) fail("llh.adaptive_average_pool: only out_size [1,1] is supported");
    Value* xv = op->operands[0];
    TV& xt = get(xv); toView(xt);
    View x = xt.view, x3;
    Expr N = xt.shape[0], C = xt.shape[1], HW = xt.shape[2] * xt.shape[3];
    std::vector<Expr> nh = nhwcStrides(xt.shape);
    bool isNhwc = true;
    for (int d = 0; d < 4; ++d) if (!xt.shape[d].isConst(1) && x.strides[d] != nh[d]) isNhwc = false;
    View res;
    if (isNhwc) {
      x3 = x; x3.shape = {N, HW, C}; x3.strides = {HW * C, C, Expr(1)};
      View out = emitReduce(x3, "mean", op->results[0]->type.elt, false);   // [N, C]
      res = out; res.shape = {N, C, Expr(1), Expr(1)}; res.strides = {C, Expr(1), Expr(1), Expr(1)};
    } else {
      View xc = contiguousViewOf(xv);
      x3 = xc; x3.shape = {N * C, HW, Expr(1)}; x3.strides = {HW, Expr(1), Expr(1)};
      View out = emitReduce(x3, "mean", op->results[0]->type.elt, false);
      res = out; res.shape = {N, C, Expr(1), Expr(1)}; res.strides = {C, Expr(1), Expr(1), Expr(1)};
    }
    tvs[op->results[0]] = makeView(res, false);
  }

  void softmax(Op* op) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    size_t r = xt.shape.size();
    const Attr* a = op->attr("axis");
    int64_t axis = a ? a->i : (int64_t)r - 1;
    if (axis < 0) axis += (int64_t)r;
    if (axis != (int64_t)r - 1) fail("llh.softmax: only the last axis is supported");
    {
      TV& x0 = raw(xv);
      settle(x0);
      if (x0.kind == TV::Pending && xv->users.size() == 1 && attentionScores(x0)) {
        // scores of an attention: wait for the consumer before emitting anything
        AttnCand c; c.pending = x0.pending; attn.push_back(c);
        View out = freshView(resultDtype(op->results[0]), x0.shape, false);
        TV t; t.kind = TV::AttnProb; t.attn = (int)attn.size() - 1; t.pending = x0.pending; t.dtype = out.dtype; t.shape = x0.shape; t.view = out;
        tvs[op->results[0]] = t;
        return;
      }
    }
    View x = contiguousLeafOrView(xv);
    Expr rows(1); for (size_t d = 0; d + 1 < r; ++d) rows = rows * xt.shape[d];
    View x2 = x; x2.shape = {rows, xt.shape[r - 1]}; x2.strides = {xt.shape[r - 1], Expr(1)};
    View out = freshView(resultDtype(op->results[0]), xt.shape, false);
    View o2 = out; o2.shape = x2.shape; o2.strides = x2.strides;
    Step s; s.kernel = "softmax"; s.views.emplace_back("x", x2); s.views.emplace_back("out", o2);
    plan.steps.push_back(s);
    tvs[op->results[0]] = makeView(out, false);
  }
  void layerNorm(Op* op) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    size_t r = xt.shape.size();
    const Attr* a = op->attr("axis");
    int64_t axis = a ? a->i : (int64_t)r - 1;
    if (axis < 0) axis += (int64_t)r;
    const Attr* e = op->attr("epsilon");
    View x = contiguousLeafOrView(xv);
    Expr rows(1), D(1);
    for (size_t d = 0; d < r; ++d) { if ((int64_t)d < axis) rows = rows * xt.shape[d]; else D = D * xt.shape[d]; }
    View x2 = x; x2.shape = {rows, D}; x2.strides = {D, Expr(1)};
    View g = contiguousViewOf(op->operands[1]), b = contiguousViewOf(op->operands[2]);
    g.shape = {D}; g.strides = {Expr(1)}; b.shape = {D}; b.strides = {Expr(1)};
    View out = freshView(resultDtype(op->results[0]), xt.shape, false);
    View o2 = out; o2.shape = x2.shape; o2.strides = x2.strides;
    Step s; s.kernel = "layernorm";
    s.views.emplace_back("x", x2); s.views.emplace_back("gamma", g); s.views.emplace_back("beta", b); s.views.emplace_back("out", o2);
    s.params.emplace_back("eps", fmtDouble(e ? e->f : 1e-5));
    plan.steps.push_back(s);
    tvs[op->results[0]] = makeView(out, false);
  }
  void embedding(Op* op) {
    View table = contiguousViewOf(op->operands[0]);
    View ids = contiguousViewOf(op->operands[1]);
    TV& it = raw(op->operands[1]);
    if (table.rank() != 2) fail("llh.embedding expects a rank-2 table");
    std::vector<Expr> oshape = it.shape; oshape.push_back(table.shape[1]);
    Expr rows = numelOf(it.shape);
    View idf = ids; idf.shape = {rows}; idf.strides = {Expr(1)};
    View out = freshView(resultDtype(op->results[0]), oshape, false);
    View o2 = out; o2.shape = {rows, table.shape[1]}; o2.strides = {table.shape[1], Expr(1)};
    Step s; s.kernel = "gather";
    s.views.emplace_back("table", table); s.views.emplace_back("ids", idf); s.views.emplace_back("out", o2);
    plan.steps.push_back(s);
    tvs[op->results[0]] = makeView(out, false);
  }
  void batchNormInference(Op* op) {
    // y = (x - mean) * gamma / sqrt(var + eps) + beta (src/Dialect/LLH/Transforms/DecomposeOps.cpp:125-144),
    // restated as a per-channel scale/shift computed once at load: scale = gamma / sqrt(var + eps),
    // shift = beta - mean * scale.
    const Attr* e = op->attr("epsilon");
    const Attr* fi = op->attr("feature_index");
    int64_t f = fi ? fi->i : 1;
    double eps = e ? e->f : 1e-5;
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    std::vector<View> p;
    for (int i = 1; i <= 4; ++i) { TV& t = get(op->operands[i]); toView(t); View v = t.view; if (v.rank() != 1) fail("batch_norm parameters must be rank 1"); p.push_back(v); }
    int gamma = leafNode(p[0]), beta = leafNode(p[1]), mean = leafNode(p[2]), var = leafNode(p[3]);
    int scale = opNode("div", gamma, opNode("sqrt", opNode("add", var, constNode(eps))));
    int shift = opNode("sub", beta, opNode("mul", mean, scale));
    settle(xt);
    if (xt.kind == TV::Pending && xv->users.size() == 1) {
      PendingK& P = pend[xt.pending];
      int cd = -1;
      for (size_t d = 0; d < xt.view.rank(); ++d) if (xt.view.strides[d].isConst(1) && xt.view.shape[d] == P.nativeOut.shape[P.chanDim]) cd = (int)d;
      if (P.stage == 0 && cd == f) {
        P.shiftRoot = P.shiftRoot < 0 ? shift : opNode("add", opNode("mul", P.shiftRoot, scale), shift);
        P.scaleRoot = P.scaleRoot < 0 ? scale : opNode("mul", P.scaleRoot, scale);
        TV r = xt; r.dtype = op->results[0]->type.elt; tvs[op->results[0]] = r;
        return;
      }
    }
    // general case: one fused elementwise pass with the vectors broadcast along feature_index
    std::vector<Expr> shape = xt.shape;
    // the vectors are materialised once (load time), then broadcast
    View sv = materializeTree(scale, DType::F32, {shape[f]}), hv = materializeTree(shift, DType::F32, {shape[f]});
    int xn = operandNode(xt, shape);
    int sn = leafNode(broadcastView(sv, shape, {f})), hn = leafNode(broadcastView(hv, shape, {f}));
    tvs[op->results[0]] = makeLazy(opNode("add", opNode("mul", xn, sn), hn), op->results[0]->type.elt, shape);
  }

  // ---- data movement
  void reshapeTo(Op* op, const std::vector<Expr>& target) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    std::vector<Expr> shape = target;
    // one -1 extent is inferred (LLHCanonicalize.cpp reshape handling)
    int neg = -1; Expr known(1);
    for (size_t d = 0; d < shape.size(); ++d) { if (shape[d].isConst(-1)) neg = (int)d; else known = known * shape[d]; }
    if (neg >= 0) shape[neg] = numelOf(xt.shape).floordiv(known);
    TV r; r.dtype = op->results[0]->type.elt == DType::None ? xt.dtype : xt.dtype; r.shape = shape; r.isConst = xt.isConst;
    settle(xt);
    if (xt.kind == TV::Lazy) {
      std::map<int, int> memo; bool ok = true;
      int root = mapLeaves(xt.root, [&](const View& l, View& o) { return reshapeView(l, shape, o); }, memo, ok);
      if (ok) { tvs[op->results[0]] = makeLazy(root, xt.dtype, shape); return; }
      toView(xt);
    }
    if (xt.kind == TV::Deferred) toView(xt);
    View nv;
    bool viewOk = reshapeView(xt.view, shape, nv);
    if (!viewOk && (xt.kind == TV::ViewK) && isContiguous(xt.view)) {
      // a dense row-major source takes any shape of the same element count, whether or not the equality of the
      // symbolic products can be proved here (the module asserts it by construction)
      nv = xt.view; nv.shape = shape; nv.strides = rowMajor(shape); viewOk = true;
    }
    if (viewOk) {
      r.kind = xt.kind; r.view = nv; r.pending = xt.pending; r.attn = xt.attn;
      tvs[op->results[0]] = r; return;
    }
    if (xt.kind == TV::Pending && xv->users.size() == 1 && relayoutPending(xt) && reshapeView(xt.view, shape, nv)) {
      r.kind = xt.kind; r.view = nv; r.pending = xt.pending;
      tvs[op->results[0]] = r; return;
    }
    if (xt.kind == TV::Pending || xt.kind == TV::AttnProb) toView(xt);
    r.kind = TV::Deferred; r.view = xt.view;
    tvs[op->results[0]] = r;
  }
  // A GEMM result that has only been permuted so far (attention's [B,H,S,D] -> [B,S,H,D]) and is now
  // reshaped: nothing has been emitted yet, so the kernel can write its tile rows straight into the
  // permuted order (it takes arbitrary batch and row strides) and the copy disappears.
  bool relayoutPending(TV& t) {
    PendingK& P = pend[t.pending];
    if (P.emitted || (P.step.kernel != "gemm" && P.step.kernel != "attention") || P.hasRes || !t.view.offset.isConst(0)) return false;
    const View& nat = P.nativeOut;
    std::vector<int> logicalOf(nat.rank(), -1);
    std::vector<bool> used(t.view.rank(), false);
    for (size_t d = 0; d < nat.rank(); ++d) {
      if (nat.shape[d].isConst(1)) continue;
      for (size_t l = 0; l < t.view.rank(); ++l)
        if (!used[l] && !t.view.shape[l].isConst(1) && t.view.shape[l] == nat.shape[d] && t.view.strides[l] == nat.strides[d]) { logicalOf[d] = (int)l; used[l] = true; break; }
      if (logicalOf[d] < 0) return false;
    }
    for (size_t l = 0; l < t.view.rank(); ++l) if (!used[l] && !t.view.shape[l].isConst(1)) return false;
    std::vector<Expr> fresh = rowMajor(t.view.shape);
    const size_t nDim = nat.rank() - 1;
    if (logicalOf[nDim] >= 0 && !fresh[logicalOf[nDim]].isConst(1)) return false;   // the kernel needs unit stride along n
    for (size_t d = 0; d < nat.rank(); ++d) if (logicalOf[d] >= 0) P.nativeOut.strides[d] = fresh[logicalOf[d]];
    t.view.strides = fresh;
    return true;
  }
  void transpose(Op* op) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    std::vector<int64_t> perms = intArray(op, "perms");
    if (perms.size() != xt.shape.size()) fail("llh.transpose: perms rank mismatch");
    auto permute = [&](const View& v) { View o = v; for (size_t i = 0; i < perms.size(); ++i) { o.shape[i] = v.shape[perms[i]]; o.strides[i] = v.strides[perms[i]]; } return o; };
    settle(xt);
    if (xt.kind == TV::Deferred) toView(xt);
    std::vector<Expr> shape(perms.size());
    for (size_t i = 0; i < perms.size(); ++i) shape[i] = xt.shape[perms[i]];
    if (xt.kind == TV::Lazy) {
      std::map<int, int> memo; bool ok = true;
      int root = mapLeaves(xt.root, [&](const View& l, View& o) { o = permute(l); return true; }, memo, ok);
      tvs[op->results[0]] = makeLazy(root, xt.dtype, shape); return;
    }
    TV r = xt; r.shape = shape; r.view = permute(xt.view);
    tvs[op->results[0]] = r;
  }
  void broadcastTo(Op* op) {
    Value* xv = op->operands[0];
    TV& xt = get(xv);
    std::vector<Expr> shape;
    for (size_t i = 1; i < op->operands.size(); ++i) shape.push_back(scalarOf(op->operands[i]));
    std::vector<int64_t> cast = intArray(op, "cast_dims");
    if (cast.empty()) for (size_t i = 0; i < xt.shape.size(); ++i) cast.push_back((int64_t)(shape.size() - xt.shape.size() + i));
    settle(xt);
    // dims that are already the target extent keep the producer's name for them
    for (size_t i = 0; i < xt.shape.size(); ++i) if (!xt.shape[i].isConst(1)) shape[cast[i]] = xt.shape[i];
    if (xt.kind == TV::Lazy) {
      std::map<int, int> memo; bool ok = true;
      int root = mapLeaves(xt.root, [&](const View& l, View& o) { o = broadcastView(l, shape, cast); return true; }, memo, ok);
      tvs[op->results[0]] = makeLazy(root, xt.dtype, shape); return;
    }
    if ((xt.kind == TV::Pending || xt.kind == TV::AttnProb) && xt.shape.size() == shape.size()) {   // identity broadcast keeps the producer open
      bool same = true; for (size_t i = 0; i < shape.size(); ++i) if (cast[i] != (int64_t)i || xt.shape[i] != shape[i]) same = false;
      if (same) { TV r = xt; tvs[op->results[0]] = r; return; }
    }
    if (xt.kind == TV::Deferred && xt.shape.size() == shape.size()) {
      bool same = true; for (size_t i = 0; i < shape.size(); ++i) if (cast[i] != (int64_t)i || xt.shape[i] != shape[i]) same = false;
      if (same) { TV r = xt; tvs[op->results[0]] = r; return; }
    }
    toView(xt);
    tvs[op->results[0]] = makeView(broadcastView(xt.view, shape, cast), xt.isConst);
  }
  void strideSlice(Op* op) {
    Value* xv = op->operands[0];
    View x = viewOf(xv);
    size_t r = x.rank();
    if (op->operands.size() != 1 + 3 * r) fail("llh.stride_slice: expects starts, ends and strides for every dim");
    View o = x;
    for (size_t d = 0; d < r; ++d) {
      Expr st = scalarOf(op->operands[1 + d]), en = scalarOf(op->operands[1 + r + d]), sp = scalarOf(op->operands[1 + 2 * r + d]);
      if (en.isConst() && en.constant() >= (int64_t)1 << 62) en = x.shape[d];
      if (st.isConst() && st.constant() < 0) st = st + x.shape[d];
      if (en.isConst() && en.constant() < 0) en = en + x.shape[d];
      o.offset = o.offset + st * x.strides[d];
      o.shape[d] = (en - st).ceildiv(sp);
      if (!(o.shape[d] == x.shape[d]))
        noteRelation(o.shape[d], sp.isConst(1) ? "(d0)[s0, s1] -> (s0 - s1)" : "(d0)[s0, s1, s2] -> ((s0 - s1) ceildiv s2)", sp.isConst(1) ? std::vector<Expr>{en, st} : std::vector<Expr>{en, st, sp});
      o.strides[d] = x.strides[d] * sp;
    }
    tvs[op->results[0]] = makeView(o, raw(xv).isConst);
  }
  // llh.cat (LLHOps.td: CatOp, `dim` attribute): the result is one buffer, every operand is written into its range of it
  // along `dim` by an elementwise step of its own (a lazy operand is evaluated straight into its range).
  void cat(Op* op) {
    if (op->operands.empty()) fail("llh.cat without operands");
    const Attr* da = op->attr("dim");
    std::vector<TV*> ts;
    for (Value* v : op->operands) { TV& t = get(v); settle(t); ts.push_back(&t); }
    const size_t r = ts[0]->shape.size();
    int64_t dim = da ? da->i : 0;
    if (dim < 0) dim += (int64_t)r;
    if (dim < 0 || dim >= (int64_t)r) fail("llh.cat: dim out of range");
    std::vector<Expr> shape = ts[0]->shape;
    Expr along(0);
    for (TV* t : ts) {
      if (t->shape.size() != r) fail("llh.cat: operands of different rank");
      for (size_t d = 0; d < r; ++d) if ((int64_t)d != dim && !(t->shape[d] == shape[d])) fail("llh.cat: operands differ outside the concatenated dim");
      along = along + t->shape[dim];
    }
    shape[dim] = along;
    DType dt = op->results[0]->type.elt == DType::None ? ts[0]->dtype : op->results[0]->type.elt;
    bool allConst = true;
    for (TV* t : ts) allConst = allConst && t->isConst;
    if (shapesOnly) { TV t; t.kind = TV::ViewK; t.dtype = dt; t.shape = shape; tvs[op->results[0]] = t; return; }
    View out = freshView(dt, shape, allConst);
    Expr at(0);
    for (TV* t : ts) {
      View part = out;
      part.offset = out.offset + at * out.strides[dim];
      part.shape = t->shape;
      emitEltwise(operandNode(*t, t->shape), part, allConst && numelOf(shape).isConst());
      at = at + t->shape[dim];
    }
    tvs[op->results[0]] = makeView(out, allConst);
  }
  void extract(Op* op) {
    View x = viewOf(op->operands[0]);
    Expr idx = scalarOf(op->operands[1]);
    if (idx.isConst() && idx.constant() < 0) idx = idx + x.shape[0];
    View o = x;
    o.offset = o.offset + idx * x.strides[0];
    o.shape.erase(o.shape.begin()); o.strides.erase(o.strides.begin());
    if (o.shape.empty()) { o.shape.push_back(Expr(1)); o.strides.push_back(Expr(1)); }
    tvs[op->results[0]] = makeView(o, raw(op->operands[0]).isConst);
  }

  // ---- constants / arguments
  void constant(Op* op) {
    const Attr* a = op->attr("value");
    if (!a) fail("llh.constant without value");
    Value* res = op->results[0];
    if (a->kind == Attr::Int || a->kind == Attr::Bool) {
      TV t; t.kind = TV::Scalar; t.scalar = Expr(a->i); t.dtype = DType::I64; t.isConst = true; tvs[res] = t; return;
    }
    if (a->kind == Attr::Float) { TV t; t.kind = TV::Scalar; t.isFloatScalar = true; t.fscalar = a->f; t.dtype = DType::F32; t.isConst = true; tvs[res] = t; return; }
    if (a->kind != Attr::Dense) fail("unsupported llh.constant value");
    std::vector<Expr> shape;
    for (auto d : a->type.dims) shape.push_back(Expr(d));
    if (shape.empty()) shape.push_back(Expr(1));
    bool isF = isFloat(a->type.elt);
    size_t n = isF ? a->floats.size() : a->ints.size();
    if (n == 1) { tvs[res] = makeLazy(constNode(isF ? a->floats[0] : (double)a->ints[0]), a->type.elt, shape); return; }
    View v = freshView(a->type.elt, shape, true);
    plan.buffers[v.buf].kind = BufferDecl::Const;
    for (size_t k = 0; k < n; ++k) plan.buffers[v.buf].values.push_back(isF ? a->floats[k] : (double)a->ints[k]);
    tvs[res] = makeView(v, true);
  }
  void weight(Op* op) {
    const Attr* f = op->attr("weight_file");
    if (!f) fail("llh.weight without weight_file");
    const Type& t = op->results[0]->type;
    std::vector<Expr> shape;
    for (auto d : t.dims) { if (d == kDynamic) fail("llh.weight with a dynamic extent"); shape.push_back(Expr(d)); }
    if (shape.empty()) shape.push_back(Expr(1));
    View v = freshView(t.elt, shape, true);
    plan.buffers[v.buf].kind = BufferDecl::Weight;
    plan.buffers[v.buf].file = f->s;
    tvs[op->results[0]] = makeView(v, true);
  }
  void scalarBinary(Op* op, const std::string& name) {
    Expr a = scalarOf(op->operands[0]), b = scalarOf(op->operands[1]);
    TV t; t.kind = TV::Scalar; t.dtype = DType::I64; t.isConst = true;
    if (name == "add") t.scalar = a + b; else if (name == "sub") t.scalar = a - b; else if (name == "mul") t.scalar = a * b;
    else if (name == "div") t.scalar = a.floordiv(b); else fail("unsupported scalar op llh." + name);
    const char* sign = name == "add" ? "+" : name == "sub" ? "-" : name == "mul" ? "*" : "floordiv";
    noteRelation(t.scalar, std::string("(d0)[s0, s1] -> (s0 ") + sign + " s1)", {a, b});
    tvs[op->results[0]] = t;
  }

  void bindArguments(Func& f) {
    int symArgs = 0, tensorArgs = 0, fresh = 0;
    std::set<std::string> seen;
    for (size_t i = 0; i < f.args.size(); ++i) {
      Value* a = f.args[i];
      const AttrList& attrs = i < f.argAttrs.size() ? f.argAttrs[i] : AttrList();
      if (a->type.kind == Type::Scalar) {
        const Attr* s = findAttr(attrs, "func.symbol_int");
        std::string name = s ? s->s : "s" + std::to_string(fresh++);
        TV t; t.kind = TV::Scalar; t.dtype = DType::I64;
        if (name.size() > 1 && name[0] == 'c' && std::isdigit((unsigned char)name[1])) t.scalar = Expr(std::stoll(name.substr(1)));
        else { t.scalar = Expr::sym(name); SymbolBinding b; b.name = name; b.symbolArg = symArgs; plan.symbols.push_back(b); }
        ++symArgs;
        tvs[a] = t;
        continue;
      }
      if (!a->type.isTensor()) fail("unsupported argument type");
      std::vector<Expr> shape;
      for (size_t d = 0; d < a->type.dims.size(); ++d) {
        const Attr* s = findAttr(attrs, "func.input_symbol_" + std::to_string(d));
        std::string name = s ? s->s : "";
        if (a->type.dims[d] != kDynamic) { shape.push_back(Expr(a->type.dims[d])); continue; }
        // an encoding the argument's type already carries names the extent (text that went through infer-symbol-shape before)
        if (name.empty() && d < a->type.encoding.size()) {
          const std::string& e = a->type.encoding[d];
          bool plain = !e.empty() && (isalpha((unsigned char)e[0]) || e[0] == '_');
          for (char ch : e) if (!isalnum((unsigned char)ch) && ch != '_') plain = false;
          if (plain) name = e;
        }
        if (name.empty()) { do name = "s" + std::to_string(fresh++); while (seen.count(name)); }
        seen.insert(name);
        if (name[0] == 'c' && name.size() > 1 && std::isdigit((unsigned char)name[1])) { shape.push_back(Expr(std::stoll(name.substr(1)))); continue; }
        // a torch symbol expression such as "2*s0" cannot name an input extent; plain names only
        shape.push_back(Expr::sym(name));
        SymbolBinding b; b.name = name; b.input = tensorArgs; b.dim = (int)d; plan.symbols.push_back(b);
      }
      if (shape.empty()) shape.push_back(Expr(1));
      View v; v.dtype = a->type.elt; v.shape = shape; v.strides = rowMajor(shape);
      v.buf = newBuffer(a->type.elt, numelOf(shape), BufferDecl::Input);
      plan.buffers[v.buf].index = tensorArgs;
      IoDecl io; io.buf = v.buf; io.dtype = a->type.elt; io.shape = shape;
      plan.inputs.push_back(io);
      ++tensorArgs;
      tvs[a] = makeView(v, false);
    }
    plan.numSymbolArgs = symArgs;
  }

  void finishOutputs(Op* ret) {
    std::set<int> taken;
    for (size_t k = 0; k < ret->operands.size(); ++k) {
      Value* v = ret->operands[k];
      TV& t = raw(v);
      settle(t);
      if (t.kind == TV::Scalar) fail("returning scalars is not supported");
      // the caller allocates the result with the declared element type
      const DType want = v->type.elt;
      if (want != DType::None && want != t.dtype) {
        if (t.kind == TV::Pending && v->users.size() == 1 && isFloat(want) && isFloat(t.dtype)) {
          PendingK& P = pend[t.pending];
          P.nativeOut.dtype = want; plan.buffers[P.buf].dtype = want; t.dtype = want; t.view.dtype = want;
        } else if (t.kind == TV::Lazy) {
          t.dtype = want;
        } else {
          toView(t);
          TV conv = makeLazy(opNode("cast", leafNode(t.view)), want, t.shape);
          t = conv;
        }
      }
      IoDecl io; io.dtype = t.dtype; io.shape = t.shape;
      std::vector<Expr> rm = rowMajor(t.shape);
      bool direct = false;
      if (t.kind == TV::Pending && v->users.size() == 1 && isContiguous(t.view) && t.view.offset.isConst(0) && !taken.count(t.view.buf)) {
        plan.buffers[t.view.buf].kind = BufferDecl::Output; plan.buffers[t.view.buf].index = (int)k;
        emitPending(t.pending); settle(t);
        io.buf = t.view.buf; direct = true;
      } else if (t.kind == TV::Lazy && nodes[t.root].kind != ENode::Leaf) {
        int buf = newBuffer(t.dtype, numelOf(t.shape), BufferDecl::Output);
        plan.buffers[buf].index = (int)k;
        materializeTree(t.root, t.dtype, t.shape, &rm, buf);
        io.buf = buf; direct = true;
      }
      if (!direct) {
        toView(t);
        const BufferDecl& b = plan.buffers[t.view.buf];
        if (b.kind == BufferDecl::Temp && isContiguous(t.view) && t.view.offset.isConst(0) && b.numel == numelOf(t.shape) && !taken.count(t.view.buf)) {
          plan.buffers[t.view.buf].kind = BufferDecl::Output; plan.buffers[t.view.buf].index = (int)k;
          io.buf = t.view.buf;
        } else {
          int buf = newBuffer(t.dtype, numelOf(t.shape), BufferDecl::Output);
          plan.buffers[buf].index = (int)k;
          materializeTree(leafNode(t.view), t.dtype, t.shape, &rm, buf);
          io.buf = buf;
        }
      }
      taken.insert(io.buf);
      plan.outputs.push_back(io);
    }
  }

  void run() {
    Func* f = m.entrance();
    if (!f) fail("module has no function");
    m.recomputeUsers();
    bindArguments(*f);
    static const std::set<std::string> binary = {"add", "sub", "mul", "div", "max", "min", "pow"};
    static const std::set<std::string> unary = {"relu", "abs", "sqrt", "rsqrt", "exp", "gelu", "tanh", "erf", "sigmoid", "neg"};
    for (Op* op : f->ops) {
      if (op->erased) continue;
      const std::string& n = op->name;
      if (n == "func.return") { if (!shapesOnly) finishOutputs(op); continue; }
      if (n.compare(0, 4, "llh.") != 0) fail("operation '" + n + "' is not part of the LLH surface");
      std::string s = n.substr(4);
      if (s == "constant") constant(op);
      else if (s == "weight") weight(op);
      else if (s == "empty") {           // uninitialised storage of the given extents (LLHOps.td: llh.empty)
        std::vector<Expr> shape;
        for (Value* d : op->operands) shape.push_back(scalarOf(d));
        DType dt = op->results[0]->type.elt == DType::None ? DType::F32 : op->results[0]->type.elt;
        tvs[op->results[0]] = makeView(freshView(dt, shape, false), false);
      }
      else if (s == "torch_symbolic_int" || s == "symbolic_int") {
        const Attr* a = op->attr("sym_name");
        if (!a) fail("symbolic int without sym_name");
        if (op->results.empty()) continue;
        TV t; t.kind = TV::Scalar; t.dtype = DType::I64;
        t.scalar = (a->s.size() > 1 && a->s[0] == 'c' && std::isdigit((unsigned char)a->s[1])) ? Expr(std::stoll(a->s.substr(1))) : Expr::sym(a->s);
        tvs[op->results[0]] = t;
      }
      else if (s == "dim") {
        TV& x = raw(op->operands[0]);
        Expr d = scalarOf(op->operands[1]);
        if (!d.isConst()) fail("llh.dim with a symbolic index");
        int64_t k = d.constant(); if (k < 0) k += (int64_t)x.shape.size();
        if (k < 0 || k >= (int64_t)x.shape.size()) fail("llh.dim index out of range");
        TV t; t.kind = TV::Scalar; t.dtype = DType::I64; t.scalar = x.shape[k]; tvs[op->results[0]] = t;
      }
      else if (binary.count(s)) {
        if (op->results[0]->type.kind == Type::Scalar) scalarBinary(op, s); else eltwise(op, s);
      }
      else if (unary.count(s)) eltwise(op, s);
      else if (s == "where") eltwise(op, "where");
      else if (s == "compare") {
        const Attr* k = op->attr("kind");
        std::string kind = k ? k->s : "EQ";
        for (auto& c : kind) c = (char)std::tolower((unsigned char)c);
        eltwise(op, kind);
      }
      else if (s == "convert_to") {
        TV& x = get(op->operands[0]);
        if (x.kind == TV::Scalar) { tvs[op->results[0]] = x; continue; }
        DType to = op->results[0]->type.elt;
        if (to == x.dtype) { TV c = x; tvs[op->results[0]] = c; continue; }
        if (isFloat(to) && isFloat(x.dtype)) {
          // float -> float: arithmetic is fp32 everywhere, only the storage type of whatever is
          // materialised next changes, so the conversion does not break a fusion
          settle(x);
          if (x.kind == TV::AttnProb) {      // probabilities keep whatever storage type is the narrowest asked for
            TV r = x;
            if (dtypeSize(to) < dtypeSize(x.dtype)) { r.dtype = to; r.view.dtype = to; plan.buffers[r.view.buf].dtype = to; }
            tvs[op->results[0]] = r; continue;
          }
          // widening (bf16 -> f32) of stored data is exact: keep the narrow storage and let the
          // consumers read it as it is (they all compute in fp32)
          if (dtypeSize(to) > dtypeSize(x.dtype) && (x.kind == TV::Pending || x.kind == TV::ViewK || x.kind == TV::Deferred)) {
            TV c = x; tvs[op->results[0]] = c; continue;
          }
          if (x.kind == TV::Pending && op->operands[0]->users.size() == 1) {
            PendingK& P = pend[x.pending];
            P.nativeOut.dtype = to; plan.buffers[P.buf].dtype = to;
            TV r = x; r.dtype = to; r.view.dtype = to; tvs[op->results[0]] = r; continue;
          }
          if (x.kind == TV::Lazy) { TV r = x; r.dtype = to; tvs[op->results[0]] = r; continue; }
          toView(x);
          tvs[op->results[0]] = makeLazy(leafNode(x.view), to, x.shape); continue;
        }
        int node = operandNode(x, x.shape);
        tvs[op->results[0]] = makeLazy(opNode(isFloat(to) ? "cast" : "trunc", node), to, x.shape);
      }
      else if (s == "scalar_cast") {
        TV& x = raw(op->operands[0]);
        if (x.kind != TV::Scalar) fail("llh.scalar_cast expects a scalar");
        if (op->results[0]->type.isTensor()) {
          if (!x.isFloatScalar && !x.scalar.isConst()) fail("llh.scalar_cast of a symbolic value to a tensor is not supported");
          tvs[op->results[0]] = makeLazy(constNode(x.isFloatScalar ? x.fscalar : (double)x.scalar.constant()), op->results[0]->type.elt, {Expr(1)});
        } else { TV c = x; tvs[op->results[0]] = c; }
      }
      else if (s == "matmul") gemm(op, false);
      else if (s == "batch_matmul") gemm(op, true);
      else if (s == "conv") conv(op, false);
      else if (s == "conv_bias") conv(op, true);
      else if (s == "batch_norm_inference") batchNormInference(op);
      else if (s == "batch_norm" && shapesOnly) {       // shapes only: the result has the input's shape, the statistics keep their declared types
        TV x = get(op->operands[0]);
        for (size_t i = 0; i < op->results.size(); ++i) {
          TV t; t.kind = TV::ViewK; t.dtype = op->results[i]->type.elt;
          if (i == 0) t.shape = x.shape; else for (auto d : op->results[i]->type.dims) t.shape.push_back(Expr(d));
          tvs[op->results[i]] = t;
        }
      }
      else if (s == "max_pool") maxPool(op);
      else if (s == "adaptive_average_pool") adaptiveAvgPool(op);
      else if (s == "reduce_sum") reduce(op, "sum");
      else if (s == "reduce_max") reduce(op, "max");
      else if (s == "reduce_min") reduce(op, "min");
      else if (s == "reduce_mean") reduce(op, "mean");
      else if (s == "softmax") softmax(op);
      else if (s == "layer_norm") layerNorm(op);
      else if (s == "embedding") embedding(op);
      else if (s == "reshape") { std::vector<Expr> t; for (size_t i = 1; i < op->operands.size(); ++i) t.push_back(scalarOf(op->operands[i])); reshapeTo(op, t); }
      else if (s == "flatten") {
        TV& x = raw(op->operands[0]);
        int64_t d = scalarOf(op->operands[1]).constant(); if (d < 0) d += (int64_t)x.shape.size();
        Expr lo(1), hi(1);
        for (size_t i = 0; i < x.shape.size(); ++i) { if ((int64_t)i < d) lo = lo * x.shape[i]; else hi = hi * x.shape[i]; }
        reshapeTo(op, d == 0 ? std::vector<Expr>{hi} : std::vector<Expr>{lo, hi});
      }
      else if (s == "transpose") transpose(op);
      else if (s == "broadcast_to" || s == "expand") broadcastTo(op);
      else if (s == "stride_slice") strideSlice(op);
      else if (s == "cat") cat(op);
      else if (s == "extract") extract(op);
      else if (s == "symbolic_bind" || s == "encoding_bind" || s == "symbol_bind" || s == "print" || s == "aot" ||
               s == "symbol_relation" || s == "symbol_relation_map" || s == "symbol_binary_relation") continue;
      else if (s == "drop") { TV c = get(op->operands[0]); tvs[op->results[0]] = c; }   // inference: identity
      else fail("no CUDA lowering for '" + n + "'");
    }
    if (!shapesOnly && opts.fuseSiblingGemms) fuseSiblingGemms();
    plan.options["precision"] = opts.precision;
    plan.options["mode"] = opts.mode;
    plan.options["target"] = opts.target;
  }

  // ---- sibling GEMMs
  // Several linear layers that read the same activation (the query, key and value projections of an attention layer)
  // become one GEMM: the weights are stacked once at load into [G*N, K], the bias vectors into [G*N], the product is
  // written as [M, G*N], and every later reader of one of the original outputs gets the matching column range of that
  // buffer as a strided view.  One launch with a G times wider N keeps the tensor pipe busier than G launches do
  // (measured on B200, bf16, M = 98304, K = 768: 1302 TFLOP/s at N = 2304 against 1144 at N = 768).
  struct SiblingGemm {
    View a, b, out, shift;
    bool hasShift = false;
    int64_t N = 0, K = 0;
  };
  bool siblingCandidate(const Step& s, SiblingGemm& g) const {
    if (s.kernel != "gemm" || s.init) return false;
    const View *a = s.view("a"), *b = s.view("b"), *o = s.view("out"), *sh = s.view("shift");
    if (!a || !b || !o) return false;
    for (auto& v : s.views) if (v.first != "a" && v.first != "b" && v.first != "out" && v.first != "shift") return false;
    if (s.param("act") != "none" || s.param("prec") == "tf32x3") return false;
    if (std::stod(s.param("alpha", "1")) != 1.0) return false;
    if (a->rank() != 4 || b->rank() != 4 || o->rank() != 4) return false;
    if (!a->shape[0].isConst(1) || !a->shape[1].isConst(1) || !b->shape[0].isConst(1) || !b->shape[1].isConst(1)) return false;
    if (!b->shape[2].isConst() || !b->shape[3].isConst() || !b->offset.isConst() || !bufIsConst(b->buf)) return false;
    g.K = b->shape[2].constant(); g.N = b->shape[3].constant();
    if (!b->strides[2].isConst(1) || !b->strides[3].isConst(g.K)) return false;        // the weight as stored: [N][K]
    if (g.N % 64 || g.K % 64) return false;
    if (plan.buffers[o->buf].kind != BufferDecl::Temp || !o->offset.isConst(0) || o->strides != rowMajor(o->shape) || !o->shape[3].isConst(g.N)) return false;
    if (sh) {
      if (sh->rank() != 1 || !sh->shape[0].isConst(g.N) || !sh->strides[0].isConst(1) || sh->dtype != DType::F32 || !bufIsConst(sh->buf)) return false;
      g.shift = *sh; g.hasShift = true;
    }
    g.a = *a; g.b = *b; g.out = *o;
    return true;
  }
  // A view over one of the original [M, N] outputs, restated over the fused [M, G*N] buffer (column block j): every dim
  // must either step through whole rows or stay inside one row.
  bool remapIntoFused(View& v, int64_t N, int64_t G, int64_t j, int fusedBuf) const {
    if (!v.offset.isConst()) return false;
    const int64_t off = v.offset.constant(), col0 = off % N;
    int64_t colSpan = col0;
    View r = v;
    for (size_t d = 0; d < v.rank(); ++d) {
      if (v.shape[d].isConst(1)) { r.strides[d] = Expr(0); continue; }
      if (!v.strides[d].isConst()) return false;
      const int64_t st = v.strides[d].constant();
      if (st % N == 0) { r.strides[d] = Expr(st / N * G * N); continue; }
      if (st < 0 || !v.shape[d].isConst()) return false;
      colSpan += (v.shape[d].constant() - 1) * st;
    }
    if (colSpan >= N) return false;
    r.offset = Expr(off / N * G * N + col0 + j * N);
    r.buf = fusedBuf;
    v = r;
    return true;
  }
  void fuseSiblingGemms() {
    for (size_t i = 0; i < plan.steps.size(); ++i) {
      SiblingGemm g0;
      if (!siblingCandidate(plan.steps[i], g0)) continue;
      std::vector<size_t> group = {i};
      std::vector<SiblingGemm> gs = {g0};
      for (size_t j = i + 1; j < plan.steps.size() && group.size() < 4; ++j) {
        const Step& sj = plan.steps[j];
        if (sj.init) continue;
        if (const View* o = sj.view("out")) if (o->buf == g0.a.buf) break;       // the activation is overwritten: stop looking
        SiblingGemm g;
        if (!siblingCandidate(sj, g)) continue;
        if (g.a.str() != g0.a.str() || g.N != g0.N || g.K != g0.K || g.b.dtype != g0.b.dtype || g.out.dtype != g0.out.dtype || g.hasShift != g0.hasShift ||
            sj.param("prec") != plan.steps[i].param("prec") || !(g.out.shape[2] == g0.out.shape[2]))
          continue;
        group.push_back(j); gs.push_back(g);
      }
      if (group.size() < 2) continue;
      bool isOutput = false;
      for (auto& g : gs) for (auto& o : plan.outputs) isOutput = isOutput || o.buf == g.out.buf;
      if (isOutput) continue;
      // every reader of the original outputs must be expressible over the fused buffer; checked before anything changes.
      // A group that does not work out is tried again without its last member.
      int64_t G = 0;
      const int64_t N = g0.N, K = g0.K;
      int fusedBuf = -1;
      std::vector<std::pair<View*, View>> rewrites;
      bool ok = false;
      for (; !ok && group.size() >= 2; ) {
      G = (int64_t)group.size();
      fusedBuf = newBuffer(g0.out.dtype, g0.out.shape[2] * Expr(G * N), BufferDecl::Temp);
      rewrites.clear();
      ok = true;
      for (size_t k = 0; k < plan.steps.size() && ok; ++k) {
        if (std::find(group.begin(), group.end(), k) != group.end()) continue;
        // the fused GEMM takes the place of the last one (where the operands of all of them are ready), so nothing in
        // between may read an output of the earlier ones
        if (k > group.front() && k < group.back())
          for (auto& nv : plan.steps[k].views) for (auto& g : gs) ok = ok && nv.second.buf != g.out.buf;
        for (auto& nv : plan.steps[k].views)
          for (int64_t j = 0; j < G && ok; ++j)
            if (nv.second.buf == gs[j].out.buf) {
              View r = nv.second;
              ok = nv.first != "out" && remapIntoFused(r, N, G, j, fusedBuf);
              rewrites.emplace_back(&nv.second, r);
            }
      }
      if (!ok) { group.pop_back(); gs.pop_back(); }
      }
      if (!ok) continue;
      for (auto& rw : rewrites) *rw.first = rw.second;
      // stacked operands, built once at load (the load-time steps are placed directly in front of the fused GEMM, behind
      // the load-time steps that make the operands of the single ones)
      const size_t before = plan.steps.size();
      View w = freshView(g0.b.dtype, {Expr(G * N), Expr(K)}, true), sh;
      if (g0.hasShift) sh = freshView(DType::F32, {Expr(G * N)}, true);
      for (int64_t j = 0; j < G; ++j) {
        View src = gs[j].b; src.shape = {Expr(N), Expr(K)}; src.strides = {Expr(K), Expr(1)};
        View dst = w; dst.offset = Expr(j * N * K); dst.shape = src.shape;
        emitEltwise(leafNode(src), dst, true);
        if (g0.hasShift) { View d = sh; d.offset = Expr(j * N); d.shape = {Expr(N)}; emitEltwise(leafNode(gs[j].shift), d, true); }
      }
      Step fused = plan.steps[i];
      for (auto& nv : fused.views) {
        if (nv.first == "b") { nv.second = w; nv.second.shape = {Expr(1), Expr(1), Expr(K), Expr(G * N)}; nv.second.strides = {Expr(G * N * K), Expr(G * N * K), Expr(1), Expr(K)}; }
        if (nv.first == "shift") nv.second = sh;
        if (nv.first == "out") { nv.second.buf = fusedBuf; nv.second.shape[3] = Expr(G * N); nv.second.strides = rowMajor(nv.second.shape); }
      }
      std::vector<Step> inits(plan.steps.begin() + (long)before, plan.steps.end());
      plan.steps.resize(before);
      plan.steps[group.back()] = fused;
      plan.steps.insert(plan.steps.begin() + (long)group.back(), inits.begin(), inits.end());
      for (size_t k = group.size() - 1; k-- > 0;) plan.steps.erase(plan.steps.begin() + (long)group[k]);
      --i;   // position i now holds whatever followed the first GEMM: look at it again
    }
  }
};

}  // namespace

Plan lowerToPlan(Module& m, const CompileOptionsData& opts) {
  runOperationLegalization(m);
  runRemoveRedundantOps(m);
  runFuseSoftmax(m);
  Lowering L(m, opts);
  L.run();
  return L.plan;
}

}  // namespace llc

namespace llc {
// infer-symbol-shape: runs the same shape rules as the lowering and writes the result back
// as static extents plus #llh.encoding<shapes = ...> on every tensor type
// (the reference pass: src/Dialect/LLH/SymbolInfer/InferSymbolShape.cpp:61-175).  Constant
// extents are named c<value>, input symbols keep their names, derived extents are printed as
// expressions where the reference would mint a fresh symbol plus a relation.
// Symbols that the input declares equal (`llh.symbol_relation` of kind EQ, usually in the nested module @__symbol__) become
// one symbol: the `relation` side is renamed to the `symbol` side wherever it occurs - encodings of types, `symbol`
// attributes, encoding attributes of bind ops, argument attributes - and its declaration is dropped (the reference folds
// such relations in its canonicalisation of the symbol ops, LLHCanonicalize of SymbolRelationOp).
static void unifyEqualSymbols(Module& m) {
  std::map<std::string, std::string> to;
  auto find = [&](std::string n) { for (auto it = to.find(n); it != to.end(); it = to.find(n)) n = it->second; return n; };
  for (auto& r : m.parsedRelations)
    if (r.kind == "EQ" && !r.symbol.empty() && !r.relation.empty()) {
      const std::string a = find(r.symbol), b = find(r.relation);
      if (a != b) to[b] = a;
    }
  if (to.empty()) return;
  auto renameText = [&](std::string& text) {           // "@name" tokens inside attribute text
    std::string out;
    for (size_t i = 0; i < text.size();) {
      if (text[i] == '@') {
        size_t j = i + 1;
        while (j < text.size() && (isalnum((unsigned char)text[j]) || text[j] == '_')) ++j;
        out += "@" + find(text.substr(i + 1, j - i - 1));
        i = j;
      } else out += text[i++];
    }
    text = out;
  };
  std::function<void(Attr&)> renameAttr = [&](Attr& a) {
    if (a.kind == Attr::SymRef) a.s = find(a.s);
    else if (a.kind == Attr::Enum || a.kind == Attr::Raw) renameText(a.s);
    else if (a.kind == Attr::Str && to.count(a.s)) a.s = find(a.s);
    for (auto& e : a.elems) renameAttr(e);
    for (auto& kv : a.dict) renameAttr(kv.second);
  };
  for (auto& v : m.valueStore) for (auto& n : v->type.encoding) n = find(n);
  for (auto& op : m.opStore) { for (auto& kv : op->props) renameAttr(kv.second); for (auto& kv : op->attrs) renameAttr(kv.second); }
  for (auto& f : m.funcs) {
    for (auto& al : f.argAttrs) for (auto& kv : al) renameAttr(kv.second);
    for (auto& t : f.resultTypes) for (auto& n : t.encoding) n = find(n);
  }
  std::vector<std::string> decls;
  for (auto& d : m.symbolDecls) if (!to.count(d)) decls.push_back(d);
  m.symbolDecls = decls;
}

void runInferSymbolShape(Module& m) {
  unifyEqualSymbols(m);
  const std::set<std::string> declaredBefore(m.symbolDecls.begin(), m.symbolDecls.end());
  runOperationLegalization(m);
  CompileOptionsData opts;
  Lowering L(m, opts);
  L.shapesOnly = true;
  L.run();
  for (auto& kv : L.tvs) {
    Value* v = kv.first;
    const TV& t = kv.second;
    if (!v->type.isTensor() || t.kind == TV::None || t.kind == TV::Scalar) continue;
    v->type.unranked = false;
    v->type.dims.clear(); v->type.encoding.clear();
    for (auto& e : t.shape) {
      v->type.dims.push_back(e.isConst() ? e.constant() : kDynamic);
      v->type.encoding.push_back(e.isConst() ? "c" + std::to_string(e.constant()) : e.str());
    }
  }
  // A derived extent gets a symbol of its own, the lowest free "s<k>", and a relation that says how it follows from its
  // operands (the reference: SymbolAnalysis::buildNewSymbol); equal expressions share one symbol.
  m.leadingLines.clear();
  std::vector<std::string> relationMaps;
  {
    auto isName = [](const std::string& n) { for (char c : n) if (!isalnum((unsigned char)c) && c != '_') return false; return !n.empty(); };
    std::set<std::string> used;
    std::vector<Value*> order;
    Func* f0 = m.entrance();
    if (f0) {
      for (Value* a : f0->args) order.push_back(a);
      for (Op* op : f0->ops) for (Value* r : op->results) order.push_back(r);
    }
    for (Value* v : order) if (v->type.isTensor()) for (auto& n : v->type.encoding) if (isName(n)) used.insert(n);
    std::map<std::string, std::string> fresh;          // printed expression -> symbol
    std::vector<std::string> created;
    auto nameOf = [&](const std::string& expr) -> std::string {
      if (isName(expr)) return expr;
      auto it = fresh.find(expr);
      if (it != fresh.end()) return it->second;
      int k = 0;
      while (used.count("s" + std::to_string(k))) ++k;
      std::string n = "s" + std::to_string(k);
      used.insert(n); fresh[expr] = n; created.push_back(expr);
      return n;
    };
    for (Value* v : order) if (v->type.isTensor()) for (auto& n : v->type.encoding) n = nameOf(n);
    // an integer scalar carries its symbol as an attribute of the op that produces it (the reference: `symbol = @c3`)
    if (f0) for (Op* op : f0->ops) {
      if (op->results.size() != 1 || op->results[0]->type.isTensor()) continue;
      auto it = L.tvs.find(op->results[0]);
      if (it == L.tvs.end() || it->second.kind != TV::Scalar || it->second.isFloatScalar) continue;
      const Expr& e = it->second.scalar;
      Attr a; a.kind = Attr::SymRef; a.s = e.isConst() ? "c" + std::to_string(e.constant()) : nameOf(e.str());
      bool set = false;
      for (auto& kv : op->props) if (kv.first == "symbol") { kv.second = a; set = true; }
      if (!set) {
        auto pos = op->props.begin();
        while (pos != op->props.end() && pos->first < "symbol") ++pos;
        op->props.insert(pos, std::make_pair(std::string("symbol"), a));
      }
    }
    std::vector<std::string> maps;
    for (size_t i = 0; i < created.size(); ++i) {      // may grow: an operand can be a derived extent that no tensor carries
      const std::string expr = created[i];
      auto it = L.relInfo.find(expr);
      if (it == L.relInfo.end()) continue;
      size_t mi = std::find(maps.begin(), maps.end(), it->second.map) - maps.begin();
      if (mi == maps.size()) maps.push_back(it->second.map);
      std::string rel;
      for (auto& o : it->second.operands) rel += (rel.empty() ? "@" : ", @") + (o.isConst() ? "c" + std::to_string(o.constant()) : nameOf(o.str()));
      relationMaps.push_back("\"llh.symbol_relation_map\"() <{express = \"" + expr + "\", relation = #map" + (mi ? std::to_string(mi) : "") + ", relations = [" + rel +
                             "], symbol = @" + fresh[expr] + "}> : () -> ()");
    }
    for (size_t i = 0; i < maps.size(); ++i) m.leadingLines.push_back("#map" + (i ? std::to_string(i) : std::string()) + " = affine_map<" + maps[i] + ">");
  }
  // every symbol an encoding names is declared once at the head of the module, arguments first, then in program order
  // (the reference's pass materialises them as llh.symbolic_int ops, SymbolAnalysis.cpp:266-330)
  m.symbolDecls.clear();
  std::set<std::string> declared;
  auto declare = [&](const Value* v) {
    if (!v->type.isTensor()) return;
    for (auto& n : v->type.encoding) if (declared.insert(n).second) m.symbolDecls.push_back(n);
  };
  Func* f = m.entrance();
  if (f) {
    for (Value* a : f->args) declare(a);
    for (Op* op : f->ops) for (Value* r : op->results) declare(r);
  }
  // an i64 argument that names no symbol yet gets the next free one (it is a symbol too: SymbolAnalysis buildNewSymbol)
  if (f) {
    int next = 0;
    for (auto& n : m.symbolDecls) if (n.size() > 1 && n[0] == 's' && isdigit((unsigned char)n[1])) next = std::max(next, atoi(n.c_str() + 1) + 1);
    if (f->argAttrs.size() < f->args.size()) f->argAttrs.resize(f->args.size());
    for (size_t i = 0; i < f->args.size(); ++i) {
      if (f->args[i]->type.isTensor() || f->args[i]->type.elt != DType::I64 || findAttr(f->argAttrs[i], "func.symbol_int")) continue;
      Attr a; a.kind = Attr::SymRef; a.s = "s" + std::to_string(next++);
      f->argAttrs[i].emplace_back("func.symbol_int", a);
      if (declared.insert(a.s).second) m.symbolDecls.push_back(a.s);
    }
  }
  // a dynamic extent is at least 1 (SymbolAnalysis.cpp:630-633 records the same relation for every new symbol)
  m.symbolRelations.clear();
  bool anyDynamic = false;
  for (auto& n : m.symbolDecls) {
    bool plain = !n.empty() && n[0] == 's';
    for (char c : n) if (!isalnum((unsigned char)c) && c != '_') plain = false;
    if (!plain || declaredBefore.count(n)) continue;     // the relation is recorded when a symbol is created, not for one the input declares
    anyDynamic = true;
    m.symbolRelations.push_back("\"llh.symbol_relation\"() <{relation = @c1, relation_kind = #llh.SymbolRelation<GE>, symbol = @" + n + "}> : () -> ()");
  }
  if (anyDynamic && declared.insert("c1").second) m.symbolDecls.push_back("c1");
  for (auto& l : relationMaps) m.symbolRelations.push_back(l);
  // relations the input came with stay, except the equalities folded above and those between constants only
  for (auto& r : m.parsedRelations) {
    auto isConstName = [](const std::string& n) { return n.size() > 1 && n[0] == 'c' && isdigit((unsigned char)n[1]); };
    if (r.kind == "EQ") continue;
    if ((r.symbol.empty() || isConstName(r.symbol)) && (r.relation.empty() || isConstName(r.relation))) continue;
    m.symbolRelations.push_back(r.text);
  }
  m.parsedRelations.clear();
  m.hasSymbolModule = true;
  if (f) {
    f->resultTypes.clear();
    for (Op* op : f->ops) if (op->name == "func.return") for (Value* v : op->operands) f->resultTypes.push_back(v->type);
  }
}
}  // namespace llc

// LLH-level rewrites of the reference that the GPU pipeline itself does not need (its stride algebra and epilogue
// absorption make them fall out), provided so that the reference's LLH surface behaves the same through llc_run_pass:
//   decompose-ops              src/Dialect/LLH/Transforms/DecomposeOps.cpp:110-148
//   transform-layout           src/Dialect/LLH/Transforms/TransformLayout.cpp:141-198
//   canonicalize               src/Dialect/LLH/IR/LLHCanonicalize.cpp:109-209 (+ the folders of LLHOps.cpp)
//   inline (folders only)      the same folders, reached through --inline in test/Dialect/LLH/fold.mlir
//   unload-and-bind-encoding   src/Dialect/LLH/Transforms/UnloadAndBindEncoding.cpp
//   cse                        MLIR's common-subexpression elimination, for pure LLH ops
#include <cmath>
#include <functional>
#include <map>
#include <set>

#include "plan.h"

namespace llc {

namespace {

struct Builder {
  Module& m;
  std::vector<Op*>& out;
  int& fresh;
  std::string name() { return "%t" + std::to_string(fresh++); }
  Value* result(Op* op, const Type& t) { Value* v = m.newValue(t, name()); v->def = op; v->index = (int)op->results.size(); op->results.push_back(v); return v; }
  Value* constI64(int64_t v) {
    Op* c = m.newOp("llh.constant"); c->setProp("value", Attr::integer(v));
    Value* r = result(c, Type::scalar(DType::I64)); out.push_back(c); return r;
  }
  Value* dim(Value* x, int64_t i) {
    Op* d = m.newOp("llh.dim"); d->operands = {x, constI64(i)};
    Value* r = result(d, Type::scalar(DType::I64)); out.push_back(d); return r;
  }
  // extent i of x as an i64 value: a constant when static, llh.dim otherwise
  Value* extent(Value* x, size_t i) { return x->type.dims[i] == kDynamic ? dim(x, (int64_t)i) : constI64(x->type.dims[i]); }
  Value* unary(const std::string& n, Value* x, const Type& t) { Op* o = m.newOp(n); o->operands = {x}; Value* r = result(o, t); out.push_back(o); return r; }
  Value* binary(const std::string& n, Value* a, Value* b, const Type& t) { Op* o = m.newOp(n); o->operands = {a, b}; Value* r = result(o, t); out.push_back(o); return r; }
  Value* transpose(Value* x, const std::vector<int64_t>& perms) {
    Type t = x->type; t.encoding.clear();
    for (size_t i = 0; i < perms.size(); ++i) t.dims[i] = x->type.dims[perms[i]];
    if (!x->type.encoding.empty()) { t.encoding.resize(perms.size()); for (size_t i = 0; i < perms.size(); ++i) t.encoding[i] = x->type.encoding[perms[i]]; }
    Op* o = m.newOp("llh.transpose"); o->operands = {x}; o->setProp("perms", Attr::array(perms));
    Value* r = result(o, t); out.push_back(o); return r;
  }
  // x (rank r) reshaped to `rank` dims with its extents placed at `at`, then broadcast to the shape of `like`
  // (DecomposeOps.cpp:76-106, LLHCanonicalize.cpp:109-209)
  Value* reshapeAndBroadcast(Value* x, const std::vector<int64_t>& at, Value* like) { return broadcastTo(reshapeTo(x, at, like->type.dims.size()), like); }
  Value* reshapeTo(Value* x, const std::vector<int64_t>& at, size_t rank) {
    Type rt = Type::tensor(x->type.elt, std::vector<int64_t>(rank, 1));
    std::vector<Value*> dims(rank, nullptr);
    for (size_t i = 0; i < at.size(); ++i) { rt.dims[at[i]] = x->type.dims[i]; dims[at[i]] = extent(x, i); }
    Value* one = nullptr;
    for (auto& d : dims) if (!d) { if (!one) one = constI64(1); d = one; }
    if (x->type.dims == rt.dims) return x;
    Op* rs = m.newOp("llh.reshape"); rs->operands.push_back(x);
    for (Value* d : dims) rs->operands.push_back(d);
    Value* cur = result(rs, rt); out.push_back(rs);
    return cur;
  }
  Value* broadcastTo(Value* cur, Value* like) {
    const size_t rank = like->type.dims.size();
    if (cur->type.dims == like->type.dims && !hasDynamic(like->type)) return cur;
    std::vector<int64_t> cast(rank), expand, keep;
    Op* bc = m.newOp("llh.broadcast_to"); bc->operands.push_back(cur);
    for (size_t i = 0; i < rank; ++i) {
      cast[i] = (int64_t)i;
      (cur->type.dims[i] == 1 && like->type.dims[i] != 1 ? expand : keep).push_back((int64_t)i);
      bc->operands.push_back(extent(like, i));
    }
    bc->setProp("cast_dims", Attr::array(cast)); bc->setProp("expand_dims", Attr::array(expand)); bc->setProp("noexpand_dims", Attr::array(keep));
    Type bt = like->type; bt.elt = cur->type.elt;
    Value* r = result(bc, bt); out.push_back(bc); return r;
  }
  static bool hasDynamic(const Type& t) { for (auto d : t.dims) if (d == kDynamic) return true; return false; }
};

void replaceUses(Module& m, Value* from, Value* to) {
  for (auto& f : m.funcs) for (Op* op : f.ops) for (auto& o : op->operands) if (o == from) o = to;
}
bool sideEffectFree(const Op* op) { return op->name != "llh.print" && op->name != "func.return" && op->name != "llh.encoding_bind" && op->name != "llh.symbol_bind" && op->name != "llh.symbolic_bind"; }
void dce(Module& m) {
  bool changed = true;
  while (changed) {
    changed = false;
    m.recomputeUsers();
    for (auto& f : m.funcs)
      for (Op* op : f.ops) {
        if (op->erased || !sideEffectFree(op) || op->results.empty()) continue;
        bool used = false;
        for (Value* r : op->results) used = used || !r->users.empty();
        if (!used) { op->erased = true; changed = true; }
      }
  }
}
// Rebuilds every function's op list through `visit`, which appends to `out` (the op itself, its replacement, or nothing).
void rewrite(Module& m, const std::function<void(Func&, Op*, Builder&)>& visit) {
  int fresh = 0;
  for (auto& v : m.valueStore) if (v->name.size() > 2 && v->name[1] == 't') fresh = std::max(fresh, atoi(v->name.c_str() + 2) + 1);
  for (auto& f : m.funcs) {
    std::vector<Op*> out;
    Builder b{m, out, fresh};
    for (Op* op : f.ops) { if (op->erased) continue; visit(f, op, b); }
    f.ops.swap(out);
  }
  m.recomputeUsers();
}

const Attr* constValue(const Value* v) { return v->def && v->def->name == "llh.constant" ? v->def->attr("value") : nullptr; }
bool constInt(const Value* v, int64_t& out) { const Attr* a = constValue(v); if (a && a->kind == Attr::Int) { out = a->i; return true; } return false; }
// a constant whose every element equals `x` (scalar or splat)
bool isConstEqual(const Value* v, double x) {
  const Attr* a = constValue(v);
  if (!a) return false;
  if (a->kind == Attr::Int) return (double)a->i == x;
  if (a->kind == Attr::Float) return a->f == x;
  if (a->kind == Attr::Dense) {
    if (!a->floats.empty()) { for (double f : a->floats) if (f != x) return false; return true; }
    if (!a->ints.empty()) { for (int64_t i : a->ints) if ((double)i != x) return false; return true; }
  }
  return false;
}
bool scalarConst(const Value* v, double& out) {
  const Attr* a = constValue(v);
  if (!a) return false;
  if (a->kind == Attr::Int) { out = (double)a->i; return true; }
  if (a->kind == Attr::Float) { out = a->f; return true; }
  return false;
}

}  // namespace

// ---- decompose-ops --------------------------------------------------------------------------------------------------
// llh.batch_norm_inference -> stddev = sqrt(var + eps); ((x - mean) * scale) / stddev + bias, every per-channel operand
// reshaped and broadcast to the input (DecomposeOps.cpp:125-144; eps becomes a tensor<1xT> constant, :65-74).
void runDecomposeOps(Module& m) {
  rewrite(m, [&](Func&, Op* op, Builder& b) {
    if (op->name != "llh.batch_norm_inference" || op->operands.size() != 5 || !op->operands[0]->type.isTensor()) { b.out.push_back(op); return; }
    Value *x = op->operands[0], *scale = op->operands[1], *bias = op->operands[2], *mean = op->operands[3], *var = op->operands[4];
    const Attr* eps = op->attr("epsilon"); const Attr* fi = op->attr("feature_index");
    const int64_t feature = fi ? fi->i : 1;
    Op* c = b.m.newOp("llh.constant");
    Attr dense; dense.kind = Attr::Dense; dense.splat = true; dense.floats = {eps ? eps->f : 1e-5}; dense.type = Type::tensor(var->type.elt, {1});
    c->setProp("value", dense);
    Value* epsV = b.result(c, Type::tensor(var->type.elt, {1})); b.out.push_back(c);
    Value* fined = b.binary("llh.add", var, epsV, var->type);
    Value* stddev = b.unary("llh.sqrt", fined, fined->type);
    Value* meanB = b.reshapeAndBroadcast(mean, {feature}, x);
    Value* scaleB = b.reshapeAndBroadcast(scale, {feature}, x);
    Value* biasB = b.reshapeAndBroadcast(bias, {feature}, x);
    Value* stdB = b.reshapeAndBroadcast(stddev, {feature}, x);
    Value* r = b.binary("llh.sub", x, meanB, x->type);
    r = b.binary("llh.mul", r, scaleB, x->type);
    r = b.binary("llh.div", r, stdB, x->type);
    r = b.binary("llh.add", r, biasB, x->type);
    r->type = op->results[0]->type;
    replaceUses(b.m, op->results[0], r);
    op->erased = true;
  });
  dce(m);
}

// ---- transform-layout -----------------------------------------------------------------------------------------------
// NCHW convolutions and poolings computed channel-last: operands transposed with perms [0,2,3,1], the op re-typed and
// marked NHWC, the result transposed back with [0,3,1,2] (TransformLayout.cpp:141-198).
void runTransformLayout(Module& m) {
  const std::vector<int64_t> toLast = {0, 2, 3, 1}, toFirst = {0, 3, 1, 2};
  rewrite(m, [&](Func&, Op* op, Builder& b) {
    const bool conv = op->name == "llh.conv" || op->name == "llh.conv_bias", pool = op->name == "llh.max_pool" || op->name == "llh.adaptive_average_pool";
    const Attr* lay = op->attr("layout");
    if ((!conv && !pool) || (lay && lay->s != "NCHW") || op->operands.empty() || op->operands[0]->type.dims.size() != 4 || op->results.empty()) { b.out.push_back(op); return; }
    op->operands[0] = b.transpose(op->operands[0], toLast);
    if (conv && op->operands.size() > 1 && op->operands[1]->type.dims.size() == 4) op->operands[1] = b.transpose(op->operands[1], toLast);
    op->setProp("layout", Attr::enumeration("Layout", "NHWC"));
    if (conv) op->setProp("weight_layout", Attr::enumeration("Layout", "FHWC"));
    Value* res = op->results[0];
    Type nchw = res->type;
    Type nhwc = nchw; nhwc.encoding.clear();
    for (size_t i = 0; i < 4; ++i) nhwc.dims[i] = nchw.dims[toLast[i]];
    if (!nchw.encoding.empty()) { nhwc.encoding.resize(4); for (size_t i = 0; i < 4; ++i) nhwc.encoding[i] = nchw.encoding[toLast[i]]; }
    Value* inner = b.m.newValue(nhwc, b.name()); inner->def = op; inner->index = 0;
    op->results[0] = inner;
    b.out.push_back(op);
    Op* back = b.m.newOp("llh.transpose"); back->operands = {inner}; back->setProp("perms", Attr::array(toFirst));
    res->def = back; back->results.push_back(res);
    b.out.push_back(back);
  });
}

// ---- cse ------------------------------------------------------------------------------------------------------------
void runCse(Module& m) {
  for (auto& f : m.funcs) {
    std::map<std::string, Op*> seen;
    for (Op* op : f.ops) {
      if (op->erased || !sideEffectFree(op) || op->results.size() != 1 || op->name == "llh.weight") continue;
      std::string key = op->name + "(";
      for (Value* v : op->operands) key += v->name + ",";
      key += ")";
      for (auto& kv : op->props) key += kv.first + "=" + kv.second.str() + ";";
      for (auto& kv : op->attrs) key += kv.first + "=" + kv.second.str() + ";";
      key += ":" + op->results[0]->type.str();
      auto it = seen.find(key);
      if (it == seen.end()) { seen[key] = op; continue; }
      replaceUses(m, op->results[0], it->second->results[0]);
      op->erased = true;
    }
  }
  dce(m);
}

// ---- folders (shared by canonicalize and inline) ---------------------------------------------------------------------
static bool foldOnce(Module& m) {
  bool changed = false;
  m.recomputeUsers();
  auto replaceWith = [&](Op* op, Value* v) { replaceUses(m, op->results[0], v); op->erased = true; changed = true; };
  for (auto& f : m.funcs) {
    std::vector<Op*> prefix;                              // constants created by folding go to the head of the function
    int fresh = 0;
    for (auto& v : m.valueStore) if (v->name.size() > 2 && v->name[1] == 'k') fresh = std::max(fresh, atoi(v->name.c_str() + 2) + 1);
    auto makeConst = [&](const Attr& value, const Type& t) {
      Op* c = m.newOp("llh.constant"); c->setProp("value", value);
      Value* r = m.newValue(t, "%k" + std::to_string(fresh++)); r->def = c; c->results.push_back(r);
      prefix.push_back(c);
      return r;
    };
    auto scalarAttr = [&](double v, const Type& t) { return isFloat(t.elt) ? Attr::floating(v, t.elt) : Attr::integer((int64_t)v, t.elt); };
    auto splatAttr = [&](double v, const Type& t) { Attr a; a.kind = Attr::Dense; a.splat = true; a.type = t; if (isFloat(t.elt)) a.floats = {v}; else a.ints = {(int64_t)v}; return a; };
    auto constLike = [&](double v, const Type& t) { return t.isTensor() ? makeConst(splatAttr(v, t), t) : makeConst(scalarAttr(v, t), t); };
    for (Op* op : f.ops) {
      if (op->erased || op->results.size() != 1) continue;
      Value* res = op->results[0];
      const std::string& n = op->name;
      // llh.dim of a static extent is that constant (LLHOps.cpp DimOp::fold)
      if (n == "llh.dim" && op->operands.size() == 2 && op->operands[0]->type.isTensor() && !op->operands[0]->type.unranked) {
        int64_t i;
        if (constInt(op->operands[1], i)) {
          const auto& dims = op->operands[0]->type.dims;
          if (i < 0) i += (int64_t)dims.size();
          if (i >= 0 && i < (int64_t)dims.size() && dims[i] != kDynamic) { replaceWith(op, makeConst(Attr::integer(dims[i]), Type::scalar(DType::I64))); continue; }
        }
      }
      if (n == "llh.abs" && op->operands[0]->def && op->operands[0]->def->name == "llh.abs") { replaceWith(op, op->operands[0]); continue; }
      if (n == "llh.convert_to" && op->operands[0]->type.str() == res->type.str()) { replaceWith(op, op->operands[0]); continue; }
      if (n == "llh.reshape" && op->operands[0]->type.isTensor() && !Builder::hasDynamic(res->type) && !res->type.unranked) {
        Value* x = op->operands[0];
        if (x->type.dims == res->type.dims) { replaceWith(op, x); continue; }
        if (const Attr* a = constValue(x)) {                // reshape of a constant: the same payload under the new type
          Attr v = *a; v.type = res->type; v.type.encoding.clear();
          replaceWith(op, makeConst(v, res->type)); continue;
        }
      }
      if (n == "llh.broadcast_to" && op->operands[0]->type.isTensor()) {
        const Attr* ex = op->attr("expand_dims");
        const bool nothing = ex && ex->kind == Attr::IntArray && ex->ints.empty() && op->operands[0]->type.dims.size() == res->type.dims.size();
        if (nothing || (!Builder::hasDynamic(res->type) && op->operands[0]->type.dims == res->type.dims)) { replaceWith(op, op->operands[0]); continue; }
      }
      if ((n == "llh.add" || n == "llh.sub" || n == "llh.mul" || n == "llh.div") && op->operands.size() == 2) {
        Value *a = op->operands[0], *c = op->operands[1];
        const bool sameType = a->type.str() == res->type.str() && c->type.str() == res->type.str();
        double x, y;
        if (scalarConst(a, x) && scalarConst(c, y) && !res->type.isTensor() && !(n == "llh.div" && y == 0)) {
          const double v = n == "llh.add" ? x + y : n == "llh.sub" ? x - y : n == "llh.mul" ? x * y : (isFloat(res->type.elt) ? x / y : (double)((int64_t)x / (int64_t)y));
          replaceWith(op, makeConst(scalarAttr(v, res->type), res->type)); continue;
        }
        if (!sameType) continue;
        if (n == "llh.add") {
          if (isConstEqual(a, 0)) { replaceWith(op, c); continue; }
          if (isConstEqual(c, 0)) { replaceWith(op, a); continue; }
          if (a->def && a->def->name == "llh.sub" && a->def->operands[1] == c) { replaceWith(op, a->def->operands[0]); continue; }   // (x - y) + y
          if (c->def && c->def->name == "llh.sub" && c->def->operands[1] == a) { replaceWith(op, c->def->operands[0]); continue; }   // y + (x - y)
        } else if (n == "llh.sub") {
          if (a == c) { replaceWith(op, constLike(0, res->type)); continue; }
          if (isConstEqual(c, 0)) { replaceWith(op, a); continue; }
          if (a->def && a->def->name == "llh.add" && a->def->operands[1] == c) { replaceWith(op, a->def->operands[0]); continue; }   // (x + y) - y
          if (a->def && a->def->name == "llh.add" && a->def->operands[0] == c) { replaceWith(op, a->def->operands[1]); continue; }
        } else if (n == "llh.mul") {
          if (isConstEqual(a, 1)) { replaceWith(op, c); continue; }
          if (isConstEqual(c, 1)) { replaceWith(op, a); continue; }
          if (isConstEqual(a, 0)) { replaceWith(op, a); continue; }
          if (isConstEqual(c, 0)) { replaceWith(op, c); continue; }
        } else if (n == "llh.div") {
          if (isConstEqual(c, 1)) { replaceWith(op, a); continue; }
        }
      }
    }
    if (!prefix.empty()) f.ops.insert(f.ops.begin(), prefix.begin(), prefix.end());
  }
  return changed;
}
static void dedupeConstants(Module& m) {
  for (auto& f : m.funcs) {
    std::map<std::string, Value*> seen;
    for (Op* op : f.ops) {
      if (op->erased || op->name != "llh.constant" || op->results.size() != 1) continue;
      const Attr* v = op->attr("value");
      if (!v) continue;
      const std::string key = v->str() + ":" + op->results[0]->type.str();
      auto it = seen.find(key);
      if (it == seen.end()) { seen[key] = op->results[0]; continue; }
      replaceUses(m, op->results[0], it->second);
      op->erased = true;
    }
  }
}
void runFold(Module& m) {
  for (int i = 0; i < 8 && foldOnce(m); ++i) {}
  dedupeConstants(m);
  dce(m);
}

// ---- canonicalize ---------------------------------------------------------------------------------------------------
// Besides the folders: negative extract indices made positive (dim + index), operands of elementwise ops and where that
// are lower in rank or have extent-1 dims reshaped and broadcast to the result (LLHCanonicalize.cpp:109-209,
// LLHUtilitys.cpp:80-163), and the layout attributes of convolutions and poolings filled in from the module's global
// layout (the reference's layout canonicalisation).
void runCanonicalize(Module& m) {
  std::string global = "NCHW";
  if (const Attr* g = findAttr(m.attrs, "builtin.gloabal_layout")) if (g->kind == Attr::Enum) global = g->s;
  rewrite(m, [&](Func&, Op* op, Builder& b) {
    const std::string& n = op->name;
    if ((n == "llh.conv" || n == "llh.conv_bias" || n == "llh.max_pool" || n == "llh.adaptive_average_pool") && !op->attr("layout")) {
      op->setProp("layout", Attr::enumeration("Layout", global));
      if (n == "llh.conv" || n == "llh.conv_bias") op->setProp("weight_layout", Attr::enumeration("Layout", global == "NCHW" ? "FCHW" : "FHWC"));
    }
    if (n == "llh.extract" && op->operands.size() == 2 && op->operands[0]->type.isTensor()) {
      int64_t i;
      if (constInt(op->operands[1], i) && i < 0) {
        Value* d0 = b.dim(op->operands[0], 0);
        op->operands[1] = b.binary("llh.add", d0, op->operands[1], Type::scalar(DType::I64));
      }
    }
    static const std::set<std::string> elementwise = {"llh.add", "llh.sub", "llh.mul", "llh.div", "llh.max", "llh.min", "llh.pow", "llh.where", "llh.compare"};
    if (elementwise.count(n) && !op->results.empty() && op->results[0]->type.isTensor() && !op->results[0]->type.unranked) {
      // the operand whose shape is the result's is the model; the others are brought to it
      const Type& rt = op->results[0]->type;
      Value* like = nullptr;
      for (Value* v : op->operands) if (v->type.isTensor() && v->type.dims == rt.dims) { like = v; break; }
      if (like) {
        // first every reshape, then every broadcast (the order the reference's patterns leave behind)
        std::vector<bool> touched(op->operands.size(), false);
        for (size_t k = 0; k < op->operands.size(); ++k) {
          Value*& v = op->operands[k];
          if (!v->type.isTensor() || v->type.unranked || v->type.dims == rt.dims) continue;
          const size_t r = v->type.dims.size(), rank = rt.dims.size();
          if (r > rank) continue;
          std::vector<int64_t> at(r);
          for (size_t i = 0; i < r; ++i) at[i] = (int64_t)(rank - r + i);      // numpy alignment: trailing dims
          v = b.reshapeTo(v, at, rank);
          touched[k] = true;
        }
        for (size_t k = 0; k < op->operands.size(); ++k) if (touched[k]) op->operands[k] = b.broadcastTo(op->operands[k], like);
      }
    }
    b.out.push_back(op);
  });
  runFold(m);
}

// ---- unload-and-bind-encoding ---------------------------------------------------------------------------------------
// Encodings leave the tensor types and are recorded by an llh.encoding_bind op after each definition; the symbol of a
// scalar op (its `symbol` attribute) is recorded by an llh.symbol_bind (UnloadAndBindEncoding.cpp).
void runUnloadAndBindEncoding(Module& m) {
  auto encodingAttr = [](const std::vector<std::string>& enc) {
    Attr a; a.kind = Attr::Raw; a.s = "#llh.encoding<shapes = ";
    for (size_t i = 0; i < enc.size(); ++i) a.s += (i ? ", @" : "@") + enc[i];
    a.s += ">";
    return a;
  };
  for (auto& f : m.funcs) {
    std::vector<Op*> out;
    auto bind = [&](Value* v) {
      if (!v->type.isTensor() || v->type.encoding.empty()) return;
      Op* b = m.newOp("llh.encoding_bind"); b->operands = {v}; b->setProp("encoding", encodingAttr(v->type.encoding));
      out.push_back(b);
    };
    for (Value* a : f.args) bind(a);
    for (Op* op : f.ops) {
      if (op->erased) continue;
      out.push_back(op);
      if (op->name == "func.return") continue;
      for (Value* r : op->results) bind(r);
      if (const Attr* s = op->attr("symbol")) {
        if (op->results.size() == 1 && !op->results[0]->type.isTensor()) {
          Op* sb = m.newOp("llh.symbol_bind"); sb->operands = {op->results[0]}; sb->setProp("symbol", *s);
          out.push_back(sb);
        }
      }
    }
    f.ops.swap(out);
    for (auto& t : f.resultTypes) t.encoding.clear();
  }
  for (auto& v : m.valueStore) v->type.encoding.clear();
  m.recomputeUsers();
}

// symbol-cse (the reference: src/Dialect/LLH/Transforms/SymbolCSE.cpp, driven by test/Dialect/LLH/symbol_infer/symbol_cse.mlir):
// after infer-symbol-shape every integer scalar carries `symbol = @...`.  Two values with the same symbol are the same
// number, so the later one is replaced by the earlier; a value whose symbol is a constant c<N> is replaced by that
// constant (written `arith.constant N : index` when the value came from the arith / tensor dialects).
void runSymbolCse(Module& m) {
  for (auto& f : m.funcs) {
    std::map<std::string, Value*> first;
    std::vector<Op*> out;
    auto replaceUses = [&](Value* from, Value* to) {
      for (Op* u : f.ops) for (auto& v : u->operands) if (v == from) v = to;
    };
    for (Op* op : f.ops) {
      if (op->erased) continue;
      const Attr* sym = op->results.size() == 1 && !op->results[0]->type.isTensor() ? op->attr("symbol") : nullptr;
      if (!sym || sym->kind != Attr::SymRef) { out.push_back(op); continue; }
      const std::string& name = sym->s;
      const bool isConstSym = name.size() > 1 && name[0] == 'c' && isdigit((unsigned char)name[1]);
      const bool isConstOp = op->name == "llh.constant";
      if (isConstSym && !isConstOp) {
        Op* c = m.newOp("llh.constant");
        if (!op->written.empty()) c->written = "arith.constant";
        Attr v = Attr::integer(std::stoll(name.substr(1)));
        if (!op->written.empty()) v.type = Type::scalar(DType::Index);
        c->props.emplace_back("value", v);
        Value* r = m.newValue(op->results[0]->type);
        r->def = c; c->results.push_back(r);
        out.push_back(c);
        replaceUses(op->results[0], r);
        op->erased = true;
        continue;
      }
      auto it = first.find(name);
      if (it != first.end() && !isConstOp) { replaceUses(op->results[0], it->second); op->erased = true; continue; }
      if (it == first.end()) first[name] = op->results[0];
      out.push_back(op);
    }
    f.ops = out;
  }
  m.recomputeUsers();
}

}  // namespace llc

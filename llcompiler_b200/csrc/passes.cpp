// LLH-level passes that run before the conversion to kernel calls.
//
// Names follow the reference pipeline (src/Pipeline/TransformPipeline.cpp:103-130):
// operation-legalization, remove-redundant-ops, then a new fuse-softmax pass that
// re-assembles the amax/sub/exp/sum/div chain the reference's decomposition
// table produces (llcompiler/compiler/torch_compile_config.py:24) into the
// llh.softmax op that the Python dialect declares (llcompiler/dialect/llh.py:406-411).
#include <set>

#include "plan.h"

namespace llc {

static bool isPure(const Op* op) { return op->name != "llh.print" && op->name != "func.return"; }

static void eraseDead(Module& m) {
  bool changed = true;
  while (changed) {
    changed = false;
    m.recomputeUsers();
    for (auto& f : m.funcs)
      for (Op* op : f.ops) {
        if (op->erased || !isPure(op) || op->results.empty()) continue;
        bool used = false;
        for (Value* r : op->results) if (!r->users.empty()) used = true;
        if (!used) { op->erased = true; changed = true; }
      }
  }
}

static void replaceAllUses(Module& m, Value* from, Value* to) {
  for (auto& f : m.funcs) for (Op* op : f.ops) for (auto& o : op->operands) if (o == from) o = to;
}

// Rank-0 tensors become tensor<1xT>, integer `axis` attributes become arrays
// (src/Dialect/LLH/Transforms/Operationlegalization.cpp:109-230 does the same normalisation).
void runOperationLegalization(Module& m) {
  // rank-0 tensors become tensor<1x..> (Operationlegalization.cpp: "weight_refine", "extract" patterns), also in the
  // function's declared result types
  for (auto& v : m.valueStore)
    if (v->type.isTensor() && !v->type.unranked && v->type.dims.empty()) v->type.dims.push_back(1);
  for (auto& f : m.funcs) {
    for (auto& t : f.resultTypes)
      if (t.isTensor() && !t.unranked && t.dims.empty()) t.dims.push_back(1);
    // the number of leading i64 (symbol) arguments is recorded on the function
    int64_t nSym = 0;
    for (Value* a : f.args) { if (a->type.isTensor()) break; ++nSym; }
    if (nSym > 0 && !findAttr(f.attrs, "symbol_int_arg_nums")) f.attrs.emplace_back("symbol_int_arg_nums", Attr::integer(nSym));
    std::vector<Op*> out;
    int fresh = 0;
    for (Op* op : f.ops) {
      if (op->name == "llh.reduce_max" || op->name == "llh.reduce_min" || op->name == "llh.reduce_sum" || op->name == "llh.reduce_mean") {
        const Attr* a = op->attr("axis");
        if (a && a->kind == Attr::Int) op->setProp("axis", Attr::array({a->i}));
      }
      // broadcast_to of a lower-rank operand: reshape it to the result's rank first (extent 1 in the new dims), so that
      // cast_dims is always the identity
      if (op->name == "llh.broadcast_to" && !op->operands.empty() && !op->results.empty()) {
        Value* x = op->operands[0];
        const size_t rank = op->operands.size() - 1;
        const Attr* cd = op->attr("cast_dims");
        if (x->type.isTensor() && !x->type.unranked && x->type.dims.size() < rank && cd && cd->kind == Attr::IntArray &&
            cd->ints.size() == x->type.dims.size()) {
          auto name = [&]() { return "%lg" + std::to_string(fresh++); };
          Op* one = m.newOp("llh.constant");
          one->setProp("value", Attr::integer(1));
          Value* oneV = m.newValue(Type::scalar(DType::I64), name()); oneV->def = one; one->results.push_back(oneV);
          out.push_back(one);
          std::vector<Value*> dims(rank, oneV);
          Type rt = x->type; rt.dims.assign(rank, 1); rt.encoding.clear();
          for (size_t i = 0; i < cd->ints.size(); ++i) {
            const int64_t d = cd->ints[i];
            if (d < 0 || (size_t)d >= rank) continue;
            rt.dims[d] = x->type.dims[i];
            if (x->type.dims[i] == kDynamic) {
              Op* idx = m.newOp("llh.constant"); idx->setProp("value", Attr::integer((int64_t)i));
              Value* idxV = m.newValue(Type::scalar(DType::I64), name()); idxV->def = idx; idx->results.push_back(idxV);
              Op* dim = m.newOp("llh.dim"); dim->operands = {x, idxV};
              Value* dimV = m.newValue(Type::scalar(DType::I64), name()); dimV->def = dim; dim->results.push_back(dimV);
              out.push_back(idx); out.push_back(dim);
              dims[d] = dimV;
            } else {
              Op* c = m.newOp("llh.constant"); c->setProp("value", Attr::integer(x->type.dims[i]));
              Value* cV = m.newValue(Type::scalar(DType::I64), name()); cV->def = c; c->results.push_back(cV);
              out.push_back(c);
              dims[d] = cV;
            }
          }
          Op* rs = m.newOp("llh.reshape");
          rs->operands.push_back(x);
          for (Value* d : dims) rs->operands.push_back(d);
          Value* rv = m.newValue(rt, name()); rv->def = rs; rs->results.push_back(rv);
          out.push_back(rs);
          op->operands[0] = rv;
          std::vector<int64_t> ident(rank); for (size_t i = 0; i < rank; ++i) ident[i] = (int64_t)i;
          op->setProp("cast_dims", Attr::array(ident));
        }
      }
      out.push_back(op);
    }
    f.ops.swap(out);
  }
  m.recomputeUsers();
}

// Drops bookkeeping ops and identity data movement
// (src/Dialect/LLH/Transforms/RemoveRedundantOps.cpp:136-268).
void runRemoveRedundantOps(Module& m) {
  for (auto& f : m.funcs)
    for (Op* op : f.ops) {
      if (op->erased) continue;
      if (op->name == "llh.symbolic_bind" || op->name == "llh.encoding_bind" || op->name == "llh.symbol_bind") op->erased = true;
      if (op->name == "llh.transpose" && op->results.size() == 1) {
        const Attr* p = op->attr("perms");
        bool identity = p && p->kind == Attr::IntArray;
        if (identity) for (size_t i = 0; i < p->ints.size(); ++i) if (p->ints[i] != (int64_t)i) identity = false;
        if (identity) { replaceAllUses(m, op->results[0], op->operands[0]); op->erased = true; }
      }
    }
  eraseDead(m);
}

static Op* skipShapeOps(Value* v) {   // looks through reshape / broadcast_to
  Op* d = v->def;
  while (d && (d->name == "llh.reshape" || d->name == "llh.broadcast_to")) d = d->operands[0]->def;
  return d;
}

static bool reducesLastAxis(const Op* op) {
  const Attr* a = op->attr("axis");
  if (!a) return false;
  int64_t rank = (int64_t)op->operands[0]->type.dims.size();
  std::vector<int64_t> ax = a->kind == Attr::IntArray ? a->ints : std::vector<int64_t>{a->i};
  return ax.size() == 1 && (ax[0] == rank - 1 || ax[0] == -1);
}

void runFuseSoftmax(Module& m) {
  m.recomputeUsers();
  for (auto& f : m.funcs)
    for (Op* div : f.ops) {
      if (div->erased || div->name != "llh.div" || div->operands.size() != 2 || !div->results[0]->type.isTensor()) continue;
      Op* e = div->operands[0]->def;
      if (!e || e->name != "llh.exp") continue;
      Op* sum = skipShapeOps(div->operands[1]);
      if (!sum || sum->name != "llh.reduce_sum" || sum->operands[0] != e->results[0] || !reducesLastAxis(sum)) continue;
      Op* sub = e->operands[0]->def;
      if (!sub || sub->name != "llh.sub") continue;
      Value* x = sub->operands[0];
      Op* mx = skipShapeOps(sub->operands[1]);
      if (!mx || mx->name != "llh.reduce_max" || mx->operands[0] != x || !reducesLastAxis(mx)) continue;
      if (e->results[0]->users.size() != 2 || sub->results[0]->users.size() != 1) continue;
      int64_t rank = (int64_t)x->type.dims.size();
      div->name = "llh.softmax";
      div->operands = {x};
      div->props.clear();
      div->props.emplace_back("axis", Attr::integer(rank - 1));
    }
  eraseDead(m);
}

}  // namespace llc

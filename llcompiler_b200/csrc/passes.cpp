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
  for (auto& v : m.valueStore)
    if (v->type.isTensor() && !v->type.unranked && v->type.dims.empty()) v->type.dims.push_back(1);
  for (auto& f : m.funcs)
    for (Op* op : f.ops) {
      if (op->name == "llh.reduce_max" || op->name == "llh.reduce_min" || op->name == "llh.reduce_sum" || op->name == "llh.reduce_mean") {
        const Attr* a = op->attr("axis");
        if (a && a->kind == Attr::Int) op->setProp("axis", Attr::array({a->i}));
      }
    }
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

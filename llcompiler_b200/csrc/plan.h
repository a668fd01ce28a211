// The kernel plan: what the GPU pipeline produces from an LLH module and what the
// executor runs.
//
// The reference lowers LLH through StableHLO/linalg/affine/LLVM into a shared
// object exporting main(void**) (src/Pipeline/TransformPipeline.cpp:100-226,
// src/Compiler/Compiler.cpp:296-348).  Here the product of compilation is a
// text plan: buffers, symbol bindings and an ordered list of kernel calls whose
// operands are strided views with symbolic extents.  Extents are kept as
// expressions over the shape symbols and evaluated when a call binds them.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "ir.h"

namespace llc {

struct View {
  int buf = -1;
  Expr offset;
  std::vector<Expr> shape, strides;
  DType dtype = DType::F32;
  size_t rank() const { return shape.size(); }
  std::string str() const;
};

struct BufferDecl {
  enum Kind { Temp, Input, Output, Weight, Const } kind = Temp;
  DType dtype = DType::F32;
  Expr numel;
  int index = -1;     // input/output position
  std::string file;   // weight .npy path
  // dense constants that are not splats (small): values in element order
  std::vector<double> values;
};

struct Step {
  std::string kernel;                              // "gemm", "conv", ...
  bool init = false;                               // runs once at load (operands are weights/constants)
  std::vector<std::pair<std::string, View>> views; // named operands
  std::vector<std::pair<std::string, std::string>> params;  // named scalars, already text
  const View* view(const std::string& n) const { for (auto& v : views) if (v.first == n) return &v.second; return nullptr; }
  std::string param(const std::string& n, const std::string& dflt = "") const { for (auto& p : params) if (p.first == n) return p.second; return dflt; }
};

struct SymbolBinding {
  std::string name;
  int symbolArg = -1;          // position among the i64 symbol arguments, or
  int input = -1, dim = -1;    // tensor input position and dim
};

struct IoDecl { int buf; DType dtype; std::vector<Expr> shape; };

struct Plan {
  std::map<std::string, std::string> options;
  std::vector<SymbolBinding> symbols;
  int numSymbolArgs = 0;
  std::vector<BufferDecl> buffers;
  std::vector<IoDecl> inputs, outputs;
  std::vector<Step> steps;
  std::string str() const;
};

Plan parsePlan(const std::string& text);

struct CompileOptionsData {
  std::string mode = "inference", target = "sm_100a", pipeline = "cuda", globalLayout = "NCHW";
  std::string logRoot, logLevel = "debug", cpu, mtriple;
  std::string precision = "auto";  // fp32 | tf32 | tf32x3 | bf16 | auto
  bool displayMlirPasses = false, displayLlvmPasses = false;
  bool mergeStemRows = true;       // narrow-channel stem convolutions read a filter row per K block (LLC_MERGE_STEM_ROWS=0 disables)
  bool fuseAttention = true;       // batch_matmul -> softmax -> batch_matmul as one attention step where the kernel's limits allow
  bool fuseSiblingGemms = true;    // linear layers over one activation (query, key, value) as one GEMM over stacked weights (LLC_FUSE_SIBLING_GEMMS=0 disables)
};

// Runs the GPU pipeline on parsed LLH text and returns the plan.
Plan lowerToPlan(Module& m, const CompileOptionsData& opts);

// LLH-level passes that are useful on their own (and are what the structure tests drive).
void runOperationLegalization(Module& m);
void runSymbolCse(Module& m);   // integer scalars that carry the same symbol become one value; a constant symbol becomes a constant
void runRemoveRedundantOps(Module& m);
void runFuseSoftmax(Module& m);
void runInferSymbolShape(Module& m);   // writes #llh.encoding onto every tensor type
// llh_transforms.cpp: the reference's LLH-level rewrites that its lit files exercise
void runDecomposeOps(Module& m);
void runTransformLayout(Module& m);
void runCanonicalize(Module& m);
void runFold(Module& m);
void runCse(Module& m);
void runUnloadAndBindEncoding(Module& m);

}  // namespace llc

// C ABI, compile side: LLH text -> kernel plan file (see include/llc_runtime.h).
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>

#include "../../include/llc_runtime.h"
#include "capi_common.h"
#include "plan.h"

namespace llc {
thread_local std::string g_lastError;
thread_local std::string g_passText;

int setError(int code, const std::string& msg) { g_lastError = msg; return code; }

int statusFor(const std::exception& e) {
  std::string w = e.what();
  if (w.find("parse error") != std::string::npos || w.find("not a kernel plan") != std::string::npos) return LLC_ERR_PARSE;
  if (w.find("llc compile:") != std::string::npos) return LLC_ERR_UNSUPPORTED;
  if (w.find("llc io:") != std::string::npos) return LLC_ERR_IO;
  if (w.find("llc cuda:") != std::string::npos) return LLC_ERR_CUDA;
  if (w.find("llc argument:") != std::string::npos || w.find("shape symbol") != std::string::npos) return LLC_ERR_ARGUMENT;
  return LLC_ERR_INTERNAL;
}

static CompileOptionsData optionsFrom(const LlcOptions* o) {
  CompileOptionsData d;
  // LLC_FUSE_ATTENTION=0 keeps attention as GEMM, softmax, GEMM (the path every shape outside the fused kernel's limits takes)
  if (const char* e = getenv("LLC_FUSE_ATTENTION")) d.fuseAttention = !(e[0] == '0');
  if (const char* e = getenv("LLC_FUSE_SIBLING_GEMMS")) d.fuseSiblingGemms = !(e[0] == '0');
  if (const char* e = getenv("LLC_MERGE_STEM_ROWS")) d.mergeStemRows = !(e[0] == '0');
  if (!o) return d;
  auto set = [](std::string& dst, const char* src) { if (src && *src) dst = src; };
  set(d.mode, o->mode); set(d.target, o->target); set(d.pipeline, o->pipeline); set(d.globalLayout, o->global_layout);
  set(d.logRoot, o->log_root); set(d.logLevel, o->log_level); set(d.cpu, o->cpu); set(d.mtriple, o->mtriple);
  set(d.precision, o->precision);
  return d;
}

static void checkOptions(const CompileOptionsData& d) {
  if (d.mode != "inference") throw std::runtime_error("llc compile: mode '" + d.mode + "' is not supported by the CUDA pipeline (inference only)");
  if (d.pipeline != "cuda" && d.pipeline != "transform") throw std::runtime_error("llc compile: unknown pipeline '" + d.pipeline + "'");
  if (d.globalLayout != "NCHW") throw std::runtime_error("llc compile: global layout '" + d.globalLayout + "' is not supported (modules are NCHW-typed; NHWC is used internally)");
  static const char* precs[] = {"auto", "fp32", "tf32", "tf32x3", "bf16"};
  bool ok = false; for (auto p : precs) if (d.precision == p) ok = true;
  if (!ok) throw std::runtime_error("llc compile: unknown precision '" + d.precision + "'");
}
}  // namespace llc

using namespace llc;

extern "C" const char* llc_last_error(void) { return g_lastError.c_str(); }
extern "C" const char* llc_version(void) { return "llcompiler-b200 0.1 (sm_100a)"; }

extern "C" int llc_run_pass(const char* text, const char* pass, const LlcOptions* options, const char** out) {
  if (!text || !pass || !out) return setError(LLC_ERR_ARGUMENT, "null argument");
  try {
    CompileOptionsData d = optionsFrom(options);
    std::string p = pass;
    std::string result;
    for (auto& part : splitInputFile(text)) {
      bool blank = part.find_first_not_of(" \t\r\n") == std::string::npos;
      if (blank) continue;
      auto m = parseModule(part);
      if (m->funcs.empty()) continue;
      // `pass` may be a comma-separated pipeline, applied in order (the reference's RUN lines chain several)
      bool printedPlan = false;
      size_t at = 0;
      while (at <= p.size()) {
        size_t comma = p.find(',', at);
        if (comma == std::string::npos) comma = p.size();
        const std::string one = p.substr(at, comma - at);
        at = comma + 1;
        if (one.empty() || one == "parse") {}
        else if (one == "operation-legalization") runOperationLegalization(*m);
        else if (one == "remove-redundant-ops") runRemoveRedundantOps(*m);
        else if (one == "fuse-softmax") runFuseSoftmax(*m);
        else if (one == "infer-symbol-shape") runInferSymbolShape(*m);
        else if (one == "decompose-ops") runDecomposeOps(*m);
        else if (one == "transform-layout") runTransformLayout(*m);
        else if (one == "canonicalize") runCanonicalize(*m);
        else if (one == "inline") runFold(*m);
        else if (one == "cse") runCse(*m);
        else if (one == "symbol-cse") runSymbolCse(*m);
        else if (one == "unload-and-bind-encoding") runUnloadAndBindEncoding(*m);
        else if (one == "lower") { checkOptions(d); result += lowerToPlan(*m, d).str(); result += "// -----\n"; printedPlan = true; break; }
        else return setError(LLC_ERR_ARGUMENT, "unknown pass '" + one + "'");
      }
      if (printedPlan) continue;
      result += m->str();
      result += "// -----\n";
    }
    g_passText = result;
    *out = g_passText.c_str();
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

extern "C" int llc_compile(const char* text, const LlcOptions* options, char* outPath, size_t outLen) {
  if (!text || !outPath) return setError(LLC_ERR_ARGUMENT, "null argument");
  try {
    CompileOptionsData d = optionsFrom(options);
    checkOptions(d);
    auto m = parseModule(text);
    auto dump = [&](const std::string& stage, const std::string& body) {
      if (d.logRoot.empty()) return;
      ::mkdir(d.logRoot.c_str(), 0755);
      std::ofstream(d.logRoot + "/" + stage) << body;
    };
    dump("00_input.mlir", m->str());
    Plan plan = lowerToPlan(*m, d);
    dump("01_llh_after_fusion.mlir", m->str());
    std::string body = plan.str();
    dump("02_kernel_plan.llcplan", body);
    // the artefact is named after a hash of the module text, like the reference's temp .so
    // (src/Compiler/Compiler.cpp:305-309)
    size_t h = std::hash<std::string>()(std::string(text) + "|" + d.precision + (d.fuseAttention ? "|fa" : "") + (d.mergeStemRows ? "|ms" : "") + (d.fuseSiblingGemms ? "|sg" : ""));
    const char* tmp = getenv("TMPDIR");
    char path[512];
    snprintf(path, sizeof path, "%s/llc_%016zx_%d.llcplan", tmp && *tmp ? tmp : "/tmp", h, (int)getpid());
    { std::ofstream f(path); if (!f) throw std::runtime_error(std::string("llc io: cannot write ") + path); f << body; }
    if (strlen(path) + 1 > outLen) return setError(LLC_ERR_ARGUMENT, "out_path buffer too small");
    strcpy(outPath, path);
    return LLC_OK;
  } catch (const std::exception& e) { return setError(statusFor(e), e.what()); }
}

// pybind11 module `llcompiler_`: the reference's Python-facing native module
// (src/Pybind/Entrance.cpp:69-120) re-bound onto the C ABI of llc_runtime.h.  Same submodules
// (tensor, compiler, executor), same class and method names, same argument order.  A non-zero
// status from the C ABI becomes a Python RuntimeError (the reference logs and carries on,
// include/llcompiler/Support/Logger.h:126-134).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "llc_runtime.h"

namespace py = pybind11;

namespace {

void check(int rc) { if (rc != LLC_OK) throw std::runtime_error(std::string("[llc status ") + std::to_string(rc) + "] " + llc_last_error()); }

// llc::compiler::Tensor (include/llcompiler/Compiler/Tensor.h:35-48) plus a device ordinal.
struct Tensor {
  uintptr_t data = 0, base = 0;
  int type = LLC_FLOAT32;
  int64_t offset = 0;
  std::vector<int64_t> size, stride;
  int device = -1;
  Tensor() {}
  Tensor(uintptr_t data_ptr, uintptr_t base_ptr, int type_, int64_t offset_, std::vector<int64_t> size_, std::vector<int64_t> stride_, int device_ = -1)
      : data(data_ptr), base(base_ptr), type(type_), offset(offset_), size(std::move(size_)), stride(std::move(stride_)), device(device_) {}
  LlcTensor desc() const { return LlcTensor{reinterpret_cast<void*>(data), type, device, (int32_t)size.size(), size.data(), stride.data()}; }
  void print() const {
    std::string s = "Tensor(data=" + std::to_string(data) + ", type=" + std::to_string(type) + ", device=" + std::to_string(device) + ", size=[";
    for (size_t i = 0; i < size.size(); ++i) s += (i ? "," : "") + std::to_string(size[i]);
    py::print(s + "])");
  }
};

// Element size and struct-module format of a dtype code (the reference's get_itemsize / get_format,
// src/Pybind/Entrance.cpp:27-58, plus the two 16-bit floats).
py::ssize_t itemSize(int type) {
  switch (type) {
    case LLC_INT8: case LLC_INT1: return 1;
    case LLC_INT16: case LLC_FLOAT16: case LLC_BFLOAT16: return 2;
    case LLC_INT32: case LLC_FLOAT32: return 4;
    default: return 8;
  }
}
std::string formatOf(int type) {
  switch (type) {
    case LLC_INT8: return "b"; case LLC_INT1: return "?"; case LLC_INT16: return "h"; case LLC_INT32: return "i"; case LLC_INT64: return "q";
    case LLC_FLOAT32: return "f"; case LLC_FLOAT64: return "d"; case LLC_FLOAT16: return "e";
    case LLC_BFLOAT16: return "H";      // no struct code for bf16: exposed as its 16-bit pattern
  }
  throw std::runtime_error("Tensor: unknown element type code " + std::to_string(type));
}
// Buffer view of a HOST tensor (the reference's tensors are always host memory, src/Pybind/Entrance.cpp:80-91);
// device memory cannot be read through the buffer protocol.
py::buffer_info bufferOf(Tensor& t) {
  if (t.device >= 0) throw std::runtime_error("Tensor: device memory has no buffer view; copy the torch tensor to the host first");
  std::vector<py::ssize_t> shape(t.size.begin(), t.size.end()), strides;
  for (auto s : t.stride) strides.push_back((py::ssize_t)s * itemSize(t.type));
  return py::buffer_info(reinterpret_cast<void*>(t.data), itemSize(t.type), formatOf(t.type), (py::ssize_t)shape.size(), shape, strides);
}

// The reference's executor.get_tool (src/Compiler/Command.cpp:13-15 over ToolPath.h.in:19-24) names the external
// programs its pipeline shells out to.  This backend runs no subprocess: "llc-opt" is the text-IR driver module, "cxx"
// the host compiler the build used; the LLVM tools have no counterpart and raise, as an unknown name does there.
std::string getTool(const std::string& name) {
  if (name == "llc-opt") return "python -m llcompiler_b200.llc_opt";
  if (name == "cxx") return "g++";
  throw py::index_error("no tool '" + name + "': the CUDA pipeline runs in-process and has no LLVM tool chain (opt, llc, llc-translate)");
}

// llc::compiler::CompileOptions (include/llcompiler/Compiler/CompileOption.h:39-71)
struct CompileOptions {
  std::string mode = "inference", target = "sm_100a", pipeline = "cuda", global_layout = "NCHW", log_root, log_level = "debug", cpu, mtriple, precision = "auto";
  bool mlir_passes = false, llvm_passes = false;
  LlcOptions c() const { return LlcOptions{mode.c_str(), target.c_str(), pipeline.c_str(), global_layout.c_str(), log_root.c_str(), log_level.c_str(), cpu.c_str(), mtriple.c_str(), precision.c_str()}; }
};

struct Compiler {
  std::string compile_mlir_to_shared_lib(const std::string& text, const CompileOptions& o) {
    char path[1024];
    LlcOptions c = o.c();
    check(llc_compile(text.c_str(), &c, path, sizeof path));
    return path;
  }
  std::string run_pass(const std::string& text, const std::string& pass, const CompileOptions& o) {
    const char* out = nullptr;
    LlcOptions c = o.c();
    check(llc_run_pass(text.c_str(), pass.c_str(), &c, &out));
    return out;
  }
};

// llc::compiler::Execution (src/Compiler/Execution.cpp:10-66)
struct Execution {
  LlcExec* exec = nullptr;
  ~Execution() { if (exec) llc_free(exec); }
  void load(const std::string& path, int device, const std::string& weight_dir) {
    if (exec) throw std::runtime_error("Execution.load may be called once per object");
    check(llc_load_from(path.c_str(), weight_dir.empty() ? nullptr : weight_dir.c_str(), device, &exec));
  }
  bool loaded_from_pool() const { need(); return llc_loaded_from_pool(exec) == 1; }
  void need() const { if (!exec) throw std::runtime_error("Execution.load has not been called"); }
  void run_impl(const std::vector<int64_t>& symbols, std::vector<Tensor*>& in, std::vector<Tensor*>& out, uintptr_t stream) {
    need();
    std::vector<LlcTensor> ci, co;
    for (auto* t : in) ci.push_back(t->desc());
    for (auto* t : out) co.push_back(t->desc());
    int rc;
    {
      py::gil_scoped_release release;
      rc = llc_run(exec, symbols.data(), (int)symbols.size(), ci.data(), (int)ci.size(), co.data(), (int)co.size(), reinterpret_cast<void*>(stream));
    }
    check(rc);
  }
  void run(std::vector<Tensor*> in, std::vector<Tensor*> out, uintptr_t stream) { run_impl({}, in, out, stream); }
  void run_with_symbols(std::vector<int64_t> symbols, std::vector<Tensor*> in, std::vector<Tensor*> out, uintptr_t stream) { run_impl(symbols, in, out, stream); }
  std::vector<std::pair<std::vector<int64_t>, int>> output_shapes(std::vector<int64_t> symbols, std::vector<Tensor*> in) {
    need();
    std::vector<LlcTensor> ci;
    for (auto* t : in) ci.push_back(t->desc());
    std::vector<std::pair<std::vector<int64_t>, int>> res;
    for (int k = 0; k < llc_num_outputs(exec); ++k) {
      int64_t sizes[8]; int32_t rank = 0, dtype = 0;
      check(llc_output_shape(exec, symbols.data(), (int)symbols.size(), ci.data(), (int)ci.size(), k, sizes, &rank, &dtype));
      res.emplace_back(std::vector<int64_t>(sizes, sizes + rank), dtype);
    }
    return res;
  }
  std::string profile(std::vector<int64_t> symbols, std::vector<Tensor*> in, std::vector<Tensor*> out, int reps, uintptr_t stream) {
    need();
    std::vector<LlcTensor> ci, co;
    for (auto* t : in) ci.push_back(t->desc());
    for (auto* t : out) co.push_back(t->desc());
    std::string report(1 << 20, '\0');
    check(llc_profile(exec, symbols.data(), (int)symbols.size(), ci.data(), (int)ci.size(), co.data(), (int)co.size(), reps,
                      reinterpret_cast<void*>(stream), &report[0], report.size()));
    report.resize(strlen(report.c_str()));
    return report;
  }
  // Raises when a kernel of an earlier call recorded a failure (see llc_status); returns the three words otherwise.
  std::vector<int> status() {
    need();
    int32_t w[3] = {0, 0, 0};
    int rc;
    {
      py::gil_scoped_release release;
      rc = llc_status(exec, w);
    }
    check(rc);
    return {w[0], w[1], w[2]};
  }
  int num_inputs() const { need(); return llc_num_inputs(exec); }
  int num_outputs() const { need(); return llc_num_outputs(exec); }
  int num_symbols() const { need(); return llc_num_symbols(exec); }
  int64_t last_launch_count() const { need(); return llc_last_launch_count(exec); }
  int64_t arena_bytes() const { need(); return llc_arena_bytes(exec); }
};

}  // namespace

PYBIND11_MODULE(llcompiler_, m) {
  m.doc() = "B200 execution backend with the llcompiler_ module surface";
  auto tensor = m.def_submodule("tensor");
  py::class_<Tensor>(tensor, "Tensor", py::buffer_protocol())
      .def(py::init<>())
      .def_buffer(&bufferOf)
      .def("to_numpy", [](Tensor& t) { return py::array(bufferOf(t)); })
      .def(py::init<uintptr_t, uintptr_t, int, int64_t, std::vector<int64_t>, std::vector<int64_t>, int>(), py::arg("data_ptr"), py::arg("base_ptr"),
           py::arg("type"), py::arg("offset"), py::arg("size"), py::arg("stride"), py::arg("device") = -1)
      .def_readwrite("data", &Tensor::data).def_readwrite("base", &Tensor::base).def_readwrite("offset", &Tensor::offset)
      .def_readwrite("size", &Tensor::size).def_readwrite("stride", &Tensor::stride).def_readwrite("type", &Tensor::type)
      .def_readwrite("device", &Tensor::device)
      .def("print", &Tensor::print);
  tensor.attr("INT8") = (int)LLC_INT8; tensor.attr("INT16") = (int)LLC_INT16; tensor.attr("INT32") = (int)LLC_INT32;
  tensor.attr("INT64") = (int)LLC_INT64; tensor.attr("FLOAT32") = (int)LLC_FLOAT32; tensor.attr("DOUBL64") = (int)LLC_FLOAT64;
  tensor.attr("INT1") = (int)LLC_INT1; tensor.attr("FLOAT16") = (int)LLC_FLOAT16; tensor.attr("BFLOAT16") = (int)LLC_BFLOAT16;

  auto compiler = m.def_submodule("compiler");
  py::class_<Compiler>(compiler, "Compiler")
      .def(py::init<>())
      .def("compile_mlir_to_shared_lib", &Compiler::compile_mlir_to_shared_lib)
      .def("run_pass", &Compiler::run_pass);
  py::class_<CompileOptions>(compiler, "CompileOptions")
      .def(py::init<>())
      .def("set_log_root", [](CompileOptions& o, const std::string& v) { o.log_root = v; })
      .def("set_mode", [](CompileOptions& o, const std::string& v) { o.mode = v; })
      .def("set_target", [](CompileOptions& o, const std::string& v) { o.target = v; })
      .def("set_log_level", [](CompileOptions& o, const std::string& v) { o.log_level = v; })
      .def("set_pipeline", [](CompileOptions& o, const std::string& v) { o.pipeline = v; })
      .def("set_global_layout", [](CompileOptions& o, const std::string& v) { o.global_layout = v; })
      .def("set_cpu", [](CompileOptions& o, const std::string& v) { o.cpu = v; })
      .def("set_mtriple", [](CompileOptions& o, const std::string& v) { o.mtriple = v; })
      .def("set_precision", [](CompileOptions& o, const std::string& v) { o.precision = v; })
      .def("display_llvm_passes", [](CompileOptions& o, bool v) { o.llvm_passes = v; })
      .def("display_mlir_passes", [](CompileOptions& o, bool v) { o.mlir_passes = v; });

  auto executor = m.def_submodule("executor");
  executor.def("get_tool", &getTool);
  py::class_<Execution>(executor, "Execution")
      .def(py::init<>())
      .def("load", &Execution::load, py::arg("path"), py::arg("device") = 0, py::arg("weight_dir") = "")
      .def("loaded_from_pool", &Execution::loaded_from_pool)
      .def("run", &Execution::run, py::arg("inputs"), py::arg("outs"), py::arg("stream") = 0)
      .def("run_with_symbols", &Execution::run_with_symbols, py::arg("symbols"), py::arg("inputs"), py::arg("outs"), py::arg("stream") = 0)
      .def("output_shapes", &Execution::output_shapes)
      .def("profile", &Execution::profile, py::arg("symbols"), py::arg("inputs"), py::arg("outs"), py::arg("reps") = 5, py::arg("stream") = 0)
      .def("status", &Execution::status)
      .def("num_inputs", &Execution::num_inputs).def("num_outputs", &Execution::num_outputs).def("num_symbols", &Execution::num_symbols)
      .def("last_launch_count", &Execution::last_launch_count).def("arena_bytes", &Execution::arena_bytes);
  m.def("version", []() { return std::string(llc_version()); });
}

/* C ABI of the B200 execution backend: compile LLH text to a kernel plan, load
 * the plan onto a GPU, run it.
 *
 * This is the boundary a binding of the reference's pybind module `llcompiler_`
 * sits on (src/Pybind/Entrance.cpp:69-120).  Each entry point names the
 * reference interface it stands in for.  Every function returns 0 on success
 * and a non-zero LlcStatus otherwise; llc_last_error() then holds a message for
 * the calling thread.  No function allocates or frees memory the caller owns,
 * and no type from any tensor library appears in a signature.
 */
#ifndef LLC_RUNTIME_H_
#define LLC_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum LlcStatus {
  LLC_OK = 0,
  LLC_ERR_PARSE = 1,        /* malformed LLH text or plan */
  LLC_ERR_UNSUPPORTED = 2,  /* an op or attribute with no CUDA lowering */
  LLC_ERR_ARGUMENT = 3,     /* wrong tensor count, rank, dtype, extent or symbol value */
  LLC_ERR_IO = 4,           /* plan or weight file missing / unreadable */
  LLC_ERR_CUDA = 5,         /* a CUDA call failed, or no CUDA device is present */
  LLC_ERR_INTERNAL = 6
} LlcStatus;

/* Element type codes.  0..6 are the reference's
 * (include/llcompiler/Compiler/Tensor.h:25-33: INT8, INT16, INT32, INT64, FLOAT32,
 * DOUBL64, INT1); 7 and 8 are new, the reference has no 16-bit float path. */
typedef enum LlcDType {
  LLC_INT8 = 0, LLC_INT16 = 1, LLC_INT32 = 2, LLC_INT64 = 3, LLC_FLOAT32 = 4,
  LLC_FLOAT64 = 5, LLC_INT1 = 6, LLC_FLOAT16 = 7, LLC_BFLOAT16 = 8
} LlcDType;

/* Replaces llc::compiler::Tensor (include/llcompiler/Compiler/Tensor.h:35-48): a
 * non-owning description of caller memory.  `sizes` and `strides` are in
 * elements.  `device` is the CUDA ordinal the memory lives on, or -1 for host
 * memory (the reference only knows host memory); host tensors are staged through
 * the device inside llc_run.  `data` already includes any storage offset. */
typedef struct LlcTensor {
  void* data;
  int32_t dtype;   /* LlcDType */
  int32_t device;  /* -1 = host */
  int32_t rank;
  const int64_t* sizes;
  const int64_t* strides;
} LlcTensor;

/* Replaces llc::compiler::CompileOptions (include/llcompiler/Compiler/CompileOption.h:39-71).
 * NULL strings mean "default".  `precision` is new: how fp32 contractions are computed,
 * one of "fp32" (FMA), "tf32", "tf32x3" (three-pass split, fp32-grade), "auto". */
typedef struct LlcOptions {
  const char* mode;          /* "inference" | "training" (training is rejected) */
  const char* target;        /* "sm_100a"; "x86_64"/"x86" are accepted and mapped to it with a warning */
  const char* pipeline;      /* "cuda" | "transform" (alias) */
  const char* global_layout; /* "NCHW" | "NHWC": layout of the module's rank-4 tensors */
  const char* log_root;      /* when non-empty the pipeline stages are dumped below this directory */
  const char* log_level;
  const char* cpu;           /* accepted, ignored */
  const char* mtriple;       /* accepted, ignored */
  const char* precision;
} LlcOptions;

typedef struct LlcExec LlcExec;

/* Replaces LLCCompiler::generateSharedLibFromMLIRStr (src/Compiler/Compiler.cpp:296-348):
 * LLH module text in, path of the compiled artefact out (a kernel plan, "<hash>.llcplan",
 * where the reference writes "<hash>.so").  `out_path` receives a NUL-terminated path. */
int llc_compile(const char* mlir_text, const LlcOptions* options, char* out_path, size_t out_path_len);

/* Runs one named LLH-level pass (or "lower") over the text and returns the printed result in
 * a buffer owned by the library (valid until the next call on this thread).  This is what the
 * reference's llc-opt driver does for its lit tests (tools/llc-opt/llc-opt.cpp:37-60).
 * Passes: "parse", "operation-legalization", "remove-redundant-ops", "fuse-softmax", "infer-symbol-shape",
 * "decompose-ops", "transform-layout", "canonicalize", "inline" (the folders), "cse", "symbol-cse",
 * "unload-and-bind-encoding", "lower" (prints the kernel plan); a comma-separated list is applied in order. */
int llc_run_pass(const char* mlir_text, const char* pass, const LlcOptions* options, const char** out_text);

/* Replaces llc::compiler::Execution::load (src/Compiler/Execution.cpp:10-19): reads the plan,
 * uploads the weights named by its llh.weight files to `device`, runs the load-time kernels
 * (weight re-layout, folded batch-norm vectors).  Allocates device memory. */
int llc_load(const char* plan_path, int device, LlcExec** out_exec);

/* llc_load with a weight directory (NULL or "" = llc_load): the .npy files the plan names are looked up in
 * `weight_dir` by file name first, and the uploaded, re-laid-out weight pool is kept there as `pool.bin` (tied to the
 * plan text, the pool size and the library build): a later load of the same plan from the same directory reads that
 * one file, uploads it and runs no load-time kernel.  This is the run side of the plan and weight cache; the
 * reference names its artefact after a hash of the module text (src/Compiler/Compiler.cpp:305-309) but rebuilds it
 * and re-dumps the weights on every compile (llcompiler/importer/fx_translate.py:416-436).
 * llc_loaded_from_pool tells which way a handle was loaded (1 = from pool.bin). */
int llc_load_from(const char* plan_path, const char* weight_dir, int device, LlcExec** out_exec);
int llc_loaded_from_pool(const LlcExec* exec);

int llc_num_inputs(const LlcExec* exec);
int llc_num_outputs(const LlcExec* exec);
int llc_num_symbols(const LlcExec* exec);

/* Output extents for a given binding, so that the caller can allocate results without
 * re-tracing the model (the reference re-runs FakeTensorProp on every call,
 * llcompiler/executor/out_put_call.py:154-170).  `sizes` must hold 8 entries. */
int llc_output_shape(LlcExec* exec, const int64_t* symbols, int n_symbols, const LlcTensor* inputs,
                     int n_inputs, int out_index, int64_t* sizes, int32_t* rank, int32_t* dtype);

/* Replaces llc::compiler::Execution::run / run_with_symbols (src/Compiler/Execution.cpp:21-66):
 * caller-allocated inputs and outputs, symbol values in the order of the function's i64
 * arguments.  Kernels are enqueued on `stream` (a cudaStream_t, NULL = the legacy default
 * stream); the call returns after enqueueing when every tensor is device memory and after
 * the results have reached the host otherwise. */
int llc_run(LlcExec* exec, const int64_t* symbols, int n_symbols, const LlcTensor* inputs, int n_inputs,
            LlcTensor* outputs, int n_outputs, void* stream);

/* Reads and clears the failure words the kernels of this executor's device write when they cannot raise an error
 * themselves: a bounded wait of a tensor-core kernel that gave up (words[0] GEMM / convolution, words[1] attention; see
 * llc_cuda_status for the codes) and the number of embedding indices that lay outside their table (words[2]; such rows
 * are written as zeros).  Returns LLC_OK when all three are zero, LLC_ERR_ARGUMENT for bad indices, LLC_ERR_CUDA for a
 * wait that gave up.  `words` may be NULL.  Synchronises the device.  llc_run and llc_profile make the same check
 * themselves whenever they wait for their results (host tensors); a caller that passes device tensors gets control
 * back before the kernels have run and calls this after its own synchronisation.  The reference has no counterpart: its
 * CHECK macros log and carry on (include/llcompiler/Support/Logger.h:126-134). */
int llc_status(LlcExec* exec, int32_t* words);

/* Threading: calls on one LlcExec are serialised by a lock inside it (bindings, arena and staging buffers are shared
 * state), so two threads may share a handle but do not overlap; different handles are independent.  Every entry point
 * leaves the calling thread's current CUDA device as it found it. */

/* Same arguments as llc_run; runs the plan `reps` times (after one warm-up pass) with CUDA events
 * around every kernel and writes a text report: one "step <i> <kernel> <ms> <flops> <bytes>" line per
 * plan step and one "kernel <name> <launches> <ms> <flops> <bytes>" line per kernel family (ms and
 * work per run; flops and bytes are the algorithmic figures).  The reference's only timing aid is a
 * wall-clock decorator (llcompiler/utility/utility.py:6-15). */
int llc_profile(LlcExec* exec, const int64_t* symbols, int n_symbols, const LlcTensor* inputs, int n_inputs,
                LlcTensor* outputs, int n_outputs, int reps, void* stream, char* report, size_t report_len);

/* Number of kernels the last llc_run on this handle launched, and arena bytes in use. */
int64_t llc_last_launch_count(const LlcExec* exec);
int64_t llc_arena_bytes(const LlcExec* exec);

void llc_free(LlcExec* exec);
const char* llc_last_error(void);
const char* llc_version(void);

#ifdef __cplusplus
}
#endif
#endif /* LLC_RUNTIME_H_ */

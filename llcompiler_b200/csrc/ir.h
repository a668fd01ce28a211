// A self-contained IR for the textual LLH dialect.
//
// The reference parses the importer's text with MLIR
// (src/Compiler/Compiler.cpp:296-304) and works on MLIR operations.  MLIR is
// not available, so this is the subset the LLH surface needs: modules,
// func.func with argument attributes, SSA values, generic-form operations with
// properties/attributes, tensor types with an optional #llh.encoding, and the
// attribute kinds the importer prints (include/llcompiler/Dialect/LLH/IR/
// LLHOps.td, LLHAttrs.td:30-51, LLHEnums.td:22-137).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "expr.h"

namespace llc {

enum class DType { F32, BF16, F16, F64, I64, I32, I16, I8, I1, Index, None };
const char* dtypeName(DType t);
int dtypeSize(DType t);
bool dtypeFromName(const std::string& s, DType& out);
inline bool isFloat(DType t) { return t == DType::F32 || t == DType::BF16 || t == DType::F16 || t == DType::F64; }

constexpr int64_t kDynamic = INT64_MIN;

struct Type {
  enum Kind { None, Scalar, Tensor } kind = None;
  DType elt = DType::None;
  std::vector<int64_t> dims;          // kDynamic for '?'
  bool unranked = false;              // tensor<*xT>
  std::vector<std::string> encoding;  // #llh.encoding<shapes = @s0, @c3>; empty = none
  static Type scalar(DType t) { Type r; r.kind = Scalar; r.elt = t; return r; }
  static Type tensor(DType t, std::vector<int64_t> d) { Type r; r.kind = Tensor; r.elt = t; r.dims = std::move(d); return r; }
  bool isTensor() const { return kind == Tensor; }
  std::string str() const;
};

struct Attr {
  enum Kind { Unit, Int, Float, Str, Bool, IntArray, Dense, Enum, SymRef, TypeAttr, Array, Dict, Raw } kind = Unit;
  int64_t i = 0;
  double f = 0;
  std::string s;               // Str / SymRef / Raw text / Enum value ("NCHW") ; enum kind in s2
  std::string s2;              // Enum kind ("Layout") ; IntArray element type ("i64")
  std::vector<int64_t> ints;   // IntArray, integer Dense payload
  std::vector<double> floats;  // float Dense payload
  Type type;                   // Int/Float/Dense type, TypeAttr
  std::vector<Attr> elems;     // Array
  std::vector<std::pair<std::string, Attr>> dict;  // Dict
  bool splat = false;
  std::string str() const;
  static Attr integer(int64_t v, DType t = DType::I64) { Attr a; a.kind = Int; a.i = v; a.type = Type::scalar(t); return a; }
  static Attr floating(double v, DType t = DType::F64) { Attr a; a.kind = Float; a.f = v; a.type = Type::scalar(t); return a; }
  static Attr string(const std::string& v) { Attr a; a.kind = Str; a.s = v; return a; }
  static Attr array(const std::vector<int64_t>& v) { Attr a; a.kind = IntArray; a.ints = v; a.s2 = "i64"; return a; }
  static Attr enumeration(const std::string& kind, const std::string& v) { Attr a; a.kind = Enum; a.s2 = kind; a.s = v; return a; }
  static Attr boolean(bool v) { Attr a; a.kind = Bool; a.i = v; return a; }
};

using AttrList = std::vector<std::pair<std::string, Attr>>;
const Attr* findAttr(const AttrList& l, const std::string& name);

struct Op;
struct Value {
  std::string name;   // "%5"
  Type type;
  Op* def = nullptr;  // null for function arguments
  int index = 0;      // result index or argument index
  std::vector<Op*> users;
};

struct Op {
  std::string name;  // "llh.conv"
  std::vector<Value*> operands;
  AttrList props;    // <{...}>
  AttrList attrs;    // {...}
  std::vector<Value*> results;
  bool erased = false;
  std::string written;   // the op's name in the input when it was read from another dialect's custom form ("tensor.dim", "arith.subi", ...)
  const Attr* attr(const std::string& n) const { const Attr* a = findAttr(props, n); return a ? a : findAttr(attrs, n); }
  void setProp(const std::string& n, const Attr& a);
};

struct Func {
  std::string name;
  std::vector<Value*> args;
  std::vector<AttrList> argAttrs;
  std::vector<Type> resultTypes;
  AttrList attrs;
  std::vector<Op*> ops;  // includes the terminator ("func.return")
};

struct Module {
  std::string symName;
  AttrList attrs;
  std::vector<Func> funcs;
  std::vector<std::unique_ptr<Value>> valueStore;
  std::vector<std::unique_ptr<Op>> opStore;
  std::vector<std::string> leadingLines;  // "#map = ..." aliases kept verbatim
  std::vector<std::string> symbolRelations;   // generic-form "llh.symbol_relation" lines printed after the functions
  std::vector<std::string> symbolDecls;   // names declared as "llh.symbolic_int" ops at the head of the module body
  // relations read from the input (module level or the nested module @__symbol__): kind ("EQ", "GE", ...), the two
  // symbols, and the op as written
  struct ParsedRelation { std::string kind, symbol, relation, text; };
  std::vector<ParsedRelation> parsedRelations;
  bool hasSymbolModule = false;           // print `module @__symbol__ { ... }` even when it holds no relation
  Value* newValue(const Type& t, const std::string& name = "");
  Op* newOp(const std::string& name);
  Func* entrance();
  void recomputeUsers();
  std::string str() const;
};

// Parses one module (or a bare list of func.func, which the reference's lit files use).
// Throws std::runtime_error with line/column on malformed input.
std::unique_ptr<Module> parseModule(const std::string& text);
// Splits a lit file at "// -----" markers.
std::vector<std::string> splitInputFile(const std::string& text);

}  // namespace llc

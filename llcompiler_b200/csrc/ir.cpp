// Parser and printer for the textual LLH surface (see ir.h).
#include "ir.h"
#include <map>

#include <cmath>
#include <cstring>
#include <sstream>

namespace llc {

// ------------------------------------------------------------------ dtypes
const char* dtypeName(DType t) {
  switch (t) {
    case DType::F32: return "f32"; case DType::BF16: return "bf16"; case DType::F16: return "f16";
    case DType::F64: return "f64"; case DType::I64: return "i64"; case DType::I32: return "i32";
    case DType::I16: return "i16"; case DType::I8: return "i8"; case DType::I1: return "i1";
    case DType::Index: return "index"; default: return "none";
  }
}
int dtypeSize(DType t) {
  switch (t) {
    case DType::F32: case DType::I32: return 4;
    case DType::BF16: case DType::F16: case DType::I16: return 2;
    case DType::F64: case DType::I64: case DType::Index: return 8;
    case DType::I8: case DType::I1: return 1;
    default: return 0;
  }
}
bool dtypeFromName(const std::string& s, DType& out) {
  static const std::pair<const char*, DType> table[] = {
      {"f32", DType::F32}, {"bf16", DType::BF16}, {"f16", DType::F16}, {"f64", DType::F64},
      {"i64", DType::I64}, {"i32", DType::I32}, {"i16", DType::I16}, {"i8", DType::I8},
      {"i1", DType::I1}, {"index", DType::Index}, {"si64", DType::I64}, {"ui8", DType::I8}};
  for (auto& e : table) if (s == e.first) { out = e.second; return true; }
  return false;
}

const Attr* findAttr(const AttrList& l, const std::string& name) {
  for (auto& kv : l) if (kv.first == name) return &kv.second;
  return nullptr;
}
void Op::setProp(const std::string& n, const Attr& a) {
  for (auto& kv : props) if (kv.first == n) { kv.second = a; return; }
  props.emplace_back(n, a);
}

// ------------------------------------------------------------------ printing
static std::string fmtFloat(double v) {
  if (std::isnan(v)) return "0x7FC00000";
  if (std::isinf(v)) return v > 0 ? "0x7F800000" : "0xFF800000";
  char buf[64];
  snprintf(buf, sizeof buf, "%.6e", v);
  if (std::strtod(buf, nullptr) != v) snprintf(buf, sizeof buf, "%.17g", v);
  std::string s = buf;
  if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
  return s;
}

std::string Type::str() const {
  if (kind == Scalar) return dtypeName(elt);
  if (kind != Tensor) return "none";
  std::string o = "tensor<";
  if (unranked) o += "*x";
  for (auto d : dims) o += (d == kDynamic ? std::string("?") : std::to_string(d)) + "x";
  o += dtypeName(elt);
  if (!encoding.empty()) {
    o += ", #llh.encoding<shapes = ";
    for (size_t i = 0; i < encoding.size(); ++i) {
      if (i) o += ", ";
      const std::string& e = encoding[i];
      bool plain = !e.empty();
      for (char c : e) if (!(std::isalnum((unsigned char)c) || c == '_')) plain = false;
      o += plain ? "@" + e : "@\"" + e + "\"";
    }
    o += ">";
  }
  return o + ">";
}

static std::string quote(const std::string& s) {
  std::string o = "\"";
  for (char c : s) { if (c == '"' || c == '\\') o += '\\'; o += c; }
  return o + "\"";
}

std::string Attr::str() const {
  switch (kind) {
    case Unit: return "unit";
    case Int: return std::to_string(i) + (type.kind == Type::None ? "" : " : " + type.str());
    case Float: return fmtFloat(f) + (type.kind == Type::None ? "" : " : " + type.str());
    case Str: return quote(s);
    case Bool: return i ? "true" : "false";
    case IntArray: {
      std::string o = "array<" + (s2.empty() ? std::string("i64") : s2);
      for (size_t k = 0; k < ints.size(); ++k) o += (k ? ", " : ": ") + std::to_string(ints[k]);
      return o + ">";
    }
    case Dense: {
      std::string o = "dense<";
      bool isF = isFloat(type.elt);
      size_t n = isF ? floats.size() : ints.size();
      auto one = [&](size_t k) {
        if (isF) return fmtFloat(floats[k]);
        if (type.elt == DType::I1) return std::string(ints[k] ? "true" : "false");
        return std::to_string(ints[k]);
      };
      if (splat || n == 1) o += n ? one(0) : "";
      else { o += "["; for (size_t k = 0; k < n; ++k) o += (k ? ", " : "") + one(k); o += "]"; }
      return o + "> : " + type.str();
    }
    case Enum: return "#llh." + s2 + "<" + s + ">";
    case SymRef: return "@" + s;
    case TypeAttr: return type.str();
    case Array: {
      std::string o = "[";
      for (size_t k = 0; k < elems.size(); ++k) o += (k ? ", " : "") + elems[k].str();
      return o + "]";
    }
    case Dict: {
      std::string o = "{";
      for (size_t k = 0; k < dict.size(); ++k) o += (k ? ", " : "") + dict[k].first + " = " + dict[k].second.str();
      return o + "}";
    }
    case Raw: return s;
  }
  return "";
}

static std::string attrListStr(const AttrList& l) {
  std::string o;
  for (size_t k = 0; k < l.size(); ++k) {
    o += (k ? ", " : "") + l[k].first;
    if (l[k].second.kind != Attr::Unit) o += " = " + l[k].second.str();
  }
  return o;
}

Value* Module::newValue(const Type& t, const std::string& name) {
  valueStore.emplace_back(new Value());
  Value* v = valueStore.back().get();
  v->type = t;
  v->name = name.empty() ? "%v" + std::to_string(valueStore.size()) : name;
  return v;
}
Op* Module::newOp(const std::string& name) {
  opStore.emplace_back(new Op());
  opStore.back()->name = name;
  return opStore.back().get();
}
Func* Module::entrance() {
  for (auto& f : funcs) if (findAttr(f.attrs, "entrance")) return &f;
  for (auto& f : funcs) if (f.name == "main") return &f;
  return funcs.empty() ? nullptr : &funcs[0];
}
void Module::recomputeUsers() {
  for (auto& v : valueStore) v->users.clear();
  for (auto& f : funcs)
    for (Op* op : f.ops) {
      if (op->erased) continue;
      for (Value* v : op->operands) v->users.push_back(op);
    }
}

std::string Module::str() const {
  std::ostringstream o;
  for (auto& l : leadingLines) o << l << "\n";
  o << "module";
  if (!symName.empty()) o << " @" << symName;
  if (!attrs.empty()) o << " attributes {" << attrListStr(attrs) << "}";
  o << " {\n";
  for (auto& n : symbolDecls) o << "  \"llh.symbolic_int\"() <{sym_name = \"" << n << "\"}> : () -> ()\n";
  for (auto& f : funcs) {
    // SSA names are assigned in print order, the way MLIR's printer does: %arg0.. for arguments, %0.. for results
    std::map<const Value*, std::string> names;
    for (size_t i = 0; i < f.args.size(); ++i) names[f.args[i]] = "%arg" + std::to_string(i);
    { int n = 0; for (Op* op : f.ops) if (!op->erased) for (Value* r : op->results) names[r] = "%" + std::to_string(n++); }
    auto nm = [&](const Value* v) -> const std::string& { auto it = names.find(v); return it == names.end() ? v->name : it->second; };
    o << "  func.func @" << f.name << "(";
    for (size_t i = 0; i < f.args.size(); ++i) {
      o << (i ? ", " : "") << nm(f.args[i]) << ": " << f.args[i]->type.str();
      if (i < f.argAttrs.size() && !f.argAttrs[i].empty()) o << " {" << attrListStr(f.argAttrs[i]) << "}";
    }
    o << ")";
    if (!f.resultTypes.empty()) {
      o << " -> ";
      if (f.resultTypes.size() > 1) o << "(";
      for (size_t i = 0; i < f.resultTypes.size(); ++i) o << (i ? ", " : "") << f.resultTypes[i].str();
      if (f.resultTypes.size() > 1) o << ")";
    }
    if (!f.attrs.empty()) o << " attributes {" << attrListStr(f.attrs) << "}";
    o << " {\n";
    for (Op* op : f.ops) {
      if (op->erased) continue;
      o << "    ";
      if (op->name == "func.return") {
        o << "return";
        for (size_t i = 0; i < op->operands.size(); ++i) o << (i ? ", " : " ") << nm(op->operands[i]);
        if (!op->operands.empty()) o << " : ";
        for (size_t i = 0; i < op->operands.size(); ++i) o << (i ? ", " : "") << op->operands[i]->type.str();
        o << "\n";
        continue;
      }
      for (size_t i = 0; i < op->results.size(); ++i) o << (i ? ", " : "") << nm(op->results[i]);
      if (!op->results.empty()) o << " = ";
      if (op->written == "arith.constant" && op->attrs.empty() && op->props.size() == 1 && op->props[0].first == "value") {
        o << "arith.constant " << op->props[0].second.str() << "\n";      // MLIR's custom form: `arith.constant 0 : index`
        continue;
      }
      o << "\"" << (op->written.empty() ? op->name : op->written) << "\"(";
      for (size_t i = 0; i < op->operands.size(); ++i) o << (i ? ", " : "") << nm(op->operands[i]);
      o << ")";
      if (!op->props.empty()) o << " <{" << attrListStr(op->props) << "}>";
      if (!op->attrs.empty()) o << " {" << attrListStr(op->attrs) << "}";
      o << " : (";
      for (size_t i = 0; i < op->operands.size(); ++i) o << (i ? ", " : "") << op->operands[i]->type.str();
      o << ") -> ";
      if (op->results.size() != 1) o << "(";
      for (size_t i = 0; i < op->results.size(); ++i) o << (i ? ", " : "") << op->results[i]->type.str();
      if (op->results.size() != 1) o << ")";
      o << "\n";
    }
    o << "  }\n";
  }
  if (!symbolRelations.empty() || hasSymbolModule) {   // the relations live in a module of their own, as in the reference's output
    o << "  module @__symbol__ {\n";
    for (auto& l : symbolRelations) o << "    " << l << "\n";
    o << "  }\n";
  }
  o << "}\n";
  return o.str();
}

// ------------------------------------------------------------------ parsing
namespace {
struct Parser {
  const std::string& s;
  size_t p = 0;
  Module* m;
  std::map<std::string, Value*> values;
  explicit Parser(const std::string& text, Module* mod) : s(text), m(mod) {}

  [[noreturn]] void fail(const std::string& msg) {
    size_t line = 1, col = 1;
    for (size_t i = 0; i < p && i < s.size(); ++i) { if (s[i] == '\n') { ++line; col = 1; } else ++col; }
    throw std::runtime_error("LLH parse error at " + std::to_string(line) + ":" + std::to_string(col) + ": " + msg);
  }
  void ws() {
    for (;;) {
      while (p < s.size() && std::isspace((unsigned char)s[p])) ++p;
      if (p + 1 < s.size() && s[p] == '/' && s[p + 1] == '/') { while (p < s.size() && s[p] != '\n') ++p; continue; }
      break;
    }
  }
  bool eof() { ws(); return p >= s.size(); }
  bool peek(const char* t) { ws(); return s.compare(p, strlen(t), t) == 0; }
  bool peekWord(const char* t) {
    ws(); size_t n = strlen(t);
    if (s.compare(p, n, t) != 0) return false;
    char c = p + n < s.size() ? s[p + n] : ' ';
    return !(std::isalnum((unsigned char)c) || c == '_' || c == '.');
  }
  bool eat(const char* t) { if (peek(t)) { p += strlen(t); return true; } return false; }
  bool eatWord(const char* t) { if (peekWord(t)) { p += strlen(t); return true; } return false; }
  void expect(const char* t) { if (!eat(t)) fail(std::string("expected '") + t + "'"); }
  static bool identChar(char c) { return std::isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$'; }
  std::string ident() {
    ws(); size_t b = p;
    while (p < s.size() && identChar(s[p])) ++p;
    if (b == p) fail("expected identifier");
    return s.substr(b, p - b);
  }
  std::string stringLit() {
    ws(); if (p >= s.size() || s[p] != '"') fail("expected string");
    ++p; std::string o;
    while (p < s.size() && s[p] != '"') { if (s[p] == '\\' && p + 1 < s.size()) ++p; o += s[p++]; }
    if (p >= s.size()) fail("unterminated string");
    ++p; return o;
  }
  std::string balanced(char open, char close) {  // consumes from the opening char
    ws(); if (s[p] != open) fail("expected opening bracket");
    size_t b = p; int depth = 0;
    while (p < s.size()) {
      if (s[p] == '"') { stringLit(); continue; }
      if (s[p] == open) ++depth;
      else if (s[p] == close && !(close == '>' && p > 0 && s[p - 1] == '-')) { if (--depth == 0) { ++p; break; } }
      ++p;
    }
    return s.substr(b, p - b);
  }
  std::string valueName() {
    ws(); if (p >= s.size() || s[p] != '%') fail("expected SSA value");
    size_t b = p++;
    while (p < s.size() && (std::isalnum((unsigned char)s[p]) || s[p] == '_' || s[p] == '.' || s[p] == '$' || s[p] == '#')) ++p;
    return s.substr(b, p - b);
  }

  Type type() {
    ws();
    if (eat("tensor<")) {
      Type t; t.kind = Type::Tensor;
      ws();
      if (eat("*x")) t.unranked = true;
      for (;;) {
        ws();
        if (s[p] == '?') { ++p; expect("x"); t.dims.push_back(kDynamic); continue; }
        if (std::isdigit((unsigned char)s[p])) {
          size_t q = p; int64_t v = 0;
          while (q < s.size() && std::isdigit((unsigned char)s[q])) v = v * 10 + (s[q++] - '0');
          if (q < s.size() && s[q] == 'x') { p = q + 1; t.dims.push_back(v); continue; }
        }
        break;
      }
      std::string e = ident();
      if (!dtypeFromName(e, t.elt)) fail("unknown element type '" + e + "'");
      if (eat(",")) {
        ws();
        if (eat("#llh.encoding<")) {
          expect("shapes"); expect("=");
          for (;;) {
            expect("@");
            ws();
            t.encoding.push_back(s[p] == '"' ? stringLit() : ident());
            if (!eat(",")) break;
          }
          expect(">");
        } else if (!peek(">")) {
          // unknown encoding: skip it
          while (p < s.size() && s[p] != '>') { if (s[p] == '<') balanced('<', '>'); else ++p; }
        }
      }
      expect(">");
      return t;
    }
    if (peek("(")) { balanced('(', ')'); ws(); if (eat("->")) type(); return Type(); }  // function type: skipped
    std::string e = ident();
    DType d;
    if (dtypeFromName(e, d)) return Type::scalar(d);
    if (peek("<")) balanced('<', '>');
    return Type();  // unknown types (memref, !llvm.ptr, ...) are carried as None
  }

  void denseBody(Attr& a) {
    ws();
    if (eat("[")) { if (eat("]")) return; for (;;) { denseBody(a); if (!eat(",")) break; } expect("]"); return; }
    if (eatWord("true")) { a.ints.push_back(1); a.floats.push_back(1); return; }
    if (eatWord("false")) { a.ints.push_back(0); a.floats.push_back(0); return; }
    if (peek("\"")) { a.s = stringLit(); return; }   // hex blob: not needed by the LLH surface
    double v; bool isInt; int64_t iv;
    number(v, isInt, iv);
    a.floats.push_back(v); a.ints.push_back(isInt ? iv : (int64_t)v);
  }
  void number(double& v, bool& isInt, int64_t& iv) {
    ws(); size_t b = p;
    if (s.compare(p, 2, "0x") == 0 || s.compare(p, 3, "-0x") == 0) {
      bool neg = s[p] == '-'; if (neg) ++p; p += 2; size_t h = p;
      while (p < s.size() && std::isxdigit((unsigned char)s[p])) ++p;
      uint64_t bits = std::stoull(s.substr(h, p - h), nullptr, 16);
      isInt = false; iv = (int64_t)bits;
      if (p - h <= 8) { uint32_t u = (uint32_t)bits; float f; memcpy(&f, &u, 4); v = f; }
      else { memcpy(&v, &bits, 8); }
      if (neg) v = -v;
      return;
    }
    if (p < s.size() && (s[p] == '-' || s[p] == '+')) ++p;
    bool fl = false;
    while (p < s.size() && (std::isdigit((unsigned char)s[p]) || s[p] == '.' || s[p] == 'e' || s[p] == 'E' ||
                            ((s[p] == '-' || s[p] == '+') && (s[p - 1] == 'e' || s[p - 1] == 'E')))) {
      if (s[p] == '.' || s[p] == 'e' || s[p] == 'E') fl = true;
      ++p;
    }
    if (p == b) fail("expected number");
    std::string t = s.substr(b, p - b);
    isInt = !fl;
    v = std::strtod(t.c_str(), nullptr);
    iv = isInt ? (int64_t)std::strtoll(t.c_str(), nullptr, 10) : (int64_t)v;
    if (isInt && t.size() > 18) iv = (int64_t)std::strtoull(t.c_str(), nullptr, 10);
  }

  Attr attrValue() {
    ws();
    Attr a;
    if (p >= s.size()) fail("expected attribute");
    char c = s[p];
    if (c == '"') { a.kind = Attr::Str; a.s = stringLit(); if (eat(":")) type(); return a; }
    if (eatWord("true")) return Attr::boolean(true);
    if (eatWord("false")) return Attr::boolean(false);
    if (eatWord("unit")) return a;
    if (eat("array<")) {
      a.kind = Attr::IntArray; a.s2 = ident();
      if (eat(":")) { for (;;) { double v; bool isI; int64_t iv; number(v, isI, iv); a.ints.push_back(iv); if (!eat(",")) break; } }
      expect(">");
      return a;
    }
    if (eat("dense<")) {
      a.kind = Attr::Dense;
      if (!peek(">")) denseBody(a);
      expect(">"); expect(":");
      a.type = type();
      int64_t n = 1; for (auto d : a.type.dims) n *= d;
      a.splat = (int64_t)a.ints.size() == 1 && n != 1;
      return a;
    }
    if (eat("#llh.")) {
      a.kind = Attr::Enum; a.s2 = ident();
      if (peek("<")) { std::string b = balanced('<', '>'); a.s = b.substr(1, b.size() - 2); }
      return a;
    }
    if (c == '#') { a.kind = Attr::Raw; size_t b = p; ++p; ident(); if (peek("<")) balanced('<', '>'); a.s = s.substr(b, p - b); return a; }
    if (c == '@') { ++p; a.kind = Attr::SymRef; ws(); a.s = s[p] == '"' ? stringLit() : ident(); return a; }
    if (c == '[') {
      ++p; a.kind = Attr::Array;
      if (!eat("]")) { for (;;) { a.elems.push_back(attrValue()); if (!eat(",")) break; } expect("]"); }
      return a;
    }
    if (c == '{') { a.kind = Attr::Dict; a.dict = attrDict("{", "}"); return a; }
    if (peek("affine_map<") || peek("affine_set<")) { a.kind = Attr::Raw; size_t b = p; ident(); balanced('<', '>'); a.s = s.substr(b, p - b); return a; }
    if (std::isdigit((unsigned char)c) || c == '-' || c == '+') {
      double v; bool isInt; int64_t iv;
      number(v, isInt, iv);
      Type t;
      if (eat(":")) t = type();
      if (t.kind == Type::Scalar && isFloat(t.elt)) { a.kind = Attr::Float; a.f = v; }
      else if (!isInt && t.kind == Type::None) { a.kind = Attr::Float; a.f = v; }
      else if (!isInt) { a.kind = Attr::Float; a.f = v; }
      else { a.kind = Attr::Int; a.i = iv; }
      a.type = t;
      return a;
    }
    // a type used as an attribute
    a.kind = Attr::TypeAttr; a.type = type();
    return a;
  }

  AttrList attrDict(const char* open, const char* close) {
    AttrList out;
    expect(open);
    if (eat(close)) return out;
    for (;;) {
      ws();
      std::string key = s[p] == '"' ? stringLit() : ident();
      Attr v;
      if (eat("=")) v = attrValue();
      out.emplace_back(key, v);
      if (!eat(",")) break;
    }
    expect(close);
    return out;
  }

  Value* use(const std::string& name) {
    auto it = values.find(name);
    if (it == values.end()) fail("use of undefined value " + name);
    return it->second;
  }

  std::vector<Type> typeList() {
    std::vector<Type> out;
    if (eat("(")) {
      if (eat(")")) return out;
      for (;;) { out.push_back(type()); if (peek("{")) attrDict("{", "}"); if (!eat(",")) break; }
      expect(")");
    } else out.push_back(type());
    return out;
  }

  void operation(Func& f) {
    std::vector<std::string> resultNames;
    ws();
    if (s[p] == '%') {
      for (;;) {
        std::string n = valueName();
        int count = 1;
        if (eat(":")) { double v; bool b; int64_t iv; number(v, b, iv); count = (int)iv; }
        if (count == 1) resultNames.push_back(n);
        else for (int k = 0; k < count; ++k) resultNames.push_back(n + "#" + std::to_string(k));
        if (!eat(",")) break;
      }
      expect("=");
    }
    ws();
    Op* op = nullptr;
    if (s[p] == '"') {
      op = m->newOp(stringLit());
      expect("(");
      if (!eat(")")) { for (;;) { op->operands.push_back(use(valueName())); if (!eat(",")) break; } expect(")"); }
      if (peek("<{")) op->props = attrDict("<{", "}>");
      if (peek("(")) fail("operations with regions are not part of the LLH surface");
      if (peek("{")) op->attrs = attrDict("{", "}");
      expect(":");
      std::vector<Type> inTypes = typeList();
      expect("->");
      std::vector<Type> outTypes = typeList();
      if (inTypes.size() != op->operands.size()) fail("operand/type count mismatch on " + op->name);
      if (outTypes.size() != resultNames.size()) fail("result/type count mismatch on " + op->name);
      for (size_t i = 0; i < outTypes.size(); ++i) {
        Value* v = m->newValue(outTypes[i], resultNames[i]);
        v->def = op; v->index = (int)i;
        op->results.push_back(v); values[resultNames[i]] = v;
      }
    } else {
      std::string name = ident();
      if (name == "return" || name == "func.return") {
        op = m->newOp("func.return");
        ws();
        if (p < s.size() && s[p] == '%') {
          for (;;) { op->operands.push_back(use(valueName())); if (!eat(",")) break; }
          expect(":");
          for (size_t i = 0; i < op->operands.size(); ++i) { type(); if (i + 1 < op->operands.size()) expect(","); }
        }
      } else if (name == "arith.constant") {
        op = m->newOp("llh.constant");
        op->written = name;
        if (peek("{")) op->attrs = attrDict("{", "}");
        Attr v = attrValue();
        op->props.emplace_back("value", v);
        if (resultNames.size() != 1) fail("arith.constant needs one result");
        Type t = v.type;
        if (t.kind == Type::Scalar && t.elt == DType::Index) t.elt = DType::I64;
        Value* r = m->newValue(t, resultNames[0]);
        r->def = op; op->results.push_back(r); values[resultNames[0]] = r;
      } else if (name == "tensor.dim" || name == "arith.addi" || name == "arith.subi" || name == "arith.muli" || name == "arith.divsi" ||
                 name == "arith.index_cast") {
        // index arithmetic around shapes, in MLIR's custom form; read as the LLH scalar ops over i64 that say the same
        // (`tensor.dim %t, %i : type`, `arith.subi %a, %b : index`, `arith.index_cast %a : index to i64`)
        static const std::map<std::string, std::string> same = {{"tensor.dim", "llh.dim"}, {"arith.addi", "llh.add"}, {"arith.subi", "llh.sub"},
                                                                {"arith.muli", "llh.mul"}, {"arith.divsi", "llh.div"}, {"arith.index_cast", "llh.scalar_cast"}};
        op = m->newOp(same.at(name));
        op->written = name;
        if (peek("{")) op->attrs = attrDict("{", "}");
        for (;;) { op->operands.push_back(use(valueName())); if (!eat(",")) break; }
        expect(":");
        type();
        if (name == "arith.index_cast") { if (!eatWord("to")) fail("arith.index_cast: expected 'to'"); type(); }
        if (resultNames.size() != 1) fail(name + " needs one result");
        Value* r = m->newValue(Type::scalar(DType::I64), resultNames[0]);
        r->def = op; op->results.push_back(r); values[resultNames[0]] = r;
      } else {
        fail("unsupported custom-form operation '" + name + "'");
      }
    }
    f.ops.push_back(op);
  }

  void function() {
    eatWord("private"); eatWord("public");
    expect("@");
    Func f;
    f.name = ident();
    values.clear();
    expect("(");
    if (!eat(")")) {
      for (;;) {
        ws();
        if (s[p] == '%') {
          std::string n = valueName();
          expect(":");
          Type t = type();
          Value* v = m->newValue(t, n);
          v->index = (int)f.args.size();
          f.args.push_back(v); values[n] = v;
          f.argAttrs.emplace_back(peek("{") ? attrDict("{", "}") : AttrList());
        } else {
          type();  // declaration without names
          if (peek("{")) attrDict("{", "}");
        }
        if (!eat(",")) break;
      }
      expect(")");
    }
    if (eat("->")) f.resultTypes = typeList();
    if (eatWord("attributes")) f.attrs = attrDict("{", "}");
    if (eat("{")) {
      while (!peek("}")) { if (eof()) fail("unterminated function body"); operation(f); }
      expect("}");
    }
    m->funcs.push_back(std::move(f));
  }

  void keepRelation(Op* op, std::string text) {
    if (op->name != "llh.symbol_relation" && op->name != "llh.symbol_relation_map" && op->name != "llh.symbol_binary_relation") return;
    Module::ParsedRelation r;
    while (!text.empty() && isspace((unsigned char)text.front())) text.erase(text.begin());
    while (!text.empty() && isspace((unsigned char)text.back())) text.pop_back();
    r.text = text;
    if (const Attr* a = op->attr("relation_kind")) { size_t lt = a->s.find('<'), gt = a->s.rfind('>'); r.kind = lt != std::string::npos && gt != std::string::npos ? a->s.substr(lt + 1, gt - lt - 1) : a->s; }
    if (const Attr* a = op->attr("symbol")) r.symbol = a->s;
    if (const Attr* a = op->attr("relation")) r.relation = a->s;
    if (op->name != "llh.symbol_relation") r.kind = op->name;
    m->parsedRelations.push_back(r);
  }

  void moduleBody() {
    for (;;) {
      if (eof() || peek("}")) return;
      if (eatWord("func.func")) { function(); continue; }
      if (peekWord("module") || peekWord("builtin.module")) {  // nested module (@__symbol__ and the like): only its symbol relations are kept
        ident(); if (eat("@")) ident();
        if (eatWord("attributes")) attrDict("{", "}");
        expect("{");
        m->hasSymbolModule = true;
        while (!peek("}")) {
          if (eof()) fail("unterminated nested module");
          const size_t b = p;
          Func dummy; operation(dummy);
          if (!dummy.ops.empty()) keepRelation(dummy.ops.back(), s.substr(b, p - b));
        }
        expect("}");
        continue;
      }
      if (peek("\"llh.symbolic_int\"") || peek("\"llh.")) {  // module-level symbol declarations: kept, in order, for printing
        const size_t opBegin = p;
        Func dummy; operation(dummy);
        if (!dummy.ops.empty()) keepRelation(dummy.ops.back(), s.substr(opBegin, p - opBegin));
        if (!dummy.ops.empty() && dummy.ops.back()->name == "llh.symbolic_int")
          if (const Attr* n = dummy.ops.back()->attr("sym_name")) {
            bool known = false;
            for (auto& d : m->symbolDecls) known = known || d == n->s;
            if (!known) m->symbolDecls.push_back(n->s);
          }
        continue;
      }
      fail("unexpected text at module level");
    }
  }

  void top() {
    // "#map = affine_map<...>" alias lines
    for (;;) {
      ws();
      if (p < s.size() && s[p] == '#') { size_t b = p; while (p < s.size() && s[p] != '\n') ++p; m->leadingLines.push_back(s.substr(b, p - b)); continue; }
      break;
    }
    if (eatWord("builtin.module") || eatWord("module")) {
      if (eat("@")) m->symName = ident();
      if (eatWord("attributes")) m->attrs = attrDict("{", "}");
      expect("{");
      moduleBody();
      expect("}");
    } else {
      moduleBody();
    }
    if (!eof()) fail("trailing text after module");
  }
};
}  // namespace

std::unique_ptr<Module> parseModule(const std::string& text) {
  std::unique_ptr<Module> m(new Module());
  Parser ps(text, m.get());
  ps.top();
  m->recomputeUsers();
  return m;
}

std::vector<std::string> splitInputFile(const std::string& text) {
  std::vector<std::string> out;
  std::string cur;
  std::istringstream in(text);
  std::string line;
  while (std::getline(in, line)) {
    size_t b = line.find_first_not_of(" \t");
    if (b != std::string::npos && line.compare(b, 8, "// -----") == 0) { out.push_back(cur); cur.clear(); continue; }
    cur += line + "\n";
  }
  out.push_back(cur);
  return out;
}

}  // namespace llc

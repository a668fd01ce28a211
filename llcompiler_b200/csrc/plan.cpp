// Text form of the kernel plan (see plan.h): printer and parser.
//
//   llcplan 1
//   option <key> <value>
//   nsymargs <n>
//   symbol <name> arg <k> | symbol <name> input <i> <dim>
//   buffer <id> <dtype> <temp|input|output|weight|const> <numel-expr> [index=<k>] [file="..."] [values=v,v,...]
//   input <k> <buf> <dtype> <d0,d1,...>
//   output <k> <buf> <dtype> <d0,d1,...>
//   step|init <kernel> <name>=<view>... <name>:<scalar>...
// A view is b<buf>@<offset>[<shape>;<strides>]:<dtype>; extents are expressions
// over the shape symbols with + - * // and parentheses, no spaces.
#include "plan.h"

#include <sstream>

namespace llc {

static std::string joinExprs(const std::vector<Expr>& v) {
  std::string o;
  for (size_t i = 0; i < v.size(); ++i) o += (i ? "," : "") + v[i].str();
  return o;
}

std::string View::str() const {
  return "b" + std::to_string(buf) + "@" + offset.str() + "[" + joinExprs(shape) + ";" + joinExprs(strides) + "]:" + dtypeName(dtype);
}

static const char* kindName(BufferDecl::Kind k) {
  switch (k) {
    case BufferDecl::Temp: return "temp"; case BufferDecl::Input: return "input";
    case BufferDecl::Output: return "output"; case BufferDecl::Weight: return "weight";
    default: return "const";
  }
}

std::string Plan::str() const {
  std::ostringstream o;
  o.precision(17);
  o << "llcplan 1\n";
  for (auto& kv : options) o << "option " << kv.first << " " << kv.second << "\n";
  o << "nsymargs " << numSymbolArgs << "\n";
  for (auto& s : symbols) {
    if (s.symbolArg >= 0) o << "symbol " << s.name << " arg " << s.symbolArg << "\n";
    else o << "symbol " << s.name << " input " << s.input << " " << s.dim << "\n";
  }
  for (size_t i = 0; i < buffers.size(); ++i) {
    auto& b = buffers[i];
    o << "buffer " << i << " " << dtypeName(b.dtype) << " " << kindName(b.kind) << " " << b.numel.str();
    if (b.index >= 0) o << " index=" << b.index;
    if (!b.file.empty()) o << " file=\"" << b.file << "\"";
    if (!b.values.empty()) { o << " values="; for (size_t k = 0; k < b.values.size(); ++k) o << (k ? "," : "") << b.values[k]; }
    o << "\n";
  }
  for (size_t i = 0; i < inputs.size(); ++i)
    o << "input " << i << " " << inputs[i].buf << " " << dtypeName(inputs[i].dtype) << " " << joinExprs(inputs[i].shape) << "\n";
  for (size_t i = 0; i < outputs.size(); ++i)
    o << "output " << i << " " << outputs[i].buf << " " << dtypeName(outputs[i].dtype) << " " << joinExprs(outputs[i].shape) << "\n";
  for (auto& s : steps) {
    o << (s.init ? "init " : "step ") << s.kernel;
    for (auto& v : s.views) o << " " << v.first << "=" << v.second.str();
    for (auto& p : s.params) o << " " << p.first << ":" << p.second;
    o << "\n";
  }
  return o.str();
}

// ---- parsing: expressions are re-read as opaque single-atom Exprs (their text) so that
// printing a parsed plan reproduces it; the executor evaluates the text with EvalExpr.
static Expr opaque(const std::string& text) {
  bool num = !text.empty();
  for (size_t i = 0; i < text.size(); ++i) if (!(std::isdigit((unsigned char)text[i]) || (i == 0 && text[i] == '-'))) num = false;
  if (num) return Expr(std::stoll(text));
  Expr e; e.terms[{text}] = 1; return e;
}
static std::vector<Expr> splitExprs(const std::string& s) {
  std::vector<Expr> out; std::string cur; int depth = 0;
  for (char c : s) {
    if (c == '(') ++depth; if (c == ')') --depth;
    if (c == ',' && depth == 0) { out.push_back(opaque(cur)); cur.clear(); } else cur += c;
  }
  if (!cur.empty()) out.push_back(opaque(cur));
  return out;
}
static View parseView(const std::string& t) {
  View v;
  size_t at = t.find('@'), lb = t.find('['), sc = t.find(';', lb), rb = t.find(']', sc), col = t.rfind(':');
  if (t[0] != 'b' || at == std::string::npos || lb == std::string::npos || sc == std::string::npos || rb == std::string::npos)
    throw std::runtime_error("bad view '" + t + "'");
  v.buf = std::stoi(t.substr(1, at - 1));
  v.offset = opaque(t.substr(at + 1, lb - at - 1));
  v.shape = splitExprs(t.substr(lb + 1, sc - lb - 1));
  v.strides = splitExprs(t.substr(sc + 1, rb - sc - 1));
  if (!dtypeFromName(t.substr(col + 1), v.dtype)) throw std::runtime_error("bad view dtype '" + t + "'");
  return v;
}

Plan parsePlan(const std::string& text) {
  Plan p;
  std::istringstream in(text);
  std::string line;
  bool header = false;
  while (std::getline(in, line)) {
    if (line.empty()) continue;
    std::istringstream ls(line);
    std::string kw; ls >> kw;
    if (kw == "llcplan") { header = true; continue; }
    if (!header) throw std::runtime_error("not a kernel plan (missing 'llcplan' header)");
    if (kw == "option") { std::string k, v; ls >> k; std::getline(ls, v); size_t b = v.find_first_not_of(' '); p.options[k] = b == std::string::npos ? "" : v.substr(b); }
    else if (kw == "nsymargs") ls >> p.numSymbolArgs;
    else if (kw == "symbol") {
      SymbolBinding s; std::string how; ls >> s.name >> how;
      if (how == "arg") ls >> s.symbolArg; else ls >> s.input >> s.dim;
      p.symbols.push_back(s);
    } else if (kw == "buffer") {
      size_t id; std::string dt, kind, numel; ls >> id >> dt >> kind >> numel;
      BufferDecl b;
      if (!dtypeFromName(dt, b.dtype)) throw std::runtime_error("bad buffer dtype " + dt);
      b.kind = kind == "temp" ? BufferDecl::Temp : kind == "input" ? BufferDecl::Input : kind == "output" ? BufferDecl::Output
             : kind == "weight" ? BufferDecl::Weight : BufferDecl::Const;
      b.numel = opaque(numel);
      std::string rest; std::getline(ls, rest);
      size_t f = rest.find("file=\"");
      if (f != std::string::npos) { size_t e = rest.find('"', f + 6); b.file = rest.substr(f + 6, e - f - 6); rest.erase(f, e - f + 1); }
      std::istringstream rs(rest); std::string tok;
      while (rs >> tok) {
        if (tok.compare(0, 6, "index=") == 0) b.index = std::stoi(tok.substr(6));
        else if (tok.compare(0, 7, "values=") == 0) { std::istringstream vs(tok.substr(7)); std::string x; while (std::getline(vs, x, ',')) b.values.push_back(std::stod(x)); }
      }
      if (id != p.buffers.size()) throw std::runtime_error("buffer ids must be dense and ordered");
      p.buffers.push_back(b);
    } else if (kw == "input" || kw == "output") {
      size_t k; IoDecl d; std::string dt, shape; ls >> k >> d.buf >> dt >> shape;
      if (!dtypeFromName(dt, d.dtype)) throw std::runtime_error("bad io dtype " + dt);
      d.shape = splitExprs(shape);
      (kw == "input" ? p.inputs : p.outputs).push_back(d);
    } else if (kw == "step" || kw == "init") {
      Step s; s.init = kw == "init"; ls >> s.kernel;
      std::string tok;
      while (ls >> tok) {
        size_t eq = tok.find('='), co = tok.find(':');
        if (eq != std::string::npos && (co == std::string::npos || eq < co) && eq + 1 < tok.size() && tok[eq + 1] == 'b' && tok.find('@') != std::string::npos)
          s.views.emplace_back(tok.substr(0, eq), parseView(tok.substr(eq + 1)));
        else if (co != std::string::npos) s.params.emplace_back(tok.substr(0, co), tok.substr(co + 1));
        else throw std::runtime_error("bad step token '" + tok + "'");
      }
      p.steps.push_back(s);
    } else throw std::runtime_error("unknown plan line '" + line + "'");
  }
  if (!header) throw std::runtime_error("not a kernel plan (empty)");
  return p;
}

}  // namespace llc

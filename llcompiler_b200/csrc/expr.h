// Symbolic integer expressions over shape symbols.
//
// The reference keeps symbolic dims as SymEngine expressions plus affine maps
// (src/Dialect/LLH/Utils/SymbolAnalysis.cpp:266-535).  SymEngine is not
// available, so this is a small canonical-polynomial replacement: an Expr is a
// sum of integer-coefficient monomials over atoms; an atom is a symbol name
// ("s0") or an opaque parenthesised floor division ("((s2+1)//2)").  The
// canonical form makes structural equality a map comparison, which is what the
// stride algebra and the broadcast checks need.  Exprs print to an infix text
// that the run-time evaluator (EvalExpr) parses again.
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>
#include <algorithm>
#include <cctype>

namespace llc {

struct Expr {
  // monomial (sorted atom names, repetition = power) -> coefficient
  std::map<std::vector<std::string>, int64_t> terms;

  Expr() {}
  Expr(int64_t c) { if (c) terms[{}] = c; }
  static Expr sym(const std::string& name) { Expr e; e.terms[{name}] = 1; return e; }

  bool isConst() const { return terms.empty() || (terms.size() == 1 && terms.begin()->first.empty()); }
  int64_t constant() const { return terms.empty() ? 0 : terms.begin()->second; }
  bool isConst(int64_t v) const { return isConst() && constant() == v; }
  bool operator==(const Expr& o) const { return terms == o.terms; }
  bool operator!=(const Expr& o) const { return !(terms == o.terms); }

  Expr operator+(const Expr& o) const {
    Expr r = *this;
    for (auto& t : o.terms) { if ((r.terms[t.first] += t.second) == 0) r.terms.erase(t.first); }
    return r;
  }
  Expr operator-() const { Expr r = *this; for (auto& t : r.terms) t.second = -t.second; return r; }
  Expr operator-(const Expr& o) const { return *this + (-o); }
  Expr operator*(const Expr& o) const {
    Expr r;
    for (auto& a : terms) for (auto& b : o.terms) {
      std::vector<std::string> m = a.first;
      m.insert(m.end(), b.first.begin(), b.first.end());
      std::sort(m.begin(), m.end());
      if ((r.terms[m] += a.second * b.second) == 0) r.terms.erase(m);
    }
    return r;
  }
  // floor division; exact when every coefficient divides, otherwise an opaque atom
  Expr floordiv(const Expr& d) const {
    if (d.isConst(1)) return *this;
    if (d.isConst() && d.constant() != 0) {
      int64_t c = d.constant();
      if (isConst()) { int64_t a = constant(); int64_t q = a / c; if ((a % c != 0) && ((a < 0) != (c < 0))) --q; return Expr(q); }
      bool all = true;
      for (auto& t : terms) if (t.second % c) all = false;
      if (all) { Expr r = *this; for (auto& t : r.terms) t.second /= c; return r; }
    }
    if (*this == d) return Expr(1);
    // single-monomial exact cancellation, e.g. (12*s0*s1) // (12*s0)
    if (terms.size() == 1 && d.terms.size() == 1) {
      auto num = *terms.begin(); auto den = *d.terms.begin();
      std::vector<std::string> rest = num.first; bool ok = den.second != 0 && num.second % den.second == 0;
      for (auto& a : den.first) {
        auto it = std::find(rest.begin(), rest.end(), a);
        if (it == rest.end()) { ok = false; break; }
        rest.erase(it);
      }
      if (ok) { Expr r; r.terms[rest] = num.second / den.second; return r; }
    }
    return Expr::sym("((" + str() + ")//(" + d.str() + "))");
  }
  Expr ceildiv(const Expr& d) const { return (*this + d - Expr(1)).floordiv(d); }

  std::string str() const {
    if (terms.empty()) return "0";
    std::string out;
    bool first = true;
    for (auto& t : terms) {
      int64_t c = t.second;
      if (!first) out += (c < 0 ? "-" : "+"); else if (c < 0) out += "-";
      first = false;
      int64_t a = c < 0 ? -c : c;
      if (t.first.empty()) { out += std::to_string(a); continue; }
      bool needMul = false;
      if (a != 1) { out += std::to_string(a); needMul = true; }
      for (auto& atom : t.first) { if (needMul) out += "*"; out += atom; needMul = true; }
    }
    return out;
  }
  void collectSymbols(std::vector<std::string>& out) const;
};

// ---- run-time evaluation of the printed form --------------------------------
struct EvalExpr {
  const std::string& s; size_t p = 0; const std::map<std::string, int64_t>& env;
  EvalExpr(const std::string& text, const std::map<std::string, int64_t>& e) : s(text), env(e) {}
  static int64_t eval(const std::string& text, const std::map<std::string, int64_t>& env) {
    EvalExpr ev(text, env); int64_t v = ev.expr();
    if (ev.p != text.size()) throw std::runtime_error("bad expression '" + text + "'");
    return v;
  }
  static int64_t fdiv(int64_t a, int64_t b) {
    if (b == 0) throw std::runtime_error("division by zero in shape expression");
    int64_t q = a / b; if ((a % b != 0) && ((a < 0) != (b < 0))) --q; return q;
  }
  int64_t expr() {
    int64_t v = term();
    while (p < s.size() && (s[p] == '+' || s[p] == '-')) { char c = s[p++]; int64_t t = term(); v = c == '+' ? v + t : v - t; }
    return v;
  }
  int64_t term() {
    int64_t v = unary();
    while (p < s.size()) {
      if (s[p] == '*') { ++p; v *= unary(); }
      else if (s[p] == '/' && p + 1 < s.size() && s[p + 1] == '/') { p += 2; v = fdiv(v, unary()); }
      else break;
    }
    return v;
  }
  int64_t unary() { if (p < s.size() && s[p] == '-') { ++p; return -unary(); } return primary(); }
  int64_t primary() {
    if (p >= s.size()) throw std::runtime_error("truncated expression '" + s + "'");
    if (s[p] == '(') { ++p; int64_t v = expr(); if (p >= s.size() || s[p] != ')') throw std::runtime_error("missing ) in '" + s + "'"); ++p; return v; }
    if (std::isdigit((unsigned char)s[p])) { int64_t v = 0; while (p < s.size() && std::isdigit((unsigned char)s[p])) v = v * 10 + (s[p++] - '0'); return v; }
    size_t b = p;
    while (p < s.size() && (std::isalnum((unsigned char)s[p]) || s[p] == '_')) ++p;
    std::string name = s.substr(b, p - b);
    auto it = env.find(name);
    if (it == env.end()) throw std::runtime_error("unbound shape symbol '" + name + "'");
    return it->second;
  }
};

inline void Expr::collectSymbols(std::vector<std::string>& out) const {
  std::string text = str();
  size_t p = 0;
  while (p < text.size()) {
    if (std::isalpha((unsigned char)text[p]) || text[p] == '_') {
      size_t b = p; while (p < text.size() && (std::isalnum((unsigned char)text[p]) || text[p] == '_')) ++p;
      std::string n = text.substr(b, p - b);
      if (std::find(out.begin(), out.end(), n) == out.end()) out.push_back(n);
    } else ++p;
  }
}

}  // namespace llc

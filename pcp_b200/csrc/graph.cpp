// General StableHLO front end, host side: text -> tensor program, gradient program, dump.  See graph.h.
#include "graph.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <map>

namespace pcpb {

namespace {

// element-type codes and sizes as in common.cuh (a CUDA header; this file is plain C++)
enum : int { DT_F32 = 0, DT_F64 = 1, DT_BF16 = 3, DT_I32 = 4, DT_I64 = 5, DT_BOOL = 6 };
size_t dtype_size(int dt) { return (dt == DT_F64 || dt == DT_I64) ? 8 : (dt == DT_F32 || dt == DT_I32) ? 4 : dt == DT_BF16 ? 2 : 1; }

// ------------------------------------------------------------------------------------------------
// text helpers
// ------------------------------------------------------------------------------------------------
bool ident_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '.'; }

std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && isspace((unsigned char)s[a])) ++a;
  while (b > a && isspace((unsigned char)s[b - 1])) --b;
  return s.substr(a, b - a);
}

int dtype_of(const std::string& e) {
  if (e == "f32") return DT_F32;
  if (e == "f64") return DT_F64;
  if (e == "bf16") return DT_BF16;
  if (e == "i64") return DT_I64;
  if (e == "i32") return DT_I32;
  if (e == "i1") return DT_BOOL;
  return -1;
}

const char* dtype_name(int dt) {
  switch (dt) {
    case DT_F32: return "f32";
    case DT_F64: return "f64";
    case DT_BF16: return "bf16";
    case DT_I64: return "i64";
    case DT_I32: return "i32";
    case DT_BOOL: return "i1";
  }
  return "?";
}

bool is_float(int dt) { return dt == DT_F32 || dt == DT_F64 || dt == DT_BF16; }

// "tensor<64x32xf32>" (text between the angle brackets given) -> shape, dtype
bool parse_tensor_body(const std::string& body, std::vector<int64_t>* shape, int* dt) {
  shape->clear();
  size_t pos = 0;
  while (true) {
    size_t x = body.find('x', pos);
    if (x == std::string::npos) break;
    const std::string tok = body.substr(pos, x - pos);
    if (tok.empty() || tok.find_first_not_of("0123456789") != std::string::npos) break;
    shape->push_back(strtoll(tok.c_str(), nullptr, 10));
    pos = x + 1;
  }
  *dt = dtype_of(body.substr(pos));
  return *dt >= 0;
}

// every tensor<...> in s, in order
bool all_types(const std::string& s, std::vector<std::vector<int64_t>>* shapes, std::vector<int>* dts) {
  size_t p = 0;
  while ((p = s.find("tensor<", p)) != std::string::npos) {
    const size_t e = s.find('>', p);
    if (e == std::string::npos) return false;
    std::vector<int64_t> sh;
    int dt;
    if (!parse_tensor_body(s.substr(p + 7, e - p - 7), &sh, &dt)) return false;
    shapes->push_back(sh);
    dts->push_back(dt);
    p = e + 1;
  }
  return true;
}

// every %name in s, in order
std::vector<std::string> ssa_names(const std::string& s) {
  std::vector<std::string> r;
  for (size_t p = s.find('%'); p != std::string::npos; p = s.find('%', p + 1)) {
    size_t e = p + 1;
    while (e < s.size() && ident_char(s[e])) ++e;
    if (e > p + 1) r.push_back(s.substr(p + 1, e - p - 1));
  }
  return r;
}

// the integers of "key = [1, 2]" / "key = array<i64: 1, 2>" after position `at`; false when the key is absent
bool int_list_after(const std::string& s, const std::string& key, std::vector<int64_t>* out, char open = '[', char close = ']') {
  out->clear();
  size_t p = 0;
  while (true) {
    p = s.find(key, p);
    if (p == std::string::npos) return false;
    if ((p == 0 || !ident_char(s[p - 1])) && (p + key.size() >= s.size() || !ident_char(s[p + key.size()]))) break;   // whole word
    p += key.size();
  }
  p = s.find(open, p);
  if (p == std::string::npos) return false;
  const size_t e = s.find(close, p);
  if (e == std::string::npos) return false;
  std::string body = s.substr(p + 1, e - p - 1);
  const size_t colon = body.find(':');
  if (open == '<' && colon != std::string::npos) body = body.substr(colon + 1);
  const char* c = body.c_str();
  while (*c) {
    while (*c && !(isdigit((unsigned char)*c) || *c == '-')) ++c;
    if (!*c) break;
    char* end;
    out->push_back(strtoll(c, &end, 10));
    c = end;
  }
  return true;
}

// the integer of "key = 3" (key as a whole word); false when absent
bool int_after(const std::string& s, const std::string& key, int64_t* out) {
  size_t p = 0;
  while (true) {
    p = s.find(key, p);
    if (p == std::string::npos) return false;
    const size_t e = p + key.size();
    if ((p == 0 || !ident_char(s[p - 1])) && (e >= s.size() || !ident_char(s[e]))) { p = e; break; }
    p = e;
  }
  while (p < s.size() && isspace((unsigned char)s[p])) ++p;
  if (p >= s.size() || s[p] != '=') return false;
  ++p;
  char* end;
  const long long v = strtoll(s.c_str() + p, &end, 10);
  if (end == s.c_str() + p) return false;
  *out = v;
  return true;
}

int64_t numel_of(const std::vector<int64_t>& s) {
  int64_t n = 1;
  for (int64_t x : s) n *= x;
  return n;
}

int hexval(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  return -1;
}

bool hex_bytes(const char* s, size_t n, std::vector<uint8_t>* out) {
  if (n % 2) return false;
  out->resize(n / 2);
  for (size_t i = 0; i < n / 2; ++i) {
    const int h = hexval(s[2 * i]), l = hexval(s[2 * i + 1]);
    if (h < 0 || l < 0) return false;
    (*out)[i] = (uint8_t)(h * 16 + l);
  }
  return true;
}

uint16_t bf16_bits_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// one scalar literal of element type dt -> its bytes appended to out
// bf16_model: the reference rewrites 32-bit hex float literals of bf16 models before compiling
// (src/compiler/sanitizer.zig:129-244): 0xFF800000 (-inf) becomes -65504, other finite values their "%.6e" decimal.
bool append_literal(const std::string& tok_in, int dt, bool bf16_model, std::vector<uint8_t>* out, double* fval, long long* ival) {
  const std::string tok = trim(tok_in);
  double f = 0.0;
  long long i = 0;
  bool from_bits = false;
  if (bf16_model && tok.size() == 10 && tok.compare(0, 2, "0x") == 0 && tok.find_first_not_of("0123456789abcdefABCDEF", 2) == std::string::npos &&
      is_float(dt)) {
    const uint32_t u = (uint32_t)strtoull(tok.c_str() + 2, nullptr, 16);
    float x;
    memcpy(&x, &u, 4);
    if (u == 0xFF800000u) f = -65504.0;
    else if (isfinite(x)) { char b[64]; snprintf(b, sizeof b, "%.6e", (double)x); f = strtod(b, nullptr); }
    else f = x;
  }
  else if (tok == "true" || tok == "false") { i = tok == "true"; f = (double)i; }
  else if (tok.size() > 2 && (tok.compare(0, 2, "0x") == 0 || tok.compare(0, 2, "0X") == 0)) {
    unsigned long long bits = strtoull(tok.c_str() + 2, nullptr, 16);
    from_bits = true;
    if (dt == DT_F32) { uint32_t u = (uint32_t)bits; float x; memcpy(&x, &u, 4); f = x; }
    else if (dt == DT_BF16) { if (bits > 0xFFFFull) bits >>= 16; uint32_t u = (uint32_t)bits << 16; float x; memcpy(&x, &u, 4); f = x; }
    else if (dt == DT_F64) { memcpy(&f, &bits, 8); }
    else { i = (long long)bits; f = (double)i; from_bits = false; }
  } else if (is_float(dt)) {
    if (tok == "inf" || tok == "+inf") f = INFINITY; else if (tok == "-inf") f = -INFINITY; else if (tok == "nan") f = NAN;
    else { char* end; f = strtod(tok.c_str(), &end); if (end == tok.c_str()) return false; }
  } else {
    char* end;
    if (tok.find_first_of(".eE") != std::string::npos) { f = strtod(tok.c_str(), &end); i = (long long)f; }
    else { i = strtoll(tok.c_str(), &end, 10); f = (double)i; }
    if (end == tok.c_str()) return false;
  }
  (void)from_bits;
  if (fval) *fval = f;
  if (ival) *ival = is_float(dt) ? (long long)0 : i;
  if (out) {
    uint8_t buf[8];
    size_t n = 0;
    switch (dt) {
      case DT_F32: { float x = (float)f; memcpy(buf, &x, 4); n = 4; break; }
      case DT_F64: { memcpy(buf, &f, 8); n = 8; break; }
      case DT_BF16: { uint16_t x = bf16_bits_rne((float)f); memcpy(buf, &x, 2); n = 2; break; }
      case DT_I64: { memcpy(buf, &i, 8); n = 8; break; }
      case DT_I32: { int32_t x = (int32_t)i; memcpy(buf, &x, 4); n = 4; break; }
      case DT_BOOL: { buf[0] = i != 0; n = 1; break; }
      default: return false;
    }
    out->insert(out->end(), buf, buf + n);
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
// program construction
// ------------------------------------------------------------------------------------------------
struct Builder {
  Graph* g;
  std::string err;

  int value(const std::vector<int64_t>& shape, int dt, const std::string& name = "") {
    GValue v;
    v.shape = shape; v.dt = dt; v.numel = numel_of(shape); v.name = name;
    g->vals.push_back(v);
    return (int)g->vals.size() - 1;
  }
  int emit(GOp op, const std::vector<int64_t>& shape, int dt, const std::string& name = "") {
    op.out = value(shape, dt, name);
    g->vals[op.out].op = (int)g->ops.size();
    g->ops.push_back(op);
    return op.out;
  }
  const GValue& V(int v) const { return g->vals[v]; }

  int splat(const std::vector<int64_t>& shape, int dt, double f) {
    GOp op; op.kind = G_CONST_SPLAT; op.fval = f; op.ival = isfinite(f) ? (long long)f : 0;
    return emit(op, shape, dt);
  }
  int zeros_like(int v) { return splat(V(v).shape, V(v).dt, 0.0); }
  int unary(int sub, int x) { GOp op; op.kind = G_UNARY; op.sub = sub; op.in = {x}; return emit(op, V(x).shape, V(x).dt); }
  int binary(int sub, int a, int b) {
    if (V(a).shape != V(b).shape || V(a).dt != V(b).dt) { if (err.empty()) err = "gradient rule: operands of different types"; }
    GOp op; op.kind = G_BINARY; op.sub = sub; op.in = {a, b};
    return emit(op, V(a).shape, V(a).dt);
  }
  int compare(int dir, int a, int b) { GOp op; op.kind = G_COMPARE; op.sub = dir; op.in = {a, b}; return emit(op, V(a).shape, DT_BOOL); }
  int select(int p, int a, int b) { GOp op; op.kind = G_SELECT; op.in = {p, a, b}; return emit(op, V(a).shape, V(a).dt); }
  int convert(int x, int dt) { if (V(x).dt == dt) return x; GOp op; op.kind = G_CONVERT; op.in = {x}; return emit(op, V(x).shape, dt); }
  int reshape(int x, const std::vector<int64_t>& shape) {
    if (V(x).shape == shape) return x;
    if (numel_of(shape) != V(x).numel) { if (err.empty()) err = "gradient rule: reshape changes the element count"; return x; }
    GOp op; op.kind = G_RESHAPE; op.in = {x};
    return emit(op, shape, V(x).dt);
  }
  int transpose(int x, const std::vector<int64_t>& perm) {
    std::vector<int64_t> shape(perm.size());
    for (size_t k = 0; k < perm.size(); ++k) shape[k] = V(x).shape[perm[k]];
    GOp op; op.kind = G_TRANSPOSE; op.in = {x}; op.a = perm;
    return emit(op, shape, V(x).dt);
  }
  int bcast(int x, const std::vector<int64_t>& dims, const std::vector<int64_t>& shape) {
    GOp op; op.kind = G_BCAST; op.in = {x}; op.a = dims;
    return emit(op, shape, V(x).dt);
  }
  int reduce(int kind, int x, const std::vector<int64_t>& dims) {
    if (dims.empty()) return x;
    std::vector<int64_t> shape;
    for (size_t i = 0; i < V(x).shape.size(); ++i) {
      bool red = false;
      for (int64_t d : dims) red |= (d == (int64_t)i);
      if (!red) shape.push_back(V(x).shape[i]);
    }
    const int init = splat({}, V(x).dt, kind == R_MAX ? -INFINITY : 0.0);
    GOp op; op.kind = G_REDUCE; op.sub = kind; op.in = {x, init}; op.a = dims;
    return emit(op, shape, V(x).dt);
  }
  int slice(int x, const std::vector<int64_t>& a, const std::vector<int64_t>& b, const std::vector<int64_t>& c) {
    std::vector<int64_t> shape(a.size());
    for (size_t i = 0; i < a.size(); ++i) shape[i] = (b[i] - a[i] + c[i] - 1) / c[i];
    GOp op; op.kind = G_SLICE; op.in = {x}; op.a = a; op.b = b; op.c = c;
    return emit(op, shape, V(x).dt);
  }
  // result dims: batch (lhs order), lhs free, rhs free
  int dot(int x, int y, const std::vector<int64_t>& lb, const std::vector<int64_t>& rb, const std::vector<int64_t>& lc,
          const std::vector<int64_t>& rc) {
    auto in = [](const std::vector<int64_t>& v, int64_t i) { for (int64_t e : v) if (e == i) return true; return false; };
    std::vector<int64_t> shape;
    for (int64_t i : lb) shape.push_back(V(x).shape[i]);
    for (size_t i = 0; i < V(x).shape.size(); ++i) if (!in(lb, i) && !in(lc, i)) shape.push_back(V(x).shape[i]);
    for (size_t i = 0; i < V(y).shape.size(); ++i) if (!in(rb, i) && !in(rc, i)) shape.push_back(V(y).shape[i]);
    for (size_t i = 0; i < lc.size(); ++i)
      if (V(x).shape[lc[i]] != V(y).shape[rc[i]]) { if (err.empty()) err = "dot_general: contracting sizes differ"; }
    GOp op; op.kind = G_DOT; op.in = {x, y}; op.a = lb; op.b = rb; op.c = lc; op.d = rc;
    return emit(op, shape, V(x).dt);
  }
};

}  // namespace

// ------------------------------------------------------------------------------------------------
// parser
// ------------------------------------------------------------------------------------------------
std::string graph_parse(const char* text, size_t n, bool sanitize, Graph* g) {
  *g = Graph();
  Builder bld{g, ""};
  const std::string all(text, n);
  // resources: name: "0x<hex>" inside {-# ... #-}; the first four bytes of a blob are its alignment header
  std::map<std::string, std::vector<uint8_t>> resources;
  size_t res_at = all.find("{-#");
  if (res_at != std::string::npos) {
    size_t p = res_at;
    while ((p = all.find("\"0x", p)) != std::string::npos) {
      const size_t e = all.find('"', p + 1);
      if (e == std::string::npos) break;
      size_t k = p;                                  // the key: identifier before the ':' preceding the string
      while (k > res_at && all[k] != ':') --k;
      size_t ke = k;
      while (ke > res_at && isspace((unsigned char)all[ke - 1])) --ke;
      size_t ks = ke;
      while (ks > res_at && ident_char(all[ks - 1])) --ks;
      std::vector<uint8_t> raw;
      if (!hex_bytes(all.c_str() + p + 3, e - p - 3, &raw) || raw.size() < 4) return "malformed resource blob";
      resources[all.substr(ks, ke - ks)] = std::vector<uint8_t>(raw.begin() + 4, raw.end());
      p = e + 1;
    }
  }
  const std::string body = res_at == std::string::npos ? all : all.substr(0, res_at);
  // the @main header
  size_t h = body.find("@main(");
  if (h == std::string::npos) return "function @main not found";
  size_t line_end = body.find('\n', h);
  if (line_end == std::string::npos) line_end = body.size();
  const std::string header = body.substr(h, line_end - h);
  const size_t arrow = header.rfind("->");
  if (arrow == std::string::npos) return "@main has no result type";
  std::map<std::string, int> env;
  {
    const std::string sig = header.substr(0, arrow);
    size_t p = 0;
    while ((p = sig.find('%', p)) != std::string::npos) {
      size_t e = p + 1;
      while (e < sig.size() && ident_char(sig[e])) ++e;
      const std::string name = sig.substr(p + 1, e - p - 1);
      const size_t t = sig.find("tensor<", e), te = sig.find('>', t);
      if (t == std::string::npos || te == std::string::npos) return "argument %" + name + " has no tensor type";
      std::vector<int64_t> sh;
      int dt;
      if (!parse_tensor_body(sig.substr(t + 7, te - t - 7), &sh, &dt)) return "argument %" + name + ": unsupported element type";
      const int v = bld.value(sh, dt, name);
      g->args.push_back(v);
      env[name] = v;
      p = te;
    }
  }
  const bool bf16_model = !g->args.empty() && g->vals[g->args[0]].dt == DT_BF16;
  // ops, one per line
  size_t pos = line_end + 1;
  bool returned = false;
  while (pos < body.size() && !returned) {
    size_t e = body.find('\n', pos);
    if (e == std::string::npos) e = body.size();
    const std::string s = trim(body.substr(pos, e - pos));
    pos = e + 1;
    if (s.empty() || s.compare(0, 2, "//") == 0) continue;
    if (s.compare(0, 6, "return") == 0 || s.compare(0, 11, "func.return") == 0) {
      const std::vector<std::string> names = ssa_names(s);
      if (names.size() != 1 || !env.count(names[0])) return "@main must return one value";
      g->ret = env[names[0]];
      returned = true;
      break;
    }
    if (s == "}") break;
    if (s[0] != '%') return "cannot parse line: " + s.substr(0, 80);
    const size_t eq = s.find('=');
    if (eq == std::string::npos) return "cannot parse line: " + s.substr(0, 80);
    const std::string res = trim(s.substr(1, eq - 1));
    if (res.find(':') != std::string::npos) return "ops with several results are not supported: " + s.substr(0, 80);
    const std::string rest = trim(s.substr(eq + 1));
    const size_t colon = rest.rfind(" : ");
    if (colon == std::string::npos) return "op without a type: " + s.substr(0, 80);
    const std::string head = rest.substr(0, colon), tail = rest.substr(colon + 3);
    std::vector<std::vector<int64_t>> tshapes;
    std::vector<int> tdts;
    if (!all_types(tail, &tshapes, &tdts) || tshapes.empty()) return "unsupported type in: " + s.substr(0, 120);
    const std::vector<int64_t> oshape = tshapes.back();
    const int odt = tdts.back();
    std::string name, after;
    if (head.empty()) return "op without a name: " + s.substr(0, 80);
    for (const auto& sh : tshapes) {
      int64_t nel = 1;
      for (int64_t dsz : sh) { if (dsz < 0 || (dsz > 0 && nel > ((int64_t)1 << 40) / dsz)) return "tensor too large: " + s.substr(0, 80); nel *= dsz; }
      if (sh.size() > 8) return "tensor rank above 8: " + s.substr(0, 80);
    }
    if (head[0] == '"') {
      const size_t q = head.find('"', 1);
      if (q == std::string::npos) return "cannot parse line: " + s.substr(0, 80);
      name = head.substr(1, q - 1);
      after = head.substr(q + 1);
    } else {
      size_t q = 0;
      while (q < head.size() && ident_char(head[q])) ++q;
      name = head.substr(0, q);
      after = head.substr(q);
    }
    GOp op;
    if (name == "stablehlo.constant" || name == "arith.constant") {
      const std::string v = trim(after);
      if (v.empty()) return "constant without a value: %" + res;
      if (v.compare(0, 15, "dense_resource<") == 0) {
        const std::string key = v.substr(15, v.find('>') - 15);
        if (!resources.count(key)) return "constant refers to an unknown resource: " + key;
        op.kind = G_CONST_DATA; op.data = resources[key];
      } else if (v.compare(0, 6, "dense<") == 0 && v.back() == '>') {
        const std::string lit = trim(v.substr(6, v.size() - 7));
        if (lit.size() > 3 && lit.compare(0, 3, "\"0x") == 0) {
          op.kind = G_CONST_DATA;
          if (!hex_bytes(lit.c_str() + 3, lit.size() - 4, &op.data)) return "malformed hex constant";
        } else if (!lit.empty() && lit[0] == '[') {
          op.kind = G_CONST_DATA;
          std::string tok;
          for (char ch : lit + ",") {
            if (ch == '[' || ch == ']' || ch == ',' || isspace((unsigned char)ch)) {
              if (!tok.empty()) { if (!append_literal(tok, odt, bf16_model, &op.data, nullptr, nullptr)) return "bad literal: " + tok; tok.clear(); }
            } else tok.push_back(ch);
          }
        } else {
          op.kind = G_CONST_SPLAT;
          if (!append_literal(lit, odt, bf16_model, nullptr, &op.fval, &op.ival)) return "bad literal: " + lit;
        }
      } else return "unsupported constant: " + v.substr(0, 60);
      if (op.kind == G_CONST_DATA && (int64_t)op.data.size() != numel_of(oshape) * (int64_t)dtype_size(odt))
        return "constant payload has the wrong size: %" + res;
      env[res] = bld.emit(op, oshape, odt, res);
      continue;
    }
    // operands
    std::string operand_text = after;
    if (head[0] == '"') operand_text = after.substr(0, after.find(')') + 1);
    std::vector<int> in;
    for (const std::string& o : ssa_names(operand_text)) {
      if (!env.count(o)) return "use of an undefined value %" + o;
      in.push_back(env[o]);
    }
    op.in = in;
    auto need = [&](size_t k) { return in.size() == k; };
    static const std::map<std::string, int> unary = {
        {"stablehlo.rsqrt", U_RSQRT}, {"stablehlo.sqrt", U_SQRT}, {"stablehlo.exponential", U_EXP}, {"stablehlo.log", U_LOG},
        {"stablehlo.tanh", U_TANH}, {"stablehlo.logistic", U_LOGISTIC}, {"stablehlo.negate", U_NEG}, {"stablehlo.ceil", U_CEIL},
        {"stablehlo.floor", U_FLOOR}, {"stablehlo.sine", U_SIN}, {"stablehlo.cosine", U_COS}, {"stablehlo.abs", U_ABS}};
    static const std::map<std::string, int> binary = {
        {"stablehlo.add", B_ADD}, {"stablehlo.subtract", B_SUB}, {"stablehlo.multiply", B_MUL}, {"stablehlo.divide", B_DIV},
        {"stablehlo.power", B_POW}, {"stablehlo.maximum", B_MAX}, {"stablehlo.minimum", B_MIN}, {"stablehlo.and", B_AND},
        {"stablehlo.or", B_OR}};
    if (unary.count(name)) {
      if (!need(1)) return name + ": one operand expected";
      op.kind = G_UNARY; op.sub = unary.at(name);
    } else if (binary.count(name)) {
      if (!need(2)) return name + ": two operands expected";
      if (bld.V(in[0]).shape != bld.V(in[1]).shape || bld.V(in[0]).dt != bld.V(in[1]).dt) return name + ": operand types differ (%" + res + ")";
      op.kind = G_BINARY; op.sub = binary.at(name);
    } else if (name == "stablehlo.compare") {
      if (!need(2)) return "compare: two operands expected";
      static const std::map<std::string, int> dirs = {{"EQ", C_EQ}, {"NE", C_NE}, {"GE", C_GE}, {"GT", C_GT}, {"LE", C_LE}, {"LT", C_LT}};
      const std::string d = trim(after).substr(0, 2);
      if (!dirs.count(d)) return "compare: unknown direction " + d;
      op.kind = G_COMPARE; op.sub = dirs.at(d);
    } else if (name == "stablehlo.select") {
      if (!need(3)) return "select: three operands expected";
      op.kind = G_SELECT;
    } else if (name == "stablehlo.convert") {
      if (!need(1)) return "convert: one operand expected";
      op.kind = G_CONVERT;
    } else if (name == "stablehlo.reshape") {
      if (!need(1) || bld.V(in[0]).numel != numel_of(oshape)) return "reshape changes the element count (%" + res + ")";
      op.kind = G_RESHAPE;
    } else if (name == "stablehlo.transpose") {
      if (!need(1) || !int_list_after(after, "dims", &op.a) || op.a.size() != bld.V(in[0]).shape.size()) return "transpose: bad dims (%" + res + ")";
      op.kind = G_TRANSPOSE;
    } else if (name == "stablehlo.broadcast_in_dim") {
      if (!need(1) || !int_list_after(after, "dims", &op.a) || op.a.size() != bld.V(in[0]).shape.size()) return "broadcast_in_dim: bad dims (%" + res + ")";
      op.kind = G_BCAST;
    } else if (name == "stablehlo.slice") {
      if (!need(1)) return "slice: one operand expected";
      const size_t lb = after.find('['), rb = after.find(']');
      if (lb == std::string::npos || rb == std::string::npos) return "slice: no ranges";
      std::string ranges = after.substr(lb + 1, rb - lb - 1) + ",";
      std::string part;
      for (char ch : ranges) {
        if (ch == ',') {
          long long a = 0, b = 0, c = 1;
          const int k = sscanf(part.c_str(), " %lld : %lld : %lld", &a, &b, &c);
          if (k < 2) return "slice: bad range " + part;
          if (k < 3) c = 1;
          op.a.push_back(a); op.b.push_back(b); op.c.push_back(c);
          part.clear();
        } else part.push_back(ch);
      }
      if (op.a.size() != bld.V(in[0]).shape.size()) return "slice: rank mismatch";
      op.kind = G_SLICE;
    } else if (name == "stablehlo.concatenate") {
      int64_t dim;
      if (in.empty() || !int_after(after, "dim", &dim)) return "concatenate: bad dim";
      op.a = {dim};
      op.kind = G_CONCAT;
    } else if (name == "stablehlo.iota" || name == "stablehlo.dynamic_iota") {
      int64_t dim;
      if (!int_after(after, "dim", &dim)) return "iota: bad dim";
      op.a = {dim};
      op.in.clear();
      op.kind = G_IOTA;
    } else if (name == "stablehlo.reduce") {
      if (!need(2)) return "reduce: operand and init expected";
      if (after.find("stablehlo.add") != std::string::npos) op.sub = R_ADD;
      else if (after.find("stablehlo.maximum") != std::string::npos) op.sub = R_MAX;
      else return "reduce: only add and maximum are supported (%" + res + ")";
      if (!int_list_after(after, "dimensions", &op.a)) return "reduce: no dimensions";
      op.kind = G_REDUCE;
    } else if (name == "stablehlo.dot_general") {
      if (!need(2)) return "dot_general: two operands expected";
      const size_t bd = after.find("batching_dims"), cd = after.find("contracting_dims");
      auto two_lists = [&](size_t at, std::vector<int64_t>* l, std::vector<int64_t>* r) {
        const std::string t = after.substr(at);
        if (!int_list_after(t, "dims", l)) return false;
        const size_t x = t.find(" x ");
        return x != std::string::npos && int_list_after("k " + t.substr(x + 3), "k", r);
      };
      if (bd != std::string::npos && !two_lists(bd + 9, &op.a, &op.b)) return "dot_general: bad batching dims";
      if (cd == std::string::npos || !two_lists(cd + 12, &op.c, &op.d)) return "dot_general: bad contracting dims";
      op.kind = G_DOT;
    } else if (name == "stablehlo.gather") {
      if (!need(2)) return "gather: two operands expected";
      std::vector<int64_t> collapsed, sim, ivd(1, 0), sizes;
      int_list_after(after, "collapsed_slice_dims", &collapsed);
      int_list_after(after, "start_index_map", &sim);
      if (!int_after(after, "index_vector_dim", &ivd[0])) return "gather: no index_vector_dim";
      int_list_after(after, "slice_sizes", &sizes, '<', '>');
      const GValue &x = bld.V(in[0]), &idx = bld.V(in[1]);
      if (idx.dt != DT_I64) return "gather: indices must be i64";
      if (collapsed == std::vector<int64_t>{0} && sim == std::vector<int64_t>{0}) {
        int64_t rows = idx.numel;
        if (ivd[0] < (int64_t)idx.shape.size()) { if (idx.shape[ivd[0]] != 1) return "gather: index vector longer than 1"; }
        if (x.shape.empty() || sizes.size() != x.shape.size() || sizes[0] != 1) return "gather: unsupported slice sizes";
        for (size_t i = 1; i < sizes.size(); ++i) if (sizes[i] != x.shape[i]) return "gather: only whole rows are supported";
        if (rows * (x.numel / x.shape[0]) != numel_of(oshape)) return "gather: result shape mismatch";
        op.kind = G_GATHER_ROWS;
      } else if (collapsed == std::vector<int64_t>{0, 1} && sim == std::vector<int64_t>{0, 1}) {
        if (x.shape.size() != 2 || idx.shape.empty() || ivd[0] != (int64_t)idx.shape.size() - 1 || idx.shape.back() != 2 ||
            idx.numel / 2 != numel_of(oshape))
          return "gather: unsupported two-index form";
        op.kind = G_GATHER2;
      } else return "gather: unsupported dimension numbers (%" + res + ")";
    } else {
      return "unsupported op " + name;
    }
    // attribute checks: everything that later code indexes with must be in range
    {
      auto in_range = [](const std::vector<int64_t>& v, int64_t n) { for (int64_t x : v) if (x < 0 || x >= n) return false; return true; };
      auto distinct = [](std::vector<int64_t> v) { std::sort(v.begin(), v.end()); return std::adjacent_find(v.begin(), v.end()) == v.end(); };
      const int64_t orank = (int64_t)oshape.size();
      const int64_t irank = in.empty() ? 0 : (int64_t)bld.V(in[0]).shape.size();
      switch (op.kind) {
        case G_TRANSPOSE:
          if (!in_range(op.a, irank) || !distinct(op.a) || orank != irank) return "transpose: not a permutation (%" + res + ")";
          for (int64_t k = 0; k < orank; ++k) if (oshape[k] != bld.V(in[0]).shape[op.a[k]]) return "transpose: result shape mismatch (%" + res + ")";
          break;
        case G_BCAST:
          if (!in_range(op.a, orank) || !distinct(op.a)) return "broadcast_in_dim: dims out of range (%" + res + ")";
          for (size_t k = 0; k < op.a.size(); ++k) {
            const int64_t sz = bld.V(in[0]).shape[k];
            if (sz != 1 && sz != oshape[op.a[k]]) return "broadcast_in_dim: operand does not fit the result (%" + res + ")";
          }
          break;
        case G_REDUCE: {
          if (!in_range(op.a, irank) || !distinct(op.a)) return "reduce: dimensions out of range (%" + res + ")";
          std::vector<int64_t> kept;
          for (int64_t k = 0; k < irank; ++k) if (std::find(op.a.begin(), op.a.end(), k) == op.a.end()) kept.push_back(bld.V(in[0]).shape[k]);
          if (kept != oshape || bld.V(in[1]).numel != 1) return "reduce: result shape mismatch (%" + res + ")";
          break;
        }
        case G_CONCAT: {
          if (!in_range(op.a, orank)) return "concatenate: dimension out of range (%" + res + ")";
          int64_t total = 0;
          for (int v : in) {
            const GValue& x = bld.V(v);
            if ((int64_t)x.shape.size() != orank || x.dt != odt) return "concatenate: operand types differ (%" + res + ")";
            for (int64_t k = 0; k < orank; ++k) if (k != op.a[0] && x.shape[k] != oshape[k]) return "concatenate: operand shapes differ (%" + res + ")";
            total += x.shape[op.a[0]];
          }
          if (total != oshape[op.a[0]]) return "concatenate: sizes do not add up (%" + res + ")";
          break;
        }
        case G_IOTA:
          if (!in_range(op.a, orank)) return "iota: dimension out of range (%" + res + ")";
          break;
        case G_SLICE:
          if (orank != irank) return "slice: rank mismatch (%" + res + ")";
          for (int64_t k = 0; k < irank; ++k)
            if (op.c[k] < 1 || op.a[k] < 0 || op.b[k] < op.a[k] || op.b[k] > bld.V(in[0]).shape[k] ||
                (op.b[k] - op.a[k] + op.c[k] - 1) / op.c[k] != oshape[k])
              return "slice: bad range (%" + res + ")";
          break;
        case G_DOT: {
          const int64_t rrank = (int64_t)bld.V(in[1]).shape.size();
          std::vector<int64_t> l = op.a, r = op.b;
          l.insert(l.end(), op.c.begin(), op.c.end());
          r.insert(r.end(), op.d.begin(), op.d.end());
          if (op.a.size() != op.b.size() || op.c.size() != op.d.size() || !in_range(l, irank) || !in_range(r, rrank) || !distinct(l) || !distinct(r))
            return "dot_general: dimension numbers out of range (%" + res + ")";
          for (size_t k = 0; k < op.a.size(); ++k)
            if (bld.V(in[0]).shape[op.a[k]] != bld.V(in[1]).shape[op.b[k]]) return "dot_general: batch sizes differ (%" + res + ")";
          break;
        }
        case G_SELECT:
          if (bld.V(in[0]).dt != 6 /* i1 */ || bld.V(in[0]).shape != oshape || bld.V(in[1]).shape != oshape || bld.V(in[1]).dt != odt)
            return "select: operand types (%" + res + ")";
          break;
        case G_COMPARE:
          if (bld.V(in[0]).shape != bld.V(in[1]).shape || bld.V(in[0]).dt != bld.V(in[1]).dt || bld.V(in[0]).shape != oshape || odt != 6)
            return "compare: operand types (%" + res + ")";
          break;
        case G_CONVERT:
          if (bld.V(in[0]).shape != oshape) return "convert changes the shape (%" + res + ")";
          break;
        default: break;
      }
    }
    if (op.kind == G_DOT) {
      const int v = bld.dot(in[0], in[1], op.a, op.b, op.c, op.d);
      if (!bld.err.empty()) return bld.err + " (%" + res + ")";
      if (g->vals[v].numel != numel_of(oshape) || g->vals[v].dt != odt) return "dot_general: result type mismatch (%" + res + ")";
      g->vals[v].shape = oshape; g->vals[v].name = res;
      env[res] = v;
      continue;
    }
    if (op.kind == G_UNARY || op.kind == G_BINARY || op.kind == G_SELECT) {
      const GValue& x = bld.V(in.back());
      if (x.shape != oshape || x.dt != odt) return name + ": result type differs from the operands (%" + res + ")";
    }
    // stability patches of the reference (src/compiler/sanitizer.zig:8-111): log(x) -> log(x + 1e-4), a / b -> a / (b + 1e-4);
    // the constant is the literal 1.000000e-4 of the op's own element type
    if (sanitize && ((op.kind == G_UNARY && op.sub == U_LOG) || (op.kind == G_BINARY && op.sub == B_DIV))) {
      const int k = (int)op.in.size() - 1;
      op.in[k] = bld.binary(B_ADD, op.in[k], bld.splat(oshape, odt, 1.000000e-4));
    }
    env[res] = bld.emit(op, oshape, odt, res);
  }
  if (!returned) return "@main has no return";
  g->n_forward_ops = (int)g->ops.size();
  return "";
}

// ------------------------------------------------------------------------------------------------
// gradient program
// ------------------------------------------------------------------------------------------------
std::string graph_add_gradients(Graph* g, int n_params, int clamp, float lo, float hi) {
  Builder B{g, ""};
  const int nfwd = g->n_forward_ops;
  if (g->ret < 0 || n_params > (int)g->args.size()) return "gradient program: bad arguments";
  // src/autodiff/engine.zig:472-530: use counts over the forward ops, reverse Kahn order from the return, FIFO queue
  std::vector<int> use_count(g->vals.size(), 0);
  for (int i = 0; i < nfwd; ++i)
    for (int o : g->ops[i].in)
      if (g->vals[o].op >= 0) use_count[o] += 1;
  std::map<int, int> adj;
  {
    GOp s; s.kind = G_SEED;
    g->seed = B.emit(s, g->vals[g->ret].shape, g->vals[g->ret].dt);
    adj[g->ret] = g->seed;
  }
  const double eps_f32 = (double)1e-4f;      // the guard constant is built in f32 and converted (src/core/ops.zig:849-854)
  auto eps_like = [&](int x) { return B.splat(B.V(x).shape, B.V(x).dt, eps_f32); };
  auto inlist = [](const std::vector<int64_t>& v, int64_t i) { for (int64_t e : v) if (e == i) return true; return false; };

  std::deque<int> queue;
  if (g->vals[g->ret].op >= 0) queue.push_back(g->vals[g->ret].op);
  while (!queue.empty()) {
    const int oi = queue.front();
    queue.pop_front();
    const GOp op = g->ops[oi];            // a copy: emitting grows g->ops
    if (adj.count(op.out)) {
      int gr = adj[op.out];
      gr = B.reshape(gr, B.V(op.out).shape);
      const std::vector<int>& p = op.in;
      std::vector<int> grads(p.size(), -1);
      bool has_rule = true;
      switch (op.kind) {
        case G_BINARY:
          switch (op.sub) {
            case B_ADD: grads[0] = gr; grads[1] = gr; break;                                     // vjp_rules.zig:29
            case B_SUB: grads[0] = gr; grads[1] = B.unary(U_NEG, gr); break;                    // :67
            case B_MUL: grads[0] = B.binary(B_MUL, gr, p[1]); grads[1] = B.binary(B_MUL, gr, p[0]); break;   // :106
            case B_DIV: {                                                                        // :154, denominator b + 1e-4
              const int bs = B.binary(B_ADD, p[1], eps_like(p[1]));
              grads[0] = B.binary(B_DIV, gr, bs);
              grads[1] = B.unary(U_NEG, B.binary(B_DIV, B.binary(B_MUL, p[0], gr), B.binary(B_MUL, bs, bs)));
              break;
            }
            case B_POW: {                                                                        // :252: e * (y / x), 0 where x == 0; the exponent gets zeros
              const int y = B.binary(B_POW, p[0], p[1]);
              const int z = B.zeros_like(y);
              const int ydb = B.select(B.compare(C_EQ, p[0], B.zeros_like(p[0])), z, B.binary(B_DIV, y, p[0]));
              grads[0] = B.binary(B_MUL, gr, B.binary(B_MUL, p[1], ydb));
              grads[1] = B.zeros_like(p[1]);
              break;
            }
            case B_MAX:                                                                          // :499: ReLU rule, operand 0 only, strict x > 0
              grads[0] = B.select(B.compare(C_GT, p[0], B.zeros_like(p[0])), gr, B.zeros_like(gr));
              break;
            default: has_rule = false;
          }
          break;
        case G_UNARY:
          switch (op.sub) {
            case U_NEG: grads[0] = B.unary(U_NEG, gr); break;                                   // :339
            case U_EXP: grads[0] = B.binary(B_MUL, gr, B.unary(U_EXP, p[0])); break;            // :1436
            case U_LOG: grads[0] = B.binary(B_DIV, gr, B.binary(B_ADD, p[0], eps_like(p[0]))); break;   // :1476
            case U_RSQRT: {                                                                      // :1529: -0.5 g rsqrt(x + 1e-4)^3
              const int r = B.unary(U_RSQRT, B.binary(B_ADD, p[0], eps_like(p[0])));
              const int cub = B.binary(B_MUL, B.binary(B_MUL, r, r), r);
              grads[0] = B.binary(B_MUL, B.binary(B_MUL, gr, B.splat(B.V(gr).shape, B.V(gr).dt, -0.5)), cub);
              break;
            }
            case U_TANH: {                                                                       // :1692
              const int y = B.unary(U_TANH, p[0]);
              grads[0] = B.binary(B_MUL, gr, B.binary(B_SUB, B.splat(B.V(y).shape, B.V(y).dt, 1.0), B.binary(B_MUL, y, y)));
              break;
            }
            case U_LOGISTIC: {                                                                   // :1019
              const int s = B.unary(U_LOGISTIC, p[0]);
              grads[0] = B.binary(B_MUL, gr, B.binary(B_MUL, s, B.binary(B_SUB, B.splat(B.V(s).shape, B.V(s).dt, 1.0), s)));
              break;
            }
            case U_SIN: grads[0] = B.binary(B_MUL, gr, B.unary(U_COS, p[0])); break;            // :937
            case U_COS: grads[0] = B.unary(U_NEG, B.binary(B_MUL, gr, B.unary(U_SIN, p[0]))); break;   // :977
            default: has_rule = false;
          }
          break;
        case G_TRANSPOSE: {                                                                      // :373
          std::vector<int64_t> inv(op.a.size());
          for (size_t i = 0; i < op.a.size(); ++i) inv[op.a[i]] = (int64_t)i;
          grads[0] = B.transpose(gr, inv);
          break;
        }
        case G_DOT: {                                                                            // :426: batch dims are the leading ones
          const int ra = (int)B.V(p[0]).shape.size(), rb = (int)B.V(p[1]).shape.size(), rg = (int)B.V(gr).shape.size();
          const int nb = std::min(ra, std::min(rb, rg)) - 2;
          if (nb < 0) return "dot_general VJP: operands of rank < 2";
          std::vector<int64_t> batch;
          for (int i = 0; i < nb; ++i) batch.push_back(i);
          grads[0] = B.dot(gr, p[1], batch, batch, {rg - 1}, {rb - 1});
          grads[1] = B.dot(p[0], gr, batch, batch, {ra - 2}, {rg - 2});
          break;
        }
        case G_RESHAPE: grads[0] = B.reshape(gr, B.V(p[0]).shape); break;                      // :565
        case G_REDUCE: {                                                                         // sum :599, max :673
          const GValue x = B.V(p[0]);
          std::vector<int64_t> kept;
          for (size_t i = 0; i < x.shape.size(); ++i) if (!inlist(op.a, (int64_t)i)) kept.push_back((int64_t)i);
          const int gb = B.bcast(gr, kept, x.shape);
          if (op.sub == R_MAX) {
            const int mx = B.bcast(B.reduce(R_MAX, p[0], op.a), kept, x.shape);
            grads[0] = B.select(B.compare(C_EQ, p[0], mx), gb, B.zeros_like(p[0]));
          } else grads[0] = gb;
          break;
        }
        case G_GATHER_ROWS: {                                                                    // :1115: scatter-add of the rows
          GOp s; s.kind = G_SCATTER_ROWS; s.in = {gr, p[1]};
          grads[0] = B.emit(s, B.V(p[0]).shape, B.V(p[0]).dt);
          break;
        }
        case G_GATHER2: {                                                                        // :779
          GOp s; s.kind = G_SCATTER2; s.in = {gr, p[1]};
          grads[0] = B.emit(s, B.V(p[0]).shape, B.V(p[0]).dt);
          break;
        }
        case G_SLICE: {                                                                          // :1260: pad with zeros
          GOp s; s.kind = G_PAD; s.in = {gr}; s.a = op.a; s.b = op.b; s.c = op.c;
          grads[0] = B.emit(s, B.V(p[0]).shape, B.V(p[0]).dt);
          break;
        }
        case G_BCAST: {                                                                          // :1336
          const GValue x = B.V(p[0]);
          const GValue gv = B.V(gr);
          for (size_t i = 1; i < op.a.size(); ++i) if (op.a[i] <= op.a[i - 1]) return "broadcast_in_dim VJP: dims must increase";
          std::vector<int64_t> red;
          for (size_t i = 0; i < gv.shape.size(); ++i) {
            bool from_operand = false, expanded = false;
            for (size_t k = 0; k < op.a.size(); ++k)
              if (op.a[k] == (int64_t)i) { from_operand = true; expanded = (x.shape[k] == 1 && gv.shape[i] != 1); }
            if (!from_operand || expanded) red.push_back((int64_t)i);
          }
          grads[0] = B.reshape(B.reduce(R_ADD, gr, red), x.shape);
          break;
        }
        case G_CONVERT: if (is_float(B.V(p[0]).dt)) grads[0] = B.convert(gr, B.V(p[0]).dt); break;      // :1584
        case G_SELECT:                                                                           // :1640
          grads[1] = B.select(p[0], gr, B.zeros_like(gr));
          grads[2] = B.select(p[0], B.zeros_like(gr), gr);
          break;
        case G_CONCAT: {                                                                         // :1071
          const int64_t d = op.a[0];
          int64_t at = 0;
          for (size_t i = 0; i < p.size(); ++i) {
            const GValue x = B.V(p[i]);
            std::vector<int64_t> a(x.shape.size(), 0), b = B.V(gr).shape, c(x.shape.size(), 1);
            a[d] = at; b[d] = at + x.shape[d];
            grads[i] = B.slice(gr, a, b, c);
            at += x.shape[d];
          }
          break;
        }
        default: has_rule = false;      // constants, iota, compare, ... stop the gradient (engine.zig:134-193)
      }
      if (!B.err.empty()) return B.err;
      if (has_rule) {
        for (size_t i = 0; i < p.size(); ++i) {
          if (grads[i] < 0 || !is_float(B.V(p[i]).dt)) continue;
          // engine.zig:604-702: shape of the operand, finite guard, clamp in f32, the edge's element type, accumulate
          int gi = grads[i];
          if (B.V(gi).numel != B.V(p[i]).numel) return "adjoint of another size than its value";
          gi = B.reshape(gi, B.V(p[i]).shape);
          if (B.V(gi).dt != B.V(p[i]).dt) return "adjoint of another element type than its value";
          GOp gc; gc.kind = G_GUARD_CLAMP; gc.sub = clamp ? 1 : 0; gc.lo = lo; gc.hi = hi; gc.in = {gi};
          gi = B.emit(gc, B.V(gi).shape, B.V(gi).dt);
          if (!B.err.empty()) return B.err;
          adj[p[i]] = adj.count(p[i]) ? B.binary(B_ADD, adj[p[i]], gi) : gi;
        }
      }
    }
    for (int o : op.in) {
      if (g->vals[o].op < 0) continue;
      if (--use_count[o] == 0) queue.push_back(g->vals[o].op);
    }
  }
  g->grad_of_arg.assign(g->args.size(), -1);
  for (int i = 0; i < n_params; ++i) {
    const int a = g->args[i];
    if (adj.count(a)) g->grad_of_arg[i] = adj[a];
  }
  return B.err;
}

// ------------------------------------------------------------------------------------------------
// dump
// ------------------------------------------------------------------------------------------------
std::string graph_dump(const Graph& g) {
  std::string s;
  char buf[256];
  auto list = [&](const char* key, const std::vector<int64_t>& v) {
    s += " "; s += key; s += "=";
    for (size_t i = 0; i < v.size(); ++i) { snprintf(buf, sizeof buf, i ? ",%lld" : "%lld", (long long)v[i]); s += buf; }
  };
  snprintf(buf, sizeof buf, "graph vals=%zu ops=%zu forward_ops=%d ret=%d seed=%d\n", g.vals.size(), g.ops.size(), g.n_forward_ops, g.ret, g.seed);
  s += buf;
  s += "args";
  for (int a : g.args) { snprintf(buf, sizeof buf, " %d", a); s += buf; }
  s += "\ngrads";
  for (int a : g.grad_of_arg) { snprintf(buf, sizeof buf, " %d", a); s += buf; }
  s += "\n";
  for (size_t i = 0; i < g.vals.size(); ++i) {
    const GValue& v = g.vals[i];
    snprintf(buf, sizeof buf, "val %zu %s", i, dtype_name(v.dt));
    s += buf;
    list("shape", v.shape);
    s += " name=" + (v.name.empty() ? std::string("-") : v.name) + "\n";
  }
  for (size_t i = 0; i < g.ops.size(); ++i) {
    const GOp& o = g.ops[i];
    snprintf(buf, sizeof buf, "op %zu kind=%d sub=%d out=%d", i, o.kind, o.sub, o.out);
    s += buf;
    std::vector<int64_t> in(o.in.begin(), o.in.end());
    list("in", in); list("a", o.a); list("b", o.b); list("c", o.c); list("d", o.d);
    snprintf(buf, sizeof buf, " f=%.17g i=%lld lo=%.9g hi=%.9g data=", o.fval, o.ival, (double)o.lo, (double)o.hi);
    s += buf;
    static const char* hex = "0123456789abcdef";
    for (uint8_t c : o.data) { s.push_back(hex[c >> 4]); s.push_back(hex[c & 15]); }
    s += "\n";
  }
  return s;
}

}  // namespace pcpb

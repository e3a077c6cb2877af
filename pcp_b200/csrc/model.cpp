#include "model.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>

namespace pcpb {

namespace {

struct ArgType {
  std::vector<int64_t> shape;
  std::string elem;
};

// "tensor<65x64xf32>" -> shape, elem
bool parse_tensor_type(const std::string& s, ArgType* out) {
  size_t a = s.find("tensor<");
  if (a == std::string::npos) return false;
  a += 7;
  size_t b = s.find('>', a);
  if (b == std::string::npos) return false;
  std::string body = s.substr(a, b - a);
  out->shape.clear();
  size_t pos = 0;
  while (true) {
    size_t x = body.find('x', pos);
    if (x == std::string::npos) break;
    std::string tok = body.substr(pos, x - pos);
    if (tok.empty() || tok.find_first_not_of("0123456789") != std::string::npos) break;
    out->shape.push_back(strtoll(tok.c_str(), nullptr, 10));
    pos = x + 1;
  }
  out->elem = body.substr(pos);
  return !out->elem.empty();
}

std::string first_operand(const std::string& line) {
  size_t eq = line.find('=');
  if (eq == std::string::npos) return "";
  size_t p = line.find('%', eq);
  if (p == std::string::npos) return "";
  size_t e = p + 1;
  while (e < line.size() && (isalnum((unsigned char)line[e]) || line[e] == '_' || line[e] == '.')) ++e;
  return line.substr(p, e - p);
}

std::string nth_operand(const std::string& line, int n) {
  size_t eq = line.find('=');
  size_t p = eq;
  std::string r;
  for (int i = 0; i <= n; ++i) {
    p = line.find('%', p == std::string::npos ? 0 : p + 1);
    if (p == std::string::npos) return "";
    size_t e = p + 1;
    while (e < line.size() && (isalnum((unsigned char)line[e]) || line[e] == '_' || line[e] == '.')) ++e;
    r = line.substr(p, e - p);
  }
  return r;
}

}  // namespace

std::string parse_artifact(const char* text, size_t n, ModelConfig* cfg) {
  std::string src(text, n);
  size_t fpos = src.find("@main(");
  if (fpos == std::string::npos) return "no func.func @main in artefact";
  size_t sig_end = src.find("->", fpos);
  size_t line_end = src.find('\n', fpos);
  if (sig_end == std::string::npos || line_end == std::string::npos || sig_end > line_end)
    return "cannot parse the @main signature";
  std::string sig = src.substr(fpos, sig_end - fpos);
  std::vector<ArgType> args;
  size_t p = 0;
  while ((p = sig.find("tensor<", p)) != std::string::npos) {
    ArgType t;
    size_t e = sig.find('>', p);
    if (!parse_tensor_type(sig.substr(p, e - p + 1), &t)) return "bad argument type in @main";
    args.push_back(t);
    p = e;
  }
  if (args.size() < 4) return "@main has too few arguments";
  const size_t nP = args.size() - 2;
  const ArgType& ids = args[nP];
  if (ids.elem != "i64" || ids.shape.size() != 2 || args[nP + 1].elem != "i64" || args[nP + 1].shape != ids.shape)
    return "the last two @main arguments must be i64 [B,T] token ids and targets";
  // ---- nanoGPT family: wte [V,d], wpe [T,d], 8 tensors per layer (4 of them rank 1), ln_f w/b, head w/b ----
  if (nP >= 14 && (nP - 6) % 8 == 0 && args[0].shape.size() == 2 && args[1].shape.size() == 2 &&
      args[2].shape.size() == 1 && args[nP - 1].shape.size() == 1) {
    ModelConfig c;
    c.family = FAMILY_NANOGPT;
    if (args[0].elem == "f32") c.dtype = 0;
    else if (args[0].elem == "bf16") c.dtype = 3;
    else return "unsupported model dtype " + args[0].elem;
    c.B = ids.shape[0]; c.T = ids.shape[1];
    c.V = args[0].shape[0]; c.d = args[0].shape[1];
    c.L = (int64_t)(nP - 6) / 8;
    if (args[1].shape[0] != c.T || args[1].shape[1] != c.d) return "wpe shape must be [T, d]";
    c.F = args[8].shape[0];
    for (int64_t l = 0; l < c.L; ++l) {
      const ArgType* a = &args[2 + 8 * l];
      auto v1 = [&](const ArgType& t) { return t.shape.size() == 1 && t.shape[0] == c.d; };
      auto m2 = [&](const ArgType& t, int64_t r, int64_t k) { return t.shape.size() == 2 && t.shape[0] == r && t.shape[1] == k; };
      if (!(v1(a[0]) && v1(a[1]) && m2(a[2], 3 * c.d, c.d) && m2(a[3], c.d, c.d) && v1(a[4]) && v1(a[5]) &&
            m2(a[6], c.F, c.d) && m2(a[7], c.d, c.F)))
        return "layer parameter shapes do not follow ln1,c_attn,c_proj,ln2,c_fc,c_proj";
    }
    const ArgType* t = &args[nP - 4];
    if (!(t[0].shape.size() == 1 && t[0].shape[0] == c.d && t[1].shape.size() == 1 && t[1].shape[0] == c.d &&
          t[2].shape.size() == 2 && t[2].shape[0] == c.V && t[2].shape[1] == c.d && t[3].shape[0] == c.V))
      return "final LayerNorm / lm_head shapes not recognised";
    for (size_t i = 0; i < nP; ++i) if (args[i].elem != args[0].elem) return "all parameters must share one dtype";
    // heads: the first reshape to [B, T, H, hd]
    {
      char pat[64];
      snprintf(pat, sizeof pat, "-> tensor<%lldx%lldx", (long long)c.B, (long long)c.T);
      size_t q = 0;
      while ((q = src.find(pat, q)) != std::string::npos) {
        ArgType rt;
        size_t e = src.find('>', q);
        if (parse_tensor_type(src.substr(q + 3, e - q - 2), &rt) && rt.shape.size() == 4 && rt.shape[2] * rt.shape[3] == c.d) {
          c.H = rt.shape[2]; c.hd = rt.shape[3];
          break;
        }
        q = e;
      }
      if (c.H == 0) return "could not find the [B,T,H,hd] reshape";
    }
    c.Hkv = c.H;
    // MLP activation: max(u, 0), or the tanh GELU written as u*u*u, 0.044715, sqrt(2/pi), tanh, +1, 0.5*u (one tanh
    // per layer and no other use of tanh in this family).  Anything else is refused.
    {
      size_t n_tanh = 0;
      for (size_t q = 0; (q = src.find("stablehlo.tanh", q)) != std::string::npos; ++q) ++n_tanh;
      if (src.find("stablehlo.power") != std::string::npos || src.find("stablehlo.erf") != std::string::npos ||
          src.find("stablehlo.logistic") != std::string::npos)
        return "nanoGPT graph with an activation other than ReLU or tanh-GELU is not supported";
      if (n_tanh == 0) c.activation = ACT_NATIVE;
      else if ((int64_t)n_tanh == c.L && src.find("dense<4.47149985e-02>") != std::string::npos &&
               src.find("dense<7.97884583e-01>") != std::string::npos)
        c.activation = ACT_GELU_TANH;
      else
        return "nanoGPT graph with an activation other than ReLU or tanh-GELU is not supported";
    }
    // Body fingerprint, as for nanochat below: per layer two rsqrt (LayerNorms), one exponential (softmax), six
    // dot_general, one select (causal mask) and, with ReLU, one maximum; the head adds one rsqrt, one exponential and
    // one log (cross entropy), one negate, one dot_general and three selects.
    {
      auto count = [&](const char* op) {
        size_t n = 0;
        const std::string pat = std::string("= stablehlo.") + op + " ";
        for (size_t q = 0; (q = src.find(pat, q)) != std::string::npos; ++q) ++n;
        return (int64_t)n;
      };
      struct { const char* op; int64_t want; } expect[] = {
          {"rsqrt", 2 * c.L + 1}, {"maximum", c.activation == ACT_NATIVE ? c.L : 0}, {"exponential", c.L + 1}, {"log", 1},
          {"dot_general", 6 * c.L + 1}, {"select", c.L + 3}, {"negate", 1}, {"sqrt", 0}, {"sine", 0}, {"cosine", 0},
          {"abs", 0}, {"minimum", 0}, {"clamp", 0}, {"convolution", 0}};
      for (auto& e : expect) {
        const int64_t got = count(e.op);
        if (got != e.want)
          return std::string("not a nanoGPT-family body: ") + std::to_string(got) + " stablehlo." + e.op +
                 " ops where the family has " + std::to_string(e.want);
      }
    }
    if (src.find("dense<-100>") == std::string::npos) return "expected ignore_index -100 in the loss";
    c.ignore_index = -100;
    c.softcap = 0.f;
    int64_t off = 0;
    for (size_t i = 0; i < nP; ++i) {
      TensorInfo ti;
      ti.shape = args[i].shape;
      ti.numel = 1;
      for (int64_t s : args[i].shape) ti.numel *= s;
      ti.offset = off;
      off += ti.numel;              // tight, like the reference's parameter blob (src/algorithms/diloco.zig:665-667)
      c.params.push_back(ti);
    }
    c.total_params = off;
    *cfg = c;
    return "";
  }
  if ((nP - 2) % 6 != 0 || nP < 8) return "not a nanochat- or nanoGPT-family graph (unexpected parameter list)";
  for (size_t i = 0; i < nP; ++i)
    if (args[i].shape.size() != 2 || args[i].elem != args[0].elem)
      return "not a nanochat-family graph (all parameters must be rank-2 of one dtype)";
  ModelConfig c;
  if (args[0].elem == "f32") c.dtype = 0;
  else if (args[0].elem == "bf16") c.dtype = 3;
  else return "unsupported model dtype " + args[0].elem;
  c.B = ids.shape[0]; c.T = ids.shape[1];
  c.V = args[0].shape[0]; c.d = args[0].shape[1];
  c.L = (int64_t)(nP - 2) / 6;
  if (args[nP - 1].shape[0] != c.V || args[nP - 1].shape[1] != c.d) return "lm_head shape does not match wte";
  int64_t dkv = args[2].shape[0];
  c.F = args[5].shape[0];
  for (int64_t l = 0; l < c.L; ++l) {
    const ArgType* a = &args[1 + 6 * l];
    const bool ok = a[0].shape[0] == c.d && a[0].shape[1] == c.d && a[1].shape[0] == dkv && a[1].shape[1] == c.d &&
                    a[2].shape[0] == dkv && a[2].shape[1] == c.d && a[3].shape[0] == c.d && a[3].shape[1] == c.d &&
                    a[4].shape[0] == c.F && a[4].shape[1] == c.d && a[5].shape[0] == c.d && a[5].shape[1] == c.F;
    if (!ok) return "layer parameter shapes do not follow q,k,v,proj,fc,proj";
  }

  // RoPE tables: the two dense_resource constants of type tensor<1xTx1x(hd/2)xbf16>
  std::vector<std::string> keys;
  {
    size_t q = 0;
    while ((q = src.find("dense_resource<", q)) != std::string::npos) {
      size_t e = src.find('>', q);
      std::string key = src.substr(q + 15, e - q - 15);
      size_t le = src.find('\n', e);
      ArgType t;
      if (parse_tensor_type(src.substr(e, le - e), &t) && t.elem == "bf16" && t.shape.size() == 4 &&
          t.shape[0] == 1 && t.shape[1] == c.T && t.shape[2] == 1) {
        c.hd = 2 * t.shape[3];
        keys.push_back(key);
      }
      q = e;
    }
  }
  if (keys.size() < 2 || c.hd <= 0) return "RoPE table resources not found";
  if (c.d % c.hd != 0 || dkv % c.hd != 0) return "head_dim does not divide the model width";
  c.H = c.d / c.hd; c.Hkv = dkv / c.hd;
  if (c.H % c.Hkv != 0) return "query heads are not a multiple of kv heads";
  size_t rs = src.find("dialect_resources");
  if (rs == std::string::npos) return "no dialect_resources section";
  const size_t half = (size_t)c.hd / 2;
  for (const std::string& key : keys) {
    size_t k = src.find(key + ":", rs);
    if (k == std::string::npos) return "resource blob missing: " + key;
    size_t h = src.find("\"0x", k);
    size_t he = src.find('"', h + 1);
    if (h == std::string::npos || he == std::string::npos) return "bad resource blob";
    const char* hex = src.c_str() + h + 3;
    size_t nhex = he - (h + 3);
    if (nhex < 8 + 4 * (size_t)c.T * half) return "resource blob too short";
    std::vector<uint16_t> vals((size_t)c.T * half);
    auto hv = [](char ch) -> int { return ch <= '9' ? ch - '0' : (ch | 32) - 'a' + 10; };
    for (size_t i = 0; i < vals.size(); ++i) {
      const char* q = hex + 8 + 4 * i;                    // skip the 4-byte alignment header
      int lo = hv(q[0]) * 16 + hv(q[1]), hi = hv(q[2]) * 16 + hv(q[3]);
      vals[i] = (uint16_t)(lo | (hi << 8));
    }
    // cos(0) = 1.0 (0x3F80), sin(0) = 0
    if (vals[0] == 0x3F80) c.rope_cos.swap(vals); else c.rope_sin.swap(vals);
  }
  if (c.rope_cos.empty() || c.rope_sin.empty()) return "could not tell the cos table from the sin table";

  // soft-cap: constant feeding the divide in front of stablehlo.tanh
  {
    std::map<std::string, std::string> defs;
    size_t q = line_end + 1;
    while (q < src.size()) {
      size_t e = src.find('\n', q);
      if (e == std::string::npos) e = src.size();
      std::string line = src.substr(q, e - q);
      size_t pc = line.find('%');
      size_t eq = line.find(" = ");
      if (pc != std::string::npos && eq != std::string::npos && pc < eq) defs[line.substr(pc, eq - pc)] = line;
      if (line.find("return") != std::string::npos && line.find("stablehlo") == std::string::npos) break;
      q = e + 1;
    }
    bool found = false;
    for (auto& kv : defs) {
      if (kv.second.find("stablehlo.tanh") == std::string::npos) continue;
      std::string cur = first_operand(kv.second);          // the divide
      auto it = defs.find(cur);
      if (it == defs.end() || it->second.find("stablehlo.divide") == std::string::npos) continue;
      cur = nth_operand(it->second, 1);                    // its denominator
      for (int hop = 0; hop < 8 && !cur.empty(); ++hop) {
        auto d2 = defs.find(cur);
        if (d2 == defs.end()) break;
        size_t dl = d2->second.find("dense<");
        if (dl != std::string::npos) {
          c.softcap = (float)strtod(d2->second.c_str() + dl + 6, nullptr);
          found = true;
          break;
        }
        cur = first_operand(d2->second);
      }
      if (found) break;
    }
    if (!found) return "soft-cap constant not found (expected tanh(z / cap) * cap before the loss)";
  }
  // Body fingerprint.  The signature alone does not tell the family: a graph with these parameter shapes but, say, a
  // GELU MLP or no QK-norm would otherwise be trained with the built-in nanochat arithmetic.  Per layer the family
  // has four rsqrt (two block norms, the q and k norms), five power (their squares and the ReLU^2), one maximum, one
  // exponential (softmax), eight dot_general and one select (causal mask); the head adds two rsqrt / power (embedding
  // and final norm), one tanh (soft-cap), one exponential and one log (cross entropy), one dot_general and two
  // selects (ignored targets), and names the ignore index -1.
  {
    auto count = [&](const char* op) {
      size_t n = 0;
      const std::string pat = std::string("= stablehlo.") + op + " ";
      for (size_t q = 0; (q = src.find(pat, q)) != std::string::npos; ++q) ++n;
      return (int64_t)n;
    };
    struct { const char* op; int64_t want; } expect[] = {
        {"rsqrt", 4 * c.L + 2}, {"power", 5 * c.L + 2}, {"maximum", c.L}, {"tanh", 1}, {"exponential", c.L + 1},
        {"log", 1}, {"dot_general", 8 * c.L + 1}, {"select", c.L + 2}, {"erf", 0}, {"logistic", 0}, {"sqrt", 0},
        {"sine", 0}, {"cosine", 0}, {"abs", 0}, {"minimum", 0}, {"clamp", 0}, {"convolution", 0}};
    for (auto& e : expect) {
      const int64_t got = count(e.op);
      if (got != e.want)
        return std::string("not a nanochat-family body: ") + std::to_string(got) + " stablehlo." + e.op +
               " ops where the family has " + std::to_string(e.want) +
               " (RMSNorm + RoPE + QK-norm + ReLU^2 + soft-capped cross entropy expected)";
    }
    if (src.find("dense<-1>") == std::string::npos) return "expected ignore_index -1 in the loss";
  }
  c.ignore_index = -1;

  int64_t off = 0;
  for (size_t i = 0; i < nP; ++i) {
    TensorInfo t;
    t.shape = args[i].shape;
    t.numel = args[i].shape[0] * args[i].shape[1];
    t.offset = off;
    off += t.numel;
    c.params.push_back(t);
  }
  c.total_params = off;
  *cfg = c;
  return "";
}

}  // namespace pcpb

// Rewriter-lite: the decisions of XLA's GemmRewriter for the quantized scaled dot, restated over
// the small subset of HLO text this repository's fixtures use, emitting this library's custom-call
// targets instead of "__cublas$lt$matmul$f8" / "__cublas$lt$matmul".
//
// What is followed (xla/backends/gpu/transforms/gemm_rewriter.cc):
//   * MatchFp8Param / FindF8SubgraphRecursive (:190-336): a dot operand must be convert(f8 x),
//     optionally times or divided by broadcast(scalar scale).
//   * CreateF8CustomCall (:1235-1591): operand types e4m3fn / e5m2 but not both e5m2; scalar scales
//     become f32 operands, inverted when the HLO divides, constant 1 when absent; exactly one
//     contracting dimension per operand; no transposes are inserted (Blackwell, :1535-1554).
//   * FuseVectorBiasAdd (:1987-2124), FuseMatrixBiasAdd (:1829-1978), FuseReluActivation
//     (:2126-2164), FuseGeluActivation (:888-1007, 2166-2249), F8ConvertD / F8AddDAmax
//     (:1635-1794): the users of the dot are folded into the epilogue in the order the HLO
//     applies them; the FP8 output cast needs clamp bounds equal to the type's +-max.
//   * GemmWorkspaceRewriteVisitor (:2774-2892): a trailing s8[32 MiB] workspace result.
//   * The s8 x s8 -> s32 dot goes to the integer target; unlike the reference (which refuses to
//     fuse it, :897-901) the following per-row x per-column dequantisation is folded in too.
// Anything outside these patterns is left alone: the function reports "not rewritten".
//
// The output is (a) the rewritten module as HLO text and (b) a small JSON "plan" that tells a
// runner how to obtain each custom-call operand from the module's parameters and which root
// outputs the results feed -- the information ThunkEmitter would read off the instruction.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <string>
#include <vector>

namespace {

struct Shape {
  std::string type;                 // "f32", "f8e4m3fn", ... or "tuple"
  std::vector<int64_t> dims;
  std::vector<Shape> elements;      // for tuples
  std::vector<int64_t> layout;      // minor_to_major as written ({1,0} row-major); empty = default (row-major)
  bool IsColumnMajor2D() const { return dims.size() == 2 && layout.size() == 2 && layout[0] == 0 && layout[1] == 1; }
  std::string ToString() const {
    if (type == "tuple") {
      std::string s = "(";
      for (size_t i = 0; i < elements.size(); ++i) s += (i ? ", " : "") + elements[i].ToString();
      return s + ")";
    }
    std::string s = type + "[";
    for (size_t i = 0; i < dims.size(); ++i) s += (i ? "," : "") + std::to_string(dims[i]);
    s += "]";
    if (!layout.empty()) {
      s += "{";
      for (size_t i = 0; i < layout.size(); ++i) s += (i ? "," : "") + std::to_string(layout[i]);
      s += "}";
    }
    return s;
  }
  bool IsScalar() const { return type != "tuple" && dims.empty(); }
};

struct Instr {
  std::string name;
  Shape shape;
  std::string opcode;
  std::vector<std::string> operands;
  std::string attrs;                // everything after the closing parenthesis, verbatim
  std::string literal;              // constant(...) / parameter(...) payload
  bool is_root = false;
};

struct Computation {
  std::string name;
  bool is_entry = false;
  std::vector<Instr> instrs;
  std::string raw;                  // original text, re-emitted verbatim for non-entry computations
};

struct Module {
  std::string name;
  std::vector<Computation> computations;
};

std::string Trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
  return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}

bool ParseShape(const std::string& text, size_t* pos, Shape* out) {
  size_t p = *pos;
  while (p < text.size() && text[p] == ' ') ++p;
  if (p < text.size() && text[p] == '(') {               // tuple shape
    out->type = "tuple";
    ++p;
    while (true) {
      while (p < text.size() && (text[p] == ' ' || text[p] == ',')) ++p;
      if (p < text.size() && text[p] == ')') { ++p; break; }
      Shape e;
      if (!ParseShape(text, &p, &e)) return false;
      out->elements.push_back(e);
    }
    *pos = p;
    return true;
  }
  size_t start = p;
  while (p < text.size() && (isalnum(static_cast<unsigned char>(text[p])) || text[p] == '_')) ++p;
  if (p == start || p >= text.size() || text[p] != '[') return false;
  out->type = text.substr(start, p - start);
  ++p;
  std::string num;
  while (p < text.size() && text[p] != ']') {
    if (text[p] == ',') { if (!num.empty()) out->dims.push_back(std::stoll(num)); num.clear(); }
    else if (text[p] != ' ') num += text[p];
    ++p;
  }
  if (p >= text.size()) return false;
  if (!num.empty()) out->dims.push_back(std::stoll(num));
  ++p;
  if (p < text.size() && text[p] == '{') {                // layout suffix: minor_to_major, e.g. {1,0}
    ++p;
    std::string v;
    while (p < text.size() && text[p] != '}') {
      if (text[p] == ',') { if (!v.empty()) out->layout.push_back(std::stoll(v)); v.clear(); }
      else if (isdigit(static_cast<unsigned char>(text[p]))) v += text[p];
      ++p;
    }
    if (!v.empty()) out->layout.push_back(std::stoll(v));
    if (p < text.size()) ++p;
  }
  *pos = p;
  return true;
}

// "name = shape opcode(operands), attrs"
bool ParseInstr(const std::string& line_in, Instr* in, std::string* err) {
  std::string line = Trim(line_in);
  if (line.rfind("ROOT ", 0) == 0) { in->is_root = true; line = Trim(line.substr(5)); }
  size_t eq = line.find(" = ");
  if (eq == std::string::npos) { *err = "no '=' in instruction: " + line; return false; }
  in->name = Trim(line.substr(0, eq));
  if (!in->name.empty() && in->name[0] == '%') in->name = in->name.substr(1);
  size_t p = eq + 3;
  if (!ParseShape(line, &p, &in->shape)) { *err = "bad shape in: " + line; return false; }
  while (p < line.size() && line[p] == ' ') ++p;
  size_t op_start = p;
  while (p < line.size() && line[p] != '(') ++p;
  if (p >= line.size()) { *err = "no '(' in: " + line; return false; }
  in->opcode = Trim(line.substr(op_start, p - op_start));
  int depth = 0;
  size_t args_start = p + 1, args_end = std::string::npos;
  for (; p < line.size(); ++p) {
    if (line[p] == '(') ++depth;
    else if (line[p] == ')') { if (--depth == 0) { args_end = p; break; } }
  }
  if (args_end == std::string::npos) { *err = "unbalanced parentheses in: " + line; return false; }
  const std::string args = line.substr(args_start, args_end - args_start);
  if (in->opcode == "constant" || in->opcode == "parameter") {
    in->literal = Trim(args);
  } else {
    std::string cur;
    int d = 0;
    for (char c : args) {
      if (c == '(' || c == '[' || c == '{') ++d;
      if (c == ')' || c == ']' || c == '}') --d;
      if (c == ',' && d == 0) { in->operands.push_back(Trim(cur)); cur.clear(); }
      else cur += c;
    }
    if (!Trim(cur).empty()) in->operands.push_back(Trim(cur));
    for (std::string& o : in->operands) {                 // "f32[4] %x" or "%x" or "x"
      size_t sp = o.find_last_of(' ');
      if (sp != std::string::npos) o = o.substr(sp + 1);
      if (!o.empty() && o[0] == '%') o = o.substr(1);
    }
  }
  in->attrs = Trim(line.substr(args_end + 1));
  if (!in->attrs.empty() && in->attrs[0] == ',') in->attrs = Trim(in->attrs.substr(1));
  return true;
}

bool ParseModule(const std::string& text, Module* m, std::string* err) {
  std::istringstream ss(text);
  std::string line;
  Computation* cur = nullptr;
  while (std::getline(ss, line)) {
    const std::string t = Trim(line);
    if (t.empty() || t.rfind("//", 0) == 0) continue;
    if (t.rfind("HloModule", 0) == 0) {
      std::istringstream ls(t);
      std::string kw;
      ls >> kw >> m->name;
      if (!m->name.empty() && m->name.back() == ',') m->name.pop_back();
      continue;
    }
    if (cur == nullptr) {
      if (t.back() != '{') { *err = "expected a computation header, got: " + t; return false; }
      m->computations.emplace_back();
      cur = &m->computations.back();
      std::string head = Trim(t.substr(0, t.size() - 1));
      if (head.rfind("ENTRY ", 0) == 0) { cur->is_entry = true; head = Trim(head.substr(6)); }
      size_t sp = head.find_first_of(" (");
      cur->name = head.substr(0, sp);
      if (!cur->name.empty() && cur->name[0] == '%') cur->name = cur->name.substr(1);
      cur->raw = line + "\n";
      continue;
    }
    cur->raw += line + "\n";
    if (t == "}") { cur = nullptr; continue; }
    Instr in;
    if (!ParseInstr(t, &in, err)) return false;
    cur->instrs.push_back(in);
  }
  for (const Computation& c : m->computations)
    if (c.is_entry) return true;
  *err = "module has no ENTRY computation";
  return false;
}

int64_t AttrDim(const std::string& attrs, const std::string& key, int64_t dflt) {
  size_t p = attrs.find(key + "={");
  if (p == std::string::npos) return dflt;
  p += key.size() + 2;
  size_t e = attrs.find('}', p);
  std::string body = attrs.substr(p, e - p);
  if (body.empty() || body.find(',') != std::string::npos) return -2;    // none or several
  return std::stoll(body);
}

bool IsF8(const std::string& t) { return t == "f8e4m3fn" || t == "f8e5m2"; }
double F8Max(const std::string& t) { return t == "f8e4m3fn" ? 448.0 : 57344.0; }
int TypeCode(const std::string& t) {       // xla::PrimitiveType numbers
  static const std::map<std::string, int> k = {{"s8", 2}, {"s32", 4}, {"f16", 10}, {"f32", 11}, {"bf16", 16},
                                               {"f8e5m2", 19}, {"f8e4m3fn", 20}};
  auto it = k.find(t);
  return it == k.end() ? 0 : it->second;
}

}  // namespace

namespace {

struct Graph {
  Computation* comp = nullptr;
  std::map<std::string, Instr*> by_name;
  std::map<std::string, std::vector<Instr*>> users;
  Instr* root = nullptr;

  explicit Graph(Computation* c) : comp(c) {
    for (Instr& i : c->instrs) by_name[i.name] = &i;
    for (Instr& i : c->instrs) {
      std::set<std::string> seen;
      for (const std::string& o : i.operands)
        if (seen.insert(o).second) users[o].push_back(&i);
      if (i.is_root) root = &i;
    }
    if (root == nullptr && !c->instrs.empty()) root = &c->instrs.back();
  }
  Instr* Get(const std::string& n) const {
    auto it = by_name.find(n);
    return it == by_name.end() ? nullptr : it->second;
  }
  Instr* Operand(const Instr* i, size_t k) const { return k < i->operands.size() ? Get(i->operands[k]) : nullptr; }
  const std::vector<Instr*>& Users(const Instr* i) const {
    static const std::vector<Instr*> none;
    auto it = users.find(i->name);
    return it == users.end() ? none : it->second;
  }
};

// broadcast(scalar) with dimensions={} -> the scalar instruction.
Instr* BroadcastedScalar(const Graph& g, Instr* x) {
  if (x == nullptr || x->opcode != "broadcast") return nullptr;
  Instr* s = g.Operand(x, 0);
  return (s != nullptr && s->shape.IsScalar()) ? s : nullptr;
}

bool ScalarConstant(const Graph& g, Instr* x, double* value) {
  if (x == nullptr) return false;
  if (x->opcode == "broadcast") x = BroadcastedScalar(g, x);
  if (x == nullptr || x->opcode != "constant" || !x->shape.IsScalar()) return false;
  const std::string& l = x->literal;
  if (l == "inf") *value = INFINITY;
  else if (l == "-inf") *value = -INFINITY;
  else {
    char* end = nullptr;
    *value = std::strtod(l.c_str(), &end);
    if (end == l.c_str()) return false;
  }
  return true;
}
bool IsConstantNear(const Graph& g, Instr* x, double want, double rel = 1e-5) {
  double v;
  return ScalarConstant(g, x, &v) && std::fabs(v - want) <= rel * std::max(1.0, std::fabs(want));
}

// For a binary instruction of `opcode` one of whose operands is `a`, the other operand.
Instr* OtherOperand(const Graph& g, Instr* bin, const char* opcode, Instr* a) {
  if (bin == nullptr || bin->opcode != opcode || bin->operands.size() != 2) return nullptr;
  Instr* l = g.Operand(bin, 0);
  Instr* r = g.Operand(bin, 1);
  if (l == a) return r;
  if (r == a) return l;
  return nullptr;
}
// The user of `x` with the given opcode whose other operand satisfies `pred`; nullptr if none.
template <typename Pred>
Instr* UserWith(const Graph& g, Instr* x, const char* opcode, Pred pred) {
  for (Instr* u : g.Users(x)) {
    if (u->opcode != opcode) continue;
    if (u->operands.size() == 2 && u->operands[0] == x->name && u->operands[1] == x->name) {
      if (pred(x)) return u;
      continue;
    }
    Instr* other = OtherOperand(g, u, opcode, x);
    if (other != nullptr && pred(other)) return u;
  }
  return nullptr;
}

// Where a custom-call operand comes from, in terms of the module's own parameters.
struct Source {
  std::string role;
  int param = -1;            // parameter number, or -1 for a constant
  bool reciprocal = false;   // operand = 1 / parameter (the HLO divided by the scale)
  double constant = 1.0;     // value when param < 0
  Shape shape;
  Shape padded;              // shape the custom call receives (dimensions rounded up to 16)
  bool reshaped = false;     // the parameter is viewed in another shape (a bitcast of the same row-major bytes)
  bool transposed = false;   // the parameter is column-major: its buffer IS the row-major matrix with the dimensions swapped
  std::string instr;         // name of the instruction in the original module
};

bool AsParameter(Instr* x, int* number) {
  if (x == nullptr || x->opcode != "parameter") return false;
  *number = std::atoi(x->literal.c_str());
  return true;
}

struct Fp8Operand {
  Instr* f8 = nullptr;       // the FP8 value (must be a parameter in the lite version)
  Instr* scale = nullptr;    // scalar the dequantised value was multiplied / divided by, or nullptr
  bool divide = false;
  bool reshaped = false;     // a bitcast / reshape sat between the dequantisation and the dot
  Shape view;                // ... and gave the operand this shape (same bytes, row-major)
};

// MatchFp8Param (gemm_rewriter.cc:190-336) for the shapes the fixtures use.
bool MatchFp8Operand(const Graph& g, Instr* x, Fp8Operand* out) {
  if (x == nullptr) return false;
  // A bitcast / reshape of the dequantised value commutes with the dequantisation (FindF8SubgraphRecursive walks
  // through it, gemm_rewriter.cc:248-336; gemm_rewriter_fp8_test.cc:579-612): the FP8 buffer is viewed in the new shape.
  while (x->opcode == "bitcast" || x->opcode == "reshape") {
    if (!x->shape.layout.empty() && !std::is_sorted(x->shape.layout.rbegin(), x->shape.layout.rend())) return false;
    if (!out->reshaped) { out->reshaped = true; out->view = x->shape; }
    x = g.Operand(x, 0);
    if (x == nullptr) return false;
  }
  if (IsF8(x->shape.type)) {        // an FP8 value fed to the dot as it is (gemm_rewriter_fp8_test.cc:313-350)
    out->f8 = x;
    return true;
  }
  Instr* conv = x;
  if (x->opcode == "multiply" || x->opcode == "divide") {
    Instr* l = g.Operand(x, 0);
    Instr* r = g.Operand(x, 1);
    Instr* sl = BroadcastedScalar(g, l);
    Instr* sr = BroadcastedScalar(g, r);
    if (sr != nullptr) { conv = l; out->scale = sr; }
    else if (sl != nullptr && x->opcode == "multiply") { conv = r; out->scale = sl; }
    else return false;
    out->divide = x->opcode == "divide";
  }
  if (conv == nullptr || conv->opcode != "convert") return false;
  Instr* src = g.Operand(conv, 0);
  if (src == nullptr || !IsF8(src->shape.type)) return false;
  out->f8 = src;
  return true;
}

// The decisions taken for one dot: everything a thunk emitter would read off the custom call.
struct Plan {
  bool rewritten = false;
  std::string reason;                  // why not, when not rewritten
  std::string target;
  int64_t m = 0, n = 0, k = 0;
  int lhs_contracting = 1, rhs_contracting = 0;
  int epilogue = 0;                    // GemmBackendConfig.Epilogue number (backend_configs.proto:106-117; DEFAULT = 0)
  double alpha = 1.0, beta = 0.0;
  bool damax = false, emit_s32 = false;
  int64_t batch = 0;                   // > 0: leading batch dimension of a, b, c and D
  bool d_viewed = false;               // a bitcast / reshape sits behind the dot: the [m, n] result is viewed as d_view
  Shape d_view;
  bool d_transposed = false;           // the result is column-major: the call computes D^T = B^T A^T into a row-major [n, m] buffer
  std::vector<Source> operands;
  Shape d_shape, d_padded;
  int d_root_index = -1, amax_root_index = -1;   // position in the ROOT tuple (-1: ROOT itself / absent)
  std::string d_instr, amax_instr;     // instructions of the original module the results replace
};

bool ScaleSource(const Graph& g, Instr* scale, bool divide, const char* role, Source* out, std::string* why) {
  out->role = role;
  out->shape.type = "f32";
  if (scale == nullptr) { out->param = -1; out->constant = 1.0; return true; }
  if (scale->shape.type != "f32") { *why = std::string(role) + " is not f32"; return false; }
  double v;
  if (ScalarConstant(g, scale, &v)) { out->param = -1; out->constant = divide ? 1.0 / v : v; return true; }
  if (!AsParameter(scale, &out->param)) { *why = std::string(role) + " is neither a parameter nor a constant"; return false; }
  out->reciprocal = divide;
  out->instr = scale->name;
  return true;
}

// Follows the single chain of users of the dot and folds what the reference folds.
void MatchF8Epilogue(const Graph& g, Instr* dot, Plan* plan) {
  Instr* cur = dot;
  bool relu = false, gelu = false, vector_bias = false;
  // -- alpha: multiply(dot, broadcast(constant)) right behind the dot (HandleMultiply, gemm_rewriter.cc:888-921;
  //    gemm_rewriter_fp8_test.cc:993-1047)
  if (g.Users(cur).size() == 1 && g.Users(cur)[0]->opcode == "multiply") {
    Instr* mul = g.Users(cur)[0];
    Instr* other = OtherOperand(g, mul, "multiply", cur);
    double c;
    if (other != nullptr && ScalarConstant(g, BroadcastedScalar(g, other), &c)) {
      plan->alpha = c;
      cur = mul;
    }
  }
  // -- a bitcast / reshape of the dot's result that keeps the minor dimension (a rank-3 x rank-2 dot written as a
  //    matrix product, gemm_rewriter_fp8_test.cc:2112-2186, 2274-2344): the epilogue continues on the view
  if (g.Users(cur).size() == 1 && (g.Users(cur)[0]->opcode == "bitcast" || g.Users(cur)[0]->opcode == "reshape")) {
    Instr* v = g.Users(cur)[0];
    const bool row_major = v->shape.layout.empty() || std::is_sorted(v->shape.layout.rbegin(), v->shape.layout.rend());
    if (row_major && !v->shape.dims.empty() && v->shape.dims.back() == plan->n) {
      plan->d_viewed = true;
      cur = v;
    }
  }
  // -- bias (vector along the minor dimension, or a full matrix with beta = 1)
  for (Instr* u : g.Users(cur)) {
    if (u->opcode != "add") continue;
    Instr* other = OtherOperand(g, u, "add", cur);
    if (other == nullptr) continue;
    int pnum;
    if (other->opcode == "broadcast" && AttrDim(other->attrs, "dimensions", -1) == int64_t(cur->shape.dims.size()) - 1) {
      Instr* v = g.Operand(other, 0);
      if (v != nullptr && v->opcode == "convert") v = g.Operand(v, 0);      // f32 bias must be convert(bf16/f16)
      if (v != nullptr && AsParameter(v, &pnum) && v->shape.dims.size() == 1 && v->shape.dims[0] == plan->n &&
          (v->shape.type == "bf16" || v->shape.type == "f16" || (v->shape.type == "f32" && g.Operand(other, 0) == v))) {
        Source s;
        s.role = "bias"; s.param = pnum; s.shape = v->shape; s.instr = v->name;
        plan->operands.push_back(s);
        vector_bias = true;
        cur = u;
        break;
      }
    } else if (AsParameter(other, &pnum) && other->shape.dims == cur->shape.dims && g.Users(cur).size() == 1) {
      Source s;
      s.role = "c"; s.param = pnum; s.shape = other->shape; s.instr = other->name;
      plan->operands.insert(plan->operands.begin() + 2, s);                 // c sits at operand index 2
      plan->beta = 1.0;
      cur = u;
      break;
    }
  }
  // -- ReLU: maximum(x, broadcast(0))
  if (Instr* mx = UserWith(g, cur, "maximum", [&](Instr* o) { return IsConstantNear(g, o, 0.0, 0.0); })) {
    if (g.Users(cur).size() == 1) { relu = true; cur = mx; }
  }
  // -- GELU, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  if (!relu) {
    Instr* x = cur;
    Instr* x2 = UserWith(g, x, "multiply", [&](Instr* o) { return o == x; });
    Instr* x3 = x2 ? UserWith(g, x, "multiply", [&](Instr* o) { return o == x2; }) : nullptr;
    Instr* t0 = x3 ? UserWith(g, x3, "multiply", [&](Instr* o) { return IsConstantNear(g, o, 0.044715); }) : nullptr;
    Instr* t1 = t0 ? UserWith(g, x, "add", [&](Instr* o) { return o == t0; }) : nullptr;
    Instr* t2 = t1 ? UserWith(g, t1, "multiply", [&](Instr* o) { return IsConstantNear(g, o, 0.7978845608); }) : nullptr;
    Instr* th = nullptr;
    if (t2) for (Instr* u : g.Users(t2)) if (u->opcode == "tanh") th = u;
    Instr* t3 = th ? UserWith(g, th, "add", [&](Instr* o) { return IsConstantNear(g, o, 1.0); }) : nullptr;
    Instr* cdf = t3 ? UserWith(g, t3, "multiply", [&](Instr* o) { return IsConstantNear(g, o, 0.5); }) : nullptr;
    Instr* out = cdf ? UserWith(g, x, "multiply", [&](Instr* o) { return o == cdf; }) : nullptr;
    // The pre-activation may have no users besides the GELU pattern itself (otherwise the
    // reference needs the GELU_AUX epilogue, gemm_rewriter.cc:2190-2192).
    if (out != nullptr && g.Users(x).size() == 4) { gelu = true; cur = out; }
  }
  // DEFAULT 0, BIAS 1, RELU 2, BIAS_RELU 3, GELU 4, BIAS_GELU 6 (backend_configs.proto:106-117)
  plan->epilogue = gelu ? (vector_bias ? 6 : 4) : relu ? (vector_bias ? 3 : 2) : (vector_bias ? 1 : 0);

  // -- amax = reduce-max(abs(x)) (abs optional after ReLU), F8AddDAmax
  Instr* amax = nullptr;
  for (Instr* u : g.Users(cur)) {
    Instr* red = nullptr;
    if (u->opcode == "abs") { for (Instr* uu : g.Users(u)) if (uu->opcode == "reduce") red = uu; }
    else if (u->opcode == "reduce" && relu) red = u;
    if (red != nullptr && red->shape.IsScalar()) {
      double init;
      if (ScalarConstant(g, g.Operand(red, 1), &init) && init <= 0.0) amax = red;
    }
  }
  // -- scaled, saturating FP8 output: [divide | multiply by broadcast(scale)] -> clamp(+-max) -> convert(f8)
  Instr* d = cur;
  for (Instr* u : g.Users(cur)) {
    Instr* scaled = nullptr;
    Instr* scale = nullptr;
    bool divide = false;
    Instr* clamp = nullptr;
    if (u->opcode == "divide" || u->opcode == "multiply") {
      Instr* other = OtherOperand(g, u, u->opcode.c_str(), cur);
      scale = BroadcastedScalar(g, other);
      if (scale == nullptr || (u->opcode == "divide" && g.Operand(u, 0) != cur)) continue;
      divide = u->opcode == "divide";
      scaled = u;
      for (Instr* uu : g.Users(scaled)) if (uu->opcode == "clamp" && g.Operand(uu, 1) == scaled) clamp = uu;
    } else if (u->opcode == "clamp" && g.Operand(u, 1) == cur) {
      clamp = u;
    }
    if (clamp == nullptr) continue;
    Instr* conv = nullptr;
    for (Instr* uu : g.Users(clamp)) if (uu->opcode == "convert" && IsF8(uu->shape.type)) conv = uu;
    if (conv == nullptr) continue;
    const double mx = F8Max(conv->shape.type);
    if (!IsConstantNear(g, g.Operand(clamp, 0), -mx, 0.0) || !IsConstantNear(g, g.Operand(clamp, 2), mx, 0.0)) continue;
    Source s;
    std::string why;
    if (!ScaleSource(g, scale, divide, "d_scale", &s, &why)) continue;
    plan->operands.push_back(s);
    d = conv;
    break;
  }
  if (!IsF8(d->shape.type) && !gelu && !vector_bias && plan->beta == 0.0 && g.Users(cur).size() == 1 &&
      plan->operands.size() >= 4 && plan->operands[2].param < 0 && plan->operands[2].constant == 1.0 && !plan->operands[2].reciprocal) {
    // F8ScaleD (gemm_rewriter.cc:1593-1633): the output is scaled by a scalar but NOT cast to FP8.  The factor is
    // forwarded as a_scale -- only when no input scale was fused there (a_scale is still the constant 1), the
    // epilogue is DEFAULT or RELU and no matrix bias was fused.
    Instr* u = g.Users(cur)[0];
    if (u->opcode == "multiply" || (u->opcode == "divide" && g.Operand(u, 0) == cur)) {
      Instr* scale = BroadcastedScalar(g, OtherOperand(g, u, u->opcode.c_str(), cur));
      Source sd;
      std::string why;
      if (scale != nullptr && ScaleSource(g, scale, u->opcode == "divide", "a_scale", &sd, &why)) {
        plan->operands[2] = sd;
        cur = u;
        d = u;
      }
    }
  }
  if (!IsF8(d->shape.type)) {
    amax = nullptr;   // amax is only produced together with an FP8 output (the delayed-scaling pattern)
    // A final narrowing convert of the f32 result simply becomes the custom call's output type.
    if (g.Users(cur).size() == 1 && g.Users(cur)[0]->opcode == "convert" &&
        (g.Users(cur)[0]->shape.type == "bf16" || g.Users(cur)[0]->shape.type == "f16"))
      d = g.Users(cur)[0];
  }
  plan->d_instr = d->name;
  plan->d_shape = d->shape;
  if (amax != nullptr) { plan->damax = true; plan->amax_instr = amax->name; }
}

Plan Decide(const Graph& g) {
  Plan plan;
  Instr* dot = nullptr;
  for (Instr& i : g.comp->instrs)
    if (i.opcode == "dot") { if (dot != nullptr) { plan.reason = "more than one dot"; return plan; } dot = &i; }
  if (dot == nullptr) { plan.reason = "no dot"; return plan; }
  Instr* lhs = g.Operand(dot, 0);
  Instr* rhs = g.Operand(dot, 1);
  const int64_t lc = AttrDim(dot->attrs, "lhs_contracting_dims", -2), rc = AttrDim(dot->attrs, "rhs_contracting_dims", -2);
  // Rank 2, or rank 3 with one leading batch dimension on both operands (the canonical batched form,
  // gemm_rewriter_fp8_test.cc:941-991).
  const bool has_batch = dot->attrs.find("batch_dims") != std::string::npos;
  const size_t rank = lhs ? lhs->shape.dims.size() : 0;
  const int64_t bo = has_batch ? 1 : 0;
  if (lhs == nullptr || rhs == nullptr || lc < bo || rc < bo || rank != size_t(2 + bo) || rhs->shape.dims.size() != rank ||
      lc > bo + 1 || rc > bo + 1 ||
      (has_batch && (AttrDim(dot->attrs, "lhs_batch_dims", -2) != 0 || AttrDim(dot->attrs, "rhs_batch_dims", -2) != 0 ||
                     lhs->shape.dims[0] != rhs->shape.dims[0]))) {
    plan.reason = "only dots of rank 2, or rank 3 with batch dimension 0 on both operands, with one contracting dimension each are handled";
    return plan;
  }
  plan.lhs_contracting = int(lc);
  plan.rhs_contracting = int(rc);
  plan.batch = has_batch ? lhs->shape.dims[0] : 0;
  plan.k = lhs->shape.dims[lc];
  plan.m = lhs->shape.dims[bo + (bo + 1 - lc)];
  plan.n = rhs->shape.dims[bo + (bo + 1 - rc)];

  if (lhs->shape.type == "s8" && rhs->shape.type == "s8" && dot->shape.type == "s32") {
    if (has_batch) { plan.reason = "batched integer dots are not handled"; return plan; }
    // Integer dot; optionally convert(f32) * broadcast(row scale) * broadcast(col scale) -> convert(bf16).
    int pa, pb;
    if (!AsParameter(lhs, &pa) || !AsParameter(rhs, &pb)) { plan.reason = "s8 operands must be parameters"; return plan; }
    plan.target = "b200$dot$s8";
    Source a; a.role = "a"; a.param = pa; a.shape = lhs->shape; a.instr = lhs->name;
    Source b; b.role = "b"; b.param = pb; b.shape = rhs->shape; b.instr = rhs->name;
    plan.operands = {a, b};
    plan.d_instr = dot->name;
    plan.d_shape = dot->shape;
    Instr* cf = nullptr;
    for (Instr* u : g.Users(dot)) if (u->opcode == "convert" && u->shape.type == "f32") cf = u;
    if (cf != nullptr && g.Users(dot).size() == 1) {
      auto scale_along = [&](Instr* x, int dim, Instr** next, Source* s) {
        for (Instr* u : g.Users(x)) {
          if (u->opcode != "multiply") continue;
          Instr* other = OtherOperand(g, u, "multiply", x);
          int pnum;
          if (other && other->opcode == "broadcast" && AttrDim(other->attrs, "dimensions", -1) == dim &&
              AsParameter(g.Operand(other, 0), &pnum) && g.Operand(other, 0)->shape.type == "f32") {
            s->param = pnum; s->shape = g.Operand(other, 0)->shape; s->instr = g.Operand(other, 0)->name;
            *next = u;
            return true;
          }
        }
        return false;
      };
      Instr* y0 = nullptr;
      Instr* y1 = nullptr;
      Source rs, cs;
      rs.role = "a_row_scale"; cs.role = "b_col_scale";
      if (scale_along(cf, 0, &y0, &rs) && scale_along(y0, 1, &y1, &cs)) {
        Instr* out = y1;
        for (Instr* u : g.Users(y1)) if (u->opcode == "convert" && u->shape.type == "bf16") out = u;
        plan.operands.push_back(rs);
        plan.operands.push_back(cs);
        plan.d_instr = out->name;
        plan.d_shape = out->shape;
      }
    }
    plan.rewritten = true;
    return plan;
  }

  Fp8Operand fa, fb;
  if (!MatchFp8Operand(g, lhs, &fa) || !MatchFp8Operand(g, rhs, &fb)) { plan.reason = "operands are not dequantised FP8 values"; return plan; }
  if (fa.f8->shape.type == "f8e5m2" && fb.f8->shape.type == "f8e5m2") { plan.reason = "both operands are f8e5m2"; return plan; }
  int pa, pb;
  if (!AsParameter(fa.f8, &pa) || !AsParameter(fb.f8, &pb)) { plan.reason = "FP8 operands must be parameters"; return plan; }
  plan.target = "b200$scaled_dot$f8";
  Source a; a.role = "a"; a.param = pa; a.shape = fa.f8->shape; a.instr = fa.f8->name;
  Source b; b.role = "b"; b.param = pb; b.shape = fb.f8->shape; b.instr = fb.f8->name;
  for (auto pr : {std::make_pair(&a, &fa), std::make_pair(&b, &fb)}) {
    if (!pr.second->reshaped) continue;
    if (!pr.first->shape.layout.empty() && !std::is_sorted(pr.first->shape.layout.rbegin(), pr.first->shape.layout.rend())) {
      plan.reason = "a reshaped operand must be in the default layout";
      return plan;
    }
    pr.first->shape.dims = pr.second->view.dims;
    pr.first->shape.layout.clear();
    pr.first->reshaped = true;
  }
  Source as, bs;
  if (!ScaleSource(g, fa.scale, fa.divide, "a_scale", &as, &plan.reason)) return plan;
  if (!ScaleSource(g, fb.scale, fb.divide, "b_scale", &bs, &plan.reason)) return plan;
  plan.operands = {a, b, as, bs};
  plan.d_instr = dot->name;
  plan.d_shape = dot->shape;
  MatchF8Epilogue(g, dot, &plan);
  if (plan.d_viewed) {
    // The call produces the [m, n] matrix; the module sees it in the shape of the view.  A matrix bias given in that
    // shape is the same bytes as an [m, n] matrix.
    plan.d_view = plan.d_shape;
    plan.d_view.layout.clear();
    plan.d_shape.dims = {plan.m, plan.n};
    plan.d_shape.layout.clear();
    for (Source& src : plan.operands) {
      if (src.role == "c" && src.shape.dims.size() != 2) {
        src.shape.dims = {plan.m, plan.n};
        src.shape.layout.clear();
        src.reshaped = true;
      }
    }
  }
  const std::string& dt = plan.d_shape.type;
  if (!(dt == "bf16" || dt == "f16" || dt == "f32" || IsF8(dt))) { plan.rewritten = false; plan.reason = "unsupported output type " + dt; return plan; }
  if (dt == "f8e5m2" && a.shape.type == "f8e4m3fn" && b.shape.type == "f8e4m3fn") { plan.reason = "e4m3 x e4m3 -> e5m2 is not in the supported type table"; return plan; }

  // Layouts (gemm_rewriter_fp8_test.cc:2825-2890 runs all 32 combinations).  The custom call takes row-major
  // buffers only: a column-major [r, c] operand IS the row-major [c, r] matrix, so it is passed as that with its
  // contracting dimension renumbered; a column-major result is D^T, obtained by swapping the operands
  // (MakeOutputColumnMajor's identity, xla/stream_executor/gpu/gpu_blas_lt.cc:271-287).
  if (plan.batch == 0) {
    auto as_row_major = [](Source* src, int* contracting) {
      std::swap(src->shape.dims[0], src->shape.dims[1]);
      src->shape.layout.clear();
      src->transposed = true;
      *contracting = 1 - *contracting;
    };
    if (plan.operands[0].shape.IsColumnMajor2D()) as_row_major(&plan.operands[0], &plan.lhs_contracting);
    if (plan.operands[1].shape.IsColumnMajor2D()) as_row_major(&plan.operands[1], &plan.rhs_contracting);
    if (plan.d_shape.IsColumnMajor2D()) {
      if (plan.epilogue != 0 || plan.beta != 0.0 || plan.damax || plan.operands.size() != 4) {
        plan.reason = "a column-major result is handled for the plain scaled dot only";
        return plan;
      }
      std::swap(plan.operands[0], plan.operands[1]);
      std::swap(plan.operands[2], plan.operands[3]);
      plan.operands[0].role = "a"; plan.operands[1].role = "b";
      plan.operands[2].role = "a_scale"; plan.operands[3].role = "b_scale";
      std::swap(plan.lhs_contracting, plan.rhs_contracting);
      std::swap(plan.m, plan.n);
      std::swap(plan.d_shape.dims[0], plan.d_shape.dims[1]);
      plan.d_shape.layout.clear();
      plan.d_transposed = true;
    }
  } else if (plan.operands[0].shape.IsColumnMajor2D() || !plan.d_shape.layout.empty() || !plan.operands[0].shape.layout.empty() ||
             !plan.operands[1].shape.layout.empty()) {
    bool default_layouts = true;
    for (const Shape* sh : {&plan.operands[0].shape, &plan.operands[1].shape, &plan.d_shape})
      for (size_t i = 0; i < sh->layout.size(); ++i) default_layouts = default_layouts && sh->layout[i] == int64_t(sh->layout.size() - 1 - i);
    if (!default_layouts) { plan.reason = "batched dots are handled in the default (row-major) layout only"; return plan; }
  }
  plan.rewritten = true;
  return plan;
}

}  // namespace


namespace {

std::string JsonStr(const std::string& s) {
  std::string o = "\"";
  for (char c : s) { if (c == '"' || c == '\\') o += '\\'; o += c; }
  return o + "\"";
}
std::string Dims(const Shape& s) {
  std::string o = "[";
  for (size_t i = 0; i < s.dims.size(); ++i) o += (i ? "," : "") + std::to_string(s.dims[i]);
  return o + "]";
}
std::string Num(double v) {
  char buf[64];
  snprintf(buf, sizeof buf, "%.17g", v);
  return buf;
}

// A value that must stay floating point when parsed back (JSON readers turn "1" into an integer).
std::string F64(double v) {
  std::string s = Num(v);
  if (s.find_first_of(".einf") == std::string::npos) s += ".0";
  return s;
}

constexpr int64_t kWorkspaceBytes = 32ll * 1024 * 1024;   // GemmConfig::kHopperWorkspace, matmul_utils.h:103

bool Emit(const Module& m, const Graph& g, Plan* plan, std::string* hlo, std::string* json) {
  // Where the results land in the module's output.
  Instr* root = g.root;
  std::vector<std::string> root_elems;
  if (root->opcode == "tuple") root_elems = root->operands;
  else root_elems = {root->name};
  for (size_t i = 0; i < root_elems.size(); ++i) {
    if (root_elems[i] == plan->d_instr) plan->d_root_index = int(i);
    else if (plan->damax && root_elems[i] == plan->amax_instr) plan->amax_root_index = int(i);
    else { plan->rewritten = false; plan->reason = "the module's output uses a value the custom call does not produce: " + root_elems[i]; return false; }
  }
  if (plan->d_root_index < 0) { plan->rewritten = false; plan->reason = "the dot's result is not an output of the module"; return false; }

  std::ostringstream o;
  o << "HloModule " << (m.name.empty() ? "module" : m.name) << "_rewritten\n\n";
  o << "ENTRY main {\n";
  for (const Instr& i : g.comp->instrs)
    if (i.opcode == "parameter") o << "  " << i.name << " = " << i.shape.ToString() << " parameter(" << i.literal << ")\n";
  std::vector<std::string> op_names;
  int tmp = 0;
  for (const Source& s : plan->operands) {
    if (s.param < 0) {
      const std::string n = s.role + "_const" + std::to_string(tmp++);
      o << "  " << n << " = f32[] constant(" << Num(s.constant) << ")\n";
      op_names.push_back(n);
    } else if (s.reciprocal) {
      const std::string one = "one" + std::to_string(tmp++), n = s.role + "_inv";
      o << "  " << one << " = f32[] constant(1)\n";
      o << "  " << n << " = f32[] divide(" << one << ", " << s.instr << ")\n";
      op_names.push_back(n);
    } else if (s.reshaped && !s.transposed) {
      const std::string n = s.role + "_view";
      o << "  " << n << " = " << s.shape.ToString() << " bitcast(" << s.instr << ")\n";
      op_names.push_back(n);
    } else if (s.transposed) {
      const std::string n = s.role + "_rm";          // the same bytes, read as the row-major matrix they are
      o << "  " << n << " = " << s.shape.ToString() << "{1,0} bitcast(" << s.instr << ")\n";
      op_names.push_back(n);
    } else {
      op_names.push_back(s.instr);
    }
  }
  // Operands whose dimensions are not multiples of 16 are zero-padded and the result is sliced back
  // (PadOperandToMultipleOf16 / PadShapeToMultipleOf16, gemm_rewriter.cc:1556-1580).  Zero rows and
  // columns add nothing to the dot, a zero bias entry keeps act(0) = 0 out of amax.
  auto round16 = [](int64_t v) { return (v + 15) / 16 * 16; };
  bool padded = false;
  for (size_t i = 0; i < plan->operands.size(); ++i) {
    Source& s = plan->operands[i];
    s.padded = s.shape;
    {
      const size_t first = (plan->batch > 0 && s.padded.dims.size() == 3) ? 1 : 0;      // the batch dimension stays
      for (size_t d = first; d < s.padded.dims.size(); ++d) s.padded.dims[d] = round16(s.padded.dims[d]);
    }
    if (s.padded.dims == s.shape.dims) continue;
    padded = true;
    const std::string z = "zero" + std::to_string(tmp++), n = s.role + "_pad";
    o << "  " << z << " = " << s.shape.type << "[] constant(0)\n";
    o << "  " << n << " = " << s.padded.ToString() << " pad(" << op_names[i] << ", " << z << "), padding=";
    for (size_t d = 0; d < s.shape.dims.size(); ++d) o << (d ? "x" : "") << "0_" << (s.padded.dims[d] - s.shape.dims[d]);
    o << "\n";
    op_names[i] = n;
  }
  plan->d_padded = plan->d_shape;
  for (size_t d = plan->batch > 0 ? 1 : 0; d < plan->d_padded.dims.size(); ++d) plan->d_padded.dims[d] = round16(plan->d_padded.dims[d]);
  const Shape d_logical = plan->d_shape;
  const bool f8 = plan->target == "b200$scaled_dot$f8";
  std::string tuple_shape = "(" + plan->d_padded.ToString();
  if (plan->damax) tuple_shape += ", f32[]";
  tuple_shape += ", s8[" + std::to_string(kWorkspaceBytes) + "]";   // appended to every cuBLASLt matmul, FP8 or not
  tuple_shape += ")";
  o << "  cc = " << tuple_shape << " custom-call(";
  for (size_t i = 0; i < op_names.size(); ++i) o << (i ? ", " : "") << op_names[i];
  o << "), custom_call_target=\"" << plan->target << "\", api_version=API_VERSION_TYPED_FFI, backend_config={";
  if (f8) {
    o << "alpha_real = " << F64(plan->alpha) << " : f64, beta = " << F64(plan->beta) << " : f64, epilogue = " << plan->epilogue
      << " : i32, lhs_contracting_dim = " << plan->lhs_contracting << " : i64, rhs_contracting_dim = " << plan->rhs_contracting
      << " : i64, damax_output = " << (plan->damax ? "true" : "false")
      << (plan->batch > 0 ? ", lhs_batch_dims = array<i64: 0>, rhs_batch_dims = array<i64: 0>" : "") << ", selected_config = 0 : i64}\n";
  } else {
    o << "lhs_contracting_dim = " << plan->lhs_contracting << " : i64, rhs_contracting_dim = " << plan->rhs_contracting
      << " : i64, emit_s32 = false}\n";
  }
  const std::string dn = plan->d_viewed ? "d_mat" : "d";      // the [m, n] result; `d` is what the module sees
  if (padded || plan->d_padded.dims != d_logical.dims) {
    o << "  d_full = " << plan->d_padded.ToString() << " get-tuple-element(cc), index=0\n";
    o << "  " << dn << " = " << d_logical.ToString() << " slice(d_full), slice={";
    for (size_t d = 0; d < d_logical.dims.size(); ++d) o << (d ? ", " : "") << "[0:" << d_logical.dims[d] << "]";
    o << "}\n";
  } else if (plan->d_transposed) {
    Shape logical = plan->d_shape;
    std::swap(logical.dims[0], logical.dims[1]);
    logical.layout = {0, 1};
    o << "  d_t = " << plan->d_shape.ToString() << " get-tuple-element(cc), index=0\n";
    o << "  " << dn << " = " << logical.ToString() << " bitcast(d_t)\n";
  } else {
    o << "  " << dn << " = " << plan->d_shape.ToString() << " get-tuple-element(cc), index=0\n";
  }
  if (plan->d_viewed) o << "  d = " << plan->d_view.ToString() << " bitcast(d_mat)\n";
  if (plan->damax) o << "  amax = f32[] get-tuple-element(cc), index=1\n";
  if (root->opcode == "tuple") {
    o << "  ROOT out = " << root->shape.ToString() << " tuple(";
    for (size_t i = 0; i < root_elems.size(); ++i) o << (i ? ", " : "") << (int(i) == plan->d_root_index ? "d" : "amax");
    o << ")\n";
  } else {
    o << "  ROOT out = " << root->shape.ToString() << " copy(d)\n";
  }
  o << "}\n";
  *hlo = o.str();

  std::ostringstream j;
  j << "{\"rewritten\": true, \"target\": " << JsonStr(plan->target) << ", \"m\": " << plan->m << ", \"n\": " << plan->n
    << ", \"k\": " << plan->k << ", \"operands\": [";
  for (size_t i = 0; i < plan->operands.size(); ++i) {
    const Source& s = plan->operands[i];
    j << (i ? ", " : "") << "{\"role\": " << JsonStr(s.role) << ", \"param\": " << s.param << ", \"reciprocal\": "
      << (s.reciprocal ? "true" : "false") << ", \"constant\": " << Num(s.constant) << ", \"dtype\": " << TypeCode(s.shape.type)
      << ", \"dims\": " << Dims(s.shape) << ", \"padded_dims\": " << Dims(s.padded) << ", \"transposed\": "
      << (s.transposed ? "true" : "false") << ", \"reshaped\": " << (s.reshaped ? "true" : "false") << "}";
  }
  j << "], \"results\": [{\"role\": \"d\", \"dtype\": " << TypeCode(plan->d_shape.type) << ", \"dims\": " << Dims(plan->d_shape)
    << ", \"padded_dims\": " << Dims(plan->d_padded) << ", \"transposed\": " << (plan->d_transposed ? "true" : "false")
    << ", \"view_dims\": " << (plan->d_viewed ? Dims(plan->d_view) : std::string("null")) << ", \"root_index\": " << (root->opcode == "tuple" ? plan->d_root_index : -1) << "}";
  if (plan->damax) j << ", {\"role\": \"amax\", \"dtype\": 11, \"dims\": [], \"root_index\": " << plan->amax_root_index << "}";
  j << ", {\"role\": \"workspace\", \"dtype\": 2, \"dims\": [" << kWorkspaceBytes << "], \"root_index\": -2}";
  j << "], \"attrs\": {\"alpha_real\": " << F64(plan->alpha) << ", \"beta\": " << F64(plan->beta) << ", \"epilogue\": " << plan->epilogue
    << ", \"lhs_contracting_dim\": " << plan->lhs_contracting << ", \"rhs_contracting_dim\": " << plan->rhs_contracting
    << ", \"damax_output\": " << (plan->damax ? "true" : "false")
    << (plan->batch > 0 ? ", \"lhs_batch_dims\": [0], \"rhs_batch_dims\": [0]" : "") << "}, \"batch\": " << plan->batch << "}";
  *json = j.str();
  return true;
}

int Copy(const std::string& s, char* out, size_t len) {
  if (out == nullptr || len == 0) return 0;
  if (s.size() + 1 > len) return 8;   // RESOURCE_EXHAUSTED
  std::memcpy(out, s.c_str(), s.size() + 1);
  return 0;
}

}  // namespace

// Rewrites the scaled-dot pattern of an HLO module (text) onto this library's custom call.
// Returns 0 when the text was understood -- whether or not anything was rewritten: `plan_json`
// then says {"rewritten": false, "reason": ...} and `out_hlo` repeats the input -- 3 on text it
// cannot parse, 8 when an output buffer is too small.
extern "C" int b200sd_rewrite_hlo(const char* hlo_text, char* out_hlo, size_t out_hlo_len, char* plan_json,
                                  size_t plan_json_len, char* err, size_t err_len) {
  auto fail = [&](int code, const std::string& msg) {
    if (err != nullptr && err_len > 0) snprintf(err, err_len, "%s", msg.c_str());
    return code;
  };
  if (hlo_text == nullptr) return fail(3, "hlo_text is null");
  Module m;
  std::string perr;
  if (!ParseModule(hlo_text, &m, &perr)) return fail(3, perr);
  Computation* entry = nullptr;
  for (Computation& c : m.computations) if (c.is_entry) entry = &c;
  Graph g(entry);
  for (const Instr& i : entry->instrs)
    for (const std::string& o : i.operands)
      if (g.Get(o) == nullptr) return fail(3, "instruction " + i.name + " uses an undefined value " + o);
  Plan plan = Decide(g);
  std::string hlo, json;
  if (plan.rewritten) Emit(m, g, &plan, &hlo, &json);
  if (!plan.rewritten) {
    hlo = hlo_text;
    json = "{\"rewritten\": false, \"reason\": " + JsonStr(plan.reason) + "}";
  }
  if (int rc = Copy(hlo, out_hlo, out_hlo_len)) return fail(rc, "out_hlo buffer too small");
  if (int rc = Copy(json, plan_json, plan_json_len)) return fail(rc, "plan_json buffer too small");
  if (err != nullptr && err_len > 0) err[0] = '\0';
  return 0;
}

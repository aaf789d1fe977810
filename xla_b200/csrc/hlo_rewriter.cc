// Rewriter-lite: the decisions of XLA's GemmRewriter for the quantized scaled dot, restated as a
// rewrite over HLO text, emitting this library's custom-call targets instead of
// "__cublas$lt$matmul$f8" / "__cublas$lt$matmul".
//
// Like the reference (xla/backends/gpu/transforms/gemm_rewriter.cc) it works bottom-up over the entry
// computation: every dot is visited first (HandleDot, :657-779), then the instructions behind it fold
// into the call one at a time.
//   * MatchFp8Param / FindF8SubgraphRecursive (:190-336): from a dot operand back to an FP8 value
//     through a convert, an optional multiply / divide by a broadcast scalar, and any number of ops
//     that commute with the dequantisation (bitcast, broadcast, copy, dynamic-slice, pad, reshape,
//     select against zero, slice, transpose), which are re-applied to the FP8 value itself.
//   * CreateF8CustomCall (:1235-1591): e4m3fn / e5m2 operands but not both e5m2; scales become f32
//     scalar operands (inverted when the HLO divides, constant 1 when absent); one contracting and one
//     non-contracting dimension per operand; operands padded to multiples of 16, result sliced back.
//     No transposes are inserted (the Blackwell branch, :1535-1554): a buffer is handed over as the
//     row-major matrix it physically is and transposition is expressed by the contracting dimension; a
//     column-major result is computed as D^T by swapping the operands (MakeOutputColumnMajor's identity,
//     xla/stream_executor/gpu/gpu_blas_lt.cc:271-287).  Only when the batch dimensions are not the
//     major-most dimensions of a buffer is a transpose needed.
//   * HandleMultiply / HandleDivide (:888-1061): alpha, the output scale without an FP8 cast (F8ScaleD,
//     :1593-1633), tanh-GELU; HandleAdd (:1063-1189) with FuseVectorBiasAdd (:1987-2124) and
//     FuseMatrixBiasAdd (:1829-1978); HandleMaximum / FuseReluActivation (:2126-2164); HandleConvert with
//     F8ConvertD / F8AddDAmax (:1635-1794).
//   * GemmWorkspaceRewriteVisitor (:2774-2892): a trailing s8[32 MiB] workspace result on every call.
//   * The s8 x s8 -> s32 dot goes to the integer target; unlike the reference (which refuses to fuse
//     into S32 gemms, :897-901, :1838-1842) the per-row x per-column dequantisation behind it is folded
//     in too.  Also beyond the reference: a narrowing convert (f32 -> bf16 / f16) right behind a call
//     becomes the call's output type.
// Dots that do not match stay as they are and the reason is reported.
//
// Output: the rewritten module as HLO text and a JSON description of the custom calls.
#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <string>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------------ IR
struct Shape {
  std::string type;                 // "f32", "f8e4m3fn", ... or "tuple"
  std::vector<int64_t> dims;
  std::vector<Shape> elements;      // for tuples
  std::vector<int64_t> layout;      // minor_to_major as written; empty = default (row-major)

  std::vector<int64_t> MinorToMajor() const {
    if (!layout.empty()) return layout;
    std::vector<int64_t> l(dims.size());
    for (size_t i = 0; i < l.size(); ++i) l[i] = int64_t(l.size()) - 1 - int64_t(i);
    return l;
  }
  // Logical dimension numbers from the major-most to the minor-most one in memory.
  std::vector<int64_t> Physical() const {
    std::vector<int64_t> l = MinorToMajor();
    std::reverse(l.begin(), l.end());
    return l;
  }
  bool IsDefaultLayout() const {
    const std::vector<int64_t> l = MinorToMajor();
    for (size_t i = 0; i < l.size(); ++i)
      if (l[i] != int64_t(l.size()) - 1 - int64_t(i)) return false;
    return true;
  }
  bool IsScalar() const { return type != "tuple" && dims.empty(); }
  std::string ToString() const {
    if (type == "tuple") {
      std::string s = "(";
      for (size_t i = 0; i < elements.size(); ++i) s += (i ? ", " : "") + elements[i].ToString();
      return s + ")";
    }
    std::string s = type + "[";
    for (size_t i = 0; i < dims.size(); ++i) s += (i ? "," : "") + std::to_string(dims[i]);
    s += "]";
    if (!layout.empty() && !IsDefaultLayout()) {
      s += "{";
      for (size_t i = 0; i < layout.size(); ++i) s += (i ? "," : "") + std::to_string(layout[i]);
      s += "}";
    }
    return s;
  }
};

Shape MakeShape(const std::string& type, std::vector<int64_t> dims) {
  Shape s;
  s.type = type;
  s.dims = std::move(dims);
  return s;
}

struct Instr;

// What a custom call of this library carries besides its operands: the GemmBackendConfig fields
// (xla/service/gpu/backend_configs.proto:88-135) this path reads, and which optional operands /
// results are present.  Operand order (xla/service/gpu/thunk_emitter.cc:776-862):
// a, b, [c], a_scale, b_scale, [bias], [d_scale];  integer target: a, b, [a_row_scale, b_col_scale].
struct Gemm {
  bool f8 = true;
  double alpha = 1.0, beta = 0.0;
  int epilogue = 0;                    // GemmBackendConfig.Epilogue number (DEFAULT = 0)
  bool damax = false, emit_s32 = false;
  int lhs_contracting = 1, rhs_contracting = 0;   // in the index space of the operands as passed
  bool batched = false;
  int64_t batch = 0, m = 0, n = 0, k = 0;         // logical (unpadded) extents; m x n is the result AS COMPUTED
  bool has_c = false, has_bias = false, has_d_scale = false, has_dequant = false;
  bool swapped = false;                // operands were exchanged to produce a column-major result as D^T
  int64_t explicit_block = 0;          // MX: the block size the source call states in its backend config (0: implied by the shapes)
  bool mx = false;                     // MX block-scaled dot: operands a, b, a_scale, b_scale (thunk_emitter.cc:939-988)
  Instr* amax = nullptr;               // the f32[] second result, when damax
  Instr* acc = nullptr;                // the s32 second result, when emit_s32
  size_t ScaleIndex() const { return has_c ? 3 : 2; }
};

struct Instr {
  std::string name;
  Shape shape;
  std::string opcode;
  std::vector<Instr*> operands;
  std::vector<std::string> operand_names;   // as parsed, before resolution
  std::vector<std::string> nested;          // operands written as whole instructions, to be parsed in front of this one
  std::string attrs;                // everything after the closing parenthesis, verbatim
  std::string literal;              // constant(...) / parameter(...) payload
  bool is_root = false;
  std::unique_ptr<Gemm> gemm;       // set on custom calls created here
};

struct Computation {
  std::string name;
  bool is_entry = false;
  std::vector<std::unique_ptr<Instr>> instrs;
  std::string raw;                  // original text, re-emitted verbatim for non-entry computations
};

struct Module {
  std::string name;
  std::vector<Computation> computations;
};

// ------------------------------------------------------------------------------------------ parsing
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
      if (p >= text.size()) return false;
      if (text[p] == ')') { ++p; break; }
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
    else if (isdigit(static_cast<unsigned char>(text[p]))) num += text[p];
    else if (text[p] != ' ') return false;
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
      else if (text[p] == ':') { while (p < text.size() && text[p] != '}') ++p; break; }   // tiling etc.: ignored
      ++p;
    }
    if (!v.empty()) out->layout.push_back(std::stoll(v));
    if (p < text.size()) ++p;
    if (out->layout.size() != out->dims.size()) out->layout.clear();
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
  {
    // The shape may be left out ("out = add(a, b)"): it is then taken from the first operand.
    const size_t paren = line.find('(', p), bracket = line.find('[', p);
    const bool has_shape = line[line.find_first_not_of(' ', p)] == '(' || (bracket != std::string::npos && bracket < paren);
    if (has_shape) {
      if (!ParseShape(line, &p, &in->shape)) { *err = "bad shape in: " + line; return false; }
    } else {
      in->shape.type = "?";
    }
  }
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
      if (c == ',' && d == 0) { in->operand_names.push_back(Trim(cur)); cur.clear(); }
      else cur += c;
    }
    if (!Trim(cur).empty()) in->operand_names.push_back(Trim(cur));
    for (size_t i = 0; i < in->operand_names.size(); ++i) {
      // An operand spelled as an instruction of its own, "f16[8] multiply(%a, %b)": the caller parses it as a
      // separate instruction under a made-up name.
      std::string& o = in->operand_names[i];
      if (!o.empty() && o.back() == ')') {
        const std::string nested_name = in->name + ".operand" + std::to_string(i);
        in->nested.emplace_back(nested_name + " = " + o);
        o = nested_name;
      }
    }
    for (std::string& o : in->operand_names) {            // "f32[4] %x" or "%x" or "x"
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
  // Instructions may run over several lines: a line that neither starts an instruction ("x = ..."),
  // nor opens or closes a computation, continues the line before it.
  std::vector<std::string> lines;
  {
    std::istringstream ss(text);
    std::string line;
    while (std::getline(ss, line)) {
      size_t c = line.find("//");
      if (c != std::string::npos) line = line.substr(0, c);
      const std::string t = Trim(line);
      if (t.empty()) continue;
      const bool header = t.rfind("HloModule", 0) == 0;
      const size_t eq = t.find(" = "), paren = t.find('(');
      const bool starts_instr = eq != std::string::npos && (paren == std::string::npos || eq < paren);
      const bool opens = !header && !starts_instr && t.back() == '{';
      const bool closes = t == "}";
      if (header || opens || closes || starts_instr || lines.empty()) lines.push_back(t);
      else lines.back() += " " + t;
    }
  }
  Computation* cur = nullptr;
  for (std::string t : lines) {
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
      cur->raw = t + "\n";
      continue;
    }
    if (t == "}") { cur->raw += "}\n"; cur = nullptr; continue; }
    bool closes_after = false;
    if (t.size() > 1 && t.back() == '}' && std::count(t.begin(), t.end(), '{') < std::count(t.begin(), t.end(), '}')) {
      t = Trim(t.substr(0, t.size() - 1));                 // an instruction followed by the computation's closing brace
      closes_after = true;
    }
    cur->raw += "  " + t + "\n";
    // Operands written as nested instructions come out as instructions of their own, in front of their user.
    std::function<bool(const std::string&)> add = [&](const std::string& line) {
      auto in = std::make_unique<Instr>();
      if (!ParseInstr(line, in.get(), err)) return false;
      for (const std::string& inner : in->nested)
        if (!add(inner)) return false;
      in->nested.clear();
      cur->instrs.push_back(std::move(in));
      return true;
    };
    if (!add(t)) return false;
    if (closes_after) { cur->raw += "}\n"; cur = nullptr; }
  }
  if (m->computations.empty()) { *err = "module has no computation"; return false; }
  bool has_entry = false;
  for (const Computation& c : m->computations) has_entry = has_entry || c.is_entry;
  if (!has_entry) m->computations.back().is_entry = true;      // a module given as a single computation
  return true;
}

std::vector<int64_t> AttrList(const std::string& attrs, const std::string& key) {
  std::vector<int64_t> out;
  size_t p = attrs.find(key + "={");
  if (p == std::string::npos) return out;
  p += key.size() + 2;
  size_t e = attrs.find('}', p);
  std::string cur;
  for (size_t i = p; i < e && i < attrs.size(); ++i) {
    if (attrs[i] == ',') { if (!Trim(cur).empty()) out.push_back(std::stoll(cur)); cur.clear(); }
    else cur += attrs[i];
  }
  if (!Trim(cur).empty()) out.push_back(std::stoll(cur));
  return out;
}

bool IsF8(const std::string& t) { return t == "f8e4m3fn" || t == "f8e5m2"; }
bool IsAnyF8(const std::string& t) { return t.rfind("f8", 0) == 0; }
double F8Max(const std::string& t) { return t == "f8e4m3fn" ? 448.0 : 57344.0; }
int TypeCode(const std::string& t) {       // xla::PrimitiveType numbers
  static const std::map<std::string, int> k = {{"pred", 1}, {"s8", 2}, {"s32", 4}, {"f16", 10}, {"f32", 11}, {"bf16", 16},
                                               {"f8e5m2", 19}, {"f8e4m3fn", 20}, {"f8e8m0fnu", 33}};
  auto it = k.find(t);
  return it == k.end() ? 0 : it->second;
}
int64_t Round16(int64_t v) { return (v + 15) / 16 * 16; }

std::string JoinInts(const std::vector<int64_t>& v, const char* sep = ",") {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) s += (i ? sep : "") + std::to_string(v[i]);
  return s;
}

constexpr int64_t kWorkspaceBytes = 32ll * 1024 * 1024;   // GemmConfig::kHopperWorkspace, matmul_utils.h:103

// ------------------------------------------------------------------------------------------ the rewriter
class Rewriter {
 public:
  Rewriter(Computation* c, const std::vector<Computation>* all) : comp_(c), all_(all) {
    for (auto& i : c->instrs) {
      names_.insert(i->name);
      if (i->is_root) root_ = i.get();
    }
    if (root_ == nullptr && !c->instrs.empty()) root_ = c->instrs.back().get();
  }

  bool Resolve(std::string* err) {
    std::map<std::string, Instr*> by_name;
    for (auto& i : comp_->instrs) by_name[i->name] = i.get();
    for (auto& i : comp_->instrs) {
      for (const std::string& o : i->operand_names) {
        auto it = by_name.find(o);
        if (it == by_name.end()) { *err = "instruction " + i->name + " uses an undefined value " + o; return false; }
        i->operands.push_back(it->second);
      }
      if (i->shape.type == "?") {
        if (i->operands.empty() || i->operands[0]->shape.type == "?") { *err = "instruction " + i->name + " has no shape"; return false; }
        i->shape = i->operands[0]->shape;
      }
    }
    return true;
  }

  void Run() {
    std::vector<Instr*> order;
    for (auto& i : comp_->instrs) order.push_back(i.get());
    for (Instr* i : order) {
      if (!IsLive(i)) continue;
      if (i->opcode == "dot") HandleDot(i);
      else if (i->opcode == "multiply") HandleMultiply(i);
      else if (i->opcode == "divide") HandleDivide(i);
      else if (i->opcode == "add") HandleAdd(i);
      else if (i->opcode == "maximum") HandleMaximum(i);
      else if (i->opcode == "convert") HandleConvert(i);
      else if (i->opcode == "custom-call" && i->attrs.find("\"__op$block_scaled_dot\"") != std::string::npos) HandleBlockScaledDot(i);
      else if (i->opcode == "scaled-dot") HandleScaledDot(i);
    }
    for (Instr* g : calls_) {
      if (!IsLive(g) || g->gemm->mx) continue;
      if (!g->gemm->f8) FoldInt8Dequantisation(g);
      FoldNarrowingConvert(g);
    }
  }

  std::string EmitHlo(const Module& m) const;
  std::string EmitJson() const;
  bool AnyRewritten() const {
    for (Instr* g : calls_) if (IsLive(g)) return true;
    return false;
  }

 private:
  // ---- graph ----
  Instr* Add(const std::string& opcode, const Shape& shape, std::vector<Instr*> operands, const std::string& attrs = "",
             const std::string& literal = "", const std::string& hint = "") {
    auto in = std::make_unique<Instr>();
    std::string base = hint.empty() ? opcode : hint;
    for (char& c : base) if (c == '-') c = '_';
    std::string name = base;
    for (int n = 1; names_.count(name); ++n) name = base + "." + std::to_string(n);
    names_.insert(name);
    in->name = name;
    in->shape = shape;
    in->opcode = opcode;
    in->operands = std::move(operands);
    in->attrs = attrs;
    in->literal = literal;
    Instr* p = in.get();
    comp_->instrs.push_back(std::move(in));
    dirty_ = true;
    return p;
  }
  void Replace(Instr* old_i, Instr* new_i) {
    if (old_i == new_i) return;
    for (auto& i : comp_->instrs)
      for (Instr*& o : i->operands)
        if (o == old_i && i.get() != new_i) o = new_i;
    if (root_ == old_i) root_ = new_i;
    dirty_ = true;
  }
  void Refresh() const {
    if (!dirty_) return;
    live_.clear();
    users_.clear();
    std::vector<Instr*> stack = {root_};
    while (!stack.empty()) {
      Instr* i = stack.back();
      stack.pop_back();
      if (!live_.insert(i).second) continue;
      std::set<Instr*> seen;
      for (Instr* o : i->operands) {
        if (seen.insert(o).second) users_[o].push_back(i);
        stack.push_back(o);
      }
    }
    dirty_ = false;
  }
  bool IsLive(Instr* i) const { Refresh(); return live_.count(i) != 0; }
  const std::vector<Instr*>& Users(Instr* i) const {
    Refresh();
    static const std::vector<Instr*> none;
    auto it = users_.find(i);
    return it == users_.end() ? none : it->second;
  }
  // Users of the value, not counting the call's own extra-result instructions; being the root counts as one.
  std::vector<Instr*> ValueUsers(Instr* i) const {
    std::vector<Instr*> out;
    for (Instr* u : Users(i)) if (u->opcode != "gemm-amax" && u->opcode != "gemm-acc") out.push_back(u);
    return out;
  }
  size_t UserCount(Instr* i) const { return ValueUsers(i).size() + (i == root_ ? 1 : 0); }

  // ---- small matchers ----
  static Instr* BroadcastOperand(Instr* x) { return (x && x->opcode == "broadcast" && x->operands.size() == 1) ? x->operands[0] : nullptr; }
  static bool ConstantValue(Instr* x, double* v) {
    if (x == nullptr || x->opcode != "constant" || !x->shape.IsScalar()) return false;
    const std::string& l = x->literal;
    if (l == "inf") { *v = INFINITY; return true; }
    if (l == "-inf") { *v = -INFINITY; return true; }
    char* end = nullptr;
    *v = std::strtod(l.c_str(), &end);
    return end != l.c_str();
  }
  static bool BcastConst(Instr* x, double* v) {           // broadcast(constant scalar)
    Instr* s = BroadcastOperand(x);
    return s != nullptr && ConstantValue(s, v);
  }
  static bool BcastConstNear(Instr* x, double want, double rel = 1e-5) {
    double v;
    return BcastConst(x, &v) && std::fabs(v - want) <= rel * std::max(1.0, std::fabs(want));
  }
  // A call this pass made that may still absorb users (the MX call takes no epilogue, thunk_emitter.cc:939-988).
  static bool IsGemm(Instr* x) { return x != nullptr && x->gemm != nullptr && !x->gemm->mx; }
  static bool IsF8Gemm(Instr* x) { return IsGemm(x) && x->gemm->f8; }
  static Instr* Other(Instr* bin, Instr* a) {             // binary op with operands {a, other} in any order -> other
    if (bin->operands.size() != 2) return nullptr;
    if (bin->operands[0] == a) return bin->operands[1];
    if (bin->operands[1] == a) return bin->operands[0];
    return nullptr;
  }
  Instr* ConstantScalar(const std::string& type, const std::string& literal, const std::string& hint) {
    return Add("constant", MakeShape(type, {}), {}, "", literal, hint);
  }
  void Refuse(Instr* dot, const std::string& why) { refusals_.push_back({dot->name, why}); }

  // ---- MatchFp8Param ----
  struct Fp8Param {
    Instr* fp8 = nullptr;
    Instr* scale = nullptr;
    bool mult_scale = false;
    std::vector<std::pair<Instr*, int>> commutative;     // (op, index of the operand that leads back to the FP8 value)
  };
  bool FindF8Subgraph(Instr* x, std::set<Instr*>* visited, std::vector<std::pair<Instr*, int>>* path) {
    if (!visited->insert(x).second) return false;
    if (IsAnyF8(x->shape.type)) { path->push_back({x, -1}); return true; }
    const std::string& op = x->opcode;
    if (x->operands.empty()) return false;
    if (x->operands.size() == 1 || op == "divide" || op == "dynamic-slice" || op == "pad") {
      if (FindF8Subgraph(x->operands[0], visited, path)) { path->push_back({x, 0}); return true; }
      return false;
    }
    if (op == "multiply" || op == "select") {
      for (int k = 0; k < 2; ++k) {
        const int idx = k + (op == "select" ? 1 : 0);
        if (idx < int(x->operands.size()) && FindF8Subgraph(x->operands[idx], visited, path)) {
          path->push_back({x, idx});
          return true;
        }
      }
    }
    return false;
  }
  bool MatchFp8Param(Instr* x, Fp8Param* out, std::string* why) {
    std::set<Instr*> visited;
    std::vector<std::pair<Instr*, int>> path;
    if (!FindF8Subgraph(x, &visited, &path)) { *why = "no FP8 value behind operand " + x->name; return false; }
    out->fp8 = path[0].first;
    if (path.size() == 1) return true;
    Instr* conv = path[1].first;
    if (conv->opcode != "convert") { *why = "the FP8 value " + path[0].first->name + " is not dequantised by a convert"; return false; }
    size_t dequant_ops = 1;
    if (path.size() > 2) {
      Instr* bin = path[2].first;
      if (bin->operands.size() == 2 && (bin->opcode == "multiply" || (bin->opcode == "divide" && bin->operands[0] == conv))) {
        Instr* s = BroadcastOperand(Other(bin, conv));
        if (s != nullptr) {
          out->scale = s;
          out->mult_scale = bin->opcode == "multiply";
          dequant_ops = 2;
        }
      }
    }
    for (size_t i = 1 + dequant_ops; i < path.size(); ++i) {
      Instr* op = path[i].first;
      const std::string& oc = op->opcode;
      const bool same_type = op->operands[path[i].second]->shape.type == op->shape.type;
      const bool ok = (oc == "bitcast" && same_type) || oc == "broadcast" || oc == "copy" || oc == "dynamic-slice" || oc == "pad" ||
                      oc == "reshape" || oc == "select" || oc == "slice" || oc == "transpose";
      if (!ok) { *why = oc + " (" + op->name + ") between the dequantisation and the dot does not commute with it"; return false; }
      if (oc == "select") {
        double v;
        if (!(BcastConst(op->operands[path[i].second == 2 ? 1 : 2], &v) && v == 0.0)) {
          *why = "select needs a zero operand to be exchanged with the dequantisation";
          return false;
        }
      }
      if (oc == "pad") {
        double v;
        if (!(ConstantValue(op->operands[1], &v) && v == 0.0)) { *why = "pad needs a zero padding value to be exchanged with the dequantisation"; return false; }
      }
      out->commutative.push_back(path[i]);
    }
    return true;
  }
  // Re-applies the commutative ops to the FP8 value (shift_ops of CreateF8CustomCall).
  Instr* ShiftOps(Instr* x, const std::vector<std::pair<Instr*, int>>& ops) {
    for (const auto& pr : ops) {
      Instr* op = pr.first;
      Shape shape = op->shape;
      shape.type = x->shape.type;
      std::vector<Instr*> operands = {x};
      if (op->opcode == "dynamic-slice") {
        for (size_t i = 1; i < op->operands.size(); ++i) operands.push_back(op->operands[i]);
      } else if (op->opcode == "pad") {
        Shape ps = op->operands[1]->shape;
        ps.type = x->shape.type;
        operands.push_back(Add("convert", ps, {op->operands[1]}, "", "", op->operands[1]->name + "_" + x->shape.type));
      } else if (op->opcode == "select") {
        const int other_idx = pr.second == 2 ? 1 : 2;
        Shape zs = op->operands[other_idx]->shape;
        zs.type = x->shape.type;
        Instr* zero = Add("convert", zs, {op->operands[other_idx]}, "", "", op->operands[other_idx]->name + "_" + x->shape.type);
        operands = {op->operands[0], nullptr, nullptr};
        operands[pr.second] = x;
        operands[other_idx] = zero;
      }
      x = Add(op->opcode, shape, operands, op->attrs, "", op->name + "_" + x->shape.type);
    }
    return x;
  }
  // f32 scalar operand for a scale: 1 when absent, 1 / s when the HLO divided, converted to f32.
  Instr* ScaleOperand(Instr* scale, bool mult, const std::string& hint) {
    if (scale == nullptr) return ConstantScalar("f32", "1", hint + "_one");
    Instr* s = scale;
    if (!mult) {
      Instr* one = ConstantScalar(scale->shape.type, "1", "one");
      s = Add("divide", scale->shape, {one, scale}, "", "", hint + "_inv");
    }
    if (s->shape.type != "f32") s = Add("convert", MakeShape("f32", {}), {s}, "", "", hint + "_f32");
    return s;
  }

  // One operand of a dot as the buffer it physically is: `value` has shape [batch?, rows, cols] in the
  // default layout and `contracting` says which of rows / cols (0 / 1) is contracted.
  struct Physical {
    Instr* value = nullptr;
    int contracting = 0;
    int64_t batch = 0, free_extent = 0, k = 0;
  };
  // `batch_dims`, `c`, `nc`: the operand's batch, contracting and non-contracting dimension numbers.
  Physical AsRowMajor(Instr* x, const std::vector<int64_t>& batch_dims, int64_t c, int64_t nc, const std::string& hint) {
    const std::vector<int64_t> phys = x->shape.Physical();
    const size_t nb = batch_dims.size();
    bool batch_leading = true;
    for (size_t i = 0; i < nb; ++i) batch_leading = batch_leading && phys[i] == batch_dims[i];
    if (!batch_leading) {
      // The batch dimensions are not the major-most ones of the buffer: a copy into [batch..., nc, c] order.
      std::vector<int64_t> perm = batch_dims;
      perm.push_back(nc);
      perm.push_back(c);
      std::vector<int64_t> dims;
      for (int64_t d : perm) dims.push_back(x->shape.dims[d]);
      x = Add("transpose", MakeShape(x->shape.type, dims), {x}, "dimensions={" + JoinInts(perm) + "}", "", hint + "_batch_major");
      std::vector<int64_t> nbd(nb);
      for (size_t i = 0; i < nb; ++i) nbd[i] = int64_t(i);
      return AsRowMajor(x, nbd, int64_t(nb) + 1, int64_t(nb), hint);
    }
    Physical p;
    p.batch = 1;
    for (int64_t b : batch_dims) p.batch *= x->shape.dims[b];
    const int64_t d0 = phys[nb], d1 = phys[nb + 1];
    p.contracting = d0 == c ? 0 : 1;
    p.k = x->shape.dims[c];
    p.free_extent = x->shape.dims[nc];
    std::vector<int64_t> dims;
    if (nb > 0) dims.push_back(p.batch);
    dims.push_back(x->shape.dims[d0]);
    dims.push_back(x->shape.dims[d1]);
    if (dims == x->shape.dims && x->shape.IsDefaultLayout()) p.value = x;
    else p.value = Add("bitcast", MakeShape(x->shape.type, dims), {x}, "", "", hint + "_rm");   // the same bytes, read as the row-major array they are
    if (nb == 0) p.batch = 0;
    return p;
  }
  Instr* PadTo16(Instr* x, bool batched, const std::string& hint) {
    Shape padded = x->shape;
    for (size_t d = batched ? 1 : 0; d < padded.dims.size(); ++d) padded.dims[d] = Round16(padded.dims[d]);
    return PadTo(x, padded.dims, hint);
  }
  Instr* PadTo(Instr* x, const std::vector<int64_t>& target, const std::string& hint) {
    if (target == x->shape.dims) return x;
    Instr* zero = ConstantScalar(x->shape.type, "0", "zero_" + x->shape.type);
    std::string padding;
    for (size_t d = 0; d < x->shape.dims.size(); ++d) padding += (d ? "x" : "") + std::string("0_") + std::to_string(target[d] - x->shape.dims[d]);
    return Add("pad", MakeShape(x->shape.type, target), {x, zero}, "padding=" + padding, "", hint + "_pad");
  }

  // An operand with several adjacent non-contracting dimensions (a rank-3 activation times a rank-2
  // weight) is viewed as a matrix and the result reshaped back, which is what XLA's DotDecomposer
  // (xla/hlo/transforms/expanders/dot_decomposer.cc:155-270) has done before GemmRewriter runs.
  // Returns the canonical dot, or `dot` itself.
  Instr* MergeFreeDimensions(Instr* dot) {
    std::vector<int64_t> contracting[2] = {AttrList(dot->attrs, "lhs_contracting_dims"), AttrList(dot->attrs, "rhs_contracting_dims")};
    std::vector<int64_t> batch[2] = {AttrList(dot->attrs, "lhs_batch_dims"), AttrList(dot->attrs, "rhs_batch_dims")};
    if (contracting[0].size() != 1 || contracting[1].size() != 1) return dot;
    Instr* ops[2] = {dot->operands[0], dot->operands[1]};
    bool changed = false;
    int64_t merged_free[2] = {1, 1};
    for (int s = 0; s < 2; ++s) {
      Instr* x = ops[s];
      std::vector<int64_t> free;
      for (int64_t d = 0; d < int64_t(x->shape.dims.size()); ++d)
        if (d != contracting[s][0] && std::find(batch[s].begin(), batch[s].end(), d) == batch[s].end()) free.push_back(d);
      for (int64_t d : free) merged_free[s] *= x->shape.dims[d];
      if (free.size() < 2) continue;
      if (!x->shape.IsDefaultLayout() || !dot->shape.IsDefaultLayout()) return dot;
      for (size_t i = 1; i < free.size(); ++i) if (free[i] != free[i - 1] + 1) return dot;
      std::vector<int64_t> dims;
      const int64_t first = free.front(), removed = int64_t(free.size()) - 1;
      for (int64_t d = 0; d < int64_t(x->shape.dims.size()); ++d) {
        if (d == first) dims.push_back(merged_free[s]);
        else if (d < first || d > free.back()) dims.push_back(x->shape.dims[d]);
      }
      ops[s] = Add("reshape", MakeShape(x->shape.type, dims), {x}, "", "", x->name + "_2d");
      auto shift = [&](int64_t d) { return d > first ? d - removed : d; };
      contracting[s][0] = shift(contracting[s][0]);
      for (int64_t& b : batch[s]) b = shift(b);
      changed = true;
    }
    if (!changed) return dot;
    std::vector<int64_t> out_dims;
    for (int64_t b : batch[0]) out_dims.push_back(ops[0]->shape.dims[b]);
    out_dims.push_back(merged_free[0]);
    out_dims.push_back(merged_free[1]);
    std::string attrs = "lhs_contracting_dims={" + JoinInts(contracting[0]) + "}, rhs_contracting_dims={" + JoinInts(contracting[1]) + "}";
    if (!batch[0].empty()) attrs = "lhs_batch_dims={" + JoinInts(batch[0]) + "}, rhs_batch_dims={" + JoinInts(batch[1]) + "}, " + attrs;
    Instr* canon = Add("dot", MakeShape(dot->shape.type, out_dims), {ops[0], ops[1]}, attrs, "", dot->name + "_2d");
    Instr* back = Add("reshape", dot->shape, {canon}, "", "", dot->name + "_view");
    Replace(dot, back);
    return canon;
  }

  // ---- HandleDot ----
  void HandleDot(Instr* dot) {
    if (dot->operands.size() != 2) return;
    dot = MergeFreeDimensions(dot);
    Instr* lhs = dot->operands[0];
    Instr* rhs = dot->operands[1];
    const std::vector<int64_t> lc = AttrList(dot->attrs, "lhs_contracting_dims"), rc = AttrList(dot->attrs, "rhs_contracting_dims");
    const std::vector<int64_t> lb = AttrList(dot->attrs, "lhs_batch_dims"), rb = AttrList(dot->attrs, "rhs_batch_dims");
    // s8 x s8 -> s32, and s8 x s8 -> f32 (both rows of the run-time type table, cuda_blas_lt.cc:444-445): the f32 form
    // is the exact s32 sum converted once.
    const bool int8 = lhs->shape.type == "s8" && rhs->shape.type == "s8" && (dot->shape.type == "s32" || dot->shape.type == "f32");

    Fp8Param a, b;
    std::string why;
    if (!int8) {
      if (!MatchFp8Param(lhs, &a, &why) || !MatchFp8Param(rhs, &b, &why)) return Refuse(dot, "operands are not dequantised FP8 values: " + why);
      const std::string &at = a.fp8->shape.type, &bt = b.fp8->shape.type;
      if (at == "f8e5m2" && bt == "f8e5m2") return Refuse(dot, "both operands are f8e5m2: one of them must be f8e4m3fn");
      if (!IsF8(at) || !IsF8(bt)) return Refuse(dot, "operand types must be f8e4m3fn or f8e5m2, got " + at + " and " + bt);
      for (Instr* s : {a.scale, b.scale})
        if (s != nullptr && !s->shape.IsScalar()) return Refuse(dot, "the scaling factors must be scalars");
      const std::string& dt = dot->shape.type;
      if (!(dt == "bf16" || dt == "f16" || dt == "f32" || IsF8(dt))) return Refuse(dot, "output type must be f8e4m3fn, f8e5m2, bf16, f16 or f32, got " + dt);
      if (dt == "f8e5m2" && at == "f8e4m3fn" && bt == "f8e4m3fn") return Refuse(dot, "f8e4m3fn x f8e4m3fn -> f8e5m2 is not in the supported type table");
    }
    if (lc.size() != 1 || rc.size() != 1) return Refuse(dot, "A and B must have one contracting dimension each");
    if (lb.size() != rb.size()) return Refuse(dot, "batch dimensions of A and B differ in number");
    const size_t nb = lb.size();
    Instr* a_in = int8 ? lhs : (a.commutative.empty() ? a.fp8 : a.commutative.back().first);
    Instr* b_in = int8 ? rhs : (b.commutative.empty() ? b.fp8 : b.commutative.back().first);
    if (a_in->shape.dims.size() != nb + 2 || b_in->shape.dims.size() != nb + 2)
      return Refuse(dot, "inputs must have exactly one contracting and one non-contracting dimension");
    if (dot->shape.dims.size() != nb + 2) return Refuse(dot, "unexpected result rank");
    auto free_dim = [&](const std::vector<int64_t>& batch, int64_t c, size_t rank) {
      for (int64_t d = 0; d < int64_t(rank); ++d)
        if (d != c && std::find(batch.begin(), batch.end(), d) == batch.end()) return d;
      return int64_t(-1);
    };
    const int64_t lnc = free_dim(lb, lc[0], nb + 2), rnc = free_dim(rb, rc[0], nb + 2);
    if (lnc < 0 || rnc < 0) return Refuse(dot, "A and B must have one non-contracting dimension");
    if (a_in->shape.dims[lc[0]] != b_in->shape.dims[rc[0]]) return Refuse(dot, "contracting extents differ");
    for (size_t i = 0; i < nb; ++i)
      if (a_in->shape.dims[lb[i]] != b_in->shape.dims[rb[i]]) return Refuse(dot, "batch extents differ");
    // The reference leaves tiny dots to its elementwise emitters ((m + n) * k below a threshold of 100,
    // xla/service/gpu/matmul_utils.cc:1171-1205).
    // Only floating-point dots can go there (IsDotSupportedByClassicalEmitters, :1207-1222).
    const bool float_dot = dot->shape.type == "f16" || dot->shape.type == "f32" || dot->shape.type == "bf16";
    if (float_dot && (a_in->shape.dims[lnc] + b_in->shape.dims[rnc]) * a_in->shape.dims[lc[0]] < 100)
      return Refuse(dot, "too small to be worth a library call ((m + n) * k < 100)");

    // How the result lies in memory decides which operand plays A: batch-major, then either [m, n] (as is)
    // or [n, m] (a column-major result, produced as D^T = B^T A^T).
    const std::vector<int64_t> ophys = dot->shape.Physical();
    bool out_batch_leading = true;
    for (size_t i = 0; i < nb; ++i) out_batch_leading = out_batch_leading && ophys[i] == int64_t(i);
    const bool swapped = out_batch_leading && ophys[nb] == int64_t(nb) + 1;      // n is the major one of the matrix dims

    Instr* a_val = int8 ? lhs : ShiftOps(a.fp8, a.commutative);
    Instr* b_val = int8 ? rhs : ShiftOps(b.fp8, b.commutative);
    Physical pa = AsRowMajor(a_val, lb, lc[0], lnc, "a");
    Physical pb = AsRowMajor(b_val, rb, rc[0], rnc, "b");
    Instr* a_scale = int8 ? nullptr : ScaleOperand(a.scale, a.mult_scale, "a_scale");
    Instr* b_scale = int8 ? nullptr : ScaleOperand(b.scale, b.mult_scale, "b_scale");
    if (swapped) {
      std::swap(pa, pb);
      std::swap(a_scale, b_scale);
    }
    auto g = std::make_unique<Gemm>();
    g->f8 = !int8;
    g->swapped = swapped;
    g->batched = nb > 0;
    g->batch = nb > 0 ? pa.batch : 0;
    g->m = pa.free_extent;
    g->n = pb.free_extent;
    g->k = pa.k;
    g->lhs_contracting = pa.contracting + (nb > 0 ? 1 : 0);
    g->rhs_contracting = pb.contracting + (nb > 0 ? 1 : 0);
    const int64_t gm = g->m, gn = g->n, gbatch = g->batch;
    Instr* a_op = PadTo16(pa.value, nb > 0, "a");
    Instr* b_op = PadTo16(pb.value, nb > 0, "b");

    std::vector<int64_t> ddims, dpad;
    if (nb > 0) { ddims.push_back(gbatch); dpad.push_back(gbatch); }
    ddims.push_back(gm); ddims.push_back(gn);
    dpad.push_back(Round16(gm)); dpad.push_back(Round16(gn));
    std::vector<Instr*> operands = {a_op, b_op};
    if (!int8) { operands.push_back(a_scale); operands.push_back(b_scale); }
    Instr* call = Add("custom-call", MakeShape(dot->shape.type, dpad), operands, "", "", "gemm");
    call->gemm = std::move(g);
    calls_.push_back(call);

    Instr* result = call;
    if (dpad != ddims) {
      std::string sl;
      for (size_t d = 0; d < ddims.size(); ++d) sl += (d ? ", " : "") + std::string("[0:") + std::to_string(ddims[d]) + "]";
      result = Add("slice", MakeShape(dot->shape.type, ddims), {result}, "slice={" + sl + "}", "", "gemm_slice");
    }
    if (!out_batch_leading) {
      // Batch-major result first, then a copy into the layout the module asked for.
      std::vector<int64_t> ldims;
      for (size_t i = 0; i < nb; ++i) ldims.push_back(dot->shape.dims[i]);
      ldims.push_back(gm); ldims.push_back(gn);
      Instr* bm = result;
      if (ldims != result->shape.dims) bm = Add("bitcast", MakeShape(dot->shape.type, ldims), {result}, "", "", "gemm_view");
      result = Add("copy", dot->shape, {bm}, "", "", "gemm_relayout");
    } else if (result->shape.dims != dot->shape.dims || !dot->shape.IsDefaultLayout()) {
      result = Add("bitcast", dot->shape, {result}, "", "", "gemm_view");
    }
    Replace(dot, result);
  }

  // `__op$block_scaled_dot` (xla/backends/gpu/transforms/block_scaling_rewriter.h:30-77): operands lhs, rhs,
  // lhs_scale, rhs_scale [, global_scale]; contracting dimension minor on both inputs, an optional batch
  // dimension major.  The reference either expands it into dequantize + dot (block_scaling_rewriter.cc:194-262)
  // or hands it to a library; with MX operands (FP8 values, one f8e8m0fnu scale per 32) it becomes this
  // library's block-scaled call, which takes the four operands as they are.  Everything else is left alone.
  // `__op$block_scaled_dot` (block_scaling_rewriter.h:30-77): the contracting dimension is the minor one of both
  // operands by definition of the call.
  void HandleBlockScaledDot(Instr* cc) {
    if (cc->operands.size() == 5) return Refuse(cc, "block-scaled dot with a global scale: not taken by the MX call (exactly four operands, thunk_emitter.cc:939-988)");
    if (cc->operands.size() != 4) return Refuse(cc, "block-scaled dot must have four operands");
    // An explicit block size comes in the backend config (block_scaling_rewriter.cc:613-621); it is what allows scale
    // arrays padded along k.  Extra scale rows are allowed either way (block_scaling_rewriter.cc:489-493).  The
    // call takes the padded arrays as they are and reads the leading [rows, k / 32] corner.
    int64_t explicit_block = 0;
    const size_t p = cc->attrs.find("block_size");
    if (p != std::string::npos) {
      size_t q = p + 10;
      while (q < cc->attrs.size() && !std::isdigit(static_cast<unsigned char>(cc->attrs[q]))) ++q;
      explicit_block = std::strtoll(cc->attrs.c_str() + q, nullptr, 10);
      if (explicit_block != 32) return Refuse(cc, "block-scaled dot: the block size must be 32 (MX), got " + std::to_string(explicit_block));
    }
    TakeMxDot(cc, "block-scaled dot", explicit_block);
  }

  // The `scaled-dot` instruction (lhs, rhs, lhs_scale, rhs_scale + dot dimension numbers), which the reference turns
  // into `__cublas$lt$matmul$mx` when a BLAS library wins its autotuning (autotuner/hipblaslt.cc:430-505; run against
  // the expansion in autotuner/mx_scaled_dot_execution_test.cc).  Taken in the form that call has: one contracting
  // dimension, the minor one of both operands, and at most one leading batch dimension.
  void HandleScaledDot(Instr* sd) {
    if (sd->operands.size() != 4) return Refuse(sd, "scaled-dot must have four operands");
    const std::vector<int64_t> lc = AttrList(sd->attrs, "lhs_contracting_dims"), rc = AttrList(sd->attrs, "rhs_contracting_dims");
    const std::vector<int64_t> lb = AttrList(sd->attrs, "lhs_batch_dims"), rb = AttrList(sd->attrs, "rhs_batch_dims");
    const int64_t rank = int64_t(sd->operands[0]->shape.dims.size());
    if (lc.size() != 1 || rc.size() != 1) return Refuse(sd, "scaled-dot: A and B must have one contracting dimension each");
    if (int64_t(sd->operands[1]->shape.dims.size()) != rank) return Refuse(sd, "scaled-dot: operand ranks differ");
    if (rank != 2 && rank != 3) return Refuse(sd, "scaled-dot: operands must have rank 2, or rank 3 with one leading batch dimension");
    const bool batch_ok = rank == 3 ? (lb == std::vector<int64_t>{0} && rb == std::vector<int64_t>{0}) : (lb.empty() && rb.empty());
    if (!batch_ok) return Refuse(sd, "scaled-dot: batch dimensions must be {0} on rank-3 operands and absent on rank-2 ones");
    const int64_t contracting[2] = {lc[0], rc[0]};
    for (int k = 0; k < 2; ++k)
      if (contracting[k] != rank - 1 && contracting[k] != rank - 2) return Refuse(sd, "scaled-dot: the contracting dimension must be one of the two matrix dimensions");
    for (int k = 2; k < 4; ++k)
      if (sd->operands[k]->shape.dims.empty()) return Refuse(sd, "scaled-dot: a scalar scale means no scaling; not the MX form");
    // The instruction's scales may be coarser in any dimension (one scale per dim / scale_dim indices,
    // hlo_evaluator_typed_visitor.h:1831-1879); the MX form has one per row and per 32 values along k.
    for (int k = 0; k < 2; ++k) {
      const Shape& v = sd->operands[k]->shape;
      const Shape& sc = sd->operands[k + 2]->shape;
      const int64_t free_dim = contracting[k] == rank - 1 ? rank - 2 : rank - 1;
      if (int64_t(sc.dims.size()) != rank || sc.dims[free_dim] != v.dims[free_dim])
        return Refuse(sd, "scaled-dot: the block size must be 32 along k and 1 along the rows (scales [rows, k / 32])");
    }
    // The MX call wants k minor on both operands.  An operand given [k, rows] is transposed in front of the call
    // together with its scales (one extra pass over that operand; the library the reference calls takes a
    // transposed operand through its matrix layouts instead).
    const std::vector<Instr*> original = sd->operands;
    for (int k = 0; k < 2; ++k) {
      if (contracting[k] == rank - 1) continue;
      for (int which : {k, k + 2}) {
        Instr* x = sd->operands[which];
        if (!x->shape.IsDefaultLayout()) { sd->operands = original; return Refuse(sd, "scaled-dot: operands must be in the default (row-major) layout"); }
        std::vector<int64_t> perm, dims;
        for (int64_t d = 0; d < rank - 2; ++d) perm.push_back(d);
        perm.push_back(rank - 1);
        perm.push_back(rank - 2);
        for (int64_t d : perm) dims.push_back(x->shape.dims[d]);
        sd->operands[which] = Add("transpose", MakeShape(x->shape.type, dims), {x}, "dimensions={" + JoinInts(perm) + "}", "", x->name + "_k_minor");
      }
    }
    if (!TakeMxDot(sd, "scaled-dot", 0)) sd->operands = original;
  }

  bool Declined(Instr* i, const std::string& why) {
    Refuse(i, why);
    return false;
  }
  bool TakeMxDot(Instr* cc, const std::string& what, int64_t explicit_block) {
    const Shape& a = cc->operands[0]->shape;
    const Shape& b = cc->operands[1]->shape;
    const Shape& sa = cc->operands[2]->shape;
    const Shape& sb = cc->operands[3]->shape;
    const Shape& d = cc->shape;
    if (!IsF8(a.type) || !IsF8(b.type)) return Declined(cc, what + ": only f8e4m3fn / f8e5m2 values are implemented, got " + a.type + " and " + b.type);
    if (sa.type != "f8e8m0fnu" || sb.type != "f8e8m0fnu") return Declined(cc, what + ": scales must be f8e8m0fnu (MX), got " + sa.type + " and " + sb.type);
    if (!(d.type == "f32" || d.type == "bf16" || d.type == "f16")) return Declined(cc, what + ": result must be f32, bf16 or f16");
    const size_t rank = a.dims.size();
    if ((rank != 2 && rank != 3) || b.dims.size() != rank || sa.dims.size() != rank || sb.dims.size() != rank || d.dims.size() != rank)
      return Declined(cc, what + ": operands must have rank 2, or rank 3 with one leading batch dimension");
    for (const Shape* sh : {&a, &b, &sa, &sb, &d})
      if (!sh->IsDefaultLayout()) return Declined(cc, what + ": operands must be in the default (row-major) layout");
    const size_t o = rank - 2;
    const int64_t m = a.dims[o], k = a.dims[o + 1], n = b.dims[o];
    if (b.dims[o + 1] != k) return Declined(cc, what + ": contracting dimensions differ");
    if (k % 32 != 0 || sa.dims[o] < m || sb.dims[o] < n) return Declined(cc, what + ": the block size must be 32 (scales [rows, k / 32])");
    if (explicit_block ? (sa.dims[o + 1] * 32 < k || sb.dims[o + 1] * 32 < k) : (sa.dims[o + 1] * 32 != k || sb.dims[o + 1] * 32 != k))
      return Declined(cc, what + ": the block size must be 32 (scales [rows, k / 32])");
    if (d.dims[o] != m || d.dims[o + 1] != n) return Declined(cc, what + ": result shape is not [m, n]");
    if (rank == 3 && !(b.dims[0] == a.dims[0] && sa.dims[0] == a.dims[0] && sb.dims[0] == a.dims[0] && d.dims[0] == a.dims[0]))
      return Declined(cc, what + ": batch dimensions differ");
    auto g = std::make_unique<Gemm>();
    g->f8 = true;
    g->mx = true;
    g->explicit_block = explicit_block;
    g->m = m; g->n = n; g->k = k;
    g->batched = rank == 3;
    g->batch = rank == 3 ? a.dims[0] : 0;
    g->lhs_contracting = int(rank) - 1;
    g->rhs_contracting = int(rank) - 1;
    Instr* call = Add("custom-call", cc->shape, cc->operands, "", "", "mx_gemm");
    call->gemm = std::move(g);
    calls_.push_back(call);
    Replace(cc, call);
    return true;
  }

  // gemm, or slice(gemm), or bitcast(gemm), or bitcast(slice(gemm)) -- with one user each below the top.
  struct Through {
    Instr* gemm = nullptr;
    Instr* slice = nullptr;
    Instr* bitcast = nullptr;
  };
  bool LookThrough(Instr* x, Through* t, bool need_one_user_each) {
    Instr* cur = x;
    if (cur->opcode == "bitcast" && cur->operands.size() == 1) { t->bitcast = cur; cur = cur->operands[0]; }
    if (cur->opcode == "slice" && cur->operands.size() == 1) { t->slice = cur; cur = cur->operands[0]; }
    if (!IsF8Gemm(cur)) return false;          // epilogues are fused into the FP8 call only
    t->gemm = cur;
    if (need_one_user_each) {
      if (UserCount(cur) != 1) return false;
      if (t->slice && t->bitcast && UserCount(t->slice) != 1) return false;
    }
    if (t->slice) {          // only slices that chop off the ends of dimensions, with stride 1
      const std::string& at = t->slice->attrs;
      for (size_t p = at.find('['); p != std::string::npos; p = at.find('[', p + 1)) {
        if (at.compare(p, 3, "[0:") != 0) return false;
        const size_t close = at.find(']', p);
        const std::string body = at.substr(p + 1, close - p - 1);
        if (std::count(body.begin(), body.end(), ':') == 2 && body.substr(body.rfind(':')) != ":1") return false;
      }
    }
    return true;
  }
  // Rebuilds slice / bitcast on top of a call whose element type (or value) changed.
  Instr* Rewrap(const Through& t, const std::string& new_type) {
    Instr* r = t.gemm;
    if (t.slice) {
      Shape s = t.slice->shape;
      s.type = new_type;
      r = Add("slice", s, {r}, t.slice->attrs, "", "gemm_slice");
    }
    if (t.bitcast) {
      Shape s = t.bitcast->shape;
      s.type = new_type;
      r = Add("bitcast", s, {r}, "", "", "gemm_view");
    }
    return r;
  }

  // ---- HandleMultiply / HandleDivide ----
  void HandleMultiply(Instr* instr) {
    if (instr->operands.size() != 2) return;
    // alpha: multiply(gemm, broadcast(constant)), each with this one user
    for (int side = 0; side < 2; ++side) {
      Instr* g = instr->operands[side];
      Instr* other = instr->operands[1 - side];
      double alpha;
      if (IsF8Gemm(g) && UserCount(g) == 1 && UserCount(other) == 1 && BcastConst(other, &alpha) &&
          g->gemm->beta == 0.0 && g->gemm->epilogue == 0 && !g->gemm->has_d_scale) {
        g->gemm->alpha *= alpha;
        Replace(instr, g);
        return;
      }
    }
    // output scale without an FP8 cast
    for (int side = 0; side < 2; ++side) {
      Instr* g = instr->operands[side];
      Instr* other = instr->operands[1 - side];
      if (IsF8Gemm(g) && UserCount(g) == 1 && UserCount(other) == 1 && BroadcastOperand(other) != nullptr) {
        if (F8ScaleD(instr, g, BroadcastOperand(other), /*divide=*/false)) return;
      }
    }
    // tanh-form GELU: x * cdf, cdf = 0.5 * (1 + tanh(sqrt(2 / pi) * (x + 0.044715 * x^3)))
    for (int side = 0; side < 2; ++side) {
      Instr* x = instr->operands[side];
      Instr* cdf = instr->operands[1 - side];
      Through t;
      if (!LookThrough(x, &t, /*need_one_user_each=*/false)) continue;
      if (t.slice && t.bitcast) continue;
      if (UserCount(cdf) != 1 || !MatchGeluCdf(cdf, x)) continue;
      FuseGelu(instr, t);
      return;
    }
  }
  void HandleDivide(Instr* instr) {
    if (instr->operands.size() != 2) return;
    Instr* g = instr->operands[0];
    Instr* other = instr->operands[1];
    if (IsF8Gemm(g) && UserCount(g) == 1 && UserCount(other) == 1 && BroadcastOperand(other) != nullptr)
      F8ScaleD(instr, g, BroadcastOperand(other), /*divide=*/true);
  }
  bool F8ScaleD(Instr* instr, Instr* g, Instr* d_scale, bool divide) {
    if (!d_scale->shape.IsScalar() || g->gemm->has_d_scale || IsF8(g->shape.type)) return false;
    Instr* a_scale = g->operands[g->gemm->ScaleIndex()];
    double v;
    if (!(ConstantValue(a_scale, &v) && v == 1.0)) return false;       // an input scale already sits there
    const int e = g->gemm->epilogue;
    if ((e != 0 && e != 2) || g->gemm->beta != 0.0) return false;      // DEFAULT or RELU only, no matrix bias
    g->operands[g->gemm->ScaleIndex()] = ScaleOperand(d_scale, !divide, "a_scale");
    dirty_ = true;
    Replace(instr, g);
    return true;
  }
  template <typename Pred>
  bool MulWith(Instr* mul, Pred pred, Instr** rest) {
    if (mul == nullptr || mul->opcode != "multiply" || mul->operands.size() != 2) return false;
    for (int s = 0; s < 2; ++s)
      if (pred(mul->operands[s])) { *rest = mul->operands[1 - s]; return true; }
    return false;
  }
  bool MatchGeluCdf(Instr* cdf, Instr* x) {
    Instr *sum1 = nullptr, *th = nullptr, *poly = nullptr, *cube_term = nullptr, *x3 = nullptr, *x2 = nullptr;
    if (!MulWith(cdf, [&](Instr* o) { return BcastConstNear(o, 0.5); }, &sum1)) return false;
    if (sum1->opcode != "add" || sum1->operands.size() != 2) return false;
    for (int s = 0; s < 2; ++s)
      if (BcastConstNear(sum1->operands[s], 1.0)) th = sum1->operands[1 - s];
    if (th == nullptr || th->opcode != "tanh" || UserCount(th) != 1) return false;
    Instr* inner = th->operands[0];
    if (UserCount(inner) != 1) return false;
    if (!MulWith(inner, [&](Instr* o) { return BcastConstNear(o, std::sqrt(2.0 / M_PI)); }, &poly)) return false;
    if (poly->opcode != "add" || poly->operands.size() != 2 || UserCount(poly) != 1) return false;
    for (int s = 0; s < 2; ++s)
      if (poly->operands[s] == x) cube_term = poly->operands[1 - s];
    if (cube_term == nullptr || UserCount(cube_term) != 1) return false;
    if (!MulWith(cube_term, [&](Instr* o) { return BcastConstNear(o, 0.044715); }, &x3)) return false;
    if (UserCount(x3) != 1) return false;
    if (!MulWith(x3, [&](Instr* o) { return o == x; }, &x2)) return false;
    if (x2->opcode != "multiply" || UserCount(x2) != 1) return false;
    return x2->operands.size() == 2 && x2->operands[0] == x && x2->operands[1] == x;
  }
  void FuseGelu(Instr* mul, const Through& t) {
    Instr* g = t.gemm;
    // The pre-activation has four users inside the GELU pattern; any other user would need the
    // auxiliary output (GELU_AUX), which this library does not produce: the pattern is left alone then.
    Instr* view = t.slice ? t.slice : t.bitcast;
    const bool has_aux = view ? (UserCount(view) > 4 || UserCount(g) > 1) : UserCount(g) > 4;
    if (has_aux || g->shape.type == "s32" || g->gemm->has_d_scale) return;
    if (g->gemm->epilogue == 0) g->gemm->epilogue = 4;              // GELU
    else if (g->gemm->epilogue == 1) g->gemm->epilogue = 6;         // BIAS_GELU
    else return;
    Replace(mul, Rewrap(t, g->shape.type));
  }

  // ---- HandleAdd ----
  void HandleAdd(Instr* instr) {
    if (instr->operands.size() != 2) return;
    for (int side = 0; side < 2; ++side) {
      Instr* x = instr->operands[side];
      Instr* other = instr->operands[1 - side];
      Through t;
      if (!LookThrough(x, &t, true)) continue;
      if ((t.slice || t.bitcast) && UserCount(x) != 1) continue;
      if (other->opcode == "broadcast") {
        if (FuseVectorBias(instr, t, x, other)) return;
        // add(bitcast(gemm), broadcast(bias)) on a batched call: the broadcast itself becomes a matrix bias
        if (t.bitcast && !t.slice && UserCount(other) == 1 && FuseMatrixBias(instr, t, x, other)) return;
        continue;
      }
      if (FuseMatrixBias(instr, t, x, other)) return;
    }
  }
  bool FuseVectorBias(Instr* instr, const Through& t, Instr* x, Instr* broadcast) {
    Instr* g = t.gemm;
    if (g->shape.type == "s32" || g->gemm->has_d_scale) return false;
    Instr* bias = broadcast->operands[0];
    Instr* convert = bias->opcode == "convert" ? bias : nullptr;
    if (UserCount(g) != 1 || g->gemm->epilogue != 0) return false;
    if (bias->shape.dims.size() != 1) return false;
    // The bias must run along the minor-most dimension of what the add sees, and that dimension must be
    // the columns of the call's result.
    const Shape& out = x->shape;
    const std::vector<int64_t> bd = AttrList(broadcast->attrs, "dimensions");
    const int64_t minor = out.MinorToMajor()[0];
    if (bd.size() != 1 || bd[0] != minor || bias->shape.dims[0] != out.dims[minor] || bias->shape.dims[0] != g->gemm->n) return false;
    if (g->gemm->f8 && g->gemm->beta != 0.0) return false;       // matrix and vector bias together: only the matrix bias is fused
    if (g->gemm->f8 && bias->shape.type == "f32") {
      if (convert == nullptr) return false;      // an f32 bias is only taken as convert(bf16 / f16)
      Instr* narrow = convert->operands[0];
      const std::string &bt = narrow->shape.type, &ot = g->shape.type;
      const bool ok = (bt == "bf16" && (IsF8(ot) || ot == "f32" || ot == "bf16")) || (bt == "f16" && (ot == "f16" || IsF8(ot)));
      if (!ok) return false;
      bias = narrow;
    }
    if (!(bias->shape.type == "bf16" || bias->shape.type == "f16" || bias->shape.type == "f32")) return false;
    bias = PadTo(bias, {g->shape.dims.back()}, "bias");
    g->operands.push_back(bias);
    g->gemm->has_bias = true;
    g->gemm->epilogue = 1;                       // BIAS
    dirty_ = true;
    Replace(instr, x);
    return true;
  }
  bool FuseMatrixBias(Instr* instr, const Through& t, Instr* x, Instr* bias) {
    Instr* g = t.gemm;
    if (g->shape.type == "s32" || IsAnyF8(bias->shape.type) || g->gemm->has_d_scale) return false;
    if (bias->shape.dims != x->shape.dims) return false;
    if (!(g->gemm->epilogue == 0 || g->gemm->epilogue == 1) || g->gemm->beta != 0.0 || UserCount(g) != 1) return false;
    if (!(bias->shape.type == "bf16" || bias->shape.type == "f16" || bias->shape.type == "f32")) return false;
    // The bias must lie in memory like the value it is added to (then the same view applies to it).
    if (bias->shape.MinorToMajor() != x->shape.MinorToMajor()) return false;
    Instr* c = bias;
    std::vector<int64_t> logical;                 // the call's unpadded result dims
    if (g->gemm->batched) logical.push_back(g->gemm->batch);
    logical.push_back(g->gemm->m);
    logical.push_back(g->gemm->n);
    if (c->shape.dims != logical || !c->shape.IsDefaultLayout()) c = Add("bitcast", MakeShape(c->shape.type, logical), {c}, "", "", "c_view");
    c = PadTo(c, g->shape.dims, "c");
    g->operands.insert(g->operands.begin() + 2, c);
    g->gemm->has_c = true;
    g->gemm->beta = 1.0;
    dirty_ = true;
    Replace(instr, x);
    return true;
  }

  // ---- HandleMaximum ----
  void HandleMaximum(Instr* instr) {
    if (instr->operands.size() != 2) return;
    for (int side = 0; side < 2; ++side) {
      Instr* x = instr->operands[side];
      Instr* zeros = instr->operands[1 - side];
      double v;
      if (!(BcastConst(zeros, &v) && v == 0.0)) continue;
      Through t;
      if (!LookThrough(x, &t, false)) continue;
      if (t.slice && t.bitcast) continue;
      Instr* g = t.gemm;
      if (g->shape.type == "s32" || UserCount(g) != 1 || UserCount(x) != 1 || g->gemm->has_d_scale) continue;
      if (g->gemm->epilogue == 0) g->gemm->epilogue = 2;            // RELU
      else if (g->gemm->epilogue == 1) g->gemm->epilogue = 3;       // BIAS_RELU
      else continue;
      Replace(instr, x);
      return;
    }
  }

  // ---- HandleConvert: scaled, saturating FP8 output and amax ----
  void HandleConvert(Instr* instr) {
    if (!IsF8(instr->shape.type) || instr->operands.size() != 1) return;
    Instr* clamp = instr->operands[0];
    if (clamp->opcode != "clamp" || clamp->operands.size() != 3 || UserCount(clamp) != 1) return;
    double lo, hi;
    if (!BcastConst(clamp->operands[0], &lo) || !BcastConst(clamp->operands[2], &hi)) return;
    Instr* mid = clamp->operands[1];
    Instr* g = nullptr;
    Instr* d_scale = nullptr;
    bool mult = false;
    if (IsF8Gemm(mid)) {
      g = mid;
    } else if ((mid->opcode == "divide" || mid->opcode == "multiply") && mid->operands.size() == 2) {
      for (int side = 0; side < 2; ++side) {
        if (mid->opcode == "divide" && side != 0) continue;
        Instr* cand = mid->operands[side];
        Instr* other = mid->operands[1 - side];
        if (IsF8Gemm(cand) && BroadcastOperand(other) != nullptr) {
          g = cand;
          d_scale = BroadcastOperand(other);
          mult = mid->opcode == "multiply";
          break;
        }
      }
    }
    if (g == nullptr || g->gemm->has_d_scale || IsF8(g->shape.type)) return;
    const double mx = F8Max(instr->shape.type);
    if (lo != -mx || hi != mx) return;                        // the clamp must be exactly the type's finite range
    if (d_scale != nullptr && !d_scale->shape.IsScalar()) return;
    const std::string &at = g->operands[0]->shape.type, &bt = g->operands[1]->shape.type;
    if (instr->shape.type == "f8e5m2" && at == "f8e4m3fn" && bt == "f8e4m3fn") return;   // not in the supported type table
    // The only other user the call may have is the maximum of its absolute values.
    const std::vector<Instr*> users = ValueUsers(g);
    Instr* reduce_damax = nullptr;
    if (UserCount(g) == 2) {
      for (Instr* u : users) {
        Instr* maybe = nullptr;
        if (u->opcode == "abs") {
          if (UserCount(u) != 1 || ValueUsers(u).empty()) continue;
          maybe = ValueUsers(u)[0];
        } else {
          if (g->gemm->epilogue != 2 && g->gemm->epilogue != 3) continue;     // without abs, ReLU must make the values non-negative
          maybe = u;
        }
        double init;
        if (maybe->opcode == "reduce" && maybe->operands.size() == 2 && ConstantValue(maybe->operands[1], &init) && init <= 0.0 &&
            maybe->shape.IsScalar() && ReducesWithMaximum(maybe))
          reduce_damax = maybe;
      }
      if (reduce_damax == nullptr) return;
    } else if (UserCount(g) > 2) {
      return;
    }
    if (g->gemm->beta != 0.0) {
      const std::string& ct = g->operands[2]->shape.type;
      if (ct != "bf16" && ct != "f16") return;
    }
    g->operands.push_back(d_scale ? ScaleOperand(d_scale, mult, "d_scale") : ConstantScalar("f32", "1", "d_scale_one"));
    g->gemm->has_d_scale = true;
    g->shape.type = instr->shape.type;
    dirty_ = true;
    if (reduce_damax != nullptr) {
      g->gemm->damax = true;
      Instr* amax = Add("gemm-amax", MakeShape("f32", {}), {g}, "", "", "amax");
      g->gemm->amax = amax;
      Instr* out = amax;
      if (reduce_damax->shape.type != "f32") out = Add("convert", reduce_damax->shape, {amax}, "", "", "amax_" + reduce_damax->shape.type);
      Replace(reduce_damax, out);
    }
    Replace(instr, g);
  }
  bool ReducesWithMaximum(Instr* reduce) const {
    size_t p = reduce->attrs.find("to_apply=");
    if (p == std::string::npos) return false;
    std::string name = reduce->attrs.substr(p + 9);
    if (!name.empty() && name[0] == '%') name = name.substr(1);
    size_t e = name.find_first_of(", ");
    if (e != std::string::npos) name = name.substr(0, e);
    for (const Computation& c : *all_)
      if (c.name == name) {
        Instr* r = nullptr;
        for (const auto& i : c.instrs) if (i->is_root) r = i.get();
        if (r == nullptr && !c.instrs.empty()) r = c.instrs.back().get();
        return r != nullptr && r->opcode == "maximum";
      }
    return false;
  }

  // ---- beyond the reference ----
  // convert(s32 call) * broadcast(row scale, dims={0}) * broadcast(col scale, dims={1}) [-> convert(bf16)]
  void FoldInt8Dequantisation(Instr* g) {
    if (g->gemm->batched || g->gemm->swapped) return;
    Instr* top = g;
    Instr* slice = nullptr;
    if (UserCount(top) == 1 && !ValueUsers(top).empty() && ValueUsers(top)[0]->opcode == "slice") { slice = ValueUsers(top)[0]; top = slice; }
    Instr* cf = nullptr;
    for (Instr* u : ValueUsers(top)) if (u->opcode == "convert" && u->shape.type == "f32") cf = u;
    if (cf == nullptr) return;
    auto scale_along = [&](Instr* x, int64_t dim, Instr** next, Instr** scale) {
      if (UserCount(x) != 1 || ValueUsers(x).empty()) return false;
      Instr* u = ValueUsers(x)[0];
      if (u->opcode != "multiply") return false;
      Instr* other = Other(u, x);
      if (other == nullptr || other->opcode != "broadcast") return false;
      const std::vector<int64_t> bd = AttrList(other->attrs, "dimensions");
      Instr* v = other->operands[0];
      if (bd.size() != 1 || bd[0] != dim || v->shape.type != "f32" || v->shape.dims.size() != 1) return false;
      *next = u;
      *scale = v;
      return true;
    };
    Instr *y0 = nullptr, *y1 = nullptr, *rs = nullptr, *cs = nullptr;
    if (!scale_along(cf, 0, &y0, &rs) || !scale_along(y0, 1, &y1, &cs)) return;
    if (rs->shape.dims[0] != g->gemm->m || cs->shape.dims[0] != g->gemm->n) return;
    Instr* out = y1;
    if (UserCount(y1) == 1 && !ValueUsers(y1).empty() && ValueUsers(y1)[0]->opcode == "convert" && ValueUsers(y1)[0]->shape.type == "bf16")
      out = ValueUsers(y1)[0];
    const bool keep_s32 = UserCount(top) > 1;          // the raw accumulator is an output too
    g->operands.push_back(PadTo(rs, {g->shape.dims[0]}, "a_row_scale"));
    g->operands.push_back(PadTo(cs, {g->shape.dims[1]}, "b_col_scale"));
    g->gemm->has_dequant = true;
    const std::string s32 = g->shape.type;
    g->shape.type = out->shape.type;
    dirty_ = true;
    Instr* result = g;
    if (slice != nullptr) {
      Shape s = slice->shape;
      s.type = out->shape.type;
      result = Add("slice", s, {g}, slice->attrs, "", "gemm_slice");
    }
    if (keep_s32) {
      g->gemm->emit_s32 = true;
      Shape as = g->shape;
      as.type = s32;
      Instr* acc = Add("gemm-acc", as, {g}, "", "", "acc");
      g->gemm->acc = acc;
      Instr* acc_out = acc;
      if (slice != nullptr) acc_out = Add("slice", slice->shape, {acc}, slice->attrs, "", "acc_slice");
      // every user of the s32 value other than the dequantisation chain now reads the second result
      for (auto& i : comp_->instrs)
        if (i.get() != cf && i.get() != result && i.get() != acc && i.get() != acc_out && i.get() != slice)
          for (Instr*& o : i->operands)
            if (o == top) o = acc_out;
      if (root_ == top) root_ = acc_out;
    }
    Replace(out, result);
  }
  // A narrowing convert right behind a call simply becomes the call's output type.
  void FoldNarrowingConvert(Instr* g) {
    if (!g->gemm->f8 || g->shape.type != "f32" || g->gemm->has_c) return;
    Instr* top = g;
    std::vector<Instr*> chain;
    while (UserCount(top) == 1 && !ValueUsers(top).empty() && (ValueUsers(top)[0]->opcode == "slice" || ValueUsers(top)[0]->opcode == "bitcast")) {
      top = ValueUsers(top)[0];
      chain.push_back(top);
    }
    if (UserCount(top) != 1 || ValueUsers(top).empty()) return;
    Instr* conv = ValueUsers(top)[0];
    if (conv->opcode != "convert" || !(conv->shape.type == "bf16" || conv->shape.type == "f16")) return;
    if (g->gemm->has_bias) {
      // the vector bias type must still go with the narrower output (compatible_bias_type of FuseVectorBiasAdd)
      const std::string& bt = g->operands[g->gemm->ScaleIndex() + 2]->shape.type;
      if (!((bt == "bf16" && conv->shape.type == "bf16") || (bt == "f16" && conv->shape.type == "f16"))) return;
    }
    g->shape.type = conv->shape.type;
    for (Instr* c : chain) c->shape.type = conv->shape.type;
    dirty_ = true;
    Replace(conv, top);
  }

  Computation* comp_;
  const std::vector<Computation>* all_;
  Instr* root_ = nullptr;
  std::set<std::string> names_;
  std::vector<Instr*> calls_;
  std::vector<std::pair<std::string, std::string>> refusals_;
  mutable bool dirty_ = true;
  mutable std::set<Instr*> live_;
  mutable std::map<Instr*, std::vector<Instr*>> users_;
};

// ------------------------------------------------------------------------------------------ output
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
std::string JsonStr(const std::string& s) {
  std::string o = "\"";
  for (char c : s) { if (c == '"' || c == '\\') o += '\\'; o += c; }
  return o + "\"";
}
std::string Dims(const Shape& s) { return "[" + JoinInts(s.dims) + "]"; }

Shape CallTupleShape(const Instr* g) {
  Shape t;
  t.type = "tuple";
  t.elements.push_back(g->shape);
  if (g->gemm->damax) t.elements.push_back(MakeShape("f32", {}));
  if (g->gemm->emit_s32) { Shape a = g->shape; a.type = "s32"; t.elements.push_back(a); }
  t.elements.push_back(MakeShape("s8", {kWorkspaceBytes}));   // appended to every cuBLASLt matmul, FP8 or not
  return t;
}

std::string Rewriter::EmitHlo(const Module& m) const {
  std::ostringstream o;
  o << "HloModule " << (m.name.empty() ? "module" : m.name) << "_rewritten\n\n";
  for (const Computation& c : m.computations)
    if (!c.is_entry) o << c.raw << "\n";
  o << "ENTRY " << comp_->name << " {\n";
  std::set<const Instr*> done;
  std::function<void(const Instr*)> emit = [&](const Instr* i) {
    if (done.count(i)) return;
    done.insert(i);
    for (const Instr* op : i->operands) emit(op);
    const char* lead = i == root_ ? "  ROOT " : "  ";
    if (i->gemm) {
      const Gemm& g = *i->gemm;
      o << "  " << i->name << ".call = " << CallTupleShape(i).ToString() << " custom-call(";
      for (size_t k = 0; k < i->operands.size(); ++k) o << (k ? ", " : "") << i->operands[k]->name;
      o << "), custom_call_target=\"" << (g.mx ? "b200$block_scaled_dot$mx" : g.f8 ? "b200$scaled_dot$f8" : "b200$dot$s8")
        << "\", api_version=API_VERSION_TYPED_FFI, backend_config={";
      // lhs_stride / rhs_stride as the reference's rewriter writes them: the dense extent of one batch entry of each
      // operand as passed (gemm_rewriter.cc:705-721).
      auto entry_extent = [](const Instr* x) {
        const auto& d = x->shape.dims;
        return d.size() >= 2 ? d[d.size() - 2] * d[d.size() - 1] : int64_t(0);
      };
      const int64_t lhs_stride = entry_extent(i->operands[0]), rhs_stride = entry_extent(i->operands[1]);
      if (g.mx) {
        o << "alpha_real = " << F64(g.alpha) << " : f64";
        if (g.explicit_block) o << ", block_size = " << g.explicit_block << " : i64";
        o << "}\n";
      } else if (g.f8) {
        o << "alpha_real = " << F64(g.alpha) << " : f64, beta = " << F64(g.beta) << " : f64, epilogue = " << g.epilogue
          << " : i32, lhs_contracting_dim = " << g.lhs_contracting << " : i64, rhs_contracting_dim = " << g.rhs_contracting
          << " : i64, damax_output = " << (g.damax ? "true" : "false")
          << (g.batched ? ", lhs_batch_dims = array<i64: 0>, rhs_batch_dims = array<i64: 0>" : "") << ", lhs_stride = " << lhs_stride
          << " : i64, rhs_stride = " << rhs_stride << " : i64, selected_config = 0 : i64}\n";
      } else {
        o << "lhs_contracting_dim = " << g.lhs_contracting << " : i64, rhs_contracting_dim = " << g.rhs_contracting
          << " : i64, emit_s32 = " << (g.emit_s32 ? "true" : "false")
          << (g.batched ? ", lhs_batch_dims = array<i64: 0>, rhs_batch_dims = array<i64: 0>" : "") << ", lhs_stride = " << lhs_stride
          << " : i64, rhs_stride = " << rhs_stride << " : i64}\n";
      }
      o << lead << i->name << " = " << i->shape.ToString() << " get-tuple-element(" << i->name << ".call), index=0\n";
      return;
    }
    if (i->opcode == "gemm-amax" || i->opcode == "gemm-acc") {
      o << lead << i->name << " = " << i->shape.ToString() << " get-tuple-element(" << i->operands[0]->name << ".call), index=1\n";
      return;
    }
    o << lead << i->name << " = " << i->shape.ToString() << " " << i->opcode << "(";
    if (i->opcode == "parameter" || i->opcode == "constant") {
      o << i->literal;
    } else {
      for (size_t k = 0; k < i->operands.size(); ++k) o << (k ? ", " : "") << i->operands[k]->name;
    }
    o << ")";
    if (!i->attrs.empty()) o << ", " << i->attrs;
    o << "\n";
  };
  // Parameters first, in their own order, whether or not anything still uses them.
  std::vector<const Instr*> params;
  for (const auto& i : comp_->instrs) if (i->opcode == "parameter") params.push_back(i.get());
  std::sort(params.begin(), params.end(), [](const Instr* a, const Instr* b) { return std::atoi(a->literal.c_str()) < std::atoi(b->literal.c_str()); });
  for (const Instr* pi : params) emit(pi);
  emit(root_);
  o << "}\n";
  return o.str();
}

std::string Rewriter::EmitJson() const {
  // Where an operand comes from, looking back through data-movement ops to a parameter or constant.
  auto describe = [&](const Instr* x, const std::string& role) {
    std::ostringstream j;
    const Instr* cur = x;
    bool reciprocal = false;
    std::vector<std::string> chain;
    while (true) {
      const std::string& oc = cur->opcode;
      if (oc == "bitcast" || oc == "reshape" || oc == "copy" || oc == "transpose" || oc == "pad" || oc == "convert" || oc == "slice" ||
          oc == "dynamic-slice" || oc == "broadcast") {
        chain.push_back(oc);
        cur = cur->operands[0];
      } else if (oc == "select") {
        chain.push_back(oc);
        cur = cur->operands[cur->operands[1]->opcode == "convert" ? 2 : 1];
      } else if (oc == "divide" && cur->operands.size() == 2 && cur->operands[0]->opcode == "constant") {
        reciprocal = true;
        chain.push_back(oc);
        cur = cur->operands[1];
      } else {
        break;
      }
    }
    int param = -1;
    double constant = 0.0;
    bool is_const = false;
    if (cur->opcode == "parameter") param = std::atoi(cur->literal.c_str());
    else if (cur->opcode == "constant" && cur->shape.IsScalar()) { is_const = true; constant = std::strtod(cur->literal.c_str(), nullptr); }
    std::reverse(chain.begin(), chain.end());
    j << "{\"role\": " << JsonStr(role) << ", \"name\": " << JsonStr(x->name) << ", \"param\": " << param << ", \"reciprocal\": "
      << (reciprocal ? "true" : "false") << ", \"constant\": " << (is_const ? F64(reciprocal ? 1.0 / constant : constant) : std::string("null"))
      << ", \"dtype\": " << TypeCode(x->shape.type) << ", \"dims\": " << Dims(x->shape) << ", \"source\": " << JsonStr(cur->name)
      << ", \"source_opcode\": " << JsonStr(cur->opcode) << ", \"source_dims\": " << Dims(cur->shape) << ", \"source_dtype\": " << TypeCode(cur->shape.type) << ", \"chain\": [";
    for (size_t i = 0; i < chain.size(); ++i) j << (i ? ", " : "") << JsonStr(chain[i]);
    j << "]}";
    return j.str();
  };
  std::ostringstream calls;
  size_t n_calls = 0;
  std::string first;
  for (Instr* g : calls_) {
    if (!IsLive(g)) continue;
    const Gemm& c = *g->gemm;
    std::vector<std::string> roles = {"a", "b"};
    if (c.mx) {
      roles.push_back("a_scale");
      roles.push_back("b_scale");
    } else if (c.f8) {
      if (c.has_c) roles.push_back("c");
      roles.push_back("a_scale");
      roles.push_back("b_scale");
      if (c.has_bias) roles.push_back("bias");
      if (c.has_d_scale) roles.push_back("d_scale");
    } else if (c.has_dequant) {
      roles.push_back("a_row_scale");
      roles.push_back("b_col_scale");
    }
    std::ostringstream j;
    j << "{\"name\": " << JsonStr(g->name) << ", \"target\": " << JsonStr(c.mx ? "b200$block_scaled_dot$mx" : c.f8 ? "b200$scaled_dot$f8" : "b200$dot$s8") << ", \"m\": " << c.m
      << ", \"n\": " << c.n << ", \"k\": " << c.k << ", \"batch\": " << c.batch << ", \"swapped\": " << (c.swapped ? "true" : "false")
      << ", \"operands\": [";
    for (size_t i = 0; i < g->operands.size(); ++i) j << (i ? ", " : "") << describe(g->operands[i], i < roles.size() ? roles[i] : "?");
    j << "], \"results\": [{\"role\": \"d\", \"dtype\": " << TypeCode(g->shape.type) << ", \"dims\": " << Dims(g->shape) << "}";
    if (c.damax) j << ", {\"role\": \"amax\", \"dtype\": 11, \"dims\": []}";
    if (c.emit_s32) j << ", {\"role\": \"acc\", \"dtype\": 4, \"dims\": " << Dims(g->shape) << "}";
    j << ", {\"role\": \"workspace\", \"dtype\": 2, \"dims\": [" << kWorkspaceBytes << "]}], \"attrs\": {";
    auto entry_extent = [](const Instr* x) {
      const auto& d = x->shape.dims;
      return d.size() >= 2 ? d[d.size() - 2] * d[d.size() - 1] : int64_t(0);
    };
    std::ostringstream strides;
    strides << ", \"lhs_stride\": " << entry_extent(g->operands[0]) << ", \"rhs_stride\": " << entry_extent(g->operands[1]);
    if (c.mx) {
      j << "\"alpha_real\": " << F64(c.alpha);
      if (c.explicit_block) j << ", \"block_size\": " << c.explicit_block;
    } else if (c.f8) {
      j << "\"alpha_real\": " << F64(c.alpha) << ", \"beta\": " << F64(c.beta) << ", \"epilogue\": " << c.epilogue
        << ", \"lhs_contracting_dim\": " << c.lhs_contracting << ", \"rhs_contracting_dim\": " << c.rhs_contracting
        << ", \"damax_output\": " << (c.damax ? "true" : "false")
        << (c.batched ? ", \"lhs_batch_dims\": [0], \"rhs_batch_dims\": [0]" : "") << strides.str();
    } else {
      j << "\"lhs_contracting_dim\": " << c.lhs_contracting << ", \"rhs_contracting_dim\": " << c.rhs_contracting << ", \"emit_s32\": "
        << (c.emit_s32 ? "true" : "false") << (c.batched ? ", \"lhs_batch_dims\": [0], \"rhs_batch_dims\": [0]" : "") << strides.str();
    }
    j << "}}";
    if (n_calls == 0) first = j.str();
    calls << (n_calls ? ", " : "") << j.str();
    ++n_calls;
  }
  std::ostringstream out;
  out << "{\"rewritten\": " << (n_calls ? "true" : "false") << ", \"calls\": [" << calls.str() << "], \"not_rewritten\": [";
  for (size_t i = 0; i < refusals_.size(); ++i)
    out << (i ? ", " : "") << "{\"dot\": " << JsonStr(refusals_[i].first) << ", \"reason\": " << JsonStr(refusals_[i].second) << "}";
  out << "]";
  if (n_calls == 0) out << ", \"reason\": " << JsonStr(refusals_.empty() ? std::string("no dot") : refusals_[0].second);
  else out << ", " << first.substr(1, first.size() - 2);     // the first call's fields again at the top level, for callers that deal with one call
  out << "}";
  return out.str();
}

int Copy(const std::string& s, char* out, size_t len) {
  if (out == nullptr || len == 0) return 0;
  if (s.size() + 1 > len) return 8;   // RESOURCE_EXHAUSTED
  std::memcpy(out, s.c_str(), s.size() + 1);
  return 0;
}

}  // namespace

// Rewrites the scaled-dot patterns of an HLO module (text) onto this library's custom calls.
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
  if (entry->instrs.empty()) return fail(3, "the entry computation is empty");
  Rewriter rw(entry, &m.computations);
  if (!rw.Resolve(&perr)) return fail(3, perr);
  rw.Run();
  const std::string json = rw.EmitJson();
  const std::string hlo = rw.AnyRewritten() ? rw.EmitHlo(m) : std::string(hlo_text);
  if (int rc = Copy(hlo, out_hlo, out_hlo_len)) return fail(rc, "out_hlo buffer too small");
  if (int rc = Copy(json, plan_json, plan_json_len)) return fail(rc, "plan_json buffer too small");
  if (err != nullptr && err_len > 0) err[0] = '\0';
  return 0;
}

// Stand-alone front end for HTile programs: reader, verifier, the dot-transpose-to-load-order rewrite,
// printer and a JSON view of the object model.  Interface and the reference files it stands in for:
// include/htile_front.h.  Host code only.
#include "htile_front.h"

#include <cctype>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace htf {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

std::string format(const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return buf;
}

// ---------------------------------------------------------------------------------------------
// object model
// ---------------------------------------------------------------------------------------------
struct Type {
  enum Kind { Scalar, MemRef, Tensor } kind = Scalar;
  std::vector<long long> shape;
  std::string elem;       // f16, bf16, f32, f64, index, i1 ... i64
  std::string placement;  // "shared", "local" or "" (tensors only)

  std::string str() const {
    if (kind == Scalar) return elem;
    std::string body;
    for (long long d : shape) body += std::to_string(d) + "x";
    body += elem;
    if (kind == MemRef) return "memref<" + body + ">";
    if (!placement.empty()) body += ", #htile.encoding<placement = " + placement + ">";
    return "tensor<" + body + ">";
  }
  bool operator==(const Type &o) const {
    return kind == o.kind && shape == o.shape && elem == o.elem && placement == o.placement;
  }
};

struct Attr {
  enum Kind { Bool, Int, Float, Str, Array } kind = Bool;
  bool b = true;  // unit attributes and the keywords true / unit read as true
  long long i = 0;
  double f = 0.0;
  std::string s;
  std::vector<Attr> arr;
};
using AttrDict = std::vector<std::pair<std::string, Attr>>;

const Attr *find(const AttrDict &d, const std::string &key) {
  for (const auto &kv : d)
    if (kv.first == key) return &kv.second;
  return nullptr;
}
void set(AttrDict &d, const std::string &key, Attr v) {
  for (auto &kv : d)
    if (kv.first == key) {
      kv.second = std::move(v);
      return;
    }
  d.emplace_back(key, std::move(v));
}
void erase(AttrDict &d, const std::string &key) {
  for (size_t i = 0; i < d.size(); ++i)
    if (d[i].first == key) {
      d.erase(d.begin() + i);
      return;
    }
}
bool truthy(const Attr *a) {
  if (!a) return false;
  switch (a->kind) {
    case Attr::Bool: return a->b;
    case Attr::Int: return a->i != 0;
    case Attr::Float: return a->f != 0.0;
    case Attr::Str: return !a->s.empty();
    case Attr::Array: return !a->arr.empty();
  }
  return false;
}

struct Op;
struct Block;
struct Value {
  int id = 0;
  std::string name;
  Type type;
  Op *owner_op = nullptr;        // result of an operation, or
  Block *owner_block = nullptr;  // block argument
};

struct Block {
  std::vector<Value *> args;
  std::vector<std::unique_ptr<Op>> ops;
  Op *parent_op = nullptr;
};

struct Op {
  std::string name;
  std::vector<Value *> operands;
  std::vector<Value *> results;
  AttrDict attrs;
  std::vector<std::unique_ptr<Block>> regions;
  Block *parent = nullptr;
};

struct Func {
  std::string name;
  AttrDict attrs;
  std::unique_ptr<Block> body;
};

struct Module {
  std::vector<std::unique_ptr<Func>> funcs;
  std::deque<Value> values;  // arena: addresses stay valid

  Value *new_value(const std::string &name, const Type &t) {
    values.emplace_back();
    Value &v = values.back();
    v.id = static_cast<int>(values.size()) - 1;
    v.name = name;
    v.type = t;
    return &v;
  }
};

template <class F> void walk(Block &b, F &&f) {
  // snapshot: the callback may insert or erase operations of this block
  std::vector<Op *> ops;
  for (auto &o : b.ops) ops.push_back(o.get());
  for (Op *o : ops) {
    f(*o);
    for (auto &r : o->regions) walk(*r, f);
  }
}
template <class F> void walk(Module &m, F &&f) {
  for (auto &fn : m.funcs) walk(*fn->body, f);
}

// ---------------------------------------------------------------------------------------------
// reader
// ---------------------------------------------------------------------------------------------
const char *const kScalars[] = {"bf16", "f16", "f32", "f64", "index", "i16", "i32", "i64", "i1", "i8"};

const std::set<std::string> kBinary = {
    "arith.addf", "arith.subf", "arith.mulf", "arith.divf", "arith.maximumf", "arith.minimumf", "arith.addi",
    "arith.subi", "arith.muli", "arith.divsi", "arith.remsi", "arith.maxsi", "arith.minsi", "arith.andi", "arith.ori"};
const std::set<std::string> kUnary = {"math.exp2", "math.exp", "math.log2", "math.log",
                                      "math.sqrt", "math.rsqrt", "math.tanh", "arith.negf"};
const std::set<std::string> kCasts = {"arith.truncf", "arith.extf", "arith.sitofp", "arith.fptosi", "arith.index_cast"};

bool ident_start(char c) { return std::isalpha(static_cast<unsigned char>(c)) || c == '_'; }
bool ident_char(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$'; }

class Parser {
 public:
  Parser(const char *text, Module &m) : t_(text), n_(std::strlen(text)), m_(m) {}

  void module() {
    scopes_.emplace_back();
    while (true) {
      ws();
      if (pos_ >= n_) break;
      if (t_[pos_] == '#' && alias_definition()) continue;
      if (keyword("module")) {
        if (keyword("attributes")) attr_dict();
        expect("{");
        while (!accept("}")) func();
        continue;
      }
      func();
    }
  }

  Type type_only() { return type(); }

 private:
  const char *t_;
  size_t n_, pos_ = 0;
  Module &m_;
  std::map<std::string, std::string> aliases_;
  std::vector<std::map<std::string, Value *>> scopes_;

  [[noreturn]] void fail(const std::string &msg) {
    int line = 1;
    for (size_t i = 0; i < pos_ && i < n_; ++i) line += t_[i] == '\n';
    std::string snippet;
    for (size_t i = pos_; i < n_ && i < pos_ + 40 && t_[i] != '\n'; ++i) snippet += t_[i];
    throw Error(format("line %d: %s (at '%s')", line, msg.c_str(), snippet.c_str()));
  }

  void ws() {
    while (pos_ < n_) {
      if (std::isspace(static_cast<unsigned char>(t_[pos_]))) {
        ++pos_;
      } else if (t_[pos_] == '/' && pos_ + 1 < n_ && t_[pos_ + 1] == '/') {
        while (pos_ < n_ && t_[pos_] != '\n') ++pos_;
      } else {
        break;
      }
    }
  }
  bool peek(const char *s) {
    ws();
    return std::strncmp(t_ + pos_, s, std::strlen(s)) == 0;
  }
  bool accept(const char *s) {
    if (!peek(s)) return false;
    pos_ += std::strlen(s);
    return true;
  }
  void expect(const char *s) {
    if (!accept(s)) fail(std::string("expected '") + s + "'");
  }
  bool try_ident(std::string &out) {
    ws();
    if (pos_ >= n_ || !ident_start(t_[pos_])) return false;
    size_t e = pos_ + 1;
    while (e < n_ && ident_char(t_[e])) ++e;
    out.assign(t_ + pos_, e - pos_);
    pos_ = e;
    return true;
  }
  bool keyword(const char *word) {
    const size_t save = pos_;
    std::string id;
    if (try_ident(id) && id == word) return true;
    pos_ = save;
    return false;
  }
  std::string ident() {
    std::string id;
    if (!try_ident(id)) fail("expected identifier");
    return id;
  }

  bool alias_definition() {  // #name = rest of the line
    size_t p = pos_ + 1;
    if (p >= n_ || !ident_start(t_[p])) return false;
    size_t e = p + 1;
    while (e < n_ && (std::isalnum(static_cast<unsigned char>(t_[e])) || t_[e] == '_')) ++e;
    size_t q = e;
    while (q < n_ && (t_[q] == ' ' || t_[q] == '\t')) ++q;
    if (q >= n_ || t_[q] != '=') return false;
    ++q;
    while (q < n_ && (t_[q] == ' ' || t_[q] == '\t')) ++q;
    size_t eol = q;
    while (eol < n_ && t_[eol] != '\n') ++eol;
    if (eol == q) return false;
    std::string rest(t_ + q, eol - q);
    while (!rest.empty() && std::isspace(static_cast<unsigned char>(rest.back()))) rest.pop_back();
    aliases_[std::string(t_ + p, e - p)] = rest;
    pos_ = eol;
    return true;
  }

  // -- SSA scopes --
  Value *define(Value *v) {
    scopes_.back()[v->name] = v;
    return v;
  }
  Value *lookup(const std::string &name) {
    for (auto it = scopes_.rbegin(); it != scopes_.rend(); ++it) {
      auto f = it->find(name);
      if (f != it->end()) return f->second;
    }
    fail("use of undefined value %" + name);
  }
  std::string ssa_name() {
    ws();
    if (pos_ >= n_ || t_[pos_] != '%') fail("expected SSA value");
    size_t e = pos_ + 1;
    while (e < n_ && (std::isalnum(static_cast<unsigned char>(t_[e])) || std::strchr("_.$-", t_[e]))) ++e;
    if (e == pos_ + 1) fail("expected SSA value");
    std::string name(t_ + pos_ + 1, e - pos_ - 1);
    pos_ = e;
    return name;
  }
  Value *ssa_use() { return lookup(ssa_name()); }
  void ssa_use_list(const char *close, std::vector<Value *> &out) {
    if (accept(close)) return;
    while (true) {
      out.push_back(ssa_use());
      if (accept(close)) return;
      expect(",");
    }
  }

  // -- types --
  static bool is_scalar(const std::string &s) {
    for (const char *k : kScalars)
      if (s == k) return true;
    return false;
  }
  Type type() {
    ws();
    for (const char *kind : {"memref", "tensor"}) {
      const size_t kl = std::strlen(kind);
      if (std::strncmp(t_ + pos_, kind, kl) == 0 && pos_ + kl < n_ && t_[pos_ + kl] == '<') {
        const size_t start = pos_ + kl + 1;
        int depth = 1;
        size_t i = start;
        while (depth) {
          if (i >= n_) fail("unterminated type");
          if (t_[i] == '<') ++depth;
          if (t_[i] == '>') --depth;
          ++i;
        }
        const std::string body(t_ + start, i - 1 - start);
        pos_ = i;
        return shaped(kind, body);
      }
    }
    std::string id;
    const size_t save = pos_;
    if (try_ident(id) && is_scalar(id)) {
      Type t;
      t.elem = id;
      return t;
    }
    pos_ = save;
    fail("expected type");
  }
  static std::string strip(const std::string &s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace(static_cast<unsigned char>(s[a]))) ++a;
    while (b > a && std::isspace(static_cast<unsigned char>(s[b - 1]))) --b;
    return s.substr(a, b - a);
  }
  Type shaped(const std::string &kind, const std::string &body) {
    const size_t comma = body.find(',');
    const std::string dims = strip(comma == std::string::npos ? body : body.substr(0, comma));
    std::string enc = comma == std::string::npos ? "" : strip(body.substr(comma + 1));
    Type t;
    t.kind = kind == "memref" ? Type::MemRef : Type::Tensor;
    size_t p = 0;
    while (true) {  // (\d+x)* element
      size_t e = p;
      while (e < dims.size() && std::isdigit(static_cast<unsigned char>(dims[e]))) ++e;
      if (e > p && e < dims.size() && dims[e] == 'x') {
        t.shape.push_back(std::atoll(dims.substr(p, e - p).c_str()));
        p = e + 1;
        continue;
      }
      break;
    }
    t.elem = dims.substr(p);
    if (t.elem.empty() || !std::isalpha(static_cast<unsigned char>(t.elem[0])))
      fail("dynamic or malformed shape in " + kind + "<" + body + ">");
    for (char c : t.elem)
      if (!std::isalnum(static_cast<unsigned char>(c))) fail("dynamic or malformed shape in " + kind + "<" + body + ">");
    if (!is_scalar(t.elem)) fail("unknown element type '" + t.elem + "'");
    if (t.kind == Type::MemRef) {
      if (!enc.empty()) fail("memref layouts / memory spaces are not supported");
      return t;
    }
    if (!enc.empty()) {
      if (enc[0] == '#') {
        auto it = aliases_.find(enc.substr(1));
        if (it != aliases_.end()) enc = it->second;
      }
      // #htile.encoding< placement = NAME >
      std::string squeezed;
      for (char c : enc)
        if (!std::isspace(static_cast<unsigned char>(c))) squeezed += c;
      const std::string head = "#htile.encoding<placement=";
      if (squeezed.compare(0, head.size(), head) != 0 || squeezed.back() != '>')
        fail("unknown tensor encoding '" + enc + "'");
      t.placement = squeezed.substr(head.size(), squeezed.size() - head.size() - 1);
      if (t.placement != "shared" && t.placement != "local") fail("unknown tensor encoding '" + enc + "'");
    }
    return t;
  }

  // -- attributes --
  bool number(Attr &out) {
    ws();
    size_t p = pos_;
    if (p < n_ && (t_[p] == '-' || t_[p] == '+')) ++p;
    const size_t digits0 = p;
    bool is_int = true;
    if (p + 1 < n_ && t_[p] == '0' && t_[p + 1] == 'x' && p + 2 < n_ && std::isxdigit(static_cast<unsigned char>(t_[p + 2]))) {
      p += 2;
      while (p < n_ && std::isxdigit(static_cast<unsigned char>(t_[p]))) ++p;
    } else {
      while (p < n_ && std::isdigit(static_cast<unsigned char>(t_[p]))) ++p;
      if (p == digits0) return false;
      auto exponent = [&](size_t q) -> size_t {  // [eE][-+]?\d+ starting at q, or q if absent
        if (q < n_ && (t_[q] == 'e' || t_[q] == 'E')) {
          size_t r = q + 1;
          if (r < n_ && (t_[r] == '-' || t_[r] == '+')) ++r;
          const size_t d0 = r;
          while (r < n_ && std::isdigit(static_cast<unsigned char>(t_[r]))) ++r;
          if (r > d0) return r;
        }
        return q;
      };
      if (p < n_ && t_[p] == '.') {
        is_int = false;
        ++p;
        while (p < n_ && std::isdigit(static_cast<unsigned char>(t_[p]))) ++p;
        p = exponent(p);
      } else {
        const size_t q = exponent(p);
        if (q != p) is_int = false;
        p = q;
      }
    }
    const std::string txt(t_ + pos_, p - pos_);
    pos_ = p;
    if (is_int) {
      out.kind = Attr::Int;
      out.i = std::strtoll(txt.c_str(), nullptr, 0);
    } else {
      out.kind = Attr::Float;
      out.f = std::strtod(txt.c_str(), nullptr);
    }
    return true;
  }
  Attr attr_value() {
    ws();
    Attr a;
    if (accept("array<")) {
      ident();  // i64 / i1
      a.kind = Attr::Array;
      if (accept(":")) {
        while (true) {
          a.arr.push_back(attr_value());
          if (!accept(",")) break;
        }
      }
      expect(">");
      return a;
    }
    if (accept("[")) {
      a.kind = Attr::Array;
      if (!accept("]")) {
        while (true) {
          a.arr.push_back(attr_value());
          if (accept("]")) break;
          expect(",");
        }
      }
      return a;
    }
    if (pos_ < n_ && t_[pos_] == '"') {
      size_t e = pos_ + 1;
      while (e < n_ && t_[e] != '"') e += (t_[e] == '\\' && e + 1 < n_) ? 2 : 1;
      if (e >= n_) fail("unterminated string");
      a.kind = Attr::Str;
      a.s.assign(t_ + pos_ + 1, e - pos_ - 1);
      pos_ = e + 1;
      return a;
    }
    if (keyword("true") || keyword("unit")) return a;
    if (keyword("false")) {
      a.b = false;
      return a;
    }
    if (number(a)) {
      if (accept(":")) type();
      return a;
    }
    fail("unsupported attribute value");
  }
  Attr attr_value_no_type() {
    Attr a;
    if (number(a)) return a;
    if (keyword("true")) return a;
    if (keyword("false")) {
      a.b = false;
      return a;
    }
    fail("expected a numeric constant");
  }
  AttrDict attr_dict() {
    AttrDict d;
    if (!accept("{")) return d;
    if (accept("}")) return d;
    while (true) {
      std::string key;
      if (!try_ident(key)) fail("expected attribute name");
      Attr v;
      if (accept("=")) v = attr_value();
      set(d, key, std::move(v));
      if (accept("}")) return d;
      expect(",");
    }
  }
  void update(AttrDict &into, const AttrDict &from) {
    for (const auto &kv : from) set(into, kv.first, kv.second);
  }

  // -- functions, blocks, operations --
  void func() {
    if (!keyword("func.func")) fail("expected func.func");
    if (!keyword("private")) keyword("public");
    expect("@");
    auto fn = std::make_unique<Func>();
    fn->name = ident();
    fn->body = std::make_unique<Block>();
    expect("(");
    scopes_.emplace_back();
    if (!accept(")")) {
      while (true) {
        const std::string an = ssa_name();
        expect(":");
        Value *v = m_.new_value(an, type());
        v->owner_block = fn->body.get();
        fn->body->args.push_back(define(v));
        if (accept(")")) break;
        expect(",");
      }
    }
    if (accept("->")) fail("functions with results are not supported");
    if (keyword("attributes")) fn->attrs = attr_dict();
    expect("{");
    block_body(*fn->body, "}");
    scopes_.pop_back();
    m_.funcs.push_back(std::move(fn));
  }
  void block_body(Block &b, const char *close) {
    while (!accept(close)) {
      std::unique_ptr<Op> op = operation();
      op->parent = &b;
      b.ops.push_back(std::move(op));
    }
  }
  std::unique_ptr<Op> operation() {
    ws();
    std::vector<std::string> result_names;
    if (peek("%")) {
      while (true) {
        result_names.push_back(ssa_name());
        if (accept(":")) fail("result packs (%x:N) are not supported; name each result");
        if (!accept(",")) break;
      }
      expect("=");
    }
    auto op = std::make_unique<Op>();
    op->name = ident();
    const std::vector<Type> types = op_body(*op);
    if (types.size() != result_names.size())
      fail(format("%s: %zu result names for %zu results", op->name.c_str(), result_names.size(), types.size()));
    for (size_t i = 0; i < types.size(); ++i) {
      Value *v = m_.new_value(result_names[i], types[i]);
      v->owner_op = op.get();
      op->results.push_back(define(v));
    }
    return op;
  }
  std::vector<Type> arrow_types() {
    expect(":");
    type();
    expect("->");
    return {type()};
  }
  void need_keyword(const char *w) {
    if (!keyword(w)) fail(std::string("expected '") + w + "'");
  }

  std::vector<Type> op_body(Op &op) {
    const std::string &n = op.name;
    if (n == "return" || n == "func.return" || n == "gpu.terminator") return {};
    if (n == "arith.constant") {
      ws();
      set(op.attrs, "value", attr_value_no_type());
      expect(":");
      return {type()};
    }
    if (kBinary.count(n)) {
      op.operands.push_back(ssa_use());
      expect(",");
      op.operands.push_back(ssa_use());
      update(op.attrs, attr_dict());
      expect(":");
      return {type()};
    }
    if (kUnary.count(n)) {
      op.operands.push_back(ssa_use());
      update(op.attrs, attr_dict());
      expect(":");
      return {type()};
    }
    if (kCasts.count(n)) {
      op.operands.push_back(ssa_use());
      expect(":");
      type();
      need_keyword("to");
      return {type()};
    }
    if (n == "arith.cmpi" || n == "arith.cmpf") {
      Attr p;
      p.kind = Attr::Str;
      p.s = ident();
      set(op.attrs, "predicate", p);
      expect(",");
      op.operands.push_back(ssa_use());
      expect(",");
      op.operands.push_back(ssa_use());
      expect(":");
      Type ty = type();
      ty.elem = "i1";
      if (ty.kind != Type::Tensor) ty = Type{Type::Scalar, {}, "i1", ""};
      return {ty};
    }
    if (n == "arith.select") {
      op.operands.push_back(ssa_use());
      for (int k = 0; k < 2; ++k) {
        expect(",");
        op.operands.push_back(ssa_use());
      }
      expect(":");
      Type ty = type();
      if (accept(",")) ty = type();
      return {ty};
    }
    if (n == "tensor.empty") {
      expect("(");
      expect(")");
      expect(":");
      return {type()};
    }
    if (n == "linalg.broadcast") {
      need_keyword("ins");
      expect("(");
      op.operands.push_back(ssa_use());
      expect(":");
      type();
      expect(")");
      need_keyword("outs");
      expect("(");
      op.operands.push_back(ssa_use());
      expect(":");
      const Type out_ty = type();
      expect(")");
      need_keyword("dimensions");
      expect("=");
      set(op.attrs, "dimensions", attr_value());
      return {out_ty};
    }
    if (n == "htile.hello") {
      update(op.attrs, attr_dict());
      return {};
    }
    if (n == "htile.load" || n == "htile.gather_nd") {
      op.operands.push_back(ssa_use());
      expect("[");
      ssa_use_list("]", op.operands);
      update(op.attrs, attr_dict());
      expect(":");
      type();
      while (accept(",")) type();
      expect("->");
      return {type()};
    }
    if (n == "htile.store") {
      op.operands.push_back(ssa_use());
      expect(",");
      op.operands.push_back(ssa_use());
      expect("[");
      ssa_use_list("]", op.operands);
      update(op.attrs, attr_dict());
      expect(":");
      type();
      expect(",");
      type();
      return {};
    }
    if (n == "htile.dot") {
      op.operands.push_back(ssa_use());
      expect(",");
      op.operands.push_back(ssa_use());
      if (accept(",")) op.operands.push_back(ssa_use());
      update(op.attrs, attr_dict());
      if (const Attr *pol = find(op.attrs, "warp_policy")) {  // include/HTile/HTileOps.td:11-19
        if (pol->kind != Attr::Str || (pol->s != "square" && pol->s != "full_row" && pol->s != "full_col"))
          fail("htile.dot: invalid warp_policy '" + pol->s + "'");
      }
      expect(":");
      for (size_t k = 0; k < op.operands.size(); ++k) {
        type();
        accept(",");
      }
      expect("->");
      return {type()};
    }
    if (n == "htile.reduce") {
      op.operands.push_back(ssa_use());
      need_keyword("axis");
      set(op.attrs, "axis", attr_value());
      need_keyword("kind");
      set(op.attrs, "kind", attr_value());
      update(op.attrs, attr_dict());
      return arrow_types();
    }
    if (n == "htile.full" || n == "htile.copy") {
      op.operands.push_back(ssa_use());
      update(op.attrs, attr_dict());
      return arrow_types();
    }
    if (n == "htile.permute" || n == "htile.unsqueeze") {
      op.operands.push_back(ssa_use());
      const char *key = n == "htile.permute" ? "permutation" : "mask";
      need_keyword(key);
      set(op.attrs, key, attr_value());
      update(op.attrs, attr_dict());
      return arrow_types();
    }
    if (n == "htile.arange") {
      op.operands.push_back(ssa_use());
      need_keyword("to");
      op.operands.push_back(ssa_use());
      update(op.attrs, attr_dict());
      expect(":");
      return {type()};
    }
    if (n == "scf.yield") {
      if (peek("%")) {
        while (true) {
          op.operands.push_back(ssa_use());
          if (!accept(",")) break;
        }
        expect(":");
        for (size_t k = 0; k < op.operands.size(); ++k) {
          type();
          if (k + 1 < op.operands.size()) expect(",");
        }
      }
      return {};
    }
    if (n == "scf.for") return scf_for(op);
    if (n == "gpu.launch") return gpu_launch(op);
    fail("unsupported operation '" + n + "'");
  }

  std::vector<Type> scf_for(Op &op) {
    const std::string iv = ssa_name();
    expect("=");
    op.operands.push_back(ssa_use());
    need_keyword("to");
    op.operands.push_back(ssa_use());
    need_keyword("step");
    op.operands.push_back(ssa_use());
    auto body = std::make_unique<Block>();
    body->parent_op = &op;
    std::vector<std::string> iter_names;
    if (keyword("iter_args")) {
      expect("(");
      while (true) {
        iter_names.push_back(ssa_name());
        expect("=");
        op.operands.push_back(ssa_use());
        if (accept(")")) break;
        expect(",");
      }
    }
    std::vector<Type> types;
    if (accept("->")) {
      expect("(");
      while (true) {
        types.push_back(type());
        if (accept(")")) break;
        expect(",");
      }
    }
    if (types.size() != iter_names.size()) fail("scf.for: iter_args and result types differ in number");
    scopes_.emplace_back();
    Value *ivv = m_.new_value(iv, Type{Type::Scalar, {}, "index", ""});
    ivv->owner_block = body.get();
    body->args.push_back(define(ivv));
    for (size_t k = 0; k < iter_names.size(); ++k) {
      Value *v = m_.new_value(iter_names[k], types[k]);
      v->owner_block = body.get();
      body->args.push_back(define(v));
    }
    expect("{");
    block_body(*body, "}");
    scopes_.pop_back();
    op.regions.push_back(std::move(body));
    update(op.attrs, attr_dict());
    return types;
  }

  std::vector<Type> gpu_launch(Op &op) {
    auto body = std::make_unique<Block>();
    body->parent_op = &op;
    scopes_.emplace_back();
    const Type index{Type::Scalar, {}, "index", ""};
    std::vector<Value *> sizes;
    for (const char *word : {"blocks", "threads"}) {
      need_keyword(word);
      expect("(");
      std::vector<std::string> ids;
      while (true) {
        ids.push_back(ssa_name());
        if (accept(")")) break;
        expect(",");
      }
      need_keyword("in");
      expect("(");
      std::vector<std::string> size_names;
      while (true) {
        size_names.push_back(ssa_name());
        expect("=");
        op.operands.push_back(ssa_use());
        if (accept(")")) break;
        expect(",");
      }
      if (ids.size() != 3 || size_names.size() != 3) fail("gpu.launch needs three ids and three sizes per level");
      for (const auto &nm : ids) {
        Value *v = m_.new_value(nm, index);
        v->owner_block = body.get();
        body->args.push_back(define(v));
      }
      for (const auto &nm : size_names) {
        Value *v = m_.new_value(nm, index);
        v->owner_block = body.get();
        sizes.push_back(v);
      }
    }
    // block arguments: 3 block ids, 3 thread ids, then the 6 sizes (as in the upstream op)
    for (Value *v : sizes) body->args.push_back(define(v));
    expect("{");
    block_body(*body, "}");
    scopes_.pop_back();
    op.regions.push_back(std::move(body));
    return {};
  }
};

// ---------------------------------------------------------------------------------------------
// verifier
// ---------------------------------------------------------------------------------------------
bool int_array(const Attr *a, std::vector<long long> &out) {
  if (!a || a->kind != Attr::Array) return false;
  out.clear();
  for (const Attr &e : a->arr) {
    if (e.kind != Attr::Int) return false;
    out.push_back(e.i);
  }
  return true;
}
bool is_permutation(const std::vector<long long> &p, size_t rank) {
  if (p.size() != rank) return false;
  std::vector<bool> seen(rank, false);
  for (long long v : p) {
    if (v < 0 || static_cast<size_t>(v) >= rank || seen[v]) return false;
    seen[v] = true;
  }
  return true;
}

void verify_op(const Op &op) {
  const std::string &n = op.name;
  auto bad = [&](const std::string &msg) { throw Error(n + ": " + msg); };
  auto tensor = [&](const Value *v, const char *what) -> const Type & {
    if (v->type.kind != Type::Tensor) bad(std::string(what) + " must be a tensor, got " + v->type.str());
    return v->type;
  };
  if (n == "htile.dot") {
    if (op.operands.size() < 2 || op.operands.size() > 3 || op.results.size() != 1) bad("expects two or three operands and one result");
    const Type &a = tensor(op.operands[0], "lhs"), &b = tensor(op.operands[1], "rhs"), &r = tensor(op.results[0], "result");
    if (a.shape.size() != 2 || b.shape.size() != 2 || r.shape.size() != 2) bad("operands and result must have rank 2");
    const bool ta = truthy(find(op.attrs, "transpose_a")), tb = truthy(find(op.attrs, "transpose_b"));
    const long long M = ta ? a.shape[1] : a.shape[0], Ka = ta ? a.shape[0] : a.shape[1];
    const long long Kb = tb ? b.shape[1] : b.shape[0], N = tb ? b.shape[0] : b.shape[1];
    if (Ka != Kb) bad(format("reduction extents differ: %lld and %lld", Ka, Kb));
    if (r.shape[0] != M || r.shape[1] != N) bad(format("result must be %lldx%lld, got %s", M, N, r.str().c_str()));
    if (a.elem != b.elem) bad("operand element types differ");
    if (op.operands.size() == 3 && !(op.operands[2]->type == r)) bad("accumulator type differs from the result type");
  } else if (n == "htile.reduce") {
    if (op.operands.size() != 1 || op.results.size() != 1) bad("expects one operand and one result");
    const Type &x = tensor(op.operands[0], "input"), &r = tensor(op.results[0], "result");
    const Attr *axis = find(op.attrs, "axis"), *kind = find(op.attrs, "kind");
    if (!axis || axis->kind != Attr::Int || axis->i < 0 || static_cast<size_t>(axis->i) >= x.shape.size()) bad("axis out of range");
    if (!kind || kind->kind != Attr::Str || (kind->s != "max" && kind->s != "sum" && kind->s != "min")) bad("kind must be \"max\", \"sum\" or \"min\"");
    std::vector<long long> want = x.shape;
    want.erase(want.begin() + axis->i);
    if (r.shape != want) bad("result shape is not the input shape without the reduced axis");
    if (r.elem != x.elem) bad("result element type differs from the input's");
  } else if (n == "htile.permute") {
    const Type &x = tensor(op.operands[0], "input"), &r = tensor(op.results[0], "result");
    std::vector<long long> perm;
    if (!int_array(find(op.attrs, "permutation"), perm) || !is_permutation(perm, x.shape.size())) bad("permutation is not a permutation of the input's dimensions");
    for (size_t k = 0; k < perm.size(); ++k)
      if (r.shape.size() != perm.size() || r.shape[k] != x.shape[perm[k]]) bad("result shape does not follow the permutation");  // lib/HTile/HTilePasses.cpp:22-29
    if (r.elem != x.elem) bad("result element type differs from the input's");
  } else if (n == "htile.load" || n == "htile.store") {
    const bool load = n == "htile.load";
    const size_t mem_at = load ? 0 : 1;
    if (op.operands.size() <= mem_at) bad("missing memref operand");
    const Type &mem = op.operands[mem_at]->type;
    if (mem.kind != Type::MemRef) bad("expects a memref, got " + mem.str());
    const Type &tile = load ? tensor(op.results.empty() ? op.operands[0] : op.results[0], "result") : tensor(op.operands[0], "value");
    if (op.operands.size() != mem_at + 1 + mem.shape.size()) bad(format("expects one offset per memref dimension (%zu)", mem.shape.size()));
    for (size_t k = mem_at + 1; k < op.operands.size(); ++k)
      if (op.operands[k]->type.kind != Type::Scalar || op.operands[k]->type.elem != "index") bad("offsets must be of type index");
    if (tile.shape.size() > mem.shape.size()) bad("tile rank exceeds the memref rank");
    if (tile.elem != mem.elem) bad("tile and memref element types differ");
    std::vector<long long> order;
    if (const Attr *o = find(op.attrs, "dimension_order")) {
      if (!int_array(o, order) || !is_permutation(order, tile.shape.size())) bad("dimension_order is not a permutation of the tile's dimensions");
    } else {
      for (size_t k = 0; k < tile.shape.size(); ++k) order.push_back(static_cast<long long>(k));
    }
    const size_t lead = mem.shape.size() - tile.shape.size();
    for (size_t k = 0; k < tile.shape.size(); ++k)  // result dim k reads memory tile-dim order[k]
      if (tile.shape[k] > mem.shape[lead + order[k]]) bad("tile extent exceeds the memref extent");
  } else if (n == "htile.full") {
    const Type &r = tensor(op.results[0], "result");
    if (op.operands[0]->type.kind != Type::Scalar || op.operands[0]->type.elem != r.elem) bad("scalar type differs from the result element type");
  } else if (n == "htile.copy") {
    const Type &x = tensor(op.operands[0], "input"), &r = tensor(op.results[0], "result");
    if (x.shape != r.shape || x.elem != r.elem) bad("copy changes shape or element type");
  } else if (n == "htile.arange") {
    const Type &r = tensor(op.results[0], "result");
    if (r.shape.size() != 1) bad("result must have rank 1");
  } else if (n == "linalg.broadcast") {
    const Type &x = tensor(op.operands[0], "input"), &r = tensor(op.results[0], "result");
    std::vector<long long> dims;
    if (!int_array(find(op.attrs, "dimensions"), dims) || x.shape.size() + dims.size() != r.shape.size()) bad("dimensions do not account for the rank difference");
  } else if (n == "scf.for") {
    if (op.regions.size() != 1) bad("expects one region");
    const Block &body = *op.regions[0];
    if (body.args.size() != op.results.size() + 1 || op.operands.size() != op.results.size() + 3) bad("iter_args, results and block arguments differ in number");
    if (!body.ops.empty() && body.ops.back()->name == "scf.yield") {
      const Op &y = *body.ops.back();
      if (y.operands.size() != op.results.size()) bad("scf.yield operand count differs from the loop's results");
      for (size_t k = 0; k < y.operands.size(); ++k)
        if (!(y.operands[k]->type == op.results[k]->type)) bad(format("scf.yield operand %zu has type %s, the loop carries %s", k, y.operands[k]->type.str().c_str(), op.results[k]->type.str().c_str()));
    } else if (!op.results.empty()) {
      bad("a loop with results must end in scf.yield");
    }
  } else if (kBinary.count(n)) {
    if (!(op.operands[0]->type == op.operands[1]->type) || !(op.operands[0]->type == op.results[0]->type)) bad("operand and result types differ");
  }
}

// ---------------------------------------------------------------------------------------------
// pass: htile-dot-transpose-to-load-order
// ---------------------------------------------------------------------------------------------
void replace_all_uses(Module &m, Value *from, Value *to) {
  walk(m, [&](Op &o) {
    for (Value *&v : o.operands)
      if (v == from) v = to;
  });
}
bool has_uses(Module &m, Value *v) {
  bool used = false;
  walk(m, [&](Op &o) {
    for (Value *x : o.operands) used = used || x == v;
  });
  return used;
}
size_t index_of(Block &b, Op *op) {
  for (size_t i = 0; i < b.ops.size(); ++i)
    if (b.ops[i].get() == op) return i;
  throw Error("internal: operation not in its block");
}
Op *insert_before(Op &anchor, std::unique_ptr<Op> op) {
  Block &b = *anchor.parent;
  op->parent = &b;
  Op *raw = op.get();
  b.ops.insert(b.ops.begin() + index_of(b, &anchor), std::move(op));
  return raw;
}
void erase_op(Op &op) {
  Block &b = *op.parent;
  b.ops.erase(b.ops.begin() + index_of(b, &op));
}
Attr int_array_attr(const std::vector<long long> &v) {
  Attr a;
  a.kind = Attr::Array;
  for (long long x : v) {
    Attr e;
    e.kind = Attr::Int;
    e.i = x;
    a.arr.push_back(e);
  }
  return a;
}

void dot_transpose_to_load_order(Module &m) {
  int counter = 0;
  auto fresh = [&]() { return "_t2lo" + std::to_string(++counter); };
  std::vector<Op *> dots, permutes;
  walk(m, [&](Op &o) {
    if (o.name == "htile.dot" && (truthy(find(o.attrs, "transpose_a")) || truthy(find(o.attrs, "transpose_b")))) dots.push_back(&o);
  });
  for (Op *dot : dots) {
    const std::pair<const char *, int> sides[] = {{"transpose_a", 0}, {"transpose_b", 1}};
    for (const auto &side : sides) {
      if (!truthy(find(dot->attrs, side.first))) continue;
      Value *src = dot->operands[side.second];
      if (src->type.kind != Type::Tensor || src->type.shape.size() != 2)  // lib/HTile/HTilePasses.cpp:96-97,108-109
        throw Error(std::string("htile.dot: ") + side.first + " fission expects a rank-2 " + (side.second == 0 ? "lhs" : "rhs"));
      auto permute = std::make_unique<Op>();
      permute->name = "htile.permute";
      permute->operands.push_back(src);
      set(permute->attrs, "permutation", int_array_attr({1, 0}));
      Type pt = src->type;
      std::swap(pt.shape[0], pt.shape[1]);
      Value *res = m.new_value(fresh(), pt);
      res->owner_op = permute.get();
      permute->results.push_back(res);
      insert_before(*dot, std::move(permute));
      dot->operands[side.second] = res;
      erase(dot->attrs, side.first);
    }
  }
  walk(m, [&](Op &o) {
    if (o.name == "htile.permute") permutes.push_back(&o);
  });
  for (Op *permute : permutes) {
    Op *load = permute->operands[0]->owner_op;
    if (!load || load->name != "htile.load") continue;
    std::vector<long long> perm, existing;
    if (!int_array(find(permute->attrs, "permutation"), perm)) continue;
    if (!int_array(find(load->attrs, "dimension_order"), existing)) {
      existing.clear();
      for (size_t k = 0; k < perm.size(); ++k) existing.push_back(static_cast<long long>(k));
    }
    auto fused = std::make_unique<Op>();
    fused->name = "htile.load";
    fused->operands = load->operands;
    fused->attrs = load->attrs;
    std::vector<long long> order;  // lib/HTile/HTilePasses.cpp:31-45
    for (long long p : perm) order.push_back(existing.at(static_cast<size_t>(p)));
    set(fused->attrs, "dimension_order", int_array_attr(order));
    Value *res = m.new_value(fresh(), permute->results[0]->type);
    res->owner_op = fused.get();
    fused->results.push_back(res);
    insert_before(*permute, std::move(fused));
    replace_all_uses(m, permute->results[0], res);
    erase_op(*permute);
    if (!has_uses(m, load->results[0])) erase_op(*load);
  }
}

void run_pipeline(Module &m, const std::string &pipeline) {
  std::string inner = pipeline;
  auto strip = [](std::string s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace(static_cast<unsigned char>(s[a]))) ++a;
    while (b > a && std::isspace(static_cast<unsigned char>(s[b - 1]))) --b;
    return s.substr(a, b - a);
  };
  inner = strip(inner);
  const std::string head = "builtin.module(";
  if (inner.compare(0, head.size(), head) == 0 && !inner.empty() && inner.back() == ')')
    inner = inner.substr(head.size(), inner.size() - head.size() - 1);
  size_t p = 0;
  while (p <= inner.size()) {
    const size_t comma = inner.find(',', p);
    const std::string name = strip(inner.substr(p, comma == std::string::npos ? std::string::npos : comma - p));
    if (name == "htile-dot-transpose-to-load-order") dot_transpose_to_load_order(m);
    else if (!name.empty() && name != "cse" && name != "canonicalize") throw Error("unknown pass '" + name + "'");
    if (comma == std::string::npos) break;
    p = comma + 1;
  }
}

// ---------------------------------------------------------------------------------------------
// JSON view and printer
// ---------------------------------------------------------------------------------------------
std::string json_string(const std::string &s) {
  std::string o = "\"";
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += static_cast<char>(c); }
    else if (c < 0x20) o += format("\\u%04x", c);
    else o += static_cast<char>(c);
  }
  return o + "\"";
}
std::string float_repr(double f) {  // shortest text that reads back as the same double, always with '.', 'e' or "inf"/"nan"
  char buf[64];
  for (int prec = 1; prec <= 17; ++prec) {
    snprintf(buf, sizeof(buf), "%.*g", prec, f);
    if (std::strtod(buf, nullptr) == f) break;
  }
  std::string s = buf;
  if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
  return s;
}
std::string json_attr(const Attr &a) {
  switch (a.kind) {
    case Attr::Bool: return a.b ? "true" : "false";
    case Attr::Int: return std::to_string(a.i);
    case Attr::Float: return float_repr(a.f);
    case Attr::Str: return json_string(a.s);
    case Attr::Array: {
      std::string o = "[";
      for (size_t k = 0; k < a.arr.size(); ++k) o += (k ? ", " : "") + json_attr(a.arr[k]);
      return o + "]";
    }
  }
  return "null";
}
std::string json_attrs(const AttrDict &d) {
  std::string o = "{";
  for (size_t k = 0; k < d.size(); ++k) o += (k ? ", " : "") + json_string(d[k].first) + ": " + json_attr(d[k].second);
  return o + "}";
}
std::string json_value_def(const Value *v) {
  return "{\"id\": " + std::to_string(v->id) + ", \"name\": " + json_string(v->name) + ", \"type\": " + json_string(v->type.str()) + "}";
}
void json_block(const Block &b, std::string &o);
void json_op(const Op &op, std::string &o) {
  o += "{\"name\": " + json_string(op.name) + ", \"operands\": [";
  for (size_t k = 0; k < op.operands.size(); ++k) o += (k ? ", " : "") + std::to_string(op.operands[k]->id);
  o += "], \"results\": [";
  for (size_t k = 0; k < op.results.size(); ++k) o += (k ? ", " : "") + json_value_def(op.results[k]);
  o += "], \"attributes\": " + json_attrs(op.attrs) + ", \"regions\": [";
  for (size_t k = 0; k < op.regions.size(); ++k) {
    if (k) o += ", ";
    json_block(*op.regions[k], o);
  }
  o += "]}";
}
void json_block(const Block &b, std::string &o) {
  o += "{\"arguments\": [";
  for (size_t k = 0; k < b.args.size(); ++k) o += (k ? ", " : "") + json_value_def(b.args[k]);
  o += "], \"operations\": [";
  for (size_t k = 0; k < b.ops.size(); ++k) {
    if (k) o += ", ";
    json_op(*b.ops[k], o);
  }
  o += "]}";
}
std::string to_json(const Module &m) {
  std::string o = "{\"functions\": [";
  for (size_t k = 0; k < m.funcs.size(); ++k) {
    if (k) o += ", ";
    o += "{\"name\": " + json_string(m.funcs[k]->name) + ", \"attributes\": " + json_attrs(m.funcs[k]->attrs) + ", \"body\": ";
    json_block(*m.funcs[k]->body, o);
    o += "}";
  }
  return o + "]}";
}

class Printer {
 public:
  std::string run(const Module &m) {
    out_ = "module {\n";
    for (const auto &fn : m.funcs) {
      counter_ = 0;
      std::string args;
      for (size_t k = 0; k < fn->body->args.size(); ++k)
        args += (k ? ", " : "") + fresh(fn->body->args[k], "arg" + std::to_string(k)) + ": " + fn->body->args[k]->type.str();
      out_ += "  func.func @" + fn->name + "(" + args + ")" + (fn->attrs.empty() ? "" : " attributes" + attr_dict(fn->attrs, {})) + " {\n";
      block(*fn->body, "    ");
      out_ += "  }\n";
    }
    return out_ + "}\n";
  }

 private:
  std::string out_;
  std::map<const Value *, std::string> names_;
  int counter_ = 0;

  std::string nm(const Value *v) { return "%" + names_.at(v); }
  std::string fresh(const Value *v, const std::string &fixed = "") {
    names_[v] = fixed.empty() ? std::to_string(counter_++) : fixed;
    return "%" + names_[v];
  }
  static std::string attr(const Attr &a) {
    switch (a.kind) {
      case Attr::Bool: return a.b ? "unit" : "false";
      case Attr::Int: return std::to_string(a.i);
      case Attr::Float: return float_repr(a.f);
      case Attr::Str: return "\"" + a.s + "\"";
      case Attr::Array: {
        std::string o = "array<i64: ";
        for (size_t k = 0; k < a.arr.size(); ++k) o += (k ? ", " : "") + std::to_string(a.arr[k].i);
        return o + ">";
      }
    }
    return "";
  }
  static std::string list(const Attr &a) {  // the bracketed form of permutation / mask / dimensions
    std::string o = "[";
    for (size_t k = 0; k < a.arr.size(); ++k)   // a mask is an array of booleans, the others of integers
      o += (k ? ", " : "") + (a.arr[k].kind == Attr::Bool ? std::string(a.arr[k].b ? "true" : "false") : std::to_string(a.arr[k].i));
    return o + "]";
  }
  static std::string attr_dict(const AttrDict &d, const std::set<std::string> &skip) {
    std::string items;
    for (const auto &kv : d) {
      if (skip.count(kv.first)) continue;
      if (!items.empty()) items += ", ";
      items += (kv.second.kind == Attr::Bool && kv.second.b) ? kv.first : kv.first + " = " + attr(kv.second);
    }
    return items.empty() ? "" : " {" + items + "}";
  }
  void block(const Block &b, const std::string &ind) {
    for (const auto &o : b.ops) op(*o, ind);
  }
  void op(const Op &o, const std::string &ind) {
    const std::string &n = o.name;
    std::vector<std::string> ops, tys;
    for (const Value *v : o.operands) {
      ops.push_back(nm(v));
      tys.push_back(v->type.str());
    }
    auto join = [](const std::vector<std::string> &v, size_t from = 0) {
      std::string s;
      for (size_t k = from; k < v.size(); ++k) s += (k > from ? ", " : "") + v[k];
      return s;
    };
    if (n == "arith.constant") {
      const Attr &v = *find(o.attrs, "value");
      const std::string text = v.kind == Attr::Bool ? (v.b ? "True" : "False") : attr(v);
      out_ += ind + fresh(o.results[0]) + " = arith.constant " + text + " : " + o.results[0]->type.str() + "\n";
      return;
    }
    if (n == "scf.for") {
      const Block &body = *o.regions[0];
      std::string res;
      for (size_t k = 0; k < o.results.size(); ++k) res += (k ? ", " : "") + fresh(o.results[k]);
      const std::string iv = fresh(body.args[0]);
      std::string iters, rtypes;
      for (size_t k = 1; k < body.args.size(); ++k) {
        iters += (k > 1 ? ", " : "") + fresh(body.args[k]) + " = " + ops[k + 2];
        rtypes += (k > 1 ? ", " : "") + o.results[k - 1]->type.str();
      }
      out_ += ind + (res.empty() ? "" : res + " = ") + "scf.for " + iv + " = " + ops[0] + " to " + ops[1] + " step " + ops[2];
      if (!iters.empty()) out_ += " iter_args(" + iters + ") -> (" + rtypes + ")";
      out_ += " {\n";
      block(body, ind + "  ");
      out_ += ind + "}" + attr_dict(o.attrs, {}) + "\n";
      return;
    }
    if (n == "gpu.launch") {
      const Block &body = *o.regions[0];
      std::vector<std::string> ids, szs;
      for (size_t k = 0; k < 6; ++k) ids.push_back(fresh(body.args[k]));
      for (size_t k = 6; k < body.args.size(); ++k) szs.push_back(fresh(body.args[k]));
      auto sizes = [&](size_t from) {
        std::string s;
        for (size_t k = from; k < from + 3; ++k) s += (k > from ? ", " : "") + szs[k] + " = " + ops[k];
        return s;
      };
      out_ += ind + "gpu.launch blocks(" + ids[0] + ", " + ids[1] + ", " + ids[2] + ") in (" + sizes(0) + ") threads(" +
              ids[3] + ", " + ids[4] + ", " + ids[5] + ") in (" + sizes(3) + ") {\n";
      block(body, ind + "  ");
      out_ += ind + "}\n";
      return;
    }
    std::string res;
    for (size_t k = 0; k < o.results.size(); ++k) res += (k ? ", " : "") + fresh(o.results[k]);
    const std::string lhs = res.empty() ? ind : ind + res + " = ";
    const std::string rty = o.results.size() == 1 ? o.results[0]->type.str() : "";
    if (n == "htile.load" || n == "htile.gather_nd") {
      out_ += lhs + n + " " + ops[0] + "[" + join(ops, 1) + "]" + attr_dict(o.attrs, {}) + " : " + tys[0] + " -> " + rty + "\n";
    } else if (n == "htile.store") {
      out_ += lhs + n + " " + ops[0] + ", " + ops[1] + "[" + join(ops, 2) + "]" + attr_dict(o.attrs, {}) + " : " + tys[0] + ", " + tys[1] + "\n";
    } else if (n == "htile.dot") {
      out_ += lhs + n + " " + join(ops) + attr_dict(o.attrs, {}) + " : " + join(tys) + " -> " + rty + "\n";
    } else if (n == "htile.reduce") {
      out_ += lhs + n + " " + ops[0] + " axis " + std::to_string(find(o.attrs, "axis")->i) + " kind \"" + find(o.attrs, "kind")->s + "\"" +
              attr_dict(o.attrs, {"axis", "kind"}) + " : " + tys[0] + " -> " + rty + "\n";
    } else if (n == "htile.permute" || n == "htile.unsqueeze") {
      const std::string key = n == "htile.permute" ? "permutation" : "mask";
      out_ += lhs + n + " " + ops[0] + " " + key + " " + list(*find(o.attrs, key)) + attr_dict(o.attrs, {key}) + " : " + tys[0] + " -> " + rty + "\n";
    } else if (n == "htile.full" || n == "htile.copy") {
      out_ += lhs + n + " " + ops[0] + attr_dict(o.attrs, {}) + " : " + tys[0] + " -> " + rty + "\n";
    } else if (n == "htile.arange") {
      out_ += lhs + n + " " + ops[0] + " to " + ops[1] + " : " + rty + "\n";
    } else if (n == "tensor.empty") {
      out_ += lhs + "tensor.empty() : " + rty + "\n";
    } else if (n == "linalg.broadcast") {
      out_ += lhs + "linalg.broadcast ins(" + ops[0] + " : " + tys[0] + ") outs(" + ops[1] + " : " + tys[1] + ") dimensions = " +
              list(*find(o.attrs, "dimensions")) + "\n";
    } else if (kCasts.count(n)) {
      out_ += lhs + n + " " + ops[0] + " : " + tys[0] + " to " + rty + "\n";
    } else if (n == "arith.cmpi" || n == "arith.cmpf") {
      out_ += lhs + n + " " + find(o.attrs, "predicate")->s + ", " + ops[0] + ", " + ops[1] + " : " + tys[0] + "\n";
    } else if (n == "scf.yield") {
      out_ += lhs + "scf.yield " + join(ops) + (ops.empty() ? "" : " : " + join(tys)) + "\n";
    } else if (n == "return" || n == "func.return" || n == "gpu.terminator" || n == "htile.hello") {
      out_ += lhs + n + attr_dict(o.attrs, {}) + "\n";
    } else {  // element-wise arith / math / select
      out_ += lhs + n + " " + join(ops) + attr_dict(o.attrs, {}) + " : " + rty + "\n";
    }
  }
};

char *dup_string(const std::string &s) {
  char *p = static_cast<char *>(std::malloc(s.size() + 1));
  if (p) std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}
void put_error(char *err, size_t err_len, const std::string &msg) {
  if (err && err_len) {
    std::strncpy(err, msg.c_str(), err_len - 1);
    err[err_len - 1] = '\0';
  }
}

}  // namespace htf

struct htf_module {
  htf::Module m;
};

extern "C" int htf_version(void) { return 100; }

extern "C" htf_module *htf_parse(const char *text, char *err, size_t err_len) {
  if (err && err_len) err[0] = '\0';
  if (!text) {
    htf::put_error(err, err_len, "null text");
    return nullptr;
  }
  auto mod = std::make_unique<htf_module>();
  try {
    htf::Parser(text, mod->m).module();
  } catch (const std::exception &e) {
    htf::put_error(err, err_len, e.what());
    return nullptr;
  }
  return mod.release();
}

extern "C" void htf_free(htf_module *m) { delete m; }

extern "C" int htf_verify(const htf_module *m, char *err, size_t err_len) {
  if (err && err_len) err[0] = '\0';
  if (!m) {
    htf::put_error(err, err_len, "null module");
    return -1;
  }
  try {
    htf::walk(const_cast<htf::Module &>(m->m), [](htf::Op &o) { htf::verify_op(o); });
  } catch (const std::exception &e) {
    htf::put_error(err, err_len, e.what());
    return -1;
  }
  return 0;
}

extern "C" int htf_run_pipeline(htf_module *m, const char *pipeline, char *err, size_t err_len) {
  if (err && err_len) err[0] = '\0';
  if (!m || !pipeline) {
    htf::put_error(err, err_len, "null argument");
    return -1;
  }
  try {
    htf::run_pipeline(m->m, pipeline);
  } catch (const std::exception &e) {
    htf::put_error(err, err_len, e.what());
    return -1;
  }
  return 0;
}

extern "C" char *htf_to_json(const htf_module *m) { return m ? htf::dup_string(htf::to_json(m->m)) : nullptr; }

extern "C" char *htf_print(const htf_module *m) {
  if (!m) return nullptr;
  try {
    return htf::dup_string(htf::Printer().run(m->m));
  } catch (const std::exception &) {
    return nullptr;
  }
}

extern "C" void htf_string_free(char *s) { std::free(s); }

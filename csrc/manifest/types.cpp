// Typed parse of manifest v7 (see types.hpp). One reader object per JSON object keeps track of the
// keys it consumed so that an unknown field is reported with its path.
#include "types.hpp"

#include <algorithm>
#include <array>

namespace kern {

// ---- enums <-> names -----------------------------------------------------------------------------
static const std::pair<const char*, DType> kDTypes[] = {
    {"bf16", DType::bf16}, {"f16", DType::f16}, {"f32", DType::f32}, {"fp8e4m3", DType::fp8e4m3},
    {"fp8e8m0", DType::fp8e8m0}, {"i8", DType::i8}, {"i32", DType::i32}, {"u32", DType::u32},
    {"i64", DType::i64}, {"u64", DType::u64}, {"u8", DType::u8}};
const char* dtype_name(DType d) {
  for (auto& p : kDTypes) if (p.second == d) return p.first;
  return "?";
}
bool dtype_parse(const std::string& s, DType& out) {
  for (auto& p : kDTypes) if (s == p.first) { out = p.second; return true; }
  return false;
}
uint64_t dtype_bytes(DType d) {
  switch (d) {
    case DType::bf16: case DType::f16: return 2;
    case DType::f32: case DType::i32: case DType::u32: return 4;
    case DType::i64: case DType::u64: return 8;
    default: return 1;
  }
}
bool dtype_is_int(DType d) {
  return d == DType::i8 || d == DType::i32 || d == DType::u32 || d == DType::i64 || d == DType::u64 || d == DType::u8;
}
bool dtype_is_float(DType d) { return !dtype_is_int(d); }

static const std::pair<const char*, Fill> kFills[] = {
    {"token", Fill::Token}, {"position", Fill::Position}, {"valid", Fill::Valid}, {"slot", Fill::Slot},
    {"seq_len", Fill::SeqLen}, {"cu_seqlens", Fill::CuSeqlens}, {"blocks", Fill::Blocks},
    {"temperature", Fill::Temperature}, {"top_k", Fill::TopK}, {"top_p", Fill::TopP}, {"min_p", Fill::MinP},
    {"seed", Fill::Seed}, {"tokens", Fill::Tokens}, {"count", Fill::Count}, {"error", Fill::Error}};
const char* fill_name(Fill f) {
  for (auto& p : kFills) if (p.second == f) return p.first;
  return "?";
}
bool fill_parse(const std::string& s, Fill& out) {
  for (auto& p : kFills) if (s == p.first) { out = p.second; return true; }
  return false;
}
std::vector<DType> fill_dtypes(Fill f) {
  switch (f) {
    case Fill::Temperature: case Fill::TopP: case Fill::MinP: return {DType::f32};
    case Fill::TopK: return {DType::i32};
    case Fill::Seed: return {DType::i64};
    default: return {DType::i32, DType::i64};
  }
}
const char* axis_name(VarAxis a) {
  switch (a) { case VarAxis::Rows: return "rows"; case VarAxis::Groups: return "groups";
               case VarAxis::Ranks: return "ranks"; default: return "none"; }
}
const char* kind_name(BufferKind k) {
  static const char* n[] = {"input", "output", "inout", "weight", "source", "workspace", "carry", "peer"};
  return n[(int)k];
}

// ---- Expr ----------------------------------------------------------------------------------------
std::optional<uint64_t> Expr::eval(const VarMap& vars, std::string* why) const {
  auto fail = [&](const std::string& w) -> std::optional<uint64_t> { if (why) *why = w; return std::nullopt; };
  switch (kind) {
    case Const: return c;
    case Var: {
      auto it = vars.find(var);
      if (it == vars.end()) return fail("unknown var `" + var + "`");
      return it->second;
    }
    case CeilDiv: {
      if (c == 0) return fail("division by zero");
      auto x = sub[0].eval(vars, why);
      if (!x) return x;
      if (*x > UINT64_MAX - (c - 1)) return fail("arithmetic overflow");
      return (*x + (c - 1)) / c;
    }
    case Mul: {
      auto x = sub[0].eval(vars, why);
      if (!x) return x;
      if (c != 0 && *x > UINT64_MAX / c) return fail("arithmetic overflow");
      return *x * c;
    }
    case Add: {
      auto a = sub[0].eval(vars, why);
      if (!a) return a;
      auto b = sub[1].eval(vars, why);
      if (!b) return b;
      if (*a > UINT64_MAX - *b) return fail("arithmetic overflow");
      return *a + *b;
    }
    case Clamp: {
      auto x = sub[0].eval(vars, why);
      if (!x) return x;
      uint64_t v = *x > c ? *x - c : 0;
      return std::min(v, c2);
    }
  }
  return std::nullopt;
}
void Expr::collect_vars(std::vector<std::string>& out) const {
  if (kind == Var) out.push_back(var);
  for (auto& s : sub) s.collect_vars(out);
}
Json Expr::to_json() const {
  Json j = Json::object(), a = Json::array();
  switch (kind) {
    case Const: return Json::uint(c);
    case Var: return Json::str(var);
    case CeilDiv: a.push(sub[0].to_json()); a.push(Json::uint(c)); j.set("ceil_div", a); return j;
    case Mul: a.push(sub[0].to_json()); a.push(Json::uint(c)); j.set("mul", a); return j;
    case Add: a.push(sub[0].to_json()); a.push(sub[1].to_json()); j.set("add", a); return j;
    case Clamp: a.push(sub[0].to_json()); a.push(Json::uint(c)); a.push(Json::uint(c2)); j.set("clamp", a); return j;
  }
  return j;
}

std::optional<double> Bound::eval(const VarMap& vars) const {
  switch (kind) {
    case Int: return (double)i;
    case Float: return f;
    case Ex: { auto v = expr.eval(vars); if (!v) return std::nullopt; return (double)*v; }
  }
  return std::nullopt;
}

// ---- HostTensor ----------------------------------------------------------------------------------
std::optional<uint64_t> HostTensor::span(uint64_t outer) const {
  if (shape.size() != strides.size()) return std::nullopt;
  unsigned __int128 acc = 0;
  for (size_t i = 0; i < shape.size(); ++i) {
    uint64_t n = (i == 0 && shape[i] == 0) ? outer : shape[i];
    if (n == 0) return std::nullopt;
    acc += (unsigned __int128)(n - 1) * strides[i];
    if (acc > UINT64_MAX) return std::nullopt;
  }
  acc = (acc + 1) * dtype_bytes(dtype);
  if (acc > UINT64_MAX) return std::nullopt;
  return (uint64_t)acc;
}
std::string HostTensor::describe() const {
  auto v = [](const std::vector<uint64_t>& a) {
    std::string s = "[";
    for (size_t i = 0; i < a.size(); ++i) s += (i ? ", " : "") + std::to_string(a[i]);
    return s + "]";
  };
  return std::string(dtype_name(dtype)) + " shape " + v(shape) + " strides " + v(strides);
}
std::optional<uint64_t> HostTensor::admit(DType dt, const std::vector<uint64_t>& shp,
                                          const std::vector<uint64_t>& str, std::string& err) const {
  auto want = [&](const std::string& got) { err = "host tensor " + got + " is not the declared " + describe(); };
  if (dt != dtype) { want(std::string("of ") + dtype_name(dt)); return std::nullopt; }
  if (shp.size() != shape.size() || str.size() != strides.size()) {
    want("of rank " + std::to_string(shp.size()) + "/" + std::to_string(str.size()));
    return std::nullopt;
  }
  bool fits = str == strides;
  for (size_t i = 0; i < shp.size() && fits; ++i)
    fits = (i == 0 && shape[i] == 0) ? shp[i] >= 1 : shp[i] == shape[i];
  if (!fits) { HostTensor got{dt, shp, str}; want(got.describe()); return std::nullopt; }
  auto s = span(shp.empty() ? 1 : shp[0]);
  if (!s) want("whose span overflows 64 bits");
  return s;
}

// ---- Buffer sizes ----------------------------------------------------------------------------------
std::optional<uint64_t> Buffer::elems(const VarMap& vars) const {
  unsigned __int128 n = 1;
  for (auto& d : shape) {
    uint64_t v = d.c;
    if (d.is_var) { auto it = vars.find(d.var); if (it == vars.end()) return std::nullopt; v = it->second; }
    n *= v;
    if (n > UINT64_MAX) return std::nullopt;
  }
  return (uint64_t)n;
}
std::optional<uint64_t> Buffer::bytes(const VarMap& vars) const {
  auto n = elems(vars);
  if (!n) return n;
  unsigned __int128 b = (unsigned __int128)*n * dtype_bytes(dtype);
  if (b > UINT64_MAX) return std::nullopt;
  return (uint64_t)b;
}

// ---- ParamType -------------------------------------------------------------------------------------
bool ParamType::parse(const std::string& s, ParamType& out) {
  out = ParamType();
  if (s == "i32" || s == "i64" || s == "f32" || s == "u8") {
    out.kind = Scalar;
    dtype_parse(s, out.dtype);
    return true;
  }
  if (s.rfind("bytes<", 0) == 0 && s.back() == '>') {
    std::string n = s.substr(6, s.size() - 7);
    if (n.empty() || n.size() > 9 || !std::all_of(n.begin(), n.end(), ::isdigit)) return false;
    out.kind = Bytes;
    out.nbytes = (uint32_t)std::stoul(n);
    return out.nbytes > 0;
  }
  size_t sp = s.find(' ');
  if (sp == std::string::npos) return false;
  std::string dir = s.substr(0, sp), rest = s.substr(sp + 1);
  if (dir == "in") out.dir = In; else if (dir == "out") out.dir = Out; else if (dir == "inout") out.dir = Inout;
  else return false;
  if (rest == "state") { out.kind = State; return true; }
  if (rest.rfind("buffer<", 0) == 0 && rest.back() == '>') {
    out.kind = Buffer;
    return dtype_parse(rest.substr(7, rest.size() - 8), out.dtype);
  }
  return false;
}
std::string ParamType::str() const {
  static const char* dirs[] = {"in", "out", "inout"};
  switch (kind) {
    case Scalar: return dtype_name(dtype);
    case Bytes: return "bytes<" + std::to_string(nbytes) + ">";
    case Buffer: return std::string(dirs[dir]) + " buffer<" + dtype_name(dtype) + ">";
    case State: return std::string(dirs[dir]) + " state";
  }
  return "?";
}
uint32_t ParamType::abi_size() const {
  switch (kind) {
    case Scalar: return (uint32_t)dtype_bytes(dtype);
    case Bytes: return nbytes;
    default: return 8;
  }
}

std::vector<LaunchArg> Op::args_of(const Launch& l) const {
  if (l.args) return *l.args;
  std::vector<LaunchArg> out(params.size());
  for (size_t i = 0; i < params.size(); ++i) { out[i].kind = LaunchArg::Param; out[i].param = i; }
  return out;
}
std::string LaunchArg::str() const {
  switch (kind) {
    case Param: return "interface param #" + std::to_string(param);
    case Scratch: return "scratch `" + name + "`";
    case I32: return "i32 literal " + std::to_string(i);
    case I64: return "i64 literal " + std::to_string(i);
    case F32: return "f32 literal " + std::to_string(f);
    case U8: return "u8 literal " + std::to_string(i);
    case Rank: return "rank in group `" + name + "`";
    case PackK: return "pack of " + std::to_string(pack.size) + " bytes";
  }
  return "?";
}
std::string Arg::str() const {
  switch (kind) {
    case Buf: return "buffer `" + name + "`" + (offset ? "+" + std::to_string(offset) : "");
    case StateK: return "state `" + name + "`" + (offset ? "+" + std::to_string(offset) : "");
    case Var: return "var `" + name + "`";
    case ExprK: return "expression";
    case I32: return "i32 literal " + std::to_string(i);
    case I64: return "i64 literal " + std::to_string(i);
    case F32: return "f32 literal " + std::to_string(f);
    case U8: return "u8 literal " + std::to_string(i);
    case Rank: return "rank in group `" + name + "`";
  }
  return "?";
}

// ---- TensorMap / Pack checks -----------------------------------------------------------------------
uint64_t TensorMapDecl::bits() const {
  if (dtype == "u4" || dtype == "u4packed") return 4;
  if (dtype == "u8") return 8;
  if (dtype == "u16" || dtype == "f16" || dtype == "bf16") return 16;
  if (dtype == "u64" || dtype == "i64") return 64;
  return 32;
}
int TensorMapDecl::cu_dtype() const {
  static const std::pair<const char*, int> t[] = {{"u8", 0}, {"u16", 1}, {"u32", 2}, {"i32", 3}, {"u64", 4},
      {"i64", 5}, {"f16", 6}, {"f32", 7}, {"bf16", 9}, {"tf32", 11}, {"u4", 14}, {"u4packed", 13}};   // u4: 16U4_ALIGN16B (16 nibbles per 16-byte chunk in shared memory), u4packed: 16U4_ALIGN8B
  for (auto& p : t) if (dtype == p.first) return p.second;
  return -1;
}
Errors TensorMapDecl::check() const {
  Errors e;
  const size_t n = dims.size();
  if (cu_dtype() < 0) e.push_back("unknown tensormap dtype `" + dtype + "`");
  if (n < 1 || n > 5) { e.push_back("dims has " + std::to_string(n) + " entries, expected 1 to 5"); return e; }
  if (strides.size() != n - 1)
    e.push_back("strides has " + std::to_string(strides.size()) + " entries, expected dims - 1 = " + std::to_string(n - 1));
  if (box.size() != n) e.push_back("box has " + std::to_string(box.size()) + " entries, expected " + std::to_string(n));
  for (size_t i = 0; i + 1 < n; ++i)
    if (dims[i] == 0) { e.push_back("dims[" + std::to_string(i) + "] is 0; only the outermost dim may span the buffer"); break; }
  if (n == 1 && dims[0] == 0) e.push_back("dims[0] is 0");
  for (size_t i = 0; i < box.size(); ++i)
    if (box[i] < 1 || box[i] > 256) { e.push_back("box[" + std::to_string(i) + "] = " + std::to_string(box[i]) + ", must be 1..=256"); break; }
  for (size_t i = 0; i < strides.size(); ++i)
    if (strides[i] == 0 || strides[i] % 16) {
      e.push_back("strides[" + std::to_string(i) + "] = " + std::to_string(strides[i]) + " is not a positive multiple of 16");
      break;
    }
  if (dtype == "u4") {       // the unpacking type: whole 128-nibble boxes, 32-byte strides
    if (!box.empty() && box[0] != 128) e.push_back("box[0] of a `u4` map must be 128 nibbles");
    if (dims[0] % 128) e.push_back("dims[0] of a `u4` map must be a multiple of 128 nibbles");
    for (size_t i = 0; i < strides.size(); ++i)
      if (strides[i] % 32) { e.push_back("strides of a `u4` map must be multiples of 32 bytes"); break; }
  }
  const uint64_t b = bits();
  if ((dims[0] * b) % 128) e.push_back("dims[0] = " + std::to_string(dims[0]) + " elements is not a multiple of 16 bytes");
  if (!box.empty()) {
    uint64_t inner = (uint64_t)box[0] * b / 8;
    if (inner % 16) e.push_back("box[0] = " + std::to_string(box[0]) + " elements spans " + std::to_string(inner) + " bytes, not a multiple of 16");
    if (swizzle != 0 && inner > swizzle)
      e.push_back("box[0] spans " + std::to_string(inner) + " bytes, more than the " + std::to_string(swizzle) + " byte swizzle span");
  }
  if (swizzle != 0 && swizzle != 32 && swizzle != 64 && swizzle != 128)
    e.push_back("swizzle " + std::to_string(swizzle) + " is not one of 0, 32, 64, 128");
  if (l2_promotion != 0 && l2_promotion != 64 && l2_promotion != 128 && l2_promotion != 256)
    e.push_back("l2_promotion " + std::to_string(l2_promotion) + " is not one of 0, 64, 128, 256");
  return e;
}
std::optional<uint64_t> TensorMapDecl::footprint() const {
  if (dims.empty() || strides.size() + 1 != dims.size()) return std::nullopt;
  size_t n = dims.size() > 1 && dims.back() == 0 ? dims.size() - 1 : dims.size();
  unsigned __int128 bytes = ((unsigned __int128)dims[0] * bits() + 7) / 8;
  for (size_t i = 1; i < n; ++i) {
    if (dims[i] == 0) return std::nullopt;
    bytes += (unsigned __int128)(dims[i] - 1) * strides[i - 1];
    if (bytes > UINT64_MAX) return std::nullopt;
  }
  return (uint64_t)bytes;
}
std::optional<uint32_t> Field::natural_width() const {
  if (width) return width;
  switch (src.kind) {
    case FieldSrc::Param: return std::nullopt;
    case FieldSrc::Scratch: case FieldSrc::I64: return 8;
    case FieldSrc::I32: case FieldSrc::F32: case FieldSrc::Var: case FieldSrc::ExprK: case FieldSrc::Rank: return 4;
    case FieldSrc::U8: return 1;
    case FieldSrc::TensorMap: return 128;
  }
  return std::nullopt;
}
Errors Pack::check(const std::vector<ParamType>& iface) const {
  Errors e;
  std::vector<std::array<uint32_t, 3>> spans;
  for (size_t i = 0; i < fields.size(); ++i) {
    const Field& f = fields[i];
    std::optional<uint32_t> w = f.natural_width();
    if (!w && f.src.kind == FieldSrc::Param && f.src.param < iface.size()) {
      const ParamType& p = iface[f.src.param];
      if (p.kind != ParamType::Bytes) w = p.abi_size();
    }
    if (!w || *w == 0) { e.push_back("field #" + std::to_string(i) + ": width unknown"); continue; }
    if (f.src.kind == FieldSrc::TensorMap) {
      if (*w != 128) e.push_back("field #" + std::to_string(i) + ": a tensormap field is 128 bytes, not " + std::to_string(*w));
      if (f.at % 64) e.push_back("field #" + std::to_string(i) + ": tensormap at " + std::to_string(f.at) + " is not 64-byte aligned");
    }
    uint64_t end = (uint64_t)f.at + *w;
    if (end <= size) spans.push_back({f.at, (uint32_t)end, (uint32_t)i});
    else e.push_back("field #" + std::to_string(i) + " at " + std::to_string(f.at) + " spans " + std::to_string(*w) +
                     " bytes, past the " + std::to_string(size) + " byte image");
  }
  std::sort(spans.begin(), spans.end());
  for (size_t i = 1; i < spans.size(); ++i)
    if (spans[i][0] < spans[i - 1][1])
      e.push_back("field #" + std::to_string(spans[i][2]) + " overlaps field #" + std::to_string(spans[i - 1][2]));
  return e;
}

VarMap Manifest::vars_at_max() const {
  VarMap v;
  for (auto& kv : vars) v[kv.first] = kv.second.max;
  return v;
}
VarMap Manifest::vars_at_min() const {
  VarMap v;
  for (auto& kv : vars) v[kv.first] = VAR_MIN;
  return v;
}

int registry_ref_parse(const std::string& s, std::string& url, std::string& err) {
  if (s.rfind("https://", 0) == 0) {
    std::string rest = s.substr(8);
    size_t slash = rest.find('/');
    bool ok = slash != std::string::npos && slash > 0 && slash + 1 < rest.size() &&
              std::none_of(rest.begin(), rest.end(), [](unsigned char c) { return std::isspace(c); });
    if (ok) { url = s; return 1; }
    err = "invalid registry ref `" + s + "`: expected https://<host>/<path>";
    return -1;
  }
  if (s.find("://") != std::string::npos) {
    err = "invalid registry ref `" + s + "`: only https:// and hf: sources are fetched";
    return -1;
  }
  if (s.rfind("hf:", 0) != 0) return 0;
  auto bad = [&] { err = "invalid registry ref `" + s + "`: expected hf:<org>/<repo>/<path>[@revision]"; return -1; };
  std::string rest = s.substr(3), rev = "main";
  size_t at = rest.rfind('@');
  if (at != std::string::npos) {
    rev = rest.substr(at + 1);
    if (rev.empty() || rev.find('/') != std::string::npos) return bad();
    rest = rest.substr(0, at);
  }
  size_t a = rest.find('/');
  if (a == std::string::npos) return bad();
  size_t b = rest.find('/', a + 1);
  if (b == std::string::npos) return bad();
  std::string org = rest.substr(0, a), repo = rest.substr(a + 1, b - a - 1), path = rest.substr(b + 1);
  if (org.empty() || repo.empty() || path.empty()) return bad();
  size_t pos = 0;
  while (pos <= path.size()) {
    size_t nx = path.find('/', pos);
    std::string seg = path.substr(pos, nx == std::string::npos ? std::string::npos : nx - pos);
    if (seg.empty() || seg == "." || seg == "..") return bad();
    if (nx == std::string::npos) break;
    pos = nx + 1;
  }
  url = "https://huggingface.co/" + org + "/" + repo + "/resolve/" + rev + "/" + path;
  return 1;
}

}  // namespace kern

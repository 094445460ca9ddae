// Wire types of manifest schema v7 and their typed parse from JSON: unknown fields and duplicate
// names are errors, `constants` are substituted for string leaves before typing, every parse error
// is collected (the caller sees all of them at once).
// Reference: crates/kern-manifest/src/types.rs:31-1653 (the schema), constants.rs:93-136 (expansion).
#pragma once
#include <array>
#include <cstring>
#include <map>
#include <optional>
#include <set>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "json.hpp"

namespace kern {

constexpr uint64_t SCHEMA_VERSION = 7;
constexpr uint64_t VAR_MIN = 1;

using Errors = std::vector<std::string>;
using VarMap = std::map<std::string, uint64_t>;

// ---- element types -------------------------------------------------------------------------------
enum class DType { bf16, f16, f32, fp8e4m3, fp8e8m0, i8, i32, u32, i64, u64, u8 };
const char* dtype_name(DType d);
bool dtype_parse(const std::string& s, DType& out);
uint64_t dtype_bytes(DType d);
bool dtype_is_int(DType d);
bool dtype_is_float(DType d);

// ---- expressions ---------------------------------------------------------------------------------
struct Expr {
  enum Kind { Const, Var, CeilDiv, Mul, Add, Clamp } kind = Const;
  uint64_t c = 0, c2 = 0;          // Const value; CeilDiv/Mul constant; Clamp start (c) and len (c2)
  std::string var;
  std::vector<Expr> sub;           // 1 child (CeilDiv, Mul, Clamp) or 2 (Add)
  // nullopt on unknown var / overflow / division by zero (why says which)
  std::optional<uint64_t> eval(const VarMap& vars, std::string* why = nullptr) const;
  void collect_vars(std::vector<std::string>& out) const;
  Json to_json() const;
};

struct Dim {
  bool is_var = false;
  uint64_t c = 0;
  std::string var;
  Json to_json() const { return is_var ? Json::str(var) : Json::uint(c); }
};

// ---- fills -----------------------------------------------------------------------------------------
enum class Fill { Token, Position, Valid, Slot, SeqLen, CuSeqlens, Blocks, Temperature, TopK, TopP, MinP,
                  Seed, Tokens, Count, Error };
const char* fill_name(Fill f);
bool fill_parse(const std::string& s, Fill& out);
inline bool fill_is_output(Fill f) { return f == Fill::Tokens || f == Fill::Count || f == Fill::Error; }
std::vector<DType> fill_dtypes(Fill f);

enum class VarAxis { None, Rows, Groups, Ranks };
const char* axis_name(VarAxis a);

struct Var {
  uint64_t max = 0;
  VarAxis axis = VarAxis::None;
};

struct HostTensor {
  DType dtype = DType::u8;
  std::vector<uint64_t> shape, strides;
  std::optional<uint64_t> span(uint64_t outer) const;   // bytes from first to last element
  // check a tensor a host engine offers against this declaration; returns bytes or sets err
  std::optional<uint64_t> admit(DType dt, const std::vector<uint64_t>& shp, const std::vector<uint64_t>& str,
                                std::string& err) const;
  std::string describe() const;
};

struct Shard {
  enum By { Position, Heads } by = Position;
  std::string group;
  std::vector<std::pair<uint64_t, uint64_t>> segments;  // heads: [rows, width]
};

struct State {
  uint64_t bytes_per_token = 0, bytes = 0, bytes_per_seq = 0;
  std::optional<HostTensor> host;
  std::optional<Shard> shard;
  bool is_per_seq() const { return bytes_per_seq > 0; }
  bool is_paged() const { return bytes_per_token > 0; }
  bool is_owned() const { return !host.has_value(); }
};

enum class BufferKind { Input, Output, Inout, Weight, Source, Workspace, Carry, Peer };
const char* kind_name(BufferKind k);

struct TensorSource {
  bool ranked = false;
  std::string name;                   // named
  std::string group;                  // ranked
  std::vector<std::string> tensors;   // ranked
};
struct Ranges {
  bool ranked = false;
  uint64_t range[2] = {0, 0};
  std::string group;
  std::vector<std::pair<uint64_t, uint64_t>> ranges;
};
struct Interleave {
  TensorSource with;
  uint64_t rows = 0;
};
struct Segment {
  TensorSource tensor;
  std::optional<Ranges> rows, cols;
  std::optional<Interleave> interleave;
};

struct Bound {
  enum Kind { Int, Float, Ex } kind = Int;
  int64_t i = 0;
  double f = 0;
  Expr expr;
  std::optional<double> eval(const VarMap& vars) const;
};
struct Domain {
  std::optional<Bound> min, max;
  std::optional<std::string> index_into;
  uint64_t stride = 1;
  bool monotone = false;
};

struct Buffer {
  DType dtype = DType::u8;
  std::vector<Dim> shape;
  BufferKind kind = BufferKind::Workspace;
  bool host_placement = false;
  std::optional<Fill> fill;
  std::optional<Domain> domain;
  bool export_ = false;
  std::optional<std::string> of, group;
  std::vector<Segment> bind;
  // bytes at the given var assignment; nullopt on overflow / unknown var
  std::optional<uint64_t> bytes(const VarMap& vars) const;
  std::optional<uint64_t> elems(const VarMap& vars) const;
};

// ---- ops -------------------------------------------------------------------------------------------
struct ParamType {
  enum Kind { Scalar, Bytes, Buffer, State } kind = Scalar;
  enum Dir { In, Out, Inout } dir = In;       // Buffer / State
  DType dtype = DType::i32;                   // Scalar (i32,i64,f32,u8) or Buffer element type
  uint32_t nbytes = 0;                        // Bytes<n>
  bool is_pointer() const { return kind == Buffer || kind == State; }
  bool writes() const { return is_pointer() && dir != In; }
  bool reads() const { return is_pointer() && dir != Out; }
  uint32_t abi_size() const;                  // bytes the kernel ABI gives this parameter
  std::string str() const;
  static bool parse(const std::string& s, ParamType& out);
};

struct Module {
  std::string source, sha256;
  bool multicast_free = false;   // declared `multicast: false`: built from sources that pass the lint
};

struct Scratch {
  DType dtype = DType::u8;
  std::vector<Dim> shape;
};

struct When {
  std::string var;
  std::optional<uint64_t> min, max;
  bool holds(uint64_t v) const { return (!min || v >= *min) && (!max || v <= *max); }
};

struct TensorMapDecl {
  size_t param = 0;
  std::string dtype;                 // u8|u16|u32|i32|u64|i64|f16|bf16|f32|tf32|u4|u4packed
  std::vector<uint64_t> dims, strides;
  std::vector<uint32_t> box;
  uint32_t swizzle = 0, l2_promotion = 0;
  bool oob_nan = false, wrap = false;
  uint64_t bits() const;
  int cu_dtype() const;              // CUtensorMapDataType code
  Errors check() const;
  std::optional<uint64_t> footprint() const;
};

struct FieldSrc {
  enum Kind { Param, Scratch, I32, I64, F32, U8, Var, ExprK, Rank, TensorMap } kind = I32;
  size_t param = 0;
  std::string name;     // scratch / var / rank group
  int64_t i = 0;
  double f = 0;
  Expr expr;
  TensorMapDecl tmap;
};
struct Field {
  uint32_t at = 0;
  std::optional<uint32_t> width;
  FieldSrc src;
  std::optional<uint32_t> natural_width() const;
};
struct Pack {
  uint32_t size = 0;
  std::vector<Field> fields;
  Errors check(const std::vector<ParamType>& iface) const;
};

struct LaunchArg {
  enum Kind { Param, Scratch, I32, I64, F32, U8, Rank, PackK } kind = Param;
  size_t param = 0;
  std::string name;     // scratch name / rank group
  int64_t i = 0;
  double f = 0;
  Pack pack;
  std::string str() const;
};

struct GemmAlgo {
  int64_t id = 0, split_k = 0;
  uint64_t tile = 0, stages = 0, reduction = 0, swizzle = 0, custom = 0, inner_shape = 0, cluster_shape = 0;
};

struct Launch {
  bool is_extern = false;
  std::string module, entry;
  std::optional<std::vector<ParamType>> params;
  uint32_t block[3] = {1, 1, 1};
  Expr grid[3];
  std::optional<Expr> shared_mem;
  std::optional<std::array<uint32_t, 3>> cluster;
  bool pdl = false;
  std::optional<When> when;
  std::optional<GemmAlgo> algo;
  std::optional<std::vector<LaunchArg>> args;
};

struct Op {
  std::vector<ParamType> params;
  std::map<std::string, Scratch> scratch;
  std::vector<Launch> launches;
  const std::vector<ParamType>& params_of(const Launch& l) const { return l.params ? *l.params : params; }
  std::vector<LaunchArg> args_of(const Launch& l) const;
};

// ---- programs --------------------------------------------------------------------------------------
struct Arg {
  enum Kind { Buf, StateK, Var, ExprK, I32, I64, F32, U8, Rank } kind = Buf;
  std::string name;       // buf / state / var / group
  uint64_t offset = 0;
  Expr expr;
  int64_t i = 0;
  double f = 0;
  std::string str() const;
};
struct Call {
  std::optional<std::string> label;
  std::string op;
  std::vector<Arg> args;
  uint8_t lane = 0;
  std::vector<uint8_t> after;
};
struct Batch {
  uint64_t groups = 0;
  Dim rows;
  std::optional<std::string> context;
};
struct Program {
  std::optional<Batch> batch;
  bool once = false, derive = false, graph = false;
  std::vector<Call> calls;
};

struct Cut {
  std::string id;
  uint64_t stage = 0, stages = 0;
};

struct Manifest {
  uint64_t schema_version = 0;
  std::string model;
  std::optional<std::string> tool_parser;
  bool has_chat = false;
  std::map<std::string, Json> constants;
  std::map<std::string, Var> vars;
  std::map<std::string, uint64_t> topology;   // group -> size
  bool has_topology = false;
  std::optional<Cut> cut;
  std::map<std::string, State> states;
  std::map<std::string, Buffer> buffers;
  std::map<std::string, Module> modules;
  std::map<std::string, Op> ops;
  std::map<std::string, Program> programs;
  // declaration order of programs as written (the order `kern verify` prints them in)
  std::vector<std::string> program_order;

  VarMap vars_at_max() const;
  VarMap vars_at_min() const;
  // per-sequence slots a state table of `width` columns addresses, etc. are derived by the pool
};

// Parse + type a manifest document. Every problem found is appended to `errs`; the returned
// manifest is usable for verification only when `errs` stayed empty.
Manifest parse_manifest(const Json& doc, Errors& errs);
Manifest parse_manifest_text(const std::string& text, Errors& errs);
// Serialise back to the wire format (constants already expanded).
Json manifest_to_json(const Manifest& m);

// `hf:org/repo/path[@rev]` or `https://…` module sources; returns 0 = not a registry ref,
// 1 = ok (url set), -1 = malformed (err set)
int registry_ref_parse(const std::string& s, std::string& url, std::string& err);

}  // namespace kern

// Whole-plan executor: the stream executor and arena allocator behind hal::Executable::run.
//
// Input is the step list ops::build_executable_plan derives from the nine-pass pipeline's output
// (include/frame/ops/executable_plan.h:42-71): per step the op name, attribute values, input and
// output slot numbers, output types, and for every intermediate the byte offset the memory
// planner assigned inside one arena (src/ir/memory_plan.cpp:37-133).  The reference executes it
// in CudaExecutable::run (src/backends/cuda/cuda_executable.cpp:41-128) by allocating the arena
// with cudaMalloc inside every run, allocating every graph output separately and copying it
// into the caller's tensor afterwards, and re-decoding attributes in every kernel call.
//
// Here, once per plan: the arena is allocated (one cudaMalloc, 256-byte aligned, the planner's
// offsets are used as they are); attributes are decoded into POD launch records; constants are
// materialised; matmul/conv2d steps absorb the elementwise group that follows them as their
// epilogue when that is provably safe under the planner's buffer reuse; reshape becomes an
// alias when no later step can overwrite the aliased bytes.  Per run: one loop of launches on
// the caller's stream, graph outputs written straight into the caller's buffers, no allocation,
// no synchronisation.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "common.cuh"

namespace fb200 {

enum class Kind {
  kMatmul, kConv2d, kConv1d, kMaxPool, kChain, kBiasAdd, kSoftmax, kLayerNorm, kScan, kMambaScan,
  kTranspose, kSlice, kConcat, kSum, kCopy, kAlias, kConstant, kSkip, kAttentionFan, kDwConvTimeMajor, kAvgPool, kGather, kScatterAdd,
  kPoolSelect, kMaxPoolGrad, kAvgPoolGrad, kConvGradInput, kConvGradFilter, kRfft, kIrfft,
  kMatmulGradLhs, kMatmulGradRhs, kMseLoss, kMseLossGrad
};

struct SlotInfo {
  int dtype = 0;
  std::vector<int64_t> dims;
  int64_t numel = 1;
  int64_t arena_offset = -1;  // >= 0: lives in the arena
  int input_index = -1;       // >= 0: graph input
  int output_index = -1;      // >= 0: graph output (first occurrence)
  int alias_of = -1;          // >= 0: same bytes as that slot
  void* constant = nullptr;   // materialised constant
  int private_index = -1;     // >= 0: lives in buffer `private_index` of the run's workspace, outside the planner's arena
  bool is_constant = false;   // produced by a `constant` step
  bool splat = false;         // constant whose elements are all equal ...
  float splat_value = 0.0f;   // ... to this value (as stored in the slot's dtype)
  size_t bytes() const { return static_cast<size_t>(numel) * itemsize_of(dtype); }
};

struct Attr {
  std::string name, kind, text;
};

struct Step {
  std::string op;
  Kind kind = Kind::kSkip;
  std::vector<int> in, out;
  std::vector<Attr> attrs;
  // decoded
  std::vector<int> chain_ops, chain_arity;   // kChain, or the absorbed epilogue of a contraction
  std::vector<int> epi_operand_slot;         // per epilogue step: slot of the operand or -1
  std::vector<int> epi_mode;
  int write_slot = -1;                       // where the (possibly fused) result goes
  int split_slot = -1;                       // kMatmul: slot that receives the columns from split_col on
  int64_t split_col = 0;
  int ln_res = -1, ln_sum = -1;              // kLayerNorm of (in[0] + ln_res): the sum is also stored to ln_sum
  int pool_mid = -1;                         // kConv2d followed by a max_pool2d: the conv's own result slot
  std::vector<int64_t> pool_iv;              //   and the pool's kernel, stride, padding (write_slot = pool result)
  std::vector<int64_t> iv;                   // op-specific integers
  double eps = 0.0;
  // kAttentionFan: the matrices the heads' q/k/v windows lie in, where the results go, and the
  // device table of per-head coordinates
  int fan_q = -1, fan_k = -1, fan_v = -1, fan_dest = -1;
  int64_t fan_heads = 0, fan_sq = 0, fan_sk = 0;
  float fan_scale = 1.0f;   // scores are multiplied by this (and rounded again) before the softmax
  void* fan_table = nullptr;
  // kDwConvTimeMajor: input matrix slot and column window, weights, bias, geometry
  int dw_x = -1, dw_w = -1, dw_bias = -1;
  int64_t dw_col = 0, dw_ld = 0, dw_batch = 0, dw_len = 0, dw_out_len = 0, dw_channels = 0, dw_k = 0, dw_shift = 0;
};

}  // namespace fb200

using namespace fb200;

struct fb200_plan {
  bool dry = false;   // parsed and rewritten for description only: owns no device memory, cannot run
  int device = 0;
  int allow_tf32 = 0;
  int opt_level = 1;
  std::vector<SlotInfo> slots;
  std::vector<Step> steps;
  std::vector<int> input_slots, output_slots;
  size_t arena_bytes = 0;
  std::vector<void*> owned;           // constants, device tables
  // Everything a run writes lives in a workspace: the arena at the planner's offsets plus the plan's
  // private buffers.  Each stream that runs the plan gets a workspace of its own (up to
  // kMaxWorkspaces), so runs on different streams from different host threads overlap on the device;
  // callers beyond that, and callers that share a stream, take turns on a workspace's mutex.  The
  // CUDA graphs captured for a stream belong to its workspace.
  struct GraphEntry {
    std::vector<const void*> key;   // input pointers, output pointers, stream
    int runs = 0;
    uint64_t last_used = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
  };
  struct Workspace {
    fb200_stream stream = nullptr;
    bool claimed = false;
    void* arena = nullptr;
    std::vector<void*> priv;
    std::mutex run_mu;
    std::vector<GraphEntry> graphs;   // a few pointer sets (the pipelined host path alternates two)
    uint64_t graph_clock = 0;
  };
  static constexpr size_t kMaxWorkspaces = 4;
  std::vector<std::unique_ptr<Workspace>> workspaces;
  std::vector<size_t> private_bytes;  // size of each private buffer
  std::vector<void*> stage_in, stage_out;  // device staging for run_host
  int launches = 0;
  std::mutex mu;
  // CUDA-graph replay of the step list: the first run with a given set of input/output pointers
  // is eager (it also performs every lazy initialisation), the second captures the launches into
  // a graph, later runs with the same pointers replay it with one cudaGraphLaunch.
  std::atomic<bool> graph_enabled{true};
  // pipelined host runs: two sets of staging buffers, a copy-in and a copy-out stream, and events
  // that order H2D(k) -> run(k) -> D2H(k) and keep a staging set from being reused too early
  std::vector<void*> stage_in2, stage_out2;
  cudaStream_t s_h2d = nullptr, s_d2h = nullptr;
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_run[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  uint64_t host_runs = 0;
  // inputs bound as device-resident parameters (fb200_plan_bind_resident): the host-buffer entry
  // points read them where they lie instead of copying them in
  std::vector<const void*> resident;
};

namespace fb200 {

// FRAME_B200_PLAN_DEBUG=1 prints to stderr why a group rewrite was not applied.
static bool plan_debug() {
  static const bool on = getenv("FRAME_B200_PLAN_DEBUG") != nullptr;
  return on;
}
#define PLAN_TRACE(...) do { if (plan_debug()) { fprintf(stderr, "[fb200 plan] " __VA_ARGS__); fputc('\n', stderr); } } while (0)

static const Attr* find_attr(const Step& s, const char* name) {
  for (const Attr& a : s.attrs) if (a.name == name) return &a;
  return nullptr;
}

static std::vector<int64_t> parse_int_list(const std::string& text) {
  std::vector<int64_t> out;
  const char* p = text.c_str();
  while (*p) {
    if ((*p >= '0' && *p <= '9') || *p == '-') {
      char* end = nullptr;
      out.push_back(strtoll(p, &end, 10));
      p = end;
    } else {
      ++p;
    }
  }
  return out;
}

static std::vector<double> parse_double_list(const std::string& text) {
  std::vector<double> out;
  const char* p = text.c_str();
  while (*p) {
    if ((*p >= '0' && *p <= '9') || *p == '-' || *p == '+' || *p == '.' || *p == 'i' || *p == 'n') {
      char* end = nullptr;
      const double v = strtod(p, &end);
      if (end == p) { ++p; continue; }
      out.push_back(v);
      p = end;
    } else {
      ++p;
    }
  }
  return out;
}

static std::string unquote(const std::string& t) {
  std::string out;
  size_t i = 0;
  while (i < t.size() && t[i] != '"') ++i;
  for (++i; i < t.size() && t[i] != '"'; ++i) {
    if (t[i] == '\\' && i + 1 < t.size()) { ++i; out += (t[i] == 'n') ? '\n' : t[i]; }
    else out += t[i];
  }
  return out;
}

static int ew_code(const std::string& name) {
  static const char* names[] = {"", "add", "mul", "relu", "square", "sigmoid", "tanh", "rsqrt",
                                "gelu", "silu", "softplus", "exp", "heaviside_surrogate", "relu_grad_internal"};
  for (int i = 1; i <= 13; ++i) if (name == names[i]) return i;
  return 0;
}

static int dtype_from_name(const std::string& text) {
  static const char* names[] = {"float32", "float64", "float16", "bfloat16", "int8", "int16",
                                "int32", "int64", "uint8", "bool"};
  for (int i = 0; i < 10; ++i) if (text.find(names[i]) != std::string::npos) return i;
  return -1;
}

// Resolves a slot to the slot whose bytes it shares.
static int root_slot(const fb200_plan& p, int s) {
  while (p.slots[s].alias_of >= 0) s = p.slots[s].alias_of;
  return s;
}

static bool ranges_overlap(const fb200_plan& p, int a, int b) {
  a = root_slot(p, a);
  b = root_slot(p, b);
  if (a == b) return true;
  const SlotInfo& x = p.slots[a];
  const SlotInfo& y = p.slots[b];
  if (x.arena_offset < 0 || y.arena_offset < 0) return false;  // distinct non-arena buffers
  const int64_t xe = x.arena_offset + static_cast<int64_t>(x.bytes());
  const int64_t ye = y.arena_offset + static_cast<int64_t>(y.bytes());
  return x.arena_offset < ye && y.arena_offset < xe;
}

static int parse_plan(const char* text, fb200_plan* p) {
  std::istringstream is(text);
  std::string line;
  int slot_count = 0;
  Step* cur = nullptr;
  while (std::getline(is, line)) {
    if (line.empty()) continue;
    std::istringstream ls(line);
    std::string tag;
    ls >> tag;
    if (tag == "plan") {
      std::string a, b;
      ls >> a >> b;
      if (a.rfind("slots=", 0) != 0 || b.rfind("arena=", 0) != 0) {
        return set_error(FB200_INVALID_ARGUMENT, "plan: malformed header '%s'", line.c_str());
      }
      slot_count = atoi(a.c_str() + 6);
      p->arena_bytes = strtoull(b.c_str() + 6, nullptr, 10);
      p->slots.assign(static_cast<size_t>(slot_count), SlotInfo{});
    } else if (tag == "in") {
      int idx, dtype, rank;
      ls >> idx >> dtype >> rank;
      if (idx < 0 || idx >= slot_count || rank < 0 || rank > 8) {
        return set_error(FB200_INVALID_ARGUMENT, "plan: bad input line '%s'", line.c_str());
      }
      SlotInfo& s = p->slots[idx];
      s.dtype = dtype;
      s.dims.resize(rank);
      s.numel = 1;
      for (int i = 0; i < rank; ++i) { ls >> s.dims[i]; s.numel *= s.dims[i]; }
      s.input_index = static_cast<int>(p->input_slots.size());
      p->input_slots.push_back(idx);
    } else if (tag == "step") {
      p->steps.emplace_back();
      cur = &p->steps.back();
      std::string tok;
      ls >> cur->op >> tok;
      if (tok.rfind("nin=", 0) != 0) return set_error(FB200_INVALID_ARGUMENT, "plan: bad step line '%s'", line.c_str());
      const int nin = atoi(tok.c_str() + 4);
      for (int i = 0; i < nin; ++i) { int s; ls >> s; cur->in.push_back(s); }
      ls >> tok;
      if (tok.rfind("nout=", 0) != 0) return set_error(FB200_INVALID_ARGUMENT, "plan: bad step line '%s'", line.c_str());
      const int nout = atoi(tok.c_str() + 5);
      for (int i = 0; i < nout; ++i) {
        int slot, dtype, rank;
        long long off;
        ls >> slot >> dtype >> off >> rank;
        if (slot < 0 || slot >= slot_count || rank < 0 || rank > 8) {
          return set_error(FB200_INVALID_ARGUMENT, "plan: bad step output in '%s'", line.c_str());
        }
        SlotInfo& s = p->slots[slot];
        s.dtype = dtype;
        s.arena_offset = off;
        s.dims.resize(rank);
        s.numel = 1;
        for (int d = 0; d < rank; ++d) { ls >> s.dims[d]; s.numel *= s.dims[d]; }
        cur->out.push_back(slot);
      }
      for (int s : cur->in) {
        if (s < 0 || s >= slot_count) return set_error(FB200_INVALID_ARGUMENT, "plan: slot out of range in '%s'", line.c_str());
      }
    } else if (tag == "attr") {
      if (cur == nullptr) return set_error(FB200_INVALID_ARGUMENT, "plan: attr before any step");
      Attr a;
      ls >> a.name >> a.kind;
      std::getline(ls, a.text);
      if (!a.text.empty() && a.text[0] == ' ') a.text.erase(0, 1);
      cur->attrs.push_back(a);
    } else if (tag == "out") {
      int s;
      ls >> s;
      if (s < 0 || s >= slot_count) return set_error(FB200_INVALID_ARGUMENT, "plan: bad out line '%s'", line.c_str());
      if (p->slots[s].output_index < 0) p->slots[s].output_index = static_cast<int>(p->output_slots.size());
      p->output_slots.push_back(s);
    } else {
      return set_error(FB200_INVALID_ARGUMENT, "plan: unknown line '%s'", line.c_str());
    }
  }
  if (p->slots.empty() && slot_count != 0) return set_error(FB200_INVALID_ARGUMENT, "plan: missing header");
  return FB200_OK;
}

// Decodes one step's attributes into its launch record.  Unknown op -> UNIMPLEMENTED with the
// op name (the contract of Backend::compile, include/frame/hal/backend.h:103-104).
static int decode_step(fb200_plan* p, Step& s) {
  const std::string& op = s.op;
  auto need = [&](const char* name) -> const Attr* {
    const Attr* a = find_attr(s, name);
    if (a == nullptr) set_error(FB200_INVALID_ARGUMENT, "op '%s' is missing required attribute '%s'", op.c_str(), name);
    return a;
  };
  if (!s.out.empty()) s.write_slot = s.out[0];
  if (op == "matmul") {
    s.kind = Kind::kMatmul;
  } else if (op == "conv2d") {
    s.kind = Kind::kConv2d;
    const Attr *st = need("stride"), *pd = need("padding"), *g = need("groups");
    if (!st || !pd || !g) return FB200_INVALID_ARGUMENT;
    auto sv = parse_int_list(st->text), pv = parse_int_list(pd->text), gv = parse_int_list(g->text);
    if (sv.size() != 2 || pv.size() != 2 || gv.size() != 1) return set_error(FB200_INVALID_ARGUMENT, "op 'conv2d': malformed attributes");
    s.iv = {sv[0], sv[1], pv[0], pv[1], gv[0]};
  } else if (op == "conv1d") {
    s.kind = Kind::kConv1d;
    const Attr *st = need("stride"), *pd = need("padding"), *g = need("groups");
    if (!st || !pd || !g) return FB200_INVALID_ARGUMENT;
    s.iv = {parse_int_list(st->text).at(0), parse_int_list(pd->text).at(0), parse_int_list(g->text).at(0)};
  } else if (op == "max_pool2d") {
    s.kind = Kind::kMaxPool;
    const Attr *k = need("kernel"), *st = need("stride"), *pd = need("padding");
    if (!k || !st || !pd) return FB200_INVALID_ARGUMENT;
    auto kv = parse_int_list(k->text), sv = parse_int_list(st->text), pv = parse_int_list(pd->text);
    if (kv.size() != 2 || sv.size() != 2 || pv.size() != 2) return set_error(FB200_INVALID_ARGUMENT, "op 'max_pool2d': malformed attributes");
    s.iv = {kv[0], kv[1], sv[0], sv[1], pv[0], pv[1]};
  } else if (op == "avg_pool2d") {
    s.kind = Kind::kAvgPool;
    const Attr *k = need("kernel"), *st = need("stride"), *pd = need("padding");
    if (!k || !st || !pd) return FB200_INVALID_ARGUMENT;
    auto kv = parse_int_list(k->text), sv = parse_int_list(st->text), pv = parse_int_list(pd->text);
    if (kv.size() != 2 || sv.size() != 2 || pv.size() != 2) return set_error(FB200_INVALID_ARGUMENT, "op 'avg_pool2d': malformed attributes");
    s.iv = {kv[0], kv[1], sv[0], sv[1], pv[0], pv[1]};
  } else if (op == "max_pool2d_select_internal" || op == "max_pool2d_grad_internal" || op == "avg_pool2d_grad_internal") {
    s.kind = op == "max_pool2d_select_internal" ? Kind::kPoolSelect
             : op == "max_pool2d_grad_internal" ? Kind::kMaxPoolGrad : Kind::kAvgPoolGrad;
    const Attr *k = need("kernel"), *st = need("stride"), *pd = need("padding");
    if (!k || !st || !pd) return FB200_INVALID_ARGUMENT;
    auto kv = parse_int_list(k->text), sv = parse_int_list(st->text), pv = parse_int_list(pd->text);
    if (kv.size() != 2 || sv.size() != 2 || pv.size() != 2) {
      return set_error(FB200_INVALID_ARGUMENT, "op '%s': malformed attributes", op.c_str());
    }
    s.iv = {kv[0], kv[1], sv[0], sv[1], pv[0], pv[1]};
  } else if (op == "conv2d_grad_input_internal" || op == "conv2d_grad_filter_internal") {
    s.kind = op == "conv2d_grad_input_internal" ? Kind::kConvGradInput : Kind::kConvGradFilter;
    const Attr *st = need("stride"), *pd = need("padding"), *g = need("groups");
    if (!st || !pd || !g) return FB200_INVALID_ARGUMENT;
    auto sv = parse_int_list(st->text), pv = parse_int_list(pd->text), gv = parse_int_list(g->text);
    if (sv.size() != 2 || pv.size() != 2 || gv.size() != 1) {
      return set_error(FB200_INVALID_ARGUMENT, "op '%s': malformed attributes", op.c_str());
    }
    s.iv = {sv[0], sv[1], pv[0], pv[1], gv[0]};
  } else if (op == "matmul_grad_lhs_internal") {
    s.kind = Kind::kMatmulGradLhs;
  } else if (op == "matmul_grad_rhs_internal") {
    s.kind = Kind::kMatmulGradRhs;
  } else if (op == "mse_loss") {
    s.kind = Kind::kMseLoss;
  } else if (op == "mse_loss_grad_internal") {
    s.kind = Kind::kMseLossGrad;
  } else if (op == "rfft") {
    s.kind = Kind::kRfft;
  } else if (op == "irfft") {
    s.kind = Kind::kIrfft;
    const Attr* n = need("n");
    if (!n) return FB200_INVALID_ARGUMENT;
    s.iv = {parse_int_list(n->text).at(0)};
  } else if (op == "gather") {
    s.kind = Kind::kGather;
    p->graph_enabled = false;   // the index check synchronises the stream
  } else if (op == "scatter_add" || op == "gather_grad_internal") {
    s.kind = Kind::kScatterAdd;
    p->graph_enabled = false;
  } else if (op == "heaviside_surrogate") {
    const Attr* a = need("alpha");
    if (!a) return FB200_INVALID_ARGUMENT;
    const double alpha = strtod(a->text.c_str(), nullptr);
    if (!(alpha > 0.0) || alpha != alpha || alpha > 1.7e308) {
      return set_error(FB200_INVALID_ARGUMENT, "op 'heaviside_surrogate': attribute 'alpha' must be finite and positive, got %g", alpha);
    }
    s.kind = Kind::kChain;
    s.chain_ops = {FB200_EW_HEAVISIDE};
    s.chain_arity = {1};
  } else if (op == "fused_elementwise_internal") {
    s.kind = Kind::kChain;
    const Attr *o = need("ops"), *a = need("arities");
    if (!o || !a) return FB200_INVALID_ARGUMENT;
    const std::string names = unquote(o->text);
    size_t start = 0;
    while (start <= names.size()) {
      const size_t semi = names.find(';', start);
      const std::string name = names.substr(start, semi == std::string::npos ? std::string::npos : semi - start);
      const int code = ew_code(name);
      if (code == 0) return set_error(FB200_UNIMPLEMENTED, "op 'fused_elementwise_internal': sub-op '%s' has no cuda kernel", name.c_str());
      s.chain_ops.push_back(code);
      if (semi == std::string::npos) break;
      start = semi + 1;
    }
    for (int64_t v : parse_int_list(a->text)) s.chain_arity.push_back(static_cast<int>(v));
    if (s.chain_arity.size() != s.chain_ops.size()) return set_error(FB200_INVALID_ARGUMENT, "op 'fused_elementwise_internal': ops/arities length mismatch");
  } else if (ew_code(op) != 0) {
    s.kind = Kind::kChain;
    s.chain_ops = {ew_code(op)};
    s.chain_arity = {ew_is_binary(ew_code(op)) ? 2 : 1};
  } else if (op == "bias_add") {
    s.kind = Kind::kBiasAdd;
  } else if (op == "softmax") {
    s.kind = Kind::kSoftmax;
  } else if (op == "layer_norm") {
    s.kind = Kind::kLayerNorm;
    const Attr* e = need("eps");
    if (!e) return FB200_INVALID_ARGUMENT;
    s.eps = strtod(e->text.c_str(), nullptr);
  } else if (op == "selective_scan") {
    s.kind = Kind::kScan;
  } else if (op == "mamba_scan") {
    s.kind = Kind::kMambaScan;
  } else if (op == "transpose") {
    s.kind = Kind::kTranspose;
    const Attr* pm = need("perm");
    if (!pm) return FB200_INVALID_ARGUMENT;
    s.iv = parse_int_list(pm->text);
  } else if (op == "slice") {
    s.kind = Kind::kSlice;
    const Attr *ax = need("axis"), *st = need("start"), *sp = need("stop");
    if (!ax || !st || !sp) return FB200_INVALID_ARGUMENT;
    s.iv = {parse_int_list(ax->text).at(0), parse_int_list(st->text).at(0), parse_int_list(sp->text).at(0)};
  } else if (op == "concat") {
    s.kind = Kind::kConcat;
    const Attr* ax = need("axis");
    if (!ax) return FB200_INVALID_ARGUMENT;
    s.iv = {parse_int_list(ax->text).at(0)};
  } else if (op == "sum") {
    s.kind = Kind::kSum;
    const Attr* ax = need("axes");
    if (!ax) return FB200_INVALID_ARGUMENT;
    s.iv = parse_int_list(ax->text);
  } else if (op == "reshape") {
    s.kind = Kind::kCopy;  // may become kAlias below
  } else if (op == "constant") {
    s.kind = Kind::kConstant;
  } else {
    return set_error(FB200_UNIMPLEMENTED, "op '%s' has no kernel registered for backend 'cuda'", op.c_str());
  }
  (void)p;
  return FB200_OK;
}

static int materialise_constant(fb200_plan* p, Step& s) {
  const Attr* v = find_attr(s, "value");
  if (v == nullptr) return set_error(FB200_INVALID_ARGUMENT, "op 'constant' is missing required attribute 'value'");
  SlotInfo& slot = p->slots[s.out[0]];
  std::vector<double> vals = parse_double_list(v->text);
  const int64_t n = slot.numel;
  if (static_cast<int64_t>(vals.size()) == 1 && n != 1) vals.assign(static_cast<size_t>(n), vals[0]);
  if (static_cast<int64_t>(vals.size()) != n) {
    return set_error(FB200_INVALID_ARGUMENT, "op 'constant': value has %zu elements, shape needs %lld", vals.size(), (long long)n);
  }
  if (n == 0) return FB200_OK;
  bool all_equal = true;
  for (int64_t i = 1; i < n && all_equal; ++i) all_equal = vals[static_cast<size_t>(i)] == vals[0];
  std::vector<uint8_t> host(slot.bytes());
  for (int64_t i = 0; i < n; ++i) {
    const double d = vals[i];
    switch (slot.dtype) {
      case FB200_F32: reinterpret_cast<float*>(host.data())[i] = static_cast<float>(d); break;
      case FB200_F64: reinterpret_cast<double*>(host.data())[i] = d; break;
      case FB200_BF16: {
        const float f = static_cast<float>(d);
        uint32_t bits; memcpy(&bits, &f, 4);
        uint16_t h;
        if ((bits & 0x7fffffffu) > 0x7f800000u) h = static_cast<uint16_t>((bits >> 16) | 0x40u);
        else h = static_cast<uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
        reinterpret_cast<uint16_t*>(host.data())[i] = h;
        break;
      }
      case FB200_F16: {
        const __half h = __float2half_rn(static_cast<float>(d));
        memcpy(host.data() + 2 * i, &h, 2);
        break;
      }
      case FB200_I32: reinterpret_cast<int32_t*>(host.data())[i] = static_cast<int32_t>(d); break;
      case FB200_I64: reinterpret_cast<int64_t*>(host.data())[i] = static_cast<int64_t>(d); break;
      default: return set_error(FB200_UNIMPLEMENTED, "op 'constant': unsupported dtype code %d", slot.dtype);
    }
  }
  // A constant that is also a graph output is copied into the caller's buffer at run time.
  slot.is_constant = true;
  if (!p->dry) {
    void* dev = nullptr;
    if (int rc = fb200_malloc(p->device, host.size(), 256, &dev)) return rc;
    p->owned.push_back(dev);
    if (int rc = fb200_memcpy(p->device, dev, host.data(), host.size(), FB200_H2D, nullptr, 1)) return rc;
    slot.constant = dev;
  }
  if (all_equal) {   // the value as the kernels will read it back from the slot's dtype
    float stored = static_cast<float>(vals[0]);
    if (slot.dtype == FB200_BF16) {
      uint32_t bits = static_cast<uint32_t>(reinterpret_cast<uint16_t*>(host.data())[0]) << 16;
      memcpy(&stored, &bits, 4);
    } else if (slot.dtype == FB200_F16) {
      __half h;
      memcpy(&h, host.data(), 2);
      stored = __half2float(h);
    }
    slot.splat = slot.dtype == FB200_F32 || slot.dtype == FB200_BF16 || slot.dtype == FB200_F16;
    slot.splat_value = stored;
  }
  return FB200_OK;
}

// Last step index that reads `slot` (through aliases too); graph outputs live to the end.
static int last_use(const fb200_plan& p, int slot) {
  int last = -1;
  const int root = root_slot(p, slot);
  for (size_t i = 0; i < p.steps.size(); ++i) {
    for (int in : p.steps[i].in) if (root_slot(p, in) == root) last = static_cast<int>(i);
  }
  for (int o : p.output_slots) if (root_slot(p, o) == root) last = static_cast<int>(p.steps.size());
  return last;
}

// A matmul whose result is only ever read through column slices, the last of which runs to the
// right edge: that last block is written by the GEMM itself into a buffer of the plan's own
// (outside the planner's arena, so no planned lifetime is disturbed) and the slice is dropped.  In
// the Mamba block this is the gate half z of in_proj: the planner reuses the bytes of the slice's
// output for the scan's result, so neither the slice nor the reshape behind it could become a view;
// with a private buffer both do (201 MB less to copy, twice, at the benchmark size).
static int split_matmul_tails(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  for (int i = 0; i < n; ++i) {
    Step& s = p->steps[static_cast<size_t>(i)];
    if (s.kind != Kind::kMatmul || s.in.size() != 2 || s.out.size() != 1 || !s.chain_ops.empty()) continue;
    const int x = s.out[0];
    const SlotInfo& xs = p->slots[static_cast<size_t>(x)];
    if (xs.output_index >= 0 || xs.dims.size() != 2 || xs.numel == 0) continue;
    const int64_t rows = xs.dims[0], cols = xs.dims[1];
    const int64_t k = p->slots[static_cast<size_t>(s.in[0])].dims.size() == 2 ? p->slots[static_cast<size_t>(s.in[0])].dims[1] : 0;
    if (!fb200_matmul_uses_tensor_cores(rows, cols, k, xs.dtype, p->allow_tf32)) continue;
    bool only_slices = true;
    int tail = -1;
    int64_t max_stop_before = 0;
    for (int o : p->output_slots) if (o == x) only_slices = false;
    for (int j = 0; j < n && only_slices; ++j) {
      const Step& t = p->steps[static_cast<size_t>(j)];
      bool reads = false;
      for (int in : t.in) if (in == x) reads = true;
      if (!reads) continue;
      if (t.kind != Kind::kSlice || t.in.size() != 1 || t.iv[0] != 1 || t.iv[1] < 0) { only_slices = false; break; }
      if (t.iv[2] == cols && tail < 0) tail = j;
      else max_stop_before = std::max(max_stop_before, t.iv[2]);
    }
    if (!only_slices || tail < 0) continue;
    const Step& ts = p->steps[static_cast<size_t>(tail)];
    const int64_t start = ts.iv[1];
    const int vec = 16 / itemsize_of(xs.dtype);
    if (start <= 0 || start % 32 != 0 || (cols - start) % vec != 0 || max_stop_before > start) continue;
    const int dst = ts.out[0];
    SlotInfo& ds = p->slots[static_cast<size_t>(dst)];
    if (ds.output_index >= 0 || ds.input_index >= 0 || ds.alias_of >= 0) continue;
    ds.private_index = static_cast<int>(p->private_bytes.size());
    p->private_bytes.push_back(ds.bytes());
    ds.arena_offset = -1;
    s.split_slot = dst;
    s.split_col = start;
    p->steps[static_cast<size_t>(tail)].kind = Kind::kSkip;
    PLAN_TRACE("matmul at step %d writes columns [%lld, %lld) straight into the output of the slice at step %d (private buffer)",
               i, (long long)start, (long long)cols, tail);
  }
  return FB200_OK;
}

static void optimise(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  // reshape -> alias when the aliased bytes cannot be overwritten while the alias is live
  for (int i = 0; i < n; ++i) {
    Step& s = p->steps[i];
    if (s.op != "reshape" || s.in.size() != 1 || s.out.size() != 1) continue;
    const int src = s.in[0], dst = s.out[0];
    if (p->slots[dst].output_index >= 0) continue;   // must land in the caller's buffer
    if (p->slots[dst].numel == 0) { s.kind = Kind::kSkip; continue; }
    const int end = last_use(*p, dst);
    bool safe = true;
    const int src_root = root_slot(*p, src);
    if (p->slots[src_root].output_index >= 0) safe = true;  // output buffers are never reused
    for (int j = i + 1; j <= end && j < n && safe; ++j) {
      for (int w : p->steps[j].out) {
        if (w != dst && p->slots[w].arena_offset >= 0 && p->slots[src_root].arena_offset >= 0 &&
            ranges_overlap(*p, w, src_root)) safe = false;
      }
    }
    if (safe) {
      p->slots[dst].alias_of = src;
      s.kind = Kind::kAlias;
    }
  }
  if (p->opt_level < 1) return;
  // matmul / conv2d absorb the elementwise group(s) that directly follow them
  for (int i = 0; i < n; ++i) {
    Step& s = p->steps[i];
    if (s.kind != Kind::kMatmul && s.kind != Kind::kConv2d) continue;
    int cur_out = s.out[0];
    for (int j = i + 1; j < n; ++j) {
      Step& t = p->steps[j];
      if (t.kind != Kind::kChain && t.kind != Kind::kBiasAdd) break;
      if (t.in.empty() || t.out.size() != 1) break;
      bool epilogue_ok = true;   // relu_grad_internal stays a chain of its own
      for (int c : t.chain_ops) epilogue_ok = epilogue_ok && ew_epilogue_ok(c);
      if (!epilogue_ok) break;
      // The contraction's result must be operand 0 of the group; add and mul commute exactly,
      // so a leading binary step may also take it as operand 1.
      size_t lhs_index = 0;
      if (t.in[0] != cur_out) {
        if (t.kind == Kind::kChain && t.chain_arity[0] == 2 && ew_commutes(t.chain_ops[0]) && t.in.size() >= 2 &&
            t.in[1] == cur_out) {
          lhs_index = 1;
        } else {
          break;
        }
      }
      std::vector<int> ext;
      for (size_t a = 0; a < t.in.size(); ++a) if (a != lhs_index) ext.push_back(t.in[a]);
      if (p->slots[cur_out].output_index >= 0) break;          // the intermediate is observable
      if (p->slots[t.out[0]].dtype != p->slots[cur_out].dtype) break;
      if (p->slots[t.out[0]].dtype == FB200_I32 || p->slots[t.out[0]].dtype == FB200_I64) break;
      // single consumer: nobody else reads cur_out
      bool single = true;
      for (int q = 0; q < n && single; ++q) {
        if (q == j) {
          for (int e : ext) if (e == cur_out) single = false;
          continue;
        }
        for (int in : p->steps[q].in) if (in == cur_out) single = false;
      }
      if (!single) break;
      const int add_ops = t.kind == Kind::kBiasAdd ? 1 : static_cast<int>(t.chain_ops.size());
      if (static_cast<int>(s.chain_ops.size()) + add_ops > FB200_MAX_CHAIN) break;
      // the fused store goes to t's output: it must not overlap anything the contraction reads
      bool overlap = false;
      for (int in : s.in) if (ranges_overlap(*p, t.out[0], in)) overlap = true;
      for (int os : s.epi_operand_slot) if (os >= 0 && ranges_overlap(*p, t.out[0], os)) overlap = true;
      for (int e : ext) if (ranges_overlap(*p, t.out[0], e)) overlap = true;
      if (overlap) {
        // The planner laid the arena out for the separate steps and reused bytes that the
        // contraction still reads (typically its own A operand) for the group's result.  A private
        // buffer for that result removes the conflict.
        SlotInfo& os = p->slots[static_cast<size_t>(root_slot(*p, t.out[0]))];
        if (os.input_index >= 0 || os.output_index >= 0 || os.constant != nullptr || os.arena_offset < 0) break;
        // a single add in front of a LayerNorm is left to that rewrite (one pass over the rows
        // instead of an epilogue that nothing overlaps)
        if (j + 1 < n && p->steps[static_cast<size_t>(j + 1)].kind == Kind::kLayerNorm &&
            !p->steps[static_cast<size_t>(j + 1)].in.empty() && p->steps[static_cast<size_t>(j + 1)].in[0] == t.out[0] &&
            t.chain_ops.size() == 1 && t.chain_ops[0] == FB200_EW_ADD) break;
        os.private_index = static_cast<int>(p->private_bytes.size());
        p->private_bytes.push_back(os.bytes());
        os.arena_offset = -1;
        PLAN_TRACE("step %d: the epilogue's result overlapped an operand of the contraction at step %d and moves to a private buffer (%zu bytes)",
                   j, i, os.bytes());
      }
      if (t.kind == Kind::kBiasAdd) {
        if (s.kind != Kind::kMatmul || ext.size() != 1) break;
        s.chain_ops.push_back(FB200_EW_ADD);
        s.epi_operand_slot.push_back(ext[0]);
        s.epi_mode.push_back(FB200_OPERAND_COL);
      } else {
        size_t next_ext = 0;
        for (size_t c = 0; c < t.chain_ops.size(); ++c) {
          s.chain_ops.push_back(t.chain_ops[c]);
          if (t.chain_arity[c] == 2) {
            s.epi_operand_slot.push_back(ext[next_ext++]);
            s.epi_mode.push_back(FB200_OPERAND_FULL);
          } else {
            s.epi_operand_slot.push_back(-1);
            s.epi_mode.push_back(FB200_OPERAND_FULL);
          }
        }
      }
      s.write_slot = t.out[0];
      t.kind = Kind::kSkip;
      cur_out = t.out[0];
    }
  }
}


// conv2d [+ epilogue] -> max_pool2d becomes one step (fb200_conv2d_max_pool) when the pool is the only
// reader of the convolution's result and that result is not a graph output.  The call itself
// decides whether the pair runs as one kernel (an image stem: the pooled rows leave the epilogue and
// the convolution's result is never written) or as the two kernels through the planned intermediate.
static void fuse_conv_pool(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  auto runs = [](const Step& s) { return s.kind != Kind::kSkip && s.kind != Kind::kAlias && s.kind != Kind::kConstant; };
  for (int i = 0; i < n; ++i) {
    Step& s = p->steps[i];
    if (s.kind != Kind::kConv2d || s.write_slot < 0 || !s.pool_iv.empty()) continue;
    const int mid = s.write_slot;
    if (p->slots[mid].output_index >= 0 || p->slots[mid].dtype != FB200_F32) continue;
    int j = i + 1;
    while (j < n && !runs(p->steps[j])) ++j;
    if (j >= n) continue;
    Step& t = p->steps[j];
    if (t.kind != Kind::kMaxPool || t.in.size() != 1 || t.out.size() != 1 || t.in[0] != mid) continue;
    bool single = true;
    for (int q = 0; q < n && single; ++q) {
      if (q == j || !runs(p->steps[q])) continue;
      for (int in : p->steps[q].in) if (in == mid) single = false;
      for (int in : p->steps[q].epi_operand_slot) if (in == mid) single = false;
    }
    if (!single) continue;
    // the pooled result must not overlap anything the convolution reads (or its intermediate, which
    // the two-kernel form still writes)
    bool overlap = ranges_overlap(*p, t.out[0], mid);
    for (int in : s.in) if (ranges_overlap(*p, t.out[0], in)) overlap = true;
    for (int os : s.epi_operand_slot) if (os >= 0 && ranges_overlap(*p, t.out[0], os)) overlap = true;
    if (overlap) continue;
    s.pool_mid = mid;
    s.pool_iv = t.iv;
    s.write_slot = t.out[0];
    t.kind = Kind::kSkip;
  }
}

// add(a, b) -> layer_norm becomes one step (fb200_add_layer_norm) when the layer_norm is the next
// step that runs: a transformer block's residual add and the normalisation behind it.  The sum is
// still stored (the block's second residual reads it); the normalisation works from registers.
static void fuse_add_layer_norm(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  auto runs = [](const Step& s) { return s.kind != Kind::kSkip && s.kind != Kind::kAlias && s.kind != Kind::kConstant; };
  for (int i = 0; i < n; ++i) {
    Step& a = p->steps[i];
    if (a.kind != Kind::kChain || a.chain_ops.size() != 1 || a.chain_ops[0] != FB200_EW_ADD || a.chain_arity[0] != 2 ||
        a.in.size() != 2 || a.out.size() != 1 || a.write_slot != a.out[0]) continue;
    const int sum = a.out[0];
    int j = i + 1;
    while (j < n && !runs(p->steps[j])) ++j;
    if (j >= n) continue;
    Step& ln = p->steps[j];
    if (ln.kind != Kind::kLayerNorm || ln.in.size() != 3 || ln.in[0] != sum || ln.ln_res >= 0) continue;
    const SlotInfo& ss = p->slots[sum];
    if (ss.dims.size() != 2) continue;
    bool same = true;
    for (int in : a.in) same = same && p->slots[in].dims == ss.dims && p->slots[in].dtype == ss.dtype;
    if (!same) continue;
    const int out = ln.write_slot;
    // One kernel reads a, b, gamma, beta and writes the sum and the result.  A warp holds its whole
    // row of a and b in registers before it writes anything, and touches no other row, so the result
    // (or the sum) may sit EXACTLY on an addend (same bytes, same row layout: the planner likes to
    // put the normalised rows where the dead addend was); any other overlap is refused.
    auto exact = [&](int x, int y) {
      const SlotInfo& sx = p->slots[root_slot(*p, x)];
      const SlotInfo& sy = p->slots[root_slot(*p, y)];
      return sx.arena_offset >= 0 && sx.arena_offset == sy.arena_offset && sx.bytes() == sy.bytes();
    };
    bool overlap = ranges_overlap(*p, out, sum);
    for (int in : a.in) {
      if (ranges_overlap(*p, out, in) && !exact(out, in)) overlap = true;
      if (ranges_overlap(*p, sum, in) && !exact(sum, in)) overlap = true;
    }
    for (size_t q = 1; q < ln.in.size(); ++q) {
      if (ranges_overlap(*p, out, ln.in[q]) || ranges_overlap(*p, sum, ln.in[q])) overlap = true;
    }
    if (overlap) continue;
    ln.in[0] = a.in[0];
    ln.ln_res = a.in[1];
    ln.ln_sum = sum;
    a.kind = Kind::kSkip;
  }
}

static bool step_runs(const Step& s) {
  return s.kind != Kind::kSkip && s.kind != Kind::kAlias && s.kind != Kind::kConstant;
}

// Index of the step that writes the bytes of `slot` (through its own output or as the fused
// result of a contraction), or -1.
static int writer_of(const fb200_plan& p, int slot) {
  const int root = root_slot(p, slot);
  for (size_t j = 0; j < p.steps.size(); ++j) {
    const Step& s = p.steps[j];
    if (!step_runs(s) || s.write_slot < 0) continue;
    if (root_slot(p, s.write_slot) == root) return static_cast<int>(j);
  }
  return -1;
}

// Does step `s` read or write bytes overlapping `slot`, other than through slots rooted at `own`?
static bool step_touches(const fb200_plan& p, const Step& s, int slot, int own) {
  auto hit = [&](int x) { return x >= 0 && root_slot(p, x) != own && ranges_overlap(p, x, slot); };
  for (int x : s.in) if (hit(x)) return true;
  for (int x : s.epi_operand_slot) if (hit(x)) return true;
  if (hit(s.write_slot)) return true;
  if (hit(s.pool_mid)) return true;
  if (hit(s.ln_res) || hit(s.ln_sum)) return true;
  for (int x : {s.fan_q, s.fan_k, s.fan_v, s.fan_dest, s.dw_x, s.dw_w, s.dw_bias}) if (hit(x)) return true;
  return false;
}

// ---- attention-fan recognition ------------------------------------------------------------------
// A window of a rank-2 matrix reached through a chain of `slice` steps.
struct Window { int base; int64_t row, col; };

static Window resolve_window(const fb200_plan& p, const std::vector<int>& producer, int slot) {
  Window w{slot, 0, 0};
  for (;;) {
    const int j = producer[static_cast<size_t>(w.base)];
    if (j < 0) break;
    const Step& s = p.steps[static_cast<size_t>(j)];
    if (s.kind != Kind::kSlice || s.in.size() != 1) break;
    const SlotInfo& src = p.slots[static_cast<size_t>(s.in[0])];
    if (src.dims.size() != 2 || s.iv[1] < 0) break;
    if (s.iv[0] == 0) w.row += s.iv[1]; else w.col += s.iv[1];
    w.base = s.in[0];
  }
  return w;
}

// Live steps that read `slot` (directly, through an alias, or as an epilogue operand).
static std::vector<std::pair<int, int>> readers_of(const fb200_plan& p, int slot) {
  std::vector<std::pair<int, int>> out;
  const int root = root_slot(p, slot);
  for (size_t j = 0; j < p.steps.size(); ++j) {
    const Step& s = p.steps[j];
    if (s.kind == Kind::kSkip || s.kind == Kind::kAlias) continue;
    for (size_t i = 0; i < s.in.size(); ++i) {
      if (root_slot(p, s.in[i]) == root) out.emplace_back(static_cast<int>(j), static_cast<int>(i));
    }
    for (int e : s.epi_operand_slot) if (e >= 0 && root_slot(p, e) == root) out.emplace_back(static_cast<int>(j), -1);
  }
  return out;
}

struct FanHead {
  int transpose, scores, softmax, values;   // step indices
  float scale;                              // 1, or the splat constant the scores are multiplied by
  int scale_step;                           // the mul step when it is a step of its own, else -1
  Window q, k, v;
  int dest;                                 // slot the result finally lands in
  int64_t dest_row, dest_col;
  std::vector<std::pair<int, int>> path;    // (concat step, input index) from the head outwards
};

// Finds groups of `matmul(q, transpose(k)) -> softmax -> matmul(p, v)` chains whose operands are
// windows of common matrices and whose results are concatenated into one matrix, and replaces each
// group by ONE attention_fan launch at the position of its last step.  The windows are read in
// place and the results are written straight into the concatenated matrix, so the slices,
// transposes and concats of the group are not executed at all.  Because that moves reads and
// writes in time relative to what the memory planner assumed, the group is only formed when
//  (1) no step that still runs between the producer of a source matrix and the launch writes
//      bytes overlapping that matrix,
//  (2) no step that still runs between the launch and the (skipped) outermost concat touches bytes
//      overlapping the destination, and every reader of the destination comes after the launch,
//  (3) every concat on the way is fed only by heads of the group (or by such concats).
// Anything else keeps the step-by-step path.
static void fuse_attention_fans(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  std::vector<int> producer(p->slots.size(), -1);
  for (int i = 0; i < n; ++i) {
    for (int o : p->steps[static_cast<size_t>(i)].out) producer[static_cast<size_t>(o)] = i;
  }
  auto sole_reader = [&](int slot, int* step, int* index) {
    if (p->slots[static_cast<size_t>(slot)].output_index >= 0) return false;
    const auto r = readers_of(*p, slot);
    if (r.size() != 1 || r[0].second < 0) return false;
    *step = r[0].first;
    *index = r[0].second;
    return true;
  };
  std::vector<FanHead> heads;
  for (int i = 0; i < n; ++i) {
    const Step& sm = p->steps[static_cast<size_t>(i)];
    if (sm.kind != Kind::kSoftmax || sm.in.size() != 1 || sm.out.size() != 1) continue;
    FanHead h{};
    h.softmax = i;
    // The scores: a matmul, possibly followed by a `mul` with a constant filled with one value (the
    // reference's own attention scales by 1/sqrt(d) there, src/nn/layers.cpp:1062-1071).  That mul
    // is either still a step of its own or has been absorbed as the matmul's epilogue.
    h.scale = 1.0f;
    h.scale_step = -1;
    int scores_slot = sm.in[0];
    int w0 = writer_of(*p, scores_slot);
    if (w0 < 0) { PLAN_TRACE("softmax step %d: no producer for its input", i); continue; }
    auto splat_of = [&](int slot, float* value) {
      const SlotInfo& c = p->slots[static_cast<size_t>(root_slot(*p, slot))];
      if (!c.is_constant || !c.splat) return false;
      *value = c.splat_value;
      return true;
    };
    if (p->steps[static_cast<size_t>(w0)].kind == Kind::kChain) {
      const Step& mu = p->steps[static_cast<size_t>(w0)];
      int sole = -1, sole_index = -1;
      if (mu.chain_ops.size() != 1 || mu.chain_ops[0] != FB200_EW_MUL || mu.in.size() != 2 ||
          !sole_reader(mu.out[0], &sole, &sole_index) || sole != i) {
        PLAN_TRACE("softmax step %d: input written by step %d (%s), not a matmul or a mul", i, w0, mu.op.c_str());
        continue;
      }
      float value = 1.0f;
      int x = -1;
      if (splat_of(mu.in[1], &value)) x = mu.in[0];
      else if (splat_of(mu.in[0], &value)) x = mu.in[1];
      if (x < 0) { PLAN_TRACE("softmax step %d: scores are multiplied by a tensor that is not a constant splat", i); continue; }
      h.scale = value;
      h.scale_step = w0;
      scores_slot = x;
      w0 = writer_of(*p, scores_slot);
      if (w0 < 0) continue;
    }
    h.scores = w0;
    const Step& m1 = p->steps[static_cast<size_t>(h.scores)];
    if (m1.kind != Kind::kMatmul || m1.in.size() != 2 || m1.write_slot != scores_slot) {
      PLAN_TRACE("softmax step %d: scores written by step %d (%s), not a matmul", i, h.scores, m1.op.c_str());
      continue;
    }
    if (!m1.chain_ops.empty()) {
      float value = 1.0f;
      if (h.scale_step >= 0 || m1.chain_ops.size() != 1 || m1.chain_ops[0] != FB200_EW_MUL ||
          m1.epi_operand_slot[0] < 0 || m1.epi_mode[0] != FB200_OPERAND_FULL ||
          !splat_of(m1.epi_operand_slot[0], &value)) {
        PLAN_TRACE("softmax step %d: scores have an epilogue other than one mul by a constant splat", i);
        continue;
      }
      h.scale = value;
    }
    if (!(h.scale > 0.0f)) { PLAN_TRACE("softmax step %d: non-positive score scale", i); continue; }
    int step = -1, index = -1;
    if (!sole_reader(m1.write_slot, &step, &index) || step != (h.scale_step >= 0 ? h.scale_step : i)) { PLAN_TRACE("softmax step %d: scores have other readers", i); continue; }
    h.transpose = producer[static_cast<size_t>(m1.in[1])];
    if (h.transpose < 0) { PLAN_TRACE("softmax step %d: k operand has no producer", i); continue; }
    const Step& tr = p->steps[static_cast<size_t>(h.transpose)];
    if (tr.kind != Kind::kTranspose || tr.iv.size() != 2 || tr.iv[0] != 1 || tr.iv[1] != 0) { PLAN_TRACE("softmax step %d: k operand is not a [1,0] transpose", i); continue; }
    if (!sole_reader(tr.out[0], &step, &index) || step != h.scores) { PLAN_TRACE("softmax step %d: transposed k has other readers", i); continue; }
    if (!sole_reader(sm.out[0], &step, &index) || index != 0) { PLAN_TRACE("softmax step %d: probabilities are not the lhs of exactly one step", i); continue; }
    h.values = step;
    const Step& m2 = p->steps[static_cast<size_t>(h.values)];
    if (m2.kind != Kind::kMatmul || !m2.chain_ops.empty() || m2.write_slot != m2.out[0] || m2.in.size() != 2) { PLAN_TRACE("softmax step %d: consumer is not a plain matmul", i); continue; }
    const SlotInfo& qs = p->slots[static_cast<size_t>(m1.in[0])];
    const SlotInfo& ks = p->slots[static_cast<size_t>(tr.in[0])];
    const SlotInfo& vs = p->slots[static_cast<size_t>(m2.in[1])];
    if (qs.dims.size() != 2 || ks.dims.size() != 2 || vs.dims.size() != 2) continue;
    if (qs.dims[1] != ks.dims[1] || vs.dims[0] != ks.dims[0] || vs.dims[1] != qs.dims[1]) continue;
    if (ks.dtype != qs.dtype || vs.dtype != qs.dtype) continue;
    if (!fb200_attention_fan_supported(qs.dims[0], ks.dims[0], qs.dims[1], qs.dtype)) { PLAN_TRACE("softmax step %d: shape/dtype outside the fused kernel (sq %lld sk %lld d %lld dtype %d)", i, (long long)qs.dims[0], (long long)ks.dims[0], (long long)qs.dims[1], qs.dtype); continue; }
    h.q = resolve_window(*p, producer, m1.in[0]);
    h.k = resolve_window(*p, producer, tr.in[0]);
    h.v = resolve_window(*p, producer, m2.in[1]);
    bool ok = true;
    for (const Window* w : {&h.q, &h.k, &h.v}) {
      const SlotInfo& b = p->slots[static_cast<size_t>(w->base)];
      if (b.dims.size() != 2 || b.dims[1] % 8 != 0 || w->col % 8 != 0 || b.dims[0] > 0x7fffffff ||
          b.dims[1] > 0x7fffffff) ok = false;
    }
    if (!ok) { PLAN_TRACE("softmax step %d: operand windows are not 16-byte addressable", i); continue; }
    // where the result finally lands
    int cur = m2.out[0];
    h.dest_row = h.dest_col = 0;
    while (sole_reader(cur, &step, &index)) {
      const Step& c = p->steps[static_cast<size_t>(step)];
      if (c.kind != Kind::kConcat || p->slots[static_cast<size_t>(c.out[0])].dims.size() != 2) break;
      const int64_t axis = c.iv[0];
      int64_t off = 0;
      for (int a = 0; a < index; ++a) off += p->slots[static_cast<size_t>(c.in[static_cast<size_t>(a)])].dims[static_cast<size_t>(axis)];
      if (axis == 0) h.dest_row += off; else h.dest_col += off;
      h.path.emplace_back(step, index);
      cur = c.out[0];
    }
    h.dest = cur;
    const SlotInfo& d = p->slots[static_cast<size_t>(h.dest)];
    if (d.dims.size() != 2 || d.dims[1] % 8 != 0 || h.dest_col % 8 != 0) { PLAN_TRACE("softmax step %d: destination not addressable", i); continue; }
    heads.push_back(h);
  }
  std::vector<char> used(heads.size(), 0);
  for (size_t g = 0; g < heads.size(); ++g) {
    if (used[g]) continue;
    // the group: every head with the same source matrices, destination and shape
    std::vector<size_t> group;
    const SlotInfo& q0 = p->slots[static_cast<size_t>(p->steps[static_cast<size_t>(heads[g].scores)].in[0])];
    const SlotInfo& k0 = p->slots[static_cast<size_t>(p->steps[static_cast<size_t>(heads[g].transpose)].in[0])];
    for (size_t o = g; o < heads.size(); ++o) {
      if (used[o]) continue;
      const SlotInfo& qo = p->slots[static_cast<size_t>(p->steps[static_cast<size_t>(heads[o].scores)].in[0])];
      const SlotInfo& ko = p->slots[static_cast<size_t>(p->steps[static_cast<size_t>(heads[o].transpose)].in[0])];
      if (heads[o].q.base == heads[g].q.base && heads[o].k.base == heads[g].k.base &&
          heads[o].v.base == heads[g].v.base && heads[o].dest == heads[g].dest &&
          qo.dims == q0.dims && ko.dims == k0.dims && qo.dtype == q0.dtype &&
          heads[o].scale == heads[g].scale) {
        group.push_back(o);
        used[o] = 1;
      }
    }
    // tentatively skip the group's steps, then check the three conditions
    std::vector<Kind> saved(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) saved[static_cast<size_t>(i)] = p->steps[static_cast<size_t>(i)].kind;
    auto restore = [&]() { for (int i = 0; i < n; ++i) p->steps[static_cast<size_t>(i)].kind = saved[static_cast<size_t>(i)]; };
    int pos = -1, outer_concat = -1;
    std::vector<int> concats;
    for (size_t o : group) {
      const FanHead& h = heads[o];
      pos = std::max(pos, h.values);
      for (const auto& pc : h.path) {
        if (std::find(concats.begin(), concats.end(), pc.first) == concats.end()) concats.push_back(pc.first);
        outer_concat = std::max(outer_concat, pc.first);
      }
    }
    // (3) every input of every concat on the way comes from the group
    bool ok = true;
    for (int c : concats) {
      const Step& cs = p->steps[static_cast<size_t>(c)];
      for (size_t a = 0; a < cs.in.size() && ok; ++a) {
        bool fed = false;
        for (size_t o : group) {
          for (const auto& pc : heads[o].path) if (pc.first == c && pc.second == static_cast<int>(a)) fed = true;
        }
        if (!fed) ok = false;
      }
    }
    if (!ok) { PLAN_TRACE("fan of %zu heads: a concat on the way has inputs from outside the fan", group.size()); continue; }
    for (size_t o : group) {
      const FanHead& h = heads[o];
      for (int j : {h.transpose, h.scores, h.softmax, h.values}) p->steps[static_cast<size_t>(j)].kind = Kind::kSkip;
      if (h.scale_step >= 0) p->steps[static_cast<size_t>(h.scale_step)].kind = Kind::kSkip;
    }
    for (int c : concats) p->steps[static_cast<size_t>(c)].kind = Kind::kSkip;
    // slices nobody reads any more
    for (bool changed = true; changed;) {
      changed = false;
      for (int i = 0; i < n; ++i) {
        Step& s = p->steps[static_cast<size_t>(i)];
        if (s.kind != Kind::kSlice || p->slots[static_cast<size_t>(s.out[0])].output_index >= 0) continue;
        if (readers_of(*p, s.out[0]).empty()) { s.kind = Kind::kSkip; changed = true; }
      }
    }
    const FanHead& first = heads[group[0]];
    // (1) the source matrices stay intact until the launch
    for (int base : {first.q.base, first.k.base, first.v.base}) {
      const int from = producer[static_cast<size_t>(root_slot(*p, base))];
      for (int j = from + 1; j < pos && ok; ++j) {
        const Step& s = p->steps[static_cast<size_t>(j)];
        if (s.kind == Kind::kSkip || s.kind == Kind::kAlias || s.kind == Kind::kConstant) continue;
        for (int w : s.out) if (ranges_overlap(*p, w, base)) ok = false;
        if (s.write_slot >= 0 && ranges_overlap(*p, s.write_slot, base)) ok = false;
      }
    }
    // (2) the destination: readers come after the launch; nothing that still runs before the
    // outermost concat's position touches its bytes
    for (const auto& r : readers_of(*p, first.dest)) if (r.first <= pos) ok = false;
    for (int j = pos + 1; j < outer_concat && ok; ++j) {
      const Step& s = p->steps[static_cast<size_t>(j)];
      if (s.kind == Kind::kSkip || s.kind == Kind::kAlias || s.kind == Kind::kConstant) continue;
      for (int w : s.out) if (ranges_overlap(*p, w, first.dest)) ok = false;
      for (int r : s.in) if (ranges_overlap(*p, r, first.dest)) ok = false;
      for (int e : s.epi_operand_slot) if (e >= 0 && ranges_overlap(*p, e, first.dest)) ok = false;
      if (s.write_slot >= 0 && ranges_overlap(*p, s.write_slot, first.dest)) ok = false;
    }
    // without a concat on the way the result stays where the planner put it, but is written later
    // than planned: its bytes must not be in use by a step that still runs in between
    if (concats.empty() && group.size() != 1) ok = false;
    std::vector<fb200_attention_head> table;
    const int64_t o_ld = p->slots[static_cast<size_t>(first.dest)].dims[1];
    for (size_t o : group) {
      const FanHead& h = heads[o];
      fb200_attention_head e{};
      const int64_t coords[6] = {h.q.row, h.q.col, h.k.row, h.k.col, h.v.row, h.v.col};
      for (int64_t c : coords) if (c < 0 || c > 0x7fffffff) ok = false;
      e.q_row = static_cast<int32_t>(h.q.row); e.q_col = static_cast<int32_t>(h.q.col);
      e.k_row = static_cast<int32_t>(h.k.row); e.k_col = static_cast<int32_t>(h.k.col);
      e.v_row = static_cast<int32_t>(h.v.row); e.v_col = static_cast<int32_t>(h.v.col);
      e.o_offset = h.dest_row * o_ld + h.dest_col;
      table.push_back(e);
    }
    // (3) the planner laid the arena out for the unfused graph, in which the source matrices are
    // dead (sliced into per-head copies) long before the concat's result is written, so it may have
    // put that result over them.  The launch reads the sources while it writes the result: a result
    // that overlaps a source moves to a private buffer.
    const int dest_root = root_slot(*p, first.dest);
    bool dest_private = false;
    for (int base : {first.q.base, first.k.base, first.v.base}) {
      if (ranges_overlap(*p, dest_root, base)) dest_private = true;
    }
    if (dest_private) {
      const SlotInfo& ds = p->slots[static_cast<size_t>(dest_root)];
      if (ds.input_index >= 0 || ds.output_index >= 0 || ds.constant != nullptr || ds.arena_offset < 0) ok = false;
      for (int base : {first.q.base, first.k.base, first.v.base}) if (root_slot(*p, base) == dest_root) ok = false;
    }
    void* dev_table = nullptr;
    if (ok && !p->dry) {
      const size_t bytes = table.size() * sizeof(fb200_attention_head);
      ok = fb200_malloc(p->device, bytes, 256, &dev_table) == FB200_OK &&
           fb200_memcpy(p->device, dev_table, table.data(), bytes, FB200_H2D, nullptr, /*blocking*/ 1) == FB200_OK;
      if (!ok && dev_table) { fb200_free(p->device, dev_table); dev_table = nullptr; }
    }
    if (!ok) { PLAN_TRACE("fan of %zu heads ending at step %d: rejected by the byte-range checks", group.size(), pos); restore(); continue; }
    PLAN_TRACE("fan of %zu heads -> one attention_fan launch at step %d (scale %g)", group.size(), pos, first.scale);
    if (dev_table != nullptr) p->owned.push_back(dev_table);
    if (dest_private) {
      SlotInfo& ds = p->slots[static_cast<size_t>(dest_root)];
      ds.private_index = static_cast<int>(p->private_bytes.size());
      p->private_bytes.push_back(ds.bytes());
      ds.arena_offset = -1;
      PLAN_TRACE("fan at step %d: its result overlapped a source matrix in the arena and moves to a private buffer (%zu bytes)",
                 pos, ds.bytes());
    }
    Step& launch = p->steps[static_cast<size_t>(pos)];
    launch.kind = Kind::kAttentionFan;
    launch.fan_q = first.q.base; launch.fan_k = first.k.base; launch.fan_v = first.v.base;
    launch.fan_dest = first.dest;
    launch.fan_heads = static_cast<int64_t>(group.size());
    launch.fan_sq = q0.dims[0];
    launch.fan_sk = k0.dims[0];
    launch.fan_table = dev_table;
    launch.fan_scale = first.scale;
  }
}

// reshape whose source could not become the view (the planner reuses the source's bytes while the
// result is live): make the SOURCE a view of the result instead, i.e. let the source's producer
// write where the planner put the reshape's output (an arena range, or the caller's output
// buffer).  Safe when no step that runs between that producer and the reshape touches those
// bytes, and the source is not read after the result's bytes may be reused.
static void alias_reshape_sources(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  // Last reshape first: in a chain a -> b -> c, b must already share c's bytes when a is considered,
  // because b's own planned bytes may be what a's producer reads.  A reshape that became a view
  // no longer reads or writes anything, which can make an earlier candidate safe: sweep until
  // nothing changes.
  for (int sweep = 0, changed = 1; changed && sweep < 8; ++sweep) {
  changed = 0;
  for (int i = n - 1; i >= 0; --i) {
    Step& s = p->steps[static_cast<size_t>(i)];
    if (s.op != "reshape" || s.kind != Kind::kCopy || s.in.size() != 1 || s.out.size() != 1) continue;
    const int dst = s.out[0];
    const int r = root_slot(*p, s.in[0]);
    const int dr = root_slot(*p, dst);
    const SlotInfo& rs = p->slots[static_cast<size_t>(r)];
    const SlotInfo& ds = p->slots[static_cast<size_t>(dr)];
    if (r == dr) continue;
    if (rs.arena_offset < 0 || rs.input_index >= 0 || rs.output_index >= 0 || rs.constant != nullptr) continue;
    if (ds.bytes() != rs.bytes() || ds.numel == 0 || ds.input_index >= 0 || ds.constant != nullptr) continue;
    if (ds.arena_offset < 0 && ds.output_index < 0) continue;
    const int d = writer_of(*p, r);
    if (d < 0 || d >= i) continue;
    const int src_last = last_use(*p, r), dst_last = std::max(i, last_use(*p, dst));
    if (src_last > dst_last) continue;
    bool safe = true;
    for (int j = d; j < i && safe; ++j) {
      const Step& t = p->steps[static_cast<size_t>(j)];
      if (step_runs(t) && step_touches(*p, t, dst, r)) safe = false;
    }
    if (!safe) continue;
    p->slots[static_cast<size_t>(r)].alias_of = dst;
    s.kind = Kind::kAlias;
    changed = 1;
  }
  }
}

// transpose(0,2,1) -> conv1d(groups = channels, stride 1) [-> slice along time] [-> unary chain]
// -> transpose(0,2,1)  becomes one time-major depthwise convolution at the position of the last
// transpose.  The input may be a column window of a wider matrix (a `slice` along the columns
// followed by a reshape that became a view): it is then read in place.  The result is written
// where and when the planner expected the last transpose's output, so only the inputs move in
// time: the group is formed when no step that still runs in between writes bytes overlapping the
// input matrix, the weights or the bias, and the result does not overlap them either.
static void fuse_time_major_convs(fb200_plan* p) {
  const int n = static_cast<int>(p->steps.size());
  std::vector<int> producer(p->slots.size(), -1);
  for (int i = 0; i < n; ++i) for (int o : p->steps[static_cast<size_t>(i)].out) producer[static_cast<size_t>(o)] = i;
  auto sole_reader = [&](int slot, int* step) {
    if (p->slots[static_cast<size_t>(slot)].output_index >= 0) return false;
    const auto r = readers_of(*p, slot);
    if (r.size() != 1 || r[0].second < 0) return false;
    *step = r[0].first;
    return true;
  };
  auto is_time_swap = [](const Step& t) {
    return t.kind == Kind::kTranspose && t.iv.size() == 3 && t.iv[0] == 0 && t.iv[1] == 2 && t.iv[2] == 1;
  };
  for (int ci = 0; ci < n; ++ci) {
    Step& cv = p->steps[static_cast<size_t>(ci)];
    if (cv.kind != Kind::kConv1d || cv.in.size() < 2) continue;
    const SlotInfo& xs = p->slots[static_cast<size_t>(cv.in[0])];
    const SlotInfo& ws = p->slots[static_cast<size_t>(cv.in[1])];
    if (xs.dims.size() != 3 || ws.dims.size() != 3) continue;
    const int64_t batch = xs.dims[0], chan = xs.dims[1], len = xs.dims[2], k = ws.dims[2];
    const int64_t stride = cv.iv[0], padding = cv.iv[1], groups = cv.iv[2];
    if (stride != 1 || groups != chan || ws.dims[0] != chan || ws.dims[1] != 1 || k < 1 || k > 8) continue;
    const int vec = 16 / itemsize_of(xs.dtype);
    if (!is_float_dtype(xs.dtype) || chan % vec != 0 || batch > 65535) continue;
    const int t1 = producer[static_cast<size_t>(cv.in[0])];
    if (t1 < 0 || !is_time_swap(p->steps[static_cast<size_t>(t1)])) continue;
    int step = -1;
    if (!sole_reader(cv.in[0], &step) || step != ci) continue;
    std::vector<int> members = {t1, ci};
    int cur = cv.out[0];
    int64_t start = 0, out_len = len + 2 * padding - k + 1;
    if (!sole_reader(cur, &step)) continue;
    if (p->steps[static_cast<size_t>(step)].kind == Kind::kSlice && p->steps[static_cast<size_t>(step)].iv[0] == 2) {
      const Step& sl = p->steps[static_cast<size_t>(step)];
      if (sl.iv[1] < 0 || sl.iv[2] > out_len || sl.iv[2] < sl.iv[1]) continue;
      start = sl.iv[1];
      out_len = sl.iv[2] - sl.iv[1];
      members.push_back(step);
      cur = sl.out[0];
      if (!sole_reader(cur, &step)) continue;
    }
    std::vector<int> ops;
    if (p->steps[static_cast<size_t>(step)].kind == Kind::kChain) {
      const Step& ch = p->steps[static_cast<size_t>(step)];
      bool unary = ch.in.size() == 1;
      for (int a : ch.chain_arity) if (a != 1) unary = false;
      if (!unary || p->slots[static_cast<size_t>(ch.out[0])].dtype != xs.dtype) continue;
      ops = ch.chain_ops;
      members.push_back(step);
      cur = ch.out[0];
      if (!sole_reader(cur, &step)) continue;
    }
    if (!is_time_swap(p->steps[static_cast<size_t>(step)])) continue;
    const int t2 = step;
    Step& last = p->steps[static_cast<size_t>(t2)];
    if (last.write_slot != last.out[0] || out_len > 65535 * 32) continue;
    // the time-major input: a matrix of its own, or a column window of a wider rank-2 matrix
    const int a_root = root_slot(*p, p->steps[static_cast<size_t>(t1)].in[0]);
    int x_slot = a_root, slice_step = -1;
    int64_t col = 0, ld = chan;
    const int ap = writer_of(*p, a_root);
    if (ap >= 0 && p->steps[static_cast<size_t>(ap)].kind == Kind::kSlice) {
      const Step& sl = p->steps[static_cast<size_t>(ap)];
      const SlotInfo& wide = p->slots[static_cast<size_t>(sl.in[0])];
      if (wide.dims.size() == 2 && sl.iv[0] == 1 && sl.iv[1] >= 0 && sl.iv[2] - sl.iv[1] == chan &&
          wide.dims[0] == batch * len && wide.dims[1] % vec == 0 && sl.iv[1] % vec == 0 &&
          readers_of(*p, a_root).size() == 1) {
        x_slot = sl.in[0];
        col = sl.iv[1];
        ld = wide.dims[1];
        slice_step = ap;
      }
    }
    // tentatively drop the group, then check that the inputs survive until the launch
    std::vector<Kind> saved(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) saved[static_cast<size_t>(i)] = p->steps[static_cast<size_t>(i)].kind;
    for (int m : members) p->steps[static_cast<size_t>(m)].kind = Kind::kSkip;
    if (slice_step >= 0) p->steps[static_cast<size_t>(slice_step)].kind = Kind::kSkip;
    bool ok = true;
    const int bias_slot = cv.in.size() > 2 ? cv.in[2] : -1;
    for (int src : {x_slot, cv.in[1], bias_slot}) {
      if (src < 0) continue;
      if (ranges_overlap(*p, src, last.out[0])) ok = false;
      const int from = std::max(writer_of(*p, src), producer[static_cast<size_t>(root_slot(*p, src))]);
      for (int j = from + 1; j < t2 && ok; ++j) {
        const Step& t = p->steps[static_cast<size_t>(j)];
        if (!step_runs(t)) continue;
        if (t.write_slot >= 0 && ranges_overlap(*p, t.write_slot, src)) ok = false;
        if (t.kind == Kind::kAttentionFan && ranges_overlap(*p, t.fan_dest, src)) ok = false;
      }
    }
    if (!ok) {
      for (int i = 0; i < n; ++i) p->steps[static_cast<size_t>(i)].kind = saved[static_cast<size_t>(i)];
      continue;
    }
    last.kind = Kind::kDwConvTimeMajor;
    last.dw_x = x_slot; last.dw_w = cv.in[1]; last.dw_bias = bias_slot;
    last.dw_col = col; last.dw_ld = ld; last.dw_batch = batch; last.dw_len = len;
    last.dw_out_len = out_len; last.dw_channels = chan; last.dw_k = k; last.dw_shift = start - padding;
    last.chain_ops = ops;
  }
}

// The workspace the calling thread is running on (set for the duration of a run).
static thread_local fb200_plan::Workspace* t_ws = nullptr;

static int workspace_alloc(fb200_plan* p, fb200_plan::Workspace* ws) {
  if (p->arena_bytes > 0) { if (int rc = fb200_malloc(p->device, p->arena_bytes, 256, &ws->arena)) return rc; }
  for (size_t bytes : p->private_bytes) {
    void* buf = nullptr;
    if (bytes > 0) { if (int rc = fb200_malloc(p->device, bytes, 256, &buf)) return rc; }
    ws->priv.push_back(buf);
  }
  return FB200_OK;
}

static void workspace_free(fb200_plan* p, fb200_plan::Workspace* ws) {
  for (auto& e : ws->graphs) {
    if (e.exec) cudaGraphExecDestroy(e.exec);
    if (e.graph) cudaGraphDestroy(e.graph);
  }
  if (ws->arena) fb200_free(p->device, ws->arena);
  for (void* q : ws->priv) if (q) fb200_free(p->device, q);
}

// The workspace of `stream`: its own if it has one or one can still be made, else the first one
// (shared; its mutex serialises the sharers).
static int acquire_workspace(fb200_plan* p, fb200_stream stream, fb200_plan::Workspace** out) {
  std::lock_guard<std::mutex> lock(p->mu);
  for (auto& w : p->workspaces) {
    if (w->claimed && w->stream == stream) { *out = w.get(); return FB200_OK; }
  }
  for (auto& w : p->workspaces) {
    if (!w->claimed) { w->claimed = true; w->stream = stream; *out = w.get(); return FB200_OK; }
  }
  if (p->workspaces.size() < fb200_plan::kMaxWorkspaces) {
    std::unique_ptr<fb200_plan::Workspace> w(new fb200_plan::Workspace());
    if (int rc = workspace_alloc(p, w.get())) { workspace_free(p, w.get()); return rc; }
    w->claimed = true;
    w->stream = stream;
    *out = w.get();
    p->workspaces.push_back(std::move(w));
    return FB200_OK;
  }
  *out = p->workspaces[0].get();
  return FB200_OK;
}

static void* slot_ptr(fb200_plan* p, int slot, const void* const* inputs, void* const* outputs) {
  const int r = root_slot(*p, slot);
  const SlotInfo& s = p->slots[r];
  if (s.input_index >= 0) return const_cast<void*>(inputs[s.input_index]);
  if (s.output_index >= 0) return outputs[s.output_index];
  if (s.constant != nullptr) return s.constant;
  if (s.private_index >= 0) return t_ws != nullptr ? t_ws->priv[static_cast<size_t>(s.private_index)] : nullptr;
  if (s.arena_offset >= 0) return t_ws != nullptr ? static_cast<char*>(t_ws->arena) + s.arena_offset : nullptr;
  return nullptr;
}

static int run_step(fb200_plan* p, Step& s, const void* const* inputs, void* const* outputs,
                    fb200_stream stream) {
  auto in_ptr = [&](size_t i) { return slot_ptr(p, s.in[i], inputs, outputs); };
  auto in_slot = [&](size_t i) -> const SlotInfo& { return p->slots[s.in[i]]; };
  void* out = s.write_slot >= 0 ? slot_ptr(p, s.write_slot, inputs, outputs) : nullptr;
  const SlotInfo& os = p->slots[s.out.empty() ? 0 : s.out[0]];
  fb200_epilogue epi{};
  const fb200_epilogue* epi_ptr = nullptr;
  if (!s.chain_ops.empty() && (s.kind == Kind::kMatmul || s.kind == Kind::kConv2d)) {
    epi.n_ops = static_cast<int>(s.chain_ops.size());
    for (int i = 0; i < epi.n_ops; ++i) {
      epi.ops[i] = s.chain_ops[i];
      epi.modes[i] = s.epi_mode[i];
      epi.operands[i] = s.epi_operand_slot[i] >= 0 ? slot_ptr(p, s.epi_operand_slot[i], inputs, outputs) : nullptr;
    }
    epi_ptr = &epi;
  }
  switch (s.kind) {
    case Kind::kSkip:
    case Kind::kAlias:
    case Kind::kConstant:
      return FB200_OK;
    case Kind::kMatmul: {
      if (s.in.size() != 2 || in_slot(0).dims.size() != 2 || in_slot(1).dims.size() != 2) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'matmul' expects two rank-2 inputs");
      }
      const int64_t m = in_slot(0).dims[0], k = in_slot(0).dims[1], n = in_slot(1).dims[1];
      if (in_slot(1).dims[0] != k) return set_error(FB200_INVALID_ARGUMENT, "op 'matmul': contraction dims differ");
      if (s.split_slot >= 0) {
        return fb200_matmul_split(in_ptr(0), in_ptr(1), out, slot_ptr(p, s.split_slot, inputs, outputs), s.split_col,
                                  m, n, k, os.dtype, p->allow_tf32, epi_ptr, stream);
      }
      // opt_level 0 is the step-by-step path in the CPU reference's own arithmetic: strict fp32
      // products keep the CPU's order of additions at any size
      const int precision = (p->opt_level == 0 && !p->allow_tf32) ? -1 : p->allow_tf32;
      return fb200_matmul(in_ptr(0), in_ptr(1), out, m, n, k, os.dtype, precision, epi_ptr, stream);
    }
    case Kind::kConv2d: {
      if (s.in.size() < 2 || in_slot(0).dims.size() != 4 || in_slot(1).dims.size() != 4) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'conv2d' expects rank-4 x and w");
      }
      fb200_conv2d_params q{};
      q.n = in_slot(0).dims[0]; q.cin = in_slot(0).dims[1]; q.h = in_slot(0).dims[2]; q.w = in_slot(0).dims[3];
      q.cout = in_slot(1).dims[0]; q.kh = in_slot(1).dims[2]; q.kw = in_slot(1).dims[3];
      q.stride_h = s.iv[0]; q.stride_w = s.iv[1]; q.pad_h = s.iv[2]; q.pad_w = s.iv[3]; q.groups = s.iv[4];
      if (!s.pool_iv.empty()) {
        return fb200_conv2d_max_pool(in_ptr(0), in_ptr(1), s.in.size() > 2 ? in_ptr(2) : nullptr,
                                     slot_ptr(p, s.pool_mid, inputs, outputs), out, &q, s.pool_iv[0], s.pool_iv[1],
                                     s.pool_iv[2], s.pool_iv[3], s.pool_iv[4], s.pool_iv[5], os.dtype, p->allow_tf32,
                                     epi_ptr, stream);
      }
      return fb200_conv2d(in_ptr(0), in_ptr(1), s.in.size() > 2 ? in_ptr(2) : nullptr, out, &q,
                          os.dtype, p->allow_tf32, epi_ptr, stream);
    }
    case Kind::kConv1d: {
      if (s.in.size() < 2 || in_slot(0).dims.size() != 3 || in_slot(1).dims.size() != 3) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'conv1d' expects rank-3 x and w");
      }
      return fb200_conv1d(in_ptr(0), in_ptr(1), s.in.size() > 2 ? in_ptr(2) : nullptr, out,
                          in_slot(0).dims[0], in_slot(0).dims[1], in_slot(0).dims[2],
                          in_slot(1).dims[0], in_slot(1).dims[2], s.iv[0], s.iv[1], s.iv[2],
                          os.dtype, stream);
    }
    case Kind::kMaxPool: {
      if (in_slot(0).dims.size() != 4) return set_error(FB200_INVALID_ARGUMENT, "op 'max_pool2d' expects rank-4 x");
      return fb200_max_pool2d(in_ptr(0), out, in_slot(0).dims[0], in_slot(0).dims[1],
                              in_slot(0).dims[2], in_slot(0).dims[3], s.iv[0], s.iv[1], s.iv[2],
                              s.iv[3], s.iv[4], s.iv[5], os.dtype, stream);
    }
    case Kind::kAvgPool: {
      if (in_slot(0).dims.size() != 4) return set_error(FB200_INVALID_ARGUMENT, "op 'avg_pool2d' expects rank-4 x");
      return fb200_avg_pool2d(in_ptr(0), out, in_slot(0).dims[0], in_slot(0).dims[1], in_slot(0).dims[2],
                              in_slot(0).dims[3], s.iv[0], s.iv[1], s.iv[2], s.iv[3], s.iv[4], s.iv[5],
                              os.dtype, stream);
    }
    case Kind::kPoolSelect:
    case Kind::kMaxPoolGrad: {
      // the forward op's input is operand 1 (x); operand 0 is g resp. dy
      if (s.in.size() != 2 || in_slot(1).dims.size() != 4) {
        return set_error(FB200_INVALID_ARGUMENT, "op '%s' expects two operands and a rank-4 x", s.op.c_str());
      }
      const auto& xd = in_slot(1).dims;
      auto fn = s.kind == Kind::kPoolSelect ? fb200_max_pool2d_select : fb200_max_pool2d_grad;
      return fn(in_ptr(0), in_ptr(1), out, xd[0], xd[1], xd[2], xd[3], s.iv[0], s.iv[1], s.iv[2], s.iv[3],
                s.iv[4], s.iv[5], os.dtype, stream);
    }
    case Kind::kAvgPoolGrad: {
      if (os.dims.size() != 4) return set_error(FB200_INVALID_ARGUMENT, "op 'avg_pool2d_grad_internal' expects a rank-4 result");
      return fb200_avg_pool2d_grad(in_ptr(0), out, os.dims[0], os.dims[1], os.dims[2], os.dims[3], s.iv[0],
                                   s.iv[1], s.iv[2], s.iv[3], s.iv[4], s.iv[5], os.dtype, stream);
    }
    case Kind::kConvGradInput:
    case Kind::kConvGradFilter: {
      // conv2d_grad_input_internal(dy, w) -> dx;  conv2d_grad_filter_internal(x, dy) -> dw
      const bool wrt_input = s.kind == Kind::kConvGradInput;
      if (s.in.size() != 2 || os.dims.size() != 4 || in_slot(wrt_input ? 1 : 0).dims.size() != 4) {
        return set_error(FB200_INVALID_ARGUMENT, "op '%s' expects rank-4 operands", s.op.c_str());
      }
      const auto& xd = wrt_input ? os.dims : in_slot(0).dims;
      const auto& wd = wrt_input ? in_slot(1).dims : os.dims;
      fb200_conv2d_params cp{xd[0], xd[1], xd[2], xd[3], wd[0], wd[2], wd[3], s.iv[0], s.iv[1], s.iv[2], s.iv[3], s.iv[4]};
      return wrt_input ? fb200_conv2d_grad_input(in_ptr(0), in_ptr(1), out, &cp, os.dtype, stream)
                       : fb200_conv2d_grad_filter(in_ptr(0), in_ptr(1), out, &cp, os.dtype, stream);
    }
    case Kind::kMatmulGradLhs: {
      // (gy [m, n], b [k, n]) -> ga [m, k]
      if (s.in.size() != 2 || in_slot(0).dims.size() != 2 || in_slot(1).dims.size() != 2 ||
          in_slot(0).dims[1] != in_slot(1).dims[1]) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'matmul_grad_lhs_internal' expects gy [m, n] and b [k, n]");
      }
      return fb200_matmul_grad_lhs(in_ptr(0), in_ptr(1), out, in_slot(0).dims[0], in_slot(0).dims[1],
                                   in_slot(1).dims[0], os.dtype, p->allow_tf32, stream);
    }
    case Kind::kMatmulGradRhs: {
      // (a [m, k], gy [m, n]) -> gb [k, n]
      if (s.in.size() != 2 || in_slot(0).dims.size() != 2 || in_slot(1).dims.size() != 2 ||
          in_slot(0).dims[0] != in_slot(1).dims[0]) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'matmul_grad_rhs_internal' expects a [m, k] and gy [m, n]");
      }
      return fb200_matmul_grad_rhs(in_ptr(0), in_ptr(1), out, in_slot(0).dims[0], in_slot(1).dims[1],
                                   in_slot(0).dims[1], os.dtype, p->allow_tf32, stream);
    }
    case Kind::kMseLoss:
    case Kind::kMseLossGrad: {
      const size_t want = s.kind == Kind::kMseLoss ? 2 : 3;
      if (s.in.size() != want || in_slot(0).dims != in_slot(1).dims) {
        return set_error(FB200_INVALID_ARGUMENT, "op '%s' requires pred and target of the same shape", s.op.c_str());
      }
      int64_t numel = 1;
      for (int64_t d : in_slot(0).dims) numel *= d;
      return s.kind == Kind::kMseLoss
                 ? fb200_mse_loss(in_ptr(0), in_ptr(1), out, numel, os.dtype, stream)
                 : fb200_mse_loss_grad(in_ptr(0), in_ptr(1), in_ptr(2), out, numel, os.dtype, stream);
    }
    case Kind::kRfft: {
      const auto& xd = in_slot(0).dims;
      if (xd.empty() || xd.back() < 2) return set_error(FB200_INVALID_ARGUMENT, "op 'rfft' requires the last dimension (n) to be >= 2");
      int64_t rows = 1;
      for (size_t d = 0; d + 1 < xd.size(); ++d) rows *= xd[d];
      return fb200_rfft(in_ptr(0), out, rows, xd.back(), os.dtype, stream);
    }
    case Kind::kIrfft: {
      const auto& zd = in_slot(0).dims;
      const int64_t n = s.iv[0];
      if (zd.size() < 2 || zd.back() != 2 || zd[zd.size() - 2] != n / 2 + 1) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'irfft' requires z [..., n/2+1, 2] for attribute n=%lld", (long long)n);
      }
      int64_t rows = 1;
      for (size_t d = 0; d + 2 < zd.size(); ++d) rows *= zd[d];
      return fb200_irfft(in_ptr(0), out, rows, n, os.dtype, stream);
    }
    case Kind::kGather: {
      if (s.in.size() != 2 || in_slot(0).dims.size() != 2 || in_slot(1).dims.size() != 1) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'gather' expects x [N, F] and indices [K]");
      }
      return fb200_gather(in_ptr(0), in_ptr(1), out, in_slot(0).dims[0], in_slot(0).dims[1],
                          in_slot(1).dims[0], os.dtype, in_slot(1).dtype, stream);
    }
    case Kind::kScatterAdd: {
      if (s.in.size() != 2 || in_slot(0).dims.size() != 2 || in_slot(1).dims.size() != 1 || os.dims.size() != 2) {
        return set_error(FB200_INVALID_ARGUMENT, "op '%s' expects updates [K, F], indices [K] and a rank-2 result", s.op.c_str());
      }
      return fb200_scatter_add(in_ptr(0), in_ptr(1), out, in_slot(0).dims[0], in_slot(0).dims[1],
                               os.dims[0], os.dtype, in_slot(1).dtype, stream);
    }
    case Kind::kChain: {
      std::vector<const void*> ptrs(s.in.size());   // groups longer than one launch's limit are split inside
      for (size_t i = 0; i < s.in.size(); ++i) ptrs[i] = in_ptr(i);
      return fb200_fused_elementwise(ptrs.data(), static_cast<int>(s.in.size()), out, os.numel, os.dtype,
                                     s.chain_ops.data(), s.chain_arity.data(),
                                     static_cast<int>(s.chain_ops.size()), stream);
    }
    case Kind::kBiasAdd: {
      const int64_t cols = os.dims.empty() ? 1 : os.dims.back();
      return fb200_bias_add(in_ptr(0), in_ptr(1), out, cols ? os.numel / cols : 0, cols, os.dtype, stream);
    }
    case Kind::kSoftmax:
      if (os.dims.size() != 2) return set_error(FB200_INVALID_ARGUMENT, "op 'softmax' requires rank-2 x");
      return fb200_softmax(in_ptr(0), out, os.dims[0], os.dims[1], os.dtype, stream);
    case Kind::kLayerNorm:
      if (os.dims.size() != 2 || s.in.size() != 3) return set_error(FB200_INVALID_ARGUMENT, "op 'layer_norm' requires rank-2 x, gamma, beta");
      if (s.ln_res >= 0) {
        return fb200_add_layer_norm(in_ptr(0), slot_ptr(p, s.ln_res, inputs, outputs), in_ptr(1), in_ptr(2),
                                    slot_ptr(p, s.ln_sum, inputs, outputs), out, os.dims[0], os.dims[1], s.eps,
                                    os.dtype, stream);
      }
      return fb200_layer_norm(in_ptr(0), in_ptr(1), in_ptr(2), out, os.dims[0], os.dims[1], s.eps, os.dtype, stream);
    case Kind::kScan: {
      if (s.in.size() != 5 || os.dims.empty()) return set_error(FB200_INVALID_ARGUMENT, "op 'selective_scan' expects 5 inputs of rank >= 1");
      const int64_t steps = os.dims.back();
      return fb200_selective_scan(in_ptr(0), in_ptr(1), in_ptr(2), in_ptr(3), in_ptr(4), out,
                                  steps ? os.numel / steps : 0, steps, os.dtype, stream);
    }
    case Kind::kMambaScan: {
      // inputs: u, delta, A, B, C, D [, z]; u: [batch, len, dm]; A: [dm, nstate]
      if (s.in.size() < 6 || in_slot(0).dims.size() != 3 || in_slot(2).dims.size() != 2) {
        return set_error(FB200_INVALID_ARGUMENT, "op 'mamba_scan' expects u[b,l,d], delta, A[d,n], B, C, D [, z]");
      }
      return fb200_mamba_scan(in_ptr(0), in_ptr(1), in_ptr(2), in_ptr(3), in_ptr(4), in_ptr(5),
                              s.in.size() > 6 ? in_ptr(6) : nullptr, out, in_slot(0).dims[0],
                              in_slot(0).dims[1], in_slot(0).dims[2], in_slot(2).dims[1], stream);
    }
    case Kind::kTranspose:
      return fb200_transpose(in_ptr(0), out, static_cast<int>(in_slot(0).dims.size()),
                             in_slot(0).dims.data(), s.iv.data(), itemsize_of(os.dtype), stream);
    case Kind::kSlice:
      return fb200_slice(in_ptr(0), out, static_cast<int>(in_slot(0).dims.size()),
                         in_slot(0).dims.data(), s.iv[0], s.iv[1], s.iv[2], itemsize_of(os.dtype), stream);
    case Kind::kConcat: {
      std::vector<const void*> ptrs(s.in.size());
      std::vector<int64_t> sizes(s.in.size());
      const int64_t axis = s.iv[0];
      for (size_t i = 0; i < s.in.size(); ++i) {
        ptrs[i] = in_ptr(i);
        sizes[i] = in_slot(i).dims[static_cast<size_t>(axis)];
      }
      return fb200_concat(ptrs.data(), static_cast<int>(ptrs.size()), sizes.data(), out,
                          static_cast<int>(os.dims.size()), os.dims.data(), axis, itemsize_of(os.dtype), stream);
    }
    case Kind::kSum:
      return fb200_sum_axes(in_ptr(0), out, static_cast<int>(in_slot(0).dims.size()),
                            in_slot(0).dims.data(), s.iv.data(), static_cast<int>(s.iv.size()), os.dtype, stream);
    case Kind::kCopy:
      return fb200_memcpy(p->device, out, in_ptr(0), os.bytes(), FB200_D2D, stream, 0);
    case Kind::kDwConvTimeMajor: {
      const char* x = static_cast<const char*>(slot_ptr(p, s.dw_x, inputs, outputs)) + s.dw_col * itemsize_of(os.dtype);
      return fb200_dwconv1d_time_major(x, s.dw_ld, slot_ptr(p, s.dw_w, inputs, outputs),
                                       s.dw_bias >= 0 ? slot_ptr(p, s.dw_bias, inputs, outputs) : nullptr, out,
                                       s.dw_channels, s.dw_batch, s.dw_len, s.dw_out_len, s.dw_channels, s.dw_k,
                                       s.dw_shift, s.chain_ops.data(), static_cast<int>(s.chain_ops.size()),
                                       os.dtype, stream);
    }
    case Kind::kAttentionFan: {
      const SlotInfo& qb = p->slots[static_cast<size_t>(s.fan_q)];
      const SlotInfo& kb = p->slots[static_cast<size_t>(s.fan_k)];
      const SlotInfo& vb = p->slots[static_cast<size_t>(s.fan_v)];
      const SlotInfo& db = p->slots[static_cast<size_t>(s.fan_dest)];
      return fb200_attention_fan(slot_ptr(p, s.fan_q, inputs, outputs), qb.dims[0], qb.dims[1],
                                 slot_ptr(p, s.fan_k, inputs, outputs), kb.dims[0], kb.dims[1],
                                 slot_ptr(p, s.fan_v, inputs, outputs), vb.dims[0], vb.dims[1],
                                 slot_ptr(p, s.fan_dest, inputs, outputs), db.dims[1],
                                 static_cast<const fb200_attention_head*>(s.fan_table), s.fan_heads,
                                 s.fan_sq, s.fan_sk, 64, s.fan_scale, db.dtype, stream);
    }
  }
  return FB200_OK;
}

}  // namespace fb200

static int plan_create_impl(const char* plan_text, int device, int allow_tf32, int opt_level, bool dry,
                            fb200_plan** plan) {
  if (plan_text == nullptr || plan == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_create: null argument");
  *plan = nullptr;
  fb200_plan* p = new fb200_plan();
  p->dry = dry;
  p->device = device;
  p->allow_tf32 = allow_tf32;
  p->opt_level = opt_level;
  int rc = parse_plan(plan_text, p);
  for (size_t i = 0; rc == FB200_OK && i < p->steps.size(); ++i) rc = decode_step(p, p->steps[i]);
  if (rc == FB200_OK) {
    // arena bounds: every intermediate must fit inside what the planner announced
    for (const SlotInfo& s : p->slots) {
      if (s.arena_offset >= 0 && s.arena_offset + s.bytes() > p->arena_bytes && s.output_index < 0 && s.numel > 0) {
        rc = set_error(FB200_INVALID_ARGUMENT, "plan: an intermediate at offset %lld (+%zu bytes) exceeds the arena of %zu bytes",
                       (long long)s.arena_offset, s.bytes(), p->arena_bytes);
        break;
      }
    }
  }
  if (rc == FB200_OK) {
    // graph outputs are written in the caller's buffers, never in the arena
    for (int o : p->output_slots) p->slots[o].arena_offset = -1;

  }
  for (size_t i = 0; rc == FB200_OK && i < p->steps.size(); ++i) {
    if (p->steps[i].kind == Kind::kConstant) rc = materialise_constant(p, p->steps[i]);
  }
  if (rc != FB200_OK) {
    fb200_plan_destroy(p);
    return rc;
  }
  if (p->opt_level >= 1) {
    if (int rc2 = split_matmul_tails(p)) {
      fb200_plan_destroy(p);
      return rc2;
    }
  }
  optimise(p);
  if (p->opt_level >= 1) {
    alias_reshape_sources(p);
    fuse_attention_fans(p);
    fuse_time_major_convs(p);
    if (p->allow_tf32) fuse_conv_pool(p);
    fuse_add_layer_norm(p);
  }
  if (!dry) {
    // the first workspace; further streams get theirs at their first run
    std::unique_ptr<fb200_plan::Workspace> w(new fb200_plan::Workspace());
    if (int rc2 = workspace_alloc(p, w.get())) {
      workspace_free(p, w.get());
      fb200_plan_destroy(p);
      return rc2;
    }
    p->workspaces.push_back(std::move(w));
  }
  if (const char* env = getenv("FRAME_B200_GRAPH")) p->graph_enabled = p->graph_enabled.load() && atoi(env) != 0;
  p->launches = 0;
  for (const Step& s : p->steps) {
    if (s.kind != Kind::kSkip && s.kind != Kind::kAlias && s.kind != Kind::kConstant && s.kind != Kind::kCopy) ++p->launches;
    // a fused group longer than one launch's limit runs as successive launches
    if (s.kind == Kind::kChain && s.chain_ops.size() > FB200_MAX_CHAIN) {
      p->launches += static_cast<int>((s.chain_ops.size() - 1) / FB200_MAX_CHAIN);
    }
  }
  *plan = p;
  return FB200_OK;
}

extern "C" int fb200_plan_create(const char* plan_text, int device, int allow_tf32, int opt_level,
                                 fb200_plan** plan) {
  return plan_create_impl(plan_text, device, allow_tf32, opt_level, false, plan);
}

extern "C" int fb200_plan_describe(const char* plan_text, int allow_tf32, int opt_level, fb200_plan** plan) {
  return plan_create_impl(plan_text, 0, allow_tf32, opt_level, true, plan);
}

extern "C" int fb200_plan_destroy(fb200_plan* p) {
  if (p == nullptr) return FB200_OK;
  for (auto& w : p->workspaces) workspace_free(p, w.get());
  for (int b = 0; b < 2; ++b) {
    if (p->ev_in[b]) cudaEventDestroy(p->ev_in[b]);
    if (p->ev_run[b]) cudaEventDestroy(p->ev_run[b]);
    if (p->ev_out[b]) cudaEventDestroy(p->ev_out[b]);
  }
  if (p->s_h2d) cudaStreamDestroy(p->s_h2d);
  if (p->s_d2h) cudaStreamDestroy(p->s_d2h);
  for (void* q : p->stage_in2) fb200_free(p->device, q);
  for (void* q : p->stage_out2) fb200_free(p->device, q);
  for (void* q : p->owned) fb200_free(p->device, q);
  for (void* q : p->stage_in) fb200_free(p->device, q);
  for (void* q : p->stage_out) fb200_free(p->device, q);
  delete p;
  return FB200_OK;
}

extern "C" int fb200_plan_num_inputs(const fb200_plan* p) { return p ? static_cast<int>(p->input_slots.size()) : 0; }
extern "C" int fb200_plan_num_outputs(const fb200_plan* p) { return p ? static_cast<int>(p->output_slots.size()) : 0; }
extern "C" size_t fb200_plan_arena_bytes(const fb200_plan* p) { return p ? p->arena_bytes : 0; }
extern "C" size_t fb200_plan_private_bytes(const fb200_plan* p) {
  size_t total = 0;
  if (p) for (size_t b : p->private_bytes) total += b;
  return total;
}
extern "C" int fb200_plan_launches_per_run(const fb200_plan* p) { return p ? p->launches : 0; }

extern "C" int fb200_plan_io_spec(const fb200_plan* p, int is_output, int index, int* dtype,
                                  int* rank, int64_t* dims) {
  if (p == nullptr || dtype == nullptr || rank == nullptr || dims == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_io_spec: null argument");
  const std::vector<int>& v = is_output ? p->output_slots : p->input_slots;
  if (index < 0 || static_cast<size_t>(index) >= v.size()) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_io_spec: index %d out of range", index);
  const SlotInfo& s = p->slots[v[static_cast<size_t>(index)]];
  *dtype = s.dtype;
  *rank = static_cast<int>(s.dims.size());
  for (size_t i = 0; i < s.dims.size(); ++i) dims[i] = s.dims[i];
  return FB200_OK;
}

extern "C" int fb200_plan_run(fb200_plan* p, const void* const* inputs, void* const* outputs,
                              fb200_stream stream) {
  if (p == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run: null plan");
  if (p->dry) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run: this plan was made by fb200_plan_describe and cannot run");
  if ((!p->input_slots.empty() && inputs == nullptr) || (!p->output_slots.empty() && outputs == nullptr)) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run: null input/output table");
  }
  for (size_t i = 0; i < p->input_slots.size(); ++i) {
    if (inputs[i] == nullptr && p->slots[p->input_slots[i]].numel > 0) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run: input %zu is null", i);
  }
  for (size_t i = 0; i < p->output_slots.size(); ++i) {
    if (outputs[i] == nullptr && p->slots[p->output_slots[i]].numel > 0) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run: output %zu is null", i);
  }
  FB200_CUDA_OK(cudaSetDevice(p->device));
  fb200_plan::Workspace* ws = nullptr;
  if (int rc = acquire_workspace(p, stream, &ws)) return rc;
  std::lock_guard<std::mutex> lock(ws->run_mu);   // callers that share a workspace take turns
  struct Scope { Scope(fb200_plan::Workspace* w) { t_ws = w; } ~Scope() { t_ws = nullptr; } } scope(ws);
  auto run_eager = [&]() -> int {
    for (Step& s : p->steps) {
      if (int rc = run_step(p, s, inputs, outputs, stream)) {
        // keep the kernel's message, prefix the op like CudaExecutable::run does
        std::string msg = fb200_last_error();
        return set_error(rc, "plan run: op '%s' kernel failed: %s", s.op.c_str(), msg.c_str());
      }
    }
    return FB200_OK;
  };
  bool done = false;
  if (p->graph_enabled && stream != nullptr && p->launches >= 2) {
    std::vector<const void*> key;
    for (size_t i = 0; i < p->input_slots.size(); ++i) key.push_back(inputs[i]);
    for (size_t i = 0; i < p->output_slots.size(); ++i) key.push_back(outputs[i]);
    key.push_back(stream);
    fb200_plan::GraphEntry* ge = nullptr;
    for (auto& e : ws->graphs) if (e.key == key) ge = &e;
    if (ge == nullptr) {
      if (ws->graphs.size() < 4) {
        ws->graphs.emplace_back();
        ge = &ws->graphs.back();
      } else {   // replace the entry used longest ago
        ge = &ws->graphs[0];
        for (auto& e : ws->graphs) if (e.last_used < ge->last_used) ge = &e;
        if (ge->exec) cudaGraphExecDestroy(ge->exec);
        if (ge->graph) cudaGraphDestroy(ge->graph);
        *ge = fb200_plan::GraphEntry();
      }
      ge->key = key;
    }
    ge->last_used = ++ws->graph_clock;
    if (ge->exec != nullptr) {
      FB200_CUDA_OK(cudaGraphLaunch(ge->exec, as_stream(stream)));
      g_launch_count.fetch_add(p->launches, std::memory_order_relaxed);
      done = true;
    } else if (ge->runs >= 1) {
      const int64_t count_before = g_launch_count.load(std::memory_order_relaxed);
      if (cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeRelaxed) == cudaSuccess) {
        const int rc = run_eager();
        cudaGraph_t captured = nullptr;
        const cudaError_t end = cudaStreamEndCapture(as_stream(stream), &captured);
        if (rc == FB200_OK && end == cudaSuccess && captured != nullptr &&
            cudaGraphInstantiate(&ge->exec, captured, 0) == cudaSuccess) {
          ge->graph = captured;
          g_launch_count.store(count_before, std::memory_order_relaxed);  // capture launched nothing
          FB200_CUDA_OK(cudaGraphLaunch(ge->exec, as_stream(stream)));
          g_launch_count.fetch_add(p->launches, std::memory_order_relaxed);
          done = true;
        } else {
          if (captured) cudaGraphDestroy(captured);
          ge->exec = nullptr;
          p->graph_enabled = false;  // this plan stays on eager launches
          (void)cudaGetLastError();
          g_launch_count.store(count_before, std::memory_order_relaxed);
          if (rc != FB200_OK) return rc;
        }
      } else {
        (void)cudaGetLastError();
        p->graph_enabled = false;
      }
    }
    ++ge->runs;
  }
  if (!done) {
    if (int rc = run_eager()) return rc;
  }
  // Outputs that are not produced by a step writing into the caller's buffer: graph inputs
  // passed through, constants, repeated outputs.
  for (size_t i = 0; i < p->output_slots.size(); ++i) {
    const int slot = p->output_slots[i];
    const int r = root_slot(*p, slot);
    const SlotInfo& s = p->slots[r];
    const void* src = nullptr;
    if (s.input_index >= 0) src = inputs[s.input_index];
    else if (s.constant != nullptr) src = s.constant;
    else if (s.output_index >= 0 && static_cast<size_t>(s.output_index) != i) src = outputs[s.output_index];
    if (src != nullptr && src != outputs[i]) {
      if (int rc = fb200_memcpy(p->device, outputs[i], src, p->slots[slot].bytes(), FB200_D2D, stream, 0)) return rc;
    }
  }
  return FB200_OK;
}

extern "C" int fb200_plan_run_host(fb200_plan* p, const void* const* host_inputs,
                                   void* const* host_outputs, fb200_stream stream) {
  if (p == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run_host: null plan");
  if (p->dry) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run_host: this plan was made by fb200_plan_describe and cannot run");
  {
    std::lock_guard<std::mutex> lock(p->mu);
    if (p->stage_in.empty() && p->stage_out.empty()) {
      for (int slot : p->input_slots) {
        void* d = nullptr;
        if (p->slots[slot].bytes() > 0) { if (int rc = fb200_malloc(p->device, p->slots[slot].bytes(), 256, &d)) return rc; }
        p->stage_in.push_back(d);
      }
      for (int slot : p->output_slots) {
        void* d = nullptr;
        if (p->slots[slot].bytes() > 0) { if (int rc = fb200_malloc(p->device, p->slots[slot].bytes(), 256, &d)) return rc; }
        p->stage_out.push_back(d);
      }
    }
  }
  std::vector<const void*> in(p->stage_in.begin(), p->stage_in.end());
  for (size_t i = 0; i < p->input_slots.size(); ++i) {
    if (i < p->resident.size() && p->resident[i] != nullptr) { in[i] = p->resident[i]; continue; }
    if (int rc = fb200_memcpy(p->device, p->stage_in[i], host_inputs[i], p->slots[p->input_slots[i]].bytes(), FB200_H2D, stream, 0)) return rc;
  }
  if (int rc = fb200_plan_run(p, in.data(), p->stage_out.data(), stream)) return rc;
  for (size_t i = 0; i < p->output_slots.size(); ++i) {
    if (int rc = fb200_memcpy(p->device, host_outputs[i], p->stage_out[i], p->slots[p->output_slots[i]].bytes(), FB200_D2H, stream, 0)) return rc;
  }
  return fb200_stream_synchronize(p->device, stream);
}

// Per-step device times of one eager run (CUDA events on `stream` around every step), for
// harness-side roofline accounting.  Steps that launch nothing report 0.  Synchronises the stream.
extern "C" int fb200_plan_profile(fb200_plan* p, const void* const* inputs, void* const* outputs,
                                  fb200_stream stream, float* step_ms, int cap, int* n_steps) {
  if (p == nullptr || step_ms == nullptr || n_steps == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_profile: null argument");
  }
  if (p->dry) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_profile: this plan was made by fb200_plan_describe and cannot run");
  const int n = static_cast<int>(p->steps.size());
  *n_steps = n;
  if (cap < n) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_profile: room for %d steps, plan has %d", cap, n);
  FB200_CUDA_OK(cudaSetDevice(p->device));
  fb200_plan::Workspace* ws = nullptr;
  if (int rc0 = acquire_workspace(p, stream, &ws)) return rc0;
  std::lock_guard<std::mutex> lock(ws->run_mu);
  struct Scope { Scope(fb200_plan::Workspace* w) { t_ws = w; } ~Scope() { t_ws = nullptr; } } scope(ws);
  std::vector<cudaEvent_t> ev(static_cast<size_t>(n) + 1);
  for (auto& e : ev) FB200_CUDA_OK(cudaEventCreate(&e));
  int rc = FB200_OK;
  FB200_CUDA_OK(cudaEventRecord(ev[0], as_stream(stream)));
  for (int i = 0; i < n && rc == FB200_OK; ++i) {
    rc = run_step(p, p->steps[i], inputs, outputs, stream);
    FB200_CUDA_OK(cudaEventRecord(ev[i + 1], as_stream(stream)));
  }
  FB200_CUDA_OK(cudaStreamSynchronize(as_stream(stream)));
  for (int i = 0; i < n && rc == FB200_OK; ++i) {
    const Kind k = p->steps[i].kind;
    step_ms[i] = 0.0f;
    if (k != Kind::kSkip && k != Kind::kAlias && k != Kind::kConstant) {
      FB200_CUDA_OK(cudaEventElapsedTime(&step_ms[i], ev[i], ev[i + 1]));
    }
  }
  for (auto& e : ev) cudaEventDestroy(e);
  return rc;
}

// Pipelined variant of fb200_plan_run_host: the call returns once its work is queued.  Run k copies
// its inputs on a copy-in stream, runs on `stream`, and copies its outputs on a copy-out stream, so
// H2D(k+1), run(k) and D2H(k-1) overlap; two sets of staging buffers alternate.  The host input
// buffers of run k may be rewritten, and its host outputs read, after fb200_plan_host_sync (or once
// two further runs have been queued, which wait for the staging set to drain).  Pinned host memory
// makes the copies asynchronous; pageable memory still works but serialises.
extern "C" int fb200_plan_run_host_async(fb200_plan* p, const void* const* host_inputs,
                                         void* const* host_outputs, fb200_stream stream) {
  if (p == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run_host_async: null plan");
  if (p->dry) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_run_host_async: this plan was made by fb200_plan_describe and cannot run");
  FB200_CUDA_OK(cudaSetDevice(p->device));
  int b = 0;
  uint64_t k = 0;
  {
    std::lock_guard<std::mutex> lock(p->mu);
    if (p->s_h2d == nullptr) {
      FB200_CUDA_OK(cudaStreamCreateWithFlags(&p->s_h2d, cudaStreamNonBlocking));
      FB200_CUDA_OK(cudaStreamCreateWithFlags(&p->s_d2h, cudaStreamNonBlocking));
      for (int i = 0; i < 2; ++i) {
        FB200_CUDA_OK(cudaEventCreateWithFlags(&p->ev_in[i], cudaEventDisableTiming));
        FB200_CUDA_OK(cudaEventCreateWithFlags(&p->ev_run[i], cudaEventDisableTiming));
        FB200_CUDA_OK(cudaEventCreateWithFlags(&p->ev_out[i], cudaEventDisableTiming));
      }
      auto fill = [&](std::vector<void*>& v, const std::vector<int>& slots) -> int {
        for (int slot : slots) {
          void* d = nullptr;
          if (p->slots[slot].bytes() > 0) { if (int rc = fb200_malloc(p->device, p->slots[slot].bytes(), 256, &d)) return rc; }
          v.push_back(d);
        }
        return FB200_OK;
      };
      if (p->stage_in.empty() && p->stage_out.empty()) {
        if (int rc = fill(p->stage_in, p->input_slots)) return rc;
        if (int rc = fill(p->stage_out, p->output_slots)) return rc;
      }
      if (int rc = fill(p->stage_in2, p->input_slots)) return rc;
      if (int rc = fill(p->stage_out2, p->output_slots)) return rc;
    }
    k = p->host_runs++;
    b = static_cast<int>(k & 1);
  }
  std::vector<void*>& stage = b == 0 ? p->stage_in : p->stage_in2;
  std::vector<const void*> in(stage.begin(), stage.end());
  std::vector<void*>& out = b == 0 ? p->stage_out : p->stage_out2;
  cudaStream_t cs = as_stream(stream);
  // the staging inputs of this set were last read by run k-2
  if (k >= 2) FB200_CUDA_OK(cudaStreamWaitEvent(p->s_h2d, p->ev_run[b], 0));
  for (size_t i = 0; i < p->input_slots.size(); ++i) {
    const size_t bytes = p->slots[p->input_slots[i]].bytes();
    if (i < p->resident.size() && p->resident[i] != nullptr) { in[i] = p->resident[i]; continue; }
    if (bytes > 0) FB200_CUDA_OK(cudaMemcpyAsync(stage[i], host_inputs[i], bytes, cudaMemcpyHostToDevice, p->s_h2d));
  }
  FB200_CUDA_OK(cudaEventRecord(p->ev_in[b], p->s_h2d));
  FB200_CUDA_OK(cudaStreamWaitEvent(cs, p->ev_in[b], 0));
  // the staging outputs of this set were last copied out by run k-2
  if (k >= 2) FB200_CUDA_OK(cudaStreamWaitEvent(cs, p->ev_out[b], 0));
  if (int rc = fb200_plan_run(p, in.data(), out.data(), stream)) return rc;
  FB200_CUDA_OK(cudaEventRecord(p->ev_run[b], cs));
  FB200_CUDA_OK(cudaStreamWaitEvent(p->s_d2h, p->ev_run[b], 0));
  for (size_t i = 0; i < p->output_slots.size(); ++i) {
    const size_t bytes = p->slots[p->output_slots[i]].bytes();
    if (bytes > 0) FB200_CUDA_OK(cudaMemcpyAsync(host_outputs[i], out[i], bytes, cudaMemcpyDeviceToHost, p->s_d2h));
  }
  FB200_CUDA_OK(cudaEventRecord(p->ev_out[b], p->s_d2h));
  return FB200_OK;
}

// Marks graph input `index` as a parameter that already lives on the device (weights, and the
// reference's full-shape biases: a Frame module keeps them on the graph's device between runs).
// fb200_plan_run_host and fb200_plan_run_host_async then read it in place and ignore the matching
// host pointer; a null `device_ptr` restores the copy.  The caller keeps the buffer alive and
// unchanged while runs are in flight.
extern "C" int fb200_plan_bind_resident(fb200_plan* p, int index, const void* device_ptr) {
  if (p == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_bind_resident: null plan");
  if (index < 0 || static_cast<size_t>(index) >= p->input_slots.size()) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_bind_resident: input %d out of range", index);
  }
  std::lock_guard<std::mutex> lock(p->mu);
  if (p->resident.size() < p->input_slots.size()) p->resident.resize(p->input_slots.size(), nullptr);
  p->resident[static_cast<size_t>(index)] = device_ptr;
  return FB200_OK;
}

// Waits until every pipelined run queued so far has delivered its outputs to the host.
extern "C" int fb200_plan_host_sync(fb200_plan* p) {
  if (p == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_plan_host_sync: null plan");
  if (p->s_d2h == nullptr) return FB200_OK;
  FB200_CUDA_OK(cudaSetDevice(p->device));
  FB200_CUDA_OK(cudaStreamSynchronize(p->s_d2h));
  return FB200_OK;
}

// Op name of step `index`; a contraction that absorbed a following group reports
// "matmul+epilogue" / "conv2d+epilogue" (+ "+max_pool2d" when the pool behind it was folded in), a
// step folded away reports "(absorbed)" or "(alias)".
extern "C" const char* fb200_plan_step_op(const fb200_plan* p, int index) {
  static thread_local std::string name;
  if (p == nullptr || index < 0 || static_cast<size_t>(index) >= p->steps.size()) return "";
  const Step& s = p->steps[static_cast<size_t>(index)];
  if (s.kind == Kind::kSkip) name = "(absorbed)";
  else if (s.kind == Kind::kAttentionFan) name = "attention_fan";
  else if (s.kind == Kind::kDwConvTimeMajor) name = "dwconv1d_time_major";
  else if (s.kind == Kind::kAlias) name = "(alias)";
  else if (s.kind == Kind::kLayerNorm && s.ln_res >= 0) name = "add+layer_norm";
  else if (s.kind == Kind::kConv2d && !s.pool_iv.empty()) name = s.chain_ops.empty() ? "conv2d+max_pool2d" : "conv2d+epilogue+max_pool2d";
  else if ((s.kind == Kind::kMatmul || s.kind == Kind::kConv2d) && !s.chain_ops.empty()) name = s.op + "+epilogue";
  else name = s.op;
  return name.c_str();
}

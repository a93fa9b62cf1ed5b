// Tuning-spec persistence: the on-disk contract of TF_MONONN_DUMP_DIR and
// TF_MONONN_EXISTING_TUNING_SPEC_DIR.
//
// The reference stores a GraphSpecification protobuf as proto3 JSON with original field
// names (mononn_engine/helpers/protobuf.cc:32-46) under
//   <dump_dir>/<cluster_N>/{<grid>_1_1__<block>_1_1.json, best_tuning_spec.json,
//                           tuning_log.log, performance_report.csv}
// (mononn_engine/module/mononn_module_tuner.cc:457-466,509-520,584-603,422-448).
// The same layout and field names are kept; the per-GEMM `cutlass_config` is replaced by
// an `sm100_config` (UMMA tile, K split, pipeline slots) and unknown fields are ignored
// on load, so a spec written by the reference parses (its tiles are simply not used).
#include <sys/stat.h>
#include <sys/types.h>

#include <cctype>
#include <cstdlib>
#include <fstream>
#include <sstream>

#include "json.h"
#include "module.h"

namespace mononn {

bool env_truthy(const char* name) {
  // mononn_engine/helpers/env_variable.cc:20-26
  const char* v = std::getenv(name);
  if (!v) return false;
  const std::string s(v);
  return s == "True" || s == "true" || s == "1";
}

// "cluster_<digits>" prefix of the module name (helpers/string_helpers.cc:34-46). A name of
// another form is kept whole (sanitised) instead of aborting the process.
std::string cluster_dir_name(const std::string& name) {
  if (name.compare(0, 8, "cluster_") == 0) {
    size_t pos = 8;
    while (pos < name.size() && std::isdigit(static_cast<unsigned char>(name[pos]))) ++pos;
    if (pos > 8) return name.substr(0, pos);
  }
  std::string out;
  for (char c : name) out.push_back(std::isalnum(static_cast<unsigned char>(c)) ? c : '_');
  return out.empty() ? std::string("cluster_0") : out;
}

static Json dim3_json(uint32_t x) {
  Json d = Json::object();
  d.set("x", Json::number(x));
  d.set("y", Json::number(1));
  d.set("z", Json::number(1));
  return d;
}

std::string spec_to_json(const Plan& plan, uint32_t sm_count) {
  Json root = Json::object();
  Json ctx = Json::object();
  Json rt = Json::object();
  rt.set("grid_dim", dim3_json(plan.grid));
  rt.set("block_dim", dim3_json(plan.block));
  rt.set("cluster_dim", dim3_json(plan.cluster));
  rt.set("smem_size", Json::number(plan.smem_bytes));
  rt.set("stream", Json::string("stream"));
  ctx.set("cuda_runtime_context", rt);
  Json dev = Json::object();
  dev.set("device_count", Json::number(1));
  dev.set("sm_count", Json::number(sm_count));
  dev.set("static_smem_size", Json::number(0));
  dev.set("max_configurable_smem_size", Json::number(232448));
  dev.set("cuda_arch", Json::string("1000"));
  dev.set("register_per_block", Json::number(65536));
  dev.set("warp_size", Json::number(32));
  dev.set("reserved_smem_per_block", Json::number(1024));
  ctx.set("cuda_device_context", dev);
  root.set("cuda_context", ctx);
  root.set("hlo_module_name", Json::string(plan.module_name));
  // "auto": Q/K/V projections are computed inside the attention items when the attention stage
  // cannot fill the GPU (batches*heads <= CTAs, sequence <= 128); "off"; "on": whenever legal
  root.set("qkv_fusion", Json::string(plan.spec.qkv_fusion == 1 ? "off" : plan.spec.qkv_fusion == 2 ? "on" : "auto"));
  root.set("row_fusion", Json::string(plan.spec.row_fusion == 1 ? "off" : "on"));
  root.set("l2_hints", Json::string(plan.spec.l2_hints == 1 ? "off" : "on"));
  root.set("row_split", Json::string(plan.spec.row_split == 1 ? "off" : "on"));
  root.set("out_fusion", Json::string(plan.spec.out_fusion == 2 ? "on" : (plan.spec.out_fusion == 3 ? "fused_qkv" : "off")));
  root.set("chain_fusion", Json::string(plan.spec.chain_fusion == 2 ? "on" : "off"));
  root.set("barrier_arrive", Json::string(plan.spec.barrier_arrive == 1 || plan.cluster > 1
                                              ? "cta"
                                              : (plan.spec.barrier_arrive == 2 ? "warp" : "last")));
  root.set("cluster_elewise_spec", Json::object());
  root.set("cluster_reduce_spec", Json::object());
  Json gemms = Json::object();
  for (const PlanOp& op : plan.ops) {
    if (op.d.kind != OP_GEMM) continue;
    Json cfg = Json::object();
    cfg.set("mma_m", Json::number(128));
    cfg.set("mma_n", Json::number(op.d.n_tile));
    cfg.set("mma_k", Json::number(16));
    cfg.set("k_split", Json::number(op.d.k_split));
    cfg.set("k_block", Json::number(64));
    cfg.set("a_stages", Json::number(kASlots));
    cfg.set("b_stages", Json::number(kBSlots));
    cfg.set("cluster_x", Json::number(plan.cluster));
    cfg.set("cluster_y", Json::number(1));
    cfg.set("cta_group", Json::number(1));
    Json fus = Json::array();
    if (op.d.flags & F_BIAS) fus.arr.push_back(Json::string("bias"));
    if (op.d.act == ACT_GELU_ERF) fus.arr.push_back(Json::string("gelu_erf"));
    if (op.d.act == ACT_RELU) fus.arr.push_back(Json::string("relu"));
    if (op.d.act == ACT_QUICK_GELU) fus.arr.push_back(Json::string("quick_gelu"));
    if (op.d.act == ACT_GELU_TANH) fus.arr.push_back(Json::string("gelu_tanh"));
    if (op.d.flags & F_RESID) fus.arr.push_back(Json::string("residual"));
    cfg.set("epilogue_fusion", fus);
    Json problem = Json::object();
    problem.set("m", Json::number(op.d.M));
    problem.set("n", Json::number(op.d.N));
    problem.set("k", Json::number(op.d.K));
    Json node = Json::object();
    node.set("sm100_config", cfg);
    node.set("problem", problem);
    gemms.set(op.name, node);
  }
  root.set("gemm_spec_list", gemms);
  root.set("conv_spec_list", Json::object());
  Json allow = Json::array(), reject = Json::array();
  for (const std::string& s : plan.spec.allow_list) allow.arr.push_back(Json::string(s));
  for (const std::string& s : plan.spec.reject_list) reject.arr.push_back(Json::string(s));
  root.set("codegen_allow_list", allow);
  root.set("codegen_reject_list", reject);
  return root.dump(2);
}

static const char* kind_name(uint32_t k) {
  switch (k) {
    case OP_GEMM: return "gemm";
    case OP_ATTENTION: return "attention";
    case OP_LAYERNORM: return "layernorm";
    case OP_EMBED: return "embed";
    case OP_ASSEMBLE: return "assemble";
    case OP_PATCHIFY: return "patchify";
    case OP_ARGMAX: return "argmax";
    case OP_ROWSEL: return "rowsel";
    case OP_PAIRDOT: return "pairdot";
    default: return "none";
  }
}
static const char* tkind_name(TKind k) {
  switch (k) {
    case TKind::ActF16: return "act_f16";
    case TKind::ActF16T: return "act_f16_t";
    case TKind::AccF32: return "acc_f32";
    case TKind::VecF32: return "vec_f32";
    case TKind::Const: return "const";
    default: return "arg";
  }
}
static Json ref_json(const BufRef& r) {
  Json j = Json::object();
  j.set("space", Json::string(r.space == SPACE_ARG ? "arg" : r.space == SPACE_CONST ? "const"
                              : r.space == SPACE_SCRATCH ? "scratch" : "none"));
  j.set("index", Json::number(r.index));
  j.set("offset", Json::number(static_cast<double>(r.offset)));
  return j;
}

// Human/test-readable description of a lowered plan: stages, operators with their tiles,
// tensor placements, constant bindings. Stands in for the `<context>_src/` dump of the
// reference (mononn_engine/module/mononn_module_tuner.cc:560-575): there is no generated
// source to dump, the table is the artefact.
std::string plan_to_json(const Plan& plan) {
  Json root = Json::object();
  root.set("module", Json::string(plan.module_name));
  root.set("grid", Json::number(plan.grid));
  root.set("block", Json::number(plan.block));
  root.set("cluster", Json::number(plan.cluster));
  root.set("smem_bytes", Json::number(plan.smem_bytes));
  root.set("temp_bytes", Json::number(static_cast<double>(plan.temp_bytes)));
  root.set("scratch_bytes", Json::number(static_cast<double>(plan.scratch_bytes)));
  root.set("const_bytes", Json::number(static_cast<double>(plan.const_bytes)));
  root.set("algorithmic_bytes", Json::number(plan.algorithmic_bytes));
  root.set("algorithmic_flops", Json::number(plan.algorithmic_flops));
  Json stages = Json::array();
  for (size_t s = 0; s < plan.stages.size(); ++s) {
    Json st = Json::object();
    st.set("name", Json::string(plan.stage_names[s]));
    st.set("n_items", Json::number(plan.stages[s].n_items));
    Json ops = Json::array();
    for (uint32_t i = 0; i < plan.stages[s].op_count; ++i) {
      const PlanOp& op = plan.ops[plan.stages[s].op_begin + i];
      Json o = Json::object();
      o.set("name", Json::string(op.name));
      o.set("kind", Json::string(kind_name(op.d.kind)));
      o.set("n_items", Json::number(op.d.n_items));
      o.set("flags", Json::number(op.d.flags));
      o.set("act", Json::number(op.d.act));
      if (op.flag_index >= 0) {
        o.set("flag", Json::number(op.flag_index));
        o.set("waits", Json::number(op.waits ? 1 : 0));
        o.set("flag_target", Json::number(op.d.flag_target));
      }
      if (op.wflag_index >= 0) {
        o.set("wait_flag", Json::number(op.wflag_index));
        o.set("wait_target", Json::number(op.d.wait_target));
      }
      if (op.d.kind == OP_GEMM) {
        o.set("M", Json::number(op.d.M));
        o.set("N", Json::number(op.d.N));
        o.set("K", Json::number(op.d.K));
        o.set("n_tile", Json::number(op.d.n_tile));
        o.set("k_split", Json::number(op.d.k_split));
        o.set("kb_per_split", Json::number(op.d.kb_per_split));
        o.set("kb_per_bslot", Json::number(op.d.kb_per_bslot));
        o.set("out_mode", Json::number(op.d.out_mode));
      }
      if (op.d.kind == OP_PATCHIFY) {
        o.set("rows", Json::number(op.d.rows));
        o.set("cols", Json::number(op.d.cols));
        o.set("window_elements", Json::number(op.d.K));
        o.set("window", Json::number(op.d.head_dim));
        o.set("stride", Json::number(op.d.M));
        o.set("pad", Json::number(op.d.rows_per_batch));
      }
      Json ptrs = Json::array();
      for (int k = 0; k < 8; ++k) ptrs.arr.push_back(ref_json(op.p[k]));
      o.set("p", ptrs);
      Json aux = Json::array();
      for (int k = 0; k < 4; ++k) aux.arr.push_back(ref_json(op.q[k]));
      o.set("q", aux);
      ops.arr.push_back(o);
    }
    st.set("ops", ops);
    stages.arr.push_back(st);
  }
  root.set("stages", stages);
  Json tensors = Json::array();
  for (const TensorPlacement& t : plan.tensors) {
    Json j = Json::object();
    j.set("name", Json::string(t.name));
    j.set("kind", Json::string(tkind_name(t.kind)));
    j.set("at", ref_json(t.at));
    j.set("rows", Json::number(t.rows));
    j.set("cols", Json::number(t.cols));
    j.set("ld", Json::number(t.ld));
    j.set("batches", Json::number(t.batches));
    j.set("seq", Json::number(t.seq));
    j.set("def_stage", Json::number(t.def_stage));
    j.set("last_stage", Json::number(t.last_stage));
    tensors.arr.push_back(j);
  }
  root.set("tensors", tensors);
  Json args = Json::array();
  for (const ArgDesc& a : plan.args) {
    Json j = Json::object();
    j.set("name", Json::string(a.name));
    j.set("bytes", Json::number(static_cast<double>(a.bytes)));
    j.set("kind", Json::number(a.kind));
    j.set("param_number", Json::number(a.param_number));
    args.arr.push_back(j);
  }
  root.set("args", args);
  Json consts = Json::array();
  for (const ConstBinding& b : plan.consts) {
    Json j = Json::object();
    j.set("name", Json::string(b.const_name));
    j.set("kind", Json::string(b.kind == ConstBinding::RAW ? "raw" : "pack_b"));
    j.set("offset", Json::number(static_cast<double>(b.offset)));
    j.set("bytes", Json::number(static_cast<double>(b.bytes)));
    j.set("src_bytes", Json::number(static_cast<double>(b.src_bytes)));
    if (b.kind == ConstBinding::PACK_B) {
      j.set("K", Json::number(b.K));
      j.set("N", Json::number(b.N));
      j.set("n_tile", Json::number(b.n_tile));
    }
    consts.arr.push_back(j);
  }
  root.set("constants", consts);
  Json tm = Json::array();
  for (const TmapSpec& t : plan.tmaps) {
    Json j = Json::object();
    j.set("base", ref_json(t.base));
    j.set("dim0", Json::number(static_cast<double>(t.dim0)));
    j.set("dim1", Json::number(static_cast<double>(t.dim1)));
    j.set("stride1_bytes", Json::number(static_cast<double>(t.stride1_bytes)));
    j.set("box0", Json::number(t.box0));
    j.set("box1", Json::number(t.box1));
    tm.arr.push_back(j);
  }
  root.set("tensor_maps", tm);
  return root.dump(1);
}

int spec_from_json(const std::string& text, TuningSpec* spec, std::string* err) {
  Json root;
  if (!Json::parse(text, &root, err)) return MONONN_ERR_PARSE;
  if (!root.is_object()) {
    if (err) *err = "tuning spec must be a JSON object";
    return MONONN_ERR_PARSE;
  }
  *spec = TuningSpec();
  if (const Json* ctx = root.find("cuda_context"))
    if (const Json* rt = ctx->find("cuda_runtime_context")) {
      if (const Json* g = rt->find("grid_dim")) spec->grid = static_cast<uint32_t>(g->get_number("x", 0));
      if (const Json* cl = rt->find("cluster_dim")) spec->cluster = static_cast<uint32_t>(cl->get_number("x", 1));
      if (const Json* b = rt->find("block_dim")) spec->block = static_cast<uint32_t>(b->get_number("x", kThreads));
    }
  if (const Json* cf = root.find("chain_fusion"))
    if (cf->type == Json::String) spec->chain_fusion = cf->str == "on" ? 2u : (cf->str == "off" ? 1u : 0u);
  if (const Json* of = root.find("out_fusion"))
    if (of->type == Json::String) spec->out_fusion = of->str == "on" ? 2u : (of->str == "fused_qkv" ? 3u : (of->str == "off" ? 1u : 0u));
  if (const Json* rs = root.find("row_split"))
    if (rs->type == Json::String) spec->row_split = rs->str == "off" ? 1u : 0u;
  if (const Json* ba = root.find("barrier_arrive"))
    if (ba->type == Json::String) spec->barrier_arrive = ba->str == "cta" ? 1u : (ba->str == "warp" ? 2u : 3u);
  if (const Json* lh = root.find("l2_hints"))
    if (lh->type == Json::String) spec->l2_hints = lh->str == "on" ? 2u : (lh->str == "off" ? 1u : 0u);
  if (const Json* rf = root.find("row_fusion"))
    if (rf->type == Json::String) spec->row_fusion = rf->str == "off" ? 1u : (rf->str == "on" ? 2u : 0u);
  if (const Json* qf = root.find("qkv_fusion"))
    if (qf->type == Json::String) spec->qkv_fusion = qf->str == "off" ? 1u : qf->str == "on" ? 2u : 0u;
  if (const Json* gl = root.find("gemm_spec_list")) {
    if (!gl->is_object()) {
      if (err) *err = "gemm_spec_list must be an object";
      return MONONN_ERR_PARSE;
    }
    for (const auto& kv : gl->obj) {
      const Json* cfg = kv.second.find("sm100_config");
      if (!cfg) continue;  // a reference spec with cutlass_config only: ignored
      GemmTileSpec t;
      t.n_tile = static_cast<uint32_t>(cfg->get_number("mma_n", 0));
      t.k_split = static_cast<uint32_t>(cfg->get_number("k_split", 0));
      spec->gemm[kv.first] = t;
    }
  }
  for (const char* key : {"codegen_allow_list", "codegen_reject_list"})
    if (const Json* l = root.find(key))
      if (l->is_array())
        for (const Json& e : l->arr)
          if (e.type == Json::String)
            (std::string(key) == "codegen_allow_list" ? spec->allow_list : spec->reject_list)
                .push_back(e.str);
  return MONONN_OK;
}

static bool read_file(const std::string& path, std::string* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  return true;
}

// Accepts either <dir>/<cluster_N>/best_tuning_spec.json or <dir>/best_tuning_spec.json.
int load_spec_dir(const std::string& dir, const std::string& module_name, TuningSpec* spec,
                  std::string* err) {
  std::string text;
  const std::string a = dir + "/" + cluster_dir_name(module_name) + "/best_tuning_spec.json";
  const std::string b = dir + "/best_tuning_spec.json";
  if (!read_file(a, &text) && !read_file(b, &text)) {
    if (err) *err = "no best_tuning_spec.json under " + dir;
    return MONONN_ERR_IO;
  }
  return spec_from_json(text, spec, err);
}

bool make_dirs(const std::string& path) {
  std::string cur;
  for (size_t i = 0; i <= path.size(); ++i) {
    if (i == path.size() || path[i] == '/') {
      if (!cur.empty() && cur != "/") {
        if (mkdir(cur.c_str(), 0777) != 0) {
          struct stat st;
          if (stat(cur.c_str(), &st) != 0 || !S_ISDIR(st.st_mode)) return false;
        }
      }
    }
    if (i < path.size()) cur.push_back(path[i]);
  }
  return true;
}

int save_spec_dir(const std::string& dir, const std::string& module_name, const std::string& json,
                  const std::vector<PerfRow>& perf, const std::string& log, std::string* err) {
  const std::string cdir = dir + "/" + cluster_dir_name(module_name);
  if (!make_dirs(cdir)) {
    if (err) *err = "cannot create " + cdir;
    return MONONN_ERR_IO;
  }
  auto write = [&](const std::string& name, const std::string& content) {
    std::ofstream f(cdir + "/" + name, std::ios::binary | std::ios::trunc);
    if (!f) return false;
    f << content;
    return static_cast<bool>(f);
  };
  if (!write("best_tuning_spec.json", json)) {
    if (err) *err = "cannot write best_tuning_spec.json in " + cdir;
    return MONONN_ERR_IO;
  }
  // per-context copy, named as the reference names it: <grid>_1_1__<block>_1_1.json
  {
    TuningSpec s;
    std::string e;
    if (spec_from_json(json, &s, &e) == MONONN_OK && s.grid) {
      std::ostringstream n;
      n << s.grid << "_1_1__" << s.block << "_1_1.json";
      write(n.str(), json);
    }
  }
  if (!perf.empty()) {
    std::ostringstream csv;
    for (const PerfRow& r : perf) csv << r.context << "," << r.node << "," << r.us << "\n";
    write("performance_report.csv", csv.str());
  }
  if (!log.empty()) write("tuning_log.log", log);
  return MONONN_OK;
}

}  // namespace mononn

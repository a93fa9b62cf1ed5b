// extern "C" surface of libmononn_b200.so (declared in include/mononn.h).
#include <cstdlib>
#include <cstring>
#include <new>

#include "builders.h"
#include "json.h"
#include "hlo_lowering.h"
#include "module.h"

using namespace mononn;

static int fail(int code, const std::string& msg) {
  set_last_error(msg);
  return code;
}

void mononn_module::refresh_descs() {
  const Plan& p = rt.plan();
  descs.clear();
  for (size_t i = 0; i < p.args.size(); ++i) {
    mononn_arg_desc d;
    d.index = static_cast<int>(i);
    d.bytes = p.args[i].bytes;
    d.kind = p.args[i].kind;
    d.param_number = p.args[i].param_number;
    descs.push_back(d);
  }
  const_names.clear();
  const_bytes.clear();
  for (const ConstBinding& b : p.consts) {
    bool seen = false;
    for (const std::string& n : const_names) seen = seen || n == b.const_name;
    if (seen) continue;
    const_names.push_back(b.const_name);
    const_bytes.push_back(b.src_bytes);
  }
  stage_name_store = p.stage_names;
  spec_json = spec_to_json(p, rt.sm_count());
  plan_json = plan_to_json(p);
}

int mononn_module::lower(const TuningSpec& spec) {
  Plan plan;
  std::string err;
  int rc = schedule(graph, spec, rt.sm_count(), &plan, &err);
  if (rc) return fail(rc, err);
  rc = rt.load_plan(plan);
  if (rc) return rc;
  refresh_descs();
  return MONONN_OK;
}

static int finish_compile(mononn_module* m, const mononn_options* opt, mononn_module** out) {
  auto env_or = [](const char* given, const char* env) -> std::string {
    if (given && *given) return given;
    const char* v = std::getenv(env);
    return v ? std::string(v) : std::string();
  };
  m->dump_dir = env_or(opt ? opt->dump_dir : nullptr, "TF_MONONN_DUMP_DIR");
  m->spec_dir = env_or(opt ? opt->spec_dir : nullptr, "TF_MONONN_EXISTING_TUNING_SPEC_DIR");
  m->threadpool_size = opt ? opt->threadpool_size : 0;
  if (m->threadpool_size <= 0) {
    const char* v = std::getenv("TF_MONONN_THREADPOOL_SIZE");
    m->threadpool_size = v ? std::atoi(v) : 0;
  }
  m->tuning_level = opt ? opt->tuning_level : 0;
  m->rt.pack_threads = m->threadpool_size;
  int rc = m->rt.init(opt ? opt->device : 0);
  if (rc) {
    delete m;
    return rc;
  }
  if (opt && opt->barrier_timeout_us) m->rt.timeout_us = opt->barrier_timeout_us;
  TuningSpec spec;
  if (!m->spec_dir.empty()) {
    std::string err;
    rc = load_spec_dir(m->spec_dir, m->graph.module_name, &spec, &err);
    if (rc) {
      delete m;
      return fail(rc, err);
    }
  }
  rc = m->lower(spec);
  if (rc) {
    delete m;
    return rc;
  }
  // constants whose values the HLO text carried need not be set by the caller
  for (const auto& kv : m->graph.literals) {
    bool wanted = false;
    for (const ConstBinding& b : m->rt.plan().consts) wanted = wanted || b.const_name == kv.first;
    if (!wanted) continue;
    rc = m->rt.set_constant(kv.first, kv.second.data(), kv.second.size());
    if (rc) {
      delete m;
      return rc;
    }
  }
  *out = m;
  return MONONN_OK;
}

extern "C" {

int mononn_compile_hlo_text(const char* hlo_text, size_t len, const char* kernel_name,
                            const mononn_options* options, mononn_module** out) {
  if (!hlo_text || !out) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  mononn_module* m = new (std::nothrow) mononn_module();
  if (!m) return fail(MONONN_ERR_INVALID_ARGUMENT, "out of memory");
  std::string err;
  int rc = hlo_text_to_fgraph(std::string(hlo_text, len), &m->graph, &err);
  if (rc) {
    delete m;
    return fail(rc, err);
  }
  m->kernel_name = kernel_name ? kernel_name : "mononn_" + m->graph.module_name;
  return finish_compile(m, options, out);
}

int mononn_compile_encoder_json(const char* config_json, const char* kernel_name,
                                const mononn_options* options, mononn_module** out) {
  if (!config_json || !out) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  EncoderConfig cfg;
  std::string err;
  int rc = encoder_config_from_json(config_json, &cfg, &err);
  if (rc) return fail(rc, err);
  mononn_module* m = new (std::nothrow) mononn_module();
  if (!m) return fail(MONONN_ERR_INVALID_ARGUMENT, "out of memory");
  rc = build_bert_encoder(cfg, &m->graph, &err);
  if (rc) {
    delete m;
    return fail(rc, err);
  }
  m->kernel_name = kernel_name ? kernel_name : "mononn_" + m->graph.module_name;
  return finish_compile(m, options, out);
}

int mononn_module_args(const mononn_module* m, const mononn_arg_desc** descs, int* n) {
  if (!m || !descs || !n) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *descs = m->descs.data();
  *n = static_cast<int>(m->descs.size());
  return MONONN_OK;
}

int mononn_module_launch_config(const mononn_module* m, unsigned grid[3], unsigned block[3],
                                unsigned* smem_bytes) {
  if (!m || !grid || !block || !smem_bytes) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  const Plan& p = m->rt.plan();
  grid[0] = p.grid;
  grid[1] = grid[2] = 1;
  block[0] = p.block;
  block[1] = block[2] = 1;
  *smem_bytes = p.smem_bytes;
  return MONONN_OK;
}

int mononn_set_constant(mononn_module* m, const char* name, const void* host, size_t bytes) {
  if (!m || !name || !host) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  return m->rt.set_constant(name, host, bytes);
}

int mononn_constant_count(const mononn_module* m, int* n) {
  if (!m || !n) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *n = static_cast<int>(m->const_names.size());
  return MONONN_OK;
}

int mononn_constant_info(const mononn_module* m, int i, const char** name, size_t* bytes) {
  if (!m || i < 0 || i >= static_cast<int>(m->const_names.size()))
    return fail(MONONN_ERR_INVALID_ARGUMENT, "constant index out of range");
  if (name) *name = m->const_names[i].c_str();
  if (bytes) *bytes = m->const_bytes[i];
  return MONONN_OK;
}

int mononn_launch(mononn_module* m, void* const* device_args, int n, void* cuda_stream) {
  if (!m || !device_args) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  return m->rt.launch_all(device_args, n, cuda_stream);
}

int mononn_infer_host(mononn_module* m, const void* const* host_inputs, int n_inputs,
                      void* const* host_outputs, int n_outputs, void* const* device_args, int n,
                      void* cuda_stream) {
  if (!m || !host_inputs || !host_outputs || !device_args) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  return m->rt.infer_host(host_inputs, n_inputs, host_outputs, n_outputs, device_args, n, cuda_stream);
}

int mononn_last_status(mononn_module* m, int* stage, int* cta) {
  if (!m) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  return m->rt.check_status(stage, cta);
}

int mononn_tune(mononn_module* m, void* const* device_args, int n, void* cuda_stream) {
  if (!m || !device_args) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  return tune_module(m, device_args, n, cuda_stream);
}

int mononn_save_spec(const mononn_module* m, const char* dir) {
  if (!m || !dir) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  std::string err;
  int rc = save_spec_dir(dir, m->graph.module_name, m->spec_json, m->perf, m->tuning_log, &err);
  return rc ? fail(rc, err) : MONONN_OK;
}

int mononn_spec_json(mononn_module* m, const char** json) {
  if (!m || !json) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *json = m->spec_json.c_str();
  return MONONN_OK;
}

int mononn_profile_stages(mononn_module* m, void* const* device_args, int n, void* cuda_stream,
                          double* us, const char** names, int cap, int* n_stages) {
  if (!m || !device_args || !n_stages) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  const uint32_t ns = static_cast<uint32_t>(m->rt.plan().stages.size());
  int rc = m->rt.launch(device_args, n, cuda_stream, 0, ns, true);
  if (rc) return rc;
  int st = 0, cta = 0;
  rc = m->rt.check_status(&st, &cta);
  if (rc) return rc;
  std::vector<double> t;
  rc = m->rt.read_stamps(&t);
  if (rc) return rc;
  *n_stages = static_cast<int>(t.size());
  m->perf.clear();
  const Plan& p = m->rt.plan();
  const std::string ctx =
      std::to_string(p.grid) + "_1_1__" + std::to_string(p.block) + "_1_1";
  for (size_t i = 0; i < t.size(); ++i) {
    if (static_cast<int>(i) < cap) {
      if (us) us[i] = t[i];
      if (names) names[i] = m->stage_name_store[i].c_str();
    }
    m->perf.push_back(PerfRow{ctx, m->stage_name_store[i], t[i]});
  }
  return MONONN_OK;
}

int mononn_plan_json(mononn_module* m, const char** json) {
  if (!m || !json) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *json = m->plan_json.c_str();
  return MONONN_OK;
}

int mononn_launch_stages(mononn_module* m, void* const* device_args, int n, void* cuda_stream,
                         unsigned stage_begin, unsigned stage_end) {
  if (!m || !device_args) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  return m->rt.launch(device_args, n, cuda_stream, stage_begin, stage_end, false);
}

int mononn_describe(const char* kind, const char* text, size_t len, const char* spec_json,
                    unsigned sm_count, char** out_json) {
  if (!kind || !text || !out_json) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  *out_json = nullptr;
  FGraph g;
  std::string err;
  int rc;
  if (std::string(kind) == "hlo") {
    rc = hlo_text_to_fgraph(std::string(text, len), &g, &err);
  } else if (std::string(kind) == "encoder") {
    EncoderConfig cfg;
    rc = encoder_config_from_json(std::string(text, len), &cfg, &err);
    if (!rc) rc = build_bert_encoder(cfg, &g, &err);
  } else {
    return fail(MONONN_ERR_INVALID_ARGUMENT, "kind must be \"hlo\" or \"encoder\"");
  }
  if (rc) return fail(rc, err);
  TuningSpec spec;
  if (spec_json && *spec_json) {
    rc = spec_from_json(spec_json, &spec, &err);
    if (rc) return fail(rc, err);
  }
  Plan plan;
  rc = schedule(g, spec, sm_count ? sm_count : 148, &plan, &err);
  if (rc) return fail(rc, err);
  Json root = Json::object();
  Json plan_j, spec_j;
  std::string e2;
  Json::parse(plan_to_json(plan), &plan_j, &e2);
  Json::parse(spec_to_json(plan, sm_count ? sm_count : 148), &spec_j, &e2);
  root.set("plan", plan_j);
  root.set("spec", spec_j);
  // constants whose values the HLO text carried: name -> their bytes in the element type, as hex
  Json lits = Json::object();
  for (const auto& kv : g.literals) {
    static const char* digits = "0123456789abcdef";
    std::string hex;
    for (uint8_t b : kv.second) {
      hex.push_back(digits[b >> 4]);
      hex.push_back(digits[b & 15]);
    }
    lits.set(kv.first, Json::string(hex));
  }
  root.set("literals", lits);
  const std::string s = root.dump(1);
  char* buf = static_cast<char*>(std::malloc(s.size() + 1));
  if (!buf) return fail(MONONN_ERR_INVALID_ARGUMENT, "out of memory");
  std::memcpy(buf, s.c_str(), s.size() + 1);
  *out_json = buf;
  return MONONN_OK;
}

void mononn_free_string(char* s) { std::free(s); }

int mononn_trace_stages(mononn_module* m, void* const* device_args, int n, void* cuda_stream,
                        double* out, size_t cap, int* grid, int* n_stages) {
  if (!m || !device_args || !out) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  std::vector<double> t;
  int rc = m->rt.trace_launch(device_args, n, cuda_stream, &t);
  if (rc) return rc;
  if (grid) *grid = static_cast<int>(m->rt.plan().grid);
  if (n_stages) *n_stages = static_cast<int>(m->rt.plan().stages.size());
  if (t.size() > cap) return fail(MONONN_ERR_TOO_LARGE, "trace buffer too small");
  std::memcpy(out, t.data(), t.size() * sizeof(double));
  return MONONN_OK;
}

int mononn_debug_skew_barrier(mononn_module* m, unsigned missing_arrivals) {
  if (!m) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  m->rt.skew_epoch(missing_arrivals);
  return MONONN_OK;
}

int mononn_module_cost(const mononn_module* m, double* bytes, double* flops) {
  if (!m) return fail(MONONN_ERR_INVALID_ARGUMENT, "null argument");
  if (bytes) *bytes = m->rt.plan().algorithmic_bytes;
  if (flops) *flops = m->rt.plan().algorithmic_flops;
  return MONONN_OK;
}

void mononn_destroy(mononn_module* m) { delete m; }

const char* mononn_strerror(int code) {
  switch (code) {
    case MONONN_OK: return "ok";
    case MONONN_ERR_INVALID_ARGUMENT: return "invalid argument";
    case MONONN_ERR_PARSE: return "parse error";
    case MONONN_ERR_UNSUPPORTED: return "unsupported operator, type, layout or pattern";
    case MONONN_ERR_CUDA: return "CUDA call failed";
    case MONONN_ERR_NO_DEVICE: return "no sm_100 device";
    case MONONN_ERR_BARRIER_TIMEOUT: return "bounded wait inside the kernel expired";
    case MONONN_ERR_CONSTANT: return "unknown constant or wrong size";
    case MONONN_ERR_IO: return "I/O error";
    case MONONN_ERR_NOT_READY: return "constants missing";
    case MONONN_ERR_TOO_LARGE: return "size beyond the documented maximum";
    default: return "unknown error";
  }
}

const char* mononn_last_error(void) { return get_last_error(); }

int mononn_enabled(void) { return env_truthy("TF_MONONN_ENABLED") ? 1 : 0; }

}  // extern "C"

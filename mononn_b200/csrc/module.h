// The object behind the opaque mononn_module handle.
//
// Counterpart of MonoNNModule (mononn_engine/module/mononn_module.h:31-87): it owns the
// fused graph, the tuning spec it was lowered with and the launchable artefact -- a stage
// table bound to device memory instead of PTX text.
#pragma once
#include <string>
#include <vector>

#include "../../include/mononn.h"
#include "plan.h"
#include "runtime.h"

struct mononn_module {
  std::string kernel_name;
  mononn::FGraph graph;
  mononn::Runtime rt;
  std::string dump_dir, spec_dir;
  int threadpool_size = 0;
  int tuning_level = 0;
  std::vector<mononn_arg_desc> descs;
  std::vector<std::string> const_names;
  std::vector<size_t> const_bytes;
  std::string spec_json;
  std::string plan_json;
  std::vector<mononn::PerfRow> perf;
  std::vector<std::string> stage_name_store;
  std::string tuning_log;

  // Lower graph with `spec` and (re)load the device state.
  int lower(const mononn::TuningSpec& spec);
  void refresh_descs();
};

namespace mononn {
// spec.cc: GraphSpecification-shaped JSON of a tuning spec and its launch context.
std::string spec_to_json(const Plan& plan, uint32_t sm_count);
std::string plan_to_json(const Plan& plan);
int spec_from_json(const std::string& text, TuningSpec* spec, std::string* err);
int load_spec_dir(const std::string& dir, const std::string& module_name, TuningSpec* spec,
                  std::string* err);
int save_spec_dir(const std::string& dir, const std::string& module_name, const std::string& json,
                  const std::vector<PerfRow>& perf, const std::string& log, std::string* err);
std::string cluster_dir_name(const std::string& module_name);
bool make_dirs(const std::string& path);
bool env_truthy(const char* name);
// tuner.cc
int tune_module(mononn_module* m, void* const* args, int n, void* stream);
}  // namespace mononn

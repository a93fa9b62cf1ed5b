// On-device schedule search.
//
// Follows the shape of MonoNNModuleTuner::tune
// (mononn_engine/module/mononn_module_tuner.cc:620-991): GEMM candidates are de-duplicated
// by problem (the reference hashes the GEMM problem, :386-408, and copies the best
// CutlassConfig to every node with that hash, :820-975), each candidate is timed on the
// device, and the winners are merged into one spec that is timed end to end against the
// heuristic default. Because a candidate here is a table, not a CUDA source to be compiled
// by an nvcc subprocess, one candidate costs a re-pack of the affected weights plus a few
// launches.
#include <algorithm>
#include <sstream>
#include <tuple>

#include "module.h"

namespace mononn {

namespace {
struct ProblemKey {
  uint32_t M, N, K, flags, act, out_mode;
  bool operator<(const ProblemKey& o) const {
    return std::tie(M, N, K, flags, act, out_mode) <
           std::tie(o.M, o.N, o.K, o.flags, o.act, o.out_mode);
  }
};
}  // namespace

int tune_module(mononn_module* m, void* const* args, int n, void* stream) {
  std::ostringstream log;
  const int warm = 3, iters = 20;
  TuningSpec best = m->rt.plan().spec;
  best.allow_list.clear();
  best.reject_list.clear();
  int rc = m->lower(best);
  if (rc) return rc;
  const uint32_t n_stages = static_cast<uint32_t>(m->rt.plan().stages.size());
  double best_us = 0;
  rc = m->rt.time_stages(args, n, stream, 0, n_stages, warm, iters, &best_us);
  if (rc) return rc;
  log << "default spec: " << best_us << " us\n";
  const double default_us = best_us;
  const TuningSpec default_spec = best;

  if (m->tuning_level >= 1) {
    // group GEMM nodes by problem
    std::map<ProblemKey, std::vector<std::string>> classes;
    std::map<ProblemKey, std::pair<bool, uint32_t>> meta;  // can_split, budget
    {
      const Plan& p = m->rt.plan();
      for (const StageDesc& sd : p.stages) {
        uint32_t gemms = 0;
        for (uint32_t i = 0; i < sd.op_count; ++i)
          if (p.ops[sd.op_begin + i].d.kind == OP_GEMM) ++gemms;
        for (uint32_t i = 0; i < sd.op_count; ++i) {
          const PlanOp& op = p.ops[sd.op_begin + i];
          if (op.d.kind != OP_GEMM) continue;
          ProblemKey k{op.d.M, op.d.N, op.d.K, op.d.flags, op.d.act, op.d.out_mode};
          classes[k].push_back(op.name);
          meta[k] = {op.d.out_mode == OUT_F32_RED && op.d.act == ACT_NONE,
                     std::max(1u, p.grid / std::max(1u, gemms))};
        }
      }
    }
    for (const auto& kv : classes) {
      const ProblemKey& k = kv.first;
      const auto cands = gemm_tile_candidates(k.M, k.N, k.K, meta[k].first, meta[k].second);
      GemmTileSpec cur = best.gemm[kv.second.front()];
      for (const GemmTileSpec& c : cands) {
        if (c.n_tile == cur.n_tile && c.k_split == cur.k_split) continue;
        TuningSpec trial = best;
        for (const std::string& node : kv.second) trial.gemm[node] = c;
        rc = m->lower(trial);
        if (rc) return rc;
        double us = 0;
        rc = m->rt.time_stages(args, n, stream, 0, n_stages, warm, iters, &us);
        if (rc) return rc;
        log << "M" << k.M << " N" << k.N << " K" << k.K << " n_tile " << c.n_tile << " k_split "
            << c.k_split << ": " << us << " us\n";
        if (us < best_us) {
          best_us = us;
          best = trial;
          cur = c;
        }
      }
    }
  }
  // final pick: the merged spec must beat the default end to end, else keep the default
  rc = m->lower(best);
  if (rc) return rc;
  double final_us = 0;
  rc = m->rt.time_stages(args, n, stream, 0, n_stages, warm, iters, &final_us);
  if (rc) return rc;
  log << "merged spec: " << final_us << " us (default " << default_us << " us)\n";
  if (final_us > default_us) {
    rc = m->lower(default_spec);
    if (rc) return rc;
    log << "kept the default spec\n";
  }
  m->tuning_log = log.str();
  if (!m->dump_dir.empty()) {
    std::string err;
    rc = save_spec_dir(m->dump_dir, m->graph.module_name, m->spec_json, m->perf, m->tuning_log,
                       &err);
    if (rc) {
      set_last_error(err);
      return rc;
    }
  }
  return MONONN_OK;
}

}  // namespace mononn

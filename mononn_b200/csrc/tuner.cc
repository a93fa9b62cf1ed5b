// On-device schedule search.
//
// Follows the shape of MonoNNModuleTuner::tune
// (mononn_engine/module/mononn_module_tuner.cc:620-991): candidates are enumerated per
// dimension of the schedule space (TuningSpaceGenerator,
// mononn_engine/tuning/tuning_space_generator.cc:52-309), GEMM candidates are de-duplicated by
// problem (the reference hashes the GEMM problem, :386-408, and copies the best CutlassConfig to
// every node with that hash, :820-975) and timed in isolation on the stage that holds one node
// of the class (the reference isolates a node with its codegen allow-list, :647-722), and the
// winners are merged into one spec that is timed end to end against the heuristic default.
// Because a candidate here is a table, not a CUDA source to be compiled by an nvcc
// subprocess, one candidate costs a re-pack of the affected weights plus a few launches.
//
// Dimensions searched, by tuning_level:
//   0  none: the heuristic spec is timed and reported
//   1  stage structure (Q/K/V projections inside the attention items or as a stage of their own;
//      LayerNorm in the stage of its split-K GEMMs or behind a grid barrier of its own), L2
//      eviction hints on the weight and activation streams, then
//      the tile width and K split of every GEMM problem class
//   2  + the cluster shape (CTAs that arrive at the grid barrier through one of them) and the
//      number of CTAs of the cooperative launch (the reference's (grid, block) contexts,
//      mononn_engine/tuning/tuning_space_generator.cc:65-101)
#include <algorithm>
#include <fstream>
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

// Per-measurement journal, <dump_dir>/<cluster_N>/tuning_progress.log: one line
// "<label>\t<microseconds>" per timed spec, flushed as it is written. The search is
// deterministic, so a tune that was interrupted (the reference cannot resume one:
// its tuning_log.log is written at the end, mononn_module_tuner.cc:560-583) replays the
// journal on its next run: measurements whose label matches, in order, are reused; from
// the first difference on everything is measured again.
struct Journal {
  std::vector<std::pair<std::string, double>> old;
  size_t next = 0;
  int reused = 0;
  std::ofstream out;

  void open(const std::string& dump_dir, const std::string& module_name) {
    if (dump_dir.empty()) return;
    const std::string dir = dump_dir + "/" + cluster_dir_name(module_name);
    if (!make_dirs(dir)) return;
    const std::string path = dir + "/tuning_progress.log";
    {
      std::ifstream in(path);
      std::string line;
      while (std::getline(in, line)) {
        const size_t tab = line.rfind('\t');
        if (tab == std::string::npos) break;
        char* end = nullptr;
        const double us = std::strtod(line.c_str() + tab + 1, &end);
        if (end == line.c_str() + tab + 1 || us <= 0) break;  // a torn last line ends the replay
        old.push_back({line.substr(0, tab), us});
      }
    }
    out.open(path, std::ios::trunc);
  }
  // Returns true and sets *us when the next journal entry is this measurement.
  bool replay(const std::string& label, double* us) {
    if (next < old.size() && old[next].first == label) {
      *us = old[next++].second;
      ++reused;
      record(label, *us);
      return true;
    }
    old.resize(next);  // diverged: nothing after this point can be trusted
    return false;
  }
  void record(const std::string& label, double us) {
    if (!out.is_open()) return;
    out << label << '\t' << us << '\n';
    out.flush();
  }
};

// Stage of the current plan that holds operator `node`, or -1.
int stage_of(const Plan& p, const std::string& node) {
  for (size_t s = 0; s < p.stages.size(); ++s)
    for (uint32_t i = 0; i < p.stages[s].op_count; ++i)
      if (p.ops[p.stages[s].op_begin + i].name == node) return static_cast<int>(s);
  return -1;
}
}  // namespace

int tune_module(mononn_module* m, void* const* args, int n, void* stream) {
  std::ostringstream log;
  const int warm = 3, iters = 20;
  Journal journal;
  journal.open(m->dump_dir, m->graph.module_name);
  // One timed spec: replayed from the journal when possible, else lowered and measured. With a
  // node name only the stage that holds the node is launched (isolation); otherwise all stages.
  auto measure = [&](const std::string& label, const TuningSpec& spec, const std::string& node,
                     double* us) -> int {
    if (journal.replay(label, us)) return MONONN_OK;
    int r = m->lower(spec);
    if (r) return r;
    uint32_t begin = 0, end = static_cast<uint32_t>(m->rt.plan().stages.size());
    if (!node.empty()) {
      const int s = stage_of(m->rt.plan(), node);
      if (s < 0) {
        set_last_error("tuner: operator " + node + " is not in the lowered plan");
        return MONONN_ERR_INVALID_ARGUMENT;
      }
      begin = static_cast<uint32_t>(s);
      end = begin + 1;
    }
    r = m->rt.time_stages(args, n, stream, begin, end, warm, iters, us);
    if (r) return r;
    journal.record(label, *us);
    return MONONN_OK;
  };
  TuningSpec best = m->rt.plan().spec;
  best.allow_list.clear();
  best.reject_list.clear();
  int rc = m->lower(best);
  if (rc) return rc;
  double best_us = 0;
  rc = measure("default", best, "", &best_us);
  if (rc) return rc;
  log << "default spec: " << best_us << " us\n";
  const double default_us = best_us;
  const TuningSpec default_spec = best;

  if (m->tuning_level >= 1) {
    // ---- stage structure: whole-graph choices, timed end to end
    struct Structural {
      const char* name;
      uint32_t TuningSpec::*field;
      uint32_t value;
    };
    const Structural choices[] = {
        {"qkv_fusion off", &TuningSpec::qkv_fusion, 1u},
        {"qkv_fusion on", &TuningSpec::qkv_fusion, 2u},
        {"row_fusion off", &TuningSpec::row_fusion, 1u},
        {"row_fusion on", &TuningSpec::row_fusion, 2u},
        {"l2_hints off", &TuningSpec::l2_hints, 1u},
        {"l2_hints on", &TuningSpec::l2_hints, 2u},
        {"barrier_arrive cta", &TuningSpec::barrier_arrive, 1u},
        {"barrier_arrive warp", &TuningSpec::barrier_arrive, 2u},
        {"row_split off", &TuningSpec::row_split, 1u},
        {"out_fusion off", &TuningSpec::out_fusion, 1u},
        {"out_fusion on", &TuningSpec::out_fusion, 2u},
        {"chain_fusion off", &TuningSpec::chain_fusion, 1u},
        {"chain_fusion on", &TuningSpec::chain_fusion, 2u},
    };
    for (const Structural& c : choices) {
      if (best.*(c.field) == c.value) continue;
      TuningSpec trial = best;
      trial.*(c.field) = c.value;
      if (c.field != &TuningSpec::l2_hints && c.field != &TuningSpec::barrier_arrive)
        trial.gemm.clear();  // the GEMM nodes and their CTA budgets change with the structure
      double us = 0;
      rc = measure(c.name, trial, "", &us);
      if (rc == MONONN_ERR_UNSUPPORTED || rc == MONONN_ERR_INVALID_ARGUMENT) {
        log << c.name << ": not applicable to this graph\n";
        continue;
      }
      if (rc) return rc;
      log << c.name << ": " << us << " us\n";
      if (us < best_us) {
        best_us = us;
        rc = m->lower(trial);
        if (rc) return rc;
        best = m->rt.plan().spec;  // with the heuristic tiles of the new structure filled in
      }
    }
    rc = m->lower(best);
    if (rc) return rc;

    // ---- GEMM tiles: group the nodes by problem, time candidates on one node's stage alone
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
      // a node from the middle of the graph: its inputs are what a steady-state layer sees
      const std::string probe = kv.second[kv.second.size() / 2];
      const auto cands = gemm_tile_candidates(k.M, k.N, k.K, meta[k].first, meta[k].second);
      GemmTileSpec cur = best.gemm[probe];
      std::ostringstream cls;
      cls << "M" << k.M << " N" << k.N << " K" << k.K << " f" << k.flags << " a" << k.act << " o" << k.out_mode;
      double cur_us = 0;
      rc = measure(cls.str() + " stage of " + probe + " as is", best, probe, &cur_us);
      if (rc) return rc;
      log << cls.str() << " n_tile " << cur.n_tile << " k_split " << cur.k_split << " (current): " << cur_us
          << " us for its stage\n";
      for (const GemmTileSpec& c : cands) {
        if (c.n_tile == cur.n_tile && c.k_split == cur.k_split) continue;
        TuningSpec trial = best;
        for (const std::string& node : kv.second) trial.gemm[node] = c;
        double us = 0;
        std::ostringstream label;
        label << cls.str() << " n_tile " << c.n_tile << " k_split " << c.k_split;
        rc = measure(label.str(), trial, probe, &us);
        if (rc) return rc;
        log << label.str() << ": " << us << " us for its stage\n";
        if (us < cur_us) {
          cur_us = us;
          best = trial;
          cur = c;
        }
      }
    }
  }
  if (m->tuning_level >= 2) {
    // ---- CTAs of the launch: fewer CTAs make the grid barrier cheaper and the tiles wider
    const uint32_t sms = m->rt.sm_count();
    rc = measure("merged tiles", best, "", &best_us);
    if (rc) return rc;
    for (uint32_t cluster : {2u, 4u}) {
      if (best.grid % cluster != 0 || cluster == best.cluster) continue;
      TuningSpec trial = best;
      trial.cluster = cluster;
      double us = 0;
      std::ostringstream label;
      label << "cluster " << cluster;
      rc = measure(label.str(), trial, "", &us);
      if (rc == MONONN_ERR_INVALID_ARGUMENT) {  // not co-resident in this shape
        log << label.str() << ": " << get_last_error() << "\n";
        continue;
      }
      if (rc) return rc;
      log << label.str() << ": " << us << " us\n";
      if (us < best_us) {
        best_us = us;
        best = trial;
      }
    }
    for (uint32_t grid : {sms - sms / 8, sms - sms / 4, sms / 2}) {
      grid -= grid % std::max(1u, best.cluster);
      if (grid == 0 || grid == best.grid) continue;
      TuningSpec trial = best;
      trial.grid = grid;
      trial.gemm.clear();  // tiles are chosen for the CTA budget
      double us = 0;
      std::ostringstream label;
      label << "grid " << grid;
      rc = measure(label.str(), trial, "", &us);
      if (rc) return rc;
      log << label.str() << ": " << us << " us\n";
      if (us < best_us) {
        best_us = us;
        rc = m->lower(trial);
        if (rc) return rc;
        best = m->rt.plan().spec;
      }
    }
  }
  // final pick: the merged spec must beat the default end to end, else keep the default
  rc = m->lower(best);
  if (rc) return rc;
  double final_us = 0;
  {
    const uint32_t ns = static_cast<uint32_t>(m->rt.plan().stages.size());
    rc = m->rt.time_stages(args, n, stream, 0, ns, warm, iters, &final_us);
    if (rc) return rc;
  }
  if (journal.reused) log << "reused " << journal.reused << " measurements of an earlier run\n";
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

// The control plane's time model: what one lane's remaining work costs at a given SM
// share, link-credit grant and kernel form for its host-resident experts.
//
// The model is the reference's (csrc/control/estimator.h:1-168, estimator.cpp:200-258;
// Eq. 1 and 2 of its paper): a layer is an attention window followed by an MoE window;
// inside a window compute and memory reads overlap, so a window costs the largest of one
// term per resource it can wait for (SM compute; HBM reads, stretched by contention; for
// MoE also the host link); the lane's estimate is the sum over its remaining layers and
// passes plus per-layer and per-pass overheads.  Every rate is a calibrated curve
// against the SM share or the credits.  What is specific to this library:
//   * the one-pass form (form 0) reads an expert once per 256-row block and keeps its
//     partial sums in TMEM, so it has no partial-sum traffic in HBM (one_pass_rows,
//     one_pass_row_bytes below are parameters of the calibration, not constants);
//   * credits are whatever unit the calibration's rho curves use: on a B200 behind PCIe
//     they are link slots (workers allowed to read host memory at once).
#pragma once
#include <algorithm>
#include <cmath>
#include <map>
#include <stdexcept>
#include <vector>

namespace mf {
namespace plan {

constexpr int kOnePass = 0;   // the form id of the weight-stationary / one-pass kernel ("asym" in the reference)

// Piecewise-linear curve through measured points (x increasing).  Flat beyond the last
// point; before the first point flat, or, for a rate that vanishes at zero, a straight
// line to the origin (csrc/control/curve.h:10-27).
struct Curve {
  std::vector<double> x, y;
  bool through_origin = false;
  bool empty() const { return x.empty(); }
  double operator()(double v) const {
    if (x.empty()) return 0.0;
    if (v >= x.back()) return y.back();
    if (v <= x.front()) return (through_origin && x.front() > 0) ? y.front() * std::max(v, 0.0) / x.front() : y.front();
    size_t hi = 1;
    while (x[hi] < v) ++hi;
    const double f = (v - x[hi - 1]) / (x[hi] - x[hi - 1]);
    return y[hi - 1] + f * (y[hi] - y[hi - 1]);
  }
  // The largest x whose value stays within `level` (infinite once the curve's plateau is within it).
  double last_within(double level) const;
};

struct ModelShape {
  int hidden = 0, intermediate = 0, experts = 0, top_k = 0, layers = 0;
  int heads = 0, kv_heads = 0, head_dim = 128, vocab = 0;
  int dense_layers = 0, dense_intermediate = 0, shared_intermediate = 0;
  double expert_weight_bytes = 2, dense_weight_bytes = 2;
  double expert_bytes() const { return 3.0 * hidden * intermediate * expert_weight_bytes; }
  double kv_bytes_per_token() const { return 2.0 * layers * kv_heads * head_dim * 2.0; }
};

struct KernelRates {
  Curve flops, bytes;     // against the SM share
  double q_per_sm = 0;    // link / memory-queue entries one SM keeps in flight under this kernel
};

struct Calibration {
  int sms = 0;
  double hbm_residency = 0, link_residency = 0;   // R_H, R_C: seconds an entry of each kind stays in flight
  Curve stretch;                                   // gamma: read-time stretch against exposure (entry-seconds)
  double q_max = 0;
  KernelRates dense, attn_prefill, attn_decode;
  std::map<int, KernelRates> expert;               // by form
  std::map<int, Curve> link_rate;                  // rho: bytes/s against credits, by form
  std::map<int, double> tile_credits;              // q(form): credits one host-expert tile keeps in flight
  double link_peak = 0;                            // beta
  int reference_form = 64;
  double layer_overhead = 0, tail_overhead = 0;
  int one_pass_rows = 64;                          // row block of form 0 in the compute term (reference: <= 64; this library: 256)
  double one_pass_row_bytes = -1;                  // HBM bytes per routed row of form 0's partial sums; < 0: the reference's K-split formula

  double rho(int form, double credits) const;
  double credits_per_tile(int form) const;
  double saturating_credits() const;               // Q^link: fewest credits at which the reference form reaches 99 % of beta
  double exposure_bound() const { return saturating_credits() * link_residency + q_max * sms * hbm_residency; }
};

struct Seq {
  int tokens = 1, context = 0;
};

struct LaneWork {
  bool decode = false;
  std::vector<std::vector<Seq>> passes;
  int first_layer = 0;
  std::vector<double> active, miss;
  int staging = 0;
  double deadline = 0;
  bool samples = true;
};

struct PassLoad {
  double tokens = 0, attn_flops = 0, kv_bytes = 0, proj_flops = 0, proj_bytes = 0, pairs = 0, moe_act_bytes = 0;
  double shared_flops = 0, shared_bytes = 0, dense_mlp_flops = 0, dense_mlp_bytes = 0;
  double link_rows_bound = 0, sampled = 0;
  std::vector<double> active, miss;
  int first_layer = 0;
};

struct LaneLoad {
  bool decode = false;
  int staging = 0;
  double deadline = 0;
  std::vector<PassLoad> passes;
};

struct Estimate {
  double total = 0, attn = 0, moe = 0, staged = 0;
  double a_cmp = 0, a_rd = 0, m_cmp = 0, m_rd = 0, m_link = 0;   // terms of the first pass's first MoE layer
};

struct EstimatorOptions {
  bool contention_aware = true;
  double ewma = 0.1;
};

PassLoad pass_load(const ModelShape& m, const LaneWork& w, const std::vector<Seq>& seqs, bool first, bool last);

class Estimator {
 public:
  Estimator(const ModelShape& m, const Calibration& c, EstimatorOptions o);
  LaneLoad load(const LaneWork& w) const;
  Estimate evaluate(const LaneLoad& l, int share, double credits, int form) const;
  double gamma_ratio(double own_exposure) const;
  void observe(bool decode, bool moe, double ratio);
  double correction(bool decode, bool moe) const { return correction_[decode][moe]; }
  const ModelShape& model() const { return model_; }
  const Calibration& calibration() const { return cal_; }
  const EstimatorOptions& options() const { return opt_; }
  double link_credits() const { return q_link_; }
  double exposure_bound() const { return x_max_; }

 private:
  struct RatesAtShare;
  const KernelRates& expert_kernel(int form) const;
  double moe_window(const LaneLoad& l, const PassLoad& p, int layer, const RatesAtShare& r, double staged_cap, int form,
                    double& staged, double terms[3]) const;
  ModelShape model_;
  Calibration cal_;
  EstimatorOptions opt_;
  double q_link_ = 0, x_max_ = 0, stretch_max_ = 1, expert_bytes_ = 0, one_pass_row_bytes_ = 0;
  double correction_[2][2] = {{1, 1}, {1, 1}};
};

// ------------------------------------------------------------------ plan search
struct SearchOptions {
  std::vector<int> forms{16, 32, 64, 128, kOnePass};
  int pour_quantum = 2, pour_candidates = 8, decode_choices = 4;
  double tolerance = 0.01;
};

struct LanePlan {
  int sms = 0;
  double credits = 0;
  int form = 64;
  int cap = 0;
  double rate = 0, slack = 0;
  Estimate est;
};

struct Plan {
  bool feasible = false;
  std::vector<LanePlan> lanes;
  double copy_rate = 0, min_slack = 0, total_time = 0;
  long evaluations = 0;
  double micros = 0;
};

// Algorithm 1 of the reference's paper (csrc/control/search.h:1-90): with the exposure bound
// fixed, lanes do not interact, so per lane, form and grant the smallest share that meets
// the deadline is found by bisection; the decode lane is settled first (its options are
// cached under a caller-given key), prefill lanes enumerate forms and a split of the
// remaining credits, spare SMs are poured onto the lane with the least slack, and the
// best candidate is re-evaluated at whole link slots.
class PlanSearch {
 public:
  PlanSearch(const Estimator* est, SearchOptions opt);
  Plan solve(const std::vector<LaneLoad>& lanes, unsigned long long decode_key);
  int deadline_floor(const LaneLoad& l, double credits, int form, long* evals) const;
  std::vector<double> grants(int form) const;
  void clear_cache() { decode_cache_.clear(); }
  const Estimator& estimator() const { return *est_; }

 private:
  struct Option {
    int form;
    double credits;
    int floor;
  };
  struct Candidate {
    std::vector<int> form, share;
    std::vector<double> credits, slack;
    std::vector<Estimate> est;
    int spare = 0;
    double min_slack = 0, total = 0;
  };
  void pour_spare(const std::vector<LaneLoad>& lanes, Candidate& c, long& evals) const;
  bool settle(const std::vector<LaneLoad>& lanes, const Candidate& c, Plan& out, long& evals) const;
  Plan fallback(const std::vector<LaneLoad>& lanes, const std::vector<Option>& decode_options, long& evals) const;
  const Estimator* est_;
  SearchOptions opt_;
  std::map<unsigned long long, std::vector<Option>> decode_cache_;
};

}  // namespace plan
}  // namespace mf

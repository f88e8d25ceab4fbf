// Host code only: the control plane's time estimator and plan search (plan_model.h).
#include "plan_model.h"

#include <chrono>
#include <limits>
#include <tuple>

namespace mf {
namespace plan {

namespace {

constexpr double kNever = 1e30;

// work / rate, where no work costs nothing and work at no rate never finishes
double time_for(double work, double rate) { return work <= 0 ? 0.0 : (rate > 0 ? work / rate : kNever); }

double round_up_rows(double rows, int block) { return std::ceil(std::max(rows, 0.0) / block) * block; }

// Row-block height the expander gives an HBM expert with `rows` routed rows (16 / 32 / 64 / 128).
int hbm_block(double rows) {
  int h = 16;
  while (h < 128 && rows > h) h *= 2;
  return h;
}

double relative_slack(const LaneLoad& l, double t) { return l.deadline > 0 ? (l.deadline - t) / l.deadline : -kNever; }

}  // namespace

double Curve::last_within(double level) const {
  if (level <= 0 || x.empty()) return 0.0;
  if (level >= y.back()) return std::numeric_limits<double>::infinity();
  if (level < y.front()) return (through_origin && y.front() > 0) ? x.front() * level / y.front() : 0.0;
  for (size_t i = 1; i < x.size(); ++i)
    if (y[i] > level) return x[i - 1] + (level - y[i - 1]) / (y[i] - y[i - 1]) * (x[i] - x[i - 1]);
  return x.back();
}

// ----------------------------------------------------------------- calibration
double Calibration::rho(int form, double credits) const {
  const auto it = link_rate.find(form);
  if (it == link_rate.end()) throw std::runtime_error("monofab: the calibration has no credit sweep for kernel form " + std::to_string(form));
  return it->second(credits);
}

double Calibration::credits_per_tile(int form) const {
  const auto it = tile_credits.find(form);
  return it == tile_credits.end() ? 1.0 : std::max(it->second, 1e-9);
}

double Calibration::saturating_credits() const {
  const auto it = link_rate.find(reference_form);
  if (it == link_rate.end() || it->second.empty()) return 0.0;
  const Curve& c = it->second;
  const double want = 0.99 * link_peak;   // a measured curve approaches the peak; "reaches" allows 1 %
  for (size_t i = 0; i < c.x.size(); ++i) {
    if (c.y[i] < want) continue;
    if (i == 0) return c.x[0];
    return c.x[i - 1] + (want - c.y[i - 1]) / std::max(c.y[i] - c.y[i - 1], 1e-30) * (c.x[i] - c.x[i - 1]);
  }
  return c.x.back();
}

// ------------------------------------------------------------------- workload
// FLOPs, bytes and routed rows of one pass, counted as the calibration runs count theirs
// (csrc/control/estimator.cpp:119-186).
PassLoad pass_load(const ModelShape& m, const LaneWork& w, const std::vector<Seq>& seqs, bool first, bool last) {
  const double H = m.hidden, D = m.head_dim, hq = m.heads, hkv = m.kv_heads, I = m.intermediate;
  const double qkv = (hq + 2 * hkv) * D;
  PassLoad p;
  double scored_keys = 0, key_reads = 0;
  for (const Seq& s : seqs) {
    const double n = std::max(s.tokens, 0), c = std::max(s.context, 0);
    p.tokens += n;
    scored_keys += n * c + n * (n + 1) / 2;   // causal: row j scores c + j + 1 keys
    if (w.decode) {
      key_reads += c + n;
    } else {   // every 128-row query block reads the keys up to its own end
      for (double q0 = 0; q0 < n; q0 += 128) key_reads += c + std::min(n, q0 + 128);
    }
  }
  p.attn_flops = 4.0 * hq * D * scored_keys;
  p.kv_bytes = key_reads * hkv * D * 4.0 * (w.decode ? 1.0 : hq / std::max(hkv, 1.0));   // K and V, bf16
  p.proj_flops = 2.0 * p.tokens * H * (qkv + hq * D);
  p.proj_bytes = (H * qkv + hq * D * H + H * m.experts) * m.dense_weight_bytes + p.tokens * (2 * H + qkv + 2 * hq * D) * 2.0;
  p.pairs = p.tokens * m.top_k;
  p.moe_act_bytes = p.pairs * (2 * H + 3 * I) * 2.0 + p.tokens * H * 8.0;
  if (m.shared_intermediate > 0) {
    p.shared_flops = 6.0 * p.tokens * H * m.shared_intermediate;
    p.shared_bytes = 3.0 * H * m.shared_intermediate * m.dense_weight_bytes;
  }
  if (m.dense_layers > 0) {
    p.dense_mlp_flops = 6.0 * p.tokens * H * m.dense_intermediate;
    p.dense_mlp_bytes = 3.0 * H * m.dense_intermediate * m.dense_weight_bytes;
  }
  p.link_rows_bound = w.decode ? p.tokens : 0.0;   // a decode batch cannot route more rows to an expert than it has
  p.sampled = (last && w.samples) ? static_cast<double>(seqs.size()) : 0.0;
  p.first_layer = first ? w.first_layer : 0;
  p.active.resize(m.layers);
  p.miss.resize(m.layers);
  for (int l = 0; l < m.layers; ++l) {
    p.active[l] = std::max(l < static_cast<int>(w.active.size()) ? w.active[l] : 0.0, 0.0);
    p.miss[l] = std::min(std::max(l < static_cast<int>(w.miss.size()) ? w.miss[l] : 0.0, 0.0), p.active[l]);
  }
  return p;
}

// ------------------------------------------------------------------ estimator
struct Estimator::RatesAtShare {
  double share;
  double attn_flops, attn_bytes, dense_flops, dense_bytes, host_flops, host_bytes;
  double hbm_flops[4], hbm_bytes[4], hbm_q[4];   // by row-block height 16, 32, 64, 128
  double link_rate, stretch_attn;
};

Estimator::Estimator(const ModelShape& m, const Calibration& c, EstimatorOptions o) : model_(m), cal_(c), opt_(o) {
  if (cal_.sms <= 0) throw std::runtime_error("monofab: the calibration has no SM count");
  q_link_ = cal_.saturating_credits();
  x_max_ = cal_.exposure_bound();
  stretch_max_ = cal_.stretch.empty() ? 1.0 : std::max(1.0, cal_.stretch(x_max_));
  expert_bytes_ = model_.expert_bytes();
  if (cal_.one_pass_row_bytes >= 0) {
    one_pass_row_bytes_ = cal_.one_pass_row_bytes;
  } else {
    // The reference's weight-stationary kernel (csrc/control/estimator.cpp:30-34): fp32 partial sums of
    // w13 per K split (splits of at most eight 64-wide K tiles), the reduce's read and zeroing, its bf16
    // output, and the w2 partial sums per K split.
    auto splits = [](int k) { return std::max(1, (k / 64 + 7) / 8); };
    const double I = model_.intermediate, H = model_.hidden;
    one_pass_row_bytes_ = 8 * I * splits(model_.hidden) + 16 * I + 2 * I + 4 * H * splits(model_.intermediate);
  }
}

double Estimator::gamma_ratio(double own_exposure) const {
  if (!opt_.contention_aware || cal_.stretch.empty()) return 1.0;
  return std::max(1.0, stretch_max_ / std::max(1.0, cal_.stretch(own_exposure)));
}

void Estimator::observe(bool decode, bool moe, double ratio) {
  if (!(ratio > 0) || !std::isfinite(ratio)) return;
  double& c = correction_[decode][moe];
  c += opt_.ewma * (std::min(std::max(ratio, 0.25), 4.0) - c);
}

const KernelRates& Estimator::expert_kernel(int form) const {
  auto it = cal_.expert.find(form);
  if (it == cal_.expert.end()) it = cal_.expert.find(cal_.reference_form);
  if (it == cal_.expert.end()) throw std::runtime_error("monofab: the calibration has no sweep of the expert kernel");
  return it->second;
}

LaneLoad Estimator::load(const LaneWork& w) const {
  LaneLoad l;
  l.decode = w.decode;
  l.staging = w.staging;
  l.deadline = w.deadline;
  const size_t n = w.passes.size();
  for (size_t i = 0; i < n; ++i) l.passes.push_back(pass_load(model_, w, w.passes[i], i == 0, i + 1 == n));
  return l;
}

// One MoE window.  terms = {compute, stretched HBM reads, link}.
double Estimator::moe_window(const LaneLoad& l, const PassLoad& p, int layer, const RatesAtShare& r, double staged_cap,
                             int form, double& staged, double terms[3]) const {
  const double H = model_.hidden, I = model_.intermediate;
  const double active = p.active[layer], miss = p.miss[layer];
  // Experts the copy engine is sure to have staged during the attention window (Eq. 3 of the reference's paper).
  staged = l.staging > 0 ? std::min(std::min(miss, static_cast<double>(l.staging)), staged_cap) : 0.0;
  const double over_link = std::max(0.0, miss - staged);
  const double from_hbm = std::max(0.0, active - over_link);
  const double rows = active > 0 ? p.pairs / active : 0.0;   // expected rows of an activated expert
  const int h = hbm_block(rows);
  const int hi = h == 16 ? 0 : h == 32 ? 1 : h == 64 ? 2 : 3;
  int host_block = form;
  if (form == kOnePass) {
    host_block = 16;
    while (host_block < cal_.one_pass_rows && rows > host_block) host_block *= 2;
  }
  const double flops_per_row = 6.0 * H * I;
  // the HBM-expert and host-expert kernels share the lane's SMs: their times add
  terms[0] = time_for(from_hbm * flops_per_row * round_up_rows(rows, h) + p.shared_flops, r.hbm_flops[hi]) +
             time_for(over_link * flops_per_row * round_up_rows(rows, host_block), r.host_flops);
  const double passes_hbm = std::ceil(std::max(rows, 1.0) / h);
  const double partial_sums = form == kOnePass ? over_link * rows * one_pass_row_bytes_ : 0.0;
  const double reads = time_for(from_hbm * expert_bytes_ * passes_hbm + p.shared_bytes, r.hbm_bytes[hi]) +
                       time_for(p.moe_act_bytes, r.dense_bytes) + time_for(partial_sums, r.host_bytes);
  terms[1] = gamma_ratio(r.hbm_q[hi] * r.share * cal_.hbm_residency) * reads;
  const double link_rows = p.link_rows_bound > 0 ? p.link_rows_bound : rows;
  const double passes_link = form == kOnePass ? 1.0 : std::ceil(std::max(link_rows, 1.0) / form);
  terms[2] = time_for(over_link * expert_bytes_ * passes_link, r.link_rate);
  return std::max(terms[0], std::max(terms[1], terms[2])) * correction(l.decode, true);
}

Estimate Estimator::evaluate(const LaneLoad& l, int share, double credits, int form) const {
  RatesAtShare r;
  r.share = std::min(std::max(share, 1), cal_.sms);
  const KernelRates& attn = l.decode ? cal_.attn_decode : cal_.attn_prefill;
  r.attn_flops = attn.flops(r.share);
  r.attn_bytes = attn.bytes(r.share);
  r.dense_flops = cal_.dense.flops(r.share);
  r.dense_bytes = cal_.dense.bytes(r.share);
  const KernelRates& host = expert_kernel(form);
  r.host_flops = host.flops(r.share);
  r.host_bytes = host.bytes(r.share);
  for (int i = 0; i < 4; ++i) {
    const KernelRates& k = expert_kernel(16 << i);
    r.hbm_flops[i] = k.flops(r.share);
    r.hbm_bytes[i] = k.bytes(r.share);
    r.hbm_q[i] = k.q_per_sm;
  }
  // Credits the lane's SMs can keep in flight, capped by the grant; without the gate (the
  // contention-blind ablation) the streams keep their full depth.
  const double depth = cal_.credits_per_tile(form) * r.share;
  r.link_rate = cal_.rho(form, opt_.contention_aware ? std::min(depth, credits) : depth);
  const double granted_rate = cal_.rho(form, opt_.contention_aware ? credits : q_link_);
  r.stretch_attn = gamma_ratio(attn.q_per_sm * r.share * cal_.hbm_residency);

  Estimate e;
  double moe_sum = 0, staged_sum = 0;
  int moe_layers = 0;
  bool first_moe = true;
  for (size_t pi = 0; pi < l.passes.size(); ++pi) {
    const PassLoad& p = l.passes[pi];
    const double a_cmp = time_for(p.attn_flops, r.attn_flops) + time_for(p.proj_flops, r.dense_flops);
    const double a_rd = time_for(p.kv_bytes, r.attn_bytes) + time_for(p.proj_bytes, r.dense_bytes);
    const double t_attn = std::max(a_cmp, r.stretch_attn * a_rd) * correction(l.decode, false);
    if (pi == 0) {
      e.attn = t_attn;
      e.a_cmp = a_cmp;
      e.a_rd = a_rd;
    }
    const double staged_cap = std::floor(granted_rate * t_attn / std::max(expert_bytes_, 1.0));
    for (int layer = p.first_layer; layer < model_.layers; ++layer) {
      double t_moe;
      if (layer < model_.dense_layers) {
        t_moe = std::max(time_for(p.dense_mlp_flops, r.dense_flops),
                         gamma_ratio(r.hbm_q[3] * r.share * cal_.hbm_residency) * time_for(p.dense_mlp_bytes, r.dense_bytes));
      } else {
        double staged, terms[3];
        t_moe = moe_window(l, p, layer, r, staged_cap, form, staged, terms);
        if (pi == 0) {
          if (first_moe) {
            e.m_cmp = terms[0];
            e.m_rd = terms[1];
            e.m_link = terms[2];
            first_moe = false;
          }
          moe_sum += t_moe;
          staged_sum += staged;
          ++moe_layers;
        }
      }
      e.total += t_attn + t_moe + cal_.layer_overhead;
    }
    if (p.sampled > 0) {   // the vocabulary projection of the rows that are sampled
      const double H = model_.hidden;
      e.total += std::max(time_for(2.0 * p.sampled * H * model_.vocab, r.dense_flops),
                          time_for(H * model_.vocab * model_.dense_weight_bytes, r.dense_bytes)) + cal_.tail_overhead;
    }
  }
  if (moe_layers > 0) {
    e.moe = moe_sum / moe_layers;
    e.staged = staged_sum / moe_layers;
  }
  return e;
}

// ----------------------------------------------------------------- plan search
PlanSearch::PlanSearch(const Estimator* est, SearchOptions opt) : est_(est), opt_(std::move(opt)) {
  if (!est_) throw std::runtime_error("monofab: a plan search needs an estimator");
  if (opt_.forms.empty()) throw std::runtime_error("monofab: a plan search needs at least one kernel form");
}

std::vector<double> PlanSearch::grants(int form) const {
  const double budget = est_->link_credits();
  std::vector<double> out;
  const auto& curves = est_->calibration().link_rate;
  const auto it = curves.find(form);
  if (est_->options().contention_aware && it != curves.end())
    for (double x : it->second.x)
      if (x > 0 && x < budget * (1 - 1e-9)) out.push_back(x);
  out.push_back(budget);
  return out;
}

int PlanSearch::deadline_floor(const LaneLoad& l, double credits, int form, long* evals) const {
  const int all = est_->calibration().sms;
  auto in_time = [&](int share) {
    if (evals) ++*evals;
    return est_->evaluate(l, share, credits, form).total <= l.deadline;
  };
  if (!in_time(all)) return all + 1;
  if (in_time(1)) return 1;
  int miss = 1, meet = all;   // the estimate falls as the share grows: bisect the boundary
  while (meet - miss > 1) {
    const int mid = miss + (meet - miss) / 2;
    (in_time(mid) ? meet : miss) = mid;
  }
  return meet;
}

// Spare SMs go, a few at a time, to whichever lane has the least slack, as long as that lane's
// estimate still improves; what is left after every lane has stopped improving also goes to the
// tightest lane, because a share is a floor, not a fence.
void PlanSearch::pour_spare(const std::vector<LaneLoad>& lanes, Candidate& c, long& evals) const {
  const size_t n = lanes.size();
  c.est.resize(n);
  c.slack.resize(n);
  int spare = est_->calibration().sms;
  for (size_t b = 0; b < n; ++b) {
    c.est[b] = est_->evaluate(lanes[b], c.share[b], c.credits[b], c.form[b]);
    ++evals;
    c.slack[b] = relative_slack(lanes[b], c.est[b].total);
    spare -= c.share[b];
  }
  auto tightest = [&](const std::vector<char>& out) {
    int best = -1;
    for (size_t b = 0; b < n; ++b)
      if (!out[b] && (best < 0 || c.slack[b] < c.slack[best])) best = static_cast<int>(b);
    return best;
  };
  std::vector<char> saturated(n, 0);
  for (int b; spare > 0 && (b = tightest(saturated)) >= 0;) {
    const int add = std::min(opt_.pour_quantum, spare);
    const Estimate e = est_->evaluate(lanes[b], c.share[b] + add, c.credits[b], c.form[b]);
    ++evals;
    if (e.total < c.est[b].total * (1 - 1e-9)) {
      c.share[b] += add;
      spare -= add;
      c.est[b] = e;
      c.slack[b] = relative_slack(lanes[b], e.total);
    } else {
      saturated[b] = 1;
    }
  }
  if (spare > 0 && n > 0) c.share[tightest(std::vector<char>(n, 0))] += spare;
  c.min_slack = n ? *std::min_element(c.slack.begin(), c.slack.end()) : 0.0;
  c.total = 0;
  for (const Estimate& e : c.est) c.total += e.total;
}

// The candidate at whole link slots (at least one per lane, so no lane can stall on a host-resident
// expert), re-evaluated exactly and checked against the SM count and the two link budgets.
bool PlanSearch::settle(const std::vector<LaneLoad>& lanes, const Candidate& c, Plan& out, long& evals) const {
  const Calibration& cal = est_->calibration();
  out.lanes.assign(lanes.size(), LanePlan{});
  out.min_slack = lanes.empty() ? 0.0 : kNever;
  out.total_time = 0;
  int sms = 0;
  double credits = 0, rate = 0;
  bool ok = true;
  for (size_t b = 0; b < lanes.size(); ++b) {
    LanePlan& p = out.lanes[b];
    const double per_tile = cal.credits_per_tile(c.form[b]);
    p.form = c.form[b];
    p.sms = c.share[b];
    p.cap = std::max(1, static_cast<int>(std::floor(c.credits[b] / per_tile + 1e-9)));
    p.credits = p.cap * per_tile;
    p.est = est_->evaluate(lanes[b], p.sms, p.credits, p.form);
    ++evals;
    p.rate = cal.rho(p.form, p.credits);
    p.slack = relative_slack(lanes[b], p.est.total);
    ok = ok && p.est.total <= lanes[b].deadline;
    sms += p.sms;
    credits += p.credits;
    rate += p.rate;
    out.min_slack = std::min(out.min_slack, p.slack);
    out.total_time += p.est.total;
  }
  ok = ok && sms <= cal.sms;
  if (est_->options().contention_aware) {   // without the gate there is nothing to hold the grants to
    const double slot_rounding = cal.credits_per_tile(cal.reference_form) * lanes.size();
    ok = ok && credits <= est_->link_credits() * (1 + opt_.tolerance) + slot_rounding;
    ok = ok && rate <= cal.link_peak * (1 + opt_.tolerance);
  }
  out.copy_rate = std::max(0.0, cal.link_peak - rate);
  out.feasible = ok;
  return ok;
}

// No candidate meets every deadline: an even split of the credits with all SMs poured, marked infeasible.
Plan PlanSearch::fallback(const std::vector<LaneLoad>& lanes, const std::vector<Option>& decode_options, long& evals) const {
  const size_t n = lanes.size();
  Candidate c;
  c.form.assign(n, est_->calibration().reference_form);
  c.credits.assign(n, est_->link_credits() / std::max<size_t>(n, 1));
  c.share.assign(n, 1);
  if (n && lanes[0].decode && !decode_options.empty()) c.form[0] = decode_options.front().form;
  pour_spare(lanes, c, evals);
  Plan out;
  settle(lanes, c, out, evals);
  out.feasible = false;
  return out;
}

Plan PlanSearch::solve(const std::vector<LaneLoad>& lanes, unsigned long long decode_key) {
  const auto started = std::chrono::steady_clock::now();
  long evals = 0;
  const Calibration& cal = est_->calibration();
  const int all = cal.sms;
  const double budget = est_->link_credits();
  const size_t n = lanes.size();
  const bool with_decode = n > 0 && lanes[0].decode;
  const size_t p0 = with_decode ? 1 : 0, n_prefill = n - p0;
  for (size_t b = p0; b < n; ++b)
    if (lanes[b].decode) throw std::runtime_error("monofab: the decode lane must be the first lane of a plan");
  if (n_prefill > 2) throw std::runtime_error("monofab: a plan has at most two prefill lanes");
  auto done = [&](Plan p) {
    p.evaluations = evals;
    p.micros = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - started).count();
    return p;
  };
  if (n == 0) {
    Plan p;
    p.feasible = true;
    p.copy_rate = cal.link_peak;
    return done(p);
  }

  // The decode lane first: every (form, grant) that can meet its deadline, cheapest share first, then
  // fewest credits.  Remembered under the caller's key until the batch's composition changes.
  std::vector<Option> decode_options;
  if (with_decode) {
    const auto hit = decode_key ? decode_cache_.find(decode_key) : decode_cache_.end();
    if (hit != decode_cache_.end()) {
      decode_options = hit->second;
    } else {
      for (int form : opt_.forms)
        for (double q : grants(form)) {
          const int floor = deadline_floor(lanes[0], q, form, &evals);
          if (floor <= all) decode_options.push_back(Option{form, q, floor});
        }
      std::sort(decode_options.begin(), decode_options.end(), [](const Option& a, const Option& b) {
        return std::tie(a.floor, a.credits) < std::tie(b.floor, b.credits);
      });
      if (decode_key) {
        if (decode_cache_.size() > 256) decode_cache_.clear();
        decode_cache_[decode_key] = decode_options;
      }
    }
    if (decode_options.empty()) return done(fallback(lanes, decode_options, evals));
  }

  std::map<std::tuple<size_t, int, long long>, int> floors;   // deadline floors of the prefill lanes, memoised
  auto prefill_floor = [&](size_t b, int form, double q) {
    const auto key = std::make_tuple(b, form, std::llround(q * 1024));
    const auto it = floors.find(key);
    if (it != floors.end()) return it->second;
    return floors[key] = deadline_floor(lanes[b], q, form, &evals);
  };
  const bool gated = est_->options().contention_aware;
  const double rate_limit = cal.link_peak * (1 + opt_.tolerance);
  // A lane's estimate never grows with its grant and no other lane's depends on it, so a prefill lane
  // takes the largest grant that the credits left and the link rate left both allow.
  auto largest_grant = [&](int form, double credits_left, double rate_left) {
    if (!gated) return credits_left;
    const auto it = cal.link_rate.find(form);
    const double by_rate = it == cal.link_rate.end() ? 0.0 : it->second.last_within(rate_left);
    return std::max(0.0, std::min(credits_left, by_rate));
  };

  const size_t attempts = with_decode ? std::min<size_t>(decode_options.size(), std::max(1, opt_.decode_choices)) : 1;
  for (size_t attempt = 0; attempt < attempts; ++attempt) {
    Candidate seed;
    seed.form.assign(n, cal.reference_form);
    seed.credits.assign(n, 0.0);
    seed.share.assign(n, 0);
    double credits_left = budget;
    if (with_decode) {
      const Option& d = decode_options[attempt];
      seed.form[0] = d.form;
      if (n_prefill == 0) {   // alone, the decode lane gets the whole budget
        seed.credits[0] = budget;
        seed.share[0] = std::min(d.floor, prefill_floor(0, d.form, budget));
      } else {
        seed.credits[0] = d.credits;
        seed.share[0] = d.floor;
      }
      credits_left = std::max(0.0, budget - seed.credits[0]);
    }
    const double decode_rate = with_decode ? cal.rho(seed.form[0], seed.credits[0]) : 0.0;

    std::vector<Candidate> pool;
    auto consider = [&](Candidate c) {
      int sms = 0;
      double rate = 0;
      for (size_t b = 0; b < n; ++b) {
        if (c.share[b] > all) return;
        sms += c.share[b];
        rate += cal.rho(c.form[b], c.credits[b]);
      }
      if (sms > all || (gated && rate > rate_limit)) return;
      c.spare = all - sms;
      pool.push_back(std::move(c));
    };
    if (n_prefill == 0) {
      consider(seed);
    } else if (n_prefill == 1) {
      for (int form : opt_.forms) {
        Candidate c = seed;
        c.form[p0] = form;
        c.credits[p0] = largest_grant(form, credits_left, rate_limit - decode_rate);
        c.share[p0] = prefill_floor(p0, form, c.credits[p0]);
        consider(std::move(c));
      }
    } else {
      for (int f1 : opt_.forms)
        for (int f2 : opt_.forms)
          for (double q1 : grants(f1)) {
            if (q1 > credits_left * (1 + 1e-9)) continue;
            const double rate_left = rate_limit - decode_rate - (gated ? cal.rho(f1, q1) : 0.0);
            if (rate_left < 0) continue;
            Candidate c = seed;
            c.form[p0] = f1;
            c.form[p0 + 1] = f2;
            c.credits[p0] = q1;
            c.credits[p0 + 1] = largest_grant(f2, credits_left - q1, rate_left);
            c.share[p0] = prefill_floor(p0, f1, q1);
            if (c.share[p0] > all) continue;
            c.share[p0 + 1] = prefill_floor(p0 + 1, f2, c.credits[p0 + 1]);
            consider(std::move(c));
          }
    }
    if (pool.empty()) continue;   // try the decode lane's next option

    // Pour into the candidates with the most spare SMs; keep the largest minimum slack, ties broken by
    // the smallest total estimated time.
    std::stable_sort(pool.begin(), pool.end(), [](const Candidate& a, const Candidate& b) { return a.spare > b.spare; });
    if (pool.size() > static_cast<size_t>(opt_.pour_candidates)) pool.resize(opt_.pour_candidates);
    for (Candidate& c : pool) pour_spare(lanes, c, evals);
    std::stable_sort(pool.begin(), pool.end(), [](const Candidate& a, const Candidate& b) {
      if (std::abs(a.min_slack - b.min_slack) > 1e-12) return a.min_slack > b.min_slack;
      return a.total < b.total;
    });
    for (const Candidate& c : pool) {
      Plan out;
      if (settle(lanes, c, out, evals)) return done(out);
    }
  }
  return done(fallback(lanes, decode_options, evals));
}

}  // namespace plan
}  // namespace mf

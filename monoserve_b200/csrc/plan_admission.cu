// Host code only: the activation-profile view and admission (plan_admission.h).
#include "plan_admission.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <limits>

namespace mf {
namespace plan {

// ------------------------------------------------------------------ ProfileView
ProfileView::ProfileView(int layers, int experts) : layers_(layers), experts_(experts) {
  if (layers <= 0 || experts <= 0) throw std::runtime_error("monofab: a profile needs layers and experts");
  const size_t n = static_cast<size_t>(layers) * experts;
  shares_[0].assign(n, 1.0 / experts);
  shares_[1] = shares_[0];
  hot_.assign(n, 0);
  tabulate(0);
  tabulate(1);
}

void ProfileView::set_profile(bool decode, const std::vector<double>& shares) {
  if (shares.size() != shares_[0].size()) throw std::runtime_error("monofab: the profile must hold layers x experts shares");
  shares_[decode] = shares;
  tabulate(decode);
}

void ProfileView::set_hot(const std::vector<uint8_t>& hot) {
  if (hot.size() != hot_.size()) throw std::runtime_error("monofab: the hot-tier mask must hold layers x experts flags");
  hot_ = hot;
  tabulate(0);
  tabulate(1);
}

void ProfileView::tabulate(int which) {
  active_[which].assign(static_cast<size_t>(layers_) * kGrid, 0.0);
  missing_[which].assign(static_cast<size_t>(layers_) * kGrid, 0.0);
  for (int l = 0; l < layers_; ++l)
    for (int g = 0; g < kGrid; ++g) {
      const double rows = std::exp2(0.5 * g);
      double on_total = 0, on_cold = 0;
      for (int e = 0; e < experts_; ++e) {
        const size_t at = static_cast<size_t>(l) * experts_ + e;
        const double p = std::min(std::max(shares_[which][at], 0.0), 1.0);
        const double on = p >= 1.0 ? 1.0 : -std::expm1(rows * std::log1p(-p));   // 1 - (1 - p)^rows
        on_total += on;
        if (!hot_[at]) on_cold += on;
      }
      active_[which][static_cast<size_t>(l) * kGrid + g] = on_total;
      missing_[which][static_cast<size_t>(l) * kGrid + g] = on_cold;
    }
}

std::pair<double, double> ProfileView::expected(bool decode, int layer, double pairs) const {
  if (pairs <= 0 || layer < 0 || layer >= layers_) return {0.0, 0.0};
  const double* a = &active_[decode][static_cast<size_t>(layer) * kGrid];
  const double* m = &missing_[decode][static_cast<size_t>(layer) * kGrid];
  if (pairs <= 1) return {a[0] * pairs, m[0] * pairs};
  const double x = 2.0 * std::log2(pairs);
  if (x >= kGrid - 1) return {a[kGrid - 1], m[kGrid - 1]};
  const int g = static_cast<int>(x);
  const double f = x - g;
  return {a[g] + f * (a[g + 1] - a[g]), m[g] + f * (m[g + 1] - m[g])};
}

// -------------------------------------------------------------------- Admission
Admission::Admission(const Estimator* est, PlanSearch* search, const ProfileView* profile, AdmissionConfig cfg)
    : est_(est), search_(search), profile_(profile), cfg_(cfg) {
  if (!est_ || !search_ || !profile_) throw std::runtime_error("monofab: admission needs an estimator, a search and a profile");
  if (cfg_.max_prefill_lanes < 1 || cfg_.max_prefill_lanes > 2) throw std::runtime_error("monofab: admission runs one or two prefill lanes");
  lanes_.resize(cfg_.max_prefill_lanes);
  decode_key_ = next_key_++;
}

int Admission::open_lanes() const {
  return static_cast<int>(std::count_if(lanes_.begin(), lanes_.end(), [](const PrefillLane& l) { return l.open; }));
}

double Admission::ttft_deadline(int64_t id) const {
  const Request& r = entries_.at(id).r;
  return r.arrival + r.ttft;
}

void Admission::sort_queue_by_deadline() {
  std::stable_sort(queue_.begin(), queue_.end(), [&](int64_t a, int64_t b) { return ttft_deadline(a) < ttft_deadline(b); });
}

bool Admission::fits_memory(const std::vector<int64_t>& ids) const {
  double kv = kv_reserved_;
  for (int64_t id : ids) kv += kv_need(entries_.at(id).r);
  if (cfg_.kv_capacity > 0 && kv > cfg_.kv_capacity) return false;
  return !(cfg_.workspace_capacity > 0 && (open_lanes() + 1) * cfg_.lane_workspace > cfg_.workspace_capacity);
}

std::vector<const Admission::PrefillLane*> Admission::open_in_order() const {
  std::vector<const PrefillLane*> out;
  for (int i : open_order_) out.push_back(&lanes_[i]);
  return out;
}

// The decode lane's next step: one token per request on top of what it has cached; the tightest TPOT
// is the lane's deadline; expected activations come from the decode profile at batch x top-k rows.
LaneWork Admission::decode_work(const std::vector<int64_t>& ids) const {
  LaneWork w;
  w.decode = true;
  w.deadline = std::numeric_limits<double>::infinity();
  std::vector<Seq> step;
  for (int64_t id : ids) {
    const Entry& e = entries_.at(id);
    Seq s;
    s.tokens = 1;
    s.context = e.r.prompt + std::max(e.generated, 1) - 1;
    step.push_back(s);
    w.deadline = std::min(w.deadline, e.r.tpot);
  }
  w.passes.push_back(std::move(step));
  const ModelShape& m = est_->model();
  for (int l = 0; l < m.layers; ++l) {
    const auto on = profile_->expected(true, l, static_cast<double>(ids.size()) * m.top_k);
    w.active.push_back(on.first);
    w.miss.push_back(on.second);
  }
  return w;
}

// What a prefill lane still has to run: its current pass from the layer it has reached, then its later passes.
LaneWork Admission::prefill_work(const PrefillLane& lane, double now) const {
  LaneWork w;
  w.staging = cfg_.staging_experts;
  w.first_layer = lane.layers_done;
  w.deadline = lane.deadline - now;
  double rows_now = 0;
  for (size_t i = lane.pass; i < lane.passes.size(); ++i) {
    const PassSpec& p = lane.passes[i];
    std::vector<Seq> seqs(p.reqs.size());
    for (size_t k = 0; k < seqs.size(); ++k) {
      seqs[k].tokens = p.tokens[k];
      seqs[k].context = p.pos0[k];
      if (i == lane.pass) rows_now += p.tokens[k];
    }
    w.passes.push_back(std::move(seqs));
  }
  const ModelShape& m = est_->model();
  for (int l = 0; l < m.layers; ++l) {
    const auto on = profile_->expected(false, l, rows_now * m.top_k);
    w.active.push_back(on.first);
    w.miss.push_back(on.second);
  }
  return w;
}

// A sealed batch is one pass; a single prompt beyond the token budget runs as the fewest even chunks
// that fit it (chunking only bounds activation memory: every chunk streams nearly the whole expert set).
std::vector<PassSpec> Admission::passes_for(const std::vector<int64_t>& ids) const {
  std::vector<PassSpec> out;
  const int first_prompt = entries_.at(ids[0]).r.prompt;
  if (ids.size() == 1 && first_prompt > cfg_.token_budget) {
    const int pieces = (first_prompt + cfg_.token_budget - 1) / cfg_.token_budget;
    const int chunk = (first_prompt + pieces - 1) / pieces;
    for (int at = 0; at < first_prompt; at += chunk) {
      const int n = std::min(chunk, first_prompt - at);
      PassSpec p;
      p.reqs.push_back(ids[0]);
      p.tokens.push_back(n);
      p.pos0.push_back(at);
      p.last.push_back(at + n == first_prompt);
      out.push_back(std::move(p));
    }
    return out;
  }
  PassSpec p;
  for (int64_t id : ids) {
    p.reqs.push_back(id);
    p.tokens.push_back(entries_.at(id).r.prompt);
    p.pos0.push_back(0);
    p.last.push_back(1);
  }
  out.push_back(std::move(p));
  return out;
}

Plan Admission::search(const std::vector<int64_t>& decode, const std::vector<const PrefillLane*>& prefill, double now,
                       unsigned long long key, Decision& d) {
  std::vector<LaneLoad> loads;
  if (!decode.empty()) loads.push_back(est_->load(decode_work(decode)));
  for (const PrefillLane* l : prefill) loads.push_back(est_->load(prefill_work(*l, now)));
  ++d.searches;
  return search_->solve(loads, decode.empty() ? 0 : key);
}

void Admission::admit_joiners(double now, Decision& d, Plan& plan, bool& have_plan, bool& changed) {
  if (joiners_.empty() || decode_.size() >= static_cast<size_t>(cfg_.max_decode)) return;
  for (size_t take = std::min(joiners_.size(), cfg_.max_decode - decode_.size()); take > 0; take /= 2) {
    std::vector<int64_t> batch = decode_;
    batch.insert(batch.end(), joiners_.begin(), joiners_.begin() + static_cast<long>(take));
    const unsigned long long key = next_key_++;
    Plan p = search(batch, open_in_order(), now, key, d);
    if (!p.feasible) continue;
    for (size_t i = 0; i < take; ++i) {
      entries_.at(joiners_.front()).stage = Stage::kDecode;
      d.joined.push_back(joiners_.front());
      joiners_.pop_front();
    }
    decode_ = std::move(batch);
    decode_key_ = key;
    d.decode_changed = true;
    plan = std::move(p);
    have_plan = changed = true;
    return;
  }
}

void Admission::open_prefill_lanes(double now, Decision& d, Plan& plan, bool& have_plan, bool& changed) {
  while (!queue_.empty()) {
    const auto free_lane = std::find_if(lanes_.begin(), lanes_.end(), [](const PrefillLane& l) { return !l.open; });
    if (free_lane == lanes_.end()) return;
    const int index = static_cast<int>(free_lane - lanes_.begin());
    sort_queue_by_deadline();
    std::vector<int64_t> prefix;
    int tokens = 0;
    for (int64_t id : queue_) {
      const int prompt = entries_.at(id).r.prompt;
      if (prefix.empty() && prompt > cfg_.token_budget) {   // a long prompt goes alone, chunked
        prefix.push_back(id);
        break;
      }
      if (tokens + prompt > cfg_.token_budget || prefix.size() >= static_cast<size_t>(cfg_.max_batch_requests)) break;
      prefix.push_back(id);
      tokens += prompt;
    }
    bool opened = false;
    size_t size = prefix.size();
    for (int trial = 0; trial < cfg_.batch_trials && size > 0 && !opened; ++trial, size = std::max<size_t>(1, size / 2)) {
      const std::vector<int64_t> batch(prefix.begin(), prefix.begin() + static_cast<long>(size));
      if (fits_memory(batch)) {
        PrefillLane lane;
        lane.open = true;
        lane.reqs = batch;
        lane.passes = passes_for(batch);
        lane.deadline = std::numeric_limits<double>::infinity();
        for (int64_t id : batch) lane.deadline = std::min(lane.deadline, ttft_deadline(id));
        std::vector<const PrefillLane*> with = open_in_order();
        with.push_back(&lane);
        Plan p = search(decode_, with, now, decode_key_, d);
        if (p.feasible) {
          for (int64_t id : batch) {
            Entry& e = entries_.at(id);
            e.stage = Stage::kPrefill;
            kv_reserved_ += kv_need(e.r);
            queue_.erase(std::find(queue_.begin(), queue_.end(), id));
          }
          lanes_[index] = std::move(lane);
          open_order_.push_back(index);
          d.pass_lanes.push_back(index + 1);
          d.passes.push_back(lanes_[index].passes[0]);
          plan = std::move(p);
          have_plan = changed = opened = true;
        }
      }
      if (size == 1) break;
    }
    if (!opened) return;
  }
}

void Admission::reject_hopeless(double now, Decision& d) {
  if (queue_.empty() || cfg_.reject_checks <= 0) return;
  double lanes_free_at = now;
  for (const PrefillLane& l : lanes_)
    if (l.open) lanes_free_at = std::max(lanes_free_at, l.expected_end);
  sort_queue_by_deadline();
  int checked = 0;
  for (size_t i = 0; i < queue_.size() && checked < cfg_.reject_checks;) {
    const int64_t id = queue_[i];
    const double deadline = ttft_deadline(id);
    bool hopeless = deadline <= lanes_free_at;
    if (!hopeless) {   // alone in a prefill lane beside the decode lane, with the time left once the lanes are free
      PrefillLane alone;
      alone.open = true;
      alone.reqs.push_back(id);
      alone.passes = passes_for(alone.reqs);
      alone.deadline = deadline;
      hopeless = !search(decode_, {&alone}, lanes_free_at, decode_key_, d).feasible;
      ++checked;
    }
    if (hopeless) {
      d.rejected.push_back(id);
      entries_.erase(id);
      queue_.erase(queue_.begin() + static_cast<long>(i));
    } else {
      ++i;
    }
  }
}

Decision Admission::decide(double now, bool changed) {
  const auto started = std::chrono::steady_clock::now();
  Decision d;
  Plan plan;
  bool have_plan = false;
  admit_joiners(now, d, plan, have_plan, changed);
  open_prefill_lanes(now, d, plan, have_plan, changed);
  reject_hopeless(now, d);
  if (changed && !have_plan) plan = search(decode_, open_in_order(), now, decode_key_, d);
  if (changed) {
    d.publish = true;
    d.feasible = plan.feasible;
    if (!decode_.empty()) d.lanes.push_back(0);
    for (int i : open_order_) d.lanes.push_back(i + 1);
    for (size_t i = 0; i < d.lanes.size() && i < plan.lanes.size(); ++i)
      if (d.lanes[i] > 0) lanes_[d.lanes[i] - 1].expected_end = now + plan.lanes[i].est.total;
    d.plan = std::move(plan);
  }
  d.decode = decode_;
  d.micros = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - started).count();
  return d;
}

Decision Admission::arrive(const Request& r, double now) {
  if (entries_.count(r.id)) throw std::runtime_error("monofab: a request with this id is already known");
  Entry e;
  e.r = r;
  entries_.emplace(r.id, e);
  queue_.push_back(r.id);
  return decide(now, false);
}

Decision Admission::pass_done(int lane, double now) {
  if (lane < 1 || lane > static_cast<int>(lanes_.size()) || !lanes_[lane - 1].open)
    throw std::runtime_error("monofab: pass_done names a prefill lane that is not open");
  PrefillLane& l = lanes_[lane - 1];
  if (l.pass + 1 < l.passes.size()) {   // a chunked prompt: its next chunk starts at once
    ++l.pass;
    l.layers_done = 0;
    Decision d = decide(now, true);
    d.pass_lanes.insert(d.pass_lanes.begin(), lane);
    d.passes.insert(d.passes.begin(), lanes_[lane - 1].passes[lanes_[lane - 1].pass]);
    return d;
  }
  // the prompts are done and their first tokens are out: they wait to join the decode batch
  for (int64_t id : l.reqs) {
    const auto it = entries_.find(id);
    if (it == entries_.end()) continue;
    if (it->second.stage == Stage::kPrefill) {
      it->second.stage = Stage::kWaitingToJoin;
      it->second.generated = std::max(it->second.generated, 1);
      joiners_.push_back(id);
    } else if (it->second.stage == Stage::kGone) {
      entries_.erase(it);
    }
  }
  l = PrefillLane{};
  open_order_.erase(std::remove(open_order_.begin(), open_order_.end(), lane - 1), open_order_.end());
  return decide(now, true);
}

Decision Admission::finished(int64_t id, double now) {
  const auto it = entries_.find(id);
  if (it == entries_.end()) return Decision{};
  Entry& e = it->second;
  auto drop = [&](auto& list) { list.erase(std::remove(list.begin(), list.end(), id), list.end()); };
  const bool left_decode = e.stage == Stage::kDecode;
  if (left_decode) {
    drop(decode_);
    decode_key_ = next_key_++;
  } else if (e.stage == Stage::kWaitingToJoin) {
    drop(joiners_);
  } else if (e.stage == Stage::kQueued) {
    drop(queue_);
  }
  if (e.stage == Stage::kDecode || e.stage == Stage::kWaitingToJoin || e.stage == Stage::kPrefill)
    kv_reserved_ = std::max(0.0, kv_reserved_ - kv_need(e.r));
  if (e.stage == Stage::kPrefill) e.stage = Stage::kGone;   // its lane's pass still runs; pass_done forgets it
  else entries_.erase(it);
  Decision d = decide(now, left_decode);
  d.decode_changed = d.decode_changed || left_decode;
  return d;
}

Decision Admission::behind(int, double now) { return decide(now, true); }

void Admission::progress(int lane, int layers_done) {
  if (lane >= 1 && lane <= static_cast<int>(lanes_.size())) lanes_[lane - 1].layers_done = layers_done;
}

void Admission::generated(int64_t id, int tokens) {
  const auto it = entries_.find(id);
  if (it != entries_.end()) it->second.generated = tokens;
}

}  // namespace plan
}  // namespace mf

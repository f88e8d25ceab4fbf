// Admission: what runs after each serving event (a request arrives, a prefill pass ends, a
// request produces its last token, a lane falls behind its plan).  Every decision is a small
// number of plan searches, one per candidate set of lanes.
//
// The policy is the reference's (csrc/control/admission.h:1-161, admission.cpp:226-448):
//   * decode first: requests whose prompt is done join the decode batch if a re-solved plan
//     still keeps every deadline (all waiting ones, else half of them, and so on), and wait
//     otherwise;
//   * then prefill: the queue in deadline order is cut into a batch under the token budget; the
//     largest prefix (whole, half, quarter ...) whose plan is feasible and whose KV reservation
//     fits opens a free prefill lane and is sealed; a prompt longer than the budget goes alone,
//     in a few even chunks;
//   * a queued request is rejected only if no plan could meet its deadline even alone, after
//     every open prefill lane has finished;
//   * whenever the lane set changed, its plan is (re)published.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <utility>
#include <vector>

#include "plan_model.h"

namespace mf {
namespace plan {

// Expected numbers of activated experts per layer for a number of routed rows, from per-layer
// activation shares and the hot-tier mask (csrc/control/admission.h:26-49).  An expert with
// share p is activated by n independent rows with probability 1 - (1 - p)^n; the expectation
// is tabulated on a grid n = 2^(i/2) and interpolated in log2 n.
class ProfileView {
 public:
  ProfileView(int layers, int experts);
  void set_profile(bool decode, const std::vector<double>& shares);   // [layers * experts]
  void set_hot(const std::vector<uint8_t>& hot);                      // [layers * experts], 1 = in the hot tier
  // (activated, of those outside the hot tier)
  std::pair<double, double> expected(bool decode, int layer, double pairs) const;
  int layers() const { return layers_; }
  int experts() const { return experts_; }

 private:
  static constexpr int kGrid = 49;
  void tabulate(int which);
  int layers_, experts_;
  std::vector<double> shares_[2];
  std::vector<uint8_t> hot_;
  std::vector<double> active_[2], missing_[2];   // [layer][grid point]
};

struct Request {
  int64_t id = 0;
  int prompt = 0, max_output = 1;
  double arrival = 0, ttft = 0, tpot = 0;
};

struct AdmissionConfig {
  int max_prefill_lanes = 2, token_budget = 16384, max_batch_requests = 64, max_decode = 256, staging_experts = 0;
  double kv_capacity = 0, kv_bytes_per_token = 0, workspace_capacity = 0, lane_workspace = 0;
  int batch_trials = 4, reject_checks = 2;
};

struct PassSpec {   // one prefill pass: per request the tokens it computes, where they start, and whether the prompt ends here
  std::vector<int64_t> reqs;
  std::vector<int> tokens, pos0;
  std::vector<uint8_t> last;
};

struct Decision {
  bool publish = false, feasible = true, decode_changed = false;
  Plan plan;
  std::vector<int> lanes;        // fabric lane of plan.lanes[i] (0 = decode)
  std::vector<int64_t> decode, joined, rejected;
  std::vector<int> pass_lanes;   // prefill passes to start: the lane ...
  std::vector<PassSpec> passes;  // ... and its pass
  int searches = 0;
  double micros = 0;
};

class Admission {
 public:
  Admission(const Estimator* est, PlanSearch* search, const ProfileView* profile, AdmissionConfig cfg);
  Decision arrive(const Request& r, double now);
  Decision pass_done(int lane, double now);
  Decision finished(int64_t id, double now);
  Decision behind(int lane, double now);
  void progress(int lane, int layers_done);
  void generated(int64_t id, int tokens);
  size_t queued() const { return queue_.size(); }
  size_t waiting() const { return joiners_.size(); }
  int open_lanes() const;
  double kv_reserved() const { return kv_reserved_; }

 private:
  enum class Stage { kQueued, kPrefill, kWaitingToJoin, kDecode, kGone };
  struct Entry {
    Request r;
    Stage stage = Stage::kQueued;
    int generated = 0;
  };
  struct PrefillLane {
    bool open = false;
    std::vector<int64_t> reqs;
    std::vector<PassSpec> passes;
    size_t pass = 0;
    int layers_done = 0;
    double deadline = 0, expected_end = 0;   // absolute seconds
  };
  Decision decide(double now, bool lanes_changed);
  void admit_joiners(double now, Decision& d, Plan& plan, bool& have_plan, bool& changed);
  void open_prefill_lanes(double now, Decision& d, Plan& plan, bool& have_plan, bool& changed);
  void reject_hopeless(double now, Decision& d);
  Plan search(const std::vector<int64_t>& decode, const std::vector<const PrefillLane*>& prefill, double now,
              unsigned long long key, Decision& d);
  std::vector<const PrefillLane*> open_in_order() const;
  LaneWork decode_work(const std::vector<int64_t>& ids) const;
  LaneWork prefill_work(const PrefillLane& lane, double now) const;
  std::vector<PassSpec> passes_for(const std::vector<int64_t>& ids) const;
  double kv_need(const Request& r) const { return (static_cast<double>(r.prompt) + (r.max_output > 1 ? r.max_output : 1)) * cfg_.kv_bytes_per_token; }
  double ttft_deadline(int64_t id) const;
  bool fits_memory(const std::vector<int64_t>& ids) const;
  void sort_queue_by_deadline();

  const Estimator* est_;
  PlanSearch* search_;
  const ProfileView* profile_;
  AdmissionConfig cfg_;
  std::map<int64_t, Entry> entries_;
  std::vector<int64_t> queue_, decode_;
  std::deque<int64_t> joiners_;
  std::vector<PrefillLane> lanes_;   // fabric lane = index + 1
  std::vector<int> open_order_;      // open prefill lanes in plan order
  unsigned long long decode_key_, next_key_ = 1;
  double kv_reserved_ = 0;
};

}  // namespace plan
}  // namespace mf

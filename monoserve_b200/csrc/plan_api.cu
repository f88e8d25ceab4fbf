// C ABI of the control plane (include/monofab.h, "plans"): flat arrays of doubles in,
// flat arrays out, opaque handles in between.  The Python mirror
// (monoserve_b200/control.py) flattens its objects with the same layouts.
#include <cstring>
#include <memory>
#include <string>

#include "../../include/monofab.h"
#include "plan_model.h"

namespace mf {
int fail(int code, const char* fmt, ...);   // api.cu
}

using namespace mf::plan;
using mf::fail;

struct monofab_plan_estimator {
  std::unique_ptr<Estimator> est;
};
struct monofab_plan_load {
  LaneLoad load;
};
struct monofab_plan_search {
  std::unique_ptr<PlanSearch> search;
};

namespace {

// A cursor over a flat array of doubles that refuses to run off its end.
struct Reader {
  const double* p;
  int left;
  bool ok = true;
  double next() {
    if (left <= 0) {
      ok = false;
      return 0.0;
    }
    --left;
    return *p++;
  }
  int count(int limit = 1 << 20) {
    const double v = next();
    if (!(v >= 0) || v > limit) {
      ok = false;
      return 0;
    }
    return static_cast<int>(v);
  }
  Curve curve() {   // n, through_origin, x[n], y[n]
    Curve c;
    const int n = count();
    c.through_origin = next() != 0;
    for (int i = 0; i < n && ok; ++i) c.x.push_back(next());
    for (int i = 0; i < n && ok; ++i) c.y.push_back(next());
    for (size_t i = 1; i < c.x.size(); ++i)
      if (!(c.x[i] > c.x[i - 1])) ok = false;   // x must increase
    return c;
  }
  KernelRates rates() {   // flops curve, bytes curve, q_per_sm
    KernelRates k;
    k.flops = curve();
    k.bytes = curve();
    k.q_per_sm = next();
    return k;
  }
};

void put_estimate(const Estimate& e, double* out) {
  const double v[9] = {e.total, e.attn, e.moe, e.staged, e.a_cmp, e.a_rd, e.m_cmp, e.m_rd, e.m_link};
  std::memcpy(out, v, sizeof v);
}

template <class F>
int guarded(const char* what, F body) {
  try {
    return body();
  } catch (const std::exception& e) {
    return fail(MONOFAB_EINVAL, "%s: %s", what, e.what());
  }
}

}  // namespace

extern "C" {

double monofab_plan_curve_at(const double* x, const double* y, int n, int through_origin, double v) {
  if (!x || !y || n <= 0) return 0.0;
  Curve c;
  c.x.assign(x, x + n);
  c.y.assign(y, y + n);
  c.through_origin = through_origin != 0;
  return c(v);
}

int monofab_plan_estimator_create(const double* model, int n_model, const double* calibration, int n_calibration,
                                  int contention_aware, double ewma, monofab_plan_estimator** out) {
  if (!model || !calibration || !out) return fail(MONOFAB_EINVAL, "plan_estimator_create: NULL argument");
  if (n_model != MONOFAB_PLAN_MODEL_FIELDS) return fail(MONOFAB_EINVAL, "plan_estimator_create: the model takes %d fields, %d given", MONOFAB_PLAN_MODEL_FIELDS, n_model);
  return guarded("plan_estimator_create", [&] {
    ModelShape m;
    m.hidden = static_cast<int>(model[0]);
    m.intermediate = static_cast<int>(model[1]);
    m.experts = static_cast<int>(model[2]);
    m.top_k = static_cast<int>(model[3]);
    m.layers = static_cast<int>(model[4]);
    m.heads = static_cast<int>(model[5]);
    m.kv_heads = static_cast<int>(model[6]);
    m.head_dim = static_cast<int>(model[7]);
    m.vocab = static_cast<int>(model[8]);
    m.dense_layers = static_cast<int>(model[9]);
    m.dense_intermediate = static_cast<int>(model[10]);
    m.shared_intermediate = static_cast<int>(model[11]);
    m.expert_weight_bytes = model[12];
    m.dense_weight_bytes = model[13];
    if (m.layers < 0 || m.layers > 4096 || m.hidden <= 0 || m.intermediate <= 0 || m.experts <= 0)
      return fail(MONOFAB_EINVAL, "plan_estimator_create: bad model shape");
    Reader r{calibration, n_calibration};
    Calibration c;
    c.sms = static_cast<int>(r.next());
    c.hbm_residency = r.next();
    c.link_residency = r.next();
    c.q_max = r.next();
    c.link_peak = r.next();
    c.reference_form = static_cast<int>(r.next());
    c.layer_overhead = r.next();
    c.tail_overhead = r.next();
    c.one_pass_rows = static_cast<int>(r.next());
    c.one_pass_row_bytes = r.next();
    c.stretch = r.curve();
    c.dense = r.rates();
    c.attn_prefill = r.rates();
    c.attn_decode = r.rates();
    for (int i = 0, n = r.count(64); i < n && r.ok; ++i) {
      const int form = static_cast<int>(r.next());
      c.expert[form] = r.rates();
    }
    for (int i = 0, n = r.count(64); i < n && r.ok; ++i) {
      const int form = static_cast<int>(r.next());
      c.link_rate[form] = r.curve();
    }
    for (int i = 0, n = r.count(64); i < n && r.ok; ++i) {
      const int form = static_cast<int>(r.next());
      c.tile_credits[form] = r.next();
    }
    if (!r.ok || r.left != 0) return fail(MONOFAB_EINVAL, "plan_estimator_create: malformed calibration array");
    if (c.one_pass_rows < 16) c.one_pass_rows = 16;
    EstimatorOptions o;
    o.contention_aware = contention_aware != 0;
    o.ewma = ewma;
    auto* h = new monofab_plan_estimator();
    h->est.reset(new Estimator(m, c, o));
    *out = h;
    return MONOFAB_OK;
  });
}

int monofab_plan_estimator_destroy(monofab_plan_estimator* e) {
  delete e;
  return MONOFAB_OK;
}

int monofab_plan_estimator_info(monofab_plan_estimator* e, double out[4]) {
  if (!e || !out) return fail(MONOFAB_EINVAL, "plan_estimator_info: NULL argument");
  out[0] = e->est->link_credits();
  out[1] = e->est->exposure_bound();
  out[2] = e->est->model().expert_bytes();
  out[3] = e->est->model().kv_bytes_per_token();
  return MONOFAB_OK;
}

double monofab_plan_gamma_ratio(monofab_plan_estimator* e, double own_exposure) { return e ? e->est->gamma_ratio(own_exposure) : 1.0; }

int monofab_plan_observe(monofab_plan_estimator* e, int decode, int moe, double ratio) {
  if (!e) return fail(MONOFAB_EINVAL, "plan_observe: NULL handle");
  e->est->observe(decode != 0, moe != 0, ratio);
  return MONOFAB_OK;
}

double monofab_plan_correction(monofab_plan_estimator* e, int decode, int moe) { return e ? e->est->correction(decode != 0, moe != 0) : 1.0; }

int monofab_plan_load_create(monofab_plan_estimator* e, const double* work, int n_work, monofab_plan_load** out) {
  if (!e || !work || !out) return fail(MONOFAB_EINVAL, "plan_load_create: NULL argument");
  return guarded("plan_load_create", [&] {
    Reader r{work, n_work};
    LaneWork w;
    w.decode = r.next() != 0;
    w.first_layer = static_cast<int>(r.next());
    w.staging = static_cast<int>(r.next());
    w.deadline = r.next();
    w.samples = r.next() != 0;
    for (int i = 0, n = r.count(); i < n && r.ok; ++i) w.active.push_back(r.next());
    for (int i = 0, n = r.count(); i < n && r.ok; ++i) w.miss.push_back(r.next());
    for (int i = 0, n = r.count(); i < n && r.ok; ++i) {
      std::vector<Seq> seqs;
      for (int j = 0, k = r.count(); j < k && r.ok; ++j) {
        Seq s;
        s.tokens = static_cast<int>(r.next());
        s.context = static_cast<int>(r.next());
        seqs.push_back(s);
      }
      w.passes.push_back(std::move(seqs));
    }
    if (!r.ok || r.left != 0) return fail(MONOFAB_EINVAL, "plan_load_create: malformed work array");
    auto* h = new monofab_plan_load();
    h->load = e->est->load(w);
    *out = h;
    return MONOFAB_OK;
  });
}

int monofab_plan_load_destroy(monofab_plan_load* l) {
  delete l;
  return MONOFAB_OK;
}

int monofab_plan_evaluate(monofab_plan_estimator* e, const monofab_plan_load* l, int share, double credits, int form,
                          double out[MONOFAB_PLAN_ESTIMATE_FIELDS]) {
  if (!e || !l || !out) return fail(MONOFAB_EINVAL, "plan_evaluate: NULL argument");
  return guarded("plan_evaluate", [&] {
    put_estimate(e->est->evaluate(l->load, share, credits, form), out);
    return MONOFAB_OK;
  });
}

int monofab_plan_search_create(monofab_plan_estimator* e, const int32_t* forms, int n_forms, int pour_quantum,
                               int pour_candidates, int decode_choices, double tolerance, monofab_plan_search** out) {
  if (!e || !out || (n_forms > 0 && !forms)) return fail(MONOFAB_EINVAL, "plan_search_create: NULL argument");
  return guarded("plan_search_create", [&] {
    SearchOptions o;
    if (n_forms > 0) o.forms.assign(forms, forms + n_forms);
    if (pour_quantum > 0) o.pour_quantum = pour_quantum;
    if (pour_candidates > 0) o.pour_candidates = pour_candidates;
    if (decode_choices > 0) o.decode_choices = decode_choices;
    if (tolerance >= 0) o.tolerance = tolerance;
    auto* h = new monofab_plan_search();
    h->search.reset(new PlanSearch(e->est.get(), o));
    *out = h;
    return MONOFAB_OK;
  });
}

int monofab_plan_search_destroy(monofab_plan_search* s) {
  delete s;
  return MONOFAB_OK;
}

int monofab_plan_deadline_floor(monofab_plan_search* s, const monofab_plan_load* l, double credits, int form, int* share) {
  if (!s || !l || !share) return fail(MONOFAB_EINVAL, "plan_deadline_floor: NULL argument");
  return guarded("plan_deadline_floor", [&] {
    *share = s->search->deadline_floor(l->load, credits, form, nullptr);
    return MONOFAB_OK;
  });
}

int monofab_plan_solve(monofab_plan_search* s, const monofab_plan_load* const* lanes, int n_lanes, uint64_t decode_key,
                       double* out, int out_cap) {
  if (!s || !out || (n_lanes > 0 && !lanes)) return fail(MONOFAB_EINVAL, "plan_solve: NULL argument");
  if (n_lanes < 0 || n_lanes > 3) return fail(MONOFAB_EINVAL, "plan_solve: %d lanes (at most one decode and two prefill lanes)", n_lanes);
  if (out_cap < MONOFAB_PLAN_HEADER_FIELDS + n_lanes * MONOFAB_PLAN_LANE_FIELDS) return fail(MONOFAB_EINVAL, "plan_solve: output array too small");
  return guarded("plan_solve", [&] {
    std::vector<LaneLoad> loads;
    for (int i = 0; i < n_lanes; ++i) {
      if (!lanes[i]) return fail(MONOFAB_EINVAL, "plan_solve: lane %d is NULL", i);
      loads.push_back(lanes[i]->load);
    }
    const Plan p = s->search->solve(loads, decode_key);
    out[0] = p.feasible;
    out[1] = static_cast<double>(p.lanes.size());
    out[2] = p.copy_rate;
    out[3] = p.min_slack;
    out[4] = p.total_time;
    out[5] = static_cast<double>(p.evaluations);
    out[6] = p.micros;
    out[7] = 0;
    double* q = out + MONOFAB_PLAN_HEADER_FIELDS;
    for (const LanePlan& l : p.lanes) {
      q[0] = l.sms;
      q[1] = l.credits;
      q[2] = l.form;
      q[3] = l.cap;
      q[4] = l.rate;
      q[5] = l.slack;
      put_estimate(l.est, q + 6);
      q += MONOFAB_PLAN_LANE_FIELDS;
    }
    return MONOFAB_OK;
  });
}

int monofab_plan_clear_cache(monofab_plan_search* s) {
  if (!s) return fail(MONOFAB_EINVAL, "plan_clear_cache: NULL handle");
  s->search->clear_cache();
  return MONOFAB_OK;
}

}  // extern "C"

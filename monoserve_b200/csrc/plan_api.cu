// C ABI of the control plane (include/monofab.h, "plans"): flat arrays of doubles in,
// flat arrays out, opaque handles in between.  The Python mirror
// (monoserve_b200/control.py) flattens its objects with the same layouts.
#include <cstring>
#include <memory>
#include <string>

#include "../../include/monofab.h"
#include "plan_admission.h"
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
struct monofab_plan_profile {
  std::unique_ptr<ProfileView> view;
};
struct monofab_plan_admission {
  std::unique_ptr<Admission> adm;
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

// header [8] + lanes x [15], as monofab_plan_solve lays a plan out
void put_plan(const Plan& p, double* out) {
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
    put_plan(s->search->solve(loads, decode_key), out);
    return MONOFAB_OK;
  });
}

int monofab_plan_clear_cache(monofab_plan_search* s) {
  if (!s) return fail(MONOFAB_EINVAL, "plan_clear_cache: NULL handle");
  s->search->clear_cache();
  return MONOFAB_OK;
}

int monofab_plan_profile_create(int layers, int experts, monofab_plan_profile** out) {
  if (!out) return fail(MONOFAB_EINVAL, "plan_profile_create: NULL argument");
  return guarded("plan_profile_create", [&] {
    auto* h = new monofab_plan_profile();
    h->view.reset(new ProfileView(layers, experts));
    *out = h;
    return MONOFAB_OK;
  });
}

int monofab_plan_profile_destroy(monofab_plan_profile* p) {
  delete p;
  return MONOFAB_OK;
}

int monofab_plan_profile_set(monofab_plan_profile* p, int decode, const double* shares, int n) {
  if (!p || !shares || n < 0) return fail(MONOFAB_EINVAL, "plan_profile_set: bad argument");
  return guarded("plan_profile_set", [&] {
    p->view->set_profile(decode != 0, std::vector<double>(shares, shares + n));
    return MONOFAB_OK;
  });
}

int monofab_plan_profile_set_hot(monofab_plan_profile* p, const uint8_t* hot, int n) {
  if (!p || !hot || n < 0) return fail(MONOFAB_EINVAL, "plan_profile_set_hot: bad argument");
  return guarded("plan_profile_set_hot", [&] {
    p->view->set_hot(std::vector<uint8_t>(hot, hot + n));
    return MONOFAB_OK;
  });
}

int monofab_plan_profile_expected(monofab_plan_profile* p, int decode, int layer, double pairs, double out[2]) {
  if (!p || !out) return fail(MONOFAB_EINVAL, "plan_profile_expected: NULL argument");
  const auto v = p->view->expected(decode != 0, layer, pairs);
  out[0] = v.first;
  out[1] = v.second;
  return MONOFAB_OK;
}

int monofab_plan_admission_create(monofab_plan_estimator* e, monofab_plan_search* s, monofab_plan_profile* p,
                                  const double* config, int n_config, monofab_plan_admission** out) {
  if (!e || !s || !p || !config || !out) return fail(MONOFAB_EINVAL, "plan_admission_create: NULL argument");
  if (n_config != MONOFAB_PLAN_ADMISSION_FIELDS) return fail(MONOFAB_EINVAL, "plan_admission_create: the configuration takes %d fields, %d given", MONOFAB_PLAN_ADMISSION_FIELDS, n_config);
  return guarded("plan_admission_create", [&] {
    AdmissionConfig c;
    c.max_prefill_lanes = static_cast<int>(config[0]);
    c.token_budget = static_cast<int>(config[1]);
    c.max_batch_requests = static_cast<int>(config[2]);
    c.max_decode = static_cast<int>(config[3]);
    c.staging_experts = static_cast<int>(config[4]);
    c.kv_capacity = config[5];
    c.kv_bytes_per_token = config[6];
    c.workspace_capacity = config[7];
    c.lane_workspace = config[8];
    c.batch_trials = static_cast<int>(config[9]);
    c.reject_checks = static_cast<int>(config[10]);
    auto* h = new monofab_plan_admission();
    h->adm.reset(new Admission(e->est.get(), s->search.get(), p->view.get(), c));
    *out = h;
    return MONOFAB_OK;
  });
}

int monofab_plan_admission_destroy(monofab_plan_admission* a) {
  delete a;
  return MONOFAB_OK;
}

int monofab_plan_admission_state(monofab_plan_admission* a, double out[4]) {
  if (!a || !out) return fail(MONOFAB_EINVAL, "plan_admission_state: NULL argument");
  out[0] = static_cast<double>(a->adm->queued());
  out[1] = static_cast<double>(a->adm->waiting());
  out[2] = a->adm->open_lanes();
  out[3] = a->adm->kv_reserved();
  return MONOFAB_OK;
}

int monofab_plan_admission_event(monofab_plan_admission* a, int kind, int64_t id, const double* args, int n_args,
                                 int64_t* out, int out_cap, int* out_n, double* plan, int plan_cap) {
  if (!a) return fail(MONOFAB_EINVAL, "plan_admission_event: NULL handle");
  auto arg = [&](int i) { return (args && i < n_args) ? args[i] : 0.0; };
  if (kind == MONOFAB_PLAN_EVENT_PROGRESS) {
    a->adm->progress(static_cast<int>(id), static_cast<int>(arg(0)));
    return MONOFAB_OK;
  }
  if (kind == MONOFAB_PLAN_EVENT_GENERATED) {
    a->adm->generated(id, static_cast<int>(arg(0)));
    return MONOFAB_OK;
  }
  if (!out || !out_n || !plan || plan_cap < MONOFAB_PLAN_HEADER_FIELDS + 3 * MONOFAB_PLAN_LANE_FIELDS)
    return fail(MONOFAB_EINVAL, "plan_admission_event: the decision needs output arrays");
  return guarded("plan_admission_event", [&] {
    Decision d;
    switch (kind) {
      case MONOFAB_PLAN_EVENT_ARRIVE: {
        Request r;
        r.id = id;
        r.prompt = static_cast<int>(arg(0));
        r.max_output = static_cast<int>(arg(1));
        r.arrival = arg(2);
        r.ttft = arg(3);
        r.tpot = arg(4);
        d = a->adm->arrive(r, arg(5));
        break;
      }
      case MONOFAB_PLAN_EVENT_PASS_DONE: d = a->adm->pass_done(static_cast<int>(id), arg(0)); break;
      case MONOFAB_PLAN_EVENT_FINISHED: d = a->adm->finished(id, arg(0)); break;
      case MONOFAB_PLAN_EVENT_BEHIND: d = a->adm->behind(static_cast<int>(id), arg(0)); break;
      default: return fail(MONOFAB_EINVAL, "plan_admission_event: unknown event %d", kind);
    }
    std::vector<int64_t> v = {d.publish, d.feasible, d.decode_changed, d.searches};
    auto list = [&](const auto& items) {
      v.push_back(static_cast<int64_t>(items.size()));
      for (auto x : items) v.push_back(static_cast<int64_t>(x));
    };
    list(d.lanes);
    list(d.decode);
    list(d.joined);
    list(d.rejected);
    v.push_back(static_cast<int64_t>(d.passes.size()));
    for (size_t i = 0; i < d.passes.size(); ++i) {
      const PassSpec& p = d.passes[i];
      v.push_back(d.pass_lanes[i]);
      v.push_back(static_cast<int64_t>(p.reqs.size()));
      for (size_t k = 0; k < p.reqs.size(); ++k) {
        v.push_back(p.reqs[k]);
        v.push_back(p.tokens[k]);
        v.push_back(p.pos0[k]);
        v.push_back(p.last[k]);
      }
    }
    if (static_cast<int>(v.size()) > out_cap) return fail(MONOFAB_EINVAL, "plan_admission_event: the decision needs %zu words, %d given", v.size(), out_cap);
    std::memcpy(out, v.data(), v.size() * sizeof(int64_t));
    *out_n = static_cast<int>(v.size());
    put_plan(d.plan, plan);
    plan[7] = d.micros;
    return MONOFAB_OK;
  });
}

}  // extern "C"

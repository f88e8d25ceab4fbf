"""The control plane over libmonofab's plan entry points: time estimator and plan search.

The classes keep the names, attributes and call signatures of the reference's
`monoserve._C.control` (csrc/control/py_control.cpp:10-254) and of the helpers in
monoserve/control/__init__.py and calibration.py, so the reference's control tests read
the same here; `as_native_module()` returns a module object with those names for
`monoserve._C.control`.  All arithmetic happens in the native library (host code); the
objects here only hold inputs and results and flatten them into the arrays the C ABI
takes (layouts in include/monofab.h).

"""
import ctypes
import json
import types

from monoserve_b200 import _C

ASYM = 0                      # the one-pass form ("asym" in the reference's calibration files)
FORMS = (16, 32, 64, 128, ASYM)
FORM_KEYS = {"16": 16, "32": 32, "64": 64, "128": 128, "asym": 0}


def _doubles(values):
    return (ctypes.c_double * len(values))(*values)


class Curve:
    """Piecewise-linear curve through measured points; Curve(x, y, origin=False)(v)."""

    def __init__(self, x=(), y=(), origin=False):
        self.x, self.y, self.origin = [float(v) for v in x], [float(v) for v in y], bool(origin)
        assert len(self.x) == len(self.y)

    def empty(self):
        return not self.x

    def __call__(self, v):
        return _C.lib.monofab_plan_curve_at(_doubles(self.x), _doubles(self.y), len(self.x), int(self.origin), float(v))

    at = __call__

    def _flat(self):
        return [float(len(self.x)), float(self.origin)] + self.x + self.y


class KernelRates:
    def __init__(self):
        self.flops, self.bytes, self.q_per_sm = Curve(), Curve(), 0.0

    def _flat(self):
        return self.flops._flat() + self.bytes._flat() + [float(self.q_per_sm)]


class ModelShape:
    _FIELDS = ("hidden", "intermediate", "experts", "top_k", "layers", "heads", "kv_heads", "head_dim", "vocab",
               "dense_layers", "dense_intermediate", "shared_intermediate", "expert_weight_bytes", "dense_weight_bytes")

    def __init__(self):
        for f in self._FIELDS:
            setattr(self, f, 0)
        self.head_dim, self.expert_weight_bytes, self.dense_weight_bytes = 128, 2.0, 2.0

    @property
    def expert_bytes(self):
        return 3.0 * self.hidden * self.intermediate * self.expert_weight_bytes

    @property
    def kv_bytes_per_token(self):
        return 2.0 * self.layers * self.kv_heads * self.head_dim * 2.0

    def _flat(self):
        return [float(getattr(self, f)) for f in self._FIELDS]


class Calibration:
    """Units as in the reference's struct: seconds, bytes/s, FLOP/s, credits."""

    def __init__(self):
        self.sms, self.R_H, self.R_C, self.q_max = 0, 0.0, 0.0, 0.0
        self.gamma = Curve()
        self.dense, self.attn_prefill, self.attn_decode = KernelRates(), KernelRates(), KernelRates()
        self.expert, self.rho, self.q_form = {}, {}, {}
        self.beta, self.reference_form = 0.0, 64
        self.layer_overhead, self.tail_overhead = 0.0, 0.0
        # the one-pass form in this library: 256-row blocks, partial sums stay in TMEM (no HBM traffic);
        # the defaults below are the reference's kernel (row blocks up to 64, K-split partial sums in HBM)
        self.one_pass_rows, self.one_pass_row_bytes = 64, -1.0

    def rho_at(self, form, credits):
        if form not in self.rho:
            raise RuntimeError("monofab: the calibration has no credit sweep for kernel form %d" % form)
        return self.rho[form](credits)

    def q_of(self, form):
        return max(self.q_form.get(form, 1.0), 1e-9)

    def _flat(self):
        out = [float(self.sms), self.R_H, self.R_C, self.q_max, self.beta, float(self.reference_form),
               self.layer_overhead, self.tail_overhead, float(self.one_pass_rows), float(self.one_pass_row_bytes)]
        out += self.gamma._flat() + self.dense._flat() + self.attn_prefill._flat() + self.attn_decode._flat()
        out.append(float(len(self.expert)))
        for form, rates in sorted(self.expert.items()):
            out += [float(form)] + rates._flat()
        out.append(float(len(self.rho)))
        for form, curve in sorted(self.rho.items()):
            out += [float(form)] + curve._flat()
        out.append(float(len(self.q_form)))
        for form, q in sorted(self.q_form.items()):
            out += [float(form), float(q)]
        return out


class Seq:
    def __init__(self, tokens=1, context=0):
        self.tokens, self.context = tokens, context


class LaneWork:
    def __init__(self):
        self.decode, self.passes, self.first_layer = False, [], 0
        self.active, self.miss, self.staging, self.deadline, self.samples = [], [], 0, 0.0, True

    def _flat(self):
        out = [float(self.decode), float(self.first_layer), float(self.staging), float(self.deadline), float(self.samples)]
        out += [float(len(self.active))] + [float(v) for v in self.active]
        out += [float(len(self.miss))] + [float(v) for v in self.miss]
        out.append(float(len(self.passes)))
        for seqs in self.passes:
            out.append(float(len(seqs)))
            for s in seqs:
                out += [float(s.tokens), float(s.context)]
        return out


class EstimatorOptions:
    def __init__(self):
        self.contention_aware, self.ewma = True, 0.1


class Estimate:
    _FIELDS = ("total", "attn", "moe", "staged", "a_cmp", "a_rd", "m_cmp", "m_rd", "m_link")

    def __init__(self, values):
        for f, v in zip(self._FIELDS, values):
            setattr(self, f, v)

    def __repr__(self):
        return "Estimate(" + ", ".join(f"{f}={getattr(self, f):.6g}" for f in self._FIELDS) + ")"


class LaneLoad:
    """A lane's work as the estimator counts it (opaque; made by Estimator.load)."""

    def __init__(self, handle, work):
        self._h, self.decode, self.staging, self.deadline = handle, work.decode, work.staging, work.deadline

    def __del__(self):
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:   # (module globals go first at exit)
            _C.lib.monofab_plan_load_destroy(self._h)
            self._h = None


class Estimator:
    def __init__(self, model, calibration, options=None):
        options = options or EstimatorOptions()
        self._model, self._cal, self._opt = model, calibration, options
        m, c = model._flat(), calibration._flat()
        self._h = ctypes.c_void_p()
        _C.check(_C.lib.monofab_plan_estimator_create(_doubles(m), len(m), _doubles(c), len(c),
                                                      int(options.contention_aware), float(options.ewma),
                                                      ctypes.byref(self._h)))
        info = (ctypes.c_double * 4)()
        _C.check(_C.lib.monofab_plan_estimator_info(self._h, ctypes.byref(info)))
        self.link_credits, self.exposure_bound = info[0], info[1]

    def __del__(self):
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:   # (module globals go first at exit)
            _C.lib.monofab_plan_estimator_destroy(self._h)
            self._h = None

    def load(self, work):
        w = work._flat()
        h = ctypes.c_void_p()
        _C.check(_C.lib.monofab_plan_load_create(self._h, _doubles(w), len(w), ctypes.byref(h)))
        return LaneLoad(h, work)

    def evaluate(self, load, s, credits, form):
        out = (ctypes.c_double * 9)()
        _C.check(_C.lib.monofab_plan_evaluate(self._h, load._h, int(s), float(credits), int(form), ctypes.byref(out)))
        return Estimate(list(out))

    def gamma_ratio(self, own):
        return _C.lib.monofab_plan_gamma_ratio(self._h, float(own))

    def observe(self, decode, moe, ratio):
        _C.check(_C.lib.monofab_plan_observe(self._h, int(decode), int(moe), float(ratio)))

    def correction(self, decode, moe):
        return _C.lib.monofab_plan_correction(self._h, int(decode), int(moe))

    model = property(lambda self: self._model)
    calibration = property(lambda self: self._cal)
    options = property(lambda self: self._opt)


class SearchOptions:
    def __init__(self):
        self.forms, self.pour_quantum, self.pour_candidates, self.decode_choices, self.tolerance = list(FORMS), 2, 8, 4, 0.01


class LanePlan:
    def __init__(self, v):
        self.sms, self.credits, self.form, self.cap = int(v[0]), v[1], int(v[2]), int(v[3])
        self.rate, self.slack, self.est = v[4], v[5], Estimate(v[6:15])


class Plan:
    def __init__(self, v):
        self.feasible, n = bool(v[0]), int(v[1])
        self.copy_rate, self.min_slack, self.total_time, self.evaluations, self.micros = v[2], v[3], v[4], int(v[5]), v[6]
        self.lanes = [LanePlan(v[8 + 15 * i:8 + 15 * (i + 1)]) for i in range(n)]


class PlanSearch:
    def __init__(self, estimator, options=None):
        options = options or SearchOptions()
        self._est, self._opt = estimator, options
        forms = (ctypes.c_int32 * len(options.forms))(*options.forms)
        self._h = ctypes.c_void_p()
        _C.check(_C.lib.monofab_plan_search_create(estimator._h, forms, len(options.forms), options.pour_quantum,
                                                   options.pour_candidates, options.decode_choices, options.tolerance,
                                                   ctypes.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:   # (module globals go first at exit)
            _C.lib.monofab_plan_search_destroy(self._h)
            self._h = None

    def deadline_floor(self, load, credits, form):
        s = ctypes.c_int32()
        _C.check(_C.lib.monofab_plan_deadline_floor(self._h, load._h, float(credits), int(form), ctypes.byref(s)))
        return s.value

    def solve(self, lanes, decode_key=0):
        n = len(lanes)
        handles = (ctypes.c_void_p * max(1, n))(*[l._h for l in lanes])
        out = (ctypes.c_double * (8 + 15 * max(1, n)))()
        _C.check(_C.lib.monofab_plan_solve(self._h, handles, n, int(decode_key), out, len(out)))
        return Plan(list(out))

    def clear_cache(self):
        _C.check(_C.lib.monofab_plan_clear_cache(self._h))

    estimator = property(lambda self: self._est)
    options = property(lambda self: self._opt)


class ProfileView:
    """Expected activated experts per layer for a number of routed rows (csrc/control/admission.h:26-49)."""

    def __init__(self, layers, experts):
        self.layers, self.experts = layers, experts
        self._h = ctypes.c_void_p()
        _C.check(_C.lib.monofab_plan_profile_create(layers, experts, ctypes.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:   # (module globals go first at exit)
            _C.lib.monofab_plan_profile_destroy(self._h)
            self._h = None

    def set_profile(self, decode, shares):
        _C.check(_C.lib.monofab_plan_profile_set(self._h, int(decode), _doubles([float(v) for v in shares]), len(shares)))

    def set_hot(self, hot):
        mask = (ctypes.c_uint8 * len(hot))(*[int(v) for v in hot])
        _C.check(_C.lib.monofab_plan_profile_set_hot(self._h, mask, len(hot)))

    def expected(self, decode, layer, pairs):
        out = (ctypes.c_double * 2)()
        _C.check(_C.lib.monofab_plan_profile_expected(self._h, int(decode), int(layer), float(pairs), ctypes.byref(out)))
        return out[0], out[1]


class Request:
    def __init__(self, id=0, prompt=0, max_output=1, arrival=0.0, ttft=0.0, tpot=0.0):
        self.id, self.prompt, self.max_output, self.arrival, self.ttft, self.tpot = id, prompt, max_output, arrival, ttft, tpot


class AdmissionConfig:
    _FIELDS = ("max_prefill_lanes", "token_budget", "max_batch_requests", "max_decode", "staging_experts", "kv_capacity",
               "kv_bytes_per_token", "workspace_capacity", "lane_workspace", "batch_trials", "reject_checks")

    def __init__(self):
        self.max_prefill_lanes, self.token_budget, self.max_batch_requests, self.max_decode = 2, 16384, 64, 256
        self.staging_experts, self.kv_capacity, self.kv_bytes_per_token = 0, 0.0, 0.0
        self.workspace_capacity, self.lane_workspace, self.batch_trials, self.reject_checks = 0.0, 0.0, 4, 2


class PassSpec:
    def __init__(self, reqs, tokens, pos0, last):
        self.reqs, self.tokens, self.pos0, self.last = reqs, tokens, pos0, last


class Decision:
    """What an admission event decided: publish / feasible / plan / lanes (the fabric lane of every plan
    lane) / decode_changed / decode / joined / rejected / pass_lanes + passes (prefill passes to start) /
    searches / micros (csrc/control/admission.h:81-95)."""

    def __init__(self, words, plan):
        it = iter(words)
        self.publish, self.feasible, self.decode_changed, self.searches = bool(next(it)), bool(next(it)), bool(next(it)), next(it)
        take = lambda: [next(it) for _ in range(next(it))]  # noqa: E731
        self.lanes, self.decode, self.joined, self.rejected = take(), take(), take(), take()
        self.pass_lanes, self.passes = [], []
        for _ in range(next(it)):
            self.pass_lanes.append(next(it))
            rows = [[next(it) for _ in range(4)] for _ in range(next(it))]
            self.passes.append(PassSpec([r[0] for r in rows], [r[1] for r in rows], [r[2] for r in rows], [r[3] for r in rows]))
        self.micros = plan[7]
        self.plan = Plan(plan)


class Admission:
    """Admission events -> decisions (csrc/control/admission.h:97-161)."""

    ARRIVE, PASS_DONE, FINISHED, BEHIND, PROGRESS, GENERATED = range(6)

    def __init__(self, estimator, search, profile, config=None):
        config = config or AdmissionConfig()
        self._keep = (estimator, search, profile)
        cfg = [float(getattr(config, f)) for f in AdmissionConfig._FIELDS]
        self._h = ctypes.c_void_p()
        _C.check(_C.lib.monofab_plan_admission_create(estimator._h, search._h, profile._h, _doubles(cfg), len(cfg),
                                                      ctypes.byref(self._h)))
        self.config = config

    def __del__(self):
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:   # (module globals go first at exit)
            _C.lib.monofab_plan_admission_destroy(self._h)
            self._h = None

    def _event(self, kind, ident, *args):
        a = _doubles([float(v) for v in args])
        if kind in (self.PROGRESS, self.GENERATED):
            _C.check(_C.lib.monofab_plan_admission_event(self._h, kind, int(ident), a, len(args), None, 0, None, None, 0))
            return None
        words, n = (ctypes.c_int64 * 65536)(), ctypes.c_int32()
        plan = (ctypes.c_double * (8 + 15 * 3))()
        _C.check(_C.lib.monofab_plan_admission_event(self._h, kind, int(ident), a, len(args), words, len(words),
                                                     ctypes.byref(n), plan, len(plan)))
        return Decision(list(words[:n.value]), list(plan))

    def arrive(self, r, now):
        return self._event(self.ARRIVE, r.id, r.prompt, r.max_output, r.arrival, r.ttft, r.tpot, now)

    def pass_done(self, lane, now):
        return self._event(self.PASS_DONE, lane, now)

    def finished(self, ident, now):
        return self._event(self.FINISHED, ident, now)

    def behind(self, lane, now):
        return self._event(self.BEHIND, lane, now)

    def progress(self, lane, layers_done):
        self._event(self.PROGRESS, lane, layers_done)

    def generated(self, ident, tokens):
        self._event(self.GENERATED, ident, tokens)

    def _state(self):
        out = (ctypes.c_double * 4)()
        _C.check(_C.lib.monofab_plan_admission_state(self._h, ctypes.byref(out)))
        return list(out)

    queued = property(lambda self: int(self._state()[0]))
    waiting = property(lambda self: int(self._state()[1]))
    open_lanes = property(lambda self: int(self._state()[2]))
    kv_reserved = property(lambda self: self._state()[3])


def profile_view(decode_p, prefill_p, hot):
    """A ProfileView from [layers, experts] activation shares of the decode and prefill profiles and the
    hot tier (a mask of the same shape, or one list of experts per layer)
    (monoserve/control/__init__.py:60-79)."""
    import numpy as np
    decode_p = np.asarray(decode_p, dtype=np.float64)
    layers, experts = decode_p.shape
    view = ProfileView(layers, experts)
    view.set_profile(True, decode_p.ravel().tolist())
    view.set_profile(False, np.asarray(prefill_p, dtype=np.float64).ravel().tolist())
    mask = np.zeros((layers, experts), dtype=np.uint8)
    if isinstance(hot, np.ndarray) and hot.shape == (layers, experts):
        mask[:] = hot != 0
    else:
        for layer, members in enumerate(hot):
            mask[layer, list(members)] = 1
    view.set_hot(mask.ravel().tolist())
    return view


# ---- helpers of monoserve/control/__init__.py and calibration.py ----------------------
def form_name(form):
    return "asym" if form == ASYM else f"sym{form}"


def model_shape(cfg, expert_weight_bytes=None, dense_weight_bytes=None):
    """ModelShape of a model configuration (one byte per weight for FP8, two for bf16, unless given)."""
    wb = 1.0 if getattr(cfg, "fp8", False) else 2.0
    m = ModelShape()
    m.hidden, m.intermediate = cfg.hidden, cfg.intermediate
    m.experts, m.top_k, m.layers = cfg.num_experts, cfg.top_k, cfg.num_layers
    m.heads, m.kv_heads, m.head_dim, m.vocab = cfg.num_heads, cfg.num_kv_heads, getattr(cfg, "head_dim", 128), cfg.vocab
    m.dense_layers = getattr(cfg, "dense_layers", 0)
    m.dense_intermediate = getattr(cfg, "dense_intermediate", 0)
    m.shared_intermediate = getattr(cfg, "shared_intermediate", 0)
    m.expert_weight_bytes = float(wb if expert_weight_bytes is None else expert_weight_bytes)
    m.dense_weight_bytes = float(wb if dense_weight_bytes is None else dense_weight_bytes)
    return m


def _rates(d):
    k = KernelRates()
    sms = [float(s) for s in d["sms"]]
    k.flops = Curve(sms, [v * 1e12 for v in d["tflops"]], True)
    k.bytes = Curve(sms, [v * 1e9 for v in d["gbps"]], True)
    k.q_per_sm = float(d["q_per_sm"])
    return k


def load_calibration(src):
    """A Calibration from a JSON file path or a parsed dict, in the reference's file format
    (monoserve/control/calibration.py:1-25: SM counts, microseconds, TFLOP/s, GB/s, credits), plus the
    optional keys one_pass_rows and one_pass_row_bytes."""
    if isinstance(src, dict):
        d = src
    else:
        with open(src) as f:
            d = json.load(f)
    c = Calibration()
    c.sms = int(d["sms"])
    c.R_H, c.R_C = float(d["R_H_us"]) * 1e-6, float(d["R_C_us"]) * 1e-6
    c.gamma = Curve([x * 1e-6 for x in d["gamma"]["exposure_entry_us"]], d["gamma"]["stretch"], False)
    c.q_max = float(d["q_max"])
    c.dense, c.attn_prefill, c.attn_decode = _rates(d["dense"]), _rates(d["attn_prefill"]), _rates(d["attn_decode"])
    c.expert = {FORM_KEYS[k]: _rates(v) for k, v in d["expert"].items()}
    c.rho = {FORM_KEYS[k]: Curve(v["credits"], [g * 1e9 for g in v["gbps"]], True) for k, v in d["rho"].items()}
    c.q_form = {FORM_KEYS[k]: float(v) for k, v in d["q_form"].items()}
    c.beta = float(d["beta_gbps"]) * 1e9
    c.reference_form = int(d.get("reference_form", 64))
    c.layer_overhead = float(d.get("layer_overhead_us", 0.0)) * 1e-6
    c.tail_overhead = float(d.get("tail_overhead_us", 0.0)) * 1e-6
    c.one_pass_rows = int(d.get("one_pass_rows", 64))
    c.one_pass_row_bytes = float(d.get("one_pass_row_bytes", -1.0))
    return c


def save_calibration(data, path):
    with open(path, "w") as f:
        json.dump(data, f, indent=1, sort_keys=True)


def as_native_module():
    """A module object with the names of the reference's monoserve._C.control."""
    m = types.ModuleType("monoserve._C.control")
    m.__doc__ = "Time estimator, plan search and admission over libmonofab."
    for name in ("ASYM", "Curve", "KernelRates", "ModelShape", "Calibration", "Seq", "LaneWork", "EstimatorOptions",
                 "Estimate", "Estimator", "SearchOptions", "LanePlan", "Plan", "PlanSearch", "ProfileView", "Request",
                 "AdmissionConfig", "PassSpec", "Decision", "Admission"):
        setattr(m, name, globals()[name])
    return m

"""ctypes binding of libmonofab.so: the module that stands where the reference
keeps its native extension `monoserve._C` (csrc/bindings.cpp:171-384).

Raw 64-bit addresses cross this boundary, as in the reference (tensors are
`.data_ptr()`'d in Python, monoserve/fabric/args.py:28-29).  There is no CPU
fallback: if the shared library is missing or cannot be loaded, importing this
module raises, and every compute call needs a CUDA device.
"""
import ctypes
import json
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MONOFAB_LIB") or os.path.join(_HERE, "libmonofab.so")

# Every symbol include/monofab.h declares; tests check that all of them resolve.
EXPORTS = [
    "monofab_version", "monofab_last_error", "monofab_struct_layouts_json", "monofab_host_device_pointer",
    "monofab_host_alloc", "monofab_host_free", "monofab_router_logits", "monofab_router_topk", "monofab_combine", "monofab_attention", "monofab_attention_trace", "monofab_pack_scratch_bytes", "monofab_pack_pairs", "monofab_pack_pairs_static",
    "monofab_moe_create", "monofab_moe_destroy", "monofab_moe_set_router", "monofab_moe_set_region",
    "monofab_moe_set_scales", "monofab_pack_w13", "monofab_moe_set_w13_packed", "monofab_moe_set_table", "monofab_moe_set_plan", "monofab_moe_forward", "monofab_moe_experts",
    "monofab_moe_forward_host", "monofab_moe_status", "monofab_moe_workspace", "monofab_moe_set_profile",
    "monofab_moe_last_times",
    "monofab_fabric_create", "monofab_fabric_destroy", "monofab_fabric_info", "monofab_fabric_start",
    "monofab_fabric_stop", "monofab_fabric_set_limits", "monofab_fabric_upload", "monofab_fabric_release",
    "monofab_fabric_program_info", "monofab_fabric_publish", "monofab_fabric_progress", "monofab_fabric_lane_stats",
    "monofab_fabric_reset_inflight_max", "monofab_fabric_wait_notes", "monofab_fabric_read", "monofab_fabric_write", "monofab_fabric_blob_alloc",
    "monofab_fabric_blob_free", "monofab_fabric_set_trace", "monofab_fabric_trace_count",
    "monofab_fabric_worker_tiles", "monofab_fabric_iteration_times", "monofab_fabric_tensor_map", "monofab_fabric_tensor_map_packed",
    "monofab_fabric_start_on", "monofab_fabric_lane_ring", "monofab_fabric_wait_note_address",
    "monofab_host_loop_create", "monofab_host_loop_add_lane", "monofab_host_loop_start", "monofab_host_loop_stop",
    "monofab_host_loop_stats", "monofab_host_loop_destroy", "monofab_host_loop_inject", "monofab_host_loop_step",
    "monofab_host_loop_log",
    "monofab_ep_create", "monofab_ep_local", "monofab_ep_export", "monofab_ep_connect", "monofab_ep_disconnect",
    "monofab_ep_destroy", "monofab_ep_set_router", "monofab_ep_forward", "monofab_ep_phase", "monofab_ep_workspace",
    "monofab_ep_set_profile", "monofab_ep_last_times", "monofab_ep_dest_base", "monofab_release_debug",
    "monofab_plan_curve_at", "monofab_plan_estimator_create", "monofab_plan_estimator_destroy", "monofab_plan_estimator_info",
    "monofab_plan_gamma_ratio", "monofab_plan_observe", "monofab_plan_correction", "monofab_plan_load_create",
    "monofab_plan_load_destroy", "monofab_plan_evaluate", "monofab_plan_search_create", "monofab_plan_search_destroy",
    "monofab_plan_deadline_floor", "monofab_plan_solve", "monofab_plan_clear_cache",
    "monofab_plan_profile_create", "monofab_plan_profile_destroy", "monofab_plan_profile_set", "monofab_plan_profile_set_hot",
    "monofab_plan_profile_expected", "monofab_plan_admission_create", "monofab_plan_admission_destroy",
    "monofab_plan_admission_state", "monofab_plan_admission_event",
]
EP_HANDLE_BYTES = 256   # MONOFAB_EP_HANDLE_BYTES


class MoEConfigC(ctypes.Structure):
    """struct monofab_moe_config of include/monofab.h."""
    _fields_ = [("hidden", ctypes.c_int32), ("intermediate", ctypes.c_int32), ("experts", ctypes.c_int32),
                ("top_k", ctypes.c_int32), ("max_tokens", ctypes.c_int32), ("scoring", ctypes.c_int32),
                ("renorm", ctypes.c_int32), ("routed_scale", ctypes.c_float), ("fp8", ctypes.c_int32),
                ("reserved", ctypes.c_int32 * 7)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m monoserve_b200.build` "
                          "(there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, f32, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_uint64
    lib.monofab_last_error.restype = ctypes.c_char_p
    lib.monofab_struct_layouts_json.restype = ctypes.c_char_p
    lib.monofab_host_device_pointer.argtypes = [vp, ctypes.POINTER(u64)]
    lib.monofab_host_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(vp)]
    lib.monofab_host_free.argtypes = [vp]
    lib.monofab_router_logits.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    lib.monofab_router_topk.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp]
    lib.monofab_pack_scratch_bytes.restype = ctypes.c_size_t
    lib.monofab_pack_scratch_bytes.argtypes = [i32, i32, i32]
    lib.monofab_pack_pairs.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
    lib.monofab_pack_pairs_static.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.monofab_attention.argtypes = [vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, vp, i32, vp, i32, vp, vp]
    lib.monofab_attention_trace.argtypes = [i32, vp]
    lib.monofab_combine.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp]
    lib.monofab_moe_create.argtypes = [ctypes.POINTER(MoEConfigC), ctypes.POINTER(vp)]
    lib.monofab_moe_destroy.argtypes = [vp]
    lib.monofab_moe_set_router.argtypes = [vp, vp, vp]
    lib.monofab_moe_set_region.argtypes = [vp, i32, vp, vp, i32]
    lib.monofab_moe_set_scales.argtypes = [vp, vp, vp]
    lib.monofab_pack_w13.argtypes = [vp, vp, i32, i32, i32, i32, vp]
    lib.monofab_moe_set_w13_packed.argtypes = [vp, i32, i32]
    lib.monofab_moe_set_table.argtypes = [vp, vp, vp]
    lib.monofab_moe_set_plan.argtypes = [vp, i32, i32, i32]
    lib.monofab_moe_forward.argtypes = [vp, vp, vp, vp, i32, vp]
    lib.monofab_moe_experts.argtypes = [vp, vp, vp, i32, vp]
    lib.monofab_moe_forward_host.argtypes = [vp, vp, vp, vp, i32, vp]
    lib.monofab_moe_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    lib.monofab_moe_workspace.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
    lib.monofab_moe_set_profile.argtypes = [vp, i32]
    lib.monofab_moe_last_times.argtypes = [vp, ctypes.POINTER(ctypes.c_float * 6)]
    u32, sz = ctypes.c_uint32, ctypes.c_size_t
    P = ctypes.POINTER
    lib.monofab_fabric_create.argtypes = [i32, i32, sz, P(vp)]
    lib.monofab_fabric_destroy.argtypes = [vp]
    lib.monofab_fabric_info.argtypes = [vp, P(ctypes.c_int32), P(ctypes.c_int32), P(ctypes.c_int32), P(u64)]
    lib.monofab_fabric_start.argtypes = [vp]
    lib.monofab_fabric_stop.argtypes = [vp]
    lib.monofab_fabric_start_on.argtypes = [vp, u64, u64, i32, i32]
    lib.monofab_fabric_lane_ring.argtypes = [vp, i32, i32, i32, P(u64 * 3), vp, P(i32)]
    lib.monofab_fabric_wait_note_address.argtypes = [vp, P(u64)]
    lib.monofab_fabric_set_limits.argtypes = [vp, u32, u64]
    lib.monofab_fabric_upload.argtypes = [vp, vp, i32, vp, i32, vp, i32, i32, i32, i32, P(u64)]
    lib.monofab_fabric_release.argtypes = [vp, u64]
    lib.monofab_fabric_program_info.argtypes = [vp, u64, P(u32 * 6)]
    lib.monofab_fabric_publish.argtypes = [vp, vp, i32, vp, vp, vp, i32, vp, P(u64)]
    lib.monofab_fabric_progress.argtypes = [vp, vp, vp, vp, P(u64)]
    lib.monofab_fabric_lane_stats.argtypes = [vp, i32, P(u32 * 7)]
    lib.monofab_fabric_reset_inflight_max.argtypes = [vp, i32]
    lib.monofab_fabric_read.argtypes = [vp, u64, vp, sz]
    lib.monofab_fabric_write.argtypes = [vp, u64, vp, sz]
    lib.monofab_fabric_blob_alloc.argtypes = [vp, sz, P(u64)]
    lib.monofab_fabric_blob_free.argtypes = [vp, u64]
    lib.monofab_fabric_set_trace.argtypes = [vp, u64, u32]
    lib.monofab_fabric_trace_count.argtypes = [vp, P(u32)]
    lib.monofab_fabric_worker_tiles.argtypes = [vp, vp, vp]
    lib.monofab_fabric_wait_notes.argtypes = [vp, vp]
    lib.monofab_fabric_iteration_times.argtypes = [vp, i32, u64, i32, ctypes.c_double, vp]
    lib.monofab_fabric_tensor_map.argtypes = [vp, u64, vp, vp, vp, i32, i32, i32, P(u64)]
    lib.monofab_fabric_tensor_map_packed.argtypes = [vp, u64, i32]
    lib.monofab_host_loop_create.argtypes = [vp, i32, i32, ctypes.c_size_t, ctypes.c_size_t, vp, vp, i32, P(vp)]
    lib.monofab_host_loop_add_lane.argtypes = [vp, i32, i32, u64, u64, i32, u64, vp, vp]
    lib.monofab_host_loop_start.argtypes = [vp, i32]
    lib.monofab_host_loop_stop.argtypes = [vp]
    lib.monofab_host_loop_stats.argtypes = [vp, vp]
    lib.monofab_host_loop_destroy.argtypes = [vp]
    lib.monofab_host_loop_inject.argtypes = [vp, i32, u64, u64, u64]
    lib.monofab_host_loop_step.argtypes = [vp]
    lib.monofab_host_loop_log.argtypes = [vp, vp, i32, P(i32)]
    lib.monofab_ep_create.argtypes = [P(MoEConfigC), i32, i32, i32, P(vp)]
    lib.monofab_ep_local.restype = vp
    lib.monofab_ep_local.argtypes = [vp]
    lib.monofab_ep_export.argtypes = [vp, vp]
    lib.monofab_ep_connect.argtypes = [vp, vp]
    lib.monofab_ep_disconnect.argtypes = [vp]
    lib.monofab_ep_destroy.argtypes = [vp]
    lib.monofab_ep_set_router.argtypes = [vp, vp, vp]
    lib.monofab_ep_forward.argtypes = [vp, vp, vp, vp, i32, vp]
    lib.monofab_ep_phase.argtypes = [vp, i32, vp, vp, vp, i32, vp]
    lib.monofab_ep_workspace.argtypes = [vp, ctypes.c_char_p, P(vp), P(sz)]
    lib.monofab_ep_set_profile.argtypes = [vp, i32]
    lib.monofab_ep_last_times.argtypes = [vp, P(ctypes.c_float * 8)]
    lib.monofab_ep_dest_base.argtypes = [vp, i32, i32, i32, i32, i32]
    lib.monofab_release_debug.argtypes = [i32, i32, P(u64 * 3)]
    f64 = ctypes.c_double
    lib.monofab_plan_curve_at.restype = f64
    lib.monofab_plan_curve_at.argtypes = [vp, vp, i32, i32, f64]
    lib.monofab_plan_estimator_create.argtypes = [vp, i32, vp, i32, i32, f64, P(vp)]
    lib.monofab_plan_estimator_destroy.argtypes = [vp]
    lib.monofab_plan_estimator_info.argtypes = [vp, P(f64 * 4)]
    lib.monofab_plan_gamma_ratio.restype = f64
    lib.monofab_plan_gamma_ratio.argtypes = [vp, f64]
    lib.monofab_plan_observe.argtypes = [vp, i32, i32, f64]
    lib.monofab_plan_correction.restype = f64
    lib.monofab_plan_correction.argtypes = [vp, i32, i32]
    lib.monofab_plan_load_create.argtypes = [vp, vp, i32, P(vp)]
    lib.monofab_plan_load_destroy.argtypes = [vp]
    lib.monofab_plan_evaluate.argtypes = [vp, vp, i32, f64, i32, P(f64 * 9)]
    lib.monofab_plan_search_create.argtypes = [vp, vp, i32, i32, i32, i32, f64, P(vp)]
    lib.monofab_plan_search_destroy.argtypes = [vp]
    lib.monofab_plan_deadline_floor.argtypes = [vp, vp, f64, i32, P(i32)]
    lib.monofab_plan_solve.argtypes = [vp, vp, i32, u64, vp, i32]
    lib.monofab_plan_clear_cache.argtypes = [vp]
    i64 = ctypes.c_int64
    lib.monofab_plan_profile_create.argtypes = [i32, i32, P(vp)]
    lib.monofab_plan_profile_destroy.argtypes = [vp]
    lib.monofab_plan_profile_set.argtypes = [vp, i32, vp, i32]
    lib.monofab_plan_profile_set_hot.argtypes = [vp, vp, i32]
    lib.monofab_plan_profile_expected.argtypes = [vp, i32, i32, f64, P(f64 * 2)]
    lib.monofab_plan_admission_create.argtypes = [vp, vp, vp, vp, i32, P(vp)]
    lib.monofab_plan_admission_destroy.argtypes = [vp]
    lib.monofab_plan_admission_state.argtypes = [vp, P(f64 * 4)]
    lib.monofab_plan_admission_event.argtypes = [vp, i32, i64, vp, i32, vp, i32, P(i32), vp, i32]
    return lib


lib = _load()


def check(code):
    """Raise RuntimeError("monofab: ...") on a failing return code, as the
    reference's native layer does (csrc/host/fabric.cpp:15-18)."""
    if code != 0:
        raise RuntimeError(lib.monofab_last_error().decode())
    return code


_layouts = None


def struct_layouts():
    """{name: (sizeof, {field: (offset, "u64" | "u32" | "f32")})}
    (csrc/bindings.cpp:66-168).  The table belongs to the build of the library: parsed once."""
    global _layouts
    if _layouts is None:
        raw = json.loads(lib.monofab_struct_layouts_json().decode())
        _layouts = {k: (v[0], {f: (o, t) for f, (o, t) in v[1].items()}) for k, v in raw.items()}
    return _layouts


def host_device_pointer(host_addr):
    out = ctypes.c_uint64()
    check(lib.monofab_host_device_pointer(ctypes.c_void_p(host_addr), ctypes.byref(out)))
    return out.value


def gemm_args(out, ld_out, k_tiles, epi, bm, n_limit, pair_token=0, pair_weight=0, residual=0, ld_res=0, bias=0,
              up_offset=0, w_fp8=0):
    """Packed GemmArgs block (csrc/bindings.cpp:332-356)."""
    from monoserve_b200.fabric.args import pack
    return pack("GemmArgs", out=out, ld_out=ld_out, k_tiles=k_tiles, epi=epi, bm=bm, n_limit=n_limit,
                pair_token=pair_token, pair_weight=pair_weight, residual=residual, ld_res=ld_res, bias=bias,
                up_offset=up_offset, w_fp8=w_fp8)

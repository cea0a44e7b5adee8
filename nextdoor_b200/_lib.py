"""ctypes bindings of libnextdoor_b200.so (the C ABI declared in include/nextdoor_b200.h).

There is no CPU fallback: if the shared library is missing the import of this module raises,
and every compute entry point fails with ND_ERR_CUDA on a machine without a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("ND_B200_LIB") or os.path.join(HERE, "libnextdoor_b200.so")  # override: another build of the same ABI

ND_OK = 0
MAX_FANOUT = 8

APP_UNIFORM_WALK, APP_DEEPWALK, APP_PPR, APP_NODE2VEC, APP_KHOP, APP_KHOP_DISTINCT = range(6)
APP_FASTGCN_REF, APP_LADIES_REF, APP_FASTGCN_IS, APP_LADIES_IS = 6, 7, 8, 9
MODE_TRANSIT_PARALLEL, MODE_TRANSIT_PARALLEL_LB, MODE_SAMPLE_PARALLEL = 0, 1, 2
PHASES = ("next", "invert", "bin", "finalize", "dedup", "collect", "tail")


class AppParams(C.Structure):
    _fields_ = [
        ("app", C.c_int32),
        ("steps", C.c_int32),
        ("fanout", C.c_int32 * MAX_FANOUT),
        ("batch", C.c_int32),
        ("n2v_ref_compat", C.c_int32),
        ("p", C.c_float),
        ("q", C.c_float),
        ("stop_prob", C.c_float),
        ("seed", C.c_uint64),
    ]


class NdError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"nextdoor_b200 error {code}: {msg}")
        self.code = code


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m nextdoor_b200.build` "
        "(the package has no fallback implementation)")

lib = C.CDLL(LIB_PATH)
VP = C.c_void_p

_SIGS = {
    "nd_last_error": (C.c_char_p, []),
    "nd_version": (C.c_int, []),
    "nd_device_count": (C.c_int, []),
    "nd_launch_count": (C.c_int64, []),
    "nd_graph_from_csr": (C.c_int, [C.c_int, C.c_int32, C.c_int64, VP, VP, VP, VP, C.POINTER(VP)]),
    "nd_graph_from_edge_records": (C.c_int, [C.c_int, C.c_int64, VP, C.POINTER(VP)]),
    "nd_graph_load_edge_list_binary": (C.c_int, [C.c_int, C.c_char_p, C.POINTER(VP)]),
    "nd_graph_load": (C.c_int, [C.c_int, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(VP)]),
    "nd_graph_rmat": (C.c_int, [C.c_int, C.c_int32, C.c_int64, C.c_uint64, C.POINTER(VP)]),
    "nd_graph_info": (C.c_int, [VP, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_int)]),
    "nd_graph_to_host": (C.c_int, [VP, VP, VP, VP, VP]),
    "nd_graph_device_ptrs": (C.c_int, [VP, C.POINTER(VP), C.POINTER(VP), C.POINTER(VP), C.POINTER(VP)]),
    "nd_graph_destroy": (C.c_int, [VP]),
    "nd_graph_partition": (C.c_int, [VP, C.c_int64, C.c_int32, VP, VP, VP, VP, C.POINTER(C.c_int32)]),
    "nd_final_sample_size": (C.c_int, [C.POINTER(AppParams)]),
    "nd_initial_sample_size": (C.c_int, [C.POINTER(AppParams)]),
    "nd_shard_range": (C.c_int, [C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "nd_sampler_create": (C.c_int, [VP, C.POINTER(AppParams), C.c_int64, C.c_int64, VP, C.POINTER(VP)]),
    "nd_sampler_set_initial": (C.c_int, [VP, VP]),
    "nd_sampler_set_stream": (C.c_int, [VP, VP]),
    "nd_sampler_sample": (C.c_int, [VP, C.c_int]),
    "nd_sampler_sync": (C.c_int, [VP]),
    "nd_sampler_final_samples": (C.c_int, [VP, VP]),
    "nd_sampler_final_samples_async": (C.c_int, [VP, VP, VP]),
    "nd_sampler_host_update_begin": (C.c_int, [VP, VP, VP, VP]),
    "nd_sampler_host_update_fetch": (C.c_int, [VP]),
    "nd_sampler_host_update_finish": (C.c_int, [VP, C.POINTER(C.c_int64)]),
    "nd_host_fill_int32": (C.c_int, [VP, C.c_int64, C.c_int32]),
    "nd_sampler_pack_rows": (C.c_int, [VP, C.POINTER(VP), C.POINTER(VP)]),
    "nd_sampler_pack_rows_total": (C.c_int, [VP, C.POINTER(C.c_int64)]),
    "nd_rows_scratch_words": (C.c_int64, [C.c_int64]),
    "nd_rows_unpack": (C.c_int, [C.c_int, VP, C.c_int64, C.c_int, C.c_int32, VP, VP, VP, VP, VP]),
    "nd_stream_sync": (C.c_int, [C.c_int, VP]),
    "nd_sampler_final_samples_device": (C.c_int, [VP, C.POINTER(VP)]),
    "nd_sampler_aux": (C.c_int, [VP, VP, VP, VP, VP]),
    "nd_sampler_stats": (C.c_int, [VP, VP, C.c_int]),
    "nd_sampler_live_pairs": (C.c_int, [VP, VP, C.c_int]),
    "nd_sampler_set_profiling": (C.c_int, [VP, C.c_int]),
    "nd_sampler_phase_ms": (C.c_int, [VP, VP, VP, C.c_int]),
    "nd_sampler_next_kernel": (C.c_int, [VP, C.c_int, C.c_char_p, C.c_int]),
    "nd_sampler_destroy": (C.c_int, [VP]),
    "nd_invert_map": (C.c_int, [C.c_int, C.c_int64, VP, VP, C.c_int32, VP, VP, C.POINTER(C.c_int64)]),
    "nd_inverter_create": (C.c_int, [C.c_int, C.c_int64, C.c_int32, C.POINTER(VP)]),
    "nd_inverter_run": (C.c_int, [VP, VP, C.c_int64, VP, VP, VP, VP, C.POINTER(VP)]),
    "nd_inverter_destroy": (C.c_int, [VP]),
    "nd_invert_map_static": (C.c_int, [C.c_int, C.c_int64, VP, VP, C.c_int32, VP, VP, C.POINTER(C.c_int64)]),
    "nd_invert_map_static_on": (C.c_int, [C.c_int, VP, C.c_int64, VP, VP, C.c_int32, VP, VP, C.POINTER(C.c_int64)]),
    "nd_static_max_pairs": (C.c_int64, []),
    "nd_distinct_segments":(C.c_int, [C.c_int, VP, C.c_int64, C.c_int32, C.c_int32, VP]),
    "nd_philox_uniform": (C.c_int, [C.c_int, C.c_uint64, C.c_int64, VP, VP]),
    "nd_walk_step": (C.c_int, [VP, C.POINTER(AppParams), C.c_int, C.c_int64, VP, VP, VP, VP]),
    "nd_walk_step_packed": (C.c_int, [VP, C.POINTER(AppParams), C.c_int, C.c_int64, VP, VP, VP]),
    "nd_walk_step_status": (C.c_int, [C.c_int, VP, C.POINTER(C.c_int)]),
    "nd_route_count": (C.c_int, [C.c_int, C.c_int64, VP, C.c_int, VP, C.c_int, VP, VP]),
    "nd_route_scatter": (C.c_int, [C.c_int, C.c_int64, VP, C.c_int, VP, C.c_int, VP, VP, VP, VP]),
    "nd_records_store": (C.c_int, [C.c_int, C.c_int64, VP, C.c_int, C.c_int64, C.c_int64, C.c_int, VP, VP]),
}

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED = tuple(_SIGS)


def check(code):
    if code != ND_OK:
        raise NdError(code, lib.nd_last_error().decode(errors="replace"))

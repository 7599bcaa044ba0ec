"""ctypes prototypes for the engine-level C ABI (include/pi05_b200.h)."""
from __future__ import annotations

import ctypes as C


class Gemma(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("width", "depth", "mlp_dim", "num_heads", "num_kv_heads", "head_dim")]


class ModelConfig(C.Structure):
    _fields_ = ([(n, C.c_int32) for n in (
        "action_dim", "action_horizon", "max_token_len", "num_flow_steps", "num_views",
        "image_size", "patch_size", "vision_width", "vision_depth", "vision_mlp_dim",
        "vision_heads", "vision_head_dim", "vocab_size")]
        + [(n, C.c_float) for n in (
            "rms_norm_eps", "layer_norm_eps", "rope_theta", "time_min_period", "time_max_period")]
        + [("language", Gemma), ("action_expert", Gemma)])


class EngineOptions(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("device", C.c_int32), ("seed", C.c_uint64),
                ("act_scale", C.c_float), ("weight_dist", C.c_int32),
                ("int8_activations", C.c_int32)]


class HostTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("elements", C.c_uint64),
                ("dtype", C.c_int32)]


class Observation(C.Structure):
    _fields_ = [("token_count", C.c_int32), ("image_layout", C.c_int32), ("images", C.c_void_p),
                ("patches", C.c_void_p), ("token_ids", C.c_void_p), ("noise", C.c_void_p),
                ("noise_dtype", C.c_int32)]


class Signature(C.Structure):
    _fields_ = [("elements", C.c_uint64), ("sum", C.c_double), ("abs_checksum", C.c_double),
                ("l2", C.c_double), ("max_abs", C.c_double), ("sample_count", C.c_int32),
                ("sample", C.c_float * 256)]


_P = C.c_void_p
_SZ = C.c_size_t

PROTOTYPES = [
    ("pi05_default_config", None, [C.POINTER(ModelConfig)]),
    ("pi05_engine_create", C.c_int,
     [C.POINTER(ModelConfig), C.c_int32, C.c_int32, C.c_uint64, C.c_float, C.POINTER(_P)]),
    ("pi05_engine_create_ex", C.c_int,
     [C.POINTER(ModelConfig), C.POINTER(EngineOptions), C.POINTER(_P)]),
    ("pi05_engine_set_activation_scale", C.c_int, [_P, C.c_char_p, C.c_float]),
    ("pi05_engine_activation_scale", C.c_float, [_P, C.c_char_p]),
    ("pi05_set_tuning", C.c_int, [C.c_char_p, C.c_int32]),
    ("pi05_engine_create_from_tensors", C.c_int,
     [C.POINTER(ModelConfig), C.POINTER(EngineOptions), C.POINTER(HostTensor), C.c_int32, C.POINTER(_P)]),
    ("pi05_device_sm", C.c_int, [C.c_int32]),
    ("pi05_runtime_create", C.c_int, [_P, C.POINTER(_P)]),
    ("pi05_runtime_destroy", None, [_P]),
    ("pi05_runtime_infer", C.c_int, [_P, C.POINTER(Observation), _P]),
    ("pi05_runtime_plan_info", C.c_int,
     [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    ("pi05_graph_signature", C.c_int, [_P, C.c_char_p, C.POINTER(Signature)]),
    ("pi05_engine_destroy", None, [_P]),
    ("pi05_engine_weight_bytes", _SZ, [_P]),
    ("pi05_engine_read_weight", C.c_int, [_P, C.c_char_p, _P, _SZ, C.POINTER(_SZ)]),
    ("pi05_engine_capture", C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.POINTER(_P)]),
    ("pi05_graph_destroy", None, [_P]),
    ("pi05_graph_update_raw_image_inputs", C.c_int, [_P, _P, _P, _P]),
    ("pi05_graph_update_patch_inputs", C.c_int, [_P, _P, _P, _P]),
    ("pi05_graph_replay", C.c_int, [_P]),
    ("pi05_graph_run_eager", C.c_int, [_P]),
    ("pi05_graph_sync", C.c_int, [_P]),
    ("pi05_graph_output", C.c_int, [_P, _P]),
    ("pi05_graph_time_replays", C.c_int, [_P, C.c_int32, _P]),
    ("pi05_graph_stage_times", C.c_int, [_P, _P]),
    ("pi05_graph_time_launches", C.c_int, [_P, C.c_char_p, _P, _P]),
    ("pi05_graph_workspace_bytes", _SZ, [_P]),
    ("pi05_graph_workspace_used_bytes", _SZ, [_P]),
    ("pi05_graph_num_launches", C.c_int32, [_P]),
    ("pi05_graph_launch_name", C.c_char_p, [_P, C.c_int32]),
    ("pi05_graph_read_tensor", C.c_int, [_P, C.c_char_p, _P, _SZ, C.POINTER(_SZ)]),
]


def declare(handle: C.CDLL) -> None:
    """Attach argtypes/restype to every exported engine-level symbol."""
    for name, restype, argtypes in PROTOTYPES:
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes

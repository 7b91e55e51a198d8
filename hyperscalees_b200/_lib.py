"""ctypes binding of libhses_b200.so (the C ABI declared in include/hses.h).

There is no fallback: if the shared object is missing or cannot be loaded the
import of any compute entry point raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhses_b200.so")

c_f32p = C.POINTER(C.c_float)
c_i32p = C.POINTER(C.c_int32)

# every symbol include/hses.h declares, in declaration order
EXPORTS = [
    "hses_last_error", "hses_version", "hses_ctx_create", "hses_ctx_destroy",
    "hses_ctx_calibration_info", "hses_ctx_device_status", "hses_profile_enable", "hses_profile_count", "hses_profile_read",
    "hses_noise_seed", "hses_normal_fill", "hses_lora_factors",
    "hses_dense_noise", "hses_poisson_encode", "hses_poisson_encode_dual", "hses_lif_scan",
    "hses_perturbed_linear_workspace_bytes", "hses_perturbed_linear", "hses_time_mean", "hses_fitness",
    "hses_peer_window_bytes", "hses_peer_alloc", "hses_peer_open", "hses_peer_close", "hses_peer_free",
    "hses_fitness_publish", "hses_fitness_wait", "hses_fitness_exchange",
    "hses_member_mean", "hses_convert_fitnesses", "hses_es_update_workspace_bytes",
    "hses_es_update", "hses_es_update_static_scratch_bytes", "hses_es_update_static",
    "hses_es_update_dense", "hses_solver_step", "hses_snn_forward_workspace_bytes", "hses_snn_forward",
    "hses_population_eval_workspace_bytes", "hses_population_eval", "hses_population_update_workspace_bytes",
    "hses_population_update", "hses_wkv7", "hses_spiking_attention",
    "hses_factor_cache_bytes", "hses_factor_cache_build", "hses_es_update_ex",
    "hses_population_grads_elems", "hses_population_grads", "hses_population_apply",
    "hses_convert_fitnesses_bs", "hses_vector_mul",
    "hses_prng_normal_half", "hses_einsum_pair_workspace_bytes", "hses_einsum_pair", "hses_layer_norm", "hses_group_norm", "hses_token_shift_mix", "hses_relu_square", "hses_rate_encode",
    "hses_rwkv_mix_prepare", "hses_rwkv_mix_finish", "hses_token_shift_mix_multi",
    "hses_embedding", "hses_lif_rate", "hses_swish", "hses_add_inplace", "hses_token_fitness",
    "hses_comm_unique_id", "hses_comm_init", "hses_comm_rank", "hses_comm_world", "hses_comm_async_error",
    "hses_comm_destroy", "hses_comm_abort", "hses_allgather_fitness", "hses_allreduce_grads",
]


class FactorCacheDesc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("key", C.c_uint64), ("true_epoch", C.c_int32),
                ("first_pair", C.c_int32), ("n_pairs", C.c_int64), ("rank", C.c_int32),
                ("a", C.c_int32), ("b", C.c_int32)]


class UpdateArgs(C.Structure):
    _fields_ = [("key", C.c_uint64), ("epoch", C.c_int32), ("noise_reuse", C.c_int32),
                ("first_thread", C.c_int32), ("n", C.c_int64), ("n_total", C.c_int64),
                ("rank", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("sigma", C.c_float),
                ("fitness", C.c_void_p), ("grad", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t), ("cache", C.POINTER(FactorCacheDesc)),
                ("mode", C.c_int32), ("sign_factors", C.c_int32), ("algo", C.c_int32)]


class LinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("t_steps", C.c_int32), ("n_pop", C.c_int64), ("bm", C.c_int32),
        ("k", C.c_int32), ("x_row_stride", C.c_int64), ("param", C.c_void_p), ("a", C.c_int32),
        ("param_row_stride", C.c_int64), ("sigma", C.c_float), ("rank", C.c_int32),
        ("key", C.c_uint64), ("epoch", C.c_int32), ("first_thread", C.c_int32),
        ("noise_reuse", C.c_int32), ("perturb", C.c_int32), ("lif", C.c_int32),
        ("tau_m", C.c_float), ("v_th", C.c_float), ("reset_mode", C.c_int32), ("out_scale", C.c_float), ("out_scale_ptr", C.c_void_p), ("out", C.c_void_p),
        ("out_row_stride", C.c_int64), ("potentials", C.c_void_p), ("algo", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("cache", C.POINTER(FactorCacheDesc)), ("precision", C.c_int32),
        ("factor_order", C.c_int32), ("x_half", C.c_void_p), ("out_half", C.c_void_p), ("x_split_valid", C.c_int32), ("n_groups", C.c_int32), ("x_op", C.c_int32),
    ]


class SnnModelDesc(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("dims", C.POINTER(C.c_int32)), ("weights", C.POINTER(C.c_void_p)),
                ("weight_strides", C.POINTER(C.c_int64)), ("keys", C.POINTER(C.c_uint64)),
                ("out_gain", C.c_float), ("out_gain_dev", C.c_void_p), ("tau_m", C.c_float),
                ("v_th", C.POINTER(C.c_float)), ("reset_mode", C.c_int32),
                ("caches", C.POINTER(C.POINTER(FactorCacheDesc)))]


class PopArgs(C.Structure):
    _fields_ = [("T", C.c_int32), ("n_pop", C.c_int64), ("bm", C.c_int32), ("perturb", C.c_int32),
                ("sigma", C.c_float), ("rank", C.c_int32), ("epoch", C.c_int32), ("first_thread", C.c_int32),
                ("noise_reuse", C.c_int32)]


class SolverDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("lr", C.c_float), ("beta1", C.c_float),
                ("beta2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float)]


class HsesError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"hses status {status}: {message}")
        self.status = status


_lib = None


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m hyperscalees_b200._build` "
            "(there is no CPU or PyTorch fallback for the CUDA path)")
    L = C.CDLL(LIB_PATH)
    vp, i32, i64, u64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_size_t
    L.hses_last_error.restype = C.c_char_p
    L.hses_last_error.argtypes = []
    L.hses_version.restype = C.c_int
    L.hses_ctx_create.argtypes = [C.c_int, C.POINTER(vp)]
    L.hses_ctx_destroy.argtypes = [vp]
    L.hses_ctx_calibration_info.argtypes = [vp, C.POINTER(u64), C.POINTER(u64)]
    L.hses_ctx_device_status.argtypes = [vp, C.POINTER(C.c_int)]
    L.hses_profile_enable.argtypes = [vp, C.c_int]
    L.hses_profile_count.argtypes = [vp]
    L.hses_profile_read.argtypes = [vp, C.c_int, C.POINTER(C.c_char_p), C.POINTER(i64), C.POINTER(C.c_double)]
    L.hses_noise_seed.restype = u64
    L.hses_noise_seed.argtypes = [u64, i32, i32]
    L.hses_normal_fill.argtypes = [vp, vp, u64, vp, sz]
    L.hses_lora_factors.argtypes = [vp, vp, u64, i32, i32, vp, i32, i64, i32, i32, i32, f32, i32, vp, vp]
    L.hses_dense_noise.argtypes = [vp, vp, u64, i32, i32, vp, i32, i64, i32, i32, f32, vp]
    L.hses_poisson_encode.argtypes = [vp, vp, vp, i64, i32, i64, i32, C.POINTER(C.c_uint32), vp]
    L.hses_poisson_encode_dual.argtypes = [vp, vp, vp, i64, i32, i64, i32, C.POINTER(C.c_uint32), vp, vp]
    L.hses_lif_scan.argtypes = [vp, vp, vp, i32, i64, i32, i64, vp, f32, f32, i32, vp]
    L.hses_perturbed_linear_workspace_bytes.restype = sz
    L.hses_perturbed_linear_workspace_bytes.argtypes = [C.POINTER(LinearArgs)]
    L.hses_perturbed_linear.argtypes = [vp, vp, C.POINTER(LinearArgs)]
    L.hses_time_mean.argtypes = [vp, vp, vp, i32, i64, i32, i64, vp, i64]
    L.hses_peer_window_bytes.argtypes = [i64]
    L.hses_peer_window_bytes.restype = C.c_size_t
    L.hses_peer_alloc.argtypes = [vp, i64, C.POINTER(vp), vp]
    L.hses_peer_open.argtypes = [vp, vp, C.POINTER(vp)]
    L.hses_peer_close.argtypes = [vp]
    L.hses_peer_free.argtypes = [vp]
    L.hses_fitness_publish.argtypes = [vp, vp, vp, i64, i64, i64, C.POINTER(vp), i32, i32, C.c_uint32]
    L.hses_fitness_wait.argtypes = [vp, vp, vp, i64, i32, C.c_uint32, vp]
    L.hses_fitness_exchange.argtypes = [vp, vp, vp, i64, i64, i64, C.POINTER(vp), i32, i32, C.c_uint32, vp]
    L.hses_fitness.argtypes = [vp, vp, vp, i64, i32, vp, i32, vp]
    L.hses_member_mean.argtypes = [vp, vp, vp, i64, i32, vp]
    L.hses_convert_fitnesses.argtypes = [vp, vp, vp, i64, i32, vp, vp]
    L.hses_es_update_workspace_bytes.restype = sz
    L.hses_es_update_workspace_bytes.argtypes = [i32, i32, i32, i64]
    L.hses_es_update.argtypes = [vp, vp, u64, i32, i32, i32, i64, i64, i32, i32, i32, f32, vp, vp, vp, sz]
    L.hses_es_update_ex.argtypes = [vp, vp, C.POINTER(UpdateArgs)]
    L.hses_factor_cache_bytes.restype = sz
    L.hses_factor_cache_bytes.argtypes = [i64, i32, i32, i32]
    L.hses_factor_cache_build.argtypes = [vp, vp, u64, i32, i32, i32, i64, i32, i32, i32, vp,
                                          C.POINTER(FactorCacheDesc)]
    L.hses_es_update_static_scratch_bytes.restype = sz
    L.hses_es_update_static_scratch_bytes.argtypes = []
    L.hses_es_update_static.argtypes = [vp, vp, u64, i32, i32, i32, i64, i64, i32, i32, i32, f32, vp, vp]
    L.hses_es_update_dense.argtypes = [vp, vp, u64, i32, i32, i32, i64, i64, i32, f32, vp, vp]
    L.hses_solver_step.argtypes = [vp, vp, C.POINTER(SolverDesc), i32, f32, vp, vp, vp, vp, i64]
    pm, pp = C.POINTER(SnnModelDesc), C.POINTER(PopArgs)
    L.hses_snn_forward_workspace_bytes.restype = sz
    L.hses_snn_forward_workspace_bytes.argtypes = [pm, pp]
    L.hses_snn_forward.argtypes = [vp, vp, pm, pp, vp, i64, vp, vp, sz]
    L.hses_population_eval_workspace_bytes.restype = sz
    L.hses_population_eval_workspace_bytes.argtypes = [pm, pp]
    L.hses_population_eval.argtypes = [vp, vp, pm, pp, vp, i64, vp, C.POINTER(C.c_uint32), i32, vp, vp, vp, sz]
    L.hses_population_update_workspace_bytes.restype = sz
    L.hses_population_update_workspace_bytes.argtypes = [pm, i32, i64]
    L.hses_population_update.argtypes = [vp, vp, pm, f32, i32, i32, i32, i32, i32, u64, vp, i64,
                                         C.POINTER(SolverDesc), i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                         vp, sz]
    L.hses_convert_fitnesses_bs.argtypes = [vp, vp, vp, i64, i32, vp, vp]
    L.hses_vector_mul.argtypes = [vp, vp, vp, vp, vp, i64]
    L.hses_prng_normal_half.argtypes = [vp, vp, vp, i64, C.c_float, C.c_float, C.POINTER(C.c_uint32)]
    L.hses_einsum_pair_workspace_bytes.restype = sz
    L.hses_einsum_pair_workspace_bytes.argtypes = [i64, i32, i32, i32]
    L.hses_einsum_pair.argtypes = [vp, vp, vp, i64, i64, vp, i64, i64, vp, i64, i32, i32, i32, vp, vp, vp, sz]
    L.hses_layer_norm.argtypes = [vp, vp, vp, i64, i32, vp, vp, f32, vp]
    L.hses_group_norm.argtypes = [vp, vp, vp, i64, i32, i32, i32, vp, vp, f32, vp]
    L.hses_token_shift_mix.argtypes = [vp, vp, vp, i32, i32, vp, vp, vp, vp]
    L.hses_relu_square.argtypes = [vp, vp, vp, i64, vp]
    L.hses_rwkv_mix_prepare.argtypes = [vp, vp, i64, i32, i32] + [vp] * 16
    L.hses_rwkv_mix_finish.argtypes = [vp, vp, i64, i32, i32] + [vp] * 7
    L.hses_token_shift_mix_multi.argtypes = [vp, vp, vp, i32, i32, vp, vp, i32, C.POINTER(vp), C.POINTER(vp)]
    L.hses_rate_encode.argtypes = [vp, vp, vp, i64, f32, vp]
    L.hses_population_grads_elems.restype = sz
    L.hses_population_grads_elems.argtypes = [pm]
    L.hses_population_grads.argtypes = [vp, vp, pm, f32, i32, i32, i32, i32, i32, u64, vp, i64, i32, i64, vp, vp, sz]
    L.hses_population_apply.argtypes = [vp, vp, pm, C.POINTER(SolverDesc), i32, C.POINTER(vp), C.POINTER(vp),
                                        C.POINTER(vp), vp]
    L.hses_wkv7.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, vp, vp]
    L.hses_spiking_attention.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, i32, f32, vp, f32, f32, f32, i32,
                                         vp, vp]
    L.hses_embedding.argtypes = [vp, vp, vp, i64, vp, i64, i32, i32, vp, i32, vp, vp, i32, i64, vp, i64]
    L.hses_lif_rate.argtypes = [vp, vp, vp, i64, i32, f32, f32, i32, vp]
    L.hses_swish.argtypes = [vp, vp, vp, i64, vp]
    L.hses_add_inplace.argtypes = [vp, vp, vp, vp, i64]
    L.hses_token_fitness.argtypes = [vp, vp, vp, i64, vp, i64, i32, i32, i32, f32, vp, vp]
    L.hses_comm_unique_id.argtypes = [vp]
    L.hses_comm_init.argtypes = [vp, vp, i32, i32, C.POINTER(vp)]
    L.hses_comm_rank.argtypes = [vp]
    L.hses_comm_world.argtypes = [vp]
    L.hses_comm_async_error.argtypes = [vp]
    L.hses_comm_destroy.argtypes = [vp]
    L.hses_comm_abort.argtypes = [vp]
    L.hses_allgather_fitness.argtypes = [vp, vp, vp, i64, vp]
    L.hses_allreduce_grads.argtypes = [vp, vp, vp, i64]
    for name in EXPORTS:
        fn = getattr(L, name)
        if fn.restype is C.c_int and name not in ("hses_version",):
            fn.restype = C.c_int
    _lib = L
    return L


def check(status: int):
    if status != 0:
        msg = load().hses_last_error()
        raise HsesError(status, msg.decode() if msg else "")

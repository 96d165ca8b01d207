"""ctypes bindings of the in-tree native libraries.

``kernels()`` loads ``libxpool_kernels.so`` (CUDA, sm_100a) and ``runtime()`` loads
``libxpool_runtime.so`` (host-only C++). Both check the ABI number baked into the library against
``EXPECTED_ABI`` — the same contract as the reference's ``EXPECTED_NATIVE_ABI_VERSION``
(src/xpool/cext.py:1-30).

On a machine with a GPU a missing kernel library is an error, never a silent fallback: the Python
operators in :mod:`crosspool_b200.ops` have no eager substitute on the hot path.
"""

from __future__ import annotations

import ctypes as C
import functools
from pathlib import Path

EXPECTED_ABI = 21
HERE = Path(__file__).resolve().parent


class NativeLibraryError(RuntimeError):
    pass


class GemmArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p),
        ("x", C.c_void_p),
        ("out", C.c_void_p),
        ("resid", C.c_void_p),
        ("bias", C.c_void_p),
        ("ws", C.c_void_p),
        ("counters", C.c_void_p),
        ("status", C.c_void_p),
        ("stream", C.c_void_p),
        ("ws_bytes", C.c_size_t),
        ("counter_bytes", C.c_size_t),
        ("w_rows_total", C.c_int),
        ("n_out", C.c_int),
        ("k", C.c_int),
        ("rows", C.c_int),
        ("ldw", C.c_int),
        ("ldx", C.c_int),
        ("ld_out", C.c_int),
        ("ld_resid", C.c_int),
        ("epilogue", C.c_int),
        ("dual", C.c_int),
        ("up_offset", C.c_int),
        ("splits", C.c_int),
        ("bn", C.c_int),
        ("num_sms", C.c_int),
        ("w_evict_first", C.c_int),
        ("w_tiled", C.c_int),
        ("gate_limit", C.c_float),
        ("up_add", C.c_float),
        ("act_alpha", C.c_float),
        ("tile_table", C.c_void_p),
        ("n_tiles", C.c_void_p),
        ("w_rows_per_group", C.c_int),
        ("smem_limit", C.c_int),
        ("fp8", C.c_int),
        ("w_scale", C.c_void_p),
        ("x_scale", C.c_void_p),
        ("ld_xscale", C.c_int),
    ]


class GemmPlan(C.Structure):
    _fields_ = [
        ("ws_bytes", C.c_size_t),
        ("counter_bytes", C.c_size_t),
        ("bn", C.c_int),
        ("nacc", C.c_int),
        ("splits", C.c_int),
        ("tiles", C.c_int),
        ("grid", C.c_int),
        ("smem_bytes", C.c_int),
        ("smem_budget", C.c_int),
        ("stages", C.c_int),
    ]


class NormArgs(C.Structure):
    _fields_ = [
        ("parts", C.c_void_p * 8),
        ("wait_flags", C.c_void_p * 8),
        ("out_peers", C.c_void_p * 8),
        ("peer_flags", C.c_void_p * 8),
        ("peer_meta", C.c_void_p * 8),
        ("resid", C.c_void_p),
        ("weight", C.c_void_p),
        ("out_local", C.c_void_p),
        ("done_counter", C.c_void_p),
        ("status", C.c_void_p),
        ("cancel", C.c_void_p),
        ("wait_ns", C.c_uint64),
        ("rows", C.c_int),
        ("hidden", C.c_int),
        ("ld_parts", C.c_int),
        ("ld_out", C.c_int),
        ("nparts", C.c_int),
        ("npeers", C.c_int),
        ("wait_seq", C.c_uint32),
        ("publish_seq", C.c_uint32),
        ("meta_layer", C.c_uint32),
        ("meta_mode", C.c_uint32),
        ("meta_deadline_us", C.c_uint32),
        ("eps", C.c_float),
        ("seq_counter", C.c_void_p),
        ("meta_deadline_ptr", C.c_void_p),
        ("trace_events", C.c_void_p),
        ("trace_state", C.c_void_p),
        ("trace_capacity", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


def _load(name: str) -> C.CDLL:
    path = HERE / name
    if not path.exists():
        raise NativeLibraryError(
            f"{path} is missing; build it with `python -m crosspool_b200.native.build`"
        )
    return C.CDLL(str(path))


@functools.lru_cache(maxsize=None)
def kernels() -> C.CDLL:
    lib = _load("libxpool_kernels.so")
    lib.xp_abi_version.restype = C.c_int
    got = lib.xp_abi_version()
    if got != EXPECTED_ABI:
        raise NativeLibraryError(f"libxpool_kernels.so has ABI {got}, expected {EXPECTED_ABI}; rebuild")
    for fn in ("xp_gemm", "xp_gemm_plan", "xp_norm_publish", "xp_swiglu", "xp_fill_u32", "xp_l2_flush",
               "xp_encode_tmap_2d"):
        getattr(lib, fn).restype = C.c_int
    lib.xp_gemm.argtypes = [C.POINTER(GemmArgs)]
    lib.xp_gemm_plan.argtypes = [C.POINTER(GemmArgs), C.POINTER(GemmPlan)]
    lib.xp_norm_publish.argtypes = [C.POINTER(NormArgs), C.c_void_p]
    lib.xp_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float,
                              C.c_void_p]
    lib.xp_fill_u32.argtypes = [C.c_void_p, C.c_uint32, C.c_size_t, C.c_void_p]
    lib.xp_l2_flush.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    lib.xp_encode_tmap_2d.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32,
                                      C.c_uint32]
    _declare_attention(lib)
    _declare_lane(lib)
    _declare_moe(lib)
    return lib


def kernels_available() -> bool:
    return (HERE / "libxpool_kernels.so").exists()


_launches = 0


def check(rc: int, what: str, kernels_launched: int = 1) -> None:
    """Raises on a non-zero native return code; counts the kernels the call launched."""
    global _launches
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}")
    _launches += kernels_launched


def launch_count() -> int:
    """Kernels of this library launched (or captured into a graph) so far by this process."""
    return _launches


class RopeArgs(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p),
        ("q_out", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("q_norm_weight", C.c_void_p),
        ("k_norm_weight", C.c_void_p),
        ("positions", C.c_void_p),
        ("slots", C.c_void_p),
        ("rows", C.c_int),
        ("ld_qkv", C.c_int),
        ("q_heads", C.c_int),
        ("kv_heads", C.c_int),
        ("head_dim", C.c_int),
        ("eps", C.c_float),
        ("log2_theta", C.c_float),
    ]


class DecodeAttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("out", C.c_void_p),
        ("ws", C.c_void_p),
        ("block_table", C.c_void_p),
        ("seq_lens", C.c_void_p),
        ("batch", C.c_int),
        ("q_heads", C.c_int),
        ("kv_heads", C.c_int),
        ("head_dim", C.c_int),
        ("page_size", C.c_int),
        ("max_blocks", C.c_int),
        ("num_splits", C.c_int),
        ("scale", C.c_float),
        ("chunk_tokens", C.c_int),
        ("num_pages", C.c_int),
        ("status", C.c_void_p),
        ("force_simt", C.c_int),
        ("reserved", C.c_int),
    ]


class PrefillAttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("out", C.c_void_p),
        ("block_table", C.c_void_p),
        ("q_starts", C.c_void_p),
        ("q_lens", C.c_void_p),
        ("ctx_lens", C.c_void_p),
        ("num_seqs", C.c_int),
        ("max_q_len", C.c_int),
        ("q_heads", C.c_int),
        ("kv_heads", C.c_int),
        ("head_dim", C.c_int),
        ("page_size", C.c_int),
        ("max_blocks", C.c_int),
        ("scale", C.c_float),
        ("num_pages", C.c_int),
        ("force_simple", C.c_int),
        ("status", C.c_void_p),
        ("total_q", C.c_int),
    ]


def _declare_attention(lib: C.CDLL) -> None:
    for fn in ("xp_rope_kv", "xp_decode_attn", "xp_prefill_attn", "xp_embedding", "xp_argmax",
               "xp_decode_attn_splits"):
        getattr(lib, fn).restype = C.c_int
    lib.xp_rope_kv.argtypes = [C.POINTER(RopeArgs), C.c_void_p]
    lib.xp_decode_attn.argtypes = [C.POINTER(DecodeAttnArgs), C.c_void_p]
    lib.xp_prefill_attn.argtypes = [C.POINTER(PrefillAttnArgs), C.c_void_p]
    lib.xp_decode_attn_splits.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.xp_embedding.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.xp_argmax.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.xp_sample.restype = C.c_int
    lib.xp_sample.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]


class WaitArgs(C.Structure):
    _fields_ = [
        ("flags", C.c_void_p * 8),
        ("want_ptr", C.c_void_p),
        ("cancel", C.c_void_p),
        ("status", C.c_void_p),
        ("wait_ns", C.c_uint64),
        ("want", C.c_uint32),
        ("n", C.c_int),
        ("failure", C.c_void_p),
        ("peer_failures", C.c_void_p * 8),
        ("n_peer_failures", C.c_int),
        ("origin_pe", C.c_uint32),
        ("instance", C.c_uint32),
        ("trace_events", C.c_void_p),
        ("trace_state", C.c_void_p),
        ("trace_capacity", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


class SignalArgs(C.Structure):
    _fields_ = [("flags", C.c_void_p * 8), ("seq_counter", C.c_void_p), ("n", C.c_int), ("reserved", C.c_int)]


class LaneInstanceDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p),
        ("act", C.c_void_p),
        ("in_flag", C.c_void_p),
        ("record", C.c_void_p),
        ("out_peer", C.c_void_p),
        ("done_record_peer", C.c_void_p),
        ("capacity_rows", C.c_int),
        ("hidden", C.c_int),
        ("num_layers", C.c_int),
        ("act_ld", C.c_int),
        ("failure_peer", C.c_void_p),
        ("pe", C.c_int),
        ("reserved", C.c_int),
    ]


class LaneLayerDesc(C.Structure):
    _fields_ = [
        ("w_gateup", C.c_void_p),
        ("w_down", C.c_void_p),
        ("bias_gateup", C.c_void_p),
        ("bias_down", C.c_void_p),
        ("inter_local", C.c_int),
        ("gated", C.c_int),
        ("w_tiled", C.c_int),
        ("gate_limit", C.c_float),
        ("up_add", C.c_float),
        ("act_alpha", C.c_float),
        ("router", C.c_void_p),
        ("correction_bias", C.c_void_p),
        ("router_bias", C.c_void_p),
        ("num_experts", C.c_int),
        ("top_k", C.c_int),
        ("expert_lo", C.c_int),
        ("expert_hi", C.c_int),
        ("sigmoid", C.c_int),
        ("renormalize", C.c_int),
        ("scale", C.c_float),
        ("shared_inter_local", C.c_int),
        ("w_shared_gateup", C.c_void_p),
        ("w_shared_down", C.c_void_p),
        ("router_raw", C.c_void_p),
        ("router_precision", C.c_int),
        ("reserved", C.c_int),
    ]


def _declare_lane(lib: C.CDLL) -> None:
    lib.xp_lane_create.restype = C.c_void_p
    lib.xp_lane_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_size_t]
    lib.xp_lane_destroy.restype = None
    lib.xp_lane_destroy.argtypes = [C.c_void_p]
    lib.xp_trace_read.restype = C.c_int64
    lib.xp_trace_read.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_uint64), C.c_uint64, C.POINTER(C.c_uint64),
                                  C.c_void_p]
    lib.xp_trace_destroy.restype = None
    lib.xp_trace_destroy.argtypes = [C.c_void_p, C.c_void_p]
    lib.xp_lane_trace_read.restype = C.c_int64
    lib.xp_lane_trace_read.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.c_uint64, C.POINTER(C.c_uint64), C.c_void_p]
    sig = {
        "xp_lane_trace_enable": [C.c_void_p, C.c_uint32],
        "xp_lane_set_instance": [C.c_void_p, C.c_int, C.POINTER(LaneInstanceDesc)],
        "xp_lane_set_layer": [C.c_void_p, C.c_int, C.c_int, C.POINTER(LaneLayerDesc)],
        "xp_lane_commit": [C.c_void_p],
        "xp_lane_launch": [C.c_void_p, C.c_int, C.c_uint64, C.c_void_p],
        "xp_lane_shutdown": [C.c_void_p, C.c_void_p],
        "xp_lane_failure": [C.c_void_p, C.POINTER(C.c_uint32), C.c_void_p],
        "xp_trace_create": [C.c_uint32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)],
        "xp_lane_threads_start": [C.c_void_p, C.c_uint64, C.c_int],
        "xp_lane_threads_stop": [C.c_void_p],
        "xp_lane_threads_state": [C.c_void_p, C.POINTER(C.c_uint64)],
        "xp_lane_stats": [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.c_void_p],
        "xp_wait_flags": [C.POINTER(WaitArgs), C.c_void_p],
        "xp_signal_flags": [C.POINTER(SignalArgs), C.c_void_p],
        "xp_dev_alloc": [C.POINTER(C.c_void_p), C.c_size_t],
        "xp_dev_free": [C.c_void_p],
        "xp_ipc_get_handle": [C.c_void_p, C.c_void_p],
        "xp_ipc_open": [C.c_void_p, C.POINTER(C.c_void_p)],
        "xp_ipc_close": [C.c_void_p],
        "xp_memset_async": [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p],
        "xp_enable_peer_access": [C.c_int],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = args


class RouterArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("logit_bias", C.c_void_p), ("correction_bias", C.c_void_p),
        ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
        ("rows", C.c_int), ("num_experts", C.c_int), ("top_k", C.c_int), ("ld_logits", C.c_int),
        ("logits_fp32", C.c_int), ("sigmoid", C.c_int), ("renormalize", C.c_int), ("round_weights_bf16", C.c_int),
        ("scale", C.c_float),
    ]


class RouteArgs(C.Structure):
    _fields_ = [
        ("topk_ids", C.c_void_p), ("counts", C.c_void_p), ("offsets", C.c_void_p), ("perm_token", C.c_void_p),
        ("route_pos", C.c_void_p), ("tiles_gateup", C.c_void_p), ("tiles_down", C.c_void_p),
        ("n_tiles_gateup", C.c_void_p), ("n_tiles_down", C.c_void_p),
        ("rows", C.c_int), ("top_k", C.c_int), ("expert_lo", C.c_int), ("expert_hi", C.c_int),
        ("tm_gateup", C.c_int), ("bn_gateup", C.c_int), ("tm_down", C.c_int), ("bn_down", C.c_int),
    ]


def _declare_moe(lib: C.CDLL) -> None:
    sig = {
        "xp_debug_options_set": [C.POINTER(C.c_uint32)],
        "xp_debug_options_get": [C.POINTER(C.c_uint32)],
        "xp_router_topk": [C.POINTER(RouterArgs), C.c_void_p],
        "xp_router_fp32": [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
        "xp_moe_route": [C.POINTER(RouteArgs), C.c_void_p],
        "xp_moe_gather": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p],
        "xp_moe_combine": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
        "xp_quant_act_fp8": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = args


DEBUG_OPTION_NAMES = ("transport_observer", "fabric_observer", "graph_observer", "ffn_routing_observer")


def set_debug_options(options: dict) -> None:
    """Uploads the process's debug options to the kernel library's constant memory on the current device."""
    four = (C.c_uint32 * 4)(*[int(bool(options.get(n, False))) for n in DEBUG_OPTION_NAMES])
    check(kernels().xp_debug_options_set(four), "xp_debug_options_set", 0)


def get_debug_options() -> dict:
    four = (C.c_uint32 * 4)()
    check(kernels().xp_debug_options_get(four), "xp_debug_options_get", 0)
    return {n: bool(four[i]) for i, n in enumerate(DEBUG_OPTION_NAMES)}

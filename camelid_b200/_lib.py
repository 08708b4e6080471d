"""Loads the C-ABI shared library and declares its entry points for ctypes."""
from __future__ import annotations

import ctypes as C
import os
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "camelid_b200.h"


class CmldError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[cmld status {code}] {message}")
        self.code = code
        self.message = message


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "n_heads", "n_kv_heads", "head_dim", "hidden", "ffn_dim", "rope_dim",
                                         "max_pos", "vocab")] + [
        ("eps", C.c_float), ("split_half_pairing", C.c_int32), ("rope_theta", C.c_float), ("max_seqs", C.c_int32),
        ("n_experts", C.c_int32), ("n_experts_used", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
        ("ep_rank", C.c_int32), ("ep_size", C.c_int32), ("device", C.c_int32), ("flags", C.c_int32)]


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("nbytes", C.c_uint64), ("qtype", C.c_int32), ("reserved", C.c_int32)]


def lib_path() -> Path:
    return PKG / "libcamelid_b200.so"


def declared_symbols() -> list[str]:
    """Every function the public header declares."""
    text = HEADER.read_text()
    return sorted(set(re.findall(r"CMLD_API\s+[\w\s\*]+?\b(cmld_\w+)\s*\(", text)))


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    p = lib_path()
    if not p.exists():
        raise ImportError(f"{p} is missing: build it with `python -m camelid_b200.build` (needs nvcc); "
                          "this package has no CPU implementation")
    if "CMLD_NCCL_PATH" not in os.environ:
        # a sharded engine binds NCCL at run time; point it at the copy PyTorch would load, so that a
        # process using both ends up with one libnccl.so.2 whichever is imported first
        try:
            import importlib.util

            spec = importlib.util.find_spec("nvidia.nccl")
            for root in (spec.submodule_search_locations if spec else []):
                cand = Path(root) / "lib" / "libnccl.so.2"
                if cand.exists():
                    os.environ["CMLD_NCCL_PATH"] = str(cand)
                    break
        except Exception:
            pass
    L = C.CDLL(str(p))
    vp, i32, i64, u64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float
    P = C.POINTER
    sig = {
        "cmld_last_error": (C.c_char_p, []),
        "cmld_version": (C.c_char_p, []),
        "cmld_device_count": (i32, []),
        "cmld_set_device": (i32, [i32]),
        "cmld_malloc": (i32, [P(vp), u64]),
        "cmld_free": (i32, [vp]),
        "cmld_memcpy_h2d": (i32, [vp, vp, u64]),
        "cmld_memcpy_d2h": (i32, [vp, vp, u64]),
        "cmld_memset": (i32, [vp, i32, u64]),
        "cmld_device_synchronize": (i32, []),
        "cmld_mem_info": (i32, [P(u64), P(u64)]),
        "cmld_engine_create": (i32, [P(Config), P(vp)]),
        "cmld_engine_destroy": (i32, [vp]),
        "cmld_comm_unique_id": (i32, [vp]),
        "cmld_engine_comm_init": (i32, [vp, vp, i32, i32]),
        "cmld_engine_set_layer": (i32, [vp, i32, P(Tensor), vp, vp]),
        "cmld_engine_set_layer_moe": (i32, [vp, i32, vp, P(Tensor), P(Tensor), P(Tensor)]),
        "cmld_engine_set_output": (i32, [vp, vp, P(Tensor)]),
        "cmld_engine_set_token_embd": (i32, [vp, P(Tensor)]),
        "cmld_engine_adopt_layer": (i32, [vp, i32, P(vp), vp, vp]),
        "cmld_engine_adopt_layer_moe": (i32, [vp, i32, vp, vp, vp, vp]),
        "cmld_engine_adopt_output": (i32, [vp, vp, vp]),
        "cmld_engine_adopt_token_embd": (i32, [vp, vp]),
        "cmld_engine_weights_ready": (i32, [vp]),
        "cmld_engine_filled": (i64, [vp]),
        "cmld_engine_set_filled": (i32, [vp, i64]),
        "cmld_engine_max_pos": (i64, [vp]),
        "cmld_engine_n_layers": (i32, [vp]),
        "cmld_engine_rope_row": (i32, [vp, i64, vp, vp]),
        "cmld_engine_set_rope_frequencies": (i32, [vp, vp, i32]),
        "cmld_engine_forward_token_sample": (i32, [vp, vp, vp, vp, i64, f32, f32, f32, C.c_uint64, vp, vp]),
        "cmld_sample_gumbel": (i32, [vp, i32, f32, C.c_uint64, vp]),
        "cmld_sample_gumbel_filtered": (i32, [vp, i32, f32, f32, C.c_uint64, vp]),
        "cmld_sample_min_p_mask": (i32, [vp, i32, f32, vp]),
        "cmld_sample_uniforms": (i32, [C.c_uint64, i32, vp]),
        "cmld_engine_verify_tree": (i32, [vp, vp, vp, vp, vp, vp, i32, i64, i32, f32, vp]),
        "cmld_engine_compact_tree_kv_path": (i32, [vp, vp, i32, i64]),
        "cmld_engine_forward_token": (i32, [vp, vp, vp, vp, i64, f32, i32, P(C.c_uint32)]),
        "cmld_engine_forward_token_logits": (i32, [vp, vp, vp, vp, i64, f32, vp]),
        "cmld_engine_forward_token_hidden": (i32, [vp, vp, vp, vp, i64, f32, vp, vp]),
        "cmld_engine_forward_layer": (i32, [vp, i32, vp, vp, vp, i64, f32, vp]),
        "cmld_engine_prefill_from": (i32, [vp, vp, vp, vp, i64, f32, i64]),
        "cmld_engine_verify_batch": (i32, [vp, vp, vp, vp, i64, i32, f32, vp]),
        "cmld_engine_seed_layer": (i32, [vp, i32, vp, vp, i64]),
        "cmld_engine_read_kv_layer": (i32, [vp, i32, i64, vp, vp]),
        "cmld_engine_prefill_tokens": (i32, [vp, i32, vp, i64, i64, P(C.c_uint32)]),
        "cmld_engine_decode_greedy": (i32, [vp, i32, vp, vp, vp, i32, vp]),
        "cmld_engine_step_batch": (i32, [vp, i32, vp, vp, vp, vp, vp, vp]),
        "cmld_engine_last_timing": (i32, [vp, P(f32), P(i64)]),
        "cmld_peer_wait_selftest": (i32, [i32]),
        "cmld_exact_sum_selftest": (i32, [vp, i32, vp]),
        "cmld_weight_create": (i32, [i32, i64, i64, vp, u64, P(vp)]),
        "cmld_weight_synth": (i32, [i32, u64, u64, i64, i64, i64, f32, P(vp)]),
        "cmld_weight_shard": (i32, [vp, i64, i64, i64, i64, i64, i64, P(vp)]),
        "cmld_weight_destroy": (i32, [vp]),
        "cmld_weight_wire_bytes": (i64, [vp]),
        "cmld_weight_export_wire": (i32, [vp, vp]),
        "cmld_weight_dequant": (i32, [vp, i64, i64, vp]),
        "cmld_act_row_bytes": (i64, [i64]),
        "cmld_act_quantize": (i32, [i32, vp, i64, i32, vp]),
        "cmld_act_export": (i32, [i32, vp, i64, i32, vp, vp]),
        "cmld_gemv": (i32, [vp, vp, i32, vp, vp]),
        "cmld_gemv_select_kernel": (i32, [i32]),
        "cmld_gemv_fused": (i32, [vp, i32, vp, vp, vp, f32, i32, vp, vp]),
        "cmld_rms_norm": (i32, [vp, vp, i64, i32, f32, vp, i32, vp]),
        "cmld_silu_mul": (i32, [vp, vp, i64, i32, vp, i32, vp]),
        "cmld_argmax": (i32, [vp, i64, i32, vp]),
        "cmld_attention_decode": (i32, [vp, vp, vp, i32, i32, i32, i64, i64, f32, vp]),
        "cmld_attention_decode_noalloc": (i32, [vp, vp, vp, i32, i32, i32, i64, i64, f32, vp]),
        "cmld_attention_decode_ordered": (i32, [vp, vp, vp, i32, i32, i32, i64, i64, f32, vp]),
        "cmld_gemv_time": (i32, [P(vp), i32, vp, i32, vp, i32, i32, P(f32)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    L._signatures = sig
    _lib = L
    return L


def check(rc: int):
    if rc != 0:
        raise CmldError(rc, lib().cmld_last_error().decode("utf-8", "replace"))

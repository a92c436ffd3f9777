"""ctypes loader for the sm_100a kernel library (``librexl3_kernels.so``, built in-tree by :mod:`rexl3_b200.ops.build`).

On a machine with a CUDA device a missing library is an error, never a silent fallback: ops raise if the
extension cannot be loaded.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librexl3_kernels.so")
_lock = threading.Lock()
_lib = None

launch_count = 0  # kernels launched through this module since import (bench.py reports it)


class KernelError(RuntimeError):
    pass


def load(build_if_missing: bool = True):
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            if not build_if_missing:
                raise KernelError(f"{LIB_PATH} is missing: run python -m rexl3_b200.ops.build")
            from . import build as _b
            _b.build()
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
        return _lib


def _declare(lib):
    c_int, c_void, c_f, c_ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_longlong
    sig = {
        "rx_exl3_plan_splits": (c_int, [c_int, c_int, c_int]),
        "rx_exl3_tile_rows": (c_int, [c_int]),
        "rx_exl3_gemm": (c_int, [c_void, c_int, c_int, c_void, c_int, c_int, c_int, c_void, c_int, c_void, c_void]),
        "rx_exl3_gemm_b4": (c_int, [c_void, c_int, c_int, c_void, c_int, c_int, c_void, c_int, c_void, c_void]),
        "rx_exl3_gemm_b4_tp": (c_int, [c_void, c_int, c_int, c_void, c_int, c_int, c_void, c_int, c_void, c_void, c_void]),
        "rx_tp_bump_epoch": (c_int, [c_void, c_void]),
        "rx_tp_finish_rs": (c_int, [c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_tp_norm_rot_push": (c_int, [c_void, c_int, c_int, c_int, c_int, c_void, c_f, c_void, c_void, c_void, c_void]),
        "rx_tp_wait_flags": (c_int, [c_void, c_int, c_void, ctypes.c_uint, c_void, c_void]),
        "rx_ipc_get_handle": (c_int, [c_void, c_void]),
        "rx_ipc_open": (c_int, [c_void, c_void]),
        "rx_ipc_close": (c_int, [c_void]),
        "rx_tp_cand_desc_size": (c_int, []),
        "rx_tp_bcast_desc_size": (c_int, []),
        "rx_tp_finish_bcast": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void]),
        "rx_tp_allsum_add_norm_rot": (c_int, [c_void, c_void, c_int, c_int, c_void, ctypes.c_uint, c_int, c_int, c_void, c_void, c_f, c_void, c_void,
                                              c_void, c_void, c_void]),
        "rx_tp_finish_bcast_mm": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void]),
        "rx_tp_allsum_add_norm_rot_mm": (c_int, [c_void, c_void, c_int, c_int, c_void, ctypes.c_uint, c_int, c_int, c_void, c_void, c_f, c_void, c_void,
                                                 c_void, c_void, c_void, c_void]),
        "rx_exl3_gemm_grouped": (c_int, [c_void, c_int, c_int, c_void, c_ll, c_int, c_int, c_int, c_void, c_int, c_void, c_int, c_int, c_void, c_void]),
        "rx_moe_router": (c_int, [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_f, c_void, c_void, c_void]),
        "rx_moe_router2": (c_int, [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_f, c_void, c_void, c_void, c_void]),
        "rx_moe_router_grouped": (c_int, [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_f, c_int, c_int, c_void, c_void, c_void, c_void]),
        "rx_moe_plan": (c_int, [c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_moe_gather_rot": (c_int, [c_void, c_void, c_void, c_int, c_int, c_int, c_void, c_void, c_void]),
        "rx_moe_swiglu_rot": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_moe_relu2_rot": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_moe_combine_desc_size": (c_int, []),
        "rx_moe_a2a_desc_size": (c_int, []),
        "rx_moe_a2a_dispatch": (c_int, [c_void, c_void, c_int, c_int, c_void, c_void, c_void]),
        "rx_moe_a2a_recv_ids": (c_int, [c_void, c_void, c_void, c_void]),
        "rx_moe_a2a_return": (c_int, [c_void, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_moe_a2a_home": (c_int, [c_void, c_int, c_int, c_void, c_void, c_void, c_void, c_void]),
        "rx_verify_desc_size": (c_int, []),
        "rx_trellis_encode_scratch_bytes": (c_ll, [c_int]),
        "rx_trellis_encode_cuda": (c_int, [c_void, c_int, c_int, c_void, c_void, c_void, c_void, c_int, c_void]),
        "rx_verify_accept": (c_int, [c_void, c_void, c_int, c_int, c_void, c_int, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_mla_scratch_floats": (c_ll, [c_int, c_int, c_int]),
        "rx_mla_attn": (c_int, [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_f, c_void, c_void, c_void]),
        "rx_head_gemm": (c_int, [c_void, c_int, c_int, c_void, c_int, c_int, c_int, c_void, c_int, c_int, c_int, c_void]),
        "rx_mla_row": (c_int, [c_void, c_void, c_void, c_f, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_void]),
        "rx_mla_q_rope": (c_int, [c_void, c_void, c_void, c_int, c_void, c_int, c_void]),
        "rx_mla_attn_sel": (c_int, [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_f, c_void, c_void, c_void, c_int, c_void]),
        "rx_mla_row_ld": (c_int, [c_void, c_int, c_void, c_void, c_f, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_void]),
        "rx_mla_q_rope_ld": (c_int, [c_void, c_int, c_void, c_void, c_int, c_void, c_int, c_void]),
        "rx_dsa_append": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_f, c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_int,
                                  c_void, c_int, c_void]),
        "rx_dsa_select": (c_int, [c_void, c_int, c_void, c_int, c_int, c_void, c_void, c_int, c_void, c_void, c_int, c_f, c_int, c_int, c_void, c_int,
                                  c_void, c_int, c_void, c_void, c_int, c_void]),
        "rx_tp_coll_desc_size": (c_int, []),
        "rx_tp_coll_push": (c_int, [c_void, c_ll, c_void, c_void]),
        "rx_tp_coll_combine": (c_int, [c_void, c_ll, c_int, c_void, c_void, c_void]),
        "rx_fp8_linear_scratch_floats": (c_ll, [c_int, c_int, c_int]),
        "rx_fp8_linear": (c_int, [c_void, c_int, c_int, c_void, c_void, c_int, c_void, c_int, c_int, c_void, c_void, c_int, c_void, c_void]),
        "rx_dsa_gather": (c_int, [c_void, c_void, c_int, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_void]),
        "rx_mxfp4_gemm_grouped": (c_int, [c_void, c_int, c_int, c_void, c_void, c_int, c_int, c_void, c_int, c_void, c_int, c_int, c_void, c_void]),
        "rx_moe_combine": (c_int, [c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_void, c_void]),
        "rx_tp_cand_push": (c_int, [c_void, c_void, c_int, c_int, c_void, c_void]),
        "rx_tp_cand_merge": (c_int, [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_void, ctypes.c_uint, c_void, c_void, c_void, c_void]),
        "rx_ssm_mixer": (c_int, [c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void,
                                 c_void, c_void, c_f, c_void, c_void, c_void, c_void, c_void, c_void, c_int]),
        "rx_gdn_mixer": (c_int, [c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_void,
                                 c_f, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_void]),
        "rx_dev_alloc": (c_int, [c_ll, ctypes.POINTER(ctypes.c_void_p)]),
        "rx_dev_free": (c_int, [c_void]),
        "rx_exl3_unpack": (c_int, [c_void, c_int, c_int, c_int, c_int, c_void, c_void]),
        "rx_set_pdl": (c_int, [c_int]),
        "rx_embed": (c_int, [c_void, c_void, c_void, c_int, c_int, c_int, c_void]),
        "rx_norm_rot_in": (c_int, [c_void, c_void, c_f, c_void, c_void, c_int, c_int, c_void]),
        "rx_finish_store": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_int, c_void]),
        "rx_finish_add_norm_rot": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_f, c_void, c_void, c_void, c_void]),
        "rx_finish_swiglu_rot": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void]),
        "rx_finish_qkv_rope": (c_int, [c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_f, c_void, c_void,
                                       c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_void, c_void, c_int]),
        "rx_state_digest": (c_int, [c_void, c_ll, c_void, c_void]),
        "rx_hc_mix": (c_int, [c_void, c_void, c_void, c_f, c_f, c_f, c_void, c_f, c_f, c_f, c_int, c_int, c_int, c_void, c_void, c_void]),
        "rx_hc_apply": (c_int, [c_void, c_void, c_void, c_int, c_int, c_void]),
        "rx_topk_scratch_bytes": (c_ll, [c_int, c_int, c_int]),
        "rx_topk": (c_int, [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void]),
        "rx_make_kv_tmap": (c_int, [c_void, c_void, c_ll, c_int]),
        "rx_make_kv_tmap8": (c_int, [c_void, c_void, c_ll, c_int]),
        "rx_attn_decode_chunk": (c_int, []),
        "rx_attn_decode_scratch_floats": (c_ll, [c_int, c_int, c_int, c_int]),
        "rx_attn_decode": (c_int, [c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_f,
                                   c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void]),
        "rx_attn_decode_q4": (c_int, [c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_f,
                                      c_void, c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void]),
        "rx_attn_vbt_width": (c_int, []),
        "rx_kv_move_rows": (c_int, [c_void, c_int, c_int, c_int, c_void, c_int, c_void]),
        "rx_attn_prefill_q4": (c_int, [c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                                       c_int, c_f, c_void, c_void, c_void, c_void]),
        "rx_attn_plan_ints": (c_int, []),
        "rx_attn_plan": (c_int, [c_void, c_void, c_int, c_int, c_int, c_int, c_void, c_void, c_void]),
        "rx_attn_prefill_tc": (c_int, [c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                                       c_int, c_f, c_void, c_void, c_int]),
        "rx_attn_prefill": (c_int, [c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                                    c_int, c_f, c_void, c_void, c_void, c_void, c_void]),
    }
    for name, (res, args) in sig.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.restype = res
        fn.argtypes = args


def check(err: int, what: str) -> None:
    if err != 0:
        raise KernelError(f"{what} failed with CUDA error {err}")


def ptr(t) -> int:
    """Device pointer of a torch tensor (None -> NULL)."""
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def count(n: int = 1) -> None:
    global launch_count
    launch_count += n

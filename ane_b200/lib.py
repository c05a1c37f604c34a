"""ctypes binding of libane_cuda.so (the C ABI declared in include/ane_cuda.h).

The library is the product; this module only loads it and declares the prototypes.  There is
no fallback: if the shared object is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libane_cuda.so")

# enums of include/ane_cuda.h
F32, BF16, F16 = 0, 1, 2
ID_U16, ID_I32 = 0, 1
NORM_BWD_REFERENCE, NORM_BWD_EXACT = 0, 1
ROPE_FORWARD, ROPE_INVERSE = 0, 1
ADAM_STORIES, ADAM_DYNAMIC = 0, 1
OOR_SKIP, OOR_ZERO = 0, 2

OK = 0
ERR_INVALID, ERR_CUDA, ERR_NOT_INIT, ERR_NOMEM, ERR_UNSUPPORTED, ERR_TIMEOUT = -1, -2, -3, -4, -5, -6


class AneCudaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libane_cuda error {code}: {msg}")
        self.code = code


class AdamState(C.Structure):
    """training/stories_config.h:56-59"""
    _fields_ = [("m", C.POINTER(C.c_float)), ("v", C.POINTER(C.c_float)), ("n", C.c_size_t)]


class Status(C.Structure):
    _fields_ = [("oor_ids", C.c_int32), ("nonfinite", C.c_int32), ("wait_giveups", C.c_int32),
                ("reserved", C.c_int32)]


_vp, _i, _u, _f, _sz = C.c_void_p, C.c_int, C.c_uint, C.c_float, C.c_size_t
_fp = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)

# name -> (restype, argtypes).  Every symbol include/ane_cuda.h declares is listed here; the CPU
# test-suite checks that the shared object exports each of them.
PROTOTYPES = {
    "ane_cuda_init": (_i, [_i]),
    "ane_cuda_shutdown": (None, []),
    "ane_cuda_version": (_i, []),
    "ane_cuda_device_count": (_i, []),
    "ane_cuda_last_error": (C.c_char_p, []),
    "ane_cuda_launch_count": (C.c_longlong, []),
    "ane_cuda_reset_launch_count": (None, []),
    "ane_cuda_set_tuning": (_i, [C.c_char_p, _i]),
    "ane_cuda_clear_tuning": (_i, [C.c_char_p]),
    "ane_cuda_alloc": (_vp, [_sz]),
    "ane_cuda_write": (_i, [_vp, _sz, _vp, _sz]),
    "ane_cuda_read": (_i, [_vp, _sz, _vp, _sz]),
    "ane_cuda_devptr": (_vp, [_vp]),
    "ane_cuda_bufsize": (_sz, [_vp]),
    "ane_cuda_free": (None, [_vp]),
    "ane_cuda_host_alloc": (_vp, [_sz]),
    "ane_cuda_host_free": (None, [_vp]),
    "ane_cuda_sync": (_i, [_vp]),
    "ane_cuda_zero_dev": (_i, [_vp, _vp, _sz]),
    "ane_cuda_copy_dev": (_i, [_vp, _vp, _vp, _sz]),
    "ane_cuda_poll_status": (_i, [C.POINTER(Status), _i]),
    "ane_cuda_workspace_bytes": (_sz, []),
    "ane_cuda_reserve_workspace": (_i, [_sz]),
    "ane_cuda_freeze": (_i, [_i]),
    "ane_cuda_release_caches": (_i, []),
    # host-pointer drop-ins
    "ane_cuda_rmsnorm": (_i, [_fp, _fp, _fp, _i, _i]),
    "ane_cuda_rmsnorm_bwd": (_i, [_fp, _fp, _fp, _fp, _fp, _i, _i]),
    "ane_cuda_adam_update": (_i, [_fp, _fp, C.POINTER(AdamState), _i, _f, _f, _f, _f]),
    "ane_cuda_adam_update_wd": (_i, [_fp, _fp, C.POINTER(AdamState), _i, _f, _f, _f, _f, _f]),
    "ane_cuda_cross_entropy_loss": (_i, [_fp, _fp, _fp, _u16p, _i, _i]),
    "ane_cuda_embed_lookup": (_i, [_fp, _fp, _u16p, _i, _i, _i]),
    "ane_cuda_embed_backward": (_i, [_fp, _fp, _u16p, _i, _i, _i]),
    "ane_cuda_rope_backward_inplace": (_i, [_fp, _i, _i, _i]),
    "ane_cuda_residual": (_i, [_fp, _fp, _fp, _f, _sz]),
    "ane_cuda_swiglu": (_i, [_fp, _fp, _fp, _sz]),
    "ane_cuda_swiglu_bwd": (_i, [_fp, _fp, _fp, _fp, _fp, _sz]),
    # batched host-buffer forms
    "ane_cuda_rmsnorm_host": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _f]),
    "ane_cuda_rmsnorm_bwd_host": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _u]),
    "ane_cuda_residual_host": (_i, [_i, _sz, _vp, _vp, _vp, _f]),
    "ane_cuda_residual_rmsnorm_host": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f]),
    "ane_cuda_swiglu_host": (_i, [_i, _sz, _vp, _vp, _vp]),
    "ane_cuda_swiglu_bwd_host": (_i, [_i, _sz, _vp, _vp, _vp, _vp, _vp]),
    "ane_cuda_rope_host": (_i, [_i, _i, _i, _i, _i, _vp, _vp, _f, _i, _u]),
    "ane_cuda_qknorm_rope_host": (_i, [_i, _i, _i, _i, _i, _vp, _vp, _vp, _f, _f, _i]),
    "ane_cuda_rope_qknorm_bwd_host": (_i, [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _u]),
    # device-resident operators
    "ane_cuda_rmsnorm_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _f]),
    "ane_cuda_rmsnorm_bwd_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _u]),
    "ane_cuda_rmsnorm_bwd_static_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _u]),
    "ane_cuda_residual_dev": (_i, [_vp, _i, _sz, _vp, _vp, _vp, _f]),
    "ane_cuda_scale_dev": (_i, [_vp, _i, _sz, _vp, _vp, _f]),
    "ane_cuda_residual_rmsnorm_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f]),
    "ane_cuda_swiglu_dev": (_i, [_vp, _i, _sz, _vp, _vp, _vp]),
    "ane_cuda_swiglu_bwd_dev": (_i, [_vp, _i, _sz, _vp, _vp, _vp, _vp, _vp]),
    "ane_cuda_rope_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _f, _i, _u]),
    "ane_cuda_qknorm_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _f]),
    "ane_cuda_qknorm_bwd_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _u]),
    "ane_cuda_qknorm_rope_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _f, _f, _i]),
    "ane_cuda_rope_qknorm_bwd_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _u]),
    "ane_cuda_qknorm_rope_pair_dev": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _i]),
    "ane_cuda_rope_qknorm_bwd_pair_dev": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _u]),
    "ane_cuda_embed_lookup_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _u]),
    "ane_cuda_embed_backward_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i]),
    "ane_cuda_cross_entropy_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _f]),
    "ane_cuda_adam_dev": (_i, [_vp, _sz, _vp, _vp, _vp, _vp, _i, _f, _f, _f, _f, _f, _f, _vp, _u]),
    "ane_cuda_grad_norm_sq_dev": (_i, [_vp, _sz, _vp, _f, _vp]),
    "ane_cuda_clip_factor_dev": (_i, [_vp, _vp, _i, _f, _vp]),
    # layout helpers
    "ane_cuda_qknorm_rope_tiled_dev": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _f, _f, _i]),
    "ane_cuda_rope_qknorm_bwd_gqa_dev": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _u]),
    "ane_cuda_gqa_tile_dev": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "ane_cuda_gqa_reduce_dev": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "ane_cuda_convert_dev": (_i, [_vp, _i, _i, _sz, _vp, _vp]),
    "ane_cuda_pack_dyn_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "ane_cuda_vocab_map_build_dev": (_i, [_vp, _i, _sz, _vp, _i, _vp, _vp, _vp]),
    "ane_cuda_vocab_compact_embed_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "ane_cuda_vocab_scatter_grads_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "ane_cuda_vocab_update_full_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    # optimizer step over peer memory
    "ane_cuda_p2p_reduce_dev": (_i, [_vp, _i, _vp, _sz, _sz, _vp, _f, _vp, _vp]),
    "ane_cuda_p2p_reduce_limited_dev": (_i, [_vp, _i, _vp, _sz, _sz, _vp, _f, _vp, _vp, _i]),
    "ane_cuda_p2p_adam_dev": (_i, [_vp, _i, _i, _vp, _sz, _sz, _vp, _vp, _vp, _i, _f, _f, _f, _f, _f, _f, _vp, _u]),
    # operator chain with host buffers
    "ane_cuda_chain_create": (_vp, [_vp, _i, _vp]),
    "ane_cuda_chain_step": (_i, [_vp, _vp]),
    "ane_cuda_chain_sync": (_i, [_vp]),
    "ane_cuda_chain_compute_stream": (_vp, [_vp]),
    "ane_cuda_chain_h2d_bytes": (_sz, [_vp]),
    "ane_cuda_chain_d2h_bytes": (_sz, [_vp]),
    "ane_cuda_chain_destroy": (None, [_vp]),
    # multi-GPU group
    "ane_cuda_comm_unique_id": (_i, [_vp]),
    "ane_cuda_comm_init": (_i, [_i, _i, _vp, C.c_double]),
    "ane_cuda_comm_size": (_i, []),
    "ane_cuda_comm_rank": (_i, []),
    "ane_cuda_comm_destroy": (_i, []),
    "ane_cuda_comm_wait": (_i, [_vp, C.c_double]),
    "ane_cuda_allreduce_f32": (_i, [_vp, _vp, _sz]),
    "ane_cuda_comm_map_peers": (_i, [_vp, _vp, _sz]),
    "ane_cuda_comm_unmap_peers": (_i, []),
    "ane_cuda_sharded_adam_step": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i, _f, _f, _f, _f, _f, _f, _f, _u, _vp]),
    # checkpoints
    "ane_cuda_ckpt_read_header": (_i, [C.c_char_p, _vp]),
    "ane_cuda_ckpt_param_count": (_sz, [_vp]),
    "ane_cuda_ckpt_load": (_i, [C.c_char_p, _vp, _vp, _vp, _vp, _sz]),
    "ane_cuda_ckpt_save": (_i, [C.c_char_p, _vp, _vp, _vp, _vp, _sz]),
    "ane_cuda_ckpt_load_flat": (_i, [C.c_char_p, _vp, _vp, _vp, _vp, _sz]),
    "ane_cuda_ckpt_save_flat": (_i, [C.c_char_p, _vp, _vp, _vp, _vp, _sz]),
    "ane_cuda_ckpt_flat_decay_count": (_sz, [_vp]),
    "ane_cuda_ckpt_tensor_offset": (_i, [_vp, _i, _i, _i, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "ane_cuda_llama2c_read_config": (_i, [C.c_char_p, _vp]),
    "ane_cuda_llama2c_to_header": (_i, [_vp, _vp]),
    "ane_cuda_llama2c_load": (_i, [C.c_char_p, _vp, _vp, _vp, _sz, _i]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared object and declare the prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m ane_b200.build` (needs nvcc). "
            "libane_cuda has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != OK:
        raise AneCudaError(rc, load().ane_cuda_last_error().decode("utf-8", "replace"))


def init(device: int = 0) -> None:
    check(load().ane_cuda_init(int(device)))
    # ANE_CUDA_TUNING="knob=value,knob=value": kernel-selection knobs for benchmarking
    for item in filter(None, os.environ.get("ANE_CUDA_TUNING", "").split(",")):
        name, _, value = item.partition("=")
        set_tuning(name.strip(), int(value))


def set_tuning(name: str, value: int) -> None:
    check(load().ane_cuda_set_tuning(name.encode(), int(value)))


def clear_tuning(name=None) -> None:
    check(load().ane_cuda_clear_tuning(name.encode() if name is not None else None))


def launch_count() -> int:
    return int(load().ane_cuda_launch_count())


def reset_launch_count() -> None:
    load().ane_cuda_reset_launch_count()


def poll_status(reset: bool = True) -> Status:
    s = Status()
    check(load().ane_cuda_poll_status(C.byref(s), int(reset)))
    return s

"""Checkpoints of the reference's training loops ("BLZT" files, version 2 of training/train_large.m and
version 4 of training/training_dynamic/train.m) to and from flat device buffers, through the C ABI
(`ane_cuda_ckpt_*`, implemented in csrc/ckpt.cu).

Device layout ("weight order"): per layer Wq Wk Wv Wo W1 W2 W3 rms_att rms_ffn, then rms_final, then
embed -- the file's order with the Adam moments taken out -- in three parallel fp32 buffers w, m, v.

"Optimizer order" (the ``*_flat`` functions) is the arrangement of ``layer_chain.FlatParams``:
[per-layer matrices | embed | rms_att of all layers | rms_ffn of all layers | rms_final | QK-norm weights], weight
decay on the first two blocks only.  The reference's files hold no QK-norm weights: a load leaves them (and their
moments) as they are in the destination buffers, a save drops them.

Also here: the llama2.c weight-file loader of training/train_large.m:13-56.
"""
from __future__ import annotations

import ctypes as C

from . import lib as _l

MAGIC = 0x424C5A54


class CkptHeader(C.Structure):
    """training/stories_config.h:95-104 (version 2), training_dynamic/config.h:78-86 (version 4); 96 bytes."""
    _fields_ = [("magic", C.c_int), ("version", C.c_int), ("step", C.c_int), ("total_steps", C.c_int),
                ("n_layers", C.c_int), ("vocab_size", C.c_int), ("dim", C.c_int), ("hidden_dim", C.c_int),
                ("n_heads", C.c_int), ("seq_len", C.c_int), ("lr", C.c_float), ("loss", C.c_float),
                ("cum_compile", C.c_double), ("cum_train", C.c_double), ("cum_wall", C.c_double),
                ("cum_steps", C.c_int), ("cum_batches", C.c_int), ("adam_t", C.c_int),
                ("kv_heads", C.c_int), ("head_dim", C.c_int), ("q_dim", C.c_int)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def read_header(path: str) -> CkptHeader:
    h = CkptHeader()
    _l.check(_l.load().ane_cuda_ckpt_read_header(path.encode(), C.byref(h)))
    return h


def param_count(h: CkptHeader) -> int:
    return int(_l.load().ane_cuda_ckpt_param_count(C.byref(h)))


def layer_tensors(h: CkptHeader):
    """(name, element count) of the nine per-layer tensors in file order."""
    q_dim, kv_dim = (h.q_dim, h.kv_heads * h.head_dim) if h.version >= 4 else (h.dim, h.dim)
    d, hid = h.dim, h.hidden_dim
    return [("Wq", q_dim * d), ("Wk", kv_dim * d), ("Wv", kv_dim * d), ("Wo", d * q_dim), ("W1", hid * d), ("W2", d * hid),
            ("W3", hid * d), ("rms_att", d), ("rms_ffn", d)]


def load(path: str, with_moments: bool = True, device="cuda"):
    """-> (header, w, m, v): flat fp32 CUDA tensors in weight order (m, v are None without moments)."""
    import torch
    h = read_header(path)
    n = param_count(h)
    w = torch.empty(n, dtype=torch.float32, device=device)
    m = torch.empty_like(w) if with_moments else None
    v = torch.empty_like(w) if with_moments else None
    _l.check(_l.load().ane_cuda_ckpt_load(path.encode(), C.byref(h), w.data_ptr(), m.data_ptr() if with_moments else None,
                                         v.data_ptr() if with_moments else None, n))
    return h, w, m, v


def save(path: str, h: CkptHeader, w, m, v) -> None:
    for t in (w, m, v):
        if not (t.is_cuda and t.is_contiguous() and t.dtype.is_floating_point and t.element_size() == 4):
            raise ValueError("expected contiguous fp32 CUDA tensors")
    _l.check(_l.load().ane_cuda_ckpt_save(path.encode(), C.byref(h), w.data_ptr(), m.data_ptr(), v.data_ptr(), w.numel()))


TENSORS = ("Wq", "Wk", "Wv", "Wo", "W1", "W2", "W3", "rms_att", "rms_ffn", "rms_final", "embed")


def tensor_range(h: CkptHeader, name: str, layer: int = 0, flat: bool = False):
    """(offset, count) in floats of one tensor in weight order (flat=False) or optimizer order (flat=True)."""
    off, cnt = C.c_size_t(), C.c_size_t()
    _l.check(_l.load().ane_cuda_ckpt_tensor_offset(C.byref(h), int(flat), TENSORS.index(name), layer, C.byref(off), C.byref(cnt)))
    return off.value, cnt.value


def flat_decay_count(h: CkptHeader) -> int:
    """Length of the leading range of optimizer order that takes weight decay (matrices and embedding)."""
    return int(_l.load().ane_cuda_ckpt_flat_decay_count(C.byref(h)))


def load_flat(path: str, w, m=None, v=None) -> CkptHeader:
    """File -> the first param_count floats of w (and m, v) in optimizer order; the rest of the buffers is untouched."""
    h = CkptHeader()
    _l.check(_l.load().ane_cuda_ckpt_load_flat(path.encode(), C.byref(h), w.data_ptr(), m.data_ptr() if m is not None else None,
                                              v.data_ptr() if v is not None else None, w.numel()))
    return h


def save_flat(path: str, h: CkptHeader, w, m, v) -> None:
    _l.check(_l.load().ane_cuda_ckpt_save_flat(path.encode(), C.byref(h), w.data_ptr(), m.data_ptr(), v.data_ptr(), w.numel()))


def header_for(cfg, step: int = 0, adam_t: int = 0, lr: float = 0.0, loss: float = 0.0) -> CkptHeader:
    """Version-4 header of a layer_chain.ChainConfig (training_dynamic/config.h:78-86)."""
    h = CkptHeader()
    h.magic, h.version, h.step, h.adam_t, h.lr, h.loss = MAGIC, 4, step, adam_t, lr, loss
    h.n_layers, h.vocab_size, h.dim, h.hidden_dim, h.n_heads, h.seq_len = cfg.layers, cfg.vocab, cfg.dim, cfg.hidden, cfg.heads, cfg.seq
    h.kv_heads, h.head_dim, h.q_dim = cfg.kv_heads, cfg.head_dim, cfg.heads * cfg.head_dim
    return h


class Llama2cConfig(C.Structure):
    """training/stories_config.h:108-110"""
    _fields_ = [(n, C.c_int) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len")]


def llama2c_read_config(path: str) -> Llama2cConfig:
    c = Llama2cConfig()
    _l.check(_l.load().ane_cuda_llama2c_read_config(path.encode(), C.byref(c)))
    return c


def llama2c_load(path: str, expect: Llama2cConfig | None = None, flat: bool = False, device="cuda", out=None):
    """-> (checkpoint header describing the model, w): the weights of a llama2.c file as a flat fp32 CUDA tensor in
    weight order, or in optimizer order when flat (then `out` may be a longer buffer, e.g. FlatParams.w)."""
    import torch
    c = llama2c_read_config(path)
    h = CkptHeader()
    _l.check(_l.load().ane_cuda_llama2c_to_header(C.byref(c), C.byref(h)))
    w = torch.empty(param_count(h), dtype=torch.float32, device=device) if out is None else out
    _l.check(_l.load().ane_cuda_llama2c_load(path.encode(), C.byref(expect) if expect is not None else None, C.byref(h), w.data_ptr(),
                                            w.numel(), int(flat)))
    return h, w

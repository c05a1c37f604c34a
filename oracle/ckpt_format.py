"""Test infrastructure: numpy restatement of the reference's checkpoint writer, used only by tests to produce files
the way save_checkpoint does (training/train_large.m:109-145 for version 2, training/training_dynamic/train.m:104-138
for version 4).  The product's reader/writer (ane_b200/csrc/ckpt.cu) is checked against files made here.

Parity unpinned against reference binaries: both writers live in Objective-C main files that do not compile here and
the repository ships no checkpoint file; the restatement follows the fwrite sequence line by line."""
import struct

import numpy as np

MAGIC = 0x424C5A54
HEADER_FMT = "<10i2f3d3i3i"          # stories_config.h:95-104 / training_dynamic/config.h:78-86
assert struct.calcsize(HEADER_FMT) == 96


def sizes(version, n_layers, vocab, dim, hidden, n_heads, kv_heads=0, head_dim=0, q_dim=0):
    """element counts of Wq Wk Wv Wo W1 W2 W3 rms_att rms_ffn (train.m:119-122; train_large.m:126-129 uses WQ_SZ
    for all of Wq, Wk, Wv)"""
    if version >= 4:
        kv_dim = kv_heads * head_dim
        return [q_dim * dim, kv_dim * dim, kv_dim * dim, dim * q_dim, hidden * dim, dim * hidden, hidden * dim, dim, dim]
    return [dim * dim] * 4 + [hidden * dim, dim * hidden, hidden * dim, dim, dim]


def write(path, hdr, layers, rms_final, embed):
    """hdr: dict of header fields; layers: list of 9 (w, m, v) triples per layer; rms_final, embed: (w, m, v)."""
    h = struct.pack(HEADER_FMT, MAGIC, hdr["version"], hdr["step"], hdr["total_steps"], hdr["n_layers"], hdr["vocab_size"],
                    hdr["dim"], hdr["hidden_dim"], hdr["n_heads"], hdr["seq_len"], hdr["lr"], hdr["loss"],
                    hdr.get("cum_compile", 0.0), hdr["cum_train"], hdr["cum_wall"], hdr["cum_steps"], hdr.get("cum_batches", 0),
                    hdr["adam_t"], hdr.get("kv_heads", 0), hdr.get("head_dim", 0), hdr.get("q_dim", 0))
    with open(path, "wb") as f:
        f.write(h)
        for tensors in layers:
            for w, _, _ in tensors:                   # weights first (train.m:119-122)
                f.write(np.ascontiguousarray(w, np.float32).tobytes())
            for _, m, v in tensors:                   # then m, v of each (train.m:123-131)
                f.write(np.ascontiguousarray(m, np.float32).tobytes())
                f.write(np.ascontiguousarray(v, np.float32).tobytes())
        for t in rms_final:                           # train.m:133-134
            f.write(np.ascontiguousarray(t, np.float32).tobytes())
        for t in embed:                               # train.m:135-136
            f.write(np.ascontiguousarray(t, np.float32).tobytes())


def weight_order(layers, rms_final, embed, which):
    """flat array of the w (which=0), m (1) or v (2) parts in weight order"""
    parts = [t[which].ravel() for tensors in layers for t in tensors] + [rms_final[which].ravel(), embed[which].ravel()]
    return np.concatenate(parts).astype(np.float32)


LLAMA2C_FMT = "<7i"                   # stories_config.h:108-110


def write_llama2c(path, dim, hidden, n_layers, n_heads, n_kv_heads, vocab, seq_len, layers, rms_final, embed, shared=True,
                  trailing=b""):
    """A llama2.c weight file in the order load_pretrained reads it (training/train_large.m:28-50): header, embed, then
    rms_att, wq, wk, wv, wo, rms_ffn, w1, w2, w3 each for all layers, rms_final.  layers: per layer the nine weight
    arrays in CHECKPOINT order (Wq Wk Wv Wo W1 W2 W3 rms_att rms_ffn).  A negative vocab_size in the header marks an
    unshared classifier (train_large.m:25-26); `trailing` stands for what follows rms_final in real files."""
    order = [7, 0, 1, 2, 3, 8, 4, 5, 6]
    with open(path, "wb") as f:
        f.write(struct.pack(LLAMA2C_FMT, dim, hidden, n_layers, n_heads, n_kv_heads, vocab if shared else -vocab, seq_len))
        f.write(np.ascontiguousarray(embed, np.float32).tobytes())
        for k in order:
            for tensors in layers:
                f.write(np.ascontiguousarray(tensors[k], np.float32).tobytes())
        f.write(np.ascontiguousarray(rms_final, np.float32).tobytes())
        f.write(trailing)


def optimizer_order(layers, rms_final, embed, which):
    """flat array of the w (which=0), m (1) or v (2) parts in optimizer order:
    [per-layer matrices | embed | rms_att[all] | rms_ffn[all] | rms_final]"""
    parts = [t[which].ravel() for tensors in layers for t in tensors[:7]] + [embed[which].ravel()]
    parts += [tensors[7][which].ravel() for tensors in layers] + [tensors[8][which].ravel() for tensors in layers]
    parts.append(rms_final[which].ravel())
    return np.concatenate(parts).astype(np.float32)

"""Test infrastructure: pure-Python restatement of the reference's on-disk formats, the checker for the
library's host-side readers and writers. Only tests import this; the product never does.
parity unpinned: the reference ships no weight file and no test vectors for these functions; the format is
pinned by its own reader and writer, restated below from their sources."""
from __future__ import annotations

import struct

import numpy as np


def write_wts(path, blobs):
    """The exporter's loop (tools/gen_wts.py:85-99): count line, then per blob `name count ` and for every
    value a space and the hex of its big-endian fp32 bytes, newline."""
    items = list(blobs.items()) if isinstance(blobs, dict) else list(blobs)
    with open(path, "w") as f:
        f.write("{}\n".format(len(items)))
        for k, v in items:
            vr = np.asarray(v, dtype=np.float32).reshape(-1)
            f.write("{} {} ".format(k, len(vr)))
            for bits in vr.view(np.uint32).tolist():       # bit pattern, so that NaN payloads survive
                f.write(" ")
                f.write(struct.pack(">I", bits).hex())
            f.write("\n")


def read_wts(path):
    """loadWeights (se-ssd-ai-trt.cpp:278-314): white-space separated tokens; decimal blob count; per blob a
    name, a decimal size and `size` hexadecimal 32-bit words that are the values' bit patterns. Returns a dict
    (a repeated name keeps the last blob, as std::map assignment does)."""
    with open(path) as f:
        tok = f.read().split()
    pos = 0
    count = int(tok[pos]); pos += 1
    assert count > 0
    out = {}
    for _ in range(count):
        name, size = tok[pos], int(tok[pos + 1]); pos += 2
        words = np.array([int(t, 16) for t in tok[pos:pos + size]], dtype=np.uint32)
        assert words.size == size
        pos += size
        out[name] = words.view(np.float32)
    return out


def fold_batchnorm(gamma, beta, mean, var, eps):
    """add_batchNorm1d_relu's scale and shift arrays (se-ssd-ai-trt.cpp:808-826), evaluated in fp32."""
    g, b, m, v = (np.asarray(a, dtype=np.float32) for a in (gamma, beta, mean, var))
    root = np.sqrt(v + np.float32(eps), dtype=np.float32)
    return (g / root).astype(np.float32), (b - m * g / root).astype(np.float32)


def read_points(path, max_points):
    """loadData (se-ssd-ai-trt.cpp:1515-1556) + the size rule at :1848: the file's bytes at the start of a
    zeroed [max_points][4] fp32 buffer, points = bytes // 16; None when the file does not fit (the reference exits)."""
    raw = open(path, "rb").read()
    if len(raw) > max_points * 16:
        return None
    buf = np.zeros(max_points * 16, np.uint8)
    buf[:len(raw)] = np.frombuffer(raw, np.uint8)
    return buf.view(np.float32).reshape(max_points, 4), len(raw) // 16

"""Expected results of the dense ternary projections (gpre_dense, gpu_pre.m:235-256) in numpy: per-token absmax int8
(maple.c:184-194), int32 dot of the unpacked codes (layout of convert.py:29-33), (float)(tot - qsum) * qs * s[r] with two fp32
roundings (maple.c:425-458).  Used by the CPU test (against the compiled reference's tdot) and the GPU parity test."""
import numpy as np


def unpack(codes, rows, cols):
    """codes: uint8 [rows][cols/4]; byte j of a 32-byte group holds columns j, j+32, j+64, j+96 at bits 0,2,4,6.  Returns t in {-1,0,1}."""
    c = np.asarray(codes, np.uint8).reshape(rows, cols // 128, 32)
    t = np.stack([(c >> s) & 3 for s in (0, 2, 4, 6)], axis=2).astype(np.int64) - 1        # [rows][group][k][j] -> column 32k + j
    return t.reshape(rows, cols)


def prep(x):
    x = np.asarray(x, np.float32)
    mx = np.abs(x).max(axis=1)
    qs = np.where(mx > 0, mx / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / qs).astype(np.float32)
    q = np.rint((x * inv[:, None]).astype(np.float32)).astype(np.int64)
    return q, qs


def dense(codes, scales, rows, cols, x):
    t = unpack(codes, rows, cols)
    q, qs = prep(x)
    d = (q @ t.T).astype(np.float32)                                  # |dot| < 2^24: exact in fp32
    return ((d * qs[:, None]).astype(np.float32) * np.asarray(scales, np.float32)[None, :]).astype(np.float32)

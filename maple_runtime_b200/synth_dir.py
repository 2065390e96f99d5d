"""A synthetic checkpoint directory in the converter's on-disk format (convert.py, layout.py of the reference): shard-0000N.bin
files plus layout.bin, filled by this package's counter-based generator, so that the loader (gmoe_load_layers), or the reference
itself, can be pointed at something when the real checkpoint is absent.

layout.bin: packed 26-byte records '<BBQQII' = kind ('t' ternary | 'b' bf16), shard 0..8, data offset, scale offset, rows, cols, in the
order embeddings, head, final norm, then per layer: input norm, post-attention norm, q norm, k norm, router, q, k, v, o and per
expert gate, up, down (layout.py:1-22).  Ternary tensors are 2-bit packed as pack_ternary does (convert.py:29-33): a 128-column
group is 32 bytes, byte j holds columns j, j+32, j+64, j+96 at bits 0, 2, 4, 6, code = t + 1; one fp32 scale per row."""
import os
import struct
import numpy as np

from . import lib as ml

C = ml.CONST


def pack_ternary(t):
    """t: int array [rows][cols] of -1, 0, +1 (cols a multiple of 128) -> uint8 [rows][cols/4] in the converter's layout."""
    rows, cols = t.shape
    c = (np.asarray(t) + 1).astype(np.uint8).reshape(rows, cols // 128, 4, 32)
    out = np.zeros((rows, cols // 128, 32), np.uint8)
    for k in range(4):
        out |= (c[:, :, k, :] << (2 * k)).astype(np.uint8)
    return np.ascontiguousarray(out.reshape(rows, cols // 4))


def write(dirname, clib, seed, layer_ids, split_experts_at=128):
    """Writes len(layer_ids) layers: directory layer i holds the synthetic layer layer_ids[i] of `seed`.  The experts of a layer
    are split over two shard files at `split_experts_at` so that a layer spans two regions, as real layers sometimes do.
    Returns {"dense": [(q, k, v, o) as (codes, scales) per layer]} for tests."""
    os.makedirs(dirname, exist_ok=True)
    shards = [bytearray() for _ in range(9)]
    recs = []

    def put(k, data):
        while len(shards[k]) % 64:
            shards[k].append(0)
        off = len(shards[k]); shards[k] += bytes(data); return off

    def bf16_rec(k, arr, rows, cols):
        recs.append((ord('b'), k, put(k, np.ascontiguousarray(arr, np.uint16).tobytes()), 0, rows, cols))
    ones = np.full(2048, 0x3F80, np.uint16)
    bf16_rec(0, ones[:64], 64, 1); bf16_rec(0, ones[:64], 64, 1); bf16_rec(0, ones, 2048, 1)       # embeddings, head (stand-ins), final norm
    rng = np.random.default_rng(seed & 0xFFFFFFFF)
    dense = []
    for i, L in enumerate(layer_ids):
        ka, kb = (2 * i) % 9, (2 * i + 1) % 9
        bf16_rec(ka, ones, 2048, 1)                                        # input norm
        bf16_rec(ka, ml.synth_norm(clib, seed, L), 2048, 1)                 # post-attention norm
        bf16_rec(ka, ones[:128], 128, 1); bf16_rec(ka, ones[:128], 128, 1)  # q norm, k norm
        bf16_rec(ka, ml.synth_router(clib, seed, L), 256, 2048)
        mats = []
        for rows in (2048, 512, 512, 2048):                                # q, k, v, o
            codes = pack_ternary(rng.choice(np.array([-1, 0, 1]), size=(rows, 2048), p=[0.3, 0.4, 0.3]))
            scales = rng.uniform(0.01, 0.05, rows).astype(np.float32)
            recs.append((ord('t'), ka, put(ka, codes.tobytes()), put(ka, scales.tobytes()), rows, 2048))
            mats.append((codes, scales))
        dense.append(mats)
        ex = np.asarray(ml.synth_experts(clib, seed, L, 0, 256), np.uint8).reshape(256, C.EXPERT_BYTES)
        for e in range(256):
            k = ka if e < split_experts_at else kb
            base = put(k, ex[e].tobytes())
            recs.append((ord('t'), k, base, base + C.GU_CODES, 512, 2048))
            recs.append((ord('t'), k, base + C.GU_BYTES, base + C.GU_BYTES + C.GU_CODES, 512, 2048))
            recs.append((ord('t'), k, base + 2 * C.GU_BYTES, base + 2 * C.GU_BYTES + C.GU_CODES, 2048, 512))
    for k in range(9):
        if shards[k]:
            with open(os.path.join(dirname, f"shard-{k + 1:05d}.bin"), "wb") as f:
                f.write(shards[k])
    with open(os.path.join(dirname, "layout.bin"), "wb") as f:
        for r in recs:
            f.write(struct.pack("<BBQQII", *r))
    return {"dense": dense}

"""The first step of the attention half on the card (gmoe_qk_rope; the reference's kernel `qkn`, gpu_full.metal:32-71, and its CPU form
maple.c:711-717): RMS norm of the query and key heads, half-rotary embedding on local layers, fp16 key and value rows.  Compared bit for
bit with the oracle's restatement (which the CPU suite pins to the compiled reference) and with the compiled reference where it is here."""
import numpy as np
import pytest

from test_oracle import attention_head_case

pytestmark = pytest.mark.gpu


def bf16_to_f32(w):
    return (w.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("nb,glob,seed", [(1, 0, 51), (64, 0, 52), (64, 1, 53), (700, 0, 54), (2048, 0, 55), (2048, 1, 56)])
def test_attention_head_equals_oracle(nb, glob, seed, gpu, oracle):
    from oracle import oracle as orc
    q, k, v, qn, kn, pos = attention_head_case(seed, nb)
    positions = 4096
    i = np.arange(32); inv = 1.0 / np.power(10000.0, (2.0 * i) / 64)                      # maple.c:1085
    f = np.arange(positions)[:, None] * inv[None, :]
    cs = np.stack([np.cos(f), np.sin(f)], -1).astype(np.float32)                          # maple.c:1151-1153
    if orc.Reference.available():
        cs = orc.Reference().rope_table(positions)                                        # the table exactly as maple.c builds it with this libm
    want_q, _, want_kc, want_vc = oracle.qk_rope(q, k, v, qn, kn, pos, cs, glob)
    gpu.rope_table(cs)
    got_q, got_kc, got_vc, _ = gpu.qk_rope(np.concatenate([q, k, v], 1), pos, glob, bf16_to_f32(qn), bf16_to_f32(kn))
    assert np.array_equal(got_q.view(np.uint32), want_q.view(np.uint32)), f"{int((got_q.view(np.uint32) != want_q.view(np.uint32)).sum())} q values differ"
    assert np.array_equal(got_kc, want_kc) and np.array_equal(got_vc, want_vc)
    if orc.Reference.available():
        ref_q, _, ref_kc, ref_vc = orc.Reference().qk_rope(q, k, v, qn, kn, pos, glob)
        assert np.array_equal(got_q.view(np.uint32), ref_q.view(np.uint32)) and np.array_equal(got_kc, ref_kc) and np.array_equal(got_vc, ref_vc)


def test_attention_head_rejects_bad_arguments(gpu, clib):
    q, k, v, qn, kn, pos = attention_head_case(57, 8)
    cs = np.zeros((16, 32, 2), np.float32); cs[..., 0] = 1.0
    gpu.rope_table(cs)
    pos[:] = 3; pos[5] = 16                                                               # one position past the table
    with pytest.raises(RuntimeError, match="outside the table"):
        gpu.qk_rope(np.concatenate([q, k, v], 1), pos, 0, bf16_to_f32(qn), bf16_to_f32(kn))
    gpu.qk_rope(np.concatenate([q, k, v], 1), pos, 1, bf16_to_f32(qn), bf16_to_f32(kn))     # a global layer does not read the table
    assert clib.gmoe_rope_table(None, 4) < 0

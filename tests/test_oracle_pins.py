"""CPU tests of the oracle itself: the reference's own pins for this path, the
C restatement against its numpy twin, and the invariants the reference's GPU
integration tests rely on (decode path == prefill path for the same token)."""
import struct

import numpy as np
import pytest

from bonsai_pot_b200 import synth
from oracle import oracle as O
from tests.helpers import build_decode_case, within_tolerance


# ---- pins taken from the reference's unit tests ---------------------------------

def test_payload_sizes_pinned_by_reference():
    # src/kv_snapshot.rs:430-449, 516-520
    assert O.payload_bytes(36, 1024, 512) == 42_467_328
    assert O.payload_bytes(36, 1024, 32768) == 2_717_908_992
    assert O.payload_bytes(36, 1024, 0) == 0


def test_payload_offsets_do_not_overlap():
    # src/kv_snapshot.rs:451-468
    n_layer, kv_dim, pos = 36, 1024, 16
    for kind in range(2):
        for il in range(n_layer):
            d_start = O.payload_offset(n_layer, kv_dim, pos, kind, il, 0)
            d_end = d_start + pos * (kv_dim // 32) * 4
            qs_start = O.payload_offset(n_layer, kv_dim, pos, kind, il, 1)
            qs_end = qs_start + pos * kv_dim
            assert d_end <= qs_start
            if il + 1 < n_layer:
                assert qs_end <= O.payload_offset(n_layer, kv_dim, pos, kind, il + 1, 0)
    assert O.payload_offset(n_layer, kv_dim, pos, 1, 0, 0) == O.payload_bytes(n_layer, kv_dim, pos) // 2


def test_snapshot_header_roundtrip_and_rejects():
    # src/kv_snapshot.rs:392-428, 470-495
    sh = O.Shape(n_layer=36, max_seq=1024)
    pos = 4
    payload = bytes(i & 0xFF for i in range(O.payload_bytes(36, 1024, pos)))
    blob = O.MAGIC + struct.pack("<6I", 1, 36, 1024, 1024, pos, 0) + payload
    assert len(blob) == 32 + len(payload)
    n_layer, kv_dim, max_seq, p, pl = O.snapshot_parse(blob)
    assert (n_layer, kv_dim, max_seq, p) == (36, 1024, 1024, pos) and pl == payload
    empty = O.MAGIC + struct.pack("<6I", 1, 36, 1024, 1024, 0, 0)
    assert len(empty) == O.HEADER_BYTES and O.snapshot_parse(empty)[3] == 0
    bad = bytearray(blob); bad[0] = 0xFF
    with pytest.raises(ValueError):
        O.snapshot_parse(bytes(bad))
    with pytest.raises(ValueError):
        O.snapshot_parse(blob[:-1])
    bad = bytearray(blob); bad[8:12] = struct.pack("<I", 2)
    with pytest.raises(ValueError):
        O.snapshot_parse(bytes(bad))
    bad = bytearray(blob); bad[28] = 1
    with pytest.raises(ValueError):
        O.snapshot_parse(bytes(bad))
    assert sh.kv_bytes == 36 * 1024 * (1024 + 128)


def test_rope_table_values_pinned_by_reference():
    # src/model.rs:2021-2045: head_dim 8, base 1e4, max_seq 4
    t = O.rope_table_f32(8, 10_000.0, 4)
    assert t.shape == (4 * 8,)
    assert abs(t[0] - 1.0) < 1e-6 and abs(t[1]) < 1e-6
    assert abs(t[8] - np.float32(np.cos(1.0))) < 1e-5
    assert abs(t[9] - np.float32(np.sin(1.0))) < 1e-5
    # position 0 is the identity rotation for every j
    assert np.all(t[0:8:2] == 1.0) and np.all(t[1:8:2] == 0.0)


def test_cache_layout_offsets():
    # src/forward.rs:48-58 and src/kv_snapshot.rs:172-180 agree
    L = O.lib()
    n_layer, max_seq, kv_dim = 36, 4096, 1024
    assert L.orc_kv_d_total(n_layer, max_seq, kv_dim) == n_layer * max_seq * 32 * 4
    for il in (0, 1, 35):
        assert L.orc_buf_d_offset(max_seq, kv_dim, il) == il * max_seq * 32 * 4
        assert L.orc_buf_qs_offset(n_layer, max_seq, kv_dim, il) == n_layer * max_seq * 128 + il * max_seq * kv_dim
    assert L.orc_kv_total_bytes(36, 32768, 1024) == 36 * 32768 * 1152


# ---- the restatement against itself ------------------------------------------------

def test_f16_conversions_match_numpy():
    L = O.lib()
    allh = np.arange(65536, dtype=np.uint16)
    back = np.array([L.orc_f16_to_f32(int(v)) for v in allh], dtype=np.float32)
    ref = allh.view(np.float16).astype(np.float32)
    same = (back.view(np.uint32) == ref.view(np.uint32)) | np.isnan(ref)
    assert same.all()
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * np.float32(8),
                        rng.standard_normal(2000).astype(np.float32) * np.float32(1e-5),
                        np.array([0, 6e-8, 3e-8, 2.98e-8, 65504, 65519.99, -65520, 5.96e-8, 8.94e-8], dtype=np.float32)])
    mine = np.array([L.orc_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(mine, x.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("pos_base,m", [(0, 1), (100, 64), (1000, 24)])
def test_c_oracle_equals_numpy_twin_bit_for_bit(pos_base, m):
    sh = O.Shape(n_layer=3, max_seq=1024)
    rope = O.rope_table_f16(sh)
    k = synth.tensor(3, 9, 1, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(3, 9, 1, synth.T_V_NEW, (m, sh.kv_dim))
    q = synth.tensor(3, 9, 1, synth.T_Q, (m, sh.q_dim))
    w = (1 + 0.1 * np.random.default_rng(5).standard_normal(128)).astype(np.float16)
    a_k, a_v, b_k, b_v = sh.new_cache(), sh.new_cache(), sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w, rope, a_k, a_v, 2, pos_base, m)
    O.np_kv_writeback(sh, k, v, w, rope, b_k, b_v, 2, pos_base, m)
    assert np.array_equal(a_k, b_k) and np.array_equal(a_v, b_v)
    qa = O.q_norm_rope(sh, q, w, rope, pos_base, m).view(np.uint16).reshape(m, sh.q_dim)
    qb = O.np_q_norm_rope(sh, q, w, rope, pos_base, m).view(np.uint16)
    assert np.array_equal(qa, qb)
    # only the addressed rows of the addressed layer were touched
    untouched = a_k.copy()
    sh.d_section(untouched, 2)[pos_base:pos_base + m] = 0
    sh.qs_section(untouched, 2)[pos_base:pos_base + m] = 0
    assert not untouched.any()


def test_quantiser_edge_cases():
    # all-zero block -> d = 0, q = 0; max magnitude maps to +-127; ties round to even
    sh = O.Shape(n_layer=1, n_head=4, n_kv_head=1, max_seq=4)
    x = np.zeros((1, 128), dtype=np.float16)
    x[0, 32:64] = np.linspace(-2, 2, 32).astype(np.float16)
    x[0, 64] = 127.0; x[0, 65] = 0.5; x[0, 66] = 1.5; x[0, 67] = 2.5; x[0, 68] = -0.5
    kv = sh.new_cache()
    O.quantize_rows(sh, x, kv, 0, 0, 1)
    d, q = sh.d_section(kv, 0)[0], sh.qs_section(kv, 0)[0]
    assert d[0] == 0 and not q[:32].any()
    assert q[32] == -127 and q[63] == 127
    assert d[2] == 1.0 and list(q[64:69]) == [127, 0, 2, 2, 0]
    # quantising the dequantised values reproduces the bytes
    deq = O.np_dequant(sh, kv, 0, 1).astype(np.float16)
    kv2 = sh.new_cache()
    O.quantize_rows(sh, deq, kv2, 0, 0, 1)
    assert np.array_equal(sh.qs_section(kv2, 0)[0], q)


def test_sensitivity_to_reduction_tree_and_contraction():
    """The V path has no freedom; the K path may move by an ulp with the order of
    the sum of squares or with FMA contraction. Report how much."""
    sh = O.Shape(n_layer=1, max_seq=64)
    rope = O.rope_table_f16(sh)
    m = 64
    k = synth.tensor(0, 0, 0, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(0, 0, 0, synth.T_V_NEW, (m, sh.kv_dim))
    w = synth.ones_weight()
    base_k, base_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w, rope, base_k, base_v, 0, 0, m)
    for tree, contract in ((1, 0), (2, 0), (0, 1)):
        a, b = sh.new_cache(), sh.new_cache()
        O.kv_writeback(sh, k, v, w, rope, a, b, 0, 0, m, tree=tree, contract=contract)
        assert np.array_equal(b, base_v)  # V bytes and scales never move
        dq = sh.qs_section(a, 0).astype(np.int32) - sh.qs_section(base_k, 0).astype(np.int32)
        assert np.abs(dq).max() <= 1
        rel = np.abs(sh.d_section(a, 0) - sh.d_section(base_k, 0)) / sh.d_section(base_k, 0)
        assert rel.max() < 1e-6  # a few ulp
        frac_scales = float((sh.d_section(a, 0) != sh.d_section(base_k, 0)).mean())
        print(f"tree={tree} contract={contract}: {frac_scales:.3f} of K scales differ, {int((dq != 0).sum())} K bytes differ")


@pytest.mark.parametrize("n_past", [0, 1, 15, 16, 17, 100, 512])
def test_decode_oracle_within_tolerance_of_exact_softmax(n_past):
    sh = O.Shape(n_layer=1, max_seq=1024)
    c = build_decode_case(sh, seed=0, cfg_id=0, layer=0, n_past=n_past)
    out = O.attn_decode(sh, c["qn"], c["kv_k"], c["kv_v"], 0, c["cur_pos"])
    exact = O.attn_exact(sh, c["qn"], c["kv_k"], c["kv_v"], 0, 1, n_past)[0]
    ok, max_abs, max_rel = within_tolerance(out.astype(np.float32), exact)
    assert ok, (max_abs, max_rel)
    parts = O.attn_split(sh, c["qn"], c["kv_k"], c["kv_v"], 0, c["cur_pos"])
    assert parts.shape == (sh.n_head, -(-c["cur_pos"] // 16), 130)
    assert np.array_equal(O.attn_merge(sh, parts).view(np.uint16), out.view(np.uint16))


def test_prefill_last_token_agrees_with_decode_path():
    """tests/gpu_integration.rs:122-139 cross-checks attention.wgsl against
    attention_split + attention_merge through the first generated token; here the
    same invariant is checked on the attention outputs directly."""
    sh = O.Shape(n_layer=1, max_seq=128)
    rope = O.rope_table_f16(sh)
    m = 70
    q = O.q_norm_rope(sh, synth.tensor(1, 2, 0, synth.T_Q, (m, sh.q_dim)), synth.ones_weight(), rope, 0, m)
    k = synth.tensor(1, 2, 0, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(1, 2, 0, synth.T_V_NEW, (m, sh.kv_dim))
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, synth.ones_weight(), rope, kv_k, kv_v, 0, 0, m)
    pre = O.attn_prefill(sh, q, kv_k, kv_v, 0, m)
    exact = O.attn_exact(sh, q, kv_k, kv_v, 0, m, 0)
    ok, max_abs, max_rel = within_tolerance(pre.astype(np.float32), exact)
    assert ok, (max_abs, max_rel)
    for tok in (0, 15, 16, 69):
        dec = O.attn_decode(sh, q[tok:tok + 1], kv_k, kv_v, 0, tok + 1)
        ok, max_abs, _ = within_tolerance(dec.astype(np.float32), pre[tok].astype(np.float32))
        assert ok and max_abs <= 1e-3


def test_oracle_is_deterministic():
    sh = O.Shape(n_layer=1, max_seq=256)
    c = build_decode_case(sh, seed=2, cfg_id=0, layer=0, n_past=200)
    a = O.attn_decode(sh, c["qn"], c["kv_k"], c["kv_v"], 0, c["cur_pos"])
    b = O.attn_decode(sh, c["qn"], c["kv_k"], c["kv_v"], 0, c["cur_pos"])
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))


def test_rsqrt_is_correctly_rounded():
    """The oracle's 1/sqrt (step 2 of kv_writeback_fused.wgsl / q_norm_rope_fused.wgsl, fixed here as
    the correctly rounded value) against an independent exact check in Python integers, on random and
    hand-picked inputs; then every float of [2^-20, 16) (201 million, the range `total / 128 + eps` can
    take for f16 inputs is inside it) through the C sweep, which re-checks the defining property and
    counts disagreements with the former long-double evaluation."""
    from fractions import Fraction
    lib = O.lib()
    rng = np.random.default_rng(11)
    xs = np.concatenate([
        np.exp(rng.uniform(np.log(1e-6), np.log(7e4), 4000)).astype(np.float32),
        np.array([1e-6, 1.0, 2.0, 4.0, 0.25, 3.0, 1.0 + 2.0 ** -23, 2.0 - 2.0 ** -23, 65504.0 ** 2 / 128], dtype=np.float32),
    ])
    for x in xs:
        r = np.float32(lib.orc_rsqrt_rn(float(x)))
        lo, hi = np.nextafter(r, np.float32(0)), np.nextafter(r, np.float32(np.inf))
        fx = Fraction(float(x))
        m_lo = (Fraction(float(lo)) + Fraction(float(r))) / 2
        m_hi = (Fraction(float(r)) + Fraction(float(hi))) / 2
        # m_lo < 1/sqrt(x) < m_hi  <=>  m_lo^2 x < 1 < m_hi^2 x
        assert m_lo * m_lo * fx < 1 < m_hi * m_hi * fx, float(x)
    first, last = 0x35800000, 0x41800000  # bit patterns of 2^-20 and 16.0
    differ = lib.orc_rsqrt_sweep(first, last - first, 1)
    assert differ != 2 ** 64 - 1, "the exact 1/sqrt violated its own rounding property"
    assert differ == 0, f"{differ} inputs where the long-double evaluation was not correctly rounded"

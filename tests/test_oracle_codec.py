"""The CPU oracle's codec against the golden vectors produced by the reference's own codec
(tests/golden/make_golden.py) and against the reference's published known answers."""
import numpy as np

from oracle import nvfp4_codec_oracle as oc


def test_edge_cases_known_scale_bytes(golden):
    # known answers of the reference's edge-case self-test (codec/nvfp4_codec.py:424-476)
    p, s = oc.encode(golden["edge_in"])
    assert s[:, 0].tolist() == [127, 127, 127, 132, 115, 127, 127]
    assert np.array_equal(p, golden["edge_packed"])
    assert np.array_equal(s, golden["edge_scales"])
    d = oc.decode(p, s)
    assert np.array_equal(d.view(np.uint16), golden["edge_dec"].view(np.uint16))
    # -0.0 is stored as +0: nibble 0
    assert np.all(p[5] == 0)


def test_random_matrices_bit_exact(golden):
    for i in range(int(golden["n_mats"])):
        m = golden[f"m{i}_in"]
        p, s = oc.encode(m)
        assert np.array_equal(p, golden[f"m{i}_packed"]), i
        assert np.array_equal(s, golden[f"m{i}_scales"]), i
        d = oc.decode(golden[f"m{i}_packed"], golden[f"m{i}_scales"])
        assert np.array_equal(d.view(np.uint16), golden[f"m{i}_dec"].view(np.uint16)), i


def test_scale_rule_exhaustive(golden):
    vals = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    assert np.array_equal(oc.block_scale_bytes(vals), golden["scale_all"])


def test_rounding_rule_exhaustive(golden):
    vals = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    for j, e in enumerate(golden["code_exps"]):
        got = oc.e2m1_codes((vals * 2.0 ** int(e)).astype(np.float32))
        assert np.array_equal(got, golden["code_all"][j]), int(e)


def test_ties_go_to_smaller_code():
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    assert oc.e2m1_codes(mids).tolist() == [0, 1, 2, 3, 4, 5, 6]
    assert oc.e2m1_codes(np.nextafter(mids, np.float32(10))).tolist() == [1, 2, 3, 4, 5, 6, 7]


def test_vectorised_decoder_rows(golden):
    d = oc.decode(golden["emb_packed"], golden["emb_scales"])
    assert np.array_equal(d[golden["emb_idx"]].view(np.uint16), golden["emb_rows"].view(np.uint16))


def test_byte_table_matches_decode():
    tbl = oc.byte_to_half_bits()
    packed = np.arange(256, dtype=np.uint8).reshape(32, 8)
    scales = np.full((32, 1), 127, dtype=np.uint8)
    d = oc.decode(packed, scales).view(np.uint16).reshape(256, 2)
    # +0 and -0 differ in bits: the codec never stores -0, the table keeps the sign bit
    same = (d == tbl) | ((d & 0x7FFF) == 0) & ((tbl & 0x7FFF) == 0)
    assert same.all()


def test_gemv_truth_recipe(golden):
    y = oc.gemv_ref_f32(golden["gemv_packed"], golden["gemv_scales"], golden["gemv_act"])
    np.testing.assert_allclose(y, golden["gemv_y_f32"], rtol=2e-6, atol=1e-7)
    y64 = oc.gemv_f64(golden["gemv_packed"], golden["gemv_scales"], golden["gemv_act"])
    assert oc.rel_error_floored(golden["gemv_y_f32"], y64).max() < 1e-5


def test_calibrated_quality_figures(golden):
    # published: cosine 0.9926, SNR 18.3 dB for the 16x16 sigma-0.3 matrix, seed 42
    cal = golden["cal_in"]
    p, s = oc.encode(cal)
    d = oc.decode(p, s)
    assert np.array_equal(d.view(np.uint16), golden["cal_dec"].view(np.uint16))
    a, b = cal.astype(np.float64).ravel(), d.astype(np.float64).ravel()
    cos = a @ b / (np.linalg.norm(a) * np.linalg.norm(b))
    snr = 10 * np.log10((a ** 2).mean() / ((a - b) ** 2).mean())
    assert abs(cos - 0.9926) < 5e-4
    assert abs(snr - 18.3) < 0.1


def test_roundtrip_error_bound():
    w = oc.synthetic_weight(64, 512, seed=3)
    p, s = oc.encode(w)
    d = oc.decode_f64(p, s)
    scale = np.exp2(s.astype(np.float64) - 127)
    err = np.abs(d - w.astype(np.float64)).reshape(64, -1, 16).max(axis=-1)
    assert np.all(err <= scale * 1.0 + 1e-12)  # half the widest code gap (4 <-> 6)


def test_empty_and_shapes():
    p, s = oc.encode(np.zeros((0, 32), dtype=np.float16))
    assert p.shape == (0, 16) and s.shape == (0, 2)
    p, s = oc.encode(np.zeros((3, 16), dtype=np.float16))
    assert np.all(s == 127) and np.all(p == 0)


def test_container_quantiser_matches_golden(golden):
    """The container writer's exact-arithmetic quantiser (frexp scale rule, midpoint counting)
    against the reference codec's bytes, and its packed-embedding reader against the reference's
    decoded rows."""
    import os
    import tempfile

    from nvfp4_v100_b200.pipeline import _qwen38_nvfp4_pack as pk

    for key in ["edge"] + [f"m{i}" for i in range(int(golden["n_mats"]))]:
        p, s = pk.encode_rows(golden[key + "_in"].astype(np.float32))
        assert np.array_equal(p, golden[key + "_packed"]), key
        assert np.array_equal(s, golden[key + "_scales"]), key
    vals = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    assert np.array_equal(pk.encode_block_scales(vals)[0], golden["scale_all"])
    for j, e in enumerate(golden["code_exps"]):
        a = (vals * 2.0 ** int(e)).astype(np.float32)
        assert np.array_equal(pk.e2m1_codes_rtn(a), golden["code_all"][j]), int(e)

    from nvfp4_v100_b200.pipeline._qwen38_infer import PackedEmb

    with tempfile.TemporaryDirectory() as d:
        np.save(os.path.join(d, "p.npy"), golden["emb_packed"])
        np.save(os.path.join(d, "s.npy"), golden["emb_scales"])
        emb = PackedEmb(os.path.join(d, "p.npy"), os.path.join(d, "s.npy"))
        rows = emb[golden["emb_idx"]].numpy()
        assert np.array_equal(rows.view(np.uint16), golden["emb_rows"].view(np.uint16))

"""launch_nvfp4_encode (device quantiser) against the codec oracle and the reference codec's golden
bytes: bit-exact, including the exhaustive scale and rounding rules."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_codec_oracle as oc
from tests.gpu_util import ptr, stream

pytestmark = pytest.mark.gpu


def encode_gpu(lib, w16: np.ndarray):
    M, K = w16.shape
    src = torch.from_numpy(np.ascontiguousarray(w16)).cuda()
    packed = torch.full((M * K // 2 + 16,), 0xAB, dtype=torch.uint8, device="cuda")
    scales = torch.full((M * K // 16 + 16,), 0xCD, dtype=torch.uint8, device="cuda")
    rc = lib.launch_nvfp4_encode(ptr(src), ptr(packed), ptr(scales), M, K, stream())
    torch.cuda.synchronize()
    assert rc == 0
    p, s = packed.cpu().numpy(), scales.cpu().numpy()
    assert (p[M * K // 2:] == 0xAB).all() and (s[M * K // 16:] == 0xCD).all()   # canaries
    return p[:M * K // 2].reshape(M, K // 2), s[:M * K // 16].reshape(M, K // 16)


def test_golden_matrices(lib, golden):
    for key in ["edge"] + [f"m{i}" for i in range(int(golden["n_mats"]))]:
        p, s = encode_gpu(lib, golden[key + "_in"])
        assert np.array_equal(p, golden[key + "_packed"]), key
        assert np.array_equal(s, golden[key + "_scales"]), key


def test_scale_rule_every_fp16_maximum(lib, golden):
    # one block per finite fp16 magnitude: that value once, zeros elsewhere
    vals = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16)
    w = np.zeros((len(vals), 16), dtype=np.float16)
    w[:, 5] = vals
    _, s = encode_gpu(lib, w)
    assert np.array_equal(s[:, 0], golden["scale_all"])


def test_rounding_rule_every_fp16_value(lib):
    # blocks whose maximum pins the scale at 2^e; the other 15 slots sweep all fp16 values that
    # do not exceed the maximum (both signs), so every value / scale combination is visited
    allv = np.arange(0, 0x10000, dtype=np.uint32).astype(np.uint16).view(np.float16)
    finite = allv[np.isfinite(allv)]
    for top in (6.0, 3.0, 0.046875, 1536.0, 6.1e-5, 65504.0):
        cand = finite[np.abs(finite.astype(np.float32)) <= top]
        n = -(-len(cand) // 15)
        w = np.zeros((n, 16), dtype=np.float16)
        w[:, 0] = top
        body = np.zeros(n * 15, dtype=np.float16)
        body[:len(cand)] = cand
        w[:, 1:] = body.reshape(n, 15)
        p, s = encode_gpu(lib, w)
        rp, rs = oc.encode(w)
        assert np.array_equal(s, rs), top
        assert np.array_equal(p, rp), top


def test_shapes_and_model_statistics(lib):
    for M, K, sigma, seed in ((1, 16, 1.0, 0), (7, 48, 0.02, 1), (100, 5120, 0.02, 2),
                              (5120, 5120, 0.02, 3), (3, 17408, 1.0, 4)):
        w = oc.synthetic_weight(M, K, seed=seed, sigma=sigma)
        p, s = encode_gpu(lib, w)
        rp, rs = oc.encode(w)
        assert np.array_equal(p, rp) and np.array_equal(s, rs), (M, K)
    # re-quantising dequantised values (many exact ties and negative zeros; a block whose
    # largest code fell below 6 moves to a smaller scale): still the codec's bytes, and after
    # that one step the representation is stable
    w = oc.synthetic_weight(64, 1024, seed=9)
    p, s = encode_gpu(lib, w)
    d = oc.decode(p, s)
    p2, s2 = encode_gpu(lib, d)
    rp2, rs2 = oc.encode(d)
    assert np.array_equal(p2, rp2) and np.array_equal(s2, rs2)
    assert np.array_equal(oc.decode(p2, s2).view(np.uint16) & 0x7FFF, d.view(np.uint16) & 0x7FFF)


def test_non_finite_inputs_follow_the_cpu_arithmetic(lib):
    w = oc.synthetic_weight(4, 64, seed=5, sigma=1.0)
    w[0, 3] = np.inf
    w[1, 20] = -np.inf
    w[2, 40] = np.nan
    p, s = encode_gpu(lib, w)
    with np.errstate(all="ignore"):
        rp, rs = oc.encode(w)
    assert np.array_equal(s, rs) and np.array_equal(p, rp)
    assert s[0, 0] == 254 and s[2, 2] == 127


def test_argument_checks(lib):
    assert lib.launch_nvfp4_encode(None, None, None, 4, 64, None) == -2
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    o = torch.zeros(64, dtype=torch.uint8, device="cuda")
    assert lib.launch_nvfp4_encode(ptr(x), ptr(o), ptr(o), 1, 24, stream()) == -2
    assert lib.launch_nvfp4_encode(ptr(x), ptr(o), ptr(o), 0, 16, stream()) == -2


def test_encoded_weights_feed_the_gemv(lib):
    from tests.gpu_util import gemv
    w = oc.synthetic_weight(96, 1024, seed=11)
    p, s = encode_gpu(lib, w)
    a = oc.synthetic_act(1024, seed=12)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    ref = oc.gemv_f64(p, s, a)
    assert oc.rel_error_floored(y, ref).max() <= 1e-3


def test_container_written_on_the_gpu_equals_the_host_container(lib, tmp_path):
    from nvfp4_v100_b200.pipeline import _qwen38_nvfp4_pack as pk

    rng = np.random.default_rng(21)
    tensors = {
        "model.language_model.layers.0.mlp.gate_proj.weight": oc.synthetic_weight(96, 256, 1),
        "model.language_model.layers.0.mlp.down_proj.weight": oc.synthetic_weight(256, 96 + 32, 2),
        "model.language_model.layers.0.input_layernorm.weight": rng.standard_normal(256).astype(np.float32),
        "model.language_model.embed_tokens.weight": oc.synthetic_weight(50, 256, 3),
        "lm_head.weight": oc.synthetic_weight(50, 256, 4),
    }
    host_dir, gpu_dir = str(tmp_path / "host"), str(tmp_path / "gpu")
    ih = pk.pack_tensors(tensors, host_dir)
    ig = pk.pack_tensors(tensors, gpu_dir, device="cuda")
    assert ih == ig and len(ih) == 3
    for name in ("nvfp4_packed.bin", "nvfp4_index.json", "fp16_embed.npy"):
        with open(f"{host_dir}/{name}", "rb") as a, open(f"{gpu_dir}/{name}", "rb") as b:
            assert a.read() == b.read(), name


def decode_gpu(lib, p, s, ids=None):
    d_p, d_s = torch.from_numpy(np.ascontiguousarray(p)).cuda(), torch.from_numpy(np.ascontiguousarray(s)).cuda()
    n = p.shape[0] if ids is None else len(ids)
    K = p.shape[1] * 2
    d_ids = None if ids is None else torch.from_numpy(np.asarray(ids, dtype=np.int64)).cuda()
    out = torch.full((n * K + 16,), 3.0, dtype=torch.float16, device="cuda")
    rc = lib.launch_nvfp4_decode_rows(ptr(d_p), ptr(d_s), None if ids is None else ptr(d_ids),
                                      ptr(out), n, K, p.shape[0], stream())
    torch.cuda.synchronize()
    assert rc == 0
    o = out.cpu().numpy()
    assert (o[n * K:] == 3.0).all()
    return o[:n * K].reshape(n, K)


def test_decode_rows_bit_exact(lib, golden):
    # the reference decoder's rows (golden), every packed byte under every scale byte, gathers
    d = decode_gpu(lib, golden["emb_packed"], golden["emb_scales"], golden["emb_idx"])
    assert np.array_equal(d.view(np.uint16), golden["emb_rows"].view(np.uint16))
    for i in range(int(golden["n_mats"])):
        d = decode_gpu(lib, golden[f"m{i}_packed"], golden[f"m{i}_scales"])
        assert np.array_equal(d.view(np.uint16), golden[f"m{i}_dec"].view(np.uint16)), i
    # 256 scale bytes x (256 packed bytes in 32 blocks of 8 bytes): row r uses scale byte r
    p = np.tile(np.arange(256, dtype=np.uint8), (256, 1))
    s = np.repeat(np.arange(256, dtype=np.uint8)[:, None], 32, axis=1)
    got = decode_gpu(lib, p, s)
    with np.errstate(over="ignore"):
        want = oc.decode(p, s)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert lib.launch_nvfp4_decode_rows(None, None, None, None, 1, 16, 1, None) == -2


def test_packed_embedding_lookup_on_the_device(lib, tmp_path):
    from nvfp4_v100_b200.pipeline import _qwen38_infer as Q

    w = oc.synthetic_weight(300, 256, seed=8)
    p, s = oc.encode(w)
    np.save(tmp_path / "p.npy", p)
    np.save(tmp_path / "s.npy", s)
    emb = Q.QEmbedding(Q.PackedEmb(str(tmp_path / "p.npy"), str(tmp_path / "s.npy")))
    ids = torch.tensor([[5, 299, 0, 5]], device="cuda")
    got = emb(ids)
    assert got.shape == (1, 4, 256) and got.dtype == torch.float16
    want = oc.decode(p, s)[[5, 299, 0, 5]]
    assert np.array_equal(got[0].cpu().numpy().view(np.uint16), want.view(np.uint16))
    dense = Q.QEmbedding(torch.from_numpy(oc.decode(p, s)))
    assert torch.equal(dense(ids), got)

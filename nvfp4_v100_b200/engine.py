"""Native decode engine: one decode step of the hybrid (Gated-DeltaNet + gated-attention) decoder
as a fixed list of C-ABI launches, captured once in a CUDA graph and replayed per token.

It plays the role of the reference's decode engine bridge — ``QLinear`` dispatch, the
``patch_fused_deltanet`` / ``patch_attn_decode`` / ``patch_rmsnorm`` forwards and ``GraphDecoder``
(reference: pipeline/_qwen38_infer.py:144-184, 425-510, 587-650, 653-729, 856-903;
experiments/_qwen38_p7_pair.py pair fusion; experiments/_qwen38_p9_fuse.py RoPE / silu fusion) —
without the third-party model code in the loop: every operator of the step is one of this
library's kernels, the token id, position and KV length live in device memory, and a replay needs
no host work.  PyTorch is used for device buffers, streams and graph capture only.

Weight layout: the engine consumes matrices in the reference container's raw layout
(packed [M, K/2] + scales [M, K/16]) and, like the reference's pair fusion, concatenates
projections that share an input by rows at load time: [q|k|v], [in_proj_qkv|z|b|a]; gate and up
rows are interleaved in groups of 8 so the GEMV epilogue can apply silu(gate)*up.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib, tp

vp = ctypes.c_void_p
HEAD_DIM = 256      # attention head dim (fixed by the kernels)
DN_DIM = 128        # DeltaNet head dim (fixed by the kernels)
CONV_K = 4
PREFILL_MAX_CONTEXT = 9600   # launch_attn_prefill: 4 query rows x context x 4 bytes <= 150 KB


@dataclass
class ModelConfig:
    """Shapes of the decoder.  Defaults are the reference's 27B model (hidden 5120,
    intermediate 17408, 24 q / 4 kv heads x 256, DeltaNet 16 key / 48 value heads x 128,
    q projection with per-head output gate, every 4th layer full attention)."""
    hidden: int = 5120
    inter: int = 17408
    vocab: int = 248320
    n_layers: int = 64
    full_attn_interval: int = 4
    hq: int = 24
    hkv: int = 4
    dn_kheads: int = 16
    dn_vheads: int = 48
    rms_eps: float = 1e-6
    rope_theta: float = 1e7
    max_len: int = 1024

    def is_attn(self, i: int) -> bool:
        return (i + 1) % self.full_attn_interval == 0

    @property
    def conv_dim(self) -> int:
        return (2 * self.dn_kheads + self.dn_vheads) * DN_DIM

    def layer_shapes(self, i: int) -> dict:
        """name -> (M, K) of the layer's linear weights, reference naming."""
        H = self.hidden
        if self.is_attn(i):
            mix = {"q_proj": (self.hq * 2 * HEAD_DIM, H), "k_proj": (self.hkv * HEAD_DIM, H),
                   "v_proj": (self.hkv * HEAD_DIM, H), "o_proj": (H, self.hq * HEAD_DIM)}
        else:
            mix = {"in_proj_qkv": (self.conv_dim, H), "in_proj_z": (self.dn_vheads * DN_DIM, H),
                   "in_proj_b": (self.dn_vheads, H), "in_proj_a": (self.dn_vheads, H),
                   "out_proj": (H, self.dn_vheads * DN_DIM)}
        mix.update({"gate_proj": (self.inter, H), "up_proj": (self.inter, H),
                    "down_proj": (H, self.inter)})
        return mix


def rope_tables(cfg: ModelConfig):
    """cos/sin fp16 [max_len, 256]: angle = pos * theta^(-2i/256), i = 0..127, duplicated over the
    two halves (the model's rotary embedding; computed in fp32, stored as fp16)."""
    inv = (1.0 / (np.float32(cfg.rope_theta) ** (np.arange(0, HEAD_DIM, 2, dtype=np.float32)
                                                 / np.float32(HEAD_DIM)))).astype(np.float32)
    ang = np.arange(cfg.max_len, dtype=np.float32)[:, None] * inv[None, :]
    emb = np.concatenate([ang, ang], axis=1)
    return np.cos(emb).astype(np.float16), np.sin(emb).astype(np.float16)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[inter, X] gate and up byte matrices -> [2*inter, X] with rows in groups of 8:
    gate rows 8j..8j+7 then up rows 8j..8j+7."""
    n, x = gate.shape
    assert n % 8 == 0 and up.shape == gate.shape
    return torch.stack([gate.view(n // 8, 8, x), up.view(n // 8, 8, x)], dim=1).reshape(2 * n, x)


@dataclass
class _Mat:
    packed: torch.Tensor
    scales: torch.Tensor
    M: int
    K: int


@dataclass
class _Layer:
    attn: bool
    in_w1: torch.Tensor            # fp32 (1 + input_layernorm.weight)
    post_w1: torch.Tensor
    w_in: _Mat = None              # [q|k|v] or [in_proj_qkv|z|b|a]
    w_out: _Mat = None             # o_proj / out_proj
    w_gu: _Mat = None
    w_down: _Mat = None
    extra: dict = field(default_factory=dict)


class ContainerWeights:
    """Read-only mapping from the engine's weight names (``layers.3.self_attn.q_proj``,
    ``layers.3.input_layernorm.weight``, ``embed_tokens``, ``norm.weight``, ``lm_head``) to the
    contents of a reference container.  Matrices come back as (packed [M, K/2], scales [M, K/16])
    numpy VIEWS of the memory-mapped ``nvfp4_packed.bin`` — nothing is read until it is sliced and
    copied; vectors come from ``fp32_misc.npz``; the embedding table is the memory-mapped
    ``fp16_embed.npy``."""

    PREFIX = "model.language_model."

    def __init__(self, directory: str):
        import json
        import os

        self.directory = directory
        with open(os.path.join(directory, "nvfp4_index.json"), encoding="utf-8") as f:
            self.index = json.load(f)
        self.blob = np.memmap(os.path.join(directory, "nvfp4_packed.bin"), dtype=np.uint8, mode="r")
        self.misc = np.load(os.path.join(directory, "fp32_misc.npz"))
        self.embed = np.load(os.path.join(directory, "fp16_embed.npy"), mmap_mode="r")
        self.bytes_viewed = 0

    def _matrix(self, key):
        e = self.index[key]
        M, K = int(e["M"]), int(e["K"])
        p = self.blob[int(e["packed_off"]):int(e["packed_off"]) + int(e["packed_bytes"])]
        s = self.blob[int(e["scales_off"]):int(e["scales_off"]) + int(e["scales_bytes"])]
        return p.reshape(M, K // 2), s.reshape(M, K // 16)

    def __getitem__(self, name):
        if name == "embed_tokens":
            return self.embed
        if name == "lm_head":
            return self._matrix("lm_head.weight")
        full = self.PREFIX + name
        if full + ".weight" in self.index:
            return self._matrix(full + ".weight")
        if full in self.misc.files:
            a = self.misc[full]
            # the depthwise conv weight is stored [channels, 1, 4]
            return a.reshape(a.shape[0], -1) if a.ndim == 3 else a
        raise KeyError(name)


class DecodeEngine:
    """Holds the prepared weights and all state of one sequence and replays the step graph."""

    def __init__(self, cfg: ModelConfig, device: str = "cuda", tp_rank: int = 0, tp_world: int = 1,
                 allreduce: str = "peer"):
        """tp_world > 1: this process holds shard tp_rank of a tensor-parallel group (one process
        per GPU, torch.distributed initialised with the NCCL backend by the caller).
        allreduce: "peer" (default, the fastest measured at 2 GPUs) = GEMV, then this library's
        one-shot all-reduce + residual kernel over NVLink peer memory; "inline" = the K-split GEMV
        writes its partial vector into the peer-visible buffer and the NEXT GEMV's prologue does
        the exchange, the sum, the residual add and the RMSNorm (no kernel of its own per
        all-reduce); "fused" = the K-split GEMV, its all-reduce and the residual add are ONE
        kernel (peer stores per tile, last CTA reduces); "nccl" = GEMV, NCCL all-reduce, then a
        residual-add kernel.  In "peer" and "inline" the greedy pick is exchanged through peer
        memory as well, so a decode step contains no library collective."""
        if not torch.cuda.is_available():
            raise RuntimeError("DecodeEngine needs a CUDA device; there is no CPU fallback")
        self.cfg = cfg
        self.dev = torch.device(device)
        self.lib = _lib.load()
        # the tensor-core GEMV's workspace must exist before any stream capture
        if self.lib.nvfp4_gemv_tc_prepare() != 0:
            raise RuntimeError("nvfp4_gemv_tc_prepare failed (no device memory for the GEMV workspace)")
        if "NVFP4_GEMM_CONFIG" in os.environ:      # W4A16 GEMM tile policy (see nvfp4_b200_gemm_config)
            self.lib.nvfp4_b200_gemm_config(int(os.environ["NVFP4_GEMM_CONFIG"]))
        self.rank, self.world = tp_rank, tp_world
        c = cfg
        W = tp_world
        if c.hq % W or c.dn_kheads % W or c.dn_vheads % W or c.inter % (W * 128):
            raise ValueError(f"model shapes do not split over {W} ranks")
        if W > c.hkv and W % c.hkv:
            raise ValueError("ranks must be a multiple of the KV heads when there are more ranks")
        # local (per-rank) sizes
        self.hq_l = c.hq // W
        self.hkv_l = max(1, c.hkv // W)
        self.nk_l, self.nv_l = c.dn_kheads // W, c.dn_vheads // W
        self.inter_l = c.inter // W
        self.conv_l = (2 * self.nk_l + self.nv_l) * DN_DIM
        self.v_lo, self.v_hi = tp.split_range(c.vocab, W, tp_rank, 16) if c.vocab % 16 == 0 \
            else tp.split_range(c.vocab, W, tp_rank, 1)
        self.layers: list[_Layer] = []
        self.graph = None
        self.n_launch = 0
        self.n_collective = 0
        f16, f32, i64 = torch.float16, torch.float32, torch.int64
        z = lambda *s, dt=f16: torch.zeros(*s, dtype=dt, device=self.dev)
        self.h = z(c.hidden)
        self.partial = z(c.hidden)          # K-split layer output before the all-reduce
        self.qkv = z(self.hq_l * 2 * HEAD_DIM + 2 * self.hkv_l * HEAD_DIM)
        self.q_out = z(self.hq_l * HEAD_DIM)
        self.gate_out = z(self.hq_l * HEAD_DIM)
        self.attn_out = z(self.hq_l * HEAD_DIM)
        self.attn_scratch = z(int(self.lib.nvfp4_attn_split_scratch_bytes(self.hq_l)), dt=torch.uint8)
        self.dn_in = z(self.conv_l + self.nv_l * DN_DIM + 2 * self.nv_l)
        self.dn_out = z(self.nv_l * DN_DIM)
        self.dn_scratch = z(self.conv_l, dt=f32)
        self.act = z(self.inter_l)
        self.logits = z(self.v_hi - self.v_lo)
        self.cand = z(2, dt=f32)
        self.cand_all = z(2 * W, dt=f32)
        self.tok = z(1, dt=i64)
        self.pos = z(1, dt=i64)            # index of the token being processed
        self.len = z(1, dt=i64)            # keys in the cache including that token
        self.hist_cap = 4096
        self.history = z(self.hist_cap, dt=i64)
        self.hist_count = z(1, dt=i64)
        cos, sin = rope_tables(c)
        self.cos = torch.from_numpy(cos).to(self.dev)
        self.sin = torch.from_numpy(sin).to(self.dev)
        self.embed = None
        self.final_w1 = None
        self.lm_head = None
        self.allreduce = allreduce if W > 1 else "none"
        # chunked prefill through the token-major GEMM entry (no transposes around the GEMMs);
        # NVFP4_PREFILL_TRANSPOSE=1 keeps the reference-shaped call with explicit layout changes
        self.prefill_token_major = os.environ.get("NVFP4_PREFILL_TRANSPOSE", "0") != "1"
        self.mlp_one_launch = os.environ.get("NVFP4_MLP_ONE_LAUNCH", "0") == "1"
        self.ar_calls = 0
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.dev)   # decode steps so far
        self._pending = None        # ("inline"): (parity, site) of the all-reduce not yet applied
        self._site = 0
        if self.allreduce in ("peer", "fused", "inline"):
            self._setup_peer_comm()

    def _setup_peer_comm(self):
        from .comm import PeerComm

        self.comm = PeerComm(self.cfg.hidden, self.rank, self.world)

    def comm_status(self) -> int:
        """0 if every peer wait of the one-shot all-reduce was answered in time."""
        if self.allreduce not in ("peer", "fused", "inline"):
            return 0
        return self.comm.status()

    def close(self):
        """Release the graph and the peer mappings (call on every rank, before tearing the
        process group down)."""
        self.graph = None
        if getattr(self, "comm", None) is not None:
            self.comm.close()
            self.comm = None

    # ------------------------------------------------------------------ weights
    def _mat(self, packed: torch.Tensor, scales: torch.Tensor, M: int, K: int) -> _Mat:
        packed = packed.contiguous().view(-1)
        scales = scales.contiguous().view(-1)
        assert packed.numel() == M * K // 2 and scales.numel() == M * K // 16
        assert packed.data_ptr() % 32 == 0 and scales.data_ptr() % 8 == 0
        return _Mat(packed, scales, M, K)

    def load_random(self, seed: int = 0, quantise: bool = True):
        """The throughput workload: seeded fp16 weights ~N(0, 0.02^2) drawn on the device and
        quantised there with ``launch_nvfp4_encode`` (``quantise=False``: random E2M1 bytes with
        scale bytes in [118, 122], the range those weights produce), fp16 embedding
        ~N(0, 0.02^2), unit norm weights."""
        c = self.cfg
        g = torch.Generator(device=self.dev)
        g.manual_seed(seed * 64 + self.rank)
        vp = ctypes.c_void_p

        def rnd(M, K):
            if not quantise:
                p = torch.randint(0, 256, (M * K // 2,), dtype=torch.uint8, device=self.dev,
                                  generator=g)
                s = torch.randint(118, 123, (M * K // 16,), dtype=torch.uint8, device=self.dev,
                                  generator=g)
                return self._mat(p, s, M, K)
            p = torch.empty(M * K // 2, dtype=torch.uint8, device=self.dev)
            s = torch.empty(M * K // 16, dtype=torch.uint8, device=self.dev)
            st = vp(torch.cuda.current_stream(self.dev).cuda_stream)
            step = max(1, (1 << 28) // K)               # at most 512 MB of fp16 at a time
            for r0 in range(0, M, step):
                r1 = min(M, r0 + step)
                w = (torch.randn((r1 - r0, K), device=self.dev, generator=g) * 0.02).half()
                rc = self.lib.launch_nvfp4_encode(
                    vp(w.data_ptr()), vp(p.data_ptr() + r0 * (K // 2)),
                    vp(s.data_ptr() + r0 * (K // 16)), r1 - r0, K, st)
                if rc != 0:
                    raise RuntimeError(f"launch_nvfp4_encode rc={rc}")
            return self._mat(p, s, M, K)

        ones = lambda n: torch.ones(n, dtype=torch.float32, device=self.dev)
        self.layers = []
        for i in range(c.n_layers):
            L = _Layer(c.is_attn(i), ones(c.hidden), ones(c.hidden))
            if L.attn:
                L.w_in = rnd(self.hq_l * 2 * HEAD_DIM + 2 * self.hkv_l * HEAD_DIM, c.hidden)
                L.w_out = rnd(c.hidden, self.hq_l * HEAD_DIM)
                L.extra = dict(
                    q_w1=ones(HEAD_DIM), k_w1=ones(HEAD_DIM),
                    keys=torch.zeros(self.hkv_l, c.max_len, HEAD_DIM, dtype=torch.float16, device=self.dev),
                    values=torch.zeros(self.hkv_l, c.max_len, HEAD_DIM, dtype=torch.float16, device=self.dev))
            else:
                L.w_in = rnd(self.conv_l + self.nv_l * DN_DIM + 2 * self.nv_l, c.hidden)
                L.w_out = rnd(c.hidden, self.nv_l * DN_DIM)
                L.extra = dict(
                    conv_w=(torch.randn(self.conv_l, CONV_K, device=self.dev, generator=g) * 0.02).half(),
                    conv_state=torch.zeros(self.conv_l, CONV_K, dtype=torch.float16, device=self.dev),
                    A_log=torch.log(torch.rand(self.nv_l, device=self.dev, generator=g) * 16 + 1e-3).half(),
                    dt_bias=torch.ones(self.nv_l, dtype=torch.float16, device=self.dev),
                    norm_w=torch.ones(DN_DIM, dtype=torch.float16, device=self.dev),
                    state=torch.zeros(self.nv_l, DN_DIM, DN_DIM, dtype=torch.float32, device=self.dev))
            L.w_gu = rnd(2 * self.inter_l, c.hidden)
            L.w_down = rnd(c.hidden, self.inter_l)
            self.layers.append(L)
        ge = torch.Generator(device=self.dev)
        ge.manual_seed(seed + 7919)          # the embedding is replicated: same on every rank
        self.embed = (torch.randn(c.vocab, c.hidden, device=self.dev, generator=ge) * 0.02).half()
        self.final_w1 = ones(c.hidden)
        self.lm_head = rnd(self.v_hi - self.v_lo, c.hidden)

    def load_weights(self, weights: dict):
        """``weights``: reference-named numpy arrays of the FULL model, e.g.
        ``layers.3.self_attn.q_proj`` -> (packed u8 [M, K/2], scales u8 [M, K/16]),
        ``layers.3.input_layernorm.weight`` -> fp16 array, ``embed_tokens`` fp16 [V, H],
        ``norm.weight``, ``lm_head`` (packed, scales).  Each rank cuts its shard out of the raw
        bytes (rows for q/k/v, in_proj, gate/up, lm_head; a K range for o_proj, out_proj,
        down_proj), uploads it and fuses projections that share an input by rows on the device."""
        c = self.cfg
        dev = self.dev
        R, W = self.rank, self.world

        def dv(a):
            return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

        def w1(name):
            return (1.0 + torch.from_numpy(np.asarray(weights[name], dtype=np.float16)).float()).to(dev)

        def f16(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float16)).to(dev)

        def mat(parts, K):
            p = torch.cat([dv(x[0]) for x in parts], 0)
            s = torch.cat([dv(x[1]) for x in parts], 0)
            return self._mat(p, s, p.shape[0], K)

        def rows(name, unit):
            p, s = weights[name]
            lo, hi = tp.split_range(p.shape[0], W, R, unit)
            return tp.shard_rows(p, s, lo, hi)

        def kslice(name, K):
            p, s = weights[name]
            pk, sk, k0, k1 = tp.shard_k(p, s, K, W, R)
            return (pk, sk), k1 - k0

        def vec_rows(a, unit):
            lo, hi = tp.split_range(a.shape[0], W, R, unit)
            return a[lo:hi]

        self.layers = []
        for i in range(c.n_layers):
            pre = f"layers.{i}."
            L = _Layer(c.is_attn(i), w1(pre + "input_layernorm.weight"),
                       w1(pre + "post_attention_layernorm.weight"))
            if L.attn:
                a = pre + "self_attn."
                kp, ks = weights[a + "k_proj"]
                vpk, vs = weights[a + "v_proj"]
                L.w_in = mat([rows(a + "q_proj", 2 * HEAD_DIM),
                              tp.shard_kv_heads(kp, ks, c.hkv, W, R)[:2],
                              tp.shard_kv_heads(vpk, vs, c.hkv, W, R)[:2]], c.hidden)
                wo, ko = kslice(a + "o_proj", c.hq * HEAD_DIM)
                L.w_out = mat([wo], ko)
                L.extra = dict(
                    q_w1=w1(a + "q_norm.weight"), k_w1=w1(a + "k_norm.weight"),
                    keys=torch.zeros(self.hkv_l, c.max_len, HEAD_DIM, dtype=torch.float16, device=dev),
                    values=torch.zeros(self.hkv_l, c.max_len, HEAD_DIM, dtype=torch.float16, device=dev))
            else:
                a = pre + "linear_attn."
                groups = (c.dn_kheads * DN_DIM, c.dn_kheads * DN_DIM, c.dn_vheads * DN_DIM)
                qp, qs = weights[a + "in_proj_qkv"]
                L.w_in = mat([tp.shard_grouped_rows(qp, qs, groups, DN_DIM, W, R, np.concatenate),
                              rows(a + "in_proj_z", DN_DIM), rows(a + "in_proj_b", 1),
                              rows(a + "in_proj_a", 1)], c.hidden)
                wo, ko = kslice(a + "out_proj", c.dn_vheads * DN_DIM)
                L.w_out = mat([wo], ko)
                cw = np.asarray(weights[a + "conv1d.weight"], dtype=np.float16).reshape(c.conv_dim, CONV_K)
                cw_l, _ = tp.shard_grouped_rows(cw, cw, groups, DN_DIM, W, R, np.concatenate)
                L.extra = dict(
                    conv_w=f16(cw_l),
                    conv_state=torch.zeros(self.conv_l, CONV_K, dtype=torch.float16, device=dev),
                    A_log=f16(vec_rows(np.asarray(weights[a + "A_log"]), 1)),
                    dt_bias=f16(vec_rows(np.asarray(weights[a + "dt_bias"]), 1)),
                    norm_w=f16(weights[a + "norm.weight"]),
                    state=torch.zeros(self.nv_l, DN_DIM, DN_DIM, dtype=torch.float32, device=dev))
            m = pre + "mlp."
            gp, gs = rows(m + "gate_proj", 128)
            upp, ups = rows(m + "up_proj", 128)
            L.w_gu = self._mat(interleave_gate_up(dv(gp), dv(upp)), interleave_gate_up(dv(gs), dv(ups)),
                               2 * self.inter_l, c.hidden)
            wd, kd = kslice(m + "down_proj", c.inter)
            L.w_down = mat([wd], kd)
            self.layers.append(L)
        self.embed = f16(weights["embed_tokens"])
        self.final_w1 = w1("norm.weight")
        lp, ls = weights["lm_head"]
        self.lm_head = mat([tp.shard_rows(lp, ls, self.v_lo, self.v_hi)], c.hidden)

    def load_container(self, directory: str):
        """Load this rank's shard straight from a reference container (``nvfp4_packed.bin`` +
        ``nvfp4_index.json`` + ``fp32_misc.npz`` + ``fp16_embed.npy``; layout:
        pipeline/_qwen38_nvfp4_pack.py:117-124, uploaded per index entry by
        pipeline/_qwen38_infer.py:91-101).  The file is memory-mapped and every matrix is a view
        into the map: a rank copies to the device only the bytes of its own shard — whole rows
        for q/k/v, in_proj, gate/up and lm_head (one contiguous range per row group), a K range
        of every row for o_proj, out_proj and down_proj (a strided range, gathered into a
        shard-sized host buffer) — and never holds the full model in host memory."""
        self.load_weights(ContainerWeights(directory))

    # ------------------------------------------------------------------ one step
    def _gemv(self, st, m: _Mat, x, out, pro_w1=None, epi=0, residual=None):
        out_ptr = out if isinstance(out, int) else out.data_ptr()
        if self._pending is not None:
            # the all-reduce of the previous K-split layer runs in this GEMV's prologue
            assert x is self.h and pro_w1 is not None and residual is None
            parity, site = self._pending
            self._pending = None
            rc = self.lib.launch_nvfp4_gemv_fused_ar(
                vp(m.packed.data_ptr()), vp(m.scales.data_ptr()), vp(self.h.data_ptr()), vp(out_ptr),
                m.M, m.K, vp(pro_w1.data_ptr()), float(self.cfg.rms_eps), epi, self.comm.ptrs,
                self.rank, self.world, self.cfg.hidden, parity, vp(self.epoch.data_ptr()), site,
                2 * self.cfg.n_layers, st)
            if rc != 0:
                raise RuntimeError(f"launch_nvfp4_gemv_fused_ar rc={rc} (M={m.M}, K={m.K})")
            self.n_launch += 1
            self.n_collective += 1
            return
        rc = self.lib.launch_nvfp4_gemv_fused(
            vp(m.packed.data_ptr()), vp(m.scales.data_ptr()), vp(x.data_ptr()), vp(out_ptr),
            m.M, m.K, 0 if pro_w1 is None else 1,
            vp(0 if pro_w1 is None else pro_w1.data_ptr()), float(self.cfg.rms_eps), epi,
            vp(0 if residual is None else residual.data_ptr()), st)
        if rc != 0:
            raise RuntimeError(f"launch_nvfp4_gemv_fused rc={rc} (M={m.M}, K={m.K})")
        self.n_launch += 1

    def _mlp_one_launch(self, st, L) -> bool:
        """One GPU, matrices large enough for the tensor-core GEMV: RMSNorm -> gate/up -> silu*mul ->
        down -> residual add as ONE kernel (launch_nvfp4_mlp_tc); the weight ring streams on from
        the first matrix into the second.  False = not taken, the caller issues the two launches.
        Off by default (NVFP4_MLP_ONE_LAUNCH=1 switches it on): measured 249 tok/s against 256 with
        two launches - the grid-wide barrier costs what the kernel boundary cost, and the second
        matrix's weight requests have to be held back behind the barrier for the same reason they
        are held back at kernel entry."""
        if self.world != 1 or not self.mlp_one_launch:
            return False
        gu, dn = L.w_gu, L.w_down
        if not (self.lib.nvfp4_gemv_tc_wanted(gu.M, gu.K) and self.lib.nvfp4_gemv_tc_wanted(dn.M, dn.K)):
            return False
        rc = self.lib.launch_nvfp4_mlp_tc(
            vp(gu.packed.data_ptr()), vp(gu.scales.data_ptr()), vp(dn.packed.data_ptr()),
            vp(dn.scales.data_ptr()), vp(self.h.data_ptr()), vp(self.act.data_ptr()),
            vp(L.post_w1.data_ptr()), float(self.cfg.rms_eps), dn.K, dn.M, st)
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"launch_nvfp4_mlp_tc rc={rc}")
        self.n_launch += 1
        return True

    def _row_parallel(self, st, m: _Mat, x):
        """o_proj / out_proj / down_proj: h += W x.  One GPU: the residual add is the GEMV's
        epilogue.  Tensor parallel: each rank's K slice gives a partial vector; all-reduce (NCCL,
        captured in the graph), then the residual add."""
        if self.world == 1:
            self._gemv(st, m, x, self.h, epi=1, residual=self.h)
            return
        if self.allreduce == "fused":
            _, parity = self.comm.next_slot()
            self.ar_calls += 1
            rc = self.lib.launch_nvfp4_gemv_allreduce(
                vp(m.packed.data_ptr()), vp(m.scales.data_ptr()), vp(x.data_ptr()),
                vp(self.h.data_ptr()), m.M, m.K, self.comm.ptrs, self.rank, self.world,
                self.cfg.hidden, parity, st)
            if rc != 0:
                raise RuntimeError(f"launch_nvfp4_gemv_allreduce rc={rc}")
            self.n_launch += 1
            self.n_collective += 1
            return
        if self.allreduce == "inline":
            slot, parity = self.comm.next_slot()
            self.ar_calls += 1
            self._gemv(st, m, x, slot)
            self._pending = (parity, self._site)
            self._site += 1
            return
        if self.allreduce == "peer":
            slot, parity = self.comm.next_slot()
            self.ar_calls += 1
            self._gemv(st, m, x, slot)
            self.comm.allreduce_residual(self.h, parity, st)
            self.n_launch += 1
            self.n_collective += 1
            return
        import torch.distributed as dist

        self._gemv(st, m, x, self.partial)
        dist.all_reduce(self.partial)
        self.n_collective += 1
        rc = self.lib.launch_residual_add(vp(self.h.data_ptr()), vp(self.partial.data_ptr()),
                                          self.cfg.hidden, st)
        assert rc == 0, rc
        self.n_launch += 1

    def enqueue_step(self):
        """Enqueue one decode step on torch's current stream (capturable)."""
        c, lib = self.cfg, self.lib
        st = vp(torch.cuda.current_stream().cuda_stream)
        self.n_launch = 0
        self.n_collective = 0
        self._site = 0
        self._pending = None
        # an even number of K-split layers per step keeps the slot parity of every call site the
        # same in every step, which a captured graph needs
        assert self.ar_calls % 2 == 0
        rc = lib.launch_embed_gather(vp(self.embed.data_ptr()), vp(self.tok.data_ptr()),
                                     vp(self.h.data_ptr()), c.hidden, c.vocab, st)
        assert rc == 0, rc
        self.n_launch += 1
        nq = self.conv_l
        for L in self.layers:
            e = L.extra
            if L.attn:
                self._gemv(st, L.w_in, self.h, self.qkv, pro_w1=L.in_w1)
                rc = lib.launch_attn_prep(
                    vp(self.qkv.data_ptr()), vp(e["q_w1"].data_ptr()), vp(e["k_w1"].data_ptr()),
                    vp(self.cos.data_ptr()), vp(self.sin.data_ptr()), vp(self.pos.data_ptr()),
                    vp(self.q_out.data_ptr()), vp(self.gate_out.data_ptr()),
                    vp(e["keys"].data_ptr()), vp(e["values"].data_ptr()), self.hq_l, self.hkv_l,
                    c.max_len, float(c.rms_eps), st)
                assert rc == 0, rc
                rc = lib.launch_attn_decode_split(
                    vp(self.q_out.data_ptr()), vp(e["keys"].data_ptr()), vp(e["values"].data_ptr()),
                    vp(self.len.data_ptr()), vp(self.gate_out.data_ptr()),
                    vp(self.attn_out.data_ptr()), vp(self.attn_scratch.data_ptr()), c.max_len,
                    self.hq_l, self.hkv_l, float(HEAD_DIM) ** -0.5, st)
                assert rc == 0, rc
                self.n_launch += 2
                self._row_parallel(st, L.w_out, self.attn_out)
            else:
                self._gemv(st, L.w_in, self.h, self.dn_in, pro_w1=L.in_w1)
                base = self.dn_in.data_ptr()
                zoff = nq * 2
                boff = zoff + self.nv_l * DN_DIM * 2
                aoff = boff + self.nv_l * 2
                rc = lib.launch_dn_fused_heads(
                    vp(base), vp(base + zoff), vp(base + boff), vp(base + aoff),
                    vp(e["conv_w"].data_ptr()), vp(e["conv_state"].data_ptr()),
                    vp(e["A_log"].data_ptr()), vp(e["dt_bias"].data_ptr()),
                    vp(e["norm_w"].data_ptr()), vp(e["state"].data_ptr()),
                    vp(self.dn_scratch.data_ptr()), vp(self.dn_out.data_ptr()),
                    self.nk_l, self.nv_l, float(c.rms_eps), st)
                assert rc == 0, rc
                self.n_launch += 2
                self._row_parallel(st, L.w_out, self.dn_out)
            if not self._mlp_one_launch(st, L):
                self._gemv(st, L.w_gu, self.h, self.act, pro_w1=L.post_w1, epi=2)
                self._row_parallel(st, L.w_down, self.act)
        self._gemv(st, self.lm_head, self.h, self.logits, pro_w1=self.final_w1)
        if self.world == 1:
            rc = lib.launch_argmax_advance(
                vp(self.logits.data_ptr()), c.vocab, vp(self.tok.data_ptr()), vp(self.pos.data_ptr()),
                vp(self.len.data_ptr()), vp(self.history.data_ptr()), vp(self.hist_count.data_ptr()),
                self.hist_cap, st)
            assert rc == 0, rc
            self.n_launch += 1
        elif self.allreduce in ("inline", "peer"):
            rc = lib.launch_argmax_exchange(
                vp(self.logits.data_ptr()), self.v_hi - self.v_lo, self.v_lo, self.comm.ptrs,
                self.rank, self.world, c.hidden, vp(self.epoch.data_ptr()), vp(self.tok.data_ptr()),
                vp(self.pos.data_ptr()), vp(self.len.data_ptr()), vp(self.history.data_ptr()),
                vp(self.hist_count.data_ptr()), self.hist_cap, st)
            assert rc == 0, rc
            self.n_launch += 1
            self.n_collective += 1
        else:
            import torch.distributed as dist

            rc = lib.launch_argmax_slice(vp(self.logits.data_ptr()), self.v_hi - self.v_lo,
                                         self.v_lo, vp(self.cand.data_ptr()), st)
            assert rc == 0, rc
            dist.all_gather_into_tensor(self.cand_all, self.cand)
            self.n_collective += 1
            rc = lib.launch_pick_global_argmax(
                vp(self.cand_all.data_ptr()), self.world, vp(self.tok.data_ptr()),
                vp(self.pos.data_ptr()), vp(self.len.data_ptr()), vp(self.history.data_ptr()),
                vp(self.hist_count.data_ptr()), self.hist_cap, st)
            assert rc == 0, rc
            self.n_launch += 2

    # ------------------------------------------------------------------ state
    def reset(self, first_token: int = 0):
        """Empty caches and recurrent state, position 0, next token to process = first_token."""
        for L in self.layers:
            e = L.extra
            if L.attn:
                e["keys"].zero_()
                e["values"].zero_()
            else:
                e["conv_state"].zero_()
                e["state"].zero_()
        self.tok.fill_(int(first_token))
        self.pos.zero_()
        self.len.fill_(1)
        self.hist_count.zero_()

    def snapshot(self):
        """Copy of every piece of mutable state (reference: snap_decode_state plus the fused
        DeltaNet buffers, pipeline/_qwen38_infer.py:530-552, 817-818)."""
        snap = {"tok": self.tok.clone(), "pos": self.pos.clone(), "len": self.len.clone(),
                "hist_count": self.hist_count.clone(), "history": self.history.clone(), "layers": []}
        n = int(self.len.item())
        for L in self.layers:
            e = L.extra
            if L.attn:
                snap["layers"].append((e["keys"][:, :n].clone(), e["values"][:, :n].clone()))
            else:
                snap["layers"].append((e["conv_state"].clone(), e["state"].clone()))
        return snap

    def restore(self, snap):
        for L, s in zip(self.layers, snap["layers"]):
            e = L.extra
            if L.attn:
                n = s[0].shape[1]
                e["keys"][:, :n].copy_(s[0])
                e["values"][:, :n].copy_(s[1])
            else:
                e["conv_state"].copy_(s[0])
                e["state"].copy_(s[1])
        for k in ("tok", "pos", "len", "hist_count", "history"):
            getattr(self, k).copy_(snap[k])

    # ------------------------------------------------------------------ graph
    def capture(self, n_warmup: int = 1):
        """Warm up on a side stream (the warm-up steps mutate state: the caller's state is saved
        and restored around them, the hygiene rule of the reference's capture protocol,
        pipeline/_qwen38_infer.py:687-701, 825-829), then capture one step."""
        snap = self.snapshot()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(n_warmup):
                self.enqueue_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.restore(snap)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.enqueue_step()
        self.restore(snap)
        torch.cuda.synchronize()
        return self.n_launch

    def step(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:
            self.enqueue_step()

    # ------------------------------------------------------------------ chunked prefill
    def _prefill_buffers(self, chunk: int):
        """Scratch for one chunk of up to ``chunk`` tokens (allocated once, reused)."""
        if getattr(self, "_pf", None) is not None and self._pf["chunk"] >= chunk:
            return self._pf
        c = self.cfg
        f16 = torch.float16
        np_max = (chunk + 7) // 8 * 8
        m_in = max(self.hq_l * 2 * HEAD_DIM + 2 * self.hkv_l * HEAD_DIM,
                   self.conv_l + self.nv_l * DN_DIM + 2 * self.nv_l)
        k_max = max(c.hidden, self.hq_l * HEAD_DIM, self.nv_l * DN_DIM)
        m_max = max(m_in, 2 * self.inter_l, c.hidden)
        e = lambda *shape, dt=f16: torch.empty(*shape, dtype=dt, device=self.dev)
        work = int(self.lib.nvfp4_dn_prefill_work_bytes(chunk, max(1, self.nk_l), max(1, self.nv_l)))
        self._pf = dict(
            chunk=chunk, ids=e(chunk, dt=torch.int64),
            h=e(chunk * c.hidden), xn=e(chunk * c.hidden),
            xT=e(k_max * np_max), yT=e(m_max * np_max), y=e(chunk * m_in),
            actT=e(self.inter_l * np_max), dT=e(c.hidden * np_max),
            q=e(chunk * self.hq_l * HEAD_DIM), gate=e(chunk * self.hq_l * HEAD_DIM),
            mix=e(chunk * max(self.hq_l * HEAD_DIM, self.nv_l * DN_DIM)),
            work=e(work, dt=torch.uint8), work_bytes=work)
        return self._pf

    def prefill(self, tokens, chunk: int = 512, start: int = 0):
        """Run ``tokens`` (host ints) through the model in chunks of up to ``chunk`` tokens with the
        tensor-core GEMM as every projection, filling the KV caches, conv windows and recurrent
        states for positions start .. start + len(tokens) - 1.  Leaves the engine ready to process
        the token at the next position (``tok`` is the caller's to set).  Tensor parallel: every
        rank runs its shard of each projection; the K-split projections' token-major partial outputs
        are summed over the ranks with an NCCL all-reduce (bandwidth-sized messages, 5 MB per
        call for 512 tokens) before the residual add.  The reference's flow is
        pipeline/_qwen38_infer.py:796-809 (512-token chunks through the third-party model code)."""
        c, lib = self.cfg, self.lib
        if self.world > 1:
            import torch.distributed as dist
        total = len(tokens)
        if start + total > c.max_len:
            raise ValueError("prompt longer than the cache")
        # the chunk attention kernel keeps a group's scores in shared memory (150 KB): checked
        # here, before the first launch, because a failure in the middle of a prompt would leave
        # the caches and states of earlier chunks and layers already advanced
        if start + total > PREFILL_MAX_CONTEXT:
            raise ValueError(f"chunked prefill handles contexts up to {PREFILL_MAX_CONTEXT} tokens "
                             f"(got {start + total}); feed the rest through step()")
        B = self._prefill_buffers(min(chunk, max(total, 1)))
        st = vp(torch.cuda.current_stream().cuda_stream)
        H = c.hidden
        ptr = lambda t: vp(t.data_ptr())

        def ok(rc, what):
            if rc != 0:
                raise RuntimeError(f"{what} rc={rc}")

        def rmsnorm(w1, n):
            ok(lib.launch_rmsnorm(ptr(B["h"]), H, ptr(w1), ptr(B["xn"]), n, H, float(c.rms_eps), st),
               "launch_rmsnorm")

        def to_gemm(src, n, feat, Np):          # token-major [n][feat] -> xT [feat][Np]
            ok(lib.launch_transpose_f16(ptr(src), feat, ptr(B["xT"]), Np, n, feat, st), "transpose")

        def gemm(m: _Mat, act, out, Np):
            ok(lib.launch_nvfp4_gemmtc_v5(ptr(m.packed), ptr(m.scales), ptr(act), ptr(out), m.M, Np,
                                          m.K, st), "launch_nvfp4_gemmtc_v5")

        def gemm_ex(m: _Mat, act, ld_act, out, ld_out, n, flags):
            # flags: 1 = act token-major, 2 = out token-major, 4 = out += (residual)
            ok(lib.launch_nvfp4_gemm_w4a16_ex(ptr(m.packed), ptr(m.scales), ptr(act), ld_act, ptr(out),
                                              ld_out, m.M, n, m.K, flags, st),
               "launch_nvfp4_gemm_w4a16_ex")

        def residual_gemm(m: _Mat, act, ld_act, in_flag, n):
            """h[t] += W . act[t]: the residual add inside the GEMM's epilogue on one GPU; over
            ranks the token-major partial products are summed first."""
            if self.world == 1:
                gemm_ex(m, act, ld_act, B["h"], H, n, in_flag | 2 | 4)
            else:
                gemm_ex(m, act, ld_act, B["dT"], H, n, in_flag | 2)
                dist.all_reduce(B["dT"][:n * H])
                B["h"][:n * H] += B["dT"][:n * H]

        for lo in range(0, total, B["chunk"]):
            n = min(B["chunk"], total - lo)
            Np = (n + 7) // 8 * 8
            p0 = start + lo
            B["ids"][:n].copy_(torch.as_tensor(np.asarray(tokens[lo:lo + n], dtype=np.int64)))
            ok(lib.launch_embed_rows(ptr(self.embed), ptr(B["ids"]), ptr(B["h"]), n, H, c.vocab, st),
               "launch_embed_rows")
            for L in self.layers:
                e = L.extra
                m_in = L.w_in.M
                rmsnorm(L.in_w1, n)
                if self.prefill_token_major:
                    # the GEMM reads the token-major rows as its K-major B operand and writes
                    # token-major: no layout change around it
                    gemm_ex(L.w_in, B["xn"], H, B["y"], m_in, n, 1 | 2)
                else:
                    to_gemm(B["xn"], n, H, Np)
                    gemm(L.w_in, B["xT"], B["yT"], Np)
                    ok(lib.launch_transpose_f16(ptr(B["yT"]), Np, ptr(B["y"]), m_in, m_in, n, st),
                       "transpose")
                if L.attn:
                    ok(lib.launch_attn_prep_tokens(
                        ptr(B["y"]), m_in, ptr(e["q_w1"]), ptr(e["k_w1"]), ptr(self.cos),
                        ptr(self.sin), p0, n, ptr(B["q"]), ptr(B["gate"]), ptr(e["keys"]),
                        ptr(e["values"]), self.hq_l, self.hkv_l, c.max_len, float(c.rms_eps), st),
                       "launch_attn_prep_tokens")
                    ok(lib.launch_attn_prefill(
                        ptr(B["q"]), ptr(e["keys"]), ptr(e["values"]), p0 + 1, n, ptr(B["gate"]),
                        ptr(B["mix"]), c.max_len, self.hq_l, self.hkv_l, float(HEAD_DIM) ** -0.5,
                        st), "launch_attn_prefill")
                else:
                    ok(lib.launch_dn_prefill(
                        ptr(B["y"]), m_in, ptr(e["conv_w"]), ptr(e["conv_state"]), ptr(e["A_log"]),
                        ptr(e["dt_bias"]), ptr(e["norm_w"]), ptr(e["state"]), ptr(B["work"]),
                        B["work_bytes"], ptr(B["mix"]), n, self.nk_l, self.nv_l, float(c.rms_eps),
                        st), "launch_dn_prefill")
                if self.prefill_token_major:
                    residual_gemm(L.w_out, B["mix"], L.w_out.K, 1, n)
                else:
                    to_gemm(B["mix"], n, L.w_out.K, Np)
                    gemm(L.w_out, B["xT"], B["dT"], Np)
                    if self.world > 1:
                        dist.all_reduce(B["dT"][:H * Np])
                    ok(lib.launch_add_transposed(ptr(B["h"]), ptr(B["dT"]), Np, n, H, st), "add")
                rmsnorm(L.post_w1, n)
                if self.prefill_token_major:
                    # gate/up leaves [2 inter][tokens] for the row-wise silu-mul; the down
                    # projection reads that layout and adds into the token-major residual
                    gemm_ex(L.w_gu, B["xn"], H, B["yT"], Np, n, 1)
                else:
                    to_gemm(B["xn"], n, H, Np)
                    gemm(L.w_gu, B["xT"], B["yT"], Np)
                ok(lib.launch_silu_mul_rows(ptr(B["yT"]), ptr(B["actT"]), self.inter_l, Np, st),
                   "launch_silu_mul_rows")
                if self.prefill_token_major:
                    residual_gemm(L.w_down, B["actT"], Np, 0, n)
                else:
                    gemm(L.w_down, B["actT"], B["dT"], Np)
                    if self.world > 1:
                        dist.all_reduce(B["dT"][:H * Np])
                    ok(lib.launch_add_transposed(ptr(B["h"]), ptr(B["dT"]), Np, n, H, st), "add")
        self.pos.fill_(start + total)
        self.len.fill_(start + total + 1)
        if lib.nvfp4_gemm_status(0) != 0:
            raise RuntimeError("a bounded wait inside the tensor-core GEMM ran out")

    def run(self, prompt, n_gen: int, native_prefill: bool = False):
        """Feed the prompt, then generate n_gen tokens greedily; returns the generated token ids
        (host list).  The prompt goes token by token through the decode step (teacher forced), or
        with ``native_prefill`` all but its last token through :meth:`prefill`."""
        self.reset(int(prompt[0]))
        if native_prefill and len(prompt) > 1:
            self.prefill([int(t) for t in prompt[:-1]])
            self.tok.fill_(int(prompt[-1]))
            prompt = prompt[-1:]
        for t in range(1, len(prompt)):
            self.step()
            self.tok.fill_(int(prompt[t]))      # overwrite the model's own prediction
        base = int(self.hist_count.item())
        for _ in range(n_gen):
            self.step()
        torch.cuda.synchronize()
        st = self.comm_status()
        if st != 0:
            raise RuntimeError(f"a bounded wait on a tensor-parallel peer ran out (status {st}): "
                               "the generated tokens are not valid")
        return self.history[base:base + n_gen].cpu().tolist()

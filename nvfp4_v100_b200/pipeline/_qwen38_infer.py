"""Decode engine bridge: the reference's monkey-patch layer over the third-party model code,
backed by this repository's sm_100a library.

Same public names and call signatures as the reference module (pipeline/_qwen38_infer.py):
``load_gemv``/``load_v5``, ``GEMV``, ``V5``, ``GEMV_T1``, ``set_gemv_t1``, ``upload_nvfp4``,
``PackedEmb``, ``QEmbedding``, ``QLinear``, ``st_name``, ``patch_linears``, ``fill_rest``,
``rebuild_rope``, ``build_model``, ``patch_fused_deltanet``, ``ensure_kv_stage``,
``snap_decode_state``, ``restore_decode_state``, ``refresh_deltanet_state``,
``patch_attn_decode``, ``patch_rmsnorm``, ``GraphDecoder`` — plus ``patch_rope`` and
``patch_mlp_silu_mul`` from experiments/_qwen38_p9_fuse.py and a ``prefill`` helper.

The libraries are loaded by the reference's file names through ``ctypes.CDLL`` (the ``.dll``
names are symlinks to the one shared library), with the reference's ``argtypes``.  Differences
that the environment forces, all behaviour-neutral:
  * the container is opened when a model is built, not at import (there is no default model
    directory on this machine); ``NVFP4_MODEL_DIR`` still names it;
  * the model skeleton is created on the ``meta`` device directly (the reference uses
    ``accelerate.init_empty_weights``);
  * the installed transformers names the layer kind ``layer_type`` (the reference's version:
    ``block_type``); both are accepted;
  * head counts are read from the module, so shards and small test models work
    (``launch_attn_decode_heads`` / ``launch_dn_fused_heads``); the 27B shapes take the
    reference-named entry points.
"""
from __future__ import annotations

import ctypes
import json
import os

import numpy as np
import torch
import torch.nn as nn

BASE = os.path.dirname(os.path.abspath(__file__))
KDIR = os.path.join(os.path.dirname(BASE), "kernels")
MODEL_DIR = os.environ.get("NVFP4_MODEL_DIR", "")

_vp = ctypes.c_void_p


def _dll(name):
    path = os.path.join(KDIR, name)
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: run `python -m nvfp4_v100_b200.build`")
    return ctypes.CDLL(path)


def load_gemv():
    lib = _dll("nvfp4_gemv.dll")
    lib.gpu_malloc.argtypes = [ctypes.c_size_t]
    lib.gpu_malloc.restype = ctypes.c_void_p
    lib.gpu_free.argtypes = [ctypes.c_void_p]
    lib.gpu_memcpy_h2d.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    lib.gpu_memcpy_h2d.restype = ctypes.c_int
    lib.gpu_memcpy_d2h.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    lib.gpu_memcpy_d2h.restype = ctypes.c_int
    for fn in (lib.launch_nvfp4_gemv, lib.launch_nvfp4_gemv_v8):
        fn.argtypes = [_vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, _vp]
        fn.restype = ctypes.c_int
    lib.launch_nvfp4_gemv2.argtypes = [_vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, _vp]
    lib.launch_nvfp4_gemv2.restype = ctypes.c_int
    return lib


def load_v5():
    lib = _dll("nvfp4_cuda_v5.dll")
    lib.launch_nvfp4_gemmtc_v5.argtypes = [_vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_int, _vp]
    lib.launch_nvfp4_gemmtc_v5.restype = ctypes.c_int
    return lib


GEMV = load_gemv()
V5 = load_v5()
H2D = GEMV.gpu_memcpy_h2d
UPLOAD_BYTES = [0]
_CONTAINER = {"dir": None, "fd": None}
GEMV_T1 = {"v1": GEMV.launch_nvfp4_gemv, "v8": GEMV.launch_nvfp4_gemv_v8}.get(
    os.environ.get("VF_GEMV", "v8"), GEMV.launch_nvfp4_gemv_v8)


def set_gemv_t1(name):
    """Switch the T=1 kernel entry at run time ('v1' or 'v8')."""
    global GEMV_T1
    fn = {"v1": GEMV.launch_nvfp4_gemv, "v8": GEMV.launch_nvfp4_gemv_v8}[name]
    GEMV_T1 = fn
    return fn


def open_container(model_dir=None):
    d = model_dir or MODEL_DIR
    if not d:
        raise RuntimeError("no model directory: pass model_dir or set NVFP4_MODEL_DIR")
    if _CONTAINER["dir"] != d:
        if _CONTAINER["fd"] is not None:
            _CONTAINER["fd"].close()
        _CONTAINER["fd"] = open(os.path.join(d, "nvfp4_packed.bin"), "rb")
        _CONTAINER["dir"] = d
    return _CONTAINER["fd"]


def upload_nvfp4(entry):
    """Raw row-major bytes of one matrix -> device (two allocations, two synchronous copies)."""
    fd = _CONTAINER["fd"]
    d_p = GEMV.gpu_malloc(entry["packed_bytes"])
    d_s = GEMV.gpu_malloc(entry["scales_bytes"])
    assert d_p and d_s, "gpu_malloc failed"
    fd.seek(entry["packed_off"])
    pb = fd.read(entry["packed_bytes"])
    fd.seek(entry["scales_off"])
    sb = fd.read(entry["scales_bytes"])
    assert H2D(d_p, pb, len(pb)) == 0 and H2D(d_s, sb, len(sb)) == 0
    UPLOAD_BYTES[0] += len(pb) + len(sb)
    return d_p, d_s


class PackedEmb:
    """NVFP4-packed embedding table on the host; ``[idx]`` decodes the rows to fp16."""
    CP = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)

    def __init__(self, path_p, path_s):
        self.packed = np.load(path_p, mmap_mode="r")
        self.scales = np.load(path_s, mmap_mode="r")
        V, Hh = self.packed.shape
        self.shape = (V, Hh * 2)
        self.lut = (np.where(np.arange(16) & 8, -1.0, 1.0) * self.CP[np.arange(16) & 7]).astype(np.float32)

    def __getitem__(self, idx):
        scalar = np.isscalar(idx) or (torch.is_tensor(idx) and idx.ndim == 0)
        idx = np.asarray(idx.cpu() if torch.is_tensor(idx) else idx).reshape(-1)
        p, sb = self.packed[idx], self.scales[idx]
        n = p.shape[0]
        nib = np.empty((n, p.shape[1] * 2), dtype=np.uint8)
        nib[:, 0::2] = p & 0x0F
        nib[:, 1::2] = p >> 4
        w = self.lut[nib].reshape(n, -1, 16)
        sc = np.exp2(sb.astype(np.float64) - 127.0)
        w = (w * sc[:, :, None]).astype(np.float16).reshape(n, -1)
        return torch.from_numpy(w[0] if scalar else w)


class QEmbedding(nn.Module):
    """Embedding kept in host memory; only the looked-up rows travel to the device."""

    def __init__(self, weight_cpu):
        super().__init__()
        self.weight_cpu = weight_cpu
        self.num_embeddings, self.embedding_dim = weight_cpu.shape

    def forward(self, ids):
        idx = ids.detach().cpu().reshape(-1)
        rows = self.weight_cpu[idx]
        return rows.to("cuda", dtype=rows.dtype).view(*ids.shape, -1)


class QLinear(nn.Module):
    """Forward-only Linear whose weight lives on the device in NVFP4 form.  T = 1: GEMV; T = 2:
    two-activation GEMV; T > 2: tensor-core GEMM on the transposed activations."""

    def __init__(self, d_p, d_s, M, K, bias=None):
        super().__init__()
        self.d_p, self.d_s, self.M, self.K = d_p, d_s, M, K
        self.bias = bias

    def forward(self, x):
        K = self.K
        lead = x.shape[:-1]
        x2 = x.reshape(-1, K).contiguous()
        if x2.dtype != torch.float16:
            x2 = x2.to(torch.float16)
        T = x2.shape[0]
        stream = torch.cuda.current_stream().cuda_stream
        if T == 1:
            out = torch.empty((1, self.M), dtype=torch.float16, device=x.device)
            rc = GEMV_T1(self.d_p, self.d_s, x2.data_ptr(), out.data_ptr(), self.M, K, _vp(stream))
            assert rc == 0, f"gemv rc={rc}"
        elif T == 2:
            out = torch.empty((2, self.M), dtype=torch.float16, device=x.device)
            rc = GEMV.launch_nvfp4_gemv2(self.d_p, self.d_s, x2[0].data_ptr(), x2[1].data_ptr(),
                                         out.data_ptr(), self.M, K, _vp(stream))
            assert rc == 0, f"gemv2 rc={rc}"
        else:
            xt = x2.t().contiguous()                                    # (K, T)
            o2 = torch.empty((self.M, T), dtype=torch.float16, device=x.device)
            rc = V5.launch_nvfp4_gemmtc_v5(self.d_p, self.d_s, xt.data_ptr(), o2.data_ptr(),
                                           self.M, T, K, _vp(stream))
            assert rc == 0, f"gemm rc={rc}"
            out = o2.t().contiguous()
        if self.bias is not None:
            out = out + self.bias
        return out.reshape(*lead, self.M)


def st_name(name):
    """Skeleton parameter name -> checkpoint name (model.* -> model.language_model.*)."""
    if name.startswith("model."):
        return "model.language_model." + name[len("model."):]
    return name


def patch_linears(model, index, misc):
    patched = 0
    misc_keys = set(misc.files)
    for pname, module in list(model.named_modules()):
        if isinstance(module, nn.Linear):
            wkey = st_name(f"{pname}.weight")
            if wkey not in index:
                print(f"  [warn] {wkey} not in the quantised index, left as is")
                continue
            e = index[wkey]
            d_p, d_s = upload_nvfp4(e)
            bias = None
            if module.bias is not None:
                bkey = st_name(f"{pname}.bias")
                bias = (torch.from_numpy(misc[bkey]).to(torch.float16).cuda() if bkey in misc_keys
                        else torch.zeros(module.bias.shape, dtype=torch.float16, device="cuda"))
            q = QLinear(d_p, d_s, e["M"], e["K"], bias=bias)
            parts = pname.split(".")
            parent = model.get_submodule(".".join(parts[:-1])) if len(parts) > 1 else model
            setattr(parent, parts[-1], q)
            patched += 1
    return patched


def fill_rest(model, misc, embed):
    filled, skipped = 0, []
    misc_keys = set(misc.files)
    for name, p in model.named_parameters():
        if "embed_tokens" in name:
            p.data.copy_(torch.from_numpy(np.asarray(embed)).to(torch.float16))
            filled += 1
            continue
        key = st_name(name)
        if key in misc_keys:
            p.data.copy_(torch.from_numpy(misc[key]).to(torch.float16).reshape(p.shape).cuda())
            filled += 1
        else:
            skipped.append(key)
    return filled, skipped


def rebuild_rope(model):
    """Recreate the non-persistent rotary buffers after ``to_empty``."""
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5TextRotaryEmbedding
    n = 0
    for mod in model.modules():
        if isinstance(mod, Qwen3_5TextRotaryEmbedding):
            fresh = Qwen3_5TextRotaryEmbedding(mod.config, torch.device("cuda"))
            mod.inv_freq = fresh.inv_freq
            mod.original_inv_freq = fresh.original_inv_freq
            mod.attention_scaling = fresh.attention_scaling
            n += 1
    return n


def _layer_kind(lyr):
    return getattr(lyr, "block_type", None) or getattr(lyr, "layer_type")


def build_model(model_dir=None):
    """Container + config.json -> (config, model) with every Linear a QLinear."""
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM

    d = model_dir or MODEL_DIR
    open_container(d)
    cfg = Qwen3_5TextConfig(**json.load(open(os.path.join(d, "config.json"), encoding="utf-8")))
    with torch.device("meta"):
        model = Qwen3_5ForCausalLM(cfg).to(torch.float16)
    index = json.load(open(os.path.join(d, "nvfp4_index.json"), encoding="utf-8"))
    misc = np.load(os.path.join(d, "fp32_misc.npz"))
    emb_p, emb_s = (os.path.join(d, "nvfp4_embed_packed.npy"), os.path.join(d, "nvfp4_embed_scales.npy"))
    emb_mode = os.environ.get("VF_EMBED", "nvfp4" if os.path.exists(emb_p) and os.path.exists(emb_s)
                              else "fp16")
    if emb_mode == "nvfp4":
        embed = PackedEmb(emb_p, emb_s)
    else:
        embed = torch.from_numpy(np.asarray(np.load(os.path.join(d, "fp16_embed.npy"), mmap_mode="r")))
    model.model.embed_tokens = QEmbedding(embed)
    n_patch = patch_linears(model, index, misc)
    model.to_empty(device="cuda")
    n_fill, skipped = fill_rest(model, misc, None)
    n_rope = rebuild_rope(model)
    model.eval()
    torch.cuda.synchronize()
    print(f"  patch {n_patch} Linear | fill {n_fill} param | rope {n_rope} | "
          f"uploaded {UPLOAD_BYTES[0] / 1e9:.2f} GB", flush=True)
    if skipped:
        print("  skipped:", skipped[:10], flush=True)
    return cfg, model


def prefill(model, cache, ids, chunk=512):
    """Chunked prefill (reference: pipeline/_qwen38_infer.py:796-809); returns the first token."""
    L = ids.shape[1]
    first = None
    with torch.no_grad():
        for i in range(0, L, chunk):
            j = min(i + chunk, L)
            out = model(ids[:, i:j], past_key_values=cache, use_cache=True,
                        cache_position=torch.arange(i, j, device="cuda"), logits_to_keep=1)
            if j == L:
                first = int(out.logits[:, -1, :].argmax(dim=-1).item())
    return first


# ------------------------------------------------------------------------------------------------
def patch_fused_deltanet(model, cache, mtp=True):
    """Replace the T <= 2 forward of every linear-attention layer by the fused step kernel.
    Call AFTER a prefill: the conv and recurrent state are copied out of the cache."""
    dn = _dll("nvfp4_dn_fused.dll")
    dn.launch_dn_fused.argtypes = [_vp] * 12 + [ctypes.c_float, _vp]
    dn.launch_dn_fused.restype = ctypes.c_int
    dn.launch_dn_fused_heads.argtypes = [_vp] * 12 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, _vp]
    dn.launch_dn_fused_heads.restype = ctypes.c_int
    mods = []
    for i, lyr in enumerate(model.model.layers):
        if _layer_kind(lyr) != "linear_attention":
            continue
        mod = lyr.linear_attn
        lay = cache.layers[i]
        nk, nv = mod.num_k_heads, mod.num_v_heads
        cdim = mod.conv_dim
        conv = lay.conv_states[0].reshape(-1)
        rec = lay.recurrent_states[0]                                # (nv, 128, 128) k x v
        mod._vf_conv = torch.zeros(cdim * 4, dtype=torch.float16, device="cuda")
        mod._vf_conv.copy_(conv.to(torch.float16))                   # layout c*4 + t
        mod._vf_S = rec.transpose(-1, -2).contiguous().float().reshape(-1).clone()
        mod._vf_scr = torch.zeros(cdim, dtype=torch.float32, device="cuda")
        mod._vf_out = torch.zeros(nv * 128, dtype=torch.float16, device="cuda")
        mod._vf_out2 = torch.zeros(nv * 128, dtype=torch.float16, device="cuda")
        mod._vf_S_bak = torch.zeros_like(mod._vf_S) if mtp else None
        mod._vf_conv_bak = torch.zeros_like(mod._vf_conv) if mtp else None
        mod._vf_eps = float(getattr(mod.norm, "variance_epsilon", getattr(mod.norm, "eps", 1e-6)))
        mod._vf_convw = mod.conv1d.weight.detach().reshape(cdim, 4).to(torch.float16).contiguous()
        if not getattr(mod, "_vf_fast", False):
            mod._vf_orig = mod.forward
        mod._vf_fast = True
        mods.append(mod)

    def launch(mod, mixed, z, b, a, obuf, st):
        p = _vp
        args = (p(mixed.data_ptr()), p(z.data_ptr()), p(b.data_ptr()), p(a.data_ptr()),
                p(mod._vf_convw.data_ptr()), p(mod._vf_conv.data_ptr()), p(mod.A_log.data_ptr()),
                p(mod.dt_bias.data_ptr()), p(mod.norm.weight.data_ptr()), p(mod._vf_S.data_ptr()),
                p(mod._vf_scr.data_ptr()), p(obuf.data_ptr()))
        if (mod.num_k_heads, mod.num_v_heads) == (16, 48):
            return dn.launch_dn_fused(*args, mod._vf_eps, st)
        return dn.launch_dn_fused_heads(*args, mod.num_k_heads, mod.num_v_heads, mod._vf_eps, st)

    def fast_fwd(mod):
        def fwd(hidden_states, cache_params=None, attention_mask=None, **kw):
            Tn = hidden_states.shape[1]
            if Tn > 2:
                return mod._vf_orig(hidden_states, cache_params=cache_params,
                                    attention_mask=attention_mask, **kw)
            st = _vp(torch.cuda.current_stream().cuda_stream)
            mixed = mod.in_proj_qkv(hidden_states)
            z = mod.in_proj_z(hidden_states)
            b = mod.in_proj_b(hidden_states)
            a = mod.in_proj_a(hidden_states)
            outs = []
            for t in range(Tn):
                if t == 0 and mod._vf_S_bak is not None:
                    mod._vf_S_bak.copy_(mod._vf_S)
                    mod._vf_conv_bak.copy_(mod._vf_conv)
                obuf = mod._vf_out if t == 0 else mod._vf_out2
                rc = launch(mod, mixed[:, t].contiguous(), z[:, t].contiguous(),
                            b[:, t].contiguous(), a[:, t].contiguous(), obuf, st)
                assert rc == 0, f"dn_fused rc={rc}"
                outs.append(obuf.view(1, 1, -1))
            return mod.out_proj(outs[0] if Tn == 1 else torch.cat(outs, dim=1))
        return fwd

    for mod in mods:
        mod.forward = fast_fwd(mod)
    return mods


_KV_STAGE = {"buf": None, "elems": 0}


def ensure_kv_stage(model, max_len):
    cfg = model.config
    H = getattr(cfg, "num_key_value_heads", None) or cfg.num_attention_heads
    D = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    n = H * max_len * D
    if _KV_STAGE["buf"] is None or _KV_STAGE["elems"] < n:
        _KV_STAGE["buf"] = torch.empty(n, dtype=torch.float16, device="cuda")
        _KV_STAGE["elems"] = n
    return _KV_STAGE["buf"]


def snap_decode_state(model, cache, prompt_len):
    """KV prefix + cumulative_length of every attention layer, to the host."""
    snap = []
    for i, lyr in enumerate(model.model.layers):
        if _layer_kind(lyr) == "linear_attention":
            continue
        lay = cache.layers[i]
        snap.append((i, lay.keys[:, :, :prompt_len].clone().cpu(),
                     lay.values[:, :, :prompt_len].clone().cpu(),
                     lay.cumulative_length.clone().cpu()))
    return snap


def restore_decode_state(model, cache, snap, prompt_len):
    for i, k, v, c in snap:
        lay = cache.layers[i]
        lay.keys[:, :, :prompt_len].copy_(k)
        lay.values[:, :, :prompt_len].copy_(v)
        lay.cumulative_length.copy_(c)


def refresh_deltanet_state(model, cache):
    """After a new prefill into the same cache: copy its states into the fused kernels' buffers."""
    for i, lyr in enumerate(model.model.layers):
        if _layer_kind(lyr) != "linear_attention":
            continue
        mod = lyr.linear_attn
        lay = cache.layers[i]
        rt = lay.recurrent_states[0].transpose(-1, -2)
        mod._vf_S.view(rt.shape).copy_(rt)
        mod._vf_conv.copy_(lay.conv_states[0].reshape(-1))


def patch_attn_decode(model, cache, max_len=3072):
    """Replace the T = 1 forward of every full-attention layer by the fused decode kernel."""
    lib = _dll("nvfp4_attn_decode.dll")
    lib.launch_attn_decode.argtypes = [_vp] * 6 + [ctypes.c_int, ctypes.c_float, _vp]
    lib.launch_attn_decode.restype = ctypes.c_int
    lib.launch_attn_decode_heads.argtypes = [_vp] * 6 + [ctypes.c_int] * 3 + [ctypes.c_float, _vp]
    lib.launch_attn_decode_heads.restype = ctypes.c_int
    from transformers.models.qwen3_5 import modeling_qwen3_5 as hf
    mods = []
    pairs = []
    for i, lyr in enumerate(model.model.layers):
        if _layer_kind(lyr) != "full_attention":
            continue
        mod, lay = lyr.self_attn, cache.layers[i]
        hq = mod.config.num_attention_heads
        mod._vf_attn_out = torch.zeros(hq * mod.head_dim, dtype=torch.float16, device="cuda")
        if not getattr(mod, "_vf_attn", False):
            mod._vf_attn_orig = mod.forward
        mod._vf_attn = True
        mods.append(mod)
        pairs.append((mod, lay))

    def fast_fwd(mod, lay):
        hq, hkv = mod.config.num_attention_heads, mod.config.num_key_value_heads

        def fwd(hidden_states, position_embeddings=None, attention_mask=None,
                past_key_values=None, **kw):
            Tn = hidden_states.shape[1]
            if Tn != 1 or past_key_values is None:
                return mod._vf_attn_orig(hidden_states, position_embeddings=position_embeddings,
                                         attention_mask=attention_mask,
                                         past_key_values=past_key_values, **kw)
            D = mod.head_dim
            input_shape = hidden_states.shape[:-1]
            hidden_shape = (*input_shape, -1, D)
            qg = mod.q_proj(hidden_states).view(*input_shape, -1, D * 2)
            query_states, gate = torch.chunk(qg, 2, dim=-1)
            gate = gate.reshape(*input_shape, -1).contiguous()
            query_states = mod.q_norm(query_states.reshape(hidden_shape)).transpose(1, 2)
            key_states = mod.k_norm(mod.k_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
            value_states = mod.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
            cos, sin = position_embeddings
            query_states, key_states = hf.apply_rotary_pos_emb(query_states, key_states, cos, sin)
            keys, values = past_key_values.update(key_states, value_states, mod.layer_idx)
            q = query_states.contiguous()
            st = _vp(torch.cuda.current_stream().cuda_stream)
            a = (_vp(q.data_ptr()), _vp(keys.data_ptr()), _vp(values.data_ptr()),
                 _vp(lay.cumulative_length.data_ptr()), _vp(gate.data_ptr()),
                 _vp(mod._vf_attn_out.data_ptr()))
            if (hq, hkv) == (24, 4):
                rc = lib.launch_attn_decode(*a, max_len, float(mod.scaling), st)
            else:
                rc = lib.launch_attn_decode_heads(*a, max_len, hq, hkv, float(mod.scaling), st)
            assert rc == 0, f"attn_decode rc={rc} layer={mod.layer_idx}"
            return mod.o_proj(mod._vf_attn_out.view(1, 1, -1)), None
        return fwd

    for mod, lay in pairs:
        mod.forward = fast_fwd(mod, lay)
    return mods


def patch_rmsnorm(model):
    """Fuse every zero-centred RMSNorm: out = f16(f32(x) * rsqrt(mean(x^2) + eps) * (1 + w))."""
    lib = _dll("nvfp4_rmsnorm.dll")
    lib.launch_rmsnorm.argtypes = [_vp, ctypes.c_longlong, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                   ctypes.c_float, _vp]
    lib.launch_rmsnorm.restype = ctypes.c_int
    norms = []
    for mod in model.modules():
        if mod.__class__.__name__ != "Qwen3_5RMSNorm":
            continue
        mod._vf_w1 = (1.0 + mod.weight.float()).contiguous()
        mod._vf_out = None
        if not getattr(mod, "_vf_norm", False):
            mod._vf_norm_orig = mod.forward
        mod._vf_norm = True
        norms.append(mod)

    def fast_norm(mod):
        def fwd(x):
            n = x.shape[-1]
            if x.dim() >= 2 and x.shape[1] != 1:            # prefill keeps the original path
                return mod._vf_norm_orig(x)
            rows = x.numel() // n
            if rows <= 0 or x.stride(-1) != 1 or x.dtype != torch.float16:
                return mod._vf_norm_orig(x)
            if mod._vf_out is None or tuple(mod._vf_out.shape) != (rows, n):
                mod._vf_out = torch.empty((rows, n), dtype=x.dtype, device=x.device)
            st = _vp(torch.cuda.current_stream().cuda_stream)
            rc = lib.launch_rmsnorm(_vp(x.data_ptr()), x.stride(-2), _vp(mod._vf_w1.data_ptr()),
                                    _vp(mod._vf_out.data_ptr()), rows, n, float(mod.eps), st)
            assert rc == 0, f"rmsnorm rc={rc}"
            return mod._vf_out.view(x.shape)
        return fwd

    for mod in norms:
        mod.forward = fast_norm(mod)
    return norms


def patch_rope():
    """Module-level apply_rotary_pos_emb -> fused kernel for the decode shapes (T = 1, full
    rotation over 256 dims, fp16); anything else falls back (experiments/_qwen38_p9_fuse.py:48-82)."""
    lib = _dll("nvfp4_rope_silu.dll")
    lib.launch_rope_qk.argtypes = [_vp] * 6 + [ctypes.c_int, ctypes.c_int, _vp]
    lib.launch_rope_qk.restype = ctypes.c_int
    from transformers.models.qwen3_5 import modeling_qwen3_5 as hf
    if getattr(hf, "_vf_rope_orig", None) is None:
        hf._vf_rope_orig = hf.apply_rotary_pos_emb

    def fused(q, k, cos, sin, unsqueeze_dim=1):
        ok = (q.dim() == 4 and q.shape[0] == 1 and q.shape[2] == 1 and q.shape[-1] == 256 and
              cos.shape[-1] == 256 and q.dtype == torch.float16 and k.dtype == torch.float16)
        if not ok:
            return hf._vf_rope_orig(q, k, cos, sin, unsqueeze_dim=unsqueeze_dim)
        hq, hkv = q.shape[1], k.shape[1]
        qc, kc = q.contiguous(), k.contiguous()
        c16 = cos.reshape(-1).to(torch.float16).contiguous()
        s16 = sin.reshape(-1).to(torch.float16).contiguous()
        qo, ko = torch.empty_like(qc), torch.empty_like(kc)
        st = _vp(torch.cuda.current_stream().cuda_stream)
        rc = lib.launch_rope_qk(_vp(qc.data_ptr()), _vp(kc.data_ptr()), _vp(c16.data_ptr()),
                                _vp(s16.data_ptr()), _vp(qo.data_ptr()), _vp(ko.data_ptr()), hq, hkv, st)
        assert rc == 0, f"rope rc={rc}"
        return qo, ko

    hf.apply_rotary_pos_emb = fused
    return fused


def patch_mlp_silu_mul(model):
    """Every MLP forward at T = 1: down(silu(gate(x)) * up(x)) with the fused silu*mul kernel
    (experiments/_qwen38_p9_fuse.py:85-116)."""
    lib = _dll("nvfp4_rope_silu.dll")
    lib.launch_silu_mul.argtypes = [_vp, _vp, _vp, ctypes.c_int, _vp]
    lib.launch_silu_mul.restype = ctypes.c_int
    mods = []
    for mod in model.modules():
        if mod.__class__.__name__ != "Qwen3_5MLP":
            continue
        if not getattr(mod, "_vf_mlp", False):
            mod._vf_mlp_orig = mod.forward
        mod._vf_mlp = True
        mod._vf_act = None
        mods.append(mod)

    def fast(mod):
        def fwd(x):
            if x.numel() != x.shape[-1] or x.dtype != torch.float16:
                return mod._vf_mlp_orig(x)
            g, u = mod.gate_proj(x), mod.up_proj(x)
            n = g.numel()
            if mod._vf_act is None or mod._vf_act.numel() != n:
                mod._vf_act = torch.empty(n, dtype=torch.float16, device=x.device)
            st = _vp(torch.cuda.current_stream().cuda_stream)
            rc = lib.launch_silu_mul(_vp(g.data_ptr()), _vp(u.data_ptr()), _vp(mod._vf_act.data_ptr()), n, st)
            assert rc == 0, f"silu_mul rc={rc}"
            return mod.down_proj(mod._vf_act.view(g.shape))
        return fwd

    for mod in mods:
        mod.forward = fast(mod)
    return mods


class GraphDecoder:
    """One whole decode step — model forward, argmax, logits copy, position increment — captured
    in a CUDA graph.  The embedding row is gathered on the host and copied in before each replay.
    Warm-up steps mutate the cache: the caller snapshots before and restores after construction."""

    def __init__(self, model, cache, first_pos, hid, n_warmup=3, static_pos=None, use_pos4=True):
        self.first_pos = first_pos
        self.rope_pos = first_pos
        self.pos4 = torch.zeros(4, 1, 1, dtype=torch.long, device="cuda")
        self.static_embeds = torch.zeros(1, 1, hid, dtype=torch.float16, device="cuda")
        if static_pos is None:
            self.static_pos = torch.tensor([first_pos, first_pos + 1], device="cuda")
            self._own_pos = True
        else:
            self.static_pos = static_pos
            self._own_pos = False
        self.pos2 = self.static_pos[:1].view(1)
        V = model.lm_head.M
        self.static_logits = torch.zeros(1, V, dtype=torch.float16, device="cuda")
        self.static_next = torch.zeros(1, dtype=torch.long, device="cuda")
        self.pin = torch.empty(hid, dtype=torch.float16, pin_memory=True)

        def one_step():
            kw = {"position_ids": self.pos4} if use_pos4 else {}
            o = model(inputs_embeds=self.static_embeds, past_key_values=cache,
                      cache_position=self.pos2, use_cache=True, **kw)
            self.static_logits.copy_(o.logits[:, -1, :])
            self.static_next.copy_(o.logits[:, -1, :].argmax(dim=-1))
            self.static_pos.add_(1)

        self._one_step = one_step
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(n_warmup):
                self.pos4.fill_(int(self.static_pos[0].item()))
                one_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            one_step()

    def reset_pos(self):
        self.static_pos.copy_(torch.tensor([self.first_pos, self.first_pos + 1]))
        self.rope_pos = self.first_pos

    def set_pos(self, p):
        self.first_pos = p
        self.rope_pos = p
        self.static_pos.copy_(torch.tensor([p, p + 1]))

    def _feed(self, tok_id, emb_w):
        self.pin.copy_(emb_w[tok_id])
        self.static_embeds.copy_(self.pin.view(1, 1, -1), non_blocking=True)
        self.pos4.fill_(self.rope_pos)
        self.graph.replay()
        self.rope_pos += 1

    def step(self, tok_id, emb_w):
        self._feed(tok_id, emb_w)
        return int(self.static_next.item())

    def step_logits(self, tok_id, emb_w):
        self._feed(tok_id, emb_w)
        return int(self.static_next.item()), self.static_logits

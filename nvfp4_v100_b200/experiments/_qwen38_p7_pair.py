"""Pair fusion of the small projections that share an input: one GEMV launch computes
``in_proj_b`` and ``in_proj_a`` (2 x 48 rows) or ``k_proj`` and ``v_proj`` (2 x 1024 rows).

Answers to the names of the reference's ``experiments/_qwen38_p7_pair.py`` (``_PairLinear``,
``_Group``, ``PAIRS``, ``patch_pair_gemv``; reference lines 29-123), so a script written against
it runs against this package.  Rows are independent, so the fused launch gives bit for bit what
the two separate launches give.

Built differently from the reference where the hardware differs: the two members' bytes are
joined by device-to-device copies (the reference reads them back to the host and uploads them
again), and a group keeps its output buffer instead of allocating one per token, so that the
fused call can sit inside a captured step graph.
"""
from __future__ import annotations

import ctypes

import torch

from ..pipeline import _qwen38_infer as _qi
from ..pipeline._qwen38_infer import GEMV, QLinear

_vp = ctypes.c_void_p


class _Group:
    """The joined weights of a pair and the output of their last fused launch."""
    __slots__ = ("d_p", "d_s", "K", "M_total", "out", "xptr")

    def __init__(self, d_p, d_s, K, M_total):
        self.d_p, self.d_s, self.K, self.M_total = d_p, d_s, K, M_total
        self.out, self.xptr = None, 0

    def compute(self, x2):
        if self.out is None or self.out.device != x2.device:
            self.out = torch.empty((1, self.M_total), dtype=torch.float16, device=x2.device)
        rc = _qi.GEMV_T1(_vp(self.d_p), _vp(self.d_s), _vp(x2.data_ptr()), _vp(self.out.data_ptr()),
                         self.M_total, self.K, _vp(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"gemv(group) rc={rc}")
        self.xptr = x2.data_ptr()
        return self.out


class _PairLinear(QLinear):
    """A member of a pair: for one token the lead member launches the whole group and returns its
    own rows, the follower takes its rows from that result when it is called on the same input;
    any other call (more tokens, unexpected order) runs the member on its own rows, which its
    ``d_p`` / ``d_s`` already point at."""

    def forward(self, x):
        K = self.K
        lead = x.shape[:-1]
        x2 = x.reshape(-1, K)
        if x2.dtype != torch.float16:
            x2 = x2.half()
        x2 = x2.contiguous()
        if x2.shape[0] == 1:
            g = self._group
            out = None
            if self._lead:
                out = g.compute(x2)
            elif g.out is not None and g.xptr == x2.data_ptr():
                out = g.out
            if out is not None:
                # a copy: the group's buffer is overwritten by the next token's launch
                y = out[:, self._row_off:self._row_off + self.M].clone()
                if self.bias is not None:
                    y = y + self.bias
                return y.reshape(*lead, self.M)
        return super().forward(x)


# attribute name -> (partner, called first?); call order as in the model's forward:
#   linear_attn: b = in_proj_b(x); a = in_proj_a(x)      self_attn: k_proj(x) ... v_proj(x)
PAIRS = {"in_proj_b": ("in_proj_a", True), "in_proj_a": ("in_proj_b", False),
         "k_proj": ("v_proj", True), "v_proj": ("k_proj", False)}


def patch_pair_gemv(model):
    """After ``build_model``: replace each (in_proj_b, in_proj_a) and (k_proj, v_proj) pair of
    ``QLinear`` modules by two ``_PairLinear`` members over one joined weight buffer; the members'
    old buffers are freed.  Returns the number of pairs fused."""
    done = set()
    n_pair = 0
    for pname, mod in list(model.named_modules()):
        if not isinstance(mod, QLinear) or isinstance(mod, _PairLinear) or pname in done:
            continue
        owner, _, attr = pname.rpartition(".")
        if attr not in PAIRS or not PAIRS[attr][1]:
            continue
        sib_attr = PAIRS[attr][0]
        parent = model.get_submodule(owner) if owner else model
        sib = getattr(parent, sib_attr, None)
        if not isinstance(sib, QLinear) or sib.K != mod.K:
            continue
        if mod.bias is not None or sib.bias is not None:
            continue
        M1, M2, K = mod.M, sib.M, mod.K
        pb1, sb1 = M1 * K // 2, M1 * K // 16
        pb2, sb2 = M2 * K // 2, M2 * K // 16
        d_p = GEMV.gpu_malloc(pb1 + pb2)
        d_s = GEMV.gpu_malloc(sb1 + sb2)
        if not d_p or not d_s:
            raise MemoryError("gpu_malloc(pair) failed")
        for dst, src, n in ((d_p, mod.d_p, pb1), (d_p + pb1, sib.d_p, pb2),
                            (d_s, mod.d_s, sb1), (d_s + sb1, sib.d_s, sb2)):
            if GEMV.gpu_memcpy_d2d(_vp(dst), _vp(src), n) != 0:
                raise RuntimeError("gpu_memcpy_d2d(pair) failed")
        for old in (mod.d_p, mod.d_s, sib.d_p, sib.d_s):
            GEMV.gpu_free(_vp(old))
        g = _Group(d_p, d_s, K, M1 + M2)
        q1 = _PairLinear(d_p, d_s, M1, K, bias=None)
        q1._group, q1._row_off, q1._lead = g, 0, True
        q2 = _PairLinear(d_p + pb1, d_s + sb1, M2, K, bias=None)
        q2._group, q2._row_off, q2._lead = g, M1, False
        setattr(parent, attr, q1)
        setattr(parent, sib_attr, q2)
        done.update({pname, (owner + "." if owner else "") + sib_attr})
        n_pair += 1
    print(f"  [pair fusion] {n_pair} pairs of small GEMVs joined ({n_pair} launches fewer per step)",
          flush=True)
    return n_pair

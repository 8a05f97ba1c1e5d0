"""CPU oracle for the masked-attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this file: it is the checker used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.  It restates, with dense fp32/fp64
torch ops on the host, what the reference computes:

* ``naive_reference``     follows chill_attention/chill.py:498-544
  (dense boolean mask -> key-padding combine -> scaled_dot_product_attention
  in fp32 -> rows beyond ``lens`` multiplied by zero).
* ``builtin_mask_dense``  restates the five mask predicates,
  chill_attention/mask.py:818-825 (Full), :904-911 (Causal), :995-1012
  (SlidingWindow), :1129-1148 (Chunkwise), :1286-1304 (PrefixLM).
* ``attention_forward``   adds what the naive path does not return: the
  log-sum-exp in log2 units, ``LSE2 = logsumexp(scaled masked scores)/ln 2``
  (chill_attention/chill_fwd.py:328), and the row conventions of the kernels
  (chill_fwd.py:70-71, :218, :288): a row with no visible key gives O = 0 and
  LSE2 = -inf; a row at or beyond ``lens[b]`` gives O = 0 and LSE2 = 0.
* ``attention_backward``  closed-form gradients of the same function
  (chill_bwd_dq.py:272-332, chill_bwd_dkdv.py:380-403): rows at or beyond
  ``lens[b]`` contribute nothing, dK/dV are summed over the GQA group.
* ``banded_forward``/``banded_backward`` evaluate the same dense formulas on the
  key slice each query block can see, so that very long sliding-window
  sequences need no L x L matrix.

Parity pin: ``tests/golden/*.npz`` holds outputs of the reference itself (run
under its CPU interpreter by tests/golden/make_golden.py); tests/test_oracle.py
checks this oracle against every one of them.
"""
from __future__ import annotations

import math

import torch

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------- masks
def builtin_mask_dense(name, args, q_pos, k_pos):
    """bool[len(q_pos), len(k_pos)] for one of the five built-in mask names.

    ``q_pos`` / ``k_pos`` are int64 tensors of *global* positions.
    """
    q = q_pos.reshape(-1, 1)
    k = k_pos.reshape(1, -1)
    if name == "FullChillMask":
        return torch.ones((q.numel(), k.numel()), dtype=torch.bool)
    if name == "CausalChillMask":
        return q >= k
    if name == "SlidingWindowChillMask":
        left, right = args
        return (k <= q + right) & (k >= q - left)
    if name == "ChunkwiseChillMask":
        cs, bc = args
        d = q // cs - k // cs
        return (d >= 0) & (d <= bc)
    if name == "PrefixLMChillMask":
        (p,) = args
        return (k < p) | (q >= k)
    raise KeyError(name)


def _expand_kv(q, k, v):
    if q.shape[1] != k.shape[1]:
        g = q.shape[1] // k.shape[1]
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    return k, v


def _lens_tensor(lens, B, T):
    if lens is None:
        return torch.full((B,), T, dtype=torch.int64)
    return lens.to(torch.int64).clamp(max=T)  # chill_fwd.py:66: lens > T is clamped


# ----------------------------------------------------------- reference's naive path
def naive_reference(mask_dense, q, k, v, lens):
    """Restatement of chill.py:498-544.  ``mask_dense`` is bool (T, T).

    Returns (O * res_mask, res_mask) in the dtype of q (call it with fp32).
    """
    import torch.nn.functional as F

    k, v = _expand_kv(q, k, v)
    T = q.size(2)
    attn_mask = mask_dense
    if lens is not None:
        kpm = (torch.arange(T).unsqueeze(0) < lens.unsqueeze(-1)).unsqueeze(-1)  # (B, T, 1)
        both = kpm & kpm.transpose(-1, -2)
        attn_mask = attn_mask.unsqueeze(0).unsqueeze(0) & both.unsqueeze(1)
        res_mask = kpm.unsqueeze(1)
    else:
        res_mask = torch.as_tensor(1)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask) * res_mask, res_mask


# ------------------------------------------------------------------ dense fwd / bwd
def _visible(mask_dense, B, T_q, T_k, lens_q, k_pos):
    """(B, 1, T_q, T_k) bool: mask AND key position < lens[b]."""
    vis = mask_dense.reshape(1, 1, T_q, T_k) & (k_pos.reshape(1, 1, 1, T_k) < lens_q.reshape(B, 1, 1, 1))
    return vis


def attention_forward(mask_dense, q, k, v, lens=None, sm_scale=None, dtype=torch.float64,
                      q_pos=None, k_pos=None, seq_len=None):
    """Dense masked attention.  Returns (O, LSE2) in ``dtype``.

    q: (B, H, Tq, D); k, v: (B, Hkv, Tk, D); mask_dense: bool (Tq, Tk).
    ``q_pos``/``k_pos`` (global positions, default arange) and ``seq_len``
    (default Tq) only matter for the ``lens`` bound.
    """
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    q_pos = torch.arange(Tq) if q_pos is None else q_pos
    k_pos = torch.arange(Tk) if k_pos is None else k_pos
    seq_len = Tq if seq_len is None else seq_len
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    L = _lens_tensor(lens, B, seq_len)
    k, v = _expand_kv(q, k, v)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sm_scale
    vis = _visible(mask_dense, B, Tq, Tk, L, k_pos)
    s = s.masked_fill(~vis, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m_safe)
    l = p.sum(dim=-1, keepdim=True)
    lse2 = (m.squeeze(-1) + torch.log(torch.where(l == 0, torch.ones_like(l), l)).squeeze(-1)) * LOG2E
    o = torch.matmul(p / torch.where(l == 0, torch.ones_like(l), l), vf)
    row_ok = (q_pos.reshape(1, 1, Tq) < L.reshape(B, 1, 1))
    o = torch.where(row_ok.unsqueeze(-1), o, torch.zeros_like(o))
    lse2 = torch.where(row_ok, lse2, torch.zeros_like(lse2))
    return o, lse2


def attention_backward(mask_dense, q, k, v, do, lens=None, sm_scale=None, dtype=torch.float64,
                       q_pos=None, k_pos=None, seq_len=None):
    """Closed-form dQ, dK, dV of ``attention_forward`` (dK/dV summed over the GQA group)."""
    B, H, Tq, D = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    q_pos = torch.arange(Tq) if q_pos is None else q_pos
    k_pos = torch.arange(Tk) if k_pos is None else k_pos
    seq_len = Tq if seq_len is None else seq_len
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    L = _lens_tensor(lens, B, seq_len)
    ke, ve = _expand_kv(q, k, v)
    qf, kf, vf, dof = q.to(dtype), ke.to(dtype), ve.to(dtype), do.to(dtype)
    row_ok = (q_pos.reshape(1, 1, Tq, 1) < L.reshape(B, 1, 1, 1))
    dof = torch.where(row_ok, dof, torch.zeros_like(dof))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sm_scale
    vis = _visible(mask_dense, B, Tq, Tk, L, k_pos)
    s = s.masked_fill(~vis, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m_safe)
    l = p.sum(dim=-1, keepdim=True)
    p = p / torch.where(l == 0, torch.ones_like(l), l)
    p = torch.where(row_ok, p, torch.zeros_like(p))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (p * dp).sum(dim=-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.matmul(ds, kf) * sm_scale
    dk = torch.matmul(ds.transpose(-1, -2), qf) * sm_scale
    if H != Hkv:
        g = H // Hkv
        dk = dk.reshape(B, Hkv, g, Tk, D).sum(dim=2)
        dv = dv.reshape(B, Hkv, g, Tk, D).sum(dim=2)
    return dq, dk, dv


# ------------------------------------------------------------ banded (long sequences)
def _band(name, args, qb, qe, T):
    """Inclusive key interval that queries [qb, qe) of a built-in mask can see."""
    if name == "SlidingWindowChillMask":
        left, right = args
        return max(0, qb - left), min(T, qe + right)
    if name == "ChunkwiseChillMask":
        cs, bc = args
        return max(0, (qb // cs - bc) * cs), min(T, ((qe - 1) // cs + 1) * cs)
    if name == "CausalChillMask":
        return 0, qe
    return 0, T


def banded_forward(name, args, q, k, v, sm_scale=None, block=2048, dtype=torch.float32):
    """``attention_forward`` for built-in masks evaluated block by block on the
    visible key band only (exact, no L x L matrix)."""
    B, H, T, D = q.shape
    o = torch.empty(q.shape, dtype=dtype)
    lse = torch.empty(q.shape[:3], dtype=dtype)
    for qb in range(0, T, block):
        qe = min(T, qb + block)
        kb, ke = _band(name, args, qb, qe, T)
        qp, kp = torch.arange(qb, qe), torch.arange(kb, ke)
        md = builtin_mask_dense(name, args, qp, kp)
        ob, lb = attention_forward(md, q[:, :, qb:qe], k[:, :, kb:ke], v[:, :, kb:ke], None, sm_scale,
                                   dtype, qp, kp, T)
        o[:, :, qb:qe] = ob
        lse[:, :, qb:qe] = lb
    return o, lse


def banded_backward(name, args, q, k, v, do, sm_scale=None, block=2048, dtype=torch.float32):
    B, H, T, D = q.shape
    dq = torch.zeros(q.shape, dtype=dtype)
    dk = torch.zeros(k.shape, dtype=dtype)
    dv = torch.zeros(v.shape, dtype=dtype)
    for qb in range(0, T, block):
        qe = min(T, qb + block)
        kb, ke = _band(name, args, qb, qe, T)
        qp, kp = torch.arange(qb, qe), torch.arange(kb, ke)
        md = builtin_mask_dense(name, args, qp, kp)
        a, b, c = attention_backward(md, q[:, :, qb:qe], k[:, :, kb:ke], v[:, :, kb:ke], do[:, :, qb:qe],
                                     None, sm_scale, dtype, qp, kp, T)
        dq[:, :, qb:qe] = a
        dk[:, :, kb:ke] += b
        dv[:, :, kb:ke] += c
    return dq, dk, dv


def unmasked_pairs(name, args, T):
    """Number of (q, k) pairs a built-in mask leaves visible on [0, T)^2 (per head)."""
    total = 0
    block = 4096
    for qb in range(0, T, block):
        qe = min(T, qb + block)
        kb, ke = _band(name, args, qb, qe, T)
        total += int(builtin_mask_dense(name, args, torch.arange(qb, qe), torch.arange(kb, ke)).sum())
    return total

"""Plain-PyTorch fp32 definitions of every op the sm_100a kernels implement.

These functions are the numerics oracle of the test-suite: each CUDA kernel is compared
with the function of the same role here, on small shapes.  They restate the math of the
reference's CPU backend (``backends/reference/__init__.py``: norms l.169-250, SwiGLU
l.253-267, rope l.335-364, KV int8 quant l.367-390, gated attention l.432-489, causal
conv l.639-696, delta-net head prep l.699-731, delta step l.847-874, record/commit
l.919-957, router l.144-166) without its dispatch table.  Everything computes in fp32 and
returns fp32 unless noted.
"""
from __future__ import annotations


import torch
import torch.nn.functional as F

NEG_INF = float("-inf")


# ---------------------------------------------------------------- norms / activations
def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * gain`` over the last axis; ``gain`` already holds
    ``1 + w`` for the zero-centred norms."""
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gain.float()


def add_rms_norm(x: torch.Tensor, add: torch.Tensor, gain: torch.Tensor,
                 eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """Residual add then norm: returns ``(x + add, norm(x + add))``."""
    s = x.float() + add.float()
    return s, rms_norm(s, gain, eps)


def rms_norm_gated(x: torch.Tensor, w: torch.Tensor, gate: torch.Tensor,
                   eps: float = 1e-6) -> torch.Tensor:
    """Per-head ``norm(x) * w * silu(gate)``; ``w`` is a plain gain ``[dv]``."""
    return rms_norm(x, w, eps) * F.silu(gate.float())


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate.float()) * up.float()


def quant_rows_int8(x: torch.Tensor, floor: float = 1e-5) -> tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-row int8: ``s = max(amax, floor) / 127``; ``q = round(x / s)``."""
    xf = x.float()
    s = xf.abs().amax(-1).clamp_min(floor) / 127.0
    q = (xf / s.unsqueeze(-1)).round().clamp_(-127, 127).to(torch.int8)
    return q, s


# ---------------------------------------------------------------- rotary
def inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def rope_tables(rotary_dim: int, theta: float, max_seq: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``[max_seq, rotary_dim]`` fp32 cos/sin in the ``cat(half, half)`` layout."""
    f = torch.arange(max_seq, dtype=torch.float32)[:, None] * inv_freq(rotary_dim, theta)[None]
    return torch.cat([f.cos(), f.cos()], -1), torch.cat([f.sin(), f.sin()], -1)


def mrope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float,
                  section=(11, 11, 10)) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[L, rotary_dim]`` for 3-axis positions ``[3, L]`` (t, h, w).

    Frequency ``j`` takes its angle from axis ``j % 3`` while ``j < 3 * section[axis]``
    allows it (interleaved sections; reference ``ops/mrope.py``), else from axis 0.  With the
    three rows equal this is the ordinary 1-D table.
    """
    inv = inv_freq(rotary_dim, theta)
    half = rotary_dim // 2
    ang = positions.float()[:, :, None] * inv[None, None, :]        # [3, L, half]
    out = ang[0].clone()
    for axis in (1, 2):
        idx = torch.arange(axis, min(3 * section[axis], half), 3)
        out[:, idx] = ang[axis][:, idx]
    return torch.cat([out.cos(), out.cos()], -1), torch.cat([out.sin(), out.sin()], -1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Rotate the leading ``rotary_dim`` channels of ``x [..., T, heads, hd]`` with
    ``cos/sin [T, rotary_dim]``; channel ``i`` pairs with ``i + rotary_dim/2``."""
    xf = x.float()
    rot, rest = xf[..., :rotary_dim], xf[..., rotary_dim:]
    h = rotary_dim // 2
    rh = torch.cat([-rot[..., h:], rot[..., :h]], -1)
    c, s = cos.float().unsqueeze(-2), sin.float().unsqueeze(-2)
    return torch.cat([rot * c + rh * s, rest], -1)


# ---------------------------------------------------------------- gated softmax attention
def gated_attention(q: torch.Tensor, gate: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    q_pos: torch.Tensor, scale: float, keep: torch.Tensor | None = None) -> torch.Tensor:
    """Causal GQA attention with a sigmoid output gate.

    Args:
        q, gate: ``[T, nh, hd]`` (q already normed and rotated).
        k, v: ``[S, nkv, hd]`` — the whole visible cache in position order.
        q_pos: ``[T]`` position of each query; key ``s`` participates when ``s <= q_pos``.
        keep: optional bool ``[T, S]`` extra key mask.
    Returns ``[T, nh, hd]`` fp32.
    """
    T, nh, hd = q.shape
    S, nkv, _ = k.shape
    rep = nh // nkv
    qf = q.float().reshape(T, nkv, rep, hd)
    scores = torch.einsum("tgrd,sgd->tgrs", qf, k.float()) * scale
    mask = torch.arange(S)[None, :] > q_pos.reshape(-1, 1).cpu()
    if keep is not None:
        mask = mask | ~keep
    scores = scores.masked_fill(mask.to(scores.device)[:, None, None, :], NEG_INF)
    out = torch.einsum("tgrs,sgd->tgrd", scores.softmax(-1), v.float()).reshape(T, nh, hd)
    return out * torch.sigmoid(gate.float())


# ---------------------------------------------------------------- gated delta net
def conv1d_silu_seq(conv_w: torch.Tensor, x: torch.Tensor, conv_state: torch.Tensor
                    ) -> tuple[torch.Tensor, torch.Tensor]:
    """Depthwise causal conv (taps ``[C, K]`` oldest first) + SiLU over ``x [T, C]``.

    ``conv_state [C, K-1]`` holds the previous ``K-1`` inputs.  Returns the outputs
    ``[T, C]`` and the new state (the last ``K-1`` rows of ``state ++ x``).
    """
    K = conv_w.shape[1]
    seq = torch.cat([conv_state.float().t(), x.float()], 0)          # [K-1+T, C]
    win = seq.unfold(0, K, 1)                                        # [T, C, K]
    return F.silu((win * conv_w.float()).sum(-1)), seq[-(K - 1):].t().contiguous()


def gdn_head_prep(q: torch.Tensor, k: torch.Tensor, b: torch.Tensor, a: torch.Tensor,
                  A_log: torch.Tensor, dt_bias: torch.Tensor, rep: int):
    """L2-normalise q/k per head (eps 1e-6 inside the sqrt), scale q by ``dk**-0.5``,
    expand key heads to value heads, ``beta = sigmoid(b)``,
    ``g = -exp(A_log) * softplus(a + dt_bias)`` (a log decay <= 0).

    q, k: ``[..., num_k, dk]``; b, a: ``[..., num_v]``.
    """
    qf, kf = q.float(), k.float()
    if rep > 1:
        qf = qf.repeat_interleave(rep, -2)
        kf = kf.repeat_interleave(rep, -2)
    qn = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * (q.shape[-1] ** -0.5)
    kn = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(b.float())
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())
    return qn, kn, beta, g


def delta_step(q, k, v, beta, g, state):
    """One gated delta-rule step on ``state [nv, dk, dv]`` (updated in place).

    ``S <- S * exp(g)``; ``d = (v - S^T k) * beta``; ``S <- S + k d^T``; ``o = S^T q``.
    Returns ``(o [nv, dv], k, d, alpha)`` — the rank-one update record of this step.
    """
    alpha = g.float().exp()
    state.mul_(alpha[:, None, None])
    kv = (state * k[:, :, None]).sum(-2)
    d = (v.float() - kv) * beta[:, None]
    state.add_(k[:, :, None] * d[:, None, :])
    return (state * q[:, :, None]).sum(-2), k, d, alpha


def delta_recurrent(q, k, v, beta, g, state):
    """Token-by-token scan; q/k ``[T, nv, dk]``, v ``[T, nv, dv]``, beta/g ``[T, nv]``."""
    outs = []
    for t in range(q.shape[0]):
        o, _, _, _ = delta_step(q[t], k[t], v[t], beta[t], g[t], state)
        outs.append(o)
    return torch.stack(outs, 0)


def delta_chunked(q, k, v, beta, g, state, chunk: int = 64):
    """Chunked (WY / UT-transform) form of the same recurrence.

    For a chunk with entry state ``S0`` and cumulative log decay ``c_t``:
    ``(I + T) U = beta*(V - diag(e^c) K S0)`` with ``T_ij = beta_i e^{c_i-c_j} k_i.k_j (j<i)``;
    ``O = diag(e^c) Q S0 + (Q K^T * D) U`` with ``D_ij = e^{c_i-c_j} (j<=i)``;
    ``S_L = e^{c_L} S0 + (K * e^{c_L-c})^T U``.  Same layouts as ``delta_recurrent``.
    The state is updated in place.
    """
    T, nv, dk = q.shape
    outs = []
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        L = e - s
        qc, kc, vc = (t[s:e].transpose(0, 1).float() for t in (q, k, v))     # [nv, L, d]
        bc, gc = beta[s:e].t().float(), g[s:e].t().float()                   # [nv, L]
        c = gc.cumsum(-1)
        diff = c[:, :, None] - c[:, None, :]
        tril = torch.tril(torch.ones(L, L, dtype=torch.bool), 0)
        D = torch.where(tril, diff, torch.full_like(diff, NEG_INF)).exp()
        strict = torch.tril(torch.ones(L, L, dtype=torch.bool), -1)
        Tm = (kc @ kc.transpose(-1, -2)) * D * bc[:, :, None]
        Tm = torch.where(strict, Tm, torch.zeros_like(Tm))
        rhs = bc[:, :, None] * (vc - c.exp()[:, :, None] * (kc @ state))
        eye = torch.eye(L).expand(nv, L, L)
        U = torch.linalg.solve_triangular(eye + Tm, rhs, upper=False, unitriangular=True)
        o = c.exp()[:, :, None] * (qc @ state) + ((qc @ kc.transpose(-1, -2)) * D) @ U
        k2 = kc * (c[:, -1:] - c).exp()[:, :, None]
        state.mul_(c[:, -1].exp()[:, None, None]).add_(k2.transpose(-1, -2) @ U)
        outs.append(o.transpose(0, 1))
    return torch.cat(outs, 0)


def delta_commit(base: torch.Tensor, rec_k, rec_d, rec_alpha, steps: int) -> torch.Tensor:
    """Replay the first ``steps`` recorded rank-one updates on a copy of ``base``."""
    st = base.clone()
    for t in range(steps):
        st.mul_(rec_alpha[t][:, None, None])
        st.add_(rec_k[t][:, :, None] * rec_d[t][:, None, :])
    return st


# ---------------------------------------------------------------- MoE
def moe_route(logits: torch.Tensor, top_k: int, normalize: bool = True):
    """fp32 softmax -> top-k -> optional renormalisation. Returns ``(index, weight)``."""
    probs = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(probs, top_k, -1)
    if normalize:
        w = w / w.sum(-1, keepdim=True)
    return idx, w


def moe_ffn(x, router_w, gate_up, down, top_k, normalize=True, shared=None):
    """Routed SwiGLU experts (+ optional shared expert with a sigmoid scalar gate).

    gate_up ``[E, 2I, H]`` (gate rows first), down ``[E, H, I]``;
    shared = ``(gate_w [S,H], up_w [S,H], down_w [H,S], gate_vec [1,H])``.
    """
    xf = x.float()
    idx, w = moe_route(xf @ router_w.float().t(), top_k, normalize)
    out = torch.zeros_like(xf)
    I = gate_up.shape[1] // 2
    for t in range(xf.shape[0]):
        for j in range(top_k):
            e = int(idx[t, j])
            gu = gate_up[e].float() @ xf[t]
            h = F.silu(gu[:I]) * gu[I:]
            out[t] += w[t, j] * (down[e].float() @ h)
    if shared is not None:
        sg, su, sdn, gv = (s.float() for s in shared)
        h = F.silu(xf @ sg.t()) * (xf @ su.t())
        out = out + torch.sigmoid(xf @ gv.reshape(-1, 1)) * (h @ sdn.t())
    return out


# ---------------------------------------------------------------- quantised GEMM oracles
def w8a8_linear(x: torch.Tensor, wq: torch.Tensor, wscale: torch.Tensor) -> torch.Tensor:
    """Dynamic per-token int8 activations x per-output-channel int8 weights.

    ``wq [N, K]`` int8, ``wscale [N]``; integer dot products are exact, then
    ``y = acc * s_x[m] * s_w[n]``.
    """
    xq, xs = quant_rows_int8(x, floor=1e-8)
    acc = xq.to(torch.int32).double() @ wq.to(torch.int32).double().t()
    return (acc * xs.double()[:, None] * wscale.double()[None, :]).float()


def w4a8_linear(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, k: int,
                group: int = 128) -> torch.Tensor:
    """int8 per-token activations x int4 group-``group`` weights.

    ``packed uint8 [ceil(K/2), N]`` (low nibble = even k, code = q + 8), ``scale [G, N]``.
    Per group: exact integer partial dot, times the group's weight scale; then the token's
    activation scale.
    """
    lo = (packed & 0xF).to(torch.int32) - 8
    hi = (packed >> 4).to(torch.int32) - 8
    w = torch.stack([lo, hi], 1).reshape(-1, packed.shape[1])[:k]          # [K, N]
    xq, xs = quant_rows_int8(x, floor=1e-8)
    out = torch.zeros(x.shape[0], packed.shape[1], dtype=torch.float64)
    for gi, s in enumerate(range(0, k, group)):
        e = min(k, s + group)
        part = xq[:, s:e].to(torch.int32).double() @ w[s:e].double()
        out += part * scale[gi].double()[None, :]
    return (out * xs.double()[:, None]).float()

"""Gated delta-rule linear attention (the token mixer of Qwen3-Next / Qwen3.5's "linear_attention" layers).

Per head the layer keeps a state S [d_k, d_v] and, for every token t with key k_t, value v_t, query q_t, decay a_t in (0, 1]
and write strength b_t in (0, 1):

    S <- a_t S                       (forget)
    u_t = b_t (v_t - k_t^T S)        (what the state does not yet predict for this key)
    S <- S + k_t u_t^T               (write)
    o_t = q_t^T S                    (read)

``gated_delta_rule`` evaluates this in chunks: inside a chunk the u_t obey a unit lower-triangular linear system
(I + L) U = B with L[t, i] = b_t (c_t / c_i) (k_t . k_i) for i < t, B[t] = b_t (v_t - c_t k_t^T S_in) and c_t the decay
accumulated since the start of the chunk, which one triangular solve handles for all tokens of the chunk; outputs and the
outgoing state are then dense products. Only the loop over chunks is sequential. ``gated_delta_rule_reference`` is the
token-by-token recurrence above, used by the tests.

``GatedDeltaNet`` is the full mixer (paddleformers/transformers/qwen3_next): fused input projections grouped by key head
(q, k, v, output gate z; write strength and decay inputs), a causal depth-wise convolution with SiLU over q | k | v, L2-normalised
q and k, decay a_t = exp(-exp(A_log) softplus(x_a + dt_bias)), a per-head RMSNorm of the read-out gated by SiLU(z), and the
output projection. It runs as tensor operations on every device; with a cache object it continues from the stored
convolution tail and recurrent state (incremental decoding).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as TF


def gated_delta_rule_reference(q, k, v, log_decay, beta, state=None):
    """q, k: [B, S, H, dk]; v: [B, S, H, dv]; log_decay, beta: [B, S, H]. Returns (o [B, S, H, dv], final state)."""
    B, S, H, dk = k.shape
    dv = v.shape[-1]
    St = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device) if state is None else state.float()
    q, k, v, log_decay, beta = (x.float() for x in (q, k, v, log_decay, beta))
    out = []
    for t in range(S):
        St = St * log_decay[:, t].exp()[..., None, None]
        u = beta[:, t][..., None] * (v[:, t] - torch.einsum("bhk,bhkv->bhv", k[:, t], St))
        St = St + torch.einsum("bhk,bhv->bhkv", k[:, t], u)
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t], St))
    return torch.stack(out, dim=1), St


def gated_delta_rule(q, k, v, log_decay, beta, chunk: int = 64, state=None):
    """Chunked evaluation of the gated delta rule (same arguments and result as ``gated_delta_rule_reference``)."""
    B, S, H, dk = k.shape
    dv = v.shape[-1]
    dtype = v.dtype
    pad = (-S) % chunk
    q, k, v, log_decay, beta = (x.float().transpose(1, 2) for x in (q, k, v, log_decay, beta))       # [B, H, S, ...]
    if pad:                     # padded steps: no decay (log 0 = 1x), no write (beta 0), outputs dropped
        q, k, v = (TF.pad(x, (0, 0, 0, pad)) for x in (q, k, v))
        log_decay, beta = TF.pad(log_decay, (0, pad)), TF.pad(beta, (0, pad))
    n = (S + pad) // chunk
    q, k, v = (x.reshape(B, H, n, chunk, -1) for x in (q, k, v))
    beta = beta.reshape(B, H, n, chunk)
    G = log_decay.reshape(B, H, n, chunk).cumsum(-1)                        # log c_t inside each chunk
    ratio = (G[..., :, None] - G[..., None, :]).tril().exp().tril()          # c_t / c_i for i <= t, 0 above the diagonal
    kk = k @ k.transpose(-1, -2)
    L = (beta[..., None] * ratio * kk).tril(-1)                              # strictly lower part
    eye = torch.eye(chunk, dtype=torch.float32, device=q.device)
    qk = (q @ k.transpose(-1, -2)) * ratio                                   # (c_t / c_i)(q_t . k_i), i <= t
    c = G.exp()                                                              # [B, H, n, chunk]
    St = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device) if state is None else state.float()
    outs = []
    for j in range(n):
        kj, cj = k[:, :, j], c[:, :, j]
        rhs = beta[:, :, j, :, None] * (v[:, :, j] - cj[..., None] * (kj @ St))
        U = torch.linalg.solve_triangular(eye + L[:, :, j], rhs, upper=False, unitriangular=True)
        outs.append(cj[..., None] * (q[:, :, j] @ St) + qk[:, :, j] @ U)
        last = cj[..., -1]                                                   # decay over the whole chunk
        w = (G[:, :, j, -1:, ] - G[:, :, j]).exp()                           # c_C / c_i
        St = St * last[..., None, None] + (kj * w[..., None]).transpose(-1, -2) @ U
    o = torch.stack(outs, dim=2).reshape(B, H, n * chunk, dv)[:, :, :S]
    return o.transpose(1, 2).to(dtype), St


class GatedDeltaNet(nn.Module):
    def __init__(self, config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = config.hidden_size
        self.nv, self.nk = config.linear_num_value_heads, config.linear_num_key_heads
        self.dk, self.dv = config.linear_key_head_dim, config.linear_value_head_dim
        self.key_dim, self.value_dim = self.nk * self.dk, self.nv * self.dv
        self.kernel = config.linear_conv_kernel_dim
        self.eps = config.rms_norm_eps
        conv_dim = 2 * self.key_dim + self.value_dim
        # Qwen3-Next fuses the input projections per key head; Qwen3.5 keeps four flat ones
        self.split_proj = bool(getattr(config, "linear_attn_split_projections", False))
        if self.split_proj:
            self.in_proj_qkv = nn.Linear(H, conv_dim, bias=False, **kw)
            self.in_proj_z = nn.Linear(H, self.value_dim, bias=False, **kw)
            self.in_proj_b = nn.Linear(H, self.nv, bias=False, **kw)
            self.in_proj_a = nn.Linear(H, self.nv, bias=False, **kw)
        else:
            self.in_proj_qkvz = nn.Linear(H, 2 * self.key_dim + 2 * self.value_dim, bias=False, **kw)
            self.in_proj_ba = nn.Linear(H, 2 * self.nv, bias=False, **kw)
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, self.kernel, groups=conv_dim, bias=False, padding=self.kernel - 1, **kw)
        self.dt_bias = nn.Parameter(torch.ones(self.nv, **kw))
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nv, dtype=torch.float32, device=device).uniform_(1, 16)).to(dtype or torch.float32))
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.dv, **kw))
        self.out_proj = nn.Linear(self.value_dim, H, bias=False, **kw)

    def forward(self, x2d: torch.Tensor, ctx, cache=None) -> torch.Tensor:
        """``cache`` (any object; attributes are added to it) keeps what incremental decoding needs between calls: the last
        ``kernel - 1`` inputs of the convolution and the recurrent state."""
        B, S = ctx.B, ctx.S
        r = self.nv // self.nk
        if self.split_proj:
            mixed = self.in_proj_qkv(x2d).view(B, S, -1).transpose(1, 2)
            z, b, a = self.in_proj_z(x2d), self.in_proj_b(x2d), self.in_proj_a(x2d)
        else:
            # projections are laid out per key head: [q (dk) | k (dk) | v (r dv) | z (r dv)] and [b (r) | a (r)]
            qkvz = self.in_proj_qkvz(x2d).view(B, S, self.nk, 2 * self.dk + 2 * r * self.dv)
            ba = self.in_proj_ba(x2d).view(B, S, self.nk, 2 * r)
            q, k, v, z = qkvz.split([self.dk, self.dk, r * self.dv, r * self.dv], dim=-1)
            b, a = ba.split([r, r], dim=-1)
            mixed = torch.cat([q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)], dim=-1).transpose(1, 2)
        if cache is None:
            mixed = TF.silu(self.conv1d(mixed)[:, :, :S]).transpose(1, 2)      # causal: left padding, right part dropped
        else:
            tail = getattr(cache, "conv_tail", None)
            if tail is None:
                tail = mixed.new_zeros(B, mixed.shape[1], self.kernel - 1)
            padded = torch.cat([tail, mixed], dim=-1)
            cache.conv_tail = padded[:, :, -(self.kernel - 1):].detach()
            mixed = TF.silu(TF.conv1d(padded, self.conv1d.weight, None, groups=padded.shape[1])).transpose(1, 2)
        q, k, v = mixed.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k = q.reshape(B, S, self.nk, self.dk), k.reshape(B, S, self.nk, self.dk)
        v, z = v.reshape(B, S, self.nv, self.dv), z.reshape(B, S, self.nv, self.dv)
        beta = torch.sigmoid(b.reshape(B, S, self.nv))
        log_decay = -self.A_log.float().exp() * TF.softplus(a.reshape(B, S, self.nv).float() + self.dt_bias.float())
        if r > 1:
            q, k = q.repeat_interleave(r, dim=2), k.repeat_interleave(r, dim=2)

        def l2(t):
            t = t.float()
            return t * torch.rsqrt(t.pow(2).sum(-1, keepdim=True) + 1e-6)

        o, state = gated_delta_rule(l2(q) * self.dk ** -0.5, l2(k), v, log_decay, beta,
                                    state=getattr(cache, "linear_state", None) if cache is not None else None)
        if cache is not None:
            cache.linear_state = state.detach()
        o = o.float()
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps)
        o = (self.norm.weight * o.to(x2d.dtype)) * TF.silu(z.float())
        return self.out_proj(o.to(x2d.dtype).reshape(B * S, self.value_dim))


def decayed_linear_attention(q, k, v, slope, chunk: int = 64, state=None):
    """Causal linear attention with a fixed exponential decay per head ("lightning attention", MiniMax-Text):
    o_t = sum_{i <= t} exp(-slope_h (t - i)) (q_t . k_i) v_i. q, k, v: [B, S, H, D]; slope: [H] (> 0).
    Inside a chunk the decayed score matrix is formed explicitly; across chunks a [D, D] state per head carries the sum of
    decayed k v^T. Returns (o [B, S, H, D], final state [B, H, D, D])."""
    B, S, H, D = q.shape
    dtype = v.dtype
    q, k, v = (x.float().transpose(1, 2) for x in (q, k, v))                       # [B, H, S, D]
    slope = slope.float().view(1, H, 1, 1)
    St = torch.zeros(B, H, D, v.shape[-1], dtype=torch.float32, device=q.device) if state is None else state.float()
    outs = []
    for lo in range(0, S, chunk):
        qc, kc, vc = q[:, :, lo:lo + chunk], k[:, :, lo:lo + chunk], v[:, :, lo:lo + chunk]
        n = qc.shape[2]
        pos = torch.arange(n, device=q.device, dtype=torch.float32)
        dist = pos[:, None] - pos[None, :]
        decay = torch.where(dist >= 0, torch.exp(-slope * dist.clamp(min=0)), torch.zeros((), device=q.device))   # [1, H, n, n]
        intra = ((qc @ kc.transpose(-1, -2)) * decay) @ vc
        inter = (qc * torch.exp(-slope * (pos + 1).view(1, 1, n, 1))) @ St          # the state is "one step before the chunk"
        outs.append(intra + inter)
        St = St * torch.exp(-slope * n) + (kc * torch.exp(-slope * (n - 1 - pos).view(1, 1, n, 1))).transpose(-1, -2) @ vc
    return torch.cat(outs, dim=2).transpose(1, 2).to(dtype), St


class LightningAttention(nn.Module):
    """MiniMax-Text's linear-attention mixer (paddleformers/transformers/minimax): SiLU on the fused q | k | v projection (laid out
    per head), decayed linear attention with head- and depth-dependent slopes, RMSNorm over all heads, a sigmoid output gate
    computed from the layer input, output projection."""

    def __init__(self, config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H, self.nh, self.hd = config.hidden_size, config.num_attention_heads, config.head_dim
        self.chunk = int(getattr(config, "block_size", 64) or 64)
        self.qkv = nn.Linear(H, 3 * self.nh * self.hd, bias=False, **kw)
        self.gate = nn.Linear(H, self.nh * self.hd, bias=False, **kw)
        self.out = nn.Linear(self.nh * self.hd, H, bias=False, **kw)
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.nh * self.hd, **kw))
        self.eps = 1e-6
        base = 1.0 / (2.0 ** (8.0 / self.nh))
        depth = 1.0 - layer_idx / (config.num_hidden_layers - 1 + 1e-5) + 1e-5
        self.register_buffer("slope", (base ** (torch.arange(self.nh, dtype=torch.float32, device=device) + 1)) * depth, persistent=False)

    def forward(self, x2d, ctx, cache=None):
        B, S = ctx.B, ctx.S
        q, k, v = TF.silu(self.qkv(x2d)).view(B, S, self.nh, 3 * self.hd).split(self.hd, dim=-1)
        o, state = decayed_linear_attention(q, k, v, self.slope, self.chunk,
                                            state=getattr(cache, "linear_state", None) if cache is not None else None)
        if cache is not None:               # incremental decoding: the decayed sum of k v^T so far
            cache.linear_state = state.detach()
        o = o.reshape(B * S, self.nh * self.hd).float()
        o = (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps)).to(x2d.dtype) * self.norm.weight
        return self.out(torch.sigmoid(self.gate(x2d)) * o)

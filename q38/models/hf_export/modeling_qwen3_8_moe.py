"""Q38 sparse MoE language model: module tree, parameter names and the plain-PyTorch math.

This single file is both

* the model definition used by training and evaluation (``q38.models`` re-exports it and
  installs the sm_100a kernel backend with :func:`set_backend`), and
* the remote-code file carried by the HF export: it depends only on ``torch`` (and, for the
  ``PreTrainedModel`` wrappers at the bottom, on ``transformers``), so a directory written by
  ``save_pretrained`` loads with ``AutoModelForCausalLM.from_pretrained(..., trust_remote_code=True)``.

Every hot function has two implementations: the PyTorch one written here, which is the
numerical specification (fp32 on CPU it is the oracle of the kernel tests), and, when a backend
is installed and the tensors live on a GPU, a hand-written CUDA kernel path.  State-dict keys and
parameter registration order match the reference model
(q38/models/qwen3_8_moe/modeling_qwen3_8_moe.py:418-461, 663-690, 740-835, 1032-1043,
1065-1071, 1168-1176, 1210-1231, 1358-1388) so `ckpt.pt` files and optimizer state dicts are
interchangeable.

Architecture in one paragraph: token embeddings are replicated into ``n_branch`` fp32 residual
streams ``X[B,S,n,h]``.  Each layer applies two mHC-wrapped sub-layers (token mixer, then MoE):
``mhc.pre`` reads a convex-ish combination of the streams, the sub-layer runs on it, ``mhc.post``
mixes the streams with a Sinkhorn-normalised 4x4 matrix and writes the output back.  Three of
four token mixers are Gated DeltaNet layers, the fourth is QSA: gated GQA attention restricted to
the top-k 64-token key blocks chosen per query block by a small MQA indexer that is trained only
by a KL term against the dense attention's block mass.  Hashed bigram/trigram embeddings are
added after layer 0.  A one-layer MTP head predicts token t+2 during training.
"""
from __future__ import annotations

import copy
import math
import os

import torch
import torch.nn.functional as F
import torch.utils.checkpoint
from torch import nn

BLK = 64                      # QSA block size, GDN chunk size and sequence padding granule

# --------------------------------------------------------------------------- kernel backend
_BACKEND = None


def set_backend(backend):
    """Install (or with ``None`` remove) the object that provides the CUDA implementations."""
    global _BACKEND
    _BACKEND = backend


def get_backend():
    return _BACKEND


def _hook(name: str, t: torch.Tensor):
    """The backend's implementation of `name` for tensors like `t`, or ``None`` to use the PyTorch path."""
    if _BACKEND is None or not t.is_cuda:
        return None
    return getattr(_BACKEND, name, None)


def _embed(table: nn.Embedding, ids):
    """Embedding lookup; on a GPU the backend scatters the gradient straight into the table's gradient buffer."""
    fast = _hook("embedding", table.weight)
    if fast is not None:
        return fast(table.weight, ids)
    return table(ids)


def _linear(x, weight, bias=None):
    """``x @ weight.T`` in the dtype of ``x`` (fp32 master weights are cast per use)."""
    fast = _hook("linear", x)
    if fast is not None and bias is None:
        return fast(x, weight)
    return F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


# --------------------------------------------------------------------------- normalisation
class Qwen3_8MoeRMSNorm(nn.Module):
    """Zero-centred RMSNorm: ``x_hat * (1 + w)`` evaluated in fp32, weight initialised to 0."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.zeros(dim))

    def forward(self, x, out_dtype=None):
        out_dtype = out_dtype or x.dtype
        fast = _hook("rmsnorm", x)
        if fast is not None:
            return fast(x, self.weight, self.eps, out_dtype)
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * (1.0 + self.weight.float())).to(out_dtype)

    def extra_repr(self):
        return f"{tuple(self.weight.shape)}, eps={self.eps}"


class Qwen3_8MoeRMSNormGated(nn.Module):
    """Per-head RMSNorm followed by a SiLU gate.

    Rounding points: normalise in fp32, round to the input dtype, multiply by the weight, then by
    ``silu(gate)`` in fp32, round again."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x, gate):
        fast = _hook("gated_rmsnorm", x)
        if fast is not None and x.dtype == torch.bfloat16 and x.shape[-1] == 64:
            return fast(x, gate, self.weight, self.variance_epsilon)
        dt = x.dtype
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        y = self.weight * xf.to(dt)
        return (y * F.silu(gate.float())).to(dt)


# --------------------------------------------------------------------------- rotary embedding
def rope_tables(positions, rotary_dim, theta, dtype):
    """cos/sin ``[.., S, rotary_dim]`` for the rotate-half convention on the leading ``rotary_dim`` dims."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=positions.device) / rotary_dim))
    ang = positions.float()[..., None] * inv
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):
    """x ``[B,H,S,D]``; rotates the first ``cos.shape[-1]`` dims, passes the rest through."""
    rd = cos.shape[-1]
    rot, rest = x[..., :rd], x[..., rd:]
    half = rd // 2
    turned = torch.cat([-rot[..., half:], rot[..., :half]], dim=-1)
    c, s = cos[:, None].to(x.dtype), sin[:, None].to(x.dtype)
    return torch.cat([rot * c + turned * s, rest], dim=-1)


# --------------------------------------------------------------------------- Gated DeltaNet
def l2norm(x, eps=1e-6):
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_chunk_operands(q, k, v, g, beta, chunk=BLK):
    """Per-chunk operands of the chunked delta rule, all ``[B,Hv,n,chunk,D]`` fp32 (``carry`` is ``[B,Hv,n]``).

    With ``gc`` the cumulative log-decay inside a chunk and ``Gamma_ij = exp(gc_i - gc_j)``:
    ``Tm = (I + tril(beta_i (k_i.k_j) Gamma_ij, -1))^-1``, ``w = Tm (beta e^gc k)``, ``u = Tm (beta v)``,
    ``P = tril((q_i.k_j) Gamma_ij)``, ``qg = q e^gc``, ``kg = k e^(gc_last - gc)``, ``carry = e^gc_last``.
    q and k are L2-normalised and q is scaled by ``D**-0.5``.  The sequence is right-padded to a multiple of the chunk.
    """
    B, S, Hk, D = k.shape
    Hv = v.shape[2]
    rep = Hv // Hk
    q = l2norm(q.float()) * D ** -0.5
    k = l2norm(k.float())
    if rep > 1:
        q = q.repeat_interleave(rep, dim=2)
        k = k.repeat_interleave(rep, dim=2)
    pad = (-S) % chunk
    tr = lambda t: F.pad(t.float().transpose(1, 2), (0, 0, 0, pad) if t.dim() == 4 else (0, pad))
    q, k, v, g, beta = tr(q), tr(k), tr(v), tr(g), tr(beta)               # [B,H,Sp,(D)]
    n = (S + pad) // chunk
    q, k, v = (t.reshape(B, Hv, n, chunk, -1) for t in (q, k, v))
    g, beta = g.reshape(B, Hv, n, chunk), beta.reshape(B, Hv, n, chunk)
    gc = g.cumsum(-1)                                                        # decay from chunk start
    diff = gc[..., :, None] - gc[..., None, :]
    lower = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    decay = torch.where(lower, diff, torch.full_like(diff, float("-inf"))).exp()
    kb, vb = k * beta[..., None], v * beta[..., None]
    system = (kb @ k.transpose(-1, -2)) * decay                             # unit lower-triangular system
    u = torch.linalg.solve_triangular(system, vb, upper=False, unitriangular=True)
    w = torch.linalg.solve_triangular(system, kb * gc.exp()[..., None], upper=False, unitriangular=True)
    return dict(w=w, u=u, P=(q @ k.transpose(-1, -2)) * decay, qg=q * gc.exp()[..., None],
                kg=k * (gc[..., -1:] - gc).exp()[..., None], carry=gc[..., -1].exp())


def gated_delta_rule_chunked(q, k, v, g, beta, chunk=BLK):
    """Chunked gated delta rule; the fp32 specification of the GDN kernels.

    q,k ``[B,S,Hk,D]``; v ``[B,S,Hv,D]``; g (log decay, <= 0) and beta ``[B,S,Hv]``.  Value head j
    reads key head ``j // (Hv/Hk)``.  Per head and token:
    ``S <- exp(g) S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q``.
    The state starts at zero and is not reset at document boundaries.
    """
    out_dtype = q.dtype
    B, S = k.shape[:2]
    ops = gdn_chunk_operands(q, k, v, g, beta, chunk)
    n = ops["w"].shape[2]
    state = ops["w"].new_zeros(B, v.shape[2], k.shape[-1], v.shape[-1])
    outs = []
    for i in range(n):
        v_new = ops["u"][:, :, i] - ops["w"][:, :, i] @ state
        outs.append(ops["qg"][:, :, i] @ state + ops["P"][:, :, i] @ v_new)
        state = state * ops["carry"][:, :, i, None, None] + ops["kg"][:, :, i].transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(B, v.shape[2], n * chunk, -1)[:, :, :S]
    return o.transpose(1, 2).contiguous().to(out_dtype)


def gated_delta_rule_recurrent(q, k, v, g, beta):
    """Token-by-token form of the same recurrence (test oracle for the chunked form)."""
    B, S, Hk, D = k.shape
    Hv = v.shape[2]
    rep = Hv // Hk
    q = (l2norm(q.float()) * D ** -0.5).repeat_interleave(rep, dim=2)
    k = l2norm(k.float()).repeat_interleave(rep, dim=2)
    v, g, beta = v.float(), g.float(), beta.float()
    state = q.new_zeros(B, Hv, D, v.shape[-1])
    outs = []
    for t in range(S):
        state = state * g[:, t].exp()[..., None, None]
        pred = torch.einsum("bhkv,bhk->bhv", state, k[:, t])
        state = state + torch.einsum("bhk,bhv->bhkv", k[:, t], (v[:, t] - pred) * beta[:, t][..., None])
        outs.append(torch.einsum("bhkv,bhk->bhv", state, q[:, t]))
    return torch.stack(outs, 1)


def causal_conv_silu(x, weight):
    """Depthwise causal conv (left padding ``K-1``) + SiLU on ``[B,S,C]``; weight ``[C,1,K]``."""
    K = weight.shape[-1]
    y = F.conv1d(x.transpose(1, 2), weight.to(x.dtype), None, padding=K - 1, groups=x.shape[-1])[..., :x.shape[1]]
    return F.silu(y).transpose(1, 2)


class Qwen3_8MoeGatedDeltaNet(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_v_heads, self.num_k_heads = config.linear_num_value_heads, config.linear_num_key_heads
        self.head_k_dim, self.head_v_dim = config.linear_key_head_dim, config.linear_value_head_dim
        self.key_dim = self.head_k_dim * self.num_k_heads
        self.value_dim = self.head_v_dim * self.num_v_heads
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_kernel_size = config.linear_conv_kernel_dim
        self.layer_idx = layer_idx
        # registration order is part of the checkpoint contract (index-based optimizer state)
        self.dt_bias = nn.Parameter(torch.ones(self.num_v_heads))
        self.A_log = nn.Parameter(torch.empty(self.num_v_heads).uniform_(0.01, 16).log_())
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, self.conv_kernel_size, groups=self.conv_dim,
                                padding=self.conv_kernel_size - 1, bias=False)
        self.norm = Qwen3_8MoeRMSNormGated(self.head_v_dim, eps=config.rms_norm_eps)
        self.out_proj = nn.Linear(self.value_dim, self.hidden_size, bias=False)
        self.in_proj_qkv = nn.Linear(self.hidden_size, self.conv_dim, bias=False)
        self.in_proj_z = nn.Linear(self.hidden_size, self.value_dim, bias=False)
        self.in_proj_b = nn.Linear(self.hidden_size, self.num_v_heads, bias=False)
        self.in_proj_a = nn.Linear(self.hidden_size, self.num_v_heads, bias=False)

    def forward(self, x):
        fast = _hook("gated_deltanet", x)
        if fast is not None:
            out = fast(self, x)
            if out is not None:
                return out
        B, S, _ = x.shape
        qkv = causal_conv_silu(_linear(x, self.in_proj_qkv.weight), self.conv1d.weight)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        z = _linear(x, self.in_proj_z.weight)
        beta = _linear(x, self.in_proj_b.weight).sigmoid()
        g = -self.A_log.float().exp() * F.softplus(_linear(x, self.in_proj_a.weight).float() + self.dt_bias.float())
        o = gated_delta_rule_chunked(q.reshape(B, S, -1, self.head_k_dim), k.reshape(B, S, -1, self.head_k_dim),
                                     v.reshape(B, S, -1, self.head_v_dim), g, beta)
        o = self.norm(o.reshape(-1, self.head_v_dim), z.reshape(-1, self.head_v_dim))
        return _linear(o.reshape(B, S, -1), self.out_proj.weight)


# --------------------------------------------------------------------------- attention (weights only) + QSA
class Qwen3_8MoeAttention(nn.Module):
    """Holds the gated-attention weights; the computation lives in :func:`qsa_attention`."""

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.head_dim = config.head_dim
        self.num_heads, self.num_kv_heads = config.num_attention_heads, config.num_key_value_heads
        self.scaling = self.head_dim ** -0.5
        h = config.hidden_size
        self.q_proj = nn.Linear(h, self.num_heads * self.head_dim * 2, bias=False)     # query || output gate per head
        self.k_proj = nn.Linear(h, self.num_kv_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(h, self.num_kv_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, h, bias=False)
        self.q_norm = Qwen3_8MoeRMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.k_norm = Qwen3_8MoeRMSNorm(self.head_dim, eps=config.rms_norm_eps)


class Indexer(nn.Module):
    """MQA "lightning indexer": ``I[t,s] = sum_j w_j(t) relu(q_j(t) . k(s)) / sqrt(d)``."""

    def __init__(self, hidden, heads=4, head_dim=64):
        super().__init__()
        self.n_ih, self.d_ih = heads, head_dim
        self.wq = nn.Linear(hidden, heads * head_dim, bias=False)
        self.wk = nn.Linear(hidden, head_dim, bias=False)
        self.ww = nn.Linear(hidden, heads, bias=False)

    def project(self, x, cos, sin):
        B, S, _ = x.shape
        q = _linear(x, self.wq.weight).view(B, S, self.n_ih, self.d_ih).transpose(1, 2)
        k = _linear(x, self.wk.weight).view(B, S, 1, self.d_ih).transpose(1, 2)
        w = _linear(x, self.ww.weight).float() * self.n_ih ** -0.5
        return apply_rope(q, cos, sin), apply_rope(k, cos, sin), w

    def forward(self, x, cos, sin, block_queries=False):
        q, k, w = self.project(x, cos, sin)
        if block_queries:
            q, w = q[:, :, ::BLK], w[:, ::BLK]
        scores = torch.matmul(q, k.transpose(-1, -2)).float()                  # [B,nh,Q,S]
        return torch.einsum("bhts,bth->bts", F.relu(scores) * self.d_ih ** -0.5, w)


@torch.no_grad()
def block_mass(q, k, scale, rows_per_pass=256):
    """Head-averaged probability mass that dense causal attention puts on each 64-key block: ``[B,S,nb]``."""
    B, nq, S, d = q.shape
    nkv = k.shape[1]
    qg = q.view(B, nkv, nq // nkv, S, d)
    cols = torch.arange(S, device=q.device)
    parts = []
    for t0 in range(0, S, rows_per_pass):
        t1 = min(S, t0 + rows_per_pass)
        s = torch.matmul(qg[:, :, :, t0:t1], k[:, :, None].transpose(-1, -2)).float() * scale
        s = s.masked_fill(cols[None, :] > torch.arange(t0, t1, device=q.device)[:, None], float("-inf"))
        p = s.softmax(-1).view(B, nkv, nq // nkv, t1 - t0, S // BLK, BLK).sum(-1)
        parts.append(p.mean(dim=(1, 2)))
    return torch.cat(parts, dim=1)


def select_blocks(lp_blk, budget):
    """Top-``budget`` key blocks per query block, scored by the first query of the block.

    ``lp_blk`` is ``[B,S,nb]`` (all queries) or ``[B,nb,nb]`` (first queries only).  The own block is
    always kept and future blocks never are.  Returns ``(count[B,nb] int32, index[B,nb,k] int32)``;
    only the first ``count`` entries of a row are meaningful.
    """
    B, Q, nb = lp_blk.shape
    k = min(budget, nb)
    p = lp_blk.detach().exp()
    if Q != nb:
        p = p.view(B, nb, BLK, nb)[:, :, 0]
    qb = torch.arange(nb, device=p.device)[:, None]
    kb = torch.arange(nb, device=p.device)[None, :]
    p = torch.where(kb > qb, torch.full_like(p, -1.0), p)
    p = torch.where(kb == qb, torch.full_like(p, 2.0), p)
    index = p.topk(k, dim=-1).indices.to(torch.int32)
    count = torch.clamp(qb[:, 0] + 1, max=k).to(torch.int32)[None].expand(B, -1).contiguous()
    return count, index


def block_sparse_mask(count, index, S):
    """Dense boolean ``[B,S,S]`` mask equivalent to the selected blocks with in-block causality."""
    B, nb, k = index.shape
    slot = torch.arange(k, device=index.device)[None, None, :]
    chosen = torch.zeros(B, nb, nb, dtype=torch.bool, device=index.device)
    chosen.scatter_(2, index.long(), slot < count[..., None])
    mask = chosen.repeat_interleave(BLK, 1).repeat_interleave(BLK, 2)
    return mask & torch.ones(S, S, dtype=torch.bool, device=index.device).tril()


QSA_STAT = {}


def qsa_attention(attn, x, cos, sin, indexer, budget, dense, want_kl):
    """Gated GQA attention, dense (warm-up) or restricted to indexer-selected blocks.

    Returns ``(output, kl)``; ``kl`` is the indexer's distillation loss (``None`` when not training).
    The indexer sees ``x.detach()`` and gets gradient from the KL term only; block selection is not
    differentiated.  (Reference: modeling_qwen3_8_moe.py:1117-1160.)
    """
    fast = _hook("qsa_attention", x)
    if fast is not None:
        out = fast(attn, x, cos, sin, indexer, budget, dense, want_kl)
        if out is not None:
            return out
    B, S, _ = x.shape
    hd = attn.head_dim
    qg = _linear(x, attn.q_proj.weight).view(B, S, -1, 2 * hd)
    q, gate = qg[..., :hd], qg[..., hd:].reshape(B, S, -1)
    q = apply_rope(attn.q_norm(q).transpose(1, 2), cos, sin)
    k = apply_rope(attn.k_norm(_linear(x, attn.k_proj.weight).view(B, S, -1, hd)).transpose(1, 2), cos, sin)
    v = _linear(x, attn.v_proj.weight).view(B, S, -1, hd).transpose(1, 2)
    kl = lp_blk = None
    if indexer is not None and (want_kl or not dense):
        first_only = not want_kl and not os.environ.get("Q38_INDEXER_BASELINE")
        score = indexer(x.detach(), cos, sin, block_queries=first_only)
        pos = torch.arange(S, device=x.device)
        qpos = pos[::BLK] if first_only else pos
        score = score.masked_fill(pos[None, :] > qpos[:, None], -1e9)         # finite: keeps the backward NaN-free
        lp = score.log_softmax(-1)
        lp_blk = lp.view(B, lp.shape[1], S // BLK, BLK).logsumexp(-1)
        if want_kl:
            P = block_mass(q.detach(), k.detach(), attn.scaling)
            kl = torch.where(P > 0, P * (P.clamp(min=1e-12).log() - lp_blk), torch.zeros_like(P)).sum(-1).mean()
            if QSA_STAT.get("on") and not dense:
                with torch.no_grad():
                    cnt, idx = select_blocks(lp_blk, budget)
                    sel = block_sparse_mask(cnt, idx, S)[:, ::BLK, ::BLK].float()
                    QSA_STAT.setdefault("recall", []).append(
                        (P.view(B, S // BLK, BLK, -1) * sel[:, :, None, :]).sum(-1).mean().item())
    if dense or indexer is None:
        o = F.scaled_dot_product_attention(q, k, v, scale=attn.scaling, is_causal=True, enable_gqa=True)
    else:
        cnt, idx = select_blocks(lp_blk, budget)
        mask = block_sparse_mask(cnt, idx, S)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask[:, None], scale=attn.scaling, enable_gqa=True)
    o = o.transpose(1, 2).reshape(B, S, -1) * torch.sigmoid(gate)
    return _linear(o, attn.o_proj.weight), kl


# --------------------------------------------------------------------------- MoE
class Qwen3_8MoeMLP(nn.Module):
    def __init__(self, config, intermediate_size):
        super().__init__()
        h = config.hidden_size
        self.gate_proj = nn.Linear(h, intermediate_size, bias=False)
        self.up_proj = nn.Linear(h, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, h, bias=False)

    def forward(self, x):
        return _linear(F.silu(_linear(x, self.gate_proj.weight)) * _linear(x, self.up_proj.weight), self.down_proj.weight)


class Qwen3_8MoeExperts(nn.Module):
    """Routed experts as 3-D tensors ``gate_up_proj[E,2f,h]`` and ``down_proj[E,h,f]``."""

    def __init__(self, config):
        super().__init__()
        self.num_experts, self.hidden_dim = config.num_experts, config.hidden_size
        self.intermediate_dim = config.moe_intermediate_size
        self.gate_up_proj = nn.Parameter(torch.empty(self.num_experts, 2 * self.intermediate_dim, self.hidden_dim))
        self.down_proj = nn.Parameter(torch.empty(self.num_experts, self.hidden_dim, self.intermediate_dim))

    def forward(self, x, top_idx, top_w):
        """Sorted-by-expert evaluation; contributions are summed in top-k slot order (no atomics)."""
        T, k = top_idx.shape
        order = torch.sort(top_idx.reshape(-1), stable=True).indices
        counts = torch.bincount(top_idx.reshape(-1), minlength=self.num_experts).tolist()
        rows = x[order // k]
        outs, start = [], 0
        for e, c in enumerate(counts):
            if c:
                xe = rows[start:start + c]
                gu = F.linear(xe, self.gate_up_proj[e].to(x.dtype))
                f = self.intermediate_dim
                outs.append(F.linear(F.silu(gu[:, :f]) * gu[:, f:], self.down_proj[e].to(x.dtype)))
            start += c
        y = torch.cat(outs) * top_w.reshape(-1)[order, None]
        pairs = torch.zeros(T * k, self.hidden_dim, dtype=y.dtype, device=y.device).index_copy(0, order, y)
        return pairs.view(T, k, -1).sum(1)


class Qwen3_8MoeTopKRouter(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.top_k, self.num_experts, self.hidden_dim = config.num_experts_per_tok, config.num_experts, config.hidden_size
        self.weight = nn.Parameter(torch.zeros(self.num_experts, self.hidden_dim))

    def forward(self, x):
        logits = _linear(x.reshape(-1, self.hidden_dim), self.weight)
        probs = logits.softmax(-1, dtype=torch.float32)
        top_p, top_idx = probs.topk(self.top_k, dim=-1)
        top_w = (top_p / top_p.sum(-1, keepdim=True)).to(logits.dtype)
        return logits, top_w, top_idx, probs


class RouterStats:
    """Accumulates, over the routers of one forward pass, what the balancing loss needs.

    ``loss = E * sum_e mean_rows(assignments_e) * mean_rows(prob_e)`` with both means taken over the
    rows of all recorded routers (L layers + the MTP block).  Only the probabilities carry gradient.
    (Reference: modeling_qwen3_8_moe.py:1289-1355 applied to the hooked router logits, q38/train.py:228-262.)
    """

    def __init__(self, num_experts):
        self.num_experts = num_experts
        self.counts, self.prob_sums, self.rows = [], [], 0

    def add(self, counts, prob_sum, rows):
        self.counts.append(counts)
        self.prob_sums.append(prob_sum)
        self.rows += rows

    def loss(self):
        if not self.counts:
            return 0
        f = torch.stack(self.counts).sum(0).float() / self.rows
        p = torch.stack(self.prob_sums).sum(0) / self.rows
        return (f * p).sum() * self.num_experts


class Qwen3_8MoeSparseMoeBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate = Qwen3_8MoeTopKRouter(config)
        self.experts = Qwen3_8MoeExperts(config)
        self.shared_expert = Qwen3_8MoeMLP(config, config.shared_expert_intermediate_size)
        self.shared_expert_gate = nn.Linear(config.hidden_size, 1, bias=False)
        self.stats_sink = None            # a RouterStats while a loss forward is recording, else None

    def _recording(self):
        return self.stats_sink is not None and self.training and torch.is_grad_enabled()

    def forward(self, x):
        fast = _hook("moe_block", x)
        if fast is not None:
            out = fast(self, x)
            if out is not None:
                return out
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        _, top_w, top_idx, probs = self.gate(x2)
        if self._recording():
            self.stats_sink.add(torch.bincount(top_idx.reshape(-1), minlength=self.gate.num_experts),
                                probs.sum(0), x2.shape[0])
        routed = self.experts(x2, top_idx, top_w)
        shared = torch.sigmoid(_linear(x2, self.shared_expert_gate.weight)) * self.shared_expert(x2)
        return (routed + shared).reshape(shape)


# --------------------------------------------------------------------------- decoder layer
class Qwen3_8MoeDecoderLayer(nn.Module):
    """Container of one layer's sub-modules.  The trunk drives them through mHC; only the MTP block
    uses :meth:`forward`, which is a plain pre-norm residual layer."""

    def __init__(self, config, layer_idx, block_type=None):
        super().__init__()
        self.block_type = block_type or config.layer_types[layer_idx]
        if self.block_type == "linear_attention":
            self.linear_attn = Qwen3_8MoeGatedDeltaNet(config, layer_idx)
        else:
            self.self_attn = Qwen3_8MoeAttention(config, layer_idx)
        self.mlp = Qwen3_8MoeSparseMoeBlock(config)
        self.input_layernorm = Qwen3_8MoeRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = Qwen3_8MoeRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, x):
        if self.block_type != "linear_attention":
            raise RuntimeError("the plain-residual layer is only defined for Gated DeltaNet blocks")
        x = x + self.linear_attn(self.input_layernorm(x))
        return x + self.mlp(self.post_attention_layernorm(x))


# --------------------------------------------------------------------------- mHC
def sinkhorn(logits, iters):
    P = torch.exp(logits - logits.amax(dim=(-2, -1), keepdim=True))
    for _ in range(iters):
        P = P / P.sum(-1, keepdim=True).clamp(min=1e-9)
        P = P / P.sum(-2, keepdim=True).clamp(min=1e-9)
    return P


class MHC(nn.Module):
    """Branch-residual coefficients of one sub-layer.

    ``pre``: ``Xf = rmsnorm(flatten(X))``, ``z = tanh(B A Xf)``; ``pre = sigmoid(b_pre + a0 z[:n])``,
    ``post = 2 sigmoid(b_post + a1 z[n:2n])``, ``res = sinkhorn(b_res + a2 z[2n:])``; returns
    ``sum_n pre_n X_n``.  ``post``: ``X'_m = sum_n res[m,n] X_n + post_m y``.  All in fp32.
    Initialisation makes the block an ordinary residual connection (B = 0, res ~ I, post = 1).
    """

    def __init__(self, h, n=4, r=None, slot=0, iters=20):
        super().__init__()
        self.n, self.iters = n, iters
        r = r or round(h / 8)
        self.A = nn.Linear(n * h, r, bias=False)
        self.B = nn.Linear(r, 2 * n + n * n, bias=False)
        nn.init.normal_(self.A.weight, std=0.02)
        nn.init.zeros_(self.B.weight)
        pre = torch.full((n,), 0.1)
        pre[slot % n] = 0.7
        self.b_pre = nn.Parameter(torch.log(pre / (1 - pre)))
        self.b_post = nn.Parameter(torch.zeros(n))
        self.b_res = nn.Parameter(torch.full((n, n), -8.0) + 8.0 * torch.eye(n))
        self.alphas = nn.Parameter(torch.full((3,), 0.1))

    def coefficients(self, X):
        n = self.n
        Xf = X.float().flatten(2)
        Xf = Xf * torch.rsqrt(Xf.pow(2).mean(-1, keepdim=True) + 1e-6)
        z = torch.tanh(F.linear(F.linear(Xf, self.A.weight.float()), self.B.weight.float()))
        a = self.alphas.float()
        pre = torch.sigmoid(self.b_pre.float() + a[0] * z[..., :n])
        post = 2 * torch.sigmoid(self.b_post.float() + a[1] * z[..., n:2 * n])
        res = sinkhorn(self.b_res.float() + a[2] * z[..., 2 * n:].reshape(*z.shape[:-1], n, n), self.iters)
        return pre, post, res

    def pre(self, X):
        pre, post, res = self.coefficients(X)
        return (pre.unsqueeze(-1) * X.float()).sum(2), (X, post, res)

    @staticmethod
    def post(y, state):
        X, post, res = state
        return torch.einsum("bsmn,bsnh->bsmh", res, X.float()) + post.unsqueeze(-1) * y.float().unsqueeze(2)


# --------------------------------------------------------------------------- n-gram hash embeddings
_P2 = (1000003, 998244353)
_P3 = (1000033, 998244353, 1000000007)
_MIX = 2654435761


class NGramEmbedding(nn.Module):
    """Hashed bigram + trigram embeddings, RMS-normalised and gated into the residual stream.

    The context never crosses an EOS: a predecessor that lies before the latest EOS (or before the
    sequence start) is replaced by the placeholder id ``vocab``.  Hashes use wrapping int64
    arithmetic with an arithmetic right shift; the row is the non-negative remainder."""

    def __init__(self, hidden, vocab, rows, eos_id, gate_bias=-1.0, init_std=0.02, norm_init=0.02):
        super().__init__()
        self.hidden, self.vocab, self.rows, self.eos_id = hidden, vocab, rows, eos_id
        self.emb2 = nn.Embedding(rows, hidden)
        self.emb3 = nn.Embedding(rows, hidden)
        nn.init.normal_(self.emb2.weight, std=init_std)
        nn.init.normal_(self.emb3.weight, std=init_std)
        self.norm = nn.RMSNorm(hidden, eps=1e-6)
        nn.init.constant_(self.norm.weight, norm_init)
        self.gate = nn.Linear(hidden, hidden, bias=True)
        nn.init.normal_(self.gate.weight, std=0.02)
        nn.init.constant_(self.gate.bias, gate_bias)
        self.collect, self.stat = False, {}

    def indices(self, ids):
        B, T = ids.shape
        ids = ids.long()
        pos = torch.arange(T, device=ids.device).expand(B, T)
        eos_id = -1 if self.eos_id is None else self.eos_id
        last = torch.where(ids == eos_id, pos, torch.full_like(pos, -1)).cummax(1).values.clamp(min=0)

        def back(k):
            shifted = F.pad(ids, (k, 0), value=self.vocab)[:, :T]
            return torch.where(pos - k >= last, shifted, torch.full_like(shifted, self.vocab))

        a, b, c = back(1), ids, back(2)
        h2 = (a * _P2[0]) ^ (b * _P2[1])
        h3 = (c * _P3[0]) ^ (a * _P3[1]) ^ (b * _P3[2])
        h2 = (h2 ^ (h2 >> 17)) * _MIX
        h3 = (h3 ^ (h3 >> 17)) * _MIX
        return h2 % self.rows, h3 % self.rows

    def delta(self, h, ids):
        """The increment ``sigmoid(W h + b) * rmsnorm(emb2[i2] + emb3[i3])`` to add to every branch."""
        fast = _hook("ngram_delta", h)
        if fast is not None and not self.collect:
            return fast(self, h, ids)
        i2, i3 = self.indices(ids)
        e = self.norm((self.emb2(i2) + self.emb3(i3)).float()).to(h.dtype)
        g = torch.sigmoid(_linear(h, self.gate.weight, self.gate.bias))
        if self.collect:
            with torch.no_grad():
                self.stat = dict(gate_mean=g.float().mean().item(), gate_frac_lt01=(g < 0.1).float().mean().item(),
                                 gate_frac_gt09=(g > 0.9).float().mean().item(),
                                 ratio=((g * e).float().norm() / h.float().norm().clamp(min=1e-9)).item())
        return g * e

    def forward(self, h, ids):
        return h + self.delta(h, ids)


# --------------------------------------------------------------------------- trunk
class Q38TextCore(nn.Module):
    """Embedding, decoder layers, final norm, mHC blocks, indexers and n-gram tables."""

    def _build(self, config):
        h, L = config.hidden_size, config.num_hidden_layers
        self.embed_tokens = nn.Embedding(config.vocab_size, h, config.pad_token_id)
        self.layers = nn.ModuleList([Qwen3_8MoeDecoderLayer(config, i) for i in range(L)])
        self.norm = Qwen3_8MoeRMSNorm(h, eps=config.rms_norm_eps)
        self.mhc = nn.ModuleList([MHC(h, config.n_branch, max(1, round(h / 8)), slot=i, iters=config.mhc_iters)
                                  for i in range(2 * L)])
        self.indexers = nn.ModuleDict({str(i): Indexer(h, config.indexer_heads, config.indexer_head_dim)
                                       for i, kind in enumerate(config.layer_types[:L]) if kind == "full_attention"})
        self.ngram = (NGramEmbedding(h, config.vocab_size, config.ngram_rows, config.eos_token_id)
                      if config.ngram_rows else None)
        self.gradient_checkpointing = False
        self.qsa_dense = False
        self.compute_dtype = None          # activation dtype of the sub-layers; None = dtype of the embedding

    def rope(self, length, device, dtype):
        rp = self.config.rope_parameters or {}
        factor = rp.get("partial_rotary_factor", getattr(self.config, "partial_rotary_factor", 0.25) or 0.25)
        pos = torch.arange(length, device=device)[None]
        return rope_tables(pos, int(self.config.head_dim * factor), rp.get("rope_theta", 1e7), dtype)

    def trunk(self, ids):
        """ids ``[B,S]`` -> (pre-final-norm hidden ``[B,S,h]``, list of per-QSA-layer KL terms)."""
        length = ids.shape[1]
        if not length:
            raise ValueError("Q38 requires at least one input token")
        if self.config.indexer_head_dim != self.config.head_dim:
            raise ValueError("Indexer and attention head dimensions must match for shared partial RoPE")
        if length % BLK:
            ids = F.pad(ids, (0, (-length) % BLK), value=self.config.pad_token_id or 0)
        e = _embed(self.embed_tokens, ids)
        dtype = self.compute_dtype or e.dtype
        cos, sin = self.rope(ids.shape[1], ids.device, e.dtype)
        X = e.float().unsqueeze(2).expand(-1, -1, self.config.n_branch, -1).contiguous()
        kls = []
        ckpt = self.gradient_checkpointing and self.training and torch.is_grad_enabled()
        for i in range(len(self.layers)):
            if ckpt:
                # the layers draw no random numbers, so the RNG state is not saved (reading it is not allowed during CUDA-graph capture)
                X, kl = torch.utils.checkpoint.checkpoint(self._layer, i, X, ids, cos, sin, dtype, use_reentrant=False, preserve_rng_state=False)
            else:
                X, kl = self._layer(i, X, ids, cos, sin, dtype)
            if kl is not None:
                kls.append(kl)
        return X.sum(2)[:, :length].to(e.dtype), kls

    def _sublayer_input(self, mhc, norm, X, dtype):
        fast = _hook("mhc_pre_norm", X)
        if fast is not None:
            return fast(mhc, norm, X, dtype)
        xin, state = mhc.pre(X)
        return norm(xin, out_dtype=dtype), state

    def _sublayer_output(self, mhc, y, state):
        fast = _hook("mhc_post", y)
        if fast is not None:
            return fast(mhc, y, state)
        return mhc.post(y, state)

    def _layer(self, i, X, ids, cos, sin, dtype):
        layer, kl = self.layers[i], None
        x, state = self._sublayer_input(self.mhc[2 * i], layer.input_layernorm, X, dtype)
        if layer.block_type == "linear_attention":
            y = layer.linear_attn(x)
        else:
            y, kl = qsa_attention(layer.self_attn, x, cos, sin, self.indexers[str(i)], self.config.qsa_blocks,
                                  self.training and self.qsa_dense, self.training and torch.is_grad_enabled())
        X = self._sublayer_output(self.mhc[2 * i], y, state)
        x, state = self._sublayer_input(self.mhc[2 * i + 1], layer.post_attention_layernorm, X, dtype)
        X = self._sublayer_output(self.mhc[2 * i + 1], layer.mlp(x), state)
        if i == 0 and self.ngram is not None:
            X = X + self.ngram.delta(X.mean(2).to(dtype), ids).float().unsqueeze(2)
        return X, kl


class _Output(dict):
    """Minimal attribute-style output record (``.logits``, ``.loss``, ``.last_hidden_state``)."""
    __getattr__ = dict.get


class Q38CausalCore(nn.Module):
    """``model`` (trunk) + tied ``lm_head`` + optional training-only ``mtp`` head."""

    def _build(self, config, text_model):
        h = config.hidden_size
        self.model = text_model
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(h, config.vocab_size, bias=False)
        self.mtp = None
        if config.mtp:
            self.mtp = nn.ModuleDict(dict(
                enorm=Qwen3_8MoeRMSNorm(h, eps=config.rms_norm_eps),
                hnorm=Qwen3_8MoeRMSNorm(h, eps=config.rms_norm_eps),
                proj=nn.Linear(2 * h, h, bias=False),
                block=Qwen3_8MoeDecoderLayer(config, config.num_hidden_layers, block_type="linear_attention"),
                norm=Qwen3_8MoeRMSNorm(h, eps=config.rms_norm_eps)))

    def tie_embeddings(self):
        self.lm_head.weight = self.model.embed_tokens.weight

    def moe_blocks(self):
        blocks = [layer.mlp for layer in self.model.layers]
        return blocks + ([self.mtp["block"].mlp] if self.mtp is not None else [])

    def mtp_hidden(self, hs, ids_next):
        """MTP trunk: ``proj([enorm(embed(next token)); hnorm(hidden)])`` -> one plain GDN+MoE layer -> norm."""
        m = self.mtp
        dtype = self.model.compute_dtype or hs.dtype
        z = torch.cat([m["enorm"](_embed(self.model.embed_tokens, ids_next), out_dtype=dtype), m["hnorm"](hs, out_dtype=dtype)], -1)
        return m["norm"](m["block"](_linear(z, m["proj"].weight)))

    def logits(self, input_ids):
        hs, _ = self.model.trunk(input_ids)
        dtype = self.model.compute_dtype or hs.dtype
        return _linear(self.model.norm(hs, out_dtype=dtype), self.lm_head.weight)

    def _causal_forward(self, input_ids=None, attention_mask=None, past_key_values=None, inputs_embeds=None,
                        labels=None, use_cache=False, **unused):
        if input_ids is None or inputs_embeds is not None:
            raise ValueError("Q38 packed prefill requires input_ids")
        if past_key_values is not None or use_cache or attention_mask is not None:
            raise ValueError("Q38 supports uncached packed prefill without attention_mask")
        logits = self.logits(input_ids)
        loss = None
        if labels is not None:
            shift = logits[:, :-1].float().reshape(-1, logits.shape[-1])
            loss = F.cross_entropy(shift, labels[:, 1:].reshape(-1), ignore_index=-100)
        return _Output(logits=logits, loss=loss)


def init_q38_weights(model, config, generator=None):
    """Random initialisation of the reference presets: N(0, 0.02) linears / embeddings / experts /
    routers (padding row zeroed), zero-centred norm weights 0, gated-norm weights 1, ``dt_bias = 1``,
    ``A_log = log U(0.01, 16)``.  mHC, indexer and n-gram modules keep their constructor init.
    (Reference: modeling_qwen3_8_moe.py:943-960, 1227-1230.)"""
    std = config.initializer_range
    own_init = (MHC, Indexer, NGramEmbedding)
    skip = {id(m) for top in model.modules() if isinstance(top, own_init) for m in top.modules()}
    with torch.no_grad():
        for module in model.modules():
            if id(module) in skip:
                continue
            if isinstance(module, (nn.Linear, nn.Conv1d)):
                module.weight.normal_(0.0, std, generator=generator)
                if module.bias is not None:
                    module.bias.zero_()
            elif isinstance(module, nn.Embedding):
                module.weight.normal_(0.0, std, generator=generator)
                if module.padding_idx is not None:
                    module.weight[module.padding_idx].zero_()
            elif isinstance(module, Qwen3_8MoeRMSNorm):
                module.weight.zero_()
            elif isinstance(module, Qwen3_8MoeRMSNormGated):
                module.weight.fill_(1.0)
            elif isinstance(module, Qwen3_8MoeExperts):
                module.gate_up_proj.normal_(0.0, std, generator=generator)
                module.down_proj.normal_(0.0, std, generator=generator)
            elif isinstance(module, Qwen3_8MoeTopKRouter):
                module.weight.normal_(0.0, std, generator=generator)
            elif isinstance(module, Qwen3_8MoeGatedDeltaNet):
                module.dt_bias.fill_(1.0)
                module.A_log.copy_(torch.empty_like(module.A_log).uniform_(0.01, 16, generator=generator).log_())


# --------------------------------------------------------------------------- plain nn.Module front ends
class Q38TextModel(Q38TextCore):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self._build(config)


class Q38ForCausalLM(Q38CausalCore):
    """Dependency-free model used by ``q38.train`` / ``q38.evaluate`` / the benchmark."""

    def __init__(self, config, init=True):
        super().__init__()
        self.config = config
        self._build(config, Q38TextModel(config))
        if init:
            init_q38_weights(self, config)
        self.tie_embeddings()

    def forward(self, input_ids=None, **kw):
        return self._causal_forward(input_ids=input_ids, **kw)

    def get_input_embeddings(self):
        return self.model.embed_tokens


# --------------------------------------------------------------------------- transformers front ends
try:
    from transformers.modeling_utils import PreTrainedModel
    from transformers.generation import GenerationMixin
    try:
        from .configuration_qwen3_8_moe import Qwen3_8MoeTextConfig
    except ImportError:                                   # flat layout inside an HF export directory
        from configuration_qwen3_8_moe import Qwen3_8MoeTextConfig
    _HAVE_TRANSFORMERS = True
except Exception:                                         # pragma: no cover - transformers is optional
    _HAVE_TRANSFORMERS = False

if _HAVE_TRANSFORMERS:
    class Qwen3_8MoePreTrainedModel(PreTrainedModel):
        config: Qwen3_8MoeTextConfig
        config_class = Qwen3_8MoeTextConfig
        base_model_prefix = "model"
        supports_gradient_checkpointing = True
        _no_split_modules = ["Qwen3_8MoeDecoderLayer"]
        _keys_to_ignore_on_load_unexpected = [r"^mtp.*"]

        def _init_weights(self, module):
            # Whole-model initialisation happens once in the constructors below; loading a checkpoint
            # overwrites it.  Per-module re-initialisation by the loader is a no-op.
            return

    class Qwen3_8MoeTextModel(Q38TextCore, Qwen3_8MoePreTrainedModel):
        def __init__(self, config):
            Qwen3_8MoePreTrainedModel.__init__(self, config)
            self._build(config)
            self.post_init()

        def forward(self, input_ids=None, attention_mask=None, past_key_values=None, inputs_embeds=None,
                    use_cache=False, **unused):
            if input_ids is None or inputs_embeds is not None:
                raise ValueError("Q38 packed prefill requires input_ids")
            if past_key_values is not None or use_cache or attention_mask is not None:
                raise ValueError("Q38 supports uncached packed prefill without attention_mask")
            hs, _ = self.trunk(input_ids)
            return _Output(last_hidden_state=self.norm(hs))

    class Qwen3_8MoeForCausalLM(Q38CausalCore, Qwen3_8MoePreTrainedModel, GenerationMixin):
        _tied_weights_keys = {"lm_head.weight": "model.embed_tokens.weight"}
        _keys_to_ignore_on_load_unexpected = [r"^mtp.*", r"^model.visual.*"]

        def __init__(self, config):
            Qwen3_8MoePreTrainedModel.__init__(self, config)
            self._build(config, Qwen3_8MoeTextModel(config))
            init_q38_weights(self, config)
            self.post_init()

        def get_input_embeddings(self):
            return self.model.embed_tokens

        def get_output_embeddings(self):
            return self.lm_head

        def forward(self, input_ids=None, **kw):
            kw.pop("return_dict", None)
            return self._causal_forward(input_ids=input_ids, **kw)

    __all__ = ["Qwen3_8MoeTextModel", "Qwen3_8MoeForCausalLM", "Qwen3_8MoePreTrainedModel", "Q38ForCausalLM"]
else:
    __all__ = ["Q38ForCausalLM"]

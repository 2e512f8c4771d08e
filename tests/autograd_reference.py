"""Native-torch model of one Ulysses attention block boundary for every rank of a context-parallel
group on ONE device: F.linear + index routes + autograd, the conformance reference the fused
operators are checked against (as benchmarks/sm90/backward/backward_torch_autograd.py of the
reference does: torch.nn.functional.linear forward, torch.autograd.grad, native route construction).

Every rank gets its own weight leaves, so the weight gradients stay per rank (the operators do no
cross-rank reduction)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def toy_attention(q, k, v, q_local_heads, kv_local_heads, head_dim):
    """A differentiable stand-in for attention on planar [rows, heads*d] tensors: per position and
    head, Q gated by its KV head's K, plus V.  Row-local, so it commutes with any row route."""
    rows = q.shape[0]
    group = q_local_heads // kv_local_heads
    ke = k.view(rows, kv_local_heads, 1, head_dim).expand(rows, kv_local_heads, group, head_dim)
    ve = v.view(rows, kv_local_heads, 1, head_dim).expand(rows, kv_local_heads, group, head_dim)
    qv = q.view(rows, kv_local_heads, group, head_dim)
    return (qv * torch.tanh(ke) + 0.5 * ve).reshape(rows, q_local_heads * head_dim)


def reference_world(xs, w_qkv, w_o, dys, *, cp, seq_local, q_heads, kv_heads, head_dim):
    """xs[r] [seq_local, hidden] and dys[r] [seq_local, hidden] of every rank (batch 1), shared
    weights.  Returns per rank a dict of y, q, k, v, dx, dw_qkv, dw_o (all BF16 math, FP32
    accumulation inside the matmuls, like the fused operators)."""
    ql, kvl = q_heads // cp, kv_heads // cp
    xs = [x.detach().clone().requires_grad_(True) for x in xs]
    wq = [w_qkv.detach().clone().requires_grad_(True) for _ in range(cp)]
    wo = [w_o.detach().clone().requires_grad_(True) for _ in range(cp)]
    ys = [F.linear(xs[r], wq[r]) for r in range(cp)]  # [seq_local, (q + 2 kv) d]
    k0, v0 = q_heads * head_dim, (q_heads + kv_heads) * head_dim
    qs, ks, vs, attn = [], [], [], []
    for d in range(cp):  # owner d holds its heads for every position, source ranks in row order
        qs.append(torch.cat([ys[r][:, d * ql * head_dim:(d + 1) * ql * head_dim] for r in range(cp)], dim=0))
        ks.append(torch.cat([ys[r][:, k0 + d * kvl * head_dim:k0 + (d + 1) * kvl * head_dim] for r in range(cp)], dim=0))
        vs.append(torch.cat([ys[r][:, v0 + d * kvl * head_dim:v0 + (d + 1) * kvl * head_dim] for r in range(cp)], dim=0))
        attn.append(toy_attention(qs[d], ks[d], vs[d], ql, kvl, head_dim))
    outs = []
    for r in range(cp):  # rank r gathers its rows of every owner's heads
        lhs = torch.cat([attn[p][r * seq_local:(r + 1) * seq_local] for p in range(cp)], dim=1)
        outs.append(F.linear(lhs, wo[r]))
    grads = torch.autograd.grad(outs, xs + wq + wo, grad_outputs=list(dys))
    return [dict(y=outs[r].detach(), q=qs[r].detach(), k=ks[r].detach(), v=vs[r].detach(),
                 dx=grads[r], dw_qkv=grads[cp + r], dw_o=grads[2 * cp + r]) for r in range(cp)]


def close(got, want, atol=0.02, rtol=0.02):
    """The reference's backward tolerance, |a - b| <= 0.02 + 0.02 |b| (backward/validation.cuh:71), on
    values scaled to the tensor's own magnitude so that sums over thousands of tokens compare alike."""
    got, want = got.detach().float(), want.detach().float()
    scale = want.abs().mean().clamp_min(1e-6)
    bad = ((got - want).abs() / scale > atol + rtol * want.abs() / scale)
    return int(bad.sum()), float(((got - want).abs() / scale).max())

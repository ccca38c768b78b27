"""Each op of the path written once more, in PyTorch, from its mathematical definition, with gradients from autograd.

These formulations deliberately share nothing with oracle/ref_chain.py (which restates the reference's thunk
chains primitive by primitive, with their rounding points): they are the textbook definitions in float64, so a
misreading of a reference formula that the oracle and the kernels share would show up against them.  Used on the CPU
against the oracle (tests/test_oracle_vs_torch.py) and on the GPU against the kernels
(tests/test_gpu_torch_crosscheck.py).  Inputs are torch tensors of any float dtype; everything is computed in float64.
"""
import torch
import torch.nn.functional as F


def _leaf(t):
    return t.detach().double().requires_grad_(True)


def rmsnorm(x, gamma, dy, eps):
    """y = gamma * x / sqrt(mean(x^2) + eps) over the last dimension; returns (y, dx, dgamma)."""
    x, gamma = _leaf(x), _leaf(gamma)
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gamma
    y.backward(dy.double())
    return y.detach(), x.grad, gamma.grad


def causal_softmax(scores, d_p, q_pos=None):
    """Row softmax where row r sees columns c <= q_pos[r] (all columns when q_pos is None); returns (P, dScores)."""
    s = _leaf(scores)
    if q_pos is None:
        masked = s
    else:
        cols = torch.arange(s.shape[-1], device=s.device)
        masked = s.masked_fill(cols[None, :] > q_pos[:, None], float("-inf"))
    p = torch.softmax(masked, dim=-1)
    p.backward(d_p.double())
    return p.detach(), s.grad


def cross_entropy(logits, targets, w):
    """loss_i = -log softmax(x_i)[k_i]; the adjoint of sum_i w * loss_i; returns (loss_rows, dlogits)."""
    x = _leaf(logits)
    loss = F.cross_entropy(x, targets.long(), reduction="none")
    (loss * w).sum().backward()
    return loss.detach(), x.grad


def swiglu(gate, up, dh):
    """h = silu(gate) * up; returns (h, dgate, dup)."""
    g, u = _leaf(gate), _leaf(up)
    h = F.silu(g) * u
    h.backward(dh.double())
    return h.detach(), g.grad, u.grad


def rope_angles(seq, head_dim, theta=10000.0, device="cpu"):
    """cos and sin tables [seq, head_dim] of rotary embedding in its rotate-half form: the angle of position p and
    feature i (and of its partner i + head_dim / 2) is p * theta^(-2 i / head_dim)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64, device=device)
    inv = theta ** (-2.0 * i / head_dim)
    ang = torch.arange(seq, dtype=torch.float64, device=device)[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return torch.cos(ang), torch.sin(ang)


def rope(x, dy, cos, sin, pos):
    """y = x * cos + rotate_half(x) * sin with rotate_half(x) = [-x2, x1]; x: [tokens, heads, head_dim], cos / sin:
    [positions, head_dim], pos: position index of every token; returns (y, dx)."""
    x = _leaf(x)
    c, s = cos.double()[pos][:, None, :], sin.double()[pos][:, None, :]
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    y = x * c + rot * s
    y.backward(dy.double())
    return y.detach(), x.grad


def causal_attention(q, k, v, d_ctx, alpha):
    """softmax(alpha q k^T, causal) v per (batch, head); q, k, v, d_ctx: [B, S, H, hd]; returns (ctx, dq, dk, dv)."""
    q, k, v = _leaf(q), _leaf(k), _leaf(v)
    ctx = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                         scale=alpha).transpose(1, 2)
    ctx.backward(d_ctx.double())
    return ctx.detach(), q.grad, k.grad, v.grad

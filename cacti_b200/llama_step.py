"""One OpenLLaMA-shaped training step (forward + backward) issued purely through the C ABI.

This is the workload of benchmark config 5: the op sequence of `Llama::apply` (src/librarium/llama.rs:420-548)
and of the adjoints the spine would stage for it (src/spine.rs:447-690), with each group of primitive thunks
replaced by its fused entry point.  It is host plumbing only: torch owns device memory and streams, every
arithmetic step is a `cacti_b200_*` call.  Differences from the reference graph, all stated:
  * the f32 probability tensor `out_lm_prob` and the arg-max (llama.rs:543,546) are not produced;
  * attention probabilities are recomputed from the saved scores in the backward instead of being kept
    (the fused softmax forward+backward entry point yields them together with dS; 2.1 GB less live memory per
    layer at B = 8);
  * each residual add (llama.rs:514,533) runs inside the RMSNorm that follows it (same bits, one pass less);
  * the diagnostics thunks the example runs on every tensor (examples/open_llama_3b_train.rs:412-425) are omitted;
  * the six block matmuls of a layer carry the causal structure as a hint: score / dP tiles above the diagonal are
    not computed (the masked softmax never reads them) and products with the exact zeros of P and dS are skipped;
    every value that is used is bit-identical to the full product.  The softmax zero-fills the masked tails of P
    and dS only as far as those matmuls read (CACTI_B200_MASK_CAUSAL_TRIM).
  * by default attention runs fused (cacti_b200_attention_fwd / _bwd_prep): scores and probabilities stay on chip in
    the forward, and the backward rebuilds P and dS per tile instead of reading stored scores, materialises them once
    and multiplies them with the three hinted block matmuls.  `attention="fused-bwd"` keeps P and dS on chip in the
    backward too (cacti_b200_attention_bwd: measured slower, 2.10 ms against 1.42 ms per layer at 8 sequences, because
    the exponentials, which bound these kernels, are then evaluated once for dQ and once for dK / dV);
    `attention="unfused"` keeps the reference's op sequence.
Layout: activations [T, D] = [B, S, H, hd]; scores [B, S, H, S] as in the reference.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from . import ops
from .capi import TRI_A_LOWER, TRI_A_UPPER, TRI_C_LOWER, lib


@dataclass
class LlamaShape:
    layers: int = 26
    d_model: int = 3200
    heads: int = 32
    head_dim: int = 100
    ffn: int = 8640
    vocab: int = 32000
    seq: int = 2048
    eps: float = 1e-6
    theta: float = 10000.0

    @staticmethod
    def open_llama_3b():
        """LlamaConfig::open_llama_3b, src/librarium/llama.rs:88-105."""
        return LlamaShape()


def init_weights(cfg: LlamaShape, device, seed=0, std=0.02, dtype=torch.float16):
    """Random-init weights ~ N(0, std^2); norm gains are 1 (a gain ~N(0, 0.02^2) would scale every residual
    branch by 0.02 and make the step degenerate)."""
    g = torch.Generator(device=device).manual_seed(seed)

    def w(*shape):
        return (torch.randn(*shape, device=device, generator=g) * std).to(dtype)

    D, F, V = cfg.d_model, cfg.ffn, cfg.vocab
    P = {"embed": w(V, D), "lm_head": w(V, D), "head_norm": torch.ones(D, device=device, dtype=dtype), "layers": []}
    for _ in range(cfg.layers):
        L = {"pre_norm": torch.ones(D, device=device, dtype=dtype), "q": w(D, D), "k": w(D, D),
             "v": w(D, D), "o": w(D, D), "post_norm": torch.ones(D, device=device, dtype=dtype),
             "up": w(F, D), "gate": w(F, D), "down": w(D, F)}
        # one flat buffer per layer, laid out like the gradient buckets of dp.alloc_bucketed_grads: q, k and v are
        # then adjacent, which lets the step run their three projections as one batched matmul
        flat = torch.empty(sum((t.numel() + 127) // 128 * 128 for t in L.values()), dtype=dtype, device=device)
        off = 0
        for name, t in L.items():
            L[name] = flat[off:off + t.numel()].view(t.shape).copy_(t)
            off += (t.numel() + 127) // 128 * 128
        P["layers"].append(L)
    return P


def stacked(*ts):
    """[n, rows, 1, cols] view over n equal 2-d tensors that lie back to back in memory (None when they do not): the
    4-d block layout of the batched matmul, one block row per tensor."""
    t0 = ts[0]
    if os.environ.get("CACTI_B200_NO_STACK") == "1":         # A/B switch: always the separate launches
        return None
    if any(t.shape != t0.shape or t.dtype != t0.dtype or not t.is_contiguous() or
           t.untyped_storage().data_ptr() != t0.untyped_storage().data_ptr() for t in ts):
        return None                                          # (neighbours by accident of the allocator do not count)
    step = t0.numel() * t0.element_size()
    if any(t.data_ptr() != t0.data_ptr() + i * step for i, t in enumerate(ts)):
        return None
    return torch.as_strided(t0, (len(ts), t0.shape[0], 1, t0.shape[1]), (t0.numel(), t0.shape[1], t0.shape[1], 1))


def zeros_like_params(P):
    out = {k: torch.zeros_like(v) for k, v in P.items() if k != "layers"}
    out["layers"] = [{k: torch.zeros_like(v) for k, v in L.items()} for L in P["layers"]]
    return out


def flat_params(P):
    """(name, tensor) pairs in a fixed order (used for gradient bucketing)."""
    out = [("embed", P["embed"]), ("lm_head", P["lm_head"]), ("head_norm", P["head_norm"])]
    for i, L in enumerate(P["layers"]):
        out += [(f"layers.{i}.{k}", v) for k, v in L.items()]
    return out


class TrainStep:
    """Forward + backward over `batch` sequences of cfg.seq tokens.  Gradients are written (Apply mode) into
    `grads`, a structure shaped like the parameters; `on_layer_done(i)` is called after layer i's weight
    gradients are complete, and with i = cfg.layers as soon as the output head's gradients are (the hook a
    data-parallel reducer attaches to; the embedding gradient is complete when the call returns)."""

    def __init__(self, cfg: LlamaShape, params, batch: int, loss_tokens: int | None = None, attention: str = "auto"):
        self.cfg, self.P, self.B = cfg, params, batch
        # "fused": attention_fwd / attention_bwd_prep (scores never reach HBM); "unfused": the reference's op sequence,
        # block matmul - softmax - block matmul; "auto": fused when the shape allows it
        can_fuse = cfg.seq % 128 == 0 and cfg.head_dim <= 128 and cfg.head_dim % 4 == 0
        if attention not in ("auto", "fused", "fused-bwd", "unfused"):
            raise ValueError(f"attention={attention!r}")
        if attention in ("fused", "fused-bwd") and not can_fuse:
            raise ValueError("fused attention needs seq % 128 == 0, head_dim <= 128 and head_dim % 4 == 0")
        self.fused = can_fuse if attention == "auto" else attention in ("fused", "fused-bwd")
        self.fused_bwd = attention == "fused-bwd"       # the backward keeps P and dS on chip as well
        dev = params["embed"].device
        self.dev = dev
        self.T = batch * cfg.seq
        self.loss_tokens = loss_tokens or self.T           # global token count: the loss is a mean over all ranks
        self.cos, self.sin = ops.rope_tables(cfg.seq, cfg.head_dim, cfg.theta, params["embed"].dtype, dev)
        L = lib()
        S, hd, H = cfg.seq, cfg.head_dim, cfg.heads
        nb = max(L.cacti_b200_gemm_workspace_bytes(S, S, hd, batch, H), L.cacti_b200_gemm_workspace_bytes(S, hd, S, batch, H),
                 L.cacti_b200_gemm_workspace_bytes(hd, S, S, batch, H))
        self.gemm_ws = torch.empty(nb, dtype=torch.uint8, device=dev)
        # dense matmuls: partial sums of the k-split schedule (all operands here are TMA-addressable, nothing is repacked)
        self.mm_ws = ops.gemm_workspace(0, 0, 0, dev)
        self.norm_ws = ops.rmsnorm_workspace(self.T, cfg.d_model, dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.launches = 0

    # -- small helpers (each is exactly one or two C-ABI calls) -----------------------------------------
    def _mm(self, a, b, ta, tb, c=None, beta=0.0):
        self.launches += 1
        return ops.gemm(a, b, ta, tb, beta=beta, c=c, workspace=self.mm_ws)

    def _bmm(self, a, b, ta, tb, alpha=1.0, tri=0, b_valid=None, c=None):
        self.launches += 3 if b_valid is None else 1       # unaligned operands are repacked first; padded ones are not
        return ops.block_gemm(a, b, ta, tb, alpha=alpha, workspace=self.gemm_ws, tri=tri, b_valid=b_valid, c=c)

    def _mm_stack(self, a, b, ta, tb, c):
        """One batched launch for matmuls that share an operand (given as a 2-d tensor, broadcast) and whose other operand
        and result are `stacked` views.  Same tiles and the same k order as the separate launches, hence the same bits;
        what changes is the tile count of the launch: 3 x 169 tiles of 256 x 256 fill 74 SM pairs for 6.85 waves, where
        169 alone fill 2.28 (the third wave a quarter full)."""
        self.launches += 1
        a4 = a if a.dim() == 4 else a.view(1, a.shape[0], 1, a.shape[1])
        b4 = b if b.dim() == 4 else b.view(1, b.shape[0], 1, b.shape[1])
        return ops.block_gemm(a4, b4, ta, tb, workspace=self.gemm_ws, c=c)

    def forward_backward(self, tokens, targets, grads, on_layer_done=None):
        cfg, P, B, T = self.cfg, self.P, self.B, self.T
        S, H, hd, D = cfg.seq, cfg.heads, cfg.head_dim, cfg.d_model
        alpha = 1.0 / math.sqrt(hd)
        # scores [B, S, H, S]: q_pos = (row / H) % S; P and dS feed only hinted block matmuls, so their masked
        # tails are zero-filled just as far as those can read
        mask = (H, S, 0, True)
        self.launches = 0
        x, _ = ops.gather_rows(P["embed"], tokens, status=self.status)
        self.launches += 1
        saved = []
        branch = None                                     # output of the previous MLP, not yet added to the stream
        for Lw in P["layers"]:
            # each residual add is fused into the norm that follows it (one pass instead of two over [T, D])
            if branch is None:
                n1 = ops.rmsnorm_fwd(x, Lw["pre_norm"], cfg.eps)
            else:
                n1, x = ops.add_rmsnorm_fwd(x, branch, Lw["pre_norm"], cfg.eps)
            w_qkv = stacked(Lw["q"], Lw["k"], Lw["v"])
            if w_qkv is not None:                         # the three projections of n1 as one batched matmul
                qkv = torch.empty(3, T, D, dtype=n1.dtype, device=n1.device)
                self._mm_stack(n1, w_qkv, False, True, qkv.view(3, T, 1, D))
                q_lin, k_lin, v_lin = qkv[0], qkv[1], qkv[2]
            else:
                q_lin, k_lin, v_lin = (self._mm(n1, Lw[name], False, True) for name in ("q", "k", "v"))
            if self.fused:
                # q, k, v with the head dimension zero-padded to 128 (RoPE writes q and k that way directly); the
                # padded copies also serve the backward pass
                q = ops.rope_fwd_pitched(q_lin.view(T, H, hd), self.cos, self.sin, 128).view(B, S, H, 128)
                k = ops.rope_fwd_pitched(k_lin.view(T, H, hd), self.cos, self.sin, 128).view(B, S, H, 128)
                v = ops.block_pad(v_lin.view(B, S, H, hd), 128)
                ctx, sc = ops.attention_fwd(q, k, v, hd, alpha)               # sc: the row statistics (m, l)
                ctx = ctx.view(T, D)
                self.launches += 2
            else:
                q = ops.rope_fwd(q_lin.view(T, H, hd), self.cos, self.sin)
                k = ops.rope_fwd(k_lin.view(T, H, hd), self.cos, self.sin)
                v = v_lin
                sc = self._bmm(q.view(B, S, H, hd), k.view(B, S, H, hd), False, True, alpha, TRI_C_LOWER)   # [B,S,H,S]
                p = ops.softmax_fwd(sc.view(B * S * H, S), mask)
                ctx = self._bmm(p.view(B, S, H, S), v.view(B, S, H, hd), False, False, tri=TRI_A_LOWER).view(T, D)
                del p
                self.launches += 1
            n2, x_mid = ops.add_rmsnorm_fwd(x, self._mm(ctx, Lw["o"], False, True), Lw["post_norm"], cfg.eps)
            up = self._mm(n2, Lw["up"], False, True)
            gate = self._mm(n2, Lw["gate"], False, True)
            h = ops.swiglu_fwd(gate, up)
            branch = self._mm(h, Lw["down"], False, True)
            self.launches += 5
            saved.append((x, n1, q, k, v, sc, ctx, x_mid, n2, up, gate, h))
            x = x_mid
        nf, x = ops.add_rmsnorm_fwd(x, branch, P["head_norm"], cfg.eps)
        del branch
        logits = self._mm(nf, P["lm_head"], False, True)
        loss, _, dlogits, _ = ops.softmax_nll_fwd_bwd(logits, targets, w_scalar=1.0 / self.loss_tokens, want_rows=False,
                                                       status=self.status)
        self.launches += 3
        del logits
        # ---------------------------------------------------------------- backward
        self._mm(dlogits, nf, True, False, c=grads["lm_head"])
        dnf = self._mm(dlogits, P["lm_head"], False, False)
        del dlogits
        dx, _ = ops.rmsnorm_bwd(x, P["head_norm"], dnf, cfg.eps, dgamma=grads["head_norm"], workspace=self.norm_ws)
        self.launches += 2
        if on_layer_done is not None:
            on_layer_done(cfg.layers)
        for li in range(cfg.layers - 1, -1, -1):
            Lw, G = P["layers"][li], grads["layers"][li]
            x_in, n1, q, k, v, sc, ctx, x_mid, n2, up, gate, h = saved.pop()
            # MLP branch: x_out = x_mid + h Wdown^T
            self._mm(dx, h, True, False, c=G["down"])
            dh = self._mm(dx, Lw["down"], False, False)
            dgate, dup = ops.swiglu_bwd(gate, up, dh)
            del dh, h
            self._mm(dup, n2, True, False, c=G["up"])
            self._mm(dgate, n2, True, False, c=G["gate"])
            dn2 = self._mm(dup, Lw["up"], False, False)
            self._mm(dgate, Lw["gate"], False, False, c=dn2, beta=1.0)
            del dgate, dup, up, gate
            ops.rmsnorm_bwd(x_mid, Lw["post_norm"], dn2, cfg.eps, dx=dx, dgamma=G["post_norm"], beta_dx=1,
                            workspace=self.norm_ws)                                  # dx += adjoint through the norm
            del dn2
            # attention branch: x_mid = x_in + ctx Wo^T
            self._mm(dx, ctx, True, False, c=G["o"])
            dctx = self._mm(dx, Lw["o"], False, False)
            # dq, dk and dv are written into one [3, T, D] buffer when the q, k, v gradients lie back to back, so that
            # the three weight-gradient matmuls below can run as one batched launch
            g_qkv = stacked(G["q"], G["k"], G["v"])
            dqkv = torch.empty(3, T, D, dtype=dx.dtype, device=dx.device) if g_qkv is not None else None
            dv_out = dqkv[2].view(B, S, H, hd) if dqkv is not None else None
            if self.fused_bwd:
                # dq, dk, dv straight from q, k, v (the padded copies), dctx and the row statistics
                dctx = ops.block_pad(dctx.view(B, S, H, hd), 128)
                dq, dk, dv = ops.attention_bwd(q, k, v, dctx, ctx.view(B, S, H, hd), sc, alpha, dv=dv_out)
                dq, dk, dv = dq.view(T, H, hd), dk.view(T, H, hd), dv.view(T, D)
                del dctx, sc
                self.launches += 4
            elif self.fused:
                # P and dS are rebuilt from q, k, v, dctx and the row statistics; q, k, v here are the padded copies
                dctx = ops.block_pad(dctx.view(B, S, H, hd), 128)
                p, ds = ops.attention_bwd_prep(q, k, v, dctx, ctx.view(B, S, H, hd), sc, alpha)
                self.launches += 3
                bv = hd
            else:
                dp = self._bmm(dctx.view(B, S, H, hd), v.view(B, S, H, hd), False, True, tri=TRI_C_LOWER)  # dctx V^T
                # one fused pass over (S, dP) yields the recomputed probabilities and dS together
                p, ds = ops.softmax_fwd_bwd(sc.view(B * S * H, S), dp.view(B * S * H, S), mask)
                del dp
                self.launches += 1
                dctx, q, k, bv = dctx.view(B, S, H, hd), q.view(B, S, H, hd), k.view(B, S, H, hd), None
            if not self.fused_bwd:
                del sc
                dv = self._bmm(p.view(B, S, H, S), dctx, True, False, tri=TRI_A_UPPER, b_valid=bv, c=dv_out).view(T, D)   # P^T dctx
                del p, dctx
                dq = self._bmm(ds.view(B, S, H, S), k, False, False, alpha, TRI_A_LOWER, b_valid=bv)               # dS K
                dk = self._bmm(ds.view(B, S, H, S), q, True, False, alpha, TRI_A_UPPER, b_valid=bv)                # dS^T Q
                del ds
            if dqkv is not None:
                dq = ops.rope_bwd(dq.view(T, H, hd), self.cos, self.sin, dx=dqkv[0].view(T, H, hd)).view(T, D)
                dk = ops.rope_bwd(dk.view(T, H, hd), self.cos, self.sin, dx=dqkv[1].view(T, H, hd)).view(T, D)
                self._mm_stack(dqkv.view(3, T, 1, D), n1, True, False, g_qkv)
            else:
                dq = ops.rope_bwd(dq.view(T, H, hd), self.cos, self.sin).view(T, D)
                dk = ops.rope_bwd(dk.view(T, H, hd), self.cos, self.sin).view(T, D)
                self._mm(dq, n1, True, False, c=G["q"])
                self._mm(dk, n1, True, False, c=G["k"])
                self._mm(dv, n1, True, False, c=G["v"])
            dn1 = self._mm(dq, Lw["q"], False, False)
            self._mm(dk, Lw["k"], False, False, c=dn1, beta=1.0)
            self._mm(dv, Lw["v"], False, False, c=dn1, beta=1.0)
            del dq, dk, dv
            ops.rmsnorm_bwd(x_in, Lw["pre_norm"], dn1, cfg.eps, dx=dx, dgamma=G["pre_norm"], beta_dx=1,
                            workspace=self.norm_ws)
            del dn1
            self.launches += 10
            if on_layer_done is not None:
                on_layer_done(li)
        ops.scatter_add_rows(dx, tokens, cfg.vocab, dtable=grads["embed"], status=self.status)
        self.launches += 5
        return loss


class GraphedStep:
    """One training step captured in a CUDA graph and replayed: the step is about 1200 kernel launches, and at one
    sequence per GPU (eight-GPU strong scaling) the gaps between them were 6 % of the step.  `body()` is called once
    under capture and must launch the whole step on the current stream (token copy from pinned memory, forward_backward,
    the gradient reduction hooks); whatever it returns is kept as `result` (tensors there are rewritten by every
    replay).  Capture needs a few eager calls first (kernel attributes, occupancy caches and the NCCL communicator are
    set up on first use), which `warmup` does.  The reference has no counterpart: it synchronises around every thunk
    (src/thunk/mod.rs:3478-3536)."""

    def __init__(self, body, warmup: int = 2):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        # the capture allocates the step's activations again, in the graph's own pool: hand the warm-up's cached blocks
        # back first, or both copies stay reserved (2 x 63 GiB at 8 sequences per GPU)
        torch.cuda.empty_cache()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.result = body()

    def replay(self):
        self.graph.replay()
        return self.result

"""CPU oracle for one training step: the composition of Llama::apply (src/librarium/llama.rs:420-548) and its
adjoints out of the per-op restatements in oracle/ref_chain.py.  Test infrastructure only; parity unpinned
(see ref_chain.py).  Every thunk output is rounded to f16, as the reference's f16 cells are."""
import math

import numpy as np

from . import ref_chain as R


def step(P, tokens, targets, cfg, loss_tokens=None):
    """P: dict of numpy f16 weights shaped like cacti_b200.llama_step.init_weights.  Returns (loss, grads)."""
    B = tokens.size // cfg.seq
    S, H, hd, D, T = cfg.seq, cfg.heads, cfg.head_dim, cfg.d_model, tokens.size
    alpha = 1.0 / math.sqrt(hd)
    cos, sin = R.ref_rope_tables(S, hd, cfg.theta, np.float16)
    pos = np.arange(T) % S
    keep = R.causal_keep_mask(B * S * H, S, H, S, 0)
    mm = lambda a, b, ta, tb: R.ref_gemm(a, b, ta, tb)
    x = R.ref_gather_rows(P["embed"], tokens)
    saved = []
    for L in P["layers"]:
        n1 = R.ref_rmsnorm_fwd(x, L["pre_norm"], cfg.eps)[0]
        q = R.ref_rope_fwd(mm(n1, L["q"], False, True).reshape(T, H, hd), cos, sin, pos)
        k = R.ref_rope_fwd(mm(n1, L["k"], False, True).reshape(T, H, hd), cos, sin, pos)
        v = mm(n1, L["v"], False, True)
        sc = R.ref_block_gemm(q.reshape(B, S, H, hd), k.reshape(B, S, H, hd), False, True, alpha)
        p = R.ref_softmax_fwd(sc.reshape(B * S * H, S), keep)[0]
        ctx = R.ref_block_gemm(p.reshape(B, S, H, S), v.reshape(B, S, H, hd)).reshape(T, D)
        x_mid = x + mm(ctx, L["o"], False, True)
        n2 = R.ref_rmsnorm_fwd(x_mid, L["post_norm"], cfg.eps)[0]
        up, gate = mm(n2, L["up"], False, True), mm(n2, L["gate"], False, True)
        h = R.ref_swiglu_fwd(gate, up)[0]
        x_out = x_mid + mm(h, L["down"], False, True)
        saved.append((x, n1, q, k, v, sc, p, ctx, x_mid, n2, up, gate, h))
        x = x_out
    nf = R.ref_rmsnorm_fwd(x, P["head_norm"], cfg.eps)[0]
    logits = mm(nf, P["lm_head"], False, True)
    w = np.float32(1.0 / (loss_tokens or T))
    loss_rows, dlogits, _ = R.ref_softmax_nll(logits, targets, w)
    loss = np.float32((loss_rows * w).sum(dtype=np.float32))
    G = {"layers": [None] * len(P["layers"])}
    G["lm_head"] = mm(dlogits, nf, True, False)
    dnf = mm(dlogits, P["lm_head"], False, False)
    dx, G["head_norm"] = R.ref_rmsnorm_bwd(x, P["head_norm"], dnf, cfg.eps)
    for li in range(len(P["layers"]) - 1, -1, -1):
        L = P["layers"][li]
        x_in, n1, q, k, v, sc, p, ctx, x_mid, n2, up, gate, h = saved.pop()
        g = {}
        g["down"] = mm(dx, h, True, False)
        dh = mm(dx, L["down"], False, False)
        dgate, dup = R.ref_swiglu_bwd(gate, up, dh)
        g["up"], g["gate"] = mm(dup, n2, True, False), mm(dgate, n2, True, False)
        dn2 = R.ref_gemm(dgate, L["gate"], False, False, beta=1.0, c=mm(dup, L["up"], False, False))
        d2, g["post_norm"] = R.ref_rmsnorm_bwd(x_mid, L["post_norm"], dn2, cfg.eps)
        dx = dx + d2
        g["o"] = mm(dx, ctx, True, False)
        dctx = mm(dx, L["o"], False, False)
        dv = R.ref_block_gemm(p.reshape(B, S, H, S), dctx.reshape(B, S, H, hd), True, False).reshape(T, D)
        dp = R.ref_block_gemm(dctx.reshape(B, S, H, hd), v.reshape(B, S, H, hd), False, True)
        ds = R.ref_softmax_bwd(sc.reshape(B * S * H, S), dp.reshape(B * S * H, S), keep)
        dq = R.ref_block_gemm(ds.reshape(B, S, H, S), k.reshape(B, S, H, hd), False, False, alpha)
        dk = R.ref_block_gemm(ds.reshape(B, S, H, S), q.reshape(B, S, H, hd), True, False, alpha)
        dq = R.ref_rope_bwd(dq.reshape(T, H, hd), cos, sin, pos).reshape(T, D)
        dk = R.ref_rope_bwd(dk.reshape(T, H, hd), cos, sin, pos).reshape(T, D)
        g["q"], g["k"], g["v"] = mm(dq, n1, True, False), mm(dk, n1, True, False), mm(dv, n1, True, False)
        dn1 = mm(dq, L["q"], False, False)
        dn1 = R.ref_gemm(dk, L["k"], False, False, beta=1.0, c=dn1)
        dn1 = R.ref_gemm(dv, L["v"], False, False, beta=1.0, c=dn1)
        d1, g["pre_norm"] = R.ref_rmsnorm_bwd(x_in, L["pre_norm"], dn1, cfg.eps)
        dx = dx + d1
        G["layers"][li] = g
    G["embed"] = R.ref_scatter_add_rows(dx, tokens, P["embed"].shape[0])
    return loss, G

"""Tensor-core workloads for cacti_b200.profile_cases: dense projection shapes, the two attention block matmuls and the
fused attention kernels (attn_fwd, attn_bwd)."""
import torch

from . import ops


def make(case, rnd, batch=2):
    if case.startswith("gemm_"):
        m, n, k = 4096, 3200, 3200
        if case == "gemm_nt":          # y = x W^T (forward projection)
            a, b = rnd(m, k), rnd(n, k, scale=0.02)
            c = torch.empty(m, n, dtype=torch.float16, device="cuda")
            return lambda: ops.gemm(a, b, False, True, c=c)
        if case == "gemm_nn":          # dx = dy W
            a, b = rnd(m, n), rnd(n, k, scale=0.02)
            c = torch.empty(m, k, dtype=torch.float16, device="cuda")
            return lambda: ops.gemm(a, b, False, False, c=c)
        if case == "gemm_tn":          # dW = dy^T x
            a, b = rnd(m, n), rnd(m, k)
            c = torch.empty(n, k, dtype=torch.float16, device="cuda")
            return lambda: ops.gemm(a, b, True, False, c=c)
    bsz, s, h, hd = batch, 2048, 32, 100
    if case == "qk":
        q, kk = rnd(bsz, s, h, hd), rnd(bsz, s, h, hd)
        c = torch.empty(bsz, s, h, s, dtype=torch.float16, device="cuda")
        ws = torch.empty(ops.lib().cacti_b200_gemm_workspace_bytes(s, s, hd, bsz, h), dtype=torch.uint8, device="cuda")
        return lambda: ops.block_gemm(q, kk, False, True, alpha=0.1, c=c, workspace=ws)
    if case == "pv":
        pr, v = rnd(bsz, s, h, s, scale=0.02), rnd(bsz, s, h, hd)
        c = torch.empty(bsz, s, h, hd, dtype=torch.float16, device="cuda")
        ws = torch.empty(ops.lib().cacti_b200_gemm_workspace_bytes(s, hd, s, bsz, h), dtype=torch.uint8, device="cuda")
        return lambda: ops.block_gemm(pr, v, False, False, c=c, workspace=ws)
    if case in ("attn_fwd", "attn_bwd"):
        alpha = hd ** -0.5
        q, kk, v, do = (ops.block_pad(rnd(bsz, s, h, hd), 128) for _ in range(4))
        ctx, st = ops.attention_fwd(q, kk, v, hd, alpha)
        if case == "attn_fwd":
            return lambda: ops.attention_fwd(q, kk, v, hd, alpha, ctx=ctx, stats=st)
        pp = torch.empty(bsz, s, h, s, dtype=torch.float16, device="cuda")
        ds = torch.empty_like(pp)
        return lambda: ops.attention_bwd_prep(q, kk, v, do, ctx, st, alpha, p=pp, ds=ds)
    raise SystemExit(f"unknown gemm case {case}")

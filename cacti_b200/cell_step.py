"""The OpenLLaMA-shaped training step of benchmark config 5 run the way the reference runs it: every tensor is a cell
of one arena under the soft-OOM policy, every op a thunk (Apply / Accumulate / Initialize) that looks its cells up,
pins them, launches and unpins.

`llama_step.TrainStep` issues the same C-ABI calls over torch-owned memory; this driver issues them through the C++
host shim (cacti_b200/host/): parameters, gradients, activations, workspaces and the status word are cells of a
`binding.Ctx`, whose arena has the reference's front / back cursors and whose allocation path is the reference's retry
loop (src/pctx/mod.rs:342-402): when a request does not fit under the soft limit (CACTI_VMEM_SOFT_LIMIT,
src/pctx/nvgpu.rs:1438-1463) resident cells are spilled to page-locked host memory, oldest first
(_try_soft_oom, src/pctx/nvgpu.rs:2004-2283), and a spilled cell is copied back when a thunk next reads it.  Saved
activations of the forward pass are what ends up on the host; the backward pass brings them back layer by layer.
Nothing here synchronises except the final read-back of the loss, and the results are bit-identical to the step
over torch memory: the kernels, their arguments and their order are the same, only the addresses differ.

The op sequence is `Llama::apply` (src/librarium/llama.rs:420-548) and the adjoints the spine stages for it
(src/spine.rs:447-690), with the fused entry points of llama_step.TrainStep(attention="fused").  Cells that are no
longer needed are freed at once (the reference's reset sweep, src/ctx.rs:150-235, does it per cycle).
"""
from __future__ import annotations

import math

import numpy as np

from .capi import R_16F, R_32F, R_32I, TRI_A_LOWER, TRI_A_UPPER, OPERAND_B_PADDED
from .host import binding as H

APPLY, ACC, INIT = H.APPLY, H.ACCUMULATE, H.INITIALIZE


class ThunkError(RuntimeError):
    pass


class CellTrainStep:
    """weights: {"embed", "lm_head", "head_norm", "layers": [{...}]} of numpy float16 arrays (llama_step.init_weights
    moved to the host).  Parameters and gradients are stable cells (they survive the step; spilled rather than dropped),
    everything else lives for part of one step."""

    def __init__(self, ctx: H.Ctx, cfg, weights, batch: int, loss_tokens: int | None = None, fused_bwd: bool = False):
        self.ctx, self.L, self.h, self.cfg, self.B = ctx, ctx.L, ctx.h, cfg, batch
        # False (llama_step's default): P and dS are cells, three block-matmul thunks; True: one attention_bwd thunk
        self.fused_bwd = fused_bwd
        self.T = batch * cfg.seq
        self.loss_tokens = loss_tokens or self.T
        assert cfg.seq % 128 == 0 and cfg.head_dim <= 128 and cfg.head_dim % 4 == 0, "the fused attention path needs these"
        self.shapes = {}

        def put(a):
            return ctx.cell(np.ascontiguousarray(a), stable=True)

        def named(prefix, d):
            out = {}
            for k, v in d.items():
                out[k] = put(v)
                self.shapes[f"{prefix}{k}"] = v.shape
            return out

        self.W = named("", {k: v for k, v in weights.items() if k != "layers"})
        self.W["layers"] = [named(f"layers.{i}.", Lw) for i, Lw in enumerate(weights["layers"])]
        self.G = {k: ctx.cell(nbytes=weights[k].nbytes, stable=True) for k in weights if k != "layers"}
        self.G["layers"] = [{k: ctx.cell(nbytes=v.nbytes, stable=True) for k, v in Lw.items()} for Lw in weights["layers"]]
        # RoPE tables (init_constants, src/librarium/llama.rs:389-411) come from the kernel library itself
        self.cos, self.sin = self._rope_tables()
        self.status = ctx.cell(np.zeros(1, np.uint32), stable=True)
        self.launches = 0

    # ---- helpers --------------------------------------------------------------------------------------------
    def _rope_tables(self):
        from . import capi
        cfg, ctx = self.cfg, self.ctx
        n = cfg.seq * cfg.head_dim * 2
        cos, sin = ctx.cell(nbytes=n, stable=True), ctx.cell(nbytes=n, stable=True)
        pc, ps = self.L.cbh_pwrite(self.h, cos), self.L.cbh_pwrite(self.h, sin)
        if not pc or not ps:
            raise ThunkError("hard OOM while placing the RoPE tables")
        capi.check(capi.lib().cacti_b200_rope_tables(pc, ps, cfg.seq, cfg.head_dim, cfg.theta, R_16F, self.L.cbh_stream(self.h)),
                   "rope_tables")
        return cos, sin

    def new(self, *shape, esize=2):
        return self.ctx.cell(nbytes=int(np.prod(shape)) * esize)

    def free(self, *cells):
        for c in cells:
            self.ctx.free(c)

    def call(self, name, *args):
        rc = getattr(self.L, "cbh_thunk_" + name)(self.h, *args)
        self.launches += 1
        if rc == -1:
            raise ThunkError(f"{name}: hard OOM (every resident cell is pinned or the request exceeds the soft limit)")
        if rc:
            raise ThunkError(f"{name}: error {rc}")

    def mm(self, a, b, m, n, k, ta, tb, out=None, mode=APPLY):
        out = self.new(m, n) if out is None else out
        self.call("matmul", mode, out, a, b, m, n, k, int(ta), int(tb), 1.0, R_16F)
        return out

    # ---- the step -------------------------------------------------------------------------------------------
    def forward_backward(self, tokens: np.ndarray, targets: np.ndarray) -> float:
        cfg, B, T, W, G = self.cfg, self.B, self.T, self.W, self.G
        S, H_, hd, D, F, V = cfg.seq, cfg.heads, cfg.head_dim, cfg.d_model, cfg.ffn, cfg.vocab
        alpha = 1.0 / math.sqrt(hd)
        ctx = self.ctx
        self.launches = 0
        tok = ctx.cell(np.ascontiguousarray(tokens, dtype=np.int32))
        tgt = ctx.cell(np.ascontiguousarray(targets, dtype=np.int32))
        x = self.new(T, D)
        self.call("gather_rows", APPLY, x, W["embed"], tok, R_32I, T, V, D, R_16F, self.status)
        saved, branch = [], None
        for Lw in W["layers"]:
            n1 = self.new(T, D)
            if branch is None:
                self.call("rmsnorm_fwd", APPLY, n1, x, Lw["pre_norm"], cfg.eps, T, D, R_16F)
            else:
                total = self.new(T, D)
                self.call("add_rmsnorm_fwd", APPLY, n1, total, x, branch, Lw["pre_norm"], cfg.eps, T, D, R_16F)
                self.free(branch)                # x is the previous layer's x_mid, which its backward still needs
                x = total
            qp, kp = self.new(T, H_, 128), self.new(T, H_, 128)
            for w, dst in ((Lw["q"], qp), (Lw["k"], kp)):
                t = self.mm(n1, w, T, D, D, False, True)
                self.call("rope_fwd", APPLY, dst, t, self.cos, self.sin, T, H_, hd, S, 128, R_16F)
                self.free(t)
            t = self.mm(n1, Lw["v"], T, D, D, False, True)
            vp = self.new(T, H_, 128)
            self.call("block_pad", APPLY, vp, t, B, S, H_, hd, 128, R_16F)
            self.free(t)
            ctxc, stats = self.new(T, D), self.new(B, H_, S, 4, esize=4)
            self.call("attention_fwd", APPLY, ctxc, stats, qp, kp, vp, B, S, H_, hd, alpha, R_16F)
            o = self.mm(ctxc, Lw["o"], T, D, D, False, True)
            n2, x_mid = self.new(T, D), self.new(T, D)
            self.call("add_rmsnorm_fwd", APPLY, n2, x_mid, x, o, Lw["post_norm"], cfg.eps, T, D, R_16F)
            self.free(o)
            up = self.mm(n2, Lw["up"], T, F, D, False, True)
            gate = self.mm(n2, Lw["gate"], T, F, D, False, True)
            h = self.new(T, F)
            self.call("swiglu_fwd", APPLY, h, gate, up, T * F, R_16F)
            branch = self.mm(h, Lw["down"], T, D, F, False, True)
            saved.append((x, n1, qp, kp, vp, stats, ctxc, x_mid, n2, up, gate, h))
            x = x_mid
        nf, total = self.new(T, D), self.new(T, D)
        self.call("add_rmsnorm_fwd", APPLY, nf, total, x, branch, W["head_norm"], cfg.eps, T, D, R_16F)
        self.free(branch)                        # x is the last layer's x_mid: freed with that layer's saved cells
        x = total                                # input of the head norm
        logits = self.mm(nf, W["lm_head"], T, V, D, False, True)
        loss, dlogits = self.new(1, esize=4), self.new(T, V)
        self.call("softmax_nll", APPLY, loss, dlogits, logits, tgt, R_32I, 1.0 / self.loss_tokens, T, V, R_16F, self.status)
        self.free(logits)
        # ---------------------------------------------------------------- backward
        self.mm(dlogits, nf, V, D, T, True, False, out=G["lm_head"])
        dnf = self.mm(dlogits, W["lm_head"], T, D, V, False, False)
        self.free(dlogits, nf)
        dx = self.new(T, D)
        self.call("rmsnorm_bwd", APPLY, APPLY, dx, G["head_norm"], dnf, x, W["head_norm"], cfg.eps, T, D, R_16F, R_16F)
        self.free(dnf, x)
        for li in range(cfg.layers - 1, -1, -1):
            Lw, Gl = W["layers"][li], G["layers"][li]
            x_in, n1, qp, kp, vp, stats, ctxc, x_mid, n2, up, gate, h = saved.pop()
            self.mm(dx, h, D, F, T, True, False, out=Gl["down"])
            dh = self.mm(dx, Lw["down"], T, F, D, False, False)
            dgate, dup = self.new(T, F), self.new(T, F)
            self.call("swiglu_bwd", APPLY, APPLY, dgate, dup, gate, up, dh, T * F, R_16F)
            self.free(dh, h, up, gate)
            self.mm(dup, n2, F, D, T, True, False, out=Gl["up"])
            self.mm(dgate, n2, F, D, T, True, False, out=Gl["gate"])
            dn2 = self.mm(dup, Lw["up"], T, D, F, False, False)
            self.mm(dgate, Lw["gate"], T, D, F, False, False, out=dn2, mode=ACC)
            self.free(dgate, dup, n2)
            self.call("rmsnorm_bwd", ACC, APPLY, dx, Gl["post_norm"], dn2, x_mid, Lw["post_norm"], cfg.eps, T, D, R_16F, R_16F)
            self.free(dn2, x_mid)
            self.mm(dx, ctxc, D, D, T, True, False, out=Gl["o"])
            dctx = self.mm(dx, Lw["o"], T, D, D, False, False)
            dctxp = self.new(T, H_, 128)
            self.call("block_pad", APPLY, dctxp, dctx, B, S, H_, hd, 128, R_16F)
            self.free(dctx)
            dv, dq, dk = self.new(T, D), self.new(T, D), self.new(T, D)
            if self.fused_bwd:
                self.call("attention_bwd", APPLY, dq, dk, dv, qp, kp, vp, dctxp, ctxc, stats, B, S, H_, hd, alpha, R_16F)
                self.free(ctxc, stats, vp, dctxp, qp, kp)
            else:
                p, ds = self.new(B, S, H_, S), self.new(B, S, H_, S)
                self.call("attention_bwd_prep", APPLY, p, ds, qp, kp, vp, dctxp, ctxc, stats, B, S, H_, hd, alpha, R_16F)
                self.free(ctxc, stats, vp)
                # P^T dO, dS K, dS^T Q on the reference's block layout; the right-hand operands are the 128-wide padded copies
                self.call("block_matmul", APPLY, dv, p, dctxp, B, H_, S, hd, S, S, 128, True, False, 1.0, TRI_A_UPPER, 0, OPERAND_B_PADDED, R_16F)
                self.free(p, dctxp)
                self.call("block_matmul", APPLY, dq, ds, kp, B, H_, S, hd, S, S, 128, False, False, alpha, TRI_A_LOWER, 0, OPERAND_B_PADDED, R_16F)
                self.call("block_matmul", APPLY, dk, ds, qp, B, H_, S, hd, S, S, 128, True, False, alpha, TRI_A_UPPER, 0, OPERAND_B_PADDED, R_16F)
                self.free(ds, qp, kp)
            unrot = []
            for d in (dq, dk):
                t = self.new(T, D)
                self.call("rope_bwd", APPLY, t, d, self.cos, self.sin, T, H_, hd, S, R_16F)
                self.free(d)
                unrot.append(t)
            dq, dk = unrot
            for d, name in ((dq, "q"), (dk, "k"), (dv, "v")):
                self.mm(d, n1, D, D, T, True, False, out=Gl[name])
            dn1 = self.mm(dq, Lw["q"], T, D, D, False, False)
            self.mm(dk, Lw["k"], T, D, D, False, False, out=dn1, mode=ACC)
            self.mm(dv, Lw["v"], T, D, D, False, False, out=dn1, mode=ACC)
            self.free(dq, dk, dv, n1)
            self.call("rmsnorm_bwd", ACC, APPLY, dx, Gl["pre_norm"], dn1, x_in, Lw["pre_norm"], cfg.eps, T, D, R_16F, R_16F)
            self.free(dn1, x_in)
        self.call("scatter_add_rows", APPLY, G["embed"], dx, tok, R_32I, T, V, D, R_16F, self.status)
        self.free(dx, tok, tgt)
        out = self.ctx.get(loss, np.zeros(1, np.float32))       # with_mem read-back: the one synchronisation of the step
        self.free(loss)
        st = self.ctx.get(self.status, np.zeros(1, np.uint32))
        if st[0]:
            raise ThunkError(f"status word {int(st[0])}: a token or target index was out of range")
        return float(out[0])

    def gradient(self, path: str) -> np.ndarray:
        """Host copy of one gradient: 'embed', 'lm_head', 'head_norm' or 'layers.<i>.<name>'."""
        parts = path.split(".")
        cell = self.G[path] if len(parts) == 1 else self.G["layers"][int(parts[1])][parts[2]]
        return self.ctx.get(cell, np.empty(self.shapes[path], np.float16))

    def adamw_init(self):
        """f32 master copies and the two running averages as stable cells (AdamW32, src/librarium/adamw.rs:20-44)."""
        self.opt = {}
        for path, shape in self.shapes.items():
            w16 = self._param_host(path)
            self.opt[path] = (self.ctx.cell(w16.astype(np.float32), stable=True),
                              self.ctx.cell(np.zeros(shape, np.float32), stable=True),
                              self.ctx.cell(np.zeros(shape, np.float32), stable=True))

    def _cells(self, path):
        parts = path.split(".")
        if len(parts) == 1:
            return self.W[path], self.G[path]
        return self.W["layers"][int(parts[1])][parts[2]], self.G["layers"][int(parts[1])][parts[2]]

    def _param_host(self, path):
        return self.ctx.get(self._cells(path)[0], np.empty(self.shapes[path], np.float16))

    def adamw_step(self, iter_nr: int, lr=1e-3, wd=0.0, a1=0.1, a2=1e-3, eps=1e-8, grad_unscale=1.0):
        """One Initialize-mode thunk per parameter: master, averages and the 16-bit copy are read and overwritten in
        place (the three in-place update thunks of AdamW32::step, src/librarium/adamw.rs:46-61, fused)."""
        for path, (master, g1, g2) in self.opt.items():
            w, g = self._cells(path)
            n = int(np.prod(self.shapes[path]))
            self.call("adamw32_step", INIT, master, g1, g2, w, g, n, R_16F, R_16F, grad_unscale, lr, wd, a1, a2, eps, iter_nr)

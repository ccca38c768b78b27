"""Small single-kernel workloads for profiling under ncu (a few GB at most, a handful of launches).

    python -m cacti_b200.profile_cases <case> [--launches N]

cases: softmax (causal fwd+bwd, 8 heads x 2048 x 2048 f16), softmax_full (config 2), nll (2048 x 32000 f16),
rmsnorm (16384 x 3200 f16), rope (16384 x 32 x 100 f16), swiglu (4096 x 8640 f16),
gemm_nt / gemm_nn / gemm_tn (4096 x 3200 x 3200 f16), qk / pv / attn_fwd / attn_bwd (--batch sequences of config 5),
train_step (one config-5 forward+backward over --batch sequences; only for the single-pass launch list).
Inputs are larger than the 126 MB L2 so DRAM counters are meaningful.
"""
from __future__ import annotations

import argparse

import torch

from . import ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--batch", type=int, default=2, help="sequences for the qk / pv cases")
    ap.add_argument("--tune", action="append", default=[], metavar="KNOB=VALUE",
                    help="set a cacti_b200_tune knob before running (repeatable), e.g. gemm_pair=1")
    a = ap.parse_args()
    for kv in a.tune:
        k, v = kv.split("=")
        if ops.lib().cacti_b200_tune(k.encode(), int(v)) != 0:
            raise SystemExit(f"tune {kv} rejected")
    gen = torch.Generator(device="cuda").manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=gen) * scale).half()

    if a.case in ("softmax", "softmax_full"):
        heads = 32 if a.case == "softmax_full" else 8
        s, dp = rnd(heads * 2048, 2048, scale=0.1), rnd(heads * 2048, 2048)
        p, ds = torch.empty_like(s), torch.empty_like(s)
        fn = lambda: ops.softmax_fwd_bwd(s, dp, (1, 2048, 0), p=p, ds=ds)
    elif a.case == "nll":
        lg = rnd(2048, 32000, scale=2.0)
        tg = torch.randint(0, 32000, (2048,), device="cuda", dtype=torch.int32, generator=gen)
        dl = torch.empty_like(lg)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        fn = lambda: ops.softmax_nll_fwd_bwd(lg, tg, w_scalar=1.0 / 2048, dlogits=dl, status=st)
    elif a.case == "rmsnorm":
        x, dy, g = rnd(16384, 3200), rnd(16384, 3200), rnd(3200)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        dg = torch.empty(3200, dtype=torch.float16, device="cuda")
        ws = ops.rmsnorm_workspace(16384, 3200, x.device)
        fn = lambda: ops.rmsnorm_fwd_bwd(x, g, dy, 1e-6, y=y, dx=dx, dgamma=dg, workspace=ws)
    elif a.case == "rope":
        cos, sin = ops.rope_tables(2048, 100)
        q, dq = rnd(16384, 32, 100), rnd(16384, 32, 100)
        yq, dxq = torch.empty_like(q), torch.empty_like(q)
        fn = lambda: ops.rope_fwd_bwd(q, dq, cos, sin, y=yq, dx=dxq)
    elif a.case == "swiglu":
        ga, up, dh = rnd(4096, 8640), rnd(4096, 8640), rnd(4096, 8640)
        h, dga, dup = torch.empty_like(ga), torch.empty_like(ga), torch.empty_like(ga)
        fn = lambda: ops.swiglu_fwd_bwd(ga, up, dh, h=h, dgate=dga, dup=dup)
    elif a.case == "train_step":
        from . import dp, llama_step as LS
        cfg = LS.LlamaShape.open_llama_3b()
        P = LS.init_weights(cfg, torch.device("cuda"))
        grads, _ = dp.alloc_bucketed_grads(P)
        step = LS.TrainStep(cfg, P, a.batch)
        tok = torch.randint(0, cfg.vocab, (a.batch * cfg.seq,), device="cuda", dtype=torch.int32, generator=gen)
        tgt = torch.randint(0, cfg.vocab, (a.batch * cfg.seq,), device="cuda", dtype=torch.int32, generator=gen)
        fn = lambda: step.forward_backward(tok, tgt, grads)
    elif a.case.startswith("gemm_") or a.case in ("qk", "pv", "attn_fwd", "attn_bwd"):
        from . import gemm_cases
        fn = gemm_cases.make(a.case, rnd, a.batch)
    else:
        raise SystemExit(f"unknown case {a.case}")
    for _ in range(a.launches):
        fn()
    torch.cuda.synchronize()
    print("done", a.case)


if __name__ == "__main__":
    main()

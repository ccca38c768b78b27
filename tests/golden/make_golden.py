"""Generate tests/golden/golden_small.npz from the CPU oracle (oracle/ref_chain.py).

The reference project has no tests or golden vectors for these ops and cannot be built without
its Rust/Futhark toolchain, so these fixtures are produced by the restatement itself: they pin the
oracle against regressions and give the GPU tests fixed targets; they do not pin it against the
reference.  Inputs are regenerated from seeds (tensor k of a case uses seed 1000*case + k), only
outputs are stored.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_chain as R  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_small.npz")


def inputs(case):
    """Seeded inputs of every golden case (shared with the tests)."""
    s = 1000 * case
    if case == 1:      # RMSNorm f32, 8 rows of benchmark config 1
        return dict(x=R.normal(s + 0, (8, 3200)), gamma=R.normal(s + 1, (3200,), scale=0.02, shift=1.0),
                    dy=R.normal(s + 2, (8, 3200)), eps=1e-6)
    if case == 2:      # RMSNorm f16
        return dict(x=R.normal(s + 0, (8, 3200), np.float16), gamma=R.normal(s + 1, (3200,), np.float16, 0.02, 1.0),
                    dy=R.normal(s + 2, (8, 3200), np.float16), eps=1e-6)
    if case == 3:      # causal softmax f16, layout [B=1, H=2, Sq=64, Sk=64] -> rows = 128, q_div 1
        return dict(s=R.normal(s + 0, (128, 64), np.float16, 0.1), dp=R.normal(s + 1, (128, 64), np.float16),
                    mask=(1, 64, 0))
    if case == 4:      # causal softmax f16, reference layout [B=1, Sq=32, H=3, Sk=32] -> q_div 3
        return dict(s=R.normal(s + 0, (96, 32), np.float16, 0.1), dp=R.normal(s + 1, (96, 32), np.float16),
                    mask=(3, 32, 0))
    if case == 5:      # RoPE f16: 40 tokens, 4 heads, head_dim 100, seq 16
        return dict(x=R.normal(s + 0, (40, 4, 100), np.float16), dy=R.normal(s + 1, (40, 4, 100), np.float16),
                    seq=16, theta=10000.0)
    if case == 6:      # SwiGLU f16
        return dict(gate=R.normal(s + 0, (8, 864), np.float16), up=R.normal(s + 1, (8, 864), np.float16),
                    dh=R.normal(s + 2, (8, 864), np.float16))
    if case == 7:      # softmax-NLL f16, vocab 32000, 3 rows
        return dict(logits=R.normal(s + 0, (3, 32000), np.float16, 2.0), targets=R.uniform_int(s + 1, 3, 32000),
                    w=np.float32(1.0 / 3))
    if case == 8:      # gather / scatter-add
        return dict(table=R.normal(s + 0, (50, 64), np.float16), tokens=R.uniform_int(s + 1, 40, 50),
                    dy=R.normal(s + 2, (40, 64), np.float16))
    raise KeyError(case)


def outputs(case):
    a = inputs(case)
    if case in (1, 2):
        y, _, _ = R.ref_rmsnorm_fwd(a["x"], a["gamma"], a["eps"])
        dx, dg = R.ref_rmsnorm_bwd(a["x"], a["gamma"], a["dy"], a["eps"])
        return dict(y=y, dx=dx, dgamma=dg)
    if case in (3, 4):
        keep = R.causal_keep_mask(a["s"].shape[0], a["s"].shape[1], *a["mask"])
        p, _ = R.ref_softmax_fwd(a["s"], keep)
        return dict(p=p, ds=R.ref_softmax_bwd(a["s"], a["dp"], keep))
    if case == 5:
        cos, sin = R.ref_rope_tables(a["seq"], 100, a["theta"], np.float16)
        pos = np.arange(40) % a["seq"]
        return dict(cos=cos, sin=sin, y=R.ref_rope_fwd(a["x"], cos, sin, pos), dx=R.ref_rope_bwd(a["dy"], cos, sin, pos))
    if case == 6:
        h, _ = R.ref_swiglu_fwd(a["gate"], a["up"])
        dg, du = R.ref_swiglu_bwd(a["gate"], a["up"], a["dh"])
        return dict(h=h, dgate=dg, dup=du)
    if case == 7:
        loss, d, picked = R.ref_softmax_nll(a["logits"], a["targets"], a["w"])
        return dict(loss_rows=loss, loss_sum=np.float32((loss * a["w"]).sum(dtype=np.float32)), dlogits=d, picked=picked)
    if case == 8:
        return dict(out=R.ref_gather_rows(a["table"], a["tokens"]),
                    dtable=R.ref_scatter_add_rows(a["dy"], a["tokens"], 50))
    raise KeyError(case)


CASES = range(1, 9)

if __name__ == "__main__":
    blob = {}
    for c in CASES:
        for k, v in outputs(c).items():
            blob[f"c{c}_{k}"] = np.asarray(v)
    np.savez_compressed(OUT, **blob)
    print(OUT, os.path.getsize(OUT), "bytes")

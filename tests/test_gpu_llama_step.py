"""The composed training step (benchmark config 5 at reduced depth/width) against the composed CPU oracle."""
import numpy as np
import pytest
import torch

from cacti_b200 import llama_step as LS
from oracle import llama_oracle, ref_chain as R
from tests.gpu_util import dev, host
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu


def _np_params(P):
    out = {k: host(v) for k, v in P.items() if k != "layers"}
    out["layers"] = [{k: host(v) for k, v in L.items()} for L in P["layers"]]
    return out


@pytest.mark.parametrize("hd,heads", [(20, 4), (16, 2)])
def test_reduced_step_matches_oracle(cuda, hd, heads):
    cfg = LS.LlamaShape(layers=2, d_model=hd * heads, heads=heads, head_dim=hd, ffn=96, vocab=160, seq=32)
    B = 2
    P = LS.init_weights(cfg, cuda, seed=0, std=0.08)
    # non-trivial norm gains so that dgamma and the gain path are exercised
    for L in P["layers"]:
        L["pre_norm"].copy_(dev(R.normal(50, (cfg.d_model,), np.float16, 0.1, 1.0)))
        L["post_norm"].copy_(dev(R.normal(51, (cfg.d_model,), np.float16, 0.1, 1.0)))
    tok = R.uniform_int(1, B * cfg.seq, cfg.vocab)
    tgt = R.uniform_int(2, B * cfg.seq, cfg.vocab)
    grads = LS.zeros_like_params(P)
    step = LS.TrainStep(cfg, P, B)
    loss = step.forward_backward(dev(tok), dev(tgt), grads)
    torch.cuda.synchronize()
    assert host(step.status)[0] == 0
    ref_loss, ref_g = llama_oracle.step(_np_params(P), tok, tgt, cfg)
    assert abs(float(host(loss)[0]) - float(ref_loss)) < 2e-3 * abs(float(ref_loss))
    # gradients pass through ~40 f16-rounded thunks; hold them to 2 % of the tensor's rms
    for name in ("lm_head", "head_norm", "embed"):
        assert_close(host(grads[name]), ref_g[name], "float16", name, rtol=2e-2, floor_frac=1.0)
    for li in range(cfg.layers):
        for name, g in grads["layers"][li].items():
            assert_close(host(g), ref_g["layers"][li][name], "float16", f"layer {li} {name}", rtol=2e-2, floor_frac=1.0)
    assert step.launches > 0


@pytest.mark.parametrize("hd,heads,seq", [(100, 2, 256), (64, 3, 128)])
def test_fused_attention_step_matches_oracle_and_unfused(cuda, hd, heads, seq):
    """Same step with attention fused (scores never in HBM, P and dS rebuilt per tile in the backward): against the
    composed CPU oracle at the tolerance of the unfused step, and against the unfused step itself."""
    cfg = LS.LlamaShape(layers=2, d_model=hd * heads, heads=heads, head_dim=hd, ffn=96, vocab=160, seq=seq)
    B = 2
    P = LS.init_weights(cfg, cuda, seed=1, std=0.08)
    for L in P["layers"]:
        L["pre_norm"].copy_(dev(R.normal(52, (cfg.d_model,), np.float16, 0.1, 1.0)))
        L["post_norm"].copy_(dev(R.normal(53, (cfg.d_model,), np.float16, 0.1, 1.0)))
    tok = R.uniform_int(3, B * cfg.seq, cfg.vocab)
    tgt = R.uniform_int(4, B * cfg.seq, cfg.vocab)
    out = {}
    for mode in ("fused", "fused-bwd", "unfused"):
        grads = LS.zeros_like_params(P)
        step = LS.TrainStep(cfg, P, B, attention=mode)
        assert step.fused == (mode != "unfused") and step.fused_bwd == (mode == "fused-bwd")
        loss = step.forward_backward(dev(tok), dev(tgt), grads)
        torch.cuda.synchronize()
        assert host(step.status)[0] == 0
        out[mode] = (float(host(loss)[0]), grads)
    auto = LS.TrainStep(cfg, P, B)
    assert auto.fused and not auto.fused_bwd                # "auto": fused forward, P and dS materialised once in the backward
    ref_loss, ref_g = llama_oracle.step(_np_params(P), tok, tgt, cfg)
    for mode, (loss, grads) in out.items():
        assert abs(loss - float(ref_loss)) < 2e-3 * abs(float(ref_loss)), mode
        for name in ("lm_head", "head_norm", "embed"):
            assert_close(host(grads[name]), ref_g[name], "float16", f"{mode} {name}", rtol=2e-2, floor_frac=1.0)
        for li in range(cfg.layers):
            for name, g in grads["layers"][li].items():
                assert_close(host(g), ref_g["layers"][li][name], "float16", f"{mode} layer {li} {name}", rtol=2e-2, floor_frac=1.0)
    assert abs(out["fused"][0] - out["unfused"][0]) < 1e-3 * abs(out["unfused"][0])
    assert out["fused"][0] == out["fused-bwd"][0]            # the forward passes are the same kernels


def test_graphed_step_replays_the_eager_step(cuda):
    """The step captured in a CUDA graph and replayed twice gives the loss and gradients of the eager step, bit for
    bit (same kernels, same order), also after the inputs in the captured buffers were replaced."""
    cfg = LS.LlamaShape(layers=2, d_model=200, heads=2, head_dim=100, ffn=96, vocab=160, seq=128)
    B = 2
    P = LS.init_weights(cfg, cuda, seed=1, std=0.08)
    toks = [R.uniform_int(3 + i, B * cfg.seq, cfg.vocab) for i in range(2)]
    tgts = [R.uniform_int(13 + i, B * cfg.seq, cfg.vocab) for i in range(2)]
    eager = []
    for tok, tgt in zip(toks, tgts):
        grads = LS.zeros_like_params(P)
        loss = LS.TrainStep(cfg, P, B).forward_backward(dev(tok), dev(tgt), grads)
        torch.cuda.synchronize()
        eager.append((host(loss).copy(), [host(g).copy() for _, g in LS.flat_params(grads)]))
    grads = LS.zeros_like_params(P)
    step = LS.TrainStep(cfg, P, B)
    tok_d, tgt_d = dev(toks[0]).clone(), dev(tgts[0]).clone()
    gs = LS.GraphedStep(lambda: step.forward_backward(tok_d, tgt_d, grads))
    for i in (0, 1, 0):
        tok_d.copy_(dev(toks[i])); tgt_d.copy_(dev(tgts[i]))
        loss = gs.replay()
        torch.cuda.synchronize()
        assert np.array_equal(host(loss), eager[i][0])
        for (_, g), ref in zip(LS.flat_params(grads), eager[i][1]):
            assert np.array_equal(host(g), ref)
    assert host(step.status)[0] == 0


def test_batched_qkv_matmuls_give_the_same_bits(cuda):
    """q, k and v projections (and their weight gradients) run as one batched matmul when the three weights (gradients)
    lie back to back in memory, as init_weights and dp.alloc_bucketed_grads lay them out; separately otherwise.  Both
    ways must give the same loss and gradients, bit for bit."""
    from cacti_b200 import dp as DP
    cfg = LS.LlamaShape(layers=2, d_model=256, heads=2, head_dim=128, ffn=128, vocab=160, seq=128)
    B = 2
    P = LS.init_weights(cfg, cuda, seed=5, std=0.08)
    assert LS.stacked(P["layers"][0]["q"], P["layers"][0]["k"], P["layers"][0]["v"]) is not None
    P_apart = {k: v.clone() for k, v in P.items() if k != "layers"}
    P_apart["layers"] = [{k: torch.cat([v.reshape(-1), v.new_zeros(8)])[:v.numel()].view(v.shape) for k, v in L.items()}
                         for L in P["layers"]]
    assert LS.stacked(P_apart["layers"][0]["q"], P_apart["layers"][0]["k"], P_apart["layers"][0]["v"]) is None
    tok, tgt = dev(R.uniform_int(3, B * cfg.seq, cfg.vocab)), dev(R.uniform_int(4, B * cfg.seq, cfg.vocab))
    res = []
    for params, bucketed in ((P, True), (P_apart, False)):
        grads = DP.alloc_bucketed_grads(params)[0] if bucketed else LS.zeros_like_params(params)
        G0 = grads["layers"][0]
        assert (LS.stacked(G0["q"], G0["k"], G0["v"]) is not None) == bucketed
        step = LS.TrainStep(cfg, params, B)
        loss = step.forward_backward(tok, tgt, grads)
        torch.cuda.synchronize()
        assert host(step.status)[0] == 0
        res.append((host(loss).copy(), [host(g).copy() for _, g in LS.flat_params(grads)], step.launches))
    assert np.array_equal(res[0][0], res[1][0])
    for a, b in zip(res[0][1], res[1][1]):
        assert np.array_equal(a, b)
    assert res[0][2] == res[1][2] - 4 * cfg.layers           # two launches instead of six per layer

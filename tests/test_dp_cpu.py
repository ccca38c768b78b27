"""World-size-2 gloo test of the data-parallel host logic (sequence sharding, bucketed gradient all-reduce)."""
import os
import socket
import subprocess
import sys

import torch

from cacti_b200 import dp

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from cacti_b200 import dp
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=int(os.environ["RANK"]), world_size=2)
rank = dist.get_rank()
params = {"embed": torch.zeros(7, 5), "head_norm": torch.zeros(5),
          "layers": [{"q": torch.zeros(5, 5), "pre_norm": torch.zeros(5)} for _ in range(3)]}
grads, buckets = dp.alloc_bucketed_grads(params)
assert len(buckets) == 5          # 3 layers, the output head, the rest
red = dp.GradReducer(buckets)
assert red.enabled
for li in (2, 1, 0):                      # backward order
    grads["layers"][li]["q"].fill_(float(rank + 1) * (li + 1))
    grads["layers"][li]["pre_norm"].fill_(float(rank + 10))
    red.reduce_bucket(li)
grads["embed"].fill_(float(rank)); grads["head_norm"].fill_(1.0)
red.reduce_bucket(3)
red.reduce_bucket(4)
red.finish()
for li in range(3):
    assert torch.all(grads["layers"][li]["q"] == 3.0 * (li + 1)), grads["layers"][li]["q"]
    assert torch.all(grads["layers"][li]["pre_norm"] == 21.0)
assert torch.all(grads["embed"] == 1.0) and torch.all(grads["head_norm"] == 2.0)
first, count = dp.shard_sequences(8, 2, rank)
t = torch.tensor([first, count]); out = [torch.zeros(2, dtype=torch.long) for _ in range(2)]
dist.all_gather(out, t)
assert [o.tolist() for o in out] == [[0, 4], [4, 4]]
dist.destroy_process_group()
print("ok", rank)
'''


def test_shard_sequences_covers_everything():
    for n in (1, 7, 8, 9):
        for world in (1, 2, 4, 8):
            got = [dp.shard_sequences(n, world, r) for r in range(world)]
            assert sum(c for _, c in got) == n
            pos = 0
            for first, count in got:
                assert first == pos
                pos += count


def test_bucketed_grads_are_views_of_the_buckets():
    params = {"embed": torch.zeros(3, 4), "lm_head": torch.zeros(3, 4), "head_norm": torch.zeros(4),
              "layers": [{"a": torch.zeros(2, 2), "b": torch.zeros(5)}]}
    grads, buckets = dp.alloc_bucketed_grads(params)
    assert len(buckets) == 3                 # layer 0, output head, embedding
    grads["lm_head"].fill_(1.0)
    assert buckets[1].sum().item() == 12.0 and buckets[2].sum().item() == 0.0
    grads["layers"][0]["b"].fill_(2.0)
    assert buckets[0].sum().item() == 10.0 and grads["layers"][0]["a"].shape == (2, 2)
    assert dp.GradReducer(buckets).enabled is False        # no process group: a single-GPU run reduces nothing


def test_gloo_world2_allreduce():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), PORT=str(port), REPO=repo)
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"ok {r}" in o, o


LOST_RANK_WORKER = r'''
import datetime, os, sys, time, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from cacti_b200 import dp
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=int(os.environ["RANK"]), world_size=2,
                        timeout=datetime.timedelta(seconds=20))
rank = dist.get_rank()
buckets = [torch.full((64,), float(rank + 1)) for _ in range(2)]
red = dp.GradReducer(buckets, timeout_s=5.0)
red.reduce_bucket(0); red.reduce_bucket(1); red.finish()          # step 1: both ranks take part
assert torch.all(buckets[0] == 3.0)
dist.barrier()
if rank == 1:
    print("ok 1 (leaving between steps)", flush=True)
    os._exit(0)                                                     # the rank is gone: no shutdown handshake
t0 = time.time()
try:                                                                # step 2: the survivor's exchange must end with an error
    red.reduce_bucket(0); red.reduce_bucket(1); red.finish()
    print("exchange completed without its peer", flush=True); sys.exit(3)
except Exception as e:
    dt = time.time() - t0
    assert dt < 15.0, dt
    print(f"ok 0 (raised {type(e).__name__} after {dt:.1f} s)", flush=True)
os._exit(0)
'''


def test_a_rank_that_leaves_between_steps_ends_the_exchange_with_an_error():
    """Failure made on the host: rank 1 exits between two steps.  Rank 0's next gradient exchange raises within the
    reducer's time-out instead of waiting for ever."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), PORT=str(port), REPO=repo)
        procs.append(subprocess.Popen([sys.executable, "-c", LOST_RANK_WORKER], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"ok {r}" in o, o


def test_stacked_views_need_adjacent_tensors_of_one_storage():
    """llama_step.stacked: the [n, rows, 1, cols] view behind the batched q / k / v matmuls exists only for equal,
    contiguous tensors that lie back to back in one storage (as init_weights and alloc_bucketed_grads lay them out)."""
    import torch
    from cacti_b200 import dp as DP, llama_step as LS
    flat = torch.arange(3 * 6 * 4, dtype=torch.float32)
    a, b, c = (flat[i * 24:(i + 1) * 24].view(6, 4) for i in range(3))
    v = LS.stacked(a, b, c)
    assert v is not None and v.shape == (3, 6, 1, 4)
    assert torch.equal(v[1, :, 0, :], b) and torch.equal(v[2, 5, 0], c[5])
    assert LS.stacked(a, c, b) is None                                   # wrong order
    assert LS.stacked(a, b.clone(), c) is None                           # another storage
    gap = torch.zeros(3 * 24 + 8)
    g0, g1 = gap[0:24].view(6, 4), gap[32:56].view(6, 4)
    assert LS.stacked(g0, g1) is None                                    # padding in between
    assert LS.stacked(a, flat[24:48].view(4, 6)) is None                 # another shape
    assert LS.stacked(a.t(), b.t()) is None                              # not contiguous
    # the layouts the step relies on
    cfg = LS.LlamaShape(layers=1, d_model=256, heads=2, head_dim=128, ffn=128, vocab=64, seq=128)
    P = LS.init_weights(cfg, torch.device("cpu"), seed=0)
    L0 = P["layers"][0]
    assert LS.stacked(L0["q"], L0["k"], L0["v"]) is not None
    G0 = DP.alloc_bucketed_grads(P)[0]["layers"][0]
    assert LS.stacked(G0["q"], G0["k"], G0["v"]) is not None
    G1 = LS.zeros_like_params(P)["layers"][0]
    assert LS.stacked(G1["q"], G1["k"], G1["v"]) is None

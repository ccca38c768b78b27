"""Checkpoint ingest onto the GPU: mmap -> pinned ring -> async H2D delivers the file's bytes."""
import pytest
import torch

from cacti_b200 import ingest
from cacti_b200.llama_step import init_weights, zeros_like_params
from tests.test_ingest_cpu import CFG, hf_state, ingest_flat, write_safetensors

pytestmark = pytest.mark.gpu


def test_load_llama_to_device(cuda, tmp_path):
    src = init_weights(CFG, torch.device("cpu"), seed=5)
    write_safetensors(tmp_path / "model.safetensors", hf_state(src))
    dst = zeros_like_params(init_weights(CFG, torch.device("cuda"), seed=6))
    # slots far smaller than the tensors: every slot is reused many times while earlier transfers are in flight
    copier = ingest.StagedCopier("cuda", slot_bytes=256, slots=2)
    ingest.load_llama(ingest.TensorsDir.open(tmp_path), dst, copier)
    want = dict(ingest_flat(src))
    total = 0
    for k, v in ingest_flat(dst):
        assert torch.equal(v.cpu(), want[k]), k
        total += v.numel() * v.element_size()
    assert copier.h2d_bytes == total
    torch.save(hf_state(src), tmp_path / "pytorch_model.bin")
    dst2 = zeros_like_params(dst)
    ingest.load_llama(ingest.PickleDir.open(tmp_path), dst2)
    for k, v in ingest_flat(dst2):
        assert torch.equal(v.cpu(), want[k]), k

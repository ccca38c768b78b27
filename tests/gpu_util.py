"""Host<->device helpers for the GPU parity tests (torch is only the owner of device memory)."""
import numpy as np
import torch

from oracle import ref_chain as R


def dev(a, device="cuda:0", bf16=False):
    """numpy array -> device tensor.  bf16=True: a is float32 and is rounded to bfloat16."""
    a = np.ascontiguousarray(a)
    if bf16:
        return torch.from_numpy(R.to_bf16_bits(a).view(np.int16)).to(device).view(torch.bfloat16).reshape(a.shape)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.uint16)
    return torch.from_numpy(a).to(device)


def host(t):
    """device tensor -> numpy (bf16 comes back as float32)."""
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    if t.dtype == torch.uint16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def offset_view(a, off, device="cuda:0"):
    """Copy `a` into a device buffer at an element offset, returning the (unaligned) view."""
    t = dev(a, device)
    buf = torch.empty(t.numel() + off + 16, dtype=t.dtype, device=device)
    v = buf[off:off + t.numel()].view(t.shape)
    v.copy_(t)
    return v


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])

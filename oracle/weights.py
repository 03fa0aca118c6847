"""Deterministic, name-keyed parameter fill (TEST INFRASTRUCTURE ONLY).

Both the golden-vector generator (reference modules) and the parity tests (the
CUDA-backed modules) fill their parameters with this function, so that no
weight file has to be stored: every tensor is drawn from a CPU generator seeded
by a CRC of its state_dict key."""
import zlib

import torch


def keyed_tensor(key, shape, seed=0):
    g = torch.Generator().manual_seed((zlib.crc32(key.encode()) + 7919 * seed) & 0x7FFFFFFF)
    return torch.randn(tuple(shape), generator=g)


def fill_state_dict(module, seed=0, prefix=""):
    """Overwrites every parameter/buffer of ``module`` in place; returns the
    resulting state_dict (fp32, CPU clones)."""
    sd = module.state_dict()
    new = {}
    for k, v in sd.items():
        name = prefix + k
        if k.endswith("num_batches_tracked"):
            new[k] = torch.zeros_like(v)
            continue
        t = keyed_tensor(name, v.shape, seed)
        if k.endswith("running_var"):
            t = 0.5 + t.abs()
        elif k.endswith("running_mean"):
            t = 0.1 * t
        elif k.endswith("bias"):
            t = 0.1 * t
        elif v.dim() == 1:                       # norm scales
            t = 1.0 + 0.1 * t
        else:                                    # weight matrices / conv kernels
            fan_in = v.numel() // v.shape[0]
            t = t / (fan_in ** 0.5)
        new[k] = t.to(v.dtype)
    module.load_state_dict(new)
    return {k: v.clone() for k, v in new.items()}

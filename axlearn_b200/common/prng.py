"""Host-side splittable PRNG keys.

A key is a CPU ``torch.uint32`` tensor of shape ``[4]`` (128 bits), the same shape and dtype
the reference stores as ``prng_key`` in its trainer state (axlearn/common/trainer.py:367 with
the "rbg" implementation selected at axlearn/common/utils_spmd.py:46).  Derivation
(``fold_in`` / ``split``) is a keyed 128-bit hash evaluated on the host — it costs a
microsecond and never touches the GPU.  Random *tensors* are drawn from a ``torch.Generator``
seeded from the key on the device that will hold the tensor, so initialisation and dropout
stay device-resident.
"""

from __future__ import annotations

import hashlib
import struct
from typing import Sequence, Union

import numpy as np
import torch

KEY_SHAPE = (4,)
KEY_DTYPE = torch.uint32


def _to_bytes(key: torch.Tensor) -> bytes:
    if key.shape != KEY_SHAPE:
        raise ValueError(f"PRNG key must have shape {KEY_SHAPE}, got {tuple(key.shape)}")
    return key.detach().cpu().numpy().astype(np.uint32).tobytes()


def _from_bytes(b: bytes) -> torch.Tensor:
    return torch.from_numpy(np.frombuffer(b, dtype=np.uint32).copy())


def PRNGKey(seed: int) -> torch.Tensor:  # pylint: disable=invalid-name
    """Creates a key from an integer seed."""
    digest = hashlib.blake2b(struct.pack("<q", int(seed)), digest_size=16, person=b"axb200-seed").digest()
    return _from_bytes(digest)


def fold_in(key: torch.Tensor, data: int) -> torch.Tensor:
    """Deterministically derives a new key from ``key`` and an integer."""
    digest = hashlib.blake2b(
        struct.pack("<q", int(data) & 0x7FFFFFFFFFFFFFFF),
        digest_size=16,
        key=_to_bytes(key),
        person=b"axb200-fold",
    ).digest()
    return _from_bytes(digest)


def split(key: torch.Tensor, num: int = 2) -> list[torch.Tensor]:
    """Derives ``num`` independent keys."""
    kb = _to_bytes(key)
    return [
        _from_bytes(
            hashlib.blake2b(
                struct.pack("<q", i), digest_size=16, key=kb, person=b"axb200-split"
            ).digest()
        )
        for i in range(num)
    ]


def seed_of(key: torch.Tensor) -> int:
    """A 63-bit integer seed for ``torch.Generator.manual_seed``."""
    lo, hi = struct.unpack("<QQ", _to_bytes(key))
    return (lo ^ (hi * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


def generator(key: torch.Tensor, device: Union[str, torch.device] = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed_of(key))
    return g


def normal(
    key: torch.Tensor, shape: Sequence[int], *, dtype=torch.float32, device="cpu", std: float = 1.0
) -> torch.Tensor:
    out = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    out.normal_(0.0, 1.0, generator=generator(key, device))
    if std != 1.0:
        out.mul_(std)
    return out.to(dtype)


def uniform(
    key: torch.Tensor,
    shape: Sequence[int],
    *,
    dtype=torch.float32,
    device="cpu",
    minval: float = 0.0,
    maxval: float = 1.0,
) -> torch.Tensor:
    out = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    out.uniform_(minval, maxval, generator=generator(key, device))
    return out.to(dtype)


def truncated_normal(
    key: torch.Tensor, shape: Sequence[int], *, dtype=torch.float32, device="cpu", std: float = 1.0
) -> torch.Tensor:
    """Normal truncated to [-2, 2] standard deviations, rescaled to unit variance before
    ``std`` is applied (the correction constant is the std of the truncated law)."""
    out = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    torch.nn.init.trunc_normal_(out, 0.0, 1.0, -2.0, 2.0, generator=generator(key, device))
    out.mul_(std / 0.87962566103423978)
    return out.to(dtype)


def randint(
    key: torch.Tensor, shape: Sequence[int], low: int, high: int, *, dtype=torch.int32, device="cpu"
) -> torch.Tensor:
    return torch.randint(
        low, high, tuple(shape), generator=generator(key, device), device=device, dtype=dtype
    )


def bernoulli(key: torch.Tensor, p: float, shape: Sequence[int], *, device="cpu") -> torch.Tensor:
    return uniform(key, shape, device=device) < p

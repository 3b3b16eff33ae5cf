"""PyTorch-CPU restatement of one depth step (TEST/BENCH INFRASTRUCTURE: the timed CPU baseline).

The reference has no CPU path for its engine (every entry point requires CUDA tensors, beam_engine.py:284), so the
CPU arm of the benchmark is the same step written with the idioms the reference itself uses on torch/numpy tensors:
gather expansion (data_loader.py:141-148), FNV-1a/fmix64 hashing (data_loader.py:192-213), uniqueness through
torch.unique + scatter_reduce, score threshold by sorting, float32 nn.Linear scorer (scorers.py:21-36).  It uses all
host threads torch is given.  It returns the same surviving set as oracle/beam_oracle.py (checked in tests).
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

_M = (1 << 64) - 1


def _i64(x: int) -> int:
    x &= _M
    return x - (1 << 64) if x >= (1 << 63) else x


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    return (x >> s) & ((1 << (64 - s)) - 1)


def _mix64(x: torch.Tensor) -> torch.Tensor:
    x = x ^ _lsr(x, 33)
    x = x * _i64(0xFF51AFD7ED558CCD)
    x = x ^ _lsr(x, 33)
    x = x * _i64(0xC4CEB9FE1A85EC53)
    return x ^ _lsr(x, 33)


def hash64(states: torch.Tensor) -> torch.Tensor:
    """int64 tensor holding the unsigned 64-bit hash bit pattern (beam_kernels.cu:38-48)."""
    s = states.to(torch.int64)
    h = torch.full((s.shape[0],), _i64(1469598103934665603), dtype=torch.int64)
    for i in range(s.shape[1]):
        h = (h ^ s[:, i]) * 1099511628211
    h = _mix64(h)
    return torch.where((h >= 0) & (h <= 2), h + 4, h)


def fingerprint64(states: torch.Tensor) -> torch.Tensor:
    """beam_kernels.cu:50-59."""
    s = states.to(torch.int64)
    g = _i64(0x9E3779B97F4A7C15)
    h = torch.full((s.shape[0],), g, dtype=torch.int64)
    for i in range(s.shape[1]):
        h = h ^ (s[:, i] + g + (h << 6) + _lsr(h, 2))
    h = _mix64(h ^ _i64(0xD6E8FEB86659FD93))
    return torch.where(h == 0, torch.full_like(h, 4), h)


class TorchMLP(torch.nn.Module):
    def __init__(self, w: Dict[str, np.ndarray]):
        super().__init__()
        h, k = w["w1"].shape
        self.l1 = torch.nn.Linear(k, h)
        self.l2 = torch.nn.Linear(h, h)
        self.l3 = torch.nn.Linear(h, 1)
        with torch.no_grad():
            self.l1.weight.copy_(torch.from_numpy(w["w1"])); self.l1.bias.copy_(torch.from_numpy(w["b1"]))
            self.l2.weight.copy_(torch.from_numpy(w["w2"])); self.l2.bias.copy_(torch.from_numpy(w["b2"]))
            self.l3.weight.copy_(torch.from_numpy(w["w3"])[None, :]); self.l3.bias.fill_(float(w["b3"]))

    def forward(self, x):
        return self.l3(torch.relu(self.l2(torch.relu(self.l1(x))))).squeeze(1)


def _unsigned_order(h: torch.Tensor) -> torch.Tensor:
    """Map the int64 bit pattern so that signed order equals unsigned order."""
    return h ^ _i64(1 << 63)


@torch.no_grad()
def depth_step(frontier: torch.Tensor, gens: torch.Tensor, solved: torch.Tensor, beam: int, num_values: int,
               models: Optional[Sequence[TorchMLP]] = None, score_offset: float = -150.0, chunk: int = 65536):
    """One depth on CPU tensors.  frontier [P, n] uint8, gens [G, n] int64.  Returns (next frontier [K, n], keys [K])."""
    p, n = frontier.shape
    g = gens.shape[0]
    children = frontier[:, gens].reshape(p * g, n)  # gather, parent-major
    h = hash64(children)
    f = fingerprint64(children)
    if models is None:
        key = (children != solved[None, :]).sum(dim=1).to(torch.int64)
    else:
        qs = []
        for c0 in range(0, children.shape[0], chunk):
            x = torch.nn.functional.one_hot(children[c0:c0 + chunk].to(torch.int64), num_values).flatten(1).float()
            q = sum(m(x) for m in models) / float(len(models))
            qs.append(q)
        q = torch.cat(qs) - score_offset
        key = (q.clamp(0.0, 300.0) * 256.0 + 0.5).to(torch.int64)
    payload = torch.arange(p * g, dtype=torch.int64)  # parent*G + move: same order as (parent, move)
    # dedup on (hash, fingerprint): winner = min (key, payload)
    hf = torch.stack([h, f], dim=1)
    _, inv = torch.unique(hf, dim=0, return_inverse=True)
    val = (key << 32) | payload
    best = torch.full((int(inv.max()) + 1,), torch.iinfo(torch.int64).max, dtype=torch.int64)
    best.scatter_reduce_(0, inv, val, reduce="amin")
    win = best & 0xFFFFFFFF
    wkey = best >> 32
    wh = _unsigned_order(h[win])
    wf = _unsigned_order(f[win])
    # exact K on (key, hash, fingerprint): three stable sorts, least significant first
    order = torch.argsort(wf, stable=True)
    order = order[torch.argsort(wh[order], stable=True)]
    order = order[torch.argsort(wkey[order], stable=True)]
    keep = win[order[:beam]]
    return children[keep], key[keep]

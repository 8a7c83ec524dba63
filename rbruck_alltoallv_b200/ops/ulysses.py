"""Sequence <-> head re-sharding for sequence-parallel attention (the "Ulysses" exchange), on top of the
uniform all-to-all.

Every rank holds a slice of the sequence with all heads, ``[S / P, H, D]``; attention wants the whole sequence
for a slice of the heads, ``[S, H / P, D]``.  Going there and back is two uniform all-to-alls of
``S / P * H / P * D`` elements per pair.  The reference has no attention or sequence code; this is an example of
the library's collective in the place a training framework would use it.  Both directions are persistent calls:
buffers and counts are fixed at construction, a call is one pack (a strided local copy) and one kernel launch.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch


class UlyssesExchange:
    def __init__(self, comm, seq_local: int, heads: int, head_dim: int, dtype=torch.bfloat16, algo: str = "spreadout",
                 **algo_kw):
        P, L = comm.P, comm.L
        if heads % P:
            raise ValueError("the number of heads must be a multiple of the number of ranks")
        self.comm, self.P, self.L = comm, P, L
        self.s_l, self.h, self.hp, self.d, self.dtype = seq_local, heads, heads // P, head_dim, dtype
        self.block = seq_local * self.hp * head_dim                  # elements per (source, destination) pair
        dev = f"cuda:{comm.device}"
        n = P * self.block
        counts = np.full((L, P), self.block, dtype=np.int32)
        displs = np.tile(np.arange(P, dtype=np.int64) * self.block, (L, 1))
        self._send = [torch.empty(n, dtype=dtype, device=dev) for _ in range(L)]
        self._recv = [comm.symm_empty(n, dtype) for _ in range(L)]
        self._call = comm.prepare(self._send, self._recv, counts, displs, counts, displs, algo=algo, **algo_kw)

    def _as_list(self, x) -> List[torch.Tensor]:
        return [x] if isinstance(x, torch.Tensor) else list(x)

    def seq_to_head(self, x: Sequence[torch.Tensor] | torch.Tensor) -> List[torch.Tensor]:
        """``[S / P, H, D]`` per local rank -> ``[S, H / P, D]`` per local rank (views of the library's buffers,
        valid until the next exchange)."""
        P, s_l, hp, d = self.P, self.s_l, self.hp, self.d
        for buf, t in zip(self._send, self._as_list(x)):
            # block for rank q = my sequence slice of head group q
            buf.view(P, s_l, hp, d).copy_(t.view(s_l, P, hp, d).permute(1, 0, 2, 3))
        self._call.launch()
        return [r.view(P * s_l, hp, d) for r in self._recv]          # block from rank q = sequence slice q

    def head_to_seq(self, y: Sequence[torch.Tensor] | torch.Tensor) -> List[torch.Tensor]:
        """``[S, H / P, D]`` per local rank -> ``[S / P, H, D]`` per local rank (fresh tensors)."""
        P, s_l, hp, d = self.P, self.s_l, self.hp, self.d
        for buf, t in zip(self._send, self._as_list(y)):
            buf.copy_(t.reshape(-1))                                 # sequence slice q is already the block for rank q
        self._call.launch()
        # block from rank q = my sequence slice of head group q
        return [r.view(P, s_l, hp, d).permute(1, 0, 2, 3).reshape(s_l, self.h, d) for r in self._recv]

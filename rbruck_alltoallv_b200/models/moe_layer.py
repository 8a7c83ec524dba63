"""MoE FFN layer as a user-facing module, plus the smoke routine used by the repository entry point."""
from __future__ import annotations

import torch

from ..ops.moe import MoEExpertParallel, reference_forward


class MoELayer:
    """Top-2 routed SwiGLU FFN with experts sharded over the communicator's ranks.

    ``router_weight`` [E, H] (optional): when given, logits are ``x @ router_weight.T`` in fp32; otherwise the
    caller passes logits to :meth:`forward`.
    """

    def __init__(self, comm, num_experts, hidden, inter, tokens, router_weight=None, **kw):
        self.ep = MoEExpertParallel(comm, num_experts, hidden, inter, tokens, **kw)
        self.router_weight = router_weight

    def forward(self, x, logits=None):
        if logits is None:
            if self.router_weight is None:
                raise ValueError("either logits or a router weight is needed")
            logits = (x.float() @ self.router_weight.float().t()).contiguous()
        return self.ep.forward(x, logits)

    __call__ = forward


def smoke_moe(comm=None):
    """Tiny single-GPU forward checked against the fp32 reference."""
    from ..parallel.comm import Communicator
    own = Communicator(nranks=1, heap_bytes=256 << 20, arena_bytes=1 << 20)
    try:
        T, H, I, E = 256, 256, 512, 8
        layer = MoELayer(own, E, H, I, T, seed=1)
        g = torch.Generator(device="cuda")
        g.manual_seed(7)
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, device="cuda", generator=g)
        out = layer(x, logits)
        layer.ep.check()
        ref, _, _ = reference_forward(x, logits, layer.ep.w13, layer.ep.w2)
        err = (out.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= 0.02 * scale + 1e-3, f"MoE smoke mismatch: max err {err} vs scale {scale}"
        # the same layer with MXFP8 expert GEMMs (hardware block scaling, fused SwiGLU + quantiser epilogue)
        mx = MoELayer(own, E, H, I, T, seed=1, fp8="mx")
        out = mx(x, logits)
        mx.ep.check()
        rel = (out.float() - ref).norm().item() / ref.norm().item()
        assert rel < 0.08, f"MXFP8 MoE smoke deviates {rel:.3f} from the fp32 reference"
    finally:
        own.close()

"""Router plug-ins with the reference's interface (models/decoder_moe.py:47-151):
`forward(logits[S,E], top_k) -> (topk_idx int64 [S,K], topk_w [S,K])` and `.name`.

All of them run on the CUDA kernels of libmoe_b200.so and reject CPU tensors.
"""
from __future__ import annotations

import torch

from . import ops


class RouterBase(torch.nn.Module):
    """Interface: route logits -> (topk_idx[int64], topk_weight[float])"""

    def forward(self, logits: torch.Tensor, top_k: int):  # noqa: D401
        raise NotImplementedError

    @property
    def name(self) -> str:
        return self.__class__.__name__


class CUDATopKRouter(RouterBase):
    """Top-k + softmax over the picked logits (models/decoder_moe.py:58-62, :126-151).
    Lowest expert index wins ties; weights are returned in the logits dtype."""

    available = True

    def forward(self, logits: torch.Tensor, top_k: int):
        if top_k <= 0:
            raise ValueError("top_k must be > 0")
        if top_k > logits.size(-1):
            raise ValueError("top_k must be <= n_experts")
        idx_i32, w_f32 = ops.topk_select(logits, int(top_k))
        return idx_i32.to(torch.int64), w_f32.to(dtype=logits.dtype)


# The reference's default router has the same contract; on this library both names run the kernel.
TorchTopKRouter = CUDATopKRouter


class SinkhornRouter(RouterBase):
    """Sinkhorn-Knopp router (models/decoder_moe.py:65-123) as one CUDA kernel."""

    def __init__(self, *, iters: int = 10, epsilon: float = 1e-6, temperature: float = 1.0):
        super().__init__()
        if iters <= 0:
            raise ValueError("SinkhornRouter.iters must be > 0")
        if epsilon <= 0:
            raise ValueError("SinkhornRouter.epsilon must be > 0")
        if temperature <= 0:
            raise ValueError("SinkhornRouter.temperature must be > 0")
        self.iters = int(iters)
        self.epsilon = float(epsilon)
        self.temperature = float(temperature)

    def forward(self, logits: torch.Tensor, top_k: int):
        if logits.dim() != 2:
            raise ValueError("SinkhornRouter expects logits of shape [tokens, experts]")
        if top_k <= 0:
            raise ValueError("top_k must be > 0")
        if top_k > logits.size(1):
            raise ValueError("top_k must be <= n_experts")
        idx, w = ops.sinkhorn(logits, int(top_k), iters=self.iters, epsilon=self.epsilon,
                              temperature=self.temperature)
        return idx.to(torch.int64), w.to(dtype=logits.dtype)

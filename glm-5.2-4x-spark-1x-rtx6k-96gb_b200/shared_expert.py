"""The dense shared expert of a sparse layer, beside the routed path.

Every sparse layer of the model adds a shared expert that all rows pass through:
``hidden + routed_moe + shared_mlp`` (python/reference/glmrt_reference/glm_moe_dsa_layer_ref.py:157-206),
with ``shared_mlp = expert_forward(normalized, shared weights)`` (moe_ref.py:17-21): the same
gate / up / SwiGLU / down arithmetic as a routed expert, but dense -- float32 math on the stored
weights, no activation quantisation -- and run by the coordinator, not by the expert workers
(``docs/balanced-path.md:53-66`` times it as "shared MLP" next to routing and dispatch).

It is three plain GEMMs over all rows, so it goes to the library GEMM (cuBLAS through
``torch.matmul``; float32 accumulation) with the SwiGLU between them, and its result enters the
routed layer's combine as the shared delta (``MoeLayer.forward_residual``), where
``out = bf16(residual + bf16(shared + routed))`` is formed in one pass
(native/cuda/kernels/residual.cu:36-62).  Nothing here touches the routed experts' kernels.
"""
from __future__ import annotations

import torch


class DenseSharedExpert:
    """Shared-expert weights resident on the current device: gate/up ``[I, H]``, down ``[H, I]``.

    ``dtype``: ``torch.float32`` reproduces the reference's float32 arithmetic exactly as stated
    (weights up-cast once at load, TF32 off); ``torch.bfloat16`` keeps the weights as stored and
    lets the GEMMs accumulate in float32 (outputs of the first two GEMMs are rounded to bf16).
    """

    def __init__(self, gate_proj: torch.Tensor, up_proj: torch.Tensor, down_proj: torch.Tensor,
                 dtype: torch.dtype = torch.float32):
        assert gate_proj.shape == up_proj.shape and down_proj.shape == gate_proj.shape[::-1]
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.gate_up = torch.cat([gate_proj, up_proj], dim=0).to(dev, dtype).contiguous()   # [2I, H]: one GEMM for both
        self.down = down_proj.to(dev, dtype).contiguous()
        self.inter = gate_proj.shape[0]

    def delta(self, normalized_bf16: torch.Tensor) -> torch.Tensor:
        """bf16 ``expert_forward(normalized)`` rows: what the layer adds as ``shared_mlp``."""
        assert normalized_bf16.dtype == torch.bfloat16 and normalized_bf16.is_cuda
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            x = normalized_bf16.to(self.dtype)
            gu = (x @ self.gate_up.T).float()
            g, u = gu[:, :self.inter], gu[:, self.inter:]
            act = torch.nn.functional.silu(g) * u
            y = act.to(self.dtype) @ self.down.T
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        return y.to(torch.bfloat16)


def sparse_layer_forward(routed_layer, shared: DenseSharedExpert, residual_bf16: torch.Tensor,
                         normalized_bf16: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``residual + routed_moe(normalized) + shared_mlp(normalized)`` with the two additions folded into
    the routed layer's combine (glm_moe_dsa_layer_ref.py:190-198)."""
    return routed_layer.forward_residual(normalized_bf16, residual_bf16, shared.delta(normalized_bf16), out)

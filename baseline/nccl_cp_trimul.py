"""Context-parallel TriMul forward the conventional way: eager PyTorch kernels + NCCL collectives.

This is the on-box comparison target for the fused path, in the spirit of the reference's DTensor
context-parallel baseline (benchmark/distributed/trimul_dtensor_reference.py:2454-3302 in the
reference project): the pair tensor is row-sharded, every rank projects its own tokens, and the
token-pair contraction gets its missing operand through a collective --

* outgoing  tri[i,j] = sum_k a[i,k] b[j,k]: all-gather of b over the row shards, local batched GEMM;
* incoming  tri[i,j] = sum_k a[k,i] b[k,j]: local partial sums over the rank's k rows for every
  (i, j), then a reduce-scatter over the row shards.

bf16 storage, fp32 accumulation inside the library GEMMs, the same twelve operations as the oracle
(fold_cp_ops/workflows/trimul_autotune.py:1505-1525).  Nothing here is used by the product path.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F


class NcclCpTriMul:
    def __init__(self, weights: Dict[str, Optional[torch.Tensor]], group=None, eps: float = 1e-5,
                 dtype: torch.dtype = torch.bfloat16):
        self.group = group
        self.eps = eps
        self.dtype = dtype
        cast = lambda t: None if t is None else t.to(dtype)
        self.w = {k: cast(v) for k, v in weights.items()}

    def _world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    @torch.no_grad()
    def forward(self, x_local: torch.Tensor, direction: str = "outgoing",
                mask_local: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x_local: (B, N/cp, N, D) rows of the pair tensor owned by this rank; returns the same shape."""
        w = self.w
        B, ni, N, D = x_local.shape
        cp = self._world()
        x = x_local.to(self.dtype)
        xn = F.layer_norm(x, (D,), w["norm_in_w"], w["norm_in_b"], self.eps)
        ab = F.linear(xn, w["p_in_w"], w["p_in_b"]) * torch.sigmoid(F.linear(xn, w["g_in_w"], w["g_in_b"]))
        if mask_local is not None:
            ab = ab * mask_local.to(self.dtype).unsqueeze(-1)
        a, b = ab.chunk(2, dim=-1)                      # (B, ni, N, D) each
        a_cm = a.permute(0, 3, 1, 2).contiguous()       # (B, D, ni, N): channel planes
        b_cm = b.permute(0, 3, 1, 2).contiguous()
        del ab, a, b
        if direction == "outgoing":
            if cp > 1:
                parts = [torch.empty_like(b_cm) for _ in range(cp)]
                dist.all_gather(parts, b_cm, group=self.group)
                b_full = torch.cat(parts, dim=2)        # (B, D, N, N): b[j, k] for every j
                del parts
            else:
                b_full = b_cm
            tri_cm = torch.matmul(a_cm, b_full.transpose(-1, -2))    # (B, D, ni, N)
            del b_full
        elif direction == "incoming":
            part = torch.matmul(a_cm.transpose(-1, -2), b_cm)         # (B, D, N, N): sum over this rank's k rows
            if cp > 1:
                send = part.permute(2, 0, 1, 3).contiguous()          # (N, B, D, N): output row i leading
                del part
                rank = dist.get_rank(self.group)
                if dist.get_backend(self.group) == "nccl":
                    recv = torch.empty((ni, B, D, N), dtype=send.dtype, device=send.device)
                    dist.reduce_scatter_tensor(recv, send, group=self.group)
                else:  # backends without reduce-scatter (CPU tests): all-reduce and keep the own rows
                    dist.all_reduce(send, group=self.group)
                    recv = send[rank * ni:(rank + 1) * ni]
                tri_cm = recv.permute(1, 2, 0, 3)                      # (B, D, ni, N)
            else:
                tri_cm = part
        else:
            raise ValueError(f"direction must be 'outgoing' or 'incoming', got {direction!r}")
        tri = tri_cm.permute(0, 2, 3, 1)                               # (B, ni, N, D) view
        y = F.linear(F.layer_norm(tri, (D,), w["norm_out_w"], w["norm_out_b"], self.eps), w["p_out_w"], w["p_out_b"])
        return y * torch.sigmoid(F.linear(xn, w["g_out_w"], w["g_out_b"]))

"""The reference's second expert-parallel strategy (moe/sglang_moe_all_gather_all_reduce.py:162-446):
every rank sees all tokens, computes only its own experts' slots and the partial outputs are summed
with an all-reduce.  `EPMoE(config)` keeps the reference's constructor and attribute names; the
compute is the fused pipeline of DeepseekV3MoE restricted to the rank's expert range."""
from typing import List, Optional

import torch

from .all2all_moe import DeepseekV3MoE, MoEGate  # noqa: F401
from .config import Config  # noqa: F401
from .group_gemm_kernel import (gelu_and_mul_triton_kernel, grouped_gemm_triton, post_reorder_triton_kernel,  # noqa: F401
                                pre_reorder_triton_kernel, run_moe_ep_preproess, silu_and_mul_triton_kernel)


class GroupedGemmRunner(torch.nn.Module):
    """reference :25-55: the module the reference's EPMoE builds once (`GroupedGemmRunner(device)`) and
    calls for both grouped GEMMs; forwards to grouped_gemm_triton with the same argument order."""

    def __init__(self, device):
        super().__init__()
        self.device = device
        self.use_flashinfer = False

    def forward(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, batch_size: int,
                weight_column_major: bool, seg_indptr: Optional[torch.Tensor] = None,
                weight_indices: Optional[torch.Tensor] = None, use_fp8_w8a8: bool = False,
                scale_a: torch.Tensor = None, scale_b: torch.Tensor = None,
                block_shape: Optional[List[int]] = None):
        return grouped_gemm_triton(a, b, c, batch_size, weight_column_major, seg_indptr, weight_indices,
                                   use_fp8_w8a8, scale_a, scale_b, block_shape=block_shape)


class EPMoE(DeepseekV3MoE):
    def __init__(self, config, device=None):
        config.ep_strategy = "allreduce"
        super().__init__(config, device=device)
        # names of the reference class (:176-196)
        self.tp_size, self.tp_rank = self.ep_size, self.ep_rank
        self.num_experts = config.n_routed_experts
        self.num_experts_per_partition = self.experts_per_rank
        self.start_expert_id = self.tp_rank * self.num_experts_per_partition
        self.end_expert_id = self.start_expert_id + self.num_experts_per_partition - 1
        self.top_k = config.num_experts_per_tok
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.moe_intermediate_size
        self.activation = config.hidden_act          # "silu" or "gelu" (reference :374-397)
        self.grouped_gemm_runner = GroupedGemmRunner(self._dev)

    def forward(self, hidden_states: torch.Tensor, router_logits=None):
        """hidden_states [batch, seq, hidden]: ALL tokens, identical on every rank (reference :275-277)."""
        return super().forward(hidden_states)

"""The reference's second expert-parallel strategy (moe/sglang_moe_all_gather_all_reduce.py:162-446):
every rank sees all tokens, computes only its own experts' slots and the partial outputs are summed
with an all-reduce.  `EPMoE(config)` keeps the reference's constructor and attribute names; the
compute is the fused pipeline of DeepseekV3MoE restricted to the rank's expert range."""
import torch

from .all2all_moe import DeepseekV3MoE, MoEGate  # noqa: F401
from .config import Config  # noqa: F401
from .group_gemm_kernel import (gelu_and_mul_triton_kernel, grouped_gemm_triton, post_reorder_triton_kernel,  # noqa: F401
                                pre_reorder_triton_kernel, run_moe_ep_preproess, silu_and_mul_triton_kernel)


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
        self.activation = config.hidden_act

    def forward(self, hidden_states: torch.Tensor, router_logits=None):
        """hidden_states [batch, seq, hidden]: ALL tokens, identical on every rank (reference :275-277)."""
        return super().forward(hidden_states)

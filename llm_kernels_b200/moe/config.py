"""Layer configuration.  The attribute names and model defaults are the ones the reference's
callers set and read (moe/config.py:3-31), so its test scripts can configure this layer unchanged.

Grouped by what they control; every attribute is set on the instance by ``Config()``.

model shape     hidden_size, intermediate_size (dense MLP width), moe_intermediate_size (expert
                width), n_routed_experts, num_experts_per_tok, n_shared_experts, hidden_act
router          scoring_func ("sigmoid" as the reference, or "softmax", which the reference rejects
                at moe/all2all_moe.py:67-72), topk_method, n_group, topk_group, norm_topk_prob,
                routed_scaling_factor, seq_aux
parallelism     ep_size; plus, read with getattr when present: ep_strategy, ep_exchange,
                ep_recv_capacity, ep_passes, ep_gemm_ctas (see moe/all2all_moe.py)
expert numerics quantize_method selects the B200 expert path:
                  "fp8_block"  e4m3 weights with 128x128 f32 scales, e4m3 activations 1x128
                  "w4a16"      asymmetric group-128 int4 weights, bf16 activations
                  "w4a8"       two-level int4 weights, int8 activations 1x128
                use_block_quant, w_quant_block_size, a_quant_block_size, w_bit, a_bit, w_dtype,
                a_dtype describe that choice the way the reference's flags do
"""
import torch

_MODEL = dict(hidden_size=7168, intermediate_size=18432, moe_intermediate_size=2048,
              n_routed_experts=256, num_experts_per_tok=8, n_shared_experts=0, hidden_act="silu")
_ROUTER = dict(scoring_func="sigmoid", topk_method="noaux_tc", n_group=8, topk_group=4,
               norm_topk_prob=True, routed_scaling_factor=2.5, seq_aux=True)
_RUNTIME = dict(ep_size=1, use_triton_group_gemm=True)   # the grouped path is the only path here
_NUMERICS = dict(quantize_method="fp8_block", use_block_quant=True, w_quant_block_size=(128, 128),
                 a_quant_block_size=(1, 128), w_bit=8, a_bit=8,
                 w_dtype=torch.float8_e4m3fn, a_dtype=torch.float8_e4m3fn)


class Config:
    def __init__(self):
        for group in (_MODEL, _ROUTER, _RUNTIME, _NUMERICS):
            for name, value in group.items():
                setattr(self, name, value)

"""Parity metrics with the definitions of the reference's moe/utils.py:131-240
(ResultAnalyzer.compare_tensors).  The reference's ResultCollector, which writes
.pt files on every forward (moe/utils.py:34-64), is kept as an inert stub so code
that calls it keeps working without touching the disk."""
import logging
from typing import Optional

import torch

EPSILON = 1e-8
DEFAULT_SIMILARITY_THRESHOLD = 0.99
DEFAULT_DIFF_THRESHOLD = 1e-3


def setup_logging(name: str = "moe", level=logging.INFO):
    logger = logging.getLogger(name)
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s - %(name)s - %(levelname)s - %(message)s"))
        logger.addHandler(h)
    logger.setLevel(level)
    return logger


class ResultCollector:
    @staticmethod
    def save(name, tensor, prefix="", rank=0, output_dir=None):
        return None


class ResultAnalyzer:
    @staticmethod
    def compare_tensors(tensor1: torch.Tensor, tensor2: torch.Tensor, var_name: Optional[str] = None,
                        rank: int = 0, verbose: bool = False,
                        similarity_threshold: float = DEFAULT_SIMILARITY_THRESHOLD,
                        diff_threshold: float = DEFAULT_DIFF_THRESHOLD, logger=None) -> dict:
        a = tensor1.reshape(-1, tensor1.shape[-1]).float()
        b = tensor2.reshape(-1, tensor2.shape[-1]).float()
        abs_diff = (a - b).abs()
        max_diff, mean_diff = abs_diff.max().item(), abs_diff.mean().item()
        rel = abs_diff / (torch.maximum(a.abs(), b.abs()) + EPSILON)
        cos = torch.nn.functional.cosine_similarity(a, b, dim=1)
        res = {
            "max_diff": max_diff, "mean_diff": mean_diff,
            "max_rel_diff": rel.max().item(), "mean_rel_diff": rel.mean().item(),
            "avg_sim_val": cos.mean().item(), "min_sim_val": cos.min().item(),
            "max_sim_val": cos.max().item(),
            "is_equivalent": (mean_diff < diff_threshold and max_diff < diff_threshold * 10
                              and rel.mean().item() < diff_threshold * 10),
            "rel_fro": ((a - b).double().norm() / b.double().norm().clamp_min(1e-300)).item(),
        }
        if verbose:
            (logger or setup_logging("tensor_metrics")).info(f"Rank {rank}: {var_name}: {res}")
        return res

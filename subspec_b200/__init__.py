"""subspec_b200 — the speculative-decoding hot path of NYCU-EDgeAi/subspec on B200 (sm_100a).

Keeps the reference's `specdecodes` call signatures for tree verification, the
draft tree and the KV-cache managers, and runs them on hand-written CUDA kernels
reached through a C-ABI shared library (include/subspec_b200.h).  No CPU fallback.
"""
from .tree import Tree
from .verify import (VerifyOutput, VerifyWorkspace, lossy_bottom_up_verify, verify_tree, verify_tree_batched)
from .wandb_logger import wandb_logger

__all__ = ["Tree", "VerifyOutput", "VerifyWorkspace", "lossy_bottom_up_verify", "verify_tree", "verify_tree_batched",
           "wandb_logger"]

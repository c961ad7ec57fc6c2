"""Small helpers shared by the all-reduce host code (reference: mini_allreduce/utils.py)."""
import logging
import os

import torch
import torch.distributed as dist


def is_cuda() -> bool:
    return torch.cuda.is_available() and torch.version.cuda is not None


def get_bool_env_var(name: str, default: str = "false") -> bool:
    return os.getenv(name, default).lower() in ("true", "1")


def log_info_on_rank0(logger: logging.Logger, msg: str) -> None:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0:
        logger.info(msg)

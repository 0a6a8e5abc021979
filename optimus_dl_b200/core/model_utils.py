"""Parameter counting that de-duplicates shared tensors (optimus_dl/core/model_utils.py:10-34)."""

from __future__ import annotations

import torch


def get_num_parameters(model: torch.nn.Module, only_trainable: bool = False) -> int:
    seen: set[int] = set()
    total = 0
    for p in model.parameters():
        if only_trainable and not p.requires_grad:
            continue
        key = p.data_ptr() if p.numel() > 0 and p.device.type != "meta" else id(p)
        if key in seen:
            continue
        seen.add(key)
        total += p.numel()
    return total

"""LinearStrassen and replace_linear_with_strassen (reference: model/layers.py:232-300, with
the constructor spellings of fixed_strassen_fp32_agg.py:128-169, main_profiling.py:51-92 and
modded_nanogpt/data_dist_train_gpt2.py:71-116).

The layer stays an ``nn.Linear`` subclass with ordinary parameters, so FSDP
(``use_orig_params=True``), autocast and ``state_dict`` treat it like any Linear. Differences
from the reference, all widenings: in_features may differ from out_features, the flattened batch
may exceed the feature size (no zero padding to D x D is made), and ``depth=None`` / ``-1`` asks the
tuner table for algorithm and depth.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import ops


class LinearStrassen(nn.Linear):
    def __init__(self, in_features: int, out_features: Optional[int] = None, bias: bool = True, dtype=None,
                 depth: Optional[int] = 1, device="cuda", algo: str = "classic") -> None:
        # main_profiling.py:51-60 spells the constructor (features, bias, dtype, depth, device)
        if isinstance(out_features, bool):
            # every later positional argument sits one slot to the left in that spelling
            new_dtype = bias if (isinstance(bias, torch.dtype) or bias is None) else dtype
            new_depth = dtype if isinstance(dtype, int) else depth
            new_device = depth if isinstance(depth, (str, torch.device)) else device
            out_features, bias, dtype, depth, device = None, out_features, new_dtype, new_depth, new_device
        if out_features is None:
            out_features = in_features
        super().__init__(in_features, out_features, bias, device, dtype)
        self.depth = depth
        self.algo = algo

    def forward(self, input: Tensor) -> Tensor:
        *batch_dims, d_in = input.shape
        assert d_in == self.in_features, "Input dim mismatch"
        x = input.reshape(-1, d_in)
        w = self.weight
        if torch.is_autocast_enabled():
            dt = torch.get_autocast_dtype("cuda")
            x, w = x.to(dt), w.to(dt)
        elif x.dtype != w.dtype:
            x = x.to(w.dtype)
        auto = self.depth is None or self.depth < 0
        if auto:
            algo, depth = "auto", -1
        elif self.depth == 0:
            algo, depth = "dense", 0
        else:
            algo, depth = self.algo, min(self.depth, 4)
            # sizes that do not split into whole 16-byte vectors use fewer levels
            while depth > 0 and any(v % (8 << depth) for v in (x.shape[0], d_in, self.out_features)):
                depth -= 1
            if depth == 0:
                algo = "dense"
        # weight.T stays a view (model/layers.py:252); the bias rides in the product's epilogue
        # instead of a separate pass over the output (model/layers.py:271-272)
        if self.bias is not None:
            out = ops.linear_autograd(x, w.t(), self.bias, algo, depth)
        else:
            out = ops.matmul_autograd(x, w.t(), algo, depth)
        return out.view(*batch_dims, self.out_features)


def replace_linear_with_strassen(module: nn.Module, min_size: int = 128, depth: int = 1):
    """model/layers.py:279-300: swap every square nn.Linear of at least ``min_size`` features
    for a LinearStrassen carrying the same weight and bias; recurse into children."""
    for name, child in module.named_children():
        if isinstance(child, nn.Linear) and not isinstance(child, LinearStrassen):
            if child.in_features == child.out_features and child.in_features >= min_size:
                print(f"Replacing '{name}' with LinearStrassen.")
                new_layer = LinearStrassen(child.in_features, child.out_features, bias=child.bias is not None,
                                           device=child.weight.device, dtype=child.weight.dtype, depth=depth)
                new_layer.weight.data.copy_(child.weight.data)
                if child.bias is not None:
                    new_layer.bias.data.copy_(child.bias.data)
                setattr(module, name, new_layer)
            else:
                print(f"Skipping '{name}': Not square or too small.")
        elif len(list(child.children())) > 0:
            replace_linear_with_strassen(child, min_size, depth)

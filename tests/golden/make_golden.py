"""Generates tests/golden/reference_outputs.npz by importing the reference project itself
(vmad18/strassen-triton, read-only checkout) and running its torch-level Strassen functions on
CPU tensors with seeded inputs. Run once in the build container:

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/reference

The archive holds, per case, the inputs' seed/shape/dtype (inputs are regenerated from the seed)
and the reference's output bits (bf16/fp16 stored as uint16 views, fp32 as float32).
"""
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def make_inputs(seed, n, dtype, dist):
    """A then B from one CPU generator, fp32, scaled, then cast: the order every implementation
    in this repository uses so that all of them see identical bits."""
    g = torch.Generator("cpu").manual_seed(seed)
    if dist == "normal":
        A = torch.randn((n, n), generator=g)
        B = torch.randn((n, n), generator=g)
    elif dist == "normal_scaled":
        A = torch.randn((n, n), generator=g) / n ** 0.5
        B = torch.randn((n, n), generator=g) / n ** 0.5
    else:  # uniform(-1, 1)
        A = 2 * torch.rand((n, n), generator=g) - 1
        B = 2 * torch.rand((n, n), generator=g) - 1
    return A.to(dtype), B.to(dtype)


def to_numpy(t):
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


CASES = [
    # name, module, function, kwargs, seed, n, dtype, dist
    ("agg_base_bf16_128", "fixed_strassen_fp32_agg", "_strassen_base", {"base_dtype": torch.bfloat16}, 0, 128, torch.bfloat16, "normal_scaled"),
    ("agg_d1_bf16_128", "fixed_strassen_fp32_agg", "strassen_matmul_n_layers", {"n_depth": 1, "base_dtype": torch.bfloat16}, 0, 128, torch.bfloat16, "normal_scaled"),
    ("agg_d2_bf16_128", "fixed_strassen_fp32_agg", "strassen_matmul_n_layers", {"n_depth": 2, "base_dtype": torch.bfloat16}, 0, 128, torch.bfloat16, "uniform"),
    ("agg_d3_bf16_128", "fixed_strassen_fp32_agg", "strassen_matmul_n_layers", {"n_depth": 3, "base_dtype": torch.bfloat16}, 1, 128, torch.bfloat16, "uniform"),
    ("agg_d2_fp16_64", "fixed_strassen_fp32_agg", "strassen_matmul_n_layers", {"n_depth": 2, "base_dtype": torch.float16}, 2, 64, torch.float16, "normal_scaled"),
    ("agg_d2_default_fp32_64", "fixed_strassen_fp32_agg", "strassen_matmul_n_layers", {}, 3, 64, torch.float32, "normal"),
    ("agg_small_16", "fixed_strassen_fp32_agg", "_strassen_base", {}, 4, 16, torch.float32, "normal"),
    ("plain_base_bf16_128", "fixed_strassen", "_strassen_base", {}, 0, 128, torch.bfloat16, "normal_scaled"),
    ("plain_d2_bf16_128", "fixed_strassen", "strassen_matmul_n_layers", {"n_depth": 2}, 0, 128, torch.bfloat16, "uniform"),
    ("plain_d3_bf16_128", "fixed_strassen", "strassen_matmul_n_layers", {"n_depth": 3}, 1, 128, torch.bfloat16, "uniform"),
    ("plain_d1_fp32_128", "fixed_strassen", "strassen_matmul_n_layers", {"n_depth": 1}, 0, 128, torch.float32, "normal"),
    ("plain_d2_fp32_128", "fixed_strassen", "strassen_matmul_n_layers", {"n_depth": 2}, 0, 128, torch.float32, "normal"),
    ("two_layers_fp32_128", "strassen", "strassen_matmul_two_layers", {}, 1234, 128, torch.float32, "normal"),
    ("strassen_base_fp32_128", "strassen", "_strassen_base", {}, 1234, 128, torch.float32, "normal"),
    ("two_layers_bf16_64", "strassen", "strassen_matmul_two_layers", {}, 3331, 64, torch.bfloat16, "normal_scaled"),
]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of vmad18/strassen-triton>")
    ref_dir = sys.argv[1]
    sys.path.insert(0, ref_dir)
    import importlib

    out = {}
    for name, mod, fn, kwargs, seed, n, dtype, dist in CASES:
        module = importlib.import_module(mod)
        A, B = make_inputs(seed, n, dtype, dist)
        C = getattr(module, fn)(A, B, **kwargs)
        out[name] = to_numpy(C)
        out[name + "__dtype"] = np.array(str(C.dtype))
        print(name, tuple(C.shape), C.dtype)
    np.savez_compressed(os.path.join(HERE, "reference_outputs.npz"), **out)


if __name__ == "__main__":
    main()

"""Seeded synthetic inputs shared by the tests (CPU generator, so that host and device see the same bits)."""
import numpy as np
import torch


def randn_fp16(shape, seed, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.float16)


def np16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().numpy()


def bits(a) -> np.ndarray:
    """fp16 array -> uint16 bit patterns (so that NaN == NaN and -0 != +0 in comparisons)."""
    if isinstance(a, torch.Tensor):
        a = np16(a)
    return np.ascontiguousarray(a).view(np.uint16)


def edge_case_matrix(seed=7):
    """(1, 12, 64) fp16 matrix whose rows exercise the out-of-domain paths of the rounding:
    all-zero row, row of fp16 subnormals (scale underflows to a subnormal / zero), a row with NaN,
    a row with +-inf, a row reaching the largest finite fp16, rows with exact .5 ties."""
    x = randn_fp16((1, 12, 64), seed).numpy().copy()
    x[0, 0, :] = 0
    x[0, 1, :] = np.float16(6e-8) * (np.arange(64) % 5)          # subnormals: amax/127 rounds to 0
    x[0, 2, :] = np.float16(2e-5) * ((np.arange(64) % 7) - 3)    # scale is an fp16 subnormal
    x[0, 3, 5] = np.float16(np.nan)
    x[0, 4, 9] = np.float16(np.inf)
    x[0, 4, 10] = -np.float16(np.inf)
    x[0, 5, 0] = np.float16(65504.0)
    x[0, 6, :] = (np.arange(64) - 32).astype(np.float16) * np.float16(0.5)   # amax 16 -> scale 0.126: many ties unlikely
    x[0, 7, :] = 0
    x[0, 7, 0] = np.float16(127.0)                                # scale exactly 1: x = k + 0.5 are exact ties
    x[0, 7, 1:40] = (np.arange(39) - 19).astype(np.float16) + np.float16(0.5)
    x[0, 8, :] = -x[0, 7, :]
    x[0, 9, :] = np.float16(-0.0)
    return torch.from_numpy(x)

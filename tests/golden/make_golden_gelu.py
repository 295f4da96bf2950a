"""Generates tests/golden/reference_gelu_sm100.npz: the reference's own cu_gelu_forward (cuda/gelu.cu:6-17, compiled
unmodified for sm_100 into oracle/_ref/gelu.fatbin by `make -C oracle ref`) evaluated on every one of the 65536 fp16
bit patterns.  GELU maps one fp16 value to one fp16 value, so this table is the complete behaviour of that kernel.

    python tests/golden/make_golden_gelu.py          (on a machine with an sm_100 GPU)
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.ref_cuda import ReferenceKernels  # noqa: E402


def main():
    out_path = os.path.join(ROOT, "tests", "golden", "reference_gelu_sm100.npz")
    if len(sys.argv) > 1:
        out_path = sys.argv[1]
    ref = ReferenceKernels()
    x = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16).reshape(16, 4096).cuda()
    y = ref.gelu_forward(x)
    torch.cuda.synchronize()
    table = y.cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    np.savez_compressed(out_path, gelu_of_every_fp16=table)
    print("wrote", out_path, table.shape)


if __name__ == "__main__":
    main()

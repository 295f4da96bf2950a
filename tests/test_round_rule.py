"""Host-side proof obligations of the quantisation kernels' arithmetic shortcuts."""
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _compile(tmp_path):
    exe = str(tmp_path / "round_rule_check")
    flags = ["-O2", "-ffp-contract=off"]
    if "fma" in open("/proc/cpuinfo").read():
        flags.append("-mfma")
    subprocess.run(["gcc"] + flags + ["-I", os.path.join(ROOT, "cpm_kernels_b200", "csrc"), "-o", exe,
                    os.path.join(ROOT, "tests", "csrc", "round_rule_check.c"), "-lm"], check=True)
    return exe


def test_division_free_rounding_rule_is_exact(tmp_path):
    """Every third fp16 scale x every fp16 value in the rule's domain (about 4.6e8 pairs): whenever the rule
    claims a code, it is the reference's (int8)nearbyintf(x / s).  The full sweep (stride 1, 1.4e9 pairs, also
    0 mismatches) is `round_rule_check 0x0400 0x7bff 1`."""
    exe = _compile(tmp_path)
    procs = [subprocess.Popen([exe, hex(0x0400 + off), "0x7bff", "3"], stdout=subprocess.PIPE, text=True) for off in (0,)]
    for p in procs:
        out = p.communicate()[0]
        assert p.returncode == 0, out
        assert "mismatches=0" in out
        pairs = int(out.split("pairs=")[1].split()[0])
        ties = int(out.split("ties=")[1].split()[0])
        assert pairs > 4e8
        assert 0 < ties < pairs * 1e-3      # the fallback to the division is rare


def test_scale_division_in_binary32_equals_the_references_double_division():
    """cuda/gemm.cu:74 computes half(amax / 127.0) with a double division narrowed to float; the kernels use a
    binary32 division.  Equal for every non-negative fp16 amax and for random binary32 amax (backward kernels)."""
    bits = np.arange(0, 0x7c01, dtype=np.uint16)
    amax = bits.view(np.float16).astype(np.float32)
    ref = (amax.astype(np.float64) / 127.0).astype(np.float32)
    got = amax / np.float32(127.0)
    assert (ref.view(np.uint32) == got.view(np.uint32)).all()
    rng = np.random.default_rng(1)
    r = (rng.random(4_000_000, dtype=np.float32) * np.float32(2.0) ** rng.integers(-30, 30, 4_000_000).astype(np.float32)).astype(np.float32)
    ref = (r.astype(np.float64) / 127.0).astype(np.float32)
    got = r / np.float32(127.0)
    assert (ref.view(np.uint32) == got.view(np.uint32)).all()

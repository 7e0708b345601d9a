"""The specification header the kernels are built from (csrc/fw_spec.cuh) compiles as plain C++
too.  Its host build is checked here, without a GPU, against the oracle's independent C code: the
Philox block function in both of its forms (key schedule in place, round keys formed ahead of time),
the exponential key and the PPR stop threshold.  This pins the header's arithmetic to the oracle's
on the CPU; the GPU parity tests then cover what nvcc makes of the same source."""
import os
import subprocess

import numpy as np

import oracle_lib as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include <cstdio>
#include <cstdint>
#include <cstring>
#include "fw_spec.cuh"
int main() {
  unsigned long long n = 0;
  if (scanf("%llu", &n) != 1) return 2;
  for (unsigned long long i = 0; i < n; ++i) {
    unsigned c[4], k[2];
    double tp;
    if (scanf("%u %u %u %u %u %u %lf", &c[0], &c[1], &c[2], &c[3], &k[0], &k[1], &tp) != 7) return 3;
    const fw::Philox4 a = fw::philox4x32_10(c[0], c[1], c[2], c[3], k[0], k[1]);
    uint32_t rk[20];
    fw::philox_round_keys(k[0], k[1], rk);
    const fw::Philox4 b = fw::philox4x32_10(c[0], c[1], c[2], c[3], rk);
    const float e = fw::exp_key(a.x);
    uint32_t ebits;
    memcpy(&ebits, &e, 4);
    printf("%u %u %u %u %u %u %u %u %u %u\n", a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, ebits,
           fw::tp_threshold(tp));
  }
  return 0;
}
"""


def test_spec_header_matches_oracle(tmp_path):
    src = tmp_path / "spec_check.cpp"
    exe = tmp_path / "spec_check"
    src.write_text(PROGRAM)
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    # -ffp-contract=off: the header's fp32 arithmetic is written with explicit fmaf where it wants one
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-x", "c++", str(src), "-o", str(exe),
                    "-I" + os.path.join(ROOT, "flowwalker_artifact_b200", "csrc")], check=True, env=env)
    rng = np.random.default_rng(23)
    n = 4000
    words = rng.integers(0, 2 ** 32, size=(n, 6), dtype=np.uint64)
    # known-answer vectors of Random123 first, then edge cases of the key function
    words[0] = 0
    words[1] = 0xFFFFFFFF
    words[2] = [0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0]
    tps = rng.random(n)
    tps[:6] = [0.0, 1.0, 0.2, 0.5, 1e-12, 0.999999999]
    lines = ["%d" % n] + ["%d %d %d %d %d %d %.17g" % (*[int(x) for x in w], tp) for w, tp in zip(words, tps)]
    res = subprocess.run([str(exe)], input="\n".join(lines) + "\n", capture_output=True, text=True, check=True)
    out = np.array([[int(x) for x in ln.split()] for ln in res.stdout.splitlines()], dtype=np.uint64)
    assert out.shape == (n, 10)
    assert out[0, :4].tolist() == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert out[1, :4].tolist() == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert out[2, :4].tolist() == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    lib = O.lib()
    import ctypes
    lib.fwo_exp_key.restype = ctypes.c_float
    lib.fwo_exp_key.argtypes = [ctypes.c_uint32]
    lib.fwo_tp_threshold.restype = ctypes.c_uint32
    lib.fwo_tp_threshold.argtypes = [ctypes.c_double]
    for i in range(n):
        ref = O.philox([int(x) for x in words[i, :4]], [int(x) for x in words[i, 4:]])
        assert out[i, :4].tolist() == ref, i
        assert out[i, 4:8].tolist() == ref, i  # round keys formed ahead of time: the same block
        e = np.float32(lib.fwo_exp_key(ref[0]))
        assert int(out[i, 8]) == int(e.view(np.uint32)), (i, ref[0])
        assert int(out[i, 9]) == lib.fwo_tp_threshold(float(tps[i])), (i, tps[i])

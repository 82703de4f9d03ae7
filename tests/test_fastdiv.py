"""Host check of the multiply-high division the kernels use to turn a pixel index into
(image, row, column): FastDiv::host_div applies the same multiplier and shift as the device
method, so checking it against `/` on the CPU checks the constants the kernels receive."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INC = "/usr/local/cuda/include"

SRC = r"""
#include <cstdio>
#include <cstdlib>
#include "common.cuh"
int main() {
  unsigned long long bad = 0, cnt = 0;
  const unsigned ds[] = {1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 29, 57, 58, 841, 3249, 3306, 65535, 65536, 65537,
                         1000003, (1u << 30) - 1, 1u << 30, (1u << 30) + 1, 0x7fffffffu};
  for (unsigned d : ds) {
    const b200::FastDiv f(d);
    for (unsigned long long n = 0; n < (1ull << 31); n += 4099) { ++cnt; bad += f.host_div((unsigned)n) != n / d; }
    for (unsigned long long n = (1ull << 31) - 3000; n < (1ull << 31); ++n) { ++cnt; bad += f.host_div((unsigned)n) != n / d; }
    for (unsigned long long k = 1; k < 2000 && k * d < (1ull << 31); ++k)
      for (int e = -1; e <= 1; ++e) {
        const unsigned long long n = k * d + e;
        if (n < (1ull << 31)) { ++cnt; bad += f.host_div((unsigned)n) != n / d; }
      }
  }
  srand(7);
  for (int i = 0; i < 2000000; ++i) {
    const unsigned d = (unsigned)rand() % 200000 + 1;
    const unsigned n = (((unsigned)rand() << 16) ^ (unsigned)rand()) & 0x7fffffffu;
    ++cnt; bad += b200::FastDiv(d).host_div(n) != n / d;
  }
  printf("%llu %llu\n", cnt, bad);
  return bad != 0;
}
"""


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC), reason="needs g++ and the CUDA headers")
def test_fastdiv_matches_integer_division(tmp_path):
    src = tmp_path / "fastdiv_check.cpp"
    src.write_text(SRC)
    exe = tmp_path / "fastdiv_check"
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([gxx, "-O2", "-std=c++17", "-x", "c++", str(src), "-o", str(exe),
                           "-I", os.path.join(ROOT, "pytorch-vulkan_b200", "csrc"), "-I", os.path.join(ROOT, "include"),
                           "-I", CUDA_INC])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    checked, bad = map(int, out.stdout.split())
    assert checked > 10_000_000 and bad == 0

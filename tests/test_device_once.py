"""The once-per-device set-up guard (csrc/device_once.h) that keeps per-device CUDA settings (a kernel's shared-memory ceiling,
a symbol's device address) from being made on the first device only.  Plain C++: compiled and run here without a GPU."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <cstdio>
#include <thread>
#include <vector>
#include "device_once.h"
int main() {
  p0p::DeviceOnce once;
  int calls[4] = {0, 0, 0, 0};
  // every device gets its own set-up, once
  for (int rep = 0; rep < 3; rep++)
    for (int d = 0; d < 4; d++)
      if (once.run(d, [&] { calls[d]++; return 0; }) != 0) return 1;
  for (int d = 0; d < 4; d++) if (calls[d] != 1 || !once.done(d)) return 2;
  // a failed set-up is reported and tried again on the next call
  p0p::DeviceOnce flaky; int tries = 0;
  if (flaky.run(1, [&] { tries++; return 7; }) != 7 || flaky.done(1)) return 3;
  if (flaky.run(1, [&] { tries++; return 0; }) != 0 || !flaky.done(1) || tries != 2) return 4;
  if (flaky.run(1, [&] { tries++; return 9; }) != 0 || tries != 2) return 5;
  // ordinals outside the table are refused, not indexed
  if (once.run(-1, [] { return 0; }) != -1 || once.run(p0p::DeviceOnce::kMaxDevices, [] { return 0; }) != -1 || once.done(999)) return 6;
  // concurrent first calls for one device: exactly one set-up
  p0p::DeviceOnce shared; int n = 0;
  std::vector<std::thread> th;
  for (int i = 0; i < 16; i++) th.emplace_back([&] { shared.run(5, [&] { n++; return 0; }); });
  for (auto& t : th) t.join();
  if (n != 1) return 7;
  std::puts("ok");
  return 0;
}
'''


def test_device_once_guard(tmp_path):
    src = tmp_path / "once.cpp"; exe = tmp_path / "once"
    src.write_text(PROGRAM)
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(ROOT, "p0pc0rn_kernels_b200", "csrc"), str(src), "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ok", (r.returncode, r.stdout, r.stderr)

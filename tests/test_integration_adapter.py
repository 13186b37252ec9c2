"""The reference-side adapter (see_ai_b200/integration/cuda_backend_adapter.cc) compiles against the
reference's own seam header (runtime/executor/backend.h:82-166) and links with the library.

Needs the reference tree for its header, so it is skipped where the tree is absent."""
import os
import shutil
import subprocess

import pytest

from see_ai_b200 import build as see_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("SEE_REFERENCE_TREE", "/root/reference")
ADAPTER = os.path.join(ROOT, "see_ai_b200", "integration", "cuda_backend_adapter.cc")

MAIN = r"""
#include "runtime/executor/backend.h"
#include <cstdio>
namespace seeml::update_rt {
std::expected<std::unique_ptr<ExecutorBackend>, std::string> CreateCudaBackend(int);
}
int main() {
  auto made = seeml::update_rt::CreateCudaBackend(0);
  if (!made) { std::printf("refused: %s\n", made.error().c_str()); return 3; }
  seeml::update_rt::ExecutorBackend& be = **made;
  std::printf("made: %s on %s relaxed=%llu fused=%llu\n", be.name(), be.device().c_str(),
              (unsigned long long)be.relaxed_executions(), (unsigned long long)be.fused_dispatches());
  return be.Flush() ? 0 : 4;
}
"""


@pytest.mark.skipif(not os.path.isfile(os.path.join(REFERENCE, "runtime/executor/backend.h")),
                    reason="the reference tree's seam header is not on this machine")
@pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")
def test_adapter_compiles_against_the_reference_seam_and_links(tmp_path):
    see_build.build()
    lib_dir = os.path.join(ROOT, "see_ai_b200")
    main_cc = tmp_path / "main.cc"
    main_cc.write_text(MAIN)
    exe = tmp_path / "adapter_check"
    cmd = ["g++", "-std=c++23", "-Wall", "-Wextra", "-Werror", "-I", REFERENCE, "-I", os.path.join(ROOT, "include"),
           ADAPTER, str(main_cc), "-L", lib_dir, "-lsee_cuda", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-4000:]
    ran = subprocess.run([str(exe)], capture_output=True, text=True)
    # With no device the library refuses to create a backend (no CPU fallback); with one it is made and flushes.
    if ran.returncode == 3:
        assert "no CPU fallback" in ran.stdout
    else:
        assert ran.returncode == 0 and ran.stdout.startswith("made: cuda on "), ran.stdout + ran.stderr

"""The C++ host adapters (tair-kvcache_b200/host/kvcm_b200_host.h), driven by a C++ program that replays the
reference's own C++ test tables the way those tests call MetaSearcher / CacheManager."""
import os
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_cpp_host_adapter_program():
    binary = os.path.join(ROOT, "tests", "cpp", "host_adapter_test.bin")
    if not os.path.exists(binary):
        import __graft_entry__ as entry
        entry._load_build_module().build_host_adapter_test()
    proc = subprocess.run([binary], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout
    assert "all checks passed" in proc.stdout

"""Sleep-mode allocator bookkeeping on CPU, against a stand-in for the driver's virtual-memory API (tests/fake_cuda_driver.cpp)."""
import ctypes
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _build(tmp_path):
    fake = str(tmp_path / "libfakecuda.so")
    subprocess.run(["g++", "-O1", "-std=c++17", "-fPIC", "-shared", os.path.join(HERE, "fake_cuda_driver.cpp"), "-o", fake], check=True)
    import importlib.util
    spec = importlib.util.spec_from_file_location("_cumem_build", os.path.join(ROOT, "1cat-vllm_b200", "csrc", "cumem", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return fake, mod.build()


_CHILD = r'''
import ctypes, os, sys
from onecat_vllm.utils.cumem import CuMemAllocator
fake = ctypes.CDLL(os.environ["ONECAT_CUMEM_DRIVER"], mode=ctypes.RTLD_GLOBAL)
fake.fake_live_phys_bytes.restype = ctypes.c_longlong
fake.cuMemcpyHtoD_v2.argtypes = [ctypes.c_ulonglong, ctypes.c_char_p, ctypes.c_size_t]
fake.cuMemcpyDtoH_v2.argtypes = [ctypes.c_char_p, ctypes.c_ulonglong, ctypes.c_size_t]
a = CuMemAllocator.get()
a.set_tag("weights"); w = a.malloc(3 << 20)          # rounded up to the 2 MiB granularity: 4 MiB
a.set_tag("kv_cache"); kv = a.malloc(1 << 20)
a.set_tag("default"); other = a.malloc(100)
assert a.stats()["mapped_bytes"] == (4 << 20) + (2 << 20) + (2 << 20) and a.stats()["allocations"] == 3
assert fake.cuMemcpyHtoD_v2(w, b"weights!" * 4, 32) == 0 and fake.cuMemcpyHtoD_v2(kv, b"kvkvkvkv", 8) == 0 and fake.cuMemcpyHtoD_v2(other, b"keepme", 6) == 0
freed = a.sleep(offload_tags=("weights",), discard_tags=("kv_cache",))
assert freed == 6 << 20, freed
s = a.stats()
assert s["asleep_bytes"] == 6 << 20 and s["host_backup_bytes"] == 4 << 20 and s["mapped_bytes"] == 2 << 20
assert fake.fake_live_phys_bytes() == 2 << 20            # the physical memory really went back
buf = ctypes.create_string_buffer(32)
assert fake.cuMemcpyDtoH_v2(buf, w, 32) == 700            # nothing is mapped under a sleeping allocation
assert fake.cuMemcpyDtoH_v2(buf, other, 6) == 0 and buf.raw[:6] == b"keepme"
assert a.sleep(("weights",), ("kv_cache",)) == 0          # sleeping twice releases nothing more
assert a.wake_up(("weights",)) == 4 << 20                 # pools wake separately, at the same addresses
assert fake.cuMemcpyDtoH_v2(buf, w, 32) == 0 and buf.raw == b"weights!" * 4
assert a.stats(("kv_cache",))["asleep_bytes"] == 2 << 20
assert a.wake_up() == 2 << 20
assert fake.cuMemcpyDtoH_v2(buf, kv, 8) == 0 and buf.raw[:8] != b"kvkvkvkv"   # a discarded pool comes back uninitialised
assert a.stats()["host_backup_bytes"] == 0 and a.stats()["asleep_bytes"] == 0
a.free(w); a.free(kv); a.free(other)
assert a.stats()["allocations"] == 0 and fake.fake_live_phys_bytes() == 0
print("OK")
'''


@pytest.mark.timeout(120)
def test_sleep_and_wake_release_and_restore_tagged_pools(tmp_path):
    fake, so = _build(tmp_path)
    assert os.path.exists(so)
    env = dict(os.environ, ONECAT_CUMEM_DRIVER=fake, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", _CHILD], env=env, capture_output=True, text=True, timeout=100)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr


def test_missing_driver_is_reported(tmp_path):
    _, so = _build(tmp_path)
    env = dict(os.environ, ONECAT_CUMEM_DRIVER=str(tmp_path / "nope.so"), PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    code = ("from onecat_vllm.utils.cumem import CuMemAllocator\na = CuMemAllocator.get()\n"
            "try:\n    a.malloc(10)\n    print('allocated')\nexcept MemoryError as e:\n    print('ERR', e)\n")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=100)
    assert "ERR cannot load the CUDA driver" in r.stdout, r.stdout + r.stderr

"""The best-fit dynamic memory pool: placement, splitting, merging, stream rules, limit and statistics on the C heap;
and (GPU) the same pool installed as the CUDA allocator of a fresh process."""
import os
import subprocess
import sys

import pytest

from mindspore_b200.utils.memory_pool import BestFitPool

KB = 1024


def test_best_fit_split_and_merge():
    pool = BestFitPool(block_size=64 * KB)
    a = pool.alloc(10 * KB)
    b = pool.alloc(20 * KB)
    c = pool.alloc(8 * KB)
    assert b == a + 10 * KB and c == b + 20 * KB            # cut from one block, in order
    st = pool.stats()
    assert st["blocks"] == 1 and st["reserved"] == 64 * KB and st["used"] == 38 * KB
    pool.free(b)                                             # a 20 KB hole and the 26 KB tail are idle
    d = pool.alloc(19 * KB)                                  # best fit: the hole, not the tail
    assert d == b
    e = pool.alloc(512)                                      # the 1 KB rest of the hole is the smallest fit
    assert e == b + 19 * KB
    pool.free(d)
    pool.free(e)
    pool.free(a)                                             # a + (d, e) merge into one 30 KB idle buffer
    assert pool.stats()["largest_idle"] == 30 * KB
    pool.free(c)                                             # and with c and the tail into the whole block
    st = pool.stats()
    assert st["used"] == 0 and st["idle_bufs"] == 1 and st["largest_idle"] == 64 * KB
    assert st["peak_used"] == 38 * KB
    assert pool.release_idle() == 64 * KB and pool.stats()["reserved"] == 0
    with pytest.raises(ValueError):
        pool.free(a)                                         # not a live buffer any more
    pool.close()


def test_requests_are_rounded_and_big_requests_get_their_own_block():
    pool = BestFitPool(block_size=16 * KB)
    a = pool.alloc(1)
    b = pool.alloc(1)
    assert b - a == 512
    big = pool.alloc(100 * KB)
    st = pool.stats()
    assert st["blocks"] == 2 and st["reserved"] == 116 * KB
    pool.free(big)
    assert pool.release_idle() == 100 * KB                   # only the block without live buffers goes back
    pool.close()


def test_limit_is_enforced():
    pool = BestFitPool(block_size=32 * KB, max_size=48 * KB)
    a = pool.alloc(30 * KB)
    b = pool.alloc(14 * KB)                                  # a full second block would pass the limit: exact size
    assert pool.stats()["reserved"] == 46 * KB
    with pytest.raises(MemoryError):
        pool.alloc(4 * KB)
    pool.free(a)
    pool.alloc(28 * KB)                                      # reuse, no growth
    assert pool.stats()["reserved"] == 46 * KB
    pool.free(b)
    pool.close()


def test_cross_stream_reuse_waits_for_synchronisation():
    pool = BestFitPool(block_size=16 * KB)
    a = pool.alloc(16 * KB, stream=1)
    pool.free(a)
    assert pool.alloc(16 * KB, stream=1) == a                # same stream: ordered, reuse at once
    pool.free(a)
    other = pool.alloc(16 * KB, stream=2)                    # another stream may not take it yet: a new block
    assert other != a and pool.stats()["blocks"] == 2
    pool.free(other)
    pool.mark_synchronized()                                 # the device finished everything: all idle is free for all
    assert pool.alloc(16 * KB, stream=3) in (a, other)
    assert pool.stats()["blocks"] == 2
    pool.close()


_GPU_SCRIPT = r"""
import torch
import mindspore_b200 as ms
from mindspore_b200.utils import memory_pool as MP
ms.set_context(device_target="GPU", mempool_block_size="256MB", max_device_memory="8GB")
MP.enable_device_pool()
x = torch.randn(4096, 4096, device="cuda")
y = x @ x
z = torch.empty(1 << 30, dtype=torch.uint8, device="cuda")      # larger than a block: gets a block of its own
st = MP.device_pool_stats()
assert st["used"] >= 2 * 64 * 2 ** 20 + (1 << 30) and st["reserved"] >= st["used"] and st["blocks"] >= 2, st
ref = float((x.cpu() @ x.cpu())[0, 0])
assert abs(float(y[0, 0]) - ref) <= 1e-2 * max(1.0, abs(ref))
del x, y, z
st2 = MP.device_pool_stats()
assert st2["used"] < st["used"], (st, st2)
freed = MP.device_pool_release_idle()      # the block of z has no live buffer left (library workspaces live elsewhere)
assert freed >= 1 << 30 and MP.device_pool_stats()["reserved"] <= st["reserved"] - (1 << 30), (freed, st)
try:
    torch.empty(9 << 30, dtype=torch.uint8, device="cuda")
except (MemoryError, RuntimeError) as e:
    print("limit ok", type(e).__name__, str(e)[:60])
else:
    raise SystemExit("the 8 GB limit was not enforced")
print("pool ok", st)
"""


@pytest.mark.gpu
def test_pool_as_the_cuda_allocator():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _GPU_SCRIPT], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "pool ok" in r.stdout and "limit ok" in r.stdout, r.stdout + r.stderr

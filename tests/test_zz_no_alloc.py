"""GPU: the entry point for callers that may not allocate device memory (b200_oft_tn_f16_static).

Such callers - a process that gave all device memory to its own pool at start-up, or a request loop
that cannot afford the device-wide synchronisation of cudaMalloc - get the same fused product with the
kernel's scratch held in a fixed array inside the library.  The test drives it through the C ABI twice
in a row, with different operands and a different block edge the second time (the array is shared and
keeps the first call's contents), and requires the bits of the ordinary entry point each time.
Collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from _util import make_oft_case
from cute_mma_b200 import ops

pytestmark = pytest.mark.gpu


def _both(lib, cuda, m, n, k, b, seed, group_size=None):
    """(result of the ordinary entry point on the route that needs no X.R scratch, result of the static one)."""
    import torch

    A, R, B = make_oft_case(m, n, k, b, group_size, seed=seed)
    dA, dB, dR = (torch.from_numpy(x).to(cuda) for x in (A, B, R))
    want = torch.full((m, n), -3.0, dtype=torch.float16, device=cuda)
    got = torch.full((m, n), -5.0, dtype=torch.float16, device=cuda)
    with ops.option("oft_route", 1, lib):
        ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, want, n, group_size=group_size, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    ops.oft_tn_static(m, n, k, dA, k, dB, k, dR, k, got, n, group_size=group_size, reconn_sz=b, lib=lib)
    assert ops.static_status(lib)[0] == 0   # synchronises; the record of a wait that ran out would show here
    return want.cpu().numpy(), got.cpu().numpy()


def test_static_scratch_entry_point_matches_the_allocating_one_twice(lib, cuda):
    want1, got1 = _both(lib, cuda, 384, 512, 512, 64, seed=21)
    assert np.array_equal(want1.view(np.uint16), got1.view(np.uint16))
    want2, got2 = _both(lib, cuda, 200, 768, 256, 32, seed=22, group_size=256)  # second call: other shape, other b
    assert np.array_equal(want2.view(np.uint16), got2.view(np.uint16))
    assert not np.array_equal(want1[:200, :512], want2[:, :512])  # the two calls really computed different things


def test_static_scratch_entry_point_validates_like_the_other(lib, cuda):
    import torch

    d = torch.zeros(64 * 64, dtype=torch.float16, device=cuda)
    with pytest.raises(ops.Error) as e:
        ops.oft_tn_static(64, 64, 60, d, 64, d, 64, d, 64, d, 64, reconn_sz=16, lib=lib)  # k not a multiple of b
    assert e.value.code == ops.EINVAL
    with pytest.raises(ops.Error) as e:
        ops.oft_tn_static(64, 64, 48, d, 64, d, 64, d, 64, d, 64, reconn_sz=24, lib=lib)  # block edge not built
    assert e.value.code == ops.EUNSUPPORTED


def test_static_scratch_entry_point_small_blocks_and_its_size_limit(lib, cuda):
    """8 x 8 blocks need an expanded copy of R as scratch: it fits the library's array for a small K and
    is refused, with both sizes in the message, when it does not."""
    want, got = _both(lib, cuda, 256, 512, 512, 8, seed=23)   # 16 rows x 512 columns of fp16 = 16 KB of scratch beside the record
    assert np.array_equal(want.view(np.uint16), got.view(np.uint16))
    import torch

    d = torch.zeros(64 * 4096, dtype=torch.float16, device=cuda)
    with pytest.raises(ops.Error) as e:
        ops.oft_tn_static(64, 64, 4096, d, 4096, d, 4096, d, 4096, d, 64, reconn_sz=8, lib=lib)  # 128 KB needed
    assert e.value.code == ops.EUNSUPPORTED and "65536" in e.value.message


def test_static_scratch_entry_point_allocates_no_device_memory(lib, cuda):
    """Free device memory as the driver reports it (cudaMemGetInfo) is the same before and after static calls that
    follow the first one on this device (which only looks up the array's address), also when the kernel uses the
    tile-round counters in the array (option tile_sync) and for 8 x 8 blocks, whose expanded R lives in the array."""
    import torch

    m, n, k = 512, 1024, 256
    A, R, B = make_oft_case(m, n, k, 64, seed=61)
    A8, R8, B8 = make_oft_case(m, n, k, 8, seed=62)
    dA, dB, dR, dA8, dB8, dR8 = (torch.from_numpy(x).to(cuda) for x in (A, B, R, A8, B8, R8))
    dC = torch.empty((m, n), dtype=torch.float16, device=cuda)
    want = torch.empty((m, n), dtype=torch.float16, device=cuda)
    ops.oft_tn_static(m, n, k, dA, k, dB, k, dR, k, dC, n, reconn_sz=64, lib=lib)   # first call on the device, if none came before
    assert ops.static_status(lib)[0] == 0
    free0, _ = torch.cuda.mem_get_info(cuda)
    ops.oft_tn_static(m, n, k, dA, k, dB, k, dR, k, dC, n, reconn_sz=64, lib=lib)
    with ops.option("tile_sync", 1, lib):
        ops.oft_tn_static(m, n, k, dA, k, dB, k, dR, k, dC, n, reconn_sz=64, lib=lib)
    assert ops.static_status(lib)[0] == 0
    out64 = dC.clone()
    ops.oft_tn_static(m, n, k, dA8, k, dB8, k, dR8, k, dC, n, reconn_sz=8, lib=lib)
    assert ops.static_status(lib)[0] == 0
    free1, _ = torch.cuda.mem_get_info(cuda)
    assert free1 == free0, (free0, free1)
    with ops.option("oft_route", 1, lib):
        ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, want, n, reconn_sz=64, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(out64.view(torch.int16), want.view(torch.int16))


_FRESH = """
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import numpy as np, torch
from _util import make_oft_case, oft_ok
from cute_mma_b200 import ops
from oracle import oracle
lib = ops.load_library()
dev = torch.device("cuda:0"); torch.cuda.set_device(0)
m, n, k, b = 256, 512, 256, 32
A, R, B = make_oft_case(m, n, k, b, seed=71)
dA, dB, dR = (torch.from_numpy(x).to(dev) for x in (A, B, R))
dC = torch.empty((m, n), dtype=torch.float16, device=dev)
ops.oft_tn_static(m, n, k, dA, k, dB, k, dR, k, dC, n, reconn_sz=b, lib=lib)   # the library's very first call in this process
assert ops.static_status(lib) == [0, 0, 0, 0]
ref = oracle.cpu_oft_tn(A, R, B, m, n, 1, k, b, threads=2)
assert oft_ok(dC.cpu().numpy(), ref, truth=oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=True))[0] == 0
print("fresh-process static call ok")
"""


def test_static_scratch_entry_point_first_in_a_fresh_process(lib, cuda):
    """In a process of its own the static entry point is the first thing the library runs (its own set-up path:
    symbol address, device attributes, the driver's tensor-map entry point), checked against the oracle."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = _FRESH.format(root=root, tests=os.path.join(root, "tests"))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "fresh-process static call ok" in res.stdout, res.stdout + res.stderr

"""GPU: the entry point for callers that may not allocate device memory (b200_oft_tn_f16_static).

Such callers - a process that gave all device memory to its own pool at start-up, or a request loop
that cannot afford the device-wide synchronisation of cudaMalloc - get the same fused product with the
kernel's scratch held in a fixed array inside the library.  The test drives it through the C ABI twice
in a row, with different operands and a different block edge the second time (the array is shared and
keeps the first call's contents), and requires the bits of the ordinary entry point each time.
Collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import numpy as np
import pytest

from _util import make_oft_case
from cute_mma_b200 import ops

pytestmark = pytest.mark.gpu


def _both(lib, cuda, m, n, k, b, seed, group_size=None):
    import torch

    A, R, B = make_oft_case(m, n, k, b, group_size, seed=seed)
    dA, dB, dR = (torch.from_numpy(x).to(cuda) for x in (A, B, R))
    want = torch.full((m, n), -3.0, dtype=torch.float16, device=cuda)
    got = torch.full((m, n), -5.0, dtype=torch.float16, device=cuda)
    ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, want, n, group_size=group_size, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    ops.oft_tn_static(m, n, k, dA, k, dB, k, dR, k, got, n, group_size=group_size, reconn_sz=b, lib=lib)
    torch.cuda.synchronize()
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

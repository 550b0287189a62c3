"""GPU test of the bounded waits inside the tensor-core kernel.

Every wait on an mbarrier in the kernel has a wall-clock limit.  Here the limit
is made short (100 ms) and the launch descriptor's self-test bit
(SM120_TUNE_STALL_KBLOCK) makes every TMA producer stop
before one k-block of its first tile, so the MMA role's wait for that k-block
runs out.  The kernel must then return normally (no trap, no fault, no hang),
report a non-zero status word, and leave the device usable: the next, ordinary
launch is checked against the oracle.  Both kernel flavours are exercised."""
import ctypes
import time

import numpy as np
import pytest
import torch

from oracle import reference as ref
from tests import _util as U

pytestmark = pytest.mark.gpu


def _status(lib, clear):
    st = ctypes.c_uint(0)
    assert lib.sm120_get_kernel_status(0, ctypes.byref(st), int(clear)) == 0
    return st.value


@pytest.mark.parametrize("cta_group", [1, 2])
def test_wait_limit_reports_status_and_device_survives(ops, binding, cta_group):
    lib = binding.load_library()
    rng = np.random.default_rng(5)
    M, N, K = 512, 512, 256                       # 4 k-blocks of 64
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, True, "bfloat16", scale=0.3)
    ta, tb = U.to_cuda(a), U.to_cuda(b)
    want = ref.matmul_oracle(a, b, transpose_b=True, out_dtype="bfloat16")
    assert _status(lib, clear=True) == 0
    flavour = binding.TUNE_CTA_GROUP_2 if cta_group == 2 else binding.TUNE_CTA_GROUP_1
    try:
        lib.sm120_set_wait_limit_ms(100)
        t0 = time.perf_counter()
        # k-block 1 of every CTA's first tile never arrives; the result is meaningless, the call must only return
        ops.fused_matmul(ta, tb, transpose_b=True, tuning=flavour | binding.tune_stall_kblock(1))
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        lib.sm120_set_wait_limit_ms(2000)
    assert binding.last_kernel_name().startswith("tc_bf16_2cta" if cta_group == 2 else "tc_bf16_128")
    assert 0.05 < elapsed < 5.0, elapsed          # gave up after the limit, not instantly and not never
    status = _status(lib, clear=True)
    assert status != 0
    assert (status >> 28) in (1, 2, 3)            # role that gave up first: producer, MMA or epilogue
    assert _status(lib, clear=False) == 0         # the read above cleared it
    got = ops.fused_matmul(ta, tb, transpose_b=True, tuning=flavour)   # same flavour, no stall: a normal launch
    torch.cuda.synchronize()
    assert ref.rel_frobenius(U.to_numpy(got), want) <= ref.TOLERANCE["bfloat16"]
    assert _status(lib, clear=False) == 0

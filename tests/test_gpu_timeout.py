"""The bounded pipeline waits of the tensor-core kernels, made to run out on purpose.

Every mbarrier wait in conv_ts_kernel / tc_gemm_kernel gives up after a cycle limit, records a status word, and the
kernel unwinds: the other warps' waits run out too, tensor memory is released, the launch returns.  The reference's own
bounded waits return VLE_Timeout (matlab/src/vl_tmove.cu:1344-1359); so does vlb_ctx_device_status here.  The test makes
a wait run out the harmless way: the warp that would fetch the filter tiles stays idle (a test switch of the context), so
the barrier behind it is never completed -- nothing traps, faults or spins without bound -- and the limit is lowered to
about a millisecond so that the launch returns at once.
"""
import numpy as np
import pytest

from conftest import bit_equal

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_returns_timeout_and_the_next_call_is_correct(gpu):
    from matconvnet_b200 import capi
    nn, mat, ctx = gpu
    rng = np.random.default_rng(21)
    x = mat.from_numpy(rng.standard_normal((16, 16, 32, 4)).astype(np.float32))
    f = mat.from_numpy((rng.standard_normal((3, 3, 32, 64)) * 0.1).astype(np.float32))
    b = mat.from_numpy(rng.standard_normal(64).astype(np.float32))
    want = mat.to_numpy(nn.vl_nnconv(x, f, b, pad=1, ctx=ctx))
    assert ctx.device_status() == 0
    lib = ctx.lib
    ctx.check(lib.vlb_ctx_set_wait_limit(ctx.handle, 2_000_000))
    ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 1))
    try:
        nn.vl_nnconv(x, f, b, pad=1, ctx=ctx)              # the launch itself succeeds; its result is undefined
        with pytest.raises(capi.VlbError) as err:
            ctx.device_status()
        assert err.value.code == capi.ERROR_NAMES.index("VLE_Timeout")
    finally:
        ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 0))
        ctx.check(lib.vlb_ctx_set_wait_limit(ctx.handle, 0))
    assert ctx.device_status() == 0                        # the word was cleared by the failed query
    got = mat.to_numpy(nn.vl_nnconv(x, f, b, pad=1, ctx=ctx))
    assert ctx.device_status() == 0
    assert bit_equal(got, want)

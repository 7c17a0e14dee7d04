"""The allocation-free RMSNorm backward (seraph_b200_rmsnorm_backward_static).

Who needs it: a host that may not call the CUDA allocator at the point where it
runs this op - a capture is open on another stream of the process, the
embedding framework bans cudaMalloc after start-up, or all device memory is
handed out by the embedder.  The regular entry point grows a scratch buffer on
demand; this one keeps the per-CTA partial sums of the scale gradient in a
fixed array inside the library.

The test calls it through the C ABI with raw device pointers, twice in a row
(the array keeps the first call's contents when the second starts), and holds
both results against cuda_train_rmsnorm_backward_batch on the same inputs.
Collected last so that a run stopping at the first failure has already run
everything else; it also passes alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev_ptr(buf):
    return C.c_void_p(buf.b.contents.data)


def ctx_stream(ctx):
    # cuda_train_context_t: int device_id, then void* stream at offset 8
    return C.c_void_p(C.c_void_p.from_address(ctx.h + 8).value)


@pytest.mark.parametrize("rows,cols", [(300, 512), (77, 2048), (1000, 8192), (5, 100)])
def test_static_scratch_matches_regular_entry_point(rows, cols):
    from seraph_b200 import api
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    ds0 = rng.standard_normal(cols).astype(np.float32)
    with api.Context(0) as ctx:
        bx, bw = ctx.upload(x), ctx.upload(w)
        for call in range(2):                       # two calls in a row, different gradients each time
            dy = rng.standard_normal((rows, cols)).astype(np.float32)
            bdy = ctx.upload(dy)
            ref_dx, ref_ds = ctx.empty(x.size), ctx.upload(ds0)
            ctx.lib.cuda_train_rmsnorm_backward_batch(ctx.h, bx.b, bw.b, bdy.b, ref_dx.b, ref_ds.b, rows, cols, 1e-5)
            new_dx, new_ds = ctx.empty(x.size), ctx.upload(ds0)
            rc = ctx.lib.seraph_b200_rmsnorm_backward_static(dev_ptr(bx), dev_ptr(bw), dev_ptr(bdy), dev_ptr(new_dx), dev_ptr(new_ds),
                                                             rows, cols, 1e-5, ctx_stream(ctx))
            assert rc == 0
            ctx.sync()
            ctx.check()
            a_dx, a_ds, b_dx, b_ds = ref_dx.numpy(), ref_ds.numpy(), new_dx.numpy(), new_ds.numpy()
            # same arithmetic, summation order may differ between the two entry points: the op tests' tolerance applies
            assert np.linalg.norm(b_dx - a_dx) <= 1e-5 * np.linalg.norm(a_dx), call
            assert np.linalg.norm(b_ds - a_ds) <= 1e-5 * np.linalg.norm(a_ds), call
            ctx.release(bdy, ref_dx, ref_ds, new_dx, new_ds)


def test_static_scratch_rejects_rows_wider_than_its_array():
    from seraph_b200 import api
    with api.Context(0) as ctx:
        b = ctx.zeros(16)
        p = dev_ptr(b)
        assert ctx.lib.seraph_b200_rmsnorm_backward_static(p, p, p, p, p, 1, 8193, 1e-5, None) == 7
        assert ctx.lib.seraph_b200_rmsnorm_backward_static(None, p, p, p, p, 1, 16, 1e-5, None) == 1

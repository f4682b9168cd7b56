"""sk_column_sums_static: the column sums for callers that must not allocate device memory
(a framework owns their device heap, or they hold only raw pointers and a stream and cannot
create a context). It keeps its partial sums in an array built into the library, so this test
calls it through the C ABI with nothing but pointers and a stream, twice in a row (the array
is reused and keeps the previous call's contents), and checks each result against the column
sums the context entry point sk_backward_grads produces for the same tensors.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SK_ERR_STATIC_LIMIT = 12


def _block(ctx, k, n, batch, norm):
    import soklyn_b200 as sk
    from soklyn_b200.configs import _GivenWeights
    rng = np.random.default_rng(11 + n)
    w = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
    cfg = sk.LayerInitConfig(norm, sk.Activation.Tanh, sk.Regularisation.none(), 0.0)
    return sk.DenseBlock(ctx, True, k, n, batch, _GivenWeights(w), cfg, sk.Precision.FP32)


@pytest.mark.parametrize("k,n,batch,norm_name", [(24, 40, 50, "LayerNorm"), (16, 1000, 333, "RMSNorm"), (8, 7, 9, "Disabled")])
def test_static_column_sums_match_context_path_twice(gpu_ctx, k, n, batch, norm_name):
    import torch
    import soklyn_b200 as sk
    from soklyn_b200 import _native
    lib = _native.lib()
    norm = getattr(sk.Normalisation, norm_name)
    blk = _block(gpu_ctx, k, n, batch, norm)
    dev = gpu_ctx.device
    stream = C.c_void_p(gpu_ctx.stream.cuda_stream)
    x = sk.Tensor.from_cpu_vector(gpu_ctx, np.random.default_rng(1).standard_normal((batch, k)).astype(np.float32), (batch, k))
    for call in range(2):   # two calls in a row, with different gradients each time
        g = torch.Generator(device="cpu").manual_seed(100 + call)
        for t in (blk.get_delta_prenorm_out(), blk.get_norm_weights_grad(), blk.get_norm_biases_grad()):
            t.data.copy_(torch.randn(t.data.shape, generator=g) * (call + 1))
        dw = torch.empty(k, n, device=dev)
        want = torch.empty(3, n, device=dev)
        gpu_ctx.gpu_backward_grads(blk, x, batch, dw, want)
        got = torch.full((3, n), float("nan"), device=dev)
        rc = lib.sk_column_sums_static(stream, blk.get_delta_prenorm_out().ptr(), blk.get_norm_weights_grad().ptr(),
                                       blk.get_norm_biases_grad().ptr(), got.data_ptr(), batch, n, norm.ordinal())
        assert rc == 0
        gpu_ctx.synchronize()
        a, b = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(a).all()
        scale = max(np.abs(b).max(), 1e-30)
        assert np.abs(a - b).max() / scale <= 1e-5   # the f32 tolerance of the parity tests
        # all three rows against float64 column sums taken on the host
        tensors = (blk.get_delta_prenorm_out(), blk.get_norm_weights_grad(), blk.get_norm_biases_grad())
        for row, t in enumerate(tensors[: 1 + min(norm.ordinal(), 2)]):
            ref = t.download(gpu_ctx)[:batch].astype(np.float64).sum(0)
            assert np.abs(a[row] - ref).max() / max(np.abs(ref).max(), 1e-30) <= 1e-5, f"sum {row}"


@pytest.mark.parametrize("n,batch", [(262144, 8), (200000, 40)])
def test_static_column_sums_at_the_limit_of_the_array(gpu_ctx, n, batch):
    """The widest N the built-in array can hold (one slab of partial sums fills it), and a width just below
    it with more rows than one slab covers: two calls in a row against float64 sums taken on the host."""
    import torch
    from soklyn_b200 import _native
    lib = _native.lib()
    dev = gpu_ctx.device
    stream = C.c_void_p(gpu_ctx.stream.cuda_stream)
    for call in range(2):
        g = torch.Generator(device="cpu").manual_seed(7 + call)
        host = [torch.randn(batch, n, generator=g) * (call + 1) for _ in range(3)]
        devs = [h.to(dev) for h in host]
        got = torch.full((3, n), float("nan"), device=dev)
        rc = lib.sk_column_sums_static(stream, devs[0].data_ptr(), devs[1].data_ptr(), devs[2].data_ptr(), got.data_ptr(),
                                       batch, n, 2)
        assert rc == 0
        gpu_ctx.synchronize()
        a = got.cpu().numpy()
        for row in range(3):
            ref = host[row].double().sum(0).numpy()
            assert np.abs(a[row] - ref).max() / max(np.abs(ref).max(), 1e-30) <= 1e-5, f"call {call} sum {row}"


def test_static_column_sums_reject_sizes_beyond_the_array():
    from soklyn_b200 import _native
    lib = _native.lib()
    dummy = C.c_void_p(256)   # never dereferenced: the size check comes first
    assert lib.sk_column_sums_static(None, dummy, dummy, dummy, dummy, 8, 262145, 2) == SK_ERR_STATIC_LIMIT
    assert lib.sk_column_sums_static(None, None, None, None, dummy, 8, 16, 0) == 9
    assert b"262144" in lib.sk_status_string(SK_ERR_STATIC_LIMIT)

"""The weight-streaming linear kernel of decode steps against an fp32 matrix product of the same bf16
operands (the reference's Linear operator is y = x W^T in the activations' dtype with fp32 accumulation
inside its GEMM back ends, pace/ops/backends/tpp.py:19-63)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _want(x, w):
    return (x.float() @ w.float().t())


@pytest.mark.parametrize("M,N,K", [(32, 4096, 4096), (32, 6144, 4096), (32, 28672, 4096), (32, 4096, 14336),
                                   (1, 128, 128), (7, 256, 384), (32, 128256, 4096), (19, 1024, 2048)])
def test_linear_matches_fp32_product(M, N, K):
    from pace_b200.ops.linear import linear_skinny as linear
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16().to(DEV)
    for call in range(2):                      # the second call finds the workspace as the first one left it
        y = linear(x, w)
        assert y.shape == (M, N) and y.dtype == torch.bfloat16
        want = _want(x, w)
        err = (y.float() - want).abs()
        # one rounding to bf16 of a value of magnitude |want|: relative 2^-8
        tol = want.abs() * 2.0 ** -7 + 1e-3
        assert bool((err <= tol).all()), (call, err.max().item(), (err - tol).max().item())
    torch.cuda.synchronize()


def test_linear_views_strides_and_fallbacks():
    from pace_b200.ops import linear as L
    g = torch.Generator().manual_seed(1)
    w_big = (torch.randn(512, 640, generator=g) * 0.05).bfloat16().to(DEV)
    w = w_big[:, :512]                                           # a row pitch larger than K
    x = torch.randn(4, 3, 512, generator=g).bfloat16().to(DEV)   # [B, n, K]: 12 token rows
    assert L.fits(x, w)
    y = L.linear_skinny(x, w)
    assert y.shape == (4, 3, 512)
    want = _want(x.reshape(12, 512), w).view(4, 3, 512)
    assert (y.float() - want).abs().max().item() < 2e-2
    # more than 32 token rows, a bias, fp32, odd sizes: the library GEMM
    xb = torch.randn(40, 512, generator=g).bfloat16().to(DEV)
    assert not L.fits(xb, w)
    assert torch.equal(L.linear(xb, w), torch.nn.functional.linear(xb, w))
    assert not L.fits(x.float(), w.float()) and not L.fits(x[..., :500], w_big[:, :500])
    with pytest.raises(RuntimeError, match="linear_skinny"):
        L.linear_skinny(xb, w)
    # linear(), what the model calls, is the library GEMM
    assert torch.equal(L.linear(x, w), torch.nn.functional.linear(x, w))


def test_linear_in_a_graph_chain():
    """Several layers back to back in one CUDA graph (each launch's weights stream while the launch in
    front still runs; they share the workspace): every layer's result as when run alone."""
    from pace_b200.ops.linear import linear_skinny as linear
    g = torch.Generator().manual_seed(2)
    shapes = [(1024, 512), (512, 1024), (2048, 512), (512, 2048)]
    ws = [(torch.randn(n, k, generator=g) * 0.05).bfloat16().to(DEV) for n, k in shapes]
    x0 = torch.randn(32, 512, generator=g).bfloat16().to(DEV)

    def chain():
        h, outs = x0, []
        for w in ws:
            h = linear(h, w)
            outs.append(h)
        return outs
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        eager = [o.clone() for o in chain()]
    s.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr, stream=s):
        outs = chain()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, outs):      # (row tiles cut between thread blocks are summed in fp32 in arrival order)
        assert (a.float() - b.float()).abs().max().item() <= a.float().abs().max().item() * 2.0 ** -6
    h = x0
    for w, o in zip(ws, eager):
        want = _want(h, w)
        assert (o.float() - want).abs().max().item() <= (want.abs().max().item() * 2.0 ** -7 + 1e-3)
        h = o

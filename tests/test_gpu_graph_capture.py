"""The single-GPU entry points take a stream and launch nothing else on the side, so a chain
of them can be captured into a CUDA graph once and replayed: same bits as the eager calls,
also after the inputs change.  (The library's workspace is allocated on an op's first use,
which must therefore happen before the capture starts - the eager pass below does that.)"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def chain(fdl, a, b, c, row, gamma, beta):
    t = fdl.binary(a, b, fdl.MUL)
    t = fdl.binary(t, c, fdl.ADD)
    r = fdl.unary(t, fdl.RELU)
    fused = fdl.mul_add_relu(a, b, c)
    g = fdl.unary(t, 2)                                   # gelu
    w = fdl.broadcast_binary(t, row, fdl.ADD)
    sm = fdl.softmax_rows(w)
    ln = fdl.layernorm_rows(w, gamma, beta)
    rs = fdl.reduce_rows(w, fdl.REDUCE_SUM)
    rm = fdl.reduce_rows(w, fdl.REDUCE_MAX)
    am = fdl.argmax_rows(w)
    cm = fdl.reduce_cols(w, fdl.REDUCE_MEAN)
    total = fdl.full_sum(w.reshape(-1))
    blocks = fdl.block_reduce_1024(w.reshape(-1))
    return [r, fused, g, w, sm, ln, rs, rm, am, cm, total, blocks]


@pytest.mark.parametrize("shape", [(1024, 1024), (300, 4100)])
def test_chain_replays_from_a_cuda_graph(fdl, cuda, shape):
    rows, cols = shape
    rng = np.random.default_rng(5)

    def fresh():
        return [cuda.from_numpy(rng.uniform(-1, 1, shape).astype(np.float32)).cuda() for _ in range(3)]

    a, b, c = fresh()
    row = cuda.from_numpy(rng.uniform(-1, 1, (1, cols)).astype(np.float32)).cuda()
    gamma = cuda.from_numpy(rng.uniform(0.9, 1.1, cols).astype(np.float32)).cuda()
    beta = cuda.from_numpy(rng.uniform(-0.1, 0.1, cols).astype(np.float32)).cuda()
    chain(fdl, a, b, c, row, gamma, beta)                 # first use: workspace, kernel attributes
    cuda.cuda.synchronize()

    graph = cuda.cuda.CUDAGraph()
    with cuda.cuda.graph(graph):
        captured = chain(fdl, a, b, c, row, gamma, beta)
    for _ in range(3):
        for dst, src in zip((a, b, c), fresh()):
            dst.copy_(src)
        graph.replay()
        cuda.cuda.synchronize()
        got = [t.clone() for t in captured]
        want = chain(fdl, a, b, c, row, gamma, beta)
        cuda.cuda.synchronize()
        for i, (g, w) in enumerate(zip(got, want)):
            assert cuda.equal(g.view(cuda.int32) if g.dtype == cuda.float32 else g,
                              w.view(cuda.int32) if w.dtype == cuda.float32 else w), f"output {i} differs"
    fdl.take_device_error()

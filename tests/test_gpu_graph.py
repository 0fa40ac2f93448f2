"""CUDA-graph capture of the block, the way the reference engine captures its decode step around the MoE
hand-off (src/infrastructure/cuda_moe.rs:1283-1286): the asynchronous calls enqueue on the caller's stream,
allocate nothing, read nothing back, and fork / join their internal stream with events, so a captured graph
replays the whole block (router, routed experts, shared expert, combine) on new activations."""
import importlib

import pytest
import torch

pkg = importlib.import_module("ferrum-torrens_b200")

pytestmark = pytest.mark.gpu

H, I, E, K, SI = 2048, 512, 256, 8, 512


@pytest.fixture(scope="module")
def stack():
    dev = torch.device("cuda:0")
    layers = 2
    moe = pkg.B200MoE(0, pkg.ExpertShapes(H, I), E * layers, experts=E, layers=layers, top_k=K, shared_inter=SI,
                      max_tokens=512)
    dense = []
    for l in range(layers):
        pkg.synth.fill_banks_on_device(moe, l, seed=50 + l, slot0=l * E)
        dense.append(pkg.synth.device_dense_weights(60 + l, dev))
    yield moe, dense, dev
    moe.close()


@pytest.mark.parametrize("tokens", [1, 8, 64, 512])
def test_captured_block_replays_on_new_activations(stack, tokens):
    """T <= 256 takes the decode kernels, T = 512 the tcgen05 grouped GEMM (tensor maps are kernel arguments)."""
    moe, dense, dev = stack
    xs = [pkg.synth.device_x(70 + i, tokens, H, dev) for i in range(3)]

    def eager(x):
        outs = []
        for l, (g, su, sd, sg) in enumerate(dense):
            o = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev)
            ids = torch.empty((tokens, K), dtype=torch.int32, device=dev)
            moe.moe_block(l, x, g, su, sd, sg, o, ids_out=ids)
            outs.append((o, ids))
        moe.sync_status()
        return outs

    want = [eager(x) for x in xs]

    x_static = xs[0].clone()
    outs = [torch.empty((tokens, H), dtype=torch.bfloat16, device=dev) for _ in dense]
    idss = [torch.empty((tokens, K), dtype=torch.int32, device=dev) for _ in dense]
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for l, (g, su, sd, sg) in enumerate(dense):      # first call outside the capture (one-time attribute setup)
            moe.moe_block(l, x_static, g, su, sd, sg, outs[l], ids_out=idss[l])
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    launches_before = moe.kernel_launches()
    with torch.cuda.graph(graph, stream=side):
        for l, (g, su, sd, sg) in enumerate(dense):
            moe.moe_block(l, x_static, g, su, sd, sg, outs[l], ids_out=idss[l])
    assert moe.kernel_launches() > launches_before, "the capture enqueued this library's kernels"

    for i in (1, 2, 0, 1):
        x_static.copy_(xs[i])
        graph.replay()
        torch.cuda.synchronize()
        moe.sync_status()
        for l in range(len(dense)):
            assert torch.equal(idss[l], want[i][l][1]), (i, l)
            assert torch.equal(outs[l], want[i][l][0]), (i, l)

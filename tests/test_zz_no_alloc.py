"""pi05_gemm_static_scratch — the GEMM entry point for callers that cannot allocate.

Some callers of the library must not call cudaMalloc where they need a GEMM (a control loop
past its set-up phase, a plugin with a fixed memory budget), so this variant keeps the
split-K scratch in a fixed array inside the library. It must give exactly what pi05_gemm
gives with caller-provided scratch, on two calls in a row (the array is shared and keeps
the previous call's contents), and must refuse requests larger than its fixed scratch.
Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("op", [0, 1, 2])
def test_static_scratch_matches_caller_scratch_twice(op):
    from apxinf_b200 import _lib as L, kernels as K
    gen = torch.Generator().manual_seed(123 + op)
    M, N, Kd = 10, 1024, 4096
    if op == L.OP_BF16:
        a = torch.randn(M, Kd, generator=gen).to(torch.bfloat16)
        b = (torch.randn(N, Kd, generator=gen) * 0.05).to(torch.bfloat16)
    elif op == L.OP_E4M3:
        a = (torch.randn(M, Kd, generator=gen) * 4).to(torch.float8_e4m3fn)
        b = (torch.randn(N, Kd, generator=gen) * 4).to(torch.float8_e4m3fn)
    else:
        a = torch.randint(-128, 128, (M, Kd), generator=gen, dtype=torch.int8)
        b = torch.randint(-128, 128, (N, Kd), generator=gen, dtype=torch.int8)
    bias = (torch.randn(N, generator=gen) * 0.1).to(torch.bfloat16).cuda()
    ad, bd = a.cuda(), b.cuda()
    alpha = {0: 1.0, 1: 1.0 / 64, 2: 1e-4}[op]
    partials = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    counters = torch.zeros(1024, dtype=torch.int32, device="cuda")
    want = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    st = K.gemm(ad, bd, want, op=op, bias=bias, alpha=alpha, partials=partials,
                tile_counters=counters, force_split_k=8)
    torch.cuda.synchronize()
    assert st.item() == 0 and want.float().abs().max().item() > 0
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    status = K.new_status()
    # first call on the device (address look-up) happens here if no earlier test made it
    K.gemm(ad, bd, outs[0], op=op, bias=bias, alpha=alpha, force_split_k=8, static_scratch=True,
           status=status)
    torch.cuda.synchronize()
    for call in range(2):
        got = outs[call]
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        # the entry point takes no device memory: the driver's free-memory figure is the same
        # before and after the call (outputs and the status word were allocated above)
        free_before, _ = torch.cuda.mem_get_info()
        st = K.gemm(ad, bd, got, op=op, bias=bias, alpha=alpha, force_split_k=8, static_scratch=True,
                    status=status)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)
        assert st.item() == 0
        # same kernel, same split order: no tolerance needed (the GEMM tests allow one bf16
        # ulp against the CPU reference; here both sides are the GPU)
        assert torch.equal(got, want), f"call {call}: max diff {(got.float() - want.float()).abs().max().item()}"


def test_static_scratch_large_rows_and_limits():
    from apxinf_b200 import Pi05Error, _lib as L, kernels as K
    gen = torch.Generator().manual_seed(9)
    M, N, Kd = 300, 256, 4096
    a = torch.randn(M, Kd, generator=gen).to(torch.bfloat16).cuda()
    b = (torch.randn(N, Kd, generator=gen) * 0.05).to(torch.bfloat16).cuda()
    partials = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    counters = torch.zeros(1024, dtype=torch.int32, device="cuda")
    want = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    K.gemm(a, b, want, op=L.OP_BF16, out_type=L.OUT_F32, partials=partials, tile_counters=counters,
           force_split_k=4, force_swap=0)
    got = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    K.gemm(a, b, got, op=L.OP_BF16, out_type=L.OUT_F32, force_split_k=4, force_swap=0,
           static_scratch=True)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # more tiles x splits than the built-in scratch holds: refused before launch
    big_a = torch.zeros(4096, 4096, dtype=torch.bfloat16, device="cuda")
    big_b = torch.zeros(4096, 4096, dtype=torch.bfloat16, device="cuda")
    big_out = torch.zeros(4096, 4096, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Pi05Error) as info:
        K.gemm(big_a, big_b, big_out, op=L.OP_BF16, force_split_k=8, static_scratch=True)
    assert info.value.code == -7 and "scratch" in str(info.value)
    with pytest.raises(Pi05Error):  # the entry point is the split-K variant only
        K.gemm(a, b, got, op=L.OP_BF16, out_type=L.OUT_F32, force_split_k=1, static_scratch=True)


def test_static_scratch_wants_a_stream_of_the_current_device():
    """The built-in array's address is the current device's; a stream of another device is
    refused before anything is launched. Needs a second GPU to see the refusal."""
    from apxinf_b200 import Pi05Error, _lib as L, kernels as K
    a = torch.zeros(16, 256, dtype=torch.bfloat16, device="cuda:0")
    b = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda:0")
    out = torch.zeros(16, 128, dtype=torch.bfloat16, device="cuda:0")
    # a non-default stream of the current device is accepted
    side = torch.cuda.Stream(device=0)
    K.gemm(a, b, out, op=L.OP_BF16, force_split_k=2, static_scratch=True, stream=side)
    side.synchronize()
    if torch.cuda.device_count() < 2:
        return
    other = torch.cuda.Stream(device=1)
    with pytest.raises(Pi05Error) as info:
        K.gemm(a, b, out, op=L.OP_BF16, force_split_k=2, static_scratch=True, stream=other)
    assert info.value.code == -1


def test_static_scratch_is_capturable_after_the_first_call():
    """After one eager call per device the entry point neither allocates nor synchronises: it
    can be captured into a CUDA graph in thread-local capture mode, the mode the engine captures
    in (an allocation or a synchronising call by the capturing thread fails the capture), and the
    graph replays to the same result."""
    from apxinf_b200 import _lib as L, kernels as K
    gen = torch.Generator().manual_seed(7)
    M, N, Kd = 24, 512, 2048
    a = torch.randn(M, Kd, generator=gen).to(torch.bfloat16).cuda()
    b = (torch.randn(N, Kd, generator=gen) * 0.05).to(torch.bfloat16).cuda()
    want = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    got = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    status = K.new_status()
    K.gemm(a, b, want, op=L.OP_BF16, force_split_k=4, static_scratch=True, status=status)  # eager, first
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
        K.gemm(a, b, got, op=L.OP_BF16, force_split_k=4, static_scratch=True, status=status)
    for _ in range(2):
        got.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert status.item() == 0
        assert torch.equal(got, want)
    del graph
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before - (4 << 20)  # the graph object itself, nothing per call

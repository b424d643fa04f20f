"""A context belongs to one CUDA device.  With tensors on cuda:1 while cuda:0 is the current device, both host faces
refuse the call on the host — nothing is launched on the wrong GPU — and under torch.cuda.device(1) the same call works
and returns what device 0 returns.  Needs two GPUs; skipped otherwise."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")


@needs_two
def test_mismatched_device_is_refused_and_matching_device_works(small_graph):
    from graph_sampling_b200 import ops
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = small_graph
    seeds = np.arange(0, 600, 3, dtype=np.int64)
    on0 = [torch.from_numpy(a).to("cuda:0") for a in (indptr, indices, seeds)]
    on1 = [torch.from_numpy(a).to("cuda:1") for a in (indptr, indices, seeds)]
    torch.cuda.set_device(0)
    want = ops.csc_col_slicing(*on0)
    with pytest.raises(GsbError) as e:                    # tensors and context of device 1, device 0 current
        ops.csc_col_slicing(*on1)
    assert e.value.status == -1 and "device" in str(e.value)
    with pytest.raises(GsbError):
        ops.fused_csc_col_slicing_sampling(on1[0], on1[1], on1[2], 4, False, seed=1)
    with torch.cuda.device(1):
        got = ops.csc_col_slicing(*on1)
        smp1 = ops.fused_csc_col_slicing_sampling(on1[0], on1[1], on1[2], 4, False, seed=1)
    smp0 = ops.fused_csc_col_slicing_sampling(on0[0], on0[1], on0[2], 4, False, seed=1)
    for w, g in zip(want, got):
        assert torch.equal(w.cpu(), g.cpu())
    for w, g in zip(smp0, smp1):
        assert torch.equal(w.cpu(), g.cpu())
    ops.default_context(torch.device("cuda", 0)).check_device()     # device 0's context saw no error


@needs_two
def test_torchscript_face_refuses_tensors_of_another_device(small_graph):
    from graph_sampling_b200 import build as b
    torch.classes.load_library(b.build_glue())
    indptr, indices = small_graph
    torch.cuda.set_device(0)
    g = torch.classes.gs_classes.Graph(False)
    with pytest.raises(RuntimeError, match="current device"):
        g._CAPI_LoadCSC(torch.from_numpy(indptr).to("cuda:1"), torch.from_numpy(indices).to("cuda:1"))
    with torch.cuda.device(1):
        g._CAPI_LoadCSC(torch.from_numpy(indptr).to("cuda:1"), torch.from_numpy(indices).to("cuda:1"))
        sub = g._CAPI_FusedColumnwiseSlicingSampling(torch.arange(50, device="cuda:1"), 3, False)
        assert int(sub._CAPI_GetNumEdges()) > 0

"""The calls of the path can be recorded into a CUDA graph and replayed: they launch on the
THCState's current stream, allocate nothing once the context's workspace has its size, and the
full reduction has a form that leaves its result on the device (sumallToDevice).  This is how a
host that issues many small tensor calls removes the per-launch cost on B200.

torch is used here only to own the capture (torch.cuda.graph) and the device buffers."""
import numpy as np
import pytest

from cutorch_b200 import thc
from common import assert_bit_equal, rng

pytestmark = pytest.mark.gpu


def test_step_recorded_in_a_cuda_graph_replays_with_new_inputs(oracle):
    import torch
    from cutorch_b200._lib import OP, RED
    dev = torch.device("cuda", 0)
    state = thc.State()
    side = torch.cuda.Stream()
    state.set_stream(side.cuda_stream, 0)
    rows, cols = 512, 4096
    x = torch.empty(rows, cols, device=dev)
    y = torch.empty(rows, cols, device=dev)
    z = torch.empty(rows, cols, device=dev)
    v = torch.empty(rows, 1, device=dev)
    i = torch.empty(rows, 1, dtype=torch.int64, device=dev)
    total = torch.zeros(1, dtype=torch.float64, device=dev)

    def W(t, kind):
        w = thc.Tensor.wrap(state, kind, t.data_ptr(), tuple(t.shape), tuple(t.stride()))
        w._owner = t
        return w

    tx, ty, tz, tv, ti = W(x, "Float"), W(y, "Float"), W(z, "Float"), W(v, "Float"), W(i, "Long")

    def step():
        tz.cmul(tx, ty)
        tz.add(tz, 1.0)
        tv.max(ti, tz, 1, 1)
        tz.sumall_to_device(total.data_ptr())

    r = rng("graph")
    with torch.cuda.stream(side):
        x.copy_(torch.from_numpy(r.standard_normal((rows, cols)).astype(np.float32)))
        y.copy_(torch.from_numpy(r.standard_normal((rows, cols)).astype(np.float32)))
        step()                      # warm-up: sizes the workspace outside the capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        for trial in range(3):
            hx = r.standard_normal((rows, cols)).astype(np.float32)
            hy = r.standard_normal((rows, cols)).astype(np.float32)
            x.copy_(torch.from_numpy(hx))
            y.copy_(torch.from_numpy(hy))
            graph.replay()
            side.synchronize()
            want_z = oracle.pointwise(OP["ADD_S"], np.zeros_like(hx),
                                      [oracle.pointwise(OP["MUL"], np.zeros_like(hx), [hx, hy])], 1.0)
            want_v, want_i = oracle.reduce_dim(RED["MAX"], 0, 0, want_z, 1, with_index=True)
            assert_bit_equal(z.cpu().numpy(), want_z, f"replay {trial}: z")
            assert_bit_equal(v.cpu().numpy(), want_v, f"replay {trial}: row max")
            assert_bit_equal(i.cpu().numpy(), want_i, f"replay {trial}: row argmax")
            want_sum = oracle.reduce_all(RED["SUM"], 0, 0, want_z)
            assert abs(float(total.item()) - want_sum) <= 1e-5 * abs(want_sum) + 1e-3, f"replay {trial}: sum"
    state.shutdown()

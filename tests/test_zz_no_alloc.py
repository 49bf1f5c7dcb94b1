"""The allocation-free value-head entry point against the regular forward.

Some callers of this library cannot allocate: a search thread in the middle of
a self-play loop (a cudaMalloc would synchronise the device under every other
engine's stream) or a process whose GPU memory was budgeted once at start-up.
For them ob200_net_value_head_noalloc keeps its intermediates in an array built
into the library.  The check: through the C ABI, on two calls in a row, its
values equal the ones ob200_net_forward_device produced from the same tower
output (same kernels, same order of operations, so equality is exact; the
tolerance of the network tests, 1e-2, is the stated bound)."""
import numpy as np
import pytest

from omoknuni_small_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [0, 1], ids=["bf16", "f16"])
def test_value_head_noalloc_matches_forward_twice(lib, dtype):
    import torch
    from omoknuni_small_b200 import capi
    shapes = synth.net_tensor_shapes(15, 17, 64, 2, 225, 2, 1)
    w = synth.make_weights(shapes, seed=5, init="torch_default", bn="random")
    B = 96
    net = capi.Net(17, 15, 2, 64, 225, 2, 1, 256, B, tower_dtype=dtype).load(w)
    policy = torch.empty((B, 225), dtype=torch.float32, device="cuda")
    value = torch.empty(B, dtype=torch.float32, device="cuda")
    for call, seed in enumerate((11, 12)):                       # two calls in a row, different inputs
        x = synth.make_stone_planes(B, 15, 17, seed=seed)
        bt = capi.planes_to_board_tensor(torch.from_numpy(x).cuda(), net.input_tensor_channels(), dtype)
        net.forward_device(bt, B, policy, value, capi.OUT_PROBS)     # the existing entry point
        torch.cuda.synchronize()
        want = value.cpu().numpy().copy()
        got = torch.full((B,), 7.0, dtype=torch.float32, device="cuda")
        net.value_head_noalloc(net.tower_output_ptr(), B, got)      # the allocation-free entry point
        torch.cuda.synchronize()
        got = got.cpu().numpy()
        assert np.abs(got - want).max() <= 1e-2, f"call {call}: {np.abs(got - want).max()}"
        assert np.array_equal(got, want), f"call {call}: same kernels must give identical values"
        assert np.all(np.abs(got) <= 1.0)


def test_value_head_noalloc_rejects_oversize(lib):
    from omoknuni_small_b200 import capi
    import torch
    shapes = synth.net_tensor_shapes(15, 17, 64, 1, 225, 32, 32)
    w = synth.make_weights(shapes, seed=6, init="torch_default")
    net = capi.Net(17, 15, 1, 64, 225, 32, 32, 256, 128).load(w)
    cap = int(capi.lib().ob200_value_head_noalloc_capacity())
    assert cap == 1 << 19
    per_board = 32 * 225 + 256
    too_many = cap // per_board + 1                                  # 71 boards of the 32-channel head
    x = synth.make_stone_planes(128, 15, 17, seed=1)
    policy = torch.empty((128, 225), dtype=torch.float32, device="cuda")
    value = torch.empty(128, dtype=torch.float32, device="cuda")
    bt = capi.planes_to_board_tensor(torch.from_numpy(x).cuda(), 64)
    net.forward_device(bt, 128, policy, value)
    out = torch.empty(128, dtype=torch.float32, device="cuda")
    with pytest.raises(capi.Error) as e:
        net.value_head_noalloc(net.tower_output_ptr(), too_many, out)
    assert e.value.code == 7 and "static array" in str(e.value)
    net.value_head_noalloc(net.tower_output_ptr(), too_many - 1, out)   # the largest batch that fits
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy()[: too_many - 1], value.cpu().numpy()[: too_many - 1])

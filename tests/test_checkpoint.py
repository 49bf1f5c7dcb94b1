"""Checkpoint import: a file written by the reference's own ResNetModel::save is read back
tensor for tensor, converted to the flat format the adapter loads, and its shape recovered."""
import numpy as np
import pytest

from omoknuni_small_b200 import checkpoint, synth


def test_flat_round_trip(tmp_path):
    shapes = synth.net_tensor_shapes(9, 17, 64, 1, 81, 2, 1)
    w = synth.make_weights(shapes, seed=1, init="torch_default", bn="random")
    checkpoint.write_flat(tmp_path / "w.bin", w)
    back = checkpoint.read_flat(tmp_path / "w.bin")
    assert list(back) == [k for k, _ in shapes]
    assert all(np.array_equal(back[k], w[k].ravel()) for k in w)
    assert checkpoint.infer_config(w) == dict(input_channels=17, board_size=9, blocks=1, filters=64, policy_size=81,
                                              policy_head_ch=2, value_head_ch=1, value_hidden=256)


def test_reads_a_checkpoint_saved_by_the_reference(tmp_path, oracle):
    if not oracle.have_ref_net():
        pytest.skip("oracle/_ref not built here (the reference checkout is absent)")
    net = oracle.RefNet(19, 15, 2, 64, 225, seed=11)
    net.save(tmp_path / "model_gomoku_15x15.pt")
    got = checkpoint.load_reference_checkpoint(tmp_path / "model_gomoku_15x15.pt")
    want = {k: v for k, v in net.state().items() if "num_batches" not in k}
    assert set(got) == set(want)
    assert all(np.array_equal(got[k].ravel(), want[k]) for k in want)
    assert checkpoint.infer_config(got) == dict(input_channels=19, board_size=15, blocks=2, filters=64, policy_size=225,
                                                policy_head_ch=32, value_head_ch=32, value_hidden=256)
    assert checkpoint.main(["checkpoint", str(tmp_path / "model_gomoku_15x15.pt"), str(tmp_path / "out.bin")]) == 0
    flat = checkpoint.read_flat(tmp_path / "out.bin")
    assert all(np.array_equal(flat[k], want[k]) for k in want)

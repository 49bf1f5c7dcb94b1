"""Drop-in check with the reference's own types: oracle/_ref/adapter_check (built where
the reference checkout exists; it travels as a binary) hands real GomokuState objects to
B200Network::inference through a NeuralNetwork pointer.  Its outputs must match the fp32
forward of the oracle on the oracle's planes for the same games."""
import os
import struct
import subprocess

import numpy as np
import pytest

from omoknuni_small_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "adapter_check")


def write_weights(path, shapes, w):
    with open(path, "wb") as f:
        for name, _ in shapes:
            a = np.ascontiguousarray(w[name], np.float32).ravel()
            f.write(struct.pack("<I", len(name)) + name.encode() + struct.pack("<Q", a.size) + a.tobytes())


@pytest.mark.skipif(not os.path.exists(BIN), reason="oracle/_ref/adapter_check not built (needs the reference checkout)")
def test_reference_states_through_cpp_adapter(tmp_path, oracle, lib):
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(15, 19, 64, 3, 225, 32, 32)
    w = synth.make_weights(shapes, seed=21, init="torch_default", bn="random")
    write_weights(tmp_path / "w.bin", shapes, w)
    games, hist, nh, tm = synth.make_gomoku_games(150, 15, seed=33)     # 150 > the adapter's max_batch of 64
    null_at = 7
    with open(tmp_path / "g.bin", "wb") as f:
        f.write(struct.pack("<i", len(games)))
        for i, mv in enumerate(games):
            if i == null_at:
                f.write(struct.pack("<i", -1))
            else:
                f.write(struct.pack("<i", len(mv)) + np.asarray(mv, np.int32).tobytes())
    r = subprocess.run([BIN, str(tmp_path / "w.bin"), str(tmp_path / "g.bin"), str(tmp_path / "o.bin"), "19", "3", "32", "32"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = np.fromfile(tmp_path / "o.bin", np.float32)
    n = len(games)
    probs, value = raw[: n * 225].reshape(n, 225), raw[n * 225:]
    planes = oracle.gomoku_encode(hist, nh, tm, 15, 19)
    planes[null_at] = 0.0                                                # a null state is all-zero planes
    ref_logits, ref_v = net_ref.forward(w, planes)
    assert np.abs(probs - net_ref.softmax(ref_logits)).max() <= 1e-3
    assert np.abs(value - ref_v).max() <= 1e-2
    assert np.allclose(probs.sum(1), 1, atol=1e-5)

"""Drop-in checks with the reference's own types and code: oracle/_ref/adapter_check (built
where the reference checkout exists; it travels as a binary) drives the C++ adapters with real
GomokuState / MCTSNode objects and with the reference's own batch collector
(SharedInferenceQueue, compiled unchanged from its source).  Network outputs must match the
fp32 forward of the oracle on the oracle's planes for the same games."""
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


needs_bin = pytest.mark.skipif(not os.path.exists(BIN), reason="oracle/_ref/adapter_check not built (needs the reference checkout)")


def write_case(tmp_path, n_games, null_at=None, seed=33):
    shapes = synth.net_tensor_shapes(15, 19, 64, 3, 225, 32, 32)
    w = synth.make_weights(shapes, seed=21, init="torch_default", bn="random")
    write_weights(tmp_path / "w.bin", shapes, w)
    games, hist, nh, tm = synth.make_gomoku_games(n_games, 15, seed=seed)
    with open(tmp_path / "g.bin", "wb") as f:
        f.write(struct.pack("<i", len(games)))
        for i, mv in enumerate(games):
            if i == null_at:
                f.write(struct.pack("<i", -1))
            else:
                f.write(struct.pack("<i", len(mv)) + np.asarray(mv, np.int32).tobytes())
    return w, games, hist, nh, tm


def check_against_fp32(tmp_path, oracle, w, games, hist, nh, tm, null_at=None):
    from oracle import net_ref
    raw = np.fromfile(tmp_path / "o.bin", np.float32)
    n = len(games)
    probs, value = raw[: n * 225].reshape(n, 225), raw[n * 225:]
    planes = oracle.gomoku_encode(hist, nh, tm, 15, 19)
    if null_at is not None:
        planes[null_at] = 0.0                                            # a null state is all-zero planes
    ref_logits, ref_v = net_ref.forward(w, planes)
    assert np.abs(probs - net_ref.softmax(ref_logits)).max() <= 1e-3
    assert np.abs(value - ref_v).max() <= 1e-2
    assert np.allclose(probs.sum(1), 1, atol=1e-5)


@needs_bin
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_reference_states_through_cpp_adapter(tmp_path, oracle, lib, dtype):
    """NeuralNetwork::inference with real GomokuState objects, a null state, more states than max_batch."""
    w, games, hist, nh, tm = write_case(tmp_path, 150, null_at=7)        # 150 > the adapter's max_batch of 64
    r = subprocess.run([BIN, "direct", str(tmp_path / "w.bin"), str(tmp_path / "g.bin"), str(tmp_path / "o.bin"), "19", "3", "32", "32", dtype],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    check_against_fp32(tmp_path, oracle, w, games, hist, nh, tm, null_at=7)


@needs_bin
def test_reference_batch_collector_in_front_of_the_network(tmp_path, oracle, lib):
    """The reference's SharedInferenceQueue::submitBatch from 6 producer threads with the B200 network behind it:
    per-request results equal direct inference (checked inside the binary, bit for bit), the reference's failure
    conventions hold (default outputs for a network that is not ready, exception at future.get() for one that
    throws), and the collected outputs match the fp32 forward."""
    w, games, hist, nh, tm = write_case(tmp_path, 230, seed=34)
    r = subprocess.run([BIN, "queue", str(tmp_path / "w.bin"), str(tmp_path / "g.bin"), str(tmp_path / "o.bin"), "19", "3", "32", "32", "6"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "equal to direct inference" in r.stdout
    check_against_fp32(tmp_path, oracle, w, games, hist, nh, tm)


@needs_bin
@pytest.mark.parametrize("seed", [1, 2])
def test_tree_adapter_against_real_mcts_nodes(lib, seed):
    """B200Tree (selectChildBatch / applyVirtualLoss / revertVirtualLoss / backup / setPriorProbabilities) against
    300 real MCTSNode families, chains of real nodes, and expand + setPriorProbabilities on a real GomokuState."""
    r = subprocess.run([BIN, "tree", str(seed)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "equal to MCTSNode" in r.stdout


@needs_bin
def test_search_adapter_fills_the_reference_result_types(tmp_path, lib):
    """B200GomokuSearch: MCTSSettings in, SearchResult / MCTSStats out, with the assertions the reference's engine
    tests make (legal action, 225 probabilities summing to one, nodes, evaluations, average batch size > 1)."""
    write_case(tmp_path, 4)
    r = subprocess.run([BIN, "engine", str(tmp_path / "w.bin"), "19", "3", "32", "32"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "MCTSSettings -> SearchResult" in r.stdout

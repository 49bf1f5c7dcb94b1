"""Encoder parity: the bf16 board tensor decodes to exactly the planes of the
CPU oracle / the reference's GomokuState (values are 0/1, so bf16 is exact)."""
import numpy as np
import pytest

from omoknuni_small_b200 import synth
from test_oracle import load_encode_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api(lib):
    from omoknuni_small_b200 import capi
    return capi


def run_encode(api, hist, nh, tm, S, planes, out_channels=64):
    import torch
    bt = api.encode_gomoku(torch.from_numpy(hist).cuda(), torch.from_numpy(nh).cuda(), torch.from_numpy(tm).cuda(), S,
                           planes, out_channels)
    torch.cuda.synchronize()
    return api.board_tensor_to_planes(bt.cpu().numpy().view(np.uint16), S, hist.shape[0], out_channels)


@pytest.mark.parametrize("planes", [17, 19])
def test_encode_matches_reference_golden(api, planes):
    games, hist, nh, tm, ref, _ = load_encode_golden()
    got, pad_zero = run_encode(api, hist, nh, tm, 15, planes)
    assert pad_zero
    assert np.array_equal(got[:, :planes], ref[:, :planes])
    assert not got[:, planes:].any()


@pytest.mark.parametrize("B,S,seed", [(1, 15, 1), (257, 15, 2), (1024, 15, 3), (40, 9, 4), (7, 19, 5)])
def test_encode_matches_oracle(api, oracle, B, S, seed):
    games, hist, nh, tm = synth.make_gomoku_games(B, S, seed=seed)
    got, pad_zero = run_encode(api, hist, nh, tm, S, 19)
    assert pad_zero and np.array_equal(got[:, :19], oracle.gomoku_encode(hist, nh, tm, S, 19))


def test_encode_edge_cases(api, oracle):
    # empty history, full 16-move history, history entries beyond n_hist are ignored
    hist = np.full((3, 16), -1, np.int16)
    hist[1] = np.arange(16) * 14
    hist[2] = np.arange(16) + 100
    nh = np.array([0, 16, 5], np.uint8)
    tm = np.array([1, 1, 2], np.uint8)
    got, pad_zero = run_encode(api, hist, nh, tm, 15, 19)
    assert pad_zero and np.array_equal(got[:, :19], oracle.gomoku_encode(hist, nh, tm, 15, 19))
    assert got[0, 16].all() and not got[0, :16].any() and not got[2, 16].any()


def test_planes_to_board_tensor_round_trip(api):
    import torch
    x = synth.make_stone_planes(33, 15, 17, seed=6)
    x[:, 3] *= 0.37                                           # a non-binary plane: must match host rounding to bf16
    bt = api.planes_to_board_tensor(torch.from_numpy(x).cuda(), 64)
    torch.cuda.synchronize()
    got = bt.cpu().numpy().view(np.uint16)
    assert np.array_equal(got, api.planes_to_board_tensor_host(x, 64))
